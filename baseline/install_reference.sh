#!/bin/bash
# Installs the unmodified reference into baseline/_ref (git-ignored): its CUDA extension is built with its own
# setup.py, its Python modules are copied verbatim.  The reference tree has no top-level setup.py / pyproject, so
# `pip install <reference root>` fails with "neither setup.py nor pyproject.toml found"; the extension directory
# is the installable part.  REF = path of the reference checkout (first argument or environment); the build writes
# into the source tree, hence the copy.  WHEELS = optional directory of offline wheels for pip.
set -e
REF=${1:-${REF:?usage: install_reference.sh <path of the reference checkout>}}
WHEELS=${WHEELS:-/opt/wheelhouse}
HERE="$(cd "$(dirname "$0")" && pwd)"
TMP=$(mktemp -d)
cp -r "$REF"/. "$TMP"/
( cd "$TMP/extensions/cuda" && TORCH_CUDA_ARCH_LIST=10.0a python -m pip install --no-index --no-build-isolation --no-deps \
    --find-links "$WHEELS" --target "$HERE/_ref" . )
for f in comm.py DDPbackend.py tensor_load_balance.py train.py utils.py; do cp "$REF/$f" "$HERE/_ref/$f"; done
mkdir -p "$HERE/_ref/extensions/cuda"
cp "$REF/extensions/cuda/functions.py" "$HERE/_ref/extensions/cuda/functions.py"
touch "$HERE/_ref/extensions/__init__.py" "$HERE/_ref/extensions/cuda/__init__.py"
echo "installed into $HERE/_ref"
