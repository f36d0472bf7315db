import pytest
import torch

from _dist_util import run_gloo


def _worker(rank, world):
    import torch.distributed as dist

    from zen_repro_b200.compat.comm import LoadBalanceAllreduce
    from zen_repro_b200.compat.DDPbackend import DDPBackend
    from zen_repro_b200.compat.tensor_load_balance import TensorPartition

    g = dist.group.WORLD
    be = DDPBackend(g, list(range(world)))
    t = torch.arange(rank + 2, dtype=torch.float32) + 10 * rank
    parts = be.allgather_padding(t)
    assert [p.numel() for p in parts] == [r + 2 for r in range(world)]
    assert torch.equal(parts[1], torch.arange(3, dtype=torch.float32) + 10)
    parts2 = be.allgatherv(t)
    assert all(torch.equal(a, b) for a, b in zip(parts, parts2))
    sends = [torch.full((rank + p + 1,), float(rank * 10 + p)) for p in range(world)]
    recv = be.alltoallv(sends)
    assert [r.numel() for r in recv] == [q + rank + 1 for q in range(world)]
    assert all(float(r[0]) == q * 10 + rank for q, r in enumerate(recv))
    lba = LoadBalanceAllreduce(g, list(range(world)), None)
    gen = torch.Generator().manual_seed(rank)
    x = torch.zeros(20000)
    idx = torch.randperm(20000, generator=gen)[:300]
    x[idx] = torch.randn(300, generator=gen)
    x[0] = 1.0
    want = x.clone()
    dist.all_reduce(want)
    for m in (1, 2, 3):
        torch.testing.assert_close(lba.zen_sparse_comm(x, m), want, atol=1e-5, rtol=0)
    own = lba.calculate_mapping(20000)
    assert sum(o.numel() for o in own) == 20000
    mine = torch.nonzero(x, as_tuple=True)[0]
    mine = mine[torch.isin(mine, own[rank])]
    bm = lba.encode_bitmap(mine, 20000)
    assert int(bm[0]) & 1 == int(bool((mine == own[rank][0]).any()))      # LSB-first
    decoded = lba.decode_bitmap(be.allgather_padding(bm), 20000)
    assert torch.equal(decoded[rank], mine)
    tp = TensorPartition(world, 1, 3)
    i, v, s = tp.load_balance(x)
    assert int(s.sum()) == int((x != 0).sum())
    tz = TensorPartition(world, 1, 3, hash="zen_poly3")
    i2, v2, s2 = tz.load_balance(x[:3000].contiguous())
    got = torch.cat(i2).sort().values
    assert torch.equal(got.long(), torch.nonzero(x[:3000], as_tuple=True)[0])
    return True


def test_reference_shaped_api_on_gloo():
    assert all(run_gloo(_worker, 2))


def test_compress_keeps_about_top_k_percent():
    from zen_repro_b200.parallel.hooks import compress, compress_with_allgather

    torch.manual_seed(0)
    g = torch.randn(200000)
    out = compress(5, g)
    frac = float((out != 0).float().mean())
    assert 0.03 < frac < 0.08
    small = torch.randn(4096)
    assert compress_with_allgather(1, small, None) is small


def test_every_native_entry_point_named_in_the_package_is_exported():
    """A C entry point whose signature mentions a type from an unnamed namespace silently gets internal linkage; catch
    that (and plain typos) without a GPU: every ``zen_*`` name the Python package calls must be a symbol of the library."""
    import ctypes
    import pathlib
    import re

    from zen_repro_b200 import build as zbuild

    path = zbuild.lib_path()
    if not path.exists():
        pytest.skip("native library not built")
    cdll = ctypes.CDLL(str(path))
    root = pathlib.Path(zbuild.__file__).parent
    names = set()
    for f in root.rglob("*.py"):
        names |= set(re.findall(r"\b(?:lib\(\)|lib|_lib)\.(zen_[a-z0-9_]+)\b", f.read_text()))
    assert len(names) > 40
    missing = sorted(n for n in names if not hasattr(cdll, n))
    assert not missing, missing
