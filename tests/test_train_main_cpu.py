"""The training entry point end to end on two CPU ranks: the reference's flags, its ``time.txt`` sink, and the
per-step metrics file, for the dense method and the ZEN hook."""
import json
import os

import pytest

from _dist_util import run_gloo


def _main_worker(rank, world, method, tmp):
    import train

    os.environ["RANK"], os.environ["WORLD_SIZE"], os.environ["LOCAL_RANK"] = str(rank), str(world), str(rank)
    train.main(["--model_name", "tiny-gpt2", "-b", "2", "-l", "16", "-s", "6", "--tp", "1", "--method", str(method),
                "--top_k", "20", "--bucket_cap", "1", "--no_grad_checkpoint", "--time_from", "2", "--time_to", "5",
                "--log_dir", tmp, "--time_file", os.path.join(tmp, "time.txt"),
                "--metrics_out", os.path.join(tmp, "metrics.jsonl"), "--metrics_every", "2"])
    return True


@pytest.mark.parametrize("method", [0, 3])
def test_train_main_writes_time_txt_and_step_metrics(method, tmp_path):
    run_gloo(_main_worker, 2, method, str(tmp_path), timeout=300)
    lines = open(tmp_path / "time.txt").read().strip().splitlines()
    assert lines[0] == f"tiny-gpt2 method {method} topk 20 dp 2"
    assert float(lines[1]) > 0
    recs = [json.loads(l) for l in open(tmp_path / "metrics.jsonl")]
    steps = [r for r in recs if r["kind"] == "step"]
    assert [r["step"] for r in steps] == list(range(7))
    assert all(r["loss"] == r["loss"] and r["step_ms"] > 0 for r in steps)
    sampled = [r for r in steps if "recoveries" in r]
    assert [r["step"] for r in sampled] == [0, 2, 4, 6]
    if method == 0:
        assert all(r["embedding_rows_sent"] > 0 and 0 < r["embedding_row_density"] <= 1 for r in sampled)
    summary = [r for r in recs if r["kind"] == "summary"]
    assert len(summary) == 1 and summary[0]["tokens_per_s"] > 0 and summary[0]["dp"] == 2
    assert steps[-1]["loss"] < steps[0]["loss"]
