"""Status mirror and agreed recovery on CPU ranks: the failure is made on the host (a status word that one rank sets),
no kernel waits or faults."""
import pytest
import torch

from _dist_util import run_gloo


def test_status_mirror_reads_one_step_late_and_in_step_order():
    from zen_repro_b200.parallel.health import StatusMirror, decode

    m = StatusMirror("cpu")
    w = torch.zeros(1, dtype=torch.int32)
    m.add("x", w)
    seen = []
    for step in range(7):
        seen.append(m.poll())
        if step == 3:
            w[0] = 4
        m.publish()
    # set during step 3, published at the end of step 3, visible to the poll at the start of step 5 (lag 1)
    assert seen[:5] == [{}, {}, {}, {}, {}] and seen[5] == {"x": 4} and seen[6] == {"x": 4}
    assert "expired" in decode(4) and decode(0) == "ok"
    m.clear()
    assert int(w) == 0


def _recover_worker(rank, world, policy):
    from zen_repro_b200.parallel.health import SyncStatusError
    from zen_repro_b200.trainer import TrainConfig, Trainer

    t = Trainer(TrainConfig(model="tiny-gpt2", micro_batch=2, seq_len=16, precision="fp32", lr=1e-2, data_pool=0,
                            sparse_embedding=True, bucket_cap_mb=0.05, on_sync_error=policy), init_dist=False)
    fake = torch.zeros(1, dtype=torch.int32)
    t.health.add("embedding_rows", fake)                 # stands in for the engine's device status word
    raised_at = None
    for step in range(8):
        if step == 2 and rank == 1:
            fake[0] = 4                                  # only rank 1 "timed out", and it also drifted
            with torch.no_grad():
                t.model.unwrap().wte.add_(0.5)
        try:
            t.step(next(t.data))
        except SyncStatusError:
            raised_at = step
            break
    w = t.model.unwrap().wte.detach().clone()
    return raised_at, t.recoveries, bool(t.model.module.embedding_sync.force_library), w


def test_every_rank_recovers_at_the_same_step_and_replicas_agree_again():
    out = run_gloo(_recover_worker, 2, "recover")
    for raised, rec, forced, _ in out:
        assert raised is None and forced and len(rec) == 1
    assert out[0][1][0]["step"] == out[1][1][0]["step"] == 4          # set in step 2, published, read at the start of step 4
    assert out[0][1][0]["status"] == out[1][1][0]["status"] == {"embedding_rows": 4}
    torch.testing.assert_close(torch.as_tensor(out[0][3]), torch.as_tensor(out[1][3]), atol=0, rtol=0)


def test_raise_policy_stops_every_rank_at_the_same_step():
    out = run_gloo(_recover_worker, 2, "raise")
    assert [o[0] for o in out] == [4, 4]
