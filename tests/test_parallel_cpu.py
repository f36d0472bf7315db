"""Reducer, embedding row sync and tensor parallelism on CPU ranks (gloo)."""
import pytest
import torch

from _dist_util import run_gloo
from zen_repro_b200.models import build_model, get_config


@pytest.mark.parametrize("name", ["tiny-gpt2", "tiny-llama", "tiny-gemma", "tiny-opt"])
def test_reducer_grads_equal_plain_autograd(name):
    from zen_repro_b200.parallel.embedding_sync import EmbeddingRowSync
    from zen_repro_b200.parallel.reducer import ZenDDP

    torch.manual_seed(0)
    ids = torch.randint(0, 1000, (2, 16))
    a = build_model(name, dtype=torch.float32)
    b = build_model(name, dtype=torch.float32)
    b.load_state_dict(a.state_dict())
    a(ids, ids).backward()
    sync = EmbeddingRowSync(b.wte.shape[0], b.wte.shape[1], 32, None, dtype=torch.float32)
    sync.target_param = b.wte
    b.sparse_sink = sync
    if b.lm_head is not None:
        b.wte.zen_sparse_only = True
    ddp = ZenDDP(b, None, 0.05, sync)
    for _ in range(2):                       # second pass checks zero_grad / re-arming
        ddp.zero_grad()
        ddp(ids, ids).backward()
        # gradient-producing ops write into the bucket views themselves: their claims were counted in forward and
        # signalled in backward, and the gradients still live in the buckets
        direct = [q for q in b.parameters() if getattr(q, "zen_expected", 0) > 0]
        assert len(direct) >= len(list(b.parameters())) - 3
        assert all(q.zen_signals == q.zen_expected for q in direct)
        assert all(q.grad.data_ptr() == ddp._view_of[id(q)].data_ptr() for q in direct)
        ddp.finalize_grads()
    for (n, p), q in zip(a.named_parameters(), b.parameters()):
        torch.testing.assert_close(q.grad, p.grad, atol=1e-6, rtol=1e-5, msg=lambda m, n=n: f"{n}: {m}")


def _dp_worker(rank, world, sparse, method):
    from zen_repro_b200.trainer import TrainConfig, Trainer

    t = Trainer(TrainConfig(model="tiny-gpt2", micro_batch=2, seq_len=16, precision="fp32", lr=1e-2, data_pool=0,
                            sparse_embedding=sparse, method=method, top_k=20, bucket_cap_mb=0.05), init_dist=False)
    losses = [t.step(next(t.data)) for _ in range(6)]
    w = t.model.unwrap().wte.detach().clone()
    return losses, w


def test_sparse_embedding_rows_match_dense_sync_on_two_ranks():
    s = run_gloo(_dp_worker, 2, True, 0)
    d = run_gloo(_dp_worker, 2, False, 0)
    for r in range(2):
        assert s[r][0] == pytest.approx(d[r][0], rel=1e-4, abs=1e-4)
        torch.testing.assert_close(torch.as_tensor(s[r][1]), torch.as_tensor(d[r][1]), atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(torch.as_tensor(s[0][1]), torch.as_tensor(s[1][1]), atol=0, rtol=0)         # replicas stay identical


def test_zen_hook_trains_on_two_ranks():
    out = run_gloo(_dp_worker, 2, False, 3)
    losses = out[0][0]
    assert losses[-1] < losses[0]
    torch.testing.assert_close(torch.as_tensor(out[0][1]), torch.as_tensor(out[1][1]), atol=0, rtol=0)


def _tp_worker(rank, world, name, sequence_parallel=False):
    import torch.distributed as dist

    from zen_repro_b200.models.sharding import shard_state_dict

    torch.manual_seed(0)
    cfg = get_config(name)
    full = build_model(cfg, dtype=torch.float32)
    ids = torch.randint(0, cfg.vocab_size, (2, 16))
    want = full(ids, ids)
    want.backward()
    g = dist.group.WORLD
    sh = build_model(cfg, tp_group=g, dtype=torch.float32)
    sh.load_state_dict(shard_state_dict(full.state_dict(), cfg, rank, world))
    if sequence_parallel:
        sh.enable_sequence_parallel()
    got = sh(ids, ids)
    got.backward()
    sh.sync_replicated_grads()
    gfull = shard_state_dict({k: p.grad for k, p in full.named_parameters()}, cfg, rank, world)
    errs = {k: float((p.grad - gfull[k]).abs().max()) for k, p in sh.named_parameters()}
    logits = sh(ids)
    ref_logits = full(ids)
    return float(want.detach()), float(got.detach()), max(errs.values()), float((logits - ref_logits).abs().max())


@pytest.mark.parametrize("name", ["tiny-llama", "tiny-gpt2", "tiny-gemma"])
def test_tensor_parallel_matches_single_rank(name):
    for want, got, gerr, lerr in run_gloo(_tp_worker, 2, name):
        assert got == pytest.approx(want, rel=1e-5, abs=1e-5)
        assert gerr < 1e-4
        assert lerr < 1e-4


@pytest.mark.parametrize("name", ["tiny-llama", "tiny-gpt2", "tiny-gemma"])
def test_sequence_parallel_matches_single_rank(name):
    """Residual stream sharded over the tokens of the TP group: all-gather before the column-parallel projections,
    reduce-scatter after the row-parallel ones, partial norm / bias gradients summed over the group."""
    for want, got, gerr, lerr in run_gloo(_tp_worker, 2, name, True):
        assert got == pytest.approx(want, rel=1e-5, abs=1e-5)
        assert gerr < 1e-4
        assert lerr < 1e-4


def _mesh_worker(rank, world):
    from zen_repro_b200.parallel.mesh import ProcessGroupMesh

    m = ProcessGroupMesh(tp_size=2)
    return m.dp_rank, m.tp_rank, m.get_ranks_in_group(m.dp_group), m.get_ranks_in_group(m.tp_group)


def test_mesh_groups():
    res = run_gloo(_mesh_worker, 4)
    assert res[0] == (0, 0, [0, 2], [0, 1])
    assert res[3] == (1, 1, [1, 3], [2, 3])


def _heartbeat_worker(rank, world):
    import time

    import torch.distributed as dist

    from zen_repro_b200.parallel.failure import Heartbeat, PeerLost

    hb = Heartbeat(interval=0.05, timeout=0.6)
    dist.barrier()
    assert hb.lost() == []
    x = torch.ones(4)
    dist.all_reduce(x)                          # a step with everybody present
    if rank == world - 1:
        hb.stop()                               # leaves between steps: nothing of its own is in flight
        time.sleep(2.5)                         # stays around so that the others' store reads keep working
        return "left"
    t0 = time.monotonic()
    while time.monotonic() - t0 < 5.0:
        try:
            hb.assert_alive()                   # what the trainer does before every step
        except PeerLost as e:
            return e.ranks                      # noticed on the host; the next collective is never launched
        time.sleep(0.05)
    return "not noticed"


def test_heartbeat_names_the_rank_that_left_between_steps():
    res = run_gloo(_heartbeat_worker, 3)
    assert res[2] == "left"
    assert res[0] == [2] and res[1] == [2]


def test_gradient_accumulation_over_micro_batches_with_no_sync():
    """Two micro-batches under ``no_sync`` and a third with synchronisation: the bucket views hold the sum of all three
    (the first writer after ``zero_grad`` overwrites, every later writer accumulates)."""
    from zen_repro_b200.parallel.reducer import ZenDDP

    torch.manual_seed(0)
    a = build_model("tiny-llama", dtype=torch.float32)
    b = build_model("tiny-llama", dtype=torch.float32)
    b.load_state_dict(a.state_dict())
    batches = [torch.randint(0, 1000, (2, 16)) for _ in range(3)]
    for ids in batches:
        a(ids, ids).backward()
    ddp = ZenDDP(b, None, 0.05, None)
    ddp.zero_grad()
    with ddp.no_sync():
        for ids in batches[:2]:
            ddp(ids, ids).backward()
    ddp(batches[2], batches[2]).backward()
    ddp.finalize_grads()
    for (n, p), q in zip(a.named_parameters(), b.parameters()):
        torch.testing.assert_close(q.grad, p.grad, atol=1e-5, rtol=1e-4, msg=lambda m, n=n: f"{n}: {m}")


def _verify_worker(rank, world):
    import torch.distributed as dist

    from zen_repro_b200.parallel.hooks import verified_or_dense

    x = torch.full((8,), float(rank + 1))
    wrong = torch.zeros(8)                                     # what a sparse call that lost records might return
    stats = {}
    ok = verified_or_dense(wrong.clone(), 0, x, None, stats)   # clean status everywhere: the sparse result stands
    bad = verified_or_dense(wrong.clone(), 4 if rank == 1 else 0, x, None, stats)   # one rank timed out: all fall back
    return ok.tolist(), bad.tolist(), stats


def test_hook_recovery_agrees_on_the_status_and_falls_back_to_dense():
    res = run_gloo(_verify_worker, 3)
    for ok, bad, stats in res:
        assert ok == [0.0] * 8
        assert bad == [6.0] * 8                                # 1 + 2 + 3 on every rank, also on those that saw no error
        assert stats["last_status"] == 4 and stats["fallbacks"] == 1


def _dense_by_density_worker(rank, world):
    from zen_repro_b200.parallel.hooks import make_zen_comm_hook
    from zen_repro_b200.parallel.reducer import GradBucket

    torch.manual_seed(rank)
    out = {}
    for top_k in (1, 30):
        hook = make_zen_comm_hook(None, None, top_k=top_k, method=3, torch_future=False)
        x = torch.randn(70000)
        thr = x.abs().kthvalue(int(x.numel() * (1 - top_k / 100.0))).values
        res = hook(None, GradBucket(0, x.clone(), [], True)).wait()
        out[top_k] = (bool(hook.state["dense_by_density"]), round(hook.state["expected_union"], 4), res.clone())
    return out


def test_hook_hands_dense_unions_to_the_dense_allreduce():
    """Three ranks: at top_k 1 % the union of the selections is about 3 % and the bucket takes the sparse exchange; at
    30 % it is 66 %, past the break-even measured against the dense all-reduce, and the thresholded bucket is summed
    densely.  Either way every rank gets the same sum of (approximately) its top fraction of entries."""
    res = run_gloo(_dense_by_density_worker, 3)
    for r in res:
        assert r[1][0] is False and r[1][1] == pytest.approx(0.0297, abs=1e-4)
        assert r[30][0] is True and r[30][1] == pytest.approx(0.657, abs=1e-3)
    for k in (1, 30):
        a = torch.as_tensor(res[0][k][2])
        for r in res[1:]:
            torch.testing.assert_close(torch.as_tensor(r[k][2]), a, atol=1e-6, rtol=1e-6)
        frac = float((a != 0).float().mean())
        assert 0.5 * res[0][k][1] < frac < 1.6 * res[0][k][1]       # sampled thresholds: about the expected union


def _tp_dp_worker(rank, world, sparse_tp):
    from zen_repro_b200.trainer import TrainConfig, Trainer

    t = Trainer(TrainConfig(model="tiny-llama", micro_batch=2, seq_len=16, precision="fp32", lr=1e-2, data_pool=0, tp=2,
                            sparse_embedding=True, sparse_embedding_under_tp=sparse_tp, bucket_cap_mb=0.05), init_dist=False)
    m = t.model.unwrap()
    assert (m.sparse_sink is not None) == sparse_tp and bool(getattr(m.wte, "zen_sparse_only", False)) == sparse_tp
    losses = [t.step(next(t.data)) for _ in range(4)]
    if sparse_tp:
        assert int(m.sparse_sink.last_count) > 0           # rows went through the sparse sink
    w = m.wte.detach().clone()
    return losses, w


def test_vocab_sharded_embedding_rows_sync_sparsely_over_dp_under_tp():
    """TP = 2 x DP = 2 on four CPU ranks: the gradient of the vocabulary-sharded embedding travels over the DP group
    as sparse rows and training follows the dense synchronisation of the same run."""
    sparse = run_gloo(_tp_dp_worker, 4, True)
    dense = run_gloo(_tp_dp_worker, 4, False)
    for r in range(4):
        assert sparse[r][0] == pytest.approx(dense[r][0], rel=1e-5, abs=1e-5)
        torch.testing.assert_close(torch.as_tensor(sparse[r][1]), torch.as_tensor(dense[r][1]), atol=1e-6, rtol=1e-5)
    # the two DP replicas of a TP coordinate hold the same embedding shard
    torch.testing.assert_close(torch.as_tensor(sparse[0][1]), torch.as_tensor(sparse[2][1]), atol=0, rtol=0)
