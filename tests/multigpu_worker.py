"""Worker run under torchrun by tests/test_multigpu.py (one process per GPU).  Prints ``OK <name>`` per check."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def make_sparse(n, density, seed, dtype, dev):
    g = torch.Generator().manual_seed(seed)
    k = max(1, int(n * density))
    idx = torch.randperm(n, generator=g)[:k]
    x = torch.zeros(n)
    x[idx] = torch.randn(k, generator=g)
    return x.to(dtype).to(dev)


def check_sparse_allreduce(rank, world, dev):
    from zen_repro_b200.sparse.engine import SparseAllReduce

    for n, dtype in [(300007, torch.float32), (1 << 22, torch.bfloat16)]:
        eng = SparseAllReduce(n, None, max_density=0.2, methods=(1, 2, 3), deterministic=True)
        for rep in range(3):
            x = make_sparse(n, 0.02 * (rep + 1), 100 * rep + rank, dtype, dev)
            want = x.clone().float()
            dist.all_reduce(want)
            for method in (1, 2, 3, "auto"):
                out = eng(x, method=method)
                st = eng.check()
                assert st == 0, (method, st)
                tol = 1e-5 if dtype == torch.float32 else 0.05
                err = (out.float() - want).abs().max().item()
                assert err <= tol, (n, dtype, method, err)
        eng.close()
    print(f"OK sparse_allreduce rank{rank}", flush=True)


def check_row_engine(rank, world, dev):
    from zen_repro_b200.sparse.row_engine import RowSparseAllReduce

    vocab, d, max_rows = 50257, 768, 4096
    eng = RowSparseAllReduce(vocab, d, max_rows, None, dtype=torch.bfloat16)
    for rep in range(2):
        g = torch.Generator().manual_seed(10 * rep + rank)
        n = 2000 + 100 * rank
        ids = torch.randperm(vocab, generator=g)[:n].sort().values.to(torch.int32)
        rows = torch.zeros(max_rows, dtype=torch.int32); rows[:n] = ids
        vals = torch.zeros(max_rows, d); vals[:n] = torch.randn(n, d, generator=g)
        rows, vals = rows.to(dev), vals.bfloat16().to(dev)
        cnt = torch.tensor([n], dtype=torch.int32, device=dev)
        dense = torch.zeros(vocab, d, device=dev)
        dense.index_add_(0, rows[:n].long(), vals[:n].float())
        dist.all_reduce(dense)
        grad = torch.zeros(vocab, d, dtype=torch.bfloat16, device=dev)
        eng(rows, cnt, vals, grad, scale=1.0)
        assert eng.check() == 0
        err = (grad.float() - dense).abs().max().item()
        assert err < 0.1, err
    eng.close()
    print(f"OK row_engine rank{rank}", flush=True)


def check_trainer_dp(rank, world, dev):
    from zen_repro_b200.trainer import TrainConfig, Trainer

    losses = {}
    for sparse in (True, False):
        torch.manual_seed(0)
        t = Trainer(TrainConfig(model="gpt2", num_layers=2, micro_batch=2, seq_len=128, sparse_embedding=sparse, lr=1e-3,
                                data_pool=0), init_dist=False)
        losses[sparse] = [t.step(next(t.data)) for _ in range(6)]
        if sparse:
            assert t.model.module.embedding_sync.check() == 0
    a, b = losses[True], losses[False]
    assert all(abs(x - y) < 0.05 for x, y in zip(a, b)), (a, b)
    assert a[-1] < a[0]
    print(f"OK trainer_dp rank{rank} {a[0]:.3f}->{a[-1]:.3f}", flush=True)


def check_zen_hook(rank, world, dev):
    from zen_repro_b200.trainer import TrainConfig, Trainer

    t = Trainer(TrainConfig(model="tiny-llama", micro_batch=2, seq_len=32, method=3, top_k=10, lr=1e-2, data_pool=0,
                            bucket_cap_mb=0.1), init_dist=False)
    ls = [t.step(next(t.data)) for _ in range(8)]
    assert ls[-1] < ls[0], ls
    m = t.collect_metrics()                      # counters of the last step's sparse all-reduces, the same on every rank
    assert m["recoveries"] == 0 and m["buckets"], m
    for b in m["buckets"].values():
        assert 0.0 < b["density_sent"] <= 0.35 and b["union_density"] >= b["density_sent"] * 0.5
        assert 1.0 <= b["partition_max_over_mean"] < 3.0 and b["calls"] >= 7
    print(f"OK zen_hook rank{rank} {ls[0]:.3f}->{ls[-1]:.3f}", flush=True)


def check_departed_rank(rank, world, dev):
    """A rank that stops taking part between steps: the others' next sparse all-reduce must return a TIMEOUT
    status within its bound (no hang, context usable afterwards)."""
    from zen_repro_b200.sparse import engine as E

    n = 100000
    eng = E.SparseAllReduce(n, None, max_density=0.2, wait_ms=300.0)
    x = make_sparse(n, 0.01, rank, torch.float32, dev)
    eng(x, method=3)
    assert eng.check() == 0
    dist.barrier()
    torch.cuda.synchronize()
    if rank == world - 1:
        print(f"OK departed_rank rank{rank} (leaving)", flush=True)
    else:
        eng(x, method=3)                       # the last rank never launches this step
        st = eng.check()
        assert st & E.ST_TIMEOUT, st
        assert float(torch.ones(8, device=dev).sum()) == 8.0
        print(f"OK departed_rank rank{rank} status={st}", flush=True)
    torch.cuda.synchronize()
    dist.barrier()                             # everybody is idle again before anyone frees peer-mapped memory
    eng.close()


def check_gemm_allreduce(rank, world, dev):
    """GEMM with the all-reduce fused into its epilogue == GEMM followed by an NCCL all-reduce, on every rank."""
    from zen_repro_b200.ops import gemm as G
    from zen_repro_b200.parallel.tp_fused import FusedTPWorkspace

    ws = FusedTPWorkspace(None, 4096, 4096, wait_ms=1000.0)
    for (M, N, K) in [(256, 384, 320), (4096, 768, 1536), (1000, 4096, 512), (77, 130, 72)]:
        for rep in range(3):
            g = torch.Generator().manual_seed(1000 * rep + rank)
            a = torch.randn(M, K, generator=g).bfloat16().to(dev)
            w = torch.randn(N, K, generator=g).bfloat16().to(dev)
            bias = torch.randn(N, generator=torch.Generator().manual_seed(7)).bfloat16().to(dev)
            got = ws.gemm_ar_nt(a, w, bias)
            want = (a.float() @ w.float().t())
            dist.all_reduce(want)
            want = want + bias.float()
            assert ws.check() == 0 and G.gemm_error() == 0
            err = (got.float() - want).abs().max().item()
            assert err <= 0.02 * want.abs().max().item() + 0.05, (M, N, K, err)
            # every rank holds the same bits
            ref = got.clone()
            dist.broadcast(ref, 0)
            assert torch.equal(ref, got)
            wt = w.t().contiguous()
            got2 = ws.gemm_ar_nn(a, wt)
            assert (got2.float() + bias.float() - want).abs().max().item() <= 0.02 * want.abs().max().item() + 0.1
    ws.close()
    print(f"OK gemm_allreduce rank{rank}", flush=True)


def check_gemm_rs_ag(rank, world, dev):
    """GEMM fused with a reduce-scatter of its output rows, and with an all-gather of its input rows, against NCCL."""
    from zen_repro_b200.ops import gemm as G
    from zen_repro_b200.parallel.tp_fused import FusedTPWorkspace

    ws = FusedTPWorkspace(None, 4096, 4096, wait_ms=1000.0)
    for (M, N, K) in [(256, 384, 320), (4096, 768, 1536), (2048, 4096, 512), (512, 130, 72)]:
        for rep in range(3):
            g = torch.Generator().manual_seed(2000 * rep + rank)
            a = torch.randn(M, K, generator=g).bfloat16().to(dev)
            w = torch.randn(N, K, generator=g).bfloat16().to(dev)
            bias = torch.randn(N, generator=torch.Generator().manual_seed(9)).bfloat16().to(dev)
            # reduce-scatter: this rank's rows of the summed product
            assert ws.fits_rs(M, N)
            got = ws.gemm_rs_nt(a, w, bias)
            full = a.float() @ w.float().t()
            dist.all_reduce(full)
            rpr = M // world
            want = full[rank * rpr:(rank + 1) * rpr] + bias.float()
            assert ws.check() == 0 and G.gemm_error() == 0
            assert got.shape == (rpr, N)
            assert (got.float() - want).abs().max().item() <= 0.02 * want.abs().max().item() + 0.05, ("rs", M, N, K)
            got_nn = ws.gemm_rs_nn(a, w.t().contiguous())
            assert (got_nn.float() + bias.float() - want).abs().max().item() <= 0.02 * want.abs().max().item() + 0.1
            # all-gather of the input rows, then the product with this rank's own weight
            assert ws.fits_ag(M, K)
            rows = [torch.empty_like(a) for _ in range(world)]
            dist.all_gather(rows, a)
            want2 = torch.cat(rows).float() @ w.float().t() + bias.float()
            got2 = ws.ag_gemm_nt(a, w, bias)
            assert ws.check() == 0 and G.gemm_error() == 0
            assert got2.shape == (world * M, N)
            assert (got2.float() - want2).abs().max().item() <= 0.02 * want2.abs().max().item() + 0.05, ("ag", M, N, K)
            got3 = ws.ag_gemm_nn(a, w.t().contiguous())
            assert (got3.float() + bias.float() - want2).abs().max().item() <= 0.02 * want2.abs().max().item() + 0.1
    ws.close()
    print(f"OK gemm_rs_ag rank{rank}", flush=True)


def check_tp_trainer(rank, world, dev):
    """TP = 2 training with fused GEMM + all-reduce tracks the NCCL-based TP path."""
    from zen_repro_b200.trainer import TrainConfig, Trainer

    out = {}
    for fused in (True, False):
        t = Trainer(TrainConfig(model="meta-llama/Llama-3.2-3B", num_layers=2, micro_batch=1, seq_len=256, tp=2, lr=1e-4,
                                data_pool=0, fused_tp=fused), init_dist=False)
        out[fused] = [t.step(next(t.data)) for _ in range(4)]
    assert all(abs(a - b) < 0.05 for a, b in zip(out[True], out[False])), out
    print(f"OK tp_trainer rank{rank} {out[True]}", flush=True)


def check_sp_trainer(rank, world, dev):
    """TP = 2 with the residual stream sharded over tokens (all-gather + GEMM, GEMM + reduce-scatter kernels) tracks
    the all-reduce form of the same model."""
    from zen_repro_b200.trainer import TrainConfig, Trainer

    out = {}
    for sp in (True, False):
        t = Trainer(TrainConfig(model="meta-llama/Llama-3.2-3B", num_layers=2, micro_batch=1, seq_len=256, tp=2, lr=1e-4,
                                data_pool=0, fused_tp=True, sequence_parallel=sp), init_dist=False)
        out[sp] = [t.step(next(t.data)) for _ in range(4)]
        ws = t.model.unwrap().tp_ws
        assert ws is None or ws.check() == 0
    assert all(abs(a - b) < 0.05 for a, b in zip(out[True], out[False])), out
    print(f"OK sp_trainer rank{rank} {out[True]}", flush=True)


def check_sparse_back_to_back(rank, world, dev):
    """Eight calls on ONE engine with no host synchronisation or collective in between, method 1 and the balanced
    methods mixed, while the last rank is held back by a finite sleep before each of its consumers: a fast rank is then
    a whole call ahead of the slow one, which is safe only because record slots and their mails alternate with the
    call parity.  Guard words around the sub-regions must survive."""
    from zen_repro_b200.sparse.engine import SparseAllReduce

    n = 1 << 20
    eng = SparseAllReduce(n, None, max_density=0.1, methods=(1, 2, 3), deterministic=True, wait_ms=5000.0)
    xs = [make_sparse(n, 0.01 + 0.004 * i, 1000 * i + rank, torch.float32, dev) for i in range(8)]
    methods = [1, 1, 3, 1, 2, 1, 1, "auto"]
    outs = []
    rs = eng.rank_state
    torch.cuda.synchronize(); dist.barrier()
    for i, (x, m) in enumerate(zip(xs, methods)):
        out = torch.empty_like(x)
        eng.epoch += 1
        e = eng.epoch
        if m == 1:
            rs.partition_push(x, e, None, broadcast=True)
            if rank == world - 1:
                torch.cuda._sleep(20_000_000)                 # about 10 ms: the peers finish this call and push the next
            rs.scatter_sources(out, e)
        else:
            from zen_repro_b200.sparse.engine import _fmt_for

            rs.partition_push(x, e, None)
            if rank == world - 1:
                torch.cuda._sleep(20_000_000)
            rs.owner_reduce(e, x.dtype, True)
            rs.gather_push(e, x.dtype, _fmt_for(m))
            rs.densify(out, e, _fmt_for(m))
        outs.append(out)
    torch.cuda.synchronize()
    assert eng.check() == 0
    for x, out in zip(xs, outs):
        want = x.clone()
        dist.all_reduce(want)
        assert torch.equal(out, want) or (out - want).abs().max().item() <= 1e-5, (out - want).abs().max().item()
    assert rs.damaged_canaries() == []
    dist.barrier()
    eng.close()
    print(f"OK sparse_back_to_back rank{rank}", flush=True)


def check_sparse_nvls(rank, world, dev):
    """Gather push through the multicast alias (one multimem store, replicated by the NVSwitch) against the dense sum."""
    from zen_repro_b200.sparse.engine import SparseAllReduce

    n = 1 << 22
    eng = SparseAllReduce(n, None, max_density=0.2, methods=(2, 3), transport="nvls")
    if eng.transport != "nvls":
        print(f"OK sparse_nvls rank{rank} (no multicast on this fabric: plain peer stores were used)", flush=True)
    for rep in range(2):
        x = make_sparse(n, 0.03 * (rep + 1), 7 * rep + rank, torch.float32, dev)
        want = x.clone().float()
        dist.all_reduce(want)
        for method in (3, 2, "auto"):
            out = eng(x, method=method)
            assert eng.check() == 0
            assert (out.float() - want).abs().max().item() <= 1e-5
    assert eng.rank_state.damaged_canaries() == []
    dist.barrier()
    eng.close()
    print(f"OK sparse_nvls rank{rank} transport={eng.transport}", flush=True)


def check_verify_fallback(rank, world, dev):
    """``verify=True`` of the hook with a failure made on the host: the last rank does not launch its push for one
    bucket.  Every rank must see the expired wait (its own or a peer's, through the agreed status), fall back, and
    return the exact dense sum of the thresholded buckets."""
    from zen_repro_b200.parallel.hooks import make_zen_comm_hook
    from zen_repro_b200.parallel.reducer import GradBucket
    from zen_repro_b200.sparse.engine import SparseAllReduce

    n = 200000
    eng = SparseAllReduce(n, None, max_density=0.3, methods=(1, 2, 3), wait_ms=300.0)
    hook = make_zen_comm_hook(None, None, top_k=100, method=3, engines={n: eng}, torch_future=False, verify=True,
                              dense_above=2.0)                  # keep the bucket on the sparse engine whatever top_k says
    x = make_sparse(n, 0.05, rank, torch.float32, dev)
    want = x.clone()
    dist.all_reduce(want)
    out = hook(None, GradBucket(0, x.clone(), [], True)).wait()
    assert hook.state.get("fallbacks", 0) == 0 and (out - want).abs().max().item() <= 1e-5
    # the failure: this rank's kernels of the next call are not launched (the engine call is replaced by a no-op)
    if rank == world - 1:
        eng.rank_state.allreduce = lambda x_, out_, *a, **k: out_.zero_()
    out = hook(None, GradBucket(0, x.clone(), [], True)).wait()
    assert hook.state["fallbacks"] == 1 and hook.state["last_status"] != 0
    assert (out - want).abs().max().item() <= 1e-5, (out - want).abs().max().item()
    assert float(torch.ones(8, device=dev).sum()) == 8.0      # the context is alive
    torch.cuda.synchronize()
    dist.barrier()
    eng.close()
    print(f"OK verify_fallback rank{rank} status={hook.state['last_status']}", flush=True)


def check_tp2dp2_sparse_embedding(rank, world, dev):
    """TP 2 x DP 2: the vocabulary-sharded embedding gradient synchronised as sparse rows over the DP group tracks
    the dense synchronisation of the same run."""
    from zen_repro_b200.trainer import TrainConfig, Trainer

    assert world % 4 == 0 or world == 4, "needs four ranks"
    out = {}
    for sparse in (True, False):
        t = Trainer(TrainConfig(model="meta-llama/Llama-3.2-3B", num_layers=2, micro_batch=1, seq_len=256, tp=2, lr=1e-4,
                                data_pool=0, sparse_embedding_under_tp=sparse), init_dist=False)
        assert (t.model.module.embedding_sync is not None) == sparse
        out[sparse] = [t.step(next(t.data)) for _ in range(4)]
        assert not t.check_health(raise_on_error=False) or not any(t.check_health(raise_on_error=False).values())
        w = t.model.unwrap().wte.detach().float()
        out[("w", sparse)] = w
        t.close()
    assert all(abs(a - b) < 0.02 for a, b in zip(out[True], out[False])), out
    assert (out[("w", True)] - out[("w", False)]).abs().max().item() < 2e-3
    print(f"OK tp2dp2_sparse_embedding rank{rank} {out[True]}", flush=True)


def check_nvls_dense_allreduce(rank, world, dev):
    """The multimem all-reduce kernel against the NCCL all-reduce: bf16 and fp32 ranges of one arena, several calls in a
    row without host synchronisation, the mean folded in; then a trainer whose dense buckets go through it against the
    same run on NCCL."""
    from zen_repro_b200.parallel.nvls_allreduce import MulticastArena
    from zen_repro_b200.trainer import TrainConfig, Trainer

    try:
        arena = MulticastArena(64 << 20, None, wait_ms=5000.0)
    except RuntimeError as ex:
        print(f"OK nvls_dense rank{rank} (skipped: {ex})", flush=True)
        return
    g = torch.Generator().manual_seed(50 + rank)
    cases = [(0, 1 << 20, torch.bfloat16), (4 << 20, 3 * 1000 * 8, torch.float32), (16 << 20, (1 << 22) + 8, torch.bfloat16)]
    wants, views = [], []
    for off, n, dt in cases:
        v = arena.view(off, n, dt)
        v.copy_(torch.randn(n, generator=g).to(dt))
        want = v.float().clone()
        dist.all_reduce(want)
        wants.append(want / world)
        views.append(v)
    torch.cuda.synchronize(); dist.barrier()
    for (off, n, dt), v in zip(cases, views):
        arena.allreduce_(off, n * v.element_size(), dt, 1.0 / world)
    torch.cuda.synchronize()
    assert arena.check() == 0
    for v, want, (_, _, dt) in zip(views, wants, cases):
        tol = 2e-2 if dt == torch.bfloat16 else 1e-5
        assert (v.float() - want).abs().max().item() <= tol * max(1.0, want.abs().max().item()), dt
        ref = v.clone()
        dist.broadcast(ref, 0)
        assert torch.equal(ref, v)                       # every rank holds the same bits
    losses = {}
    for tr in ("nvls", "nccl"):
        t = Trainer(TrainConfig(model="gpt2", num_layers=2, micro_batch=2, seq_len=128, lr=1e-3, data_pool=4, dense_transport=tr,
                                cuda_graph=True, graph_warmup=2), init_dist=False)
        assert (t.model.module.arena is not None) == (tr == "nvls")
        losses[tr] = [t.step(next(t.data)) for _ in range(6)]
        assert not any(t.check_health(raise_on_error=False).values())
        t.close()
    assert all(abs(a - b) < 0.03 for a, b in zip(losses["nvls"], losses["nccl"])), losses
    print(f"OK nvls_dense rank{rank} {losses['nvls'][0]:.3f}->{losses['nvls'][-1]:.3f}", flush=True)


def check_sample_exchange(rank, world, dev):
    """Threshold samples exchanged through peer memory equal an NCCL all-gather, five calls in a row without host
    synchronisation; the TP-aware threshold is then the same number on every rank of the group."""
    from zen_repro_b200.parallel.hooks import SampleExchange, sampled_threshold

    ns = 3001
    ex = SampleExchange(None, ns, dev, wait_ms=5000.0)
    xs = [torch.rand(ns, generator=torch.Generator().manual_seed(10 * i + rank)).to(dev) for i in range(5)]
    got = [ex(x).clone() for x in xs]
    torch.cuda.synchronize()
    assert int(ex.status.item()) == 0
    for x, g in zip(xs, got):
        want = torch.empty(world * ns, device=dev)
        dist.all_gather_into_tensor(want, x)
        assert torch.equal(g, want)
    t = torch.randn(200000, generator=torch.Generator().manual_seed(rank)).to(dev).bfloat16()
    thr = sampled_threshold(t, 1.0, group=dist.group.WORLD).clone()
    every = [torch.empty_like(thr) for _ in range(world)]
    dist.all_gather(every, thr)
    assert all(torch.equal(e, every[0]) for e in every) and float(thr) > 0
    dist.barrier()
    ex.region.close()
    print(f"OK sample_exchange rank{rank} thr={float(thr):.4f}", flush=True)


CHECKS = {"samples": check_sample_exchange, "nvls_dense": check_nvls_dense_allreduce, "b2b": check_sparse_back_to_back, "nvls": check_sparse_nvls, "verify": check_verify_fallback,
          "tp2dp2": check_tp2dp2_sparse_embedding, "gemm_ar": check_gemm_allreduce, "sp_trainer": check_sp_trainer, "gemm_rs_ag": check_gemm_rs_ag, "tp_trainer": check_tp_trainer,"sparse": check_sparse_allreduce, "rows": check_row_engine, "trainer": check_trainer_dp,
          "hook": check_zen_hook, "departed": check_departed_rank}

if __name__ == "__main__":
    from zen_repro_b200.parallel import launch_from_torch

    rank, world, dev = launch_from_torch()
    names = sys.argv[1:] or list(CHECKS)
    for nme in names:
        CHECKS[nme](rank, world, dev)
        dist.barrier()
    dist.destroy_process_group()
