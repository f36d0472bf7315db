"""CUDA sparse all-reduce kernels against the pure-PyTorch oracle (all ranks on one GPU, phase by phase)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def make_sparse(n, density, seed, dtype, device, zipf=None):
    g = torch.Generator().manual_seed(seed)
    k = min(n, max(1, int(n * density))) if density > 0 else 0
    x = torch.zeros(n, dtype=torch.float32)
    if k:
        if zipf:
            w = 1.0 / torch.arange(1, n + 1, dtype=torch.float64) ** zipf
            idx = torch.multinomial(w, k, replacement=False, generator=g)
        else:
            idx = torch.randperm(n, generator=g)[:k]
        x[idx] = torch.randn(k, generator=g)
    return x.to(dtype).to(device)


def dense_sum(xs):
    acc = torch.zeros_like(xs[0], dtype=torch.float32)
    for x in xs:                      # rank order, the order the deterministic reduction uses
        acc += x.float()
    return acc


@pytest.mark.parametrize("P", [1, 2, 4, 8])
@pytest.mark.parametrize("n", [1, 63, 4097, 300007, (1 << 20) + 5])
@pytest.mark.parametrize("method", [1, 2, 3, "auto"])
def test_fp32_matches_dense_sum(P, n, method):
    from zen_repro_b200.sparse.engine import VirtualSparseAllReduce

    dev = torch.device("cuda")
    eng = VirtualSparseAllReduce(n, P, max_density=0.3, methods=(1, 2, 3), deterministic=True)
    for rep, density in enumerate([0.01, 0.2, 0.0]):
        xs = [make_sparse(n, density, seed=17 * r + rep, dtype=torch.float32, device=dev, zipf=1.1 if n > 4097 else None)
              for r in range(P)]
        if n > 1:
            xs[0][0] = 3.0            # position 0 must be transmittable
        outs = eng(xs, method=method)
        assert eng.status() == [0] * P
        want = dense_sum(xs)
        for o in outs:
            torch.testing.assert_close(o, want, atol=0, rtol=0)


@pytest.mark.parametrize("P", [2, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_half_types(P, dtype):
    from zen_repro_b200.sparse.engine import VirtualSparseAllReduce

    n = 500000
    dev = torch.device("cuda")
    eng = VirtualSparseAllReduce(n, P, max_density=0.12, methods=(3,))
    xs = [make_sparse(n, 0.05, seed=r, dtype=dtype, device=dev) for r in range(P)]
    outs = eng(xs, method=3)
    assert eng.status() == [0] * P
    want = dense_sum(xs)
    for o in outs:
        torch.testing.assert_close(o.float(), want, atol=0.05, rtol=0.01)   # one rounding of the fp32 sum


def test_dense_input_takes_the_direct_path_and_stays_correct():
    from zen_repro_b200.sparse.engine import VirtualSparseAllReduce

    n, P = 200000, 4
    dev = torch.device("cuda")
    eng = VirtualSparseAllReduce(n, P, max_density=1.0, methods=(3,), deterministic=True)
    xs = [torch.randn(n, device=dev) for _ in range(P)]
    outs = eng(xs, method=3)
    assert eng.status() == [0] * P
    torch.testing.assert_close(outs[0], dense_sum(xs), atol=1e-5, rtol=0)


def test_threshold_is_applied_in_the_scan():
    from zen_repro_b200.sparse.engine import VirtualSparseAllReduce

    n, P = 100000, 2
    dev = torch.device("cuda")
    eng = VirtualSparseAllReduce(n, P, max_density=1.0, methods=(3,), deterministic=True)
    xs = [torch.randn(n, device=dev) for _ in range(P)]
    thr = torch.tensor([1.5], device=dev)
    outs = eng(xs, method=3, threshold=thr)
    want = dense_sum([torch.where(x.abs() >= 1.5, x, torch.zeros_like(x)) for x in xs])
    torch.testing.assert_close(outs[1], want, atol=1e-6, rtol=0)


def test_overflow_is_reported_not_written_out_of_bounds():
    from zen_repro_b200.sparse import engine as E

    n, P = 400000, 2
    dev = torch.device("cuda")
    eng = E.VirtualSparseAllReduce(n, P, max_density=0.001, methods=(3,))
    xs = [torch.randn(n, device=dev) for _ in range(P)]      # 100 % dense into 0.1 % slots
    eng(xs, method=3)
    st = eng.status()
    assert all(s & (E.ST_REC_OVERFLOW | E.ST_PEER_OVERFLOW | E.ST_GATHER_OVERFLOW) for s in st), st
    # the engine stays usable afterwards
    ys = [make_sparse(n, 0.0005, seed=r, dtype=torch.float32, device=dev) for r in range(P)]
    outs = eng(ys, method=3)
    assert eng.status() == [0] * P
    torch.testing.assert_close(outs[0], dense_sum(ys), atol=1e-6, rtol=0)


def test_bounded_wait_times_out_and_context_survives():
    from zen_repro_b200.sparse import engine as E

    n, P = 10000, 2
    dev = torch.device("cuda")
    eng = E.VirtualSparseAllReduce(n, P, methods=(3,))
    x = make_sparse(n, 0.01, 0, torch.float32, dev)
    eng.epoch += 1
    eng.ranks[0].partition_push(x, eng.epoch)          # rank 1 never pushes: its mail keeps the old epoch
    eng.ranks[0].owner_reduce(eng.epoch, torch.float32)
    st = eng.ranks[0].read_status()
    assert st & E.ST_TIMEOUT
    assert float(torch.ones(4, device=dev).sum()) == 4.0   # context still healthy


def test_owner_map_kernel_matches_python():
    import ctypes
    from zen_repro_b200 import _native
    from zen_repro_b200.sparse.engine import perm_struct
    from zen_repro_b200.sparse.hashing import BlockPermutation, zen_poly3_owner

    n, P = 123457, 8
    dev = torch.device("cuda")
    perm = BlockPermutation.make(n, P, 64)
    out = torch.empty(n, dtype=torch.int32, device=dev)
    ps = perm_struct(perm)
    lib = _native.lib()
    _native.check(lib.zen_owner_map(_native.ptr(out), ctypes.c_uint64(n), ctypes.byref(ps), 0, ctypes.c_uint32(0), P,
                                    _native.stream_ptr()), "owner_map")
    want, _ = perm.owner_slot(torch.arange(n))
    assert torch.equal(out.cpu().long(), want)
    table = n // P * P
    _native.check(lib.zen_owner_map(_native.ptr(out), ctypes.c_uint64(n), ctypes.byref(ps), 1, ctypes.c_uint32(table), P,
                                    _native.stream_ptr()), "owner_map")
    assert torch.equal(out.cpu().long(), zen_poly3_owner(torch.arange(n), table, P))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sampled_threshold_kernels(dtype):
    import ctypes

    from zen_repro_b200 import _native
    from zen_repro_b200.parallel.hooks import sampled_threshold

    dev = torch.device("cuda")
    lib = _native.lib()
    # exact k-th largest against torch.topk
    torch.manual_seed(0)
    v = torch.rand(100003, device=dev) * 5
    hist = torch.zeros(2048, dtype=torch.int32, device=dev)
    state = torch.zeros(2, dtype=torch.int32, device=dev)
    out = torch.empty(1, device=dev)
    for k in (1, 17, 5000, 100003):
        _native.check(lib.zen_select_kth(_native.ptr(v), ctypes.c_uint32(v.numel()), ctypes.c_uint32(k), _native.ptr(hist),
                                         _native.ptr(state), _native.ptr(out), _native.stream_ptr()), "select")
        want = torch.topk(v, k, sorted=True)[0][-1]
        assert float(out) == float(want), (k, float(out), float(want))
        assert int(hist.abs().sum()) == 0
    # the sampled threshold keeps about top_k percent
    g = torch.randn(1 << 21, device=dev).to(dtype)
    thr = sampled_threshold(g, 5)
    frac = float((g.abs().float() >= thr).float().mean())
    assert 0.04 < frac < 0.06, frac
