import pytest
import torch
from hypothesis import given, settings, strategies as st

from zen_repro_b200.sparse import torch_pipeline as tp
from _dist_util import run_gloo


def make_sparse(n, density, seed, dtype=torch.float32, zipf=None):
    g = torch.Generator().manual_seed(seed)
    k = max(1, int(n * density))
    if zipf:
        w = 1.0 / torch.arange(1, n + 1, dtype=torch.float64) ** zipf
        idx = torch.multinomial(w, k, replacement=False, generator=g)
    else:
        idx = torch.randperm(n, generator=g)[:k]
    x = torch.zeros(n, dtype=torch.float32)
    x[idx] = torch.randn(k, generator=g)
    return x.to(dtype)


@settings(max_examples=25, deadline=None)
@given(st.integers(1, 5000), st.integers(1, 8), st.sampled_from([1, 2, 3]), st.floats(0.0, 0.6))
def test_simulate_equals_dense_sum(n, p, method, density):
    xs = [make_sparse(n, density, seed=r) if density > 0 else torch.zeros(n) for r in range(p)]
    want = torch.stack(xs).sum(0)
    for got in tp.simulate(xs, method=method):
        torch.testing.assert_close(got, want, atol=1e-5, rtol=0)


def test_index_zero_and_awkward_sizes():
    for n, p in [(1, 2), (7, 8), (2999999 // 64, 8), (4097, 3)]:
        xs = [torch.zeros(n) for _ in range(p)]
        for r in range(p):
            xs[r][0] = r + 1.0
            xs[r][n - 1] += 0.5
        want = torch.stack(xs).sum(0)
        for m in (1, 2, 3):
            torch.testing.assert_close(tp.simulate(xs, method=m)[0], want)


def _worker(rank, world, n, density, method, dtype_name):
    import torch.distributed as dist

    dtype = getattr(torch, dtype_name)
    x = make_sparse(n, density, seed=rank, dtype=dtype, zipf=1.1)
    got = tp.dist_sparse_allreduce(x, method=method)
    want = x.clone().float()
    dist.all_reduce(want)
    return float((got.float() - want).abs().max())


@pytest.mark.parametrize("method", [1, 2, 3])
def test_gloo_two_ranks_zipf_one_percent(method):
    # 2**20 fp32 elements per rank, 1 % nonzeros at Zipf(1.1) positions (seed = rank), values N(0,1):
    # hash-partition -> all-to-all -> reduce -> all-gather must equal the dense all-reduce sum.
    errs = run_gloo(_worker, 2, 1 << 20, 0.01, method, "float32")
    assert max(errs) <= 1e-5


def test_gloo_four_ranks_bf16():
    errs = run_gloo(_worker, 4, 100003, 0.05, 3, "bfloat16")
    assert max(errs) <= 0.07      # one bf16 rounding of a sum of up to four N(0,1) values


def _emul_worker(rank, world, faults, density, max_density):
    import torch.distributed as dist

    from zen_repro_b200.sparse.emulated import EmulatedSparseAllReduce

    n = 1 << 14
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.zeros(n)
    idx = torch.randperm(n, generator=g)[: int(n * density)]
    x[idx] = torch.randn(idx.numel(), generator=g)
    want = x.clone()
    dist.all_reduce(want)
    eng = EmulatedSparseAllReduce(n, None, max_density=max_density, wait_s=0.6, faults=faults)
    got = eng(x, method=3)
    again = eng(x, method=2)                              # the next call starts from a clean epoch
    return (float((got - want).abs().max()), eng.last_status if faults else 0, float((again - want).abs().max()),
            eng.last_fallback)


def test_emulated_push_protocol_matches_dense_sum():
    from _dist_util import run_gloo

    for err, status, err2, fb in run_gloo(_emul_worker, 3, None, 0.01, 0.12):
        assert err < 1e-5 and err2 < 1e-5 and status == 0 and not fb


@pytest.mark.parametrize("faults,bit", [({"mute": [1]}, 4), ({"short": [2]}, 8), ({"slow": {0: 1.5}}, 4)])
def test_emulated_faults_raise_status_bits_and_fall_back_to_dense(faults, bit):
    """A peer that never pushes (or pushes late) makes the bounded waits expire (bit 4); a mail that claims fewer
    records than were sent is flagged as loss at a peer (bit 8).  Every rank sees the agreed status and returns the
    dense all-reduce instead, so the result is still the exact sum."""
    from _dist_util import run_gloo

    res = run_gloo(_emul_worker, 3, faults, 0.01, 0.12)
    for err, status, err2, fb in res:
        assert status & bit, (status, bit)
        assert fb and err < 1e-5 and err2 < 1e-5


def test_emulated_capacity_overflow_is_reported_not_written_past_the_inbox():
    from _dist_util import run_gloo

    # 20 % non-zeros against inboxes sized for 1 %: senders truncate and flag, receivers learn of it through the mail
    res = run_gloo(_emul_worker, 2, {"none": []}, 0.2, 0.01)
    for err, status, err2, fb in res:
        assert status & (1 | 8) and fb and err < 1e-5
