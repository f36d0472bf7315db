import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("P", [1, 2, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("vocab,d", [(50257, 768), (1000, 64), (256000, 256)])
def test_row_sparse_allreduce_matches_oracle(P, dtype, vocab, d):
    from zen_repro_b200.sparse import row_engine as R

    dev = "cuda"
    max_rows = 2048
    eng = R.VirtualRowSparseAllReduce(vocab, d, max_rows, P, dtype=dtype)
    for rep in range(2):
        rows_l, cnt_l, vals_l = [], [], []
        for r in range(P):
            g = torch.Generator().manual_seed(100 * rep + r)
            w = 1.0 / torch.arange(1, vocab + 1, dtype=torch.float64) ** 1.1
            n = min(vocab // 2, 1500 - 100 * r)
            ids = torch.multinomial(w, n, replacement=False, generator=g).sort().values.to(torch.int32)
            ids[0] = 0 if r == 0 else ids[0]
            rows = torch.zeros(max_rows, dtype=torch.int32); rows[:n] = ids
            vals = torch.zeros(max_rows, d); vals[:n] = torch.randn(n, d, generator=g)
            rows_l.append(rows.to(dev)); cnt_l.append(torch.tensor([n], dtype=torch.int32, device=dev))
            vals_l.append(vals.to(dtype).to(dev))
        grads = [torch.ones(vocab, d, dtype=dtype, device=dev) for _ in range(P)]
        eng(rows_l, cnt_l, vals_l, grads, scale=0.5)
        assert eng.status() == [0] * P
        want = R.rows_oracle(rows_l, cnt_l, vals_l, vocab, d, scale=0.5) + 1.0
        tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=0.06, rtol=0.02)
        for gsum in grads:
            torch.testing.assert_close(gsum.float().cpu(), want, **tol)
