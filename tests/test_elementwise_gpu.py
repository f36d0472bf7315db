"""Elementwise / normalisation / loss kernels against their PyTorch fp32 restatements."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from zen_repro_b200.ops import elementwise as E  # noqa: E402

DEV = "cuda"


def tol(dtype):
    return dict(atol=2e-2, rtol=2e-2) if dtype != torch.float32 else dict(atol=2e-5, rtol=2e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layer", [False, True])
@pytest.mark.parametrize("rows,cols", [(5, 64), (300, 768), (64, 2048), (33, 4096)])
def test_norm_fwd_bwd(dtype, layer, rows, cols):
    g = torch.Generator().manual_seed(0)
    x = torch.randn(rows, cols, generator=g).to(dtype)
    res = torch.randn(rows, cols, generator=g).to(dtype)
    w = (torch.randn(cols, generator=g) * 0.1 + (0.0 if not layer else 1.0)).to(dtype)
    b = (torch.randn(cols, generator=g) * 0.1).to(dtype) if layer else None
    dy = torch.randn(rows, cols, generator=g).to(dtype)
    dres = torch.randn(rows, cols, generator=g).to(dtype)
    unit = not layer
    y0, h0, r0, m0 = E.norm_fwd(x, w, b, res, eps=1e-6, layer=layer, unit_offset=unit)
    y1, h1, r1, m1 = E.norm_fwd(x.to(DEV), w.to(DEV), b.to(DEV) if b is not None else None, res.to(DEV), eps=1e-6,
                                layer=layer, unit_offset=unit)
    torch.testing.assert_close(h1.cpu().float(), h0.float(), **tol(dtype))
    torch.testing.assert_close(y1.cpu().float(), y0.float(), **tol(dtype))
    torch.testing.assert_close(r1.cpu(), r0, atol=1e-4, rtol=1e-3)
    dh0, dw0, db0 = E.norm_bwd(dy, h0, w, r0, m0, dres, layer=layer, unit_offset=unit, has_bias=layer)
    dh1, dw1, db1 = E.norm_bwd(dy.to(DEV), h1, w.to(DEV), r1, m1, dres.to(DEV), layer=layer, unit_offset=unit,
                               has_bias=layer)
    torch.testing.assert_close(dh1.cpu().float(), dh0.float(), **tol(dtype))
    wt = dict(atol=0.3, rtol=3e-2) if dtype != torch.float32 else dict(atol=1e-3, rtol=1e-4)
    torch.testing.assert_close(dw1.cpu().float(), dw0.float(), **wt)
    if layer:
        torch.testing.assert_close(db1.cpu().float(), db0.float(), **wt)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind", ["gelu_tanh", "relu", "swiglu", "geglu"])
def test_activations(dtype, kind):
    g = torch.Generator().manual_seed(1)
    rows, inner = 77, 1024
    gu = torch.randn(rows, 2 * inner, generator=g).to(dtype)
    dout = torch.randn(rows, inner, generator=g).to(dtype)
    gated = kind in ("swiglu", "geglu")
    a, b = gu[:, :inner], (gu[:, inner:] if gated else None)
    o0 = E.act_fwd(a, b, kind)
    gud = gu.to(DEV)
    ad, bd = gud[:, :inner], (gud[:, inner:] if gated else None)
    o1 = E.act_fwd(ad, bd, kind)
    # the kernels use tanh.approx (relative error about 2^-11), so fp32 is compared at 3e-3
    t = tol(dtype) if dtype != torch.float32 else dict(atol=3e-3, rtol=3e-3)
    torch.testing.assert_close(o1.cpu().float(), o0.float(), **t)
    da0, db0 = E.act_bwd(a, b, dout, kind)
    da1, db1 = E.act_bwd(ad, bd, dout.to(DEV), kind)
    torch.testing.assert_close(da1.cpu().float(), da0.float(), **t)
    if gated:
        torch.testing.assert_close(db1.cpu().float(), db0.float(), **t)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rope_and_inverse(dtype):
    g = torch.Generator().manual_seed(2)
    tokens, heads, hd, seq = 96, 4, 128, 48
    x = torch.randn(tokens, heads, hd, generator=g).to(dtype)
    y0 = E.rope_(x.clone(), seq, 10000.0)
    xd = x.to(DEV)
    y1 = E.rope_(xd.clone(), seq, 10000.0)
    torch.testing.assert_close(y1.cpu().float(), y0.float(), **tol(dtype))
    back = E.rope_(y1.clone(), seq, 10000.0, inverse=True)
    torch.testing.assert_close(back.cpu().float(), x.float(), **tol(dtype))
    # strided view (q inside a fused qkv buffer)
    qkv = torch.randn(tokens, 3 * heads * hd, generator=g).to(dtype).to(DEV)
    q = qkv.view(tokens, 3 * heads, hd)[:, :heads]
    want = E.rope_(q.cpu().contiguous(), seq, 500000.0)
    E.rope_(q, seq, 500000.0)
    torch.testing.assert_close(q.cpu().float(), want.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_fwd_and_row_sparse_bwd(dtype):
    g = torch.Generator().manual_seed(3)
    vocab, d, seq, bsz = 5003, 256, 64, 5
    ids = torch.randint(0, 50, (bsz * seq,), generator=g)
    ids[::7] = torch.randint(0, vocab, (ids[::7].numel(),), generator=g)
    wte = torch.randn(vocab, d, generator=g).to(dtype)
    wpe = torch.randn(seq + 2, d, generator=g).to(dtype)
    o0 = E.embedding_fwd(ids, wte, wpe, seq=seq, pos_offset=2, scale=1.5)
    o1 = E.embedding_fwd(ids.to(DEV), wte.to(DEV), wpe.to(DEV), seq=seq, pos_offset=2, scale=1.5)
    torch.testing.assert_close(o1.cpu().float(), o0.float(), **tol(dtype))
    dy = torch.randn(bsz * seq, d, generator=g).to(dtype)
    r0, c0, v0 = E.embedding_bwd_rows(ids, dy, vocab, scale=0.5)
    for _ in range(2):                                   # second call checks that the scratch was left clean
        sc = E.RowSparseScratch(vocab, d, min(ids.numel(), vocab), dtype, DEV) if _ == 0 else sc
        r1, c1, v1 = E.embedding_bwd_rows(ids.to(DEV), dy.to(DEV), vocab, scale=0.5, scratch=sc)
        n = int(c1.item())
        assert n == int(c0.item())
        assert torch.equal(r1[:n].cpu(), r0)
        torch.testing.assert_close(v1[:n].cpu().float(), v0.float(), **tol(dtype))
    grad = torch.randn(vocab, d, generator=g).to(dtype)
    want = grad.clone().float()
    want.index_add_(0, r0.long(), v0.float())
    gd = grad.to(DEV)
    E.rows_add_(gd, r1, c1, v1)
    torch.testing.assert_close(gd.cpu().float(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("vocab", [50257, 1000, 32000])
def test_cross_entropy(dtype, vocab):
    g = torch.Generator().manual_seed(4)
    rows = 37
    pad = (-vocab) % 8
    buf = (torch.randn(rows, vocab + pad, generator=g) * 3).to(dtype)
    logits = buf[:, :vocab]
    labels = torch.randint(0, vocab, (rows,), generator=g)
    labels[3] = -100
    l0, d0 = E.cross_entropy(logits.clone(), labels, grad_scale=1.0 / rows)
    bd = buf.to(DEV)
    l1, d1 = E.cross_entropy(bd[:, :vocab], labels.to(DEV), grad_scale=1.0 / rows)
    torch.testing.assert_close(l1.cpu(), l0, atol=2e-3, rtol=1e-3)
    torch.testing.assert_close(d1.cpu().float(), d0.float(), atol=1e-3 if dtype != torch.float32 else 1e-6, rtol=2e-2)
    assert float(d1[3].abs().max()) == 0.0


def test_colsum():
    a = torch.randn(1000, 3072).to(torch.bfloat16)
    got = E.colsum(a.to(DEV))
    torch.testing.assert_close(got.cpu().float(), a.float().sum(0), atol=0.3, rtol=2e-2)


@pytest.mark.parametrize("kind", ["gelu_tanh", "relu"])
@pytest.mark.parametrize("rows,inner", [(1000, 3072), (77, 256), (8192, 10240)])
def test_activation_backward_with_column_sums(kind, rows, inner):
    """The activation backward that also leaves the bias gradient of the layer before it: same da as the plain kernel,
    and the column sums of exactly those stored values; the linear layer's backward picks them up from the tensor."""
    torch.manual_seed(3)
    x = torch.randn(rows, inner, device=DEV).bfloat16()
    g = torch.randn(rows, inner, device=DEV).bfloat16()
    want, _ = E.act_bwd(x, None, g, kind)
    da, part = E.act_bwd_with_colsum(x, g, kind)
    assert torch.equal(da, want)
    out = torch.full((inner,), 1.0, device=DEV, dtype=torch.bfloat16)
    E.colsum_from_parts(part, out, accumulate=True)
    torch.testing.assert_close(out.float(), da.float().sum(0) + 1.0, atol=0.3, rtol=2e-2)
    E.colsum_from_parts(part, out, accumulate=False)
    torch.testing.assert_close(out.float(), da.float().sum(0), atol=0.3, rtol=2e-2)


def test_bias_gradient_rides_with_the_activation_backward():
    from zen_repro_b200.ops import autograd as AG
    torch.manual_seed(4)
    x = torch.randn(4, 64, 256, device=DEV).bfloat16()
    w = (torch.randn(512, 256, device=DEV) * 0.05).bfloat16().requires_grad_(True)
    b = torch.zeros(512, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    grads = []
    for fuse in (True, False):
        AG._FUSE_ACT_COLSUM = fuse
        try:
            w.grad = b.grad = None
            y = AG.activation(AG.linear(x, w, b), "gelu_tanh")
            (y.float() ** 2).sum().backward()
            grads.append((w.grad.clone(), b.grad.clone()))
        finally:
            AG._FUSE_ACT_COLSUM = True
    assert torch.equal(grads[0][0], grads[1][0])
    torch.testing.assert_close(grads[0][1].float(), grads[1][1].float(), atol=0.05, rtol=2e-2)
    h = (x.float() @ w.detach().float().t() + b.detach().float()).requires_grad_(True)
    (torch.nn.functional.gelu(h, approximate="tanh") ** 2).sum().backward()
    torch.testing.assert_close(grads[0][1].float(), h.grad.sum((0, 1)), atol=0.5, rtol=5e-2)


def test_queued_column_reductions_go_out_as_one_launch():
    """Reductions of different widths and part counts, one with a second (part, out) pair, one accumulating: the grouped
    kernel gives what the single reductions give, callbacks fire in order after the launch."""
    torch.manual_seed(6)
    specs = [(256, 768, False, False), (256, 3072, True, False), (37, 2304, False, True), (256, 768, True, True), (8, 64, False, False)]
    jobs, fired = [], []
    for i, (parts, cols, acc, pair) in enumerate(specs):
        part = torch.randn(parts, cols, device=DEV)
        out = torch.full((cols,), 0.5, device=DEV, dtype=torch.bfloat16)
        part2 = torch.randn(parts, cols, device=DEV) if pair else None
        out2 = torch.full((cols,), -1.0, device=DEV, dtype=torch.bfloat16) if pair else None
        jobs.append((part, out, acc, part2, out2))
        E._queue_reduce(part, parts, out, acc, (lambda i=i: fired.append(i)), part2, out2)
    assert fired == []
    E.flush_colreduce()
    assert fired == list(range(len(specs)))
    for part, out, acc, part2, out2 in jobs:
        want = part.sum(0) + (0.5 if acc else 0.0)
        torch.testing.assert_close(out.float(), want, atol=0.15, rtol=2e-2)
        if part2 is not None:
            want2 = part2.sum(0) + (-1.0 if acc else 0.0)
            torch.testing.assert_close(out2.float(), want2, atol=0.15, rtol=2e-2)


def test_cuda_graph_step_matches_eager_steps():
    """The captured training step (replayed) follows the same loss trajectory as launching every kernel from the host."""
    from zen_repro_b200.trainer import TrainConfig, Trainer

    def run(graph):
        torch.manual_seed(0)
        t = Trainer(TrainConfig(model="gpt2", num_layers=2, micro_batch=2, seq_len=256, lr=1e-3, data_pool=4, cuda_graph=graph,
                                graph_warmup=2), init_dist=False)
        ids = [next(t.data)["input_ids"].cuda() for _ in range(4)]
        out = [float(t.step_device(i, i, read_loss=True)) for i in ids + ids]
        return out, t

    eager, _ = run(False)
    graph, tg = run(True)
    assert tg._graph is not None and tg.graph_launches_per_step > 20
    assert graph[-1] < graph[0]
    for a, b in zip(eager, graph):
        assert abs(a - b) < 0.05, (eager, graph)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_vocab_parallel_xent_kernels(dtype):
    g = torch.Generator().manual_seed(5)
    rows, vl, valid, start = 33, 1000, 993, 2000
    buf = (torch.randn(rows, vl + 0, generator=g) * 3).to(dtype)
    labels = torch.randint(1500, 3500, (rows,), generator=g)
    labels[1] = -100
    labels[2] = start + 5
    m0, s0, t0 = E.xent_partial(buf, labels, valid, start)
    m1, s1, t1 = E.xent_partial(buf.to(DEV), labels.to(DEV), valid, start)
    torch.testing.assert_close(m1.cpu(), m0, atol=1e-5, rtol=0)
    torch.testing.assert_close(s1.cpu(), s0, atol=1e-2, rtol=1e-3)
    torch.testing.assert_close(t1.cpu(), t0, atol=1e-5, rtol=0)
    lse = m0 + s0.log() + 0.3
    scale = torch.tensor([0.25])
    d0 = E.xent_apply_(buf.clone(), labels, lse, valid, start, grad_scale_dev=scale)
    d1 = E.xent_apply_(buf.to(DEV), labels.to(DEV), lse.to(DEV), valid, start, grad_scale_dev=scale.to(DEV))
    torch.testing.assert_close(d1.cpu().float(), d0.float(), atol=2e-3, rtol=2e-2)
    assert float(d1[1].abs().max()) == 0.0 and float(d1[:, valid:].abs().max()) == 0.0
