"""tcgen05 GEMM against an fp32 matmul of the same bf16 operands."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from zen_repro_b200.ops import gemm as G  # noqa: E402


def _check(got, want, K):
    err = (got.float() - want).abs().max().item()
    scale = want.abs().max().item() + 1e-6
    assert err <= 0.01 * scale + 0.02, (err, scale)


SHAPES = [(128, 128, 64), (128, 256, 128), (256, 512, 256), (1000, 768, 768), (8192, 2304, 768), (300, 50257, 768),
          (77, 130, 72), (4096, 4096, 4096)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("bn", [0, 128, 256, 512])     # 512 selects the CTA-pair kernel
def test_nt(M, N, K, bn):
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    got = G.gemm_nt(a, b, bn=bn)
    assert G.gemm_error() == 0
    _check(got, a.float() @ b.float().t(), K)


@pytest.mark.parametrize("M,N,K", SHAPES[:6])
def test_nn_and_tn(M, N, K):
    torch.manual_seed(1)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(K, N, device="cuda").bfloat16()
    _check(G.gemm_nn(a, b), a.float() @ b.float(), K)
    at = torch.randn(K, M, device="cuda").bfloat16()
    _check(G.gemm_tn(at, b), at.float().t() @ b.float(), K)
    assert G.gemm_error() == 0


def test_bias_accumulate_fp32_out():
    torch.manual_seed(2)
    M, N, K = 512, 384, 320
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    want = a.float() @ b.float().t() + bias.float()
    _check(G.gemm_nt(a, b, bias=bias), want, K)
    acc = torch.ones(M, N, device="cuda", dtype=torch.float32)
    G.gemm_nt(a, b, out=acc, accumulate=True)
    _check(acc, a.float() @ b.float().t() + 1.0, K)
    accb = torch.ones(M, N, device="cuda", dtype=torch.bfloat16)
    G.gemm_nt(a, b, out=accb, accumulate=True)
    _check(accb, a.float() @ b.float().t() + 1.0, K)
    assert G.gemm_error() == 0


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (1000, 1304, 200), (8192, 768, 768), (384, 50257, 128)])
def test_pair_kernel_store_through_shared_memory(M, N, K):
    """Plain bf16 output of the CTA-pair kernel goes through TMA stores: edges are clipped, padding columns of a wider
    buffer stay untouched, the bias is added."""
    torch.manual_seed(6)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    ld = (N + 7) // 8 * 8 + 8
    buf = torch.full((M + 1, ld), 7.0, device="cuda", dtype=torch.bfloat16)
    out = buf[:M, :N]
    G.gemm_nt(a, b, bias=bias, out=out, bn=512)
    _check(out, a.float() @ b.float().t() + bias.float(), K)
    assert bool((buf[:M, N:] == 7.0).all()) and bool((buf[M] == 7.0).all())
    # the caller may give up the columns to the next multiple of 8 (an odd N then takes the store path too)
    G.gemm_nt(a, b, bias=bias, out=out, bn=512, pad_ok=True)
    _check(out, a.float() @ b.float().t() + bias.float(), K)
    n8 = (N + 7) // 8 * 8
    assert bool((buf[:M, n8:] == 7.0).all()) and bool((buf[M] == 7.0).all())
    assert G.gemm_error() == 0


def test_strided_operands_inside_a_wider_buffer():
    torch.manual_seed(3)
    buf = torch.randn(256, 3 * 128, device="cuda").bfloat16()
    q, k = buf[:, :128], buf[:, 128:256]
    w = torch.randn(64, 128, device="cuda").bfloat16()
    _check(G.gemm_nt(q, w), q.float() @ w.float().t(), 128)
    _check(G.gemm_nt(k, w), k.float() @ w.float().t(), 128)


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 320), (8192, 2304, 768), (1000, 1300, 264)])
def test_pair_kernel_all_layouts(M, N, K):
    torch.manual_seed(4)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(K, N, device="cuda").bfloat16()
    at = torch.randn(K, M, device="cuda").bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    _check(G.gemm_nn(a, b, bias=bias, bn=512), a.float() @ b.float() + bias.float(), K)
    _check(G.gemm_tn(at, b, bn=512), at.float().t() @ b.float(), K)
    acc = torch.ones(M, N, device="cuda", dtype=torch.bfloat16)
    G.gemm_nt(a, b.t().contiguous(), out=acc, accumulate=True, bn=512)
    _check(acc, a.float() @ b.float() + 1.0, K)
    assert G.gemm_error() == 0


@pytest.mark.parametrize("M,N,K", [(768, 2304, 8192), (768, 768, 8192), (3072, 768, 4096), (700, 1000, 2112)])
def test_split_k_weight_gradient_shapes(M, N, K, monkeypatch):
    """Few output tiles and a long K: the K slices meet through the workspace, summed in slice order."""
    monkeypatch.setattr(G, "_SPLITK_MIN_K", 2048)          # the default only splits much longer K
    torch.manual_seed(5)
    assert G.split_k_choice(M, N, K) > 1
    at = torch.randn(K, M, device="cuda").bfloat16()
    b = torch.randn(K, N, device="cuda").bfloat16()
    want = at.float().t() @ b.float()
    got = G.gemm_tn(at, b)
    _check(got, want, K)
    again = G.gemm_tn(at, b)                       # same slices, same order: bit-identical, counters were left at zero
    assert torch.equal(got, again)
    acc = torch.ones(M, N, device="cuda", dtype=torch.bfloat16)
    G.gemm_tn(at, b, out=acc, accumulate=True)
    _check(acc, want + 1.0, K)
    acc32 = torch.full((M, N), 2.0, device="cuda", dtype=torch.float32)
    G.gemm_tn(at, b, out=acc32, accumulate=True)
    _check(acc32, want + 2.0, K)
    a = at.t().contiguous()
    _check(G.gemm_nt(a, b.t().contiguous()), want, K)
    assert G.gemm_error() == 0


@pytest.mark.parametrize("M,N,K", [(256, 128, 64), (8192, 768, 768), (1000, 1304, 200), (512, 50257, 128)])
def test_pair_kernel_with_128_wide_tiles(M, N, K):
    """The CTA-pair kernel with 256 x 128 tiles (chosen when 256-wide tiles fill the GPU unevenly), all layouts."""
    from zen_repro_b200 import _native

    old = _native.lib().zen_gemm2_force_bn(128)
    try:
        torch.manual_seed(7)
        a = torch.randn(M, K, device="cuda").bfloat16()
        b = torch.randn(K, N, device="cuda").bfloat16()
        at = torch.randn(K, M, device="cuda").bfloat16()
        bias = torch.randn(N, device="cuda").bfloat16()
        _check(G.gemm_nn(a, b, bias=bias, bn=512), a.float() @ b.float() + bias.float(), K)
        _check(G.gemm_nt(a, b.t().contiguous(), bn=512), a.float() @ b.float(), K)
        _check(G.gemm_tn(at, b, bn=512), at.float().t() @ b.float(), K)
        acc = torch.ones(M, N, device="cuda", dtype=torch.float32)
        G.gemm_nn(a, b, out=acc, accumulate=True, bn=512)
        _check(acc, a.float() @ b.float() + 1.0, K)
        assert G.gemm_error() == 0
    finally:
        _native.lib().zen_gemm2_force_bn(old)


@pytest.mark.parametrize("M,N,K", [(256, 192, 64), (8192, 768, 768), (8192, 768, 3072), (1000, 1304, 200), (512, 960, 4096)])
def test_pair_kernel_with_192_wide_tiles(M, N, K):
    """The CTA-pair kernel with 256 x 192 tiles (K-major B only; picked when 192-wide tiles need fewer tile-widths of
    time than 256-wide ones, e.g. 8192 x 768 outputs), K-major and MN-major A, bias, fp32 accumulate output."""
    from zen_repro_b200 import _native

    old = _native.lib().zen_gemm2_force_bn(192)
    try:
        torch.manual_seed(8)
        a = torch.randn(M, K, device="cuda").bfloat16()
        w = torch.randn(N, K, device="cuda").bfloat16()               # [N, K]: K-major B for gemm_nt
        at = torch.randn(K, M, device="cuda").bfloat16()
        bias = torch.randn(N, device="cuda").bfloat16()
        _check(G.gemm_nt(a, w, bias=bias, bn=512), a.float() @ w.float().t() + bias.float(), K)
        acc = torch.ones(M, N, device="cuda", dtype=torch.float32)
        G.gemm_nt(a, w, out=acc, accumulate=True, bn=512)
        _check(acc, a.float() @ w.float().t() + 1.0, K)
        # MN-major B falls back to 256-wide tiles under the same setting and must stay correct
        _check(G.gemm_nn(a, w.t().contiguous(), bn=512), a.float() @ w.float().t(), K)
        _check(G.gemm_tn(at, w.t().contiguous(), bn=512), at.float().t() @ w.float().t(), K)
        assert G.gemm_error() == 0
    finally:
        _native.lib().zen_gemm2_force_bn(old)


@pytest.mark.parametrize("M,N,K", [(8192, 768, 3072), (8192, 2048, 1024), (8000, 760, 1100), (8192, 768, 1024)])
def test_tail_split_of_the_last_round(M, N, K):
    """Outputs whose 256 x 256 tiles leave the last wave of clusters less than half full: those tiles run as two K
    slices that exchange half an accumulator.  Same result as without the split (fp32 sums of two halves), the same
    bits on every call, flags left clear for the next launch, all operand layouts, with and without bias."""
    from zen_repro_b200 import _native
    torch.manual_seed(11)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    want = a.float() @ b.float().t()
    lib = _native.lib()
    old = lib.zen_gemm2_tail_split(2)
    try:
        got = G.gemm_nt(a, b, bn=512)
        _check(got, want, K)
        assert torch.equal(got, G.gemm_nt(a, b, bn=512))
        _check(G.gemm_nt(a, b, bias=bias, bn=512), want + bias.float(), K)
        _check(G.gemm_nn(a, b.t().contiguous(), bn=512), want, K)
        _check(G.gemm_tn(a.t().contiguous(), b.t().contiguous(), bn=512), want, K)
        lib.zen_gemm2_tail_split(0)
        plain = G.gemm_nt(a, b, bn=512)
        assert (got.float() - plain.float()).abs().max() <= 0.02 * want.abs().max()
        lib.zen_gemm2_tail_split(2)
        _check(G.gemm_nt(a, b, bn=512), want, K)           # split again after an unsplit launch on the same workspace
    finally:
        lib.zen_gemm2_tail_split(old)
    assert G.gemm_error() == 0


@pytest.mark.parametrize("shapes", [
    [(768, 2304, 8192), (768, 768, 8192), (768, 3072, 8192), (3072, 768, 8192)],      # a GPT-2 layer: 108 tiles, tail of 34
    [(768, 768, 2048), (520, 1000, 1100)],                                            # fewer tiles than clusters: all split
    [(2048, 2560, 1024), (2048, 2048, 1024), (2048, 4096, 1024), (4096, 2048, 1024), (768, 768, 1024), (256, 256, 1024)],
])
def test_grouped_weight_gradients_in_one_launch(shapes):
    """Several a^T @ b products queued by defer_tn go out as one launch over one list of tiles; each equals its own
    GEMM, the callbacks run after the launch, accumulation and fp32 outputs keep the plain store path."""
    torch.manual_seed(13)
    ops, outs, wants, fired = [], [], [], []
    for i, (M, N, K) in enumerate(shapes):
        a = torch.randn(K, M, device="cuda").bfloat16()
        b = torch.randn(K, N, device="cuda").bfloat16()
        want = a.float().t() @ b.float()
        if i == 1:                                       # accumulated into an existing bf16 gradient
            out = torch.ones(M, N, device="cuda", dtype=torch.bfloat16)
            want = want + 1.0
            acc = True
        elif i == 2 and len(shapes) > 2:                 # fp32 output
            out = torch.empty(M, N, device="cuda", dtype=torch.float32)
            acc = False
        else:
            out = torch.full((M, N), 7.0, device="cuda", dtype=torch.bfloat16)     # overwritten
            acc = False
        ops.append((a, b, out, acc)); outs.append(out); wants.append((want, K))
    old = G.GROUP_SIZE
    G.GROUP_SIZE = 6
    try:
        for i, (a, b, out, acc) in enumerate(ops):
            G.defer_tn(a, b, out, acc, done=lambda i=i: fired.append(i))
        if len(ops) < 6:
            assert fired == []                           # still queued
        G.flush_deferred()
    finally:
        G.GROUP_SIZE = old
    assert fired == list(range(len(ops)))
    for out, (want, K) in zip(outs, wants):
        _check(out, want, K)
    assert G.gemm_error() == 0
    # the same outputs again, everything overwritten this time: bit-identical to separate launches without tail split
    from zen_repro_b200 import _native
    G.GROUP_SIZE = 6
    try:
        fresh = [torch.empty(M, N, device="cuda", dtype=torch.bfloat16) for (M, N, K) in shapes]
        for (a, b, _o, _acc), o in zip(ops, fresh):
            G.defer_tn(a, b, o, False)
        G.flush_deferred()
        again = [torch.empty(M, N, device="cuda", dtype=torch.bfloat16) for (M, N, K) in shapes]
        for (a, b, _o, _acc), o in zip(ops, again):
            G.defer_tn(a, b, o, False)
        G.flush_deferred()
    finally:
        G.GROUP_SIZE = old
    for x, y, (want, K) in zip(fresh, again, [( (a.float().t() @ b.float()), a.shape[0]) for (a, b, _o, _c) in ops]):
        assert torch.equal(x, y)
        _check(x, want, K)
    assert G.gemm_error() == 0
