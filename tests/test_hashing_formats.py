import torch
from hypothesis import given, settings, strategies as st

from zen_repro_b200.sparse import formats, hashing
from zen_repro_b200.sparse.hashing import BlockPermutation


@settings(max_examples=60, deadline=None)
@given(st.integers(1, 200000), st.integers(1, 8), st.sampled_from([1, 64, 128]))
def test_block_permutation_is_bijection(n, p, g):
    perm = BlockPermutation.make(n, p, g)
    idx = torch.arange(n)
    owner, slot = perm.owner_slot(idx)
    assert owner.min() >= 0 and owner.max() < p
    assert slot.min() >= 0 and slot.max() < perm.slots_per_part
    flat = owner * perm.slots_per_part + slot
    assert flat.unique().numel() == n
    back = torch.empty_like(idx)
    for o in range(p):
        m = owner == o
        back[m] = perm.index_of(o, slot[m])
    assert torch.equal(back, idx)


def _zipf_positions(n, count, s, seed):
    g = torch.Generator().manual_seed(seed)
    w = 1.0 / torch.arange(1, n + 1, dtype=torch.float64) ** s
    return torch.multinomial(w, count, replacement=False, generator=g)


def test_partition_balance_on_zipf_positions():
    n = 1 << 20
    for p in (2, 4, 8):
        perm = BlockPermutation.make(n, p, 64)
        idx = _zipf_positions(n, n // 100, 1.1, seed=p)
        owner, _ = perm.owner_slot(idx)
        imb = hashing.partition_imbalance(owner, p)
        contiguous = hashing.partition_imbalance(idx // (n // p), p)
        assert imb < 1.10, (p, imb)
        assert contiguous > 1.5


def test_zen_poly3_matches_wrapping_arithmetic():
    idx = torch.tensor([0, 1, 2, 12345, 2 ** 20 + 7])
    h = hashing.zen_poly3(idx, 10001861)
    for i, k in enumerate(idx.tolist()):
        want = (573729859 * k ** 3 + 0xCC9E2D51 * k ** 2 + 0x1B873593 * k + 10001861) % (1 << 32)
        assert int(h[i]) == want
    own = hashing.zen_poly3_owner(torch.arange(100000), 100000 // 8 * 8, 8)
    assert own.min() >= 0 and own.max() < 8
    assert hashing.partition_imbalance(own, 8) < 1.1


@settings(max_examples=50, deadline=None)
@given(st.lists(st.booleans(), min_size=1, max_size=300))
def test_bitmap_roundtrip_lsb_first(bits):
    m = torch.tensor(bits)
    packed = formats.pack_bitmap(m)
    assert packed.numel() == (len(bits) + 7) // 8
    assert torch.equal(formats.unpack_bitmap(packed, len(bits)), m)
    if bits[0]:
        assert int(packed[0]) & 1        # slot 0 is the least significant bit of byte 0


def test_coo_and_format_choice():
    d = torch.tensor([0.0, 1.5, 0.0, -2.0])
    i, v = formats.coo_encode(d)
    assert i.tolist() == [1, 3]
    assert torch.equal(formats.coo_decode(i, v, 4), d)
    assert formats.choose_index_format(10, 100000) == "coo"
    assert formats.choose_index_format(5000, 100000) == "bitmap"
    assert formats.choose_index_format(60000, 100000) == "dense"


def test_murmur3_known_vectors_and_split_k_choice():
    from zen_repro_b200.sparse.hashing import fmix32, murmur3_32

    # published verification values of MurmurHash3_x86_32 for 4-byte keys
    keys = torch.tensor([0x00000000, 0xFFFFFFFF, 0x87654321], dtype=torch.int64)
    got = murmur3_32(keys, 0).tolist()
    assert got == [0x2362F9DE, 0x76293B50, 0xF55B516B], [hex(v) for v in got]
    assert int(murmur3_32(torch.tensor([0x87654321]), 0x5082EDEE)) == 0x2362F9DE
    assert int(fmix32(torch.tensor([0]))) == 0
    # spreads consecutive indices over 8 owners within a few percent
    own = murmur3_32(torch.arange(1 << 16), 0) % 8
    cnt = torch.bincount(own, minlength=8).float()
    assert float(cnt.max() / cnt.mean()) < 1.05


def test_split_k_choice_is_limited_to_weight_gradient_shapes():
    from zen_repro_b200.ops import gemm as G

    assert G.split_k_choice(768, 2304, 8192) == 2          # 27 tiles, long K
    assert G.split_k_choice(768, 768, 8192) == 2
    assert G.split_k_choice(8192, 2304, 768) == 1          # plenty of tiles
    assert G.split_k_choice(768, 2304, 1024) == 1          # short K
    assert G.split_k_choice(4096, 4096, 8192) == 1
    assert G.split_k_choice(100, 2304, 8192) == 1          # too narrow for a 256-row pair tile


def test_packed_bf16_threshold_pretest_matches_the_exact_compare():
    """The partition kernel's cheap per-vector test for bf16 (both halves of a 32-bit word against the threshold with one
    add and one mask, `Raw8<bf16>::hit` in csrc/sparse_kernels.cu), restated on integers: it must never reject a value
    that the exact compare |x| >= thr keeps, and must reject everything below the threshold rounded up to bf16."""
    import numpy as np

    rng = np.random.default_rng(0)
    for thr in [0.0, 1e-30, 0.003, 0.5, 0.50001, 1.0, 3.1e38, float("inf")]:
        tbits = max(int(np.float32(thr).view(np.uint32)), 1)
        t16 = min((tbits + 0xFFFF) >> 16, 0x8000) or 1
        addc = ((0x8000 - t16) * 0x00010001) & 0xFFFFFFFF
        x16 = rng.integers(0, 1 << 16, size=4096, dtype=np.uint32)
        x16[:8] = [0, 0x8000, 1, 0x3F00, 0x3F01, 0x7F80, 0xFF80, t16]          # +0, -0, tiny, 0.5, next, +inf, -inf, threshold
        words = x16[0::2] | (x16[1::2] << 16)
        got = (((words & 0x7FFF7FFF) + addc) & 0x80008000) != 0
        mag32 = (x16 & 0x7FFF).astype(np.uint64) << 16
        exact = mag32 >= tbits                                                 # the kernel's keep test on magnitude bits
        want = exact[0::2] | exact[1::2]
        assert np.array_equal(got, want), thr
