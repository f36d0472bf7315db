"""tcgen05 attention kernels against an fp32 softmax(QK^T)V restatement."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from zen_repro_b200.ops import attention as A  # noqa: E402


def _ref(qkv, B, S, hq, hkv, hd, scale):
    t = qkv.float().view(B, S, hq + 2 * hkv, hd)
    q, k, v = t[:, :, :hq].transpose(1, 2), t[:, :, hq:hq + hkv].transpose(1, 2), t[:, :, hq + hkv:].transpose(1, 2)
    rep = hq // hkv
    k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    s = (q @ k.transpose(-1, -2)) * scale
    mask = torch.ones(S, S, dtype=torch.bool, device=qkv.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, -1)
    o = torch.softmax(s, -1) @ v
    return o.transpose(1, 2).reshape(B * S, hq * hd), lse


@pytest.mark.parametrize("B,S,hq,hkv,hd", [(2, 128, 2, 2, 64), (1, 512, 4, 4, 64), (2, 1024, 12, 12, 64),
                                           (1, 384, 8, 2, 128), (1, 256, 4, 1, 256), (2, 256, 8, 8, 128)])
def test_forward(B, S, hq, hkv, hd):
    torch.manual_seed(0)
    qkv = (torch.randn(B * S, (hq + 2 * hkv) * hd, device="cuda") * 0.7).bfloat16()
    scale = 1.0 / math.sqrt(hd)
    out, lse2 = A.attention_fwd_kernel(qkv, B, S, hq, hkv, hd, scale)
    torch.cuda.synchronize()
    assert A.attention_error() == 0
    want, lse = _ref(qkv, B, S, hq, hkv, hd, scale)
    torch.testing.assert_close(out.float(), want, atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(lse2 * math.log(2.0), lse, atol=2e-2, rtol=1e-3)
