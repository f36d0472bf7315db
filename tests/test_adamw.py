import pytest
import torch

from zen_repro_b200.optim import FusedAdamW


def _run(device, dtype, steps=4):
    torch.manual_seed(0)
    ps = [torch.randn(n).to(dtype).to(device).requires_grad_(True) for n in (7, 70000, 131072 + 3)]
    ref = [p.detach().float().cpu().clone().requires_grad_(True) for p in ps]
    opt = FusedAdamW(ps, lr=1e-2, weight_decay=0.1)
    ropt = torch.optim.AdamW(ref, lr=1e-2, weight_decay=0.1)
    for s in range(steps):
        for p, r in zip(ps, ref):
            g = torch.randn(p.shape, generator=torch.Generator().manual_seed(s * 10 + p.numel() % 7))
            p.grad = g.to(dtype).to(device)
            r.grad = g.to(dtype).float()
        opt.step()
        ropt.step()
    return ps, ref, opt


def test_cpu_matches_torch_adamw():
    ps, ref, _ = _run("cpu", torch.float32)
    for p, r in zip(ps, ref):
        torch.testing.assert_close(p.detach(), r.detach(), atol=1e-6, rtol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gpu_matches_torch_adamw(dtype):
    ps, ref, opt = _run("cuda", dtype)
    for p, r in zip(ps, ref):
        if dtype == torch.float32:
            torch.testing.assert_close(p.detach().cpu(), r.detach(), atol=1e-6, rtol=1e-5)
        else:
            torch.testing.assert_close(opt.state[p]["master"].cpu(), r.detach(), atol=1e-5, rtol=1e-4)
            torch.testing.assert_close(p.detach().cpu().float(), r.detach(), atol=1e-2, rtol=1e-2)
