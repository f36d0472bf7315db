"""AdamW state across save / resume with the device step counter (the counter a captured step reads)."""
import torch


def test_load_state_dict_restores_device_step_counter_and_state_dict_reads_it():
    from zen_repro_b200.optim import FusedAdamW

    p = torch.nn.Parameter(torch.randn(8))
    opt = FusedAdamW([p], lr=1e-2)
    opt.enable_device_step("cpu")
    for _ in range(3):
        p.grad = torch.randn(8)
        opt.step()
    opt._step_dev += 2                     # what two graph replays do: the host side of step() does not run
    sd = opt.state_dict()
    assert sd["zen_step"] == 5
    q = torch.nn.Parameter(p.detach().clone())
    opt2 = FusedAdamW([q], lr=1e-2)
    opt2.enable_device_step("cpu")
    opt2.load_state_dict(sd)
    assert int(opt2._step_dev) == 5 and opt2._step == 5


def test_moments_and_master_weights_keep_fp32_through_load_state_dict():
    """torch's own loader would cast optimizer state to the parameter's dtype (bf16); the kernel reads fp32."""
    from zen_repro_b200.optim import FusedAdamW

    p = torch.nn.Parameter(torch.randn(16).bfloat16())
    opt = FusedAdamW([p], lr=1e-2)
    p.grad = torch.randn(16).bfloat16()
    opt.step()
    sd = opt.state_dict()
    q = torch.nn.Parameter(p.detach().clone())
    opt2 = FusedAdamW([q], lr=1e-2)
    opt2.load_state_dict(sd)
    st = opt2.state[q]
    assert st["exp_avg"].dtype == st["exp_avg_sq"].dtype == st["master"].dtype == torch.float32
    torch.testing.assert_close(st["master"], opt.state[p]["master"], atol=0, rtol=0)
