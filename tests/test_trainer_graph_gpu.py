"""Whole-step CUDA graph on one GPU: the status mirror inside a replayed step, resume of the device step counter, and
the Gemma-2 block (soft-capped attention on the head_dim 256 kernels) against the fp32 restatement."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _trainer(**kw):
    from zen_repro_b200.trainer import TrainConfig, Trainer

    cfg = dict(model="gpt2", num_layers=2, micro_batch=2, seq_len=128, data_pool=4, cuda_graph=True, graph_warmup=2, lr=1e-3)
    cfg.update(kw)
    return Trainer(TrainConfig(**cfg), init_dist=False)


def test_status_mirror_follows_graph_replays_and_recovers_two_steps_later():
    t = _trainer()
    fake = torch.zeros(1, dtype=torch.int32, device=t.device)
    t.health.add("embedding_rows", fake)                 # stands in for an engine's status word
    losses = []
    for step in range(10):
        if step == 6:
            fake.fill_(4)                                # "a wait expired" during step 6 (set on the host, between steps)
        losses.append(t.step(next(t.data), read_loss=(step % 2 == 0)))
    torch.cuda.synchronize()
    assert len(t.recoveries) == 1 and t.recoveries[0]["step"] == 8 and t.recoveries[0]["status"] == {"embedding_rows": 4}
    assert t._graph is None and not t.graph_ok           # replays stopped at the recovery
    assert int(fake.item()) == 0


def test_replayed_steps_match_eager_steps():
    a, b = _trainer(cuda_graph=True), _trainer(cuda_graph=False)
    la = [a.step(next(a.data)) for _ in range(6)]
    lb = [b.step(next(b.data)) for _ in range(6)]
    assert a._graph is not None and b._graph is None
    assert la == pytest.approx(lb, rel=2e-3, abs=2e-3)
    assert a.optimizer.steps_done == 6                   # the device counter advanced in the replays too


def test_resume_under_cuda_graph_continues_like_an_uninterrupted_run(tmp_path):
    from zen_repro_b200.ckpt import load_checkpoint, save_checkpoint

    a = _trainer()
    for _ in range(5):
        a.step(next(a.data))
    save_checkpoint(str(tmp_path), a)
    want = [a.step(next(a.data)) for _ in range(4)]
    b = _trainer()
    assert load_checkpoint(str(tmp_path), b) == 5
    got = [b.step(next(b.data)) for _ in range(4)]
    assert b._graph is not None                          # two eager steps after the resume, then captured again
    assert got == pytest.approx(want, rel=2e-3, abs=2e-3)
    assert b.optimizer.steps_done == 9


@pytest.mark.parametrize("B,S,hq,hkv", [(1, 256, 4, 2), (2, 384, 8, 8)])
def test_softcapped_attention_hd256(B, S, hq, hkv):
    from zen_repro_b200.ops import attention as A
    from zen_repro_b200.ops import autograd as O

    hd, cap = 256, 50.0
    torch.manual_seed(5)
    qkv = (torch.randn(B * S, (hq + 2 * hkv) * hd, device="cuda") * 2.0).bfloat16().requires_grad_(True)   # scores beyond the cap
    dout = (torch.randn(B * S, hq * hd, device="cuda") * 0.5).bfloat16()
    out = O.attention(qkv, B, S, hq, hkv, hd, softcap=cap)
    out.backward(dout)
    torch.cuda.synchronize()
    assert A.attention_error() == 0
    x = qkv.detach().float().requires_grad_(True)
    want = A.reference_attention(x, B, S, hq, hkv, hd, 1.0 / math.sqrt(hd), cap)
    torch.testing.assert_close(out.float(), want.float(), atol=3e-2, rtol=3e-2)
    (g,) = torch.autograd.grad(want, x, dout.float())
    rel = (qkv.grad.float() - g).norm() / g.norm()
    assert rel < 0.03, float(rel)
    plain = O.attention(qkv.detach(), B, S, hq, hkv, hd)
    assert (plain.float() - out.float()).abs().max() > 0.05          # the cap really changed the result


def test_gemma2_block_trains_on_the_kernels():
    t = _trainer(model="google/gemma-2-2b", num_layers=2, micro_batch=1, seq_len=256, cuda_graph=False, lr=1e-4)
    losses = [t.step(next(t.data)) for _ in range(4)]
    assert all(l == l for l in losses) and losses[-1] < losses[0]
    assert not any(t.check_health(raise_on_error=False).values())
