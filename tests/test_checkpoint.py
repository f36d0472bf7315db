import pytest
import torch

from zen_repro_b200.ckpt import load_checkpoint, save_checkpoint
from zen_repro_b200.trainer import TrainConfig, Trainer


def _mk():
    return Trainer(TrainConfig(model="tiny-llama", micro_batch=2, seq_len=16, precision="fp32", lr=1e-2, data_pool=0),
                   init_dist=False)


def test_resume_continues_identically(tmp_path):
    a = _mk()
    for _ in range(3):
        a.step(next(a.data))
    save_checkpoint(str(tmp_path), a)
    want = [a.step(next(a.data)) for _ in range(3)]
    b = _mk()
    assert load_checkpoint(str(tmp_path), b) == 3
    got = [b.step(next(b.data)) for _ in range(3)]
    assert got == pytest.approx(want, rel=1e-6)


def test_hf_checkpoint_loads_into_transformers(tmp_path):
    transformers = pytest.importorskip("transformers")
    a = _mk()
    save_checkpoint(str(tmp_path), a)
    sd = torch.load(tmp_path / "pytorch_model.bin", weights_only=True)
    cfg = a.model_cfg
    hf = transformers.LlamaForCausalLM(transformers.LlamaConfig(
        vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
        num_hidden_layers=cfg.num_layers, num_attention_heads=cfg.num_heads, num_key_value_heads=cfg.num_kv_heads,
        head_dim=cfg.head_dim, tie_word_embeddings=False))
    missing, unexpected = hf.load_state_dict(sd, strict=False)
    assert not unexpected and all("inv_freq" in m for m in missing)
    ids = torch.randint(0, cfg.vocab_size, (2, 16))
    ours = a.model.unwrap()(ids, ids)
    theirs = hf(input_ids=ids, labels=ids).loss
    torch.testing.assert_close(ours, theirs, atol=1e-4, rtol=1e-4)


def _tp2_save_worker(rank, world, path):
    t = Trainer(TrainConfig(model="tiny-llama", micro_batch=2, seq_len=16, precision="fp32", lr=1e-2, data_pool=0, tp=2),
                init_dist=False)
    for _ in range(2):
        t.step(next(t.data))
    save_checkpoint(path, t)
    return [t.step(next(t.data)) for _ in range(2)]


def test_checkpoint_written_with_tp2_resumes_on_one_rank(tmp_path):
    """Model shards and optimizer moments of a TP = 2 run are joined for a TP = 1 resume; the HF-format file holds the
    full model either way."""
    from _dist_util import run_gloo

    want = run_gloo(_tp2_save_worker, 2, str(tmp_path))[0]
    b = _mk()
    assert load_checkpoint(str(tmp_path), b) == 2
    got = [b.step(next(b.data)) for _ in range(2)]
    assert got == pytest.approx(want, rel=1e-4, abs=1e-4)
    sd = torch.load(tmp_path / "pytorch_model.bin", weights_only=True)
    cfg = b.model_cfg
    assert sd["model.embed_tokens.weight"].shape == (cfg.vocab_size, cfg.hidden_size)


def test_check_health_is_clean_on_cpu():
    a = _mk()
    a.step(next(a.data))
    assert not any(a.check_health().values())
