"""Model configurations.  One dataclass describes every decoder family the framework trains:
GPT-2 (learned positions, LayerNorm, GELU, Conv1D weight layout), OPT (learned positions with offset 2,
LayerNorm, ReLU), Llama (RMSNorm, RoPE, GQA, SwiGLU) and Gemma (RMSNorm with unit offset, RoPE, MQA,
GeGLU, scaled embeddings).  The reference builds these from HuggingFace configs
(train.py:141-152); the presets below carry the same shapes so that no hub access is needed.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass


@dataclass
class ModelConfig:
    family: str = "gpt2"              # gpt2 | opt | llama | gemma
    vocab_size: int = 50257
    hidden_size: int = 768
    num_layers: int = 12
    num_heads: int = 12
    num_kv_heads: int = 12
    head_dim: int = 64
    intermediate_size: int = 3072
    max_position: int = 1024
    norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    tie_embeddings: bool = True
    init_std: float = 0.02
    grad_checkpoint: bool = False
    name: str = "gpt2"
    # Gemma-2 additions (all off for the other families)
    post_norms: bool = False          # a second RMSNorm on the output of the attention and of the MLP branch
    attn_softcap: float = 0.0         # scores -> cap * tanh(scores / cap) before the softmax
    final_softcap: float = 0.0        # logits -> cap * tanh(logits / cap) before the loss
    sliding_window: int = 0           # every other layer attends to the last `sliding_window` positions only

    # ---- derived behaviour -------------------------------------------------------------
    @property
    def layer_norm(self) -> bool:
        return self.family in ("gpt2", "opt")

    @property
    def norm_unit_offset(self) -> bool:
        return self.family == "gemma"

    @property
    def act(self) -> str:
        return {"gpt2": "gelu_tanh", "opt": "relu", "llama": "swiglu", "gemma": "geglu"}[self.family]

    @property
    def gated(self) -> bool:
        return self.family in ("llama", "gemma")

    @property
    def learned_positions(self) -> bool:
        return self.family in ("gpt2", "opt")

    @property
    def pos_offset(self) -> int:
        return 2 if self.family == "opt" else 0

    @property
    def has_bias(self) -> bool:
        return self.family in ("gpt2", "opt")

    @property
    def weight_layout(self) -> str:
        return "in_out" if self.family == "gpt2" else "out_in"

    @property
    def embed_scale(self) -> float:
        return float(self.hidden_size) ** 0.5 if self.family == "gemma" else 1.0

    def replace(self, **kw) -> "ModelConfig":
        return dataclasses.replace(self, **kw)

    def num_params(self) -> int:
        d, i, L = self.hidden_size, self.intermediate_size, self.num_layers
        qkv = d * (self.num_heads + 2 * self.num_kv_heads) * self.head_dim
        o = self.num_heads * self.head_dim * d
        mlp = d * i * (3 if self.gated else 2)
        emb = self.vocab_size * d * (1 if self.tie_embeddings else 2)
        pos = (self.max_position + self.pos_offset) * d if self.learned_positions else 0
        return L * (qkv + o + mlp) + emb + pos

    def flops_per_token(self, seq: int) -> float:
        """Training FLOPs per token (forward + backward), matmuls and attention only."""
        d, i, L = self.hidden_size, self.intermediate_size, self.num_layers
        qkv = d * (self.num_heads + 2 * self.num_kv_heads) * self.head_dim
        o = self.num_heads * self.head_dim * d
        mlp = d * i * (3 if self.gated else 2)
        attn = 2 * seq * self.num_heads * self.head_dim * 0.5          # causal: half of QK^T and PV
        per_layer = qkv + o + mlp + attn
        return 6.0 * (L * per_layer + self.vocab_size * d)


PRESETS = {
    # headline benchmark config 2: GPT-2 small
    "gpt2": ModelConfig(family="gpt2", name="gpt2", vocab_size=50257, hidden_size=768, num_layers=12, num_heads=12,
                        num_kv_heads=12, head_dim=64, intermediate_size=3072, max_position=1024, norm_eps=1e-5),
    # benchmark config 3: Gemma-2B (18 layers, MQA, head_dim 256, GeGLU 16384, vocab 256000)
    "gemma-2b": ModelConfig(family="gemma", name="gemma-2b", vocab_size=256000, hidden_size=2048, num_layers=18,
                            num_heads=8, num_kv_heads=1, head_dim=256, intermediate_size=16384, max_position=8192,
                            norm_eps=1e-6, tie_embeddings=True),
    # benchmark config 4: Llama-3-8B
    "llama-3-8b": ModelConfig(family="llama", name="llama-3-8b", vocab_size=128256, hidden_size=4096, num_layers=32,
                              num_heads=32, num_kv_heads=8, head_dim=128, intermediate_size=14336, max_position=8192,
                              norm_eps=1e-5, rope_theta=500000.0, tie_embeddings=False),
    # the reference's sweep (run_all.sh:5)
    "facebook/opt-2.7b": ModelConfig(family="opt", name="facebook/opt-2.7b", vocab_size=50272, hidden_size=2560,
                                     num_layers=32, num_heads=32, num_kv_heads=32, head_dim=80, intermediate_size=10240,
                                     max_position=2048, norm_eps=1e-5),
    "meta-llama/Llama-3.2-3B": ModelConfig(family="llama", name="meta-llama/Llama-3.2-3B", vocab_size=128256,
                                           hidden_size=3072, num_layers=28, num_heads=24, num_kv_heads=8, head_dim=128,
                                           intermediate_size=8192, max_position=8192, norm_eps=1e-5,
                                           rope_theta=500000.0, tie_embeddings=True),
    # Gemma-2 2B: pre + post norms around both branches, soft-capped attention scores (50) and final logits (30),
    # sliding-window attention (4096) on every other layer; the reference forces 8 KV heads for any gemma model
    # (train.py:146-147)
    "google/gemma-2-2b": ModelConfig(family="gemma", name="google/gemma-2-2b", vocab_size=256000, hidden_size=2304,
                                     num_layers=26, num_heads=8, num_kv_heads=8, head_dim=256, intermediate_size=9216,
                                     max_position=8192, norm_eps=1e-6, tie_embeddings=True, post_norms=True,
                                     attn_softcap=50.0, final_softcap=30.0, sliding_window=4096),
    # tiny models for tests and smoke runs
    "tiny-gpt2": ModelConfig(family="gpt2", name="tiny-gpt2", vocab_size=1000, hidden_size=64, num_layers=2,
                             num_heads=4, num_kv_heads=4, head_dim=16, intermediate_size=256, max_position=64),
    "tiny-llama": ModelConfig(family="llama", name="tiny-llama", vocab_size=1000, hidden_size=64, num_layers=2,
                              num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=128, max_position=64,
                              tie_embeddings=False),
    "tiny-gemma": ModelConfig(family="gemma", name="tiny-gemma", vocab_size=1000, hidden_size=64, num_layers=2,
                              num_heads=4, num_kv_heads=1, head_dim=32, intermediate_size=128, max_position=64,
                              norm_eps=1e-6),
    "tiny-gemma2": ModelConfig(family="gemma", name="tiny-gemma2", vocab_size=1000, hidden_size=64, num_layers=2,
                               num_heads=4, num_kv_heads=2, head_dim=32, intermediate_size=128, max_position=64,
                               norm_eps=1e-6, post_norms=True, attn_softcap=50.0, final_softcap=30.0, sliding_window=4096),
    "tiny-opt": ModelConfig(family="opt", name="tiny-opt", vocab_size=1000, hidden_size=64, num_layers=2, num_heads=4,
                            num_kv_heads=4, head_dim=16, intermediate_size=256, max_position=64),
}
PRESETS["gpt2-small"] = PRESETS["gpt2"]
PRESETS["google/gemma-2b"] = PRESETS["gemma-2b"]
PRESETS["meta-llama/Meta-Llama-3-8B"] = PRESETS["llama-3-8b"]


def get_config(name: str, **overrides) -> ModelConfig:
    if name not in PRESETS:
        raise KeyError(f"unknown model {name!r}; known: {sorted(PRESETS)}")
    cfg = PRESETS[name]
    overrides = {k: v for k, v in overrides.items() if v is not None}
    return cfg.replace(**overrides) if overrides else cfg
