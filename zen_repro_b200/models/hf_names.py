"""HuggingFace parameter names and shapes <-> this framework's fused parameters.

``to_hf`` splits the fused qkv and gate|up matrices and renames everything so that the result loads
into ``transformers``' GPT2LMHeadModel / OPTForCausalLM / LlamaForCausalLM / GemmaForCausalLM / Gemma2ForCausalLM with
``load_state_dict``; ``from_hf`` is the inverse.  Only full (TP = 1) models are converted; sharded
models are gathered first by the checkpoint code.
"""
from __future__ import annotations

import torch


def _split_rows(w, sizes, layout):
    """Split the output dimension of a weight (rows for [out, in], columns for [in, out])."""
    return torch.split(w, sizes, dim=1 if layout == "in_out" else 0)


def to_hf(model) -> dict:
    cfg = model.cfg
    fam = cfg.family
    hd = cfg.head_dim
    qs, ks = cfg.num_heads * hd, cfg.num_kv_heads * hd
    sd = {}
    V = cfg.vocab_size

    def put(k, t):
        sd[k] = t.detach().clone()

    if fam == "gpt2":
        put("transformer.wte.weight", model.wte[:V])
        put("transformer.wpe.weight", model.wpe)
        for i, b in enumerate(model.blocks):
            p = f"transformer.h.{i}."
            put(p + "ln_1.weight", b.norm1_w); put(p + "ln_1.bias", b.norm1_b)
            put(p + "attn.c_attn.weight", b.qkv_w); put(p + "attn.c_attn.bias", b.qkv_b)
            put(p + "attn.c_proj.weight", b.o_w); put(p + "attn.c_proj.bias", b.o_b)
            put(p + "ln_2.weight", b.norm2_w); put(p + "ln_2.bias", b.norm2_b)
            put(p + "mlp.c_fc.weight", b.up_w); put(p + "mlp.c_fc.bias", b.up_b)
            put(p + "mlp.c_proj.weight", b.down_w); put(p + "mlp.c_proj.bias", b.down_b)
        put("transformer.ln_f.weight", model.norm_f_w); put("transformer.ln_f.bias", model.norm_f_b)
        put("lm_head.weight", model.head_weight()[:V])
    elif fam == "opt":
        put("model.decoder.embed_tokens.weight", model.wte[:V])
        put("model.decoder.embed_positions.weight", model.wpe)
        for i, b in enumerate(model.blocks):
            p = f"model.decoder.layers.{i}."
            q, k, v = _split_rows(b.qkv_w, [qs, ks, ks], "out_in")
            qb, kb, vb = torch.split(b.qkv_b, [qs, ks, ks])
            put(p + "self_attn.q_proj.weight", q); put(p + "self_attn.q_proj.bias", qb)
            put(p + "self_attn.k_proj.weight", k); put(p + "self_attn.k_proj.bias", kb)
            put(p + "self_attn.v_proj.weight", v); put(p + "self_attn.v_proj.bias", vb)
            put(p + "self_attn.out_proj.weight", b.o_w); put(p + "self_attn.out_proj.bias", b.o_b)
            put(p + "self_attn_layer_norm.weight", b.norm1_w); put(p + "self_attn_layer_norm.bias", b.norm1_b)
            put(p + "fc1.weight", b.up_w); put(p + "fc1.bias", b.up_b)
            put(p + "fc2.weight", b.down_w); put(p + "fc2.bias", b.down_b)
            put(p + "final_layer_norm.weight", b.norm2_w); put(p + "final_layer_norm.bias", b.norm2_b)
        put("model.decoder.final_layer_norm.weight", model.norm_f_w)
        put("model.decoder.final_layer_norm.bias", model.norm_f_b)
        put("lm_head.weight", model.head_weight()[:V])
    else:  # llama, gemma
        put("model.embed_tokens.weight", model.wte[:V])
        for i, b in enumerate(model.blocks):
            p = f"model.layers.{i}."
            q, k, v = _split_rows(b.qkv_w, [qs, ks, ks], "out_in")
            gate, up = _split_rows(b.up_w, [cfg.intermediate_size] * 2, "out_in")
            put(p + "self_attn.q_proj.weight", q); put(p + "self_attn.k_proj.weight", k)
            put(p + "self_attn.v_proj.weight", v); put(p + "self_attn.o_proj.weight", b.o_w)
            put(p + "mlp.gate_proj.weight", gate); put(p + "mlp.up_proj.weight", up)
            put(p + "mlp.down_proj.weight", b.down_w)
            put(p + "input_layernorm.weight", b.norm1_w)
            if cfg.post_norms:       # Gemma-2 names: post_attention = norm on the attention output, pre_feedforward = MLP input
                put(p + "post_attention_layernorm.weight", b.postnorm1_w)
                put(p + "pre_feedforward_layernorm.weight", b.norm2_w)
                put(p + "post_feedforward_layernorm.weight", b.postnorm2_w)
            else:
                put(p + "post_attention_layernorm.weight", b.norm2_w)
        put("model.norm.weight", model.norm_f_w)
        put("lm_head.weight", model.head_weight()[:V])
    return sd


@torch.no_grad()
def from_hf(model, sd: dict, strict: bool = True):
    cfg = model.cfg
    fam = cfg.family
    V = cfg.vocab_size
    used = set()

    def get(k):
        used.add(k)
        return sd[k]

    def cp(dst, src):
        dst.copy_(src.to(dst.dtype))

    if fam == "gpt2":
        cp(model.wte[:V], get("transformer.wte.weight")); cp(model.wpe, get("transformer.wpe.weight"))
        for i, b in enumerate(model.blocks):
            p = f"transformer.h.{i}."
            for ours, theirs in (("norm1_w", "ln_1.weight"), ("norm1_b", "ln_1.bias"), ("qkv_w", "attn.c_attn.weight"),
                                 ("qkv_b", "attn.c_attn.bias"), ("o_w", "attn.c_proj.weight"), ("o_b", "attn.c_proj.bias"),
                                 ("norm2_w", "ln_2.weight"), ("norm2_b", "ln_2.bias"), ("up_w", "mlp.c_fc.weight"),
                                 ("up_b", "mlp.c_fc.bias"), ("down_w", "mlp.c_proj.weight"), ("down_b", "mlp.c_proj.bias")):
                cp(getattr(b, ours), get(p + theirs))
        cp(model.norm_f_w, get("transformer.ln_f.weight")); cp(model.norm_f_b, get("transformer.ln_f.bias"))
    elif fam == "opt":
        cp(model.wte[:V], get("model.decoder.embed_tokens.weight"))
        cp(model.wpe, get("model.decoder.embed_positions.weight"))
        for i, b in enumerate(model.blocks):
            p = f"model.decoder.layers.{i}."
            cp(b.qkv_w, torch.cat([get(p + f"self_attn.{n}_proj.weight") for n in "qkv"], 0))
            cp(b.qkv_b, torch.cat([get(p + f"self_attn.{n}_proj.bias") for n in "qkv"], 0))
            for ours, theirs in (("o_w", "self_attn.out_proj.weight"), ("o_b", "self_attn.out_proj.bias"),
                                 ("norm1_w", "self_attn_layer_norm.weight"), ("norm1_b", "self_attn_layer_norm.bias"),
                                 ("up_w", "fc1.weight"), ("up_b", "fc1.bias"), ("down_w", "fc2.weight"),
                                 ("down_b", "fc2.bias"), ("norm2_w", "final_layer_norm.weight"),
                                 ("norm2_b", "final_layer_norm.bias")):
                cp(getattr(b, ours), get(p + theirs))
        cp(model.norm_f_w, get("model.decoder.final_layer_norm.weight"))
        cp(model.norm_f_b, get("model.decoder.final_layer_norm.bias"))
    else:
        cp(model.wte[:V], get("model.embed_tokens.weight"))
        for i, b in enumerate(model.blocks):
            p = f"model.layers.{i}."
            cp(b.qkv_w, torch.cat([get(p + f"self_attn.{n}_proj.weight") for n in "qkv"], 0))
            cp(b.up_w, torch.cat([get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight")], 0))
            norms = ((("norm1_w", "input_layernorm.weight"), ("postnorm1_w", "post_attention_layernorm.weight"),
                      ("norm2_w", "pre_feedforward_layernorm.weight"), ("postnorm2_w", "post_feedforward_layernorm.weight"))
                     if cfg.post_norms else
                     (("norm1_w", "input_layernorm.weight"), ("norm2_w", "post_attention_layernorm.weight")))
            for ours, theirs in (("o_w", "self_attn.o_proj.weight"), ("down_w", "mlp.down_proj.weight")) + norms:
                cp(getattr(b, ours), get(p + theirs))
        cp(model.norm_f_w, get("model.norm.weight"))
    if model.lm_head is not None:
        cp(model.lm_head[:V], get("lm_head.weight"))
    else:
        used.add("lm_head.weight")
    if strict:
        extra = [k for k in sd if k not in used and not k.endswith(("attn.bias", "attn.masked_bias", "inv_freq"))]
        if extra:
            raise KeyError(f"unexpected keys in HF state dict: {extra[:5]}")
    return model
