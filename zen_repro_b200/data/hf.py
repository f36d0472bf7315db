"""Optional HuggingFace data path with the behaviour of the reference's loader (utils.py:11-31): first 10 000
documents of RedPajama-1T-Sample, tokenised to a fixed length with padding (pad = eos), labels = input ids
shifted left by one with the pad id appended.  Needs network access and the ``datasets`` package."""
from __future__ import annotations


def hf_token_stream(model_name: str, max_length: int, batch_size: int, plugin, seed: int = 0):
    from datasets import load_dataset
    from transformers import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(model_name, trust_remote_code=True)
    tok.pad_token = tok.eos_token
    ds = load_dataset("togethercomputer/RedPajama-Data-1T-Sample", split="train[:10000]")

    def encode(ex):
        out = tok(ex["text"], truncation=True, max_length=max_length, padding="max_length")
        out["labels"] = [ids[1:] + [tok.pad_token_id] for ids in out["input_ids"]]
        return out

    ds = ds.map(encode, batched=True, remove_columns=ds.column_names)
    ds.set_format("torch", columns=["input_ids", "labels"])
    loader = plugin.prepare_dataloader(ds, batch_size=batch_size, shuffle=True, drop_last=True, seed=seed)

    def gen():
        while True:
            for b in loader:
                yield {"input_ids": b["input_ids"], "labels": b["labels"]}

    return gen()
