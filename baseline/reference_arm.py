"""Reference arm of the benchmark: the unmodified reference code on the same metric and config.

What runs: HuggingFace ``AutoModelForCausalLM.from_config`` (eager attention, gradient checkpointing on, as
train.py:148-155), stock ``torch.nn.parallel.DistributedDataParallel`` over NCCL, and the reference's own
``compress_with_allgather`` (source taken verbatim from its train.py) and ``LoadBalanceAllreduce`` (its comm.py,
DDPbackend.py, tensor_load_balance.py and compiled extension, all loaded from ``baseline/_ref``) wired into a DDP
communication hook exactly as train.py:162-185 does.  ColossalAI, apex and the ``nvtx`` pip package are not
installable offline, so ``Booster``/``HybridParallelPlugin`` are replaced by plain DDP, ``HybridAdam`` by
``torch.optim.Adam(fused=True)`` and ``nvtx`` by a shim; tensor parallelism (ColossalAI shardformer) is therefore
unavailable and configs that need it report so.  Nothing from ``zen_repro_b200`` is imported here.
"""
from __future__ import annotations

import ast
import json
import logging
import math
import os
import subprocess
import sys
import threading
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def _unavailable(why: str):
    print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
    sys.exit(0)


def _load_reference():
    if not os.path.exists(os.path.join(REF, "comm.py")):
        _unavailable("baseline/_ref is not installed (run baseline/install_reference.sh)")
    sys.path.insert(0, os.path.join(HERE, "shims"))
    sys.path.insert(0, REF)
    try:
        import comm  # noqa: F401  (imports DDPbackend, tensor_load_balance, extensions.cuda.functions, functions_cuda)
    except Exception as e:  # pragma: no cover
        _unavailable(f"reference modules failed to import: {type(e).__name__}: {e}")
    src = open(os.path.join(REF, "train.py")).read()
    tree = ast.parse(src)
    ns = {}
    import nvtx
    import torch
    import torch.distributed as dist

    ns.update(torch=torch, dist=dist, math=math, nvtx=nvtx)
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in ("compress_with_allgather", "compress"):
            exec(compile(ast.Module([node], []), os.path.join(REF, "train.py"), "exec"), ns)
    return comm, ns["compress_with_allgather"]


def _hf_config(name: str):
    import transformers

    if name == "gpt2":
        return transformers.GPT2Config()                                   # GPT-2 small defaults
    if name == "gemma-2b":
        return transformers.GemmaConfig(vocab_size=256000, hidden_size=2048, intermediate_size=16384, num_hidden_layers=18,
                                        num_attention_heads=8, num_key_value_heads=1, head_dim=256,
                                        max_position_embeddings=8192)
    return None


def _zipf_batches(vocab, seq, batch, s, seed, rank, n):
    import torch

    w = 1.0 / torch.arange(1, vocab + 1, dtype=torch.float64) ** s
    cdf = torch.cumsum(w / w.sum(), 0)
    out = []
    for i in range(n):
        g = torch.Generator().manual_seed((seed * 1_000_003 + rank) * 1_000_003 + i)
        u = torch.rand(batch * seq, generator=g, dtype=torch.float64)
        out.append(torch.searchsorted(cdf, u).clamp_(max=vocab - 1).view(batch, seq).pin_memory())
    return out


class _Clocks:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, idx):
        self.lines = []
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i", str(idx),
                                       "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: [self.lines.append(l) for l in self.p.stdout], daemon=True).start()
        except Exception:
            self.p = None

    def stop(self):
        if self.p is None:
            return None
        self.p.terminate()
        sm, mx, reasons = [], [], set()
        for l in self.lines:
            f = [x.strip() for x in l.split(",")]
            if len(f) >= 9:
                try:
                    sm.append(float(f[1])); mx.append(float(f[2]))
                except ValueError:
                    continue
                for n, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons)}


def run_reference(args, preset, models=None):
    import torch

    if not torch.cuda.is_available():
        _unavailable("no CUDA device")
    if preset.get("tp", 1) > 1:
        _unavailable("needs tensor parallelism from ColossalAI's shardformer, which cannot be installed offline")
    comm, compress_with_allgather = _load_reference()
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1"); os.environ.setdefault("MASTER_PORT", "29511")
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    out = _measure_reference(args, preset, comm, compress_with_allgather, dev, rank, world, local)
    if out is None:
        _unavailable(f"no HuggingFace config for {preset['model']} in the reference arm")
    if preset["model"] == "gpt2" and models and not getattr(args, "no_extra", False):
        # the second model of the benchmark, measured in the same process after the headline with the same K and W
        try:
            r = _measure_reference(args, models["gemma-2b"], comm, compress_with_allgather, dev, rank, world, local)
            out["extra"] = {"gemma-2b": {k: r[k] for k in ("value", "unit", "ms_per_step", "config", "e2e")}}
        except Exception as ex:
            out["extra"] = {"gemma-2b": {"error": f"{type(ex).__name__}: {ex}"[:300]}}
    if rank == 0:
        print(json.dumps(out), flush=True)
    dist.destroy_process_group()


def _measure_reference(args, preset, comm, compress_with_allgather, dev, rank, world, local):
    import gc

    import torch
    import torch.distributed as dist
    import transformers
    from torch.nn.parallel import DistributedDataParallel as DDP

    cfg = _hf_config(preset["model"])
    if cfg is None:
        return None
    if args.num_layers:
        cfg.num_hidden_layers = args.num_layers
    torch.manual_seed(0)
    model = transformers.AutoModelForCausalLM.from_config(cfg)
    model.gradient_checkpointing_enable()                                  # train.py:153-154 (always on)
    model.config._attn_implementation = "eager"                            # train.py:155
    model = model.to(torch.bfloat16).to(dev)
    optimizer = torch.optim.Adam(model.parameters(), fused=True)           # HybridAdam defaults
    ddp = DDP(model, device_ids=[local], bucket_cap_mb=512)                # train.py:104 default bucket cap
    dp_group = dist.group.WORLD
    tp_groups = [dist.new_group([r]) for r in range(world)]
    tp_group = tp_groups[rank]
    method = args.method if args.method else 3                              # train.py:100 default
    top_k = int(args.top_k) if args.top_k else 1
    logger = logging.getLogger("reference")
    lba = comm.LoadBalanceAllreduce(dp_group, list(range(world)), logger)
    stream = torch.cuda.Stream()
    state = {"skip": True}

    def custom_comm_hook(_state, bucket):                                   # train.py:167-183
        tensors = bucket.buffer()
        future = torch.futures.Future()
        if state["skip"]:
            future.set_result(tensors)
            state["skip"] = False
            return future
        with torch.cuda.stream(stream):
            compressed = compress_with_allgather(top_k, tensors, tp_group)
            if dp_group.size() > 1:
                tensors = lba.zen_sparse_comm(compressed, method)
        future.set_result(tensors)
        return future

    if method != 0:
        ddp.register_comm_hook(None, custom_comm_hook)
    seq, mb = preset["seq_len"], (args.micro_batch or preset["micro_batch"])
    nb = max(4, min(8, args.steps))
    batches = _zipf_batches(cfg.vocab_size, seq, mb, preset["zipf_s"], 0, rank, nb)
    dev_batches = [b.to(dev) for b in batches]

    def step(ids):
        out = ddp(input_ids=ids, labels=ids)
        loss = out[0]
        loss.backward()
        optimizer.step()
        optimizer.zero_grad()
        return loss

    for i in range(args.warmup):
        step(dev_batches[i % nb])
    dist.barrier(); torch.cuda.synchronize()
    clocks = _Clocks(local) if rank == 0 else None
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for i in range(args.steps):
        step(dev_batches[i % nb])
    e.record()
    dist.barrier(); torch.cuda.synchronize()
    ms = s.elapsed_time(e)
    t0 = time.perf_counter()
    for i in range(args.steps):
        loss = step(batches[i % nb].to(dev, non_blocking=True))
        float(loss.item())
    dist.barrier(); torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    ck = clocks.stop() if clocks else None
    t = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = t.tolist()
    tokens = mb * seq * world * args.steps
    out = {"metric": "train tokens/sec", "value": tokens / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
           "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
           "vs_baseline": None, "dtype": "bf16", "data": "synthetic Zipf tokens, random-init weights", "impl": "reference",
           "config": {"model": preset["model"], "global_batch": mb * world, "seq_len": seq, "parallelism": f"dp{world}",
                      "method": method, "top_k": top_k, "grad_checkpoint": True, "attention": "eager",
                      "stand_ins": "torch DDP for ColossalAI plugin, torch Adam(fused) for HybridAdam, nvtx shim"},
           "clocks": ck,
           "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": mb * seq * 8, "d2h_bytes_per_step": 4},
           "gpu_launches": None}
    del ddp, model, optimizer, dev_batches, lba, step, custom_comm_hook
    gc.collect()
    torch.cuda.empty_cache()
    return out
