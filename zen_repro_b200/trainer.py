"""Training engine: the public entry point that scripts, the benchmark and the smoke test share.

    trainer = Trainer(TrainConfig(model="gpt2", micro_batch=8, seq_len=1024))
    loss = trainer.step(next(trainer.data))          # H2D copy, forward, backward, gradient sync, AdamW, loss read

It wires together what the reference's ``train.py`` assembles by hand (plugin, booster, model,
optimizer, hook registration: train.py:109-185) and runs the same loop body (train.py:198-211).
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass

import torch
import torch.distributed as dist

from .data import ZipfTokenStream
from .models import build_model, get_config
from .optim import FusedAdamW
from .parallel import Booster, DistCoordinator, HybridParallelPlugin, launch_from_torch, make_zen_comm_hook
from .utils.trace import trace_range


@dataclass
class TrainConfig:
    model: str = "gpt2"
    micro_batch: int = 8
    seq_len: int = 1024
    tp: int = 1
    method: int = 0                   # 0 dense buckets (+ sparse embedding rows); 1/2/3 ZEN top-k hook on all buckets
    top_k: float = 1.0
    bucket_cap_mb: float = 64.0
    sparse_embedding: bool = True
    grad_checkpoint: bool = False
    lr: float = 1e-3
    weight_decay: float = 0.0
    zipf_s: float = 1.1
    seed: int = 0
    num_layers: int | None = None
    kv_heads: int | None = None
    precision: str = "bf16"
    data_pool: int = 8                # pre-generated pinned batches that the stream cycles through (0 = generate per step)
    overlap: bool = True
    fused_tp: bool = True             # TP all-reduces fused into the GEMM epilogues (peer memory) instead of NCCL
    sequence_parallel: bool = False   # TP with the residual stream sharded over tokens: all-gather + GEMM / GEMM + reduce-scatter
    sparse_embedding_under_tp: bool = False   # TP > 1: sync the vocabulary-sharded embedding gradient as sparse rows over DP
    heartbeat_s: float = 0.0          # > 0: host heartbeat between ranks, checked before every step (PeerLost is raised)
    cuda_graph: bool = False          # capture forward + backward + sync + optimizer once, then replay it every step
    graph_warmup: int = 2             # real steps launched from the host before the capture
    dense_transport: str = "auto"     # dense buckets: "nccl" (library all-reduce), "nvls" (own multimem kernel through the
                                      # NVSwitch), "auto" = nvls for pure data-parallel runs when the fabric has multicast
    status_mirror: bool = True        # mirror the kernels' status words to the host every step (read one step late)
    on_sync_error: str = "recover"    # "recover": resync the replicas and switch the failing path to its library form;
                                      # "raise": stop with SyncStatusError

    def to_dict(self):
        return dataclasses.asdict(self)


class Trainer:
    def __init__(self, cfg: TrainConfig, init_dist: bool = True):
        self.cfg = cfg
        if init_dist and not dist.is_initialized():
            launch_from_torch()
        self.coordinator = DistCoordinator()
        self.plugin = HybridParallelPlugin(tp_size=cfg.tp, pp_size=1, precision=cfg.precision,
                                           ddp_bucket_cap_mb=cfg.bucket_cap_mb,
                                           sparse_embedding=cfg.sparse_embedding and cfg.method == 0, overlap=cfg.overlap,
                                           sparse_embedding_under_tp=cfg.sparse_embedding_under_tp,
                                           dense_transport=("nvls" if cfg.tp == 1 else "nccl") if cfg.dense_transport == "auto"
                                           else cfg.dense_transport)
        self.booster = Booster(self.plugin)
        self.device = self.plugin.device
        mc = get_config(cfg.model, num_layers=cfg.num_layers, num_kv_heads=cfg.kv_heads,
                        grad_checkpoint=cfg.grad_checkpoint or None)
        self.model_cfg = mc
        torch.manual_seed(cfg.seed)
        model = build_model(mc, tp_group=self.plugin.tp_group if cfg.tp > 1 else None, device=self.device,
                            dtype=self.plugin.dtype)
        model.reset_parameters(seed=cfg.seed + 1000 * self.plugin.pg_mesh.tp_rank)
        if cfg.tp > 1 and self.device.type == "cuda" and cfg.fused_tp:
            model.enable_fused_tp(cfg.micro_batch * cfg.seq_len)
        if cfg.tp > 1 and cfg.sequence_parallel:
            model.enable_sequence_parallel()
        optimizer = FusedAdamW(model.parameters(), lr=cfg.lr, weight_decay=cfg.weight_decay)
        self.data = ZipfTokenStream(mc.vocab_size, cfg.seq_len, cfg.micro_batch, s=cfg.zipf_s, seed=cfg.seed,
                                    dp_rank=self.plugin.dp_rank, pool=cfg.data_pool)
        self.model, self.optimizer, _, _, _ = self.booster.boost(model, optimizer, dataloader=self.data,
                                                                 max_tokens=cfg.micro_batch * cfg.seq_len)
        if cfg.method != 0:
            hook = make_zen_comm_hook(self.model.dp_group, self.model.tp_group, top_k=cfg.top_k, method=cfg.method,
                                      torch_future=False)
            if self.device.type == "cuda" and self.plugin.dp_size > 1:
                for b in self.model.module.buckets:          # allocate peer buffers outside backward
                    if b.buffer.numel() > 4096:
                        hook.engine_for(b.buffer.numel(), self.device)
            self.model.module.register_comm_hook(None, hook)
            self._hook = hook
        self.step_count = 0                  # optimizer steps since the start of training (restored by a resume)
        self._steps_here = 0                 # steps run by this process; the graph capture waits for graph_warmup of them
        self.heartbeat = None
        if cfg.heartbeat_s > 0 and dist.is_initialized() and dist.get_world_size() > 1:
            from .parallel.failure import Heartbeat

            self.heartbeat = Heartbeat(interval=cfg.heartbeat_s / 4, timeout=cfg.heartbeat_s)
        self.health = None
        self.recoveries: list = []
        if cfg.status_mirror:
            from .parallel.health import StatusMirror

            self.health = StatusMirror(self.device, self.plugin.dp_group if dist.is_initialized() else None)
            emb = self.model.module.embedding_sync
            if emb is not None and emb._engine is not None:
                self.health.add("embedding_rows", emb._engine.state.status_t)
            if getattr(self, "_hook", None) is not None:
                for numel, eng in self._hook.state["engines"].items():
                    self.health.add(f"sparse_{numel}", eng.rank_state.status_t)
            ws = getattr(self.model.unwrap(), "tp_ws", None)
            if ws is not None:
                self.health.add("tp_fused", ws.status)
            if getattr(self.model.module, "arena", None) is not None:
                self.health.add("dense_nvls", self.model.module.arena.status)
        self._graph = None
        self.graph_launches_per_step = 0
        self._static_ids = self._static_loss = None
        self.graph_ok = cfg.cuda_graph and self.device.type == "cuda"
        if self.graph_ok:
            # everything a replayed step must see change lives on the device: AdamW's step count and the call counters
            # of the sparse engines (row granule for the embedding, element granule for the top-k hook)
            self.optimizer.enable_device_step(self.device)
            emb = self.model.module.embedding_sync
            if emb is not None and emb._engine is not None:
                emb._engine.enable_device_epoch()
            if getattr(self, "_hook", None) is not None:
                for eng in self._hook.state["engines"].values():
                    eng.enable_device_epoch()

    @property
    def tokens_per_step(self) -> int:
        """Tokens consumed per optimizer step by the whole job."""
        return self.cfg.micro_batch * self.cfg.seq_len * self.plugin.dp_size

    def step(self, batch: dict, read_loss: bool = True):
        """One optimizer step on a host batch.  Returns the loss as a float (read_loss) or a device tensor."""
        if self.heartbeat is not None:
            self.heartbeat.assert_alive()        # a peer that left between steps is noticed here, before any launch
        with trace_range("h2d"):
            ids = batch["input_ids"].to(self.device, non_blocking=True)
            labels = batch["labels"].to(self.device, non_blocking=True) if batch["labels"] is not batch["input_ids"] else ids
        return self.step_device(ids, labels, read_loss)

    def _capture(self, ids: torch.Tensor):
        """Capture one full training step (forward, backward, gradient synchronisation, AdamW, zero-grad) in a CUDA
        graph.  Everything the step reads at run time lives on the device: the token buffer, the optimizer's step
        count and the sparse engine's call counter."""
        self._static_ids = ids.clone()
        ws = getattr(self.model.unwrap(), "tp_ws", None)
        if ws is not None and ws._step_dev is None:
            # the fused TP GEMMs counted their calls during the eager steps; from here on the counter lives on the device
            even = ws.enable_device_epoch(ws.calls_in_step or ws.calls_last_step)
            if self.cfg.sequence_parallel and not even:
                self.graph_ok = False
                ws._step_dev, ws.ctx.epoch_dev = None, None
                return False
        torch.cuda.synchronize()
        from . import _native

        g = torch.cuda.CUDAGraph()
        before = _native.launch_count()
        published = self.health.published if self.health is not None else 0
        with torch.cuda.graph(g):
            self._static_loss = self._eager_step(self._static_ids, self._static_ids)
        if self.health is not None:
            self.health.published = published      # recorded, not run: the host counts a publish at every replay instead
        self.graph_launches_per_step = _native.launch_count() - before      # this library's kernels inside the graph
        self._graph = g
        return True

    def _recover(self, bad: dict) -> None:
        """A communication kernel reported overflow or an expired wait in an earlier step (same step and same value on
        every rank).  That step used incomplete gradients on some rank, so the replicas may differ: re-broadcast
        parameters and optimizer state from data-parallel rank 0, switch the failing path to its library form (dense
        all-reduce of the thresholded bucket, all-gather of the embedding rows, NCCL all-reduce after the TP GEMMs) and
        go on.  The step is no longer replayed from a graph afterwards."""
        from .parallel.health import SyncStatusError, decode

        msg = ", ".join(f"{k}: {decode(v)}" for k, v in bad.items())
        if self.cfg.on_sync_error == "raise":
            raise SyncStatusError(f"gradient synchronisation reported errors: {msg}")
        self.coordinator.print_on_master(f"[zen] step {self.step_count}: {msg}; resynchronising replicas and falling back")
        self._graph = None
        self.graph_ok = False
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        if dist.is_initialized() and self.plugin.dp_size > 1:
            src = dist.get_global_rank(self.plugin.dp_group, 0) if self.plugin.dp_group is not None else 0
            for p in self.model.parameters():
                dist.broadcast(p.data, src, group=self.plugin.dp_group)
                for v in self.optimizer.state.get(p, {}).values():
                    if torch.is_tensor(v):
                        dist.broadcast(v, src, group=self.plugin.dp_group)
        for name in bad:
            if name == "embedding_rows":
                self.model.module.embedding_sync.force_library = True
            elif name == "tp_fused":
                self.model.unwrap().disable_fused_tp()
            elif name == "dense_nvls":
                self.model.module.arena = None            # the buckets stay where they are; the library all-reduce takes over
            elif getattr(self, "_hook", None) is not None:
                self._hook.state["force_dense"] = True
        self.health.clear()
        self.recoveries.append({"step": self.step_count, "status": dict(bad)})

    def step_device(self, ids: torch.Tensor, labels: torch.Tensor, read_loss: bool = False):
        if self.health is not None and self.health.sources:
            bad = self.health.poll()
            if bad:
                self._recover(bad)
        if self.graph_ok and labels is ids and self._steps_here >= self.cfg.graph_warmup:
            if self._graph is None and not self._capture(ids):   # the first steps ran eagerly (tables, scratch, peers): record now
                return self.step_device(ids, labels, read_loss)
            self._static_ids.copy_(ids, non_blocking=True)
            self._graph.replay()
            if self.health is not None and self.health.sources:
                self.health.published += 1         # the replayed step published its status words
            self.step_count += 1
            self._steps_here += 1
            return float(self._static_loss.item()) if read_loss else self._static_loss
        loss = self._eager_step(ids, labels)
        self.step_count += 1
        self._steps_here += 1
        return float(loss.item()) if read_loss else loss

    def _eager_step(self, ids: torch.Tensor, labels: torch.Tensor):
        ws = getattr(self.model.unwrap(), "tp_ws", None)
        if ws is not None:
            ws.begin_step()
        with trace_range("forward"):
            loss = self.model(ids, labels)
        with trace_range("backward"):
            self.booster.backward(loss, self.optimizer)
        if self.health is not None and self.health.sources:
            self.health.publish()
        with trace_range("optimizer_step"):
            self.optimizer.step()
            self.model.module.zero_grad()
        return loss.detach()

    def check_health(self, raise_on_error: bool = True) -> dict:
        """Read (and clear) the status words that the kernels set instead of faulting: capacity overflow or an expired
        wait in the sparse engines (element and row granule) and in the fused tensor-parallel GEMMs, and the error
        codes of the tcgen05 GEMM / attention kernels.  Synchronises the device; meant for every N-th step and the end
        of a run, not for the hot loop.  Non-zero entries mean that a step used incomplete data."""
        out = {}
        if self.device.type != "cuda":
            return out
        from .ops import attention as A
        from .ops import gemm as G

        torch.cuda.synchronize()
        out["gemm"] = int(G.gemm_error())
        out["attention"] = int(A.attention_error())
        emb = getattr(self.model.module, "embedding_sync", None)
        if emb is not None:
            out["embedding_rows"] = int(emb.check())
        hook = getattr(self, "_hook", None)
        if hook is not None:
            for numel, eng in hook.state["engines"].items():
                out[f"sparse_{numel}"] = int(eng.check())
        ws = getattr(self.model.unwrap(), "tp_ws", None)
        if ws is not None:
            out["tp_fused"] = int(ws.check())
        arena = getattr(self.model.module, "arena", None)
        if arena is not None:
            out["dense_nvls"] = int(arena.check())
        bad = {k: v for k, v in out.items() if v}
        if bad and raise_on_error:
            raise RuntimeError(f"kernel status words report errors: {bad} (1 = record overflow, 2 = gather overflow, "
                               f"4 = wait expired, 8 = overflow at a peer, 16 = bad argument)")
        return out

    def collect_metrics(self) -> dict:
        """Counters of the sparse synchronisation paths after the last step: density of what was sent, density of the
        union, load balance across owners (max / mean of the records each owner received), bytes pushed over the links,
        index formats, reported overflow / timeout bits and the number of fallbacks so far.  Synchronises the device
        and runs one small all-gather: every rank calls it at the same step (every N-th step, not in the hot loop)."""
        out: dict = {"optimizer_steps": self.step_count, "recoveries": len(self.recoveries)}
        if self.health is not None:
            out["status_bits"] = dict(self.health.last)
        world = self.plugin.dp_size
        emb = getattr(self.model.module, "embedding_sync", None)
        if emb is not None and emb.last_count is not None:
            rows = int(emb.last_count.item())
            out["embedding_rows_sent"] = rows
            out["embedding_row_density"] = rows / emb.vocab
            out["embedding_bytes_pushed"] = rows * (emb.d * 2 + 4)
        hook = getattr(self, "_hook", None)
        if hook is not None:
            out["fallbacks"] = hook.state.get("fallbacks", 0)
            per_bucket = {}
            for numel, eng in hook.state["engines"].items():
                m = eng.metrics()
                loads = torch.tensor([float(m["owner_recv_records"])], device=self.device)
                if world > 1:
                    every = [torch.zeros_like(loads) for _ in range(world)]
                    dist.all_gather(every, loads, group=self.plugin.dp_group)
                    loads = torch.cat(every)
                mean = float(loads.mean())
                m["partition_max_over_mean"] = float(loads.max()) / mean if mean > 0 else 1.0
                m["density_sent"] = float(loads.sum()) / (numel * max(1, world))
                per_bucket[str(numel)] = m
            out["buckets"] = per_bucket
        return out

    def close(self) -> None:
        """Drop the captured graph and release the peer-visible regions (sparse engines, fused TP workspace).  A
        collective over the groups that own those regions: every rank calls it, between steps."""
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        self._graph = None
        self._static_ids = self._static_loss = None
        if self.heartbeat is not None and hasattr(self.heartbeat, "stop"):
            self.heartbeat.stop()
        emb = getattr(self.model.module, "embedding_sync", None)
        if emb is not None and emb._engine is not None:
            emb._engine.close()
            emb._engine = None
        hook = getattr(self, "_hook", None)
        if hook is not None:
            for eng in hook.state["engines"].values():
                eng.close()
            hook.state["engines"].clear()
        ws = getattr(self.model.unwrap(), "tp_ws", None) or getattr(self.model.unwrap(), "_tp_ws_off", None)
        if ws is not None:
            ws.close()

    def bytes_per_step(self, batch: dict) -> tuple[int, int]:
        h2d = batch["input_ids"].numel() * batch["input_ids"].element_size()
        if batch["labels"] is not batch["input_ids"]:
            h2d += batch["labels"].numel() * batch["labels"].element_size()
        return h2d, 4
