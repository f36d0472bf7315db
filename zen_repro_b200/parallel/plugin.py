"""Plugin / booster facade with the entry points the reference's training script uses.

``HybridParallelPlugin(tp_size, pp_size=1, precision="bf16", ddp_bucket_cap_mb=...)`` builds the
DP x TP mesh; ``Booster(plugin).boost(model, optimizer, dataloader=...)`` moves the model to the device
in the plugin's precision, wraps it for data parallelism and returns the five-tuple the reference
unpacks (train.py:117-123, 157); the boosted model exposes ``dp_group``, ``tp_group`` and ``module``
(the reducer, with ``register_comm_hook`` and ``device``) as train.py:162-185 expects;
``booster.backward(loss, optimizer)`` runs backward and joins the gradient communication
(train.py:205).  Models are built already sharded (``build_model(..., tp_group=plugin.tp_group)``).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .embedding_sync import EmbeddingRowSync
from .mesh import ProcessGroupMesh
from .reducer import ZenDDP


class HybridParallelPlugin:
    def __init__(self, tp_size: int = 1, pp_size: int = 1, precision: str = "bf16", ddp_bucket_cap_mb: float = 25,
                 sparse_embedding: bool = True, overlap: bool = True, enable_sequence_parallelism: bool = False,
                 sparse_embedding_under_tp: bool = False, dense_transport: str = "nccl"):
        self.tp_size, self.pp_size, self.precision = tp_size, pp_size, precision
        self.enable_sequence_parallelism = enable_sequence_parallelism    # same switch as ColossalAI's plugin
        # row-sparse synchronisation of the vocabulary-sharded embedding gradient over the DP group when TP > 1
        self.sparse_embedding_under_tp = sparse_embedding_under_tp
        self.ddp_bucket_cap_mb = ddp_bucket_cap_mb
        # dense buckets: "nccl" (library all-reduce) or "nvls" (this library's multimem kernel through the NVSwitch)
        self.dense_transport = dense_transport
        self.sparse_embedding = sparse_embedding
        self.overlap = overlap
        self.pg_mesh = ProcessGroupMesh(tp_size, pp_size)
        self.dp_group, self.tp_group = self.pg_mesh.dp_group, self.pg_mesh.tp_group
        self.dp_size, self.dp_rank = self.pg_mesh.dp_size, self.pg_mesh.dp_rank
        self.dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[precision]
        self.device = torch.device(f"cuda:{torch.cuda.current_device()}") if torch.cuda.is_available() else torch.device("cpu")

    def prepare_dataloader(self, dataset, batch_size: int, shuffle: bool = False, drop_last: bool = True, seed: int = 0,
                           **kw):
        """DP-sharded loader over a map-style dataset (train.py:134).  Streams are returned unchanged."""
        if not hasattr(dataset, "__len__"):
            return dataset
        from torch.utils.data import DataLoader
        from torch.utils.data.distributed import DistributedSampler

        sampler = DistributedSampler(dataset, num_replicas=self.dp_size, rank=self.dp_rank, shuffle=shuffle, seed=seed,
                                     drop_last=drop_last)
        return DataLoader(dataset, batch_size=batch_size, sampler=sampler, drop_last=drop_last, pin_memory=torch.cuda.is_available(), **kw)


class BoostedModel(nn.Module):
    def __init__(self, ddp: ZenDDP, plugin: HybridParallelPlugin):
        super().__init__()
        self.module = ddp
        self.dp_group, self.tp_group = plugin.dp_group, plugin.tp_group

    def forward(self, *a, **kw):
        return self.module(*a, **kw)

    def unwrap(self):
        return self.module.module


class Booster:
    def __init__(self, plugin: HybridParallelPlugin):
        self.plugin = plugin
        self._models: list = []

    def boost(self, model, optimizer=None, criterion=None, dataloader=None, lr_scheduler=None, max_tokens: int | None = None):
        pl = self.plugin
        if isinstance(model, BoostedModel):
            return model, optimizer, criterion, dataloader, lr_scheduler
        model = model.to(device=pl.device, dtype=pl.dtype)
        if pl.enable_sequence_parallelism and pl.tp_size > 1 and hasattr(model, "enable_sequence_parallel"):
            model.enable_sequence_parallel()
        emb_sync = None
        wte = getattr(model, "wte", None)
        if pl.sparse_embedding and wte is not None and (pl.tp_size == 1 or pl.sparse_embedding_under_tp) and max_tokens:
            emb_sync = EmbeddingRowSync(wte.shape[0], wte.shape[1], max_tokens, pl.dp_group, dtype=pl.dtype,
                                        device=pl.device)
            emb_sync.target_param = wte
            model.sparse_sink = emb_sync
            if getattr(model, "lm_head", None) is not None:
                wte.zen_sparse_only = True
            else:
                wte.zen_early = True         # tied: only the LM-head product is left in the dense gradient
        ddp = ZenDDP(model, pl.dp_group, pl.ddp_bucket_cap_mb, emb_sync, overlap=pl.overlap,
                     dense_transport=pl.dense_transport)
        if emb_sync is not None:
            emb_sync.prepare(pl.device)
        if optimizer is not None:
            # the optimizer was built on the unboosted parameters; they were moved in place by .to() only when
            # device/dtype did not change, so rebind the groups to the live parameters
            live = [p for p in model.parameters() if p.requires_grad]
            flat = [p for g in optimizer.param_groups for p in g["params"]]
            if len(flat) == len(live) and any(a is not b for a, b in zip(flat, live)):
                it = iter(live)
                for g in optimizer.param_groups:
                    g["params"] = [next(it) for _ in g["params"]]
        boosted = BoostedModel(ddp, pl)
        self._models.append(boosted)
        return boosted, optimizer, criterion, dataloader, lr_scheduler

    def backward(self, loss: torch.Tensor, optimizer=None) -> None:
        """Backward pass, then join the bucket communication and apply the sparse embedding rows."""
        loss.backward()
        for m in self._models:
            m.module.finalize_grads()
