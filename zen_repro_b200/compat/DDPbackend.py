"""Collective wrapper with the reference's surface (DDPbackend.py:4-81): ``allgather``, ``allgather_padding``,
``allgatherv`` and ``alltoallv`` over a process group.  Works on NCCL and on gloo (which lacks the list form
of all-to-all, so ``alltoallv`` is built on ``all_to_all_single`` with uneven splits); a group of one rank
returns lists, not bare tensors, so callers need no special case."""
from __future__ import annotations

import torch
import torch.distributed as dist


class DDPBackend:
    def __init__(self, process_group, global_ranks=None, logger=None):
        self.process_group = process_group
        self.group_size = dist.get_world_size(group=process_group)
        self.local_rank = dist.get_rank(group=process_group)
        self.global_ranks = list(global_ranks) if global_ranks is not None else list(range(self.group_size))
        self.logger = logger

    def allgather(self, tensor: torch.Tensor, async_op: bool = True) -> list:
        """Same-size all-gather -> list of ``group_size`` tensors."""
        if self.group_size == 1:
            return [tensor]
        flat = torch.empty((self.group_size,) + tuple(tensor.shape), dtype=tensor.dtype, device=tensor.device)
        work = dist.all_gather_into_tensor(flat.view(-1), tensor.contiguous().view(-1), group=self.process_group,
                                           async_op=async_op)
        if async_op:
            work.wait()
        return list(flat.unbind(0))

    def allgather_padding(self, tensor: torch.Tensor, async_op: bool = True) -> list:
        """Variable-size all-gather: exchange lengths, pad to the maximum, gather, trim."""
        n = torch.tensor([tensor.numel()], dtype=torch.int64, device=tensor.device)
        sizes = [int(s) for s in torch.stack(self.allgather(n, async_op)).view(-1).tolist()]
        if self.group_size == 1:
            return [tensor]
        mx = max(max(sizes), 1)
        padded = torch.zeros(mx, dtype=tensor.dtype, device=tensor.device)
        padded[: tensor.numel()] = tensor.reshape(-1)
        parts = self.allgather(padded, async_op)
        return [p[:s] for p, s in zip(parts, sizes)]

    def allgatherv(self, tensor: torch.Tensor) -> list:
        """Variable-size all-gather by pairwise send/recv, lower rank sends first (DDPbackend.py:46-69)."""
        if self.group_size == 1:
            return [tensor]
        n = torch.tensor([tensor.numel()], dtype=torch.int64, device=tensor.device)
        sizes = [int(s) for s in torch.stack(self.allgather(n)).view(-1).tolist()]
        out = [torch.empty(s, dtype=tensor.dtype, device=tensor.device) for s in sizes]
        out[self.local_rank] = tensor
        reqs = []
        for r in range(self.group_size):
            if r == self.local_rank:
                continue
            peer = self.global_ranks[r]
            ops = [dist.P2POp(dist.isend, tensor, peer, self.process_group), dist.P2POp(dist.irecv, out[r], peer, self.process_group)]
            if r < self.local_rank:
                ops.reverse()
            reqs.extend(dist.batch_isend_irecv(ops))
        for q in reqs:
            q.wait()
        return out

    def alltoallv(self, tensors: list, gather_splits=None) -> list:
        """tensors[p] goes to rank p; returns what every rank sent here.  ``gather_splits`` (the all-gathered split
        table of the reference) is accepted and used for the receive sizes when given."""
        if self.group_size == 1:
            return list(tensors)
        assert len(tensors) == self.group_size
        dev, dtype = tensors[0].device, tensors[0].dtype
        send_counts = [t.numel() for t in tensors]
        if gather_splits is not None:
            recv_counts = [int(s[self.local_rank]) for s in gather_splits]
        else:
            sc = torch.tensor(send_counts, dtype=torch.int64, device=dev)
            rc = torch.empty_like(sc)
            dist.all_to_all_single(rc, sc, group=self.process_group)
            recv_counts = rc.tolist()
        send = torch.cat([t.reshape(-1) for t in tensors])
        recv = torch.empty(sum(recv_counts), dtype=dtype, device=dev)
        dist.all_to_all_single(recv, send, output_split_sizes=recv_counts, input_split_sizes=send_counts,
                               group=self.process_group)
        return list(torch.split(recv, recv_counts))
