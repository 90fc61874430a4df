"""Tensor-parallel reductions for the row-split projections and the vocab-sharded greedy pick.

Two interchangeable reducers:

* ``NcclReducer``   -- torch.distributed all_reduce / all_gather on the current stream.  The baseline
  and the correctness oracle; works under gloo on CPU too (multi-process tests).
* ``PeerReducer``   -- (``dgpp_b200.parallel.peer``) one-shot all-reduce over NVLink peer memory done by
  our own kernel: every rank pushes its bf16 partial into every peer's symmetric buffer, raises a
  flag, and folds the W partials in ascending rank order in fp32, so all ranks hold bit-identical
  results.  Graph-capturable (epoch counters, no host arm).

Contract (reference: src/net/bus_kernel.cu:361 block_fold_vectors, src/kernels/pick.cu:84-157):
the fold order is rank-ascending fp32 with one final bf16 rounding; the greedy pick keeps the
strictly greater value scanning ranks in ascending order, so ties go to the lowest token id.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class NcclReducer:
    launches_per_all_reduce = 1

    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self._gather_val = None
        self._gather_id = None

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if t.device.type == "cpu" and t.dtype == torch.bfloat16:
            # gloo: fold in fp32, ascending rank order, one rounding -- the same contract as the GPU kernels
            parts = [torch.empty_like(t, dtype=torch.float32) for _ in range(self.world)]
            dist.all_gather(parts, t.float(), group=self.group)
            acc = parts[0].clone()
            for p in parts[1:]:
                acc += p
            t.copy_(acc.to(torch.bfloat16))
            return t
        dist.all_reduce(t, group=self.group)
        return t

    def merge_picks(self, ids: torch.Tensor, vals: torch.Tensor) -> None:
        """Every rank holds (best id, best value) of its vocab slice; afterwards every rank holds the
        global pick (ties -> lowest rank -> lowest id)."""
        n = ids.numel()
        if self._gather_val is None or self._gather_val.shape[1] < n:
            self._gather_val = torch.empty(self.world, max(n, 256), dtype=torch.float32, device=ids.device)
            self._gather_id = torch.empty(self.world, max(n, 256), dtype=torch.int32, device=ids.device)
        gv, gi = self._gather_val[:, :n].contiguous(), self._gather_id[:, :n].contiguous()
        dist.all_gather_into_tensor(gv, vals.contiguous(), group=self.group)
        dist.all_gather_into_tensor(gi, ids.contiguous(), group=self.group)
        best = torch.argmax(gv, dim=0)  # first maximal rank
        ids.copy_(gi.gather(0, best.unsqueeze(0)).squeeze(0))
        vals.copy_(gv.gather(0, best.unsqueeze(0)).squeeze(0))
