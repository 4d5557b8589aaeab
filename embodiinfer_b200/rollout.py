"""Data-parallel rollout: one process per GPU, weights replicated, observations sharded, one gather.

Behavioural counterpart of the reference's ``DataParallelEngine`` (embodiinfer/engine/parallel/
data_parallel.py:422-517): every observation is served by exactly one replica, results come back in
the caller's order with the caller's request ids, and a failing replica makes the call fail with
``ReplicaExecutionError`` instead of returning partial results.  The reference runs its replicas as
threads of one process and collects Python lists on the host; here each replica is a rank of a
``torch.distributed`` group, shards are contiguous (so rank order is caller order) and the only
collective on the data path is one ``all_gather_into_tensor`` of the fp32 action chunks.

A rank learns that another rank failed from a one-word health reduction that precedes the gather, on
the host side of the step: no kernel waits on another rank.
"""

from __future__ import annotations

from collections.abc import Callable, Sequence
from dataclasses import dataclass

import torch
import torch.distributed as dist


class ReplicaExecutionError(RuntimeError):
    """A replica failed; no partial result is returned (data_parallel.py:492-513)."""

    def __init__(self, failed_ranks: Sequence[int], message: str = "") -> None:
        self.failed_ranks = tuple(failed_ranks)
        super().__init__(message or f"replica(s) {list(self.failed_ranks)} failed; no actions were produced")


def shard_bounds(total: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous shard [begin, end) of ``total`` items for ``rank``; the first ``total % world`` ranks
    take one extra item, so concatenating the shards in rank order restores the caller's order."""
    if total < 0 or world <= 0 or not 0 <= rank < world:
        raise ValueError("need total >= 0 and 0 <= rank < world")
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


@dataclass
class RolloutResult:
    actions: torch.Tensor          # [total, horizon, action_dim] fp32, caller order, on this rank's device
    request_ids: list[str]         # caller's ids, same order
    owner_rank: list[int]          # which replica produced each row


class DataParallelRollout:
    """Run ``policy(observations_shard) -> [n, horizon, action_dim]`` on every rank and gather.

    ``policy`` is this rank's replica (weights already on its device).  ``observations`` is any
    indexable batch (a tensor or a dict of tensors sharing dimension 0); every rank passes the same
    full batch (or at least its own shard's rows) and receives the full result.
    """

    def __init__(self, policy: Callable[..., torch.Tensor], *, group: dist.ProcessGroup | None = None,
                 device: torch.device | None = None) -> None:
        self.policy = policy
        self.group = group
        self.distributed = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if self.distributed else 1
        self.rank = dist.get_rank(group) if self.distributed else 0
        self.device = device or torch.device("cpu")
        self.healthy = True

    @staticmethod
    def _slice(observations, begin: int, end: int):
        if isinstance(observations, dict):
            return {key: value[begin:end] for key, value in observations.items()}
        return observations[begin:end]

    @staticmethod
    def _count(observations) -> int:
        if isinstance(observations, dict):
            return len(next(iter(observations.values())))
        return len(observations)

    def run(self, observations, request_ids: Sequence[str] | None = None) -> RolloutResult:
        total = self._count(observations)
        if request_ids is None:
            request_ids = [f"r{index}" for index in range(total)]
        elif len(request_ids) != total:
            raise ValueError("request_ids length must match observations length")
        begin, end = shard_bounds(total, self.world, self.rank)
        local, failure = None, None
        if not self.healthy:
            failure = RuntimeError(f"replica {self.rank} is not healthy")
        elif end > begin:
            try:
                local = self.policy(self._slice(observations, begin, end))
                if local.ndim != 3 or local.shape[0] != end - begin:
                    raise ValueError("a replica must return [n, horizon, action_dim] for its n observations")
            except Exception as error:      # fence this replica off, then tell the others
                self.healthy = False
                failure = error
        # health word first: every rank learns of a failure before it would enter the gather
        flags = torch.zeros(self.world, dtype=torch.int32, device=self.device)
        flags[self.rank] = 0 if failure is None else 1
        if self.distributed and self.world > 1:
            dist.all_reduce(flags, op=dist.ReduceOp.MAX, group=self.group)
        failed = [rank for rank, flag in enumerate(flags.tolist()) if flag]
        if failed:
            error = ReplicaExecutionError(failed)
            if failure is not None:
                raise error from failure
            raise error
        owner = [rank for rank in range(self.world) for _ in range(*shard_bounds(total, self.world, rank))]
        if self.world == 1:
            actions = local if local is not None else torch.zeros((0, 0, 0), device=self.device)
            return RolloutResult(actions.float(), list(request_ids), owner)
        # shapes: every rank has at least the metadata of its own result; share horizon/action_dim
        meta = torch.tensor(list(local.shape[1:]) if local is not None else [0, 0], dtype=torch.int64, device=self.device)
        dist.all_reduce(meta, op=dist.ReduceOp.MAX, group=self.group)
        horizon, action_dim = (int(v) for v in meta.tolist())
        longest = shard_bounds(total, self.world, 0)[1]          # rank 0 holds a longest shard
        padded = torch.zeros((longest, horizon, action_dim), dtype=torch.float32, device=self.device)
        if local is not None:
            padded[: end - begin] = local.float()
        gathered = torch.empty((self.world * longest, horizon, action_dim), dtype=torch.float32, device=self.device)
        dist.all_gather_into_tensor(gathered, padded, group=self.group)
        pieces = []
        for rank in range(self.world):
            rank_begin, rank_end = shard_bounds(total, self.world, rank)
            pieces.append(gathered[rank * longest: rank * longest + (rank_end - rank_begin)])
        return RolloutResult(torch.cat(pieces), list(request_ids), owner)
