"""Data-parallel rollout: one process per GPU, weights replicated, observations sharded, ONE gather.

Behavioural counterpart of the reference's ``DataParallelEngine`` (embodiinfer/engine/parallel/
data_parallel.py:422-517): every observation is served by exactly one replica, results come back in
the caller's order with the caller's request ids, a failing replica makes the call fail with
``ReplicaExecutionError`` instead of returning partial results, and a replica that failed is fenced: later
calls are served by the healthy replicas only (data_parallel.py:227, 578).  The reference runs its replicas as
threads of one process and collects Python lists on the host; here each replica is a rank of a
``torch.distributed`` group, shards are contiguous over the healthy ranks (so rank order is caller order) and
the only collective of a call is one ``all_gather_into_tensor``.

What is gathered is a fixed-size record per rank: ``slots`` action chunks of ``[horizon, action_dim]`` fp32
followed by a two-word header (failed flag, rows produced).  Every rank therefore learns
of a failure from the same collective that carries the actions, on the host side of the step; no kernel waits
on another rank.  A rank whose process has gone makes the collective fail or time out; that is reported as a
``ReplicaExecutionError`` too (the group is then unusable and has to be rebuilt by the caller).
"""

from __future__ import annotations

from collections.abc import Callable, Sequence
from dataclasses import dataclass
from datetime import timedelta

import torch
import torch.distributed as dist

HEADER_WORDS = 2      # failed (0/1), rows produced


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


def healthy_shard_bounds(total: int, healthy: Sequence[bool], rank: int) -> tuple[int, int]:
    """Shard of ``rank`` when only the ranks marked healthy take observations: the healthy ranks split the batch
    in rank order, a fenced rank gets the empty shard at the position where its shard would start."""
    if not 0 <= rank < len(healthy):
        raise ValueError("need 0 <= rank < world")
    serving = [index for index, ok in enumerate(healthy) if ok]
    if not serving:
        raise ReplicaExecutionError(tuple(range(len(healthy))), "every replica is fenced; no replica can serve the batch")
    if healthy[rank]:
        return shard_bounds(total, len(serving), serving.index(rank))
    position = sum(1 for index in serving if index < rank)
    edge = shard_bounds(total, len(serving), position)[0] if position < len(serving) else total
    return edge, edge


@dataclass
class RolloutResult:
    actions: torch.Tensor          # [total, horizon, action_dim] fp32, caller order, on this rank's device
    request_ids: list[str]         # caller's ids, same order
    owner_rank: list[int]          # which replica produced each row


class DataParallelRollout:
    """Run ``policy(observations_shard) -> [n, horizon, action_dim]`` on every healthy rank and gather.

    ``policy`` is this rank's replica (weights already on its device).  ``observations`` is any
    indexable batch (a tensor or a dict of tensors sharing dimension 0); every rank passes the same
    full batch (or at least its own shard's rows) and receives the full result.  ``horizon`` and
    ``action_dim`` fix the gathered record (a rank with an empty shard has no output to learn them from).
    ``status_check`` is called after the policy ran and before the gather; it raises when a kernel of this
    rank reported an expired wait (default on CUDA: ``embodiinfer_b200.kernels.check_status``).
    ``timeout`` (seconds) bounds the gather on back ends that support a per-call limit (gloo); with NCCL the
    limit is the process group's own timeout.
    """

    def __init__(self, policy: Callable[..., torch.Tensor], *, group: dist.ProcessGroup | None = None,
                 device: torch.device | None = None, horizon: int = 10, action_dim: int = 32,
                 status_check: Callable[[], None] | None = None, timeout: float | None = None) -> None:
        self.policy = policy
        self.group = group
        self.distributed = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if self.distributed else 1
        self.rank = dist.get_rank(group) if self.distributed else 0
        self.device = device or torch.device("cpu")
        self.horizon, self.action_dim = horizon, action_dim
        self.timeout = timeout
        self.healthy_ranks = [True] * self.world      # the same on every rank: updated from each call's gather
        if status_check is None and self.device.type == "cuda":
            from . import kernels

            status_check = lambda: kernels.check_status(self.device)
        self.status_check = status_check

    @property
    def healthy(self) -> bool:
        return self.healthy_ranks[self.rank]

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

    def _gather(self, record: torch.Tensor) -> torch.Tensor:
        gathered = torch.empty(self.world * record.numel(), dtype=torch.float32, device=self.device)
        try:
            work = dist.all_gather_into_tensor(gathered, record, group=self.group, async_op=True)
            if self.timeout is not None and dist.get_backend(self.group) == "gloo":
                work.wait(timedelta(seconds=self.timeout))
            else:
                work.wait()
        except Exception as error:          # a peer is gone or the call timed out: nobody's result is usable
            others = tuple(rank for rank in range(self.world) if rank != self.rank)
            self.healthy_ranks = [rank == self.rank for rank in range(self.world)]
            raise ReplicaExecutionError(others, f"the gather of the action chunks failed ({type(error).__name__}: "
                                                f"{str(error)[:120]}); replica(s) {list(others)} did not answer") from error
        return gathered.view(self.world, record.numel())

    def run(self, observations, request_ids: Sequence[str] | None = None) -> RolloutResult:
        total = self._count(observations)
        if request_ids is None:
            request_ids = [f"r{index}" for index in range(total)]
        elif len(request_ids) != total:
            raise ValueError("request_ids length must match observations length")
        healthy = list(self.healthy_ranks)
        bounds = [healthy_shard_bounds(total, healthy, rank) for rank in range(self.world)]
        begin, end = bounds[self.rank]
        local, failure = None, None
        if end > begin:
            try:
                local = self.policy(self._slice(observations, begin, end))
                if local.ndim != 3 or local.shape[0] != end - begin:
                    raise ValueError("a replica must return [n, horizon, action_dim] for its n observations")
                if self.world > 1 and tuple(local.shape[1:]) != (self.horizon, self.action_dim):
                    raise ValueError(f"a replica must return [n, {self.horizon}, {self.action_dim}] action chunks")
                if self.status_check is not None:
                    self.status_check()
            except Exception as error:      # this replica is fenced from the next call on; the others learn it below
                failure = error
        if self.world == 1:
            if failure is not None:
                self.healthy_ranks = [False]
                raise ReplicaExecutionError((0,)) from failure
            actions = local if local is not None else torch.zeros((0, self.horizon, self.action_dim), device=self.device)
            return RolloutResult(actions.float(), list(request_ids), [0] * total)
        # one fixed-size record per rank: [slots x horizon x action_dim | failed, rows]
        slots = max(1, max(stop - start for start, stop in bounds))
        chunk = self.horizon * self.action_dim
        record = torch.zeros(slots * chunk + HEADER_WORDS, dtype=torch.float32, device=self.device)
        if local is not None and failure is None:
            record[: (end - begin) * chunk] = local.reshape(-1).float()
        record[slots * chunk] = 0.0 if failure is None else 1.0
        record[slots * chunk + 1] = float(end - begin)
        gathered = self._gather(record)
        headers = gathered[:, slots * chunk:].tolist()          # the call's one read of the device
        failed = [rank for rank, header in enumerate(headers) if header[0] != 0.0]
        if failed:
            for rank in failed:
                self.healthy_ranks[rank] = False
            error = ReplicaExecutionError(failed)
            if failure is not None:
                raise error from failure
            raise error
        pieces = [gathered[rank, : (stop - start) * chunk].reshape(stop - start, self.horizon, self.action_dim)
                  for rank, (start, stop) in enumerate(bounds)]
        owner = [rank for rank, (start, stop) in enumerate(bounds) for _ in range(stop - start)]
        return RolloutResult(torch.cat(pieces), list(request_ids), owner)
