"""Data-parallel rollout on CPU ranks (gloo): contiguous sharding, order-preserving gather, failure fencing.
Follows the reference's fake-replica tests (tests/test_data_parallel.py:34-80): no GPU, no model."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from embodiinfer_b200.rollout import DataParallelRollout, ReplicaExecutionError, shard_bounds


def test_shard_bounds_partition_in_order():
    for total in (0, 1, 7, 8, 256, 257):
        for world in (1, 2, 3, 8):
            bounds = [shard_bounds(total, world, rank) for rank in range(world)]
            assert bounds[0][0] == 0 and bounds[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(bounds, bounds[1:]))
            sizes = [end - begin for begin, end in bounds]
            assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)
    with pytest.raises(ValueError):
        shard_bounds(4, 2, 2)


def test_single_process_rollout_echoes_order():
    def policy(observations):
        return observations["tag"].float()[:, None, None].expand(-1, 10, 32)

    rollout = DataParallelRollout(policy)
    result = rollout.run({"tag": torch.arange(5)}, request_ids=[f"req{i}" for i in range(5)])
    assert result.actions[:, 0, 0].tolist() == [0.0, 1.0, 2.0, 3.0, 4.0]
    assert result.request_ids == ["req0", "req1", "req2", "req3", "req4"] and result.owner_rank == [0] * 5
    with pytest.raises(ValueError, match="request_ids length"):
        rollout.run({"tag": torch.arange(5)}, request_ids=["a"])

    def broken(observations):
        raise RuntimeError("device lost")

    failing = DataParallelRollout(broken)
    with pytest.raises(ReplicaExecutionError) as info:
        failing.run({"tag": torch.arange(3)})
    assert info.value.failed_ranks == (0,) and not failing.healthy
    with pytest.raises(ReplicaExecutionError):       # stays fenced
        failing.run({"tag": torch.arange(3)})


def test_healthy_shards_skip_fenced_ranks():
    from embodiinfer_b200.rollout import healthy_shard_bounds

    healthy = [True, False, True, True]
    bounds = [healthy_shard_bounds(10, healthy, rank) for rank in range(4)]
    assert bounds == [(0, 4), (4, 4), (4, 7), (7, 10)]                       # rank 1 serves nothing, order is kept
    assert [healthy_shard_bounds(5, [False, True], rank) for rank in range(2)] == [(0, 0), (0, 5)]
    assert [healthy_shard_bounds(5, [True, False], rank) for rank in range(2)] == [(0, 5), (5, 5)]
    with pytest.raises(ReplicaExecutionError, match="every replica is fenced"):
        healthy_shard_bounds(5, [False, False], 0)


def test_expired_device_wait_is_reported_and_cleared():
    """The status word every tensor-core launch receives: a non-zero code (here written by hand, as an expired
    bounded wait would) raises at the next check, names the wait, and is cleared."""
    from embodiinfer_b200 import kernels as K

    device = torch.device("cuda", 0)
    K._status_words[0] = torch.tensor([0x102], dtype=torch.int32)            # a host tensor stands in for the device word
    try:
        with pytest.raises(RuntimeError, match=r"status 0x102: the MMA issuer waited for a filled stage"):
            K.check_status(device)
        K.check_status(device)                                                 # cleared
        seen = []
        rollout = DataParallelRollout(lambda obs: obs["tag"].float()[:, None, None].expand(-1, 10, 32),
                                      status_check=lambda: K.check_status(device))
        K._status_words[0][0] = 0x104
        with pytest.raises(ReplicaExecutionError) as info:                     # the replica is fenced like any failing one
            rollout.run({"tag": torch.arange(3)})
        assert "0x104" in str(info.value.__cause__) and not rollout.healthy and not seen
    finally:
        del K._status_words[0]


def _free_port() -> int:
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def _worker(rank: int, world: int, port: int, total: int, fail_rank: int, results) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        def policy(observations):
            if rank == fail_rank:
                raise RuntimeError("injected replica failure")
            tags = observations["tag"].float()
            return torch.stack((tags, torch.full_like(tags, float(rank))), dim=-1)[:, None, :].expand(-1, 10, 2).contiguous()

        rollout = DataParallelRollout(policy, horizon=10, action_dim=2)
        try:
            result = rollout.run({"tag": torch.arange(total)}, request_ids=[f"id{i}" for i in range(total)])
            results[rank] = ("ok", result.actions[:, 0, 0].tolist(), result.actions[:, 3, 1].tolist(), result.owner_rank, result.request_ids)
        except ReplicaExecutionError as error:
            results[rank] = ("failed", error.failed_ranks)
    finally:
        dist.destroy_process_group()


def _run(world: int, total: int, fail_rank: int = -1):
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), total, fail_rank, results), nprocs=world, join=True)
    return dict(results)


@pytest.mark.parametrize("total", (7, 8, 1))
def test_two_rank_gather_preserves_caller_order(total):
    results = _run(2, total)
    for rank in (0, 1):
        status, tags, owners_from_actions, owner, ids = results[rank]
        assert status == "ok"
        assert tags == [float(i) for i in range(total)]            # caller order
        assert owners_from_actions == [float(r) for r in owner]    # each row came from its shard's rank
        assert owner == [0] * ((total + 1) // 2) + [1] * (total // 2)
        assert ids == [f"id{i}" for i in range(total)]


def test_failure_on_one_rank_fails_the_call_everywhere():
    results = _run(2, 6, fail_rank=1)
    assert results[0] == ("failed", (1,)) and results[1] == ("failed", (1,))


def _fencing_worker(rank: int, world: int, port: int, results) -> None:
    """Rank 1 fails in the first call; the second call is served by ranks 0 and 2; rank 2 then leaves between
    steps and the third call reports it instead of blocking."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    calls = {"n": 0}

    def policy(observations):
        calls["n"] += 1
        if rank == 1 and calls["n"] == 1:
            raise RuntimeError("injected replica failure")
        tags = observations["tag"].float()
        return torch.stack((tags, torch.full_like(tags, float(rank))), dim=-1)[:, None, :].expand(-1, 10, 2).contiguous()

    rollout = DataParallelRollout(policy, horizon=10, action_dim=2, timeout=5.0)
    batch = {"tag": torch.arange(7)}
    log = []
    try:
        rollout.run(batch)
    except ReplicaExecutionError as error:
        log.append(("first", error.failed_ranks))
    second = rollout.run(batch)                       # the fenced rank takes part in the gather with an empty shard
    log.append(("second", second.actions[:, 0, 0].tolist(), second.owner_rank, list(rollout.healthy_ranks), calls["n"]))
    if rank == 2:                                     # leaves between steps: none of its collectives is in flight
        results[rank] = log
        dist.destroy_process_group()
        return
    try:
        rollout.run(batch)
        log.append(("third", "returned"))
    except ReplicaExecutionError as error:
        log.append(("third", error.failed_ranks))
    results[rank] = log
    try:
        dist.destroy_process_group()
    except Exception:
        pass


def test_fenced_replica_is_skipped_and_a_departed_rank_is_reported():
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_fencing_worker, args=(3, _free_port(), results), nprocs=3, join=True)
    for rank in range(3):
        log = results[rank]
        assert log[0] == ("first", (1,))
        name, tags, owner, healthy, calls = log[1]
        assert tags == [float(i) for i in range(7)]                    # caller order, nothing missing
        assert owner == [0, 0, 0, 0, 2, 2, 2] and healthy == [True, False, True]
        assert calls == (1 if rank == 1 else 2)                        # the fenced replica was not asked again
    for rank in (0, 1):
        assert results[rank][2][0] == "third" and results[rank][2][1] != "returned"      # reported, not blocked
