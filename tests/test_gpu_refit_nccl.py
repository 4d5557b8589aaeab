"""Weight refit over NCCL between two GPUs: the quantised state of a calibrated plan is broadcast from the learner's
rank and refreshed in place on the replica (counterpart of ``NCCLBroadcastSync``,
embodiinfer/engine/rollout/weight_sync.py:58-80).  Needs two CUDA devices; skipped on a single-GPU box."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import nn

pytestmark = pytest.mark.gpu


class Holder(nn.Module):
    """A module whose only refit state is a calibrated plan's packed operands."""

    def __init__(self, plan) -> None:
        super().__init__()
        self.plan = plan
        self.register_buffer("step", torch.zeros((), device=plan.gate_up.device))

    def refit_tensors(self):
        return self.plan.refit_tensors("mlp.")


def _worker(rank: int, world: int, port: int, results) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        from embodiinfer_b200 import layers as L
        from embodiinfer_b200.backend.mlp import FusedMlpPlan
        from embodiinfer_b200.layers.registry import OperatorRequest
        from embodiinfer_b200.refit import BroadcastWeightSync

        quantizer = L.quantization_backends.get("cuda", OperatorRequest(device, torch.bfloat16, bits=4))
        generator = torch.Generator().manual_seed(100 + rank)          # every rank starts from different weights
        weights = [(0.05 * torch.randn(shape, generator=generator)).to(device=device, dtype=torch.bfloat16)
                   for shape in ((512, 256), (512, 256), (256, 512))]
        plan = FusedMlpPlan(*weights, gate_up_max=6.0, down_max=4.0, gate_up="nvfp4", down="fp8", quantizer=quantizer)
        holder = Holder(plan)
        x = torch.randn((300, 256), generator=torch.Generator().manual_seed(7)).to(device=device, dtype=torch.bfloat16)
        before = plan(x).clone()
        pointers = {name: tensor.data_ptr() for name, tensor in holder.refit_tensors().items()}
        sync = BroadcastWeightSync(holder, src_rank=0, bucket_bytes=64 << 10)
        broadcasts = sync.update()
        torch.cuda.synchronize(device)
        after = plan(x).clone()
        gathered = [torch.empty_like(after) for _ in range(world)]
        dist.all_gather(gathered, after)
        same_everywhere = bool(torch.equal(gathered[0], gathered[1]))
        in_place = pointers == {name: tensor.data_ptr() for name, tensor in holder.refit_tensors().items()}
        changed = not torch.equal(before, after)
        results[rank] = (sync.policy_version, broadcasts >= 2, same_everywhere, in_place, changed)
    finally:
        dist.destroy_process_group()


def test_refit_broadcast_over_nccl():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(2, port, results), nprocs=2, join=True)
    assert results[0] == (1, True, True, True, False)       # the learner keeps its own weights
    assert results[1] == (1, True, True, True, True)        # the replica now computes with the learner's
