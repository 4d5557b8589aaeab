"""Refit broadcast of quantised bundle state between two gloo ranks on CPU."""

from __future__ import annotations

import os
import tempfile

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import nn

from embodiinfer_b200.refit import BroadcastWeightSync


class Bundle(nn.Module):
    """Buffers shaped like an NVFP4Linear's: packed codes, block scales, a global scale, a bf16 bias."""

    def __init__(self, seed: int) -> None:
        super().__init__()
        generator = torch.Generator().manual_seed(seed)
        self.register_buffer("weight", torch.randint(0, 256, (64, 32), dtype=torch.uint8, generator=generator))
        self.register_buffer("weight_scale", torch.randint(0, 127, (64, 4), dtype=torch.uint8, generator=generator))
        self.register_buffer("weight_global_scale", torch.rand((), generator=generator))
        self.bias = nn.Parameter(torch.randn(64, generator=generator).to(torch.bfloat16), requires_grad=False)
        self.inner = nn.Linear(8, 8)
        with torch.no_grad():
            self.inner.weight.copy_(torch.randn(8, 8, generator=generator))
        # what a calibrated plan holds outside the state dict: packed codes (e4m3) and a derived copy
        self.plan_codes = torch.randint(0, 120, (16, 8), dtype=torch.uint8, generator=generator).view(torch.float8_e4m3fn)
        self.derived = self.plan_codes.view(torch.uint8).clone()

    def refit_tensors(self):
        return {"proj.weight": self.plan_codes}


def _worker(rank: int, world: int, init_file: str, results) -> None:
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world)
    try:
        module = Bundle(seed=100 + rank)                      # every rank starts from different weights
        pointers = {name: tensor.data_ptr() for name, tensor in module.state_dict(keep_vars=True).items()}
        seen_versions = []

        def rebuild_derived():                                 # runs after the copies, before the version advances
            seen_versions.append(sync.policy_version)
            module.derived.copy_(module.plan_codes.view(torch.uint8))

        plan_pointer = module.plan_codes.data_ptr()
        sync = BroadcastWeightSync(module, src_rank=0, bucket_bytes=1024, on_refit=[rebuild_derived])      # small buckets: several broadcasts per dtype
        count = sync.update()
        assert sync.policy_version == 1 and count >= 4 and seen_versions == [0]
        # the plan's packed operand (not in the state dict) was refreshed in place, and the derived state with it
        assert module.plan_codes.data_ptr() == plan_pointer
        assert torch.equal(module.plan_codes.view(torch.uint8), Bundle(seed=100).plan_codes.view(torch.uint8))
        assert torch.equal(module.derived, Bundle(seed=100).plan_codes.view(torch.uint8))
        assert all(tensor.data_ptr() == pointers[name] for name, tensor in module.state_dict(keep_vars=True).items()), "in place"
        reference = Bundle(seed=100)
        for name, tensor in module.state_dict().items():
            assert torch.equal(tensor, reference.state_dict()[name]) or name == "inner.bias", name
        sync.update(["bias"])
        assert sync.policy_version == 2
        results.put((rank, "ok"))
    except Exception as error:                                # reported to the parent instead of a silent exit code
        results.put((rank, repr(error)))
    finally:
        dist.destroy_process_group()


def test_broadcast_refit_two_ranks():
    context = mp.get_context("spawn")
    results = context.Queue()
    with tempfile.TemporaryDirectory() as directory:
        init_file = os.path.join(directory, "rendezvous")
        workers = [context.Process(target=_worker, args=(rank, 2, init_file, results)) for rank in range(2)]
        for worker in workers:
            worker.start()
        outcomes = dict(results.get(timeout=120) for _ in workers)
        for worker in workers:
            worker.join(timeout=60)
    assert outcomes == {0: "ok", 1: "ok"}, outcomes
