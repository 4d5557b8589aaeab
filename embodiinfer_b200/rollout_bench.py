"""Observations per second of the data-parallel rollout (the rollout benchmark configuration: 256 observations, synthetic inputs).

    python -m embodiinfer_b200.rollout_bench --observations 256 [--layer-scale 1.0] [--quantization fp8]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m embodiinfer_b200.rollout_bench --observations 256

Every rank builds the same random-init policy (weights replicated), takes its contiguous shard of the
batch (pinned host uint8 frames -> device inside the timed region), runs SigLIP -> prefix -> 10 denoise
steps and joins one NCCL gather (the only collective of a call) of the fixed-size per-rank records that carry
the [n, 10, 32] fp32 action chunks.  Prints one JSON line on rank 0.

``--fused-mlp`` calibrates the Gemma MLPs on the first micro-batch and runs them as the calibrated fused
plan; ``--graphs`` replays one CUDA graph per micro-batch (host-to-device copy of the frames included)
instead of launching every kernel from Python.
"""

from __future__ import annotations

import argparse
import json
import os
import torch
import torch.distributed as dist

from .pi05_shaped import Pi05ShapedPolicy, synthetic_observations
from .rollout import DataParallelRollout


class GraphedReplica:
    """One CUDA graph of the whole policy step for a fixed micro-batch: pinned host staging buffers ->
    device copies -> SigLIP -> prefix -> denoise.  A short last micro-batch is padded with stale rows."""

    def __init__(self, policy: Pi05ShapedPolicy, example: dict, micro_batch: int) -> None:
        device = policy.device_
        self.micro_batch = micro_batch
        self.host = {key: torch.empty((micro_batch, *value.shape[1:]), dtype=value.dtype).pin_memory() for key, value in example.items()}
        self.device = {key: torch.empty_like(value, device=device) for key, value in self.host.items()}
        for key, value in self.host.items():
            value.copy_(example[key][:micro_batch])
        self.noise = policy.noise(micro_batch)
        self.stream = torch.cuda.Stream(device)
        self.stream.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(self.stream):
            for _ in range(2):                      # plan buffers, workspaces, library heuristics: before capture
                self._step(policy)
        self.stream.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=self.stream):
            self.output = self._step(policy)
        torch.cuda.synchronize(device)

    def _step(self, policy: Pi05ShapedPolicy) -> torch.Tensor:
        for key, value in self.host.items():
            self.device[key].copy_(value, non_blocking=True)
        return policy(self.device, self.noise)

    def __call__(self, piece: dict) -> torch.Tensor:
        count = len(piece["tokens"])
        torch.cuda.current_stream().synchronize()           # the previous replay has consumed the staging buffers
        for key, value in piece.items():
            self.host[key][:count].copy_(value)
        self.graph.replay()
        return self.output[:count].clone()


def measure_rollout(device: torch.device, *, observations: int = 256, micro_batch: int = 32, quantization: str = "fp8",
                    layer_scale: float = 1.0, repeats: int = 3, fused_mlp: bool = True, graphs: bool = True,
                    policy: Pi05ShapedPolicy | None = None) -> tuple[dict, Pi05ShapedPolicy]:
    """Observations per second of the 256-observation rollout on the ranks of the initialised process group (or one
    GPU).  Device time: CUDA events around each pass on the launching stream, maximum over ranks, best of ``repeats``.
    Returns the result record (meaningful on rank 0) and the policy, for further measurements on it."""
    world = dist.get_world_size() if dist.is_initialized() else 1
    if policy is None:
        policy = Pi05ShapedPolicy(quantization, device=device, layer_scale=layer_scale)
    batch = synthetic_observations(observations)
    batch = {key: value.pin_memory() for key, value in batch.items()}
    first = {key: value[:micro_batch] for key, value in batch.items()}
    if fused_mlp and not getattr(policy, "calibrated", False):
        policy.calibrate_fused_mlp(first, margin=1.25)
        policy.calibrated = True
    step = GraphedReplica(policy, first, micro_batch) if graphs else policy

    def replica(shard):
        chunks = []
        count = len(shard["tokens"])
        for begin in range(0, count, micro_batch):
            piece = {key: value[begin: begin + micro_batch] for key, value in shard.items()}
            chunks.append(step(piece))
        return torch.cat(chunks)

    rollout = DataParallelRollout(replica, device=device)
    rollout.run(batch)                             # warm-up: workspaces, library heuristics, NCCL
    torch.cuda.synchronize(device)
    milliseconds = []
    result = None
    for _ in range(repeats):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        result = rollout.run(batch)
        stop.record()
        torch.cuda.synchronize(device)
        elapsed = torch.tensor(start.elapsed_time(stop), device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
        milliseconds.append(elapsed.item())
    best = min(milliseconds) * 1e-3
    flops = policy.flops_per_observation() * observations
    record = {
        "metric": "rollout_observations_per_s", "value": observations / best, "unit": "obs/s", "n_gpus": world,
        "observations": observations, "ms": milliseconds, "quantization": quantization,
        "layer_scale": layer_scale, "micro_batch": micro_batch, "scaling": "strong",
        "fused_mlp": fused_mlp, "cuda_graphs": graphs, "collectives_per_call": 1 if world > 1 else 0,
        "quantised_linear_tflops": flops / best / 1e12, "actions_checksum": float(result.actions.double().sum()),
        "gathered_bytes": result.actions.numel() * 4,
        "h2d_bytes_per_observation": sum(value[0].numel() * value.element_size() for value in batch.values()),
    }
    return record, policy


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--observations", type=int, default=256)
    parser.add_argument("--micro-batch", type=int, default=16)
    parser.add_argument("--layer-scale", type=float, default=1.0)
    parser.add_argument("--quantization", default="fp8")
    parser.add_argument("--repeats", type=int, default=3)
    parser.add_argument("--fused-mlp", action="store_true")
    parser.add_argument("--graphs", action="store_true")
    args = parser.parse_args()
    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", 0), ("WORLD_SIZE", 1), ("LOCAL_RANK", 0)))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    record, _ = measure_rollout(device, observations=args.observations, micro_batch=args.micro_batch, quantization=args.quantization,
                                layer_scale=args.layer_scale, repeats=args.repeats, fused_mlp=args.fused_mlp, graphs=args.graphs)
    if rank == 0:
        print(json.dumps(record))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
