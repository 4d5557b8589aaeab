"""Observations per second of the data-parallel rollout (the rollout benchmark configuration: 256 observations, synthetic inputs).

    python -m embodiinfer_b200.rollout_bench --observations 256 [--layer-scale 1.0] [--quantization fp8]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m embodiinfer_b200.rollout_bench --observations 256

Every rank builds the same random-init policy (weights replicated), takes its contiguous shard of the
batch (pinned host uint8 frames -> device inside the timed region), runs SigLIP -> prefix -> 10 denoise
steps and joins one NCCL gather of the [n, 10, 32] fp32 action chunks.  Prints one JSON line on rank 0.

``--fused-mlp`` calibrates the Gemma MLPs on the first micro-batch and runs them as the calibrated fused
plan; ``--graphs`` replays one CUDA graph per micro-batch (host-to-device copy of the frames included)
instead of launching every kernel from Python.
"""

from __future__ import annotations

import argparse
import json
import os
import time

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
    policy = Pi05ShapedPolicy(args.quantization, device=device, layer_scale=args.layer_scale)
    observations = synthetic_observations(args.observations)
    observations = {key: value.pin_memory() for key, value in observations.items()}
    first = {key: value[: args.micro_batch] for key, value in observations.items()}
    if args.fused_mlp:
        policy.calibrate_fused_mlp(first, margin=1.25)
    step = GraphedReplica(policy, first, args.micro_batch) if args.graphs else policy

    def replica(shard):
        chunks = []
        count = len(shard["tokens"])
        for begin in range(0, count, args.micro_batch):
            piece = {key: value[begin: begin + args.micro_batch] for key, value in shard.items()}
            chunks.append(step(piece))
        return torch.cat(chunks)

    rollout = DataParallelRollout(replica, device=device)
    rollout.run(observations)                      # warm-up: workspaces, cuDNN/SDPA heuristics, NCCL
    torch.cuda.synchronize()
    seconds = []
    for _ in range(args.repeats):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        start = time.perf_counter()
        result = rollout.run(observations)
        torch.cuda.synchronize()
        elapsed = torch.tensor(time.perf_counter() - start, device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
        seconds.append(elapsed.item())
    if rank == 0:
        best = min(seconds)
        flops = policy.flops_per_observation() * args.observations
        print(json.dumps({
            "metric": "rollout_observations_per_s", "value": args.observations / best, "unit": "obs/s", "n_gpus": world,
            "observations": args.observations, "seconds": seconds, "quantization": args.quantization,
            "layer_scale": args.layer_scale, "micro_batch": args.micro_batch, "scaling": "strong",
            "fused_mlp": args.fused_mlp, "cuda_graphs": args.graphs,
            "quantised_linear_tflops": flops / best / 1e12, "actions_checksum": float(result.actions.double().sum()),
            "gathered_bytes": result.actions.numel() * 4,
        }))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
