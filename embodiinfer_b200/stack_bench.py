"""Milliseconds of the pi0.5-shaped stacks on one B200 (the prefix-stack and action-expert benchmark configurations, synthetic inputs).

    python -m embodiinfer_b200.stack_bench [--quantization fp8|nvfp4] [--batches 1 8 64] [--registry-route]

* prefix stack: 18 Gemma-2B-shaped layers over 560 prefix tokens (one observation), random-init weights,
  input ~N(0, 1) bf16;
* action-expert denoise: 18 Gemma-300M-shaped layers over a 10-token action chunk, 10 Euler steps,
  batch B, attending to random prefix keys/values [B, 1, 560, 256] per layer.

Each measurement is one CUDA graph replayed 20 times between CUDA events (after 3 warm-up replays); the
MLPs run as the calibrated fused plan unless ``--registry-route`` is given.  One JSON line per case.
Attention, norms and RoPE are torch operations and are inside the timed region: the numbers are stack
latencies, not GEMM times (``kernel_bench`` has those).
"""

from __future__ import annotations

import argparse
import json

import torch

from .pi05_shaped import (ACTION_DIM, ACTION_HORIZON, GEMMA_2B, GEMMA_300M, Pi05ShapedPolicy, rope_tables,
                          synthetic_observations)

PREFIX_TOKENS = 560


def graph_milliseconds(function, replays: int = 20) -> float:
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(2):
            function()
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        function()
    torch.cuda.synchronize()
    for _ in range(3):
        graph.replay()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(replays):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / replays


def linear_flops(shape, tokens: int, layers: int) -> float:
    q_dim, kv_dim = shape.heads * shape.head_dim, shape.kv_heads * shape.head_dim
    per_token = shape.width * (q_dim + 2 * kv_dim) + q_dim * shape.width + 3 * shape.width * shape.mlp
    return 2.0 * tokens * per_token * layers


@torch.no_grad()
def measure_denoise(policy: Pi05ShapedPolicy, batches=(1, 8, 64), seed: int = 1004) -> dict[str, float]:
    """Milliseconds of the 10-step action-expert denoise (18 layers, 10-token chunk) per batch size, on ``policy``'s
    expert tower with random prefix keys/values: one CUDA graph per batch size, 20 replays between CUDA events."""
    device = policy.device_
    generator = torch.Generator(device=device).manual_seed(seed)
    found = {}
    for batch in batches:
        cache = [tuple(torch.randn((batch, 1, PREFIX_TOKENS, GEMMA_300M.head_dim), device=device, generator=generator).to(torch.bfloat16)
                       for _ in range(2)) for _ in policy.expert]
        noise = torch.randn((batch, ACTION_HORIZON, ACTION_DIM), device=device, generator=generator)
        found[f"B{batch}"] = graph_milliseconds(lambda: policy.denoise(cache, PREFIX_TOKENS, noise))
    return found


@torch.no_grad()
def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--quantization", default="fp8")
    parser.add_argument("--batches", type=int, nargs="*", default=[1, 8, 64])
    parser.add_argument("--registry-route", action="store_true", help="dynamic scales, unfused MLP (QuantizedLinear.forward)")
    parser.add_argument("--layer-scale", type=float, default=1.0)
    args = parser.parse_args()
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    policy = Pi05ShapedPolicy(args.quantization, device=device, layer_scale=args.layer_scale, vocabulary=4096)
    if not args.registry_route:
        policy.calibrate_fused_mlp(synthetic_observations(2, vocabulary=4096), margin=1.5)
    generator = torch.Generator(device=device).manual_seed(1003)
    common = {"quantization": args.quantization, "route": "registry" if args.registry_route else "calibrated fused MLP",
              "layers": len(policy.prefix), "data": "synthetic", "timing": "CUDA-graph replay, CUDA events, 20 replays"}

    hidden = torch.randn((1, PREFIX_TOKENS, GEMMA_2B.width), device=device, generator=generator).to(torch.bfloat16)
    rope = rope_tables(torch.arange(PREFIX_TOKENS, device=device), GEMMA_2B.head_dim)

    def prefix_stack():
        x = hidden
        for block in policy.prefix:
            x, _ = block(x, rope)
        return x

    milliseconds = graph_milliseconds(prefix_stack)
    flops = linear_flops(GEMMA_2B, PREFIX_TOKENS, len(policy.prefix))
    print(json.dumps({"case": "prefix_stack_560_tokens", "ms": round(milliseconds, 4),
                      "quantised_linear_tflops": round(flops / milliseconds / 1e9, 1), **common}), flush=True)

    for batch in args.batches:
        cache = [tuple(torch.randn((batch, 1, PREFIX_TOKENS, GEMMA_300M.head_dim), device=device, generator=generator).to(torch.bfloat16)
                       for _ in range(2)) for _ in policy.expert]
        noise = torch.randn((batch, ACTION_HORIZON, ACTION_DIM), device=device, generator=generator)
        milliseconds = graph_milliseconds(lambda: policy.denoise(cache, PREFIX_TOKENS, noise))
        flops = 10 * linear_flops(GEMMA_300M, ACTION_HORIZON * batch, len(policy.expert))
        print(json.dumps({"case": f"expert_denoise_10_steps_B{batch}", "ms": round(milliseconds, 4),
                          "ms_per_step": round(milliseconds / 10, 4),
                          "quantised_linear_tflops": round(flops / milliseconds / 1e9, 2), **common}), flush=True)


if __name__ == "__main__":
    main()
