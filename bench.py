"""Benchmark of the quantised-Linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (benchmark configuration 2): the NVFP4 W4A4 linear pair of a Gemma-2B-shaped MLP at M = 560 tokens:
encode x (bf16 -> NVFP4, calibrated scale) -> [gate;up] 2048 -> 2x16384 with the gated GELU-tanh
epilogue that re-encodes the hidden activation to NVFP4 -> down 16384 -> 2048 (bf16 out).
Inputs are seeded synthetic tensors with the config's shapes and distributions (x ~ N(0,1) with 1 %
outliers x20, weights ~ N(0, 0.02)).  One "step" is one pass of that chain over one batch.

Metric: quant GEMM TFLOP/s = 2*M*K*N summed over the two GEMMs / time, whole job over all ranks.
  value  device time only: operands resident in HBM, CUDA events around every step on the launching
         stream, four copies of the weights used in rotation (228 MB > 126 MB L2), max over ranks.
  e2e    the same chain through the public API with host buffers: pinned-host x -> device, the three
         launches, bf16 result -> pinned host, all inside the timed region; four steps are in flight (the
         copies of neighbouring steps overlap the kernels).
With N > 1 every rank runs the same chain on its own batch (weights replicated, no collective on the
data path): weak scaling.

The same line carries the other two parts of the benchmark metric, measured in the same process after the
timed cfg2 region: "rollout" (observations/s of the 256-observation data-parallel rollout, strong scaling over
the N ranks, one NCCL gather per call) and, at N = 1, "denoise_ms" (10-step action-expert denoise at B = 1, 8, 64).

`--impl reference` times the CPU restatement of the reference's route (oracle/, numpy + BLAS on all
host threads) on the same workload and prints the same line with "impl": "reference".
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

TOKENS, HIDDEN, INTER = 560, 2048, 16384
SEED = 1002
SETS = 4            # copies of the quantised weights used in rotation: 4 x 57 MB > 126 MB L2
FLOPS_GATE_UP = 2.0 * TOKENS * HIDDEN * 2 * INTER
FLOPS_DOWN = 2.0 * TOKENS * INTER * HIDDEN
FLOPS_STEP = FLOPS_GATE_UP + FLOPS_DOWN
METRIC = "quant_gemm_tflops"
UNIT = "TFLOP/s"
WORKLOAD = "cfg2: NVFP4 W4A4 MLP pair, M=560, gate_up 2048->2x16384 (+GELU-tanh, NVFP4 re-encode), down 16384->2048"
NOMINAL_NVFP4_TFLOPS = 9000.0


def synthetic_inputs(seed: int):
    """Seeded tensors with the shapes and value distributions of benchmark configuration 2."""
    generator = torch.Generator().manual_seed(seed)
    x = torch.randn((TOKENS, HIDDEN), generator=generator)
    x = torch.where(torch.rand((TOKENS, HIDDEN), generator=generator) < 0.01, x * 20, x).to(torch.bfloat16)
    gate = (0.02 * torch.randn((INTER, HIDDEN), generator=generator)).to(torch.bfloat16)
    up = (0.02 * torch.randn((INTER, HIDDEN), generator=generator)).to(torch.bfloat16)
    down = (0.02 * torch.randn((HIDDEN, INTER), generator=generator)).to(torch.bfloat16)
    return x, gate, up, down


def measured_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text())
    return {}


# ---------------------------------------------------------------------------------------------------
# CPU leg: the oracle port of the reference's route


def bits(tensor: torch.Tensor) -> np.ndarray:
    return tensor.contiguous().view(torch.uint16).numpy()


def cpu_port_step(x, gate, up, down, gate_up_max: float, down_max: float, table: np.ndarray):
    """One pass of the chain with the numpy oracle; returns (bf16 bits of y, seconds)."""
    from oracle import quant_oracle as O

    if not hasattr(cpu_port_step, "weights"):
        cpu_port_step.weights = [O.nvfp4_quantize_C(bits(w)) for w in (gate, up, down)]   # one-time, not timed
    (gp, gsl, _, g_s), (up_, usl, _, u_s), (dp, dsl, _, d_s) = cpu_port_step.weights
    start = time.perf_counter()
    ap, asl, _, a_s = O.nvfp4_quantize_C(bits(x), np.float32(gate_up_max / 2688.0))
    g = O.nvfp4_linear_plan(ap, asl, a_s, gp, gsl, g_s)
    u = O.nvfp4_linear_plan(ap, asl, a_s, up_, usl, u_s)
    hidden = O.gelu_mul(g, u, table)
    hp, hsl, _, h_s = O.nvfp4_quantize_C(hidden, np.float32(down_max / 2688.0))
    y = O.nvfp4_linear_plan(hp, hsl, h_s, dp, dsl, d_s)
    cpu_port_step.hidden_codes = hp
    return y, time.perf_counter() - start


def cpu_table() -> np.ndarray:
    codes = torch.arange(65536, dtype=torch.int32).to(torch.uint16).view(torch.bfloat16)
    return torch.nn.functional.gelu(codes, approximate="tanh").view(torch.uint16).numpy()


def parity_record(got_bits: np.ndarray, want_bits: np.ndarray) -> dict:
    """Whole-output comparison against the CPU oracle under the benchmark's tolerance: relative Frobenius <= 1e-3 and,
    per element, |difference| <= 2e-2 or, where one bf16 unit in the last place of the expected value is already
    larger than 2e-2 (magnitudes from 4 up), one such unit: an fp32 and an fp64 accumulation of the same products
    can land on adjacent bf16 values."""
    from oracle import quant_oracle as O

    got = O.bf16_to_f32(got_bits).astype(np.float64)
    want = O.bf16_to_f32(want_bits).astype(np.float64)
    difference = np.abs(got - want)
    ulp = np.exp2(np.floor(np.log2(np.maximum(np.abs(want), 1e-30))) - 7)
    over = difference > 2e-2
    rel = float(O.rel_frobenius(got_bits, want_bits))
    max_ulp = float((difference[over] / ulp[over]).max()) if over.any() else 0.0
    return {"rel_frobenius": rel, "max_abs": float(difference.max()), "n_over_2e-2": int(over.sum()), "elements": int(over.size),
            "max_ulp_of_those": max_ulp, "within_tolerance": bool(rel <= 1e-3 and max_ulp <= 1.0),
            "rule": "rel-Frobenius <= 1e-3; per element <= max(2e-2, one bf16 ulp of the expected value)",
            "against": "CPU oracle, whole output of this workload"}


def calibrate_on_cpu(x, gate, up):
    """Calibrated maxima the way a calibration pass would record them: amax of the MLP input and of
    the hidden activation (bf16 reference math on a 64-token sample)."""
    gate_up_max = float(x.float().abs().max())
    sample = x[:64].float()
    hidden = torch.nn.functional.gelu(sample @ gate.float().t(), approximate="tanh") * (sample @ up.float().t())
    return gate_up_max, float(hidden.abs().max()) * 2.0


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    x, gate, up, down = synthetic_inputs(SEED)
    gate_up_max, down_max = calibrate_on_cpu(x, gate, up)
    table = cpu_table()
    threads = torch.get_num_threads()
    # A full step is ~10 s of host work: bound the run to a few minutes whatever K says.
    steps = max(1, min(args.steps, 3))
    warmup = max(0, min(args.warmup, 1))
    for _ in range(warmup):
        cpu_port_step(x, gate, up, down, gate_up_max, down_max, table)
    seconds = [cpu_port_step(x, gate, up, down, gate_up_max, down_max, table)[1] for _ in range(steps)]
    mean = float(np.mean(seconds))
    value = FLOPS_STEP / mean / 1e12
    sample = f"{steps} full step(s) of the workload (bounded from --steps {args.steps}); weights quantised once, untimed"
    line = {
        "impl": "reference",
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
        "ms_per_step": mean * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "nvfp4", "data": "synthetic",
        "config": {"workload": WORKLOAD, "host": "numpy/BLAS port of the reference's route (oracle/quant_oracle.py)"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------------
# GPU leg


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    REASONS = {
        0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
        0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown",
        0x100: "display_clock_setting",
    }

    def __init__(self, index: int) -> None:
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._halt = threading.Event()
        self.error = None

    def run(self) -> None:
        try:
            import pynvml

            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            physical = int(visible.split(",")[self.index]) if visible and visible.split(",")[self.index].isdigit() else self.index
            handle = pynvml.nvmlDeviceGetHandleByIndex(physical)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM)
            while not self._halt.is_set():
                self.samples.append(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM))
                mask = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                self.reasons.update(name for bit, name in self.REASONS.items() if mask & bit and bit != 0x1)
                time.sleep(0.002)
        except Exception as error:   # NVML missing: report it instead of failing the benchmark
            self.error = repr(error)

    def stop(self) -> dict:
        self._halt.set()
        self.join(timeout=2.0)
        out = {"sm_mhz": float(np.median(self.samples)) if self.samples else None, "sm_max_mhz": self.max_mhz,
               "reasons": sorted(self.reasons), "samples": len(self.samples)}
        if self.error:
            out["error"] = self.error
        return out


def run_ours(args) -> None:
    import torch.distributed as dist

    from embodiinfer_b200 import _native as N
    from embodiinfer_b200 import kernels as K
    from embodiinfer_b200 import layers as L
    from embodiinfer_b200.backend.mlp import FusedMlpPlan, _ShapeOnly
    from embodiinfer_b200.layers.registry import OperatorRequest

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU fallback (use --impl reference for the CPU leg)")
    if world != args.gpus:
        raise RuntimeError(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    x, gate, up, down = synthetic_inputs(SEED + rank)       # every rank its own batch; same weights' distribution
    gate_up_max, down_max = calibrate_on_cpu(x, gate, up)
    quantizer = L.quantization_backends.get("cuda", OperatorRequest(device, torch.bfloat16, shape=(TOKENS, HIDDEN), bits=4))
    # SETS copies of the quantised weights (57 MB each) are used in rotation, so that every step streams its
    # weights from HBM: 4 x 57 MB exceeds the 126 MB L2.  (Flushing the L2 with a large write instead would also
    # evict the kernels' code, which no real caller does between two layers.)
    gate_d, up_d, down_d = gate.to(device), up.to(device), down.to(device)
    mlps = [FusedMlpPlan(gate_d, up_d, down_d, gate_up_max=gate_up_max, down_max=down_max, gate_up="nvfp4", down="nvfp4",
                         quantizer=quantizer, approximate="tanh") for _ in range(SETS)]
    del gate_d, up_d, down_d
    mlp = mlps[0]
    x_device = x.to(device)
    x_host = x.pin_memory()
    y_host = torch.empty((TOKENS, HIDDEN), dtype=torch.bfloat16).pin_memory()
    stream = torch.cuda.current_stream(device)

    mlp_shape = _ShapeOnly((TOKENS, INTER), x_device)

    def gate_up_launch(plan, source, encoded=None):
        return plan.gate_up.apply_gated(source, plan.encode(source) if encoded is None else encoded, table=plan.table, bits=4,
                                        scale=plan.down.maximum / 2688.0, table_range=plan.table_range)

    def step_device(index=0):
        return mlps[index].down.apply(mlp_shape, gate_up_launch(mlps[index], x_device))

    # End-to-end slots: the copies of step i+1 and i-1 overlap the kernels of step i (three streams, events
    # between them); every step still moves its own input from pinned host memory and its own result back.
    SLOTS = SETS                     # slot k runs on weight set k
    x_hosts = [x_host] + [x.clone().pin_memory() for _ in range(SLOTS - 1)]
    y_hosts = [y_host] + [torch.empty_like(y_host).pin_memory() for _ in range(SLOTS - 1)]
    x_slots = [torch.empty_like(x_device) for _ in range(SLOTS)]
    y_slots = [torch.empty((TOKENS, HIDDEN), device=device, dtype=torch.bfloat16) for _ in range(SLOTS)]

    def step_e2e(slot):
        y_slots[slot].copy_(mlps[slot](x_slots[slot]))

    hidden_first = gate_up_launch(mlps[0], x_device)          # encoded hidden activation of the first step, kept for the parity check
    y_first = mlps[0].down.apply(mlp_shape, hidden_first).clone()
    hidden_codes, hidden_scales = hidden_first.output.clone(), hidden_first.scales.clone()
    torch.cuda.synchronize()

    # The step is replayed from a CUDA graph (three kernel nodes; the e2e graph adds the two copies), as the
    # reference replays its captured request graphs: launch latency of the host is not part of the metric.
    side = torch.cuda.Stream(device)
    side.wait_stream(stream)
    with torch.cuda.stream(side):
        for _ in range(3):                     # warm the side stream's workspaces before capture
            for index in range(SETS):
                step_device(index)
                step_e2e(index)
        side.synchronize()
        graphs_device = [torch.cuda.CUDAGraph() for _ in range(SETS)]
        graphs_e2e = [torch.cuda.CUDAGraph() for _ in range(SLOTS)]
        for index in range(SETS):
            with torch.cuda.graph(graphs_device[index], stream=side):
                step_device(index)
        for slot in range(SLOTS):
            with torch.cuda.graph(graphs_e2e[slot], stream=side):
                step_e2e(slot)
    stream.wait_stream(side)
    torch.cuda.synchronize()

    copy_in, copy_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    landed = [torch.cuda.Event() for _ in range(SLOTS)]       # input of the slot is on the device
    computed = [torch.cuda.Event() for _ in range(SLOTS)]     # result of the slot is in y_slots
    returned = [torch.cuda.Event() for _ in range(SLOTS)]     # result of the slot is back on the host

    def run_e2e(steps, first_event=None, last_event=None):
        for i in range(steps):
            slot = i % SLOTS
            with torch.cuda.stream(copy_in):
                if i == 0 and first_event is not None:
                    first_event.record(copy_in)
                if i >= SLOTS:
                    copy_in.wait_event(computed[slot])          # the kernels of step i - SLOTS have read x_slots[slot]
                x_slots[slot].copy_(x_hosts[slot], non_blocking=True)
                landed[slot].record(copy_in)
            stream.wait_event(landed[slot])
            if i >= SLOTS:
                stream.wait_event(returned[slot])               # y_slots[slot] of step i - SLOTS has left the device
            graphs_e2e[slot].replay()
            computed[slot].record(stream)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(computed[slot])
                y_hosts[slot].copy_(y_slots[slot], non_blocking=True)
                returned[slot].record(copy_out)
                if i == steps - 1 and last_event is not None:
                    last_event.record(copy_out)

    for i in range(max(args.warmup, 3)):
        graphs_device[i % SETS].replay()
    run_e2e(max(args.warmup, 3))
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    new_event = lambda: torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)
    sampler.start()
    # keep the clocks under load for the sampler and out of their idle state before timing
    spin_until = time.time() + 0.5
    while time.time() < spin_until:
        graphs_device[0].replay()
    starts, ends = ([new_event() for _ in range(args.steps)] for _ in range(2))
    barrier()
    for i in range(args.steps):
        starts[i].record(stream)
        graphs_device[i % SETS].replay()
        ends[i].record(stream)
    barrier()
    device_ms = sum(s.elapsed_time(e) for s, e in zip(starts, ends))

    # End to end: K steps in flight over three streams, one start and one end event.
    e2e_start, e2e_end = new_event(), new_event()
    barrier()
    run_e2e(args.steps, e2e_start, e2e_end)
    barrier()
    e2e_ms = e2e_start.elapsed_time(e2e_end)

    # dominant kernel alone (gate_up + GELU + re-encode): one CUDA graph of GATE_UP_BATCH launches over the
    # weight sets in rotation, CUDA events around its replays (eager launches would put the host's launch
    # latency, and single-kernel graphs their launch gaps, between the events)
    GATE_UP_BATCH = 4 * SETS
    encoded_once = [plan.encode(x_device) for plan in mlps]
    graph_gate_up = torch.cuda.CUDAGraph()
    side.wait_stream(stream)
    with torch.cuda.stream(side):
        for index in range(SETS):
            gate_up_launch(mlps[index], x_device, encoded_once[index])
        side.synchronize()
        with torch.cuda.graph(graph_gate_up, stream=side):
            for launch in range(GATE_UP_BATCH):
                gate_up_launch(mlps[launch % SETS], x_device, encoded_once[launch % SETS])
    stream.wait_stream(side)
    torch.cuda.synchronize()
    k_start, k_end = new_event(), new_event()
    barrier()
    gate_up_replays = max(1, -(-args.steps // GATE_UP_BATCH))
    k_start.record(stream)
    for _ in range(gate_up_replays):
        graph_gate_up.replay()
    k_end.record(stream)
    barrier()
    gate_up_ms = k_start.elapsed_time(k_end) / (gate_up_replays * GATE_UP_BATCH)
    clocks = sampler.stop()

    # One step alone, end to end, nothing in flight beside it: what a control loop that waits for each result sees.
    torch.cuda.synchronize()
    lat_start, lat_end = new_event(), new_event()
    LATENCY_STEPS = 10
    lat_start.record(stream)
    for i in range(LATENCY_STEPS):
        slot = i % SLOTS
        x_slots[slot].copy_(x_hosts[slot], non_blocking=True)
        graphs_e2e[slot].replay()
        y_hosts[slot].copy_(y_slots[slot], non_blocking=True)
        stream.synchronize()
    lat_end.record(stream)
    torch.cuda.synchronize()
    latency_ms = lat_start.elapsed_time(lat_end) / LATENCY_STEPS

    if world > 1:
        times = torch.tensor([device_ms, e2e_ms, gate_up_ms, latency_ms], device=device, dtype=torch.float64)
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        device_ms, e2e_ms, gate_up_ms, latency_ms = times.tolist()

    # The other parts of the metric.  Every rank takes part (the rollout gathers across ranks); the cfg2 objects are
    # released first.  A failure here is reported inside the block and never costs the cfg2 line.
    library_us = library_gemm_microseconds(device) if world == 1 and not args.skip_library else None
    del mlps, graphs_device, graphs_e2e, graph_gate_up, encoded_once
    torch.cuda.empty_cache()
    rollout_block, denoise_block = None, None
    if not args.skip_rollout:
        try:
            from embodiinfer_b200.rollout_bench import measure_rollout
            from embodiinfer_b200.stack_bench import measure_denoise

            record, policy = measure_rollout(device, observations=256, micro_batch=32, quantization="fp8", repeats=2)
            rollout_block = {"obs_per_s": record["value"], "observations": 256, "scaling": "strong", "n_gpus": world,
                             "gathered_bytes": record["gathered_bytes"], "checksum": record["actions_checksum"],
                             "collectives_per_call": record["collectives_per_call"], "micro_batch": record["micro_batch"],
                             "ms": record["ms"], "quantised_linear_tflops": record["quantised_linear_tflops"],
                             "h2d_bytes_per_observation": record["h2d_bytes_per_observation"],
                             "workload": "cfg5: SigLIP-So400m-shaped tower + Gemma-2B-shaped prefix + 10-step expert denoise, FP8 linears, "
                                         "uint8 frames from pinned host memory inside the timed region"}
            if world == 1:
                denoise_block = {key: round(value, 4) for key, value in measure_denoise(policy).items()}
                denoise_block["workload"] = "cfg4: 18 Gemma-300M-shaped layers, 10-token chunk, 10 Euler steps, FP8 linears, one CUDA graph"
        except Exception as error:          # noqa: BLE001 - reported, the main metric stands
            rollout_block = {"error": f"{type(error).__name__}: {str(error)[:300]}"}
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    value = world * args.steps * FLOPS_STEP / (device_ms * 1e-3) / 1e12
    e2e_value = world * args.steps * FLOPS_STEP / (e2e_ms * 1e-3) / 1e12
    peaks = measured_peaks()
    achieved = FLOPS_GATE_UP / (gate_up_ms * 1e-3) / 1e12
    if "bf16_tflops" in peaks:
        peak = 4.0 * float(peaks["bf16_tflops"])
        peak_source = "4 x measured cuBLAS bf16 burst (MEASURED_PEAKS.json has no NVFP4 figure; 4x is the nominal NVFP4:bf16 ratio)"
    else:
        peak = 4.0 * 1590.0
        peak_source = "4 x fallback bf16 burst 1590 TFLOP/s (MEASURED_PEAKS.json absent)"
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": device_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "nvfp4", "data": "synthetic",
        "config": {"workload": WORKLOAD, "l2": f"{SETS} weight sets of 57 MB in rotation (working set {SETS * 57} MB > 126 MB L2), no flush", "launches_per_step": 3,
                   "replay": "each step is one CUDA-graph replay",
                   "calibrated_max": {"gate_up": gate_up_max, "down": down_max}},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2,
                "ms_per_step": e2e_ms / args.steps, "in_flight": SLOTS,
                "single_step_latency_ms": latency_ms,
                "note": "throughput with 4 steps in flight on three streams; single_step_latency_ms is one step alone (copy in, three launches, copy out, host wait)"},
        "gpu_launches": 3 * args.steps + 3 * args.steps + gate_up_replays * GATE_UP_BATCH,   # device steps + e2e steps + gate_up-only launches
        "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "linear_kernel<NVFP4, GEGLU->NVFP4> (gate_up)", "achieved": achieved, "peak": peak,
                     "unit": "TFLOP/s", "frac": achieved / peak, "frac_of_nominal_9000": achieved / NOMINAL_NVFP4_TFLOPS,
                     "peak_source": peak_source, "us_per_launch": gate_up_ms * 1e3, "traffic": gate_up_traffic_bytes()},
    }
    if rollout_block is not None:
        line["rollout"] = rollout_block
    if denoise_block is not None:
        line["denoise_ms"] = denoise_block
    if library_us is not None:
        line["library_gemm_us"] = library_us
    if world == 1:
        table = cpu_table()
        x0, gate0, up0, down0 = synthetic_inputs(SEED)
        y_cpu, seconds = cpu_port_step(x0, gate0, up0, down0, gate_up_max, down_max, table)
        y_gpu = y_first.cpu().view(torch.uint16).numpy()
        # (1) the whole chain against the oracle's chain; (2) the down GEMM on IDENTICAL quantised operands (the GPU's own
        # encoded hidden activation fed to the oracle), judged element by element; (3) how many of the hidden NVFP4 codes
        # equal the oracle's (a one-ulp difference of gate or up can move a code, which (1) then carries into y)
        from oracle import quant_oracle as O

        codes_gpu = hidden_codes.cpu().view(torch.uint8).numpy()
        scales_gpu = hidden_scales.cpu().view(torch.uint8).numpy()
        weights = cpu_port_step.weights[2]
        y_same_operands = O.nvfp4_linear_plan(codes_gpu, scales_gpu, np.float32(down_max / 2688.0), weights[0], weights[1], weights[3])
        line["parity"] = parity_record(y_gpu, y_same_operands)
        line["parity"]["against"] = "CPU oracle of the down GEMM on the GPU's own encoded hidden activation (identical quantised operands), whole output"
        line["parity"]["chain"] = {"rel_frobenius": float(O.rel_frobenius(y_gpu, y_cpu)), "max_abs": float(O.max_abs(y_gpu, y_cpu)),
                                   "hidden_codes_equal_to_oracle": float((codes_gpu == cpu_port_step.hidden_codes).mean()),
                                   "against": "CPU oracle of the whole chain (its own hidden activation): differences include re-encoded hidden codes that moved"}
        line["cpu_baseline"] = {"value": FLOPS_STEP / seconds / 1e12, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                                "sample": "one full step of the same workload with the numpy/BLAS oracle (weights quantised once, untimed)"}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def library_gemm_microseconds(device) -> dict:
    """torch's scaled_mm (cuBLASLt; the GEMM the reference calls on this GPU, backend/torch/nvfp4.py:109-119) on the two
    GEMM shapes of the workload, operands rotated like the benchmark's weight sets.  GEMMs only: the reference adds an
    activation encoder, the GELU*up + re-encode pass (41.9 MB of traffic) and the global-scale multiply around them."""
    def codes(shape):
        return (torch.randint(0, 255, shape, device=device, dtype=torch.uint8) & 0x77)

    def blocked(rows, blocks):
        return -(-rows // 128) * 128 * (-(-blocks // 4) * 4)

    found = {}
    try:
        for name, rows, width in (("gate_up", 2 * INTER, HIDDEN), ("down", HIDDEN, INTER)):
            sets = []
            for _ in range(SETS):
                a = codes((TOKENS, width // 2)).view(torch.float4_e2m1fn_x2)
                w = codes((rows, width // 2)).view(torch.float4_e2m1fn_x2)
                sa = torch.randint(40, 72, (blocked(TOKENS, width // 16),), device=device, dtype=torch.uint8).view(torch.float8_e4m3fn)
                sw = torch.randint(40, 72, (blocked(rows, width // 16),), device=device, dtype=torch.uint8).view(torch.float8_e4m3fn)
                sets.append((a, w, sa, sw))
            for a, w, sa, sw in sets:
                torch._scaled_mm(a, w.t(), sa, sw, out_dtype=torch.bfloat16)
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            launches = 10 * SETS
            start.record()
            for index in range(launches):
                a, w, sa, sw = sets[index % SETS]
                torch._scaled_mm(a, w.t(), sa, sw, out_dtype=torch.bfloat16)
            stop.record()
            torch.cuda.synchronize()
            found[name] = round(start.elapsed_time(stop) * 1e3 / launches, 2)
        found["what"] = "torch._scaled_mm NVFP4 GEMM only (bf16 out), eager launches, CUDA events"
    except Exception as error:          # noqa: BLE001 - this torch build may lack the kernel
        found = {"unavailable": f"{type(error).__name__}: {str(error)[:160]}"}
    return found


def gate_up_traffic_bytes():
    """dram__bytes_read.sum + dram__bytes_write.sum of one gate_up launch as the last ncu capture recorded it
    (profiles/roofline_traffic.json, rewritten whenever that capture is refreshed); None without the file."""
    path = ROOT / "profiles" / "roofline_traffic.json"
    if not path.exists():
        return None
    return json.loads(path.read_text()).get("gate_up_cfg2", {}).get("dram_bytes_per_launch")


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=20)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--skip-rollout", action="store_true", help="only the cfg2 metric (no rollout / denoise blocks)")
    parser.add_argument("--skip-library", action="store_true", help="do not time torch's scaled_mm beside the kernels")
    args = parser.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
