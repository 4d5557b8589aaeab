"""Per-kernel timings on one B200: the quantisers, the stand-alone gated epilogue, the norm producer and the tensor-core
Linear at the shapes of the pi0.5-style towers.  One JSON line per case.

    python -m embodiinfer_b200.kernel_bench                       # every case
    python -m embodiinfer_b200.kernel_bench --case 'linear/fp8'   # cases whose name matches the regex
    python -m embodiinfer_b200.kernel_bench --case cfg1 --library # also time torch's scaled_mm on the same shape
    python -m embodiinfer_b200.kernel_bench --case cfg1 --eager 3 # three plain launches and no timing: the form to run under a profiler
    python -m embodiinfer_b200.kernel_bench --case 'quant|geglu|norm' --reference   # the reference's own kernels beside each case

Method: each case is launched ``--launches`` times inside one CUDA graph, rotating over as many
operand sets as it takes to exceed the L2 capacity (capped at 16 sets; ``"l2": "warm"`` marks the
cases whose rotation stays below it), the graph is replayed for 0.5 s to settle the clocks and then
timed with CUDA events.  ``gbs`` counts each operand and result once (algorithmic bytes), ``tflops``
is 2*M*N*K.  Operands are Gaussian matrices (activations ~N(0,1), weights ~N(0,0.02)) quantised by the
package's own kernels, so the gated epilogue sees realistic gate values.
"""

from __future__ import annotations

import argparse
import json
import re
import time

import torch

from . import _native as N
from . import kernels as K
from .backend.activation import gelu_table

L2_BYTES = 126 * 2**20
MAX_SETS = 16


def _codes(shape, device):
    return torch.randint(0, 255, shape, device=device, dtype=torch.uint8) & 0x77      # no NaN codes


def _scale_codes(shape, device):
    return torch.randint(40, 72, shape, device=device, dtype=torch.uint8)              # e4m3 around 1


def _blocked_bytes(rows: int, blocks: int) -> int:
    return -(-rows // 128) * 128 * (-(-blocks // 4) * 4)


def run_eager(make, set_bytes: int, launches: int) -> int:
    """``launches`` plain launches over rotating operand sets (no graph, no timing): what a profiler should see."""
    sets = max(1, min(MAX_SETS, launches, -(-2 * L2_BYTES // max(set_bytes, 1))))
    closures = [make(index) for index in range(sets)]
    torch.cuda.synchronize()
    for index in range(launches):
        closures[index % sets]()
    torch.cuda.synchronize()
    return sets


FORCED_SETS = 0       # --sets: 1 keeps every operand in the L2 between launches (warm), 0 = enough sets to exceed it


def time_graph(make, set_bytes: int, launches: int, settle: float = 0.5) -> tuple[float, int]:
    """Average microseconds per launch; ``make(i)`` returns the launch closure of operand set ``i``."""
    sets = FORCED_SETS or max(1, min(MAX_SETS, -(-2 * L2_BYTES // max(set_bytes, 1))))
    closures = [make(index) for index in range(sets)]
    for closure in closures[:2]:
        closure()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side), torch.cuda.graph(graph, stream=side):
        for index in range(launches):
            closures[index % sets]()
    torch.cuda.synchronize()
    begin = time.time()
    while time.time() - begin < settle:
        graph.replay()
        torch.cuda.synchronize()
    replays = 20
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(replays):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) * 1e3 / (replays * launches), sets


# ---- cases -----------------------------------------------------------------------------------

def quantiser_cases(device):
    for rows in (560, 17920):
        columns = 2048
        count = rows * columns

        def amax(_i, rows=rows):
            x = torch.randn((rows, columns), device=device).to(torch.bfloat16)
            scratch, scale = K.new_scale_scratch(device), torch.ones((), device=device)
            return lambda: K.tensor_scale(x, 448.0, N.SCALAR_RCP, scratch, scale)

        def fp8(flags):
            def make(_i, rows=rows):
                x = torch.randn((rows, columns), device=device).to(torch.bfloat16)
                out, scale = torch.empty((rows, columns), device=device, dtype=torch.uint8), torch.full((), 0.01, device=device)
                return lambda: K.fp8_quantize(x, out, scale, flags)
            return make

        def nvfp4(flags):
            def make(_i, rows=rows):
                x = torch.randn((rows, columns), device=device).to(torch.bfloat16)
                out = torch.empty((rows, columns // 2), device=device, dtype=torch.uint8)
                blocked = torch.zeros(_blocked_bytes(rows, columns // 16), device=device, dtype=torch.uint8)
                scale = torch.full((), 0.002, device=device)
                return lambda: K.nvfp4_quantize(x, out, None, blocked, scale, flags)
            return make

        yield f"quant/tensor_scale/{rows}x{columns}", amax, 2 * count, 2 * count, 0
        yield f"quant/fp8_C/{rows}x{columns}", fp8(N.SPEC_C), 3 * count, 3 * count, 0
        yield f"quant/fp8_T/{rows}x{columns}", fp8(N.SPEC_T | N.DIVISOR_BF16), 3 * count, 3 * count, 0
        nv = 2 * count + count // 2 + count // 16
        yield f"quant/nvfp4_C/{rows}x{columns}", nvfp4(N.SPEC_C), nv, nv, 0
        yield f"quant/nvfp4_T/{rows}x{columns}", nvfp4(N.SPEC_T | N.SCALAR_RCP), nv, nv, 0


def geglu_cases(device):
    rows, features = 560, 16384
    table = gelu_table(device, "tanh")
    for bits, out_bytes in ((16, 2.0), (8, 1.0), (4, 0.5 + 1 / 16)):
        def make(_i, bits=bits):
            packed = torch.randn((rows, 2 * features), device=device).to(torch.bfloat16)
            gate, up = packed[:, :features], packed[:, features:]
            out = torch.empty((rows, features * (2 if bits == 16 else 1) // (2 if bits == 4 else 1)), device=device, dtype=torch.uint8)
            scale = torch.full((), 0.01, device=device)
            blocked = torch.zeros(_blocked_bytes(rows, features // 16), device=device, dtype=torch.uint8) if bits == 4 else None
            return lambda: K.geglu(gate, up, out, bits=bits, table=table, rows=rows, columns=features, row_stride=2 * features,
                                   scale=scale, blocked=blocked)
        total = int(rows * features * (4 + out_bytes))
        yield f"geglu/standalone_bits{bits}/{rows}x{features}", make, total, total, 0


def norm_cases(device):
    """Residual update + RMSNorm + encoder in one launch (bytes: input, update, residual out, codes out)."""
    columns = 2048
    for rows in (560, 17920):
        for bits, out_bytes in ((8, 1.0), (4, 0.5 + 1 / 16), (16, 2.0)):
            def make(_i, rows=rows, bits=bits):
                x = torch.randn((rows, columns), device=device).to(torch.bfloat16)
                update = torch.randn((rows, columns), device=device).to(torch.bfloat16)
                residual = torch.empty_like(x)
                weight = torch.randn(columns, device=device) * 0.1
                width = {16: 2 * columns, 8: columns, 4: columns // 2}[bits]
                out = torch.empty((rows, width), device=device, dtype=torch.uint8)
                blocked = torch.zeros(_blocked_bytes(rows, columns // 16), device=device, dtype=torch.uint8) if bits == 4 else None
                scale = torch.full((), 0.01, device=device)
                return lambda: K.norm_quant(x, out, bits=bits, tokens=560, scale=weight, update=update, residual=residual,
                                            global_scale=None if bits == 16 else scale, blocked=blocked)
            total = int(rows * columns * (6 + out_bytes))
            yield f"norm/residual_rms_bits{bits}/{rows}x{columns}", make, total, total, 0
    columns = 1152
    for rows in (768, 24576):
        for bits, out_bytes in ((8, 1.0), (4, 0.5 + 1 / 16)):
            def make(_i, rows=rows, bits=bits):
                x = torch.randn((rows, columns), device=device).to(torch.bfloat16)
                update = torch.randn((rows, columns), device=device).to(torch.bfloat16)
                residual = torch.empty_like(x)
                weight = torch.randn(columns, device=device).to(torch.bfloat16)
                bias = torch.randn(columns, device=device).to(torch.bfloat16)
                out = torch.empty((rows, columns if bits == 8 else columns // 2), device=device, dtype=torch.uint8)
                blocked = torch.zeros(_blocked_bytes(rows, columns // 16), device=device, dtype=torch.uint8) if bits == 4 else None
                return lambda: K.layer_norm_quant(x, weight, bias, out, bits=bits, scale_value=40.0 if bits == 8 else 0.004,
                                                  update=update, residual=residual, blocked=blocked)
            total = int(rows * columns * (6 + out_bytes))
            yield f"norm/residual_layer_norm_bits{bits}/{rows}x{columns}", make, total, total, 0


def layout_cases(device):
    """The transposing encoder behind the attention and the frame-to-patch producer."""
    heads, head_dim = 8, 256
    for batch, tokens in ((1, 560), (32, 560)):
        for bits, out_bytes in ((8, 1.0), (4, 0.5 + 1 / 16)):
            def make(_i, batch=batch, tokens=tokens, bits=bits):
                attended = torch.randn((batch, heads, tokens, head_dim), device=device).to(torch.bfloat16)
                rows, columns = batch * tokens, heads * head_dim
                out = torch.empty((rows, columns if bits == 8 else columns // 2), device=device, dtype=torch.uint8)
                blocked = torch.zeros(_blocked_bytes(rows, columns // 16), device=device, dtype=torch.uint8) if bits == 4 else None
                return lambda: K.bhsd_quant(attended, out, bits=bits, scale_value=40.0 if bits == 8 else 0.004, blocked=blocked)
            total = int(batch * tokens * heads * head_dim * (2 + out_bytes))
            yield f"layout/bhsd_bits{bits}/{batch}x{heads}x{tokens}x{head_dim}", make, total, total, 0
    for cameras in (3, 96):
        def make(_i, cameras=cameras):
            frames = torch.randint(0, 256, (cameras, 224, 224, 3), device=device, dtype=torch.uint8)
            patches = torch.empty((cameras * 256, 588), device=device, dtype=torch.bfloat16)
            return lambda: K.frames_to_patches(frames, patches, 14)
        total = cameras * 224 * 224 * 3 * 3
        yield f"layout/frames_to_patches/{cameras}x224x224", make, total, total, 0


LINEAR_SHAPES = [
    # name, kind, M, N (features; GEGLU: gate features), K, epilogue
    ("cfg1_fp8_560x16384x2048", "fp8", 560, 16384, 2048, "linear"),
    ("cfg2_nvfp4_gate_up_geglu_560x2x16384x2048", "nvfp4", 560, 16384, 2048, "geglu"),
    ("cfg2_nvfp4_down_560x2048x16384", "nvfp4", 560, 2048, 16384, "linear"),
    ("nvfp4_gate_up_plain_560x32768x2048", "nvfp4", 560, 32768, 2048, "linear"),
    ("fp8_gate_up_geglu_560x2x16384x2048", "fp8", 560, 16384, 2048, "geglu"),
    ("fp8_down_560x2048x16384", "fp8", 560, 2048, 16384, "linear"),
    ("prefix_qkv_fp8_560x2560x2048", "fp8", 560, 2560, 2048, "linear"),
    ("prefix_o_fp8_560x2048x2048", "fp8", 560, 2048, 2048, "linear"),
    ("prefix_qkv_nvfp4_560x2560x2048", "nvfp4", 560, 2560, 2048, "linear"),
    ("siglip_qkv_fp8_8192x3456x1152", "fp8", 8192, 3456, 1152, "linear"),
    ("siglip_fc1_fp8_8192x4304x1152", "fp8", 8192, 4304, 1152, "linear"),
    ("siglip_fc2_fp8_8192x1152x4304", "fp8", 8192, 1152, 4304, "linear"),
    ("prefix_mb16_gate_up_fp8_geglu_8960x2x16384x2048", "fp8", 8960, 16384, 2048, "geglu"),
    ("prefix_mb16_down_fp8_8960x2048x16384", "fp8", 8960, 2048, 16384, "linear"),
    ("prefix_mb16_gate_up_nvfp4_geglu_8960x2x16384x2048", "nvfp4", 8960, 16384, 2048, "geglu"),
    ("prefix_mb16_down_nvfp4_8960x2048x16384", "nvfp4", 8960, 2048, 16384, "linear"),
] + [
    (f"expert_B{batch}_{name}_{kind}_{10 * batch}x{n}x{k}", kind, 10 * batch, n, k, epilogue)
    for batch in (1, 2, 4, 8, 12, 64) for kind in ("fp8", "nvfp4")
    for name, n, k, epilogue in (("qkv", 2560, 1024, "linear"), ("o", 1024, 2048, "linear"),
                                 ("gate_up_geglu", 4096, 1024, "geglu"), ("down", 1024, 4096, "linear"))
]


def quantised_operand(kind: str, rows: int, width: int, std: float, device):
    """Codes, tiled block scales and the global scale of a Gaussian matrix, through the package's own
    quantiser (random codes where the width is not a multiple of 64, which the quantiser plans require)."""
    if width % 64 != 0:
        codes = _codes((rows, width if kind == "fp8" else width // 2), device)
        scales = _scale_codes((_blocked_bytes(rows, width // 16),), device) if kind == "nvfp4" else None
        return codes, scales, torch.full((), 1e-3 if kind == "fp8" else 3e-2, device=device)
    from .backend.quantization import B200Quantizer
    matrix = (std * torch.randn((rows, width), device=device)).to(torch.bfloat16)
    plan = B200Quantizer().plan(matrix, 8 if kind == "fp8" else 4)
    plan.quantize(matrix)
    torch.cuda.synchronize()
    scales = plan.blocked.view(torch.uint8).clone() if kind == "nvfp4" else None
    return plan.output.view(torch.uint8).clone(), scales, plan.scale.reshape(()).clone()


def linear_cases(device, options=None):
    options = options or {}
    table = gelu_table(device, "tanh")
    table_range = K.gelu_table_range(table)
    for name, kind, tokens, features, width, epilogue in LINEAR_SHAPES:
        gated = epilogue == "geglu"
        rows = 2 * features if gated else features
        operand = 1.0 if kind == "fp8" else 0.5 + 1 / 16
        out_bytes = (1.0 if kind == "fp8" else 0.5 + 1 / 16) if gated else 2.0
        total = int(tokens * width * operand + rows * width * operand + tokens * features * out_bytes)

        def make(_i, kind=kind, tokens=tokens, features=features, width=width, gated=gated, rows=rows):
            status = torch.zeros(4, device=device, dtype=torch.int32)
            act, act_scales, act_scale = quantised_operand(kind, tokens, width, 1.0, device)
            weight, weight_scales, weight_scale = quantised_operand(kind, rows, width, 0.02, device)
            arguments = dict(tokens=tokens, features=features, width=width, act=act, weight=weight, act_scale=act_scale,
                             weight_scale=weight_scale, status=status, kind=N.KIND_FP8 if kind == "fp8" else N.KIND_NVFP4)
            if kind == "nvfp4":
                arguments.update(act_scales=act_scales, weight_scales=weight_scales)
            if gated:
                out_format = N.OUT_FP8 if kind == "fp8" else N.OUT_NVFP4
                out = torch.empty((tokens, features if kind == "fp8" else features // 2), device=device, dtype=torch.uint8)
                arguments.update(epilogue=N.EPI_GEGLU, out_format=out_format, out=out, gelu_table=table, gelu_range=table_range,
                                 out_scale=torch.full((), 0.02 if kind == "fp8" else 0.003, device=device))
                if kind == "nvfp4":
                    if not options.get("unpaired"):
                        arguments.update(flags=N.LINEAR_PAIRED_GATE_UP_SCALES)
                    arguments.update(out_blocked=torch.zeros(_blocked_bytes(tokens, features // 16), device=device, dtype=torch.uint8),
                                     out_scales=torch.empty((tokens, features // 16), device=device, dtype=torch.uint8))
            else:
                arguments.update(epilogue=N.EPI_LINEAR, out_format=N.OUT_BF16,
                                 out=torch.empty((tokens, features), device=device, dtype=torch.bfloat16))
            if options.get("workspace") and not gated:
                arguments["workspace"] = K.linear_workspace(device)
            arguments["flags"] = arguments.get("flags", 0) | options.get("flags", 0)
            arguments["feature_tile"] = options.get("feature_tile", 0)
            return lambda: K.linear(**arguments)

        yield f"linear/{name}", make, total, total, 2.0 * tokens * rows * width


ATTENTION_SHAPES = [
    # name, batch, query heads, queries, keys (head dimension 256, one key/value head)
    ("prefix_B1_8x560x560", 1, 8, 560, 560),
    ("prefix_B32_8x560x560", 32, 8, 560, 560),
    ("expert_B1_8x10x570", 1, 8, 10, 570),
    ("expert_B2_8x10x570", 2, 8, 10, 570),
    ("expert_B4_8x10x570", 4, 8, 10, 570),
    ("expert_B8_8x10x570", 8, 8, 10, 570),
    ("expert_B16_8x10x570", 16, 8, 10, 570),
    ("expert_B32_8x10x570", 32, 8, 10, 570),
    ("expert_B64_8x10x570", 64, 8, 10, 570),
]


def attention_cases(device, library: bool):
    """b2_attention; with ``library`` torch's scaled_dot_product_attention on the same tensors instead (name suffix)."""
    import torch.nn.functional as F
    for name, batch, heads, queries, keys in ATTENTION_SHAPES:
        total = 2 * (2 * batch * heads * queries * 256 + 2 * batch * keys * 256)
        flops = 4.0 * batch * heads * queries * keys * 256

        def make(_i, batch=batch, heads=heads, queries=queries, keys=keys, library=library):
            q = torch.randn((batch, heads, queries, 256), device=device).to(torch.bfloat16)
            k = torch.randn((batch, 1, keys, 256), device=device).to(torch.bfloat16)
            v = torch.randn((batch, 1, keys, 256), device=device).to(torch.bfloat16)
            out = torch.empty_like(q)
            if library:
                return lambda: F.scaled_dot_product_attention(q, k, v, enable_gqa=True)
            return lambda: K.attention(q, k, v, out)

        yield f"attention/{name}" + ("/torch_sdpa" if library else ""), make, total, total, flops


def library_time(kind: str, tokens: int, rows: int, width: int, device, launches: int) -> float | None:
    """torch's scaled_mm (the GEMM the reference calls on this GPU) at the same shape; None when this
    torch build has no such kernel for the operand type."""
    try:
        if kind == "fp8":
            def make(_i):
                a = _codes((tokens, width), device).view(torch.float8_e4m3fn)
                w = _codes((rows, width), device).view(torch.float8_e4m3fn)
                one = torch.ones((), device=device)
                return lambda: torch._scaled_mm(a, w.t(), one, one, out_dtype=torch.bfloat16)
            set_bytes = tokens * width + rows * width + 2 * tokens * rows
        else:
            def make(_i):
                a = _codes((tokens, width // 2), device).view(torch.float4_e2m1fn_x2)
                w = _codes((rows, width // 2), device).view(torch.float4_e2m1fn_x2)
                sa = _scale_codes((_blocked_bytes(tokens, width // 16),), device).view(torch.float8_e4m3fn)
                sw = _scale_codes((_blocked_bytes(rows, width // 16),), device).view(torch.float8_e4m3fn)
                return lambda: torch._scaled_mm(a, w.t(), sa, sw, out_dtype=torch.bfloat16)
            set_bytes = (tokens + rows) * width // 2 + 2 * tokens * rows
        return time_graph(make, set_bytes, launches)[0]
    except Exception as error:                      # no kernel for this type/shape in this torch build
        print(json.dumps({"library_unavailable": f"{kind}: {type(error).__name__}: {str(error)[:120]}"}))
        return None


# ---- the reference's own CUDA kernels, timed by the same harness ---------------------------------------

def reference_cases(device):
    """The reference's SIMT kernels for this path (its quantiser, GELU*up epilogue, norm + encoder, LayerNorm + encoder and
    transposing encoder), imported unmodified from ``baseline/_ref`` and compiled by the reference's own loader, at the
    shapes of the cases above.  Yields (name of the matching case here, make, set_bytes)."""
    import ctypes
    import os
    import sys
    import tempfile
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent / "baseline" / "_ref"
    if not (root / "embodiinfer").exists():
        raise SystemExit("--reference needs the reference under baseline/_ref (python baseline/install_reference.py <checkout>)")
    os.environ.setdefault("EMBODIINFER_CUDA_CACHE_DIR", tempfile.mkdtemp(prefix="embodiinfer_ref_cache_"))
    sys.path.insert(0, str(root))
    from embodiinfer.backend.cuda.activation import GeluMulFusion
    from embodiinfer.backend.cuda.norm_quant import NormQuantReduceFusion
    from embodiinfer.backend.cuda.normalization import NormFusion
    from embodiinfer.backend.cuda.quantization import CudaQuantizer

    quantizer = CudaQuantizer()
    fusion = GeluMulFusion(quantizer, approximate="tanh")
    norm_quant = NormQuantReduceFusion(quantizer, NormFusion())
    library = norm_quant.library
    pointer = ctypes.c_void_p
    library.cc_layer_norm_fp8.argtypes = [pointer] * 6 + [ctypes.c_float, ctypes.c_int, ctypes.c_int, pointer]
    library.cc_layer_norm_fp4.argtypes = [pointer] * 7 + [ctypes.c_float, ctypes.c_int, ctypes.c_int, pointer]
    stream = lambda: torch.cuda.current_stream(device).cuda_stream

    for rows in (560, 17920):
        columns = 2048
        for bits, name, out_bytes in ((8, "fp8_C", 1.0), (4, "nvfp4_C", 0.5 + 1 / 16)):
            def make(_i, rows=rows, bits=bits):
                x = torch.randn((rows, columns), device=device).to(torch.bfloat16)
                plan = quantizer.plan(x, bits, 0.01 if bits == 8 else 0.002)
                return lambda: plan.quantize(x)
            yield f"quant/{name}/{rows}x{columns}", make, int(rows * columns * (2 + out_bytes))
        for bits, out_bytes in ((8, 1.0), (4, 0.5 + 1 / 16)):
            def make(_i, rows=rows, bits=bits):
                x = torch.randn((rows // 560, 560, columns), device=device).to(torch.bfloat16)
                update = torch.randn_like(x)
                weight = torch.randn(columns, device=device) * 0.1
                plan = norm_quant.plan(x, bits=bits, calibrated_scale=0.01, adaptive=False)
                return lambda: plan.residual_normalize(x, update, None, scale=weight)
            yield f"norm/residual_rms_bits{bits}/{rows}x{columns}", make, int(rows * columns * (6 + out_bytes))
    rows, features = 560, 16384
    for bits, out_bytes in ((16, 2.0), (8, 1.0), (4, 0.5 + 1 / 16)):
        def make(_i, bits=bits):
            packed = torch.randn((rows, 2 * features), device=device).to(torch.bfloat16)
            gate, up = packed[:, :features].contiguous(), packed[:, features:].contiguous()
            plan = fusion.plan(gate, bits, None if bits == 16 else 0.01)
            return lambda: plan.encode(gate, up)
        yield f"geglu/standalone_bits{bits}/{rows}x{features}", make, int(rows * features * (4 + out_bytes))
    columns = 1152
    for rows in (768, 24576):
        for bits, out_bytes in ((8, 1.0), (4, 0.5 + 1 / 16)):
            def make(_i, rows=rows, bits=bits):
                x = torch.randn((rows, columns), device=device).to(torch.bfloat16)
                update = torch.randn_like(x)
                residual = torch.empty_like(x)
                weight = torch.randn(columns, device=device).to(torch.bfloat16)
                bias = torch.randn(columns, device=device).to(torch.bfloat16)
                out = torch.empty((rows, columns if bits == 8 else columns // 2), device=device, dtype=torch.uint8)
                blocked = torch.zeros(_blocked_bytes(rows, columns // 16), device=device, dtype=torch.uint8)
                if bits == 8:
                    return lambda: library.cc_layer_norm_fp8(x.data_ptr(), update.data_ptr(), weight.data_ptr(), bias.data_ptr(),
                                                             residual.data_ptr(), out.data_ptr(), 40.0, rows, columns, stream())
                return lambda: library.cc_layer_norm_fp4(x.data_ptr(), update.data_ptr(), weight.data_ptr(), bias.data_ptr(),
                                                         residual.data_ptr(), out.data_ptr(), blocked.data_ptr(), 0.004, rows, columns, stream())
            yield f"norm/residual_layer_norm_bits{bits}/{rows}x{columns}", make, int(rows * columns * (6 + out_bytes))


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--case", default=".", help="regex over case names")
    parser.add_argument("--launches", type=int, default=32)
    parser.add_argument("--library", action="store_true", help="also time torch's scaled_mm at each linear shape")
    parser.add_argument("--list", action="store_true")
    parser.add_argument("--reference", action="store_true",
                        help="also time the reference's own CUDA kernels (baseline/_ref) at the quantiser / epilogue / norm cases")
    parser.add_argument("--sets", type=int, default=0, help="operand sets in rotation (1 = warm L2; default: enough to exceed the L2)")
    parser.add_argument("--eager", type=int, default=0, help="run this many plain launches per case and no timing (for profilers)")
    parser.add_argument("--flags", type=int, default=0, help="OR-ed into the b2_linear flags (8 = stream the token tile, 64 = one CTA per tile)")
    parser.add_argument("--feature-tile", type=int, default=0, help="features per tile (0 = the library's choice)")
    parser.add_argument("--workspace", action="store_true", help="give the plain launches split-K scratch (the library then decides)")
    parser.add_argument("--unpaired", action="store_true", help="gated NVFP4 cases without the paired gate/up scale layout")
    args = parser.parse_args()
    pattern = re.compile(args.case)
    global FORCED_SETS
    FORCED_SETS = max(0, args.sets)
    if args.list:
        for name, *_ in LINEAR_SHAPES:
            print("linear/" + name)
        return
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    peaks = {"hbm_gbs": 6541.5, "fp8_tflops": 4500.0, "nvfp4_tflops": 9000.0}
    options = {"flags": args.flags, "feature_tile": args.feature_tile, "unpaired": args.unpaired, "workspace": args.workspace}
    sources = (quantiser_cases, geglu_cases, norm_cases, layout_cases, lambda dev: linear_cases(dev, options),
               lambda dev: attention_cases(dev, False), lambda dev: attention_cases(dev, True) if args.library else iter(()))
    reference_us = {}
    if args.reference:
        for name, make, set_bytes in reference_cases(device):
            if pattern.search(name):
                reference_us[name] = round(time_graph(make, set_bytes, args.launches)[0], 2)
    for source in sources:
        for name, make, set_bytes, algorithmic_bytes, flops in source(device):
            if not pattern.search(name):
                continue
            if args.eager > 0:
                print(json.dumps({"case": name, "eager_launches": args.eager, "sets": run_eager(make, set_bytes, args.eager)}), flush=True)
                continue
            microseconds, sets = time_graph(make, set_bytes, args.launches)
            line = {"case": name, "us": round(microseconds, 2), "gbs": round(algorithmic_bytes / microseconds / 1e3, 1),
                    "sets": sets, "l2": "cold" if sets * set_bytes >= L2_BYTES else "warm"}
            if name.startswith("attention/"):
                line["tflops"] = round(flops / microseconds / 1e6, 1)
            elif flops:
                line["tflops"] = round(flops / microseconds / 1e6, 1)
                nominal = peaks["fp8_tflops"] if "fp8" in name else peaks["nvfp4_tflops"]
                line["frac_of_nominal_tensor_peak"] = round(line["tflops"] / nominal, 3)
                if args.library:
                    _, kind, tokens, features, width, epilogue = next(s for s in LINEAR_SHAPES if "linear/" + s[0] == name)
                    rows = 2 * features if epilogue == "geglu" else features
                    library = library_time(kind, tokens, rows, width, device, args.launches)
                    if library is not None:
                        line["torch_scaled_mm_us"] = round(library, 2)
                        line["torch_scaled_mm_tflops"] = round(flops / library / 1e6, 1)
            else:
                line["frac_of_measured_hbm"] = round(line["gbs"] / peaks["hbm_gbs"], 3)
                if name in reference_us:
                    line["reference_kernel_us"] = reference_us[name]
                    line["reference_kernel_gbs"] = round(algorithmic_bytes / reference_us[name] / 1e3, 1)
            print(json.dumps(line), flush=True)
            torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
