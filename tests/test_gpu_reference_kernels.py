"""This library's kernels against the reference's OWN CUDA kernels, run on the same GPU on the same seeded inputs.

The reference package is imported unmodified from ``baseline/_ref`` (installed there by
``baseline/install_reference.py``; the folder is not tracked).  Its quantiser, GELU*up epilogue and norm + encoder
kernels are plain SIMT kernels that the package compiles with nvcc on first use
(embodiinfer/backend/cuda/native.py:43-119); they are called through the reference's own classes
(``CudaQuantizer``, ``GeluMulFusion``, ``NormQuantFusion`` / ``NormQuantReduceFusion``) or, where the reference
binds them inside a policy (``cc_layer_norm_*``, ``cc_bhsd_*``: policies/pi05/inference/vision.py:68-110), through
the compiled library with the argument lists written there.  Every output (codes, per-tensor scale, row-major and
tiled block scales, residual, gate) must be byte-equal.  This pins the CUDA-route NVFP4 encoder, the LayerNorm
arithmetic and the kernels' row-sum order on reference output; the CPU oracle restates the same sources.

The tests skip when ``baseline/_ref`` or nvcc is missing.  The reference's kernels that wait on other blocks
(action bridge, decode attention) are not touched.
"""

from __future__ import annotations

import ctypes
import os
import shutil
import sys
import tempfile
from pathlib import Path

import numpy as np
import pytest
import torch

from embodiinfer_b200 import _native as N
from embodiinfer_b200 import kernels as K
from tests.util import make_input, u8

pytestmark = pytest.mark.gpu

REFERENCE = Path(__file__).resolve().parent.parent / "baseline" / "_ref"


@pytest.fixture(scope="module")
def reference():
    """The reference's CUDA back ends, compiled into a scratch cache."""
    if not (REFERENCE / "embodiinfer").exists():
        pytest.skip("baseline/_ref is not installed (python baseline/install_reference.py <checkout>)")
    if shutil.which("nvcc") is None and not Path("/usr/local/cuda/bin/nvcc").exists():
        pytest.skip("the reference compiles its kernels with nvcc")
    cache = tempfile.mkdtemp(prefix="embodiinfer_ref_cache_")
    os.environ["EMBODIINFER_CUDA_CACHE_DIR"] = cache
    sys.path.insert(0, str(REFERENCE))
    try:
        from embodiinfer.backend.cuda.activation import GeluMulFusion
        from embodiinfer.backend.cuda.norm_quant import NormQuantFusion, NormQuantReduceFusion
        from embodiinfer.backend.cuda.normalization import NormFusion
        from embodiinfer.backend.cuda.quantization import CudaQuantizer

        quantizer = CudaQuantizer()
        norm = NormFusion()
        yield dict(quantizer=quantizer, gelu=GeluMulFusion(quantizer, approximate="tanh"), norm_quant=NormQuantFusion(quantizer, norm),
                   norm_reduce=NormQuantReduceFusion(quantizer, norm))
        torch.cuda.synchronize()
    finally:
        sys.path.remove(str(REFERENCE))
        shutil.rmtree(cache, ignore_errors=True)


def blocked_bytes(rows, blocks):
    return -(-rows // 128) * 128 * (-(-blocks // 4) * 4)


def same(ours: torch.Tensor, theirs: torch.Tensor, what: str) -> None:
    a, b = u8(ours).reshape(-1), u8(theirs).reshape(-1)
    assert a.shape == b.shape, what
    assert np.array_equal(a, b), f"{what}: {(a != b).sum()} of {a.size} bytes differ"


@pytest.mark.parametrize("rows,columns", [(560, 2048), (37, 64), (130, 1152), (1, 16384)])
@pytest.mark.parametrize("dynamic", (False, True))
def test_quantizer_fp8(device, reference, rows, columns, dynamic):
    """cc_scale + cc_fp8 (csrc/quantize.cu:38-67, 116-133) vs b2_tensor_scale + b2_fp8_quantize."""
    x = make_input((rows, columns), 7 + rows, multiplier=3.0).to(device)
    plan = reference["quantizer"].plan(x, 8, None if dynamic else 0.0173).quantize(x)
    scale = torch.full((), 0.0173, device=device)
    if dynamic:
        K.tensor_scale(x, 448.0, N.SCALAR_RCP, K.new_scale_scratch(device), scale)
    out = torch.empty((rows, columns), device=device, dtype=torch.uint8)
    K.fp8_quantize(x, out, scale, N.SPEC_C)
    torch.cuda.synchronize()
    same(scale.reshape(1), plan.scale.reshape(1), "per-tensor scale")
    same(out, plan.output, "e4m3 codes")


@pytest.mark.parametrize("rows,columns", [(560, 2048), (37, 64), (130, 1152), (200, 16384)])
@pytest.mark.parametrize("dynamic", (False, True))
def test_quantizer_nvfp4(device, reference, rows, columns, dynamic):
    """cc_scale + cc_fp4 (csrc/quantize.cu:69-104, 135-142) vs b2_tensor_scale + b2_nvfp4_quantize: packed codes,
    row-major block scales and the 128x4-tile layout including its zero padding."""
    x = make_input((rows, columns), 11 + rows, multiplier=2.0).to(device)
    plan = reference["quantizer"].plan(x, 4, None if dynamic else 0.0031).quantize(x)
    scale = torch.full((), 0.0031, device=device)
    if dynamic:
        K.tensor_scale(x, 448.0 * 6.0, N.SCALAR_RCP, K.new_scale_scratch(device), scale)
    out = torch.empty((rows, columns // 2), device=device, dtype=torch.uint8)
    scales = torch.empty((rows, columns // 16), device=device, dtype=torch.uint8)
    blocked = torch.zeros(blocked_bytes(rows, columns // 16), device=device, dtype=torch.uint8)
    K.nvfp4_quantize(x, out, scales, blocked, scale, N.SPEC_C)
    torch.cuda.synchronize()
    same(scale.reshape(1), plan.scale.reshape(1), "global scale")
    same(out, plan.output, "e2m1 codes")
    same(scales, plan.scales, "row-major block scales")
    same(blocked, plan.blocked, "tiled block scales")


@pytest.mark.parametrize("bits", (16, 8, 4))
@pytest.mark.parametrize("rows,columns", [(560, 4096), (33, 64), (130, 1152)])
def test_gelu_mul(device, reference, bits, rows, columns):
    """cc_geglu / cc_geglu_fp4 / cc_geglu_packed (csrc/fusion.cu:5-200) vs b2_geglu, separate and packed operands."""
    packed = make_input((rows, 2 * columns), 5 + columns, multiplier=1.5).to(device)
    gate, up = packed[:, :columns].contiguous(), packed[:, columns:].contiguous()
    fusion = reference["gelu"]
    scale_value = {16: None, 8: 0.0213, 4: 0.0041}[bits]
    theirs = fusion.plan(gate, bits, scale_value).encode(gate, up)
    width = {16: 2 * columns, 8: columns, 4: columns // 2}[bits]
    scale = None if bits == 16 else torch.full((), scale_value, device=device)
    scales = torch.empty((rows, columns // 16), device=device, dtype=torch.uint8) if bits == 4 else None
    blocked = torch.zeros(blocked_bytes(rows, columns // 16), device=device, dtype=torch.uint8) if bits == 4 else None
    out = torch.empty((rows, width), device=device, dtype=torch.uint8)
    K.geglu(gate, up, out, bits=bits, table=fusion.table, rows=rows, columns=columns, row_stride=columns, scale=scale,
            scales=scales, blocked=blocked, flags=N.GEGLU_TRUE_DIV if bits == 8 and (rows * columns) % 8 else 0)
    torch.cuda.synchronize()
    same(out, theirs.output, "hidden activation")
    if bits == 4:
        same(scales, theirs.scales, "row-major block scales")
        same(blocked, theirs.blocked, "tiled block scales")
    if bits != 4:
        theirs_packed = fusion.plan(gate, bits, scale_value).encode_packed(packed)
        ours_packed = torch.empty_like(out)
        K.geglu(packed, packed[:, columns:], ours_packed, bits=bits, table=fusion.table, rows=rows, columns=columns,
                row_stride=2 * columns, scale=scale)
        torch.cuda.synchronize()
        same(ours_packed, theirs_packed.output, "hidden activation from the packed matrix")


@pytest.mark.parametrize("bits", (8, 4))
@pytest.mark.parametrize("batch,tokens,columns,adaptive", [(2, 35, 2048, False), (3, 10, 1024, True), (2, 9, 1152, False), (2, 7, 320, True)])
def test_norm_quant_given_mean(device, reference, bits, batch, tokens, columns, adaptive):
    """cc_norm_quant (csrc/norm_quant.cu:91-112; torch computes the mean of squares) vs b2_norm_quant with that mean."""
    generator = torch.Generator().manual_seed(columns + tokens)
    x = (torch.randn((batch, tokens, columns), generator=generator) * 3).to(torch.bfloat16).to(device)
    scale = None if adaptive else (torch.randn((columns,), generator=generator) * 0.2).to(device)
    modulation = (torch.randn((batch, 3 * columns), generator=generator) * 0.3).to(device) if adaptive else None
    calibrated = {8: 0.011, 4: 0.0023}[bits]
    plan = reference["norm_quant"].plan(x, bits=bits, calibrated_scale=calibrated, adaptive=adaptive)
    plan.normalize(x, scale=scale, modulation=modulation)
    rows = batch * tokens
    out = torch.empty((rows, columns if bits == 8 else columns // 2), device=device, dtype=torch.uint8)
    scales = torch.empty((rows, columns // 16), device=device, dtype=torch.uint8) if bits == 4 else None
    blocked = torch.zeros(blocked_bytes(rows, columns // 16), device=device, dtype=torch.uint8) if bits == 4 else None
    gate = torch.empty((batch, columns), device=device, dtype=torch.bfloat16) if adaptive else None
    K.norm_quant(x, out, bits=bits, tokens=tokens, scale=scale, modulation=modulation, mean=plan.mean.reshape(-1).contiguous(),
                 global_scale=plan.scale, scales=scales, blocked=blocked, gate=gate)
    torch.cuda.synchronize()
    same(out, plan.output, "codes")
    if bits == 4:
        same(scales, plan.scales, "row-major block scales")
        same(blocked, plan.blocked, "tiled block scales")
    if adaptive:
        same(gate, plan.gate, "gate")


@pytest.mark.parametrize("bits", (8, 4))
@pytest.mark.parametrize("batch,tokens,columns,adaptive,gated", [(2, 35, 2048, False, False), (3, 10, 1024, True, True), (2, 9, 1152, False, False),
                                                                 (2, 7, 320, True, True), (8, 560, 2048, False, False)])
def test_norm_quant_single_pass(device, reference, bits, batch, tokens, columns, adaptive, gated):
    """cc_norm_quant_reduce (csrc/norm_quant.cu:114-562: residual update, in-kernel row sums, affine, encoder) vs
    b2_norm_quant without a mean: the same GPU evaluates the same reciprocal root, so everything is byte-equal."""
    generator = torch.Generator().manual_seed(3 * columns + tokens)
    x = (torch.randn((batch, tokens, columns), generator=generator) * 3).to(torch.bfloat16).to(device)
    update = torch.randn((batch, tokens, columns), generator=generator).to(torch.bfloat16).to(device)
    update_gate = torch.randn((batch, 1, columns), generator=generator).to(torch.bfloat16).to(device) if gated else None
    scale = None if adaptive else (torch.randn((columns,), generator=generator) * 0.2).to(device)
    modulation = (torch.randn((batch, 3 * columns), generator=generator) * 0.3).to(device) if adaptive else None
    calibrated = {8: 0.011, 4: 0.0023}[bits]
    plan = reference["norm_reduce"].plan(x, bits=bits, calibrated_scale=calibrated, adaptive=adaptive)
    residual_theirs, _, gate_theirs = plan.residual_normalize(x, update, update_gate, scale=scale, modulation=modulation)
    rows = batch * tokens
    out = torch.empty((rows, columns if bits == 8 else columns // 2), device=device, dtype=torch.uint8)
    scales = torch.empty((rows, columns // 16), device=device, dtype=torch.uint8) if bits == 4 else None
    blocked = torch.zeros(blocked_bytes(rows, columns // 16), device=device, dtype=torch.uint8) if bits == 4 else None
    gate = torch.empty((batch, columns), device=device, dtype=torch.bfloat16) if adaptive else None
    residual = torch.empty_like(x)
    K.norm_quant(x, out, bits=bits, tokens=tokens, scale=scale, modulation=modulation, update=update,
                 update_gate=None if update_gate is None else update_gate.reshape(batch, columns), global_scale=plan.scale,
                 residual=residual, scales=scales, blocked=blocked, gate=gate)
    torch.cuda.synchronize()
    same(residual, residual_theirs, "residual")
    same(out, plan.output, "codes")
    if bits == 4:
        same(scales, plan.scales, "row-major block scales")
        same(blocked, plan.blocked, "tiled block scales")
    if adaptive:
        same(gate, gate_theirs, "gate")


@pytest.mark.parametrize("bits", (8, 4))
@pytest.mark.parametrize("rows,columns,with_update", [(37, 1152, True), (130, 2048, False), (512, 1152, True), (9, 1024, True)])
def test_layer_norm(device, reference, bits, rows, columns, with_update):
    """cc_layer_norm_fp8 / cc_layer_norm_fp4 (csrc/norm_quant.cu:564-687, 797-931) vs b2_layer_norm_quant."""
    library = reference["norm_quant"].library
    pointer = ctypes.c_void_p
    library.cc_layer_norm_fp8.argtypes = [pointer] * 6 + [ctypes.c_float, ctypes.c_int, ctypes.c_int, pointer]
    library.cc_layer_norm_fp4.argtypes = [pointer] * 7 + [ctypes.c_float, ctypes.c_int, ctypes.c_int, pointer]
    library.cc_layer_norm_fp8.restype = library.cc_layer_norm_fp4.restype = ctypes.c_int
    generator = torch.Generator().manual_seed(rows + columns)
    x = (torch.randn((rows, columns), generator=generator) * 2 + 0.3).to(torch.bfloat16).to(device)
    update = torch.randn((rows, columns), generator=generator).to(torch.bfloat16).to(device) if with_update else None
    weight = torch.randn((columns,), generator=generator).to(torch.bfloat16).to(device)
    bias = torch.randn((columns,), generator=generator).to(torch.bfloat16).to(device)
    scale_value = {8: 448.0 / 11.0, 4: 11.0 / 2688.0}[bits]
    stream = torch.cuda.current_stream(device).cuda_stream
    width = columns if bits == 8 else columns // 2
    out_theirs = torch.zeros((rows, width), device=device, dtype=torch.uint8)
    residual_theirs = torch.zeros((rows, columns), device=device, dtype=torch.bfloat16)
    blocked_theirs = torch.zeros(blocked_bytes(rows, columns // 16), device=device, dtype=torch.uint8)
    update_pointer = None if update is None else update.data_ptr()
    if bits == 8:
        status = library.cc_layer_norm_fp8(x.data_ptr(), update_pointer, weight.data_ptr(), bias.data_ptr(), residual_theirs.data_ptr(),
                                           out_theirs.data_ptr(), scale_value, rows, columns, stream)
    else:
        status = library.cc_layer_norm_fp4(x.data_ptr(), update_pointer, weight.data_ptr(), bias.data_ptr(), residual_theirs.data_ptr(),
                                           out_theirs.data_ptr(), blocked_theirs.data_ptr(), scale_value, rows, columns, stream)
    assert status == 0
    out = torch.zeros_like(out_theirs)
    residual = torch.zeros_like(residual_theirs)
    blocked = torch.zeros_like(blocked_theirs) if bits == 4 else None
    K.layer_norm_quant(x, weight, bias, out, bits=bits, scale_value=scale_value, update=update, residual=residual, blocked=blocked)
    torch.cuda.synchronize()
    same(out, out_theirs, "codes")
    if with_update:
        same(residual, residual_theirs, "residual")
    if bits == 4:
        same(blocked, blocked_theirs, "tiled block scales")


@pytest.mark.parametrize("bits", (8, 4))
@pytest.mark.parametrize("batch,heads,tokens,head_dim", [(1, 8, 560, 256), (3, 8, 10, 256), (2, 16, 256, 72)])
def test_attention_output_encoder(device, reference, bits, batch, heads, tokens, head_dim):
    """cc_bhsd_fp8 / cc_bhsd_fp4 (csrc/norm_quant.cu:689-795) vs b2_bhsd_quant."""
    if bits == 4 and head_dim % 16:
        pytest.skip("NVFP4 blocks need head_dim % 16 == 0")
    library = reference["norm_quant"].library
    generator = torch.Generator().manual_seed(head_dim + tokens)
    attended = (torch.randn((batch, heads, tokens, head_dim), generator=generator) * 2).to(torch.bfloat16).to(device)
    rows, columns = batch * tokens, heads * head_dim
    scale_value = {8: 448.0 / 9.0, 4: 9.0 / 2688.0}[bits]
    stream = torch.cuda.current_stream(device).cuda_stream
    out_theirs = torch.zeros((rows, columns if bits == 8 else columns // 2), device=device, dtype=torch.uint8)
    blocked_theirs = torch.zeros(blocked_bytes(rows, columns // 16), device=device, dtype=torch.uint8)
    strides = attended.stride()
    if bits == 8:
        status = library.cc_bhsd_fp8(attended.data_ptr(), out_theirs.data_ptr(), scale_value, strides[0], strides[1], strides[2],
                                     batch, heads, tokens, head_dim, stream)
    else:
        status = library.cc_bhsd_fp4(attended.data_ptr(), out_theirs.data_ptr(), blocked_theirs.data_ptr(), scale_value, strides[0],
                                     strides[1], strides[2], batch, heads, tokens, head_dim, stream)
    assert status == 0
    out = torch.zeros_like(out_theirs)
    blocked = torch.zeros_like(blocked_theirs) if bits == 4 else None
    K.bhsd_quant(attended, out, bits=bits, scale_value=scale_value, blocked=blocked)
    torch.cuda.synchronize()
    same(out, out_theirs, "codes")
    if bits == 4:
        same(blocked, blocked_theirs, "tiled block scales")
