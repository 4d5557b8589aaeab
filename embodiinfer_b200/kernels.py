"""Tensor-level wrappers over the C ABI: raw pointers, the caller's current stream, no allocation.

These are the calls the plan objects (``embodiinfer_b200.backend``) and the registry kernels
(``embodiinfer_b200.layers.linear``) are built from.  Every function launches on
``torch.cuda.current_stream(device)`` like the reference's ctypes wrappers
(embodiinfer/backend/cuda/quantization.py:139-166) and raises ``RuntimeError`` on a non-zero status.
"""

from __future__ import annotations

import ctypes

import torch

from . import _native as N


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _ptr(tensor: torch.Tensor | None) -> int | None:
    return None if tensor is None else tensor.data_ptr()


def _require_cuda(*tensors: torch.Tensor | None) -> torch.device:
    device = None
    for tensor in tensors:
        if tensor is None:
            continue
        if not tensor.is_cuda:
            raise ValueError("embodiinfer_b200 kernels require CUDA tensors; there is no CPU fallback")
        if device is None:
            device = tensor.device
        elif tensor.device != device:
            raise ValueError("all operands must live on one CUDA device")
    if device is None:
        raise ValueError("no tensor operands")
    return device


def gelu_table_range(table: torch.Tensor) -> tuple[int, int]:
    """Magnitude-code range of a GELU table that the fused epilogue must keep in shared memory
    (``b2_gelu_table_range``); ``(0, 0)`` when the table has no closed-form tails.  Copies the table
    to the host: call it once per table, outside graph capture."""
    host = table.detach().to("cpu").contiguous().view(torch.uint16)
    if host.numel() != 65536:
        raise ValueError("a GELU table has 65536 entries")
    lo, hi = ctypes.c_int32(0), ctypes.c_int32(0)
    status = N.load().b2_gelu_table_range(host.data_ptr(), ctypes.byref(lo), ctypes.byref(hi))
    if status == N.E_UNSUPPORTED:
        return (0, 0)
    N.check(status, "b2_gelu_table_range")
    return (lo.value, hi.value)


def new_scale_scratch(device: torch.device) -> torch.Tensor:
    """Zeroed scratch for :func:`tensor_scale`; allocate once per plan, outside graph capture."""
    return torch.zeros(N.SCALE_SCRATCH_BYTES // 4, device=device, dtype=torch.int32)


def tensor_scale(x: torch.Tensor, bound: float, flags: int, scratch: torch.Tensor, scale: torch.Tensor) -> None:
    """``scale <- amax(|x|) / bound`` (device fp32), see ``b2_tensor_scale``."""
    device = _require_cuda(x, scratch, scale)
    if x.dtype != torch.bfloat16 or not x.is_contiguous():
        raise ValueError("tensor_scale requires a contiguous bf16 tensor")
    with torch.cuda.device(device):
        status = N.load().b2_tensor_scale(
            x.data_ptr(), x.numel(), float(bound), int(flags), scratch.data_ptr(), scale.data_ptr(), _stream(device)
        )
    N.check(status, "b2_tensor_scale")


def tensor_scale_static(x: torch.Tensor, bound: float, flags: int, scale: torch.Tensor) -> None:
    """``tensor_scale`` for callers that may not allocate or pass scratch memory: the scratch is a static
    array inside the library (``b2_tensor_scale_static``).  At most ``STATIC_SCALE_MAX_COUNT`` elements;
    calls that overlap on one GPU race on the shared array; make the first call on a device outside
    any stream capture."""
    device = _require_cuda(x, scale)
    if x.dtype != torch.bfloat16 or not x.is_contiguous():
        raise ValueError("tensor_scale_static requires a contiguous bf16 tensor")
    with torch.cuda.device(device):
        status = N.load().b2_tensor_scale_static(
            x.data_ptr(), x.numel(), float(bound), int(flags), scale.data_ptr(), _stream(device)
        )
    N.check(status, "b2_tensor_scale_static")


def fp8_quantize(x: torch.Tensor, out: torch.Tensor, scale: torch.Tensor, flags: int) -> None:
    """bf16 -> e4m3 at ``*scale``, see ``b2_fp8_quantize``."""
    device = _require_cuda(x, out, scale)
    if x.dtype != torch.bfloat16 or not x.is_contiguous() or not out.is_contiguous() or out.numel() != x.numel():
        raise ValueError("fp8_quantize requires contiguous bf16 input and a same-sized 1-byte output")
    with torch.cuda.device(device):
        status = N.load().b2_fp8_quantize(
            x.data_ptr(), out.data_ptr(), scale.data_ptr(), x.numel(), int(flags), _stream(device)
        )
    N.check(status, "b2_fp8_quantize")


def nvfp4_quantize(
    x: torch.Tensor,
    out: torch.Tensor,
    scales: torch.Tensor | None,
    blocked: torch.Tensor | None,
    global_scale: torch.Tensor,
    flags: int,
) -> None:
    """bf16 [R, K] -> packed e2m1 + e4m3 block scales, see ``b2_nvfp4_quantize``."""
    device = _require_cuda(x, out, scales, blocked, global_scale)
    if x.dtype != torch.bfloat16 or x.ndim != 2 or not x.is_contiguous():
        raise ValueError("nvfp4_quantize requires a contiguous bf16 matrix")
    rows, columns = x.shape
    with torch.cuda.device(device):
        status = N.load().b2_nvfp4_quantize(
            x.data_ptr(),
            out.data_ptr(),
            _ptr(scales),
            _ptr(blocked),
            global_scale.data_ptr(),
            rows,
            columns,
            int(flags),
            _stream(device),
        )
    N.check(status, "b2_nvfp4_quantize")


def geglu(
    gate: torch.Tensor,
    up: torch.Tensor | None,
    out: torch.Tensor,
    *,
    bits: int,
    table: torch.Tensor,
    rows: int,
    columns: int,
    row_stride: int,
    scale: torch.Tensor | None = None,
    scales: torch.Tensor | None = None,
    blocked: torch.Tensor | None = None,
    flags: int = 0,
) -> None:
    """GELU(gate) * up with the reference's two bf16 roundings, see ``b2_geglu``."""
    device = _require_cuda(gate, up, out, table, scale, scales, blocked)
    with torch.cuda.device(device):
        status = N.load().b2_geglu(
            gate.data_ptr(),
            _ptr(up),
            out.data_ptr(),
            _ptr(scales),
            _ptr(blocked),
            _ptr(scale),
            rows,
            columns,
            row_stride,
            bits,
            table.data_ptr(),
            int(flags),
            _stream(device),
        )
    N.check(status, "b2_geglu")


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor | None = None, *, status: torch.Tensor | None = None,
              codes: torch.Tensor | None = None, multiplier: float | None = None, blocked: torch.Tensor | None = None,
              scales: torch.Tensor | None = None, global_scale: float | None = None) -> torch.Tensor:
    """Unmasked multi-query attention, ``softmax(q k^T / sqrt(D)) v``: q [B, H, T, 256], k / v [B, 1, S, 256], all
    contiguous bf16; returns [B, H, T, 256] (``b2_attention``; the reference's ``SDPAAttention``).  With ``codes`` (a
    contiguous 1-byte [B*T, H*256] tensor) and ``multiplier`` the output is written as the e4m3 rows of the output
    projection instead (``b2_attention_fp8``) and ``codes`` is returned.  With ``codes`` ([B*T, H*128] bytes), ``blocked``
    (the tiled block scales, padding zeroed), ``global_scale`` and optionally ``scales`` (row-major [B*T, H*16]) it is
    written as the projection's NVFP4 rows (``b2_attention_nvfp4``)."""
    _require_cuda(q, k, v)
    if q.dim() != 4 or k.shape != v.shape or k.dim() != 4 or k.shape[1] != 1 or k.shape[0] != q.shape[0] or k.shape[3] != q.shape[3]:
        raise ValueError("attention requires q [B, H, T, D] and k, v [B, 1, S, D]")
    if any(t.dtype != torch.bfloat16 or not t.is_contiguous() for t in (q, k, v)):
        raise ValueError("attention requires contiguous bf16 tensors")
    batch, heads, queries, head_dim = q.shape
    if status is None:
        status = status_word(q.device)
    if codes is not None and blocked is not None:
        rows, blocks = batch * queries, heads * head_dim // 16
        if global_scale is None or codes.element_size() != 1 or not codes.is_contiguous() or codes.numel() * 2 != q.numel() or \
                codes.device != q.device or blocked.element_size() != 1 or not blocked.is_contiguous() or blocked.device != q.device or \
                blocked.numel() < (rows + 127) // 128 * ((blocks + 3) // 4) * 512:
            raise ValueError("NVFP4 attention output needs contiguous codes [B*T, H*D/2], tiled block scales and a global scale")
        if scales is not None and (scales.element_size() != 1 or not scales.is_contiguous() or scales.numel() != rows * blocks or
                                   scales.device != q.device):
            raise ValueError("row-major block scales must be a contiguous 1-byte [B*T, H*D/16] tensor")
        with torch.cuda.device(q.device):
            code = N.load().b2_attention_nvfp4(q.data_ptr(), k.data_ptr(), v.data_ptr(), codes.data_ptr(),
                                               None if scales is None else scales.data_ptr(), blocked.data_ptr(), float(global_scale),
                                               batch, heads, queries, k.shape[2], head_dim, status.data_ptr(), _stream(q.device))
        N.check(code, "b2_attention_nvfp4")
        return codes
    if codes is not None:
        if multiplier is None or codes.element_size() != 1 or not codes.is_contiguous() or codes.numel() != q.numel() or codes.device != q.device:
            raise ValueError("encoded attention output must be a contiguous 1-byte [B*T, H*D] tensor with a multiplier")
        with torch.cuda.device(q.device):
            code = N.load().b2_attention_fp8(q.data_ptr(), k.data_ptr(), v.data_ptr(), codes.data_ptr(), float(multiplier), batch, heads,
                                             queries, k.shape[2], head_dim, status.data_ptr(), _stream(q.device))
        N.check(code, "b2_attention_fp8")
        return codes
    if out is None:
        out = torch.empty_like(q)
    elif out.shape != q.shape or out.dtype != torch.bfloat16 or not out.is_contiguous():
        raise ValueError("attention output must be a contiguous bf16 tensor of the queries' shape")
    with torch.cuda.device(q.device):
        code = N.load().b2_attention(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), batch, heads, queries, k.shape[2],
                                     head_dim, status.data_ptr(), _stream(q.device))
    N.check(code, "b2_attention")
    return out


def _rope_desc(sine: torch.Tensor, cosine: torch.Tensor, q_out: torch.Tensor, k_out: torch.Tensor, v_out: torch.Tensor, *,
               batch: int, tokens: int, heads: int, kv_heads: int, head_dim: int, kv_offset: int = 0) -> "N.RopeDesc":
    """The ``b2_rope_desc`` of these arguments (checked like :func:`rope_split`'s)."""
    _require_cuda(sine, cosine, q_out, k_out, v_out)
    for factor in (sine, cosine):
        if factor.dtype != torch.float32 or not factor.is_contiguous() or factor.shape[-2:] != (tokens, head_dim // 2):
            raise ValueError("rope requires contiguous fp32 factors [tokens, head_dim/2] (optionally with a batch dimension)")
    if q_out.shape != (batch, heads, tokens, head_dim) or not q_out.is_contiguous() or q_out.dtype != torch.bfloat16:
        raise ValueError("q_out must be a contiguous bf16 [batch, heads, tokens, head_dim] tensor")
    for cache in (k_out, v_out):
        if cache.ndim != 4 or cache.shape[0] != batch or cache.shape[1] != kv_heads or cache.shape[3] != head_dim or \
                not cache.is_contiguous() or cache.dtype != torch.bfloat16 or cache.shape != k_out.shape:
            raise ValueError("key/value buffers must be contiguous bf16 [batch, kv_heads, capacity, head_dim] tensors")
    return N.RopeDesc(sine=sine.data_ptr(), cosine=cosine.data_ptr(), q_out=q_out.data_ptr(), k_out=k_out.data_ptr(),
                      v_out=v_out.data_ptr(), factor_batch_stride=tokens * (head_dim // 2) if sine.ndim == 3 else 0,
                      batch=batch, tokens=tokens, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                      kv_capacity=k_out.shape[2], kv_offset=kv_offset)


def rope_split(qkv: torch.Tensor, sine: torch.Tensor, cosine: torch.Tensor, q_out: torch.Tensor, k_out: torch.Tensor,
               v_out: torch.Tensor, *, batch: int, tokens: int, heads: int, kv_heads: int, head_dim: int, kv_offset: int = 0) -> None:
    """Split a packed QKV projection, rotate queries and keys, write ``q_out`` [B, heads, T, D] and the
    keys / values into ``k_out`` / ``v_out`` [B, kv_heads, S, D] at ``kv_offset``; see ``b2_rope_split``.
    ``sine`` / ``cosine``: fp32 [T, D/2] or [B, T, D/2]."""
    device = _require_cuda(qkv, sine, cosine, q_out, k_out, v_out)
    width = (heads + 2 * kv_heads) * head_dim
    if qkv.dtype != torch.bfloat16 or not qkv.is_contiguous() or qkv.numel() != batch * tokens * width:
        raise ValueError("rope_split requires a contiguous bf16 [batch*tokens, (heads + 2*kv_heads)*head_dim] projection")
    for factor in (sine, cosine):
        if factor.dtype != torch.float32 or not factor.is_contiguous() or factor.shape[-2:] != (tokens, head_dim // 2):
            raise ValueError("rope_split requires contiguous fp32 factors [tokens, head_dim/2] (optionally with a batch dimension)")
    if q_out.shape != (batch, heads, tokens, head_dim) or not q_out.is_contiguous() or q_out.dtype != torch.bfloat16:
        raise ValueError("q_out must be a contiguous bf16 [batch, heads, tokens, head_dim] tensor")
    for cache in (k_out, v_out):
        if cache.ndim != 4 or cache.shape[0] != batch or cache.shape[1] != kv_heads or cache.shape[3] != head_dim or \
                not cache.is_contiguous() or cache.dtype != torch.bfloat16:
            raise ValueError("key/value buffers must be contiguous bf16 [batch, kv_heads, capacity, head_dim] tensors")
    stride = tokens * (head_dim // 2) if sine.ndim == 3 else 0
    with torch.cuda.device(device):
        status = N.load().b2_rope_split(qkv.data_ptr(), sine.data_ptr(), cosine.data_ptr(), q_out.data_ptr(), k_out.data_ptr(),
                                        v_out.data_ptr(), batch, tokens, heads, kv_heads, head_dim, stride, k_out.shape[2],
                                        kv_offset, _stream(device))
    N.check(status, "b2_rope_split")


def norm_quant(inputs: torch.Tensor, output: torch.Tensor, *, bits: int, tokens: int, scale: torch.Tensor | None = None,
               modulation: torch.Tensor | None = None, update: torch.Tensor | None = None,
               update_gate: torch.Tensor | None = None, mean: torch.Tensor | None = None,
               global_scale: torch.Tensor | None = None, residual: torch.Tensor | None = None,
               scales: torch.Tensor | None = None, blocked: torch.Tensor | None = None, gate: torch.Tensor | None = None,
               inverse: torch.Tensor | None = None, flags: int = 0) -> None:
    """Residual update + RMSNorm (offset scale or adaptive modulation) + bf16 rounding + encoder over the
    contiguous bf16 rows of ``inputs`` [..., columns]; see ``b2_norm_quant`` for every argument."""
    present = [t for t in (inputs, output, scale, modulation, update, update_gate, mean, global_scale, residual, scales,
                           blocked, gate, inverse) if t is not None]
    device = _require_cuda(*present)
    if inputs.dtype != torch.bfloat16 or not inputs.is_contiguous():
        raise ValueError("norm_quant requires contiguous bf16 rows")
    for other in (update, residual):
        if other is not None and (other.shape != inputs.shape or other.dtype != torch.bfloat16 or not other.is_contiguous()):
            raise ValueError("update and residual must match the input's shape, dtype and layout")
    for affine in (scale, modulation, mean, inverse):
        if affine is not None and (affine.dtype != torch.float32 or not affine.is_contiguous()):
            raise ValueError("scale, modulation, mean and inverse must be contiguous fp32 tensors")
    columns = inputs.shape[-1]
    rows = inputs.numel() // columns
    desc = N.NormDesc(
        input=inputs.data_ptr(), update=_ptr(update), update_gate=_ptr(update_gate), scale=_ptr(scale),
        modulation=_ptr(modulation), mean=_ptr(mean), global_scale=_ptr(global_scale), residual=_ptr(residual),
        output=output.data_ptr(), scales=_ptr(scales), blocked=_ptr(blocked), gate=_ptr(gate), inverse=_ptr(inverse),
        rows=rows, columns=columns, tokens=tokens, bits=bits, flags=int(flags))
    with torch.cuda.device(device):
        status = N.load().b2_norm_quant(ctypes.byref(desc), _stream(device))
    N.check(status, "b2_norm_quant")


def layer_norm_quant(inputs: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, output: torch.Tensor, *, bits: int,
                     scale_value: float = 1.0, update: torch.Tensor | None = None, residual: torch.Tensor | None = None,
                     scales: torch.Tensor | None = None, blocked: torch.Tensor | None = None,
                     statistics: torch.Tensor | None = None) -> None:
    """Residual update + LayerNorm + bf16 rounding + encoder over the contiguous bf16 rows of ``inputs``
    [..., columns]; ``scale_value`` is the e4m3 multiplier (bits 8) or the NVFP4 global scale (bits 4); see
    ``b2_layer_norm_quant``."""
    device = _require_cuda(inputs, weight, bias, output, update, residual, scales, blocked, statistics)
    if inputs.dtype != torch.bfloat16 or not inputs.is_contiguous():
        raise ValueError("layer_norm_quant requires contiguous bf16 rows")
    columns = inputs.shape[-1]
    for affine in (weight, bias):
        if affine.dtype != torch.bfloat16 or affine.shape != (columns,) or not affine.is_contiguous():
            raise ValueError("weight and bias must be contiguous bf16 [columns] tensors")
    for other in (update, residual):
        if other is not None and (other.shape != inputs.shape or other.dtype != torch.bfloat16 or not other.is_contiguous()):
            raise ValueError("update and residual must match the input's shape, dtype and layout")
    with torch.cuda.device(device):
        status = N.load().b2_layer_norm_quant(inputs.data_ptr(), _ptr(update), weight.data_ptr(), bias.data_ptr(), _ptr(residual),
                                              output.data_ptr(), _ptr(scales), _ptr(blocked), _ptr(statistics), float(scale_value),
                                              inputs.numel() // columns, columns, bits, _stream(device))
    N.check(status, "b2_layer_norm_quant")


def bhsd_quant(attended: torch.Tensor, output: torch.Tensor, *, bits: int, scale_value: float = 1.0,
               scales: torch.Tensor | None = None, blocked: torch.Tensor | None = None) -> None:
    """Attention output [B, H, S, D] (any strides with D contiguous) -> encoded rows [B*S, H*D]; ``scale_value`` is
    the e4m3 multiplier (bits 8) or the NVFP4 global scale (bits 4); see ``b2_bhsd_quant``."""
    device = _require_cuda(attended, output, scales, blocked)
    if attended.dtype != torch.bfloat16 or attended.ndim != 4 or attended.stride(3) != 1:
        raise ValueError("bhsd_quant requires a bf16 [B, H, S, D] tensor whose last dimension is contiguous")
    batch, heads, tokens, head_dim = attended.shape
    with torch.cuda.device(device):
        status = N.load().b2_bhsd_quant(attended.data_ptr(), output.data_ptr(), _ptr(scales), _ptr(blocked), float(scale_value),
                                        attended.stride(0), attended.stride(1), attended.stride(2), batch, heads, tokens,
                                        head_dim, bits, _stream(device))
    N.check(status, "b2_bhsd_quant")


def normalize_frames(frames: torch.Tensor, images: torch.Tensor) -> None:
    """``(frames / 255) * 2 - 1`` into fp32 ``images`` [cameras, 3, H, W]; ``frames`` is contiguous uint8
    [cameras, H, W, 3] (same checks and errors as the reference's ``normalize_frames``)."""
    if frames.dtype != torch.uint8 or frames.ndim != 4 or frames.shape[3] != 3 or not frames.is_contiguous():
        raise ValueError("frames must be contiguous uint8 [cameras, height, width, 3]")
    if images.dtype != torch.float32 or images.ndim != 4 or tuple(images.shape[:2]) != (frames.shape[0], 3) or \
            not images.is_contiguous():
        raise ValueError("images must be contiguous float32 [cameras, 3, height, width]")
    if frames.device.type != "cuda" or images.device != frames.device:
        raise ValueError("frames and images must share a CUDA device")
    if tuple(images.shape[2:]) != tuple(frames.shape[1:3]):
        raise ValueError("images must have the frame height and width")
    with torch.cuda.device(frames.device):
        status = N.load().b2_normalize_frames(frames.data_ptr(), images.data_ptr(), frames.shape[0],
                                              frames.shape[1] * frames.shape[2], _stream(frames.device))
    N.check(status, "b2_normalize_frames")


def frames_to_patches(frames: torch.Tensor, patches: torch.Tensor, patch: int) -> None:
    """uint8 frames [cameras, H, W, 3] -> bf16 patch rows [cameras * (H/patch) * (W/patch), 3*patch*patch] holding
    ``bf16((x / 255) * 2 - 1)`` in (channel, y, x) order; see ``b2_frames_to_patches``."""
    device = _require_cuda(frames, patches)
    if frames.dtype != torch.uint8 or frames.ndim != 4 or frames.shape[3] != 3 or not frames.is_contiguous():
        raise ValueError("frames must be contiguous uint8 [cameras, height, width, 3]")
    cameras, height, width, _ = frames.shape
    expected = (cameras * (height // patch) * (width // patch), 3 * patch * patch)
    if patches.dtype != torch.bfloat16 or tuple(patches.shape) != expected or not patches.is_contiguous():
        raise ValueError("patches must be contiguous bf16 [cameras * grid_h * grid_w, 3 * patch * patch]")
    with torch.cuda.device(device):
        status = N.load().b2_frames_to_patches(frames.data_ptr(), patches.data_ptr(), cameras, height, width, patch,
                                               _stream(device))
    N.check(status, "b2_frames_to_patches")


# ---- the status word of the bounded waits -------------------------------------------------------------
# Every wait inside the tensor-core kernels is bounded; a wait that runs out leaves a code in the launch's status
# word and the kernel drains with a wrong result instead of hanging.  The plan objects and the registry kernels
# pass ONE word per device to every launch (a launch only ever writes a non-zero code into a zero word), and the
# host reads it where it synchronises anyway: at the end of a rollout step, when a workspace scope is released.
STATUS_NAMES = {0x101: "the TMA producer waited for a free stage", 0x102: "the MMA issuer waited for a filled stage",
                0x103: "the MMA issuer waited for a drained accumulator", 0x104: "the epilogue waited for a finished accumulator",
                0x105: "the producer waited for its copies in flight", 0x106: "a CTA waited for the other K ranges of its tile",
                0x107: "a CTA waited for the partial sums of its cluster",
                0x108: "a CTA waited for the partial attention rows of its cluster"}
_status_words: dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """The device's status word (int32, zero unless a bounded wait expired since the last check).  Created on first
    use: touch it once before capturing a CUDA graph, as with every plan buffer."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    word = _status_words.get(index)
    if word is None:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("Warm tensor-core launches before graph capture")
        word = _status_words[index] = torch.zeros(1, device=torch.device("cuda", index), dtype=torch.int32)
    return word


def check_status(device: torch.device) -> None:
    """Read the device's status word (this synchronises with the device) and raise ``RuntimeError`` naming the wait
    that expired; the word is cleared so that later launches are judged on their own."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    word = _status_words.get(index)
    if word is None:
        return
    code = int(word.item())
    if code != 0:
        word.zero_()
        what = STATUS_NAMES.get(code, "an unknown wait")
        raise RuntimeError(f"a tensor-core launch on cuda:{index} gave up a bounded wait (status {code:#x}: {what} for longer than "
                           "its limit); its result and those of the launches after it are invalid")


_WORKSPACE_BYTES = 32 << 20
_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def linear_workspace(device: torch.device) -> torch.Tensor:
    """Zeroed split-K scratch for launches on the current stream of ``device`` (one per device and stream,
    created on first use: warm a shape up before capturing it, as with every plan buffer).  Launches that
    follow one another on a stream can share it: each leaves its ticket words zero again."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), _stream(device))
    workspace = _workspaces.get(key)
    if workspace is None:
        workspace = _workspaces[key] = torch.zeros(_WORKSPACE_BYTES, device=device, dtype=torch.uint8)
    return workspace


def linear(
    *,
    kind: int,
    epilogue: int,
    out_format: int,
    tokens: int,
    features: int,
    width: int,
    act: torch.Tensor,
    act_scale: torch.Tensor,
    weight: torch.Tensor,
    weight_scale: torch.Tensor,
    out: torch.Tensor,
    act_scales: torch.Tensor | None = None,
    weight_scales: torch.Tensor | None = None,
    weight_scale_up: torch.Tensor | None = None,
    bias: torch.Tensor | None = None,
    residual: torch.Tensor | None = None,
    gelu_table: torch.Tensor | None = None,
    out_scale: torch.Tensor | None = None,
    out_scales: torch.Tensor | None = None,
    out_blocked: torch.Tensor | None = None,
    status: torch.Tensor | None = None,
    flags: int = 0,
    feature_tile: int = 0,
    gelu_range: tuple[int, int] = (0, 0),
    workspace: torch.Tensor | None | bool = None,
    rope: dict | None = None,
) -> None:
    """One fused tensor-core launch, see ``b2_linear``.  ``status``: the word an expired bounded wait is reported in
    (default: the device's word, read by :func:`check_status`).  ``workspace``: zeroed split-K scratch, e.g.
    :func:`linear_workspace`; without one (the default) K is never split.  The fix-up through the L2 costs
    more than the shorter K loop saves at every shape of the pi0.5 stacks measured so far (560x2048x16384:
    35 vs 28 us; 10x2560x1024: 12.5 vs 5.6 us), so the plans do not pass one."""
    device = _require_cuda(
        act, act_scale, weight, weight_scale, out, act_scales, weight_scales, weight_scale_up, bias, residual, gelu_table, out_scale,
        out_scales, out_blocked, status,
    )
    if status is None:
        status = status_word(device)
    desc = N.LinearDesc(
        kind=kind,
        epilogue=epilogue,
        out_format=out_format,
        flags=flags,
        tokens=tokens,
        features=features,
        width=width,
        feature_tile=feature_tile,
        gelu_lo=gelu_range[0],
        gelu_hi=gelu_range[1],
        act=act.data_ptr(),
        act_scales=_ptr(act_scales),
        act_scale=act_scale.data_ptr(),
        weight=weight.data_ptr(),
        weight_scales=_ptr(weight_scales),
        weight_scale=weight_scale.data_ptr(),
        weight_scale_up=_ptr(weight_scale_up),
        bias=_ptr(bias),
        residual=_ptr(residual),
        gelu_table=_ptr(gelu_table),
        out_scale=_ptr(out_scale),
        out=out.data_ptr(),
        out_scales=_ptr(out_scales),
        out_blocked=_ptr(out_blocked),
        status=_ptr(status),
    )
    if isinstance(workspace, torch.Tensor):
        desc.workspace, desc.workspace_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
    preparation = None
    if rope is not None:
        # the attention preparation as this projection's epilogue (``b2_linear_desc.rope``); `out` is not written
        preparation = _rope_desc(**rope)
        desc.rope = ctypes.addressof(preparation)
    with torch.cuda.device(device):
        code = N.load().b2_linear(ctypes.byref(desc), _stream(device))
    N.check(code, "b2_linear")
