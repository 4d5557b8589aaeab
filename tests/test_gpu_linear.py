"""The fused tensor-core Linear through the C ABI against the oracle on identical quantised operands.

Tolerance: relative Frobenius <= 1e-3 and max-abs <= 2e-2 in bf16 (tests/util.py explains the one-ulp
allowance for large magnitudes).  Encoded outputs of the fused epilogues (e4m3 / e2m1 codes and block
scales) are compared bit for bit against the stand-alone epilogue run on the kernel's own bf16 gate/up.
"""

from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

from embodiinfer_b200 import _native as N
from embodiinfer_b200 import kernels as K
from embodiinfer_b200.backend.quantization import blocked_scale_bytes
from oracle import quant_oracle as O
from tests.util import assert_gated_close, assert_gemm_close, bits, gelu_table_cpu, make_input, make_weight, u8

pytestmark = pytest.mark.gpu


def operands(kind, tokens, rows, width, seed, device):
    x = bits(make_input((tokens, width), seed))
    w = bits(make_weight((rows, width), seed).to(torch.bfloat16))
    if kind == "fp8":
        aq, a_s = O.fp8_quantize_C(x)
        wq, w_s = O.fp8_quantize_C(w)
        host = dict(a=aq, a_s=a_s, w=wq, w_s=w_s)
        dev = dict(kind=N.KIND_FP8, act=torch.from_numpy(aq).to(device), weight=torch.from_numpy(wq).to(device))
    else:
        ap, asl, abl, a_s = O.nvfp4_quantize_C(x)
        wp, wsl, wbl, w_s = O.nvfp4_quantize_C(w)
        host = dict(a=ap, a_sl=asl, a_s=a_s, w=wp, w_sl=wsl, w_s=w_s)
        dev = dict(kind=N.KIND_NVFP4, act=torch.from_numpy(ap).to(device), weight=torch.from_numpy(wp).to(device),
                   act_scales=torch.from_numpy(abl).to(device), weight_scales=torch.from_numpy(wbl).to(device))
    dev["act_scale"] = torch.tensor(float(host["a_s"]), device=device)
    dev["weight_scale"] = torch.tensor(float(host["w_s"]), device=device)
    return host, dev


def accumulate(kind, host):
    if kind == "fp8":
        return O.e4m3_decode(host["a"]).astype(np.float64) @ O.e4m3_decode(host["w"]).astype(np.float64).T
    return O.nvfp4_block_acc(host["a"], host["a_sl"], host["w"], host["w_sl"])


LINEAR_CASES = [
    # tokens, features, width, tile
    (32, 128, 128, 64), (200, 256, 1024, 64), (10, 2560, 1024, 0), (80, 1024, 2048, 0), (640, 4096, 1024, 0),
    (560, 2048, 2048, 0), (560, 2048, 2048, 64), (560, 2048, 2048, 128), (560, 2048, 2048, 192), (560, 2048, 2048, 256),
    (1, 64, 64, 0), (17, 72, 192, 0), (129, 200, 320, 0), (559, 1152, 1152, 0), (561, 1024, 2048, 0),
    # one tile per CTA and a long K: several K atoms per ring slot, with a short last slot and a ragged last atom
    (10, 1024, 4096, 0), (100, 256, 1152, 0), (64, 128, 2304, 0), (50, 192, 2240, 0), (128, 64, 8192, 0),
    # 32 features per tile: every 32-row quarter of a 128-row feature-scale block, a ragged last tile, two token tiles
    (10, 160, 256, 32), (70, 96, 512, 32), (200, 256, 1024, 32), (24, 200, 2048, 32), (80, 1024, 4096, 0),
    # cluster schedule: 1 .. 128 tokens, every cluster size (8 / 4 / 2 / 1 by the number of feature tiles and K atoms),
    # K ranges of unequal length, a ragged last K atom, features that end inside a tile, more tiles than one wave
    (5, 128, 128, 0), (16, 128, 256, 0), (33, 256, 640, 0), (128, 1024, 4096, 0), (127, 2176, 1024, 0), (9, 4352, 1152, 0),
    (3, 9600, 512, 0), (48, 20480, 256, 0), (96, 1032, 3392, 0), (2, 136, 16384, 0),
]


@pytest.mark.parametrize("kind", ("fp8", "nvfp4"))
@pytest.mark.parametrize("tokens,features,width,tile", LINEAR_CASES)
def test_linear_matches_oracle(device, kind, tokens, features, width, tile):
    host, dev = operands(kind, tokens, features, width, tokens + features, device)
    status = torch.zeros(1, device=device, dtype=torch.int32)
    out = torch.full((tokens + 1, features), float("nan"), device=device, dtype=torch.bfloat16)
    call = dict(epilogue=N.EPI_LINEAR, out_format=N.OUT_BF16, tokens=tokens, features=features, width=width, out=out[:tokens],
                status=status, feature_tile=tile, **dev)
    if kind == "nvfp4" and tile == 32:        # 32-feature tiles are FP8 only
        with pytest.raises(RuntimeError, match="error -2"):
            K.linear(**call)
        return
    if kind == "fp8":
        want = O.fp8_linear(host["a"], host["a_s"], host["w"], host["w_s"])
    else:
        want = O.nvfp4_linear_plan(host["a"], host["a_sl"], host["a_s"], host["w"], host["w_sl"], host["w_s"])
    # up to 128 tokens with no tile asked for: the library's own choice, the cluster schedule (weights as the MMA's "A"
    # operand) and the tile schedule, whose single-tile paths these cases also cover
    schedules = (0, N.LINEAR_CLUSTER, N.LINEAR_SINGLE_CTA) if tokens <= 128 and tile == 0 else (0,)
    for flags in schedules:
        out.fill_(float("nan"))
        K.linear(flags=flags, **call)
        torch.cuda.synchronize()
        assert status.item() == 0
        assert torch.isnan(out[tokens]).all(), "wrote past the last token row"
        assert_gemm_close(bits(out[:tokens]), want)


@pytest.mark.parametrize("kind", ("fp8", "nvfp4"))
def test_siglip_shapes_with_bias(device, kind):
    """K = 4304 is not a multiple of 128 (ragged last K slice); N = 4304 is not a multiple of any tile."""
    for tokens, features, width in ((512, 1152, 4304 if kind == "fp8" else 4288), (512, 4304, 1152), (256, 3456, 1152)):
        host, dev = operands(kind, tokens, features, width, 7 + features, device)
        bias = make_weight((1, features), 9, std=0.1).to(torch.bfloat16).reshape(-1)
        out = torch.empty((tokens, features), device=device, dtype=torch.bfloat16)
        K.linear(epilogue=N.EPI_LINEAR, out_format=N.OUT_BF16, tokens=tokens, features=features, width=width, out=out,
                 bias=bias.to(device), **dev)
        if kind == "fp8":
            want = O.fp8_linear(host["a"], host["a_s"], host["w"], host["w_s"], bits(bias))
        else:
            want = O.nvfp4_linear_plan(host["a"], host["a_sl"], host["a_s"], host["w"], host["w_sl"], host["w_s"])
            want = O.f32_to_bf16(O.bf16_to_f32(want) + O.bf16_to_f32(bits(bias))[None, :])
        assert_gemm_close(bits(out), want)


def test_registry_rounding_bias_and_residual(device):
    """NVFP4 registry route: bf16(bf16(acc) * bf16(g_a*g_w)), then bias and residual as separate bf16 adds."""
    tokens, features, width = 80, 1024, 2048
    host, dev = operands("nvfp4", tokens, features, width, 5, device)
    bias = make_weight((1, features), 3, std=0.1).to(torch.bfloat16).reshape(-1)
    residual = make_input((tokens, features), 4, outliers=False)
    out = torch.empty((tokens, features), device=device, dtype=torch.bfloat16)
    K.linear(epilogue=N.EPI_LINEAR, out_format=N.OUT_BF16, tokens=tokens, features=features, width=width, out=out,
             bias=bias.to(device), residual=residual.to(device), flags=N.LINEAR_ROUND_SCALE_BF16, **dev)
    want = O.nvfp4_linear_registry(host["a"], host["a_sl"], host["a_s"], host["w"], host["w_sl"], host["w_s"], bits(bias))
    want = O.f32_to_bf16(O.bf16_to_f32(want) + O.bf16_to_f32(bits(residual)))
    assert_gemm_close(bits(out), want)


@pytest.mark.parametrize("kind", ("fp8", "nvfp4"))
@pytest.mark.parametrize("tokens,features,width,tile", [(64, 256, 512, 64), (200, 256, 512, 128), (560, 2048, 2048, 0), (130, 384, 1024, 0)])
def test_gated_epilogues(device, kind, tokens, features, width, tile):
    host, dev = operands(kind, tokens, 2 * features, width, 21 + tokens, device)
    table_host = gelu_table_cpu("tanh")
    table = torch.from_numpy(table_host.view(np.int16).copy()).view(torch.uint16).to(device)
    common = dict(epilogue=N.EPI_GEGLU, tokens=tokens, features=features, width=width, gelu_table=table, feature_tile=tile, **dev)
    # bf16 hidden against the oracle (two GEMM outputs, GELU table, product rounding)
    hidden = torch.empty((tokens, features), device=device, dtype=torch.bfloat16)
    K.linear(out_format=N.OUT_BF16, out=hidden, **common)
    y = O.f32_to_bf16((accumulate(kind, host) * float(host["a_s"]) * float(host["w_s"])).astype(np.float32))
    want_hidden = O.gelu_mul(y[:, :features], y[:, features:], table_host)
    assert_gemm_close(bits(hidden), want_hidden)
    got_hidden = bits(hidden)
    peak = float(np.abs(O.bf16_to_f32(got_hidden)).max())
    # e4m3 output: identical to encoding the kernel's own bf16 hidden with the reciprocal scale (fusion.cu:87-92)
    scale8 = np.float32(peak / 448.0)
    out8 = torch.empty((tokens, features), device=device, dtype=torch.uint8)
    K.linear(out_format=N.OUT_FP8, out=out8, out_scale=torch.tensor(float(scale8), device=device), **common)
    want8 = O.e4m3_encode_satfinite((O.bf16_to_f32(got_hidden) * (np.float32(1.0) / scale8)).astype(np.float32))
    assert np.array_equal(u8(out8), want8)
    K.linear(out_format=N.OUT_FP8, out=out8, out_scale=torch.tensor(float(scale8), device=device), flags=N.GEGLU_TRUE_DIV, **common)
    assert np.array_equal(u8(out8), O.fp8_quantize_C(got_hidden, scale8)[0])
    # NVFP4 output: codes, row-major scales and tiled scales of the CUDA-route encoder on the same hidden
    scale4 = np.float32(peak / (448.0 * 6.0))
    out4 = torch.empty((tokens, features // 2), device=device, dtype=torch.uint8)
    linear = torch.empty((tokens, features // 16), device=device, dtype=torch.uint8)
    blocked = torch.zeros(blocked_scale_bytes(tokens, features), device=device, dtype=torch.uint8)
    K.linear(out_format=N.OUT_NVFP4, out=out4, out_scales=linear, out_blocked=blocked,
             out_scale=torch.tensor(float(scale4), device=device), **common)
    want4 = O.nvfp4_quantize_C(got_hidden, scale4)
    assert np.array_equal(u8(out4), want4[0]) and np.array_equal(u8(linear), want4[1]) and np.array_equal(u8(blocked), want4[2])


@pytest.mark.parametrize("tokens,features,width", [(513, 512, 256), (640, 384, 512), (1100, 256, 1024), (560, 16384, 2048)])
def test_gated_nvfp4_ragged_last_token_pair(device, tokens, features, width):
    """Gated NVFP4 launches whose last token pair is mostly padding (1, 128, 76 and 48 rows of its 256): every row
    against the oracle, nothing past the last row, and codes, row-major and blocked scales exactly the encodings of the
    launch's own bf16 hidden, with and without the row-major scale output."""
    host, dev = operands("nvfp4", tokens, 2 * features, width, 77 + tokens, device)
    table_host = gelu_table_cpu("tanh")
    table = torch.from_numpy(table_host.view(np.int16).copy()).view(torch.uint16).to(device)
    status = torch.zeros(1, device=device, dtype=torch.int32)
    common = dict(epilogue=N.EPI_GEGLU, tokens=tokens, features=features, width=width, gelu_table=table,
                  gelu_range=K.gelu_table_range(table), status=status, **dev)
    hidden = torch.full((tokens + 1, features), float("nan"), device=device, dtype=torch.bfloat16)
    K.linear(out_format=N.OUT_BF16, out=hidden[:tokens], **common)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert torch.isnan(hidden[tokens]).all(), "wrote past the last token row"
    got_hidden = bits(hidden[:tokens])
    if features <= 512:
        y = O.f32_to_bf16((accumulate("nvfp4", host) * float(host["a_s"]) * float(host["w_s"])).astype(np.float32))
        assert_gemm_close(got_hidden, O.gelu_mul(y[:, :features], y[:, features:], table_host))
    else:       # the benchmark's size: a launch with the pair schedule forced must agree to the same tolerance
        paired = torch.empty((tokens, features), device=device, dtype=torch.bfloat16)
        K.linear(out_format=N.OUT_BF16, out=paired, flags=N.LINEAR_PAIRS, **common)
        assert_gemm_close(got_hidden, bits(paired))
    scale4 = np.float32(float(np.abs(O.bf16_to_f32(got_hidden)).max()) / (448.0 * 6.0))
    want4 = O.nvfp4_quantize_C(got_hidden, scale4)
    for with_rows in (True, False):
        out4 = torch.full((tokens + 1, features // 2), 0xA5, device=device, dtype=torch.uint8)
        linear = torch.empty((tokens, features // 16), device=device, dtype=torch.uint8) if with_rows else None
        blocked = torch.zeros(blocked_scale_bytes(tokens, features), device=device, dtype=torch.uint8)
        K.linear(out_format=N.OUT_NVFP4, out=out4[:tokens], out_scales=linear, out_blocked=blocked,
                 out_scale=torch.tensor(float(scale4), device=device), **common)
        torch.cuda.synchronize()
        assert status.item() == 0
        assert (out4[tokens] == 0xA5).all()
        assert np.array_equal(u8(out4[:tokens]), want4[0]) and np.array_equal(u8(blocked), want4[2])
        if with_rows:
            assert np.array_equal(u8(linear), want4[1])


@pytest.mark.parametrize("kind", ("fp8", "nvfp4"))
@pytest.mark.parametrize("tokens,features,width", [(10, 4096, 1024), (37, 384, 1536), (128, 256, 4096), (3, 128, 64)])
def test_cluster_schedule_epilogues(device, kind, tokens, features, width):
    """B2_LINEAR_CLUSTER: the weights are the MMA's "A" operand and a thread-block cluster shares the K of a feature tile.
    Its partial sums meet in a fixed order, so a launch repeats its bits; against the oracle it is held to the GEMM
    tolerance, and the encoded outputs must be exactly the encodings of its own bf16 hidden.  Gated NVFP4 takes the
    paired gate / up scale layout there."""
    host, dev = operands(kind, tokens, 2 * features, width, 31 + tokens, device)
    table_host = gelu_table_cpu("tanh")
    table = torch.from_numpy(table_host.view(np.int16).copy()).view(torch.uint16).to(device)
    flags = N.LINEAR_CLUSTER
    if kind == "nvfp4":
        scales = host["w_sl"]
        blocks = scales.shape[1]
        paired = np.stack((scales[:features].reshape(features // 64, 64, blocks),
                           scales[features:].reshape(features // 64, 64, blocks)), axis=1).reshape(2 * features, blocks)
        dev = {**dev, "weight_scales": torch.from_numpy(O.swizzle_scales(paired)).to(device)}
        flags |= N.LINEAR_PAIRED_GATE_UP_SCALES
    status = torch.zeros(1, device=device, dtype=torch.int32)
    for table_range in (K.gelu_table_range(table), (0x3B4B - 1277, 0x40A2 + 3), (0, 0)):     # bulk-copied, entry by entry, none
        common = dict(epilogue=N.EPI_GEGLU, tokens=tokens, features=features, width=width, gelu_table=table, gelu_range=table_range,
                      status=status, **dev)
        hidden = torch.empty((tokens + 1, features), device=device, dtype=torch.bfloat16).fill_(float("nan"))
        K.linear(out_format=N.OUT_BF16, out=hidden[:tokens], flags=flags, **common)
        again = torch.empty((tokens, features), device=device, dtype=torch.bfloat16)
        K.linear(out_format=N.OUT_BF16, out=again, flags=flags, **common)
        torch.cuda.synchronize()
        assert status.item() == 0
        assert torch.isnan(hidden[tokens]).all(), "wrote past the last token row"
        assert np.array_equal(bits(hidden[:tokens]), bits(again))
        y = O.f32_to_bf16((accumulate(kind, host) * float(host["a_s"]) * float(host["w_s"])).astype(np.float32))
        assert_gemm_close(bits(hidden[:tokens]), O.gelu_mul(y[:, :features], y[:, features:], table_host))
    got_hidden = bits(hidden[:tokens])
    peak = float(np.abs(O.bf16_to_f32(got_hidden)).max())
    scale8 = np.float32(peak / 448.0)
    out8 = torch.empty((tokens, features), device=device, dtype=torch.uint8)
    K.linear(out_format=N.OUT_FP8, out=out8, out_scale=torch.tensor(float(scale8), device=device), flags=flags | N.GEGLU_TRUE_DIV, **common)
    assert np.array_equal(u8(out8), O.fp8_quantize_C(got_hidden, scale8)[0])
    scale4 = np.float32(peak / (448.0 * 6.0))
    out4 = torch.empty((tokens, features // 2), device=device, dtype=torch.uint8)
    linear = torch.empty((tokens, features // 16), device=device, dtype=torch.uint8)
    blocked = torch.zeros(blocked_scale_bytes(tokens, features), device=device, dtype=torch.uint8)
    K.linear(out_format=N.OUT_NVFP4, out=out4, out_scales=linear, out_blocked=blocked,
             out_scale=torch.tensor(float(scale4), device=device), flags=flags, **common)
    want4 = O.nvfp4_quantize_C(got_hidden, scale4)
    assert np.array_equal(u8(out4), want4[0]) and np.array_equal(u8(linear), want4[1]) and np.array_equal(u8(blocked), want4[2])
    assert status.item() == 0
    # plain epilogue with bias and residual, and the GELU epilogue (bias + table), on the first `features` weight rows
    bias = make_weight((1, features), 3, std=0.1).to(torch.bfloat16).reshape(-1)
    residual = make_input((tokens, features), 4, outliers=False)
    plain_dev = {**dev, "weight": dev["weight"][:features].contiguous()}
    if kind == "nvfp4":
        plain_dev["weight_scales"] = torch.from_numpy(O.swizzle_scales(host["w_sl"][:features])).to(device)
    y = y[:, :features]
    with_bias = O.f32_to_bf16(O.bf16_to_f32(y) + O.bf16_to_f32(bits(bias))[None, :])
    out = torch.empty((tokens, features), device=device, dtype=torch.bfloat16)
    shape = dict(tokens=tokens, features=features, width=width, status=status)
    K.linear(epilogue=N.EPI_LINEAR, out_format=N.OUT_BF16, out=out, bias=bias.to(device), residual=residual.to(device),
             flags=N.LINEAR_CLUSTER, **shape, **plain_dev)
    assert_gemm_close(bits(out), O.f32_to_bf16(O.bf16_to_f32(with_bias) + O.bf16_to_f32(bits(residual))))
    K.linear(epilogue=N.EPI_GELU, out_format=N.OUT_BF16, out=out, bias=bias.to(device), gelu_table=table,
             gelu_range=K.gelu_table_range(table), flags=N.LINEAR_CLUSTER, **shape, **plain_dev)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert_gemm_close(bits(out), table_host[with_bias])


@pytest.mark.parametrize("kind", ("fp8", "nvfp4"))
def test_gated_zero_gate_reads_the_full_table(device, kind):
    """A gate of exactly zero lies below every compact range and, with no range at all, must still come
    from the table: zero activations give gelu(0) * 0 = 0 everywhere."""
    tokens, features, width = 200, 256, 512
    host, dev = operands(kind, tokens, 2 * features, width, 5, device)
    dev["act"] = torch.zeros_like(dev["act"])
    table = torch.from_numpy(gelu_table_cpu("tanh").view(np.int16).copy()).view(torch.uint16).to(device)
    # dirty the shared memory of every SM first: 200 KB of non-zero bytes per CTA
    K.linear(epilogue=N.EPI_LINEAR, out_format=N.OUT_BF16, tokens=tokens, features=2 * features, width=width,
             out=torch.empty((tokens, 2 * features), device=device, dtype=torch.bfloat16), **operands(kind, tokens, 2 * features, width, 6, device)[1])
    for table_range in ((0, 0), K.gelu_table_range(table)):
        hidden = torch.full((tokens, features), 7.0, device=device, dtype=torch.bfloat16)
        K.linear(epilogue=N.EPI_GEGLU, out_format=N.OUT_BF16, tokens=tokens, features=features, width=width, out=hidden,
                 gelu_table=table, gelu_range=table_range, **dev)
        assert not (bits(hidden) & 0x7fff).any()


@pytest.mark.parametrize("kind", ("fp8", "nvfp4"))
@pytest.mark.parametrize("epilogue,tokens,features,width", [("linear", 560, 8192, 1024), ("linear", 300, 12288, 768), ("geglu", 300, 8192, 512)])
def test_token_resident_order_matches_streaming_and_oracle(device, kind, epilogue, tokens, features, width):
    """Enough feature tiles per CTA for the kernel to keep its token tile on chip (the default there);
    B2_LINEAR_STREAM_TOKENS forces the streaming order: both must give the same bits, and match the oracle."""
    gated = epilogue == "geglu"
    host, dev = operands(kind, tokens, (2 if gated else 1) * features, width, 77 + tokens, device)
    outputs = []
    for flags in (0, N.LINEAR_STREAM_TOKENS):
        out = torch.empty((tokens, features), device=device, dtype=torch.bfloat16)
        status = torch.zeros(1, device=device, dtype=torch.int32)
        if gated:
            table_host = gelu_table_cpu("tanh")
            table = torch.from_numpy(table_host.view(np.int16).copy()).view(torch.uint16).to(device)
            K.linear(epilogue=N.EPI_GEGLU, out_format=N.OUT_BF16, tokens=tokens, features=features, width=width, out=out,
                     gelu_table=table, gelu_range=K.gelu_table_range(table), flags=flags, status=status, **dev)
        else:
            K.linear(epilogue=N.EPI_LINEAR, out_format=N.OUT_BF16, tokens=tokens, features=features, width=width, out=out,
                     flags=flags, status=status, **dev)
        assert int(status.item()) == 0
        outputs.append(bits(out))
    assert np.array_equal(outputs[0], outputs[1])
    y = O.f32_to_bf16((accumulate(kind, host) * float(host["a_s"]) * float(host["w_s"])).astype(np.float32))
    want = O.gelu_mul(y[:, :features], y[:, features:], gelu_table_cpu("tanh")) if gated else y
    assert_gemm_close(outputs[0], want)


@pytest.mark.parametrize("kind", ("fp8", "nvfp4"))
@pytest.mark.parametrize("epilogue,tokens,features,width", [("linear", 10, 1024, 4096), ("linear", 80, 1024, 2048), ("linear", 10, 2560, 1024),
                                                            ("linear", 560, 2048, 16384), ("linear", 10, 128, 32768), ("linear", 80, 256, 16384),
                                                            ("geglu", 10, 4096, 1024)])
def test_split_k_is_deterministic_and_matches_oracle(device, kind, epilogue, tokens, features, width):
    """Few tiles and a long K: K is cut across CTAs when a workspace is given and the library's estimate says it
    pays (the two long-K cases; the others run unsplit).  Same bits on every run (the partial sums are added in
    split order), tickets back at zero, within tolerance of the oracle like the unsplit launch."""
    gated = epilogue == "geglu"
    host, dev = operands(kind, tokens, (2 if gated else 1) * features, width, 11 + tokens, device)
    table_host = gelu_table_cpu("tanh")
    table = torch.from_numpy(table_host.view(np.int16).copy()).view(torch.uint16).to(device)
    workspace = torch.zeros(32 << 20, device=device, dtype=torch.uint8)
    outputs = []
    for ws in (workspace, workspace, False):
        out = torch.empty((tokens, features), device=device, dtype=torch.bfloat16)
        status = torch.zeros(1, device=device, dtype=torch.int32)
        extra = dict(epilogue=N.EPI_GEGLU, gelu_table=table, gelu_range=K.gelu_table_range(table)) if gated else dict(epilogue=N.EPI_LINEAR)
        K.linear(out_format=N.OUT_BF16, tokens=tokens, features=features, width=width, out=out, status=status, workspace=ws, **extra, **dev)
        assert int(status.item()) == 0
        outputs.append(bits(out))
    assert np.array_equal(outputs[0], outputs[1])
    assert not workspace[:1024].any()                       # ticket words
    plan = N.LinearDesc(kind=dev["kind"], epilogue=N.EPI_GEGLU if gated else N.EPI_LINEAR, out_format=N.OUT_BF16, tokens=tokens,
                        features=features, width=width)
    planned = N.load().b2_linear_workspace_bytes(ctypes.byref(plan))
    assert bool(workspace.any()) == (planned > 0)           # partial sums were written exactly when the library plans a split
    y = O.f32_to_bf16((accumulate(kind, host) * float(host["a_s"]) * float(host["w_s"])).astype(np.float32))
    want = O.gelu_mul(y[:, :features], y[:, features:], table_host) if gated else y
    assert_gemm_close(outputs[0], want)
    assert_gemm_close(outputs[2], want)


def run_linear(device, dev, *, tokens, features, width, flags=0, tile=0, **extra):
    """One plain launch with a guard row behind the output and the status word checked."""
    out = torch.full((tokens + 1, features), float("nan"), device=device, dtype=torch.bfloat16)
    status = torch.zeros(1, device=device, dtype=torch.int32)
    K.linear(epilogue=N.EPI_LINEAR, out_format=N.OUT_BF16, tokens=tokens, features=features, width=width, out=out[:tokens],
             status=status, flags=flags, feature_tile=tile, **extra, **dev)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.isnan(out[tokens]).all(), "wrote past the last token row"
    return out[:tokens]


@pytest.mark.parametrize("kind", ("fp8", "nvfp4"))
@pytest.mark.parametrize("tokens,features,width,tile", [(129, 256, 256, 0), (256, 512, 1024, 256), (257, 384, 512, 128), (560, 2048, 2048, 0),
                                                         (560, 2048, 2048, 256), (700, 1152, 1152, 128), (1024, 4096, 512, 0), (300, 200, 320, 0)])
def test_paired_schedule_equals_single_cta(device, kind, tokens, features, width, tile):
    """More than 128 tokens: pairs of SMs compute 256-token tiles (`tcgen05.mma.cta_group::2`), each CTA loading its
    own token rows and half of the weight tile.  B2_LINEAR_SINGLE_CTA keeps one CTA per 128-token tile.  The two
    schedules accumulate along K in the same order: identical bits, with bias and residual, and within the GEMM
    tolerance of the oracle."""
    host, dev = operands(kind, tokens, features, width, 3 + tokens + features, device)
    bias = make_weight((1, features), 91, std=0.5).reshape(-1).to(torch.bfloat16).to(device)
    residual = make_input((tokens, features), 92, outliers=False).to(device)
    common = dict(tokens=tokens, features=features, width=width, tile=tile)
    paired = run_linear(device, dev, flags=N.LINEAR_PAIRS, **common)
    single = run_linear(device, dev, flags=N.LINEAR_SINGLE_CTA, **common)
    assert torch.equal(paired.view(torch.int16), single.view(torch.int16))
    want = O.f32_to_bf16((accumulate(kind, host) * float(host["a_s"]) * float(host["w_s"])).astype(np.float32))
    assert_gemm_close(bits(paired), want)
    full = run_linear(device, dev, flags=N.LINEAR_PAIRS, bias=bias, residual=residual, **common)
    assert torch.equal(full, (paired + bias) + residual)


@pytest.mark.parametrize("kind", ("fp8", "nvfp4"))
@pytest.mark.parametrize("out_format", ("bf16", "fp8", "nvfp4"))
def test_paired_schedule_gated_equals_single_cta(device, kind, out_format):
    """The gated epilogue on pairs: the leader CTA loads the gate rows of a tile, its peer the up rows; every encoded
    output (codes, row-major and tiled block scales) equals the single-CTA schedule's bit for bit."""
    tokens, features, width = 330, 512, 1024
    host, dev = operands(kind, tokens, 2 * features, width, 17, device)
    table = torch.from_numpy(gelu_table_cpu("tanh").view(np.int16).copy()).view(torch.uint16).to(device)
    common = dict(epilogue=N.EPI_GEGLU, tokens=tokens, features=features, width=width, gelu_table=table,
                  gelu_range=K.gelu_table_range(table), **dev)
    results = []
    for flags in (N.LINEAR_PAIRS, N.LINEAR_SINGLE_CTA):
        status = torch.zeros(1, device=device, dtype=torch.int32)
        if out_format == "bf16":
            out = torch.empty((tokens, features), device=device, dtype=torch.bfloat16)
            K.linear(out_format=N.OUT_BF16, out=out, flags=flags, status=status, **common)
            results.append((bits(out),))
        elif out_format == "fp8":
            out = torch.empty((tokens, features), device=device, dtype=torch.uint8)
            K.linear(out_format=N.OUT_FP8, out=out, out_scale=torch.tensor(0.01, device=device), flags=flags, status=status, **common)
            results.append((u8(out),))
        else:
            out = torch.empty((tokens, features // 2), device=device, dtype=torch.uint8)
            linear = torch.empty((tokens, features // 16), device=device, dtype=torch.uint8)
            blocked = torch.zeros(blocked_scale_bytes(tokens, features), device=device, dtype=torch.uint8)
            K.linear(out_format=N.OUT_NVFP4, out=out, out_scales=linear, out_blocked=blocked,
                     out_scale=torch.tensor(0.002, device=device), flags=flags, status=status, **common)
            results.append((u8(out), u8(linear), u8(blocked)))
        assert int(status.item()) == 0
    for got, want in zip(*results):
        assert np.array_equal(got, want)


@pytest.mark.parametrize("kind,width", [("fp8", 1024), ("nvfp4", 2048), ("nvfp4", 320)])
def test_resident_pair_order_equals_single_cta(device, kind, width):
    """Short K and at least two tiles per SM pair: each pair keeps its 256 token rows (and their scales) on chip for
    all of K and streams weights only.  Same accumulation order as the other schedules: identical bits, also with the
    streaming order forced, with the ragged third token pair of 560 rows and a ragged last feature tile."""
    tokens, features = 560, 12800 - 64
    host, dev = operands(kind, tokens, features, width, 7 + width, device)
    common = dict(tokens=tokens, features=features, width=width)
    resident = run_linear(device, dev, **common)
    single = run_linear(device, dev, flags=N.LINEAR_SINGLE_CTA, **common)
    streaming = run_linear(device, dev, flags=N.LINEAR_PAIRS | N.LINEAR_STREAM_TOKENS, **common)
    assert torch.equal(resident.view(torch.int16), single.view(torch.int16))
    assert torch.equal(streaming.view(torch.int16), single.view(torch.int16))
    rows = slice(500, 560)
    want = O.f32_to_bf16((accumulate(kind, {**host, "a": host["a"][rows], **({"a_sl": host["a_sl"][rows]} if kind == "nvfp4" else {})})
                          * float(host["a_s"]) * float(host["w_s"])).astype(np.float32))
    assert_gemm_close(bits(resident[rows]), want)


@pytest.mark.parametrize("layout", ("paired", "bundle", "fp8"))
@pytest.mark.parametrize("out_format", ("bf16", "nvfp4"))
def test_resident_pair_order_gated(device, layout, out_format):
    """The gated epilogue in the resident order: 64 + 64-feature tiles with the paired gate/up scale layout (two
    accumulators in tensor memory), 128 + 128-feature tiles with the bundle's layout, and FP8; every output equals the
    single-CTA schedule's bit for bit."""
    kind = "fp8" if layout == "fp8" else "nvfp4"
    tokens, features, width = 330, 4864 if layout == "paired" else 9600, 1024 if kind == "fp8" else 2048
    host, dev = operands(kind, tokens, 2 * features, width, 23, device)
    flags = 0
    if layout == "paired":
        scales = host["w_sl"]
        blocks = scales.shape[1]
        paired = np.stack((scales[:features].reshape(features // 64, 64, blocks),
                           scales[features:].reshape(features // 64, 64, blocks)), axis=1).reshape(2 * features, blocks)
        dev = {**dev, "weight_scales": torch.from_numpy(O.swizzle_scales(paired)).to(device)}
        flags = N.LINEAR_PAIRED_GATE_UP_SCALES
    table = torch.from_numpy(gelu_table_cpu("tanh").view(np.int16).copy()).view(torch.uint16).to(device)
    common = dict(epilogue=N.EPI_GEGLU, tokens=tokens, features=features, width=width, gelu_table=table,
                  gelu_range=K.gelu_table_range(table), **dev)
    results = []
    for extra in (0, N.LINEAR_SINGLE_CTA):
        status = torch.zeros(1, device=device, dtype=torch.int32)
        if out_format == "bf16":
            out = torch.full((tokens + 1, features), float("nan"), device=device, dtype=torch.bfloat16)
            K.linear(out_format=N.OUT_BF16, out=out[:tokens], flags=flags | extra, status=status, **common)
            assert torch.isnan(out[tokens]).all()
            results.append((bits(out[:tokens]),))
        else:
            out = torch.empty((tokens, features // 2), device=device, dtype=torch.uint8)
            linear = torch.empty((tokens, features // 16), device=device, dtype=torch.uint8)
            blocked = torch.zeros(blocked_scale_bytes(tokens, features), device=device, dtype=torch.uint8)
            K.linear(out_format=N.OUT_NVFP4, out=out, out_scales=linear, out_blocked=blocked,
                     out_scale=torch.tensor(0.002, device=device), flags=flags | extra, status=status, **common)
            results.append((u8(out), u8(linear), u8(blocked)))
        torch.cuda.synchronize()
        assert int(status.item()) == 0
    for got, want in zip(*results):
        assert np.array_equal(got, want)


TAIL_TOKENS = list(range(1, 18)) + [127, 128, 129, 255, 256, 257, 559, 560, 561]


@pytest.mark.parametrize("kind", ("fp8", "nvfp4"))
def test_token_tail_sweep(device, kind):
    """Every token count around the tile boundaries (1..17, 127..129, 255..257, 559..561) at one small shape: each
    launch is the oracle's result on its own rows and writes nothing behind its last row."""
    features, width = 192, 256
    host, dev = operands(kind, max(TAIL_TOKENS), features, width, 41, device)
    want = O.f32_to_bf16((accumulate(kind, host) * float(host["a_s"]) * float(host["w_s"])).astype(np.float32))
    for tokens in TAIL_TOKENS:
        sliced = dict(dev)
        sliced["act"] = dev["act"][:tokens].contiguous()
        out = run_linear(device, sliced, tokens=tokens, features=features, width=width)
        assert_gemm_close(bits(out), want[:tokens])
        if tokens > 128:        # and on pairs of SMs, whatever the padding
            paired = run_linear(device, sliced, tokens=tokens, features=features, width=width, flags=N.LINEAR_PAIRS)
            assert torch.equal(paired.view(torch.int16), out.view(torch.int16))


def test_config1_full_size(device):
    """Benchmark configuration 1 at full size: FP8 W8A8 560 x 16384 x 2048, every output element against the oracle;
    then with a bias."""
    tokens, features, width = 560, 16384, 2048
    host, dev = operands("fp8", tokens, features, width, 1001, device)
    out = run_linear(device, dev, tokens=tokens, features=features, width=width)
    assert_gemm_close(bits(out), O.fp8_linear(host["a"], host["a_s"], host["w"], host["w_s"]))
    paired = run_linear(device, dev, tokens=tokens, features=features, width=width, flags=N.LINEAR_PAIRS)
    assert torch.equal(paired.view(torch.int16), out.view(torch.int16))
    # the bias is a separate bf16 addition on that result (fp8.py:139-140)
    bias = make_weight((1, features), 1001, std=0.1).to(torch.bfloat16).reshape(-1).to(device)
    assert torch.equal(run_linear(device, dev, tokens=tokens, features=features, width=width, bias=bias), out + bias)


def test_config2_full_size(device):
    """Benchmark configuration 2 at full size, all 560 rows: the gated launch's bf16 hidden activation against the
    oracle, its NVFP4 re-encoding bit for bit against the CUDA-route encoder on that hidden activation, and the down
    projection of the re-encoded activation against the oracle."""
    tokens, hidden_width, inter = 560, 2048, 16384
    host, dev = operands("nvfp4", tokens, 2 * inter, hidden_width, 1002, device)
    table_host = gelu_table_cpu("tanh")
    table = torch.from_numpy(table_host.view(np.int16).copy()).view(torch.uint16).to(device)
    common = dict(epilogue=N.EPI_GEGLU, tokens=tokens, features=inter, width=hidden_width, gelu_table=table,
                  gelu_range=K.gelu_table_range(table), **dev)
    hidden = torch.empty((tokens, inter), device=device, dtype=torch.bfloat16)
    K.linear(out_format=N.OUT_BF16, out=hidden, **common)
    y = O.f32_to_bf16((accumulate("nvfp4", host) * float(host["a_s"]) * float(host["w_s"])).astype(np.float32))
    assert_gated_close(bits(hidden), y[:, :inter], y[:, inter:], table_host)
    got_hidden = bits(hidden)
    scale4 = np.float32(float(np.abs(O.bf16_to_f32(got_hidden)).max()) / (448.0 * 6.0))
    out4 = torch.empty((tokens, inter // 2), device=device, dtype=torch.uint8)
    linear = torch.empty((tokens, inter // 16), device=device, dtype=torch.uint8)
    blocked = torch.zeros(blocked_scale_bytes(tokens, inter), device=device, dtype=torch.uint8)
    K.linear(out_format=N.OUT_NVFP4, out=out4, out_scales=linear, out_blocked=blocked,
             out_scale=torch.tensor(float(scale4), device=device), **common)
    want4 = O.nvfp4_quantize_C(got_hidden, scale4)
    assert np.array_equal(u8(out4), want4[0]) and np.array_equal(u8(linear), want4[1]) and np.array_equal(u8(blocked), want4[2])
    # down projection of the re-encoded activation (K = 16384)
    w = bits(make_weight((hidden_width, inter), 1003).to(torch.bfloat16))
    wp, wsl, wbl, w_s = O.nvfp4_quantize_C(w)
    down = dict(kind=N.KIND_NVFP4, act=out4, act_scales=blocked, act_scale=torch.tensor(float(scale4), device=device),
                weight=torch.from_numpy(wp).to(device), weight_scales=torch.from_numpy(wbl).to(device),
                weight_scale=torch.tensor(float(w_s), device=device))
    out = run_linear(device, down, tokens=tokens, features=hidden_width, width=inter)
    assert_gemm_close(bits(out), O.nvfp4_linear_plan(want4[0], want4[1], scale4, wp, wsl, w_s))


@pytest.mark.parametrize("kind,tokens,features,width", [("fp8", 256, 4304, 1152), ("fp8", 130, 384, 1024), ("nvfp4", 130, 384, 1024)])
def test_bias_gelu_epilogue(device, kind, tokens, features, width):
    """out = gelu(x W^T + bias): bf16 against the oracle; e4m3 output identical to encoding the kernel's own
    bf16 result (reciprocal multiply, and true division with B2_GEGLU_TRUE_DIV), with and without a table range."""
    host, dev = operands(kind, tokens, features, width, 31 + features, device)
    bias = make_weight((1, features), 9, std=0.5).to(torch.bfloat16).reshape(-1)
    table_host = gelu_table_cpu("tanh")
    table = torch.from_numpy(table_host.view(np.int16).copy()).view(torch.uint16).to(device)
    common = dict(epilogue=N.EPI_GELU, tokens=tokens, features=features, width=width, bias=bias.to(device), gelu_table=table, **dev)
    hidden = torch.empty((tokens, features), device=device, dtype=torch.bfloat16)
    K.linear(out_format=N.OUT_BF16, out=hidden, **common)
    y = O.f32_to_bf16((accumulate(kind, host) * float(host["a_s"]) * float(host["w_s"])).astype(np.float32))
    y = O.f32_to_bf16(O.bf16_to_f32(y) + O.bf16_to_f32(bits(bias))[None, :])
    assert_gemm_close(bits(hidden), table_host[y])
    got = bits(hidden)
    ranged = torch.empty_like(hidden)
    K.linear(out_format=N.OUT_BF16, out=ranged, gelu_range=K.gelu_table_range(table), **common)
    assert np.array_equal(bits(ranged), got)
    scale = np.float32(float(np.abs(O.bf16_to_f32(got)).max()) / 448.0)
    out8 = torch.empty((tokens, features), device=device, dtype=torch.uint8)
    K.linear(out_format=N.OUT_FP8, out=out8, out_scale=torch.tensor(float(scale), device=device), **common)
    assert np.array_equal(u8(out8), O.e4m3_encode_satfinite((O.bf16_to_f32(got) * (np.float32(1.0) / scale)).astype(np.float32)))
    K.linear(out_format=N.OUT_FP8, out=out8, out_scale=torch.tensor(float(scale), device=device), flags=N.GEGLU_TRUE_DIV,
             gelu_range=K.gelu_table_range(table), **common)
    assert np.array_equal(u8(out8), O.fp8_quantize_C(got, scale)[0])


def test_gated_with_separate_up_scale(device):
    """gate and up quantised separately (two per-tensor scales) give the same result as two Linears."""
    tokens, features, width = 96, 128, 256
    x = bits(make_input((tokens, width), 1))
    wg = bits(make_weight((features, width), 2).to(torch.bfloat16))
    wu = bits(make_weight((features, width), 3, std=0.05).to(torch.bfloat16))
    aq, a_s = O.fp8_quantize_C(x)
    gq, g_s = O.fp8_quantize_C(wg)
    uq, u_s = O.fp8_quantize_C(wu)
    table_host = gelu_table_cpu("tanh")
    table = torch.from_numpy(table_host.view(np.int16).copy()).view(torch.uint16).to(device)
    hidden = torch.empty((tokens, features), device=device, dtype=torch.bfloat16)
    scalar = lambda v: torch.tensor(float(v), device=device)
    K.linear(kind=N.KIND_FP8, epilogue=N.EPI_GEGLU, out_format=N.OUT_BF16, tokens=tokens, features=features, width=width,
             act=torch.from_numpy(aq).to(device), act_scale=scalar(a_s), weight=torch.from_numpy(np.concatenate([gq, uq])).to(device),
             weight_scale=scalar(g_s), weight_scale_up=scalar(u_s), gelu_table=table, out=hidden)
    want = O.gelu_mul(O.fp8_linear(aq, a_s, gq, g_s), O.fp8_linear(aq, a_s, uq, u_s), table_host)
    assert_gemm_close(bits(hidden), want)


def test_full_size_properties(device):
    """Config-2 sizes: zero activations give zero; doubling the activation scale doubles the output."""
    tokens, features, width = 560, 16384, 2048
    host, dev = operands("nvfp4", tokens, features, width, 1002, device)
    out = torch.empty((tokens, features), device=device, dtype=torch.bfloat16)
    common = dict(epilogue=N.EPI_LINEAR, out_format=N.OUT_BF16, tokens=tokens, features=features, width=width)
    K.linear(out=out, **common, **dev)
    doubled = torch.empty_like(out)
    K.linear(out=doubled, **common, **{**dev, "act_scale": dev["act_scale"] * 2})
    assert torch.equal(out.float() * 2, doubled.float())
    zero = {**dev, "act": torch.zeros_like(dev["act"])}
    K.linear(out=doubled, **common, **zero)
    assert not doubled.any()
    rows = slice(300, 316)
    want = O.nvfp4_linear_plan(host["a"][rows], host["a_sl"][rows], host["a_s"], host["w"], host["w_sl"], host["w_s"])
    assert_gemm_close(bits(out[rows]), want)


def test_rejections(device):
    x = torch.zeros((8, 64), device=device, dtype=torch.uint8)
    with pytest.raises(RuntimeError, match="error -1"):     # a flag bit the library does not know
        K.linear(kind=N.KIND_FP8, epilogue=N.EPI_LINEAR, out_format=N.OUT_BF16, tokens=8, features=16, width=64, act=x,
                 act_scale=torch.ones((), device=device), weight=torch.zeros((16, 64), device=device, dtype=torch.uint8),
                 weight_scale=torch.ones((), device=device), out=torch.zeros((8, 16), device=device, dtype=torch.bfloat16), flags=0x1000)
    w = torch.zeros((16, 64), device=device, dtype=torch.uint8)
    one = torch.ones((), device=device)
    out = torch.zeros((8, 16), device=device, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="error -2"):
        K.linear(kind=N.KIND_FP8, epilogue=N.EPI_LINEAR, out_format=N.OUT_FP8, tokens=8, features=16, width=64, act=x,
                 act_scale=one, weight=w, weight_scale=one, out=out)
    with pytest.raises(RuntimeError, match="error -2"):
        K.linear(kind=N.KIND_FP8, epilogue=N.EPI_LINEAR, out_format=N.OUT_BF16, tokens=8, features=16, width=64, act=x,
                 act_scale=one, weight=w, weight_scale=one, out=out, feature_tile=48)
    with pytest.raises(RuntimeError, match="error -1"):
        K.linear(kind=N.KIND_NVFP4, epilogue=N.EPI_LINEAR, out_format=N.OUT_BF16, tokens=8, features=16, width=128, act=x,
                 act_scale=one, weight=w, weight_scale=one, out=out)      # NVFP4 without block scales
    with pytest.raises(ValueError, match="no CPU fallback"):
        K.linear(kind=N.KIND_FP8, epilogue=N.EPI_LINEAR, out_format=N.OUT_BF16, tokens=8, features=16, width=64, act=x.cpu(),
                 act_scale=one, weight=w, weight_scale=one, out=out)


@pytest.mark.parametrize("std", (1e-7, 0.02, 0.5, 20.0))
def test_compact_gelu_table_matches_full_table(device, std):
    """Keeping only the non-trivial part of the GELU table in shared memory (b2_gelu_table_range)
    gives the same bits as gathering from the full table, for tiny, ordinary and huge gate values."""
    tokens, features, width = 200, 256, 512
    x = bits(make_input((tokens, width), 3))
    w = bits(make_weight((2 * features, width), 4, std=std).to(torch.bfloat16))
    aq, a_s = O.fp8_quantize_C(x)
    wq, w_s = O.fp8_quantize_C(w)
    table_host = gelu_table_cpu("tanh")
    table = torch.from_numpy(table_host.view(np.int16).copy()).view(torch.uint16).to(device)
    table_range = K.gelu_table_range(table)
    # the closed forms hold outside [0x3B4B, 0x40A2); lo comes back ten binades lower, hi four binades higher, both on a
    # multiple of eight codes
    assert table_range == ((0x3B4B - 1280) & ~7, (0x40A2 + 512 + 7) & ~7)
    scalar = lambda v: torch.tensor(float(v), device=device)
    common = dict(kind=N.KIND_FP8, epilogue=N.EPI_GEGLU, out_format=N.OUT_BF16, tokens=tokens, features=features, width=width,
                  act=torch.from_numpy(aq).to(device), act_scale=scalar(a_s), weight=torch.from_numpy(wq).to(device),
                  weight_scale=scalar(w_s), gelu_table=table)
    full = torch.empty((tokens, features), device=device, dtype=torch.bfloat16)
    compact = torch.empty_like(full)
    K.linear(out=full, **common)
    K.linear(out=compact, gelu_range=table_range, **common)
    assert torch.equal(full.view(torch.int16), compact.view(torch.int16))
    gate = O.bf16_to_f32(O.fp8_linear(aq, a_s, wq[:features], w_s))
    magnitudes = (O.f32_to_bf16(gate) & 0x7FFF)
    if std == 1e-7:
        assert (magnitudes < 0x3B4B - 1280).mean() > 0.3       # the x/2 tail is exercised
    if std == 0.5:
        assert (magnitudes >= 0x40A2).mean() > 0.2      # the identity / -0 values inside the widened range
    if std == 20.0:
        assert (magnitudes >= 0x40A2 + 512).mean() > 0.2      # the identity / -0 tail beyond it


def test_gelu_table_range_rejects_unstructured_tables(device):
    generator = torch.Generator().manual_seed(0)
    noise = torch.randint(0, 65535, (65536,), generator=generator, dtype=torch.int32).to(torch.uint16)
    assert K.gelu_table_range(noise) == (0, 0)


def test_paired_gate_up_scale_layout(device):
    """B2_LINEAR_PAIRED_GATE_UP_SCALES: same bits as the bundle-order scale layout, fewer tensor-core operations."""
    tokens, features, width = 200, 256, 512
    host, dev = operands("nvfp4", tokens, 2 * features, width, 77, device)
    scales = host["w_sl"]                                    # row-major [2F, K/16]: gate rows, then up rows
    blocks = scales.shape[1]
    paired = np.stack((scales[:features].reshape(features // 64, 64, blocks),
                       scales[features:].reshape(features // 64, 64, blocks)), axis=1).reshape(2 * features, blocks)
    table_host = gelu_table_cpu("tanh")
    table = torch.from_numpy(table_host.view(np.int16).copy()).view(torch.uint16).to(device)
    common = dict(epilogue=N.EPI_GEGLU, out_format=N.OUT_BF16, tokens=tokens, features=features, width=width, gelu_table=table)
    plain = torch.empty((tokens, features), device=device, dtype=torch.bfloat16)
    K.linear(out=plain, feature_tile=64, **common, **dev)
    fast = torch.empty_like(plain)
    paired_dev = {**dev, "weight_scales": torch.from_numpy(O.swizzle_scales(paired)).to(device)}
    K.linear(out=fast, flags=N.LINEAR_PAIRED_GATE_UP_SCALES, **common, **paired_dev)
    assert torch.equal(plain.view(torch.int16), fast.view(torch.int16))
    with pytest.raises(RuntimeError, match="error -2"):
        K.linear(out=fast, flags=N.LINEAR_PAIRED_GATE_UP_SCALES, feature_tile=128, **common, **paired_dev)
    fp8_host, fp8_dev = operands("fp8", tokens, 2 * features, width, 77, device)
    with pytest.raises(RuntimeError, match="error -1"):
        K.linear(out=fast, flags=N.LINEAR_PAIRED_GATE_UP_SCALES, **common, **fp8_dev)
