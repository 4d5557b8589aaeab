"""The pi0.5-shaped random-init stack on the GPU: every quantised projection at its real width, towers
shortened to one layer.  Checker: the same stack with the registry kernels swapped for a composed
"dequantised" route (the reference's torch-route expressions evaluated by torch on the device, fp32 GEMM),
i.e. the W8A8 oracle composition applied layer by layer."""

from __future__ import annotations

import pytest
import torch

from embodiinfer_b200.layers import linear as registry
from embodiinfer_b200.pi05_shaped import ACTION_DIM, ACTION_HORIZON, Pi05ShapedPolicy, synthetic_observations
from embodiinfer_b200.rollout import DataParallelRollout

pytestmark = pytest.mark.gpu


def composed_fp8_linear(inputs, weight, weight_scale, bias=None):
    """fp8.py:66-73 + 118-141 with torch ops: quantise, dequantise both operands, fp32 matmul, bf16, + bias."""
    rows = inputs.reshape(-1, inputs.shape[-1])
    peak = rows.float().abs().amax()
    scale = torch.where(peak > 0, peak / 448.0, torch.ones_like(peak))
    codes = (rows / scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    product = (codes.float() @ weight.float().t()) * (scale * weight_scale)
    output = product.to(torch.bfloat16)
    if bias is not None:
        output = output + bias
    return output.reshape(*inputs.shape[:-1], weight.shape[0])


def test_one_layer_policy_matches_composed_route(device, monkeypatch):
    policy = Pi05ShapedPolicy("fp8", device=device, layer_scale=0.01, vocabulary=4096)
    assert len(policy.vision) == len(policy.prefix) == len(policy.expert) == 1
    observations = synthetic_observations(3, vocabulary=4096)
    actions = policy(observations)
    assert actions.shape == (3, ACTION_HORIZON, ACTION_DIM) and actions.dtype == torch.float32
    assert torch.isfinite(actions).all()
    assert torch.equal(actions, policy(observations)), "the rollout step must be deterministic"
    native = registry._resolve("fp8_native")
    monkeypatch.setitem(registry._REGISTRY, "fp8_native", (composed_fp8_linear, native[1]))
    expected = policy(observations)
    monkeypatch.setitem(registry._REGISTRY, "fp8_native", native)
    # Ten Euler steps through requantising layers amplify single-ulp differences of the bf16 GEMM outputs;
    # the per-Linear tolerance (1e-3) is checked in test_gpu_linear / test_gpu_plans.
    error = (actions - expected).norm() / expected.norm()
    assert error < 2e-2, float(error)
    result = DataParallelRollout(policy, device=device).run(observations)
    assert torch.equal(result.actions, actions) and result.owner_rank == [0, 0, 0]
    assert policy.flops_per_observation() > 1e11


@pytest.mark.parametrize("quantization", ("fp8", "nvfp4"))
def test_calibrated_fused_mlp_route_stays_close_to_the_registry_route(device, quantization):
    """After calibration on the same observations the Gemma MLPs run as encode + fused gate_up/GELU/re-encode
    + down(+residual).  Static scales and the CUDA-route weight encoder change roundings, not the result:
    the action chunks stay within a few percent of the registry route's, and the step is deterministic."""
    policy = Pi05ShapedPolicy(quantization, device=device, layer_scale=0.01, vocabulary=4096)
    observations = synthetic_observations(3, vocabulary=4096)
    reference = policy(observations)
    policy.calibrate_fused_mlp(observations)
    assert all(block.fused_mlp is not None for block in [*policy.vision, *policy.prefix, *policy.expert])
    fused = policy(observations)
    assert torch.isfinite(fused).all() and torch.equal(fused, policy(observations))
    error = (fused - reference).norm() / reference.norm()
    assert error < 0.1, float(error)
    gemma = [*policy.prefix, *policy.expert]
    # the attention kernel writes the output projection's encoded rows (e4m3 or NVFP4): the same bits as attention and
    # encoder in two launches
    for block in gemma:
        block.encode_in_attention = False
    assert torch.equal(policy(observations), fused)
    for block in gemma:
        block.encode_in_attention = True
    # the norm + encoder launch in front of the calibrated plans against torch's rms_norm + the separate encoder
    assert all(block.mlp_norm is not None and block.qkv.norm is not None for block in gemma)
    assert all(block.mlp_norm is not None and block.qkv.layer_norm is not None for block in policy.vision)
    for block in [*gemma, *policy.vision]:
        block.fused_norm = False
    separate = policy(observations)
    error = (fused - separate).norm() / separate.norm()
    assert error < 0.05, float(error)


def test_graph_replay_of_the_policy_step_equals_eager(device):
    from embodiinfer_b200.rollout_bench import GraphedReplica
    policy = Pi05ShapedPolicy("fp8", device=device, layer_scale=0.01, vocabulary=4096)
    observations = {key: value.pin_memory() for key, value in synthetic_observations(4, vocabulary=4096).items()}
    policy.calibrate_fused_mlp(observations)
    eager = policy(observations)
    graphed = GraphedReplica(policy, observations, 4)
    assert torch.equal(graphed(observations), eager)
    half = {key: value[:2] for key, value in observations.items()}
    assert torch.equal(graphed(half), eager[:2])


def _linear_records(block):
    """Forward hooks on every quantised Linear bundle of one block: (name, input, output) of the real forward pass."""
    records, handles = [], []
    bundles = {"qkv": block.qkv.bundle, "o_proj": block.o_proj.bundle, "gate_up": block.gate_up, "down": block.down}
    for name, module in bundles.items():
        handles.append(module.register_forward_hook(
            lambda mod, args, output, name=name: records.append((name, mod, args[0].detach().clone(), output.detach().clone()))))
    return records, handles


@pytest.mark.parametrize("quantization", ("fp8", "nvfp4"))
@pytest.mark.parametrize("tower,batch,tokens", [("prefix", 1, 560), ("expert", 8, 10)])
def test_full_width_layer_linears_match_the_oracle(device, quantization, tower, batch, tokens):
    """One layer at its real width (Gemma-2B-shaped prefix layer over 560 tokens; Gemma-300M-shaped expert layer over
    a 10-token chunk at B = 8): every quantised Linear of the forward pass -- packed QKV, output projection, packed
    gate/up, down -- is compared with the CPU oracle of the registry route ON THE ACTIVATIONS THE LAYER ACTUALLY
    PRODUCED, whole output, relative Frobenius <= 1e-3 and the per-element bound of the GEMM tests.  Same idea as
    the reference's operator-equality test (tests/pi05/test_graphs.py:238-313), with the oracle as the other side."""
    import numpy as np

    from embodiinfer_b200 import layers as L
    from embodiinfer_b200.pi05_shaped import GEMMA_2B, GEMMA_300M, GemmaBlock, rope_tables
    from oracle import quant_oracle as O
    from tests.util import assert_gemm_close, bits, u8

    shape = GEMMA_2B if tower == "prefix" else GEMMA_300M
    config = L.FP8Config(backend="native") if quantization == "fp8" else L.NVFP4Config(backend="native")
    generator = torch.Generator(device=device).manual_seed(1003 if tower == "prefix" else 1004)
    block = GemmaBlock(shape, shape.heads * shape.head_dim, config, generator, device)
    x = torch.randn((batch, tokens, shape.width), device=device, generator=generator).to(torch.bfloat16)
    rope = rope_tables(torch.arange(tokens, device=device), shape.head_dim)
    records, handles = _linear_records(block)
    with torch.no_grad():
        output, _ = block(x, rope)
    for handle in handles:
        handle.remove()
    assert torch.isfinite(output).all() and [name for name, *_ in records] == ["qkv", "o_proj", "gate_up", "down"]
    for name, bundle, inputs, result in records:
        rows = bits(inputs.reshape(-1, inputs.shape[-1]))
        got = bits(result.reshape(-1, result.shape[-1]))
        if quantization == "fp8":
            codes, scale = O.fp8_quantize_T(rows, scalar_div="rcp", divisor_bf16=True)
            want = O.fp8_linear(codes, scale, u8(bundle.weight), np.float32(bundle.weight_scale.item()))
        else:
            packed, block_scales, global_scale = O.nvfp4_quantize_T(rows, "rcp")
            want = O.nvfp4_linear_registry(packed, block_scales, global_scale, u8(bundle.weight), u8(bundle.weight_scale),
                                           np.float32(bundle.weight_global_scale.item()))
        assert got.shape == want.shape, name
        assert_gemm_close(got, want)


def test_expert_runs_on_adaptive_norms(device):
    """The action expert's norms are AdaRMS norms: one modulation (scale | shift | gate, fp32 [B, 3 width]) per norm and
    Euler step, from the flow time only (policies/pi05/inference/runtime.py:366-401); the calibrated route feeds them
    to the fused norm + encoder launches (gated residual update, modulation, gate output) and stays close to the
    tensor-operation route; the actions do depend on the modulation."""
    from embodiinfer_b200.pi05_shaped import DENOISE_STEPS, GEMMA_300M
    policy = Pi05ShapedPolicy("fp8", device=device, layer_scale=0.12, vocabulary=4096)
    observations = synthetic_observations(4, vocabulary=4096)
    schedule = policy.modulation_schedule(4)
    assert len(schedule) == DENOISE_STEPS and len(schedule[0]) == 2 * len(policy.expert) + 1
    assert all(m.shape == (4, 3 * GEMMA_300M.width) and m.dtype == torch.float32 for m in schedule[0])
    assert not torch.equal(schedule[0][0], schedule[1][0]), "the modulation follows the flow time"
    reference = policy(observations)
    policy.calibrate_fused_mlp(observations)
    assert all(block.adaptive and block.qkv.norm is not None for block in policy.expert)
    fused = policy(observations)
    assert torch.isfinite(fused).all() and torch.equal(fused, policy(observations))
    assert float((fused - reference).norm() / reference.norm()) < 0.1
    for block in policy.expert:
        block.fused_norm = False
    unfused = policy(observations)
    assert float((fused - unfused).norm() / unfused.norm()) < 0.05
    for block in policy.expert:
        block.fused_norm = True
    with torch.no_grad():
        policy.final_dense.bias[: GEMMA_300M.width] += 0.5          # a different scale in the last norm
    policy.schedules.clear()
    assert float((policy(observations) - fused).norm() / fused.norm()) > 0.05
