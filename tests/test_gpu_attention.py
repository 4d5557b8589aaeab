"""b2_attention (tcgen05 multi-query attention, head dimension 256) against a float32 PyTorch attention on the same
bf16 inputs.  Tolerance: the output is bf16 (relative rounding error up to 2^-9, about 1.1e-3 rms) and the probabilities
enter the second product as bf16, as in torch's own flash kernels; the test asks for a relative Frobenius error of at
most 3e-3 against the float32 result and for an error no larger than 1.5 times torch's bf16 scaled_dot_product_attention
on the same inputs (reference semantics: embodiinfer/backend/torch/attention.py:97-106)."""

from __future__ import annotations

import pytest
import torch
import torch.nn.functional as F

from embodiinfer_b200 import kernels as K

pytestmark = pytest.mark.gpu


def reference(q, k, v):
    scores = torch.einsum("bhtd,bsd->bhts", q.float(), k[:, 0].float()) / 16.0
    return torch.einsum("bhts,bsd->bhtd", scores.softmax(-1), v[:, 0].float())


def relative(a, b):
    return float((a.float() - b).norm() / b.norm())


@pytest.mark.parametrize("batch,heads,queries,keys", [
    (2, 8, 560, 560),       # prefix tower: 4480 query rows per batch element, 35 tiles, 9 key tiles (the last one ragged)
    (3, 8, 10, 570),        # action expert: ten-token chunk over prefix + chunk
    (1, 8, 10, 570),
    (1, 1, 1, 1),           # a single key: softmax is 1
    (2, 3, 77, 64),         # exactly one key tile, ragged rows
    (2, 8, 16, 65),         # one key in the second tile
    (1, 8, 128, 128),
    # one tile per batch element and several key tiles: the keys are cut across a cluster of 8 / 4 / 2 CTAs
    (1, 8, 10, 580),        # ten key tiles, one per CTA where clusters of ten are available (else unequal key ranges over eight)
    (1, 8, 13, 130),        # 104 rows, three key tiles over three CTAs
    (1, 8, 16, 200),        # a full tile of 128 rows
    (1, 2, 5, 1000),        # sixteen key tiles: the largest cluster
    (2, 4, 7, 300),         # 28 rows over four CTAs, a ragged last key tile
    (1, 1, 3, 1030),        # fewer rows than CTAs: most CTAs own none
    (9, 8, 10, 570),        # nine clusters of eight
    (20, 8, 10, 570),       # clusters of two
])
@pytest.mark.parametrize("spread", (1.0, 6.0))
def test_attention_matches_float32(device, batch, heads, queries, keys, spread):
    generator = torch.Generator(device=device).manual_seed(7 * batch + heads + queries + keys)
    q = (torch.randn((batch, heads, queries, 256), device=device, generator=generator) * spread).to(torch.bfloat16)
    k = torch.randn((batch, 1, keys, 256), device=device, generator=generator).to(torch.bfloat16)
    v = torch.randn((batch, 1, keys, 256), device=device, generator=generator).to(torch.bfloat16)
    status = torch.zeros(1, device=device, dtype=torch.int32)
    out = torch.full((batch * heads * queries + 1, 256), float("nan"), device=device, dtype=torch.bfloat16)
    result = K.attention(q, k, v, out[:-1].view(batch, heads, queries, 256), status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.isnan(out[-1]).all(), "wrote past the last row"
    want = reference(q, k, v)
    error = relative(result, want)
    library = relative(F.scaled_dot_product_attention(q, k, v, enable_gqa=heads > 1), want)
    assert torch.isfinite(result.float()).all()
    assert error <= 3e-3, (error, library)
    assert error <= 1.5 * library + 1e-4, (error, library)


@pytest.mark.parametrize("batch,heads,queries,keys", [(1, 8, 10, 580), (3, 8, 10, 570), (2, 8, 560, 560), (40, 8, 10, 70), (2, 3, 77, 64)])
def test_encoded_output_matches_attention_then_encoder(device, batch, heads, queries, keys):
    """b2_attention_fp8 writes the e4m3 rows [B*T, H*256] of the output projection: the same bytes as b2_attention followed
    by b2_bhsd_quant, on the split (clusters over the keys) and the one-CTA-per-tile paths."""
    generator = torch.Generator(device=device).manual_seed(batch + heads + queries + keys)
    q = torch.randn((batch, heads, queries, 256), device=device, generator=generator).to(torch.bfloat16)
    k = torch.randn((batch, 1, keys, 256), device=device, generator=generator).to(torch.bfloat16)
    v = (3.0 * torch.randn((batch, 1, keys, 256), device=device, generator=generator)).to(torch.bfloat16)
    multiplier = 448.0 / 2.5                    # values beyond 2.5 saturate
    status = torch.zeros(1, device=device, dtype=torch.int32)
    out = K.attention(q, k, v, status=status)
    want = torch.zeros((batch * queries, heads * 256), device=device, dtype=torch.uint8)
    K.bhsd_quant(out, want, bits=8, scale_value=multiplier)
    got = torch.full((batch * queries + 1, heads * 256), 0x7f, device=device, dtype=torch.uint8)
    K.attention(q, k, v, codes=got[:-1], multiplier=multiplier, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(got[:-1], want)
    assert (got[-1] == 0x7f).all(), "wrote past the last row"
    assert want.any()


@pytest.mark.parametrize("batch,heads,queries,keys", [(1, 8, 10, 580), (3, 8, 10, 570), (2, 8, 560, 560), (40, 8, 10, 70), (2, 3, 77, 64)])
@pytest.mark.parametrize("with_rows", (True, False))
def test_nvfp4_output_matches_attention_then_encoder(device, batch, heads, queries, keys, with_rows):
    """b2_attention_nvfp4 writes the NVFP4 rows of the output projection (e2m1 pairs, tiled and row-major e4m3 block scales):
    the same bytes as b2_attention followed by b2_bhsd_quant (bits 4), on the split and the one-CTA-per-tile paths.  The
    global scale is small enough for some block scales to saturate at 448 and some rows are zero (block scale 0)."""
    generator = torch.Generator(device=device).manual_seed(batch + heads + queries + keys)
    q = torch.randn((batch, heads, queries, 256), device=device, generator=generator).to(torch.bfloat16)
    k = torch.randn((batch, 1, keys, 256), device=device, generator=generator).to(torch.bfloat16)
    v = (3.0 * torch.randn((batch, 1, keys, 256), device=device, generator=generator)).to(torch.bfloat16)
    v[:, :, :, 32:48] = 0                        # a block of zeros in every row
    v[:, :, :, 100] *= 64.0                      # a block whose scale saturates
    global_scale = 2.5 / (448.0 * 6.0)
    rows, blocks = batch * queries, heads * 16
    tiled = (rows + 127) // 128 * ((blocks + 3) // 4) * 512
    status = torch.zeros(1, device=device, dtype=torch.int32)
    out = K.attention(q, k, v, status=status)
    want = torch.zeros((rows, heads * 128), device=device, dtype=torch.uint8)
    want_rows = torch.zeros((rows, blocks), device=device, dtype=torch.uint8)
    want_tiled = torch.zeros(tiled, device=device, dtype=torch.uint8)
    K.bhsd_quant(out, want, bits=4, scale_value=global_scale, scales=want_rows, blocked=want_tiled)
    got = torch.full((rows + 1, heads * 128), 0x7f, device=device, dtype=torch.uint8)
    got_rows = torch.full((rows + 1, blocks), 0x7f, device=device, dtype=torch.uint8) if with_rows else None
    got_tiled = torch.zeros(tiled, device=device, dtype=torch.uint8)
    K.attention(q, k, v, codes=got[:-1], blocked=got_tiled, scales=None if got_rows is None else got_rows[:-1],
                global_scale=global_scale, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(got[:-1], want) and torch.equal(got_tiled, want_tiled)
    assert (got[-1] == 0x7f).all(), "wrote past the last row"
    if with_rows:
        assert torch.equal(got_rows[:-1], want_rows) and (got_rows[-1] == 0x7f).all()
    assert want.any() and (want_rows == 0).any() and (want_rows == 0x7e).any()


def test_attention_rejects_other_shapes(device):
    q = torch.zeros((1, 2, 4, 128), device=device, dtype=torch.bfloat16)
    k = torch.zeros((1, 1, 4, 128), device=device, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="error -2"):
        K.attention(q, k, k.clone())
    with pytest.raises(ValueError):
        K.attention(q, torch.zeros((1, 2, 4, 128), device=device, dtype=torch.bfloat16), k)
