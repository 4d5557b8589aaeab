"""The fused split + rotary + key/value write against the reference's rotation evaluated by torch on the device."""

from __future__ import annotations

import pytest
import torch

from embodiinfer_b200 import kernels as K
from embodiinfer_b200.pi05_shaped import rope_reference, rope_tables

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("batch,tokens,heads,kv_heads,head_dim,prefix", [(1, 560, 8, 1, 256, 0), (3, 10, 8, 1, 256, 560), (2, 7, 4, 2, 64, 5)])
def test_rope_split_is_bit_exact(device, batch, tokens, heads, kv_heads, head_dim, prefix):
    generator = torch.Generator(device=device).manual_seed(tokens + head_dim)
    width = (heads + 2 * kv_heads) * head_dim
    qkv = torch.randn((batch * tokens, width), device=device, generator=generator).to(torch.bfloat16)
    tables = rope_tables(prefix + torch.arange(tokens, device=device), head_dim)
    q = torch.empty((batch, heads, tokens, head_dim), device=device, dtype=torch.bfloat16)
    keys = torch.full((batch, kv_heads, prefix + tokens, head_dim), 3.0, device=device, dtype=torch.bfloat16)
    values = torch.full_like(keys, -2.0)
    K.rope_split(qkv, tables[0], tables[1], q, keys, values, batch=batch, tokens=tokens, heads=heads, kv_heads=kv_heads,
                 head_dim=head_dim, kv_offset=prefix)
    rows = qkv.view(batch, tokens, heads + 2 * kv_heads, head_dim).transpose(1, 2)         # [B, H_total, T, D]
    assert torch.equal(q, rope_reference(rows[:, :heads], tables))
    assert torch.equal(keys[:, :, prefix:], rope_reference(rows[:, heads: heads + kv_heads], tables))
    assert torch.equal(values[:, :, prefix:], rows[:, heads + kv_heads:])
    assert (keys[:, :, :prefix] == 3.0).all() and (values[:, :, :prefix] == -2.0).all()    # earlier positions untouched


def test_rope_split_rejects_bad_arguments(device):
    qkv = torch.zeros((4, 3 * 24), device=device, dtype=torch.bfloat16)
    sine = cosine = torch.zeros((4, 12), device=device)
    q = torch.empty((1, 1, 4, 24), device=device, dtype=torch.bfloat16)
    cache = torch.empty((1, 1, 4, 24), device=device, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):          # head_dim must be a multiple of 16
        K.rope_split(qkv, sine, cosine, q, cache, cache.clone(), batch=1, tokens=4, heads=1, kv_heads=1, head_dim=24)


@pytest.mark.parametrize("batch,tokens,heads,kv_heads,prefix,per_batch_tables", [
    (1, 10, 8, 1, 570, False), (3, 10, 8, 1, 560, False), (8, 10, 8, 1, 30, True), (1, 1, 2, 2, 0, False), (2, 64, 3, 1, 7, False)])
def test_rope_epilogue_of_the_projection_matches_two_launches(device, batch, tokens, heads, kv_heads, prefix, per_batch_tables):
    """``b2_linear_desc.rope``: the packed FP8 QKV projection writes rotated queries, keys and values itself.  Same bits as
    the projection followed by b2_rope_split (the projection on the same schedule both times)."""
    from embodiinfer_b200 import _native as N
    head_dim, width = 256, 1024
    rows, features = batch * tokens, (heads + 2 * kv_heads) * head_dim
    generator = torch.Generator(device=device).manual_seed(rows + features)
    act = torch.randint(0, 256, (rows, width), device=device, dtype=torch.uint8, generator=generator)
    weight = torch.randint(0, 256, (features, width), device=device, dtype=torch.uint8, generator=generator)
    for codes in (act, weight):
        codes[(codes & 0x7f) == 0x7f] = 0x30           # no NaN codes
    act_scale, weight_scale = torch.tensor(2.0 ** -6, device=device), torch.tensor(2.0 ** -9, device=device)
    tables = rope_tables(prefix + torch.arange(tokens, device=device), head_dim)
    if per_batch_tables:
        tables = tuple(torch.stack([torch.roll(t, b, dims=0) for b in range(batch)]).contiguous() for t in tables)
    common = dict(kind=N.KIND_FP8, epilogue=N.EPI_LINEAR, out_format=N.OUT_BF16, tokens=rows, features=features, width=width,
                  act=act, act_scale=act_scale, weight=weight, weight_scale=weight_scale, flags=N.LINEAR_CLUSTER)
    results = []
    for fused in (False, True):
        q = torch.zeros((batch, heads, tokens, head_dim), device=device, dtype=torch.bfloat16)
        keys = torch.full((batch, kv_heads, prefix + tokens, head_dim), 3.0, device=device, dtype=torch.bfloat16)
        values = torch.full_like(keys, -2.0)
        out = torch.zeros((rows, features), device=device, dtype=torch.bfloat16)
        preparation = dict(sine=tables[0], cosine=tables[1], q_out=q, k_out=keys, v_out=values, batch=batch, tokens=tokens, heads=heads,
                           kv_heads=kv_heads, head_dim=head_dim, kv_offset=prefix)
        if fused:
            K.linear(out=out, rope=preparation, **common)
        else:
            K.linear(out=out, **common)
            K.rope_split(out, **preparation)
        torch.cuda.synchronize()
        K.check_status(device)
        results.append((q, keys, values))
    for a, b in zip(*results):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    assert results[0][0].view(torch.int16).any()
    assert (results[1][1][:, :, :prefix] == 3.0).all() and (results[1][2][:, :, :prefix] == -2.0).all()


def test_rope_epilogue_refuses_what_it_does_not_handle(device):
    from embodiinfer_b200 import _native as N
    act = torch.zeros((10, 1024), device=device, dtype=torch.uint8)
    weight = torch.zeros((2560, 1024), device=device, dtype=torch.uint8)
    one = torch.tensor(1.0, device=device)
    tables = rope_tables(torch.arange(10, device=device), 256)
    q = torch.zeros((1, 8, 10, 256), device=device, dtype=torch.bfloat16)
    cache = torch.zeros((1, 1, 10, 256), device=device, dtype=torch.bfloat16)
    out = torch.zeros((10, 2560), device=device, dtype=torch.bfloat16)
    preparation = dict(sine=tables[0], cosine=tables[1], q_out=q, k_out=cache, v_out=cache.clone(), batch=1, tokens=10, heads=8, kv_heads=1, head_dim=256)
    common = dict(kind=N.KIND_FP8, epilogue=N.EPI_LINEAR, out_format=N.OUT_BF16, tokens=10, features=2560, width=1024, act=act, act_scale=one,
                  weight=weight, weight_scale=one, out=out)
    K.linear(rope=preparation, **common)                                                       # the supported form
    with pytest.raises(RuntimeError, match="error -2"):                                       # the tile schedule was asked for
        K.linear(rope=preparation, flags=N.LINEAR_SINGLE_CTA, **common)
    with pytest.raises(RuntimeError, match="error -2"):                                       # a bias
        K.linear(rope=preparation, bias=torch.zeros(2560, device=device, dtype=torch.bfloat16), **common)
    with pytest.raises(RuntimeError, match="error -2"):                                       # features do not match the heads
        K.linear(rope={**preparation, "heads": 7, "q_out": q[:, :7].contiguous()}, **common)
    torch.cuda.synchronize()
