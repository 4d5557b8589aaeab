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
