"""The scratch-free scale entry point (b2_tensor_scale_static) against b2_tensor_scale.

Some callers of this library can neither allocate device memory nor hand over a scratch buffer when
they need an activation scale: they run inside a fixed arena of raw device pointers owned by another
runtime, or in a process where cudaMalloc is off limits after start-up because it stalls every stream.
For them the library keeps the scratch in a static device array.  This file is collected last so that
a run stopping at the first failure has already executed every other test; it also passes when run on
its own in a fresh process.
"""

from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

from embodiinfer_b200 import _native as N

pytestmark = pytest.mark.gpu


def call_both(x: torch.Tensor, bound: float, flags: int) -> tuple[float, float]:
    """Both entry points through the C ABI on the current stream; returns (static, with caller scratch)."""
    library = N.load()
    device = x.device
    stream = torch.cuda.current_stream(device).cuda_stream
    scratch = torch.zeros(2, device=device, dtype=torch.int32)
    with_scratch = torch.full((), -1.0, device=device)
    static = torch.full((), -2.0, device=device)
    N.check(library.b2_tensor_scale(x.data_ptr(), x.numel(), bound, flags, scratch.data_ptr(), with_scratch.data_ptr(), stream),
            "b2_tensor_scale")
    N.check(library.b2_tensor_scale_static(x.data_ptr(), x.numel(), bound, flags, static.data_ptr(), stream),
            "b2_tensor_scale_static")
    torch.cuda.synchronize(device)
    return static.item(), with_scratch.item()


def test_two_calls_in_a_row_match_the_existing_entry_point(device):
    generator = torch.Generator().manual_seed(31)
    first = (torch.randn((560, 2048), generator=generator) * 3.0).to(torch.bfloat16).to(device)
    second = (torch.randn((17, 4099), generator=generator) * 0.01).to(torch.bfloat16).to(device)   # ragged count, smaller amax
    for x in (first, second):                       # the second call must not see the first call's leftovers
        for bound, flags in ((448.0, N.SCALAR_RCP), (2688.0, N.SCALAR_RCP | N.CLAMP_TINY), (448.0, 0)):
            static, reference = call_both(x, bound, flags)
            assert np.float32(static) == np.float32(reference)    # same bits, like the other scale tests
    zero = torch.zeros(4096, device=device, dtype=torch.bfloat16)
    assert call_both(zero, 448.0, N.SCALAR_RCP) == (1.0, 1.0)


def test_size_limit_and_argument_checks(device):
    library = N.load()
    scale = torch.zeros((), device=device)
    x = torch.zeros(64, device=device, dtype=torch.bfloat16)
    too_many = N.STATIC_SCALE_MAX_COUNT + 1
    assert library.b2_tensor_scale_static(x.data_ptr(), too_many, 448.0, 0, scale.data_ptr(), None) == N.E_TOO_LARGE
    with pytest.raises(RuntimeError, match="size beyond the entry point's maximum"):
        N.check(N.E_TOO_LARGE, "b2_tensor_scale_static")
    assert library.b2_tensor_scale_static(None, 64, 448.0, 0, scale.data_ptr(), None) == N.E_INVALID
    assert library.b2_tensor_scale_static(ctypes.c_void_p(x.data_ptr() + 2), 32, 448.0, 0, scale.data_ptr(), None) == N.E_INVALID


def test_largest_supported_tensor(device):
    """A 32 Mi-element tensor (half the documented maximum) uses 2048 of the 4096 slots."""
    x = torch.randn(32 * 1024 * 1024, device=device).to(torch.bfloat16)
    static, reference = call_both(x, 448.0, N.SCALAR_RCP)
    assert np.float32(static) == np.float32(reference)
    assert np.float32(static) == np.float32((x.float().abs().amax() * torch.tensor(1.0 / 448.0, device=device)).item())


def test_documented_maximum_uses_every_slot(device):
    """Exactly B2_STATIC_SCALE_MAX_COUNT elements (64 Mi bf16, 128 MB): the last of the 4096 slots of the static
    array is in use, with the largest magnitude placed in the very last element, and a second call at the boundary
    right behind it sees none of the first one's state."""
    count = N.STATIC_SCALE_MAX_COUNT
    x = torch.randn(count, device=device).to(torch.bfloat16)
    x[-1] = 300.0
    static, reference = call_both(x, 448.0, N.SCALAR_RCP)
    assert np.float32(static) == np.float32(reference) == np.float32(np.float32(300.0) * np.float32(1.0 / 448.0))
    x[-1] = 0.5
    static, reference = call_both(x, 448.0, N.SCALAR_RCP)
    assert np.float32(static) == np.float32(reference)
    assert np.float32(static) == np.float32((x.float().abs().amax() * torch.tensor(1.0 / 448.0, device=device)).item())
