"""Weight refit for rollout replicas: one rank (the learner) broadcasts, every replica copies in place.

Counterpart of ``NCCLBroadcastSync`` (embodiinfer/engine/rollout/weight_sync.py:59-80), which broadcasts
every parameter tensor on its own and then advances the policy version (``commit_refit``).  Here the
state that moves is the *quantised* bundle state (packed codes, block scales, global scales, biases:
``FP8Linear`` / ``NVFP4Linear`` buffers, a quarter to a half of the bf16 bytes), tensors of one dtype are
packed into buckets of ``bucket_bytes`` so that NVLink sees a few large broadcasts instead of hundreds of
small ones, and the copy back is in place: device pointers held by captured CUDA graphs and by the plan
objects stay valid.  Rank order, names and shapes must agree on all ranks (same model definition).

Plan objects keep their packed operands outside the module's state dict.  A module (or any of its
submodules) that defines ``refit_tensors() -> dict[name, tensor]`` has those tensors broadcast and refreshed
in place as well, under the prefix ``plans.``; ``on_refit`` callbacks run after the copies and BEFORE the
version advances, like the reference's hook (embodiinfer/engine/rollout/refit.py:122-137), so a reader that
sees the new version never computes with stale derived state.
"""

from __future__ import annotations

from collections.abc import Callable, Iterable

import torch
import torch.distributed as dist
from torch import nn


class BroadcastWeightSync:
    def __init__(self, module: nn.Module, src_rank: int = 0, group: dist.ProcessGroup | None = None,
                 bucket_bytes: int = 64 << 20, on_refit: Iterable[Callable[[], None]] = ()) -> None:
        if bucket_bytes <= 0:
            raise ValueError("bucket_bytes must be positive")
        self.module, self.src_rank, self.group, self.bucket_bytes = module, src_rank, group, bucket_bytes
        self.on_refit = list(on_refit)
        self.version = 0

    @property
    def policy_version(self) -> int:
        """Monotonic count of completed refits (weight_sync.py:67-70)."""
        return self.version

    def _tensors(self, names: Iterable[str] | None) -> list[tuple[str, torch.Tensor]]:
        state = {name: tensor for name, tensor in self.module.state_dict(keep_vars=True).items()}
        owners = [self.module] if hasattr(self.module, "refit_tensors") else [
            child for child in self.module.modules() if child is not self.module and hasattr(child, "refit_tensors")]
        for owner in owners:
            for name, tensor in owner.refit_tensors().items():
                state.setdefault(f"plans.{name}", tensor)
        if names is None:
            selected = sorted(state)
        else:
            selected = list(names)
            missing = [name for name in selected if name not in state]
            if missing:
                raise KeyError(f"unknown parameter or buffer names: {missing[:4]}")
        return [(name, state[name].data) for name in selected]

    @torch.no_grad()
    def update(self, names: Iterable[str] | None = None) -> int:
        """Broadcast the named tensors (default: the whole state dict) from ``src_rank`` and copy them into
        the live module in place.  Returns the number of broadcasts issued."""
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed not initialized")
        by_dtype: dict[tuple[torch.dtype, torch.device], list[torch.Tensor]] = {}
        for _, tensor in self._tensors(names):
            by_dtype.setdefault((tensor.dtype, tensor.device), []).append(tensor)
        broadcasts = 0
        for (dtype, device), tensors in by_dtype.items():
            bucket: list[torch.Tensor] = []
            size = 0
            for tensor in [*tensors, None]:
                nbytes = 0 if tensor is None else tensor.numel() * tensor.element_size()
                if bucket and (tensor is None or size + nbytes > self.bucket_bytes):
                    flat = torch.cat([piece.reshape(-1) for piece in bucket]) if len(bucket) > 1 else bucket[0].reshape(-1).clone()
                    carrier = flat.view(torch.uint8) if dtype in (torch.float8_e4m3fn,) else flat
                    dist.broadcast(carrier, src=self.src_rank, group=self.group)
                    offset = 0
                    for piece in bucket:
                        piece.copy_(flat[offset: offset + piece.numel()].view(piece.shape))
                        offset += piece.numel()
                    broadcasts += 1
                    bucket, size = [], 0
                if tensor is not None:
                    bucket.append(tensor)
                    size += nbytes
        for hook in self.on_refit:          # derived state is rebuilt before a reader can see the new version
            hook()
        self.version += 1
        return broadcasts
