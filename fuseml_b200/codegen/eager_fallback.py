"""``EagerFallbackGuard``: run a launch, and on failure run an eager function instead.

Kept as a class for API compatibility (fuseml/codegen/eager_fallback.py:63-298) and for
user code that wraps its *own* experimental kernels.  It is **not** installed on any
launcher this package builds: a matched chain that fails to launch raises, it is never
silently recomputed with PyTorch ops.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch

from .._logging import logger


class EagerFallbackGuard:
    def __init__(self, eager_fn: Callable[..., torch.Tensor], clone_inputs: bool = True) -> None:
        if not callable(eager_fn):
            raise TypeError("eager_fn must be callable")
        self._eager_fn = eager_fn
        self._clone_inputs = clone_inputs
        self._fallback_count = 0
        self._last_error: BaseException | None = None

    @property
    def fallback_count(self) -> int:
        return self._fallback_count

    @property
    def last_error(self) -> BaseException | None:
        return self._last_error

    def execute(self, launch_fn: Callable[[], torch.Tensor], input_tensors: Sequence[torch.Tensor],
                triton_buffers: Sequence[torch.Tensor] | None = None) -> torch.Tensor:
        """``launch_fn()``; on ``RuntimeError`` synchronise, drop the failed launch's buffers and
        return ``eager_fn(*inputs)`` computed from copies taken before the launch."""
        saved = [t.clone() if (self._clone_inputs and isinstance(t, torch.Tensor)) else t for t in input_tensors]
        try:
            return launch_fn()
        except RuntimeError as exc:
            self._fallback_count += 1
            self._last_error = exc
            logger.warning("fused launch failed (%s); running the eager function instead", exc)
            if torch.cuda.is_available():
                try:
                    torch.cuda.synchronize()
                except RuntimeError:
                    pass
                if "out of memory" in str(exc).lower():
                    torch.cuda.empty_cache()
            if triton_buffers is not None:
                del triton_buffers
            return self._eager_fn(*saved)

    def reset(self) -> None:
        self._fallback_count = 0
        self._last_error = None
