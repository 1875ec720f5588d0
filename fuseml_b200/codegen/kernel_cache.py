"""Identity of a compiled fused chain, and the per-compiler launcher cache.

Same API as the reference (fuseml/codegen/kernel_cache.py:65-531): ``TensorFingerprint``
(shape, stride, storage offset, 16-byte alignment, dtype, stride-0 dims),
``KernelCacheKey`` (op chain + input fingerprints + output shape/dtype + device
capability), ``KernelCache`` with hit / miss counters, ``build_op_chain`` and
``build_cache_key``.  Two things are added because a precompiled sm_100a kernel is
selected by them: the fingerprint records whether TMA can address the tensor
directly (``tma_legal``), and the key carries the plan the router chose
(tile width, stages, cluster) so that two shapes landing on different kernel
instances never share a launcher.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

import torch

from .._logging import logger

_ELEM_BYTES = {"torch.float32": 4, "torch.float16": 2, "torch.bfloat16": 2}


def _materialize_ints(vals) -> tuple[int, ...]:
    """Concrete, hashable ints from a shape / stride that may hold ``torch.SymInt``."""
    return tuple(int(v) for v in vals)


def _materialize_int(val) -> int:
    return int(val)


def _tma_legal(shape: tuple, stride: tuple, aligned: bool, dtype: str) -> bool:
    """Can a 2-D TMA map with one unit stride describe this tensor?  (16-byte aligned base,
    the other stride a multiple of 16 bytes.)  1-D / 0-D tensors are read by plain loads."""
    if len(shape) != 2:
        return True
    eb = _ELEM_BYTES.get(dtype)
    if eb is None or not aligned:
        return False
    s0, s1 = stride
    if s1 == 1:
        return shape[0] == 1 or (s0 * eb) % 16 == 0
    if s0 == 1:
        return shape[1] == 1 or (s1 * eb) % 16 == 0
    return False


@dataclass(frozen=True)
class TensorFingerprint:
    shape: tuple
    stride: tuple
    storage_offset: int
    aligned: bool
    dtype: str
    broadcast_dims: tuple = ()

    def _key(self):
        return (self.shape, self.stride, self.storage_offset, self.aligned, self.dtype, self.broadcast_dims)

    def __hash__(self) -> int:
        return hash(self._key())

    def __eq__(self, other: object) -> bool:
        if not isinstance(other, TensorFingerprint):
            return NotImplemented
        return self._key() == other._key()

    def __lt__(self, other: object) -> bool:
        if not isinstance(other, TensorFingerprint):
            return NotImplemented
        return self._key() < other._key()

    @property
    def tma_legal(self) -> bool:
        return _tma_legal(self.shape, self.stride, self.aligned, self.dtype)

    @classmethod
    def from_tensor(cls, t: torch.Tensor) -> "TensorFingerprint":
        stride = _materialize_ints(t.stride())
        try:
            aligned = t.data_ptr() % 16 == 0
        except RuntimeError:       # FakeTensor / FunctionalTensor: no storage
            aligned = True
        return cls(_materialize_ints(t.shape), stride, _materialize_int(t.storage_offset()), aligned,
                   str(t.dtype), tuple(s == 0 for s in stride))

    @classmethod
    def from_node(cls, node: torch.fx.Node) -> Optional["TensorFingerprint"]:
        """From FX metadata: ``tensor_meta`` (ShapeProp) first, then ``val`` (FakeTensor).
        Intermediate results are fresh allocations: offset 0, aligned."""
        meta = node.meta.get("tensor_meta")
        if meta is not None and not hasattr(meta, "shape"):
            meta = meta[0] if isinstance(meta, (tuple, list)) and len(meta) > 0 else None
        if meta is not None and hasattr(meta, "shape"):
            stride = _materialize_ints(meta.stride)
            return cls(_materialize_ints(meta.shape), stride, 0, True, str(meta.dtype),
                       tuple(s == 0 for s in stride))
        val = node.meta.get("val")
        if val is not None and hasattr(val, "shape"):
            stride = (_materialize_ints(val.stride()) if callable(getattr(val, "stride", None))
                      else (1,) * len(val.shape))
            offset = (_materialize_int(val.storage_offset()) if callable(getattr(val, "storage_offset", None))
                      else 0)
            return cls(_materialize_ints(val.shape), stride, offset, True, str(val.dtype),
                       tuple(s == 0 for s in stride))
        return None


@dataclass(frozen=True)
class KernelCacheKey:
    op_chain: tuple
    input_fingerprints: tuple
    output_shapes: tuple
    output_dtypes: tuple
    device_capability: tuple
    plan: tuple = ()        # (tile_n, stages, cluster) chosen by the router; () when not planned yet

    def _key(self):
        # fingerprints compare as a sorted multiset, as in the reference: the launcher is
        # positional and re-prepares per live shape, so input order carries no kernel identity
        return (self.op_chain, tuple(sorted(self.input_fingerprints)), self.output_shapes, self.output_dtypes,
                self.device_capability, self.plan)

    def __hash__(self) -> int:
        return hash(self._key())

    def __eq__(self, other: object) -> bool:
        if not isinstance(other, KernelCacheKey):
            return NotImplemented
        return self._key() == other._key()


class KernelCache:
    """In-memory map key -> launcher, owned by one ``FuseMLCompiler``."""

    def __init__(self) -> None:
        self._store: dict[KernelCacheKey, Any] = {}
        self._hits = 0
        self._misses = 0

    def lookup(self, key: KernelCacheKey) -> Any | None:
        launcher = self._store.get(key)
        if launcher is not None:
            self._hits += 1
            logger.debug("kernel cache hit (%d entries)", len(self._store))
            return launcher
        self._misses += 1
        return None

    def store(self, key: KernelCacheKey, launcher: Any) -> None:
        self._store[key] = launcher

    @property
    def size(self) -> int:
        return len(self._store)

    @property
    def hits(self) -> int:
        return self._hits

    @property
    def misses(self) -> int:
        return self._misses

    def clear(self) -> None:
        self._store.clear()
        self._hits = 0
        self._misses = 0


_cached_device_capability: tuple | None = None


def _get_device_capability(tensor_map: dict) -> tuple:
    """Capability of the first CUDA tensor in ``tensor_map``; ``(0, 0)`` for CPU-only maps."""
    global _cached_device_capability
    if _cached_device_capability is not None:
        return _cached_device_capability
    for t in tensor_map.values():
        if isinstance(t, torch.Tensor) and t.is_cuda:
            _cached_device_capability = tuple(torch.cuda.get_device_capability(t.device))
            return _cached_device_capability
    return (0, 0)


def build_op_chain(group: Any) -> tuple:
    from ..passes.topology import canonicalize_target

    return tuple(canonicalize_target(n.target) for n in group.all_nodes if n.op == "call_function")


def build_cache_key(group: Any, tensor_map: dict, output_shape: tuple | None = None,
                    output_dtype: str | None = None, plan: tuple = ()) -> KernelCacheKey | None:
    """Key for ``group``: live tensors from ``tensor_map`` (by input node name) where present,
    FX metadata otherwise; None when an input or the output cannot be described."""
    fingerprints = []
    for node in group.inputs:
        t = tensor_map.get(node.name)
        fp = TensorFingerprint.from_tensor(t) if t is not None else TensorFingerprint.from_node(node)
        if fp is None:
            logger.debug("cannot fingerprint input %s: no cache key", node.name)
            return None
        fingerprints.append(fp)
    shape, dtype = output_shape, output_dtype
    if shape is None or dtype is None:
        meta = getattr(group, "output_metadata", None) or {}
        if "shape" in meta:
            shape = shape or tuple(meta["shape"])
            dtype = dtype or str(meta["dtype"])
        else:
            fp = TensorFingerprint.from_node(group.output_node)
            if fp is None:
                logger.debug("cannot determine output metadata: no cache key")
                return None
            shape = shape or fp.shape
            dtype = dtype or fp.dtype
    return KernelCacheKey(build_op_chain(group), tuple(fingerprints), (shape,), (dtype,),
                          _get_device_capability(tensor_map), tuple(plan))
