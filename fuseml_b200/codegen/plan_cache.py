"""Measured launch plans, persisted on disk.

The native router (``fuseml_sm100_plan``) chooses tile width, CTA pairing, rasterisation group
and split-K from a roofline model in microseconds, so nothing *has* to be tuned or cached.  For
shapes whose tile count does not fill whole waves of the 74 CTA pairs (row shards of a few
hundred to a few thousand rows) a measured choice can beat the model: :func:`tune_plan` times
a handful of candidate plans on the live tensors of the first call and keeps the fastest, and
:class:`PlanCache` persists it as JSON so that the next process starts from the measured plan
without measuring again.

The reference persists only generated Triton source (a SHA-256 keyed temp directory,
fuseml/codegen/kernel_generator.py:1067-1172) and re-runs Triton's autotuner in every process
(27-98 s per kernel on first call, fuseml/codegen/kernel_launcher.py:640-670 describes the frozen
launch it is building towards); here the tuned result itself is what is stored.

File format: ``{"version": 1, "plans": {key: {"tile_n", "cluster", "grid", "group_m",
"split_k", "stream_k", "group_n", "us", "candidates"}}}``.  The key names the device, the library build, the problem
(M, N, K, dtypes, B layout) and the epilogue signature, so a rebuilt library or another GPU
never picks up a stale entry.  Writes are atomic (temp file + rename).
"""
from __future__ import annotations

import json
import os
import tempfile
import threading
from pathlib import Path
from typing import Callable, Iterable

from .. import _native as N
from .._logging import logger

ENV_PATH = "FUSEML_PLAN_CACHE"
ENV_AUTOTUNE = "FUSEML_AUTOTUNE"
_FIELDS = ("tile_n", "cluster", "grid", "group_m", "split_k")


def default_path() -> Path:
    p = os.environ.get(ENV_PATH)
    if p:
        return Path(p)
    base = os.environ.get("XDG_CACHE_HOME") or os.path.join(os.path.expanduser("~"), ".cache")
    return Path(base) / "fuseml_b200" / "plan_cache.json"


def autotune_requested() -> bool:
    return os.environ.get(ENV_AUTOTUNE, "").strip() not in ("", "0", "false", "False")


def plan_key(device_name: str, build_id: str, M: int, Ncols: int, Kd: int, ab_dtype: int, out_dtype: int,
             b_layout: str, signature: str) -> str:
    return "|".join((device_name, build_id, f"{M}x{Ncols}x{Kd}", f"ab{ab_dtype}", f"out{out_dtype}", b_layout, signature))


class PlanCache:
    """JSON file of measured plans; safe to share between threads of one process.  Several
    processes may write the same file: each write re-reads it first and replaces it atomically, so
    a lost update costs one re-measurement, never a corrupt file."""

    def __init__(self, path: os.PathLike | str | None = None) -> None:
        self.path = Path(path) if path is not None else default_path()
        self._lock = threading.Lock()
        self._plans: dict[str, dict] = {}
        self.hits = 0
        self.misses = 0
        self._load()

    def _load(self) -> None:
        try:
            data = json.loads(self.path.read_text())
            if data.get("version") == 1 and isinstance(data.get("plans"), dict):
                self._plans.update(data["plans"])
        except FileNotFoundError:
            pass
        except Exception as exc:       # an unreadable cache is ignored, not fatal
            logger.warning("plan cache %s ignored: %r", self.path, exc)

    def __len__(self) -> int:
        return len(self._plans)

    def get(self, key: str) -> dict | None:
        with self._lock:
            e = self._plans.get(key)
            if e is None:
                self.misses += 1
            else:
                self.hits += 1
            return dict(e) if e is not None else None

    def put(self, key: str, entry: dict) -> None:
        with self._lock:
            self._load()               # merge what other processes wrote since
            self._plans[key] = dict(entry)
            try:
                self.path.parent.mkdir(parents=True, exist_ok=True)
                fd, tmp = tempfile.mkstemp(dir=str(self.path.parent), prefix=self.path.name, suffix=".tmp")
                with os.fdopen(fd, "w") as f:
                    json.dump({"version": 1, "plans": self._plans}, f, indent=1, sort_keys=True)
                os.replace(tmp, self.path)
            except OSError as exc:     # read-only home, full disk: keep the entry in memory
                logger.warning("plan cache %s not written: %r", self.path, exc)


def apply_entry(plan: N.Plan, entry: dict) -> bool:
    """Copy a stored choice into ``plan``; False (plan untouched) when the entry is malformed."""
    try:
        vals = {k: int(entry[k]) for k in _FIELDS}
    except (KeyError, TypeError, ValueError):
        return False
    if vals["tile_n"] % 32 or not 32 <= vals["tile_n"] <= 256 or vals["cluster"] not in (1, 2) or vals["grid"] <= 0 \
            or vals["group_m"] <= 0 or not 0 <= vals["split_k"] <= 64:
        return False
    for k, v in vals.items():
        setattr(plan, k, v)
    # flag entries are absent in files written before the flag existed: the router's choice stands
    for name, bit in (("stream_k", N.PLAN_STREAM_K), ("group_n", N.PLAN_GROUP_N)):
        if name in entry:
            plan.flags = (plan.flags & ~bit) | (bit if entry[name] else 0)
    return True


def entry_of(plan: N.Plan, us: float | None = None, candidates: int = 0) -> dict:
    e = {k: int(getattr(plan, k)) for k in _FIELDS}
    e["stream_k"] = int(bool(plan.flags & N.PLAN_STREAM_K))
    e["group_n"] = int(bool(plan.flags & N.PLAN_GROUP_N))
    if us is not None:
        e["us"] = round(float(us), 3)
    e["candidates"] = int(candidates)
    return e


def candidate_plans(base: N.Plan, M: int, Ncols: int, sm_count: int = 148, has_reduction: bool = False) -> list[N.Plan]:
    """The router's plan first, then its neighbours: narrower CTA-pair tiles whose tile count fills
    the last wave better, other rasterisation groups, other split-K factors.  A handful at most."""
    out = [N.Plan.from_buffer_copy(base)]

    def add(**kw) -> None:
        p = N.Plan.from_buffer_copy(base)
        for k, v in kw.items():
            setattr(p, k, v)
        if all(any(getattr(p, f) != getattr(q, f) for f in _FIELDS + ("flags",)) for q in out):
            out.append(p)

    if base.cluster == 2:
        units = max(1, sm_count // 2)
        tiles_m = (M + 255) // 256
        base_waves = -(-(tiles_m * -(-Ncols // base.tile_n)) // units) * base.tile_n
        for bn in (224, 192, 160):
            tiles = tiles_m * -(-Ncols // bn)
            if -(-tiles // units) * bn < base_waves:          # fewer column-waves of work
                add(tile_n=bn, grid=min(tiles, units) * 2)
        along = -(-Ncols // base.tile_n) if base.flags & N.PLAN_GROUP_N else tiles_m     # what group_m counts
        for gm in (max(1, base.group_m // 2), min(along, base.group_m * 2)):
            add(group_m=gm)
        tiles_n = -(-Ncols // base.tile_n)
        if tiles_m * tiles_n >= 2 * units:                    # the other walk: bands of columns <-> groups of rows
            other = tiles_m if base.flags & N.PLAN_GROUP_N else tiles_n
            add(flags=base.flags ^ N.PLAN_GROUP_N, group_m=max(1, min(other, base.group_m)))
        rem = (tiles_m * -(-Ncols // base.tile_n)) % units
        if 0 < rem and not has_reduction:                     # the last wave shared by K ranges, or not
            if base.flags & N.PLAN_STREAM_K:
                add(flags=base.flags & ~N.PLAN_STREAM_K)
            else:                                             # every pair takes part in the last wave
                add(flags=base.flags | N.PLAN_STREAM_K, grid=units * 2)
    elif base.split_k > 1 and not has_reduction:
        for sk in (max(2, base.split_k // 2), min(32, base.split_k * 2)):
            tiles = -(-Ncols // base.tile_n)
            add(split_k=sk, grid=tiles * sk)
    return out


def tune_plan(launch: Callable[[N.Plan], None], candidates: Iterable[N.Plan], *, warmup: int = 3, iters: int = 10):
    """Time ``launch(plan)`` for every candidate with CUDA events on the current stream and return
    ``(best_plan, best_us, n_tried)``.  A candidate whose launch raises is skipped."""
    import torch

    best, best_us, tried = None, float("inf"), 0
    for plan in candidates:
        try:
            for _ in range(warmup):
                launch(plan)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                launch(plan)
            e1.record()
            e1.synchronize()
        except RuntimeError as exc:
            logger.debug("candidate plan rejected: %r", exc)
            continue
        tried += 1
        us = e0.elapsed_time(e1) * 1e3 / iters
        if us < best_us:
            best, best_us = plan, us
    return best, best_us, tried
