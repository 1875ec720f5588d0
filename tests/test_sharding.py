"""Row sharding across ranks, exercised with two ``gloo`` processes on CPU: the partition, the
scalar all-reduce and the end-to-end equivalence "sharded + combined == unsharded"."""
from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fuseml_b200.sharding import RowShardedModule, allreduce_scalars, row_range, shard_rows


def test_row_range_partitions_exactly():
    for M in (0, 1, 7, 128, 8192, 32768 + 5):
        for world in (1, 2, 3, 8):
            spans = [row_range(M, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == M
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        row_range(10, 2, 2)


def test_single_process_is_a_no_op():
    s, m = allreduce_scalars(torch.tensor(3.0), torch.tensor(5.0))
    assert float(s) == 3.0 and float(m) == 5.0
    x = torch.arange(12.0).reshape(6, 2)
    assert torch.equal(shard_rows(x, 3, 1), x[2:4])


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import configs

        case = configs.make("cfg5", small=True)
        x = case.args[0]
        stack = case.module

        def fn(x_local):
            with torch.no_grad():
                y, _, _ = stack(x_local)
            return y, y.sum(), y.amax(), y.mean()

        runner = RowShardedModule(fn, reductions=("sum", "max", "mean"))
        y, s, m, mean = runner(shard_rows(x, world, rank), global_rows=x.shape[0])
        results[rank] = (row_range(x.shape[0], world, rank), y, float(s), float(m), float(mean))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_matches_unsharded():
    from oracle import configs

    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    case = configs.make("cfg5", small=True)
    with torch.no_grad():
        y_ref, s_ref, m_ref = case.module(*case.args)
    rows = torch.empty_like(y_ref)
    for rank in range(world):
        (a, b), y, s, m, mean = results[rank]
        rows[a:b] = y
        # every rank holds the same combined scalars
        assert abs(s - float(s_ref)) <= 1e-4 * abs(float(s_ref)) + 1e-3
        assert m == pytest.approx(float(m_ref), rel=1e-6)
        assert mean == pytest.approx(float(y_ref.mean()), rel=1e-4, abs=1e-6)
    assert torch.allclose(rows, y_ref, rtol=1e-5, atol=1e-5)


def test_numa_binding_uses_nvml_mask_and_respects_allowed_cores(monkeypatch):
    """bind_to_device_numa against a fake NVML: the mask is intersected with the cores this
    process may use; an empty intersection or a failing NVML leaves the affinity alone."""
    import os
    import types

    from fuseml_b200 import sharding

    if not hasattr(os, "sched_setaffinity"):
        pytest.skip("no sched_setaffinity on this platform")
    allowed = sorted(os.sched_getaffinity(0))
    calls = []
    monkeypatch.setattr(os, "sched_setaffinity", lambda pid, cpus: calls.append((pid, sorted(cpus))))
    props = types.SimpleNamespace(pci_domain_id=0, pci_bus_id=0x1b, pci_device_id=0)
    monkeypatch.setattr(sharding.torch.cuda, "get_device_properties", lambda i: props)

    def fake(mask_words, seen):
        def by_bus(b):
            seen.append(b)
            return "h"
        return types.SimpleNamespace(nvmlInit=lambda: None, nvmlDeviceGetHandleByPciBusId=by_bus,
                                     nvmlDeviceGetCpuAffinity=lambda h, n: mask_words[:n] + [0] * max(0, n - len(mask_words)))

    seen: list = []
    want = allowed[: max(1, len(allowed) // 2)]
    words = [0] * ((max(allowed) // 64) + 1)
    for c in want:
        words[c // 64] |= 1 << (c % 64)
    got = sharding.bind_to_device_numa(0, nvml=fake(words, seen))
    assert got == want and seen == [b"00000000:1b:00.0"]
    if len(want) < len(allowed):
        assert calls == [(0, want)]
    # cores outside the allowed set only: nothing changes
    calls.clear()
    far = [0] * ((max(allowed) // 64) + 2)
    far[-1] = 1 << 63
    assert sharding.bind_to_device_numa(0, nvml=fake(far, seen)) is None and calls == []
    # NVML raising: nothing changes
    broken = types.SimpleNamespace(nvmlInit=lambda: (_ for _ in ()).throw(RuntimeError("no driver")))
    assert sharding.bind_to_device_numa(0, nvml=broken) is None and calls == []
