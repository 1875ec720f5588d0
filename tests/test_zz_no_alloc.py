"""The allocation-free entry point, ``fuseml_sm100_gemm_epilogue_noalloc``.

Who needs it: callers that are not allowed to allocate device memory at launch time —
code running while another framework holds its memory pool locked, plugins given a
fixed memory budget when they were loaded, serving loops that must never hit an
allocator.  Their reduction scratch comes from an 8 MiB array compiled into the
library instead of a workspace tensor.

The test drives the entry point through the C ABI exactly as such a caller would
(inputs and outputs are ordinary buffers, no workspace is passed) and compares with the
regular entry point on the same inputs, on two calls in a row: the second call reuses
the scratch array with the first call's leftovers in it.  The file name sorts last so
that a run stopping at the first failure has already executed every other test.
"""
from __future__ import annotations

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _launch(lib, N, K, entry, a, b, out_max, out_mean, workspace=None):
    desc = N.GemmDesc()
    prog = K.EpilogueProgram().relu()
    K.fill_desc(desc, a, b, prog, None, torch.bfloat16)
    desc.reduce.kinds = N.RED_MAX | N.RED_MEAN
    desc.reduce.axis = N.AXIS_N
    desc.reduce.out_max = out_max.data_ptr()
    desc.reduce.out_mean = out_mean.data_ptr()
    plan = K.plan_for(desc, K.device_props())
    if workspace is not None:
        desc.reduce.workspace = workspace.data_ptr()
        desc.reduce.workspace_bytes = workspace.numel()
    stream = torch.cuda.current_stream().cuda_stream
    rc = getattr(lib, entry)(C.byref(desc), C.byref(plan), C.c_void_p(stream))
    return rc, desc, plan


def test_noalloc_entry_matches_regular_entry_twice(native_lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from fuseml_b200 import _native as N, kernels as K

    lib = native_lib
    assert lib.fuseml_sm100_noalloc_scratch_bytes() == 8 << 20
    g = torch.Generator().manual_seed(123)
    M, Kd, Nn = 1000, 520, 1304          # ragged on every side; 6 column tiles of partials
    for call in range(2):
        a = torch.randn(M, Kd, generator=g).to(torch.bfloat16).cuda()
        b = (torch.randn(Kd, Nn, generator=g) / Kd ** 0.5).to(torch.bfloat16).cuda()
        ref_max = torch.empty(M, dtype=torch.float32, device="cuda")
        ref_mean = torch.empty(M, dtype=torch.float32, device="cuda")
        got_max = torch.full((M,), float("nan"), dtype=torch.float32, device="cuda")
        got_mean = torch.full((M,), float("nan"), dtype=torch.float32, device="cuda")

        # regular entry point, caller-provided workspace
        ws = torch.empty(1 << 20, dtype=torch.uint8, device="cuda")
        rc, _, _ = _launch(lib, N, K, "fuseml_sm100_gemm_epilogue", a, b, ref_max, ref_mean, ws)
        assert rc == N.OK, N.strerror(rc)

        # allocation-free entry point: no workspace at all
        before = torch.cuda.memory_allocated()
        rc, _, _ = _launch(lib, N, K, "fuseml_sm100_gemm_epilogue_noalloc", a, b, got_max, got_mean)
        assert rc == N.OK, N.strerror(rc)
        assert torch.cuda.memory_allocated() == before
        torch.cuda.synchronize()
        assert K.device_status() == 0

        # same kernel, same tiling, same partial order: identical results; the stated
        # tolerance of the reduction tests (1e-3 relative) is the bound that matters
        scale = ref_mean.abs().max().item()
        assert (got_mean - ref_mean).abs().max().item() <= 1e-3 * scale, f"call {call}"
        assert (got_max - ref_max).abs().max().item() <= 1e-3 * ref_max.abs().max().item(), f"call {call}"
        # and both agree with PyTorch on the same inputs
        c = torch.relu(a.float() @ b.float())
        assert (got_max - c.amax(-1)).abs().max().item() <= 1e-3 * c.amax().item()
        assert (got_mean - c.mean(-1)).abs().max().item() <= 1e-3 * scale


def test_noalloc_entry_rejects_oversized_scratch(native_lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from fuseml_b200 import _native as N, kernels as K

    # 65536 rows x 64 column tiles x 4 bytes = 16 MiB of partials: beyond the 8 MiB array
    M, Kd, Nn = 65536, 64, 16384
    a = torch.zeros(M, Kd, dtype=torch.bfloat16, device="cuda")
    b = torch.zeros(Kd, Nn, dtype=torch.bfloat16, device="cuda")
    o1 = torch.zeros(M, dtype=torch.float32, device="cuda")
    o2 = torch.zeros(M, dtype=torch.float32, device="cuda")
    rc, _, _ = _launch(native_lib, N, K, "fuseml_sm100_gemm_epilogue_noalloc", a, b, o1, o2)
    assert rc == N.E_LIMIT
    assert "maximum" in N.strerror(rc)
