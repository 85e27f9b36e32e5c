"""GPU: the entry point for callers that cannot allocate device memory (sfb_max_avg_forward_static).

Some users of this library run where cudaMalloc is off limits: inside a CUDA-graph capture, inside a
serving loop whose memory is owned by another pool, or in a host application that only passes input and
output buffers.  For them the library carries its own fixed scratch array.  This file (collected last)
calls that entry point through the C ABI, twice in a row on different data, and checks both results
bit for bit against the ordinary entry point, which uses a caller-provided workspace, and against the
float64 oracle; after each call it reads the device status word of the built-in scratch.  It also checks
that a shape too large for the built-in scratch is refused with a clear message.
"""
import ctypes

import pytest
import torch

from separableflowthesis_b200 import _lib, ops
from oracle import separation_oracle as orc

pytestmark = pytest.mark.gpu


def _call_static(lib, F1, F2):
    B, H1, W1, C = F1.shape
    _, H2, W2, _ = F2.shape
    shape = _lib.SfbShape(B, H1, W1, H2, W2, C, 0)
    MA_u = torch.empty(B, H1, W1, 2, H2, dtype=torch.float32, device=F1.device)
    MA_v = torch.empty(B, H1, W1, 2, W2, dtype=torch.float32, device=F1.device)
    stream = torch.cuda.current_stream(F1.device).cuda_stream
    P = ctypes.c_void_p
    rc = lib.sfb_max_avg_forward_static(P(F1.data_ptr()), P(F2.data_ptr()), P(MA_u.data_ptr()), P(MA_v.data_ptr()),
                                        ctypes.byref(shape), P(stream))
    return rc, MA_u, MA_v


def test_static_scratch_entry_point_matches_workspace_entry_point(cuda_device):
    lib = _lib.load()
    assert lib.sfb_static_scratch_bytes() == 32 << 20
    g = torch.Generator().manual_seed(2024)
    # two calls in a row with different sizes and data: the second must not see anything of the first
    for (B, H1, W1, H2, W2, C) in ((1, 48, 64, 48, 64, 256), (2, 21, 37, 10, 18, 64)):
        F1 = (torch.randn(B, H1, W1, C, generator=g) / C ** 0.5).to(cuda_device)
        F2 = torch.randn(B, H2, W2, C, generator=g).to(cuda_device)
        rc, MA_u, MA_v = _call_static(lib, F1, F2)
        assert rc == _lib.SFB_OK, lib.sfb_last_error()
        # no bounded device-side wait gave up: the status word of the built-in scratch is 0
        status = ctypes.c_int32(-1)
        stream = torch.cuda.current_stream(cuda_device).cuda_stream
        assert lib.sfb_static_device_status(ctypes.c_void_p(stream), ctypes.byref(status)) == _lib.SFB_OK
        assert status.value == 0
        with ops.sweep_operands("tf32"):   # the static entry point always computes with TF32 operands
            ref_u, ref_v = ops.max_avg_forward(F1, F2)
        torch.cuda.synchronize()
        # same kernels, same arithmetic: identical bits (tolerance of the other GPU tests: 1e-3 relative)
        assert torch.equal(MA_u, ref_u) and torch.equal(MA_v, ref_v)
        # and both within the TF32 tolerance of the float64 oracle
        o_u, o_v = orc.max_avg_forward(F1.double().cpu(), F2.double().cpu())
        for x, r in ((MA_u, o_u), (MA_v, o_v)):
            err = (x.double().cpu() - r).abs().max().item() / max(r.abs().max().item(), 1e-30)
            assert err < 1e-3, err


def test_static_scratch_rejects_shapes_that_do_not_fit(cuda_device):
    lib = _lib.load()
    F = torch.zeros(1, 135, 240, 256, device=cuda_device)  # needs far more than 32 MiB of scratch
    rc, _, _ = _call_static(lib, F, F)
    assert rc == _lib.SFB_ERR_UNSUPPORTED_SHAPE
    assert b"built-in scratch" in lib.sfb_last_error()
