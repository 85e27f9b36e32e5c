"""GPU: the path a kernel takes when one of its bounded device-side waits runs out.

Nothing here faults, traps or hangs the GPU.  A test hook of the library (sfb_debug_wait_timeout) shortens the time
limit of one wait from 2 s to 20 ms and tells the correlation sweep's producer to leave out the last block it would
load, on a problem of ONE CTA.  The tensor-core issuer then waits for a block that never comes; its wait runs out,
it writes its code to the status word, the other roles of the CTA see the abort flag and leave their loops, tensor
memory is freed and the kernel returns by itself.  The host reads the status word (SFB_ERR_DEVICE_TIMEOUT), and
the next ordinary call on the same workspace must pass its parity check: the context stays usable.
"""
import ctypes

import pytest
import torch

from separableflowthesis_b200 import _lib, ops
from oracle import separation_oracle as orc

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_sets_the_status_word_and_the_next_call_works(cuda_device):
    lib = _lib.load()
    dev = cuda_device
    g = torch.Generator().manual_seed(3)
    B, H1, W1, H2, W2, C = 1, 8, 12, 8, 12, 32          # 96 image-1 pixels: one CTA, one correlation tile + the mean tile
    F1 = (torch.randn(B, H1, W1, C, generator=g) / C ** 0.5).to(dev)
    F2 = torch.randn(B, H2, W2, C, generator=g).to(dev)
    shape = _lib.SfbShape(B, H1, W1, H2, W2, C, 0)
    nbytes = lib.sfb_workspace_bytes(_lib.OP_MAX_AVG_FORWARD, ctypes.byref(shape))
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    MA_u = torch.empty(B, H1, W1, 2, H2, device=dev)
    MA_v = torch.empty(B, H1, W1, 2, W2, device=dev)
    P = ctypes.c_void_p
    stream = torch.cuda.current_stream(dev).cuda_stream

    def call():
        return lib.sfb_max_avg_forward(P(F1.data_ptr()), P(F2.data_ptr()), P(MA_u.data_ptr()), P(MA_v.data_ptr()),
                                       ctypes.byref(shape), P(ws.data_ptr()), ctypes.c_size_t(nbytes), P(stream))

    status = ctypes.c_int32(0)
    try:
        assert lib.sfb_debug_wait_timeout(20_000_000, 1) == _lib.SFB_OK     # 20 ms per wait, last load left out
        assert call() == _lib.SFB_OK                                       # the launch itself succeeds
        rc = lib.sfb_device_status(P(ws.data_ptr()), P(stream), ctypes.byref(status))
    finally:
        lib.sfb_debug_wait_timeout(0, 0)
    assert rc == _lib.SFB_ERR_DEVICE_TIMEOUT
    assert status.value in (102, 103)            # the MMA issuer's wait ran out (or the epilogue's, first one wins)
    assert b"bounded device-side wait" in lib.sfb_last_error()
    torch.cuda.synchronize()                     # no sticky CUDA error: the kernel returned normally

    # normal operation on the same workspace: status cleared by the call, results within tolerance of the oracle
    assert call() == _lib.SFB_OK
    assert lib.sfb_device_status(P(ws.data_ptr()), P(stream), ctypes.byref(status)) == _lib.SFB_OK
    assert status.value == 0
    r_u, r_v = orc.max_avg_forward(F1.double().cpu(), F2.double().cpu())
    for x, r in ((MA_u, r_u), (MA_v, r_v)):
        err = (x.double().cpu() - r).abs().max().item() / r.abs().max().item()
        assert err < 1e-3, err
    # and through the Python layer
    u2, v2 = ops.max_avg_forward(F1, F2)
    assert torch.equal(u2, MA_u) and torch.equal(v2, MA_v)
