"""The five native ops, under the names and signatures of the reference's pybind11 module
``MemorySaver`` (libs/MemorySaver/src/MemorySaver_cuda.cpp:105-112): tensors in, a list of freshly
allocated tensors out.  Each function validates its inputs the way the reference's CHECK_INPUT does
(CUDA + contiguous, MemorySaver_cuda.cpp:6-8; plus the shape/dtype checks the reference lacks),
allocates the outputs and calls the C ABI of ``libsepflow_b200.so`` on the current CUDA stream.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Dict, List, Tuple

import torch

from . import _lib

# Scratch buffers handed to the library, one per (device, stream): calls that share a workspace must be ordered on
# one stream.  A buffer grows to the largest size asked for and is kept for reuse (7.5 GB for a level backward of
# B=8, 135x240, Kc=4); release_workspaces() drops them.  The lock covers DataParallel-style callers that run the ops
# from several threads.
_workspaces: Dict[Tuple[int, int], torch.Tensor] = {}
_workspaces_lock = threading.Lock()


def _check(t: torch.Tensor, name: str, dtype: torch.dtype, ndim: int) -> None:
    if not isinstance(t, torch.Tensor):
        raise RuntimeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if t.dtype != dtype:
        raise RuntimeError(f"{name} must have dtype {dtype}, got {t.dtype}")
    if t.dim() != ndim:
        raise RuntimeError(f"{name} must have {ndim} dimensions, got {t.dim()}")


def _check_pair(F1: torch.Tensor, F2: torch.Tensor) -> _lib.SfbShape:
    _check(F1, "img1_features_l0", torch.float32, 4)
    _check(F2, "img2_features_lk", torch.float32, 4)
    if F1.device != F2.device:
        raise RuntimeError("img1_features_l0 and img2_features_lk must be on the same device")
    if F1.shape[0] != F2.shape[0] or F1.shape[3] != F2.shape[3]:
        raise RuntimeError(f"batch / feature dimensions differ: {tuple(F1.shape)} vs {tuple(F2.shape)}")
    B, H1, W1, C = F1.shape
    _, H2, W2, _ = F2.shape
    return _lib.SfbShape(B, H1, W1, H2, W2, C, 0)


def _check_like(t: torch.Tensor, name: str, shape, dtype, device) -> None:
    _check(t, name, dtype, len(shape))
    if tuple(t.shape) != tuple(shape):
        raise RuntimeError(f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")
    if t.device != device:
        raise RuntimeError(f"{name} is on {t.device}, expected {device}")


def _workspace(nbytes: int, device: torch.device, stream: int) -> torch.Tensor:
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream)
    with _workspaces_lock:
        ws = _workspaces.get(key)
        if ws is None or ws.numel() < nbytes:
            ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
            _workspaces[key] = ws
        return ws


def release_workspaces(device=None) -> int:
    """Drop the cached scratch buffers (of one device, or of all) and return the bytes released to torch's
    allocator.  Work already enqueued keeps its buffer alive through torch's stream-ordered allocator only if the
    caller synchronises first: call this between steps, not while ops are in flight."""
    index = None if device is None else torch.device(device).index
    freed = 0
    with _workspaces_lock:
        for key in [k for k in _workspaces if index is None or k[0] == index]:
            freed += _workspaces.pop(key).numel()
    return freed


def _ptr(t):
    if isinstance(t, float):
        return ctypes.c_float(t)
    if isinstance(t, int):
        return ctypes.c_int32(t)
    return ctypes.c_void_p(t.data_ptr() if t is not None else None)


def _call(name: str, op: int, shape: _lib.SfbShape, device: torch.device, tensors) -> None:
    lib = _lib.load()
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream(device).cuda_stream
        nbytes = lib.sfb_workspace_bytes(op, ctypes.byref(shape))
        if nbytes == 0:
            # run the entry point anyway so that the library reports the precise reason
            nbytes = 256
        ws = _workspace(nbytes, device, stream)
        rc = getattr(lib, name)(*[_ptr(t) for t in tensors], ctypes.byref(shape),
                                ctypes.c_void_p(ws.data_ptr()), ctypes.c_size_t(ws.numel()),
                                ctypes.c_void_p(stream))
        if rc != _lib.SFB_OK:
            raise RuntimeError(f"{name}: {lib.sfb_status_string(rc).decode()}: {lib.sfb_last_error().decode()}")
        if os.environ.get("SFB_CHECK_DEVICE_STATUS", "0") == "1":
            dev_status = ctypes.c_int32(0)
            rc = lib.sfb_device_status(ctypes.c_void_p(ws.data_ptr()), ctypes.c_void_p(stream),
                                       ctypes.byref(dev_status))
            if rc != _lib.SFB_OK:
                raise RuntimeError(f"{name}: {lib.sfb_last_error().decode()}")


def max_avg_forward(img1_features_l0: torch.Tensor, img2_features_lk: torch.Tensor) -> List[torch.Tensor]:
    """MemorySaver.max_avg_forward (MemorySaver_cuda.cpp:10-21): returns [MA_u, MA_v]."""
    F1, F2 = img1_features_l0, img2_features_lk
    s = _check_pair(F1, F2)
    MA_u = torch.empty(s.B, s.H1, s.W1, 2, s.H2, dtype=torch.float32, device=F1.device)
    MA_v = torch.empty(s.B, s.H1, s.W1, 2, s.W2, dtype=torch.float32, device=F1.device)
    _call("sfb_max_avg_forward", _lib.OP_MAX_AVG_FORWARD, s, F1.device, (F1, F2, MA_u, MA_v))
    return [MA_u, MA_v]


def max_argmax_avg_forward(img1_features_l0: torch.Tensor, img2_features_lk: torch.Tensor) -> List[torch.Tensor]:
    """MemorySaver.max_argmax_avg_forward (MemorySaver_cuda.cpp:23-34): returns [MA_u, MA_v, AM_u, AM_v]."""
    F1, F2 = img1_features_l0, img2_features_lk
    s = _check_pair(F1, F2)
    MA_u = torch.empty(s.B, s.H1, s.W1, 2, s.H2, dtype=torch.float32, device=F1.device)
    MA_v = torch.empty(s.B, s.H1, s.W1, 2, s.W2, dtype=torch.float32, device=F1.device)
    AM_u = torch.empty(s.B, s.H1, s.W1, 1, s.H2, dtype=torch.int32, device=F1.device)
    AM_v = torch.empty(s.B, s.H1, s.W1, 1, s.W2, dtype=torch.int32, device=F1.device)
    _call("sfb_max_argmax_avg_forward", _lib.OP_MAX_AVG_FORWARD, s, F1.device, (F1, F2, MA_u, MA_v, AM_u, AM_v))
    return [MA_u, MA_v, AM_u, AM_v]


def max_argmax_avg_backward(img1_features_l0, img2_features_lk, argmax_output_u, argmax_output_v,
                            grad_MaxAvg_u, grad_MaxAvg_v) -> List[torch.Tensor]:
    """MemorySaver.max_argmax_avg_backward (MemorySaver_cuda.cpp:55-78): returns [gF1, gF2]."""
    F1, F2 = img1_features_l0, img2_features_lk
    s = _check_pair(F1, F2)
    dev = F1.device
    _check_like(argmax_output_u, "argmax_output_u", (s.B, s.H1, s.W1, 1, s.H2), torch.int32, dev)
    _check_like(argmax_output_v, "argmax_output_v", (s.B, s.H1, s.W1, 1, s.W2), torch.int32, dev)
    _check_like(grad_MaxAvg_u, "grad_MaxAvg_u", (s.B, s.H1, s.W1, 2, s.H2), torch.float32, dev)
    _check_like(grad_MaxAvg_v, "grad_MaxAvg_v", (s.B, s.H1, s.W1, 2, s.W2), torch.float32, dev)
    gF1 = torch.empty_like(F1)
    gF2 = torch.empty_like(F2)
    _call("sfb_max_argmax_avg_backward", _lib.OP_MAX_ARGMAX_AVG_BACKWARD, s, dev,
          (F1, F2, argmax_output_u, argmax_output_v, grad_MaxAvg_u, grad_MaxAvg_v, gF1, gF2))
    return [gF1, gF2]


def _check_attention(s: _lib.SfbShape, A_u, A_v, dev, names=("attention_weights_u", "attention_weights_v")):
    _check(A_u, names[0], torch.float32, 5)
    s.Kc = A_u.shape[3]
    _check_like(A_u, names[0], (s.B, s.H1, s.W1, s.Kc, s.W2), torch.float32, dev)
    _check_like(A_v, names[1], (s.B, s.H1, s.W1, s.Kc, s.H2), torch.float32, dev)
    if s.Kc < 1:
        raise RuntimeError("attention weights need at least one channel")


def compression_forward(img1_features_l0, img2_features_lk, attention_weights_u, attention_weights_v) -> List[torch.Tensor]:
    """MemorySaver.compression_forward (MemorySaver_cuda.cpp:36-53), any Kc >= 1: returns [C_u, C_v]."""
    F1, F2 = img1_features_l0, img2_features_lk
    s = _check_pair(F1, F2)
    dev = F1.device
    _check_attention(s, attention_weights_u, attention_weights_v, dev)
    C_u = torch.empty(s.B, s.H1, s.W1, s.Kc, s.H2, dtype=torch.float32, device=dev)
    C_v = torch.empty(s.B, s.H1, s.W1, s.Kc, s.W2, dtype=torch.float32, device=dev)
    _call("sfb_compression_forward", _lib.OP_COMPRESSION_FORWARD, s, dev,
          (F1, F2, attention_weights_u, attention_weights_v, C_u, C_v))
    return [C_u, C_v]


def compression_backward(img1_features_l0, img2_features_lk, attention_weights_u, attention_weights_v,
                         grad_compressed_output_u, grad_compressed_output_v) -> List[torch.Tensor]:
    """MemorySaver.compression_backward (MemorySaver_cuda.cpp:80-103): returns [gF1, gF2, gA_u, gA_v]."""
    F1, F2 = img1_features_l0, img2_features_lk
    s = _check_pair(F1, F2)
    dev = F1.device
    _check_attention(s, attention_weights_u, attention_weights_v, dev)
    _check_like(grad_compressed_output_u, "grad_compressed_output_u", (s.B, s.H1, s.W1, s.Kc, s.H2), torch.float32, dev)
    _check_like(grad_compressed_output_v, "grad_compressed_output_v", (s.B, s.H1, s.W1, s.Kc, s.W2), torch.float32, dev)
    gF1 = torch.empty_like(F1)
    gF2 = torch.empty_like(F2)
    gA_u = torch.empty_like(attention_weights_u)
    gA_v = torch.empty_like(attention_weights_v)
    _call("sfb_compression_backward", _lib.OP_COMPRESSION_BACKWARD, s, dev,
          (F1, F2, attention_weights_u, attention_weights_v, grad_compressed_output_u, grad_compressed_output_v,
           gF1, gF2, gA_u, gA_v))
    return [gF1, gF2, gA_u, gA_v]


def separation_backward(img1_features_l0, img2_features_lk, argmax_output_u, argmax_output_v, grad_MaxAvg_u,
                        grad_MaxAvg_v, attention_weights_u, attention_weights_v, grad_compressed_output_u,
                        grad_compressed_output_v) -> List[torch.Tensor]:
    """Both backward ops in one call (no counterpart in the reference's module): returns
    [gF1, gF2, gA_u, gA_v] with gF1/gF2 the sum of what max_argmax_avg_backward and compression_backward
    return, computed with one pair of gradient GEMMs."""
    F1, F2 = img1_features_l0, img2_features_lk
    s = _check_pair(F1, F2)
    dev = F1.device
    _check_attention(s, attention_weights_u, attention_weights_v, dev)
    _check_like(argmax_output_u, "argmax_output_u", (s.B, s.H1, s.W1, 1, s.H2), torch.int32, dev)
    _check_like(argmax_output_v, "argmax_output_v", (s.B, s.H1, s.W1, 1, s.W2), torch.int32, dev)
    _check_like(grad_MaxAvg_u, "grad_MaxAvg_u", (s.B, s.H1, s.W1, 2, s.H2), torch.float32, dev)
    _check_like(grad_MaxAvg_v, "grad_MaxAvg_v", (s.B, s.H1, s.W1, 2, s.W2), torch.float32, dev)
    _check_like(grad_compressed_output_u, "grad_compressed_output_u", (s.B, s.H1, s.W1, s.Kc, s.H2), torch.float32, dev)
    _check_like(grad_compressed_output_v, "grad_compressed_output_v", (s.B, s.H1, s.W1, s.Kc, s.W2), torch.float32, dev)
    gF1 = torch.empty_like(F1)
    gF2 = torch.empty_like(F2)
    gA_u = torch.empty_like(attention_weights_u)
    gA_v = torch.empty_like(attention_weights_v)
    _call("sfb_separation_backward", _lib.OP_SEPARATION_BACKWARD, s, dev,
          (F1, F2, argmax_output_u, argmax_output_v, grad_MaxAvg_u, grad_MaxAvg_v, attention_weights_u,
           attention_weights_v, grad_compressed_output_u, grad_compressed_output_v, gF1, gF2, gA_u, gA_v))
    return [gF1, gF2, gA_u, gA_v]


def compression_attention_backward(img1_features_l0, img2_features_lk, grad_compressed_output_u,
                                   grad_compressed_output_v) -> List[torch.Tensor]:
    """First half of separation_backward: [gA_u, gA_v] only."""
    F1, F2 = img1_features_l0, img2_features_lk
    s = _check_pair(F1, F2)
    dev = F1.device
    _check(grad_compressed_output_u, "grad_compressed_output_u", torch.float32, 5)
    s.Kc = grad_compressed_output_u.shape[3]
    _check_like(grad_compressed_output_u, "grad_compressed_output_u", (s.B, s.H1, s.W1, s.Kc, s.H2), torch.float32, dev)
    _check_like(grad_compressed_output_v, "grad_compressed_output_v", (s.B, s.H1, s.W1, s.Kc, s.W2), torch.float32, dev)
    gA_u = torch.empty(s.B, s.H1, s.W1, s.Kc, s.W2, dtype=torch.float32, device=dev)
    gA_v = torch.empty(s.B, s.H1, s.W1, s.Kc, s.H2, dtype=torch.float32, device=dev)
    _call("sfb_compression_attention_backward", _lib.OP_COMPRESSION_FORWARD, s, dev,
          (F1, F2, grad_compressed_output_u, grad_compressed_output_v, gA_u, gA_v))
    return [gA_u, gA_v]


def separation_feature_backward(img1_features_l0, img2_features_lk, argmax_output_u, argmax_output_v,
                                grad_MaxAvg_u, grad_MaxAvg_v, attention_weights_u, attention_weights_v,
                                grad_compressed_output_u, grad_compressed_output_v) -> List[torch.Tensor]:
    """Second half of separation_backward: [gF1, gF2], the summed feature gradients of both backward ops."""
    F1, F2 = img1_features_l0, img2_features_lk
    s = _check_pair(F1, F2)
    dev = F1.device
    _check_attention(s, attention_weights_u, attention_weights_v, dev)
    _check_like(argmax_output_u, "argmax_output_u", (s.B, s.H1, s.W1, 1, s.H2), torch.int32, dev)
    _check_like(argmax_output_v, "argmax_output_v", (s.B, s.H1, s.W1, 1, s.W2), torch.int32, dev)
    _check_like(grad_MaxAvg_u, "grad_MaxAvg_u", (s.B, s.H1, s.W1, 2, s.H2), torch.float32, dev)
    _check_like(grad_MaxAvg_v, "grad_MaxAvg_v", (s.B, s.H1, s.W1, 2, s.W2), torch.float32, dev)
    _check_like(grad_compressed_output_u, "grad_compressed_output_u", (s.B, s.H1, s.W1, s.Kc, s.H2), torch.float32, dev)
    _check_like(grad_compressed_output_v, "grad_compressed_output_v", (s.B, s.H1, s.W1, s.Kc, s.W2), torch.float32, dev)
    gF1 = torch.empty_like(F1)
    gF2 = torch.empty_like(F2)
    _call("sfb_separation_feature_backward", _lib.OP_SEPARATION_BACKWARD, s, dev,
          (F1, F2, argmax_output_u, argmax_output_v, grad_MaxAvg_u, grad_MaxAvg_v, attention_weights_u,
           attention_weights_v, grad_compressed_output_u, grad_compressed_output_v, gF1, gF2))
    return [gF1, gF2]


# ------------------------------------------------------------------------------------------------------
# Channels-first variants (no counterpart in the reference's module): the tensors have the layout the
# call site feeds to / gets from its Conv3d modules, (B, K, D, H1, W1), so it needs no permute copies.
def max_argmax_avg_forward_cf(img1_features_l0, img2_features_lk, with_argmax=True) -> List[torch.Tensor]:
    """[sep_v (B,2,H2,H1,W1), sep_u (B,2,W2,H1,W1), AM_u (B,H2,H1,W1), AM_v (B,W2,H1,W1)]: channel 0 = max,
    1 = mean; sep_v holds the per-u channels (the reference's maxavg_u permuted, core/corr.py:428-429)."""
    F1, F2 = img1_features_l0, img2_features_lk
    s = _check_pair(F1, F2)
    dev = F1.device
    sep_v = torch.empty(s.B, 2, s.H2, s.H1, s.W1, dtype=torch.float32, device=dev)
    sep_u = torch.empty(s.B, 2, s.W2, s.H1, s.W1, dtype=torch.float32, device=dev)
    am_u = torch.empty(s.B, s.H2, s.H1, s.W1, dtype=torch.int32, device=dev) if with_argmax else None
    am_v = torch.empty(s.B, s.W2, s.H1, s.W1, dtype=torch.int32, device=dev) if with_argmax else None
    _call("sfb_max_argmax_avg_forward_cf", _lib.OP_MAX_AVG_FORWARD_CF, s, dev, (F1, F2, sep_v, sep_u, am_u, am_v))
    return [sep_v, sep_u, am_u, am_v]


def _check_attention_cf(s, a_u, a_v, dev, names=("attention_weights_u", "attention_weights_v")):
    _check(a_u, names[0], torch.float32, 5)
    s.Kc = a_u.shape[1]
    _check_like(a_u, names[0], (s.B, s.Kc, s.W2, s.H1, s.W1), torch.float32, dev)
    _check_like(a_v, names[1], (s.B, s.Kc, s.H2, s.H1, s.W1), torch.float32, dev)
    if s.Kc < 1:
        raise RuntimeError("attention weights need at least one channel")


def compression_forward_cf(img1_features_l0, img2_features_lk, a_u, a_v) -> List[torch.Tensor]:
    """a_u (B,Kc,W2,H1,W1), a_v (B,Kc,H2,H1,W1) -> [c_u (B,Kc,H2,H1,W1), c_v (B,Kc,W2,H1,W1)]."""
    F1, F2 = img1_features_l0, img2_features_lk
    s = _check_pair(F1, F2)
    dev = F1.device
    _check_attention_cf(s, a_u, a_v, dev)
    c_u = torch.empty(s.B, s.Kc, s.H2, s.H1, s.W1, dtype=torch.float32, device=dev)
    c_v = torch.empty(s.B, s.Kc, s.W2, s.H1, s.W1, dtype=torch.float32, device=dev)
    _call("sfb_compression_forward_cf", _lib.OP_COMPRESSION_CF, s, dev, (F1, F2, a_u, a_v, c_u, c_v))
    return [c_u, c_v]


def compression_attention_backward_cf(img1_features_l0, img2_features_lk, gc_u, gc_v) -> List[torch.Tensor]:
    """gc_u (B,Kc,H2,H1,W1), gc_v (B,Kc,W2,H1,W1) -> [ga_u (B,Kc,W2,H1,W1), ga_v (B,Kc,H2,H1,W1)]."""
    F1, F2 = img1_features_l0, img2_features_lk
    s = _check_pair(F1, F2)
    dev = F1.device
    _check_attention_cf(s, gc_v, gc_u, dev, ("grad_compressed_output_v", "grad_compressed_output_u"))
    ga_u = torch.empty(s.B, s.Kc, s.W2, s.H1, s.W1, dtype=torch.float32, device=dev)
    ga_v = torch.empty(s.B, s.Kc, s.H2, s.H1, s.W1, dtype=torch.float32, device=dev)
    _call("sfb_compression_attention_backward_cf", _lib.OP_COMPRESSION_CF, s, dev, (F1, F2, gc_u, gc_v, ga_u, ga_v))
    return [ga_u, ga_v]


def separation_feature_backward_cf(img1_features_l0, img2_features_lk, am_u, am_v, g_sep_v, g_sep_u, a_u, a_v,
                                   gc_u, gc_v) -> List[torch.Tensor]:
    """[gF1, gF2] summed over the max/avg and the compression node, all per-pixel tensors channels-first."""
    F1, F2 = img1_features_l0, img2_features_lk
    s = _check_pair(F1, F2)
    dev = F1.device
    _check_attention_cf(s, a_u, a_v, dev)
    _check_like(am_u, "argmax_u", (s.B, s.H2, s.H1, s.W1), torch.int32, dev)
    _check_like(am_v, "argmax_v", (s.B, s.W2, s.H1, s.W1), torch.int32, dev)
    _check_like(g_sep_v, "grad_sep_v", (s.B, 2, s.H2, s.H1, s.W1), torch.float32, dev)
    _check_like(g_sep_u, "grad_sep_u", (s.B, 2, s.W2, s.H1, s.W1), torch.float32, dev)
    _check_like(gc_u, "grad_c_u", (s.B, s.Kc, s.H2, s.H1, s.W1), torch.float32, dev)
    _check_like(gc_v, "grad_c_v", (s.B, s.Kc, s.W2, s.H1, s.W1), torch.float32, dev)
    gF1 = torch.empty_like(F1)
    gF2 = torch.empty_like(F2)
    _call("sfb_separation_feature_backward_cf", _lib.OP_SEPARATION_FEATURE_BACKWARD_CF, s, dev,
          (F1, F2, am_u, am_v, g_sep_v, g_sep_u, a_u, a_v, gc_u, gc_v, gF1, gF2))
    return [gF1, gF2]


# ------------------------------------------------------------------------------------------------------
# Attention weights of the call site and the whole level in one call (no counterpart in the reference's
# module; the reference runs torch's Conv3d and softmax between its ops, core/corr.py:437-442).
def _check_attention_params(weight, bias, name, dev):
    _check(weight, name + ".weight", torch.float32, 5)
    Kc = weight.shape[0]
    _check_like(weight, name + ".weight", (Kc, 2, 3, 3, 3), torch.float32, dev)
    _check_like(bias, name + ".bias", (Kc,), torch.float32, dev)
    return Kc


def _raise_on(rc, name):
    if rc != _lib.SFB_OK:
        lib = _lib.load()
        raise RuntimeError(f"{name}: {lib.sfb_status_string(rc).decode()}: {lib.sfb_last_error().decode()}")


def attention_forward(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """softmax(Conv3d(2 -> Kc, 3, padding=1)(x), dim=2) for x (B,2,D,H1,W1); x may be a channel slice
    ``t[:, :2]`` of a contiguous (B,K,D,H1,W1) tensor."""
    if not (isinstance(x, torch.Tensor) and x.is_cuda and x.dtype == torch.float32 and x.dim() == 5 and x.shape[1] == 2):
        raise RuntimeError("x must be a CUDA float32 tensor of shape (B, 2, D, H1, W1)")
    B, _, D, H1, W1 = x.shape
    if not x[0].is_contiguous():
        raise RuntimeError("x must be contiguous within a sample")
    Kc = _check_attention_params(weight, bias, "attention", x.device)
    a = torch.empty(B, Kc, D, H1, W1, dtype=torch.float32, device=x.device)
    lib = _lib.load()
    with torch.cuda.device(x.device):
        stream = torch.cuda.current_stream(x.device).cuda_stream
        _raise_on(lib.sfb_attention_forward(_ptr(x), x.stride(0), _ptr(weight), _ptr(bias), _ptr(a), B, Kc, D, H1, W1,
                                            ctypes.c_void_p(stream)), "sfb_attention_forward")
    return a


def attention_backward(x, weight, a, grad_a, add=None) -> List[torch.Tensor]:
    """[gx (B,2,D,H1,W1), gweight, gbias] of ``attention_forward`` for upstream gradient ``grad_a``; ``add`` (shape
    of x, may be a channel slice) is added to gx.  ``grad_a`` is left untouched (a copy is consumed)."""
    B, _, D, H1, W1 = x.shape
    dev = x.device
    Kc = weight.shape[0]
    _check_like(weight, "weight", (Kc, 2, 3, 3, 3), torch.float32, dev)
    _check_like(a, "a", (B, Kc, D, H1, W1), torch.float32, dev)
    _check_like(grad_a, "grad_a", (B, Kc, D, H1, W1), torch.float32, dev)
    g = grad_a.clone()
    gx = torch.empty(B, 2, D, H1, W1, dtype=torch.float32, device=dev)
    gw = torch.empty_like(weight)
    gb = torch.empty(Kc, dtype=torch.float32, device=dev)
    lib = _lib.load()
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        nbytes = lib.sfb_attention_backward_workspace_bytes(B, Kc, D, H1, W1)
        ws = _workspace(max(nbytes, 256), dev, stream)
        _raise_on(lib.sfb_attention_backward(_ptr(x), x.stride(0), _ptr(weight), _ptr(a), _ptr(g), _ptr(add),
                                             add.stride(0) if add is not None else 0, _ptr(gx), _ptr(gw), _ptr(gb),
                                             B, Kc, D, H1, W1, ctypes.c_void_p(ws.data_ptr()),
                                             ctypes.c_size_t(ws.numel()), ctypes.c_void_p(stream)),
                  "sfb_attention_backward")
    return [gx, gw, gb]


def _check_fmaps(fmap1: torch.Tensor, fmap2: torch.Tensor) -> _lib.SfbShape:
    """The model's feature maps (B, C, H, W), as core/corr.py:340-382 holds them."""
    _check(fmap1, "fmap1", torch.float32, 4)
    _check(fmap2, "fmap2", torch.float32, 4)
    if fmap1.device != fmap2.device:
        raise RuntimeError("fmap1 and fmap2 must be on the same device")
    if fmap1.shape[0] != fmap2.shape[0] or fmap1.shape[1] != fmap2.shape[1]:
        raise RuntimeError(f"batch / feature dimensions differ: {tuple(fmap1.shape)} vs {tuple(fmap2.shape)}")
    B, C, H1, W1 = fmap1.shape
    _, _, H2, W2 = fmap2.shape
    return _lib.SfbShape(B, H1, W1, H2, W2, C, 0)


def separation_level_forward(img1_features_l0, img2_features_lk, weight_u, bias_u, weight_v, bias_v,
                             with_argmax=True, fmaps=False, scale1=1.0, place=None) -> List[torch.Tensor]:
    """One pyramid level of the call site (core/corr.py:419-457 up to the upsampling):
    [sep_u (B,2+Kc,W2,H1,W1), sep_v (B,2+Kc,H2,H1,W1), am_u, am_v, a_u (B,Kc,W2,H1,W1), a_v (B,Kc,H2,H1,W1)];
    (weight_u, bias_u) are the parameters of the reference's ``attention1``, which acts on sep_u.
    With ``fmaps`` the two feature arguments are the model's maps (B,C,H,W) and image 1's is multiplied by
    ``scale1`` inside the library (the permute + division of core/corr.py:419-422).  ``place`` = (sep_u_all,
    sep_v_all, c0) (fmaps only) writes the volumes into channels c0.. of those larger contiguous tensors (the
    concatenation over pyramid levels, core/corr.py:473-475) and returns None in their place."""
    F1, F2 = img1_features_l0, img2_features_lk
    s = _check_fmaps(F1, F2) if fmaps else _check_pair(F1, F2)
    dev = F1.device
    s.Kc = _check_attention_params(weight_u, bias_u, "attention1", dev)
    if _check_attention_params(weight_v, bias_v, "attention2", dev) != s.Kc:
        raise RuntimeError("attention1 and attention2 must have the same number of output channels")
    f32 = dict(dtype=torch.float32, device=dev)
    Ktot = c0 = 0
    if place is not None:
        if not fmaps:
            raise RuntimeError("place needs fmaps=True")
        sep_u, sep_v, c0 = place
        Ktot = _check_placed(s, sep_u, sep_v, c0, dev, "sep")
    else:
        sep_u = torch.empty(s.B, 2 + s.Kc, s.W2, s.H1, s.W1, **f32)
        sep_v = torch.empty(s.B, 2 + s.Kc, s.H2, s.H1, s.W1, **f32)
    am_u = torch.empty(s.B, s.H2, s.H1, s.W1, dtype=torch.int32, device=dev) if with_argmax else None
    am_v = torch.empty(s.B, s.W2, s.H1, s.W1, dtype=torch.int32, device=dev) if with_argmax else None
    a_u = torch.empty(s.B, s.Kc, s.W2, s.H1, s.W1, **f32)
    a_v = torch.empty(s.B, s.Kc, s.H2, s.H1, s.W1, **f32)
    if fmaps:
        _call("sfb_separation_level_forward_fmaps", _lib.OP_SEPARATION_LEVEL_FORWARD, s, dev,
              (F1, F2, float(scale1), weight_u, bias_u, weight_v, bias_v, sep_u, sep_v, int(Ktot), int(c0), am_u, am_v,
               a_u, a_v))
        if place is not None:
            return [None, None, am_u, am_v, a_u, a_v]
    else:
        _call("sfb_separation_level_forward", _lib.OP_SEPARATION_LEVEL_FORWARD, s, dev,
              (F1, F2, weight_u, bias_u, weight_v, bias_v, sep_u, sep_v, am_u, am_v, a_u, a_v))
    return [sep_u, sep_v, am_u, am_v, a_u, a_v]


def _check_placed(s, t_u, t_v, c0, dev, name):
    """Larger tensors (B,Ktot,D,H1,W1) holding this level's 2+Kc channels from channel c0; returns Ktot."""
    _check(t_u, name + "_u", torch.float32, 5)
    Ktot = t_u.shape[1]
    _check_like(t_u, name + "_u", (s.B, Ktot, s.W2, s.H1, s.W1), torch.float32, dev)
    _check_like(t_v, name + "_v", (s.B, Ktot, s.H2, s.H1, s.W1), torch.float32, dev)
    if c0 < 0 or c0 + 2 + s.Kc > Ktot:
        raise RuntimeError(f"channels {c0}..{c0 + 2 + s.Kc} do not fit in {Ktot}")
    return Ktot


def separation_level_backward(img1_features_l0, img2_features_lk, weight_u, weight_v, sep_u, sep_v, am_u, am_v,
                              a_u, a_v, g_sep_u, g_sep_v, fmaps=False, scale1=1.0, c0=None) -> List[torch.Tensor]:
    """[gF1, gF2, gweight_u, gbias_u, gweight_v, gbias_v] of ``separation_level_forward`` (feature gradients in the
    layout of the feature arguments).  With ``c0`` (fmaps only) sep_u, sep_v, g_sep_u, g_sep_v are the larger
    tensors of a forward with ``place`` and the level occupies their channels c0.. ."""
    F1, F2 = img1_features_l0, img2_features_lk
    s = _check_fmaps(F1, F2) if fmaps else _check_pair(F1, F2)
    dev = F1.device
    _check_attention_cf(s, a_u, a_v, dev)
    _check_like(weight_u, "attention1.weight", (s.Kc, 2, 3, 3, 3), torch.float32, dev)
    _check_like(weight_v, "attention2.weight", (s.Kc, 2, 3, 3, 3), torch.float32, dev)
    _check_like(am_u, "argmax_u", (s.B, s.H2, s.H1, s.W1), torch.int32, dev)
    _check_like(am_v, "argmax_v", (s.B, s.W2, s.H1, s.W1), torch.int32, dev)
    Ktot = 0
    if c0 is not None:
        if not fmaps:
            raise RuntimeError("c0 needs fmaps=True")
        Ktot = _check_placed(s, sep_u, sep_v, c0, dev, "sep")
        if _check_placed(s, g_sep_u, g_sep_v, c0, dev, "grad_sep") != Ktot:
            raise RuntimeError("sep and grad_sep have different channel counts")
    else:
        for t, name, D in ((sep_u, "sep_u", s.W2), (sep_v, "sep_v", s.H2), (g_sep_u, "grad_sep_u", s.W2),
                           (g_sep_v, "grad_sep_v", s.H2)):
            _check_like(t, name, (s.B, 2 + s.Kc, D, s.H1, s.W1), torch.float32, dev)
    gF1 = torch.empty_like(F1)
    gF2 = torch.empty_like(F2)
    gw_u, gw_v = torch.empty_like(weight_u), torch.empty_like(weight_v)
    gb_u = torch.empty(s.Kc, dtype=torch.float32, device=dev)
    gb_v = torch.empty(s.Kc, dtype=torch.float32, device=dev)
    name = "sfb_separation_level_backward_fmaps" if fmaps else "sfb_separation_level_backward"
    head = (F1, F2, float(scale1)) if fmaps else (F1, F2)
    place = (int(Ktot), int(c0 or 0)) if fmaps else ()
    _call(name, _lib.OP_SEPARATION_LEVEL_BACKWARD, s, dev,
          head + (weight_u, weight_v, sep_u, sep_v) + place + (am_u, am_v, a_u, a_v, g_sep_u, g_sep_v, gF1, gF2, gw_u,
                                                               gb_u, gw_v, gb_v))
    return [gF1, gF2, gw_u, gb_u, gw_v, gb_v]


# ------------------------------------------------------------------------------------------------------
# Placement of a level's volumes into the concatenated, level-0-sized outputs (core/corr.py:459-475).
def upsample_displacement_into(src: torch.Tensor, dst: torch.Tensor, c0: int) -> None:
    """dst[:, c0:c0+K] = F.interpolate(src, dst.shape[2:], mode='trilinear', align_corners=True) for src
    (B,K,Dl,H1,W1) and a contiguous dst (B,Ktot,D0,H1,W1) with the same H1, W1 and Dl <= D0."""
    _check(src, "src", torch.float32, 5)
    _check(dst, "dst", torch.float32, 5)
    B, K, Dl, H1, W1 = src.shape
    if dst.shape[0] != B or tuple(dst.shape[3:]) != (H1, W1) or c0 < 0 or c0 + K > dst.shape[1] or dst.device != src.device:
        raise RuntimeError(f"cannot place {tuple(src.shape)} at channel {c0} of {tuple(dst.shape)}")
    D0 = dst.shape[2]
    lib = _lib.load()
    with torch.cuda.device(src.device):
        stream = torch.cuda.current_stream(src.device).cuda_stream
        out = ctypes.c_void_p(dst.data_ptr() + 4 * c0 * D0 * H1 * W1)
        _raise_on(lib.sfb_upsample_displacement(_ptr(src), out, dst.stride(0), B, K, Dl, D0, H1, W1,
                                                ctypes.c_void_p(stream)), "sfb_upsample_displacement")


def upsample_displacement_backward(grad_dst: torch.Tensor, c0: int, K: int, Dl: int) -> torch.Tensor:
    """Gradient of ``src`` (B,K,Dl,H1,W1) of ``upsample_displacement_into`` from the gradient of the whole dst."""
    _check(grad_dst, "grad_dst", torch.float32, 5)
    B, Ktot, D0, H1, W1 = grad_dst.shape
    if c0 < 0 or c0 + K > Ktot:
        raise RuntimeError(f"channels {c0}..{c0 + K} outside {Ktot}")
    gsrc = torch.empty(B, K, Dl, H1, W1, dtype=torch.float32, device=grad_dst.device)
    lib = _lib.load()
    with torch.cuda.device(grad_dst.device):
        stream = torch.cuda.current_stream(grad_dst.device).cuda_stream
        g = ctypes.c_void_p(grad_dst.data_ptr() + 4 * c0 * D0 * H1 * W1)
        _raise_on(lib.sfb_upsample_displacement_backward(g, grad_dst.stride(0), _ptr(gsrc), B, K, Dl, D0, H1, W1,
                                                         ctypes.c_void_p(stream)), "sfb_upsample_displacement_backward")
    return gsrc


# ------------------------------------------------------------------------------------------------------
# Lookup on an aggregated 3D cost volume (the reference's CorrBlock1D, core/corr.py:513-624), one volume at a time.
def _check_volume(corr):
    _check(corr, "corr", torch.float32, 5)
    return tuple(corr.shape)


def _check_coord(coord, B, H1, W1, dev):
    if not (isinstance(coord, torch.Tensor) and coord.is_cuda and coord.dtype == torch.float32
            and tuple(coord.shape) == (B, H1, W1) and coord.device == dev):
        raise RuntimeError(f"coord must be a CUDA float32 tensor of shape {(B, H1, W1)} on {dev}")
    if not coord[0].is_contiguous():
        raise RuntimeError("coord must be contiguous within a sample")


def lookup_build_pyramid(corr: torch.Tensor, levels: int) -> torch.Tensor:
    """Levels 1 .. levels-1 of the displacement pyramid of corr (B,dim,D,H1,W1), back to back in one flat tensor."""
    B, dim, D, H1, W1 = _check_volume(corr)
    lib = _lib.load()
    nbytes = lib.sfb_lookup_pyramid_bytes(B, dim, D, H1, W1, levels)
    pyr = torch.empty(max(nbytes // 4, 1), dtype=torch.float32, device=corr.device)
    with torch.cuda.device(corr.device):
        stream = torch.cuda.current_stream(corr.device).cuda_stream
        _raise_on(lib.sfb_lookup_build_pyramid(_ptr(corr), _ptr(pyr), B, dim, D, H1, W1, levels,
                                               ctypes.c_void_p(stream)), "sfb_lookup_build_pyramid")
    return pyr


def lookup_forward(corr, pyramid, coord, levels=4, radius=4, clamp_unit=False) -> torch.Tensor:
    """out (B, levels*dim*(2r+1), H1, W1): 2r+1 interpolated samples per level around coord / 2^level
    (core/corr.py:576-594); coord (B,H1,W1) may be a component slice ``coords[:, i]``."""
    B, dim, D, H1, W1 = _check_volume(corr)
    _check_coord(coord, B, H1, W1, corr.device)
    out = torch.empty(B, levels * dim * (2 * radius + 1), H1, W1, dtype=torch.float32, device=corr.device)
    lib = _lib.load()
    with torch.cuda.device(corr.device):
        stream = torch.cuda.current_stream(corr.device).cuda_stream
        _raise_on(lib.sfb_lookup_forward(_ptr(corr), _ptr(pyramid), _ptr(coord), coord.stride(0), _ptr(out), B, dim, D,
                                         H1, W1, levels, radius, int(bool(clamp_unit)), ctypes.c_void_p(stream)),
                  "sfb_lookup_forward")
    return out


def lookup_backward(corr_shape, coord, grad_out, levels=4, radius=4, clamp_unit=False) -> torch.Tensor:
    """Gradient of the volume (B,dim,D,H1,W1) for upstream gradient grad_out."""
    B, dim, D, H1, W1 = corr_shape
    dev = grad_out.device
    _check_like(grad_out, "grad_out", (B, levels * dim * (2 * radius + 1), H1, W1), torch.float32, dev)
    _check_coord(coord, B, H1, W1, dev)
    gcorr = torch.empty(B, dim, D, H1, W1, dtype=torch.float32, device=dev)
    lib = _lib.load()
    nbytes = lib.sfb_lookup_pyramid_bytes(B, dim, D, H1, W1, levels)
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        ws = _workspace(max(nbytes, 256), dev, stream)
        _raise_on(lib.sfb_lookup_backward(_ptr(grad_out), _ptr(coord), coord.stride(0), _ptr(gcorr),
                                          ctypes.c_void_p(ws.data_ptr()), B, dim, D, H1, W1, levels, radius,
                                          int(bool(clamp_unit)), ctypes.c_void_p(stream)), "sfb_lookup_backward")
    return gcorr


class sweep_operands:
    """Context manager / setter for the operand type of every contraction (correlation sweeps and gradient GEMMs) of
    the ops and the level calls: ``with ops.sweep_operands("tf32"): ...`` (process-wide).  "fp16" is the default (TF32's
    mantissa at twice the tensor-core rate, inputs scaled by powers of two on the device), "tf32" the same precision
    without scaling, "bf16" the lower-precision type of BASELINE's bf16 configuration."""
    _codes = {"tf32": 0, "bf16": 1, "fp16": 2}

    def __init__(self, kind: str):
        if kind not in self._codes:
            raise ValueError(f"operand type must be 'tf32', 'bf16' or 'fp16', got {kind!r}")
        self.prev = _lib.load().sfb_set_sweep_operands(self._codes[kind])

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        _lib.load().sfb_set_sweep_operands(self.prev)
        return False


def corr_volume(img1_features_l0, img2_features_lk) -> torch.Tensor:
    """Test aid: the dense volume S (B,H1,W1,H2,W2) of a small problem, through the tensor-core pipeline."""
    F1, F2 = img1_features_l0, img2_features_lk
    s = _check_pair(F1, F2)
    S = torch.empty(s.B, s.H1, s.W1, s.H2, s.W2, dtype=torch.float32, device=F1.device)
    _call("sfb_corr_volume", _lib.OP_CORR_VOLUME, s, F1.device, (F1, F2, S))
    return S


def _check_lookup4d(F1, F2_levels, coords, radius):
    if not (isinstance(F1, torch.Tensor) and F1.is_cuda and F1.dtype == torch.float32 and F1.dim() == 4
            and F1.is_contiguous()):
        raise RuntimeError("F1 must be a contiguous CUDA float32 tensor of shape (B, H1, W1, C)")
    B, H1, W1, C = F1.shape
    if C % 4 != 0 or C > 512:
        raise RuntimeError("the 4D lookup needs C % 4 == 0 and C <= 512")
    if not 0 <= radius <= 4:
        raise RuntimeError("radius must be in [0, 4]")
    if not 1 <= len(F2_levels) <= 8:
        raise RuntimeError("between 1 and 8 pyramid levels")
    for l, f2 in enumerate(F2_levels):
        if not (isinstance(f2, torch.Tensor) and f2.device == F1.device and f2.dtype == torch.float32 and f2.dim() == 4
                and f2.is_contiguous() and f2.shape[0] == B and f2.shape[3] == C):
            raise RuntimeError(f"F2_levels[{l}] must be a contiguous float32 tensor of shape (B, H2, W2, C) on {F1.device}")
        if f2.shape[1] < 2 or f2.shape[2] < 2:
            raise RuntimeError("every pyramid level needs H2 >= 2 and W2 >= 2")
    _check_like(coords, "coords", (B, 2, H1, W1), torch.float32, F1.device)
    if not coords.is_contiguous():
        raise RuntimeError("coords must be contiguous")
    return B, H1, W1, C


def _level_arrays(tensors):
    n = len(tensors)
    ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in tensors])
    H2 = (ctypes.c_int32 * n)(*[t.shape[1] for t in tensors])
    W2 = (ctypes.c_int32 * n)(*[t.shape[2] for t in tensors])
    return ptrs, H2, W2


def lookup4d_forward(F1, F2_levels, coords, radius=4, scale=1.0) -> torch.Tensor:
    """Lookup on the 4D correlation volume without storing it (the call core/corr.py:491-510 leaves
    unimplemented; same result as the dense block's lookup, core/corr.py:192-247).  F1 (B,H1,W1,C),
    F2_levels[l] (B,H2_l,W2_l,C) channels-last, coords (B,2,H1,W1) -> (B, levels*(2r+1)^2, H1, W1)."""
    B, H1, W1, C = _check_lookup4d(F1, F2_levels, coords, radius)
    n = len(F2_levels)
    out = torch.empty(B, n * (2 * radius + 1) ** 2, H1, W1, dtype=torch.float32, device=F1.device)
    ptrs, H2, W2 = _level_arrays(F2_levels)
    lib = _lib.load()
    with torch.cuda.device(F1.device):
        stream = torch.cuda.current_stream(F1.device).cuda_stream
        _raise_on(lib.sfb_lookup4d_forward(_ptr(F1), ptrs, H2, W2, n, _ptr(coords), _ptr(out), B, H1, W1, C, radius,
                                           float(scale), ctypes.c_void_p(stream)), "sfb_lookup4d_forward")
    return out


def lookup4d_backward(F1, F2_levels, coords, grad_out, radius=4, scale=1.0):
    """(gF1, [gF2_l]) for upstream gradient grad_out of lookup4d_forward."""
    B, H1, W1, C = _check_lookup4d(F1, F2_levels, coords, radius)
    n = len(F2_levels)
    _check_like(grad_out, "grad_out", (B, n * (2 * radius + 1) ** 2, H1, W1), torch.float32, F1.device)
    if not grad_out.is_contiguous():
        raise RuntimeError("grad_out must be contiguous")
    gF1 = torch.empty_like(F1)
    gF2 = [torch.empty_like(f2) for f2 in F2_levels]
    ptrs, H2, W2 = _level_arrays(F2_levels)
    gptrs, _, _ = _level_arrays(gF2)
    lib = _lib.load()
    with torch.cuda.device(F1.device):
        stream = torch.cuda.current_stream(F1.device).cuda_stream
        _raise_on(lib.sfb_lookup4d_backward(_ptr(F1), ptrs, H2, W2, n, _ptr(coords), _ptr(grad_out), _ptr(gF1), gptrs,
                                            B, H1, W1, C, radius, float(scale), ctypes.c_void_p(stream)),
                  "sfb_lookup4d_backward")
    return gF1, gF2
