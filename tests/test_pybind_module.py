"""The native Python module ``MemorySaver`` (separableflowthesis_b200/pybind): the five names of the reference's
pybind11 module (libs/MemorySaver/src/MemorySaver_cuda.cpp:105-112) over the C ABI.

CPU: the module imports, exports exactly those names and validates its inputs like the reference's CHECK_INPUT
(MemorySaver_cuda.cpp:6-8).  GPU: the same results as the ctypes layer, and -- where a checkout of the reference lies
beside this repository (or SFB_REFERENCE_ROOT points at one) -- the reference's own ``core/corr.py`` and
``libs/MemorySaver/functions/MemorySaver.py``, unmodified, running on top of the module and compared with the
stored vectors of the reference's dense path.
"""
import os
import sys
import types

import numpy as np
import pytest
import torch

from separableflowthesis_b200 import build as sfb_build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NAMES = ["compression_backward", "compression_forward", "max_argmax_avg_backward", "max_argmax_avg_forward",
         "max_avg_forward"]


@pytest.fixture(scope="module")
def memorysaver():
    sfb_build.build_pybind_module()
    return sfb_build.load_pybind_module()


def test_module_exports_the_reference_names_and_checks_inputs(memorysaver):
    assert sorted(n for n in dir(memorysaver) if not n.startswith("_")) == NAMES
    z = torch.zeros(1, 2, 2, 4)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        memorysaver.max_avg_forward(z, z)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        memorysaver.compression_backward(z, z, z, z, z, z)


def _reference_root():
    root = os.environ.get("SFB_REFERENCE_ROOT", os.path.join(os.path.dirname(ROOT), "reference"))
    return root if os.path.isdir(os.path.join(root, "libs", "MemorySaver", "functions")) else None


@pytest.mark.gpu
def test_module_matches_the_ctypes_layer(memorysaver, cuda_device):
    from separableflowthesis_b200 import ops
    g = torch.Generator().manual_seed(8)
    B, H1, W1, H2, W2, C, Kc = 2, 11, 19, 9, 21, 64, 3
    dev = cuda_device
    F1 = (torch.randn(B, H1, W1, C, generator=g) / C ** 0.5).to(dev)
    F2 = torch.randn(B, H2, W2, C, generator=g).to(dev)
    A_u = torch.randn(B, H1, W1, Kc, W2, generator=g).softmax(-1).to(dev)
    A_v = torch.randn(B, H1, W1, Kc, H2, generator=g).softmax(-1).to(dev)
    gMu, gMv = torch.randn(B, H1, W1, 2, H2, generator=g).to(dev), torch.randn(B, H1, W1, 2, W2, generator=g).to(dev)
    gCu, gCv = torch.randn(B, H1, W1, Kc, H2, generator=g).to(dev), torch.randn(B, H1, W1, Kc, W2, generator=g).to(dev)
    a = memorysaver.max_argmax_avg_forward(F1, F2)
    b = ops.max_argmax_avg_forward(F1, F2)
    assert len(a) == 4 and a[2].dtype == torch.int32 and tuple(a[2].shape) == (B, H1, W1, 1, H2)
    pairs = list(zip(a, b))
    pairs += list(zip(memorysaver.max_avg_forward(F1, F2), ops.max_avg_forward(F1, F2)))
    pairs += list(zip(memorysaver.compression_forward(F1, F2, A_u, A_v), ops.compression_forward(F1, F2, A_u, A_v)))
    pairs += list(zip(memorysaver.max_argmax_avg_backward(F1, F2, a[2], a[3], gMu, gMv),
                      ops.max_argmax_avg_backward(F1, F2, a[2], a[3], gMu, gMv)))
    pairs += list(zip(memorysaver.compression_backward(F1, F2, A_u, A_v, gCu, gCv),
                      ops.compression_backward(F1, F2, A_u, A_v, gCu, gCv)))
    for x, y in pairs:
        assert x.shape == y.shape and x.dtype == y.dtype and torch.equal(x, y)
    with pytest.raises(RuntimeError, match="must have shape"):
        memorysaver.compression_forward(F1, F2, A_v, A_u)
    with pytest.raises(RuntimeError, match="contiguous"):
        memorysaver.max_avg_forward(F1.transpose(1, 2), F2)


def _import_reference_block(memorysaver):
    """The reference's AlternateCorrBlockSepflow, imported unmodified from a checkout, with `memorysaver` in the place
    of ``libs/MemorySaver/build/lib/MemorySaver`` (functions/MemorySaver.py:3); None without a checkout."""
    ref_root = _reference_root()
    if ref_root is None:
        return None
    for pkg in ("libs.MemorySaver.build", "libs.MemorySaver.build.lib", "libs.GANet.build", "libs.GANet.build.lib"):
        m = types.ModuleType(pkg)
        m.__path__ = []
        sys.modules[pkg] = m
    sys.modules["libs.MemorySaver.build.lib.MemorySaver"] = memorysaver
    sys.modules["libs.MemorySaver.build.lib"].MemorySaver = memorysaver
    ga = types.ModuleType("libs.GANet.build.lib.GANet")      # imported by core/nlf.py, never called with guid=None
    sys.modules["libs.GANet.build.lib.GANet"] = ga
    sys.modules["libs.GANet.build.lib"].GANet = ga
    sys.path[:0] = [ref_root, os.path.join(ref_root, "core")]
    try:
        from core.corr import AlternateCorrBlockSepflow as RefBlock
    finally:
        del sys.path[:2]
    return RefBlock


def test_reference_call_site_reaches_the_module(memorysaver):
    """CPU: the reference's call site and autograd Functions import with this module in the place of their own build
    and hand it their tensors -- shown by the module's own input check answering (CPU tensors are refused exactly as
    the reference's CHECK_INPUT refuses them, MemorySaver_cuda.cpp:6-8), for the training and the inference Function."""
    RefBlock = _import_reference_block(memorysaver)
    if RefBlock is None:
        pytest.skip("no checkout of the reference beside this repository (set SFB_REFERENCE_ROOT)")
    g = torch.Generator().manual_seed(0)
    f1 = torch.randn(1, 16, 9, 11, generator=g)
    f2 = torch.randn(1, 16, 9, 11, generator=g)
    convs = tuple(torch.nn.Conv3d(2, 2, 3, padding=1) for _ in range(2))
    for support_backward in (True, False):
        blk = RefBlock(f1, f2, None, support_backward=support_backward)
        with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
            blk(None, sep=True, attention_weights=convs)


@pytest.mark.gpu
def test_reference_call_site_runs_on_the_module(memorysaver, cuda_device, golden_dir):
    """The drop-in: the reference's AlternateCorrBlockSepflow (core/corr.py:335-510) and its three autograd Functions
    (libs/MemorySaver/functions/MemorySaver.py), imported unmodified, with this module in the place of
    ``libs/MemorySaver/build/lib/MemorySaver``; outputs and gradients against the vectors its dense CorrBlock produced
    (tests/golden/make_golden.py).  Kc = 2, as the stored case."""
    RefBlock = _import_reference_block(memorysaver)
    if RefBlock is None:
        pytest.skip("no checkout of the reference beside this repository (set SFB_REFERENCE_ROOT)")
    z = np.load(os.path.join(golden_dir, "block_dense_b2_c16_9x11_k2.npz"))
    dev = cuda_device
    f1 = torch.from_numpy(z["f1"]).float().to(dev).requires_grad_(True)
    f2 = torch.from_numpy(z["f2"]).float().to(dev).requires_grad_(True)
    convs = []
    for i in range(2):
        conv = torch.nn.Conv3d(2, z["w0"].shape[0], 3, padding=1)
        with torch.no_grad():
            conv.weight.copy_(torch.from_numpy(z[f"w{i}"]).float())
            conv.bias.copy_(torch.from_numpy(z[f"b{i}"]).float())
        convs.append(conv.to(dev))
    torch.backends.cudnn.allow_tf32 = False
    blk = RefBlock(f1, f2, None, support_backward=True)
    sep_u, sep_v = blk(None, sep=True, attention_weights=tuple(convs))
    gen = torch.Generator().manual_seed(int(z["loss_seed"]))
    wu = torch.randn(sep_u.shape, generator=gen, dtype=torch.float64).float().to(dev)
    wv = torch.randn(sep_v.shape, generator=gen, dtype=torch.float64).float().to(dev)
    ((sep_u * wu).sum() + (sep_v * wv).sum()).backward()

    def relerr(x, name):
        r = torch.from_numpy(z[name]).double()
        return (x.detach().double().cpu() - r).abs().max().item() / max(r.abs().max().item(), 1e-30)

    assert relerr(sep_u, "sep_u") < 1e-3 and relerr(sep_v, "sep_v") < 1e-3
    assert relerr(f1.grad, "g_f1") < 2e-3 and relerr(f2.grad, "g_f2") < 2e-3
    assert relerr(convs[0].weight.grad, "g_w0") < 2e-3 and relerr(convs[1].weight.grad, "g_w1") < 2e-3
