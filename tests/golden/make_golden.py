"""Generate the golden vectors under tests/golden/ from the reference's own Python code.

Run once in a container that holds the reference checkout:

    python tests/golden/make_golden.py /path/to/SeparableFlowThesis

What it does
  1. Puts stub modules in ``sys.modules`` for the two compiled extensions the reference
     imports at module top (libs/MemorySaver/functions/MemorySaver.py:3,
     libs/GANet/functions/GANet.py:3).  The GANet stub is empty (never called when
     ``guid is None``); the MemorySaver stub exposes the five op names backed by
     ``oracle/separation_oracle.py`` so the reference's own autograd wrappers and its own
     ``AlternateCorrBlockSepflow`` (core/corr.py:335-510) run on CPU.
  2. Runs the reference's dense ``CorrBlock`` (core/corr.py:15-302), pure reference code, in
     float64 on seeded inputs: separated volumes and, for a weighted-sum loss, the gradients
     of f1, f2 and both Conv3d modules.  These are the golden end-to-end vectors.
  3. Runs ``AlternateCorrBlockSepflow`` on top of the oracle and asserts that it reproduces
     (2) to 1e-11 -- this pins the oracle's five ops (values, layouts, argmax shapes,
     gradient definitions) against the reference.
  4. Stores op-level vectors from the reference's own test definitions
     ``compute_maxavg_torch`` (scripts/test_maxavg_cuda.py:118-146) and
     ``compute_compression_torch`` (scripts/test_compression_cuda.py:105-159), levels 0-2.

  5. Runs the reference's ``CorrBlock1D`` (core/corr.py:513-624) on seeded volumes and coordinates, stores outputs
     and volume gradients, and asserts that the oracle's lookup reproduces them to 1e-11.

The CPU tests load the stored ``.npz`` files and never need the reference checkout.
"""
from __future__ import annotations

import os
import sys
import types

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, REPO)

from oracle import separation_oracle as oracle  # noqa: E402


def install_stubs(ref_root: str):
    ms = types.ModuleType("libs.MemorySaver.build.lib.MemorySaver")
    for name in ("max_avg_forward", "max_argmax_avg_forward", "max_argmax_avg_backward",
                 "compression_forward", "compression_backward"):
        setattr(ms, name, getattr(oracle, name))
    for pkg in ("libs.MemorySaver.build", "libs.MemorySaver.build.lib",
                "libs.GANet.build", "libs.GANet.build.lib"):
        m = types.ModuleType(pkg)
        m.__path__ = []
        sys.modules[pkg] = m
    sys.modules["libs.MemorySaver.build.lib.MemorySaver"] = ms
    sys.modules["libs.MemorySaver.build.lib"].MemorySaver = ms
    ga = types.ModuleType("libs.GANet.build.lib.GANet")
    sys.modules["libs.GANet.build.lib.GANet"] = ga
    sys.modules["libs.GANet.build.lib"].GANet = ga
    sys.path.insert(0, ref_root)
    sys.path.insert(0, os.path.join(ref_root, "core"))


def seeded_case(B, C, H, W, Kc, seed=1234, dtype=torch.float64):
    g = torch.Generator().manual_seed(seed)
    f1 = torch.randn(B, C, H, W, generator=g, dtype=dtype)
    f2 = torch.randn(B, C, H, W, generator=g, dtype=dtype)
    convs = []
    for _ in range(2):
        conv = torch.nn.Conv3d(2, Kc, 3, padding=1).to(dtype)
        with torch.no_grad():
            conv.weight.copy_(torch.randn(conv.weight.shape, generator=g, dtype=dtype) * 0.02)
            conv.bias.copy_(torch.randn(conv.bias.shape, generator=g, dtype=dtype) * 0.02)
        convs.append(conv)
    return f1, f2, convs, g


def run_block(block_cls, f1, f2, convs, gen_seed, **kw):
    f1 = f1.clone().requires_grad_(True)
    f2 = f2.clone().requires_grad_(True)
    for c in convs:
        c.zero_grad()
    blk = block_cls(f1, f2, None, **kw)
    sep_u, sep_v = blk(None, sep=True, attention_weights=tuple(convs))
    g = torch.Generator().manual_seed(gen_seed)
    wu = torch.randn(sep_u.shape, generator=g, dtype=sep_u.dtype)
    wv = torch.randn(sep_v.shape, generator=g, dtype=sep_v.dtype)
    loss = (sep_u * wu).sum() + (sep_v * wv).sum()
    loss.backward()
    out = dict(sep_u=sep_u.detach(), sep_v=sep_v.detach(), g_f1=f1.grad, g_f2=f2.grad)
    for i, c in enumerate(convs):
        out[f"g_w{i}"] = c.weight.grad.clone()
        out[f"g_b{i}"] = c.bias.grad.clone()
    return out


def main(ref_root: str):
    install_stubs(ref_root)
    from core.corr import CorrBlock, AlternateCorrBlockSepflow  # reference code

    # ---- end-to-end block vectors (reference dense path) + oracle pin ----
    B, C, H, W, Kc = 2, 16, 9, 11, 2
    f1, f2, convs, _ = seeded_case(B, C, H, W, Kc)
    dense = run_block(CorrBlock, f1, f2, convs, 77)
    memsave = run_block(AlternateCorrBlockSepflow, f1, f2, convs, 77, support_backward=True)
    for k in dense:
        err = (dense[k] - memsave[k]).abs().max().item()
        assert err < 1e-11, (k, err)
        print(f"oracle-under-reference-wrappers vs reference dense  {k:6s} max|diff| = {err:.2e}")
    np.savez_compressed(
        os.path.join(HERE, "block_dense_b2_c16_9x11_k2.npz"),
        f1=f1.numpy(), f2=f2.numpy(),
        w0=convs[0].weight.detach().numpy(), b0=convs[0].bias.detach().numpy(),
        w1=convs[1].weight.detach().numpy(), b1=convs[1].bias.detach().numpy(),
        loss_seed=np.int64(77),
        **{k: v.numpy() for k, v in dense.items()})

    # ---- op-level vectors from the reference's own test definitions ----
    sys.path.insert(0, os.path.join(ref_root, "scripts"))
    import importlib
    t_maxavg = importlib.import_module("test_maxavg_cuda")
    t_comp = importlib.import_module("test_compression_cuda")
    B, C, H, W, Kc = 2, 12, 8, 12, 3
    g = torch.Generator().manual_seed(4321)
    F1 = torch.randn(B, H, W, C, generator=g, dtype=torch.float64) / C ** 0.5
    F2 = torch.randn(B, H, W, C, generator=g, dtype=torch.float64)
    store = dict(F1=F1.numpy(), F2=F2.numpy())
    for level in range(3):
        mu, au, mv, av = t_maxavg.compute_maxavg_torch(F1, F2, level)
        h2, w2 = H // 2 ** level, W // 2 ** level
        A_u = torch.randn(B, H, W, Kc, w2, generator=g, dtype=torch.float64).softmax(-1)
        A_v = torch.randn(B, H, W, Kc, h2, generator=g, dtype=torch.float64).softmax(-1)
        cu, cv = t_comp.compute_compression_torch(F1, F2, A_u, A_v, level)
        store.update({
            f"l{level}_max_u": mu.numpy(), f"l{level}_avg_u": au.numpy(),
            f"l{level}_max_v": mv.numpy(), f"l{level}_avg_v": av.numpy(),
            f"l{level}_A_u": A_u.numpy(), f"l{level}_A_v": A_v.numpy(),
            f"l{level}_C_u": cu.numpy(), f"l{level}_C_v": cv.numpy(),
        })
    np.savez_compressed(os.path.join(HERE, "ops_b2_c12_8x12_k3.npz"), **store)
    lookup_vectors()
    lookup4d_vectors()
    print("golden vectors written to", HERE)


def lookup_vectors():
    """The reference's CorrBlock1D (core/corr.py:513-624, pure torch) on seeded volumes and coordinates that reach
    inside, across and beyond the displacement range: outputs and the gradients of both volumes."""
    from core.corr import CorrBlock1D  # reference code
    B, dim, H, W, levels, radius = 1, 2, 16, 24, 4, 4
    g = torch.Generator().manual_seed(2468)
    corr1 = torch.randn(B, dim, W, H, W, generator=g, dtype=torch.float64).requires_grad_(True)
    corr2 = torch.randn(B, dim, H, H, W, generator=g, dtype=torch.float64).requires_grad_(True)
    coords = torch.stack((torch.rand(B, H, W, generator=g, dtype=torch.float64) * (W + 10) - 5,
                          torch.rand(B, H, W, generator=g, dtype=torch.float64) * (H + 10) - 5), dim=1)
    coords[0, :, 0, 0] = torch.tensor([3.0, 7.0], dtype=torch.float64)      # exact integers
    coords[0, :, 0, 1] = torch.tensor([-0.5, float(H - 1)], dtype=torch.float64)
    out1, out2 = CorrBlock1D(corr1, corr2, num_levels=levels, radius=radius)(coords)
    w1 = torch.randn(out1.shape, generator=g, dtype=torch.float64)
    w2 = torch.randn(out2.shape, generator=g, dtype=torch.float64)
    ((out1.double() * w1).sum() + (out2.double() * w2).sum()).backward()
    np.savez_compressed(os.path.join(HERE, "lookup1d_b1_dim2_16x24.npz"),
                        corr1=corr1.detach().numpy(), corr2=corr2.detach().numpy(), coords=coords.numpy(),
                        out1=out1.detach().numpy(), out2=out2.detach().numpy(),
                        w1=w1.float().numpy(), w2=w2.float().numpy(),
                        g_corr1=corr1.grad.float().numpy(), g_corr2=corr2.grad.float().numpy(),
                        levels=np.int64(levels), radius=np.int64(radius))
    # pin the oracle's restatement against the reference's outputs
    o1 = oracle.lookup_forward(corr1.detach(), coords[:, 0], levels, radius, clamp_unit=True)
    o2 = oracle.lookup_forward(corr2.detach(), coords[:, 1], levels, radius, clamp_unit=False)
    e1, e2 = (o1 - out1.detach()).abs().max().item(), (o2 - out2.detach()).abs().max().item()
    g1 = oracle.lookup_backward(corr1.shape, coords[:, 0], w1, levels, radius, True)
    g2 = oracle.lookup_backward(corr2.shape, coords[:, 1], w2, levels, radius, False)
    e3, e4 = (g1 - corr1.grad).abs().max().item(), (g2 - corr2.grad).abs().max().item()
    print(f"oracle lookup vs reference CorrBlock1D: out1 {e1:.2e} out2 {e2:.2e} g_corr1 {e3:.2e} g_corr2 {e4:.2e}")
    # the reference returns float32 (core/corr.py:602,623: ``.float()``), so its outputs and the gradients that
    # pass through that cast carry float32 rounding; the float64 oracle agrees to that rounding
    assert max(e1, e2, e3, e4) < 1e-6




def lookup4d_vectors():
    """The reference's dense block (core/corr.py:15-247, pure torch with guid=None) looked up at seeded coordinates
    that reach inside, across and beyond the image: the result the memory-saving block's unimplemented branch
    (core/corr.py:491-510) would have to return, and the gradients of both feature maps."""
    from core.corr import CorrBlock  # reference code
    B, C, H, W, levels, radius = 1, 8, 12, 16, 3, 4
    g = torch.Generator().manual_seed(1357)
    f1 = torch.randn(B, C, H, W, generator=g, dtype=torch.float64).requires_grad_(True)
    f2 = torch.randn(B, C, H, W, generator=g, dtype=torch.float64).requires_grad_(True)
    coords = torch.stack((torch.rand(B, H, W, generator=g, dtype=torch.float64) * (W + 8) - 4,
                          torch.rand(B, H, W, generator=g, dtype=torch.float64) * (H + 8) - 4), dim=1)
    coords[0, :, 0, 0] = torch.tensor([3.0, 7.0], dtype=torch.float64)      # exact integers
    coords[0, :, 0, 1] = torch.tensor([-0.5, float(H - 1)], dtype=torch.float64)
    coords[0, :, 0, 2] = torch.tensor([float(W - 1), 0.0], dtype=torch.float64)
    coords[0, :, 0, 3] = torch.tensor([-40.0, 55.0], dtype=torch.float64)   # window entirely in the padding
    out = CorrBlock(f1, f2, None, num_levels=levels, radius=radius)(coords)
    w = torch.randn(out.shape, generator=g, dtype=torch.float64)
    (out.double() * w).sum().backward()
    np.savez_compressed(os.path.join(HERE, "lookup4d_b1_c8_12x16.npz"),
                        f1=f1.detach().numpy(), f2=f2.detach().numpy(), coords=coords.numpy(),
                        out=out.detach().numpy(), w=w.float().numpy(),
                        g_f1=f1.grad.float().numpy(), g_f2=f2.grad.float().numpy(),
                        levels=np.int64(levels), radius=np.int64(radius))
    o = oracle.lookup4d_dense_forward(f1.detach(), f2.detach(), coords, levels, radius)
    g1, g2 = oracle.lookup4d_dense_backward(f1.detach(), f2.detach(), coords, w, levels, radius)
    print(f"oracle lookup4d vs reference CorrBlock: out {(o - out.detach()).abs().max().item():.2e} "
          f"g_f1 {(g1 - f1.grad).abs().max().item():.2e} g_f2 {(g2 - f2.grad).abs().max().item():.2e}")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/SeparableFlowThesis")
    main(sys.argv[1])
