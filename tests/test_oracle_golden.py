"""CPU: the oracle against the vectors generated from the reference's own Python code
(tests/golden/make_golden.py)."""
import os

import numpy as np
import torch
import torch.nn.functional as F

from oracle import separation_oracle as orc

TOL = 1e-11  # float64 vectors


def _t(x):
    return torch.from_numpy(np.ascontiguousarray(x))


def _pool(F2, level):
    x = F2.permute(0, 3, 1, 2)
    for _ in range(level):
        x = F.avg_pool2d(x, 2, stride=2)
    return x.permute(0, 2, 3, 1).contiguous()


def test_ops_match_reference_test_definitions(golden_dir):
    g = np.load(os.path.join(golden_dir, "ops_b2_c12_8x12_k3.npz"))
    F1, F2 = _t(g["F1"]), _t(g["F2"])
    for level in range(3):
        F2l = _pool(F2, level)
        MA_u, MA_v, AM_u, AM_v = orc.max_argmax_avg_forward(F1, F2l)
        # golden layout (B, disp, H1, W1) -- scripts/test_maxavg_cuda.py:136-144
        for name, ours in (("max_u", MA_u[..., 0, :]), ("avg_u", MA_u[..., 1, :]),
                           ("max_v", MA_v[..., 0, :]), ("avg_v", MA_v[..., 1, :])):
            ref = _t(g[f"l{level}_{name}"]).permute(0, 2, 3, 1)
            assert (ours - ref).abs().max().item() < TOL, (level, name)
        A_u, A_v = _t(g[f"l{level}_A_u"]), _t(g[f"l{level}_A_v"])
        C_u, C_v = orc.compression_forward(F1, F2l, A_u, A_v)
        # golden layout (B, Kc, disp, H1, W1) -- scripts/test_compression_cuda.py:151-157
        assert (C_u - _t(g[f"l{level}_C_u"]).permute(0, 3, 4, 1, 2)).abs().max().item() < TOL
        assert (C_v - _t(g[f"l{level}_C_v"]).permute(0, 3, 4, 1, 2)).abs().max().item() < TOL
        # the argmax really points at the maximum and is the first such index
        S = orc.corr_volume(F1, F2l)
        assert torch.equal(S.gather(4, AM_u[..., 0, :].long().unsqueeze(-1)).squeeze(-1), MA_u[..., 0, :])
        assert torch.equal(S.gather(3, AM_v[..., 0, :].long().unsqueeze(-2)).squeeze(-2), MA_v[..., 0, :])


def test_argmax_lowest_index_on_ties():
    F1 = torch.ones(1, 2, 3, 4, dtype=torch.float64)
    F2 = torch.ones(1, 3, 5, 4, dtype=torch.float64)  # every S entry identical: ties everywhere
    _, _, AM_u, AM_v = orc.max_argmax_avg_forward(F1, F2)
    assert AM_u.dtype == torch.int32 and AM_u.shape == (1, 2, 3, 1, 3) and AM_v.shape == (1, 2, 3, 1, 5)
    assert (AM_u == 0).all() and (AM_v == 0).all()


def test_backward_ops_match_autograd_of_dense_definition():
    g = torch.Generator().manual_seed(7)
    B, H1, W1, H2, W2, C, Kc = 2, 5, 7, 4, 6, 8, 3
    F1 = torch.randn(B, H1, W1, C, generator=g, dtype=torch.float64, requires_grad=True)
    F2 = torch.randn(B, H2, W2, C, generator=g, dtype=torch.float64, requires_grad=True)
    A_u = torch.randn(B, H1, W1, Kc, W2, generator=g, dtype=torch.float64, requires_grad=True)
    A_v = torch.randn(B, H1, W1, Kc, H2, generator=g, dtype=torch.float64, requires_grad=True)
    S = orc.corr_volume(F1, F2)
    # max/avg
    outs = [S.max(4).values, S.mean(4), S.max(3).values, S.mean(3)]
    gs = [torch.randn(o.shape, generator=g, dtype=torch.float64) for o in outs]
    ref = torch.autograd.grad(sum((o * w).sum() for o, w in zip(outs, gs)), (F1, F2), retain_graph=True)
    fw = orc.max_argmax_avg_forward(F1.detach(), F2.detach())
    gMA_u = torch.stack((gs[0], gs[1]), dim=3)
    gMA_v = torch.stack((gs[2], gs[3]), dim=3)
    got = orc.max_argmax_avg_backward(F1.detach(), F2.detach(), fw[2], fw[3], gMA_u, gMA_v)
    for a, b in zip(got, ref):
        assert (a - b).abs().max().item() < 1e-10
    # compression
    C_u = torch.einsum("bijuv,bijkv->bijku", S, A_u)
    C_v = torch.einsum("bijuv,bijku->bijkv", S, A_v)
    gC_u = torch.randn(C_u.shape, generator=g, dtype=torch.float64)
    gC_v = torch.randn(C_v.shape, generator=g, dtype=torch.float64)
    ref = torch.autograd.grad((C_u * gC_u).sum() + (C_v * gC_v).sum(), (F1, F2, A_u, A_v))
    got = orc.compression_backward(F1.detach(), F2.detach(), A_u.detach(), A_v.detach(), gC_u, gC_v)
    for a, b in zip(got, ref):
        assert (a - b).abs().max().item() < 1e-10


def test_row_chunking_is_transparent(monkeypatch):
    g = torch.Generator().manual_seed(9)
    F1 = torch.randn(1, 6, 5, 8, generator=g, dtype=torch.float64)
    F2 = torch.randn(1, 4, 7, 8, generator=g, dtype=torch.float64)
    whole = orc.max_argmax_avg_forward(F1, F2)
    real = orc._row_chunks
    monkeypatch.setattr(orc, "_row_chunks", lambda H1, W1, H2, W2, budget_elems=0: real(H1, W1, H2, W2, 1))
    chunked = orc.max_argmax_avg_forward(F1, F2)
    for a, b in zip(whole, chunked):
        assert torch.equal(a, b)


def test_lookup_matches_reference_corrblock1d(golden_dir):
    """The oracle's lookup against the outputs and volume gradients of the reference's own CorrBlock1D
    (core/corr.py:513-624; float32 outputs, hence 1e-6)."""
    g = np.load(os.path.join(golden_dir, "lookup1d_b1_dim2_16x24.npz"))
    levels, radius = int(g["levels"]), int(g["radius"])
    coords = torch.from_numpy(g["coords"])
    for i, clamp in ((1, True), (2, False)):
        corr = torch.from_numpy(g[f"corr{i}"])
        out = orc.lookup_forward(corr, coords[:, i - 1], levels, radius, clamp_unit=clamp)
        ref = torch.from_numpy(g[f"out{i}"]).double()
        assert out.shape == ref.shape and (out - ref).abs().max().item() < 1e-6
        gc = orc.lookup_backward(corr.shape, coords[:, i - 1], torch.from_numpy(g[f"w{i}"]).double(), levels, radius, clamp)
        assert (gc - torch.from_numpy(g[f"g_corr{i}"]).double()).abs().max().item() < 1e-6


def test_lookup4d_matches_reference_dense_block(golden_dir):
    """The oracle's 4D lookup (stored-volume form and memory-saving form) against the output and feature gradients
    of the reference's own dense CorrBlock (core/corr.py:192-247), generated by tests/golden/make_golden.py."""
    g = np.load(os.path.join(golden_dir, "lookup4d_b1_c8_12x16.npz"))
    levels, radius = int(g["levels"]), int(g["radius"])
    f1, f2 = torch.from_numpy(g["f1"]), torch.from_numpy(g["f2"])
    coords, w = torch.from_numpy(g["coords"]), torch.from_numpy(g["w"]).double()
    out = orc.lookup4d_dense_forward(f1, f2, coords, levels, radius)
    assert (out - torch.from_numpy(g["out"]).double()).abs().max().item() < 1e-6
    g1, g2 = orc.lookup4d_dense_backward(f1, f2, coords, w, levels, radius)
    assert (g1 - torch.from_numpy(g["g_f1"]).double()).abs().max().item() < 1e-5
    assert (g2 - torch.from_numpy(g["g_f2"]).double()).abs().max().item() < 1e-5

    # memory-saving form: pooled features instead of a pooled volume
    pyr = [f2]
    for _ in range(levels - 1):
        pyr.append(torch.nn.functional.avg_pool2d(pyr[-1], 2, stride=2))
    F1 = f1.permute(0, 2, 3, 1).contiguous()
    F2s = [t.permute(0, 2, 3, 1).contiguous() for t in pyr]
    scale = 1.0 / f1.shape[1] ** 0.5
    out2 = orc.lookup4d_forward(F1, F2s, coords, radius, scale)
    assert (out2 - out).abs().max().item() < 1e-12
    gF1, gF2s = orc.lookup4d_backward(F1, F2s, coords, w, radius, scale)
    assert (gF1.permute(0, 3, 1, 2) - g1).abs().max().item() < 1e-12
    with torch.enable_grad():
        x = f2.clone().requires_grad_(True)
        p = [x]
        for _ in range(levels - 1):
            p.append(torch.nn.functional.avg_pool2d(p[-1], 2, stride=2))
        torch.autograd.backward(p, [t.permute(0, 3, 1, 2) for t in gF2s])
    assert (x.grad - g2).abs().max().item() < 1e-12
