"""GPU parity tests: the CUDA ops (called through the ctypes binding of the C ABI) against the
oracle on the same seeded inputs.

Tolerances.  The device path multiplies TF32-rounded operands (round-to-nearest, 2^-11 relative)
and accumulates in FP32; for S ~ N(0,1) that is ~4e-4 absolute per entry.  Values and gradients
must agree with the float64 oracle to TOL = 1e-3 in the reference's own error measure
max|x - ref| / max(|x|max, |ref|max) (scripts/test_model.py:251-256).  An argmax must be
bit-identical wherever the float64 gap between the best and second-best entry exceeds
MARGIN = 5e-3, and must always point at an entry within TOL of the maximum.
"""
import os

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import separableflowthesis_b200 as sfb
from separableflowthesis_b200 import ops
from oracle import separation_oracle as orc

pytestmark = pytest.mark.gpu

TOL = 1e-3
MARGIN = 5e-3

# (B, H1, W1, H2, W2, C, Kc): tiny, ragged/odd, pooled levels, C not a multiple of 32, Kc above one sweep
SHAPES = [
    (1, 1, 1, 1, 1, 4, 1),
    (1, 3, 5, 3, 5, 8, 1),
    (1, 8, 16, 8, 16, 32, 2),
    (2, 11, 19, 9, 21, 100, 3),
    (1, 17, 23, 8, 11, 64, 5),     # level-1 sized image 2, Kc > 4 -> two compression sweeps
    (3, 16, 16, 2, 2, 256, 2),     # level-3 sized image 2
    (1, 9, 130, 9, 130, 36, 4),    # more than one 128-pixel row tile per image row, W2 > 128
    (2, 48, 64, 48, 64, 256, 2),   # BASELINE config 2 at full size
]


def relerr(x, ref):
    x = x.detach().double().cpu()
    ref = ref.detach().double().cpu()
    den = max(x.abs().max().item(), ref.abs().max().item(), 1e-30)
    return (x - ref).abs().max().item() / den


def make_inputs(shape, seed):
    B, H1, W1, H2, W2, C, Kc = shape
    g = torch.Generator().manual_seed(seed)
    F1 = torch.randn(B, H1, W1, C, generator=g) / C ** 0.5
    F2 = torch.randn(B, H2, W2, C, generator=g)
    A_u = torch.randn(B, H1, W1, Kc, W2, generator=g).softmax(-1)
    A_v = torch.randn(B, H1, W1, Kc, H2, generator=g).softmax(-1)
    return F1, F2, A_u, A_v, g


@pytest.mark.parametrize("shape", SHAPES)
def test_corr_volume(shape, cuda_device):
    if shape[1] * shape[2] * shape[3] * shape[4] > 1 << 22:
        pytest.skip("dense dump only for small cases")
    F1, F2, *_ = make_inputs(shape, 0)
    S = ops.corr_volume(F1.to(cuda_device), F2.to(cuda_device))
    assert relerr(S, orc.corr_volume(F1.double(), F2.double())) < TOL


@pytest.mark.parametrize("shape", SHAPES)
def test_max_argmax_avg_forward(shape, cuda_device):
    F1, F2, *_ = make_inputs(shape, 1)
    MA_u, MA_v, AM_u, AM_v = ops.max_argmax_avg_forward(F1.to(cuda_device), F2.to(cuda_device))
    r_u, r_v, ra_u, ra_v = orc.max_argmax_avg_forward(F1.double(), F2.double())
    assert MA_u.shape == r_u.shape and MA_v.shape == r_v.shape
    assert AM_u.shape == ra_u.shape and AM_v.shape == ra_v.shape and AM_u.dtype == torch.int32
    for ch in (0, 1):
        assert relerr(MA_u[..., ch, :], r_u[..., ch, :]) < TOL
        assert relerr(MA_v[..., ch, :], r_v[..., ch, :]) < TOL
    gap_u, gap_v = orc.top2_margins(F1, F2)
    AM_u, AM_v = AM_u.cpu(), AM_v.cpu()
    assert ((AM_u[..., 0, :] == ra_u[..., 0, :]) | (gap_u <= MARGIN)).all()
    assert ((AM_v[..., 0, :] == ra_v[..., 0, :]) | (gap_v <= MARGIN)).all()
    # whatever index was chosen holds a value within tolerance of the maximum, and is in range
    S = orc.corr_volume(F1.double(), F2.double())
    assert (AM_u >= 0).all() and (AM_u < shape[4]).all() and (AM_v >= 0).all() and (AM_v < shape[3]).all()
    scale = max(S.abs().max().item(), 1e-30)
    picked_u = S.gather(4, AM_u[..., 0, :].long().unsqueeze(-1)).squeeze(-1)
    picked_v = S.gather(3, AM_v[..., 0, :].long().unsqueeze(-2)).squeeze(-2)
    assert ((r_u[..., 0, :] - picked_u).abs().max() / scale) < TOL
    assert ((r_v[..., 0, :] - picked_v).abs().max() / scale) < TOL
    # the inference variant returns the same max/mean channels, bit for bit
    MA_u2, MA_v2 = ops.max_avg_forward(F1.to(cuda_device), F2.to(cuda_device))
    assert torch.equal(MA_u2, MA_u) and torch.equal(MA_v2, MA_v)


def test_argmax_ties_lowest_index(cuda_device):
    """Duplicated image-2 pixels give bit-identical S entries; the lower index must win
    (MemorySaver_kernel_forward.cu:498-507)."""
    g = torch.Generator().manual_seed(3)
    B, H1, W1, H2, W2, C = 1, 6, 9, 20, 40, 64
    F1 = torch.randn(B, H1, W1, C, generator=g) / 8
    base = torch.randn(B, 1, 1, C, generator=g)
    F2 = base.expand(B, H2, W2, C).contiguous()          # all pixels equal: every row/column is one big tie
    _, _, AM_u, AM_v = ops.max_argmax_avg_forward(F1.to(cuda_device), F2.to(cuda_device))
    assert (AM_u == 0).all() and (AM_v == 0).all()
    F2 = torch.randn(B, H2, W2, C, generator=g)
    F2[:, :, 17] = F2[:, :, 3]                            # column 17 duplicates column 3
    F2[:, 12] = F2[:, 5]                                  # row 12 duplicates row 5 (after the column copy)
    _, _, AM_u, AM_v = ops.max_argmax_avg_forward(F1.to(cuda_device), F2.to(cuda_device))
    assert not (AM_u == 17).any() and not (AM_v == 12).any()


@pytest.mark.parametrize("shape", SHAPES)
def test_compression_forward(shape, cuda_device):
    F1, F2, A_u, A_v, _ = make_inputs(shape, 2)
    C_u, C_v = ops.compression_forward(*[t.to(cuda_device) for t in (F1, F2, A_u, A_v)])
    r_u, r_v = orc.compression_forward(F1.double(), F2.double(), A_u.double(), A_v.double())
    assert C_u.shape == r_u.shape and C_v.shape == r_v.shape
    assert relerr(C_u, r_u) < TOL and relerr(C_v, r_v) < TOL


@pytest.mark.parametrize("shape", SHAPES)
def test_max_argmax_avg_backward(shape, cuda_device):
    """The backward op takes the argmax as an input (MemorySaver_cuda.cpp:55-61), so it is tested in
    isolation with the oracle's argmax."""
    B, H1, W1, H2, W2, C, Kc = shape
    F1, F2, _, _, g = make_inputs(shape, 4)
    _, _, AM_u, AM_v = orc.max_argmax_avg_forward(F1.double(), F2.double())
    gMA_u = torch.randn(B, H1, W1, 2, H2, generator=g)
    gMA_v = torch.randn(B, H1, W1, 2, W2, generator=g)
    gF1, gF2 = ops.max_argmax_avg_backward(*[t.to(cuda_device) for t in (F1, F2, AM_u, AM_v, gMA_u, gMA_v)])
    r1, r2 = orc.max_argmax_avg_backward(F1.double(), F2.double(), AM_u, AM_v, gMA_u.double(), gMA_v.double())
    assert relerr(gF1, r1) < TOL and relerr(gF2, r2) < TOL


@pytest.mark.parametrize("shape", SHAPES)
def test_compression_backward(shape, cuda_device):
    B, H1, W1, H2, W2, C, Kc = shape
    F1, F2, A_u, A_v, g = make_inputs(shape, 5)
    gC_u = torch.randn(B, H1, W1, Kc, H2, generator=g)
    gC_v = torch.randn(B, H1, W1, Kc, W2, generator=g)
    args = (F1, F2, A_u, A_v, gC_u, gC_v)
    out = ops.compression_backward(*[t.to(cuda_device) for t in args])
    ref = orc.compression_backward(*[t.double() for t in args])
    for name, x, r in zip(("gF1", "gF2", "gA_u", "gA_v"), out, ref):
        assert x.shape == r.shape, name
        assert relerr(x, r) < TOL, name


@pytest.mark.parametrize("shape", SHAPES)
def test_separation_backward_is_the_sum_of_both_backward_ops(shape, cuda_device):
    """The one-call backward returns gA_u, gA_v of the compression op and gF1, gF2 = the sum of the two
    ops' feature gradients (what autograd accumulates for the reference's two Functions)."""
    B, H1, W1, H2, W2, C, Kc = shape
    F1, F2, A_u, A_v, g = make_inputs(shape, 8)
    _, _, AM_u, AM_v = orc.max_argmax_avg_forward(F1.double(), F2.double())
    gMA_u = torch.randn(B, H1, W1, 2, H2, generator=g)
    gMA_v = torch.randn(B, H1, W1, 2, W2, generator=g)
    gC_u = torch.randn(B, H1, W1, Kc, H2, generator=g)
    gC_v = torch.randn(B, H1, W1, Kc, W2, generator=g)
    out = ops.separation_backward(*[t.to(cuda_device) for t in (F1, F2, AM_u, AM_v, gMA_u, gMA_v, A_u, A_v, gC_u, gC_v)])
    r_m = orc.max_argmax_avg_backward(F1.double(), F2.double(), AM_u, AM_v, gMA_u.double(), gMA_v.double())
    r_c = orc.compression_backward(*[t.double() for t in (F1, F2, A_u, A_v, gC_u, gC_v)])
    assert relerr(out[0], r_m[0] + r_c[0]) < TOL and relerr(out[1], r_m[1] + r_c[1]) < TOL
    assert relerr(out[2], r_c[2]) < TOL and relerr(out[3], r_c[3]) < TOL


@pytest.mark.parametrize("shape", SHAPES)
def test_channels_first_ops(shape, cuda_device):
    """The (B,K,D,H1,W1)-layout entry points against the oracle's channels-first definitions (= the
    reference-layout results permuted the way core/corr.py:428-429,445-446 permutes them)."""
    B, H1, W1, H2, W2, C, Kc = shape
    F1, F2, A_u, A_v, g = make_inputs(shape, 9)
    a_u = A_u.permute(0, 3, 4, 1, 2).contiguous()
    a_v = A_v.permute(0, 3, 4, 1, 2).contiguous()
    dev = cuda_device
    sep_v, sep_u, am_u, am_v = ops.max_argmax_avg_forward_cf(F1.to(dev), F2.to(dev))
    r_sep_v, r_sep_u, r_am_u, r_am_v = orc.max_argmax_avg_forward_cf(F1.double(), F2.double())
    assert sep_v.shape == r_sep_v.shape and sep_u.shape == r_sep_u.shape and am_u.shape == r_am_u.shape
    assert relerr(sep_v, r_sep_v) < TOL and relerr(sep_u, r_sep_u) < TOL
    gap_u, gap_v = orc.top2_margins(F1, F2)   # (B,H1,W1,H2) and (B,H1,W1,W2)
    assert ((am_u.cpu() == r_am_u) | (gap_u.permute(0, 3, 1, 2) <= MARGIN)).all()
    assert ((am_v.cpu() == r_am_v) | (gap_v.permute(0, 3, 1, 2) <= MARGIN)).all()
    s2_v, s2_u, none_u, none_v = ops.max_argmax_avg_forward_cf(F1.to(dev), F2.to(dev), with_argmax=False)
    assert none_u is None and torch.equal(s2_v, sep_v) and torch.equal(s2_u, sep_u)
    c_u, c_v = ops.compression_forward_cf(F1.to(dev), F2.to(dev), a_u.to(dev), a_v.to(dev))
    r_c_u, r_c_v = orc.compression_forward_cf(F1.double(), F2.double(), a_u.double(), a_v.double())
    assert relerr(c_u, r_c_u) < TOL and relerr(c_v, r_c_v) < TOL
    gc_u = torch.randn(r_c_u.shape, generator=g)
    gc_v = torch.randn(r_c_v.shape, generator=g)
    ga_u, ga_v = ops.compression_attention_backward_cf(F1.to(dev), F2.to(dev), gc_u.to(dev), gc_v.to(dev))
    r_ga_u, r_ga_v = orc.compression_attention_backward_cf(F1.double(), F2.double(), gc_u.double(), gc_v.double())
    assert relerr(ga_u, r_ga_u) < TOL and relerr(ga_v, r_ga_v) < TOL
    g_sep_v = torch.randn(r_sep_v.shape, generator=g)
    g_sep_u = torch.randn(r_sep_u.shape, generator=g)
    gF1, gF2 = ops.separation_feature_backward_cf(*[t.to(dev) for t in (F1, F2, r_am_u, r_am_v, g_sep_v, g_sep_u,
                                                                         a_u, a_v, gc_u, gc_v)])
    r1, r2 = orc.separation_feature_backward_cf(F1.double(), F2.double(), r_am_u, r_am_v, g_sep_v.double(),
                                                g_sep_u.double(), a_u.double(), a_v.double(), gc_u.double(),
                                                gc_v.double())
    assert relerr(gF1, r1) < TOL and relerr(gF2, r2) < TOL


ATT_TOL = 2e-5   # fp32 stencil + softmax against the float64 oracle

# (B, Kc, D, H1, W1)
ATT_SHAPES = [(1, 1, 1, 1, 1), (2, 2, 3, 2, 5), (1, 3, 7, 9, 11), (2, 4, 24, 13, 37), (1, 5, 9, 6, 130), (1, 9, 4, 5, 7)]


@pytest.mark.parametrize("shape", ATT_SHAPES)
def test_attention_forward_backward(shape, cuda_device):
    """Conv3d(2 -> Kc, 3, padding 1) + softmax over the displacement axis (core/corr.py:437-442) and its
    backward, against torch's own float64 conv3d / softmax / autograd.  The input is a channel slice of a
    wider tensor, as at the call site."""
    B, Kc, D, H1, W1 = shape
    g = torch.Generator().manual_seed(21)
    wide = torch.randn(B, 2 + Kc, D, H1, W1, generator=g)
    weight = torch.randn(Kc, 2, 3, 3, 3, generator=g) * 0.3
    bias = torch.randn(Kc, generator=g)
    grad_a = torch.randn(B, Kc, D, H1, W1, generator=g)
    add = torch.randn(B, 2 + Kc, D, H1, W1, generator=g)
    dev = cuda_device
    wide_d, add_d = wide.to(dev), add.to(dev)
    a = ops.attention_forward(wide_d[:, :2], weight.to(dev), bias.to(dev))
    r_a = orc.attention_forward(wide[:, :2].double(), weight.double(), bias.double())
    assert a.shape == r_a.shape and relerr(a, r_a) < ATT_TOL
    assert (a.sum(dim=2) - 1).abs().max().item() < 1e-5
    gx, gw, gb = ops.attention_backward(wide_d[:, :2], weight.to(dev), a, grad_a.to(dev), add_d[:, :2])
    r_gx, r_gw, r_gb = orc.attention_backward(wide[:, :2].double(), weight.double(), a.double().cpu(), grad_a.double(),
                                              add[:, :2].double())
    assert relerr(gx, r_gx) < ATT_TOL and relerr(gw, r_gw) < ATT_TOL
    assert (gb.double().cpu() - r_gb).abs().max().item() < ATT_TOL * max(r_gw.abs().max().item(), 1.0)
    gx0, gw0, gb0 = ops.attention_backward(wide_d[:, :2], weight.to(dev), a, grad_a.to(dev))
    assert relerr(gx0, r_gx - add[:, :2].double()) < ATT_TOL and torch.equal(gw0, gw) and torch.equal(gb0, gb)


LEVEL_SHAPES = [s for s in SHAPES if s[1] * s[2] >= 15]


@pytest.mark.parametrize("shape", LEVEL_SHAPES)
def test_separation_level(shape, cuda_device):
    """One pyramid level in one call (core/corr.py:419-457) against the oracle's chain of the three ops and the
    two attention modules; the backward is checked with the device forward's own argmax / attention weights."""
    B, H1, W1, H2, W2, C, Kc = shape
    F1, F2, _, _, g = make_inputs(shape, 13)
    params = [torch.randn(Kc, 2, 3, 3, 3, generator=g) * 0.3, torch.randn(Kc, generator=g) * 0.1,
              torch.randn(Kc, 2, 3, 3, 3, generator=g) * 0.3, torch.randn(Kc, generator=g) * 0.1]
    dev = cuda_device
    F1d, F2d = F1.to(dev), F2.to(dev)
    wu, bu, wv, bv = [t.to(dev) for t in params]
    sep_u, sep_v, am_u, am_v, a_u, a_v = ops.separation_level_forward(F1d, F2d, wu, bu, wv, bv)
    ref = orc.separation_level_forward(F1.double(), F2.double(), *[t.double() for t in params])
    assert sep_u.shape == ref[0].shape and sep_v.shape == ref[1].shape
    # the attention weights see max/avg values that carry the TF32 error, through a softmax: same budget
    assert relerr(sep_u, ref[0]) < 2 * TOL and relerr(sep_v, ref[1]) < 2 * TOL
    assert relerr(a_u, ref[4]) < 2 * TOL and relerr(a_v, ref[5]) < 2 * TOL
    inf = ops.separation_level_forward(F1d, F2d, wu, bu, wv, bv, with_argmax=False)
    assert inf[2] is None and torch.equal(inf[0], sep_u) and torch.equal(inf[1], sep_v)
    g_sep_u = torch.randn(sep_u.shape, generator=g)
    g_sep_v = torch.randn(sep_v.shape, generator=g)
    out = ops.separation_level_backward(F1d, F2d, wu, wv, sep_u, sep_v, am_u, am_v, a_u, a_v, g_sep_u.to(dev),
                                        g_sep_v.to(dev))
    r = orc.separation_level_backward(F1.double(), F2.double(), params[0].double(), params[2].double(),
                                      sep_u.double().cpu(), sep_v.double().cpu(), am_u.cpu(), am_v.cpu(),
                                      a_u.double().cpu(), a_v.double().cpu(), g_sep_u.double(), g_sep_v.double())
    assert relerr(out[0], r[0]) < TOL and relerr(out[1], r[1]) < TOL
    for i in (2, 4):
        assert relerr(out[i], r[i]) < TOL
        assert (out[i + 1].double().cpu() - r[i + 1]).abs().max().item() < TOL * max(r[i].abs().max().item(), 1.0)
    again = ops.separation_level_backward(F1d, F2d, wu, wv, sep_u, sep_v, am_u, am_v, a_u, a_v, g_sep_u.to(dev),
                                          g_sep_v.to(dev))
    for x, y in zip(out, again):
        assert torch.equal(x, y)
    # the same level from the model's (B,C,H,W) feature maps, scale applied inside (core/corr.py:419-422)
    scale = 1.0 / C ** 0.5
    fmap1 = (F1 * C ** 0.5).permute(0, 3, 1, 2).contiguous()
    fmap2 = F2.permute(0, 3, 1, 2).contiguous()
    fw = ops.separation_level_forward(fmap1.to(dev), fmap2.to(dev), wu, bu, wv, bv, fmaps=True, scale1=scale)
    assert relerr(fw[0], ref[0]) < 2 * TOL and relerr(fw[1], ref[1]) < 2 * TOL
    outm = ops.separation_level_backward(fmap1.to(dev), fmap2.to(dev), wu, wv, *fw, g_sep_u.to(dev), g_sep_v.to(dev),
                                         fmaps=True, scale1=scale)
    rm = orc.separation_level_backward(fmap1.double(), fmap2.double(), params[0].double(), params[2].double(),
                                       fw[0].double().cpu(), fw[1].double().cpu(), fw[2].cpu(), fw[3].cpu(),
                                       fw[4].double().cpu(), fw[5].double().cpu(), g_sep_u.double(), g_sep_v.double(),
                                       fmaps=True, scale1=scale)
    assert outm[0].shape == fmap1.shape and outm[1].shape == fmap2.shape
    assert relerr(outm[0], rm[0]) < TOL and relerr(outm[1], rm[1]) < TOL
    assert relerr(outm[2], rm[2]) < TOL and relerr(outm[4], rm[4]) < TOL
    # ... and written into / read from channels 3.. of larger tensors (the concatenation over pyramid levels)
    Kt, Ktot, c0 = 2 + Kc, 2 + Kc + 4, 3
    big_u = torch.full((B, Ktot, W2, H1, W1), 5.0, device=dev)
    big_v = torch.full((B, Ktot, H2, H1, W1), 5.0, device=dev)
    fp = ops.separation_level_forward(fmap1.to(dev), fmap2.to(dev), wu, bu, wv, bv, fmaps=True, scale1=scale,
                                      place=(big_u, big_v, c0))
    assert fp[0] is None and torch.equal(big_u[:, c0:c0 + Kt], fw[0]) and torch.equal(big_v[:, c0:c0 + Kt], fw[1])
    assert (big_u[:, :c0] == 5.0).all() and (big_u[:, c0 + Kt:] == 5.0).all()
    gbig_u = torch.zeros_like(big_u)
    gbig_v = torch.zeros_like(big_v)
    gbig_u[:, c0:c0 + Kt] = g_sep_u.to(dev)
    gbig_v[:, c0:c0 + Kt] = g_sep_v.to(dev)
    outp = ops.separation_level_backward(fmap1.to(dev), fmap2.to(dev), wu, wv, big_u, big_v, fp[2], fp[3], fp[4], fp[5],
                                         gbig_u, gbig_v, fmaps=True, scale1=scale, c0=c0)
    for x, y in zip(outp, outm):
        assert torch.equal(x, y)


# positions pass through grid_sample's normalisation and back in float32, as in the reference's own float32 run:
# position error ~ D * 2^-24, i.e. ~1.4e-5 of a displacement step at D = 240
LOOKUP_TOL = 5e-5


@pytest.mark.parametrize("shape", [(1, 1, 1, 1, 1, 1), (2, 3, 5, 11, 4, 7), (1, 6, 30, 240, 9, 33), (2, 2, 16, 16, 5, 130)])
def test_upsample_displacement(shape, cuda_device):
    """Resampling of a level's volumes along the displacement axis into a channel slice of the concatenated output
    and its adjoint, against F.interpolate(mode='trilinear', align_corners=True) (core/corr.py:459-467)."""
    B, K, Dl, D0, H1, W1 = shape
    g = torch.Generator().manual_seed(41)
    src = torch.randn(B, K, Dl, H1, W1, generator=g)
    dev = cuda_device
    dst = torch.full((B, K + 3, D0, H1, W1), 7.0, device=dev)
    ops.upsample_displacement_into(src.to(dev), dst, 2)
    ref = F.interpolate(src.double(), [D0, H1, W1], mode="trilinear", align_corners=True)
    # the source position d*(Dl-1)/(D0-1) is formed in float32, as in torch's own float32 kernel: ~D0 * 2^-24
    assert relerr(dst[:, 2:2 + K], ref) < 2e-5
    assert (dst[:, :2] == 7.0).all() and (dst[:, 2 + K:] == 7.0).all()     # neighbours untouched
    gd = torch.randn(B, K + 3, D0, H1, W1, generator=g)
    gs = ops.upsample_displacement_backward(gd.to(dev), 2, K, Dl)
    assert relerr(gs, orc.upsample_displacement_backward(gd.double(), 2, K, Dl)) < 2e-5

# (B, dim, D, H1, W1, levels, radius)
LOOKUP_SHAPES = [(1, 1, 2, 1, 1, 1, 1), (2, 1, 16, 5, 7, 4, 4), (1, 3, 37, 9, 11, 3, 2), (2, 2, 240, 13, 37, 4, 4)]


@pytest.mark.parametrize("shape", LOOKUP_SHAPES)
@pytest.mark.parametrize("clamp", [False, True])
def test_lookup_forward_backward(shape, clamp, cuda_device):
    """Displacement pyramid + interpolated lookup of one aggregated volume and its backward against the oracle's
    restatement of the reference's avg_pool2d / grid_sample chain (core/corr.py:543-594)."""
    B, dim, D, H1, W1, levels, radius = shape
    g = torch.Generator().manual_seed(31)
    corr = torch.randn(B, dim, D, H1, W1, generator=g)
    coords = torch.rand(B, 2, H1, W1, generator=g) * (D + 12) - 6     # inside, across and beyond the range
    coords[0, 0].view(-1)[0] = 3.0                                     # an exact integer position
    gout = torch.randn(B, levels * dim * (2 * radius + 1), H1, W1, generator=g)
    dev = cuda_device
    corr_d, coords_d = corr.to(dev), coords.to(dev)
    pyr = ops.lookup_build_pyramid(corr_d, levels)
    out = ops.lookup_forward(corr_d, pyr, coords_d[:, 0], levels, radius, clamp)
    ref = orc.lookup_forward(corr.double(), coords[:, 0].double(), levels, radius, clamp)
    assert out.shape == ref.shape and relerr(out, ref) < LOOKUP_TOL
    gc = ops.lookup_backward(tuple(corr.shape), coords_d[:, 0], gout.to(dev), levels, radius, clamp)
    rg = orc.lookup_backward(corr.shape, coords[:, 0].double(), gout.double(), levels, radius, clamp)
    assert relerr(gc, rg) < LOOKUP_TOL
    assert torch.equal(gc, ops.lookup_backward(tuple(corr.shape), coords_d[:, 0], gout.to(dev), levels, radius, clamp))


def test_corrblock1d_against_reference_vectors(golden_dir, cuda_device):
    """The CorrBlock1D drop-in (both volumes, autograd) against the vectors of the reference's own class."""
    gold = np.load(os.path.join(golden_dir, "lookup1d_b1_dim2_16x24.npz"))
    dev = cuda_device
    corr1 = torch.from_numpy(gold["corr1"]).float().to(dev).requires_grad_(True)
    corr2 = torch.from_numpy(gold["corr2"]).float().to(dev).requires_grad_(True)
    coords = torch.from_numpy(gold["coords"]).float().to(dev)
    blk = sfb.CorrBlock1D(corr1, corr2, num_levels=int(gold["levels"]), radius=int(gold["radius"]))
    out1, out2 = blk(coords)
    assert relerr(out1, torch.from_numpy(gold["out1"])) < LOOKUP_TOL
    assert relerr(out2, torch.from_numpy(gold["out2"])) < LOOKUP_TOL
    w1 = torch.from_numpy(gold["w1"]).to(dev)
    w2 = torch.from_numpy(gold["w2"]).to(dev)
    ((out1 * w1).sum() + (out2 * w2).sum()).backward()
    assert relerr(corr1.grad, torch.from_numpy(gold["g_corr1"])) < LOOKUP_TOL
    assert relerr(corr2.grad, torch.from_numpy(gold["g_corr2"])) < LOOKUP_TOL


def _lookup4d_coords(kind, B, H1, W1, H2, W2, gen):
    """(B,2,H1,W1) positions in image 2: 'smooth' = the pixel grid plus a slowly varying displacement (neighbouring
    windows overlap, four pixels per pass), 'random' = anywhere inside and around the image (one pixel per pass),
    'mixed' = smooth with a block of random ones, exact integers and far-away positions."""
    ys, xs = torch.meshgrid(torch.arange(H1, dtype=torch.float32), torch.arange(W1, dtype=torch.float32), indexing="ij")
    sx, sy = (W2 - 1) / max(W1 - 1, 1), (H2 - 1) / max(H1 - 1, 1)
    smooth = torch.stack((xs * sx + 2.5 * torch.sin(ys / 3.0) + 0.3, ys * sy + 1.5 * torch.cos(xs / 4.0) - 0.2))
    smooth = smooth.unsqueeze(0).repeat(B, 1, 1, 1)
    rnd = torch.stack((torch.rand(B, H1, W1, generator=gen) * (W2 + 12) - 6,
                       torch.rand(B, H1, W1, generator=gen) * (H2 + 12) - 6), dim=1)
    if kind == "smooth":
        return smooth
    if kind == "random":
        return rnd
    out = smooth.clone()
    out[:, :, : max(H1 // 3, 1)] = rnd[:, :, : max(H1 // 3, 1)]
    out[0, :, -1, 0] = torch.tensor([3.0, 2.0])
    out[0, :, -1, -1] = torch.tensor([-500.0, 1.0e7])
    return out


# (B, C, H1, W1, H2, W2, levels, radius, coordinates)
LOOKUP4D_CASES = [
    (1, 4, 1, 1, 2, 2, 1, 0, "random"),
    (1, 8, 12, 16, 12, 16, 3, 4, "mixed"),
    (2, 256, 20, 28, 20, 28, 3, 4, "smooth"),
    (2, 256, 9, 13, 9, 13, 2, 4, "random"),
    (1, 100, 9, 13, 16, 11, 2, 2, "mixed"),       # C not a multiple of 128, N1 not a multiple of 32, H2 != H1
    (1, 384, 8, 12, 8, 12, 2, 3, "smooth"),
    (1, 512, 5, 7, 17, 33, 4, 1, "mixed"),
]


@pytest.mark.parametrize("case", LOOKUP4D_CASES)
def test_lookup4d_forward_backward(case, cuda_device):
    """4D lookup without the stored volume, and its feature gradients, against the oracle's restatement of the
    dense block's einsum / avg_pool2d / grid_sample chain (core/corr.py:286-296, 32-39, 200-247) in float64."""
    B, C, H1, W1, H2, W2, levels, radius, kind = case
    dev = cuda_device
    gen = torch.Generator().manual_seed(4242 + C + H1)
    f1 = torch.randn(B, H1, W1, C, generator=gen)
    f2 = torch.randn(B, C, H2, W2, generator=gen)
    pyr = [f2]
    for _ in range(levels - 1):
        pyr.append(F.avg_pool2d(pyr[-1], 2, stride=2))
    F2s = [t.permute(0, 2, 3, 1).contiguous() for t in pyr]
    coords = _lookup4d_coords(kind, B, H1, W1, H2, W2, gen)
    scale = 1.0 / C ** 0.5
    out = ops.lookup4d_forward(f1.to(dev), [t.to(dev) for t in F2s], coords.to(dev), radius, scale)
    ref = orc.lookup4d_forward(f1.double(), [t.double() for t in F2s], coords.double(), radius, scale)
    assert out.shape == ref.shape and relerr(out, ref) < LOOKUP_TOL
    gout = torch.randn(out.shape, generator=gen)
    gF1, gF2 = ops.lookup4d_backward(f1.to(dev), [t.to(dev) for t in F2s], coords.to(dev), gout.to(dev), radius, scale)
    rF1, rF2 = orc.lookup4d_backward(f1.double(), [t.double() for t in F2s], coords.double(), gout.double(), radius, scale)
    assert relerr(gF1, rF1) < LOOKUP_TOL
    for a, b in zip(gF2, rF2):
        assert relerr(a, b) < LOOKUP_TOL


def test_block_lookup_against_reference_vectors(golden_dir, cuda_device):
    """AlternateCorrBlockSepflow(...)(coords): the branch the reference leaves unimplemented (core/corr.py:491-510),
    against the output and feature gradients of the reference's own dense CorrBlock (core/corr.py:192-247)."""
    gold = np.load(os.path.join(golden_dir, "lookup4d_b1_c8_12x16.npz"))
    dev = cuda_device
    f1 = torch.from_numpy(gold["f1"]).float().to(dev).requires_grad_(True)
    f2 = torch.from_numpy(gold["f2"]).float().to(dev).requires_grad_(True)
    blk = sfb.AlternateCorrBlockSepflow(f1, f2, None, num_levels=int(gold["levels"]), radius=int(gold["radius"]),
                                        support_backward=True)
    coords = torch.from_numpy(gold["coords"]).float().to(dev)
    out = blk(coords)
    assert relerr(out, torch.from_numpy(gold["out"])) < LOOKUP_TOL
    assert torch.equal(out, blk(coords))
    (out * torch.from_numpy(gold["w"]).to(dev)).sum().backward()
    assert relerr(f1.grad, torch.from_numpy(gold["g_f1"])) < LOOKUP_TOL
    assert relerr(f2.grad, torch.from_numpy(gold["g_f2"])) < LOOKUP_TOL


def test_ops_from_a_fresh_thread(cuda_device):
    """A thread that has not touched CUDA yet (an autograd worker whose first node is one of these ops) can call
    every entry point: the library binds the device context itself before it builds tensor maps."""
    import threading
    shape = (1, 6, 9, 6, 9, 16, 2)
    F1, F2, _, _, g = make_inputs(shape, 17)
    params = [torch.randn(2, 2, 3, 3, 3, generator=g) * 0.3, torch.randn(2, generator=g) * 0.1,
              torch.randn(2, 2, 3, 3, 3, generator=g) * 0.3, torch.randn(2, generator=g) * 0.1]
    dev = cuda_device
    F1d, F2d = F1.to(dev), F2.to(dev)
    wu, bu, wv, bv = [t.to(dev) for t in params]
    fw = ops.separation_level_forward(F1d, F2d, wu, bu, wv, bv)
    gs = [torch.randn(fw[0].shape, generator=g).to(dev), torch.randn(fw[1].shape, generator=g).to(dev)]
    ref = ops.separation_level_backward(F1d, F2d, wu, wv, *fw, *gs)
    torch.cuda.synchronize()
    box = {}

    def work():
        try:
            box["out"] = ops.separation_level_backward(F1d, F2d, wu, wv, *fw, *gs)
            torch.cuda.synchronize()
        except Exception as e:  # surfaced below
            box["err"] = e

    t = threading.Thread(target=work)
    t.start()
    t.join()
    assert "err" not in box, box.get("err")
    for x, y in zip(ref, box["out"]):
        assert torch.equal(x, y)


def test_two_threads_on_their_own_streams(cuda_device):
    """Two host threads, each on its own CUDA stream, run the ops on different shapes at the same time (the
    DataParallel / serving-worker pattern).  Workspaces are kept per (device, stream), so neither sees the other's
    operand copies, scales or status word: every result equals the one the same call gives when it runs alone."""
    import threading
    shapes = [(2, 17, 23, 8, 11, 64, 5), (1, 9, 130, 9, 130, 40, 4)]

    def run_all(job):
        a, params, ups = job
        fw = ops.separation_level_forward(a[0], a[1], *params)
        bw = ops.separation_level_backward(a[0], a[1], params[0], params[2], *fw, *ups)
        return list(ops.max_argmax_avg_forward(*a[:2])) + list(ops.compression_forward(*a[:4])) + \
            list(ops.compression_backward(*a)) + list(fw) + list(bw)

    jobs = []
    for i, shape in enumerate(shapes):
        B, H1, W1, H2, W2, C, Kc = shape
        F1, F2, A_u, A_v, g = make_inputs(shape, 60 + i)
        gC_u = torch.randn(B, H1, W1, Kc, H2, generator=g)
        gC_v = torch.randn(B, H1, W1, Kc, W2, generator=g)
        args = [t.to(cuda_device) for t in (F1, F2, A_u, A_v, gC_u, gC_v)]
        # the level calls stage their Conv3d weights in one per-device constant array: each thread has its own weights
        params = [t.to(cuda_device) for t in (torch.randn(Kc, 2, 3, 3, 3, generator=g) * 0.3, torch.randn(Kc, generator=g) * 0.1,
                                              torch.randn(Kc, 2, 3, 3, 3, generator=g) * 0.3, torch.randn(Kc, generator=g) * 0.1)]
        fw = ops.separation_level_forward(args[0], args[1], *params)
        ups = [torch.randn(fw[0].shape, generator=g).to(cuda_device), torch.randn(fw[1].shape, generator=g).to(cuda_device)]
        args = (args, params, ups)
        alone = run_all(args)
        jobs.append((args, alone))
    torch.cuda.synchronize()
    errors, mismatches = [], []

    def work(i):
        try:
            args, alone = jobs[i]
            stream = torch.cuda.Stream(device=cuda_device)
            with torch.cuda.stream(stream):
                for _ in range(6):
                    out = run_all(args)
                    stream.synchronize()
                    mismatches.extend((i, j) for j, (x, y) in enumerate(zip(out, alone)) if not torch.equal(x, y))
        except Exception as e:  # surfaced below
            errors.append(e)

    threads = [threading.Thread(target=work, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    assert not mismatches, mismatches


@pytest.mark.parametrize("shape", [(2, 11, 19, 9, 21, 104, 3), (1, 24, 40, 24, 40, 256, 2)])
def test_separation_level_with_bf16_sweep_operands(shape, cuda_device):
    """BF16 operands in the sweeps of the level calls (BASELINE's bf16 configuration): products of BF16 values are
    exact in FP32, so the max channel must match the float64 oracle evaluated on the BF16-rounded features to
    accumulation-order accuracy; the mean rows of F2 are rounded once more (BF16), which the mean, attention and
    compression channels inherit; the backward (BF16 gradient GEMMs and attention-gradient sweep) stays within BF16
    accuracy of the default path."""
    B, H1, W1, H2, W2, C, Kc = shape
    F1, F2, _, _, g = make_inputs(shape, 23)
    params = [torch.randn(Kc, 2, 3, 3, 3, generator=g) * 0.3, torch.randn(Kc, generator=g) * 0.1,
              torch.randn(Kc, 2, 3, 3, 3, generator=g) * 0.3, torch.randn(Kc, generator=g) * 0.1]
    dev = cuda_device
    F1d, F2d = F1.to(dev), F2.to(dev)
    wu, bu, wv, bv = [t.to(dev) for t in params]
    before = _lib_operands()
    with ops.sweep_operands("bf16"):
        fw = ops.separation_level_forward(F1d, F2d, wu, bu, wv, bv)
        g_sep_u = torch.randn(fw[0].shape, generator=g).to(dev)
        g_sep_v = torch.randn(fw[1].shape, generator=g).to(dev)
        bw = ops.separation_level_backward(F1d, F2d, wu, wv, *fw, g_sep_u, g_sep_v)
    assert _lib_operands() == before                              # restored
    F1b, F2b = F1.bfloat16().double(), F2.bfloat16().double()
    ref = orc.separation_level_forward(F1b, F2b, *[t.double() for t in params])
    assert relerr(fw[0][:, 0], ref[0][:, 0]) < 2e-5 and relerr(fw[1][:, 0], ref[1][:, 0]) < 2e-5
    assert relerr(fw[0], ref[0]) < 4e-3 and relerr(fw[1], ref[1]) < 4e-3
    gap_u, gap_v = orc.top2_margins(F1b.float(), F2b.float())
    assert ((fw[2].cpu() == ref[2]) | (gap_u.permute(0, 3, 1, 2) <= 1e-4)).all()
    assert ((fw[3].cpu() == ref[3]) | (gap_v.permute(0, 3, 1, 2) <= 1e-4)).all()
    # against the unrounded float64 oracle the BF16 path is a BF16-accuracy result
    ref32 = orc.separation_level_forward(F1.double(), F2.double(), *[t.double() for t in params])
    assert relerr(fw[0], ref32[0]) < 1e-2 and relerr(fw[1], ref32[1]) < 1e-2
    # backward with the BF16 forward's own argmax / attention weights: BF16 accuracy against the float64 oracle
    rb = orc.separation_level_backward(F1.double(), F2.double(), params[0].double(), params[2].double(),
                                       fw[0].double().cpu(), fw[1].double().cpu(), fw[2].cpu(), fw[3].cpu(),
                                       fw[4].double().cpu(), fw[5].double().cpu(), g_sep_u.double().cpu(),
                                       g_sep_v.double().cpu())
    for i in (0, 1, 2, 4):
        assert relerr(bw[i], rb[i]) < 1e-2, i


def _lib_operands():
    from separableflowthesis_b200 import _lib
    return _lib.load().sfb_get_sweep_operands()


def test_backward_is_deterministic(cuda_device):
    """Gradients accumulate in TMEM, not with atomics: two runs are bit-identical."""
    shape = (2, 24, 40, 24, 40, 128, 2)
    B, H1, W1, H2, W2, C, Kc = shape
    F1, F2, A_u, A_v, g = make_inputs(shape, 6)
    gC_u = torch.randn(B, H1, W1, Kc, H2, generator=g)
    gC_v = torch.randn(B, H1, W1, Kc, W2, generator=g)
    args = [t.to(cuda_device) for t in (F1, F2, A_u, A_v, gC_u, gC_v)]
    a = ops.compression_backward(*args)
    b = ops.compression_backward(*args)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def test_golden_op_vectors(golden_dir, cuda_device):
    """CUDA ops against the vectors produced by the reference's own test definitions."""
    gold = np.load(os.path.join(golden_dir, "ops_b2_c12_8x12_k3.npz"))
    F1 = torch.from_numpy(gold["F1"]).float().to(cuda_device)
    F2 = torch.from_numpy(gold["F2"]).float().to(cuda_device)
    for level in range(3):
        x = F2.permute(0, 3, 1, 2)
        for _ in range(level):
            x = F.avg_pool2d(x, 2, stride=2)
        F2l = x.permute(0, 2, 3, 1).contiguous()
        MA_u, MA_v = ops.max_avg_forward(F1, F2l)
        for name, ours in (("max_u", MA_u[..., 0, :]), ("avg_u", MA_u[..., 1, :]),
                           ("max_v", MA_v[..., 0, :]), ("avg_v", MA_v[..., 1, :])):
            ref = torch.from_numpy(gold[f"l{level}_{name}"]).permute(0, 2, 3, 1)
            assert relerr(ours, ref) < TOL, (level, name)
        A_u = torch.from_numpy(gold[f"l{level}_A_u"]).float().to(cuda_device)
        A_v = torch.from_numpy(gold[f"l{level}_A_v"]).float().to(cuda_device)
        C_u, C_v = ops.compression_forward(F1, F2l, A_u, A_v)
        assert relerr(C_u, torch.from_numpy(gold[f"l{level}_C_u"]).permute(0, 3, 4, 1, 2)) < TOL
        assert relerr(C_v, torch.from_numpy(gold[f"l{level}_C_v"]).permute(0, 3, 4, 1, 2)) < TOL


@pytest.mark.parametrize("fuse_backward,channels_first,fuse_attention",
                         [(True, True, True), (True, True, False), (True, False, False), (False, False, False)])
def test_block_against_reference_dense_vectors(golden_dir, cuda_device, fuse_backward, channels_first, fuse_attention):
    """The whole call site (4 pyramid levels, Conv3d attention, autograd) on the GPU against the
    vectors of the reference's dense CorrBlock.  Gradients flow through argmax choices; the seeded
    case has no near-ties at the MARGIN level, so the same tolerance applies."""
    gold = np.load(os.path.join(golden_dir, "block_dense_b2_c16_9x11_k2.npz"))
    f1 = torch.from_numpy(gold["f1"]).float().to(cuda_device).requires_grad_(True)
    f2 = torch.from_numpy(gold["f2"]).float().to(cuda_device).requires_grad_(True)
    convs = []
    for i in range(2):
        conv = torch.nn.Conv3d(2, gold["w0"].shape[0], 3, padding=1).to(cuda_device)
        with torch.no_grad():
            conv.weight.copy_(torch.from_numpy(gold[f"w{i}"]).float())
            conv.bias.copy_(torch.from_numpy(gold[f"b{i}"]).float())
        convs.append(conv)
    blk = sfb.AlternateCorrBlockSepflow(f1, f2, None, support_backward=True, fuse_backward=fuse_backward,
                                        channels_first=channels_first, fuse_attention=fuse_attention)
    sep_u, sep_v = blk(None, sep=True, attention_weights=tuple(convs))
    assert relerr(sep_u, torch.from_numpy(gold["sep_u"])) < TOL
    assert relerr(sep_v, torch.from_numpy(gold["sep_v"])) < TOL
    gen = torch.Generator().manual_seed(int(gold["loss_seed"]))
    wu = torch.randn(sep_u.shape, generator=gen, dtype=torch.float64).float().to(cuda_device)
    wv = torch.randn(sep_v.shape, generator=gen, dtype=torch.float64).float().to(cuda_device)
    ((sep_u * wu).sum() + (sep_v * wv).sum()).backward()
    assert relerr(f1.grad, torch.from_numpy(gold["g_f1"])) < 2 * TOL
    assert relerr(f2.grad, torch.from_numpy(gold["g_f2"])) < 2 * TOL
    for i, conv in enumerate(convs):
        gw = torch.from_numpy(gold[f"g_w{i}"])
        assert relerr(conv.weight.grad, gw) < 2 * TOL
        # a bias shifts all logits of a softmax equally, so its gradient is ~0: compare on the weights' scale
        gb_err = (conv.bias.grad.double().cpu() - torch.from_numpy(gold[f"g_b{i}"])).abs().max().item()
        assert gb_err < 2 * TOL * gw.abs().max().item()


def test_ops_reject_bad_inputs(cuda_device):
    F1 = torch.randn(1, 4, 4, 8, device=cuda_device)
    with pytest.raises(RuntimeError, match="contiguous"):
        ops.max_avg_forward(F1.permute(0, 2, 1, 3), F1)
    with pytest.raises(RuntimeError, match="dtype"):
        ops.max_avg_forward(F1.half(), F1.half())
    with pytest.raises(RuntimeError, match="feature dimensions differ"):
        ops.max_avg_forward(F1, torch.randn(1, 4, 4, 12, device=cuda_device))
    with pytest.raises(RuntimeError, match="unsupported"):
        ops.max_avg_forward(torch.randn(1, 4, 4, 6, device=cuda_device), torch.randn(1, 4, 4, 6, device=cuda_device))
    with pytest.raises(RuntimeError, match="shape"):
        ops.compression_forward(F1, F1, torch.randn(1, 4, 4, 2, 5, device=cuda_device),
                                torch.randn(1, 4, 4, 2, 4, device=cuda_device))
