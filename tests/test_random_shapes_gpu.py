"""GPU parity on seeded random shapes: the five ops of the reference's extension plus the one-call backward, against
the float64 oracle, with each 10-bit operand type (TF32 and the default scaled FP16).

The shapes are drawn so that the ragged cases meet each other: image widths that are not a multiple of the 16-column
tile, image-1 pixel counts that are not a multiple of the 128-pixel CTA tile, image 2 larger and smaller than image 1,
channel counts that are not a multiple of 8 (where FP16 operands fall back to TF32) or of 32 (a partial K block), and
compression channel counts on both sides of the four-per-sweep limit.  Inputs get a random overall scale between 1e-3
and 1e3, which the error measure (max error over max magnitude, scripts/test_model.py:251-256) is blind to and the
FP16 scaling has to follow.
"""
import numpy as np
import pytest
import torch

from separableflowthesis_b200 import ops
from oracle import separation_oracle as orc

pytestmark = pytest.mark.gpu

TOL = 1e-3


def relerr(x, ref):
    x = x.detach().double().cpu()
    ref = ref.detach().double().cpu()
    den = max(x.abs().max().item(), ref.abs().max().item(), 1e-300)
    return (x - ref).abs().max().item() / den


def draw_shapes(n, seed):
    rng = np.random.default_rng(seed)
    shapes = []
    for _ in range(n):
        B = int(rng.integers(1, 4))
        H1, W1 = int(rng.integers(1, 30)), int(rng.integers(1, 45))
        H2, W2 = int(rng.integers(1, 30)), int(rng.integers(1, 45))
        C = 4 * int(rng.integers(1, 66))
        Kc = int(rng.integers(1, 7))
        s1, s2, sg = (float(10.0 ** rng.uniform(-3, 3)) for _ in range(3))
        shapes.append((B, H1, W1, H2, W2, C, Kc, s1, s2, sg))
    return shapes


SHAPES = draw_shapes(24, 20240611)


def shape_id(s):
    return "b%d_%dx%d_%dx%d_c%d_k%d" % s[:7]


@pytest.mark.parametrize("operands", ["tf32", "fp16"])
@pytest.mark.parametrize("shape", SHAPES, ids=shape_id)
def test_all_ops_on_a_random_shape(shape, operands, cuda_device):
    B, H1, W1, H2, W2, C, Kc, s1, s2, sg = shape
    g = torch.Generator().manual_seed(int(np.dot(shape[:7], [1, 7, 49, 343, 2401, 16807, 117649])))
    F1 = torch.randn(B, H1, W1, C, generator=g) * (s1 / C ** 0.5)
    F2 = torch.randn(B, H2, W2, C, generator=g) * s2
    A_u = torch.randn(B, H1, W1, Kc, W2, generator=g).softmax(-1)
    A_v = torch.randn(B, H1, W1, Kc, H2, generator=g).softmax(-1)
    gMA_u = torch.randn(B, H1, W1, 2, H2, generator=g) * sg
    gMA_v = torch.randn(B, H1, W1, 2, W2, generator=g) * sg
    gC_u = torch.randn(B, H1, W1, Kc, H2, generator=g) * sg
    gC_v = torch.randn(B, H1, W1, Kc, W2, generator=g) * sg
    dev = lambda *ts: [t.to(cuda_device) for t in ts]
    dbl = lambda *ts: [t.double() for t in ts]

    r_u, r_v, AM_u, AM_v = orc.max_argmax_avg_forward(*dbl(F1, F2))
    S = orc.corr_volume(*dbl(F1, F2))
    scale = max(S.abs().max().item(), 1e-300)
    with ops.sweep_operands(operands):
        MA_u, MA_v, am_u, am_v = ops.max_argmax_avg_forward(*dev(F1, F2))
        MA_u2, MA_v2 = ops.max_avg_forward(*dev(F1, F2))
        C_u, C_v = ops.compression_forward(*dev(F1, F2, A_u, A_v))
        gm = ops.max_argmax_avg_backward(*dev(F1, F2, AM_u, AM_v, gMA_u, gMA_v))
        gc = ops.compression_backward(*dev(F1, F2, A_u, A_v, gC_u, gC_v))
        gs = ops.separation_backward(*dev(F1, F2, AM_u, AM_v, gMA_u, gMA_v, A_u, A_v, gC_u, gC_v))

    # forward: both channels of both directions; the chosen arg-max entries hold the maximum to tolerance
    assert relerr(MA_u, r_u) < TOL and relerr(MA_v, r_v) < TOL
    assert torch.equal(MA_u2, MA_u) and torch.equal(MA_v2, MA_v)
    am_u, am_v = am_u.cpu(), am_v.cpu()
    assert (am_u >= 0).all() and (am_u < W2).all() and (am_v >= 0).all() and (am_v < H2).all()
    picked_u = S.gather(4, am_u[..., 0, :].long().unsqueeze(-1)).squeeze(-1)
    picked_v = S.gather(3, am_v[..., 0, :].long().unsqueeze(-2)).squeeze(-2)
    assert (r_u[..., 0, :] - picked_u).abs().max().item() / scale < TOL
    assert (r_v[..., 0, :] - picked_v).abs().max().item() / scale < TOL
    rc_u, rc_v = orc.compression_forward(*dbl(F1, F2, A_u, A_v))
    assert relerr(C_u, rc_u) < TOL and relerr(C_v, rc_v) < TOL

    # backward: each op alone, and the one-call sum of both
    rm = orc.max_argmax_avg_backward(F1.double(), F2.double(), AM_u, AM_v, gMA_u.double(), gMA_v.double())
    rc = orc.compression_backward(*dbl(F1, F2, A_u, A_v, gC_u, gC_v))
    assert relerr(gm[0], rm[0]) < TOL and relerr(gm[1], rm[1]) < TOL
    for name, x, r in zip(("gF1", "gF2", "gA_u", "gA_v"), gc, rc):
        assert x.shape == r.shape and relerr(x, r) < TOL, name
    assert relerr(gs[0], rm[0] + rc[0]) < TOL and relerr(gs[1], rm[1] + rc[1]) < TOL
    assert relerr(gs[2], rc[2]) < TOL and relerr(gs[3], rc[3]) < TOL
