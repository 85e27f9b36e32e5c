"""GPU tests at BASELINE.json's full image sizes.

Two kinds of check: (1) the same oracle code run on the GPU in FP32 (plain torch matmul/einsum,
TF32 disabled) on image-1 row chunks, which is exact enough to act as the reference at sizes the
CPU cannot finish in seconds; (2) size-independent identities of the math:
  * scaling F2 by 2 scales every output by exactly 2 (power-of-two scaling commutes with rounding),
  * mean_u(mean_v S) computed from MA_u's mean channel equals the one from MA_v's,
  * uniform attention weights turn the compression channels into the mean channels,
  * <gF1, F1> = <gF2, F2> = <G, S> (S is bilinear), and for the compression op
    <G, S> = <gC_u, C_u> + <gC_v, C_v>, <gA_u, A_u> = <gC_u... see the asserts.
"""
import pytest
import torch

from separableflowthesis_b200 import ops
from oracle import separation_oracle as orc

pytestmark = pytest.mark.gpu
TOL = 1e-3


def relerr(x, ref):
    den = max(x.abs().max().item(), ref.abs().max().item(), 1e-30)
    return (x.double() - ref.double()).abs().max().item() / den


def features(B, H, W, C, Kc, dev, seed=1234):
    g = torch.Generator().manual_seed(seed)
    F1 = (torch.randn(B, H, W, C, generator=g) / C ** 0.5).to(dev)
    F2 = torch.randn(B, H, W, C, generator=g).to(dev)
    A_u = torch.randn(B, H, W, Kc, W, generator=g).softmax(-1).to(dev)
    A_v = torch.randn(B, H, W, Kc, H, generator=g).softmax(-1).to(dev)
    return F1, F2, A_u, A_v


# one sample each of configs 3 (55x128, Kc=4), 4 (47x156, Kc=2) and 5 (135x240, Kc=4)
FULL = [(55, 128, 4), (47, 156, 2), (135, 240, 4)]


@pytest.mark.parametrize("H,W,Kc", FULL)
def test_forward_against_fp32_torch_on_gpu(H, W, Kc, cuda_device):
    torch.backends.cuda.matmul.allow_tf32 = False
    F1, F2, A_u, A_v = features(1, H, W, 256, Kc, cuda_device)
    MA_u, MA_v, AM_u, AM_v = ops.max_argmax_avg_forward(F1, F2)
    C_u, C_v = ops.compression_forward(F1, F2, A_u, A_v)
    rows = slice(H // 2, H // 2 + 4)  # a 4-row band of image 1 through the dense FP32 path
    r_u, r_v, ra_u, ra_v = orc.max_argmax_avg_forward(F1[:, rows].contiguous(), F2)
    assert relerr(MA_u[:, rows], r_u) < TOL and relerr(MA_v[:, rows], r_v) < TOL
    S = orc.corr_volume(F1[:, rows].contiguous(), F2)
    picked = S.gather(4, AM_u[:, rows, :, 0, :].long().unsqueeze(-1)).squeeze(-1)
    assert relerr(picked, r_u[..., 0, :]) < TOL
    picked = S.gather(3, AM_v[:, rows, :, 0, :].long().unsqueeze(-2)).squeeze(-2)
    assert relerr(picked, r_v[..., 0, :]) < TOL
    agree = (AM_u[:, rows] == ra_u).float().mean().item()
    assert agree > 0.995  # the rest are near-ties flipped by TF32 rounding
    rc_u, rc_v = orc.compression_forward(F1[:, rows].contiguous(), F2, A_u[:, rows].contiguous(),
                                         A_v[:, rows].contiguous())
    assert relerr(C_u[:, rows], rc_u) < TOL and relerr(C_v[:, rows], rc_v) < TOL


@pytest.mark.parametrize("H,W,Kc", FULL)
def test_forward_identities(H, W, Kc, cuda_device):
    F1, F2, _, _ = features(1, H, W, 256, Kc, cuda_device, seed=7)
    MA_u, MA_v, AM_u, AM_v = ops.max_argmax_avg_forward(F1, F2)
    MA_u2, MA_v2, AM_u2, AM_v2 = ops.max_argmax_avg_forward(F1, F2 * 2)
    assert torch.equal(MA_u2, MA_u * 2) and torch.equal(MA_v2, MA_v * 2)
    assert torch.equal(AM_u2, AM_u) and torch.equal(AM_v2, AM_v)
    assert (MA_u[..., 0, :] >= MA_u[..., 1, :]).all() and (MA_v[..., 0, :] >= MA_v[..., 1, :]).all()
    m1 = MA_u[..., 1, :].double().mean(-1)
    m2 = MA_v[..., 1, :].double().mean(-1)
    assert (m1 - m2).abs().max().item() < TOL * MA_u[..., 1, :].abs().max().item()
    A_u = torch.full((1, H, W, Kc, W), 1.0 / W, device=cuda_device)
    A_v = torch.full((1, H, W, Kc, H), 1.0 / H, device=cuda_device)
    C_u, C_v = ops.compression_forward(F1, F2, A_u, A_v)
    for k in range(Kc):
        assert relerr(C_u[..., k, :], MA_u[..., 1, :]) < TOL
        assert relerr(C_v[..., k, :], MA_v[..., 1, :]) < TOL


@pytest.mark.parametrize("H,W,Kc", FULL)
def test_backward_identities_and_band(H, W, Kc, cuda_device):
    torch.backends.cuda.matmul.allow_tf32 = False
    F1, F2, A_u, A_v = features(1, H, W, 256, Kc, cuda_device, seed=11)
    g = torch.Generator(device=cuda_device).manual_seed(5)
    MA_u, MA_v, AM_u, AM_v = ops.max_argmax_avg_forward(F1, F2)
    gMA_u = torch.randn(MA_u.shape, generator=g, device=cuda_device)
    gMA_v = torch.randn(MA_v.shape, generator=g, device=cuda_device)
    gF1, gF2 = ops.max_argmax_avg_backward(F1, F2, AM_u, AM_v, gMA_u, gMA_v)
    lhs = (gF1.double() * F1.double()).sum().item()
    rhs = (gF2.double() * F2.double()).sum().item()
    gs = (gMA_u.double() * MA_u.double()).sum().item() + (gMA_v.double() * MA_v.double()).sum().item()
    scale = gF1.double().abs().sum().item() * F1.abs().max().item()
    assert abs(lhs - rhs) < TOL * scale and abs(lhs - gs) < TOL * scale
    rows = slice(H // 3, H // 3 + 3)
    r1, _ = orc.max_argmax_avg_backward(F1[:, rows].contiguous(), F2, AM_u[:, rows].contiguous(),
                                        AM_v[:, rows].contiguous(), gMA_u[:, rows].contiguous(),
                                        gMA_v[:, rows].contiguous())
    assert relerr(gF1[:, rows], r1) < TOL

    C_u, C_v = ops.compression_forward(F1, F2, A_u, A_v)
    gC_u = torch.randn(C_u.shape, generator=g, device=cuda_device)
    gC_v = torch.randn(C_v.shape, generator=g, device=cuda_device)
    gF1, gF2, gA_u, gA_v = ops.compression_backward(F1, F2, A_u, A_v, gC_u, gC_v)
    lhs = (gF1.double() * F1.double()).sum().item()
    rhs = (gF2.double() * F2.double()).sum().item()
    cu = (gC_u.double() * C_u.double()).sum().item()
    cv = (gC_v.double() * C_v.double()).sum().item()
    scale = gF1.double().abs().sum().item() * F1.abs().max().item()
    assert abs(lhs - rhs) < TOL * scale and abs(lhs - (cu + cv)) < TOL * scale
    sa = gA_u.double().abs().sum().item() * A_u.max().item()
    assert abs((gA_u.double() * A_u.double()).sum().item() - cv) < TOL * sa
    assert abs((gA_v.double() * A_v.double()).sum().item() - cu) < TOL * sa
    band = [t[:, rows].contiguous() for t in (F1, A_u, A_v, gC_u, gC_v)]
    r = orc.compression_backward(band[0], F2, band[1], band[2], band[3], band[4])
    assert relerr(gF1[:, rows], r[0]) < TOL
    assert relerr(gA_u[:, rows], r[2]) < TOL and relerr(gA_v[:, rows], r[3]) < TOL


def test_gF2_against_fp32_torch_full_sum(cuda_device):
    """gF2 sums over ALL image-1 pixels, so check it whole on the config-3 size via row chunks."""
    torch.backends.cuda.matmul.allow_tf32 = False
    H, W, Kc = 55, 128, 4
    F1, F2, A_u, A_v = features(1, H, W, 256, Kc, cuda_device, seed=13)
    g = torch.Generator(device=cuda_device).manual_seed(6)
    gC_u = torch.randn(1, H, W, Kc, H, generator=g, device=cuda_device)
    gC_v = torch.randn(1, H, W, Kc, W, generator=g, device=cuda_device)
    out = ops.compression_backward(F1, F2, A_u, A_v, gC_u, gC_v)
    ref = orc.compression_backward(F1, F2, A_u, A_v, gC_u, gC_v)
    for x, r in zip(out, ref):
        assert relerr(x, r) < TOL
    MA_u, MA_v, AM_u, AM_v = ops.max_argmax_avg_forward(F1, F2)
    gMA_u = torch.randn(MA_u.shape, generator=g, device=cuda_device)
    gMA_v = torch.randn(MA_v.shape, generator=g, device=cuda_device)
    out = ops.max_argmax_avg_backward(F1, F2, AM_u, AM_v, gMA_u, gMA_v)
    ref = orc.max_argmax_avg_backward(F1, F2, AM_u, AM_v, gMA_u, gMA_v)
    for x, r in zip(out, ref):
        assert relerr(x, r) < TOL


def test_call_site_variants_agree_at_full_size(cuda_device):
    """One sample of config 5 (135x240, C=256, Kc=4), two pyramid levels: the call site as one autograd node (library
    stencil kernels for the attention modules, library resampling + concatenation) against the op-by-op call site
    (torch's Conv3d / softmax / F.interpolate / torch.cat around the same sweeps).  Both use the same TF32 sweeps,
    so they must agree far inside the TF32 tolerance: this checks the attention, resampling and placement kernels
    and the one-call backward at the full image size."""
    import separableflowthesis_b200 as sfb
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    H, W, C, Kc = 135, 240, 256, 4
    g = torch.Generator().manual_seed(99)
    f1 = torch.randn(1, C, H, W, generator=g).to(cuda_device)
    f2 = torch.randn(1, C, H, W, generator=g).to(cuda_device)
    convs = []
    for _ in range(2):
        conv = torch.nn.Conv3d(2, Kc, 3, padding=1)
        with torch.no_grad():
            conv.weight.copy_(torch.randn(conv.weight.shape, generator=g) * 0.1)
            conv.bias.copy_(torch.randn(conv.bias.shape, generator=g) * 0.1)
        convs.append(conv.to(cuda_device))
    gd = torch.Generator(device=cuda_device).manual_seed(7)
    results = []
    for fuse_attention in (True, False):
        a = f1.clone().requires_grad_(True)
        b = f2.clone().requires_grad_(True)
        for c in convs:
            c.zero_grad()
        blk = sfb.AlternateCorrBlockSepflow(a, b, None, num_levels=2, support_backward=True,
                                            fuse_attention=fuse_attention)
        su, sv = blk(None, sep=True, attention_weights=tuple(convs))
        if not results:
            up = (torch.randn(su.shape, generator=gd, device=cuda_device),
                  torch.randn(sv.shape, generator=gd, device=cuda_device))
        torch.autograd.backward([su, sv], list(up))
        results.append([su.detach(), sv.detach(), a.grad, b.grad] + [c.weight.grad.clone() for c in convs])
        del su, sv, blk
    names = ("sep_u", "sep_v", "g_fmap1", "g_fmap2", "g_weight1", "g_weight2")
    for name, x, y in zip(names, results[0], results[1]):
        assert x.shape == y.shape and relerr(x, y) < 2e-4, (name, relerr(x, y))
