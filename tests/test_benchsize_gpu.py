"""GPU: the entry points the benchmark times, checked against the oracle at the sizes it times them.

``bench.py`` measures ``sfb_separation_level_forward`` / ``_backward`` (one pyramid level of the call site,
core/corr.py:416-457, in one library call each way) on BASELINE config 5 (135x240, C=256, Kc=4) and, for the BF16
configuration, config 4 (B=8, 47x156, Kc=2).  The CPU oracle cannot finish those sizes in seconds, so the same
oracle code (oracle/separation_oracle.py: dense matmul -> max/mean -> Conv3d/softmax -> einsum, image-1 row
chunks) runs on the GPU in FP32 with TF32 switched off everywhere; its own error (~1e-6) is far inside the
tolerances below.  The comparison is the one the reference's tests make (scripts/test_compression_autograd.py:442-484,
scripts/test_model.py:251-256): max |x - ref| over max(|x|max, |ref|max).

Tolerances: 1e-3 for gradients and attention gradients (FP16 operands by default, TF32 on request: both keep 10
mantissa bits; FP32 accumulation), 2e-3 for whole-level outputs (their attention weights are a softmax of
max/avg values of that accuracy); for BF16 operands 2e-5 on
the max channel against the oracle on BF16-rounded features (products of BF16 values are exact in FP32), 4e-3 on the
other forward outputs and 1e-2 on the backward against the unrounded oracle.
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


def no_tf32():
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False


def level_inputs(B, H, W, C, Kc, dev, seed):
    """Seeded N(0,1) features (image 1 pre-scaled by 1/sqrt(C), core/corr.py:419), N(0, 0.02)-grade attention
    parameters as BASELINE config 2 states them, N(0,1) upstream gradients."""
    g = torch.Generator().manual_seed(seed)
    F1 = (torch.randn(B, H, W, C, generator=g) / C ** 0.5).to(dev)
    F2 = torch.randn(B, H, W, C, generator=g).to(dev)
    params = [(torch.randn(Kc, 2, 3, 3, 3, generator=g) * 0.02).to(dev), (torch.randn(Kc, generator=g) * 0.02).to(dev),
              (torch.randn(Kc, 2, 3, 3, 3, generator=g) * 0.02).to(dev), (torch.randn(Kc, generator=g) * 0.02).to(dev)]
    gd = torch.Generator(device=dev).manual_seed(seed + 1)
    g_sep_u = torch.randn(B, 2 + Kc, W, H, W, generator=gd, device=dev)
    g_sep_v = torch.randn(B, 2 + Kc, H, H, W, generator=gd, device=dev)
    return F1, F2, params, g_sep_u, g_sep_v


def check_level(F1, F2, params, g_sep_u, g_sep_v, fmaps):
    """Forward and backward of one level through the library, every output against the oracle run on the same
    device in FP32; the backward is evaluated with the device forward's own argmax / attention weights, as autograd
    does.  gF2 is compared whole: the oracle accumulates it over all image-1 row chunks."""
    wu, bu, wv, bv = params
    C = F1.shape[-1]
    scale = 1.0
    a1, a2 = F1, F2
    if fmaps:   # the model's (B, C, H, W) maps, unscaled; the library scales image 1 on the way in
        scale = 1.0 / C ** 0.5
        a1 = (F1 * C ** 0.5).permute(0, 3, 1, 2).contiguous()
        a2 = F2.permute(0, 3, 1, 2).contiguous()
    fw = ops.separation_level_forward(a1, a2, wu, bu, wv, bv, fmaps=fmaps, scale1=scale)
    ref = orc.separation_level_forward(a1, a2, wu, bu, wv, bv, fmaps=fmaps, scale1=scale)
    for name, i in (("sep_u", 0), ("sep_v", 1), ("a_u", 4), ("a_v", 5)):
        assert fw[i].shape == ref[i].shape
        assert relerr(fw[i], ref[i]) < 2 * TOL, (name, relerr(fw[i], ref[i]))
    agree = (fw[2] == ref[2]).float().mean().item()
    assert agree > 0.995, agree   # the rest are near-ties flipped by TF32 rounding
    del ref
    bw = ops.separation_level_backward(a1, a2, wu, wv, *fw, g_sep_u, g_sep_v, fmaps=fmaps, scale1=scale)
    rb = orc.separation_level_backward(a1, a2, wu, wv, *fw, g_sep_u, g_sep_v, fmaps=fmaps, scale1=scale)
    for name, i in (("gF1", 0), ("gF2", 1), ("gweight_u", 2), ("gweight_v", 4)):
        assert bw[i].shape == rb[i].shape
        assert relerr(bw[i], rb[i]) < TOL, (name, relerr(bw[i], rb[i]))
    for name, i in (("gbias_u", 3), ("gbias_v", 5)):   # measured against the scale of the weight gradients
        den = max(rb[i - 1].abs().max().item(), 1.0)
        assert (bw[i].double() - rb[i].double()).abs().max().item() < TOL * den, name


@pytest.mark.parametrize("fmaps", [False, True])
def test_level_at_config5_size_one_sample(fmaps, cuda_device):
    """One sample of BASELINE config 5 (135x240, C=256, Kc=4): the per-sample work of the benchmarked step."""
    no_tf32()
    F1, F2, params, gu, gv = level_inputs(1, 135, 240, 256, 4, cuda_device, seed=501)
    check_level(F1, F2, params, gu, gv, fmaps)


def test_level_at_benchmarked_batch(cuda_device):
    """B=8, the benchmarked batch (sample strides of every view), at BASELINE config 4's size (47x156, Kc=2)."""
    no_tf32()
    F1, F2, params, gu, gv = level_inputs(8, 47, 156, 256, 2, cuda_device, seed=502)
    check_level(F1, F2, params, gu, gv, fmaps=True)


def test_level_bf16_operands_at_config4_size(cuda_device):
    """BASELINE config 4's operand type at its image size (two samples): BF16 operands in the sweeps."""
    no_tf32()
    F1, F2, params, gu, gv = level_inputs(2, 47, 156, 256, 2, cuda_device, seed=503)
    wu, bu, wv, bv = params
    with ops.sweep_operands("bf16"):
        fw = ops.separation_level_forward(F1, F2, wu, bu, wv, bv)
        bw = ops.separation_level_backward(F1, F2, wu, wv, *fw, gu, gv)
    F1b, F2b = F1.bfloat16().float(), F2.bfloat16().float()
    ref = orc.separation_level_forward(F1b, F2b, wu, bu, wv, bv)
    # channel 0 = max: exact products, only the accumulation order differs
    assert relerr(fw[0][:, 0], ref[0][:, 0]) < 2e-5 and relerr(fw[1][:, 0], ref[1][:, 0]) < 2e-5
    assert relerr(fw[0], ref[0]) < 4e-3 and relerr(fw[1], ref[1]) < 4e-3
    ref32 = orc.separation_level_forward(F1, F2, wu, bu, wv, bv)
    assert relerr(fw[0], ref32[0]) < 1e-2 and relerr(fw[1], ref32[1]) < 1e-2
    rb = orc.separation_level_backward(F1, F2, wu, wv, *fw, gu, gv)
    for i in (0, 1, 2, 4):
        assert relerr(bw[i], rb[i]) < 1e-2, i


def test_lookup_radius_beyond_register_window(cuda_device):
    """CorrBlock1D lookup (core/corr.py:576-624) with radius 6: more taps than the kernel's in-register window
    holds, which takes its general path."""
    B, dim, D, H1, W1, levels, radius = 2, 1, 48, 9, 14, 3, 6
    g = torch.Generator().manual_seed(77)
    corr = torch.randn(B, dim, D, H1, W1, generator=g)
    coord = torch.rand(B, H1, W1, generator=g) * (D + 6) - 3      # some positions outside the volume
    gout = torch.randn(B, levels * dim * (2 * radius + 1), H1, W1, generator=g)
    dev = cuda_device
    for clamp in (False, True):
        c = coord / D if clamp else coord
        pyr = ops.lookup_build_pyramid(corr.to(dev), levels)
        out = ops.lookup_forward(corr.to(dev), pyr, c.to(dev), levels, radius, clamp)
        ref = orc.lookup_forward(corr.double(), c.double(), levels, radius, clamp)
        assert relerr(out.cpu(), ref) < 5e-5
        gc = ops.lookup_backward(tuple(corr.shape), c.to(dev), gout.to(dev), levels, radius, clamp)
        rg = orc.lookup_backward(tuple(corr.shape), c.double(), gout.double(), levels, radius, clamp)
        assert relerr(gc.cpu(), rg) < 5e-5


@pytest.mark.parametrize("shape", [(2, 47, 156, 47, 156, 256, 2), (1, 13, 22, 11, 19, 64, 3)])
def test_five_ops_with_bf16_operands(shape, cuda_device):
    """The five reference-layout ops (MemorySaver_cuda.cpp:105-112) with BF16 operands in every contraction (BASELINE
    config 4's operand type), at its image size and on a ragged small case.  Forward ops against the oracle on
    BF16-rounded features (max channel: exact products, 2e-5; sums 4e-3); backward ops, whose generated operand is
    rounded to BF16 as well, against the unrounded oracle with 1e-2."""
    no_tf32()
    B, H1, W1, H2, W2, C, Kc = shape
    dev = cuda_device
    g = torch.Generator(device=dev).manual_seed(601)
    F1 = torch.randn(B, H1, W1, C, generator=g, device=dev) / C ** 0.5
    F2 = torch.randn(B, H2, W2, C, generator=g, device=dev)
    A_u = torch.softmax(torch.randn(B, H1, W1, Kc, W2, generator=g, device=dev), -1)
    A_v = torch.softmax(torch.randn(B, H1, W1, Kc, H2, generator=g, device=dev), -1)
    gMA_u = torch.randn(B, H1, W1, 2, H2, generator=g, device=dev)
    gMA_v = torch.randn(B, H1, W1, 2, W2, generator=g, device=dev)
    gC_u = torch.randn(B, H1, W1, Kc, H2, generator=g, device=dev)
    gC_v = torch.randn(B, H1, W1, Kc, W2, generator=g, device=dev)
    with ops.sweep_operands("bf16"):
        MA_u, MA_v, AM_u, AM_v = ops.max_argmax_avg_forward(F1, F2)
        MA_u2, MA_v2 = ops.max_avg_forward(F1, F2)
        C_u, C_v = ops.compression_forward(F1, F2, A_u, A_v)
        gF1m, gF2m = ops.max_argmax_avg_backward(F1, F2, AM_u, AM_v, gMA_u, gMA_v)
        gF1c, gF2c, gA_u, gA_v = ops.compression_backward(F1, F2, A_u, A_v, gC_u, gC_v)
    F1b, F2b = F1.bfloat16().float(), F2.bfloat16().float()
    rMA_u, rMA_v, rAM_u, rAM_v = orc.max_argmax_avg_forward(F1b, F2b)
    assert torch.equal(MA_u, MA_u2) and torch.equal(MA_v, MA_v2)
    assert relerr(MA_u[..., 0, :], rMA_u[..., 0, :]) < 2e-5 and relerr(MA_v[..., 0, :], rMA_v[..., 0, :]) < 2e-5
    assert relerr(MA_u, rMA_u) < 4e-3 and relerr(MA_v, rMA_v) < 4e-3
    assert (AM_u == rAM_u).float().mean().item() > 0.99 and (AM_v == rAM_v).float().mean().item() > 0.99
    rC_u, rC_v = orc.compression_forward(F1b, F2b, A_u, A_v)
    assert relerr(C_u, rC_u) < 4e-3 and relerr(C_v, rC_v) < 4e-3
    r1, r2 = orc.max_argmax_avg_backward(F1, F2, AM_u, AM_v, gMA_u, gMA_v)
    assert relerr(gF1m, r1) < 1e-2 and relerr(gF2m, r2) < 1e-2
    rc = orc.compression_backward(F1, F2, A_u, A_v, gC_u, gC_v)
    for name, x, r in zip(("gF1", "gF2", "gA_u", "gA_v"), (gF1c, gF2c, gA_u, gA_v), rc):
        assert relerr(x, r) < 1e-2, name


@pytest.mark.parametrize("kind", ["tf32", "fp16"])
def test_level_with_each_10_bit_operand_type(kind, cuda_device):
    """The default (FP16 operands with per-tensor power-of-two scaling) and the TF32 path, one sample at BASELINE
    config 4's size, against the same oracle with the same tolerances."""
    no_tf32()
    F1, F2, params, gu, gv = level_inputs(1, 47, 156, 256, 2, cuda_device, seed=504)
    with ops.sweep_operands(kind):
        check_level(F1, F2, params, gu, gv, fmaps=False)
        check_level(F1, F2, params, gu, gv, fmaps=True)


@pytest.mark.parametrize("scales", [(1e4, 3e3, 1e-7), (1e-5, 1e-6, 1e5), (1.0, 1.0, 1e-10)])
def test_fp16_operands_follow_the_scale_of_the_inputs(scales, cuda_device):
    """FP16 has five exponent bits; the library multiplies every tensor that becomes an FP16 operand by a power of two
    found on the device from its largest magnitude, and undoes it when results are stored.  Features and upstream
    gradients far outside FP16's range must therefore give the same accuracy as at unit scale (the attention filters are
    scaled inversely so that the softmax stays unsaturated)."""
    no_tf32()
    fs1, fs2, gs = scales
    F1, F2, params, gu, gv = level_inputs(1, 24, 40, 256, 2, cuda_device, seed=505)
    wu, bu, wv, bv = params
    params = [wu / (fs1 * fs2), bu, wv / (fs1 * fs2), bv]
    with ops.sweep_operands("fp16"):
        check_level(F1 * fs1, F2 * fs2, params, gu * gs, gv * gs, fmaps=False)


def test_five_ops_with_tf32_and_fp16_operands_agree(cuda_device):
    """The five reference-layout ops under the two 10-bit operand types, including weights far above 1 in the
    compression backward (the weights of that op need not be softmax outputs): each within 1e-3 of the oracle."""
    no_tf32()
    B, H1, W1, H2, W2, C, Kc = 1, 13, 22, 11, 19, 64, 3
    dev = cuda_device
    g = torch.Generator(device=dev).manual_seed(602)
    F1 = torch.randn(B, H1, W1, C, generator=g, device=dev) / C ** 0.5
    F2 = torch.randn(B, H2, W2, C, generator=g, device=dev)
    A_u = torch.randn(B, H1, W1, Kc, W2, generator=g, device=dev) * 300.0
    A_v = torch.randn(B, H1, W1, Kc, H2, generator=g, device=dev) * 300.0
    gMA_u = torch.randn(B, H1, W1, 2, H2, generator=g, device=dev) * 1e-6
    gMA_v = torch.randn(B, H1, W1, 2, W2, generator=g, device=dev) * 1e-6
    gC_u = torch.randn(B, H1, W1, Kc, H2, generator=g, device=dev) * 1e-6
    gC_v = torch.randn(B, H1, W1, Kc, W2, generator=g, device=dev) * 1e-6
    _, _, AM_u, AM_v = orc.max_argmax_avg_forward(F1, F2)
    r_ma = orc.max_argmax_avg_forward(F1, F2)
    r_c = orc.compression_forward(F1, F2, A_u, A_v)
    r_mb = orc.max_argmax_avg_backward(F1, F2, AM_u, AM_v, gMA_u, gMA_v)
    r_cb = orc.compression_backward(F1, F2, A_u, A_v, gC_u, gC_v)
    r_sb = orc.separation_backward(F1, F2, AM_u, AM_v, gMA_u, gMA_v, A_u, A_v, gC_u, gC_v)
    for kind in ("tf32", "fp16"):
        with ops.sweep_operands(kind):
            ma = ops.max_argmax_avg_forward(F1, F2)
            c = ops.compression_forward(F1, F2, A_u, A_v)
            mb = ops.max_argmax_avg_backward(F1, F2, AM_u, AM_v, gMA_u, gMA_v)
            cb = ops.compression_backward(F1, F2, A_u, A_v, gC_u, gC_v)
            sb = ops.separation_backward(F1, F2, AM_u, AM_v, gMA_u, gMA_v, A_u, A_v, gC_u, gC_v)
        for got, ref in ((ma[:2], r_ma[:2]), (c, r_c), (mb, r_mb), (cb, r_cb), (sb, r_sb)):
            for x, r in zip(got, ref):
                assert relerr(x, r) < TOL, kind


def test_fp16_operand_scaling_edge_cases(cuda_device):
    """Inputs that give the scale search nothing to work with: all-zero features (largest magnitude 0: scale 1, every
    output 0, the arg-max the lowest index as for any tie), and all-zero upstream gradients (every gradient exactly 0).
    No NaN or Inf may come out of the scale arithmetic."""
    dev = cuda_device
    F1, F2, params, gu, gv = level_inputs(1, 9, 14, 64, 2, dev, seed=506)
    wu, bu, wv, bv = params
    with ops.sweep_operands("fp16"):
        fw0 = ops.separation_level_forward(torch.zeros_like(F1), torch.zeros_like(F2), wu, bu, wv, bv)
        assert all(torch.isfinite(t.float()).all() for t in fw0)
        assert fw0[0][:, :2].abs().max().item() == 0.0 and fw0[1][:, :2].abs().max().item() == 0.0
        assert fw0[2].abs().max().item() == 0 and fw0[3].abs().max().item() == 0
        fw = ops.separation_level_forward(F1, F2, wu, bu, wv, bv)
        bw0 = ops.separation_level_backward(F1, F2, wu, wv, *fw, torch.zeros_like(gu), torch.zeros_like(gv))
        for t in bw0:
            assert torch.isfinite(t).all() and t.abs().max().item() == 0.0
        # one feature map zero, the other not: S = 0 everywhere, gradients flow only to the zero map
        bwz = ops.separation_level_backward(torch.zeros_like(F1), F2, wu, wv,
                                            *ops.separation_level_forward(torch.zeros_like(F1), F2, wu, bu, wv, bv), gu, gv)
        assert all(torch.isfinite(t).all() for t in bwz)
        assert bwz[1].abs().max().item() == 0.0      # gF2 = G^T * F1 with F1 = 0
        assert bwz[0].abs().max().item() > 0.0       # gF1 = G * F2
