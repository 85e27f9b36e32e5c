"""GPU: the image-1 row partition on the device (what ``sharding.make_shard(prefer="rows")`` hands each rank).

One GPU plays every rank in turn: the call site runs on each rank's block of image-1 rows extended by its halo rows
(so the image-1 extent differs from image 2's and the blocks start in the middle of 128-pixel tiles), with no upstream
gradient on the halo rows, and the pieces are combined by hand the way the collectives combine them: interior rows of
the outputs, sum of the partial image-2 gradients, halo rows of the image-1 gradient added to the neighbouring block,
sum of the attention-parameter gradients.  The result must equal the unsharded run on the device and the float64 dense
path (autograd through oracle/separation_oracle.py, which restates core/corr.py:416-457).
"""
import pytest
import torch

import separableflowthesis_b200 as sfb
from separableflowthesis_b200 import sharding
from oracle import separation_oracle as orc

pytestmark = pytest.mark.gpu


def relerr(x, ref):
    den = max(x.abs().max().item(), ref.abs().max().item(), 1e-30)
    return (x.double().cpu() - ref.double().cpu()).abs().max().item() / den


def make_convs(Kc, g, dev):
    convs = []
    for _ in range(2):
        conv = torch.nn.Conv3d(2, Kc, 3, padding=1)
        with torch.no_grad():
            conv.weight.copy_(torch.randn(conv.weight.shape, generator=g) * 0.3)
            conv.bias.copy_(torch.randn(conv.bias.shape, generator=g) * 0.1)
        convs.append(conv.to(dev))
    return convs


def run_block(f1, f2, convs, gu, gv, keep=None):
    """Call site on (f1, f2); upstream gradients gu / gv apply to image-1 rows keep = (i0, i1) of the outputs."""
    a = f1.clone().requires_grad_(True)
    b = f2.clone().requires_grad_(True)
    for c in convs:
        c.zero_grad()
    blk = sfb.AlternateCorrBlockSepflow(a, b, None, num_levels=1, support_backward=True)
    su, sv = blk(None, sep=True, attention_weights=tuple(convs))
    if keep is not None:
        su, sv = su[:, :, :, keep[0]:keep[1]], sv[:, :, :, keep[0]:keep[1]]
    torch.autograd.backward([su, sv], [gu, gv])
    return (su.detach(), sv.detach(), a.grad, b.grad, [c.weight.grad.clone() for c in convs],
            [c.bias.grad.clone() for c in convs])


@pytest.mark.parametrize("blocks,kind", [(2, "tf32"), (3, "tf32"), (2, "fp16"), (3, "fp16")])
def test_row_blocks_combine_to_the_unsharded_result(blocks, kind, cuda_device):
    from separableflowthesis_b200 import ops
    with ops.sweep_operands(kind):
        _row_blocks_combine(blocks, kind, cuda_device)


def _row_blocks_combine(blocks, kind, cuda_device):
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    dev = cuda_device
    B, C, H, W, Kc = 2, 64, 21, 30, 2
    g = torch.Generator().manual_seed(2718)
    f1 = torch.randn(B, C, H, W, generator=g).to(dev)
    f2 = torch.randn(B, C, H, W, generator=g).to(dev)
    convs = make_convs(Kc, g, dev)
    gu = torch.randn(B, 2 + Kc, W, H, W, generator=g).to(dev)
    gv = torch.randn(B, 2 + Kc, H, H, W, generator=g).to(dev)
    full = run_block(f1, f2, convs, gu, gv)

    su = torch.zeros_like(full[0])
    sv = torch.zeros_like(full[1])
    g1 = torch.zeros_like(f1)
    g2 = torch.zeros_like(f2)
    gw = [torch.zeros_like(c.weight) for c in convs]
    gb = [torch.zeros_like(c.bias) for c in convs]
    for ri in range(blocks):
        sh = sharding.make_shard(B, H, blocks, ri, prefer="rows")
        assert (sh.b0, sh.b1) == (0, B)
        e0, e1, i0, i1 = sharding.halo_range(sh, H)
        part = run_block(f1[:, :, e0:e1].contiguous(), f2, convs, gu[:, :, :, sh.r0:sh.r1].contiguous(),
                         gv[:, :, :, sh.r0:sh.r1].contiguous(), keep=(i0, i1))
        su[:, :, :, sh.r0:sh.r1] = part[0]
        sv[:, :, :, sh.r0:sh.r1] = part[1]
        g1[:, :, e0:e1] += part[2]          # halo rows land on the neighbouring blocks' rows
        g2 += part[3]                       # partial sums over this block's image-1 pixels
        for i in range(2):
            gw[i] += part[4][i]
            gb[i] += part[5][i]
    # Same sweeps on the same features: with TF32 operands the outputs are identical.  With FP16 operands a block's
    # image-1 rows get their own power-of-two scale; scaling is exact except for the few values that land in FP16's
    # subnormal range under one scale and not the other, so the outputs agree to 1e-6 instead of bit for bit.  The
    # gradients are not bit-identical either way: at a block border dLoss/dS of a pixel is the sum of what two blocks
    # generate (the stencil's transpose reaches across the border), and each part is rounded on its own before its GEMM.
    if kind == "tf32":
        assert torch.equal(su, full[0]) and torch.equal(sv, full[1])
    else:
        assert relerr(su, full[0]) < 1e-6 and relerr(sv, full[1]) < 1e-6
    errs = {"g_fmap1": relerr(g1, full[2]), "g_fmap2": relerr(g2, full[3]), "g_weight1": relerr(gw[0], full[4][0]),
            "g_weight2": relerr(gw[1], full[4][1])}
    assert max(errs.values()) < 1e-3, errs
    for i in range(2):
        assert (gb[i] - full[5][i]).abs().max().item() < 1e-4 * max(full[4][i].abs().max().item(), 1.0)

    # and both against the float64 oracle: forward outputs directly; gradients with the oracle's backward evaluated on
    # the device forward's own argmax / attention weights (what autograd does), because a float64 forward breaks
    # near-ties of the max differently than TF32 operands and would route a few gradients elsewhere
    from separableflowthesis_b200 import ops
    scale = 1.0 / C ** 0.5
    params = []
    for c in convs:
        params += [c.weight.detach(), c.bias.detach()]
    fw = ops.separation_level_forward(f1, f2, *params, fmaps=True, scale1=scale)
    assert torch.equal(fw[0], full[0]) and torch.equal(fw[1], full[1])
    p64 = [t.double().cpu() for t in params]
    ref = orc.separation_level_forward(f1.double().cpu(), f2.double().cpu(), *p64, fmaps=True, scale1=scale)
    assert relerr(su, ref[0]) < 2e-3 and relerr(sv, ref[1]) < 2e-3
    rb = orc.separation_level_backward(f1.double().cpu(), f2.double().cpu(), p64[0], p64[2], fw[0].double().cpu(),
                                       fw[1].double().cpu(), fw[2].cpu(), fw[3].cpu(), fw[4].double().cpu(),
                                       fw[5].double().cpu(), gu.double().cpu(), gv.double().cpu(), fmaps=True, scale1=scale)
    assert relerr(g1, rb[0]) < 2e-3 and relerr(g2, rb[1]) < 2e-3
    assert relerr(gw[0], rb[2]) < 2e-3 and relerr(gw[1], rb[4]) < 2e-3
