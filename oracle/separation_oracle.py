"""CPU restatement of the reference's cost-volume separation ops.  TEST INFRASTRUCTURE ONLY.

This file is the checker for the CUDA path and the timed CPU baseline; the
product (``separableflowthesis_b200``) never imports it.  It restates, with
dense torch CPU tensor algebra, what the reference's five ``MemorySaver.*``
native ops compute (libs/MemorySaver/src/MemorySaver_cuda.cpp:105-112) in the
formulation the reference's own dense path uses
(core/corr.py:251-302 ``CorrBlock.corr_compute`` and core/corr.py:40-165
``CorrBlock.separate``: matmul -> max/mean over one displacement axis ->
einsum with the attention weights).

Parity pin: ``tests/golden/make_golden.py`` imports the reference's own
``CorrBlock`` and ``AlternateCorrBlockSepflow`` (core/corr.py) in a container
that has the reference checkout, runs them on seeded inputs (with these
functions plugged under the reference's own ``functions/MemorySaver.py``
wrappers for the memory-saving block) and stores the outputs; the CPU test
suite checks this file against those stored vectors.

Conventions (identical to the reference ops):
  F1   (B, H1, W1, C)   image-1 features, already scaled by 1/sqrt(C) by the caller
                        (core/corr.py:419)
  F2   (B, H2, W2, C)   image-2 features of one pyramid level (core/corr.py:422)
  S[b,i,j,u,v] = sum_c F1[b,i,j,c] * F2[b,u,v,c]   (never stored by the product)
  MA_u (B, H1, W1, 2, H2): [...,0,u] = max_v S, [...,1,u] = mean_v S
  MA_v (B, H1, W1, 2, W2): [...,0,v] = max_u S, [...,1,v] = mean_u S
  AM_u (B, H1, W1, 1, H2) int32 = argmax_v S (lowest v on ties,
        MemorySaver_kernel_forward.cu:498-507), AM_v likewise over u
  A_u  (B, H1, W1, Kc, W2), A_v (B, H1, W1, Kc, H2): attention weights
  C_u  (B, H1, W1, Kc, H2) = sum_v S * A_u ; C_v (B, H1, W1, Kc, W2) = sum_u S * A_v
        (MemorySaver_kernel_forward.cu:712-726)

Every function works on row chunks of image 1 so that the dense volume of one
chunk, not of the whole image, is what lives in host memory.
"""
from __future__ import annotations

import torch

__all__ = [
    "corr_volume",
    "max_avg_forward",
    "max_argmax_avg_forward",
    "max_argmax_avg_backward",
    "compression_forward",
    "compression_backward",
    "compression_attention_backward",
    "separation_feature_backward",
    "separation_backward",
    "max_argmax_avg_forward_cf",
    "compression_forward_cf",
    "compression_attention_backward_cf",
    "separation_feature_backward_cf",
    "top2_margins",
]


def _row_chunks(H1: int, W1: int, H2: int, W2: int, budget_elems: int = 1 << 26):
    """Yield (r0, r1) image-1 row ranges whose dense volume stays under ``budget_elems``."""
    per_row = max(1, W1 * H2 * W2)
    step = max(1, budget_elems // per_row)
    r0 = 0
    while r0 < H1:
        yield r0, min(H1, r0 + step)
        r0 += step


def corr_volume(F1: torch.Tensor, F2: torch.Tensor) -> torch.Tensor:
    """S (B,H1,W1,H2,W2) as in core/corr.py:286-289 (scale already folded into F1)."""
    B, H1, W1, C = F1.shape
    _, H2, W2, _ = F2.shape
    S = torch.matmul(F1.reshape(B, H1 * W1, C), F2.reshape(B, H2 * W2, C).transpose(1, 2))
    return S.reshape(B, H1, W1, H2, W2)


def _first_argmax(S: torch.Tensor, dim: int) -> torch.Tensor:
    """Index of the maximum along ``dim`` with the LOWEST index winning ties.

    The reference kernel updates on strict ``<`` while scanning upward
    (MemorySaver_kernel_forward.cu:498-507), hence first occurrence.
    """
    m = S.max(dim=dim, keepdim=True).values
    n = S.shape[dim]
    shape = [1] * S.dim()
    shape[dim] = n
    idx = torch.arange(n, dtype=torch.int64, device=S.device).reshape(shape)
    cand = torch.where(S == m, idx, torch.full_like(idx, n))
    return cand.min(dim=dim).values


def max_argmax_avg_forward(F1: torch.Tensor, F2: torch.Tensor):
    """Restates MemorySaver.max_argmax_avg_forward (MemorySaver_cuda.cpp:23-34;
    kernel MemorySaver_kernel_forward.cu:328-533).  Returns [MA_u, MA_v, AM_u, AM_v]."""
    B, H1, W1, C = F1.shape
    _, H2, W2, _ = F2.shape
    MA_u = F1.new_empty(B, H1, W1, 2, H2)
    MA_v = F1.new_empty(B, H1, W1, 2, W2)
    AM_u = torch.empty(B, H1, W1, 1, H2, dtype=torch.int32, device=F1.device)
    AM_v = torch.empty(B, H1, W1, 1, W2, dtype=torch.int32, device=F1.device)
    for r0, r1 in _row_chunks(H1, W1, H2, W2):
        S = corr_volume(F1[:, r0:r1], F2)
        MA_u[:, r0:r1, :, 0] = S.max(dim=4).values
        MA_u[:, r0:r1, :, 1] = S.mean(dim=4)
        MA_v[:, r0:r1, :, 0] = S.max(dim=3).values
        MA_v[:, r0:r1, :, 1] = S.mean(dim=3)
        AM_u[:, r0:r1, :, 0] = _first_argmax(S, 4).to(torch.int32)
        AM_v[:, r0:r1, :, 0] = _first_argmax(S, 3).to(torch.int32)
    return [MA_u, MA_v, AM_u, AM_v]


def max_avg_forward(F1: torch.Tensor, F2: torch.Tensor):
    """Restates MemorySaver.max_avg_forward (MemorySaver_cuda.cpp:10-21; kernel
    MemorySaver_kernel_forward.cu:128-313).  Returns [MA_u, MA_v]."""
    return max_argmax_avg_forward(F1, F2)[:2]


def _maxavg_G(AM_u, AM_v, gMA_u, gMA_v, H2, W2):
    """Dense gradient of the loss w.r.t. S for a chunk of image-1 rows:
    one-hot of the argmax times the max-gradient plus the spread mean-gradient
    (MemorySaver_kernel_max_avg_argmax_backward.cu:200-251)."""
    B, h, W1 = AM_u.shape[:3]
    G = gMA_u.new_zeros(B, h, W1, H2, W2)
    G += (gMA_u[..., 1, :] / W2).unsqueeze(-1)
    G += (gMA_v[..., 1, :] / H2).unsqueeze(-2)
    G.scatter_add_(4, AM_u[..., 0, :].to(torch.int64).unsqueeze(-1), gMA_u[..., 0, :].unsqueeze(-1))
    G.scatter_add_(3, AM_v[..., 0, :].to(torch.int64).unsqueeze(-2), gMA_v[..., 0, :].unsqueeze(-2))
    return G


def max_argmax_avg_backward(F1, F2, AM_u, AM_v, gMA_u, gMA_v):
    """Restates MemorySaver.max_argmax_avg_backward (MemorySaver_cuda.cpp:55-78;
    kernel MemorySaver_kernel_max_avg_argmax_backward.cu:47-317).  Returns [gF1, gF2]."""
    B, H1, W1, C = F1.shape
    _, H2, W2, _ = F2.shape
    gF1 = torch.zeros_like(F1)
    gF2 = torch.zeros_like(F2)
    F2f = F2.reshape(B, H2 * W2, C)
    for r0, r1 in _row_chunks(H1, W1, H2, W2):
        G = _maxavg_G(AM_u[:, r0:r1], AM_v[:, r0:r1], gMA_u[:, r0:r1], gMA_v[:, r0:r1], H2, W2)
        Gf = G.reshape(B, (r1 - r0) * W1, H2 * W2)
        gF1[:, r0:r1] = torch.matmul(Gf, F2f).reshape(B, r1 - r0, W1, C)
        gF2 += torch.matmul(Gf.transpose(1, 2), F1[:, r0:r1].reshape(B, -1, C)).reshape(B, H2, W2, C)
    return [gF1, gF2]


def compression_forward(F1, F2, A_u, A_v):
    """Restates MemorySaver.compression_forward for ANY Kc (MemorySaver_cuda.cpp:36-53).
    The reference kernel hard-codes Kc=2 (MemorySaver_kernel_forward.cu:20,1061); for other
    Kc the definition is the dense einsum of core/corr.py:128,140.  Returns [C_u, C_v]."""
    B, H1, W1, C = F1.shape
    _, H2, W2, _ = F2.shape
    Kc = A_u.shape[3]
    C_u = F1.new_empty(B, H1, W1, Kc, H2)
    C_v = F1.new_empty(B, H1, W1, Kc, W2)
    for r0, r1 in _row_chunks(H1, W1, H2, W2):
        S = corr_volume(F1[:, r0:r1], F2)
        C_u[:, r0:r1] = torch.einsum("bijuv,bijkv->bijku", S, A_u[:, r0:r1])
        C_v[:, r0:r1] = torch.einsum("bijuv,bijku->bijkv", S, A_v[:, r0:r1])
    return [C_u, C_v]


def compression_backward(F1, F2, A_u, A_v, gC_u, gC_v):
    """Restates MemorySaver.compression_backward (MemorySaver_cuda.cpp:80-103; kernel
    MemorySaver_kernel_compression_backward.cu:417-508).  Returns [gF1, gF2, gA_u, gA_v]."""
    B, H1, W1, C = F1.shape
    _, H2, W2, _ = F2.shape
    gF1 = torch.zeros_like(F1)
    gF2 = torch.zeros_like(F2)
    gA_u = torch.empty_like(A_u)
    gA_v = torch.empty_like(A_v)
    F2f = F2.reshape(B, H2 * W2, C)
    for r0, r1 in _row_chunks(H1, W1, H2, W2):
        S = corr_volume(F1[:, r0:r1], F2)
        gA_u[:, r0:r1] = torch.einsum("bijuv,bijku->bijkv", S, gC_u[:, r0:r1])
        gA_v[:, r0:r1] = torch.einsum("bijuv,bijkv->bijku", S, gC_v[:, r0:r1])
        G = torch.einsum("bijku,bijkv->bijuv", gC_u[:, r0:r1], A_u[:, r0:r1])
        G = G + torch.einsum("bijku,bijkv->bijuv", A_v[:, r0:r1], gC_v[:, r0:r1])
        Gf = G.reshape(B, (r1 - r0) * W1, H2 * W2)
        gF1[:, r0:r1] = torch.matmul(Gf, F2f).reshape(B, r1 - r0, W1, C)
        gF2 += torch.matmul(Gf.transpose(1, 2), F1[:, r0:r1].reshape(B, -1, C)).reshape(B, H2, W2, C)
    return [gF1, gF2, gA_u, gA_v]


def compression_attention_backward(F1, F2, gC_u, gC_v):
    """[gA_u, gA_v] of compression_backward alone (they do not depend on the attention weights)."""
    B, H1, W1, C = F1.shape
    _, H2, W2, _ = F2.shape
    Kc = gC_u.shape[3]
    gA_u = F1.new_empty(B, H1, W1, Kc, W2)
    gA_v = F1.new_empty(B, H1, W1, Kc, H2)
    for r0, r1 in _row_chunks(H1, W1, H2, W2):
        S = corr_volume(F1[:, r0:r1], F2)
        gA_u[:, r0:r1] = torch.einsum("bijuv,bijku->bijkv", S, gC_u[:, r0:r1])
        gA_v[:, r0:r1] = torch.einsum("bijuv,bijkv->bijku", S, gC_v[:, r0:r1])
    return [gA_u, gA_v]


def separation_feature_backward(F1, F2, AM_u, AM_v, gMA_u, gMA_v, A_u, A_v, gC_u, gC_v):
    """[gF1, gF2] summed over the two backward ops, i.e. what autograd accumulates for the reference's
    ComputeMaxArgmaxAvgFunction and ComputeSelfCompressionFunction
    (libs/MemorySaver/functions/MemorySaver.py:71-105, 140-177) applied to the same F1, F2."""
    a = max_argmax_avg_backward(F1, F2, AM_u, AM_v, gMA_u, gMA_v)
    b = compression_backward(F1, F2, A_u, A_v, gC_u, gC_v)
    return [a[0] + b[0], a[1] + b[1]]


def separation_backward(F1, F2, AM_u, AM_v, gMA_u, gMA_v, A_u, A_v, gC_u, gC_v):
    """[gF1, gF2, gA_u, gA_v]: both backward ops, feature gradients summed."""
    return (separation_feature_backward(F1, F2, AM_u, AM_v, gMA_u, gMA_v, A_u, A_v, gC_u, gC_v)
            + compression_attention_backward(F1, F2, gC_u, gC_v))


# Channels-first variants: the same results with every per-pixel tensor permuted the way the call site
# permutes it for its Conv3d modules, (B,H1,W1,K,D) -> (B,K,D,H1,W1) (core/corr.py:428-429, 445-446).
def _to_cf(x):
    return x.permute(0, 3, 4, 1, 2).contiguous()


def _from_cf(x):
    return x.permute(0, 3, 4, 1, 2).contiguous()


def max_argmax_avg_forward_cf(F1, F2, with_argmax=True):
    MA_u, MA_v, AM_u, AM_v = max_argmax_avg_forward(F1, F2)
    am_u = _to_cf(AM_u)[:, 0].contiguous() if with_argmax else None
    am_v = _to_cf(AM_v)[:, 0].contiguous() if with_argmax else None
    return [_to_cf(MA_u), _to_cf(MA_v), am_u, am_v]


def compression_forward_cf(F1, F2, a_u, a_v):
    C_u, C_v = compression_forward(F1, F2, _from_cf(a_u), _from_cf(a_v))
    return [_to_cf(C_u), _to_cf(C_v)]


def compression_attention_backward_cf(F1, F2, gc_u, gc_v):
    gA_u, gA_v = compression_attention_backward(F1, F2, _from_cf(gc_u), _from_cf(gc_v))
    return [_to_cf(gA_u), _to_cf(gA_v)]


def separation_feature_backward_cf(F1, F2, am_u, am_v, g_sep_v, g_sep_u, a_u, a_v, gc_u, gc_v):
    return separation_feature_backward(F1, F2, _from_cf(am_u.unsqueeze(1)), _from_cf(am_v.unsqueeze(1)),
                                       _from_cf(g_sep_v), _from_cf(g_sep_u), _from_cf(a_u), _from_cf(a_v),
                                       _from_cf(gc_u), _from_cf(gc_v))


# Attention weights of the call site and one whole pyramid level, exactly as the reference chains them
# (core/corr.py:425-457 with the Conv3d(2, Kc, 3, padding=1) modules of core/sepflow.py:59-60).
def attention_forward(x, weight, bias):
    """a = softmax over the displacement axis of Conv3d(x) (core/corr.py:437-442); x (B,2,D,H1,W1)."""
    return torch.nn.functional.conv3d(x, weight, bias, padding=1).softmax(dim=2)


def attention_backward(x, weight, a, grad_a, add=None):
    """[gx (+ add), gweight, gbias] of attention_forward, given its output ``a``: the softmax backward in
    closed form, the convolution's by autograd."""
    gl = a * (grad_a - (grad_a * a).sum(dim=2, keepdim=True))
    with torch.enable_grad():   # callers may sit inside an autograd backward, where grad mode is off
        x = x.detach().clone().requires_grad_(True)
        weight = weight.detach().clone().requires_grad_(True)
        bias = torch.zeros(weight.shape[0], dtype=weight.dtype, device=weight.device, requires_grad=True)
        torch.nn.functional.conv3d(x, weight, bias, padding=1).backward(gl)
    return [x.grad if add is None else x.grad + add, weight.grad, bias.grad]


def _from_fmaps(fmap1, fmap2, scale1):
    """core/corr.py:419-422: channels-last copies, image 1 scaled."""
    return fmap1.permute(0, 2, 3, 1).contiguous() * scale1, fmap2.permute(0, 2, 3, 1).contiguous()


def separation_level_forward(F1, F2, weight_u, bias_u, weight_v, bias_v, with_argmax=True, fmaps=False, scale1=1.0,
                             place=None):
    """[sep_u (B,2+Kc,W2,H1,W1), sep_v (B,2+Kc,H2,H1,W1), am_u, am_v, a_u, a_v] (core/corr.py:425-457); with
    ``fmaps`` from the model's (B,C,H,W) maps (core/corr.py:419-422)."""
    if fmaps:
        F1, F2 = _from_fmaps(F1, F2, scale1)
    ma_v2, ma_u2, am_u, am_v = max_argmax_avg_forward_cf(F1, F2, with_argmax)   # sep_v (per u), sep_u (per v)
    a_u = attention_forward(ma_u2, weight_u, bias_u)
    a_v = attention_forward(ma_v2, weight_v, bias_v)
    c_u, c_v = compression_forward_cf(F1, F2, a_u, a_v)
    sep_u, sep_v = torch.cat((ma_u2, c_v), dim=1), torch.cat((ma_v2, c_u), dim=1)
    if place is not None:   # channels c0.. of the concatenated outputs of all levels
        big_u, big_v, c0 = place
        big_u[:, c0:c0 + sep_u.shape[1]] = sep_u
        big_v[:, c0:c0 + sep_v.shape[1]] = sep_v
        return [None, None, am_u, am_v, a_u, a_v]
    return [sep_u, sep_v, am_u, am_v, a_u, a_v]


def separation_level_backward(F1, F2, weight_u, weight_v, sep_u, sep_v, am_u, am_v, a_u, a_v, g_sep_u, g_sep_v,
                              fmaps=False, scale1=1.0, c0=None):
    """[gF1, gF2, gweight_u, gbias_u, gweight_v, gbias_v]: the chain rule through the three ops and the two
    attention modules, with the forward's argmax and attention weights given."""
    if fmaps:
        F1, F2 = _from_fmaps(F1, F2, scale1)
    if c0 is not None:
        Kt = 2 + a_u.shape[1]
        sep_u, sep_v = sep_u[:, c0:c0 + Kt], sep_v[:, c0:c0 + Kt]
        g_sep_u, g_sep_v = g_sep_u[:, c0:c0 + Kt], g_sep_v[:, c0:c0 + Kt]
    gc_v = g_sep_u[:, 2:].contiguous()
    gc_u = g_sep_v[:, 2:].contiguous()
    ga_u, ga_v = compression_attention_backward_cf(F1, F2, gc_u, gc_v)
    gm_u, gw_u, gb_u = attention_backward(sep_u[:, :2], weight_u, a_u, ga_u, g_sep_u[:, :2])
    gm_v, gw_v, gb_v = attention_backward(sep_v[:, :2], weight_v, a_v, ga_v, g_sep_v[:, :2])
    gm_u, gm_v = gm_u.contiguous(), gm_v.contiguous()
    gF1, gF2 = separation_feature_backward_cf(F1, F2, am_u, am_v, gm_v, gm_u, a_u, a_v, gc_u, gc_v)
    if fmaps:
        gF1 = (gF1 * scale1).permute(0, 3, 1, 2).contiguous()
        gF2 = gF2.permute(0, 3, 1, 2).contiguous()
    return [gF1, gF2, gw_u, gb_u, gw_v, gb_v]


# Placement of a level's volumes into the concatenated outputs, as the reference does it (core/corr.py:459-475).
def upsample_displacement_into(src, dst, c0):
    K = src.shape[1]
    dst[:, c0:c0 + K] = torch.nn.functional.interpolate(src, list(dst.shape[2:]), mode="trilinear", align_corners=True)


def upsample_displacement_backward(grad_dst, c0, K, Dl):
    B, _, D0, H1, W1 = grad_dst.shape
    with torch.enable_grad():
        src = torch.zeros(B, K, Dl, H1, W1, dtype=grad_dst.dtype, device=grad_dst.device, requires_grad=True)
        out = torch.nn.functional.interpolate(src, [D0, H1, W1], mode="trilinear", align_corners=True)
        out.backward(grad_dst[:, c0:c0 + K])
    return src.grad


# Lookup on the aggregated 3D volumes: the reference's CorrBlock1D (core/corr.py:513-624), one volume at a time.
def lookup_pyramid(corr, levels):
    """Levels 0 .. levels-1 of the displacement pyramid of corr (B,dim,D,H1,W1): average pooling by two along the
    displacement axis (core/corr.py:543-548; the reference builds one level more than it reads)."""
    pyr = [corr]
    for _ in range(levels - 1):
        B, dim, D, H1, W1 = pyr[-1].shape
        x = pyr[-1].permute(0, 3, 4, 1, 2).reshape(B * H1 * W1, dim, 1, D)
        x = torch.nn.functional.avg_pool2d(x, [1, 2], stride=[1, 2])
        pyr.append(x.reshape(B, H1, W1, dim, D // 2).permute(0, 3, 4, 1, 2).contiguous())
    return pyr


def lookup_forward(corr, coord, levels=4, radius=4, clamp_unit=False):
    """out (B, levels*dim*(2r+1), H1, W1) for one volume corr (B,dim,D,H1,W1) and one coordinate component coord
    (B,H1,W1), with the reference's own chain of operations (core/corr.py:550-594): positions coord/2^l + dx, the
    clamp to [-1,1] the reference applies to its first volume (core/corr.py:586), grid_sample with
    align_corners=True."""
    B, dim, D, H1, W1 = corr.shape
    outs = []
    for l, vol in enumerate(lookup_pyramid(corr, levels)):
        Dl = vol.shape[2]
        img = vol.permute(0, 3, 4, 1, 2).reshape(B * H1 * W1, dim, 1, Dl)
        dx = torch.linspace(-radius, radius, 2 * radius + 1, dtype=corr.dtype, device=corr.device).view(1, 1, -1, 1)
        x0 = dx + coord.reshape(B * H1 * W1, 1, 1, 1) / 2 ** l
        y0 = torch.zeros_like(x0)
        pos = torch.cat([x0, y0], dim=-1)
        if clamp_unit:
            pos = torch.clamp(pos, -1, 1)
        xgrid, ygrid = pos.split([1, 1], dim=-1)
        xgrid = 2 * xgrid / (Dl - 1) - 1
        smp = torch.nn.functional.grid_sample(img, torch.cat([xgrid, ygrid], dim=-1), align_corners=True)
        outs.append(smp.view(B, H1, W1, -1))
    return torch.cat(outs, dim=-1).permute(0, 3, 1, 2).contiguous()


def lookup_backward(corr_shape, coord, gout, levels=4, radius=4, clamp_unit=False):
    """Gradient of the volume for upstream gradient gout (the lookup is linear in the volume)."""
    with torch.enable_grad():
        corr = torch.zeros(corr_shape, dtype=gout.dtype, device=gout.device, requires_grad=True)
        lookup_forward(corr, coord, levels, radius, clamp_unit).backward(gout)
    return corr.grad


def lookup4d_dense_forward(fmap1, fmap2, coords, levels=4, radius=4):
    """Lookup on the stored 4D correlation volume pyramid, the dense block's chain of operations: volume
    fmap1 . fmap2 / sqrt(C) (core/corr.py:286-296), pyramid by 2x2 average pooling over the image-2 axes
    (core/corr.py:32-39), per level a (2r+1)^2 window around coords / 2^l sampled with grid_sample
    (core/corr.py:200-247, core/utils/utils.py:110-118).  fmap1, fmap2 (B,C,H,W); coords (B,2,H1,W1) ->
    (B, levels*(2r+1)^2, H1, W1).  This is what the memory-saving block's unimplemented branch
    (core/corr.py:491-510) has to return."""
    B, C, H1, W1 = fmap1.shape
    H2, W2 = fmap2.shape[2:]
    corr = torch.einsum("bcij,bcuv->bijuv", fmap1, fmap2) / torch.sqrt(torch.tensor(float(C), dtype=fmap1.dtype))
    corr = corr.reshape(B * H1 * W1, 1, H2, W2)
    r = radius
    pos = coords.permute(0, 2, 3, 1)
    outs = []
    for l in range(levels):
        if l > 0:
            corr = torch.nn.functional.avg_pool2d(corr, 2, stride=2)
        d = torch.linspace(-r, r, 2 * r + 1, dtype=coords.dtype, device=coords.device)
        delta = torch.stack(torch.meshgrid(d, d, indexing="ij"), dim=-1)
        at = pos.reshape(B * H1 * W1, 1, 1, 2) / 2 ** l + delta.view(1, 2 * r + 1, 2 * r + 1, 2)
        Hl, Wl = corr.shape[-2:]
        xgrid, ygrid = at.split([1, 1], dim=-1)
        grid = torch.cat([2 * xgrid / (Wl - 1) - 1, 2 * ygrid / (Hl - 1) - 1], dim=-1)
        smp = torch.nn.functional.grid_sample(corr, grid.to(corr.dtype), align_corners=True)
        outs.append(smp.view(B, H1, W1, -1))
    return torch.cat(outs, dim=-1).permute(0, 3, 1, 2).contiguous()


def lookup4d_dense_backward(fmap1, fmap2, coords, gout, levels=4, radius=4):
    """(gfmap1, gfmap2) of lookup4d_dense_forward for upstream gradient gout, by autograd through the dense chain."""
    with torch.enable_grad():
        a = fmap1.detach().clone().requires_grad_(True)
        b = fmap2.detach().clone().requires_grad_(True)
        lookup4d_dense_forward(a, b, coords, levels, radius).backward(gout)
    return a.grad, b.grad


def lookup4d_forward(F1, F2_levels, coords, radius=4, scale=1.0):
    """The same lookup in the memory-saving formulation, with the interface of the call the reference sketches
    (core/corr.py:497-510): channels-last F1 (B,H1,W1,C) and one channels-last image-2 feature map per level
    (B,H2_l,W2_l,C), level l being the 2x2 average pooling of level l-1 (core/corr.py:377-382).  Averaging the
    volume over image-2 blocks equals correlating with the averaged features, so this returns what
    lookup4d_dense_forward returns when scale = 1/sqrt(C)."""
    B, H1, W1, C = F1.shape
    r = radius
    pos = coords.permute(0, 2, 3, 1)
    outs = []
    for l, F2 in enumerate(F2_levels):
        Hl, Wl = F2.shape[1:3]
        corr = (torch.einsum("bijc,buvc->bijuv", F1, F2) * scale).reshape(B * H1 * W1, 1, Hl, Wl)
        d = torch.linspace(-r, r, 2 * r + 1, dtype=coords.dtype, device=coords.device)
        delta = torch.stack(torch.meshgrid(d, d, indexing="ij"), dim=-1)
        at = pos.reshape(B * H1 * W1, 1, 1, 2) / 2 ** l + delta.view(1, 2 * r + 1, 2 * r + 1, 2)
        xgrid, ygrid = at.split([1, 1], dim=-1)
        grid = torch.cat([2 * xgrid / (Wl - 1) - 1, 2 * ygrid / (Hl - 1) - 1], dim=-1)
        smp = torch.nn.functional.grid_sample(corr, grid.to(corr.dtype), align_corners=True)
        outs.append(smp.view(B, H1, W1, -1))
    return torch.cat(outs, dim=-1).permute(0, 3, 1, 2).contiguous()


def lookup4d_backward(F1, F2_levels, coords, gout, radius=4, scale=1.0):
    """(gF1, [gF2_l]) of lookup4d_forward: the gradient of every level's feature map separately, as the
    device path returns them (the pooling between levels is the caller's)."""
    with torch.enable_grad():
        a = F1.detach().clone().requires_grad_(True)
        bs = [f.detach().clone().requires_grad_(True) for f in F2_levels]
        lookup4d_forward(a, bs, coords, radius, scale).backward(gout)
    return a.grad, [b.grad for b in bs]


def top2_margins(F1: torch.Tensor, F2: torch.Tensor):
    """Gap between the largest and second-largest entry of S along v (per (p,u)) and
    along u (per (p,v)), computed in float64.  An argmax is required to be bit-exact only
    where this gap exceeds the operand-rounding tolerance of the device path."""
    S = corr_volume(F1.double(), F2.double())
    def gap(dim):
        if S.shape[dim] < 2:
            return torch.full(S.max(dim=dim).values.shape, float("inf"), dtype=torch.float64, device=S.device)
        t = S.topk(2, dim=dim).values
        return t.select(dim, 0) - t.select(dim, 1)
    return gap(4), gap(3)
