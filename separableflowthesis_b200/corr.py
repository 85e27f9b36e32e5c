"""Call site of the separation ops: a drop-in for ``AlternateCorrBlockSepflow`` of the reference
(core/corr.py:335-510), producing the two separated 3D cost volumes for all pyramid levels without
ever holding the 4D correlation volume.

Differences from the reference that do not change results: the scaled channels-last copy of
``fmap1`` is made once instead of once per level (core/corr.py:419 recomputes it inside the loop); with
``fuse_backward`` (default) the feature gradients of the max/avg node and the compression node of a level,
which autograd would add, come out of one pair of gradient GEMMs instead of two; with ``channels_first``
(default, used whenever attention weights are given) the ops read and write the (B,K,D,H1,W1) tensors of the
Conv3d attention directly, which removes the permute copies of core/corr.py:428-429,445-446,451-452; with
``fuse_attention`` (default) a level whose attention modules are the Conv3d(2, Kc, 3, padding=1) of
core/sepflow.py:59-60 is one autograd node whose forward and backward are one library call each (the
Conv3d + softmax run in the library's stencil kernels, the concatenations of core/corr.py:454-457 are written
in place, and the (B,C,H,W) feature maps are read directly, which removes the channels-last and scaled copies of
core/corr.py:419-422); a level that already has the level-0 displacement range skips the trilinear resampling, which is
the identity there.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from .functions import (ComputeMaxArgmaxAvgFunction, ComputeMaxAvgFunction, ComputeSelfCompressionFunction,
                        FusedMaxArgmaxAvgFunction, FusedSelfCompressionFunction, SeparationCompressionCF,
                        Lookup4dFunction, LookupFunction, SeparationLevelFunction, SeparationMaxAvgCF, SeparationPyramidFunction,
                        SeparationState)
from . import ops as _ops


def _is_standard_attention(m) -> bool:
    """True for the module the reference builds: Conv3d(2, Kc, 3, padding=1) (core/sepflow.py:59-60)."""
    return (isinstance(m, torch.nn.Conv3d) and m.in_channels == 2 and tuple(m.kernel_size) == (3, 3, 3)
            and tuple(m.padding) == (1, 1, 1) and tuple(m.stride) == (1, 1, 1) and tuple(m.dilation) == (1, 1, 1)
            and m.groups == 1 and m.padding_mode == "zeros" and m.bias is not None and m.out_channels <= 64)


class AlternateCorrBlockSepflow:
    """Separation of the correlation volume of ``fmap1`` (B,C,H,W) against the average-pooled pyramid
    of ``fmap2``; ``guid`` must be None because non-local 4D filtering needs the stored volume
    (core/corr.py:356-358)."""

    def __init__(self, fmap1, fmap2, guid, num_levels=4, radius=4, support_backward=False, fuse_backward=True,
                 channels_first=True, fuse_attention=True):
        if guid is not None:
            raise Exception("Cannot use NLF while not storing the 4d correlation volume")
        self.max_avg_function = ComputeMaxArgmaxAvgFunction if support_backward else ComputeMaxAvgFunction
        self.support_backward = support_backward
        self.fuse_backward = fuse_backward
        self.channels_first = channels_first
        self.fuse_attention = fuse_attention
        self.num_levels = num_levels
        self.radius = radius
        self.fmap1_l0 = fmap1
        self.pyramid = [fmap2]
        for _ in range(num_levels - 1):
            fmap2 = F.avg_pool2d(fmap2, 2, stride=2)
            self.pyramid.append(fmap2)
        self._channels_last = None

    def _one_node_per_level(self, attention_weights) -> bool:
        return (self.channels_first and self.fuse_backward and self.fuse_attention and attention_weights is not None
                and all(_is_standard_attention(m) for m in attention_weights)
                and attention_weights[0].out_channels == attention_weights[1].out_channels)

    def separate_level(self, F1, level, attention_weights):
        """One pyramid level: returns (sep_u (B,K,W2,H1,W1), sep_v (B,K,H2,H1,W1)) before upsampling."""
        if self._one_node_per_level(attention_weights):
            # the library reads the (B,C,H,W) maps themselves: no channels-last copies, no scaled copy of fmap1
            attention1, attention2 = attention_weights
            return SeparationLevelFunction.apply(self.fmap1_l0.contiguous(), self.pyramid[level].contiguous(),
                                                 attention1.weight, attention1.bias, attention2.weight,
                                                 attention2.bias, self.support_backward, True,
                                                 1.0 / math.sqrt(self.fmap1_l0.shape[1]))
        F2 = self.pyramid[level].permute(0, 2, 3, 1).contiguous()
        if self.channels_first and self.fuse_backward and attention_weights is not None:
            state = SeparationState()
            sep_v, sep_u = SeparationMaxAvgCF.apply(F1, F2, state, self.support_backward)
            attention1, attention2 = attention_weights
            a_u = attention1(sep_u).softmax(dim=2)
            a_v = attention2(sep_v).softmax(dim=2)
            c_u, c_v = SeparationCompressionCF.apply(F1, F2, a_u.contiguous(), a_v.contiguous(), state)
            return torch.cat((sep_u, c_v), dim=1), torch.cat((sep_v, c_u), dim=1)
        fused = self.support_backward and self.fuse_backward and attention_weights is not None
        state = SeparationState() if fused else None
        if fused:
            maxavg_u, maxavg_v = FusedMaxArgmaxAvgFunction.apply(F1, F2, state)
        else:
            maxavg_u, maxavg_v = self.max_avg_function.apply(F1, F2)
        # naming follows the reference: sep_v holds the per-u channels, sep_u the per-v channels
        sep_v = maxavg_u.permute(0, 3, 4, 1, 2).contiguous()
        sep_u = maxavg_v.permute(0, 3, 4, 1, 2).contiguous()
        if attention_weights is not None:
            attention1, attention2 = attention_weights
            a_u = attention1(sep_u).softmax(dim=2).permute(0, 3, 4, 1, 2).contiguous()
            a_v = attention2(sep_v).softmax(dim=2).permute(0, 3, 4, 1, 2).contiguous()
            if fused:
                c_u, c_v = FusedSelfCompressionFunction.apply(F1, F2, a_u, a_v, state)
            else:
                c_u, c_v = ComputeSelfCompressionFunction.apply(F1, F2, a_u, a_v)
            sep_v = torch.cat((sep_v, c_u.permute(0, 3, 4, 1, 2)), dim=1)
            sep_u = torch.cat((sep_u, c_v.permute(0, 3, 4, 1, 2)), dim=1)
        return sep_u, sep_v

    def separate(self, attention_weights):
        """All levels, each trilinearly resampled to the level-0 displacement range and concatenated
        over channels: sep_u (B, K*levels, W, H, W), sep_v (B, K*levels, H, H, W) (core/corr.py:384-477)."""
        batch, fdim, h1, w1 = self.fmap1_l0.shape
        h2, w2 = self.pyramid[0].shape[2:]
        if self._one_node_per_level(attention_weights) and self.num_levels > 1:
            # one node for the whole pyramid: levels are resampled along the displacement axis and written into
            # their channel slices of the outputs by the library (no F.interpolate, no torch.cat)
            attention1, attention2 = attention_weights
            return SeparationPyramidFunction.apply(self.support_backward, 1.0 / math.sqrt(fdim), attention1.weight,
                                                   attention1.bias, attention2.weight, attention2.bias,
                                                   self.fmap1_l0.contiguous(), *[f.contiguous() for f in self.pyramid])
        F1 = None
        if not self._one_node_per_level(attention_weights):
            F1 = self.fmap1_l0.permute(0, 2, 3, 1).contiguous() / math.sqrt(fdim)
        sep_u_lvls, sep_v_lvls = [], []
        for level in range(self.num_levels):
            sep_u, sep_v = self.separate_level(F1, level, attention_weights)
            # align_corners resampling to the size a tensor already has copies it: skip.  The target displacement
            # ranges are those of level 0 of image 2 (the reference writes [w1, h1, w1] / [h1, h1, w1], the same
            # thing for its equally sized images; with image-1 rows sharded over ranks only image 2 has them all).
            if sep_u.shape[2] != w2:
                sep_u = F.interpolate(sep_u, [w2, h1, w1], mode="trilinear", align_corners=True)
            if sep_v.shape[2] != h2:
                sep_v = F.interpolate(sep_v, [h2, h1, w1], mode="trilinear", align_corners=True)
            sep_u_lvls.append(sep_u)
            sep_v_lvls.append(sep_v)
        if self.num_levels == 1:
            return sep_u_lvls[0], sep_v_lvls[0]
        return torch.cat(sep_u_lvls, dim=1), torch.cat(sep_v_lvls, dim=1)

    def __call__(self, coords, sep=False, attention_weights=None):
        if sep:
            return self.separate(attention_weights)
        return self.lookup(coords)

    def lookup(self, coords):
        """Lookup on the 4D correlation volume pyramid without storing it: the branch the reference leaves as
        NotImplementedError (core/corr.py:491-510).  coords (B,2,H1,W1) -> (B, levels*(2r+1)^2, H1, W1), equal to
        the dense block's lookup (core/corr.py:192-247).  The channels-last copies that the reference's sketch makes
        on every call (core/corr.py:500-501) are made once per block."""
        if self._channels_last is None:
            self._channels_last = [t.permute(0, 2, 3, 1).contiguous() for t in [self.fmap1_l0] + self.pyramid]
        F1, *F2_levels = self._channels_last
        scale = 1.0 / math.sqrt(self.fmap1_l0.shape[1])
        return Lookup4dFunction.apply(coords.to(F1.dtype).contiguous(), self.radius, scale, F1, *F2_levels)


class CorrBlock1D:
    """Lookup on the two aggregated 3D cost volumes: a drop-in for ``CorrBlock1D`` of the reference
    (core/corr.py:513-624).  corr1 (B,dim,W2,H1,W1) is read with the x component of the coordinates, corr2
    (B,dim,H2,H1,W1) with the y component; each call returns (out1, out2) of shape (B, levels*dim*(2r+1), H1, W1).

    The volumes stay in the layout they arrive in (the reference permutes and reshapes them to one row per pixel,
    core/corr.py:531-541); their displacement pyramids are built once, here.  As in the reference, the sampling
    positions of the FIRST volume are clamped to [-1, 1] before the lookup (core/corr.py:586) and those of the second
    are not; gradients flow to the volumes, not to the coordinates (the model detaches them, core/sepflow.py:192).
    """

    def __init__(self, corr1, corr2, num_levels=4, radius=4):
        assert corr1.shape[:2] == corr2.shape[:2] and corr1.shape[3:] == corr2.shape[3:]
        assert corr1.shape[2] == corr1.shape[4] and corr2.shape[2] == corr2.shape[3]  # h1 == h2 and w1 == w2
        self.num_levels = num_levels
        self.radius = radius
        self.corr1 = corr1.contiguous()
        self.corr2 = corr2.contiguous()
        with torch.no_grad():
            self.pyramid1 = _ops.lookup_build_pyramid(self.corr1, num_levels)
            self.pyramid2 = _ops.lookup_build_pyramid(self.corr2, num_levels)

    def __call__(self, coords):
        out1 = LookupFunction.apply(self.corr1, self.pyramid1, coords[:, 0], self.num_levels, self.radius, True)
        out2 = LookupFunction.apply(self.corr2, self.pyramid2, coords[:, 1], self.num_levels, self.radius, False)
        return out1, out2
