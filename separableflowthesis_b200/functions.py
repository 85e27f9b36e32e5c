"""The three autograd Functions of libs/MemorySaver/functions/MemorySaver.py, same names, argument
order, outputs and error behaviour, on top of the B200 ops."""
from __future__ import annotations

import torch
from torch.autograd import Function
from torch.autograd.function import once_differentiable

from . import ops as MemorySaver


class ComputeMaxAvgFunction(Function):
    """Max and mean channels without argmax; inference only (functions/MemorySaver.py:6-38)."""

    @staticmethod
    def forward(ctx, img1_features_l0, img2_features_lk):
        assert img1_features_l0.is_contiguous() and img2_features_lk.is_contiguous()
        with torch.cuda.device_of(img1_features_l0):
            max_avg_output_u, max_avg_output_v = MemorySaver.max_avg_forward(img1_features_l0, img2_features_lk)
        return max_avg_output_u, max_avg_output_v

    @staticmethod
    def backward(ctx, gradOutput_u, gradOutput_v):
        raise NotImplementedError("max avg backward pass is not implemented: use max argmax avg")


class ComputeMaxArgmaxAvgFunction(Function):
    """Max (+argmax kept for backward) and mean channels (functions/MemorySaver.py:40-105)."""

    @staticmethod
    def forward(ctx, img1_features_l0, img2_features_lk):
        assert img1_features_l0.is_contiguous() and img2_features_lk.is_contiguous()
        with torch.cuda.device_of(img1_features_l0):
            ma_u, ma_v, am_u, am_v = MemorySaver.max_argmax_avg_forward(img1_features_l0, img2_features_lk)
        ctx.save_for_backward(img1_features_l0, img2_features_lk, am_u, am_v)
        return ma_u, ma_v

    @staticmethod
    def backward(ctx, grad_MaxAvg_u, grad_MaxAvg_v):
        img1_features_l0, img2_features_lk, am_u, am_v = ctx.saved_tensors
        grad_MaxAvg_u = grad_MaxAvg_u.contiguous()
        grad_MaxAvg_v = grad_MaxAvg_v.contiguous()
        with torch.cuda.device_of(grad_MaxAvg_u):
            g1, g2 = MemorySaver.max_argmax_avg_backward(img1_features_l0, img2_features_lk, am_u, am_v,
                                                         grad_MaxAvg_u, grad_MaxAvg_v)
        return g1, g2


class ComputeSelfCompressionFunction(Function):
    """Attention-weighted compression channels (functions/MemorySaver.py:107-177)."""

    @staticmethod
    def forward(ctx, img1_features_l0, img2_features_lk, attention_weights_u, attention_weights_v):
        assert img1_features_l0.is_contiguous() and img2_features_lk.is_contiguous()
        assert attention_weights_u.is_contiguous() and attention_weights_v.is_contiguous()
        with torch.cuda.device_of(img1_features_l0):
            c_u, c_v = MemorySaver.compression_forward(img1_features_l0, img2_features_lk,
                                                       attention_weights_u, attention_weights_v)
        ctx.save_for_backward(img1_features_l0, img2_features_lk, attention_weights_u, attention_weights_v)
        return c_u, c_v

    @staticmethod
    def backward(ctx, grad_compressed_output_u, grad_compressed_output_v):
        f1, f2, a_u, a_v = ctx.saved_tensors
        grad_compressed_output_u = grad_compressed_output_u.contiguous()
        grad_compressed_output_v = grad_compressed_output_v.contiguous()
        with torch.cuda.device_of(grad_compressed_output_u):
            g1, g2, ga_u, ga_v = MemorySaver.compression_backward(f1, f2, a_u, a_v, grad_compressed_output_u,
                                                                  grad_compressed_output_v)
        return g1, g2, ga_u, ga_v


# --------------------------------------------------------------------------------------------------
# Fused backward for the call site.  Not part of the reference's surface.
#
# When the max/avg node and the compression node act on the same (F1, F2) -- which is how
# AlternateCorrBlockSepflow.separate uses them (core/corr.py:425,448) -- their two feature gradients are
# summed by autograd.  The pair of Functions below produces that sum with ONE pair of gradient GEMMs:
# the compression node's backward returns only the attention gradients (they are needed at once, the
# Conv3d/softmax backward sits between the two nodes) and parks its inputs in a shared state object; the
# max/avg node's backward, which autograd always runs later because its outputs feed the attention
# weights, then computes the summed feature gradients.
class SeparationState:
    """Shared between the two fused Functions of one pyramid level."""

    def __init__(self):
        self.pending = None          # (A_u, A_v, gC_u, gC_v) parked by the compression node's backward
        self.collected = True


def _guard_pending(state):
    # runs when the backward pass that parked the tensors ends: they must have been consumed by then
    def check():
        if state.pending is not None:
            state.pending = None
            raise RuntimeError(
                "fused separation backward: the compression node deferred its feature gradients but the "
                "max/avg node's backward never ran (its outputs do not reach the loss); use "
                "AlternateCorrBlockSepflow(..., fuse_backward=False)")
    return check


class FusedMaxArgmaxAvgFunction(Function):
    @staticmethod
    def forward(ctx, img1_features_l0, img2_features_lk, state):
        assert img1_features_l0.is_contiguous() and img2_features_lk.is_contiguous()
        with torch.cuda.device_of(img1_features_l0):
            ma_u, ma_v, am_u, am_v = MemorySaver.max_argmax_avg_forward(img1_features_l0, img2_features_lk)
        ctx.save_for_backward(img1_features_l0, img2_features_lk, am_u, am_v)
        ctx.state = state
        return ma_u, ma_v

    @staticmethod
    def backward(ctx, grad_MaxAvg_u, grad_MaxAvg_v):
        f1, f2, am_u, am_v = ctx.saved_tensors
        grad_MaxAvg_u = grad_MaxAvg_u.contiguous()
        grad_MaxAvg_v = grad_MaxAvg_v.contiguous()
        pending, ctx.state.pending = ctx.state.pending, None
        with torch.cuda.device_of(grad_MaxAvg_u):
            if pending is None:
                g1, g2 = MemorySaver.max_argmax_avg_backward(f1, f2, am_u, am_v, grad_MaxAvg_u, grad_MaxAvg_v)
            else:
                a_u, a_v, gc_u, gc_v = pending
                g1, g2 = MemorySaver.separation_feature_backward(f1, f2, am_u, am_v, grad_MaxAvg_u, grad_MaxAvg_v,
                                                                 a_u, a_v, gc_u, gc_v)
        return g1, g2, None


class FusedSelfCompressionFunction(Function):
    @staticmethod
    def forward(ctx, img1_features_l0, img2_features_lk, attention_weights_u, attention_weights_v, state):
        assert img1_features_l0.is_contiguous() and img2_features_lk.is_contiguous()
        assert attention_weights_u.is_contiguous() and attention_weights_v.is_contiguous()
        with torch.cuda.device_of(img1_features_l0):
            c_u, c_v = MemorySaver.compression_forward(img1_features_l0, img2_features_lk,
                                                       attention_weights_u, attention_weights_v)
        ctx.save_for_backward(img1_features_l0, img2_features_lk, attention_weights_u, attention_weights_v)
        ctx.state = state
        return c_u, c_v

    @staticmethod
    def backward(ctx, grad_compressed_output_u, grad_compressed_output_v):
        f1, f2, a_u, a_v = ctx.saved_tensors
        gc_u = grad_compressed_output_u.contiguous()
        gc_v = grad_compressed_output_v.contiguous()
        with torch.cuda.device_of(gc_u):
            if not (ctx.needs_input_grad[0] or ctx.needs_input_grad[1]):
                ga_u, ga_v = MemorySaver.compression_attention_backward(f1, f2, gc_u, gc_v)
                return None, None, ga_u, ga_v, None
            if not (ctx.needs_input_grad[2] or ctx.needs_input_grad[3]):
                # the attention weights do not depend on the max/avg node: nothing guarantees that node's
                # backward runs after this one, so do not defer
                g1, g2, ga_u, ga_v = MemorySaver.compression_backward(f1, f2, a_u, a_v, gc_u, gc_v)
                return g1, g2, ga_u, ga_v, None
            ga_u, ga_v = MemorySaver.compression_attention_backward(f1, f2, gc_u, gc_v)
            ctx.state.pending = (a_u, a_v, gc_u, gc_v)
            torch.autograd.Variable._execution_engine.queue_callback(_guard_pending(ctx.state))
        return None, None, ga_u, ga_v, None


# --------------------------------------------------------------------------------------------------
# Channels-first pair for the call site: same fused backward, and every per-pixel tensor already has the
# (B, K, D, H1, W1) layout of the Conv3d attention modules, so the call site's permute copies disappear.
class SeparationMaxAvgCF(Function):
    @staticmethod
    def forward(ctx, img1_features_l0, img2_features_lk, state, with_argmax):
        assert img1_features_l0.is_contiguous() and img2_features_lk.is_contiguous()
        with torch.cuda.device_of(img1_features_l0):
            sep_v, sep_u, am_u, am_v = MemorySaver.max_argmax_avg_forward_cf(img1_features_l0, img2_features_lk,
                                                                             with_argmax)
        if with_argmax:
            ctx.save_for_backward(img1_features_l0, img2_features_lk, am_u, am_v)
        ctx.state = state
        ctx.with_argmax = with_argmax
        return sep_v, sep_u

    @staticmethod
    def backward(ctx, grad_sep_v, grad_sep_u):
        if not ctx.with_argmax:
            raise NotImplementedError("max avg backward pass is not implemented: use max argmax avg")
        f1, f2, am_u, am_v = ctx.saved_tensors
        pending, ctx.state.pending = ctx.state.pending, None
        if pending is None:
            raise RuntimeError("channels-first separation backward needs the compression node's backward first "
                               "(use AlternateCorrBlockSepflow(..., channels_first=False) for max/avg alone)")
        a_u, a_v, gc_u, gc_v = pending
        with torch.cuda.device_of(grad_sep_v):
            g1, g2 = MemorySaver.separation_feature_backward_cf(f1, f2, am_u, am_v, grad_sep_v.contiguous(),
                                                                grad_sep_u.contiguous(), a_u, a_v, gc_u, gc_v)
        return g1, g2, None, None


class SeparationCompressionCF(Function):
    @staticmethod
    def forward(ctx, img1_features_l0, img2_features_lk, a_u, a_v, state):
        assert img1_features_l0.is_contiguous() and img2_features_lk.is_contiguous()
        assert a_u.is_contiguous() and a_v.is_contiguous()
        with torch.cuda.device_of(img1_features_l0):
            c_u, c_v = MemorySaver.compression_forward_cf(img1_features_l0, img2_features_lk, a_u, a_v)
        ctx.save_for_backward(img1_features_l0, img2_features_lk, a_u, a_v)
        ctx.state = state
        return c_u, c_v

    @staticmethod
    def backward(ctx, grad_c_u, grad_c_v):
        f1, f2, a_u, a_v = ctx.saved_tensors
        gc_u, gc_v = grad_c_u.contiguous(), grad_c_v.contiguous()
        with torch.cuda.device_of(gc_u):
            ga_u, ga_v = MemorySaver.compression_attention_backward_cf(f1, f2, gc_u, gc_v)
        if ctx.needs_input_grad[0] or ctx.needs_input_grad[1]:
            ctx.state.pending = (a_u, a_v, gc_u, gc_v)
            torch.autograd.Variable._execution_engine.queue_callback(_guard_pending(ctx.state))
        return None, None, ga_u, ga_v, None


# --------------------------------------------------------------------------------------------------
# One pyramid level as a single autograd node: max/avg sweep, both attention modules (Conv3d(2, Kc, 3,
# padding=1) + softmax over the displacement axis, core/corr.py:437-442) and the compression sweep, writing
# the concatenated tensors of core/corr.py:454-457 directly.  The backward is one call as well.
class SeparationLevelFunction(Function):
    @staticmethod
    def forward(ctx, img1_features_l0, img2_features_lk, weight_u, bias_u, weight_v, bias_v, with_argmax,
                fmaps=False, scale1=1.0):
        """With ``fmaps`` the features are the model's maps (B,C,H,W) and ``scale1`` multiplies image 1's."""
        assert img1_features_l0.is_contiguous() and img2_features_lk.is_contiguous()
        ctx.fmaps, ctx.scale1 = fmaps, scale1
        with torch.cuda.device_of(img1_features_l0):
            sep_u, sep_v, am_u, am_v, a_u, a_v = MemorySaver.separation_level_forward(
                img1_features_l0, img2_features_lk, weight_u.contiguous(), bias_u.contiguous(),
                weight_v.contiguous(), bias_v.contiguous(), with_argmax, fmaps, scale1)
        if with_argmax:
            ctx.save_for_backward(img1_features_l0, img2_features_lk, weight_u, weight_v, sep_u, sep_v, am_u, am_v,
                                  a_u, a_v)
        ctx.with_argmax = with_argmax
        return sep_u, sep_v

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_sep_u, grad_sep_v):
        if not ctx.with_argmax:
            raise NotImplementedError("max avg backward pass is not implemented: use max argmax avg")
        f1, f2, weight_u, weight_v, sep_u, sep_v, am_u, am_v, a_u, a_v = ctx.saved_tensors
        with torch.cuda.device_of(grad_sep_u):
            g1, g2, gw_u, gb_u, gw_v, gb_v = MemorySaver.separation_level_backward(
                f1, f2, weight_u.contiguous(), weight_v.contiguous(), sep_u, sep_v, am_u, am_v, a_u, a_v,
                grad_sep_u.contiguous(), grad_sep_v.contiguous(), ctx.fmaps, ctx.scale1)
        return g1, g2, gw_u, gb_u, gw_v, gb_v, None, None, None


# --------------------------------------------------------------------------------------------------
# All pyramid levels as one autograd node (core/corr.py:416-475): per level the one-call forward from the feature
# maps, then its volumes are resampled along the displacement axis and written straight into their channel slice of
# the concatenated outputs (the reference runs F.interpolate per level and torch.cat over levels).
class SeparationPyramidFunction(Function):
    @staticmethod
    def forward(ctx, with_argmax, scale1, weight_u, bias_u, weight_v, bias_v, fmap1, *fmap2_levels):
        assert fmap1.is_contiguous() and all(f.is_contiguous() for f in fmap2_levels)
        params = [t.contiguous() for t in (weight_u, bias_u, weight_v, bias_v)]
        B, _, H1, W1 = fmap1.shape
        H2, W2 = fmap2_levels[0].shape[2:]     # displacement ranges of the outputs (= H1, W1 unless image-1 rows are sharded)
        L, Kt = len(fmap2_levels), 2 + weight_u.shape[0]
        saved = []
        with torch.cuda.device_of(fmap1):
            sep_u = torch.empty(B, Kt * L, W2, H1, W1, dtype=fmap1.dtype, device=fmap1.device)
            sep_v = torch.empty(B, Kt * L, H2, H1, W1, dtype=fmap1.dtype, device=fmap1.device)
            for l, fmap2 in enumerate(fmap2_levels):
                if tuple(fmap2.shape[2:]) == (H2, W2):   # displacement range of the output: written in place
                    su, sv, am_u, am_v, a_u, a_v = MemorySaver.separation_level_forward(
                        fmap1, fmap2, *params, with_argmax, True, scale1, (sep_u, sep_v, l * Kt))
                else:
                    su, sv, am_u, am_v, a_u, a_v = MemorySaver.separation_level_forward(fmap1, fmap2, *params,
                                                                                        with_argmax, True, scale1)
                    MemorySaver.upsample_displacement_into(su, sep_u, l * Kt)
                    MemorySaver.upsample_displacement_into(sv, sep_v, l * Kt)
                saved.append((su, sv, am_u, am_v, a_u, a_v))
        ctx.with_argmax, ctx.scale1, ctx.levels = with_argmax, scale1, L
        if with_argmax:
            # volumes written in place are saved as the outputs themselves
            ctx.in_place = [t[0] is None for t in saved]
            flat = [x for t in saved for x in t if x is not None]
            ctx.save_for_backward(fmap1, weight_u, weight_v, sep_u, sep_v, *fmap2_levels, *flat)
        return sep_u, sep_v

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_sep_u, grad_sep_v):
        if not ctx.with_argmax:
            raise NotImplementedError("max avg backward pass is not implemented: use max argmax avg")
        L = ctx.levels
        fmap1, weight_u, weight_v, sep_u, sep_v = ctx.saved_tensors[:5]
        fmap2_levels = ctx.saved_tensors[5:5 + L]
        flat = list(ctx.saved_tensors[5 + L:])
        wu, wv = weight_u.contiguous(), weight_v.contiguous()
        gu, gv = grad_sep_u.contiguous(), grad_sep_v.contiguous()
        Kt = 2 + weight_u.shape[0]
        g1 = gw_u = gb_u = gw_v = gb_v = None
        g2 = []
        with torch.cuda.device_of(gu):
            for l in range(L):
                if ctx.in_place[l]:
                    am_u, am_v, a_u, a_v = flat[:4]
                    del flat[:4]
                    out = MemorySaver.separation_level_backward(fmap1, fmap2_levels[l], wu, wv, sep_u, sep_v, am_u, am_v,
                                                                a_u, a_v, gu, gv, True, ctx.scale1, l * Kt)
                else:
                    su, sv, am_u, am_v, a_u, a_v = flat[:6]
                    del flat[:6]
                    gsu = MemorySaver.upsample_displacement_backward(gu, l * Kt, Kt, su.shape[2])
                    gsv = MemorySaver.upsample_displacement_backward(gv, l * Kt, Kt, sv.shape[2])
                    out = MemorySaver.separation_level_backward(fmap1, fmap2_levels[l], wu, wv, su, sv, am_u, am_v, a_u,
                                                                a_v, gsu, gsv, True, ctx.scale1)
                g2.append(out[1])
                if l == 0:
                    g1, gw_u, gb_u, gw_v, gb_v = out[0], out[2], out[3], out[4], out[5]
                else:
                    g1 += out[0]; gw_u += out[2]; gb_u += out[3]; gw_v += out[4]; gb_v += out[5]
        return (None, None, gw_u, gb_u, gw_v, gb_v, g1, *g2)


# --------------------------------------------------------------------------------------------------
# Lookup on one aggregated 3D volume (CorrBlock1D, core/corr.py:576-594).  The volume's pyramid is passed in so that
# it is built once per volume, not once per refinement iteration.  No gradient for the coordinates: the model
# detaches them before every lookup (core/sepflow.py:192).
class LookupFunction(Function):
    @staticmethod
    def forward(ctx, corr, pyramid, coord, levels, radius, clamp_unit):
        with torch.cuda.device_of(corr):
            out = MemorySaver.lookup_forward(corr, pyramid, coord, levels, radius, clamp_unit)
        ctx.save_for_backward(coord)
        ctx.cfg = (tuple(corr.shape), levels, radius, clamp_unit)
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_out):
        (coord,) = ctx.saved_tensors
        shape, levels, radius, clamp_unit = ctx.cfg
        with torch.cuda.device_of(grad_out):
            gcorr = MemorySaver.lookup_backward(shape, coord, grad_out.contiguous(), levels, radius, clamp_unit)
        return gcorr, None, None, None, None, None


class Lookup4dFunction(Function):
    """Lookup on the 4D correlation volume without storing it.  ``apply(coords, radius, scale, F1, *F2_levels)`` with
    channels-last features -> (B, levels*(2r+1)^2, H1, W1); gradients for the features only (the model detaches
    the coordinates, core/sepflow.py:193)."""

    @staticmethod
    def forward(ctx, coords, radius, scale, F1, *F2_levels):
        with torch.cuda.device_of(F1):
            out = MemorySaver.lookup4d_forward(F1, list(F2_levels), coords, radius, scale)
        ctx.save_for_backward(coords, F1, *F2_levels)
        ctx.cfg = (radius, scale)
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_out):
        coords, F1, *F2_levels = ctx.saved_tensors
        radius, scale = ctx.cfg
        with torch.cuda.device_of(grad_out):
            gF1, gF2 = MemorySaver.lookup4d_backward(F1, F2_levels, coords, grad_out.contiguous(), radius, scale)
        return (None, None, None, gF1, *gF2)
