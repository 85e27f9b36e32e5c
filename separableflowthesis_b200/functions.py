"""The three autograd Functions of libs/MemorySaver/functions/MemorySaver.py, same names, argument
order, outputs and error behaviour, on top of the B200 ops."""
from __future__ import annotations

import torch
from torch.autograd import Function

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
