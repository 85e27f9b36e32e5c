"""CPU: the host-side mirror of the reference call site (separableflowthesis_b200/corr.py and
functions.py) with the oracle plugged in where the CUDA ops go, against the golden vectors of the
reference's dense CorrBlock.  This tests glue (permutes, conv+softmax, concatenation, upsampling,
autograd wiring); the CUDA ops themselves are tested in the gpu-marked files."""
import os

import numpy as np
import pytest
import torch

import separableflowthesis_b200 as sfb
from separableflowthesis_b200 import functions
from oracle import separation_oracle as orc


def _t(x):
    return torch.from_numpy(np.ascontiguousarray(x))


@pytest.fixture()
def oracle_backend(monkeypatch):
    monkeypatch.setattr(functions, "MemorySaver", orc)


VARIANTS = [(True, True, True), (True, True, False), (True, False, False), (False, False, False)]


@pytest.mark.parametrize("fuse_backward,channels_first,fuse_attention", VARIANTS)
def test_block_matches_reference_dense_path(golden_dir, oracle_backend, fuse_backward, channels_first, fuse_attention):
    g = np.load(os.path.join(golden_dir, "block_dense_b2_c16_9x11_k2.npz"))
    f1 = _t(g["f1"]).requires_grad_(True)
    f2 = _t(g["f2"]).requires_grad_(True)
    convs = []
    for i in range(2):
        conv = torch.nn.Conv3d(2, g["w0"].shape[0], 3, padding=1).double()
        with torch.no_grad():
            conv.weight.copy_(_t(g[f"w{i}"]))
            conv.bias.copy_(_t(g[f"b{i}"]))
        convs.append(conv)
    blk = sfb.AlternateCorrBlockSepflow(f1, f2, None, support_backward=True, fuse_backward=fuse_backward,
                                        channels_first=channels_first, fuse_attention=fuse_attention)
    sep_u, sep_v = blk(None, sep=True, attention_weights=tuple(convs))
    assert (sep_u - _t(g["sep_u"])).abs().max().item() < 1e-11
    assert (sep_v - _t(g["sep_v"])).abs().max().item() < 1e-11
    gen = torch.Generator().manual_seed(int(g["loss_seed"]))
    wu = torch.randn(sep_u.shape, generator=gen, dtype=torch.float64)
    wv = torch.randn(sep_v.shape, generator=gen, dtype=torch.float64)
    ((sep_u * wu).sum() + (sep_v * wv).sum()).backward()
    assert (f1.grad - _t(g["g_f1"])).abs().max().item() < 1e-10
    assert (f2.grad - _t(g["g_f2"])).abs().max().item() < 1e-10
    for i, conv in enumerate(convs):
        assert (conv.weight.grad - _t(g[f"g_w{i}"])).abs().max().item() < 1e-10
        assert (conv.bias.grad - _t(g[f"g_b{i}"])).abs().max().item() < 1e-10


def test_inference_block_has_no_backward(oracle_backend):
    f1 = torch.randn(1, 8, 4, 6, dtype=torch.float64, requires_grad=True)
    f2 = torch.randn(1, 8, 4, 6, dtype=torch.float64)
    blk = sfb.AlternateCorrBlockSepflow(f1, f2, None, num_levels=2, support_backward=False)
    sep_u, sep_v = blk(None, sep=True, attention_weights=None)
    assert sep_u.shape == (1, 4, 6, 4, 6) and sep_v.shape == (1, 4, 4, 4, 6)
    with pytest.raises(NotImplementedError):
        sep_u.sum().backward()


def test_block_error_behaviour(oracle_backend):
    f = torch.randn(1, 8, 4, 6)
    with pytest.raises(Exception, match="NLF"):
        sfb.AlternateCorrBlockSepflow(f, f, guid=torch.zeros(1))


def test_block_lookup_matches_reference_dense_block(golden_dir, oracle_backend):
    """sep=False: the branch the reference leaves unimplemented (core/corr.py:491-510) returns the dense block's
    lookup (core/corr.py:192-247), and its gradients reach both feature maps through the pooling pyramid."""
    g = np.load(os.path.join(golden_dir, "lookup4d_b1_c8_12x16.npz"))
    f1 = _t(g["f1"]).requires_grad_(True)
    f2 = _t(g["f2"]).requires_grad_(True)
    blk = sfb.AlternateCorrBlockSepflow(f1, f2, None, num_levels=int(g["levels"]), radius=int(g["radius"]),
                                        support_backward=True)
    monkey_out = blk(_t(g["coords"]), sep=False)
    assert (monkey_out - _t(g["out"]).double()).abs().max().item() < 1e-6
    (monkey_out * _t(g["w"]).double()).sum().backward()
    assert (f1.grad - _t(g["g_f1"]).double()).abs().max().item() < 1e-5
    assert (f2.grad - _t(g["g_f2"]).double()).abs().max().item() < 1e-5


def test_ops_reject_cpu_and_malformed_tensors():
    F1 = torch.randn(1, 4, 4, 8)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        sfb.MemorySaver.max_avg_forward(F1, F1)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        sfb.MemorySaver.compression_forward(F1, F1, F1, F1)


def test_fused_backward_without_feature_gradients(oracle_backend):
    """Only the attention parameters need gradients: nothing is deferred and nothing is lost."""
    f1 = torch.randn(1, 8, 5, 6, dtype=torch.float64)
    f2 = torch.randn(1, 8, 5, 6, dtype=torch.float64)
    convs = [torch.nn.Conv3d(2, 2, 3, padding=1).double() for _ in range(2)]
    outs = []
    for fuse, cf, fa in VARIANTS:
        for c in convs:
            c.zero_grad()
        blk = sfb.AlternateCorrBlockSepflow(f1, f2, None, num_levels=1, support_backward=True, fuse_backward=fuse,
                                            channels_first=cf, fuse_attention=fa)
        su, sv = blk(None, sep=True, attention_weights=tuple(convs))
        (su.sum() + (sv * sv).sum()).backward()
        outs.append([c.weight.grad.clone() for c in convs])
    for other in outs[1:]:
        for a, b in zip(outs[0], other):
            assert torch.allclose(a, b, atol=1e-12)


def test_corrblock1d_host_logic(golden_dir, monkeypatch):
    """CorrBlock1D drop-in (component slicing, clamp on the first volume only, pyramid reuse, autograd) with the
    oracle in place of the CUDA ops, against the vectors of the reference's own class."""
    from separableflowthesis_b200 import corr as corr_mod

    class OracleOps:
        @staticmethod
        def lookup_build_pyramid(corr, levels):
            return None

        @staticmethod
        def lookup_forward(corr, pyramid, coord, levels, radius, clamp_unit):
            return orc.lookup_forward(corr, coord, levels, radius, clamp_unit)

        @staticmethod
        def lookup_backward(shape, coord, grad_out, levels, radius, clamp_unit):
            return orc.lookup_backward(shape, coord, grad_out, levels, radius, clamp_unit)

    monkeypatch.setattr(corr_mod, "_ops", OracleOps)
    monkeypatch.setattr(functions, "MemorySaver", OracleOps)
    g = np.load(os.path.join(golden_dir, "lookup1d_b1_dim2_16x24.npz"))
    corr1 = _t(g["corr1"]).requires_grad_(True)
    corr2 = _t(g["corr2"]).requires_grad_(True)
    blk = sfb.CorrBlock1D(corr1, corr2, num_levels=int(g["levels"]), radius=int(g["radius"]))
    out1, out2 = blk(_t(g["coords"]))
    assert (out1 - _t(g["out1"]).double()).abs().max().item() < 1e-6
    assert (out2 - _t(g["out2"]).double()).abs().max().item() < 1e-6
    ((out1 * _t(g["w1"]).double()).sum() + (out2 * _t(g["w2"]).double()).sum()).backward()
    assert (corr1.grad - _t(g["g_corr1"]).double()).abs().max().item() < 1e-6
    assert (corr2.grad - _t(g["g_corr2"]).double()).abs().max().item() < 1e-6
