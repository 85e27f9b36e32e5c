"""GPU: the CUDA ops against the reference's OWN CUDA extension (libs/MemorySaver/src, built unmodified by
oracle/build_ref_cuda.py into oracle/_ref/MemorySaver.so) as a second oracle, at the sizes the reference's kernels
are written for (Kc = 2: MemorySaver_kernel_forward.cu:20 compiles the channel count in).  Skipped when that file
has not been built.  The reference accumulates gF2 with atomicAdd, so comparisons are to tolerance, not bits."""
import importlib.util
import os

import pytest
import torch

from separableflowthesis_b200 import ops
from oracle import separation_oracle as orc

pytestmark = pytest.mark.gpu

REF_SO = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "MemorySaver.so")
TOL = 1e-3
MARGIN = 5e-3


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF_SO):
        pytest.skip("oracle/_ref/MemorySaver.so not built (python oracle/build_ref_cuda.py <reference checkout>)")
    spec = importlib.util.spec_from_file_location("MemorySaver", REF_SO)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def relerr(x, ref):
    x, ref = x.double(), ref.double()
    return ((x - ref).abs().max() / max(x.abs().max().item(), ref.abs().max().item(), 1e-30)).item()


# (B, H1, W1, H2, W2, C): BASELINE config 2, an odd size, a pooled image 2
@pytest.mark.parametrize("shape", [(2, 48, 64, 48, 64, 256), (1, 17, 23, 17, 23, 64), (1, 16, 24, 8, 12, 32)])
def test_ops_match_the_reference_cuda_extension(ref, shape, cuda_device):
    B, H1, W1, H2, W2, C = shape
    Kc = 2
    dev = cuda_device
    g = torch.Generator().manual_seed(1234)
    F1 = (torch.randn(B, H1, W1, C, generator=g) / C ** 0.5).to(dev)
    F2 = torch.randn(B, H2, W2, C, generator=g).to(dev)
    A_u = torch.randn(B, H1, W1, Kc, W2, generator=g).softmax(-1).to(dev)
    A_v = torch.randn(B, H1, W1, Kc, H2, generator=g).softmax(-1).to(dev)
    gMA_u = torch.randn(B, H1, W1, 2, H2, generator=g).to(dev)
    gMA_v = torch.randn(B, H1, W1, 2, W2, generator=g).to(dev)
    gC_u = torch.randn(B, H1, W1, Kc, H2, generator=g).to(dev)
    gC_v = torch.randn(B, H1, W1, Kc, W2, generator=g).to(dev)

    r_mu, r_mv, r_au, r_av = ref.max_argmax_avg_forward(F1, F2)
    mu, mv, au, av = ops.max_argmax_avg_forward(F1, F2)
    assert relerr(mu, r_mu) < TOL and relerr(mv, r_mv) < TOL
    gap_u, gap_v = orc.top2_margins(F1.cpu(), F2.cpu())
    sure_u, sure_v = (gap_u > MARGIN).to(dev), (gap_v > MARGIN).to(dev)
    assert torch.equal(au[:, :, :, 0][sure_u], r_au[:, :, :, 0][sure_u])
    assert torch.equal(av[:, :, :, 0][sure_v], r_av[:, :, :, 0][sure_v])

    r_g1, r_g2 = ref.max_argmax_avg_backward(F1, F2, r_au, r_av, gMA_u, gMA_v)
    g1, g2 = ops.max_argmax_avg_backward(F1, F2, r_au, r_av, gMA_u, gMA_v)
    assert relerr(g1, r_g1) < TOL and relerr(g2, r_g2) < TOL

    r_cu, r_cv = ref.compression_forward(F1, F2, A_u, A_v)
    cu, cv = ops.compression_forward(F1, F2, A_u, A_v)
    assert relerr(cu, r_cu) < TOL and relerr(cv, r_cv) < TOL

    r = ref.compression_backward(F1, F2, A_u, A_v, gC_u, gC_v)
    o = ops.compression_backward(F1, F2, A_u, A_v, gC_u, gC_v)
    for a, b in zip(o, r):
        assert relerr(a, b) < TOL
    torch.cuda.synchronize()
