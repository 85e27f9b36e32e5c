"""CPU: the C-ABI library loads without a GPU, exports every symbol include/sepflow_b200.h
declares, and rejects bad arguments before touching CUDA."""
import ctypes
import os
import re

import pytest

from separableflowthesis_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build_library()
    return _lib.load()


def test_exports_every_declared_symbol(lib):
    header = open(os.path.join(ROOT, "include", "sepflow_b200.h")).read()
    declared = set(re.findall(r"\b(sfb_[a-z_0-9]+)\s*\(", header))
    assert declared == set(_lib.EXPORTED_SYMBOLS)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.sfb_version() >= 100


def test_workspace_query(lib):
    s = _lib.SfbShape(2, 48, 64, 48, 64, 256, 2)
    fwd = lib.sfb_workspace_bytes(_lib.OP_MAX_AVG_FORWARD, ctypes.byref(s))
    bwd = lib.sfb_workspace_bytes(_lib.OP_COMPRESSION_BACKWARD, ctypes.byref(s))
    feat = 2 * 48 * 64 * 256 * 4                      # one rounded feature copy
    packed = 2 * 48 * 64 * (48 + 64) * 4              # one packed slot of every (pixel, displacement) pair
    assert fwd >= 2 * feat + 2 * (48 + 64) * 256 * 4 + 3 * packed   # + mean rows of F2 + max/mean/argmax slots
    assert bwd >= 2 * feat + (4 + 2) * packed                      # + 2*Kc input slots + Kc output slots
    bad = _lib.SfbShape(2, 48, 64, 48, 64, 258, 2)
    assert lib.sfb_workspace_bytes(_lib.OP_MAX_AVG_FORWARD, ctypes.byref(bad)) == 0
    assert lib.sfb_workspace_bytes(99, ctypes.byref(s)) == 0


def test_argument_validation(lib):
    s = _lib.SfbShape(1, 4, 4, 4, 4, 32, 2)
    P = ctypes.c_void_p
    buf = (ctypes.c_char * 4096)()
    a16 = (ctypes.addressof(buf) + 255) // 256 * 256
    rc = lib.sfb_max_avg_forward(None, P(a16), P(a16), P(a16), ctypes.byref(s), P(a16), 1 << 20, None)
    assert rc == _lib.SFB_ERR_INVALID_ARGUMENT and b"F1 is NULL" in lib.sfb_last_error()
    rc = lib.sfb_max_avg_forward(P(a16 + 4), P(a16), P(a16), P(a16), ctypes.byref(s), P(a16), 1 << 20, None)
    assert rc == _lib.SFB_ERR_INVALID_ARGUMENT and b"aligned" in lib.sfb_last_error()
    rc = lib.sfb_max_avg_forward(P(a16), P(a16), P(a16), P(a16), ctypes.byref(s), P(a16), 16, None)
    assert rc == _lib.SFB_ERR_WORKSPACE_TOO_SMALL
    bad_c = _lib.SfbShape(1, 4, 4, 4, 4, 300, 2)
    rc = lib.sfb_compression_forward(P(a16), P(a16), P(a16), P(a16), P(a16), P(a16), ctypes.byref(bad_c), P(a16),
                                     1 << 20, None)
    assert rc == _lib.SFB_ERR_UNSUPPORTED_SHAPE
    no_k = _lib.SfbShape(1, 4, 4, 4, 4, 32, 0)
    rc = lib.sfb_compression_forward(P(a16), P(a16), P(a16), P(a16), P(a16), P(a16), ctypes.byref(no_k), P(a16),
                                     1 << 20, None)
    assert rc == _lib.SFB_ERR_INVALID_ARGUMENT
    assert lib.sfb_status_string(_lib.SFB_ERR_DEVICE_TIMEOUT) == b"device-side wait timed out"


def test_argument_validation_of_the_call_site_entry_points(lib):
    """Attention, lookup, resampling and placed level calls reject bad sizes before any CUDA work."""
    P = ctypes.c_void_p
    buf = (ctypes.c_char * 4096)()
    a16 = (ctypes.addressof(buf) + 255) // 256 * 256
    p = P(a16)
    assert lib.sfb_attention_forward(p, 0, p, p, p, 1, 0, 4, 4, 4, None) == _lib.SFB_ERR_INVALID_ARGUMENT
    assert lib.sfb_attention_forward(p, 0, p, p, p, 1, 65, 4, 4, 4, None) == _lib.SFB_ERR_UNSUPPORTED_SHAPE
    assert lib.sfb_attention_forward(None, 0, p, p, p, 1, 2, 4, 4, 4, None) == _lib.SFB_ERR_INVALID_ARGUMENT
    assert lib.sfb_attention_backward_workspace_bytes(1, 2, 4, 4, 4) > 0
    assert lib.sfb_attention_backward(p, 0, p, p, p, None, 0, p, p, p, 1, 2, 4, 4, 4, p, 16, None) \
        == _lib.SFB_ERR_WORKSPACE_TOO_SMALL
    assert lib.sfb_lookup_pyramid_bytes(2, 1, 16, 3, 5, 4) == 4 * 2 * (8 + 4 + 2) * 15
    assert lib.sfb_lookup_pyramid_bytes(2, 1, 16, 3, 5, 5) == 0          # coarsest level would have one entry
    assert lib.sfb_lookup_forward(p, p, p, 15, p, 2, 1, 1, 3, 5, 1, 4, 0, None) == _lib.SFB_ERR_INVALID_ARGUMENT
    assert lib.sfb_lookup_forward(p, p, p, 15, p, 2, 1, 16, 3, 5, 9, 4, 0, None) == _lib.SFB_ERR_UNSUPPORTED_SHAPE
    levels = (P * 2)(a16, a16)
    H2, W2 = (ctypes.c_int32 * 2)(8, 4), (ctypes.c_int32 * 2)(8, 4)
    f = ctypes.c_float(1.0)
    assert lib.sfb_lookup4d_forward(p, levels, H2, W2, 2, p, p, 1, 8, 8, 30, 4, f, None) == _lib.SFB_ERR_INVALID_ARGUMENT
    assert b"C % 4" in lib.sfb_last_error()
    assert lib.sfb_lookup4d_forward(p, levels, H2, W2, 2, p, p, 1, 8, 8, 32, 5, f, None) == _lib.SFB_ERR_INVALID_ARGUMENT
    assert lib.sfb_lookup4d_forward(p, levels, H2, W2, 9, p, p, 1, 8, 8, 32, 4, f, None) == _lib.SFB_ERR_INVALID_ARGUMENT
    one = (ctypes.c_int32 * 2)(8, 1)
    assert lib.sfb_lookup4d_forward(p, levels, H2, one, 2, p, p, 1, 8, 8, 32, 4, f, None) == _lib.SFB_ERR_INVALID_ARGUMENT
    assert b"H2 >= 2" in lib.sfb_last_error()
    holes = (P * 2)(a16, None)
    assert lib.sfb_lookup4d_backward(p, levels, H2, W2, 2, p, p, p, holes, 1, 8, 8, 32, 4, f, None) \
        == _lib.SFB_ERR_INVALID_ARGUMENT
    assert lib.sfb_upsample_displacement(p, p, 100, 1, 2, 8, 4, 3, 5, None) == _lib.SFB_ERR_UNSUPPORTED_SHAPE
    assert b"upsampling" in lib.sfb_last_error()
    assert lib.sfb_upsample_displacement(p, None, 100, 1, 2, 4, 8, 3, 5, None) == _lib.SFB_ERR_INVALID_ARGUMENT
    s = _lib.SfbShape(1, 4, 4, 4, 4, 32, 2)
    rc = lib.sfb_separation_level_forward_fmaps(p, p, ctypes.c_float(1.0), p, p, p, p, p, p, 5, 3, None, None, p, p,
                                                ctypes.byref(s), p, 1 << 30, None)
    assert rc == _lib.SFB_ERR_INVALID_ARGUMENT and b"do not fit" in lib.sfb_last_error()


def test_max_avg_ops_ignore_an_uninitialised_kc():
    """The max/avg entry points do not read Kc (the header says so): a garbage value must neither be rejected nor
    overflow the size checks."""
    lib = _lib.load()
    for kc in (0x7fffffff, -5, 0):
        s = _lib.SfbShape(1, 48, 64, 48, 64, 256, kc)
        assert lib.sfb_workspace_bytes(_lib.OP_MAX_AVG_FORWARD, ctypes.byref(s)) > 0
        assert lib.sfb_workspace_bytes(_lib.OP_MAX_ARGMAX_AVG_BACKWARD, ctypes.byref(s)) > 0
    # ops that do use Kc still check it
    s = _lib.SfbShape(1, 48, 64, 48, 64, 256, 0)
    assert lib.sfb_workspace_bytes(_lib.OP_COMPRESSION_FORWARD, ctypes.byref(s)) == 0


def test_operand_switch(lib):
    """sfb_set_sweep_operands: FP16 (2) is the default, TF32 (0) and BF16 (1) can be chosen, anything else is refused
    with -1 and leaves the setting alone; the call returns the previous value."""
    if "SFB_OPERANDS" not in os.environ:
        assert lib.sfb_get_sweep_operands() == 2
    lib.sfb_set_sweep_operands(2)
    assert lib.sfb_set_sweep_operands(0) == 2 and lib.sfb_get_sweep_operands() == 0
    assert lib.sfb_set_sweep_operands(7) == -1 and lib.sfb_get_sweep_operands() == 0
    assert lib.sfb_set_sweep_operands(1) == 0
    assert lib.sfb_set_sweep_operands(2) == 1 and lib.sfb_get_sweep_operands() == 2


def test_missing_library_fails_loudly(tmp_path):
    """No CPU or PyTorch fallback: with the shared library out of reach, loading raises and says how to build it."""
    import subprocess
    import sys
    code = (
        "import separableflowthesis_b200._lib as L\n"
        f"L.LIB_PATH = {str(tmp_path / 'absent' / 'libsepflow_b200.so')!r}\n"
        "L._lib = None\n"
        "try:\n"
        "    L.load()\n"
        "except RuntimeError as e:\n"
        "    assert 'is missing' in str(e) and 'no CPU or PyTorch fallback' in str(e), str(e)\n"
        "    print('raised')\n"
    )
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-c", code], cwd=root, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    assert out.stdout.strip().endswith("raised")
