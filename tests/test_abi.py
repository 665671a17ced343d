"""The C-ABI library without a GPU: it loads, exports every declared symbol, and validates arguments."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def tk():
    import tacker_b200
    from tacker_b200 import _build

    _build.build_library()
    return tacker_b200


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "tacker_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tk_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(tk):
    lib = tk.lib()
    names = _declared_symbols()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/tacker_b200.h but not exported"


def test_registry_mirrors_fmap_keys(tk):
    lib = tk.lib()
    keys = [lib.tk_key(i).decode() for i in range(lib.tk_num_keys())]
    assert set(keys) == set(tk.KEYS)
    for k in keys:
        assert lib.tk_lookup(k.encode())
    assert not lib.tk_lookup(b"gptb_hot3d")        # outside the hot path: not registered
    assert lib.tk_key(99) is None
    from tacker_b200 import ops

    with pytest.raises(KeyError, match="load kernel"):
        ops.lookup("cp_sgemm")


def test_status_strings_and_options(tk):
    lib = tk.lib()
    assert lib.tk_status_string(0) == b"ok"
    for s in range(-8, 0):
        assert lib.tk_status_string(s) != b"unknown status"
    from tacker_b200 import ops

    assert ops.get_option("cp_ppt") == 8
    ops.set_option("cp_ppt", 4)
    assert ops.get_option("cp_ppt") == 4
    ops.set_option("cp_ppt", 8)
    assert lib.tk_set_option(b"cp_ppt", 3) == -1
    assert lib.tk_set_option(b"tzgemm_bn", 64) == -1
    assert lib.tk_set_option(b"nope", 1) == -4


def test_argument_validation_needs_no_gpu(tk):
    from tacker_b200 import ops

    ints = [C.c_int(1)] * 20
    assert ops.raw_launch("gptb_tzgemm", ints[:5], (1, 1, 1), (192, 1, 1)) == -1      # wrong count
    assert ops.raw_launch("tzgemm_stencil", ints[:31], (1, 1, 1), (448, 1, 1)) == -1
    p = [C.c_void_p(256), C.c_void_p(256), C.c_void_p(256), C.c_int(128), C.c_int(100), C.c_int(128),
         C.c_float(1.0)] + [C.c_int(1)] * 6 + [C.c_int(0), C.c_int(1), C.c_int(4), C.c_int(0)]
    assert ops.raw_launch("gptb_tzgemm", p, (1, 1, 1), (192, 1, 1)) == -3             # N not a multiple of 64
    assert ops.raw_launch("gptb_tzgemm", p, (0, 1, 1), (192, 1, 1)) == -6


def test_shape_helpers(tk):
    from tacker_b200 import ops

    assert ops.tzgemm_dims(1024, 1024, 1024) == (1024, 1024, 1024, 256)
    assert ops.tzgemm_dims(1, 1000, 4096) == (128, 896, 4096, 28)
    assert ops.conv_mnk([1, 3, 224, 224, 64, 3, 3, 3, 1, 1, 1, 1, 1, 1]) == (50176, 64, 27)


def test_python_mirror_marshals_like_the_reference(tk):
    """GPTB = solo params + 6 geometry ints (+4 at launch); Mix = k1 + 3 ++ k2 + 3 (src/MixKernel.h:55-73)."""
    from tacker_b200 import ops

    tz = ops.GPTBKernel("tzgemm", "gptb_tzgemm", ops.OriTZGEMMKernel(0, 0, 0, 300, 200, 130), (148, 1, 1), (192, 1, 1), 0, 6)
    assert (tz.kernel_.M_GLOBAL, tz.kernel_.N_GLOBAL, tz.kernel_.K_GLOBAL, tz.kernel_.ori_blks) == (256, 128, 128, 8)
    assert len(tz.kernelParams) == 7 + 6 and tz.ptb_iter_block_step == 148
    st = ops.GPTBKernel("stencil", "gptb_stencil", ops.OriSTENCILKernel(1, 2, 0, 0, 512, 512, 64), (444, 1, 1), (128, 1, 1), 0, 1024)
    assert [p.value for p in st.kernelParams[7:]] == [8, 128, 1, 32, 4, 1]
    mk = ops.MixKernel("tzgemm_stencil", st, tz, (148, 1, 1), (448, 1, 1), 0, 100, 0, 6)
    assert len(mk.kernelParams) == 32
    assert [p.value for p in mk.kernelParams[13:16]] == [0, 148, 100]
    assert [p.value for p in mk.kernelParams[29:32]] == [0, 148, 6]
    assert ops.query is not None
