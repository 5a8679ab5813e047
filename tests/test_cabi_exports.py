"""CPU-only checks of the drop-in boundary: the library builds for sm_100a without a GPU, loads,
exports every symbol include/kvcomp_b200.h declares, and its host-side argument checks return
error codes (never abort).  No kernel is launched here."""
import ctypes as C
import os
import re

import pytest

from kvcomp_b200 import _lib

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    return _lib.load()


def declared_symbols():
    with open(os.path.join(REPO, "include", "kvcomp_b200.h")) as f:
        text = f.read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(kvc_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(lib):
    names = declared_symbols()
    assert len(names) >= 18
    for n in names:
        assert hasattr(lib, n), "library does not export %s" % n
    assert sorted(_lib.EXPORTS) == names


def test_constants_match_header():
    with open(os.path.join(REPO, "include", "kvcomp_b200.h")) as f:
        text = f.read()
    assert int(re.search(r"#define KVC_LUT_BITS\s+(\d+)", text).group(1)) == _lib.LUT_BITS
    for bit, name in _lib.FLAGS.items():
        m = re.search(r"#define KVC_FLAG_%s\s+0x([0-9a-fA-F]+)" % name, text)
        assert m and int(m.group(1), 16) == bit, name
    assert _lib.BOOK_BYTES == 64 + 2048 + 1536 + 2048 + 4 * (1 << _lib.LUT_BITS)


def test_version_and_buffer_sizes(lib):
    assert lib.kvc_version() == 1
    out = (C.c_int64 * 4)()
    # kernels.cu:893-917 on a [16,64,1,32,128] K tensor: (4096, 65536, 8, 4194304)
    assert lib.kvc_buffer_sizes(1024, 32 * 128, 1, out) == 0
    assert tuple(out) == (4096, 65536, 8, 4194304)
    assert lib.kvc_buffer_sizes(1024, 32 * 128, 0, out) == 0
    assert tuple(out) == (4096, 65536, 8, 4194304)
    # the reference aborts on these (tcom_assert); here they are error codes with a message
    assert lib.kvc_buffer_sizes(1000, 32 * 128, 1, out) == 1
    assert b"K_VEC_PER_BLK" in lib.kvc_last_error()
    assert lib.kvc_buffer_sizes(1088, 32 * 128, 0, out) == 1
    assert b"V_VEC_LEN" in lib.kvc_last_error()


def test_qmeta_make(lib):
    q = _lib.QMeta()
    n = C.c_int64()
    T, B, H, D = 256, 2, 4, 128
    expect = {  # mode, shared -> (tok_div, sj, sb, sh, sc, units)
        (0, 1): (64, 1, 0, 0, 0, 4), (0, 0): (64, 2, 1, 0, 0, 8),
        (1, 0): (64, B * H * D, H * D, D, 1, 4 * B * H * D),
        (2, 1): (1, 1, 0, 0, 0, 256), (2, 0): (1, 2, 1, 0, 0, 512),
        (3, 0): (1, B * H, H, 1, 0, 256 * B * H),
    }
    for (mode, shared), e in expect.items():
        assert lib.kvc_qmeta_make(mode, shared, T, B, H, D, 64, C.byref(q), C.byref(n)) == 0
        assert (q.tok_div, q.sj, q.sb, q.sh, q.sc, n.value) == e
    assert lib.kvc_qmeta_make(9, 0, T, B, H, D, 64, C.byref(q), C.byref(n)) == 1
    assert lib.kvc_qmeta_make(0, 0, 100, B, H, D, 64, C.byref(q), C.byref(n)) == 1


def test_null_and_shape_errors_return_codes(lib):
    z = C.c_void_p(0)
    assert lib.kvc_histogram(z, 10, z, z) == 1
    assert lib.kvc_build_codebook(z, z, z) == 1
    assert lib.kvc_book_from_tree(z, 6, z, z) == 1
    assert lib.kvc_quantize(z, 64, 1, 1, 128, 0, 1, 64, 0.05, z, z, 1, z, z, z, 0, z, z) == 1
    assert lib.kvc_encode(z, 64, 1, 1, z, 256, 0, z, z, z, 0, z, z, 0, z, z) == 1
    assert lib.kvc_decode(z, 0, z, z, z, 64, 1, 1, z, z, z) == 1
    assert lib.kvc_attn_decode(None, None, 128, 1, 1, 1, z, 1.0, z, z, 0, z, 0, z, 0, z, z) == 1
    assert lib.kvc_last_error() != b""
    assert lib.kvc_encode_workspace(1024, 32, 1) >= 512 * 4
    assert lib.kvc_attn_workspace(8, 32, 4) >= 8 * 32 * 4 * 130 * 4
    assert lib.kvc_attn_splits(4096, 8, 32, 148) >= 2
    assert lib.kvc_attn_splits(128, 1, 1, 148) == 1


def test_no_cpu_path():
    import torch
    from kvcomp_b200 import ops
    with pytest.raises(_lib.KvcError):
        ops.quantize(torch.zeros(64, 1, 1, 128, dtype=torch.float16), 0, 64, 0.05)
    with pytest.raises(_lib.KvcError):
        ops.histogram(torch.zeros(64, dtype=torch.uint8))


def test_header_is_valid_c_and_links_from_c(lib, tmp_path):
    """include/kvcomp_b200.h compiled as C by gcc and linked against the library: the boundary a cgo, JNI or
    FFI binding would use.  Host-only entry points are called; no kernel is launched."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if not gcc:
        pytest.skip("no C compiler")
    exe = str(tmp_path / "cabi_check")
    libdir = os.path.dirname(_lib.lib_path())
    r = subprocess.run([gcc, "-std=c11", "-Wall", "-Werror", "-I", os.path.join(REPO, "include"),
                        os.path.join(REPO, "tests", "cabi_check.c"), "-L", libdir, "-lkvcomp_b200",
                        "-Wl,-rpath," + libdir, "-o", exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([exe], capture_output=True, text=True)
    import ctypes
    want = "ok %d %d %d" % (_lib.BOOK_BYTES, ctypes.sizeof(_lib.Cache), ctypes.sizeof(_lib.QMeta))
    assert r.returncode == 0 and r.stdout.strip() == want, (r.returncode, r.stdout, r.stderr, want)
