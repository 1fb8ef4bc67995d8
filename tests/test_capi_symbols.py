"""The C-ABI library loads on a machine without a GPU, exports every symbol the header declares, and
validates arguments on the host (negative status codes) before touching any device."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from daisy_b200 import _lib
    if not os.path.exists(_lib.LIB_PATH):
        from daisy_b200.build import build
        build()
    return _lib.lib()


def test_header_symbols_exported(lib):
    from daisy_b200 import _lib
    hdr = open(os.path.join(ROOT, "include", "daisy_b200.h")).read()
    declared = set(re.findall(r"\b(daisy_b200_\w+)\s*\(", hdr))
    assert declared, "no declarations parsed"
    assert declared == set(_lib.SIGNATURES), (declared ^ set(_lib.SIGNATURES))
    for name in declared:
        assert hasattr(lib, name), name


def test_version_and_strerror(lib):
    assert lib.daisy_b200_version() == 100
    for code in range(0, -8, -1):
        assert lib.daisy_b200_strerror(code)
    assert b"unknown" in lib.daisy_b200_strerror(-99)


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    from daisy_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.lib()


def test_argument_validation_without_gpu(lib):
    from daisy_b200 import _lib
    buf = (C.c_char * 4096)()
    a = C.addressof(buf)
    a = (a + 255) & ~255                                    # 256-byte aligned scratch address, never dereferenced
    # head_dim != 128
    assert lib.daisy_b200_qkv_prep(a, a, a, 0, 0, 0, 0, 0, 0, 0, 0, 0, a, a, a, a, a, None, 0, 0, 0, None, 1, 1, 1, 64, 1e-6, 15, None) == _lib.EUNSUPPORTED
    # null pointers / bad sizes
    assert lib.daisy_b200_qkv_prep(None, None, None, 0, 0, 0, 0, 0, 0, 0, 0, 0, a, a, None, None, None, None, 0, 0, 0, None, 1, 1, 1, 128, 1e-6, 15, None) == _lib.EINVAL
    assert lib.daisy_b200_swa_attend(None, a, a, 0, 0, 0, 0, 0, 0, 0, 0, 0, a, 0, 0, 0, 1, 1, 1, 128, 0, 0.12, None, 0, 0, None, None) == _lib.EINVAL
    assert lib.daisy_b200_swa_attend(a, a, a, 128, 128, 128, 128, 128, 128, 128, 128, 128, a, 128, 128, 128, 1, 1, 1, 128, 0, -1.0, None, 0, 0, None, None) == _lib.EINVAL
    # misaligned pointer / stride
    assert lib.daisy_b200_swa_attend(a + 2, a, a, 128, 128, 128, 128, 128, 128, 128, 128, 128, a, 128, 128, 128, 1, 1, 1, 128, 0, 0.12, None, 0, 0, None, None) == _lib.EALIGN
    assert lib.daisy_b200_swa_attend(a, a, a, 128, 132, 128, 128, 128, 128, 128, 128, 128, a, 128, 128, 128, 1, 1, 1, 128, 0, 0.12, None, 0, 0, None, None) == _lib.EALIGN
    # a broadcast (zero-stride) head or batch dimension longer than 1 is refused, not read at overlapping offsets
    assert lib.daisy_b200_swa_attend(a, a, a, 128, 128, 0, 128, 128, 128, 128, 128, 128, a, 256, 256, 128, 1, 1, 2, 128, 0, 0.12, None, 0, 0, None, None) == _lib.EINVAL
    assert lib.daisy_b200_swa_attend(a, a, a, 128, 128, 128, 0, 128, 128, 128, 128, 128, a, 128, 128, 128, 2, 1, 1, 128, 0, 0.12, None, 0, 0, None, None) == _lib.EINVAL
    # workspace too small
    need = lib.daisy_b200_swa_prefill_workspace_bytes(1, 128, 2, 128)
    assert need == 3 * 128 * 2 * 128 * 2
    assert lib.daisy_b200_swa_prefill_fwd(a, a, a, 256, 256, 128, 256, 256, 128, 256, 256, 128, a, a, a, 256, 256, 128, None, None,
                                          1, 128, 2, 128, 64, 0.12, 1e-6, None, 0, 15, a, need - 1, None, None) == _lib.EWORKSPACE
    # decode: workspace, D, negative t
    w = lib.daisy_b200_swa_decode_workspace_bytes(2, 3, 128, 4)
    assert w == 2 * 3 * 4 * 130 * 4
    args = [a, a, a, 384, 128, 384, 128, 384, 128, a, a, 0, 0, 128, 10, 64, 16, a, a, a, 384, 128, None, None, 2, 3, 128, 0.12, 1e-6, 15]
    assert lib.daisy_b200_swa_decode_step(*args, a, w - 1, 4, None, None) == _lib.EWORKSPACE
    bad = list(args); bad[26] = 64
    assert lib.daisy_b200_swa_decode_step(*bad, a, w, 4, None, None) == _lib.EUNSUPPORTED
    bad = list(args); bad[14] = -1
    assert lib.daisy_b200_swa_decode_step(*bad, a, w, 4, None, None) == _lib.EINVAL
    # KDA: K != 128, chunk != 64, workspace
    kw = lib.daisy_b200_kda_workspace_bytes(1, 100, 2, 128, 128)
    assert kw == 1 * 2 * 2 * 83456
    assert lib.daisy_b200_kda_workspace_bytes(1, 100, 2, 64, 128) == 0
    assert lib.daisy_b200_kda_chunk_fwd(a, a, a, a, a, None, a, None, 1, 100, 2, 64, 128, 64, 0.0, 1, a, kw, None, None) == _lib.EUNSUPPORTED
    assert lib.daisy_b200_kda_chunk_fwd(a, a, a, a, a, None, a, None, 1, 100, 2, 128, 128, 32, 0.0, 1, a, kw, None, None) == _lib.EUNSUPPORTED
    assert lib.daisy_b200_kda_chunk_fwd(a, a, a, a, a, None, a, None, 1, 100, 2, 128, 128, 64, 0.0, 1, a, kw - 1, None, None) == _lib.EWORKSPACE
    # packed KDA: the same records per chunk; tables are required; then the dense checks apply
    assert lib.daisy_b200_kda_varlen_workspace_bytes(2, 2, 128, 128) == kw
    assert lib.daisy_b200_kda_varlen_workspace_bytes(0, 2, 128, 128) == 0
    assert lib.daisy_b200_kda_chunk_fwd_varlen(a, a, a, a, a, None, a, None, 100, 2, 128, 128, 64, 0.0, 1, None, 2, a, 1,
                                               a, kw, None, None) == _lib.EINVAL
    assert lib.daisy_b200_kda_chunk_fwd_varlen(a, a, a, a, a, None, a, None, 100, 2, 128, 128, 64, 0.0, 1, a + 4, 2, a, 1,
                                               a, kw, None, None) == _lib.EALIGN
    assert lib.daisy_b200_kda_chunk_fwd_varlen(a, a, a, a, a, None, a, None, 100, 2, 128, 128, 64, 0.0, 1, a, 2, a, 1,
                                               a, kw - 1, None, None) == _lib.EWORKSPACE
    assert lib.daisy_b200_kda_short_conv_varlen(a, 256, a, None, None, None, a, 256, 8, 256, 4, None, 1, None) == _lib.EINVAL
    assert lib.daisy_b200_kda_short_conv_varlen(a, 256, a, None, a, a, a, 256, 8, 256, 4, a, 1, None) == _lib.EINVAL
    # ring copy: n > cap, bad element size
    assert lib.daisy_b200_ring_copy_rows(a, 1024, 512, 128, a, 1024, 512, 128, 1, 2, 128, 4, 0, 5, 2, 1, None) == _lib.EINVAL
    assert lib.daisy_b200_ring_copy_rows(a, 1024, 512, 128, a, 1024, 512, 128, 1, 2, 128, 4, 0, 2, 3, 1, None) == _lib.EINVAL
    # self-test entry: K must be 64 or 128
    assert lib.daisy_b200_selftest_umma(a, a, a, 96, 0, None, None) == _lib.EINVAL


def test_decode_split_heuristic(lib):
    s = lib.daisy_b200_swa_decode_splits
    assert s(64, 16, 4095, 148) >= 1
    assert s(8, 16, 4095, 148) > s(64, 16, 4095, 148)        # fewer (batch, head) pairs -> more splits
    assert s(1, 1, 100, 148) == 1                             # short contexts are not split
    assert s(1, 1, 100000, 148) == 64                         # capped
    assert s(0, 16, 10, 148) == 1
