"""The C-ABI library builds for sm_100a, loads without a GPU, and exports every
symbol include/gorch_cuda_shim.h declares. No compute calls here."""
import ctypes as C
import os
import re

from gorch_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "gorch_cuda_shim.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gorch_cuda_\w+)\s*\(", text)))


def test_library_builds_and_exports_header_symbols():
    path = build.build()
    assert os.path.exists(path)
    lib = C.CDLL(path)
    names = declared_symbols()
    assert len(names) >= 19
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert sorted(_lib.EXPORTS) == names


def test_no_device_is_a_clean_error():
    """Without a GPU the context constructor returns NULL plus a message (the
    NULL + errOut convention of metal/shim.h:30-35); with one it succeeds."""
    lib = _lib.load()
    err = C.c_void_p()
    ctx = lib.gorch_cuda_create_ctx(0, C.byref(err))
    if ctx:
        lib.gorch_cuda_release(ctx)
    else:
        assert err.value
        msg = C.string_at(err.value)
        assert b"gorch_cuda" in msg
        lib.gorch_cuda_free_string(err)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    import pytest
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "libgorchcuda.so"))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _lib.load()


def test_product_does_not_touch_the_oracle():
    """Nothing under gorch_b200/ may import, link or mention the oracle."""
    pkg = os.path.join(ROOT, "gorch_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp", ".hpp")):
                text = open(os.path.join(dirpath, f), errors="replace").read()
                assert "oracle" not in text.lower(), os.path.join(dirpath, f)


def test_comm_entry_points_fail_cleanly():
    """The multi-GPU entry points without a context or a buffer: an error code and a message, never
    a crash or a hang; making a unique id either works or reports an NCCL error (no GPU here)."""
    lib = _lib.load()
    err = C.c_void_p()
    assert lib.gorch_cuda_comm_init(None, 0, 2, None, C.byref(err)) == 1          # GORCH_CUDA_ERR_BAD_ARG
    assert b"null context" in C.string_at(err.value)
    lib.gorch_cuda_free_string(err)
    err = C.c_void_p()
    assert lib.gorch_cuda_comm_release(None, C.byref(err)) == 1
    lib.gorch_cuda_free_string(err)
    err = C.c_void_p()
    assert lib.gorch_cuda_comm_unique_id(None, C.byref(err)) == 1
    lib.gorch_cuda_free_string(err)
    err = C.c_void_p()
    rc = lib.gorch_cuda_sample_vocab_sharded_dev(None, None, 0, 1, 1, 1, 0, 1, 0, None, None, None, None, C.byref(err))
    assert rc == 1
    lib.gorch_cuda_free_string(err)
