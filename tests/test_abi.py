"""The C-ABI library loads and exports exactly what include/*.h declares (no compute, no GPU)."""
import ctypes
import glob
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = open(h).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(mograd_b200_\w+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    import mograd_b200
    from mograd_b200 import _lib

    lib = mograd_b200.load()
    decl = declared_symbols()
    assert decl, "no declarations found in include/*.h"
    for name in sorted(decl):
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert decl == set(_lib.SIGNATURES), "ctypes prototypes and header disagree"


def test_abi_version_and_error_text():
    import mograd_b200

    lib = mograd_b200.load()
    assert lib.mograd_b200_abi_version() == 1
    # argument validation happens before any CUDA call, so it works without a GPU
    rc = lib.mograd_b200_layer_norm_fwd(None, None, None, None, None, None, 4, 4, ctypes.c_float(1e-5), 0, None)
    assert rc == -1
    assert b"NULL" in lib.mograd_b200_last_error()


def test_bad_arguments_return_status_without_launching():
    from mograd_b200 import _lib

    lib = _lib.load()
    one = ctypes.c_void_p(256)  # never dereferenced: validation fails first
    f = ctypes.c_float
    assert lib.mograd_b200_layer_norm_bwd(one, one, one, one, one, one, 0, 8, f(1e-5), 0, None, 0, None) == _lib.EINVAL
    assert lib.mograd_b200_layer_norm_fwd(one, one, one, one, None, None, 4, 4, f(1e-5), 7, None) == _lib.EDTYPE
    assert lib.mograd_b200_layer_norm_fwd(one, one, one, one, None, None, 4, 1 << 20, f(1e-5), 0, None) == _lib.EUNSUPPORTED
    assert lib.mograd_b200_softmax_xent_fwd_bwd(one, one, one, one, 8, 8, 8, 8, f(1.0), 0, None, 0, None) == _lib.EWORKSPACE
    assert lib.mograd_b200_matmul_bias_bt(one, one, None, one, 4, 4, 4, 2, 4, 4, 0, 0, None) == _lib.EINVAL
    assert lib.mograd_b200_matmul_bias_bt(one, one, None, one, 4, 4, 4, 4, 4, 4, 0, 9, None) == _lib.EDTYPE


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from mograd_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    try:
        _lib.load()
    except ImportError as e:
        assert "no CPU or PyTorch fallback" in str(e)
    else:
        raise AssertionError("load() must fail when the shared object is missing")
