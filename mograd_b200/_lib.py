"""ctypes binding of libmograd_b200.so (the C ABI declared in include/mograd_b200.h).

The library is required: importing the symbols fails loudly when the shared
object has not been built (``python -m mograd_b200.build``); there is no
fallback implementation of any operator.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("MOGRAD_B200_SO", os.path.join(_HERE, "libmograd_b200.so"))

_p = ctypes.c_void_p
_i64 = ctypes.c_int64
_int = ctypes.c_int
_f32 = ctypes.c_float
_sz = ctypes.c_size_t

BF16 = 0
F32 = 1
F16 = 2

OK = 0
EINVAL = -1
EDTYPE = -2
EALIGN = -3
EWORKSPACE = -4
ECUDA = -5
EUNSUPPORTED = -6

# name -> (restype, argtypes); mirrors include/mograd_b200.h declaration by declaration
SIGNATURES = {
    "mograd_b200_abi_version": (_int, []),
    "mograd_b200_launch_count": (ctypes.c_ulonglong, []),
    "mograd_b200_last_error": (ctypes.c_char_p, []),
    "mograd_b200_device_status": (_int, [ctypes.POINTER(_int), ctypes.POINTER(_int)]),
    "mograd_b200_device_status_async": (_int, [_p, _p]),
    "mograd_b200_selftest_wait_expiry": (_int, [ctypes.c_uint, _p]),
    "mograd_b200_matmul_bias_bt": (_int, [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _int, _int, _p]),
    "mograd_b200_matmul_bias_bt_bwd_workspace_bytes": (_sz, [_i64, _i64, _i64, _int]),
    "mograd_b200_matmul_bias_bt_bwd": (_int, [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i64,
                                              _i64, _int, _p, _sz, _p]),
    "mograd_b200_layer_norm_fwd": (_int, [_p, _p, _p, _p, _p, _p, _i64, _i64, _f32, _int, _p]),
    "mograd_b200_layer_norm_bwd_workspace_bytes": (_sz, [_i64, _i64, _int]),
    "mograd_b200_layer_norm_bwd": (_int, [_p, _p, _p, _p, _p, _p, _i64, _i64, _f32, _int, _p, _sz, _p]),
    "mograd_b200_layer_norm_bwd_static": (_int, [_p, _p, _p, _p, _p, _p, _i64, _i64, _f32, _int, _p]),
    "mograd_b200_cross_entropy_workspace_bytes": (_sz, [_i64, _i64, _int]),
    "mograd_b200_cross_entropy": (_int, [_p, _p, _p, _i64, _i64, _i64, _i64, _int, _p, _sz, _p]),
    "mograd_b200_cross_entropy_grad": (_int, [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _int, _p]),
    "mograd_b200_softmax_xent_workspace_bytes": (_sz, [_i64, _i64, _int]),
    "mograd_b200_softmax_xent_fwd_bwd": (_int, [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _f32, _int, _p, _sz, _p]),
    "mograd_b200_flash_attn_fwd": (_int, [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _f32, _int, _int, _int,
                                          _p]),
    "mograd_b200_flash_attn_bwd_workspace_bytes": (_sz, [_i64, _i64, _i64, _i64, _int]),
    "mograd_b200_flash_attn_bwd": (_int, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _f32,
                                          _int, _int, _int, _p, _sz, _p]),
    "mograd_b200_matmul_bias_bt_ex": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _int, _int,
                                             _p]),
    "mograd_b200_matmul_bias_bt_bwd_ex": (_int, [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64,
                                                 _i64, _i64, _i64, _i64, _int, _p, _sz, _p]),
    "mograd_b200_matmul_bias_bt_relu_bits": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _int,
                                                    _p]),
    "mograd_b200_matmul_bias_bt_bwd_relu_bits": (_int, [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64,
                                                        _i64, _i64, _i64, _i64, _i64, _int, _p, _sz, _p]),
    "mograd_b200_layer_norm_bwd_ex": (_int, [_p, _p, _p, _p, _p, _p, _p, _i64, _i64, _f32, _int, _p, _sz, _p]),
    "mograd_b200_flash_attn_fwd_ex": (_int, [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _f32, _int, _int, _i64,
                                             _int, _int, _p]),
    "mograd_b200_flash_attn_bwd_ex": (_int, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _f32,
                                             _int, _int, _i64, _i64, _int, _int, _p, _sz, _p]),
    "mograd_b200_relu_grad": (_int, [_p, _p, _p, _i64, _int, _p]),
    "mograd_b200_add": (_int, [_p, _p, _p, _i64, _int, _p]),
    "mograd_b200_gather_rows": (_int, [_p, _p, _p, _i64, _i64, _i64, _int, _p]),
    "mograd_b200_scatter_add_rows_workspace_bytes": (_sz, [_i64, _i64, _int]),
    "mograd_b200_scatter_add_rows": (_int, [_p, _p, _p, _i64, _i64, _i64, _int, _p, _sz, _p]),
    "mograd_b200_adamw_step": (_int, [_p, _p, _p, _p, _p, _i64, _f32, _f32, _f32, _f32, _f32, _int, _f32, _int, _p]),
    "mograd_b200_adamw_step_dev": (_int, [_p, _p, _p, _p, _p, _i64, _f32, _f32, _f32, _f32, _f32, _p, _int, _f32, _int,
                                          _p]),
}


class KernelError(RuntimeError):
    """A C-ABI call returned a negative status (the Mojo host would raise Error)."""

    def __init__(self, name: str, code: int, message: str):
        super().__init__(f"{name} failed with status {code}: {message}")
        self.code = code
        self.message = message


_lib = None


def load() -> ctypes.CDLL:
    """dlopen the kernel library once and attach the prototypes."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m mograd_b200.build` "
                "(mograd_b200 has no CPU or PyTorch fallback)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError = header and library disagree
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def call(name: str, *args) -> None:
    """Call a status-returning entry point; raise KernelError on a negative status."""
    lib = load()
    rc = getattr(lib, name)(*args)
    if rc != OK:
        raise KernelError(name, rc, lib.mograd_b200_last_error().decode("utf-8", "replace"))


def query(name: str, *args) -> int:
    return int(getattr(load(), name)(*args))


def device_status() -> tuple[int, int]:
    """(code, detail) of the device status word, cleared by the read; synchronises the device."""
    code, detail = _int(0), _int(0)
    call("mograd_b200_device_status", ctypes.byref(code), ctypes.byref(detail))
    return code.value, detail.value


def check_device_status(where: str) -> None:
    """Raise KernelError when a kernel's bounded wait gave up since the last check (its outputs are garbage)."""
    code, detail = device_status()
    if code != 0:
        raise KernelError(where, ECUDA, f"a bounded device-side wait gave up (status {code}, detail {detail}); "
                                        "the results of the kernels launched since the last check are invalid")
