"""ctypes loader for libtinyfa_b200.so (the C ABI declared in include/tinyfa_b200.h).

There is no CPU fallback: if the shared library is missing the import fails loudly.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtinyfa_b200.so")

STATUS_NAMES = {
    0: "OK",
    1: "BAD_DTYPE",
    2: "BAD_HEAD_DIM",
    3: "BAD_ARGUMENT",
    4: "CUDA_ERROR",
    5: "WRONG_DEVICE",
    6: "TOO_LARGE",
    7: "DEVICE_TIMEOUT",
}

# every symbol include/tinyfa_b200.h declares
EXPORTED_SYMBOLS = (
    "tfa_b200_fwd",
    "tfa_b200_fwd_varlen",
    "tfa_b200_head_dim_supported",
    "tfa_b200_last_error_string",
    "tfa_b200_device_status",
    "tfa_b200_set_option",
    "tfa_b200_version",
    "tfa_b200_fwd_decode_noalloc",
)

_lib = None


def load():
    """Load the shared library once and declare the argument types of its entry points."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `make -C tinyfa_b200/csrc` (or __graft_entry__.build()). "
            "This package has no fallback path."
        )
    lib = ctypes.CDLL(LIB_PATH)
    vp, ci, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    lib.tfa_b200_fwd.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, ci, vp]
    lib.tfa_b200_fwd.restype = ci
    lib.tfa_b200_fwd_varlen.argtypes = [vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ll, ll, ci, ci, ci, ci, vp]
    lib.tfa_b200_fwd_varlen.restype = ci
    lib.tfa_b200_head_dim_supported.argtypes = [ci]
    lib.tfa_b200_head_dim_supported.restype = ci
    lib.tfa_b200_last_error_string.argtypes = []
    lib.tfa_b200_last_error_string.restype = ctypes.c_char_p
    lib.tfa_b200_device_status.argtypes = [ctypes.POINTER(ci)]
    lib.tfa_b200_device_status.restype = ci
    lib.tfa_b200_set_option.argtypes = [ctypes.c_char_p, ci]
    lib.tfa_b200_set_option.restype = ci
    lib.tfa_b200_fwd_decode_noalloc.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, ci, ci, vp]
    lib.tfa_b200_fwd_decode_noalloc.restype = ci
    lib.tfa_b200_version.argtypes = []
    lib.tfa_b200_version.restype = ctypes.c_char_p
    _lib = lib
    return lib


def last_error():
    return load().tfa_b200_last_error_string().decode("utf-8", "replace")


def check(status, what):
    if status != 0:
        raise RuntimeError(f"{what} failed: {STATUS_NAMES.get(status, status)}: {last_error()}")
