"""TEST INFRASTRUCTURE ONLY: Python face of the CPU oracle (oracle/attention_oracle.c).

Only tests/, the smoke run and the benchmark's CPU-baseline / reference legs may import this module;
the product package (tinyfa_b200/, tiny_flash_attn/) never does.

`fixed()` / `varlen()` compute attention forward on the host in fp64 (default) or in fp32 with the
reference CPU code's operation order (reference tests/cpp/cpu_reference.h:14-66, 68-129).  Inputs are
numpy float32 arrays holding the (already dtype-rounded) values the device kernel sees.

`ref_cpu()` gives access to the reference's own cpu_reference.h compiled behind a C shim
(oracle/_ref/libtinyfa_refcpu.so, built by `make -C oracle ref_cpu` where the reference is present);
`ref_gpu()` to the reference's CUDA kernels built for sm_100a (oracle/_ref/libtinyfa_ref.so).
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_PORT = os.path.join(_HERE, "liboracle.so")
_REF_CPU = os.path.join(_HERE, "_ref", "libtinyfa_refcpu.so")
_REF_GPU = os.path.join(_HERE, "_ref", "libtinyfa_ref.so")

_fp = ctypes.POINTER(ctypes.c_float)
_dp = ctypes.POINTER(ctypes.c_double)
_ip = ctypes.POINTER(ctypes.c_int)
_ci = ctypes.c_int


def build(targets=("port",)):
    """Compile the oracle with the Makefile beside this file (building the checker is not using it)."""
    subprocess.run(["make", "-C", _HERE, "-j8", *targets], check=True, capture_output=True)


_port = None


def port():
    global _port
    if _port is None:
        if not os.path.exists(_PORT):
            build(("port",))
        lib = ctypes.CDLL(_PORT)
        lib.tfa_oracle_fixed_f32.argtypes = [_fp, _fp, _fp, _fp] + [_ci] * 8
        lib.tfa_oracle_fixed_f64.argtypes = [_fp, _fp, _fp, _dp] + [_ci] * 8
        lib.tfa_oracle_varlen_f32.argtypes = [_fp, _fp, _fp, _fp, _ip, _ip] + [_ci] * 5
        lib.tfa_oracle_varlen_f64.argtypes = [_fp, _fp, _fp, _dp, _ip, _ip] + [_ci] * 5
        lib.tfa_oracle_num_threads.restype = _ci
        _port = lib
    return _port


def num_threads():
    return int(port().tfa_oracle_num_threads())


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def fixed(Q, K, V, causal=False, precision="f64", q_rows=0):
    """Q [B,Sq,Hq,D], K,V [B,Skv,Hkv,D] float32 -> O [B,Sq,Hq,D] (float64 or float32)."""
    Q, K, V = _f32(Q), _f32(K), _f32(V)
    B, Sq, Hq, D = Q.shape
    Skv, Hkv = K.shape[1], K.shape[2]
    assert K.shape == (B, Skv, Hkv, D) and V.shape == K.shape and Hq % Hkv == 0
    lib = port()
    if precision == "f64":
        O = np.zeros(Q.shape, dtype=np.float64)
        lib.tfa_oracle_fixed_f64(Q.ctypes.data_as(_fp), K.ctypes.data_as(_fp), V.ctypes.data_as(_fp),
                                 O.ctypes.data_as(_dp), B, Sq, Skv, Hq, Hkv, D, int(causal), int(q_rows))
    else:
        O = np.zeros(Q.shape, dtype=np.float32)
        lib.tfa_oracle_fixed_f32(Q.ctypes.data_as(_fp), K.ctypes.data_as(_fp), V.ctypes.data_as(_fp),
                                 O.ctypes.data_as(_fp), B, Sq, Skv, Hq, Hkv, D, int(causal), int(q_rows))
    return O


def varlen(Q, K, V, cu_q, cu_kv, causal=False, precision="f64"):
    """Q [Tq,Hq,D], K,V [Tkv,Hkv,D] float32, cu_* int32 [B+1] -> O [Tq,Hq,D]."""
    Q, K, V = _f32(Q), _f32(K), _f32(V)
    cu_q = np.ascontiguousarray(cu_q, dtype=np.int32)
    cu_kv = np.ascontiguousarray(cu_kv, dtype=np.int32)
    Tq, Hq, D = Q.shape
    Hkv = K.shape[1]
    B = cu_q.shape[0] - 1
    assert cu_kv.shape[0] == B + 1 and Hq % Hkv == 0 and V.shape == K.shape
    lib = port()
    if precision == "f64":
        O = np.zeros(Q.shape, dtype=np.float64)
        lib.tfa_oracle_varlen_f64(Q.ctypes.data_as(_fp), K.ctypes.data_as(_fp), V.ctypes.data_as(_fp),
                                  O.ctypes.data_as(_dp), cu_q.ctypes.data_as(_ip), cu_kv.ctypes.data_as(_ip), B, Hq,
                                  Hkv, D, int(causal))
    else:
        O = np.zeros(Q.shape, dtype=np.float32)
        lib.tfa_oracle_varlen_f32(Q.ctypes.data_as(_fp), K.ctypes.data_as(_fp), V.ctypes.data_as(_fp),
                                  O.ctypes.data_as(_fp), cu_q.ctypes.data_as(_ip), cu_kv.ctypes.data_as(_ip), B, Hq,
                                  Hkv, D, int(causal))
    return O


# --------------------------------------------------------------------------- the reference itself
_ref_cpu = None


def ref_cpu_available():
    return os.path.exists(_REF_CPU)


def ref_cpu():
    """The reference's own cpu_reference.h (compiled where it lies) behind a C shim."""
    global _ref_cpu
    if _ref_cpu is None:
        lib = ctypes.CDLL(_REF_CPU)
        lib.tfa_refcpu_fixed.argtypes = [_fp, _fp, _fp, _fp] + [_ci] * 7
        lib.tfa_refcpu_varlen.argtypes = [_fp, _fp, _fp, _fp, _ip, _ip] + [_ci] * 5
        lib.tfa_refcpu_fixed_mt.argtypes = [_fp, _fp, _fp, _fp] + [_ci] * 8
        lib.tfa_refcpu_num_threads.restype = _ci
        _ref_cpu = lib
    return _ref_cpu


def ref_cpu_fixed(Q, K, V, causal=False, threads=False, q_rows=0):
    Q, K, V = _f32(Q), _f32(K), _f32(V)
    B, Sq, Hq, D = Q.shape
    Skv, Hkv = K.shape[1], K.shape[2]
    O = np.zeros(Q.shape, dtype=np.float32)
    lib = ref_cpu()
    args = [Q.ctypes.data_as(_fp), K.ctypes.data_as(_fp), V.ctypes.data_as(_fp), O.ctypes.data_as(_fp), B, Sq, Skv, Hq,
            Hkv, D, int(causal)]
    if threads:
        lib.tfa_refcpu_fixed_mt(*args, int(q_rows))
    else:
        lib.tfa_refcpu_fixed(*args)
    return O


def ref_cpu_varlen(Q, K, V, cu_q, cu_kv, causal=False):
    Q, K, V = _f32(Q), _f32(K), _f32(V)
    cu_q = np.ascontiguousarray(cu_q, dtype=np.int32)
    cu_kv = np.ascontiguousarray(cu_kv, dtype=np.int32)
    O = np.zeros(Q.shape, dtype=np.float32)
    ref_cpu().tfa_refcpu_varlen(Q.ctypes.data_as(_fp), K.ctypes.data_as(_fp), V.ctypes.data_as(_fp),
                                O.ctypes.data_as(_fp), cu_q.ctypes.data_as(_ip), cu_kv.ctypes.data_as(_ip),
                                cu_q.shape[0] - 1, Q.shape[1], K.shape[1], Q.shape[2], int(causal))
    return O


_ref_gpu = None


def ref_gpu_available():
    return os.path.exists(_REF_GPU)


def ref_gpu():
    """The reference's CUDA kernels (its SM8x tile table) compiled for sm_100a, behind a C shim."""
    global _ref_gpu
    if _ref_gpu is None:
        lib = ctypes.CDLL(_REF_GPU)
        vp = ctypes.c_void_p
        lib.tfa_ref_fwd.argtypes = [vp, vp, vp, vp] + [_ci] * 8 + [vp]
        lib.tfa_ref_fwd.restype = _ci
        lib.tfa_ref_fwd_varlen.argtypes = [vp, vp, vp, vp, vp, vp] + [_ci] * 8 + [vp]
        lib.tfa_ref_fwd_varlen.restype = _ci
        _ref_gpu = lib
    return _ref_gpu


_TORCH_CODE = None


def _code(t):
    import torch

    return {torch.float16: 1, torch.bfloat16: 2, torch.float32: 3}[t.dtype]


def ref_gpu_fixed(Q, K, V, causal=False, out=None):
    """Run the reference kernels on torch CUDA tensors [B,S,H,D]; returns O (zero-initialised like the binding)."""
    import torch

    O = torch.zeros_like(Q) if out is None else out
    B, Sq, Hq, D = Q.shape
    rc = ref_gpu().tfa_ref_fwd(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), _code(Q), B, Sq, K.shape[1], Hq,
                               K.shape[2], D, int(causal), torch.cuda.current_stream().cuda_stream)
    if rc != 0:
        raise RuntimeError(f"reference library returned {rc}")
    return O


def ref_gpu_varlen(Q, K, V, cu_q, cu_kv, max_q, max_kv, causal=False):
    import torch

    O = torch.zeros_like(Q)
    rc = ref_gpu().tfa_ref_fwd_varlen(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), cu_q.data_ptr(),
                                      cu_kv.data_ptr(), _code(Q), cu_q.shape[0] - 1, int(max_q), int(max_kv),
                                      Q.shape[1], K.shape[1], Q.shape[2], int(causal),
                                      torch.cuda.current_stream().cuda_stream)
    if rc != 0:
        raise RuntimeError(f"reference library returned {rc}")
    return O
