"""Build-time kernel selection and packaging (no GPU needed).

The reference selects kernels with TFA_TARGET_HEADDIM_<N> and TFA_TARGET_DTYPE in both of its build systems
(reference python/setup.py:77-132, CMakeLists.txt:72-79,160-177) and reports the result through
tfa::isHeadDimCompiled (reference csrc/flash_attn/config.cuh:102-131).  The same switches drive
tinyfa_b200/csrc/Makefile, setup.py and CMakeLists.txt here.
"""
import ctypes
import os
import shutil
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "tinyfa_b200", "csrc")
HEAD_DIMS = (32, 64, 96, 128, 192, 256)


def _load(path):
    lib = ctypes.CDLL(path)
    vp, ci = ctypes.c_void_p, ctypes.c_int
    lib.tfa_b200_fwd.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, ci, vp]
    lib.tfa_b200_last_error_string.restype = ctypes.c_char_p
    return lib


def _make(tmp_path, **env):
    out = tmp_path / "libfiltered.so"
    e = dict(os.environ)
    e.update(env)
    r = subprocess.run(["make", "-C", CSRC, "-j8", f"BUILD={tmp_path / 'obj'}", f"OUT={out}"], env=e,
                       capture_output=True, text=True)
    return r, out


def test_default_build_has_every_head_dim():
    from tinyfa_b200 import _lib
    lib = _lib.load()
    assert [lib.tfa_b200_head_dim_supported(d) for d in HEAD_DIMS] == [1] * 6
    assert lib.tfa_b200_head_dim_supported(48) == 0


def test_makefile_filters_head_dims_and_dtype(tmp_path):
    off = {f"TFA_TARGET_HEADDIM_{d}": "0" for d in HEAD_DIMS if d != 64}
    r, out = _make(tmp_path, TFA_TARGET_DTYPE="fp32", **off)
    assert r.returncode == 0, r.stdout + r.stderr
    # fp32 only: no tensor-core kernel object was compiled
    assert not [f for f in os.listdir(tmp_path / "obj") if f.startswith("fwd_tc_")]
    lib = _load(str(out))
    assert [lib.tfa_b200_head_dim_supported(d) for d in HEAD_DIMS] == [0, 1, 0, 0, 0, 0]
    # argument checks come before any CUDA call, so they can be exercised without a device
    assert lib.tfa_b200_fwd(16, 16, 16, 16, 1, 1, 8, 8, 2, 2, 64, 0, None) == 1      # fp16 left out -> BAD_DTYPE
    assert b"not compiled" in lib.tfa_b200_last_error_string()
    assert lib.tfa_b200_fwd(16, 16, 16, 16, 3, 1, 8, 8, 2, 2, 128, 0, None) == 2     # hd128 left out -> BAD_HEAD_DIM
    assert b"TFA_TARGET_HEADDIM_128" in lib.tfa_b200_last_error_string()
    assert lib.tfa_b200_fwd(16, 16, 16, 16, 3, 1, 8, 8, 2, 2, 100, 0, None) == 2     # never a valid head dim
    assert b"unsupported headDim" in lib.tfa_b200_last_error_string()


def test_makefile_off_spellings_and_shared_instantiation(tmp_path):
    # 32 and 64 share one tensor-core instantiation: leaving out 64 alone must keep the object, but not the head dim
    off = {"TFA_TARGET_HEADDIM_64": "OFF", "TFA_TARGET_HEADDIM_96": "false", "TFA_TARGET_HEADDIM_128": "No",
           "TFA_TARGET_HEADDIM_192": "0", "TFA_TARGET_HEADDIM_256": "0"}
    r, out = _make(tmp_path, TFA_TARGET_DTYPE="BF16", **off)
    assert r.returncode == 0, r.stdout + r.stderr
    objs = sorted(f for f in os.listdir(tmp_path / "obj") if f.startswith("fwd_tc_") and f.endswith(".o"))
    assert objs == ["fwd_tc_hdp64_bf1.o"]
    lib = _load(str(out))
    assert [lib.tfa_b200_head_dim_supported(d) for d in HEAD_DIMS] == [1, 0, 0, 0, 0, 0]
    assert lib.tfa_b200_fwd(16, 16, 16, 16, 3, 1, 8, 8, 2, 2, 32, 0, None) == 1      # fp32 left out


def test_makefile_rejects_bad_selection(tmp_path):
    r, _ = _make(tmp_path, TFA_TARGET_DTYPE="fp8")
    assert r.returncode != 0 and "fp16, bf16, fp32" in (r.stdout + r.stderr)
    r, _ = _make(tmp_path, **{f"TFA_TARGET_HEADDIM_{d}": "0" for d in HEAD_DIMS})
    assert r.returncode != 0 and "All head dims are disabled" in (r.stdout + r.stderr)


def test_setup_py_reads_the_same_switches():
    """setup.py validates the switches before anything is built (reference python/setup.py:109-112, 124-128)."""
    code = "import runpy, sys; sys.argv = ['setup.py', '--version']; runpy.run_path('setup.py')"
    env = dict(os.environ, TFA_TARGET_DTYPE="int8")
    r = subprocess.run([sys.executable, "-c", code], cwd=ROOT, env=env, capture_output=True, text=True)
    assert r.returncode != 0 and "fp16, bf16, fp32" in r.stderr
    env = dict(os.environ, **{f"TFA_TARGET_HEADDIM_{d}": "OFF" for d in HEAD_DIMS})
    r = subprocess.run([sys.executable, "-c", code], cwd=ROOT, env=env, capture_output=True, text=True)
    assert r.returncode != 0 and "All HeadDims are disabled" in r.stderr
    r = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True)
    assert r.returncode == 0 and "0.1.0" in r.stdout


@pytest.mark.skipif(shutil.which("cmake") is None, reason="cmake not installed")
def test_cmake_package_and_consumer(tmp_path):
    """CMake build with a filter, install, then a downstream project that does find_package(TinyFA) and links
    TinyFA::tinyfa (the reference's target, reference CMakeLists.txt:147-148) against the reference's include path."""
    bdir, prefix, cdir = tmp_path / "b", tmp_path / "prefix", tmp_path / "c"
    flags = ["-DTFA_TARGET_DTYPE=bf16"] + [f"-DTFA_TARGET_HEADDIM_{d}=OFF" for d in HEAD_DIMS if d != 128]
    for cmd in (["cmake", "-S", ROOT, "-B", str(bdir)] + flags,
                ["cmake", "--build", str(bdir), "-j8"],
                ["cmake", "--install", str(bdir), "--prefix", str(prefix)],
                ["cmake", "-S", os.path.join(ROOT, "tests", "cmake_consumer"), "-B", str(cdir),
                 f"-DCMAKE_PREFIX_PATH={prefix}"],
                ["cmake", "--build", str(cdir), "-j8"]):
        r = subprocess.run(cmd, capture_output=True, text=True)
        assert r.returncode == 0, " ".join(cmd) + "\n" + r.stdout[-3000:] + r.stderr[-3000:]
    lib = _load(str(prefix / "lib" / "libtinyfa_b200.so"))
    assert [lib.tfa_b200_head_dim_supported(d) for d in HEAD_DIMS] == [0, 0, 0, 1, 0, 0]
    # the consumer only asks which head dims are compiled: runs without a device
    r = subprocess.run([str(cdir / "consumer")], capture_output=True, text=True,
                       env=dict(os.environ, LD_LIBRARY_PATH=str(prefix / "lib")))
    assert r.returncode == 0 and "head dims compiled: 1" in r.stdout
