"""Packaging of the B200 attention-forward library:  pip install --no-build-isolation .

Takes the place of the reference's python/setup.py.  The native library is built with
`make -C tinyfa_b200/csrc`, which reads the same build switches from the environment as the reference
(reference python/setup.py:77-132):

    TFA_TARGET_HEADDIM_<N>=0|OFF|FALSE|NO    leave head dim N out (default: 32, 64, 96, 128, 192, 256 all in)
    TFA_TARGET_DTYPE=fp16|bf16|fp32         compile one dtype only (default: all)

e.g.  TFA_TARGET_DTYPE=bf16 TFA_TARGET_HEADDIM_32=0 pip install --no-build-isolation .

There is no TFA_TARGET_SM here: the library targets sm_100a only.  Two packages are installed: `tinyfa_b200`
(ctypes binding + libtinyfa_b200.so) and `tiny_flash_attn` (the reference's module name, re-exporting
flash_attn_forward / flash_attn_varlen_forward).  The C header and the drop-in C++ header are installed as package
data under tinyfa_b200/include.
"""
import os
import shutil
import subprocess

from setuptools import Distribution, setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(ROOT, "tinyfa_b200", "csrc")

_all_headdims = [32, 64, 96, 128, 192, 256]
_enabled = [hd for hd in _all_headdims
            if os.environ.get(f"TFA_TARGET_HEADDIM_{hd}", "1").strip().upper() not in ("0", "OFF", "FALSE", "NO")]
_dtype = os.environ.get("TFA_TARGET_DTYPE", "").strip().lower()
if not _enabled:
    raise ValueError("All HeadDims are disabled. At least one TFA_TARGET_HEADDIM_<N> must be enabled.")
if _dtype not in ("", "fp16", "bf16", "fp32"):
    raise ValueError(f"TFA_TARGET_DTYPE='{_dtype}' cannot be mapped. Valid values: fp16, bf16, fp32")


class BuildNative(build_py):
    """Builds libtinyfa_b200.so before the Python files are collected."""

    def run(self):
        print("=" * 40)
        print(f"[TinyFA-B200] TFA_TARGET_DTYPE   = '{_dtype}'")
        print(f"[TinyFA-B200] HeadDims enabled   = {_enabled}")
        print("=" * 40)
        jobs = str(os.cpu_count() or 4)
        subprocess.check_call(["make", "-C", CSRC, "-j", jobs])
        inc_dst = os.path.join(ROOT, "tinyfa_b200", "include")
        if os.path.isdir(inc_dst):
            shutil.rmtree(inc_dst)
        shutil.copytree(os.path.join(ROOT, "include"), inc_dst)
        try:
            super().run()
        finally:
            shutil.rmtree(inc_dst, ignore_errors=True)


class BinaryDistribution(Distribution):
    """The wheel carries a native library: tag it for this platform."""

    def has_ext_modules(self):
        return True


setup(
    name="tinyfa_b200",
    version="0.1.0",
    description="B200-native (sm_100a) Flash Attention forward behind the TinyFA API",
    packages=["tinyfa_b200", "tiny_flash_attn"],
    package_data={"tinyfa_b200": ["libtinyfa_b200.so", "include/*.h", "include/flash_attn/*.cuh"]},
    python_requires=">=3.9",
    install_requires=["torch"],
    cmdclass={"build_py": BuildNative},
    distclass=BinaryDistribution,
    zip_safe=False,
)
