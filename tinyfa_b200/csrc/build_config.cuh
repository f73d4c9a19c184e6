// Build-time kernel selection, with the reference's switches: TFA_TARGET_HEADDIM_<N> (defined = that head dim is
// compiled; reference csrc/flash_attn/config.cuh:44-131) and TFA_TARGET_DTYPE (1 = fp16 only, 2 = bf16 only,
// 3 = fp32 only, undefined = all; reference csrc/flash_attn/flash_api.cuh:27-41 via python/setup.py:100-132 and
// CMakeLists.txt:160-177).  The build files define one TFA_TARGET_HEADDIM_<N> per enabled head dim; a translation
// unit compiled without any of them gets all six.
#pragma once

#if !defined(TFA_TARGET_HEADDIM_32) && !defined(TFA_TARGET_HEADDIM_64) && !defined(TFA_TARGET_HEADDIM_96) && \
    !defined(TFA_TARGET_HEADDIM_128) && !defined(TFA_TARGET_HEADDIM_192) && !defined(TFA_TARGET_HEADDIM_256)
#define TFA_TARGET_HEADDIM_32 1
#define TFA_TARGET_HEADDIM_64 1
#define TFA_TARGET_HEADDIM_96 1
#define TFA_TARGET_HEADDIM_128 1
#define TFA_TARGET_HEADDIM_192 1
#define TFA_TARGET_HEADDIM_256 1
#endif

#ifdef TFA_TARGET_HEADDIM_32
#define TFA_HAVE_HD32 1
#else
#define TFA_HAVE_HD32 0
#endif
#ifdef TFA_TARGET_HEADDIM_64
#define TFA_HAVE_HD64 1
#else
#define TFA_HAVE_HD64 0
#endif
#ifdef TFA_TARGET_HEADDIM_96
#define TFA_HAVE_HD96 1
#else
#define TFA_HAVE_HD96 0
#endif
#ifdef TFA_TARGET_HEADDIM_128
#define TFA_HAVE_HD128 1
#else
#define TFA_HAVE_HD128 0
#endif
#ifdef TFA_TARGET_HEADDIM_192
#define TFA_HAVE_HD192 1
#else
#define TFA_HAVE_HD192 0
#endif
#ifdef TFA_TARGET_HEADDIM_256
#define TFA_HAVE_HD256 1
#else
#define TFA_HAVE_HD256 0
#endif

// The tensor-core kernels are instantiated per padded head dim: 32 and 64 share one, 96 and 128 share one.
#define TFA_HAVE_HDP64 (TFA_HAVE_HD32 || TFA_HAVE_HD64)
#define TFA_HAVE_HDP128 (TFA_HAVE_HD96 || TFA_HAVE_HD128)
#define TFA_HAVE_HDP192 TFA_HAVE_HD192
#define TFA_HAVE_HDP256 TFA_HAVE_HD256

#ifdef TFA_TARGET_DTYPE
#define TFA_HAVE_FP16 (TFA_TARGET_DTYPE == 1)
#define TFA_HAVE_BF16 (TFA_TARGET_DTYPE == 2)
#define TFA_HAVE_FP32 (TFA_TARGET_DTYPE == 3)
#else
#define TFA_HAVE_FP16 1
#define TFA_HAVE_BF16 1
#define TFA_HAVE_FP32 1
#endif

namespace tfa_b200 {

constexpr bool head_dim_compiled(int d) {
  return (d == 32 && TFA_HAVE_HD32) || (d == 64 && TFA_HAVE_HD64) || (d == 96 && TFA_HAVE_HD96) ||
         (d == 128 && TFA_HAVE_HD128) || (d == 192 && TFA_HAVE_HD192) || (d == 256 && TFA_HAVE_HD256);
}
constexpr bool dtype_compiled(int code) {
  return (code == 1 && TFA_HAVE_FP16) || (code == 2 && TFA_HAVE_BF16) || (code == 3 && TFA_HAVE_FP32);
}

}  // namespace tfa_b200
