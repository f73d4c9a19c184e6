// Types shared by the host launchers and the C-ABI of the B200 attention-forward library.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace tfa_b200 {

// Status codes returned by every C-ABI entry point (0 = success).
enum Status : int {
  kOk = 0,
  kBadDtype = 1,       // dtype code is not 1 (fp16), 2 (bf16) or 3 (fp32)
  kBadHeadDim = 2,     // head dim not in {32, 64, 96, 128, 192, 256}
  kBadArgument = 3,    // null pointer, negative size, Hq % Hkv != 0, misaligned pointer ...
  kCudaError = 4,      // a CUDA runtime / driver call failed (see tfa_b200_last_error_string)
  kWrongDevice = 5,    // current device is not compute capability 10.x
  kTooLarge = 6,       // a size exceeds what an entry point supports
  kDeviceTimeout = 7,  // a bounded wait inside a kernel gave up (reported by tfa_b200_device_status)
};

// dtype codes follow the reference binding (reference csrc/binding/flash_attn_binding.cu:22).
enum DType : int { kFp16 = 1, kBf16 = 2, kFp32 = 3 };

// One attention-forward problem, fixed-length or packed variable-length.
// Layouts (reference csrc/flash_attn/params.cuh:49-68, 97-116):
//   fixed : Q,O [B,Sq,Hq,D]   K,V [B,Skv,Hkv,D]        cuQ == cuKV == nullptr
//   varlen: Q,O [totalQ,Hq,D] K,V [totalKV,Hkv,D]      cuQ/cuKV = int32 [B+1] prefix sums on the device;
//           seqLenQ / seqLenKV then hold the maximum lengths and only size the grid
//           (reference csrc/flash_attn/launcher.cuh:94-98).
struct FwdProblem {
  const void* Q;
  const void* K;
  const void* V;
  void* O;
  const int* cuQ;
  const int* cuKV;
  int dtype;
  int batch;
  int seqLenQ;
  int seqLenKV;
  long long totalQ;   // rows of Q/O  (fixed: B*Sq; varlen: upper bound known on the host, or -1)
  long long totalKV;  // rows of K/V
  int headsQ;
  int headsKV;
  int headDim;
  int causal;
  cudaStream_t stream;
};

// The device status word holds 0, or (launch epoch << 8) | site code once a bounded wait inside a kernel gave up.

int launch_fwd_fp32(const FwdProblem& p);    // fp32: CUDA-core FMA kernel
void set_error_string(const char* fmt, ...);
// argument checks shared by every entry point (c_abi.cu); both return a Status
int validate_common(const void* Q, const void* K, const void* V, void* O, int dtype, int batch, int sq, int skv, int hq,
                    int hkv, int d);
int check_device();  // current device must be compute capability 10.x

}  // namespace tfa_b200
