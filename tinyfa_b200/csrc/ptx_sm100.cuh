// Inline-PTX wrappers for the sm_100a features the attention kernels use: mbarrier, bulk tensor
// copies (TMA), tensor memory (TMEM) management, tcgen05 MMA / load / store, register reallocation.
//
// Replaces the role of the reference's cp.async wrappers (reference csrc/flash_attn/ptx.cuh:13-38):
// where the reference stages tiles with 16-byte cp.async and synchronises with __syncthreads, these
// kernels stage whole tiles with one TMA instruction and synchronise through mbarriers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace tfa_b200 {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Non-blocking probe of a phase (try_wait may suspend the thread and wake it up late).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---------------------------------------------------------------- TMA (no cluster broadcast forms)
__device__ __forceinline__ void prefetch_tensormap(const void* desc) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(desc) : "memory");
}

// 4-D tiled load global -> shared (head dim, head, row within the batch entry, batch entry).
__device__ __forceinline__ void tma_load_4d(uint32_t smemDst, const void* desc, uint32_t bar, int x, int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smemDst), "l"(desc), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_4d(const void* desc, int x, int y, int z, int w) {
  asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global [%0, {%1, %2, %3, %4}];" ::"l"(desc), "r"(x), "r"(y), "r"(z),
               "r"(w)
               : "memory");
}

// Tensor maps that are completed on the device (the host cannot know a dimension without reading it back):
// the map is edited in shared memory, published to global memory with a release that orders the generic-proxy
// writes before later tensor-map-proxy reads, and acquired by the thread that will issue TMA copies through it.
__device__ __forceinline__ void tensormap_set_dim2(uint32_t smemMap, uint32_t extent) {
  asm volatile("tensormap.replace.tile.global_dim.shared::cta.b1024.b32 [%0], 2, %1;" ::"r"(smemMap), "r"(extent) : "memory");
}
// warp-collective: copies the 128-byte map from shared to global memory
__device__ __forceinline__ void tensormap_publish(void* globalMap, uint32_t smemMap) {
  asm volatile("tensormap.cp_fenceproxy.global.shared::cta.tensormap::generic.release.gpu.sync.aligned [%0], [%1], 128;" ::"l"(globalMap),
               "r"(smemMap)
               : "memory");
}
__device__ __forceinline__ void tensormap_acquire(const void* globalMap) {
  asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(globalMap) : "memory");
}

// ---------------------------------------------------------------- CTA pairs (cluster of two)
// The kernels that run one tcgen05.mma over two SMs launch clusters of two CTAs.  Rank 0 issues the MMAs; barriers
// that it waits on are reached from the other CTA through the cluster window of the shared address space.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cta address of this CTA -> shared::cluster address of the same offset in CTA `rank`
__device__ __forceinline__ uint32_t mapa(uint32_t localAddr, uint32_t rank) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(localAddr), "r"(rank));
  return a;
}
// Arrival on a barrier of either CTA of the pair.  Plain form: it hands over no generic-proxy data (what it orders -
// tensor-memory stores against the other CTA's MMAs - is covered by the tcgen05 fences around it); a cluster-scope
// release here was measured at ~1000 clocks per arrival in the softmax loop.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t clusterAddr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(clusterAddr) : "memory");
}
// Arrival that publishes this thread's earlier stores into the other CTA's shared memory (pairs with mbar_try_wait_cluster).
__device__ __forceinline__ void mbar_arrive_cluster_release(uint32_t clusterAddr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(clusterAddr) : "memory");
}
// wait that also makes the other CTA's plain stores (made before its cluster-scope arrival) visible
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void st_cluster_u32(uint32_t clusterAddr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(clusterAddr), "r"(v) : "memory");
}
// all threads of both CTAs
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// 4-D tiled load into this CTA's shared memory whose completion bytes are counted on a barrier that may live in
// the other CTA of the pair (clusterBar: a shared::cluster address).  No broadcast: every CTA loads its own data.
__device__ __forceinline__ void tma_load_4d_pair(uint32_t smemDst, const void* desc, uint32_t clusterBar, int x, int y, int z,
                                                 int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smemDst), "l"(desc), "r"(clusterBar), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}

// ---------------------------------------------------------------- register reallocation
template <int kRegs>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegs));
}
template <int kRegs>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegs));
}

// ---------------------------------------------------------------- tensor memory
// Allocate nCols (power of two, 32..512) TMEM columns; the base address is written to *smemDst.
// Warp-collective.
__device__ __forceinline__ void tmem_alloc(uint32_t smemDst, uint32_t nCols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemDst), "r"(nCols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t nCols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(nCols) : "memory");
}

// CTA-pair forms: one warp of each CTA of the pair executes them, with the same shared-memory offset.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smemDst, uint32_t nCols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemDst), "r"(nCols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t nCols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(nCols) : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Values loaded by tcgen05.ld are defined only after tcgen05.wait::ld, but the compiler sees no dependence between
// the wait and the destination registers.  Passing the registers through an empty volatile asm placed after the
// wait pins every later use behind it (volatile asm statements keep their order); it emits no instruction.
template <int N>
__device__ __forceinline__ void tmem_ld_fence(uint32_t (&r)[N]) {
#pragma unroll
  for (int i = 0; i < N; i++) asm volatile("" : "+r"(r[i]));
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// mbarrier arrives once every tcgen05.mma previously issued by this thread has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// CTA-pair form (the two CTAs of a cluster of two issue one MMA over both SMs): the arrival is delivered to the
// barrier at the same shared-memory offset in every CTA of ctaMask.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t ctaMask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"(ctaMask)
               : "memory");
}

// D[tmem] (+)= A * B, 16-bit inputs, fp32 accumulate, one thread issues; A from shared memory (mma_ss_lohi) or from
// tensor memory (mma_ts_lohi).  The 64-bit shared-memory descriptors are passed as (lo, hi) words, so that stepping a
// descriptor through a tile is a single 32-bit add on the lo word (start address field, 16-byte units).
__device__ __forceinline__ void mma_ss_lohi(uint32_t dTmem, uint32_t aLo, uint32_t aHi, uint32_t bLo, uint32_t bHi,
                                            uint32_t iDesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t"
      "}\n" ::"r"(dTmem),
      "r"(aLo), "r"(aHi), "r"(bLo), "r"(bHi), "r"(iDesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_ts_lohi(uint32_t dTmem, uint32_t aTmem, uint32_t bLo, uint32_t bHi, uint32_t iDesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 db;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t"
      "}\n" ::"r"(dTmem),
      "r"(aTmem), "r"(bLo), "r"(bHi), "r"(iDesc), "r"(accumulate)
      : "memory");
}

// CTA-pair forms (M = 256: rows 0-127 are this CTA's, 128-255 the other's; each CTA supplies its 128 rows of A and
// half of B's N columns from the same shared-memory offsets, and receives its 128 rows of D in its own tensor memory).
__device__ __forceinline__ void mma_ss_lohi_pair(uint32_t dTmem, uint32_t aLo, uint32_t aHi, uint32_t bLo, uint32_t bHi,
                                                 uint32_t iDesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n\t"
      "}\n" ::"r"(dTmem),
      "r"(aLo), "r"(aHi), "r"(bLo), "r"(bHi), "r"(iDesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_ts_lohi_pair(uint32_t dTmem, uint32_t aTmem, uint32_t bLo, uint32_t bHi, uint32_t iDesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 db;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], db, %4, p;\n\t"
      "}\n" ::"r"(dTmem),
      "r"(aTmem), "r"(bLo), "r"(bHi), "r"(iDesc), "r"(accumulate)
      : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives TMEM lane (base lane + i).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// ---------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor for tcgen05.mma, 128-byte swizzle (layout code 2 in bits 61-63,
// descriptor version 1 in bits 46-47).  lbo / sbo are byte offsets (multiples of 16).
__host__ __device__ __forceinline__ constexpr uint64_t smem_desc_sw128(uint32_t lboBytes, uint32_t sboBytes) {
  return (static_cast<uint64_t>((lboBytes >> 4) & 0x3FFF) << 16) |
         (static_cast<uint64_t>((sboBytes >> 4) & 0x3FFF) << 32) | (static_cast<uint64_t>(1) << 46) |
         (static_cast<uint64_t>(2) << 61);
}
// Instruction descriptor for kind::f16, fp32 accumulate.  fmt: 0 = fp16, 1 = bf16.
__host__ __device__ __forceinline__ constexpr uint32_t instr_desc_f16(int fmt, int M, int N, int aMajorMN,
                                                                      int bMajorMN) {
  return (1u << 4) | (static_cast<uint32_t>(fmt) << 7) | (static_cast<uint32_t>(fmt) << 10) |
         (static_cast<uint32_t>(aMajorMN) << 15) | (static_cast<uint32_t>(bMajorMN) << 16) |
         (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

}  // namespace ptx
}  // namespace tfa_b200
