// Shared device helpers for the sm_100a kernels: PTX wrappers for mbarrier, TMA (bulk tensor
// copies, never with cluster multicast), tcgen05 (TMEM allocation, UMMA issue, commit, TMEM loads),
// shared-memory matrix descriptors, the 128-byte swizzle, and bounded waits.
//
// Every wait in this code base is bounded: a spin gives up after SSM_WAIT_NS nanoseconds, records a
// status word in global memory, and the kernel unwinds (frees TMEM, returns).  The host reads the
// status after synchronising and raises.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cuda.h>
#include <stdint.h>

#define SSM_OK 0
#define SSM_ERR_TIMEOUT_MBAR 1      // an mbarrier phase never completed
#define SSM_ERR_TIMEOUT_FLAG 2      // a global-memory flag (peer or local) never arrived
#define SSM_ERR_BAD_ARG 3
#define SSM_ERR_BOUNDS 4            // debug build only: an index check failed (the access was skipped)


namespace ssm {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One poll of an mbarrier phase.  The form WITH a suspend-time hint matters: the thread sleeps in hardware until the
// phase completes (or the hint runs out) and is woken by the completion itself.  Without the hint, the same loop cost the
// GEMM main loop 8-10 % (2048 x 18560 x 4096: 214 us -> 194 us with it), and a software spin before it another 15 %.
#ifndef SSM_MBAR_HINT_NS
#define SSM_MBAR_HINT_NS 1000
#endif
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"((uint32_t)SSM_MBAR_HINT_NS) : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t) :: "memory");      // not to be moved across barriers
  return t;
}
// Bounded wait: gives up after SSM_WAIT_NS nanoseconds (or when another thread already recorded an
// error), stores `code` in *status and returns false.
#ifndef SSM_WAIT_NS
#define SSM_WAIT_NS 2000000000ull
#endif
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code = SSM_ERR_TIMEOUT_MBAR) {
  const uint64_t t0 = global_timer_ns();
  for (uint32_t i = 1;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 0u) {
      if (status != nullptr && *((volatile int*)status) != 0) return false;
      if (global_timer_ns() - t0 > SSM_WAIT_NS) break;
    }
  }
  if (status != nullptr) atomicCAS(status, 0, code);
  return false;
}

// ---------------------------------------------------------------- thread-block clusters (CTA pairs)
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Full barrier over all threads of all CTAs of the cluster, with release/acquire ordering of shared memory.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// In a cluster of two CTAs the shared-memory windows of the pair differ in bit 24 of the shared::cluster address:
// clearing it turns the address of an object of this CTA into the address of the same object of the even CTA.
constexpr uint32_t PAIR_LEADER_MASK = 0xFEFFFFFFu;
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// ---------------------------------------------------------------- fences
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() {
  asm volatile("fence.proxy.async;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------- TMA (no multicast anywhere)
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2D tile load global -> shared, completion signalled on `bar` (complete_tx bytes).
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
// Same for one CTA of a cta_group::2 pair: `bar_cluster_addr` may name the mbarrier of either CTA of the pair (the
// loads of both CTAs complete on the leader's barrier).  No multicast: each CTA fetches its own half of the tile.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, int x, int y,
                                                 uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
// Prefetch of a 2D tile into L2 only (no shared-memory destination, no completion to wait for).
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* m, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// 2D tile store shared -> global (bulk group completion).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---------------------------------------------------------------- tcgen05 / TMEM
// Allocate `cols` TMEM columns (power of two >= 32); the base address is written to *smem_out.
// Must be executed by one full warp.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_out, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_out)), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]; issued by ONE thread.
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on `bar` when all MMAs issued so far by this thread have completed (implies
// tcgen05.fence::before_thread_sync).  Issued by ONE thread.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// ---- cta_group::2: one accumulator tile of 256 rows spread over the TMEM of a CTA pair (128 rows each); A rows and
// B rows are split between the two CTAs' shared memory; the even CTA of the pair issues the MMAs.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_out, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_out)), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the mbarrier at the same shared-memory offset in both CTAs of the pair once all MMAs issued so far have
// completed (a signal to two barriers, not a data copy).
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}
// Load 32 consecutive fp32 columns of this warp's 32 TMEM lanes: thread t gets lane (base_lane + t).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// TMEM address: bits [31:16] lane, [15:0] column.
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, uint32_t lane, uint32_t col) {
  return base + (lane << 16) + col;
}

// ---------------------------------------------------------------- UMMA descriptors
// Instruction descriptor for kind::f16 with bf16 A/B and fp32 accumulate.
//   bits [4,6) D format (1 = f32), [7,10) A format (1 = bf16), [10,13) B format (1 = bf16),
//   bit 15 A major (0 = K-major, 1 = MN-major), bit 16 B major, [17,23) N>>3, [24,29) M>>4.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int M, int N, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) |
         ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// Shared-memory matrix descriptor, 128-byte swizzle.  The tile is made of "atoms" of 8 rows x 128 bytes
// (1024 B, base 1024-B aligned); `sbo_bytes` is the distance between consecutive 8-row groups and
// `lbo_bytes` the distance between consecutive 128-byte column blocks (used by MN-major operands; K-major
// swizzled operands ignore it).
//   bits [0,14) start >> 4, [16,30) LBO >> 4, [32,46) SBO >> 4, [46,48) version = 1, [61,64) layout = 2 (SW128).
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Byte offset of 16-byte chunk `chunk` (0..7) of row `row` inside a [rows][128 B] tile stored with the
// 128-byte swizzle (what TMA SWIZZLE_128B writes and what the SW128 descriptors expect).  The tile base
// must be 1024-byte aligned.
__device__ __forceinline__ uint32_t sw128_offset(uint32_t row, uint32_t chunk) {
  return row * 128u + ((chunk ^ (row & 7u)) << 4);
}

// ---------------------------------------------------------------- misc
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + __expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.0f ? x : log1pf(__expf(x)); }

}  // namespace ssm

// ---------------------------------------------------------------- debug build: index checks
// Compiled with -DSSM_DEBUG_BOUNDS (a second library next to the regular one, ops/native.py build(debug=True)),
// SSM_INDEX_OK(index, limit) checks 0 <= index < limit on the device.  A failed check records
// {SSM_ERR_BOUNDS, source line, index, limit} once in a per-file device array and evaluates to false, and the
// kernel skips that access: no trap, no fault, the context stays usable and the host reads the record through the
// file's ssm_debug_bounds_* function.  In the regular build the macro is the constant `true` and costs nothing.
#ifdef SSM_DEBUG_BOUNDS
namespace ssm {
static __device__ int g_debug_bounds[4];
__device__ __forceinline__ bool debug_index_ok(long long idx, long long limit, int line) {
  if (idx >= 0 && idx < limit) return true;
  if (atomicCAS(&g_debug_bounds[0], 0, SSM_ERR_BOUNDS) == 0) {
    g_debug_bounds[1] = line;
    g_debug_bounds[2] = (int)idx;
    g_debug_bounds[3] = (int)limit;
  }
  return false;
}
}  // namespace ssm
#define SSM_INDEX_OK(idx, limit) ssm::debug_index_ok((long long)(idx), (long long)(limit), __LINE__)
#define SSM_DEBUG_BOUNDS_GETTER(name)                                                          \
  extern "C" int name(int* out4, int reset) {                                                  \
    cudaError_t e = cudaMemcpyFromSymbol(out4, ssm::g_debug_bounds, 4 * sizeof(int));          \
    if (e == cudaSuccess && reset) {                                                           \
      const int z[4] = {0, 0, 0, 0};                                                           \
      e = cudaMemcpyToSymbol(ssm::g_debug_bounds, z, sizeof(z));                               \
    }                                                                                          \
    return (int)e;                                                                             \
  }
#else
#define SSM_INDEX_OK(idx, limit) true
#define SSM_DEBUG_BOUNDS_GETTER(name)                                                          \
  extern "C" int name(int* out4, int reset) {                                                  \
    out4[0] = out4[1] = out4[2] = out4[3] = 0;                                                 \
    (void)reset;                                                                               \
    return 0;                                                                                  \
  }
#endif

// ---------------------------------------------------------------- host side
#include <cudaTypedefs.h>
#include <stdio.h>
namespace ssm {
// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda).
// The driver call needs the primary context current on the calling thread; threads that have only been
// handed work by another runtime (autograd worker threads) may not have it yet.
inline void bind_primary_context() {
  static thread_local bool bound = false;
  if (!bound) { cudaFree(0); bound = true; }
}
inline PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
  bind_primary_context();
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }
  return fn;
}
// 2D bf16 tensor map: `inner` contiguous elements, `outer` rows of `row_stride_bytes`; box {box_inner, box_outer}
// with 128-byte swizzle (box_inner * 2 bytes must be 128).  Returns 0 on success.
inline int make_tmap_2d(CUtensorMap* map, CUtensorMapDataType dtype, int elem_bytes, const void* base, uint64_t inner,
                        uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer,
                        CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  auto enc = tensor_map_encoder();
  if (enc == nullptr) return -1;
  (void)elem_bytes;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, dtype, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}
inline int make_tmap_2d_bf16(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer,
                             uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer,
                             CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  return make_tmap_2d(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, inner, outer, row_stride_bytes, box_inner,
                      box_outer, swizzle);
}
}  // namespace ssm
