// Peer-memory building blocks for the tensor-parallel collectives over NVLink / NVSwitch (sm_100a).
// All ranks of a TP group hold a symmetric workspace; kernels receive the peers' base pointers and use plain
// P2P loads/stores plus release/acquire flags at system scope.  Nothing here uses TMA multicast or NVLS.
//
//   push (all-gather building block)   copy a local [rows, cols] bf16 shard into every rank's gather buffer at
//                                      this rank's row offset, then publish flag[src = me] = seq on every rank
//   reduce (reduce-scatter consumer)   wait until all T sources have published, then sum the T partial tiles
//                                      that landed in this rank's landing zone (fp32 accumulate) -> bf16
//   small all-reduce                   packed fp32 vector (cross-entropy statistics, norm-weight grads):
//                                      every rank writes its vector into every rank's slot, waits, sums
// Flag waits are bounded (SSM_WAIT_NS); on time-out the status word is set and the kernel returns.
// The collectives the reference triggers implicitly through neuronx-distributed are listed with their call
// sites in mamba2/mamba2_mixer.py:228,233 and mamba2/modeling_mamba2.py:276,300-301,498-510.
#include "common.cuh"

namespace ssm {

constexpr int MAX_RANKS = 8;

struct PeerPtrs {
  void* p[MAX_RANKS];
};

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Bounded wait until *flag >= seq.
__device__ __forceinline__ bool wait_flag_ge(const int* flag, int seq, int* status) {
  if (ld_acquire_sys(flag) >= seq) return true;
  const uint64_t t0 = global_timer_ns();
  for (uint32_t i = 1;; ++i) {
    if (ld_acquire_sys(flag) >= seq) return true;
    if ((i & 63u) == 0u) {
      if (status != nullptr && *((volatile int*)status) != 0) return false;
      if (global_timer_ns() - t0 > SSM_WAIT_NS) break;
    }
  }
  if (status != nullptr) atomicCAS(status, 0, SSM_ERR_TIMEOUT_FLAG);
  return false;
}

// ---------------------------------------------------------------------------------------------------
// push: src [rows, cols] (row stride src_ld) -> dst[t] + (row_off + r) * dst_ld + c   for every rank t
// grid: any; block 256.  counter: local int (zero on entry; reset by the last block).  flags[t] points at rank
// t's flag array; this rank's slot is flags[t][flag_base + me].
// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
push_shard_kernel(const __nv_bfloat16* __restrict__ src, long long src_ld, PeerPtrs dst, long long dst_ld,
                  long long row_off, int rows, int cols, int nranks, int me, PeerPtrs flags, int flag_base, int seq_off,
                  const int* seq_base, int* counter) {
  const int seq = seq_off + (seq_base ? *seq_base : 0);
  const int vec_per_row = cols / 8;
  const long long total = (long long)rows * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = (int)(i % vec_per_row) * 8;
    const uint4 v = *reinterpret_cast<const uint4*>(src + r * src_ld + c);
    #pragma unroll
    for (int k = 0; k < MAX_RANKS; ++k) {
      const int t = (me + k) % MAX_RANKS;     // start with the local copy, then peers in ring order
      if (t < nranks)
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dst.p[t]) + (row_off + r) * dst_ld + c) = v;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(counter, 1) + 1;
    if (done == (int)gridDim.x) {
      __threadfence_system();
      for (int t = 0; t < nranks; ++t) st_release_sys(reinterpret_cast<int*>(flags.p[t]) + flag_base + me, seq);
      *counter = 0;
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// reduce: out[r, c] = sum_s land[s][r][c]  after flags[flag_base + s] >= seq for all s.
// land: local landing zone [nranks][rows][ld] bf16.  grid: any; block 256.
// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
reduce_partials_kernel(const __nv_bfloat16* __restrict__ land, long long ld, long long slot_stride,
                       __nv_bfloat16* __restrict__ out, long long out_ld, int rows, int cols, int nranks,
                       const int* flags, int flag_base, int seq_off, const int* seq_base, int* status) {
  const int seq = seq_off + (seq_base ? *seq_base : 0);
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < nranks) {
    if (!wait_flag_ge(flags + flag_base + threadIdx.x, seq, status)) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) return;
  const int vec_per_row = cols / 8;
  const long long total = (long long)rows * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = (int)(i % vec_per_row) * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < nranks; ++s) {
      const uint4 u = *reinterpret_cast<const uint4*>(land + s * slot_stride + r * ld + c);
      acc[0] += bf16_lo(u.x); acc[1] += bf16_hi(u.x); acc[2] += bf16_lo(u.y); acc[3] += bf16_hi(u.y);
      acc[4] += bf16_lo(u.z); acc[5] += bf16_hi(u.z); acc[6] += bf16_lo(u.w); acc[7] += bf16_hi(u.w);
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + r * out_ld + c) = o;
  }
}

// ---------------------------------------------------------------------------------------------------
// small all-reduce (sum or max) of n fp32 values, n <= a few thousand.  Every rank writes its vector into
// slot[me] of every rank, publishes, waits for all, reduces.  slots[t] -> rank t's slot array [nranks][n_max].
// One block.  op: 0 sum, 1 max.
// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
small_allreduce_kernel(float* __restrict__ data, int n, int n_max, PeerPtrs slots, PeerPtrs flags, int flag_base,
                       int nranks, int me, int seq_off, const int* seq_base, int op, int* status) {
  const int seq = seq_off + (seq_base ? *seq_base : 0);
  __shared__ int s_ok;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = data[i];
    for (int t = 0; t < nranks; ++t) reinterpret_cast<float*>(slots.p[t])[(long long)me * n_max + i] = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    s_ok = 1;
    for (int t = 0; t < nranks; ++t) st_release_sys(reinterpret_cast<int*>(flags.p[t]) + flag_base + me, seq);
  }
  __syncthreads();
  if (threadIdx.x < nranks) {
    if (!wait_flag_ge(reinterpret_cast<int*>(flags.p[me]) + flag_base + threadIdx.x, seq, status)) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) return;
  const float* mine = reinterpret_cast<const float*>(slots.p[me]);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float acc = mine[i];
    for (int s = 1; s < nranks; ++s) {
      const float v = mine[(long long)s * n_max + i];
      acc = op == 0 ? acc + v : fmaxf(acc, v);
    }
    data[i] = acc;
  }
}

// *base += stride  (one thread); launched once per training step so that sequence numbers grow across replays of
// a captured CUDA graph although every kernel node keeps its fixed offset
__global__ void advance_counter_kernel(int* base, int stride) { *base += stride; }

}  // namespace ssm

using namespace ssm;

static PeerPtrs to_peers(const void* const* ptrs, int n) {
  PeerPtrs p;
  for (int i = 0; i < MAX_RANKS; ++i) p.p[i] = i < n ? const_cast<void*>(ptrs[i]) : nullptr;
  return p;
}

extern "C" int ssm_comm_max_ranks() { return MAX_RANKS; }

extern "C" int ssm_push_shard(const void* src, long long src_ld, const void* const* dst_ptrs, long long dst_ld,
                              long long row_off, int rows, int cols, int nranks, int me, const void* const* flag_ptrs,
                              int flag_base, int seq, const int* seq_base, int* counter, int blocks, cudaStream_t st) {
  if (cols % 8 || src_ld % 8 || dst_ld % 8 || nranks > MAX_RANKS || nranks < 1) return -SSM_ERR_BAD_ARG;
  push_shard_kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(src), src_ld,
                                            to_peers(dst_ptrs, nranks), dst_ld, row_off, rows, cols, nranks, me,
                                            to_peers(flag_ptrs, nranks), flag_base, seq, seq_base, counter);
  return (int)cudaGetLastError();
}

extern "C" int ssm_reduce_partials(const void* land, long long ld, long long slot_stride, void* out, long long out_ld,
                                   int rows, int cols, int nranks, const void* flags, int flag_base, int seq,
                                   const int* seq_base, int* status, int blocks, cudaStream_t st) {
  if (cols % 8 || ld % 8 || out_ld % 8 || slot_stride % 8 || nranks > MAX_RANKS) return -SSM_ERR_BAD_ARG;
  reduce_partials_kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(land), ld, slot_stride,
                                                 reinterpret_cast<__nv_bfloat16*>(out), out_ld, rows, cols, nranks,
                                                 reinterpret_cast<const int*>(flags), flag_base, seq, seq_base, status);
  return (int)cudaGetLastError();
}

extern "C" int ssm_small_allreduce(void* data, int n, int n_max, const void* const* slot_ptrs,
                                   const void* const* flag_ptrs, int flag_base, int nranks, int me, int seq,
                                   const int* seq_base, int op, int* status, cudaStream_t st) {
  if (n > n_max || nranks > MAX_RANKS) return -SSM_ERR_BAD_ARG;
  small_allreduce_kernel<<<1, 256, 0, st>>>(reinterpret_cast<float*>(data), n, n_max, to_peers(slot_ptrs, nranks),
                                            to_peers(flag_ptrs, nranks), flag_base, nranks, me, seq, seq_base, op, status);
  return (int)cudaGetLastError();
}

extern "C" int ssm_advance_counter(int* base, int stride, cudaStream_t st) {
  advance_counter_kernel<<<1, 1, 0, st>>>(base, stride);
  return (int)cudaGetLastError();
}
