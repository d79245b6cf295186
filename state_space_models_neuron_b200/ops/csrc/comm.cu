// Peer-memory building blocks for the tensor-parallel collectives over NVLink / NVSwitch (sm_100a).
// All ranks of a TP group hold a symmetric workspace; kernels receive the peers' base pointers and use plain
// P2P loads/stores plus release/acquire flags at system scope.  Nothing here uses TMA multicast or NVLS.
//
//   push (all-gather building block)   copy a local [rows, cols] bf16 shard into every rank's gather buffer at
//                                      this rank's row offset, then publish flag[src = me] = seq on every rank
//                                      (the all-gather and reduce-scatter of the linear layers live inside the GEMM
//                                      kernel, gemm.cu; this stand-alone push serves the embedding backward)
//   small all-reduce                   packed fp32 vector (cross-entropy statistics, norm-weight grads):
//                                      every rank writes its vector into every rank's slot, waits, sums
//   ZeRO-1                             peer reduce of the owned gradient shard fused with scaling and the norm
//                                      partial; AdamW on the shard fused with the push of the new bf16 parameters
//   one-shot bf16 all-reduce           decode-time sum of a [batch, d_model] activation over the TP group
//   vocabulary-parallel embedding      the rank that holds a token's row stores it into the sequence owner's
//                                      buffer; backward scatter-adds gathered output gradients in fp32
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
// Flags for several ranks: ONE system-scope fence, then relaxed system-scope stores that go out back to back.  A loop of
// release stores instead pays one NVLink round trip per destination, in series (measured in the all-gather GEMM at 4
// ranks: the CTA that published a flag set was 35 us late, and every later flag set waited for it).
__device__ __forceinline__ void st_relaxed_sys(int* p, int v) {
  asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Sequence numbers wrap around: "flag has reached seq" is a signed distance, valid while the two are less than 2^31
// apart (advance_counter_kernel keeps idle flags within that distance).
__device__ __forceinline__ bool seq_reached(int flag, int seq) {
  return (int)((unsigned)flag - (unsigned)seq) >= 0;
}
__device__ __forceinline__ int seq_add(int off, const int* base) {
  return (int)((unsigned)off + (base != nullptr ? (unsigned)*base : 0u));
}
// Bounded wait until *flag has reached seq.
__device__ __forceinline__ bool wait_flag_ge(const int* flag, int seq, int* status) {
  if (seq_reached(ld_acquire_sys(flag), seq)) return true;
  const uint64_t t0 = global_timer_ns();
  for (uint32_t i = 1;; ++i) {
    if (seq_reached(ld_acquire_sys(flag), seq)) return true;
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
  const int seq = seq_add(seq_off, seq_base);
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
      for (int t = 0; t < nranks; ++t) st_relaxed_sys(reinterpret_cast<int*>(flags.p[t]) + flag_base + me, seq);
      *counter = 0;
    }
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
  const int seq = seq_add(seq_off, seq_base);
  __shared__ int s_ok;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = data[i];
    for (int t = 0; t < nranks; ++t) reinterpret_cast<float*>(slots.p[t])[(long long)me * n_max + i] = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    s_ok = 1;
    __threadfence_system();                   // orders the whole block's (already fenced) stores before the flags
    for (int t = 0; t < nranks; ++t) st_relaxed_sys(reinterpret_cast<int*>(flags.p[t]) + flag_base + me, seq);
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

// *base += stride (modulo 2^32); launched once per training step so that sequence numbers grow across replays of a
// captured CUDA graph although every kernel node keeps its fixed offset.  The waits compare by signed distance,
// which is only meaningful within 2^31: whenever the base crosses a multiple of 2^29, every local flag that has
// fallen more than 2^29 behind (a collective kind that has not run for a long time) is pulled up to the new base,
// which no wait of the new block can mistake for "arrived" (their sequence numbers are base + position, position
// >= 1).  A flag that a peer stores to at the same moment keeps the peer's (newer) value: the update is a
// compare-and-swap against the stale value.
__global__ void advance_counter_kernel(int* base, int stride, int* flags, int nflags) {
  __shared__ unsigned s_old, s_new;
  if (threadIdx.x == 0) {
    s_old = (unsigned)*base;
    s_new = s_old + (unsigned)stride;
    *base = (int)s_new;
  }
  __syncthreads();
  if (flags == nullptr || (s_old >> 29) == (s_new >> 29)) return;
  for (int i = threadIdx.x; i < nflags; i += blockDim.x) {
    const int f = *((volatile int*)(flags + i));
    if ((int)(s_new - (unsigned)f) > (1 << 29)) atomicCAS(flags + i, f, (int)s_new);
  }
}

}  // namespace ssm

using namespace ssm;

static PeerPtrs to_peers(const void* const* ptrs, int n) {
  PeerPtrs p;
  for (int i = 0; i < MAX_RANKS; ++i) p.p[i] = i < n ? const_cast<void*>(ptrs[i]) : nullptr;
  return p;
}

extern "C" int ssm_comm_max_ranks() { return MAX_RANKS; }
SSM_DEBUG_BOUNDS_GETTER(ssm_debug_bounds_comm)

extern "C" int ssm_push_shard(const void* src, long long src_ld, const void* const* dst_ptrs, long long dst_ld,
                              long long row_off, int rows, int cols, int nranks, int me, const void* const* flag_ptrs,
                              int flag_base, int seq, const int* seq_base, int* counter, int blocks, cudaStream_t st) {
  if (cols % 8 || src_ld % 8 || dst_ld % 8 || nranks > MAX_RANKS || nranks < 1) return -SSM_ERR_BAD_ARG;
  push_shard_kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(src), src_ld,
                                            to_peers(dst_ptrs, nranks), dst_ld, row_off, rows, cols, nranks, me,
                                            to_peers(flag_ptrs, nranks), flag_base, seq, seq_base, counter);
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

// flags / nflags: this rank's flag array that belongs to the counter (may be null: no refresh of idle flags)
extern "C" int ssm_advance_counter(int* base, int stride, int* flags, int nflags, cudaStream_t st) {
  advance_counter_kernel<<<1, 128, 0, st>>>(base, stride, flags, nflags);
  return (int)cudaGetLastError();
}

// =====================================================================================================
// ZeRO-1 over peer memory: gradient reduce-scatter fused with scaling and the squared-norm partial, and the
// sharded AdamW update fused with the all-gather of the updated low-precision parameters.
// Every data-parallel rank keeps its flat fp32 gradient buffer and its flat bf16 parameter buffer in symmetric
// memory.  Rank r owns elements [r*S, (r+1)*S).
//   zero1_reduce   : publish "my gradients are final", wait for all ranks (bounded), then for the owned shard
//                    g = (1/dp) * sum over ranks of their gradient (P2P loads), store g locally, add sum(g^2)
//   zero1_adamw_push: AdamW on the owned fp32 master shard with the clip coefficient, store the new bf16 values
//                    into every rank's parameter buffer (P2P stores), then publish "my shard has landed"
//   zero1_wait     : wait until every rank's shard has landed (bounded) before later kernels read parameters
// These replace reduce_scatter + scale + norm + AdamW + all_gather of the NxD ZeRO-1 wrapper the reference
// enables with zero_one_enabled (train.py:73,129-138).
// =====================================================================================================
namespace ssm {

__global__ void __launch_bounds__(256)
zero1_reduce_kernel(PeerPtrs grads, float* __restrict__ shard_out, long long shard_start, long long n4, int nranks,
                    int me, float scale, float* __restrict__ sumsq, PeerPtrs flags, int flag_base, int seq_off,
                    const int* seq_base, int* status) {
  const int seq = seq_add(seq_off, seq_base);
  __shared__ int s_ok;
  __shared__ float red[8];
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x < nranks)      // this rank's backward is complete (stream order)
    st_release_sys(reinterpret_cast<int*>(flags.p[threadIdx.x]) + flag_base + me, seq);
  if (threadIdx.x < nranks) {
    if (!wait_flag_ge(reinterpret_cast<const int*>(flags.p[me]) + flag_base + threadIdx.x, seq, status)) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) return;
  float local = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    #pragma unroll
    for (int k = 0; k < MAX_RANKS; ++k) {
      const int r = (me + k) % MAX_RANKS;
      if (r < nranks) {
        const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[r]) + shard_start + i * 4);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
    }
    acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    *reinterpret_cast<float4*>(shard_out + i * 4) = acc;
    local += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  #pragma unroll
  for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x == 0 && sumsq != nullptr) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[w];
    atomicAdd(sumsq, t);
  }
}

__global__ void __launch_bounds__(256)
zero1_adamw_push_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                        const float* __restrict__ g, PeerPtrs params, long long param_off, long long n4, int nranks,
                        int me, const float* __restrict__ clip, float lr, float b1, float b2, float eps, float wd,
                        const float* __restrict__ lr_dev, const int* __restrict__ step_dev, int step, PeerPtrs flags,
                        int flag_base, int seq_off, const int* seq_base, int* counter, int publish) {
  const int seq = seq_add(seq_off, seq_base);
  const float c = clip ? *clip : 1.f;
  if (lr_dev != nullptr) lr = *lr_dev;
  const float st = step_dev != nullptr ? (float)(*step_dev) : (float)step;
  const float ib1 = 1.f / (1.f - powf(b1, st)), ib2 = 1.f / (1.f - powf(b2, st));
  const float decay = 1.f - lr * wd;
  // a negative or NaN clip coefficient means "skip this step" (non-finite gradients): nothing is updated or pushed,
  // the parameters every rank holds stay valid, and the completion flag is still published
  const long long n_eff = (c >= 0.f) ? n4 : 0;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_eff; i += (long long)gridDim.x * blockDim.x) {
    const float4 gi = *reinterpret_cast<const float4*>(g + i * 4);
    float4 mi = *reinterpret_cast<const float4*>(m + i * 4);
    float4 vi = *reinterpret_cast<const float4*>(v + i * 4);
    float4 wv = *reinterpret_cast<const float4*>(master + i * 4);
    #define SSM_ADAM(f)                                             \
      { const float gg = gi.f * c;                                  \
        mi.f = b1 * mi.f + (1.f - b1) * gg;                         \
        vi.f = b2 * vi.f + (1.f - b2) * gg * gg;                    \
        wv.f = wv.f * decay - lr * (mi.f * ib1) / (sqrtf(vi.f * ib2) + eps); }
    SSM_ADAM(x) SSM_ADAM(y) SSM_ADAM(z) SSM_ADAM(w)
    #undef SSM_ADAM
    *reinterpret_cast<float4*>(m + i * 4) = mi;
    *reinterpret_cast<float4*>(v + i * 4) = vi;
    *reinterpret_cast<float4*>(master + i * 4) = wv;
    uint2 o;
    o.x = pack_bf16(wv.x, wv.y); o.y = pack_bf16(wv.z, wv.w);
    #pragma unroll
    for (int k = 0; k < MAX_RANKS; ++k) {
      const int r = (me + k) % MAX_RANKS;
      if (r < nranks) *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(params.p[r]) + param_off + i * 4) = o;
    }
  }
  if (!publish) return;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(counter, 1) + 1;
    if (done == (int)gridDim.x) {
      __threadfence_system();
      for (int t = 0; t < nranks; ++t) st_relaxed_sys(reinterpret_cast<int*>(flags.p[t]) + flag_base + me, seq);
      *counter = 0;
    }
  }
}

__global__ void zero1_wait_kernel(const int* flags, int flag_base, int nranks, int seq_off, const int* seq_base,
                                  int* status) {
  const int seq = seq_add(seq_off, seq_base);
  if ((int)threadIdx.x < nranks) wait_flag_ge(flags + flag_base + threadIdx.x, seq, status);
}

}  // namespace ssm

extern "C" int ssm_zero1_reduce(const void* const* grad_ptrs, void* shard_out, long long shard_start, long long n,
                                int nranks, int me, float scale, void* sumsq, const void* const* flag_ptrs,
                                int flag_base, int seq, const int* seq_base, int* status, cudaStream_t st) {
  if (n % 4 || shard_start % 4 || nranks > MAX_RANKS) return -SSM_ERR_BAD_ARG;
  const long long n4 = n / 4;
  const int blocks = (int)((n4 + 255) / 256 < 148 * 8 ? (n4 + 255) / 256 : 148 * 8);
  zero1_reduce_kernel<<<blocks, 256, 0, st>>>(to_peers(grad_ptrs, nranks), reinterpret_cast<float*>(shard_out),
                                              shard_start, n4, nranks, me, scale, reinterpret_cast<float*>(sumsq),
                                              to_peers(flag_ptrs, nranks), flag_base, seq, seq_base, status);
  return (int)cudaGetLastError();
}

extern "C" int ssm_zero1_adamw_push(void* master, void* m, void* v, const void* g, const void* const* param_ptrs,
                                    long long param_off, long long n, int nranks, int me, const void* clip, float lr,
                                    float b1, float b2, float eps, float wd, const void* lr_dev, const void* step_dev,
                                    int step, const void* const* flag_ptrs, int flag_base, int seq, const int* seq_base,
                                    int* counter, int publish, cudaStream_t st) {
  if (n % 4 || param_off % 4 || nranks > MAX_RANKS) return -SSM_ERR_BAD_ARG;
  const long long n4 = n / 4;
  const int blocks = (int)((n4 + 255) / 256 < 148 * 8 ? (n4 + 255) / 256 : 148 * 8);
  zero1_adamw_push_kernel<<<blocks, 256, 0, st>>>(
      reinterpret_cast<float*>(master), reinterpret_cast<float*>(m), reinterpret_cast<float*>(v),
      reinterpret_cast<const float*>(g), to_peers(param_ptrs, nranks), param_off, n4, nranks, me,
      reinterpret_cast<const float*>(clip), lr, b1, b2, eps, wd, reinterpret_cast<const float*>(lr_dev),
      reinterpret_cast<const int*>(step_dev), step, to_peers(flag_ptrs, nranks), flag_base, seq, seq_base, counter,
      publish);
  return (int)cudaGetLastError();
}

extern "C" int ssm_zero1_wait(const void* flags, int flag_base, int nranks, int seq, const int* seq_base, int* status,
                              cudaStream_t st) {
  zero1_wait_kernel<<<1, 32, 0, st>>>(reinterpret_cast<const int*>(flags), flag_base, nranks, seq, seq_base, status);
  return (int)cudaGetLastError();
}

namespace ssm {

// =====================================================================================================
// One-shot all-reduce (sum) of a bf16 activation over the TP group, for the latency-bound decode path
// (row-parallel out_proj of one token per sequence: [batch, d_model] per layer).  Every rank stores its vector
// into slot[me] of every rank, the last CTA publishes the flag, all CTAs wait (bounded) for the T sources and sum
// the T slots in fp32.  The grid must be co-resident (<= number of SMs): CTAs wait for peers, not for each other.
// =====================================================================================================
__global__ void __launch_bounds__(256)
oneshot_allreduce_bf16_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, long long nvec,
                              PeerPtrs slots, long long slot_stride, int nranks, int me, PeerPtrs flags,
                              int flag_base, int seq_off, const int* seq_base, int* counter, int* status) {
  const int seq = seq_add(seq_off, seq_base);
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += step) {
    const uint4 v = reinterpret_cast<const uint4*>(in)[i];
    #pragma unroll
    for (int k = 0; k < MAX_RANKS; ++k) {
      const int t = (me + k) % MAX_RANKS;
      if (t < nranks) reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(slots.p[t]) + me * slot_stride)[i] = v;
    }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    s_ok = 1;
    const int done = atomicAdd(counter, 1) + 1;
    if (done == (int)gridDim.x) {
      __threadfence_system();
      for (int t = 0; t < nranks; ++t) st_relaxed_sys(reinterpret_cast<int*>(flags.p[t]) + flag_base + me, seq);
      *counter = 0;
    }
  }
  __syncthreads();
  if (threadIdx.x < nranks) {
    if (!wait_flag_ge(reinterpret_cast<const int*>(flags.p[me]) + flag_base + threadIdx.x, seq, status)) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) return;
  const __nv_bfloat16* mine = reinterpret_cast<const __nv_bfloat16*>(slots.p[me]);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += step) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < nranks; ++s) {
      const uint4 u = reinterpret_cast<const uint4*>(mine + s * slot_stride)[i];
      acc[0] += bf16_lo(u.x); acc[1] += bf16_hi(u.x); acc[2] += bf16_lo(u.y); acc[3] += bf16_hi(u.y);
      acc[4] += bf16_lo(u.z); acc[5] += bf16_hi(u.z); acc[6] += bf16_lo(u.w); acc[7] += bf16_hi(u.w);
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

// =====================================================================================================
// Vocabulary-parallel embedding over peer memory.
// The reference sums T masked partial lookups with an all-reduce and then keeps one sequence slice
// (mamba2/modeling_mamba2.py:276,300-301).  Every token's row lives on exactly one rank, so nothing has to be
// summed: the rank that holds row ids[t] stores it straight into the output buffer of the rank that owns token
// t's sequence slice, and a flag per source says "all my rows have landed".
//   embed_lookup    : local masked lookup (ids outside [vocab_start, vocab_start + vloc) give zero rows)
//   vocab_embed_push: for token (b, l) with a local id: dst[l / Ls][(b * Ls + l % Ls), :] = weight[id - vocab_start]
//   embed_wait_copy : wait (bounded) for all sources, copy the landing buffer to the output tensor
//   embed_bwd       : grad32[id - vocab_start, :] += g[row(t), :] for the local ids; g is either the local
//                     gradient (one rank) or the gather buffer that the push kernel above filled (waits first)
// =====================================================================================================
__global__ void __launch_bounds__(256)
embed_lookup_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ weight, long long vocab_start,
                    long long vloc, __nv_bfloat16* __restrict__ out, long long ntok, int D) {
  const int vec = D / 8;
  for (long long t = blockIdx.x; t < ntok; t += gridDim.x) {
    const long long id = ids[t] - vocab_start;
    const bool in = id >= 0 && id < vloc;
    for (int c = threadIdx.x; c < vec; c += blockDim.x) {
      const uint4 v = in ? *reinterpret_cast<const uint4*>(weight + id * D + c * 8) : make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4*>(out + t * D + c * 8) = v;
    }
  }
}

__global__ void __launch_bounds__(256)
vocab_embed_push_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ weight,
                        long long vocab_start, long long vloc, PeerPtrs dst, int B, int L, int Ls, int D, int nranks,
                        int me, PeerPtrs flags, int flag_base, int seq_off, const int* seq_base, int* counter) {
  const int seq = seq_add(seq_off, seq_base);
  const int vec = D / 8;
  const long long ntok = (long long)B * L;
  for (long long t = blockIdx.x; t < ntok; t += gridDim.x) {
    const long long id = ids[t] - vocab_start;
    if (id < 0 || id >= vloc) continue;
    const int b = (int)(t / L), l = (int)(t % L);
    const int owner = l / Ls;
    if (!SSM_INDEX_OK(owner, nranks)) continue;
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(dst.p[owner]) + ((long long)b * Ls + (l % Ls)) * D;
    for (int c = threadIdx.x; c < vec; c += blockDim.x)
      *reinterpret_cast<uint4*>(o + c * 8) = *reinterpret_cast<const uint4*>(weight + id * D + c * 8);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(counter, 1) + 1;
    if (done == (int)gridDim.x) {
      __threadfence_system();
      for (int t = 0; t < nranks; ++t) st_relaxed_sys(reinterpret_cast<int*>(flags.p[t]) + flag_base + me, seq);
      *counter = 0;
    }
  }
}

__global__ void __launch_bounds__(256)
embed_wait_copy_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ out, long long nvec,
                       int nranks, const int* flags, int flag_base, int seq_off, const int* seq_base, int* status) {
  const int seq = seq_add(seq_off, seq_base);
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < nranks) {
    if (!wait_flag_ge(flags + flag_base + threadIdx.x, seq, status)) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) return;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x)
    reinterpret_cast<uint4*>(out)[i] = reinterpret_cast<const uint4*>(src)[i];
}

__global__ void __launch_bounds__(256)
embed_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ g, long long g_ld,
                 float* __restrict__ grad32, long long vocab_start, long long vloc, int B, int L, int Ls, int D,
                 int nranks, const int* flags, int flag_base, int seq_off, const int* seq_base, int* status) {
  if (nranks > 1) {
    const int seq = seq_add(seq_off, seq_base);
    __shared__ int s_ok;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (threadIdx.x < nranks) {
      if (!wait_flag_ge(flags + flag_base + threadIdx.x, seq, status)) s_ok = 0;
    }
    __syncthreads();
    if (!s_ok) return;
  }
  const int vec = D / 4;
  const long long ntok = (long long)B * L;
  for (long long t = blockIdx.x; t < ntok; t += gridDim.x) {
    const long long id = ids[t] - vocab_start;
    if (id < 0 || id >= vloc) continue;
    const int b = (int)(t / L), l = (int)(t % L);
    // row of token (b, l) in g: [B, L] order on one rank, [owner][b][l % Ls] in the gather buffer
    const long long r = nranks > 1 ? ((long long)(l / Ls) * B + b) * Ls + (l % Ls) : t;
    if (!SSM_INDEX_OK(r, ntok) || !SSM_INDEX_OK(D - 1, g_ld)) continue;
    const __nv_bfloat16* src = g + r * g_ld;
    float* dstp = grad32 + id * D;
    for (int c = threadIdx.x; c < vec; c += blockDim.x) {
      const uint2 u = *reinterpret_cast<const uint2*>(src + c * 4);
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dstp + c * 4), "f"(bf16_lo(u.x)),
                   "f"(bf16_hi(u.x)), "f"(bf16_lo(u.y)), "f"(bf16_hi(u.y)) : "memory");
    }
  }
}

}  // namespace ssm
using namespace ssm;

extern "C" int ssm_embed_lookup(const void* ids, const void* weight, long long vocab_start, long long vloc, void* out,
                                long long ntok, int D, cudaStream_t st) {
  if (D % 8 || ntok < 1) return -SSM_ERR_BAD_ARG;
  const int blocks = (int)(ntok < 148 * 8 ? ntok : 148 * 8);
  embed_lookup_kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<const long long*>(ids),
                                              reinterpret_cast<const __nv_bfloat16*>(weight), vocab_start, vloc,
                                              reinterpret_cast<__nv_bfloat16*>(out), ntok, D);
  return (int)cudaGetLastError();
}

extern "C" int ssm_vocab_embed_push(const void* ids, const void* weight, long long vocab_start, long long vloc,
                                    const void* const* dst_ptrs, int B, int L, int Ls, int D, int nranks, int me,
                                    const void* const* flag_ptrs, int flag_base, int seq, const int* seq_base,
                                    int* counter, cudaStream_t st) {
  if (D % 8 || nranks > MAX_RANKS || nranks < 1 || Ls < 1 || L != Ls * nranks) return -SSM_ERR_BAD_ARG;
  const long long ntok = (long long)B * L;
  const int blocks = (int)(ntok < 148 * 4 ? ntok : 148 * 4);
  vocab_embed_push_kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<const long long*>(ids),
                                                  reinterpret_cast<const __nv_bfloat16*>(weight), vocab_start, vloc,
                                                  to_peers(dst_ptrs, nranks), B, L, Ls, D, nranks, me,
                                                  to_peers(flag_ptrs, nranks), flag_base, seq, seq_base, counter);
  return (int)cudaGetLastError();
}

extern "C" int ssm_embed_wait_copy(const void* src, void* out, long long nelem, int nranks, const void* flags,
                                   int flag_base, int seq, const int* seq_base, int* status, cudaStream_t st) {
  if (nelem % 8 || nranks > MAX_RANKS) return -SSM_ERR_BAD_ARG;
  const long long nvec = nelem / 8;
  const int blocks = (int)((nvec + 255) / 256 < 148 * 4 ? (nvec + 255) / 256 : 148 * 4);
  embed_wait_copy_kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(src),
                                                 reinterpret_cast<__nv_bfloat16*>(out), nvec, nranks,
                                                 reinterpret_cast<const int*>(flags), flag_base, seq, seq_base, status);
  return (int)cudaGetLastError();
}

extern "C" int ssm_embed_bwd(const void* ids, const void* g, long long g_ld, void* grad32, long long vocab_start,
                             long long vloc, int B, int L, int Ls, int D, int nranks, const void* flags, int flag_base,
                             int seq, const int* seq_base, int* status, cudaStream_t st) {
  if (D % 4 || g_ld % 4 || nranks > MAX_RANKS || nranks < 1) return -SSM_ERR_BAD_ARG;
  const long long ntok = (long long)B * L;
  const int blocks = (int)(ntok < 148 * 8 ? ntok : 148 * 8);
  embed_bwd_kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<const long long*>(ids),
                                           reinterpret_cast<const __nv_bfloat16*>(g), g_ld,
                                           reinterpret_cast<float*>(grad32), vocab_start, vloc, B, L, Ls, D, nranks,
                                           reinterpret_cast<const int*>(flags), flag_base, seq, seq_base, status);
  return (int)cudaGetLastError();
}

extern "C" int ssm_allreduce_bf16(const void* in, void* out, long long n, const void* const* slot_ptrs,
                                  long long slot_stride, int nranks, int me, const void* const* flag_ptrs,
                                  int flag_base, int seq, const int* seq_base, int* counter, int* status,
                                  cudaStream_t st) {
  if (n % 8 || slot_stride % 8 || n > slot_stride || nranks > MAX_RANKS || nranks < 1) return -SSM_ERR_BAD_ARG;
  const long long nvec = n / 8;
  long long blocks = (nvec + 255) / 256;
  if (blocks > 64) blocks = 64;            // co-resident by a wide margin; 64 x 256 x 16 B per pass
  oneshot_allreduce_bf16_kernel<<<(int)blocks, 256, 0, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(in), reinterpret_cast<__nv_bfloat16*>(out), nvec,
      to_peers(slot_ptrs, nranks), slot_stride, nranks, me, to_peers(flag_ptrs, nranks), flag_base, seq, seq_base,
      counter, status);
  return (int)cudaGetLastError();
}
