// bf16 GEMM for sm_100a: TMA (no multicast) -> 128B-swizzled smem ring -> tcgen05.mma with fp32 accumulators in
// TMEM -> epilogue.  Persistent, warp-specialised, 7 warps:
//     warp 0      TMA producer (one elected thread): the A loads of every stage (all loads in the fused variants)
//     warp 1      MMA issuer (one elected thread), owns the TMEM allocation
//     warps 2..5  epilogue: tcgen05.ld -> bf16 (plain, or +bias / GELU) -> swizzled smem -> TMA store,
//                 or fp32 TMA store / TMA reduce-add for gradient outputs (optionally adding sum(C^2) to a scalar),
//                 or TMA stores into the peers' landing zones (reduce-scatter)
//     warp 6      second TMA producer: the B loads of every stage (plain GEMMs)
// Two accumulator stages in TMEM let the epilogue of tile i overlap the main loop of tile i+1.
// Tiles 128 x {256, 192, 128} x 64, chosen per problem by wave count.
// C[M,N] = A * B with A given as [M,K] row-major ("K-major") or [K,M] row-major ("MN-major") and B as
// [N,K] row-major (K-major) or [K,N] row-major (MN-major); the MN-major forms serve the transposed products
// of the backward pass (dX = dY W, dW = dY^T X) without any explicit transpose.
// Replaces the XLA-compiled `dot` of every Linear layer of the reference (mamba2/mamba2_mixer.py:228,233,
// mamba2/modeling_mamba2.py:498, mamba2hybrid/mamba2hybrid_attn.py:411-413,463, mamba2hybrid/mamba2hybrid_mlp.py:121,134).
#include "common.cuh"
#include <stdlib.h>
#include <string.h>

namespace ssm {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_THREADS = 224;                       // warp 0: TMA (A), 1: MMA, 2-5: epilogue, 6: TMA (B) when dual
constexpr int EPI_BLOCK_COLS = 64;                       // bf16 columns per TMA store block (128 bytes)
constexpr int EPI_BUF_BYTES = GEMM_BM * EPI_BLOCK_COLS * 2;  // 16 KiB

struct GemmParams {
  int M, N, K;
  int a_mn, b_mn;        // operand majorness
  int mode;              // 0: bf16 via TMA store, 1: fp32 store, 2: fp32 accumulate (red.add)
  int act;               // 0 none, 1 GELU (mode 0 only)
  const __nv_bfloat16* bias;  // [N] or null (mode 0 only)
  float* c32;            // modes 1, 2
  long long ldc32;
  __nv_bfloat16* c16;    // mode 0 (direct-store epilogue)
  long long ldc16;
  float* sumsq;          // mode 1 only: += sum of squares of every stored element (gradient-norm contribution)
  int dual;              // 1: two producer warps, one issues the A loads and one the B loads of every stage
  int prefetch;          // k-blocks that the TMA producer prefetches into L2 ahead of its loads (0 = off)
  unsigned long long* trace;   // optional [grid][16] timestamps (ns) for pipeline analysis, else null
  int direct;            // 1: epilogue warps store their rows straight from registers (no smem staging / TMA store)
  int* status;
  int tiles_m, tiles_n;
  int gemm_ctas;         // CTAs that run GEMM tiles (the grid may hold extra communication CTAs)
};

constexpr int MAX_RANKS = 8;
struct PeerPtrs { void* p[MAX_RANKS]; };

// Fusion of the GEMM with the tensor-parallel collectives over peer memory.
//  * all-gather side (ag): the A operand is a gather buffer [nranks * rows_per_shard, K] in local memory that
//    every rank fills by pushing its shard into all ranks' buffers.  The last `comm_ctas` CTAs of this grid do
//    this rank's push (P2P stores) and publish flag[me] = seq on every rank; the TMA producer of the GEMM CTAs
//    waits (bounded) for flag[shard] before the first load of a shard's rows and visits the local shard first.
//  * reduce-scatter side (rs, epilogue mode 3): output rows belong to owner = row / rows_per_owner; each tile is
//    TMA-stored into the owner's landing slot for this rank (one tensor map per owner, peer memory), remote
//    owners first; when all of this rank's tiles for an owner have landed, flag[me] = seq is published there.
struct GemmComm {
  int nranks, me, seq;          // sequence number of this call = *seq_base + seq (seq_base may be null)
  const int* seq_base;          // device counter advanced once per training step (keeps CUDA-graph replays unique)
  // all-gather side
  int ag, rows_per_shard, comm_ctas, ag_flag_base, ag_cols;
  const int* ag_flags;                 // local flag array
  const __nv_bfloat16* ag_src; long long ag_src_ld;
  PeerPtrs ag_dst; long long ag_dst_ld;
  PeerPtrs flag_ptrs;                  // every rank's flag array
  int* ag_counter;
  // reduce-scatter side
  int rs, rows_per_owner, rs_flag_base;
  int* rs_counters;                    // local [nranks]
  PeerPtrs rs_land; long long rs_land_ld;   // landing slots as plain pointers (direct-store epilogue)
};
struct RsMaps { CUtensorMap m[MAX_RANKS]; };

__device__ __forceinline__ void st_release_sys_s32(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys_s32(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool wait_flag(const int* flag, int seq, int* status) {
  if (ld_acquire_sys_s32(flag) >= seq) return true;
  const uint64_t t0 = global_timer_ns();
  for (uint32_t i = 1;; ++i) {
    if (ld_acquire_sys_s32(flag) >= seq) return true;
    if ((i & 63u) == 0u) {
      if (status != nullptr && *((volatile int*)status) != 0) return false;
      if (global_timer_ns() - t0 > SSM_WAIT_NS) break;
    }
  }
  if (status != nullptr) atomicCAS(status, 0, SSM_ERR_TIMEOUT_FLAG);
  return false;
}
// m-tile visiting order: rotate so that `first_block` (a shard / owner index) comes first
__device__ __forceinline__ int rotate_m(int tm, int tiles_m, int tiles_per_block, int first_block) {
  int v = tm + first_block * tiles_per_block;
  return v >= tiles_m ? v - tiles_m : v;
}

__device__ __forceinline__ void trace_mark(const GemmParams& p, int slot) {
  if (p.trace != nullptr) p.trace[(size_t)blockIdx.x * 16 + slot] = global_timer_ns();
}

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;   // 16 KiB
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_OFF = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFF = EPI_OFF + 2 * EPI_BUF_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;      // barriers + alignment slack
};

__device__ __forceinline__ float gelu_f(float x) {
  return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_tcgen05(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_c, const GemmParams p, const GemmComm cm,
                  const __grid_constant__ RsMaps rsm) {
  using L = GemmSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int kblocks = (p.K + GEMM_BK - 1) / GEMM_BK;
  const int nctas = p.gemm_ctas;
  const int seqv = cm.seq + (cm.seq_base != nullptr ? *cm.seq_base : 0);

  if (cm.ag && cm.comm_ctas == 0) {
    // ------------------------------------------------------------------ cooperative all-gather push
    // Every CTA first moves a slice of the local shard into all ranks' gather buffers (P2P stores), the last one
    // to finish publishes this rank's flag everywhere; only then do the CTAs turn to their tiles.  The tiles of
    // remote shards could not start before the data has crossed NVLink anyway, and all SMs storing together get
    // the shard out several times faster than a few dedicated CTAs.
    const int vec_per_row = cm.ag_cols / 8;
    const long long total = (long long)cm.rows_per_shard * vec_per_row;
    const long long row_off = (long long)cm.me * cm.rows_per_shard;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
      const long long r = i / vec_per_row;
      const int c = (int)(i % vec_per_row) * 8;
      const uint4 v = *reinterpret_cast<const uint4*>(cm.ag_src + r * cm.ag_src_ld + c);
      #pragma unroll
      for (int k = 0; k < MAX_RANKS; ++k) {
        const int t = (cm.me + k) % MAX_RANKS;
        if (t < cm.nranks)
          *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(cm.ag_dst.p[t]) + (row_off + r) * cm.ag_dst_ld + c) = v;
      }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      const int done = atomicAdd(cm.ag_counter, 1) + 1;
      if (done == (int)gridDim.x) {
        __threadfence_system();
        for (int t = 0; t < cm.nranks; ++t)
          st_release_sys_s32(reinterpret_cast<int*>(cm.flag_ptrs.p[t]) + cm.ag_flag_base + cm.me, seqv);
        *cm.ag_counter = 0;
      }
    }
  }
  if ((int)blockIdx.x >= nctas) {
    // ------------------------------------------------------------------ communication CTA (all-gather push)
    const int ci = blockIdx.x - nctas;
    const int vec_per_row = cm.ag_cols / 8;
    const long long total = (long long)cm.rows_per_shard * vec_per_row;
    const long long row_off = (long long)cm.me * cm.rows_per_shard;
    for (long long i = (long long)ci * blockDim.x + threadIdx.x; i < total; i += (long long)cm.comm_ctas * blockDim.x) {
      const long long r = i / vec_per_row;
      const int c = (int)(i % vec_per_row) * 8;
      const uint4 v = *reinterpret_cast<const uint4*>(cm.ag_src + r * cm.ag_src_ld + c);
      #pragma unroll
      for (int k = 0; k < MAX_RANKS; ++k) {
        const int t = (cm.me + k) % MAX_RANKS;
        if (t < cm.nranks)
          *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(cm.ag_dst.p[t]) + (row_off + r) * cm.ag_dst_ld + c) = v;
      }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      const int done = atomicAdd(cm.ag_counter, 1) + 1;
      if (done == cm.comm_ctas) {
        __threadfence_system();
        for (int t = 0; t < cm.nranks; ++t)
          st_release_sys_s32(reinterpret_cast<int*>(cm.flag_ptrs.p[t]) + cm.ag_flag_base + cm.me, seqv);
        *cm.ag_counter = 0;
      }
    }
    return;
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], p.dual ? 2 : 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull_bar[a], 1); mbar_init(&tempty_bar[a], 4); }
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (p.mode != 3) tma_prefetch_desc(&tmap_c);
    if (p.mode == 3) for (int t = 0; t < cm.nranks; ++t) tma_prefetch_desc(&rsm.m[t]);
  }
  constexpr int TMEM_COLS = 2 * BN <= 256 ? 256 : 512;      // allocation sizes are powers of two
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) trace_mark(p, 0);

  if (warp == 0 || (warp == 6 && p.dual)) {
    // ------------------------------------------------------------------ TMA producer(s)
    // One thread issuing every load of a stage is a bottleneck of its own: a tensor-map copy takes that thread a few
    // hundred cycles to issue, and a stage needs 2 (K-major operands) to 6 (MN-major) of them.  With `dual` warp 0
    // issues the A loads and warp 6 the B loads; both arm the same full barrier (two arrivals) with their byte counts.
    const bool do_a = warp == 0, do_b = warp == 6 || !p.dual;
    const uint32_t tx_bytes = (do_a ? L::A_BYTES : 0) + (do_b ? L::B_BYTES : 0);
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      int armed[STAGES];
      #pragma unroll
      for (int s = 0; s < STAGES; ++s) armed[s] = -1;
      bool ok = true;
      uint32_t shard_seen = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += nctas) {
        int tm = tile % p.tiles_m;
        if (cm.ag) tm = rotate_m(tm, p.tiles_m, cm.rows_per_shard / GEMM_BM, cm.me);
        if (cm.rs) tm = rotate_m(tm, p.tiles_m, cm.rows_per_owner / GEMM_BM, (cm.me + 1) % cm.nranks);
        const int m0 = tm * GEMM_BM;
        const int n0 = (tile / p.tiles_m) * BN;
        if (cm.ag) {
          const int shard = m0 / cm.rows_per_shard;
          if (!(shard_seen & (1u << shard))) {
            if (!wait_flag(cm.ag_flags + cm.ag_flag_base + shard, seqv, p.status)) { ok = false; break; }
            fence_proxy_async_all();      // rows were written by generic-proxy stores (local or peer SMs)
            shard_seen |= 1u << shard;
          }
        }
        for (int kb = 0; kb < kblocks; ++kb) {
          if (p.prefetch > 0 && !p.dual) {
            // L2 prefetch of the operand tiles this CTA will load `prefetch` k-blocks from now (possibly in its next
            // tile): the ring of STAGES loads then completes at L2 latency instead of HBM latency
            int pk = kb + p.prefetch, ptile = tile;
            while (pk >= kblocks) { pk -= kblocks; ptile += nctas; }
            if (ptile < num_tiles) {
              int ptm = ptile % p.tiles_m;
              if (cm.ag) ptm = rotate_m(ptm, p.tiles_m, cm.rows_per_shard / GEMM_BM, cm.me);
              if (cm.rs) ptm = rotate_m(ptm, p.tiles_m, cm.rows_per_owner / GEMM_BM, (cm.me + 1) % cm.nranks);
              const int pm0 = ptm * GEMM_BM, pn0 = (ptile / p.tiles_m) * BN, pk0 = pk * GEMM_BK;
              if (!cm.ag) {                       // gathered rows may not have arrived yet: weights only in that case
                if (!p.a_mn) tma_prefetch_l2_2d(&tmap_a, pk0, pm0);
                else { tma_prefetch_l2_2d(&tmap_a, pm0, pk0); tma_prefetch_l2_2d(&tmap_a, pm0 + 64, pk0); }
              }
              if (!p.b_mn) tma_prefetch_l2_2d(&tmap_b, pk0, pn0);
              else {
                #pragma unroll
                for (int j = 0; j < BN / 64; ++j) tma_prefetch_l2_2d(&tmap_b, pn0 + 64 * j, pk0);
              }
            }
          }
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status)) { ok = false; break; }
          uint8_t* sa = smem + stage * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          mbar_expect_tx(&full_bar[stage], tx_bytes);
          armed[stage] = (int)phase;
          const int k0 = kb * GEMM_BK;
          if (do_a) {
            if (!p.a_mn) {
              tma_load_2d(sa, &tmap_a, k0, m0, &full_bar[stage]);                 // box {64 k, 128 m}
            } else {
              tma_load_2d(sa, &tmap_a, m0, k0, &full_bar[stage]);                 // box {64 m, 64 k} x 2
              tma_load_2d(sa + 8192, &tmap_a, m0 + 64, k0, &full_bar[stage]);
            }
          }
          if (do_b) {
            if (!p.b_mn) {
              tma_load_2d(sb, &tmap_b, k0, n0, &full_bar[stage]);                 // box {64 k, BN n}
            } else {
              #pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_2d(sb + j * 8192, &tmap_b, n0 + 64 * j, k0, &full_bar[stage]);  // box {64 n, 64 k}
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
          if (do_a && tile == (int)blockIdx.x && kb == 0) trace_mark(p, 8);
        }
      }
      if (do_a) trace_mark(p, 9);
      if (!ok) {
        // error path: let copies that are still in flight land before the CTA's shared memory goes away
        #pragma unroll
        for (int s = 0; s < STAGES; ++s)
          if (armed[s] >= 0) mbar_wait(&full_bar[s], (uint32_t)armed[s], nullptr);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(GEMM_BM, BN, p.a_mn, p.b_mn);
      const uint32_t a_step = p.a_mn ? (16 * 128) >> 4 : 32 >> 4;  // descriptor start-address step per UMMA_K=16
      const uint32_t b_step = p.b_mn ? (16 * 128) >> 4 : 32 >> 4;
      const uint32_t a_lbo = p.a_mn ? 8192u : 16u, b_lbo = p.b_mn ? 8192u : 16u;
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += nctas) {
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, p.status)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.status)) { ok = false; break; }
          tc_fence_after_sync();
          if (tile == (int)blockIdx.x && kb == 0) trace_mark(p, 1);
          const uint32_t sa = smem_u32(smem + stage * L::STAGE_BYTES);
          const uint32_t sb = sa + L::A_BYTES;
          const uint64_t da = make_smem_desc_sw128(sa, a_lbo, 1024);
          const uint64_t db = make_smem_desc_sw128(sb, b_lbo, 1024);
          #pragma unroll
          for (int kk = 0; kk < GEMM_BK / 16; ++kk)
            umma_bf16(d_tmem, da + (uint64_t)(kk * a_step), db + (uint64_t)(kk * b_step), idesc, (kb | kk) != 0);
          umma_commit(&empty_bar[stage]);          // frees the smem stage once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tfull_bar[acc]);      // accumulator complete
        trace_mark(p, tile == (int)blockIdx.x ? 2 : 3);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp >= 2 && warp < 6) {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;                        // TMEM lane quarter this warp may access
    const int epi_tid = threadIdx.x - 64;          // 0..127
    const int row = q * 32 + lane;                 // row of the tile held by this thread
    uint8_t* epi_buf = smem + L::EPI_OFF;
    int acc = 0; uint32_t acc_phase = 0;
    bool ok = true;
    int stores_issued = 0;
    float ssq = 0.f;                               // this thread's share of sum(C^2) (mode 1 with p.sumsq)
    int rs_count[MAX_RANKS];
    #pragma unroll
    for (int t = 0; t < MAX_RANKS; ++t) rs_count[t] = 0;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += nctas) {
      int tm = tile % p.tiles_m;
      if (cm.ag) tm = rotate_m(tm, p.tiles_m, cm.rows_per_shard / GEMM_BM, cm.me);
      if (cm.rs) tm = rotate_m(tm, p.tiles_m, cm.rows_per_owner / GEMM_BM, (cm.me + 1) % cm.nranks);
      const int m0 = tm * GEMM_BM;
      const int n0 = (tile / p.tiles_m) * BN;
      const int owner = cm.rs ? m0 / cm.rows_per_owner : 0;
      if (cm.rs && ok) {
        #pragma unroll
        for (int t = 0; t < MAX_RANKS; ++t) if (t == owner) rs_count[t] += 1;
      }
      if (!mbar_wait(&tfull_bar[acc], acc_phase, p.status)) { ok = false; }
      {
        // the four epilogue warps must agree on the outcome before they meet at named barriers
        uint32_t mine = ok ? 1u : 0u, all;
        asm volatile(
            "{\n\t"
            ".reg .pred p, q;\n\t"
            "setp.ne.u32 p, %1, 0;\n\t"
            "bar.red.and.pred q, 1, 128, p;\n\t"
            "selp.u32 %0, 1, 0, q;\n\t"
            "}\n"
            : "=r"(all) : "r"(mine) : "memory");
        ok = all != 0;
      }
      tc_fence_after_sync();
      if (epi_tid == 0) trace_mark(p, tile == (int)blockIdx.x ? 4 : 6);
      if (ok) {
        #pragma unroll 1
        for (int j = 0; j < BN / EPI_BLOCK_COLS; ++j) {
          const int nb = n0 + j * EPI_BLOCK_COLS;
          if (nb >= p.N) break;
          uint32_t v[2][32];
          tmem_ld32(tmem_addr(tmem_base, q * 32, acc * BN + j * 64), v[0]);
          tmem_ld32(tmem_addr(tmem_base, q * 32, acc * BN + j * 64 + 32), v[1]);
          tmem_ld_wait();
          if (p.direct && p.mode == 3) {
            // reduce-scatter: the row goes straight into the owner's landing slot (peer memory, P2P stores)
            __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(cm.rs_land.p[owner]) +
                                  (long long)(m0 - owner * cm.rows_per_owner + row) * cm.rs_land_ld;
            #pragma unroll
            for (int h = 0; h < 2; ++h) {
              #pragma unroll
              for (int c = 0; c < 4; ++c) {
                const int col = nb + h * 32 + c * 8;
                if (col >= p.N) break;
                uint4 o;
                o.x = pack_bf16(__uint_as_float(v[h][c * 8 + 0]), __uint_as_float(v[h][c * 8 + 1]));
                o.y = pack_bf16(__uint_as_float(v[h][c * 8 + 2]), __uint_as_float(v[h][c * 8 + 3]));
                o.z = pack_bf16(__uint_as_float(v[h][c * 8 + 4]), __uint_as_float(v[h][c * 8 + 5]));
                o.w = pack_bf16(__uint_as_float(v[h][c * 8 + 6]), __uint_as_float(v[h][c * 8 + 7]));
                *reinterpret_cast<uint4*>(base + col) = o;        // N % 8 == 0 on this path
              }
            }
          } else if (p.direct) {
            // every thread owns one output row: 64 consecutive columns = 128 B (bf16) or 2 x 128 B (fp32)
            const int r = m0 + row;
            if (r < p.M) {
              #pragma unroll
              for (int h = 0; h < 2; ++h) {
                #pragma unroll
                for (int c = 0; c < 4; ++c) {
                  const int col = nb + h * 32 + c * 8;
                  if (col >= p.N) break;
                  float f[8];
                  #pragma unroll
                  for (int e = 0; e < 8; ++e) {
                    float x = __uint_as_float(v[h][c * 8 + e]);
                    if (p.mode == 0) {
                      if (p.bias != nullptr && col + e < p.N) x += __bfloat162float(p.bias[col + e]);
                      if (p.act == 1) x = gelu_f(x);
                    }
                    f[e] = x;
                  }
                  if (p.mode == 0) {
                    __nv_bfloat16* dst = p.c16 + (long long)r * p.ldc16 + col;
                    if (col + 8 <= p.N) {
                      uint4 o;
                      o.x = pack_bf16(f[0], f[1]); o.y = pack_bf16(f[2], f[3]);
                      o.z = pack_bf16(f[4], f[5]); o.w = pack_bf16(f[6], f[7]);
                      *reinterpret_cast<uint4*>(dst) = o;
                    } else {
                      for (int e = 0; e < 8 && col + e < p.N; ++e) dst[e] = __float2bfloat16(f[e]);
                    }
                  } else {
                    float* dst = p.c32 + (long long)r * p.ldc32 + col;
                    #pragma unroll
                    for (int q4 = 0; q4 < 2; ++q4) {
                      const int cc = col + q4 * 4;
                      if (cc + 4 <= p.N) {
                        if (p.mode == 1)
                          *reinterpret_cast<float4*>(dst + q4 * 4) = make_float4(f[q4 * 4], f[q4 * 4 + 1], f[q4 * 4 + 2], f[q4 * 4 + 3]);
                        else
                          asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + q4 * 4), "f"(f[q4 * 4]),
                                       "f"(f[q4 * 4 + 1]), "f"(f[q4 * 4 + 2]), "f"(f[q4 * 4 + 3]) : "memory");
                      } else {
                        for (int e = 0; e < 4 && cc + e < p.N; ++e) {
                          if (p.mode == 1) dst[q4 * 4 + e] = f[q4 * 4 + e];
                          else atomicAdd(dst + q4 * 4 + e, f[q4 * 4 + e]);
                        }
                      }
                    }
                  }
                }
              }
            }
          } else if (p.mode == 0 || p.mode == 3) {
            uint8_t* buf = epi_buf + (stores_issued & 1) * EPI_BUF_BYTES;
            if (epi_tid == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (p.bias == nullptr && p.act == 0) {
              // plain output (every GEMM of the training step except the MLP up-projection): convert and stage only;
              // keeping the bias / GELU arithmetic out of this loop matters, the compiler otherwise evaluates it
              // for every element and selects
              #pragma unroll
              for (int h = 0; h < 2; ++h) {
                #pragma unroll
                for (int c = 0; c < 4; ++c) {           // 16-byte chunk = 8 bf16
                  uint4 o;
                  o.x = pack_bf16(__uint_as_float(v[h][c * 8 + 0]), __uint_as_float(v[h][c * 8 + 1]));
                  o.y = pack_bf16(__uint_as_float(v[h][c * 8 + 2]), __uint_as_float(v[h][c * 8 + 3]));
                  o.z = pack_bf16(__uint_as_float(v[h][c * 8 + 4]), __uint_as_float(v[h][c * 8 + 5]));
                  o.w = pack_bf16(__uint_as_float(v[h][c * 8 + 6]), __uint_as_float(v[h][c * 8 + 7]));
                  *reinterpret_cast<uint4*>(buf + sw128_offset(row, h * 4 + c)) = o;
                }
              }
            } else {
              #pragma unroll
              for (int h = 0; h < 2; ++h) {
                #pragma unroll
                for (int c = 0; c < 4; ++c) {
                  float f[8];
                  #pragma unroll
                  for (int e = 0; e < 8; ++e) {
                    float x = __uint_as_float(v[h][c * 8 + e]);
                    const int col = nb + h * 32 + c * 8 + e;
                    if (p.bias != nullptr && col < p.N) x += __bfloat162float(p.bias[col]);
                    if (p.act == 1) x = gelu_f(x);
                    f[e] = x;
                  }
                  uint4 o;
                  o.x = pack_bf16(f[0], f[1]); o.y = pack_bf16(f[2], f[3]);
                  o.z = pack_bf16(f[4], f[5]); o.w = pack_bf16(f[6], f[7]);
                  *reinterpret_cast<uint4*>(buf + sw128_offset(row, h * 4 + c)) = o;
                }
              }
            }
            fence_proxy_async_smem();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (epi_tid == 0) {
              if (p.mode == 0) tma_store_2d(&tmap_c, buf, nb, m0);
              else tma_store_2d(&rsm.m[owner], buf, nb, m0 - owner * cm.rows_per_owner);
              tma_store_commit();
            }
            ++stores_issued;
          } else {
            // fp32 output: 32 columns (128 bytes) per staging block, TMA store or TMA reduce-add (grad accumulation)
            #pragma unroll
            for (int h = 0; h < 2; ++h) {
              if (nb + h * 32 >= p.N) break;
              uint8_t* buf = epi_buf + (stores_issued & 1) * EPI_BUF_BYTES;
              if (epi_tid == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
              asm volatile("bar.sync 1, 128;" ::: "memory");
              #pragma unroll
              for (int c = 0; c < 8; ++c)
                *reinterpret_cast<uint4*>(buf + sw128_offset(row, c)) =
                    make_uint4(v[h][c * 4], v[h][c * 4 + 1], v[h][c * 4 + 2], v[h][c * 4 + 3]);
              if (p.sumsq != nullptr) {            // rows / columns beyond M, N hold exact zeros (TMA zero fill)
                #pragma unroll
                for (int e = 0; e < 32; ++e) ssq += __uint_as_float(v[h][e]) * __uint_as_float(v[h][e]);
              }
              fence_proxy_async_smem();
              asm volatile("bar.sync 1, 128;" ::: "memory");
              if (epi_tid == 0) {
                if (p.mode == 1) {
                  tma_store_2d(&tmap_c, buf, nb + h * 32, m0);
                } else {
                  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                               ::"l"(reinterpret_cast<uint64_t>(&tmap_c)), "r"(smem_u32(buf)), "r"(nb + h * 32), "r"(m0)
                               : "memory");
                }
                tma_store_commit();
              }
              ++stores_issued;
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (epi_tid == 0) trace_mark(p, tile == (int)blockIdx.x ? 5 : 7);
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (p.sumsq != nullptr && p.mode == 1) {
      #pragma unroll
      for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
      if (lane == 0) atomicAdd(p.sumsq, ssq);
    }
    if (cm.rs && p.direct) {
      // the rows were written with ordinary stores by all epilogue threads: make them visible system-wide before
      // thread 0 reports this CTA's tiles
      __threadfence_system();
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    if (epi_tid == 0) {
      tma_store_wait_all();
      if (cm.rs && ok) {
        // all tiles of this CTA have landed: publish per owner once every CTA has reported its share
        fence_proxy_async_all();
        __threadfence_system();
        const int per_owner = (cm.rows_per_owner / GEMM_BM) * p.tiles_n;
        #pragma unroll
        for (int t = 0; t < MAX_RANKS; ++t) {
          if (t < cm.nranks && rs_count[t] > 0) {
            const int done = atomicAdd(cm.rs_counters + t, rs_count[t]) + rs_count[t];
            if (done == per_owner) {
              cm.rs_counters[t] = 0;
              __threadfence_system();
              st_release_sys_s32(reinterpret_cast<int*>(cm.flag_ptrs.p[t]) + cm.rs_flag_base + cm.me, seqv);
            }
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0) trace_mark(p, 10);
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ------------------------------------------------------------------------------------ host
static int g_num_sms = 0;

// SSM_GEMM_EPI=direct makes the epilogue warps store their rows straight from registers instead of staging them in
// shared memory for a TMA store (measured slower: each lane then writes its own 128-byte row segment, which costs
// most for the fp32 gradient outputs; kept for experiments).
static unsigned long long* g_trace = nullptr;

// SSM_GEMM_DUAL=0 goes back to one producer thread for all loads of a stage.
static int gemm_dual_producers() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("SSM_GEMM_DUAL");
    v = (e && atoi(e) == 0) ? 0 : 1;
  }
  return v;
}

// SSM_GEMM_PREFETCH=n: the producer prefetches operand tiles n k-blocks ahead into L2 (0 = off).
static int gemm_prefetch_distance() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("SSM_GEMM_PREFETCH");
    v = e ? atoi(e) : 0;
    if (v < 0) v = 0;
  }
  return v;
}

static int epilogue_direct() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("SSM_GEMM_EPI");
    v = (e && strcmp(e, "direct") == 0) ? 1 : 0;
  }
  return v;
}

// Tile width.  128x256 tiles have the best operand reuse; 128x192 and 128x128 tiles fill the SMs better when the
// 256-wide tiling leaves the last wave mostly empty (the per-rank shapes of tensor parallelism).  Compare the
// SM-time of the tilings: waves x relative tile cost (measured: a 128-wide tile costs 0.8 of a 256-wide one, a
// 192-wide one is taken as 0.8 = 0.75 / 0.94); a narrower tiling must win by 10 % to be chosen.
// SSM_GEMM_FORCE_BN=128|192|256 overrides the choice (experiments).
static int pick_tile_n(int M, int N) {
  static int forced = -1;
  if (forced < 0) {
    const char* e = getenv("SSM_GEMM_FORCE_BN");
    forced = e ? atoi(e) : 0;
  }
  if (N <= 128) return 128;
  if (forced == 128 || forced == 192 || forced == 256) return forced;
  const int sms = g_num_sms > 0 ? g_num_sms : 148;
  const long long tm = (M + GEMM_BM - 1) / GEMM_BM;
  auto cost = [&](int bn, double tile_cost) {
    const long long t = tm * ((N + bn - 1) / bn);
    return (double)((t + sms - 1) / sms) * tile_cost;
  };
  // fewer 128-wide tiles than SMs (decode-time GEMMs with a handful of rows, thin per-rank projections): every CTA
  // is bound by its own operand stream, so the tiling with the most CTAs wins
  if (tm * ((N + 127) / 128) <= sms) return 128;
  const double c256 = cost(256, 1.0), c192 = cost(192, 0.8), c128 = cost(128, 0.8);
  int best = 256;
  double cb = c256;
  if (c192 < 0.9 * cb) { best = 192; cb = c192; }
  if (c128 < 0.9 * c256 && c128 < cb) best = 128;
  return best;
}

template <int BN, int STAGES>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, GemmParams p,
                       cudaStream_t stream, const GemmComm* comm = nullptr, const RsMaps* maps = nullptr) {
  using L = GemmSmem<BN, STAGES>;
  static bool configured = false;
  auto kern = gemm_bf16_tcgen05<BN, STAGES>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  p.tiles_m = (p.M + GEMM_BM - 1) / GEMM_BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  const int tiles = p.tiles_m * p.tiles_n;
  static GemmComm no_comm;       // zero-initialised: no fusion
  static RsMaps no_maps;
  GemmComm cm = comm ? *comm : no_comm;
  int extra = (comm && cm.ag) ? cm.comm_ctas : 0;
  const int avail = g_num_sms - extra;
  p.gemm_ctas = tiles < avail ? tiles : avail;
  kern<<<p.gemm_ctas + extra, GEMM_THREADS, L::TOTAL, stream>>>(ta, tb, tc, p, cm, maps ? *maps : no_maps);
  return (int)cudaGetLastError();
}

}  // namespace ssm

// C[M,N] = A * B.  a_mn = 0: A is [M,K] with row stride lda; a_mn = 1: A is [K,M] with row stride lda.
// b_mn = 0: B is [N,K] with row stride ldb; b_mn = 1: B is [K,N] with row stride ldb.
// mode 0: C bf16 [M, ldc] (ldc * 2 bytes must be a multiple of 16); 1: C fp32 store; 2: C fp32 += .
// All leading dimensions in elements; operand bases 16-byte aligned, operand row strides multiples of 8.
static int gemm_bf16_impl(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                          long long ldc, int a_mn, int b_mn, int mode, const void* bias, int act, int* status,
                          cudaStream_t stream, float* sumsq);

extern "C" int ssm_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                             long long ldb, long long ldc, int a_mn, int b_mn, int mode, const void* bias, int act,
                             int* status, cudaStream_t stream) {
  return gemm_bf16_impl(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, mode, bias, act, status, stream, nullptr);
}

// Same, and with mode 1 (fp32 store) the sum of squares of the stored matrix is added to *sumsq (fp32, device):
// the wgrad GEMM then delivers its share of the global gradient norm without a second pass over the gradient.
extern "C" int ssm_gemm_bf16_ex(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                long long ldb, long long ldc, int a_mn, int b_mn, int mode, const void* bias, int act,
                                int* status, cudaStream_t stream, void* sumsq) {
  if (sumsq != nullptr && mode != 1) return -SSM_ERR_BAD_ARG;
  return gemm_bf16_impl(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, mode, bias, act, status, stream,
                        reinterpret_cast<float*>(sumsq));
}

static int gemm_bf16_impl(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                          long long ldc, int a_mn, int b_mn, int mode, const void* bias, int act, int* status,
                          cudaStream_t stream, float* sumsq) {
  using namespace ssm;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -SSM_ERR_BAD_ARG;
  if (mode == 0 && ((ldc % 8) || (reinterpret_cast<uintptr_t>(C) & 15))) return -SSM_ERR_BAD_ARG;
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int BN = pick_tile_n(M, N);
  CUtensorMap ta, tb, tc;
  int r;
  if (!a_mn) r = make_tmap_2d_bf16(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, 64, 128);
  else       r = make_tmap_2d_bf16(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, 64, 64);
  if (r) return -100 - r;
  if (!b_mn) r = make_tmap_2d_bf16(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, 64, BN);
  else       r = make_tmap_2d_bf16(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, 64);
  if (r) return -200 - r;
  if (mode == 0) {
    r = make_tmap_2d_bf16(&tc, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc * 2, 64, 128);
    if (r) return -300 - r;
  } else {
    if ((ldc % 4) || (reinterpret_cast<uintptr_t>(C) & 15)) return -SSM_ERR_BAD_ARG;
    r = make_tmap_2d(&tc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc * 4, 32, 128);
    if (r) return -300 - r;
  }
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.a_mn = a_mn; p.b_mn = b_mn; p.mode = mode; p.act = act;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.c32 = mode == 0 ? nullptr : reinterpret_cast<float*>(C);
  p.ldc32 = ldc; p.status = status; p.tiles_m = 0; p.tiles_n = 0; p.gemm_ctas = 0;
  p.c16 = mode == 0 ? reinterpret_cast<__nv_bfloat16*>(C) : nullptr;
  p.ldc16 = ldc; p.direct = epilogue_direct(); p.trace = g_trace; p.prefetch = gemm_prefetch_distance(); p.sumsq = sumsq;
  p.dual = gemm_dual_producers();
  if (sumsq != nullptr) p.direct = 0;      // the sum of squares is formed in the staged (TMA-store) epilogue
  if (BN == 256) return launch_gemm<256, 4>(ta, tb, tc, p, stream);
  if (BN == 192) return launch_gemm<192, 4>(ta, tb, tc, p, stream);
  return launch_gemm<128, 6>(ta, tb, tc, p, stream);
}

// GEMM fused with a tensor-parallel collective over peer memory (see GemmComm).
//   ag = 1: A must be this rank's gather buffer [nranks * rows_per_shard, K] (= ag_dst_ptrs[me], row stride
//           ag_dst_ld); ag_src is the local shard [rows_per_shard, K]; flag_ptrs[t] is rank t's flag array.
//   rs = 1: mode is forced to 3; land_ptrs[o] is the base of the [rows_per_owner, N] slot this rank owns inside
//           rank o's landing zone (row stride land_ld); C is ignored.
// rows_per_shard / rows_per_owner must be multiples of 128 and M = nranks * rows.
extern "C" int ssm_gemm_bf16_fused(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                   long long ldb, long long ldc, int a_mn, int b_mn, int mode, const void* bias,
                                   int act, int* status, cudaStream_t stream, int nranks, int me, int seq,
                                   const int* seq_base, const void* const* flag_ptrs, int ag, int rows_per_shard, int comm_ctas,
                                   int ag_flag_base, const void* ag_src, long long ag_src_ld,
                                   const void* const* ag_dst_ptrs, long long ag_dst_ld, int* ag_counter, int rs,
                                   int rows_per_owner, int rs_flag_base, const void* const* land_ptrs,
                                   long long land_ld, int* rs_counters) {
  using namespace ssm;
  if (M <= 0 || N <= 0 || K <= 0 || nranks < 1 || nranks > MAX_RANKS || me < 0 || me >= nranks) return -SSM_ERR_BAD_ARG;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -SSM_ERR_BAD_ARG;
  if (ag && (a_mn || rows_per_shard % GEMM_BM || (long long)rows_per_shard * nranks != M || K % 8 || comm_ctas < 0 ||
             ag_src_ld % 8 || ag_dst_ld % 8))
    return -SSM_ERR_BAD_ARG;
  if (rs && (rows_per_owner % GEMM_BM || (long long)rows_per_owner * nranks != M || land_ld % 8)) return -SSM_ERR_BAD_ARG;
  if (rs) mode = 3;
  if (mode == 0 && ((ldc % 8) || (reinterpret_cast<uintptr_t>(C) & 15))) return -SSM_ERR_BAD_ARG;
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int BN = pick_tile_n(M, N);
  CUtensorMap ta, tb, tc;
  int r;
  if (!a_mn) r = make_tmap_2d_bf16(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, 64, 128);
  else       r = make_tmap_2d_bf16(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, 64, 64);
  if (r) return -100 - r;
  if (!b_mn) r = make_tmap_2d_bf16(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, 64, BN);
  else       r = make_tmap_2d_bf16(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, 64);
  if (r) return -200 - r;
  if (mode == 0) {
    r = make_tmap_2d_bf16(&tc, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc * 2, 64, 128);
    if (r) return -300 - r;
  } else if (mode == 1 || mode == 2) {
    if ((ldc % 4) || (reinterpret_cast<uintptr_t>(C) & 15)) return -SSM_ERR_BAD_ARG;
    r = make_tmap_2d(&tc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc * 4, 32, 128);
    if (r) return -300 - r;
  } else {
    tc = ta;
  }
  RsMaps maps;
  GemmComm cm;
  memset(&cm, 0, sizeof(cm));
  memset(&maps, 0, sizeof(maps));
  cm.nranks = nranks; cm.me = me; cm.seq = seq; cm.seq_base = seq_base;
  for (int t = 0; t < MAX_RANKS; ++t) cm.flag_ptrs.p[t] = t < nranks ? const_cast<void*>(flag_ptrs[t]) : nullptr;
  if (ag) {
    cm.ag = 1; cm.rows_per_shard = rows_per_shard; cm.comm_ctas = comm_ctas; cm.ag_flag_base = ag_flag_base;
    cm.ag_cols = K; cm.ag_flags = reinterpret_cast<const int*>(flag_ptrs[me]);
    cm.ag_src = reinterpret_cast<const __nv_bfloat16*>(ag_src); cm.ag_src_ld = ag_src_ld;
    for (int t = 0; t < MAX_RANKS; ++t) cm.ag_dst.p[t] = t < nranks ? const_cast<void*>(ag_dst_ptrs[t]) : nullptr;
    cm.ag_dst_ld = ag_dst_ld; cm.ag_counter = ag_counter;
  }
  if (rs) {
    cm.rs = 1; cm.rows_per_owner = rows_per_owner; cm.rs_flag_base = rs_flag_base; cm.rs_counters = rs_counters;
    cm.rs_land_ld = land_ld;
    for (int t = 0; t < nranks; ++t) cm.rs_land.p[t] = const_cast<void*>(land_ptrs[t]);
    for (int t = 0; t < nranks; ++t) {
      r = make_tmap_2d_bf16(&maps.m[t], land_ptrs[t], (uint64_t)N, (uint64_t)rows_per_owner, (uint64_t)land_ld * 2, 64, 128);
      if (r) return -400 - r;
    }
  }
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.a_mn = a_mn; p.b_mn = b_mn; p.mode = mode; p.act = act;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.c32 = (mode == 1 || mode == 2) ? reinterpret_cast<float*>(C) : nullptr;
  p.ldc32 = ldc; p.status = status; p.tiles_m = 0; p.tiles_n = 0; p.gemm_ctas = 0;
  p.c16 = mode == 0 ? reinterpret_cast<__nv_bfloat16*>(C) : nullptr;
  p.ldc16 = ldc; p.direct = epilogue_direct(); p.trace = g_trace; p.prefetch = gemm_prefetch_distance(); p.sumsq = nullptr;
  p.dual = 0;      // the fused variants keep the single producer that their flag protocol was validated with
  if (BN == 256) return launch_gemm<256, 4>(ta, tb, tc, p, stream, &cm, &maps);
  if (BN == 192) return launch_gemm<192, 4>(ta, tb, tc, p, stream, &cm, &maps);
  return launch_gemm<128, 6>(ta, tb, tc, p, stream, &cm, &maps);
}

// Pipeline analysis: buf = device array of gridDim * 16 uint64 (or null to switch tracing off).  Slots (ns, global
// timer): 0 CTA set-up done, 8 first TMA load issued, 1 first stage landed, 2/3 MMAs of the first / a later tile
// issued, 4/6 first / later accumulator complete (seen by the epilogue), 5/7 epilogue of that tile done, 9 producer
// finished, 10 CTA done.
extern "C" int ssm_gemm_set_trace(void* buf) {
  ssm::g_trace = reinterpret_cast<unsigned long long*>(buf);
  return 0;
}
