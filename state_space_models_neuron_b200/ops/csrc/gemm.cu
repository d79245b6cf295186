// bf16 GEMM for sm_100a: TMA (no multicast) -> 128B-swizzled smem ring -> tcgen05.mma with fp32 accumulators in
// TMEM -> epilogue.  Persistent, warp-specialised, 7 warps per CTA:
//     warp 0      TMA producer (one elected thread): the A loads of every stage
//     warp 1      MMA issuer (one elected thread), owns the TMEM allocation
//     warps 2..5  epilogue: tcgen05.ld -> bf16 (plain, or +bias / GELU) -> swizzled smem -> TMA store,
//                 or fp32 TMA store / TMA reduce-add for gradient outputs (optionally adding sum(C^2) to a scalar),
//                 or TMA stores into the peers' landing zones (reduce-scatter);
//                 in the all-gather variant their first thread first pushes this rank's shard to the peers
//     warp 6      second TMA producer: the B loads of every stage
// Two accumulator stages in TMEM let the epilogue of tile i overlap the main loop of tile i+1.
//
// Two tile families:
//   * one CTA per tile, 128 x {256, 192, 128} x 64 (cta_group::1)
//   * a CTA pair per tile, 256 x {256, 128} x 64 (cta_group::2, clusters of two CTAs): every CTA loads its own 128
//     rows of A and its own half of the B rows, the even CTA issues MMAs that read both CTAs' shared memory and
//     write 128 accumulator rows into each CTA's TMEM.  Per FLOP a CTA then pulls 2/3 of the operand bytes of
//     a 128 x 256 tile through its L2 port, which is what bounds the single-CTA main loop.
// Scheduling: whole tiles round-robin over the CTAs (or pairs) for as many full waves as there are; the tiles of
// the last, partial wave are split along K over the idle units (at most 4 slices, 8 for accumulating outputs).
// Slices of a tile leave their fp32 partial sums in a scratch buffer; whichever slice finishes last sums all of them
// in slice order (the result does not depend on the arrival order) and runs the epilogue; no slice ever waits for
// another one.
//
// C[M,N] = A * B with A given as [M,K] row-major ("K-major") or [K,M] row-major ("MN-major") and B as
// [N,K] row-major (K-major) or [K,N] row-major (MN-major); the MN-major forms serve the transposed products
// of the backward pass (dX = dY W, dW = dY^T X) without any explicit transpose.
// Replaces the XLA-compiled `dot` of every Linear layer of the reference (mamba2/mamba2_mixer.py:228,233,
// mamba2/modeling_mamba2.py:498, mamba2hybrid/mamba2hybrid_attn.py:411-413,463, mamba2hybrid/mamba2hybrid_mlp.py:121,134).
#include "common.cuh"
#include <stdlib.h>
#include <string.h>

namespace ssm {

constexpr int GEMM_BM = 128;                             // accumulator rows per CTA
constexpr int GEMM_BK = 64;
constexpr int GEMM_THREADS = 224;                       // warp 0: TMA (A), 1: MMA, 2-5: epilogue, 6: TMA (B)
constexpr int EPI_BLOCK_COLS = 64;                       // bf16 columns per TMA store block (128 bytes)
constexpr int EPI_BUF_BYTES = GEMM_BM * EPI_BLOCK_COLS * 2;  // 16 KiB
constexpr int MAX_SPLIT = 8;                             // K slices of a tail tile (upper bound of GemmParams::split)
constexpr int MAX_UNITS = 160;                           // scheduling units (CTAs or pairs) the scratch is sized for
constexpr int AG_MAX_GROUPS = 4;                         // column (K) groups of a shard with a ready flag of their own

struct GemmParams {
  int M, N, K;
  int a_mn, b_mn;        // operand majorness
  int mode;              // 0: bf16 via TMA store, 1: fp32 store, 2: fp32 accumulate (red.add), 3: reduce-scatter push
  int act;               // 0 none, 1 GELU (mode 0 only)
  const __nv_bfloat16* bias;  // [N] or null (mode 0 only)
  float* c32;            // modes 1, 2
  long long ldc32;
  __nv_bfloat16* c16;    // mode 0 (direct-store epilogue)
  long long ldc16;
  float* sumsq;          // mode 1 only: += sum of squares of every stored element (gradient-norm contribution)
  int dual;              // 1: two producer warps, one issues the A loads and one the B loads of every stage
  unsigned long long* trace;   // optional [grid][16] timestamps (ns) for pipeline analysis, else null
  int direct;            // 1: epilogue warps store their rows straight from registers (no smem staging / TMA store)
  int* status;
  int tiles_m, tiles_n;
  // schedule: `units` CTAs (or CTA pairs) take whole tiles [0, full_tiles) round-robin; the `rem` tiles after them
  // are cut into `split` K slices each, one slice per unit
  int units, full_tiles, rem, split;
  float* ws;             // scratch for partial sums of split tiles: [rem][split][CTAs per unit][128 x BN] fp32
                         // (rem * split <= units, so it never exceeds one 128 x 256 block per CTA of the grid)
  int* ws_counters;      // [rem][CTAs per unit] arrival counters (zero between launches)
  // cross-entropy statistics of the rows of C (mode 0, LM head): per n-tile (max, sum exp(x - max)) of the bf16-rounded
  // logits and the logit at the row's label
  const long long* ce_labels;   // [M] global ids, negative = ignored; null = off
  long long ce_vocab_start;
  float* ce_max;         // [tiles_n][M]
  float* ce_sum;         // [tiles_n][M]
  float* ce_tgt;         // [M], written only for rows whose label lies in [vocab_start, vocab_start + N)
};

constexpr int MAX_RANKS = 8;
struct PeerPtrs { void* p[MAX_RANKS]; };

// Fusion of the GEMM with the tensor-parallel collectives over peer memory.
//  * all-gather side (ag): the A operand is a gather buffer [nranks * rows_per_shard, K] in local memory that
//    every rank fills by pushing its shard into all ranks' buffers.  One thread per CTA moves boxes of the local
//    shard through shared memory (TMA load, then one TMA store per destination rank over NVLink) before the
//    epilogue warps turn to their tiles.  The shard travels in up to four groups of columns (ranges of K), first
//    columns first; the CTA that completes a group publishes flag[me][group] = seq on every rank.  Meanwhile the
//    producer and MMA warps already work: tiles of the local shard read the shard itself (second tensor map);
//    the main loop of a tile of a remote shard waits (bounded) for a column group only when it reaches that
//    group's first k-block, so it starts when a quarter of the shard has landed and computes on it while the rest
//    is still crossing NVLink.  (No TMA load touches peer memory.)
//  * reduce-scatter side (rs, epilogue mode 3): output rows belong to owner = row / rows_per_owner; each tile is
//    TMA-stored into the owner's landing slot for this rank (one tensor map per owner, peer memory), remote
//    owners first; when all of this rank's tiles for an owner have landed, flag[me] = seq is published there.
//    Tiles are visited owner by owner, this rank's own rows last.  With rs_out set the kernel also finishes the
//    collective, in one of two ways.  Two ranks (rs_tail = 0): the epilogue of a tile of this rank's own rows
//    waits (bounded, once) for the flag of the other source, adds its partial block from the landing zone to the
//    fp32 accumulators and stores the reduced rows into rs_out.  More ranks (rs_tail = 1): summing T - 1 blocks in
//    the epilogues of the few CTAs that hold own tiles would be a long chain of dependent loads, so the own tiles
//    store their partial into rs_out, and after its tiles every CTA of the grid waits (bounded) for the flags of
//    all sources (this rank's included) and sums a slice: rs_out += the T - 1 landed blocks, fp32 accumulate.
//    The waits are for flags that peers (or this grid's epilogues, which never wait for the tail) publish.
struct GemmComm {
  int nranks, me, seq;          // sequence number of this call = *seq_base + seq (seq_base may be null)
  const int* seq_base;          // device counter advanced once per training step (keeps CUDA-graph replays unique)
  // all-gather side
  int ag, rows_per_shard, ag_group_kb, ag_flag_base, ag_cols;   // ag_group_kb: 64-column blocks per flag group
  int ag_push_rows;                    // rows of a push box (128, 64 or 32)
  const int* ag_flags;                 // local flag array
  const __nv_bfloat16* ag_src; long long ag_src_ld;
  PeerPtrs ag_dst; long long ag_dst_ld;
  PeerPtrs flag_ptrs;                  // every rank's flag array
  int* ag_counter;                     // local [AG_MAX_GROUPS], zero between launches
  // reduce-scatter side
  int rs, rows_per_owner, rs_flag_base;
  int* rs_counters;                    // local [nranks]
  PeerPtrs rs_land; long long rs_land_ld;   // landing slots as plain pointers (direct-store epilogue)
  const __nv_bfloat16* rs_land_local; long long rs_slot_stride;   // this rank's landing zone [nranks][rows][ld]
  __nv_bfloat16* rs_out; long long rs_out_ld;                     // reduced block [rows_per_owner, N] or null
  int rs_tail;                         // how the partial blocks are summed into rs_out: 0 in the epilogues of this
                                       // rank's own tiles, 1 by all CTAs after their tiles (see below)
};
// one tensor map per rank: the owners' landing slots (reduce-scatter) or the ranks' gather buffers (all-gather push)
struct RsMaps { CUtensorMap m[MAX_RANKS]; };

__device__ __forceinline__ void st_release_sys_s32(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// after ONE system-scope fence, flags for several ranks go out back to back; a loop of release stores pays one NVLink
// round trip per destination in series
__device__ __forceinline__ void st_relaxed_sys_s32(int* p, int v) {
  asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys_s32(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Sequence numbers wrap around: "flag has reached seq" is a signed distance, valid while the two are less than
// 2^31 apart.
__device__ __forceinline__ bool seq_reached(int flag, int seq) {
  return (int)((unsigned)flag - (unsigned)seq) >= 0;
}
__device__ __forceinline__ bool wait_flag(const int* flag, int seq, int* status) {
  if (seq_reached(ld_acquire_sys_s32(flag), seq)) return true;
  const uint64_t t0 = global_timer_ns();
  for (uint32_t i = 1;; ++i) {
    if (seq_reached(ld_acquire_sys_s32(flag), seq)) return true;
    if ((i & 63u) == 0u) {
      if (status != nullptr && *((volatile int*)status) != 0) return false;
      if (global_timer_ns() - t0 > SSM_WAIT_NS) break;
    }
  }
  if (status != nullptr) atomicCAS(status, 0, SSM_ERR_TIMEOUT_FLAG);
  return false;
}
constexpr int GEMM_TRACE_SLOTS = 24;      // int64 time stamps per CTA in the trace buffer (ssm_gemm_set_trace)
__device__ __forceinline__ void trace_mark(const GemmParams& p, int slot) {
  if (p.trace != nullptr) p.trace[(size_t)blockIdx.x * GEMM_TRACE_SLOTS + slot] = global_timer_ns();
}

template <int BN, int STAGES, bool PAIR>
struct GemmSmem {
  static constexpr int B_ROWS = PAIR ? BN / 2 : BN;       // rows of B that this CTA loads
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;   // 16 KiB
  static constexpr int B_BYTES = B_ROWS * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_OFF = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFF = EPI_OFF + 2 * EPI_BUF_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;      // barriers + alignment slack
};

__device__ __forceinline__ float gelu_f(float x) {
  return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
}

struct Work { int tile, kb0, kb1, slice, nslices, tail; };

__device__ __forceinline__ bool get_work(const GemmParams& p, int unit, int it, int kblocks, Work& w) {
  const int idx = unit + it * p.units;
  if (idx < p.full_tiles) {
    w.tile = idx; w.kb0 = 0; w.kb1 = kblocks; w.slice = 0; w.nslices = 1; w.tail = 0;
    return true;
  }
  if (it != p.full_tiles / p.units || unit >= p.rem * p.split) return false;
  w.tail = unit / p.split;
  w.tile = p.full_tiles + w.tail;
  w.slice = unit - w.tail * p.split;
  w.nslices = p.split;
  w.kb0 = (int)((long long)w.slice * kblocks / p.split);
  w.kb1 = (int)((long long)(w.slice + 1) * kblocks / p.split);
  return true;
}

// (first row of this CTA's 128 accumulator rows, first column of the tile).  Plain GEMMs walk the tiles column by
// column inside bands of 8 m-tiles.  The collective variants walk them block by block, a block being the rows of one source shard (all-gather)
// or of one owner (reduce-scatter): the all-gather starts with the local shard, whose rows need no transfer, and
// takes the remote shards in ring order behind it; the reduce-scatter starts with the next rank's rows, so that
// every partial block is on its way as early as possible, and ends with this rank's own rows.  With whole tiles
// dealt round-robin every unit therefore begins with work that does not wait for a peer, as far as there is any.
template <int BN, bool PAIR>
__device__ __forceinline__ void tile_origin(const GemmParams& p, const GemmComm& cm, int tile, int cta_rank, int& m0, int& n0) {
  constexpr int TILE_M = PAIR ? 256 : 128;
  int tm, tn;
  if (cm.ag || cm.rs) {
    const int tpb = (cm.ag ? cm.rows_per_shard : cm.rows_per_owner) / TILE_M;    // m-tiles per block (host: divisible)
    const int per_block = tpb * p.tiles_n;
    const int bi = tile / per_block, within = tile - bi * per_block;
    int block = (cm.ag ? cm.me : (cm.me + 1 == cm.nranks ? 0 : cm.me + 1)) + bi;
    if (block >= cm.nranks) block -= cm.nranks;
    tn = within / tpb;
    tm = block * tpb + (within - tn * tpb);
  } else {
    // bands of RASTER_M m-tiles, column by column inside a band: the tiles of one wave then share a few A row blocks
    // and a few B column blocks instead of all of A (tall outputs like the wgrad of in_proj re-read A from DRAM once
    // per wave otherwise: ncu showed 7.6x the operand bytes)
    constexpr int RASTER_M = 8;
    const int band = tile / (RASTER_M * p.tiles_n);
    const int within = tile - band * (RASTER_M * p.tiles_n);
    const int first_m = band * RASTER_M;
    const int rows_in_band = p.tiles_m - first_m < RASTER_M ? p.tiles_m - first_m : RASTER_M;
    tn = within / rows_in_band;
    tm = first_m + (within - tn * rows_in_band);
  }
  m0 = tm * TILE_M + cta_rank * GEMM_BM;
  n0 = tn * BN;
}

template <int BN, int STAGES, bool PAIR>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_tcgen05(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CUtensorMap tmap_a_local,
                  const __grid_constant__ CUtensorMap tmap_push, const GemmParams p, const GemmComm cm,
                  const __grid_constant__ RsMaps rsm) {
  using L = GemmSmem<BN, STAGES, PAIR>;
  constexpr int CTAS_PER_UNIT = PAIR ? 2 : 1;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint64_t* push_bar = tempty_bar + 2;                         // all-gather push: shard tile landed in shared memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(push_bar + 1);
  int* epi_flag = reinterpret_cast<int*>(tmem_slot + 1);      // epilogue warps: "this slice arrived last"

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta_rank = PAIR ? (int)cluster_ctarank() : 0;
  const int unit = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const bool leader = cta_rank == 0;
  const int kblocks = (p.K + GEMM_BK - 1) / GEMM_BK;
  const int seqv = (int)((unsigned)cm.seq + (cm.seq_base != nullptr ? (unsigned)*cm.seq_base : 0u));

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], p.dual ? 2 : 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull_bar[a], 1); mbar_init(&tempty_bar[a], 4 * CTAS_PER_UNIT); }
    mbar_init(push_bar, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (p.mode != 3 || cm.rs_out != nullptr) tma_prefetch_desc(&tmap_c);
    if (p.mode == 3 || cm.ag) for (int t = 0; t < cm.nranks; ++t) tma_prefetch_desc(&rsm.m[t]);
    if (cm.ag) { tma_prefetch_desc(&tmap_a_local); tma_prefetch_desc(&tmap_push); }
  }
  constexpr int TMEM_COLS = 2 * BN <= 256 ? 256 : 512;      // allocation sizes are powers of two
  if (warp == 1) {
    if (PAIR) { tmem_alloc_pair(tmem_slot, TMEM_COLS); tmem_relinquish_pair(); }
    else { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  }
  tc_fence_before_sync();
  if (PAIR) cluster_sync_all(); else __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) trace_mark(p, 0);

  if (warp == 0 || (warp == 6 && p.dual)) {
    // ------------------------------------------------------------------ TMA producer(s)
    // A tensor-map copy takes the issuing thread a few hundred cycles, and a stage needs 2 (K-major operands) to 6
    // (MN-major) of them: warp 0 issues the A loads and warp 6 the B loads; both arm the same full barrier.  In a
    // pair both CTAs' loads complete on the leader's barrier, which its producers arm with the bytes of both CTAs.
    const bool do_a = warp == 0, do_b = warp == 6 || !p.dual;
    const uint32_t tx_bytes = ((do_a ? L::A_BYTES : 0) + (do_b ? L::B_BYTES : 0)) * CTAS_PER_UNIT;
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      int armed[STAGES];
      #pragma unroll
      for (int s = 0; s < STAGES; ++s) armed[s] = -1;
      bool ok = true;
      uint32_t group_seen = 0;
      Work w;
      for (int it = 0; ok && get_work(p, unit, it, kblocks, w); ++it) {
        int m0, n0;
        tile_origin<BN, PAIR>(p, cm, w.tile, cta_rank, m0, n0);
        const int nb0 = n0 + cta_rank * L::B_ROWS;         // first B row (= output column) this CTA loads
        const CUtensorMap* ta = &tmap_a;
        int am0 = m0;
        int remote_shard = -1;                             // >= 0: the rows come from that rank's push
        if (cm.ag) {
          const int shard = m0 / cm.rows_per_shard;
          if (shard == cm.me) {
            ta = &tmap_a_local;                            // the local shard is read in place
            am0 = m0 - shard * cm.rows_per_shard;
          } else if (m0 < p.M && do_a) {
            remote_shard = shard;
          }
        }
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (remote_shard >= 0) {
            const int grp = kb / cm.ag_group_kb;
            const uint32_t bit = 1u << (remote_shard * AG_MAX_GROUPS + grp);
            if (!(group_seen & bit)) {
              if (!wait_flag(cm.ag_flags + cm.ag_flag_base + remote_shard * AG_MAX_GROUPS + grp, seqv, p.status)) { ok = false; break; }
              fence_proxy_async_all();      // the columns were written by the peer's bulk stores; TMA reads them
              if (group_seen == 0) trace_mark(p, 12);
              group_seen |= bit;
            }
          }
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status)) { ok = false; break; }
          uint8_t* sa = smem + stage * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          if (leader) mbar_expect_tx(&full_bar[stage], tx_bytes);
          armed[stage] = (int)phase;
          const int k0 = kb * GEMM_BK;
          if (!PAIR) {
            if (do_a) {
              if (!p.a_mn) {
                tma_load_2d(sa, ta, k0, am0, &full_bar[stage]);                 // box {64 k, 128 m}
              } else {
                tma_load_2d(sa, ta, am0, k0, &full_bar[stage]);                 // box {64 m, 64 k} x 2
                tma_load_2d(sa + 8192, ta, am0 + 64, k0, &full_bar[stage]);
              }
            }
            if (do_b) {
              if (!p.b_mn) {
                tma_load_2d(sb, &tmap_b, k0, nb0, &full_bar[stage]);            // box {64 k, BN n}
              } else {
                #pragma unroll
                for (int j = 0; j < L::B_ROWS / 64; ++j)
                  tma_load_2d(sb + j * 8192, &tmap_b, nb0 + 64 * j, k0, &full_bar[stage]);  // box {64 n, 64 k}
              }
            }
          } else {
            const uint32_t bar = smem_u32(&full_bar[stage]) & PAIR_LEADER_MASK;
            if (do_a) {
              if (!p.a_mn) {
                tma_load_2d_pair(sa, ta, k0, am0, bar);
              } else {
                tma_load_2d_pair(sa, ta, am0, k0, bar);
                tma_load_2d_pair(sa + 8192, ta, am0 + 64, k0, bar);
              }
            }
            if (do_b) {
              if (!p.b_mn) {
                tma_load_2d_pair(sb, &tmap_b, k0, nb0, bar);                    // box {64 k, BN/2 n}
              } else {
                #pragma unroll
                for (int j = 0; j < L::B_ROWS / 64; ++j)
                  tma_load_2d_pair(sb + j * 8192, &tmap_b, nb0 + 64 * j, k0, bar);
              }
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
          if (do_a && it == 0 && kb == w.kb0) trace_mark(p, 8);
        }
      }
      if (do_a) trace_mark(p, 9);
      if (!ok) {
        // error path: let copies that are still in flight land before the CTA's shared memory goes away
        if (leader) {
          #pragma unroll
          for (int s = 0; s < STAGES; ++s)
            if (armed[s] >= 0) mbar_wait(&full_bar[s], (uint32_t)armed[s], nullptr);
        } else {
          const uint64_t t0 = global_timer_ns();           // the peer's copies complete on the leader's barriers
          while (global_timer_ns() - t0 < 50000ull) { }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (even CTA of a pair only)
    if (lane == 0 && leader) {
      const uint32_t idesc = make_idesc_bf16(PAIR ? 256 : 128, BN, p.a_mn, p.b_mn);
      const uint32_t a_step = p.a_mn ? (16 * 128) >> 4 : 32 >> 4;  // descriptor start-address step per UMMA_K=16
      const uint32_t b_step = p.b_mn ? (16 * 128) >> 4 : 32 >> 4;
      const uint32_t a_lbo = p.a_mn ? 8192u : 16u, b_lbo = p.b_mn ? 8192u : 16u;
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      bool ok = true;
      Work w;
      for (int it = 0; ok && get_work(p, unit, it, kblocks, w); ++it) {
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, p.status)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.status)) { ok = false; break; }
          tc_fence_after_sync();
          if (it == 0 && kb == w.kb0) trace_mark(p, 1);
          const uint32_t sa = smem_u32(smem + stage * L::STAGE_BYTES);
          const uint32_t sb = sa + L::A_BYTES;
          const uint64_t da = make_smem_desc_sw128(sa, a_lbo, 1024);
          const uint64_t db = make_smem_desc_sw128(sb, b_lbo, 1024);
          #pragma unroll
          for (int kk = 0; kk < GEMM_BK / 16; ++kk) {
            const uint32_t accum = (kb != w.kb0 || kk != 0) ? 1u : 0u;
            if (PAIR) umma_bf16_pair(d_tmem, da + (uint64_t)(kk * a_step), db + (uint64_t)(kk * b_step), idesc, accum);
            else umma_bf16(d_tmem, da + (uint64_t)(kk * a_step), db + (uint64_t)(kk * b_step), idesc, accum);
          }
          // frees the smem stage (in both CTAs of a pair) once these MMAs have read it
          if (PAIR) umma_commit_pair(&empty_bar[stage]); else umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) { if (PAIR) umma_commit_pair(&tfull_bar[acc]); else umma_commit(&tfull_bar[acc]); }   // accumulator complete
        trace_mark(p, it == 0 ? 2 : 3);
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

    if (cm.ag) {
      // -------- all-gather push: the local shard goes to every rank's gather buffer in boxes of 128 / 64 / 32 rows x
      // 64 columns: TMA load into the (still idle) epilogue staging buffers, one TMA store per destination.  One
      // thread per CTA drives it.  The boxes are dealt round-robin over the CTAs of the grid, column group by column
      // group, and the host picks the box height so that every CTA gets about one box per group: all SMs push the
      // first columns first, which is what lets remote tiles start early.  The CTA that completes a group publishes
      // its flag on every rank.  The bulk copies leave the load/store units and their path to L2 alone, which the
      // main loop running next to them needs.
      if (epi_tid == 0) {
        const int col_blocks = (cm.ag_cols + 63) / 64;                 // 64-column blocks of the shard
        const int row_blocks = cm.rows_per_shard / cm.ag_push_rows;
        const uint32_t box_bytes = (uint32_t)cm.ag_push_rows * 128u;
        const int ngroups = (col_blocks + cm.ag_group_kb - 1) / cm.ag_group_kb;
        const int grid = (int)gridDim.x;
        uint32_t phase = 0;
        int committed = 0;                          // boxes (bulk groups) committed so far
        bool pok = true;
        // A remote bulk store takes about 10 us until `wait_group` sees it complete (measured at 4 ranks), far longer
        // than loading a box (about 1 us), so what counts is how many boxes a CTA has in flight.  The two epilogue
        // staging buffers are cut into as many slots as boxes fit (2 of 128 rows, 4 of 64, 8 of 32): the 3-4 boxes a
        // CTA typically owns are all issued within a few microseconds, and only then does the CTA wait, group by
        // group, and report.  (Waiting for group g before issuing group g + 2 was tried: it serialised the store
        // latency, 10 us per group.)
        const int nslots = (2 * EPI_BUF_BYTES) / (int)box_bytes;
        int group_last[AG_MAX_GROUPS];              // value of `committed` after the last box of each column group
        int dealt = 0;                              // boxes dealt so far over all CTAs (round-robin start of a group)
        for (int g = 0; g < ngroups && pok; ++g) {
          const int cols_g = min(cm.ag_group_kb, col_blocks - g * cm.ag_group_kb);
          const int boxes_g = cols_g * row_blocks;
          const int start = ((int)blockIdx.x - dealt % grid + grid) % grid;
          dealt += boxes_g;
          for (int b = start; b < boxes_g; b += grid) {
            const int row = (b / cols_g) * cm.ag_push_rows;
            const int col = (g * cm.ag_group_kb + b % cols_g) * 64;
            uint8_t* buf = epi_buf + (committed % nslots) * box_bytes;
            if (committed >= nslots) {              // the stores that last read this slot: nslots - 1 newer groups may pend
              if (nslots >= 8)      asm volatile("cp.async.bulk.wait_group.read 7;" ::: "memory");
              else if (nslots >= 4) asm volatile("cp.async.bulk.wait_group.read 3;" ::: "memory");
              else                  asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            }
            mbar_expect_tx(push_bar, box_bytes);
            tma_load_2d(buf, &tmap_push, col, row, push_bar);
            if (!mbar_wait(push_bar, phase, p.status)) { pok = false; break; }
            phase ^= 1;
            if (committed == 0) trace_mark(p, 16);
            #pragma unroll 1
            for (int k = 1; k <= cm.nranks; ++k) {
              // peers first, the local copy last; rank me - 1 consumes this shard earliest (right after its own)
              int t = cm.me - k;
              if (t < 0) t += cm.nranks;
              tma_store_2d(&rsm.m[t], buf, col, cm.me * cm.rows_per_shard + row);
            }
            tma_store_commit();
            ++committed;
          }
          group_last[g] = committed;
        }
        trace_mark(p, 17);
        // then, group by group: once this CTA's boxes of the group have landed, report; the CTA that completes the
        // count publishes the group's flag on every rank
        for (int g = 0; g < ngroups && pok; ++g) {
          const int after = committed - group_last[g];      // boxes committed after the group's last one may pend
          if (after <= 0)      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
          else if (after == 1) asm volatile("cp.async.bulk.wait_group 1;" ::: "memory");
          else if (after == 2) asm volatile("cp.async.bulk.wait_group 2;" ::: "memory");
          else if (after == 3) asm volatile("cp.async.bulk.wait_group 3;" ::: "memory");
          else                 asm volatile("cp.async.bulk.wait_group 4;" ::: "memory");
          fence_proxy_async_all();
          __threadfence_system();
          if (g == 0) trace_mark(p, 18);
          const int done = atomicAdd(cm.ag_counter + g, 1) + 1;
          if (done == grid) {                       // this CTA completed the group: publish its flag on every rank
            if (g == 0) trace_mark(p, 20);
            cm.ag_counter[g] = 0;
            __threadfence_system();
            for (int t = 0; t < cm.nranks; ++t)
              st_relaxed_sys_s32(reinterpret_cast<int*>(cm.flag_ptrs.p[t]) + cm.ag_flag_base + cm.me * AG_MAX_GROUPS + g, seqv);
          }
        }
        tma_store_wait_all();
        trace_mark(p, 11);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");       // the staging buffers are free for the epilogue again
    }

    int acc = 0; uint32_t acc_phase = 0;
    bool ok = true;
    int stores_issued = 0;
    float ssq = 0.f;                               // this thread's share of sum(C^2) (mode 1 with p.sumsq)
    // reduce-scatter: tiles are visited owner by owner; when this CTA has stored its last tile for an owner it
    // reports them, and the CTA that completes an owner's count publishes the flag there: a partial block is
    // announced as soon as it has landed, not when the whole GEMM is over
    int rs_owner = -1, rs_pending = 0;
    bool rs_seen = false;
    auto rs_report = [&](int owner_, int count_) {
      if (p.direct) {                                // rows were written with ordinary stores by all epilogue threads
        __threadfence_system();
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      if (epi_tid == 0) {
        tma_store_wait_all();
        fence_proxy_async_all();
        __threadfence_system();
        const int per_owner = (cm.rows_per_owner / GEMM_BM) * p.tiles_n;
        const int done = atomicAdd(cm.rs_counters + owner_, count_) + count_;
        if (done == per_owner) {
          cm.rs_counters[owner_] = 0;
          __threadfence_system();
          st_relaxed_sys_s32(reinterpret_cast<int*>(cm.flag_ptrs.p[owner_]) + cm.rs_flag_base + cm.me, seqv);
        }
      }
    };
    Work w;
    for (int it = 0; ok && get_work(p, unit, it, kblocks, w); ++it) {
      int m0, n0;
      tile_origin<BN, PAIR>(p, cm, w.tile, cta_rank, m0, n0);
      const int owner = cm.rs ? m0 / cm.rows_per_owner : 0;
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
      if (epi_tid == 0) trace_mark(p, it == 0 ? 4 : 6);
      // ---- reduce-scatter, tiles of this rank's own rows: the other ranks' partial blocks are added right here in
      // the epilogue (they computed this rank's rows before their own, so their data is normally waiting); the first
      // such tile makes sure of it (bounded wait for the flags of all other sources)
      const bool own = cm.rs && cm.rs_out != nullptr && owner == cm.me;
      const bool own_sum = own && !cm.rs_tail;        // this epilogue adds the other sources' blocks itself
      if (own_sum && !rs_seen && ok) {
        uint32_t mine = 1u, all;
        if (epi_tid < cm.nranks && epi_tid != cm.me) {
          const int* flags = reinterpret_cast<const int*>(cm.flag_ptrs.p[cm.me]);
          mine = wait_flag(flags + cm.rs_flag_base + epi_tid, seqv, p.status) ? 1u : 0u;
        }
        asm volatile(
            "{\n\t"
            ".reg .pred p, q;\n\t"
            "setp.ne.u32 p, %1, 0;\n\t"
            "bar.red.and.pred q, 1, 128, p;\n\t"
            "selp.u32 %0, 1, 0, q;\n\t"
            "}\n"
            : "=r"(all) : "r"(mine) : "memory");
        ok = all != 0;
        rs_seen = true;
        if (epi_tid == 0) trace_mark(p, 13);
      }
      // ---- tail tiles cut along K: exchange partial sums, the slice that arrives last runs the epilogue
      bool run_epilogue = ok && m0 < p.M;
      const float* others = nullptr;       // partial sums of the other slices (this CTA's rows), null: none
      if (ok && w.nslices > 1 && p.mode != 2) {
        float* mine = p.ws + ((size_t)(w.tail * p.split + w.slice) * CTAS_PER_UNIT + cta_rank) * (GEMM_BM * BN);
        #pragma unroll 1
        for (int j = 0; j < BN / 32; ++j) {
          if (n0 + j * 32 >= p.N) break;
          uint32_t v[32];
          tmem_ld32(tmem_addr(tmem_base, q * 32, acc * BN + j * 32), v);
          tmem_ld_wait();
          if (m0 + row < p.M) {
            #pragma unroll
            for (int c = 0; c < 8; ++c)         // layout [BN / 4][128 rows][4]: a warp writes 512 contiguous bytes
              *reinterpret_cast<uint4*>(mine + ((size_t)(j * 8 + c) * GEMM_BM + row) * 4) =
                  make_uint4(v[c * 4], v[c * 4 + 1], v[c * 4 + 2], v[c * 4 + 3]);
          }
        }
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (epi_tid == 0) {
          int* ctr = p.ws_counters + w.tail * CTAS_PER_UNIT + cta_rank;
          const int ticket = atomicAdd(ctr, 1);
          const int last = ticket == w.nslices - 1;
          if (last) { *ctr = 0; __threadfence(); }
          *epi_flag = last;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        run_epilogue = run_epilogue && (*epi_flag != 0);
        others = p.ws + ((size_t)(w.tail * p.split) * CTAS_PER_UNIT + cta_rank) * (GEMM_BM * BN);
      }
      if (run_epilogue && cm.rs && !own_sum) {
        if (owner != rs_owner) {
          if (rs_pending > 0) rs_report(rs_owner, rs_pending);
          rs_owner = owner;
          rs_pending = 0;
        }
        rs_pending += 1;
      }
      float ce_m = -INFINITY, ce_s = 0.f;
      long long ce_lbl = -1;
      if (p.ce_labels != nullptr && run_epilogue && m0 + row < p.M) {
        const long long lb = p.ce_labels[m0 + row];
        ce_lbl = lb >= 0 ? lb - p.ce_vocab_start : -1;
      }
      if (run_epilogue) {
        #pragma unroll 1
        for (int j = 0; j < BN / EPI_BLOCK_COLS; ++j) {
          const int nb = n0 + j * EPI_BLOCK_COLS;
          if (nb >= p.N) break;
          uint32_t v[2][32];
          if (others == nullptr) {
            tmem_ld32(tmem_addr(tmem_base, q * 32, acc * BN + j * 64), v[0]);
            tmem_ld32(tmem_addr(tmem_base, q * 32, acc * BN + j * 64 + 32), v[1]);
            tmem_ld_wait();
          } else {
            // sum of all slices in slice order (this CTA's own partial is read back like the others), so the result
            // does not depend on which slice happened to arrive last
            #pragma unroll
            for (int h = 0; h < 2; ++h) {
              #pragma unroll
              for (int e = 0; e < 32; ++e) v[h][e] = 0u;
            }
            if (m0 + row < p.M) {                  // rows beyond M hold nothing anyone reads
              #pragma unroll
              for (int h = 0; h < 2; ++h) {
                if (nb + h * 32 >= p.N) break;
                for (int s0 = 0; s0 < w.nslices; s0 += 2) {      // two slices (16 vector loads) in flight per thread
                  float4 o[2][8];
                  #pragma unroll
                  for (int t = 0; t < 2; ++t) {
                    const float* src = others + (size_t)(s0 + t) * CTAS_PER_UNIT * (GEMM_BM * BN);
                    #pragma unroll
                    for (int c = 0; c < 8; ++c)
                      o[t][c] = (s0 + t < w.nslices)
                                    ? __ldcg(reinterpret_cast<const float4*>(src + ((size_t)(j * 16 + h * 8 + c) * GEMM_BM + row) * 4))
                                    : make_float4(0.f, 0.f, 0.f, 0.f);
                  }
                  #pragma unroll
                  for (int t = 0; t < 2; ++t) {
                    #pragma unroll
                    for (int c = 0; c < 8; ++c) {
                      v[h][c * 4 + 0] = __float_as_uint(__uint_as_float(v[h][c * 4 + 0]) + o[t][c].x);
                      v[h][c * 4 + 1] = __float_as_uint(__uint_as_float(v[h][c * 4 + 1]) + o[t][c].y);
                      v[h][c * 4 + 2] = __float_as_uint(__uint_as_float(v[h][c * 4 + 2]) + o[t][c].z);
                      v[h][c * 4 + 3] = __float_as_uint(__uint_as_float(v[h][c * 4 + 3]) + o[t][c].w);
                    }
                  }
                }
              }
            }
          }
          if (p.direct) {
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
            if (own_sum) {
              const long long r_in = (long long)(m0 - owner * cm.rows_per_owner + row);
              for (int src_rank = 0; src_rank < cm.nranks; ++src_rank) {      // fixed order: reproducible sums
                if (src_rank == cm.me) continue;
                const __nv_bfloat16* src = cm.rs_land_local + src_rank * cm.rs_slot_stride + r_in * cm.rs_land_ld + nb;
                uint4 u[8];
                #pragma unroll
                for (int c = 0; c < 8; ++c)
                  u[c] = (nb + c * 8 < p.N) ? __ldcg(reinterpret_cast<const uint4*>(src + c * 8)) : make_uint4(0u, 0u, 0u, 0u);
                #pragma unroll
                for (int c = 0; c < 8; ++c) {
                  const uint32_t pk[4] = {u[c].x, u[c].y, u[c].z, u[c].w};
                  #pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    uint32_t& lo = v[c >> 2][(c & 3) * 8 + 2 * e];
                    uint32_t& hi = v[c >> 2][(c & 3) * 8 + 2 * e + 1];
                    lo = __float_as_uint(__uint_as_float(lo) + bf16_lo(pk[e]));
                    hi = __float_as_uint(__uint_as_float(hi) + bf16_hi(pk[e]));
                  }
                }
              }
            }
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
                  if (p.ce_labels != nullptr) {
                    // statistics of the values the consumer of C will read: the bf16-rounded logits
                    const uint32_t pk[4] = {o.x, o.y, o.z, o.w};
                    float mx = ce_m;
                    #pragma unroll
                    for (int e = 0; e < 8; ++e) {
                      const int col = nb + h * 32 + c * 8 + e;
                      const float x = (e & 1) ? bf16_hi(pk[e >> 1]) : bf16_lo(pk[e >> 1]);
                      if (col < p.N) mx = fmaxf(mx, x);
                    }
                    if (mx > ce_m) { ce_s *= __expf(ce_m - mx); ce_m = mx; }
                    #pragma unroll
                    for (int e = 0; e < 8; ++e) {
                      const int col = nb + h * 32 + c * 8 + e;
                      const float x = (e & 1) ? bf16_hi(pk[e >> 1]) : bf16_lo(pk[e >> 1]);
                      if (col < p.N) {
                        ce_s += __expf(x - ce_m);
                        if ((long long)col == ce_lbl) p.ce_tgt[m0 + row] = x;
                      }
                    }
                  }
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
              else if (own) tma_store_2d(&tmap_c, buf, nb, m0 - owner * cm.rows_per_owner);     // reduced block
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
        if (p.ce_labels != nullptr && m0 + row < p.M) {
          const size_t o = (size_t)(n0 / BN) * p.M + (m0 + row);
          p.ce_max[o] = ce_m;
          p.ce_sum[o] = ce_s;
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (epi_tid == 0) trace_mark(p, it == 0 ? 5 : 7);
      if (lane == 0) {
        if (PAIR) mbar_arrive_cluster(smem_u32(&tempty_bar[acc]) & PAIR_LEADER_MASK);
        else mbar_arrive(&tempty_bar[acc]);
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      if (cm.rs && ok && rs_pending > 0) {
        // last tile of this CTA for the current owner?  then report it now, while the next tile's main loop runs
        Work nw;
        int next_owner = -1;
        if (get_work(p, unit, it + 1, kblocks, nw)) {
          int nm0, nn0;
          tile_origin<BN, PAIR>(p, cm, nw.tile, cta_rank, nm0, nn0);
          next_owner = nm0 / cm.rows_per_owner;
        }
        if (next_owner != rs_owner) { rs_report(rs_owner, rs_pending); rs_pending = 0; }
      }
    }
    if (p.sumsq != nullptr && p.mode == 1) {
      #pragma unroll
      for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
      if (lane == 0) atomicAdd(p.sumsq, ssq);
    }
    if (cm.rs && ok && rs_pending > 0) rs_report(rs_owner, rs_pending);
    if (epi_tid == 0) {
      tma_store_wait_all();
      trace_mark(p, 14);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (cm.rs && cm.rs_out != nullptr && cm.rs_tail) {
    // ------------------------------------------------------------------ reduce-scatter tail (more than two ranks)
    // rs_out holds this rank's own partial block; every CTA adds a slice of the T - 1 blocks that the other sources
    // stored into this rank's landing zone.  The wait is for flags only.
    if ((int)threadIdx.x < cm.nranks) {
      const int* flags = reinterpret_cast<const int*>(cm.flag_ptrs.p[cm.me]);
      if (!wait_flag(flags + cm.rs_flag_base + threadIdx.x, seqv, p.status)) *epi_flag = -1;
    }
    __syncthreads();
    if (threadIdx.x == 0) trace_mark(p, 13);
    if (*epi_flag != -1) {
      const int vec_per_row = p.N / 8;
      const long long total = (long long)cm.rows_per_owner * vec_per_row;
      const long long stride = (long long)gridDim.x * GEMM_THREADS;
      constexpr int U = 4;                       // vectors in flight per thread and source
      for (long long i0 = (long long)blockIdx.x * GEMM_THREADS + threadIdx.x; i0 < total; i0 += stride * U) {
        float a[U][8];
        long long off_in[U], off_out[U];
        #pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + u * stride;
          const long long r = i / vec_per_row;
          const int c = (int)(i - r * vec_per_row) * 8;
          off_in[u] = r * cm.rs_land_ld + c;
          off_out[u] = r * cm.rs_out_ld + c;
        }
        for (int s = -1; s < cm.nranks; ++s) {     // own partial first, then the sources in rank order: reproducible
          if (s == cm.me) continue;
          uint4 v[U];
          #pragma unroll
          for (int u = 0; u < U; ++u)
            if (i0 + u * stride < total)
              v[u] = __ldcg(reinterpret_cast<const uint4*>(s < 0 ? cm.rs_out + off_out[u]
                                                                   : cm.rs_land_local + s * cm.rs_slot_stride + off_in[u]));
          #pragma unroll
          for (int u = 0; u < U; ++u) {
            if (i0 + u * stride < total) {
              if (s < 0) {
                a[u][0] = bf16_lo(v[u].x); a[u][1] = bf16_hi(v[u].x); a[u][2] = bf16_lo(v[u].y); a[u][3] = bf16_hi(v[u].y);
                a[u][4] = bf16_lo(v[u].z); a[u][5] = bf16_hi(v[u].z); a[u][6] = bf16_lo(v[u].w); a[u][7] = bf16_hi(v[u].w);
              } else {
                a[u][0] += bf16_lo(v[u].x); a[u][1] += bf16_hi(v[u].x); a[u][2] += bf16_lo(v[u].y); a[u][3] += bf16_hi(v[u].y);
                a[u][4] += bf16_lo(v[u].z); a[u][5] += bf16_hi(v[u].z); a[u][6] += bf16_lo(v[u].w); a[u][7] += bf16_hi(v[u].w);
              }
            }
          }
        }
        #pragma unroll
        for (int u = 0; u < U; ++u) {
          if (i0 + u * stride < total) {
            uint4 o;
            o.x = pack_bf16(a[u][0], a[u][1]); o.y = pack_bf16(a[u][2], a[u][3]);
            o.z = pack_bf16(a[u][4], a[u][5]); o.w = pack_bf16(a[u][6], a[u][7]);
            *reinterpret_cast<uint4*>(cm.rs_out + off_out[u]) = o;
          }
        }
      }
    }
  }
  if (threadIdx.x == 0) trace_mark(p, 10);
  if (PAIR) {
    // neither CTA may leave (or free TMEM) while its partner can still signal its barriers or read its shared memory
    tc_fence_before_sync();
    cluster_sync_all();
    if (warp == 1) tmem_dealloc_pair(tmem_base, TMEM_COLS);
  } else {
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------ host
static int g_num_sms = 0;
static unsigned long long* g_trace = nullptr;

static int env_int(const char* name, int dflt) {
  const char* e = getenv(name);
  return e ? atoi(e) : dflt;
}
// SSM_GEMM_DUAL=0 goes back to one producer thread for all loads of a stage.
static int gemm_dual_producers() {
  static int v = -1;
  if (v < 0) v = env_int("SSM_GEMM_DUAL", 1) ? 1 : 0;
  return v;
}
// SSM_GEMM_EPI=direct makes the epilogue warps store their rows straight from registers instead of staging them in
// shared memory for a TMA store (measured slower; kept for experiments).
static int epilogue_direct() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("SSM_GEMM_EPI");
    v = (e && strcmp(e, "direct") == 0) ? 1 : 0;
  }
  return v;
}
// Scheduling options: environment defaults (SSM_GEMM_PAIR=0|1|2: never / by cost / whenever possible use CTA pairs;
// SSM_GEMM_SPLIT=0|1|2: never / where it pays / wherever possible cut tail tiles along K; SSM_GEMM_FORCE_BN=128|192|256: tile width), overridden at run time
// by ssm_gemm_set_options (tests and benchmarks).
static int g_opt_pair = -1, g_opt_split = -1, g_opt_bn = -1;
static int gemm_pair_mode() {
  if (g_opt_pair < 0) g_opt_pair = env_int("SSM_GEMM_PAIR", 1);
  return g_opt_pair;
}
static int gemm_pairs_enabled() { return gemm_pair_mode() != 0; }
static int gemm_split_enabled() {
  if (g_opt_split < 0) { g_opt_split = env_int("SSM_GEMM_SPLIT", 1); if (g_opt_split < 0 || g_opt_split > 2) g_opt_split = 1; }
  return g_opt_split;
}
static int gemm_forced_bn() {
  if (g_opt_bn < 0) g_opt_bn = env_int("SSM_GEMM_FORCE_BN", 0);
  return g_opt_bn;
}

// Scratch for the split tail (allocated once per device, on first use): partial sums and arrival counters.
struct Scratch { float* ws; int* counters; };
static Scratch g_scratch[16] = {};
static int scratch_for_current_device(Scratch* out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return -1;
  if (g_scratch[dev].ws == nullptr) {
    const size_t ws_bytes = (size_t)MAX_UNITS * 2 * GEMM_BM * 256 * sizeof(float);   // one slice per CTA and launch
    void* a = nullptr; void* b = nullptr;
    if (cudaMalloc(&a, ws_bytes) != cudaSuccess) return -1;
    if (cudaMalloc(&b, MAX_UNITS * 2 * sizeof(int)) != cudaSuccess) { cudaFree(a); return -1; }
    if (cudaMemset(b, 0, MAX_UNITS * 2 * sizeof(int)) != cudaSuccess) { cudaFree(a); cudaFree(b); return -1; }
    g_scratch[dev].ws = reinterpret_cast<float*>(a);
    g_scratch[dev].counters = reinterpret_cast<int*>(b);
  }
  *out = g_scratch[dev];
  return 0;
}

struct TileChoice { int bn; int pair; };

// Tile shape.  The cost of a tiling is (full waves + the split tail) x time of one tile; tile times relative to a
// 128 x 256 single-CTA tile are measured values (a CTA's main loop is bound by the operand bytes it pulls per
// k-block: 48 KB for 128x256, 32 KB for a 128x128 tile or for its half of a 256x256 pair tile, 24 KB for its half
// of a 256x128 pair tile).  SSM_GEMM_FORCE_BN=128|192|256 and SSM_GEMM_PAIR=0|1|2 (2 = always) override.
// K slices for the `rem` tiles left after the full waves (or for all tiles when there are fewer tiles than units).
// Cutting a tile into s slices saves (1 - 1/s) of its main loop but adds the exchange of partial sums: every slice
// writes its fp32 block to scratch and the last arriver reads the others back, a latency-bound pass measured at
// 8-10 us for a 256 x 256 pair tile (2320 x 4096 x 2048 fp32 out: 59.5 us with the split, 51.7 us without), half of
// that for a 128-row tile.  Accumulate mode adds its slices into C directly and has no read-back.  Costs are in units
// of one single-CTA 128 x 256 k-block (about 0.42 us); the split is taken only where it pays.
static int tail_split(long long rem, int units, int kblocks, int mode, int pair, double cost_kb, double* exchange) {
  if (exchange) *exchange = 0.0;
  if (rem <= 0) return 1;
  int split = (int)(units / rem);
  const int cap = mode == 2 ? MAX_SPLIT : 4;
  if (split > cap) split = cap;
  if (split > kblocks / 4) split = kblocks / 4;
  if (split <= 1) return 1;
  const double exch = mode == 2 ? 4.0 : (pair ? 22.0 : 12.0);
  if (gemm_split_enabled() != 2 && (1.0 - 1.0 / split) * kblocks * cost_kb <= exch) return 1;   // 2: split wherever possible
  if (exchange) *exchange = exch;
  return split;
}

static double tile_cost_kb(int bn, int pair) {
  // cost of one tile per k-block, relative to the single-CTA 128 x 256 tile
  if (pair) return bn == 256 ? 0.68 : 0.52;
  return bn == 256 ? 1.00 : 0.80;
}

// Work distribution of one launch: `units` CTAs (or CTA pairs) take the whole tiles [0, full_tiles) round-robin; the
// `rem` tiles after them are cut into `split` K slices each, one slice per unit.  With fewer tiles than units all
// tiles are tail tiles and only the units that get a slice are launched.
struct Schedule { int units, full_tiles, rem, split; };
static Schedule plan_schedule(int tiles, int max_units, int kblocks, int mode, int pair, int bn) {
  Schedule s;
  s.units = tiles < max_units ? tiles : max_units;
  s.full_tiles = (tiles / s.units) * s.units;
  s.rem = tiles - s.full_tiles;
  s.split = 1;
  if (gemm_split_enabled() && (s.rem > 0 || tiles < max_units)) {
    if (tiles < max_units) { s.units = max_units; s.full_tiles = 0; s.rem = tiles; }
    s.split = tail_split(s.rem, s.units, kblocks, mode, pair, tile_cost_kb(bn, pair), nullptr);
    if (tiles < max_units) s.units = s.rem * s.split;
  }
  return s;
}

static TileChoice pick_tile(int M, int N, int K, int b_mn, int allow_pair, int mode = 0) {
  const int forced_bn = gemm_forced_bn(), forced_pair = gemm_pair_mode();
  const int sms = g_num_sms > 0 ? g_num_sms : 148;
  const int kblocks = (K + GEMM_BK - 1) / GEMM_BK;
  struct Cand { int bn, pair; double cost; };
  const Cand cands[5] = {{256, 0, tile_cost_kb(256, 0)}, {192, 0, tile_cost_kb(192, 0)}, {128, 0, tile_cost_kb(128, 0)},
                         {256, 1, tile_cost_kb(256, 1)}, {128, 1, tile_cost_kb(128, 1)}};
  TileChoice best = {256, 0};
  double best_t = 1e30;
  for (const Cand& c : cands) {
    if (c.pair && (!allow_pair || forced_pair == 0 || M <= 128)) continue;
    if (!c.pair && forced_pair == 2 && allow_pair && M > 128) continue;
    if (forced_bn && c.bn != forced_bn) continue;
    if (c.bn > 128 && N <= 128) continue;
    const int tile_m = c.pair ? 256 : 128;
    const int units = c.pair ? sms / 2 : sms;
    const long long tiles = (long long)((M + tile_m - 1) / tile_m) * ((N + c.bn - 1) / c.bn);
    const long long full = tiles / units, rem = tiles % units;
    double waves = (double)full, exchange = 0.0;
    if (tiles < units) {
      waves = 1.0 / tail_split(tiles, units, kblocks, mode, c.pair, c.cost, &exchange);
    } else if (rem) {
      waves += 1.0 / tail_split(rem, units, kblocks, mode, c.pair, c.cost, &exchange);
    }
    // per-tile fixed cost (pipeline fill, epilogue tail) in k-block units
    const double t = waves * (kblocks * c.cost + 6.0) + exchange;
    if (t < best_t) { best_t = t; best = {c.bn, c.pair}; }
  }
  (void)b_mn;
  return best;
}

template <int BN, int STAGES, bool PAIR>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, GemmParams p,
                       cudaStream_t stream, const GemmComm* comm = nullptr, const RsMaps* maps = nullptr,
                       const CUtensorMap* ta_local = nullptr, const CUtensorMap* ta_push = nullptr) {
  using L = GemmSmem<BN, STAGES, PAIR>;
  static bool configured = false;
  auto kern = gemm_bf16_tcgen05<BN, STAGES, PAIR>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  constexpr int TILE_M = PAIR ? 256 : 128;
  p.tiles_m = (p.M + TILE_M - 1) / TILE_M;
  p.tiles_n = (p.N + BN - 1) / BN;
  const int tiles = p.tiles_m * p.tiles_n;
  static GemmComm no_comm;       // zero-initialised: no fusion
  static RsMaps no_maps;
  GemmComm cm = comm ? *comm : no_comm;
  int max_units = PAIR ? g_num_sms / 2 : g_num_sms;
  if (PAIR) {
    // every CTA of the grid must be resident at once (CTAs of different ranks wait for one another's pushes)
    static int max_clusters = -1;
    if (max_clusters < 0) {
      cudaLaunchConfig_t q = {};
      q.gridDim = dim3((unsigned)g_num_sms, 1, 1);
      q.blockDim = dim3(GEMM_THREADS, 1, 1);
      q.dynamicSmemBytes = L::TOTAL;
      cudaLaunchAttribute qa[1];
      qa[0].id = cudaLaunchAttributeClusterDimension;
      qa[0].val.clusterDim.x = 2; qa[0].val.clusterDim.y = 1; qa[0].val.clusterDim.z = 1;
      q.attrs = qa; q.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &q) != cudaSuccess || n < 1) n = g_num_sms / 2;
      max_clusters = n;
    }
    if (max_units > max_clusters) max_units = max_clusters;
  }
  if (max_units > MAX_UNITS) max_units = MAX_UNITS;
  const int kblocks = (p.K + GEMM_BK - 1) / GEMM_BK;
  Schedule sc = plan_schedule(tiles, max_units, kblocks, p.mode, PAIR ? 1 : 0, BN);
  p.ws = nullptr; p.ws_counters = nullptr;
  if (sc.split > 1 && p.mode != 2) {             // slices exchange fp32 partial sums through a per-device scratch buffer
    Scratch s;
    if (scratch_for_current_device(&s) != 0) {
      if (tiles < max_units) sc.units = sc.rem;   // no scratch: whole tail tiles, one per unit
      sc.split = 1;
    } else {
      p.ws = s.ws; p.ws_counters = s.counters;
    }
  }
  const int units = sc.units;
  p.full_tiles = sc.full_tiles; p.rem = sc.rem; p.split = sc.split;
  p.units = units;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(units * (PAIR ? 2 : 1)), 1, 1);
  cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = L::TOTAL;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = PAIR ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ta, tb, tc, ta_local ? *ta_local : ta, ta_push ? *ta_push : ta, p, cm,
                                     maps ? *maps : no_maps);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaGetLastError();
}

}  // namespace ssm

struct GemmExtra {                     // optional outputs of ssm_gemm_bf16_ex2
  const void* ce_labels; long long ce_vocab_start; void* ce_max; void* ce_sum; void* ce_tgt;
};

static int gemm_bf16_impl(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                          long long ldc, int a_mn, int b_mn, int mode, const void* bias, int act, int* status,
                          cudaStream_t stream, float* sumsq, const GemmExtra* extra, const ssm::GemmComm* comm,
                          const void* const* land_ptrs, long long land_ld, int* tiles_n_out);

// C[M,N] = A * B.  a_mn = 0: A is [M,K] with row stride lda; a_mn = 1: A is [K,M] with row stride lda.
// b_mn = 0: B is [N,K] with row stride ldb; b_mn = 1: B is [K,N] with row stride ldb.
// mode 0: C bf16 [M, ldc] (ldc * 2 bytes must be a multiple of 16); 1: C fp32 store; 2: C fp32 += .
// All leading dimensions in elements; operand bases 16-byte aligned, operand row strides multiples of 8.
extern "C" int ssm_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                             long long ldb, long long ldc, int a_mn, int b_mn, int mode, const void* bias, int act,
                             int* status, cudaStream_t stream) {
  return gemm_bf16_impl(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, mode, bias, act, status, stream, nullptr, nullptr,
                        nullptr, nullptr, 0, nullptr);
}

// Same, and with mode 1 (fp32 store) the sum of squares of the stored matrix is added to *sumsq (fp32, device):
// the wgrad GEMM then delivers its share of the global gradient norm without a second pass over the gradient.
extern "C" int ssm_gemm_bf16_ex(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                long long ldb, long long ldc, int a_mn, int b_mn, int mode, const void* bias, int act,
                                int* status, cudaStream_t stream, void* sumsq) {
  if (sumsq != nullptr && mode != 1) return -SSM_ERR_BAD_ARG;
  return gemm_bf16_impl(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, mode, bias, act, status, stream,
                        reinterpret_cast<float*>(sumsq), nullptr, nullptr, nullptr, 0, nullptr);
}

// Number of column tiles the kernel will use for an [M, N] x K product with K-major operands: the leading extent of
// the per-tile cross-entropy statistics that ssm_gemm_bf16_ce / the fused variant write.
// (rows_per_shard: shard rows of the all-gather variant, 0 for the plain GEMM).
extern "C" int ssm_gemm_ce_tiles(int M, int N, int K, int rows_per_shard) {
  using namespace ssm;
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const TileChoice c = pick_tile(M, N, K, 0, gemm_pairs_enabled() && rows_per_shard % 256 == 0);
  return (N + c.bn - 1) / c.bn;
}

// The tiling and work distribution that a plain GEMM of this shape gets, without launching anything (host only; also
// callable without a GPU, where 148 SMs are assumed): out[8] = {tile width BN, 1 if CTA-pair tiles, tiles along M,
// tiles along N, units launched, whole tiles in the full waves, tail tiles, K slices per tail tile}.
// mode as in ssm_gemm_bf16 (2 = accumulate).  For debugging, tests of the schedule and `kernel_bench gemm --plan`.
extern "C" int ssm_gemm_plan(int M, int N, int K, int mode, int allow_pair, int* out) {
  using namespace ssm;
  if (M <= 0 || N <= 0 || K <= 0 || out == nullptr) return -SSM_ERR_BAD_ARG;
  const int sms = g_num_sms > 0 ? g_num_sms : 148;
  const TileChoice c = pick_tile(M, N, K, 0, allow_pair && gemm_pairs_enabled(), mode);
  const int tile_m = c.pair ? 256 : 128;
  const int tiles_m = (M + tile_m - 1) / tile_m, tiles_n = (N + c.bn - 1) / c.bn;
  int max_units = c.pair ? sms / 2 : sms;
  if (max_units > MAX_UNITS) max_units = MAX_UNITS;
  const Schedule sc = plan_schedule(tiles_m * tiles_n, max_units, (K + GEMM_BK - 1) / GEMM_BK, mode, c.pair, c.bn);
  out[0] = c.bn; out[1] = c.pair; out[2] = tiles_m; out[3] = tiles_n;
  out[4] = sc.units; out[5] = sc.full_tiles; out[6] = sc.rem; out[7] = sc.split;
  return 0;
}

// bf16 GEMM (mode 0, no bias / activation) whose epilogue also emits cross-entropy statistics of the rows of C:
// ce_max / ce_sum [tiles_n][M] (maximum and sum of exp(x - max) over the tile's columns, from the bf16-rounded
// values) and ce_tgt[row] = C[row, labels[row] - vocab_start] where that column exists (other rows untouched).
extern "C" int ssm_gemm_bf16_ce(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                long long ldb, long long ldc, int* status, cudaStream_t stream, const void* labels,
                                long long vocab_start, void* ce_max, void* ce_sum, void* ce_tgt) {
  GemmExtra ex = {labels, vocab_start, ce_max, ce_sum, ce_tgt};
  return gemm_bf16_impl(A, B, C, M, N, K, lda, ldb, ldc, 0, 0, 0, nullptr, 0, status, stream, nullptr, &ex, nullptr,
                        nullptr, 0, nullptr);
}

static int gemm_bf16_impl(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                          long long ldc, int a_mn, int b_mn, int mode, const void* bias, int act, int* status,
                          cudaStream_t stream, float* sumsq, const GemmExtra* extra, const ssm::GemmComm* comm,
                          const void* const* land_ptrs, long long land_ld, int* tiles_n_out) {
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
  // the collective variants walk the tiles block by block (rows of one shard / owner): pair tiles need whole blocks
  int allow_pair = gemm_pairs_enabled();
  if (comm != nullptr && comm->ag && comm->rows_per_shard % 256) allow_pair = 0;
  if (comm != nullptr && comm->rs && comm->rows_per_owner % 256) allow_pair = 0;
  const TileChoice tcw = pick_tile(M, N, K, b_mn, allow_pair, mode);
  const int BN = tcw.bn;
  const bool pair = tcw.pair != 0;
  if (tiles_n_out) *tiles_n_out = (N + BN - 1) / BN;
  const uint32_t b_rows = pair ? BN / 2 : BN;
  CUtensorMap ta, tb, tc, ta_local;
  int r;
  if (!a_mn) r = make_tmap_2d_bf16(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, 64, 128);
  else       r = make_tmap_2d_bf16(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, 64, 64);
  if (r) return -100 - r;
  if (!b_mn) r = make_tmap_2d_bf16(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, 64, b_rows);
  else       r = make_tmap_2d_bf16(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, 64);
  if (r) return -200 - r;
  if (mode == 0) {
    r = make_tmap_2d_bf16(&tc, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc * 2, 64, 128);
    if (r) return -300 - r;
  } else if (mode == 1 || mode == 2) {
    if ((ldc % 4) || (reinterpret_cast<uintptr_t>(C) & 15)) return -SSM_ERR_BAD_ARG;
    r = make_tmap_2d(&tc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc * 4, 32, 128);
    if (r) return -300 - r;
  } else if (comm != nullptr && comm->rs && comm->rs_out != nullptr) {
    r = make_tmap_2d_bf16(&tc, comm->rs_out, (uint64_t)N, (uint64_t)comm->rows_per_owner, (uint64_t)comm->rs_out_ld * 2, 64, 128);
    if (r) return -300 - r;
  } else {
    tc = ta;
  }
  ta_local = ta;
  RsMaps maps;
  memset(&maps, 0, sizeof(maps));
  CUtensorMap ta_push = ta;
  GemmComm cm_local;
  if (comm != nullptr) cm_local = *comm;
  if (comm != nullptr && comm->ag) {
    r = make_tmap_2d_bf16(&ta_local, comm->ag_src, (uint64_t)K, (uint64_t)comm->rows_per_shard,
                          (uint64_t)comm->ag_src_ld * 2, 64, 128);
    if (r) return -500 - r;
    // push boxes: as tall as possible while every CTA still gets about one box per column group
    const int col_blocks = (K + GEMM_BK - 1) / GEMM_BK;
    int push_rows = 128;
    while (push_rows > 32 && (long long)(comm->rows_per_shard / push_rows) * col_blocks < 3LL * g_num_sms) push_rows /= 2;
    cm_local.ag_push_rows = push_rows;
    r = make_tmap_2d_bf16(&ta_push, comm->ag_src, (uint64_t)K, (uint64_t)comm->rows_per_shard,
                          (uint64_t)comm->ag_src_ld * 2, 64, (uint32_t)push_rows);
    if (r) return -500 - r;
    for (int t = 0; t < comm->nranks; ++t) {      // every rank's gather buffer: destinations of the shard push
      r = make_tmap_2d_bf16(&maps.m[t], comm->ag_dst.p[t], (uint64_t)K, (uint64_t)M, (uint64_t)comm->ag_dst_ld * 2, 64,
                            (uint32_t)push_rows);
      if (r) return -600 - r;
    }
    comm = &cm_local;
  }
  if (comm != nullptr && comm->rs) {
    for (int t = 0; t < comm->nranks; ++t) {
      r = make_tmap_2d_bf16(&maps.m[t], land_ptrs[t], (uint64_t)N, (uint64_t)comm->rows_per_owner, (uint64_t)land_ld * 2, 64, 128);
      if (r) return -400 - r;
    }
  }
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K; p.a_mn = a_mn; p.b_mn = b_mn; p.mode = mode; p.act = act;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.c32 = (mode == 1 || mode == 2) ? reinterpret_cast<float*>(C) : nullptr;
  p.ldc32 = ldc; p.status = status;
  p.c16 = mode == 0 ? reinterpret_cast<__nv_bfloat16*>(C) : nullptr;
  p.ldc16 = ldc; p.direct = epilogue_direct(); p.trace = g_trace; p.sumsq = sumsq;
  p.dual = gemm_dual_producers();
  if (sumsq != nullptr || mode == 3) p.direct = 0;   // sum of squares / peer stores go through the staged epilogue
  if (extra != nullptr && extra->ce_labels != nullptr) {
    if (mode != 0 || bias != nullptr || act != 0) return -SSM_ERR_BAD_ARG;
    p.direct = 0;
    p.ce_labels = reinterpret_cast<const long long*>(extra->ce_labels);
    p.ce_vocab_start = extra->ce_vocab_start;
    p.ce_max = reinterpret_cast<float*>(extra->ce_max);
    p.ce_sum = reinterpret_cast<float*>(extra->ce_sum);
    p.ce_tgt = reinterpret_cast<float*>(extra->ce_tgt);
  }
  const RsMaps* mp = (comm != nullptr && (comm->rs || comm->ag)) ? &maps : nullptr;
  if (pair) {
    if (BN == 256) return launch_gemm<256, 6, true>(ta, tb, tc, p, stream, comm, mp, &ta_local, &ta_push);
    return launch_gemm<128, 8, true>(ta, tb, tc, p, stream, comm, mp, &ta_local, &ta_push);
  }
  if (BN == 256) return launch_gemm<256, 4, false>(ta, tb, tc, p, stream, comm, mp, &ta_local, &ta_push);
  if (BN == 192) return launch_gemm<192, 4, false>(ta, tb, tc, p, stream, comm, mp, &ta_local, &ta_push);
  return launch_gemm<128, 6, false>(ta, tb, tc, p, stream, comm, mp, &ta_local, &ta_push);
}

// GEMM fused with a tensor-parallel collective over peer memory (see GemmComm).
//   ag = 1: A must be this rank's gather buffer [nranks * rows_per_shard, K] (= ag_dst_ptrs[me], row stride
//           ag_dst_ld); ag_src is the local shard [rows_per_shard, K]; flag_ptrs[t] is rank t's flag array; the
//           ready flags of this call are flag_ptrs[t][ag_flag_base + source * 4 + column group]; ag_counter points at
//           4 local ints that are zero between launches.
//   rs = 1: mode is forced to 3; land_ptrs[o] is the base of the [rows_per_owner, N] slot this rank owns inside
//           rank o's landing zone (row stride land_ld); C is ignored.  With rs_out the kernel also reduces: the
//           partial blocks of the other sources are read from this rank's landing zone (rs_land_local: [nranks]
//           slots, rs_slot_stride elements apart) and the sum goes to rs_out [rows_per_owner, N] (row stride
//           rs_out_ld); N % 8 == 0 then.
//   ce_labels: as in ssm_gemm_bf16_ce (all-gather + LM head).
// rows_per_shard / rows_per_owner must be multiples of 128 and M = nranks * rows.
extern "C" int ssm_gemm_bf16_fused(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                   long long ldb, long long ldc, int a_mn, int b_mn, int mode, const void* bias,
                                   int act, int* status, cudaStream_t stream, int nranks, int me, int seq,
                                   const int* seq_base, const void* const* flag_ptrs, int ag, int rows_per_shard,
                                   int ag_flag_base, const void* ag_src, long long ag_src_ld,
                                   const void* const* ag_dst_ptrs, long long ag_dst_ld, int* ag_counter, int rs,
                                   int rows_per_owner, int rs_flag_base, const void* const* land_ptrs,
                                   long long land_ld, int* rs_counters, const void* rs_land_local,
                                   long long rs_slot_stride, void* rs_out, long long rs_out_ld, const void* ce_labels,
                                   long long ce_vocab_start, void* ce_max, void* ce_sum, void* ce_tgt) {
  using namespace ssm;
  if (M <= 0 || N <= 0 || K <= 0 || nranks < 1 || nranks > MAX_RANKS || me < 0 || me >= nranks) return -SSM_ERR_BAD_ARG;
  if (ag && (a_mn || rows_per_shard % GEMM_BM || (long long)rows_per_shard * nranks != M || K % 8 ||
             ag_src_ld % 8 || ag_dst_ld % 8 || (reinterpret_cast<uintptr_t>(ag_src) & 15)))
    return -SSM_ERR_BAD_ARG;
  if (rs && (rows_per_owner % GEMM_BM || (long long)rows_per_owner * nranks != M || land_ld % 8)) return -SSM_ERR_BAD_ARG;
  if (rs && rs_out != nullptr && (N % 8 || rs_out_ld % 8 || rs_slot_stride % 8)) return -SSM_ERR_BAD_ARG;
  if (rs) mode = 3;
  GemmComm cm;
  memset(&cm, 0, sizeof(cm));
  cm.nranks = nranks; cm.me = me; cm.seq = seq; cm.seq_base = seq_base;
  for (int t = 0; t < MAX_RANKS; ++t) cm.flag_ptrs.p[t] = t < nranks ? const_cast<void*>(flag_ptrs[t]) : nullptr;
  if (ag) {
    cm.ag = 1; cm.rows_per_shard = rows_per_shard; cm.ag_flag_base = ag_flag_base;
    // at most AG_MAX_GROUPS column groups per shard, each a whole number of 64-column blocks
    const int col_blocks = (K + GEMM_BK - 1) / GEMM_BK;
    cm.ag_group_kb = (col_blocks + AG_MAX_GROUPS - 1) / AG_MAX_GROUPS;
    cm.ag_cols = K; cm.ag_flags = reinterpret_cast<const int*>(flag_ptrs[me]);
    cm.ag_src = reinterpret_cast<const __nv_bfloat16*>(ag_src); cm.ag_src_ld = ag_src_ld;
    for (int t = 0; t < MAX_RANKS; ++t) cm.ag_dst.p[t] = t < nranks ? const_cast<void*>(ag_dst_ptrs[t]) : nullptr;
    cm.ag_dst_ld = ag_dst_ld; cm.ag_counter = ag_counter;
  }
  if (rs) {
    cm.rs = 1; cm.rows_per_owner = rows_per_owner; cm.rs_flag_base = rs_flag_base; cm.rs_counters = rs_counters;
    cm.rs_land_ld = land_ld;
    for (int t = 0; t < nranks; ++t) cm.rs_land.p[t] = const_cast<void*>(land_ptrs[t]);
    cm.rs_land_local = reinterpret_cast<const __nv_bfloat16*>(rs_land_local);
    cm.rs_slot_stride = rs_slot_stride;
    cm.rs_out = reinterpret_cast<__nv_bfloat16*>(rs_out); cm.rs_out_ld = rs_out_ld;
    cm.rs_tail = env_int("SSM_RS_TAIL", nranks > 2 ? 1 : 0) ? 1 : 0;
  }
  GemmExtra ex = {ce_labels, ce_vocab_start, ce_max, ce_sum, ce_tgt};
  return gemm_bf16_impl(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, mode, bias, act, status, stream, nullptr,
                        ce_labels != nullptr ? &ex : nullptr, &cm, land_ptrs, land_ld, nullptr);
}

// pair: 0 never / 1 by cost / 2 whenever possible use CTA-pair tiles; split: 0/1 K-split of tail tiles; bn: 0 (by cost)
// or 128 / 192 / 256.  A negative value leaves that option as it is.
extern "C" int ssm_gemm_set_options(int pair, int split, int bn) {
  if (pair >= 0) ssm::g_opt_pair = pair;
  if (split >= 0) ssm::g_opt_split = split > 2 ? 1 : split;
  if (bn >= 0) ssm::g_opt_bn = bn;
  return 0;
}

// Pipeline analysis: buf = device array of gridDim * GEMM_TRACE_SLOTS (24) uint64 (or null to switch tracing off).  Slots (ns, global
// timer): 0 CTA set-up done, 8 first TMA load issued, 1 first stage landed, 2/3 MMAs of the first / a later tile
// issued, 4/6 first / later accumulator complete (seen by the epilogue), 5/7 epilogue of that tile done, 9 producer
// finished, 10 CTA done (after the reduce-scatter tail); collective variants: 11 all-gather push finished, 12 first
// wait for a remote row group over, 13 reduce-scatter tail: flags of all sources seen, 14 epilogue warps done with
// their tiles (stores complete, flags published); all-gather push thread: 16 first box in shared memory, 17 all boxes
// issued, 18 own boxes of column group 0 complete, 20 flag of group 0 published (only the CTA that completed the count).
extern "C" int ssm_gemm_set_trace(void* buf) {
  ssm::g_trace = reinterpret_cast<unsigned long long*>(buf);
  return 0;
}
