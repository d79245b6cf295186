// Causal grouped-query flash attention for sm_100a, head_dim 128, forward and backward, on tcgen05.
//   forward  : one CTA per (128-query tile, query head, batch); K/V tiles of 128 keys arrive by TMA (double
//              buffered); S = Q K^T and P V run on tcgen05 with TMEM accumulators; thread i owns query row i, so
//              the online softmax needs no cross-thread reductions; O stays in registers until the end.
//   backward : one CTA per (128-key tile, kv head, batch) walks the query heads of its group and the query tiles
//              at or below the diagonal; dK and dV accumulate in TMEM over the whole walk (deterministic), dQ is
//              added to an fp32 buffer with red.add.
// K/V heads are indexed (kv head = q head / ratio), never replicated in memory (the reference materialises
// repeat_kv before its NKI flash kernel: mamba2hybrid/mamba2hybrid_attn.py:440-447).
// q [B*L, Hq*128], k/v [B*L, Hkv*128], out [B*L, Hq*128], lse [B, Hq, L] (natural log, of scaled scores).
#include "common.cuh"

namespace ssm {

constexpr int AT = 128;                  // tile (queries / keys)
constexpr int AD = 128;                  // head dim
constexpr int ATILE = AT * AD * 2;       // bytes of one [128][128] bf16 tile (two 16 KiB swizzle blocks)
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint64_t adesc_k(uint32_t base, int kk) {     // K-major, two 64-wide atoms
  return make_smem_desc_sw128(base + (kk >> 2) * (ATILE / 2) + (kk & 3) * 32, 16, 1024);
}
__device__ __forceinline__ uint64_t adesc_mn(uint32_t base, int kk) {    // MN-major, two 64-wide blocks
  return make_smem_desc_sw128(base + kk * 2048, ATILE / 2, 1024);
}
__device__ __forceinline__ uint4 apack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16(f[0], f[1]); u.y = pack_bf16(f[2], f[3]); u.z = pack_bf16(f[4], f[5]); u.w = pack_bf16(f[6], f[7]);
  return u;
}
// store 8 values of row `row`, columns [col, col+8) into a [128][128] swizzled tile
__device__ __forceinline__ void tile_store8(uint8_t* tile, int row, int col, const float (&f)[8]) {
  *reinterpret_cast<uint4*>(tile + (col >> 6) * (ATILE / 2) + sw128_offset(row, (col & 63) >> 3)) = apack8(f);
}

struct AttnFwdParams {
  float* lse;
  int L, Hq, Hkv;
  float scale;
  int* status;
};

__global__ void __launch_bounds__(128, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                const AttnFwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK0 = smem + ATILE;             // K stages at +1, +2 tiles; V stages at +3, +4 tiles
  uint8_t* sV0 = smem + 3 * ATILE;
  uint8_t* sP = smem + 5 * ATILE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * ATILE);   // [0] q, [1..2] kv stage, [3] S ready, [4] PV ready
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z, tid = threadIdx.x, warp = tid >> 5;
  const int hk = h / (p.Hq / p.Hkv);
  const int row0 = b * p.L + qt * AT;

  if (tid == 0) {
    for (int k = 0; k < 5; ++k) mbar_init(&bars[k], 1);
    mbar_fence_init();
    tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); tma_prefetch_desc(&tm_o);
  }
  if (warp == 0) { tmem_alloc(tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const int ntiles = qt + 1;

  auto load_kv = [&](int j, int stage) {
    mbar_expect_tx(&bars[1 + stage], 2 * ATILE);
    const int r = b * p.L + j * AT;
    uint8_t* dk = sK0 + stage * ATILE;
    uint8_t* dv = sV0 + stage * ATILE;
    tma_load_2d(dk, &tm_k, hk * AD, r, &bars[1 + stage]);
    tma_load_2d(dk + ATILE / 2, &tm_k, hk * AD + 64, r, &bars[1 + stage]);
    tma_load_2d(dv, &tm_v, hk * AD, r, &bars[1 + stage]);
    tma_load_2d(dv + ATILE / 2, &tm_v, hk * AD + 64, r, &bars[1 + stage]);
  };
  if (tid == 0) {
    mbar_expect_tx(&bars[0], ATILE);
    tma_load_2d(sQ, &tm_q, h * AD, row0, &bars[0]);
    tma_load_2d(sQ + ATILE / 2, &tm_q, h * AD + 64, row0, &bars[0]);
    load_kv(0, 0);
  }
  float o[AD];
  #pragma unroll
  for (int d = 0; d < AD; ++d) o[d] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  const float c = p.scale * LOG2E;
  bool ok = true;
  const uint32_t aQ = smem_u32(sQ), aP = smem_u32(sP);

  for (int j = 0; j < ntiles && ok; ++j) {
    const int st = j & 1;
    const uint32_t kv_par = (j >> 1) & 1, par = j & 1;
    if (tid == 0) {
      if (j + 1 < ntiles) load_kv(j + 1, st ^ 1);        // stage st^1 was released by the barrier ending tile j-1
      bool good = (j > 0) || mbar_wait(&bars[0], 0, p.status);
      good = good && mbar_wait(&bars[1 + st], kv_par, p.status);
      if (good) {
        tc_fence_after_sync();
        const uint32_t aK = smem_u32(sK0 + st * ATILE);
        const uint32_t id = make_idesc_bf16(128, 128, 0, 0);
        #pragma unroll
        for (int kk = 0; kk < 8; ++kk) umma_bf16(tmem, adesc_k(aQ, kk), adesc_k(aK, kk), id, kk != 0);
        umma_commit(&bars[3]);
      }
    }
    __syncwarp();
    ok = __syncthreads_and(mbar_wait(&bars[3], par, p.status));
    tc_fence_after_sync();
    if (!ok) break;
    // ---- online softmax, row = tid
    const bool diag = (j == qt);
    float m_new = m_run;
    #pragma unroll 1
    for (int jb = 0; jb < 4; ++jb) {
      uint32_t v[32];
      tmem_ld32(tmem_addr(tmem, warp * 32, jb * 32), v);
      tmem_ld_wait();
      #pragma unroll
      for (int e = 0; e < 32; ++e)
        if (!diag || jb * 32 + e <= tid) m_new = fmaxf(m_new, __uint_as_float(v[e]));
    }
    const float alpha = exp2f((m_run - m_new) * c);       // m_run = -inf on the first tile -> 0
    float rsum = 0.f;
    #pragma unroll 1
    for (int jb = 0; jb < 4; ++jb) {
      uint32_t v[32];
      tmem_ld32(tmem_addr(tmem, warp * 32, jb * 32), v);
      tmem_ld_wait();
      #pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        float f[8];
        #pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int col = jb * 32 + ch * 8 + e;
          const float pv = (!diag || col <= tid) ? exp2f((__uint_as_float(v[ch * 8 + e]) - m_new) * c) : 0.f;
          f[e] = pv;
          rsum += pv;
        }
        tile_store8(sP, tid, jb * 32 + ch * 8, f);
      }
    }
    l_run = l_run * alpha + rsum;
    m_run = m_new;
    #pragma unroll
    for (int d = 0; d < AD; ++d) o[d] *= alpha;
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after_sync();
      const uint32_t aV = smem_u32(sV0 + st * ATILE);
      const uint32_t id = make_idesc_bf16(128, 128, 0, 1);
      #pragma unroll
      for (int kk = 0; kk < 8; ++kk) umma_bf16(tmem + 128, adesc_k(aP, kk), adesc_mn(aV, kk), id, kk != 0);
      umma_commit(&bars[4]);
    }
    __syncwarp();
    ok = __syncthreads_and(mbar_wait(&bars[4], par, p.status));
    tc_fence_after_sync();
    if (!ok) break;
    #pragma unroll
    for (int db = 0; db < 4; ++db) {
      uint32_t v[32];
      tmem_ld32(tmem_addr(tmem, warp * 32, 128 + db * 32), v);
      tmem_ld_wait();
      #pragma unroll
      for (int e = 0; e < 32; ++e) o[db * 32 + e] += __uint_as_float(v[e]);
    }
    tc_fence_before_sync();
    __syncthreads();          // all reads of S / PV and of this K/V stage are done
  }
  if (ok) {
    const float inv = 1.f / l_run;
    #pragma unroll
    for (int ch = 0; ch < 16; ++ch) {
      float f[8];
      #pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = o[ch * 8 + e] * inv;
      tile_store8(sP, tid, ch * 8, f);
    }
    p.lse[((long long)b * p.Hq + h) * p.L + qt * AT + tid] = m_run * p.scale + logf(l_run);
  }
  fence_proxy_async_smem();
  __syncthreads();
  if (tid == 0 && ok) {
    tma_store_2d(&tm_o, sP, h * AD, row0);
    tma_store_2d(&tm_o, sP + ATILE / 2, h * AD + 64, row0);
    tma_store_commit();
    tma_store_wait_all();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

// ---------------------------------------------------------------------------------------------------
struct AttnBwdParams {
  const float* lse; const float* delta;     // [B, Hq, L]
  float* dq32;                              // [B*L, Hq*128] fp32, zero on entry
  __nv_bfloat16* dk; __nv_bfloat16* dv;     // [B*L, Hkv*128]
  int L, Hq, Hkv;
  float scale;
  int* status;
};

__global__ void __launch_bounds__(128, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                const AttnBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + ATILE;
  uint8_t* sQ = smem + 2 * ATILE;
  uint8_t* sDO = smem + 3 * ATILE;
  uint8_t* sP = smem + 4 * ATILE;
  uint8_t* sDS = smem + 5 * ATILE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * ATILE);   // [0] kv, [1] q/do, [2] S,dP, [3] dV,dK,dQ
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  const int kt = blockIdx.x, hk = blockIdx.y, b = blockIdx.z, tid = threadIdx.x, warp = tid >> 5;
  const int ratio = p.Hq / p.Hkv;
  const int qtiles = p.L / AT;
  const int krow0 = b * p.L + kt * AT;

  if (tid == 0) {
    for (int k = 0; k < 4; ++k) mbar_init(&bars[k], 1);
    mbar_fence_init();
    tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); tma_prefetch_desc(&tm_do);
  }
  if (warp == 0) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ = smem_u32(sQ), aDO = smem_u32(sDO), aP = smem_u32(sP),
                 aDS = smem_u32(sDS);
  if (tid == 0) {
    mbar_expect_tx(&bars[0], 2 * ATILE);
    tma_load_2d(sK, &tm_k, hk * AD, krow0, &bars[0]);
    tma_load_2d(sK + ATILE / 2, &tm_k, hk * AD + 64, krow0, &bars[0]);
    tma_load_2d(sV, &tm_v, hk * AD, krow0, &bars[0]);
    tma_load_2d(sV + ATILE / 2, &tm_v, hk * AD + 64, krow0, &bars[0]);
  }
  const float c = p.scale * LOG2E;
  bool ok = true;
  int it = 0;
  for (int hr = 0; hr < ratio && ok; ++hr) {
    const int h = hk * ratio + hr;
    for (int qt = kt; qt < qtiles && ok; ++qt, ++it) {
      const uint32_t par = it & 1;
      const int qrow0 = b * p.L + qt * AT;
      if (tid == 0) {
        mbar_expect_tx(&bars[1], 2 * ATILE);
        tma_load_2d(sQ, &tm_q, h * AD, qrow0, &bars[1]);
        tma_load_2d(sQ + ATILE / 2, &tm_q, h * AD + 64, qrow0, &bars[1]);
        tma_load_2d(sDO, &tm_do, h * AD, qrow0, &bars[1]);
        tma_load_2d(sDO + ATILE / 2, &tm_do, h * AD + 64, qrow0, &bars[1]);
        bool good = (it > 0) || mbar_wait(&bars[0], 0, p.status);
        good = good && mbar_wait(&bars[1], par, p.status);
        if (good) {
          tc_fence_after_sync();
          const uint32_t id = make_idesc_bf16(128, 128, 0, 0);
          #pragma unroll
          for (int kk = 0; kk < 8; ++kk) umma_bf16(tmem, adesc_k(aQ, kk), adesc_k(aK, kk), id, kk != 0);           // S
          #pragma unroll
          for (int kk = 0; kk < 8; ++kk) umma_bf16(tmem + 128, adesc_k(aDO, kk), adesc_k(aV, kk), id, kk != 0);   // dP
          umma_commit(&bars[2]);
        }
      }
      __syncwarp();
      ok = __syncthreads_and(mbar_wait(&bars[2], par, p.status));
      tc_fence_after_sync();
      if (!ok) break;
      const long long so = ((long long)b * p.Hq + h) * p.L + qt * AT + tid;
      const float lse2 = p.lse[so] * LOG2E, dlt = p.delta[so];
      const bool diag = (qt == kt);
      #pragma unroll 1
      for (int jb = 0; jb < 4; ++jb) {
        uint32_t sv[32], dp[32];
        tmem_ld32(tmem_addr(tmem, warp * 32, jb * 32), sv);
        tmem_ld32(tmem_addr(tmem, warp * 32, 128 + jb * 32), dp);
        tmem_ld_wait();
        #pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          float pf[8], df[8];
          #pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int col = jb * 32 + ch * 8 + e;
            const float pv = (!diag || col <= tid) ? exp2f(__uint_as_float(sv[ch * 8 + e]) * c - lse2) : 0.f;
            pf[e] = pv;
            df[e] = pv * (__uint_as_float(dp[ch * 8 + e]) - dlt) * p.scale;
          }
          tile_store8(sP, tid, jb * 32 + ch * 8, pf);
          tile_store8(sDS, tid, jb * 32 + ch * 8, df);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncthreads();
      if (tid == 0) {
        tc_fence_after_sync();
        const uint32_t id_t = make_idesc_bf16(128, 128, 1, 1);
        #pragma unroll
        for (int kk = 0; kk < 8; ++kk)      // dV[key][d] += sum_i P[i][key] dO[i][d]
          umma_bf16(tmem + 256, adesc_mn(aP, kk), adesc_mn(aDO, kk), id_t, (it | kk) != 0);
        #pragma unroll
        for (int kk = 0; kk < 8; ++kk)      // dK[key][d] += sum_i dS[i][key] Q[i][d]
          umma_bf16(tmem + 384, adesc_mn(aDS, kk), adesc_mn(aQ, kk), id_t, (it | kk) != 0);
        const uint32_t id_q = make_idesc_bf16(128, 128, 0, 1);
        #pragma unroll
        for (int kk = 0; kk < 8; ++kk)      // dQ[i][d] = sum_key dS[i][key] K[key][d]
          umma_bf16(tmem, adesc_k(aDS, kk), adesc_mn(aK, kk), id_q, kk != 0);
        umma_commit(&bars[3]);
      }
      __syncwarp();
      ok = __syncthreads_and(mbar_wait(&bars[3], par, p.status));
      tc_fence_after_sync();
      if (!ok) break;
      float* dq = p.dq32 + (long long)(qrow0 + tid) * (p.Hq * AD) + h * AD;
      #pragma unroll 1
      for (int db = 0; db < 4; ++db) {
        uint32_t v[32];
        tmem_ld32(tmem_addr(tmem, warp * 32, db * 32), v);
        tmem_ld_wait();
        #pragma unroll
        for (int k4 = 0; k4 < 8; ++k4)
          asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dq + db * 32 + k4 * 4),
                       "f"(__uint_as_float(v[k4 * 4])), "f"(__uint_as_float(v[k4 * 4 + 1])),
                       "f"(__uint_as_float(v[k4 * 4 + 2])), "f"(__uint_as_float(v[k4 * 4 + 3])) : "memory");
      }
      tc_fence_before_sync();
      __syncthreads();       // Q, dO, P, dS tiles and TMEM[0,256) are free for the next iteration
    }
  }
  if (ok) {
    tc_fence_after_sync();
    #pragma unroll 1
    for (int which = 0; which < 2; ++which) {
      __nv_bfloat16* dst = (which == 0 ? p.dv : p.dk) + (long long)(krow0 + tid) * (p.Hkv * AD) + hk * AD;
      #pragma unroll 1
      for (int db = 0; db < 4; ++db) {
        uint32_t v[32];
        tmem_ld32(tmem_addr(tmem, warp * 32, 256 + which * 128 + db * 32), v);
        tmem_ld_wait();
        #pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          float f[8];
          #pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(v[ch * 8 + e]);
          *reinterpret_cast<uint4*>(dst + db * 32 + ch * 8) = apack8(f);
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace ssm

using namespace ssm;

static int attn_maps(CUtensorMap* tq, CUtensorMap* tk, CUtensorMap* tv, CUtensorMap* tx, const void* q, const void* k,
                     const void* v, const void* x, int B, int L, int Hq, int Hkv) {
  int r = make_tmap_2d_bf16(tq, q, (uint64_t)Hq * AD, (uint64_t)B * L, (uint64_t)Hq * AD * 2, 64, 128);
  if (r) return -100 - r;
  r = make_tmap_2d_bf16(tk, k, (uint64_t)Hkv * AD, (uint64_t)B * L, (uint64_t)Hkv * AD * 2, 64, 128);
  if (r) return -200 - r;
  r = make_tmap_2d_bf16(tv, v, (uint64_t)Hkv * AD, (uint64_t)B * L, (uint64_t)Hkv * AD * 2, 64, 128);
  if (r) return -300 - r;
  r = make_tmap_2d_bf16(tx, x, (uint64_t)Hq * AD, (uint64_t)B * L, (uint64_t)Hq * AD * 2, 64, 128);
  if (r) return -400 - r;
  return 0;
}

extern "C" int ssm_attn_fwd(const void* q, const void* k, const void* v, void* out, void* lse, int B, int L, int Hq,
                            int Hkv, int D, float scale, int* status, cudaStream_t st) {
  if (D != AD || L % AT || Hq % Hkv) return -SSM_ERR_BAD_ARG;
  static bool cfg = false;
  const int smem = 6 * ATILE + 128 + 1024;
  if (!cfg) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    cfg = true;
  }
  CUtensorMap tq, tk, tv, to;
  int r = attn_maps(&tq, &tk, &tv, &to, q, k, v, out, B, L, Hq, Hkv);
  if (r) return r;
  AttnFwdParams p;
  p.lse = reinterpret_cast<float*>(lse); p.L = L; p.Hq = Hq; p.Hkv = Hkv; p.scale = scale; p.status = status;
  dim3 grid(L / AT, Hq, B);
  attn_fwd_kernel<<<grid, 128, smem, st>>>(tq, tk, tv, to, p);
  return (int)cudaGetLastError();
}

extern "C" int ssm_attn_bwd(const void* q, const void* k, const void* v, const void* dout, const void* lse,
                            const void* delta, void* dq32, void* dk, void* dv, int B, int L, int Hq, int Hkv, int D,
                            float scale, int* status, cudaStream_t st) {
  if (D != AD || L % AT || Hq % Hkv) return -SSM_ERR_BAD_ARG;
  static bool cfg = false;
  const int smem = 6 * ATILE + 128 + 1024;
  if (!cfg) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    cfg = true;
  }
  CUtensorMap tq, tk, tv, tdo;
  int r = attn_maps(&tq, &tk, &tv, &tdo, q, k, v, dout, B, L, Hq, Hkv);
  if (r) return r;
  AttnBwdParams p;
  p.lse = reinterpret_cast<const float*>(lse); p.delta = reinterpret_cast<const float*>(delta);
  p.dq32 = reinterpret_cast<float*>(dq32);
  p.dk = reinterpret_cast<__nv_bfloat16*>(dk); p.dv = reinterpret_cast<__nv_bfloat16*>(dv);
  p.L = L; p.Hq = Hq; p.Hkv = Hkv; p.scale = scale; p.status = status;
  dim3 grid(L / AT, Hkv, B);
  attn_bwd_kernel<<<grid, 128, smem, st>>>(tq, tk, tv, tdo, p);
  return (int)cudaGetLastError();
}
