// SSD (state-space duality) chunked scan for sm_100a, forward and backward, chunk = 128 tokens,
// d_state N = 128, head slices of P = 64 channels (a head of 128 channels is two slices sharing dt/A/D).
//
// Per (batch b, head slice h, chunk c), with l_i = cumsum(A dt) inside the chunk:
//   forward   Y = (CB^T o Lambda o dt_j) X + exp(l_i) C S_in + D x           (Lambda_ij = exp(l_i - l_j), j <= i)
//             S_local = sum_j exp(l_T - l_j) dt_j B_j (x) x_j ;  S_in[c+1] = exp(l_T) S_in[c] + S_local[c]
//   backward  see ssd_chunk_scan_bwd_kernel.
// All 128x128x{64,128} products run on tcgen05 with fp32 accumulators in TMEM; operands come straight from
// TMA (B, C, x, dY, states) or are built by the 128 threads of the CTA in the 128-byte-swizzled layout
// (decay-weighted CB^T, scaled x / dY).  The decay factors are always formed as exp of a difference of
// cumulative sums, never as a ratio of exponentials.
// Reference math: mamba2/mamba2_kernel.py:15-62,138-169 (forward), :358-480 (backward).
#include "common.cuh"

namespace ssm {

constexpr int CT = 128;      // chunk length
constexpr int NS = 128;      // d_state
constexpr int PS = 64;       // channels per head slice
constexpr int TILE128 = 128 * 128 * 2;   // bytes of a [128][128] bf16 tile (two 16 KiB swizzle blocks)
constexpr int TILE64 = 128 * 64 * 2;     // bytes of a [128][64] bf16 tile

// descriptor helpers ------------------------------------------------------------------------------
// K-major operand tile [rows][K] made of 64-wide K atoms of [rows][128 B]; k-step kk covers K = 16*kk..
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t base, int kk, uint32_t atom_bytes) {
  return make_smem_desc_sw128(base + (kk >> 2) * atom_bytes + (kk & 3) * 32, 16, 1024);
}
// MN-major operand tile [K rows][MN] made of 64-wide MN blocks of [K rows][128 B] `block_bytes` apart.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t base, int kk, uint32_t block_bytes) {
  return make_smem_desc_sw128(base + kk * 2048, block_bytes, 1024);
}

__device__ __forceinline__ void unpack8(const uint4 u, float (&f)[8]) {
  f[0] = bf16_lo(u.x); f[1] = bf16_hi(u.x); f[2] = bf16_lo(u.y); f[3] = bf16_hi(u.y);
  f[4] = bf16_lo(u.z); f[5] = bf16_hi(u.z); f[6] = bf16_lo(u.w); f[7] = bf16_hi(u.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16(f[0], f[1]); u.y = pack_bf16(f[2], f[3]); u.z = pack_bf16(f[4], f[5]); u.w = pack_bf16(f[6], f[7]);
  return u;
}

// block-wide helpers for 128 threads -----------------------------------------------------------------
__device__ __forceinline__ float warp_sum128(float v) {
  #pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// sum over the 128 threads, result to all; red has >= 4 floats; contains two __syncthreads
__device__ __forceinline__ float block_sum128(float v, float* red) {
  v = warp_sum128(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  return red[0] + red[1] + red[2] + red[3];
}

// =====================================================================================
// dt = softplus(dt_raw + bias), l = inclusive cumsum of A*dt within each chunk.   grid (nc, H, B), 128 threads
// =====================================================================================
__global__ void __launch_bounds__(128)
ssd_dt_prep_kernel(const __nv_bfloat16* __restrict__ dt_raw, long long row_stride, const float* __restrict__ dt_bias,
                   const float* __restrict__ A, float* __restrict__ dt_out, float* __restrict__ l_out, int L, int H) {
  __shared__ float wsum[4];
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z, j = threadIdx.x;
  const long long t = (long long)c * CT + j;
  const float v = __bfloat162float(dt_raw[((long long)b * L + t) * row_stride + h]) + dt_bias[h];
  const float dt = softplus_f(v);
  float a = A[h] * dt;
  const int lane = j & 31, w = j >> 5;
  #pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, a, o);
    if (lane >= o) a += n;
  }
  if (lane == 31) wsum[w] = a;
  __syncthreads();
  float off = 0.f;
  for (int k = 0; k < w; ++k) off += wsum[k];
  const long long o = ((long long)b * H + h) * L + t;
  dt_out[o] = dt;
  l_out[o] = a + off;
}

// =====================================================================================
// chunk states:  S[n][p] = sum_j W[j][n] * s_j * V[j][p]
//   mode 0 (forward):   W = B, V = x,  s_j = exp(l_T - l_j) * dt_j
//   mode 1 (backward):  W = C, V = dY, s_j = exp(l_j)
// grid (nc, Hv, B), 128 threads.  out fp32 [B, Hv, nc, 128, 64].
// =====================================================================================
struct ChunkStateParams {
  const __nv_bfloat16* v; long long v_row_stride;  // V rows: (b*L + t) * v_row_stride + hv*64
  const float* dt; const float* l;                 // [B, H, L]
  float* out;
  int L, H, Hv, G, nc, w_col0, mode;
  int* status;
};

__global__ void __launch_bounds__(128)
ssd_chunk_state_kernel(const __grid_constant__ CUtensorMap tm_w, const ChunkStateParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sW = smem;                      // [128 j][128 n]  (two blocks)
  uint8_t* sV = smem + TILE128;            // [128 j][64 p]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TILE128 + TILE64);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
  const int c = blockIdx.x, hv = blockIdx.y, b = blockIdx.z, tid = threadIdx.x, warp = tid >> 5;
  const int psplit = p.Hv / p.H, h = hv / psplit, g = h / (p.H / p.G);
  const long long row0 = (long long)b * p.L + (long long)c * CT;

  if (tid == 0) { mbar_init(&bars[0], 1); mbar_init(&bars[1], 1); mbar_fence_init(); }
  if (warp == 0) { tmem_alloc(tmem_slot, 64); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  if (tid == 0) {
    mbar_expect_tx(&bars[0], TILE128);
    tma_load_2d(sW, &tm_w, p.w_col0 + g * NS, (int)row0, &bars[0]);
    tma_load_2d(sW + TILE128 / 2, &tm_w, p.w_col0 + g * NS + 64, (int)row0, &bars[0]);
  }
  // scaled V row j -> smem (MN-major B operand: rows = j (K), 64 contiguous p)
  {
    const long long lo = ((long long)b * p.H + h) * p.L + (long long)c * CT;
    const float lj = p.l[lo + tid];
    float s;
    if (p.mode == 0) s = __expf(p.l[lo + CT - 1] - lj) * p.dt[lo + tid];
    else s = __expf(lj);
    const __nv_bfloat16* vr = p.v + (row0 + tid) * p.v_row_stride + (long long)hv * PS;
    #pragma unroll
    for (int ch = 0; ch < 8; ++ch) {
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(vr + ch * 8), f);
      #pragma unroll
      for (int e = 0; e < 8; ++e) f[e] *= s;
      *reinterpret_cast<uint4*>(sV + sw128_offset(tid, ch)) = pack8(f);
    }
  }
  fence_proxy_async_smem();
  __syncthreads();
  bool ok = true;
  if (tid == 0) {
    ok = mbar_wait(&bars[0], 0, p.status);
    if (ok) {
      tc_fence_after_sync();
      const uint32_t idesc = make_idesc_bf16(128, PS, 1, 1);
      const uint32_t a = smem_u32(sW), bb = smem_u32(sV);
      #pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        umma_bf16(tmem, desc_mnmajor(a, kk, TILE128 / 2), desc_mnmajor(bb, kk, 0), idesc, kk != 0);
      umma_commit(&bars[1]);
    }
  }
  __syncwarp();
  ok = __syncthreads_and(mbar_wait(&bars[1], 0, p.status));
  tc_fence_after_sync();
  if (ok) {
    float* o = p.out + ((((long long)b * p.Hv + hv) * p.nc + c) * NS + tid) * PS;
    #pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint32_t v[32];
      tmem_ld32(tmem_addr(tmem, warp * 32, half * 32), v);
      tmem_ld_wait();
      #pragma unroll
      for (int q = 0; q < 8; ++q)
        *reinterpret_cast<float4*>(o + half * 32 + q * 4) =
            make_float4(__uint_as_float(v[q * 4]), __uint_as_float(v[q * 4 + 1]), __uint_as_float(v[q * 4 + 2]),
                        __uint_as_float(v[q * 4 + 3]));
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 64);
}

// =====================================================================================
// inter-chunk recurrence (elementwise over the N*P state entries):
//   forward:  in[c] = run ; run = exp(l_T[c]) * run + local[c]       c = 0 .. nc-1
//   reverse:  in[c] = run ; run = exp(l_T[c]) * run + local[c]       c = nc-1 .. 0
// in: bf16 [B,Hv,nc,N*P] (MMA operand), final: fp32 [B,Hv,N*P] (optional), init fp32 [B,Hv,N*P] (optional).
// grid (N*P/4/256, Hv, B), 256 threads.
// =====================================================================================
__global__ void __launch_bounds__(256)
ssd_state_pass_kernel(const float* __restrict__ local, const float* __restrict__ l, const float* __restrict__ init,
                      __nv_bfloat16* __restrict__ in16, float* __restrict__ fin, int L, int H, int Hv, int nc,
                      int reverse) {
  const int hv = blockIdx.y, b = blockIdx.z;
  const int h = hv / (Hv / H);
  const int e = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  const long long base = ((long long)b * Hv + hv) * nc;
  const float* lrow = l + ((long long)b * H + h) * L;
  float4 run = make_float4(0.f, 0.f, 0.f, 0.f);
  if (init) run = *reinterpret_cast<const float4*>(init + ((long long)b * Hv + hv) * (NS * PS) + e);
  for (int k = 0; k < nc; ++k) {
    const int c = reverse ? nc - 1 - k : k;
    const long long o = (base + c) * (NS * PS) + e;
    uint2 pk;
    pk.x = pack_bf16(run.x, run.y); pk.y = pack_bf16(run.z, run.w);
    *reinterpret_cast<uint2*>(in16 + o) = pk;
    const float dec = __expf(lrow[(long long)c * CT + CT - 1]);
    const float4 s = *reinterpret_cast<const float4*>(local + o);
    run.x = dec * run.x + s.x; run.y = dec * run.y + s.y; run.z = dec * run.z + s.z; run.w = dec * run.w + s.w;
  }
  if (fin) *reinterpret_cast<float4*>(fin + ((long long)b * Hv + hv) * (NS * PS) + e) = run;
}

// =====================================================================================
// forward chunk scan.  grid (nc, Hv, B), 128 threads, 2 CTAs / SM.
// TMEM: [0,128) CB^T product, [128,192) Y_diag, [192,256) Y_off.
// smem: C tile | B tile | x tile | S_in tile ; the decay-weighted matrix reuses the C tile, the output
// staging reuses the B tile.
// =====================================================================================
struct ScanFwdParams {
  const float* dt; const float* l; const float* D;   // dt,l [B,H,L]; D [H]
  int L, H, Hv, G, nc, d_in;
  int* status;
};

__global__ void __launch_bounds__(128)
ssd_chunk_scan_fwd_kernel(const __grid_constant__ CUtensorMap tm_xbc, const __grid_constant__ CUtensorMap tm_sin,
                          const __grid_constant__ CUtensorMap tm_y, const ScanFwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sC = smem;                          // [128 i][128 n]; later M [128 i][128 j]
  uint8_t* sB = smem + TILE128;                // [128 j][128 n]; later y staging [128 i][64 p]
  uint8_t* sX = smem + 2 * TILE128;            // [128 j][64 p]
  uint8_t* sS = smem + 2 * TILE128 + TILE64;   // [128 n][64 p]
  float* s_l = reinterpret_cast<float*>(smem + 2 * TILE128 + 2 * TILE64);
  float* s_dt = s_l + CT;
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_dt + CT);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);
  const int c = blockIdx.x, hv = blockIdx.y, b = blockIdx.z, tid = threadIdx.x, warp = tid >> 5;
  const int psplit = p.Hv / p.H, h = hv / psplit, g = h / (p.H / p.G);
  const int row0 = b * p.L + c * CT;

  if (tid == 0) {
    mbar_init(&bars[0], 1); mbar_init(&bars[1], 1); mbar_init(&bars[2], 1);
    mbar_fence_init();
    tma_prefetch_desc(&tm_xbc); tma_prefetch_desc(&tm_sin); tma_prefetch_desc(&tm_y);
  }
  if (warp == 0) { tmem_alloc(tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  if (tid == 0) {
    mbar_expect_tx(&bars[0], 2 * TILE128 + 2 * TILE64);
    const int cB = p.d_in + g * NS, cC = p.d_in + p.G * NS + g * NS;
    tma_load_2d(sC, &tm_xbc, cC, row0, &bars[0]);
    tma_load_2d(sC + TILE128 / 2, &tm_xbc, cC + 64, row0, &bars[0]);
    tma_load_2d(sB, &tm_xbc, cB, row0, &bars[0]);
    tma_load_2d(sB + TILE128 / 2, &tm_xbc, cB + 64, row0, &bars[0]);
    tma_load_2d(sX, &tm_xbc, hv * PS, row0, &bars[0]);
    tma_load_2d(sS, &tm_sin, 0, ((b * p.Hv + hv) * p.nc + c) * NS, &bars[0]);
  }
  {
    const long long lo = ((long long)b * p.H + h) * p.L + (long long)c * CT;
    s_l[tid] = p.l[lo + tid];
    s_dt[tid] = p.dt[lo + tid];
  }
  __syncthreads();
  bool ok = true;
  if (tid == 0) {
    ok = mbar_wait(&bars[0], 0, p.status);
    if (ok) {
      tc_fence_after_sync();
      const uint32_t aC = smem_u32(sC), aB = smem_u32(sB), aS = smem_u32(sS);
      const uint32_t id_cb = make_idesc_bf16(128, 128, 0, 0);
      #pragma unroll
      for (int kk = 0; kk < 8; ++kk)      // CB^T[i][j] = sum_n C[i][n] B[j][n]
        umma_bf16(tmem, desc_kmajor(aC, kk, TILE128 / 2), desc_kmajor(aB, kk, TILE128 / 2), id_cb, kk != 0);
      const uint32_t id_off = make_idesc_bf16(128, PS, 0, 1);
      #pragma unroll
      for (int kk = 0; kk < 8; ++kk)      // Y_off[i][p] = sum_n C[i][n] S_in[n][p]
        umma_bf16(tmem + 192, desc_kmajor(aC, kk, TILE128 / 2), desc_mnmajor(aS, kk, 0), id_off, kk != 0);
      umma_commit(&bars[1]);
    }
  }
  __syncwarp();
  ok = __syncthreads_and(mbar_wait(&bars[1], 0, p.status));
  tc_fence_after_sync();
  const int i = tid;
  if (ok) {
    // decay-weighted lower-triangular matrix, row i, written over the C tile (K-major A operand, K = j)
    const float li = s_l[i];
    #pragma unroll 1
    for (int jb = 0; jb < 4; ++jb) {
      if (jb > warp) {      // columns j > i for every row of this warp: the causal mask zeroes the whole block
        #pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const int jc = jb * 32 + ch * 8;
          *reinterpret_cast<uint4*>(sC + (jc >> 6) * (TILE128 / 2) + sw128_offset(i, (jc & 63) >> 3)) = make_uint4(0, 0, 0, 0);
        }
        continue;
      }
      uint32_t v[32];
      tmem_ld32(tmem_addr(tmem, warp * 32, jb * 32), v);
      tmem_ld_wait();
      #pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        float f[8];
        #pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int j = jb * 32 + ch * 8 + e;
          f[e] = (j <= i) ? __uint_as_float(v[ch * 8 + e]) * __expf(li - s_l[j]) * s_dt[j] : 0.f;
        }
        const int jc = jb * 32 + ch * 8;
        *reinterpret_cast<uint4*>(sC + (jc >> 6) * (TILE128 / 2) + sw128_offset(i, (jc & 63) >> 3)) = pack8(f);
      }
    }
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && ok) {
    tc_fence_after_sync();
    const uint32_t aM = smem_u32(sC), aX = smem_u32(sX);
    const uint32_t id = make_idesc_bf16(128, PS, 0, 1);
    #pragma unroll
    for (int kk = 0; kk < 8; ++kk)        // Y_diag[i][p] = sum_j M[i][j] x[j][p]
      umma_bf16(tmem + 128, desc_kmajor(aM, kk, TILE128 / 2), desc_mnmajor(aX, kk, 0), id, kk != 0);
    umma_commit(&bars[2]);
  }
  __syncwarp();
  ok = __syncthreads_and(ok && mbar_wait(&bars[2], 0, p.status));
  tc_fence_after_sync();
  if (ok) {
    const float al = __expf(s_l[i]);
    const float Dh = p.D[h];
    #pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint32_t yd[32], yo[32];
      tmem_ld32(tmem_addr(tmem, warp * 32, 128 + half * 32), yd);
      tmem_ld32(tmem_addr(tmem, warp * 32, 192 + half * 32), yo);
      tmem_ld_wait();
      #pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        float xv[8], f[8];
        unpack8(*reinterpret_cast<const uint4*>(sX + sw128_offset(i, half * 4 + ch)), xv);
        #pragma unroll
        for (int e = 0; e < 8; ++e)
          f[e] = __uint_as_float(yd[ch * 8 + e]) + al * __uint_as_float(yo[ch * 8 + e]) + Dh * xv[e];
        *reinterpret_cast<uint4*>(sB + sw128_offset(i, half * 4 + ch)) = pack8(f);
      }
    }
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && ok) {
    tma_store_2d(&tm_y, sB, hv * PS, row0);
    tma_store_commit();
    tma_store_wait_all();
  }
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

// =====================================================================================
// backward chunk scan.  grid (nc, G * splits, B), 256 threads (two warpgroups), 1 CTA / SM; the CTA walks `hpc` head slices
// of one group.  Given dY and, per chunk, S_in (state entering the chunk) and dS_out (gradient of the state
// leaving the chunk):
//   CB = C B^T ; dM = dY X^T ; M0 = CB o Lambda ; dCB = dM o Lambda o dt_j
//   dU   = M0^T dY + exp(l_T - l_j) (B dS_out)                      dx = dt_j dU + D dY
//   dB  += dCB^T C + (exp(l_T - l_j) dt_j X) dS_out^T               dC += dCB B + (exp(l_i) dY) S_in^T
//   ddt_j = sum_p x dU + A da_j ;  da_j = sum_{k >= j} dl_k + E
//   dl_k = sum_{j<k} W[k][j] - sum_{i>k} W[i][k] + exp(l_k) sum_p dY (C S_in) - exp(l_T - l_k) dt_k sum_p x (B dS_out),
//          W = dM o M0 o dt_j   (row sums in-thread, column sums by a warp butterfly; no cancellation of large terms)
//   E = exp(l_T) <dS_out, S_in> + sum_j exp(l_T - l_j) dt_j sum_p x (B dS_out)
//   dA += sum_j dt_j da_j ; dD += sum dY x ; d(dt_raw) = ddt sigmoid(dt_raw + bias)
// TMEM: [0,128) CB then dU_diag | dU_state, [128,256) dM then C S_in, [256,384) dB, [384,512) dC
// (dB, dC accumulate over the CTA's heads and are added to the fp32 output with red.add).
// =====================================================================================
struct ScanBwdParams {
  const float* dt; const float* l; const float* D; const float* A; const float* dt_bias;
  const __nv_bfloat16* dt_raw; long long dt_raw_stride;     // [B*L rows], column h
  __nv_bfloat16* ddt_raw; long long ddt_stride;             // d(dt_raw): row (b*L+t)*stride + h  (bf16, atomic-free when psplit == 1)
  float* ddt32;                                             // [B, Hv, L] fp32 per head slice (summed on the host when psplit > 1)
  float* dBC;                                               // fp32 [B*L, 2*G*128]
  float* hpart;                                             // fp32 [B*nc, Hv, 3]  (dA, dD, d dt_bias partials)
  int L, H, Hv, G, nc, d_in, hpc;
  int* status;
};

constexpr int BWD_SMEM = 2 * TILE128 /*C,B*/ + 4 * TILE64 /*X,dY,Sin,dSout*/ + 2 * TILE128 /*M0,dCB*/ + TILE64 /*dY'*/;

// 256 threads = two warpgroups.  Row r = tid & 127 of every 128-row tile is shared by the two threads (r, wg = 0/1):
// in the operand-building phase warpgroup wg handles the 32-column blocks jb with (jb & 1) == wg, in the scaling
// and epilogue phases it handles channel half wg (32 of the 64 channels).  Two warps per scheduler hide the
// TMEM-load / MUFU / shared-memory latencies that a single warpgroup leaves exposed.
__device__ __forceinline__ float block_sum256(float v, float* red) {   // red: >= 8 floats; two __syncthreads
  v = warp_sum128(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  return red[0] + red[1] + red[2] + red[3] + red[4] + red[5] + red[6] + red[7];
}

__global__ void __launch_bounds__(256, 1)
ssd_chunk_scan_bwd_kernel(const __grid_constant__ CUtensorMap tm_xbc, const __grid_constant__ CUtensorMap tm_dy,
                          const __grid_constant__ CUtensorMap tm_sin, const __grid_constant__ CUtensorMap tm_dsout,
                          const __grid_constant__ CUtensorMap tm_dx, const ScanBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sC = smem;
  uint8_t* sB = sC + TILE128;
  uint8_t* sX = sB + TILE128;          // x, later scaled in place, later dx staging
  uint8_t* sDY = sX + TILE64;
  uint8_t* sSin = sDY + TILE64;
  uint8_t* sDS = sSin + TILE64;
  uint8_t* sM0 = sDS + TILE64;
  uint8_t* sDCB = sM0 + TILE128;
  uint8_t* sDYs = sDCB + TILE128;      // exp(l_i) * dY
  float* s_l = reinterpret_cast<float*>(sDYs + TILE64);
  float* s_dt = s_l + CT;
  float* s_red = s_dt + CT;            // 16 floats
  float* s_col = s_red + 16;           // [4 row-warps][128] column sums of W
  float* s_pair = s_col + 4 * CT;      // [5][128] per-row partials handed from warpgroup 1 to warpgroup 0
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_pair + 5 * CT);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);

  const int c = blockIdx.x, b = blockIdx.z, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row = tid & 127, wg = tid >> 7, rw = warp & 3;      // tile row, warpgroup, row-warp (TMEM lane quarter)
  const int psplit = p.Hv / p.H;
  const int hv_per_group = (p.H / p.G) * psplit;
  const int splits = hv_per_group / p.hpc;
  const int g = blockIdx.y / splits;
  const int hv0 = g * hv_per_group + (blockIdx.y % splits) * p.hpc;
  const int row0 = b * p.L + c * CT;

  if (tid == 0) {
    for (int k = 0; k < 4; ++k) mbar_init(&bars[k], 1);
    mbar_fence_init();
    tma_prefetch_desc(&tm_xbc); tma_prefetch_desc(&tm_dy); tma_prefetch_desc(&tm_sin);
    tma_prefetch_desc(&tm_dsout); tma_prefetch_desc(&tm_dx);
  }
  if (warp == 0) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t aC = smem_u32(sC), aB = smem_u32(sB), aX = smem_u32(sX), aDY = smem_u32(sDY), aSin = smem_u32(sSin),
                 aDS = smem_u32(sDS), aM0 = smem_u32(sM0), aDCB = smem_u32(sDCB), aDYs = smem_u32(sDYs);
  bool ok = true;

  for (int it = 0; it < p.hpc && ok; ++it) {
    const int hv = hv0 + it, h = hv / psplit;
    const uint32_t par = it & 1;
    // ---------------------------------------------------------------- loads
    if (tid == 0) {
      uint32_t bytes = 4 * TILE64;
      if (it == 0) bytes += 2 * TILE128;
      mbar_expect_tx(&bars[0], bytes);
      if (it == 0) {
        const int cB = p.d_in + g * NS, cC = p.d_in + p.G * NS + g * NS;
        tma_load_2d(sC, &tm_xbc, cC, row0, &bars[0]);
        tma_load_2d(sC + TILE128 / 2, &tm_xbc, cC + 64, row0, &bars[0]);
        tma_load_2d(sB, &tm_xbc, cB, row0, &bars[0]);
        tma_load_2d(sB + TILE128 / 2, &tm_xbc, cB + 64, row0, &bars[0]);
      }
      const int srow = ((b * p.Hv + hv) * p.nc + c) * NS;
      tma_load_2d(sX, &tm_xbc, hv * PS, row0, &bars[0]);
      tma_load_2d(sDY, &tm_dy, hv * PS, row0, &bars[0]);
      tma_load_2d(sSin, &tm_sin, 0, srow, &bars[0]);
      tma_load_2d(sDS, &tm_dsout, 0, srow, &bars[0]);
    }
    const long long lo = ((long long)b * p.H + h) * p.L + (long long)c * CT;
    if (wg == 0) s_l[row] = p.l[lo + row];
    else s_dt[row] = p.dt[lo + row];
    __syncthreads();
    // ---------------------------------------------------------------- phase 1: CB, dM
    if (tid == 0) {
      ok = mbar_wait(&bars[0], par, p.status);
      if (ok) {
        tc_fence_after_sync();
        const uint32_t id_cb = make_idesc_bf16(128, 128, 0, 0);
        #pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_bf16(tmem, desc_kmajor(aC, kk, TILE128 / 2), desc_kmajor(aB, kk, TILE128 / 2), id_cb, kk != 0);
        #pragma unroll
        for (int kk = 0; kk < 4; ++kk)                            // dM[i][j] = sum_p dY[i][p] x[j][p]
          umma_bf16(tmem + 128, desc_kmajor(aDY, kk, 0), desc_kmajor(aX, kk, 0), id_cb, kk != 0);
        umma_commit(&bars[1]);
      }
    }
    __syncwarp();
    ok = __syncthreads_and(mbar_wait(&bars[1], par, p.status));   // uniform outcome for the whole CTA
    tc_fence_after_sync();
    if (!ok) break;
    // ---------------------------------------------------------------- thread-built operands
    const float li = s_l[row], dti = s_dt[row], lT = s_l[CT - 1];
    const float a_left = __expf(li), a_right = __expf(lT - li);
    float r1 = 0.f;                      // this thread's share of sum_{j<i} W[i][j]
    #pragma unroll 1
    for (int jq = 0; jq < 2; ++jq) {
      const int jb = wg + 2 * jq;        // 32-column block handled by this warpgroup
      if (jb > rw) {                     // fully masked block (j > i for all rows of this warp)
        #pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const int jc = jb * 32 + ch * 8;
          const uint32_t off = (jc >> 6) * (TILE128 / 2) + sw128_offset(row, (jc & 63) >> 3);
          *reinterpret_cast<uint4*>(sM0 + off) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(sDCB + off) = make_uint4(0, 0, 0, 0);
        }
        s_col[rw * CT + jb * 32 + lane] = 0.f;
        continue;
      }
      uint32_t cb[32], dm[32];
      float wv[32];
      tmem_ld32(tmem_addr(tmem, rw * 32, jb * 32), cb);
      tmem_ld32(tmem_addr(tmem, rw * 32, 128 + jb * 32), dm);
      tmem_ld_wait();
      #pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        float m0[8], dc[8];
        #pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int j = jb * 32 + ch * 8 + e;
          const float lam = (j <= row) ? __expf(li - s_l[j]) : 0.f;
          m0[e] = __uint_as_float(cb[ch * 8 + e]) * lam;
          dc[e] = __uint_as_float(dm[ch * 8 + e]) * lam * s_dt[j];
          // W[i][j] = dM[i][j] * (CB Lambda dt_j)[i][j], strictly below the diagonal
          wv[ch * 8 + e] = (j < row) ? __uint_as_float(dm[ch * 8 + e]) * m0[e] * s_dt[j] : 0.f;
        }
        const int jc = jb * 32 + ch * 8;
        const uint32_t off = (jc >> 6) * (TILE128 / 2) + sw128_offset(row, (jc & 63) >> 3);
        *reinterpret_cast<uint4*>(sM0 + off) = pack8(m0);
        *reinterpret_cast<uint4*>(sDCB + off) = pack8(dc);
      }
      #pragma unroll
      for (int e = 0; e < 32; ++e) r1 += wv[e];
      // column sums of this 32x32 block over the warp's rows: recursive halving, lane c ends with column c
      #pragma unroll
      for (int sft = 16; sft >= 1; sft >>= 1) {
        const bool up = (lane & sft) != 0;
        #pragma unroll
        for (int k = 0; k < sft; ++k) {
          const float keep = up ? wv[k + sft] : wv[k];
          const float send = up ? wv[k] : wv[k + sft];
          wv[k] = keep + __shfl_xor_sync(0xffffffffu, send, sft);
        }
      }
      s_col[rw * CT + jb * 32 + lane] = wv[0];
    }
    // scaled copies of this thread's channel half (4 chunks of 8): x in place, dY into its own tile
    uint4 xrow[4];
    float dot_ss = 0.f;                  // share of <dS_out, S_in> (row n = `row`, channel half wg)
    {
      const float sx = a_right * dti;
      #pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t off = sw128_offset(row, wg * 4 + q);
        xrow[q] = *reinterpret_cast<const uint4*>(sX + off);
        float f[8], f2[8];
        unpack8(xrow[q], f);
        #pragma unroll
        for (int e = 0; e < 8; ++e) f[e] *= sx;
        *reinterpret_cast<uint4*>(sX + off) = pack8(f);
        unpack8(*reinterpret_cast<const uint4*>(sDY + off), f);
        #pragma unroll
        for (int e = 0; e < 8; ++e) f[e] *= a_left;
        *reinterpret_cast<uint4*>(sDYs + off) = pack8(f);
        unpack8(*reinterpret_cast<const uint4*>(sSin + off), f);
        unpack8(*reinterpret_cast<const uint4*>(sDS + off), f2);
        #pragma unroll
        for (int e = 0; e < 8; ++e) dot_ss += f[e] * f2[e];
      }
    }
    if (wg == 1) s_pair[row] = r1;
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    // ---------------------------------------------------------------- phase 2 MMAs
    if (tid == 0) {
      tc_fence_after_sync();
      const uint32_t id_u1 = make_idesc_bf16(128, PS, 1, 1);     // dU_diag[j][p] = sum_i M0[i][j] dY[i][p]
      #pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        umma_bf16(tmem, desc_mnmajor(aM0, kk, TILE128 / 2), desc_mnmajor(aDY, kk, 0), id_u1, kk != 0);
      const uint32_t id_u2 = make_idesc_bf16(128, PS, 0, 1);     // dU_state[j][p] = sum_n B[j][n] dS_out[n][p]
      #pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        umma_bf16(tmem + 64, desc_kmajor(aB, kk, TILE128 / 2), desc_mnmajor(aDS, kk, 0), id_u2, kk != 0);
      #pragma unroll
      for (int kk = 0; kk < 8; ++kk)                             // Yoff[i][p] = sum_n C[i][n] S_in[n][p]
        umma_bf16(tmem + 128, desc_kmajor(aC, kk, TILE128 / 2), desc_mnmajor(aSin, kk, 0), id_u2, kk != 0);
      const uint32_t id_b1 = make_idesc_bf16(128, 128, 1, 1);    // dB[j][n] += sum_i dCB[i][j] C[i][n]
      #pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        umma_bf16(tmem + 256, desc_mnmajor(aDCB, kk, TILE128 / 2), desc_mnmajor(aC, kk, TILE128 / 2), id_b1,
                  (it | kk) != 0);
      const uint32_t id_kk = make_idesc_bf16(128, 128, 0, 0);    // dB[j][n] += sum_p xs[j][p] dS_out[n][p]
      #pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        umma_bf16(tmem + 256, desc_kmajor(aX, kk, 0), desc_kmajor(aDS, kk, 0), id_kk, 1);
      const uint32_t id_c1 = make_idesc_bf16(128, 128, 0, 1);    // dC[i][n] += sum_j dCB[i][j] B[j][n]
      #pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        umma_bf16(tmem + 384, desc_kmajor(aDCB, kk, TILE128 / 2), desc_mnmajor(aB, kk, TILE128 / 2), id_c1,
                  (it | kk) != 0);
      #pragma unroll
      for (int kk = 0; kk < 4; ++kk)                             // dC[i][n] += sum_p dYs[i][p] S_in[n][p]
        umma_bf16(tmem + 384, desc_kmajor(aDYs, kk, 0), desc_kmajor(aSin, kk, 0), id_kk, 1);
      umma_commit(&bars[2]);
    }
    __syncwarp();
    ok = __syncthreads_and(mbar_wait(&bars[2], par, p.status));
    tc_fence_after_sync();
    if (!ok) break;
    // ---------------------------------------------------------------- epilogue (row j = `row`, channel half wg)
    const float Dh = p.D[h];
    float ddt_direct = 0.f, r2 = 0.f, q = 0.f, dD = 0.f;
    {
      uint32_t ud[32], us[32], yo[32];
      tmem_ld32(tmem_addr(tmem, rw * 32, wg * 32), ud);
      tmem_ld32(tmem_addr(tmem, rw * 32, 64 + wg * 32), us);
      tmem_ld32(tmem_addr(tmem, rw * 32, 128 + wg * 32), yo);
      tmem_ld_wait();
      #pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        float xv[8], gy[8], o[8];
        unpack8(xrow[ch], xv);
        unpack8(*reinterpret_cast<const uint4*>(sDY + sw128_offset(row, wg * 4 + ch)), gy);
        #pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float usr = __uint_as_float(us[ch * 8 + e]);
          const float dU = __uint_as_float(ud[ch * 8 + e]) + a_right * usr;
          ddt_direct += xv[e] * dU;
          q += xv[e] * usr;
          r2 += gy[e] * __uint_as_float(yo[ch * 8 + e]);
          dD += gy[e] * xv[e];
          o[e] = dti * dU + Dh * gy[e];
        }
        *reinterpret_cast<uint4*>(sX + sw128_offset(row, wg * 4 + ch)) = pack8(o);   // dx staging (x tile is dead)
      }
    }
    fence_proxy_async_smem();
    if (wg == 1) {                        // hand the per-row partials of the upper channel half to warpgroup 0
      s_pair[CT + row] = ddt_direct;
      s_pair[2 * CT + row] = r2;
      s_pair[3 * CT + row] = q;
    }
    // E = exp(l_T) <dS_out, S_in> + sum_j a_right dt_j q_j   (both are plain sums over all 256 threads)
    const float E = block_sum256(__expf(lT) * dot_ss + a_right * dti * q, s_red);
    if (tid == 0) { tma_store_2d(&tm_dx, sX, hv * PS, row0); tma_store_commit(); }
    float dl = 0.f;
    if (wg == 0) {
      r1 += s_pair[row];
      ddt_direct += s_pair[CT + row];
      r2 += s_pair[2 * CT + row];
      q += s_pair[3 * CT + row];
      const float c1 = s_col[row] + s_col[CT + row] + s_col[2 * CT + row] + s_col[3 * CT + row];
      dl = r1 + a_left * r2 - c1 - a_right * dti * q;
    }
    // suffix sum of dl over the 128 rows (warpgroup 0; warpgroup 1 carries zeros through the same barriers)
    float suf = dl;
    #pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float n = __shfl_down_sync(0xffffffffu, suf, o);
      if (lane + o < 32) suf += n;
    }
    __syncthreads();
    if (lane == 0 && wg == 0) s_red[8 + rw] = suf;      // warp totals
    __syncthreads();
    float ddr = 0.f, dta = 0.f;
    if (wg == 0) {
      float tail = 0.f;
      for (int w = rw + 1; w < 4; ++w) tail += s_red[8 + w];
      const float da = suf + tail + E;
      const float ddt = ddt_direct + p.A[h] * da;
      const float sig = sigmoid_f(__bfloat162float(p.dt_raw[(long long)(row0 + row) * p.dt_raw_stride + h]) + p.dt_bias[h]);
      ddr = ddt * sig;
      dta = dti * da;
      if (p.ddt32 != nullptr) p.ddt32[((long long)b * p.Hv + hv) * p.L + (long long)c * CT + row] = ddr;
      else p.ddt_raw[(long long)(row0 + row) * p.ddt_stride + h] = __float2bfloat16(ddr);
    }
    const float sA = block_sum256(dta, s_red);
    const float sD = block_sum256(dD, s_red);
    const float sb = block_sum256(ddr, s_red);
    if (tid == 0) {
      float* hp = p.hpart + (((long long)b * p.nc + c) * p.Hv + hv) * 3;
      hp[0] = sA; hp[1] = sD; hp[2] = sb;
      tma_store_wait_read();      // the dx staging tile is reloaded as x by the next head
    }
    tc_fence_before_sync();
    __syncthreads();
  }
  // ---------------------------------------------------------------- flush dB (warpgroup 0), dC (warpgroup 1)
  if (ok) {
    tc_fence_after_sync();
    const int GN = p.G * NS;
    float* dst = p.dBC + (long long)(row0 + row) * (2 * GN) + wg * GN + g * NS;
    #pragma unroll 1
    for (int nb = 0; nb < 4; ++nb) {
      uint32_t v[32];
      tmem_ld32(tmem_addr(tmem, rw * 32, 256 + wg * 128 + nb * 32), v);
      tmem_ld_wait();
      #pragma unroll
      for (int k4 = 0; k4 < 8; ++k4)
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + nb * 32 + k4 * 4),
                     "f"(__uint_as_float(v[k4 * 4])), "f"(__uint_as_float(v[k4 * 4 + 1])),
                     "f"(__uint_as_float(v[k4 * 4 + 2])), "f"(__uint_as_float(v[k4 * 4 + 3])) : "memory");
    }
  }
  if (tid == 0) tma_store_wait_all();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace ssm

// ------------------------------------------------------------------------------------ C API
using namespace ssm;

static int smem_opt_in(const void* fn, int bytes) {
  return (int)cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

extern "C" int ssm_ssd_dt_prep(const void* dt_raw, long long row_stride, const void* dt_bias, const void* A,
                               void* dt_out, void* l_out, int B, int L, int H, cudaStream_t st) {
  if (L % CT) return -SSM_ERR_BAD_ARG;
  dim3 grid(L / CT, H, B);
  ssd_dt_prep_kernel<<<grid, 128, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(dt_raw), row_stride,
                                           reinterpret_cast<const float*>(dt_bias), reinterpret_cast<const float*>(A),
                                           reinterpret_cast<float*>(dt_out), reinterpret_cast<float*>(l_out), L, H);
  return (int)cudaGetLastError();
}

// w_src: bf16 [B*L, w_cols] (row stride w_stride) holding W (B or C of every group) starting at column w_col0.
// v: bf16 rows (b*L+t)*v_stride + hv*64.   out fp32 [B,Hv,nc,128,64].
extern "C" int ssm_ssd_chunk_state(const void* w_src, long long w_stride, int w_cols, int w_col0, const void* v,
                                   long long v_stride, const void* dt, const void* l, void* out, int B, int L, int H,
                                   int Hv, int G, int mode, int* status, cudaStream_t st) {
  if (L % CT || Hv % H || H % G || w_stride % 8 || v_stride % 8) return -SSM_ERR_BAD_ARG;
  static bool cfg = false;
  const int smem = TILE128 + TILE64 + 64 + 1024;
  if (!cfg) { int e = smem_opt_in((const void*)ssd_chunk_state_kernel, smem); if (e) return e; cfg = true; }
  CUtensorMap tm;
  int r = make_tmap_2d_bf16(&tm, w_src, (uint64_t)w_cols, (uint64_t)B * L, (uint64_t)w_stride * 2, 64, 128);
  if (r) return -100 - r;
  ChunkStateParams p;
  p.v = reinterpret_cast<const __nv_bfloat16*>(v); p.v_row_stride = v_stride;
  p.dt = reinterpret_cast<const float*>(dt); p.l = reinterpret_cast<const float*>(l);
  p.out = reinterpret_cast<float*>(out);
  p.L = L; p.H = H; p.Hv = Hv; p.G = G; p.nc = L / CT; p.w_col0 = w_col0; p.mode = mode; p.status = status;
  dim3 grid(L / CT, Hv, B);
  ssd_chunk_state_kernel<<<grid, 128, smem, st>>>(tm, p);
  return (int)cudaGetLastError();
}

extern "C" int ssm_ssd_state_pass(const void* local, const void* l, const void* init, void* in16, void* fin, int B,
                                  int L, int H, int Hv, int reverse, cudaStream_t st) {
  dim3 grid(NS * PS / 4 / 256, Hv, B);
  ssd_state_pass_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const float*>(local), reinterpret_cast<const float*>(l),
                                              reinterpret_cast<const float*>(init),
                                              reinterpret_cast<__nv_bfloat16*>(in16), reinterpret_cast<float*>(fin), L,
                                              H, Hv, L / CT, reverse);
  return (int)cudaGetLastError();
}

// xbc: conv output bf16 [B*L, xbc_cols] (x | B | C), row stride xbc_stride.  s_in bf16 [B*Hv*nc*128, 64].
// y: bf16 [B*L, Hv*64] row stride y_stride (written).
extern "C" int ssm_ssd_chunk_scan_fwd(const void* xbc, long long xbc_stride, int xbc_cols, const void* s_in, void* y,
                                      long long y_stride, const void* dt, const void* l, const void* D, int B, int L,
                                      int H, int Hv, int G, int d_in, int* status, cudaStream_t st) {
  if (L % CT || Hv % H || H % G || xbc_stride % 8 || y_stride % 8) return -SSM_ERR_BAD_ARG;
  static bool cfg = false;
  const int smem = 2 * TILE128 + 2 * TILE64 + 2 * CT * 4 + 64 + 1024;
  if (!cfg) { int e = smem_opt_in((const void*)ssd_chunk_scan_fwd_kernel, smem); if (e) return e; cfg = true; }
  const int nc = L / CT;
  CUtensorMap tx, ts, ty;
  int r = make_tmap_2d_bf16(&tx, xbc, (uint64_t)xbc_cols, (uint64_t)B * L, (uint64_t)xbc_stride * 2, 64, 128);
  if (r) return -100 - r;
  r = make_tmap_2d_bf16(&ts, s_in, 64, (uint64_t)B * Hv * nc * NS, 128, 64, 128);
  if (r) return -200 - r;
  r = make_tmap_2d_bf16(&ty, y, (uint64_t)Hv * PS, (uint64_t)B * L, (uint64_t)y_stride * 2, 64, 128);
  if (r) return -300 - r;
  ScanFwdParams p;
  p.dt = reinterpret_cast<const float*>(dt); p.l = reinterpret_cast<const float*>(l);
  p.D = reinterpret_cast<const float*>(D);
  p.L = L; p.H = H; p.Hv = Hv; p.G = G; p.nc = nc; p.d_in = d_in; p.status = status;
  dim3 grid(nc, Hv, B);
  ssd_chunk_scan_fwd_kernel<<<grid, 128, smem, st>>>(tx, ts, ty, p);
  return (int)cudaGetLastError();
}

// dy: bf16 [B*L, Hv*64] (row stride dy_stride).  dx: bf16 [B*L, Hv*64] written (row stride dx_stride).
// dBC: fp32 [B*L, 2*G*128], must be zero on entry.  hpart: fp32 [B*nc, Hv, 3].
// ddt: if ddt32 != null it receives fp32 [B,Hv,L]; else bf16 values are written to ddt_raw rows.
extern "C" int ssm_ssd_chunk_scan_bwd(const void* xbc, long long xbc_stride, int xbc_cols, const void* dy,
                                      long long dy_stride, const void* s_in,
                                      const void* ds_out, void* dx, long long dx_stride, void* dBC, void* hpart,
                                      void* ddt_raw, long long ddt_stride, void* ddt32, const void* dt_raw,
                                      long long dt_raw_stride, const void* dt_bias, const void* A, const void* dt,
                                      const void* l, const void* D, int B, int L, int H, int Hv, int G, int d_in,
                                      int hpc, int* status, cudaStream_t st) {
  if (L % CT || Hv % H || H % G || xbc_stride % 8 || dy_stride % 8 || dx_stride % 8)
    return -SSM_ERR_BAD_ARG;
  const int hv_per_group = Hv / G;
  if (hpc <= 0 || hv_per_group % hpc) return -SSM_ERR_BAD_ARG;
  static bool cfg = false;
  const int smem = BWD_SMEM + (11 * CT + 16) * 4 + 64 + 1024;
  if (!cfg) { int e = smem_opt_in((const void*)ssd_chunk_scan_bwd_kernel, smem); if (e) return e; cfg = true; }
  const int nc = L / CT;
  CUtensorMap tx, tdy, ts, tds, tdx;
  int r = make_tmap_2d_bf16(&tx, xbc, (uint64_t)xbc_cols, (uint64_t)B * L, (uint64_t)xbc_stride * 2, 64, 128);
  if (r) return -100 - r;
  r = make_tmap_2d_bf16(&tdy, dy, (uint64_t)Hv * PS, (uint64_t)B * L, (uint64_t)dy_stride * 2, 64, 128);
  if (r) return -200 - r;
  r = make_tmap_2d_bf16(&ts, s_in, 64, (uint64_t)B * Hv * nc * NS, 128, 64, 128);
  if (r) return -300 - r;
  r = make_tmap_2d_bf16(&tds, ds_out, 64, (uint64_t)B * Hv * nc * NS, 128, 64, 128);
  if (r) return -400 - r;
  r = make_tmap_2d_bf16(&tdx, dx, (uint64_t)Hv * PS, (uint64_t)B * L, (uint64_t)dx_stride * 2, 64, 128);
  if (r) return -500 - r;
  ScanBwdParams p;
  p.dt = reinterpret_cast<const float*>(dt); p.l = reinterpret_cast<const float*>(l);
  p.D = reinterpret_cast<const float*>(D); p.A = reinterpret_cast<const float*>(A);
  p.dt_bias = reinterpret_cast<const float*>(dt_bias);
  p.dt_raw = reinterpret_cast<const __nv_bfloat16*>(dt_raw); p.dt_raw_stride = dt_raw_stride;
  p.ddt_raw = reinterpret_cast<__nv_bfloat16*>(ddt_raw); p.ddt_stride = ddt_stride;
  p.ddt32 = reinterpret_cast<float*>(ddt32);
  p.dBC = reinterpret_cast<float*>(dBC); p.hpart = reinterpret_cast<float*>(hpart);
  p.L = L; p.H = H; p.Hv = Hv; p.G = G; p.nc = nc; p.d_in = d_in; p.hpc = hpc; p.status = status;
  dim3 grid(nc, G * (hv_per_group / hpc), B);
  ssd_chunk_scan_bwd_kernel<<<grid, 256, smem, st>>>(tx, tdy, ts, tds, tdx, p);
  return (int)cudaGetLastError();
}
