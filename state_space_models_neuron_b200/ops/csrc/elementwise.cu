// Memory-bound kernels of the Mamba-2 block for sm_100a: causal depthwise conv1d + SiLU (fwd/bwd),
// gated group RMSNorm (fwd/bwd), residual-add + RMSNorm (fwd/bwd), GELU (fwd/bwd), vocab-shard cross
// entropy statistics and gradient, fused AdamW and sum of squares.  All io is 16-byte vectorised bf16,
// all arithmetic fp32.  Reference counterparts: mamba2/conv1d_grouped.py:65-194 (conv),
// mamba2/fused_kernel.py:76-175 (gated norm), mamba2/modeling_mamba2.py:94-103 (RMSNorm).
#include "common.cuh"

namespace ssm {

struct alignas(16) bf16x8 { __nv_bfloat162 v[4]; };

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  f[0] = bf16_lo(u.x); f[1] = bf16_hi(u.x); f[2] = bf16_lo(u.y); f[3] = bf16_hi(u.y);
  f[4] = bf16_lo(u.z); f[5] = bf16_hi(u.z); f[6] = bf16_lo(u.w); f[7] = bf16_hi(u.w);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16(f[0], f[1]); u.y = pack_bf16(f[2], f[3]); u.z = pack_bf16(f[4], f[5]); u.w = pack_bf16(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ void load8f(const float* p, float (&f)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ void store8f(float* p, const float (&f)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}

__device__ __forceinline__ float warp_sum(float v) {
  #pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
  #pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Sum over the block; every thread gets the result.  `red` holds >= 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : -INFINITY;
  t = warp_max(t);
  return t;
}

// =====================================================================================
// causal depthwise conv1d (4 taps) + SiLU, channels-last
// =====================================================================================
constexpr int CONV_TOK = 32;   // tokens per thread at full size; small problems use shorter tiles (more CTAs)
constexpr int CONV_K = 4;

// x [B, L, C] with row stride xs (elements); out row stride os.  init [B, 3, C] (tokens preceding x) or null.
template <int TOK>
__global__ void __launch_bounds__(128)
conv1d_silu_fwd_kernel(const __nv_bfloat16* __restrict__ x, long long xs, const __nv_bfloat16* __restrict__ w,
                       const __nv_bfloat16* __restrict__ bias, const __nv_bfloat16* __restrict__ init,
                       __nv_bfloat16* __restrict__ out, long long os, int L, int C) {
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c0 >= C) return;
  if (!SSM_INDEX_OK(c0 + 7, C) || !SSM_INDEX_OK(C - 1, xs) || !SSM_INDEX_OK(C - 1, os)) return;   // whole 8-channel vectors inside a row
  const int t0 = blockIdx.y * TOK;
  const int b = blockIdx.z;
  float wt[CONV_K][8], bs[8];
  #pragma unroll
  for (int e = 0; e < 8; ++e) {
    #pragma unroll
    for (int k = 0; k < CONV_K; ++k) wt[k][e] = __bfloat162float(w[(c0 + e) * CONV_K + k]);
    bs[e] = bias ? __bfloat162float(bias[c0 + e]) : 0.f;
  }
  const __nv_bfloat16* xb = x + (long long)b * L * xs + c0;
  __nv_bfloat16* ob = out + (long long)b * L * os + c0;
  float h[3][8];   // x[t-3], x[t-2], x[t-1]
  #pragma unroll
  for (int k = 0; k < 3; ++k) {
    const int t = t0 - 3 + k;
    if (t >= 0) load8(xb + (long long)t * xs, h[k]);
    else if (init != nullptr) load8(init + ((long long)b * 3 + (t + 3)) * C + c0, h[k]);
    else {
      #pragma unroll
      for (int e = 0; e < 8; ++e) h[k][e] = 0.f;
    }
  }
  #pragma unroll 4
  for (int i = 0; i < TOK; ++i) {
    const int t = t0 + i;
    if (t >= L) break;
    float cur[8], o[8];
    load8(xb + (long long)t * xs, cur);
    #pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float pre = bs[e] + wt[0][e] * h[0][e] + wt[1][e] * h[1][e] + wt[2][e] * h[2][e] + wt[3][e] * cur[e];
      o[e] = silu_f(pre);
      h[0][e] = h[1][e]; h[1][e] = h[2][e]; h[2][e] = cur[e];
    }
    store8(ob + (long long)t * os, o);
  }
}

// Backward.  dy for channels [0, c_split) comes from dy16 (bf16, row stride ds16); channels >= c_split from
// dy32 (fp32, row stride ds32, indexed by channel - c_split).  dx is written with row stride dxs.
// part [gridDim.z * gridDim.y, C, 5] receives per-tile partial sums (dw[0..3], db).
// Each thread owns 4 channels and walks CONV_TOK (+3 halo) tokens; loads are issued four tokens at a time before
// any arithmetic so that every thread keeps 8 requests in flight.
constexpr int CONV_CPT = 4;

__device__ __forceinline__ void unpack4(const uint2 u, float (&f)[4]) {
  f[0] = bf16_lo(u.x); f[1] = bf16_hi(u.x); f[2] = bf16_lo(u.y); f[3] = bf16_hi(u.y);
}

template <int TOK>
__global__ void __launch_bounds__(128, 4)
conv1d_silu_bwd_kernel(const __nv_bfloat16* __restrict__ x, long long xs, const __nv_bfloat16* __restrict__ w,
                       const __nv_bfloat16* __restrict__ bias, const __nv_bfloat16* __restrict__ dy16, long long ds16,
                       const float* __restrict__ dy32, long long ds32, int c_split,
                       __nv_bfloat16* __restrict__ dx, long long dxs, float* __restrict__ part, int L, int C) {
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * CONV_CPT;
  if (c0 >= C) return;
  const int t0 = blockIdx.y * TOK;
  const int b = blockIdx.z;
  float wt[CONV_K][CONV_CPT], bs[CONV_CPT];
  #pragma unroll
  for (int e = 0; e < CONV_CPT; ++e) {
    #pragma unroll
    for (int k = 0; k < CONV_K; ++k) wt[k][e] = __bfloat162float(w[(c0 + e) * CONV_K + k]);
    bs[e] = bias ? __bfloat162float(bias[c0 + e]) : 0.f;
  }
  const __nv_bfloat16* xb = x + (long long)b * L * xs + c0;
  const bool lo = c0 < c_split;
  float xw[3][CONV_CPT], dp[CONV_K][CONV_CPT], dw[CONV_K][CONV_CPT], db[CONV_CPT];
  #pragma unroll
  for (int e = 0; e < CONV_CPT; ++e) {
    db[e] = 0.f;
    #pragma unroll
    for (int k = 0; k < CONV_K; ++k) { dw[k][e] = 0.f; dp[k][e] = 0.f; }
  }
  #pragma unroll
  for (int k = 0; k < 3; ++k) {
    const int t = t0 - 3 + k;
    if (t >= 0) unpack4(*reinterpret_cast<const uint2*>(xb + (long long)t * xs), xw[k]);
    else {
      #pragma unroll
      for (int e = 0; e < CONV_CPT; ++e) xw[k][e] = 0.f;
    }
  }
  constexpr int NSTEP = TOK + 3;
  constexpr int NB = (NSTEP + 3) / 4;
  #pragma unroll 1
  for (int ib = 0; ib < NB; ++ib) {
    uint2 xr[4], g16[4];
    float4 g32[4];
    #pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int t = t0 + ib * 4 + k;
      if (t < L && ib * 4 + k < NSTEP) {
        xr[k] = *reinterpret_cast<const uint2*>(xb + (long long)t * xs);
        if (lo) g16[k] = *reinterpret_cast<const uint2*>(dy16 + ((long long)b * L + t) * ds16 + c0);
        else g32[k] = *reinterpret_cast<const float4*>(dy32 + ((long long)b * L + t) * ds32 + (c0 - c_split));
      }
    }
    #pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int i = ib * 4 + k;
      const int t = t0 + i;
      if (i >= NSTEP) break;
      const bool valid = t < L;
      float cur[CONV_CPT], g[CONV_CPT], d[CONV_CPT];
      if (valid) {
        unpack4(xr[k], cur);
        if (lo) unpack4(g16[k], g);
        else { g[0] = g32[k].x; g[1] = g32[k].y; g[2] = g32[k].z; g[3] = g32[k].w; }
      }
      #pragma unroll
      for (int e = 0; e < CONV_CPT; ++e) {
        float dpre = 0.f;
        if (valid) {
          const float pre = bs[e] + wt[0][e] * xw[0][e] + wt[1][e] * xw[1][e] + wt[2][e] * xw[2][e] + wt[3][e] * cur[e];
          const float sg = sigmoid_f(pre);
          dpre = g[e] * sg * (1.f + pre * (1.f - sg));
          if (i < TOK) {
            dw[0][e] += xw[0][e] * dpre; dw[1][e] += xw[1][e] * dpre; dw[2][e] += xw[2][e] * dpre;
            dw[3][e] += cur[e] * dpre; db[e] += dpre;
          }
        } else {
          cur[e] = 0.f;
        }
        dp[0][e] = dp[1][e]; dp[1][e] = dp[2][e]; dp[2][e] = dp[3][e]; dp[3][e] = dpre;
        // dx[t-3] = w3*dpre[t-3] + w2*dpre[t-2] + w1*dpre[t-1] + w0*dpre[t]
        d[e] = wt[3][e] * dp[0][e] + wt[2][e] * dp[1][e] + wt[1][e] * dp[2][e] + wt[0][e] * dp[3][e];
        xw[0][e] = xw[1][e]; xw[1][e] = xw[2][e]; xw[2][e] = cur[e];
      }
      const int td = t - 3;
      if (i >= 3 && td < L) {
        uint2 o;
        o.x = pack_bf16(d[0], d[1]); o.y = pack_bf16(d[2], d[3]);
        *reinterpret_cast<uint2*>(dx + ((long long)b * L + td) * dxs + c0) = o;
      }
    }
  }
  float* pp = part + ((long long)(blockIdx.z * gridDim.y + blockIdx.y) * C + c0) * 5;
  #pragma unroll
  for (int e = 0; e < CONV_CPT; ++e) {
    pp[e * 5 + 0] = dw[0][e]; pp[e * 5 + 1] = dw[1][e]; pp[e * 5 + 2] = dw[2][e]; pp[e * 5 + 3] = dw[3][e];
    pp[e * 5 + 4] = db[e];
  }
}

// =====================================================================================
// gated group RMSNorm:  out = w * h * rsqrt(mean_g(h^2) + eps),  h = y * silu(z)
// one block per (row, group); thread handles vectors v = tid, tid + blockDim, ... of 8 elements
// =====================================================================================
// MAXV = 16-byte vectors per thread.  Rows up to 8192 elements run with one vector per thread and up to 1024
// threads (few registers, full occupancy); longer rows use four vectors per thread.

template <int NORM_MAXV>
__global__ void __launch_bounds__(NORM_MAXV == 1 ? 1024 : 256)
gated_rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ y, long long ys, const __nv_bfloat16* __restrict__ z,
                         long long zs, const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out,
                         long long os, int gs, float eps) {
  __shared__ float red[33];
  const long long row = blockIdx.x;
  const int g = blockIdx.y;
  const int nvec = gs / 8;
  const __nv_bfloat16* yr = y + row * ys + (long long)g * gs;
  const __nv_bfloat16* zr = z ? z + row * zs + (long long)g * gs : nullptr;
  float h[NORM_MAXV][8];
  float ss = 0.f;
  #pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      float a[8];
      load8(yr + v * 8, a);
      if (zr) {
        float zz[8];
        load8(zr + v * 8, zz);
        #pragma unroll
        for (int e = 0; e < 8; ++e) a[e] *= silu_f(zz[e]);
      }
      #pragma unroll
      for (int e = 0; e < 8; ++e) { h[i][e] = a[e]; ss += a[e] * a[e]; }
    }
  }
  const float rstd = rsqrtf(block_sum(ss, red) / gs + eps);
  #pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      float ww[8], o[8];
      load8(w + (long long)g * gs + v * 8, ww);
      #pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = ww[e] * h[i][e] * rstd;
      store8(out + row * os + (long long)g * gs + v * 8, o);
    }
  }
}

// grid (row_slices, groups); each block walks rows r = blockIdx.x, blockIdx.x + gridDim.x, ...
// dwpart [gridDim.x, d] fp32 partial sums of dout * h * rstd.
template <int NORM_MAXV>
__global__ void __launch_bounds__(NORM_MAXV == 1 ? 1024 : 256)
gated_rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ y, long long ys, const __nv_bfloat16* __restrict__ z,
                         long long zs, const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ dout,
                         long long dos, __nv_bfloat16* __restrict__ dy, long long dys, __nv_bfloat16* __restrict__ dz,
                         long long dzs, float* __restrict__ dwpart, long long rows, int d, int gs, float eps) {
  __shared__ float red[33];
  const int g = blockIdx.y;
  const int nvec = gs / 8;
  float ww[NORM_MAXV][8], dwacc[NORM_MAXV][8];
  #pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    #pragma unroll
    for (int e = 0; e < 8; ++e) dwacc[i][e] = 0.f;
    if (v < nvec) load8(w + (long long)g * gs + v * 8, ww[i]);
  }
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const long long off = (long long)g * gs;
    float h[NORM_MAXV][8], dn[NORM_MAXV][8];
    float ss = 0.f, dot = 0.f;
    #pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        float a[8], go[8];
        load8(y + row * ys + off + v * 8, a);
        load8(dout + row * dos + off + v * 8, go);
        if (z) {
          float zz[8];
          load8(z + row * zs + off + v * 8, zz);
          #pragma unroll
          for (int e = 0; e < 8; ++e) a[e] *= silu_f(zz[e]);
        }
        #pragma unroll
        for (int e = 0; e < 8; ++e) {
          h[i][e] = a[e]; dn[i][e] = go[e] * ww[i][e];
          ss += a[e] * a[e]; dot += dn[i][e] * a[e];
        }
      }
    }
    const float rstd = rsqrtf(block_sum(ss, red) / gs + eps);
    const float mdot = block_sum(dot, red) * rstd / gs;     // mean(dn * n), n = h * rstd
    #pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        float yy[8], zz[8], oy[8], oz[8];
        load8(y + row * ys + off + v * 8, yy);
        if (z) load8(z + row * zs + off + v * 8, zz);
        #pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float n = h[i][e] * rstd;
          const float dh = rstd * (dn[i][e] - n * mdot);
          if (z) {
            const float s = sigmoid_f(zz[e]);
            oy[e] = dh * zz[e] * s;
            oz[e] = dh * yy[e] * s * (1.f + zz[e] * (1.f - s));
          } else {
            oy[e] = dh; oz[e] = 0.f;
          }
        }
        // dw += dout * n
        float go[8];
        load8(dout + row * dos + off + v * 8, go);
        #pragma unroll
        for (int e = 0; e < 8; ++e) dwacc[i][e] += go[e] * h[i][e] * rstd;
        store8(dy + row * dys + off + v * 8, oy);
        if (z) store8(dz + row * dzs + off + v * 8, oz);
      }
    }
  }
  #pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) store8f(dwpart + (long long)blockIdx.x * d + (long long)g * gs + v * 8, dwacc[i]);
  }
}

// =====================================================================================
// residual add + RMSNorm:  r' = r + x ;  out = w * r' * rsqrt(mean(r'^2) + eps)
// one block per row.  Residual stream may be bf16 or fp32.
// =====================================================================================
template <typename RT>
__device__ __forceinline__ void load8r(const RT* p, float (&f)[8]);
template <> __device__ __forceinline__ void load8r<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[8]) { load8(p, f); }
template <> __device__ __forceinline__ void load8r<float>(const float* p, float (&f)[8]) { load8f(p, f); }
template <typename RT>
__device__ __forceinline__ void store8r(RT* p, const float (&f)[8]);
template <> __device__ __forceinline__ void store8r<__nv_bfloat16>(__nv_bfloat16* p, const float (&f)[8]) { store8(p, f); }
template <> __device__ __forceinline__ void store8r<float>(float* p, const float (&f)[8]) { store8f(p, f); }

template <typename RT, int NORM_MAXV>
__global__ void __launch_bounds__(NORM_MAXV == 1 ? 1024 : 256)
add_rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const RT* __restrict__ res, const __nv_bfloat16* __restrict__ w,
                       __nv_bfloat16* __restrict__ out, RT* __restrict__ res_out, int D, float eps) {
  __shared__ float red[33];
  const long long row = blockIdx.x;
  const int nvec = D / 8;
  float r[NORM_MAXV][8];
  float ss = 0.f;
  #pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      float a[8];
      load8(x + row * D + v * 8, a);
      if (res) {
        float b[8];
        load8r<RT>(res + row * D + v * 8, b);
        #pragma unroll
        for (int e = 0; e < 8; ++e) a[e] += b[e];
      }
      if (res_out) store8r<RT>(res_out + row * D + v * 8, a);
      #pragma unroll
      for (int e = 0; e < 8; ++e) { r[i][e] = a[e]; ss += a[e] * a[e]; }
    }
  }
  const float rstd = rsqrtf(block_sum(ss, red) / D + eps);
  #pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      float ww[8], o[8];
      load8(w + v * 8, ww);
      #pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = ww[e] * r[i][e] * rstd;
      store8(out + row * D + v * 8, o);
    }
  }
}

// d_sum = d_res_out + rmsnorm_bwd(d_out);  dwpart [gridDim.x, D].  res = the summed residual r' saved by fwd.
template <typename RT, int NORM_MAXV>
__global__ void __launch_bounds__(NORM_MAXV == 1 ? 1024 : 256)
add_rmsnorm_bwd_kernel(const RT* __restrict__ res, const __nv_bfloat16* __restrict__ w,
                       const __nv_bfloat16* __restrict__ dout, const RT* __restrict__ dres_out,
                       RT* __restrict__ dsum, float* __restrict__ dwpart, long long rows, int D, float eps) {
  __shared__ float red[33];
  const int nvec = D / 8;
  float ww[NORM_MAXV][8], dwacc[NORM_MAXV][8];
  #pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    #pragma unroll
    for (int e = 0; e < 8; ++e) dwacc[i][e] = 0.f;
    if (v < nvec) load8(w + v * 8, ww[i]);
  }
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    float r[NORM_MAXV][8], go[NORM_MAXV][8];
    float ss = 0.f, dot = 0.f;
    #pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        load8r<RT>(res + row * D + v * 8, r[i]);
        load8(dout + row * D + v * 8, go[i]);
        #pragma unroll
        for (int e = 0; e < 8; ++e) { ss += r[i][e] * r[i][e]; dot += go[i][e] * ww[i][e] * r[i][e]; }
      }
    }
    const float rstd = rsqrtf(block_sum(ss, red) / D + eps);
    const float mdot = block_sum(dot, red) * rstd / D;
    #pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        float o[8];
        if (dres_out) load8r<RT>(dres_out + row * D + v * 8, o);
        else {
          #pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = 0.f;
        }
        #pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float n = r[i][e] * rstd;
          o[e] += rstd * (go[i][e] * ww[i][e] - n * mdot);
          dwacc[i][e] += go[i][e] * n;
        }
        store8r<RT>(dsum + row * D + v * 8, o);
      }
    }
  }
  #pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) store8f(dwpart + (long long)blockIdx.x * D + v * 8, dwacc[i]);
  }
}

// =====================================================================================
// GELU (erf) forward / backward, 8 elements per thread
// =====================================================================================
__global__ void gelu_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n8) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float a[8];
    load8(x + i * 8, a);
    #pragma unroll
    for (int e = 0; e < 8; ++e) a[e] = 0.5f * a[e] * (1.f + erff(a[e] * 0.70710678118654752f));
    store8(y + i * 8, a);
  }
}
__global__ void gelu_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                __nv_bfloat16* __restrict__ dx, long long n8) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float a[8], g[8];
    load8(x + i * 8, a);
    load8(dy + i * 8, g);
    #pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float cdf = 0.5f * (1.f + erff(a[e] * 0.70710678118654752f));
      const float pdf = 0.3989422804014327f * __expf(-0.5f * a[e] * a[e]);
      g[e] *= cdf + a[e] * pdf;
    }
    store8(dx + i * 8, g);
  }
}

// =====================================================================================
// vocab-shard cross entropy: per row (max, sum exp(l - max), target logit), and the gradient
// =====================================================================================
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__global__ void __launch_bounds__(256)
ce_partials_kernel(const T* __restrict__ logits, long long ld, const long long* __restrict__ labels, int V,
                   int vocab_start, float* __restrict__ omax, float* __restrict__ osum, float* __restrict__ otgt) {
  __shared__ float red[33];
  const long long row = blockIdx.x;
  const T* lr = logits + row * ld;
  float m = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) m = fmaxf(m, to_f<T>(lr[i]));
  m = block_max(m, red);
  float s = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) s += __expf(to_f<T>(lr[i]) - m);
  s = block_sum(s, red);
  if (threadIdx.x == 0) {
    const long long loc = labels[row] - vocab_start;
    omax[row] = m; osum[row] = s;
    otgt[row] = (loc >= 0 && loc < V) ? to_f<T>(lr[loc]) : 0.f;
  }
}

// grad[row, i] = (exp(l - gmax) / gsum - [i == label]) * g[row];  gmax/gsum are the global statistics.
template <typename T>
__global__ void __launch_bounds__(256)
ce_backward_kernel(const T* __restrict__ logits, long long ld, const long long* __restrict__ labels, int V,
                   int vocab_start, long long ignore_index, const float* __restrict__ gmax,
                   const float* __restrict__ gsum, const float* __restrict__ grow, T* __restrict__ grad, long long gld) {
  const long long row = blockIdx.x;
  const long long lab = labels[row];
  const float g = (lab == ignore_index) ? 0.f : grow[row];
  const float m = gmax[row], inv = 1.f / gsum[row];
  const long long loc = lab - vocab_start;
  const T* lr = logits + row * ld;
  T* gr = grad + row * gld;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float p = __expf(to_f<T>(lr[i]) - m) * inv;
    if (i == loc) p -= 1.f;
    p *= g;
    if constexpr (sizeof(T) == 2) gr[i] = __float2bfloat16(p); else gr[i] = p;
  }
}

// =====================================================================================
// Rotary position embedding (rotate-half convention) on the first `rd` channels of every head:
//   out[:, :rd/2] = x1 * cos - sign * x2 * sin,   out[:, rd/2:rd] = x2 * cos + sign * x1 * sin
// x, out: [tokens, H, Dh] bf16 with a token stride; cos / sin: fp32 tables [L, rd/2], position = token % L + offset
// already folded into the table.  sign = +1 applies the rotation (forward), -1 its inverse (the backward pass:
// the Jacobian of a rotation is the rotation by the opposite angle).  Channels >= rd are copied.
// The reference's rotary helpers are mamba2hybrid/mamba2hybrid_attn.py:101-226 (applied at :428-430).
// =====================================================================================
__global__ void __launch_bounds__(256)
rope_kernel(const __nv_bfloat16* __restrict__ x, long long x_ld, __nv_bfloat16* __restrict__ out, long long out_ld,
            const float* __restrict__ cs, const float* __restrict__ sn, long long tokens, int L, int H, int Dh, int rd,
            float sign) {
  const int half = rd / 2;
  const int vec_rot = half / 8;                 // 8-channel vectors in each rotated half
  const int vec_rest = (Dh - rd) / 8;
  const int per_head = vec_rot + vec_rest;
  const long long total = tokens * H * per_head;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(i % per_head);
    const long long th = i / per_head;
    const int h = (int)(th % H);
    const long long t = th / H;
    const __nv_bfloat16* xr = x + t * x_ld + (long long)h * Dh;
    __nv_bfloat16* orow = out + t * out_ld + (long long)h * Dh;
    if (v >= vec_rot) {                          // pass-through channels
      const int c = rd + (v - vec_rot) * 8;
      *reinterpret_cast<uint4*>(orow + c) = *reinterpret_cast<const uint4*>(xr + c);
      continue;
    }
    const int c = v * 8;
    const uint4 a = *reinterpret_cast<const uint4*>(xr + c);
    const uint4 b = *reinterpret_cast<const uint4*>(xr + half + c);
    if (!SSM_INDEX_OK((long long)h * Dh + half + c + 7, x_ld) || !SSM_INDEX_OK((long long)h * Dh + half + c + 7, out_ld)) continue;
    const float* cp = cs + (t % L) * half + c;
    const float* sp = sn + (t % L) * half + c;
    const float4 c0 = *reinterpret_cast<const float4*>(cp), c1 = *reinterpret_cast<const float4*>(cp + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(sp), s1 = *reinterpret_cast<const float4*>(sp + 4);
    const float cc[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float ss[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    const uint32_t ap[4] = {a.x, a.y, a.z, a.w}, bp[4] = {b.x, b.y, b.z, b.w};
    uint32_t o1[4], o2[4];
    #pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float x1l = bf16_lo(ap[e]), x1h = bf16_hi(ap[e]), x2l = bf16_lo(bp[e]), x2h = bf16_hi(bp[e]);
      const float sl = sign * ss[2 * e], sh = sign * ss[2 * e + 1];
      o1[e] = pack_bf16(x1l * cc[2 * e] - x2l * sl, x1h * cc[2 * e + 1] - x2h * sh);
      o2[e] = pack_bf16(x2l * cc[2 * e] + x1l * sl, x2h * cc[2 * e + 1] + x1h * sh);
    }
    *reinterpret_cast<uint4*>(orow + c) = make_uint4(o1[0], o1[1], o1[2], o1[3]);
    *reinterpret_cast<uint4*>(orow + half + c) = make_uint4(o2[0], o2[1], o2[2], o2[3]);
  }
}

// Row statistics that a GEMM epilogue produced per column tile -> one (max, sum exp(x - max)) per row.
// tmax / tsum: [tiles][rows].
__global__ void __launch_bounds__(256)
ce_merge_tiles_kernel(const float* __restrict__ tmax, const float* __restrict__ tsum, int tiles, long long rows,
                      float* __restrict__ omax, float* __restrict__ osum) {
  const long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float m = -INFINITY;
  for (int t = 0; t < tiles; ++t) m = fmaxf(m, tmax[(long long)t * rows + r]);
  float s = 0.f;
  for (int t = 0; t < tiles; ++t) s += tsum[(long long)t * rows + r] * __expf(tmax[(long long)t * rows + r] - m);
  omax[r] = m;
  osum[r] = s;
}

// =====================================================================================
// AdamW on a flat fp32 master shard + low-precision copy; sum of squares
// =====================================================================================
// 4 elements per thread per iteration, 16-byte loads/stores; n4 = n / 4 (segments are multiples of 128 elements)
template <typename GT> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    return make_float4(bf16_lo(u.x), bf16_hi(u.x), bf16_lo(u.y), bf16_hi(u.y));
  }
};

template <typename GT>
__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
             const GT* __restrict__ g, __nv_bfloat16* __restrict__ out16, float* __restrict__ out32,
             long long n4, const float* __restrict__ clip, float lr, float b1, float b2, float eps,
             float wd, float bc1, float bc2, const float* __restrict__ lr_dev, const int* __restrict__ step_dev) {
  const float c = clip ? *clip : 1.f;
  if (!(c >= 0.f)) return;                               // negative or NaN coefficient: the optimizer skips this step
  if (lr_dev != nullptr) lr = *lr_dev;                   // device-resident hyper-parameters: a captured graph
  if (step_dev != nullptr) {                             // replays with the current learning rate and step
    const float st = (float)(*step_dev);
    bc1 = 1.f - powf(b1, st);
    bc2 = 1.f - powf(b2, st);
  }
  const float decay = 1.f - lr * wd, ib1 = 1.f / bc1, ib2 = 1.f / bc2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 gi = Vec4<GT>::load(g + i * 4);
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
    if (out16) {
      uint2 o;
      o.x = pack_bf16(wv.x, wv.y); o.y = pack_bf16(wv.z, wv.w);
      *reinterpret_cast<uint2*>(out16 + i * 4) = o;
    }
    if (out32) *reinterpret_cast<float4*>(out32 + i * 4) = wv;
  }
}

template <typename GT>
__global__ void __launch_bounds__(256)
sumsq_kernel(const GT* __restrict__ g, long long n4, float* __restrict__ total) {
  __shared__ float red[33];
  float s = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 x = Vec4<GT>::load(g + i * 4);
    s += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) atomicAdd(total, s);
}

// sum of squares over a list of [lo, hi) element ranges of one fp32 buffer (lo, hi multiples of 4), one launch:
// grid (x, number of ranges); blocks beyond the end of a short range leave at once
__global__ void __launch_bounds__(256)
sumsq_ranges_kernel(const float* __restrict__ g, const long long* __restrict__ ranges, float* __restrict__ total) {
  __shared__ float red[33];
  const long long lo = ranges[2 * blockIdx.y], n4 = (ranges[2 * blockIdx.y + 1] - lo) / 4;
  if ((long long)blockIdx.x * blockDim.x >= n4) return;
  const float* base = g + lo;
  float s = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 x = *reinterpret_cast<const float4*>(base + i * 4);
    s += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) atomicAdd(total, s);
}

// =====================================================================================
// finalisation of small parameter gradients: column sums of per-CTA partial buffers written straight into the
// fp32 main-gradient buffers (store or accumulate per parameter), so the mixer backward issues one launch
// instead of ~20 reduction / cast / copy kernels
// =====================================================================================
struct SmallGradArgs {
  const float* conv_part; int T1, C;          // [T1][C][5]  (dw0..dw3, db)
  const float* gated_part; int S, d_in;       // [S][d_in]
  const float* hpart; int T2, Hv, H;          // [T2][Hv][3] (dA, dD, d dt_bias)
  const float* A;                             // [H]  (dA_log = dA * A)
  float *g_conv_w, *g_conv_b, *g_norm_w, *g_A_log, *g_D, *g_dt_bias;
  int acc_mask;                               // bit i set: add into parameter i's buffer, else overwrite
};

__device__ __forceinline__ void put(float* dst, float v, bool acc) { *dst = acc ? *dst + v : v; }

// fp32 copies of the per-head mixer parameters in one launch: out[0:H] = -exp(A_log), out[H:2H] = D,
// out[2H:3H] = dt_bias (the three parameters may be bf16 or fp32)
__global__ void mixer_param_prep_kernel(const void* A_log, const void* D, const void* dt_bias, int bf16_mask, int H,
                                        float* __restrict__ out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= 3 * H) return;
  const int which = i / H, h = i % H;
  const void* src = which == 0 ? A_log : which == 1 ? D : dt_bias;
  const float v = (bf16_mask >> which) & 1 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(src)[h])
                                           : reinterpret_cast<const float*>(src)[h];
  out[i] = which == 0 ? -expf(v) : v;
}

// Column sums with the rows split over 8 thread groups: block = 32 columns x 8 row groups, each thread adds
// every 8th row of its column (coalesced 128-byte row reads), the 8 partial sums meet in shared memory.
// A one-thread-per-column loop over all rows is latency-bound on these small matrices.
constexpr int CS_COLS = 32, CS_GROUPS = 8;

__device__ __forceinline__ float colsum_groups(float s, float (*red)[CS_COLS + 1]) {
  const int tx = threadIdx.x & (CS_COLS - 1), tg = threadIdx.x / CS_COLS;
  red[tg][tx] = s;
  __syncthreads();
  float r = 0.f;
  if (tg == 0) {
    #pragma unroll
    for (int k = 0; k < CS_GROUPS; ++k) r += red[k][tx];
  }
  return r;
}

__global__ void __launch_bounds__(256) mixer_small_grads_kernel(const SmallGradArgs a) {
  __shared__ float red[CS_GROUPS][CS_COLS + 1];
  const int tx = threadIdx.x & (CS_COLS - 1), tg = threadIdx.x / CS_COLS;
  const long long n_conv = (long long)a.C * 5, n_gated = a.d_in, n_h = (long long)a.H * 3;
  long long i = (long long)blockIdx.x * CS_COLS + tx;
  int seg = 3;
  float s = 0.f;
  if (i < n_conv) {
    seg = 0;
    for (int t = tg; t < a.T1; t += CS_GROUPS) s += a.conv_part[(long long)t * n_conv + i];
  } else if (i - n_conv < n_gated) {
    seg = 1;
    i -= n_conv;
    for (int t = tg; t < a.S; t += CS_GROUPS) s += a.gated_part[(long long)t * n_gated + i];
  } else if (i - n_conv - n_gated < n_h) {
    seg = 2;
    i -= n_conv + n_gated;
    const int h = (int)(i / 3), which = (int)(i % 3);
    const int psplit = a.Hv / a.H;
    for (int t = tg; t < a.T2; t += CS_GROUPS)
      for (int ps = 0; ps < psplit; ++ps) s += a.hpart[((long long)t * a.Hv + h * psplit + ps) * 3 + which];
  }
  s = colsum_groups(s, red);
  if (tg != 0) return;
  if (seg == 0) {
    const int c = (int)(i / 5), k = (int)(i % 5);
    if (k < 4) put(a.g_conv_w + c * 4 + k, s, a.acc_mask & 1);
    else if (a.g_conv_b) put(a.g_conv_b + c, s, a.acc_mask & 2);
  } else if (seg == 1) {
    put(a.g_norm_w + i, s, a.acc_mask & 4);
  } else if (seg == 2) {
    const int h = (int)(i / 3), which = (int)(i % 3);
    if (which == 0) put(a.g_A_log + h, s * a.A[h], a.acc_mask & 8);
    else if (which == 1) put(a.g_D + h, s, a.acc_mask & 16);
    else put(a.g_dt_bias + h, s, a.acc_mask & 32);
  }
}

// dst[c] (+)= sum_s part[s][c]
__global__ void __launch_bounds__(256) colsum_kernel(const float* __restrict__ part, int S, int n, float* dst, int acc) {
  __shared__ float red[CS_GROUPS][CS_COLS + 1];
  const int tx = threadIdx.x & (CS_COLS - 1), tg = threadIdx.x / CS_COLS;
  const int c = blockIdx.x * CS_COLS + tx;
  float s = 0.f;
  if (c < n)
    for (int t = tg; t < S; t += CS_GROUPS) s += part[(long long)t * n + c];
  s = colsum_groups(s, red);
  if (tg == 0 && c < n) dst[c] = acc ? dst[c] + s : s;
}

}  // namespace ssm

// ------------------------------------------------------------------------------------ C API
using namespace ssm;
#define LAUNCH_MV(kern, T, grid, t, st, ...)                                     \
  do {                                                                          \
    if (mv == 1) kern<T, 1><<<grid, t, 0, st>>>(__VA_ARGS__);                   \
    else kern<T, 4><<<grid, t, 0, st>>>(__VA_ARGS__);                           \
  } while (0)
#define BF(p) reinterpret_cast<const __nv_bfloat16*>(p)
#define BFM(p) reinterpret_cast<__nv_bfloat16*>(p)

// Token-tile length: 32 at full size; shorter tiles when that grid would leave most warp slots empty (the
// per-rank channel counts of tensor parallelism), at the price of re-reading the 3-token halo more often.
static int conv_tok_for(int B, int L, int C, int ch_per_thread, int min_tok) {
  const long long warps = (long long)((C / ch_per_thread + 31) / 32) * ((L + 31) / 32) * B;
  int tok = warps >= 2048 ? 32 : warps >= 1024 ? 16 : 8;
  return tok < min_tok ? min_tok : tok;
}

extern "C" int ssm_conv1d_silu_fwd(const void* x, long long xs, const void* w, const void* bias, const void* init,
                                   void* out, long long os, int B, int L, int C, cudaStream_t st) {
  if (C % 8 || xs % 8 || os % 8) return -SSM_ERR_BAD_ARG;
  const int tok = conv_tok_for(B, L, C, 8, 8);
  dim3 grid((C / 8 + 127) / 128, (L + tok - 1) / tok, B);
  if (tok == 32) conv1d_silu_fwd_kernel<32><<<grid, 128, 0, st>>>(BF(x), xs, BF(w), BF(bias), BF(init), BFM(out), os, L, C);
  else if (tok == 16) conv1d_silu_fwd_kernel<16><<<grid, 128, 0, st>>>(BF(x), xs, BF(w), BF(bias), BF(init), BFM(out), os, L, C);
  else conv1d_silu_fwd_kernel<8><<<grid, 128, 0, st>>>(BF(x), xs, BF(w), BF(bias), BF(init), BFM(out), os, L, C);
  return (int)cudaGetLastError();
}

// tokens per partial-sum tile of the backward kernel for this problem size
extern "C" int ssm_conv_bwd_tok_tile(int B, int L, int C) { return conv_tok_for(B, L, C, CONV_CPT, 16); }

// part must hold B * ceil(L / tile) * C * 5 floats, tile = ssm_conv_bwd_tok_tile(B, L, C).
extern "C" int ssm_conv1d_silu_bwd(const void* x, long long xs, const void* w, const void* bias, const void* dy16,
                                   long long ds16, const void* dy32, long long ds32, int c_split, void* dx,
                                   long long dxs, void* part, int B, int L, int C, cudaStream_t st) {
  if (C % 8 || xs % 8 || dxs % 8 || c_split % 8 || ds16 % 4 || ds32 % 4) return -SSM_ERR_BAD_ARG;
  const int tok = conv_tok_for(B, L, C, CONV_CPT, 16);
  dim3 grid((C / CONV_CPT + 127) / 128, (L + tok - 1) / tok, B);
  if (tok == 32)
    conv1d_silu_bwd_kernel<32><<<grid, 128, 0, st>>>(BF(x), xs, BF(w), BF(bias), BF(dy16), ds16,
                                                     reinterpret_cast<const float*>(dy32), ds32, c_split, BFM(dx), dxs,
                                                     reinterpret_cast<float*>(part), L, C);
  else
    conv1d_silu_bwd_kernel<16><<<grid, 128, 0, st>>>(BF(x), xs, BF(w), BF(bias), BF(dy16), ds16,
                                                     reinterpret_cast<const float*>(dy32), ds32, c_split, BFM(dx), dxs,
                                                     reinterpret_cast<float*>(part), L, C);
  return (int)cudaGetLastError();
}

// threads per block and vectors per thread for a row (or group) of n elements; -1 if unsupported
static int norm_threads(int n, int* maxv = nullptr) {
  const int v = n / 8;
  int mv, t = 32;
  if (v <= 1024) { mv = 1; while (t < v) t <<= 1; }
  else if (v <= 4096) { mv = 4; t = 256; while (t * 4 < v) t <<= 1; if (t > 256) return -1; }
  else return -1;
  if (maxv) *maxv = mv;
  return t;
}

extern "C" int ssm_gated_rmsnorm_fwd(const void* y, long long ys, const void* z, long long zs, const void* w,
                                     void* out, long long os, long long rows, int d, int gs, float eps, cudaStream_t st) {
  int mv = 1;
  const int t = norm_threads(gs, &mv);
  if (gs % 8 || d % gs || t < 0 || ys % 8 || zs % 8 || os % 8) return -SSM_ERR_BAD_ARG;
  dim3 grid((unsigned)rows, d / gs);
  if (mv == 1) gated_rmsnorm_fwd_kernel<1><<<grid, t, 0, st>>>(BF(y), ys, BF(z), zs, BF(w), BFM(out), os, gs, eps);
  else gated_rmsnorm_fwd_kernel<4><<<grid, t, 0, st>>>(BF(y), ys, BF(z), zs, BF(w), BFM(out), os, gs, eps);
  return (int)cudaGetLastError();
}
// dwpart must hold row_slices * d floats.
extern "C" int ssm_gated_rmsnorm_bwd(const void* y, long long ys, const void* z, long long zs, const void* w,
                                     const void* dout, long long dos, void* dy, long long dys, void* dz, long long dzs,
                                     void* dwpart, int row_slices, long long rows, int d, int gs, float eps,
                                     cudaStream_t st) {
  int mv = 1;
  const int t = norm_threads(gs, &mv);
  if (gs % 8 || d % gs || t < 0 || ys % 8 || zs % 8 || dos % 8 || dys % 8 || dzs % 8) return -SSM_ERR_BAD_ARG;
  dim3 grid(row_slices, d / gs);
  if (mv == 1)
    gated_rmsnorm_bwd_kernel<1><<<grid, t, 0, st>>>(BF(y), ys, BF(z), zs, BF(w), BF(dout), dos, BFM(dy), dys, BFM(dz), dzs,
                                                    reinterpret_cast<float*>(dwpart), rows, d, gs, eps);
  else
    gated_rmsnorm_bwd_kernel<4><<<grid, t, 0, st>>>(BF(y), ys, BF(z), zs, BF(w), BF(dout), dos, BFM(dy), dys, BFM(dz), dzs,
                                                    reinterpret_cast<float*>(dwpart), rows, d, gs, eps);
  return (int)cudaGetLastError();
}

extern "C" int ssm_add_rmsnorm_fwd(const void* x, const void* res, const void* w, void* out, void* res_out,
                                   long long rows, int D, float eps, int res_fp32, cudaStream_t st) {
  int mv = 1;
  const int t = norm_threads(D, &mv);
  if (D % 8 || t < 0) return -SSM_ERR_BAD_ARG;
  if (res_fp32)
    LAUNCH_MV(add_rmsnorm_fwd_kernel, float, (unsigned)rows, t, st, BF(x), reinterpret_cast<const float*>(res), BF(w), BFM(out),
                                                                reinterpret_cast<float*>(res_out), D, eps);
  else
    LAUNCH_MV(add_rmsnorm_fwd_kernel, __nv_bfloat16, (unsigned)rows, t, st, BF(x), BF(res), BF(w), BFM(out), BFM(res_out), D, eps);
  return (int)cudaGetLastError();
}
extern "C" int ssm_add_rmsnorm_bwd(const void* res, const void* w, const void* dout, const void* dres_out, void* dsum,
                                   void* dwpart, int row_slices, long long rows, int D, float eps, int res_fp32,
                                   cudaStream_t st) {
  int mv = 1;
  const int t = norm_threads(D, &mv);
  if (D % 8 || t < 0) return -SSM_ERR_BAD_ARG;
  if (res_fp32)
    LAUNCH_MV(add_rmsnorm_bwd_kernel, float, row_slices, t, st, reinterpret_cast<const float*>(res), BF(w), BF(dout),
                                                            reinterpret_cast<const float*>(dres_out),
                                                            reinterpret_cast<float*>(dsum),
                                                            reinterpret_cast<float*>(dwpart), rows, D, eps);
  else
    LAUNCH_MV(add_rmsnorm_bwd_kernel, __nv_bfloat16, row_slices, t, st, BF(res), BF(w), BF(dout), BF(dres_out), BFM(dsum),
                                                                    reinterpret_cast<float*>(dwpart), rows, D, eps);
  return (int)cudaGetLastError();
}

// -------------------------------------------------------------------------------------
// gated linear unit of the MLP: h = [gate | up] (row stride ld, halves of S columns), out = act(gate) * up.
// act: 0 GELU (erf), 1 SiLU.  Backward writes d(gate) | d(up) into dh with the same layout.
// (the reference's gated variant is mamba2hybrid/mamba2hybrid_mlp.py:118-134 in ATen ops)
// -------------------------------------------------------------------------------------
namespace ssm {
__device__ __forceinline__ float glu_act(float x, int act) {
  return act == 0 ? 0.5f * x * (1.f + erff(x * 0.70710678118654752f)) : x / (1.f + __expf(-x));
}
__device__ __forceinline__ float glu_act_grad(float x, int act) {
  if (act == 0) return 0.5f * (1.f + erff(x * 0.70710678118654752f)) + x * 0.3989422804014327f * __expf(-0.5f * x * x);
  const float sg = 1.f / (1.f + __expf(-x));
  return sg * (1.f + x * (1.f - sg));
}
__global__ void __launch_bounds__(256)
glu_fwd_kernel(const __nv_bfloat16* __restrict__ h, long long ld, __nv_bfloat16* __restrict__ out, long long rows, int S, int act) {
  const int vec = S / 8;
  const long long total = rows * vec;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec;
    const int c = (int)(i - r * vec) * 8;
    float g[8], u[8];
    load8(h + r * ld + c, g);
    load8(h + r * ld + S + c, u);
    #pragma unroll
    for (int e = 0; e < 8; ++e) g[e] = glu_act(g[e], act) * u[e];
    store8(out + r * S + c, g);
  }
}
__global__ void __launch_bounds__(256)
glu_bwd_kernel(const __nv_bfloat16* __restrict__ h, long long ld, const __nv_bfloat16* __restrict__ dout,
               __nv_bfloat16* __restrict__ dh, long long rows, int S, int act) {
  const int vec = S / 8;
  const long long total = rows * vec;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec;
    const int c = (int)(i - r * vec) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    load8(h + r * ld + c, g);
    load8(h + r * ld + S + c, u);
    load8(dout + r * S + c, d);
    #pragma unroll
    for (int e = 0; e < 8; ++e) {
      dg[e] = d[e] * u[e] * glu_act_grad(g[e], act);
      du[e] = d[e] * glu_act(g[e], act);
    }
    store8(dh + r * 2 * S + c, dg);
    store8(dh + r * 2 * S + S + c, du);
  }
}
}  // namespace ssm
extern "C" int ssm_glu_fwd(const void* h, long long ld, void* out, long long rows, int S, int act, cudaStream_t st) {
  if (S % 8 || ld % 8 || rows < 1 || act < 0 || act > 1) return -SSM_ERR_BAD_ARG;
  const long long total = rows * (S / 8);
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  glu_fwd_kernel<<<blocks, 256, 0, st>>>(BF(h), ld, BFM(out), rows, S, act);
  return (int)cudaGetLastError();
}
extern "C" int ssm_glu_bwd(const void* h, long long ld, const void* dout, void* dh, long long rows, int S, int act,
                           cudaStream_t st) {
  if (S % 8 || ld % 8 || rows < 1 || act < 0 || act > 1) return -SSM_ERR_BAD_ARG;
  const long long total = rows * (S / 8);
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  glu_bwd_kernel<<<blocks, 256, 0, st>>>(BF(h), ld, BF(dout), BFM(dh), rows, S, act);
  return (int)cudaGetLastError();
}

extern "C" int ssm_gelu_fwd(const void* x, void* y, long long n, cudaStream_t st) {
  if (n % 8) return -SSM_ERR_BAD_ARG;
  const long long n8 = n / 8;
  const int blocks = (int)((n8 + 255) / 256 < 148 * 16 ? (n8 + 255) / 256 : 148 * 16);
  gelu_fwd_kernel<<<blocks, 256, 0, st>>>(BF(x), BFM(y), n8);
  return (int)cudaGetLastError();
}
extern "C" int ssm_gelu_bwd(const void* x, const void* dy, void* dx, long long n, cudaStream_t st) {
  if (n % 8) return -SSM_ERR_BAD_ARG;
  const long long n8 = n / 8;
  const int blocks = (int)((n8 + 255) / 256 < 148 * 16 ? (n8 + 255) / 256 : 148 * 16);
  gelu_bwd_kernel<<<blocks, 256, 0, st>>>(BF(x), BF(dy), BFM(dx), n8);
  return (int)cudaGetLastError();
}

extern "C" int ssm_ce_partials(const void* logits, long long ld, int is_fp32, const void* labels, long long rows, int V,
                               int vocab_start, void* omax, void* osum, void* otgt, cudaStream_t st) {
  auto lb = reinterpret_cast<const long long*>(labels);
  auto a = reinterpret_cast<float*>(omax); auto b = reinterpret_cast<float*>(osum); auto c = reinterpret_cast<float*>(otgt);
  if (is_fp32) ce_partials_kernel<float><<<(unsigned)rows, 256, 0, st>>>(reinterpret_cast<const float*>(logits), ld, lb, V, vocab_start, a, b, c);
  else ce_partials_kernel<__nv_bfloat16><<<(unsigned)rows, 256, 0, st>>>(BF(logits), ld, lb, V, vocab_start, a, b, c);
  return (int)cudaGetLastError();
}
SSM_DEBUG_BOUNDS_GETTER(ssm_debug_bounds_elementwise)

extern "C" int ssm_rope(const void* x, long long x_ld, void* out, long long out_ld, const void* cos_tab, const void* sin_tab,
                        long long tokens, int L, int H, int Dh, int rd, int inverse, cudaStream_t st) {
  if (tokens < 1 || L < 1 || H < 1 || rd < 16 || rd > Dh || rd % 16 || Dh % 8 || x_ld % 8 || out_ld % 8 ||
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(cos_tab) |
        reinterpret_cast<uintptr_t>(sin_tab)) & 15))
    return -SSM_ERR_BAD_ARG;
  const long long total = tokens * H * (rd / 16 + (Dh - rd) / 8);
  const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  rope_kernel<<<blocks, 256, 0, st>>>(BF(x), x_ld, BFM(out), out_ld, reinterpret_cast<const float*>(cos_tab),
                                      reinterpret_cast<const float*>(sin_tab), tokens, L, H, Dh, rd, inverse ? -1.f : 1.f);
  return (int)cudaGetLastError();
}

extern "C" int ssm_ce_merge_tiles(const void* tmax, const void* tsum, int tiles, long long rows, void* omax, void* osum,
                                  cudaStream_t st) {
  if (tiles < 1 || rows < 1) return -SSM_ERR_BAD_ARG;
  ce_merge_tiles_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, st>>>(
      reinterpret_cast<const float*>(tmax), reinterpret_cast<const float*>(tsum), tiles, rows,
      reinterpret_cast<float*>(omax), reinterpret_cast<float*>(osum));
  return (int)cudaGetLastError();
}
extern "C" int ssm_ce_backward(const void* logits, long long ld, int is_fp32, const void* labels, long long rows, int V,
                               int vocab_start, long long ignore_index, const void* gmax, const void* gsum,
                               const void* grow, void* grad, long long gld, cudaStream_t st) {
  auto lb = reinterpret_cast<const long long*>(labels);
  auto a = reinterpret_cast<const float*>(gmax); auto b = reinterpret_cast<const float*>(gsum);
  auto c = reinterpret_cast<const float*>(grow);
  if (is_fp32) ce_backward_kernel<float><<<(unsigned)rows, 256, 0, st>>>(reinterpret_cast<const float*>(logits), ld, lb, V, vocab_start, ignore_index, a, b, c, reinterpret_cast<float*>(grad), gld);
  else ce_backward_kernel<__nv_bfloat16><<<(unsigned)rows, 256, 0, st>>>(BF(logits), ld, lb, V, vocab_start, ignore_index, a, b, c, BFM(grad), gld);
  return (int)cudaGetLastError();
}

extern "C" int ssm_adamw(void* master, void* m, void* v, const void* g, int g_fp32, void* out16, void* out32,
                         long long n, const void* clip, float lr, float b1, float b2, float eps, float wd, int step,
                         const void* lr_dev, const void* step_dev, cudaStream_t st) {
  auto lrd = reinterpret_cast<const float*>(lr_dev);
  auto std_ = reinterpret_cast<const int*>(step_dev);
  const float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  if (n % 4 || (reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
                reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(out32)) & 15 ||
      (reinterpret_cast<uintptr_t>(out16) & 7))
    return -SSM_ERR_BAD_ARG;
  n /= 4;
  const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
  auto M = reinterpret_cast<float*>(master); auto mm = reinterpret_cast<float*>(m); auto vv = reinterpret_cast<float*>(v);
  auto cl = reinterpret_cast<const float*>(clip);
  if (g_fp32) adamw_kernel<float><<<blocks, 256, 0, st>>>(M, mm, vv, reinterpret_cast<const float*>(g), BFM(out16), reinterpret_cast<float*>(out32), n, cl, lr, b1, b2, eps, wd, bc1, bc2, lrd, std_);
  else adamw_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(M, mm, vv, BF(g), BFM(out16), reinterpret_cast<float*>(out32), n, cl, lr, b1, b2, eps, wd, bc1, bc2, lrd, std_);
  return (int)cudaGetLastError();
}
extern "C" int ssm_sumsq(const void* g, int g_fp32, long long n, void* total, cudaStream_t st) {
  if (n % 4 || (reinterpret_cast<uintptr_t>(g) & 15)) return -SSM_ERR_BAD_ARG;
  n /= 4;
  const int blocks = (int)((n + 255) / 256 < 148 * 4 ? (n + 255) / 256 : 148 * 4);
  if (g_fp32) sumsq_kernel<float><<<blocks, 256, 0, st>>>(reinterpret_cast<const float*>(g), n, reinterpret_cast<float*>(total));
  else sumsq_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(BF(g), n, reinterpret_cast<float*>(total));
  return (int)cudaGetLastError();
}

// =====================================================================================
// allocation-free variant of add_rmsnorm_bwd (declared in ssm_noalloc.h)
// =====================================================================================
#include "ssm_noalloc.h"
#include <mutex>

// Partial weight-gradient sums, [SSM_NOALLOC_SLICES][D] packed with the call's D.  In host code this name is
// only a handle for the runtime's symbol table, never an address to pass to a kernel.
static __device__ __align__(256) float g_noalloc_scratch[SSM_NOALLOC_SLICES * SSM_NOALLOC_MAX_D];

namespace ssm {
// dw[c] = sum_s part[s][c]; device code may name the array directly.
__global__ void __launch_bounds__(256) noalloc_colsum_kernel(float* __restrict__ dw, int slices, int D) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= D) return;
  float s = 0.f;
  for (int r = 0; r < slices; ++r) s += g_noalloc_scratch[(long long)r * D + c];
  dw[c] = s;
}
}  // namespace ssm

static float* noalloc_scratch_for_current_device(int* err) {
  constexpr int kMaxDevices = 64;
  static float* ptrs[kMaxDevices] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) { *err = e != cudaSuccess ? (int)e : -SSM_NOALLOC_ERR_BAD_ARG; return nullptr; }
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);   // device address of the array on the current device
    if (e != cudaSuccess) { *err = (int)e; return nullptr; }
    ptrs[dev] = static_cast<float*>(p);
  }
  *err = 0;
  return ptrs[dev];
}

extern "C" int ssm_add_rmsnorm_bwd_noalloc(const void* res, const void* w, const void* dout, const void* dres_out,
                                           void* dsum, void* dw, long long rows, int D, float eps, int res_fp32,
                                           cudaStream_t st) {
  if (D > SSM_NOALLOC_MAX_D) return -SSM_NOALLOC_ERR_TOO_LARGE;
  int mv = 1;
  const int t = norm_threads(D, &mv);
  if (D <= 0 || D % 8 || t < 0 || rows < 1 || !res || !w || !dout || !dsum || !dw) return -SSM_NOALLOC_ERR_BAD_ARG;
  // the kernels move rows with 16-byte vector loads and stores: a misaligned base would fault on the device
  const uintptr_t vec16 = reinterpret_cast<uintptr_t>(res) | reinterpret_cast<uintptr_t>(w) |
                          reinterpret_cast<uintptr_t>(dout) | reinterpret_cast<uintptr_t>(dres_out) |
                          reinterpret_cast<uintptr_t>(dsum);
  if ((vec16 & 15) || (reinterpret_cast<uintptr_t>(dw) & 3)) return -SSM_NOALLOC_ERR_BAD_ARG;
  int err = 0;
  float* scratch = noalloc_scratch_for_current_device(&err);
  if (scratch == nullptr) return err;
  const int slices = rows < SSM_NOALLOC_SLICES ? (int)rows : SSM_NOALLOC_SLICES;
  if (res_fp32)
    LAUNCH_MV(add_rmsnorm_bwd_kernel, float, slices, t, st, reinterpret_cast<const float*>(res), BF(w), BF(dout),
                                                        reinterpret_cast<const float*>(dres_out),
                                                        reinterpret_cast<float*>(dsum), scratch, rows, D, eps);
  else
    LAUNCH_MV(add_rmsnorm_bwd_kernel, __nv_bfloat16, slices, t, st, BF(res), BF(w), BF(dout), BF(dres_out), BFM(dsum),
                                                                scratch, rows, D, eps);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  noalloc_colsum_kernel<<<(D + 255) / 256, 256, 0, st>>>(reinterpret_cast<float*>(dw), slices, D);
  return (int)cudaGetLastError();
}

extern "C" int ssm_mixer_small_grads(const void* conv_part, int T1, int C, const void* gated_part, int S, int d_in,
                                     const void* hpart, int T2, int Hv, int H, const void* A, void* g_conv_w,
                                     void* g_conv_b, void* g_norm_w, void* g_A_log, void* g_D, void* g_dt_bias,
                                     int acc_mask, cudaStream_t st) {
  SmallGradArgs a;
  a.conv_part = reinterpret_cast<const float*>(conv_part); a.T1 = T1; a.C = C;
  a.gated_part = reinterpret_cast<const float*>(gated_part); a.S = S; a.d_in = d_in;
  a.hpart = reinterpret_cast<const float*>(hpart); a.T2 = T2; a.Hv = Hv; a.H = H;
  a.A = reinterpret_cast<const float*>(A);
  a.g_conv_w = reinterpret_cast<float*>(g_conv_w); a.g_conv_b = reinterpret_cast<float*>(g_conv_b);
  a.g_norm_w = reinterpret_cast<float*>(g_norm_w); a.g_A_log = reinterpret_cast<float*>(g_A_log);
  a.g_D = reinterpret_cast<float*>(g_D); a.g_dt_bias = reinterpret_cast<float*>(g_dt_bias);
  a.acc_mask = acc_mask;
  const long long n = (long long)C * 5 + d_in + (long long)H * 3;
  mixer_small_grads_kernel<<<(unsigned)((n + CS_COLS - 1) / CS_COLS), 256, 0, st>>>(a);
  return (int)cudaGetLastError();
}
extern "C" int ssm_sumsq_ranges(const void* g, const void* ranges, int nranges, void* total, cudaStream_t st) {
  if (nranges < 1 || (reinterpret_cast<uintptr_t>(g) & 15)) return nranges == 0 ? 0 : -SSM_ERR_BAD_ARG;
  dim3 grid(148 * 2, nranges);
  sumsq_ranges_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const float*>(g), reinterpret_cast<const long long*>(ranges),
                                            reinterpret_cast<float*>(total));
  return (int)cudaGetLastError();
}
extern "C" int ssm_mixer_param_prep(const void* A_log, const void* D, const void* dt_bias, int bf16_mask, int H,
                                    void* out, cudaStream_t st) {
  mixer_param_prep_kernel<<<(3 * H + 127) / 128, 128, 0, st>>>(A_log, D, dt_bias, bf16_mask, H,
                                                              reinterpret_cast<float*>(out));
  return (int)cudaGetLastError();
}
extern "C" int ssm_colsum(const void* part, int S, int n, void* dst, int acc, cudaStream_t st) {
  colsum_kernel<<<(n + CS_COLS - 1) / CS_COLS, 256, 0, st>>>(reinterpret_cast<const float*>(part), S, n,
                                                 reinterpret_cast<float*>(dst), acc);
  return (int)cudaGetLastError();
}
