// Single-token decode over cached states for sm_100a (memory-bound: one pass over the SSM state).
//   conv step : roll the [C][4] window, depthwise conv + bias + SiLU for x, B and C alike
//   ssm step  : S <- S exp(A dt) + (dt x) (x) B ;  y = S C + D x ;  dt = softplus(dt_raw + bias) fused
// State layouts as in the cache: conv_state [B, C, 4] (oldest first), ssm_state [B, H, P, N] fp32, both
// updated in place.  Reference: mamba2/mamba2_kernel_inference.py:13-23,26-104 (grid over batch only, softplus
// and gated norm outside); here the grid is (head, batch) and the state makes exactly one round trip.
#include "common.cuh"

namespace ssm {

__global__ void __launch_bounds__(256)
decode_conv_step_kernel(const __nv_bfloat16* __restrict__ xnew, long long xs, __nv_bfloat16* __restrict__ state,
                        const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ bias,
                        float* __restrict__ act, int C) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  if (c >= C) return;
  if (!SSM_INDEX_OK(c, xs)) return;               // the new token's row must hold all C channels
  uint2* sp = reinterpret_cast<uint2*>(state + ((long long)b * C + c) * 4);
  const uint2 s = *sp;
  const float x1 = bf16_hi(s.x), x2 = bf16_lo(s.y), x3 = bf16_hi(s.y);
  const __nv_bfloat16 xn = xnew[(long long)b * xs + c];
  const float x4 = __bfloat162float(xn);
  uint2 ns;
  ns.x = pack_bf16(x1, x2);
  ns.y = pack_bf16(x3, x4);
  *sp = ns;
  const uint2 wv = *reinterpret_cast<const uint2*>(w + (long long)c * 4);
  float pre = bias ? __bfloat162float(bias[c]) : 0.f;
  pre += bf16_lo(wv.x) * x1 + bf16_hi(wv.x) * x2 + bf16_lo(wv.y) * x3 + bf16_hi(wv.y) * x4;
  act[(long long)b * C + c] = silu_f(pre);
}

// grid (H, B), 128 threads: warp w owns rows p = 4w .. 4w+3, 4w+16 .., ...; lanes own n = 4*lane + 128*r.
__global__ void __launch_bounds__(128)
decode_ssm_step_kernel(const float* __restrict__ act, const __nv_bfloat16* __restrict__ dt_raw, long long dts,
                       const float* __restrict__ dt_bias, const float* __restrict__ A, const float* __restrict__ D,
                       float* __restrict__ state, __nv_bfloat16* __restrict__ y, int C, int H, int P, int N, int G,
                       int d_in) {
  const int h = blockIdx.x, b = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = h / (H / G);
  const float dt = softplus_f(__bfloat162float(dt_raw[(long long)b * dts + h]) + dt_bias[h]);
  const float decay = __expf(A[h] * dt);
  const float Dh = D[h];
  const float* ab = act + (long long)b * C;
  const float* Bv = ab + d_in + g * N;
  const float* Cv = ab + d_in + G * N + g * N;
  // the activation row [x | B | C] must hold d_in + 2 G N values and the head's x slice must lie inside d_in
  if (!SSM_INDEX_OK(d_in + 2 * G * N - 1, C) || !SSM_INDEX_OK(h * P + P - 1, d_in)) return;
  float* S = state + (((long long)b * H + h) * P) * N;
  // four rows per warp iteration: four independent 16-byte loads per lane are in flight before any arithmetic,
  // and the four row sums are reduced together (the state makes one round trip; this loop is latency-bound otherwise)
  for (int p0 = warp * 4; p0 < P; p0 += 16) {
    float4 s[4];
    float xs[4], acc[4];
    #pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int pp = p0 + r;
      xs[r] = pp < P ? ab[h * P + pp] : 0.f;
      acc[r] = 0.f;
    }
    for (int n = lane * 4; n < N; n += 128) {
      #pragma unroll
      for (int r = 0; r < 4; ++r)
        if (p0 + r < P) s[r] = *reinterpret_cast<const float4*>(S + (long long)(p0 + r) * N + n);
      const float4 bv = *reinterpret_cast<const float4*>(Bv + n);
      const float4 cv = *reinterpret_cast<const float4*>(Cv + n);
      #pragma unroll
      for (int r = 0; r < 4; ++r) {
        if (p0 + r < P) {
          const float dx = dt * xs[r];
          s[r].x = s[r].x * decay + dx * bv.x; s[r].y = s[r].y * decay + dx * bv.y;
          s[r].z = s[r].z * decay + dx * bv.z; s[r].w = s[r].w * decay + dx * bv.w;
          *reinterpret_cast<float4*>(S + (long long)(p0 + r) * N + n) = s[r];
          acc[r] += s[r].x * cv.x + s[r].y * cv.y + s[r].z * cv.z + s[r].w * cv.w;
        }
      }
    }
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      #pragma unroll
      for (int r = 0; r < 4; ++r) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], o);
    }
    if (lane < 4 && p0 + lane < P) {
      const float a = lane == 0 ? acc[0] : lane == 1 ? acc[1] : lane == 2 ? acc[2] : acc[3];
      const float x = lane == 0 ? xs[0] : lane == 1 ? xs[1] : lane == 2 ? xs[2] : xs[3];
      y[(long long)b * d_in + h * P + p0 + lane] = __float2bfloat16(a + Dh * x);
    }
  }
}

}  // namespace ssm

using namespace ssm;
SSM_DEBUG_BOUNDS_GETTER(ssm_debug_bounds_decode)

extern "C" int ssm_decode_conv_step(const void* xnew, long long xs, void* state, const void* w, const void* bias,
                                    void* act, int B, int C, cudaStream_t st) {
  dim3 grid((C + 255) / 256, B);
  decode_conv_step_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(xnew), xs,
                                                reinterpret_cast<__nv_bfloat16*>(state),
                                                reinterpret_cast<const __nv_bfloat16*>(w),
                                                reinterpret_cast<const __nv_bfloat16*>(bias),
                                                reinterpret_cast<float*>(act), C);
  return (int)cudaGetLastError();
}

extern "C" int ssm_decode_ssm_step(const void* act, const void* dt_raw, long long dts, const void* dt_bias,
                                   const void* A, const void* D, void* state, void* y, int B, int C, int H, int P,
                                   int N, int G, int d_in, cudaStream_t st) {
  if (N % 4 || H % G) return -SSM_ERR_BAD_ARG;
  dim3 grid(H, B);
  decode_ssm_step_kernel<<<grid, 128, 0, st>>>(reinterpret_cast<const float*>(act),
                                               reinterpret_cast<const __nv_bfloat16*>(dt_raw), dts,
                                               reinterpret_cast<const float*>(dt_bias),
                                               reinterpret_cast<const float*>(A), reinterpret_cast<const float*>(D),
                                               reinterpret_cast<float*>(state), reinterpret_cast<__nv_bfloat16*>(y), C, H,
                                               P, N, G, d_in);
  return (int)cudaGetLastError();
}
