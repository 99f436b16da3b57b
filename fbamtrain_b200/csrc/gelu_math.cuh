// Exact-erf GELU and its derivative on pairs of fp32 values (sm_100 executes add / mul / fma on two packed fp32
// values per instruction), shared by the GEMM epilogues and the bandwidth kernels.
//
// erf by Abramowitz-Stegun 7.1.26 (|error| < 1.5e-7, far below bf16 resolution):
//   erf(|v|) = 1 - t (a1 + t (a2 + t (a3 + t (a4 + t a5)))) exp(-v^2),  t = 1 / (1 + p v),  v = |x| / sqrt(2).
// The coefficients below carry the minus sign so that the last step is one fused multiply-add; exp(-v^2) is also
// the Gaussian factor of gelu'(x) = Phi(x) + x phi(x).  (reference: exact-erf GELU and its gradient in
// kernel_gen/kernel_gen/kernels/act.py:43-86.)
#pragma once
#include <cuda_runtime.h>

namespace gelu_math {

__device__ __forceinline__ float2 f2(float a) { return make_float2(a, a); }
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// erf(x / sqrt(2)) of both halves; e receives exp(-x^2 / 2)
__device__ __forceinline__ float2 erf_core2(float2 x, float2& e) {
  const float2 u = __fmul2_rn(make_float2(fabsf(x.x), fabsf(x.y)), f2(0.70710678118654752f));
  const float2 den = __ffma2_rn(u, f2(0.3275911f), f2(1.0f));
  const float2 t = make_float2(rcp_approx(den.x), rcp_approx(den.y));
  const float2 w = __fmul2_rn(__fmul2_rn(u, u), f2(-1.4426950408889634f));
  e = make_float2(ex2_approx(w.x), ex2_approx(w.y));
  float2 poly = __ffma2_rn(t, f2(-1.061405429f), f2(1.453152027f));
  poly = __ffma2_rn(poly, t, f2(-1.421413741f));
  poly = __ffma2_rn(poly, t, f2(0.284496736f));
  poly = __ffma2_rn(poly, t, f2(-0.254829592f));
  poly = __fmul2_rn(poly, t);
  const float2 er_abs = __ffma2_rn(poly, e, f2(1.0f));
  return make_float2(copysignf(er_abs.x, x.x), copysignf(er_abs.y, x.y));
}

__device__ __forceinline__ float2 gelu2(float2 x) {
  float2 e;
  const float2 er = erf_core2(x, e);
  const float2 hx = __fmul2_rn(x, f2(0.5f));
  return __ffma2_rn(hx, er, hx);
}

__device__ __forceinline__ float2 gelu_grad2(float2 x) {
  float2 e;
  const float2 er = erf_core2(x, e);
  const float2 cdf = __ffma2_rn(er, f2(0.5f), f2(0.5f));
  return __ffma2_rn(__fmul2_rn(x, f2(0.3989422804014327f)), e, cdf);
}

__device__ __forceinline__ float gelu1(float x) { return gelu2(make_float2(x, 0.0f)).x; }
__device__ __forceinline__ float gelu_grad1(float x) { return gelu_grad2(make_float2(x, 0.0f)).x; }

}  // namespace gelu_math
