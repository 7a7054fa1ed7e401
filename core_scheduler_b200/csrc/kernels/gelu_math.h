// SPDX-License-Identifier: Apache-2.0
// GELU in its exact (erf) form, shared by the GEMM epilogues and the stand-alone GELU kernels.
#pragma once

namespace cs::kernels {
namespace {
// erf uses the rational approximation 7.1.26 of
// Abramowitz & Stegun (absolute error < 1.5e-7, far below bf16 resolution): one reciprocal, one
// exponential and five FMAs. GELU'(x) needs exp(-x^2/2) as well, which is the exponential the
// erf of x/sqrt(2) already computed, so the derivative costs two special-function ops per element
// instead of the ~45 instructions of erff + expf: the dGELU epilogue stays hidden behind a
// K = 768 main loop.
struct ErfParts {
  float erf_abs;  // erf(|x| / sqrt(2))
  float e;        // exp(-x^2 / 2)
};
__device__ __forceinline__ ErfParts erf_parts(float x) {
  const float z = fabsf(x) * 0.70710678118654752440f;
  float t;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.3275911f, z, 1.0f)));
  float poly = fmaf(1.061405429f, t, -1.453152027f);
  poly = fmaf(poly, t, 1.421413741f);
  poly = fmaf(poly, t, -0.284496736f);
  poly = fmaf(poly, t, 0.254829592f);
  poly *= t;
  ErfParts r;
  // exp(-z^2) = 2^(-z^2 * log2 e)
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r.e) : "f"(z * z * -1.4426950408889634f));
  r.erf_abs = fmaf(-poly, r.e, 1.0f);
  return r;
}
__device__ __forceinline__ float gelu_f(float x) {
  const ErfParts p = erf_parts(x);
  return 0.5f * x * (1.0f + copysignf(p.erf_abs, x));
}
__device__ __forceinline__ float gelu_grad_f(float x) {
  const ErfParts p = erf_parts(x);
  const float cdf = 0.5f * (1.0f + copysignf(p.erf_abs, x));
  return fmaf(x * 0.39894228040143267794f, p.e, cdf);
}
}  // namespace
}  // namespace cs::kernels
