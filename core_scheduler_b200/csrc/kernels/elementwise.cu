// SPDX-License-Identifier: Apache-2.0
// Memory-bound sm_100a kernels: AdamW, GELU, residual add, casts/transposes, LayerNorm,
// embedding, cross-entropy helpers and gradient-norm reductions. All are vectorised to 128-bit
// accesses and sized so that a launch covers the 148 SMs with several resident CTAs each.
//
// What they replace in the reference project: src/optimizer/adamw.cu:35-90 (scalar, one
// element per thread, one launch per tensor) and the ATen library calls listed for
// LayerNorm / GeLU / Embedding / CrossEntropy / clip_grad_norm in src/compute/*.cpp.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <mutex>

#include "api.h"
#include "bounds_check.h"
#include "gelu_math.h"

namespace cs::kernels {
namespace {
std::atomic<int64_t> g_launches{0};
}
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
int64_t launch_count() { return g_launches.load(std::memory_order_relaxed); }
int finish_launch(int n) {
  count_launch(n);
  return static_cast<int>(cudaGetLastError());
}
CS_DEFINE_BOUNDS_GETTER(bounds_report_elementwise)
bool bounds_check_enabled() {
#ifdef CS_BOUNDS_CHECK
  return true;
#else
  return false;
#endif
}
int bounds_report(BoundsReport *out, bool reset) {
  *out = BoundsReport{};
  if (!bounds_check_enabled()) return 0;
  int rc = static_cast<int>(cudaDeviceSynchronize());
  if (rc != 0) return rc;
  using Getter = int (*)(BoundsReport *, bool);
  const Getter getters[] = {bounds_report_elementwise, bounds_report_collectives, bounds_report_gemm, bounds_report_attention};
  for (Getter g : getters) {
    BoundsReport r{};
    rc = g(&r, reset);
    if (rc != 0) return rc;
    if (r.code != 0 && out->code == 0) *out = r;
  }
  return 0;
}
namespace {
constexpr int kSmCount = 148;

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

struct alignas(16) Bf16x8 {
  __nv_bfloat162 v[4];
};
__device__ __forceinline__ void unpack(const Bf16x8 &p, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ Bf16x8 pack(const float (&f)[8]) {
  Bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}
__device__ __forceinline__ void load8(const void *base, int64_t elem, int dtype, float (&f)[8]) {
  if (dtype == 1) {
    unpack(*reinterpret_cast<const Bf16x8 *>(static_cast<const __nv_bfloat16 *>(base) + elem), f);
  } else {
    const float4 a = *reinterpret_cast<const float4 *>(static_cast<const float *>(base) + elem);
    const float4 b = *reinterpret_cast<const float4 *>(static_cast<const float *>(base) + elem + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
}

int grid_for(int64_t work_items, int threads, int max_ctas_per_sm = 8) {
  const int64_t blocks = (work_items + threads - 1) / threads;
  const int64_t cap = static_cast<int64_t>(kSmCount) * max_ctas_per_sm;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}
}  // namespace

// ------------------------------------------------------------------------------- AdamW ----
namespace {
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

template <typename P, typename G, int VEC>
__global__ void __launch_bounds__(256) adamw_kernel(P *__restrict__ w, const G *__restrict__ g, P *__restrict__ m,
                                                    P *__restrict__ v, P *__restrict__ vmax,
                                                    __nv_bfloat16 *__restrict__ lp, int64_t n, float lr, float b1,
                                                    float b2, float eps, float wd, float ibc1, float ibc2,
                                                    float gscale, const float *__restrict__ clip) {
  const float scale = clip ? gscale * clip[0] : gscale;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x * VEC;
  for (int64_t base = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * VEC; base < n; base += stride) {
    P wv[VEC], mv[VEC], vv[VEC], xv[VEC];
    G gv[VEC];
    const bool full = base + VEC <= n;
    if (!CS_IN_BOUNDS(kKidAdamW, base, n)) continue;
    if (full) {
      // 128-bit (fp32 x4) or 64-bit (16-bit x4) vector accesses
      using PV = typename std::conditional<sizeof(P) == 4, float4, float2>::type;
      using GV = typename std::conditional<sizeof(G) == 4, float4, float2>::type;
      *reinterpret_cast<PV *>(wv) = *reinterpret_cast<const PV *>(w + base);
      *reinterpret_cast<PV *>(mv) = *reinterpret_cast<const PV *>(m + base);
      *reinterpret_cast<PV *>(vv) = *reinterpret_cast<const PV *>(v + base);
      *reinterpret_cast<GV *>(gv) = *reinterpret_cast<const GV *>(g + base);
      if (vmax) *reinterpret_cast<PV *>(xv) = *reinterpret_cast<const PV *>(vmax + base);
    } else {
      for (int i = 0; i < VEC; ++i) {
        if (base + i < n) {
          wv[i] = w[base + i]; mv[i] = m[base + i]; vv[i] = v[base + i]; gv[i] = g[base + i];
          if (vmax) xv[i] = vmax[base + i];
        }
      }
    }
    __nv_bfloat16 lo[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const float grad = to_f<G>(gv[i]) * scale;
      float wt = to_f<P>(wv[i]);
      wt -= lr * wd * wt;
      const float mt = b1 * to_f<P>(mv[i]) + (1.0f - b1) * grad;
      const float vt = b2 * to_f<P>(vv[i]) + (1.0f - b2) * grad * grad;
      const float mhat = mt * ibc1;
      float vhat = vt * ibc2;
      if (vmax) {
        vhat = fmaxf(to_f<P>(xv[i]), vhat);
        xv[i] = from_f<P>(vhat);
      }
      wt -= lr * mhat / (sqrtf(vhat) + eps);
      wv[i] = from_f<P>(wt);
      mv[i] = from_f<P>(mt);
      vv[i] = from_f<P>(vt);
      lo[i] = __float2bfloat16_rn(to_f<P>(wv[i]));
    }
    if (full) {
      using PV = typename std::conditional<sizeof(P) == 4, float4, float2>::type;
      *reinterpret_cast<PV *>(w + base) = *reinterpret_cast<PV *>(wv);
      *reinterpret_cast<PV *>(m + base) = *reinterpret_cast<PV *>(mv);
      *reinterpret_cast<PV *>(v + base) = *reinterpret_cast<PV *>(vv);
      if (vmax) *reinterpret_cast<PV *>(vmax + base) = *reinterpret_cast<PV *>(xv);
      if (lp) *reinterpret_cast<float2 *>(lp + base) = *reinterpret_cast<float2 *>(lo);
    } else {
      for (int i = 0; i < VEC; ++i) {
        if (base + i < n) {
          w[base + i] = wv[i]; m[base + i] = mv[i]; v[base + i] = vv[i];
          if (vmax) vmax[base + i] = xv[i];
          if (lp) lp[base + i] = lo[i];
        }
      }
    }
  }
}

template <typename P, typename G>
int launch_adamw(cudaStream_t s, const AdamWArgs &a) {
  constexpr int VEC = 4;
  // vector accesses need 16-byte (fp32) / 8-byte (16-bit) alignment of every base pointer
  const uintptr_t mask = (reinterpret_cast<uintptr_t>(a.param) | reinterpret_cast<uintptr_t>(a.grad) |
                          reinterpret_cast<uintptr_t>(a.exp_avg) | reinterpret_cast<uintptr_t>(a.exp_avg_sq) |
                          reinterpret_cast<uintptr_t>(a.max_exp_avg_sq) | reinterpret_cast<uintptr_t>(a.lp));
  const int threads = 256;
  if (mask & 15) {
    adamw_kernel<P, G, 1><<<grid_for(a.n, threads), threads, 0, s>>>(
        static_cast<P *>(a.param), static_cast<const G *>(a.grad), static_cast<P *>(a.exp_avg),
        static_cast<P *>(a.exp_avg_sq), static_cast<P *>(a.max_exp_avg_sq), static_cast<__nv_bfloat16 *>(a.lp), a.n,
        a.lr, a.beta1, a.beta2, a.eps, a.weight_decay, a.inv_bias_correction1, a.inv_bias_correction2, a.grad_scale,
        a.clip_coef);
  } else {
    adamw_kernel<P, G, VEC><<<grid_for((a.n + VEC - 1) / VEC, threads), threads, 0, s>>>(
        static_cast<P *>(a.param), static_cast<const G *>(a.grad), static_cast<P *>(a.exp_avg),
        static_cast<P *>(a.exp_avg_sq), static_cast<P *>(a.max_exp_avg_sq), static_cast<__nv_bfloat16 *>(a.lp), a.n,
        a.lr, a.beta1, a.beta2, a.eps, a.weight_decay, a.inv_bias_correction1, a.inv_bias_correction2, a.grad_scale,
        a.clip_coef);
  }
  return finish_launch();
}
}  // namespace

int adamw_step(stream_t stream, const AdamWArgs &a) {
  auto s = static_cast<cudaStream_t>(stream);
  if (a.n == 0) return 0;
  switch (a.param_dtype * 3 + a.grad_dtype) {
    case 0: return launch_adamw<float, float>(s, a);
    case 1: return launch_adamw<float, __nv_bfloat16>(s, a);
    case 2: return launch_adamw<float, __half>(s, a);
    case 4: return launch_adamw<__nv_bfloat16, __nv_bfloat16>(s, a);
    case 3: return launch_adamw<__nv_bfloat16, float>(s, a);
    case 8: return launch_adamw<__half, __half>(s, a);
    case 6: return launch_adamw<__half, float>(s, a);
    default: return static_cast<int>(cudaErrorInvalidValue);
  }
}

// ------------------------------------------------------------------ GELU / add / casts ----
namespace {
__global__ void __launch_bounds__(256) gelu_fwd_kernel(const Bf16x8 *__restrict__ x, Bf16x8 *__restrict__ y, int64_t n8) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    if (!CS_IN_BOUNDS(kKidElementwise, i, n8)) continue;
    float f[8];
    unpack(x[i], f);
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = gelu_f(f[k]);
    y[i] = pack(f);
  }
}
__global__ void __launch_bounds__(256) gelu_bwd_kernel(const Bf16x8 *__restrict__ dy, const Bf16x8 *__restrict__ x,
                                                       Bf16x8 *__restrict__ dx, int64_t n8) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float f[8], g[8];
    unpack(x[i], f);
    unpack(dy[i], g);
#pragma unroll
    for (int k = 0; k < 8; ++k) g[k] *= gelu_grad_f(f[k]);
    dx[i] = pack(g);
  }
}
__global__ void __launch_bounds__(256) add_kernel(const Bf16x8 *__restrict__ a, const Bf16x8 *__restrict__ b,
                                                  Bf16x8 *__restrict__ o, int64_t n8) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float f[8], g[8];
    unpack(a[i], f);
    unpack(b[i], g);
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] += g[k];
    o[i] = pack(f);
  }
}
__global__ void tail_kernel(const __nv_bfloat16 *a, const __nv_bfloat16 *b, __nv_bfloat16 *o, int64_t begin, int64_t n,
                            int mode) {
  const int64_t i = begin + threadIdx.x;
  if (i >= n) return;
  const float x = __bfloat162float(a[i]);
  if (mode == 0) o[i] = __float2bfloat16_rn(gelu_f(x));
  if (mode == 1) o[i] = __float2bfloat16_rn(x * gelu_grad_f(__bfloat162float(b[i])));  // a = dy, b = x
  if (mode == 2) o[i] = __float2bfloat16_rn(x + __bfloat162float(b[i]));
}
__global__ void __launch_bounds__(256) cast_kernel(const float *__restrict__ src, __nv_bfloat16 *__restrict__ dst, int64_t n) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    dst[i] = __float2bfloat16_rn(src[i]);
}
// 32x32 tile transpose through shared memory; src [rows, cols] (fp32 or bf16) -> dst [cols, rows] bf16
template <typename T>
__global__ void __launch_bounds__(256) transpose_kernel(const T *__restrict__ src, __nv_bfloat16 *__restrict__ dst,
                                                        int64_t rows, int64_t cols) {
  __shared__ float tile[32][33];
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * 32, c0 = static_cast<int64_t>(blockIdx.x) * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int64_t r = r0 + ty + 8 * k, c = c0 + tx;
    if (r < rows && c < cols && CS_IN_BOUNDS(kKidTranspose, r * cols + c, rows * cols)) tile[ty + 8 * k][tx] = to_f<T>(src[r * cols + c]);
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int64_t c = c0 + ty + 8 * k, r = r0 + tx;
    if (r < rows && c < cols && CS_IN_BOUNDS(kKidTranspose, c * rows + r, rows * cols)) dst[c * rows + r] = __float2bfloat16_rn(tile[tx][ty + 8 * k]);
  }
}
}  // namespace

int gelu_forward(stream_t stream, const void *x, void *y, int64_t n) {
  auto s = static_cast<cudaStream_t>(stream);
  const int64_t n8 = n / 8;
  if (n8) gelu_fwd_kernel<<<grid_for(n8, 256), 256, 0, s>>>(static_cast<const Bf16x8 *>(x), static_cast<Bf16x8 *>(y), n8);
  if (n % 8)
    tail_kernel<<<1, 8, 0, s>>>(static_cast<const __nv_bfloat16 *>(x), nullptr, static_cast<__nv_bfloat16 *>(y), n8 * 8, n, 0);
  return finish_launch();
}
int gelu_backward(stream_t stream, const void *dy, const void *x, void *dx, int64_t n) {
  auto s = static_cast<cudaStream_t>(stream);
  const int64_t n8 = n / 8;
  if (n8)
    gelu_bwd_kernel<<<grid_for(n8, 256), 256, 0, s>>>(static_cast<const Bf16x8 *>(dy), static_cast<const Bf16x8 *>(x),
                                                      static_cast<Bf16x8 *>(dx), n8);
  if (n % 8)
    tail_kernel<<<1, 8, 0, s>>>(static_cast<const __nv_bfloat16 *>(dy), static_cast<const __nv_bfloat16 *>(x),
                                static_cast<__nv_bfloat16 *>(dx), n8 * 8, n, 1);
  return finish_launch();
}
int add_bf16(stream_t stream, const void *a, const void *b, void *out, int64_t n) {
  auto s = static_cast<cudaStream_t>(stream);
  const int64_t n8 = n / 8;
  if (n8)
    add_kernel<<<grid_for(n8, 256), 256, 0, s>>>(static_cast<const Bf16x8 *>(a), static_cast<const Bf16x8 *>(b),
                                                 static_cast<Bf16x8 *>(out), n8);
  if (n % 8)
    tail_kernel<<<1, 8, 0, s>>>(static_cast<const __nv_bfloat16 *>(a), static_cast<const __nv_bfloat16 *>(b),
                                static_cast<__nv_bfloat16 *>(out), n8 * 8, n, 2);
  return finish_launch();
}
namespace {
__global__ void __launch_bounds__(256) acc_residual_kernel(const float *__restrict__ acc, const Bf16x8 *__restrict__ res,
                                                           Bf16x8 *__restrict__ out, int64_t n8) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float f[8];
    load8(acc, i * 8, 0, f);
    if (res) {
      float r[8];
      unpack(res[i], r);
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] += r[k];
    }
    out[i] = pack(f);
  }
}
}  // namespace

int add_f32_residual_to_bf16(stream_t stream, const float *acc, const void *residual, void *out, int64_t n) {
  if (n % 8 != 0) return static_cast<int>(cudaErrorInvalidValue);
  if (n == 0) return 0;
  acc_residual_kernel<<<grid_for(n / 8, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      acc, static_cast<const Bf16x8 *>(residual), static_cast<Bf16x8 *>(out), n / 8);
  return finish_launch();
}

int cast_fp32_to_bf16(stream_t stream, const float *src, void *dst, int64_t n) {
  if (n) cast_kernel<<<grid_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(src, static_cast<__nv_bfloat16 *>(dst), n);
  return finish_launch();
}
int transpose_cast_to_bf16(stream_t stream, const void *src, int src_dtype, void *dst_t, int64_t rows, int64_t cols) {
  auto s = static_cast<cudaStream_t>(stream);
  dim3 grid(static_cast<unsigned>((cols + 31) / 32), static_cast<unsigned>((rows + 31) / 32));
  if (src_dtype == 0)
    transpose_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float *>(src), static_cast<__nv_bfloat16 *>(dst_t), rows, cols);
  else if (src_dtype == 1)
    transpose_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16 *>(src),
                                                         static_cast<__nv_bfloat16 *>(dst_t), rows, cols);
  else
    return static_cast<int>(cudaErrorInvalidValue);
  return finish_launch();
}

namespace {
__global__ void __launch_bounds__(256) pack_qkv_kernel(const Bf16x8 *__restrict__ q, const Bf16x8 *__restrict__ k,
                                                       const Bf16x8 *__restrict__ v, Bf16x8 *__restrict__ out, int64_t B,
                                                       int64_t H, int64_t T, int d8, int src_bthd) {
  // one thread per 16-byte piece of the output, output-major so that writes are fully coalesced
  const int64_t total = B * T * 3 * H * d8;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    int64_t r = i;
    const int c = static_cast<int>(r % d8);
    r /= d8;
    const int64_t h = r % H;
    r /= H;
    const int which = static_cast<int>(r % 3);
    r /= 3;
    const int64_t t = r % T;
    const int64_t b = r / T;
    const Bf16x8 *src = which == 0 ? q : (which == 1 ? k : v);
    const int64_t from = src_bthd ? ((b * T + t) * H + h) * d8 + c : ((b * H + h) * T + t) * d8 + c;
    if (!CS_IN_BOUNDS(kKidPackQkv, from, B * H * T * d8)) continue;
    out[i] = src[from];
  }
}
}  // namespace

int pack_qkv(stream_t stream, const void *q, const void *k, const void *v, void *packed, int64_t B, int64_t H, int64_t T,
             int64_t D, int src_bthd) {
  if (D % 8 != 0) return static_cast<int>(cudaErrorInvalidValue);
  const int64_t total = B * T * 3 * H * (D / 8);
  if (total == 0) return 0;
  pack_qkv_kernel<<<grid_for(total, 256, 16), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const Bf16x8 *>(q), static_cast<const Bf16x8 *>(k), static_cast<const Bf16x8 *>(v),
      static_cast<Bf16x8 *>(packed), B, H, T, static_cast<int>(D / 8), src_bthd);
  return finish_launch();
}

// --------------------------------------------------------------------------- LayerNorm ----
namespace {
constexpr int kLnWarps = 4;       // rows per CTA iteration
constexpr int kLnMaxChunks = 8;   // register-resident path: d <= 8 * 256 = 2048
constexpr int kLnBwdCtas = kSmCount * 3;

// One warp per row, grid-stride over rows. Lane l owns the 8-element chunks l, l+32, ... of the
// row. The next row (still packed, in its 128-bit load registers) is fetched before the current
// one is reduced, so that loads stay in flight during the shuffles; the grid is one resident wave.
constexpr int ln_fwd_ctas_per_sm(int chunks) { return chunks <= 5 ? 4 : 1; }
template <int CHUNKS>
__global__ void __launch_bounds__(kLnWarps * 32, ln_fwd_ctas_per_sm(CHUNKS))
ln_fwd_kernel(const __nv_bfloat16 *__restrict__ x, const void *__restrict__ gamma, const void *__restrict__ beta, int pdt,
              __nv_bfloat16 *__restrict__ y, float *__restrict__ mean, float *__restrict__ rstd, int64_t rows, int d, float eps) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nchunks = d / 8;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kLnWarps;
  int64_t row = static_cast<int64_t>(blockIdx.x) * kLnWarps + warp;
  Bf16x8 cur[CHUNKS], nxt[CHUNKS];
  auto load_row = [&](Bf16x8(&dst)[CHUNKS], int64_t r) {
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int chunk = lane + 32 * c;
      if (chunk < nchunks && CS_IN_BOUNDS(kKidLayerNormFwd, r * d + chunk * 8 + 7, rows * d))
        dst[c] = *reinterpret_cast<const Bf16x8 *>(x + r * d + chunk * 8);
    }
  };
  // gamma / beta of this lane's chunks stay in registers for narrow rows (they would otherwise be
  // re-read from L1 for every row: four times the bytes of the row itself)
  constexpr bool kHoist = CHUNKS <= 3;
  float gw[kHoist ? CHUNKS : 1][8], bw[kHoist ? CHUNKS : 1][8];
  if (kHoist) {
#pragma unroll
    for (int c = 0; c < (kHoist ? CHUNKS : 1); ++c) {
      const int chunk = lane + 32 * c;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        gw[c][k] = 0.f;
        bw[c][k] = 0.f;
      }
      if (chunk < nchunks) {
        load8(gamma, chunk * 8, pdt, gw[c]);
        if (beta) load8(beta, chunk * 8, pdt, bw[c]);
      }
    }
  }
  if (row < rows) load_row(cur, row);
  while (row < rows) {
    const int64_t next = row + stride;
    if (next < rows) load_row(nxt, next);
    float v[CHUNKS][8];
    float sum = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      if (lane + 32 * c < nchunks) {
        unpack(cur[c], v[c]);
#pragma unroll
        for (int k = 0; k < 8; ++k) sum += v[c][k];
      }
    }
    const float mu = warp_sum(sum) / d;
    float sq = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      if (lane + 32 * c < nchunks) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float t = v[c][k] - mu;
          sq += t * t;
        }
      }
    }
    const float rs = rsqrtf(warp_sum(sq) / d + eps);
    if (lane == 0) {
      mean[row] = mu;
      rstd[row] = rs;
    }
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int chunk = lane + 32 * c;
      if (chunk < nchunks) {
        float g[8], b[8], o[8];
        if (kHoist) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            g[k] = gw[kHoist ? c : 0][k];
            b[k] = bw[kHoist ? c : 0][k];
          }
        } else {
          load8(gamma, chunk * 8, pdt, g);
          if (beta) {
            load8(beta, chunk * 8, pdt, b);
          } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) b[k] = 0.f;
          }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = (v[c][k] - mu) * rs * g[k] + b[k];
        if (CS_IN_BOUNDS(kKidLayerNormFwd, row * d + chunk * 8 + 7, rows * d)) *reinterpret_cast<Bf16x8 *>(y + row * d + chunk * 8) = pack(o);
      }
    }
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) cur[c] = nxt[c];
    row = next;
  }
}

// Backward: one warp per row, grid-stride over rows, with the next row's operands (packed bf16,
// still in their 128-bit load registers) fetched while the current row is reduced, so that
// global loads stay in flight during the shuffles. Each lane keeps dgamma/dbeta partials for
// its chunks in registers; gamma sits in shared memory. At the end the warps of a CTA combine
// through shared memory and the CTA writes one partial row to scratch; ln_bwd_reduce_kernel
// sums the partial rows.
template <int CHUNKS>
struct LnRowRegs {
  Bf16x8 x[CHUNKS], dy[CHUNKS], res[CHUNKS];
  float mu, rs;
};

template <int CHUNKS>
__device__ __forceinline__ void ln_load_row(LnRowRegs<CHUNKS> &r, const __nv_bfloat16 *x, const __nv_bfloat16 *dy,
                                            const __nv_bfloat16 *dres, const float *mean, const float *rstd, int64_t row,
                                            int64_t rows, int d, int nchunks, int lane) {
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int chunk = lane + 32 * c;
    if (chunk < nchunks && CS_IN_BOUNDS(kKidLayerNormBwd, row * d + chunk * 8 + 7, rows * d)) {
      r.x[c] = *reinterpret_cast<const Bf16x8 *>(x + row * d + chunk * 8);
      r.dy[c] = *reinterpret_cast<const Bf16x8 *>(dy + row * d + chunk * 8);
      if (dres) r.res[c] = *reinterpret_cast<const Bf16x8 *>(dres + row * d + chunk * 8);
    }
  }
  r.mu = mean[row];
  r.rs = rstd[row];
}

template <int CHUNKS>
__global__ void __launch_bounds__(kLnWarps * 32) ln_bwd_kernel(
    const __nv_bfloat16 *__restrict__ dy, const __nv_bfloat16 *__restrict__ x, const void *__restrict__ gamma, int pdt,
    const float *__restrict__ mean, const float *__restrict__ rstd, const __nv_bfloat16 *__restrict__ dres,
    __nv_bfloat16 *__restrict__ dx, float *__restrict__ scratch, int64_t rows, int d) {
  extern __shared__ float smem[];  // [d] gamma, then [kLnWarps][2][d] partials
  float *gamma_s = smem;
  float *partial_s = smem + d;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nchunks = d / 8;
  for (int i = threadIdx.x; i < nchunks; i += blockDim.x) {
    float g[8];
    load8(gamma, i * 8, pdt, g);
#pragma unroll
    for (int k = 0; k < 8; ++k) gamma_s[i * 8 + k] = g[k];
  }
  __syncthreads();
  float dg[CHUNKS][8], db[CHUNKS][8];
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      dg[c][k] = 0.f;
      db[c][k] = 0.f;
    }
  }
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kLnWarps;
  int64_t row = static_cast<int64_t>(blockIdx.x) * kLnWarps + warp;
  LnRowRegs<CHUNKS> cur, nxt;
  if (row < rows) ln_load_row<CHUNKS>(cur, x, dy, dres, mean, rstd, row, rows, d, nchunks, lane);
  while (row < rows) {
    const int64_t next = row + stride;
    if (next < rows) ln_load_row<CHUNKS>(nxt, x, dy, dres, mean, rstd, next, rows, d, nchunks, lane);
    const float mu = cur.mu, rs = cur.rs;
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int chunk = lane + 32 * c;
      if (chunk < nchunks) {
        float xv[8], dyv[8];
        unpack(cur.x[c], xv);
        unpack(cur.dy[c], dyv);
        const float4 g0 = *reinterpret_cast<const float4 *>(gamma_s + chunk * 8);
        const float4 g1 = *reinterpret_cast<const float4 *>(gamma_s + chunk * 8 + 4);
        const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float xh = (xv[k] - mu) * rs;
          const float gy = dyv[k] * g[k];
          s1 += gy * xh;
          s2 += gy;
          dg[c][k] += dyv[k] * xh;
          db[c][k] += dyv[k];
        }
      }
    }
    const float c1 = warp_sum(s1) / d, c2 = warp_sum(s2) / d;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int chunk = lane + 32 * c;
      if (chunk < nchunks) {
        float xv[8], dyv[8], o[8];
        unpack(cur.x[c], xv);
        unpack(cur.dy[c], dyv);
        const float4 g0 = *reinterpret_cast<const float4 *>(gamma_s + chunk * 8);
        const float4 g1 = *reinterpret_cast<const float4 *>(gamma_s + chunk * 8 + 4);
        const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = rs * (dyv[k] * g[k] - c2 - (xv[k] - mu) * rs * c1);
        if (dres) {
          float r[8];
          unpack(cur.res[c], r);
#pragma unroll
          for (int k = 0; k < 8; ++k) o[k] += r[k];
        }
        *reinterpret_cast<Bf16x8 *>(dx + row * d + chunk * 8) = pack(o);
      }
    }
    cur = nxt;
    row = next;
  }
  float *my = partial_s + warp * 2 * d;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int chunk = lane + 32 * c;
    if (chunk < nchunks) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        my[chunk * 8 + k] = dg[c][k];
        my[d + chunk * 8 + k] = db[c][k];
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * d; i += blockDim.x) {
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < kLnWarps; ++w) acc += partial_s[w * 2 * d + i];
    scratch[static_cast<int64_t>(blockIdx.x) * 2 * d + i] = acc;
  }
}

__global__ void __launch_bounds__(1024) ln_bwd_reduce_kernel(const float *__restrict__ scratch, int parts, int d,
                                                             float *__restrict__ dgamma, float *__restrict__ dbeta,
                                                             int accumulate) {
  // blockDim = (32, 32): 32 columns per CTA, 32 row-groups summed through shared memory
  __shared__ float red[32][33];
  const int col = blockIdx.x * 32 + threadIdx.x;
  const int which = blockIdx.y;  // 0 = dgamma, 1 = dbeta
  float acc = 0.f;
  if (col < d)
    for (int p = threadIdx.y; p < parts; p += 32) acc += scratch[static_cast<int64_t>(p) * 2 * d + which * d + col];
  red[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && col < d) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) t += red[i][threadIdx.x];
    float *out = which == 0 ? dgamma : dbeta;
    out[col] = accumulate ? out[col] + t : t;
  }
}

template <int CHUNKS>
int launch_ln_fwd(cudaStream_t s, const void *x, const void *gamma, const void *beta, int pdt, void *y, float *mean,
                  float *rstd, int64_t rows, int d, float eps) {
  const int64_t blocks = (rows + kLnWarps - 1) / kLnWarps;
  const int64_t wave = static_cast<int64_t>(kSmCount) * (CHUNKS <= 8 ? ln_fwd_ctas_per_sm(CHUNKS) * (CHUNKS <= 5 ? 1 : 2) : 2);
  const int grid = static_cast<int>(blocks > wave ? wave : blocks);
  ln_fwd_kernel<CHUNKS><<<grid, kLnWarps * 32, 0, s>>>(static_cast<const __nv_bfloat16 *>(x), gamma, beta, pdt,
                                                       static_cast<__nv_bfloat16 *>(y), mean, rstd, rows, d, eps);
  return finish_launch();
}
template <int CHUNKS>
int launch_ln_bwd(cudaStream_t s, const void *dy, const void *x, const void *gamma, int pdt, const float *mean,
                  const float *rstd, const void *dres, void *dx, float *scratch, int64_t rows, int d, int parts) {
  const size_t smem = (static_cast<size_t>(kLnWarps) * 2 * d + d) * sizeof(float);
  if (smem > 48 * 1024) {
    // Opt in to the larger dynamic shared memory once per width class and device, and report a refusal.
    constexpr int kMaxDevices = 64;
    static std::atomic<size_t> granted[kMaxDevices];
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (device < 0 || device >= kMaxDevices || granted[device].load(std::memory_order_acquire) < smem) {
      e = cudaFuncSetAttribute(ln_bwd_kernel<CHUNKS>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
      if (device >= 0 && device < kMaxDevices) granted[device].store(smem, std::memory_order_release);
    }
  }
  ln_bwd_kernel<CHUNKS><<<parts, kLnWarps * 32, smem, s>>>(
      static_cast<const __nv_bfloat16 *>(dy), static_cast<const __nv_bfloat16 *>(x), gamma, pdt, mean, rstd,
      static_cast<const __nv_bfloat16 *>(dres), static_cast<__nv_bfloat16 *>(dx), scratch, rows, d);
  return finish_launch();
}
}  // namespace

int layernorm_forward(stream_t stream, const void *x, const void *gamma, const void *beta, int param_dtype, void *y,
                      float *mean, float *rstd, int64_t rows, int64_t d, float eps) {
  auto s = static_cast<cudaStream_t>(stream);
  if (d % 8 != 0 || d > 8192 || rows == 0) return rows == 0 ? 0 : static_cast<int>(cudaErrorInvalidValue);
  const int chunks = static_cast<int>((d / 8 + 31) / 32);
  const int di = static_cast<int>(d);
  if (chunks <= 2) return launch_ln_fwd<2>(s, x, gamma, beta, param_dtype, y, mean, rstd, rows, di, eps);
  if (chunks <= 3) return launch_ln_fwd<3>(s, x, gamma, beta, param_dtype, y, mean, rstd, rows, di, eps);
  if (chunks <= 4) return launch_ln_fwd<4>(s, x, gamma, beta, param_dtype, y, mean, rstd, rows, di, eps);
  if (chunks <= 5) return launch_ln_fwd<5>(s, x, gamma, beta, param_dtype, y, mean, rstd, rows, di, eps);
  if (chunks <= 8) return launch_ln_fwd<8>(s, x, gamma, beta, param_dtype, y, mean, rstd, rows, di, eps);
  if (chunks <= 16) return launch_ln_fwd<16>(s, x, gamma, beta, param_dtype, y, mean, rstd, rows, di, eps);
  return launch_ln_fwd<32>(s, x, gamma, beta, param_dtype, y, mean, rstd, rows, di, eps);
}

int64_t layernorm_backward_scratch_rows() { return kLnBwdCtas; }

int layernorm_backward(stream_t stream, const void *dy, const void *x, const void *gamma, int param_dtype,
                       const float *mean, const float *rstd, const void *grad_residual, void *dx, float *dgamma,
                       float *dbeta, int accumulate, float *scratch, int64_t rows, int64_t d) {
  auto s = static_cast<cudaStream_t>(stream);
  if (d % 8 != 0 || d > 8192) return static_cast<int>(cudaErrorInvalidValue);
  if (rows == 0) return 0;
  const int chunks = static_cast<int>((d / 8 + 31) / 32);
  const int di = static_cast<int>(d);
  const int64_t blocks = (rows + kLnWarps - 1) / kLnWarps;
  const int parts = static_cast<int>(blocks > kLnBwdCtas ? kLnBwdCtas : blocks);
  int code;
  if (chunks <= 2) code = launch_ln_bwd<2>(s, dy, x, gamma, param_dtype, mean, rstd, grad_residual, dx, scratch, rows, di, parts);
  else if (chunks <= 3) code = launch_ln_bwd<3>(s, dy, x, gamma, param_dtype, mean, rstd, grad_residual, dx, scratch, rows, di, parts);
  else if (chunks <= 4) code = launch_ln_bwd<4>(s, dy, x, gamma, param_dtype, mean, rstd, grad_residual, dx, scratch, rows, di, parts);
  else if (chunks <= 5) code = launch_ln_bwd<5>(s, dy, x, gamma, param_dtype, mean, rstd, grad_residual, dx, scratch, rows, di, parts);
  else if (chunks <= 8) code = launch_ln_bwd<8>(s, dy, x, gamma, param_dtype, mean, rstd, grad_residual, dx, scratch, rows, di, parts);
  else return static_cast<int>(cudaErrorInvalidValue);  // wider rows use the library path
  if (code != 0) return code;
  dim3 grid(static_cast<unsigned>((d + 31) / 32), 2);
  ln_bwd_reduce_kernel<<<grid, dim3(32, 32), 0, s>>>(scratch, parts, di, dgamma, dbeta, accumulate);
  return finish_launch(1);
}

// --------------------------------------------------------------------------- embedding ----
namespace {
__global__ void __launch_bounds__(256) embedding_fwd_kernel(const int64_t *__restrict__ idx, const void *__restrict__ wte,
                                                            const void *__restrict__ wpe, int tdt,
                                                            __nv_bfloat16 *__restrict__ out, int64_t rows,
                                                            int64_t seq_len, int d, int64_t vocab) {
  const int chunks = d / 8;
  const int64_t total = rows * chunks;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = i / chunks;
    const int chunk = static_cast<int>(i - row * chunks);
    int64_t token = idx[row];
    (void)CS_IN_BOUNDS(kKidEmbeddingFwd, token, vocab);  // diagnostic build: remember the first bad id
    token = token < 0 ? 0 : (token >= vocab ? vocab - 1 : token);  // clamp instead of faulting
    float a[8];
    load8(wte, token * d + chunk * 8, tdt, a);
    if (wpe) {
      float p[8];
      load8(wpe, (row % seq_len) * d + chunk * 8, tdt, p);
#pragma unroll
      for (int k = 0; k < 8; ++k) a[k] += p[k];
    }
    *reinterpret_cast<Bf16x8 *>(out + row * d + chunk * 8) = pack(a);
  }
}

__global__ void __launch_bounds__(256) embedding_bwd_wte_kernel(const int64_t *__restrict__ idx,
                                                                const __nv_bfloat16 *__restrict__ dy,
                                                                float *__restrict__ dwte, int64_t rows, int d,
                                                                int64_t vocab, int64_t padding_idx) {
  const int chunks = d / 8;
  const int64_t total = rows * chunks;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = i / chunks;
    const int chunk = static_cast<int>(i - row * chunks);
    const int64_t token = idx[row];
    if (token != padding_idx) (void)CS_IN_BOUNDS(kKidEmbeddingBwd, token, vocab);
    if (token < 0 || token >= vocab || token == padding_idx) continue;
    float g[8];
    unpack(*reinterpret_cast<const Bf16x8 *>(dy + row * d + chunk * 8), g);
    float *dst = dwte + token * d + chunk * 8;
#pragma unroll
    for (int k = 0; k < 8; ++k) atomicAdd(dst + k, g[k]);
  }
}

__global__ void __launch_bounds__(256) embedding_bwd_wpe_kernel(const __nv_bfloat16 *__restrict__ dy,
                                                                float *__restrict__ dwpe, int accumulate,
                                                                int64_t batch, int64_t seq_len, int d) {
  const int chunks = d / 8;
  const int64_t total = seq_len * chunks;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = i / chunks;
    const int chunk = static_cast<int>(i - t * chunks);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int64_t b = 0; b < batch; ++b) {
      float g[8];
      unpack(*reinterpret_cast<const Bf16x8 *>(dy + (b * seq_len + t) * d + chunk * 8), g);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += g[k];
    }
    float *dst = dwpe + t * d + chunk * 8;
#pragma unroll
    for (int k = 0; k < 8; ++k) dst[k] = accumulate ? dst[k] + acc[k] : acc[k];
  }
}
}  // namespace

int embedding_forward(stream_t stream, const int64_t *idx, const void *wte, const void *wpe, int table_dtype, void *out,
                      int64_t rows, int64_t seq_len, int64_t d, int64_t vocab) {
  if (rows == 0) return 0;
  if (d % 8 != 0) return static_cast<int>(cudaErrorInvalidValue);
  embedding_fwd_kernel<<<grid_for(rows * (d / 8), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      idx, wte, wpe, table_dtype, static_cast<__nv_bfloat16 *>(out), rows, seq_len, static_cast<int>(d), vocab);
  return finish_launch();
}

int embedding_backward(stream_t stream, const int64_t *idx, const void *dy, float *dwte, float *dwpe, int accumulate_wpe,
                       int64_t rows, int64_t seq_len, int64_t d, int64_t vocab, int64_t padding_idx) {
  auto s = static_cast<cudaStream_t>(stream);
  if (rows == 0) return 0;
  if (d % 8 != 0) return static_cast<int>(cudaErrorInvalidValue);
  if (dwte)
    embedding_bwd_wte_kernel<<<grid_for(rows * (d / 8), 256), 256, 0, s>>>(idx, static_cast<const __nv_bfloat16 *>(dy), dwte,
                                                                          rows, static_cast<int>(d), vocab, padding_idx);
  if (dwpe)
    embedding_bwd_wpe_kernel<<<grid_for(seq_len * (d / 8), 256), 256, 0, s>>>(static_cast<const __nv_bfloat16 *>(dy), dwpe,
                                                                             accumulate_wpe, rows / seq_len, seq_len,
                                                                             static_cast<int>(d));
  return finish_launch((dwte ? 1 : 0) + (dwpe ? 1 : 0));
}

// ----------------------------------------------------------------------- cross entropy ----
namespace {
// One warp per row: merge the per-tile (max, sum-exp) partials, emit lse and the row loss.
__global__ void __launch_bounds__(256) ce_finalize_kernel(const float *__restrict__ stats, int64_t n_tiles,
                                                          const __nv_bfloat16 *__restrict__ logits, int64_t ld,
                                                          const int64_t *__restrict__ target, float *__restrict__ lse,
                                                          float *__restrict__ loss_sum, float *__restrict__ count,
                                                          int64_t rows, int64_t ignore_index) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  float row_loss = 0.f, row_valid = 0.f;
  if (row < rows) {
    const float *st = stats + row * n_tiles * 2;
    float mx = -INFINITY;
    for (int64_t t = lane; t < n_tiles; t += 32) mx = fmaxf(mx, st[2 * t]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int64_t t = lane; t < n_tiles; t += 32) {
      const float m = st[2 * t];
      if (m > -INFINITY) sum += st[2 * t + 1] * __expf(m - mx);
    }
    sum = warp_sum(sum);
    const float l = mx + __logf(sum);
    if (lane == 0) {
      lse[row] = l;
      const int64_t tg = target[row];
      if (tg != ignore_index && tg >= 0) (void)CS_IN_BOUNDS(kKidCrossEntropy, tg, ld);
      if (tg != ignore_index && tg >= 0 && tg < ld) {  // a label beyond the row is skipped, never dereferenced
        row_loss = l - __bfloat162float(logits[row * ld + tg]);
        row_valid = 1.f;
      }
    }
  }
  __shared__ float red[2][8];
  if (lane == 0) {
    red[0][threadIdx.x >> 5] = row_loss;
    red[1][threadIdx.x >> 5] = row_valid;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.f, b = 0.f;
    for (int i = 0; i < static_cast<int>(blockDim.x >> 5); ++i) {
      a += red[0][i];
      b += red[1][i];
    }
    if (b > 0.f) {
      atomicAdd(loss_sum, a);
      atomicAdd(count, b);
    }
  }
}
__global__ void ce_mean_kernel(float *loss, const float *count) { loss[0] = loss[0] / fmaxf(count[0], 1.f); }

__global__ void __launch_bounds__(256) ce_backward_kernel(__nv_bfloat16 *__restrict__ logits, int64_t ld,
                                                          const float *__restrict__ lse, const int64_t *__restrict__ target,
                                                          const float *__restrict__ count, float grad_scale, int64_t rows,
                                                          int64_t n, int64_t n_valid, int64_t ignore_index, int64_t col_offset) {
  // One CTA walks whole rows (no per-element division); target and lse are read once per row.
  const int chunks = static_cast<int>(n / 8);
  const float inv = grad_scale / fmaxf(count[0], 1.f);
  const float log2e = 1.4426950408889634f;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const int64_t tg = target[row];
    const bool ignored = tg == ignore_index || tg < 0;
    if (!ignored && col_offset == 0) (void)CS_IN_BOUNDS(kKidCrossEntropy, tg, n_valid);
    const float l2 = ignored ? 0.f : lse[row] * log2e;
    __nv_bfloat16 *row_ptr = logits + row * ld;
    for (int c8 = threadIdx.x; c8 < chunks; c8 += blockDim.x) {
      const int64_t col = static_cast<int64_t>(c8) * 8;
      if (!CS_IN_BOUNDS(kKidCrossEntropy, row * ld + col + 7, rows * ld)) continue;
      Bf16x8 *p = reinterpret_cast<Bf16x8 *>(row_ptr + col);
      float f[8];
      if (ignored) {
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] = 0.f;
      } else {
        unpack(*p, f);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int64_t c = col + k + col_offset;
          float v = c < n_valid ? exp2f(fmaf(f[k], log2e, -l2)) : 0.f;
          if (c == tg) v -= 1.f;
          f[k] = v * inv;
        }
      }
      *p = pack(f);
    }
  }
}
}  // namespace

int cross_entropy_finalize(stream_t stream, const float *stats, int64_t n_tiles, const void *logits, int64_t ld,
                           const int64_t *target, float *lse, float *loss, float *count, int64_t rows,
                           int64_t ignore_index) {
  auto s = static_cast<cudaStream_t>(stream);
  cudaMemsetAsync(loss, 0, sizeof(float), s);
  cudaMemsetAsync(count, 0, sizeof(float), s);
  const int threads = 256;
  const int64_t blocks = (rows * 32 + threads - 1) / threads;
  ce_finalize_kernel<<<static_cast<unsigned>(blocks), threads, 0, s>>>(stats, n_tiles, static_cast<const __nv_bfloat16 *>(logits),
                                                                     ld, target, lse, loss, count, rows, ignore_index);
  ce_mean_kernel<<<1, 1, 0, s>>>(loss, count);
  return finish_launch(2);
}

namespace {
__global__ void __launch_bounds__(256) ce_slice_stats_kernel(const float *__restrict__ stats, int64_t n_tiles,
                                                             const __nv_bfloat16 *__restrict__ logits, int64_t ld,
                                                             const int64_t *__restrict__ target, int64_t col_offset,
                                                             int64_t n_valid_local, float *__restrict__ out, int64_t rows) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (row >= rows) return;
  const float *st = stats + row * n_tiles * 2;
  float mx = -INFINITY;
  for (int64_t t = lane; t < n_tiles; t += 32) mx = fmaxf(mx, st[2 * t]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int64_t t = lane; t < n_tiles; t += 32) {
    const float m = st[2 * t];
    if (m > -INFINITY) sum += st[2 * t + 1] * __expf(m - mx);
  }
  sum = warp_sum(sum);
  if (lane == 0) {
    out[row * 2] = (n_valid_local > 0 && mx > -INFINITY) ? mx + __logf(sum) : -INFINITY;
    const int64_t local = target[row] - col_offset;
    out[row * 2 + 1] = (local >= 0 && local < n_valid_local) ? __bfloat162float(logits[row * ld + local]) : 0.f;
  }
}
}  // namespace

int cross_entropy_slice_stats(stream_t stream, const float *stats, int64_t n_tiles, const void *logits, int64_t ld,
                              const int64_t *target, int64_t col_offset, int64_t n_valid_local, float *out, int64_t rows) {
  if (rows == 0) return 0;
  const int threads = 256;
  const int64_t blocks = (rows * 32 + threads - 1) / threads;
  ce_slice_stats_kernel<<<static_cast<unsigned>(blocks), threads, 0, static_cast<cudaStream_t>(stream)>>>(
      stats, n_tiles, static_cast<const __nv_bfloat16 *>(logits), ld, target, col_offset, n_valid_local, out, rows);
  return finish_launch();
}

int cross_entropy_backward_inplace(stream_t stream, void *logits, int64_t ld, const float *lse, const int64_t *target,
                                   const float *count, float grad_scale, int64_t rows, int64_t n, int64_t n_valid,
                                   int64_t ignore_index, int64_t col_offset) {
  if (n % 8 != 0 || ld % 8 != 0) return static_cast<int>(cudaErrorInvalidValue);
  const int64_t cap = static_cast<int64_t>(kSmCount) * 8;
  ce_backward_kernel<<<static_cast<unsigned>(rows < cap ? rows : cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16 *>(logits), ld, lse, target, count, grad_scale, rows, n, n_valid, ignore_index, col_offset);
  return finish_launch();
}

// ----------------------------------------------------------------------- gradient norm ----
namespace {
// 16-byte loads where the pointer allows it; the scalar loop covers the tail (or everything).
template <typename T>
__global__ void __launch_bounds__(256) sumsq_kernel(const T *__restrict__ x, int64_t n, float *__restrict__ out) {
  constexpr int V = 16 / sizeof(T);
  const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t nv = (reinterpret_cast<uintptr_t>(x) & 15) == 0 ? n / V : 0;
  float acc0 = 0.f, acc1 = 0.f;
  for (int64_t i = gid; i < nv; i += stride) {
    const uint4 raw = *reinterpret_cast<const uint4 *>(x + i * V);
    const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
    for (int k = 0; k < V; k += 2) {
      const float a = to_f<T>(e[k]), b = to_f<T>(e[k + 1]);
      acc0 = fmaf(a, a, acc0);
      acc1 = fmaf(b, b, acc1);
    }
  }
  for (int64_t i = nv * V + gid; i < n; i += stride) {
    const float v = to_f<T>(x[i]);
    acc0 = fmaf(v, v, acc0);
  }
  float acc = warp_sum(acc0 + acc1);
  __shared__ float red[8];
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += red[i];
    atomicAdd(out, t);
  }
}
__global__ void clip_coef_kernel(const float *sumsq, float max_norm, float *coef, float *norm_out) {
  const float norm = sqrtf(sumsq[0]);
  norm_out[0] = norm;
  coef[0] = fminf(1.f, max_norm / (norm + 1e-6f));
}
template <typename T>
__global__ void __launch_bounds__(256) scale_kernel(T *__restrict__ x, int64_t n, const float *__restrict__ coef) {
  const float c = coef[0];
  if (c == 1.f) return;
  constexpr int V = 16 / sizeof(T);
  const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t nv = (reinterpret_cast<uintptr_t>(x) & 15) == 0 ? n / V : 0;
  for (int64_t i = gid; i < nv; i += stride) {
    uint4 raw = *reinterpret_cast<const uint4 *>(x + i * V);
    T *e = reinterpret_cast<T *>(&raw);
#pragma unroll
    for (int k = 0; k < V; ++k) e[k] = from_f<T>(to_f<T>(e[k]) * c);
    *reinterpret_cast<uint4 *>(x + i * V) = raw;
  }
  for (int64_t i = nv * V + gid; i < n; i += stride) x[i] = from_f<T>(to_f<T>(x[i]) * c);
}
}  // namespace

int sum_squares(stream_t stream, const void *x, int dtype, int64_t n, float *sumsq) {
  auto s = static_cast<cudaStream_t>(stream);
  if (n == 0) return 0;
  if (dtype == 0) sumsq_kernel<float><<<grid_for((n + 3) / 4, 256, 8), 256, 0, s>>>(static_cast<const float *>(x), n, sumsq);
  else if (dtype == 1) sumsq_kernel<__nv_bfloat16><<<grid_for((n + 7) / 8, 256, 8), 256, 0, s>>>(static_cast<const __nv_bfloat16 *>(x), n, sumsq);
  else return static_cast<int>(cudaErrorInvalidValue);
  return finish_launch();
}
int clip_coefficient(stream_t stream, const float *sumsq, float max_norm, float *coef, float *norm_out) {
  clip_coef_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(sumsq, max_norm, coef, norm_out);
  return finish_launch();
}
int scale_by_device_scalar(stream_t stream, void *x, int dtype, int64_t n, const float *coef) {
  auto s = static_cast<cudaStream_t>(stream);
  if (n == 0) return 0;
  if (dtype == 0) scale_kernel<float><<<grid_for((n + 3) / 4, 256, 8), 256, 0, s>>>(static_cast<float *>(x), n, coef);
  else if (dtype == 1) scale_kernel<__nv_bfloat16><<<grid_for((n + 7) / 8, 256, 8), 256, 0, s>>>(static_cast<__nv_bfloat16 *>(x), n, coef);
  else return static_cast<int>(cudaErrorInvalidValue);
  return finish_launch();
}
}  // namespace cs::kernels

// ------------------------------------------------------------- allocation-free entry ----
// LayerNorm backward for callers that cannot allocate (see no_alloc.h). Same kernels as
// layernorm_backward() above; the partial dgamma/dbeta rows go to a file-scope device array.
#include "no_alloc.h"

namespace {
static __device__ __align__(256) float g_noalloc_ln_scratch[CS_NOALLOC_LN_PARTS * 2 * CS_NOALLOC_LN_MAX_D];

constexpr int kNoAllocMaxDevices = 64;
std::mutex g_noalloc_mutex;
float *g_noalloc_scratch_ptr[kNoAllocMaxDevices] = {};

// In host code `g_noalloc_ln_scratch` is only a handle for the runtime; the address a kernel
// can use has to be asked for, once per device, with that device current.
int noalloc_scratch(float **out) {
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (device < 0 || device >= kNoAllocMaxDevices) return static_cast<int>(cudaErrorInvalidDevice);
  std::lock_guard<std::mutex> lock{g_noalloc_mutex};
  if (!g_noalloc_scratch_ptr[device]) {
    float *ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_noalloc_ln_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    g_noalloc_scratch_ptr[device] = ptr;
  }
  *out = g_noalloc_scratch_ptr[device];
  return 0;
}
}  // namespace

extern "C" __attribute__((visibility("default"))) int cs_layernorm_backward_noalloc(
    const void *dy, const void *x, const float *gamma, const float *mean, const float *rstd, const void *grad_residual,
    void *dx, float *dgamma, float *dbeta, int accumulate, int64_t rows, int64_t d, void *stream) {
  using namespace cs::kernels;
  if (!dy || !x || !gamma || !mean || !rstd || !dx || !dgamma || !dbeta || rows < 0) return -2;
  if (d <= 0 || d % 8 != 0 || d > CS_NOALLOC_LN_MAX_D) return -1;
  if (rows == 0) return 0;
  float *scratch = nullptr;
  const int rc = noalloc_scratch(&scratch);
  if (rc != 0) return rc;
  auto s = static_cast<cudaStream_t>(stream);
  const int chunks = static_cast<int>((d / 8 + 31) / 32);
  const int di = static_cast<int>(d);
  const int64_t blocks = (rows + kLnWarps - 1) / kLnWarps;
  const int parts = static_cast<int>(blocks > CS_NOALLOC_LN_PARTS ? CS_NOALLOC_LN_PARTS : blocks);
  int code;
  if (chunks <= 2) code = launch_ln_bwd<2>(s, dy, x, gamma, 0, mean, rstd, grad_residual, dx, scratch, rows, di, parts);
  else if (chunks <= 3) code = launch_ln_bwd<3>(s, dy, x, gamma, 0, mean, rstd, grad_residual, dx, scratch, rows, di, parts);
  else if (chunks <= 4) code = launch_ln_bwd<4>(s, dy, x, gamma, 0, mean, rstd, grad_residual, dx, scratch, rows, di, parts);
  else if (chunks <= 5) code = launch_ln_bwd<5>(s, dy, x, gamma, 0, mean, rstd, grad_residual, dx, scratch, rows, di, parts);
  else code = launch_ln_bwd<8>(s, dy, x, gamma, 0, mean, rstd, grad_residual, dx, scratch, rows, di, parts);
  if (code != 0) return code;
  dim3 grid(static_cast<unsigned>((d + 31) / 32), 2);
  ln_bwd_reduce_kernel<<<grid, dim3(32, 32), 0, s>>>(scratch, parts, di, dgamma, dbeta, accumulate);
  return finish_launch(1);
}
