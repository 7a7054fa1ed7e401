// Collectives and fused compute+collective kernels over peer-mapped symmetric memory
// (NVLink 5 through NVSwitch). See collectives.h for the protocol.
//
// The reference project reaches NCCL through c10d for every collective
// (src/communication/{all_reduce,all_gather,reduce_scatter,all_to_all}.cpp) and stages
// multi-tensor all-reduces with at::cat / copy_ (all_reduce.cpp:149-163); its kNVP2P backend
// is declared but not implemented (include/communication/communication.h:51). These kernels
// are that backend: the reduction, the scale/cast and, for ZeRO, the AdamW update happen in
// the same kernel that moves the data.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>

#include "collectives.h"
#include "bounds_check.h"

namespace cs::kernels {
namespace {
std::atomic<long long> g_wait_budget{4000000000LL};

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Diagnostic build: a peer offset must stay inside the arena (arena_bytes 0 = size unknown).
#define CS_PEER_OK(t, byte_offset) ((t).arena_bytes == 0 || CS_IN_BOUNDS(kKidCollective, (byte_offset) + 15, (t).arena_bytes))

__global__ void barrier_kernel(PeerTable t, int slot_base, uint32_t epoch, long long budget, DeviceStatus *status) {
  const int p = threadIdx.x;
  if (p >= t.size) return;
  __threadfence_system();
  st_release_sys(t.flags[p] + slot_base + t.rank, epoch);
  const uint32_t *mine = t.flags[t.rank] + slot_base + p;
  const long long t0 = clock64();
  // epochs only grow; a later epoch also satisfies an earlier wait
  while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
    if (clock64() - t0 > budget) {
      status->code = 2;
      status->kernel_id = 10;
      status->block = p;
      status->detail = static_cast<int>(epoch);
      return;
    }
    __nanosleep(64);
  }
}

struct alignas(16) V4 {
  uint32_t x, y, z, w;
};
__device__ __forceinline__ V4 ld_v4(const void *p) { return *reinterpret_cast<const V4 *>(p); }
__device__ __forceinline__ void st_v4(void *p, const V4 &v) { *reinterpret_cast<V4 *>(p) = v; }

template <int DTYPE>
__device__ __forceinline__ void accumulate(float (&acc)[8], const V4 &v, int &n) {
  if (DTYPE == 0) {
    acc[0] += __uint_as_float(v.x);
    acc[1] += __uint_as_float(v.y);
    acc[2] += __uint_as_float(v.z);
    acc[3] += __uint_as_float(v.w);
    n = 4;
  } else {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&w[i]));
      acc[2 * i] += f.x;
      acc[2 * i + 1] += f.y;
    }
    n = 8;
  }
}
template <int DTYPE>
__device__ __forceinline__ V4 finish(const float (&acc)[8], float scale) {
  V4 o;
  if (DTYPE == 0) {
    o.x = __float_as_uint(acc[0] * scale);
    o.y = __float_as_uint(acc[1] * scale);
    o.z = __float_as_uint(acc[2] * scale);
    o.w = __float_as_uint(acc[3] * scale);
  } else {
    __nv_bfloat162 t0 = __floats2bfloat162_rn(acc[0] * scale, acc[1] * scale);
    __nv_bfloat162 t1 = __floats2bfloat162_rn(acc[2] * scale, acc[3] * scale);
    __nv_bfloat162 t2 = __floats2bfloat162_rn(acc[4] * scale, acc[5] * scale);
    __nv_bfloat162 t3 = __floats2bfloat162_rn(acc[6] * scale, acc[7] * scale);
    o.x = *reinterpret_cast<uint32_t *>(&t0);
    o.y = *reinterpret_cast<uint32_t *>(&t1);
    o.z = *reinterpret_cast<uint32_t *>(&t2);
    o.w = *reinterpret_cast<uint32_t *>(&t3);
  }
  return o;
}

// Slice [begin, end) in 16-byte vectors owned by `rank` out of `vecs` vectors.
__device__ __forceinline__ void slice_of(int64_t vecs, int size, int rank, int64_t &begin, int64_t &end) {
  const int64_t per = (vecs + size - 1) / size;
  begin = per * rank;
  end = begin + per < vecs ? begin + per : vecs;
  if (begin > vecs) begin = vecs;
}

// Vectors each thread keeps in flight per peer. NVLink round trips are a few microseconds, so
// hundreds of kilobytes per SM must be outstanding to fill the links from a few dozen CTAs.
constexpr int kUnroll = 4;

template <int DTYPE>
__global__ void __launch_bounds__(256) all_reduce_twoshot_kernel(PeerTable t, int64_t offset, int64_t vecs, float scale) {
  int64_t begin, end;
  slice_of(vecs, t.size, t.rank, begin, end);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i0 = begin + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < end; i0 += stride * kUnroll) {
    V4 v[kUnroll][kMaxPeers];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < end && CS_PEER_OK(t, offset + i * 16)) {
#pragma unroll
        for (int p = 0; p < kMaxPeers; ++p)
          if (p < t.size) v[u][p] = ld_v4(t.base[(t.rank + p) % t.size] + offset + i * 16);  // all loads in flight first
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < end && CS_PEER_OK(t, offset + i * 16)) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        int n;
#pragma unroll
        for (int p = 0; p < kMaxPeers; ++p)
          if (p < t.size) accumulate<DTYPE>(acc, v[u][p], n);
        const V4 o = finish<DTYPE>(acc, scale);
#pragma unroll
        for (int p = 0; p < kMaxPeers; ++p)
          if (p < t.size) st_v4(t.base[(t.rank + p) % t.size] + offset + i * 16, o);
      }
    }
  }
}

template <int DTYPE>
__global__ void __launch_bounds__(256) pull_reduce_kernel(PeerTable t, int64_t src_offset, char *dst, int64_t vecs, float scale) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < vecs; i0 += stride * kUnroll) {
    V4 v[kUnroll][kMaxPeers];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < vecs && CS_PEER_OK(t, src_offset + i * 16)) {
#pragma unroll
        for (int p = 0; p < kMaxPeers; ++p)
          if (p < t.size) v[u][p] = ld_v4(t.base[(t.rank + p) % t.size] + src_offset + i * 16);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < vecs && CS_PEER_OK(t, src_offset + i * 16)) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        int n;
#pragma unroll
        for (int p = 0; p < kMaxPeers; ++p)
          if (p < t.size) accumulate<DTYPE>(acc, v[u][p], n);
        st_v4(dst + i * 16, finish<DTYPE>(acc, scale));
      }
    }
  }
}

__global__ void __launch_bounds__(512) pull_copy_kernel(PeerTable t, PullCopyArgs a) {
  // blockIdx.y = peer (starting with ourselves so that local data is ready first)
  const int p = (t.rank + blockIdx.y) % t.size;
  const char *src = t.base[p] + a.src_offset[p];
  char *dst = a.dst[p];
  const int64_t vec_per_row = a.row_bytes / 16;
  const int64_t total = a.rows * vec_per_row;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  constexpr int U = 8;  // eight 16-byte loads in flight per thread
  for (int64_t i0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < total; i0 += stride * U) {
    V4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < total) {
        const int64_t r = i / vec_per_row, c = i - r * vec_per_row;
        if (!CS_PEER_OK(t, a.src_offset[p] + r * a.src_stride + c * 16)) continue;
        v[u] = ld_v4(src + r * a.src_stride + c * 16);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < total) {
        const int64_t r = i / vec_per_row, c = i - r * vec_per_row;
        st_v4(dst + r * a.dst_stride + c * 16, v[u]);
      }
    }
  }
}

__global__ void __launch_bounds__(512) rs_adamw_ag_kernel(PeerTable t, ShardedAdamWArgs a) {
  const float gscale = a.clip_coef ? a.grad_scale * a.clip_coef[0] : a.grad_scale;
  const int64_t vecs = a.shard_count / 4;  // four fp32 per vector
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < vecs;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t elem = a.shard_begin + i * 4;
    V4 gv[kMaxPeers];
#pragma unroll
    for (int p = 0; p < kMaxPeers; ++p)
      if (p < t.size) gv[p] = ld_v4(t.base[(t.rank + p) % t.size] + a.grad_offset_bytes + elem * 4);
    float g[4] = {0, 0, 0, 0};
#pragma unroll
    for (int p = 0; p < kMaxPeers; ++p) {
      if (p < t.size) {
        g[0] += __uint_as_float(gv[p].x);
        g[1] += __uint_as_float(gv[p].y);
        g[2] += __uint_as_float(gv[p].z);
        g[3] += __uint_as_float(gv[p].w);
      }
    }
    float4 w = *reinterpret_cast<float4 *>(a.master + i * 4);
    float4 m = *reinterpret_cast<float4 *>(a.exp_avg + i * 4);
    float4 v = *reinterpret_cast<float4 *>(a.exp_avg_sq + i * 4);
    float *wp = &w.x, *mp = &m.x, *vp = &v.x;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float grad = g[k] * gscale;
      float wt = wp[k];
      wt -= a.lr * a.weight_decay * wt;
      const float mt = a.beta1 * mp[k] + (1.f - a.beta1) * grad;
      const float vt = a.beta2 * vp[k] + (1.f - a.beta2) * grad * grad;
      wt -= a.lr * (mt * a.inv_bias_correction1) / (sqrtf(vt * a.inv_bias_correction2) + a.eps);
      wp[k] = wt;
      mp[k] = mt;
      vp[k] = vt;
    }
    *reinterpret_cast<float4 *>(a.master + i * 4) = w;
    *reinterpret_cast<float4 *>(a.exp_avg + i * 4) = m;
    *reinterpret_cast<float4 *>(a.exp_avg_sq + i * 4) = v;
    if (a.lp_offset_bytes >= 0) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(w.x, w.y), hi = __floats2bfloat162_rn(w.z, w.w);
      uint2 packed;
      packed.x = *reinterpret_cast<uint32_t *>(&lo);
      packed.y = *reinterpret_cast<uint32_t *>(&hi);
#pragma unroll
      for (int p = 0; p < kMaxPeers; ++p)
        if (p < t.size)
          *reinterpret_cast<uint2 *>(t.base[(t.rank + p) % t.size] + a.lp_offset_bytes + elem * 2) = packed;
    }
  }
}

int comm_grid(int64_t vecs, int threads, int cap = 64) {
  // A bounded number of CTAs, each with many loads in flight, fills NVLink; keeping the grid
  // below the SM count leaves room for the GEMMs that run next to the collective.
  const int64_t blocks = (vecs + threads - 1) / threads;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}
}  // namespace

void set_peer_wait_budget(long long cycles) { g_wait_budget.store(cycles); }
long long peer_wait_budget() { return g_wait_budget.load(); }

int symm_barrier(stream_t stream, const PeerTable &t, int slot_base, uint32_t epoch, DeviceStatus *status) {
  barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(t, slot_base, epoch, g_wait_budget.load(), status);
  return finish_launch(1);
}

int symm_all_reduce_inplace(stream_t stream, const PeerTable &t, int64_t offset_bytes, int64_t count, int dtype, float scale) {
  const int64_t bytes = count * (dtype == 0 ? 4 : 2);
  if (bytes % 16 != 0 || offset_bytes % 16 != 0) return static_cast<int>(cudaErrorInvalidValue);
  const int64_t vecs = bytes / 16;
  const int64_t per = (vecs + t.size - 1) / t.size;
  auto s = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    all_reduce_twoshot_kernel<0><<<comm_grid((per + kUnroll - 1) / kUnroll, 256, 128), 256, 0, s>>>(t, offset_bytes, vecs, scale);
  else
    all_reduce_twoshot_kernel<1><<<comm_grid((per + kUnroll - 1) / kUnroll, 256, 128), 256, 0, s>>>(t, offset_bytes, vecs, scale);
  return finish_launch(1);
}

int symm_pull_reduce(stream_t stream, const PeerTable &t, int64_t src_offset_bytes, void *dst, int64_t count, int dtype,
                     float scale) {
  const int64_t bytes = count * (dtype == 0 ? 4 : 2);
  if (bytes % 16 != 0 || src_offset_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(dst) & 15))
    return static_cast<int>(cudaErrorInvalidValue);
  auto s = static_cast<cudaStream_t>(stream);
  const int64_t vecs = bytes / 16;
  if (dtype == 0)
    pull_reduce_kernel<0><<<comm_grid((vecs + kUnroll - 1) / kUnroll, 256, 128), 256, 0, s>>>(t, src_offset_bytes, static_cast<char *>(dst), vecs, scale);
  else
    pull_reduce_kernel<1><<<comm_grid((vecs + kUnroll - 1) / kUnroll, 256, 128), 256, 0, s>>>(t, src_offset_bytes, static_cast<char *>(dst), vecs, scale);
  return finish_launch(1);
}

int symm_all_reduce_oneshot(stream_t stream, const PeerTable &t, int64_t staging_offset, void *dst, int64_t count, int dtype,
                            float scale) {
  return symm_pull_reduce(stream, t, staging_offset, dst, count, dtype, scale);
}

int symm_pull_copy(stream_t stream, const PeerTable &t, const PullCopyArgs &a) {
  if (a.row_bytes % 16 != 0 || a.src_stride % 16 != 0 || a.dst_stride % 16 != 0) return static_cast<int>(cudaErrorInvalidValue);
  for (int p = 0; p < t.size; ++p)
    if ((a.src_offset[p] % 16) != 0 || (reinterpret_cast<uintptr_t>(a.dst[p]) & 15)) return static_cast<int>(cudaErrorInvalidValue);
  const int64_t vecs = a.rows * (a.row_bytes / 16);
  int gx = comm_grid((vecs + 7) / 8, 512);
  const int per_peer_cap = 64 / t.size > 8 ? 64 / t.size : 8;
  if (gx > per_peer_cap) gx = per_peer_cap;  // x peers
  dim3 grid(gx, t.size);
  pull_copy_kernel<<<grid, 512, 0, static_cast<cudaStream_t>(stream)>>>(t, a);
  return finish_launch(1);
}

int symm_reduce_scatter_adamw_all_gather(stream_t stream, const PeerTable &t, const ShardedAdamWArgs &a) {
  if (a.shard_count % 4 != 0 || a.shard_begin % 4 != 0 || a.grad_offset_bytes % 16 != 0 ||
      (a.lp_offset_bytes >= 0 && a.lp_offset_bytes % 16 != 0))
    return static_cast<int>(cudaErrorInvalidValue);
  if (a.shard_count == 0) return 0;
  rs_adamw_ag_kernel<<<comm_grid(a.shard_count / 4, 512) * 2, 512, 0, static_cast<cudaStream_t>(stream)>>>(t, a);
  return finish_launch(1);
}
CS_DEFINE_BOUNDS_GETTER(bounds_report_collectives)
}  // namespace cs::kernels
