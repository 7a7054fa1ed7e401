// SPDX-License-Identifier: Apache-2.0
// Collectives and fused compute+collective kernels over peer-mapped symmetric memory
// (NVLink 5 through NVSwitch). See collectives.h for the protocol.
//
// The reference project reaches NCCL through c10d for every collective
// (src/communication/{all_reduce,all_gather,reduce_scatter,all_to_all}.cpp) and stages
// multi-tensor all-reduces with at::cat / copy_ (all_reduce.cpp:149-163); its kNVP2P backend
// is declared but not implemented (include/communication/communication.h:51). These kernels
// are that backend: the cross-rank barriers, the reduction (inside the switch when the arena has
// a multicast mapping), the scale/cast and, for ZeRO, the AdamW update happen in the one kernel
// that moves the data.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <mutex>

#include "collectives.h"
#include "bounds_check.h"

namespace cs::kernels {
namespace {
std::atomic<long long> g_wait_budget{4000000000LL};
std::atomic<int> g_grid_cap{256};
std::atomic<int> g_multicast_min_ranks{3};

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t *p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Diagnostic build: a peer offset must stay inside the arena (arena_bytes 0 = size unknown).
#define CS_PEER_OK(t, byte_offset) ((t).arena_bytes == 0 || CS_IN_BOUNDS(kKidCollective, (byte_offset) + 15, (t).arena_bytes))

constexpr int kThreads = 256;
// Light blocks (256 threads, at most 40 registers, no shared memory to speak of): many of them fit on an SM, and a
// collective never needs more than a fraction of the machine to fill NVLink.
#define CS_COMM_BOUNDS __launch_bounds__(kThreads, 6)

__device__ __forceinline__ uint32_t *channel_words(const PeerTable &t, int peer, int channel) {
  return t.flags[peer] + kChannelBase + channel * kChannelWords;
}

// epochs only grow; a later epoch also satisfies an earlier wait
__device__ __forceinline__ bool reached(uint32_t seen, uint32_t epoch) { return static_cast<int32_t>(seen - epoch) >= 0; }

__device__ __forceinline__ void report_timeout(const Handshake &h, int kernel_id, int who) {
  h.status->code = 2;
  h.status->kernel_id = kernel_id;
  h.status->block = who;
  h.status->detail = static_cast<int>(h.epoch);
}

// Flag exchange with every peer through slots [first, first + size) of the channel: "this rank reached
// the point" is stored into slot `rank` of every peer, then this rank's own slots are polled.
// Run by the first `size` threads of one block. A wait that exceeds the budget records a status and gives up.
__device__ __forceinline__ void exchange_flags(const PeerTable &t, const Handshake &h, int first, int kernel_id) {
  const int p = threadIdx.x;
  if (p >= t.size) return;
  __threadfence_system();
  st_release_sys(channel_words(t, p, h.channel) + first + t.rank, h.epoch);
  const uint32_t *mine = channel_words(t, t.rank, h.channel) + first + p;
  const long long t0 = clock64();
  while (!reached(ld_acquire_sys(mine), h.epoch)) {
    if (clock64() - t0 > h.budget) {
      report_timeout(h, kernel_id, p);
      return;
    }
    __nanosleep(32);
  }
}

// Opening barrier: every rank's contribution to this launch is complete (the peers' kernels have started,
// which their streams allow only after the producers of their data). Block 0 talks to the peers and
// releases the other blocks through a local flag.
__device__ __forceinline__ void open_collective(const PeerTable &t, const Handshake &h, int kernel_id) {
  uint32_t *local = channel_words(t, t.rank, h.channel);
  if (blockIdx.x == 0) {
    exchange_flags(t, h, 0, kernel_id);
    __syncthreads();
    if (threadIdx.x == 0) st_release_gpu(local + 16, h.epoch);
  } else {
    if (threadIdx.x == 0) {
      const long long t0 = clock64();
      while (!reached(ld_acquire_gpu(local + 16), h.epoch)) {
        if (clock64() - t0 > h.budget) {
          report_timeout(h, kernel_id, 100 + static_cast<int>(blockIdx.x));
          break;
        }
        __nanosleep(64);
      }
    }
    __syncthreads();
  }
}

// Closing barrier: the last block of this rank to finish tells the peers "everything this rank wrote into
// your memory has landed, and it no longer reads yours" and waits for the same word from them, so that the
// kernel ends only when this rank's buffers are complete and free to be overwritten.
__device__ __forceinline__ void close_collective(const PeerTable &t, const Handshake &h, int kernel_id) {
  __shared__ int last;
  // The block barrier orders every thread's stores before thread 0's system-scope fence, which then covers them
  // all (cumulativity): one fence per block instead of one per warp.
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    uint32_t *local = channel_words(t, t.rank, h.channel);
    const uint32_t done = atomicAdd(local + 17, 1u) + 1u;
    last = done == h.blocks_before + gridDim.x;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  exchange_flags(t, h, 8, kernel_id);
}

struct alignas(16) V4 {
  uint32_t x, y, z, w;
};
__device__ __forceinline__ V4 ld_v4(const void *p) { return *reinterpret_cast<const V4 *>(p); }
__device__ __forceinline__ void st_v4(void *p, const V4 &v) { *reinterpret_cast<V4 *>(p) = v; }

// ---- multimem (NVLink multicast) accesses: one instruction addresses every rank's copy ----
__device__ __forceinline__ V4 mc_ld_reduce_f32(const void *p) {
  V4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ V4 mc_ld_reduce_bf16(const void *p) {
  V4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void mc_st(void *p, const V4 &v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void mc_st_v2(void *p, uint32_t a, uint32_t b) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}

template <int DTYPE>
__device__ __forceinline__ void accumulate(float (&acc)[8], const V4 &v) {
  if (DTYPE == 0) {
    acc[0] += __uint_as_float(v.x);
    acc[1] += __uint_as_float(v.y);
    acc[2] += __uint_as_float(v.z);
    acc[3] += __uint_as_float(v.w);
  } else {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&w[i]));
      acc[2 * i] += f.x;
      acc[2 * i + 1] += f.y;
    }
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
// scale applied to a vector that the switch already summed
template <int DTYPE>
__device__ __forceinline__ V4 scaled(const V4 &v, float scale) {
  if (scale == 1.0f) return v;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  accumulate<DTYPE>(acc, v);
  return finish<DTYPE>(acc, scale);
}

// Sum over all ranks of the 16-byte vector at `offset`: one switch-side reduction, or one load per peer.
// Peer loads are issued in groups of four so that the register budget of the kernel holds.
template <int DTYPE>
__device__ __forceinline__ V4 reduce_vector(const PeerTable &t, int64_t offset, float scale) {
  if (t.mc) return scaled<DTYPE>(DTYPE == 0 ? mc_ld_reduce_f32(t.mc + offset) : mc_ld_reduce_bf16(t.mc + offset), scale);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
  for (int g = 0; g < kMaxPeers; g += 4) {
    if (g >= t.size) break;
    V4 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (g + j < t.size) v[j] = ld_v4(t.base[(t.rank + g + j) % t.size] + offset);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (g + j < t.size) accumulate<DTYPE>(acc, v[j]);
  }
  return finish<DTYPE>(acc, scale);
}
// Writes a 16-byte vector into every rank's arena at `offset`.
__device__ __forceinline__ void broadcast_vector(const PeerTable &t, int64_t offset, const V4 &v) {
  if (t.mc) {
    mc_st(t.mc + offset, v);
    return;
  }
#pragma unroll
  for (int p = 0; p < kMaxPeers; ++p)
    if (p < t.size) st_v4(t.base[(t.rank + p) % t.size] + offset, v);
}

// Slice [begin, end) in 16-byte vectors owned by `rank` out of `vecs` vectors.
__device__ __forceinline__ void slice_of(int64_t vecs, int size, int rank, int64_t &begin, int64_t &end) {
  const int64_t per = (vecs + size - 1) / size;
  begin = per * rank;
  end = begin + per < vecs ? begin + per : vecs;
  if (begin > vecs) begin = vecs;
}

__global__ void barrier_kernel(PeerTable t, int slot_base, uint32_t epoch, long long budget, DeviceStatus *status) {
  const int p = threadIdx.x;
  if (p >= t.size) return;
  __threadfence_system();
  st_release_sys(t.flags[p] + slot_base + t.rank, epoch);
  const uint32_t *mine = t.flags[t.rank] + slot_base + p;
  const long long t0 = clock64();
  while (!reached(ld_acquire_sys(mine), epoch)) {
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

// Vectors each thread keeps in flight. NVLink round trips are a few microseconds, so megabytes must be
// outstanding per GPU; the grid supplies them (up to one light block per SM), not the per-thread depth.
constexpr int kUnroll = 4;

// How a reducing kernel reaches the other copies. One instantiation per path, so that each gets its own
// register allocation: the switch path holds kUnroll reduced vectors, the pair path both copies of
// kUnroll vectors (and trades two resident blocks per SM for them), the general path one vector per peer.
enum : int { kPathSwitch = 0, kPathPair = 1, kPathPeers = 2 };
#define CS_REDUCE_BOUNDS(PATH) __launch_bounds__(kThreads, (PATH) == kPathPair ? 4 : 6)

// Sums of the vectors at base + i * 16 for i = i0, i0 + stride, ... (kUnroll of them, those below `end`).
template <int DTYPE, int PATH>
__device__ __forceinline__ void reduce_strip(const PeerTable &t, int64_t base, int64_t i0, int64_t stride, int64_t end, float scale,
                                             V4 (&out)[kUnroll]) {
  if (PATH == kPathSwitch) {
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < end && CS_PEER_OK(t, base + i * 16)) out[u] = DTYPE == 0 ? mc_ld_reduce_f32(t.mc + base + i * 16) : mc_ld_reduce_bf16(t.mc + base + i * 16);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) out[u] = scaled<DTYPE>(out[u], scale);
  } else if (PATH == kPathPair) {
    const char *mine = t.base[t.rank] + base, *theirs = t.base[t.rank ^ 1] + base;
    V4 other[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < end && CS_PEER_OK(t, base + i * 16)) {
        other[u] = ld_v4(theirs + i * 16);
        out[u] = ld_v4(mine + i * 16);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      accumulate<DTYPE>(acc, out[u]);
      accumulate<DTYPE>(acc, other[u]);
      out[u] = finish<DTYPE>(acc, scale);
    }
  } else {
#pragma unroll 1
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < end && CS_PEER_OK(t, base + i * 16)) out[u] = reduce_vector<DTYPE>(t, base + i * 16, scale);
    }
  }
}

template <int DTYPE, int PATH>
__global__ void CS_REDUCE_BOUNDS(PATH) all_reduce_kernel(PeerTable t, Handshake h, int64_t offset, int64_t vecs, float scale) {
  open_collective(t, h, 11);
  int64_t begin, end;
  slice_of(vecs, t.size, t.rank, begin, end);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i0 = begin + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < end; i0 += stride * kUnroll) {
    V4 v[kUnroll];
    reduce_strip<DTYPE, PATH>(t, offset, i0, stride, end, scale, v);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < end && CS_PEER_OK(t, offset + i * 16)) broadcast_vector(t, offset + i * 16, v[u]);
    }
  }
  close_collective(t, h, 11);
}

// out = v + residual, elementwise on eight bf16 values (fp32 math)
__device__ __forceinline__ V4 add_bf16x8(const V4 &v, const V4 &r) {
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  accumulate<1>(acc, v);
  accumulate<1>(acc, r);
  return finish<1>(acc, 1.0f);
}

template <int DTYPE, int PATH>
__global__ void CS_REDUCE_BOUNDS(PATH) reduce_scatter_kernel(PeerTable t, Handshake h, int64_t src_offset, char *dst, const char *residual,
                                                             int64_t vecs, float scale) {
  open_collective(t, h, 12);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < vecs; i0 += stride * kUnroll) {
    V4 v[kUnroll];
    reduce_strip<DTYPE, PATH>(t, src_offset, i0, stride, vecs, scale, v);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < vecs && CS_PEER_OK(t, src_offset + i * 16)) {
        if (DTYPE == 1 && residual) v[u] = add_bf16x8(v[u], ld_v4(residual + i * 16));
        st_v4(dst + i * 16, v[u]);
      }
    }
  }
  close_collective(t, h, 12);
}

__global__ void CS_COMM_BOUNDS all_gather_push_kernel(PeerTable t, Handshake h, const char *src, int64_t dst_offset, int64_t vecs) {
  open_collective(t, h, 13);
  const int64_t mine = dst_offset + static_cast<int64_t>(t.rank) * vecs * 16;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < vecs; i0 += stride * kUnroll) {
    V4 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < vecs) v[u] = ld_v4(src + i * 16);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < vecs && CS_PEER_OK(t, mine + i * 16)) broadcast_vector(t, mine + i * 16, v[u]);
    }
  }
  close_collective(t, h, 13);
}

// Runs beside the GEMM that consumes the chunks, on the SMs that GEMM leaves free: few blocks, many threads.
// Measured alternatives on 2 and 4 GPUs (774M tensor-parallel step): 128 light blocks sharing the GEMM's SMs made the
// gather itself faster on two GPUs (21.7 against 27.1 ms per step) but the GEMM slower (37.3 against 33.9 ms) and the
// step 4 % longer; the same copies on the bulk engine (16 single-warp blocks) were 2-3 % slower than this kernel.
__global__ void __launch_bounds__(1024, 1) all_gather_chunked_kernel(PeerTable t, Handshake h, const char *src, int64_t dst_offset, int64_t vecs_per_chunk,
                                                         int chunks) {
  open_collective(t, h, 16);
  __shared__ int last_of_chunk;
  uint32_t *local = channel_words(t, t.rank, h.channel);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int c = 0; c < chunks; ++c) {
    const char *from = src + static_cast<int64_t>(c) * vecs_per_chunk * 16;
    const int64_t to = dst_offset + (static_cast<int64_t>(t.rank) * chunks + c) * vecs_per_chunk * 16;
    for (int64_t i0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < vecs_per_chunk; i0 += stride * kUnroll) {
      V4 v[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int64_t i = i0 + u * stride;
        if (i < vecs_per_chunk) v[u] = ld_v4(from + i * 16);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int64_t i = i0 + u * stride;
        if (i < vecs_per_chunk && CS_PEER_OK(t, to + i * 16)) broadcast_vector(t, to + i * 16, v[u]);
      }
    }
    // the block that completes the chunk on this rank announces it to every rank (its own included)
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();  // covers the whole block's stores, which the barrier ordered before it
      last_of_chunk = atomicAdd(local + kChunkCounters + c, 1u) + 1u == gridDim.x;
      if (last_of_chunk) atomicExch(local + kChunkCounters + c, 0u);  // every block has counted: ready for the next launch
    }
    __syncthreads();
    if (last_of_chunk && threadIdx.x < t.size) {
      __threadfence_system();
      st_release_sys(channel_words(t, threadIdx.x, h.channel) + kChunkFlags + t.rank * kMaxChunks + c, h.epoch);
    }
  }
  close_collective(t, h, 16);
}

__global__ void CS_COMM_BOUNDS slot_sum_kernel(PeerTable t, Handshake h, const char *slots, int64_t slot_bytes, char *dst, const char *residual,
                                               int64_t vecs) {
  open_collective(t, h, 17);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < vecs; i += stride) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
    for (int g = 0; g < kMaxPeers; g += 4) {
      if (g >= t.size) break;
      V4 v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (g + j < t.size) v[j] = ld_v4(slots + (g + j) * slot_bytes + i * 16);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (g + j < t.size) accumulate<1>(acc, v[j]);
    }
    if (residual) accumulate<1>(acc, ld_v4(residual + i * 16));
    st_v4(dst + i * 16, finish<1>(acc, 1.0f));
  }
}

// Blocks [p * per_peer_blocks, (p + 1) * per_peer_blocks) copy from the p-th peer, counted from this rank (local data
// first, no two ranks start on the same peer). Eight 16-byte loads per thread are in flight.
__global__ void __launch_bounds__(512) pull_copy_kernel(PeerTable t, Handshake h, PullCopyArgs a, int per_peer_blocks) {
  open_collective(t, h, 14);
  const int p = (t.rank + static_cast<int>(blockIdx.x) / per_peer_blocks) % t.size;
  const int bx = static_cast<int>(blockIdx.x) % per_peer_blocks;
  const char *src = t.base[p] + a.src_offset[p];
  char *dst = a.dst[p];
  const int64_t vec_per_row = a.row_bytes / 16;
  const int64_t total = a.rows * vec_per_row;
  const int64_t stride = static_cast<int64_t>(per_peer_blocks) * blockDim.x;
  constexpr int U = 8;
  const bool flat = a.rows == 1;
  for (int64_t i0 = static_cast<int64_t>(bx) * blockDim.x + threadIdx.x; i0 < total; i0 += stride * U) {
    V4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < total) {
        const int64_t r = flat ? 0 : i / vec_per_row, c = i - r * vec_per_row;
        if (!CS_PEER_OK(t, a.src_offset[p] + r * a.src_stride + c * 16)) continue;
        v[u] = ld_v4(src + r * a.src_stride + c * 16);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < total) {
        const int64_t r = flat ? 0 : i / vec_per_row, c = i - r * vec_per_row;
        st_v4(dst + r * a.dst_stride + c * 16, v[u]);
      }
    }
  }
  close_collective(t, h, 14);
}

// ---- bulk copy engine ----------------------------------------------------------------------------------------
// Copies whose source and destination are plain byte ranges (all-gather, all-to-all, strided pulls) do not need an
// SM's load/store units: one thread per block drives cp.async.bulk transfers through a ring of shared-memory stages,
// global (local or a peer's) -> shared completing on an mbarrier, shared -> global (local and peers') as bulk groups.
// NVLink then carries full-size packets instead of 16-byte vector accesses, and a few dozen single-warp blocks keep
// megabytes in flight. No load here carries a cluster-multicast qualifier; the sources may be peer memory.
constexpr int kBulkStages = 4;
constexpr int kBulkStageBytes = 32 * 1024;
constexpr int kBulkSmemBytes = kBulkStages * kBulkStageBytes + 128;  // ring + mbarriers
constexpr int kBulkThreads = 32;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes),
               "r"(bar)
               : "memory");
}
__device__ __forceinline__ void bulk_store(void *dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// The ring as seen by the driving thread. Item i uses stage i % kBulkStages; its load is issued kBulkStages - 1 items
// ahead of its stores. A stage is loaded again only after every store group committed so far has read its source.
struct BulkRing {
  uint32_t data, bars;
  int64_t loaded{0}, stored{0};
  bool failed{false};

  __device__ void init(unsigned char *smem) {
    data = smem_u32(smem);
    bars = data + kBulkStages * kBulkStageBytes;
    for (int s = 0; s < kBulkStages; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bars + 8u * s) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __device__ void load(const void *src, uint32_t bytes) {
    const int s = static_cast<int>(loaded % kBulkStages);
    if (loaded >= kBulkStages) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    bulk_load(data + s * kBulkStageBytes, src, bytes, bars + 8u * s);
    ++loaded;
  }
  // Waits (bounded) for the oldest loaded item and returns its shared-memory address; 0 after a timeout.
  __device__ uint32_t arrived(const Handshake &h, int kernel_id) {
    const int s = static_cast<int>(stored % kBulkStages);
    const uint32_t parity = static_cast<uint32_t>((stored / kBulkStages) & 1);
    const long long t0 = clock64();
    while (!mbar_try_wait(bars + 8u * s, parity)) {
      if (clock64() - t0 > h.budget) {
        report_timeout(h, kernel_id, 200 + static_cast<int>(blockIdx.x));
        failed = true;
        return 0;
      }
    }
    ++stored;
    return data + s * kBulkStageBytes;
  }
  // After a timeout: loads still in flight target this block's shared memory, so let them land (bounded again).
  __device__ void settle(const Handshake &h) {
    while (stored < loaded) {
      const int s = static_cast<int>(stored % kBulkStages);
      const uint32_t parity = static_cast<uint32_t>((stored / kBulkStages) & 1);
      const long long t0 = clock64();
      while (!mbar_try_wait(bars + 8u * s, parity))
        if (clock64() - t0 > h.budget) return;
      ++stored;
    }
  }
  // Every store has been performed (not only read from shared memory) and is ordered before what this thread does next.
  __device__ void drain() {
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    asm volatile("fence.proxy.async;" ::: "memory");
  }
};

// All-gather push: this rank's `bytes` at `src` into every rank's arena at dst_offset + rank * bytes.
// Pieces of at most one stage are dealt to the blocks round-robin.
__global__ void __launch_bounds__(kBulkThreads) bulk_gather_push_kernel(PeerTable t, Handshake h, const char *src, int64_t dst_offset,
                                                                        int64_t bytes) {
  extern __shared__ __align__(128) unsigned char bulk_smem[];
  open_collective(t, h, 18);
  if (threadIdx.x == 0) {
    BulkRing ring;
    ring.init(bulk_smem);
    const int64_t pieces = (bytes + kBulkStageBytes - 1) / kBulkStageBytes;
    const int64_t mine = pieces > blockIdx.x ? (pieces - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const int64_t to = dst_offset + static_cast<int64_t>(t.rank) * bytes;
    auto offset_of = [&](int64_t k) { return (static_cast<int64_t>(blockIdx.x) + k * gridDim.x) * kBulkStageBytes; };
    auto size_of = [&](int64_t k) {
      const int64_t rest = bytes - offset_of(k);
      return static_cast<uint32_t>(rest < kBulkStageBytes ? rest : kBulkStageBytes);
    };
    for (int64_t k = 0; k < mine + kBulkStages - 1 && !ring.failed; ++k) {
      if (k < mine) ring.load(src + offset_of(k), size_of(k));
      const int64_t j = k - (kBulkStages - 1);
      if (j >= 0) {
        const uint32_t from = ring.arrived(h, 18);
        if (!from) break;  // failed is set
        for (int p = 0; p < t.size; ++p) {
          const int peer = (t.rank + p) % t.size;
          if (CS_PEER_OK(t, to + offset_of(j) + size_of(j) - 16)) bulk_store(t.base[peer] + to + offset_of(j), from, size_of(j));
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      }
    }
    if (ring.failed) ring.settle(h);
    ring.drain();
  }
  close_collective(t, h, 18);
}

// Strided pulls (all-to-all, all-gather from memory outside the arena): blocks [p * per_peer, (p + 1) * per_peer)
// copy from the p-th peer counted from this rank. A row longer than one stage is cut into pieces.
__global__ void __launch_bounds__(kBulkThreads) bulk_pull_copy_kernel(PeerTable t, Handshake h, PullCopyArgs a, int per_peer_blocks) {
  extern __shared__ __align__(128) unsigned char bulk_smem[];
  open_collective(t, h, 19);
  if (threadIdx.x == 0) {
    BulkRing ring;
    ring.init(bulk_smem);
    const int p = (t.rank + static_cast<int>(blockIdx.x) / per_peer_blocks) % t.size;
    const int bx = static_cast<int>(blockIdx.x) % per_peer_blocks;
    const char *src = t.base[p] + a.src_offset[p];
    char *dst = a.dst[p];
    const int64_t pieces_per_row = (a.row_bytes + kBulkStageBytes - 1) / kBulkStageBytes;
    const int64_t pieces = a.rows * pieces_per_row;
    const int64_t mine = pieces > bx ? (pieces - bx + per_peer_blocks - 1) / per_peer_blocks : 0;
    auto piece_of = [&](int64_t k, int64_t &row, int64_t &col, uint32_t &size) {
      const int64_t i = bx + k * per_peer_blocks;
      row = i / pieces_per_row;
      col = (i - row * pieces_per_row) * kBulkStageBytes;
      const int64_t rest = a.row_bytes - col;
      size = static_cast<uint32_t>(rest < kBulkStageBytes ? rest : kBulkStageBytes);
    };
    for (int64_t k = 0; k < mine + kBulkStages - 1 && !ring.failed; ++k) {
      int64_t row, col;
      uint32_t size;
      if (k < mine) {
        piece_of(k, row, col, size);
        if (!CS_PEER_OK(t, a.src_offset[p] + row * a.src_stride + col + size - 16)) {
          ring.failed = true;
          break;
        }
        ring.load(src + row * a.src_stride + col, size);
      }
      const int64_t j = k - (kBulkStages - 1);
      if (j >= 0) {
        piece_of(j, row, col, size);
        const uint32_t from = ring.arrived(h, 19);
        if (!from) break;
        bulk_store(dst + row * a.dst_stride + col, from, size);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      }
    }
    if (ring.failed) ring.settle(h);
    ring.drain();
  }
  close_collective(t, h, 19);
}

__global__ void CS_COMM_BOUNDS rs_adamw_ag_kernel(PeerTable t, Handshake h, ShardedAdamWArgs a) {
  open_collective(t, h, 15);
  const float gscale = a.clip_coef ? a.grad_scale * a.clip_coef[0] : a.grad_scale;
  // this rank's blocks that intersect the range: j0, j0 + size, ...
  const int64_t first = a.range_begin / a.block, last = (a.range_end - 1) / a.block;
  const int64_t j0 = first + ((t.rank - first % t.size) + t.size) % t.size;
  const int64_t mine = j0 > last ? 0 : (last - j0) / t.size + 1;
  const int64_t vecs_per_block = a.block / 4;  // four fp32 per vector
  const int64_t items = mine * vecs_per_block;
  for (int64_t w = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; w < items;
       w += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t k = w / vecs_per_block, q = w - k * vecs_per_block;
    const int64_t j = j0 + k * t.size;
    const int64_t elem = j * a.block + q * 4;              // position in the arenas
    if (elem < a.range_begin || elem >= a.range_end) continue;  // the range may start or end inside a block
    const int64_t local = (j / t.size) * a.block + q * 4;  // position in this rank's shards
    const V4 gsum = reduce_vector<0>(t, a.grad_offset_bytes + elem * 4, 1.0f);
    const float g[4] = {__uint_as_float(gsum.x), __uint_as_float(gsum.y), __uint_as_float(gsum.z), __uint_as_float(gsum.w)};
    float4 wv = *reinterpret_cast<float4 *>(a.master + local);
    float4 m = *reinterpret_cast<float4 *>(a.exp_avg + local);
    float4 v = *reinterpret_cast<float4 *>(a.exp_avg_sq + local);
    float *wp = &wv.x, *mp = &m.x, *vp = &v.x;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float grad = g[i] * gscale;
      float wt = wp[i];
      wt -= a.lr * a.weight_decay * wt;
      const float mt = a.beta1 * mp[i] + (1.f - a.beta1) * grad;
      const float vt = a.beta2 * vp[i] + (1.f - a.beta2) * grad * grad;
      wt -= a.lr * (mt * a.inv_bias_correction1) / (sqrtf(vt * a.inv_bias_correction2) + a.eps);
      wp[i] = wt;
      mp[i] = mt;
      vp[i] = vt;
    }
    *reinterpret_cast<float4 *>(a.master + local) = wv;
    *reinterpret_cast<float4 *>(a.exp_avg + local) = m;
    *reinterpret_cast<float4 *>(a.exp_avg_sq + local) = v;
    if (a.lp_offset_bytes >= 0) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(wv.x, wv.y), hi = __floats2bfloat162_rn(wv.z, wv.w);
      const uint32_t p0 = *reinterpret_cast<uint32_t *>(&lo), p1 = *reinterpret_cast<uint32_t *>(&hi);
      const int64_t off = a.lp_offset_bytes + elem * 2;
      if (t.mc) {
        mc_st_v2(t.mc + off, p0, p1);
      } else {
#pragma unroll
        for (int p = 0; p < kMaxPeers; ++p)
          if (p < t.size) *reinterpret_cast<uint2 *>(t.base[(t.rank + p) % t.size] + off) = make_uint2(p0, p1);
      }
    }
  }
  close_collective(t, h, 15);
}

// The bulk engine takes over from the vector kernels where its fixed cost (one 32 KB piece per block and trip) pays.
constexpr int64_t kBulkMinBytes = 512 * 1024;
constexpr int64_t kBulkMinRowBytes = 4096;
int bulk_grid_cap() {
  const int cap = g_grid_cap.load() / 2;  // one block per SM (shared memory), so half the light kernels' share
  return cap < 8 ? 8 : cap;
}
// Opts the bulk kernels in to their shared-memory size, once per device.
bool bulk_engine_ready() {
  static std::mutex mu;
  static bool done[64] = {};
  static bool ok[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return false;
  std::lock_guard<std::mutex> lock(mu);
  if (!done[device]) {
    done[device] = true;
    ok[device] = cudaFuncSetAttribute(bulk_gather_push_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBulkSmemBytes) == cudaSuccess &&
                 cudaFuncSetAttribute(bulk_pull_copy_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBulkSmemBytes) == cudaSuccess;
  }
  return ok[device];
}

int reduce_path(const PeerTable &t) { return t.mc ? kPathSwitch : (t.size == 2 ? kPathPair : kPathPeers); }
#define CS_DISPATCH_REDUCE(LAUNCH, dtype, path)                 \
  do {                                                          \
    const int path_ = (path);                                   \
    if ((dtype) == 0) {                                         \
      if (path_ == kPathSwitch) LAUNCH(0, kPathSwitch);         \
      else if (path_ == kPathPair) LAUNCH(0, kPathPair);        \
      else LAUNCH(0, kPathPeers);                               \
    } else {                                                    \
      if (path_ == kPathSwitch) LAUNCH(1, kPathSwitch);         \
      else if (path_ == kPathPair) LAUNCH(1, kPathPair);        \
      else LAUNCH(1, kPathPeers);                               \
    }                                                           \
  } while (0)

// Small messages get proportionally fewer blocks than the cap.
int comm_grid(int64_t vecs_per_rank) {
  const int cap = g_grid_cap.load();
  const int64_t per_block = static_cast<int64_t>(kThreads) * kUnroll;
  const int64_t blocks = (vecs_per_rank + per_block - 1) / per_block;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}
}  // namespace

void set_peer_wait_budget(long long cycles) { g_wait_budget.store(cycles); }
long long peer_wait_budget() { return g_wait_budget.load(); }
void set_collective_grid_cap(int blocks) { g_grid_cap.store(blocks < 1 ? 1 : (blocks > 1024 ? 1024 : blocks)); }
int collective_grid_cap() { return g_grid_cap.load(); }
void set_multicast_min_ranks(int ranks) { g_multicast_min_ranks.store(ranks < 2 ? 2 : ranks); }
int multicast_min_ranks() { return g_multicast_min_ranks.load(); }

int symm_barrier(stream_t stream, const PeerTable &t, int slot_base, uint32_t epoch, DeviceStatus *status) {
  barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(t, slot_base, epoch, g_wait_budget.load(), status);
  return finish_launch(1);
}

int symm_all_reduce(stream_t stream, const PeerTable &t, const Handshake &h, int64_t offset_bytes, int64_t count, int dtype,
                    float scale, int *blocks) {
  const int64_t bytes = count * (dtype == 0 ? 4 : 2);
  if (bytes % 16 != 0 || offset_bytes % 16 != 0) return static_cast<int>(cudaErrorInvalidValue);
  const int64_t vecs = bytes / 16;
  const int grid = comm_grid((vecs + t.size - 1) / t.size);
  *blocks = grid;
  auto s = static_cast<cudaStream_t>(stream);
#define CS_LAUNCH_ALL_REDUCE(DTYPE, PATH) all_reduce_kernel<DTYPE, PATH><<<grid, kThreads, 0, s>>>(t, h, offset_bytes, vecs, scale)
  CS_DISPATCH_REDUCE(CS_LAUNCH_ALL_REDUCE, dtype, reduce_path(t));
#undef CS_LAUNCH_ALL_REDUCE
  return finish_launch(1);
}

int symm_reduce_scatter(stream_t stream, const PeerTable &t, const Handshake &h, int64_t src_offset_bytes, void *dst, int64_t count,
                        int dtype, float scale, int *blocks, const void *residual) {
  const int64_t bytes = count * (dtype == 0 ? 4 : 2);
  if (bytes % 16 != 0 || src_offset_bytes % 16 != 0 || ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(residual)) & 15) ||
      (residual && dtype != 1))
    return static_cast<int>(cudaErrorInvalidValue);
  const int64_t vecs = bytes / 16;
  const int grid = comm_grid(vecs);
  *blocks = grid;
  auto s = static_cast<cudaStream_t>(stream);
#define CS_LAUNCH_REDUCE_SCATTER(DTYPE, PATH)                                                                                    \
  reduce_scatter_kernel<DTYPE, PATH><<<grid, kThreads, 0, s>>>(t, h, src_offset_bytes, static_cast<char *>(dst),                  \
                                                               DTYPE == 1 ? static_cast<const char *>(residual) : nullptr, vecs, scale)
  CS_DISPATCH_REDUCE(CS_LAUNCH_REDUCE_SCATTER, dtype, reduce_path(t));
#undef CS_LAUNCH_REDUCE_SCATTER
  return finish_launch(1);
}

int symm_all_gather_push(stream_t stream, const PeerTable &t, const Handshake &h, const void *src, int64_t dst_offset_bytes,
                         int64_t bytes, int *blocks) {
  if (bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(src) & 15) || dst_offset_bytes % 16 != 0) return static_cast<int>(cudaErrorInvalidValue);
  if (bytes >= kBulkMinBytes && bulk_engine_ready()) {
    const int64_t pieces = (bytes + kBulkStageBytes - 1) / kBulkStageBytes;
    const int cap = bulk_grid_cap();
    const int grid = static_cast<int>(pieces > cap ? cap : pieces);
    *blocks = grid;
    bulk_gather_push_kernel<<<grid, kBulkThreads, kBulkSmemBytes, static_cast<cudaStream_t>(stream)>>>(t, h, static_cast<const char *>(src),
                                                                                                       dst_offset_bytes, bytes);
    return finish_launch(1);
  }
  const int64_t vecs = bytes / 16;
  const int grid = comm_grid(vecs);
  *blocks = grid;
  all_gather_push_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(t, h, static_cast<const char *>(src), dst_offset_bytes, vecs);
  return finish_launch(1);
}

int symm_all_gather_chunked(stream_t stream, const PeerTable &t, const Handshake &h, const void *src, int64_t dst_offset_bytes,
                            int64_t bytes, int chunks, int *blocks) {
  if (chunks < 1 || chunks > kMaxChunks || bytes % (16 * chunks) != 0 || (reinterpret_cast<uintptr_t>(src) & 15) || dst_offset_bytes % 16 != 0)
    return static_cast<int>(cudaErrorInvalidValue);
  const int64_t vecs_per_chunk = bytes / 16 / chunks;
  const int64_t wanted = (vecs_per_chunk + 1024 * kUnroll - 1) / (1024 * kUnroll);
  const int grid = static_cast<int>(wanted < 1 ? 1 : (wanted > kGatherBesideGemmBlocks ? kGatherBesideGemmBlocks : wanted));
  *blocks = grid;
  all_gather_chunked_kernel<<<grid, 1024, 0, static_cast<cudaStream_t>(stream)>>>(t, h, static_cast<const char *>(src), dst_offset_bytes,
                                                                                      vecs_per_chunk, chunks);
  return finish_launch(1);
}

int symm_slot_sum(stream_t stream, const PeerTable &t, const Handshake &h, const void *slots_base, int64_t slot_bytes, void *dst,
                  const void *residual, int64_t count) {
  if (count % 8 != 0 || slot_bytes % 16 != 0 ||
      ((reinterpret_cast<uintptr_t>(slots_base) | reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(residual)) & 15))
    return static_cast<int>(cudaErrorInvalidValue);
  const int64_t vecs = count / 8;
  // local reads at full memory bandwidth: more and fuller blocks than the link-bound kernels use
  const int64_t blocks = (vecs + kThreads - 1) / kThreads;
  const int grid = static_cast<int>(blocks < 1 ? 1 : (blocks > 1184 ? 1184 : blocks));
  slot_sum_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(t, h, static_cast<const char *>(slots_base), slot_bytes,
                                                                            static_cast<char *>(dst), static_cast<const char *>(residual), vecs);
  return finish_launch(1);
}

int symm_pull_copy(stream_t stream, const PeerTable &t, const Handshake &h, const PullCopyArgs &a, int *blocks) {
  if (a.row_bytes % 16 != 0 || a.src_stride % 16 != 0 || a.dst_stride % 16 != 0) return static_cast<int>(cudaErrorInvalidValue);
  for (int p = 0; p < t.size; ++p)
    if ((a.src_offset[p] % 16) != 0 || (reinterpret_cast<uintptr_t>(a.dst[p]) & 15)) return static_cast<int>(cudaErrorInvalidValue);
  if (a.row_bytes >= kBulkMinRowBytes && a.rows * a.row_bytes >= kBulkMinBytes && bulk_engine_ready()) {
    const int64_t pieces = a.rows * ((a.row_bytes + kBulkStageBytes - 1) / kBulkStageBytes);
    const int cap = bulk_grid_cap() / t.size > 4 ? bulk_grid_cap() / t.size : 4;  // blocks per peer
    const int per_peer = static_cast<int>(pieces > cap ? cap : pieces);
    *blocks = per_peer * t.size;
    bulk_pull_copy_kernel<<<per_peer * t.size, kBulkThreads, kBulkSmemBytes, static_cast<cudaStream_t>(stream)>>>(t, h, a, per_peer);
    return finish_launch(1);
  }
  const int64_t vecs = a.rows * (a.row_bytes / 16);
  const int64_t wanted = (vecs + 512 * 8 - 1) / (512 * 8);
  const int total = g_grid_cap.load();
  const int cap = total / t.size > 8 ? total / t.size : 8;  // blocks per peer
  const int per_peer = static_cast<int>(wanted < 1 ? 1 : (wanted > cap ? cap : wanted));
  *blocks = per_peer * t.size;
  pull_copy_kernel<<<per_peer * t.size, 512, 0, static_cast<cudaStream_t>(stream)>>>(t, h, a, per_peer);
  return finish_launch(1);
}

int symm_reduce_scatter_adamw_all_gather(stream_t stream, const PeerTable &t, const Handshake &h, const ShardedAdamWArgs &a,
                                         int *blocks) {
  if (a.block < 8 || (a.block & (a.block - 1)) != 0 || a.range_begin % 4 != 0 || a.range_end % 4 != 0 || a.range_end <= a.range_begin ||
      a.grad_offset_bytes % 16 != 0 || (a.lp_offset_bytes >= 0 && a.lp_offset_bytes % 16 != 0))
    return static_cast<int>(cudaErrorInvalidValue);
  const int64_t per_rank = (a.range_end - a.range_begin + t.size - 1) / t.size;
  const int grid = comm_grid(per_rank / 4 * kUnroll);  // one vector per thread and trip: more blocks per byte
  *blocks = grid;
  rs_adamw_ag_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(t, h, a);
  return finish_launch(1);
}
CS_DEFINE_BOUNDS_GETTER(bounds_report_collectives)
}  // namespace cs::kernels
