// SPDX-License-Identifier: Apache-2.0
// bf16 GEMM on the 5th-generation tensor cores (tcgen05) with fp32 accumulators in tensor
// memory (TMEM), operands staged in shared memory by TMA, and fused epilogues.
//
//   D[M,N] = A * B^T     kTN: A [M,K] and B [N,K] row-major (K contiguous)   forward
//                        kNT: A [K,M] and B [K,N] row-major (M/N contiguous) weight gradient
//                        kTM: A [M,K] row-major, B [K,N] row-major           input gradient (dY * W)
//
// Structure (one persistent CTA per SM, 320 threads):
//   warp 0      TMA producer: cp.async.bulk.tensor tiles -> 4-stage shared-memory ring
//   warp 1      allocates TMEM and issues tcgen05.mma (one elected lane); 128x256 fp32
//               accumulators, two of them (512 TMEM columns) so the epilogue of tile i overlaps
//               the main loop of tile i+1
//   warps 2-9   epilogue: tcgen05.ld the accumulator (each warp owns a 32-row lane quadrant
//               and a 128-column half), apply the fused op, store to global memory
// Shared-memory tiles use the 128-byte swizzle; the K-major operands of kTN are described to
// the MMA with SBO = 1024 B (8 rows x 128 B), the MN-major operands of kNT with LBO = 8192 B
// (next 64-element block) and SBO = 1024 B (next 8 k-rows).
// Every mbarrier wait is bounded: a wait that runs out raises an abort flag, the CTA drains,
// frees its TMEM and returns; the host sees DeviceStatus.code != 0.
//
// What it replaces in the reference project: the cuBLAS calls behind at::linear / at::matmul in
// src/compute/linear.cpp:178-207,245,286-296 and the cuDNN-frontend fused graphs of
// src/compute/gelu_linear_cudnn.cpp:123-311 (GELU+matmul, matmul+GELU', GELU+wgrad), plus the
// log_softmax pass of src/compute/cross_entropy.cpp:57-63 (folded into the classifier epilogue).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "api.h"
#include "bounds_check.h"
#include "gelu_math.h"
#include "collectives.h"

namespace cs::kernels {
namespace {
constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int EPI_WARPS = 8;
constexpr int THREADS = 64 + EPI_WARPS * 32;
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr long long kWaitBudgetCycles = 4000000000LL;  // ~2 s at 2 GHz

struct KParams {
  void *d;
  void *d2;
  const void *aux;
  const void *bias;
  float *stats;
  long long m, n, k, ldd, n_valid;
  int layout, epilogue;
  int m_tiles, n_tiles, splits, kb_total, kb_per_split;
  int atomic_out;     // fp32 output accumulated with red.global.add (split-K or accumulate mode)
  unsigned lbo_mn, sbo_mn, kstep_mn;  // MN-major descriptor parameters (bytes)
  int peer_mode;       // 0 none, 1 = A row blocks come from peers, 2 = D row blocks go to peers,
                       // 3 = A is local but arrives in row chunks announced by flags (all-gather in flight)
  int peer_rank, peer_count;
  int rows_per_peer;
  const uint32_t *ready_flags;  // peer_mode 3: word [owner * 8 + chunk] reaches ready_epoch when that chunk has landed
  uint32_t ready_epoch;
  int ready_chunks;             // chunks per owner (rows_per_peer / ready_chunks rows each, a multiple of 256)
  DeviceStatus *status;
};

struct PeerMaps {
  CUtensorMap m[8];
};

__device__ DeviceStatus g_gemm_status;

// ------------------------------------------------------------------------- PTX helpers ----
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
// Bounded wait: false when the budget ran out or another role already aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitBudgetCycles) {
      *abort_flag = 1;
      return false;
    }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tcgen05_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tcgen05_ld_32x32b_x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tcgen05_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (tcgen05): start address, leading/stride byte offsets in
// 16-byte units, descriptor version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((addr & 0x3FFFF) >> 4);
  desc |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  desc |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
  desc |= static_cast<uint64_t>(1) << 46;  // version
  desc |= static_cast<uint64_t>(2) << 61;  // SWIZZLE_128B
  return desc;
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&t);
}
__device__ __forceinline__ float2 unpack_bf16(uint32_t u) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&u));
}
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

struct TileCoord {
  int m0, n0, kb_begin, kb_end, n_tile;
};
__device__ __forceinline__ TileCoord tile_coord(const KParams &p, int tile) {
  const int mn = p.m_tiles * p.n_tiles;
  const int split = tile / mn;
  const int rem = tile - split * mn;
  const int n_tile = rem / p.m_tiles;
  const int m_tile = rem - n_tile * p.m_tiles;
  TileCoord c;
  c.m0 = m_tile * BM;
  c.n0 = n_tile * BN;
  c.n_tile = n_tile;
  c.kb_begin = split * p.kb_per_split;
  c.kb_end = min(p.kb_total, c.kb_begin + p.kb_per_split);
  return c;
}

// One warp's share of a finished accumulator tile: lane quadrant q (rows m0 + 32q .. +32) and
// column half `half` (128 of the 256 columns). tmem_acc is the TMEM address of the tile.
__device__ __forceinline__ void epilogue_tile(const KParams &p, int m0, int n0, int n_tile, uint32_t tmem_acc, int q,
                                              int half, int lane) {
  const long long row = m0 + q * 32 + lane;
  const bool row_ok = row < p.m;
  float run_max = -INFINITY, run_sum = 0.f;
#pragma unroll 1
  for (int ch = 0; ch < 4; ++ch) {
    const int col0 = half * 128 + ch * 32;
    uint32_t v[32];
    tcgen05_ld_32x32b_x32(tmem_acc + col0 + (static_cast<uint32_t>(q * 32) << 16), v);
    tcgen05_wait_ld();
    const long long gcol = n0 + col0;
    if (!row_ok || gcol >= p.n) continue;
    if (!CS_IN_BOUNDS(kKidGemmEpilogue, row * p.ldd + gcol, static_cast<long long>(p.m) * p.ldd)) continue;
    float f[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]);
    if (p.epilogue == kEpiStoreF32 || p.epilogue == kEpiAccumF32) {
      float *dst = static_cast<float *>(p.d) + row * p.ldd + gcol;
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        if (gcol + g * 4 + 4 > p.n) break;
        if (p.atomic_out) {
          asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + g * 4), "f"(f[4 * g]),
                       "f"(f[4 * g + 1]), "f"(f[4 * g + 2]), "f"(f[4 * g + 3])
                       : "memory");
        } else {
          float4 o = make_float4(f[4 * g], f[4 * g + 1], f[4 * g + 2], f[4 * g + 3]);
          if (p.epilogue == kEpiAccumF32) {
            const float4 old = *reinterpret_cast<const float4 *>(dst + g * 4);
            o.x += old.x;
            o.y += old.y;
            o.z += old.z;
            o.w += old.w;
          }
          *reinterpret_cast<float4 *>(dst + g * 4) = o;
        }
      }
      continue;
    }
    if (p.bias) {
      const uint4 *bp = reinterpret_cast<const uint4 *>(static_cast<const __nv_bfloat16 *>(p.bias) + gcol);
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        if (gcol + g * 8 + 8 > p.n) break;
        const uint4 b = __ldg(bp + g);
        const uint32_t w[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 t = unpack_bf16(w[i]);
          f[g * 8 + 2 * i] += t.x;
          f[g * 8 + 2 * i + 1] += t.y;
        }
      }
    }
    __nv_bfloat16 *dst = static_cast<__nv_bfloat16 *>(p.d) + row * p.ldd + gcol;
    if (p.epilogue == kEpiResidualBf16 || p.epilogue == kEpiDGelu) {
      const uint4 *ap = reinterpret_cast<const uint4 *>(static_cast<const __nv_bfloat16 *>(p.aux) + row * p.ldd + gcol);
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        if (gcol + g * 8 + 8 > p.n) break;
        const uint4 a = *(ap + g);
        const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 t = unpack_bf16(w[i]);
          if (p.epilogue == kEpiResidualBf16) {
            f[g * 8 + 2 * i] += t.x;
            f[g * 8 + 2 * i + 1] += t.y;
          } else {
            f[g * 8 + 2 * i] *= gelu_grad_f(t.x);
            f[g * 8 + 2 * i + 1] *= gelu_grad_f(t.y);
          }
        }
      }
    }
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      if (gcol + g * 8 + 8 > p.n) break;
      uint4 o;
      o.x = pack_bf16(f[g * 8 + 0], f[g * 8 + 1]);
      o.y = pack_bf16(f[g * 8 + 2], f[g * 8 + 3]);
      o.z = pack_bf16(f[g * 8 + 4], f[g * 8 + 5]);
      o.w = pack_bf16(f[g * 8 + 6], f[g * 8 + 7]);
      *reinterpret_cast<uint4 *>(dst + g * 8) = o;
    }
    if (p.epilogue == kEpiGeluDual) {
      __nv_bfloat16 *dst2 = static_cast<__nv_bfloat16 *>(p.d2) + row * p.ldd + gcol;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        if (gcol + g * 8 + 8 > p.n) break;
        uint4 o;
        // GELU of the value as stored (bf16-rounded), so that backward sees the same input
        o.x = pack_bf16(gelu_f(bf16_round(f[g * 8 + 0])), gelu_f(bf16_round(f[g * 8 + 1])));
        o.y = pack_bf16(gelu_f(bf16_round(f[g * 8 + 2])), gelu_f(bf16_round(f[g * 8 + 3])));
        o.z = pack_bf16(gelu_f(bf16_round(f[g * 8 + 4])), gelu_f(bf16_round(f[g * 8 + 5])));
        o.w = pack_bf16(gelu_f(bf16_round(f[g * 8 + 6])), gelu_f(bf16_round(f[g * 8 + 7])));
        *reinterpret_cast<uint4 *>(dst2 + g * 8) = o;
      }
    }
    if (p.epilogue == kEpiCrossEntropy) {
      // running (max, sum-exp) over the valid columns, on the bf16-rounded logits
      float cmax = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        f[i] = bf16_round(f[i]);
        if (gcol + i < p.n_valid) cmax = fmaxf(cmax, f[i]);
      }
      if (cmax > -INFINITY) {
        const float new_max = fmaxf(run_max, cmax);
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (gcol + i < p.n_valid) s += __expf(f[i] - new_max);
        run_sum = run_sum * __expf(run_max - new_max) + s;
        run_max = new_max;
      }
    }
  }
  if (p.epilogue == kEpiCrossEntropy && row_ok) {
    float *st = p.stats + (row * (2LL * p.n_tiles) + 2LL * n_tile + half) * 2;
    st[0] = run_max;
    st[1] = run_sum;
  }
}

// ------------------------------------------------------------------------------ kernel ----
__global__ void __launch_bounds__(THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const KParams p) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the 128-byte swizzle pattern is a function of the absolute address.
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem_aligned + STAGES * STAGE_BYTES);
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  // barrier slots: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tmem_full_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto tmem_empty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(bars + 2 * STAGES + 4);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(bars + 2 * STAGES + 5);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_tiles = p.m_tiles * p.n_tiles * p.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tmem_full_bar(b), 1);
      mbar_init(tmem_empty_bar(b), EPI_WARPS);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_b)) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(const_cast<uint32_t *>(tmem_slot))),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer ----
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const TileCoord c = tile_coord(p, tile);
        for (int kb = c.kb_begin; kb < c.kb_end; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t a_dst = smem_base + stage * STAGE_BYTES;
          const uint32_t b_dst = a_dst + A_BYTES;
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          // K-major operands: one box; MN-major operands: 64-element (128-byte) wide boxes of
          // 64 k-rows, 8 KB each
          if (p.layout == kNT) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(a_dst + j * 8192, &map_a, full_bar(stage), c.m0 + j * 64, kb * BK);
          } else {
            tma_load_2d(a_dst, &map_a, full_bar(stage), kb * BK, c.m0);
          }
          if (p.layout == kTN) {
            tma_load_2d(b_dst, &map_b, full_bar(stage), kb * BK, c.n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * 8192, &map_b, full_bar(stage), c.n0 + j * 64, kb * BK);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // Abort path: give loads that are still in flight a bounded chance to land before the
        // shared memory goes away.
        for (int s = 0; s < STAGES; ++s) {
          const long long t0 = clock64();
          while (!mbar_try_wait(full_bar(s), 0) && !mbar_try_wait(full_bar(s), 1) && clock64() - t0 < 2000000LL) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------------- MMA issuer ----
    if (lane == 0) {
      const uint32_t a_major = p.layout == kNT ? 1u : 0u;
      const uint32_t b_major = p.layout == kTN ? 0u : 1u;
      const uint32_t idesc = (1u << 4) /*fp32 accum*/ | (1u << 7) /*A bf16*/ | (1u << 10) /*B bf16*/ | (a_major << 15) |
                             (b_major << 16) | (static_cast<uint32_t>(BN >> 3) << 17) |
                             (static_cast<uint32_t>(BM >> 4) << 24);
      const uint32_t lbo_a = a_major ? p.lbo_mn : 16u, lbo_b = b_major ? p.lbo_mn : 16u;
      const uint32_t sbo_a = a_major ? p.sbo_mn : 1024u, sbo_b = b_major ? p.sbo_mn : 1024u;
      const uint32_t kstep_a = a_major ? p.kstep_mn : static_cast<uint32_t>(UMMA_K * 2);
      const uint32_t kstep_b = b_major ? p.kstep_mn : static_cast<uint32_t>(UMMA_K * 2);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const TileCoord c = tile_coord(p, tile);
        if (!mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1u, abort_flag)) break;
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = c.kb_begin; kb < c.kb_end; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const uint32_t a_src = smem_base + stage * STAGE_BYTES;
          const uint32_t b_src = a_src + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = make_smem_desc(a_src + k * kstep_a, lbo_a, sbo_a);
            const uint64_t db = make_smem_desc(b_src + k * kstep_b, lbo_b, sbo_b);
            tcgen05_mma(d_tmem, da, db, idesc, (kb > c.kb_begin || k > 0) ? 1u : 0u);
          }
          tcgen05_commit(empty_bar(stage));  // frees the stage once these MMAs retired
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        tcgen05_commit(tmem_full_bar(acc));
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else {
    // ---------------------------------------------------------------------- epilogue ----
    const int q = warp & 3;                 // TMEM lane quadrant this warp may access
    const int half = (warp - 2) >> 2;       // which 128 columns of the tile
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      const TileCoord c = tile_coord(p, tile);
      if (!mbar_wait(tmem_full_bar(acc), acc_phase, abort_flag)) break;
      tcgen05_fence_after();
      epilogue_tile(p, c.m0, c.n0, c.n_tile, tmem_base + acc * BN, q, half, lane);
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty_bar(acc));
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
  }

  // ------------------------------------------------------------------------- teardown ----
  tcgen05_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) {
    p.status->code = 1;
    p.status->kernel_id = 1;
    p.status->block = blockIdx.x;
    p.status->detail = p.layout;
  }
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}



// ----------------------------------------------------- epilogue through shared memory + TMA ----
// The accumulator rows a thread reads from TMEM are 64-byte pieces of different output rows;
// storing them directly makes every store instruction touch 32 half-filled sectors. Instead each
// epilogue warp stages 32 rows x 128 bytes in shared memory (128-byte swizzle, conflict-free
// for 16-byte accesses) and one lane issues a TMA store (or, for fp32 gradients, a TMA
// reduce-add) of that box: full 128-byte lines, bounds clipped by the tensor map.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(reinterpret_cast<uint64_t>(map)),
               "r"(src), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap *map, uint32_t src, int c0, int c1) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(src), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

constexpr int EPI_BUF_BYTES = 4096;  // 32 rows x 128 bytes
constexpr int EPI_STAGING_BYTES = EPI_WARPS * 2 * EPI_BUF_BYTES;

struct EpilogueStaging {
  uint32_t buf[2];  // shared-memory addresses of this warp's two staging boxes
  int next;         // which one the next fill uses
};

// Claims a staging box: the TMA operation that last read it (two fills ago) must have finished
// reading shared memory.
__device__ __forceinline__ uint32_t staging_acquire(EpilogueStaging &st, int lane, bool drain_all = false) {
  if (lane == 0) {
    if (drain_all)
      asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    else
      bulk_wait_read_1();
  }
  __syncwarp();
  const uint32_t b = st.buf[st.next];
  st.next ^= 1;
  return b;
}
// 16-byte piece `piece` (0..7) of row `lane` inside a swizzled 32 x 128-byte box.
__device__ __forceinline__ uint32_t staging_addr(uint32_t box, int lane, int piece) {
  return box + lane * 128 + ((piece ^ (lane & 7)) << 4);
}
// Makes the box visible to the async proxy and lets lane 0 issue the store / reduce.
__device__ __forceinline__ void staging_release(const CUtensorMap *map, uint32_t box, int c0, int c1, bool in_range, bool reduce,
                                                int lane) {
  fence_async_smem();
  __syncwarp();
  if (lane == 0) {
    if (in_range) {
      if (reduce)
        tma_reduce_add_2d(map, box, c0, c1);
      else
        tma_store_2d(map, box, c0, c1);
    }
    bulk_commit();  // an empty group keeps the acquire/commit pairing uniform
  }
}

// The 64 bytes of the auxiliary operand (residual / pre-activation) that belong to this thread's
// row in one 32-column chunk. Loaded one chunk ahead of its use so that the global-memory
// latency overlaps the TMEM read and the math of the previous chunk.
struct AuxChunk {
  uint4 v[4];
};
__device__ __forceinline__ AuxChunk load_aux_chunk(const KParams &p, long long row, bool row_ok, long long gcol) {
  AuxChunk a;
#pragma unroll
  for (int g = 0; g < 4; ++g) a.v[g] = make_uint4(0u, 0u, 0u, 0u);
  if (row_ok && gcol < p.n) {
    const uint4 *ap = reinterpret_cast<const uint4 *>(static_cast<const __nv_bfloat16 *>(p.aux) + row * p.ldd + gcol);
#pragma unroll
    for (int g = 0; g < 4; ++g)
      if (gcol + g * 8 + 8 <= p.n) a.v[g] = __ldg(ap + g);
  }
  return a;
}

__device__ __forceinline__ void epilogue_tile_tma(const KParams &p, const CUtensorMap *map_d, const CUtensorMap *map_d2, int m0,
                                                  int n0, int n_tile, uint32_t tmem_acc, int q, int half, int lane,
                                                  EpilogueStaging &st, int store_row_base, AuxChunk aux_next) {
  // store_row_base: first row of the destination tensor map inside the logical output (non-zero
  // when the rows are scattered to per-owner buffers)
  const int row0 = m0 + q * 32;
  const long long row = row0 + lane;
  const bool row_ok = row < p.m;
  const bool rows_in_range = row0 < p.m;
  float run_max = -INFINITY, run_sum = 0.f;
  const bool f32_out = p.epilogue == kEpiStoreF32 || p.epilogue == kEpiAccumF32;
  const bool reduce = f32_out && (p.atomic_out || p.epilogue == kEpiAccumF32);
  uint32_t box = 0, box2 = 0;
  const bool uses_aux = p.epilogue == kEpiResidualBf16 || p.epilogue == kEpiDGelu;
#pragma unroll 1
  for (int ch = 0; ch < 4; ++ch) {
    const int col0 = half * 128 + ch * 32;
    const AuxChunk aux = aux_next;
    if (uses_aux && ch < 3) aux_next = load_aux_chunk(p, row, row_ok, n0 + col0 + 32);
    uint32_t v[32];
    tcgen05_ld_32x32b_x32(tmem_acc + col0 + (static_cast<uint32_t>(q * 32) << 16), v);
    tcgen05_wait_ld();
    const long long gcol = n0 + col0;
    const bool cols_in_range = gcol < p.n;
    float f[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]);
    if (f32_out) {
      // one box per 32 fp32 columns
      box = staging_acquire(st, lane);
#pragma unroll
      for (int g = 0; g < 8; ++g)
        st_shared_v4(staging_addr(box, lane, g), v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
      staging_release(map_d, box, static_cast<int>(gcol), row0 - store_row_base, rows_in_range && cols_in_range, reduce, lane);
      continue;
    }
    if (p.bias && cols_in_range) {
      const uint4 *bp = reinterpret_cast<const uint4 *>(static_cast<const __nv_bfloat16 *>(p.bias) + gcol);
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        if (gcol + g * 8 + 8 > p.n) break;
        const uint4 b = __ldg(bp + g);
        const uint32_t w[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 t = unpack_bf16(w[i]);
          f[g * 8 + 2 * i] += t.x;
          f[g * 8 + 2 * i + 1] += t.y;
        }
      }
    }
    if (uses_aux && row_ok && cols_in_range) {
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        if (gcol + g * 8 + 8 > p.n) break;
        const uint4 a = aux.v[g];
        const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 t = unpack_bf16(w[i]);
          if (p.epilogue == kEpiResidualBf16) {
            f[g * 8 + 2 * i] += t.x;
            f[g * 8 + 2 * i + 1] += t.y;
          } else {
            f[g * 8 + 2 * i] *= gelu_grad_f(t.x);
            f[g * 8 + 2 * i + 1] *= gelu_grad_f(t.y);
          }
        }
      }
    }
    // two 32-column chunks share one 64-column (128-byte) box
    const int sub = ch & 1;
    if (sub == 0) {
      // the dual-output epilogue fills both boxes at once, so both previous stores must be done
      box = staging_acquire(st, lane, p.epilogue == kEpiGeluDual);
      if (p.epilogue == kEpiGeluDual) box2 = staging_acquire(st, lane, true);
    }
#pragma unroll
    for (int g = 0; g < 4; ++g)
      st_shared_v4(staging_addr(box, lane, sub * 4 + g), pack_bf16(f[g * 8 + 0], f[g * 8 + 1]), pack_bf16(f[g * 8 + 2], f[g * 8 + 3]),
                   pack_bf16(f[g * 8 + 4], f[g * 8 + 5]), pack_bf16(f[g * 8 + 6], f[g * 8 + 7]));
    if (p.epilogue == kEpiGeluDual) {
#pragma unroll
      for (int g = 0; g < 4; ++g)
        st_shared_v4(staging_addr(box2, lane, sub * 4 + g), pack_bf16(gelu_f(f[g * 8 + 0]), gelu_f(f[g * 8 + 1])),
                     pack_bf16(gelu_f(f[g * 8 + 2]), gelu_f(f[g * 8 + 3])), pack_bf16(gelu_f(f[g * 8 + 4]), gelu_f(f[g * 8 + 5])),
                     pack_bf16(gelu_f(f[g * 8 + 6]), gelu_f(f[g * 8 + 7])));
    }
    if (p.epilogue == kEpiCrossEntropy && row_ok && cols_in_range) {
      float cmax = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        f[i] = bf16_round(f[i]);
        if (gcol + i < p.n_valid) cmax = fmaxf(cmax, f[i]);
      }
      if (cmax > -INFINITY) {
        const float new_max = fmaxf(run_max, cmax);
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (gcol + i < p.n_valid) s += __expf(f[i] - new_max);
        run_sum = run_sum * __expf(run_max - new_max) + s;
        run_max = new_max;
      }
    }
    if (sub == 1) {
      const int c0 = n0 + half * 128 + (ch - 1) * 32;
      const bool in_range = rows_in_range && c0 < p.n;
      staging_release(map_d, box, c0, row0 - store_row_base, in_range, false, lane);
      if (p.epilogue == kEpiGeluDual) staging_release(map_d2, box2, c0, row0 - store_row_base, in_range, false, lane);
    }
  }
  if (p.epilogue == kEpiCrossEntropy && row_ok) {
    float *stp = p.stats + (row * (2LL * p.n_tiles) + 2LL * n_tile + half) * 2;
    stp[0] = run_max;
    stp[1] = run_sum;
  }
}

// ===================================================================================
// 2-CTA variant: a thread-block cluster of two CTAs on neighbouring SMs computes one 256x256
// tile with tcgen05.mma.cta_group::2. CTA r of the pair loads rows [128r, 128r+128) of the A
// tile and rows [128r, 128r+128) of the B tile (plain TMA loads, no multicast), so every CTA
// moves 32 KB per 256x256x64 block instead of 48 KB per 128x256x64 block: one third less
// L2-to-shared-memory traffic per FLOP, which is what bounds the 1-CTA kernel.
// The leader CTA (cluster rank 0) issues the MMAs for the pair; barriers:
//   full[s]       in the leader: the leader's producer arrives with the byte count of both
//                 CTAs, both CTAs' TMA loads complete on it
//   empty[s]      in each CTA: tcgen05.commit multicasts the arrival to both
//   tmem_full[b]  in each CTA (multicast commit); tmem_empty[b] in the leader, counted by the
//                 epilogue warps of both CTAs
// ===================================================================================
constexpr int STAGES2 = 5;
constexpr int B2_BYTES = 128 * BK * 2;               // this CTA's half of the B tile
constexpr int STAGE2_BYTES = A_BYTES + B2_BYTES;     // 32 KB
constexpr int SMEM2_BYTES = STAGES2 * STAGE2_BYTES + EPI_STAGING_BYTES + 1024 + 256;
constexpr int BM2 = 256;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t cta) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(cta));
  return out;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar_cluster_addr, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tcgen05_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"(mask)
               : "memory");
}
__device__ __forceinline__ void tcgen05_mma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ TileCoord tile_coord2(const KParams &p, int tile) {
  const int mn = p.m_tiles * p.n_tiles;
  const int split = tile / mn;
  const int rem = tile - split * mn;
  int n_tile = rem / p.m_tiles;
  int m_tile = rem - n_tile * p.m_tiles;
  if (p.peer_mode == 3) {
    // Rows arrive chunk by chunk from every owner at once: walk the row tiles in arrival order (chunk 0 of every
    // owner starting with this rank, then chunk 1, ...) and finish all column tiles of a row tile before the next.
    const int order = rem / p.n_tiles;
    n_tile = rem - order * p.n_tiles;
    const int per_peer = p.rows_per_peer / BM2;
    const int per_chunk = per_peer / p.ready_chunks;
    const int chunk = order / (p.peer_count * per_chunk);
    const int within = order - chunk * (p.peer_count * per_chunk);
    const int owner = (within / per_chunk + p.peer_rank) % p.peer_count;
    m_tile = owner * per_peer + chunk * per_chunk + (within % per_chunk);
  } else if (p.peer_mode) {
    // walk the owners' blocks in ring order so that no two ranks hammer the same peer: gathering starts with the
    // rows this rank owns (local data is consumed while remote traffic ramps up), scattering with the next rank's
    // rows (remote traffic starts at once, the local block comes last)
    const int per_peer = p.rows_per_peer / BM2;
    m_tile = (m_tile + (p.peer_rank + (p.peer_mode == 2 ? 1 : 0)) * per_peer) % p.m_tiles;
  }
  TileCoord c;
  c.m0 = m_tile * BM2;
  c.n0 = n_tile * BN;
  c.n_tile = n_tile;
  c.kb_begin = split * p.kb_per_split;
  c.kb_end = min(p.kb_total, c.kb_begin + p.kb_per_split);
  return c;
}

// 128 registers per thread (no spills): the SM's four register files are filled by warps, and a partition that
// holds three of this block's ten warps then still has room for two warps of a light kernel (collectives, AdamW),
// so those really run beside a resident GEMM block instead of waiting for it to retire.
__global__ void __maxnreg__(128)
gemm2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
             const __grid_constant__ CUtensorMap map_d, const __grid_constant__ CUtensorMap map_d2,
             const __grid_constant__ PeerMaps peer_maps, const KParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t staging_base = smem_base + STAGES2 * STAGE2_BYTES;
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem_aligned + STAGES2 * STAGE2_BYTES + EPI_STAGING_BYTES);
  const uint32_t bar_base = staging_base + EPI_STAGING_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES2 + s); };
  auto tmem_full_bar = [&](int b) { return bar_base + 8u * (2 * STAGES2 + b); };
  auto tmem_empty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES2 + 2 + b); };
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(bars + 2 * STAGES2 + 4);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(bars + 2 * STAGES2 + 5);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();
  const bool leader = cta == 0;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int total_tiles = p.m_tiles * p.n_tiles * p.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES2; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tmem_full_bar(b), 1);
      mbar_init(tmem_empty_bar(b), 2 * EPI_WARPS);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_b)) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(const_cast<uint32_t *>(tmem_slot))),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anyone signals across the pair
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------- TMA producer (one per CTA) ----
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int ready_key = -1;
      for (int tile = pair; ok && tile < total_tiles; tile += num_pairs) {
        const TileCoord c = tile_coord2(p, tile);
        const int m0 = c.m0 + static_cast<int>(cta) * 128;   // this CTA's rows of A / D
        const int nb0 = c.n0 + static_cast<int>(cta) * 128;  // this CTA's rows of the B tile
        if (p.peer_mode == 3) {
          // the rows of this tile are written by the all-gather that runs beside this kernel: wait for their chunk
          const int owner = c.m0 / p.rows_per_peer;
          const int chunk = (c.m0 - owner * p.rows_per_peer) / (p.rows_per_peer / p.ready_chunks);
          const int key = owner * 8 + chunk;
          if (key != ready_key) {
            const uint32_t *flag = p.ready_flags + key;
            const long long t0 = clock64();
            for (;;) {
              uint32_t seen;
              asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
              if (static_cast<int32_t>(seen - p.ready_epoch) >= 0) break;
              if (*abort_flag || clock64() - t0 > kWaitBudgetCycles) {
                *abort_flag = 1;
                ok = false;
                break;
              }
              __nanosleep(100);
            }
            if (!ok) break;
            // the chunk was written by other GPUs through the generic proxy; the loads below go through the async proxy
            asm volatile("fence.proxy.async.global;" ::: "memory");
            ready_key = key;
          }
        }
        for (int kb = c.kb_begin; kb < c.kb_end; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t a_dst = smem_base + stage * STAGE2_BYTES;
          const uint32_t b_dst = a_dst + A_BYTES;
          const uint32_t full_leader = mapa_shared(full_bar(stage), 0);
          if (leader) mbar_expect_tx(full_bar(stage), 2 * STAGE2_BYTES);
          if (p.layout == kNT) {
#pragma unroll
            for (int j = 0; j < 2; ++j) tma_load_2d_pair(a_dst + j * 8192, &map_a, full_leader, m0 + j * 64, kb * BK);
          } else if (p.peer_mode == 1) {
            // all-gather fused into the load: this tile's rows live in their owner's memory
            const int owner = m0 / p.rows_per_peer;
            tma_load_2d_pair(a_dst, &peer_maps.m[owner], full_leader, kb * BK, m0 - owner * p.rows_per_peer);
          } else {
            tma_load_2d_pair(a_dst, &map_a, full_leader, kb * BK, m0);
          }
          if (p.layout == kTN) {
            tma_load_2d_pair(b_dst, &map_b, full_leader, kb * BK, nb0);
          } else {
#pragma unroll
            for (int j = 0; j < 2; ++j) tma_load_2d_pair(b_dst + j * 8192, &map_b, full_leader, nb0 + j * 64, kb * BK);
          }
          if (++stage == STAGES2) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer (leader CTA only) ----
    if (lane == 0 && leader) {
      const uint32_t a_major = p.layout == kNT ? 1u : 0u;
      const uint32_t b_major = p.layout == kTN ? 0u : 1u;
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (a_major << 15) | (b_major << 16) |
                             (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(BM2 >> 4) << 24);
      const uint32_t lbo_a = a_major ? p.lbo_mn : 16u, lbo_b = b_major ? p.lbo_mn : 16u;
      const uint32_t sbo_a = a_major ? p.sbo_mn : 1024u, sbo_b = b_major ? p.sbo_mn : 1024u;
      const uint32_t kstep_a = a_major ? p.kstep_mn : static_cast<uint32_t>(UMMA_K * 2);
      const uint32_t kstep_b = b_major ? p.kstep_mn : static_cast<uint32_t>(UMMA_K * 2);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < total_tiles; tile += num_pairs) {
        const TileCoord c = tile_coord2(p, tile);
        if (!mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1u, abort_flag)) break;
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = c.kb_begin; kb < c.kb_end; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const uint32_t a_src = smem_base + stage * STAGE2_BYTES;
          const uint32_t b_src = a_src + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = make_smem_desc(a_src + k * kstep_a, lbo_a, sbo_a);
            const uint64_t db = make_smem_desc(b_src + k * kstep_b, lbo_b, sbo_b);
            tcgen05_mma_pair(d_tmem, da, db, idesc, (kb > c.kb_begin || k > 0) ? 1u : 0u);
          }
          tcgen05_commit_pair(empty_bar(stage));
          if (++stage == STAGES2) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        tcgen05_commit_pair(tmem_full_bar(acc));
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else {
    // ------------------------------------------------------- epilogue (each CTA) ----
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    int acc = 0;
    uint32_t acc_phase = 0;
    EpilogueStaging st;
    st.buf[0] = staging_base + (warp - 2) * 2 * EPI_BUF_BYTES;
    st.buf[1] = st.buf[0] + EPI_BUF_BYTES;
    st.next = 0;
    for (int tile = pair; tile < total_tiles; tile += num_pairs) {
      const TileCoord c = tile_coord2(p, tile);
      const int m0_cta = c.m0 + static_cast<int>(cta) * 128;
      // first chunk of the auxiliary operand is requested before waiting for the accumulator
      AuxChunk aux0{};
      if (p.epilogue == kEpiResidualBf16 || p.epilogue == kEpiDGelu) {
        const long long r = m0_cta + q * 32 + lane;
        aux0 = load_aux_chunk(p, r, r < p.m, c.n0 + half * 128);
      }
      if (!mbar_wait(tmem_full_bar(acc), acc_phase, abort_flag)) break;
      tcgen05_fence_after();
      if (p.peer_mode == 2) {
        // reduce-scatter fused into the epilogue: add this tile into its owner's accumulator
        const int owner = m0_cta / p.rows_per_peer;
        epilogue_tile_tma(p, &peer_maps.m[owner], &map_d2, m0_cta, c.n0, c.n_tile, tmem_base + acc * BN, q, half, lane, st,
                          owner * p.rows_per_peer, aux0);
      } else {
        epilogue_tile_tma(p, &map_d, &map_d2, m0_cta, c.n0, c.n_tile, tmem_base + acc * BN, q, half, lane, st, 0, aux0);
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(tmem_empty_bar(acc), 0));
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    if (lane == 0) bulk_wait_all();  // this warp's stores have left shared memory and are complete
  }

  // ------------------------------------------------------------------------- teardown ----
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer may still be signalling our barriers or reading our shared memory
  if (threadIdx.x == 0 && *abort_flag) {
    p.status->code = 1;
    p.status->kernel_id = 2;
    p.status->block = blockIdx.x;
    p.status->detail = p.layout;
  }
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------ host: tensor maps ----
using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                              const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess) {
      (void)cudaGetLastError();
      return static_cast<EncodeFn>(nullptr);
    }
    return reinterpret_cast<EncodeFn>(ptr);
  }();
  return fn;
}

struct MapKey {
  const void *ptr;
  uint64_t inner, outer, stride_bytes;
  uint32_t box_inner, box_outer;
  int elem_bytes;
  bool operator==(const MapKey &o) const {
    return ptr == o.ptr && inner == o.inner && outer == o.outer && stride_bytes == o.stride_bytes &&
           box_inner == o.box_inner && box_outer == o.box_outer && elem_bytes == o.elem_bytes;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey &k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    auto mix = [&h](uint64_t v) { h ^= v + 0x9e3779b97f4a7c15ULL + (h << 6) + (h >> 2); };
    mix(k.inner);
    mix(k.outer);
    mix(k.stride_bytes);
    mix((static_cast<uint64_t>(k.box_inner) << 32) | k.box_outer);
    return h;
  }
};

// 2-D bf16 tensor map: `inner` contiguous elements per row, `outer` rows, row stride in
// elements; box = box_inner x box_outer with the 128-byte swizzle (box_inner == 64).
bool get_tensor_map(const void *ptr, uint64_t inner, uint64_t outer, uint64_t stride_elems, uint32_t box_inner,
                    uint32_t box_outer, CUtensorMap *out, int elem_bytes = 2) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{ptr, inner, outer, stride_elems * elem_bytes, box_inner, box_outer, elem_bytes};
  std::lock_guard<std::mutex> lock{mu};
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return true;
  }
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {stride_elems * elem_bytes};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t elem_strides[2] = {1, 1};
  CUtensorMap map;
  const CUresult r = fn(&map, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(ptr), dims, strides, box, elem_strides,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, map);
  *out = map;
  return true;
}

}  // namespace

int64_t gemm_ce_stat_tiles(int64_t n) { return 2 * ((n + BN - 1) / BN); }  // one (max, sum) pair per 128-column half tile

int gemm_status(DeviceStatus *out) {
  return static_cast<int>(cudaMemcpyFromSymbol(out, g_gemm_status, sizeof(DeviceStatus)));
}
int gemm_status_reset() {
  DeviceStatus zero{};
  return static_cast<int>(cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(DeviceStatus)));
}

int gemm_bf16(stream_t stream, const GemmArgs &a) {
  auto s = static_cast<cudaStream_t>(stream);
  if (a.m <= 0 || a.n <= 0 || a.k <= 0) return -1;
  if (a.n % 8 != 0 || a.ldd % 8 != 0 || a.lda % 8 != 0 || a.ldb % 8 != 0) return -1;
  if ((reinterpret_cast<uintptr_t>(a.a) | reinterpret_cast<uintptr_t>(a.b) | reinterpret_cast<uintptr_t>(a.d)) & 15) return -1;
  if (!a.b || (!a.a && !(a.peer_count > 1 && a.a_peers[0])) || (!a.d && !(a.peer_count > 1 && a.d_peers[0]))) return -1;
  if (a.aux && (reinterpret_cast<uintptr_t>(a.aux) & 15)) return -1;
  if (a.d2 && (reinterpret_cast<uintptr_t>(a.d2) & 15)) return -1;
  if (a.bias && (reinterpret_cast<uintptr_t>(a.bias) & 15)) return -1;
  const bool f32_out = a.epilogue == kEpiStoreF32 || a.epilogue == kEpiAccumF32;
  if (a.layout != kNT && a.k % 8 != 0) return -1;
  if (a.layout < 0 || a.layout > kTM) return -1;
  if (a.layout == kNT && (a.m % 8 != 0)) return -1;
  if (f32_out && a.n % 4 != 0) return -1;
  if (a.m > 0x7fffffffLL || a.n > 0x7fffffffLL || a.k > 0x7fffffffLL) return -1;
  static const bool disabled = std::getenv("CS_DISABLE_TCGEN05_GEMM") != nullptr;
  if (disabled) return -1;

  static const bool one_cta_only = std::getenv("CS_GEMM_1CTA") != nullptr;
  const bool pair_kernel = !one_cta_only && a.m > 128;  // a single 128-row tile gains nothing from pairing
  const int tile_m = pair_kernel ? BM2 : BM;
  const uint32_t b_box_rows = pair_kernel ? 128u : static_cast<uint32_t>(BN);
  PeerMaps peer_maps{};
  int peer_mode = 0;
  int rows_per_peer = 0;
  if (a.peer_count > 1) {
    if (!pair_kernel || a.peer_count > 8 || a.m % a.peer_count != 0) return -1;
    rows_per_peer = static_cast<int>(a.m / a.peer_count);
    if (rows_per_peer % BM2 != 0) return -1;
    if (a.a_peers[0]) {
      if (a.layout == kNT) return -1;
      peer_mode = 1;
      for (int j = 0; j < a.peer_count; ++j)
        if (!a.a_peers[j] || (reinterpret_cast<uintptr_t>(a.a_peers[j]) & 15) ||
            !get_tensor_map(a.a_peers[j], a.k, rows_per_peer, a.lda, BK, BM, &peer_maps.m[j]))
          return -1;
    } else if (a.d_peers[0]) {
      if (a.epilogue != kEpiAccumF32 && a.epilogue != kEpiStoreBf16) return -1;
      peer_mode = 2;
      const bool f32 = a.epilogue == kEpiAccumF32;
      for (int j = 0; j < a.peer_count; ++j)
        if (!a.d_peers[j] || (reinterpret_cast<uintptr_t>(a.d_peers[j]) & 15) ||
            !get_tensor_map(a.d_peers[j], a.n, rows_per_peer, a.ldd, f32 ? 32 : 64, 32, &peer_maps.m[j], f32 ? 4 : 2))
          return -1;
    } else if (a.ready_flags) {
      if (a.layout == kNT || a.ready_chunks < 1 || a.ready_chunks > 8 || rows_per_peer % (BM2 * a.ready_chunks) != 0) return -1;
      peer_mode = 3;
    }
  }
  CUtensorMap map_a, map_b;
  if (peer_mode == 1) {
    map_a = peer_maps.m[0];
  } else if (a.layout == kNT) {
    if (!get_tensor_map(a.a, a.m, a.k, a.lda, 64, BK, &map_a)) return -1;
  } else {
    if (!get_tensor_map(a.a, a.k, a.m, a.lda, BK, BM, &map_a)) return -1;
  }
  if (a.layout == kTN) {
    if (!get_tensor_map(a.b, a.k, a.n, a.ldb, BK, b_box_rows, &map_b)) return -1;
  } else {
    if (!get_tensor_map(a.b, a.n, a.k, a.ldb, 64, BK, &map_b)) return -1;
  }
  CUtensorMap map_d{}, map_d2{};
  if (pair_kernel) {
    // output boxes of the TMA-store epilogue: 32 rows x 128 bytes
    if (peer_mode == 2) {
      map_d = peer_maps.m[0];
    } else if (f32_out) {
      if (!get_tensor_map(a.d, a.n, a.m, a.ldd, 32, 32, &map_d, 4)) return -1;
    } else {
      if (!get_tensor_map(a.d, a.n, a.m, a.ldd, 64, 32, &map_d)) return -1;
    }
    map_d2 = map_d;
    if (a.d2 && !get_tensor_map(a.d2, a.n, a.m, a.ldd, 64, 32, &map_d2)) return -1;
  }

  KParams p{};
  p.d = a.d;
  p.d2 = a.d2;
  p.aux = a.aux;
  p.bias = a.bias;
  p.stats = a.stats;
  p.m = a.m;
  p.n = a.n;
  p.k = a.k;
  p.ldd = a.ldd;
  p.n_valid = a.n_valid > 0 ? a.n_valid : a.n;
  p.layout = a.layout;
  p.epilogue = a.epilogue;
  p.m_tiles = static_cast<int>((a.m + tile_m - 1) / tile_m);
  p.n_tiles = static_cast<int>((a.n + BN - 1) / BN);
  p.kb_total = static_cast<int>((a.k + BK - 1) / BK);
  p.splits = 1;
  static const int sm_count = [] {
    int dev = 0, n = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n;
  }();
  if (f32_out) {
    // Weight gradients have few output tiles and a long reduction: split K so that every SM
    // has work; partial sums meet in the fp32 output through vector atomics.
    const int mn = p.m_tiles * p.n_tiles;
    const int workers = pair_kernel ? sm_count / 2 : sm_count;
    // Pick the split count whose tile total fills whole waves of `workers` best, keeping at
    // least 8 k-blocks per split; ties go to fewer splits (fewer reduce-adds).
    const int max_splits = p.kb_total / 8 > 0 ? p.kb_total / 8 : 1;
    int best = 1;
    double best_eff = 0.0;
    for (int sp = 1; sp <= max_splits && sp <= 64; ++sp) {
      const int tiles = mn * sp;
      const int waves = (tiles + workers - 1) / workers;
      const double eff = static_cast<double>(tiles) / (static_cast<double>(waves) * workers);
      if (eff > best_eff + 0.02) {
        best_eff = eff;
        best = sp;
      }
      if (tiles >= 4 * workers) break;
    }
    p.splits = best;
  }
  p.kb_per_split = (p.kb_total + p.splits - 1) / p.splits;
  p.splits = (p.kb_total + p.kb_per_split - 1) / p.kb_per_split;
  p.atomic_out = 0;
  if (f32_out && p.splits > 1) {
    p.atomic_out = 1;
    if (a.epilogue == kEpiStoreF32) {
      // every split adds into a zeroed output
      const cudaError_t e = cudaMemset2DAsync(a.d, static_cast<size_t>(a.ldd) * 4, 0, static_cast<size_t>(a.n) * 4,
                                              static_cast<size_t>(a.m), s);
      if (e != cudaSuccess) return static_cast<int>(e);
    }
  }
  p.peer_mode = peer_mode;
  p.peer_rank = a.peer_rank;
  p.peer_count = a.peer_count;
  p.rows_per_peer = rows_per_peer;
  if (peer_mode == 2) {
    p.splits = 1;  // the cross-rank sum happens in (or after) the destination
    p.kb_per_split = p.kb_total;
    p.atomic_out = f32_out ? 1 : 0;
  }
  p.ready_flags = a.ready_flags;
  p.ready_epoch = a.ready_epoch;
  p.ready_chunks = a.ready_chunks;
  // MN-major operand descriptors: next 64-element block 8192 B on, next 8 k-rows 1024 B on, one UMMA_K step = 16 k-rows
  p.lbo_mn = 8192;
  p.sbo_mn = 1024;
  p.kstep_mn = 2048;
  static DeviceStatus *status_ptr = [] {
    void *ptr = nullptr;
    cudaGetSymbolAddress(&ptr, g_gemm_status);
    return static_cast<DeviceStatus *>(ptr);
  }();
  p.status = status_ptr;

  static const bool attr_set = [] {
    return cudaFuncSetAttribute(gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) == cudaSuccess &&
           cudaFuncSetAttribute(gemm2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM2_BYTES) == cudaSuccess;
  }();
  if (!attr_set) return -1;
  const int total_tiles = p.m_tiles * p.n_tiles * p.splits;
  if (pair_kernel) {
    // a GEMM that waits for chunks of an all-gather in flight leaves SMs free for that gather's blocks
    const int pairs = (sm_count - (peer_mode == 3 ? kGatherBesideGemmBlocks : 0)) / 2;
    const int grid = 2 * (total_tiles < pairs ? total_tiles : pairs);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM2_BYTES;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm2_kernel, map_a, map_b, map_d, map_d2, peer_maps, p);
    if (e != cudaSuccess) return static_cast<int>(e);
    return finish_launch(1);
  }
  const int grid = total_tiles < sm_count ? total_tiles : sm_count;
  gemm_kernel<<<grid, THREADS, SMEM_BYTES, s>>>(map_a, map_b, p);
  return finish_launch(1);
}
CS_DEFINE_BOUNDS_GETTER(bounds_report_gemm)
}  // namespace cs::kernels
