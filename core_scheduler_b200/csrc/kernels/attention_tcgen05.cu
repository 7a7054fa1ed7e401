// SPDX-License-Identifier: Apache-2.0
// Causal self-attention forward on tcgen05 tensor cores for head dimension 64, reading the packed
// qkv tensor [B, T, 3, H, 64] (the c_attn output) directly and writing [B, T, H*64] plus the
// per-row log-sum-exp.
//
// One CTA per (batch, head, 128-query block), 192 threads:
//   warp 0     TMA producer: Q once, then K and V tiles of 64 keys (one stage each)
//   warp 1     MMA issuer: S = Q K^T (128x64x64, fp32 in TMEM) and
//              O += P V (128x64x64; P from shared memory, V as an MN-major operand)
//   warps 2-5  softmax: one thread per query row reads its S row from TMEM, keeps the reference
//              max / running sum and writes P (bf16, 128-byte swizzled) to shared memory for the
//              second MMA. O accumulates in TMEM across key blocks; a warp rescales its 32 rows of
//              O in place only when a row maximum has grown by more than 2^8 since the reference
//              was taken (probabilities stay below 256, exact after the final division)
// Four CTAs share an SM (49 KB of shared memory, 128 TMEM columns and at most 85 registers per
// thread each): sixteen softmax warps per SM hide each other's TMEM, exp and barrier latencies. Scores never touch global memory. Every mbarrier wait is bounded (abort flag + status word).
//
// What it replaces in the reference project: at::_scaled_dot_product_flash_attention
// (src/compute/sdpa_flash_attn.cpp:56-60) and the cuDNN-frontend SDPA graph
// (src/compute/sdpa_cudnn.cpp:84-172) together with the split/view glue around them.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "api.h"
#include "bounds_check.h"

namespace cs::kernels {
namespace {
constexpr int BQ = 128;      // queries per CTA
constexpr int BKV = 64;      // keys per step
constexpr int HD = 64;       // head dimension
constexpr int TILE_BYTES = 128 * HD * 2;      // 16 KB: a 128-row tile (Q; resident tiles of the backward)
constexpr int KV_TILE_BYTES = BKV * HD * 2;   // 8 KB: K or V tile of the forward
constexpr int P_BYTES = BQ * BKV * 2;         // 16 KB
constexpr int THREADS = 192;
constexpr int FWD_CTAS_PER_SM = 4;
constexpr int SMEM_BYTES = TILE_BYTES + 2 * KV_TILE_BYTES + P_BYTES + 1024 + 256;  // ~49 KB: four CTAs per SM
constexpr int FWD_TMEM_COLS = 128;         // forward: S 64 columns + O 64 columns; four CTAs share the SM's 512
constexpr int TMEM_COLS = 256;             // backward: S', dP' and two accumulators of 64 columns each
constexpr long long kWaitBudgetCycles = 4000000000LL;

__device__ DeviceStatus g_attn_status;

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
// Brings a tile into L2 ahead of the TMA load that will need it (no shared memory, no barrier).
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap *map, int c0, int c1) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
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
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
        "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((addr & 0x3FFFF) >> 4);
  desc |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  desc |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
  desc |= static_cast<uint64_t>(1) << 46;
  desc |= static_cast<uint64_t>(2) << 61;  // 128-byte swizzle
  return desc;
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&t);
}

struct AttnParams {
  __nv_bfloat16 *out;   // [B, T, H*64]
  float *lse;           // [B, H, T]
  int B, T, H;
  float scale_log2e;    // softmax scale * log2(e)
  float scale;
  DeviceStatus *status;
  int causal;           // 1: keys after the query are masked; 0: every query sees every key
};

__global__ void __launch_bounds__(THREADS, FWD_CTAS_PER_SM) attention_fwd_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                                 const __grid_constant__ CUtensorMap map_kv,
                                                                                 const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *aligned = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_smem = base;                       // 128 x 64
  const uint32_t k_smem = q_smem + TILE_BYTES;        // 64 x 64 (one stage: four CTAs per SM hide the reload)
  const uint32_t v_smem = k_smem + KV_TILE_BYTES;     // 64 x 64
  const uint32_t p_smem = v_smem + KV_TILE_BYTES;     // 128 x 64 probabilities
  const uint32_t bar_base = p_smem + P_BYTES;
  uint64_t *bars = reinterpret_cast<uint64_t *>(aligned + (bar_base - base));
  enum { Q_FULL = 0, K_FULL, K_EMPTY, V_FULL, V_EMPTY, S_FULL, S_EMPTY, P_FULL, P_EMPTY, O_FULL, NUM_BARS };
  auto bar = [&](int i) { return bar_base + 8u * i; };
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(bars + NUM_BARS);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(bars + NUM_BARS + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qb = gridDim.x - 1 - blockIdx.x;  // longest rows first
  const int h = blockIdx.y, b = blockIdx.z;
  const int q0 = qb * BQ;
  const int num_kv = p.causal ? 2 * (qb + 1) : p.T / BKV;  // causal: 64-key blocks 0 .. 2 qb + 1
  const int row_base = b * p.T;

  if (threadIdx.x == 0) {
    mbar_init(bar(Q_FULL), 1);
    mbar_init(bar(K_FULL), 1);
    mbar_init(bar(K_EMPTY), 1);
    mbar_init(bar(V_FULL), 1);
    mbar_init(bar(V_EMPTY), 1);
    mbar_init(bar(S_FULL), 1);
    mbar_init(bar(S_EMPTY), 4);  // one arrival per softmax warp
    mbar_init(bar(P_FULL), 4);
    mbar_init(bar(P_EMPTY), 1);
    mbar_init(bar(O_FULL), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(const_cast<uint32_t *>(tmem_slot))),
                 "r"(FWD_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t s_tmem = tmem_base;        // 64 columns of scores
  const uint32_t o_tmem = tmem_base + BKV;  // 64 columns of output accumulator

  if (warp == 0) {
    if (lane == 0) {
      const int q_col = h * HD, k_col = (p.H + h) * HD, v_col = (2 * p.H + h) * HD;
      mbar_expect_tx(bar(Q_FULL), TILE_BYTES);
      tma_load_2d(q_smem, &map_q, bar(Q_FULL), q_col, row_base + q0);
      constexpr int kAhead = 3;  // tiles requested into L2 before their shared-memory stage is free
      for (int j = 1; j < kAhead && j < num_kv; ++j) {
        tma_prefetch_2d(&map_kv, k_col, row_base + j * BKV);
        tma_prefetch_2d(&map_kv, v_col, row_base + j * BKV);
      }
      for (int j = 0; j < num_kv; ++j) {
        const uint32_t ph = j & 1;
        if (j + kAhead < num_kv) {
          tma_prefetch_2d(&map_kv, k_col, row_base + (j + kAhead) * BKV);
          tma_prefetch_2d(&map_kv, v_col, row_base + (j + kAhead) * BKV);
        }
        if (!mbar_wait(bar(K_EMPTY), ph ^ 1u, abort_flag)) break;
        mbar_expect_tx(bar(K_FULL), KV_TILE_BYTES);
        tma_load_2d(k_smem, &map_kv, bar(K_FULL), k_col, row_base + j * BKV);
        if (!mbar_wait(bar(V_EMPTY), ph ^ 1u, abort_flag)) break;
        mbar_expect_tx(bar(V_FULL), KV_TILE_BYTES);
        tma_load_2d(v_smem, &map_kv, bar(V_FULL), v_col, row_base + j * BKV);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // S = Q K^T: M=128, N=64, both operands K-major. O += P V: M=128, N=64, B (= V) MN-major.
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BKV >> 3) << 17) | (8u << 24);
      const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | (static_cast<uint32_t>(HD >> 3) << 17) | (8u << 24);
      // descriptors are built once; a k-step only advances the 16-byte-unit address field
      const uint64_t d_q = smem_desc(q_smem, 16, 1024), d_k = smem_desc(k_smem, 16, 1024);
      const uint64_t d_p = smem_desc(p_smem, 16, 1024), d_v = smem_desc(v_smem, 8192, 1024);
      constexpr uint64_t kStepK = 32 >> 4, kStepMN = 2048 >> 4;
      bool ok = mbar_wait(bar(Q_FULL), 0, abort_flag);
      auto issue_s = [&](int j) -> bool {
        const uint32_t ph = j & 1;
        if (!mbar_wait(bar(K_FULL), ph, abort_flag)) return false;
        if (!mbar_wait(bar(S_EMPTY), ph ^ 1u, abort_flag)) return false;  // softmax of block j-1 has read S
        fence_after();
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) umma(s_tmem, d_q + k * kStepK, d_k + k * kStepK, idesc_s, k > 0 ? 1u : 0u);
        umma_commit(bar(K_EMPTY));
        umma_commit(bar(S_FULL));
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; ok && j < num_kv; ++j) {
        const uint32_t ph = j & 1;
        if (j + 1 < num_kv) ok = issue_s(j + 1);  // as soon as the softmax warps have read S of block j (S_EMPTY)
        if (!ok) break;
        if (!mbar_wait(bar(P_FULL), ph, abort_flag)) break;
        if (!mbar_wait(bar(V_FULL), ph, abort_flag)) break;
        fence_after();
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k)  // P: one K-major tile; V: MN-major, 16 keys = 2 KB per step
          umma(o_tmem, d_p + k * kStepK, d_v + k * kStepMN, idesc_o, (j | k) ? 1u : 0u);
        umma_commit(bar(V_EMPTY));
        umma_commit(bar(P_EMPTY));
        umma_commit(bar(O_FULL));
      }
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;  // query row inside the block
    const int q_idx = q0 + r;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    float m_run = -INFINITY, l_run = 0.f;  // m_run: the maximum the exponents refer to (may lag the true one)
    bool ok = true;
    for (int j = 0; ok && j < num_kv; ++j) {
      const uint32_t ph = j & 1;
      if (!mbar_wait(bar(S_FULL), ph, abort_flag)) break;
      fence_after();
      const int k0 = j * BKV;
      const bool diagonal = p.causal && k0 + BKV - 1 > q0;  // some key of this block lies beyond some query of the tile
      // pass 1: row maximum of the (masked) scores. Four independent partial maxima / sums keep the
      // dependent chains short; the TMEM load of the next 16 columns is in flight meanwhile.
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      auto max_chunk = [&](const uint32_t (&v)[16], int c) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float x = __uint_as_float(v[i]);
          if (!diagonal || (k0 + c * 16 + i) <= q_idx) mx[i & 3] = fmaxf(mx[i & 3], x);
        }
      };
      uint32_t va[16], vb[16];
      tmem_ld16(s_tmem + 0 + lane_addr, va);
      tmem_wait_ld();
      tmem_ld16(s_tmem + 16 + lane_addr, vb);
      max_chunk(va, 0);
      tmem_wait_ld();
      tmem_ld16(s_tmem + 32 + lane_addr, va);
      max_chunk(vb, 1);
      tmem_wait_ld();
      tmem_ld16(s_tmem + 48 + lane_addr, vb);
      max_chunk(va, 2);
      tmem_wait_ld();
      tmem_ld16(s_tmem + 0 + lane_addr, va);  // first chunk of the second pass
      max_chunk(vb, 3);
      const float m_blk = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      // Move the reference maximum only when it lags by more than 2^8 (always on the first block).
      // A fully masked row of a diagonal block has m_blk = -inf and never moves it.
      const bool grow = j == 0 || (m_blk - m_run) * p.scale_log2e > 8.0f;
      float alpha = 1.0f;
      if (grow) {
        alpha = fast_exp2((m_run - m_blk) * p.scale_log2e);  // first block: exp2(-inf) = 0
        m_run = m_blk;
        l_run *= alpha;
      }
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        // rescale this warp's 32 rows of O in place; block j-1's P V must have landed first
        if (!__all_sync(0xffffffffu, mbar_wait(bar(O_FULL), ph ^ 1u, abort_flag))) {  // the warp leaves as one
          tmem_wait_ld();
          break;
        }
        fence_after();
        tmem_wait_ld();  // the prefetched S chunk in `va` is complete before more loads are issued
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t ov[16];
          tmem_ld16(o_tmem + c * 16 + lane_addr, ov);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
          tmem_st16(o_tmem + c * 16 + lane_addr, ov);
        }
        tmem_wait_st();
      }
      const float m_scaled = m_run * p.scale_log2e;
      // pass 2: probabilities -> shared memory (bf16, swizzled) and their sum
      if (!mbar_wait(bar(P_EMPTY), ph ^ 1u, abort_flag)) {
        tmem_wait_ld();  // no load may be outstanding when the kernel unwinds
        break;
      }
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
      auto exp_chunk = [&](const uint32_t (&v)[16], int c) {
        float e[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float x = __uint_as_float(v[i]);
          const bool keep = !diagonal || (k0 + c * 16 + i) <= q_idx;
          e[i] = keep ? fast_exp2(fmaf(x, p.scale_log2e, -m_scaled)) : 0.f;
          ls[i & 3] += e[i];
        }
        // 16 keys = 32 bytes = two 16-byte pieces of this row
        const uint32_t row_addr = p_smem + r * 128;
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          const int piece = c * 2 + g;
          const uint32_t addr = row_addr + ((piece ^ (r & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pack2(e[g * 8 + 0], e[g * 8 + 1])),
                       "r"(pack2(e[g * 8 + 2], e[g * 8 + 3])), "r"(pack2(e[g * 8 + 4], e[g * 8 + 5])),
                       "r"(pack2(e[g * 8 + 6], e[g * 8 + 7]))
                       : "memory");
        }
      };
      tmem_wait_ld();
      tmem_ld16(s_tmem + 16 + lane_addr, vb);
      exp_chunk(va, 0);
      tmem_wait_ld();
      tmem_ld16(s_tmem + 32 + lane_addr, va);
      exp_chunk(vb, 1);
      tmem_wait_ld();
      tmem_ld16(s_tmem + 48 + lane_addr, vb);
      exp_chunk(va, 2);
      tmem_wait_ld();
      // every score of this block has been read: the tensor core may start the next block's S
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(S_EMPTY));
      exp_chunk(vb, 3);
      fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(P_FULL));
      l_run += (ls[0] + ls[1]) + (ls[2] + ls[3]);
    }
    // the last block's P V completes the accumulator
    const bool done = ok && mbar_wait(bar(O_FULL), (num_kv - 1) & 1, abort_flag);
    if (done && !*abort_flag && q_idx < p.T &&
        CS_IN_BOUNDS(kKidAttention, (static_cast<long long>(row_base + q_idx) * p.H + h) * HD + HD - 1,
                     static_cast<long long>(p.B) * p.T * p.H * HD)) {
      fence_after();
      const float inv = 1.f / l_run;
      __nv_bfloat16 *dst = p.out + (static_cast<long long>(row_base + q_idx) * p.H + h) * HD;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[16];
        tmem_ld16(o_tmem + c * 16 + lane_addr, v);
        tmem_wait_ld();
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          uint4 w;
          w.x = pack2(__uint_as_float(v[g * 8 + 0]) * inv, __uint_as_float(v[g * 8 + 1]) * inv);
          w.y = pack2(__uint_as_float(v[g * 8 + 2]) * inv, __uint_as_float(v[g * 8 + 3]) * inv);
          w.z = pack2(__uint_as_float(v[g * 8 + 4]) * inv, __uint_as_float(v[g * 8 + 5]) * inv);
          w.w = pack2(__uint_as_float(v[g * 8 + 6]) * inv, __uint_as_float(v[g * 8 + 7]) * inv);
          *reinterpret_cast<uint4 *>(dst + c * 16 + g * 8) = w;
        }
      }
      p.lse[(static_cast<long long>(b) * p.H + h) * p.T + q_idx] = m_run * p.scale + __logf(l_run);
    }
  }

  fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) {
    p.status->code = 1;
    p.status->kernel_id = 3;
    p.status->block = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    p.status->detail = 0;
  }
  if (warp == 1) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(FWD_TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------------ backward ----
// dQ, dK, dV of causal attention from the packed qkv, the forward output, its gradient and the
// per-row log-sum-exp; results go straight into the packed dqkv [B, T, 3, H, 64].
//
// Three launches: (1) delta[b,h,t] = sum_d dO*O; (2) kDKV = true: one CTA per 128-key block keeps
// K_j, V_j resident and streams 64-query tiles (Q_i, dO_i), accumulating dV_j and dK_j in TMEM;
// (3) kDKV = false: one CTA per 128-query block keeps Q_i, dO_i resident and streams 64-key tiles
// (K_j, V_j), accumulating dQ_i in TMEM. No atomics, deterministic. Per streamed tile:
//   S' = R1 C1^T, dP' = R2 C2^T              (128 x 64 x 64 each, fp32 in TMEM; rows = resident side)
//   P' = exp(scale S' - lse), dS' = scale P' (dP' - delta)   (softmax warps, one thread per row)
//   [dV += P' C2]   acc += dS' C1            (128 x 64 x 64; P'/dS' from swizzled shared memory, C as
//                                             MN-major operands)
// 256 TMEM columns and ~99 KB of shared memory per CTA: two CTAs per SM; eight softmax warps per CTA
// (two threads per row, 32 of the 64 streamed columns each: the backward needs no row reductions).
constexpr int BC = 64;                          // streamed rows per step
constexpr int C_TILE_BYTES = BC * HD * 2;       // 8 KB
constexpr int PS_BYTES = 128 * BC * 2;          // 16 KB: P' or dS'
// streamed-tile stages: the dQ kernel has room for three (no P' tile); the dK/dV kernel for two
constexpr int bwd_stages(bool dkv) { return dkv ? 2 : 3; }
constexpr int BWD_THREADS = 320;  // TMA warp, MMA warp, eight softmax warps (two threads per row: 32 columns each)
constexpr int bwd_smem_bytes(bool dkv) {
  return 2 * TILE_BYTES + bwd_stages(dkv) * (2 * C_TILE_BYTES + 512) + (dkv ? 2 : 1) * PS_BYTES + 1024 + 256;
}

struct AttnBwdParams {
  __nv_bfloat16 *dqkv;  // [B, T, 3, H, 64]
  const float *lse;     // [B, H, T]: lse * log2(e)
  const float *delta;   // [B, H, T]: delta * scale
  int B, T, H;
  float scale, scale_log2e;
  DeviceStatus *status;
  int causal;
};

__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
               "r"(bytes), "r"(bar)
               : "memory");
}

__global__ void __launch_bounds__(256) attention_delta_kernel(const __nv_bfloat16 *__restrict__ out, const __nv_bfloat16 *__restrict__ dout,
                                                              const float *__restrict__ lse, float *__restrict__ delta, int B, int T,
                                                              int H, float scale) {
  // eight threads per (b, t, h) row of 64 values
  const long long gid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long row = gid >> 3;
  const int part = static_cast<int>(gid & 7);
  const long long rows = static_cast<long long>(B) * T * H;
  float acc = 0.f;
  if (row < rows) {
    const uint4 a = *reinterpret_cast<const uint4 *>(out + row * HD + part * 8);
    const uint4 g = *reinterpret_cast<const uint4 *>(dout + row * HD + part * 8);
    const __nv_bfloat162 *pa = reinterpret_cast<const __nv_bfloat162 *>(&a);
    const __nv_bfloat162 *pg = reinterpret_cast<const __nv_bfloat162 *>(&g);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = __bfloat1622float2(pa[i]), y = __bfloat1622float2(pg[i]);
      acc = fmaf(x.x, y.x, acc);
      acc = fmaf(x.y, y.y, acc);
    }
  }
  acc += __shfl_xor_sync(0xffffffffu, acc, 1);
  acc += __shfl_xor_sync(0xffffffffu, acc, 2);
  acc += __shfl_xor_sync(0xffffffffu, acc, 4);
  if (row < rows && part == 0) {
    const long long bt = row / H;
    const int h = static_cast<int>(row - bt * H);
    const long long b = bt / T;
    const int t = static_cast<int>(bt - b * T);
    // plane 0: delta; plane 1: lse * log2(e); plane 2: delta * scale (what the two backward kernels consume)
    const long long plane = static_cast<long long>(B) * H * T, at = (b * H + h) * T + t;
    delta[at] = acc;
    delta[plane + at] = lse[at] * 1.4426950408889634f;
    delta[2 * plane + at] = acc * scale;
  }
}

template <bool kDKV>
__global__ void __launch_bounds__(BWD_THREADS, 2)
attention_bwd_kernel(const __grid_constant__ CUtensorMap qkv_r, const __grid_constant__ CUtensorMap qkv_c,
                     const __grid_constant__ CUtensorMap do_r, const __grid_constant__ CUtensorMap do_c, const AttnBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *aligned = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t r1_smem = base;                      // resident operand of S'
  const uint32_t r2_smem = r1_smem + TILE_BYTES;      // resident operand of dP'
  const uint32_t c_smem = r2_smem + TILE_BYTES;       // per stage: C1 tile, C2 tile
  constexpr int STAGES = bwd_stages(kDKV);
  const uint32_t p_smem = c_smem + STAGES * 2 * C_TILE_BYTES;  // P' exists only in the dK/dV kernel
  const uint32_t ds_smem = p_smem + (kDKV ? PS_BYTES : 0);
  const uint32_t vec_smem = ds_smem + PS_BYTES;       // per stage: lse[64], delta[64] of the streamed queries
  const uint32_t bar_base = vec_smem + STAGES * 512;
  uint64_t *bars = reinterpret_cast<uint64_t *>(aligned + (bar_base - base));
  const float *vec = reinterpret_cast<const float *>(aligned + (vec_smem - base));
  enum { R_FULL = 0, C_FULL = 1, C_EMPTY = 4, SDP_FULL = 7, SDP_EMPTY = 8, PDS_FULL = 9, PDS_EMPTY = 10, ACC_FULL = 11, NUM_BARS = 12 };
  auto bar = [&](int i) { return bar_base + 8u * i; };
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(bars + NUM_BARS);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(bars + NUM_BARS + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Longest loops first: key block 0 streams all queries, query block T/128-1 streams all keys.
  const int rb = kDKV ? blockIdx.x : gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int r0 = rb * 128;
  const int row_base = b * p.T;
  // streamed 64-row tiles: queries r0 .. T (kDKV) or keys 0 .. r0+128
  const int c_first = (kDKV && p.causal) ? 2 * rb : 0;
  const int n_iter = kDKV ? p.T / BC - c_first : (p.causal ? 2 * (rb + 1) : p.T / BC);

  if (threadIdx.x == 0) {
    mbar_init(bar(R_FULL), 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar(C_FULL + s), 1);
      mbar_init(bar(C_EMPTY + s), 1);
    }
    mbar_init(bar(SDP_FULL), 1);
    mbar_init(bar(SDP_EMPTY), 8);  // one arrival per softmax warp
    mbar_init(bar(PDS_FULL), 8);
    mbar_init(bar(PDS_EMPTY), 1);
    mbar_init(bar(ACC_FULL), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(const_cast<uint32_t *>(tmem_slot))),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t s_tmem = tmem_base;             // S'   64 columns
  const uint32_t dp_tmem = tmem_base + BC;       // dP'  64 columns
  const uint32_t acc1_tmem = tmem_base + 2 * BC; // dV (kDKV only)
  const uint32_t acc2_tmem = tmem_base + 3 * BC; // dK or dQ

  const int q_col = h * HD, k_col = (p.H + h) * HD, v_col = (2 * p.H + h) * HD;
  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar(R_FULL), 2 * TILE_BYTES);
      if (kDKV) {
        tma_load_2d(r1_smem, &qkv_r, bar(R_FULL), k_col, row_base + r0);
        tma_load_2d(r2_smem, &qkv_r, bar(R_FULL), v_col, row_base + r0);
      } else {
        tma_load_2d(r1_smem, &qkv_r, bar(R_FULL), q_col, row_base + r0);
        tma_load_2d(r2_smem, &do_r, bar(R_FULL), q_col, row_base + r0);
      }
      const float *lse_row = p.lse + (static_cast<long long>(b) * p.H + h) * p.T;
      const float *delta_row = p.delta + (static_cast<long long>(b) * p.H + h) * p.T;
      constexpr int kAhead = 4;  // tiles requested into L2 before their shared-memory stage is free
      auto prefetch = [&](int t) {
        const int c0 = (c_first + t) * BC;
        if (kDKV) {
          tma_prefetch_2d(&qkv_c, q_col, row_base + c0);
          tma_prefetch_2d(&do_c, q_col, row_base + c0);
        } else {
          tma_prefetch_2d(&qkv_c, k_col, row_base + c0);
          tma_prefetch_2d(&qkv_c, v_col, row_base + c0);
        }
      };
      for (int t = STAGES; t < kAhead && t < n_iter; ++t) prefetch(t);
      for (int t = 0; t < n_iter; ++t) {
        const int s = t % STAGES;
        const uint32_t ph = (t / STAGES) & 1;
        const int c0 = (c_first + t) * BC;
        if (t + kAhead < n_iter) prefetch(t + kAhead);
        if (!mbar_wait(bar(C_EMPTY + s), ph ^ 1u, abort_flag)) break;
        const uint32_t c1 = c_smem + s * 2 * C_TILE_BYTES, c2 = c1 + C_TILE_BYTES;
        if (kDKV) {
          mbar_expect_tx(bar(C_FULL + s), 2 * C_TILE_BYTES + 512);
          tma_load_2d(c1, &qkv_c, bar(C_FULL + s), q_col, row_base + c0);
          tma_load_2d(c2, &do_c, bar(C_FULL + s), q_col, row_base + c0);
          bulk_load(vec_smem + s * 512, lse_row + c0, 256, bar(C_FULL + s));
          bulk_load(vec_smem + s * 512 + 256, delta_row + c0, 256, bar(C_FULL + s));
        } else {
          mbar_expect_tx(bar(C_FULL + s), 2 * C_TILE_BYTES);
          tma_load_2d(c1, &qkv_c, bar(C_FULL + s), k_col, row_base + c0);
          tma_load_2d(c2, &qkv_c, bar(C_FULL + s), v_col, row_base + c0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // S', dP': M=128, N=64, both operands K-major. Accumulators: M=128, N=64, B MN-major.
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BC >> 3) << 17) | (8u << 24);
      const uint32_t idesc_a = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | (static_cast<uint32_t>(HD >> 3) << 17) | (8u << 24);
      // Descriptors are built once; a k-step only advances the 16-byte-unit address field (the MMA thread
      // shares its scheduler with softmax warps, so every instruction it saves shortens the critical path).
      const uint64_t d_r1 = smem_desc(r1_smem, 16, 1024), d_r2 = smem_desc(r2_smem, 16, 1024);
      const uint64_t d_p = smem_desc(p_smem, 16, 1024), d_ds = smem_desc(ds_smem, 16, 1024);
      // stage 1 lies 2 * C_TILE_BYTES behind stage 0: one more constant added to the address field
      const uint64_t d_c1k0 = smem_desc(c_smem, 16, 1024), d_c2k0 = smem_desc(c_smem + C_TILE_BYTES, 16, 1024);
      const uint64_t d_c1m0 = smem_desc(c_smem, 8192, 1024), d_c2m0 = smem_desc(c_smem + C_TILE_BYTES, 8192, 1024);
      constexpr uint64_t kStage = (2 * C_TILE_BYTES) >> 4;
      constexpr uint64_t kStepK = 32 >> 4, kStepMN = 2048 >> 4;  // 16 elements along K: 32 bytes K-major, 2 KB MN-major
      bool ok = mbar_wait(bar(R_FULL), 0, abort_flag);
      auto issue_sdp = [&](int t) -> bool {
        const int s = t % STAGES;
        if (!mbar_wait(bar(C_FULL + s), (t / STAGES) & 1, abort_flag)) return false;
        if (!mbar_wait(bar(SDP_EMPTY), (t & 1) ^ 1u, abort_flag)) return false;
        fence_after();
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) umma(s_tmem, d_r1 + k * kStepK, d_c1k0 + s * kStage + k * kStepK, idesc_s, k > 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) umma(dp_tmem, d_r2 + k * kStepK, d_c2k0 + s * kStage + k * kStepK, idesc_s, k > 0 ? 1u : 0u);
        umma_commit(bar(SDP_FULL));
        return true;
      };
      if (ok) ok = issue_sdp(0);
      int t = 0;
      for (; ok && t < n_iter; ++t) {
        const int s = t % STAGES;
        // The scores of tile t+1 are issued as soon as the softmax warps hold tile t's S' / dP' in registers
        // (SDP_EMPTY), i.e. while they still compute; the accumulating MMAs of tile t follow once P' / dS' exist.
        if (t + 1 < n_iter) ok = issue_sdp(t + 1);
        if (!ok) break;
        if (!mbar_wait(bar(PDS_FULL), t & 1, abort_flag)) break;
        fence_after();
#pragma unroll
        for (int k = 0; k < BC / 16; ++k) {
          if (kDKV) umma(acc1_tmem, d_p + k * kStepK, d_c2m0 + s * kStage + k * kStepMN, idesc_a, (t | k) ? 1u : 0u);
          umma(acc2_tmem, d_ds + k * kStepK, d_c1m0 + s * kStage + k * kStepMN, idesc_a, (t | k) ? 1u : 0u);
        }
        umma_commit(bar(PDS_EMPTY));
        umma_commit(bar(C_EMPTY + s));
      }
      if (ok && t == n_iter) umma_commit(bar(ACC_FULL));
    }
  } else {
    const int q = warp & 3;            // TMEM lane quarter this warp may access
    const int half = (warp - 2) >> 2;  // which 32 of the 64 streamed columns this thread handles
    const int r = q * 32 + lane;       // row of the resident block
    const int r_idx = r0 + r;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    float lse_r = 0.f, delta_r = 0.f;
    if (!kDKV) {
      lse_r = p.lse[(static_cast<long long>(b) * p.H + h) * p.T + r_idx];
      delta_r = p.delta[(static_cast<long long>(b) * p.H + h) * p.T + r_idx];
    }
    bool ok = true;
    for (int t = 0; ok && t < n_iter; ++t) {
      const int s = t % STAGES;
      const int c0 = (c_first + t) * BC;
      if (kDKV && !mbar_wait(bar(C_FULL + s), (t / STAGES) & 1, abort_flag)) break;  // lse / delta of the streamed queries
      if (!mbar_wait(bar(SDP_FULL), t & 1, abort_flag)) break;
      fence_after();
      // rows are keys and columns queries (kDKV), or rows queries and columns keys: keep key <= query
      const bool near_diag = p.causal && (kDKV ? (c0 < r0 + 128) : (c0 + BC > r0));
      const float *lse_c = vec + s * 128, *delta_c = lse_c + 64;
      // 16 columns at a time; the TMEM loads of the next 16 are in flight while these are processed
      // per element: P' = exp2(S' * scale*log2e - lse*log2e), dS' = P' * (dP' * scale - delta*scale); the per-column
      // constants (dK/dV kernel) come from shared memory four at a time
      auto compute = [&](const uint32_t (&sv)[16], const uint32_t (&dv)[16], int c, uint32_t (&pp)[8], uint32_t (&dd)[8]) {
#pragma unroll
        for (int i = 0; i < 16; i += 4) {
          float l2[4] = {lse_r, lse_r, lse_r, lse_r}, dl[4] = {delta_r, delta_r, delta_r, delta_r};
          if (kDKV) {
            const float4 a = *reinterpret_cast<const float4 *>(lse_c + c * 16 + i);
            const float4 d = *reinterpret_cast<const float4 *>(delta_c + c * 16 + i);
            l2[0] = a.x; l2[1] = a.y; l2[2] = a.z; l2[3] = a.w;
            dl[0] = d.x; dl[1] = d.y; dl[2] = d.z; dl[3] = d.w;
          }
          float e4[4], d4[4];
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int col = c0 + c * 16 + i + v;
            const bool keep = !near_diag || (kDKV ? (r_idx <= col) : (col <= r_idx));
            e4[v] = keep ? fast_exp2(fmaf(__uint_as_float(sv[i + v]), p.scale_log2e, -l2[v])) : 0.f;
            d4[v] = e4[v] * fmaf(__uint_as_float(dv[i + v]), p.scale, -dl[v]);
          }
          pp[i >> 1] = pack2(e4[0], e4[1]);
          pp[(i >> 1) + 1] = pack2(e4[2], e4[3]);
          dd[i >> 1] = pack2(d4[0], d4[1]);
          dd[(i >> 1) + 1] = pack2(d4[2], d4[3]);
        }
      };
      auto store = [&](const uint32_t (&pp)[8], const uint32_t (&dd)[8], int c) {
        // 16 columns = 32 bytes = two 16-byte pieces of this row
        const uint32_t row_off = r * 128;
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          const int piece = c * 2 + g;
          const uint32_t off = row_off + ((piece ^ (r & 7)) << 4);
          if (kDKV)
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(p_smem + off), "r"(pp[g * 4 + 0]), "r"(pp[g * 4 + 1]),
                         "r"(pp[g * 4 + 2]), "r"(pp[g * 4 + 3])
                         : "memory");
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(ds_smem + off), "r"(dd[g * 4 + 0]), "r"(dd[g * 4 + 1]),
                       "r"(dd[g * 4 + 2]), "r"(dd[g * 4 + 3])
                       : "memory");
        }
      };
      uint32_t sa[16], da[16], sb[16], db[16];
      uint32_t pa[8], qa[8], pb[8], qb2[8];
      const int cb = half * 2;  // first 16-column chunk of this thread
      tmem_ld16(s_tmem + cb * 16 + lane_addr, sa);
      tmem_ld16(dp_tmem + cb * 16 + lane_addr, da);
      tmem_wait_ld();
      tmem_ld16(s_tmem + cb * 16 + 16 + lane_addr, sb);
      tmem_ld16(dp_tmem + cb * 16 + 16 + lane_addr, db);
      compute(sa, da, cb, pa, qa);
      tmem_wait_ld();
      // S' and dP' of this tile now live in registers: the tensor core may overwrite them with the next tile
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(SDP_EMPTY));
      compute(sb, db, cb + 1, pb, qb2);
      // the previous tile's accumulating MMAs must have read P' / dS' before they are overwritten
      if (!mbar_wait(bar(PDS_EMPTY), (t & 1) ^ 1u, abort_flag)) break;
      store(pa, qa, cb);
      store(pb, qb2, cb + 1);
      fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(PDS_FULL));
    }
    if (mbar_wait(bar(ACC_FULL), 0, abort_flag) && !*abort_flag) {
      fence_after();
      const long long row = static_cast<long long>(row_base + r_idx) * 3 * p.H;
      const bool row_in_range =
          CS_IN_BOUNDS(kKidAttention, (row + 2LL * p.H + h) * HD + HD - 1, static_cast<long long>(p.B) * p.T * 3 * p.H * HD);
      auto store = [&](uint32_t tmem, int part) {
        __nv_bfloat16 *dst = p.dqkv + (row + static_cast<long long>(part) * p.H + h) * HD + half * 32;
        uint32_t v[32];
        tmem_ld32(tmem + half * 32 + lane_addr, v);
        tmem_wait_ld();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 w;
          w.x = pack2(__uint_as_float(v[g * 8 + 0]), __uint_as_float(v[g * 8 + 1]));
          w.y = pack2(__uint_as_float(v[g * 8 + 2]), __uint_as_float(v[g * 8 + 3]));
          w.z = pack2(__uint_as_float(v[g * 8 + 4]), __uint_as_float(v[g * 8 + 5]));
          w.w = pack2(__uint_as_float(v[g * 8 + 6]), __uint_as_float(v[g * 8 + 7]));
          *reinterpret_cast<uint4 *>(dst + g * 8) = w;
        }
      };
      if (row_in_range) {
        if (kDKV) {
          store(acc1_tmem, 2);  // dV
          store(acc2_tmem, 1);  // dK
        } else {
          store(acc2_tmem, 0);  // dQ
        }
      }
    }
  }

  fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) {
    p.status->code = 1;
    p.status->kernel_id = kDKV ? 4 : 5;
    p.status->block = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    p.status->detail = 0;
  }
  if (warp == 1) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                              const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn attn_encode_fn() {
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
}  // namespace

int attention_status(DeviceStatus *out) {
  return static_cast<int>(cudaMemcpyFromSymbol(out, g_attn_status, sizeof(DeviceStatus)));
}

namespace {
// [rows, cols] bf16 row-major viewed through 64-column boxes of `box_rows` rows, 128-byte swizzle.
bool attn_map(CUtensorMap *out, const void *ptr, int64_t cols, int64_t rows, int box_rows) {
  EncodeFn fn = attn_encode_fn();
  if (!fn) return false;
  static std::mutex mu;
  static std::unordered_map<uint64_t, CUtensorMap> cache;
  std::lock_guard<std::mutex> lock{mu};
  const uint64_t key = reinterpret_cast<uint64_t>(ptr) ^ (static_cast<uint64_t>(rows) << 40) ^ (static_cast<uint64_t>(cols) << 20) ^
                       (static_cast<uint64_t>(box_rows) << 56);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return true;
  }
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols * 2)};
  const cuuint32_t box[2] = {HD, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  if (fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(ptr), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return true;
}
DeviceStatus *attn_status_ptr() {
  static DeviceStatus *ptr = [] {
    void *p = nullptr;
    cudaGetSymbolAddress(&p, g_attn_status);
    return static_cast<DeviceStatus *>(p);
  }();
  return ptr;
}
}  // namespace

int attention_forward_packed(stream_t stream, const void *qkv, void *out, float *lse, int64_t B, int64_t T, int64_t H, int64_t D,
                             float scale, int causal) {
  if (D != HD || T % BQ != 0 || B <= 0 || H <= 0 || T <= 0) return -1;
  if ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(out)) & 15) return -1;
  static const bool disabled = std::getenv("CS_DISABLE_TCGEN05_ATTENTION") != nullptr;
  if (disabled) return -1;
  CUtensorMap map_q, map_kv;
  if (!attn_map(&map_q, qkv, 3 * H * D, B * T, BQ) || !attn_map(&map_kv, qkv, 3 * H * D, B * T, BKV)) return -1;
  static const bool attr_set =
      cudaFuncSetAttribute(attention_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) == cudaSuccess;
  if (!attr_set) return -1;
  AttnParams p{};
  p.out = static_cast<__nv_bfloat16 *>(out);
  p.lse = lse;
  p.B = static_cast<int>(B);
  p.T = static_cast<int>(T);
  p.H = static_cast<int>(H);
  p.scale = scale;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.status = attn_status_ptr();
  p.causal = causal ? 1 : 0;
  dim3 grid(static_cast<unsigned>(T / BQ), static_cast<unsigned>(H), static_cast<unsigned>(B));
  attention_fwd_kernel<<<grid, THREADS, SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(map_q, map_kv, p);
  return finish_launch(1);
}

int attention_backward_packed(stream_t stream, const void *qkv, const void *out, const void *dout, const float *lse, float *delta,
                              void *dqkv, int64_t B, int64_t T, int64_t H, int64_t D, float scale, int causal) {
  if (D != HD || T % 128 != 0 || B <= 0 || H <= 0 || T <= 0) return -1;
  if ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(dout) |
       reinterpret_cast<uintptr_t>(dqkv) | reinterpret_cast<uintptr_t>(lse) | reinterpret_cast<uintptr_t>(delta)) & 15)
    return -1;
  static const bool disabled = std::getenv("CS_DISABLE_TCGEN05_ATTENTION") != nullptr;
  if (disabled) return -1;
  CUtensorMap qkv_r, qkv_c, do_r, do_c;
  if (!attn_map(&qkv_r, qkv, 3 * H * D, B * T, 128) || !attn_map(&qkv_c, qkv, 3 * H * D, B * T, BC) ||
      !attn_map(&do_r, dout, H * D, B * T, 128) || !attn_map(&do_c, dout, H * D, B * T, BC))
    return -1;
  static const bool attr_set =
      cudaFuncSetAttribute(attention_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bwd_smem_bytes(true)) == cudaSuccess &&
      cudaFuncSetAttribute(attention_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bwd_smem_bytes(false)) == cudaSuccess;
  if (!attr_set) return -1;
  auto s = static_cast<cudaStream_t>(stream);
  const long long threads = B * T * H * 8;
  attention_delta_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, s>>>(
      static_cast<const __nv_bfloat16 *>(out), static_cast<const __nv_bfloat16 *>(dout), lse, delta, static_cast<int>(B),
      static_cast<int>(T), static_cast<int>(H), scale);
  AttnBwdParams p{};
  p.dqkv = static_cast<__nv_bfloat16 *>(dqkv);
  p.lse = delta + B * H * T;        // plane 1 of the workspace: lse * log2(e)
  p.delta = delta + 2 * B * H * T;  // plane 2: delta * scale
  p.B = static_cast<int>(B);
  p.T = static_cast<int>(T);
  p.H = static_cast<int>(H);
  p.scale = scale;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.status = attn_status_ptr();
  p.causal = causal ? 1 : 0;
  dim3 grid(static_cast<unsigned>(T / 128), static_cast<unsigned>(H), static_cast<unsigned>(B));
  attention_bwd_kernel<true><<<grid, BWD_THREADS, bwd_smem_bytes(true), s>>>(qkv_r, qkv_c, do_r, do_c, p);
  attention_bwd_kernel<false><<<grid, BWD_THREADS, bwd_smem_bytes(false), s>>>(qkv_r, qkv_c, do_r, do_c, p);
  return finish_launch(3);
}
CS_DEFINE_BOUNDS_GETTER(bounds_report_attention)
}  // namespace cs::kernels
