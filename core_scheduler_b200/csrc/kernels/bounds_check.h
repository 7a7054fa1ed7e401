// SPDX-License-Identifier: Apache-2.0
// Checked index accessors for the diagnostic build of the kernels (-DCS_BOUNDS_CHECK).
//
// In that build every derived global index (row * stride + column, a token id used as a table
// row, a peer offset, ...) goes through CS_IN_BOUNDS: the first violation is recorded in a small
// device-side report (kernel id, block, thread, index, limit) and the access is skipped. Nothing
// traps and no device assert fires, so the context stays usable and the host reads the report
// after the launch with cs::kernels::bounds_report(). In the normal build the macro is the
// constant `true` and the checks cost nothing.
//
// The reference project has no counterpart: it relies on the libraries' own device asserts.
#pragma once

#include <cuda_runtime.h>

#include "api.h"

namespace cs::kernels {
enum BoundsKernelId : int {
  kKidAdamW = 10, kKidLayerNormFwd = 11, kKidLayerNormBwd = 12, kKidEmbeddingFwd = 13, kKidEmbeddingBwd = 14,
  kKidCrossEntropy = 15, kKidPackQkv = 16, kKidTranspose = 17, kKidCollective = 18, kKidGemmEpilogue = 19,
  kKidAttention = 20, kKidElementwise = 21,
};

#ifdef CS_BOUNDS_CHECK
namespace {
__device__ BoundsReport g_bounds_report;  // one per translation unit; bounds_report() merges them
}
__device__ __forceinline__ bool cs_in_bounds(int kernel_id, long long index, long long limit) {
  if (index >= 0 && index < limit) return true;
  if (atomicCAS(&g_bounds_report.code, 0, 1) == 0) {
    g_bounds_report.kernel_id = kernel_id;
    g_bounds_report.block = static_cast<int>(blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z));
    g_bounds_report.thread = static_cast<int>(threadIdx.x);
    g_bounds_report.index = index;
    g_bounds_report.limit = limit;
  }
  return false;
}
#define CS_IN_BOUNDS(kernel_id, index, limit) ::cs::kernels::cs_in_bounds(kernel_id, static_cast<long long>(index), static_cast<long long>(limit))
#define CS_DEFINE_BOUNDS_GETTER(name)                                                                         \
  int name(BoundsReport *out, bool reset) {                                                                   \
    int rc = static_cast<int>(cudaMemcpyFromSymbol(out, g_bounds_report, sizeof(BoundsReport)));              \
    if (rc == 0 && reset) {                                                                                   \
      const BoundsReport zero{};                                                                              \
      rc = static_cast<int>(cudaMemcpyToSymbol(g_bounds_report, &zero, sizeof(BoundsReport)));                \
    }                                                                                                         \
    return rc;                                                                                                \
  }
#else
#define CS_IN_BOUNDS(kernel_id, index, limit) true
#define CS_DEFINE_BOUNDS_GETTER(name)          \
  int name(BoundsReport *out, bool) {          \
    *out = BoundsReport{};                     \
    return 0;                                  \
  }
#endif

// per translation unit (defined with CS_DEFINE_BOUNDS_GETTER)
int bounds_report_elementwise(BoundsReport *out, bool reset);
int bounds_report_collectives(BoundsReport *out, bool reset);
int bounds_report_gemm(BoundsReport *out, bool reset);
int bounds_report_attention(BoundsReport *out, bool reset);
}  // namespace cs::kernels
