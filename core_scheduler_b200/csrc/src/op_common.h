// SPDX-License-Identifier: Apache-2.0
// Helpers shared by the op implementation files (not part of the public surface).
#pragma once
#include "cs/compute.h"
#include "kernels/api.h"

namespace cs::compute::detail {
bool fused_enabled();
void *current_stream();
void check_kernel(int code, const char *what);
int dtype_code(at::ScalarType t);  // 0 fp32, 1 bf16, 2 fp16, -1 otherwise
// Writes `value` into a gradient slot: assign when empty, overwrite when fresh, else add.
void store_grad(const Tensor &slot, const at::Tensor &value, at::ScalarType store_dtype);
bool grad_slot_ready_for_fused(const Tensor &slot);
at::Tensor as2d(const at::Tensor &t);
bool fused_gemm(const kernels::GemmArgs &args);
// An op that was expected on this library's kernels (CUDA, bf16, fused backend) runs a library
// kernel instead: warns once per (op, reason) and counts every occurrence.
void note_library_fallback(const char *op, const char *reason);
int64_t library_fallback_count();
}  // namespace cs::compute::detail
