#include "api.h"
namespace cs::kernels {
int gemm_bf16(stream_t, const GemmArgs &) { return -1; }
int gemm_tile_n() { return 256; }
}  // namespace cs::kernels
