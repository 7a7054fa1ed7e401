// Launch interface of the peer-memory collective kernels (kernels/collectives.cu).
// All ranks of one NVSwitch domain map each other's symmetric arena; a kernel on rank r
// addresses rank p's copy of a buffer as table.base[p] + offset. No kernel here uses TMA or
// multicast loads: remote data moves with plain 128-bit peer loads and stores.
#pragma once
#include <cstdint>

#include "api.h"

namespace cs::kernels {
constexpr int kMaxPeers = 8;

struct PeerTable {
  char *base[kMaxPeers];       // arena of every rank as mapped here
  uint32_t *flags[kMaxPeers];  // signal pad of every rank
  int rank;
  int size;
  long long arena_bytes;       // size of every arena (0 = unknown); limit of the diagnostic build's offset checks
};

// Wait budget of every peer-flag wait, in clock64() cycles (default ~2 s). Tests shrink it to
// provoke the timeout path: the kernel then records DeviceStatus{code=2} and returns.
void set_peer_wait_budget(long long cycles);
long long peer_wait_budget();

// All ranks arrive and leave together: rank r stores `epoch` into slot (slot_base + r) of every
// peer's pad and waits until its own pad shows `epoch` from every peer. One CTA.
int symm_barrier(stream_t stream, const PeerTable &t, int slot_base, uint32_t epoch, DeviceStatus *status);

// Two-shot all-reduce in place on the same arena range of every rank. Rank r sums slice r of all
// ranks (fp32 accumulation), multiplies by `scale` and stores the result into slice r of every
// rank's buffer. dtype: 0 fp32, 1 bf16. The caller brackets it with symm_barrier.
int symm_all_reduce_inplace(stream_t stream, const PeerTable &t, int64_t offset_bytes, int64_t count, int dtype, float scale);

// One-shot variant for small messages: every rank sums all copies into its own (no peer stores).
// `staging_offset` is where every rank put its contribution; dst is local memory.
int symm_all_reduce_oneshot(stream_t stream, const PeerTable &t, int64_t staging_offset, void *dst, int64_t count, int dtype,
                            float scale);

// dst[i] = scale * sum_p src_p[src_offset + i] for count elements (pull reduce-scatter: pass the
// offset of this rank's slice inside every peer's send buffer). dst is local memory.
int symm_pull_reduce(stream_t stream, const PeerTable &t, int64_t src_offset_bytes, void *dst, int64_t count, int dtype,
                     float scale);

// Strided chunk copies from peers (pull all-gather / all-to-all with pack and unpack fused):
// for each peer p: rows x row_bytes from base[p] + src_offset[p] (row stride src_stride) to
// dst[p] (row stride dst_stride). row_bytes, strides and addresses are multiples of 16.
struct PullCopyArgs {
  int64_t src_offset[kMaxPeers];
  char *dst[kMaxPeers];
  int64_t rows, row_bytes, src_stride, dst_stride;
};
int symm_pull_copy(stream_t stream, const PeerTable &t, const PullCopyArgs &args);

// ZeRO step in one kernel: reduce-scatter of the gradient arena (pull, fp32 accumulate),
// AdamW on this rank's shard of (master weights, moments), and all-gather of the updated bf16
// working copy by pushing it into every rank's bf16 arena.
struct ShardedAdamWArgs {
  int64_t grad_offset_bytes;   // gradient arena inside the symmetric arena (fp32)
  int64_t lp_offset_bytes;     // bf16 working-copy arena inside the symmetric arena (may be < 0: none)
  float *master;               // this rank's shard: fp32 master weights, length shard_count
  float *exp_avg, *exp_avg_sq;
  int64_t shard_begin;         // first element of this rank's shard inside the arenas
  int64_t shard_count;
  float lr, beta1, beta2, eps, weight_decay, inv_bias_correction1, inv_bias_correction2, grad_scale;
  const float *clip_coef;
};
int symm_reduce_scatter_adamw_all_gather(stream_t stream, const PeerTable &t, const ShardedAdamWArgs &args);
}  // namespace cs::kernels
