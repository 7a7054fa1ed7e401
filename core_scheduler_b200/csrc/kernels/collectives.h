// SPDX-License-Identifier: Apache-2.0
// Launch interface of the peer-memory collective kernels (kernels/collectives.cu).
// All ranks of one NVSwitch domain map each other's symmetric arena; a kernel on rank r
// addresses rank p's copy of a buffer as table.base[p] + offset and, when the arena has an
// NVLink multicast mapping, every rank's copy at once as table.mc + offset (multimem.ld_reduce
// sums the copies inside the switch, multimem.st writes all of them). No kernel here uses TMA:
// remote data moves with plain 128-bit peer loads and stores or with multimem instructions.
//
// Every collective is ONE launch: the cross-rank barrier that must precede it (all contributions
// complete) and the one that must follow it (all results written, all sources read) are part of
// the kernel. Block 0 exchanges flags with the peers, the other blocks wait on a local flag; at
// the end the last block to finish does the closing exchange.
//
// Residency. The pair GEMM is compiled for 128 registers per thread, which leaves room on every SM for light blocks
// of these kernels (256 threads, at most 40 registers, no shared memory to speak of): a collective proceeds beside a
// running GEMM. The one GEMM that itself waits for a collective (it consumes rows while symm_all_gather_chunked is
// still delivering them) launches on all but kGatherBesideGemmBlocks SMs, and that gather uses at most
// kGatherBesideGemmBlocks blocks of 1024 threads: both kernels are always resident together and neither can starve
// the other. The bulk-engine kernels need an SM's shared memory and wait for a free SM; nothing waits for them on
// the device.
#pragma once
#include <cstdint>

#include "api.h"

namespace cs::kernels {
constexpr int kMaxPeers = 8;

struct PeerTable {
  char *base[kMaxPeers];       // arena of every rank as mapped here
  uint32_t *flags[kMaxPeers];  // signal pad of every rank
  char *mc;                    // multicast mapping of the arena (null: none)
  int rank;
  int size;
  long long arena_bytes;       // size of every arena (0 = unknown); limit of the diagnostic build's offset checks
};

// Signal-pad layout (32-bit words). Words [0, 64) belong to the stand-alone barrier below. From
// kChannelBase on, every "channel" owns kChannelWords words:
//   [0, 8)    entry flags, one per source rank      [8, 16)   exit flags, one per source rank
//   [16]      local go flag (epoch)                  [17]      local count of finished blocks
//   [20, 28)  local counts of blocks that finished chunk c (chunked gather)
//   [32, 96)  chunk-ready flags [source rank * 8 + chunk], written by the source rank (chunked gather)
// Two kernels may be in flight at the same time only on different channels.
constexpr int kChannelBase = 64;
constexpr int kChannelWords = 128;
constexpr int kChunkCounters = 20;
constexpr int kChunkFlags = 32;
constexpr int kMaxChunks = 8;
constexpr int kGatherBesideGemmBlocks = 16;
enum Channel : int {
  kChanAllReduce = 0,
  kChanReduceScatter = 1,
  kChanAllGather = 2,
  kChanAllToAll = 3,
  kChanZero = 4,
  kChanGatherRows = 5,   // tensor parallel: row gathers on the main stream
  kChanScatterRows = 6,  // tensor parallel: row reduce-scatters on the main stream
  kChanGemmGather = 7,   // all-gather -> GEMM kernel
  kChanGemmScatter = 8,  // GEMM -> reduce-scatter kernel
  kChanCrossEntropy = 9, // vocabulary-parallel loss statistics
  kNumChannels = 16,
};

// What the host passes for the in-kernel barriers of one launch.
struct Handshake {
  int channel;
  uint32_t epoch;          // grows by one per launch on the channel (same on every rank)
  uint32_t blocks_before;  // blocks launched on this channel before this launch (local counter target base)
  long long budget;        // wait budget in clock64() cycles
  DeviceStatus *status;
};

// Wait budget of every peer-flag wait, in clock64() cycles (default ~2 s). Tests shrink it to
// provoke the timeout path: the kernel then records DeviceStatus{code=2} and returns.
void set_peer_wait_budget(long long cycles);
long long peer_wait_budget();

// Launch tuning of the link-bound kernels, process-wide (every rank must use the same values).
// grid cap: most blocks one collective launches (default 256; more blocks keep more bytes in flight on
// NVLink, fewer leave more of each SM to a GEMM running beside the collective).
// multicast threshold: smallest group that uses the NVLink multicast mapping when one exists (default 3).
// In a group of two a multimem access also fetches the local copy through the switch, which doubles the
// bytes on the wire, so pairs use plain peer loads and stores.
void set_collective_grid_cap(int blocks);
int collective_grid_cap();
void set_multicast_min_ranks(int ranks);
int multicast_min_ranks();

// All ranks arrive and leave together: rank r stores `epoch` into slot (slot_base + r) of every
// peer's pad and waits until its own pad shows `epoch` from every peer. One CTA.
int symm_barrier(stream_t stream, const PeerTable &t, int slot_base, uint32_t epoch, DeviceStatus *status);

// All-reduce in place on the same arena range of every rank, one launch. Rank r owns slice r:
// with a multicast mapping it loads the sum of all copies from the switch (multimem.ld_reduce,
// fp32 accumulation), scales, and writes all copies with one multimem.st; without one it pulls
// the slice from every peer, sums in fp32 and pushes the result to every peer. dtype: 0 fp32, 1 bf16.
// `blocks` receives the grid size (the caller advances Handshake::blocks_before by it).
int symm_all_reduce(stream_t stream, const PeerTable &t, const Handshake &h, int64_t offset_bytes, int64_t count, int dtype,
                    float scale, int *blocks);

// dst[i] = scale * sum_p src_p[src_offset + i] (+ residual[i]) for count elements (reduce-scatter: pass the
// offset of this rank's slice inside every rank's send buffer). dst and the optional bf16 residual are local
// memory. One launch.
int symm_reduce_scatter(stream_t stream, const PeerTable &t, const Handshake &h, int64_t src_offset_bytes, void *dst, int64_t count,
                        int dtype, float scale, int *blocks, const void *residual = nullptr);

// All-gather into a symmetric destination: this rank's `bytes` at `src` (any local memory) are written to
// dst_offset + rank * bytes of every rank (multimem.st, or one peer store per rank). One launch.
int symm_all_gather_push(stream_t stream, const PeerTable &t, const Handshake &h, const void *src, int64_t dst_offset_bytes,
                         int64_t bytes, int *blocks);

// The same all-gather in `chunks` row chunks: after chunk c of this rank's shard has been written everywhere,
// word kChunkFlags + rank * 8 + c of the channel is set to the epoch on every rank, so that a consumer kernel
// running beside the gather (the GEMM that multiplies the gathered rows) can start on the chunks that have landed.
int symm_all_gather_chunked(stream_t stream, const PeerTable &t, const Handshake &h, const void *src, int64_t dst_offset_bytes,
                            int64_t bytes, int chunks, int *blocks);

// Second half of a GEMM -> reduce-scatter whose GEMM epilogue stored every rank's partial rows (bf16) into the slot
// their owner keeps for that rank: dst[i] = sum over `slots` local slots (+ residual[i]), fp32 accumulation, bf16
// out. The kernel opens with the cross-rank barrier ("every rank's GEMM has finished writing"); it reads local
// memory only, so nothing has to follow it. `slots_base` is local memory: slot s starts at slots_base + s * slot_bytes.
int symm_slot_sum(stream_t stream, const PeerTable &t, const Handshake &h, const void *slots_base, int64_t slot_bytes, void *dst,
                  const void *residual, int64_t count);

// Strided chunk copies from peers (pull all-gather / all-to-all with pack and unpack fused):
// for each peer p: rows x row_bytes from base[p] + src_offset[p] (row stride src_stride) to
// dst[p] (row stride dst_stride). row_bytes, strides and addresses are multiples of 16. One launch.
struct PullCopyArgs {
  int64_t src_offset[kMaxPeers];
  char *dst[kMaxPeers];
  int64_t rows, row_bytes, src_stride, dst_stride;
};
int symm_pull_copy(stream_t stream, const PeerTable &t, const Handshake &h, const PullCopyArgs &args, int *blocks);

// ZeRO step in one kernel for the arena range [range_begin, range_end) (elements): reduce-scatter of the gradients
// (switch reduction or pull, fp32 accumulate), AdamW on the part of the range this rank owns, and all-gather of the
// updated bf16 working copy by writing it into every rank's bf16 arena.
// Ownership is interleaved in blocks of `block` elements (a power of two): block j of the arena belongs to rank
// j % size and is element range [(j / size) * block, ...) of that rank's local master / moment shards. Any range
// therefore splits evenly over the ranks, whatever its position, and the shard layout does not depend on how the
// gradients are bucketed.
struct ShardedAdamWArgs {
  int64_t grad_offset_bytes;   // gradient arena inside the symmetric arena (fp32)
  int64_t lp_offset_bytes;     // bf16 working-copy arena inside the symmetric arena (may be < 0: none)
  float *master;               // this rank's shard: fp32 master weights
  float *exp_avg, *exp_avg_sq; // this rank's shard of the moments
  int64_t range_begin, range_end;
  int64_t block;
  float lr, beta1, beta2, eps, weight_decay, inv_bias_correction1, inv_bias_correction2, grad_scale;
  const float *clip_coef;
};
int symm_reduce_scatter_adamw_all_gather(stream_t stream, const PeerTable &t, const Handshake &h, const ShardedAdamWArgs &args,
                                         int *blocks);
}  // namespace cs::kernels
