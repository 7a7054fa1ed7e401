// SPDX-License-Identifier: Apache-2.0
// Glue between the symmetric-memory context and the kernel launch interface (not part of the public surface).
#pragma once
#include "cs/symmetric.h"
#include "kernels/collectives.h"

namespace cs::communication {
inline kernels::PeerTable table_of(const SymmetricContext &ctx) {
  kernels::PeerTable t{};
  for (int p = 0; p < ctx.size; ++p) {
    t.base[p] = ctx.bases[p];
    t.flags[p] = ctx.flags[p];
  }
  t.mc = ctx.size >= kernels::multicast_min_ranks() ? ctx.multicast_base : nullptr;
  t.rank = ctx.rank;
  t.size = ctx.size;
  t.arena_bytes = ctx.arena_bytes;
  return t;
}

// The in-kernel barriers of the next launch on `channel`: a fresh epoch and the number of blocks the channel
// has run so far. Every rank calls this in the same order, so the numbers agree everywhere.
inline kernels::Handshake begin_collective(SymmetricContext &ctx, int channel) {
  kernels::Handshake h{};
  h.channel = channel;
  h.epoch = ++ctx.channel_epoch[channel];
  h.blocks_before = ctx.channel_blocks[channel];
  h.budget = kernels::peer_wait_budget();
  h.status = static_cast<kernels::DeviceStatus *>(ctx.status);
  return h;
}
inline void end_collective(SymmetricContext &ctx, int channel, int blocks) {
  ctx.channel_blocks[channel] += static_cast<uint32_t>(blocks);
}
}  // namespace cs::communication
