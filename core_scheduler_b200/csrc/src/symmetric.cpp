// SPDX-License-Identifier: Apache-2.0
// Symmetric memory context and peer-memory collectives (host side). See cs/symmetric.h.
#include "cs/symmetric.h"

#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <thread>

#include "kernels/collectives.h"
#include "symm_internal.h"
#include "vmm.h"

namespace cs::communication {
namespace {
constexpr int64_t kAlign = 256;
int64_t round_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

void *cur_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

void check(int code, const char *what) {
  CS_ASSERT_TRUE(code == 0, "`", what, "` failed: ", cuda_error_string(code));
}

std::vector<uint8_t> to_bytes(const cudaIpcMemHandle_t &h) {
  const auto *p = reinterpret_cast<const uint8_t *>(&h);
  return std::vector<uint8_t>(p, p + sizeof(h));
}
cudaIpcMemHandle_t from_bytes(const std::vector<uint8_t> &b) {
  cudaIpcMemHandle_t h;
  CS_ASSERT_TRUE(b.size() == sizeof(h), "malformed IPC handle in the store");
  std::memcpy(&h, b.data(), sizeof(h));
  return h;
}

int dtype_code(at::ScalarType t) { return t == at::kFloat ? 0 : (t == at::kBFloat16 ? 1 : -1); }
}  // namespace

SymmetricContext::~SymmetricContext() {
  if (!owns_) return;
  // Errors at teardown are ignored on purpose.
  cudaDeviceSynchronize();
  if (virtual_memory) {
    vmm_.reset();  // unbinds the multicast object, unmaps every range, releases the handles
  } else {
    // Mappings of peers first, then our own memory.
    for (void *p : opened_) cudaIpcCloseMemHandle(p);
    if (!bases.empty() && bases[rank]) cudaFree(bases[rank]);
    if (!flags.empty() && flags[rank]) cudaFree(flags[rank]);
  }
  if (status) cudaFree(status);
  (void)cudaGetLastError();
}

SymmetricBlock SymmetricContext::allocate(int64_t bytes) {
  // Every rank issues the same sequence of calls, so the deterministic policy below (best fit,
  // split the remainder, otherwise bump) yields the same offsets everywhere.
  bytes = round_up(std::max<int64_t>(bytes, 1), kAlign);
  int best = -1;
  for (size_t i = 0; i < free_.size(); ++i)
    if (free_[i].bytes >= bytes && (best < 0 || free_[i].bytes < free_[best].bytes)) best = static_cast<int>(i);
  if (best >= 0) {
    SymmetricBlock b = free_[best];
    free_.erase(free_.begin() + best);
    if (b.bytes > bytes) {
      free_.push_back(SymmetricBlock{b.offset + bytes, b.bytes - bytes});
      b.bytes = bytes;
    }
    in_use_ += b.bytes;
    return b;
  }
  CS_ASSERT_TRUE(bump_ + bytes <= arena_bytes, "symmetric arena exhausted: ", bump_, " + ", bytes, " > ", arena_bytes);
  SymmetricBlock b{bump_, bytes};
  bump_ += bytes;
  in_use_ += bytes;
  return b;
}

void SymmetricContext::release(const SymmetricBlock &block) {
  if (block.bytes <= 0) return;
  in_use_ -= block.bytes;
  SymmetricBlock merged = block;
  // unite with free neighbours, then give the top of the arena back to the bump pointer
  for (bool again = true; again;) {
    again = false;
    for (size_t i = 0; i < free_.size(); ++i) {
      const auto &f = free_[i];
      if (f.offset + f.bytes == merged.offset || merged.offset + merged.bytes == f.offset) {
        merged = SymmetricBlock{std::min(f.offset, merged.offset), f.bytes + merged.bytes};
        free_.erase(free_.begin() + static_cast<std::ptrdiff_t>(i));
        again = true;
        break;
      }
    }
  }
  if (merged.offset + merged.bytes == bump_)
    bump_ = merged.offset;
  else
    free_.push_back(merged);
}

SymmetricBlock SymmetricContext::staging(int64_t bytes) {
  if (staging_.bytes >= bytes) return staging_;
  if (staging_.bytes > 0) release(staging_);
  staging_ = allocate(std::max<int64_t>(bytes, 32 << 20));
  return staging_;
}

at::Tensor SymmetricContext::tensor(const SymmetricBlock &block, at::IntArrayRef sizes, at::ScalarType dtype) const {
  int64_t numel = 1;
  for (auto s : sizes) numel *= s;
  CS_ASSERT_TRUE(numel * static_cast<int64_t>(c10::elementSize(dtype)) <= block.bytes, "tensor does not fit its symmetric block");
  return at::from_blob(bases[rank] + block.offset, sizes, [](void *) {},
                       at::TensorOptions().dtype(dtype).device(at::kCUDA, static_cast<c10::DeviceIndex>(device)));
}

bool SymmetricContext::locate(const void *ptr, int64_t bytes, int64_t *offset) const {
  const char *p = static_cast<const char *>(ptr);
  const char *lo = bases[rank];
  if (p < lo || p + bytes > lo + arena_bytes) return false;
  *offset = p - lo;
  return true;
}

void SymmetricContext::barrier() {
  ++epoch;
  check(kernels::symm_barrier(cur_stream(), table_of(*this), 0, epoch, static_cast<kernels::DeviceStatus *>(status)),
        "symm_barrier");
}

namespace {
// vmm::Exchange over the communicator's key/value store
struct StoreExchange : vmm::Exchange {
  c10d::Store &store;
  std::string prefix;
  int size;
  StoreExchange(c10d::Store &s, std::string p, int n) : store{s}, prefix{std::move(p)}, size{n} {}
  void put(const std::string &key, const std::string &value) override {
    store.set(prefix + key, std::vector<uint8_t>(value.begin(), value.end()));
  }
  std::string get(const std::string &key) override {
    auto raw = store.get(prefix + key);  // blocks until the key exists (store timeout applies)
    return std::string(raw.begin(), raw.end());
  }
  void barrier(const std::string &name) override {
    store.add(prefix + name, 1);
    const auto t0 = std::chrono::steady_clock::now();
    while (store.add(prefix + name, 0) < size) {
      CS_ASSERT_TRUE(std::chrono::steady_clock::now() - t0 < std::chrono::seconds(120), "timed out in the store barrier `", name, "`");
      std::this_thread::sleep_for(std::chrono::milliseconds(2));
    }
  }
};

bool env_is(const char *name, const char *value) {
  const char *e = std::getenv(name);
  return e != nullptr && std::string(e) == value;
}
}  // namespace

std::shared_ptr<SymmetricContext> create_symmetric_context(const Comm &comm, int64_t arena_bytes) {
  auto &impl = *comm.impl();
  CS_ASSERT_TRUE(impl.size <= kernels::kMaxPeers, "symmetric memory supports up to ", kernels::kMaxPeers, " ranks");
  auto ctx = std::make_shared<SymmetricContext>();
  ctx->rank = static_cast<int>(impl.rank);
  ctx->size = static_cast<int>(impl.size);
  int device = 0;
  CS_CHECK_CUDART(cudaGetDevice(&device));
  ctx->device = device;
  ctx->arena_bytes = round_up(arena_bytes, kAlign);
  ctx->bases.assign(ctx->size, nullptr);
  ctx->flags.assign(ctx->size, nullptr);
  ctx->owns_ = true;
  CS_CHECK_CUDART(cudaMalloc(&ctx->status, sizeof(kernels::DeviceStatus)));
  CS_CHECK_CUDART(cudaMemset(ctx->status, 0, sizeof(kernels::DeviceStatus)));
  const int64_t pad_bytes = SymmetricContext::kFlagWords * static_cast<int64_t>(sizeof(uint32_t));
  static int generation = 0;
  const std::string prefix = str_cat("cs/symm/", generation++, "/");
  CS_ASSERT_TRUE(ctx->size == 1 || impl.store != nullptr, "symmetric memory needs the communicator's store to exchange handles");

  // ---- preferred: one cuMemCreate allocation per rank (arena followed by the signal pad), shared as file
  //      descriptors, with an NVLink multicast object over the same pages --------------------------------
  if (ctx->size > 1 && !env_is("CS_SYMMETRIC_IPC", "1")) {
    StoreExchange exchange{*impl.store, prefix, ctx->size};
    auto arena = std::make_shared<vmm::Arena>();
    std::string why;
    const bool want_multicast = !env_is("NCCL_NVLS_ENABLE", "0");
    if (vmm::create(arena.get(), ctx->rank, ctx->size, device, ctx->arena_bytes + pad_bytes, want_multicast, exchange, &why)) {
      for (int p = 0; p < ctx->size; ++p) {
        ctx->bases[p] = arena->peer_va[p];
        ctx->flags[p] = reinterpret_cast<uint32_t *>(arena->peer_va[p] + ctx->arena_bytes);
      }
      ctx->multicast_base = arena->multicast_va;
      ctx->virtual_memory = true;
      ctx->vmm_ = std::shared_ptr<void>(arena.get(), [arena](void *) { vmm::destroy(arena.get()); });
      CS_CHECK_CUDART(cudaMemset(ctx->flags[ctx->rank], 0, static_cast<size_t>(pad_bytes)));
      CS_CHECK_CUDART(cudaDeviceSynchronize());
      exchange.barrier("pads_cleared");  // nobody signals into a pad that is still being cleared
      impl.symmetric = ctx;
      return ctx;
    }
    logger().warn("symmetric arena: virtual-memory path unavailable (", why, "); using cudaMalloc + CUDA IPC without multicast");
  }

  // ---- fallback: cudaMalloc + CUDA IPC (no multicast) -----------------------------------------------------
  void *base = nullptr, *pad = nullptr;
  CS_CHECK_CUDART(cudaMalloc(&base, ctx->arena_bytes));
  CS_CHECK_CUDART(cudaMalloc(&pad, static_cast<size_t>(pad_bytes)));
  CS_CHECK_CUDART(cudaMemset(pad, 0, static_cast<size_t>(pad_bytes)));
  CS_CHECK_CUDART(cudaDeviceSynchronize());
  ctx->bases[ctx->rank] = static_cast<char *>(base);
  ctx->flags[ctx->rank] = static_cast<uint32_t *>(pad);
  if (ctx->size > 1) {
    cudaIpcMemHandle_t h_base, h_pad;
    CS_CHECK_CUDART(cudaIpcGetMemHandle(&h_base, base));
    CS_CHECK_CUDART(cudaIpcGetMemHandle(&h_pad, pad));
    impl.store->set(str_cat(prefix, "arena/", ctx->rank), to_bytes(h_base));
    impl.store->set(str_cat(prefix, "flags/", ctx->rank), to_bytes(h_pad));
    for (int p = 0; p < ctx->size; ++p) {
      if (p == ctx->rank) continue;
      auto hb = from_bytes(impl.store->get(str_cat(prefix, "arena/", p)));
      auto hp = from_bytes(impl.store->get(str_cat(prefix, "flags/", p)));
      void *pb = nullptr, *pp = nullptr;
      CS_CHECK_CUDART(cudaIpcOpenMemHandle(&pb, hb, cudaIpcMemLazyEnablePeerAccess));
      CS_CHECK_CUDART(cudaIpcOpenMemHandle(&pp, hp, cudaIpcMemLazyEnablePeerAccess));
      ctx->bases[p] = static_cast<char *>(pb);
      ctx->flags[p] = static_cast<uint32_t *>(pp);
      ctx->opened_.push_back(pb);
      ctx->opened_.push_back(pp);
    }
    // host rendezvous: nobody proceeds (and possibly frees) before everyone mapped everything
    impl.store->add(str_cat(prefix, "mapped"), 1);
    const auto t0 = std::chrono::steady_clock::now();
    while (impl.store->add(str_cat(prefix, "mapped"), 0) < ctx->size) {
      CS_ASSERT_TRUE(std::chrono::steady_clock::now() - t0 < std::chrono::seconds(120),
                     "timed out waiting for all ranks to map the symmetric arena");
      std::this_thread::sleep_for(std::chrono::milliseconds(2));
    }
  }
  impl.symmetric = ctx;
  return ctx;
}

std::vector<std::shared_ptr<SymmetricContext>> create_loopback_contexts(int ranks, int64_t arena_bytes) {
  CS_ASSERT_TRUE(ranks >= 1 && ranks <= kernels::kMaxPeers, "loopback emulation supports 1 to ", kernels::kMaxPeers, " ranks");
  int device = 0;
  CS_CHECK_CUDART(cudaGetDevice(&device));
  struct Holder {
    std::vector<void *> blocks;
    ~Holder() {
      for (void *p : blocks) cudaFree(p);
      (void)cudaGetLastError();
    }
  };
  auto holder = std::make_shared<Holder>();
  const int64_t bytes = round_up(arena_bytes, kAlign);
  const size_t pad_bytes = SymmetricContext::kFlagWords * sizeof(uint32_t);
  std::vector<char *> bases(ranks);
  std::vector<uint32_t *> pads(ranks);
  for (int r = 0; r < ranks; ++r) {
    void *base = nullptr, *pad = nullptr;
    CS_CHECK_CUDART(cudaMalloc(&base, static_cast<size_t>(bytes)));
    holder->blocks.push_back(base);
    CS_CHECK_CUDART(cudaMalloc(&pad, pad_bytes));
    holder->blocks.push_back(pad);
    CS_CHECK_CUDART(cudaMemset(pad, 0, pad_bytes));
    bases[r] = static_cast<char *>(base);
    pads[r] = static_cast<uint32_t *>(pad);
  }
  std::vector<std::shared_ptr<SymmetricContext>> out;
  for (int r = 0; r < ranks; ++r) {
    auto ctx = std::make_shared<SymmetricContext>();
    ctx->rank = r;
    ctx->size = ranks;
    ctx->device = device;
    ctx->arena_bytes = bytes;
    ctx->bases = bases;
    ctx->flags = pads;
    ctx->loopback_ = holder;
    void *status = nullptr;
    CS_CHECK_CUDART(cudaMalloc(&status, sizeof(kernels::DeviceStatus)));
    holder->blocks.push_back(status);
    CS_CHECK_CUDART(cudaMemset(status, 0, sizeof(kernels::DeviceStatus)));
    ctx->status = status;
    out.push_back(ctx);
  }
  CS_CHECK_CUDART(cudaDeviceSynchronize());
  return out;
}

void SymmetricContext::prime_loopback() {
  CS_ASSERT_TRUE(loopback_ != nullptr, "prime_loopback is for contexts made by create_loopback_contexts");
  // "already set" for every epoch this context will use: flags are compared as signed distances
  std::vector<uint32_t> words(kFlagWords, 0);
  constexpr uint32_t kSet = 0x3fffffffu;
  for (int i = 0; i < kernels::kChannelBase; ++i) words[i] = kSet;  // stand-alone barrier slots
  for (int c = 0; c < kernels::kNumChannels; ++c) {
    uint32_t *w = words.data() + kernels::kChannelBase + c * kernels::kChannelWords;
    for (int i = 0; i <= 16; ++i) w[i] = kSet;                                            // entry, exit, local go flag
    for (int i = kernels::kChunkFlags; i < kernels::kChunkFlags + 64; ++i) w[i] = kSet;   // chunk-ready flags
    w[17] = channel_blocks[c];  // blocks counted so far: the closing barrier's count stays consistent
  }
  auto stream = static_cast<cudaStream_t>(cur_stream());
  CS_CHECK_CUDART(cudaMemcpyAsync(flags[rank], words.data(), words.size() * sizeof(uint32_t), cudaMemcpyHostToDevice, stream));
  CS_CHECK_CUDART(cudaStreamSynchronize(stream));  // `words` is a local
}

void check_device_status(SymmetricContext &ctx, const char *where) {
  kernels::DeviceStatus st{};
  CS_CHECK_CUDART(cudaMemcpy(&st, ctx.status, sizeof(st), cudaMemcpyDeviceToHost));
  if (st.code == 0) return;
  CS_CHECK_CUDART(cudaMemset(ctx.status, 0, sizeof(st)));
  fail(__FILE__, __LINE__,
       str_cat("device-side wait timed out in ", where, ": code=", st.code, " kernel=", st.kernel_id, " peer/block=", st.block,
               " detail=", st.detail, " (rank ", ctx.rank, ")"));
}

// ------------------------------------------------------------------------ collectives ----
// Every collective below is one kernel launch on the current stream; the barriers are inside the kernels.
bool symmetric_all_reduce(SymmetricContext &ctx, const std::vector<at::Tensor> &ranges, Operation op) {
  for (auto &r : ranges)
    if (!r.is_cuda() || !r.is_contiguous() || dtype_code(r.scalar_type()) < 0 || r.nbytes() % 16 != 0 ||
        (reinterpret_cast<uintptr_t>(r.data_ptr()) & 15))
      return false;
  const float scale = op == kAVG ? 1.0f / static_cast<float>(ctx.size) : 1.0f;
  const auto table = table_of(ctx);
  auto stream = static_cast<cudaStream_t>(cur_stream());
  for (auto &r : ranges) {
    int64_t offset = 0;
    const int dt = dtype_code(r.scalar_type());
    int blocks = 0;
    if (ctx.locate(r.data_ptr(), static_cast<int64_t>(r.nbytes()), &offset)) {
      const auto h = begin_collective(ctx, kernels::kChanAllReduce);
      check(kernels::symm_all_reduce(stream, table, h, offset, r.numel(), dt, scale, &blocks), "symm_all_reduce");
      end_collective(ctx, kernels::kChanAllReduce, blocks);
    } else {
      // Not in the arena: stage the contribution, reduce straight into the destination (every rank sums all copies).
      const SymmetricBlock st = ctx.staging(static_cast<int64_t>(r.nbytes()));
      CS_CHECK_CUDART(cudaMemcpyAsync(ctx.bases[ctx.rank] + st.offset, r.data_ptr(), r.nbytes(), cudaMemcpyDeviceToDevice, stream));
      const auto h = begin_collective(ctx, kernels::kChanReduceScatter);
      check(kernels::symm_reduce_scatter(stream, table, h, st.offset, r.data_ptr(), r.numel(), dt, scale, &blocks),
            "symm_reduce_scatter (one-shot all-reduce)");
      end_collective(ctx, kernels::kChanReduceScatter, blocks);
    }
  }
  return true;
}

bool symmetric_all_gather(SymmetricContext &ctx, const std::vector<std::vector<at::Tensor>> &recv,
                          const std::vector<at::Tensor> &send) {
  for (size_t i = 0; i < send.size(); ++i) {
    if (!send[i].is_cuda() || !send[i].is_contiguous() || send[i].nbytes() % 16 != 0) return false;
    for (auto &r : recv[i])
      if (!r.is_contiguous() || r.nbytes() != send[i].nbytes() || (reinterpret_cast<uintptr_t>(r.data_ptr()) & 15)) return false;
  }
  const auto table = table_of(ctx);
  auto stream = static_cast<cudaStream_t>(cur_stream());
  for (size_t i = 0; i < send.size(); ++i) {
    const int64_t bytes = static_cast<int64_t>(send[i].nbytes());
    // Destination slots that form one block of the arena (slot p at dst + p * bytes, the same offset on every
    // rank) are written by their owners: one multicast store per vector instead of size - 1 pulls.
    int64_t dst_offset = 0;
    bool push = ctx.locate(recv[i][0].data_ptr(), bytes * ctx.size, &dst_offset);
    for (int p = 1; push && p < ctx.size; ++p)
      push = static_cast<const char *>(recv[i][p].data_ptr()) == static_cast<const char *>(recv[i][0].data_ptr()) + p * bytes;
    int blocks = 0;
    if (push) {
      // the source may be any local memory: every rank writes its own shard
      const auto h = begin_collective(ctx, kernels::kChanAllGather);
      check(kernels::symm_all_gather_push(stream, table, h, send[i].data_ptr(), dst_offset, bytes, &blocks), "symm_all_gather_push");
      end_collective(ctx, kernels::kChanAllGather, blocks);
      continue;
    }
    int64_t offset = 0;
    if (!ctx.locate(send[i].data_ptr(), bytes, &offset)) {
      const SymmetricBlock st = ctx.staging(bytes);
      offset = st.offset;
      CS_CHECK_CUDART(cudaMemcpyAsync(ctx.bases[ctx.rank] + offset, send[i].data_ptr(), bytes, cudaMemcpyDeviceToDevice, stream));
    }
    const auto h = begin_collective(ctx, kernels::kChanAllGather);
    {
      kernels::PullCopyArgs a{};
      for (int p = 0; p < ctx.size; ++p) {
        a.src_offset[p] = offset;
        a.dst[p] = static_cast<char *>(recv[i][p].data_ptr());
      }
      a.rows = 1;
      a.row_bytes = bytes;
      a.src_stride = bytes;
      a.dst_stride = bytes;
      check(kernels::symm_pull_copy(stream, table, h, a, &blocks), "symm_pull_copy");
    }
    end_collective(ctx, kernels::kChanAllGather, blocks);
  }
  return true;
}

bool symmetric_reduce_scatter(SymmetricContext &ctx, const std::vector<at::Tensor> &recv,
                              const std::vector<std::vector<at::Tensor>> &send, Operation op) {
  for (size_t i = 0; i < recv.size(); ++i) {
    if (!recv[i].is_cuda() || !recv[i].is_contiguous() || dtype_code(recv[i].scalar_type()) < 0 || recv[i].nbytes() % 16 != 0 ||
        (reinterpret_cast<uintptr_t>(recv[i].data_ptr()) & 15))
      return false;
    for (auto &s : send[i])
      if (!s.is_contiguous() || s.nbytes() != recv[i].nbytes() || s.scalar_type() != recv[i].scalar_type()) return false;
  }
  const float scale = op == kAVG ? 1.0f / static_cast<float>(ctx.size) : 1.0f;
  const auto table = table_of(ctx);
  auto stream = static_cast<cudaStream_t>(cur_stream());
  for (size_t i = 0; i < recv.size(); ++i) {
    const int64_t chunk = static_cast<int64_t>(recv[i].nbytes());
    // Contiguous send chunks already in the arena are read in place; otherwise stage them.
    int64_t first = 0;
    bool in_place = ctx.locate(send[i][0].data_ptr(), chunk * ctx.size, &first);
    for (int p = 1; in_place && p < ctx.size; ++p)
      in_place = static_cast<const char *>(send[i][p].data_ptr()) == static_cast<const char *>(send[i][0].data_ptr()) + p * chunk;
    int64_t offset = first;
    if (!in_place) {
      const SymmetricBlock st = ctx.staging(chunk * ctx.size);
      offset = st.offset;
      for (int p = 0; p < ctx.size; ++p)
        CS_CHECK_CUDART(cudaMemcpyAsync(ctx.bases[ctx.rank] + offset + p * chunk, send[i][p].data_ptr(), chunk,
                                        cudaMemcpyDeviceToDevice, stream));
    }
    int blocks = 0;
    const auto h = begin_collective(ctx, kernels::kChanReduceScatter);
    check(kernels::symm_reduce_scatter(stream, table, h, offset + ctx.rank * chunk, recv[i].data_ptr(), recv[i].numel(),
                                       dtype_code(recv[i].scalar_type()), scale, &blocks),
          "symm_reduce_scatter");
    end_collective(ctx, kernels::kChanReduceScatter, blocks);
  }
  return true;
}

bool symmetric_all_to_all(SymmetricContext &ctx, const std::vector<at::Tensor> &recv, const std::vector<at::Tensor> &send) {
  // Chunks may be 2-D row-strided views (pack/unpack fused into the transfer) as long as every
  // chunk has the same [rows, row_bytes] and, when read in place, the same row stride.
  auto rows_of = [](const at::Tensor &t) { return t.dim() == 2 ? t.size(0) : 1; };
  auto row_bytes_of = [](const at::Tensor &t) {
    return static_cast<int64_t>((t.dim() == 2 ? t.size(1) : t.numel()) * t.element_size());
  };
  auto row_stride_of = [&](const at::Tensor &t) {
    return t.dim() == 2 ? static_cast<int64_t>(t.stride(0) * t.element_size()) : row_bytes_of(t);
  };
  auto row_major = [](const at::Tensor &t) { return t.dim() == 2 ? t.stride(1) == 1 : t.is_contiguous(); };
  const int64_t rows = rows_of(send[0]), row_bytes = row_bytes_of(send[0]);
  for (int p = 0; p < ctx.size; ++p) {
    if (!send[p].is_cuda() || !row_major(send[p]) || !row_major(recv[p])) return false;
    if (rows_of(send[p]) != rows || rows_of(recv[p]) != rows || row_bytes_of(send[p]) != row_bytes || row_bytes_of(recv[p]) != row_bytes)
      return false;
    if (row_bytes % 16 != 0 || row_stride_of(send[p]) % 16 != 0 || row_stride_of(recv[p]) % 16 != 0) return false;
    if (row_stride_of(recv[p]) != row_stride_of(recv[0])) return false;
    if ((reinterpret_cast<uintptr_t>(recv[p].data_ptr()) | reinterpret_cast<uintptr_t>(send[p].data_ptr())) & 15) return false;
  }
  const auto table = table_of(ctx);
  auto stream = static_cast<cudaStream_t>(cur_stream());
  // Source of the chunk this rank wants from peer p = peer p's send[rank]; it must sit at an
  // offset that is the same on every rank, so either all send chunks are equally strided views
  // of one arena block, or they are packed into the staging block.
  std::vector<int64_t> send_offsets(ctx.size);
  bool in_place = true;
  const int64_t src_stride = row_stride_of(send[0]);
  for (int p = 0; p < ctx.size && in_place; ++p) {
    in_place = row_stride_of(send[p]) == src_stride &&
               ctx.locate(send[p].data_ptr(), (rows - 1) * src_stride + row_bytes, &send_offsets[p]);
  }
  kernels::PullCopyArgs a{};
  a.rows = rows;
  a.row_bytes = row_bytes;
  a.dst_stride = row_stride_of(recv[0]);
  if (in_place) {
    // every rank laid its chunks out identically, so peer p's chunk for us is at our own offset of send[rank]
    a.src_stride = src_stride;
    for (int p = 0; p < ctx.size; ++p) a.src_offset[p] = send_offsets[ctx.rank];
  } else {
    const int64_t chunk = rows * row_bytes;
    const SymmetricBlock st = ctx.staging(chunk * ctx.size);
    for (int p = 0; p < ctx.size; ++p)
      CS_CHECK_CUDART(cudaMemcpy2DAsync(ctx.bases[ctx.rank] + st.offset + p * chunk, row_bytes, send[p].data_ptr(),
                                        row_stride_of(send[p]), row_bytes, rows, cudaMemcpyDeviceToDevice, stream));
    a.src_stride = row_bytes;
    for (int p = 0; p < ctx.size; ++p) a.src_offset[p] = st.offset + ctx.rank * chunk;
  }
  for (int p = 0; p < ctx.size; ++p) a.dst[p] = static_cast<char *>(recv[p].data_ptr());
  int blocks = 0;
  const auto h = begin_collective(ctx, kernels::kChanAllToAll);
  check(kernels::symm_pull_copy(stream, table, h, a, &blocks), "symm_pull_copy");
  end_collective(ctx, kernels::kChanAllToAll, blocks);
  return true;
}
}  // namespace cs::communication
