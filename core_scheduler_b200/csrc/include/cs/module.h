// SPDX-License-Identifier: Apache-2.0
// Stateful module layer: parameter-owning op states, the module tree with dotted parameter
// names, optimizer modules and Parquet checkpoints.
//
// Capability parity: include/module/state.h:28-52, include/module/module.h:27-108,
// include/module/pimpl.h:21-30, include/module/optimizer_module.h:29-59,
// include/module/{linear,gelu_linear,layer_norm,embedding,adamw}.h (reference project paths).
//
// Additions: flatten_parameters() re-homes every parameter, gradient and low-precision
// working copy of a tree into contiguous arenas (one fused optimizer launch, contiguous
// collective buckets, 16-byte aligned TMA bases); save/load also cover optimizer state and
// training metadata in side files, leaving the model file layout untouched.
#pragma once
#include <map>
#include <unordered_map>

#include "cs/core.h"

namespace cs {
// Insertion-ordered string-keyed dictionary (the subset of torch::OrderedDict the API needs).
template <typename Key, typename Value>
class OrderedDict {
 public:
  struct Item {
    Key first;
    Value second;
    const Key &key() const { return first; }
    Value &value() { return second; }
    const Value &value() const { return second; }
    std::pair<Key, Value> pair() const { return {first, second}; }
  };
  Value &insert(Key key, Value value) {
    CS_ASSERT_TRUE(index_.find(key) == index_.end(), "key `", key, "` already present");
    index_.emplace(key, items_.size());
    items_.push_back(Item{std::move(key), std::move(value)});
    return items_.back().second;
  }
  [[nodiscard]] bool contains(const Key &key) const { return index_.find(key) != index_.end(); }
  Value *find(const Key &key) {
    auto it = index_.find(key);
    return it == index_.end() ? nullptr : &items_[it->second].second;
  }
  const Value *find(const Key &key) const {
    auto it = index_.find(key);
    return it == index_.end() ? nullptr : &items_[it->second].second;
  }
  Value &operator[](const Key &key) {
    auto *v = find(key);
    CS_ASSERT_TRUE(v != nullptr, "key `", key, "` is not defined");
    return *v;
  }
  const Value &operator[](const Key &key) const {
    auto *v = find(key);
    CS_ASSERT_TRUE(v != nullptr, "key `", key, "` is not defined");
    return *v;
  }
  [[nodiscard]] size_t size() const { return items_.size(); }
  [[nodiscard]] bool is_empty() const { return items_.empty(); }
  auto begin() { return items_.begin(); }
  auto end() { return items_.end(); }
  auto begin() const { return items_.begin(); }
  auto end() const { return items_.end(); }
  [[nodiscard]] std::vector<Key> keys() const {
    std::vector<Key> k;
    for (auto &i : items_) k.push_back(i.first);
    return k;
  }
  [[nodiscard]] std::vector<Value> values() const {
    std::vector<Value> v;
    for (auto &i : items_) v.push_back(i.second);
    return v;
  }

 private:
  std::vector<Item> items_;
  std::unordered_map<Key, size_t> index_;
};
}  // namespace cs

namespace cs::module {
struct CS_API OptimizerState {
  virtual ~OptimizerState() = default;
  virtual void set_lr(double lr) const = 0;
  [[nodiscard]] virtual double get_lr() const = 0;
};

// What a parameter-owning op exposes to the module tree and the optimizer.
struct CS_API State {
  struct Increment {
    Tensor parameter;
    Tensor gradient;
  };
  virtual ~State() = default;
  [[nodiscard]] virtual OrderedDict<std::string, Tensor> parameters() const = 0;
  [[nodiscard]] virtual OrderedDict<std::string, Tensor> gradients() const = 0;
  [[nodiscard]] virtual OrderedDict<std::string, Increment> increments() const = 0;
  virtual void zero_grad() = 0;
};

// Drops a gradient slot (set-to-none) unless it is arena-backed, in which case the slot is
// only marked fresh so the next backward overwrites it.
CS_API void clear_gradient(Tensor &grad);

struct CS_API Module {
  virtual ~Module() = default;

  void apply_to_submodules(const std::function<void(const std::string &, const std::shared_ptr<Module> &)> &fn,
                           const std::string &prefix = std::string()) const;
  void apply(const std::function<void(const std::string &, const Module &)> &fn,
             const std::string &prefix = std::string()) const;

  void register_state(std::shared_ptr<State> state);

  template <typename M>
  std::shared_ptr<M> register_module(std::string name, std::shared_ptr<M> module) {
    insert_child(std::move(name), module);
    return module;
  }
  template <typename Holder, typename = decltype(std::declval<Holder>().ptr())>
  auto register_module(std::string name, const Holder &holder) {
    return register_module(std::move(name), holder.ptr());
  }

  [[nodiscard]] OrderedDict<std::string, std::shared_ptr<State>> named_states() const;
  [[nodiscard]] OrderedDict<std::string, Tensor> named_parameters(bool recurse = true) const;
  [[nodiscard]] OrderedDict<std::string, Tensor> named_gradients() const;
  [[nodiscard]] OrderedDict<std::string, State::Increment> named_increments() const;
  [[nodiscard]] const OrderedDict<std::string, std::shared_ptr<Module>> &children() const { return children_; }
  [[nodiscard]] const std::shared_ptr<State> &own_state() const { return state_; }

  void zero_grad() const;
  // Moves/casts every parameter (and drops gradients); optimizer states created before the
  // call must be re-created.
  void to(const Scheduler &scheduler, TensorOptions options) const;

 private:
  void insert_child(std::string name, std::shared_ptr<Module> module);
  OrderedDict<std::string, std::shared_ptr<Module>> children_;
  std::shared_ptr<State> state_;
};

// shared_ptr-backed value-semantics handle, `Name x{args...}; x->forward(...)`.
template <typename ImplT>
class ModuleHolder {
 public:
  using ContainedType = ImplT;
  ModuleHolder() = default;
  /* implicit */ ModuleHolder(std::nullptr_t) {}
  /* implicit */ ModuleHolder(std::shared_ptr<ImplT> impl) : impl_{std::move(impl)} {}
  template <typename Head, typename... Tail,
            typename = std::enable_if_t<!(std::is_same_v<std::decay_t<Head>, ModuleHolder> && sizeof...(Tail) == 0) &&
                                        !std::is_same_v<std::decay_t<Head>, std::shared_ptr<ImplT>> &&
                                        !std::is_same_v<std::decay_t<Head>, std::nullptr_t>>>
  explicit ModuleHolder(Head &&head, Tail &&...tail)
      : impl_{std::make_shared<ImplT>(std::forward<Head>(head), std::forward<Tail>(tail)...)} {}
  ImplT *operator->() const { return get(); }
  ImplT &operator*() const { return *get(); }
  [[nodiscard]] const std::shared_ptr<ImplT> &ptr() const {
    CS_ASSERT_TRUE(impl_ != nullptr, "accessing an empty module holder");
    return impl_;
  }
  [[nodiscard]] ImplT *get() const {
    CS_ASSERT_TRUE(impl_ != nullptr, "accessing an empty module holder");
    return impl_.get();
  }
  [[nodiscard]] bool is_empty() const { return impl_ == nullptr; }
  explicit operator bool() const { return impl_ != nullptr; }

 private:
  std::shared_ptr<ImplT> impl_;
};

#define CS_MODULE_IMPL(Name, ImplType)                         \
  class Name : public ::cs::module::ModuleHolder<ImplType> {   \
   public:                                                     \
    using ::cs::module::ModuleHolder<ImplType>::ModuleHolder;  \
    using Impl = ImplType;                                     \
  }
#define CS_MODULE(Name) CS_MODULE_IMPL(Name, Name##Impl)

// ---------------------------------------------------------------------------------------
// Flat parameter arenas
// ---------------------------------------------------------------------------------------
struct CS_API FlatParameters {
  struct Slot {
    std::string key;
    int64_t offset;   // in elements, multiple of `alignment`
    int64_t numel;
    bool matrix;      // 2-D parameter (gets low-precision copies when requested)
  };
  Tensor params;      // fp32 (or the parameter dtype) master values, 1-D
  Tensor grads;       // same dtype/size, 1-D
  Tensor lp;          // low-precision working copies (undefined when not requested)
  Tensor lp_t;        // transposed low-precision copies of the 2-D parameters
  std::vector<Slot> slots;
  std::vector<Tensor> grad_handles;  // gradient slot of each entry of `slots`
  int64_t total{0};
  static constexpr int64_t alignment = 128;  // elements; keeps every slot 256-byte aligned in bf16
};

struct FlattenOptions {
  FlattenOptions() {}
  // When set, gradient and low-precision arenas are taken from this allocator (used to place
  // them in peer-mapped symmetric memory): (bytes) -> 1-D uint8 tensor of that many bytes.
  CS_ARG(std::function<at::Tensor(int64_t)>, arena_allocator) = {};
  CS_ARG(optional<at::ScalarType>, lp_dtype) = {};  // e.g. kBFloat16 for mixed precision
  CS_ARG(bool, transposed_copies) = false;          // only needed by consumers that want W^T laid out K-major
  CS_ARG(int64_t, pad_total_to) = 1;                // pad arena length (e.g. world size * 128 for sharding)
  // Parameter names laid out first, in this order, ahead of the others (which keep the module's order). A group of
  // parameters that is communicated or updated together then forms ONE contiguous range of each arena.
  CS_ARG(std::vector<std::string>, first) = {};
};

// Re-homes all parameters of `module` into one contiguous buffer (values preserved), makes
// every gradient slot a persistent view of a second buffer, and optionally creates
// low-precision working copies. Parameters shared by two states (tied weights) get one slot.
CS_API std::shared_ptr<FlatParameters> flatten_parameters(const Scheduler &scheduler, const Module &module,
                                                         const FlattenOptions &options = {});

// ---------------------------------------------------------------------------------------
// Optimizer modules
// ---------------------------------------------------------------------------------------
struct CS_API OptimizerModule {
  virtual ~OptimizerModule() = default;
  [[nodiscard]] const OrderedDict<std::string, std::shared_ptr<OptimizerState>> &named_states() const { return states_; }
  void set_lr(double lr) const;
  [[nodiscard]] double get_lr() const;
  virtual void step(const Scheduler &scheduler) = 0;
  void zero_grad(const Scheduler &scheduler) const;
  virtual void to(const Scheduler &scheduler, TensorOptions options);
  // Named tensors that make up the optimizer state (for checkpoints).
  [[nodiscard]] virtual OrderedDict<std::string, Tensor> named_state_tensors() const { return {}; }
  [[nodiscard]] virtual int64_t step_count() const { return 0; }
  virtual void set_step_count(int64_t) {}

 protected:
  void bind(const std::shared_ptr<Module> &module) { module_ = module; }
  void bind(const Module *module) { module_raw_ = module; }
  [[nodiscard]] const Module *model() const;
  OrderedDict<std::string, std::shared_ptr<OptimizerState>> states_;
  std::weak_ptr<Module> module_;
  const Module *module_raw_{nullptr};
};
}  // namespace cs::module

namespace cs {
// Model checkpoint: one Parquet file, columns `key: utf8`, `value: list<item: float32>`, one
// row per named parameter (dotted names), values flattened to fp32.
CS_API void save(const module::Module &module, const std::string &path);
CS_API void load(const module::Module &module, const std::string &path);
template <typename ImplT>
void save(const module::ModuleHolder<ImplT> &holder, const std::string &path) { save(*holder, path); }
template <typename ImplT>
void load(const module::ModuleHolder<ImplT> &holder, const std::string &path) { load(*holder, path); }

// Optimizer checkpoint (same two-column layout; keys `<param>.m`, `<param>.v`, ... plus the
// scalar row `__step__`).
CS_API void save(const module::OptimizerModule &optimizer, const std::string &path);
CS_API void load(module::OptimizerModule &optimizer, const std::string &path);

// Generic named-tensor table in the checkpoint layout (used by both overloads above).
CS_API void save_tensors(const OrderedDict<std::string, at::Tensor> &tensors, const std::string &path);
CS_API OrderedDict<std::string, at::Tensor> load_tensors(const std::string &path);
}  // namespace cs
