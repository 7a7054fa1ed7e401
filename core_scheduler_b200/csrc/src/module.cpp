// SPDX-License-Identifier: Apache-2.0
// Module tree, flat parameter arenas, optimizer-module base and checkpoints.
// Reference behaviour studied in src/module/module.cpp:32-220 and
// src/module/optimizer_module.cpp:22-51 of the reference project: depth-first traversal in
// registration order, keys "<module.path>.<parameter>" (a root state therefore yields
// ".weight"), names must be non-empty and dot-free, one state per module.
#include "cs/module.h"

#include <cstring>
#include <fstream>

#include "cs/compute.h"
#include "parquet_io.h"

namespace cs::module {
void clear_gradient(Tensor &grad) {
  if (grad.impl()->persistent) {
    grad.impl()->fresh = true;
  } else {
    grad = Tensor{};
  }
}

void Module::insert_child(std::string name, std::shared_ptr<Module> module) {
  CS_ASSERT_TRUE(!name.empty(), "a submodule name must not be empty");
  CS_ASSERT_TRUE(name.find('.') == std::string::npos, "a submodule name must not contain a dot: `", name, "`");
  CS_ASSERT_TRUE(module != nullptr, "cannot register a null submodule `", name, "`");
  children_.insert(std::move(name), std::move(module));
}

void Module::register_state(std::shared_ptr<State> state) {
  CS_ASSERT_TRUE(state_ == nullptr, "a module holds at most one state");
  state_ = std::move(state);
}

void Module::apply_to_submodules(const std::function<void(const std::string &, const std::shared_ptr<Module> &)> &fn,
                                 const std::string &prefix) const {
  for (auto &child : children_) {
    const std::string name = prefix.empty() ? child.first : prefix + "." + child.first;
    fn(name, child.second);
    child.second->apply_to_submodules(fn, name);
  }
}

void Module::apply(const std::function<void(const std::string &, const Module &)> &fn, const std::string &prefix) const {
  fn(prefix, *this);
  apply_to_submodules([&fn](const std::string &name, const std::shared_ptr<Module> &m) { fn(name, *m); }, prefix);
}

OrderedDict<std::string, std::shared_ptr<State>> Module::named_states() const {
  OrderedDict<std::string, std::shared_ptr<State>> out;
  apply([&out](const std::string &name, const Module &m) {
    if (m.state_) out.insert(name, m.state_);
  });
  return out;
}

namespace {
template <typename Value, typename Getter>
OrderedDict<std::string, Value> collect(const Module &root, bool recurse, Getter getter) {
  OrderedDict<std::string, Value> out;
  auto visit = [&](const std::string &name, const Module &m) {
    if (!m.own_state()) return;
    for (auto &item : getter(*m.own_state())) out.insert(name + "." + item.first, item.second);
  };
  if (recurse) {
    root.apply(visit);
  } else {
    visit(std::string(), root);
  }
  return out;
}
}  // namespace

OrderedDict<std::string, Tensor> Module::named_parameters(bool recurse) const {
  return collect<Tensor>(*this, recurse, [](const State &s) { return s.parameters(); });
}
OrderedDict<std::string, Tensor> Module::named_gradients() const {
  return collect<Tensor>(*this, true, [](const State &s) { return s.gradients(); });
}
OrderedDict<std::string, State::Increment> Module::named_increments() const {
  return collect<State::Increment>(*this, true, [](const State &s) { return s.increments(); });
}

void Module::zero_grad() const {
  apply([](const std::string &, const Module &m) {
    if (m.state_) m.state_->zero_grad();
  });
}

void Module::to(const Scheduler &scheduler, TensorOptions options) const {
  for (auto &item : named_parameters()) {
    Tensor p = item.second;
    submit(scheduler, "cs::module::Module::to", Task::Impl::kMain, Task::Impl::kCompute, {p}, {}, [p, options](const FnTask &) {
      auto &impl = *p.impl();
      impl.tensor = impl.tensor.to(options);
      impl.lp = at::Tensor{};
      impl.lp_t = at::Tensor{};
      impl.persistent = false;
      ++impl.version;
    });
  }
  apply([](const std::string &, const Module &m) {
    if (!m.state_) return;
    for (auto &g : m.state_->gradients()) g.second.impl()->persistent = false;
    m.state_->zero_grad();
  });
}

// ------------------------------------------------------------------------- flat arenas ----
std::shared_ptr<FlatParameters> flatten_parameters(const Scheduler &scheduler, const Module &module,
                                                   const FlattenOptions &options) {
  auto flat = std::make_shared<FlatParameters>();
  auto params = module.named_parameters();
  auto grads = module.named_gradients();
  CS_ASSERT_TRUE(params.size() > 0, "nothing to flatten");
  // Slots: one per distinct parameter handle (tied weights share an Impl and get one slot).
  std::unordered_map<const void *, size_t> seen;
  int64_t offset = 0;
  at::ScalarType dtype = at::kFloat;
  bool first = true;
  std::vector<Tensor> param_handles, grad_handles;
  // layout order: the names of options.first(), then everything else in the module's order
  std::vector<std::pair<std::string, Tensor>> ordered;
  {
    std::unordered_map<std::string, size_t> rank_of;
    for (size_t i = 0; i < options.first().size(); ++i) rank_of.emplace(options.first()[i], i);
    std::vector<std::pair<std::string, Tensor>> head(options.first().size()), tail;
    std::vector<bool> found(options.first().size(), false);
    for (auto &item : params) {
      auto it = rank_of.find(item.first);
      if (it == rank_of.end()) {
        tail.emplace_back(item.first, item.second);
      } else {
        head[it->second] = {item.first, item.second};
        found[it->second] = true;
      }
    }
    for (size_t i = 0; i < head.size(); ++i) {
      CS_ASSERT_TRUE(found[i], "flatten_parameters: `", options.first()[i], "` is not a parameter of the module");
      ordered.push_back(head[i]);
    }
    for (auto &t : tail) ordered.push_back(t);
  }
  for (auto &item : ordered) {
    item.second.wait();
    const at::Tensor &t = item.second.impl()->tensor;
    CS_ASSERT_TRUE(t.defined(), "parameter `", item.first, "` is not initialised yet");
    if (first) {
      dtype = t.scalar_type();
      first = false;
    }
    CS_ASSERT_TRUE(t.scalar_type() == dtype, "flat arenas need a single parameter dtype");
    if (seen.count(item.second.impl().get())) continue;
    seen.emplace(item.second.impl().get(), flat->slots.size());
    flat->slots.push_back({item.first, offset, t.numel(), t.dim() == 2});
    param_handles.push_back(item.second);
    grad_handles.push_back(grads[item.first]);
    offset += (t.numel() + FlatParameters::alignment - 1) / FlatParameters::alignment * FlatParameters::alignment;
  }
  const int64_t pad = std::max<int64_t>(1, options.pad_total_to());
  flat->total = (offset + pad - 1) / pad * pad;
  flat->grad_handles = grad_handles;

  std::vector<Tensor> outs{flat->params, flat->grads};
  const bool want_lp = options.lp_dtype().has_value() && *options.lp_dtype() != dtype;
  if (want_lp) {
    outs.push_back(flat->lp);
    if (options.transposed_copies()) outs.push_back(flat->lp_t);
  }
  for (auto &p : param_handles) outs.push_back(p);
  for (auto &g : grad_handles) outs.push_back(g);
  submit(scheduler, "cs::module::flatten_parameters", Task::Impl::kMain, Task::Impl::kCompute, outs, {},
         [flat, param_handles, grad_handles, dtype, want_lp, lp_dtype = options.lp_dtype().value_or(at::kBFloat16),
          transposed = options.transposed_copies(), device = scheduler.device(),
          alloc = options.arena_allocator()](const FnTask &) {
           auto opts = at::TensorOptions().device(device).dtype(dtype);
           auto arena = [&](at::ScalarType dt) {
             if (!alloc) return at::zeros({flat->total}, opts.dtype(dt));
             at::Tensor raw = alloc(flat->total * static_cast<int64_t>(c10::elementSize(dt)));
             at::Tensor typed = raw.view(dt);
             typed.zero_();
             return typed;
           };
           at::Tensor P = at::zeros({flat->total}, opts);
           at::Tensor G = arena(dtype);
           at::Tensor L, LT;
           if (want_lp) {
             L = arena(lp_dtype);
             if (transposed) LT = at::zeros({flat->total}, opts.dtype(lp_dtype));
           }
           for (size_t i = 0; i < flat->slots.size(); ++i) {
             const auto &slot = flat->slots[i];
             auto &pi = *param_handles[i].impl();
             const auto sizes = pi.tensor.sizes().vec();
             at::Tensor view = P.narrow(0, slot.offset, slot.numel).view(sizes);
             view.copy_(pi.tensor);
             pi.tensor = view;
             ++pi.version;
             auto &gi = *grad_handles[i].impl();
             gi.tensor = G.narrow(0, slot.offset, slot.numel).view(sizes);
             gi.persistent = true;
             gi.fresh = true;
             if (want_lp) {
               pi.lp = L.narrow(0, slot.offset, slot.numel).view(sizes);
               pi.lp.copy_(view);
               pi.lp_version = pi.version;
               if (transposed && slot.matrix) {
                 pi.lp_t = LT.narrow(0, slot.offset, slot.numel).view({sizes[1], sizes[0]});
                 pi.lp_t.copy_(view.t());
                 pi.lp_t_version = pi.version;
               }
             }
           }
           flat->params.impl()->tensor = P;
           flat->grads.impl()->tensor = G;
           if (want_lp) {
             flat->lp.impl()->tensor = L;
             if (transposed) flat->lp_t.impl()->tensor = LT;
           }
         });
  return flat;
}

// --------------------------------------------------------------------- optimizer module ----
const Module *OptimizerModule::model() const {
  if (auto sp = module_.lock()) return sp.get();
  return module_raw_;
}
void OptimizerModule::set_lr(double lr) const {
  for (auto &s : states_) s.second->set_lr(lr);
}
double OptimizerModule::get_lr() const {
  CS_ASSERT_TRUE(states_.size() > 0, "optimizer has no state");
  return states_.begin()->second->get_lr();
}
void OptimizerModule::zero_grad(const Scheduler &) const {
  const Module *m = model();
  CS_ASSERT_TRUE(m != nullptr, "the optimised module is gone");
  m->zero_grad();
}
void OptimizerModule::to(const Scheduler &scheduler, TensorOptions options) {
  for (auto &item : named_state_tensors()) {
    Tensor t = item.second;
    submit(scheduler, "cs::module::OptimizerModule::to", Task::Impl::kAssist, Task::Impl::kCompute, {t}, {},
           [t, options](const FnTask &) {
             if (t.impl()->tensor.defined()) t.impl()->tensor = t.impl()->tensor.to(options);
           });
  }
}
}  // namespace cs::module

// ---------------------------------------------------------------------------- checkpoint ----
namespace cs {
void save_tensors(const OrderedDict<std::string, at::Tensor> &tensors, const std::string &path) {
  std::vector<std::string> keys;
  std::vector<at::Tensor> host;  // keeps the fp32 CPU copies alive while Arrow reads them
  std::vector<const float *> data;
  std::vector<int64_t> lengths;
  for (auto &item : tensors) {
    keys.push_back(item.first);
    host.push_back(item.second.detach().to(at::kCPU, at::kFloat).contiguous().view({-1}));
    data.push_back(host.back().data_ptr<float>());
    lengths.push_back(host.back().numel());
  }
  io::write_float_list_table(path, keys, data, lengths);
}

OrderedDict<std::string, at::Tensor> load_tensors(const std::string &path) {
  auto table = io::read_float_list_table(path);
  OrderedDict<std::string, at::Tensor> out;
  for (size_t i = 0; i < table.keys.size(); ++i) {
    at::Tensor t = at::empty({static_cast<int64_t>(table.values[i].size())}, at::kFloat);
    std::memcpy(t.data_ptr<float>(), table.values[i].data(), table.values[i].size() * sizeof(float));
    out.insert(table.keys[i], t);
  }
  return out;
}

void save(const module::Module &module, const std::string &path) {
  OrderedDict<std::string, at::Tensor> tensors;
  for (auto &item : module.named_parameters()) {
    item.second.wait();  // the last writer (init, optimizer step, load) must have finished
    tensors.insert(item.first, item.second.impl()->tensor);
  }
  save_tensors(tensors, path);
}

void load(const module::Module &module, const std::string &path) {
  auto table = load_tensors(path);
  auto params = module.named_parameters();
  for (auto &item : table) {
    auto *p = params.find(item.first);
    CS_ASSERT_TRUE(p != nullptr, "checkpoint key `", item.first, "` does not name a parameter of this module");
    p->wait();
    auto &impl = *p->impl();
    CS_ASSERT_TRUE(impl.tensor.numel() == item.second.numel(), "checkpoint entry `", item.first, "` has ",
                   item.second.numel(), " values, the parameter has ", impl.tensor.numel());
    impl.tensor.copy_(item.second.view(impl.tensor.sizes()));
    ++impl.version;
  }
}

void save(const module::OptimizerModule &optimizer, const std::string &path) {
  OrderedDict<std::string, at::Tensor> tensors;
  for (auto &item : optimizer.named_state_tensors()) {
    item.second.wait();
    tensors.insert(item.first, item.second.impl()->tensor);
  }
  tensors.insert("__step__", at::full({1}, static_cast<double>(optimizer.step_count()), at::kFloat));
  tensors.insert("__lr__", at::full({1}, optimizer.get_lr(), at::kFloat));
  save_tensors(tensors, path);
}

void load(module::OptimizerModule &optimizer, const std::string &path) {
  auto table = load_tensors(path);
  auto states = optimizer.named_state_tensors();
  for (auto &item : table) {
    if (item.first == "__step__") {
      optimizer.set_step_count(static_cast<int64_t>(item.second.item<float>()));
      continue;
    }
    if (item.first == "__lr__") {
      optimizer.set_lr(item.second.item<float>());
      continue;
    }
    auto *t = states.find(item.first);
    CS_ASSERT_TRUE(t != nullptr, "optimizer checkpoint key `", item.first, "` is unknown");
    t->wait();
    auto &impl = *t->impl();
    impl.tensor.copy_(item.second.view(impl.tensor.sizes()));
  }
}
}  // namespace cs
