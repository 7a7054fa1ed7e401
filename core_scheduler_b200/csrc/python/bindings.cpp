// SPDX-License-Identifier: Apache-2.0
// Python bindings of the C++ framework (module core_scheduler_b200._C). The Python layer adds
// no behaviour of its own to these calls: tests, the benchmark and the examples drive the same
// C++ objects a C++ program would.
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/GroupRegistry.hpp>
#include <torch/csrc/distributed/c10d/ProcessGroup.hpp>
#include <torch/extension.h>
#include <c10/cuda/CUDAStream.h>

#include "cs/communication.h"
#include "cs/compute.h"
#include "cs/core.h"
#include "cs/data.h"
#include "cs/models.h"
#include "cs/modules.h"
#include "cs/observability.h"
#include "cs/optimizer.h"
#include "cs/parallel.h"
#include "cs/symmetric.h"
#include "src/vmm.h"
#include "src/symm_internal.h"
#include "kernels/collectives.h"
#include "kernels/api.h"

namespace py = pybind11;
using namespace cs;

namespace {
struct AutocastCtx {
  Scheduler scheduler;
  at::ScalarType dtype;
  std::unique_ptr<autocast::ContextGuard> guard;
};

template <typename Dict>
py::dict tensor_dict(const Dict &d) {
  py::dict out;
  for (auto &item : d) out[py::str(item.first)] = item.second;
  return out;
}

// The group is looked up by name in libtorch's process-group registry (torch.distributed registers
// every group it creates), which avoids sharing pybind11 type registrations with torch._C.
communication::Comm comm_from_process_group(const std::string &group_name, const std::string &device, bool nvp2p) {
  auto pg = c10d::resolve_process_group(group_name);
  const bool cuda = device == "cuda";
  auto backend = pg->getBackend(cuda ? c10::DeviceType::CUDA : c10::DeviceType::CPU);
  auto type = cuda ? (nvp2p ? communication::kNVP2P : communication::kNCCL) : communication::kGLOO;
  return communication::wrap_backend(backend, pg->getRank(), pg->getSize(), type, pg->getStore());
}
}  // namespace

PYBIND11_MODULE(_C, m) {
  m.doc() = "core_scheduler_b200 native runtime";
  py::register_exception<cs::Error>(m, "Error", PyExc_RuntimeError);

  // ---- core ------------------------------------------------------------------------------
  py::class_<ReadOnlyTensor>(m, "ReadOnlyTensor")
      .def(py::init<>())
      .def("defined", &ReadOnlyTensor::defined)
      .def("wait", &ReadOnlyTensor::wait, py::call_guard<py::gil_scoped_release>())
      .def("reset", &ReadOnlyTensor::reset)
      .def("numel", &ReadOnlyTensor::numel)
      .def("sizes", [](const ReadOnlyTensor &t) { return t.sizes().vec(); })
      .def("raw", [](const ReadOnlyTensor &t) { return t.impl()->tensor; },
           "the underlying torch tensor without any synchronisation")
      .def("companion", [](const ReadOnlyTensor &t) { return t.impl()->companion; })
      .def("stream_class", [](const ReadOnlyTensor &t) { return static_cast<int>(t.impl()->stream_class); })
      .def("version", [](const ReadOnlyTensor &t) { return t.impl()->version; })
      .def("lp", [](const ReadOnlyTensor &t) { return t.impl()->lp; })
      .def("lp_t", [](const ReadOnlyTensor &t) { return t.impl()->lp_t; })
      .def("is_persistent", [](const ReadOnlyTensor &t) { return t.impl()->persistent; })
      .def("is_fresh", [](const ReadOnlyTensor &t) { return t.impl()->fresh; });
  py::class_<Tensor, ReadOnlyTensor>(m, "Tensor")
      .def(py::init<>())
      .def_static("wrap", &Tensor::wrap)
      .def("set_raw", [](Tensor &t, at::Tensor v) {
        t.impl()->tensor = std::move(v);
        ++t.impl()->version;
      });
  m.def("from_torch", &Tensor::wrap);
  m.def("manual_seed", &cs::manual_seed);
  m.def("event_pool_size", &Event::pooled);
  m.def("kernel_launch_count", &cs::kernels::launch_count);
  m.def("gemm_status", [] {
    cs::kernels::DeviceStatus st{};
    cs::kernels::gemm_status(&st);
    return std::vector<int>{st.code, st.kernel_id, st.block, st.detail};
  });
  m.def("gemm_status_reset", [] { cs::kernels::gemm_status_reset(); });
  // Raw access to the tcgen05 GEMM for kernel tests and microbenchmarks (current torch stream).
  m.def("gemm_bf16",
        [](const at::Tensor &a, const at::Tensor &b, at::Tensor d, int layout, int epilogue, py::object aux, py::object bias,
           py::object d2, py::object stats, int64_t n_valid) {
          cs::kernels::GemmArgs g{};
          g.a = a.data_ptr();
          g.b = b.data_ptr();
          g.d = d.data_ptr();
          at::Tensor aux_t, bias_t, d2_t, stats_t;
          if (!aux.is_none()) { aux_t = py::cast<at::Tensor>(aux); g.aux = aux_t.data_ptr(); }
          if (!bias.is_none()) { bias_t = py::cast<at::Tensor>(bias); g.bias = bias_t.data_ptr(); }
          if (!d2.is_none()) { d2_t = py::cast<at::Tensor>(d2); g.d2 = d2_t.data_ptr(); }
          if (!stats.is_none()) { stats_t = py::cast<at::Tensor>(stats); g.stats = stats_t.data_ptr<float>(); }
          g.layout = layout;
          g.epilogue = epilogue;
          if (layout == cs::kernels::kTN) {
            g.m = a.size(0); g.k = a.size(1); g.n = b.size(0);
            g.lda = a.stride(0); g.ldb = b.stride(0);
          } else if (layout == cs::kernels::kNT) {
            g.k = a.size(0); g.m = a.size(1); g.n = b.size(1);
            g.lda = a.stride(0); g.ldb = b.stride(0);
          } else {
            g.m = a.size(0); g.k = a.size(1); g.n = b.size(1);
            g.lda = a.stride(0); g.ldb = b.stride(0);
          }
          g.ldd = d.stride(0);
          g.n_valid = n_valid;
          return cs::kernels::gemm_bf16(c10::cuda::getCurrentCUDAStream().stream(), g);
        },
        py::arg("a"), py::arg("b"), py::arg("d"), py::arg("layout") = 0, py::arg("epilogue") = 0, py::arg("aux") = py::none(),
        py::arg("bias") = py::none(), py::arg("d2") = py::none(), py::arg("stats") = py::none(), py::arg("n_valid") = -1);
  m.def("gemm_ce_stat_tiles", &cs::kernels::gemm_ce_stat_tiles);
  // Raw access to the tcgen05 attention forward kernel (current torch stream).
  m.def("attention_forward_tcgen05", [](const at::Tensor &qkv, int64_t heads, double scale, bool causal) {
    const int64_t B = qkv.size(0), T = qkv.size(1), D = qkv.size(2) / (3 * heads);
    at::Tensor out = at::empty({B, T, heads * D}, qkv.options());
    at::Tensor lse = at::empty({B, heads, T}, qkv.options().dtype(at::kFloat));
    const int rc = cs::kernels::attention_forward_packed(c10::cuda::getCurrentCUDAStream().stream(), qkv.data_ptr(), out.data_ptr(),
                                                        lse.data_ptr<float>(), B, T, heads, D, static_cast<float>(scale), causal ? 1 : 0);
    return py::make_tuple(rc, out, lse);
  }, py::arg("qkv"), py::arg("heads"), py::arg("scale"), py::arg("causal") = true);
  m.def("attention_backward_tcgen05", [](const at::Tensor &qkv, const at::Tensor &out, const at::Tensor &dout, const at::Tensor &lse,
                                         int64_t heads, double scale, bool causal) {
    const int64_t B = qkv.size(0), T = qkv.size(1), D = qkv.size(2) / (3 * heads);
    at::Tensor dqkv = at::empty_like(qkv);
    at::Tensor delta = at::empty({3, B, heads, T}, qkv.options().dtype(at::kFloat));
    const int rc = cs::kernels::attention_backward_packed(c10::cuda::getCurrentCUDAStream().stream(), qkv.data_ptr(), out.data_ptr(),
                                                          dout.data_ptr(), lse.data_ptr<float>(), delta.data_ptr<float>(),
                                                          dqkv.data_ptr(), B, T, heads, D, static_cast<float>(scale), causal ? 1 : 0);
    CS_ASSERT_TRUE(rc == 0, "attention_backward_packed returned ", rc);
    return py::make_tuple(dqkv, delta.select(0, 0));
  }, py::arg("qkv"), py::arg("out"), py::arg("dout"), py::arg("lse"), py::arg("heads"), py::arg("scale"), py::arg("causal") = true);
  m.def("bounds_check_enabled", &cs::kernels::bounds_check_enabled);
  m.def("bounds_report", [](bool reset) {
    cs::kernels::BoundsReport r{};
    const int rc = cs::kernels::bounds_report(&r, reset);
    CS_ASSERT_TRUE(rc == 0, "bounds_report failed: ", rc);
    return py::make_tuple(r.code, r.kernel_id, r.block, r.thread, static_cast<int64_t>(r.index), static_cast<int64_t>(r.limit));
  }, py::arg("reset") = true, "(code, kernel id, block, thread, index, limit) of the first out-of-range index; code 0 = none");
  m.def("attention_status", [] {
    cs::kernels::DeviceStatus st{};
    cs::kernels::attention_status(&st);
    return std::vector<int>{st.code, st.kernel_id, st.block, st.detail};
  });

  py::class_<TaskTiming>(m, "TaskTiming")
      .def_readonly("name", &TaskTiming::name)
      .def_readonly("stream_class", &TaskTiming::stream_class)
      .def_readonly("device_ms", &TaskTiming::device_ms)
      .def_readonly("start_ms", &TaskTiming::start_ms);

  py::class_<Scheduler>(m, "Scheduler")
      .def("get_device_rank", &Scheduler::get_device_rank)
      .def("device", [](const Scheduler &s) { return s.device().str(); })
      .def("synchronize", [](const Scheduler &s) { s.impl()->synchronize(); }, py::call_guard<py::gil_scoped_release>())
      .def("submitted", [](const Scheduler &s) {
        return std::vector<int64_t>(s.impl()->submitted, s.impl()->submitted + 4);
      })
      .def("set_profiling", [](const Scheduler &s, bool on) { s.impl()->set_profiling(on); })
      .def("drain_timings", [](const Scheduler &s) { return s.impl()->drain_timings(); })
      .def("autocast_enabled", [](const Scheduler &s) { return s.impl()->autocast_enabled; })
      .def("raw_stream", [](const Scheduler &s, int cls) {
        return reinterpret_cast<uintptr_t>(s.impl()->raw_stream(static_cast<StreamClass>(cls)));
      })
      // Test hook: run a Python callable as a task with declared inputs/outputs.
      .def("submit_python",
           [](const Scheduler &s, const std::string &name, int priority, std::vector<Tensor> outs,
              std::vector<ReadOnlyTensor> ins, py::function fn) {
             auto keep = std::make_shared<std::string>(name);
             cs::submit(s, keep->c_str(), static_cast<Task::Impl::Priority>(priority), Task::Impl::kCompute, outs, ins,
                        [fn, keep](const FnTask &) {
                          py::gil_scoped_acquire gil;
                          fn();
                        });
           });
  py::class_<DynamicScheduler, Scheduler>(m, "DynamicScheduler")
      .def(py::init([](int local_rank, const std::string &device, int assist_gap, int comm_gap) {
             DynamicScheduler::Options o;
             o.assist_task_gap(assist_gap).comm_task_gap(comm_gap);
             if (device == "cuda") o.device_type(at::kCUDA);
             if (device == "cpu") o.device_type(at::kCPU);
             return DynamicScheduler(local_rank, o);
           }),
           py::arg("local_rank") = 0, py::arg("device") = "auto", py::arg("assist_task_gap") = 2,
           py::arg("comm_task_gap") = 5);

  py::class_<AutocastCtx>(m, "autocast")
      .def(py::init([](const Scheduler &s, at::ScalarType dtype) { return AutocastCtx{s, dtype, nullptr}; }),
           py::arg("scheduler"), py::arg("dtype") = at::kBFloat16)
      .def("__enter__", [](AutocastCtx &c) { c.guard = std::make_unique<autocast::ContextGuard>(c.scheduler, c.dtype); })
      .def("__exit__", [](AutocastCtx &c, py::object, py::object, py::object) { c.guard.reset(); });

  m.def("to_torch", &memory::to_torch, py::call_guard<py::gil_scoped_release>());
  m.def("allclose",
        [](const ReadOnlyTensor &a, const at::Tensor &b, double rtol, double atol) { return at::allclose(a, b, rtol, atol); },
        py::arg("a"), py::arg("b"), py::arg("rtol") = 1e-5, py::arg("atol") = 1e-8);
  m.def("set_backend", [](const std::string &name) {
    compute::set_backend(name == "library" ? compute::Backend::kLibrary : compute::Backend::kFused);
  });
  m.def("library_fallbacks", &compute::library_fallbacks);
  m.def("get_backend", [] { return compute::get_backend() == compute::Backend::kFused ? "fused" : "library"; });
  m.def("working_copy", [](const Scheduler &s, const Tensor &p, at::ScalarType dt) {
    Tensor out;
    cs::submit(s, "working_copy", Task::Impl::kMain, Task::Impl::kCompute, {out}, {p},
               [out, p, dt](const FnTask &) { out.impl()->tensor = compute::working_copy(p, dt); });
    return out;
  });
  m.def("working_copy_transposed", [](const Scheduler &s, const Tensor &p, at::ScalarType dt) {
    Tensor out;
    cs::submit(s, "working_copy_transposed", Task::Impl::kMain, Task::Impl::kCompute, {out}, {p},
               [out, p, dt](const FnTask &) { out.impl()->tensor = compute::working_copy_transposed(p, dt); });
    return out;
  });

  // ---- module base -------------------------------------------------------------------------
  py::class_<module::State, std::shared_ptr<module::State>>(m, "State")
      .def("parameters", [](const module::State &s) { return tensor_dict(s.parameters()); })
      .def("gradients", [](const module::State &s) { return tensor_dict(s.gradients()); })
      .def("zero_grad", &module::State::zero_grad);
  py::class_<module::Module, std::shared_ptr<module::Module>>(m, "Module")
      .def("named_parameters", [](const module::Module &mod) { return tensor_dict(mod.named_parameters()); })
      .def("named_gradients", [](const module::Module &mod) { return tensor_dict(mod.named_gradients()); })
      .def("parameter_names", [](const module::Module &mod) { return mod.named_parameters().keys(); })
      .def("state_names", [](const module::Module &mod) { return mod.named_states().keys(); })
      .def("zero_grad", &module::Module::zero_grad)
      .def("to", [](const module::Module &mod, const Scheduler &s, at::ScalarType dt) {
        mod.to(s, at::TensorOptions().dtype(dt));
      })
      .def("save", [](const module::Module &mod, const std::string &path) { cs::save(mod, path); })
      .def("load", [](const module::Module &mod, const std::string &path) { cs::load(mod, path); });
  m.def("save", [](const module::Module &mod, const std::string &path) { cs::save(mod, path); });
  m.def("load", [](const module::Module &mod, const std::string &path) { cs::load(mod, path); });

  py::class_<module::FlatParameters, std::shared_ptr<module::FlatParameters>>(m, "FlatParameters")
      .def_readonly("params", &module::FlatParameters::params)
      .def_readonly("grads", &module::FlatParameters::grads)
      .def_readonly("lp", &module::FlatParameters::lp)
      .def_readonly("lp_t", &module::FlatParameters::lp_t)
      .def_readonly("total", &module::FlatParameters::total)
      .def("slots", [](const module::FlatParameters &f) {
        std::vector<std::tuple<std::string, int64_t, int64_t>> out;
        for (auto &s : f.slots) out.emplace_back(s.key, s.offset, s.numel);
        return out;
      });
  m.def("flatten_parameters",
        [](const Scheduler &s, const module::Module &mod, py::object lp_dtype, bool transposed, int64_t pad_to,
           const std::vector<std::string> &first) {
          module::FlattenOptions o;
          if (!lp_dtype.is_none()) o.lp_dtype(py::cast<at::ScalarType>(lp_dtype));
          o.transposed_copies(transposed).pad_total_to(pad_to).first(first);
          return module::flatten_parameters(s, mod, o);
        },
        py::arg("scheduler"), py::arg("module"), py::arg("lp_dtype") = py::none(), py::arg("transposed_copies") = false,
        py::arg("pad_total_to") = 1, py::arg("first") = std::vector<std::string>{});

  // ---- compute ops ---------------------------------------------------------------------------
  using compute::Linear;
  py::class_<Linear::State, module::State, std::shared_ptr<Linear::State>>(m, "LinearState")
      .def_property_readonly("weight", [](const Linear::State &s) { return s.forward.weight; })
      .def_property_readonly("bias", [](const Linear::State &s) { return s.forward.bias; })
      .def_property_readonly("grad_weight", [](const Linear::State &s) { return s.forward.grad_weight; })
      .def_property_readonly("grad_bias", [](const Linear::State &s) { return s.forward.grad_bias; });
  auto linear_opts = [](int64_t in, int64_t out, bool bias, py::object dtype, py::object device, bool gelu) {
    Linear::Options o{in, out};
    o.bias(bias).gelu_epilogue(gelu);
    if (!dtype.is_none()) o.dtype(py::cast<at::ScalarType>(dtype));
    if (!device.is_none()) o.device(py::cast<at::Device>(device));
    return o;
  };
  m.def("linear_init",
        [linear_opts](const Scheduler &s, int64_t in, int64_t out, bool bias, py::object dtype, py::object device, bool gelu) {
          return Linear::init(s, linear_opts(in, out, bias, dtype, device, gelu));
        },
        py::arg("scheduler"), py::arg("in_features"), py::arg("out_features"), py::arg("bias") = true,
        py::arg("dtype") = py::none(), py::arg("device") = py::none(), py::arg("gelu_epilogue") = false);
  m.def("linear_forward", [](const Scheduler &s, const std::shared_ptr<Linear::State> &st, const ReadOnlyTensor &x,
                             py::object residual) {
    if (residual.is_none()) return Linear::forward(s, st, x);
    return Linear::forward(s, st, x, py::cast<ReadOnlyTensor>(residual));
  }, py::arg("scheduler"), py::arg("state"), py::arg("input"), py::arg("residual") = py::none());
  m.def("linear_backward_input", &Linear::backward_input);
  m.def("linear_backward_parameter", &Linear::backward_parameter);

  using compute::GeluLinear;
  py::class_<GeluLinear::State, module::State, std::shared_ptr<GeluLinear::State>>(m, "GeluLinearState")
      .def_property_readonly("weight", [](const GeluLinear::State &s) { return s.forward.weight; })
      .def_property_readonly("bias", [](const GeluLinear::State &s) { return s.forward.bias; })
      .def_property_readonly("grad_weight", [](const GeluLinear::State &s) { return s.forward.grad_weight; })
      .def_property_readonly("grad_bias", [](const GeluLinear::State &s) { return s.forward.grad_bias; });
  m.def("gelu_linear_init",
        [linear_opts](const Scheduler &s, int64_t in, int64_t out, bool bias, py::object dtype, py::object device) {
          return GeluLinear::init(s, linear_opts(in, out, bias, dtype, device, false));
        },
        py::arg("scheduler"), py::arg("in_features"), py::arg("out_features"), py::arg("bias") = true,
        py::arg("dtype") = py::none(), py::arg("device") = py::none());
  m.def("gelu_linear_forward", [](const Scheduler &s, const std::shared_ptr<GeluLinear::State> &st,
                                  const ReadOnlyTensor &x, py::object residual) {
    if (residual.is_none()) return GeluLinear::forward(s, st, x);
    return GeluLinear::forward(s, st, x, py::cast<ReadOnlyTensor>(residual));
  }, py::arg("scheduler"), py::arg("state"), py::arg("input"), py::arg("residual") = py::none());
  m.def("gelu_linear_backward_input", &GeluLinear::backward_input);
  m.def("gelu_linear_backward_parameter", &GeluLinear::backward_parameter);

  using compute::LayerNorm;
  py::class_<LayerNorm::State, module::State, std::shared_ptr<LayerNorm::State>>(m, "LayerNormState")
      .def_property_readonly("weight", [](const LayerNorm::State &s) { return s.forward.weight; })
      .def_property_readonly("bias", [](const LayerNorm::State &s) { return s.forward.bias; })
      .def_property_readonly("grad_weight", [](const LayerNorm::State &s) { return s.forward.grad_weight; })
      .def_property_readonly("grad_bias", [](const LayerNorm::State &s) { return s.forward.grad_bias; });
  m.def("layer_norm_init",
        [](const Scheduler &s, std::vector<int64_t> shape, double eps, py::object dtype, py::object device) {
          LayerNorm::Options o{at::IntArrayRef(shape)};
          o.eps(eps);
          if (!dtype.is_none()) o.dtype(py::cast<at::ScalarType>(dtype));
          if (!device.is_none()) o.device(py::cast<at::Device>(device));
          return LayerNorm::init(s, o);
        },
        py::arg("scheduler"), py::arg("normalized_shape"), py::arg("eps") = 1e-5, py::arg("dtype") = py::none(),
        py::arg("device") = py::none());
  m.def("layer_norm_forward", &LayerNorm::forward);
  m.def("layer_norm_backward", [](const Scheduler &s, const std::shared_ptr<LayerNorm::State> &st,
                                  const ReadOnlyTensor &dy, py::object grad_residual) {
    if (grad_residual.is_none()) return LayerNorm::backward(s, st, dy);
    return LayerNorm::backward(s, st, dy, py::cast<ReadOnlyTensor>(grad_residual));
  }, py::arg("scheduler"), py::arg("state"), py::arg("grad_output"), py::arg("grad_residual") = py::none());

  using compute::GeLU;
  py::class_<GeLU::State, std::shared_ptr<GeLU::State>>(m, "GeLUState");
  m.def("gelu_init", &GeLU::init);
  m.def("gelu_forward", &GeLU::forward);
  m.def("gelu_backward", &GeLU::backward);

  using compute::Embedding;
  py::class_<Embedding::State, module::State, std::shared_ptr<Embedding::State>>(m, "EmbeddingState")
      .def_property_readonly("weight", [](const Embedding::State &s) { return s.forward.weight; })
      .def_property_readonly("grad_weight", [](const Embedding::State &s) { return s.forward.grad_weight; });
  m.def("embedding_init",
        [](const Scheduler &s, int64_t n, int64_t d, py::object padding_idx, py::object dtype, py::object device) {
          Embedding::Options o{n, d};
          if (!padding_idx.is_none()) o.padding_idx(py::cast<int64_t>(padding_idx));
          if (!dtype.is_none()) o.dtype(py::cast<at::ScalarType>(dtype));
          if (!device.is_none()) o.device(py::cast<at::Device>(device));
          return Embedding::init(s, o);
        },
        py::arg("scheduler"), py::arg("num_embeddings"), py::arg("embedding_dim"), py::arg("padding_idx") = py::none(),
        py::arg("dtype") = py::none(), py::arg("device") = py::none());
  m.def("embedding_forward", &Embedding::forward);
  m.def("embedding_backward", &Embedding::backward);
  m.def("embedding_forward_token_position", &Embedding::forward_token_position);
  m.def("embedding_backward_token_position", &Embedding::backward_token_position);

  using compute::CrossEntropy;
  py::class_<CrossEntropy::State, std::shared_ptr<CrossEntropy::State>>(m, "CrossEntropyState");
  m.def("cross_entropy_init",
        [](const Scheduler &s, const std::string &reduction, int64_t ignore_index) {
          CrossEntropy::Options o;
          o.reduction(reduction == "sum" ? compute::Reduction::kSum
                                         : (reduction == "none" ? compute::Reduction::kNone : compute::Reduction::kMean));
          o.ignore_index(ignore_index);
          return CrossEntropy::init(s, o);
        },
        py::arg("scheduler"), py::arg("reduction") = "mean", py::arg("ignore_index") = -100);
  m.def("cross_entropy_forward", &CrossEntropy::forward);
  m.def("cross_entropy_backward", &CrossEntropy::backward);

  using compute::LinearCrossEntropy;
  py::class_<LinearCrossEntropy::State, std::shared_ptr<LinearCrossEntropy::State>>(m, "LinearCrossEntropyState");
  m.def("linear_cross_entropy_init", &LinearCrossEntropy::init, py::arg("scheduler"), py::arg("linear"),
        py::arg("valid_classes") = -1, py::arg("ignore_index") = -100);
  m.def("linear_cross_entropy_forward", &LinearCrossEntropy::forward);
  m.def("linear_cross_entropy_backward", &LinearCrossEntropy::backward);

  using compute::ScaledDotProductAttention;
  py::class_<ScaledDotProductAttention::State, std::shared_ptr<ScaledDotProductAttention::State>>(m, "AttentionState");
  m.def("attention_init",
        [](const Scheduler &s, bool causal, double dropout, py::object scale) {
          ScaledDotProductAttention::Options o;
          o.is_causal(causal).dropout_p(dropout);
          if (!scale.is_none()) o.scale(py::cast<double>(scale));
          return ScaledDotProductAttention::init(s, o);
        },
        py::arg("scheduler"), py::arg("is_causal") = false, py::arg("dropout_p") = 0.0, py::arg("scale") = py::none());
  m.def("attention_forward", &ScaledDotProductAttention::forward);
  m.def("attention_backward", [](const Scheduler &s, const std::shared_ptr<ScaledDotProductAttention::State> &st,
                                 const ReadOnlyTensor &dout) {
    auto r = ScaledDotProductAttention::backward(s, st, dout);
    return std::vector<Tensor>{r[0], r[1], r[2]};
  });
  m.def("attention_forward_packed", &ScaledDotProductAttention::forward_packed);
  m.def("attention_backward_packed", &ScaledDotProductAttention::backward_packed);

  // Utils (the subset tests and examples use from Python; everything is reachable from C++)
  namespace Utils = compute::Utils;
  m.def("utils_sum", [](const Scheduler &s, const ReadOnlyTensor &x, std::vector<int64_t> dim, bool keep) {
    return Utils::sum(s, x, at::IntArrayRef(dim), keep);
  }, py::arg("scheduler"), py::arg("input"), py::arg("dim"), py::arg("keep_dim") = false);
  m.def("utils_cat", &Utils::cat);
  m.def("utils_add", &Utils::add);
  m.def("utils_view", [](const Scheduler &s, const ReadOnlyTensor &x, std::vector<int64_t> size) {
    return Utils::view(s, x, at::IntArrayRef(size));
  });
  m.def("utils_split", &Utils::split);
  m.def("utils_randn", [](const Scheduler &s, std::vector<int64_t> size, at::ScalarType dt) {
    return Utils::randn(s, at::IntArrayRef(size), at::TensorOptions().dtype(dt));
  });
  m.def("utils_rand", [](const Scheduler &s, std::vector<int64_t> size, at::ScalarType dt) {
    return Utils::rand(s, at::IntArrayRef(size), at::TensorOptions().dtype(dt));
  });
  m.def("utils_zeros", [](const Scheduler &s, std::vector<int64_t> size, at::ScalarType dt) {
    return Utils::zeros(s, at::IntArrayRef(size), at::TensorOptions().dtype(dt));
  });
  m.def("utils_ones", [](const Scheduler &s, std::vector<int64_t> size, at::ScalarType dt) {
    return Utils::ones(s, at::IntArrayRef(size), at::TensorOptions().dtype(dt));
  });
  m.def("utils_arange", [](const Scheduler &s, int64_t a, int64_t b) {
    return Utils::arange(s, a, b, at::TensorOptions().dtype(at::kLong));
  });
  m.def("utils_randint", [](const Scheduler &s, int64_t lo, int64_t hi, std::vector<int64_t> size) {
    return Utils::randint(s, lo, hi, at::IntArrayRef(size));
  });
  m.def("utils_broadcast_to", [](const Scheduler &s, const ReadOnlyTensor &x, std::vector<int64_t> size) {
    return Utils::broadcast_to(s, x, at::IntArrayRef(size));
  });
  m.def("utils_clone", &Utils::clone);
  m.def("utils_zero_", &Utils::zero_);
  m.def("utils_normal_", &Utils::normal_);
  m.def("utils_uniform_", &Utils::uniform_);
  m.def("utils_linalg_vector_norm", [](const Scheduler &s, const ReadOnlyTensor &x, double ord) {
    return Utils::linalg_vector_norm(s, x, ord);
  });
  m.def("utils_clip_grad_norm_", &Utils::clip_grad_norm_, py::arg("scheduler"), py::arg("tensors"), py::arg("max_norm"),
        py::arg("norm_type") = 2.0);
  m.def("init_kaiming_uniform_", [](const Scheduler &s, const Tensor &t, double a) { compute::Init::kaiming_uniform_(s, t, a); });
  m.def("init_kaiming_normal_", [](const Scheduler &s, const Tensor &t, double a) { compute::Init::kaiming_normal_(s, t, a); });

  // ---- modules -------------------------------------------------------------------------------
  py::class_<module::LinearImpl, module::Module, std::shared_ptr<module::LinearImpl>>(m, "LinearModule")
      .def(py::init([linear_opts](const Scheduler &s, int64_t in, int64_t out, bool bias, py::object dtype, py::object device) {
             return std::make_shared<module::LinearImpl>(s, linear_opts(in, out, bias, dtype, device, false));
           }),
           py::arg("scheduler"), py::arg("in_features"), py::arg("out_features"), py::arg("bias") = true,
           py::arg("dtype") = py::none(), py::arg("device") = py::none())
      .def("forward", [](const module::LinearImpl &l, const Scheduler &s, const ReadOnlyTensor &x) { return l.forward(s, x); })
      .def("backward", &module::LinearImpl::backward)
      .def("state", &module::LinearImpl::state);
  py::class_<module::LayerNormImpl, module::Module, std::shared_ptr<module::LayerNormImpl>>(m, "LayerNormModule")
      .def(py::init([](const Scheduler &s, int64_t d, py::object dtype) {
             compute::LayerNorm::Options o{d};
             if (!dtype.is_none()) o.dtype(py::cast<at::ScalarType>(dtype));
             return std::make_shared<module::LayerNormImpl>(s, o);
           }),
           py::arg("scheduler"), py::arg("normalized_shape"), py::arg("dtype") = py::none())
      .def("forward", &module::LayerNormImpl::forward)
      .def("backward", [](const module::LayerNormImpl &l, const Scheduler &s, const ReadOnlyTensor &dy) { return l.backward(s, dy); })
      .def("state", &module::LayerNormImpl::state);

  py::class_<module::OptimizerModule, std::shared_ptr<module::OptimizerModule>>(m, "OptimizerModule")
      .def("set_lr", &module::OptimizerModule::set_lr)
      .def("get_lr", &module::OptimizerModule::get_lr)
      .def("step", &module::OptimizerModule::step)
      .def("zero_grad", &module::OptimizerModule::zero_grad)
      .def("state_names", [](const module::OptimizerModule &o) { return o.named_states().keys(); })
      .def("named_state_tensors", [](const module::OptimizerModule &o) { return tensor_dict(o.named_state_tensors()); })
      .def("step_count", &module::OptimizerModule::step_count)
      .def("save", [](const module::OptimizerModule &o, const std::string &p) { cs::save(o, p); })
      .def("load", [](module::OptimizerModule &o, const std::string &p) { cs::load(o, p); });
  py::class_<module::AdamWImpl, module::OptimizerModule, std::shared_ptr<module::AdamWImpl>>(m, "AdamW")
      .def(py::init([](const Scheduler &s, const std::shared_ptr<module::Module> &mod, double lr, double beta1, double beta2,
                       double eps, double wd, bool amsgrad, std::shared_ptr<module::FlatParameters> flat) {
             optimizer::AdamW::Options o;
             o.lr(lr).beta1(beta1).beta2(beta2).eps(eps).weight_decay(wd).amsgrad(amsgrad);
             if (flat) return std::make_shared<module::AdamWImpl>(s, *mod, flat, o);
             return std::make_shared<module::AdamWImpl>(s, mod, o);
           }),
           py::keep_alive<1, 3>(), py::arg("scheduler"), py::arg("module"), py::arg("lr") = 1e-3, py::arg("beta1") = 0.9,
           py::arg("beta2") = 0.999, py::arg("eps") = 1e-8, py::arg("weight_decay") = 1e-2, py::arg("amsgrad") = false,
           py::arg("flat") = nullptr)
      .def("set_grad_scale", &module::AdamWImpl::set_grad_scale)
      .def("set_clip_coefficient", &module::AdamWImpl::set_clip_coefficient);

  py::class_<optimizer::AdamW::State, std::shared_ptr<optimizer::AdamW::State>>(m, "AdamWState")
      .def_property_readonly("m", [](const optimizer::AdamW::State &s) { return s.tensors.m; })
      .def_property_readonly("v", [](const optimizer::AdamW::State &s) { return s.tensors.v; })
      .def_property_readonly("v_max", [](const optimizer::AdamW::State &s) { return s.tensors.v_max; })
      .def("set_lr", &optimizer::AdamW::State::set_lr)
      .def("get_lr", &optimizer::AdamW::State::get_lr);
  auto adamw_opts = [](double lr, double beta1, double beta2, double eps, double wd, bool amsgrad) {
    optimizer::AdamW::Options o;
    o.lr(lr).beta1(beta1).beta2(beta2).eps(eps).weight_decay(wd).amsgrad(amsgrad);
    return o;
  };
  m.def("adamw_init",
        [adamw_opts](const Scheduler &s, const ReadOnlyTensor &p, double lr, double beta1, double beta2, double eps, double wd,
                     bool amsgrad) { return optimizer::AdamW::init(s, p, adamw_opts(lr, beta1, beta2, eps, wd, amsgrad)); },
        py::arg("scheduler"), py::arg("parameter"), py::arg("lr") = 1e-3, py::arg("beta1") = 0.9, py::arg("beta2") = 0.999,
        py::arg("eps") = 1e-8, py::arg("weight_decay") = 1e-2, py::arg("amsgrad") = false);
  m.def("adamw_step", &optimizer::AdamW::step);
  m.def("amp_adamw_step", &optimizer::AmpAdamW::step);

  // ---- models --------------------------------------------------------------------------------
  using models::GPT2Config;
  py::class_<GPT2Config>(m, "GPT2Config")
      .def(py::init([](int64_t n_layer, int64_t n_head, int64_t n_embd, int64_t block_size, int64_t vocab_size,
                       int64_t padded_vocab_size, bool use_bias, at::ScalarType dtype, double init_std,
                       bool fused_classifier, bool scale_residual_init) {
             GPT2Config c;
             c.n_layer(n_layer).n_head(n_head).n_embd(n_embd).block_size(block_size).vocab_size(vocab_size)
                 .padded_vocab_size(padded_vocab_size).use_bias(use_bias).dtype(dtype).init_std(init_std)
                 .fused_classifier(fused_classifier).scale_residual_init(scale_residual_init);
             return c;
           }),
           py::arg("n_layer") = 12, py::arg("n_head") = 12, py::arg("n_embd") = 768, py::arg("block_size") = 1024,
           py::arg("vocab_size") = 50257, py::arg("padded_vocab_size") = 50304, py::arg("use_bias") = false,
           py::arg("dtype") = at::kFloat, py::arg("init_std") = 0.02, py::arg("fused_classifier") = true,
           py::arg("scale_residual_init") = false)
      .def("parameter_count", &GPT2Config::parameter_count)
      .def("train_flops_per_token", &GPT2Config::train_flops_per_token)
      .def_property_readonly("n_layer", [](const GPT2Config &c) { return c.n_layer(); })
      .def_property_readonly("n_embd", [](const GPT2Config &c) { return c.n_embd(); })
      .def_property_readonly("n_head", [](const GPT2Config &c) { return c.n_head(); })
      .def_property_readonly("vocab_size", [](const GPT2Config &c) { return c.vocab_size(); })
      .def_property_readonly("padded_vocab_size", [](const GPT2Config &c) { return c.padded_vocab_size(); })
      .def_property_readonly("block_size", [](const GPT2Config &c) { return c.block_size(); });

  py::class_<models::GradientSync>(m, "GradientSync")
      .def(py::init([](const communication::Comm &comm, const communication::AllReduceBucket *bucket, bool last) {
             return models::GradientSync{comm, bucket, last};
           }),
           py::keep_alive<1, 3>(), py::arg("comm"), py::arg("bucket"), py::arg("last_micro_step") = true);

  py::class_<models::GPT2Impl, module::Module, std::shared_ptr<models::GPT2Impl>>(m, "GPT2")
      .def(py::init<const Scheduler &, const GPT2Config &>())
      .def("forward", &models::GPT2Impl::forward)
      .def("backward", [](models::GPT2Impl &g, const Scheduler &s, const ReadOnlyTensor &dl, py::object sync) {
        g.backward(s, dl, sync.is_none() ? models::GradientSync{} : py::cast<models::GradientSync>(sync));
      }, py::arg("scheduler"), py::arg("grad_logits"), py::arg("sync") = py::none())
      .def("forward_loss", &models::GPT2Impl::forward_loss)
      .def("backward_loss", [](models::GPT2Impl &g, const Scheduler &s, py::object sync) {
        g.backward_loss(s, sync.is_none() ? models::GradientSync{} : py::cast<models::GradientSync>(sync));
      }, py::arg("scheduler"), py::arg("sync") = py::none())
      .def("config", &models::GPT2Impl::config);

  // ---- communication ---------------------------------------------------------------------------
  using communication::Comm;
  py::class_<Comm>(m, "Comm")
      .def("get_rank", &Comm::get_rank)
      .def("get_size", &Comm::get_size)
      .def("inject_failure_after", [](const Comm &c, int64_t n) { c.impl()->fail_after = n; })
      .def("has_symmetric", [](const Comm &c) { return c.impl()->symmetric != nullptr; })
      .def("release_symmetric", [](const Comm &c) { c.impl()->symmetric.reset(); },
           "Drops the communicator's reference to its symmetric arena (the arena is unmapped once the last holder is gone). "
           "Call it on every rank, after the last kernel that uses the arena, before the process group is destroyed.");
  m.def("comm_from_process_group", &comm_from_process_group, py::arg("group_name"), py::arg("device") = "cuda",
        py::arg("nvp2p") = false);
  m.def("get_comm_world", [](const std::string &backend) {
    return communication::get_comm_world(backend == "nvp2p" ? communication::kNVP2P : communication::kNCCL);
  }, py::arg("backend") = "nccl");
  m.def("get_comm_self", &communication::get_comm_self);
  m.def("finalize_communicators", &communication::finalize);
  m.def("all_reduce", [](const Scheduler &s, const Comm &c, const std::vector<Tensor> &t, const std::string &op) {
    communication::AllReduce::run_inplace(s, c, t, op == "avg" ? communication::kAVG : communication::kSUM);
  }, py::arg("scheduler"), py::arg("comm"), py::arg("tensors"), py::arg("op") = "sum");
  py::class_<communication::AllReduceBucket>(m, "AllReduceBucket")
      .def(py::init([](int64_t bytes, const std::string &op) {
             return communication::AllReduceBucket(bytes, op == "avg" ? communication::kAVG : communication::kSUM);
           }),
           py::arg("byte_threshold"), py::arg("op") = "sum")
      .def("push_back", &communication::AllReduceBucket::push_back)
      .def("sync", &communication::AllReduceBucket::sync)
      .def("launches", &communication::AllReduceBucket::launches)
      .def("attach_optimizer", [](const communication::AllReduceBucket &b, const std::shared_ptr<module::AdamWImpl> &opt) {
        // the optimizer updates each bucket's parameters right after the bucket was reduced
        std::weak_ptr<module::AdamWImpl> weak = opt;
        b.on_reduced([weak](const Scheduler &s, const std::vector<Tensor> &grads, Task::Impl::Priority prio) {
          if (auto o = weak.lock()) o->step_partial(s, grads, prio);
        });
      }, "AdamW over flat arenas: update every bucket's parameters as soon as the bucket has been reduced")
      .def("attach_sharded_optimizer", [](const communication::AllReduceBucket &b, const std::shared_ptr<parallel::ZeroAdamWImpl> &opt) {
        // the bucket only groups the gradients; the optimizer's kernel reduce-scatters them itself
        std::weak_ptr<parallel::ZeroAdamWImpl> weak = opt;
        b.skip_reduction(true);
        b.on_reduced([weak](const Scheduler &s, const std::vector<Tensor> &grads, Task::Impl::Priority prio) {
          if (auto o = weak.lock()) o->step_partial(s, grads, prio);
        });
      }, "ZeroAdamW: reduce-scatter + AdamW + all-gather of every bucket as soon as the backward pass has produced it");
  m.def("all_gather", &communication::AllGather::run);
  m.def("reduce_scatter", [](const Scheduler &s, const Comm &c, const std::vector<Tensor> &recv,
                             const std::vector<std::vector<ReadOnlyTensor>> &send, const std::string &op) {
    communication::ReduceScatter::run(s, c, recv, send, op == "avg" ? communication::kAVG : communication::kSUM);
  }, py::arg("scheduler"), py::arg("comm"), py::arg("recv"), py::arg("send"), py::arg("op") = "sum");
  m.def("all_to_all", &communication::AllToAll::run);
  py::class_<communication::Heartbeat>(m, "Heartbeat")
      .def(py::init<const Comm &, int64_t>())
      .def("beat", &communication::Heartbeat::beat)
      .def("stale_ranks", &communication::Heartbeat::stale_ranks);

  // ---- metrics, watchdog, resumable state ---------------------------------------------------
  py::class_<metrics::StepRecord>(m, "StepRecord")
      .def(py::init<>())
      .def_readwrite("step", &metrics::StepRecord::step)
      .def_readwrite("loss", &metrics::StepRecord::loss)
      .def_readwrite("lr", &metrics::StepRecord::lr)
      .def_readwrite("grad_norm", &metrics::StepRecord::grad_norm)
      .def_readwrite("dt_host_ms", &metrics::StepRecord::dt_host_ms)
      .def_readwrite("dt_device_ms", &metrics::StepRecord::dt_device_ms)
      .def_readwrite("tokens_per_sec", &metrics::StepRecord::tokens_per_sec)
      .def_readwrite("mfu", &metrics::StepRecord::mfu)
      .def_readwrite("comm_bytes", &metrics::StepRecord::comm_bytes)
      .def_readwrite("extra", &metrics::StepRecord::extra);
  py::class_<metrics::MetricsLogger>(m, "MetricsLogger")
      .def(py::init([](const std::string &jsonl, const std::string &csv, bool console, int64_t rank, int64_t writer) {
             return std::make_unique<metrics::MetricsLogger>(
                 metrics::MetricsLogger::Options{}.jsonl_path(jsonl).csv_path(csv).console(console).rank(rank).writer_rank(writer));
           }),
           py::arg("jsonl_path") = "", py::arg("csv_path") = "", py::arg("console") = true, py::arg("rank") = 0,
           py::arg("writer_rank") = 0)
      .def("log", &metrics::MetricsLogger::log)
      .def("records_written", &metrics::MetricsLogger::records_written)
      .def_static("to_json", &metrics::MetricsLogger::to_json)
      .def_static("console_line", &metrics::MetricsLogger::console_line);
  m.def("mfu", &metrics::mfu);
  py::class_<fault::Watchdog>(m, "Watchdog")
      .def(py::init([](std::optional<Comm> comm, int64_t timeout_ms, int64_t poll_ms) {
             auto o = fault::Watchdog::Options{}.timeout_ms(timeout_ms).poll_ms(poll_ms);
             return comm ? std::make_unique<fault::Watchdog>(*comm, o) : std::make_unique<fault::Watchdog>(o);
           }),
           py::arg("comm") = py::none(), py::arg("timeout_ms") = 60000, py::arg("poll_ms") = 50)
      .def("progress", &fault::Watchdog::progress)
      .def("stop", &fault::Watchdog::stop, py::call_guard<py::gil_scoped_release>())
      .def("tripped", &fault::Watchdog::tripped)
      .def("last_step", &fault::Watchdog::last_step)
      .def("failed_peers", &fault::Watchdog::failed_peers)
      .def("check", &fault::Watchdog::check);
  py::class_<checkpoint::Meta>(m, "CheckpointMeta")
      .def(py::init<>())
      .def_readwrite("step", &checkpoint::Meta::step)
      .def_readwrite("lr", &checkpoint::Meta::lr)
      .def_readwrite("seed", &checkpoint::Meta::seed)
      .def_readwrite("data_cursor", &checkpoint::Meta::data_cursor)
      .def_readwrite("world_size", &checkpoint::Meta::world_size)
      .def_readwrite("tp_size", &checkpoint::Meta::tp_size)
      .def_readwrite("zero", &checkpoint::Meta::zero)
      .def_readwrite("model", &checkpoint::Meta::model);
  m.def("save_meta", &checkpoint::save_meta);
  m.def("load_meta", &checkpoint::load_meta);
  m.def("save_training_state",
        [](const Scheduler &s, const std::string &dir, const module::Module &model, std::shared_ptr<module::OptimizerModule> opt,
           const checkpoint::Meta &meta, int64_t rank, int64_t writer_rank) {
          checkpoint::save_training_state(s, dir, model, opt.get(), meta, rank, writer_rank);
        },
        py::arg("scheduler"), py::arg("dir"), py::arg("model"), py::arg("optimizer"), py::arg("meta"), py::arg("rank") = 0,
        py::arg("writer_rank") = 0);
  m.def("load_training_state",
        [](const Scheduler &s, const std::string &dir, const module::Module &model, std::shared_ptr<module::OptimizerModule> opt) {
          return checkpoint::load_training_state(s, dir, model, opt.get());
        },
        py::arg("scheduler"), py::arg("dir"), py::arg("model"), py::arg("optimizer"));

  // ---- symmetric memory / parallel strategies -------------------------------------------------
  using communication::SymmetricContext;
  py::class_<SymmetricContext, std::shared_ptr<SymmetricContext>>(m, "SymmetricContext")
      .def(py::init([](int64_t arena_bytes) {  // offset bookkeeping only (no device memory): allocator tests
             auto c = std::make_shared<SymmetricContext>();
             c->arena_bytes = arena_bytes;
             return c;
           }),
           py::arg("arena_bytes"))
      .def("allocate", [](SymmetricContext &c, int64_t bytes) {
        const auto b = c.allocate(bytes);
        return py::make_tuple(b.offset, b.bytes);
      })
      .def_readonly("rank", &SymmetricContext::rank)
      .def_readonly("size", &SymmetricContext::size)
      .def_readonly("arena_bytes", &SymmetricContext::arena_bytes)
      .def_readonly("virtual_memory", &SymmetricContext::virtual_memory)
      .def_property_readonly("has_multicast", [](const SymmetricContext &c) { return c.multicast_base != nullptr; })
      .def("bytes_in_use", &SymmetricContext::bytes_in_use)
      .def("cached_blocks", &SymmetricContext::cached_blocks)
      .def("empty", [](SymmetricContext &c, std::vector<int64_t> sizes, at::ScalarType dt) {
        int64_t numel = 1;
        for (auto v : sizes) numel *= v;
        const auto block = c.allocate(numel * static_cast<int64_t>(c10::elementSize(dt)));
        return py::make_tuple(c.tensor(block, sizes, dt), block.offset, block.bytes);
      })
      .def("release", [](SymmetricContext &c, int64_t offset, int64_t bytes) {
        c.release(communication::SymmetricBlock{offset, bytes});
      })
      .def("check_status", [](SymmetricContext &c) { communication::check_device_status(c, "python"); })
      // ---- direct calls on torch's current stream: for the single-GPU loopback contexts and kernel tests ----
      .def("prime_loopback", &SymmetricContext::prime_loopback)
      .def("all_reduce_", [](SymmetricContext &c, std::vector<at::Tensor> ranges, const std::string &op) {
        return communication::symmetric_all_reduce(c, ranges, op == "avg" ? communication::kAVG : communication::kSUM);
      }, py::arg("ranges"), py::arg("op") = "sum")
      .def("all_gather_", [](SymmetricContext &c, std::vector<at::Tensor> recv, at::Tensor send) {
        return communication::symmetric_all_gather(c, {recv}, {send});
      })
      .def("reduce_scatter_", [](SymmetricContext &c, at::Tensor recv, std::vector<at::Tensor> send, const std::string &op) {
        return communication::symmetric_reduce_scatter(c, {recv}, {send}, op == "avg" ? communication::kAVG : communication::kSUM);
      }, py::arg("recv"), py::arg("send"), py::arg("op") = "sum")
      .def("all_to_all_", [](SymmetricContext &c, std::vector<at::Tensor> recv, std::vector<at::Tensor> send) {
        return communication::symmetric_all_to_all(c, recv, send);
      })
      .def("gather_rows_chunked", [](SymmetricContext &c, at::Tensor shard, at::Tensor full, int chunks) {
        const auto sig = parallel::gather_rows_chunked(c, shard, full, chunks);
        return py::make_tuple(sig.epoch, reinterpret_cast<uintptr_t>(sig.flags), sig.chunks);
      })
      .def("gemm_on_gathered_chunks", [](SymmetricContext &c, at::Tensor full, at::Tensor weight, bool weight_is_rhs, int epilogue,
                                          py::object aux, py::tuple signal) {
        parallel::GatherSignal sig;
        sig.epoch = signal[0].cast<uint32_t>();
        sig.flags = reinterpret_cast<const uint32_t *>(signal[1].cast<uintptr_t>());
        sig.chunks = signal[2].cast<int>();
        auto r = parallel::gemm_on_gathered_chunks(c, full, weight, weight_is_rhs, epilogue, aux.is_none() ? at::Tensor{} : aux.cast<at::Tensor>(), sig);
        return py::make_tuple(r.first, r.second.defined() ? py::cast(r.second) : py::none());
      }, py::arg("full"), py::arg("weight"), py::arg("weight_is_rhs") = false, py::arg("epilogue") = 0, py::arg("aux") = py::none(),
           py::arg("signal"))
      .def("gemm_scatter_to_slots", &parallel::gemm_scatter_to_slots)
      .def("sum_slots", [](SymmetricContext &c, at::Tensor slots, py::object residual) {
        return parallel::sum_slots(c, slots, residual.is_none() ? at::Tensor{} : residual.cast<at::Tensor>());
      }, py::arg("slots"), py::arg("residual") = py::none())
      .def("sharded_adamw_", [](SymmetricContext &c, at::Tensor grads, py::object lp, at::Tensor master_shard, at::Tensor m, at::Tensor v,
                                int64_t range_begin, int64_t range_end, int64_t block, double lr, double beta1, double beta2, double eps,
                                double wd, int64_t step, double grad_scale) {
        // reduce-scatter + AdamW + all-gather in one kernel for the arena range [range_begin, range_end): this rank updates
        // the blocks it owns (block j belongs to rank j % size; grads fp32 and lp bf16 are arena tensors, the shards local)
        kernels::ShardedAdamWArgs a{};
        int64_t g_off = 0, l_off = -1;
        CS_ASSERT_TRUE(c.locate(grads.data_ptr(), static_cast<int64_t>(grads.nbytes()), &g_off), "grads must live in the arena");
        if (!lp.is_none()) {
          at::Tensor l = lp.cast<at::Tensor>();
          CS_ASSERT_TRUE(c.locate(l.data_ptr(), static_cast<int64_t>(l.nbytes()), &l_off), "the bf16 copy must live in the arena");
        }
        a.grad_offset_bytes = g_off;
        a.lp_offset_bytes = l_off;
        a.master = master_shard.data_ptr<float>();
        a.exp_avg = m.data_ptr<float>();
        a.exp_avg_sq = v.data_ptr<float>();
        a.range_begin = range_begin;
        a.range_end = range_end;
        a.block = block;
        a.lr = static_cast<float>(lr);
        a.beta1 = static_cast<float>(beta1);
        a.beta2 = static_cast<float>(beta2);
        a.eps = static_cast<float>(eps);
        a.weight_decay = static_cast<float>(wd);
        a.inv_bias_correction1 = static_cast<float>(1.0 / (1.0 - std::pow(beta1, static_cast<double>(step))));
        a.inv_bias_correction2 = static_cast<float>(1.0 / (1.0 - std::pow(beta2, static_cast<double>(step))));
        a.grad_scale = static_cast<float>(grad_scale);
        int blocks = 0;
        const auto h = communication::begin_collective(c, kernels::kChanZero);
        const int code = kernels::symm_reduce_scatter_adamw_all_gather(c10::cuda::getCurrentCUDAStream().stream(), communication::table_of(c), h, a, &blocks);
        CS_ASSERT_TRUE(code == 0, "fused reduce-scatter/AdamW/all-gather launch failed: ", cuda_error_string(code));
        communication::end_collective(c, kernels::kChanZero, blocks);
      });
  m.def("create_loopback_contexts", &communication::create_loopback_contexts, py::arg("ranks"), py::arg("arena_bytes"),
        "One symmetric context per emulated rank, all on the current GPU (kernel tests and profiling on a single device)");
  m.def("duplicate_descriptor", &communication::vmm::duplicate_descriptor, py::arg("pid"), py::arg("fd"),
        "Duplicates descriptor `fd` of process `pid` into this process (how arena handles cross process boundaries); -1 on failure");
  m.def("create_symmetric_context", &communication::create_symmetric_context, py::arg("comm"), py::arg("arena_bytes"));
  m.def("symmetric_barrier", [](const Scheduler &s, const Comm &c) {
    cs::submit(s, "cs::communication::barrier", Task::Impl::kComm, Task::Impl::kNccl, {}, {},
               [c](const FnTask &) { c.impl()->symmetric->barrier(); });
  });
  m.def("set_peer_wait_budget", &cs::kernels::set_peer_wait_budget);
  m.def("set_collective_grid_cap", &cs::kernels::set_collective_grid_cap);
  m.def("collective_grid_cap", &cs::kernels::collective_grid_cap);
  m.def("set_multicast_min_ranks", &cs::kernels::set_multicast_min_ranks);
  m.def("multicast_min_ranks", &cs::kernels::multicast_min_ranks);
  m.def("flatten_symmetric",
        [](const Scheduler &s, const module::Module &mod, const Comm &c, const std::vector<std::string> &first, bool unequal_shards) {
          return parallel::flatten_symmetric(s, mod, c, at::kBFloat16, first, unequal_shards);
        },
        py::arg("scheduler"), py::arg("module"), py::arg("comm"), py::arg("first") = std::vector<std::string>{},
        py::arg("unequal_shards") = false);
  py::class_<parallel::ZeroAdamWImpl, module::OptimizerModule, std::shared_ptr<parallel::ZeroAdamWImpl>>(m, "ZeroAdamW")
      .def(py::init([](const Scheduler &s, const std::shared_ptr<module::Module> &mod,
                       std::shared_ptr<module::FlatParameters> flat, const Comm &c, double lr, double beta1, double beta2,
                       double eps, double wd) {
             optimizer::AdamW::Options o;
             o.lr(lr).beta1(beta1).beta2(beta2).eps(eps).weight_decay(wd);
             return std::make_shared<parallel::ZeroAdamWImpl>(s, *mod, flat, c, o);
           }),
           py::keep_alive<1, 3>(), py::arg("scheduler"), py::arg("module"), py::arg("flat"), py::arg("comm"),
           py::arg("lr") = 1e-3, py::arg("beta1") = 0.9, py::arg("beta2") = 0.999, py::arg("eps") = 1e-8,
           py::arg("weight_decay") = 1e-2)
      .def("gather_master", &parallel::ZeroAdamWImpl::gather_master)
      .def("shard_count", &parallel::ZeroAdamWImpl::shard_count)
      .def_property_readonly_static("block", [](py::object) { return parallel::ZeroAdamWImpl::kBlock; });

  py::class_<parallel::TPGPT2Impl, module::Module, std::shared_ptr<parallel::TPGPT2Impl>>(m, "TPGPT2")
      .def(py::init<const Scheduler &, const models::GPT2Config &, const Comm &>())
      .def("forward_loss", &parallel::TPGPT2Impl::forward_loss)
      .def("backward_loss", [](parallel::TPGPT2Impl &g, const Scheduler &s, py::object sync) {
        g.backward_loss(s, sync.is_none() ? models::GradientSync{} : py::cast<models::GradientSync>(sync));
      }, py::arg("scheduler"), py::arg("sync") = py::none())
      .def("replicated_parameters", &parallel::TPGPT2Impl::replicated_parameters)
      .def("vocab_parallel", &parallel::TPGPT2Impl::vocab_parallel)
      .def("head_range", &parallel::TPGPT2Impl::head_range, "(first head, number of heads) of this rank");
  m.def("all_gather_rows", &parallel::all_gather_rows);
  m.def("fused_tp_launches", &parallel::fused_tp_launches);
  m.def("reduce_scatter_rows", [](const Scheduler &s, const Comm &c, const ReadOnlyTensor &full) {
    return parallel::reduce_scatter_rows(s, c, full, nullptr);
  });

  // ---- data ---------------------------------------------------------------------------------------
  py::class_<data::LlmDataset>(m, "LlmDataset")
      .def(py::init<const std::string &>())
      .def("size", &data::LlmDataset::size)
      .def("files", &data::LlmDataset::files)
      .def("file_offsets", &data::LlmDataset::file_offsets);
  py::class_<data::LlmDataLoader>(m, "LlmDataLoader")
      .def(py::init<const data::LlmDataset &, int64_t, int64_t, bool>(), py::arg("dataset"), py::arg("batch_size"),
           py::arg("num_workers"), py::arg("shuffle") = false)
      .def(py::init<const data::LlmDataset &, const Comm &, int64_t, int64_t, bool>(), py::arg("dataset"), py::arg("comm"),
           py::arg("batch_size"), py::arg("num_workers"), py::arg("shuffle") = false)
      .def("load", [](const data::LlmDataLoader &l, const Scheduler &s) {
        auto r = l.load(s);
        py::dict d;
        for (auto &kv : r) d[py::str(kv.first)] = kv.second;
        return d;
      })
      .def("iterations_per_epoch", &data::LlmDataLoader::iterations_per_epoch);
  py::class_<data::SyntheticDataLoader>(m, "SyntheticDataLoader")
      .def(py::init<int64_t, int64_t, int64_t, uint64_t>(), py::arg("batch_size"), py::arg("seq_len"), py::arg("vocab"),
           py::arg("seed") = 0)
      .def("load", [](const data::SyntheticDataLoader &l, const Scheduler &s) {
        auto r = l.load(s);
        py::dict d;
        for (auto &kv : r) d[py::str(kv.first)] = kv.second;
        return d;
      })
      .def("bytes_per_batch", &data::SyntheticDataLoader::bytes_per_batch);
}
