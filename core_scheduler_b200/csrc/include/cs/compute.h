// SPDX-License-Identifier: Apache-2.0
// Functional compute ops. Every op is a struct with a State, an Options builder and static
// init / forward / backward functions that build a task and submit it to a scheduler.
//
// Capability parity (reference project paths): include/compute/linear.h:24-75,
// gelu_linear.h:24-76, layer_norm.h:24-86, gelu.h:22-42, embedding.h:24-78,
// cross_entropy.h:25-60, scaled_dot_product_attention.h:23-117, utils.h:22-108, init.h:23-33.
//
// Execution: bf16 CUDA tensors run on this library's sm_100a kernels (tcgen05 GEMM with fused
// epilogues, fused LayerNorm/GeLU/embedding/cross-entropy kernels); every other dtype/device
// goes through ATen, which is also the numerical oracle used by the tests.
// Extensions over the reference surface are marked "extension".
#pragma once
#include <array>

#include "cs/core.h"
#include "cs/module.h"

namespace cs::compute {
// Which implementation CUDA bf16 tensors use. kFused = this library's kernels;
// kLibrary = ATen/cuBLAS/flash-attention calls (the reference-equivalent path).
enum class Backend : int { kFused = 0, kLibrary = 1 };
CS_API void set_backend(Backend backend);
CS_API Backend get_backend();
// Number of ops that ran a library kernel although the fused backend was selected (each distinct case is
// also logged once as a warning): a benchmark on an uncovered shape shows up here instead of passing silently.
CS_API int64_t library_fallbacks();

struct CS_API Linear {
  struct State : virtual module::State {
    struct Forward {
      Tensor weight;
      Tensor bias{};
      Tensor grad_weight{};
      Tensor grad_bias{};
    } forward;
    struct Backward {
      ReadOnlyTensor input;
    } backward;
    struct Args {
      bool bias;
      bool gelu_epilogue;  // extension: forward also emits GELU(y) as the output's companion
    } args;
    State(const Forward &forward, const Backward &backward, const Args &args)
        : forward{forward}, backward{backward}, args{args} {}
    [[nodiscard]] OrderedDict<std::string, Tensor> parameters() const override;
    [[nodiscard]] OrderedDict<std::string, Tensor> gradients() const override;
    [[nodiscard]] OrderedDict<std::string, Increment> increments() const override;
    void zero_grad() override;
  };
  struct Options {
    Options(const int64_t in_futures, const int64_t out_futures) : in_futures_{in_futures}, out_futures_{out_futures} {}
    CS_ARG(int64_t, in_futures);
    CS_ARG(int64_t, out_futures);
    CS_ARG(bool, bias) = true;
    CS_ARG(optional<at::Device>, device) = {};
    CS_ARG(optional<at::ScalarType>, dtype) = {};
    CS_ARG(bool, gelu_epilogue) = false;  // extension
  };
  static std::shared_ptr<State> init(const Scheduler &scheduler, const Options &options);
  static Tensor forward(const Scheduler &scheduler, const std::shared_ptr<State> &state, const ReadOnlyTensor &input);
  // extension: y = x W^T (+ b) + residual, the add runs in the GEMM epilogue.
  static Tensor forward(const Scheduler &scheduler, const std::shared_ptr<State> &state, const ReadOnlyTensor &input,
                        const ReadOnlyTensor &residual);
  static Tensor backward_input(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                               const ReadOnlyTensor &grad_output);
  static void backward_parameter(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                                 const ReadOnlyTensor &grad_output);
};

// y = GELU(x) W^T (+ b). When x carries GELU(x) as a companion (produced by a Linear with
// gelu_epilogue) no activation kernel runs at all.
struct CS_API GeluLinear {
  struct State : virtual module::State {
    struct Forward {
      Tensor weight;
      Tensor bias{};
      Tensor grad_weight{};
      Tensor grad_bias{};
    } forward;
    struct Backward {
      ReadOnlyTensor input;
      ReadOnlyTensor activated;  // GELU(input) kept for the weight gradient (bf16 fused path)
      int input_count{0};
    } backward;
    struct Args {
      bool bias;
    } args;
    State(const Forward &forward, const Backward &backward, const Args &args)
        : forward{forward}, backward{backward}, args{args} {}
    [[nodiscard]] OrderedDict<std::string, Tensor> parameters() const override;
    [[nodiscard]] OrderedDict<std::string, Tensor> gradients() const override;
    [[nodiscard]] OrderedDict<std::string, Increment> increments() const override;
    void zero_grad() override;
  };
  using Options = Linear::Options;
  static std::shared_ptr<State> init(const Scheduler &scheduler, const Options &options);
  static Tensor forward(const Scheduler &scheduler, const std::shared_ptr<State> &state, const ReadOnlyTensor &input);
  static Tensor forward(const Scheduler &scheduler, const std::shared_ptr<State> &state, const ReadOnlyTensor &input,
                        const ReadOnlyTensor &residual);  // extension
  static Tensor backward_input(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                               const ReadOnlyTensor &grad_output);
  static void backward_parameter(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                                 const ReadOnlyTensor &grad_output);
};

struct CS_API LayerNorm {
  struct State : virtual module::State {
    struct Forward {
      Tensor weight;
      Tensor bias;
      Tensor grad_weight{};
      Tensor grad_bias{};
    } forward;
    struct Backward {
      ReadOnlyTensor input;
      ReadOnlyTensor mean;
      ReadOnlyTensor rstd;
    } backward;
    struct Args {
      IntArray normalized_shape;
      double eps;
      bool elementwise_affine;
      bool bias;
    } args;
    State(const Forward &forward, const Backward &backward, const Args &args)
        : forward{forward}, backward{backward}, args{args} {}
    [[nodiscard]] OrderedDict<std::string, Tensor> parameters() const override;
    [[nodiscard]] OrderedDict<std::string, Tensor> gradients() const override;
    [[nodiscard]] OrderedDict<std::string, Increment> increments() const override;
    void zero_grad() override;
  };
  struct Options {
    Options(IntArrayRef normalized_shape) : normalized_shape_{normalized_shape.begin(), normalized_shape.end()} {}
    Options(int64_t normalized_shape) : normalized_shape_{normalized_shape} {}
    CS_ARG(IntArray, normalized_shape);
    CS_ARG(double, eps) = 1e-5;
    CS_ARG(bool, elementwise_affine) = true;
    CS_ARG(bool, bias) = true;
    CS_ARG(optional<at::Device>, device) = {};
    CS_ARG(optional<at::ScalarType>, dtype) = {};
  };
  static std::shared_ptr<State> init(const Scheduler &scheduler, const Options &options);
  static Tensor forward(const Scheduler &scheduler, const std::shared_ptr<State> &state, const ReadOnlyTensor &input);
  // dγ/dβ and dx in one pass on the fused path (two tasks on the library path).
  static Tensor backward(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                         const ReadOnlyTensor &grad_output);
  // extension: returns dx + grad_residual (the residual-branch add is fused into the kernel).
  static Tensor backward(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                         const ReadOnlyTensor &grad_output, const ReadOnlyTensor &grad_residual);
  static Tensor backward_input(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                               const ReadOnlyTensor &grad_output);
  static void backward_parameter(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                                 const ReadOnlyTensor &grad_output);
};

struct CS_API GeLU {
  struct State {
    struct Backward {
      ReadOnlyTensor input;
    } backward;
  };
  static std::shared_ptr<State> init(const Scheduler &scheduler);
  static Tensor forward(const Scheduler &scheduler, const std::shared_ptr<State> &state, const ReadOnlyTensor &input);
  static Tensor backward(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                         const ReadOnlyTensor &grad_output);
};

struct CS_API Embedding {
  struct State : virtual module::State {
    struct Forward {
      Tensor weight;
      Tensor grad_weight{};
    } forward;
    struct Backward {
      ReadOnlyTensor indices;
    } backward;
    struct Args {
      int64_t num_embeddings;
      int64_t padding_idx;
      optional<double> max_norm;
      double norm_type;
      bool scale_grad_by_freq;
      bool sparse;
    } args;
    State(const Forward &forward, const Backward &backward, const Args &args)
        : forward{forward}, backward{backward}, args{args} {}
    [[nodiscard]] OrderedDict<std::string, Tensor> parameters() const override;
    [[nodiscard]] OrderedDict<std::string, Tensor> gradients() const override;
    [[nodiscard]] OrderedDict<std::string, Increment> increments() const override;
    void zero_grad() override;
  };
  struct Options {
    Options(const int64_t num_embeddings, const int64_t embedding_dim)
        : num_embeddings_{num_embeddings}, embedding_dim_{embedding_dim} {}
    CS_ARG(int64_t, num_embeddings);
    CS_ARG(int64_t, embedding_dim);
    CS_ARG(optional<int64_t>, padding_idx) = {};
    CS_ARG(optional<double>, max_norm) = {};
    CS_ARG(double, norm_type) = 2.;
    CS_ARG(bool, scale_grad_by_freq) = false;
    CS_ARG(bool, sparse) = false;
    CS_ARG(optional<at::Device>, device) = {};
    CS_ARG(optional<at::ScalarType>, dtype) = {};
  };
  static std::shared_ptr<State> init(const Scheduler &scheduler, const Options &options);
  static Tensor forward(const Scheduler &scheduler, const std::shared_ptr<State> &state, const ReadOnlyTensor &indices);
  static void backward(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                       const ReadOnlyTensor &grad_output);
  // extension: token + position embedding in one kernel, out[b,t,:] = wte[idx[b,t]] + wpe[t].
  static Tensor forward_token_position(const Scheduler &scheduler, const std::shared_ptr<State> &token,
                                       const std::shared_ptr<State> &position, const ReadOnlyTensor &indices);
  static void backward_token_position(const Scheduler &scheduler, const std::shared_ptr<State> &token,
                                      const std::shared_ptr<State> &position, const ReadOnlyTensor &grad_output);
};

enum class Reduction : int { kNone = 0, kMean = 1, kSum = 2 };

struct CS_API CrossEntropy {
  struct State {
    struct Forward {
      Tensor weight{};  // optional per-class weights
    } forward;
    struct Backward {
      ReadOnlyTensor log_probs;
      ReadOnlyTensor target;
      ReadOnlyTensor total_weight;
      ReadOnlyTensor loss;
      // fused path: logits + per-row log-sum-exp instead of log-probs
      ReadOnlyTensor logits;
      ReadOnlyTensor lse;
    } backward;
    struct Args {
      Reduction reduction;
      int64_t ignore_index;
      double label_smoothing;
    } args;
  };
  struct Options {
    Options() {}
    CS_ARG(Reduction, reduction) = Reduction::kMean;
    CS_ARG(int64_t, ignore_index) = -100;
    CS_ARG(double, label_smoothing) = 0.0;
  };
  static std::shared_ptr<State> init(const Scheduler &scheduler, const Options &options = {});
  static Tensor forward(const Scheduler &scheduler, const std::shared_ptr<State> &state, const ReadOnlyTensor &input,
                        const ReadOnlyTensor &target);
  static Tensor backward(const Scheduler &scheduler, const std::shared_ptr<State> &state);
};

// extension: classifier GEMM fused with the cross-entropy. The forward GEMM's epilogue keeps
// running (max, sum-exp) per row while it stores bf16 logits once; backward turns the logits
// into dlogits in place and feeds the two gradient GEMMs. No fp32 [rows, vocab] tensor exists.
struct CS_API LinearCrossEntropy {
  struct State {
    std::shared_ptr<Linear::State> linear;
    struct Backward {
      ReadOnlyTensor input;
      ReadOnlyTensor target;
      ReadOnlyTensor logits;
      ReadOnlyTensor lse;
    } backward;
    int64_t ignore_index{-100};
    int64_t valid_classes{-1};  // columns >= valid_classes are padding and never predicted
  };
  static std::shared_ptr<State> init(const Scheduler &scheduler, const std::shared_ptr<Linear::State> &linear,
                                     int64_t valid_classes = -1, int64_t ignore_index = -100);
  // input [rows, d], target [rows] int64 -> mean loss (fp32 scalar)
  static Tensor forward(const Scheduler &scheduler, const std::shared_ptr<State> &state, const ReadOnlyTensor &input,
                        const ReadOnlyTensor &target);
  // returns d(input); accumulates the classifier weight gradient (assist stream)
  static Tensor backward(const Scheduler &scheduler, const std::shared_ptr<State> &state);
};

struct CS_API ScaledDotProductAttention {
  struct State {
    struct Forward {
    } forward;
    struct Backward {
      ReadOnlyTensor query, key, value, out, logsumexp;
      ReadOnlyTensor cum_seq_q, cum_seq_k;
      int64_t max_q{0}, max_k{0};
      ReadOnlyTensor philox_seed, philox_offset;
      bool packed{false};
      ReadOnlyTensor qkv;
    } backward;
    struct Args {
      double dropout_p;
      bool is_causal;
      bool return_debug_mask;
      optional<double> scale;
    } args;
  };
  struct Options {
    Options() {}
    CS_ARG(double, dropout_p) = 0;
    CS_ARG(bool, is_causal) = false;
    CS_ARG(bool, return_debug_mask) = false;
    CS_ARG(optional<double>, scale) = {};
  };
  static std::shared_ptr<State> init(const Scheduler &scheduler, const Options &options = {});
  // query/key/value: [B, T, H, D]; returns [B, T, H, D]
  static Tensor forward(const Scheduler &scheduler, const std::shared_ptr<State> &state, const ReadOnlyTensor &query,
                        const ReadOnlyTensor &key, const ReadOnlyTensor &value);
  static std::array<Tensor, 3> backward(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                                        const ReadOnlyTensor &grad_out);
  // extension: qkv packed as [B, T, 3*H*D] (the c_attn output); backward returns packed dqkv.
  static Tensor forward_packed(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                               const ReadOnlyTensor &qkv, int64_t num_heads);
  static Tensor backward_packed(const Scheduler &scheduler, const std::shared_ptr<State> &state,
                                const ReadOnlyTensor &grad_out);
};
// The reference exposes two attention classes (flash-attention and cuDNN engines) with the
// same interface; here both names resolve to the single implementation.
using ScaledDotProductFlashAttention = ScaledDotProductAttention;
using ScaledDotProductCuDnn = ScaledDotProductAttention;

// A namespace, as in the reference (include/compute/utils.h:21): `namespace U = cs::compute::Utils;` must compile.
namespace Utils {
  CS_API Tensor sum(const Scheduler &scheduler, const ReadOnlyTensor &input, IntArrayRef dim, bool keep_dim = false,
                    optional<at::ScalarType> dtype = {});
  CS_API Tensor sum(const Scheduler &scheduler, const ReadOnlyTensor &input, int64_t dim, bool keep_dim = false,
                    optional<at::ScalarType> dtype = {});
  CS_API Tensor range(const Scheduler &scheduler, const Scalar &start, const Scalar &end, TensorOptions options = {});
  CS_API Tensor arange(const Scheduler &scheduler, const Scalar &start, const Scalar &end, TensorOptions options = {});
  CS_API Tensor arange(const Scheduler &scheduler, const Scalar &start, const Scalar &end, const Scalar &step,
                       TensorOptions options = {});
  CS_API Tensor randint(const Scheduler &scheduler, int64_t low, int64_t high, IntArrayRef size,
                        TensorOptions options = at::kLong);
  CS_API Tensor empty(const Scheduler &scheduler, IntArrayRef size, TensorOptions options = {});
  CS_API Tensor empty_like(const Scheduler &scheduler, const ReadOnlyTensor &src);
  CS_API Tensor ones(const Scheduler &scheduler, IntArrayRef size, TensorOptions options = {});
  CS_API Tensor ones_like(const Scheduler &scheduler, const ReadOnlyTensor &src);
  CS_API Tensor zeros(const Scheduler &scheduler, IntArrayRef size, TensorOptions options = {});
  CS_API Tensor zeros_like(const Scheduler &scheduler, const ReadOnlyTensor &src);
  CS_API Tensor rand(const Scheduler &scheduler, IntArrayRef size, TensorOptions options = {});
  CS_API Tensor rand_like(const Scheduler &scheduler, const ReadOnlyTensor &src);
  CS_API Tensor randn(const Scheduler &scheduler, IntArrayRef size, TensorOptions options = {});
  CS_API Tensor randn_like(const Scheduler &scheduler, const ReadOnlyTensor &src);
  CS_API std::vector<Tensor> split(const Scheduler &scheduler, const ReadOnlyTensor &src, int64_t split_size,
                                   int64_t dim);
  CS_API Tensor view(const Scheduler &scheduler, const ReadOnlyTensor &input, IntArrayRef size);
  CS_API Tensor as_strided(const Scheduler &scheduler, const ReadOnlyTensor &input, IntArrayRef size,
                           IntArrayRef stride, optional<int64_t> storage_offset = {});
  CS_API Tensor broadcast_to(const Scheduler &scheduler, const ReadOnlyTensor &input, IntArrayRef size);
  CS_API Tensor cat(const Scheduler &scheduler, const std::vector<ReadOnlyTensor> &input, int64_t dim);
  CS_API Tensor add(const Scheduler &scheduler, const ReadOnlyTensor &x, const ReadOnlyTensor &y);
  CS_API void zero_(const Scheduler &scheduler, const Tensor &tensor);
  CS_API void uniform_(const Scheduler &scheduler, const Tensor &tensor, double from = 0, double to = 1);
  CS_API void normal_(const Scheduler &scheduler, const Tensor &tensor, double mean = 0, double std = 1);
  CS_API Tensor clone(const Scheduler &scheduler, const Tensor &tensor);
  CS_API Tensor linalg_vector_norm(const Scheduler &scheduler, const ReadOnlyTensor &self, const Scalar &ord = 2,
                                   at::OptionalIntArrayRef dim = c10::nullopt, bool keepdim = false,
                                   optional<at::ScalarType> dtype = {});
  // Scales the gradients in place so that their joint norm is at most max_norm; returns the
  // norm measured before scaling.
  CS_API Tensor clip_grad_norm_(const Scheduler &scheduler, const std::vector<Tensor> &tensors, double max_norm,
                                double norm_type = 2.0);
  // extension: casts/moves a tensor.
  CS_API Tensor to(const Scheduler &scheduler, const ReadOnlyTensor &input, TensorOptions options);
}  // namespace Utils

enum class FanMode : int { kFanIn = 0, kFanOut = 1 };
enum class Nonlinearity : int { kLinear = 0, kSigmoid, kTanh, kReLU, kLeakyReLU };

namespace Init {  // a namespace in the reference too (include/compute/init.h:23)
  CS_API void kaiming_normal_(const Scheduler &scheduler, const Tensor &tensor, double a = 0,
                              FanMode mode = FanMode::kFanIn, Nonlinearity nonlinearity = Nonlinearity::kLeakyReLU);
  CS_API void kaiming_uniform_(const Scheduler &scheduler, const Tensor &tensor, double a = 0,
                               FanMode mode = FanMode::kFanIn, Nonlinearity nonlinearity = Nonlinearity::kLeakyReLU);
}  // namespace Init

// Marks a parameter as changed (invalidates low-precision working copies).
CS_API void bump_version(const Tensor &parameter);
// Returns the parameter cast to `dtype`, using/refreshing the cached working copy. Must be
// called inside a task body on the stream that will consume the copy.
CS_API at::Tensor working_copy(const ReadOnlyTensor &parameter, at::ScalarType dtype);
// Same for the [in, out] transpose of a 2-D parameter.
CS_API at::Tensor working_copy_transposed(const ReadOnlyTensor &parameter, at::ScalarType dtype);
}  // namespace cs::compute
