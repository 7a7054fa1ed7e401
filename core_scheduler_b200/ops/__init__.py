# SPDX-License-Identifier: Apache-2.0
"""Ops with explicit backward, as Python objects over the native library.

Each class owns the native State of one op of the reference project's `cs::compute` layer and exposes the same
calls (include/compute/linear.h, gelu_linear.h, layer_norm.h, gelu.h, embedding.h, cross_entropy.h,
scaled_dot_product_attention.h, include/optimizer/adamw.h): `forward` stores what `backward` needs, the
parameter-gradient half runs on the scheduler's assist stream, the input-gradient half on the main stream.
Inputs and outputs are `core_scheduler_b200.Tensor` handles (`from_torch` / `.raw()` cross to PyTorch).

    s = cs.DynamicScheduler(0)
    fc = ops.Linear(s, 768, 3072, bias=False)
    y = fc.forward(cs.from_torch(x))
    dx = fc.backward(cs.from_torch(dy))          # weight gradient in fc.grad_weight
"""
from __future__ import annotations

from .. import _C

__all__ = ["Linear", "GeluLinear", "LayerNorm", "GeLU", "Embedding", "CrossEntropy", "LinearCrossEntropy", "Attention", "AdamW",
           "clip_grad_norm_"]


class _Parametrised:
    """Common accessors of ops that own parameters (the native `module::State`)."""

    state = None

    @property
    def weight(self):
        return self.state.weight

    @property
    def grad_weight(self):
        return self.state.grad_weight

    def zero_grad(self):
        self.state.zero_grad()


class Linear(_Parametrised):
    """y = x W^T (+ b); weight [out, in], kaiming-uniform initialised as in the reference (src/compute/linear.cpp:95-106)."""

    def __init__(self, scheduler, in_features, out_features, bias=True, dtype=None, device=None):
        self.scheduler = scheduler
        self.state = _C.linear_init(scheduler, in_features, out_features, bias=bias, dtype=dtype, device=device)

    @property
    def bias(self):
        return self.state.bias

    @property
    def grad_bias(self):
        return self.state.grad_bias

    def forward(self, x, residual=None):
        """`residual`, when given, is added in the same kernel (an extension of the reference's interface)."""
        return _C.linear_forward(self.scheduler, self.state, x, residual)

    def backward_input(self, grad_output):
        return _C.linear_backward_input(self.scheduler, self.state, grad_output)

    def backward_parameter(self, grad_output):
        _C.linear_backward_parameter(self.scheduler, self.state, grad_output)

    def backward(self, grad_output):
        """Parameter gradients (assist stream) then the input gradient (main stream), the reference's order."""
        self.backward_parameter(grad_output)
        return self.backward_input(grad_output)


class GeluLinear(_Parametrised):
    """y = GELU(x) W^T (+ b) as one op (include/compute/gelu_linear.h in the reference)."""

    def __init__(self, scheduler, in_features, out_features, bias=True, dtype=None, device=None):
        self.scheduler = scheduler
        self.state = _C.gelu_linear_init(scheduler, in_features, out_features, bias=bias, dtype=dtype, device=device)

    @property
    def bias(self):
        return self.state.bias

    @property
    def grad_bias(self):
        return self.state.grad_bias

    def forward(self, x, residual=None):
        return _C.gelu_linear_forward(self.scheduler, self.state, x, residual)

    def backward_input(self, grad_output):
        return _C.gelu_linear_backward_input(self.scheduler, self.state, grad_output)

    def backward_parameter(self, grad_output):
        _C.gelu_linear_backward_parameter(self.scheduler, self.state, grad_output)

    def backward(self, grad_output):
        """Input gradient first: the saved input is released after both halves ran (the reference's order for this op)."""
        dx = self.backward_input(grad_output)
        self.backward_parameter(grad_output)
        return dx


class LayerNorm(_Parametrised):
    """Affine LayerNorm over the trailing `normalized_shape`; statistics in fp32 (include/compute/layer_norm.h)."""

    def __init__(self, scheduler, normalized_shape, eps=1e-5, dtype=None, device=None):
        self.scheduler = scheduler
        shape = [normalized_shape] if isinstance(normalized_shape, int) else list(normalized_shape)
        self.state = _C.layer_norm_init(scheduler, shape, eps=eps, dtype=dtype, device=device)

    @property
    def bias(self):
        return self.state.bias

    @property
    def grad_bias(self):
        return self.state.grad_bias

    def forward(self, x):
        return _C.layer_norm_forward(self.scheduler, self.state, x)

    def backward(self, grad_output, grad_residual=None):
        """dx (+ `grad_residual`, added in the same pass) and the gamma/beta gradients."""
        return _C.layer_norm_backward(self.scheduler, self.state, grad_output, grad_residual)


class GeLU:
    """Exact (erf) GELU; saves its input for the backward pass (include/compute/gelu.h)."""

    def __init__(self, scheduler):
        self.scheduler = scheduler
        self.state = _C.gelu_init(scheduler)

    def forward(self, x):
        return _C.gelu_forward(self.scheduler, self.state, x)

    def backward(self, grad_output):
        return _C.gelu_backward(self.scheduler, self.state, grad_output)


class Embedding(_Parametrised):
    """Row gather with a dense weight gradient; weight ~ N(0, 1) (include/compute/embedding.h)."""

    def __init__(self, scheduler, num_embeddings, embedding_dim, padding_idx=None, dtype=None, device=None):
        self.scheduler = scheduler
        self.state = _C.embedding_init(scheduler, num_embeddings, embedding_dim, padding_idx=padding_idx, dtype=dtype, device=device)

    def forward(self, indices):
        return _C.embedding_forward(self.scheduler, self.state, indices)

    def backward(self, grad_output):
        _C.embedding_backward(self.scheduler, self.state, grad_output)


class CrossEntropy:
    """Softmax cross-entropy over [rows, classes] logits with int64 targets (include/compute/cross_entropy.h)."""

    def __init__(self, scheduler, reduction="mean", ignore_index=-100):
        self.scheduler = scheduler
        self.state = _C.cross_entropy_init(scheduler, reduction=reduction, ignore_index=ignore_index)

    def forward(self, logits, target):
        return _C.cross_entropy_forward(self.scheduler, self.state, logits, target)

    def backward(self):
        """d(loss)/d(logits) for a loss gradient of one."""
        return _C.cross_entropy_backward(self.scheduler, self.state)


class LinearCrossEntropy:
    """Classifier and loss in one op: the logits are written once in the activation type and never as fp32
    (no counterpart in the reference, which materialises fp32 log-probabilities). `valid_classes` masks padded
    vocabulary columns."""

    def __init__(self, scheduler, linear: Linear, valid_classes=-1, ignore_index=-100):
        self.scheduler = scheduler
        self.linear = linear
        self.state = _C.linear_cross_entropy_init(scheduler, linear.state, valid_classes=valid_classes, ignore_index=ignore_index)

    def forward(self, x, target):
        return _C.linear_cross_entropy_forward(self.scheduler, self.state, x, target)

    def backward(self):
        """Returns d(loss)/dx; the classifier's weight gradient lands in `linear.grad_weight`."""
        return _C.linear_cross_entropy_backward(self.scheduler, self.state)


class Attention:
    """Scaled dot-product attention on [B, T, H, D] tensors (both of the reference's attention classes,
    include/compute/scaled_dot_product_attention.h); the packed forms take the c_attn output [B, T, 3*H*D]."""

    def __init__(self, scheduler, is_causal=False, dropout_p=0.0, scale=None):
        self.scheduler = scheduler
        self.state = _C.attention_init(scheduler, is_causal=is_causal, dropout_p=dropout_p, scale=scale)

    def forward(self, query, key, value):
        return _C.attention_forward(self.scheduler, self.state, query, key, value)

    def backward(self, grad_output):
        """[dq, dk, dv]"""
        return _C.attention_backward(self.scheduler, self.state, grad_output)

    def forward_packed(self, qkv, num_heads):
        return _C.attention_forward_packed(self.scheduler, self.state, qkv, num_heads)

    def backward_packed(self, grad_output):
        return _C.attention_backward_packed(self.scheduler, self.state, grad_output)


class AdamW:
    """Functional AdamW for one parameter tensor (include/optimizer/adamw.h); `step_amp` updates fp32 master weights
    and writes the low-precision working copy (the reference declares that variant without defining it)."""

    def __init__(self, scheduler, parameter, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=1e-2, amsgrad=False):
        self.scheduler = scheduler
        self.state = _C.adamw_init(scheduler, parameter, lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay,
                                   amsgrad=amsgrad)

    def step(self, parameter, gradient):
        _C.adamw_step(self.scheduler, self.state, parameter, gradient)

    def step_amp(self, working_copy, master, gradient):
        _C.amp_adamw_step(self.scheduler, self.state, working_copy, master, gradient)


def clip_grad_norm_(scheduler, gradients, max_norm, norm_type=2.0):
    """Scales the gradients in place so that their joint norm is at most `max_norm`; returns the norm before scaling."""
    return _C.utils_clip_grad_norm_(scheduler, list(gradients), max_norm, norm_type)
