"""nn modules and functions used by the model zoo.

Each wrapper keeps PyTorch's parameter layout (so state dicts are
interchangeable with torch / torchvision checkpoints) and dispatches its math to
this library's sm_100a kernel when one exists for the case at hand, else to the
PyTorch operator. The list of cases served by own kernels grows in
``gcow_b200.ops.kernels``.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import backend
from . import kernels as K


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    if backend.get_backend() == "own" and K.gemm_usable(x, weight):
        return K.linear(x, weight, bias)
    return F.linear(x, weight, bias)


def linear_residual(x: torch.Tensor, lin: nn.Linear, residual: torch.Tensor) -> torch.Tensor:
    """``residual + lin(x)``; on the own backend the addition happens in the GEMM epilogue."""
    if (backend.get_backend() == "own" and lin.bias is not None and residual.shape[-1] == lin.out_features
            and K.fused_mlp_usable(x, lin.weight)):
        return K.linear_residual(x, lin.weight, lin.bias, residual)
    return residual + linear(x, lin.weight, lin.bias)


def ffn_residual(x: torch.Tensor, fc1: nn.Linear, fc2: nn.Linear) -> torch.Tensor:
    """``x + fc2(gelu(fc1(x)))`` - the transformer feed-forward block. On the own backend bias, GELU, its
    gradient and both residual additions run inside the epilogues of the four GEMMs involved."""
    if (backend.get_backend() == "own" and fc1.bias is not None and fc2.bias is not None
            and K.fused_mlp_usable(x, fc1.weight, fc2.weight)):
        return K.ffn_residual(x, fc1.weight, fc1.bias, fc2.weight, fc2.bias)
    return x + linear(gelu(linear(x, fc1.weight, fc1.bias)), fc2.weight, fc2.bias)


class Linear(nn.Linear):
    def forward(self, x):
        return linear(x, self.weight, self.bias)


_last_conv_path = ""


def last_conv_path() -> str:
    """Path of the most recent Conv2d call (see kernels.conv_route); benchmarks print it per layer."""
    return _last_conv_path


class Conv2d(nn.Conv2d):
    """Convolution routed to this library's kernels (kernels.conv_route): the tcgen05 GEMM for 1x1 layers, the
    implicit-GEMM kernel for stride-1 KxK layers and 3x3 stride-2 layers, im2col + GEMM for other strided KxK layers and
    the stem; cuDNN only on
    request (GCOW_CONV=lib / mixed) or for configurations no own kernel covers (groups, dilation, tiny inputs)."""

    def forward(self, x):
        global _last_conv_path
        path = _last_conv_path = K.conv_route(x, self)
        if path == "gemm1x1":
            return K.conv1x1(x, self.weight, self.bias)
        if path == "gemm1x1_strided":
            s = self.stride[0]          # a strided 1x1 convolution reads every s-th pixel: subsample, then the GEMM
            return K.conv1x1(K.subsample(x, s), self.weight, self.bias)
        if path == "igemm":
            return K.conv_igemm(x, self.weight, self.bias, self.padding)
        if path == "igemm1x1_s2":
            return K.conv1x1_s2(x, self.weight, self.bias)
        if path == "igemm_s2":
            return K.conv_igemm_s2(x, self.weight, self.bias)
        if path == "im2col":
            return K.conv_gemm(x, self.weight, self.bias, self.stride[0], self.padding[0])
        return super().forward(x)


class BatchNorm2d(nn.BatchNorm2d):
    """BatchNorm2d whose forward can also take the residual to add and apply the
    ReLU that follows: ``bn(x, residual=idt, relu=True)`` is ``relu(bn(x) + idt)`` in
    one fused kernel on the own backend, and the same three PyTorch ops otherwise.
    With ``fork=True`` the result comes back as a pair of tensors on the same memory, one per consumer, so that the
    backward kernel receives the two gradients separately and adds them while reading (otherwise the pair is just
    the same tensor twice)."""

    def flush_batch_count(self):
        """Add the training steps counted on the host (kernels.batchnorm_act) to ``num_batches_tracked``."""
        n = getattr(self, "_gcow_pending_batches", 0)
        if n and self.num_batches_tracked is not None:
            self.num_batches_tracked += n
        self._gcow_pending_batches = 0

    def _save_to_state_dict(self, destination, prefix, keep_vars):
        self.flush_batch_count()
        super()._save_to_state_dict(destination, prefix, keep_vars)

    def _load_from_state_dict(self, *args, **kw):
        self._gcow_pending_batches = 0
        super()._load_from_state_dict(*args, **kw)

    def forward(self, x, residual=None, relu=False, fork=False):
        if backend.get_backend() == "own" and K.batchnorm_usable(x, self, residual):
            return K.batchnorm_act(x, self, residual, relu, fork)
        self.flush_batch_count()           # PyTorch's own path reads and increments the tensor itself
        y = super().forward(x)
        if residual is not None:
            y = y + residual
        y = F.relu(y) if relu else y
        return (y, y) if fork else y


class MaxPool3x3s2(nn.Module):
    """3x3 / stride 2 / padding 1 max pooling (the ResNet stem pool)."""

    def forward(self, x):
        if backend.get_backend() == "own" and K.pool_usable(x):
            return K.maxpool3x3s2(x)
        return F.max_pool2d(x, 3, 2, 1)


class GlobalAvgPool(nn.Module):
    def forward(self, x):
        if backend.get_backend() == "own" and K.pool_usable(x):
            return K.global_avgpool(x)
        return F.adaptive_avg_pool2d(x, 1)


class LayerNorm(nn.LayerNorm):
    def forward(self, x):
        if backend.get_backend() == "own" and K.layernorm_usable(x, self):
            return K.layernorm(x, self.weight, self.bias, self.eps)
        return super().forward(x)


class Embedding(nn.Embedding):
    pass


def embed_sum3(ids: torch.Tensor, type_ids: torch.Tensor, tok: nn.Embedding, pos: nn.Embedding, typ: nn.Embedding):
    """``tok(ids) + pos(arange(S)) + typ(type_ids)`` for ids [B, S]: the BERT input embedding. One gather kernel and
    a deterministic backward on the own backend."""
    if backend.get_backend() == "own" and K.embed3_usable(ids, tok.weight, pos.weight, typ.weight):
        return K.embed3(ids, type_ids, tok.weight, pos.weight, typ.weight)
    position = torch.arange(ids.shape[1], device=ids.device).unsqueeze(0)
    return tok(ids) + pos(position) + typ(type_ids)


def gelu(x: torch.Tensor) -> torch.Tensor:
    if backend.get_backend() == "own" and K.gelu_usable(x):
        return K.gelu(x)
    return F.gelu(x)


class _PackedSdpaFn(torch.autograd.Function):
    """scaled_dot_product_attention on a packed [B, S, 3, H, D] tensor. Autograd through
    three slices of one tensor costs three zero-filled buffers, three copies and two adds per
    layer; here the three gradients are written into one packed tensor with a single copy."""

    @staticmethod
    def forward(ctx, qkv):
        B, S, _, H, D = qkv.shape
        with torch.enable_grad():
            q, k, v = (qkv[:, :, i].transpose(1, 2).detach().requires_grad_(True) for i in range(3))
            o = F.scaled_dot_product_attention(q, k, v)                # [B, H, S, D]
        ctx.inner = (q, k, v, o)
        ctx.shape = (B, S, H, D)
        return o.detach().transpose(1, 2).reshape(B, S, H * D)

    @staticmethod
    def backward(ctx, go):
        q, k, v, o = ctx.inner
        ctx.inner = None
        B, S, H, D = ctx.shape
        dq, dk, dv = torch.autograd.grad(o, (q, k, v), go.reshape(B, S, H, D).transpose(1, 2))
        return torch.stack((dq.transpose(1, 2), dk.transpose(1, 2), dv.transpose(1, 2)), dim=2)


def attention(qkv: torch.Tensor) -> torch.Tensor:
    """qkv: [B, S, 3, heads, head_dim] -> context [B, S, heads*head_dim] (no mask, no dropout)."""
    B, S, _, H, D = qkv.shape
    if backend.get_backend() == "own" and K.fused_attention_usable(qkv) and K.attention_mode() != "lib":
        return K.fused_attention(qkv)           # one tcgen05 kernel forward, two backward
    if backend.get_backend() == "own" and K.attention_mode() != "lib" and K.attention_usable(qkv):
        return K.attention(qkv)                 # other shapes: batched tcgen05 GEMMs + softmax kernels
    if qkv.is_cuda and qkv.requires_grad and backend.get_backend() == "own":
        return _PackedSdpaFn.apply(qkv)
    q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))     # [B, H, S, D]
    ctx = F.scaled_dot_product_attention(q, k, v)
    return ctx.transpose(1, 2).reshape(B, S, H * D)


def cross_entropy(logits: torch.Tensor, target: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """Mean cross-entropy. With the own backend a non-leaf bf16 logits buffer is
    consumed (overwritten with its gradient) by the fused kernel."""
    if backend.get_backend() == "own" and K.xent_usable(logits):
        return K.softmax_xent(logits, target, ignore_index)
    return F.cross_entropy(logits.float(), target, ignore_index=ignore_index)
