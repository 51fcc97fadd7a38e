"""autograd.Function wrappers around the sm_100a compute kernels.

``*_usable`` predicates say whether a kernel covers a given call (dtype, layout,
alignment); callers fall back to PyTorch otherwise.
"""
from __future__ import annotations

import torch

from .. import _native

_launches = 0
_err_words: dict = {}

OUT_F32, BIAS, GELU, RESIDUAL, ACCUMULATE = 1, 2, 4, 8, 16


def launch_count() -> int:
    """How many compute kernels of this library were launched through this module."""
    return _launches


def _have(name: str) -> bool:
    if not _native.cuda_available():
        return False
    try:
        return hasattr(_native.cuda(), name)
    except Exception:
        return False


def _error_word(device: torch.device) -> torch.Tensor:
    w = _err_words.get(device)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=device)
        _err_words[device] = w
    return w


def check_errors(device: torch.device | None = None) -> None:
    """Raise if any compute kernel gave up on an internal wait (synchronises)."""
    for dev, w in _err_words.items():
        if device is not None and dev != device:
            continue
        code = int(w.item())
        if code:
            w.zero_()
            raise RuntimeError(f"gcow compute kernel on {dev} abandoned a wait (role code {code})")


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, *, bias: torch.Tensor | None = None,
              residual: torch.Tensor | None = None, gelu: bool = False, out_dtype=torch.bfloat16,
              out: torch.Tensor | None = None, accumulate: bool = False, max_ctas: int = 0) -> torch.Tensor:
    """C[M,N] = A[M,K] @ B[N,K]^T (+bias) (GELU) (+residual) on the tcgen05 kernel.

    a, b: bf16, last dimension contiguous, leading dimension and K multiples of 8.
    bias: fp32 [N]. residual/out: [M,N] of ``out_dtype`` (bf16 or fp32)."""
    global _launches
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.dim() == 2 and b.dim() == 2
    assert a.stride(1) == 1 and b.stride(1) == 1 and a.shape[1] == b.shape[1]
    M, K = a.shape
    N = b.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    flags = (OUT_F32 if out.dtype == torch.float32 else 0) | (BIAS if bias is not None else 0) | \
        (GELU if gelu else 0) | (RESIDUAL if residual is not None else 0) | (ACCUMULATE if accumulate else 0)
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == N
    if residual is not None:
        assert residual.dtype == out.dtype and residual.stride() == out.stride()
    err = _native.cuda().gcow_gemm_bf16(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0),
        bias.data_ptr() if bias is not None else None, residual.data_ptr() if residual is not None else None,
        flags, _error_word(a.device).data_ptr(), max_ctas, torch.cuda.current_stream(a.device).cuda_stream)
    if err:
        raise RuntimeError(f"gcow_gemm_bf16 refused the call: {err}")
    _launches += 1
    return out


def _gemm_ok(x2d: torch.Tensor, w: torch.Tensor) -> bool:
    return (x2d.is_cuda and x2d.shape[1] % 8 == 0 and w.shape[1] % 8 == 0 and w.shape[0] % 8 == 0
            and x2d.shape[0] >= 64)


class _LinearFn(torch.autograd.Function):
    """y = x W^T + b with all three GEMMs (forward, dgrad, wgrad) on the tcgen05 kernel."""

    @staticmethod
    def forward(ctx, x, w, b):
        xb = x.reshape(-1, x.shape[-1]).to(torch.bfloat16).contiguous()
        wb = w.to(torch.bfloat16).contiguous()
        bias = b.float().contiguous() if b is not None else None
        y = gemm_bf16(xb, wb, bias=bias)
        ctx.save_for_backward(xb, wb)
        ctx.has_bias = b is not None
        ctx.x_shape = x.shape
        ctx.w_dtype = w.dtype
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        xb, wb = ctx.saved_tensors
        g = gy.reshape(-1, gy.shape[-1]).to(torch.bfloat16).contiguous()
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            # dx[M,K] = g[M,N] @ W[N,K]  ->  A = g, B = W^T stored [K,N]
            gx = gemm_bf16(g, wb.t().contiguous()).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            # dW[N,K] = g^T[N,M] @ x[M,K]  ->  A = g^T stored [N,M], B = x^T stored [K,M]
            M = g.shape[0]
            if M % 8 == 0:
                gw = gemm_bf16(g.t().contiguous(), xb.t().contiguous(), out_dtype=torch.float32).to(ctx.w_dtype)
            else:
                gw = (g.float().t() @ xb.float()).to(ctx.w_dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            gb = g.float().sum(0)
        return gx, gw, gb


def gemm_usable(x: torch.Tensor, w: torch.Tensor) -> bool:
    if not (x.is_cuda and _have("gcow_gemm_bf16")):
        return False
    x2 = x.reshape(-1, x.shape[-1])
    return _gemm_ok(x2, w)


def linear(x, w, b):
    return _LinearFn.apply(x, w, b)


def conv1x1_usable(x: torch.Tensor, w: torch.Tensor) -> bool:
    return False


def conv1x1(x, w, b):  # pragma: no cover
    raise NotImplementedError


def layernorm_usable(x: torch.Tensor, mod) -> bool:
    return False


def layernorm(x, w, b, eps):  # pragma: no cover
    raise NotImplementedError
