"""autograd.Function wrappers around the sm_100a compute kernels.

``*_usable`` predicates say whether a kernel covers a given call (dtype, layout,
alignment); callers fall back to PyTorch otherwise.
"""
from __future__ import annotations

import os

import torch

from .. import _native

_launches = 0
_err_words: dict = {}

OUT_F32, BIAS, GELU, RESIDUAL, ACCUMULATE, AUX_OUT, GELU_GRAD = 1, 2, 4, 8, 16, 32, 64


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


_arena: dict = {}


def _ws(tag: str, shape, dtype, device) -> torch.Tensor:
    """Scratch tensor from a per-(device, stream, purpose) arena that grows to the largest request and is then
    reused: partial sums of split reductions and similar buffers that live only between two kernels of one
    operation. Operations on one stream run in order, so two of them never use the same scratch at the same time;
    nothing that is returned to the caller or saved for the backward pass may come from here."""
    n = 1
    for d in (shape if isinstance(shape, (tuple, list)) else (shape,)):
        n *= int(d)
    key = (tag, dtype, device, torch.cuda.current_stream(device).cuda_stream)
    buf = _arena.get(key)
    if buf is None or buf.numel() < n:
        buf = torch.empty(max(n, 1), dtype=dtype, device=device)
        _arena[key] = buf
    return buf[:n].view(shape)


def workspace_bytes() -> int:
    """Bytes currently held by the scratch arena."""
    return sum(b.numel() * b.element_size() for b in _arena.values())


def _error_word(device: torch.device) -> torch.Tensor:
    w = _err_words.get(device)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=device)
        _err_words[device] = w
    return w


class KernelWaitAbandoned(RuntimeError):
    """A tcgen05 GEMM / convolution kernel gave up on one of its bounded mbarrier waits, so a tile of its
    output was not written."""


def check_errors(device: torch.device | None = None, raise_on_error: bool = True) -> int:
    """Read the error word of the compute kernels (synchronises). Raises KernelWaitAbandoned if a kernel gave up on
    an internal wait, or returns the code when ``raise_on_error`` is false. The word is cleared."""
    worst = 0
    for dev, w in _err_words.items():
        if device is not None and dev != device:
            continue
        code = int(w.item())
        if code:
            w.zero_()
            if raise_on_error:
                raise KernelWaitAbandoned(f"gcow compute kernel on {dev} abandoned a wait (role code {code})")
            worst = code
    return worst


def error_word(device: torch.device) -> torch.Tensor:
    """The device word that the tensor-core kernels set when they abandon a wait (one int32). Training loops copy it
    to the host next to the loss, so a kernel that gave up is noticed one step later without an extra synchronisation."""
    return _error_word(device)


def bf16_weight(w: torch.Tensor) -> torch.Tensor:
    """bf16 copy of a float32 weight in the same element order. The fused optimizers keep one up to date in their
    update kernel (``w._gcow_bf16``, valid while ``w._version`` has not moved since), so a training step runs no cast
    kernel per layer; a stale or missing copy is refreshed or made here. (Writes that bypass the version counter,
    i.e. through ``w.data``, are not seen: such code has to drop ``w._gcow_bf16`` itself.)"""
    sh = getattr(w, "_gcow_bf16", None)          # Python attributes live on the parameter object, not on a detached view
    if sh is None or sh.shape != w.shape or sh.device != w.device or w.dtype != torch.float32:
        w = w.detach()
        return w if w.dtype == torch.bfloat16 else w.to(torch.bfloat16)
    if w._gcow_bf16_version != w._version:
        sh.copy_(w.detach())
        w._gcow_bf16_version = w._version
    return sh


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, *, bias: torch.Tensor | None = None,
              residual: torch.Tensor | None = None, gelu: bool = False, out_dtype=torch.bfloat16,
              out: torch.Tensor | None = None, accumulate: bool = False, max_ctas: int = 0,
              a_t: bool = False, b_t: bool = False, tile_rows: int = 0,
              pre_gelu_out: torch.Tensor | None = None, gelu_grad_of: torch.Tensor | None = None) -> torch.Tensor:
    """C[M,N] = op(A) @ op(B)^T (+bias) (GELU) (+residual) on the tcgen05 kernel.

    ``pre_gelu_out`` (bf16 [M,N], with ``gelu``): also receives the value before the GELU, which its
    gradient needs. ``gelu_grad_of`` (bf16 [M,N]): the product is multiplied by GELU'(that tensor) before
    the residual is added, i.e. the backward of a GELU fused into the GEMM that produces its input gradient.

    a: bf16 [M,K] (or [K,M] with ``a_t``: the stored matrix is used transposed without a
    copy). b: bf16 [N,K] (or [K,N] with ``b_t``). Last dimension contiguous, leading
    dimensions multiples of 8. bias: fp32 [N]. residual/out: [M,N] of ``out_dtype``.
    ``tile_rows`` forces the 128- or 256-row tile (0: chosen from the problem size)."""
    global _launches
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.dim() == 2 and b.dim() == 2
    assert a.stride(1) == 1 and b.stride(1) == 1
    (K, M) = a.shape if a_t else a.shape[::-1]
    (Kb, N) = b.shape if b_t else b.shape[::-1]
    assert K == Kb, (a.shape, b.shape, a_t, b_t)
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    flags = (OUT_F32 if out.dtype == torch.float32 else 0) | (BIAS if bias is not None else 0) | \
        (GELU if gelu else 0) | (RESIDUAL if residual is not None else 0) | (ACCUMULATE if accumulate else 0)
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == N
    if residual is not None:
        assert residual.dtype == out.dtype and residual.stride() == out.stride()
    aux = pre_gelu_out if pre_gelu_out is not None else gelu_grad_of
    if aux is not None:
        assert pre_gelu_out is None or gelu_grad_of is None
        flags |= AUX_OUT if pre_gelu_out is not None else GELU_GRAD
    if (_pair_gemm_enabled() and not a_t and out.dtype == torch.bfloat16 and not accumulate and max_ctas == 0
            and tile_rows == 0 and K % 64 == 0 and K >= 512 and N % (64 if b_t else 32) == 0 and M >= 1024 and N >= 256
            and a.stride(0) % 8 == 0 and b.stride(0) % 8 == 0 and out.stride(0) % 8 == 0
            and not (K >= 2048 and -(-M // 256) * -(-N // 256) >= 118)):
        # large product with a short reduction: the CTA-pair kernel (two SMs per 256 x 256 tile) has the one-CTA
        # 256 x 256 tile's traffic per flop AND an overlapped epilogue; long reductions stay on the one-CTA tile, and
        # so do reductions below 512 (the 1x1 convolutions of a ResNet), which are bound by the output stream: there
        # the one-CTA kernel's TMA-store epilogue is 15-30 % faster
        err = _native.cuda().gcow_gemm2_bf16(
            a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0),
            bias.data_ptr() if bias is not None else None, residual.data_ptr() if residual is not None else None,
            aux.data_ptr() if aux is not None else None, flags, _error_word(a.device).data_ptr(), int(b_t),
            torch.cuda.current_stream(a.device).cuda_stream)
        if err == 0:
            _launches += 1
            return out
        if err != -2:
            raise RuntimeError(f"gcow_gemm2_bf16 refused the call: {err}")
    if aux is not None:
        assert aux.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and aux.shape == out.shape
        assert aux.stride() == out.stride() and N % 32 == 0 and max_ctas == 0
        err = _native.cuda().gcow_gemm_bf16_aux(
            a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0),
            bias.data_ptr() if bias is not None else None, residual.data_ptr() if residual is not None else None,
            aux.data_ptr(), flags, _error_word(a.device).data_ptr(), int(a_t), int(b_t), int(tile_rows),
            torch.cuda.current_stream(a.device).cuda_stream)
    else:
        err = _native.cuda().gcow_gemm_bf16(
            a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0),
            bias.data_ptr() if bias is not None else None, residual.data_ptr() if residual is not None else None,
            flags, _error_word(a.device).data_ptr(), max_ctas, int(a_t), int(b_t), int(tile_rows),
            torch.cuda.current_stream(a.device).cuda_stream)
    if err:
        raise RuntimeError(f"gcow_gemm_bf16 refused the call: {err}")
    _launches += 1
    return out


_pair_gemm = None


def _pair_gemm_enabled() -> bool:
    """The CTA-pair GEMM (cta_group::2) serves large products with a short reduction unless GCOW_GEMM2=0, provided
    the device can co-schedule clusters of two CTAs with its shared-memory footprint."""
    global _pair_gemm
    if _pair_gemm is None:
        import os
        _pair_gemm = (os.environ.get("GCOW_GEMM2", "1") != "0" and _have("gcow_gemm2_bf16")
                      and _native.cuda().gcow_gemm2_max_pairs() > 0)
    return _pair_gemm


def take_grad_view(w: torch.Tensor):
    """The float32 tensor this step's gradient of ``w`` may be written into, or None. A trainer that knows where the
    gradient will end up (DDP's bucket view, i.e. last step's ``w.grad``) leaves it in ``w._gcow_grad_view`` before it
    drops the gradients; the first layer to use ``w`` in a forward pass takes it, so two uses of one weight never share
    it. The weight-gradient kernels then write there and the backward returns an alias of that memory: autograd adopts
    it as ``w.grad`` and DDP, seeing its own bucket memory, copies nothing."""
    gv = getattr(w, "_gcow_grad_view", None)
    if gv is None:
        return None
    w._gcow_grad_view = None
    if gv.dtype != torch.float32 or gv.shape != w.shape or gv.device != w.device:
        return None
    return (gv, w)


def _grad_target(taken, rows: int, cols: int, align: int = 16):
    """(flat [rows, cols] view to write into, tensor to return as the gradient) or (None, None). ``align``: what the
    writing kernel needs of the address (the GEMM and convolution epilogues store 16 bytes at a time)."""
    if taken is None:
        return None, None
    gv, w = taken
    if w.grad is not None:                       # gradients are being accumulated: that memory is in use
        return None, None
    flat = gv.permute(0, 2, 3, 1) if gv.dim() == 4 else gv
    if not flat.is_contiguous() or flat.numel() != rows * cols:
        return None, None
    flat = flat.reshape(rows, cols)
    if flat.data_ptr() != gv.data_ptr() or gv.data_ptr() % align:
        return None, None
    global _grad_view_hits
    _grad_view_hits += 1
    return flat, gv.as_strided(gv.shape, gv.stride())


_grad_view_hits = 0


def grad_view_hits() -> int:
    """How many weight gradients were written straight into the tensor the trainer pointed at (see take_grad_view)."""
    return _grad_view_hits


def wgrad_gemm(g: torch.Tensor, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """dW[N, K] = g^T x for g [M, N], x [M, K] (both stored with the reduction dimension M outermost), fp32.
    The output has few tiles while M is long, so the reduction is split across CTAs: the rows are cut into
    ``s`` slabs that run as one batched launch, and the ``s`` partial products are added in a fixed order.
    ``out`` (contiguous fp32 [N, K]): where the result goes."""
    global _launches
    M, N = g.shape
    K = x.shape[1]
    tiles = -(-N // 128) * -(-K // 256)
    s = 1        # doubled while the tiles still fit one wave of 148 CTAs and a slab keeps at least 512 rows
    while s < 64 and tiles * s * 2 <= 148 and M % (2 * s) == 0 and (M // (2 * s)) % 64 == 0 and M // (2 * s) >= 512:
        s *= 2
    if s == 1 or g.stride(0) != N or x.stride(0) != K:
        return gemm_bf16(g, x, a_t=True, b_t=True, out_dtype=torch.float32, out=out)
    lib = _native.cuda()
    part = _ws("wgrad_part", (s, N, K), torch.float32, g.device)
    err = lib.gcow_gemm_bf16_batched(
        g.data_ptr(), x.data_ptr(), part.data_ptr(), N, K, M // s, N, K, K, s, (M // s) * N, (M // s) * K, N * K,
        None, None, OUT_F32, _error_word(g.device).data_ptr(), 1, 1, 0, _stream(g.device))
    _chk(err, "gcow_gemm_bf16_batched")
    if out is None:
        out = torch.empty((N, K), dtype=torch.float32, device=g.device)
    _chk(lib.gcow_reduce_partials(part.data_ptr(), out.data_ptr(), s, N * K, _stream(g.device)), "gcow_reduce_partials")
    _launches += 2
    return out


def _gemm_ok(x2d: torch.Tensor, w: torch.Tensor) -> bool:
    return x2d.is_cuda and x2d.shape[1] % 8 == 0 and w.shape[1] % 8 == 0 and x2d.shape[0] >= 64


def _pad_rows(t: torch.Tensor, rows: int) -> torch.Tensor:
    if t.shape[0] == rows:
        return t
    out = torch.zeros((rows,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    out[:t.shape[0]] = t
    return out


class _LinearFn(torch.autograd.Function):
    """y = x W^T + b with all three GEMMs (forward, dgrad, wgrad) on the tcgen05 kernel.
    An output width that is not a multiple of 8 (e.g. a 30522-word vocabulary) is
    padded internally: the result is a [.., N] view of a [M, N8] buffer whose pad
    columns are zero-weighted."""

    @staticmethod
    def forward(ctx, x, w, b):
        N = w.shape[0]
        N8 = (N + 7) // 8 * 8
        xb = x.reshape(-1, x.shape[-1]).to(torch.bfloat16).contiguous()
        wb = _pad_rows(bf16_weight(w).contiguous(), N8)
        bias = _pad_rows(b.float().contiguous(), N8) if b is not None else None
        y = gemm_bf16(xb, wb, bias=bias)
        ctx.save_for_backward(xb, wb)
        ctx.meta = (x.shape, w.dtype, b is not None, N, N8)
        ctx.grad_view = take_grad_view(w) if (N == N8 and w.dtype == torch.float32) else None
        return y[:, :N].view(*x.shape[:-1], N) if N == N8 else y[:, :N].unflatten(0, x.shape[:-1])

    @staticmethod
    def backward(ctx, gy):
        xb, wb = ctx.saved_tensors
        x_shape, w_dtype, has_bias, N, N8 = ctx.meta
        M = xb.shape[0]
        g = gy.reshape(M, N) if gy.is_contiguous() or N == N8 else gy.flatten(0, -2)
        if (g.dtype == torch.bfloat16 and g.stride(1) == 1 and g.stride(0) == N8 and g.storage_offset() == 0
                and g.untyped_storage().nbytes() >= M * N8 * 2):
            g = g.as_strided((M, N8), (N8, 1))          # the padded buffer itself (pad columns are zero)
        else:
            g = g.to(torch.bfloat16)
            if N != N8:
                gp = torch.zeros((M, N8), dtype=torch.bfloat16, device=g.device)
                gp[:, :N] = g
                g = gp
            else:
                g = g.contiguous()
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            # dx[M,K] = g[M,N] @ W[N,K]: W is stored [reduction N][K], i.e. the B operand transposed
            gx = gemm_bf16(g, wb, b_t=True).view(x_shape)
        if ctx.needs_input_grad[1]:
            # dW[N,K] = g^T @ x: both g [M,N] and x [M,K] are stored [reduction M][rows]
            flat, alias = _grad_target(ctx.grad_view, N, xb.shape[1])
            if flat is not None:
                wgrad_gemm(g, xb, out=flat)
                gw = alias
            else:
                gw = wgrad_gemm(g, xb)[:N].to(w_dtype)
        if has_bias and ctx.needs_input_grad[2]:
            gb = colsum(g)[:N]
        return gx, gw, gb


class _LinearResidualFn(torch.autograd.Function):
    """y = r + x W^T + b with the residual added in the GEMM epilogue."""

    @staticmethod
    def forward(ctx, x, w, b, r):
        xb = x.reshape(-1, x.shape[-1]).to(torch.bfloat16).contiguous()
        wb = bf16_weight(w).contiguous()
        rb = r.reshape(-1, r.shape[-1]).to(torch.bfloat16).contiguous()
        y = gemm_bf16(xb, wb, bias=b.float().contiguous() if b is not None else None, residual=rb)
        ctx.save_for_backward(xb, wb)
        ctx.meta = (x.shape, r.shape, b is not None)
        ctx.grad_view = take_grad_view(w)
        return y.view(r.shape)

    @staticmethod
    def backward(ctx, gy):
        xb, wb = ctx.saved_tensors
        x_shape, r_shape, has_bias = ctx.meta
        g = gy.reshape(-1, gy.shape[-1]).to(torch.bfloat16).contiguous()
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            gx = gemm_bf16(g, wb, b_t=True).view(x_shape)
        if ctx.needs_input_grad[1]:
            flat, alias = _grad_target(ctx.grad_view, wb.shape[0], wb.shape[1])
            gw = wgrad_gemm(g, xb, out=flat)
            if flat is not None:
                gw = alias
        if has_bias and ctx.needs_input_grad[2]:
            gb = colsum(g)
        return gx, gw, gb, (gy if ctx.needs_input_grad[3] else None)


class _FfnResidualFn(torch.autograd.Function):
    """y = x + GELU(x W1^T + b1) W2^T + b2 as two GEMMs forward and four backward, with every elementwise
    step in a GEMM epilogue: bias + GELU (keeping the pre-activation), bias + residual, GELU' on the way
    back, and the sum of the two gradient paths into x."""

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2):
        xb = x.reshape(-1, x.shape[-1]).to(torch.bfloat16).contiguous()
        w1b, w2b = bf16_weight(w1).contiguous(), bf16_weight(w2).contiguous()
        M, F = xb.shape[0], w1b.shape[0]
        pre = torch.empty((M, F), dtype=torch.bfloat16, device=xb.device)
        act = gemm_bf16(xb, w1b, bias=b1.float().contiguous(), gelu=True, pre_gelu_out=pre)
        y = gemm_bf16(act, w2b, bias=b2.float().contiguous(), residual=xb)
        ctx.save_for_backward(xb, w1b, w2b, pre, act)
        ctx.shape = x.shape
        ctx.grad_views = (take_grad_view(w1), take_grad_view(w2))
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, gy):
        xb, w1b, w2b, pre, act = ctx.saved_tensors
        g = gy.reshape(-1, gy.shape[-1]).to(torch.bfloat16).contiguous()
        dpre = gemm_bf16(g, w2b, b_t=True, gelu_grad_of=pre)                 # (g W2) * GELU'(pre)
        gw1 = gw2 = None
        if ctx.needs_input_grad[3]:
            flat, alias = _grad_target(ctx.grad_views[1], w2b.shape[0], w2b.shape[1])
            gw2 = wgrad_gemm(g, act, out=flat)
            if flat is not None:
                gw2 = alias
        gb2 = colsum(g) if ctx.needs_input_grad[4] else None
        gx = gemm_bf16(dpre, w1b, b_t=True, residual=g).view(ctx.shape) if ctx.needs_input_grad[0] else None
        if ctx.needs_input_grad[1]:
            flat, alias = _grad_target(ctx.grad_views[0], w1b.shape[0], w1b.shape[1])
            gw1 = wgrad_gemm(dpre, xb, out=flat)
            if flat is not None:
                gw1 = alias
        gb1 = colsum(dpre) if ctx.needs_input_grad[2] else None
        return gx, gw1, gb1, gw2, gb2


def fused_mlp_usable(x: torch.Tensor, *weights: torch.Tensor) -> bool:
    """Inputs on the GPU, the aux-epilogue entry built, every width a multiple of 32."""
    if not (x.is_cuda and _have("gcow_gemm_bf16_aux") and x.shape[-1] % 32 == 0):
        return False
    return all(w.shape[0] % 32 == 0 and w.shape[1] % 32 == 0 for w in weights) and x.numel() // x.shape[-1] >= 64


def linear_residual(x, w, b, r):
    return _LinearResidualFn.apply(x, w, b, r)


def ffn_residual(x, w1, b1, w2, b2):
    return _FfnResidualFn.apply(x, w1, b1, w2, b2)


def gemm_usable(x: torch.Tensor, w: torch.Tensor) -> bool:
    if not (x.is_cuda and _have("gcow_gemm_bf16")):
        return False
    x2 = x.reshape(-1, x.shape[-1])
    return _gemm_ok(x2, w)


def linear(x, w, b):
    return _LinearFn.apply(x, w, b)


def _stream(dev):
    return torch.cuda.current_stream(dev).cuda_stream


def _chk(err: int, what: str) -> None:
    if err:
        raise RuntimeError(f"{what} refused the call: {err}")


def colsum(g: torch.Tensor) -> torch.Tensor:
    """fp32 column sums of a bf16 [rows, cols] matrix (bias gradient)."""
    global _launches
    rows, cols = g.shape
    lib = _native.cuda()
    if cols % 2 or g.stride(1) != 1 or g.stride(0) % 2:
        return g.float().sum(0)
    parts = lib.gcow_colsum_parts(rows)
    part = _ws("colsum_part", parts * cols, torch.float32, g.device)
    out = torch.empty(cols, dtype=torch.float32, device=g.device)
    _chk(lib.gcow_colsum(g.data_ptr(), part.data_ptr(), out.data_ptr(), rows, cols, g.stride(0), _stream(g.device)),
         "gcow_colsum")
    _launches += 2
    return out


# ------------------------------------------------------------------ 1x1 conv
class _Conv1x1Fn(torch.autograd.Function):
    """1x1 stride-1 convolution on channels-last activations as a GEMM:
    [N*H*W, Cin] x [Cout, Cin]^T."""

    @staticmethod
    def forward(ctx, x, w, b):
        N, C, H, W = x.shape
        xm = x.permute(0, 2, 3, 1).reshape(-1, C)          # a view for channels-last input
        if xm.dtype != torch.bfloat16 or not xm.is_contiguous():
            xm = xm.to(torch.bfloat16).contiguous()
        wb = bf16_weight(w).reshape(w.shape[0], C).contiguous()
        y = gemm_bf16(xm, wb, bias=b.float().contiguous() if b is not None else None)
        ctx.save_for_backward(xm, wb)
        ctx.meta = (N, C, H, W, w.shape, w.dtype, b is not None)
        ctx.grad_view = take_grad_view(w) if w.dtype == torch.float32 else None
        return y.view(N, H, W, w.shape[0]).permute(0, 3, 1, 2)

    @staticmethod
    def backward(ctx, gy):
        xm, wb = ctx.saved_tensors
        N, C, H, W, wshape, wdtype, has_bias = ctx.meta
        g = gy.permute(0, 2, 3, 1).reshape(-1, wshape[0])
        if g.dtype != torch.bfloat16 or not g.is_contiguous():
            g = g.to(torch.bfloat16).contiguous()
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            gx = gemm_bf16(g, wb, b_t=True).view(N, H, W, C).permute(0, 3, 1, 2)
        if ctx.needs_input_grad[1]:
            flat, alias = _grad_target(ctx.grad_view, wshape[0], C)
            if flat is not None:
                wgrad_gemm(g, xm, out=flat)
                gw = alias
            else:
                gw = wgrad_gemm(g, xm)
                gw = gw.view(wshape).to(wdtype).contiguous(memory_format=torch.channels_last)
        if has_bias and ctx.needs_input_grad[2]:
            gb = colsum(g)
        return gx, gw, gb


class _SubsampleFn(torch.autograd.Function):
    """x[:, :, ::s, ::s] of a channels-last bf16 tensor as a dense channels-last tensor (what a strided 1x1 convolution
    reads); the backward writes the gradient at the sampled pixels and zeros elsewhere in one kernel."""

    @staticmethod
    def forward(ctx, x, s):
        global _launches
        N, C, H, W = x.shape
        if x.dtype != torch.bfloat16 or not x.is_contiguous(memory_format=torch.channels_last):
            x = x.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        OH, OW = (H + s - 1) // s, (W + s - 1) // s
        y = torch.empty((N, C, OH, OW), dtype=torch.bfloat16, device=x.device, memory_format=torch.channels_last)
        _chk(_native.cuda().gcow_subsample(x.data_ptr(), y.data_ptr(), N, H, W, C, s, 0, _stream(x.device)), "gcow_subsample")
        _launches += 1
        ctx.meta = (N, C, H, W, s)
        return y

    @staticmethod
    def backward(ctx, gy):
        global _launches
        N, C, H, W, s = ctx.meta
        if gy.dtype != torch.bfloat16 or not gy.is_contiguous(memory_format=torch.channels_last):
            gy = gy.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        gx = torch.empty((N, C, H, W), dtype=torch.bfloat16, device=gy.device, memory_format=torch.channels_last)
        _chk(_native.cuda().gcow_subsample(gy.data_ptr(), gx.data_ptr(), N, H, W, C, s, 1, _stream(gy.device)),
             "gcow_subsample (gradient)")
        _launches += 1
        return gx, None


def subsample(x: torch.Tensor, s: int) -> torch.Tensor:
    return _SubsampleFn.apply(x, s)


def conv1x1_usable(x: torch.Tensor, w: torch.Tensor) -> bool:
    if not (x.is_cuda and x.dim() == 4 and _have("gcow_gemm_bf16")):
        return False
    cin, cout = x.shape[1], w.shape[0]
    rows = x.shape[0] * x.shape[2] * x.shape[3]
    return cin % 8 == 0 and cout % 8 == 0 and rows % 8 == 0 and rows >= 128 and \
        x.is_contiguous(memory_format=torch.channels_last)


def conv1x1(x, w, b):
    return _Conv1x1Fn.apply(x, w, b)


# ----------------------------------------------------------------- LayerNorm
class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, eps):
        global _launches
        H = x.shape[-1]
        xb = x.reshape(-1, H).to(torch.bfloat16).contiguous()
        rows = xb.shape[0]
        y = torch.empty_like(xb)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty_like(mean)
        g32, b32 = gamma.float().contiguous(), beta.float().contiguous()
        _chk(_native.cuda().gcow_layernorm_fwd(xb.data_ptr(), g32.data_ptr(), b32.data_ptr(), y.data_ptr(),
                                               mean.data_ptr(), rstd.data_ptr(), rows, H, eps, _stream(x.device)),
             "gcow_layernorm_fwd")
        _launches += 1
        ctx.save_for_backward(xb, g32, mean, rstd)
        ctx.shape, ctx.pdtype = x.shape, gamma.dtype
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, gy):
        global _launches
        xb, g32, mean, rstd = ctx.saved_tensors
        rows, H = xb.shape
        g = gy.reshape(rows, H).to(torch.bfloat16).contiguous()
        lib = _native.cuda()
        dx = torch.empty_like(xb)
        parts = lib.gcow_layernorm_bwd_parts(rows)
        part = _ws("ln_part", parts * 2 * H, torch.float32, xb.device)
        dgb = torch.empty(2 * H, dtype=torch.float32, device=xb.device)
        _chk(lib.gcow_layernorm_bwd(g.data_ptr(), xb.data_ptr(), g32.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                    dx.data_ptr(), part.data_ptr(), dgb.data_ptr(), rows, H, _stream(xb.device)),
             "gcow_layernorm_bwd")
        _launches += 2
        return dx.view(ctx.shape), dgb[:H].to(ctx.pdtype), dgb[H:].to(ctx.pdtype), None


def layernorm_usable(x: torch.Tensor, mod) -> bool:
    H = x.shape[-1]
    return x.is_cuda and _have("gcow_layernorm_fwd") and H % 8 == 0 and H <= 4096 and \
        mod.elementwise_affine and mod.bias is not None and len(mod.normalized_shape) == 1


def layernorm(x, w, b, eps):
    return _LayerNormFn.apply(x, w, b, eps)


# ---------------------------------------------------------------------- GELU
class _GeluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        global _launches
        xb = x.to(torch.bfloat16).contiguous()
        y = torch.empty_like(xb)
        _chk(_native.cuda().gcow_gelu_fwd(xb.data_ptr(), y.data_ptr(), xb.numel(), _stream(x.device)), "gcow_gelu_fwd")
        _launches += 1
        ctx.save_for_backward(xb)
        return y

    @staticmethod
    def backward(ctx, gy):
        global _launches
        (xb,) = ctx.saved_tensors
        g = gy.to(torch.bfloat16).contiguous()
        dx = torch.empty_like(xb)
        _chk(_native.cuda().gcow_gelu_bwd(g.data_ptr(), xb.data_ptr(), dx.data_ptr(), xb.numel(), _stream(xb.device)),
             "gcow_gelu_bwd")
        _launches += 1
        return dx


def gelu_usable(x: torch.Tensor) -> bool:
    return x.is_cuda and _have("gcow_gelu_fwd") and x.numel() % 8 == 0


def gelu(x):
    return _GeluFn.apply(x)


# ------------------------------------------------------ softmax cross-entropy
class _XentFn(torch.autograd.Function):
    """Mean cross-entropy over non-ignored rows. The forward kernel leaves the
    gradient (softmax - onehot) / count in the logits buffer, which therefore must
    not be used again by the caller."""

    @staticmethod
    def forward(ctx, logits, target, ignore_index, valid_cols):
        global _launches
        rows, ld = logits.shape[0], logits.stride(0)
        count = (target != ignore_index).sum().float().reshape(1)
        row_loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
        _chk(_native.cuda().gcow_softmax_xent(logits.data_ptr(), target.data_ptr(), row_loss.data_ptr(),
                                              count.data_ptr(), rows, valid_cols, ld, ignore_index,
                                              _stream(logits.device)), "gcow_softmax_xent")
        _launches += 1
        # the kernel has turned `logits` into its own gradient; keep that buffer
        ctx.grad_buf = logits.detach()
        return row_loss.sum()

    @staticmethod
    def backward(ctx, g):
        grad = ctx.grad_buf
        ctx.grad_buf = None
        # Scale in place (the buffer is this function's own since the forward overwrote it), and over the whole
        # padded rows when they are one block of memory: the result is then still a view of that buffer, which the
        # linear layer below can hand to its GEMMs without re-padding a [rows, vocabulary] tensor.
        rows, ld = grad.shape[0], grad.stride(0)
        scale = g.to(grad.dtype)
        if grad.storage_offset() == 0 and grad.untyped_storage().nbytes() >= rows * ld * grad.element_size():
            grad.as_strided((rows, ld), (ld, 1)).mul_(scale)
        else:
            grad.mul_(scale)
        return grad, None, None, None


def xent_usable(logits: torch.Tensor) -> bool:
    return (logits.is_cuda and _have("gcow_softmax_xent") and logits.dtype == torch.bfloat16 and logits.dim() == 2
            and logits.stride(1) == 1 and logits.stride(0) % 8 == 0 and logits.requires_grad
            and not logits.is_leaf)


def softmax_xent(logits, target, ignore_index=-100, valid_cols=None):
    return _XentFn.apply(logits, target, ignore_index, valid_cols or logits.shape[1])


# ------------------------------------------------------- image normalisation
def u8_to_bf16_norm(x_u8: torch.Tensor, mean255, std255) -> torch.Tensor:
    """uint8 NHWC [N,H,W,3] -> normalised bf16 tensor of logical shape [N,3,H,W] in
    channels-last memory."""
    global _launches
    import ctypes as C_
    N, H, W, C = x_u8.shape
    assert C == 3 and x_u8.is_contiguous()
    y = torch.empty((N, H, W, 3), dtype=torch.bfloat16, device=x_u8.device)
    m = (C_.c_float * 3)(*mean255)
    s = (C_.c_float * 3)(*std255)
    _chk(_native.cuda().gcow_u8_to_bf16_norm(x_u8.data_ptr(), y.data_ptr(), N * H * W, 3, m, s, _stream(x_u8.device)),
         "gcow_u8_to_bf16_norm")
    _launches += 1
    return y.permute(0, 3, 1, 2)


# ------------------------------------------------- BatchNorm (+add) (+ReLU)
def _nhwc_rows(x: torch.Tensor):
    N, C, H, W = x.shape
    return N * H * W, C


class _BatchNormActFn(torch.autograd.Function):
    """y = relu?(bn(x) (+ residual)) on channels-last bf16 tensors, training statistics.

    With ``fork`` the result is returned twice, as two tensors on the same memory: a layer output that feeds two
    consumers (the next block's first convolution and its identity branch) then gets its two gradients delivered
    separately, and the first backward sweep adds them while it reads them - instead of autograd's addition kernel
    (two reads and a write of the whole tensor) followed by a third read here."""

    @staticmethod
    def forward(ctx, x, gamma, beta, run_mean, run_var, residual, relu, momentum, eps, fork=False):
        global _launches
        R, C = _nhwc_rows(x)
        lib = _native.cuda()
        y = torch.empty_like(x, memory_format=torch.channels_last)
        stats = torch.empty(4 * C, dtype=torch.float32, device=x.device)
        part = _ws("bn_part", lib.gcow_bn_parts(R, C) * 2 * C, torch.float32, x.device)
        g32, b32 = gamma.float().contiguous(), beta.float().contiguous()
        mask = torch.empty(R * C // 8, dtype=torch.uint8, device=x.device) if relu else None
        _chk(lib.gcow_bn_fwd_train(x.data_ptr(), residual.data_ptr() if residual is not None else None, y.data_ptr(),
                                   mask.data_ptr() if mask is not None else None, g32.data_ptr(), b32.data_ptr(),
                                   run_mean.data_ptr() if run_mean is not None else None,
                                   run_var.data_ptr() if run_var is not None else None,
                                   stats.data_ptr(), part.data_ptr(), R, C, eps, momentum, int(relu), _stream(x.device)),
             "gcow_bn_fwd_train")
        _launches += 3
        ctx.save_for_backward(x, mask, g32, stats)      # the ReLU bit mask stands in for y in the backward
        ctx.grad_views = (take_grad_view(gamma), take_grad_view(beta)) if gamma.dtype == torch.float32 else (None, None)
        ctx.meta = (R, C, bool(relu), residual is not None, gamma.dtype)
        if not fork:
            return y
        # a second tensor on the same storage (not an autograd view of the first)
        y2 = torch.empty(0, dtype=y.dtype, device=y.device).set_(y.untyped_storage(), y.storage_offset(), y.size(), y.stride())
        return y, y2

    @staticmethod
    def backward(ctx, gy, gy2=None):
        global _launches
        x, mask, g32, stats = ctx.saved_tensors
        R, C, relu, has_res, pdtype = ctx.meta
        lib = _native.cuda()
        if gy is None:
            gy, gy2 = gy2, None

        def _cl(t):
            if t.dtype != torch.bfloat16 or not t.is_contiguous(memory_format=torch.channels_last):
                t = t.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
            return t
        gy = _cl(gy)
        gy2 = _cl(gy2) if gy2 is not None else None
        dx = torch.empty_like(x, memory_format=torch.channels_last)
        # the masked (summed) gradient: the residual input's gradient, and what the second sweep reads
        dres = torch.empty_like(x, memory_format=torch.channels_last) if (has_res or gy2 is not None) else None
        part = _ws("bn_part", lib.gcow_bn_parts(R, C) * 2 * C, torch.float32, x.device)
        # dgamma and dbeta go straight into the two parameters' gradient tensors when the trainer pointed at them
        fg, ag = _grad_target(ctx.grad_views[0], 1, C, align=4)
        fb, ab = _grad_target(ctx.grad_views[1], 1, C, align=4) if fg is not None else (None, None)
        if fb is not None and _have("gcow_bn_bwd3"):
            dgamma, dbeta = ag, ab
            pg, pb = fg.data_ptr(), fb.data_ptr()
        else:
            dgb = torch.empty(2 * C, dtype=torch.float32, device=x.device)
            dgamma, dbeta = dgb[:C].to(pdtype), dgb[C:].to(pdtype)
            pg, pb = dgb.data_ptr(), dgb.data_ptr() + 4 * C
        _chk(lib.gcow_bn_bwd3(gy.data_ptr(), gy2.data_ptr() if gy2 is not None else None,
                              mask.data_ptr() if mask is not None else None, x.data_ptr(), g32.data_ptr(),
                              stats.data_ptr(), dx.data_ptr(),
                              dres.data_ptr() if dres is not None else None, pg, pb, part.data_ptr(), R, C,
                              int(relu), _stream(x.device)), "gcow_bn_bwd3")
        _launches += 3
        return dx, dgamma, dbeta, None, None, (dres if has_res else None), None, None, None, None


def batchnorm_usable(x: torch.Tensor, mod, residual=None) -> bool:
    if not (x.is_cuda and x.dim() == 4 and x.dtype == torch.bfloat16 and _have("gcow_bn_fwd_train")):
        return False
    if not x.is_contiguous(memory_format=torch.channels_last) or not mod.affine:
        return False
    if residual is not None and not (residual.dtype == torch.bfloat16 and residual.shape == x.shape
                                     and residual.is_contiguous(memory_format=torch.channels_last)):
        return False
    return bool(_native.cuda().gcow_bn_supported(x.shape[1]))


def batchnorm_act(x, mod, residual=None, relu=False, fork=False):
    """Fused BN(+add)(+ReLU) using ``mod``'s parameters and running statistics. ``fork``: return the result as two
    tensors on the same memory (see _BatchNormActFn)."""
    global _launches
    if mod.training or not mod.track_running_stats:
        if mod.training and mod.track_running_stats and mod.num_batches_tracked is not None:
            # counted on the host and added to the tensor when somebody looks (state_dict, ops.nn.BatchNorm2d): one
            # tiny kernel per layer and step otherwise, 53 of them in a ResNet-50 step
            mod._gcow_pending_batches = getattr(mod, "_gcow_pending_batches", 0) + 1
        mom = mod.momentum if mod.momentum is not None else 0.1
        rm = mod.running_mean if (mod.training and mod.track_running_stats) else None
        rv = mod.running_var if (mod.training and mod.track_running_stats) else None
        return _BatchNormActFn.apply(x, mod.weight, mod.bias, rm, rv, residual, relu, mom, mod.eps, fork)
    R, C = _nhwc_rows(x)
    y = torch.empty_like(x, memory_format=torch.channels_last)
    scratch = torch.empty(2 * C, dtype=torch.float32, device=x.device)
    _chk(_native.cuda().gcow_bn_fwd_eval(x.data_ptr(), residual.data_ptr() if residual is not None else None, y.data_ptr(),
                                         mod.weight.float().data_ptr(), mod.bias.float().data_ptr(),
                                         mod.running_mean.data_ptr(), mod.running_var.data_ptr(), scratch.data_ptr(),
                                         R, C, mod.eps, int(relu), _stream(x.device)), "gcow_bn_fwd_eval")
    _launches += 2
    return (y, y) if fork else y


# ------------------------------------------------------------------- pooling
class _MaxPool3x3s2Fn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        global _launches
        N, C, H, W = x.shape
        OH, OW = (H - 1) // 2 + 1, (W - 1) // 2 + 1
        y = torch.empty((N, C, OH, OW), dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
        idx = torch.empty((N, OH, OW, C), dtype=torch.uint8, device=x.device)
        _chk(_native.cuda().gcow_maxpool3x3s2_fwd(x.data_ptr(), y.data_ptr(), idx.data_ptr(), N, H, W, C, _stream(x.device)),
             "gcow_maxpool3x3s2_fwd")
        _launches += 1
        ctx.save_for_backward(idx)
        ctx.shape = (N, C, H, W)
        return y

    @staticmethod
    def backward(ctx, gy):
        global _launches
        (idx,) = ctx.saved_tensors
        N, C, H, W = ctx.shape
        if gy.dtype != torch.bfloat16 or not gy.is_contiguous(memory_format=torch.channels_last):
            gy = gy.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        dx = torch.empty((N, C, H, W), dtype=torch.bfloat16, device=gy.device, memory_format=torch.channels_last)
        _chk(_native.cuda().gcow_maxpool3x3s2_bwd(gy.data_ptr(), idx.data_ptr(), dx.data_ptr(), N, H, W, C, _stream(gy.device)),
             "gcow_maxpool3x3s2_bwd")
        _launches += 1
        return dx


class _GlobalAvgPoolFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        global _launches
        N, C, H, W = x.shape
        y = torch.empty((N, C, 1, 1), dtype=x.dtype, device=x.device)
        _chk(_native.cuda().gcow_avgpool_fwd(x.data_ptr(), y.data_ptr(), N, H * W, C, _stream(x.device)), "gcow_avgpool_fwd")
        _launches += 1
        ctx.shape = (N, C, H, W)
        return y

    @staticmethod
    def backward(ctx, gy):
        global _launches
        N, C, H, W = ctx.shape
        g = gy.reshape(N, C).to(torch.bfloat16).contiguous()
        dx = torch.empty((N, C, H, W), dtype=torch.bfloat16, device=gy.device, memory_format=torch.channels_last)
        _chk(_native.cuda().gcow_avgpool_bwd(g.data_ptr(), dx.data_ptr(), N, H * W, C, _stream(gy.device)), "gcow_avgpool_bwd")
        _launches += 1
        return dx


def pool_usable(x: torch.Tensor) -> bool:
    return (x.is_cuda and x.dim() == 4 and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.is_contiguous(memory_format=torch.channels_last) and _have("gcow_maxpool3x3s2_fwd"))


def maxpool3x3s2(x):
    return _MaxPool3x3s2Fn.apply(x)


def global_avgpool(x):
    return _GlobalAvgPoolFn.apply(x)


# ------------------------------------------------ convolution as im2col + GEMM
class _ConvGemmFn(torch.autograd.Function):
    """KxK convolution (any stride/padding, groups = 1) on channels-last bf16 input:
    own im2col -> tcgen05 GEMM -> (backward) GEMMs + own col2im."""

    @staticmethod
    def forward(ctx, x, w, b, stride, pad):
        global _launches
        N, C, H, W = x.shape
        Co, _, KH, KW = w.shape
        OH, OW = (H + 2 * pad - KH) // stride + 1, (W + 2 * pad - KW) // stride + 1
        lib = _native.cuda()
        if x.dtype != torch.bfloat16 or not x.is_contiguous(memory_format=torch.channels_last):
            x = x.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        K = KH * KW * C
        Kp = (K + 7) // 8 * 8          # row length of the patch matrix: a multiple of 8 (16-byte rows for TMA)
        col = torch.empty((N * OH * OW, Kp), dtype=torch.bfloat16, device=x.device)
        if C % 8 == 0:
            _chk(lib.gcow_im2col(x.data_ptr(), col.data_ptr(), N, H, W, C, KH, KW, stride, pad, _stream(x.device)), "gcow_im2col")
        else:                          # e.g. the 3-channel image in front of the stem; padded columns are zero
            _chk(lib.gcow_im2col_anyc(x.data_ptr(), col.data_ptr(), N, H, W, C, KH, KW, stride, pad, Kp, _stream(x.device)),
                 "gcow_im2col_anyc")
        _launches += 1
        wr = bf16_weight(w).permute(0, 2, 3, 1).reshape(Co, K)                                   # [Co, (kh,kw,c)]
        if Kp != K:
            wr = torch.nn.functional.pad(wr, (0, Kp - K))
        wr = wr.contiguous()
        y = gemm_bf16(col, wr, bias=b.float().contiguous() if b is not None else None)
        ctx.save_for_backward(col, wr)
        ctx.meta = (N, C, H, W, Co, KH, KW, OH, OW, stride, pad, w.dtype, b is not None)
        return y.view(N, OH, OW, Co).permute(0, 3, 1, 2)

    @staticmethod
    def backward(ctx, gy):
        global _launches
        col, wr = ctx.saved_tensors
        N, C, H, W, Co, KH, KW, OH, OW, stride, pad, wdtype, has_bias = ctx.meta
        g = gy.permute(0, 2, 3, 1).reshape(-1, Co)
        if g.dtype != torch.bfloat16 or not g.is_contiguous():
            g = g.to(torch.bfloat16).contiguous()
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            if C % 8:
                raise NotImplementedError("data gradient of a convolution whose input channels are not a multiple of 8")
            dcol = gemm_bf16(g, wr, b_t=True)                                   # [pixels, K]
            gx = torch.empty((N, C, H, W), dtype=torch.bfloat16, device=g.device, memory_format=torch.channels_last)
            _chk(_native.cuda().gcow_col2im(dcol.data_ptr(), gx.data_ptr(), N, H, W, C, KH, KW, stride, pad,
                                            _stream(g.device)), "gcow_col2im")
            _launches += 1
        if ctx.needs_input_grad[1]:
            gw = wgrad_gemm(g, col)                                               # [Co, Kp]
            if gw.shape[1] != KH * KW * C:
                gw = gw[:, :KH * KW * C]
            gw = gw.reshape(Co, KH, KW, C).permute(0, 3, 1, 2).to(wdtype).contiguous(memory_format=torch.channels_last)
        if has_bias and ctx.needs_input_grad[2]:
            gb = colsum(g)
        return gx, gw, gb, None, None


def conv_gemm_usable(x: torch.Tensor, w: torch.Tensor, stride: int, pad: int, groups: int, dilation) -> bool:
    """im2col + GEMM covers any stride and filter size; an input whose channel count is not a multiple of 8 only
    when no gradient flows into it (the image in front of the stem)."""
    if not (x.is_cuda and x.dim() == 4 and _have("gcow_im2col_anyc") and groups == 1 and tuple(dilation) == (1, 1)):
        return False
    if x.shape[1] % 8 and x.requires_grad:
        return False
    KH, KW = w.shape[2], w.shape[3]
    OH, OW = (x.shape[2] + 2 * pad - KH) // stride + 1, (x.shape[3] + 2 * pad - KW) // stride + 1
    return w.shape[0] % 8 == 0 and OH > 0 and OW > 0 and x.shape[0] * OH * OW >= 128


def conv_gemm(x, w, b, stride, pad):
    return _ConvGemmFn.apply(x, w, b, stride, pad)


# ------------------------------------------------ fused input embeddings
class _Embed3Fn(torch.autograd.Function):
    """tok[ids] + pos[position] + typ[type_ids] -> bf16 [B, S, H] in one kernel; deterministic backward
    (ordered sums for the position and type tables, a sorted segmented sum for the token table)."""

    @staticmethod
    def forward(ctx, ids, type_ids, tok, pos, typ):
        global _launches
        B, S = ids.shape
        H = tok.shape[1]
        ids_c, ty_c = ids.contiguous(), type_ids.contiguous()
        y = torch.empty((B, S, H), dtype=torch.bfloat16, device=tok.device)
        _chk(_native.cuda().gcow_embed3_fwd(ids_c.data_ptr(), ty_c.data_ptr(), tok.data_ptr(), pos.data_ptr(), typ.data_ptr(),
                                            y.data_ptr(), B * S, S, H, _stream(tok.device)), "gcow_embed3_fwd")
        _launches += 1
        ctx.save_for_backward(ids_c, ty_c)
        ctx.meta = (B, S, H, tok.shape[0], pos.shape[0], typ.shape[0])
        return y

    @staticmethod
    def backward(ctx, gy):
        global _launches
        ids, ty = ctx.saved_tensors
        B, S, H, V, P, NT = ctx.meta
        lib, dev = _native.cuda(), gy.device
        g = gy.to(torch.bfloat16).contiguous()
        order = torch.argsort(ids.view(-1), stable=True)
        dtok = torch.zeros((V, H), dtype=torch.float32, device=dev)
        dpos = torch.zeros((P, H), dtype=torch.float32, device=dev)
        parts = lib.gcow_embed_type_parts(B * S)
        tpart = _ws("embed_type_part", (parts, NT * H), torch.float32, dev)
        dtyp = torch.empty((NT, H), dtype=torch.float32, device=dev)
        _chk(lib.gcow_embed3_bwd(g.data_ptr(), ids.data_ptr(), ty.data_ptr(), order.data_ptr(), dtok.data_ptr(), dpos.data_ptr(),
                                 tpart.data_ptr(), B, S, H, NT, _stream(dev)), "gcow_embed3_bwd")
        _chk(lib.gcow_reduce_partials(tpart.data_ptr(), dtyp.data_ptr(), parts, NT * H, _stream(dev)), "gcow_reduce_partials")
        _launches += 4
        return None, None, dtok, dpos, dtyp


def embed3_usable(ids: torch.Tensor, tok: torch.Tensor, pos: torch.Tensor, typ: torch.Tensor) -> bool:
    return (ids.is_cuda and ids.dim() == 2 and ids.dtype == torch.int64 and _have("gcow_embed3_fwd")
            and tok.dtype == torch.float32 and pos.dtype == torch.float32 and typ.dtype == torch.float32
            and tok.is_contiguous() and pos.is_contiguous() and typ.is_contiguous()
            and tok.shape[1] % 4 == 0 and typ.shape[0] <= 4 and ids.shape[1] <= pos.shape[0])


def embed3(ids, type_ids, tok, pos, typ):
    return _Embed3Fn.apply(ids, type_ids, tok, pos, typ)


# ------------------------------------------------ implicit-GEMM convolution (stride 1)
def conv_ws_usable(N, H, W, C, Co, KH, KW, pad_h, pad_w):
    """64 -> 64 channels, 3x3, stride 1, padding 1: the weight-stationary kernel (pixels as the MMA's N) applies."""
    return (C == 64 and Co == 64 and KH == 3 and KW == 3 and pad_h == 1 and pad_w == 1
            and os.environ.get("GCOW_CONV_WS", "1") != "0" and _have("gcow_conv_fwd_ws")
            and bool(_native.cuda().gcow_conv_ws_usable(N, H, W)))


_HALO_WGRAD_MIN_W = 15      # narrowest image rows the halo-tile weight gradient is routed for


def conv_halo_usable(N, H, W, C, Co, KH, KW, pad_h, pad_w):
    """Ci -> 128 channels, 3x3, stride 1, padding 1, tiles that fit the shared memory: the halo-tile kernel applies."""
    return (Co == 128 and KH == 3 and KW == 3 and pad_h == 1 and pad_w == 1
            and os.environ.get("GCOW_CONV_HALO", "1") != "0" and _have("gcow_conv_fwd_halo")
            and bool(_native.cuda().gcow_conv_halo_usable(N, H, W, C)))


def _conv_fwd_s1(lib, x_ptr, w_ptr, y_ptr, bias_ptr, N, H, W, C, Co, KH, KW, pad_h, pad_w, err, st, what):
    """Stride-1 forward kernel for these extents: the weight-stationary or halo-tile one where it applies, else the
    general one."""
    if conv_ws_usable(N, H, W, C, Co, KH, KW, pad_h, pad_w):
        _chk(lib.gcow_conv_fwd_ws(x_ptr, w_ptr, y_ptr, bias_ptr, N, H, W, err, st), what + " (ws)")
    elif conv_halo_usable(N, H, W, C, Co, KH, KW, pad_h, pad_w):
        _chk(lib.gcow_conv_fwd_halo(x_ptr, w_ptr, y_ptr, bias_ptr, N, H, W, C, err, st), what + " (halo)")
    else:
        _chk(lib.gcow_conv_fwd(x_ptr, w_ptr, y_ptr, bias_ptr, N, H, W, C, Co, KH, KW, pad_h, pad_w, err, st), what)


class _ConvIgemmFn(torch.autograd.Function):
    """Stride-1 KxK convolution, channels-last bf16, as an implicit GEMM on the tcgen05 kernel
    (csrc/ops/conv_tcgen05.cu): forward, data gradient (the same kernel on dY with the flipped
    filter) and weight gradient (split over pixel ranges + ordered sum). No patch matrix."""

    @staticmethod
    def forward(ctx, x, w, b, pad_h, pad_w):
        global _launches
        N, C, H, W = x.shape
        Co, _, KH, KW = w.shape
        lib = _native.cuda()
        if x.dtype != torch.bfloat16 or not x.is_contiguous(memory_format=torch.channels_last):
            x = x.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        wr = bf16_weight(w).permute(0, 2, 3, 1).contiguous()                                       # [Co, kh, kw, Ci]
        OH, OW = H + 2 * pad_h - KH + 1, W + 2 * pad_w - KW + 1
        y = torch.empty((N, Co, OH, OW), dtype=torch.bfloat16, device=x.device, memory_format=torch.channels_last)
        bias = b.detach().float().contiguous() if b is not None else None
        _conv_fwd_s1(lib, x.data_ptr(), wr.data_ptr(), y.data_ptr(), bias.data_ptr() if bias is not None else None,
                     N, H, W, C, Co, KH, KW, pad_h, pad_w, _error_word(x.device).data_ptr(), _stream(x.device),
                     "gcow_conv_fwd")
        _launches += 1
        ctx.save_for_backward(x, wr)
        ctx.meta = (N, C, H, W, Co, KH, KW, OH, OW, pad_h, pad_w, b is not None)
        ctx.grad_view = take_grad_view(w)
        return y

    @staticmethod
    def backward(ctx, gy):
        global _launches
        x, wr = ctx.saved_tensors
        N, C, H, W, Co, KH, KW, OH, OW, pad_h, pad_w, has_bias = ctx.meta
        lib = _native.cuda()
        if gy.dtype != torch.bfloat16 or not gy.is_contiguous(memory_format=torch.channels_last):
            gy = gy.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        dev, st, err = gy.device, _stream(gy.device), _error_word(gy.device).data_ptr()
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            wt = torch.empty((C, KH, KW, Co), dtype=torch.bfloat16, device=dev)
            _chk(lib.gcow_conv_flip_weights(wr.data_ptr(), wt.data_ptr(), Co, KH, KW, C, st), "gcow_conv_flip_weights")
            gx = torch.empty((N, C, H, W), dtype=torch.bfloat16, device=dev, memory_format=torch.channels_last)
            _conv_fwd_s1(lib, gy.data_ptr(), wt.data_ptr(), gx.data_ptr(), None, N, OH, OW, Co, C, KH, KW,
                         KH - 1 - pad_h, KW - 1 - pad_w, err, st, "gcow_conv_fwd (dgrad)")
            _launches += 2
        if ctx.needs_input_grad[1]:
            # 64 -> 64 channels, 3x3, padding 1: the halo-tile kernel, when the image rows fit its slot pitch
            ws_split = (lib.gcow_conv_wgrad_ws_split(N, H, W) if conv_ws_usable(N, H, W, C, Co, KH, KW, pad_h, pad_w)
                        and os.environ.get("GCOW_CONV_WS_WGRAD", "1") != "0" and _have("gcow_conv_wgrad_ws") else 0)
            # channel counts that are multiples of 128, 3x3, padding 1, rows of at least 15 pixels: the halo-tile kernel
            # with one CTA group per (filter row, 128 x 128 channels). Measured at batch 256: 128 channels at 28 x 28 wins
            # (layer 0.221 -> 0.189 ms), 256 channels at 14 x 14 ties with the general kernel, 512 channels at 7 x 7
            # loses (slots of pitch 16 for rows of 7, 48 groups re-reading the tiles)
            halo_split = (lib.gcow_conv_wgrad_halo_split(N, H, W, C, Co) if C % 128 == 0 and Co % 128 == 0 and KH == 3
                          and KW == 3 and pad_h == 1 and pad_w == 1 and W >= _HALO_WGRAD_MIN_W
                          and os.environ.get("GCOW_CONV_HALO_WGRAD", "1") != "0" and _have("gcow_conv_wgrad_halo") else 0)
            split = (ws_split if ws_split > 0 else halo_split if halo_split > 0 else
                     lib.gcow_conv_wgrad_split(N, H, W, C, Co, KH, KW, pad_h, pad_w))
            flat, alias = _grad_target(ctx.grad_view, Co, KH * KW * C)
            # the partial sums are scratch when an ordered sum follows; a single part IS the result
            part = (_ws("conv_wgrad_part", (split, Co, KH * KW * C), torch.float32, dev) if split > 1 else
                    (flat.unsqueeze(0) if flat is not None else torch.empty((1, Co, KH * KW * C), dtype=torch.float32, device=dev)))
            if ws_split > 0:
                _chk(lib.gcow_conv_wgrad_ws(gy.data_ptr(), x.data_ptr(), part.data_ptr(), N, H, W, err, st), "gcow_conv_wgrad_ws")
            elif halo_split > 0:
                _chk(lib.gcow_conv_wgrad_halo(gy.data_ptr(), x.data_ptr(), part.data_ptr(), N, H, W, C, Co, err, st),
                     "gcow_conv_wgrad_halo")
            else:
                _chk(lib.gcow_conv_wgrad(gy.data_ptr(), x.data_ptr(), part.data_ptr(), N, H, W, C, Co, KH, KW, pad_h, pad_w,
                                         err, st), "gcow_conv_wgrad")
            _launches += 1
            if split > 1:
                out = flat if flat is not None else torch.empty((Co, KH * KW * C), dtype=torch.float32, device=dev)
                _chk(lib.gcow_reduce_partials(part.data_ptr(), out.data_ptr(), split, out.numel(), st), "gcow_reduce_partials")
                _launches += 1
            else:
                out = part[0]
            # logical [Co, Ci, kh, kw], channels-last memory
            gw = alias if flat is not None else out.view(Co, KH, KW, C).permute(0, 3, 1, 2)
        if has_bias and ctx.needs_input_grad[2]:
            gb = colsum(gy.permute(0, 2, 3, 1).reshape(-1, Co))
        return gx, gw, gb, None, None


class _Conv1x1Stride2Fn(torch.autograd.Function):
    """1x1 convolution with stride 2 (the down-sampling shortcut of a ResNet stage) on the implicit-GEMM kernel with
    one tap: forward and weight gradient read every second pixel through a tensor map with element strides, the input
    gradient is one launch that stores to the sampled pixels of a zero-filled tensor. No subsampled copy of the input
    and no scatter pass."""

    @staticmethod
    def forward(ctx, x, w, b):
        global _launches
        N, C, H, W = x.shape
        Co = w.shape[0]
        lib = _native.cuda()
        if x.dtype != torch.bfloat16 or not x.is_contiguous(memory_format=torch.channels_last):
            x = x.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        wr = bf16_weight(w).reshape(Co, C).contiguous()                                             # [Co, Ci]
        OH, OW = (H - 1) // 2 + 1, (W - 1) // 2 + 1
        y = torch.empty((N, Co, OH, OW), dtype=torch.bfloat16, device=x.device, memory_format=torch.channels_last)
        bias = b.detach().float().contiguous() if b is not None else None
        _chk(lib.gcow_conv_fwd_strided(x.data_ptr(), wr.data_ptr(), y.data_ptr(), bias.data_ptr() if bias is not None else None,
                                       N, H, W, C, Co, 1, 1, 0, 0, 2, _error_word(x.device).data_ptr(), _stream(x.device)),
             "gcow_conv_fwd_strided")
        _launches += 1
        ctx.save_for_backward(x, wr)
        ctx.meta = (N, C, H, W, Co, b is not None)
        ctx.grad_view = take_grad_view(w)
        return y

    @staticmethod
    def backward(ctx, gy):
        global _launches
        x, wr = ctx.saved_tensors
        N, C, H, W, Co, has_bias = ctx.meta
        lib = _native.cuda()
        if gy.dtype != torch.bfloat16 or not gy.is_contiguous(memory_format=torch.channels_last):
            gy = gy.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        dev, st, err = gy.device, _stream(gy.device), _error_word(gy.device).data_ptr()
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            wt = torch.empty((C, Co), dtype=torch.bfloat16, device=dev)
            _chk(lib.gcow_conv_flip_weights(wr.data_ptr(), wt.data_ptr(), Co, 1, 1, C, st), "gcow_conv_flip_weights")
            gx = torch.empty((N, C, H, W), dtype=torch.bfloat16, device=dev, memory_format=torch.channels_last)
            _chk(lib.gcow_conv_dgrad_1x1_s2(gy.data_ptr(), wt.data_ptr(), gx.data_ptr(), N, H, W, C, Co, err, st),
                 "gcow_conv_dgrad_1x1_s2")
            _launches += 2
        if ctx.needs_input_grad[1]:
            split = lib.gcow_conv_wgrad_split_strided(N, H, W, C, Co, 1, 1, 0, 0, 2)
            flat, alias = _grad_target(ctx.grad_view, Co, C)
            part = (_ws("conv_wgrad_part", (split, Co, C), torch.float32, dev) if split > 1 else
                    (flat.unsqueeze(0) if flat is not None else torch.empty((1, Co, C), dtype=torch.float32, device=dev)))
            _chk(lib.gcow_conv_wgrad_strided(gy.data_ptr(), x.data_ptr(), part.data_ptr(), N, H, W, C, Co, 1, 1, 0, 0, 2,
                                             err, st), "gcow_conv_wgrad_strided")
            _launches += 1
            if split > 1:
                out = flat if flat is not None else torch.empty((Co, C), dtype=torch.float32, device=dev)
                _chk(lib.gcow_reduce_partials(part.data_ptr(), out.data_ptr(), split, out.numel(), st), "gcow_reduce_partials")
                _launches += 1
            else:
                out = part[0]
            gw = alias if flat is not None else out.view(Co, C, 1, 1)
        if has_bias and ctx.needs_input_grad[2]:
            gb = colsum(gy.permute(0, 2, 3, 1).reshape(-1, Co))
        return gx, gw, gb


def conv1x1_s2_usable(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Both channel counts whole 64-channel rows (the kernel's reduction rows forward, backward and in the weight gradient)."""
    return (x.is_cuda and x.dim() == 4 and _have("gcow_conv_dgrad_1x1_s2") and tuple(w.shape[2:]) == (1, 1)
            and x.shape[1] % 64 == 0 and w.shape[0] % 64 == 0)


def conv1x1_s2(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None = None) -> torch.Tensor:
    return _Conv1x1Stride2Fn.apply(x, w, b)


class _ConvStride2Fn(torch.autograd.Function):
    """3x3 convolution with stride 2 and padding 1 over even extents (the down-sampling layer of every ResNet stage)
    on the implicit-GEMM kernel: the forward and the weight gradient read every second input pixel through a tensor
    map with element strides; the input gradient is four stride-1 convolutions of dY, one per parity of the dX pixel,
    with 1, 2, 2 and 4 of the nine taps. No patch matrix and no col2im scatter."""

    @staticmethod
    def forward(ctx, x, w, b):
        global _launches
        N, C, H, W = x.shape
        Co = w.shape[0]
        lib = _native.cuda()
        if x.dtype != torch.bfloat16 or not x.is_contiguous(memory_format=torch.channels_last):
            x = x.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        wr = bf16_weight(w).permute(0, 2, 3, 1).contiguous()                                       # [Co, 3, 3, Ci]
        y = torch.empty((N, Co, H // 2, W // 2), dtype=torch.bfloat16, device=x.device, memory_format=torch.channels_last)
        bias = b.detach().float().contiguous() if b is not None else None
        _chk(lib.gcow_conv_fwd_strided(x.data_ptr(), wr.data_ptr(), y.data_ptr(), bias.data_ptr() if bias is not None else None,
                                       N, H, W, C, Co, 3, 3, 1, 1, 2, _error_word(x.device).data_ptr(), _stream(x.device)),
             "gcow_conv_fwd_strided")
        _launches += 1
        ctx.save_for_backward(x, wr)
        ctx.meta = (N, C, H, W, Co, b is not None)
        ctx.grad_view = take_grad_view(w)
        return y

    @staticmethod
    def backward(ctx, gy):
        global _launches
        x, wr = ctx.saved_tensors
        N, C, H, W, Co, has_bias = ctx.meta
        lib = _native.cuda()
        if gy.dtype != torch.bfloat16 or not gy.is_contiguous(memory_format=torch.channels_last):
            gy = gy.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        dev, st, err = gy.device, _stream(gy.device), _error_word(gy.device).data_ptr()
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            wp = _ws("conv_s2_phase_w", (9 * C * Co,), torch.bfloat16, dev)
            gx = torch.empty((N, C, H, W), dtype=torch.bfloat16, device=dev, memory_format=torch.channels_last)
            _chk(lib.gcow_conv_dgrad_s2(gy.data_ptr(), wr.data_ptr(), wp.data_ptr(), gx.data_ptr(), N, H, W, C, Co, err, st),
                 "gcow_conv_dgrad_s2")
            _launches += 5
        if ctx.needs_input_grad[1]:
            split = lib.gcow_conv_wgrad_split_strided(N, H, W, C, Co, 3, 3, 1, 1, 2)
            flat, alias = _grad_target(ctx.grad_view, Co, 9 * C)
            part = (_ws("conv_wgrad_part", (split, Co, 9 * C), torch.float32, dev) if split > 1 else
                    (flat.unsqueeze(0) if flat is not None else torch.empty((1, Co, 9 * C), dtype=torch.float32, device=dev)))
            _chk(lib.gcow_conv_wgrad_strided(gy.data_ptr(), x.data_ptr(), part.data_ptr(), N, H, W, C, Co, 3, 3, 1, 1, 2,
                                             err, st), "gcow_conv_wgrad_strided")
            _launches += 1
            if split > 1:
                out = flat if flat is not None else torch.empty((Co, 9 * C), dtype=torch.float32, device=dev)
                _chk(lib.gcow_reduce_partials(part.data_ptr(), out.data_ptr(), split, out.numel(), st), "gcow_reduce_partials")
                _launches += 1
            else:
                out = part[0]
            gw = alias if flat is not None else out.view(Co, 3, 3, C).permute(0, 3, 1, 2)
        if has_bias and ctx.needs_input_grad[2]:
            gb = colsum(gy.permute(0, 2, 3, 1).reshape(-1, Co))
        return gx, gw, gb


def conv_igemm_s2_usable(x: torch.Tensor, w: torch.Tensor, stride, padding, groups: int, dilation) -> bool:
    """3x3, stride 2, padding 1, dense, even input extents, both channel counts whole 64-channel rows."""
    return (x.is_cuda and x.dim() == 4 and _have("gcow_conv_dgrad_s2") and groups == 1 and tuple(dilation) == (1, 1)
            and tuple(stride) == (2, 2) and tuple(padding) == (1, 1) and tuple(w.shape[2:]) == (3, 3)
            and x.shape[2] % 2 == 0 and x.shape[3] % 2 == 0 and x.shape[1] % 64 == 0 and w.shape[0] % 64 == 0)


def conv_igemm_s2(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None = None) -> torch.Tensor:
    return _ConvStride2Fn.apply(x, w, b)


def conv_mode() -> str:
    """GCOW_CONV selects the convolution routing of the own backend:
    ``auto`` (default) - every convolution on this library's kernels: 1x1 layers on the tcgen05 GEMM (strided ones
    after a pixel subsample), stride-1 KxK layers with whole 64-channel rows and 3x3 stride-2 layers on the
    implicit-GEMM kernel, everything else (other strided KxK, the stem) as im2col + GEMM;
    ``mixed`` - own kernels only where they are at least on par with cuDNN (stride-1 KxK with >= 128 channels), cuDNN
    for the rest;
    ``lib`` - cuDNN everywhere (the comparison arm)."""
    import os
    return os.environ.get("GCOW_CONV", "auto")


_conv_paths: dict = {}


def conv_path_counts(reset: bool = False) -> dict:
    """How many convolution calls took which path since the last reset: gemm1x1, gemm1x1_strided, igemm1x1_s2, igemm,
    igemm_s2, im2col, cudnn. Benchmarks report it; a test asserts that a ResNet-50 step sends nothing to cudnn."""
    out = dict(_conv_paths)
    if reset:
        _conv_paths.clear()
    return out


def conv_route(x: torch.Tensor, m) -> str:
    """Which kernel family serves this convolution call (see conv_mode)."""
    from . import backend
    mode = conv_mode()
    path = "cudnn"
    if (backend.get_backend() == "own" and mode != "lib" and m.groups == 1 and tuple(m.dilation) == (1, 1)
            and all(isinstance(p, int) for p in m.padding) and m.stride[0] == m.stride[1]
            and m.padding[0] == m.padding[1] and m.kernel_size[0] == m.kernel_size[1] and x.is_cuda and x.dim() == 4):
        k, s, p, w = m.kernel_size[0], m.stride[0], m.padding[0], m.weight
        if (k == 1 and p == 0 and s == 1 and mode == "auto" and _onebyone_on_igemm(x, w.shape[0])
                and conv_igemm_usable(x, w, m.stride, m.padding, 1, (1, 1), True)):
            path = "igemm"
        elif k == 1 and p == 0 and s == 2 and mode == "auto" and conv1x1_s2_usable(x, w):
            path = "igemm1x1_s2"
        elif k == 1 and p == 0:
            if mode == "auto":
                oh, ow = (x.shape[2] - 1) // s + 1, (x.shape[3] - 1) // s + 1
                rows = x.shape[0] * oh * ow
                if (_have("gcow_gemm_bf16") and x.shape[1] % 8 == 0 and w.shape[0] % 8 == 0 and rows % 8 == 0 and rows >= 128
                        and x.is_contiguous(memory_format=torch.channels_last)):
                    path = "gemm1x1" if s == 1 else "gemm1x1_strided"
        elif s == 1 and conv_igemm_usable(x, w, m.stride, m.padding, m.groups, m.dilation) and (
                mode == "auto" or min(w.shape[0], w.shape[1]) >= 128):
            path = "igemm"
        elif mode == "auto" and conv_igemm_s2_usable(x, w, m.stride, m.padding, m.groups, m.dilation):
            path = "igemm_s2"
        elif mode == "auto" and conv_gemm_usable(x, w, s, p, m.groups, m.dilation):
            path = "im2col"
    _conv_paths[path] = _conv_paths.get(path, 0) + 1
    return path


def _onebyone_on_igemm(x: torch.Tensor, out_channels: int = 64) -> bool:
    """A 1x1 layer with at most 64 input and output channels over very many pixels (64 -> 64 in the 56 x 56 stage of a ResNet at
    batch 256) runs about 10 % faster as a one-tap implicit GEMM, whose tile is as wide as the layer's output
    channels, than on the 256-column GEMM tile; every other 1x1 layer is faster on the GEMM (whose plain bf16
    results leave through the TMA). GCOW_CONV1X1=gemm|igemm forces either."""
    import os
    forced = os.environ.get("GCOW_CONV1X1", "")
    if forced in ("gemm", "igemm"):
        return forced == "igemm"
    return out_channels <= 64 and x.shape[1] <= 64 and x.shape[0] * x.shape[2] * x.shape[3] >= 500_000


def conv_igemm_usable(x: torch.Tensor, w: torch.Tensor, stride, padding, groups: int, dilation, allow_1x1: bool = False) -> bool:
    """Stride 1, dense, input channels a multiple of 64 (whole 128-byte channel rows per filter tap),
    output channels a multiple of 8, padding below the filter size."""
    if not (x.is_cuda and x.dim() == 4 and _have("gcow_conv_fwd") and groups == 1 and tuple(dilation) == (1, 1)):
        return False
    if tuple(stride) != (1, 1) or not all(isinstance(p, int) for p in padding):
        return False
    KH, KW = w.shape[2], w.shape[3]
    if (KH * KW == 1 and not allow_1x1) or padding[0] >= KH or padding[1] >= KW:
        return False
    # the data gradient swaps the channel roles, so both counts must be whole 64-channel rows
    return x.shape[1] % 64 == 0 and w.shape[0] % 64 == 0


def conv_igemm(x, w, b, padding):
    return _ConvIgemmFn.apply(x, w, b, int(padding[0]), int(padding[1]))


# ------------------------------------------------ batched GEMM and attention
def bmm_bf16(a: torch.Tensor, b: torch.Tensor, *, a_t: bool = False, b_t: bool = False,
             out_dtype=torch.bfloat16) -> torch.Tensor:
    """Batched C[i] = op(A[i]) @ op(B[i])^T on the tcgen05 kernel. a, b: bf16 [batch, rows, cols]
    with contiguous matrices (row length and batch stride multiples of 8)."""
    global _launches
    assert a.dim() == 3 and b.dim() == 3 and a.shape[0] == b.shape[0]
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.stride(2) == 1 and b.stride(2) == 1
    batch = a.shape[0]
    (K, M) = (a.shape[1], a.shape[2]) if a_t else (a.shape[2], a.shape[1])
    (Kb, N) = (b.shape[1], b.shape[2]) if b_t else (b.shape[2], b.shape[1])
    assert K == Kb
    out = torch.empty((batch, M, N), dtype=out_dtype, device=a.device)
    flags = OUT_F32 if out_dtype == torch.float32 else 0
    err = _native.cuda().gcow_gemm_bf16_batched(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(1), b.stride(1), out.stride(1), batch,
        a.stride(0), b.stride(0), out.stride(0), None, None, flags, _error_word(a.device).data_ptr(),
        int(a_t), int(b_t), 128, _stream(a.device))
    _chk(err, "gcow_gemm_bf16_batched")
    _launches += 1
    return out


class _AttentionFn(torch.autograd.Function):
    """Unfused multi-head self-attention on own kernels: batched QK^T GEMM, row softmax,
    batched PV GEMM; the backward is five batched GEMMs and the softmax backward.
    q, k, v: bf16 [batch*heads, S, D] contiguous."""

    @staticmethod
    def forward(ctx, q, k, v, scale):
        global _launches
        lib = _native.cuda()
        s = bmm_bf16(q, k)                                   # [BH, S, S] = Q K^T
        p = torch.empty_like(s)
        _chk(lib.gcow_softmax_fwd(s.data_ptr(), p.data_ptr(), s.shape[0] * s.shape[1], s.shape[2], scale,
                                  _stream(q.device)), "gcow_softmax_fwd")
        _launches += 1
        o = bmm_bf16(p, v, b_t=True)                         # [BH, S, D] = P V   (V stored [S(red), D])
        ctx.save_for_backward(q, k, v, p)
        ctx.scale = scale
        return o

    @staticmethod
    def backward(ctx, go):
        global _launches
        q, k, v, p = ctx.saved_tensors
        go = go.to(torch.bfloat16).contiguous()
        dv = bmm_bf16(p, go, a_t=True, b_t=True)             # P^T dO
        dp = bmm_bf16(go, v)                                 # dO V^T
        ds = torch.empty_like(p)
        _chk(_native.cuda().gcow_softmax_bwd(dp.data_ptr(), p.data_ptr(), ds.data_ptr(), p.shape[0] * p.shape[1],
                                             p.shape[2], ctx.scale, _stream(q.device)), "gcow_softmax_bwd")
        _launches += 1
        dq = bmm_bf16(ds, k, b_t=True)                       # dS K
        dk = bmm_bf16(ds, q, a_t=True, b_t=True)             # dS^T Q
        return dq, dk, dv, None


class _FusedAttentionFn(torch.autograd.Function):
    """Fused self-attention on the tcgen05 kernels of csrc/ops/attention_tcgen05.cu: packed qkv [B, S, 3, H, 64] in,
    context [B, S, H*64] out; the backward recomputes the probabilities from the stored log-sum-exp and writes
    the packed gradient [B, S, 3, H, 64]."""

    @staticmethod
    def forward(ctx, qkv, scale):
        global _launches
        B, S, _, H, D = qkv.shape
        q = qkv if (qkv.dtype == torch.bfloat16 and qkv.is_contiguous()) else qkv.to(torch.bfloat16).contiguous()
        out = torch.empty((B, S, H * D), dtype=torch.bfloat16, device=q.device)
        lse = torch.empty((B, H, S), dtype=torch.float32, device=q.device)
        _chk(_native.cuda().gcow_attention_fwd(q.data_ptr(), out.data_ptr(), lse.data_ptr(), B, S, H, D, scale,
                                               _error_word(q.device).data_ptr(), _stream(q.device)), "gcow_attention_fwd")
        _launches += 1
        ctx.save_for_backward(q, out, lse)
        ctx.scale = scale
        return out

    @staticmethod
    def backward(ctx, go):
        global _launches
        q, out, lse = ctx.saved_tensors
        B, S, _, H, D = q.shape
        g = go if (go.dtype == torch.bfloat16 and go.is_contiguous()) else go.to(torch.bfloat16).contiguous()
        dqkv = torch.empty_like(q)
        delta = _ws("attn_delta", (B, H, S), torch.float32, q.device)
        _chk(_native.cuda().gcow_attention_bwd(q.data_ptr(), out.data_ptr(), g.data_ptr(), lse.data_ptr(), delta.data_ptr(),
                                               dqkv.data_ptr(), B, S, H, D, ctx.scale, _error_word(q.device).data_ptr(),
                                               _stream(q.device)), "gcow_attention_bwd")
        _launches += 3
        return dqkv, None


def fused_attention_usable(qkv: torch.Tensor) -> bool:
    """Head dimension 64 and a sequence length that is a multiple of 128, at most 512."""
    if not (qkv.is_cuda and qkv.dim() == 5 and _have("gcow_attention_fwd")):
        return False
    B, S, three, H, D = qkv.shape
    return three == 3 and bool(_native.cuda().gcow_attention_supported(B, S, H, D))


def fused_attention(qkv: torch.Tensor) -> torch.Tensor:
    """qkv: [B, S, 3, H, 64] -> context [B, S, H*64]."""
    return _FusedAttentionFn.apply(qkv, 1.0 / (qkv.shape[-1] ** 0.5))


def attention_mode() -> str:
    """GCOW_ATTENTION=lib sends self-attention to PyTorch's scaled_dot_product_attention (the comparison arm);
    by default the own backend uses the fused tcgen05 kernels where they apply (head dimension 64, sequence a
    multiple of 128 up to 512) and batched tcgen05 GEMMs with softmax kernels elsewhere."""
    import os
    return os.environ.get("GCOW_ATTENTION", "own")


def attention_usable(qkv: torch.Tensor) -> bool:
    B, S, _, H, D = qkv.shape
    return qkv.is_cuda and _have("gcow_gemm_bf16_batched") and S % 8 == 0 and D % 8 == 0 and S <= 4096


def attention(qkv: torch.Tensor) -> torch.Tensor:
    """qkv: [B, S, 3, H, D] -> context [B, S, H*D]."""
    B, S, _, H, D = qkv.shape
    t = qkv.to(torch.bfloat16).permute(2, 0, 3, 1, 4).contiguous().view(3, B * H, S, D)
    o = _AttentionFn.apply(t[0], t[1], t[2], 1.0 / (D ** 0.5))
    return o.view(B, H, S, D).permute(0, 2, 1, 3).reshape(B, S, H * D)
