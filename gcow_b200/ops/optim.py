"""Fused multi-tensor optimizers backed by csrc/ops/optim_kernels.cu.

Drop-in ``torch.optim.Optimizer`` subclasses (state_dict / load_state_dict work,
so checkpoints resume) whose ``step`` is ONE kernel launch over a device table of
parameter chunks. On CPU tensors they fall back to the plain PyTorch arithmetic.
SGD defaults are the reference's (hw/models/train_imagenet.py:251-253).
"""
from __future__ import annotations

import math
import struct

import torch

from .. import _native

_CHUNK = 1 << 16


def _dense(t: torch.Tensor) -> bool:
    """Memory is one gap-free run (row-major or channels-last), so an elementwise
    update may walk it linearly."""
    if t.is_contiguous():
        return True
    return t.dim() == 4 and t.is_contiguous(memory_format=torch.channels_last)


class _FusedBase(torch.optim.Optimizer):
    n_states = 1

    def _ensure_state(self, p):
        st = self.state[p]
        if "s0" not in st:
            st["s0"] = torch.zeros_like(p, memory_format=torch.preserve_format)
            if self.n_states == 2:
                st["s1"] = torch.zeros_like(p, memory_format=torch.preserve_format)
            st["step"] = 0
        return st

    def _table(self, group):
        """Device chunk table for one param group; rebuilt only when a pointer changes."""
        params = [p for p in group["params"] if p.grad is not None]
        for p in params:
            self._ensure_state(p)
        for p in params:                 # bf16 copies of the matrices and filters, written by the update kernel
            if p.is_cuda and p.dim() >= 2 and getattr(p, "_gcow_bf16", None) is None and _dense(p) and p.dtype == torch.float32:
                p._gcow_bf16 = torch.empty_like(p, dtype=torch.bfloat16, memory_format=torch.preserve_format)
                p._gcow_bf16_version = -1
        key = tuple((p.data_ptr(), p.grad.data_ptr(), self.state[p]["s0"].data_ptr(),
                     p._gcow_bf16.data_ptr() if getattr(p, "_gcow_bf16", None) is not None else 0) for p in params)
        cache = self.__dict__.setdefault("_tables", {})
        ent = cache.get(id(group))
        if ent is not None and ent[0] == key:
            return ent[1], ent[2], params
        rows = []
        if params and params[0].is_cuda and _native.cuda().gcow_opt_chunk_bytes() != struct.calcsize("<QQQQIIQ"):
            raise RuntimeError("the optimizer library's chunk layout differs from this file's")
        for p in params:
            if not (_dense(p) and p.grad.stride() == p.stride() and p.dtype == torch.float32
                    and p.grad.dtype == torch.float32):
                raise TypeError("fused optimizers need dense float32 parameters whose gradients share their strides")
            st = self._ensure_state(p)
            n = p.numel()
            for lo in range(0, n, _CHUNK):
                c = min(_CHUNK, n - lo)
                s1 = st["s1"].data_ptr() + 4 * lo if self.n_states == 2 else 0
                sh = getattr(p, "_gcow_bf16", None)
                rows.append(struct.pack("<QQQQIIQ", p.data_ptr() + 4 * lo, p.grad.data_ptr() + 4 * lo,
                                        st["s0"].data_ptr() + 4 * lo, s1, c, 0,
                                        sh.data_ptr() + 2 * lo if sh is not None else 0))
        raw = b"".join(rows)
        dev = params[0].device if params else torch.device("cpu")
        table = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(dev) if rows else None
        cache[id(group)] = (key, table, len(rows))
        return table, len(rows), params


class FusedSGD(_FusedBase):
    n_states = 1

    def __init__(self, params, lr=0.1, momentum=0.9, weight_decay=1e-4, dampening=0.0, nesterov=False):
        super().__init__(params, dict(lr=lr, momentum=momentum, weight_decay=weight_decay,
                                      dampening=dampening, nesterov=nesterov))
        self.launches = 0

    @torch.no_grad()
    def step(self, closure=None, grad_scale: float = 1.0):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            ps = [p for p in group["params"] if p.grad is not None]
            if not ps:
                continue
            if not ps[0].is_cuda:
                self._step_cpu(group, ps, grad_scale)
                continue
            table, n, ps = self._table(group)
            first = all(self.state[p]["step"] == 0 for p in ps)
            err = _native.cuda().gcow_sgd_step(
                table.data_ptr(), n, group["lr"], group["momentum"], group["weight_decay"], group["dampening"],
                int(group["nesterov"]), int(first), grad_scale, torch.cuda.current_stream().cuda_stream)
            if err:
                raise RuntimeError(f"gcow_sgd_step failed: {err}")
            self.launches += 1
            for p in ps:
                self.state[p]["step"] += 1
                if getattr(p, "_gcow_bf16", None) is not None:
                    p._gcow_bf16_version = p._version        # the kernel wrote through raw pointers: no version bump
        return loss

    def _step_cpu(self, group, ps, grad_scale):
        for p in ps:
            st = self._ensure_state(p)
            g = p.grad * grad_scale + group["weight_decay"] * p
            if group["momentum"]:
                if st["step"] == 0:
                    st["s0"].copy_(g)
                else:
                    st["s0"].mul_(group["momentum"]).add_(g, alpha=1 - group["dampening"])
                g = g + group["momentum"] * st["s0"] if group["nesterov"] else st["s0"]
            p.add_(g, alpha=-group["lr"])
            st["step"] += 1


class FusedAdamW(_FusedBase):
    n_states = 2

    def __init__(self, params, lr=1e-4, betas=(0.9, 0.999), eps=1e-6, weight_decay=0.01):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.launches = 0

    @torch.no_grad()
    def step(self, closure=None, grad_scale: float = 1.0):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            ps = [p for p in group["params"] if p.grad is not None]
            if not ps:
                continue
            b1, b2 = group["betas"]
            if not ps[0].is_cuda:
                for p in ps:
                    st = self._ensure_state(p)
                    st["step"] += 1
                    g = p.grad * grad_scale
                    p.mul_(1 - group["lr"] * group["weight_decay"])
                    st["s0"].mul_(b1).add_(g, alpha=1 - b1)
                    st["s1"].mul_(b2).addcmul_(g, g, value=1 - b2)
                    t = st["step"]
                    denom = st["s1"].sqrt() / math.sqrt(1 - b2 ** t) + group["eps"]
                    p.addcdiv_(st["s0"], denom, value=-group["lr"] / (1 - b1 ** t))
                continue
            table, n, ps = self._table(group)
            t = self.state[ps[0]]["step"] + 1
            err = _native.cuda().gcow_adamw_step(
                table.data_ptr(), n, group["lr"], b1, b2, group["eps"], group["weight_decay"],
                1 - b1 ** t, math.sqrt(1 - b2 ** t), grad_scale, torch.cuda.current_stream().cuda_stream)
            if err:
                raise RuntimeError(f"gcow_adamw_step failed: {err}")
            self.launches += 1
            for p in ps:
                self.state[p]["step"] = t
                if getattr(p, "_gcow_bf16", None) is not None:
                    p._gcow_bf16_version = p._version
        return loss
