"""Stand-alone compress / decompress API of the ZFP float32 block codec.

CUDA tensors go through the hand-written sm_100a kernels
(csrc/codec/codec_kernels.cu); CPU tensors through the C++ oracle
(csrc/codec/oracle.cpp). Both produce the reference's header-less stream:
blocks concatenated LSB-first into little-endian 64-bit words, zero padded to a
word (sw/src/zfp.c:10-28, sw/src/stream.c:61-138).

The reference exposes ``zfp_compress(output, input)`` on a 2-D float array with
the four expert parameters set by hand or by its accuracy setter
(sw/include/zfp.h:4-7, sw/src/common.c:6-21); its training study calls zfpy with
``rate=``, ``precision=`` or ``tolerance=`` on a flat gradient
(hw/models/train_imagenet.py:459-465). Both call styles are covered here.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Optional

import torch

from . import _native

_NTHREADS = max(1, min(16, os.cpu_count() or 1))
_FAST_BITS = (16, 32, 64, 128)


@dataclass(frozen=True)
class ZfpParams:
    """The four codec parameters (sw/include/types.h:58-65)."""
    minbits: int = 1
    maxbits: int = 16658
    maxprec: int = 64
    minexp: int = -1074

    @staticmethod
    def _from_native(fill) -> "ZfpParams":
        a = (C.c_int32 * 4)()
        fill(a)
        return ZfpParams(int(a[0]), int(a[1]), int(a[2]), int(a[3]))

    @classmethod
    def from_rate(cls, rate: float, dim: int = 1) -> "ZfpParams":
        """Fixed rate: ``rate`` bits per value. A block is never shorter than its
        9-bit header, so 1-D rates below 2.25 are floored to 9 bits per block."""
        return cls._from_native(lambda a: _native.cpu().gcow_params_rate(float(rate), int(dim), a))

    @classmethod
    def from_accuracy(cls, tolerance: float) -> "ZfpParams":
        """Fixed accuracy: absolute error bound (sw/src/common.c:6-21)."""
        return cls._from_native(lambda a: _native.cpu().gcow_params_accuracy(float(tolerance), a))

    @classmethod
    def from_precision(cls, precision: int) -> "ZfpParams":
        """Fixed precision: number of bit planes kept per block."""
        return cls._from_native(lambda a: _native.cpu().gcow_params_precision(int(precision), a))

    @property
    def fixed_rate(self) -> bool:
        return self.minbits == self.maxbits

    def as_c(self):
        return (C.c_int32 * 4)(self.minbits, self.maxbits, self.maxprec, self.minexp)

    def block_precision(self, emax: int, dim: int) -> int:
        return int(_native.cpu().gcow_block_precision(emax, self.maxprec, self.minexp, dim))


@dataclass
class Compressed:
    """A compressed array: ``stream`` is a uint8 tensor of exactly ``nbytes``."""
    stream: torch.Tensor
    params: ZfpParams
    shape: tuple            # (n,) for 1-D, (ny, nx) for 2-D
    index: Optional[torch.Tensor] = None  # start bit of every block + end (int64), variable-rate only

    @property
    def nbytes(self) -> int:
        return int(self.stream.numel())

    @property
    def dim(self) -> int:
        return len(self.shape)


def _nxny(shape: tuple) -> tuple[int, int]:
    if len(shape) == 1:
        return int(shape[0]), 0
    return int(shape[1]), int(shape[0])


def _blocks(shape: tuple) -> int:
    if len(shape) == 1:
        return (shape[0] + 3) // 4
    return ((shape[0] + 3) // 4) * ((shape[1] + 3) // 4)


def max_compressed_nbytes(shape: tuple, params: ZfpParams) -> int:
    """Worst-case stream size (sw/src/common.c:187-224), a multiple of 8."""
    nx, ny = _nxny(tuple(shape))
    return int(_native.cpu().gcow_max_output_bytes(params.as_c(), nx, ny))


def compressed_nbytes(shape: tuple, params: ZfpParams) -> int:
    """Exact size of a fixed-rate stream."""
    if not params.fixed_rate:
        raise ValueError("only fixed-rate streams have a size known in advance")
    bits = _blocks(tuple(shape)) * params.maxbits
    return ((bits + 63) // 64) * 8


def _resolve_params(rate, tolerance, precision, params, dim) -> ZfpParams:
    given = [v is not None for v in (rate, tolerance, precision, params)]
    if sum(given) != 1:
        raise ValueError("give exactly one of rate=, tolerance=, precision=, params=")
    if params is not None:
        return params
    if rate is not None:
        return ZfpParams.from_rate(rate, dim)
    if tolerance is not None:
        return ZfpParams.from_accuracy(tolerance)
    return ZfpParams.from_precision(precision)


def _check(err: int, what: str) -> None:
    if err != 0:
        raise RuntimeError(f"{what} failed with CUDA/launcher error {err}")


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def compress(x: torch.Tensor, *, rate: float | None = None, tolerance: float | None = None,
             precision: int | None = None, params: ZfpParams | None = None, dim: int = 1,
             return_index: bool = False) -> Compressed:
    """Compress a float32 tensor.

    ``dim=1`` treats ``x`` as a flat vector cut into blocks of 4 (what the
    training study does with gradients); ``dim=2`` takes a 2-D tensor
    ``[ny, nx]`` cut into 4x4 blocks (the reference CPU/FPGA codec).
    Variable-rate modes (tolerance / precision) on CUDA synchronise once to
    learn the stream length; pass ``return_index=True`` to keep the per-block
    bit offsets needed for a parallel decode.
    """
    if x.dtype != torch.float32:
        raise TypeError("the codec takes float32 input")
    if dim == 2:
        if x.dim() != 2:
            raise ValueError("dim=2 needs a 2-D tensor [ny, nx]")
        shape = (int(x.shape[0]), int(x.shape[1]))
    elif dim == 1:
        shape = (int(x.numel()),)
    else:
        raise ValueError("dim must be 1 or 2")
    p = _resolve_params(rate, tolerance, precision, params, dim)
    x = x.contiguous()
    nx, ny = _nxny(shape)
    blocks = _blocks(shape)
    cap = max_compressed_nbytes(shape, p)

    if not x.is_cuda:
        out = torch.zeros(cap // 8, dtype=torch.int64)
        idx = torch.zeros(blocks + 1, dtype=torch.int64) if (return_index or not p.fixed_rate) else None
        nbytes = _native.cpu().gcow_oracle_compress(
            x.data_ptr(), nx, ny, p.as_c(), out.data_ptr(), idx.data_ptr() if idx is not None else None,
            _NTHREADS)
        stream = out.view(torch.uint8)[:nbytes]
        return Compressed(stream, p, shape, idx if (return_index or not p.fixed_rate) else None)

    lib = _native.cuda()
    with torch.cuda.device(x.device):
        if dim == 1 and p.fixed_rate and p.maxbits in _FAST_BITS:
            nbytes = compressed_nbytes(shape, p)
            out = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
            tail = blocks * p.maxbits // 8
            if tail < nbytes:
                out[tail:].zero_()
            _check(lib.gcow_encode_1d_fixed(x.data_ptr(), nx, p.maxbits, out.data_ptr(), _stream_ptr()),
                   "gcow_encode_1d_fixed")
            return Compressed(out, p, shape, None)
        if p.fixed_rate and p.maxbits % 64 == 0:
            # whole words per block: one pass, no scratch
            nbytes = compressed_nbytes(shape, p)
            out = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
            _check(lib.gcow_encode_fixed_direct(x.data_ptr(), nx, ny, p.as_c(), out.data_ptr(), _stream_ptr()),
                   "gcow_encode_fixed_direct")
            idx = (torch.arange(blocks + 1, dtype=torch.int64, device=x.device) * p.maxbits) if return_index else None
            return Compressed(out, p, shape, idx)
        scratch_bytes = lib.gcow_encode_generic_scratch_bytes(p.as_c(), blocks, dim)
        scratch = torch.empty(scratch_bytes, dtype=torch.uint8, device=x.device)
        out = torch.empty(cap, dtype=torch.uint8, device=x.device)
        idx = torch.empty(blocks + 1, dtype=torch.int64, device=x.device)
        _check(lib.gcow_encode_generic(x.data_ptr(), nx, ny, p.as_c(), out.data_ptr(), cap,
                                       scratch.data_ptr(), idx.data_ptr(), _stream_ptr()),
               "gcow_encode_generic")
        if p.fixed_rate:
            nbytes = compressed_nbytes(shape, p)
        else:
            nbytes = ((int(idx[-1].item()) + 63) // 64) * 8
        keep_index = return_index or not p.fixed_rate
        return Compressed(out[:nbytes], p, shape, idx if keep_index else None)


def decompress(c: Compressed, out: torch.Tensor | None = None, *, shift: int = 0) -> torch.Tensor:
    """Inverse of :func:`compress`. ``shift`` divides every value by 2**shift
    exactly (used to average over a power-of-two number of ranks)."""
    p, shape = c.params, tuple(c.shape)
    nx, ny = _nxny(shape)
    dev = c.stream.device
    if out is None:
        out = torch.empty(shape, dtype=torch.float32, device=dev)
    if out.dtype != torch.float32 or not out.is_contiguous() or out.numel() != (nx * (ny or 1)):
        raise ValueError("out must be a contiguous float32 tensor of the original size")
    if out.numel() == 0:
        return out
    stream = c.stream.contiguous()

    if not stream.is_cuda:
        buf = _padded_words(stream)
        _native.cpu().gcow_oracle_decompress(buf.data_ptr(), out.data_ptr(), nx, ny, p.as_c(), shift,
                                             _NTHREADS)
        return out

    lib = _native.cuda()
    with torch.cuda.device(dev):
        if len(shape) == 1 and p.fixed_rate and p.maxbits in _FAST_BITS:
            _check(lib.gcow_decode_1d_fixed(stream.data_ptr(), out.data_ptr(), nx, p.maxbits, shift,
                                            _stream_ptr()), "gcow_decode_1d_fixed")
            return out
        if not p.fixed_rate and c.index is None:
            # block offsets of a variable-rate stream are only known by walking
            # it; without an index that walk is serial, so it runs on the host
            host = decompress(Compressed(stream.cpu(), p, shape, None), shift=shift)
            out.copy_(host)
            return out
        idx = None if p.fixed_rate else c.index.to(dev)
        _check(lib.gcow_decode_generic(stream.data_ptr(), out.data_ptr(), nx, ny, p.as_c(),
                                       idx.data_ptr() if idx is not None else None, shift, _stream_ptr()),
               "gcow_decode_generic")
        return out


def _padded_words(stream: torch.Tensor) -> torch.Tensor:
    """Host copy of a byte stream, zero padded by one word so that readers may
    touch the word after the last bit."""
    n = stream.numel()
    buf = torch.zeros(((n + 7) // 8 + 1) * 8, dtype=torch.uint8)
    buf[:n] = stream
    return buf
