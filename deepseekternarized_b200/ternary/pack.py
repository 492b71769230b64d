"""TQ2 / TQ1 packing on the GPU: the surface of the reference's ``boilerplate/ternary/pack.py``.

A ternary matrix ``[N, K]`` with entries in {-1, 0, +1} is stored row-major, each trit as the digit
``u = t + 1``. TQ2: ``byte = u0 | u1 << 2 | u2 << 4 | u3 << 6`` (``ceil(K/4)`` bytes per row). TQ1:
``byte = u0 + 3 u1 + 9 u2 + 27 u3 + 81 u4`` (``ceil(K/5)`` bytes per row; values 243..255 decode to
zeros). Rows are padded to a whole byte with digit 1. Both directions run as CUDA kernels through
the C-ABI library and are bit-exact with the reference (``pack.py:34-82``); CPU tensors raise.
"""

from __future__ import annotations

import ctypes

import torch

from .. import _lib
from ..kernels.ternary_b200 import _fmt_code, _require, _stream

FORMATS = ("tq2", "tq1")


def bits_per_weight(fmt: str) -> float:
    """reference ``pack.py:26-27``"""
    return {"tq2": 2.0, "tq1": 1.6}[fmt]


def packed_cols(fmt: str, K: int) -> int:
    """reference ``pack.py:30-31``"""
    return -(-K // (4 if fmt == "tq2" else 5))


def _check(t: torch.Tensor, dtype, what: str):
    if not t.is_cuda:
        raise RuntimeError(f"B200 ternary kernel unavailable for CPU tensors: {what} must be on a CUDA device")
    if t.dtype != dtype or t.dim() != 2:
        raise RuntimeError(f"{what} must be a rank-2 {dtype} tensor")


def pack(t: torch.Tensor, fmt: str) -> torch.Tensor:
    """int8 trits [N, K] -> uint8 [N, packed_cols] (reference ``pack.py:43-45,54-59,77-78``)."""
    code = _fmt_code(fmt)
    lib = _require("auto")
    _check(t, torch.int8, "trits")
    t = t.contiguous()
    N, K = t.shape
    out = torch.empty(N, packed_cols(fmt, K), dtype=torch.uint8, device=t.device)
    with torch.cuda.device(t.device):
        _lib.check(lib.dst_pack(t.data_ptr(), N, K, code, out.data_ptr(), _stream(t)))
    return out


def unpack(p: torch.Tensor, fmt: str, K: int) -> torch.Tensor:
    """uint8 [N, packed_cols] -> int8 trits [N, K] (reference ``pack.py:48-51,70-74,81-82``)."""
    code = _fmt_code(fmt)
    lib = _require("auto")
    _check(p, torch.uint8, "packed weights")
    if p.size(1) != packed_cols(fmt, K):
        raise RuntimeError("inconsistent ternary tensor sizes")
    p = p.contiguous()
    out = torch.empty(p.size(0), K, dtype=torch.int8, device=p.device)
    with torch.cuda.device(p.device):
        _lib.check(lib.dst_unpack(p.data_ptr(), p.size(0), K, code, out.data_ptr(), _stream(p)))
    return out


def tq1_lut(device="cuda") -> torch.Tensor:
    """[256, 5] int8 trits of every byte value, rows >= 243 zero (reference ``pack.py:62-67``),
    produced by the unpack kernel itself."""
    v = torch.arange(256, dtype=torch.uint8, device=device).view(256, 1)
    return unpack(v, "tq1", 5)
