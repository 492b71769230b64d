"""Ternary GEMM and grouped (MoE expert) GEMM on B200: the call surface of the reference's
``boilerplate/kernels/ternary_cuda.py``, backed by ``libdst_b200.so``.

Contract (reference ``boilerplate/kernels/ternary_cuda.py:3-9``)::

    out[t, n] = x_scale[t] * sum_g w_scale[e(t), n, g] * sum_{k in g} x[t, k] * trit[e(t), n, k]

Two activation flavours share it:

* int8 activations + float32 scales: the reference's CUDA contract. ``ternary_gemm`` /
  ``grouped_ternary_gemm`` keep the reference signatures (``ternary_cuda.py:67-111``).
* bf16 activations + fp16 scales, fp32 accumulation: the Mode C/D path the reference only runs on
  its C++ CPU kernel (``boilerplate/ternary/ops.py:63-66,75-79``). ``ternary_gemm_bf16`` /
  ``grouped_ternary_gemm_bf16`` take the stacked terms in one call.

Every function here launches CUDA kernels. There is no CPU path: CPU tensors, a missing library or
a missing GPU raise ``RuntimeError("... unavailable ...")`` as the reference's ``backend="cuda"``
does (``ternary_cuda.py:76-77``).
"""

from __future__ import annotations

import ctypes
import os
from functools import lru_cache
from typing import Sequence

import torch

from .. import _lib

BACKENDS = ("auto", "b200", "cuda")
_ALGO = {"auto": _lib.ALGO_AUTO, "generic": _lib.ALGO_GENERIC, "decode": _lib.ALGO_DECODE, "prefill": _lib.ALGO_PREFILL}
_OUT = {torch.float32: _lib.OUT_F32, torch.bfloat16: _lib.OUT_BF16, torch.float16: _lib.OUT_F16}
_ACT = {torch.bfloat16: _lib.ACT_BF16, torch.float16: _lib.ACT_F16, torch.int8: _lib.ACT_I8}
_SCALE = {torch.float16: _lib.SCALE_F16, torch.float32: _lib.SCALE_F32, torch.bfloat16: _lib.SCALE_BF16}
_UNAVAILABLE = "B200 ternary kernel unavailable (no GPU, library not built, or DST_NO_CUDA)"


@lru_cache(1)
def ext():
    """The loaded C-ABI library, or None when ``DST_NO_CUDA`` is set or no GPU is visible
    (reference ``ternary_cuda.py:32-43``). A library that exists but fails to load raises."""
    if os.environ.get("DST_NO_CUDA") or torch.version.cuda is None or not torch.cuda.is_available():
        return None
    return _lib.load()


def _fmt_code(fmt: str) -> int:
    if fmt not in ("tq1", "tq2"):
        raise ValueError(f"unknown ternary packing {fmt!r}")
    return _lib.FMT_TQ2 if fmt == "tq2" else _lib.FMT_TQ1


def packed_cols(fmt: str, K: int) -> int:
    return -(-K // (4 if fmt == "tq2" else 5))


def _require(backend: str):
    if backend not in BACKENDS:
        raise RuntimeError(f"{_UNAVAILABLE}: backend {backend!r} is not served by this package")
    lib = ext()
    if lib is None:
        raise RuntimeError(_UNAVAILABLE)
    return lib


class TiledWeights:
    """Packed ternary weights of E experts in the tiled device layout (see ``include/dst_b200.h``):
    a byte permutation of the canonical ``[E, N, packed_cols]`` tensor built once by ``tile_weights``;
    ``untile`` restores the canonical bytes bit for bit.

    ``decode``: for TQ1 weights, optionally the SAME trits once more as tiled TQ2 (2 bits per trit instead of 1.6:
    +25 % device bytes for that copy). The TQ2 decode GEMV unpacks four trits with one AND, the TQ1 one needs a table
    read and ~4.5 integer instructions per byte, so few-row calls are served from this copy when it exists."""

    def __init__(self, data: torch.Tensor, E: int, N: int, K: int, fmt: str, decode: "TiledWeights | None" = None):
        self.data, self.E, self.N, self.K, self.fmt, self.decode = data, E, N, K, fmt, decode

    @property
    def device(self):
        return self.data.device

    def size(self, dim: int) -> int:
        return (self.E, self.N, packed_cols(self.fmt, self.K))[dim]

    def untile(self) -> torch.Tensor:
        lib = _require("auto")
        out = torch.empty(self.E, self.N, packed_cols(self.fmt, self.K), dtype=torch.uint8, device=self.data.device)
        with torch.cuda.device(self.data.device):
            _lib.check(lib.dst_untile_weights(self.data.data_ptr(), self.E, self.N, self.K, _fmt_code(self.fmt), out.data_ptr(),
                                              _stream(self.data)))
        return out


class NormRows:
    """Token rows in the tcgen05 kernel's input format: fp16 ``data`` [rows, K], each row scaled by a power of
    two so its largest magnitude lies in [128, 256), and ``factor`` [rows] float32 holding that power of two
    (``dst_gather_rows_norm`` / ``dst_swiglu_norm`` produce them; see ``include/dst_b200.h``)."""

    def __init__(self, data: torch.Tensor, factor: torch.Tensor):
        self.data, self.factor = data, factor

    def size(self, dim: int) -> int:
        return self.data.size(dim)

    @property
    def device(self):
        return self.data.device


def tile_weights(packed: torch.Tensor, fmt: str, K: int, decode_copy: bool = False) -> TiledWeights:
    """Canonical packed weights ``[E, N, packed_cols]`` (or ``[N, packed_cols]``) -> ``TiledWeights``: the one-time
    device re-layout the fast kernels read (the reference copies weights to the device at the same
    point, ``boilerplate/ternary/ops.py:41-45``). ``decode_copy`` (TQ1 with K % 512 == 0 only): also keep the trits
    as tiled TQ2 for the decode GEMV (see ``TiledWeights.decode``)."""
    code = _fmt_code(fmt)
    lib = _require("auto")
    if packed.dim() == 2:
        packed = packed[None]
    if not packed.is_cuda or packed.dtype != torch.uint8 or packed.dim() != 3 or packed.size(2) != packed_cols(fmt, K):
        raise RuntimeError("tile_weights takes a CUDA uint8 tensor [E, N, packed_cols]")
    packed = packed.contiguous()
    E, N, _ = packed.shape
    nbytes = lib.dst_tiled_bytes(code, E, N, K)
    data = torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=packed.device)
    with torch.cuda.device(packed.device):
        _lib.check(lib.dst_tile_weights(packed.data_ptr(), E, N, K, code, data.data_ptr(), _stream(packed)))
    dec = None
    if decode_copy and fmt == "tq1" and K % 512 == 0:
        dec = TiledWeights(_reencode_tq2_tiled(lib, packed, K), E, N, K, "tq2")
    return TiledWeights(data, E, N, K, fmt, dec)


def _reencode_tq2_tiled(lib, packed_tq1: torch.Tensor, K: int) -> torch.Tensor:
    """Canonical TQ1 ``[E, N, ceil(K/5)]`` -> the tiled TQ2 buffer of the same trits (unpack, pack as TQ2, tile), a few
    experts at a time so the int8 trits in between stay small."""
    E, N, _ = packed_tq1.shape
    dev = packed_tq1.device
    out = torch.empty(max(int(lib.dst_tiled_bytes(_lib.FMT_TQ2, E, N, K)), 16), dtype=torch.uint8, device=dev)
    per_expert = int(lib.dst_tiled_bytes(_lib.FMT_TQ2, 1, N, K))
    step = max(1, (256 << 20) // max(N * K, 1))
    with torch.cuda.device(dev):
        st = _stream(packed_tq1)
        for e0 in range(0, E, step):
            n = min(step, E - e0)
            trits = torch.empty(n * N, K, dtype=torch.int8, device=dev)
            tq2 = torch.empty(n * N, K // 4, dtype=torch.uint8, device=dev)
            _lib.check(lib.dst_unpack(packed_tq1[e0:e0 + n].data_ptr(), n * N, K, _lib.FMT_TQ1, trits.data_ptr(), st))
            _lib.check(lib.dst_pack(trits.data_ptr(), n * N, K, _lib.FMT_TQ2, tq2.data_ptr(), st))
            _lib.check(lib.dst_tile_weights(tq2.data_ptr(), n, N, K, _lib.FMT_TQ2, out[e0 * per_expert:].data_ptr(), st))
    return out


def fast_path_covers(K: int, group: int, scale_dtype, act_dtype=torch.bfloat16) -> bool:
    """Shapes the decode and prefill kernels accept (everything else runs on the generic kernel)."""
    return group == 128 and K % 128 == 0 and scale_dtype == torch.float16 and act_dtype in (torch.bfloat16, torch.float16, torch.int8)


def _stream(t: torch.Tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _check_dev(ts: Sequence[torch.Tensor]):
    dev = ts[0].device
    for t in ts:
        if not t.is_cuda or not t.is_contiguous():
            raise RuntimeError("ternary GEMM tensors must be contiguous CUDA tensors")
        if t.device != dev:
            raise RuntimeError("ternary GEMM tensors must share one device")


def _offsets(offsets, E: int, T: int, device, validate: bool):
    """(device int64 tensor, host ctypes array or None). Host validation as ``ternary_cuda.py:94-97``."""
    if isinstance(offsets, torch.Tensor) and offsets.is_cuda and not validate:
        if offsets.dtype != torch.int64 or offsets.numel() != E + 1:
            raise ValueError("offsets must be nondecreasing, start at 0, end at the row count, one per expert + 1")
        return offsets.contiguous(), None
    offs = torch.as_tensor(offsets, dtype=torch.int64).cpu().contiguous()
    if offs.dim() != 1 or offs.numel() != E + 1 or int(offs[0]) != 0 or int(offs[-1]) != T or bool((offs.diff() < 0).any()):
        raise ValueError("offsets must be nondecreasing, start at 0, end at the row count, one per expert + 1")
    host = (ctypes.c_int64 * (E + 1))(*offs.tolist())
    dev = offsets.contiguous() if isinstance(offsets, torch.Tensor) and offsets.is_cuda and offsets.dtype == torch.int64 \
        else offs.to(device)
    return dev, host


def _decode_row_limit(E: int, N: int) -> int:
    """Rows per expert up to which the 2-bit decode copy of TQ1 weights is the faster path (the library's AUTO rule for
    TQ2 tiles)."""
    return int(_require("auto").dst_decode_row_limit(_lib.FMT_TQ2, E, N))


def _grouped(lib, x, row_scale, offsets, packed_terms, scale_terms, K, group, fmt, out, accumulate, algo,
             validate_offsets=True, act_code=None):
    """Shared launcher. packed_terms[i] [E, N, Kp] uint8, scale_terms[i] [E, N, G]."""
    code = _fmt_code(fmt)
    n_terms = len(packed_terms)
    if n_terms < 1 or n_terms > _lib.MAX_TERMS or len(scale_terms) != n_terms:
        raise RuntimeError(f"between 1 and {_lib.MAX_TERMS} stacked terms are supported")
    tiled = isinstance(packed_terms[0], TiledWeights)
    if any(isinstance(p, TiledWeights) != tiled for p in packed_terms):
        raise RuntimeError("stacked terms must share one weight layout")
    if not isinstance(K, int) or not isinstance(group, int) or K <= 0 or group <= 0:
        raise RuntimeError("invalid ternary GEMM K or group")
    if tiled:
        if any(p.K != K or p.fmt != fmt for p in packed_terms):
            raise RuntimeError("inconsistent ternary GEMM shapes")
        # few rows per expert and a 2-bit copy of the TQ1 trits on the device: the decode GEMV reads that copy
        if fmt == "tq1" and algo in ("auto", "decode") and act_code != _lib.ACT_F16_NORM and all(p.decode is not None for p in packed_terms) \
                and x.size(0) <= _decode_row_limit(packed_terms[0].E, packed_terms[0].N) * packed_terms[0].E:
            packed_terms, fmt, code, algo = [p.decode for p in packed_terms], "tq2", _lib.FMT_TQ2, "decode"
    elif algo != "generic" and fast_path_covers(K, group, scale_terms[0].dtype, x.dtype) and all(
            p.is_cuda and p.dtype == torch.uint8 and p.dim() == 3 for p in packed_terms) and (
            algo != "auto" or 2 * x.size(0) * packed_terms[0].size(1) * K >= (1 << 28)):
        # canonical weights handed to a fast kernel: re-layout for this call (callers that reuse weights
        # tile them once with tile_weights / TernaryLinear / ExpertWeights.prepare instead)
        packed_terms = [tile_weights(p, fmt, K) for p in packed_terms]
        tiled = True
    elif algo == "auto":
        algo = "generic"
    raw = [p.data if tiled else p for p in packed_terms]
    tensors = [out, x, *raw, *scale_terms] + ([row_scale] if row_scale is not None else [])
    _check_dev(tensors)
    if x.dtype not in _ACT or out.dtype not in _OUT or any(p.dtype != torch.uint8 for p in raw):
        raise RuntimeError("unexpected ternary GEMM dtype")
    sdt = scale_terms[0].dtype
    if sdt not in _SCALE or any(s.dtype != sdt for s in scale_terms):
        raise RuntimeError("unexpected ternary GEMM scale dtype")
    if x.dim() != 2 or out.dim() != 2 or (not tiled and any(p.dim() != 3 for p in packed_terms)) or any(s.dim() != 3 for s in scale_terms):
        raise RuntimeError("bad ranks")
    E, N = packed_terms[0].size(0), packed_terms[0].size(1)
    G = -(-K // group)
    T = x.size(0)
    for p, s in zip(packed_terms, scale_terms):
        if (p.size(0), p.size(1), p.size(2)) != (E, N, packed_cols(fmt, K)) or tuple(s.shape) != (E, N, G):
            raise RuntimeError("inconsistent ternary GEMM shapes")
    if x.size(1) != K or tuple(out.shape) != (T, N) or (row_scale is not None and (row_scale.numel() != T or row_scale.dtype != torch.float32)):
        raise RuntimeError("inconsistent ternary GEMM shapes")
    if accumulate and out.dtype != torch.float32:
        raise RuntimeError("accumulation needs a float32 output")
    if E == 1 and offsets is None:
        offs_dev, offs_host = None, None
    else:
        offs_dev, offs_host = _offsets(offsets, E, T, x.device, validate_offsets)
    pk = (ctypes.c_void_p * n_terms)(*[p.data_ptr() for p in raw])
    sc = (ctypes.c_void_p * n_terms)(*[s.data_ptr() for s in scale_terms])
    act = _ACT[x.dtype] if act_code is None else act_code
    ws_bytes = int(lib.dst_gemm_workspace_bytes(_ALGO[algo], act, T, K)) if tiled and act != _lib.ACT_F16_NORM else 0
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device) if ws_bytes else None
    with torch.cuda.device(x.device):
        rc = lib.dst_ternary_grouped_gemm(
            out.data_ptr(), _OUT[out.dtype], int(bool(accumulate)), x.data_ptr(), act,
            row_scale.data_ptr() if row_scale is not None else None,
            offs_dev.data_ptr() if offs_dev is not None else None, offs_host,
            pk, _lib.LAYOUT_TILED if tiled else _lib.LAYOUT_CANONICAL, sc, n_terms, _SCALE[sdt], E, T, N, K, group, code,
            _ALGO[algo], ws.data_ptr() if ws is not None else None, ws_bytes, _stream(x))
    if ws is not None:
        ws.record_stream(torch.cuda.current_stream(x.device))
    _lib.check(rc)
    return out


# --------------------------------------------------------------------------- reference signatures (int8 contract)
def ternary_gemm(x: torch.Tensor, x_scale: torch.Tensor, packed: torch.Tensor, w_scale: torch.Tensor,
                 K: int, group: int, fmt: str, backend: str = "auto") -> torch.Tensor:
    """[T, K] int8 activations x [N, Kp] packed weights -> [T, N] float32 (reference ``ternary_cuda.py:67-87``)."""
    _fmt_code(fmt)
    if x.dtype != torch.int8:
        raise TypeError("ternary_gemm takes int8 activations (see quant_act_int8)")
    if not x.is_cuda:
        raise RuntimeError(_UNAVAILABLE + ": activations are not on a CUDA device and this backend has no CPU path")
    return grouped_ternary_gemm(x, x_scale, None, packed[None], w_scale[None], K, group, fmt, backend=backend)


def grouped_ternary_gemm(x: torch.Tensor, x_scale: torch.Tensor, offsets, packed: torch.Tensor, w_scale: torch.Tensor,
                         K: int, group: int, fmt: str, backend: str = "auto", algo: str = "auto") -> torch.Tensor:
    """Rows of ``x`` sorted by expert; ``packed`` [E, N, Kp], ``w_scale`` [E, N, G] -> [T, N] float32
    (reference ``ternary_cuda.py:90-111``)."""
    _fmt_code(fmt)
    E = packed.size(0)
    if offsets is not None and not (isinstance(offsets, torch.Tensor) and offsets.is_cuda):
        _offsets(offsets, E, x.size(0), "cpu", True)  # host offsets are validated before anything else, as the reference does
    lib = _require(backend)
    if not x.is_cuda:
        raise RuntimeError(_UNAVAILABLE + ": activations are not on a CUDA device and this backend has no CPU path")
    out = torch.empty(x.size(0), packed.size(1), dtype=torch.float32, device=x.device)
    ws = w_scale if w_scale.dtype in _SCALE else w_scale.float()
    # fp16 scales and shapes the tcgen05 kernel covers: int8 activations go to the tensor cores (exact products,
    # fp32 accumulation); anything else to the generic kernel with the reference's integer group sums
    fast = isinstance(packed, TiledWeights) or fast_path_covers(K, group, ws.dtype, x.dtype)
    return _grouped(lib, x.contiguous(), x_scale.float().contiguous(), offsets, [packed if isinstance(packed, TiledWeights) else packed.contiguous()],
                    [ws.contiguous()], K, group, fmt, out, False, ("auto" if fast else "generic") if algo == "auto" else algo)


def sort_by_expert(expert_ids: torch.Tensor, n_experts: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Flattened top-k expert ids [T*k] -> (row order sorting them by expert, offsets [E + 1])
    (reference ``ternary_cuda.py:114-118``): a stable counting sort in three small kernels."""
    lib = _require("auto")
    if not expert_ids.is_cuda:
        raise RuntimeError(_UNAVAILABLE + ": expert ids are not on a CUDA device")
    if expert_ids.dtype not in (torch.int64, torch.int32):
        raise RuntimeError("expert ids must be int64 or int32")
    ids = expert_ids.contiguous().view(-1)
    n = ids.numel()
    order = torch.empty(n, dtype=torch.int64, device=ids.device)
    offsets = torch.empty(n_experts + 1, dtype=torch.int64, device=ids.device)
    ws = torch.empty(max(1, lib.dst_sort_workspace_bytes(n, n_experts)), dtype=torch.uint8, device=ids.device)
    bad = torch.zeros(1, dtype=torch.int32, device=ids.device)
    with torch.cuda.device(ids.device):
        rc = lib.dst_sort_by_expert(ids.data_ptr(), int(ids.dtype == torch.int32), n, n_experts, order.data_ptr(),
                                    offsets.data_ptr(), bad.data_ptr(), ws.data_ptr(), _stream(ids))
    _lib.check(rc)
    return order, offsets


# --------------------------------------------------------------------------- bf16-activation path (Mode C/D)
def _as3(t: torch.Tensor) -> torch.Tensor:
    return t[None] if t.dim() == 2 else t


def ternary_gemm_bf16(x: torch.Tensor, packed_terms, scale_terms, K: int, group: int, fmt: str,
                      out_dtype=torch.float32, row_scale: torch.Tensor | None = None, algo: str = "auto",
                      out: torch.Tensor | None = None, accumulate: bool = False, backend: str = "auto") -> torch.Tensor:
    """[T, K] bf16 (or fp16) activations x k stacked terms ([N, Kp] uint8 + [N, G] fp16) -> [T, N].

    All terms are summed inside one launch (the reference makes one kernel pass per term and adds,
    ``boilerplate/ternary/ops.py:71-79``). ``accumulate=True`` adds into a float32 ``out``.
    """
    return grouped_ternary_gemm_bf16(x, None, [p if isinstance(p, TiledWeights) else _as3(p) for p in packed_terms],
                                     [_as3(s) for s in scale_terms], K, group,
                                     fmt, out_dtype, row_scale, algo, out, accumulate, backend)


def grouped_ternary_gemm_bf16(x: torch.Tensor, offsets, packed_terms, scale_terms, K: int, group: int, fmt: str,
                              out_dtype=torch.float32, row_scale: torch.Tensor | None = None, algo: str = "auto",
                              out: torch.Tensor | None = None, accumulate: bool = False, backend: str = "auto",
                              validate_offsets: bool = True) -> torch.Tensor:
    """Grouped form: rows of ``x`` sorted by expert, ``packed_terms[i]`` [E, N, Kp], ``scale_terms[i]`` [E, N, G].

    ``validate_offsets=False`` accepts a device ``offsets`` tensor without copying it to the host
    (the kernels then clamp row ranges to the row count instead).
    """
    _fmt_code(fmt)
    norm = isinstance(x, NormRows)
    if norm:
        if row_scale is not None:
            raise RuntimeError("normalised rows carry their own row factors")
        x, row_scale = x.data, x.factor
    if x.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError("the bf16 path takes bf16 or fp16 activations")
    lib = _require(backend)
    if not x.is_cuda:
        raise RuntimeError(_UNAVAILABLE + ": activations are not on a CUDA device and this backend has no CPU path")
    if out is None:
        out = torch.empty(x.size(0), packed_terms[0].size(1), dtype=out_dtype, device=x.device)
        accumulate = False
    if norm:
        if x.dtype != torch.float16 or not all(isinstance(p, TiledWeights) for p in packed_terms):
            raise RuntimeError("normalised rows are fp16 and go with tiled weights")
        return _grouped(lib, x.contiguous(), row_scale, offsets, list(packed_terms), [s.contiguous() for s in scale_terms], K, group,
                        fmt, out, accumulate, "prefill", validate_offsets, act_code=_lib.ACT_F16_NORM)
    return _grouped(lib, x.contiguous(), row_scale, offsets,
                    [p if isinstance(p, TiledWeights) else p.contiguous() for p in packed_terms],
                    [s.contiguous() for s in scale_terms], K, group, fmt, out, accumulate, algo, validate_offsets)
