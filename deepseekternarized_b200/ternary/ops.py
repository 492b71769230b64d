"""Ternary linear layers (Mode C with k terms, Mode D with k = 1) on B200: the surface of the
reference's ``boilerplate/ternary/ops.py`` (``quant_act_int8``, ``PackedTerm``, ``TernaryLinear``).

The engines hold one ``TernaryLinear`` per weight (reference ``engine/model.py:361-370``,
``engine/standard.py:37-42``) and call it with activations of any leading shape. Here every call
is one CUDA launch that sums all stacked terms; ``act="bf16"`` feeds bf16 activations with fp16
group scales and fp32 accumulation, ``act="int8"`` quantises per token first (one more kernel, which
for many rows writes the tensor-core kernel's input format directly) and follows the reference's int8
contract. Both modes keep their weights in the tiled device layout. There is no CPU or dequantised fallback.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import _lib
from ..kernels import ternary_b200 as kb
from .pack import unpack


def quant_act_int8(x: torch.Tensor, as_f16: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-token absmax int8: x ~= q * s, q in [-127, 127] (reference ``ops.py:20-25``), one kernel.
    ``as_f16``: q comes back as fp16 holding the same integers, the row format the tcgen05 GEMM reads directly."""
    lib = kb._require("auto")
    if not x.is_cuda:
        raise RuntimeError("B200 ternary kernel unavailable for CPU tensors")
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.size(-1))
    if x2.dtype not in (torch.float32, torch.bfloat16):
        x2 = x2.float()
    x2 = x2.contiguous()
    q = torch.empty(x2.shape, dtype=torch.float16 if as_f16 else torch.int8, device=x.device)
    s = torch.empty(x2.size(0), dtype=torch.float32, device=x.device)
    fn = lib.dst_quant_act_int8_f16 if as_f16 else lib.dst_quant_act_int8
    with torch.cuda.device(x.device):
        _lib.check(fn(x2.data_ptr(), int(x2.dtype == torch.float32), x2.size(0), x2.size(1), q.data_ptr(), s.data_ptr(), kb._stream(x2)))
    return q.view(*lead, -1), s.view(lead)


@dataclass
class PackedTerm:
    """One term of a stacked ternary weight (reference ``ops.py:28-31``)."""

    packed: torch.Tensor  # [N, ceil(K / per_byte)] uint8
    scale: torch.Tensor  # [N, G] fp16/bf16 as stored


class TernaryLinear:
    """Drop-in for the reference class (``ops.py:34-86``): same constructor, same call.

    ``backend`` accepts "auto", "b200" or "cuda"; anything else (the reference's "cpp"/"torch")
    raises, since this package has no CPU path. Weights are copied to the activation's device once
    and kept there, as the reference's ``_on`` does (``ops.py:41-45``); scales stay in their stored
    16-bit type (fp16 -> fp32 is exact, so reading fp16 in the kernel equals the reference's upcast,
    ``ops.py:37``).
    """

    def __init__(self, terms: list[PackedTerm], K: int, fmt: str, group: int, act: str = "int8", backend: str = "auto",
                 algo: str = "auto", decode_copy: bool = False):
        kb._fmt_code(fmt)
        if act not in ("int8", "bf16"):
            raise ValueError(f"unknown activation mode {act!r}")
        if backend not in kb.BACKENDS:
            raise RuntimeError(f"backend {backend!r} is unavailable in this package (no CPU path)")
        self.terms, self.K, self.fmt, self.group, self.act = terms, K, fmt, group, act
        self.backend, self.algo = backend, algo
        self.decode_copy = decode_copy  # TQ1: keep a tiled TQ2 copy of the trits on the device for few-row calls
        self._dev = None

    def _on(self, device):
        """([packed], [scale [1,N,G]]) on ``device``, copied once and kept. Shapes the fast kernels cover
        (group 128, K % 128 == 0, fp16 scales; both activation modes) are kept in the tiled device layout,
        everything else as the canonical ``[1, N, Kp]`` bytes."""
        if self._dev is None or self._dev[0] != device:
            packed = [t.packed.to(device).contiguous()[None] for t in self.terms]
            scales = []
            for t in self.terms:
                s = t.scale.to(device)
                if s.dtype not in (torch.float16, torch.float32, torch.bfloat16):
                    s = s.float()
                scales.append(s.contiguous()[None])
            if len({s.dtype for s in scales}) > 1:
                scales = [s.float() for s in scales]
            if self.algo != "generic" and kb.fast_path_covers(self.K, self.group, scales[0].dtype):
                packed = [kb.tile_weights(p, self.fmt, self.K, self.decode_copy) for p in packed]
            self._dev = (device, packed, scales)
        return self._dev[1], self._dev[2]

    @property
    def out_features(self) -> int:
        return self.terms[0].packed.size(0)

    def dequantized(self) -> torch.Tensor:
        """fp32 [N, K] ``sum_i unpack(packed_i) * scale_i`` (reference ``ops.py:51-58``), built with the unpack kernel."""
        dev = self._dev[0] if self._dev is not None else "cuda"
        packed, scales = self._on(torch.device(dev))
        w = None
        for p, s in zip(packed, scales):
            p = p.untile() if isinstance(p, kb.TiledWeights) else p
            d = unpack(p[0], self.fmt, self.K).float() * s[0].float().repeat_interleave(self.group, -1)[:, : self.K]
            w = d if w is None else w + d
        return w

    def __call__(self, x: torch.Tensor, out_dtype=torch.bfloat16) -> torch.Tensor:
        if not x.is_cuda:
            raise RuntimeError("B200 ternary kernel unavailable for CPU tensors (this backend has no CPU path)")
        shape = x.shape
        x2 = x.reshape(-1, self.K)
        packed, scales = self._on(x2.device)
        if self.act == "int8":
            lib = kb._require(self.backend)
            out = torch.empty(x2.size(0), self.out_features, dtype=torch.float32, device=x2.device)
            tiled = isinstance(packed[0], kb.TiledWeights)
            if tiled and self.algo in ("auto", "prefill") and x2.size(0) > 16:
                # many rows: quantise straight into the tcgen05 kernel's row format (2 launches per linear)
                qh, s = quant_act_int8(x2, as_f16=True)
                kb.grouped_ternary_gemm_bf16(kb.NormRows(qh, s), None, packed, scales, self.K, self.group, self.fmt, out=out,
                                             backend=self.backend)
            else:
                q, s = quant_act_int8(x2)
                kb._grouped(lib, q, s, None, packed, scales, self.K, self.group, self.fmt, out, False, self.algo)
        else:
            xa = x2 if x2.dtype in (torch.bfloat16, torch.float16) else x2.bfloat16()
            od = out_dtype if out_dtype in (torch.float32, torch.bfloat16, torch.float16) else torch.float32
            out = kb.grouped_ternary_gemm_bf16(xa, None, packed, scales, self.K, self.group, self.fmt, out_dtype=od,
                                               algo=self.algo, backend=self.backend)
        return out.view(*shape[:-1], -1).to(out_dtype)


def _gather_call(packed_ptrs, scale_ptrs, sdt, ids: torch.Tensor, V: int, K: int, fmt: str, group: int, pstride: int, sstride: int,
                 check: bool) -> torch.Tensor:
    import ctypes

    from .. import _lib
    from ..kernels import ternary_b200 as kb

    lib = kb._require("auto")
    flat = ids.reshape(-1).to(torch.int64).contiguous()
    out = torch.empty(flat.numel(), K, dtype=torch.bfloat16, device=flat.device)
    bad = torch.zeros(1, dtype=torch.int32, device=flat.device) if check else None
    n = len(packed_ptrs)
    pk = (ctypes.c_void_p * n)(*packed_ptrs)
    sc = (ctypes.c_void_p * n)(*scale_ptrs)
    with torch.cuda.device(flat.device):
        _lib.check(lib.dst_gather_dequant_rows_strided(pk, sc, n, kb._SCALE[sdt], flat.data_ptr(), flat.numel(), V, K, group, kb._fmt_code(fmt),
                                                       pstride, sstride, out.data_ptr(), bad.data_ptr() if check else None, kb._stream(flat)))
    if check and int(bad.item()):
        raise IndexError("table row index out of range")
    return out.view(*ids.shape, K)


def gather_dequant_rows(terms, ids: torch.Tensor, K: int, fmt: str, group: int, check: bool = True) -> torch.Tensor:
    """Rows ``ids`` of a ternary lookup table as bf16: ``sum_i unpack(packed_i[ids]) * scale_i[ids].repeat(group)``
    in fp32, then the cast (the engram-table lookup of ``boilerplate/engine/model.py:458-464``).

    ``terms``: PackedTerm list (canonical ``packed`` [V, Kp], ``scale`` [V, G]) on the device of ``ids``.
    ``check``: read the count of out-of-range ids back and raise IndexError as ``index_select`` does (a host
    synchronisation); without it such rows come back as zeros."""
    from ..kernels import ternary_b200 as kb

    if not ids.is_cuda:
        raise RuntimeError("the B200 ternary backend is unavailable: ids are not on a CUDA device and this backend has no CPU path")
    packed = [t.packed.contiguous() for t in terms]
    scales = [t.scale.contiguous() for t in terms]
    V = packed[0].size(0)
    G = -(-K // group)
    sdt = scales[0].dtype
    if sdt not in kb._SCALE or any(s.dtype != sdt for s in scales):
        raise RuntimeError("unexpected table scale dtype")
    for p_, s_ in zip(packed, scales):
        if p_.dtype != torch.uint8 or tuple(p_.shape) != (V, kb.packed_cols(fmt, K)) or tuple(s_.shape) != (V, G) or p_.device != ids.device or s_.device != ids.device:
            raise RuntimeError("inconsistent ternary table shapes")
    return _gather_call([p_.data_ptr() for p_ in packed], [s_.data_ptr() for s_ in scales], sdt, ids, V, K, fmt, group,
                        kb.packed_cols(fmt, K), G, check)


class LookupTable:
    """A ternary lookup table (the engram tables of ``boilerplate/engine/model.py:343-346``) laid out for random
    row reads: ONE record per table row holding the packed bytes of every stacked term followed by their scales, padded
    to 16 bytes. The canonical arrays put a row's pieces into 2 x terms distant places; the record makes a lookup one
    stretch of DRAM (two TQ1 terms of 256-wide rows: 112 bytes per record against 104 + 8 canonical; measured 1.2x
    faster, one term: no gain). ``rows(ids)`` returns what ``gather_dequant_rows`` returns, bit for bit."""

    def __init__(self, terms, K: int, fmt: str, group: int):
        from ..kernels import ternary_b200 as kb

        packed = [t.packed for t in terms]
        scales = [t.scale for t in terms]
        self.K, self.fmt, self.group, self.n_terms = K, fmt, group, len(terms)
        self.V = packed[0].size(0)
        Kp, G = kb.packed_cols(fmt, K), -(-K // group)
        self.sdt = scales[0].dtype
        if self.sdt not in kb._SCALE or any(s.dtype != self.sdt for s in scales):
            raise RuntimeError("unexpected table scale dtype")
        for p_, s_ in zip(packed, scales):
            if p_.dtype != torch.uint8 or tuple(p_.shape) != (self.V, Kp) or tuple(s_.shape) != (self.V, G) or not p_.is_cuda or s_.device != p_.device:
                raise RuntimeError("inconsistent ternary table shapes")
        esz = scales[0].element_size()
        self.scale_off = -(-(self.n_terms * Kp) // 4) * 4               # the scales start 4-byte aligned
        self.record = -(-(self.scale_off + self.n_terms * G * esz) // 16) * 16
        rec = torch.zeros(self.V, self.record, dtype=torch.uint8, device=packed[0].device)
        for i, (p_, s_) in enumerate(zip(packed, scales)):
            rec[:, i * Kp:(i + 1) * Kp] = p_
            rec[:, self.scale_off + i * G * esz: self.scale_off + (i + 1) * G * esz] = s_.contiguous().view(torch.uint8).view(self.V, G * esz)
        self.records, self._Kp, self._G, self._esz = rec, Kp, G, esz

    def rows(self, ids: torch.Tensor, check: bool = True) -> torch.Tensor:
        if not ids.is_cuda or ids.device != self.records.device:
            raise RuntimeError("the B200 ternary backend is unavailable: ids are not on the table's CUDA device and this backend has no CPU path")
        base = self.records.data_ptr()
        return _gather_call([base + i * self._Kp for i in range(self.n_terms)],
                            [base + self.scale_off + i * self._G * self._esz for i in range(self.n_terms)], self.sdt, ids, self.V, self.K,
                            self.fmt, self.group, self.record, self.record // self._esz, check)
