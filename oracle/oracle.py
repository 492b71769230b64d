"""numpy front end of the CPU oracle (``ternary_oracle.c``).

TEST INFRASTRUCTURE ONLY. This module is the checker that ``tests/``, the smoke check and the
bench's CPU-baseline leg compare the CUDA library against; the product package never imports it.
Parity is pinned against outputs of the reference itself (fixtures under ``tests/golden/``).

Every function names the reference lines (paths inside Vedant-Sood/DeepSeekTernarized) it follows.
Arrays are numpy; bf16 values are carried as float32 arrays that hold bf16-representable numbers
(``bf16_round`` produces them), fp16 scales as float16 or float32 arrays.
"""

from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "libternary_oracle.so"
_lib = None

FMT_CODE = {"tq1": 1, "tq2": 2}  # boilerplate/kernels/ternary_cuda.py:46-49


def build(force: bool = False) -> Path:
    """Compile the C oracle with the system gcc (``make -C oracle oracle``)."""
    src = _HERE / "ternary_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "oracle"], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(str(_LIB_PATH))
        i64, i32, p = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p
        L.orc_packed_cols.restype = i64
        L.orc_packed_cols.argtypes = [i32, i64]
        L.orc_tq1_lut.argtypes = [p]
        L.orc_pack.argtypes = [p, i64, i64, i32, p]
        L.orc_unpack.argtypes = [p, i64, i64, i32, p]
        L.orc_gemm.argtypes = [p, p, p, p, p, p, i64, i64, i64, i64, i32]
        L.orc_gemm_ref_i8.argtypes = [p, p, p, p, p, i64, i64, i64, i64, i32]
        L.orc_gemm_f64.argtypes = [p, p, p, p, i64, i64, i64, i64, i32]
        L.orc_grouped_gemm.argtypes = [p, p, p, p, p, p, p, i64, i64, i64, i64, i64, i32]
        L.orc_sort_by_expert.argtypes = [p, i64, i64, p, p]
        L.orc_quant_act_int8.argtypes = [p, i64, i64, p, p]
        _lib = L
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


def _check(rc, what):
    if rc != 0:
        raise ValueError(f"oracle {what}: invalid arguments")


# ------------------------------------------------------------------------------------ bf16 / fp16
def bf16_round(x) -> np.ndarray:
    """float32 -> nearest bf16 (ties to even), returned as float32 (what ``tensor.bfloat16()`` does)."""
    a = _c(x, np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    out = (r & 0xFFFFFFFF).astype(np.uint32).view(np.float32).reshape(a.shape)
    return np.where(np.isnan(a), a, out)


def bf16_bits(x) -> np.ndarray:
    """bf16-representable float32 array -> uint16 bit patterns."""
    return (bf16_round(x).view(np.uint32) >> 16).astype(np.uint16)


def from_bf16_bits(b) -> np.ndarray:
    return (_c(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


# ------------------------------------------------------------------------------------ format
def packed_cols(fmt: str, K: int) -> int:
    """boilerplate/ternary/pack.py:30-31"""
    return int(lib().orc_packed_cols(FMT_CODE[fmt], K))


def tq1_lut() -> np.ndarray:
    """boilerplate/ternary/pack.py:62-67"""
    out = np.empty((256, 5), np.int8)
    lib().orc_tq1_lut(_ptr(out))
    return out


def pack(trits, fmt: str) -> np.ndarray:
    """boilerplate/ternary/pack.py:43-45,54-59,77-78: int8 trits [N, K] -> uint8 [N, packed_cols]."""
    t = _c(trits, np.int8)
    N, K = t.shape
    out = np.empty((N, packed_cols(fmt, K)), np.uint8)
    _check(lib().orc_pack(_ptr(t), N, K, FMT_CODE[fmt], _ptr(out)), "pack")
    return out


def unpack(packed, fmt: str, K: int) -> np.ndarray:
    """boilerplate/ternary/pack.py:48-51,70-74,81-82"""
    p = _c(packed, np.uint8)
    N = p.shape[0]
    assert p.shape[1] == packed_cols(fmt, K)
    out = np.empty((N, K), np.int8)
    _check(lib().orc_unpack(_ptr(p), N, K, FMT_CODE[fmt], _ptr(out)), "unpack")
    return out


def dequantized(terms, K: int, group: int, fmt: str) -> np.ndarray:
    """boilerplate/ternary/ops.py:51-58: fp64 ``sum_i unpack(packed_i) * scale_i`` (scale repeated per group)."""
    w = None
    for packed, scale in terms:
        s = np.repeat(np.asarray(scale, np.float64), group, axis=-1)[:, :K]
        d = unpack(packed, fmt, K).astype(np.float64) * s
        w = d if w is None else w + d
    return w


# ------------------------------------------------------------------------------------ GEMM
def gemm_f32(x, packed, w_scale, K: int, group: int, fmt: str, out=None) -> np.ndarray:
    """The reference C++ kernel's float-activation path, boilerplate/kernels/csrc/boilerplate_cpu.cpp:70-77,109-127.

    ``x`` [M, K] float32 (bf16 activations upcast, boilerplate/ternary/ops.py:66). Accumulates into ``out``.
    """
    x = _c(x, np.float32)
    p = _c(packed, np.uint8)
    s = _c(w_scale, np.float32)
    M, N = x.shape[0], p.shape[0]
    if out is None:
        out = np.zeros((M, N), np.float32)
    _check(lib().orc_gemm(_ptr(out), _ptr(x), None, None, _ptr(p), _ptr(s), M, N, K, group, FMT_CODE[fmt]), "gemm_f32")
    return out


def gemm_i8(x_i8, x_scale, packed, w_scale, K: int, group: int, fmt: str, out=None) -> np.ndarray:
    """The reference C++ kernel's int8 path, boilerplate/kernels/csrc/boilerplate_cpu.cpp:34-68,109-127."""
    x = _c(x_i8, np.int8)
    xs = _c(x_scale, np.float32)
    p = _c(packed, np.uint8)
    s = _c(w_scale, np.float32)
    M, N = x.shape[0], p.shape[0]
    if out is None:
        out = np.zeros((M, N), np.float32)
    _check(lib().orc_gemm(_ptr(out), None, _ptr(x), _ptr(xs), _ptr(p), _ptr(s), M, N, K, group, FMT_CODE[fmt]), "gemm_i8")
    return out


def gemm_ref_i8(x_i8, x_scale, packed, w_scale, K: int, group: int, fmt: str) -> np.ndarray:
    """boilerplate/kernels/ternary_cuda.py:52-64 (ternary_gemm_ref)."""
    x = _c(x_i8, np.int8)
    xs = _c(x_scale, np.float32)
    p = _c(packed, np.uint8)
    s = _c(w_scale, np.float32)
    M, N = x.shape[0], p.shape[0]
    out = np.empty((M, N), np.float32)
    _check(lib().orc_gemm_ref_i8(_ptr(out), _ptr(x), _ptr(xs), _ptr(p), _ptr(s), M, N, K, group, FMT_CODE[fmt]), "gemm_ref_i8")
    return out


def gemm_f64(x, terms, K: int, group: int, fmt: str) -> np.ndarray:
    """fp64 dequantized product ``X @ W.T`` summed over the terms: the tolerance target."""
    x = _c(x, np.float32)
    M = x.shape[0]
    N = np.asarray(terms[0][0]).shape[0]
    out = np.zeros((M, N), np.float64)
    for packed, scale in terms:
        p = _c(packed, np.uint8)
        s = _c(scale, np.float32)
        _check(lib().orc_gemm_f64(_ptr(out), _ptr(x), _ptr(p), _ptr(s), M, N, K, group, FMT_CODE[fmt]), "gemm_f64")
    return out


def grouped_gemm_f32(x, offsets, packed, w_scale, K: int, group: int, fmt: str, out=None) -> np.ndarray:
    """boilerplate/kernels/ternary_cuda.py:90-111 with float activations: packed [E,N,Kp], w_scale [E,N,G]."""
    x = _c(x, np.float32)
    offs = _c(offsets, np.int64)
    p = _c(packed, np.uint8)
    s = _c(w_scale, np.float32)
    E, N = p.shape[0], p.shape[1]
    if offs.size != E + 1:
        raise ValueError("offsets must be nondecreasing, start at 0, end at the row count, one per expert + 1")
    if out is None:
        out = np.zeros((x.shape[0], N), np.float32)
    rc = lib().orc_grouped_gemm(_ptr(out), _ptr(x), None, None, _ptr(offs), _ptr(p), _ptr(s), E, x.shape[0], N, K, group, FMT_CODE[fmt])
    if rc:
        raise ValueError("offsets must be nondecreasing, start at 0, end at the row count, one per expert + 1")
    return out


def grouped_gemm_i8(x_i8, x_scale, offsets, packed, w_scale, K: int, group: int, fmt: str) -> np.ndarray:
    x = _c(x_i8, np.int8)
    xs = _c(x_scale, np.float32)
    offs = _c(offsets, np.int64)
    p = _c(packed, np.uint8)
    s = _c(w_scale, np.float32)
    E, N = p.shape[0], p.shape[1]
    if offs.size != E + 1:
        raise ValueError("offsets must be nondecreasing, start at 0, end at the row count, one per expert + 1")
    out = np.zeros((x.shape[0], N), np.float32)
    rc = lib().orc_grouped_gemm(_ptr(out), None, _ptr(x), _ptr(xs), _ptr(offs), _ptr(p), _ptr(s), E, x.shape[0], N, K, group, FMT_CODE[fmt])
    if rc:
        raise ValueError("offsets must be nondecreasing, start at 0, end at the row count, one per expert + 1")
    return out


def sort_by_expert(expert_ids, n_experts: int):
    """boilerplate/kernels/ternary_cuda.py:114-118: (stable order, offsets[E+1])."""
    ids = _c(expert_ids, np.int64).ravel()
    order = np.empty(ids.size, np.int64)
    offsets = np.empty(n_experts + 1, np.int64)
    _check(lib().orc_sort_by_expert(_ptr(ids), ids.size, n_experts, _ptr(order), _ptr(offsets)), "sort_by_expert")
    return order, offsets


def quant_act_int8(x):
    """boilerplate/ternary/ops.py:20-25"""
    x = _c(x, np.float32)
    M, K = x.shape
    q = np.empty((M, K), np.int8)
    s = np.empty(M, np.float32)
    lib().orc_quant_act_int8(_ptr(x), M, K, _ptr(q), _ptr(s))
    return q, s


def ternary_linear(x, terms, K: int, group: int, fmt: str, out_bf16: bool = True) -> np.ndarray:
    """boilerplate/ternary/ops.py:60-86 with act="bf16", backend="cpp": k kernel passes accumulated in
    one fp32 buffer (lines 75-79), then the cast to ``out_dtype`` (line 86; default bf16)."""
    x = _c(x, np.float32)
    lead = x.shape[:-1]
    x2 = x.reshape(-1, K)
    out = None
    for packed, scale in terms:
        out = gemm_f32(x2, packed, np.asarray(scale, np.float32), K, group, fmt, out=out)
    out = bf16_round(out) if out_bf16 else out
    return out.reshape(*lead, -1)


# ------------------------------------------------------------------------------------ MoE layer
def route_softmax_topk(x, gate_w, top_k: int, route_scale: float = 1.0):
    """boilerplate/engine/model.py:389-405 with score_func="softmax", gate_temp=1, no bias,
    norm_topk_prob=True: fp32 gate GEMM -> softmax -> top-k (descending score; on equal scores the
    lower expert id first) -> gather -> renormalise by (sum + 1e-20) -> x route_scale."""
    logits = _c(x, np.float32) @ _c(gate_w, np.float32).T
    return route_from_logits(logits, top_k, route_scale)


def route_from_logits(logits, top_k: int, route_scale: float = 1.0, score_func: str = "softmax", bias=None,
                      gate_temp: float = 1.0, norm_topk_prob: bool = True):
    """boilerplate/engine/model.py:391-405 from ``logits = F.linear(x.float(), gate_w)``: divide by the temperature,
    score function, top-k of (scores + bias) (descending; on equal values the lower expert id first), weights from
    the unbiased scores, optional renormalisation by (sum + 1e-20), times route_scale."""
    z = (_c(logits, np.float32) / np.float32(gate_temp)).astype(np.float32)
    if score_func == "softmax":
        z = z - z.max(-1, keepdims=True)
        e = np.exp(z, dtype=np.float32)
        scores = (e / e.sum(-1, keepdims=True, dtype=np.float32)).astype(np.float32)
    elif score_func == "sigmoid":
        scores = (np.float32(1.0) / (np.float32(1.0) + np.exp(-z, dtype=np.float32))).astype(np.float32)
    elif score_func == "sqrtsoftplus":
        sp = np.where(z > 20, z, np.log1p(np.exp(np.minimum(z, 20), dtype=np.float32), dtype=np.float32))
        scores = np.sqrt(sp, dtype=np.float32)
    else:
        raise ValueError(f"unknown score function {score_func!r}")
    biased = scores if bias is None else (scores + _c(bias, np.float32)).astype(np.float32)
    idx = np.argsort(-biased, axis=-1, kind="stable")[:, :top_k]
    w = np.take_along_axis(scores, idx, -1)
    if norm_topk_prob and top_k > 1:
        w = w / (w.sum(-1, keepdims=True, dtype=np.float32) + np.float32(1e-20))
    return (w * np.float32(route_scale)).astype(np.float32), idx.astype(np.int64)


def silu(x):
    x = _c(x, np.float32)
    return (x / (np.float32(1.0) + np.exp(-x, dtype=np.float32))).astype(np.float32)


def swiglu_expert(x, w1, w2, w3, weights, K_hidden, K_inter, group, fmt, swiglu_limit=0.0):
    """boilerplate/engine/model.py:376-387. w1/w3: hidden->inter (gate/up), w2: inter->hidden; each a
    list of (packed, scale) terms. ``weights`` [rows, 1] multiplies before w2. Linears return bf16."""
    gate = ternary_linear(x, w1, K_hidden, group, fmt)
    up = ternary_linear(x, w3, K_hidden, group, fmt)
    if swiglu_limit > 0:
        up = np.clip(up, -swiglu_limit, swiglu_limit)
        gate = np.minimum(gate, swiglu_limit)
    h = silu(gate) * up
    if weights is not None:
        h = (weights.astype(np.float32) * h).astype(np.float32)
    return ternary_linear(bf16_round(h), w2, K_inter, group, fmt)


def moe_layer(x, weights, indices, experts, hidden, inter, group, fmt, swiglu_limit=0.0, shared=None):
    """boilerplate/engine/model.py:407-422: experts in increasing id, each over its tokens in token order, fp32
    accumulation ``y[idx] += w2(...)``, then ``y += swiglu(shared, x)`` (``shared`` = (w1, w2, w3) terms or None),
    final cast to bf16.

    ``experts[e] = (w1_terms, w2_terms, w3_terms)``; ``weights``/``indices`` [T, k] from routing.
    """
    x = _c(x, np.float32)
    y = np.zeros_like(x, dtype=np.float32)
    for e in range(len(experts)):
        idx, top = np.nonzero(indices == e)
        if idx.size == 0:
            continue
        w1, w2, w3 = experts[e]
        y[idx] += swiglu_expert(x[idx], w1, w2, w3, weights[idx, top, None], hidden, inter, group, fmt, swiglu_limit)
    if shared is not None:
        y += swiglu_expert(x, shared[0], shared[1], shared[2], None, hidden, inter, group, fmt, swiglu_limit)
    return bf16_round(y)


def gather_dequant_rows(ids, terms, K: int, group: int, fmt: str) -> np.ndarray:
    """boilerplate/engine/model.py:458-464 (ternary engram-table lookup): for every id the row
    ``sum_i unpack(packed_i[id]) * scale_i[id].repeat(group)[:K]`` in fp32 (terms added in order), cast to bf16
    (returned as float32 holding bf16 values)."""
    flat = np.asarray(ids, np.int64).reshape(-1)
    vals = None
    for packed, scale in terms:
        t = unpack(np.ascontiguousarray(packed[flat]), fmt, K).astype(np.float32)
        sc = np.repeat(np.asarray(scale)[flat].astype(np.float32), group, axis=-1)[:, :K]
        v = (t * sc).astype(np.float32)
        vals = v if vals is None else (vals + v).astype(np.float32)
    return bf16_round(vals).reshape(*np.asarray(ids).shape, K)


def moe_layer_standard(x, logits, experts, top_k, hidden, inter, group, fmt, norm_topk_prob=True):
    """boilerplate/engine/standard.py:154-176 (OLMoE-style layer) with bf16 as the model dtype: softmax over all
    experts -> top-k -> optional renormalisation -> weights to bf16; per expert in increasing id
    ``down(silu(gate(x)) * up(x)) * w`` with every intermediate a bf16 tensor; ``index_add_`` into a bf16 output.
    Returns (y as float32 holding bf16 values, weights [T, k] float32 before the bf16 cast, indices)."""
    x = _c(x, np.float32)
    logits = _c(logits, np.float32)
    z = logits - logits.max(-1, keepdims=True)
    ez = np.exp(z, dtype=np.float32)
    scores = (ez / ez.sum(-1, keepdims=True, dtype=np.float32)).astype(np.float32)
    idx = np.argsort(-scores, axis=-1, kind="stable")[:, :top_k]
    w = np.take_along_axis(scores, idx, -1)
    if norm_topk_prob:
        w = (w / w.sum(-1, keepdims=True, dtype=np.float32)).astype(np.float32)
    wb = bf16_round(w)
    y = np.zeros_like(x, dtype=np.float32)
    for e in range(len(experts)):
        tok, slot = np.nonzero(idx == e)
        if tok.size == 0:
            continue
        w1, w2, w3 = experts[e]
        gate = ternary_linear(x[tok], w1, hidden, group, fmt)
        up = ternary_linear(x[tok], w3, hidden, group, fmt)
        h = bf16_round(bf16_round(silu(gate)) * up)
        d = ternary_linear(h, w2, inter, group, fmt)
        r = bf16_round(d * wb[tok, slot, None])
        y[tok] = bf16_round(y[tok] + r)
    return y, w, idx.astype(np.int64)


def moe_layer_f64(x, weights, indices, experts, hidden, inter, group, fmt, swiglu_limit=0.0, shared=None):
    """The same layer in fp64 with no intermediate rounding (dequantized weights, boilerplate/ternary/ops.py:51-58):
    the yardstick for how much of a layer-level difference is bf16 rounding noise."""
    x = np.asarray(x, np.float64)
    y = np.zeros_like(x)
    for e in range(len(experts)):
        idx, top = np.nonzero(indices == e)
        if idx.size == 0:
            continue
        w1, w2, w3 = (dequantized(t, K, group, fmt) for t, K in zip(experts[e], (hidden, inter, hidden)))
        g, u = x[idx] @ w1.T, x[idx] @ w3.T
        if swiglu_limit > 0:
            u, g = np.clip(u, -swiglu_limit, swiglu_limit), np.minimum(g, swiglu_limit)
        h = np.asarray(weights, np.float64)[idx, top, None] * (g / (1.0 + np.exp(-g))) * u
        y[idx] += h @ w2.T
    if shared is not None:
        w1, w2, w3 = (dequantized(t, K, group, fmt) for t, K in zip(shared, (hidden, inter, hidden)))
        g, u = x @ w1.T, x @ w3.T
        if swiglu_limit > 0:
            u, g = np.clip(u, -swiglu_limit, swiglu_limit), np.minimum(g, swiglu_limit)
        y += ((g / (1.0 + np.exp(-g))) * u) @ w2.T
    return y


# ------------------------------------------------------------------------------------ metrics
def rel_fro(a, ref) -> float:
    """boilerplate/reference/compare.py:61-62: ||a - ref||_F / ||ref||_F"""
    a, ref = np.asarray(a, np.float64), np.asarray(ref, np.float64)
    d = np.linalg.norm(ref)
    return float(np.linalg.norm(a - ref) / d) if d > 0 else float(np.linalg.norm(a - ref))


def cosine(a, ref) -> float:
    a, ref = np.asarray(a, np.float64).ravel(), np.asarray(ref, np.float64).ravel()
    d = np.linalg.norm(a) * np.linalg.norm(ref)
    return float(a @ ref / d) if d > 0 else 1.0


# ------------------------------------------------------------------------------------ seeded inputs
def synth_trits(rng: np.random.Generator, shape, p_zero=0.4) -> np.ndarray:
    """i.i.d. trits with P(0)=p_zero and P(+1)=P(-1)=(1-p_zero)/2."""
    u = rng.random(shape)
    half = (1.0 - p_zero) / 2
    return np.where(u < p_zero, 0, np.where(u < p_zero + half, 1, -1)).astype(np.int8)


def synth_scales(rng: np.random.Generator, shape, mu=-4.0, sigma=0.3) -> np.ndarray:
    """lognormal(mu, sigma) group scales rounded to fp16."""
    return np.exp(rng.normal(mu, sigma, shape)).astype(np.float16)


def synth_acts(rng: np.random.Generator, shape) -> np.ndarray:
    """N(0,1) activations rounded to bf16 (returned as float32)."""
    return bf16_round(rng.standard_normal(shape).astype(np.float32))


def reference_module():
    """The reference's own C++ CPU kernel built into ``oracle/_ref`` (None when it was not built)."""
    path = _HERE / "_ref" / "boilerplate_cpu_ref.so"
    if not path.exists() or os.environ.get("DST_NO_REF"):
        return None
    import importlib.util

    import torch  # noqa: F401  (the module links against torch)

    spec = importlib.util.spec_from_file_location("boilerplate_cpu_ref", str(path))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod
