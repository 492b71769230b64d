"""The C-ABI library builds for sm_100a, loads, and exports every symbol the public header declares.
No compute entry is called with real work here: only argument checks that return before any launch."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

from deepseekternarized_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    _lib.build()
    return _lib.load()


def declared_symbols():
    text = (ROOT / "include" / "dst_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dst_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    names = declared_symbols()
    assert len(names) >= 14
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/dst_b200.h but not exported"
    assert set(names) == set(_lib._SIGNATURES), "ctypes signatures and header disagree"


def test_version_and_strings(lib):
    assert lib.dst_abi_version() == 1
    assert lib.dst_status_string(0) == b"ok"
    assert b"offsets" in lib.dst_status_string(_lib.ERR_BAD_OFFSETS)
    assert lib.dst_last_cuda_error() == b""


@pytest.mark.parametrize("fmt,K,want", [(2, 4096, 1024), (1, 4096, 820), (1, 2048, 410), (2, 1, 1), (1, 7, 2), (3, 8, -1), (1, 0, -1)])
def test_packed_cols(lib, fmt, K, want):
    assert lib.dst_packed_cols(fmt, K) == want


def _gemm(lib, **kw):
    """Call the grouped GEMM entry with placeholder (never dereferenced) pointers; only argument checks run."""
    a = dict(out=0x1000, out_dtype=0, accumulate=0, x=0x1000, act=0, row_scale=None, offsets=None, offsets_host=None,
             layout=0, n_terms=1, scale_dtype=0, E=1, T=4, N=8, K=128, group=128, fmt=2, algo=1, ws=None, ws_bytes=0)
    a.update(kw)
    pk = (ctypes.c_void_p * 4)(0x1000, 0x1000, 0x1000, 0x1000)
    return lib.dst_ternary_grouped_gemm(a["out"], a["out_dtype"], a["accumulate"], a["x"], a["act"], a["row_scale"], a["offsets"],
                                        a["offsets_host"], pk, a["layout"], pk, a["n_terms"], a["scale_dtype"], a["E"], a["T"],
                                        a["N"], a["K"], a["group"], a["fmt"], a["algo"], a["ws"], a["ws_bytes"], None)


@pytest.mark.parametrize("kw,want", [
    (dict(K=0), _lib.ERR_BAD_ARG), (dict(K=2**62), _lib.ERR_BAD_SHAPE), (dict(group=0), _lib.ERR_BAD_ARG),
    (dict(fmt=0), _lib.ERR_BAD_ARG), (dict(fmt=3), _lib.ERR_BAD_ARG), (dict(n_terms=0), _lib.ERR_BAD_ARG),
    (dict(n_terms=5), _lib.ERR_BAD_ARG), (dict(out_dtype=7), _lib.ERR_BAD_ARG), (dict(act=9), _lib.ERR_BAD_ARG),
    (dict(scale_dtype=-1), _lib.ERR_BAD_ARG), (dict(algo=9), _lib.ERR_BAD_ARG), (dict(E=70000, offsets=0x1000), _lib.ERR_BAD_SHAPE),
    (dict(E=2), _lib.ERR_BAD_ARG),  # several experts need offsets
    (dict(accumulate=1, out_dtype=1), _lib.ERR_BAD_ARG), (dict(T=-1), _lib.ERR_BAD_ARG), (dict(out=None), _lib.ERR_BAD_ARG),
    (dict(x=None), _lib.ERR_BAD_ARG), (dict(T=0), _lib.OK), (dict(N=0), _lib.OK),
    (dict(layout=2), _lib.ERR_BAD_ARG),
    (dict(layout=1, algo=1), _lib.ERR_UNSUPPORTED),                      # the generic kernel reads canonical weights only
    (dict(layout=0, algo=3), _lib.ERR_UNSUPPORTED),                      # the tcgen05 kernel reads tiled weights only
    (dict(layout=1, algo=3, ws=None), _lib.ERR_UNSUPPORTED),             # ... and needs its workspace
    (dict(layout=1, algo=3, group=64, ws=0x1000, ws_bytes=1 << 20), _lib.ERR_UNSUPPORTED),
    (dict(layout=1, algo=3, K=192, ws=0x1000, ws_bytes=1 << 20), _lib.ERR_UNSUPPORTED),
])
def test_grouped_gemm_rejects_bad_arguments_before_launch(lib, kw, want):
    """The reference's native entries refuse malformed arguments before touching memory
    (tests/test_kernel_security.py:25-38 of the reference); so does the C ABI."""
    assert _gemm(lib, **kw) == want


@pytest.mark.parametrize("offs,T,want", [([0, 2, 1, 4], 4, _lib.ERR_BAD_OFFSETS), ([1, 2, 3, 4], 4, _lib.ERR_BAD_OFFSETS),
                                         ([0, 1, 2, 3], 4, _lib.ERR_BAD_OFFSETS), ([0, 0, 0, 0], 0, _lib.OK)])
def test_host_offsets_are_validated(lib, offs, T, want):
    host = (ctypes.c_int64 * 4)(*offs)
    assert _gemm(lib, E=3, T=T, offsets=0x1000, offsets_host=host) == want


def test_other_entries_reject_bad_arguments(lib):
    assert lib.dst_pack(None, 1, 0, 2, None, None) == _lib.ERR_BAD_ARG
    assert lib.dst_pack(None, 1, 8, 5, None, None) == _lib.ERR_BAD_ARG
    assert lib.dst_pack(None, 0, 8, 2, None, None) == _lib.OK
    assert lib.dst_unpack(None, 4, 8, 2, None, None) == _lib.ERR_BAD_ARG
    assert lib.dst_unpack(None, 0, 8, 1, None, None) == _lib.OK
    assert lib.dst_quant_act_int8(None, 0, 1, 0, None, None, None) == _lib.ERR_BAD_ARG
    assert lib.dst_route_softmax_topk(None, 4, 2000, 2, 1.0, None, None, None) == _lib.ERR_UNSUPPORTED
    assert lib.dst_route_softmax_topk(None, 4, 8, 9, 1.0, None, None, None) == _lib.ERR_UNSUPPORTED
    assert lib.dst_route_softmax_topk(None, 0, 8, 2, 1.0, None, None, None) == _lib.OK
    assert lib.dst_sort_by_expert(None, 0, 5, 0, None, None, None, None, None) == _lib.ERR_BAD_ARG
    assert lib.dst_sort_workspace_bytes(2048, 384) == 2 * 384 * 4
    assert lib.dst_gather_rows(None, None, 4, 0, 1, None, None) == _lib.ERR_BAD_ARG
    assert lib.dst_swiglu(None, None, None, 4, 0, 0.0, None, None) == _lib.ERR_BAD_ARG
    assert lib.dst_combine(None, None, None, 4, 9, 8, None, None, None) == _lib.ERR_BAD_ARG
    assert lib.dst_tiled_bytes(1, 384, 4096, 4096) == 384 * 32 * 13 * 8192
    assert lib.dst_tiled_bytes(2, 1, 70, 4160) == 1 * 1 * 17 * 8192
    assert lib.dst_tiled_bytes(3, 1, 8, 8) == -1
    assert lib.dst_tile_weights(None, 1, 8, 0, 2, None, None) == _lib.ERR_BAD_ARG
    assert lib.dst_tile_weights(0x1000, 1, 8, 64, 2, 0x1004, None) == _lib.ERR_ALIGNMENT
    assert lib.dst_untile_weights(None, 0, 8, 64, 1, None, None) == _lib.OK
    # the scatter form of the grouped GEMM: a destination table and at least one two-byte-typed buffer
    peers = (ctypes.c_void_p * 2)(0x1000, 0x2000)
    args = (0x1000, 0, None, None, None, 0x1000, 0x1000, 1, 0, 4, 64, 128, 128, 128, 1, None, 0, None)
    assert lib.dst_ternary_grouped_gemm_scatter(None, 2, 64, 0x1000, 1, *args) == _lib.ERR_BAD_ARG
    assert lib.dst_ternary_grouped_gemm_scatter(peers, 2, 64, None, 1, *args) == _lib.ERR_BAD_ARG
    assert lib.dst_ternary_grouped_gemm_scatter(peers, 0, 64, 0x1000, 1, *args) == _lib.ERR_BAD_ARG
    assert lib.dst_ternary_grouped_gemm_scatter(peers, 2, -1, 0x1000, 1, *args) == _lib.ERR_BAD_ARG
    assert lib.dst_ternary_grouped_gemm_scatter(peers, 2, 64, 0x1000, 0, *args) == _lib.ERR_UNSUPPORTED  # fp32 rows
    assert lib.dst_ep_combine_returned(None, None, None, None, 4, 9, 8, None, None, None, None) == _lib.ERR_BAD_ARG
    assert lib.dst_ep_combine_returned(None, None, None, None, 0, 6, 8, None, None, None, None) == _lib.OK
    assert lib.dst_ep_combine_returned(None, None, None, None, 4, 6, 12, None, None, None, None) == _lib.ERR_UNSUPPORTED
    assert lib.dst_gather_dequant_rows_strided(None, None, 1, 0, None, 4, 10, 256, 128, 1, 10, 2, None, None, None) == _lib.ERR_BAD_ARG  # rows overlap
    assert lib.dst_decode_row_limit(1, 384, 4096) == 16 and lib.dst_decode_row_limit(2, 1, 4096) == 16
    assert lib.dst_gemm_workspace_bytes(_lib.ALGO_GENERIC, 0, 100, 4096) == 0
    assert lib.dst_gemm_workspace_bytes(_lib.ALGO_PREFILL, 0, 100, 4096) >= 100 * 4096 * 2 + 400
