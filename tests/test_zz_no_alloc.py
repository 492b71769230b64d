"""The no-allocation entry point ``dst_ternary_grouped_gemm_noalloc`` against the regular entry point.

Some callers of this library cannot allocate device memory when they need a GEMM: a serving loop
whose memory was handed out at start-up, a thread that must not take the allocator's lock or stall
on the device-wide synchronisation ``cudaMalloc``/``cudaFree`` may perform, a plug-in that only ever
receives pointers. For them the library carries a fixed scratch array inside its own image. This
test calls that entry directly through the C ABI (ctypes, no helper in between), twice in a row with
different problem sizes so the second call meets the first call's leftovers in the shared array,
and checks each result against ``dst_ternary_grouped_gemm`` (tcgen05 kernel, caller-provided
workspace) and against the fp64 dequantized product within the tolerance the other parity tests use.
The file is named so pytest collects it last.
"""

from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.helpers import bf16_tensor, check_gemm, make_terms

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _run_both(lib, _lib, kb, fmt, E, rows_per_expert, N, K, k_terms, seed):
    rng = np.random.default_rng(seed)
    terms = make_terms(rng, N, K, 128, fmt, k_terms, lead=(E,))
    counts = np.array(rows_per_expert)
    offsets = np.concatenate([[0], counts.cumsum()]).astype(np.int64)
    T = int(offsets[-1])
    x = O.synth_acts(rng, (T, K))
    xt = bf16_tensor(x, DEV)
    tiled = [kb.tile_weights(torch.from_numpy(p).to(DEV), fmt, K) for p, _ in terms]
    scales = [torch.from_numpy(s).to(DEV) for _, s in terms]
    offs_dev = torch.from_numpy(offsets).to(DEV)
    offs_host = (ctypes.c_int64 * (E + 1))(*offsets.tolist())
    pk = (ctypes.c_void_p * k_terms)(*[t.data.data_ptr() for t in tiled])
    sc = (ctypes.c_void_p * k_terms)(*[s.data_ptr() for s in scales])
    code = _lib.FMT_TQ2 if fmt == "tq2" else _lib.FMT_TQ1
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    # existing entry: tcgen05 kernel with a workspace allocated by the caller (torch)
    want = torch.empty(T, N, dtype=torch.float32, device=DEV)
    ws_bytes = lib.dst_gemm_workspace_bytes(_lib.ALGO_PREFILL, _lib.ACT_BF16, T, K)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=DEV)
    rc = lib.dst_ternary_grouped_gemm(want.data_ptr(), _lib.OUT_F32, 0, xt.data_ptr(), _lib.ACT_BF16, None, offs_dev.data_ptr(), offs_host,
                                      pk, _lib.LAYOUT_TILED, sc, k_terms, _lib.SCALE_F16, E, T, N, K, 128, code, _lib.ALGO_PREFILL,
                                      ws.data_ptr(), ws_bytes, stream)
    assert rc == _lib.OK, _lib.status_string(rc)

    # new entry: same kernel, scratch inside the library, nothing allocated by the call
    got = torch.full((T, N), float("nan"), dtype=torch.float32, device=DEV)
    torch.cuda.synchronize()
    reserved_before = torch.cuda.memory_reserved()
    rc = lib.dst_ternary_grouped_gemm_noalloc(got.data_ptr(), _lib.OUT_F32, 0, xt.data_ptr(), _lib.ACT_BF16, None, offs_dev.data_ptr(),
                                              offs_host, pk, sc, k_terms, E, T, N, K, code, stream)
    assert rc == _lib.OK, _lib.status_string(rc)
    torch.cuda.synchronize()
    assert torch.cuda.memory_reserved() == reserved_before  # torch's allocator was not involved
    assert lib.dst_check_device_status(stream) == _lib.OK

    got_np, want_np = got.cpu().numpy(), want.cpu().numpy()
    assert np.isfinite(got_np).all()
    assert O.rel_fro(got_np, want_np) <= 2e-3 and O.cosine(got_np, want_np) >= 0.99999
    assert np.array_equal(got_np, want_np)  # same kernel, same inputs: in fact bit-identical
    for e in range(E):  # and both within the north-star tolerance of the fp64 dequantized product
        a, b = int(offsets[e]), int(offsets[e + 1])
        if b > a:
            check_gemm(got_np[a:b], x[a:b], [(p[e], s[e]) for p, s in terms], K, 128, fmt)
    return T


def test_noalloc_entry_matches_regular_entry_on_two_calls_in_a_row():
    from deepseekternarized_b200 import _lib
    from deepseekternarized_b200.kernels import ternary_b200 as kb

    lib = kb.ext()
    assert lib is not None, "CUDA library not loaded: no fallback exists"
    # call 1: TQ1, three experts (one empty), K = 4096 -> fills most of the scratch (8 MiB for 1000 rows)
    _run_both(lib, _lib, kb, "tq1", 3, [700, 0, 300], 256, 4096, 1, seed=101)
    # call 2, straight after: TQ2 with two stacked terms, fewer rows and a shorter K, so the array still holds
    # call 1's bytes beyond what this call rewrites
    _run_both(lib, _lib, kb, "tq2", 2, [37, 150], 384, 2048, 2, seed=202)


def test_noalloc_entry_refuses_what_does_not_fit():
    from deepseekternarized_b200 import _lib
    from deepseekternarized_b200.kernels import ternary_b200 as kb

    lib = kb.ext()
    assert lib is not None
    pk = (ctypes.c_void_p * 1)(0x1000)
    # 1025 rows of K = 4096 need 8 MiB + 8 KiB of fp16 activations alone: beyond the fixed array
    rc = lib.dst_ternary_grouped_gemm_noalloc(0x1000, _lib.OUT_F32, 0, 0x1000, _lib.ACT_BF16, None, None, None, pk, pk, 1, 1, 1100, 128,
                                              4096, _lib.FMT_TQ1, None)
    assert rc == _lib.ERR_TOO_LARGE
    assert b"scratch" in lib.dst_status_string(rc)
    # malformed arguments are refused before anything else happens, as in the regular entry
    assert lib.dst_ternary_grouped_gemm_noalloc(0x1000, _lib.OUT_F32, 0, 0x1000, _lib.ACT_I8, None, None, None, pk, pk, 1, 1, 8, 128, 4096,
                                                _lib.FMT_TQ1, None) == _lib.ERR_BAD_ARG
    assert lib.dst_ternary_grouped_gemm_noalloc(0x1000, _lib.OUT_F32, 0, 0x1000, _lib.ACT_BF16, None, None, None, pk, pk, 1, 1, 8, 128, 200,
                                                _lib.FMT_TQ1, None) == _lib.ERR_UNSUPPORTED
