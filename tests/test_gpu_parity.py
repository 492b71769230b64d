"""GPU parity: the CUDA library, called through the C ABI by the drop-in modules, against the CPU
oracle and the reference-generated golden fixtures. Bit-exact for packing, sorting and int8
quantisation; for GEMM outputs the north-star tolerance (relative Frobenius error <= 2e-3, cosine
>= 0.99999 against the fp64 dequantized product) plus the reference's own allclose bounds
(rtol 1e-4, atol 1e-3: tests/test_ternary.py:98, tests/test_ternary_cuda.py:80 of the reference)."""

from __future__ import annotations

import os

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.helpers import bf16_numpy, bf16_tensor, check_gemm, check_layer, make_experts, make_terms, stack_experts

pytestmark = pytest.mark.gpu
FMT = {1: "tq1", 2: "tq2"}
DEV = "cuda"


def fast_algos(K, group, scale_dtype=np.float16, fmt="tq1"):
    """Kernels that must accept a shape: the tcgen05 kernel and the TQ1 decode GEMV cover group 128, K % 128 == 0,
    fp16 scales; the TQ2 decode GEMV additionally needs K % 512 == 0."""
    ok = group == 128 and K % 128 == 0 and scale_dtype == np.float16
    return ["generic", "auto"] + (["prefill"] if ok else []) + (["decode"] if ok and (fmt == "tq1" or K % 512 == 0) else [])


@pytest.fixture(scope="module")
def kb():
    from deepseekternarized_b200.kernels import ternary_b200

    assert ternary_b200.ext() is not None, "CUDA library not loaded: no fallback exists"
    return ternary_b200


# ------------------------------------------------------------------------------------------ format
@pytest.mark.parametrize("fmt", ["tq2", "tq1"])
@pytest.mark.parametrize("K", [1, 4, 5, 7, 128, 131, 640])
def test_pack_unpack_bit_exact(golden, fmt, K):
    from deepseekternarized_b200.ternary import pack as P

    g = golden("format")
    t, p = g[f"trits_{fmt}_{K}"], g[f"packed_{fmt}_{K}"]
    got = P.pack(torch.from_numpy(t).to(DEV), fmt)
    assert got.dtype == torch.uint8 and tuple(got.shape) == (9, P.packed_cols(fmt, K))
    assert np.array_equal(got.cpu().numpy(), p)
    assert np.array_equal(P.unpack(torch.from_numpy(p).to(DEV), fmt, K).cpu().numpy(), t)


def test_tq1_every_pattern_and_every_byte(golden):
    from deepseekternarized_b200.ternary import pack as P

    g = golden("format")
    p = P.pack(torch.from_numpy(g["tq1_patterns"]).to(DEV), "tq1")
    assert np.array_equal(p.cpu().numpy(), g["tq1_patterns_packed"])
    assert p.unique().numel() == 243 and int(p.max()) < 243
    assert np.array_equal(P.unpack(p, "tq1", 5).cpu().numpy(), g["tq1_patterns"])
    assert np.array_equal(P.tq1_lut().cpu().numpy(), g["tq1_lut"])
    allb = torch.arange(256, dtype=torch.uint8, device=DEV).view(256, 1)
    assert np.array_equal(P.unpack(allb, "tq1", 5).cpu().numpy(), g["unpack_all_bytes_tq1"])
    assert np.array_equal(P.unpack(allb, "tq2", 4).cpu().numpy(), g["unpack_all_bytes_tq2"])


@pytest.mark.parametrize("fmt,N,K", [("tq1", 4096, 4096), ("tq2", 2048, 4096), ("tq1", 333, 4097), ("tq2", 0, 64)])
def test_pack_roundtrip_large_and_empty(fmt, N, K):
    from deepseekternarized_b200.ternary import pack as P

    t = O.synth_trits(np.random.default_rng(N + K), (N, K))
    p = P.pack(torch.from_numpy(t).to(DEV), fmt)
    assert np.array_equal(p.cpu().numpy(), O.pack(t, fmt))
    assert np.array_equal(P.unpack(p, fmt, K).cpu().numpy(), t)


@pytest.mark.parametrize("fmt", ["tq1", "tq2"])
@pytest.mark.parametrize("E,N,K", [(1, 128, 256), (3, 70, 4160), (2, 300, 4096), (1, 5, 7), (4, 2048, 2048)])
def test_tiled_layout_roundtrip_bit_exact(kb, fmt, E, N, K):
    """canonical -> tiled -> canonical restores every byte, also for rows and K that need padding and for
    byte values the packer never writes. TQ1 bytes >= 243 (five zero trits by definition) are re-grouped as
    trits and therefore come back as the canonical byte of five zero trits, 121."""
    rng = np.random.default_rng(E * N + K)
    Kp = O.packed_cols(fmt, K)
    p = rng.integers(0, 256, (E, N, Kp), dtype=np.uint8)
    tw = kb.tile_weights(torch.from_numpy(p).to(DEV), fmt, K)
    assert tw.data.numel() == E * -(-N // 128) * -(-K // (256 if fmt == "tq2" else 320)) * 8192
    expect = np.where(p >= 243, 121, p).astype(np.uint8) if fmt == "tq1" else p
    assert np.array_equal(tw.untile().cpu().numpy(), expect)


# ------------------------------------------------------------------------------------------ linear, bf16 acts
def test_bf16_linear_against_reference_golden(golden, kb):
    from deepseekternarized_b200.ternary.ops import PackedTerm, TernaryLinear

    g = golden("linear_f32")
    for c in range(int(g["n_cases"])):
        K, group, N, M, k_terms, code = (int(v) for v in g[f"c{c}_meta"])
        fmt = FMT[code]
        x = O.from_bf16_bits(g[f"c{c}_x_bits"])
        terms = [(g[f"c{c}_packed{i}"], g[f"c{c}_scale{i}"]) for i in range(k_terms)]
        for algo in fast_algos(K, group, fmt=fmt):
            lin = TernaryLinear([PackedTerm(torch.from_numpy(p), torch.from_numpy(s)) for p, s in terms], K, fmt, group,
                                act="bf16", backend="b200", algo=algo)
            xt = bf16_tensor(x, DEV).view(-1, K)
            y = lin(xt.view(1, -1, K), out_dtype=torch.float32)
            assert tuple(y.shape) == (1, M, N)
            y = y.view(M, N).cpu().numpy()
            np.testing.assert_allclose(y, g[f"c{c}_y_f32"], rtol=1e-4, atol=1e-3, err_msg=f"case {c} {algo}")
            check_gemm(y, x, terms, K, group, fmt)
            ybf = lin(xt)  # default bf16 output: at most the last bit may differ from the reference's rounding
            ref_bf = O.from_bf16_bits(g[f"c{c}_y_bf16_bits"])
            assert O.rel_fro(bf16_numpy(ybf), ref_bf) < 2e-3
            deq = lin.dequantized().cpu().numpy()
            assert np.allclose(deq, O.dequantized(terms, K, group, fmt), rtol=1e-6, atol=0)


@pytest.mark.parametrize("case", range(5))
def test_baseline_shapes_against_oracle_and_golden(golden, kb, case):
    """BASELINE configs 0 and 1 (single TQ2 / TQ1 linears, K = 4096): seeded inputs rebuilt here, the
    reference output known through its strided sample in the fixture."""
    g = golden("baseline_shapes")
    code, N, K, M = (int(v) for v in g[f"c{case}_meta"])
    fmt = FMT[code]
    rng = np.random.default_rng(6000 + case)
    t = O.synth_trits(rng, (N, K))
    s = O.synth_scales(rng, (N, K // 128))
    x = O.synth_acts(rng, (M, K))
    p = O.pack(t, fmt)
    for algo in fast_algos(K, 128, fmt=fmt):
        y = kb.ternary_gemm_bf16(bf16_tensor(x, DEV), [torch.from_numpy(p).to(DEV)], [torch.from_numpy(s).to(DEV)], K, 128,
                                 fmt, algo=algo).cpu().numpy()
        np.testing.assert_allclose(y.reshape(-1)[::61], g[f"c{case}_sample"], rtol=1e-4, atol=1e-3)
        check_gemm(y, x, [(p, s)], K, 128, fmt)


@pytest.mark.parametrize("fmt", ["tq1", "tq2"])
@pytest.mark.parametrize("M", [1, 4, 8, 32])
@pytest.mark.parametrize("N", [2048, 11008])
def test_config1_decode_sweep_tq1_equals_tq2_on_same_trits(kb, fmt, M, N):
    K = 4096
    rng = np.random.default_rng(N + M)
    t = O.synth_trits(rng, (N, K))
    s = O.synth_scales(rng, (N, K // 128))
    x = O.synth_acts(rng, (M, K))
    xt = bf16_tensor(x, DEV)
    st = torch.from_numpy(s).to(DEV)
    y = {}
    for f in ("tq1", "tq2"):
        y[f] = kb.ternary_gemm_bf16(xt, [torch.from_numpy(O.pack(t, f)).to(DEV)], [st], K, 128, f).cpu().numpy()
    check_gemm(y[fmt], x, [(O.pack(t, fmt), s)], K, 128, fmt)
    # same trits through two kernels (TQ2 decode: 15-bit integer activations; the others: fp16): both far inside the tolerance
    assert O.rel_fro(y["tq1"], y["tq2"]) < 2e-4


@pytest.mark.parametrize("fmt", ["tq1", "tq2"])
@pytest.mark.parametrize("M", [1, 8, 64])
def test_config3_stacked_k2_decode(kb, fmt, M):
    for (N, K) in [(2048, 4096), (4096, 2048)]:
        rng = np.random.default_rng(M + N)
        terms = make_terms(rng, N, K, 128, fmt, k_terms=2)
        x = O.synth_acts(rng, (M, K))
        for algo in fast_algos(K, 128, fmt=fmt):
            y = kb.ternary_gemm_bf16(bf16_tensor(x, DEV), [torch.from_numpy(p).to(DEV) for p, _ in terms],
                                     [torch.from_numpy(s).to(DEV) for _, s in terms], K, 128, fmt, algo=algo).cpu().numpy()
            check_gemm(y, x, terms, K, 128, fmt)
            want = O.ternary_linear(x, terms, K, 128, fmt, out_bf16=False)
            np.testing.assert_allclose(y, want, rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize("fmt,K", [("tq1", 384), ("tq2", 512)])
def test_accumulate_row_scale_and_output_types(kb, fmt, K):
    rng = np.random.default_rng(5)
    N, M = 96, 5
    terms = make_terms(rng, N, K, 128, fmt, 1)
    x = O.synth_acts(rng, (M, K))
    rs = rng.random(M).astype(np.float32) + 0.5
    p, s = [torch.from_numpy(terms[0][0]).to(DEV)], [torch.from_numpy(terms[0][1]).to(DEV)]
    base = O.gemm_f32(x, terms[0][0], terms[0][1].astype(np.float32), K, 128, fmt)
    for algo in fast_algos(K, 128, fmt=fmt):
        out = torch.full((M, N), 2.0, device=DEV)
        kb.ternary_gemm_bf16(bf16_tensor(x, DEV), p, s, K, 128, fmt, row_scale=torch.from_numpy(rs).to(DEV), out=out,
                             accumulate=True, algo=algo)
        np.testing.assert_allclose(out.cpu().numpy(), 2.0 + base * rs[:, None], rtol=1e-4, atol=1e-3)
        for dt in (torch.bfloat16, torch.float16):
            y = kb.ternary_gemm_bf16(bf16_tensor(x, DEV), p, s, K, 128, fmt, out_dtype=dt, algo=algo)
            assert y.dtype == dt and O.rel_fro(y.float().cpu().numpy(), base) < 4e-3


# ------------------------------------------------------------------------------------------ int8 contract
def test_int8_contract_against_reference_golden(golden, kb):
    from deepseekternarized_b200.ternary.ops import quant_act_int8

    g = golden("linear_i8")
    for c in range(int(g["n_cases"])):
        K, group, N, M, code = (int(v) for v in g[f"c{c}_meta"])
        fmt = FMT[code]
        q, xs = quant_act_int8(torch.from_numpy(g[f"c{c}_x_f32"]).to(DEV))
        assert np.array_equal(q.cpu().numpy(), g[f"c{c}_q"]) and np.array_equal(xs.cpu().numpy(), g[f"c{c}_xs"])
        got = kb.ternary_gemm(q, xs, torch.from_numpy(g[f"c{c}_packed"]).to(DEV), torch.from_numpy(g[f"c{c}_scale_f32"]).to(DEV),
                              K, group, fmt, backend="cuda")
        np.testing.assert_allclose(got.cpu().numpy(), g[f"c{c}_y_ref"], rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize("fmt", ["tq1", "tq2"])
def test_int8_contract_on_the_tensor_core_path(kb, fmt):
    """int8 activations with fp16 scales and tiled weights run on the tcgen05 kernel (int8 values and scale * trit are
    exact in fp16, products exact in fp32): same contract, the reference's own tolerance (tests/test_ternary_cuda.py:80)."""
    E, N, K, group = 4, 384, 1024, 128
    rng = np.random.default_rng(31)
    terms = make_terms(rng, N, K, group, fmt, 1, lead=(E,))
    counts = np.array([300, 0, 40, 7])
    offsets = np.concatenate([[0], counts.cumsum()]).astype(np.int64)
    q, xs = O.quant_act_int8(rng.standard_normal((int(offsets[-1]), K)).astype(np.float32))
    want = O.grouped_gemm_i8(q, xs, offsets, terms[0][0], terms[0][1].astype(np.float32), K, group, fmt)
    tiled = kb.tile_weights(torch.from_numpy(terms[0][0]).to(DEV), fmt, K)
    for algo in ("auto", "prefill"):
        got = kb.grouped_ternary_gemm(torch.from_numpy(q).to(DEV), torch.from_numpy(xs).to(DEV), offsets, tiled,
                                      torch.from_numpy(terms[0][1]).to(DEV), K, group, fmt, algo=algo)
        np.testing.assert_allclose(got.cpu().numpy(), want, rtol=1e-4, atol=1e-3)
        assert O.rel_fro(got.cpu().numpy(), want) < 1e-5


@pytest.mark.parametrize("fmt", ["tq1", "tq2"])
def test_grouped_and_routing_sort_against_reference_golden(golden, kb, fmt):
    g = golden("grouped")
    ids = torch.from_numpy(g[f"{fmt}_ids"]).to(DEV)
    order, offsets = kb.sort_by_expert(ids, 6)
    assert np.array_equal(order.cpu().numpy(), g[f"{fmt}_order"]) and np.array_equal(offsets.cpu().numpy(), g[f"{fmt}_offsets"])
    rows = (order // 2).cpu()
    q, xs = torch.from_numpy(g[f"{fmt}_q"])[rows].to(DEV), torch.from_numpy(g[f"{fmt}_xs"])[rows].to(DEV)
    packed, scale = torch.from_numpy(g[f"{fmt}_packed"]).to(DEV), torch.from_numpy(g[f"{fmt}_scale_f32"]).to(DEV)
    for offs in (offsets, offsets.cpu(), offsets.cpu().tolist()):
        out = kb.grouped_ternary_gemm(q, xs, offs, packed, scale, 192, 64, fmt)
        np.testing.assert_allclose(out.cpu().numpy(), g[f"{fmt}_out"], rtol=1e-5, atol=1e-4)
    with pytest.raises(ValueError, match="offsets"):
        kb.grouped_ternary_gemm(q, xs, [0, 9], packed, scale, 192, 64, fmt)
    with pytest.raises(ValueError, match="offsets"):
        kb.grouped_ternary_gemm(q, xs, torch.tensor([0, 5, 4, 9, 12, 15, 18], device=DEV), packed, scale, 192, 64, fmt)


@pytest.mark.parametrize("fmt", ["tq1", "tq2"])
@pytest.mark.parametrize("T", [1, 3, 37])
def test_reference_cuda_parity_shapes(kb, fmt, T):
    """The shapes of the reference's own (never run) CUDA test, tests/test_ternary_cuda.py:69-87:
    N not a multiple of any tile, K not a multiple of the group, one empty expert."""
    E, N, K, group = 5, 70, 4160, 128
    rng = np.random.default_rng(7 + T)
    t = O.synth_trits(rng, (E, N, K), p_zero=1 / 3)
    packed = np.stack([O.pack(t[e], fmt) for e in range(E)])
    scales = (rng.random((E, N, -(-K // group))).astype(np.float16).astype(np.float32) + np.float32(0.01))
    counts = np.array([T, 0, 2 * T, 1, T])
    offsets = np.concatenate([[0], counts.cumsum()]).astype(np.int64)
    R = int(offsets[-1])
    q, xs = O.quant_act_int8(rng.standard_normal((R, K)).astype(np.float32))
    want = O.grouped_gemm_i8(q, xs, offsets, packed, scales, K, group, fmt)
    got = kb.grouped_ternary_gemm(torch.from_numpy(q).to(DEV), torch.from_numpy(xs).to(DEV), offsets, torch.from_numpy(packed).to(DEV),
                                  torch.from_numpy(scales).to(DEV), K, group, fmt, backend="cuda")
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=1e-4, atol=1e-3)
    # the same shapes on the bf16 path, fp16 scales
    x = O.synth_acts(rng, (R, K))
    s16 = scales.astype(np.float16)
    want = O.grouped_gemm_f32(x, offsets, packed, s16.astype(np.float32), K, group, fmt)
    got = kb.grouped_ternary_gemm_bf16(bf16_tensor(x, DEV), offsets, [torch.from_numpy(packed).to(DEV)],
                                       [torch.from_numpy(s16).to(DEV)], K, group, fmt)
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=1e-4, atol=2e-3)


@pytest.mark.parametrize("fmt", ["tq2", "tq1"])
@pytest.mark.parametrize("algo", ["decode", "prefill", "auto"])
def test_grouped_decode_sizes_with_empty_and_ragged_experts(kb, algo, fmt):
    """Grouped GEMV as a MoE decode step sees it: few rows per expert, some experts empty, one above 16 rows."""
    E, N, K = 7, 200, 1024
    rng = np.random.default_rng(21)
    terms = make_terms(rng, N, K, 128, fmt, 2, lead=(E,))
    counts = np.array([1, 0, 8, 3, 19, 0, 2])
    offsets = np.concatenate([[0], counts.cumsum()]).astype(np.int64)
    x = O.synth_acts(rng, (int(offsets[-1]), K))
    tiled = [kb.tile_weights(torch.from_numpy(p).to(DEV), fmt, K) for p, _ in terms]
    y = kb.grouped_ternary_gemm_bf16(bf16_tensor(x, DEV), offsets, tiled, [torch.from_numpy(s).to(DEV) for _, s in terms], K, 128, fmt,
                                     algo=algo).cpu().numpy()
    for e in range(E):
        a, b = int(offsets[e]), int(offsets[e + 1])
        if b > a:
            check_gemm(y[a:b], x[a:b], [(p[e], s[e]) for p, s in terms], K, 128, fmt)
            want = O.ternary_linear(x[a:b], [(p[e], s[e]) for p, s in terms], K, 128, fmt, out_bf16=False)
            np.testing.assert_allclose(y[a:b], want, rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize("N,K,terms_k", [(1024, 1024, 1), (384, 512, 2)])
def test_grouped_decode_many_row_ctas(kb, N, K, terms_k):
    """Five or more rows per expert with at least one 256-row item per SM: the decode GEMV runs as one CTA per SM whose
    eight consumer warps own two MMA tiles each (8 or 16 staged rows per pass). Ragged row counts around the pass
    sizes, empty experts, an odd number of 128-row tiles (the last item has one tile only)."""
    E = 160
    rng = np.random.default_rng(N + K)
    terms = make_terms(rng, N, K, 128, "tq2", terms_k, lead=(E,))
    for top, algo in ((8, "decode"), (16, "decode"), (21, "decode"), (30, "auto")):  # 30 rows: two passes, chosen by AUTO
        counts = rng.integers(max(1, top - 7), top + 1, E)
        counts[[3, 77]] = 0
        counts[5] = top
        offsets = np.concatenate([[0], counts.cumsum()]).astype(np.int64)
        x = O.synth_acts(rng, (int(offsets[-1]), K))
        tiled = [kb.tile_weights(torch.from_numpy(p).to(DEV), "tq2", K) for p, _ in terms]
        scales = [torch.from_numpy(s).to(DEV) for _, s in terms]
        y = kb.grouped_ternary_gemm_bf16(bf16_tensor(x, DEV), offsets, tiled, scales, K, 128, "tq2", algo=algo)
        torch.cuda.synchronize()
        assert kb.ext().dst_check_device_status(None) == 0
        y = y.cpu().numpy()
        assert np.isfinite(y).all()
        for e in (0, 4, 5, 76, 78, E - 1):
            a, b = int(offsets[e]), int(offsets[e + 1])
            check_gemm(y[a:b], x[a:b], [(p[e], s[e]) for p, s in terms], K, 128, "tq2")
        want = O.grouped_gemm_f32(O.bf16_round(x), offsets, terms[0][0], terms[0][1].astype(np.float32), K, 128, "tq2")
        for p_, s_ in terms[1:]:
            want = want + O.grouped_gemm_f32(O.bf16_round(x), offsets, p_, s_.astype(np.float32), K, 128, "tq2")
        np.testing.assert_allclose(y, want, rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize("top", [1, 4, 8, 16])
def test_decode_without_a_workspace_quantises_inside_the_kernel(kb, top, monkeypatch):
    """A C-ABI caller may pass no workspace to the decode GEMV: the consumer warps then quantise each expert's token rows
    themselves (stage_tokens inside decode_kernel, all CTA shapes) instead of reading what decode_quant_kernel wrote:
    same integers, so the same outputs bit for bit."""
    E, N, K = 160, 512, 512
    rng = np.random.default_rng(top)
    terms = make_terms(rng, N, K, 128, "tq2", 1, lead=(E,))
    counts = rng.integers(max(0, top - 3), top + 1, E)
    offsets = np.concatenate([[0], counts.cumsum()]).astype(np.int64)
    x = bf16_tensor(O.synth_acts(rng, (int(offsets[-1]), K)), DEV)
    tiled = [kb.tile_weights(torch.from_numpy(terms[0][0]).to(DEV), "tq2", K)]
    sc = [torch.from_numpy(terms[0][1]).to(DEV)]
    with_ws = kb.grouped_ternary_gemm_bf16(x, offsets, tiled, sc, K, 128, "tq2", algo="decode")
    lib = kb.ext()
    real = lib.dst_gemm_workspace_bytes
    monkeypatch.setattr(lib, "dst_gemm_workspace_bytes", lambda *a: 0)
    try:
        without = kb.grouped_ternary_gemm_bf16(x, offsets, tiled, sc, K, 128, "tq2", algo="decode")
    finally:
        monkeypatch.setattr(lib, "dst_gemm_workspace_bytes", real)
    torch.cuda.synchronize()
    assert lib.dst_check_device_status(None) == 0
    assert torch.equal(with_ws, without)


@pytest.mark.parametrize("fmt", ["tq1", "tq2"])
def test_prefill_many_tiles_per_cta(kb, fmt):
    """More tiles than SMs, so every persistent CTA of the tcgen05 kernel walks several tiles (ring phases, the
    packed-slab ring and the accumulator hand-over all wrap across tile borders); ragged rows per expert around the
    one-MMA (256 rows) and the tile (320 rows) limits, one empty expert. Checked on sampled experts against the
    oracle, all rows for finiteness."""
    E, N, K = 15, 2048, 1024
    rng = np.random.default_rng(77)
    terms = make_terms(rng, N, K, 128, fmt, 1, lead=(E,))
    counts = np.array([257, 300, 0, 129, 256, 512, 31, 270, 255, 1, 513, 240, 320, 321, 641])
    offsets = np.concatenate([[0], counts.cumsum()]).astype(np.int64)
    x = O.synth_acts(rng, (int(offsets[-1]), K))
    tiled = [kb.tile_weights(torch.from_numpy(terms[0][0]).to(DEV), fmt, K)]
    y = kb.grouped_ternary_gemm_bf16(bf16_tensor(x, DEV), torch.from_numpy(offsets).to(DEV), tiled, [torch.from_numpy(terms[0][1]).to(DEV)],
                                     K, 128, fmt, algo="prefill", validate_offsets=False)
    torch.cuda.synchronize()
    assert kb.ext().dst_check_device_status(None) == 0
    y = y.cpu().numpy()
    assert np.isfinite(y).all()
    for e in (0, 5, 9, 10, 12, 13, 14):
        a, b = int(offsets[e]), int(offsets[e + 1])
        check_gemm(y[a:b], x[a:b], [(terms[0][0][e], terms[0][1][e])], K, 128, fmt)


@pytest.mark.parametrize("N", [200, 196, 384])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16])
def test_prefill_sixteen_bit_outputs_equal_rounded_fp32_outputs(kb, N, out_dtype):
    """16-bit outputs of the tcgen05 kernel leave through transposed tiles and 128-bit stores when N % 8 == 0 (else one
    store per element): either way they are the fp32 outputs rounded once. Ragged experts around the tile sizes, one
    empty, columns that end inside a 128-column tile."""
    E, K = 9, 512
    rng = np.random.default_rng(N)
    terms = make_terms(rng, N, K, 128, "tq1", 1, lead=(E,))
    counts = np.array([40, 0, 257, 31, 320, 1, 96, 300, 17])
    offsets = np.concatenate([[0], counts.cumsum()]).astype(np.int64)
    x = bf16_tensor(O.synth_acts(rng, (int(offsets[-1]), K)), DEV)
    tiled = [kb.tile_weights(torch.from_numpy(terms[0][0]).to(DEV), "tq1", K)]
    sc = [torch.from_numpy(terms[0][1]).to(DEV)]
    y32 = kb.grouped_ternary_gemm_bf16(x, offsets, tiled, sc, K, 128, "tq1", algo="prefill", out_dtype=torch.float32)
    y16 = kb.grouped_ternary_gemm_bf16(x, offsets, tiled, sc, K, 128, "tq1", algo="prefill", out_dtype=out_dtype)
    torch.cuda.synchronize()
    assert kb.ext().dst_check_device_status(None) == 0
    assert torch.equal(y16, y32.to(out_dtype))


@pytest.mark.parametrize("fmt", ["tq1", "tq2"])
def test_prefill_more_experts_than_one_launch_holds(kb, fmt):
    """The tcgen05 kernel keeps per-expert tables for at most 1023 experts in shared memory; a call with more is
    split into launches over runs of experts. 1030 experts with 0..3 rows each, every row checked."""
    E, N, K = 1030, 128, 256
    rng = np.random.default_rng(5)
    terms = make_terms(rng, N, K, 128, fmt, 1, lead=(E,))
    counts = rng.integers(0, 4, E)
    offsets = np.concatenate([[0], counts.cumsum()]).astype(np.int64)
    x = O.synth_acts(rng, (int(offsets[-1]), K))
    tiled = [kb.tile_weights(torch.from_numpy(terms[0][0]).to(DEV), fmt, K)]
    y = kb.grouped_ternary_gemm_bf16(bf16_tensor(x, DEV), torch.from_numpy(offsets).to(DEV), tiled, [torch.from_numpy(terms[0][1]).to(DEV)],
                                     K, 128, fmt, algo="prefill")
    torch.cuda.synchronize()
    assert kb.ext().dst_check_device_status(None) == 0
    y = y.cpu().numpy()
    ref = O.grouped_gemm_f32(O.bf16_round(x), offsets, terms[0][0], terms[0][1].astype(np.float32), K, 128, fmt)
    assert O.rel_fro(y, ref) < 2e-3 and O.cosine(y, ref) > 0.99999


def test_native_entry_rejects_malformed_tensors(kb):
    """tests/test_kernel_security.py:19-38 of the reference, against this backend: every malformed
    argument raises RuntimeError before any launch."""
    def args():
        return dict(x=torch.ones(1, 5, dtype=torch.int8, device=DEV), x_scale=torch.ones(1, device=DEV),
                    packed=torch.ones(2, 2, dtype=torch.uint8, device=DEV), w_scale=torch.ones(2, 2, device=DEV), K=5, group=3, fmt="tq2")
    kb.ternary_gemm(**args())
    bad = [("K", 0), ("K", 2**62), ("group", 0), ("x", torch.ones(1, 4, dtype=torch.int8, device=DEV)),
           ("packed", torch.ones(2, 1, dtype=torch.uint8, device=DEV)), ("packed", torch.ones(2, 2, device=DEV)),
           ("w_scale", torch.ones(2, 1, device=DEV)), ("w_scale", torch.ones(1, 2, device=DEV)), ("x_scale", torch.ones(0, device=DEV)),
           ("packed", torch.ones(2, 2, dtype=torch.uint8))]
    for key, value in bad:
        a = args()
        a[key] = value
        with pytest.raises(RuntimeError):
            kb.ternary_gemm(**a)
    with pytest.raises(ValueError):
        kb.ternary_gemm(**{**args(), "fmt": "tq0"})


# ------------------------------------------------------------------------------------------ MoE layer
@pytest.mark.parametrize("fmt", ["tq1", "tq2"])
def test_moe_layer_against_reference_golden(golden, fmt):
    from deepseekternarized_b200.moe import B200Ops, ExpertWeights, MoELayer

    g = golden("moe_layer")
    T, hidden, inter, E, topk, group, k_terms = (int(v) for v in g[f"{fmt}_meta"])
    x = O.from_bf16_bits(g[f"{fmt}_x_bits"])
    experts = [tuple([(g[f"{fmt}_e{e}_{wn}_packed{i}"], g[f"{fmt}_e{e}_{wn}_scale{i}"]) for i in range(k_terms)]
                     for wn in ("w1", "w2", "w3")) for e in range(E)]
    logits = torch.from_numpy(x @ g[f"{fmt}_gate_w"].T).to(DEV)
    ops = B200Ops()
    w, ids = ops.route(logits, topk, 1.0)
    assert np.array_equal(ids.cpu().numpy(), g[f"{fmt}_route_indices"])
    np.testing.assert_allclose(w.cpu().numpy(), g[f"{fmt}_route_weights"], rtol=1e-5, atol=1e-7)
    ew = ExpertWeights(*stack_experts(experts, k_terms, DEV), hidden, inter, group, fmt)
    y = MoELayer(ew, topk)(bf16_tensor(x, DEV), logits)
    want = O.from_bf16_bits(g[f"{fmt}_y_bits"])
    y64 = O.moe_layer_f64(x, g[f"{fmt}_route_weights"], g[f"{fmt}_route_indices"], experts, hidden, inter, group, fmt)
    check_layer(bf16_numpy(y), want, y64)


@pytest.mark.parametrize("fmt", ["tq1", "tq2"])
def test_moe_layer_standard_flavour_against_reference_golden(golden, fmt):
    """The OLMoE-style layer of boilerplate/engine/standard.py:154-176 on the GPU against the reference's output."""
    from deepseekternarized_b200.moe import B200Ops, ExpertWeights, MoELayer

    g = golden("moe_layer_standard")
    T, hidden, inter, E, topk, group, k_terms, renorm = (int(v) for v in g[f"{fmt}_meta"])
    x = O.from_bf16_bits(g[f"{fmt}_x_bits"])
    experts = [tuple([(g[f"{fmt}_e{e}_{wn}_packed{i}"], g[f"{fmt}_e{e}_{wn}_scale{i}"]) for i in range(k_terms)]
                     for wn in ("w1", "w2", "w3")) for e in range(E)]
    logits = torch.from_numpy(g[f"{fmt}_logits"]).to(DEV)
    _, w_ref, idx_ref = O.moe_layer_standard(x, g[f"{fmt}_logits"], experts, topk, hidden, inter, group, fmt, bool(renorm))
    w, ids = B200Ops().route(logits, topk, 1.0, renorm=bool(renorm))
    assert np.array_equal(ids.cpu().numpy(), g[f"{fmt}_route_indices"])
    np.testing.assert_allclose(w.cpu().numpy(), w_ref, rtol=1e-5, atol=1e-7)
    ew = ExpertWeights(*stack_experts(experts, k_terms, DEV), hidden, inter, group, fmt)
    y = MoELayer(ew, topk, flavour="standard", norm_topk_prob=bool(renorm))(bf16_tensor(x, DEV), logits)
    want = O.from_bf16_bits(g[f"{fmt}_y_bits"])
    check_layer(bf16_numpy(y), want, O.moe_layer_f64(x, w_ref, idx_ref, experts, hidden, inter, group, fmt))
    # larger case (the tcgen05 kernel and the fused fp16 rows): against the oracle
    T2, E2 = 700, 4
    rng = np.random.default_rng(17)
    experts2 = make_experts(rng, E2, hidden, inter, group, fmt, k_terms)
    x2 = O.synth_acts(rng, (T2, hidden))
    lg2 = rng.standard_normal((T2, E2)).astype(np.float32)
    want2, w2, idx2 = O.moe_layer_standard(x2, lg2, experts2, 2, hidden, inter, group, fmt, bool(renorm))
    ew2 = ExpertWeights(*stack_experts(experts2, k_terms, DEV), hidden, inter, group, fmt).prepare()
    y2 = MoELayer(ew2, 2, flavour="standard", norm_topk_prob=bool(renorm))(bf16_tensor(x2, DEV), torch.from_numpy(lg2).to(DEV))
    check_layer(bf16_numpy(y2), want2, O.moe_layer_f64(x2, w2, idx2, experts2, hidden, inter, group, fmt))


@pytest.mark.parametrize("fmt,k_terms", [("tq1", 1), ("tq2", 2)])
def test_moe_layer_steps_against_oracle(fmt, k_terms):
    """A mid-sized layer (T=300, 16 experts, top-6): every step against the oracle."""
    from deepseekternarized_b200.moe import B200Ops, ExpertWeights, MoELayer

    T, hidden, inter, E, topk, group = 300, 512, 256, 16, 6, 128
    rng = np.random.default_rng(11)
    experts = make_experts(rng, E, hidden, inter, group, fmt, k_terms)
    x = O.synth_acts(rng, (T, hidden))
    logits = rng.standard_normal((T, E)).astype(np.float32)
    logits[:, 3] = -40.0  # an empty expert
    ops = B200Ops()
    w, ids = ops.route(torch.from_numpy(logits).to(DEV), topk, 1.0)
    w_ref, idx_ref = O.route_from_logits(logits, topk)
    assert np.array_equal(ids.cpu().numpy(), idx_ref)
    np.testing.assert_allclose(w.cpu().numpy(), w_ref, rtol=1e-5, atol=1e-7)
    order, offsets = ops.sort(ids, E)
    order_ref, offsets_ref = O.sort_by_expert(idx_ref.reshape(-1), E)
    assert np.array_equal(order.cpu().numpy(), order_ref) and np.array_equal(offsets.cpu().numpy(), offsets_ref)
    xs = ops.gather(bf16_tensor(x, DEV), order, topk)
    assert np.array_equal(bf16_numpy(xs), x[order_ref // topk])
    ew = ExpertWeights(*stack_experts(experts, k_terms, DEV), hidden, inter, group, fmt)
    y = MoELayer(ew, topk)(bf16_tensor(x, DEV), torch.from_numpy(logits).to(DEV))
    want = O.moe_layer(x, w_ref, idx_ref, experts, hidden, inter, group, fmt)
    check_layer(bf16_numpy(y), want, O.moe_layer_f64(x, w_ref, idx_ref, experts, hidden, inter, group, fmt))
    y2 = MoELayer(ew.prepare(), topk)(bf16_tensor(x, DEV), torch.from_numpy(logits).to(DEV))  # weights tiled once
    assert torch.equal(y, y2)


def test_host_pipeline_equals_direct_calls():
    """Batches fed from pinned host buffers through the three-stream pipeline (ragged sizes, more batches than
    slots, distinct output buffers) equal the layer called on device-resident copies of the same batches."""
    from deepseekternarized_b200.moe import ExpertWeights, HostPipeline, MoELayer

    hidden, inter, E, topk, group = 512, 256, 16, 6, 128
    rng = np.random.default_rng(23)
    experts = make_experts(rng, E, hidden, inter, group, "tq1", 1)
    layer = MoELayer(ExpertWeights(*stack_experts(experts, 1, DEV), hidden, inter, group, "tq1").prepare(), topk)
    sizes = [300, 1, 257, 300, 64, 129, 300]
    pipe = HostPipeline(layer, max(sizes), hidden, E, DEV)
    xs = [bf16_tensor(O.synth_acts(rng, (t, hidden)), "cpu").pin_memory() for t in sizes]
    lgs = [torch.from_numpy(rng.standard_normal((t, E)).astype(np.float32)).pin_memory() for t in sizes]
    ys = [torch.empty(t, hidden, dtype=torch.bfloat16).pin_memory() for t in sizes]
    for x, lg, y in zip(xs, lgs, ys):
        pipe.submit(x, lg, y)
    pipe.drain()
    for x, lg, y in zip(xs, lgs, ys):
        assert torch.equal(y, layer(x.to(DEV), lg.to(DEV)).cpu())
    with pytest.raises(ValueError):
        pipe.submit(torch.empty(301, hidden, dtype=torch.bfloat16), torch.empty(301, E), torch.empty(301, hidden, dtype=torch.bfloat16))


def test_sort_large_and_bad_ids(kb):
    rng = np.random.default_rng(3)
    ids = rng.integers(0, 384, 98304).astype(np.int64)
    order, offsets = kb.sort_by_expert(torch.from_numpy(ids).to(DEV), 384)
    o_ref, f_ref = O.sort_by_expert(ids, 384)
    assert np.array_equal(order.cpu().numpy(), o_ref) and np.array_equal(offsets.cpu().numpy(), f_ref)
    order, offsets = kb.sort_by_expert(torch.from_numpy(ids.astype(np.int32)).to(DEV), 384)
    assert np.array_equal(order.cpu().numpy(), o_ref)
    order, offsets = kb.sort_by_expert(torch.zeros(0, dtype=torch.int64, device=DEV), 4)
    assert order.numel() == 0 and offsets.cpu().tolist() == [0] * 5


@pytest.mark.parametrize("fmt", ["tq1", "tq2"])
def test_table_row_lookup_against_reference_golden(golden, fmt):
    """Ternary lookup-table rows (boilerplate/engine/model.py:458-464) on the GPU: bit-exact with the reference."""
    from deepseekternarized_b200.ternary.ops import LookupTable, PackedTerm, gather_dequant_rows

    g = golden("table_rows")
    V, K, group, k_terms = (int(v) for v in g[f"{fmt}_meta"])
    terms = [PackedTerm(torch.from_numpy(g[f"{fmt}_packed{i}"]).to(DEV), torch.from_numpy(g[f"{fmt}_scale{i}"]).to(DEV)) for i in range(k_terms)]
    ids = torch.from_numpy(g[f"{fmt}_ids"]).to(DEV)
    vals = gather_dequant_rows(terms, ids, K, fmt, group)
    assert tuple(vals.shape) == (*ids.shape, K) and vals.dtype == torch.bfloat16
    assert np.array_equal(O.bf16_bits(bf16_numpy(vals)).reshape(-1, K), g[f"{fmt}_vals_bits"])
    with pytest.raises(IndexError):
        gather_dequant_rows(terms, torch.tensor([0, V], device=DEV), K, fmt, group)
    # larger tables against the oracle: a long row, the engram tables' row (head_dim 256, group 128, two stacked terms:
    # boilerplate/configs/policy/experts_engram_k2.yaml), a row whose last TQ1 byte is partly padding, and a row
    # width the 8-trit kernel does not take
    rng = np.random.default_rng(9)
    for V2, K2, group2, k2 in ((3000, 1024, 128, 2), (5000, 256, 128, 2), (700, 136, 8, 1), (700, 100, 128, 3)):
        big = make_terms(rng, V2, K2, group2, fmt, k2)
        ids2 = rng.integers(0, V2, 4096)
        ids2[:2] = (0, V2 - 1)
        got = gather_dequant_rows([PackedTerm(torch.from_numpy(p).to(DEV), torch.from_numpy(s).to(DEV)) for p, s in big],
                                  torch.from_numpy(ids2).to(DEV), K2, fmt, group2)
        assert np.array_equal(bf16_numpy(got), O.gather_dequant_rows(ids2, big, K2, group2, fmt))
        # the same table as one record per row
        table = LookupTable([PackedTerm(torch.from_numpy(p).to(DEV), torch.from_numpy(s).to(DEV)) for p, s in big], K2, fmt, group2)
        assert table.record % 16 == 0 and torch.equal(table.rows(torch.from_numpy(ids2).to(DEV)), got)
        with pytest.raises(IndexError):
            table.rows(torch.tensor([-1], device=DEV))
        assert not table.rows(torch.tensor([V2], device=DEV), check=False).any()


def test_expert_parallel_peer_transport_single_rank():
    """The peer-memory dispatch / combine kernels and the placement arithmetic in a one-rank job (every routed row is
    local): bit-identical to the single-device layer, also through the all-to-all transport. Runs in a child
    process because it initialises torch.distributed; several ranks are run by hand (see tests/ep_peer_check.py)."""
    import subprocess
    import sys
    from pathlib import Path

    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29541", RANK="0", WORLD_SIZE="1", LOCAL_RANK="0")
    res = subprocess.run([sys.executable, str(Path(__file__).with_name("ep_peer_check.py"))], env=env, capture_output=True, text=True,
                         timeout=600)
    assert res.returncode == 0 and "EP_PEER_CHECK PASS" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]


def test_scatter_gemm_stores_nothing_outside_its_buffers(kb):
    """The scattering form of the tcgen05 grouped GEMM: rows go where their targets say (a permutation here), and a
    negative target, a buffer index beyond the table or a row beyond the buffer is dropped, not stored."""
    import ctypes

    from deepseekternarized_b200.moe import B200Ops

    E, N, K, rows_per = 3, 256, 512, 70
    rng = np.random.default_rng(12)
    terms = make_terms(rng, N, K, 128, "tq1", 1, lead=(E,))
    T = E * rows_per
    tiled = [kb.tile_weights(torch.from_numpy(terms[0][0]).to(DEV), "tq1", K)]
    sc = [torch.from_numpy(terms[0][1]).to(DEV)]
    xh = torch.from_numpy((O.synth_acts(rng, (T, K)) * 30).astype(np.float16)).to(DEV)
    x = kb.NormRows(xh, torch.full((T,), 0.5, device=DEV))
    offs = torch.arange(E + 1, device=DEV, dtype=torch.int64) * rows_per
    ops = B200Ops()
    plain = ops.gemm(x, offs, tiled, sc, K, 128, "tq1")
    target = torch.randperm(T, device=DEV)
    dropped = {3: -1, 5: (1 << 48) | 5, 7: T + 5, 100: (15 << 48), 209: -7}
    kept = torch.ones(T, dtype=torch.bool, device=DEV)
    for r, v in dropped.items():
        target[r] = v
        kept[r] = False
    out = torch.full((T + 8, N), -3.0, dtype=torch.bfloat16, device=DEV)  # eight rows of margin behind the buffer
    peer = (ctypes.c_void_p * 1)(out.data_ptr())
    ops.gemm_scatter(x, offs, tiled, sc, K, 128, "tq1", peer, 1, T, target)
    torch.cuda.synchronize()
    assert kb.ext().dst_check_device_status(None) == 0
    assert torch.equal(out[target[kept]], plain[kept])
    written = torch.zeros(T + 8, dtype=torch.bool, device=DEV)
    written[target[kept]] = True
    assert (out[~written] == -3.0).all()


@pytest.mark.parametrize("W", [4, 8])
def test_ep_peer_kernels_with_emulated_ranks(W):
    """The peer-memory dispatch / combine entries for 4 and 8 ranks on ONE GPU: every "rank" has its own buffers on
    this device and the ranks' steps run one after the other (none of the kernels waits on another rank), with the
    same placement arithmetic, pointer tables and grouped GEMMs as ExpertParallelMoE. Both ways back (the owners' rows
    pulled; the second GEMM's epilogue scattering them to the tokens' ranks) = the single-device layer."""
    import ctypes

    from deepseekternarized_b200 import _lib
    from deepseekternarized_b200.kernels import ternary_b200 as kb
    from deepseekternarized_b200.moe import B200Ops, ExpertWeights, MoELayer, ep_placement

    E, hidden, inter, topk, group, fmt, tl = 16, 256, 128, 4, 128, "tq1", 96
    El, T = E // W, 96 * W
    rng = np.random.default_rng(40 + W)
    experts = make_experts(rng, E, hidden, inter, group, fmt, 1)
    x = bf16_tensor(O.synth_acts(rng, (T, hidden)), DEV)
    logits = rng.standard_normal((T, E)).astype(np.float32)
    logits[:, 5] = -40.0
    logits = torch.from_numpy(logits).to(DEV)
    ops, lib = B200Ops(), kb.ext()
    cap = tl * topk * W
    bufs = [dict(rows=torch.empty(cap, hidden, dtype=torch.float16, device=DEV), fac=torch.empty(cap, device=DEV),
                 wts=torch.empty(cap, device=DEV), down=torch.empty(cap, hidden, dtype=torch.bfloat16, device=DEV),
                 origin=torch.full((cap,), -1, dtype=torch.int64, device=DEV),
                 back=torch.full((tl * topk, hidden), float("nan"), dtype=torch.bfloat16, device=DEV)) for _ in range(W)]
    ptrs = {k: (ctypes.c_void_p * W)(*[b[k].data_ptr() for b in bufs]) for k in ("rows", "fac", "wts", "down", "origin", "back")}
    stream = kb._stream(x)
    routed = []
    for r in range(W):  # route and sort per rank; all-gather of the counts = stack
        w, ids = ops.route(logits[r * tl:(r + 1) * tl], topk, 1.0)
        order, offsets = ops.sort(ids, E)
        routed.append((w.reshape(-1).contiguous(), ids, order, offsets))
    counts_all = torch.stack([o[3].diff() for o in routed])
    place = [ep_placement(counts_all, r, El) for r in range(W)]
    dests = [torch.empty(tl * topk, dtype=torch.int64, device=DEV) for _ in range(W)]
    for r in range(W):  # push
        w, ids, order, offsets = routed[r]
        xr = x[r * tl:(r + 1) * tl].contiguous()
        _lib.check(lib.dst_ep_push_rows(xr.data_ptr(), order.data_ptr(), offsets.data_ptr(), w.data_ptr(), place[r][0].data_ptr(),
                                        order.numel(), E, El, topk, hidden, ptrs["rows"], ptrs["fac"], ptrs["wts"], ptrs["origin"], W, r,
                                        dests[r].data_ptr(), stream))
    for r in range(W):  # experts of rank r on the rows it received
        offsets2 = place[r][1]
        R = int(offsets2[-1])
        wl = ExpertWeights(*stack_experts(experts[r * El:(r + 1) * El], 1, DEV), hidden, inter, group, fmt).prepare()
        if R:
            MoELayer(wl, topk).experts_forward(kb.NormRows(bufs[r]["rows"][:R], bufs[r]["fac"][:R]), offsets2, bufs[r]["wts"][:R], None,
                                               out=bufs[r]["down"][:R])
            # the fused way back: the second GEMM stores every output row into the slot of the rank that owns the token
            MoELayer(wl, topk).experts_forward(kb.NormRows(bufs[r]["rows"], bufs[r]["fac"]), offsets2, bufs[r]["wts"], None,
                                               n_rows_dev=offsets2[-1:], scatter=(ptrs["back"], W, tl * topk, bufs[r]["origin"]))
    ys = []
    for r in range(W):  # pull + combine
        w, ids, order, offsets = routed[r]
        inv = torch.empty(tl * topk, dtype=torch.int64, device=DEV)
        y = torch.empty(tl, hidden, dtype=torch.bfloat16, device=DEV)
        ids32 = ids.reshape(-1).to(torch.int32).contiguous()
        _lib.check(lib.dst_ep_combine_pull(ptrs["down"], order.data_ptr(), ids32.data_ptr(), offsets.data_ptr(), place[r][0].data_ptr(),
                                           tl, El, topk, hidden, inv.data_ptr(), y.data_ptr(), W, stream))
        ys.append(y)
        y2 = torch.empty(tl, hidden, dtype=torch.bfloat16, device=DEV)
        _lib.check(lib.dst_ep_combine_returned(bufs[r]["back"].data_ptr(), order.data_ptr(), dests[r].data_ptr(), ids32.data_ptr(), tl, topk,
                                               hidden, inv.data_ptr(), None, y2.data_ptr(), stream))
        assert torch.equal(y2, y)
    torch.cuda.synchronize()
    assert lib.dst_check_device_status(None) == 0
    w_all = ExpertWeights(*stack_experts(experts, 1, DEV), hidden, inter, group, fmt).prepare()
    want = torch.cat([MoELayer(w_all, topk)(x[r * tl:(r + 1) * tl].contiguous(), logits[r * tl:(r + 1) * tl].contiguous()) for r in range(W)])
    assert torch.equal(torch.cat(ys), want)


# ------------------------------------------------------------------------------------------ act = "int8" as a resident path
@pytest.mark.parametrize("fmt", ["tq1", "tq2"])
def test_int8_linear_keeps_tiled_weights_and_matches_the_reference_contract(kb, fmt, monkeypatch):
    """TernaryLinear(act="int8"), the mode every shipped policy selects (configs/policy/*.yaml of the reference): the
    weights are tiled once, a few rows go to the decode GEMV as int8 (integer group sums, as ternary_gemm_ref has them,
    boilerplate/kernels/ternary_cuda.py:52-64), many rows are quantised straight into the tcgen05 kernel's row format."""
    from deepseekternarized_b200.ternary import ops

    N, K, group = 320, 1024, 128
    rng = np.random.default_rng(77)
    terms = make_terms(rng, N, K, group, fmt, 2)
    calls = []
    real_tile = kb.tile_weights
    monkeypatch.setattr(kb, "tile_weights", lambda *a, **k: (calls.append(1), real_tile(*a, **k))[1])
    lin = ops.TernaryLinear([ops.PackedTerm(torch.from_numpy(p), torch.from_numpy(s)) for p, s in terms], K, fmt, group, act="int8",
                            decode_copy=True)
    for M in (3, 300, 3):
        x = rng.standard_normal((M, K)).astype(np.float32) * 2
        q, xs = O.quant_act_int8(x)
        want = sum(O.gemm_ref_i8(q, xs, p, s.astype(np.float32), K, group, fmt) for p, s in terms)
        got = lin(torch.from_numpy(x).to(DEV), out_dtype=torch.float32).cpu().numpy()
        np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-3)
        # decode rows: exact integer group sums. Many rows: the tcgen05 kernel merges the two stacked terms into one
        # fp16 weight (s1 t1 + s2 t2, one rounding of 2^-12 relative) before the exact products
        assert O.rel_fro(got, want) < (1e-5 if M <= 16 else 5e-4)
    assert len(calls) == 2  # one re-layout per term, at the first call only
    qh, s16 = ops.quant_act_int8(torch.from_numpy(x).to(DEV), as_f16=True)
    qi, s8 = ops.quant_act_int8(torch.from_numpy(x).to(DEV))
    assert qh.dtype == torch.float16 and torch.equal(qh.to(torch.int8), qi) and torch.equal(s16, s8)
    assert np.array_equal(qi.cpu().numpy(), q) and np.array_equal(s8.cpu().numpy(), xs)


@pytest.mark.parametrize("M", [1, 2, 4, 8, 16, 19])
def test_tq1_weights_with_a_two_bit_decode_copy(kb, M):
    """TQ1 weights that also keep their trits as tiled TQ2 on the device: few-row calls read that copy (same trits, the
    TQ2 decode kernel), many-row calls the TQ1 tiles; both inside the tolerance, and the copy equals packing the
    trits as TQ2 in the first place."""
    E, N, K = 3, 200, 1024
    rng = np.random.default_rng(M)
    t = O.synth_trits(rng, (E, N, K))
    s = O.synth_scales(rng, (E, N, K // 128))
    p1 = np.stack([O.pack(t[e], "tq1") for e in range(E)])
    p2 = np.stack([O.pack(t[e], "tq2") for e in range(E)])
    w1 = kb.tile_weights(torch.from_numpy(p1).to(DEV), "tq1", K, decode_copy=True)
    w2 = kb.tile_weights(torch.from_numpy(p2).to(DEV), "tq2", K)
    assert w1.decode is not None and torch.equal(w1.decode.data, w2.data)
    counts = np.array([M, 0, max(1, M // 2)])
    offsets = np.concatenate([[0], counts.cumsum()]).astype(np.int64)
    x = O.synth_acts(rng, (int(offsets[-1]), K))
    sd = torch.from_numpy(s).to(DEV)
    y1 = kb.grouped_ternary_gemm_bf16(bf16_tensor(x, DEV), offsets, [w1], [sd], K, 128, "tq1").cpu().numpy()
    y2 = kb.grouped_ternary_gemm_bf16(bf16_tensor(x, DEV), offsets, [w2], [sd], K, 128, "tq2", algo="decode").cpu().numpy()
    if offsets[-1] <= 16 * E:
        assert np.array_equal(y1, y2)  # the very same kernel on the very same bytes
    for e in range(E):
        a, b = int(offsets[e]), int(offsets[e + 1])
        if b > a:
            check_gemm(y1[a:b], x[a:b], [(p1[e], s[e])], K, 128, "tq1")
            np.testing.assert_allclose(y1[a:b], O.gemm_f32(x[a:b], p1[e], s[e].astype(np.float32), K, 128, "tq1"), rtol=1e-4, atol=1e-3)


def test_decode_kernel_int8_activations_are_exact_integer_sums(kb):
    """int8 activations through the decode GEMV: the group sums are exact integers (int8 tensor-core MMAs), so the result
    equals the reference-of-record up to the order of the fp32 additions over groups."""
    E, N, K, group = 5, 136, 1536, 128
    rng = np.random.default_rng(41)
    terms = make_terms(rng, N, K, group, "tq2", 1, lead=(E,))
    counts = np.array([1, 4, 0, 16, 9])
    offsets = np.concatenate([[0], counts.cumsum()]).astype(np.int64)
    q, xs = O.quant_act_int8(rng.standard_normal((int(offsets[-1]), K)).astype(np.float32) * 3)
    want = O.grouped_gemm_i8(q, xs, offsets, terms[0][0], terms[0][1].astype(np.float32), K, group, "tq2")
    tiled = kb.tile_weights(torch.from_numpy(terms[0][0]).to(DEV), "tq2", K)
    got = kb.grouped_ternary_gemm(torch.from_numpy(q).to(DEV), torch.from_numpy(xs).to(DEV), offsets, tiled,
                                  torch.from_numpy(terms[0][1]).to(DEV), K, group, "tq2", algo="decode").cpu().numpy()
    np.testing.assert_allclose(got, want, rtol=2e-6, atol=1e-6)


def test_a_bounded_wait_that_runs_out_is_reported_and_leaves_the_gpu_usable(kb):
    """Failure detection in the form a shared GPU allows: through the library's test hook the epilogue warps of the tcgen05
    kernel withhold one signal and the wait limit is ~1 ms, so a wait runs out BY DESIGN at the CTA's second tile. The
    kernel must return (no fault, no endless spin), dst_check_device_status must say DST_ERR_TIMEOUT once, and an
    ordinary launch right afterwards must give the right answer."""
    from deepseekternarized_b200 import _lib

    lib = kb.ext()
    N, K, M, fmt = 512, 256, 64, "tq2"  # four 128-row tiles for one CTA
    rng = np.random.default_rng(9)
    terms = make_terms(rng, N, K, 128, fmt, 1)
    x = O.synth_acts(rng, (M, K))
    tiled = kb.tile_weights(torch.from_numpy(terms[0][0]).to(DEV), fmt, K)
    sc = [torch.from_numpy(terms[0][1]).to(DEV)]
    run = lambda: kb.ternary_gemm_bf16(bf16_tensor(x, DEV), [tiled], sc, K, 128, fmt, algo="prefill")
    assert lib.dst_check_device_status(None) == _lib.OK
    _lib.check(lib.dst_debug_prefill_timeout(2_000_000, 1, 1))
    try:
        run()  # the second tile's wait for the accumulator gives up after ~1 ms; the CTA aborts in order
        assert lib.dst_check_device_status(None) == _lib.ERR_TIMEOUT
        assert lib.dst_check_device_status(None) == _lib.OK  # the status word is cleared by the read
    finally:
        _lib.check(lib.dst_debug_prefill_timeout(0, 0, 0))
    y = run().cpu().numpy()
    assert lib.dst_check_device_status(None) == _lib.OK
    check_gemm(y, x, terms, K, 128, fmt)


def test_ep_placement_kernel_swiglu_with_device_row_count_and_barrier():
    """The pieces that keep an expert-parallel step free of host round trips: the placement kernel against the host
    formula (deepseekternarized_b200.moe.ep_placement), SwiGLU over a buffer of larger capacity with the row count read
    on the device, and the peer-memory barrier with one rank (its own flag word)."""
    import ctypes

    from deepseekternarized_b200 import _lib
    from deepseekternarized_b200.kernels import ternary_b200 as kb
    from deepseekternarized_b200.moe import ep_placement

    lib = kb.ext()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rng = np.random.default_rng(2)
    W, E = 4, 24
    El = E // W
    counts = torch.from_numpy(rng.integers(0, 9, (W, E))).to(DEV)
    offs_all = torch.cat([torch.zeros(W, 1, dtype=torch.int64, device=DEV), counts.cumsum(1)], 1).contiguous()
    for rank in range(W):
        want_start, want_local = ep_placement(counts, rank, El)
        dst_start = torch.empty(E, dtype=torch.int64, device=DEV)
        local = torch.empty(El + 1, dtype=torch.int64, device=DEV)
        _lib.check(lib.dst_ep_placement(offs_all.data_ptr(), W, E, El, rank, dst_start.data_ptr(), local.data_ptr(), stream))
        assert torch.equal(dst_start, want_start) and torch.equal(local, want_local)
    # SwiGLU with the row count on the device: the first n rows equal the plain call, the rest of the buffer is not written
    cap, n, inter = 700, 333, 256
    gu = bf16_tensor(rng.standard_normal((cap, 2 * inter)).astype(np.float32), DEV)
    wts = torch.from_numpy(rng.random(cap).astype(np.float32)).to(DEV)
    h0, f0 = torch.empty(n, inter, dtype=torch.float16, device=DEV), torch.empty(n, device=DEV)
    _lib.check(lib.dst_swiglu_norm(gu.data_ptr(), wts.data_ptr(), None, n, inter, ctypes.c_float(0.0), h0.data_ptr(), f0.data_ptr(), stream))
    h1 = torch.full((cap, inter), 7.0, dtype=torch.float16, device=DEV)
    f1 = torch.full((cap,), 7.0, device=DEV)
    n_dev = torch.tensor([n], dtype=torch.int64, device=DEV)
    _lib.check(lib.dst_swiglu_norm_dev(gu.data_ptr(), wts.data_ptr(), None, cap, n_dev.data_ptr(), inter, ctypes.c_float(0.0), h1.data_ptr(),
                                       f1.data_ptr(), stream))
    assert torch.equal(h1[:n], h0) and torch.equal(f1[:n], f0) and bool((h1[n:] == 7.0).all()) and bool((f1[n:] == 7.0).all())
    # one-rank barrier: stores its own flag and returns at once; the status stays clean
    flags = torch.zeros(16, dtype=torch.int64, device=DEV)
    table = (ctypes.c_void_p * 1)(flags.data_ptr())
    for seq in (1, 2, 3):
        _lib.check(lib.dst_ep_barrier(table, 1, 0, seq, stream))
    torch.cuda.synchronize()
    assert int(flags[0]) == 3 and lib.dst_check_device_status(None) == _lib.OK
