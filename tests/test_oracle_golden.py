"""The CPU oracle against fixtures produced by the reference's own code (tests/golden/make_golden.py)."""

from __future__ import annotations

import hashlib

import numpy as np
import pytest

from oracle import oracle as O

FMT = {1: "tq1", 2: "tq2"}


@pytest.mark.parametrize("fmt", ["tq2", "tq1"])
@pytest.mark.parametrize("K", [1, 4, 5, 7, 128, 131, 640])
def test_pack_unpack_match_reference(golden, fmt, K):
    g = golden("format")
    t, p = g[f"trits_{fmt}_{K}"], g[f"packed_{fmt}_{K}"]
    got = O.pack(t, fmt)
    assert got.dtype == np.uint8 and got.shape == (9, O.packed_cols(fmt, K))
    assert np.array_equal(got, p)
    assert np.array_equal(O.unpack(p, fmt, K), t)


def test_tq1_lut_and_every_pattern(golden):
    g = golden("format")
    assert np.array_equal(O.tq1_lut(), g["tq1_lut"])
    assert np.all(O.tq1_lut()[243:] == 0)
    p = O.pack(g["tq1_patterns"], "tq1")
    assert np.array_equal(p, g["tq1_patterns_packed"])
    assert np.unique(p).size == 243 and p.max() < 243
    assert np.array_equal(O.unpack(p, "tq1", 5), g["tq1_patterns"])


def test_unpack_every_byte_value(golden):
    g = golden("format")
    allb = np.arange(256, dtype=np.uint8).reshape(256, 1)
    assert np.array_equal(O.unpack(allb, "tq1", 5), g["unpack_all_bytes_tq1"])
    assert np.array_equal(O.unpack(allb, "tq2", 4), g["unpack_all_bytes_tq2"])


def _linear_cases(g):
    for c in range(int(g["n_cases"])):
        yield c


def test_float_linear_bit_exact_with_reference_cpu_kernel(golden):
    g = golden("linear_f32")
    for c in range(int(g["n_cases"])):
        K, group, N, M, k_terms, code = (int(v) for v in g[f"c{c}_meta"])
        fmt = FMT[code]
        x = O.from_bf16_bits(g[f"c{c}_x_bits"])
        terms = [(g[f"c{c}_packed{i}"], g[f"c{c}_scale{i}"]) for i in range(k_terms)]
        y = O.ternary_linear(x, terms, K, group, fmt, out_bf16=False)
        assert np.array_equal(y, g[f"c{c}_y_f32"]), f"case {c}"
        assert np.array_equal(O.bf16_bits(O.ternary_linear(x, terms, K, group, fmt)), g[f"c{c}_y_bf16_bits"])
        y64 = O.gemm_f64(x, terms, K, group, fmt)
        assert O.rel_fro(y, y64) < 1e-6 and O.cosine(y, y64) > 0.9999999
        w = O.dequantized(terms, K, group, fmt)
        assert np.allclose(x.astype(np.float64) @ w.T, y64, rtol=1e-12, atol=1e-12)


def test_int8_paths_match_reference(golden):
    g = golden("linear_i8")
    for c in range(int(g["n_cases"])):
        K, group, N, M, code = (int(v) for v in g[f"c{c}_meta"])
        fmt = FMT[code]
        q, xs = O.quant_act_int8(g[f"c{c}_x_f32"])
        assert np.array_equal(q, g[f"c{c}_q"]) and np.array_equal(xs, g[f"c{c}_xs"])
        ref = O.gemm_ref_i8(q, xs, g[f"c{c}_packed"], g[f"c{c}_scale_f32"], K, group, fmt)
        assert np.array_equal(ref, g[f"c{c}_y_ref"]), f"case {c}"
        cpp = O.gemm_i8(q, xs, g[f"c{c}_packed"], g[f"c{c}_scale_f32"], K, group, fmt)
        assert np.array_equal(cpp, g[f"c{c}_y_cpp"]), f"case {c}"


@pytest.mark.parametrize("fmt", ["tq1", "tq2"])
def test_grouped_and_routing_sort(golden, fmt):
    g = golden("grouped")
    order, offsets = O.sort_by_expert(g[f"{fmt}_ids"], 6)
    assert np.array_equal(order, g[f"{fmt}_order"]) and np.array_equal(offsets, g[f"{fmt}_offsets"])
    rows = order // 2
    out = O.grouped_gemm_i8(g[f"{fmt}_q"][rows], g[f"{fmt}_xs"][rows], offsets, g[f"{fmt}_packed"], g[f"{fmt}_scale_f32"], 192, 64, fmt)
    assert np.array_equal(out, g[f"{fmt}_out"])
    with pytest.raises(ValueError, match="offsets"):
        O.grouped_gemm_i8(g[f"{fmt}_q"], g[f"{fmt}_xs"], [0, 9], g[f"{fmt}_packed"], g[f"{fmt}_scale_f32"], 192, 64, fmt)


@pytest.mark.parametrize("fmt", ["tq1", "tq2"])
def test_moe_layer_matches_reference(golden, fmt):
    g = golden("moe_layer")
    T, hidden, inter, E, topk, group, k_terms = (int(v) for v in g[f"{fmt}_meta"])
    x = O.from_bf16_bits(g[f"{fmt}_x_bits"])
    w, idx = O.route_softmax_topk(x, g[f"{fmt}_gate_w"], topk)
    assert np.array_equal(idx, g[f"{fmt}_route_indices"])
    assert np.allclose(w, g[f"{fmt}_route_weights"], rtol=1e-5, atol=1e-7)
    experts = [tuple([(g[f"{fmt}_e{e}_{wn}_packed{i}"], g[f"{fmt}_e{e}_{wn}_scale{i}"]) for i in range(k_terms)]
                     for wn in ("w1", "w2", "w3")) for e in range(E)]
    # with the reference's own routing weights the layer must reproduce the reference bit for bit
    y = O.moe_layer(x, g[f"{fmt}_route_weights"], g[f"{fmt}_route_indices"], experts, hidden, inter, group, fmt)
    want = O.from_bf16_bits(g[f"{fmt}_y_bits"])
    assert O.rel_fro(y, want) < 2e-3
    mism = np.mean(O.bf16_bits(y) != g[f"{fmt}_y_bits"])
    assert mism < 0.02, mism


def test_baseline_shapes_hash(golden):
    g = golden("baseline_shapes")
    for c in range(int(g["n_cases"])):
        code, N, K, M = (int(v) for v in g[f"c{c}_meta"])
        if N * M > 4096 * 4:  # keep the CPU suite short: the largest cases run in the gpu suite's oracle leg
            continue
        fmt = FMT[code]
        rng = np.random.default_rng(6000 + c)
        t = O.synth_trits(rng, (N, K))
        s = O.synth_scales(rng, (N, K // 128))
        x = O.synth_acts(rng, (M, K))
        p = O.pack(t, fmt)
        assert hashlib.sha256(p.tobytes()).digest() == g[f"c{c}_packed_sha256"].tobytes()
        y = O.gemm_f32(x, p, s.astype(np.float32), K, 128, fmt)
        assert np.array_equal(y.reshape(-1)[::61], g[f"c{c}_sample"])
        assert hashlib.sha256(y.tobytes()).digest() == g[f"c{c}_sha256"].tobytes()


@pytest.mark.parametrize("fmt", ["tq1", "tq2"])
def test_moe_layer_standard_flavour_matches_reference(golden, fmt):
    """boilerplate/engine/standard.py:154-176 (OLMoE-style: bf16 intermediates, weight after the down projection,
    bf16 accumulation; norm_topk_prob on for the TQ1 case, off for the TQ2 k = 2 case)."""
    g = golden("moe_layer_standard")
    T, hidden, inter, E, topk, group, k_terms, renorm = (int(v) for v in g[f"{fmt}_meta"])
    x = O.from_bf16_bits(g[f"{fmt}_x_bits"])
    experts = [tuple([(g[f"{fmt}_e{e}_{wn}_packed{i}"], g[f"{fmt}_e{e}_{wn}_scale{i}"]) for i in range(k_terms)]
                     for wn in ("w1", "w2", "w3")) for e in range(E)]
    y, w, idx = O.moe_layer_standard(x, g[f"{fmt}_logits"], experts, topk, hidden, inter, group, fmt, norm_topk_prob=bool(renorm))
    assert np.array_equal(idx, g[f"{fmt}_route_indices"])
    want = O.from_bf16_bits(g[f"{fmt}_y_bits"])
    assert O.rel_fro(y, want) < 2e-3
    mism = np.mean(O.bf16_bits(y) != g[f"{fmt}_y_bits"])
    assert mism < 0.02, mism


@pytest.mark.parametrize("fmt", ["tq1", "tq2"])
def test_table_row_lookup_matches_reference(golden, fmt):
    """boilerplate/engine/model.py:458-464: rows of a ternary lookup table, dequantised and summed over terms."""
    g = golden("table_rows")
    V, K, group, k_terms = (int(v) for v in g[f"{fmt}_meta"])
    terms = [(g[f"{fmt}_packed{i}"], g[f"{fmt}_scale{i}"]) for i in range(k_terms)]
    vals = O.gather_dequant_rows(g[f"{fmt}_ids"], terms, K, group, fmt)
    assert vals.shape == (*g[f"{fmt}_ids"].shape, K)
    assert np.array_equal(O.bf16_bits(vals).reshape(-1, K), g[f"{fmt}_vals_bits"])


def variant_case(g, name):
    """One case of the moe_layer_variants fixture (tests/golden/make_golden.py, section 5d) as plain values."""
    T, hidden, inter, E, topk, group, k_terms, code, norm, with_shared = (int(v) for v in g[f"{name}_meta"])
    gate_temp, route_scale, limit = (float(v) for v in g[f"{name}_params"])
    fmt = FMT[code]

    def terms(tag, wn):
        return [(g[f"{name}_{tag}_{wn}_packed{i}"], g[f"{name}_{tag}_{wn}_scale{i}"]) for i in range(k_terms)]

    experts = [tuple(terms(f"e{e}", wn) for wn in ("w1", "w2", "w3")) for e in range(E)]
    shared = tuple(terms("shared", wn) for wn in ("w1", "w2", "w3")) if with_shared else None
    bias = g[f"{name}_gate_b"] if f"{name}_gate_b" in g.files else None
    return dict(T=T, hidden=hidden, inter=inter, E=E, topk=topk, group=group, k_terms=k_terms, fmt=fmt, norm=bool(norm),
                gate_temp=gate_temp, route_scale=route_scale, limit=limit, score_func=str(g[f"{name}_score_func"]), bias=bias,
                experts=experts, shared=shared, x=O.from_bf16_bits(g[f"{name}_x_bits"]), logits=g[f"{name}_logits"],
                weights=g[f"{name}_route_weights"], indices=g[f"{name}_route_indices"], y_bits=g[f"{name}_y_bits"])


@pytest.mark.parametrize("name", ["sigmoid", "sqrtsoftplus", "softmax_limit"])
def test_moe_layer_variants_match_reference(golden, name):
    """boilerplate/engine/model.py:376-422 with the options the plain fixture leaves off: sigmoid and sqrt-softplus
    scores, a gate bias (selection only), a temperature, no renormalisation, route_scale, the SwiGLU clamp and the
    shared expert, each produced by the reference's own V4Model.route / swiglu / moe."""
    c = variant_case(golden("moe_layer_variants"), name)
    w, idx = O.route_from_logits(c["logits"], c["topk"], c["route_scale"], c["score_func"], c["bias"], c["gate_temp"], c["norm"])
    assert np.array_equal(idx, c["indices"])
    assert np.allclose(w, c["weights"], rtol=1e-5, atol=1e-7)
    y = O.moe_layer(c["x"], c["weights"], c["indices"], c["experts"], c["hidden"], c["inter"], c["group"], c["fmt"],
                    swiglu_limit=c["limit"], shared=c["shared"])
    want = O.from_bf16_bits(c["y_bits"])
    assert O.rel_fro(y, want) < 2e-3
    assert np.mean(O.bf16_bits(y) != c["y_bits"]) < 0.02
