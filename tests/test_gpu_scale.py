"""GPU parity at the BASELINE configurations' own sizes, and the router / layer options of the V4 engine.

At full size (384 experts, up to 98 304 routed rows) the oracle cannot run the whole layer in seconds, so every stage is
checked where its result can be known exactly or from a sample:
  routing and the routing sort     against the oracle on ALL tokens (ids and order bit-exact, weights rtol 1e-5)
  the two grouped GEMMs            float32 outputs of six sampled experts (fewest rows, most rows, first, last, two
                                   random) against the fp64 dequantized product (rel. Frobenius <= 2e-3, cosine >=
                                   0.99999) and, on a few rows each, against the CPU kernel's order of operations
                                   (rtol 1e-4 / atol 1e-3, the reference's own bounds)
  SwiGLU and its rounding points   the sampled experts' rows recomputed on the host from the GPU's own gate/up rows
  combine                          sampled tokens recomputed on the host from the GPU's own expert outputs: bit-exact
Weights are the seeded synthetic experts of deepseekternarized_b200/synth.py, regenerated one expert at a time for the host side.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.helpers import bf16_numpy, bf16_tensor, check_gemm, check_layer
from tests.test_oracle_golden import variant_case

pytestmark = pytest.mark.gpu
DEV = "cuda"
SEED = 20261125


def _host_terms(seed, e, hidden, inter, fmt, k_terms):
    """Expert e of the synthetic model as oracle term lists: (w13 terms, w2 terms)."""
    from deepseekternarized_b200.synth import expert_tensors

    ts = expert_tensors(seed, e, hidden, inter, fmt, k_terms, DEV)
    w13 = [(a.cpu().numpy(), b.cpu().numpy()) for a, b, _, _ in ts]
    w2 = [(c.cpu().numpy(), d.cpu().numpy()) for _, _, c, d in ts]
    return w13, w2


def _layer_at_scale(T, E, hidden, inter, fmt, k_terms, top_k, n_tokens_checked=64):
    from deepseekternarized_b200.kernels import ternary_b200 as kb
    from deepseekternarized_b200.moe import B200Ops, MoELayer
    from deepseekternarized_b200.synth import synth_expert_weights

    w = synth_expert_weights(E, 0, DEV, fmt, hidden, inter, SEED, k_terms=k_terms)
    assert isinstance(w.w13_packed[0], kb.TiledWeights)
    g = torch.Generator().manual_seed(SEED + 7)
    x_t = torch.randn(T, hidden, generator=g).bfloat16()
    logits_t = torch.randn(T, E, generator=g)
    x, logits = x_t.float().numpy(), logits_t.numpy()
    xd, ld = x_t.to(DEV), logits_t.to(DEV)
    ops = B200Ops()
    layer = MoELayer(w, top_k, ops=ops)

    # routing and sort: all tokens
    wts, ids = ops.route(ld, top_k, 1.0)
    w_ref, idx_ref = O.route_from_logits(logits, top_k)
    assert np.array_equal(ids.cpu().numpy(), idx_ref)
    np.testing.assert_allclose(wts.cpu().numpy(), w_ref, rtol=1e-5, atol=1e-7)
    order, offsets = ops.sort(ids, E)
    order_ref, offsets_ref = O.sort_by_expert(idx_ref.reshape(-1), E)
    assert np.array_equal(order.cpu().numpy(), order_ref) and np.array_equal(offsets.cpu().numpy(), offsets_ref)

    # the layer's own steps, keeping the intermediates; float32 copies of the two GEMM outputs for the tolerance checks
    xs = layer.gather_for_experts(xd, order, top_k)
    gu = ops.gemm(xs, offsets, w.w13_packed, w.w13_scale, hidden, 128, fmt)
    gu32 = kb.grouped_ternary_gemm_bf16(xs, offsets, w.w13_packed, w.w13_scale, hidden, 128, fmt, out_dtype=torch.float32,
                                        validate_offsets=False)
    h = ops.swiglu(gu, wts.reshape(-1), order, inter, 0.0, for_weights=w.w2_packed)
    down = ops.gemm(h, offsets, w.w2_packed, w.w2_scale, inter, 128, fmt)
    down32 = kb.grouped_ternary_gemm_bf16(h, offsets, w.w2_packed, w.w2_scale, inter, 128, fmt, out_dtype=torch.float32,
                                          validate_offsets=False)
    y = ops.combine(down, order, ids, T, top_k)
    assert torch.equal(y, layer(xd, ld))  # the public call is these steps
    assert torch.equal(gu, gu32.bfloat16()) and torch.equal(down, down32.bfloat16())  # one kernel, two output types

    counts = np.diff(offsets_ref)
    rng = np.random.default_rng(5)
    nonempty = np.nonzero(counts)[0]
    picks = {int(nonempty[np.argmin(counts[nonempty])]), int(np.argmax(counts)), int(nonempty[0]), int(nonempty[-1])}
    picks |= {int(v) for v in rng.choice(nonempty, 2, replace=False)}
    h_rows = (h.data.float() * h.factor[:, None]).cpu().numpy() if isinstance(h, kb.NormRows) else bf16_numpy(h)
    for e in sorted(picks):
        a, b = int(offsets_ref[e]), int(offsets_ref[e + 1])
        w13, w2 = _host_terms(SEED, e, hidden, inter, fmt, k_terms)
        rows = x[order_ref[a:b] // top_k]
        check_gemm(gu32[a:b].cpu().numpy(), rows, w13, hidden, 128, fmt)
        few = slice(a, min(b, a + 4))
        want = O.ternary_linear(x[order_ref[few] // top_k], w13, hidden, 128, fmt, out_bf16=False)
        np.testing.assert_allclose(gu32[few].cpu().numpy(), want, rtol=1e-4, atol=1e-3)
        # SwiGLU from the GPU's own bf16 gate/up rows: bf16(weight * silu(gate) * up), at most a rounding flip apart
        gun = bf16_numpy(gu[a:b])
        hw = O.bf16_round((w_ref.reshape(-1)[order_ref[a:b], None] * (O.silu(gun[:, :inter]) * gun[:, inter:])).astype(np.float32))
        assert np.mean(O.bf16_bits(h_rows[a:b]) != O.bf16_bits(hw)) < 0.02 and O.rel_fro(h_rows[a:b], hw) < 1e-3
        check_gemm(down32[a:b].cpu().numpy(), h_rows[a:b], w2, inter, 128, fmt)
        want = O.ternary_linear(h_rows[few], w2, inter, 128, fmt, out_bf16=False)
        np.testing.assert_allclose(down32[few].cpu().numpy(), want, rtol=1e-4, atol=1e-3)

    # combine: sampled tokens from the GPU's own bf16 expert outputs, fp32 sums in increasing expert id
    inv = np.empty(T * top_k, np.int64)
    inv[order_ref] = np.arange(T * top_k)
    toks = rng.choice(T, n_tokens_checked, replace=False)
    pos = np.stack([inv[t * top_k + np.argsort(idx_ref[t], kind="stable")] for t in toks])  # [n, k] rows of `down`
    d = down[torch.from_numpy(pos.reshape(-1)).to(DEV)].float().cpu().numpy().reshape(len(toks), top_k, hidden)
    acc = np.zeros((len(toks), hidden), np.float32)
    for s in range(top_k):
        acc += d[:, s]
    assert np.array_equal(O.bf16_bits(bf16_numpy(y[torch.from_numpy(toks).to(DEV)])), O.bf16_bits(O.bf16_round(acc)))


def test_config2_layer_at_full_size():
    """BASELINE config 2: 4096 tokens, 384 TQ1 experts (4096 -> 2048 -> 4096), top-6: 24 576 rows, ~64 per expert."""
    _layer_at_scale(4096, 384, 4096, 2048, "tq1", 1, 6)


def test_config3_prefill_at_full_size():
    """BASELINE config 3, prefill: the config-2 shapes with two stacked TQ2 terms per weight (second scales 0.25x)."""
    _layer_at_scale(4096, 384, 4096, 2048, "tq2", 2, 6)


def test_config4_layer_at_full_size_on_one_gpu():
    """BASELINE config 4 at one GPU: 16 384 tokens -> 98 304 rows, ~256 per expert."""
    _layer_at_scale(16384, 384, 4096, 2048, "tq1", 1, 6)


# ------------------------------------------------------------------------------------------ router and layer options
@pytest.mark.parametrize("name", ["sigmoid", "sqrtsoftplus", "softmax_limit"])
def test_moe_layer_variants_against_reference_golden(golden, name):
    """The reference's V4Model.route / swiglu / moe with sigmoid and sqrt-softplus scores, gate bias, temperature, no
    renormalisation, route_scale, SwiGLU clamp and shared expert (fixture generated from the reference)."""
    from deepseekternarized_b200.moe import B200Ops, ExpertWeights, MoELayer
    from tests.helpers import stack_experts

    c = variant_case(golden("moe_layer_variants"), name)
    ld = torch.from_numpy(c["logits"]).to(DEV)
    bias = torch.from_numpy(c["bias"]).to(DEV) if c["bias"] is not None else None
    w, ids = B200Ops().route(ld, c["topk"], c["route_scale"], renorm=c["norm"], score_func=c["score_func"], bias=bias,
                             gate_temp=c["gate_temp"])
    assert np.array_equal(ids.cpu().numpy(), c["indices"])
    np.testing.assert_allclose(w.cpu().numpy(), c["weights"], rtol=1e-5, atol=1e-7)
    args = (c["hidden"], c["inter"], c["group"], c["fmt"])
    ew = ExpertWeights(*stack_experts(c["experts"], c["k_terms"], DEV), *args).prepare()
    shared = ExpertWeights(*stack_experts([c["shared"]], c["k_terms"], DEV), *args).prepare() if c["shared"] is not None else None
    layer = MoELayer(ew, c["topk"], route_scale=c["route_scale"], swiglu_limit=c["limit"], norm_topk_prob=c["norm"],
                     score_func=c["score_func"], gate_bias=bias, gate_temp=c["gate_temp"], shared=shared)
    xd = bf16_tensor(c["x"], DEV)
    y = layer(xd, ld)
    want = O.from_bf16_bits(c["y_bits"])
    exact = O.moe_layer_f64(c["x"], c["weights"], c["indices"], c["experts"], *args, swiglu_limit=c["limit"], shared=c["shared"])
    check_layer(bf16_numpy(y), want, exact)
    # the entry an engine calls with the routing it has already computed
    y2 = layer.forward_routed(xd, torch.from_numpy(c["weights"]).to(DEV), torch.from_numpy(c["indices"]).to(DEV))
    check_layer(bf16_numpy(y2), want, exact)
    assert O.rel_fro(bf16_numpy(y2), bf16_numpy(y)) < 2e-3


def test_routing_never_leaves_the_expert_range():
    """Rows of NaN, of -inf, of +inf and rows with fewer finite logits than top_k: k distinct ids inside [0, E) for
    every token, nothing dropped by the sort, a complete order; and a layer step over them that touches no memory it
    should not (the result rows of the poisoned tokens may be NaN, the others must be the clean layer's)."""
    from deepseekternarized_b200.kernels import ternary_b200 as kb
    from deepseekternarized_b200.moe import B200Ops, ExpertWeights, MoELayer
    from tests.helpers import make_experts, stack_experts

    T, E, top_k, hidden, inter = 64, 16, 6, 256, 128
    rng = np.random.default_rng(3)
    logits = rng.standard_normal((T, E)).astype(np.float32)
    logits[0] = np.nan
    logits[1] = -np.inf
    logits[2] = np.inf
    logits[3, 4:] = np.nan        # four finite logits, top-6 asked
    logits[4, :] = -np.inf
    logits[4, 7] = 0.5            # one finite logit
    logits[5, 3] = np.nan         # one NaN among numbers: ranks first, as in torch.topk
    ld = torch.from_numpy(logits).to(DEV)
    for score_func in ("softmax", "sigmoid", "sqrtsoftplus"):
        w, ids = B200Ops().route(ld, top_k, 1.0, score_func=score_func)
        idn = ids.cpu().numpy()
        assert idn.min() >= 0 and idn.max() < E
        assert all(len(set(r)) == top_k for r in idn.tolist())
        if score_func != "softmax":  # one NaN makes a whole softmax row NaN; elsewhere only that expert's score
            assert idn[5, 0] == 3
        want = torch.topk(torch.from_numpy(logits[6:]), top_k, dim=-1)[1].numpy()  # monotone scores: the clean rows follow the logits
        assert np.array_equal(idn[6:], want)
        order, offsets = kb.sort_by_expert(ids.reshape(-1), E)
        assert int(offsets[-1]) == T * top_k
        assert np.array_equal(np.sort(order.cpu().numpy()), np.arange(T * top_k))
    experts = make_experts(rng, E, hidden, inter, 128, "tq1", 1)
    ew = ExpertWeights(*stack_experts(experts, 1, DEV), hidden, inter, 128, "tq1").prepare()
    x = O.synth_acts(rng, (T, hidden))
    layer = MoELayer(ew, top_k)
    y = layer(bf16_tensor(x, DEV), ld)
    clean = logits.copy()
    clean[:6] = 0.0
    y_clean = layer(bf16_tensor(x, DEV), torch.from_numpy(clean).to(DEV))
    torch.cuda.synchronize()
    assert torch.equal(y[6:], y_clean[6:])
    # ids a caller computed, some outside the range: those slots are dropped, nothing else moves
    w_ok, ids_ok = B200Ops().route(torch.from_numpy(clean).to(DEV), top_k, 1.0)
    ids_bad = ids_ok.clone()
    ids_bad[10, 2] = E + 5
    ids_bad[11, 0] = -1
    y_bad = layer.forward_routed(bf16_tensor(x, DEV), w_ok, ids_bad)
    torch.cuda.synchronize()
    keep = torch.ones(T, dtype=torch.bool, device=DEV)
    keep[10] = keep[11] = False
    assert torch.equal(y_bad[keep], y_clean[keep]) and bool(torch.isfinite(y_bad.float()).all())
