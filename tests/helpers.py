"""Shared test helpers: numpy<->torch bf16 conversion, seeded inputs, and an ops object that runs the
MoE layer's steps on the CPU oracle (used to exercise the expert-parallel host logic on gloo ranks)."""

from __future__ import annotations

import numpy as np
import torch

from oracle import oracle as O


def bf16_tensor(a: np.ndarray, device="cpu") -> torch.Tensor:
    """float32 numpy array holding bf16-representable values -> torch bf16 tensor."""
    return torch.from_numpy(O.bf16_bits(a).view(np.int16)).view(torch.bfloat16).reshape(a.shape).to(device)


def bf16_numpy(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def make_terms(rng, N, K, group, fmt, k_terms=1, lead=()):
    """k stacked terms of seeded trits / lognormal fp16 scales; second and later terms 0.25x."""
    terms = []
    for i in range(k_terms):
        t = O.synth_trits(rng, (*lead, N, K))
        s = O.synth_scales(rng, (*lead, N, -(-K // group)))
        if i:
            s = (s.astype(np.float32) * 0.25).astype(np.float16)
        p = O.pack(t.reshape(-1, K), fmt).reshape(*lead, N, -1)
        terms.append((p, s))
    return terms


def check_gemm(got: np.ndarray, x: np.ndarray, terms, K, group, fmt, tol=2e-3, cos_min=0.99999):
    """The north-star tolerance: relative Frobenius error <= 2e-3 and cosine >= 0.99999 against the fp64
    dequantized product; returns (rel, cos)."""
    y64 = O.gemm_f64(x, terms, K, group, fmt)
    rel, cos = O.rel_fro(got, y64), O.cosine(got, y64)
    assert rel <= tol and cos >= cos_min, (rel, cos)
    return rel, cos


def check_layer(got: np.ndarray, want: np.ndarray, exact64: np.ndarray):
    """Layer-level parity. The reference layer rounds to bf16 after each of its three linears and at
    the end, so two correct implementations differ by rounding flips; measure both against the
    unrounded fp64 layer: ours may be at most 25 % further from it than the reference-order oracle is,
    and must stay within twice that distance of the oracle itself. Returns (ours, oracle's) distance."""
    e_ref, e_got = O.rel_fro(want, exact64), O.rel_fro(got, exact64)
    assert e_got <= max(1.25 * e_ref, 2e-3), (e_got, e_ref)
    assert O.rel_fro(got, want) <= max(2.0 * e_ref, 2e-3), (O.rel_fro(got, want), e_ref)
    assert O.cosine(got, want) >= 0.9999
    return e_got, e_ref


class OracleOps:
    """The MoE layer's compute steps on the CPU oracle, torch CPU tensors in and out."""

    def route(self, logits, top_k, route_scale, renorm=True, score_func="softmax", bias=None, gate_temp=1.0):
        w, idx = O.route_from_logits(logits.float().numpy(), top_k, route_scale, score_func,
                                     None if bias is None else bias.float().numpy(), gate_temp, renorm)
        return torch.from_numpy(w), torch.from_numpy(idx.astype(np.int32))

    def sort(self, ids, n_experts):
        order, offsets = O.sort_by_expert(ids.reshape(-1).numpy().astype(np.int64), n_experts)
        return torch.from_numpy(order), torch.from_numpy(offsets)

    def gather(self, x, order, top_k):
        return x if order is None else x[order // top_k].contiguous()

    def gemm(self, x, offsets, packed, scales, K, group, fmt):
        out = None
        xf = x.float().numpy()
        offs = np.array([0, x.size(0)], np.int64) if offsets is None else offsets.numpy()  # None: one expert over all rows
        for p, s in zip(packed, scales):
            out = O.grouped_gemm_f32(xf, offs, p.numpy(), s.float().numpy(), K, group, fmt, out=out)
        return bf16_tensor(O.bf16_round(out))

    def swiglu(self, gu, row_weights, order, inter, limit):
        g, u = gu[:, :inter].float().numpy(), gu[:, inter:].float().numpy()
        if limit > 0:
            u = np.clip(u, -limit, limit)
            g = np.minimum(g, limit)
        h = O.silu(g) * u
        if row_weights is not None:
            w = row_weights.numpy()
            w = w[order.numpy()] if order is not None else w
            h = (w[:, None].astype(np.float32) * h).astype(np.float32)
        return bf16_tensor(O.bf16_round(h))

    def combine(self, down, order, ids, T, top_k, add=None):
        d = down.float().numpy()
        inv = np.empty(T * top_k, np.int64)
        inv[order.numpy()] = np.arange(T * top_k)
        idn = ids.reshape(T, top_k).numpy()
        y = np.zeros((T, d.shape[1]), np.float32)
        for t in range(T):
            for s in np.argsort(idn[t], kind="stable"):
                y[t] += d[inv[t * top_k + s]]
        if add is not None:
            y += add.float().numpy()
        return bf16_tensor(O.bf16_round(y))


def make_experts(rng, E, hidden, inter, group, fmt, k_terms=1):
    """(oracle expert list, stacked arrays for ExpertWeights)."""
    experts = []
    for _ in range(E):
        w1 = make_terms(rng, inter, hidden, group, fmt, k_terms)
        w2 = make_terms(rng, hidden, inter, group, fmt, k_terms)
        w3 = make_terms(rng, inter, hidden, group, fmt, k_terms)
        experts.append((w1, w2, w3))
    return experts


def stack_experts(experts, k_terms, device="cpu"):
    from deepseekternarized_b200.moe import ExpertWeights  # noqa: F401  (import kept local: package import is light)

    w13p = [torch.from_numpy(np.stack([np.concatenate([e[0][i][0], e[2][i][0]]) for e in experts])).to(device) for i in range(k_terms)]
    w13s = [torch.from_numpy(np.stack([np.concatenate([e[0][i][1], e[2][i][1]]) for e in experts])).to(device) for i in range(k_terms)]
    w2p = [torch.from_numpy(np.stack([e[1][i][0] for e in experts])).to(device) for i in range(k_terms)]
    w2s = [torch.from_numpy(np.stack([e[1][i][1] for e in experts])).to(device) for i in range(k_terms)]
    return w13p, w13s, w2p, w2s
