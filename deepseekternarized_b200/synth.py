"""Seeded synthetic routed experts, generated on the device: the stand-in for a checkpoint in benchmarks and in the
parity tests at full model size (there is no public weight file for the layer shapes being measured).

Distributions: trits i.i.d. with P(0) = 0.4, P(+1) = P(-1) = 0.3; one fp16 scale per 128 K-elements drawn from
lognormal(mu = -4, sigma = 0.3); the second and later terms of a stacked (Mode C) weight carry 0.25x scales.
Expert ``e``'s tensors depend only on ``(seed, e)``, so every sharding of the experts sees the same global model and a
single expert can be regenerated on its own (``expert_tensors``) for a check on the host.
"""

from __future__ import annotations

import torch

from .moe import ExpertWeights
from .ternary.pack import pack, packed_cols

GROUP = 128


def expert_tensors(seed: int, e: int, hidden: int, inter: int, fmt: str, k_terms: int, device):
    """Canonical tensors of expert ``e``: per term ``(w13_packed [2I, Kp(hidden)], w13_scale [2I, hidden/128],
    w2_packed [hidden, Kp(I)], w2_scale [hidden, I/128])``; rows 0..I-1 of w13 are the gate projection w1, the
    rest the up projection w3."""
    g = torch.Generator(device=device)
    g.manual_seed(seed + 1000 * e)
    terms = []
    for i in range(k_terms):
        out = []
        for (Nw, Kw) in ((2 * inter, hidden), (hidden, inter)):
            u = torch.rand(Nw, Kw, generator=g, device=device)
            t = torch.where(u < 0.4, 0, torch.where(u < 0.7, 1, -1)).to(torch.int8)
            s = torch.exp(torch.randn(Nw, Kw // GROUP, generator=g, device=device) * 0.3 - 4.0)
            if i:
                s = s * 0.25
            out += [pack(t, fmt), s.half()]
        terms.append(tuple(out))
    return terms


def synth_expert_weights(n_local: int, expert0: int, device, fmt: str, hidden: int, inter: int, seed: int, k_terms: int = 1,
                         prepare: bool = True) -> ExpertWeights:
    """Experts ``expert0 .. expert0 + n_local - 1`` stacked as ``ExpertWeights`` (tiled once when ``prepare``)."""
    w13p = [torch.empty(n_local, 2 * inter, packed_cols(fmt, hidden), dtype=torch.uint8, device=device) for _ in range(k_terms)]
    w13s = [torch.empty(n_local, 2 * inter, hidden // GROUP, dtype=torch.float16, device=device) for _ in range(k_terms)]
    w2p = [torch.empty(n_local, hidden, packed_cols(fmt, inter), dtype=torch.uint8, device=device) for _ in range(k_terms)]
    w2s = [torch.empty(n_local, hidden, inter // GROUP, dtype=torch.float16, device=device) for _ in range(k_terms)]
    for j in range(n_local):
        for i, (a, b, c, d) in enumerate(expert_tensors(seed, expert0 + j, hidden, inter, fmt, k_terms, device)):
            w13p[i][j], w13s[i][j], w2p[i][j], w2s[i][j] = a, b, c, d
    w = ExpertWeights(w13p, w13s, w2p, w2s, hidden, inter, GROUP, fmt)
    return w.prepare() if prepare else w
