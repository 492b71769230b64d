"""Manifest-driven loader (deepseekternarized_b200/loader.py) against a small export written here in the layout of
the reference's docs/architecture/format.md (Mode C tensors `X.tq{i}.packed` / `X.tq{i}.scale`, manifest.json with
per-tensor file and SHA-256)."""

from __future__ import annotations

import hashlib
import json

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.helpers import bf16_numpy, bf16_tensor, check_layer, make_experts, stack_experts


def write_export(root, experts, prefix, fmt, group, k_terms, hidden, inter, n_files=2):
    from safetensors.torch import save_file

    shards = [dict() for _ in range(n_files)]
    manifest = {"format": "boilerplate", "version": 1, "tensors": {}}
    for e, (w1, w2, w3) in enumerate(experts):
        for name, terms, shape in (("w1", w1, [inter, hidden]), ("w2", w2, [hidden, inter]), ("w3", w3, [inter, hidden])):
            base = f"{prefix}.{e}.{name}"
            stored = {}
            for i, (p, s) in enumerate(terms):
                for suffix, arr in ((f"{base}.tq{i}.packed", p), (f"{base}.tq{i}.scale", s)):
                    f = (e + i) % n_files
                    shards[f][suffix] = torch.from_numpy(np.ascontiguousarray(arr))
                    stored[suffix] = {"dtype": str(arr.dtype), "shape": list(arr.shape), "sha256": hashlib.sha256(arr.tobytes()).hexdigest(),
                                      "file": f"model-{f + 1:05d}-of-{n_files:05d}.safetensors"}
            manifest["tensors"][base] = {"mode": "C", "shape": shape, "packing": fmt, "terms": k_terms, "group": group,
                                         "scale_dtype": "fp16", "act": "bf16", "stored": stored}
    manifest["tensors"]["layers.0.attn.0.wq"] = {"mode": "A"}
    for f, tensors in enumerate(shards):
        save_file(tensors, str(root / f"model-{f + 1:05d}-of-{n_files:05d}.safetensors"))
    (root / "manifest.json").write_text(json.dumps(manifest))


@pytest.mark.parametrize("fmt,k_terms", [("tq1", 1), ("tq2", 2)])
def test_loader_stacks_the_experts_of_an_export(tmp_path, fmt, k_terms):
    from deepseekternarized_b200.loader import ManifestError, load_expert_weights

    E, hidden, inter, group = 6, 256, 128, 128
    rng = np.random.default_rng(3)
    experts = make_experts(rng, E, hidden, inter, group, fmt, k_terms)
    write_export(tmp_path, experts, "layers.1.ffn.experts", fmt, group, k_terms, hidden, inter)
    w = load_expert_weights(tmp_path, "layers.1.ffn.experts", E, verify=True, prepare=False)
    want = stack_experts(experts, k_terms)
    assert (w.hidden, w.inter, w.group, w.fmt, w.n_experts) == (hidden, inter, group, fmt, E)
    for got_list, want_list in zip((w.w13_packed, w.w13_scale, w.w2_packed, w.w2_scale), want):
        assert len(got_list) == k_terms
        for a, b in zip(got_list, want_list):
            assert a.dtype == b.dtype and torch.equal(a, b)
    # a rank's shard for expert parallelism
    half = load_expert_weights(tmp_path, "layers.1.ffn.experts", 3, first_expert=3, prepare=False)
    assert torch.equal(half.w2_packed[0], want[2][0][3:])
    with pytest.raises(ManifestError, match="not in the manifest"):
        load_expert_weights(tmp_path, "layers.1.ffn.experts", E + 1, prepare=False)
    with pytest.raises(ManifestError, match="mode"):
        load_expert_weights(tmp_path, "layers.0.attn", 1, names=("wq", "wq", "wq"), prepare=False)
    # a corrupted byte is caught by the checksum
    m = json.loads((tmp_path / "manifest.json").read_text())
    key = "layers.1.ffn.experts.0.w2"
    first = next(iter(m["tensors"][key]["stored"]))
    m["tensors"][key]["stored"][first]["sha256"] = "0" * 64
    (tmp_path / "manifest.json").write_text(json.dumps(m))
    with pytest.raises(ManifestError, match="SHA-256"):
        load_expert_weights(tmp_path, "layers.1.ffn.experts", E, verify=True, prepare=False)


@pytest.mark.gpu
def test_loaded_export_runs_the_moe_layer(tmp_path):
    from deepseekternarized_b200.loader import load_expert_weights
    from deepseekternarized_b200.moe import MoELayer

    E, hidden, inter, group, fmt, topk, T = 8, 512, 256, 128, "tq1", 2, 400
    rng = np.random.default_rng(8)
    experts = make_experts(rng, E, hidden, inter, group, fmt, 1)
    write_export(tmp_path, experts, "layers.2.ffn.experts", fmt, group, 1, hidden, inter)
    w = load_expert_weights(tmp_path, "layers.2.ffn.experts", E, device="cuda")
    x = O.synth_acts(rng, (T, hidden))
    logits = rng.standard_normal((T, E)).astype(np.float32)
    y = MoELayer(w, topk)(bf16_tensor(x, "cuda"), torch.from_numpy(logits).to("cuda"))
    wr, idx = O.route_from_logits(logits, topk)
    check_layer(bf16_numpy(y), O.moe_layer(x, wr, idx, experts, hidden, inter, group, fmt),
                O.moe_layer_f64(x, wr, idx, experts, hidden, inter, group, fmt))
