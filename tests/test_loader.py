"""Manifest-driven loader (deepseekternarized_b200/loader.py) against a small export written here in the layout of
the reference's docs/architecture/format.md (Mode C tensors `X.tq{i}.packed` / `X.tq{i}.scale`, manifest.json with
per-tensor file and SHA-256), and against tests/golden/export_tiny: a directory written by the reference's own
boilerplate.format.export.export (one Mode C k = 2 rule, two Mode D rules, fp16 and bf16 scales)."""

from __future__ import annotations

import hashlib
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.helpers import bf16_numpy, bf16_tensor, check_layer, make_experts, stack_experts

EXPORT = Path(__file__).resolve().parent / "golden" / "export_tiny"
# (layer, mode, terms, packing, scale dtype, act) of the export's three ternary layers
EXPORT_LAYERS = [(3, "C", 2, "tq1", torch.float16, "bf16"), (4, "D", 1, "tq2", torch.bfloat16, "int8"),
                 (5, "D", 1, "tq1", torch.float16, "bf16")]


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


def _weightstore(name):
    """Tensor `name` as the reference's own reader (boilerplate/engine/weights.py, WeightStore.get) returned it when the
    fixture was made: uint8 packed bytes, or the raw 16 bits of an fp16 / bf16 scale."""
    g = np.load(EXPORT / "weightstore_tensors.npz")
    return g[name]


@pytest.mark.parametrize("layer,mode,k_terms,fmt,scale_dtype,act", EXPORT_LAYERS)
def test_loader_reads_an_export_written_by_the_reference(layer, mode, k_terms, fmt, scale_dtype, act):
    from deepseekternarized_b200.loader import load_expert_weights

    manifest = json.loads((EXPORT / "manifest.json").read_text())
    assert manifest["tensors"][f"layers.{layer}.ffn.experts.0.w1"]["mode"] == mode
    E = 8
    w = load_expert_weights(EXPORT, f"layers.{layer}.ffn.experts", E, verify=True, prepare=False)
    assert (w.hidden, w.inter, w.group, w.fmt, w.n_experts, w.act) == (128, 128, 128, fmt, E, act)
    assert len(w.w13_packed) == k_terms and w.w13_scale[0].dtype == scale_dtype
    for i in range(k_terms):
        for e in range(E):
            pre = f"layers.{layer}.ffn.experts.{e}"
            gate_p, up_p, down_p = (_weightstore(f"{pre}.{n}.tq{i}.packed") for n in ("w1", "w3", "w2"))
            gate_s, up_s, down_s = (_weightstore(f"{pre}.{n}.tq{i}.scale") for n in ("w1", "w3", "w2"))
            assert np.array_equal(w.w13_packed[i][e].numpy(), np.concatenate([gate_p, up_p]))
            assert np.array_equal(w.w2_packed[i][e].numpy(), down_p)
            assert np.array_equal(w.w13_scale[i][e].view(torch.int16).numpy().view(np.uint16), np.concatenate([gate_s, up_s]))
            assert np.array_equal(w.w2_scale[i][e].view(torch.int16).numpy().view(np.uint16), down_s)
    # a rank's shard
    part = load_expert_weights(EXPORT, f"layers.{layer}.ffn.experts", 2, first_expert=6, prepare=False)
    assert torch.equal(part.w2_packed[0], w.w2_packed[0][6:])


def _export_experts(layer, k_terms, fmt, scale_dtype):
    """The export's experts of one layer as oracle term lists (scales as float16, or float32 for bf16 scales)."""
    def sc(bits):
        t = torch.from_numpy(bits.view(np.int16).copy()).view(scale_dtype)
        return t.numpy() if scale_dtype == torch.float16 else t.float().numpy()

    return [tuple([(_weightstore(f"layers.{layer}.ffn.experts.{e}.{n}.tq{i}.packed"),
                    sc(_weightstore(f"layers.{layer}.ffn.experts.{e}.{n}.tq{i}.scale"))) for i in range(k_terms)]
                  for n in ("w1", "w2", "w3")) for e in range(8)]


@pytest.mark.gpu
@pytest.mark.parametrize("layer,mode,k_terms,fmt,scale_dtype,act", EXPORT_LAYERS)
def test_reference_written_export_runs_the_moe_layer(layer, mode, k_terms, fmt, scale_dtype, act):
    """Mode C and Mode D layers of the reference-written export through the loader and the layer, against the oracle
    on the tensors the reference's reader returned (the bf16-scale layer stays canonical and runs on the generic kernel)."""
    from deepseekternarized_b200.kernels import ternary_b200 as kb
    from deepseekternarized_b200.loader import load_expert_weights
    from deepseekternarized_b200.moe import MoELayer

    E, hidden, inter, group, topk, T = 8, 128, 128, 128, 2, 300
    w = load_expert_weights(EXPORT, f"layers.{layer}.ffn.experts", E, device="cuda", verify=True)
    assert isinstance(w.w13_packed[0], kb.TiledWeights) == (scale_dtype == torch.float16)
    rng = np.random.default_rng(80 + layer)
    x = O.synth_acts(rng, (T, hidden))
    logits = rng.standard_normal((T, E)).astype(np.float32)
    y = MoELayer(w, topk)(bf16_tensor(x, "cuda"), torch.from_numpy(logits).to("cuda"))
    experts = _export_experts(layer, k_terms, fmt, scale_dtype)
    wr, idx = O.route_from_logits(logits, topk)
    check_layer(bf16_numpy(y), O.moe_layer(x, wr, idx, experts, hidden, inter, group, fmt),
                O.moe_layer_f64(x, wr, idx, experts, hidden, inter, group, fmt))
