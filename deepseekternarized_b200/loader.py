"""Manifest-driven loader: routed-expert weights of a Boilerplate export -> the stacked device layout.

A Boilerplate-format directory (``docs/architecture/format.md`` of the reference, section "manifest.json")
holds ``manifest.json`` and safetensors shards. A Mode C weight (k stacked terms) or Mode D weight (one QAT-trained
term; the exporter writes ``"mode": rule.mode`` for both, ``boilerplate/format/export.py:202-234``, and the engine reads
both through the same branch, ``boilerplate/engine/model.py:364``) ``X`` is stored per term ``i`` as
``X.tq{i}.packed`` uint8 ``[N, ceil(K / per_byte)]`` and ``X.tq{i}.scale`` fp16/bf16 ``[N, ceil(K / group)]``
(``format.md:87-92``); its manifest entry names the packing, the number of terms, the group, the scale type
and, per stored tensor, the shard file and a SHA-256 of its bytes (``format.md:108-134``). The reference reads
them one tensor at a time through ``WeightStore.get`` (``boilerplate/engine/weights.py:115-132,139-``) and builds
one ``TernaryLinear`` per expert and projection (``engine/model.py:365-366``).

Here the experts of one MoE layer are read straight into the stacked ``[E, N, Kp]`` tensors the grouped kernels
take (gate and up projections stacked along N), one stack per term, and re-laid-out once on the device.
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch

from .moe import ExpertWeights

_PER_BYTE = {"tq1": 5, "tq2": 4}


class ManifestError(ValueError):
    """The export does not hold what the caller asked for (missing weight, wrong mode, inconsistent experts)."""


def _read(root: Path, file: str, name: str, cache: dict) -> torch.Tensor:
    from safetensors import safe_open

    if file not in cache:
        cache[file] = safe_open(str(root / file), framework="pt", device="cpu")
    return cache[file].get_tensor(name)


def _entry(manifest: dict, base: str) -> dict:
    meta = manifest["tensors"].get(base)
    if meta is None:
        raise ManifestError(f"{base}: not in the manifest")
    if meta.get("mode") not in ("C", "D"):
        raise ManifestError(f"{base}: mode {meta.get('mode')!r}, the ternary backend takes Mode C (stacked ternary) and "
                            "Mode D (single ternary term) weights")
    if meta.get("packing") not in _PER_BYTE:
        raise ManifestError(f"{base}: unknown packing {meta.get('packing')!r}")
    return meta


def _terms(root: Path, manifest: dict, base: str, cache: dict, verify: bool):
    """[(packed [N, Kp] uint8, scale [N, G])] of weight ``base`` plus its manifest entry."""
    meta = _entry(manifest, base)
    N, K = (int(v) for v in meta["shape"])
    per, group = _PER_BYTE[meta["packing"]], int(meta["group"])
    out = []
    for i in range(int(meta["terms"])):
        pair = []
        for suffix, shape in ((f"{base}.tq{i}.packed", (N, -(-K // per))), (f"{base}.tq{i}.scale", (N, -(-K // group)))):
            stored = meta["stored"].get(suffix)
            if stored is None:
                raise ManifestError(f"{suffix}: not listed under {base}")
            t = _read(root, stored["file"], suffix, cache)
            if tuple(t.shape) != shape or tuple(int(v) for v in stored["shape"]) != shape:
                raise ManifestError(f"{suffix}: shape {tuple(t.shape)}, expected {shape}")
            if verify and "sha256" in stored:
                raw = t.contiguous().view(torch.uint8).numpy().tobytes()
                if hashlib.sha256(raw).hexdigest() != stored["sha256"]:
                    raise ManifestError(f"{suffix}: SHA-256 mismatch")
            pair.append(t)
        if pair[0].dtype != torch.uint8:
            raise ManifestError(f"{base}.tq{i}.packed: dtype {pair[0].dtype}, expected uint8")
        out.append(tuple(pair))
    return out, meta


def load_expert_weights(root, experts_prefix: str, n_experts: int, device=None, first_expert: int = 0,
                        names=("w1", "w2", "w3"), verify: bool = False, prepare: bool = True) -> ExpertWeights:
    """Experts ``first_expert .. first_expert + n_experts - 1`` of one MoE layer as stacked ``ExpertWeights``.

    ``experts_prefix``: e.g. ``"layers.3.ffn.experts"``; the weights are ``{prefix}.{e}.{w1|w2|w3}`` (gate, down, up:
    ``boilerplate/engine/model.py:365-387``; pass ``names=("gate_proj", "down_proj", "up_proj")`` for the standard
    engine's naming, ``engine/standard.py:130-133``). ``first_expert`` / ``n_experts`` select a rank's shard for
    expert parallelism. ``verify`` checks every tensor's SHA-256 against the manifest. With ``prepare`` (and a CUDA
    ``device``) the packed stacks are re-laid-out once into the tiled device layout (fp16 scales; bf16 scales stay
    canonical and run on the generic kernel). The returned object carries the manifest's ``act`` entry as ``.act``.
    """
    root = Path(root)
    mpath = root / "manifest.json"
    if not mpath.exists():
        raise ManifestError(f"{mpath}: no manifest (not a Boilerplate-format directory)")
    manifest = json.loads(mpath.read_text())
    cache: dict = {}
    g_name, d_name, u_name = names
    stacks = None  # per term: (w13 packed rows, w13 scales, w2 packed, w2 scales), one list entry per expert
    ref = None
    for e in range(first_expert, first_expert + n_experts):
        got = {w: _terms(root, manifest, f"{experts_prefix}.{e}.{w}", cache, verify) for w in names}
        gate, gm = got[g_name]
        down, dm = got[d_name]
        up, um = got[u_name]
        key = (gm["packing"], int(gm["group"]), int(gm["terms"]), tuple(gm["shape"]), tuple(dm["shape"]), gm.get("scale_dtype"),
               gm.get("act"))
        for m in (dm, um):
            if (m["packing"], int(m["group"]), int(m["terms"])) != key[:3]:
                raise ManifestError(f"{experts_prefix}.{e}: projections differ in packing, group or number of terms")
        if tuple(um["shape"]) != tuple(gm["shape"]) or tuple(dm["shape"]) != (gm["shape"][1], gm["shape"][0]):
            raise ManifestError(f"{experts_prefix}.{e}: projection shapes do not form a SwiGLU FFN")
        if ref is None:
            ref = key
            stacks = [([], [], [], []) for _ in range(key[2])]
        elif key != ref:
            raise ManifestError(f"{experts_prefix}.{e}: differs from expert {first_expert} in format or shape")
        for i in range(key[2]):
            stacks[i][0].append(torch.cat([gate[i][0], up[i][0]]))
            stacks[i][1].append(torch.cat([gate[i][1], up[i][1]]))
            stacks[i][2].append(down[i][0])
            stacks[i][3].append(down[i][1])
    if ref is None:
        raise ManifestError("no experts requested")
    fmt, group, _, (inter, hidden), _, _, act = ref
    dev = torch.device(device) if device is not None else torch.device("cpu")
    w = ExpertWeights([torch.stack(s[0]).to(dev) for s in stacks], [torch.stack(s[1]).to(dev) for s in stacks],
                      [torch.stack(s[2]).to(dev) for s in stacks], [torch.stack(s[3]).to(dev) for s in stacks],
                      int(hidden), int(inter), group, fmt)
    w.act = act  # the manifest's activation mode of these weights ("int8" or "bf16", boilerplate/format/policy.py:73), for the caller
    return w.prepare() if prepare and dev.type == "cuda" else w
