"""Generates the golden fixtures in this folder by running the REFERENCE project's own code.

Run it where the reference tree is mounted (it cannot travel with the fixtures)::

    CXX=/usr/bin/g++ CC=/usr/bin/gcc TORCH_EXTENSIONS_DIR=/tmp/dst_ref_ext \
        PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --reference <path of the reference tree> \
        [--only format,linear,int8,grouped,moe,moe_standard,moe_variants,tables,baseline,export]

(``--only`` regenerates the named fixture files and leaves the others as they are; the path may also come from the
environment variable ``REFERENCE_ROOT``.)

Every expectation is produced by reference functions, unmodified, imported from that tree:
``boilerplate.ternary.pack`` (pack/unpack/LUT), ``boilerplate.ternary.ops`` (TernaryLinear with
act="bf16", backend="cpp"; quant_act_int8), ``boilerplate.kernels.ternary_cuda`` (ternary_gemm_ref,
grouped_ternary_gemm, sort_by_expert), the C++ kernel ``boilerplate.kernels.cpu.ext().ternary_gemm``
and ``boilerplate.engine.model.V4Model`` (route / swiglu / moe, called on a stand-in object that
carries only the attributes those three methods read) and ``boilerplate.engine.standard.StandardDecoder._moe``
(the OLMoE-style layer, on a stand-in likewise). ``export_tiny/`` is a whole Boilerplate-format directory written by
``boilerplate.format.export.export`` from the reference's own tiny random-init checkpoint
(``boilerplate.testing.tiny.write_tiny_checkpoint``) under a policy with one Mode C (k = 2) and one Mode D rule,
with the tensors the reference's ``WeightStore`` hands back for two of its experts stored beside it.

Inputs come from numpy generators with fixed seeds so the tests can rebuild them without the
reference; the fixtures hold the inputs that are cheap to store and every expected output
(large outputs as SHA-256 plus a strided sample).
"""

from __future__ import annotations

import argparse
import hashlib
import itertools
import os
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def trits_of(rng, shape):
    u = rng.random(shape)
    return np.where(u < 0.4, 0, np.where(u < 0.7, 1, -1)).astype(np.int8)


def scales_of(rng, shape):
    return np.exp(rng.normal(-4.0, 0.3, shape)).astype(np.float16)


def acts_of(rng, shape):
    return torch.from_numpy(rng.standard_normal(shape).astype(np.float32)).bfloat16()


def bits(t_bf16: torch.Tensor) -> np.ndarray:
    return t_bf16.view(torch.int16).numpy().view(np.uint16)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("REFERENCE_ROOT"), help="root of the reference project's tree")
    ap.add_argument("--only", default="", help="comma-separated fixture sections to regenerate (default: all)")
    args = ap.parse_args()
    if not args.reference:
        raise SystemExit("make_golden.py: pass --reference <tree> or set REFERENCE_ROOT")
    only = {v for v in args.only.split(",") if v}

    def want(section):
        return not only or section in only

    os.environ.setdefault("CXX", "/usr/bin/g++")
    os.environ.setdefault("CC", "/usr/bin/gcc")
    os.environ.setdefault("TORCH_EXTENSIONS_DIR", "/tmp/dst_ref_ext")
    sys.dont_write_bytecode = True
    sys.path.insert(0, args.reference)

    from boilerplate.engine.model import V4Model
    from boilerplate.engine.standard import StandardDecoder
    from boilerplate.kernels.cpu import ext
    from boilerplate.kernels.ternary_cuda import grouped_ternary_gemm, sort_by_expert, ternary_gemm, ternary_gemm_ref
    from boilerplate.ternary.ops import PackedTerm, TernaryLinear, quant_act_int8
    from boilerplate.ternary.pack import _TQ1_LUT, pack, packed_cols, unpack

    cpp = ext()
    assert cpp is not None, "reference C++ extension did not build"
    torch.set_num_threads(max(1, os.cpu_count() or 1))

    # ---------------------------------------------------------------- 1. format
    def sec_format():
        fmt_out = {"tq1_lut": _TQ1_LUT.numpy()}
        rng = np.random.default_rng(1001)
        for fmt in ("tq2", "tq1"):
            for K in (1, 4, 5, 7, 128, 131, 640):
                t = trits_of(rng, (9, K))
                p = pack(torch.from_numpy(t), fmt)
                assert tuple(p.shape) == (9, packed_cols(fmt, K))
                assert torch.equal(unpack(p, fmt, K), torch.from_numpy(t))
                fmt_out[f"trits_{fmt}_{K}"] = t
                fmt_out[f"packed_{fmt}_{K}"] = p.numpy()
        pats = np.array(list(itertools.product([-1, 0, 1], repeat=5)), dtype=np.int8)
        fmt_out["tq1_patterns"] = pats
        fmt_out["tq1_patterns_packed"] = pack(torch.from_numpy(pats), "tq1").numpy()
        allb = torch.arange(256, dtype=torch.uint8).view(256, 1)
        fmt_out["unpack_all_bytes_tq1"] = unpack(allb, "tq1", 5).numpy()
        fmt_out["unpack_all_bytes_tq2"] = unpack(allb, "tq2", 4).numpy()
        np.savez_compressed(HERE / "format.npz", **fmt_out)

    if want("format"):
        sec_format()

    # ---------------------------------------------------------------- 2. linear, float activations, k terms
    def sec_linear():
        lin_out = {}
        case = 0
        for fmt in ("tq2", "tq1"):
            for (K, group, N, M, k_terms) in [(256, 128, 37, 15, 2), (640, 128, 37, 15, 2), (200, 64, 37, 15, 2),
                                              (1024, 256, 37, 15, 2), (4160, 128, 70, 3, 1), (130, 128, 24, 5, 1),
                                              (300, 64, 24, 5, 1), (2048, 128, 64, 8, 2)]:
                rng = np.random.default_rng(2000 + case)
                terms = []
                for i in range(k_terms):
                    t = trits_of(rng, (N, K))
                    s = scales_of(rng, (N, -(-K // group)))
                    if i == 1:
                        s = (s.astype(np.float32) * 0.25).astype(np.float16)
                    if case % 3 == 0:
                        s[0, 0] = 0  # an all-zero group scale is legal (fit.py:46-48)
                    terms.append((t, s))
                x = acts_of(rng, (M, K))
                lin = TernaryLinear([PackedTerm(pack(torch.from_numpy(t), fmt), torch.from_numpy(s)) for t, s in terms],
                                    K, fmt, group, act="bf16", backend="cpp")
                y32 = lin(x, out_dtype=torch.float32)
                ybf = lin(x)  # default bf16 output
                ydq = TernaryLinear(lin.terms, K, fmt, group, act="bf16", backend="torch")(x, out_dtype=torch.float32)
                torch.testing.assert_close(y32, ydq, rtol=1e-4, atol=1e-3)
                pre = f"c{case}_"
                lin_out[pre + "meta"] = np.array([K, group, N, M, k_terms, 2 if fmt == "tq2" else 1], np.int64)
                lin_out[pre + "x_bits"] = bits(x)
                for i, (t, s) in enumerate(terms):
                    lin_out[pre + f"packed{i}"] = lin.terms[i].packed.numpy()
                    lin_out[pre + f"scale{i}"] = s
                lin_out[pre + "y_f32"] = y32.numpy()
                lin_out[pre + "y_bf16_bits"] = bits(ybf)
                case += 1
        lin_out["n_cases"] = np.array(case)
        np.savez_compressed(HERE / "linear_f32.npz", **lin_out)

    if want("linear"):
        sec_linear()

    # ---------------------------------------------------------------- 3. int8 activations
    def sec_int8():
        i8_out = {}
        case = 0
        for fmt in ("tq1", "tq2"):
            for (K, group, N, M) in [(256, 128, 24, 5), (300, 64, 24, 5), (130, 128, 24, 5), (4160, 128, 70, 3)]:
                rng = np.random.default_rng(3000 + case)
                t = trits_of(rng, (N, K))
                s = (rng.random((N, -(-K // group))).astype(np.float16).astype(np.float32) + np.float32(0.01))
                xf = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32) * 3)
                q, xs = quant_act_int8(xf)
                p = pack(torch.from_numpy(t), fmt)
                ref = ternary_gemm_ref(q, xs, p, torch.from_numpy(s), K, group, fmt)
                got = ternary_gemm(q, xs, p, torch.from_numpy(s), K, group, fmt, backend="cpp")
                pre = f"c{case}_"
                i8_out[pre + "meta"] = np.array([K, group, N, M, 2 if fmt == "tq2" else 1], np.int64)
                i8_out[pre + "x_f32"] = xf.numpy()
                i8_out[pre + "q"] = q.numpy()
                i8_out[pre + "xs"] = xs.numpy()
                i8_out[pre + "packed"] = p.numpy()
                i8_out[pre + "scale_f32"] = s
                i8_out[pre + "y_ref"] = ref.numpy()
                i8_out[pre + "y_cpp"] = got.numpy()
                case += 1
        i8_out["n_cases"] = np.array(case)
        np.savez_compressed(HERE / "linear_i8.npz", **i8_out)

    if want("int8"):
        sec_int8()

    # ---------------------------------------------------------------- 4. grouped + routing sort
    def sec_grouped():
        g_out = {}
        for ci, fmt in enumerate(("tq1", "tq2")):
            E, N, K, group, T, k = 6, 16, 192, 64, 9, 2
            rng = np.random.default_rng(4000 + ci)
            t = trits_of(rng, (E, N, K))
            s = (rng.random((E, N, K // group)).astype(np.float16).astype(np.float32) + np.float32(0.01))
            packed = torch.stack([pack(torch.from_numpy(t[e]), fmt) for e in range(E)])
            xf = torch.from_numpy(rng.standard_normal((T, K)).astype(np.float32))
            q, xs = quant_act_int8(xf)
            ids = np.stack([rng.permutation(E)[:k] for _ in range(T)]).reshape(-1).astype(np.int64)
            ids[ids == 5] = 4  # expert 5 stays empty
            order, offsets = sort_by_expert(torch.from_numpy(ids), E)
            rows = order // k
            out = grouped_ternary_gemm(q[rows], xs[rows], offsets, packed, torch.from_numpy(s), K, group, fmt, backend="cpp")
            pre = f"{fmt}_"
            g_out[pre + "packed"] = packed.numpy()
            g_out[pre + "scale_f32"] = s
            g_out[pre + "q"] = q.numpy()
            g_out[pre + "xs"] = xs.numpy()
            g_out[pre + "ids"] = ids
            g_out[pre + "order"] = order.numpy()
            g_out[pre + "offsets"] = offsets.numpy()
            g_out[pre + "out"] = out.numpy()
        np.savez_compressed(HERE / "grouped.npz", **g_out)

    if want("grouped"):
        sec_grouped()

    # ---------------------------------------------------------------- 5. MoE layer (V4 flavour)
    def sec_moe():
        m_out = {}
        for ci, (fmt, k_terms) in enumerate((("tq1", 1), ("tq2", 2))):
            T, hidden, inter, E, topk, group = 24, 256, 128, 8, 2, 128
            rng = np.random.default_rng(5000 + ci)
            x = acts_of(rng, (T, hidden))
            gate_w = torch.from_numpy(rng.standard_normal((E, hidden)).astype(np.float32) * 0.2)

            def make(Nw, Kw):
                terms = []
                for i in range(k_terms):
                    t = trits_of(rng, (Nw, Kw))
                    s = scales_of(rng, (Nw, Kw // group))
                    if i == 1:
                        s = (s.astype(np.float32) * 0.25).astype(np.float16)
                    terms.append((pack(torch.from_numpy(t), fmt).numpy(), s))
                return terms

            experts = [(make(inter, hidden), make(hidden, inter), make(inter, hidden)) for _ in range(E)]  # w1, w2, w3

            def lin(terms, Kw):
                return TernaryLinear([PackedTerm(torch.from_numpy(p), torch.from_numpy(s)) for p, s in terms], Kw, fmt, group,
                                     act="bf16", backend="cpp")

            built = [(lin(w1, hidden), lin(w2, inter), lin(w3, hidden)) for w1, w2, w3 in experts]
            cfg = types.SimpleNamespace(dim=hidden, n_routed_experts=E, n_activated_experts=topk, score_func="softmax",
                                        norm_topk_prob=True, route_scale=1.0, swiglu_limit=0.0, gate_temp=1.0)
            zero = (lambda v: torch.zeros(*v.shape[:-1], inter, dtype=torch.bfloat16),
                    lambda v: torch.zeros(*v.shape[:-1], hidden, dtype=torch.bfloat16),
                    lambda v: torch.zeros(*v.shape[:-1], inter, dtype=torch.bfloat16))
            L = types.SimpleNamespace(gate_w=gate_w, gate_b=None, shared=zero, expert_prefix="e")
            fake = types.SimpleNamespace(cfg=cfg, routing_capture=None,
                                         expert_cache=types.SimpleNamespace(touch=lambda key: None))
            fake.route = types.MethodType(V4Model.route, fake)
            fake.swiglu = types.MethodType(V4Model.swiglu, fake)
            fake.expert = lambda L_, e: built[e]
            weights, indices = fake.route(L, x)
            y = V4Model.moe(fake, L, x)
            pre = f"{fmt}_"
            m_out[pre + "meta"] = np.array([T, hidden, inter, E, topk, group, k_terms], np.int64)
            m_out[pre + "x_bits"] = bits(x)
            m_out[pre + "gate_w"] = gate_w.numpy()
            for e, ws in enumerate(experts):
                for wi, terms in zip(("w1", "w2", "w3"), ws):
                    for i, (p, s) in enumerate(terms):
                        m_out[pre + f"e{e}_{wi}_packed{i}"] = p
                        m_out[pre + f"e{e}_{wi}_scale{i}"] = s
            m_out[pre + "route_weights"] = weights.numpy()
            m_out[pre + "route_indices"] = indices.numpy()
            m_out[pre + "y_bits"] = bits(y)
        np.savez_compressed(HERE / "moe_layer.npz", **m_out)

    if want("moe"):
        sec_moe()

    # ---------------------------------------------------------------- 5b. MoE layer (standard / OLMoE flavour)
    def sec_moe_standard():
        s_out = {}
        for ci, (fmt, k_terms, renorm) in enumerate((("tq1", 1, True), ("tq2", 2, False))):
            T, hidden, inter, E, topk, group = 24, 256, 128, 8, 2, 128
            rng = np.random.default_rng(5500 + ci)
            x = acts_of(rng, (T, hidden))
            gate_w = torch.from_numpy(rng.standard_normal((E, hidden)).astype(np.float32) * 0.2)

            def make_s(Nw, Kw):
                terms = []
                for i in range(k_terms):
                    t = trits_of(rng, (Nw, Kw))
                    s = scales_of(rng, (Nw, Kw // group))
                    if i == 1:
                        s = (s.astype(np.float32) * 0.25).astype(np.float16)
                    terms.append((pack(torch.from_numpy(t), fmt).numpy(), s))
                return terms

            experts = [(make_s(inter, hidden), make_s(hidden, inter), make_s(inter, hidden)) for _ in range(E)]  # gate, down, up

            def lin_s(terms, Kw):
                return TernaryLinear([PackedTerm(torch.from_numpy(p), torch.from_numpy(s)) for p, s in terms], Kw, fmt, group,
                                     act="bf16", backend="cpp")

            built = [(lin_s(w1, hidden), lin_s(w3, hidden), lin_s(w2, inter)) for w1, w2, w3 in experts]  # (gate, up, down)
            logits = x.float() @ gate_w.T
            fake = types.SimpleNamespace(hidden=hidden, config={"num_experts_per_tok": topk, "norm_topk_prob": renorm, "num_experts": E},
                                         expert_cache=types.SimpleNamespace(get=lambda key, factory: built[key[1]], touch=lambda key: None))
            fake._run_mlp = StandardDecoder._run_mlp
            layer = types.SimpleNamespace(prefix="l", router=lambda v: logits)
            routing = []
            y = StandardDecoder._moe(fake, layer, x, routing)
            pre = f"{fmt}_"
            s_out[pre + "meta"] = np.array([T, hidden, inter, E, topk, group, k_terms, int(renorm)], np.int64)
            s_out[pre + "x_bits"] = bits(x)
            s_out[pre + "logits"] = logits.numpy()
            for e, ws in enumerate(experts):
                for wi, terms in zip(("w1", "w2", "w3"), ws):
                    for i, (p, s) in enumerate(terms):
                        s_out[pre + f"e{e}_{wi}_packed{i}"] = p
                        s_out[pre + f"e{e}_{wi}_scale{i}"] = s
            s_out[pre + "route_indices"] = routing[0].numpy()
            s_out[pre + "y_bits"] = bits(y)
        np.savez_compressed(HERE / "moe_layer_standard.npz", **s_out)

    if want("moe_standard"):
        sec_moe_standard()

    # ---------------------------------------------------------------- 5c. ternary lookup-table rows (engram tables)
    def sec_tables():
        # the expression of boilerplate/engine/model.py:458-464 with the reference's own unpack
        t_out = {}
        for ci, (fmt, k_terms, K, group) in enumerate((("tq1", 1, 192, 64), ("tq2", 2, 203, 128))):
            rng = np.random.default_rng(5800 + ci)
            V = 50
            terms = []
            for i in range(k_terms):
                t = trits_of(rng, (V, K))
                s = scales_of(rng, (V, -(-K // group)))
                if i == 1:
                    s = (s.astype(np.float32) * 0.25).astype(np.float16)
                terms.append((pack(torch.from_numpy(t), fmt), torch.from_numpy(s)))
            ids = torch.from_numpy(rng.integers(0, V, (3, 7)))
            flat = ids.reshape(-1)
            vals = None
            for packed, sc in terms:
                t = unpack(packed.index_select(0, flat), fmt, K).float()
                v = t * sc.index_select(0, flat).float().repeat_interleave(group, -1)[:, :K]
                vals = v if vals is None else vals + v
            vals = vals.to(torch.bfloat16)
            pre = f"{fmt}_"
            t_out[pre + "meta"] = np.array([V, K, group, k_terms], np.int64)
            t_out[pre + "ids"] = ids.numpy()
            for i, (p, s) in enumerate(terms):
                t_out[pre + f"packed{i}"] = p.numpy()
                t_out[pre + f"scale{i}"] = s.numpy()
            t_out[pre + "vals_bits"] = bits(vals)
        np.savez_compressed(HERE / "table_rows.npz", **t_out)

    if want("tables"):
        sec_tables()

    # ---------------------------------------------------------------- 6. BASELINE config-0/1 shapes (hash + sample)
    def sec_baseline():
        big = {}
        for ci, (fmt, N, K, M) in enumerate([("tq2", 4096, 4096, 1), ("tq2", 4096, 4096, 16), ("tq1", 4096, 4096, 1),
                                             ("tq1", 2048, 4096, 4), ("tq1", 11008, 4096, 8)]):
            rng = np.random.default_rng(6000 + ci)
            t = trits_of(rng, (N, K))
            s = scales_of(rng, (N, K // 128))
            x = acts_of(rng, (M, K))
            p = pack(torch.from_numpy(t), fmt)
            out = torch.zeros(M, N)
            cpp.ternary_gemm(out, x.float().contiguous(), torch.ones(M), p, torch.from_numpy(s).float().contiguous(), K, 128,
                             2 if fmt == "tq2" else 1, _TQ1_LUT)
            o = out.numpy()
            big[f"c{ci}_meta"] = np.array([2 if fmt == "tq2" else 1, N, K, M], np.int64)
            big[f"c{ci}_sha256"] = np.frombuffer(hashlib.sha256(o.tobytes()).digest(), np.uint8)
            big[f"c{ci}_packed_sha256"] = np.frombuffer(hashlib.sha256(p.numpy().tobytes()).digest(), np.uint8)
            big[f"c{ci}_sample"] = o.reshape(-1)[::61].copy()
        big["n_cases"] = np.array(5)
        np.savez_compressed(HERE / "baseline_shapes.npz", **big)

    if want("baseline"):
        sec_baseline()

    # ---------------------------------------------------------------- 5d. V4 layer variants: the other routers, clamp, shared expert
    def sec_moe_variants():
        v_out = {}
        variants = (
            # name, fmt, k_terms, score_func, bias, gate_temp, norm_topk_prob, route_scale, swiglu_limit, shared expert
            ("sigmoid", "tq1", 1, "sigmoid", True, 1.0, True, 1.5, 0.75, True),
            ("sqrtsoftplus", "tq2", 2, "sqrtsoftplus", True, 0.7, False, 2.5, 0.0, False),
            ("softmax_limit", "tq2", 1, "softmax", False, 1.3, True, 1.0, 0.5, True),
        )
        for ci, (name, fmt, k_terms, score_func, with_bias, gate_temp, norm, route_scale, limit, with_shared) in enumerate(variants):
            T, hidden, inter, E, topk, group = 24, 256, 128, 8, 3, 128
            rng = np.random.default_rng(5900 + ci)
            x = acts_of(rng, (T, hidden))
            gate_w = torch.from_numpy(rng.standard_normal((E, hidden)).astype(np.float32) * 0.2)
            gate_b = torch.from_numpy(rng.standard_normal(E).astype(np.float32) * 0.3) if with_bias else None

            def make(Nw, Kw):
                terms = []
                for i in range(k_terms):
                    t = trits_of(rng, (Nw, Kw))
                    s = scales_of(rng, (Nw, Kw // group))
                    if i == 1:
                        s = (s.astype(np.float32) * 0.25).astype(np.float16)
                    terms.append((pack(torch.from_numpy(t), fmt).numpy(), s))
                return terms

            experts = [(make(inter, hidden), make(hidden, inter), make(inter, hidden)) for _ in range(E)]  # w1, w2, w3
            shared = (make(inter, hidden), make(hidden, inter), make(inter, hidden)) if with_shared else None

            def lin(terms, Kw):
                return TernaryLinear([PackedTerm(torch.from_numpy(p), torch.from_numpy(s)) for p, s in terms], Kw, fmt, group,
                                     act="bf16", backend="cpp")

            built = [(lin(w1, hidden), lin(w2, inter), lin(w3, hidden)) for w1, w2, w3 in experts]
            cfg = types.SimpleNamespace(dim=hidden, n_routed_experts=E, n_activated_experts=topk, score_func=score_func,
                                        norm_topk_prob=norm, route_scale=route_scale, swiglu_limit=limit, gate_temp=gate_temp)
            zero = (lambda v: torch.zeros(*v.shape[:-1], inter, dtype=torch.bfloat16),
                    lambda v: torch.zeros(*v.shape[:-1], hidden, dtype=torch.bfloat16),
                    lambda v: torch.zeros(*v.shape[:-1], inter, dtype=torch.bfloat16))
            sh = (lin(shared[0], hidden), lin(shared[1], inter), lin(shared[2], hidden)) if with_shared else zero
            L = types.SimpleNamespace(gate_w=gate_w, gate_b=gate_b, shared=sh, expert_prefix="e")
            fake = types.SimpleNamespace(cfg=cfg, routing_capture=None,
                                         expert_cache=types.SimpleNamespace(touch=lambda key: None))
            fake.route = types.MethodType(V4Model.route, fake)
            fake.swiglu = types.MethodType(V4Model.swiglu, fake)
            fake.expert = lambda L_, e: built[e]
            weights, indices = fake.route(L, x)
            y = V4Model.moe(fake, L, x)
            pre = f"{name}_"
            v_out[pre + "meta"] = np.array([T, hidden, inter, E, topk, group, k_terms, 2 if fmt == "tq2" else 1, int(norm), int(with_shared)],
                                           np.int64)
            v_out[pre + "params"] = np.array([gate_temp, route_scale, limit], np.float64)
            v_out[pre + "score_func"] = np.array(score_func)
            v_out[pre + "x_bits"] = bits(x)
            v_out[pre + "logits"] = (x.float() @ gate_w.T).numpy()  # F.linear(x.float(), gate_w), before the temperature
            if with_bias:
                v_out[pre + "gate_b"] = gate_b.numpy()
            for e, ws in enumerate(experts + ([shared] if with_shared else [])):
                tag = f"e{e}" if e < E else "shared"
                for wi, terms in zip(("w1", "w2", "w3"), ws):
                    for i, (p, s) in enumerate(terms):
                        v_out[pre + f"{tag}_{wi}_packed{i}"] = p
                        v_out[pre + f"{tag}_{wi}_scale{i}"] = s
            v_out[pre + "route_weights"] = weights.numpy()
            v_out[pre + "route_indices"] = indices.numpy()
            v_out[pre + "y_bits"] = bits(y)
        v_out["names"] = np.array([v[0] for v in variants])
        np.savez_compressed(HERE / "moe_layer_variants.npz", **v_out)

    if want("moe_variants"):
        sec_moe_variants()

    # ---------------------------------------------------------------- 7. a Boilerplate-format export written by the reference
    def sec_export():
        import shutil
        import tempfile

        from boilerplate.engine.weights import WeightStore
        from boilerplate.format.export import export
        from boilerplate.format.policy import Policy
        from boilerplate.testing.tiny import tiny_config, write_tiny_checkpoint

        out = HERE / "export_tiny"
        if out.exists():
            shutil.rmtree(out)
        with tempfile.TemporaryDirectory() as tmp:
            src = write_tiny_checkpoint(Path(tmp) / "ckpt", tiny_config(), seed=3)
            policy = Policy.from_dict({
                "name": "golden-c-and-d", "default": {"mode": "A"},
                "rules": [
                    {"match": r"^layers\.3\.ffn\.experts\.\d+\.w[123]$", "mode": "C", "k": 2, "group": 128, "packing": "tq1",
                     "scale_dtype": "fp16", "act": "bf16"},
                    {"match": r"^layers\.4\.ffn\.experts\.\d+\.w[123]$", "mode": "D", "group": 128, "packing": "tq2",
                     "scale_dtype": "bf16", "act": "int8", "allow_larger": True},
                    {"match": r"^layers\.5\.ffn\.experts\.\d+\.w[123]$", "mode": "D", "group": 128, "packing": "tq1",
                     "scale_dtype": "fp16", "act": "bf16"},
                ]})
            export(src, out, policy, log=lambda *a: None)
        # what the reference's own reader hands back for the routed experts of the three layers
        ws = WeightStore(out)
        want_t = {}
        for layer, k_terms in ((3, 2), (4, 1), (5, 1)):
            for e in range(8):
                for w in ("w1", "w2", "w3"):
                    for i in range(k_terms):
                        for kind in ("packed", "scale"):
                            n = f"layers.{layer}.ffn.experts.{e}.{w}.tq{i}.{kind}"
                            t = ws.get(n)
                            want_t[n] = t.view(torch.int16).numpy().view(np.uint16) if t.dtype in (torch.bfloat16, torch.float16) else t.numpy()
        np.savez_compressed(out / "weightstore_tensors.npz", **want_t)

    if want("export"):
        sec_export()

    # SECTIONS_END
    print("wrote", sorted(str(p.relative_to(HERE)) for p in HERE.rglob("*") if p.is_file() and p.suffix in (".npz", ".safetensors", ".json")))


if __name__ == "__main__":
    main()
