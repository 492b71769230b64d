"""Expert-parallel host logic on two CPU ranks (gloo): dispatch / combine bookkeeping of
``ExpertParallelMoE`` with the compute steps supplied by the CPU oracle. The result must equal the
single-process layer over all tokens (same summation order per token), bit for bit."""

from __future__ import annotations

import os
import socket
import tempfile

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as O
from tests.helpers import OracleOps, bf16_tensor, make_experts, stack_experts

T_TOTAL, HIDDEN, INTER, E, TOPK, GROUP = 24, 256, 128, 8, 3, 128


def _inputs(fmt, k_terms):
    rng = np.random.default_rng(77)
    experts = make_experts(rng, E, HIDDEN, INTER, GROUP, fmt, k_terms)
    x = O.synth_acts(rng, (T_TOTAL, HIDDEN))
    logits = rng.standard_normal((T_TOTAL, E)).astype(np.float32)
    logits[:, 5] = -30.0  # expert 5 receives nothing
    return experts, x, logits


def _worker(rank, world, port, fmt, k_terms, outdir):
    from deepseekternarized_b200.moe import ExpertParallelMoE, ExpertWeights

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        experts, x, logits = _inputs(fmt, k_terms)
        El = E // world
        mine = experts[rank * El:(rank + 1) * El]
        w = ExpertWeights(*stack_experts(mine, k_terms), HIDDEN, INTER, GROUP, fmt)
        layer = ExpertParallelMoE(w, E, TOPK, ops=OracleOps())
        # uneven token split: rank 0 gets 10 tokens, rank 1 the other 14
        lo, hi = (0, 10) if rank == 0 else (10, T_TOTAL)
        y = layer(bf16_tensor(x[lo:hi]), torch.from_numpy(logits[lo:hi]))
        np.save(os.path.join(outdir, f"y{rank}.npy"), y.float().numpy())
        np.save(os.path.join(outdir, f"rows{rank}.npy"), np.array(layer.last_dispatch_rows))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fmt,k_terms", [("tq1", 1), ("tq2", 2)])
def test_two_rank_expert_parallel_equals_single_process(fmt, k_terms):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_worker, args=(2, port, fmt, k_terms, d), nprocs=2, join=True)
        y = np.concatenate([np.load(os.path.join(d, f"y{r}.npy")) for r in range(2)])
        rows = sum(int(np.load(os.path.join(d, f"rows{r}.npy"))) for r in range(2))
    experts, x, logits = _inputs(fmt, k_terms)
    w, idx = O.route_from_logits(logits, TOPK)
    want = O.moe_layer(x, w, idx, experts, HIDDEN, INTER, GROUP, fmt)
    assert rows == T_TOTAL * TOPK
    assert np.array_equal(y, want)


def test_single_process_layer_with_oracle_ops_equals_oracle_layer():
    """The sort/gather/grouped/combine decomposition itself, against the per-expert loop of the reference layer."""
    from deepseekternarized_b200.moe import ExpertWeights, MoELayer

    experts, x, logits = _inputs("tq1", 1)
    w = ExpertWeights(*stack_experts(experts, 1), HIDDEN, INTER, GROUP, "tq1")
    y = MoELayer(w, TOPK, ops=OracleOps())(bf16_tensor(x), torch.from_numpy(logits))
    wts, idx = O.route_from_logits(logits, TOPK)
    want = O.moe_layer(x, wts, idx, experts, HIDDEN, INTER, GROUP, "tq1")
    assert np.array_equal(y.float().numpy(), want)


def test_uneven_expert_split_is_refused():
    from deepseekternarized_b200.moe import expert_owner_split

    assert expert_owner_split(384, 8) == 48
    with pytest.raises(ValueError):
        expert_owner_split(10, 4)


@pytest.mark.parametrize("name", ["sigmoid", "sqrtsoftplus", "softmax_limit"])
def test_layer_options_with_oracle_ops_equal_the_reference_fixture(golden, name):
    """The layer's host logic for the V4 engine's options (score functions, gate bias, temperature, renormalisation
    switch, route_scale, SwiGLU clamp, shared expert, and the entry that takes the engine's own routing) on CPU with
    the oracle as compute: the output must be the oracle layer's, which the fixture pins to the reference's V4Model.moe."""
    from deepseekternarized_b200.moe import ExpertWeights, MoELayer
    from tests.test_oracle_golden import variant_case

    c = variant_case(golden("moe_layer_variants"), name)
    args = (c["hidden"], c["inter"], c["group"], c["fmt"])
    w = ExpertWeights(*stack_experts(c["experts"], c["k_terms"]), *args)
    shared = ExpertWeights(*stack_experts([c["shared"]], c["k_terms"]), *args) if c["shared"] is not None else None
    bias = torch.from_numpy(c["bias"]) if c["bias"] is not None else None
    layer = MoELayer(w, c["topk"], route_scale=c["route_scale"], swiglu_limit=c["limit"], ops=OracleOps(), norm_topk_prob=c["norm"],
                     score_func=c["score_func"], gate_bias=bias, gate_temp=c["gate_temp"], shared=shared)
    want = O.moe_layer(c["x"], c["weights"], c["indices"], c["experts"], *args, swiglu_limit=c["limit"], shared=c["shared"])
    y = layer(bf16_tensor(c["x"]), torch.from_numpy(c["logits"]))
    assert O.rel_fro(y.float().numpy(), want) < 2e-3  # the routing weights are recomputed here: last-bit differences allowed
    y2 = layer.forward_routed(bf16_tensor(c["x"]), torch.from_numpy(c["weights"]), torch.from_numpy(c["indices"]))
    assert np.array_equal(y2.float().numpy(), want)
    assert np.mean(O.bf16_bits(want) != c["y_bits"]) < 0.02
