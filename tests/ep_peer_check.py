"""Run as a rank of a torch.distributed job on CUDA (world size >= 1): the expert-parallel layer with the peer-memory
transport must equal the single-device layer on the same global problem, bit for bit. Prints one line per job.

Used by tests/test_gpu_parity.py (one process, world size 1) and by hand under torchrun on several GPUs:
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 tests/ep_peer_check.py
"""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from deepseekternarized_b200.moe import ExpertParallelMoE, ExpertWeights, MoELayer  # noqa: E402
from oracle import oracle as O  # noqa: E402
from tests.helpers import bf16_tensor, make_experts, stack_experts  # noqa: E402


def main():
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    T, hidden, inter, E, topk, group, fmt = 768, 512, 256, 16, 6, 128, "tq1"
    rng = np.random.default_rng(5)
    experts = make_experts(rng, E, hidden, inter, group, fmt, 1)
    x = O.synth_acts(rng, (T, hidden))
    logits = rng.standard_normal((T, E)).astype(np.float32)
    logits[:, 7] = -40.0  # an expert nobody routes to
    El, tl = E // world, T // world
    w_local = ExpertWeights(*stack_experts(experts[rank * El:(rank + 1) * El], 1, dev), hidden, inter, group, fmt).prepare()
    ok = True
    # both ways back of the peer transport (the second GEMM scattering its rows to the tokens' ranks; the rows pulled from
    # the owners), then NCCL all-to-all
    for transport, combine in (("peer", "scatter"), ("peer", "pull"), ("nccl", "auto")):
        ep = ExpertParallelMoE(w_local, E, topk, transport=transport, combine=combine)
        for step in range(3):  # both buffer sets of the peer transport, and a reuse
            y = ep(bf16_tensor(x[rank * tl:(rank + 1) * tl], dev), torch.from_numpy(logits[rank * tl:(rank + 1) * tl]).to(dev))
        ys = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(ys, y)
        if rank == 0:
            w_all = ExpertWeights(*stack_experts(experts, 1, dev), hidden, inter, group, fmt).prepare()
            y1 = MoELayer(w_all, topk)(bf16_tensor(x, dev), torch.from_numpy(logits).to(dev))
            same = torch.equal(torch.cat(ys), y1)
            ok = ok and same
            print(f"transport {transport} ({combine}): world {world}, identical to the single-device layer: {same}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("EP_PEER_CHECK", "PASS" if ok else "FAIL", flush=True)
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
