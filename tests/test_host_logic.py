"""Host-side behaviour of the drop-in modules without a GPU: the error contract of the reference's
kernel backend (boilerplate/kernels/ternary_cuda.py, tests/test_ternary_cuda.py:60-66 of the reference)."""

from __future__ import annotations

import pytest
import torch

from deepseekternarized_b200.kernels import ternary_b200 as kb
from deepseekternarized_b200.ternary import ops, pack

NO_GPU = not torch.cuda.is_available()


def test_format_helpers():
    assert pack.packed_cols("tq2", 4096) == 1024 and pack.packed_cols("tq1", 4096) == 820
    assert pack.packed_cols("tq1", 2048) == 410 and pack.packed_cols("tq2", 1) == 1
    assert pack.bits_per_weight("tq1") == 1.6 and pack.bits_per_weight("tq2") == 2.0
    assert pack.FORMATS == ("tq2", "tq1")


def test_unknown_format_is_a_value_error():
    with pytest.raises(ValueError, match="unknown ternary packing"):
        kb.ternary_gemm(torch.zeros(1, 4, dtype=torch.int8), torch.ones(1), torch.zeros(2, 1, dtype=torch.uint8),
                        torch.ones(2, 1), 4, 4, "tq3")


def test_non_int8_activations_are_a_type_error():
    with pytest.raises(TypeError, match="int8"):
        kb.ternary_gemm(torch.zeros(1, 4), torch.ones(1), torch.zeros(2, 1, dtype=torch.uint8), torch.ones(2, 1), 4, 4, "tq2")
    with pytest.raises(TypeError, match="bf16"):
        kb.ternary_gemm_bf16(torch.zeros(1, 4), [torch.zeros(2, 1, dtype=torch.uint8)], [torch.ones(2, 1).half()], 4, 4, "tq2")


def test_bad_offsets_are_a_value_error_before_anything_else():
    x = torch.zeros(9, 8, dtype=torch.int8)
    packed = torch.zeros(6, 4, 2, dtype=torch.uint8)
    scales = torch.ones(6, 4, 1)
    for offs in ([0, 9], [0, 1, 2, 3, 4, 5, 8], [1, 1, 2, 3, 4, 5, 9], [0, 3, 2, 3, 4, 5, 9]):
        with pytest.raises(ValueError, match="offsets"):
            kb.grouped_ternary_gemm(x, torch.ones(9), offs, packed, scales, 8, 8, "tq2")


@pytest.mark.skipif(not NO_GPU, reason="checks the no-GPU behaviour")
def test_backend_absence_is_clean_and_loud():
    assert kb.ext() is None
    x = torch.zeros(2, 64, dtype=torch.int8)
    packed, scales = torch.zeros(4, 16, dtype=torch.uint8), torch.ones(4, 1)
    for backend in ("auto", "cuda", "b200"):
        with pytest.raises(RuntimeError, match="unavailable"):
            kb.ternary_gemm(x, torch.ones(2), packed, scales, 64, 64, "tq2", backend=backend)
    with pytest.raises(RuntimeError, match="unavailable"):
        kb.grouped_ternary_gemm(x, torch.ones(2), [0, 2], packed[None], scales[None], 64, 64, "tq2")
    with pytest.raises(RuntimeError, match="unavailable"):
        kb.ternary_gemm_bf16(x.bfloat16(), [packed], [scales.half()], 64, 64, "tq2")
    with pytest.raises(RuntimeError, match="unavailable"):
        kb.sort_by_expert(torch.zeros(4, dtype=torch.int64), 2)
    with pytest.raises(RuntimeError, match="unavailable"):
        pack.pack(torch.zeros(2, 8, dtype=torch.int8), "tq1")
    with pytest.raises(RuntimeError, match="unavailable"):
        pack.unpack(torch.zeros(2, 2, dtype=torch.uint8), "tq2", 8)
    with pytest.raises(RuntimeError, match="unavailable"):
        ops.quant_act_int8(torch.zeros(2, 8))


def test_ternary_linear_has_no_cpu_or_foreign_backend():
    term = ops.PackedTerm(torch.zeros(4, 16, dtype=torch.uint8), torch.ones(4, 1).half())
    for backend in ("cpp", "torch"):
        with pytest.raises(RuntimeError, match="unavailable"):
            ops.TernaryLinear([term], 64, "tq2", 64, act="bf16", backend=backend)
    with pytest.raises(ValueError):
        ops.TernaryLinear([term], 64, "tq9", 64)
    with pytest.raises(ValueError):
        ops.TernaryLinear([term], 64, "tq2", 64, act="fp8")
    lin = ops.TernaryLinear([term], 64, "tq2", 64, act="bf16")
    assert lin.out_features == 4
    with pytest.raises(RuntimeError, match="unavailable"):
        lin(torch.zeros(3, 64, dtype=torch.bfloat16))


def test_ep_placement_matches_brute_force():
    """Peer-memory expert parallelism: every (source rank, expert, row) gets a distinct row of the owner's buffer,
    sorted by local expert and, inside an expert, by source rank; the owner's offsets are the expert totals."""
    import numpy as np
    import torch

    from deepseekternarized_b200.moe import ep_placement

    rng = np.random.default_rng(0)
    W, El = 3, 4
    E = W * El
    counts = rng.integers(0, 5, (W, E))
    counts[:, 5] = 0  # an expert nobody routes to
    c = torch.from_numpy(counts)
    # brute force: the owner lists its rows as (local expert, source rank, index)
    want_start = np.zeros((W, E), np.int64)
    want_offsets = np.zeros((W, El + 1), np.int64)
    for d in range(W):
        pos = 0
        for e in range(El):
            want_offsets[d, e] = pos
            for s_rank in range(W):
                want_start[s_rank, d * El + e] = pos
                pos += counts[s_rank, d * El + e]
        want_offsets[d, El] = pos
    for r in range(W):
        dst_start, offsets_local = ep_placement(c, r, El)
        assert np.array_equal(dst_start.numpy(), want_start[r])
        assert np.array_equal(offsets_local.numpy(), want_offsets[r])


def test_ep_push_block_order_visits_every_row_once():
    """The push kernel's block -> sorted-row mapping (csrc/ep_kernels.cu, ep_push_kernel): the rows of the other ranks
    in cyclic order starting behind this rank's own rows [o0, o1), the own rows spread evenly among them. Restated
    here in integers: it must be a permutation of the rows, keep both sub-sequences in order, and never run more than
    one own row behind or ahead of an even spread."""
    import random

    def row_of_block(b, n, o0, o1):
        L = max(o1 - o0, 0)
        before, upto = b * L // n, (b + 1) * L // n
        if upto > before:
            return o0 + before
        p = o1 + (b - upto)
        return p - n if p >= n else p

    rnd = random.Random(4)
    cases = [(1, 0, 0), (1, 0, 1), (7, 0, 7), (7, 3, 3), (12, 0, 4), (12, 8, 12), (98304, 12288, 24576)]
    cases += [(n, *sorted((rnd.randint(0, n), rnd.randint(0, n)))) for n in (2, 5, 33, 1000, 4097) for _ in range(4)]
    for n, o0, o1 in cases:
        rows = [row_of_block(b, n, o0, o1) for b in range(n)]
        assert sorted(rows) == list(range(n)), (n, o0, o1)
        own = [r for r in rows if o0 <= r < o1]
        assert own == list(range(o0, o1))
        others = [r for r in rows if not (o0 <= r < o1)]
        assert others == [(o1 + i) % n for i in range(n - (o1 - o0))]
        L = o1 - o0
        seen = 0
        for b, r in enumerate(rows):
            seen += o0 <= r < o1
            assert abs(seen - (b + 1) * L / n) <= 1.0


def test_lookup_kernel_tq1_window_arithmetic():
    """The eight-trit window of the table-lookup kernel (csrc/format_kernels.cu, gather_dequant8_kernel): trits
    k .. k + 7 of a TQ1 row are read from bytes k / 5 .. k / 5 + 2 (the third only from k % 5 = 3 on), whose base-3
    digits as 2-bit fields, laid side by side and shifted down by 2 (k % 5), are the eight digits u = trit + 1."""
    import numpy as np

    from oracle import oracle as O

    rng = np.random.default_rng(8)
    K = 256
    t = O.synth_trits(rng, (3, K))
    packed = O.pack(t, "tq1")
    Kp = packed.shape[1]

    def fields(v):  # five base-3 digits as 2-bit fields
        f = 0
        for i in range(5):
            f |= (v % 3) << (2 * i)
            v //= 3
        return f

    for row in range(3):
        for k in range(0, K, 8):
            b0, r = divmod(k, 5)
            w = fields(int(packed[row, b0]))
            if b0 + 1 < Kp:
                w |= fields(int(packed[row, b0 + 1])) << 10
            if r > 2 and b0 + 2 < Kp:
                w |= fields(int(packed[row, b0 + 2])) << 20
            f = w >> (2 * r)
            got = [((f >> (2 * q)) & 3) - 1 for q in range(8)]
            assert got == t[row, k:k + 8].tolist()


def test_wide_drain_tile_addressing():
    """Index arithmetic of the tcgen05 kernel's 128-bit drain (csrc/gemm_prefill.cu, drain_tile_wide), restated in
    integers: the 16 transposed 8 x 8 matrices of a 32-token x 32-column chunk land on distinct 16-byte pieces of the
    warp's 2 KB tile, every piece (token row, eight columns) is where the read-back looks for it, and neither the
    eight row addresses of a stored matrix nor the eight addresses of a quarter-warp's 128-bit loads share a bank."""
    def piece_addr(tok, piece):
        return tok * 64 + ((piece ^ ((tok >> 1) & 3)) << 4)

    written = {}
    for h in range(2):           # lane half of the quarter: columns 16 h ..
        for x in range(2):       # one stmatrix.x4: token blocks 2 x, 2 x + 1
            for k in range(4):   # matrix k of the instruction: lanes 8 k .. 8 k + 7 give its row addresses
                addrs = []
                for st_r in range(8):
                    lane = 8 * k + st_r
                    st_g, st_b = (lane >> 3) & 1, lane >> 4
                    tok, piece = 8 * (2 * x + st_b) + st_r, 2 * h + st_g
                    a = piece_addr(tok, piece)
                    assert a % 16 == 0 and 0 <= a < 2048
                    addrs.append(a)
                    # row st_r of the transposed matrix = token row 8 b + st_r, columns 8 piece .. 8 piece + 7
                    assert (tok, piece) not in written
                    written[(tok, piece)] = a
                banks = {(a // 4) % 32 // 4 for a in addrs}  # groups of four banks = one 16-byte piece
                assert len(banks) == 8
    assert len(written) == 128 and len(set(written.values())) == 128
    for i in range(4):           # read-back: piece 32 i + lane
        for q in range(4):       # a 128-bit load is served a quarter-warp at a time
            addrs = []
            for lane in range(8 * q, 8 * q + 8):
                tok, piece = 8 * i + (lane >> 2), lane & 3
                assert written[(tok, piece)] == piece_addr(tok, piece)
                addrs.append(piece_addr(tok, piece))
            assert len({(a // 4) % 32 // 4 for a in addrs}) == 8


def test_host_pipeline_has_no_cpu_path():
    from deepseekternarized_b200.moe import HostPipeline

    with pytest.raises(RuntimeError, match="CUDA"):
        HostPipeline(lambda x, lg: x, 8, 16, 4, "cpu")
    with pytest.raises(ValueError):
        HostPipeline(lambda x, lg: x, 8, 16, 4, "cpu", slots=1)
