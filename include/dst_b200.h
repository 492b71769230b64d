/*
 * dst_b200.h - C ABI of the B200 (sm_100a) ternary expert-GEMM library (libdst_b200.so).
 *
 * The library replaces ONE path of the reference project Vedant-Sood/DeepSeekTernarized
 * ("Boilerplate"): the Mode C/D ternary linear and the MoE routed-expert GEMM. Every entry point
 * takes plain pointers and sizes, launches on the CUDA stream it is given and returns a status
 * code; nothing here allocates device memory unless its comment says so. All device pointers must
 * belong to the device that is current when the call is made.
 *
 * Formats (reference: boilerplate/ternary/pack.py:1-17). A trit t in {-1,0,+1} is stored as the
 * digit u = t + 1. Weights are [N, K] row-major, K contiguous; each row is packed on its own and
 * padded to a whole byte with digit 1 (t = 0).
 *   fmt 2 = TQ2: byte = u0 | u1<<2 | u2<<4 | u3<<6      -> ceil(K/4) bytes per row
 *   fmt 1 = TQ1: byte = u0 + 3 u1 + 9 u2 + 27 u3 + 81 u4 -> ceil(K/5) bytes per row (values 243..255
 *                decode to five zeros)
 * Scales: one per output row per `group` consecutive K entries, [N, ceil(K/group)].
 * Stacked (Mode C) weights are `n_terms` such (packed, scale) pairs; their products are summed.
 */
#ifndef DST_B200_H
#define DST_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* A CUDA stream handle (cudaStream_t / CUstream) passed as an opaque pointer; NULL = default stream. */
typedef void* dst_stream_t;

/* Status codes. The Python shim maps them to the exception types the reference raises:
 * BAD_ARG/BAD_SHAPE/UNSUPPORTED/ALIGNMENT -> RuntimeError (the reference's TORCH_CHECK failures,
 * boilerplate/kernels/csrc/ternary_cuda_kernel.cu:109-141), BAD_OFFSETS -> ValueError("offsets ...")
 * (boilerplate/kernels/ternary_cuda.py:94-97). */
enum {
  DST_OK = 0,
  DST_ERR_BAD_ARG = 1,     /* null pointer, K <= 0, group <= 0, fmt not 1/2, bad enum value */
  DST_ERR_BAD_SHAPE = 2,   /* sizes inconsistent with each other or beyond documented bounds */
  DST_ERR_BAD_OFFSETS = 3, /* offsets not nondecreasing from 0 to T */
  DST_ERR_UNSUPPORTED = 4, /* the requested kernel does not cover this shape (see each entry) */
  DST_ERR_ALIGNMENT = 5,   /* a pointer misses the alignment the requested kernel needs */
  DST_ERR_CUDA = 6,        /* a CUDA runtime call failed; see dst_last_cuda_error() */
  DST_ERR_TIMEOUT = 7,     /* a bounded device-side wait expired (reported by dst_check_device_status) */
  DST_ERR_TOO_LARGE = 8    /* the call needs more scratch than the no-allocation entry point's fixed array holds */
};

enum { DST_FMT_TQ1 = 1, DST_FMT_TQ2 = 2 };           /* boilerplate/kernels/ternary_cuda.py:46-49 */
enum { DST_SCALE_F16 = 0, DST_SCALE_F32 = 1, DST_SCALE_BF16 = 2 };
enum { DST_OUT_F32 = 0, DST_OUT_BF16 = 1, DST_OUT_F16 = 2 };
/* F16_NORM: fp16 rows the caller has already scaled by a power of two per row (row maximum in [128, 256)), with
 * the factors in row_scale; dst_gather_rows_norm / dst_swiglu_norm produce them. The tcgen05 kernel then needs
 * no conversion pass and no workspace. */
enum { DST_ACT_BF16 = 0, DST_ACT_F16 = 1, DST_ACT_I8 = 2, DST_ACT_F16_NORM = 3 };
/* Kernel choice. AUTO picks DECODE for few rows per expert, PREFILL for many, and GENERIC for
 * shapes the two fast kernels do not cover. */
enum { DST_ALGO_AUTO = 0, DST_ALGO_GENERIC = 1, DST_ALGO_DECODE = 2, DST_ALGO_PREFILL = 3 };
/* Weight layout: CANONICAL is the reference's [E, N, packed_cols]; TILED is the device layout built
 * once by dst_tile_weights (below), which the two fast kernels read. */
enum { DST_LAYOUT_CANONICAL = 0, DST_LAYOUT_TILED = 1 };

#define DST_MAX_TERMS 4
#define DST_MAX_PEERS 16 /* ranks of one node whose buffers a kernel can address (expert-parallel entries) */
#define DST_MAX_EXPERTS 65535 /* the reference's bound, ternary_cuda_kernel.cu:128 */

int dst_abi_version(void);
const char* dst_status_string(int status);
/* Text of the last CUDA runtime error seen by this library on the calling thread ("" if none). */
const char* dst_last_cuda_error(void);

/* ceil(K / 4) for TQ2, ceil(K / 5) for TQ1; -1 for a bad fmt or K <= 0.
 * Replaces boilerplate/ternary/pack.py:30-31 (packed_cols). */
int64_t dst_packed_cols(int fmt, int64_t K);

/* Device pack: int8 trits [N, K] -> uint8 [N, packed_cols]. Trits outside {-1,0,1} -> DST_ERR_BAD_ARG
 * is NOT detected on the device; the caller guarantees the range, as the reference's packer does.
 * Replaces boilerplate/ternary/pack.py:34-45,54-59,77-78 (_digits, pack_tq2, pack_tq1, pack). */
int dst_pack(const int8_t* trits, int64_t N, int64_t K, int fmt, uint8_t* packed, dst_stream_t stream);

/* Device unpack: uint8 [N, packed_cols] -> int8 trits [N, K], bit-exact with the reference table
 * (TQ1 bytes 243..255 -> 0; a TQ2 field of 3 -> +2, as the reference's shift-and-mask gives).
 * Replaces boilerplate/ternary/pack.py:48-51,62-74,81-82 (unpack_tq2, tq1_lut, unpack_tq1, unpack). */
int dst_unpack(const uint8_t* packed, int64_t N, int64_t K, int fmt, int8_t* trits, dst_stream_t stream);

/*
 * Tiled device layout: tiled[e][n / 128][sb][n % 128][64 bytes], a superblock sb being 64 bytes of one
 * row (256 trits in TQ2, 320 in TQ1). Rows are padded to a multiple of 128 and K to whole superblocks
 * with zero trits. TQ1 bytes keep their base-3 value; TQ2 32-bit words are bit-permuted so that the
 * low and the high half hold the even and the odd trits of 16 consecutive ones; the sixteen words of a
 * row-superblock are stored transposed 4 x 4 and swizzled by the row (see csrc/layout_kernels.cu). dst_tiled_bytes gives
 * the buffer size (-1 on bad arguments); dst_untile_weights restores the canonical bytes bit for bit.
 * `tiled` must be 16-byte aligned. The conversion is the one-time copy the reference makes when a
 * linear first meets a device (boilerplate/ternary/ops.py:41-45, TernaryLinear._on).
 */
int64_t dst_tiled_bytes(int fmt, int64_t E, int64_t N, int64_t K);
int dst_tile_weights(const uint8_t* canonical, int64_t E, int64_t N, int64_t K, int fmt, uint8_t* tiled,
                     dst_stream_t stream);
int dst_untile_weights(const uint8_t* tiled, int64_t E, int64_t N, int64_t K, int fmt, uint8_t* canonical,
                       dst_stream_t stream);

/* Per-token absmax int8 quantisation: s = max(absmax/127, 1e-8), q = clamp(rint(x/s), -127, 127).
 * x is bf16 or f32 ([M, K]); q int8 [M, K]; s f32 [M].
 * Replaces boilerplate/ternary/ops.py:20-25 (quant_act_int8). */
int dst_quant_act_int8(const void* x, int x_is_f32, int64_t M, int64_t K, int8_t* q, float* s,
                       dst_stream_t stream);
/* The same quantisation with q stored as fp16 (every |q| <= 127 is exact in fp16): (q_f16, s) is then a
 * DST_ACT_F16_NORM activation (rows + per-row factors), so an act = "int8" linear over many rows is this kernel and the
 * tcgen05 GEMM, with no conversion pass in between. Same rounding as dst_quant_act_int8, value for value. */
int dst_quant_act_int8_f16(const void* x, int x_is_f32, int64_t M, int64_t K, void* q_f16, float* s,
                           dst_stream_t stream);

/*
 * The ternary grouped GEMM.
 *
 *   out[t, n] (+)= row_scale[t] * sum_{i < n_terms} sum_g scale_i[e(t), n, g]
 *                                  * sum_{k in group g} x[t, k] * trit_i[e(t), n, k]
 *
 * Rows of x are sorted by expert: expert e owns rows offsets[e] .. offsets[e+1]. A plain linear is
 * the case E = 1 with offsets = NULL.
 *
 *   out          [T, N], type out_dtype; overwritten, or accumulated into when accumulate != 0
 *                (f32 only), which is how the reference sums Mode C terms (ternary/ops.py:71-79).
 *   x            [T, K] activations of type act_dtype (bf16 for the Mode C/D north-star path; int8
 *                for the reference's CUDA contract, boilerplate/kernels/ternary_cuda.py:3-9).
 *   row_scale    [T] f32 or NULL (= 1). For int8 activations this is x_scale.
 *   offsets      device int64 [E+1], or NULL when E == 1.
 *   offsets_host optional host copy of the same E+1 values. When given it is validated exactly as
 *                the reference does (ternary_cuda_kernel.cu:129-139) before anything is launched;
 *                when NULL the kernels clamp every row range to [0, T] instead.
 *   weight_layout DST_LAYOUT_CANONICAL or DST_LAYOUT_TILED
 *   packed       n_terms device pointers, each [E, N, packed_cols] uint8 (canonical) or a buffer of
 *                dst_tiled_bytes(fmt, E, N, K) bytes made by dst_tile_weights (tiled)
 *   scales       n_terms device pointers, each [E, N, ceil(K/group)] of scale_dtype
 *   algo         DST_ALGO_*; a fast kernel asked for explicitly returns DST_ERR_UNSUPPORTED /
 *                DST_ERR_ALIGNMENT when it does not cover the call (AUTO falls back to GENERIC).
 *   workspace    device scratch of at least dst_gemm_workspace_bytes(...) bytes, 256-byte aligned, or
 *                NULL. The prefill kernel keeps the fp16 copy of the activations and the per-row
 *                factors there (it needs it unless the activations are DST_ACT_F16_NORM); the decode
 *                GEMV uses it, when given, to quantise every token once ahead of itself instead of
 *                once per expert and CTA (same results). It is free again when the launched work
 *                has finished.
 *
 * Fast-kernel coverage: tiled weights, group == 128, K % 128 == 0 (TQ2 decode: K % 256 == 0), fp16 scales, bf16,
 * f16 or int8 activations. GENERIC reads canonical weights only.
 * Bounds: E <= DST_MAX_EXPERTS, K <= 2^24, N <= 2^24, T <= 2^31 - 1.
 *
 * Replaces the native entry ternary_grouped_gemm (boilerplate/kernels/csrc/ternary_cuda.cpp:7-10,
 * ternary_cuda_kernel.cu:106-152) and the CPU entry ternary_gemm it shadows
 * (boilerplate/kernels/csrc/boilerplate_cpu.cpp:80-128).
 */
int dst_ternary_grouped_gemm(void* out, int out_dtype, int accumulate, const void* x, int act_dtype,
                             const float* row_scale, const int64_t* offsets, const int64_t* offsets_host,
                             const void* const* packed, int weight_layout, const void* const* scales,
                             int n_terms, int scale_dtype, int64_t E, int64_t T, int64_t N, int64_t K,
                             int64_t group, int fmt, int algo, void* workspace, size_t workspace_bytes,
                             dst_stream_t stream);

/* Scratch bytes dst_ternary_grouped_gemm needs for `algo` (AUTO: the largest any kernel may need). */
size_t dst_gemm_workspace_bytes(int algo, int act_dtype, int64_t T, int64_t K);

/* Token rows per expert up to which DST_ALGO_AUTO sends tiled weights of `fmt` (E experts of N rows) to the
 * decode GEMV rather than the tcgen05 kernel: 16, or 32 where the decode GEMV's many-row form applies. A caller
 * that keeps a second, decode-friendly copy of its weights (the Python layer's 2-bit copy of TQ1 trits) picks
 * the copy by the same rule. No reference counterpart: the reference has one kernel for every row count
 * (boilerplate/kernels/csrc/ternary_cuda_kernel.cu:44-99). */
int64_t dst_decode_row_limit(int fmt, int64_t E, int64_t N);

/*
 * Routing sort: flattened expert ids [n] (int64 or int32) -> the stable order that sorts them by
 * expert and offsets[E+1] (int64). Ids outside [0, E) are counted in *bad_count (device int32, may
 * be NULL) and dropped: order[offsets[E] .. n) is then -1. Runs three small kernels; `workspace` must hold dst_sort_workspace_bytes(n, E).
 * Replaces boilerplate/kernels/ternary_cuda.py:114-118 (sort_by_expert).
 */
size_t dst_sort_workspace_bytes(int64_t n, int64_t E);
int dst_sort_by_expert(const void* ids, int ids_are_i32, int64_t n, int64_t E, int64_t* order,
                       int64_t* offsets, int32_t* bad_count, void* workspace, dst_stream_t stream);

/*
 * Router: softmax over E logits per token, top-k by score (ties: lower expert id first), weights
 * renormalised by (sum + 1e-20) and multiplied by route_scale.
 * logits [T, E] f32 -> weights [T, k] f32, ids [T, k] int32. E <= 1024, k <= 8.
 * Replaces boilerplate/engine/model.py:389-405 (route) for score_func = "softmax", no bias.
 */
int dst_route_softmax_topk(const float* logits, int64_t T, int64_t E, int top_k, float route_scale,
                           float* weights, int32_t* ids, dst_stream_t stream);
/*
 * The general router of boilerplate/engine/model.py:389-405:
 *   score   = f(logit / gate_temp), f = softmax over the E logits | sigmoid | sqrt(softplus)   (score_func)
 *   ids     = the top_k experts by score + bias[e] (bias [E] f32 or NULL; ties: lower expert id first; a NaN ranks
 *             above every number as in torch.topk)
 *   weights = the UNBIASED scores of the picked experts, divided by (their sum + 1e-20) when renorm != 0 and
 *             top_k > 1, times route_scale
 * The top_k ids of a token are always distinct and inside [0, E), whatever the logits hold (NaN, +-inf).
 * E <= 1024, top_k <= 8, gate_temp != 0.
 */
enum { DST_SCORE_SOFTMAX = 0, DST_SCORE_SIGMOID = 1, DST_SCORE_SQRTSOFTPLUS = 2 };
int dst_route_topk(const float* logits, const float* bias, int64_t T, int64_t E, int top_k, int score_func, float gate_temp,
                   int renorm, float route_scale, float* weights, int32_t* ids, dst_stream_t stream);
/* The same with the renormalisation optional (renorm = 0: the softmax scores of the selected experts as they are):
 * the `norm_topk_prob` switch of boilerplate/engine/standard.py:159-165. */
int dst_route_softmax_topk_ex(const float* logits, int64_t T, int64_t E, int top_k, int renorm, float route_scale,
                              float* weights, int32_t* ids, dst_stream_t stream);

/*
 * Gather token rows into expert-sorted order: dst[p, :] = src[order[p] / top_k, :] (16-bit elements,
 * bf16 stays bf16). Replaces the x[idx] gathers of boilerplate/engine/model.py:418-419.
 */
int dst_gather_rows(const void* src, const int64_t* order, int64_t n_rows, int64_t K, int top_k,
                    void* dst, dst_stream_t stream);

/*
 * SwiGLU between the up and down projections, reference rounding points included:
 * gate/up are the bf16 outputs of w1/w3 laid out as gu[p, 0:I] = gate, gu[p, I:2I] = up;
 * h = bf16( weight[order[p]] * silu(gate) * up ), with optional clamps (limit > 0: up to +-limit,
 * gate to <= limit). Replaces boilerplate/engine/model.py:376-386 (swiglu, up to the w2 call).
 */
int dst_swiglu(const void* gu_bf16, const float* route_weights, const int64_t* order, int64_t n_rows,
               int64_t inter, float limit, void* h_bf16, dst_stream_t stream);

/*
 * The same two steps producing the tcgen05 kernel's input format directly (DST_ACT_F16_NORM): fp16 rows scaled
 * by 2^-e per row so the row maximum lies in [128, 256), and row_factor[p] = 2^e. Values are the reference's
 * (bf16 activations; bf16-rounded SwiGLU output) times an exact power of two. `order` may be NULL in
 * dst_gather_rows_norm (identity: convert rows in place order).
 */
int dst_gather_rows_norm(const void* src_bf16, const int64_t* order, int64_t n_rows, int64_t K, int top_k,
                         void* dst_f16, float* row_factor, dst_stream_t stream);
int dst_swiglu_norm(const void* gu_bf16, const float* route_weights, const int64_t* order, int64_t n_rows,
                    int64_t inter, float limit, void* h_f16, float* row_factor, dst_stream_t stream);
/* dst_swiglu_norm over the first min(n_rows_max, *n_rows_dev) rows, the count read on the device: an expert-parallel
 * rank learns how many rows the others sent it without a host round trip. inter % 8 == 0, inter <= 8192. */
int dst_swiglu_norm_dev(const void* gu_bf16, const float* route_weights, const int64_t* order, int64_t n_rows_max,
                        const int64_t* n_rows_dev, int64_t inter, float limit, void* h_f16, float* row_factor,
                        dst_stream_t stream);

/*
 * Combine: y[t, :] = bf16( sum over the token's top_k slots, in increasing expert id, of
 * down[pos(t, slot), :] ), fp32 accumulation; `order` is the routing sort's order and `ids` the
 * flattened expert ids [T * top_k]. Replaces the `y[idx] += ...` accumulation and the final cast of
 * boilerplate/engine/model.py:413-422. `inv` is an int64 [T * top_k] scratch the call fills.
 */
int dst_combine(const void* down_bf16, const int64_t* order, const int32_t* ids, int64_t T, int top_k,
                int64_t hidden, int64_t* inv, void* y_bf16, dst_stream_t stream);
/* The same with one more bf16 row per token added in fp32 after the experts' rows and before the cast: the shared
 * expert's output, `y += self.swiglu(L.shared, x)` of boilerplate/engine/model.py:421. add_bf16 [T, hidden] or NULL.
 * A (token, slot) whose expert id the routing sort dropped (outside [0, E)) contributes nothing. */
int dst_combine_add(const void* down_bf16, const int64_t* order, const int32_t* ids, int64_t T, int top_k,
                    int64_t hidden, int64_t* inv, const void* add_bf16, void* y_bf16, dst_stream_t stream);

/*
 * The standard (OLMoE-style) MoE flavour, boilerplate/engine/standard.py:149-176, which keeps every intermediate in
 * bf16: h = bf16( bf16(silu(gate)) * up ) without a routing weight (dst_swiglu_std: bf16 rows;
 * dst_swiglu_std_norm: the DST_ACT_F16_NORM format), and the combine
 * y[t] = sum over the token's slots in increasing expert id of bf16( down * bf16(weight) ), every partial sum
 * rounded to bf16 (index_add_ into a bf16 tensor). `weights` [T * top_k] f32 as the router wrote them.
 */
int dst_swiglu_std(const void* gu_bf16, int64_t n_rows, int64_t inter, void* h_bf16, dst_stream_t stream);
int dst_swiglu_std_norm(const void* gu_bf16, int64_t n_rows, int64_t inter, void* h_f16, float* row_factor,
                        dst_stream_t stream);
int dst_combine_weighted(const void* down_bf16, const int64_t* order, const int32_t* ids, const float* weights, int64_t T,
                         int top_k, int64_t hidden, int64_t* inv, void* y_bf16, dst_stream_t stream);

/*
 * Rows of a ternary lookup table (the Mode C/D engram tables): out[i, :] = bf16( sum over terms of
 * trit[ids[i], :] * scale[ids[i], : / group] ), fp32 products added in term order. packed[t] [V, ceil(K / per)]
 * canonical rows, scales[t] [V, ceil(K / group)] of scale_dtype. An id outside [0, V) is counted in *bad_count
 * (device int32, may be NULL) and its row is written as zeros. Replaces boilerplate/engine/model.py:458-464.
 */
int dst_gather_dequant_rows(const void* const* packed, const void* const* scales, int n_terms, int scale_dtype,
                            const int64_t* ids, int64_t n_ids, int64_t V, int64_t K, int64_t group, int fmt, void* out_bf16,
                            int32_t* bad_count, dst_stream_t stream);
/*
 * The same lookup over rows that are not densely stored: row r of term t starts at packed[t] + r * packed_row_stride
 * bytes and its scales at element r * scale_row_stride of scales[t]. With one record per table row that holds the
 * packed bytes of every term followed by their scales (both strides = the record's size, in bytes and in scale
 * elements), a looked-up row is ONE stretch of DRAM instead of two per term (measured on 256-wide rows: 1.2x faster
 * for two stacked TQ1 terms, no gain for one term).
 */
int dst_gather_dequant_rows_strided(const void* const* packed, const void* const* scales, int n_terms, int scale_dtype,
                                    const int64_t* ids, int64_t n_ids, int64_t V, int64_t K, int64_t group, int fmt,
                                    int64_t packed_row_stride, int64_t scale_row_stride, void* out_bf16, int32_t* bad_count,
                                    dst_stream_t stream);

/*
 * Expert-parallel dispatch and combine over peer memory (the reference has no expert-parallel exchange of routed
 * rows: its EP form replicates tokens and all-reduces, third_party/deepseek_v41_inference/model.py:897-905; these
 * two entries serve the sharding of the same file, :869-872, expert e on rank e / experts_per_rank).
 * The peer_* arrays hold, per rank of the node, the address AS MAPPED IN THIS PROCESS of that rank's buffer
 * (e.g. torch symmetric memory): receive rows [cap, K] f16, row factors [cap] f32, routing weights [cap] f32,
 * expert outputs [cap, hidden] bf16. `offsets` [E + 1] is this rank's routing-sort offsets over the GLOBAL experts,
 * dst_start [E] the first row, in the owning rank's receive buffer, of this rank's rows of each expert.
 * dst_ep_push_rows: for every sorted row p, the token row order[p] / top_k as fp16 scaled by a power of two
 * (DST_ACT_F16_NORM) -> the owner's buffers (rows, factor, routing weight route_weights[order[p]]). row_dest is an
 * int64 [n_rows] scratch the call fills (each row's owner and row there, found once by a small kernel of its own);
 * `rank` is this rank's index: it starts with the rows of the rank after it, so the ranks do not all store into the
 * same GPU at the same time, and spreads its own rows among the others', so the local copies run under the transfers.
 * peer_row_origin (may be NULL): per rank an int64 [cap] array; the push also records there, beside every row it
 * delivers, (rank << 48) | slot, slot = order[p] = token * top_k + choice: the row_target of the scatter GEMM below.
 * dst_ep_combine_pull: y[t] = bf16( sum over the token's slots, in increasing expert id, of the owner's output row ).
 * Neither waits on another GPU; the caller orders the steps (a stream-ordered collective between them).
 *
 * The fused form of the way back (GEMM + combine transfer in one kernel): dst_ternary_grouped_gemm_scatter is the
 * tcgen05 grouped GEMM whose epilogue stores output row r at row (row_target[r] & (2^48 - 1)) of the two-byte-typed
 * buffer peer_out[row_target[r] >> 48] [peer_rows, N] (a negative target, a buffer index >= n_peers or a row >= peer_rows:
 * not stored), with plain stores over NVLink
 * while the tensor pipe works on the next tile; with row_target = the origins the push recorded, the second expert
 * GEMM delivers every output row to slot token * top_k + choice of the rank that owns the token, and after a barrier
 * dst_ep_combine_returned sums each token's slots locally (same order, same values as dst_ep_combine_pull_add).
 * Tiled weights only; DST_ERR_UNSUPPORTED where the tcgen05 kernel does not cover the call.
 */
int dst_ternary_grouped_gemm_scatter(void* const* peer_out, int n_peers, int64_t peer_rows, const int64_t* row_target, int out_dtype, const void* x,
                                     int act_dtype, const float* row_scale, const int64_t* offsets, const int64_t* offsets_host,
                                     const void* const* packed, const void* const* scales, int n_terms, int scale_dtype, int64_t E,
                                     int64_t T, int64_t N, int64_t K, int64_t group, int fmt, void* workspace, size_t workspace_bytes,
                                     dst_stream_t stream);
/* y[t] = bf16( sum over the token's slots, in increasing expert id, of rows_bf16[t * top_k + slot] (+ add_bf16[t]) ):
 * the rows as the scatter GEMM delivered them. order / row_dest: the routing sort's order and the row destinations
 * dst_ep_push_rows filled (a negative destination: the slot has no row). inv: int64 [T * top_k] scratch. */
int dst_ep_combine_returned(const void* rows_bf16, const int64_t* order, const int64_t* row_dest, const int32_t* ids, int64_t T,
                            int top_k, int64_t hidden, int64_t* inv, const void* add_bf16, void* y_bf16, dst_stream_t stream);
/* Barrier among the ranks of one node over peer memory, in stream order: peer_flags[r] is rank r's flag array (int64
 * [world], zero at the start) as mapped in this process; seq = 1, 2, 3, ... counts the barriers of the job, the same on
 * every rank. The wait for the other ranks is bounded (~2 s), after which dst_check_device_status reports DST_ERR_TIMEOUT. */
int dst_ep_barrier(const void* const* peer_flags, int world, int rank, int64_t seq, dst_stream_t stream);
/* Where this rank's routed rows go: offsets_all [world][E + 1] holds every rank's routing-sort offsets over the global
 * experts (an all-gather of `offsets`); writes dst_start [E] and offsets_local [experts_per_rank + 1] (the row offsets
 * of this rank's own experts in its receive buffer = the grouped GEMM's offsets). One small kernel, no host step. */
int dst_ep_placement(const int64_t* offsets_all, int world, int64_t E, int64_t experts_per_rank, int rank, int64_t* dst_start,
                     int64_t* offsets_local, dst_stream_t stream);
int dst_ep_push_rows(const void* x_bf16, const int64_t* order, const int64_t* offsets, const float* route_weights,
                     const int64_t* dst_start, int64_t n_rows, int64_t E, int64_t experts_per_rank, int top_k, int64_t K,
                     const void* const* peer_rows_f16, const void* const* peer_row_factor, const void* const* peer_row_weight,
                     const void* const* peer_row_origin, int world, int rank, int64_t* row_dest, dst_stream_t stream);
int dst_ep_combine_pull(const void* const* peer_down_bf16, const int64_t* order, const int32_t* ids, const int64_t* offsets,
                        const int64_t* dst_start, int64_t T, int64_t experts_per_rank, int top_k, int64_t hidden, int64_t* inv,
                        void* y_bf16, int world, dst_stream_t stream);
/* dst_ep_combine_pull with the token's row of add_bf16 [T, hidden] (this rank's shared-expert output, or NULL) added
 * in fp32 after the experts' rows, as dst_combine_add does. */
int dst_ep_combine_pull_add(const void* const* peer_down_bf16, const int64_t* order, const int32_t* ids, const int64_t* offsets,
                            const int64_t* dst_start, int64_t T, int64_t experts_per_rank, int top_k, int64_t hidden, int64_t* inv,
                            const void* add_bf16, void* y_bf16, int world, dst_stream_t stream);

/*
 * The grouped GEMM for callers that must not allocate device memory. (This entry has no counterpart
 * in the reference project.)
 *
 * Who needs it: code that runs where cudaMalloc is off limits - a serving loop whose memory was
 * carved up at start-up and handed to other owners, a host thread that may not take the allocator's
 * lock or synchronise the device (cudaMalloc and cudaFree can do both), or a plug-in that is only
 * given pointers and has no allocator of its own. dst_ternary_grouped_gemm needs a workspace from
 * such a caller; this entry brings its own: DST_NOALLOC_SCRATCH_BYTES of device memory that are part
 * of the library image (every GPU that loads the library holds them until the process exits).
 *
 * It is the tcgen05 kernel of dst_ternary_grouped_gemm (algo DST_ALGO_PREFILL) and returns the same
 * results: tiled weights (dst_tile_weights), fp16 scales, group 128, K % 128 == 0, bf16 or fp16
 * activations; inputs and outputs are still the caller's. The call itself performs no cudaMalloc,
 * cudaFree or other allocating routine.
 *
 * Limits and rules:
 *   - T * K * 2 + T * 4 bytes (plus up to 512 bytes of alignment slack) must fit DST_NOALLOC_SCRATCH_BYTES,
 *     8 MiB + 16 KiB: 1024 rows at K = 4096, 2048 rows at K = 2048. A larger call returns DST_ERR_TOO_LARGE
 *     and launches nothing.
 *   - The first call on a device looks up the scratch array's device address
 *     (cudaGetSymbolAddress, with that device current) and keeps it. Make that first call before
 *     any stream capture begins.
 *   - All calls on a device share the one array and it keeps whatever the previous call left there.
 *     Nothing in it has to start at zero (every byte a call reads, it has written first), but two calls
 *     whose GPU work overlaps - different streams, or different host threads - race on it. Keep the
 *     calls of one device on one stream, or order them with events.
 */
#define DST_NOALLOC_SCRATCH_BYTES (8u * 1024u * 1024u + 16384u)
int dst_ternary_grouped_gemm_noalloc(void* out, int out_dtype, int accumulate, const void* x, int act_dtype,
                                     const float* row_scale, const int64_t* offsets, const int64_t* offsets_host,
                                     const void* const* packed_tiled, const void* const* scales, int n_terms,
                                     int64_t E, int64_t T, int64_t N, int64_t K, int fmt, dst_stream_t stream);

/* Reads (and clears) the device-side status words that bounded waits in the tcgen05, decode and barrier kernels write when
 * they give up. Synchronises `stream`. Returns DST_OK or DST_ERR_TIMEOUT. */
int dst_check_device_status(dst_stream_t stream);

/*
 * Test hook for the failure path of the tcgen05 kernel (this device, until called again with zeros): wait_cycles > 0
 * shortens the bounded waits from ~2 s to that many clock cycles; drop_drain_arrivals != 0 makes the warps that drain
 * the accumulator withhold their "drained" signal, so at a CTA's second tile the MMA warps' wait runs out, the CTA
 * aborts in order (every role leaves, TMEM is freed) and dst_check_device_status reports DST_ERR_TIMEOUT; max_ctas > 0
 * caps the grid so that one CTA is sure to own several tiles. Nothing in this path faults or waits without a bound.
 * dst_debug_prefill_timeout(0, 0, 0) restores normal operation. Synchronises the device.
 */
int dst_debug_prefill_timeout(long long wait_cycles, int drop_drain_arrivals, int max_ctas);

#ifdef __cplusplus
}
#endif
#endif /* DST_B200_H */
