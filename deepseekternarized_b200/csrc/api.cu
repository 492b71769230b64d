// C-ABI entry points of the ternary grouped GEMM: argument validation and kernel choice.
// The checks mirror the reference launcher's (boilerplate/kernels/csrc/ternary_cuda_kernel.cu:109-141):
// exact sizes only, offsets validated on the host whenever a host copy is supplied.
#include <algorithm>
#include <cstdio>
#include <cstring>

#include "dst_common.cuh"

namespace dst {

static thread_local char g_last_error[256] = "";

int record_cuda_error(cudaError_t err, const char* where) {
  std::snprintf(g_last_error, sizeof(g_last_error), "%s: %s (%s)", where, cudaGetErrorName(err),
                cudaGetErrorString(err));
  return DST_ERR_CUDA;
}

}  // namespace dst

extern "C" int dst_abi_version(void) { return 1; }

extern "C" const char* dst_last_cuda_error(void) { return dst::g_last_error; }

extern "C" const char* dst_status_string(int status) {
  switch (status) {
    case DST_OK: return "ok";
    case DST_ERR_BAD_ARG: return "invalid argument (null pointer, non-positive K or group, unknown format or dtype)";
    case DST_ERR_BAD_SHAPE: return "inconsistent ternary GEMM shapes";
    case DST_ERR_BAD_OFFSETS: return "offsets must be nondecreasing, start at 0, end at the row count, one per expert + 1";
    case DST_ERR_UNSUPPORTED: return "shape not covered by the requested kernel";
    case DST_ERR_ALIGNMENT: return "pointer alignment not sufficient for the requested kernel";
    case DST_ERR_CUDA: return "CUDA runtime error";
    case DST_ERR_TIMEOUT: return "a bounded device-side wait expired";
    case DST_ERR_TOO_LARGE: return "the call needs more scratch than the no-allocation entry point's fixed array holds";
    default: return "unknown status";
  }
}

// The grouped GEMM behind both entry points. row_target / peer_out: the scatter form (see GemmArgs), else null.
static int grouped_gemm(void* out, int out_dtype, int accumulate, const void* x, int act_dtype, const float* row_scale,
                        const int64_t* offsets, const int64_t* offsets_host, const void* const* packed, int weight_layout,
                        const void* const* scales, int n_terms, int scale_dtype, int64_t E, int64_t T, int64_t N, int64_t K,
                        int64_t group, int fmt, int algo, void* workspace, size_t workspace_bytes, dst_stream_t stream,
                        const int64_t* row_target, void* const* peer_out, int n_peers, int64_t peer_rows) {
  using namespace dst;
  if (K <= 0 || group <= 0 || (fmt != DST_FMT_TQ1 && fmt != DST_FMT_TQ2)) return DST_ERR_BAD_ARG;
  if (out_dtype < DST_OUT_F32 || out_dtype > DST_OUT_F16 || act_dtype < DST_ACT_BF16 || act_dtype > DST_ACT_F16_NORM ||
      scale_dtype < DST_SCALE_F16 || scale_dtype > DST_SCALE_BF16 || algo < DST_ALGO_AUTO || algo > DST_ALGO_PREFILL)
    return DST_ERR_BAD_ARG;
  if (n_terms < 1 || n_terms > DST_MAX_TERMS || E < 0 || T < 0 || N < 0) return DST_ERR_BAD_ARG;
  if (weight_layout != DST_LAYOUT_CANONICAL && weight_layout != DST_LAYOUT_TILED) return DST_ERR_BAD_ARG;
  if (accumulate && out_dtype != DST_OUT_F32) return DST_ERR_BAD_ARG;
  if (act_dtype == DST_ACT_F16_NORM && (row_scale == nullptr || algo == DST_ALGO_GENERIC || algo == DST_ALGO_DECODE))
    return act_dtype == DST_ACT_F16_NORM && row_scale == nullptr ? DST_ERR_BAD_ARG : DST_ERR_UNSUPPORTED;
  if (E > DST_MAX_EXPERTS || K > (int64_t(1) << 24) || N > (int64_t(1) << 24) || T > 0x7fffffff ||
      group > (int64_t(1) << 24))
    return DST_ERR_BAD_SHAPE;
  if (E != 1 && offsets == nullptr && E != 0) return DST_ERR_BAD_ARG;
  if (offsets_host) {
    if (offsets_host[0] != 0 || offsets_host[E] != T) return DST_ERR_BAD_OFFSETS;
    for (int64_t e = 0; e < E; ++e)
      if (offsets_host[e + 1] < offsets_host[e]) return DST_ERR_BAD_OFFSETS;
  }
  if (E == 0) return T == 0 ? DST_OK : DST_ERR_BAD_OFFSETS;
  if (T == 0 || N == 0) return DST_OK;
  if (!out || !x || !packed || !scales) return DST_ERR_BAD_ARG;

  GemmArgs a;
  std::memset(&a, 0, sizeof(a));
  a.out = out;
  a.out_dtype = out_dtype;
  a.accumulate = accumulate;
  a.x = x;
  a.act_dtype = act_dtype;
  a.row_scale = row_scale;
  a.offsets = offsets;
  a.terms.n = n_terms;
  for (int i = 0; i < n_terms; ++i) {
    if (!packed[i] || !scales[i]) return DST_ERR_BAD_ARG;
    a.terms.packed[i] = static_cast<const uint8_t*>(packed[i]);
    a.terms.scale[i] = scales[i];
  }
  a.scale_dtype = scale_dtype;
  a.E = E;
  a.T = T;
  a.N = N;
  a.K = K;
  a.group = group;
  a.Kp = cdiv64(K, fmt == DST_FMT_TQ2 ? 4 : 5);
  a.G = cdiv64(K, group);
  a.fmt = fmt;
  a.max_rows = -1;
  a.weight_layout = weight_layout;
  a.workspace = workspace;
  a.workspace_bytes = workspace ? workspace_bytes : 0;
  a.row_target = row_target;
  for (int i = 0; i < n_peers; ++i) a.peer_out[i] = peer_out[i];
  a.n_peer_out = n_peers;
  a.peer_rows = peer_rows;
  if (offsets_host) {
    int64_t widest = 0;
    for (int64_t e = 0; e < E; ++e) widest = std::max(widest, offsets_host[e + 1] - offsets_host[e]);
    a.max_rows = widest;
  } else if (E == 1) {
    a.max_rows = T;
  }
  auto st = static_cast<cudaStream_t>(stream);
  if (weight_layout == DST_LAYOUT_TILED && algo == DST_ALGO_GENERIC) return DST_ERR_UNSUPPORTED;
  switch (algo) {
    case DST_ALGO_GENERIC: return launch_generic(a, st);
    case DST_ALGO_DECODE: return launch_decode(a, st);
    case DST_ALGO_PREFILL: return launch_prefill(a, st);
    default: break;
  }
  if (act_dtype == DST_ACT_F16_NORM) return launch_prefill(a, st);  // only the tcgen05 kernel reads this format
  // AUTO: few rows per expert -> decode GEMV; many -> tcgen05 grouped GEMM; otherwise generic.
  const int64_t avg_rows = a.max_rows >= 0 ? a.max_rows : cdiv64(T, E);
  if (avg_rows <= decode_row_limit(fmt, E, N) && decode_supports(a)) return launch_decode(a, st);
  if (prefill_supports(a)) return launch_prefill(a, st);
  if (decode_supports(a)) return launch_decode(a, st);
  if (weight_layout == DST_LAYOUT_TILED) return DST_ERR_UNSUPPORTED;
  return launch_generic(a, st);
}

extern "C" int dst_ternary_grouped_gemm(void* out, int out_dtype, int accumulate, const void* x, int act_dtype,
                                        const float* row_scale, const int64_t* offsets, const int64_t* offsets_host,
                                        const void* const* packed, int weight_layout, const void* const* scales,
                                        int n_terms, int scale_dtype, int64_t E, int64_t T, int64_t N, int64_t K,
                                        int64_t group, int fmt, int algo, void* workspace, size_t workspace_bytes,
                                        dst_stream_t stream) {
  return grouped_gemm(out, out_dtype, accumulate, x, act_dtype, row_scale, offsets, offsets_host, packed, weight_layout, scales, n_terms,
                      scale_dtype, E, T, N, K, group, fmt, algo, workspace, workspace_bytes, stream, nullptr, nullptr, 0, 0);
}

extern "C" int dst_ternary_grouped_gemm_scatter(void* const* peer_out, int n_peers, int64_t peer_rows, const int64_t* row_target, int out_dtype,
                                                const void* x, int act_dtype, const float* row_scale, const int64_t* offsets,
                                                const int64_t* offsets_host, const void* const* packed, const void* const* scales,
                                                int n_terms, int scale_dtype, int64_t E, int64_t T, int64_t N, int64_t K,
                                                int64_t group, int fmt, void* workspace, size_t workspace_bytes,
                                                dst_stream_t stream) {
  if (!peer_out || !row_target || n_peers < 1 || n_peers > DST_MAX_PEERS || peer_rows < 0) return DST_ERR_BAD_ARG;
  if (out_dtype != DST_OUT_BF16 && out_dtype != DST_OUT_F16) return DST_ERR_UNSUPPORTED;  // two-byte rows only
  for (int i = 0; i < n_peers; ++i)
    if (!peer_out[i] || (reinterpret_cast<uintptr_t>(peer_out[i]) & 1) != 0) return DST_ERR_BAD_ARG;
  return grouped_gemm(peer_out[0], out_dtype, 0, x, act_dtype, row_scale, offsets, offsets_host, packed, DST_LAYOUT_TILED, scales, n_terms,
                      scale_dtype, E, T, N, K, group, fmt, DST_ALGO_PREFILL, workspace, workspace_bytes, stream, row_target, peer_out,
                      n_peers, peer_rows);
}

extern "C" int64_t dst_decode_row_limit(int fmt, int64_t E, int64_t N) { return dst::decode_row_limit(fmt, E, N); }

extern "C" size_t dst_gemm_workspace_bytes(int algo, int act_dtype, int64_t T, int64_t K) {
  if (T <= 0 || K <= 0 || algo == DST_ALGO_GENERIC) return 0;
  const size_t dec = K % 128 == 0 ? dst::decode_workspace_bytes(T, K) : 0;  // optional for the decode GEMV (it is faster with it)
  if (algo == DST_ALGO_DECODE) return dec;
  const size_t pre = dst::prefill_workspace_bytes(act_dtype, T, K);
  return algo == DST_ALGO_PREFILL ? pre : (pre > dec ? pre : dec);
}
