// Shared device/host helpers of the sm_100a ternary expert-GEMM library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/dst_b200.h"

namespace dst {

// Records a failed CUDA runtime call for dst_last_cuda_error(); returns DST_ERR_CUDA.
int record_cuda_error(cudaError_t err, const char* where);

#define DST_CUDA_TRY(expr)                                              \
  do {                                                                  \
    cudaError_t e__ = (expr);                                           \
    if (e__ != cudaSuccess) return ::dst::record_cuda_error(e__, #expr); \
  } while (0)

inline int64_t cdiv64(int64_t a, int64_t b) { return a / b + (a % b != 0); }

// One term-set of a stacked (Mode C) weight, passed to kernels by value.
struct Terms {
  const uint8_t* packed[DST_MAX_TERMS];
  const void* scale[DST_MAX_TERMS];
  int n;
};

// Arguments of a grouped ternary GEMM launch, shared by the three kernel families.
struct GemmArgs {
  void* out;
  int out_dtype;
  int accumulate;
  const void* x;
  int act_dtype;
  const float* row_scale;
  const int64_t* offsets;  // device, may be null when E == 1
  Terms terms;
  int scale_dtype;
  int64_t E, T, N, K, group, Kp, G;
  int fmt;
  int64_t max_rows;  // largest expert row count if known on the host, else -1
  int weight_layout;  // DST_LAYOUT_CANONICAL or DST_LAYOUT_TILED (terms.packed then points at tiled buffers)
  void* workspace;    // caller-provided scratch (may be null when the kernel needs none)
  size_t workspace_bytes;
  // optional scatter of the output rows (tcgen05 kernel only): row r goes to row (row_target[r] & (2^48 - 1)) of
  // peer_out[row_target[r] >> 48] (a negative target: the row is not stored); `out` is unused then
  const int64_t* row_target;
  void* peer_out[DST_MAX_PEERS];
  int n_peer_out;     // targets naming a buffer >= n_peer_out or a row >= peer_rows are not stored
  int64_t peer_rows;
};

int64_t tiled_superblocks(int fmt, int64_t K);
size_t prefill_workspace_bytes(int act_dtype, int64_t T, int64_t K);
size_t decode_workspace_bytes(int64_t T, int64_t K);  // optional: lets the decode GEMV quantise each token once, ahead of itself

int launch_generic(const GemmArgs& a, cudaStream_t stream);
int launch_decode(const GemmArgs& a, cudaStream_t stream);    // DST_ERR_UNSUPPORTED when not covered
int launch_prefill(const GemmArgs& a, cudaStream_t stream);   // DST_ERR_UNSUPPORTED when not covered
bool decode_supports(const GemmArgs& a);
int64_t decode_row_limit(int fmt, int64_t E, int64_t N);  // rows per expert up to which AUTO prefers the decode GEMV
int launch_decode_tq1(const GemmArgs& a, cudaStream_t stream);  // TQ1 decode kernel (gemm_decode_tq1.cu); reached through launch_decode
bool decode_tq1_supports(const GemmArgs& a);
bool prefill_supports(const GemmArgs& a);
int decode_take_status(int* status);
int ep_take_status(int* status);      // the same for the expert-parallel barrier kernel  // reads and clears the decode kernel's status word (0 or DST_ERR_TIMEOUT)

// ---------------------------------------------------------------------------------------------
// Trit decoding. TQ1 digit i of byte v: ((v / 3^i) % 3) - 1 for v < 243, else 0
// (reference table: boilerplate/ternary/pack.py:62-67).
// ---------------------------------------------------------------------------------------------

// 5 base-3 digits of v (< 243) as 2-bit fields d0 | d1<<2 | ... | d4<<8; 0b01 fields (t = 0) for v >= 243.
__host__ __device__ inline uint32_t tq1_fields(uint32_t v) {
  if (v >= 243u) return 0x155u;
  uint32_t f = 0;
#pragma unroll
  for (int i = 0; i < 5; ++i) {
    f |= (v % 3u) << (2 * i);
    v /= 3u;
  }
  return f;
}

__device__ __forceinline__ float scale_to_float(const void* p, int64_t idx, int scale_dtype) {
  if (scale_dtype == DST_SCALE_F16) return __half2float(reinterpret_cast<const __half*>(p)[idx]);
  if (scale_dtype == DST_SCALE_F32) return reinterpret_cast<const float*>(p)[idx];
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[idx]);
}

__device__ __forceinline__ void row_range(const int64_t* offsets, int64_t e, int64_t T, int64_t& a, int64_t& b) {
  if (offsets == nullptr) {
    a = 0;
    b = T;
    return;
  }
  a = offsets[e];
  b = offsets[e + 1];
  // Offsets that were not validated on the host are clamped so no row index leaves [0, T).
  a = a < 0 ? 0 : (a > T ? T : a);
  b = b < a ? a : (b > T ? T : b);
}

}  // namespace dst
