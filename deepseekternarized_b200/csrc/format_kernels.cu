// TQ1 / TQ2 pack and unpack on the device, plus per-token int8 activation quantisation.
// Format contract: boilerplate/ternary/pack.py:1-82 of the reference project.
#include "dst_common.cuh"

namespace dst {
namespace {

// One thread per packed byte: gathers `per` trits (digit 1 where k >= K) into one byte.
template <int FMT>
__global__ void pack_kernel(const int8_t* __restrict__ trits, int64_t N, int64_t K, int64_t Kp,
                            uint8_t* __restrict__ packed) {
  constexpr int PER = FMT == 2 ? 4 : 5;
  const int64_t total = N * Kp;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t n = i / Kp, b = i - n * Kp;
    const int8_t* row = trits + n * K;
    uint32_t v = 0, mul = 1;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int64_t k = b * PER + j;
      const uint32_t u = k < K ? (uint32_t)(row[k] + 1) : 1u;
      if (FMT == 2) {
        v |= (u & 3u) << (2 * j);
      } else {
        v += u * mul;
        mul *= 3u;
      }
    }
    packed[i] = (uint8_t)v;
  }
}

// One thread per packed byte: writes its (up to) `per` trits.
template <int FMT>
__global__ void unpack_kernel(const uint8_t* __restrict__ packed, int64_t N, int64_t K, int64_t Kp,
                              int8_t* __restrict__ trits) {
  constexpr int PER = FMT == 2 ? 4 : 5;
  const int64_t total = N * Kp;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t n = i / Kp, b = i - n * Kp;
    const uint32_t v = packed[i];
    const uint32_t f = FMT == 2 ? v : tq1_fields(v);
    int8_t* row = trits + n * K;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int64_t k = b * PER + j;
      if (k < K) row[k] = (int8_t)((int)((f >> (2 * j)) & 3u) - 1);
    }
  }
}

// One block per token row: absmax, then q = clamp(rint(x / s)), stored as int8 or as the same integers in fp16.
template <typename XT, typename QT>
__global__ void quant_act_kernel(const XT* __restrict__ x, int64_t K, QT* __restrict__ q,
                                 float* __restrict__ s) {
  __shared__ float red[32];
  const int64_t m = blockIdx.x;
  const XT* row = x + m * K;
  float amax = 0.f;
  for (int64_t k = threadIdx.x; k < K; k += blockDim.x) amax = fmaxf(amax, fabsf((float)row[k]));
  for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x + 31) / 32 ? red[threadIdx.x] : 0.f;
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    if (threadIdx.x == 0) red[0] = v;
  }
  __syncthreads();
  const float sc = fmaxf(__fdiv_rn(red[0], 127.0f), 1e-8f);
  if (threadIdx.x == 0) s[m] = sc;
  for (int64_t k = threadIdx.x; k < K; k += blockDim.x) {
    float r = rintf(__fdiv_rn((float)row[k], sc));  // round half to even, as torch.round
    r = fminf(fmaxf(r, -127.f), 127.f);
    q[m * K + k] = (QT)r;  // int8, or the same integer as fp16 (exact: |r| <= 127)
  }
}

int grid_for(int64_t total, int block) {
  int64_t g = (total + block - 1) / block;
  const int64_t cap = 148 * 16;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

// Ternary lookup table rows: out[i, :] = bf16( sum over terms of trit * scale ), fp32 products added in term order
// (boilerplate/engine/model.py:458-464: unpack(packed[ids]) * scale[ids].repeat_interleave(group), summed, -> bf16).
// One block per looked-up row; an id outside [0, V) is counted and its row written as zeros.
// Row r of term t starts at packed[t] + r * pstride bytes and its scales at element r * sstride of scale[t] (canonical
// arrays: Kp and G; one record per row holding all terms: the record's size in bytes and in scale elements).
template <int FMT>
__global__ void gather_dequant_kernel(Terms terms, int scale_dtype, const int64_t* __restrict__ ids, int64_t V, int64_t K, int64_t Kp,
                                      int64_t pstride, int64_t sstride, int64_t group, __nv_bfloat16* __restrict__ out,
                                      int32_t* __restrict__ bad_count) {
  constexpr int PER = FMT == 2 ? 4 : 5;
  const int64_t i = blockIdx.x;
  const int64_t row = ids[i];
  __nv_bfloat16* o = out + i * K;
  if (row < 0 || row >= V) {
    if (threadIdx.x == 0 && bad_count) atomicAdd(bad_count, 1);
    for (int64_t k = threadIdx.x; k < K; k += blockDim.x) o[k] = __float2bfloat16_rn(0.f);
    return;
  }
  for (int64_t b = threadIdx.x; b < Kp; b += blockDim.x) {
    float acc[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) acc[j] = 0.f;
    for (int t = 0; t < terms.n; ++t) {
      const uint32_t v = terms.packed[t][row * pstride + b];
      const uint32_t f = FMT == 2 ? v : tq1_fields(v);
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int64_t k = b * PER + j;
        if (k < K) {
          const float val = (float)((int)((f >> (2 * j)) & 3u) - 1) * scale_to_float(terms.scale[t], row * sstride + k / group, scale_dtype);
          acc[j] = t == 0 ? val : acc[j] + val;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int64_t k = b * PER + j;
      if (k < K) o[k] = __float2bfloat16_rn(acc[j]);
    }
  }
}

// The same lookup for K % 8 == 0 and group % 8 == 0 (the engram tables: K = 256, group 128): one thread per eight
// adjacent outputs = one 16-byte store, a warp per 256-wide row. TQ2: the eight trits are one aligned 16-bit load.
// TQ1: they lie in two or three bytes; the bytes' digit fields (a 256-entry table in shared memory) laid side by side
// are 15 two-bit digits in one word, shifted down to the first wanted trit. A thread takes ROWS looked-up rows at a
// time and issues all their loads (ids, then packed bytes and scales of every term) before it uses any: the lookup is
// a chain of dependent random reads, and only many of them in flight fill the memory system.
template <int FMT, int ROWS, int TERMS>
__global__ void __launch_bounds__(256)
gather_dequant8_kernel(Terms terms, int scale_dtype, const int64_t* __restrict__ ids, int64_t n_ids, int64_t V, int K, int Kp,
                       int64_t pstride, int64_t sstride, int group, __nv_bfloat16* __restrict__ out, int32_t* __restrict__ bad_count) {
  __shared__ uint16_t lut[256];
  if (FMT == 1) {
    for (int v = threadIdx.x; v < 256; v += blockDim.x) lut[v] = (uint16_t)tq1_fields((uint32_t)v);
    __syncthreads();
  }
  const int per_row = K >> 3;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t i0 = (tid / per_row) * ROWS;  // this thread's first looked-up row; the block of ROWS rows is its warp's (K = 256)
  if (i0 >= n_ids) return;
  const int c = (int)(tid % per_row), k = c << 3;
  const int b0 = k / 5, r = k - 5 * b0, g = k / group;
  int64_t row[ROWS];
#pragma unroll
  for (int j = 0; j < ROWS; ++j) row[j] = i0 + j < n_ids ? ids[i0 + j] : -1;
  uint32_t raw[ROWS][TERMS];  // TQ2: the 16 bits; TQ1: three bytes
  float sc[ROWS][TERMS];
#pragma unroll
  for (int j = 0; j < ROWS; ++j) {
    const bool ok = row[j] >= 0 && row[j] < V;
#pragma unroll
    for (int t = 0; t < TERMS; ++t) {
      raw[j][t] = 0u;
      sc[j][t] = 0.f;
      if (ok) {
        const uint8_t* pr = terms.packed[t] + row[j] * pstride;
        if (FMT == 2) {
          raw[j][t] = *reinterpret_cast<const uint16_t*>(pr + (k >> 2));
        } else {
          uint32_t w = pr[b0];
          if (b0 + 1 < Kp) w |= (uint32_t)pr[b0 + 1] << 8;
          if (r > 2 && b0 + 2 < Kp) w |= (uint32_t)pr[b0 + 2] << 16;  // trits 5 b0 + 10 ... are wanted from r = 3 on
          raw[j][t] = w;  // a byte not read holds trits beyond the eight wanted ones (K % 8 == 0 keeps those inside the row)
        }
        sc[j][t] = scale_to_float(terms.scale[t], row[j] * sstride + g, scale_dtype);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < ROWS; ++j) {
    if (i0 + j >= n_ids) break;
    uint4* o = reinterpret_cast<uint4*>(out + (i0 + j) * K + k);
    if (row[j] < 0 || row[j] >= V) {
      if (c == 0 && bad_count) atomicAdd(bad_count, 1);
      *o = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    float acc[8];
#pragma unroll
    for (int t = 0; t < TERMS; ++t) {
      uint32_t f;  // eight 2-bit digits u = trit + 1
      if (FMT == 2) {
        f = raw[j][t];
      } else {
        const uint32_t w = raw[j][t];
        f = ((uint32_t)lut[w & 0xff] | ((uint32_t)lut[(w >> 8) & 0xff] << 10) | ((uint32_t)lut[(w >> 16) & 0xff] << 20)) >> (2 * r);
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float val = (float)((int)((f >> (2 * q)) & 3u) - 1) * sc[j][t];
        acc[q] = t == 0 ? val : acc[q] + val;
      }
    }
    uint32_t w[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
      w[q] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *o = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

template <int FMT, int TERMS>
void launch_gather8(const Terms& terms, int scale_dtype, const int64_t* ids, int64_t n_ids, int64_t V, int K, int Kp, int64_t pstride,
                    int64_t sstride, int group, __nv_bfloat16* out, int32_t* bad_count, cudaStream_t st) {
  constexpr int ROWS = 4;
  const int64_t threads = ((n_ids + ROWS - 1) / ROWS) * (K / 8);
  gather_dequant8_kernel<FMT, ROWS, TERMS><<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(terms, scale_dtype, ids, n_ids, V, K, Kp, pstride,
                                                                                           sstride, group, out, bad_count);
}
template <int FMT>
void launch_gather8(const Terms& terms, int scale_dtype, const int64_t* ids, int64_t n_ids, int64_t V, int K, int Kp, int64_t pstride,
                    int64_t sstride, int group, __nv_bfloat16* out, int32_t* bad_count, cudaStream_t st) {
  switch (terms.n) {
    case 1: return launch_gather8<FMT, 1>(terms, scale_dtype, ids, n_ids, V, K, Kp, pstride, sstride, group, out, bad_count, st);
    case 2: return launch_gather8<FMT, 2>(terms, scale_dtype, ids, n_ids, V, K, Kp, pstride, sstride, group, out, bad_count, st);
    case 3: return launch_gather8<FMT, 3>(terms, scale_dtype, ids, n_ids, V, K, Kp, pstride, sstride, group, out, bad_count, st);
    default: return launch_gather8<FMT, 4>(terms, scale_dtype, ids, n_ids, V, K, Kp, pstride, sstride, group, out, bad_count, st);
  }
}

}  // namespace dst

extern "C" int64_t dst_packed_cols(int fmt, int64_t K) {
  if ((fmt != DST_FMT_TQ1 && fmt != DST_FMT_TQ2) || K <= 0) return -1;
  return dst::cdiv64(K, fmt == DST_FMT_TQ2 ? 4 : 5);
}

extern "C" int dst_pack(const int8_t* trits, int64_t N, int64_t K, int fmt, uint8_t* packed,
                        dst_stream_t stream) {
  if ((fmt != DST_FMT_TQ1 && fmt != DST_FMT_TQ2) || K <= 0 || N < 0) return DST_ERR_BAD_ARG;
  if (N == 0) return DST_OK;
  if (!trits || !packed) return DST_ERR_BAD_ARG;
  if (K > (int64_t(1) << 40) || N > (int64_t(1) << 40) / K) return DST_ERR_BAD_SHAPE;
  const int64_t Kp = dst_packed_cols(fmt, K);
  auto st = static_cast<cudaStream_t>(stream);
  const int grid = dst::grid_for(N * Kp, 256);
  if (fmt == DST_FMT_TQ2) dst::pack_kernel<2><<<grid, 256, 0, st>>>(trits, N, K, Kp, packed);
  else dst::pack_kernel<1><<<grid, 256, 0, st>>>(trits, N, K, Kp, packed);
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}

extern "C" int dst_unpack(const uint8_t* packed, int64_t N, int64_t K, int fmt, int8_t* trits,
                          dst_stream_t stream) {
  if ((fmt != DST_FMT_TQ1 && fmt != DST_FMT_TQ2) || K <= 0 || N < 0) return DST_ERR_BAD_ARG;
  if (N == 0) return DST_OK;
  if (!trits || !packed) return DST_ERR_BAD_ARG;
  if (K > (int64_t(1) << 40) || N > (int64_t(1) << 40) / K) return DST_ERR_BAD_SHAPE;
  const int64_t Kp = dst_packed_cols(fmt, K);
  auto st = static_cast<cudaStream_t>(stream);
  const int grid = dst::grid_for(N * Kp, 256);
  if (fmt == DST_FMT_TQ2) dst::unpack_kernel<2><<<grid, 256, 0, st>>>(packed, N, K, Kp, trits);
  else dst::unpack_kernel<1><<<grid, 256, 0, st>>>(packed, N, K, Kp, trits);
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}

extern "C" int dst_quant_act_int8(const void* x, int x_is_f32, int64_t M, int64_t K, int8_t* q, float* s,
                                  dst_stream_t stream) {
  if (K <= 0 || M < 0) return DST_ERR_BAD_ARG;
  if (M == 0) return DST_OK;
  if (!x || !q || !s) return DST_ERR_BAD_ARG;
  if (M > 0x7fffffff) return DST_ERR_BAD_SHAPE;
  auto st = static_cast<cudaStream_t>(stream);
  if (x_is_f32)
    dst::quant_act_kernel<float, int8_t><<<(unsigned)M, 256, 0, st>>>(static_cast<const float*>(x), K, q, s);
  else
    dst::quant_act_kernel<__nv_bfloat16, int8_t><<<(unsigned)M, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), K, q, s);
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}

extern "C" int dst_quant_act_int8_f16(const void* x, int x_is_f32, int64_t M, int64_t K, void* q_f16, float* s,
                                      dst_stream_t stream) {
  if (K <= 0 || M < 0) return DST_ERR_BAD_ARG;
  if (M == 0) return DST_OK;
  if (!x || !q_f16 || !s) return DST_ERR_BAD_ARG;
  if (M > 0x7fffffff) return DST_ERR_BAD_SHAPE;
  auto st = static_cast<cudaStream_t>(stream);
  if (x_is_f32)
    dst::quant_act_kernel<float, __half><<<(unsigned)M, 256, 0, st>>>(static_cast<const float*>(x), K, static_cast<__half*>(q_f16), s);
  else
    dst::quant_act_kernel<__nv_bfloat16, __half><<<(unsigned)M, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), K,
                                                                             static_cast<__half*>(q_f16), s);
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}

extern "C" int dst_gather_dequant_rows_strided(const void* const* packed, const void* const* scales, int n_terms, int scale_dtype,
                                               const int64_t* ids, int64_t n_ids, int64_t V, int64_t K, int64_t group, int fmt,
                                               int64_t packed_row_stride, int64_t scale_row_stride, void* out_bf16, int32_t* bad_count,
                                               dst_stream_t stream) {
  if ((fmt != DST_FMT_TQ1 && fmt != DST_FMT_TQ2) || K <= 0 || group <= 0 || V < 0 || n_ids < 0) return DST_ERR_BAD_ARG;
  if (n_terms < 1 || n_terms > DST_MAX_TERMS || scale_dtype < DST_SCALE_F16 || scale_dtype > DST_SCALE_BF16) return DST_ERR_BAD_ARG;
  const int64_t Kp = dst_packed_cols(fmt, K), G = (K + group - 1) / group;
  if (packed_row_stride < Kp || scale_row_stride < G) return DST_ERR_BAD_ARG;
  if (n_ids == 0) return DST_OK;
  if (!packed || !scales || !ids || !out_bf16) return DST_ERR_BAD_ARG;
  if (n_ids > 0x7fffffff || K > (int64_t(1) << 24)) return DST_ERR_BAD_SHAPE;
  dst::Terms terms;
  terms.n = n_terms;
  bool even = packed_row_stride % 2 == 0;  // TQ2 rows are read 16 bits at a time
  for (int i = 0; i < n_terms; ++i) {
    if (!packed[i] || !scales[i]) return DST_ERR_BAD_ARG;
    terms.packed[i] = static_cast<const uint8_t*>(packed[i]);
    terms.scale[i] = scales[i];
    even = even && (reinterpret_cast<uintptr_t>(packed[i]) & 1) == 0;
  }
  auto st = static_cast<cudaStream_t>(stream);
  auto o = static_cast<__nv_bfloat16*>(out_bf16);
  // rows of whole 8-trit pieces that share a scale, output 16-byte aligned: one 16-byte store per thread
  const bool by8 = K % 8 == 0 && group % 8 == 0 && (reinterpret_cast<uintptr_t>(out_bf16) & 15) == 0 && (fmt == DST_FMT_TQ1 || even) &&
                   n_ids * (K / 8) / 256 < 0x7fffffff;
  if (by8) {
    if (fmt == DST_FMT_TQ2)
      dst::launch_gather8<2>(terms, scale_dtype, ids, n_ids, V, (int)K, (int)Kp, packed_row_stride, scale_row_stride, (int)group, o, bad_count, st);
    else
      dst::launch_gather8<1>(terms, scale_dtype, ids, n_ids, V, (int)K, (int)Kp, packed_row_stride, scale_row_stride, (int)group, o, bad_count, st);
  } else if (fmt == DST_FMT_TQ2) {
    dst::gather_dequant_kernel<2><<<(unsigned)n_ids, 128, 0, st>>>(terms, scale_dtype, ids, V, K, Kp, packed_row_stride, scale_row_stride, group, o, bad_count);
  } else {
    dst::gather_dequant_kernel<1><<<(unsigned)n_ids, 128, 0, st>>>(terms, scale_dtype, ids, V, K, Kp, packed_row_stride, scale_row_stride, group, o, bad_count);
  }
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}

extern "C" int dst_gather_dequant_rows(const void* const* packed, const void* const* scales, int n_terms, int scale_dtype,
                                       const int64_t* ids, int64_t n_ids, int64_t V, int64_t K, int64_t group, int fmt, void* out_bf16,
                                       int32_t* bad_count, dst_stream_t stream) {
  if ((fmt != DST_FMT_TQ1 && fmt != DST_FMT_TQ2) || K <= 0 || group <= 0) return DST_ERR_BAD_ARG;
  return dst_gather_dequant_rows_strided(packed, scales, n_terms, scale_dtype, ids, n_ids, V, K, group, fmt, dst_packed_cols(fmt, K),
                                         (K + group - 1) / group, out_bf16, bad_count, stream);
}
