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

// One block per token row: absmax, then q = clamp(rint(x / s)).
template <typename XT>
__global__ void quant_act_kernel(const XT* __restrict__ x, int64_t K, int8_t* __restrict__ q,
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
    q[m * K + k] = (int8_t)r;
  }
}

int grid_for(int64_t total, int block) {
  int64_t g = (total + block - 1) / block;
  const int64_t cap = 148 * 16;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace
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
    dst::quant_act_kernel<float><<<(unsigned)M, 256, 0, st>>>(static_cast<const float*>(x), K, q, s);
  else
    dst::quant_act_kernel<__nv_bfloat16><<<(unsigned)M, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), K, q, s);
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}
