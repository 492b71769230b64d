// Generic ternary grouped GEMM on CUDA cores: covers every shape the C ABI accepts (any K, group,
// N, row count, 1..4 stacked terms, bf16 / f16 / int8 activations, f16 / f32 / bf16 scales).
// It is the kernel for shapes the two fast kernels do not cover (ragged K, short last group,
// group != 128) and the one the fast kernels are first validated against on the device.
//
// Work split: one warp per output row n, eight rows per block, one block column per expert; the
// block walks its expert's token rows in tiles of TOK. Inside a scale group the lanes stride over k,
// so activation loads are coalesced and each lane keeps a partial group sum (exact int32 for int8
// activations); the lane multiplies its partial by the group scale and the warp reduces once per
// token tile. Same contract as the reference kernels
// (boilerplate/kernels/csrc/ternary_cuda_kernel.cu:44-99, boilerplate_cpu.cpp:109-127).
#include "dst_common.cuh"

namespace dst {
namespace {

constexpr int WARPS = 8;
constexpr int TOK = 8;

template <int ACT>
struct ActT;
template <>
struct ActT<DST_ACT_BF16> { using type = __nv_bfloat16; using acc = float; };
template <>
struct ActT<DST_ACT_F16> { using type = __half; using acc = float; };
template <>
struct ActT<DST_ACT_I8> { using type = int8_t; using acc = int; };

template <int FMT, int ACT>
__global__ void __launch_bounds__(WARPS * 32)
generic_kernel(GemmArgs a) {
  using XT = typename ActT<ACT>::type;
  using AccT = typename ActT<ACT>::acc;
  __shared__ uint16_t lut[256];
  if (FMT == 1) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) lut[i] = (uint16_t)tq1_fields(i);
    __syncthreads();
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t e = blockIdx.y;
  const int64_t n = (int64_t)blockIdx.x * WARPS + warp;
  int64_t ra, rb;
  row_range(a.offsets, e, a.T, ra, rb);
  if (n >= a.N || ra >= rb) return;  // no block-wide barrier below this point
  const XT* __restrict__ x = static_cast<const XT*>(a.x);
  const int64_t K = a.K, G = a.G, group = a.group;

  for (int64_t row0 = ra; row0 < rb; row0 += TOK) {
    const int rows = (int)(rb - row0 < TOK ? rb - row0 : TOK);
    float y[TOK];
#pragma unroll
    for (int r = 0; r < TOK; ++r) y[r] = 0.f;
    for (int i = 0; i < a.terms.n; ++i) {
      const uint8_t* __restrict__ wrow = a.terms.packed[i] + (e * a.N + n) * a.Kp;
      const int64_t sbase = (e * a.N + n) * G;
      for (int64_t g = 0; g < G; ++g) {
        const int64_t k0 = g * group, k1 = k0 + group < K ? k0 + group : K;
        AccT acc[TOK];
#pragma unroll
        for (int r = 0; r < TOK; ++r) acc[r] = 0;
        for (int64_t k = k0 + lane; k < k1; k += 32) {
          int t;
          if (FMT == 2) {
            t = (int)((wrow[k >> 2] >> ((k & 3) * 2)) & 3) - 1;
          } else {
            const int64_t b = k / 5;
            t = (int)((lut[wrow[b]] >> ((int)(k - b * 5) * 2)) & 3) - 1;
          }
          if (t == 0) continue;
#pragma unroll
          for (int r = 0; r < TOK; ++r) {
            if (r < rows) {
              if (ACT == DST_ACT_I8) acc[r] += (AccT)t * (AccT)x[(row0 + r) * K + k];
              else acc[r] = (AccT)fmaf((float)t, (float)x[(row0 + r) * K + k], (float)acc[r]);
            }
          }
        }
        const float s = scale_to_float(a.terms.scale[i], sbase + g, a.scale_dtype);
#pragma unroll
        for (int r = 0; r < TOK; ++r) y[r] = fmaf(s, (float)acc[r], y[r]);
      }
    }
#pragma unroll
    for (int r = 0; r < TOK; ++r) {
      float v = y[r];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
      y[r] = v;
    }
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < TOK; ++r) {
        if (r < rows) {
          const int64_t o = (row0 + r) * a.N + n;
          float v = y[r];
          if (a.row_scale) v *= a.row_scale[row0 + r];
          if (a.out_dtype == DST_OUT_F32) {
            float* out = static_cast<float*>(a.out);
            out[o] = a.accumulate ? out[o] + v : v;
          } else if (a.out_dtype == DST_OUT_BF16) {
            static_cast<__nv_bfloat16*>(a.out)[o] = __float2bfloat16_rn(v);
          } else {
            static_cast<__half*>(a.out)[o] = __float2half_rn(v);
          }
        }
      }
    }
  }
}

template <int FMT>
int launch_fmt(const GemmArgs& a, dim3 grid, cudaStream_t st) {
  switch (a.act_dtype) {
    case DST_ACT_BF16: generic_kernel<FMT, DST_ACT_BF16><<<grid, WARPS * 32, 0, st>>>(a); break;
    case DST_ACT_F16: generic_kernel<FMT, DST_ACT_F16><<<grid, WARPS * 32, 0, st>>>(a); break;
    case DST_ACT_I8: generic_kernel<FMT, DST_ACT_I8><<<grid, WARPS * 32, 0, st>>>(a); break;
    default: return DST_ERR_BAD_ARG;
  }
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}

}  // namespace

int launch_generic(const GemmArgs& a, cudaStream_t stream) {
  if (a.T == 0 || a.N == 0 || a.E == 0) return DST_OK;
  const dim3 grid((unsigned)cdiv64(a.N, WARPS), (unsigned)a.E, 1);
  return a.fmt == DST_FMT_TQ2 ? launch_fmt<2>(a, grid, stream) : launch_fmt<1>(a, grid, stream);
}

}  // namespace dst
