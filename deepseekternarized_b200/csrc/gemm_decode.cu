// Decode GEMV / grouped GEMV for few token rows per expert: bound by HBM bandwidth on the packed weights.
//
//     out[m, n] = row_scale[m] * sum_i sum_g scale_i[e, n, g] * sum_{k in g} x[m, k] * trit_i[e, n, k]
//
// Every packed byte is read once, with 128-bit loads that are contiguous across a warp (tiled layout, see
// layout_kernels.cu: a quad of lanes reads one weight row's 64-byte superblock, eight rows are 512 contiguous
// bytes). The multiply-adds run on mma.sync.m16n8k16 (fp16 in, fp32 accumulate) fed straight from registers:
//
//   A fragment  a weight row's packed word ANDed with a 2-bit field mask IS the operand: the fp16 bit pattern
//               with only mantissa bits set is the denormal u * 4^j * 2^-24 (u = t + 1 in {0,1,2}). The tensor
//               core takes fp16 denormals exactly on this hardware (measured), so unpacking costs one AND per
//               two weights and no conversion.
//   B fragment  the token rows, staged once per expert in shared memory as fp16 multiplied by the matching
//               4^-j (and a per-token power of two that brings the row's maximum below 256), so the product
//               is u * x * 2^-17 for every field position.
//   offset      sum_k u_k x_k = sum_k t_k x_k + sum_k x_k: the per-(token, group) sums of x are computed at
//               staging time from the same rounded values and subtracted per scale group.
//
// One warp owns 16 weight rows of a 128-row tile and walks K in 256-trit superblocks (two scale groups); per
// 128-trit group the fp32 accumulator is scaled by the group's fp16 scale and added to the row's result, the
// structure of the reference kernels (boilerplate/kernels/csrc/boilerplate_cpu.cpp:116-124). Work items
// (expert, row tile) are dealt to CTAs in contiguous ranges so an expert's token rows are staged once per CTA.
//
// Coverage: TQ2 tiled weights, group 128, K % 256 == 0, fp16 scales, bf16 or fp16 activations, any row count
// per expert (rows are processed 16 at a time; beyond that the weights are re-read, from L2).
#include "dst_common.cuh"

namespace dst {
namespace {

constexpr int DC_WARPS = 8;
constexpr int DC_THREADS = DC_WARPS * 32;

struct DecodeParams {
  const uint8_t* tiled[DST_MAX_TERMS];
  const __half* scale[DST_MAX_TERMS];
  int n_terms;
  const void* x;
  int act_dtype;
  const float* row_scale;
  const int64_t* offsets;
  void* out;
  int out_dtype, accumulate;
  int E, T, N, K, G, NT, S;
  int xstride;  // bytes between staged token rows: K * 2 + 16 (an odd multiple of 16 bytes: conflict-free B loads)
};

__device__ __forceinline__ void mma_f16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Field j (0..7) of a tiled TQ2 word pairs trits 2j (low half) and 2j+1 (high half). Fields 0..4 are used in
// place (value u * 4^j * 2^-24), fields 5..7 after a shift by 10 (value u * 4^(j-5) * 2^-24).
__device__ __forceinline__ int field_shift(int j) { return j < 5 ? j : j - 5; }

// Stage the token rows [m0, m0 + mc) of x into shared memory:
//   xs[m][k] = fp16( x[m][k] * 2^(7 - e_m - 2 f(j)) ),  j = (k % 16) / 2,  e_m = floor(log2(rowmax)) - 7
//   xsum[m][g] = sum over group g of the values the tensor core will see, undone to x * 2^-e_m
//   xexp[m] = 2^e_m * row_scale[m]
template <int MT, typename XT>
__device__ void stage_tokens(const DecodeParams& p, const XT* __restrict__ x, int64_t m0, int mc, uint8_t* xs, float* xsum, float* xexp,
                             int* xex) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // pass 1, one warp per token row: the row's power of two. Token slots beyond mc are never read (their B
  // fragments are zero registers), so nothing is written for them.
  for (int m = warp; m < mc; m += DC_WARPS) {
    const XT* row = x + (m0 + m) * p.K;
    float amax = 0.f;
    for (int k = lane; k < p.K; k += 32) amax = fmaxf(amax, fabsf((float)row[k]));
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    int ex = 0;
    if (amax > 0.f && isfinite(amax)) {
      (void)frexpf(amax, &ex);
      ex -= 8;  // amax * 2^-ex in [128, 256)
    }
    if (lane == 0) {
      xex[m] = ex;
      xexp[m] = ldexpf(1.f, ex) * (p.row_scale ? p.row_scale[m0 + m] : 1.f);
    }
  }
  __syncthreads();
  // pass 2, one warp per (token row, 128-trit group): 32 lanes x 4 consecutive k
  for (int u = warp; u < mc * p.G; u += DC_WARPS) {
    const int m = u / p.G, g = u - m * p.G;
    const XT* row = x + (m0 + m) * p.K;
    __half* dst = reinterpret_cast<__half*>(xs + (size_t)m * p.xstride);
    const int ex = xex[m];
    const int k = g * 128 + lane * 4;
    float part = 0.f;
    uint32_t packed[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int kk = k + 2 * h;
      const int f = field_shift((kk & 15) >> 1);
      const float mul = ldexpf(1.f, 7 - ex - 2 * f), undo = ldexpf(1.f, 2 * f - 7);
      const __half v0 = __float2half_rn((float)row[kk] * mul), v1 = __float2half_rn((float)row[kk + 1] * mul);
      part += (__half2float(v0) + __half2float(v1)) * undo;
      packed[h] = (uint32_t)__half_as_ushort(v0) | ((uint32_t)__half_as_ushort(v1) << 16);
    }
    *reinterpret_cast<uint2*>(dst + k) = make_uint2(packed[0], packed[1]);
    for (int off = 16; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
    if (lane == 0) xsum[m * p.G + g] = part;
  }
}

template <int NB>  // NB = 1: up to 8 token rows per pass, NB = 2: up to 16
__global__ void __launch_bounds__(DC_THREADS)
decode_kernel(const DecodeParams p) {
  extern __shared__ __align__(16) uint8_t dsm[];
  constexpr int MT = NB * 8;                                        // token rows staged per pass
  uint8_t* xs = dsm;                                                // MT staged token rows
  float* xsum = reinterpret_cast<float*>(dsm + (size_t)MT * p.xstride);  // [MT][G]
  float* xexp = xsum + MT * p.G;                                    // [MT]
  int* xex = reinterpret_cast<int*>(xexp + MT);                     // [MT] exponent of the row's power of two
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g8 = lane >> 2, c = lane & 3;

  // contiguous range of (expert, row tile) items for this CTA
  const long long items = (long long)p.E * p.NT;
  const long long per = (items + gridDim.x - 1) / gridDim.x;
  const long long i0 = (long long)blockIdx.x * per, i1 = i0 + per < items ? i0 + per : items;
  int staged_e = -1;
  int64_t staged_m0 = -1;

  for (long long item = i0; item < i1; ++item) {
    const int e = (int)(item / p.NT), nt = (int)(item - (long long)e * p.NT);
    int64_t ra, rb;
    row_range(p.offsets, e, p.T, ra, rb);
    for (int64_t m0 = ra; m0 < rb; m0 += NB * 8) {
      const int mc = (int)(rb - m0 < NB * 8 ? rb - m0 : NB * 8);
      if (staged_e != e || staged_m0 != m0) {
        __syncthreads();  // everyone is done with the previous rows
        if (p.act_dtype == DST_ACT_BF16) stage_tokens<MT>(p, static_cast<const __nv_bfloat16*>(p.x), m0, mc, xs, xsum, xexp, xex);
        else stage_tokens<MT>(p, static_cast<const __half*>(p.x), m0, mc, xs, xsum, xexp, xex);
        __syncthreads();
        staged_e = e;
        staged_m0 = m0;
      }
      const int r0 = warp * 16 + g8;  // this lane's rows inside the tile: r0 and r0 + 8 (same swizzle)
      const int swz = (r0 >> 1) & 3;
      const int n_lo = nt * 128 + r0, n_hi = n_lo + 8;
      float y[NB][4];
#pragma unroll
      for (int b = 0; b < NB; ++b)
#pragma unroll
        for (int i = 0; i < 4; ++i) y[b][i] = 0.f;

      for (int term = 0; term < p.n_terms; ++term) {
        const uint8_t* wbase = p.tiled[term] + (((int64_t)e * p.NT + nt) * p.S) * 8192 + ((c ^ swz) << 4);
        const __half* s_lo = p.scale[term] + ((int64_t)e * p.N + (n_lo < p.N ? n_lo : 0)) * p.G;
        const __half* s_hi = p.scale[term] + ((int64_t)e * p.N + (n_hi < p.N ? n_hi : 0)) * p.G;
        // words c, 4 + c, 8 + c, 12 + c of rows r0 and r0 + 8, prefetched two superblocks ahead
        const uint8_t* wl_ptr = wbase + (size_t)r0 * 64;
        const uint8_t* wh_ptr = wbase + (size_t)(r0 + 8) * 64;
        const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
        uint4 w_lo = *reinterpret_cast<const uint4*>(wl_ptr), w_hi = *reinterpret_cast<const uint4*>(wh_ptr);
        uint4 w_lo2 = p.S > 1 ? *reinterpret_cast<const uint4*>(wl_ptr + 8192) : zero4;
        uint4 w_hi2 = p.S > 1 ? *reinterpret_cast<const uint4*>(wh_ptr + 8192) : zero4;
        for (int sb = 0; sb < p.S; ++sb) {
          const uint4 cur_lo = w_lo, cur_hi = w_hi;
          w_lo = w_lo2;
          w_hi = w_hi2;
          if (sb + 2 < p.S) {
            w_lo2 = *reinterpret_cast<const uint4*>(wl_ptr + (size_t)(sb + 2) * 8192);
            w_hi2 = *reinterpret_cast<const uint4*>(wh_ptr + (size_t)(sb + 2) * 8192);
          }
          const uint32_t wl[4] = {cur_lo.x, cur_lo.y, cur_lo.z, cur_lo.w}, wh[4] = {cur_hi.x, cur_hi.y, cur_hi.z, cur_hi.w};
#pragma unroll
          for (int half = 0; half < 2; ++half) {  // one 128-trit scale group: chunks 2 half, 2 half + 1
            const int grp = sb * 2 + half;
            float acc[NB][4];
#pragma unroll
            for (int b = 0; b < NB; ++b)
#pragma unroll
              for (int i = 0; i < 4; ++i) acc[b][i] = 0.f;
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
              const int ch = half * 2 + cc;
              const uint32_t a_lo = wl[ch], a_hi = wh[ch], a_lo2 = a_lo >> 10, a_hi2 = a_hi >> 10;
              // this lane's 16 k of the chunk: k = 256 sb + 64 ch + 16 c .. + 15, as 8 fp16 pairs per token
              const int koff = (sb * 256 + ch * 64 + c * 16) * 2;
              uint4 q[NB][2];
#pragma unroll
              for (int b = 0; b < NB; ++b) {
                // token columns that do not exist are zero registers: no shared-memory traffic for them
                if (b * 8 + g8 < mc) {
                  const uint8_t* xr = xs + (size_t)(b * 8 + g8) * p.xstride + koff;
                  q[b][0] = *reinterpret_cast<const uint4*>(xr);
                  q[b][1] = *reinterpret_cast<const uint4*>(xr + 16);
                } else {
                  q[b][0] = zero4;
                  q[b][1] = zero4;
                }
              }
#pragma unroll
              for (int jj = 0; jj < 4; ++jj) {
                // pairs jj (in place) and jj + 4 (jj = 0 in place at field 4, else from the shifted word)
                const uint32_t m_a = 0x00030003u << (2 * jj);
                const uint32_t a0 = a_lo & m_a, a1 = a_hi & m_a;
                uint32_t a2, a3;
                if (jj == 0) {
                  a2 = a_lo & 0x03000300u;
                  a3 = a_hi & 0x03000300u;
                } else {
                  const uint32_t m_b = 0x00030003u << (2 * (jj - 1));
                  a2 = a_lo2 & m_b;
                  a3 = a_hi2 & m_b;
                }
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                  const uint32_t b0 = jj == 0 ? q[b][0].x : jj == 1 ? q[b][0].y : jj == 2 ? q[b][0].z : q[b][0].w;
                  const uint32_t b1 = jj == 0 ? q[b][1].x : jj == 1 ? q[b][1].y : jj == 2 ? q[b][1].z : q[b][1].w;
                  mma_f16(acc[b], a0, a1, a2, a3, b0, b1);
                }
              }
            }
            // group done: y += scale[row][grp] * (2^17 acc - sum_k x); C fragment = (row r0 | r0 + 8) x (token 2c | 2c + 1)
            const float sl = grp < p.G ? __half2float(s_lo[grp]) : 0.f, sh = grp < p.G ? __half2float(s_hi[grp]) : 0.f;
#pragma unroll
            for (int b = 0; b < NB; ++b) {
              const float x0 = xsum[(b * 8 + 2 * c) * p.G + grp], x1 = xsum[(b * 8 + 2 * c + 1) * p.G + grp];
              y[b][0] = fmaf(sl, fmaf(acc[b][0], 131072.f, -x0), y[b][0]);
              y[b][1] = fmaf(sl, fmaf(acc[b][1], 131072.f, -x1), y[b][1]);
              y[b][2] = fmaf(sh, fmaf(acc[b][2], 131072.f, -x0), y[b][2]);
              y[b][3] = fmaf(sh, fmaf(acc[b][3], 131072.f, -x1), y[b][3]);
            }
          }
        }
      }
      // store: rows n_lo / n_hi, tokens m0 + b * 8 + 2c (+1)
#pragma unroll
      for (int b = 0; b < NB; ++b) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int tok = b * 8 + 2 * c + (i & 1);
          const int n = i < 2 ? n_lo : n_hi;
          if (tok < mc && n < p.N) {
            const float v = y[b][i] * xexp[tok];
            const int64_t o = (m0 + tok) * p.N + n;
            if (p.out_dtype == DST_OUT_F32) {
              float* out = static_cast<float*>(p.out);
              out[o] = p.accumulate ? out[o] + v : v;
            } else if (p.out_dtype == DST_OUT_BF16) {
              static_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(v);
            } else {
              static_cast<__half*>(p.out)[o] = __float2half_rn(v);
            }
          }
        }
      }
    }
  }
}

}  // namespace

bool decode_supports(const GemmArgs& a) {
  if (a.fmt == DST_FMT_TQ1) return decode_tq1_supports(a);
  return a.weight_layout == DST_LAYOUT_TILED && a.fmt == DST_FMT_TQ2 && a.group == 128 && a.K % 256 == 0 &&
         a.scale_dtype == DST_SCALE_F16 && (a.act_dtype == DST_ACT_BF16 || a.act_dtype == DST_ACT_F16) &&
         (size_t)16 * (a.K * 2 + 16) + (size_t)16 * (a.G + 2) * 4 <= 200 * 1024 && a.T < (int64_t(1) << 31);
}

int launch_decode(const GemmArgs& a, cudaStream_t stream) {
  if (a.T == 0 || a.N == 0 || a.E == 0) return DST_OK;
  if (a.fmt == DST_FMT_TQ1) return launch_decode_tq1(a, stream);
  if (!decode_supports(a)) return DST_ERR_UNSUPPORTED;
  for (int i = 0; i < a.terms.n; ++i)
    if ((reinterpret_cast<uintptr_t>(a.terms.packed[i]) & 15) != 0 || (reinterpret_cast<uintptr_t>(a.terms.scale[i]) & 1) != 0)
      return DST_ERR_ALIGNMENT;
  DecodeParams p;
  for (int i = 0; i < DST_MAX_TERMS; ++i) {
    p.tiled[i] = i < a.terms.n ? a.terms.packed[i] : nullptr;
    p.scale[i] = i < a.terms.n ? static_cast<const __half*>(a.terms.scale[i]) : nullptr;
  }
  p.n_terms = a.terms.n;
  p.x = a.x;
  p.act_dtype = a.act_dtype;
  p.row_scale = a.row_scale;
  p.offsets = a.offsets;
  p.out = a.out;
  p.out_dtype = a.out_dtype;
  p.accumulate = a.accumulate;
  p.E = (int)a.E;
  p.T = (int)a.T;
  p.N = (int)a.N;
  p.K = (int)a.K;
  p.G = (int)a.G;
  p.NT = (int)cdiv64(a.N, 128);
  p.S = (int)tiled_superblocks(a.fmt, a.K);
  p.xstride = (int)(a.K * 2 + 16);
  // up to 8 rows per expert (known on the host, or guessed from the mean) -> one token block per pass
  const int64_t rows_hint = a.max_rows >= 0 ? a.max_rows : cdiv64(a.T, a.E);
  int dev = 0, sms = 148;
  DST_CUDA_TRY(cudaGetDevice(&dev));
  DST_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const long long items = (long long)p.E * p.NT;
  const int nb = rows_hint <= 8 ? 1 : 2;
  const size_t smem = (size_t)nb * 8 * p.xstride + (size_t)nb * 8 * (p.G + 2) * 4;
  // as many CTAs per SM as the staged token rows allow (up to 3: 24 warps keep enough loads in flight)
  int per_sm = (int)((220 * 1024) / (smem + 1024));
  per_sm = per_sm < 1 ? 1 : (per_sm > 3 ? 3 : per_sm);
  const long long want = (long long)sms * per_sm;
  const int grid = (int)(items < want ? items : want);
  if (nb == 1) {
    DST_CUDA_TRY(cudaFuncSetAttribute(decode_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    decode_kernel<1><<<grid, DC_THREADS, smem, stream>>>(p);
  } else {
    DST_CUDA_TRY(cudaFuncSetAttribute(decode_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    decode_kernel<2><<<grid, DC_THREADS, smem, stream>>>(p);
  }
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}

}  // namespace dst
