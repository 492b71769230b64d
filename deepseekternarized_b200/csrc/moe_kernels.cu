// The small kernels around the expert GEMMs of a MoE layer: router (softmax + top-k), stable routing
// sort, row gather, SwiGLU and the per-token combine. Semantics follow the reference's V4 MoE layer
// (boilerplate/engine/model.py:376-422) and routing sort (boilerplate/kernels/ternary_cuda.py:114-118).
#include <algorithm>

#include "dst_common.cuh"

namespace dst {
namespace {

// ------------------------------------------------------------------------------------------ router
// One warp per token. score = f(logit / gate_temp) with f = softmax over the E logits, sigmoid, or
// sqrt(softplus) (boilerplate/engine/model.py:389-399); the k experts are picked by k rounds of warp arg-max over
// score + bias (equal keys: lower expert id wins), the weights are the UNBIASED scores of the picked experts,
// optionally renormalised, times route_scale (model.py:400-405).
// A NaN key ranks above every number, as in torch.topk, and every round picks among the experts not picked yet,
// so the k ids of a token are always distinct and inside [0, E) whatever the logits hold (all-NaN and all -inf
// rows included: their weights are NaN, their ids 0..k-1).
constexpr int ROUTE_MAX_PER_LANE = 32;  // E <= 1024

// a ranks above b: NaN above everything, NaNs equal among themselves
__device__ __forceinline__ bool route_above(float a, float b) {
  const bool an = a != a, bn = b != b;
  return an ? !bn : (!bn && a > b);
}

// PL: experts per lane (E <= 32 PL); the loops over a lane's experts are unrolled to that count
template <int PL>
__global__ void route_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int64_t T, int E, int top_k,
                             int score_func, float inv_temp, int renorm, float route_scale, float* __restrict__ weights,
                             int32_t* __restrict__ ids) {
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  const float* row = logits + t * E;
  float v[PL];  // unbiased scores
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < PL; ++j) {
    const int e = j * 32 + lane;
    v[j] = e < E ? row[e] * inv_temp : -INFINITY;
    mx = fmaxf(mx, v[j]);
  }
  if (score_func == DST_SCORE_SOFTMAX) {
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < PL; ++j) {
      const int e = j * 32 + lane;
      v[j] = expf(v[j] - mx);
      if (e < E) sum += v[j];
    }
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    const float inv = 1.f / sum;
#pragma unroll
    for (int j = 0; j < PL; ++j) v[j] *= inv;
  } else if (score_func == DST_SCORE_SIGMOID) {
#pragma unroll
    for (int j = 0; j < PL; ++j) v[j] = 1.f / (1.f + expf(-v[j]));
  } else {  // sqrt(softplus), softplus(x) = x above 20 as torch computes it
#pragma unroll
    for (int j = 0; j < PL; ++j) v[j] = sqrtf(v[j] > 20.f ? v[j] : log1pf(expf(v[j])));
  }
  uint32_t taken = 0;  // bit j: expert j * 32 + lane has been picked
  float wsel[8];
  int isel[8];
  float wsum = 0.f;
  for (int r = 0; r < top_k; ++r) {
    float best = 0.f, best_w = 0.f;
    int bi = 0x7fffffff;  // no candidate in this lane yet
#pragma unroll
    for (int j = 0; j < PL; ++j) {
      const int e = j * 32 + lane;
      if (e < E && !((taken >> j) & 1u)) {
        const float key = bias ? v[j] + bias[e] : v[j];
        if (bi == 0x7fffffff || route_above(key, best)) {  // ascending e within a lane: the first maximum is the lowest id
          best = key;
          best_w = v[j];
          bi = e;
        }
      }
    }
    for (int off = 16; off > 0; off >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, off);
      const float ow = __shfl_xor_sync(0xffffffffu, best_w, off);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
      const bool take = oi != 0x7fffffff && (bi == 0x7fffffff || route_above(ob, best) || (!route_above(best, ob) && oi < bi));
      if (take) {
        best = ob;
        best_w = ow;
        bi = oi;
      }
    }
    // top_k <= E, so some lane always had a candidate: 0 <= bi < E
    if ((bi & 31) == lane) taken |= 1u << (bi >> 5);
    wsel[r] = best_w;
    isel[r] = bi;
    wsum += best_w;
  }
  if (lane == 0) {
    const float d = (renorm && top_k > 1) ? 1.f / (wsum + 1e-20f) : 1.f;
    for (int r = 0; r < top_k; ++r) {
      weights[t * top_k + r] = ((renorm && top_k > 1) ? wsel[r] * d : wsel[r]) * route_scale;
      ids[t * top_k + r] = isel[r];
    }
  }
}

// ------------------------------------------------------------------------------------ routing sort
// Stable counting sort in three steps over chunks of SORT_CHUNK consecutive ids, one warp per chunk:
//   1. per-chunk histogram               hist[c][e]; also presets order[] to -1, so the tail that dropped ids leave
//                                         unwritten is recognisable (every reader clamps or skips it) instead of
//                                         holding whatever was in memory
//   2. one block: offsets[e] and the start of every (chunk, expert) run, in place in hist
//   3. per chunk, in input order: warp match on the expert id gives each entry its rank among equal
//      ids of the same 32-entry step; a per-expert cursor in shared memory carries across steps.
constexpr int SORT_CHUNK = 1024;

template <typename IdT>
__global__ void sort_hist_kernel(const IdT* __restrict__ ids, int64_t n, int E, int32_t* __restrict__ hist,
                                 int32_t* __restrict__ bad_count, int64_t* __restrict__ order) {
  extern __shared__ int32_t sh[];
  for (int e = threadIdx.x; e < E; e += 32) sh[e] = 0;
  __syncwarp();
  const int64_t c = blockIdx.x, i0 = c * SORT_CHUNK;
  int bad = 0;
  for (int s = 0; s < SORT_CHUNK; s += 32) {
    const int64_t i = i0 + s + threadIdx.x;
    if (i < n) {
      const int64_t e = (int64_t)ids[i];
      if (e >= 0 && e < E) atomicAdd(&sh[e], 1);
      else ++bad;
      order[i] = -1;
    }
  }
  __syncwarp();
  for (int e = threadIdx.x; e < E; e += 32) hist[c * E + e] = sh[e];
  if (bad && bad_count) atomicAdd(bad_count, bad);
}

__global__ void sort_scan_kernel(int32_t* __restrict__ hist, int64_t chunks, int E, int64_t* __restrict__ offsets) {
  // thread e: total of expert e; then an exclusive scan over experts; then run starts per chunk.
  extern __shared__ int64_t tot[];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int64_t s = 0;
    for (int64_t c = 0; c < chunks; ++c) s += hist[c * E + e];
    tot[e] = s;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int64_t run = 0;
    for (int e = 0; e < E; ++e) {
      const int64_t v = tot[e];
      tot[e] = run;
      offsets[e] = run;
      run += v;
    }
    offsets[E] = run;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int64_t run = tot[e];
    for (int64_t c = 0; c < chunks; ++c) {
      const int32_t v = hist[c * E + e];
      hist[c * E + e] = (int32_t)run;  // total rows < 2^31
      run += v;
    }
  }
}

template <typename IdT>
__global__ void sort_place_kernel(const IdT* __restrict__ ids, int64_t n, int E, const int32_t* __restrict__ hist,
                                  int64_t* __restrict__ order) {
  extern __shared__ int32_t cur[];
  const int lane = threadIdx.x;
  const int64_t c = blockIdx.x, i0 = c * SORT_CHUNK;
  for (int e = lane; e < E; e += 32) cur[e] = hist[c * E + e];
  __syncwarp();
  for (int s = 0; s < SORT_CHUNK; s += 32) {
    const int64_t i = i0 + s + lane;
    int64_t e = i < n ? (int64_t)ids[i] : -1;
    const bool ok = e >= 0 && e < E;
    const unsigned active = __ballot_sync(0xffffffffu, ok);
    if (ok) {
      const unsigned peers = __match_any_sync(active, (int)e);
      const int rank = __popc(peers & ((1u << lane) - 1u));
      const int leader = __ffs(peers) - 1;
      int base = 0;
      if (lane == leader) {
        base = cur[e];
        cur[e] = base + __popc(peers);
      }
      base = __shfl_sync(peers, base, leader);
      order[base + rank] = i;
    }
    __syncwarp();
  }
}

// ------------------------------------------------------------------------------------------ gather
// Every kernel that follows `order` clamps the entry to [0, n): an order array that was not produced by the routing
// sort (or one whose tail belongs to dropped ids) can then make a row wrong, but cannot make an access leave the buffers.
__device__ __forceinline__ int64_t clamp_slot(int64_t f, int64_t n) { return f < 0 ? 0 : (f >= n ? n - 1 : f); }

// dst[p, :] = src[order[p] / top_k, :], 16-byte vectors where the row length allows.
__global__ void gather_rows_kernel(const uint16_t* __restrict__ src, const int64_t* __restrict__ order, int64_t n_rows,
                                   int64_t K, int top_k, uint16_t* __restrict__ dst) {
  const int64_t p = blockIdx.x;
  if (p >= n_rows) return;
  const int64_t t = clamp_slot(order[p], n_rows) / top_k;
  const uint16_t* s = src + t * K;
  uint16_t* d = dst + p * K;
  if ((K & 7) == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
    const uint4* s4 = reinterpret_cast<const uint4*>(s);
    uint4* d4 = reinterpret_cast<uint4*>(d);
    for (int64_t i = threadIdx.x; i < K / 8; i += blockDim.x) d4[i] = s4[i];
  } else {
    for (int64_t i = threadIdx.x; i < K; i += blockDim.x) d[i] = s[i];
  }
}

// ------------------------------------------------------------------------------------------ swiglu
__device__ __forceinline__ float silu_fast(float g) {
  // g * sigmoid(g) with the hardware's exp2 and reciprocal approximations (2 ulp each; the result is rounded to bf16)
  return __fdividef(g, 1.f + __expf(-g));
}

// gu[p, 0:I] = gate (bf16), gu[p, I:2I] = up (bf16); h = bf16(w * silu(gate) * up), fp32 in between.
__global__ void swiglu_kernel(const __nv_bfloat16* __restrict__ gu, const float* __restrict__ route_weights,
                              const int64_t* __restrict__ order, int64_t n_rows, int64_t inter, float limit,
                              __nv_bfloat16* __restrict__ h) {
  const int64_t p = blockIdx.x;
  if (p >= n_rows) return;
  const float w = route_weights ? route_weights[order ? clamp_slot(order[p], n_rows) : p] : 1.f;
  const __nv_bfloat16* g = gu + p * 2 * inter;
  const __nv_bfloat16* u = g + inter;
  for (int64_t i = threadIdx.x; i < inter; i += blockDim.x) {
    float gate = __bfloat162float(g[i]), up = __bfloat162float(u[i]);
    if (limit > 0.f) {
      up = fminf(fmaxf(up, -limit), limit);
      gate = fminf(gate, limit);
    }
    const float sg = silu_fast(gate);
    float v = sg * up;
    if (route_weights) v = w * v;
    h[p * inter + i] = __float2bfloat16_rn(v);
  }
}

// ------------------------------------------------------------------------------ fp16-normalised rows
// The tcgen05 kernel takes fp16 token rows scaled by a power of two per row (row maximum in [128, 256), exact
// for every element within 2^-22 of the maximum) plus that factor. Producing them directly here saves the
// separate conversion pass over the activations.
__device__ __forceinline__ float block_max(float v, float* red) {
  for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float w = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    for (int off = 16; off > 0; off >>= 1) w = fmaxf(w, __shfl_xor_sync(0xffffffffu, w, off));
    if (threadIdx.x == 0) red[0] = w;
  }
  __syncthreads();
  const float r = red[0];
  __syncthreads();
  return r;
}

__device__ __forceinline__ int norm_exponent(float amax) {
  int ex = 0;
  if (amax > 0.f && isfinite(amax)) {
    (void)frexpf(amax, &ex);
    ex -= 8;  // amax * 2^-ex in [128, 256)
  }
  return ex;
}

// Eight bf16 (one 128-bit load) <-> floats, eight floats -> eight fp16 / bf16 (one 128-bit store).
__device__ __forceinline__ void bf16x8_to_float(const uint4& q, float* f) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ uint4 float8_to_f16(const float* f, float mul) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 h = __floats2half2_rn(f[2 * i] * mul, f[2 * i + 1] * mul);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ uint4 float8_to_bf16(const float* f) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// Single-pass forms of the two kernels below for rows of K % 8 == 0, K <= 2048 J elements: a thread keeps its J
// 16-byte chunks in registers between the maximum and the store, so every byte is read once, 128 bits at a time.
template <int J>
__global__ void __launch_bounds__(256)
gather_rows_norm_vec_kernel(const __nv_bfloat16* __restrict__ src, const int64_t* __restrict__ order, int64_t K, int top_k,
                            __half* __restrict__ dst, float* __restrict__ factor) {
  __shared__ float red[32];
  const int64_t p = blockIdx.x;
  const int64_t t = order ? clamp_slot(order[p], (int64_t)gridDim.x) / top_k : p;
  const uint4* s = reinterpret_cast<const uint4*>(src + t * K);
  const int chunks = (int)(K >> 3);
  float v[J][8];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < J; ++j) {
    const int c = threadIdx.x + j * 256;
    if (c < chunks) {
      bf16x8_to_float(s[c], v[j]);
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[j][i]));
    }
  }
  const int ex = norm_exponent(block_max(amax, red));
  const float down = ldexpf(1.f, -ex);
  uint4* d = reinterpret_cast<uint4*>(dst + p * K);
#pragma unroll
  for (int j = 0; j < J; ++j) {
    const int c = threadIdx.x + j * 256;
    if (c < chunks) d[c] = float8_to_f16(v[j], down);
  }
  if (threadIdx.x == 0) factor[p] = ldexpf(1.f, ex);
}

// Warp-per-row forms (rows of at most 256 J elements, K % 8 == 0): a block-wide maximum costs three block barriers
// per row and leaves eight rows in flight per SM, which bounds these passes by latency (gather: 0.25 ms for 98 304
// rows of 4096 against 0.15 ms of HBM time). Here a warp owns a row, keeps its J 16-byte chunks per lane in registers
// between the maximum (shuffles) and the store, and the eight warps of a block advance independently.
__device__ __forceinline__ float warp_max(float v) {
  for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}

template <int J>
__global__ void __launch_bounds__(256)
gather_rows_norm_warp_kernel(const __nv_bfloat16* __restrict__ src, const int64_t* __restrict__ order, int64_t n_rows, int64_t K,
                             int top_k, __half* __restrict__ dst, float* __restrict__ factor) {
  const int lane = threadIdx.x & 31;
  const int chunks = (int)(K >> 3);
  for (int64_t p = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); p < n_rows; p += (int64_t)gridDim.x * 8) {
    const int64_t t = order ? clamp_slot(order[p], n_rows) / top_k : p;
    const uint4* s = reinterpret_cast<const uint4*>(src + t * K);
    uint4 raw[J];
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int c = lane + j * 32;
      raw[j] = c < chunks ? s[c] : make_uint4(0u, 0u, 0u, 0u);
    }
    // the largest magnitude from the bit patterns: |bf16| orders as its low 15 bits (a NaN ranks above everything and
    // ends as "not finite" below, like an infinity: such a row's outputs are NaN whatever its scale)
    uint32_t mx = 0u;
#pragma unroll
    for (int j = 0; j < J; ++j)
      mx = __vmaxu2(mx, __vmaxu2(__vmaxu2(raw[j].x & 0x7fff7fffu, raw[j].y & 0x7fff7fffu), __vmaxu2(raw[j].z & 0x7fff7fffu, raw[j].w & 0x7fff7fffu)));
    mx = max(mx & 0xffffu, mx >> 16);
    const float amax = __uint_as_float(mx << 16);
    const int ex = norm_exponent(warp_max(amax));
    const float down = ldexpf(1.f, -ex);
    uint4* d = reinterpret_cast<uint4*>(dst + p * K);
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int c = lane + j * 32;
      if (c < chunks) {
        float v[8];
        bf16x8_to_float(raw[j], v);
        d[c] = float8_to_f16(v, down);
      }
    }
    if (lane == 0) factor[p] = ldexpf(1.f, ex);
  }
}

// h = bf16(w * silu(gate) * up) (the reference's rounding point) normalised to fp16, a warp per row; the count of rows
// as in the block-per-row form below
template <int J>
__global__ void __launch_bounds__(256)
swiglu_norm_warp_kernel(const __nv_bfloat16* __restrict__ gu, const float* __restrict__ route_weights, const int64_t* __restrict__ order,
                        int64_t n_rows, const int64_t* __restrict__ n_rows_dev, int64_t inter, float limit, __half* __restrict__ h,
                        float* __restrict__ factor) {
  int64_t n = n_rows;
  if (n_rows_dev) {
    const int64_t m = *n_rows_dev;
    n = m < 0 ? 0 : (m < n ? m : n);
  }
  const int lane = threadIdx.x & 31;
  const int chunks = (int)(inter >> 3);
  for (int64_t p = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); p < n; p += (int64_t)gridDim.x * 8) {
    const float w = route_weights ? route_weights[order ? clamp_slot(order[p], n_rows) : p] : 1.f;
    const uint4* g = reinterpret_cast<const uint4*>(gu + p * 2 * inter);
    const uint4* u = reinterpret_cast<const uint4*>(gu + p * 2 * inter + inter);
    uint4 rg[J], ru[J];
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int c = lane + j * 32;
      rg[j] = c < chunks ? g[c] : make_uint4(0u, 0u, 0u, 0u);
      ru[j] = c < chunks ? u[c] : make_uint4(0u, 0u, 0u, 0u);
    }
    uint4 hv[J];  // the products, rounded to bf16 (held as such: exact)
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < J; ++j) {
      float gate[8], up[8], x[8];
      bf16x8_to_float(rg[j], gate);
      bf16x8_to_float(ru[j], up);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float ga = gate[i], uu = up[i];
        if (limit > 0.f) {
          uu = fminf(fmaxf(uu, -limit), limit);
          ga = fminf(ga, limit);
        }
        x[i] = silu_fast(ga) * uu;
        if (route_weights) x[i] = w * x[i];
      }
      hv[j] = float8_to_bf16(x);
      bf16x8_to_float(hv[j], x);
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(x[i]));
    }
    const int ex = norm_exponent(warp_max(amax));
    const float down = ldexpf(1.f, -ex);
    uint4* d = reinterpret_cast<uint4*>(h + p * inter);
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int c = lane + j * 32;
      if (c < chunks) {
        float x[8];
        bf16x8_to_float(hv[j], x);
        d[c] = float8_to_f16(x, down);
      }
    }
    if (lane == 0) factor[p] = ldexpf(1.f, ex);
  }
}

// Rows p = blockIdx.x, blockIdx.x + gridDim.x, ... below the row count; the count is n_rows, or the smaller of n_rows and
// *n_rows_dev when the caller only knows it on the device (expert-parallel steps: rows received from the other ranks).
template <int J>
__global__ void __launch_bounds__(256)
swiglu_norm_vec_kernel(const __nv_bfloat16* __restrict__ gu, const float* __restrict__ route_weights, const int64_t* __restrict__ order,
                       int64_t n_rows, const int64_t* __restrict__ n_rows_dev, int64_t inter, float limit, __half* __restrict__ h,
                       float* __restrict__ factor) {
  __shared__ float red[32];
  int64_t n = n_rows;
  if (n_rows_dev) {
    const int64_t m = *n_rows_dev;
    n = m < 0 ? 0 : (m < n ? m : n);
  }
  const int chunks = (int)(inter >> 3);
  for (int64_t p = blockIdx.x; p < n; p += gridDim.x) {
    const float w = route_weights ? route_weights[order ? clamp_slot(order[p], n_rows) : p] : 1.f;
    const uint4* g = reinterpret_cast<const uint4*>(gu + p * 2 * inter);
    const uint4* u = reinterpret_cast<const uint4*>(gu + p * 2 * inter + inter);
    float v[J][8];
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int c = threadIdx.x + j * 256;
      if (c < chunks) {
        float gate[8], up[8];
        bf16x8_to_float(g[c], gate);
        bf16x8_to_float(u[c], up);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float ga = gate[i], uu = up[i];
          if (limit > 0.f) {
            uu = fminf(fmaxf(uu, -limit), limit);
            ga = fminf(ga, limit);
          }
          float x = silu_fast(ga) * uu;
          if (route_weights) x = w * x;
          x = __bfloat162float(__float2bfloat16_rn(x));  // the reference's rounding point
          v[j][i] = x;
          amax = fmaxf(amax, fabsf(x));
        }
      }
    }
    const int ex = norm_exponent(block_max(amax, red));
    const float down = ldexpf(1.f, -ex);
    uint4* d = reinterpret_cast<uint4*>(h + p * inter);
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int c = threadIdx.x + j * 256;
      if (c < chunks) d[c] = float8_to_f16(v[j], down);
    }
    if (threadIdx.x == 0) factor[p] = ldexpf(1.f, ex);
  }
}

// dst[p, :] = fp16(src[order[p] / top_k, :] * 2^-e_p), factor[p] = 2^e_p; one block per row, K <= 8 * 1024 per thread loop
__global__ void gather_rows_norm_kernel(const __nv_bfloat16* __restrict__ src, const int64_t* __restrict__ order, int64_t K,
                                        int top_k, __half* __restrict__ dst, float* __restrict__ factor) {
  __shared__ float red[32];
  const int64_t p = blockIdx.x;
  const int64_t t = order ? clamp_slot(order[p], (int64_t)gridDim.x) / top_k : p;
  const __nv_bfloat16* s = src + t * K;
  float amax = 0.f;
  for (int64_t k = threadIdx.x; k < K; k += blockDim.x) amax = fmaxf(amax, fabsf(__bfloat162float(s[k])));
  const int ex = norm_exponent(block_max(amax, red));
  const float down = ldexpf(1.f, -ex);
  for (int64_t k = threadIdx.x; k < K; k += blockDim.x) dst[p * K + k] = __float2half_rn(__bfloat162float(s[k]) * down);
  if (threadIdx.x == 0) factor[p] = ldexpf(1.f, ex);
}

// h = bf16(w * silu(gate) * up) (the reference's rounding point), then the row normalised to fp16 as above
__global__ void swiglu_norm_kernel(const __nv_bfloat16* __restrict__ gu, const float* __restrict__ route_weights,
                                   const int64_t* __restrict__ order, int64_t inter, float limit, __half* __restrict__ h,
                                   float* __restrict__ factor) {
  __shared__ float red[32];
  const int64_t p = blockIdx.x;
  const float w = route_weights ? route_weights[order ? clamp_slot(order[p], (int64_t)gridDim.x) : p] : 1.f;
  const __nv_bfloat16* g = gu + p * 2 * inter;
  const __nv_bfloat16* u = g + inter;
  float amax = 0.f;
  for (int pass = 0; pass < 2; ++pass) {
    int ex = 0;
    float down = 1.f;
    if (pass == 1) {
      ex = norm_exponent(block_max(amax, red));
      down = ldexpf(1.f, -ex);
      if (threadIdx.x == 0) factor[p] = ldexpf(1.f, ex);
    }
    for (int64_t i = threadIdx.x; i < inter; i += blockDim.x) {
      float gate = __bfloat162float(g[i]), up = __bfloat162float(u[i]);
      if (limit > 0.f) {
        up = fminf(fmaxf(up, -limit), limit);
        gate = fminf(gate, limit);
      }
      float v = silu_fast(gate) * up;
      if (route_weights) v = w * v;
      v = __bfloat162float(__float2bfloat16_rn(v));
      if (pass == 0) amax = fmaxf(amax, fabsf(v));
      else h[p * inter + i] = __float2half_rn(v * down);
    }
  }
}

// ----------------------------------------------------------------------------------------- combine
// inv[] is preset to -1 by the entry points; a (token, slot) whose expert id was dropped by the routing sort keeps
// -1 and contributes nothing.
__global__ void invert_order_kernel(const int64_t* __restrict__ order, int64_t n, int64_t* __restrict__ inv) {
  const int64_t p = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (p < n) {
    const int64_t f = order[p];
    if (f >= 0 && f < n) inv[f] = p;
  }
}

// A token's positions in `down` in increasing expert id (the ids of one token are distinct) -> pos[0 .. top_k) in
// shared memory; positions that are negative (dropped ids) or beyond the n_pos rows of `down` are marked -1. One
// thread sorts (its arrays are indexed at run time, so they live in local memory: one thread's worth, not a block's).
__device__ __forceinline__ void token_slots(const int64_t* __restrict__ inv, const int32_t* __restrict__ ids, int64_t t, int top_k,
                                            int64_t n_pos, int64_t* pos_shared) {
  if (threadIdx.x == 0) {
    int64_t pos[8];
    int eid[8];
    for (int s = 0; s < top_k; ++s) {
      const int64_t q = inv[t * top_k + s];
      pos[s] = (q >= 0 && q < n_pos) ? q : -1;
      eid[s] = ids[t * top_k + s];
    }
    for (int i = 1; i < top_k; ++i) {  // insertion sort by expert id
      const int e = eid[i];
      const int64_t q = pos[i];
      int j = i - 1;
      while (j >= 0 && eid[j] > e) {
        eid[j + 1] = eid[j];
        pos[j + 1] = pos[j];
        --j;
      }
      eid[j + 1] = e;
      pos[j + 1] = q;
    }
    for (int s = 0; s < top_k; ++s) pos_shared[s] = pos[s];
  }
  __syncthreads();
}

// One block per token: its top_k rows of `down`, visited in increasing expert id, summed in fp32; then the optional
// row of `add` (the shared expert's bf16 output, boilerplate/engine/model.py:421) in fp32, then the cast.
__global__ void combine_kernel(const __nv_bfloat16* __restrict__ down, const int64_t* __restrict__ inv,
                               const int32_t* __restrict__ ids, int top_k, int64_t hidden, const __nv_bfloat16* __restrict__ add,
                               __nv_bfloat16* __restrict__ y) {
  const int64_t t = blockIdx.x;
  __shared__ int64_t pos[8];
  token_slots(inv, ids, t, top_k, (int64_t)gridDim.x * top_k, pos);
  for (int64_t c = threadIdx.x; c < hidden; c += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < top_k; ++s)
      if (pos[s] >= 0) acc += __bfloat162float(down[pos[s] * hidden + c]);
    if (add) acc += __bfloat162float(add[t * hidden + c]);
    y[t * hidden + c] = __float2bfloat16_rn(acc);
  }
}

// inv for expert outputs that were sent back to their tokens' slots (the scatter form of the expert-parallel step):
// slot f = order[p] holds its row at position f itself, unless the routing sort dropped it (dest[p] < 0). inv is
// preset to -1 by the caller.
__global__ void returned_slots_kernel(const int64_t* __restrict__ order, const int64_t* __restrict__ dest, int64_t n,
                                      int64_t* __restrict__ inv) {
  const int64_t p = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (p < n) {
    const int64_t f = order[p];
    if (f >= 0 && f < n && dest[p] >= 0) inv[f] = f;
  }
}

// combine_kernel for hidden % 8 == 0: 128-bit loads and stores.
__global__ void __launch_bounds__(256)
combine_vec_kernel(const __nv_bfloat16* __restrict__ down, const int64_t* __restrict__ inv, const int32_t* __restrict__ ids, int top_k,
                   int64_t hidden, const __nv_bfloat16* __restrict__ add, __nv_bfloat16* __restrict__ y) {
  const int64_t t = blockIdx.x;
  __shared__ int64_t pos[8];
  token_slots(inv, ids, t, top_k, (int64_t)gridDim.x * top_k, pos);
  const int chunks = (int)(hidden >> 3);
  for (int c = threadIdx.x; c < chunks; c += 256) {
    // all of the token's rows are requested before any is added: one memory latency per chunk, not one per row
    // (a slot without a row reads zeros: the sum starts at +0 and so is never -0, and adding +0 to it changes nothing)
    uint4 raw[8];
#pragma unroll
    for (int s = 0; s < 8; ++s)
      raw[s] = (s < top_k && pos[s] >= 0) ? reinterpret_cast<const uint4*>(down + pos[s] * hidden)[c] : make_uint4(0u, 0u, 0u, 0u);
    uint4 radd = make_uint4(0u, 0u, 0u, 0u);
    if (add) radd = reinterpret_cast<const uint4*>(add + t * hidden)[c];
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      if (s < top_k) {
        float f[8];
        bf16x8_to_float(raw[s], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += f[i];
      }
    }
    if (add) {
      float f[8];
      bf16x8_to_float(radd, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
    reinterpret_cast<uint4*>(y + t * hidden)[c] = float8_to_bf16(acc);
  }
}


// ---------------------------------------------------------------------- standard (OLMoE-style) flavour
// boilerplate/engine/standard.py:149-176 keeps every intermediate in the model dtype (bf16): the expert output is
// down( bf16( bf16(silu(gate)) * up ) ), multiplied by the bf16 routing weight (rounded to bf16) and added into a
// bf16 output row, one rounding per addition, experts in increasing id.
template <bool NORM>
__global__ void swiglu_std_kernel(const __nv_bfloat16* __restrict__ gu, int64_t inter, __nv_bfloat16* __restrict__ h_bf16,
                                  __half* __restrict__ h_f16, float* __restrict__ factor) {
  __shared__ float red[32];
  const int64_t p = blockIdx.x;
  const __nv_bfloat16* g = gu + p * 2 * inter;
  const __nv_bfloat16* u = g + inter;
  auto value = [&](int64_t i) {
    const float gate = __bfloat162float(g[i]);
    const float sg = __bfloat162float(__float2bfloat16_rn(silu_fast(gate)));  // silu in fp32, stored as bf16
    return __bfloat162float(__float2bfloat16_rn(sg * __bfloat162float(u[i])));           // bf16 * bf16 -> bf16
  };
  if (!NORM) {
    for (int64_t i = threadIdx.x; i < inter; i += blockDim.x) h_bf16[p * inter + i] = __float2bfloat16_rn(value(i));
    return;
  }
  float amax = 0.f;
  for (int64_t i = threadIdx.x; i < inter; i += blockDim.x) amax = fmaxf(amax, fabsf(value(i)));
  const int ex = norm_exponent(block_max(amax, red));
  const float down = ldexpf(1.f, -ex);
  for (int64_t i = threadIdx.x; i < inter; i += blockDim.x) h_f16[p * inter + i] = __float2half_rn(value(i) * down);
  if (threadIdx.x == 0) factor[p] = ldexpf(1.f, ex);
}

// One block per token: y = sum over its slots in increasing expert id of bf16(down * bf16(weight)), every partial
// sum rounded to bf16 (the reference accumulates with index_add_ into a bf16 tensor).
__global__ void combine_weighted_kernel(const __nv_bfloat16* __restrict__ down, const int64_t* __restrict__ inv,
                                        const int32_t* __restrict__ ids, const float* __restrict__ weights, int top_k, int64_t hidden,
                                        __nv_bfloat16* __restrict__ y) {
  const int64_t t = blockIdx.x;
  int64_t pos[8];
  int eid[8];
  float wv[8];
  const int64_t n_pos = (int64_t)gridDim.x * top_k;
  for (int s = 0; s < top_k; ++s) {
    const int64_t q = inv[t * top_k + s];
    pos[s] = (q >= 0 && q < n_pos) ? q : -1;  // -1: the slot's expert id was dropped by the routing sort
    eid[s] = ids[t * top_k + s];
    wv[s] = __bfloat162float(__float2bfloat16_rn(weights[t * top_k + s]));
  }
  for (int i = 1; i < top_k; ++i) {  // insertion sort by expert id (ids of one token are distinct)
    const int e = eid[i];
    const int64_t p = pos[i];
    const float w = wv[i];
    int j = i - 1;
    while (j >= 0 && eid[j] > e) {
      eid[j + 1] = eid[j];
      pos[j + 1] = pos[j];
      wv[j + 1] = wv[j];
      --j;
    }
    eid[j + 1] = e;
    pos[j + 1] = p;
    wv[j + 1] = w;
  }
  for (int64_t c = threadIdx.x; c < hidden; c += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < top_k; ++s) {
      if (pos[s] < 0) continue;
      const float r = __bfloat162float(__float2bfloat16_rn(__bfloat162float(down[pos[s] * hidden + c]) * wv[s]));
      acc = __bfloat162float(__float2bfloat16_rn(acc + r));
    }
    y[t * hidden + c] = __float2bfloat16_rn(acc);
  }
}

}  // namespace
}  // namespace dst

using namespace dst;

extern "C" int dst_route_topk(const float* logits, const float* bias, int64_t T, int64_t E, int top_k, int score_func, float gate_temp,
                              int renorm, float route_scale, float* weights, int32_t* ids, dst_stream_t stream) {
  if (T < 0 || E <= 0 || top_k <= 0 || score_func < DST_SCORE_SOFTMAX || score_func > DST_SCORE_SQRTSOFTPLUS || !(gate_temp != 0.f))
    return DST_ERR_BAD_ARG;
  if (E > 32 * ROUTE_MAX_PER_LANE || top_k > 8 || top_k > E) return DST_ERR_UNSUPPORTED;
  if (T == 0) return DST_OK;
  if (!logits || !weights || !ids) return DST_ERR_BAD_ARG;
  const int warps = 4;
  const unsigned grid = (unsigned)cdiv64(T, warps);
  auto st = static_cast<cudaStream_t>(stream);
  const float inv_temp = 1.f / gate_temp;
  if (E <= 128) route_kernel<4><<<grid, warps * 32, 0, st>>>(logits, bias, T, (int)E, top_k, score_func, inv_temp, renorm, route_scale, weights, ids);
  else if (E <= 256) route_kernel<8><<<grid, warps * 32, 0, st>>>(logits, bias, T, (int)E, top_k, score_func, inv_temp, renorm, route_scale, weights, ids);
  else if (E <= 384) route_kernel<12><<<grid, warps * 32, 0, st>>>(logits, bias, T, (int)E, top_k, score_func, inv_temp, renorm, route_scale, weights, ids);
  else if (E <= 512) route_kernel<16><<<grid, warps * 32, 0, st>>>(logits, bias, T, (int)E, top_k, score_func, inv_temp, renorm, route_scale, weights, ids);
  else route_kernel<ROUTE_MAX_PER_LANE><<<grid, warps * 32, 0, st>>>(logits, bias, T, (int)E, top_k, score_func, inv_temp, renorm, route_scale, weights, ids);
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}

extern "C" int dst_route_softmax_topk_ex(const float* logits, int64_t T, int64_t E, int top_k, int renorm, float route_scale,
                                         float* weights, int32_t* ids, dst_stream_t stream) {
  return dst_route_topk(logits, nullptr, T, E, top_k, DST_SCORE_SOFTMAX, 1.f, renorm, route_scale, weights, ids, stream);
}

extern "C" int dst_route_softmax_topk(const float* logits, int64_t T, int64_t E, int top_k, float route_scale,
                                      float* weights, int32_t* ids, dst_stream_t stream) {
  return dst_route_topk(logits, nullptr, T, E, top_k, DST_SCORE_SOFTMAX, 1.f, 1, route_scale, weights, ids, stream);
}

extern "C" size_t dst_sort_workspace_bytes(int64_t n, int64_t E) {
  if (n < 0 || E <= 0) return 0;
  const int64_t chunks = cdiv64(n > 0 ? n : 1, SORT_CHUNK);
  return (size_t)(chunks * E) * sizeof(int32_t);
}

extern "C" int dst_sort_by_expert(const void* ids, int ids_are_i32, int64_t n, int64_t E, int64_t* order,
                                  int64_t* offsets, int32_t* bad_count, void* workspace, dst_stream_t stream) {
  if (n < 0 || E <= 0 || !offsets) return DST_ERR_BAD_ARG;
  if (E > 4096 || n > 0x7fffffff) return DST_ERR_BAD_SHAPE;  // per-expert tables live in shared memory
  auto st = static_cast<cudaStream_t>(stream);
  if (bad_count) DST_CUDA_TRY(cudaMemsetAsync(bad_count, 0, sizeof(int32_t), st));
  if (n == 0) {
    DST_CUDA_TRY(cudaMemsetAsync(offsets, 0, (size_t)(E + 1) * sizeof(int64_t), st));
    return DST_OK;
  }
  if (!ids || !order || !workspace) return DST_ERR_BAD_ARG;
  const int64_t chunks = cdiv64(n, SORT_CHUNK);
  int32_t* hist = static_cast<int32_t*>(workspace);
  const size_t sh32 = (size_t)E * sizeof(int32_t);
  if (ids_are_i32)
    sort_hist_kernel<int32_t><<<(unsigned)chunks, 32, sh32, st>>>(static_cast<const int32_t*>(ids), n, (int)E, hist, bad_count, order);
  else
    sort_hist_kernel<int64_t><<<(unsigned)chunks, 32, sh32, st>>>(static_cast<const int64_t*>(ids), n, (int)E, hist, bad_count, order);
  DST_CUDA_TRY(cudaGetLastError());
  sort_scan_kernel<<<1, 512, (size_t)E * sizeof(int64_t), st>>>(hist, chunks, (int)E, offsets);
  DST_CUDA_TRY(cudaGetLastError());
  if (ids_are_i32)
    sort_place_kernel<int32_t><<<(unsigned)chunks, 32, sh32, st>>>(static_cast<const int32_t*>(ids), n, (int)E, hist, order);
  else
    sort_place_kernel<int64_t><<<(unsigned)chunks, 32, sh32, st>>>(static_cast<const int64_t*>(ids), n, (int)E, hist, order);
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}

extern "C" int dst_gather_rows(const void* src, const int64_t* order, int64_t n_rows, int64_t K, int top_k,
                               void* dst_, dst_stream_t stream) {
  if (n_rows < 0 || K <= 0 || top_k <= 0) return DST_ERR_BAD_ARG;
  if (n_rows == 0) return DST_OK;
  if (!src || !order || !dst_) return DST_ERR_BAD_ARG;
  if (n_rows > 0x7fffffff) return DST_ERR_BAD_SHAPE;
  gather_rows_kernel<<<(unsigned)n_rows, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t*>(src), order, n_rows, K, top_k, static_cast<uint16_t*>(dst_));
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}

extern "C" int dst_swiglu(const void* gu_bf16, const float* route_weights, const int64_t* order, int64_t n_rows,
                          int64_t inter, float limit, void* h_bf16, dst_stream_t stream) {
  if (n_rows < 0 || inter <= 0) return DST_ERR_BAD_ARG;
  if (n_rows == 0) return DST_OK;
  if (!gu_bf16 || !h_bf16) return DST_ERR_BAD_ARG;
  if (n_rows > 0x7fffffff) return DST_ERR_BAD_SHAPE;
  swiglu_kernel<<<(unsigned)n_rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gu_bf16), route_weights, order, n_rows, inter, limit,
      static_cast<__nv_bfloat16*>(h_bf16));
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}

extern "C" int dst_gather_rows_norm(const void* src_bf16, const int64_t* order, int64_t n_rows, int64_t K, int top_k,
                                    void* dst_f16, float* row_factor, dst_stream_t stream) {
  if (n_rows < 0 || K <= 0 || top_k <= 0) return DST_ERR_BAD_ARG;
  if (n_rows == 0) return DST_OK;
  if (!src_bf16 || !dst_f16 || !row_factor) return DST_ERR_BAD_ARG;
  if (n_rows > 0x7fffffff) return DST_ERR_BAD_SHAPE;
  const bool vec = K % 8 == 0 && K <= 8192 && (reinterpret_cast<uintptr_t>(src_bf16) & 15) == 0 && (reinterpret_cast<uintptr_t>(dst_f16) & 15) == 0;
  if (vec) {
    auto st = static_cast<cudaStream_t>(stream);
    auto a = static_cast<const __nv_bfloat16*>(src_bf16);
    auto d = static_cast<__half*>(dst_f16);
    const unsigned wgrid = (unsigned)std::min<int64_t>((n_rows + 7) / 8, 148 * 64);  // eight rows per block, the blocks walk the rows
    if (K <= 1024) gather_rows_norm_warp_kernel<4><<<wgrid, 256, 0, st>>>(a, order, n_rows, K, top_k, d, row_factor);
    else if (K <= 2048) gather_rows_norm_warp_kernel<8><<<wgrid, 256, 0, st>>>(a, order, n_rows, K, top_k, d, row_factor);
    else if (K <= 4096) gather_rows_norm_warp_kernel<16><<<wgrid, 256, 0, st>>>(a, order, n_rows, K, top_k, d, row_factor);
    else gather_rows_norm_vec_kernel<4><<<(unsigned)n_rows, 256, 0, st>>>(a, order, K, top_k, d, row_factor);
    DST_CUDA_TRY(cudaGetLastError());
    return DST_OK;
  }
  gather_rows_norm_kernel<<<(unsigned)n_rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(src_bf16), order, K, top_k, static_cast<__half*>(dst_f16), row_factor);
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}

namespace {
// grid of the row-looping SwiGLU kernel: a block per row up to a few waves, then the blocks walk the rows
unsigned swiglu_grid(int64_t n_rows, bool count_on_device) {
  const int64_t cap = count_on_device ? 148 * 8 : 148 * 64;
  return (unsigned)(n_rows < cap ? n_rows : cap);
}
int swiglu_norm_launch(const void* gu_bf16, const float* route_weights, const int64_t* order, int64_t n_rows, const int64_t* n_rows_dev,
                       int64_t inter, float limit, void* h_f16, float* row_factor, cudaStream_t st) {
  auto a = static_cast<const __nv_bfloat16*>(gu_bf16);
  auto d = static_cast<__half*>(h_f16);
  const unsigned grid = swiglu_grid(n_rows, n_rows_dev != nullptr);
  const unsigned wgrid = (grid + 7) / 8;  // eight rows per block
  if (inter <= 1024) swiglu_norm_warp_kernel<4><<<wgrid, 256, 0, st>>>(a, route_weights, order, n_rows, n_rows_dev, inter, limit, d, row_factor);
  else if (inter <= 2048) swiglu_norm_warp_kernel<8><<<wgrid, 256, 0, st>>>(a, route_weights, order, n_rows, n_rows_dev, inter, limit, d, row_factor);
  else if (inter <= 4096) swiglu_norm_vec_kernel<2><<<grid, 256, 0, st>>>(a, route_weights, order, n_rows, n_rows_dev, inter, limit, d, row_factor);
  else swiglu_norm_vec_kernel<4><<<grid, 256, 0, st>>>(a, route_weights, order, n_rows, n_rows_dev, inter, limit, d, row_factor);
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}
}  // namespace

extern "C" int dst_swiglu_norm(const void* gu_bf16, const float* route_weights, const int64_t* order, int64_t n_rows,
                               int64_t inter, float limit, void* h_f16, float* row_factor, dst_stream_t stream) {
  if (n_rows < 0 || inter <= 0) return DST_ERR_BAD_ARG;
  if (n_rows == 0) return DST_OK;
  if (!gu_bf16 || !h_f16 || !row_factor) return DST_ERR_BAD_ARG;
  if (n_rows > 0x7fffffff) return DST_ERR_BAD_SHAPE;
  const bool vec = inter % 8 == 0 && inter <= 8192 && (reinterpret_cast<uintptr_t>(gu_bf16) & 15) == 0 && (reinterpret_cast<uintptr_t>(h_f16) & 15) == 0;
  if (vec) return swiglu_norm_launch(gu_bf16, route_weights, order, n_rows, nullptr, inter, limit, h_f16, row_factor, static_cast<cudaStream_t>(stream));
  swiglu_norm_kernel<<<(unsigned)n_rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gu_bf16), route_weights, order, inter, limit, static_cast<__half*>(h_f16), row_factor);
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}

extern "C" int dst_swiglu_norm_dev(const void* gu_bf16, const float* route_weights, const int64_t* order, int64_t n_rows_max,
                                   const int64_t* n_rows_dev, int64_t inter, float limit, void* h_f16, float* row_factor,
                                   dst_stream_t stream) {
  if (n_rows_max < 0 || inter <= 0) return DST_ERR_BAD_ARG;
  if (n_rows_max == 0) return DST_OK;
  if (!gu_bf16 || !h_f16 || !row_factor || !n_rows_dev) return DST_ERR_BAD_ARG;
  if (n_rows_max > 0x7fffffff) return DST_ERR_BAD_SHAPE;
  if (inter % 8 != 0 || inter > 8192) return DST_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(gu_bf16) & 15) != 0 || (reinterpret_cast<uintptr_t>(h_f16) & 15) != 0) return DST_ERR_ALIGNMENT;
  return swiglu_norm_launch(gu_bf16, route_weights, order, n_rows_max, n_rows_dev, inter, limit, h_f16, row_factor,
                            static_cast<cudaStream_t>(stream));
}

extern "C" int dst_combine_add(const void* down_bf16, const int64_t* order, const int32_t* ids, int64_t T, int top_k,
                               int64_t hidden, int64_t* inv, const void* add_bf16, void* y_bf16, dst_stream_t stream) {
  if (T < 0 || top_k <= 0 || top_k > 8 || hidden <= 0) return DST_ERR_BAD_ARG;
  if (T == 0) return DST_OK;
  if (!down_bf16 || !order || !ids || !inv || !y_bf16) return DST_ERR_BAD_ARG;
  if (T > 0x7fffffff / top_k) return DST_ERR_BAD_SHAPE;
  auto st = static_cast<cudaStream_t>(stream);
  const int64_t n = T * top_k;
  DST_CUDA_TRY(cudaMemsetAsync(inv, 0xff, (size_t)n * sizeof(int64_t), st));  // -1: no row (see invert_order_kernel)
  invert_order_kernel<<<(unsigned)cdiv64(n, 256), 256, 0, st>>>(order, n, inv);
  DST_CUDA_TRY(cudaGetLastError());
  auto add = static_cast<const __nv_bfloat16*>(add_bf16);
  if (hidden % 8 == 0 && (reinterpret_cast<uintptr_t>(down_bf16) & 15) == 0 && (reinterpret_cast<uintptr_t>(y_bf16) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(add_bf16) & 15) == 0)
    combine_vec_kernel<<<(unsigned)T, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(down_bf16), inv, ids, top_k, hidden, add,
                                                   static_cast<__nv_bfloat16*>(y_bf16));
  else
    combine_kernel<<<(unsigned)T, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(down_bf16), inv, ids, top_k, hidden, add,
                                               static_cast<__nv_bfloat16*>(y_bf16));
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}

extern "C" int dst_ep_combine_returned(const void* rows_bf16, const int64_t* order, const int64_t* row_dest, const int32_t* ids, int64_t T,
                                       int top_k, int64_t hidden, int64_t* inv, const void* add_bf16, void* y_bf16, dst_stream_t stream) {
  if (T < 0 || top_k <= 0 || top_k > 8 || hidden <= 0) return DST_ERR_BAD_ARG;
  if (hidden % 8 != 0) return DST_ERR_UNSUPPORTED;
  if (T == 0) return DST_OK;
  if (!rows_bf16 || !order || !row_dest || !ids || !inv || !y_bf16) return DST_ERR_BAD_ARG;
  if (T > 0x7fffffff / top_k) return DST_ERR_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(rows_bf16) & 15) != 0 || (reinterpret_cast<uintptr_t>(y_bf16) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(add_bf16) & 15) != 0)
    return DST_ERR_ALIGNMENT;
  auto st = static_cast<cudaStream_t>(stream);
  const int64_t n = T * top_k;
  DST_CUDA_TRY(cudaMemsetAsync(inv, 0xff, (size_t)n * sizeof(int64_t), st));  // -1: no row
  returned_slots_kernel<<<(unsigned)cdiv64(n, 256), 256, 0, st>>>(order, row_dest, n, inv);
  DST_CUDA_TRY(cudaGetLastError());
  combine_vec_kernel<<<(unsigned)T, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(rows_bf16), inv, ids, top_k, hidden,
                                                 static_cast<const __nv_bfloat16*>(add_bf16), static_cast<__nv_bfloat16*>(y_bf16));
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}

extern "C" int dst_combine(const void* down_bf16, const int64_t* order, const int32_t* ids, int64_t T, int top_k,
                           int64_t hidden, int64_t* inv, void* y_bf16, dst_stream_t stream) {
  return dst_combine_add(down_bf16, order, ids, T, top_k, hidden, inv, nullptr, y_bf16, stream);
}

extern "C" int dst_swiglu_std(const void* gu_bf16, int64_t n_rows, int64_t inter, void* h_bf16, dst_stream_t stream) {
  if (n_rows < 0 || inter <= 0) return DST_ERR_BAD_ARG;
  if (n_rows == 0) return DST_OK;
  if (!gu_bf16 || !h_bf16) return DST_ERR_BAD_ARG;
  if (n_rows > 0x7fffffff) return DST_ERR_BAD_SHAPE;
  swiglu_std_kernel<false><<<(unsigned)n_rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gu_bf16), inter, static_cast<__nv_bfloat16*>(h_bf16), nullptr, nullptr);
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}

extern "C" int dst_swiglu_std_norm(const void* gu_bf16, int64_t n_rows, int64_t inter, void* h_f16, float* row_factor,
                                   dst_stream_t stream) {
  if (n_rows < 0 || inter <= 0) return DST_ERR_BAD_ARG;
  if (n_rows == 0) return DST_OK;
  if (!gu_bf16 || !h_f16 || !row_factor) return DST_ERR_BAD_ARG;
  if (n_rows > 0x7fffffff) return DST_ERR_BAD_SHAPE;
  swiglu_std_kernel<true><<<(unsigned)n_rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gu_bf16), inter, nullptr, static_cast<__half*>(h_f16), row_factor);
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}

extern "C" int dst_combine_weighted(const void* down_bf16, const int64_t* order, const int32_t* ids, const float* weights, int64_t T,
                                    int top_k, int64_t hidden, int64_t* inv, void* y_bf16, dst_stream_t stream) {
  if (T < 0 || top_k <= 0 || top_k > 8 || hidden <= 0) return DST_ERR_BAD_ARG;
  if (T == 0) return DST_OK;
  if (!down_bf16 || !order || !ids || !weights || !inv || !y_bf16) return DST_ERR_BAD_ARG;
  if (T > 0x7fffffff / top_k) return DST_ERR_BAD_SHAPE;
  auto st = static_cast<cudaStream_t>(stream);
  const int64_t n = T * top_k;
  DST_CUDA_TRY(cudaMemsetAsync(inv, 0xff, (size_t)n * sizeof(int64_t), st));  // -1: no row
  invert_order_kernel<<<(unsigned)cdiv64(n, 256), 256, 0, st>>>(order, n, inv);
  DST_CUDA_TRY(cudaGetLastError());
  combine_weighted_kernel<<<(unsigned)T, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(down_bf16), inv, ids, weights, top_k, hidden,
                                                      static_cast<__nv_bfloat16*>(y_bf16));
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}
