// Expert-parallel dispatch and combine over peer memory (NVLink / NVSwitch, plain P2P loads and stores).
//
// Each rank holds the routed experts [rank * El, (rank + 1) * El) and its own tokens. After routing and the
// stable sort by global expert, every rank knows from an all-gather of the per-expert counts where each of its
// sorted rows belongs in the destination rank's expert-sorted receive buffer:
//     row p of expert g  ->  rank g / El, row dst_start[g] + (p - offsets[g])
// (dst_start[g] = rows of the destination's earlier experts from all ranks + rows of expert g from lower ranks).
//
//   ep_push_kernel     gathers the token row of sorted row p, normalises it to the tcgen05 kernel's fp16 row
//                      format (power of two per row, DST_ACT_F16_NORM) and STORES it, with its row factor and its
//                      routing weight, straight into the destination GPU's buffers: gather + conversion +
//                      dispatch in one pass, no staging copy, no re-sort on the receiver.
//                      Beside every row it also records where the row came from (rank, slot): the destination table
//                      of the scattering second expert GEMM (gemm_prefill.cu), which sends every output row back
//                      from its epilogue; the combine is then local (moe_kernels.cu, returned_slots_kernel).
//   ep_combine_kernel  the other way back: per token, LOADS its top_k expert outputs from the GPUs that computed
//                      them, in increasing expert id, sums in fp32 and writes bf16.
//   ep_barrier_kernel  the ranks' stream-ordered barrier over symmetric flag words; its wait is bounded.
//
// The buffers are mapped into every rank (torch symmetric memory). Only the barrier kernel waits on another GPU.
// Plain loads and stores: no TMA copies here.
#include <algorithm>

#include "dst_common.cuh"

namespace dst {
namespace {

struct PeerPtrs {
  void* p[DST_MAX_PEERS];
};
// Entry d of a by-value parameter table. Indexing the array with a run-time value would make the compiler copy the
// whole table into every thread's local memory (measured: 384 bytes of stack per thread made the push kernel 7x
// slower than its single-GPU counterpart); a chain of selects over compile-time indices reads the constant bank.
__device__ __forceinline__ void* peer_ptr(const PeerPtrs& t, int d) {
  void* r = t.p[0];
#pragma unroll
  for (int i = 1; i < DST_MAX_PEERS; ++i)
    if (d == i) r = t.p[i];
  return r;
}

__device__ __forceinline__ void bf16x8_to_float(const uint4& q, float* f) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

// index of the expert whose row range [offsets[g], offsets[g + 1]) holds row p (offsets nondecreasing, E + 1 entries)
__device__ __forceinline__ int expert_of_row(const int64_t* __restrict__ offsets, int E, int64_t p) {
  int lo = 0, hi = E;  // invariant: offsets[lo] <= p < offsets[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (offsets[mid] <= p) lo = mid;
    else hi = mid;
  }
  return lo;
}

// One thread per sorted row: the rank that owns its expert and its row in that rank's receive buffer, packed as
// (rank << 48) | row; -1 for rows past the last expert's range (ids the routing sort dropped). Doing the search here,
// once, in parallel, keeps a chain of dependent loads out of every block of the push kernel.
__global__ void ep_row_dest_kernel(const int64_t* __restrict__ offsets, const int64_t* __restrict__ dst_start, int64_t n_rows, int E, int El,
                                   int64_t* __restrict__ dest) {
  const int64_t p = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (p >= n_rows) return;
  if (p >= offsets[E]) {
    dest[p] = -1;
    return;
  }
  const int g = expert_of_row(offsets, E, p);
  dest[p] = ((int64_t)(g / El) << 48) | (dst_start[g] + (p - offsets[g]));
}

template <int J>  // 16-byte chunks per thread: rows of K <= 2048 J elements
__global__ void __launch_bounds__(256)
ep_push_kernel(const __nv_bfloat16* __restrict__ x, const int64_t* __restrict__ order, const int64_t* __restrict__ dest,
               const float* __restrict__ route_weights, const int64_t* __restrict__ own0, const int64_t* __restrict__ own1, int top_k,
               int64_t K, PeerPtrs rows, PeerPtrs fac, PeerPtrs wts, PeerPtrs back, int rank) {
  __shared__ float red[32];
  // The rows are sorted by destination rank. Blocks take the rows of the OTHER ranks in order starting with the rank
  // after this one (with every rank starting at rank 0's rows all of them would store into the same GPU at the same
  // time: measured at 8 ranks 300 GB/s per sender instead of the link's 770), and this rank's own rows [*own0, *own1)
  // spread evenly among them, so the local copies run under the transfers instead of after them.
  const int64_t n = (int64_t)gridDim.x, b = (int64_t)blockIdx.x;
  const int64_t o0 = own0 ? *own0 : 0, o1 = own1 ? *own1 : 0;
  const int64_t L = o1 > o0 ? o1 - o0 : 0;
  const int64_t before = b * L / n, upto = (b + 1) * L / n;  // own rows among the blocks before this one / up to it
  int64_t p;
  if (upto > before) {
    p = o0 + before;
  } else {
    p = o1 + (b - upto);
    if (p >= n) p -= n;
  }
  const int64_t dst = dest[p];
  if (dst < 0) return;  // a row of an id the routing sort dropped
  int64_t slot = order[p];
  slot = slot < 0 ? 0 : (slot >= (int64_t)gridDim.x ? (int64_t)gridDim.x - 1 : slot);  // never leaves the token rows
  const uint4* s = reinterpret_cast<const uint4*>(x + (slot / top_k) * K);
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
  // block maximum
  for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, red[i]);
  int ex = 0;
  if (amax > 0.f && isfinite(amax)) {
    (void)frexpf(amax, &ex);
    ex -= 8;  // amax * 2^-ex in [128, 256)
  }
  const float down = ldexpf(1.f, -ex);
  const int d = (int)(dst >> 48);
  const int64_t dr = dst & ((int64_t(1) << 48) - 1);
  uint4* out = reinterpret_cast<uint4*>(static_cast<__half*>(peer_ptr(rows, d)) + dr * K);
#pragma unroll
  for (int j = 0; j < J; ++j) {
    const int c = threadIdx.x + j * 256;
    if (c < chunks) {
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __half2 h = __floats2half2_rn(v[j][2 * i] * down, v[j][2 * i + 1] * down);
        w[i] = *reinterpret_cast<const uint32_t*>(&h);
      }
      out[c] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
  if (threadIdx.x == 0) {
    static_cast<float*>(peer_ptr(fac, d))[dr] = ldexpf(1.f, ex);
    static_cast<float*>(peer_ptr(wts, d))[dr] = route_weights[slot];
    // where the expert's output row for this routed row is to be sent back: (this rank, its slot token * top_k + choice)
    if (back.p[0] != nullptr) static_cast<int64_t*>(peer_ptr(back, d))[dr] = ((int64_t)rank << 48) | slot;
  }
}

__global__ void ep_invert_order_kernel(const int64_t* __restrict__ order, int64_t n, int64_t* __restrict__ inv) {
  const int64_t p = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (p < n) {
    const int64_t f = order[p];
    if (f >= 0 && f < n) inv[f] = p;
  }
}

// One block per token: its top_k rows, read from the ranks that own the experts, in increasing expert id, then the
// optional local row of `add` (the shared expert's output). A slot whose expert id is outside [0, E) or whose row
// was dropped by the routing sort (inv = -1) contributes nothing.
__global__ void __launch_bounds__(256)
ep_combine_kernel(PeerPtrs down, const int64_t* __restrict__ inv, const int32_t* __restrict__ ids, const int64_t* __restrict__ offsets,
                  const int64_t* __restrict__ dst_start, int E, int El, int top_k, int64_t hidden, const __nv_bfloat16* __restrict__ add,
                  __nv_bfloat16* __restrict__ y) {
  const int64_t t = blockIdx.x;
  __shared__ const __nv_bfloat16* src[8];
  if (threadIdx.x < 32) {
    // lane s looks up slot s (the slots' chains of dependent loads run side by side), then the slots are ranked by
    // expert id with shuffles (ids of one token are distinct; equal keys, which only slots without a row can have,
    // keep their order)
    const int s = threadIdx.x;
    int eid = 0x7fffffff;
    const __nv_bfloat16* sp = nullptr;
    if (s < top_k) {
      const int g = ids[t * top_k + s];
      const int64_t p = inv[t * top_k + s];
      eid = g;
      if (g >= 0 && g < E && p >= 0)
        sp = static_cast<const __nv_bfloat16*>(peer_ptr(down, g / El)) + (dst_start[g] + (p - offsets[g])) * hidden;
    }
    int rank = 0;
    for (int j = 0; j < top_k; ++j) {
      const int ej = __shfl_sync(0xffffffffu, eid, j);
      rank += (ej < eid || (ej == eid && j < s)) ? 1 : 0;
    }
    if (s < top_k) src[rank] = sp;
  }
  __syncthreads();
  const int chunks = (int)(hidden >> 3);
  for (int c = threadIdx.x; c < chunks; c += 256) {
    // all of the token's rows are requested before any is added: one trip over the links per chunk, not one per row
    // (a slot without a row reads zeros: the sum starts at +0 and so is never -0, and adding +0 to it changes nothing)
    uint4 raw[8];
#pragma unroll
    for (int s = 0; s < 8; ++s)
      raw[s] = (s < top_k && src[s] != nullptr) ? reinterpret_cast<const uint4*>(src[s])[c] : make_uint4(0u, 0u, 0u, 0u);
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
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    reinterpret_cast<uint4*>(y + t * hidden)[c] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// Placement of this rank's routed rows in their owners' buffers, from every rank's routing-sort offsets over the
// global experts (offsets_all [W][E + 1], the all-gathered `offsets` arrays). One block; thread g handles expert g:
//   dst_start[g]      = rows of the owner's earlier experts from all ranks + rows of expert g from lower ranks
//   offsets_local[i]  = row offsets of THIS rank's own experts in its receive buffer (the grouped GEMM's offsets)
__global__ void ep_placement_kernel(const int64_t* __restrict__ offsets_all, int W, int E, int El, int rank,
                                    int64_t* __restrict__ dst_start, int64_t* __restrict__ offsets_local) {
  extern __shared__ int64_t tot[];  // [E] rows of expert g from all ranks
  for (int g = threadIdx.x; g < E; g += blockDim.x) {
    int64_t t = 0;
    for (int r = 0; r < W; ++r) t += offsets_all[(int64_t)r * (E + 1) + g + 1] - offsets_all[(int64_t)r * (E + 1) + g];
    tot[g] = t;
  }
  __syncthreads();
  for (int g = threadIdx.x; g < E; g += blockDim.x) {
    const int first = (g / El) * El;
    int64_t base = 0;
    for (int j = first; j < g; ++j) base += tot[j];
    int64_t before = 0;
    for (int r = 0; r < rank; ++r) before += offsets_all[(int64_t)r * (E + 1) + g + 1] - offsets_all[(int64_t)r * (E + 1) + g];
    dst_start[g] = base + before;
    if (g / El == rank) {
      offsets_local[g - first] = base;
      if (g == first + El - 1) offsets_local[El] = base + tot[g];
    }
  }
}

// Barrier among the ranks of a node over peer memory: thread r stores `seq` into slot `rank` of rank r's flag array,
// then waits until slot r of this rank's own array has reached `seq`. Everything this rank's stream did before the
// launch (its pushes into the peers' buffers) has completed before the kernel starts, and the fence orders it before
// the flag. The wait is bounded (~2 s of clock cycles): on expiry the kernel records DST_ERR_TIMEOUT in the status word
// and returns, so a rank that never arrives cannot hang the others' GPUs.
__device__ int g_ep_status = 0;
__global__ void ep_barrier_kernel(PeerPtrs flags, int world, int rank, long long seq) {
  const int r = threadIdx.x;
  if (r >= world) return;
  __threadfence_system();
  volatile long long* theirs = static_cast<volatile long long*>(peer_ptr(flags, r));
  theirs[rank] = seq;
  volatile long long* mine = static_cast<volatile long long*>(peer_ptr(flags, rank));
  const long long t0 = clock64();
  while (mine[r] < seq) {
    if (clock64() - t0 > 4000000000LL) {
      atomicExch(&g_ep_status, DST_ERR_TIMEOUT);
      break;
    }
  }
  __threadfence_system();
}

bool fill_peers(PeerPtrs& out, const void* const* ptrs, int world) {
  for (int i = 0; i < DST_MAX_PEERS; ++i) out.p[i] = nullptr;
  for (int i = 0; i < world; ++i) {
    if (!ptrs[i] || (reinterpret_cast<uintptr_t>(ptrs[i]) & 15) != 0) return false;
    out.p[i] = const_cast<void*>(ptrs[i]);
  }
  return true;
}

}  // namespace
}  // namespace dst

using namespace dst;

extern "C" int dst_ep_barrier(const void* const* peer_flags, int world, int rank, int64_t seq, dst_stream_t stream) {
  if (world < 1 || world > DST_MAX_PEERS || rank < 0 || rank >= world || seq <= 0 || !peer_flags) return DST_ERR_BAD_ARG;
  PeerPtrs flags;
  if (!fill_peers(flags, peer_flags, world)) return DST_ERR_ALIGNMENT;
  ep_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flags, world, rank, (long long)seq);
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}

namespace dst {
int ep_take_status(int* status) {
  int st = 0;
  DST_CUDA_TRY(cudaMemcpyFromSymbol(&st, g_ep_status, sizeof(int)));
  if (st != 0) {
    const int zero = 0;
    DST_CUDA_TRY(cudaMemcpyToSymbol(g_ep_status, &zero, sizeof(int)));
  }
  *status = st;
  return DST_OK;
}
}  // namespace dst

extern "C" int dst_ep_placement(const int64_t* offsets_all, int world, int64_t E, int64_t experts_per_rank, int rank, int64_t* dst_start,
                                int64_t* offsets_local, dst_stream_t stream) {
  if (world < 1 || world > DST_MAX_PEERS || E <= 0 || experts_per_rank <= 0 || rank < 0 || rank >= world) return DST_ERR_BAD_ARG;
  if (E > 4096 || experts_per_rank * world != E) return DST_ERR_BAD_SHAPE;  // the per-expert totals live in shared memory
  if (!offsets_all || !dst_start || !offsets_local) return DST_ERR_BAD_ARG;
  ep_placement_kernel<<<1, 512, (size_t)E * sizeof(int64_t), static_cast<cudaStream_t>(stream)>>>(
      offsets_all, world, (int)E, (int)experts_per_rank, rank, dst_start, offsets_local);
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}

extern "C" int dst_ep_push_rows(const void* x_bf16, const int64_t* order, const int64_t* offsets, const float* route_weights,
                                const int64_t* dst_start, int64_t n_rows, int64_t E, int64_t experts_per_rank, int top_k, int64_t K,
                                const void* const* peer_rows_f16, const void* const* peer_row_factor, const void* const* peer_row_weight,
                                const void* const* peer_row_origin, int world, int rank, int64_t* row_dest, dst_stream_t stream) {
  if (n_rows < 0 || E <= 0 || experts_per_rank <= 0 || top_k <= 0 || K <= 0 || world < 1 || world > DST_MAX_PEERS || rank < 0 || rank >= world)
    return DST_ERR_BAD_ARG;
  if (E > DST_MAX_EXPERTS || experts_per_rank * world < E) return DST_ERR_BAD_SHAPE;
  if (K % 8 != 0 || K > 8192) return DST_ERR_UNSUPPORTED;
  if (n_rows == 0) return DST_OK;
  if (!x_bf16 || !order || !offsets || !route_weights || !dst_start || !peer_rows_f16 || !peer_row_factor || !peer_row_weight || !row_dest)
    return DST_ERR_BAD_ARG;
  if (n_rows > 0x7fffffff) return DST_ERR_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x_bf16) & 15) != 0) return DST_ERR_ALIGNMENT;
  PeerPtrs rows, fac, wts, back;
  if (!fill_peers(rows, peer_rows_f16, world) || !fill_peers(fac, peer_row_factor, world) || !fill_peers(wts, peer_row_weight, world))
    return DST_ERR_ALIGNMENT;
  for (int i = 0; i < DST_MAX_PEERS; ++i) back.p[i] = nullptr;
  if (peer_row_origin != nullptr && !fill_peers(back, peer_row_origin, world)) return DST_ERR_ALIGNMENT;
  auto st = static_cast<cudaStream_t>(stream);
  auto xp = static_cast<const __nv_bfloat16*>(x_bf16);
  ep_row_dest_kernel<<<(unsigned)cdiv64(n_rows, 256), 256, 0, st>>>(offsets, dst_start, n_rows, (int)E, (int)experts_per_rank, row_dest);
  DST_CUDA_TRY(cudaGetLastError());
  // this rank's own rows in the sorted order: [offsets[rank * El], offsets[min((rank + 1) * El, E)])
  const int64_t* own0 = offsets + std::min<int64_t>((int64_t)rank * experts_per_rank, E);
  const int64_t* own1 = offsets + std::min<int64_t>((int64_t)(rank + 1) * experts_per_rank, E);
  if (K <= 2048)
    ep_push_kernel<1><<<(unsigned)n_rows, 256, 0, st>>>(xp, order, row_dest, route_weights, own0, own1, top_k, K, rows, fac, wts, back, rank);
  else if (K <= 4096)
    ep_push_kernel<2><<<(unsigned)n_rows, 256, 0, st>>>(xp, order, row_dest, route_weights, own0, own1, top_k, K, rows, fac, wts, back, rank);
  else
    ep_push_kernel<4><<<(unsigned)n_rows, 256, 0, st>>>(xp, order, row_dest, route_weights, own0, own1, top_k, K, rows, fac, wts, back, rank);
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}

extern "C" int dst_ep_combine_pull_add(const void* const* peer_down_bf16, const int64_t* order, const int32_t* ids, const int64_t* offsets,
                                       const int64_t* dst_start, int64_t T, int64_t experts_per_rank, int top_k, int64_t hidden,
                                       int64_t* inv, const void* add_bf16, void* y_bf16, int world, dst_stream_t stream) {
  if (T < 0 || experts_per_rank <= 0 || top_k <= 0 || top_k > 8 || hidden <= 0 || world < 1 || world > DST_MAX_PEERS) return DST_ERR_BAD_ARG;
  if (hidden % 8 != 0) return DST_ERR_UNSUPPORTED;
  if (T == 0) return DST_OK;
  if (!peer_down_bf16 || !order || !ids || !offsets || !dst_start || !inv || !y_bf16) return DST_ERR_BAD_ARG;
  if (T > 0x7fffffff / top_k || experts_per_rank * world > DST_MAX_EXPERTS) return DST_ERR_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(y_bf16) & 15) != 0 || (reinterpret_cast<uintptr_t>(add_bf16) & 15) != 0) return DST_ERR_ALIGNMENT;
  PeerPtrs down;
  if (!fill_peers(down, peer_down_bf16, world)) return DST_ERR_ALIGNMENT;
  auto st = static_cast<cudaStream_t>(stream);
  const int64_t n = T * top_k;
  DST_CUDA_TRY(cudaMemsetAsync(inv, 0xff, (size_t)n * sizeof(int64_t), st));  // -1: the slot has no row
  ep_invert_order_kernel<<<(unsigned)cdiv64(n, 256), 256, 0, st>>>(order, n, inv);
  DST_CUDA_TRY(cudaGetLastError());
  ep_combine_kernel<<<(unsigned)T, 256, 0, st>>>(down, inv, ids, offsets, dst_start, (int)(experts_per_rank * world), (int)experts_per_rank,
                                                top_k, hidden, static_cast<const __nv_bfloat16*>(add_bf16),
                                                static_cast<__nv_bfloat16*>(y_bf16));
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}

extern "C" int dst_ep_combine_pull(const void* const* peer_down_bf16, const int64_t* order, const int32_t* ids, const int64_t* offsets,
                                   const int64_t* dst_start, int64_t T, int64_t experts_per_rank, int top_k, int64_t hidden, int64_t* inv,
                                   void* y_bf16, int world, dst_stream_t stream) {
  return dst_ep_combine_pull_add(peer_down_bf16, order, ids, offsets, dst_start, T, experts_per_rank, top_k, hidden, inv, nullptr, y_bf16,
                                 world, stream);
}
