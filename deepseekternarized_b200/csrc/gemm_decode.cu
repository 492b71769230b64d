// Decode GEMV / grouped GEMV for few token rows per expert: bound by HBM bandwidth on the packed weights.
//
//     out[m, n] = row_scale[m] * sum_i sum_g scale_i[e, n, g] * sum_{k in g} x[m, k] * trit_i[e, n, k]
//
// Every packed byte crosses HBM once: one thread per CTA streams the item's rows of the tiled layout's 8 KB slabs
// (layout_kernels.cu), two superblocks at a time, into a shared-memory ring with cp.async.bulk + mbarrier; the consumer
// warps read them from there with 128-bit loads. The multiply-adds are exact integer arithmetic on mma.sync.m16n8k32 (u8 x s8 -> s32)
// fed straight from registers:
//
//   A fragment  a weight row's packed word ANDed with a byte-wise 2-bit field mask IS the operand: four u8 digits
//               u = t + 1 in {0,1,2} (mask 0x03030303) or four digits times 4 (mask 0x0c0c0c0c); the other two
//               fields of every byte come from the word shifted right by 4. Unpacking costs one AND per four
//               weights and one shift per sixteen; the x1 and x4 operands accumulate apart and are merged once per
//               scale group.
//   B fragment  the token rows, staged once per expert in shared memory as 15-bit integers q = rint(x / s),
//               s = rowmax / 16256, split into two s8 columns q = 128 hi + lo (|x - s q| <= rowmax / 32512), laid
//               out in the order the lanes consume them so a lane's B registers of two MMAs are one 128-bit load.
//               int8 activations (the reference's CUDA contract) go in as they are (hi = 0): that path is exact.
//   offset      sum_k u_k q_k = sum_k t_k q_k + sum_k q_k: the per-(token, group) integer sums of q are computed
//               at staging time and subtracted per scale group.
//   columns     an MMA has eight B columns = four (hi, lo) pairs. With four or more token rows a pair is a token.
//               With one (two) token rows the four pairs are four (two) CONSECUTIVE SCALE GROUPS of the same
//               token: a lane feeds real activations only to the MMAs of its own group and reads zeros for the
//               others, so four groups accumulate side by side and the per-group epilogue (merge, subtract the
//               offset, convert, multiply by the group's fp16 scale: the structure of the reference kernels,
//               boilerplate/kernels/csrc/boilerplate_cpu.cpp:116-124) runs once per four groups, each lane of a
//               quad doing one of them; the quad's partial results are added with two shuffles at the end of K.
//
// Up to four token rows per expert: four consumer warps of 16 weight rows each and several CTAs per SM; a work item
// is (expert, 64-row half tile) over the whole of K. Five or more: the staged token rows take most of an SM's shared
// memory, so one CTA per SM of eight consumer warps that own two 16-row tiles each (a 256-row item; see the kernel).
// Items are dealt to CTAs in contiguous, equally sized ranges so an expert's token rows are staged once per CTA and run.
// Every mbarrier wait is bounded by elapsed clock cycles; on expiry the CTA raises its abort flag, all warps leave
// and the kernel records DST_ERR_TIMEOUT in the status word dst_check_device_status reads.
//
// Coverage: TQ2 tiled weights, group 128, K % 512 == 0 (a ring slot is two 256-trit superblocks), fp16 scales, bf16 / fp16 / int8 activations, any row
// count per expert (rows are processed up to 16 at a time; beyond that the weights are streamed again, from L2).
#include "dst_common.cuh"

namespace dst {
namespace {

// CW consumer warps of RW 16-row MMA tiles each (+ the producer warp) make a CTA; a work item is CW * RW * 16 rows of one
// expert over the whole of K. Few token rows: CW = 4, RW = 1 and several CTAs per SM. Five or more: the staged token rows
// take most of an SM's shared memory, so ONE CTA of 8 consumer warps with two tiles each shares them (cw below counts
// 16-row tiles: CW * RW).
constexpr int DC_QWARPS = 4;                      // warps per block of decode_quant_kernel
__host__ __device__ constexpr int dc_part(int cw) { return cw * 16 * 64; }           // bytes of one item's share of a superblock: 64 B per row
__host__ __device__ constexpr int dc_slot_data(int cw) { return 2 * dc_part(cw); }   // a ring slot holds the item's share of TWO superblocks (four scale groups)
__host__ __device__ constexpr int dc_slot(int cw) { return dc_slot_data(cw) + 16; }  // ... followed by its own "full" and "empty" mbarriers (one address register serves all)
#ifndef DC_RING_SLOTS
#define DC_RING_SLOTS 4
#endif
constexpr int DC_RING_MAX = DC_RING_SLOTS;        // slots of the slab ring (fewer, at least 2, when shared memory is short)
#ifndef DC_PRODUCER_SLEEP
#define DC_PRODUCER_SLEEP true
#endif
#ifndef DC_PREQ_ABOVE
#define DC_PREQ_ABOVE 0
#endif
constexpr int DC_ZERO = 512;                      // bytes of zeros the lanes without a column read
constexpr long long DC_WAIT_CYCLES = 4000000000LL;  // ~2 s

__device__ int g_decode_status = 0;

struct DecodeParams {
  const uint8_t* tiled[DST_MAX_TERMS];
  const __half* scale[DST_MAX_TERMS];
  int n_terms;
  const void* x;
  const float* row_scale;
  const int64_t* offsets;
  void* out;
  int out_dtype, accumulate;
  int E, T, N, K, G, NT, S;
  int ring;     // slots of the slab ring
  int GP;       // ints between the staged per-group sums of consecutive token rows: odd, so the four tokens a quad reads hit four banks
  int xstride;  // bytes between staged activation rows: K + 64 (= 64 mod 128: two rows read together hit all banks once)
  // activations quantised ahead of the GEMV by decode_quant_kernel (null: the GEMV's consumer warps do it per expert)
  const uint8_t* q_rows;  // [T][2][K] s8: the hi and the lo row of every token, bytes in the staged order
  const int* q_xsum4;     // [T][G]
  const float* q_xexp;    // [T]
};

// ------------------------------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// One try_wait: the thread may be suspended by the hardware for up to the hinted time (nanoseconds) while the phase
// is incomplete, so a waiting warp takes few issue slots from the warps that have work.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(done) : "r"(bar), "r"(parity), "r"(2000u) : "memory");
  return done != 0;
}
// Bounded wait: false when the abort flag is up or ~2 s of clock cycles have passed. BACKOFF sleeps between polls (the
// producer, which runs slabs ahead of the consumers and has no reason to poll fast).
template <bool BACKOFF = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_test(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t it = 1;; ++it) {
    if (BACKOFF) __nanosleep(256);
    if (mbar_test(bar, parity)) return true;
    if ((it & 63u) == 0u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > DC_WAIT_CYCLES) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// 128-bit shared-memory load from a shared-window address. Not volatile: the compiler may move it among the
// arithmetic around it; the mbarrier waits and arrives carry memory clobbers, which it does not cross.
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
// d = a * b + c, u8 x s8 -> s32; ZERO: c = 0
template <bool ZERO>
__device__ __forceinline__ void mma_u8s8(int* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  if (ZERO)
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
  else
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ------------------------------------------------------------------------------------------ work items
// Item -> (expert, block of RI = 64, 128 or 256 weight rows starting at row n0). Token rows [ra, rb) of the expert.
struct Item {
  int e, n0;
  int64_t ra, rb;
};
template <int RI>
__host__ __device__ __forceinline__ int items_per_expert(int NT) { return (NT * 128 + RI - 1) / RI; }
template <int RI>
__device__ __forceinline__ Item item_of(const DecodeParams& p, long long item) {
  Item it;
  const int ipe = items_per_expert<RI>(p.NT);
  it.e = (int)(item / ipe);
  it.n0 = (int)(item - (long long)it.e * ipe) * RI;
  row_range(p.offsets, it.e, p.T, it.ra, it.rb);
  return it;
}

// ------------------------------------------------------------------------------------------ staging
// Two adjacent activations (k, k + 1) as floats, one 32-bit (16-bit for int8) load.
__device__ __forceinline__ float2 load_pair(const __nv_bfloat16* p) {
  const uint32_t w = *reinterpret_cast<const uint32_t*>(p);
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
}
__device__ __forceinline__ float2 load_pair(const __half* p) { return __half22float2(*reinterpret_cast<const __half2*>(p)); }
__device__ __forceinline__ float2 load_pair(const int8_t* p) {
  const uint16_t w = *reinterpret_cast<const uint16_t*>(p);
  return make_float2((float)(int8_t)(w & 0xff), (float)(int8_t)(w >> 8));
}
// Largest magnitude of 8 adjacent 16-bit activations (one 128-bit load); non-finite values come back as +inf or NaN
__device__ __forceinline__ float amax8(const __nv_bfloat16* p) {
  const uint4 q = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float a = fabsf(__uint_as_float(w[i] << 16)), b = fabsf(__uint_as_float(w[i] & 0xFFFF0000u));
    m = (a > m || a != a) ? a : m;  // keeps a NaN once seen
    m = (b > m || b != b) ? b : m;
  }
  return m;
}
__device__ __forceinline__ float amax8(const __half* p) {
  const uint4 q = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    const float a = fabsf(f.x), b = fabsf(f.y);
    m = (a > m || a != a) ? a : m;
    m = (b > m || b != b) ? b : m;
  }
  return m;
}
__device__ __forceinline__ float amax8(const int8_t*) { return 0.f; }

// Token rows [m0, m0 + mc) of x -> shared memory, by the consumer warps:
//   xs[(2 tok + part)][..]  s8, part 0 = hi, 1 = lo of q = rint(x / s_tok); byte order inside a 256-trit superblock:
//                           position q4 * 64 + c * 16 + (m & 1) * 8 + h * 4 + b holds trit 16 (c + 4 (2 gi + h)) + tw,
//                           tw = {2 j, 8 + 2 j, 2 j + 1, 9 + 2 j}[b], MMA m = 4 gi + j of the superblock, q4 = m / 2
//                           (lane c's B registers b0 (h = 0) and b1 (h = 1) of MMAs 2 q4 and 2 q4 + 1 = 16 bytes)
//   xsum4[tok * xsum_stride + g]  4 * sum of q over scale group g (int32); zero for token slots beyond mc
//   xexp[tok]               s_tok * row_scale / 4 (NaN when the row holds a non-finite value)
template <int MT, int CW, typename XT, typename Sync>
__device__ bool stage_tokens(const DecodeParams& p, const XT* __restrict__ x, int64_t m0, int mc, uint8_t* xs, size_t xstride, int* xsum4,
                             int xsum_stride, float* xexp, float* xinv, Sync&& consumer_sync) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr bool IS_I8 = sizeof(XT) == 1;
  // pass 1: row maxima. Every consumer thread takes 128-bit pieces of every row; the warps' partial maxima meet in
  // xinv[m * CW + warp] (xinv has room for that: see the shared-memory plan in the kernel)
  if (!IS_I8) {
    for (int m = 0; m < mc; ++m) {
      const XT* row = x + (m0 + m) * p.K;
      float am = 0.f;
      for (int i = threadIdx.x * 8; i < p.K; i += CW * 32 * 8) {
        const float a = amax8(row + i);
        am = (a > am || a != a) ? a : am;
      }
      for (int off = 16; off > 0; off >>= 1) {
        const float o = __shfl_xor_sync(0xffffffffu, am, off);
        am = (o > am || o != o) ? o : am;
      }
      if (lane == 0) xinv[m * CW + warp] = am;
    }
    if (!consumer_sync()) return false;
  }
  float my_inv = 0.f;  // of token slot `lane` (lanes below MT)
  if (lane < MT) {
    float inv = 0.f, ex = 0.f;
    if (lane < mc) {
      const float rs = p.row_scale ? p.row_scale[m0 + lane] : 1.f;
      if (IS_I8) {
        inv = 1.f;
        ex = 0.25f * rs;
      } else {
        float amax = 0.f;
#pragma unroll
        for (int w = 0; w < CW; ++w) {
          const float o = xinv[lane * CW + w];
          amax = (o > amax || o != o) ? o : amax;
        }
        if (!(amax <= 3.0e38f)) {
          ex = __int_as_float(0x7fc00000);  // a non-finite activation: the token's outputs are NaN
        } else if (amax > 0.f) {
          inv = 16256.f / amax;
          ex = 0.25f * (amax / 16256.f) * rs;
        }
      }
    }
    my_inv = inv;
    if (warp == 0) xexp[lane] = ex;
  }
  // pass 2: one warp per (token slot, 128-trit group): lane = position / 4 inside the group's 128 bytes
  const int c = (lane >> 2) & 3, j = ((lane >> 4) & 1) * 2 + ((lane >> 1) & 1), h = lane & 1;
  for (int u = warp; u < MT * p.G; u += CW) {
    const int m = u / p.G, g = u - m * p.G;
    const float inv = __shfl_sync(0xffffffffu, my_inv, m);
    int sum = 0;
    if (m < mc) {
      const XT* row = x + (m0 + m) * p.K + (g * 128 + 16 * c + 64 * h + 2 * j);
      const float2 f0 = load_pair(row), f1 = load_pair(row + 8);  // trits (2j, 2j + 1) and (8 + 2j, 9 + 2j) of the word
      const float v[4] = {f0.x, f1.x, f0.y, f1.y};                   // byte order b = 0..3
      uint32_t whi = 0, wlo = 0;
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        int q;
        if (IS_I8) {
          q = (int)v[b];
        } else {
          q = (int)fminf(fmaxf(rintf(v[b] * inv), -16256.f), 16256.f);  // NaN -> 0; such a row's result is NaN through xexp
        }
        sum += q;
        const int hi = IS_I8 ? 0 : (q + 64) >> 7;
        const int lo = q - (hi << 7);
        whi |= (uint32_t)(hi & 0xff) << (8 * b);
        wlo |= (uint32_t)(lo & 0xff) << (8 * b);
      }
      // lane bits: (q4 & 1) c1 c0 (m & 1) h -> byte position (g & 1) * 128 + (q4 & 1) * 64 + c * 16 + (m & 1) * 8 + h * 4
      const int pos = (g >> 1) * 256 + (g & 1) * 128 + lane * 4;
      *reinterpret_cast<uint32_t*>(xs + (size_t)(2 * m) * xstride + pos) = whi;
      *reinterpret_cast<uint32_t*>(xs + (size_t)(2 * m + 1) * xstride + pos) = wlo;
    }
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    if (lane == 0) xsum4[m * xsum_stride + g] = 4 * sum;
  }
  return true;
}

// The staging above done ONCE per token, ahead of the GEMV, into global memory: with more than a few rows per expert
// the GEMV's CTAs would otherwise repeat it for every expert they touch (measured at 8 rows: a quarter to a half of
// their instructions). One block of DC_QWARPS warps per token row.
template <typename XT>
__global__ void __launch_bounds__(DC_QWARPS * 32)
decode_quant_kernel(const DecodeParams p, uint8_t* __restrict__ q_rows, int* __restrict__ q_xsum4, float* __restrict__ q_xexp) {
  __shared__ float xinv[DC_QWARPS];
  const int64_t t = blockIdx.x;
  auto sync = []() -> bool {
    __syncthreads();
    return true;
  };
  // token t as a "pass" of one row: row_scale, the row pointer and the outputs are all indexed by t through m0 = t
  stage_tokens<1, DC_QWARPS>(p, static_cast<const XT*>(p.x), t, 1, q_rows + (size_t)t * 2 * p.K, (size_t)p.K, q_xsum4 + t * p.G, p.G, q_xexp + t, xinv, sync);
}

// ------------------------------------------------------------------------------------------ the kernel
// GS = scale groups that share an MMA's columns (4: one token row per pass, 2: two, 1: four per column block);
// NB = column blocks (GS == 1 only): 4 NB token rows per pass; CW = consumer warps; RW = 16-row MMA tiles per warp.
//
// Many rows (RW == 2): every MMA needs 256 B of token columns from shared memory, which at the MMA rate of an SM is
// all of its shared-memory bandwidth; a warp that owns two 16-row tiles feeds both from one read. There the x1 / x4
// field trick is dropped as well: all four fields of a byte are shifted down to plain digits (three shifts per word
// more) and accumulate together, so the per-group epilogue has one merge less per output and the second set of
// accumulators is gone.
#ifndef DC_MINB
#define DC_MINB 4
#endif
#ifndef DC_MINB2
#define DC_MINB2 3
#endif
#ifndef DC_MINB4
#define DC_MINB4 2
#endif
__host__ __device__ constexpr int dc_min_blocks(int nb, int cw) { return cw > 4 ? 1 : (nb == 1 ? DC_MINB : (nb == 2 ? DC_MINB2 : DC_MINB4)); }

template <int GS, int NB, int CW, int RW, typename XT>
__global__ void __launch_bounds__((CW + 1) * 32, dc_min_blocks(NB, CW))
decode_kernel(const DecodeParams p) {
  constexpr int MT = 4 * NB / GS;  // token rows per pass
  constexpr int TPB = 4 / GS;      // token rows per column block
  constexpr int THREADS = (CW + 1) * 32;
  constexpr int RI = CW * RW * 16;  // weight rows of an item
  constexpr int PART = dc_part(CW * RW), SLOT_DATA = dc_slot_data(CW * RW), SLOT = dc_slot(CW * RW);
  constexpr bool ONEACC = RW > 1;
  static_assert(GS == 1 || NB == 1, "column blocks only with one scale group per MMA");
  static_assert(RW == 1 || NB % 2 == 0, "two-tile warps take the column blocks in pairs");
  static_assert(RI == 64 || RI == 128 || RI == 256, "an item is half a tile, a tile or two tiles");
  extern __shared__ __align__(128) uint8_t dsm[];
  uint8_t* ring = dsm;                                           // p.ring x SLOT: [two parts][full barrier][empty barrier]
  uint8_t* zero = ring + p.ring * SLOT;                          // DC_ZERO
  uint8_t* xs = zero + DC_ZERO;                                  // 2 MT staged rows
  int* xsum4 = reinterpret_cast<int*>(xs + (size_t)2 * MT * p.xstride);  // [MT][GP]
  float* xexp = reinterpret_cast<float*>(xsum4 + MT * p.GP);     // [MT]
  float* xinv = xexp + MT;                                       // [MT][CW] partial row maxima
  __shared__ uint64_t bar_stage, bar_rows;
  __shared__ int abort_s;
  volatile int* abort_flag = &abort_s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int s = 0; s < p.ring; ++s) {
      mbar_init(smem_u32(ring + s * SLOT + SLOT_DATA), 1);            // full: the producer's expect_tx arrive
      mbar_init(smem_u32(ring + s * SLOT + SLOT_DATA + 8), CW * 32);  // empty: one arrive per consumer thread
    }
    mbar_init(smem_u32(&bar_stage), CW);              // the consumer warps' own barrier (bounded, unlike bar.sync)
    mbar_init(smem_u32(&bar_rows), 1);                // pre-quantised token rows have landed (expect_tx arrive of the thread that copies)
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = threadIdx.x; i < DC_ZERO / 4; i += THREADS) reinterpret_cast<uint32_t*>(zero)[i] = 0u;
  __syncthreads();

  // contiguous, equally sized (+-1) range of items for this CTA
  const long long items = (long long)p.E * items_per_expert<RI>(p.NT);
  const long long i0 = items * blockIdx.x / gridDim.x, i1 = items * (blockIdx.x + 1) / gridDim.x;

  if (warp == CW) {
    // ------------------------------------------------------------------ producer: packed slabs -> ring
    if (lane == 0) {
      const uint32_t ring_a = smem_u32(ring), ring_end = ring_a + p.ring * SLOT;
      uint32_t sbase = ring_a, ph = 0;
      bool ok = true;
      for (long long item = i0; ok && item < i1; ++item) {
        const Item it = item_of<RI>(p, item);
        const int passes = (int)((it.rb - it.ra + MT - 1) / MT);
        // the item's rows inside the slab of their tile; 256 rows: two whole tiles (the second may not exist)
        const int tile = it.n0 >> 7;
        const int64_t off0 = (((int64_t)it.e * p.NT + tile) * p.S) * 8192 + (it.n0 & 127) * 64;
        const bool two = RI == 256 && tile + 1 < p.NT;
        const int64_t tile_step = (int64_t)p.S * 8192;
        for (int ps = 0; ok && ps < passes; ++ps)
          for (int term = 0; ok && term < p.n_terms; ++term)
            for (int sb = 0; sb < p.S; sb += 2) {
              if (!mbar_wait<DC_PRODUCER_SLEEP>(sbase + SLOT_DATA + 8, ph ^ 1u, abort_flag)) { ok = false; break; }
              const uint32_t full = sbase + SLOT_DATA;
              const uint8_t* src = p.tiled[term] + off0 + (int64_t)sb * 8192;
              if (RI == 256) {
                mbar_arrive_expect_tx(full, two ? SLOT_DATA : SLOT_DATA / 2);
                bulk_load(sbase, src, 8192, full);
                bulk_load(sbase + PART, src + 8192, 8192, full);
                if (two) {
                  bulk_load(sbase + 8192, src + tile_step, 8192, full);
                  bulk_load(sbase + PART + 8192, src + tile_step + 8192, 8192, full);
                }
              } else {
                mbar_arrive_expect_tx(full, SLOT_DATA);
                bulk_load(sbase, src, PART, full);
                bulk_load(sbase + PART, src + 8192, PART, full);
              }
              sbase += SLOT;
              if (sbase == ring_end) { sbase = ring_a; ph ^= 1u; }
            }
      }
    }
  } else {
    // ------------------------------------------------------------------ consumers
    const int g8 = lane >> 2, c = lane & 3;
    const int swz = (g8 >> 1) & 3;
    // this lane's unit of row g8 of the warp's first 16-row tile; row g8 + 8: + 512; the second tile: + 1024
    const uint32_t a_off = (uint32_t)((warp * 16 * RW + g8) * 64 + ((c ^ swz) << 4));
    const uint32_t ring_a = smem_u32(ring), zero_a = smem_u32(zero), xs_a = smem_u32(xs);
    // B column of this lane: pair g8 / 2, part g8 & 1; C columns of this lane: pair c
    const int col_pair = g8 >> 1, col_part = g8 & 1;
    const int tok_c = c / GS, slot_c = c % GS;  // (+ b * TPB) the token and the group slot of this lane's C columns
    const uint32_t ring_end = ring_a + p.ring * SLOT;
    uint32_t sbase = ring_a, ph = 0, stage_ph = 0, rows_ph = 0;  // the current ring slot and the parity of its "full" phase
    int staged_e = -1;
    int64_t staged_m0 = -1;
    auto consumer_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_stage));
      const bool r = mbar_wait(smem_u32(&bar_stage), stage_ph, abort_flag);
      stage_ph ^= 1u;
      __syncwarp();
      return r;
    };

    for (long long item = i0; item < i1; ++item) {
      const Item it = item_of<RI>(p, item);
      const int n_first = it.n0 + warp * 16 * RW + g8;  // this lane's output rows: n_first + 8 i, i < 2 RW
      for (int64_t m0 = it.ra; m0 < it.rb; m0 += MT) {
        const int mc = (int)(it.rb - m0 < MT ? it.rb - m0 : MT);
        if (staged_e != it.e || staged_m0 != m0) {
          // every consumer is done with the previous rows; then stage; then everyone sees the new ones
          if (!consumer_sync()) goto aborted;  // every consumer is done with the previous rows
          if (p.q_rows != nullptr) {
            // quantised ahead of this kernel: one thread has the rows copied in (bulk copies onto the staging barrier), the
            // others fetch the small per-(token, group) sums and the row factors
            if (warp == 0 && lane == 0) {
              const uint32_t bar = smem_u32(&bar_rows);
              mbar_arrive_expect_tx(bar, (uint32_t)mc * 2u * (uint32_t)p.K);
              for (int m = 0; m < 2 * mc; ++m)
                bulk_load(xs_a + (uint32_t)m * (uint32_t)p.xstride, p.q_rows + ((size_t)m0 * 2 + m) * p.K, (uint32_t)p.K, bar);
            }
            for (int m = warp; m < MT; m += CW)
              for (int g = lane; g < p.G; g += 32) xsum4[m * p.GP + g] = m < mc ? p.q_xsum4[(m0 + m) * p.G + g] : 0;
            if (threadIdx.x < MT) xexp[threadIdx.x] = threadIdx.x < mc ? p.q_xexp[m0 + threadIdx.x] : 0.f;
            if (!mbar_wait(smem_u32(&bar_rows), rows_ph, abort_flag)) goto aborted;
            rows_ph ^= 1u;
          } else if (!stage_tokens<MT, CW>(p, static_cast<const XT*>(p.x), m0, mc, xs, (size_t)p.xstride, xsum4, p.GP, xexp, xinv, consumer_sync)) {
            goto aborted;
          }
          if (!consumer_sync()) goto aborted;
          staged_e = it.e;
          staged_m0 = m0;
        }
        // B pointers. Shared columns (GS > 1): for phase s (= group % GS) the lane reads its column's staged row when
        // the column's pair belongs to that phase and its token exists, else the zeros. One group per MMA (GS == 1):
        // column pair j of block b is token 4 b + j; the columns of tokens that do not exist read whatever the staged
        // rows hold there (integers: an MMA column only reaches its own outputs, which are not stored).
        constexpr int NPTR = GS > 1 ? GS : 1;
        uint32_t bbase[NPTR], bstep[NPTR];
        uint32_t bblock = 0;  // GS == 1: bytes between the staged rows of consecutive column blocks
        if (GS > 1) {
#pragma unroll
          for (int s = 0; s < NPTR; ++s) {
            const int tok = col_pair / GS;
            const bool act = (col_pair % GS) == s && tok < mc;
            bbase[s] = act ? xs_a + (uint32_t)(2 * tok + col_part) * (uint32_t)p.xstride + (uint32_t)c * 16u : zero_a;
            bstep[s] = act ? 256u : 0u;
          }
        } else {
          bbase[0] = xs_a + (uint32_t)(2 * col_pair + col_part) * (uint32_t)p.xstride + (uint32_t)c * 16u;
          bstep[0] = 256u;
          bblock = 8u * (uint32_t)p.xstride;
        }
        float y[RW][NB][2];
#pragma unroll
        for (int t = 0; t < RW; ++t)
#pragma unroll
          for (int b = 0; b < NB; ++b) y[t][b][0] = y[t][b][1] = 0.f;

        for (int term = 0; term < p.n_terms; ++term) {
          // scale rows of this lane's outputs (rows beyond N read row 0 and are not stored)
          const __half* srow[2 * RW];
#pragma unroll
          for (int i = 0; i < 2 * RW; ++i) {
            const int n = n_first + 8 * i;
            srow[i] = p.scale[term] + ((int64_t)it.e * p.N + (n < p.N ? n : 0)) * p.G;
          }
          int accA[1][ONEACC ? 1 : NB][4], accB[ONEACC ? 1 : NB][4];  // the x1 and the x4 fields' sums (one tile per warp)
#pragma unroll
          for (int b = 0; b < (ONEACC ? 1 : NB); ++b)
#pragma unroll
            for (int i = 0; i < 4; ++i) accA[0][b][i] = accB[b][i] = 0;
          // scales of the lane's group of the next epilogue, requested ahead: a block of GS groups (shared columns), or
          // two groups at a time, two groups ahead, as one 32-bit load per output row (GS == 1; G is a multiple of 4)
          auto scale_at = [&](const __half* s, int grp) { return grp < p.G ? __half2float(s[grp]) : 0.f; };
          auto scale2_at = [&](const __half* s, int grp) { return grp < p.G ? *reinterpret_cast<const uint32_t*>(s + grp) : 0u; };
          float s_next[2 * RW];
          uint32_t s2_cur[2 * RW], s2_next[2 * RW];
#pragma unroll
          for (int i = 0; i < 2 * RW; ++i) {
            s_next[i] = GS > 1 ? scale_at(srow[i], slot_c) : 0.f;
            s2_cur[i] = 0u;
            s2_next[i] = GS == 1 ? scale2_at(srow[i], 0) : 0u;
          }
          // Epilogue of the block of GS groups whose first group is g_first: this lane's group is g_first + slot_c.
          // First the group's scales (odd: g_first & 1 as a compile-time value) ...
          float sc[2 * RW];
          auto take_scales = [&](int g_first, bool odd) {
            const int g_mine = g_first + slot_c;
#pragma unroll
            for (int i = 0; i < 2 * RW; ++i) {
              if (GS > 1) {
                sc[i] = s_next[i];
                s_next[i] = scale_at(srow[i], g_mine + GS);
              } else {
                if (!odd) {
                  s2_cur[i] = s2_next[i];
                  s2_next[i] = scale2_at(srow[i], g_first + 2);
                }
                const __half2 h2 = *reinterpret_cast<const __half2*>(&s2_cur[i]);
                sc[i] = odd ? __high2float(h2) : __low2float(h2);
              }
            }
          };
          // ... then per column block: 4 * sum_k u_k q_k - 4 * sum_k q_k as one integer, converted and multiplied.
          // x1 / x4 accumulators: 128 * (4 A_hi + B_hi) + (4 A_lo + B_lo)
          auto epilogue = [&](int g_first) {
            const int g_mine = g_first + slot_c;
#pragma unroll
            for (int b = 0; b < NB; ++b) {
              const int xs4 = g_mine < p.G ? xsum4[(b * TPB + tok_c) * p.GP + g_mine] : 0;
              const int v_lo = ((((accA[0][b][0] << 2) + accB[b][0]) << 7) + ((accA[0][b][1] << 2) + accB[b][1])) - xs4;
              const int v_hi = ((((accA[0][b][2] << 2) + accB[b][2]) << 7) + ((accA[0][b][3] << 2) + accB[b][3])) - xs4;
              y[0][b][0] = fmaf(sc[0], (float)v_lo, y[0][b][0]);
              y[0][b][1] = fmaf(sc[1], (float)v_hi, y[0][b][1]);
            }
          };
          // plain digits, one accumulator set, a pair of column blocks: 4 * (128 * A_hi + A_lo)
          auto epilogue_pair = [&](int g, int b0, const int (&acc)[RW][2][4]) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const int xs4 = xsum4[((b0 + j) * TPB + tok_c) * p.GP + g];
#pragma unroll
              for (int t = 0; t < RW; ++t) {
                const int v_lo = (acc[t][j][0] << 9) + ((acc[t][j][1] << 2) - xs4);
                const int v_hi = (acc[t][j][2] << 9) + ((acc[t][j][3] << 2) - xs4);
                y[t][b0 + j][0] = fmaf(sc[2 * t], (float)v_lo, y[t][b0 + j][0]);
                y[t][b0 + j][1] = fmaf(sc[2 * t + 1], (float)v_hi, y[t][b0 + j][1]);
              }
            }
          };

          // two superblocks (one ring slot, four scale groups) per iteration: the phase of every group (group % GS) is a
          // compile-time value, and the barrier traffic and slot arithmetic are paid once per 2 KB of a 16-row tile
          for (int sb0 = 0; sb0 < p.S; sb0 += 2) {
            if (!mbar_wait(sbase + SLOT_DATA, ph, abort_flag)) goto aborted;
            const uint32_t sa = sbase + a_off;
            // [superblock][tile]: rows g8 and g8 + 8. One tile per warp: both superblocks' words are read up front and the
            // slot is handed back at once; two tiles: the second superblock's words are read after the first one's MMAs
            // (registers), and the slot goes back then
            uint4 w_lo2[2][RW], w_hi2[2][RW];
            const uint32_t slot_bar = sbase + SLOT_DATA + 8;
#pragma unroll
            for (int u = 0; u < (RW == 1 ? 2 : 1); ++u)
#pragma unroll
              for (int t = 0; t < RW; ++t) {
                w_lo2[u][t] = lds128(sa + u * PART + t * 1024);
                w_hi2[u][t] = lds128(sa + u * PART + t * 1024 + 512);
              }
            if (RW == 1) mbar_arrive(slot_bar);  // every lane arrives for itself: its loads above are done
            sbase += SLOT;
            if (sbase == ring_end) { sbase = ring_a; ph ^= 1u; }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const int sb = sb0 + u;
              if (RW > 1 && u == 1) {
#pragma unroll
                for (int t = 0; t < RW; ++t) {
                  w_lo2[1][t] = lds128(sa + PART + t * 1024);
                  w_hi2[1][t] = lds128(sa + PART + t * 1024 + 512);
                }
                mbar_arrive(slot_bar);
              }
#pragma unroll
              for (int gi = 0; gi < 2; ++gi) {
                constexpr uint32_t M1 = 0x03030303u, M4 = 0x0c0c0c0cu;
                const int phase = (u * 2 + gi) % GS;   // group % GS
                const bool fresh = phase == 0;         // first group of an epilogue block: the accumulators restart
                const uint32_t bgrp = bbase[phase] + (uint32_t)sb * bstep[phase] + (uint32_t)gi * 128u;
                if (ONEACC) {
                  // operands of both tiles: [tile][field][a0..a3]
                  uint32_t op[RW][4][4];
#pragma unroll
                  for (int t = 0; t < RW; ++t) {
                    const uint4 w_lo = w_lo2[u][t], w_hi = w_hi2[u][t];
                    const uint32_t wd[4] = {gi ? w_lo.z : w_lo.x, gi ? w_hi.z : w_hi.x, gi ? w_lo.w : w_lo.y, gi ? w_hi.w : w_hi.y};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                      op[t][0][i] = wd[i] & M1;
                      op[t][1][i] = (wd[i] >> 2) & M1;
                      op[t][2][i] = (wd[i] >> 4) & M1;
                      op[t][3][i] = (wd[i] >> 6) & M1;
                    }
                  }
                  // two column blocks at a time, field by field: consecutive MMAs go to different accumulators (four
                  // independent chains), so none waits for the one before it; a pair's epilogue follows its MMAs, so
                  // it can run under the next pair's
                  take_scales(sb * 2 + gi, gi == 1);
#pragma unroll
                  for (int b0 = 0; b0 < NB; b0 += 2) {
                    if (b0 > 0 && b0 * TPB >= mc) continue;  // a short last pass: no token rows in this pair of blocks
                    uint32_t bq[2][4][2];  // [block][field][b0, b1]
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                      const uint32_t ba = bgrp + (uint32_t)(b0 + j) * bblock;
                      const uint4 q0 = lds128(ba), q1 = lds128(ba + 64);
                      bq[j][0][0] = q0.x; bq[j][0][1] = q0.y; bq[j][1][0] = q0.z; bq[j][1][1] = q0.w;
                      bq[j][2][0] = q1.x; bq[j][2][1] = q1.y; bq[j][3][0] = q1.z; bq[j][3][1] = q1.w;
                    }
                    int acc[RW][2][4];
#pragma unroll
                    for (int f = 0; f < 4; ++f)
#pragma unroll
                      for (int j = 0; j < 2; ++j)
#pragma unroll
                        for (int t = 0; t < RW; ++t) {
                          if (f == 0) mma_u8s8<true>(acc[t][j], op[t][f][0], op[t][f][1], op[t][f][2], op[t][f][3], bq[j][f][0], bq[j][f][1]);
                          else mma_u8s8<false>(acc[t][j], op[t][f][0], op[t][f][1], op[t][f][2], op[t][f][3], bq[j][f][0], bq[j][f][1]);
                        }
                    epilogue_pair(sb * 2 + gi, b0, acc);
                  }
                } else {
                  const uint4 w_lo = w_lo2[u][0], w_hi = w_hi2[u][0];
                  const uint32_t l0 = gi ? w_lo.z : w_lo.x, l1 = gi ? w_lo.w : w_lo.y, h0 = gi ? w_hi.z : w_hi.x, h1 = gi ? w_hi.w : w_hi.y;
                  const uint32_t l0s = l0 >> 4, l1s = l1 >> 4, h0s = h0 >> 4, h1s = h1 >> 4;
#pragma unroll
                  for (int b = 0; b < NB; ++b) {
                    const uint32_t ba = bgrp + (uint32_t)b * bblock;
                    const uint4 q0 = lds128(ba), q1 = lds128(ba + 64);
                    if (fresh) {
                      mma_u8s8<true>(accA[0][b], l0 & M1, h0 & M1, l1 & M1, h1 & M1, q0.x, q0.y);
                      mma_u8s8<true>(accB[b], l0 & M4, h0 & M4, l1 & M4, h1 & M4, q0.z, q0.w);
                    } else {
                      mma_u8s8<false>(accA[0][b], l0 & M1, h0 & M1, l1 & M1, h1 & M1, q0.x, q0.y);
                      mma_u8s8<false>(accB[b], l0 & M4, h0 & M4, l1 & M4, h1 & M4, q0.z, q0.w);
                    }
                    mma_u8s8<false>(accA[0][b], l0s & M1, h0s & M1, l1s & M1, h1s & M1, q1.x, q1.y);
                    mma_u8s8<false>(accB[b], l0s & M4, h0s & M4, l1s & M4, h1s & M4, q1.z, q1.w);
                  }
                }
                if (!ONEACC && phase == GS - 1) {
                  take_scales(sb * 2 + gi - (GS - 1), gi == 1);
                  epilogue(sb * 2 + gi - (GS - 1));
                }
              }
            }
          }
        }
        // the quad's lanes hold the partial sums of their group slots
#pragma unroll
        for (int t = 0; t < RW; ++t)
#pragma unroll
          for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              if (GS >= 2) y[t][b][i] += __shfl_xor_sync(0xffffffffu, y[t][b][i], 1);
              if (GS == 4) y[t][b][i] += __shfl_xor_sync(0xffffffffu, y[t][b][i], 2);
            }
        if (slot_c == 0) {
#pragma unroll
          for (int b = 0; b < NB; ++b) {
            const int tok = b * TPB + tok_c;
            if (tok < mc) {
              const float f = xexp[tok];
#pragma unroll
              for (int i = 0; i < 2 * RW; ++i) {
                const int n = n_first + 8 * i;
                if (n < p.N) {
                  const float v = y[i >> 1][b][i & 1] * f;
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
    }
  aborted:;  // a bounded wait gave up (the abort flag is up): leave without touching anything else
  }

  // ------------------------------------------------------------------ teardown
  if (*abort_flag) {
    // give bulk copies still in flight time to land before the CTA's shared memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < 4000000LL) __nanosleep(1000);
  }
  __syncthreads();
  if (threadIdx.x == 0 && abort_s) atomicExch(&g_decode_status, DST_ERR_TIMEOUT);
}

// Shared memory of a CTA apart from its ring
template <int GS, int NB, int CW>
size_t decode_fixed_smem(const DecodeParams& p) {
  constexpr int MT = 4 * NB / GS;
  return DC_ZERO + (size_t)2 * MT * p.xstride + (size_t)MT * p.GP * 4 + (size_t)MT * 4 * (1 + CW);
}

template <int GS, int NB, int CW, int RW, typename XT>
int launch_one(DecodeParams p, int sms, cudaStream_t stream) {
  constexpr int THREADS = (CW + 1) * 32, RI = CW * RW * 16, SLOT = dc_slot(CW * RW);
  const size_t budget = 226 * 1024, fixed = decode_fixed_smem<GS, NB, CW>(p);  // 227 KB per CTA less the static barriers
  if (fixed + (size_t)2 * SLOT > budget) return DST_ERR_UNSUPPORTED;
  // small CTAs: the full ring, and as many CTAs per SM as fit; the 256-row CTA: one per SM, the ring takes what is left
  const size_t room = (budget - fixed) / SLOT;
  p.ring = (int)(room < (size_t)DC_RING_MAX ? room : (size_t)DC_RING_MAX);
  const size_t smem = (size_t)p.ring * SLOT + fixed;
  auto kernel = decode_kernel<GS, NB, CW, RW, XT>;
  DST_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int per_sm = 0;
  DST_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, THREADS, smem));
  if (per_sm < 1) return DST_ERR_UNSUPPORTED;
  const long long items = (long long)p.E * items_per_expert<RI>(p.NT);
  const long long want = (long long)sms * per_sm;
  const int grid = (int)(items < want ? items : want);
  kernel<<<grid, THREADS, smem, stream>>>(p);
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}

#ifndef DC_WIDE_FROM
#define DC_WIDE_FROM 5
#endif
template <typename XT>
int launch_rows(const DecodeParams& p, int64_t rows_hint, int sms, cudaStream_t stream) {
  if (rows_hint <= 1) return launch_one<4, 1, 4, 1, XT>(p, sms, stream);
  if (rows_hint <= 2) return launch_one<2, 1, 4, 1, XT>(p, sms, stream);
  if (rows_hint < DC_WIDE_FROM && rows_hint <= 4) return launch_one<1, 1, 4, 1, XT>(p, sms, stream);
  // five or more rows: one CTA per SM whose eight consumer warps own 32 weight rows each and share the staged token
  // rows (8, then 16 per pass), when there is a 256-row item for every SM; else the small CTAs
  const long long wide_items = (long long)p.E * items_per_expert<256>(p.NT);
  if (wide_items >= sms) {
    int rc = rows_hint <= 8 ? DST_ERR_UNSUPPORTED : launch_one<1, 4, 8, 2, XT>(p, sms, stream);
    if (rc == DST_ERR_UNSUPPORTED) rc = launch_one<1, 2, 8, 2, XT>(p, sms, stream);
    if (rc != DST_ERR_UNSUPPORTED) return rc;
  }
  if (rows_hint <= 4) return launch_one<1, 1, 4, 1, XT>(p, sms, stream);
  const int rc = launch_one<1, 2, 4, 1, XT>(p, sms, stream);
  return rc == DST_ERR_UNSUPPORTED ? launch_one<1, 1, 4, 1, XT>(p, sms, stream) : rc;  // 16 staged rows of a long K may not fit
}

}  // namespace

// Scratch of the pre-quantised activations: [T][2][K] s8 rows, [T][G] int32 sums, [T] float factors (each part 256-byte aligned).
size_t decode_workspace_bytes(int64_t T, int64_t K) {
  const size_t G = (size_t)(K / 128);
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  return up((size_t)T * 2 * (size_t)K) + up((size_t)T * G * 4) + up((size_t)T * 4);
}

// Up to how many token rows per expert the decode GEMV beats the tcgen05 kernel (measured on 4096 x 4096 experts): 32
// where the many-row CTAs apply (TQ2 tiles, a 256-row item for every SM; two passes of 16 rows), else 16.
int64_t decode_row_limit(int fmt, int64_t E, int64_t N) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return fmt == DST_FMT_TQ2 && E * ((N + 255) / 256) >= sms ? 32 : 16;
}

bool decode_supports(const GemmArgs& a) {
  if (a.fmt == DST_FMT_TQ1) return decode_tq1_supports(a);
  return a.weight_layout == DST_LAYOUT_TILED && a.fmt == DST_FMT_TQ2 && a.group == 128 && a.K % 512 == 0 &&
         a.scale_dtype == DST_SCALE_F16 && (a.act_dtype == DST_ACT_BF16 || a.act_dtype == DST_ACT_F16 || a.act_dtype == DST_ACT_I8) &&
         (size_t)2 * dc_slot(4) + DC_ZERO + (size_t)8 * (a.K + 64) + (size_t)4 * (a.G + 8) * 4 <= 220 * 1024 &&
         a.T < (int64_t(1) << 31);
}

int launch_decode(const GemmArgs& a, cudaStream_t stream) {
  if (a.T == 0 || a.N == 0 || a.E == 0) return DST_OK;
  if (a.fmt == DST_FMT_TQ1) return launch_decode_tq1(a, stream);
  if (!decode_supports(a)) return DST_ERR_UNSUPPORTED;
  for (int i = 0; i < a.terms.n; ++i)
    if ((reinterpret_cast<uintptr_t>(a.terms.packed[i]) & 15) != 0 || (reinterpret_cast<uintptr_t>(a.terms.scale[i]) & 3) != 0)
      return DST_ERR_ALIGNMENT;  // slabs are bulk-copied (16 bytes); scales are read two groups (32 bits) at a time
  if ((reinterpret_cast<uintptr_t>(a.x) & 15) != 0) return DST_ERR_ALIGNMENT;  // rows are read with 128-bit loads
  DecodeParams p;
  for (int i = 0; i < DST_MAX_TERMS; ++i) {
    p.tiled[i] = i < a.terms.n ? a.terms.packed[i] : nullptr;
    p.scale[i] = i < a.terms.n ? static_cast<const __half*>(a.terms.scale[i]) : nullptr;
  }
  p.n_terms = a.terms.n;
  p.x = a.x;
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
  p.xstride = (int)(a.K + 64);
  p.ring = DC_RING_MAX;
  p.GP = p.G | 1;
  p.q_rows = nullptr;
  p.q_xsum4 = nullptr;
  p.q_xexp = nullptr;
  // rows per expert: known on the host, or guessed from the mean (an expert with more rows takes several passes)
  const int64_t rows_hint = a.max_rows >= 0 ? a.max_rows : cdiv64(a.T, a.E);
  int dev = 0, sms = 148;
  DST_CUDA_TRY(cudaGetDevice(&dev));
  DST_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  // More than two rows per expert and a workspace: quantise every token once, ahead of the GEMV
  if (rows_hint > DC_PREQ_ABOVE && a.workspace != nullptr && a.workspace_bytes >= decode_workspace_bytes(a.T, a.K) &&
      (reinterpret_cast<uintptr_t>(a.workspace) & 255) == 0) {
    auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
    uint8_t* base = static_cast<uint8_t*>(a.workspace);
    uint8_t* q_rows = base;
    int* q_xsum4 = reinterpret_cast<int*>(base + up((size_t)a.T * 2 * (size_t)a.K));
    float* q_xexp = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(q_xsum4) + up((size_t)a.T * (size_t)a.G * 4));
    if (a.act_dtype == DST_ACT_BF16) decode_quant_kernel<__nv_bfloat16><<<(unsigned)a.T, DC_QWARPS * 32, 0, stream>>>(p, q_rows, q_xsum4, q_xexp);
    else if (a.act_dtype == DST_ACT_F16) decode_quant_kernel<__half><<<(unsigned)a.T, DC_QWARPS * 32, 0, stream>>>(p, q_rows, q_xsum4, q_xexp);
    else decode_quant_kernel<int8_t><<<(unsigned)a.T, DC_QWARPS * 32, 0, stream>>>(p, q_rows, q_xsum4, q_xexp);
    DST_CUDA_TRY(cudaGetLastError());
    p.q_rows = q_rows;
    p.q_xsum4 = q_xsum4;
    p.q_xexp = q_xexp;
  }
  if (a.act_dtype == DST_ACT_BF16) return launch_rows<__nv_bfloat16>(p, rows_hint, sms, stream);
  if (a.act_dtype == DST_ACT_F16) return launch_rows<__half>(p, rows_hint, sms, stream);
  return launch_rows<int8_t>(p, rows_hint, sms, stream);
}

// Reads and clears the decode kernel's status word (DST_OK or DST_ERR_TIMEOUT in *status).
int decode_take_status(int* status) {
  int st = 0;
  DST_CUDA_TRY(cudaMemcpyFromSymbol(&st, g_decode_status, sizeof(int)));
  if (st != 0) {
    const int zero = 0;
    DST_CUDA_TRY(cudaMemcpyToSymbol(g_decode_status, &zero, sizeof(int)));
  }
  *status = st;
  return DST_OK;
}

}  // namespace dst
