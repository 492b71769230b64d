// Prefill grouped ternary GEMM for sm_100a: tcgen05 MMA with TMEM accumulators, TMA-fed activations,
// warp-specialised dequantisation of packed trits into fp16 shared-memory tiles.
//
// Problem (per expert e, rows ra..rb of the expert-sorted activations):
//     out[m, n] = row_scale[m] * sum_k x[m, k] * W_e[n, k],   W_e[n, k] = sum_i scale_i[e, n, k/128] * trit_i[e, n, k]
//
// Mapping ("swap AB"): the 128 weight rows of a tile are the MMA M dimension (TMEM lanes), up to 256
// token rows are the MMA N dimension (TMEM columns), so tiles stay full when an expert has few rows.
// Both operands are fp16, 64 K-elements per pipeline stage:
//   A (weights)      packed 8 KB slabs of the tiled layout (layout_kernels.cu) arrive by cp.async.bulk in a
//                    two-slot ring; 16 dequant warps turn them into scale * trit, exact in fp16, and write
//                    them with tcgen05.st straight into TENSOR MEMORY (lane = weight row, one 32-bit column
//                    = two consecutive K elements; 32 columns per stage, ring of 8 stages): the MMA takes A
//                    from TMEM, so the dequantised tile never passes through shared memory
//   B (activations)  fp16 rows fetched by one thread with cp.async.bulk.tensor (TMA) into K-major,
//                    128-byte-swizzled shared-memory stages
//   D (accumulator)  fp32 in TMEM columns 0..255; columns 256..511 are the A ring
// Shared-memory bandwidth is what bounds this kernel when A goes through shared memory (measured: the MMA
// issuer stalled ~1100 cycles per 512-cycle stage); with A in TMEM only B is written and read there.
// bf16 activations are converted once to fp16 with a power-of-two factor per row (exact for every
// element within 2^-22 of the row's absolute maximum); the factor comes back through row_scale.
// tcgen05 kind::f16 refuses an fp16 A with a bf16 B (illegal instruction), hence the conversion.
//
// CTA pairs (template parameter CG = 2, used when N is a multiple of 256): two CTAs of a cluster share
// one tile of 256 weight rows x up to 256 token rows. Each CTA dequantises its own 128 weight rows and
// loads HALF of the token rows; the pair's leader issues tcgen05.mma.cta_group::2 (M = 256), which reads
// the A tile of both CTAs and both halves of B. Per SM this halves the activation bytes fetched from L2
// and held in shared memory per FLOP, which is what bounds the single-CTA form (its 32 KB B stages are
// too few to cover the TMA latency). The stage-full barrier lives in the leader and collects the TMA
// bytes and the dequant arrivals of both CTAs; tcgen05.commit multicasts the stage-free and
// accumulator-full signals to both. Every TMA load writes into the shared memory of the CTA that issues it.
//
// Warp roles (704 threads, one CTA per SM, persistent over tiles):
//   warp 0      TMA producer for B and bulk copies of packed slabs
//   warp 1      MMA issuer, owns the TMEM allocation (in the non-leader CTA of a pair: relays "my A tile is ready")
//   warps 2-5   epilogue (TMEM -> registers -> global)
//   warps 6-21  dequant producers for A, in four groups of four warps: group g owns the stages with index = g
//               (mod 4), so four stages are dequantised at once (each warp's instruction stream is a long
//               dependent chain; one group per stage could not keep up with the MMAs); inside a group warp w
//               owns the 32 weight rows of TMEM lane quarter w % 4, one thread per row per 64-trit stage
//
// Every mbarrier wait is bounded by elapsed clock cycles; on expiry the CTA raises its abort flag, all
// roles leave their loops, the CTA frees TMEM and the kernel records DST_ERR_TIMEOUT in the status word.
#include <cuda.h>

#include <cstring>

#include "dst_common.cuh"

namespace dst {
namespace {

constexpr int PF_THREADS = 704;            // 6 control/epilogue warps + 16 dequant warps
constexpr int PF_DQ_WARPS = 16;
constexpr int PF_TN = 256;            // token rows per tile (TMEM columns per accumulator buffer)
constexpr int PF_A_COLS = 32;         // TMEM columns of one A stage: 64 fp16 per weight row
constexpr int PF_A_RING = 8;          // A stages in TMEM (columns 256..511)
constexpr int PF_B_BYTES = PF_TN * 128;
constexpr int PF_LUT_BYTES = 2 * 256 * 8 * 16;  // TQ1: two alignments x 256 byte values x 8 bank replicas x 16 B
constexpr int PF_SLAB = 8192;                   // one (row tile, superblock) slab of packed weights
constexpr bool kUseCtaPairs = false;
constexpr int PF_SMEM_MAX = 232448;             // 227 KB of dynamic shared memory per CTA
constexpr long long PF_WAIT_CYCLES = 4000000000LL;  // ~2 s

__device__ int g_device_status = 0;

// Optional per-role cycle accounting (build with -DDST_ROLE_TIMERS): where each warp role of the tcgen05
// kernel spends its time, summed over CTAs. Read with dst_role_timers(). Off in the shipped library.
#ifdef DST_ROLE_TIMERS
__device__ unsigned long long g_role_timers[64];
#define RT_DECL(...) long long __VA_ARGS__
#define RT_NOW() clock64()
#define RT_ADD(slot, v) atomicAdd(&g_role_timers[slot], (unsigned long long)(v))
#define RT_WAIT(acc, call) [&]() { const long long t0__ = clock64(); const bool r__ = (call); acc += clock64() - t0__; return r__; }()
#else
#define RT_DECL(...)
#define RT_NOW() 0
#define RT_ADD(slot, v)
#define RT_WAIT(acc, call) (call)
#endif

// One tensor map per TMA box height (16, 32, ... 256 token rows), so a stage is always one TMA instruction.
struct TmaMaps {
  CUtensorMap m[16];
};

struct PrefillParams {
  const uint8_t* tiled[DST_MAX_TERMS];
  const __half* scale[DST_MAX_TERMS];
  int n_terms;
  const float* row_scale;
  const int64_t* offsets;
  void* out;
  int out_dtype, accumulate;
  int E, T, N, K, G, NT, S, kstages;
  int nstage_log2;  // log2 of the stage ring depth (2, 4 or 8 stages), chosen by the host from the shared-memory budget
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
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
// Bounded wait: false when the abort flag is up or ~2 s of clock cycles have passed. BACKOFF sleeps between
// polls: for roles that wait long (epilogue, producer), so their polling does not take issue slots from the
// dequant warps.
template <bool BACKOFF = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_test(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t it = 1;; ++it) {
    if (BACKOFF) __nanosleep(40);
    if (mbar_test(bar, parity)) return true;
    if ((it & 63u) == 0u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > PF_WAIT_CYCLES) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
  // K-major, SWIZZLE_128B: start address >> 4, LBO unused (1), SBO = 1024 B (8 rows x 128 B), version 1.
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}

// A operand from tensor memory (lane = row, 32-bit column = 2 K elements), B from shared memory
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
               ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_f16_ts_2cta(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
               ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
// 8 consecutive 32-bit columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_st_8(uint32_t taddr, const uint32_t* v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) in the CTA of rank `rank`
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrives on the barrier at this shared-memory offset in BOTH CTAs of the pair once the MMAs issued so far are done
__device__ __forceinline__ void umma_commit_2cta(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((uint16_t)3) : "memory");
}
// TMA load into this CTA's shared memory whose completion bytes are counted on a barrier of the pair's leader
__device__ __forceinline__ void tma_load_2d_2cta(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t leader_bar) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(leader_bar) : "memory");
}

#define TMEM_LD_32(v, taddr)                                                                                              \
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                                  \
               "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,"   \
               "%28,%29,%30,%31}, [%32];"                                                                                 \
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),          \
                 "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),    \
                 "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),  \
                 "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])   \
               : "r"(taddr))
#define TMEM_LD_16(v, taddr)                                                                                             \
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"  \
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),         \
                 "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])    \
               : "r"(taddr))

// ------------------------------------------------------------------------------------------ tile walk
// Tiles are numbered expert-major, then token tile, then weight-row tile (fastest), so the CTAs that run
// at the same time share an expert's activation rows and packed weights in L2. Every role walks the
// same sequence with its own copy of this state.
struct TileWalker {
  const int64_t* offsets;
  int E, T, NT;      // NT: tiles along the weight rows (pairs of 128-row tiles when CTA pairs are used)
  int row_round;     // token rows per tile are a multiple of this (16, or 32 for CTA pairs)
  int e = -1, mt_count = 0, mt_rows = 0;
  long long before = 0;
  int64_t ra = 0, rb = 0;
  __device__ bool seek(long long t, int& e_out, int& nt, int& row0, int& rows) {
    while (e < 0 || t >= before + (long long)mt_count * NT) {
      if (e >= 0) before += (long long)mt_count * NT;
      if (++e >= E) return false;
      row_range(offsets, e, T, ra, rb);
      mt_count = (int)((rb - ra + PF_TN - 1) / PF_TN);
      // an expert with more rows than one tile holds is split evenly (whole multiples of row_round), so no
      // tile repeats the dequantisation of the weights for a handful of left-over rows
      mt_rows = mt_count > 0 ? (int)((((rb - ra + mt_count - 1) / mt_count) + row_round - 1) / row_round * row_round) : 0;
    }
    const long long local = t - before;
    const int mt = (int)(local / NT);
    nt = (int)(local - (long long)mt * NT);
    row0 = (int)ra + mt * mt_rows;
    rows = (int)(rb - row0 < mt_rows ? rb - row0 : mt_rows);
    if (rows < 0) rows = 0;
    e_out = e;
    return true;
  }
};

// ------------------------------------------------------------------------------------------ dequant
__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 bits_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// TQ2, tiled word format: trit 2j in bits [2j, 2j+1], trit 2j+1 in bits [16+2j, 17+2j] (digit u = t + 1).
// (w & (0x00030003 << 2j')) | 0x64006400 is the fp16 pair 1024 + u * 4^j'; one fused multiply-add maps it
// to u - 1 exactly; one multiply applies the group scale exactly.
template <bool FIRST>
__device__ __forceinline__ void tq2_word(uint32_t w, __half2 s2, __half2* acc /* 8 */) {
  const uint32_t magic = 0x64006400u;
  const uint32_t w2 = w >> 10;
  const __half2 m0 = __floats2half2_rn(1.f, 1.f), m1 = __floats2half2_rn(0.25f, 0.25f), m2 = __floats2half2_rn(0.0625f, 0.0625f),
                m3 = __floats2half2_rn(0.015625f, 0.015625f), m4 = __floats2half2_rn(0.00390625f, 0.00390625f);
  const __half2 a0 = __floats2half2_rn(-1025.f, -1025.f), a1 = __floats2half2_rn(-257.f, -257.f), a2 = __floats2half2_rn(-65.f, -65.f),
                a3 = __floats2half2_rn(-17.f, -17.f), a4 = __floats2half2_rn(-5.f, -5.f);
  __half2 t[8];
  t[0] = __hfma2(bits_h2((w & 0x00030003u) | magic), m0, a0);
  t[1] = __hfma2(bits_h2((w & 0x000C000Cu) | magic), m1, a1);
  t[2] = __hfma2(bits_h2((w & 0x00300030u) | magic), m2, a2);
  t[3] = __hfma2(bits_h2((w & 0x00C000C0u) | magic), m3, a3);
  t[4] = __hfma2(bits_h2((w & 0x03000300u) | magic), m4, a4);
  t[5] = __hfma2(bits_h2((w2 & 0x00030003u) | magic), m0, a0);
  t[6] = __hfma2(bits_h2((w2 & 0x000C000Cu) | magic), m1, a1);
  t[7] = __hfma2(bits_h2((w2 & 0x00300030u) | magic), m2, a2);
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = FIRST ? __hmul2(t[j], s2) : __hfma2(t[j], s2, acc[j]);
}

// TQ1: the thread needs the 16 trits [tau, tau + 16) of its row-superblock, tau = 16 q. They start at
// trit `o` of byte b0 = tau / 5 and always lie inside 4 consecutive bytes. Bytes go through a shared-memory
// table of unscaled fp16 trits in two alignments (first trit in the low or the high half of a pair), so
// pairs never need re-alignment: entry even = (v0,v1)(v2,v3)(v4,0), entry odd = (0,v0)(v1,v2)(v3,v4).
// Byte i lands at pair index floor((5 i - o) / 2); neighbouring bytes share one pair, merged with OR.
template <int O, bool FIRST>
__device__ __forceinline__ void tq1_decode(uint32_t win, uint32_t lut_addr, __half2 s2, __half2* acc /* 8 */) {
  uint32_t out[8];
#pragma unroll
  for (int h = 0; h < 8; ++h) out[h] = 0u;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t idx = (i == 0 ? (win << 7) : (win >> (8 * i - 7))) & 0x7F80u;
    const int p = 5 * i - O;                       // position of the byte's first trit
    const int odd = ((p % 2) + 2) % 2;             // first trit lands in the high half
    const int h0 = (p - odd) / 2;                  // floor(p / 2), exact for negative p too
    uint32_t t0, t1, t2, t3;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(t0), "=r"(t1), "=r"(t2), "=r"(t3) : "r"(lut_addr + idx + odd * 32768u));
    (void)t3;
    if (h0 >= 0 && h0 < 8) out[h0] |= t0;
    if (h0 + 1 >= 0 && h0 + 1 < 8) out[h0 + 1] |= t1;
    if (h0 + 2 >= 0 && h0 + 2 < 8) out[h0 + 2] |= t2;
  }
#pragma unroll
  for (int h = 0; h < 8; ++h) acc[h] = FIRST ? __hmul2(bits_h2(out[h]), s2) : __hfma2(bits_h2(out[h]), s2, acc[h]);
}

template <bool FIRST>
__device__ __forceinline__ void tq1_dispatch(int o, uint32_t win, uint32_t lut_addr, __half2 s2, __half2* acc) {
  switch (o) {
    case 0: tq1_decode<0, FIRST>(win, lut_addr, s2, acc); break;
    case 1: tq1_decode<1, FIRST>(win, lut_addr, s2, acc); break;
    case 2: tq1_decode<2, FIRST>(win, lut_addr, s2, acc); break;
    case 3: tq1_decode<3, FIRST>(win, lut_addr, s2, acc); break;
    default: tq1_decode<4, FIRST>(win, lut_addr, s2, acc); break;
  }
}

// ------------------------------------------------------------------------------------------ the kernel
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// Scale of group g (0..7 inside the 8 scales held in `sc`), as an fp16 pair.
__device__ __forceinline__ __half2 pick_scale(const uint4& sc, int g) {
  const uint32_t w = (g & 4) ? ((g & 2) ? sc.w : sc.z) : ((g & 2) ? sc.y : sc.x);
  const uint32_t h = (g & 1) ? (w >> 16) : (w & 0xFFFFu);
  return bits_h2(h | (h << 16));
}

// Shared memory map (dynamic, 1024-byte aligned), per CTA:
//   [0, nstage * stage_bytes)      B stage ring: 256 token rows x 64 fp16 = 32 KB for one CTA, 128 rows = 16 KB for
//                                  each CTA of a pair; nstage <= 8 and stage s pairs with A ring slot s in TMEM
//   then 2 * n_terms * 8 KB        packed-weight slabs: slot-major, one 8 KB slab per stacked term
//   then 64 KB (TQ1 only)          table of unscaled fp16 trits
template <int FMT, int CG, int TERMS>
__global__ void __launch_bounds__(PF_THREADS, 1)
prefill_kernel(const __grid_constant__ TmaMaps xmaps, const PrefillParams p) {
  constexpr int SPB = FMT == 2 ? 4 : 5;  // 64-trit stages per 64-byte superblock
  constexpr int MAX_STAGE = PF_A_RING;
  constexpr int B_BYTES = PF_B_BYTES / CG;
  constexpr int STAGE_BYTES = B_BYTES;
  constexpr int ROUND = CG == 2 ? 32 : 16;  // token rows per tile are padded to this for the MMA N
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int NSTAGE = 1 << p.nstage_log2;
  const uint32_t smask = (uint32_t)NSTAGE - 1u, sshift = (uint32_t)p.nstage_log2;
  uint8_t* slabs = smem + NSTAGE * STAGE_BYTES;
  uint8_t* lut = slabs + 2 * p.n_terms * PF_SLAB;  // TQ1 only
  __shared__ uint64_t bar_full[MAX_STAGE], bar_afull[MAX_STAGE], bar_empty[MAX_STAGE], bar_tfull[1], bar_tempty[1], bar_pfull[2], bar_pempty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  volatile int* abort_flag = &abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = CG == 2 ? cluster_ctarank() : 0u;  // 0 = the pair's leader
  const bool leader = rank == 0;
  if (tid == 0) {
    abort_s = 0;
    for (int s = 0; s < MAX_STAGE; ++s) {
      // stage full (leader): the TMA producer's expect_tx arrive + one arrive per warp of the dequant group that owns the stage
      // + one relayed arrive for the peer's A tile
      mbar_init(smem_u32(&bar_full[s]), 1 + 4 + (CG - 1));
      mbar_init(smem_u32(&bar_afull[s]), 4);  // non-leader CTA of a pair: its own A tile is written (4 warps per stage)
      mbar_init(smem_u32(&bar_empty[s]), 1);  // tcgen05.commit (multicast to both CTAs of a pair)
    }
    mbar_init(smem_u32(&bar_tfull[0]), 1);        // tcgen05.commit after the tile's last MMA
    mbar_init(smem_u32(&bar_tempty[0]), 4 * CG);  // leader: one arrive per epilogue warp of every CTA of the pair
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bar_pfull[a]), 1);        // bulk-copy producer's expect_tx arrive
      mbar_init(smem_u32(&bar_pempty[a]), PF_DQ_WARPS);  // one arrive per dequant warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (FMT == 1) {
    // table of unscaled fp16 trits: [alignment][byte value][replica] x 16 B
    for (int i = tid; i < 2 * 256 * 8; i += PF_THREADS) {
      const int odd = i >> 11, v = (i >> 3) & 255;
      const uint32_t f = tq1_fields((uint32_t)v);
      uint32_t h[6];
#pragma unroll
      for (int d = 0; d < 5; ++d) {
        const int t = (int)((f >> (2 * d)) & 3u) - 1;
        h[d + 1] = t > 0 ? 0x3C00u : (t < 0 ? 0xBC00u : 0u);
      }
      h[0] = 0u;
      uint4 ent;
      if (odd) ent = make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16), 0u);
      else ent = make_uint4(h[1] | (h[2] << 16), h[3] | (h[4] << 16), h[5], 0u);
      *reinterpret_cast<uint4*>(lut + (size_t)i * 16) = ent;
    }
  }
  __syncwarp();
  if (warp == 1) {
    if (CG == 2) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(512));
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(512));
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (CG == 2) cluster_sync_all();  // the peer's barriers are initialised before anyone arrives on them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_base_s;

  TileWalker walk;
  walk.offsets = p.offsets;
  walk.E = p.E;
  walk.T = p.T;
  walk.NT = p.NT / CG;
  walk.row_round = ROUND;
  int e, ntp, row0, rows;
  const int nsb = (p.kstages + SPB - 1) / SPB;  // superblocks a tile touches
  const long long t_first = blockIdx.x / CG, t_step = gridDim.x / CG;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer: TMA for B, bulk copies for packed slabs
    if (lane == 0) {
      uint32_t it = 0, pit = 0;  // stage counter, packed-slab counter (both run across tiles)
      bool ok = true;
      RT_DECL(w_pempty = 0, w_empty = 0, t_begin = RT_NOW());
      // One slab (all stacked terms of one superblock) is always requested one superblock ahead of the
      // stage loads, so the dequant warps find it in shared memory when they get there.
      TileWalker ahead = walk;
      int ae, antp, arow0, arows, asb = 0;
      long long at = t_first;
      bool have = ahead.seek(at, ae, antp, arow0, arows);
      auto issue_slab = [&]() -> bool {
        while (have && arows <= 0) { at += t_step; have = ahead.seek(at, ae, antp, arow0, arows); }
        if (!have) return true;
        const int slot = pit & 1;
        if (!RT_WAIT(w_pempty, mbar_wait<true>(smem_u32(&bar_pempty[slot]), ((pit >> 1) & 1u) ^ 1u, abort_flag))) return false;
        const uint32_t full = smem_u32(&bar_pfull[slot]);
        mbar_arrive_expect_tx(full, (uint32_t)p.n_terms * PF_SLAB);
        const int64_t off = (((int64_t)ae * p.NT + antp * CG + rank) * p.S + asb) * PF_SLAB;
        for (int i = 0; i < p.n_terms; ++i)
          bulk_load(smem_u32(slabs + (slot * p.n_terms + i) * PF_SLAB), p.tiled[i] + off, PF_SLAB, full);
        ++pit;
        if (++asb >= nsb) {
          asb = 0;
          at += t_step;
          have = ahead.seek(at, ae, antp, arow0, arows);
        }
        return true;
      };
      ok = issue_slab();
      const uint32_t full0 = smem_u32(&bar_full[0]), empty0 = smem_u32(&bar_empty[0]), dst0 = smem_u32(smem);
      const uint32_t lfull0 = CG == 2 ? mapa(full0, 0) : full0;  // the stage-full barriers of the pair's leader
      for (long long t = t_first; ok && walk.seek(t, e, ntp, row0, rows); t += t_step) {
        if (rows <= 0) continue;
        const int n_eff = (rows + ROUND - 1) / ROUND * ROUND;
        const int my_rows = n_eff / CG;                    // token rows this CTA stages (a multiple of 16)
        const int my_row0 = row0 + (int)rank * my_rows;
        const CUtensorMap* map = &xmaps.m[my_rows / 16 - 1];
        const uint32_t bytes = (uint32_t)my_rows * 128u;
        int sbk = 0;
        for (int ks = 0; ks < p.kstages; ++ks, ++it) {
          if (sbk == 0 && !issue_slab()) { ok = false; break; }
          if (++sbk == SPB) sbk = 0;
          const uint32_t s = it & smask;
          if (!RT_WAIT(w_empty, mbar_wait(empty0 + s * 8, ((it >> sshift) & 1u) ^ 1u, abort_flag))) { ok = false; break; }
          if (CG == 2) {
            if (leader) mbar_arrive_expect_tx(full0 + s * 8, bytes * 2u);  // both CTAs stage the same number of bytes
            tma_load_2d_2cta(dst0 + s * STAGE_BYTES, map, ks * 64, my_row0, lfull0 + s * 8);
          } else {
            mbar_arrive_expect_tx(full0 + s * 8, bytes);
            tma_load_2d(dst0 + s * STAGE_BYTES, map, ks * 64, my_row0, full0 + s * 8);
          }
        }
      }
      RT_ADD(0, RT_NOW() - t_begin); RT_ADD(1, w_pempty); RT_ADD(2, w_empty); RT_ADD(3, it); RT_ADD(4, 1);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (the leader CTA of a pair only)
    if (lane == 0 && leader) {
      uint32_t it = 0, tile = 0;
      bool ok = true;
      const uint64_t b_desc0 = umma_desc(smem_u32(smem));
      const uint32_t b_desc_lo = (uint32_t)b_desc0, b_desc_hi = (uint32_t)(b_desc0 >> 32);
      RT_DECL(w_tempty = 0, w_full = 0, t_begin = RT_NOW());
      for (long long t = t_first; ok && walk.seek(t, e, ntp, row0, rows); t += t_step) {
        if (rows <= 0) continue;
        // one accumulator: the epilogue of the previous tile must have drained it
        if (!RT_WAIT(w_tempty, mbar_wait(smem_u32(&bar_tempty[0]), (tile & 1u) ^ 1u, abort_flag))) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t n_eff = (uint32_t)((rows + ROUND - 1) / ROUND * ROUND);
        // instruction descriptor: D f32, A f16, B f16, both K-major, N >> 3 at bit 17, M >> 4 at bit 24
        const uint32_t idesc = (1u << 4) | ((n_eff >> 3) << 17) | (((128u * CG) >> 4) << 24);
        const uint32_t d_tmem = tmem;
        for (int ks = 0; ks < p.kstages; ++ks, ++it) {
          const int s = (int)(it & smask);
          if (!RT_WAIT(w_full, mbar_wait(smem_u32(&bar_full[s]), (it >> sshift) & 1u, abort_flag))) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_tmem = tmem + PF_TN + s * PF_A_COLS;  // this stage's slot of the A ring
          // only the start-address field of the B descriptor changes with the stage and the K step
          const uint32_t b_lo = b_desc_lo + (uint32_t)s * (STAGE_BYTES >> 4);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            uint64_t db;
            asm volatile("mov.b64 %0, {%1, %2};" : "=l"(db) : "r"(b_lo + kk * 2), "r"(b_desc_hi));
            if (CG == 2) umma_f16_ts_2cta(d_tmem, a_tmem + kk * 8, db, idesc, (ks > 0 || kk > 0) ? 1u : 0u);
            else umma_f16_ts(d_tmem, a_tmem + kk * 8, db, idesc, (ks > 0 || kk > 0) ? 1u : 0u);
          }
          // frees the stage (in both CTAs of a pair) when these MMAs have read it
          if (CG == 2) umma_commit_2cta(smem_u32(&bar_empty[s]));
          else umma_commit(smem_u32(&bar_empty[s]));
        }
        if (ok) {
          if (CG == 2) umma_commit_2cta(smem_u32(&bar_tfull[0]));
          else umma_commit(smem_u32(&bar_tfull[0]));
        }
        ++tile;
      }
      RT_ADD(8, RT_NOW() - t_begin); RT_ADD(9, w_tempty); RT_ADD(10, w_full); RT_ADD(11, it); RT_ADD(12, 1); RT_ADD(13, tile);
    } else if (CG == 2 && lane == 0) {
      // non-leader CTA of a pair: when this CTA's dequant warps have written their A tile of a stage, tell the
      // leader's stage-full barrier (one cluster-scope arrive per stage instead of one per dequant warp)
      uint32_t it = 0;
      bool ok = true;
      for (long long t = t_first; ok && walk.seek(t, e, ntp, row0, rows); t += t_step) {
        if (rows <= 0) continue;
        for (int ks = 0; ks < p.kstages; ++ks, ++it) {
          const int s = (int)(it & smask);
          if (!mbar_wait(smem_u32(&bar_afull[s]), (it >> sshift) & 1u, abort_flag)) { ok = false; break; }
          mbar_arrive_cluster(mapa(smem_u32(&bar_full[s]), 0));
        }
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    uint32_t tile = 0;
    RT_DECL(w_tfull = 0, t_begin = RT_NOW());
    for (long long t = t_first; walk.seek(t, e, ntp, row0, rows); t += t_step) {
      if (rows <= 0) continue;
      if (!RT_WAIT(w_tfull, mbar_wait<true>(smem_u32(&bar_tfull[0]), tile & 1u, abort_flag))) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int n = (ntp * CG + (int)rank) * 128 + q * 32 + lane;
      const bool n_ok = n < p.N;
      const uint32_t taddr0 = tmem + ((uint32_t)(q * 32) << 16);
      const int n_eff = (rows + 15) & ~15;
      // this thread owns output column n; consecutive token rows are p.N elements apart
      const size_t esz = p.out_dtype == DST_OUT_F32 ? 4 : 2;
      uint8_t* optr = static_cast<uint8_t*>(p.out) + ((size_t)row0 * p.N + (n_ok ? n : 0)) * esz;
      const size_t ostep = (size_t)p.N * esz;
      for (int c0 = 0; c0 < n_eff; c0 += 32) {
        uint32_t v[32];
        if (c0 + 32 <= n_eff) {
          TMEM_LD_32(v, taddr0 + c0);
        } else {
          TMEM_LD_16(v, taddr0 + c0);
#pragma unroll
          for (int j = 16; j < 32; ++j) v[j] = 0u;
        }
        const float rs_lane = (p.row_scale && c0 + lane < rows) ? p.row_scale[row0 + c0 + lane] : 1.f;
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int lim = n_ok ? rows - c0 : 0;  // token rows of this chunk that exist (and a column that exists)
        if (p.out_dtype == DST_OUT_BF16) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float val = __uint_as_float(v[j]) * __shfl_sync(0xffffffffu, rs_lane, j);
            if (j < lim) *reinterpret_cast<__nv_bfloat16*>(optr + j * ostep) = __float2bfloat16_rn(val);
          }
        } else if (p.out_dtype == DST_OUT_F16) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float val = __uint_as_float(v[j]) * __shfl_sync(0xffffffffu, rs_lane, j);
            if (j < lim) *reinterpret_cast<__half*>(optr + j * ostep) = __float2half_rn(val);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float val = __uint_as_float(v[j]) * __shfl_sync(0xffffffffu, rs_lane, j);
            if (j < lim) {
              float* o = reinterpret_cast<float*>(optr + j * ostep);
              *o = p.accumulate ? *o + val : val;
            }
          }
        }
        optr += 32 * ostep;
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        if (CG == 2) mbar_arrive_cluster(mapa(smem_u32(&bar_tempty[0]), 0));
        else mbar_arrive(smem_u32(&bar_tempty[0]));
      }
      ++tile;
    }
    if (warp == 2 && lane == 0) { RT_ADD(16, RT_NOW() - t_begin); RT_ADD(17, w_tfull); RT_ADD(18, 1); }
  } else {
    // ------------------------------------------------------------------ dequant producers (weights)
    // A warp may only write the TMEM lanes of its own quarter (warp id % 4): it owns those 32 weight rows.
    const int r = (warp & 3) * 32 + lane;
    const uint32_t grp = (uint32_t)(warp - 6) >> 2;  // this warp dequantises the stages with (stage index & 3) == grp
    const int swz = (r >> 1) & 3;  // swizzle of the tiled layout: logical word w sits at physical word (((w & 3) ^ swz) << 2) | (w >> 2)
    const uint32_t lut_addr = smem_u32(lut) + (uint32_t)(lane & 7) * 16u;
    const bool vec_scales = (p.G & 7) == 0;  // rows of 8 k scales are 16-byte aligned
    uint32_t it = 0, pit = 0;
    bool ok = true;
    RT_DECL(w_pfull = 0, w_dempty = 0, w_tail = 0, t_begin = RT_NOW());
    // scales of the row for 8 groups (16 stages) at a time, fetched one block ahead (also across tiles)
    uint4 sc_next[TERMS];
    TileWalker ahead = walk;
    int ae, antp, arow0, arows;
    long long at = t_first;
    bool have = ahead.seek(at, ae, antp, arow0, arows);
    while (have && arows <= 0) { at += t_step; have = ahead.seek(at, ae, antp, arow0, arows); }
    auto load_scales = [&](int ee, int nn, int g0, uint4* dst) {
      const bool n_ok = nn < p.N;
#pragma unroll
      for (int i = 0; i < TERMS; ++i) {
        if (i < p.n_terms) {
          if (!n_ok || g0 >= p.G) {
            dst[i] = make_uint4(0u, 0u, 0u, 0u);
          } else if (vec_scales) {
            dst[i] = *reinterpret_cast<const uint4*>(p.scale[i] + ((int64_t)ee * p.N + nn) * p.G + g0);
          } else {
            uint32_t h[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
              h[j] = g0 + j < p.G ? (uint32_t)__half_as_ushort(p.scale[i][((int64_t)ee * p.N + nn) * p.G + g0 + j]) : 0u;
            dst[i] = make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16), h[6] | (h[7] << 16));
          }
        }
      }
    };
    if (have) load_scales(ae, (antp * CG + (int)rank) * 128 + r, 0, sc_next);
    for (long long t = t_first; ok && walk.seek(t, e, ntp, row0, rows); t += t_step) {
      if (rows <= 0) continue;
      const int nt = ntp * CG + (int)rank;
      // the tile after this one (for the scale prefetch at the end of this tile)
      at = t + t_step;
      have = ahead.seek(at, ae, antp, arow0, arows);
      while (have && arows <= 0) { at += t_step; have = ahead.seek(at, ae, antp, arow0, arows); }
      uint4 sc[TERMS];
      int sbk = -1;
      for (int ks = 0; ks < p.kstages; ++ks, ++it) {
        if (++sbk == SPB) sbk = 0;
        const int s = (int)(it & smask);
        if ((ks & 15) == 0) {
#pragma unroll
          for (int i = 0; i < TERMS; ++i) sc[i] = sc_next[i];
          if (ks + 16 < p.kstages) load_scales(e, nt * 128 + r, (ks + 16) >> 1, sc_next);
          else if (have) load_scales(ae, (antp * CG + (int)rank) * 128 + r, 0, sc_next);
        }
        const uint32_t slot = pit & 1u;
        if (sbk == 0 && !RT_WAIT(w_pfull, mbar_wait(smem_u32(&bar_pfull[slot]), (pit >> 1) & 1u, abort_flag))) { ok = false; break; }
        const uint8_t* slab = slabs + (size_t)slot * p.n_terms * PF_SLAB + r * 64;
        const bool last_of_slab = sbk == SPB - 1 || ks == p.kstages - 1;
        if ((it & 3u) != grp) {  // another group's stage: only keep the slab ring's bookkeeping in step
          if (last_of_slab) {
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_pempty[slot]));
            ++pit;
          }
          continue;
        }
        const int g = (ks >> 1) & 7;  // 64-trit stage -> 128-trit scale group, inside the 8 held in sc
        uint32_t v[32];               // the row's 64 weights of this stage: 32 fp16 pairs = 32 TMEM columns
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          __half2 acc[8];
          if (FMT == 2) {
            const int boff = ((q4 ^ swz) << 4) + sbk * 4;  // logical word 4 sbk + q4
#pragma unroll
            for (int i = 0; i < TERMS; ++i) {
              if (i < p.n_terms) {
                const uint32_t w = *reinterpret_cast<const uint32_t*>(slab + i * PF_SLAB + boff);
                const __half2 s2 = pick_scale(sc[i], g);
                if (i == 0) tq2_word<true>(w, s2, acc);
                else tq2_word<false>(w, s2, acc);
              }
            }
          } else {
            const int qq = sbk * 4 + q4;  // 16-trit slot 0..19 inside the 320-trit superblock
            const int tau = qq * 16, b0 = tau / 5, o = tau - b0 * 5;
            const int wi = b0 >> 2, sh = (b0 & 3) * 8;
#pragma unroll
            for (int i = 0; i < TERMS; ++i) {
              if (i < p.n_terms) {
                const uint32_t* wp = reinterpret_cast<const uint32_t*>(slab + i * PF_SLAB);
                const uint32_t w0 = wp[(((wi & 3) ^ swz) << 2) | (wi >> 2)];
                const uint32_t w1 = wi + 1 < 16 ? wp[((((wi + 1) & 3) ^ swz) << 2) | ((wi + 1) >> 2)] : 0u;
                const uint32_t win = __funnelshift_r(w0, w1, sh);  // bytes b0 .. b0 + 3 of the row-superblock
                const __half2 s2 = pick_scale(sc[i], g);
                if (i == 0) tq1_dispatch<true>(o, win, lut_addr, s2, acc);
                else tq1_dispatch<false>(o, win, lut_addr, s2, acc);
              }
            }
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) v[q4 * 8 + j] = h2_bits(acc[j]);
        }
        if (last_of_slab) {  // last read of this slab: hand the slot back
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bar_pempty[slot]));
          ++pit;
        }
        if (!RT_WAIT(w_dempty, mbar_wait<true>(smem_u32(&bar_empty[s]), ((it >> sshift) & 1u) ^ 1u, abort_flag))) { ok = false; break; }
        RT_DECL(t_tail = RT_NOW());
        {
          const uint32_t taddr = tmem + ((uint32_t)((warp & 3) * 32) << 16) + PF_TN + s * PF_A_COLS;
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) tmem_st_8(taddr + q4 * 8, v + q4 * 8);
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(CG == 2 && !leader ? &bar_afull[s] : &bar_full[s]));
#ifdef DST_ROLE_TIMERS
        w_tail += RT_NOW() - t_tail;
#endif
      }
    }
    if (warp == 6 && lane == 0) { RT_ADD(24, RT_NOW() - t_begin); RT_ADD(25, w_pfull); RT_ADD(26, w_dempty); RT_ADD(27, it); RT_ADD(28, 1); RT_ADD(29, w_tail); }
  }

  // ------------------------------------------------------------------ teardown
  if (*abort_flag) {
    // give copies and MMAs still in flight time to land before shared memory and TMEM are released
    const long long t0 = clock64();
    while (clock64() - t0 < 4000000LL) __nanosleep(1000);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (CG == 2) cluster_sync_all();  // neither CTA leaves while its peer may still read its shared memory or signal it
  if (warp == 1) {
    __syncwarp();
    if (CG == 2) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512));
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512));
  }
  if (tid == 0 && abort_s) atomicExch(&g_device_status, DST_ERR_TIMEOUT);
}

// ------------------------------------------------------------------------------------------ activation conversion
// bf16 (or fp16) rows -> fp16 rows scaled by 2^-e with e = floor(log2(absmax)) - 7, so every row's
// largest magnitude lies in [128, 256); row_scale_out[m] = 2^e * row_scale_in[m].
template <typename XT>
__global__ void convert_rows_kernel(const XT* __restrict__ x, int64_t K, const float* __restrict__ rs_in, __half* __restrict__ y,
                                    float* __restrict__ rs_out) {
  __shared__ float red[32];
  const int64_t m = blockIdx.x;
  const XT* row = x + m * K;
  float amax = 0.f;
  for (int64_t k = threadIdx.x; k < K; k += blockDim.x) amax = fmaxf(amax, fabsf((float)row[k]));
  for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    if (threadIdx.x == 0) red[0] = v;
  }
  __syncthreads();
  amax = red[0];
  int ex = 0;
  if (amax > 0.f && isfinite(amax)) {
    (void)frexpf(amax, &ex);  // amax = f * 2^ex, f in [0.5, 1)
    ex -= 8;                  // amax * 2^-ex in [128, 256)
  }
  const float down = ldexpf(1.f, -ex);
  for (int64_t k = threadIdx.x; k < K; k += blockDim.x) y[m * K + k] = __float2half_rn((float)row[k] * down);
  if (threadIdx.x == 0) rs_out[m] = ldexpf(1.f, ex) * (rs_in ? rs_in[m] : 1.f);
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(sym);
  }
  return fn;
}

template <int FMT, int CG, int TERMS>
int launch_fmt(const TmaMaps& maps, PrefillParams p, long long tiles_upper, cudaStream_t st) {
  // deepest stage ring the shared-memory budget allows next to the packed slabs and the TQ1 table
  const size_t stage_bytes = PF_B_BYTES / CG;
  const size_t fixed = 1024 + (size_t)2 * p.n_terms * PF_SLAB + (FMT == 1 ? PF_LUT_BYTES : 0);
  const int fit = (int)((PF_SMEM_MAX - fixed) / stage_bytes);
  if (fit < 2) return DST_ERR_UNSUPPORTED;
  p.nstage_log2 = fit >= 8 ? 3 : (fit >= 4 ? 2 : 1);  // a power of two, so ring indices are a mask and a shift
  const int nstage = 1 << p.nstage_log2;
  const size_t smem = fixed + (size_t)nstage * stage_bytes;
  auto kernel = prefill_kernel<FMT, CG, TERMS>;
  DST_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int dev = 0, sms = 148;
  DST_CUDA_TRY(cudaGetDevice(&dev));
  DST_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(PF_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  int n_attr = 0;
  long long units = tiles_upper / CG;  // tiles (CG = 1) or pair tiles (CG = 2) at most
  if (units < 1) units = 1;
  int groups = sms / CG;
  if (CG == 2) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    n_attr = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cfg.gridDim = dim3((unsigned)sms / 2 * 2, 1, 1);
    int max_clusters = 0;
    DST_CUDA_TRY(cudaOccupancyMaxActiveClusters(&max_clusters, kernel, &cfg));
    if (max_clusters < 1) return DST_ERR_UNSUPPORTED;
    groups = max_clusters < groups ? max_clusters : groups;
  }
  if (units < groups) groups = (int)units;
  cfg.gridDim = dim3((unsigned)(groups * CG), 1, 1);
  cfg.attrs = n_attr ? attr : nullptr;
  cfg.numAttrs = n_attr;
  DST_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, maps, p));
  return DST_OK;
}

}  // namespace

size_t prefill_workspace_bytes(int act_dtype, int64_t T, int64_t K) {
  (void)act_dtype;  // fp16 activations are re-scaled per row as well, so every input type is converted
  return (size_t)T * (size_t)K * 2 + (((size_t)T * 4 + 255) & ~(size_t)255) + 256;
}

bool prefill_supports(const GemmArgs& a) {
  return a.weight_layout == DST_LAYOUT_TILED && a.group == 128 && a.K % 128 == 0 && a.scale_dtype == DST_SCALE_F16 &&
         ((a.act_dtype == DST_ACT_F16_NORM && a.row_scale != nullptr) ||
          ((a.act_dtype == DST_ACT_BF16 || a.act_dtype == DST_ACT_F16) && a.workspace != nullptr &&
           a.workspace_bytes >= prefill_workspace_bytes(a.act_dtype, a.T, a.K))) &&
         a.T < (int64_t(1) << 30) &&
         a.N <= (int64_t(1) << 22) && encode_fn() != nullptr;
}

int launch_prefill(const GemmArgs& a, cudaStream_t stream) {
  if (a.T == 0 || a.N == 0 || a.E == 0) return DST_OK;
  if (!prefill_supports(a)) return DST_ERR_UNSUPPORTED;
  const bool prenorm = a.act_dtype == DST_ACT_F16_NORM;
  if (!prenorm && (reinterpret_cast<uintptr_t>(a.workspace) & 255) != 0) return DST_ERR_ALIGNMENT;
  if (prenorm && (reinterpret_cast<uintptr_t>(a.x) & 15) != 0) return DST_ERR_ALIGNMENT;
  for (int i = 0; i < a.terms.n; ++i)
    if ((reinterpret_cast<uintptr_t>(a.terms.packed[i]) & 15) != 0 || (reinterpret_cast<uintptr_t>(a.terms.scale[i]) & 15) != 0)
      return DST_ERR_ALIGNMENT;

  // 1. activations -> fp16 rows + per-row power-of-two factor, in the workspace
  //    (skipped when the caller hands in rows that are in that format already)
  const __half* xh = prenorm ? static_cast<const __half*>(a.x) : static_cast<const __half*>(a.workspace);
  const float* rs = prenorm ? a.row_scale
                            : reinterpret_cast<const float*>(static_cast<const uint8_t*>(a.workspace) + (((size_t)a.T * a.K * 2 + 255) & ~(size_t)255));
  if (prenorm) {
    // nothing to convert
  } else if (a.act_dtype == DST_ACT_BF16)
    convert_rows_kernel<__nv_bfloat16><<<(unsigned)a.T, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(a.x), a.K, a.row_scale,
                                                                          static_cast<__half*>(a.workspace), const_cast<float*>(rs));
  else
    convert_rows_kernel<__half><<<(unsigned)a.T, 256, 0, stream>>>(static_cast<const __half*>(a.x), a.K, a.row_scale,
                                                                   static_cast<__half*>(a.workspace), const_cast<float*>(rs));
  DST_CUDA_TRY(cudaGetLastError());

  // 2. tensor maps over the fp16 rows: [T, K], boxes of 64 K-elements x 16 i token rows, 128-byte swizzle, zero fill outside
  TmaMaps maps;
  const cuuint64_t dims[2] = {(cuuint64_t)a.K, (cuuint64_t)a.T};
  const cuuint64_t strides[1] = {(cuuint64_t)a.K * 2};
  const cuuint32_t estr[2] = {1, 1};
  for (int i = 0; i < 16; ++i) {
    const cuuint32_t box[2] = {64, (cuuint32_t)(16 * (i + 1))};
    const CUresult cr = encode_fn()(&maps.m[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(xh), dims, strides, box, estr,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return record_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
  }

  PrefillParams p;
  for (int i = 0; i < DST_MAX_TERMS; ++i) {
    p.tiled[i] = i < a.terms.n ? a.terms.packed[i] : nullptr;
    p.scale[i] = i < a.terms.n ? static_cast<const __half*>(a.terms.scale[i]) : nullptr;
  }
  p.n_terms = a.terms.n;
  p.row_scale = rs;
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
  p.kstages = (int)(a.K / 64);
  const long long tiles_upper = ((long long)cdiv64(a.T, PF_TN) + a.E) * p.NT;
  // CTA pairs (cta_group::2) need an even number of 128-row weight tiles. They are correct but measured SLOWER
  // than single CTAs here (2.51 M vs 1.58 M cycles per launch on the same case): the cross-CTA barrier traffic
  // (remote arrives, multicast commits) costs more than the halved activation traffic saves while the kernel is
  // bound by its per-stage handshakes. Kept compiled and tested behind this switch for when that changes.
  const bool pairs = kUseCtaPairs && a.N % 256 == 0;
#define DST_PF_LAUNCH(FMT_, CG_)                                                                          \
  (a.terms.n == 1 ? launch_fmt<FMT_, CG_, 1>(maps, p, tiles_upper, stream)                       \
                  : a.terms.n == 2 ? launch_fmt<FMT_, CG_, 2>(maps, p, tiles_upper, stream)      \
                                   : launch_fmt<FMT_, CG_, 4>(maps, p, tiles_upper, stream))
  if (a.fmt == DST_FMT_TQ2) return pairs ? DST_PF_LAUNCH(2, 2) : DST_PF_LAUNCH(2, 1);
  return pairs ? DST_PF_LAUNCH(1, 2) : DST_PF_LAUNCH(1, 1);
#undef DST_PF_LAUNCH
}

}  // namespace dst

#ifdef DST_ROLE_TIMERS
// Profiling builds only: copies (and optionally clears) the 64 role-timer slots. Slots: 0-4 producer (total
// cycles, wait packed-slot free, wait stage free, stages, threads), 8-13 MMA issuer (total, wait accumulator
// free, wait stage full, stages, threads, tiles), 16-18 epilogue warp (total, wait accumulator full, threads),
// 24-29 one dequant warp (total, wait packed slab, wait stage free, stages, threads, store+fence+arrive).
extern "C" int dst_role_timers(unsigned long long* out, int reset) {
  DST_CUDA_TRY(cudaDeviceSynchronize());
  DST_CUDA_TRY(cudaMemcpyFromSymbol(out, dst::g_role_timers, sizeof(unsigned long long) * 64));
  if (reset) {
    unsigned long long z[64] = {0};
    DST_CUDA_TRY(cudaMemcpyToSymbol(dst::g_role_timers, z, sizeof(z)));
  }
  return DST_OK;
}
#endif

extern "C" int dst_check_device_status(dst_stream_t stream) {
  DST_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  int st = 0;
  DST_CUDA_TRY(cudaMemcpyFromSymbol(&st, dst::g_device_status, sizeof(int)));
  if (st != 0) {
    const int zero = 0;
    DST_CUDA_TRY(cudaMemcpyToSymbol(dst::g_device_status, &zero, sizeof(int)));
    return DST_ERR_TIMEOUT;
  }
  return DST_OK;
}

// ------------------------------------------------------------------------------------------ no-allocation entry
// Scratch for dst_ternary_grouped_gemm_noalloc: the fp16 copy of the activations and the per-row factors
// that the tcgen05 kernel otherwise keeps in a caller-provided workspace. It is part of the library
// image, so every GPU that loads the library holds these bytes until the process exits.
static __device__ __align__(256) unsigned char g_noalloc_scratch[DST_NOALLOC_SCRATCH_BYTES];

namespace dst {
namespace {
constexpr int kMaxDevices = 64;
void* g_noalloc_ptr[kMaxDevices] = {nullptr};  // device address of g_noalloc_scratch, per device ordinal
}  // namespace
}  // namespace dst

extern "C" int dst_ternary_grouped_gemm_noalloc(void* out, int out_dtype, int accumulate, const void* x, int act_dtype,
                                                const float* row_scale, const int64_t* offsets, const int64_t* offsets_host,
                                                const void* const* packed_tiled, const void* const* scales, int n_terms,
                                                int64_t E, int64_t T, int64_t N, int64_t K, int fmt, dst_stream_t stream) {
  using namespace dst;
  if (K <= 0 || (fmt != DST_FMT_TQ1 && fmt != DST_FMT_TQ2)) return DST_ERR_BAD_ARG;
  if (out_dtype < DST_OUT_F32 || out_dtype > DST_OUT_F16 || (act_dtype != DST_ACT_BF16 && act_dtype != DST_ACT_F16))
    return DST_ERR_BAD_ARG;
  if (n_terms < 1 || n_terms > DST_MAX_TERMS || E < 0 || T < 0 || N < 0) return DST_ERR_BAD_ARG;
  if (accumulate && out_dtype != DST_OUT_F32) return DST_ERR_BAD_ARG;
  if (E > DST_MAX_EXPERTS || K > (int64_t(1) << 24) || N > (int64_t(1) << 22) || T >= (int64_t(1) << 30)) return DST_ERR_BAD_SHAPE;
  if (K % 128 != 0) return DST_ERR_UNSUPPORTED;
  if (E != 1 && E != 0 && offsets == nullptr) return DST_ERR_BAD_ARG;
  if (offsets_host) {
    if (offsets_host[0] != 0 || offsets_host[E] != T) return DST_ERR_BAD_OFFSETS;
    for (int64_t e = 0; e < E; ++e)
      if (offsets_host[e + 1] < offsets_host[e]) return DST_ERR_BAD_OFFSETS;
  }
  if (E == 0) return T == 0 ? DST_OK : DST_ERR_BAD_OFFSETS;
  if (T == 0 || N == 0) return DST_OK;
  if (!out || !x || !packed_tiled || !scales) return DST_ERR_BAD_ARG;
  // The whole scratch need of this call must fit the static array: refuse anything larger.
  if (prefill_workspace_bytes(act_dtype, T, K) > (size_t)DST_NOALLOC_SCRATCH_BYTES) return DST_ERR_TOO_LARGE;

  // Set-up, once per device, with that device current: in host code the array's name is only a
  // stand-in for the symbol, so ask the runtime for its device address and hand THAT to the kernels.
  int dev = -1;
  DST_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return DST_ERR_UNSUPPORTED;
  if (g_noalloc_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    DST_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
    if (ptr == nullptr) return record_cuda_error(cudaErrorInvalidSymbol, "cudaGetSymbolAddress(g_noalloc_scratch)");
    g_noalloc_ptr[dev] = ptr;
  }

  GemmArgs a;
  memset(&a, 0, sizeof(a));
  a.out = out;
  a.out_dtype = out_dtype;
  a.accumulate = accumulate;
  a.x = x;
  a.act_dtype = act_dtype;
  a.row_scale = row_scale;
  a.offsets = offsets;
  a.terms.n = n_terms;
  for (int i = 0; i < n_terms; ++i) {
    if (!packed_tiled[i] || !scales[i]) return DST_ERR_BAD_ARG;
    a.terms.packed[i] = static_cast<const uint8_t*>(packed_tiled[i]);
    a.terms.scale[i] = scales[i];
  }
  a.scale_dtype = DST_SCALE_F16;
  a.E = E;
  a.T = T;
  a.N = N;
  a.K = K;
  a.group = 128;
  a.Kp = cdiv64(K, fmt == DST_FMT_TQ2 ? 4 : 5);
  a.G = K / 128;
  a.fmt = fmt;
  a.max_rows = -1;
  a.weight_layout = DST_LAYOUT_TILED;
  a.workspace = g_noalloc_ptr[dev];
  a.workspace_bytes = DST_NOALLOC_SCRATCH_BYTES;
  return launch_prefill(a, static_cast<cudaStream_t>(stream));
}
