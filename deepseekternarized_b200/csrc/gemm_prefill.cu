// Prefill grouped ternary GEMM for sm_100a: tcgen05 MMA with TMEM accumulators, TMA-fed activations,
// warp-specialised dequantisation of packed trits straight into tensor memory.
//
// Problem (per expert e, rows ra..rb of the expert-sorted activations):
//     out[m, n] = row_scale[m] * sum_k x[m, k] * W_e[n, k],   W_e[n, k] = sum_i scale_i[e, n, k/128] * trit_i[e, n, k]
//
// Mapping ("swap AB"): the 128 weight rows of a tile are the MMA M dimension (TMEM lanes), the token rows of
// one expert (up to 320 per tile) are the MMA N dimension (TMEM columns), so tiles stay full when an expert
// has few rows and an expert with up to 320 rows has its weights dequantised ONCE per 128-row weight tile.
// Both operands are fp16, 64 K-elements per pipeline stage:
//   A (weights)      packed 8 KB slabs of the tiled layout (layout_kernels.cu) arrive by cp.async.bulk in a
//                    small ring; 16 dequant warps turn them into scale * trit, exact in fp16, and write them
//                    with tcgen05.st straight into TENSOR MEMORY (lane = weight row, one 32-bit column = two
//                    consecutive K elements; 32 columns per stage): the MMA takes A from TMEM, so the
//                    dequantised tile never passes through shared memory
//   B (activations)  fp16 rows fetched by one thread with cp.async.bulk.tensor (TMA) into K-major,
//                    128-byte-swizzled shared-memory stages (one box for up to 256 rows, two for more)
//   D (accumulator)  fp32 in TMEM columns 0..319 (two MMAs per K step, each over half of the token rows, from two
//                    issuing threads); columns 320..511 hold the A ring (stage s = slot s)
// Shared-memory bandwidth is what bounds this kernel when A goes through shared memory (measured: the MMA
// issuer stalled ~1100 cycles per 512-cycle stage); with A in TMEM only B is written and read there.
// bf16 activations are converted once to fp16 with a power-of-two factor per row (exact for every
// element within 2^-22 of the row's absolute maximum); the factor comes back through row_scale.
// tcgen05 kind::f16 refuses an fp16 A with a bf16 B (illegal instruction), hence the conversion.
//
// Warp roles (896 threads, one CTA per SM, persistent over tiles):
//   warp 0      TMA producer for B (one thread)
//   warp 1, 3   MMA issuers (one thread each, each over half of a tile's token rows); warp 1 owns the TMEM allocation
//   warp 2      bulk-copy producer of the packed slabs (one thread)
//   warps 4-11  epilogue: TMEM -> registers -> global, two warps per TMEM lane quarter (warp id % 4) taking
//               alternate 32-column chunks
//   warps 12-27 dequant producers for A, in four groups of four warps: group g owns the stages with global
//               index = g (mod 4), so four stages are dequantised at once (each warp's instruction stream is a
//               long dependent chain; one group per stage could not keep up with the MMAs); inside a group
//               the warp with id % 4 == q owns the 32 weight rows of TMEM lane quarter q, one thread per row
//               per 64-trit stage
// The accumulator is drained by warps that do nothing else. A variant in which the 20 dequant warps also drained
// it (tcgen05.ld in the same, register-starved instruction stream as the dequantisation) raised "unspecified
// launch failure" on the GPU although the same code with extra progress stores passed; tcgen05.ld writes its
// destination registers asynchronously, so that role keeps few live registers and nothing between the load and
// tcgen05.wait::ld.
//
// Every mbarrier wait is bounded by elapsed clock cycles; on expiry the CTA raises its abort flag, all
// roles leave their loops, the CTA frees TMEM and the kernel records DST_ERR_TIMEOUT in the status word.
#include <cuda.h>

#include <cstring>

#include "dst_common.cuh"

namespace dst {
namespace {

constexpr int PF_CTRL_WARPS = 4;
constexpr int PF_EPI_WARPS = 8;              // accumulator drain, two warps per TMEM lane quarter
constexpr int PF_GROUPS = 4;                 // dequant warp groups (4 warps each, one per TMEM lane quarter)
constexpr int PF_DQ_WARPS = 4 * PF_GROUPS;
constexpr int PF_DQ_WARP0 = PF_CTRL_WARPS + PF_EPI_WARPS;
constexpr int PF_THREADS = 32 * (PF_DQ_WARP0 + PF_DQ_WARPS);
constexpr int PF_TN_MAX = 320;               // token rows per tile at most = accumulator columns in TMEM
constexpr int PF_A_COLS = 32;                // TMEM columns of one A stage: 64 fp16 per weight row
constexpr int PF_MAX_STAGES = 12;            // stage ring depth at most; tn_max + depth * 32 <= 512 TMEM columns
constexpr int PF_MAX_SLABS = 3;
constexpr int PF_LUT_BYTES = 256 * 16 * 4;   // TQ1: 256 byte values x 16 bank replicas x 4 B
constexpr int PF_SLAB = 8192;                // one (row tile, superblock) slab of packed weights
constexpr int PF_MAX_E = 1023;               // experts per launch: two int arrays of E + 1 entries live in shared memory
constexpr int PF_EPI_TILE = 2048;             // bytes of an epilogue warp's transposition tile (32 token rows x 32 columns x 2 bytes)
constexpr int PF_SMEM_MAX = 232448;          // 227 KB of shared memory per CTA
constexpr int PF_SMEM_STATIC = 6144;         // allowance for the statically declared barriers, flags and the scatter form's row pointers
constexpr long long PF_WAIT_CYCLES = 4000000000LL;  // ~2 s

__device__ int g_device_status = 0;
// Test hooks (dst_debug_prefill_timeout): the cycle limit of the bounded waits, and a switch that makes the epilogue
// warps keep their "accumulator drained" arrivals to themselves, so that the MMA warps' wait for the accumulator runs
// out by design at a CTA's second tile. Nothing faults or spins unbounded: the wait gives up, the abort flag goes up,
// every role leaves, the CTA frees its TMEM and the status word says DST_ERR_TIMEOUT.
__device__ long long g_wait_cycles = PF_WAIT_CYCLES;
__device__ int g_drop_drain_arrivals = 0;
int g_debug_max_ctas = 0;  // host side: caps the grid when positive (so one CTA is sure to own several tiles)

// Optional per-role cycle accounting (build with -DDST_ROLE_TIMERS): where each warp role of the tcgen05
// kernel spends its time, summed over CTAs. Read with dst_role_timers(). Off in the shipped library.
#ifdef DST_ROLE_TIMERS
__device__ unsigned long long g_role_timers[64];
#define RT_DECL(...) long long __VA_ARGS__
#define RT_NOW() clock64()
#define RT_ADD(slot, v) atomicAdd(&g_role_timers[slot], (unsigned long long)(v))
#define RT_WAIT(acc, call) [&]() { const long long t0__ = clock64(); const bool r__ = (call); acc += clock64() - t0__; return r__; }()
#define RT_SPAN(acc, t0) acc += clock64() - (t0)
#else
#define RT_DECL(...)
#define RT_NOW() 0
#define RT_ADD(slot, v)
#define RT_WAIT(acc, call) (call)
#define RT_SPAN(acc, t0)
#endif

// One tensor map per TMA box height (16, 32, ... 256 token rows), so half a stage or a whole one is one TMA instruction.
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
  // chosen by the host from the shared-memory budget
  int tn_max;       // token rows per tile at most (a multiple of 32, <= PF_TN_MAX): accumulator columns 0 .. tn_max - 1, the A ring after them
  int rows_hint;    // most rows an expert is expected to have (host knowledge or twice the mean), sizes tn_max
  int nb;           // depth of the stage ring (B stage in shared memory + A slot in TMEM), 2..6
  int nslab;        // slots of the packed-slab ring, 2 or 3
  int wide_drain;   // 16-bit outputs, N % 8 == 0, 16-byte aligned rows: the accumulator is drained with 128-bit stores (drain_tile_wide)
  int small;        // token tiles of at most 128 rows: four warps drain the accumulator and the other four of that role join
                    // the dequantisation as a fifth group (the MMAs of such tiles are short, the dequantisation is the limit)
  // Scatter of the output rows (null: rows go to `out` in place). Row r is stored at row (row_target[r] & (2^48 - 1)) of
  // peer_out[row_target[r] >> 48]: the buffers of the GPUs whose tokens the rows belong to, written from the epilogue
  // with plain stores over NVLink while the tensor pipe works on the next tile. A negative target drops the row.
  const int64_t* row_target;
  void* peer_out[DST_MAX_PEERS];
  int n_peer_out;      // a target that names a buffer >= n_peer_out or a row >= peer_rows is dropped as well
  int64_t peer_rows;
};

// Entry d of the by-value pointer table, as a chain of selects over compile-time indices (indexing a parameter array
// with a run-time value copies the table into every thread's local memory).
__device__ __forceinline__ void* pf_peer_out(const PrefillParams& p, int d) {
  void* r = p.peer_out[0];
#pragma unroll
  for (int i = 1; i < DST_MAX_PEERS; ++i)
    if (d == i) r = p.peer_out[i];
  return r;
}

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
// Up to PF_SPIN_TRIES try_waits in a loop written in PTX: three to five instructions per poll. The same loop in C++
// compiles to about nine (convergence bookkeeping around a divergent loop), and with every role of the CTA polling
// some barrier most of the time the polls were ~40 % of all instructions this kernel issued at 64 rows per expert
// (per-opcode counters: 147 try_waits, 350 branches, 135 BSSY/BSYNC pairs and 138 YIELDs per 64-K stage).
#ifndef PF_SPLIT_MIN
#define PF_SPLIT_MIN 64
#endif
#ifndef PF_SPIN_TRIES
#define PF_SPIN_TRIES 64
#endif
__device__ __forceinline__ bool mbar_spin(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      ".reg .u32 n;\n"
      "mov.u32 n, %3;\n"
      "PF_SPIN:\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "@p bra PF_SPIN_DONE;\n"
      "sub.u32 n, n, 1;\n"
      "setp.ne.u32 q, n, 0;\n"
      "@q bra PF_SPIN;\n"
      "PF_SPIN_DONE:\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done) : "r"(bar), "r"(parity), "n"(PF_SPIN_TRIES) : "memory");
  return done != 0;
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
// Bounded wait: false when the abort flag is up or ~2 s of clock cycles have passed (checked between bursts of polls).
// BACKOFF sleeps between bursts: for roles that wait long, so their polling does not take issue slots from the dequant warps.
template <bool BACKOFF = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_test(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    if (mbar_spin(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > g_wait_cycles) {
      *abort_flag = 1;
      return false;
    }
    if (BACKOFF) __nanosleep(40);
  }
}

__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
  // K-major, SWIZZLE_128B: start address >> 4, LBO unused (1), SBO = 1024 B (8 rows x 128 B), version 1.
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}

// tcgen05.mma: A operand from tensor memory (lane = row, 32-bit column = 2 K elements), B from shared memory.
// Executed by a whole (converged) warp: one elected lane issues. The issuing warps run their loops with
// all 32 lanes so that addresses and descriptors are warp-uniform values (a single-lane branch keeps them in
// per-thread registers and every MMA then pays for moving them to the uniform registers the instruction reads).
__device__ __forceinline__ void umma_f16_ts_elect(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p, e;\nsetp.ne.b32 p, %4, 0;\nelect.sync _|e, 0xffffffff;\n"
               "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
               ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit_elect(uint32_t bar) {
  asm volatile("{\n.reg .pred e;\nelect.sync _|e, 0xffffffff;\n"
               "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n}\n" ::"r"(bar) : "memory");
}
// 8 consecutive 32-bit columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_st_8(uint32_t taddr, const uint32_t* v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
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

// 16 TMEM lanes x 32 columns in the layout of an MMA accumulator fragment: registers 4 b + {0, 1} = lane t / 4 of the 16,
// columns 8 b + 2 (t % 4) + {0, 1}; registers 4 b + {2, 3} = lane t / 4 + 8, the same columns (t = lane of the warp).
#define TMEM_LD_16x256_X4(v, taddr)                                                                                        \
  asm volatile("tcgen05.ld.sync.aligned.16x256b.x4.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"    \
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),           \
                 "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])      \
               : "r"(taddr))
// Four 8 x 8 matrices of 16-bit elements from registers (thread t: row t / 4, columns 2 (t % 4) + {0, 1} of each) to
// shared memory, TRANSPOSED: lanes 8 k .. 8 k + 7 give the addresses of the eight 16-byte rows of matrix k.
__device__ __forceinline__ void stmatrix_x4_trans(uint32_t addr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3) {
  asm volatile("stmatrix.sync.aligned.x4.trans.m8n8.shared.b16 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(r0), "r"(r1), "r"(r2), "r"(r3)
               : "memory");
}

// ------------------------------------------------------------------------------------------ tile walk
// Token rows a tile of `rows` rows occupies in the MMA N dimension: a multiple of 16 up to 256 (one MMA per K
// step), a multiple of 32 above (two MMAs, each over half of the rows, and N must be a multiple of 16).
__device__ __forceinline__ int tile_neff(int rows) { return rows <= 256 ? (rows + 15) & ~15 : (rows + 31) & ~31; }

// Tiles are numbered expert-major, then token tile, then weight-row tile (fastest), so the CTAs that run
// at the same time share an expert's activation rows in L2. The kernel keeps two int arrays in shared memory:
// offs[e] = first token row of expert e (clamped to [0, T]) and tpre[e] = number of tiles of the experts
// before e. A tile index is resolved with a short forward scan from the expert of the previous tile.
__device__ __forceinline__ int expert_tiles(const int* offs, int e, int tn_max, int NT) {
  const int n = offs[e + 1] - offs[e];
  return n > 0 ? (n + tn_max - 1) / tn_max * NT : 0;
}
// e: in = an expert at or before the tile's expert, out = the tile's expert. t must be < tpre[E].
__device__ __forceinline__ void tile_seek(const PrefillParams& p, const int* offs, const int* tpre, int t, int& e, int& nt, int& row0,
                                          int& rows) {
  while (tpre[e + 1] <= t) ++e;
  const int ra = offs[e], rb = offs[e + 1];  // rb > ra: the expert has tiles
  const int n = rb - ra;
  const int mt_count = (n + p.tn_max - 1) / p.tn_max;
  // an expert with more rows than one tile holds is split evenly, so no tile repeats the dequantisation
  // of the weights for a handful of left-over rows
  const int mt_rows = tile_neff((n + mt_count - 1) / mt_count);
  const unsigned local = (unsigned)(t - tpre[e]);
  const unsigned mt = local / (unsigned)p.NT;
  nt = (int)(local - mt * (unsigned)p.NT);
  row0 = ra + (int)mt * mt_rows;
  rows = rb - row0 < mt_rows ? rb - row0 : mt_rows;
}

// ------------------------------------------------------------------------------------------ dequant
__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 bits_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// Field f (0..4) of a word that holds trit digits u = t + 1 as 2-bit fields, an even trit in bits [2f, 2f+1]
// and the odd trit after it in bits [16+2f, 17+2f]: (w & (0x00030003 << 2f)) | 0x64006400 is the fp16 pair
// 1024 + u * 4^f; one fused multiply-add maps it to u - 1 exactly.
template <int F>
__device__ __forceinline__ __half2 trit_pair(uint32_t w) {
  constexpr float m = F == 0 ? 1.f : F == 1 ? 0.25f : F == 2 ? 0.0625f : F == 3 ? 0.015625f : 0.00390625f;
  constexpr float a = F == 0 ? -1025.f : F == 1 ? -257.f : F == 2 ? -65.f : F == 3 ? -17.f : -5.f;
  return __hfma2(bits_h2((w & (0x00030003u << (2 * F))) | 0x64006400u), __floats2half2_rn(m, m), __floats2half2_rn(a, a));
}
template <bool FIRST>
__device__ __forceinline__ void put(__half2& acc, __half2 t, __half2 s2) {
  acc = FIRST ? __hmul2(t, s2) : __hfma2(t, s2, acc);  // the group scale is applied exactly (trit in {-1, 0, 1})
}

// TQ2, tiled word format: 16 trits, trit 2j in field j of the low half, trit 2j+1 in field j of the high half.
template <bool FIRST>
__device__ __forceinline__ void tq2_word(uint32_t w, __half2 s2, __half2* acc /* 8 */) {
  const uint32_t w2 = w >> 10;
  put<FIRST>(acc[0], trit_pair<0>(w), s2);
  put<FIRST>(acc[1], trit_pair<1>(w), s2);
  put<FIRST>(acc[2], trit_pair<2>(w), s2);
  put<FIRST>(acc[3], trit_pair<3>(w), s2);
  put<FIRST>(acc[4], trit_pair<4>(w), s2);
  put<FIRST>(acc[5], trit_pair<0>(w2), s2);
  put<FIRST>(acc[6], trit_pair<1>(w2), s2);
  put<FIRST>(acc[7], trit_pair<2>(w2), s2);
}

// TQ1, tiled grouping (layout_kernels.cu): the 64 trits of stage s of a row-superblock are the 12 bytes
// 12 s .. 12 s + 11 (5 trits each) plus digit s of the 4 bytes 60..63. A shared-memory table maps a byte to its
// five digits as 2-bit fields placed for BOTH positions a byte can have in a pair of bytes (10 trits = 5 fp16
// pairs): as the first byte its digits 0,2,4 are the even trits of pairs 0,1,2 and digits 1,3 the odd trits of
// pairs 0,1; as the second byte digit 0 is the odd trit of pair 2, digits 1,3 the even and digits 2,4 the odd
// trits of pairs 3,4. The two placements use disjoint bits, so one AND-OR merges two table entries into a
// word of the TQ2 pair format above.
constexpr uint32_t TQ1_FIRST_MASK = 0x000F003Fu, TQ1_SECOND_MASK = 0x03F003C0u;
__host__ __device__ inline uint32_t tq1_table_entry(uint32_t byte) {
  const uint32_t f = tq1_fields(byte);
  const uint32_t d0 = f & 3u, d1 = (f >> 2) & 3u, d2 = (f >> 4) & 3u, d3 = (f >> 6) & 3u, d4 = (f >> 8) & 3u;
  const uint32_t first = d0 | (d2 << 2) | (d4 << 4) | (d1 << 16) | (d3 << 18);
  const uint32_t second = (d0 << 20) | (d1 << 6) | (d2 << 22) | (d3 << 8) | (d4 << 24);
  return first | second;
}
__device__ __forceinline__ uint32_t tq1_lookup(uint32_t lut_addr, uint32_t word, int byte) {
  const uint32_t idx = byte == 0 ? (word << 6) & 0x3FC0u : (word >> (8 * byte - 6)) & 0x3FC0u;  // byte value * 64
  uint32_t v;
  asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(lut_addr + idx));
  return v;
}
// w[0..2]: the stage's 12 own bytes, w[3]: bytes 60..63 of the row-superblock; sbk: stage inside the superblock
template <bool FIRST>
__device__ __forceinline__ void tq1_stage(const uint32_t* w, int sbk, uint32_t lut_addr, __half2 s2, __half2* acc /* 32 */) {
#pragma unroll
  for (int q = 0; q < 6; ++q) {
    const uint32_t c0 = tq1_lookup(lut_addr, w[(2 * q) >> 2], (2 * q) & 3);
    const uint32_t c1 = tq1_lookup(lut_addr, w[(2 * q + 1) >> 2], (2 * q + 1) & 3);
    const uint32_t m = (c0 & TQ1_FIRST_MASK) | (c1 & TQ1_SECOND_MASK);
    put<FIRST>(acc[5 * q + 0], trit_pair<0>(m), s2);
    put<FIRST>(acc[5 * q + 1], trit_pair<1>(m), s2);
    put<FIRST>(acc[5 * q + 2], trit_pair<2>(m), s2);
    put<FIRST>(acc[5 * q + 3], trit_pair<3>(m), s2);
    put<FIRST>(acc[5 * q + 4], trit_pair<4>(m), s2);
  }
  // trits 60..63: digit sbk of bytes 60..63; as a "first byte" entry digit d sits at bit (d >> 1) * 2 + (d & 1) * 16
  const int sh = (sbk >> 1) * 2 + (sbk & 1) * 16;
  const uint32_t e0 = (tq1_lookup(lut_addr, w[3], 0) >> sh) & 3u, e1 = (tq1_lookup(lut_addr, w[3], 1) >> sh) & 3u;
  const uint32_t e2 = (tq1_lookup(lut_addr, w[3], 2) >> sh) & 3u, e3 = (tq1_lookup(lut_addr, w[3], 3) >> sh) & 3u;
  put<FIRST>(acc[30], trit_pair<0>(e0 | (e1 << 16)), s2);
  put<FIRST>(acc[31], trit_pair<0>(e2 | (e3 << 16)), s2);
}

// Scale of group g (0..7 inside the 8 scales held in `sc`), as an fp16 pair.
__device__ __forceinline__ __half2 pick_scale(const uint4& sc, int g) {
  const uint32_t w = (g & 4) ? ((g & 2) ? sc.w : sc.z) : ((g & 2) ? sc.y : sc.x);
  const uint32_t h = (g & 1) ? (w >> 16) : (w & 0xFFFFu);
  return bits_h2(h | (h << 16));
}

// Drains a finished tile's accumulator: 32-column chunks col_first, col_first + col_step, ... of the warp's
// TMEM lane quarter -> registers -> global (thread = output column n, chunk column j = token row j).
__device__ __forceinline__ bool drain_tile(const PrefillParams& p, uint32_t tmem, int col_first, int col_step, int r, uint32_t tfull_bar,
                                        uint32_t tempty_bar, volatile int* abort_flag, int d_nt, int d_row0, int d_rows,
                                        uint32_t d_tile, const uint64_t* __restrict__ row_ptr) {
  const int lane = r & 31;
  const uint32_t lane_base = (uint32_t)(r & ~31) << 16;
  if (!mbar_wait(tfull_bar, d_tile & 1u, abort_flag)) return false;
  // Lanes leave the polling loop (and its per-thread sleeps) one by one; the .sync.aligned tcgen05 instructions
  // below must be executed by the whole warp together.
  __syncwarp();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const int dn = d_nt * 128 + r;
  const bool n_ok = dn < p.N;
  const int n_eff = tile_neff(d_rows);
  // this thread owns output column dn; consecutive token rows are p.N elements apart
  const size_t esz = p.out_dtype == DST_OUT_F32 ? 4 : 2;
  const size_t ostep = (size_t)p.N * esz;
  uint8_t* obase = static_cast<uint8_t*>(p.out) + ((size_t)d_row0 * p.N + (n_ok ? dn : 0)) * esz;
  for (int c0 = col_first; c0 < n_eff; c0 += col_step) {
    const float rs_lane = (p.row_scale && c0 + lane < d_rows) ? p.row_scale[d_row0 + c0 + lane] : 1.f;
    uint32_t v[32];
    if (c0 + 32 <= n_eff) {
      TMEM_LD_32(v, tmem + lane_base + c0);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    } else {
      TMEM_LD_16(v, tmem + lane_base + c0);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int j = 16; j < 32; ++j) v[j] = 0u;
    }
    const int lim = n_ok ? d_rows - c0 : 0;  // token rows of this chunk that exist (and a column that exists)
    uint8_t* optr = obase + (size_t)c0 * ostep;
    if (row_ptr != nullptr) {
      // scatter form: row_ptr[j] = where token row j of the tile goes (0: nowhere), looked up by this role while it
      // waited for the accumulator; every thread stores its column of the row there
      const size_t col = (size_t)(n_ok ? dn : 0) * esz;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float val = __uint_as_float(v[j]) * __shfl_sync(0xffffffffu, rs_lane, j);
        if (j < lim) {
          const uint64_t rowp = row_ptr[c0 + j];
          if (rowp != 0) {
            if (p.out_dtype == DST_OUT_BF16) *reinterpret_cast<__nv_bfloat16*>(rowp + col) = __float2bfloat16_rn(val);
            else *reinterpret_cast<__half*>(rowp + col) = __float2half_rn(val);
          }
        }
      }
    } else if (p.out_dtype == DST_OUT_BF16) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float val = __uint_as_float(v[j]) * __shfl_sync(0xffffffffu, rs_lane, j);
        if (j < lim) *reinterpret_cast<__nv_bfloat16*>(optr) = __float2bfloat16_rn(val);
        optr += ostep;
      }
    } else if (p.out_dtype == DST_OUT_F16) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float val = __uint_as_float(v[j]) * __shfl_sync(0xffffffffu, rs_lane, j);
        if (j < lim) *reinterpret_cast<__half*>(optr) = __float2half_rn(val);
        optr += ostep;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float val = __uint_as_float(v[j]) * __shfl_sync(0xffffffffu, rs_lane, j);
        if (j < lim) {
          float* o = reinterpret_cast<float*>(optr);
          *o = p.accumulate ? *o + val : val;
        }
        optr += ostep;
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncwarp();
  if (lane == 0 && !g_drop_drain_arrivals) mbar_arrive(tempty_bar);
  return true;
}

// The same drain for 16-bit outputs with N % 8 == 0: 128-bit stores. A thread of the plain drain owns one output
// column and stores 2 bytes per token row, ~5 instructions each, and the drain of the single accumulator is on the
// critical path (a fifth of the second expert GEMM's time). Here the accumulator is read as MMA-style fragments
// (16 lanes x 256 bits), scaled, packed to pairs and turned by stmatrix.trans into a [32 token rows][32 columns] tile
// in this warp's 2 KB of shared memory (16-byte pieces XOR-swizzled by the row pair: no bank conflicts either way);
// every lane then moves four 16-byte pieces = eight adjacent columns of a token row each to global memory. The
// scatter form (row_ptr) needs one destination lookup per piece instead of one per element.
__device__ __forceinline__ bool drain_tile_wide(const PrefillParams& p, uint32_t tmem, int col_first, int col_step, int warp_q, int lane,
                                                uint32_t tfull_bar, uint32_t tempty_bar, volatile int* abort_flag, int d_nt, int d_row0,
                                                int d_rows, uint32_t d_tile, const uint64_t* __restrict__ row_ptr, uint8_t* tile_smem) {
  if (!mbar_wait(tfull_bar, d_tile & 1u, abort_flag)) return false;
  __syncwarp();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const int n_eff = tile_neff(d_rows);
  const int n0 = d_nt * 128 + warp_q * 32;  // first output column of this warp's lane quarter
  const int t0 = lane & 3, t1 = lane >> 2;
  const uint32_t tile_a = smem_u32(tile_smem);
  // stmatrix: lane L addresses row r = L % 8 of matrix k = L / 8 of a group of four: (token block 2 x + k / 2, columns 16 h + 8 (k % 2) ..)
  const int st_r = lane & 7, st_g = (lane >> 3) & 1, st_b = lane >> 4;
  // read-back: piece q = 32 i + lane -> token row 8 i + lane / 4, columns 8 (lane % 4) ..
  const int rb_p = lane & 3, rb_t = lane >> 2;
  const size_t ostep = (size_t)p.N * 2;
  for (int c0 = col_first; c0 < n_eff; c0 += col_step) {
    const float rs_lane = (p.row_scale && c0 + lane < d_rows) ? p.row_scale[d_row0 + c0 + lane] : 1.f;
    float rs[8];  // of the token rows 8 b + 2 t0 + {0, 1} of the chunk
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      rs[2 * b] = __shfl_sync(0xffffffffu, rs_lane, 8 * b + 2 * t0);
      rs[2 * b + 1] = __shfl_sync(0xffffffffu, rs_lane, 8 * b + 2 * t0 + 1);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {  // lanes 16 h .. 16 h + 15 of the quarter = output columns n0 + 16 h ..
      uint32_t v[16];
      TMEM_LD_16x256_X4(v, tmem + ((uint32_t)(warp_q * 32 + 16 * h) << 16) + (uint32_t)c0);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      uint32_t m[8];  // m[2 b + g]: token block b, columns 16 h + 8 g ..: (row = column t1, pair = token rows 2 t0, 2 t0 + 1)
#pragma unroll
      for (int b = 0; b < 4; ++b)
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          const float lo = __uint_as_float(v[4 * b + 2 * g]) * rs[2 * b], hi = __uint_as_float(v[4 * b + 2 * g + 1]) * rs[2 * b + 1];
          if (p.out_dtype == DST_OUT_BF16) {
            const __nv_bfloat162 q = __floats2bfloat162_rn(lo, hi);
            m[2 * b + g] = *reinterpret_cast<const uint32_t*>(&q);
          } else {
            const __half2 q = __floats2half2_rn(lo, hi);
            m[2 * b + g] = *reinterpret_cast<const uint32_t*>(&q);
          }
        }
#pragma unroll
      for (int x = 0; x < 2; ++x) {  // token blocks 2 x, 2 x + 1
        const int tok = 8 * (2 * x + st_b) + st_r, piece = 2 * h + st_g;
        stmatrix_x4_trans(tile_a + (uint32_t)(tok * 64 + ((piece ^ ((tok >> 1) & 3)) << 4)), m[4 * x], m[4 * x + 1], m[4 * x + 2], m[4 * x + 3]);
      }
    }
    __syncwarp();
    const int n = n0 + 8 * rb_p;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int tok = 8 * i + rb_t;
      const uint4 q = *reinterpret_cast<const uint4*>(tile_smem + tok * 64 + ((rb_p ^ ((tok >> 1) & 3)) << 4));
      if (c0 + tok < d_rows && n < p.N) {
        if (row_ptr != nullptr) {
          const uint64_t rowp = row_ptr[c0 + tok];
          if (rowp != 0) *reinterpret_cast<uint4*>(rowp + (size_t)n * 2) = q;
        } else {
          *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.out) + (size_t)(d_row0 + c0 + tok) * ostep + (size_t)n * 2) = q;
        }
      }
    }
    __syncwarp();  // the tile is read before the next chunk overwrites it
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncwarp();
  if (lane == 0 && !g_drop_drain_arrivals) mbar_arrive(tempty_bar);
  return true;
}

// ------------------------------------------------------------------------------------------ the kernel
// Shared memory map (dynamic, 1024-byte aligned), per CTA:
//   [0, nb * tn_max * 128)          B stage ring: tn_max token rows x 64 fp16 per stage; stage s pairs with A slot s in TMEM
//   then nslab * n_terms * 8 KB     packed-weight slabs: slot-major, one 8 KB slab per stacked term
//   then 16 KB (TQ1 only)           table of digit fields, see tq1_table_entry
//   then 2 x 4 KB                   offs[E + 1], tpre[E + 1] (see tile_seek)
template <int FMT, int TERMS>
__global__ void __launch_bounds__(PF_THREADS, 1)
prefill_kernel(const __grid_constant__ TmaMaps xmaps, const PrefillParams p) {
  constexpr int SPB = FMT == 2 ? 4 : 5;  // 64-trit stages per 64-byte row-superblock
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t NB = (uint32_t)p.nb;
  const uint32_t stage_bytes = (uint32_t)p.tn_max * 128u;
  uint8_t* slabs = smem + NB * stage_bytes;
  uint8_t* lut = slabs + (size_t)p.nslab * p.n_terms * PF_SLAB;  // TQ1 only
  int* offs = reinterpret_cast<int*>(lut + (FMT == 1 ? PF_LUT_BYTES : 0));
  int* tpre = offs + (PF_MAX_E + 1);
  uint8_t* epi_tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(tpre + (PF_MAX_E + 1)) + 127) & ~static_cast<uintptr_t>(127));  // PF_EPI_WARPS x 2 KB
  __shared__ uint64_t bar_full[PF_MAX_STAGES], bar_empty[PF_MAX_STAGES], bar_tfull[1], bar_tempty[1], bar_pfull[PF_MAX_SLABS],
      bar_pempty[PF_MAX_SLABS];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ uint64_t bar_epi;                      // scatter form: the epilogue warps' own barrier, once per tile
  __shared__ uint64_t rowptr_s[2][PF_TN_MAX];       // scatter form: destination of every token row of a tile, two tiles alternating
  volatile int* abort_flag = &abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    abort_s = 0;
    for (int s = 0; s < PF_MAX_STAGES; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1 + 4);  // the TMA producer's expect_tx arrive + one arrive per warp of the dequant group that owns the stage
      mbar_init(smem_u32(&bar_empty[s]), 2);     // one tcgen05.commit per MMA issuer: the MMAs that read the stage are done
    }
    mbar_init(smem_u32(&bar_tfull[0]), 2);             // one tcgen05.commit per MMA issuer after the tile's last MMA
    mbar_init(smem_u32(&bar_tempty[0]), p.small ? 4 : PF_EPI_WARPS);  // every epilogue warp has drained its share of the accumulator
    mbar_init(smem_u32(&bar_epi), p.small ? 4 : PF_EPI_WARPS);
    for (int a = 0; a < PF_MAX_SLABS; ++a) {
      mbar_init(smem_u32(&bar_pfull[a]), 1);         // bulk-copy producer's expect_tx arrive
      mbar_init(smem_u32(&bar_pempty[a]), 4 * SPB);  // one arrive per (stage of the superblock, warp of its group)
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (FMT == 1) {
    uint32_t* lut32 = reinterpret_cast<uint32_t*>(lut);  // [byte value][replica]
    for (int i = tid; i < 256 * 16; i += PF_THREADS) lut32[i] = tq1_table_entry((uint32_t)i >> 4);
  }
  for (int i = tid; i <= p.E; i += PF_THREADS) {
    // offsets that were not validated on the host are clamped so no row index leaves [0, T)
    int64_t v = p.offsets ? p.offsets[i] : (i == 0 ? 0 : (int64_t)p.T);
    offs[i] = (int)(v < 0 ? 0 : (v > p.T ? p.T : v));
  }
  __syncthreads();
  if (warp == 0) {
    // tpre: exclusive prefix sum of the experts' tile counts; each lane takes a contiguous run of experts
    const int per = (p.E + 31) / 32, b0 = lane * per, b1 = b0 + per < p.E ? b0 + per : p.E;
    int sum = 0;
    for (int i = b0; i < b1; ++i) sum += expert_tiles(offs, i, p.tn_max, p.NT);
    int incl = sum;
    for (int d = 1; d < 32; d <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += up;
    }
    int run = incl - sum;
    for (int i = b0; i < b1; ++i) {
      tpre[i] = run;
      run += expert_tiles(offs, i, p.tn_max, p.NT);
    }
    if (lane == 31) tpre[p.E] = incl;
  } else if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_base_s;

  int e = 0, nt, row0, rows;
  const int nsb = (p.kstages + SPB - 1) / SPB;  // superblocks a tile touches
  const int t_step = (int)gridDim.x, n_tiles = tpre[p.E];

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer for B (activations)
    if (lane == 0) {
      uint32_t s = 0, ph = 0;
      bool ok = true;
      RT_DECL(w_empty = 0, n_it = 0, t_begin = RT_NOW());
      const uint32_t full0 = smem_u32(&bar_full[0]), empty0 = smem_u32(&bar_empty[0]), dst0 = smem_u32(smem);
      for (int t = (int)blockIdx.x; ok && t < n_tiles; t += t_step) {
        tile_seek(p, offs, tpre, t, e, nt, row0, rows);
        const int n_eff = tile_neff(rows);
        const int h = n_eff > 256 ? n_eff >> 1 : n_eff;  // token rows per TMA box and per MMA (a multiple of 16)
        const CUtensorMap* map = &xmaps.m[h / 16 - 1];
        const uint32_t bytes = (uint32_t)n_eff * 128u;
        for (int ks = 0; ks < p.kstages; ++ks) {
          if (!RT_WAIT(w_empty, mbar_wait(empty0 + s * 8, ph ^ 1u, abort_flag))) { ok = false; break; }
          mbar_arrive_expect_tx(full0 + s * 8, bytes);
          tma_load_2d(dst0 + s * stage_bytes, map, ks * 64, row0, full0 + s * 8);
          if (h != n_eff) tma_load_2d(dst0 + s * stage_bytes + (uint32_t)h * 128u, map, ks * 64, row0 + h, full0 + s * 8);
          if (++s == NB) { s = 0; ph ^= 1u; }
#ifdef DST_ROLE_TIMERS
          ++n_it;
#endif
        }
      }
      RT_ADD(0, RT_NOW() - t_begin); RT_ADD(2, w_empty); RT_ADD(3, n_it); RT_ADD(4, 1);
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------------ bulk-copy producer for the packed slabs
    if (lane == 0) {
      uint32_t slot = 0, ph = 0;
      bool ok = true;
      RT_DECL(w_pempty = 0, t_begin = RT_NOW());
      for (int t = (int)blockIdx.x; ok && t < n_tiles; t += t_step) {
        tile_seek(p, offs, tpre, t, e, nt, row0, rows);
        const int64_t off0 = ((int64_t)e * p.NT + nt) * p.S * PF_SLAB;
        for (int sb = 0; sb < nsb; ++sb) {
          if (!RT_WAIT(w_pempty, mbar_wait<true>(smem_u32(&bar_pempty[slot]), ph ^ 1u, abort_flag))) { ok = false; break; }
          const uint32_t full = smem_u32(&bar_pfull[slot]);
          mbar_arrive_expect_tx(full, (uint32_t)p.n_terms * PF_SLAB);
          for (int i = 0; i < p.n_terms; ++i)
            bulk_load(smem_u32(slabs + ((size_t)slot * p.n_terms + i) * PF_SLAB), p.tiled[i] + off0 + (int64_t)sb * PF_SLAB, PF_SLAB, full);
          if (++slot == (uint32_t)p.nslab) { slot = 0; ph ^= 1u; }
        }
      }
      RT_ADD(5, RT_NOW() - t_begin); RT_ADD(1, w_pempty);
    }
  } else if (warp == 1 || warp == 3) {
    // ------------------------------------------------------------------ MMA issuers
    // Two threads (in two warps, on two scheduler partitions) issue the MMAs of a stage: each owns half of the token
    // rows (its own accumulator columns and its own half of the B stage), so a stage costs each of them four
    // instructions instead of eight; a single thread could not issue them as fast as the tensor pipe runs them.
    // Tiles whose row count (padded to 16) is not a multiple of 32, or below 64, are issued by the first thread
    // alone; the second then only adds its arrivals to the barriers.
    {
      // all 32 lanes run this loop (see umma_f16_ts_elect); the elected lane issues the MMAs and the commits
      const uint32_t who = warp == 1 ? 0u : 1u;
      uint32_t s = 0, ph = 0, tile = 0;
      bool ok = true;
      const uint64_t b_desc0 = umma_desc(smem_u32(smem));
      const uint32_t b_desc_lo = (uint32_t)b_desc0, b_desc_hi = (uint32_t)(b_desc0 >> 32);
      RT_DECL(w_tempty = 0, w_full = 0, n_it = 0, t_begin = RT_NOW());
      for (int t = (int)blockIdx.x; ok && t < n_tiles; t += t_step) {
        tile_seek(p, offs, tpre, t, e, nt, row0, rows);
        // one accumulator: the previous tile must have been drained
        if (!__all_sync(0xffffffffu, RT_WAIT(w_tempty, mbar_wait(smem_u32(&bar_tempty[0]), (tile & 1u) ^ 1u, abort_flag)))) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t n_eff = (uint32_t)tile_neff(rows);
        const bool split = n_eff >= (uint32_t)PF_SPLIT_MIN && (n_eff & 31u) == 0u;  // tiles above 256 rows are padded to 32: always split
        const uint32_t h = split ? n_eff >> 1 : n_eff;           // token rows per MMA (a multiple of 16, at most 256)
        const bool active = split || who == 0u;
        // instruction descriptor: D f32, A f16, B f16, both K-major, N >> 3 at bit 17, M >> 4 at bit 24
        const uint32_t idesc = (1u << 4) | ((h >> 3) << 17) | ((128u >> 4) << 24);
        const uint32_t mine = split ? who * h : 0u;              // first token row (= accumulator column) of this warp's MMAs
        const uint32_t d_tmem = tmem + mine;
        const uint32_t b_off = (mine * 128u) >> 4;               // descriptor start-address units
        for (int ks = 0; ks < p.kstages; ++ks) {
          if (!__all_sync(0xffffffffu, RT_WAIT(w_full, mbar_wait(smem_u32(&bar_full[s]), ph, abort_flag)))) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          if (active) {
            const uint32_t a_tmem = tmem + (uint32_t)p.tn_max + s * PF_A_COLS;  // this stage's slot of the A ring
            // only the start-address field of the B descriptor changes with the stage, the K step and the half
            const uint32_t b_lo = b_desc_lo + s * (stage_bytes >> 4) + b_off;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              uint64_t db;
              asm volatile("mov.b64 %0, {%1, %2};" : "=l"(db) : "r"(b_lo + kk * 2), "r"(b_desc_hi));
              umma_f16_ts_elect(d_tmem, a_tmem + kk * 8, db, idesc, (ks > 0 || kk > 0) ? 1u : 0u);
            }
          }
          umma_commit_elect(smem_u32(&bar_empty[s]));  // this warp's MMAs (if any) have read the stage
          if (++s == NB) { s = 0; ph ^= 1u; }
#ifdef DST_ROLE_TIMERS
          ++n_it;
#endif
        }
        if (ok) umma_commit_elect(smem_u32(&bar_tfull[0]));
        ++tile;
      }
      if (who == 0u && lane == 0) {
        RT_ADD(8, RT_NOW() - t_begin); RT_ADD(9, w_tempty); RT_ADD(10, w_full); RT_ADD(11, n_it); RT_ADD(12, 1); RT_ADD(13, tile);
      }
    }
  } else if (warp < PF_CTRL_WARPS + (p.small ? 4 : PF_EPI_WARPS)) {
    // ------------------------------------------------------------------ epilogue: TMEM -> registers -> global
    const int r = (warp & 3) * 32 + lane;  // a warp may only read the TMEM lanes of its own quarter (warp id % 4)
    uint32_t tile = 0;
    const int epi_threads = 32 * (p.small ? 4 : PF_EPI_WARPS), epi_tid = tid - 32 * PF_CTRL_WARPS;
    for (int t = (int)blockIdx.x; t < n_tiles; t += t_step, ++tile) {
      tile_seek(p, offs, tpre, t, e, nt, row0, rows);
      const uint64_t* row_ptr = nullptr;
      if (p.row_target != nullptr) {
        // scatter form: while the tile is computed, look up where its token rows go (a global load and a pointer
        // per row, shared by the role's warps through shared memory; the buffer of the tile before stays intact for
        // warps still draining it, and nobody passes the barrier before all are done with the tile before that)
        uint64_t* rp = rowptr_s[tile & 1u];
        const size_t ostep = (size_t)p.N * 2;
        for (int j = epi_tid; j < rows; j += epi_threads) {
          const int64_t tg = p.row_target[row0 + j];
          const int64_t dr = tg & 0xFFFFFFFFFFFFLL;
          const bool ok = tg >= 0 && (tg >> 48) < p.n_peer_out && dr < p.peer_rows;  // nothing is stored outside the buffers
          rp[j] = ok ? (uint64_t)reinterpret_cast<uintptr_t>(pf_peer_out(p, (int)(tg >> 48))) + (uint64_t)dr * ostep : 0ull;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_epi));
        if (!mbar_wait(smem_u32(&bar_epi), tile & 1u, abort_flag)) break;
        __syncwarp();
        row_ptr = rp;
      }
      // the two warps of a lane quarter take alternate 32-column chunks
      const int col_first = ((warp - PF_CTRL_WARPS) >> 2) * 32, col_step = p.small ? 32 : 32 * (PF_EPI_WARPS / 4);
      if (p.wide_drain) {
        if (!drain_tile_wide(p, tmem, col_first, col_step, warp & 3, lane, smem_u32(&bar_tfull[0]), smem_u32(&bar_tempty[0]), abort_flag, nt,
                             row0, rows, tile, row_ptr, epi_tiles + (warp - PF_CTRL_WARPS) * PF_EPI_TILE))
          break;
      } else if (!drain_tile(p, tmem, col_first, col_step, r, smem_u32(&bar_tfull[0]), smem_u32(&bar_tempty[0]), abort_flag, nt, row0,
                             rows, tile, row_ptr)) {
        break;
      }
    }
  } else {
    // ------------------------------------------------------------------ dequant producers (weights)
    // A warp may only touch the TMEM lanes of its own quarter (warp id % 4): it owns those 32 weight rows.
    const int q = warp & 3;
    const int r = q * 32 + lane;
    // groups 0..3: warps 12..27; with small token tiles warps 8..11 (epilogue warps otherwise) are group 4
    const uint32_t n_groups = p.small ? PF_GROUPS + 1 : PF_GROUPS;
    const uint32_t grp = warp >= PF_DQ_WARP0 ? (uint32_t)(warp - PF_DQ_WARP0) >> 2 : (uint32_t)PF_GROUPS;
    const int swz = (r >> 1) & 3;  // swizzle of the tiled layout: logical word w sits at physical word (((w & 3) ^ swz) << 2) | (w >> 2)
    const uint32_t lut_addr = smem_u32(lut) + (uint32_t)(lane & 15) * 4u;
    const uint32_t lane_base = (uint32_t)(q * 32) << 16;
    const bool vec_scales = (p.G & 7) == 0;  // rows of 8 k scales are 16-byte aligned
    const int kstages = p.kstages;
    uint32_t own = grp;  // global index (counted over all tiles of this CTA) of this group's next stage
    uint32_t s = grp % NB, ph = (grp / NB) & 1u;
    uint32_t it0 = 0, gs0 = 0;  // first stage / first slab of the current tile
    bool ok = true;
    RT_DECL(w_pfull = 0, w_dempty = 0, w_drain = 0, w_comp = 0, w_st = 0, w_pre = 0, n_it = 0, t_begin = RT_NOW(), w_lds = 0, w_tail = 0, t_tail = RT_NOW());

    // scales of the row: 8 groups (16 stages) per 128-bit load; when a block of 8 is taken into use the tile's next block
    // is requested, so only a tile's first block is waited for (once per tile and warp; the per-stage cost is a compare)
    uint4 sc[TERMS], scn[TERMS];
    int cur_b = -1, nxt_b = -1;              // block of 8 groups held in sc / requested into scn, of the current tile
    const __half* srow[TERMS];               // the row's scales of the current tile (null: a row beyond N, scales read as 0)
    auto load_scales = [&](int g0, uint4* dst) {
#pragma unroll
      for (int i = 0; i < TERMS; ++i) {
        if (i < p.n_terms) {
          if (srow[i] == nullptr || g0 >= p.G) {
            dst[i] = make_uint4(0u, 0u, 0u, 0u);
          } else if (vec_scales) {
            dst[i] = *reinterpret_cast<const uint4*>(srow[i] + g0);
          } else {
            uint32_t h[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) h[j] = g0 + j < p.G ? (uint32_t)__half_as_ushort(srow[i][g0 + j]) : 0u;
            dst[i] = make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16), h[6] | (h[7] << 16));
          }
        }
      }
    };
    int t = (int)blockIdx.x - t_step;  // tile being dequantised; before the first one here
    bool in_tile = false;
    int n = 0;
    for (;;) {
      if (!(in_tile && (int32_t)(own - it0) < kstages)) {
        // past the end of the current tile (or before the first): look up the next one
        if (in_tile) {
          it0 += (uint32_t)kstages;
          gs0 += (uint32_t)nsb;
          in_tile = false;
        }
        if (t + t_step >= n_tiles) break;
        t += t_step;
        tile_seek(p, offs, tpre, t, e, nt, row0, rows);
        n = nt * 128 + r;
#pragma unroll
        for (int i = 0; i < TERMS; ++i)
          if (i < p.n_terms) srow[i] = n < p.N ? p.scale[i] + ((int64_t)e * p.N + n) * p.G : nullptr;
        cur_b = nxt_b = -1;
        in_tile = true;
        continue;
      }
      const int ks = (int)(own - it0);
        RT_DECL(t_pre = RT_NOW());
        RT_SPAN(w_tail, t_tail);
        const int sb = ks / SPB, sbk = ks - sb * SPB;
        const uint32_t gs = gs0 + (uint32_t)sb;
        const uint32_t slot = p.nslab == 2 ? (gs & 1u) : gs % 3u, sround = p.nslab == 2 ? (gs >> 1) : gs / 3u;
        // scales
        const int blk = ks >> 4;
        if (blk != cur_b) {
          if (nxt_b == blk) {
#pragma unroll
            for (int i = 0; i < TERMS; ++i) sc[i] = scn[i];
          } else {
            load_scales(blk * 8, sc);
          }
          cur_b = blk;
          if ((blk + 1) * 8 < p.G) {  // the tile's next block, needed a few of this warp's stages from now
            load_scales((blk + 1) * 8, scn);
            nxt_b = blk + 1;
          }
        }
        const int g = (ks >> 1) & 7;  // 64-trit stage -> 128-trit scale group, inside the 8 held in sc

        // packed words of this row for this stage, then the slab can go back to the producer
        RT_SPAN(w_pre, t_pre);
        if (!RT_WAIT(w_pfull, mbar_wait(smem_u32(&bar_pfull[slot]), sround & 1u, abort_flag))) { ok = false; break; }
        RT_DECL(t_lds = RT_NOW());
        uint32_t w[TERMS][4];
#pragma unroll
        for (int i = 0; i < TERMS; ++i) {
          if (i < p.n_terms) {
            const uint32_t* wp = reinterpret_cast<const uint32_t*>(slabs + ((size_t)slot * p.n_terms + i) * PF_SLAB + r * 64);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int lw = FMT == 2 ? 4 * sbk + j : (j < 3 ? 3 * sbk + j : 15);  // logical word of the row-superblock
              w[i][j] = wp[(((lw & 3) ^ swz) << 2) | (lw >> 2)];
            }
          }
        }
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(smem_u32(&bar_pempty[slot]));
          // the tile's last superblock may hold fewer than SPB stages: make up for the stages that do not exist
          if (ks == kstages - 1)
            for (int x = nsb * SPB - kstages; x > 0; --x) mbar_arrive(smem_u32(&bar_pempty[slot]));
        }

#ifdef DST_ROLE_TIMERS
#pragma unroll
        for (int i = 0; i < TERMS; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) asm volatile("" : "+r"(w[i][j]));
#endif
        RT_SPAN(w_lds, t_lds);
        RT_DECL(t_c = RT_NOW());
        __half2 acc[32];
#pragma unroll
        for (int i = 0; i < TERMS; ++i) {
          if (i < p.n_terms) {
            const __half2 s2 = pick_scale(sc[i], g);
            if (FMT == 2) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (i == 0) tq2_word<true>(w[i][j], s2, acc + 8 * j);
                else tq2_word<false>(w[i][j], s2, acc + 8 * j);
              }
            } else {
              if (i == 0) tq1_stage<true>(w[i], sbk, lut_addr, s2, acc);
              else tq1_stage<false>(w[i], sbk, lut_addr, s2, acc);
            }
          }
        }
        uint32_t v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = h2_bits(acc[j]);
#ifdef DST_ROLE_TIMERS
#pragma unroll
        for (int j = 0; j < 32; ++j) asm volatile("" : "+r"(v[j]));
        RT_SPAN(w_comp, t_c);
        ++n_it;
#endif
        // the A slot must be free (the MMAs that last read it are done) before the store into it
        // no sleep between polls here: these warps are the critical path, and a sleeping lane wakes up to a
        // microsecond late (the whole warp then waits for it at the next convergence point)
        if (!RT_WAIT(w_dempty, mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, abort_flag))) { ok = false; break; }
        __syncwarp();  // re-converge after the polling loop: tcgen05.st is .sync.aligned
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t taddr = tmem + lane_base + (uint32_t)p.tn_max + s * PF_A_COLS;
        RT_DECL(t_st = RT_NOW());
        tmem_st_8(taddr, v);
        tmem_st_8(taddr + 8, v + 8);
        tmem_st_8(taddr + 16, v + 16);
        tmem_st_8(taddr + 24, v + 24);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_full[s]));
        RT_SPAN(w_st, t_st);
#ifdef DST_ROLE_TIMERS
        t_tail = RT_NOW();
#endif
        own += n_groups;
        s += n_groups;
        while (s >= NB) { s -= NB; ph ^= 1u; }
    }
    if (warp == PF_DQ_WARP0 && lane == 0) {
      RT_ADD(24, RT_NOW() - t_begin); RT_ADD(25, w_pfull); RT_ADD(26, w_dempty); RT_ADD(27, n_it); RT_ADD(28, 1);
      RT_ADD(29, w_drain); RT_ADD(30, w_comp); RT_ADD(31, w_st); RT_ADD(32, w_pre); RT_ADD(33, w_lds); RT_ADD(34, w_tail);
    }
  }

  // ------------------------------------------------------------------ teardown
  if (*abort_flag) {
    // give copies and MMAs still in flight time to land before shared memory and TMEM are released
    const long long t0 = clock64();
    while (clock64() - t0 < 4000000LL) __nanosleep(1000);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512));
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

template <int FMT, int TERMS>
int launch_fmt(const TmaMaps& maps, PrefillParams p, cudaStream_t st) {
  // Shared-memory and TMEM plan: the token tile is as large as the experts are expected to need (up to 320 rows) as
  // long as a stage ring of depth 4 fits; smaller tiles leave room for a deeper ring (each B stage is tn_max * 128
  // bytes, each A slot 32 TMEM columns next to tn_max accumulator columns), which is what hides the TMA latency
  // when the MMAs of a stage are short. Then a third packed-slab slot if there is room for it.
  const long long budget = PF_SMEM_MAX - PF_SMEM_STATIC;
  const long long fixed = 1024 + (FMT == 1 ? PF_LUT_BYTES : 0) + 2 * (PF_MAX_E + 1) * 4 + (p.wide_drain ? 128 + PF_EPI_WARPS * PF_EPI_TILE : 0);
  const long long slab2 = 2LL * p.n_terms * PF_SLAB;
  int tn_cap = (p.rows_hint + 31) / 32 * 32;
  tn_cap = tn_cap < 64 ? 64 : (tn_cap > PF_TN_MAX ? PF_TN_MAX : tn_cap);
  p.tn_max = 0;
  for (int tn = tn_cap; tn >= 64; tn -= 32) {
    long long nb = (budget - fixed - slab2) / (tn * 128LL);
    if (nb >= 4 || tn == 64) {
      const long long tmem_fit = (512 - tn) / PF_A_COLS;
      nb = nb > tmem_fit ? tmem_fit : nb;
      p.tn_max = tn;
      p.nb = (int)(nb > PF_MAX_STAGES ? PF_MAX_STAGES : nb);
      break;
    }
  }
  if (p.tn_max == 0 || p.nb < 2) return DST_ERR_UNSUPPORTED;
  p.nslab = fixed + 3LL * p.n_terms * PF_SLAB + (long long)p.nb * p.tn_max * 128 <= budget ? 3 : 2;
  p.small = p.tn_max <= 128 ? 1 : 0;
  const size_t smem = (size_t)(fixed + (long long)p.nslab * p.n_terms * PF_SLAB + (long long)p.nb * p.tn_max * 128);
  auto kernel = prefill_kernel<FMT, TERMS>;
  DST_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int dev = 0, sms = 148;
  DST_CUDA_TRY(cudaGetDevice(&dev));
  DST_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  // persistent CTAs, one per SM, fewer when there cannot be that many tiles
  long long tiles_upper = ((long long)cdiv64(p.T, p.tn_max) + p.E) * p.NT;
  if (tiles_upper >= (1LL << 30)) return DST_ERR_UNSUPPORTED;  // tile indices are 32-bit in the kernel
  if (tiles_upper < 1) tiles_upper = 1;
  unsigned grid = (unsigned)(tiles_upper < sms ? tiles_upper : sms);
  if (g_debug_max_ctas > 0 && grid > (unsigned)g_debug_max_ctas) grid = (unsigned)g_debug_max_ctas;
  prefill_kernel<FMT, TERMS><<<grid, PF_THREADS, smem, st>>>(maps, p);
  DST_CUDA_TRY(cudaGetLastError());
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
          ((a.act_dtype == DST_ACT_BF16 || a.act_dtype == DST_ACT_F16 || a.act_dtype == DST_ACT_I8) && a.workspace != nullptr &&
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
  else if (a.act_dtype == DST_ACT_I8)
    // the int8-activation contract (per-token absmax quantisation, row_scale = the token's scale): int8 values are
    // exact in fp16, scale * trit is exact in fp16, every product is exact in fp32; only the fp32 accumulation
    // order differs from the reference's integer group sums (relative difference ~1e-6)
    convert_rows_kernel<int8_t><<<(unsigned)a.T, 256, 0, stream>>>(static_cast<const int8_t*>(a.x), a.K, a.row_scale,
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
  p.row_target = a.row_target;
  for (int i = 0; i < DST_MAX_PEERS; ++i) p.peer_out[i] = a.peer_out[i];
  p.n_peer_out = a.n_peer_out;
  p.peer_rows = a.peer_rows;
  // 128-bit stores from the epilogue: two-byte outputs, whole 8-column pieces, 16-byte aligned rows
  p.wide_drain = (a.out_dtype != DST_OUT_F32 && !a.accumulate && a.N % 8 == 0 && (reinterpret_cast<uintptr_t>(a.out) & 15) == 0) ? 1 : 0;
  if (a.row_target != nullptr)
    for (int i = 0; i < DST_MAX_PEERS; ++i)
      if ((reinterpret_cast<uintptr_t>(a.peer_out[i]) & 15) != 0) p.wide_drain = 0;
  if (a.row_target != nullptr && (a.out_dtype == DST_OUT_F32 || a.accumulate)) return DST_ERR_UNSUPPORTED;
  p.E = (int)a.E;
  p.T = (int)a.T;
  p.N = (int)a.N;
  p.K = (int)a.K;
  p.G = (int)a.G;
  p.NT = (int)cdiv64(a.N, 128);
  p.S = (int)tiled_superblocks(a.fmt, a.K);
  p.kstages = (int)(a.K / 64);
  // rows per expert: known when the caller passed host offsets, else assumed below twice the mean
  p.rows_hint = (int)(a.max_rows >= 0 ? a.max_rows : 2 * cdiv64(a.T, a.E));
  if (p.rows_hint < 1) p.rows_hint = 1;
#define DST_PF_LAUNCH(FMT_)                                                            \
  (a.terms.n == 1 ? launch_fmt<FMT_, 1>(maps, p, stream)                               \
                  : a.terms.n == 2 ? launch_fmt<FMT_, 2>(maps, p, stream) : launch_fmt<FMT_, 4>(maps, p, stream))
  // The kernel keeps per-expert tables in shared memory: more experts than fit there are served by one launch
  // per run of PF_MAX_E experts (offsets are absolute token rows, so only the per-expert pointers move).
  const int64_t tiled_per_expert = (int64_t)p.NT * p.S * PF_SLAB, scales_per_expert = a.N * a.G;
  for (int64_t e0 = 0; e0 < a.E; e0 += PF_MAX_E) {
    p.E = (int)(a.E - e0 < PF_MAX_E ? a.E - e0 : PF_MAX_E);
    p.offsets = a.offsets ? a.offsets + e0 : nullptr;
    for (int i = 0; i < a.terms.n; ++i) {
      p.tiled[i] = a.terms.packed[i] + e0 * tiled_per_expert;
      p.scale[i] = static_cast<const __half*>(a.terms.scale[i]) + e0 * scales_per_expert;
    }
    const int rc = a.fmt == DST_FMT_TQ2 ? DST_PF_LAUNCH(2) : DST_PF_LAUNCH(1);
    if (rc != DST_OK) return rc;
  }
  return DST_OK;
#undef DST_PF_LAUNCH
}

}  // namespace dst

#ifdef DST_ROLE_TIMERS
// Profiling builds only: copies (and optionally clears) the 64 role-timer slots. Slots: 0-5 producers (B producer
// total cycles, slab producer wait slot free, B producer wait stage free, stages, threads, slab producer total),
// 8-13 MMA issuer (total, wait accumulator free, wait stage full, stages, threads, tiles), 24-30 one dequant warp
// (total, wait packed slab, wait stage free, own stages, threads, accumulator drain, dequant arithmetic, TMEM store +
// arrive, scale bookkeeping before the slab wait), 33 its reads of the packed words + slab hand-back, 34 loop tail and
// head (tile lookup included). The clock reads themselves cost: a build with them runs ~20 % slower.
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

extern "C" int dst_debug_prefill_timeout(long long wait_cycles, int drop_drain_arrivals, int max_ctas) {
  const long long cycles = wait_cycles > 0 ? wait_cycles : dst::PF_WAIT_CYCLES;
  const int drop = drop_drain_arrivals ? 1 : 0;
  DST_CUDA_TRY(cudaDeviceSynchronize());
  DST_CUDA_TRY(cudaMemcpyToSymbol(dst::g_wait_cycles, &cycles, sizeof(cycles)));
  DST_CUDA_TRY(cudaMemcpyToSymbol(dst::g_drop_drain_arrivals, &drop, sizeof(drop)));
  dst::g_debug_max_ctas = max_ctas > 0 ? max_ctas : 0;
  return DST_OK;
}

extern "C" int dst_check_device_status(dst_stream_t stream) {
  DST_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  int st = 0;
  DST_CUDA_TRY(cudaMemcpyFromSymbol(&st, dst::g_device_status, sizeof(int)));
  if (st != 0) {
    const int zero = 0;
    DST_CUDA_TRY(cudaMemcpyToSymbol(dst::g_device_status, &zero, sizeof(int)));
  }
  int st_decode = 0;  // the decode kernel keeps a status word of its own
  const int rc = dst::decode_take_status(&st_decode);
  if (rc != DST_OK) return rc;
  int st_ep = 0;  // and so does the expert-parallel barrier
  const int rc2 = dst::ep_take_status(&st_ep);
  if (rc2 != DST_OK) return rc2;
  return (st != 0 || st_decode != 0 || st_ep != 0) ? DST_ERR_TIMEOUT : DST_OK;
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
