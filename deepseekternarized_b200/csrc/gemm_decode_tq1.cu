// Decode GEMV / grouped GEMV for TQ1 (5 trits per byte) weights and few token rows per expert.
//
//     out[m, n] = row_scale[m] * sum_i sum_g scale_i[e, n, g] * sum_{k in g} x[m, k] * trit_i[e, n, k]
//
// Same scheme as the TQ2 decode kernel (gemm_decode.cu): mma.sync.m16n8k16 fed from registers, the A operand is
// a word of 2-bit digit fields ANDed with a field mask (the fp16 denormal u * 4^f * 2^-24, exact on this
// hardware), the token rows are staged once per expert in shared memory pre-scaled by 4^-f, and the per-(token,
// group) sums of x remove the u = t + 1 offset. What TQ1 adds:
//
//   bytes -> fields   a shared-memory table (the entries the tcgen05 kernel uses, gemm_prefill.cu) maps a byte
//                     to its five digits as 2-bit fields, placed for both positions a byte can take in a pair of
//                     bytes; one AND-OR merges two entries into a word of five (even, odd) trit pairs, and five
//                     ANDs give five A registers. Per byte: one table read and ~4.5 integer instructions, which
//                     is what bounds this kernel (the packed bytes of a TQ1 stream carry 25 % more trits than
//                     TQ2's and every trit pair costs one instruction more than there).
//   groups            a 64-byte row-superblock of the tiled layout (layout_kernels.cu) is five 64-trit stages =
//                     2.5 scale groups, and the lane that holds words c, 4+c, 8+c, 12+c of a row (one 128-bit
//                     load) holds stages of different groups. Every MMA accumulates ONE group: the four lanes of
//                     a row take part in a "set" of five MMAs only if their word of that step belongs to the
//                     set's group; the others multiply by ZERO activations, which the staging code writes into
//                     their slots, so the selection costs no instruction. Superblocks are processed in pairs
//                     (five whole groups); three fp32 accumulators per superblock, the middle group of a pair is
//                     carried from the even to the odd superblock.
//   bytes 60..63      of a row-superblock hold one trit of each of the five stages (digit s = stage s); lane 3
//                     owns them and feeds them through extra sets with single-digit masks.
//
// One warp owns 16 weight rows of a 128-row tile; a CTA of 16 warps works on two neighbouring row tiles of one
// expert at a time, so 8 staged token rows (up to ~17 KB each for K = 4096: the slots are laid out in the order
// the lanes consume them, zeros included) serve 256 weight rows. Up to 8 token rows per pass; an expert with
// more rows is processed in several passes (the weights are re-read, from L2).
//
// Coverage: TQ1 tiled weights, group 128, K % 128 == 0, fp16 scales, bf16 or fp16 activations.
#include "dst_common.cuh"

namespace dst {
namespace {

constexpr int D1_WARPS = 16;
constexpr int D1_THREADS = D1_WARPS * 32;
constexpr int D1_MT = 8;                       // token rows staged per pass
constexpr int D1_LUT_BYTES = 256 * 32 * 4;     // 256 byte values x 32 bank replicas x 4 B: every lane reads its own bank
constexpr int D1_EVEN_REGS = 5 * 48 + 3 * 16;  // 32-bit activation slots of an even superblock, per token
constexpr int D1_ODD_REGS = 6 * 48 + 16 + 32 + 32;
constexpr uint32_t D1_FIRST_MASK = 0x000F003Fu, D1_SECOND_MASK = 0x03F003C0u;

struct Decode1Params {
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
  int xstride;  // bytes between staged token rows (= 64 mod 128: conflict-free 128-bit reads of two token rows)
};

__host__ __device__ inline int d1_sb_offset(int sb) { return (sb >> 1) * (D1_EVEN_REGS + D1_ODD_REGS) + (sb & 1) * D1_EVEN_REGS; }
__host__ __device__ inline int d1_token_regs(int S) { return d1_sb_offset(S); }

__host__ __device__ inline uint32_t d1_table_entry(uint32_t byte) {
  const uint32_t f = tq1_fields(byte);
  const uint32_t d0 = f & 3u, d1 = (f >> 2) & 3u, d2 = (f >> 4) & 3u, d3 = (f >> 6) & 3u, d4 = (f >> 8) & 3u;
  return (d0 | (d2 << 2) | (d4 << 4) | (d1 << 16) | (d3 << 18)) | ((d0 << 20) | (d1 << 6) | (d2 << 22) | (d3 << 8) | (d4 << 24));
}

__device__ __forceinline__ void mma_f16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ------------------------------------------------------------------------------------------ slot map
// Scale group (0..2, relative to the superblock's first group) of stage s in a superblock of parity p.
__host__ __device__ inline int d1_rel_group(int p, int s) { return p == 0 ? s >> 1 : (s + 1) >> 1; }
// Field (0..4) of trit j (0..63) of a stage: the position of its pair in the merged word of its two bytes, or
// (j >= 60) the field of the shared byte's digit for stage s.
__host__ __device__ inline int d1_trit_field(int s, int j) {
  if (j >= 60) return s >> 1;
  const int b = j / 5, u = 5 * (b & 1) + j % 5;
  return u >> 1;
}

// Activation slot r (0 .. regs of a superblock of parity p) -> the trits of the superblock (0..319, -1 = none)
// that its low and high fp16 multiply, and their field. The order is the order in which lane c consumes slots:
// regular set q: 48 slots = 4 lanes x 12 (10 used: MMA i takes slots 2i, 2i + 1); then the shared-byte sets.
__host__ __device__ inline void d1_slot(int p, int r, int& klo, int& khi, int& f) {
  klo = khi = -1;
  f = 0;
  const int nreg = p == 0 ? 240 : 288;
  if (r < nreg) {
    const int q = r / 48, rem = r % 48, c = rem / 12, t = rem % 12;
    if (t >= 10) return;
    int j, a;
    if (p == 0) {  // sets (step, group): (0,0) (1,0) (1,1) (2,1) (3,2)
      j = q == 0 ? 0 : q <= 2 ? 1 : q == 3 ? 2 : 3;
      a = q <= 1 ? 0 : q <= 3 ? 1 : 2;
    } else {  // (0,0) (0,1) (1,1) (2,1) (2,2) (3,2)
      j = q <= 1 ? 0 : q == 2 ? 1 : q <= 4 ? 2 : 3;
      a = q == 0 ? 0 : q <= 3 ? 1 : 2;
    }
    const int w = 4 * j + c;
    if (w == 15) return;
    const int s = w / 3;
    if (d1_rel_group(p, s) != a) return;  // this lane's word belongs to another group: its slots stay zero
    f = t % 5;
    klo = 64 * s + 10 * (2 * (w % 3) + t / 5) + 2 * f;
    khi = klo + 1;
    return;
  }
  r -= nreg;
  if (p == 0) {  // three sets of 4 lanes x 4 slots: digits (2a, 2a + 1) of byte 60 + m, field a
    const int a = r / 16, c = (r % 16) / 4, m = r % 4;
    if (c != 3) return;
    f = a;
    klo = 64 * (2 * a) + 60 + m;
    if (2 * a + 1 <= 4) khi = 64 * (2 * a + 1) + 60 + m;
    return;
  }
  // odd superblock: single digits. group 0: digit 0; group 1: digits 1, 2; group 2: digits 3, 4
  if (r < 16) {
    const int c = r / 4, m = r % 4;
    if (c != 3) return;
    klo = 60 + m;
    return;
  }
  r -= 16;
  const int a = r / 32, c = (r % 32) / 8, t = r % 8, m = t >> 1;
  if (c != 3) return;
  if (a == 0) {  // group 1
    if (t & 1) { f = 1; klo = 64 * 2 + 60 + m; } else { f = 0; khi = 64 * 1 + 60 + m; }
  } else {  // group 2
    if (t & 1) { f = 2; klo = 64 * 4 + 60 + m; } else { f = 1; khi = 64 * 3 + 60 + m; }
  }
}

// ------------------------------------------------------------------------------------------ staging
// Token rows [m0, m0 + mc) of x -> shared memory, in slot order:
//   slot value = fp16( x[m][k] * 2^(7 - e_m - 2 f) ),  e_m = floor(log2(rowmax)) - 7
//   xsum[m][g] = sum over group g of the values the tensor core will see, undone to x * 2^-e_m
//   xexp[m]    = 2^e_m * row_scale[m]
template <typename XT>
__device__ void d1_stage_tokens(const Decode1Params& p, const XT* __restrict__ x, int64_t m0, int mc, uint8_t* xs, float* xsum,
                                float* xexp, int* xex) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int regs = d1_token_regs(p.S);
  // pass 1, one warp per token row: the row's power of two. Token slots beyond mc are never read (their B
  // fragments are zero registers), so nothing is written for them.
  for (int m = warp; m < mc; m += D1_WARPS) {
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
  // pass 2, one warp per (token row, group): group sums in natural k order, 32 lanes x 4 consecutive k
  for (int u = warp; u < mc * p.G; u += D1_WARPS) {
    const int m = u / p.G, g = u - m * p.G;
    const XT* row = x + (m0 + m) * p.K;
    const int ex = xex[m];
    float part = 0.f;
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      const int k = g * 128 + lane * 4 + h;
      const int f = d1_trit_field((k % 320) >> 6, k & 63);
      const __half v = __float2half_rn((float)row[k] * ldexpf(1.f, 7 - ex - 2 * f));
      part += __half2float(v) * ldexpf(1.f, 2 * f - 7);
    }
    for (int off = 16; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
    if (lane == 0) xsum[m * p.G + g] = part;
  }
  // pass 3, one thread per slot: the rows in consumption order (zeros where a lane sits out a set)
  for (int idx = threadIdx.x; idx < mc * regs; idx += D1_THREADS) {
    const int m = idx / regs, r = idx - m * regs;
    const XT* row = x + (m0 + m) * p.K;
    const int pair = r / (D1_EVEN_REGS + D1_ODD_REGS), rr = r - pair * (D1_EVEN_REGS + D1_ODD_REGS);
    const int par = rr >= D1_EVEN_REGS ? 1 : 0, sb = 2 * pair + par;
    int klo, khi, f;
    d1_slot(par, par ? rr - D1_EVEN_REGS : rr, klo, khi, f);
    const float mul = ldexpf(1.f, 7 - xex[m] - 2 * f);
    uint32_t lo = 0u, hi = 0u;
    if (klo >= 0 && sb * 320 + klo < p.K) lo = __half_as_ushort(__float2half_rn((float)row[sb * 320 + klo] * mul));
    if (khi >= 0 && sb * 320 + khi < p.K) hi = __half_as_ushort(__float2half_rn((float)row[sb * 320 + khi] * mul));
    reinterpret_cast<uint32_t*>(xs + (size_t)m * p.xstride)[r] = lo | (hi << 16);
  }
}

// ------------------------------------------------------------------------------------------ the kernel
__device__ __forceinline__ uint32_t d1_lookup(uint32_t lut_addr, uint32_t word, int byte) {
  const uint32_t idx = byte == 0 ? (word << 7) & 0x7F80u : (word >> (8 * byte - 7)) & 0x7F80u;  // byte value * 128
  uint32_t v;
  asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(lut_addr + idx));
  return v;
}

// The ten A registers of a regular word (bytes b0 b1 | b2 b3 -> two merged words of five trit pairs each).
__device__ __forceinline__ void d1_word_regs(uint32_t word, uint32_t lut_addr, uint32_t* a /* 10 */) {
  const uint32_t c0 = d1_lookup(lut_addr, word, 0), c1 = d1_lookup(lut_addr, word, 1);
  const uint32_t c2 = d1_lookup(lut_addr, word, 2), c3 = d1_lookup(lut_addr, word, 3);
  const uint32_t m01 = (c0 & D1_FIRST_MASK) | (c1 & D1_SECOND_MASK), m23 = (c2 & D1_FIRST_MASK) | (c3 & D1_SECOND_MASK);
#pragma unroll
  for (int f = 0; f < 5; ++f) {
    a[f] = m01 & (0x00030003u << (2 * f));
    a[5 + f] = m23 & (0x00030003u << (2 * f));
  }
}

// One regular set: five MMAs of this lane's ten A registers (two weight rows) against its twelve-slot block.
// live: this lane's token column exists; the others feed zero registers and cause no shared-memory traffic.
__device__ __forceinline__ void d1_set(float* acc, const uint32_t* al, const uint32_t* ah, const uint8_t* xblock, bool live) {
  uint4 b0 = make_uint4(0u, 0u, 0u, 0u), b1 = b0;
  uint2 b2 = make_uint2(0u, 0u);
  if (live) {
    b0 = *reinterpret_cast<const uint4*>(xblock);
    b1 = *reinterpret_cast<const uint4*>(xblock + 16);
    b2 = *reinterpret_cast<const uint2*>(xblock + 32);
  }
  mma_f16(acc, al[0], ah[0], al[1], ah[1], b0.x, b0.y);
  mma_f16(acc, al[2], ah[2], al[3], ah[3], b0.z, b0.w);
  mma_f16(acc, al[4], ah[4], al[5], ah[5], b1.x, b1.y);
  mma_f16(acc, al[6], ah[6], al[7], ah[7], b1.z, b1.w);
  mma_f16(acc, al[8], ah[8], al[9], ah[9], b2.x, b2.y);
}

// One superblock of parity P: four steps over the lane's four words, then the shared-byte sets.
// xsb: this token row's slots of the superblock, already offset by the lane's quad position (c * 48 bytes for
// the regular sets is added here, as are the shared sets' offsets).
template <int P>
__device__ __forceinline__ void d1_superblock(const uint4& wl4, const uint4& wh4, const uint8_t* xsb, int c, bool live,
                                              uint32_t lut_addr, float (&acc)[3][4]) {
  const uint32_t wl[4] = {wl4.x, wl4.y, wl4.z, wl4.w}, wh[4] = {wh4.x, wh4.y, wh4.z, wh4.w};
  const uint8_t* xreg = xsb + c * 48;
  int q = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t al[10], ah[10];
    d1_word_regs(wl[j], lut_addr, al);
    d1_word_regs(wh[j], lut_addr, ah);
    // groups that the four lanes' words of this step belong to (compile-time, see d1_slot)
    const int a_first = P == 0 ? (j == 0 ? 0 : j == 1 ? 0 : j == 2 ? 1 : 2) : (j == 0 ? 0 : j == 1 ? 1 : j == 2 ? 1 : 2);
    const bool two = P == 0 ? j == 1 : (j == 0 || j == 2);
    d1_set(acc[a_first], al, ah, xreg + q * 192, live);
    ++q;
    if (two) {
      d1_set(acc[a_first + 1], al, ah, xreg + q * 192, live);
      ++q;
    }
  }
  // bytes 60..63 (word 15, held by quad lane 3; the other lanes run the same code against zero activations)
  const uint32_t sl[4] = {d1_lookup(lut_addr, wl[3], 0), d1_lookup(lut_addr, wl[3], 1), d1_lookup(lut_addr, wl[3], 2), d1_lookup(lut_addr, wl[3], 3)};
  const uint32_t sh[4] = {d1_lookup(lut_addr, wh[3], 0), d1_lookup(lut_addr, wh[3], 1), d1_lookup(lut_addr, wh[3], 2), d1_lookup(lut_addr, wh[3], 3)};
  if (P == 0) {
    const uint8_t* xsh = xsb + 240 * 4 + c * 16;
#pragma unroll
    for (int a = 0; a < 3; ++a) {
      const uint32_t mask = a == 0 ? 0x00030003u : a == 1 ? 0x000C000Cu : 0x00000030u;  // digits (2a, 2a+1) of a "first byte" entry
      const uint4 b = live ? *reinterpret_cast<const uint4*>(xsh + a * 64) : make_uint4(0u, 0u, 0u, 0u);
      mma_f16(acc[a], sl[0] & mask, sh[0] & mask, sl[1] & mask, sh[1] & mask, b.x, b.y);
      mma_f16(acc[a], sl[2] & mask, sh[2] & mask, sl[3] & mask, sh[3] & mask, b.z, b.w);
    }
  } else {
    // digit masks of a "first byte" entry: d0 0x3, d1 0x30000, d2 0xC, d3 0xC0000, d4 0x30
    const uint8_t* x0 = xsb + 288 * 4 + c * 16;
    {
      const uint4 b = live ? *reinterpret_cast<const uint4*>(x0) : make_uint4(0u, 0u, 0u, 0u);
      mma_f16(acc[0], sl[0] & 0x3u, sh[0] & 0x3u, sl[1] & 0x3u, sh[1] & 0x3u, b.x, b.y);
      mma_f16(acc[0], sl[2] & 0x3u, sh[2] & 0x3u, sl[3] & 0x3u, sh[3] & 0x3u, b.z, b.w);
    }
#pragma unroll
    for (int a = 0; a < 2; ++a) {  // group 1: digits 1, 2; group 2: digits 3, 4 (slot t: byte t >> 1, first or second digit)
      const uint32_t me = a == 0 ? 0x00030000u : 0x000C0000u, mo = a == 0 ? 0x0000000Cu : 0x00000030u;
      const uint8_t* xa = xsb + (288 + 16) * 4 + a * 128 + c * 32;
      const uint4 b0 = live ? *reinterpret_cast<const uint4*>(xa) : make_uint4(0u, 0u, 0u, 0u);
      const uint4 b1 = live ? *reinterpret_cast<const uint4*>(xa + 16) : make_uint4(0u, 0u, 0u, 0u);
      mma_f16(acc[1 + a], sl[0] & me, sh[0] & me, sl[0] & mo, sh[0] & mo, b0.x, b0.y);
      mma_f16(acc[1 + a], sl[1] & me, sh[1] & me, sl[1] & mo, sh[1] & mo, b0.z, b0.w);
      mma_f16(acc[1 + a], sl[2] & me, sh[2] & me, sl[2] & mo, sh[2] & mo, b1.x, b1.y);
      mma_f16(acc[1 + a], sl[3] & me, sh[3] & me, sl[3] & mo, sh[3] & mo, b1.z, b1.w);
    }
  }
}

__global__ void __launch_bounds__(D1_THREADS)
decode_tq1_kernel(const Decode1Params p) {
  extern __shared__ __align__(16) uint8_t dsm[];
  uint8_t* lut = dsm;                                                            // digit-field table
  uint8_t* xs = dsm + D1_LUT_BYTES;                                              // D1_MT staged token rows
  float* xsum = reinterpret_cast<float*>(xs + (size_t)D1_MT * p.xstride);        // [D1_MT][G]
  float* xexp = xsum + D1_MT * p.G;                                              // [D1_MT]
  int* xex = reinterpret_cast<int*>(xexp + D1_MT);                               // [D1_MT] exponent of the row's power of two
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g8 = lane >> 2, c = lane & 3;
  {
    uint32_t* lut32 = reinterpret_cast<uint32_t*>(lut);  // [byte value][replica]
    for (int i = threadIdx.x; i < 256 * 32; i += D1_THREADS) lut32[i] = d1_table_entry((uint32_t)i >> 5);
  }
  const uint32_t lut_addr = (uint32_t)__cvta_generic_to_shared(lut) + (uint32_t)lane * 4u;

  // work items: (expert, pair of neighbouring 128-row tiles); a contiguous range per CTA
  const int NTP = (p.NT + 1) >> 1;
  const long long items = (long long)p.E * NTP;
  const long long per = (items + gridDim.x - 1) / gridDim.x;
  const long long i0 = (long long)blockIdx.x * per, i1 = i0 + per < items ? i0 + per : items;
  int staged_e = -1;
  int64_t staged_m0 = -1;

  for (long long item = i0; item < i1; ++item) {
    const int e = (int)(item / NTP), ntp = (int)(item - (long long)e * NTP);
    const int nt = ntp * 2 + (warp >> 3);  // warps 0-7: first tile of the pair, warps 8-15: second
    int64_t ra, rb;
    row_range(p.offsets, e, p.T, ra, rb);
    for (int64_t m0 = ra; m0 < rb; m0 += D1_MT) {
      const int mc = (int)(rb - m0 < D1_MT ? rb - m0 : D1_MT);
      if (staged_e != e || staged_m0 != m0) {
        __syncthreads();  // everyone is done with the previous rows (and the table is written)
        if (p.act_dtype == DST_ACT_BF16) d1_stage_tokens(p, static_cast<const __nv_bfloat16*>(p.x), m0, mc, xs, xsum, xexp, xex);
        else d1_stage_tokens(p, static_cast<const __half*>(p.x), m0, mc, xs, xsum, xexp, xex);
        __syncthreads();
        staged_e = e;
        staged_m0 = m0;
      }
      if (nt >= p.NT) continue;  // odd number of row tiles: the second half of the CTA idles on the last pair
      const int r0 = (warp & 7) * 16 + g8;  // this lane's rows inside the tile: r0 and r0 + 8 (same swizzle)
      const int swz = (r0 >> 1) & 3;
      const int n_lo = nt * 128 + r0, n_hi = n_lo + 8;
      const uint8_t* xtok = xs + (size_t)g8 * p.xstride;  // the token column this lane feeds (B fragment column g8)
      const bool live = g8 < mc;
      float y[4] = {0.f, 0.f, 0.f, 0.f};

      auto flush = [&](const float* acc, int grp, float sl, float sh) {
        // group done: y += scale[row][grp] * (2^17 acc - sum_k x); C fragment = (row r0 | r0 + 8) x (token 2c | 2c + 1)
        if (grp < p.G) {
          const float x0 = xsum[(2 * c) * p.G + grp], x1 = xsum[(2 * c + 1) * p.G + grp];
          y[0] = fmaf(sl, fmaf(acc[0], 131072.f, -x0), y[0]);
          y[1] = fmaf(sl, fmaf(acc[1], 131072.f, -x1), y[1]);
          y[2] = fmaf(sh, fmaf(acc[2], 131072.f, -x0), y[2]);
          y[3] = fmaf(sh, fmaf(acc[3], 131072.f, -x1), y[3]);
        }
      };

      for (int term = 0; term < p.n_terms; ++term) {
        const uint8_t* wbase = p.tiled[term] + (((int64_t)e * p.NT + nt) * p.S) * 8192 + ((c ^ swz) << 4);
        const __half* s_lo = p.scale[term] + ((int64_t)e * p.N + (n_lo < p.N ? n_lo : 0)) * p.G;
        const __half* s_hi = p.scale[term] + ((int64_t)e * p.N + (n_hi < p.N ? n_hi : 0)) * p.G;
        // words c, 4 + c, 8 + c, 12 + c of rows r0 and r0 + 8, prefetched two superblocks ahead
        const uint8_t* wl_ptr = wbase + (size_t)r0 * 64;
        const uint8_t* wh_ptr = wbase + (size_t)(r0 + 8) * 64;
        const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
        auto ldw = [&](const uint8_t* ptr, int sb) { return sb < p.S ? *reinterpret_cast<const uint4*>(ptr + (size_t)sb * 8192) : zero4; };
        uint4 l0 = ldw(wl_ptr, 0), h0 = ldw(wh_ptr, 0), l1 = ldw(wl_ptr, 1), h1 = ldw(wh_ptr, 1);
        for (int sb = 0; sb < p.S; sb += 2) {
          const uint4 cl0 = l0, ch0 = h0, cl1 = l1, ch1 = h1;
          l0 = ldw(wl_ptr, sb + 2);
          h0 = ldw(wh_ptr, sb + 2);
          l1 = ldw(wl_ptr, sb + 3);
          h1 = ldw(wh_ptr, sb + 3);
          // the five groups of this pair of superblocks: their scales for both rows, requested before the MMAs
          const int gb = (5 * sb) >> 1;
          float sl[5], sh[5];
#pragma unroll
          for (int i = 0; i < 5; ++i) {
            sl[i] = gb + i < p.G ? __half2float(s_lo[gb + i]) : 0.f;
            sh[i] = gb + i < p.G ? __half2float(s_hi[gb + i]) : 0.f;
          }
          float acc[3][4];
#pragma unroll
          for (int a = 0; a < 3; ++a)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[a][i] = 0.f;
          d1_superblock<0>(cl0, ch0, xtok + (size_t)d1_sb_offset(sb) * 4, c, live, lut_addr, acc);
          flush(acc[0], gb, sl[0], sh[0]);
          flush(acc[1], gb + 1, sl[1], sh[1]);
#pragma unroll
          for (int i = 0; i < 4; ++i) {  // the third group continues in the odd superblock
            acc[0][i] = acc[2][i];
            acc[1][i] = 0.f;
            acc[2][i] = 0.f;
          }
          if (sb + 1 < p.S) d1_superblock<1>(cl1, ch1, xtok + (size_t)d1_sb_offset(sb + 1) * 4, c, live, lut_addr, acc);
          flush(acc[0], gb + 2, sl[2], sh[2]);
          flush(acc[1], gb + 3, sl[3], sh[3]);
          flush(acc[2], gb + 4, sl[4], sh[4]);
        }
      }
      // store: rows n_lo / n_hi, tokens m0 + 2c (+1)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int tok = 2 * c + (i & 1);
        const int n = i < 2 ? n_lo : n_hi;
        if (tok < mc && n < p.N) {
          const float v = y[i] * xexp[tok];
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

int d1_xstride(int S) {
  int bytes = d1_token_regs(S) * 4;
  while (bytes % 128 != 64) bytes += 16;
  return bytes;
}

size_t d1_smem(int S, int G) { return (size_t)D1_LUT_BYTES + (size_t)D1_MT * d1_xstride(S) + (size_t)D1_MT * (G + 2) * 4; }

}  // namespace

bool decode_tq1_supports(const GemmArgs& a) {
  return a.weight_layout == DST_LAYOUT_TILED && a.fmt == DST_FMT_TQ1 && a.group == 128 && a.K % 128 == 0 &&
         a.scale_dtype == DST_SCALE_F16 && (a.act_dtype == DST_ACT_BF16 || a.act_dtype == DST_ACT_F16) &&
         d1_smem((int)tiled_superblocks(a.fmt, a.K), (int)a.G) <= 220 * 1024 && a.T < (int64_t(1) << 31);
}

int launch_decode_tq1(const GemmArgs& a, cudaStream_t stream) {
  if (a.T == 0 || a.N == 0 || a.E == 0) return DST_OK;
  if (!decode_tq1_supports(a)) return DST_ERR_UNSUPPORTED;
  for (int i = 0; i < a.terms.n; ++i)
    if ((reinterpret_cast<uintptr_t>(a.terms.packed[i]) & 15) != 0 || (reinterpret_cast<uintptr_t>(a.terms.scale[i]) & 1) != 0)
      return DST_ERR_ALIGNMENT;
  Decode1Params p;
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
  p.xstride = d1_xstride(p.S);
  int dev = 0, sms = 148;
  DST_CUDA_TRY(cudaGetDevice(&dev));
  DST_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const long long items = (long long)p.E * ((p.NT + 1) >> 1);
  const size_t smem = d1_smem(p.S, p.G);
  int per_sm = (int)((220 * 1024) / (smem + 1024));
  per_sm = per_sm < 1 ? 1 : (per_sm > 2 ? 2 : per_sm);
  const long long want = (long long)sms * per_sm;
  const int grid = (int)(items < want ? items : want);
  DST_CUDA_TRY(cudaFuncSetAttribute(decode_tq1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  decode_tq1_kernel<<<grid, D1_THREADS, smem, stream>>>(p);
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}

}  // namespace dst
