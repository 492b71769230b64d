// Tiled device layout of packed ternary weights, built once when weights are placed on the GPU
// (the hook the reference has in TernaryLinear._on, boilerplate/ternary/ops.py:41-45).
//
// The canonical [N, ceil(K/per)] layout has rows of 820 B (TQ1, K = 4096) or 410 B (K = 2048): no row
// starts on a 16-byte boundary, and a 128-trit scale group is 25.6 B. The two fast kernels therefore
// read a byte permutation of it:
//
//   tiled[e][nt][sb][r][0..63]   nt = n / 128, r = n % 128, sb = superblock along K
//
// A superblock is 64 bytes of one row: 256 trits in TQ2, 320 trits in TQ1 (five 64-trit MMA stages).
// One (nt, sb) slab is 8 KB contiguous and 16-byte aligned, so a thread reads its row with 128-bit
// loads and a whole slab can be fetched with one bulk copy. Rows beyond N and trits beyond K are
// padding digits (t = 0). K is padded to whole superblocks: TQ1 K = 4096 -> 4160 trits (+1.6 %).
//
//   TQ1: the 320 trits of a row-superblock are five 64-trit MMA stages; 64 is not a multiple of 5, so the
//        trits are RE-GROUPED into base-3 bytes (same digit weights 1, 3, 9, 27, 81 as the canonical format)
//        such that every stage decodes from whole bytes: bytes 12 s .. 12 s + 11 hold trits 0..59 of stage s
//        in order (byte m = trits 5 m .. 5 m + 4), and byte 60 + m (m = 0..3) holds trit 60 + m of each of the
//        five stages (digit s = stage s). A canonical byte >= 243 (never written by the packer; all trits 0
//        by definition) is re-encoded as five zero trits, so it comes back from dst_untile_weights as 121.
//   TQ2: 32-bit word q of a row-superblock holds trits k = 256 sb + 16 q + (0..15), re-ordered so that a
//        (low half, high half) pair is two consecutive trits: trit 2j sits in bits [2j, 2j+1], trit 2j+1
//        in bits [16+2j, 17+2j]. One AND then yields an fp16x2 of adjacent weights.
//
// Inside a row-superblock the sixteen 32-bit words are transposed 4 x 4 and swizzled: logical word w (trits
// 16 w .. 16 w + 15 in TQ2, bytes 4 w .. 4 w + 3 in TQ1) is stored at physical word (((w & 3) ^ s) << 2) | (w >> 2)
// with s = (r >> 1) & 3. One 128-bit load of physical unit (c ^ s) therefore returns words c, 4 + c, 8 + c,
// 12 + c: the decode kernel's lane c of a quad gets its k-slots of all four 64-trit chunks in one load, and a
// quad reads the row's 64 bytes contiguously. The swizzle spreads the accesses of 32 threads that read the
// same word of 32 consecutive rows of a slab in shared memory (64-byte stride) over 8 bank groups instead of 2.
//
// dst_untile_weights inverts the permutation bit for bit.
#include "dst_common.cuh"

namespace dst {

int64_t tiled_superblocks(int fmt, int64_t K) { return cdiv64(K, fmt == DST_FMT_TQ2 ? 256 : 320); }

namespace {

// Raw 2-bit field of trit k; fields of the row's last byte beyond K are kept as stored (the packer writes
// digit 1 there), fields beyond the last byte are padding digits.
__device__ __forceinline__ uint32_t tq2_digit(const uint8_t* row, int64_t k, int64_t Kp) {
  return k < 4 * Kp ? (uint32_t)((row[k >> 2] >> ((k & 3) * 2)) & 3) : 1u;
}

// Digit (0..2) of trit k of a canonical TQ1 row; trits beyond the row's last byte are padding digits.
__device__ __forceinline__ uint32_t tq1_digit(const uint8_t* row, int64_t k, int64_t Kp) {
  const int64_t b = k / 5;
  return b < Kp ? (tq1_fields(row[b]) >> (2 * (int)(k - b * 5))) & 3u : 1u;
}

// Position of trit kk (0..319) of a row-superblock in the tiled TQ1 grouping: byte index and digit index.
__device__ __forceinline__ void tq1_tiled_pos(int kk, int& byte, int& digit) {
  const int s = kk >> 6, j = kk & 63;
  if (j < 60) {
    byte = 12 * s + j / 5;
    digit = j % 5;
  } else {
    byte = j;  // 60 + (j - 60)
    digit = s;
  }
}

// One thread per 32-bit word of the tiled buffer.
template <int FMT>
__global__ void tile_kernel(const uint8_t* __restrict__ canon, int64_t E, int64_t N, int64_t K, int64_t Kp, int64_t NT,
                            int64_t S, uint32_t* __restrict__ tiled) {
  const int64_t total = E * NT * S * 128 * 16;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int q = (int)(i & 15);
    const int r = (int)((i >> 4) & 127);
    int64_t rest = i >> 11;
    const int64_t sb = rest % S;
    rest /= S;
    const int64_t nt = rest % NT, e = rest / NT;
    const int64_t n = nt * 128 + r;
    uint32_t w;
    if (n >= N) {
      w = FMT == 2 ? 0x55555555u : 0x79797979u;  // all digits 1 (t = 0); 0x79 = 121 = 1+3+9+27+81
    } else {
      const uint8_t* row = canon + (e * N + n) * Kp;
      if (FMT == 2) {
        const int64_t k0 = sb * 256 + q * 16;
        w = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          w |= tq2_digit(row, k0 + 2 * j, Kp) << (2 * j);
          w |= tq2_digit(row, k0 + 2 * j + 1, Kp) << (16 + 2 * j);
        }
      } else {
        w = 0;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const int bi = q * 4 + b;
          uint32_t v = 0, pw = 1;
#pragma unroll
          for (int d = 0; d < 5; ++d) {
            // trit of the superblock that lives in digit d of tiled byte bi
            const int kk = bi < 60 ? 64 * (bi / 12) + 5 * (bi % 12) + d : 64 * d + bi;
            v += tq1_digit(row, sb * 320 + kk, Kp) * pw;
            pw *= 3;
          }
          w |= v << (8 * b);
        }
      }
    }
    tiled[(i & ~15LL) | (((q & 3) ^ ((r >> 1) & 3)) << 2) | (q >> 2)] = w;
  }
}

// One thread per canonical byte.
template <int FMT>
__global__ void untile_kernel(const uint8_t* __restrict__ tiled, int64_t E, int64_t N, int64_t K, int64_t Kp, int64_t NT,
                              int64_t S, uint8_t* __restrict__ canon) {
  const int64_t total = E * N * Kp;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t b = i % Kp;
    int64_t rest = i / Kp;
    const int64_t n = rest % N, e = rest / N;
    const int64_t nt = n >> 7, r = n & 127;
    uint8_t v;
    if (FMT == 1) {
      uint32_t acc = 0, pw = 1;
#pragma unroll
      for (int d = 0; d < 5; ++d) {
        const int64_t k = b * 5 + d;
        const int64_t sb = k / 320;
        int bi, di;
        tq1_tiled_pos((int)(k - sb * 320), bi, di);
        const int w = bi >> 2;
        const uint8_t tb =
            tiled[(((e * NT + nt) * S + sb) * 128 + r) * 64 + ((((w & 3) ^ ((int)(r >> 1) & 3)) << 4) | ((w >> 2) << 2) | (bi & 3))];
        acc += ((tq1_fields(tb) >> (2 * di)) & 3u) * pw;
        pw *= 3;
      }
      v = (uint8_t)acc;
    } else {
      uint32_t acc = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int64_t k = b * 4 + j;
        const int64_t sb = k >> 8;
        const int kk = (int)(k & 255), q = kk >> 4, t = kk & 15;
        const uint32_t w = reinterpret_cast<const uint32_t*>(tiled)[(((e * NT + nt) * S + sb) * 128 + r) * 16 +
                                                                    ((((q & 3) ^ ((int)(r >> 1) & 3)) << 2) | (q >> 2))];
        const int bit = (t & 1) ? 16 + (t >> 1) * 2 : (t >> 1) * 2;
        acc |= ((w >> bit) & 3u) << (2 * j);
      }
      v = (uint8_t)acc;
    }
    canon[i] = v;
  }
}

int grid_for(int64_t total) {
  int64_t g = (total + 255) / 256;
  const int64_t cap = 148 * 32;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace
}  // namespace dst

using namespace dst;

extern "C" int64_t dst_tiled_bytes(int fmt, int64_t E, int64_t N, int64_t K) {
  if ((fmt != DST_FMT_TQ1 && fmt != DST_FMT_TQ2) || E < 0 || N < 0 || K <= 0) return -1;
  return E * cdiv64(N, 128) * tiled_superblocks(fmt, K) * 8192;
}

extern "C" int dst_tile_weights(const uint8_t* canonical, int64_t E, int64_t N, int64_t K, int fmt, uint8_t* tiled,
                                dst_stream_t stream) {
  if ((fmt != DST_FMT_TQ1 && fmt != DST_FMT_TQ2) || K <= 0 || E < 0 || N < 0) return DST_ERR_BAD_ARG;
  if (E == 0 || N == 0) return DST_OK;
  if (!canonical || !tiled) return DST_ERR_BAD_ARG;
  if (E > DST_MAX_EXPERTS || K > (int64_t(1) << 24) || N > (int64_t(1) << 24)) return DST_ERR_BAD_SHAPE;
  if (reinterpret_cast<uintptr_t>(tiled) & 15) return DST_ERR_ALIGNMENT;
  const int64_t Kp = cdiv64(K, fmt == DST_FMT_TQ2 ? 4 : 5), NT = cdiv64(N, 128), S = tiled_superblocks(fmt, K);
  auto st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(E * NT * S * 2048);
  if (fmt == DST_FMT_TQ2) tile_kernel<2><<<grid, 256, 0, st>>>(canonical, E, N, K, Kp, NT, S, reinterpret_cast<uint32_t*>(tiled));
  else tile_kernel<1><<<grid, 256, 0, st>>>(canonical, E, N, K, Kp, NT, S, reinterpret_cast<uint32_t*>(tiled));
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}

extern "C" int dst_untile_weights(const uint8_t* tiled, int64_t E, int64_t N, int64_t K, int fmt, uint8_t* canonical,
                                  dst_stream_t stream) {
  if ((fmt != DST_FMT_TQ1 && fmt != DST_FMT_TQ2) || K <= 0 || E < 0 || N < 0) return DST_ERR_BAD_ARG;
  if (E == 0 || N == 0) return DST_OK;
  if (!canonical || !tiled) return DST_ERR_BAD_ARG;
  if (E > DST_MAX_EXPERTS || K > (int64_t(1) << 24) || N > (int64_t(1) << 24)) return DST_ERR_BAD_SHAPE;
  if (reinterpret_cast<uintptr_t>(tiled) & 15) return DST_ERR_ALIGNMENT;
  const int64_t Kp = cdiv64(K, fmt == DST_FMT_TQ2 ? 4 : 5), NT = cdiv64(N, 128), S = tiled_superblocks(fmt, K);
  auto st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(E * N * Kp);
  if (fmt == DST_FMT_TQ2) untile_kernel<2><<<grid, 256, 0, st>>>(tiled, E, N, K, Kp, NT, S, canonical);
  else untile_kernel<1><<<grid, 256, 0, st>>>(tiled, E, N, K, Kp, NT, S, canonical);
  DST_CUDA_TRY(cudaGetLastError());
  return DST_OK;
}
