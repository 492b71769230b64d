/*
 * CPU oracle for the ternary expert GEMM path. TEST INFRASTRUCTURE ONLY: it is the checker the
 * parity tests, the smoke check and the bench's CPU-baseline leg compare the CUDA library
 * against. Nothing in the product package may link, import or execute it.
 *
 * It restates, in plain C, the arithmetic of the reference project (Vedant-Sood/DeepSeekTernarized,
 * "Boilerplate"); each function names the reference lines it follows. Parity is pinned: the
 * functions here are checked against outputs of the reference itself (committed fixtures under
 * tests/golden/, produced by tests/golden/make_golden.py from the reference's Python and C++ code).
 *
 * Formats (boilerplate/ternary/pack.py:1-17): a trit t in {-1,0,+1} is the digit u = t + 1.
 *   TQ2: byte = u0 | u1<<2 | u2<<4 | u3<<6, ceil(K/4) bytes per row.
 *   TQ1: byte = u0 + 3 u1 + 9 u2 + 27 u3 + 81 u4, ceil(K/5) bytes per row.
 * Rows are padded to a whole byte with digit 1 (t = 0). fmt code: 1 = TQ1, 2 = TQ2
 * (boilerplate/kernels/ternary_cuda.py:46-49).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_OK 0
#define ORC_BAD_ARG 1

static int64_t cdiv(int64_t a, int64_t b) { return a / b + (a % b != 0); }

/* boilerplate/ternary/pack.py:30-31 */
int64_t orc_packed_cols(int fmt, int64_t K) { return cdiv(K, fmt == 2 ? 4 : 5); }

/* boilerplate/ternary/pack.py:62-67: LUT[v][i] = ((v / 3^i) % 3) - 1 for v < 243, rows 243..255 all 0 */
void orc_tq1_lut(int8_t* lut /* [256*5] */) {
  static const int pow3[5] = {1, 3, 9, 27, 81};
  for (int v = 0; v < 256; ++v)
    for (int i = 0; i < 5; ++i) lut[v * 5 + i] = v < 243 ? (int8_t)((v / pow3[i]) % 3 - 1) : 0;
}

/* boilerplate/ternary/pack.py:34-45,54-59 (_digits + pack_tq2 / pack_tq1) */
int orc_pack(const int8_t* trits, int64_t N, int64_t K, int fmt, uint8_t* packed) {
  if ((fmt != 1 && fmt != 2) || N < 0 || K <= 0) return ORC_BAD_ARG;
  const int per = fmt == 2 ? 4 : 5;
  const int64_t Kp = cdiv(K, per);
  for (int64_t n = 0; n < N; ++n) {
    for (int64_t b = 0; b < Kp; ++b) {
      unsigned v = 0, mul = 1;
      for (int i = 0; i < per; ++i) {
        int64_t k = b * per + i;
        unsigned u = k < K ? (unsigned)(trits[n * K + k] + 1) : 1u; /* pad digit 1 */
        if (fmt == 2) v |= u << (2 * i); else { v += u * mul; mul *= 3; }
      }
      packed[n * Kp + b] = (uint8_t)v;
    }
  }
  return ORC_OK;
}

/* boilerplate/ternary/pack.py:48-51,70-74; boilerplate/kernels/csrc/boilerplate_cpu.cpp:19-32 */
static void decode_row(const uint8_t* p, int64_t Kp, int fmt, int8_t* out, const int8_t* lut) {
  if (fmt == 2) {
    for (int64_t b = 0; b < Kp; ++b)
      for (int i = 0; i < 4; ++i) out[4 * b + i] = (int8_t)(((p[b] >> (2 * i)) & 3) - 1);
  } else {
    for (int64_t b = 0; b < Kp; ++b) memcpy(out + 5 * b, lut + 5 * p[b], 5);
  }
}

int orc_unpack(const uint8_t* packed, int64_t N, int64_t K, int fmt, int8_t* trits) {
  if ((fmt != 1 && fmt != 2) || N < 0 || K <= 0) return ORC_BAD_ARG;
  const int per = fmt == 2 ? 4 : 5;
  const int64_t Kp = cdiv(K, per);
  int8_t lut[256 * 5];
  orc_tq1_lut(lut);
  int8_t* row = (int8_t*)malloc((size_t)(Kp * per + 8));
  if (!row) return ORC_BAD_ARG;
  for (int64_t n = 0; n < N; ++n) {
    decode_row(packed + n * Kp, Kp, fmt, row, lut);
    memcpy(trits + n * K, row, (size_t)K);
  }
  free(row);
  return ORC_OK;
}

/* boilerplate/kernels/csrc/boilerplate_cpu.cpp:70-77: sequential fp32 pos / neg sums, then pos - neg */
static float tdot_f32(const float* x, const int8_t* t, int64_t n) {
  float pos = 0.f, neg = 0.f;
  for (int64_t i = 0; i < n; ++i) {
    pos += t[i] > 0 ? x[i] : 0.f;
    neg += t[i] < 0 ? x[i] : 0.f;
  }
  return pos - neg;
}

/* boilerplate/kernels/csrc/boilerplate_cpu.cpp:34-68: exact integer group sum */
static int64_t tdot_i8(const int8_t* x, const int8_t* t, int64_t n) {
  int64_t acc = 0;
  for (int64_t i = 0; i < n; ++i) acc += (t[i] > 0 ? x[i] : 0) - (t[i] < 0 ? x[i] : 0);
  return acc;
}

/*
 * boilerplate/kernels/csrc/boilerplate_cpu.cpp:80-128. out [M,N] f32 is ACCUMULATED into.
 * x_f32 != NULL: float activations, x_scale ignored (line 124). Otherwise x_i8 with x_scale [M].
 * w_scale [N,G] f32 (the reference upcasts fp16 scales once, boilerplate/ternary/ops.py:37).
 * Per row n, per token m: y = 0; for g ascending: y += s[g] * dot(group g); out[m,n] += y (or y * xs[m]).
 * The reference is built with -O3 -march=native (boilerplate/kernels/cpu.py:23), under which gcc
 * contracts both multiply-adds into fused multiply-adds on any FMA-capable x86 host; they are written
 * as fmaf here so the oracle reproduces that build bit for bit whatever flags it is compiled with.
 */
int orc_gemm(float* out, const float* x_f32, const int8_t* x_i8, const float* x_scale,
             const uint8_t* packed, const float* w_scale, int64_t M, int64_t N, int64_t K,
             int64_t group, int fmt) {
  if (K <= 0 || group <= 0 || (fmt != 1 && fmt != 2) || M < 0 || N < 0) return ORC_BAD_ARG;
  if ((x_f32 == NULL) == (x_i8 == NULL)) return ORC_BAD_ARG;
  if (x_i8 && !x_scale) return ORC_BAD_ARG;
  const int per = fmt == 2 ? 4 : 5;
  const int64_t Kp = cdiv(K, per), G = cdiv(K, group);
  int8_t lut[256 * 5];
  orc_tq1_lut(lut);
  int fail = 0;
#pragma omp parallel
  {
    int8_t* trow = (int8_t*)malloc((size_t)(Kp * per + 64));
    if (!trow) {
#pragma omp atomic write
      fail = 1;
    }
#pragma omp for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
      if (!trow) continue;
      decode_row(packed + n * Kp, Kp, fmt, trow, lut);
      const float* s = w_scale + n * G;
      for (int64_t m = 0; m < M; ++m) {
        float y = 0.f;
        for (int64_t g = 0; g < G; ++g) {
          int64_t k0 = g * group, len = group < K - k0 ? group : K - k0;
          float a = x_i8 ? (float)tdot_i8(x_i8 + m * K + k0, trow + k0, len)
                         : tdot_f32(x_f32 + m * K + k0, trow + k0, len);
          y = fmaf(s[g], a, y);
        }
        out[m * N + n] = x_i8 ? fmaf(y, x_scale[m], out[m * N + n]) : out[m * N + n] + y;
      }
    }
    free(trow);
  }
  return fail ? ORC_BAD_ARG : ORC_OK;
}

/*
 * boilerplate/kernels/ternary_cuda.py:52-64 (ternary_gemm_ref): the reference-of-record for int8
 * activations. Group sums are exact integers; out (f32, starts at 0) += f32(acc) * w_scale[:, g]
 * for g ascending; finally out *= x_scale[:, None]. Overwrites out.
 */
int orc_gemm_ref_i8(float* out, const int8_t* x, const float* x_scale, const uint8_t* packed,
                    const float* w_scale, int64_t M, int64_t N, int64_t K, int64_t group, int fmt) {
  if (K <= 0 || group <= 0 || (fmt != 1 && fmt != 2) || M < 0 || N < 0) return ORC_BAD_ARG;
  const int per = fmt == 2 ? 4 : 5;
  const int64_t Kp = cdiv(K, per), G = cdiv(K, group);
  int8_t lut[256 * 5];
  orc_tq1_lut(lut);
#pragma omp parallel
  {
    int8_t* trow = (int8_t*)malloc((size_t)(Kp * per + 64));
#pragma omp for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
      if (!trow) continue;
      decode_row(packed + n * Kp, Kp, fmt, trow, lut);
      for (int64_t m = 0; m < M; ++m) {
        float o = 0.f;
        for (int64_t g = 0; g < G; ++g) {
          int64_t k0 = g * group, len = group < K - k0 ? group : K - k0;
          o += (float)tdot_i8(x + m * K + k0, trow + k0, len) * w_scale[n * G + g];
        }
        out[m * N + n] = o * x_scale[m];
      }
    }
    free(trow);
  }
  return ORC_OK;
}

/*
 * fp64 dequantized product, the tolerance target (boilerplate/ternary/ops.py:51-58 defines
 * W = sum_i unpack(packed_i) * scale_i repeated over each group; boilerplate/reference/compare.py:61-62
 * defines the error metrics). out64 [M,N] is ACCUMULATED into so k terms can be summed.
 */
int orc_gemm_f64(double* out64, const float* x, const uint8_t* packed, const float* w_scale,
                 int64_t M, int64_t N, int64_t K, int64_t group, int fmt) {
  if (K <= 0 || group <= 0 || (fmt != 1 && fmt != 2) || M < 0 || N < 0) return ORC_BAD_ARG;
  const int per = fmt == 2 ? 4 : 5;
  const int64_t Kp = cdiv(K, per), G = cdiv(K, group);
  int8_t lut[256 * 5];
  orc_tq1_lut(lut);
#pragma omp parallel
  {
    int8_t* trow = (int8_t*)malloc((size_t)(Kp * per + 64));
#pragma omp for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
      if (!trow) continue;
      decode_row(packed + n * Kp, Kp, fmt, trow, lut);
      for (int64_t m = 0; m < M; ++m) {
        double y = 0.0;
        for (int64_t k = 0; k < K; ++k)
          y += (double)x[m * K + k] * ((double)trow[k] * (double)w_scale[n * G + k / group]);
        out64[m * N + n] += y;
      }
    }
    free(trow);
  }
  return ORC_OK;
}

/*
 * boilerplate/kernels/ternary_cuda.py:90-111 (grouped_ternary_gemm, non-CUDA branch): rows of x are
 * sorted by expert, expert e owns rows offsets[e]..offsets[e+1]; packed [E,N,Kp], w_scale [E,N,G].
 * out [T,N] is accumulated into. Offsets are validated as lines 94-97 do.
 */
int orc_grouped_gemm(float* out, const float* x_f32, const int8_t* x_i8, const float* x_scale,
                     const int64_t* offsets, const uint8_t* packed, const float* w_scale, int64_t E,
                     int64_t T, int64_t N, int64_t K, int64_t group, int fmt) {
  if (K <= 0 || group <= 0 || (fmt != 1 && fmt != 2) || E < 0) return ORC_BAD_ARG;
  if (offsets[0] != 0 || offsets[E] != T) return ORC_BAD_ARG;
  for (int64_t e = 0; e < E; ++e)
    if (offsets[e + 1] < offsets[e]) return ORC_BAD_ARG;
  const int64_t Kp = orc_packed_cols(fmt, K), G = cdiv(K, group);
  for (int64_t e = 0; e < E; ++e) {
    int64_t a = offsets[e], b = offsets[e + 1];
    if (a >= b) continue;
    int rc = orc_gemm(out + a * N, x_f32 ? x_f32 + a * K : NULL, x_i8 ? x_i8 + a * K : NULL,
                      x_scale ? x_scale + a : NULL, packed + e * N * Kp, w_scale + e * N * G, b - a, N,
                      K, group, fmt);
    if (rc) return rc;
  }
  return ORC_OK;
}

/*
 * boilerplate/kernels/ternary_cuda.py:114-118 (sort_by_expert): stable argsort of the flattened
 * expert ids plus bincount/cumsum. A counting sort is the same permutation.
 */
int orc_sort_by_expert(const int64_t* ids, int64_t n, int64_t E, int64_t* order, int64_t* offsets) {
  for (int64_t e = 0; e <= E; ++e) offsets[e] = 0;
  for (int64_t i = 0; i < n; ++i) {
    if (ids[i] < 0 || ids[i] >= E) return ORC_BAD_ARG;
    offsets[ids[i] + 1]++;
  }
  for (int64_t e = 0; e < E; ++e) offsets[e + 1] += offsets[e];
  int64_t* cur = (int64_t*)malloc((size_t)(E + 1) * sizeof(int64_t));
  if (!cur) return ORC_BAD_ARG;
  memcpy(cur, offsets, (size_t)(E + 1) * sizeof(int64_t));
  for (int64_t i = 0; i < n; ++i) order[cur[ids[i]]++] = i;
  free(cur);
  return ORC_OK;
}

/*
 * boilerplate/ternary/ops.py:20-25 (quant_act_int8): s = max(absmax / 127, 1e-8);
 * q = clamp(round_half_even(x / s), -127, 127). torch.round rounds half to even, as nearbyintf does
 * in the default rounding mode.
 */
void orc_quant_act_int8(const float* x, int64_t M, int64_t K, int8_t* q, float* s) {
  for (int64_t m = 0; m < M; ++m) {
    float amax = 0.f;
    for (int64_t k = 0; k < K; ++k) {
      float a = fabsf(x[m * K + k]);
      if (a > amax) amax = a;
    }
    float sc = amax / 127.0f;
    if (sc < 1e-8f) sc = 1e-8f;
    s[m] = sc;
    for (int64_t k = 0; k < K; ++k) {
      float r = nearbyintf(x[m * K + k] / sc);
      if (r > 127.f) r = 127.f;
      if (r < -127.f) r = -127.f;
      q[m * K + k] = (int8_t)r;
    }
  }
}
