/*
 * CPU oracle for the sparse-convolution hot path (TEST INFRASTRUCTURE ONLY).
 *
 * This file restates, in plain scalar C, what the reference's gather-GEMM-scatter GEMM
 * and mask-based implicit-GEMM sparse convolution compute.  It is the checker the GPU
 * kernels are compared with.  Nothing in the shipped library links, loads or calls it.
 *
 * Parity status.
 *   - fp16 <-> fp32 conversion and fp32 -> int8 saturating round-half-even are pinned
 *     against the reference's own host converters (tv::half_t and
 *     NumericConverter<int8_t,float>), compiled from the reference headers by
 *     oracle/Makefile into oracle/_ref, and against golden vectors generated from them.
 *   - mnk / tile-count / workspace arithmetic is pinned the same way.
 *   - The convolution loops follow the reference's numpy definition of the op and the
 *     device kernel's control flow (citations at each function).  The reference stores
 *     no golden vectors for these loops and its fixture for them is not distributed with
 *     it, so for the loops themselves: PARITY UNPINNED (self-consistency only: the
 *     device-semantics restatement here is cross-checked against an independent
 *     per-offset numpy gather-matmul-scatter in oracle/oracle.py).
 *   - int8 requantisation epilogue: the reference has no test of it at all; the
 *     definition below is read from its source.  PARITY UNPINNED beyond the converters.
 *   - Pair / mask / argsort generation is not part of the reference (it lives in a
 *     downstream project); the convention used is documented at orc_build_pairs.
 *
 * All fp16 tensors are passed as uint16_t bit patterns.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------------------------
 * Scalar numerics
 * ---------------------------------------------------------------------------------- */

/* fp16 bits -> fp32.  Same value map as the reference's half_t::convert (
 * include/tensorview/gemm/dtypes/half.h, host branch): exact widening. */
float orc_half_to_float(uint16_t h) {
  uint32_t sign = (uint32_t)(h >> 15) << 31;
  int exp = (h >> 10) & 0x1f;
  uint32_t man = h & 0x3ff;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      /* subnormal: normalise */
      int e = -1;
      do {
        man <<= 1;
        ++e;
      } while (!(man & 0x400));
      man &= 0x3ff;
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((uint32_t)(exp - 15 + 127) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

/* fp32 -> fp16 bits, round-to-nearest-even, overflow to infinity, NaN kept quiet.
 * Value map of the reference's half_t(float) host constructor
 * (include/tensorview/gemm/dtypes/half.h) and of the device cvt.rn.f16.f32 used by the
 * epilogue's NumericConverter (include/tensorview/gemm/math/numeric_convert.h). */
uint16_t orc_float_to_half(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
  uint32_t ax = x & 0x7fffffffu;
  if (ax >= 0x7f800000u) { /* inf / nan */
    if (ax > 0x7f800000u)
      return (uint16_t)(sign | 0x7fffu); /* reference returns canonical NaN 0x7fff */
    return (uint16_t)(sign | 0x7c00u);
  }
  int exp = (int)(ax >> 23) - 127;
  uint32_t man = ax & 0x7fffffu;
  if (exp > 15) {
    return (uint16_t)(sign | 0x7c00u);
  }
  if (exp >= -14) {
    /* normal half */
    uint32_t hman = man >> 13;
    uint32_t rest = man & 0x1fffu;
    uint32_t h = ((uint32_t)(exp + 15) << 10) | hman;
    if (rest > 0x1000u || (rest == 0x1000u && (h & 1u)))
      ++h; /* may carry into exponent, incl. to inf: correct */
    return (uint16_t)(sign | h);
  }
  if (exp < -25) {
    return sign; /* underflow to zero (values below half of the smallest subnormal) */
  }
  /* subnormal half */
  man |= 0x800000u;
  int shift = -14 - exp + 13; /* 14..24 */
  uint32_t hman = man >> shift;
  uint32_t rest = man & ((1u << shift) - 1u);
  uint32_t half = 1u << (shift - 1);
  if (rest > half || (rest == half && (hman & 1u)))
    ++hman;
  return (uint16_t)(sign | hman);
}

/* fp32 -> int8: round half to even, saturate, NaN -> 0.
 * Reference: NumericConverter<int8_t,float,round_to_nearest>, device cvt.rni.sat.s8.f32
 * (include/tensorview/gemm/math/numeric_convert.h:173-193) and host twin (:263-283). */
int8_t orc_float_to_s8(float t) {
  if (t != t)
    return 0;
  float r = nearbyintf(t); /* default rounding mode = nearest even */
  if (r > 127.f)
    r = 127.f;
  if (r < -128.f)
    r = -128.f;
  return (int8_t)r;
}

/* Activation on the fp32 intermediate.  Reference: UnaryActivation
 * (cumm/gemm/gemmmath/__init__.py:151-216); codes from
 * include/tensorview/gemm/core/constants.h:40-56 (0 none, 1 ReLU, 2 Sigmoid, 3 LeakyReLU). */
static float orc_act(float x, int act_type, float act_alpha) {
  switch (act_type) {
  case 1:
    return x > 0.f ? x : 0.f;
  case 2:
    return 1.f / (1.f + expf(-x));
  case 3:
    return x >= 0.f ? x : x * act_alpha;
  default:
    return x;
  }
}

/* Linear-combination epilogue for floating outputs.
 * Reference: LinearCombination (cumm/gemm/output_op/linear.py:105-144): with a source,
 * t = beta*src, then t = alpha*acc + t (a fused multiply-add on device); without
 * (beta == 0, cumm/gemm/outputs/__init__.py:155-164) t = alpha*acc. */
static float orc_lincomb(float acc, float alpha, float beta, int has_src, float src) {
  if (has_src && beta != 0.f)
    return fmaf(alpha, acc, beta * src);
  return alpha * acc;
}

/* ------------------------------------------------------------------------------------
 * Gather-GEMM-scatter GEMM  (GemmParams with a_inds / c_inds, "ShuffleAC")
 *
 * Reference: cumm/gemm/kernel.py:640-932 with the gathering A iterator
 * (cumm/gemm/mask_iters.py:971-988) and scattering output iterator
 * (cumm/gemm/out_iters.py:541-553); numpy statement at cumm/gemm/main_real.py:196-232.
 *
 *   for i < m:  C[c_inds[i], :] = act(alpha * A[a_inds[i], :] @ B' + beta * D[c_inds[i], :])
 *
 * b is [n,k] when trans_b (row n holds the k-vector) else [k,n]; d_is_bias: D is a
 * length-n vector read without the scatter index (cumm/gemm/nvrtc_code.py:126-128,160-161).
 * a_inds or c_inds may be NULL = identity.  Strides in elements.
 * ---------------------------------------------------------------------------------- */
void orc_gemm_shuffle_ac_f16(int m, int n, int k, const uint16_t *a, int64_t lda,
                             const uint16_t *b, int64_t ldb, int trans_b, uint16_t *c,
                             int64_t ldc, const uint16_t *d, int64_t ldd, int d_is_bias,
                             const int32_t *a_inds, const int32_t *c_inds, float alpha,
                             float beta, int act_type, float act_alpha) {
  float *bt = (float *)malloc(sizeof(float) * (size_t)n * k); /* [n][k] */
  for (int j = 0; j < n; ++j)
    for (int p = 0; p < k; ++p)
      bt[(size_t)j * k + p] =
          orc_half_to_float(trans_b ? b[(int64_t)j * ldb + p] : b[(int64_t)p * ldb + j]);
  float *arow = (float *)malloc(sizeof(float) * k);
  uint16_t *orow = (uint16_t *)malloc(sizeof(uint16_t) * n);
  for (int i = 0; i < m; ++i) {
    int64_t ia = a_inds ? a_inds[i] : i;
    int64_t ic = c_inds ? c_inds[i] : i;
    for (int p = 0; p < k; ++p)
      arow[p] = orc_half_to_float(a[ia * lda + p]);
    for (int j = 0; j < n; ++j) {
      float acc = 0.f;
      const float *bj = bt + (size_t)j * k;
      for (int p = 0; p < k; ++p)
        acc += arow[p] * bj[p];
      float src = 0.f;
      int has_src = (d != NULL) && beta != 0.f;
      if (has_src)
        src = orc_half_to_float(d_is_bias ? d[j] : d[ic * ldd + j]);
      float t = orc_act(orc_lincomb(acc, alpha, beta, has_src, src), act_type, act_alpha);
      orow[j] = orc_float_to_half(t);
    }
    memcpy(c + ic * ldc, orow, sizeof(uint16_t) * n);
  }
  free(bt);
  free(arow);
  free(orow);
}

/* Gather-gather GEMM for weight gradients ("ShuffleAB", trans_a && !trans_b).
 * Reference: cumm/gemm/nvrtc_code.py:98-112 (shapes), cumm/gemm/kernel.py:833-871;
 * numpy statement cumm/gemm/main_real.py:196-232 (a[a_inds].T @ b[b_inds]).
 *   C[i, j] = act(alpha * sum_p A[a_inds[p], i] * B[b_inds[p], j] + beta * D[i, j])
 * a is [*, m], b is [*, n], p runs over kk pairs. */
void orc_gemm_shuffle_ab_f16(int m, int n, int kk, const uint16_t *a, int64_t lda,
                             const uint16_t *b, int64_t ldb, uint16_t *c, int64_t ldc,
                             const uint16_t *d, int64_t ldd, const int32_t *a_inds,
                             const int32_t *b_inds, float alpha, float beta, int act_type,
                             float act_alpha) {
  float *acc = (float *)calloc((size_t)m * n, sizeof(float));
  float *ar = (float *)malloc(sizeof(float) * m);
  float *br = (float *)malloc(sizeof(float) * n);
  for (int p = 0; p < kk; ++p) {
    int64_t ia = a_inds[p], ib = b_inds[p];
    for (int i = 0; i < m; ++i)
      ar[i] = orc_half_to_float(a[ia * lda + i]);
    for (int j = 0; j < n; ++j)
      br[j] = orc_half_to_float(b[ib * ldb + j]);
    for (int i = 0; i < m; ++i) {
      float av = ar[i];
      float *row = acc + (size_t)i * n;
      for (int j = 0; j < n; ++j)
        row[j] += av * br[j];
    }
  }
  for (int i = 0; i < m; ++i)
    for (int j = 0; j < n; ++j) {
      int has_src = (d != NULL) && beta != 0.f;
      float src = has_src ? orc_half_to_float(d[(int64_t)i * ldd + j]) : 0.f;
      float t = orc_act(orc_lincomb(acc[(size_t)i * n + j], alpha, beta, has_src, src),
                        act_type, act_alpha);
      c[(int64_t)i * ldc + j] = orc_float_to_half(t);
    }
  free(acc);
  free(ar);
  free(br);
}

/* ------------------------------------------------------------------------------------
 * Mask-based implicit GEMM, forward and input-gradient (device control flow)
 *
 * Reference: cumm/conv/kernel.py:825-920 (tile mask OR, mask_filter, mask_out store,
 * dgrad early exit, reverse_mask), cumm/conv/sparse_iters.py:317-356,626-631 (row r of a
 * tile is valid iff r < N and indices[f, mask_argsort[r]] >= 0), cumm/gemm/blockmma/mma.py
 * :445-578 (visit set bits of the tile mask in ascending order), cumm/conv/kernel.py
 * :446-448 (rows are written at mask_argsort[r]; source = output row or bias vector).
 *
 * is_dgrad = 0: out[o, n] = sum_f sum_c  X[idx[f,o], c] * W[n, f, c]     (red = C_in, nn = K_out)
 * is_dgrad = 1: out[o, n] = sum_f sum_k  X[idx[f,o], k] * W[k, f, n]     (red = K_out, nn = C_in)
 * where X is `a` (features, resp. output gradients), W is [K_out, kv, C_in] and `red`,
 * `nn` are the reduction and output widths.  tile_m is the number of sorted rows that
 * share one OR-ed mask.  mask is in sorted order, indices in original order.
 * d (may be NULL): source rows (same layout as out) or, when d_is_bias, a length-nn vector.
 *
 * Kernel volumes above 32 (cumm/gemm/blockmma/mma.py:78-270, the dynamic mask loader): a row's
 * mask is `words` = ceil(kv / 32) consecutive 32-bit words, word w covering offsets 32w..32w+31;
 * each OR-ed word is ANDed with mask_filter; mask_out[tile * words + w]; the input gradient
 * leaves a tile untouched when all words are zero, and reverse_mask makes step `pos` (weight
 * offset pos) depend on the mask bit of offset kv - 1 - pos.
 * ---------------------------------------------------------------------------------- */
/* OR of the mask words of the rows of a tile, filtered; returns whether any bit is left. */
static int orc_tile_masks(const uint32_t *mask, int r0, int rows, int words, uint32_t mask_filter,
                          uint32_t *kmask) {
  int any = 0;
  for (int w = 0; w < words; ++w) {
    uint32_t m = 0;
    for (int r = 0; r < rows; ++r)
      m |= mask[(size_t)(r0 + r) * words + w];
    kmask[w] = m & mask_filter;
    any |= kmask[w] != 0;
  }
  return any;
}
/* Is step `pos` (weight offset pos) of a tile taken?  With reverse, the bit of offset kv-1-pos. */
static int orc_step_on(const uint32_t *kmask, int kv, int pos, int reverse) {
  int f = reverse ? kv - 1 - pos : pos;
  return (kmask[f >> 5] >> (f & 31)) & 1u;
}

void orc_mask_igemm_f16(int is_dgrad, int N, int a_rows, int C_in, int K_out, int kv,
                        const uint16_t *a, const uint16_t *w, uint16_t *out,
                        const uint16_t *d, int d_is_bias, const int32_t *indices,
                        const uint32_t *mask, const int32_t *mask_argsort,
                        uint32_t *mask_out, uint32_t mask_filter, int reverse_mask,
                        int tile_m, float alpha, float beta, int act_type,
                        float act_alpha) {
  (void)a_rows;
  const int words = (kv + 31) / 32;
  uint32_t kmask[8];
  int red = is_dgrad ? K_out : C_in;
  int nn = is_dgrad ? C_in : K_out;
  /* weights as float, laid out [f][n][red] for contiguous dot products */
  float *wf = (float *)malloc(sizeof(float) * (size_t)kv * nn * red);
  for (int f = 0; f < kv; ++f)
    for (int n = 0; n < nn; ++n)
      for (int p = 0; p < red; ++p) {
        size_t src = is_dgrad ? ((size_t)p * kv + f) * C_in + n : ((size_t)n * kv + f) * C_in + p;
        wf[((size_t)f * nn + n) * red + p] = orc_half_to_float(w[src]);
      }
  float *acc = (float *)malloc(sizeof(float) * (size_t)tile_m * nn);
  float *arow = (float *)malloc(sizeof(float) * red);
  int tiles = (N + tile_m - 1) / tile_m;
  for (int t = 0; t < tiles; ++t) {
    int r0 = t * tile_m;
    int rows = N - r0 < tile_m ? N - r0 : tile_m;
    int any = orc_tile_masks(mask, r0, rows, words, mask_filter, kmask);
    if (!is_dgrad) {
      if (mask_out)
        for (int w = 0; w < words; ++w)
          mask_out[(size_t)t * words + w] = kmask[w];
    } else if (!any) {
      continue; /* tile left untouched */
    }
    memset(acc, 0, sizeof(float) * (size_t)tile_m * nn);
    for (int f = 0; f < kv; ++f) {
      if (!orc_step_on(kmask, kv, f, is_dgrad && reverse_mask))
        continue;
      const float *wff = wf + (size_t)f * nn * red;
      for (int r = 0; r < rows; ++r) {
        int o = mask_argsort[r0 + r];
        int i = indices[(size_t)f * N + o];
        if (i < 0)
          continue;
        const uint16_t *ap = a + (size_t)i * red;
        for (int p = 0; p < red; ++p)
          arow[p] = orc_half_to_float(ap[p]);
        float *ar = acc + (size_t)r * nn;
        for (int n = 0; n < nn; ++n) {
          const float *wn = wff + (size_t)n * red;
          float s = 0.f;
          for (int p = 0; p < red; ++p)
            s += arow[p] * wn[p];
          ar[n] += s;
        }
      }
    }
    for (int r = 0; r < rows; ++r) {
      int o = mask_argsort[r0 + r];
      uint16_t *op = out + (size_t)o * nn;
      for (int n = 0; n < nn; ++n) {
        int has_src = (d != NULL) && beta != 0.f;
        float src = 0.f;
        if (has_src)
          src = orc_half_to_float(d_is_bias ? d[n] : d[(size_t)o * nn + n]);
        float tt = orc_act(orc_lincomb(acc[(size_t)r * nn + n], alpha, beta, has_src, src),
                           act_type, act_alpha);
        op[n] = orc_float_to_half(tt);
      }
    }
  }
  free(wf);
  free(acc);
  free(arow);
}

/* ------------------------------------------------------------------------------------
 * Mask-based implicit GEMM, weight gradient.
 *
 * Reference: cumm/conv/kernel.py:890-897 (a filter offset excluded by mask_filter leaves
 * its slice untouched), cumm/gemm/blockmma/mma.py:608-648,722-740 (sorted rows are walked
 * in chunks; a chunk whose reduced mask word lacks bit f is skipped; one reduced-mask
 * word covers mask_width sorted rows), cumm/conv/sparse_iters.py:284-316 (A = dout rows at
 * mask_argsort[r], B = X rows at indices[f, mask_argsort[r]], -1 -> zeros),
 * cumm/conv/kernel.py:970-974 (block of dW viewed [K, kv*C]).
 *
 *   dW[k, f, c] = alpha * sum_r dout[o_r, k] * X[idx[f, o_r], c] + beta * dW_prev[k, f, c]
 *
 * out_f32 != NULL: write fp32 results there instead of fp16 `dw` (used for the multi-GPU
 * partial sums); the source for beta is then out_f32 itself.
 * ---------------------------------------------------------------------------------- */
void orc_mask_igemm_wgrad_f16(int N, int C_in, int K_out, int kv, const uint16_t *dout,
                              const uint16_t *x, uint16_t *dw, float *out_f32,
                              const int32_t *indices, const uint32_t *reduced_mask,
                              const int32_t *mask_argsort, uint32_t mask_filter,
                              int mask_width, float alpha, float beta) {
  float *acc = (float *)malloc(sizeof(float) * (size_t)K_out * C_in);
  float *dor = (float *)malloc(sizeof(float) * K_out);
  float *xr = (float *)malloc(sizeof(float) * C_in);
  const int words = (kv + 31) / 32; /* reduced_mask[chunk * words + f / 32], filter bit f % 32 */
  for (int f = 0; f < kv; ++f) {
    if (!((mask_filter >> (f & 31)) & 1u))
      continue;
    memset(acc, 0, sizeof(float) * (size_t)K_out * C_in);
    for (int r = 0; r < N; ++r) {
      if (!((reduced_mask[(size_t)(r / mask_width) * words + (f >> 5)] >> (f & 31)) & 1u))
        continue;
      int o = mask_argsort[r];
      int i = indices[(size_t)f * N + o];
      if (i < 0)
        continue;
      for (int k = 0; k < K_out; ++k)
        dor[k] = orc_half_to_float(dout[(size_t)o * K_out + k]);
      for (int c = 0; c < C_in; ++c)
        xr[c] = orc_half_to_float(x[(size_t)i * C_in + c]);
      for (int k = 0; k < K_out; ++k) {
        float dv = dor[k];
        float *row = acc + (size_t)k * C_in;
        for (int c = 0; c < C_in; ++c)
          row[c] += dv * xr[c];
      }
    }
    for (int k = 0; k < K_out; ++k)
      for (int c = 0; c < C_in; ++c) {
        size_t off = ((size_t)k * kv + f) * C_in + c;
        float a = acc[(size_t)k * C_in + c];
        if (out_f32) {
          out_f32[off] = beta != 0.f ? fmaf(alpha, a, beta * out_f32[off]) : alpha * a;
        } else {
          float src = beta != 0.f ? orc_half_to_float(dw[off]) : 0.f;
          dw[off] = orc_float_to_half(orc_lincomb(a, alpha, beta, beta != 0.f, src));
        }
      }
  }
  free(acc);
  free(dor);
  free(xr);
}

/* ------------------------------------------------------------------------------------
 * int8 inference forward with fused requantisation.
 *
 * Reference: Int8Inference output op (cumm/gemm/output_op/linear.py:279-360):
 *   t = fma(scale[n], float(acc_s32), bias[n]);
 *   if beta != 0: t = fma(beta, float(src_s8), t);   src = output_add row, or the output
 *                 row itself when no output_add is given (cumm/conv/nvrtc_code.py:78-90)
 *   t = act(t); out = sat_s8(round_half_even(t))
 * float(acc_s32) is the default int->float conversion (round to nearest even,
 * include/tensorview/gemm/math/numeric_convert.h:59-82).  The multiply-adds are fused
 * (functional.h:225-229 `a*b+c`, compiled with the default contraction).
 * alpha is not used.  Control flow as in orc_mask_igemm_f16 (forward only).
 * ---------------------------------------------------------------------------------- */
void orc_mask_igemm_s8(int N, int C_in, int K_out, int kv, const int8_t *x, const int8_t *w,
                       int8_t *out, const int8_t *output_add, const float *scale,
                       const float *bias, const int32_t *indices, const uint32_t *mask,
                       const int32_t *mask_argsort, uint32_t *mask_out, uint32_t mask_filter,
                       int tile_m, float beta, int act_type, float act_alpha) {
  int32_t *acc = (int32_t *)malloc(sizeof(int32_t) * (size_t)tile_m * K_out);
  int tiles = (N + tile_m - 1) / tile_m;
  const int words = (kv + 31) / 32;
  uint32_t kmask[8];
  for (int t = 0; t < tiles; ++t) {
    int r0 = t * tile_m;
    int rows = N - r0 < tile_m ? N - r0 : tile_m;
    orc_tile_masks(mask, r0, rows, words, mask_filter, kmask);
    if (mask_out)
      for (int w = 0; w < words; ++w)
        mask_out[(size_t)t * words + w] = kmask[w];
    memset(acc, 0, sizeof(int32_t) * (size_t)tile_m * K_out);
    for (int f = 0; f < kv; ++f) {
      if (!orc_step_on(kmask, kv, f, 0))
        continue;
      for (int r = 0; r < rows; ++r) {
        int o = mask_argsort[r0 + r];
        int i = indices[(size_t)f * N + o];
        if (i < 0)
          continue;
        const int8_t *xp = x + (size_t)i * C_in;
        for (int n = 0; n < K_out; ++n) {
          const int8_t *wp = w + ((size_t)n * kv + f) * C_in;
          int32_t s = 0;
          for (int c = 0; c < C_in; ++c)
            s += (int32_t)xp[c] * (int32_t)wp[c];
          acc[(size_t)r * K_out + n] += s;
        }
      }
    }
    for (int r = 0; r < rows; ++r) {
      int o = mask_argsort[r0 + r];
      for (int n = 0; n < K_out; ++n) {
        float tt = fmaf(scale[n], (float)acc[(size_t)r * K_out + n], bias[n]);
        if (beta != 0.f) {
          const int8_t *sp = output_add ? output_add : out;
          tt = fmaf(beta, (float)sp[(size_t)o * K_out + n], tt);
        }
        tt = orc_act(tt, act_type, act_alpha);
        out[(size_t)o * K_out + n] = orc_float_to_s8(tt);
      }
    }
  }
  free(acc);
}

/* Requantise a caller-provided int32 accumulator matrix (used to check the epilogue
 * separately from the contraction, e.g. against a BLAS-computed accumulator). */
void orc_requant_s8(int rows, int K_out, const int32_t *acc, const float *scale,
                    const float *bias, float beta, const int8_t *src, int act_type,
                    float act_alpha, int8_t *out) {
  for (int r = 0; r < rows; ++r)
    for (int n = 0; n < K_out; ++n) {
      float tt = fmaf(scale[n], (float)acc[(size_t)r * K_out + n], bias[n]);
      if (beta != 0.f && src)
        tt = fmaf(beta, (float)src[(size_t)r * K_out + n], tt);
      tt = orc_act(tt, act_type, act_alpha);
      out[(size_t)r * K_out + n] = orc_float_to_s8(tt);
    }
}

/* The fp16 output operator on a caller-provided fp32 accumulator array (used to check the
 * epilogue separately from the contraction): LinearCombination,
 * cumm/gemm/output_op/linear.py:105-144.  src / out are raw fp16 bit patterns; src may be
 * NULL (no beta term). */
void orc_lincomb_f16(long long n, const float *acc, float alpha, float beta, const uint16_t *src,
                     int act_type, float act_alpha, uint16_t *out) {
  for (long long i = 0; i < n; ++i) {
    int has_src = src != NULL && beta != 0.f;
    float sv = has_src ? orc_half_to_float(src[i]) : 0.f;
    float t = orc_act(orc_lincomb(acc[i], alpha, beta, has_src, sv), act_type, act_alpha);
    out[i] = orc_float_to_half(t);
  }
}

/* ------------------------------------------------------------------------------------
 * Pair / mask generation (convention documented here; the reference does not contain
 * this step).
 *
 * Cross-correlation, per axis  in = out*stride - pad + r*dilation  (the reference's
 * dense-conv coordinate rule, cumm/conv/input_iters.py:2666,2684, mode fixed to
 * cross-correlation at cumm/conv/nvrtc_code.py:204).  Filter offset f is the row-major
 * index of (r_z, r_y, r_x).  coords are (b, z, y, x) int32 rows.
 * indices[f, o] = row of the input voxel at that coordinate in the same batch, else -1.
 * mask[o] bit f set iff indices[f, o] >= 0.
 *
 * Open-addressing hash on the linearised coordinate; returns 0 on success.
 * ---------------------------------------------------------------------------------- */
typedef struct {
  int64_t *keys;
  int32_t *vals;
  uint64_t cap;
} orc_hash;

static uint64_t orc_mix(uint64_t k) {
  k ^= k >> 33;
  k *= 0xff51afd7ed558ccdULL;
  k ^= k >> 33;
  k *= 0xc4ceb9fe1a85ec53ULL;
  k ^= k >> 33;
  return k;
}

static int orc_hash_init(orc_hash *h, int n) {
  uint64_t cap = 16;
  while (cap < (uint64_t)n * 2 + 1)
    cap <<= 1;
  h->cap = cap;
  h->keys = (int64_t *)malloc(sizeof(int64_t) * cap);
  h->vals = (int32_t *)malloc(sizeof(int32_t) * cap);
  if (!h->keys || !h->vals)
    return -1;
  for (uint64_t i = 0; i < cap; ++i)
    h->keys[i] = -1;
  return 0;
}

static void orc_hash_put(orc_hash *h, int64_t key, int32_t val) {
  uint64_t p = orc_mix((uint64_t)key) & (h->cap - 1);
  while (h->keys[p] != -1 && h->keys[p] != key)
    p = (p + 1) & (h->cap - 1);
  if (h->keys[p] == -1) { /* first occurrence wins */
    h->keys[p] = key;
    h->vals[p] = val;
  }
}

static int32_t orc_hash_get(const orc_hash *h, int64_t key) {
  uint64_t p = orc_mix((uint64_t)key) & (h->cap - 1);
  while (h->keys[p] != -1) {
    if (h->keys[p] == key)
      return h->vals[p];
    p = (p + 1) & (h->cap - 1);
  }
  return -1;
}

static void orc_hash_free(orc_hash *h) {
  free(h->keys);
  free(h->vals);
}

/* in_coords [n_in,4], out_coords [n_out,4] (b,z,y,x); grid = input spatial shape.
 * ksize/stride/pad/dil: 3 ints each (z,y,x).  indices: [kv, n_out]; mask: [n_out]. */
int orc_build_pairs(int n_in, const int32_t *in_coords, int n_out, const int32_t *out_coords,
                    const int32_t *grid, const int32_t *ksize, const int32_t *stride,
                    const int32_t *pad, const int32_t *dil, int32_t *indices,
                    uint32_t *mask) {
  orc_hash h;
  if (orc_hash_init(&h, n_in))
    return -1;
  int64_t gz = grid[0], gy = grid[1], gx = grid[2];
  for (int i = 0; i < n_in; ++i) {
    const int32_t *c = in_coords + 4 * (size_t)i;
    int64_t key = (((int64_t)c[0] * gz + c[1]) * gy + c[2]) * gx + c[3];
    orc_hash_put(&h, key, i);
  }
  int kv = ksize[0] * ksize[1] * ksize[2];
  const int words = (kv + 31) / 32; /* mask words per output row */
  if (words > 1)
    memset(mask, 0, sizeof(uint32_t) * (size_t)n_out * words);
  for (int o = 0; o < n_out; ++o) {
    const int32_t *c = out_coords + 4 * (size_t)o;
    uint32_t mk = 0;
    int f = 0;
    for (int rz = 0; rz < ksize[0]; ++rz)
      for (int ry = 0; ry < ksize[1]; ++ry)
        for (int rx = 0; rx < ksize[2]; ++rx, ++f) {
          int64_t z = (int64_t)c[1] * stride[0] - pad[0] + (int64_t)rz * dil[0];
          int64_t y = (int64_t)c[2] * stride[1] - pad[1] + (int64_t)ry * dil[1];
          int64_t x = (int64_t)c[3] * stride[2] - pad[2] + (int64_t)rx * dil[2];
          int32_t v = -1;
          if (z >= 0 && z < gz && y >= 0 && y < gy && x >= 0 && x < gx) {
            int64_t key = (((int64_t)c[0] * gz + z) * gy + y) * gx + x;
            v = orc_hash_get(&h, key);
          }
          indices[(size_t)f * n_out + o] = v;
          if (v >= 0) {
            if (words == 1) {
              if (f < 32)
                mk |= 1u << f;
            } else {
              mask[(size_t)o * words + (f >> 5)] |= 1u << (f & 31);
            }
          }
        }
    if (words == 1)
      mask[o] = mk;
  }
  orc_hash_free(&h);
  return 0;
}
