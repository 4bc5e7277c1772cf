/*
 * Recipe source for oracle/_ref/libref_host.so (TEST INFRASTRUCTURE ONLY).
 *
 * Compiles, as HOST code, the parts of the reference's own headers that carry the
 * arithmetic and the operator contract of the sparse-conv hot path, directly from where
 * they lie in the reference tree (-I<reference>/include).  No reference source is
 * copied: this file only includes those headers and exposes a few of their functions
 * with C linkage, so the CPU oracle and the Python operator mirror can be pinned to them.
 *
 * Exposed:
 *   tv::half_t float<->half                      include/tensorview/gemm/dtypes/half.h
 *   NumericConverter<int8_t,float>               include/tensorview/gemm/math/numeric_convert.h:263-283
 *   implicit_gemm_mnk, get_spconv_logical_tile_count, get_logical_tile_count,
 *   get_gemm_k_size_per_split                    include/tensorview/gemm/core/utils.h:20-122
 *   GemmAlgoDesp / ConvAlgoDesp __repr__, supported, query_*workspace_size
 *                                                include/tensorview/gemm/core/params.h:24-327
 */
#include <tensorview/gemm/dtypes/all.h>
#include <tensorview/gemm/math/all.h>
#include <tensorview/gemm/core/params.h>
#include <cstdint>
#include <cstring>
#include <string>

extern "C" {

uint16_t ref_float_to_half(float f) { return tv::half_t(f).raw(); }

float ref_half_to_float(uint16_t h) { return float(tv::half_t::bitcast(h)); }

int ref_float_to_s8(float f) {
  tv::gemm::NumericConverter<int8_t, float, tv::gemm::FloatRoundStyle::round_to_nearest> cv;
  return int(cv(f));
}

void ref_implicit_gemm_mnk(int op_type, int N, int C, int K, int kv, int *mnk) {
  auto r = tv::gemm::implicit_gemm_mnk(tv::gemm::ConvOpType(op_type), N, C, K, kv, -1, -1, true);
  mnk[0] = r[0];
  mnk[1] = r[1];
  mnk[2] = r[2];
}

void ref_spconv_tile_count(int m, int n, int k, int tile_m, int tile_n, int split_k, int kv,
                           int op_type, int *out) {
  auto r = tv::gemm::get_spconv_logical_tile_count(m, n, k, tile_m, tile_n, split_k, kv,
                                                   tv::gemm::ConvOpType(op_type));
  out[0] = r[0];
  out[1] = r[1];
  out[2] = r[2];
}

int ref_gemm_k_size_per_split(int k, int split_k, int tile_k) {
  return tv::gemm::get_gemm_k_size_per_split(k, split_k, tile_k);
}

struct ref_desp_fields {
  int dtype_a, dtype_b, dtype_c, dacc, dcomp;
  int trans_a, trans_b, trans_c;
  int tile_shape[3], warp_tile_shape[3], tensorop[3];
  int num_stage, split_k_serial, split_k_parallel, shuffle_type;
  int epa_a, epa_b, epa_c, access_per_vector;
  /* conv part */
  int ndim, op_type, mask_sparse, increment_k_first, dynamic_mask, is_int8_inference;
};

static void fill_gemm(tv::gemm::GemmAlgoDesp &d, const ref_desp_fields *f, const char *algo) {
  d.dtype_a = f->dtype_a;
  d.dtype_b = f->dtype_b;
  d.dtype_c = f->dtype_c;
  d.dacc = f->dacc;
  d.dcomp = f->dcomp;
  d.trans_a_set(f->trans_a);
  d.trans_b_set(f->trans_b);
  d.trans_c_set(f->trans_c);
  for (int i = 0; i < 3; ++i) {
    d.tile_shape[i] = f->tile_shape[i];
    d.warp_tile_shape[i] = f->warp_tile_shape[i];
    d.tensorop[i] = f->tensorop[i];
  }
  d.num_stage = f->num_stage;
  d.split_k_serial_set(f->split_k_serial);
  d.split_k_parallel_set(f->split_k_parallel);
  d.shuffle_type = tv::gemm::ShuffleStrideType(f->shuffle_type);
  d.element_per_access_a = f->epa_a;
  d.element_per_access_b = f->epa_b;
  d.element_per_access_c = f->epa_c;
  d.access_per_vector = f->access_per_vector;
  d.algo = algo;
}

static tv::gemm::ConvAlgoDesp make_conv(const ref_desp_fields *f, const char *algo) {
  tv::gemm::ConvAlgoDesp d(f->ndim, tv::gemm::ConvOpType(f->op_type));
  fill_gemm(d, f, algo);
  d.mask_sparse = f->mask_sparse;
  d.increment_k_first = f->increment_k_first;
  d.dynamic_mask = f->dynamic_mask;
  d.is_int8_inference = f->is_int8_inference;
  return d;
}

int ref_gemm_desp_repr(const ref_desp_fields *f, const char *algo, char *buf, int buflen) {
  try {
    tv::gemm::GemmAlgoDesp d;
    fill_gemm(d, f, algo);
    std::string s = d.__repr__();
    std::strncpy(buf, s.c_str(), buflen - 1);
    buf[buflen - 1] = 0;
    return 0;
  } catch (std::exception &) {
    return 1;
  }
}

int ref_conv_desp_repr(const ref_desp_fields *f, const char *algo, char *buf, int buflen) {
  try {
    auto d = make_conv(f, algo);
    std::string s = d.__repr__();
    std::strncpy(buf, s.c_str(), buflen - 1);
    buf[buflen - 1] = 0;
    return 0;
  } catch (std::exception &) {
    return 1;
  }
}

int ref_gemm_desp_supported(const ref_desp_fields *f, int m, int n, int k) {
  tv::gemm::GemmAlgoDesp d;
  fill_gemm(d, f, "x");
  return d.supported(m, n, k) ? 1 : 0;
}

int ref_conv_desp_supported(const ref_desp_fields *f, int m, int n, int k, int C, int K,
                            int mask_width) {
  auto d = make_conv(f, "x");
  return d.supported(m, n, k, C, K, mask_width) ? 1 : 0;
}

int ref_gemm_workspace(const ref_desp_fields *f, int m, int n, int k, int split_k) {
  tv::gemm::GemmAlgoDesp d;
  fill_gemm(d, f, "x");
  return d.query_workspace_size(m, n, k, split_k);
}

int ref_conv_workspace(const ref_desp_fields *f, int m, int n, int k, int split_k, int kv) {
  auto d = make_conv(f, "x");
  return d.query_conv_workspace_size(m, n, k, split_k, kv);
}

} // extern "C"
