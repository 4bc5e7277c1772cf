/*
 * Recipe source for oracle/_ref/libref_device.so (TEST INFRASTRUCTURE ONLY; needs a GPU to run).
 *
 * Instantiates, as DEVICE code for sm_100a, the reference's own epilogue arithmetic from the
 * headers where they lie in the reference tree (-I<reference>/include) and runs it on caller
 * data, so the CPU oracle's restatement of the two output operators can be checked bit for bit
 * against what the reference's kernels compute on this GPU.  Nothing is copied from the
 * reference: this file includes its headers and calls its functors in the order its output
 * operators prescribe.
 *
 *   int8 inference   cumm/gemm/output_op/linear.py:279-360 (Int8Inference, scale_bias = False):
 *       NumericArrayConverter<float, int32_t, N>   accumulator -> float
 *       multiply_add<array<float, N>>              scale * acc + bias        (functional.h:225-229,618-640)
 *       NumericArrayConverter<float, int8_t, N>    source -> float            (when beta != 0)
 *       multiply_add                               beta * source + t
 *       activation                                 maximum<array<float, N>> for ReLU (gemmmath/__init__.py:151-216)
 *       NumericArrayConverter<int8_t, float, N>    float -> int -> packed saturating int8
 *                                                  (numeric_convert.h:100,1107-1138,2164-2186)
 *     N = 16 = 128 bit / 8 bit, the access width of the tensor-op int8 kernels
 *     (cumm/gemm/algospec/turing.py:356); N > 1, so the operator's own clamp is not compiled in.
 *   fp16 linear combination   cumm/gemm/output_op/linear.py:105-144:
 *       NumericArrayConverter<float, half_t, N> source, <float, float, N> accumulator,
 *       multiplies (beta * source), multiply_add (alpha * acc + that), activation,
 *       NumericArrayConverter<half_t, float, N>;  without a source: multiplies (alpha * acc).
 *     N = 8.
 * LeakyReLU and Sigmoid are generated code in the reference (no header to instantiate) and are
 * not covered here.
 */
#include <tensorview/gemm/dtypes/all.h>
#include <tensorview/gemm/math/all.h>
#include <cstdint>
#include <cuda_runtime.h>

namespace {

constexpr auto kRound = tv::gemm::FloatRoundStyle::round_to_nearest;

template <int N>
__global__ void requant_kernel(long long n_vec, int width, const int32_t *acc, const float *scale, const float *bias,
                               float beta, const int8_t *src, int act_type, int8_t *out) {
  using FragF = tv::array<float, N>;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_vec)
    return;
  const long long e0 = i * N;
  const int col0 = (int)(e0 % width);
  tv::array<int32_t, N> a;
  FragF sc, bi;
  for (int j = 0; j < N; ++j) {
    a[j] = acc[e0 + j];
    sc[j] = scale[col0 + j];
    bi[j] = bias[col0 + j];
  }
  tv::gemm::NumericArrayConverter<float, int32_t, N, kRound> accumulator_converter;
  FragF converted = accumulator_converter(a);
  tv::math::multiply_add<FragF> mul_add;
  FragF t = mul_add(sc, converted, bi);
  if (src != nullptr) {
    tv::array<int8_t, N> s;
    for (int j = 0; j < N; ++j)
      s[j] = src[e0 + j];
    tv::gemm::NumericArrayConverter<float, int8_t, N, kRound> source_converter;
    FragF cs = source_converter(s);
    t = mul_add(beta, cs, t);
  }
  if (act_type == 1) {
    tv::math::maximum<FragF> max_op;
    t = max_op(t, 0.f);
  }
  tv::gemm::NumericArrayConverter<int8_t, float, N, kRound> destination_converter;
  tv::array<int8_t, N> r = destination_converter(t);
  for (int j = 0; j < N; ++j)
    out[e0 + j] = r[j];
}

template <int N>
__global__ void lincomb_kernel(long long n_vec, const float *acc, float alpha, float beta, const uint16_t *src,
                               int act_type, uint16_t *out) {
  using FragF = tv::array<float, N>;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_vec)
    return;
  const long long e0 = i * N;
  FragF a;
  for (int j = 0; j < N; ++j)
    a[j] = acc[e0 + j];
  tv::gemm::NumericArrayConverter<float, float, N, kRound> accumulator_converter;
  FragF converted = accumulator_converter(a);
  tv::math::multiplies<FragF> mul;
  FragF t;
  if (src != nullptr) {
    tv::array<tv::half_t, N> s;
    for (int j = 0; j < N; ++j)
      s[j] = tv::half_t::bitcast(src[e0 + j]);
    tv::gemm::NumericArrayConverter<float, tv::half_t, N, kRound> source_converter;
    FragF cs = source_converter(s);
    tv::math::multiply_add<FragF> mul_add;
    t = mul(beta, cs);
    t = mul_add(alpha, converted, t);
  } else {
    t = mul(alpha, converted);
  }
  if (act_type == 1) {
    tv::math::maximum<FragF> max_op;
    t = max_op(t, 0.f);
  }
  tv::gemm::NumericArrayConverter<tv::half_t, float, N, kRound> destination_converter;
  tv::array<tv::half_t, N> r = destination_converter(t);
  for (int j = 0; j < N; ++j)
    out[e0 + j] = r[j].raw();
}

struct DevBuf {
  void *p = nullptr;
  ~DevBuf() {
    if (p)
      cudaFree(p);
  }
  int up(const void *host, size_t bytes) {
    if (cudaMalloc(&p, bytes ? bytes : 1) != cudaSuccess)
      return 1;
    if (host && bytes && cudaMemcpy(p, host, bytes, cudaMemcpyHostToDevice) != cudaSuccess)
      return 1;
    return 0;
  }
};

} // namespace

extern "C" {

/* All pointers are HOST pointers; n must be a multiple of 16 and of `width` (scale and bias
 * hold `width` entries, element e uses column e % width); src may be null (no beta term).
 * Returns 0 on success, a cudaError_t otherwise. */
int ref_dev_requant_s8(long long n, int width, const int32_t *acc, const float *scale, const float *bias, float beta,
                       const int8_t *src, int act_type, int8_t *out) {
  if (n <= 0 || n % 16 || width % 16 || n % width)
    return -1;
  DevBuf d_acc, d_scale, d_bias, d_src, d_out;
  if (d_acc.up(acc, n * 4) || d_scale.up(scale, width * 4) || d_bias.up(bias, width * 4) || d_out.up(nullptr, n) ||
      (src && d_src.up(src, n)))
    return (int)cudaGetLastError();
  const long long n_vec = n / 16;
  requant_kernel<16><<<(unsigned)((n_vec + 255) / 256), 256>>>(
      n_vec, width, (const int32_t *)d_acc.p, (const float *)d_scale.p, (const float *)d_bias.p, beta,
      src ? (const int8_t *)d_src.p : nullptr, act_type, (int8_t *)d_out.p);
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess)
    e = cudaMemcpy(out, d_out.p, n, cudaMemcpyDeviceToHost);
  return (int)e;
}

/* fp16 linear combination; src / out are raw fp16 bit patterns; n a multiple of 8. */
int ref_dev_lincomb_f16(long long n, const float *acc, float alpha, float beta, const uint16_t *src, int act_type,
                        uint16_t *out) {
  if (n <= 0 || n % 8)
    return -1;
  DevBuf d_acc, d_src, d_out;
  if (d_acc.up(acc, n * 4) || d_out.up(nullptr, n * 2) || (src && d_src.up(src, n * 2)))
    return (int)cudaGetLastError();
  const long long n_vec = n / 8;
  lincomb_kernel<8><<<(unsigned)((n_vec + 255) / 256), 256>>>(n_vec, (const float *)d_acc.p, alpha, beta,
                                                            src ? (const uint16_t *)d_src.p : nullptr, act_type,
                                                            (uint16_t *)d_out.p);
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess)
    e = cudaMemcpy(out, d_out.p, n * 2, cudaMemcpyDeviceToHost);
  return (int)e;
}

} // extern "C"
