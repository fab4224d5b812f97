// Row-wise steps of feed-forwards that are not gated: an activation that is a polynomial of
// normed powers, the exact GELU, and the look-up of a token's experts in a table.
#include "common.cuh"

namespace nf {

// out = a N(z) + b N(z^2) + c N(z^3) + e, powers element by element, N(v) = v / sqrt(mean(v^2) + eps)
// over the row.  One CTA a row; the three means in one pass; float32 throughout, the result in T.
template <typename T>
__global__ void poly_norm_act_kernel(const float* __restrict__ z, const float* __restrict__ coef, float eps,
                                     T* __restrict__ out, int n) {
  __shared__ float red[33];
  const int r = blockIdx.x;
  chain_wait(z);
  const float* zr = z + (size_t)r * n;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = zr[i], v2 = v * v, v3 = v2 * v;
    s2 = fmaf(v, v, s2);
    s4 = fmaf(v2, v2, s4);
    s6 = fmaf(v3, v3, s6);
  }
  s2 = block_sum(s2, red);
  s4 = block_sum(s4, red);
  s6 = block_sum(s6, red);
  const float a = coef[0] / sqrtf(s2 / (float)n + eps), b = coef[1] / sqrtf(s4 / (float)n + eps),
              c = coef[2] / sqrtf(s6 / (float)n + eps), e = coef[3];
  T* o = out + (size_t)r * n;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = zr[i], v2 = v * v;
    o[i] = from_float<T>(a * v + b * v2 + c * (v2 * v) + e);
  }
}

// x <- 0.5 x (1 + erf(x / sqrt 2)), in place
template <typename T>
__global__ void gelu_erf_kernel(T* __restrict__ x, size_t n) {
  chain_wait(x);
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const float v = to_float(x[i]);
    x[i] = from_float<T>(0.5f * v * (1.f + erff(v * 0.70710678118654752440f)));
  }
}

// idx[t, j] = table[ids[t], j]: the experts of a token stand in a table by its id.  The loader has
// checked that every entry names an expert and the step that every id lies in the table; an entry
// that does not is read as expert 0 rather than followed.
__global__ void table_route_kernel(const int* __restrict__ table, const int* __restrict__ ids, int* __restrict__ idx,
                                   int T, int k, int rows, int E) {
  chain_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * k) return;
  const int id = ids[i / k];
  const int e = (id >= 0 && id < rows) ? table[(size_t)id * k + i % k] : 0;
  idx[i] = (e >= 0 && e < E) ? e : 0;
}

// out[r, i] = T(y[r, i] + bias[i]): the bias of a projection whose float32 sums were kept
template <typename T>
__global__ void add_bias_rows_kernel(const float* __restrict__ y, const float* __restrict__ bias, T* __restrict__ out,
                                     size_t total, int n) {
  chain_wait(y);
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) out[i] = from_float<T>(y[i] + bias[i % n]);
}

}  // namespace nf

using namespace nf;

extern "C" int nf_poly_norm_act(const float* z, const float* coef, float eps, void* out, int R, int n, int dtype,
                                cudaStream_t stream) {
  if (R == 0) return 0;
  NF_REQUIRE(R > 0 && n > 0, "poly_norm_act: bad sizes R=%d n=%d", R, n);
  int th = 32;
  while (th < n && th < 512) th <<= 1;
  if (dtype == kF32)
    launch_chained(poly_norm_act_kernel<float>, dim3(R), dim3(th), 0, stream, z, coef, eps, (float*)out, n);
  else
    launch_chained(poly_norm_act_kernel<__nv_bfloat16>, dim3(R), dim3(th), 0, stream, z, coef, eps, (__nv_bfloat16*)out, n);
  return check_launch("poly_norm_act");
}

extern "C" int nf_gelu_erf(void* x, long long n, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  NF_REQUIRE(n > 0, "gelu_erf: bad size %lld", n);
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (dtype == kF32)
    launch_chained(gelu_erf_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)x, (size_t)n);
  else
    launch_chained(gelu_erf_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)x, (size_t)n);
  return check_launch("gelu_erf");
}

extern "C" int nf_table_route(const int* table, const int* ids, int* idx, int T, int k, int rows, int E,
                              cudaStream_t stream) {
  if (T == 0) return 0;
  NF_REQUIRE(T > 0 && k > 0 && rows > 0 && E > 0, "table_route: bad sizes T=%d k=%d rows=%d E=%d", T, k, rows, E);
  launch_chained(table_route_kernel, dim3((T * k + 127) / 128), dim3(128), 0, stream, table, ids, idx, T, k, rows, E);
  return check_launch("table_route");
}

extern "C" int nf_add_bias_rows(const float* y, const float* bias, void* out, int R, int n, int dtype, cudaStream_t stream) {
  if (R == 0) return 0;
  NF_REQUIRE(R > 0 && n > 0, "add_bias_rows: bad sizes R=%d n=%d", R, n);
  const size_t total = (size_t)R * n;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == kF32)
    launch_chained(add_bias_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, y, bias, (float*)out, total, n);
  else
    launch_chained(add_bias_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, y, bias, (__nv_bfloat16*)out, total, n);
  return check_launch("add_bias_rows");
}
