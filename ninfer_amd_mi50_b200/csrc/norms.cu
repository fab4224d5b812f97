// Row-wise kernels beside those of elementwise.cu: a layer norm (mean taken off, weight, no
// bias) fused with the residual sum; an RMS norm of a column slice; the gated RMS norm in
// equal parts that follows a state-space mixer; a vector added to every row of the stream; a
// sigmoid gate; rows gathered in the experts' order and scaled by their routing weight.
//
// All statistics are float32 whatever the activations' type.  The layer norm's variance is the
// mean of the squared deviations from the mean (two passes over a row kept in shared memory),
// not E[x^2] - mean^2.
#define NF_CHAIN_CLASS 2
#include "common.cuh"

namespace nf {

// h[t] += delta[t] (if delta); out[t] = (h[t] - mean) * rsqrt(var + eps) * w.
// With `rows`, row r reads h[rows[r]] / delta[rows[r]], writes out[r] and leaves h alone.
// With `y`, delta[t] is the routed experts' sum that was left pending,
// sum_j wts[t, j] * y[inv[t * k + j]] (j ascending; wts null: unit weights), rounded to T as the
// separate combine kernel rounds it, so both ways give the same bits.
// VEC: the row's width is a multiple of 4 and every operand's rows start on 16 bytes (8 for bfloat16): a thread
// owns runs of four consecutive elements and moves each run in one access.  Which elements a thread owns, and the
// order in which it adds them up, is the same whether the sum that is added comes from `delta` or from `y`.
template <typename T, bool GATHER, bool VEC>
__global__ void add_layernorm_kernel(float* __restrict__ h, const T* __restrict__ delta,
                                     const int* __restrict__ rows, const float* __restrict__ w,
                                     float eps, T* __restrict__ out, int hidden, const T* __restrict__ y,
                                     const int* __restrict__ inv, const float* __restrict__ wts, int k) {
  extern __shared__ __align__(16) float row[];      // [hidden]
  __shared__ float red[33];
  const int r = blockIdx.x;
  chain_release_if_small();
  chain_wait(h, delta, rows, y, inv, wts);
  const int src = GATHER ? rows[r] : r;
  float* hr = h + (size_t)src * hidden;
  const T* dr = delta ? delta + (size_t)src * hidden : nullptr;
  T* o = out + (size_t)r * hidden;
  constexpr int W = VEC ? 4 : 1;
  const int units = hidden / W;
  float s = 0.f;
  for (int u = threadIdx.x; u < units; u += blockDim.x) {
    const int i = u * W;
    float v[W];
    if constexpr (VEC) {
      const float4 hv = *reinterpret_cast<const float4*>(hr + i);
      v[0] = hv.x; v[1] = hv.y; v[2] = hv.z; v[3] = hv.w;
    } else {
      v[0] = hr[i];
    }
    if (y) {
      float acc[W];
#pragma unroll
      for (int e = 0; e < W; ++e) acc[e] = 0.f;
      for (int j = 0; j < k; ++j) {
        const float wt = wts ? wts[(size_t)src * k + j] : 1.f;
        const T* yr = y + (size_t)inv[(size_t)src * k + j] * hidden + i;
        float yv[W];
        if constexpr (VEC) load4(yr, yv); else yv[0] = to_float(yr[0]);
#pragma unroll
        for (int e = 0; e < W; ++e) acc[e] += wt * yv[e];
      }
#pragma unroll
      for (int e = 0; e < W; ++e) v[e] += to_float(from_float<T>(acc[e]));
    } else if (dr) {
      float dv[W];
      if constexpr (VEC) load4(dr + i, dv); else dv[0] = to_float(dr[i]);
#pragma unroll
      for (int e = 0; e < W; ++e) v[e] += dv[e];
    }
    if (!GATHER && (y || dr)) {
      if constexpr (VEC) *reinterpret_cast<float4*>(hr + i) = make_float4(v[0], v[1], v[2], v[3]);
      else hr[i] = v[0];
    }
#pragma unroll
    for (int e = 0; e < W; ++e) { row[i + e] = v[e]; s += v[e]; }
  }
  const float mean = block_sum(s, red) / (float)hidden;
  float ss = 0.f;
  for (int u = threadIdx.x; u < units; u += blockDim.x) {
#pragma unroll
    for (int e = 0; e < W; ++e) {
      const float d = row[u * W + e] - mean;
      ss += d * d;
    }
  }
  const float rstd = rsqrtf(block_sum(ss, red) / (float)hidden + eps);
  for (int u = threadIdx.x; u < units; u += blockDim.x) {
    const int i = u * W;
    if constexpr (VEC) {
      const float4 wv = *reinterpret_cast<const float4*>(w + i);
      const float ov[4] = {(row[i] - mean) * rstd * wv.x, (row[i + 1] - mean) * rstd * wv.y,
                           (row[i + 2] - mean) * rstd * wv.z, (row[i + 3] - mean) * rstd * wv.w};
      store4(o + i, ov);
    } else {
      o[i] = from_float<T>((row[i] - mean) * rstd * w[i]);
    }
  }
}

// out[t, 0:n] = x[t, col0:col0+n] * rsqrt(mean(x^2) + eps) * w   (w may be null: weight 1)
template <typename T>
__global__ void rms_norm_slice_kernel(const T* __restrict__ x, int ldx, int col0, int n,
                                      const float* __restrict__ w, float eps, T* __restrict__ out, int ldo) {
  __shared__ float red[33];
  const int t = blockIdx.x;
  chain_release_if_small();
  chain_wait(x);
  const T* xr = x + (size_t)t * ldx + col0;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = to_float(xr[i]);
    ss += v * v;
  }
  const float inv = rsqrtf(block_sum(ss, red) / (float)n + eps);
  T* o = out + (size_t)t * ldo;
  for (int i = threadIdx.x; i < n; i += blockDim.x)
    o[i] = from_float<T>(to_float(xr[i]) * inv * (w ? w[i] : 1.f));
}

// g = y * silu(z); each of `parts` equal parts of a row over its own root mean square; times w.
// y float32 [T, inner]; z = zsrc[t, zcol0 + i]; out [T, inner].
template <typename T>
__global__ void gated_group_rmsnorm_kernel(const float* __restrict__ y, const T* __restrict__ zsrc, int ldz,
                                           int zcol0, const float* __restrict__ w, float eps,
                                           T* __restrict__ out, int inner, int parts) {
  extern __shared__ float row[];      // [inner / parts]
  __shared__ float red[33];
  const int t = blockIdx.x, part = blockIdx.y;
  const int n = inner / parts, c0 = part * n;
  chain_release_if_small();
  chain_wait(y, zsrc);
  const float* yr = y + (size_t)t * inner + c0;
  const T* zr = zsrc + (size_t)t * ldz + zcol0 + c0;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float z = to_float(zr[i]);
    const float g = yr[i] * (z / (1.f + expf(-z)));
    row[i] = g;
    ss += g * g;
  }
  const float inv = rsqrtf(block_sum(ss, red) / (float)n + eps);
  T* o = out + (size_t)t * inner + c0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) o[i] = from_float<T>(row[i] * inv * w[c0 + i]);
}

__global__ void add_row_vector_kernel(float* __restrict__ h, const float* __restrict__ vec, int hidden) {
  chain_wait(h);
  float* hr = h + (size_t)blockIdx.x * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) hr[i] += vec[i];
}

// out[t, hd * n + i] = v[hd, t, i] * sigmoid(g[t, gcol0 + hd * n + i]):  v is laid out head by head
// ([heads, T, n], what a batched product over heads leaves), out token by token.
template <typename T>
__global__ void heads_sigmoid_gate_kernel(const T* __restrict__ v, const T* __restrict__ g, int ldg, int gcol0,
                                          T* __restrict__ out, int rows, int heads, int n) {
  const int t = blockIdx.x;
  chain_wait(v, g);
  const int width = heads * n;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const int hd = c / n, i = c - hd * n;
    const float gv = to_float(g[(size_t)t * ldg + gcol0 + c]);
    const float vv = to_float(v[((size_t)hd * rows + t) * n + i]);
    out[(size_t)t * width + c] = from_float<T>(vv * (1.f / (1.f + expf(-gv))));
  }
}

// out[p] = scale[order[p]] * x[order[p] / div]: the tokens in the experts' order, each times the
// weight of its (token, choice) pair.  VEC: 16 bytes a thread and step (rows are 16-byte aligned).
template <typename T, bool VEC>
__global__ void scale_gather_rows_kernel(const T* __restrict__ x, const int* __restrict__ order, int div,
                                         const float* __restrict__ scale, T* __restrict__ out, int hidden,
                                         int n_pairs) {
  constexpr int VE = 16 / (int)sizeof(T);
  const int p = blockIdx.x;
  chain_wait(x, order, scale);
  const int pair = order[p];
  T* o = out + (size_t)p * hidden;
  const bool bad = pair < 0 || pair >= n_pairs;
  const float s = bad ? 0.f : scale[pair];
  const T* xr = x + (size_t)(bad ? 0 : pair / div) * hidden;
  if (VEC) {
    for (int i = threadIdx.x * VE; i < hidden; i += blockDim.x * VE) {
      float v[8];
      if (sizeof(T) == 2) load8(reinterpret_cast<const __nv_bfloat16*>(xr) + i, v);
      else load4(reinterpret_cast<const float*>(xr) + i, v);
#pragma unroll
      for (int e = 0; e < VE; ++e) v[e] = bad ? 0.f : s * v[e];
      if (sizeof(T) == 2) {
        store4(reinterpret_cast<__nv_bfloat16*>(o) + i, v);
        store4(reinterpret_cast<__nv_bfloat16*>(o) + i + 4, v + 4);
      } else {
        store4(reinterpret_cast<float*>(o) + i, v);
      }
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_float<T>(bad ? 0.f : s * to_float(xr[i]));
  }
}

}  // namespace nf

using namespace nf;

extern "C" int nf_add_layernorm(float* h, const void* delta, const int* rows, const float* w, float eps, void* out,
                                int R, int hidden, int dtype, const void* y, const int* inv, const float* wts, int k,
                                cudaStream_t stream) {
  if (R == 0) return 0;
  NF_REQUIRE(R > 0 && hidden > 0, "add_layernorm: bad sizes R=%d hidden=%d", R, hidden);
  const size_t smem = (size_t)hidden * sizeof(float);
  NF_REQUIRE(smem <= 160 * 1024, "add_layernorm: a row of %d does not fit shared memory", hidden);
  const int threads = hidden >= 2048 ? 512 : 256;
#define NF_LN(T, G, V)                                                                                      \
  do {                                                                                                      \
    if (smem > 48 * 1024)                                                                                   \
      cudaFuncSetAttribute(add_layernorm_kernel<T, G, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    launch_chained(add_layernorm_kernel<T, G, V>, dim3(R), dim3(threads), smem, stream, h, (const T*)delta, rows, w, \
                   eps, (T*)out, hidden, (const T*)y, inv, wts, k);                                         \
  } while (0)
#define NF_LN_V(T, G) do { if (vec) NF_LN(T, G, true); else NF_LN(T, G, false); } while (0)
  const size_t tsize = dtype == kF32 ? 4 : 2;
  const bool vec = hidden % 4 == 0 && (uintptr_t)h % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)out % (4 * tsize) == 0 &&
                   (!delta || (uintptr_t)delta % (4 * tsize) == 0) && (!y || (uintptr_t)y % (4 * tsize) == 0);
  if (dtype == kF32) { if (rows) NF_LN_V(float, true); else NF_LN_V(float, false); }
  else { if (rows) NF_LN_V(__nv_bfloat16, true); else NF_LN_V(__nv_bfloat16, false); }
#undef NF_LN_V
#undef NF_LN
  return check_launch("add_layernorm");
}

extern "C" int nf_rms_norm_slice(const void* x, int ldx, int col0, int n, const float* w, float eps, void* out,
                                 int ldo, int R, int dtype, cudaStream_t stream) {
  if (R == 0) return 0;
  NF_REQUIRE(R > 0 && n > 0 && col0 >= 0 && col0 + n <= ldx && ldo >= n, "rms_norm_slice: bad sizes");
  if (dtype == kF32)
    launch_chained(rms_norm_slice_kernel<float>, dim3(R), dim3(128), 0, stream, (const float*)x, ldx, col0, n, w, eps, (float*)out, ldo);
  else
    launch_chained(rms_norm_slice_kernel<__nv_bfloat16>, dim3(R), dim3(128), 0, stream, (const __nv_bfloat16*)x, ldx, col0, n, w, eps, (__nv_bfloat16*)out, ldo);
  return check_launch("rms_norm_slice");
}

extern "C" int nf_gated_group_rmsnorm(const float* y, const void* z, int ldz, int zcol0, const float* w, float eps,
                                      void* out, int R, int inner, int parts, int dtype, cudaStream_t stream) {
  if (R == 0) return 0;
  NF_REQUIRE(R > 0 && inner > 0 && parts > 0 && inner % parts == 0, "gated_group_rmsnorm: %d does not split into %d parts", inner, parts);
  const size_t smem = (size_t)(inner / parts) * sizeof(float);
  NF_REQUIRE(smem <= 160 * 1024, "gated_group_rmsnorm: a part of %d does not fit shared memory", inner / parts);
#define NF_GN(T)                                                                                               \
  do {                                                                                                         \
    if (smem > 48 * 1024)                                                                                      \
      cudaFuncSetAttribute(gated_group_rmsnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    launch_chained(gated_group_rmsnorm_kernel<T>, dim3(R, parts), dim3(256), smem, stream, y, (const T*)z, ldz, zcol0, \
                   w, eps, (T*)out, inner, parts);                                                             \
  } while (0)
  if (dtype == kF32) NF_GN(float); else NF_GN(__nv_bfloat16);
#undef NF_GN
  return check_launch("gated_group_rmsnorm");
}

extern "C" int nf_add_row_vector(float* h, const float* vec, int R, int hidden, cudaStream_t stream) {
  if (R == 0) return 0;
  launch_chained(add_row_vector_kernel, dim3(R), dim3(256), 0, stream, h, vec, hidden);
  return check_launch("add_row_vector");
}

extern "C" int nf_heads_sigmoid_gate(const void* v, const void* g, int ldg, int gcol0, void* out, int R, int heads,
                                     int n, int dtype, cudaStream_t stream) {
  if (R == 0) return 0;
  NF_REQUIRE(heads > 0 && n > 0 && gcol0 >= 0 && gcol0 + heads * n <= ldg, "heads_sigmoid_gate: bad sizes");
  if (dtype == kF32)
    launch_chained(heads_sigmoid_gate_kernel<float>, dim3(R), dim3(256), 0, stream, (const float*)v, (const float*)g, ldg, gcol0, (float*)out, R, heads, n);
  else
    launch_chained(heads_sigmoid_gate_kernel<__nv_bfloat16>, dim3(R), dim3(256), 0, stream, (const __nv_bfloat16*)v, (const __nv_bfloat16*)g, ldg, gcol0, (__nv_bfloat16*)out, R, heads, n);
  return check_launch("heads_sigmoid_gate");
}

extern "C" int nf_scale_gather_rows(const void* x, const int* order, int div, const float* scale, void* out,
                                    int n_rows, int hidden, int dtype, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NF_REQUIRE(div > 0 && hidden > 0, "scale_gather_rows: bad sizes");
  const int threads = hidden >= 2048 ? 256 : 128;
  if (dtype == kF32) {
    if (hidden % 4 == 0) launch_chained(scale_gather_rows_kernel<float, true>, dim3(n_rows), dim3(threads), 0, stream, (const float*)x, order, div, scale, (float*)out, hidden, n_rows);
    else launch_chained(scale_gather_rows_kernel<float, false>, dim3(n_rows), dim3(256), 0, stream, (const float*)x, order, div, scale, (float*)out, hidden, n_rows);
  } else {
    if (hidden % 8 == 0) launch_chained(scale_gather_rows_kernel<__nv_bfloat16, true>, dim3(n_rows), dim3(threads), 0, stream, (const __nv_bfloat16*)x, order, div, scale, (__nv_bfloat16*)out, hidden, n_rows);
    else launch_chained(scale_gather_rows_kernel<__nv_bfloat16, false>, dim3(n_rows), dim3(256), 0, stream, (const __nv_bfloat16*)x, order, div, scale, (__nv_bfloat16*)out, hidden, n_rows);
  }
  return check_launch("scale_gather_rows");
}

// ---------------------------------------------------------------------------------------------
// Norm on a sublayer's output: h[t] += ls * (d / rms(d)) * w with d = delta[t] (+ bias), and, if
// `out`, out[t] = h[t] in the engine's type (the next sublayer's input).  delta may be float32 or
// the engine's type; the sum, the mean of squares and the products are float32.
// ---------------------------------------------------------------------------------------------
namespace nf {

template <typename TD, typename TO>
__global__ void scaled_norm_add_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                       const float* __restrict__ bias, const float* __restrict__ w,
                                       const float* __restrict__ ls, float eps, TO* __restrict__ out, int hidden) {
  __shared__ float red[33];
  const int r = blockIdx.x;
  chain_release_if_small();
  chain_wait(h, delta);
  float* hr = h + (size_t)r * hidden;
  const TD* dr = delta + (size_t)r * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float d = to_float(dr[i]) + (bias ? bias[i] : 0.f);
    ss += d * d;
  }
  const float inv = rsqrtf(block_sum(ss, red) / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float d = to_float(dr[i]) + (bias ? bias[i] : 0.f);
    float v = d * inv * w[i];
    if (ls) v *= ls[i];
    v += hr[i];
    hr[i] = v;
    if (out) out[(size_t)r * hidden + i] = from_float<TO>(v);
  }
}

// The same with the routed experts' pending sum as the sublayer's output:
// d = sum_j wts[t, j] * y[inv[t * k + j]] (j ascending; wts null: unit weights), rounded to T as the separate
// combine kernel rounds it, so both ways give the same bits.  The row is kept in shared memory.
template <typename T, typename TO>
__global__ void routed_scaled_norm_add_kernel(float* __restrict__ h, const T* __restrict__ y, const int* __restrict__ inv,
                                              const float* __restrict__ wts, int k, const float* __restrict__ w,
                                              const float* __restrict__ ls, float eps, TO* __restrict__ out, int hidden) {
  extern __shared__ float row[];      // [hidden]
  __shared__ float red[33];
  const int r = blockIdx.x;
  chain_release_if_small();
  chain_wait(h, y, inv, wts);
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < k; ++j) {
      const int p = inv[r * k + j];
      acc += (wts ? wts[r * k + j] : 1.f) * to_float(y[(size_t)p * hidden + i]);
    }
    const float d = to_float(from_float<T>(acc));
    row[i] = d;
    ss += d * d;
  }
  const float invr = rsqrtf(block_sum(ss, red) / (float)hidden + eps);
  float* hr = h + (size_t)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = row[i] * invr * w[i];
    if (ls) v *= ls[i];
    v += hr[i];
    hr[i] = v;
    if (out) out[(size_t)r * hidden + i] = from_float<TO>(v);
  }
}

// out[t] = (1 / n) * sum_m (x_m[t] / rms(x_m[t])) * w_m: the mean of several mixers' outputs, each
// first over its own root mean square and times its own weight.  out is float32.
struct NormedInputs {
  const void* x[4];
  const float* w[4];
  int n;
};

template <typename T>
__global__ void mean_of_rmsnorms_kernel(NormedInputs in, float eps, float* __restrict__ out, int hidden) {
  __shared__ float red[33];
  const int r = blockIdx.x;
  chain_release_if_small();
  chain_wait();
  float inv[4];
  for (int m = 0; m < in.n; ++m) {
    const T* xr = reinterpret_cast<const T*>(in.x[m]) + (size_t)r * hidden;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const float v = to_float(xr[i]);
      ss += v * v;
    }
    inv[m] = rsqrtf(block_sum(ss, red) / (float)hidden + eps);
  }
  const float share = 1.f / (float)in.n;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float s = 0.f;
    for (int m = 0; m < in.n; ++m)
      s += to_float(reinterpret_cast<const T*>(in.x[m])[(size_t)r * hidden + i]) * inv[m] * in.w[m][i];
    out[(size_t)r * hidden + i] = s * share;
  }
}

// out[t, c] = y[t, c] / rms(part of c) * w[c] * act(z[t, zcol0 + c]): an RMS norm in `parts` equal
// parts of a row (w null: no weight), then a gate.  act 0: silu, 1: sigmoid.  y is float32; z is of the
// output's type or float32 sums.
template <typename T, typename TZ = T>
__global__ void group_rmsnorm_gate_kernel(const float* __restrict__ y, const TZ* __restrict__ zsrc, int ldz, int zcol0,
                                          const float* __restrict__ w, float eps, T* __restrict__ out, int inner,
                                          int parts, int act) {
  __shared__ float red[33];
  const int t = blockIdx.x, part = blockIdx.y;
  const int n = inner / parts, c0 = part * n;
  chain_release_if_small();
  chain_wait(y, zsrc);
  const float* yr = y + (size_t)t * inner + c0;
  const TZ* zr = zsrc + (size_t)t * ldz + zcol0 + c0;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) ss += yr[i] * yr[i];
  const float inv = rsqrtf(block_sum(ss, red) / (float)n + eps);
  T* o = out + (size_t)t * inner + c0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float z = to_float(zr[i]);
    const float sg = 1.f / (1.f + expf(-z));
    const float gate = act == 1 ? sg : z * sg;
    o[i] = from_float<T>(yr[i] * inv * (w ? w[c0 + i] : 1.f) * gate);
  }
}

static inline int norm_threads(int n) {
  int t = 32;
  while (t < n && t < 512) t <<= 1;
  return t;
}

}  // namespace nf

// delta_dtype: 0 float32, 1 bfloat16; out (may be null) has out_dtype.
extern "C" int nf_scaled_norm_add(float* h, const void* delta, int delta_dtype, const float* bias, const float* w,
                                  const float* ls, float eps, void* out, int out_dtype, int R, int hidden,
                                  cudaStream_t stream) {
  if (R == 0) return 0;
  NF_REQUIRE(R > 0 && hidden > 0 && h && delta && w, "scaled_norm_add: bad arguments R=%d hidden=%d", R, hidden);
  const dim3 grid(R), block(norm_threads(hidden));
#define NF_SNA(TD, TO) \
  launch_chained(scaled_norm_add_kernel<TD, TO>, grid, block, 0, stream, h, (const TD*)delta, bias, w, ls, eps, (TO*)out, hidden)
  if (delta_dtype == kF32) { if (out_dtype == kF32) NF_SNA(float, float); else NF_SNA(float, __nv_bfloat16); }
  else { if (out_dtype == kF32) NF_SNA(__nv_bfloat16, float); else NF_SNA(__nv_bfloat16, __nv_bfloat16); }
#undef NF_SNA
  return check_launch("scaled_norm_add");
}

// y [pairs, hidden] of `dtype`, inv int32 [R * k], wts float32 [R, k] or null; out (may be null) has out_dtype.
extern "C" int nf_routed_scaled_norm_add(float* h, const void* y, const int* inv, const float* wts, int k, int dtype,
                                         const float* w, const float* ls, float eps, void* out, int out_dtype, int R,
                                         int hidden, cudaStream_t stream) {
  if (R == 0) return 0;
  NF_REQUIRE(R > 0 && hidden > 0 && k > 0 && h && y && inv && w, "routed_scaled_norm_add: bad arguments");
  const size_t smem = (size_t)hidden * sizeof(float);
  NF_REQUIRE(smem <= 160 * 1024, "routed_scaled_norm_add: a row of %d does not fit shared memory", hidden);
  const dim3 grid(R), block(norm_threads(hidden));
#define NF_RSNA(T, TO)                                                                                              \
  do {                                                                                                              \
    if (smem > 48 * 1024)                                                                                           \
      cudaFuncSetAttribute(routed_scaled_norm_add_kernel<T, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    launch_chained(routed_scaled_norm_add_kernel<T, TO>, grid, block, smem, stream, h, (const T*)y, inv, wts, k, w, ls, eps, \
                   (TO*)out, hidden);                                                                               \
  } while (0)
  if (dtype == kF32) NF_RSNA(float, float);
  else if (out_dtype == kF32) NF_RSNA(__nv_bfloat16, float);
  else NF_RSNA(__nv_bfloat16, __nv_bfloat16);
#undef NF_RSNA
  return check_launch("routed_scaled_norm_add");
}

extern "C" int nf_mean_of_rmsnorms(const void* const* xs, const float* const* ws, int n, float eps, float* out, int R,
                                   int hidden, int dtype, cudaStream_t stream) {
  if (R == 0) return 0;
  NF_REQUIRE(n >= 1 && n <= 4 && R > 0 && hidden > 0, "mean_of_rmsnorms: %d inputs (1 to 4), R=%d hidden=%d", n, R, hidden);
  NormedInputs in;
  in.n = n;
  for (int m = 0; m < 4; ++m) { in.x[m] = m < n ? xs[m] : nullptr; in.w[m] = m < n ? ws[m] : nullptr; }
  if (dtype == kF32) launch_chained(mean_of_rmsnorms_kernel<float>, dim3(R), dim3(norm_threads(hidden)), 0, stream, in, eps, out, hidden);
  else launch_chained(mean_of_rmsnorms_kernel<__nv_bfloat16>, dim3(R), dim3(norm_threads(hidden)), 0, stream, in, eps, out, hidden);
  return check_launch("mean_of_rmsnorms");
}

// z_dtype: the gate's type, the output's or float32.
extern "C" int nf_group_rmsnorm_gate(const float* y, const void* z, int ldz, int zcol0, const float* w, float eps,
                                     void* out, int R, int inner, int parts, int act, int dtype, int z_dtype,
                                     cudaStream_t stream) {
  if (R == 0) return 0;
  NF_REQUIRE(R > 0 && inner > 0 && parts > 0 && inner % parts == 0 && parts <= 65535,
             "group_rmsnorm_gate: %d does not split into %d parts", inner, parts);
  NF_REQUIRE(act == 0 || act == 1, "group_rmsnorm_gate: gate %d (0 silu, 1 sigmoid)", act);
  NF_REQUIRE(z_dtype == dtype || z_dtype == kF32, "group_rmsnorm_gate: the gate is of the output's type or float32");
  const dim3 grid(R, parts), block(norm_threads(inner / parts));
  if (dtype == kF32) launch_chained(group_rmsnorm_gate_kernel<float>, grid, block, 0, stream, y, (const float*)z, ldz, zcol0, w, eps, (float*)out, inner, parts, act);
  else if (z_dtype == kF32) launch_chained(group_rmsnorm_gate_kernel<__nv_bfloat16, float>, grid, block, 0, stream, y, (const float*)z, ldz, zcol0, w, eps, (__nv_bfloat16*)out, inner, parts, act);
  else launch_chained(group_rmsnorm_gate_kernel<__nv_bfloat16>, grid, block, 0, stream, y, (const __nv_bfloat16*)z, ldz, zcol0, w, eps, (__nv_bfloat16*)out, inner, parts, act);
  return check_launch("group_rmsnorm_gate");
}
