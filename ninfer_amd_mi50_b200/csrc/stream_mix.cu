// Several residual streams a token (hyper-connections), and the RMS norm in groups.
//
// A token carries S streams x_0 .. x_{S-1} of `hidden` floats, stored [T, S, hidden] in float32.
// A sublayer reads u = sum_s in[s] x_s, normed; its output y then changes all streams at once:
//
//     x_t <- sum_s mix[s, t] x_s + out[t] * y            (mix is indexed [from, to])
//
// One kernel does what lies between two sublayers: it applies the previous sublayer's update
// (if there is a y), writes the streams back, forms the next sublayer's u and norms it.  The norm
// cuts the row into `groups` equal consecutive parts and divides each by its own
// sqrt(mean(part^2) + eps) before the weight multiplies.  With S = 1, in = mix = out = 1 this is the
// ordinary residual sum fused with a (grouped) RMS norm; with `in` absent u is the plain sum of the
// streams, which is what the model's last norm reads.  Everything is float32; only y and the
// normed output have the engine's type.
#include "common.cuh"

namespace nf {

constexpr int kMaxStreams = 8;

struct StreamMixParams {
  float mix[kMaxStreams * kMaxStreams];   // [from][to]
  float out[kMaxStreams];
  float in[kMaxStreams];
};

// One CTA a row.  Dynamic shared memory: u [hidden] floats, then inv [groups].
template <typename T>
__global__ void streams_mix_norm_kernel(float* __restrict__ streams, const T* __restrict__ y,
                                        const int* __restrict__ rows, const float* __restrict__ mix,
                                        const float* __restrict__ out_w, const float* __restrict__ in_w,
                                        const float* __restrict__ weight, float eps, int groups,
                                        T* __restrict__ normed, int S, int hidden, int write_back) {
  extern __shared__ float smem[];
  float* u = smem;
  float* inv = smem + hidden;
  __shared__ float c_mix[kMaxStreams * kMaxStreams], c_out[kMaxStreams], c_in[kMaxStreams];
  const int r = blockIdx.x;
  if (threadIdx.x < S * S) c_mix[threadIdx.x] = (y && mix) ? mix[threadIdx.x] : (threadIdx.x / S == threadIdx.x % S ? 1.f : 0.f);
  if (threadIdx.x < S) {
    c_out[threadIdx.x] = (y && out_w) ? out_w[threadIdx.x] : (y ? 1.f : 0.f);
    c_in[threadIdx.x] = in_w ? in_w[threadIdx.x] : 1.f;
  }
  chain_wait(streams, y);
  const int src = rows ? rows[r] : r;
  float* xr = streams + (size_t)src * S * hidden;
  const T* yr = y ? y + (size_t)src * hidden : nullptr;
  __syncthreads();
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float x[kMaxStreams];
#pragma unroll
    for (int s = 0; s < kMaxStreams; ++s) x[s] = s < S ? xr[(size_t)s * hidden + i] : 0.f;
    float acc = 0.f;
    if (yr) {
      const float yv = to_float(yr[i]);
#pragma unroll
      for (int t = 0; t < kMaxStreams; ++t) {
        if (t < S) {
          float v = 0.f;
#pragma unroll
          for (int s = 0; s < kMaxStreams; ++s)
            if (s < S) v = fmaf(c_mix[s * S + t], x[s], v);
          v = fmaf(c_out[t], yv, v);
          if (write_back) xr[(size_t)t * hidden + i] = v;
          acc = fmaf(c_in[t], v, acc);
        }
      }
    } else {
#pragma unroll
      for (int s = 0; s < kMaxStreams; ++s)
        if (s < S) acc = fmaf(c_in[s], x[s], acc);
    }
    u[i] = acc;
  }
  __syncthreads();
  if (!normed) return;
  // a warp a group (in turn): the group's mean of squares
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  const int gs = hidden / groups;
  for (int g = warp; g < groups; g += nwarp) {
    float ss = 0.f;
    for (int i = lane; i < gs; i += 32) {
      const float v = u[g * gs + i];
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) inv[g] = 1.f / sqrtf(ss / (float)gs + eps);
  }
  __syncthreads();
  T* o = normed + (size_t)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    o[i] = from_float<T>(u[i] * inv[i / gs] * (weight ? weight[i] : 1.f));
}

// out[t, c] = float32(table[ids[t]]) for every copy c < copies: the streams all start as the embedding.
template <typename T>
__global__ void embed_copies_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                                    int hidden, int vocab, int copies) {
  const int t = blockIdx.x;
  chain_wait();
  const int id = ids[t];
  const bool ok = id >= 0 && id < vocab;
  const T* row = table + (size_t)(ok ? id : 0) * hidden;
  float* o = out + (size_t)t * copies * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = ok ? to_float(row[i]) : 0.f;
    for (int c = 0; c < copies; ++c) o[(size_t)c * hidden + i] = v;
  }
}

// x[i] <- cap * tanh(x[i] / cap)
__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap) {
  chain_wait(x);
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

static inline int mix_threads(int n) {
  int t = 32;
  while (t < n && t < 256) t <<= 1;
  return t;
}

}  // namespace nf

using namespace nf;

// streams float32 [T, S, hidden] (updated in place when y is given and write_back is set);
// y [T, hidden] or null; rows int32 [R] or null (then R = T and row r is token r); mix [S, S],
// out_w [S], in_w [S] float32 on the device (null: identity / ones); weight [hidden] or null;
// normed [R, hidden] in `dtype` or null (then only the update is applied).
extern "C" int nf_streams_mix_norm(float* streams, const void* y, const int* rows, const float* mix,
                                   const float* out_w, const float* in_w, const float* weight, float eps,
                                   int groups, void* normed, int R, int S, int hidden, int write_back, int dtype,
                                   cudaStream_t stream) {
  if (R == 0) return 0;
  NF_REQUIRE(R > 0 && hidden > 0 && S >= 1 && S <= kMaxStreams, "streams_mix_norm: bad sizes R=%d S=%d hidden=%d (at most %d streams)", R, S, hidden, kMaxStreams);
  NF_REQUIRE(groups >= 1 && hidden % groups == 0, "streams_mix_norm: %d groups do not divide a row of %d", groups, hidden);
  NF_REQUIRE(!(rows && write_back && y), "streams_mix_norm: a call on chosen rows does not write the streams back");
  const int th = mix_threads(hidden) < 64 ? 64 : mix_threads(hidden);     // S * S <= 64 threads load the constants
  const size_t smem = (size_t)(hidden + groups) * sizeof(float);
  NF_REQUIRE(smem <= 200 * 1024, "streams_mix_norm: a row of %d does not fit shared memory", hidden);
  if (dtype == kF32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(streams_mix_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_chained(streams_mix_norm_kernel<float>, dim3(R), dim3(th), smem, stream, streams, (const float*)y, rows, mix, out_w, in_w, weight, eps, groups, (float*)normed, S, hidden, write_back);
  } else {
    if (smem > 48 * 1024) cudaFuncSetAttribute(streams_mix_norm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_chained(streams_mix_norm_kernel<__nv_bfloat16>, dim3(R), dim3(th), smem, stream, streams, (const __nv_bfloat16*)y, rows, mix, out_w, in_w, weight, eps, groups, (__nv_bfloat16*)normed, S, hidden, write_back);
  }
  return check_launch("streams_mix_norm");
}

extern "C" int nf_embed_copies(const void* table, const int* ids, float* out, int T, int hidden, int vocab,
                               int copies, int dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  NF_REQUIRE(T > 0 && hidden > 0 && vocab > 0 && copies >= 1, "embed_copies: bad sizes T=%d hidden=%d vocab=%d copies=%d", T, hidden, vocab, copies);
  if (dtype == kF32)
    launch_chained(embed_copies_kernel<float>, dim3(T), dim3(mix_threads(hidden)), 0, stream, (const float*)table, ids, out, hidden, vocab, copies);
  else
    launch_chained(embed_copies_kernel<__nv_bfloat16>, dim3(T), dim3(mix_threads(hidden)), 0, stream, (const __nv_bfloat16*)table, ids, out, hidden, vocab, copies);
  return check_launch("embed_copies");
}

extern "C" int nf_softcap(float* x, long long n, float cap, cudaStream_t stream) {
  if (n == 0) return 0;
  NF_REQUIRE(n > 0 && cap > 0.f, "softcap: bad arguments n=%lld cap=%g", n, (double)cap);
  launch_chained(softcap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, (size_t)n, cap);
  return check_launch("softcap");
}
