// Grouped-query attention whose heads' scores are mixed before the softmax, over chunks, with a
// sink; and the kernel that prepares its queries, keys and values.
//
//   q, k: bias, RMS norm per head over the head's `D` numbers (one weight vector for all heads),
//         then the first `rot` dimensions turned by the position (pairs (i, i + rot/2));
//   s_g(i, j)  = (q_g(i) . k_{g / rep}(j)) * scale                      rep = H / G
//   s'_h(i, j) = sum_g talk[h, g] s_g(i, j)                             all H heads' scores of a pair meet
//   j is seen from i  iff  j <= i and (chunk == 0 or i / chunk == j / chunk)
//   p_h(i, j)  = exp(s'_h(i, j)) / (exp(sink_h) + sum_j' exp(s'_h(i, j')))
//   o_h(i)     = sum_j p_h(i, j) v_{h / rep}(j)
//
// The cache keeps one row a token, [k: G * D | v: G * Dv] (keys as they are after norm and
// rotation), in pages of `page_size` rows; key and value sizes may differ.  Scores, the mixing,
// the softmax with its sink and the weighted sum of values are float32 whatever the cache's type.
// Keys are visited in blocks of 32 aligned to absolute positions, in ascending order, so a row's
// sums depend on its own position alone: not on how a prompt was cut, nor on its neighbours in
// the step.  One CTA serves one row with all its heads, because every head's softmax needs every
// head's scores.
#include "common.cuh"

namespace nf {

constexpr int kKeyBlock = 32;
constexpr int kMaxAcc = 16;          // outputs a thread: H * Dv <= kMaxAcc * threads

template <typename T>
__global__ void talking_attention_kernel(const T* __restrict__ q, const T* __restrict__ pages,
                                         const int* __restrict__ block_table, int bt_width,
                                         const int* __restrict__ positions, const int* __restrict__ row_seg,
                                         const int* __restrict__ row_list, const float* __restrict__ talk,
                                         const float* __restrict__ sink, T* __restrict__ out, int H, int G, int D,
                                         int Dv, int page_size, int num_pages, int chunk, float scale) {
  extern __shared__ float smem[];
  float* q_s = smem;                         // [H * D]
  float* s_raw = q_s + H * D;                // [H][32]
  float* p_s = s_raw + H * kKeyBlock;        // [H][32]
  float* m_s = p_s + H * kKeyBlock;          // [H]
  float* l_s = m_s + H;                      // [H]
  float* a_s = l_s + H;                      // [H]
  float* talk_s = a_s + H;                   // [H * H]
  __shared__ const T* vrow_s[kKeyBlock];
  const int tid = threadIdx.x, nth = blockDim.x;
  const int warp = tid >> 5, lane = tid & 31, nwarp = nth >> 5;
  const int rep = H / G;
  const int row_width = G * (D + Dv);
  for (int i = tid; i < H * H; i += nth) talk_s[i] = talk ? talk[i] : (i / H == i % H ? 1.f : 0.f);
  for (int h = tid; h < H; h += nth) {
    m_s[h] = sink ? sink[h] : -INFINITY;     // the sink counts once in the denominator: exp(sink - m) = 1
    l_s[h] = sink ? 1.f : 0.f;
  }
  chain_wait(q, pages);
  const int t = row_list ? row_list[blockIdx.x] : blockIdx.x;
  const int pos = positions[t];
  const int* bt = block_table + (size_t)row_seg[t] * bt_width;
  const T* qrow = q + (size_t)t * H * D;
  for (int i = tid; i < H * D; i += nth) q_s[i] = to_float(qrow[i]);
  const int lo = chunk > 0 ? (pos / chunk) * chunk : 0;
  float acc[kMaxAcc];
#pragma unroll
  for (int n = 0; n < kMaxAcc; ++n) acc[n] = 0.f;
  __syncthreads();

  for (int j0 = (lo / kKeyBlock) * kKeyBlock; j0 <= pos; j0 += kKeyBlock) {
    // (a) the raw scores of all heads for the block's keys: one thread a (key head, key)
    for (int item = tid; item < G * kKeyBlock; item += nth) {
      const int g = item / kKeyBlock, jj = item % kKeyBlock;
      const int j = j0 + jj;
      const T* krow = nullptr;
      if (j >= lo && j <= pos) {
        const int lp = j / page_size;
        const int page = lp < bt_width ? bt[lp] : -1;
        if (page >= 0 && page < num_pages)
          krow = pages + ((size_t)page * page_size + (size_t)(j % page_size)) * row_width;
      }
      if (g == 0) vrow_s[jj] = krow ? krow + (size_t)G * D : nullptr;
      for (int r0 = 0; r0 < rep; r0 += 4) {
        float dot[4] = {0.f, 0.f, 0.f, 0.f};
        if (krow) {
          const T* kh = krow + (size_t)g * D;
          const float* qh = q_s + (size_t)(g * rep + r0) * D;
          for (int d = 0; d < D; ++d) {
            const float kv = to_float(kh[d]);
#pragma unroll
            for (int r = 0; r < 4; ++r)
              if (r0 + r < rep) dot[r] = fmaf(qh[r * D + d], kv, dot[r]);
          }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r)
          if (r0 + r < rep) s_raw[(g * rep + r0 + r) * kKeyBlock + jj] = dot[r] * scale;
      }
    }
    __syncthreads();
    // (b) mixing over heads, mask, running maximum and sum: one warp a head, one lane a key
    for (int h = warp; h < H; h += nwarp) {
      const int j = j0 + lane;
      float s = -INFINITY;
      if (j >= lo && j <= pos && vrow_s[lane] != nullptr) {
        s = 0.f;
        for (int g = 0; g < H; ++g) s = fmaf(talk_s[h * H + g], s_raw[g * kKeyBlock + lane], s);
      }
      const float m_old = m_s[h];
      const float m_new = fmaxf(m_old, warp_max(s));
      const float p = (s == -INFINITY || m_new == -INFINITY) ? 0.f : expf(s - m_new);
      const float alpha = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
      const float psum = warp_sum(p);
      p_s[h * kKeyBlock + lane] = p;
      if (lane == 0) {
        m_s[h] = m_new;
        l_s[h] = l_s[h] * alpha + psum;
        a_s[h] = alpha;
      }
    }
    __syncthreads();
    // (c) the weighted sum of values: a thread owns outputs (head, column)
    const int nkeys = min(kKeyBlock, pos - j0 + 1);
#pragma unroll
    for (int n = 0; n < kMaxAcc; ++n) {
      const int idx = tid + n * nth;
      if (idx < H * Dv) {
        const int h = idx / Dv, d = idx % Dv;
        const int off = (h / rep) * Dv + d;
        float a = acc[n] * a_s[h];
        const float* ph = p_s + h * kKeyBlock;
        for (int jj = 0; jj < nkeys; ++jj) {
          const T* vr = vrow_s[jj];
          if (vr) a = fmaf(ph[jj], to_float(vr[off]), a);
        }
        acc[n] = a;
      }
    }
    __syncthreads();
  }
  T* o = out + (size_t)t * H * Dv;
#pragma unroll
  for (int n = 0; n < kMaxAcc; ++n) {
    const int idx = tid + n * nth;
    if (idx < H * Dv) {
      const float l = l_s[idx / Dv];
      o[idx] = from_float<T>(l > 0.f ? acc[n] / l : 0.f);
    }
  }
}

// One CTA a row: biases, the per-head norm of queries and keys, the rotation, and the writes of the
// queries (engine type) and of the row [k | v] into its page.  `proj` holds the float32 sums of
// the projections, a row [q: H * D | k: G * D | v: G * Dv] (or the queries alone when the layer reads
// another layer's keys and values: G = 0 then).
template <typename T>
__global__ void head_norm_rope_append_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ bias,
                                             const float* __restrict__ q_norm, const float* __restrict__ k_norm,
                                             float eps, const float* __restrict__ inv_freq, int rot,
                                             const int* __restrict__ positions, const int* __restrict__ row_seg,
                                             T* __restrict__ q_out, T* __restrict__ pages,
                                             const int* __restrict__ block_table, int bt_width, int H, int G, int D,
                                             int Dv, int page_size, int num_pages) {
  extern __shared__ float smem[];            // [warps][D]
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  float* y = smem + (size_t)warp * D;
  chain_wait(proj);
  const int pos = positions[t];
  const float* row = proj + (size_t)t * ld;
  T* cache_row = nullptr;
  if (G > 0) {
    const int lp = pos / page_size;
    const int page = lp < bt_width ? block_table[(size_t)row_seg[t] * bt_width + lp] : -1;
    if (page >= 0 && page < num_pages)
      cache_row = pages + ((size_t)page * page_size + (size_t)(pos % page_size)) * ((size_t)G * (D + Dv));
  }
  const int half = rot / 2;
  for (int head = warp; head < H + G; head += nwarp) {
    const bool is_q = head < H;
    const float* x = row + (size_t)head * D;
    const float* b = bias ? bias + (size_t)head * D : nullptr;
    const float* w = is_q ? q_norm : k_norm;
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) {
      const float v = x[d] + (b ? b[d] : 0.f);
      y[d] = v;
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)D + eps);
    __syncwarp();
    T* dst = is_q ? q_out + (size_t)t * H * D + (size_t)head * D
                  : (cache_row ? cache_row + (size_t)(head - H) * D : nullptr);
    if (dst) {
      for (int d = lane; d < D; d += 32) {
        float v = y[d] * inv * (w ? w[d] : 1.f);
        if (d < rot) {
          const int i = d < half ? d : d - half;
          const int partner = d < half ? d + half : d - half;
          const float other = y[partner] * inv * (w ? w[partner] : 1.f);
          float sn, cs;
          sincosf((float)pos * inv_freq[i], &sn, &cs);
          v = d < half ? v * cs - other * sn : v * cs + other * sn;
        }
        dst[d] = from_float<T>(v);
      }
    }
    __syncwarp();
  }
  if (cache_row) {
    const float* x = row + (size_t)(H + G) * D;
    const float* b = bias ? bias + (size_t)(H + G) * D : nullptr;
    T* dst = cache_row + (size_t)G * D;
    for (int i = threadIdx.x; i < G * Dv; i += blockDim.x) dst[i] = from_float<T>(x[i] + (b ? b[i] : 0.f));
  }
}

}  // namespace nf

using namespace nf;

extern "C" int nf_talking_attention(const void* q, const void* pages, const int* block_table, int bt_width,
                                    const int* positions, const int* row_seg, const int* row_list, const float* talk,
                                    const float* sink, void* out, int R, int H, int G, int D, int Dv, int page_size,
                                    int num_pages, int chunk, float scale, int dtype, cudaStream_t stream) {
  if (R == 0) return 0;
  NF_REQUIRE(R > 0 && H > 0 && G > 0 && H % G == 0 && D > 0 && Dv > 0, "talking_attention: bad sizes R=%d H=%d G=%d D=%d Dv=%d", R, H, G, D, Dv);
  NF_REQUIRE(chunk >= 0 && page_size > 0, "talking_attention: bad chunk %d or page size %d", chunk, page_size);
  int th = H * Dv > 512 ? 256 : 128;
  while (th < 1024 && th * kMaxAcc < H * Dv) th <<= 1;
  NF_REQUIRE(th * kMaxAcc >= H * Dv, "talking_attention: %d heads of %d values are more than a CTA serves (%d)", H, Dv, 1024 * kMaxAcc);
  const size_t smem = ((size_t)H * D + 2 * (size_t)H * kKeyBlock + 3 * (size_t)H + (size_t)H * H) * sizeof(float);
  NF_REQUIRE(smem <= 200 * 1024, "talking_attention: %d heads of %d do not fit shared memory", H, D);
  if (dtype == kF32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(talking_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_chained(talking_attention_kernel<float>, dim3(R), dim3(th), smem, stream, (const float*)q, (const float*)pages, block_table, bt_width, positions, row_seg, row_list, talk, sink, (float*)out, H, G, D, Dv, page_size, num_pages, chunk, scale);
  } else {
    if (smem > 48 * 1024) cudaFuncSetAttribute(talking_attention_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_chained(talking_attention_kernel<__nv_bfloat16>, dim3(R), dim3(th), smem, stream, (const __nv_bfloat16*)q, (const __nv_bfloat16*)pages, block_table, bt_width, positions, row_seg, row_list, talk, sink, (__nv_bfloat16*)out, H, G, D, Dv, page_size, num_pages, chunk, scale);
  }
  return check_launch("talking_attention");
}

extern "C" int nf_head_norm_rope_append(const float* proj, int ld, const float* bias, const float* q_norm,
                                        const float* k_norm, float eps, const float* inv_freq, int rot,
                                        const int* positions, const int* row_seg, void* q_out, void* pages,
                                        const int* block_table, int bt_width, int T, int H, int G, int D, int Dv,
                                        int page_size, int num_pages, int dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  NF_REQUIRE(T > 0 && H > 0 && G >= 0 && D > 0 && Dv >= 0, "head_norm_rope_append: bad sizes T=%d H=%d G=%d D=%d Dv=%d", T, H, G, D, Dv);
  NF_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= D && (rot == 0 || inv_freq), "head_norm_rope_append: %d turned dimensions of %d", rot, D);
  NF_REQUIRE(ld >= H * D + G * (D + Dv), "head_norm_rope_append: rows of %d are shorter than the projections", ld);
  NF_REQUIRE(G == 0 || (pages && block_table), "head_norm_rope_append: keys without a cache");
  const int th = 128;
  const size_t smem = (size_t)(th / 32) * D * sizeof(float);
  NF_REQUIRE(smem <= 48 * 1024, "head_norm_rope_append: head size %d", D);
  if (dtype == kF32)
    launch_chained(head_norm_rope_append_kernel<float>, dim3(T), dim3(th), smem, stream, proj, ld, bias, q_norm, k_norm, eps, inv_freq, rot, positions, row_seg, (float*)q_out, (float*)pages, block_table, bt_width, H, G, D, Dv, page_size, num_pages);
  else
    launch_chained(head_norm_rope_append_kernel<__nv_bfloat16>, dim3(T), dim3(th), smem, stream, proj, ld, bias, q_norm, k_norm, eps, inv_freq, rot, positions, row_seg, (__nv_bfloat16*)q_out, (__nv_bfloat16*)pages, block_table, bt_width, H, G, D, Dv, page_size, num_pages);
  return check_launch("head_norm_rope_append");
}
