// The stage after the projection of an attention whose values are its keys: add the biases, take
// the queries and the keys each over the root mean square of the WHOLE projection (all heads'
// rows at once, before they are split into heads) times a weight, write the normed keys into the
// key half of the request's cache page and the keys as projected (bias added, not normed) into the
// value half.  Nothing is rotated.  The projection arrives as float32 sums, so a key is rounded
// to the cache's type once.
//
// Cache page layout: [2 (k, v)][kv_heads][page_size][head_dim], as rope_append.cu writes it.
//
// A second kernel serves an attention with values of their own and a rotation after the same
// whole-projection norms (in either page layout), and a third its elementwise output gate.
#define NF_CHAIN_CLASS 4
#include "common.cuh"

namespace nf {

template <typename T>
__global__ void __launch_bounds__(256)
qk_whole_norm_append_kernel(const float* __restrict__ proj, int ld, int q_col0, int k_col0,
                            const float* __restrict__ bias_q, const float* __restrict__ bias_k,
                            const float* __restrict__ wq, const float* __restrict__ wk, float eps,
                            const int* __restrict__ positions, const int* __restrict__ row_seg,
                            T* __restrict__ q_out, int Hq, int Hkv, int D, T* __restrict__ pages,
                            const int* __restrict__ block_table, int bt_width, int page_size, int num_pages,
                            int append) {
  __shared__ float red[33];
  const int t = blockIdx.x;
  chain_release_if_small();
  chain_wait(proj);
  const float* row = proj + (size_t)t * ld;
  const int QW = Hq * D, KW = Hkv * D;
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < QW; i += blockDim.x) {
    const float v = row[q_col0 + i] + (bias_q ? bias_q[i] : 0.f);
    sq += v * v;
  }
  for (int i = threadIdx.x; i < KW; i += blockDim.x) {
    const float v = row[k_col0 + i] + (bias_k ? bias_k[i] : 0.f);
    sk += v * v;
  }
  const float inv_q = rsqrtf(block_sum(sq, red) / (float)QW + eps);
  const float inv_k = rsqrtf(block_sum(sk, red) / (float)KW + eps);
  T* qo = q_out + (size_t)t * QW;
  for (int i = threadIdx.x; i < QW; i += blockDim.x) {
    const float v = row[q_col0 + i] + (bias_q ? bias_q[i] : 0.f);
    qo[i] = from_float<T>(v * inv_q * wq[i]);
  }
  if (!append) return;
  const int pos = positions[t], seg = row_seg[t];
  const int lp = pos / page_size;
  const int page = (lp >= 0 && lp < bt_width) ? block_table[(size_t)seg * bt_width + lp] : -1;
  if (page < 0 || page >= num_pages) return;               // no page reserved: never write out of bounds
  T* kdst = pages + ((size_t)page * 2 * Hkv * page_size + (size_t)(pos - lp * page_size)) * D;
  const size_t head_stride = (size_t)page_size * D;
  for (int i = threadIdx.x; i < KW; i += blockDim.x) {
    const int head = i / D, d = i - head * D;
    const float v = row[k_col0 + i] + (bias_k ? bias_k[i] : 0.f);
    kdst[(size_t)head * head_stride + d] = from_float<T>(v * inv_k * wk[i]);
    kdst[(size_t)(Hkv + head) * head_stride + d] = from_float<T>(v);
  }
}


// The same stage for an attention with values of their own and a rotation: biases; q and k each over
// the root mean square of the WHOLE projection times a weight of the projection's width; then the first
// `rot` dimensions of every q and k head turned by the row's position (pair (i, i + rot/2), angle
// pos * inv_freq[i] in float32), cosine and sine both times `mag`; q goes out in the cache's type, the
// key and the value (bias added) into the request's page.  Two page layouts:
//   rows == 0: [2 (k, v)][kv_heads][page_size][D] (needs Dv == D), what the flash and decode kernels read;
//   rows == 1: [page_size][kv_heads * D | kv_heads * Dv], one row a token, for key and value sizes that differ.
// Hkv == 0: a layer that reads another layer's keys brings queries only.
// The row's normed values wait in shared memory (float32) between the two passes.
template <typename T>
__global__ void __launch_bounds__(256)
whole_norm_rope_append_kernel(const float* __restrict__ proj, int ld, int q_col0, int k_col0, int v_col0,
                              const float* __restrict__ bias_q, const float* __restrict__ bias_k,
                              const float* __restrict__ bias_v, const float* __restrict__ wq,
                              const float* __restrict__ wk, float eps, const float* __restrict__ inv_freq, int rot,
                              float mag, const int* __restrict__ positions, const int* __restrict__ row_seg,
                              T* __restrict__ q_out, int Hq, int Hkv, int D, int Dv, T* __restrict__ pages,
                              const int* __restrict__ block_table, int bt_width, int page_size, int num_pages,
                              int rows_layout) {
  extern __shared__ __align__(16) float y[];   // [Hq * D + Hkv * D], then cosine and sine of the row's rot / 2 angles
  __shared__ float red[33];
  const int t = blockIdx.x;
  const int QW = Hq * D, KW = Hkv * D;
  const int half = rot / 2;
  float* cs_s = y + QW + KW;
  float* sn_s = cs_s + half;
  chain_release_if_small();
  // the angles depend on the position alone (a step's input, not the kernel before's output): all heads share them
  const int pos = positions[t];
  for (int u = threadIdx.x; u < half; u += blockDim.x) {
    float sn, cs;
    sincosf((float)pos * inv_freq[u], &sn, &cs);
    cs_s[u] = cs * mag;
    sn_s[u] = sn * mag;
  }
  chain_wait(proj);
  const float* row = proj + (size_t)t * ld;
  float sq = 0.f, sk = 0.f;
  // (which of the two forms runs depends on sizes and addresses that are the same in every step of a model)
  const bool vec = (ld | q_col0 | k_col0 | QW | KW) % 4 == 0 && (uintptr_t)proj % 16 == 0 &&
                   (!bias_q || (uintptr_t)bias_q % 16 == 0) && (!bias_k || (uintptr_t)bias_k % 16 == 0);
  if (vec) {
    for (int i = threadIdx.x * 4; i < QW + KW; i += blockDim.x * 4) {
      const bool is_q = i < QW;
      const int c = is_q ? i : i - QW;
      const float* bp = is_q ? bias_q : bias_k;
      float4 v = *reinterpret_cast<const float4*>(row + (is_q ? q_col0 : k_col0) + c);
      if (bp) {
        const float4 b = *reinterpret_cast<const float4*>(bp + c);
        v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
      }
      *reinterpret_cast<float4*>(y + i) = v;
      const float s4 = fmaf(v.w, v.w, fmaf(v.z, v.z, fmaf(v.y, v.y, v.x * v.x)));
      if (is_q) sq += s4; else sk += s4;
    }
  } else {
    for (int i = threadIdx.x; i < QW; i += blockDim.x) {
      const float v = row[q_col0 + i] + (bias_q ? bias_q[i] : 0.f);
      y[i] = v;
      sq = fmaf(v, v, sq);
    }
    for (int i = threadIdx.x; i < KW; i += blockDim.x) {
      const float v = row[k_col0 + i] + (bias_k ? bias_k[i] : 0.f);
      y[QW + i] = v;
      sk = fmaf(v, v, sk);
    }
  }
  const float inv_q = 1.f / sqrtf(block_sum(sq, red) / (float)QW + eps);
  const float inv_k = KW ? 1.f / sqrtf(block_sum(sk, red) / (float)KW + eps) : 0.f;
  for (int i = threadIdx.x; i < QW; i += blockDim.x) y[i] = y[i] * inv_q * wq[i];
  for (int i = threadIdx.x; i < KW; i += blockDim.x) y[QW + i] = y[QW + i] * inv_k * wk[i];
  __syncthreads();
  T* krow = nullptr;                           // where head 0's key of this token starts
  size_t k_head_stride = 0, v_head_stride = 0;
  T* vrow = nullptr;
  if (Hkv > 0) {
    const int lp = pos / page_size;
    const int page = (lp >= 0 && lp < bt_width) ? block_table[(size_t)row_seg[t] * bt_width + lp] : -1;
    if (page >= 0 && page < num_pages) {       // no page reserved: never write out of bounds
      const int in_page = pos - lp * page_size;
      if (rows_layout) {
        krow = pages + ((size_t)page * page_size + in_page) * ((size_t)Hkv * (D + Dv));
        vrow = krow + (size_t)Hkv * D;
        k_head_stride = D; v_head_stride = Dv;
      } else {
        krow = pages + ((size_t)page * 2 * Hkv * page_size + in_page) * D;
        k_head_stride = v_head_stride = (size_t)page_size * D;
        vrow = krow + (size_t)Hkv * k_head_stride;
      }
    }
  }
  // a unit is a turned pair (u, u + rot/2) of a head, whose angle is worked out once, or a single dimension beyond
  const int units = D - half;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  for (int hh = warp; hh < Hq + Hkv; hh += nwarp) {       // a warp a head: q heads first, then k heads, as they lie in y
    const bool is_q = hh < Hq;
    const float* yy = y + (size_t)hh * D;
    T* dst = is_q ? q_out + (size_t)t * QW + (size_t)hh * D
                  : (krow ? krow + (size_t)(hh - Hq) * k_head_stride : nullptr);
    if (!dst) continue;
    for (int u = lane; u < units; u += 32) {
      if (u < half) {
        const float a = yy[u], b = yy[u + half];
        const float sn = sn_s[u], cs = cs_s[u];
        dst[u] = from_float<T>(a * cs - b * sn);
        dst[u + half] = from_float<T>(b * cs + a * sn);
      } else {
        const int d = rot + (u - half);
        dst[d] = from_float<T>(yy[d]);
      }
    }
  }
  if (vrow) {
    for (int head = warp; head < Hkv; head += nwarp)
      for (int d = lane; d < Dv; d += 32) {
        const int i = head * Dv + d;
        vrow[(size_t)head * v_head_stride + d] = from_float<T>(row[v_col0 + i] + (bias_v ? bias_v[i] : 0.f));
      }
  }
}

// out[t, c] = o[t, c] * sigmoid(g[t, g_col0 + c]): an output gate element by element; the gate's
// logits are float32 sums or of the rows' type.
// VEC: four consecutive elements a thread, each operand's run in one access.
template <typename T, typename TG, bool VEC>
__global__ void sigmoid_gate_rows_kernel(const T* __restrict__ o, const TG* __restrict__ g, int ldg, int g_col0,
                                         T* __restrict__ out, int width) {
  const int t = blockIdx.y;
  chain_wait(o, g);
  constexpr int W = VEC ? 4 : 1;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * W;
  if (c >= width) return;
  if constexpr (VEC) {
    float ov[4], gv[4];
    load4(o + (size_t)t * width + c, ov);
    load4(g + (size_t)t * ldg + g_col0 + c, gv);
#pragma unroll
    for (int e = 0; e < 4; ++e) ov[e] = ov[e] * (1.f / (1.f + expf(-gv[e])));
    store4(out + (size_t)t * width + c, ov);
  } else {
    const float gv = to_float(g[(size_t)t * ldg + g_col0 + c]);
    out[(size_t)t * width + c] = from_float<T>(to_float(o[(size_t)t * width + c]) * (1.f / (1.f + expf(-gv))));
  }
}

}  // namespace nf

using namespace nf;

extern "C" int nf_qk_whole_norm_append(const float* proj, int ld, int q_col0, int k_col0, const float* bias_q,
                                       const float* bias_k, const float* wq, const float* wk, float eps,
                                       const int* positions, const int* row_seg, void* q_out, int T, int Hq, int Hkv,
                                       int D, void* pages, const int* block_table, int bt_width, int page_size,
                                       int num_pages, int append, int dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  NF_REQUIRE(T > 0 && Hq > 0 && Hkv > 0 && D > 0 && wq && wk, "qk_whole_norm_append: bad arguments");
  NF_REQUIRE(q_col0 >= 0 && k_col0 >= 0 && q_col0 + Hq * D <= ld && k_col0 + Hkv * D <= ld,
             "qk_whole_norm_append: the column ranges leave the projection");
  if (dtype == kF32)
    launch_chained(qk_whole_norm_append_kernel<float>, dim3(T), dim3(256), 0, stream, proj, ld, q_col0, k_col0, bias_q, bias_k, wq, wk, eps, positions, row_seg, (float*)q_out, Hq, Hkv, D, (float*)pages, block_table, bt_width, page_size, num_pages, append);
  else
    launch_chained(qk_whole_norm_append_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, proj, ld, q_col0, k_col0, bias_q, bias_k, wq, wk, eps, positions, row_seg, (__nv_bfloat16*)q_out, Hq, Hkv, D, (__nv_bfloat16*)pages, block_table, bt_width, page_size, num_pages, append);
  return check_launch("qk_whole_norm_append");
}

// proj float32 [T, ld]: q (Hq x D) at q_col0, and with Hkv > 0 k (Hkv x D) at k_col0 and v (Hkv x Dv) at
// v_col0.  rows_layout 0: pages [.., 2, Hkv, page_size, D] (Dv == D); 1: pages [.., page_size, Hkv * (D + Dv)].
extern "C" int nf_whole_norm_rope_append(const float* proj, int ld, int q_col0, int k_col0, int v_col0,
                                         const float* bias_q, const float* bias_k, const float* bias_v,
                                         const float* wq, const float* wk, float eps, const float* inv_freq, int rot,
                                         float mag, const int* positions, const int* row_seg, void* q_out, int T,
                                         int Hq, int Hkv, int D, int Dv, void* pages, const int* block_table,
                                         int bt_width, int page_size, int num_pages, int rows_layout, int dtype,
                                         cudaStream_t stream) {
  if (T == 0) return 0;
  NF_REQUIRE(T > 0 && Hq > 0 && Hkv >= 0 && D > 0 && Dv > 0 && wq && (Hkv == 0 || wk), "whole_norm_rope_append: bad arguments");
  NF_REQUIRE(q_col0 >= 0 && q_col0 + Hq * D <= ld, "whole_norm_rope_append: the queries leave the projection");
  NF_REQUIRE(Hkv == 0 || (k_col0 >= 0 && v_col0 >= 0 && k_col0 + Hkv * D <= ld && v_col0 + Hkv * Dv <= ld),
             "whole_norm_rope_append: keys or values leave the projection");
  NF_REQUIRE(Hkv == 0 || (pages && block_table), "whole_norm_rope_append: keys without a cache");
  NF_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= D && (rot == 0 || inv_freq), "whole_norm_rope_append: %d turned dimensions of %d", rot, D);
  NF_REQUIRE(rows_layout || Hkv == 0 || D == Dv, "whole_norm_rope_append: the head-major page needs equal key and value sizes");
  const size_t smem = ((size_t)(Hq + Hkv) * D + rot) * sizeof(float);
  NF_REQUIRE(smem <= 200 * 1024, "whole_norm_rope_append: %d values a row do not fit shared memory", (Hq + Hkv) * D);
  if (dtype == kF32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(whole_norm_rope_append_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_chained(whole_norm_rope_append_kernel<float>, dim3(T), dim3(256), smem, stream, proj, ld, q_col0, k_col0, v_col0, bias_q, bias_k, bias_v, wq, wk, eps, inv_freq, rot, mag, positions, row_seg, (float*)q_out, Hq, Hkv, D, Dv, (float*)pages, block_table, bt_width, page_size, num_pages, rows_layout);
  } else {
    if (smem > 48 * 1024) cudaFuncSetAttribute(whole_norm_rope_append_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_chained(whole_norm_rope_append_kernel<__nv_bfloat16>, dim3(T), dim3(256), smem, stream, proj, ld, q_col0, k_col0, v_col0, bias_q, bias_k, bias_v, wq, wk, eps, inv_freq, rot, mag, positions, row_seg, (__nv_bfloat16*)q_out, Hq, Hkv, D, Dv, (__nv_bfloat16*)pages, block_table, bt_width, page_size, num_pages, rows_layout);
  }
  return check_launch("whole_norm_rope_append");
}

// o, out [T, width] of `dtype`; g [T, ldg] float32 (g_dtype 0) or of `dtype`.
extern "C" int nf_sigmoid_gate_rows(const void* o, const void* g, int g_dtype, int ldg, int g_col0, void* out, int T,
                                    int width, int dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  NF_REQUIRE(T > 0 && T <= 65535 * 1024 && width > 0 && g_col0 >= 0 && g_col0 + width <= ldg, "sigmoid_gate_rows: bad sizes");
  NF_REQUIRE(g_dtype == kF32 || g_dtype == dtype, "sigmoid_gate_rows: the gate is float32 or of the rows' type");
  const size_t tsize = dtype == kF32 ? 4 : 2, gsize = g_dtype == kF32 ? 4 : 2;
  const bool vec = width % 4 == 0 && ldg % 4 == 0 && g_col0 % 4 == 0 && (uintptr_t)o % (4 * tsize) == 0 &&
                   (uintptr_t)out % (4 * tsize) == 0 && (uintptr_t)g % (4 * gsize) == 0;
  for (int t0 = 0; t0 < T; t0 += 65535) {
    const int rows = T - t0 < 65535 ? T - t0 : 65535;
    const dim3 grid(((vec ? width / 4 : width) + 255) / 256, rows);
    const size_t off = (size_t)t0 * width, goff = (size_t)t0 * ldg;
#define NF_SG(TT, TG_, V) \
  launch_chained(sigmoid_gate_rows_kernel<TT, TG_, V>, grid, dim3(256), 0, stream, (const TT*)o + off, (const TG_*)g + goff, ldg, g_col0, (TT*)out + off, width)
    if (dtype == kF32) { if (vec) NF_SG(float, float, true); else NF_SG(float, float, false); }
    else if (g_dtype == kF32) { if (vec) NF_SG(__nv_bfloat16, float, true); else NF_SG(__nv_bfloat16, float, false); }
    else { if (vec) NF_SG(__nv_bfloat16, __nv_bfloat16, true); else NF_SG(__nv_bfloat16, __nv_bfloat16, false); }
#undef NF_SG
  }
  return check_launch("sigmoid_gate_rows");
}
