// The attention of attention_talking.cu (heads' scores mixed before the softmax, chunks, a sink) on
// tensor cores, in bfloat16, for prompt portions and decoded tokens alike.
//
// The mixing ties all heads of a (row, key) pair together, so a tile is 32 (or 16) consecutive rows of one
// request with ALL heads, and the heads are dealt out over the CTAs of a thread-block cluster: CTA r
// of C owns heads [r * HC, (r + 1) * HC), as score heads and as output heads.  Keys come in blocks
// of 32 aligned to absolute positions, in ascending order.  For every block a CTA
//   1. computes its own heads' raw scores S_g = Q_g K^T * scale [rows x 32] with mma.sync into its
//      shared memory (float32): a warp takes (head, 16 keys), all the rows,
//   2. meets the others at a cluster barrier and reads ALL heads' raw scores, its own and the other
//      CTAs' through distributed shared memory, to mix them for its output heads:
//      S'_h = sum_g talk[h, g] S_g, in float32 on the vector units; a thread owns one row, four (or
//      two) consecutive keys and all of the CTA's heads, so every raw score is read once a CTA,
//   3. masks (j <= i, same chunk), updates the row's maximum and sum (a shuffle among the 8 or 16
//      threads of a row), and writes the weights as two bfloat16 halves (the rounding and what it
//      left: 16 bits of mantissa together),
//   4. adds P_h V to its output heads' accumulators (registers) with mma.sync: a warp takes
//      (head, 16 columns), all the rows.
// The raw scores are double buffered, so one cluster barrier a block is enough: a CTA that writes
// block b + 2 has passed barrier b + 1, which every CTA reaches only after it has mixed block b.
// Keys and values of the CTA's heads arrive by cp.async, the next block's keys while this block is
// mixed and multiplied, the next values while the next scores are computed.
//
// A step of single rows may cut a row's keys into `nsplit` runs of blocks counted from the row's own
// first block (its chunk's start), one cluster each; partial (m, l, O) go to a workspace and a second
// kernel merges them in ascending order and adds the sink.  A step with few tiles may cut the keys
// into runs counted from position 0 in the same way, so that a long tile's blocks spread over SMs.
// Either way a row's sums depend on its own position and on the runs' length only.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace nf {

namespace {

constexpr int kTmKeys = 32;        // keys a block
constexpr int kTmThreads = 256;
constexpr int kTmPad = 8;          // bfloat16 elements of padding a shared-memory row
constexpr int kTmSP = 36;          // floats a row of raw scores (consecutive rows' float4 reads meet no conflict)
constexpr int kTmPP = 40;          // bfloat16 a row of weights

__device__ __forceinline__ unsigned tm_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tm_ldm4(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void tm_ldm4t(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void tm_mma(float* c, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// another CTA's shared memory: the address of the same offset in CTA `rank` of the cluster, and a 16-byte read
__device__ __forceinline__ unsigned tm_mapa(unsigned addr, unsigned rank) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ float4 tm_ld_cluster4(unsigned addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}
// a row of the mixing weights [HC] from shared memory (16 bytes a read where the rows are so aligned)
template <int HC>
__device__ __forceinline__ void tm_talk_row(const float* p, float* w) {
  if constexpr (HC % 4 == 0) {
#pragma unroll
    for (int i = 0; i < HC / 4; ++i) {
      const float4 v = *reinterpret_cast<const float4*>(p + i * 4);
      w[i * 4] = v.x; w[i * 4 + 1] = v.y; w[i * 4 + 2] = v.z; w[i * 4 + 3] = v.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < HC; ++i) w[i] = p[i];
  }
}
__device__ __forceinline__ float2 tm_ld_cluster2(unsigned addr) {
  float2 v;
  asm volatile("ld.shared::cluster.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
  return v;
}
template <int KPT>
__device__ __forceinline__ void tm_ld_remote(unsigned addr, float* v) {
  if constexpr (KPT == 4) {
    const float4 t = tm_ld_cluster4(addr);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else {
    const float2 t = tm_ld_cluster2(addr);
    v[0] = t.x; v[1] = t.y;
  }
}
template <int KPT>
__device__ __forceinline__ void tm_ld_local(const float* p, float* v) {
  if constexpr (KPT == 4) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else {
    const float2 t = *reinterpret_cast<const float2*>(p);
    v[0] = t.x; v[1] = t.y;
  }
}
__device__ __forceinline__ void tm_cp16(unsigned dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}


struct TmLayout {
  int nkv, QS, KS, VS;
  size_t q, k, v, s, p, talk, alpha, l, pos, lo, total;
};

__host__ __device__ inline TmLayout tm_layout(int H, int G, int D, int Dv, int HC, int rows) {
  TmLayout L;
  const int rep = H / G;
  L.nkv = (HC + rep - 1) / rep + ((HC % rep != 0 && rep % HC != 0) ? 1 : 0);
  if (L.nkv > G) L.nkv = G;
  L.QS = HC * D + kTmPad;
  L.KS = L.nkv * D + kTmPad;
  L.VS = L.nkv * Dv + kTmPad;
  size_t o = 0;
  L.q = o; o += (size_t)rows * L.QS * 2;
  L.k = o; o += (size_t)kTmKeys * L.KS * 2;
  L.v = o; o += (size_t)kTmKeys * L.VS * 2;
  L.s = o; o += (size_t)2 * HC * rows * kTmSP * 4;
  L.p = o; o += (size_t)2 * HC * rows * kTmPP * 2;
  L.talk = o; o += (size_t)H * HC * 4;
  L.alpha = o; o += (size_t)HC * rows * 4;
  L.l = o; o += (size_t)HC * rows * 4;
  L.pos = o; o += rows * 4;
  L.lo = o; o += rows * 4;
  L.total = (o + 15) & ~(size_t)15;
  return L;
}

}  // namespace

// tiles: int32 [n_tiles, 2] of (segment, first row); null when every segment brings one row (tile i is
// segment i).  ws_o float32 [T * H, nsplit, Dv], ws_ml float32 [T * H, nsplit, 2], or both null: with them
// the CTAs of run `blockIdx.y` write partial sums there, which the merge kernel adds up with the sink.
template <int HC, int NU, int ROWS>      // heads a CTA; (head, 16 columns) units of the second product a warp; rows a tile (32 or 16)
__global__ void __launch_bounds__(kTmThreads, 1)
talking_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ pages,
                             const int* __restrict__ block_table, int bt_width, const int* __restrict__ positions,
                             const int* __restrict__ seg_row0, const int* __restrict__ tiles,
                             const float* __restrict__ talk, const float* __restrict__ sink,
                             __nv_bfloat16* __restrict__ out, float* __restrict__ ws_o, float* __restrict__ ws_ml,
                             int H, int G, int D, int Dv, int page_size, int num_pages, int chunk, float scale,
                             int nsplit, int blocks_per_split) {
  constexpr int MT = ROWS / 16;
  constexpr int KPT = kTmKeys * ROWS / kTmThreads;     // keys a mixing thread: 4 or 2
  constexpr int LPR = kTmKeys / KPT;                   // mixing threads a row
  constexpr int NW = kTmThreads / 32;
  extern __shared__ __align__(16) unsigned char tm_raw[];
  cg::cluster_group cluster = cg::this_cluster();
  const int C = (int)cluster.num_blocks();
  const int rank = (int)cluster.block_rank();
  const int tile = blockIdx.x / C, split = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const TmLayout L = tm_layout(H, G, D, Dv, HC, ROWS);
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(tm_raw + L.q);
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(tm_raw + L.k);
  __nv_bfloat16* Vs = reinterpret_cast<__nv_bfloat16*>(tm_raw + L.v);
  float* Ss = reinterpret_cast<float*>(tm_raw + L.s);                    // [2][HC][32][kTmSP]
  __nv_bfloat16* Ps = reinterpret_cast<__nv_bfloat16*>(tm_raw + L.p);    // [2: rounding, remainder][HC][32][kTmPP]
  float* talk_s = reinterpret_cast<float*>(tm_raw + L.talk);             // [H][HC]: talk[h0 + hl][g] at [g][hl]
  float* alpha_s = reinterpret_cast<float*>(tm_raw + L.alpha);           // [HC][32]
  float* l_s = reinterpret_cast<float*>(tm_raw + L.l);                   // [HC][32]
  int* row_pos = reinterpret_cast<int*>(tm_raw + L.pos);
  int* row_lo = reinterpret_cast<int*>(tm_raw + L.lo);
  const int QS = L.QS, KS = L.KS, VS = L.VS;
  const int rep = H / G;
  const int h0 = rank * HC;                            // this CTA's first head
  const int kv0 = h0 / rep;                            // ... and its first key/value head
  const int nkv = (h0 + HC - 1) / rep - kv0 + 1;
  const int row_width = G * (D + Dv);

  for (int i = tid; i < H * HC; i += kTmThreads) {
    const int g = i / HC, hl = i - g * HC;
    talk_s[i] = talk ? talk[(size_t)(h0 + hl) * H + g] : (g == h0 + hl ? 1.f : 0.f);
  }
  chain_wait(q, pages);
  const int seg = tiles ? tiles[2 * tile] : tile;
  const int row0 = tiles ? tiles[2 * tile + 1] : seg_row0[tile];
  const int nrows = min(ROWS, seg_row0[seg + 1] - row0);
  if (tid < ROWS) {
    const int p = tid < nrows ? positions[row0 + tid] : -1;
    row_pos[tid] = p;
    row_lo[tid] = p < 0 ? INT_MAX : (chunk > 0 ? (p / chunk) * chunk : 0);
  }
  // the tile's queries of this CTA's heads, 16 bytes a copy
  {
    const int chunks = HC * D / 8;
    for (int i = tid; i < ROWS * chunks; i += kTmThreads) {
      const int r = i / chunks, c = (i - r * chunks) * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < nrows) v = *reinterpret_cast<const uint4*>(q + (size_t)(row0 + r) * H * D + (size_t)h0 * D + c);
      *reinterpret_cast<uint4*>(Qs + r * QS + c) = v;
    }
  }
  __syncthreads();
  int j_lo = INT_MAX, j_hi = -1;
  for (int r = 0; r < ROWS; ++r) {
    j_lo = min(j_lo, row_lo[r]);
    j_hi = max(j_hi, row_pos[r]);
  }
  const int b_first = j_lo / kTmKeys;
  // runs of blocks whose sums a second kernel merges: counted from the row's first block for steps of single
  // rows, from position 0 for tiles of several rows (so that a row's runs do not depend on its neighbours)
  const bool partial = ws_o != nullptr;
  const int b_begin = !partial ? b_first : tiles ? max(b_first, split * blocks_per_split) : b_first + split * blocks_per_split;
  const int b_end = !partial ? j_hi / kTmKeys + 1
                             : min(j_hi / kTmKeys + 1, (tiles ? split * blocks_per_split : b_begin) + blocks_per_split);
  const int* bt = block_table + (size_t)seg * bt_width;

  if (partial && b_begin >= b_end) {                    // none of the tile's keys in this run (the whole cluster leaves)
    for (int i = tid; i < nrows * HC; i += kTmThreads) {
      const size_t slot = ((size_t)(row0 + i / HC) * H + h0 + i % HC) * nsplit + split;
      ws_ml[slot * 2] = -INFINITY;
      ws_ml[slot * 2 + 1] = 0.f;
    }
    return;
  }

  // eight threads a key row: the row's page is looked up once, then 16-byte copies at a stride of eight
  const int n16_k = nkv * D / 8, n16_v = nkv * Dv / 8;
  auto fetch = [&](int blk, bool values) {
    if (blk < b_end) {
      const int r = tid >> 3;
      const int j = blk * kTmKeys + r;
      const int lp = j / page_size;
      const int page = (j >= j_lo && j <= j_hi && lp < bt_width) ? bt[lp] : -1;
      const int n16 = values ? n16_v : n16_k;
      __nv_bfloat16* d = values ? Vs + (size_t)r * VS : Ks + (size_t)r * KS;
      if (page >= 0 && page < num_pages) {
        const __nv_bfloat16* src = pages + ((size_t)page * page_size + (j - lp * page_size)) * row_width +
                                   (values ? (size_t)G * D + (size_t)kv0 * Dv : (size_t)kv0 * D);
        for (int c = tid & 7; c < n16; c += 8) tm_cp16(tm_smem(d + c * 8), src + c * 8);
      } else {
        for (int c = tid & 7; c < n16; c += 8) *reinterpret_cast<uint4*>(d + c * 8) = make_uint4(0, 0, 0, 0);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  // the mixing thread's place: row mi, keys KPT kq .. of the block (four with 32 rows a tile, two with 16), all
  // of this CTA's heads (so every raw score is read once a CTA, and a row's reads are 128 consecutive bytes)
  const int mi = tid / LPR, kq = tid % LPR;
  const int my_pos = row_pos[mi], my_lo = row_lo[mi];
  const bool with_sink = sink != nullptr && !partial;
  float m_run[HC], l_run[HC];
#pragma unroll
  for (int h = 0; h < HC; ++h) {
    m_run[h] = with_sink ? sink[h0 + h] : -INFINITY;    // the sink counts once: exp(sink - m) = 1
    l_run[h] = with_sink ? 1.f : 0.f;
  }

  // the units of the second product: (head, 16 columns), fixed for the whole tile
  const int v16 = Dv / 16;
  const int n_units = HC * v16;
  int unit_h[NU], unit_v[NU];
#pragma unroll
  for (int k = 0; k < NU; ++k) {
    const int u = min(warp + k * NW, n_units - 1);
    unit_h[k] = u / v16;
    unit_v[k] = ((h0 + unit_h[k]) / rep - kv0) * Dv + (u - unit_h[k] * v16) * 16;
  }
  float o[NU][MT][2][4];
#pragma unroll
  for (int a = 0; a < NU; ++a)
#pragma unroll
    for (int b = 0; b < MT; ++b)
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[a][b][c][e] = 0.f;

  fetch(b_begin, false);
  fetch(b_begin, true);
  for (int blk = b_begin; blk < b_end; ++blk) {
    const int buf = (blk - b_begin) & 1;
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();                                    // the block's keys are in
    // ---- 1. raw scores of this CTA's heads: a warp takes (head, 16 keys) ----
    for (int u = warp; u < HC * 2; u += NW) {
      const int g = u >> 1, kh = u & 1;
      const int kvl = (h0 + g) / rep - kv0;
      float s[MT][2][4];
#pragma unroll
      for (int a = 0; a < MT; ++a)
#pragma unroll
        for (int b = 0; b < 2; ++b)
#pragma unroll
          for (int e = 0; e < 4; ++e) s[a][b][e] = 0.f;
      const unsigned qa = tm_smem(Qs + (lane & 15) * QS + g * D + (lane >> 4) * 8);
      const unsigned ka = tm_smem(Ks + (kh * 16 + (lane & 7) + (lane >> 4) * 8) * KS + kvl * D + ((lane >> 3) & 1) * 8);
      for (int k0 = 0; k0 < D; k0 += 16) {
        unsigned b0, b1, b2, b3;
        tm_ldm4(ka + k0 * 2, b0, b1, b2, b3);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          unsigned a0, a1, a2, a3;
          tm_ldm4(qa + (mt * 16 * QS + k0) * 2, a0, a1, a2, a3);
          tm_mma(s[mt][0], a0, a1, a2, a3, b0, b1);
          tm_mma(s[mt][1], a0, a1, a2, a3, b2, b3);
        }
      }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        float* dst = Ss + ((size_t)(buf * HC + g) * ROWS + mt * 16 + (lane >> 2)) * kTmSP + kh * 16 + (lane & 3) * 2;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          *reinterpret_cast<float2*>(dst + nt * 8) = make_float2(s[mt][nt][0] * scale, s[mt][nt][1] * scale);
          *reinterpret_cast<float2*>(dst + 8 * kTmSP + nt * 8) = make_float2(s[mt][nt][2] * scale, s[mt][nt][3] * scale);
        }
      }
    }
    cluster.sync();                                     // every CTA's raw scores of this block are written
    fetch(blk + 1, false);                              // the keys' buffer is free
    // ---- 2. and 3. mixing, mask, maxima, sums, weights ----
    {
      float acc[HC][KPT];
#pragma unroll
      for (int h = 0; h < HC; ++h)
#pragma unroll
        for (int k = 0; k < KPT; ++k) acc[h][k] = 0.f;
      const unsigned s_ofs = (unsigned)((((size_t)buf * HC * ROWS + mi) * kTmSP + kq * KPT) * sizeof(float));
      // own scores first, then the other CTAs' in a round that starts behind this CTA's rank, so that no
      // CTA's shared memory is asked by all the others at once; the reads of the next CTA's scores are
      // in flight while this one's are mixed
      float sv[HC][KPT];
      if (C > 1) {
        const unsigned src = tm_mapa(tm_smem(Ss), (unsigned)(rank + 1 < C ? rank + 1 : 0)) + s_ofs;
#pragma unroll
        for (int gl = 0; gl < HC; ++gl) tm_ld_remote<KPT>(src + (unsigned)(gl * ROWS * kTmSP * sizeof(float)), sv[gl]);
      }
      {
        const float* src = Ss + s_ofs / sizeof(float);
        const float* tk = talk_s + (size_t)rank * HC * HC;
#pragma unroll
        for (int gl = 0; gl < HC; ++gl) {
          float lv[KPT], w[HC];
          tm_ld_local<KPT>(src + (size_t)gl * ROWS * kTmSP, lv);
          tm_talk_row<HC>(tk + gl * HC, w);
#pragma unroll
          for (int h = 0; h < HC; ++h)
#pragma unroll
            for (int k = 0; k < KPT; ++k) acc[h][k] = fmaf(w[h], lv[k], acc[h][k]);
        }
      }
      for (int step = 1; step < C; ++step) {
        const int c = rank + step < C ? rank + step : rank + step - C;
        const float* tk = talk_s + (size_t)c * HC * HC;
        float cur[HC][KPT];
#pragma unroll
        for (int gl = 0; gl < HC; ++gl)
#pragma unroll
          for (int k = 0; k < KPT; ++k) cur[gl][k] = sv[gl][k];
        if (step + 1 < C) {
          const int cn = c + 1 < C ? c + 1 : 0;
          const unsigned src = tm_mapa(tm_smem(Ss), (unsigned)cn) + s_ofs;
#pragma unroll
          for (int gl = 0; gl < HC; ++gl) tm_ld_remote<KPT>(src + (unsigned)(gl * ROWS * kTmSP * sizeof(float)), sv[gl]);
        }
#pragma unroll
        for (int gl = 0; gl < HC; ++gl) {
          float w[HC];
          tm_talk_row<HC>(tk + gl * HC, w);
#pragma unroll
          for (int h = 0; h < HC; ++h)
#pragma unroll
            for (int k = 0; k < KPT; ++k) acc[h][k] = fmaf(w[h], cur[gl][k], acc[h][k]);
        }
      }
      const int j = blk * kTmKeys + kq * KPT;
      bool seen[KPT];
#pragma unroll
      for (int k = 0; k < KPT; ++k) seen[k] = j + k >= my_lo && j + k <= my_pos;
#pragma unroll
      for (int h = 0; h < HC; ++h) {
        float mx = -INFINITY;
#pragma unroll
        for (int k = 0; k < KPT; ++k) {
          if (!seen[k]) acc[h][k] = -INFINITY;
          mx = fmaxf(mx, acc[h][k]);
        }
#pragma unroll
        for (int d = 1; d < LPR; d <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
        const float m_new = fmaxf(m_run[h], mx);
        const float alpha = (m_run[h] == -INFINITY) ? 0.f : __expf(m_run[h] - m_new);
        float sum = 0.f;
#pragma unroll
        for (int k = 0; k < KPT; ++k) {
          acc[h][k] = seen[k] ? __expf(acc[h][k] - m_new) : 0.f;
          sum += acc[h][k];
        }
#pragma unroll
        for (int d = 1; d < LPR; d <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
        m_run[h] = m_new;
        l_run[h] = l_run[h] * alpha + sum;
        __nv_bfloat16* pd = Ps + ((size_t)h * ROWS + mi) * kTmPP + kq * KPT;
#pragma unroll
        for (int k = 0; k < KPT; k += 2) {
          const __nv_bfloat162 hi = __floats2bfloat162_rn(acc[h][k], acc[h][k + 1]);
          const __nv_bfloat162 lo = __floats2bfloat162_rn(acc[h][k] - __bfloat162float(hi.x), acc[h][k + 1] - __bfloat162float(hi.y));
          *reinterpret_cast<__nv_bfloat162*>(pd + k) = hi;
          *reinterpret_cast<__nv_bfloat162*>(pd + (size_t)HC * ROWS * kTmPP + k) = lo;
        }
        if (kq == 0) alpha_s[h * ROWS + mi] = alpha;
      }
    }
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();                                    // the block's values are in, the weights written
    // ---- 4. O += P V: a warp takes (head, 16 columns) ----
#pragma unroll
    for (int k = 0; k < NU; ++k) {
      if (warp + k * NW < n_units) {
        const int h = unit_h[k];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const float a_lo = alpha_s[h * ROWS + mt * 16 + (lane >> 2)], a_hi = alpha_s[h * ROWS + mt * 16 + 8 + (lane >> 2)];
#pragma unroll
          for (int nt = 0; nt < 2; ++nt) {
            o[k][mt][nt][0] *= a_lo; o[k][mt][nt][1] *= a_lo;
            o[k][mt][nt][2] *= a_hi; o[k][mt][nt][3] *= a_hi;
          }
        }
        const unsigned pa = tm_smem(Ps + (h * ROWS + (lane & 15)) * kTmPP + (lane >> 4) * 8);
        const unsigned va = tm_smem(Vs + ((lane & 7) + ((lane >> 3) & 1) * 8) * VS + unit_v[k] + (lane >> 4) * 8);
#pragma unroll
        for (int ks = 0; ks < kTmKeys / 16; ++ks) {
          unsigned b0, b1, b2, b3;
          tm_ldm4t(va + (ks * 16 * VS) * 2, b0, b1, b2, b3);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            unsigned a0, a1, a2, a3, l0, l1, l2, l3;
            tm_ldm4(pa + (mt * 16 * kTmPP + ks * 16) * 2, a0, a1, a2, a3);
            tm_ldm4(pa + (HC * ROWS * kTmPP + mt * 16 * kTmPP + ks * 16) * 2, l0, l1, l2, l3);
            tm_mma(o[k][mt][0], a0, a1, a2, a3, b0, b1);
            tm_mma(o[k][mt][1], a0, a1, a2, a3, b2, b3);
            tm_mma(o[k][mt][0], l0, l1, l2, l3, b0, b1);
            tm_mma(o[k][mt][1], l0, l1, l2, l3, b2, b3);
          }
        }
      }
    }
    __syncthreads();                                    // values, weights and factors are free
    fetch(blk + 1, true);
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  // ---- results ----
  if (kq == 0) {
#pragma unroll
    for (int h = 0; h < HC; ++h) {
      l_s[h * ROWS + mi] = l_run[h];
      if (partial && mi < nrows) {
        const size_t slot = ((size_t)(row0 + mi) * H + h0 + h) * nsplit + split;
        ws_ml[slot * 2] = m_run[h];
        ws_ml[slot * 2 + 1] = l_run[h];
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < NU; ++k) {
    const int u = warp + k * NW;
    if (u >= n_units) continue;
    const int h = unit_h[k], col = (u - h * v16) * 16 + (lane & 3) * 2;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int r = mt * 16 + half * 8 + (lane >> 2);
        if (r >= nrows) continue;
        if (partial) {
          float* dst = ws_o + (((size_t)(row0 + r) * H + h0 + h) * nsplit + split) * Dv + col;
#pragma unroll
          for (int nt = 0; nt < 2; ++nt)
            *reinterpret_cast<float2*>(dst + nt * 8) = make_float2(o[k][mt][nt][half * 2], o[k][mt][nt][half * 2 + 1]);
        } else {
          const float l = l_s[h * ROWS + r];
          const float inv = l > 0.f ? 1.f / l : 0.f;
          __nv_bfloat16* dst = out + (size_t)(row0 + r) * H * Dv + (size_t)(h0 + h) * Dv + col;
#pragma unroll
          for (int nt = 0; nt < 2; ++nt)
            *reinterpret_cast<__nv_bfloat162*>(dst + nt * 8) =
                __floats2bfloat162_rn(o[k][mt][nt][half * 2] * inv, o[k][mt][nt][half * 2 + 1] * inv);
        }
      }
    }
  }
  cluster.sync();                                       // no CTA leaves while another may still read its scores
}

// out[t, h, :] = (sum_s e^{m_s - M} O_s) / (sum_s e^{m_s - M} l_s + e^{sink_h - M}),  M the maximum of the
// m_s and the sink; runs in ascending order.
__global__ void talking_attention_merge_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_ml,
                                               const float* __restrict__ sink, __nv_bfloat16* __restrict__ out,
                                               int H, int Dv, int nsplit) {
  const int h = blockIdx.x % H;
  chain_wait(ws_o, ws_ml);
  const size_t base = (size_t)blockIdx.x * nsplit;
  float M = sink ? sink[h] : -INFINITY;
  for (int s = 0; s < nsplit; ++s) M = fmaxf(M, ws_ml[(base + s) * 2]);
  float l = (sink && M != -INFINITY) ? expf(sink[h] - M) : 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float m = ws_ml[(base + s) * 2];
    if (m != -INFINITY) l += expf(m - M) * ws_ml[(base + s) * 2 + 1];
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  for (int d = threadIdx.x; d < Dv; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const float m = ws_ml[(base + s) * 2];
      if (m != -INFINITY) acc += expf(m - M) * ws_o[(base + s) * Dv + d];
    }
    out[(size_t)blockIdx.x * Dv + d] = __float2bfloat16_rn(acc * inv);
  }
}

static int g_tm_max_heads = 8;
static int g_tm_rows = 0;      // 0: 32 rows a tile where they fit, else 16; 16 or 32: only that

// Heads a CTA and rows a tile.  The most heads that fit with the given rows (fewer CTAs a cluster: what crosses
// between the SMs of a cluster falls with their number); hc = 0 if no split of the heads fits.
struct TmShape {
  int hc, rows;
};
static TmShape tm_shape_rows(int H, int G, int D, int Dv, int rows) {
  if (g_tm_rows != 0 && rows != g_tm_rows) return {0, 0};
  for (int hc = 8; hc >= 1; --hc) {
    if (H % hc != 0 || hc > g_tm_max_heads) continue;
    const int c = H / hc;
    if (c != 1 && c != 2 && c != 4 && c != 8) continue;
    if (hc * Dv * rows > 512 * 32) continue;            // 64 accumulators a thread
    if (tm_layout(H, G, D, Dv, hc, rows).total > 227 * 1024) continue;
    return {hc, rows};
  }
  return {0, 0};
}
// Steps of single rows take tiles of 16 rows (a tile holds one row, and more heads a CTA fit).  Prompt portions
// take tiles of 32 rows, unless that makes clusters of 8 CTAs where tiles of 16 rows make smaller ones (measured,
// a prompt of 2,048 tokens at head size 128: 205 / 319 / 842 us a layer with 32 rows and 4 heads a CTA at 8 / 16 /
// 32 heads, 241 / 360 / 735 us with 16 rows and 8 heads a CTA).
static TmShape tm_shape(int H, int G, int D, int Dv, bool single) {
  if (H <= 0 || G <= 0 || H % G != 0 || D < 16 || Dv < 16 || D % 16 != 0 || Dv % 16 != 0) return {0, 0};
  const TmShape tall = tm_shape_rows(H, G, D, Dv, 32), flat = tm_shape_rows(H, G, D, Dv, 16);
  if (tall.hc == 0) return flat;
  if (flat.hc == 0) return tall;
  if (single) return flat;
  return (H / tall.hc == 8 && H / flat.hc < 8) ? flat : tall;
}

}  // namespace nf

using namespace nf;

// The heads a CTA of the tensor-core kernel takes at these sizes (a tile's cluster is H / that many CTAs);
// 0: the kernel does not take them, and the plain kernel serves.
// `single`: for a step whose segments bring one row each.
extern "C" int nf_talking_attention_mma_heads_per_cta(int H, int G, int D, int Dv, int single) {
  return tm_shape(H, G, D, Dv, single != 0).hc;
}
// ... and the rows of its tiles (32 or 16).
extern "C" int nf_talking_attention_mma_tile_rows(int H, int G, int D, int Dv, int single) {
  return tm_shape(H, G, D, Dv, single != 0).rows;
}
// Tiles of 16 or of 32 rows only; 0: the larger that fits.
extern "C" int nf_set_talking_attention_mma_tile_rows(int rows) {
  g_tm_rows = rows == 16 || rows == 32 ? rows : 0;
  return 0;
}

// At most this many heads a CTA (1 to 8): fewer heads make larger clusters of lighter CTAs.
extern "C" int nf_set_talking_attention_mma_max_heads(int n) {
  g_tm_max_heads = n < 1 ? 1 : n > 8 ? 8 : n;
  return 0;
}

extern "C" int nf_talking_attention_mma(const void* q, const void* pages, const int* block_table, int bt_width,
                                        const int* positions, const int* seg_row0, const int* tiles, int n_tiles,
                                        const float* talk, const float* sink, void* out, float* ws_o, float* ws_ml,
                                        int T, int H, int G, int D, int Dv, int page_size, int num_pages, int chunk,
                                        float scale, int nsplit, int blocks_per_split, cudaStream_t stream) {
  if (T == 0 || n_tiles == 0) return 0;
  const TmShape shape = tm_shape(H, G, D, Dv, tiles == nullptr);
  const int hc = shape.hc;
  NF_REQUIRE(hc > 0, "talking attention (tensor cores): sizes H=%d G=%d D=%d Dv=%d do not fit", H, G, D, Dv);
  NF_REQUIRE(chunk >= 0 && page_size > 0 && nsplit >= 1 && blocks_per_split >= 1, "talking attention: bad chunk, page size or split");
  NF_REQUIRE((ws_o == nullptr) == (ws_ml == nullptr), "talking attention: one workspace without the other");
  NF_REQUIRE(ws_o || nsplit == 1, "talking attention: runs of keys need the workspace");
  const int C = H / hc;
  const size_t smem = tm_layout(H, G, D, Dv, hc, shape.rows).total;
  const dim3 grid(n_tiles * C, nsplit);
  const int units = hc * (Dv / 16);
  const __nv_bfloat16* qq = (const __nv_bfloat16*)q;
  const __nv_bfloat16* pg = (const __nv_bfloat16*)pages;
#define NF_TM(HC, NU, ROWS)                                                                                           \
  do {                                                                                                                \
    cudaFuncSetAttribute(talking_attention_mma_kernel<HC, NU, ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                         (int)smem);                                                                                  \
    launch_chained_cluster(talking_attention_mma_kernel<HC, NU, ROWS>, grid, dim3(kTmThreads), smem, stream, C, qq,   \
                           pg, block_table, bt_width, positions, seg_row0, tiles, talk, sink, (__nv_bfloat16*)out,    \
                           ws_o, ws_ml, H, G, D, Dv, page_size, num_pages, chunk, scale, nsplit, blocks_per_split);   \
  } while (0)
#define NF_TM_HC(HC)                                   \
  do {                                                 \
    if (shape.rows == 32) {                            \
      if (units <= 8) NF_TM(HC, 1, 32);                \
      else if (units <= 16) NF_TM(HC, 2, 32);          \
      else NF_TM(HC, 4, 32);                           \
    } else {                                           \
      if (units <= 16) NF_TM(HC, 2, 16);               \
      else if (units <= 32) NF_TM(HC, 4, 16);          \
      else NF_TM(HC, 8, 16);                           \
    }                                                  \
  } while (0)
  switch (hc) {
    case 1: NF_TM_HC(1); break;
    case 2: NF_TM_HC(2); break;
    case 3: NF_TM_HC(3); break;
    case 4: NF_TM_HC(4); break;
    case 5: NF_TM_HC(5); break;
    case 6: NF_TM_HC(6); break;
    case 7: NF_TM_HC(7); break;
    default: NF_TM_HC(8); break;
  }
#undef NF_TM_HC
#undef NF_TM
  if (ws_o)
    launch_chained(talking_attention_merge_kernel, dim3(T * H), dim3(64), 0, stream, (const float*)ws_o,
                   (const float*)ws_ml, sink, (__nv_bfloat16*)out, H, Dv, nsplit);
  return check_launch("talking_attention_mma");
}
