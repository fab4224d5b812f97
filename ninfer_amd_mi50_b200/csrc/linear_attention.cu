// Linear attention with a fixed decay per head: a recurrence over each request's rows, from and
// into the request's state slot.
//
//   S_t = g_h S_{t-1} + k_t v_t^T        (S is D x V per head, float32, zero for a new request)
//   o_t = S_t^T q_t
//
// q, k (heads x D) and v (heads x V) are column ranges of one projection.  Before they enter the
// recurrence they may pass SiLU (all three), a rotation of the first `rot` dimensions of every
// q and k head (pair (i, i + rot/2) by the angle pos * f_i), and k a scale.  Everything after
// the projection is float32: angles, the rotated and scaled vectors, the state, the sums.
//
// One CTA of 128 threads serves 128 / LANES value columns of one (request, head) and walks the
// request's rows of the step in order.  A column's D state entries lie in the registers of LANES
// lanes (8, or 16 for heads wider than 64), EPL consecutive entries a lane.  The step's q, k, v
// are staged CH tokens at a time in shared memory (activation, rotation and scale applied while
// staging), so the token loop itself has no block-wide barrier; the next chunk's raw values are
// asked for before the current chunk's token loop and wait in registers, so that their way from
// memory lies under the arithmetic.  A lane reads its entries of k and q as 16-byte pieces (rows
// padded by 4 floats every EPL, which keeps the lanes of a column on different banks); the sum
// over a column is log2(LANES) shuffles.  A token's result depends on earlier tokens only
// through S, which holds the same bits however the request was cut.
//
// The state of a slot is laid out [head][value column][D]: a column's entries are contiguous, so
// the lanes of a column read and write whole 32-byte sectors.
//
// The same kernel serves a matrix-memory recurrence with gates a row (mLSTM): the decay, a factor on
// k v^T and a factor on the output are then numbers a (row, head), which a pass of its own
// (`mlstm_gates_kernel`: capped exponential gates, a running maximum, the normaliser) leaves for it.
#define NF_CHAIN_CLASS 2
#include "common.cuh"

namespace nf {

constexpr int kLaThreads = 128;

__device__ __forceinline__ float la_act(float x, int use_silu) { return use_silu ? x / (1.f + expf(-x)) : x; }
// One rotated pair of q and of k (already through `la_act`), by the angle pos * f, k scaled after
// the turn.  The products are written out so that both kernels below round alike.
__device__ __forceinline__ void la_turn(float q0, float q1, float k0, float k1, float angle, float k_scale, float q_scale,
                                        float& oq0, float& oq1, float& ok0, float& ok1) {
  const float cs = cosf(angle), sn = sinf(angle);
  oq0 = __fmul_rn(__fsub_rn(__fmul_rn(q0, cs), __fmul_rn(q1, sn)), q_scale);      // (a scale of 1 changes no bit)
  oq1 = __fmul_rn(__fadd_rn(__fmul_rn(q1, cs), __fmul_rn(q0, sn)), q_scale);
  ok0 = __fmul_rn(__fsub_rn(__fmul_rn(k0, cs), __fmul_rn(k1, sn)), k_scale);
  ok1 = __fmul_rn(__fadd_rn(__fmul_rn(k1, cs), __fmul_rn(k0, sn)), k_scale);
}

// For steps with prompt portions: q and k of every row, activated, turned and scaled ONCE, as
// float32 [T, q: H x D | k: H x D].  (The recurrence kernel's CTAs each serve a few value columns
// of a head; left to them, every one of them would repeat this work for the whole head.)
template <typename T>
__global__ void linear_attention_prepare_kernel(const T* __restrict__ src, int ld, int q_col0, int k_col0,
                                                const float* __restrict__ inv_freq, int rot, float k_scale, float q_scale,
                                                int use_silu, const int* __restrict__ positions, float* __restrict__ out,
                                                int H, int D) {
  const int t = blockIdx.x;
  chain_wait(src);
  const int half = rot / 2, units = half + (D - rot);
  const T* row = src + (size_t)t * ld;
  float* o = out + (size_t)t * 2 * H * D;
  const float fpos = (float)positions[t];
  for (int x = blockIdx.y * blockDim.x + threadIdx.x; x < H * units; x += gridDim.y * blockDim.x) {
    const int head = x / units, u = x - head * units;
    const int base = head * D;
    if (u < half) {
      float a, b, c, d;
      la_turn(la_act(to_float(row[q_col0 + base + u]), use_silu), la_act(to_float(row[q_col0 + base + u + half]), use_silu),
              la_act(to_float(row[k_col0 + base + u]), use_silu), la_act(to_float(row[k_col0 + base + u + half]), use_silu),
              fpos * inv_freq[u], k_scale, q_scale, a, b, c, d);
      o[base + u] = a; o[base + u + half] = b;
      o[H * D + base + u] = c; o[H * D + base + u + half] = d;
    } else {
      const int i = rot + (u - half);
      o[base + i] = __fmul_rn(la_act(to_float(row[q_col0 + base + i]), use_silu), q_scale);
      o[H * D + base + i] = __fmul_rn(la_act(to_float(row[k_col0 + base + i]), use_silu), k_scale);
    }
  }
}

// PREP: q and k come from `prepared` (float32, final; D a multiple of 4), four dimensions a copy.
// GATED: the decay is not a constant of the head but a number a (row, head), and so are a factor on
// the row's k v^T and one on its output: S_t = a_t S_{t-1} + b_t k_t v_t^T, o_t = c_t S_t^T q_t, with
// (a_t, b_t, c_t) at gates[(t * H + head) * 3] (what `mlstm_gates_kernel` below leaves).
template <typename T, int EPL, int LANES, int CH, bool PREP, bool GATED>    // D <= LANES * EPL; CH tokens staged at a time
__global__ void __launch_bounds__(kLaThreads)
decay_linear_attention_kernel(const T* __restrict__ src, int ld, int q_col0, int k_col0, int v_col0,
                              const float* __restrict__ decay, const float* __restrict__ inv_freq, int rot,
                              float k_scale, float q_scale, int use_silu, float* __restrict__ state, long slot_stride,
                              const int* __restrict__ seg_row0, const int* __restrict__ seg_slot,
                              const int* __restrict__ seg_pos0, float* __restrict__ out, int H, int D, int V,
                              const float* __restrict__ prepared, const float* __restrict__ gates) {
  constexpr int COLS = kLaThreads / LANES;                 // value columns a CTA
  constexpr bool VEC = EPL % 4 == 0;
  constexpr int PAD = VEC ? 4 : 0;
  constexpr int DPAD = LANES * EPL;                        // D rounded up
  constexpr int DP = LANES * (EPL + PAD);                  // padded row of q or k in shared memory
  constexpr int RMAX = (CH * DPAD + kLaThreads - 1) / kLaThreads;    // staging units a thread
  constexpr int VMAX = (CH * COLS + kLaThreads - 1) / kLaThreads;
  __shared__ __align__(16) float sq[CH][DP];
  __shared__ __align__(16) float sk[CH][DP];
  __shared__ float sv[CH][COLS];
  __shared__ float sg[GATED ? CH : 1][3];
  const int seg = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * COLS;
  const int tid = threadIdx.x, lane = tid % LANES, cidx = tid / LANES, col = col0 + cidx;
  const bool live = col < V;
  chain_release_if_small();
  chain_wait(src, state, prepared, gates);
  const int row0 = seg_row0[seg], rows = seg_row0[seg + 1] - row0;
  const int pos0 = seg_pos0[seg];
  const float g = GATED ? 0.f : decay[head];
  float* sp = state + (size_t)seg_slot[seg] * slot_stride + ((size_t)head * V + (live ? col : 0)) * D + lane * EPL;
  float s[EPL];
  const bool vec_state = VEC && D % 4 == 0 && (slot_stride % 4 == 0) && ((uintptr_t)state % 16 == 0);
  if (vec_state) {
#pragma unroll
    for (int e = 0; e < EPL; e += 4) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (live && lane * EPL + e < D) v = *reinterpret_cast<const float4*>(sp + e);
      s[e] = v.x; s[e + 1] = v.y; s[e + 2] = v.z; s[e + 3] = v.w;
    }
  } else {
#pragma unroll
    for (int e = 0; e < EPL; ++e) s[e] = (live && lane * EPL + e < D) ? sp[e] : 0.f;
  }
  const int half = rot / 2;
  auto at = [](int i) { return i + PAD * (i / EPL); };      // where dimension i lies in a padded row
  // A staging unit is a rotated pair (u, u + rot/2) for u < rot/2, or the single dimension
  // rot + (u - rot/2) beyond; unit x of a chunk belongs to token x / DPAD.
  const int units = half + (DPAD - rot);
  // raw values wait in registers unconverted, so that nothing has to wait for them before its time
  constexpr int RRAW = PREP ? 1 : RMAX;
  constexpr int RP = PREP ? (CH * (DPAD / 4) + kLaThreads - 1) / kLaThreads : 1;
  T rq0[RRAW], rq1[RRAW], rk0[RRAW], rk1[RRAW], rv[VMAX];
  float4 fq[RP], fk[RP];
  float rg[3] = {0.f, 0.f, 0.f};
  auto fetch = [&](int c0, int n) {
    if constexpr (GATED) {
      if (tid < n) {
        const float* gp = gates + ((size_t)(row0 + c0 + tid) * H + head) * 3;
        rg[0] = gp[0]; rg[1] = gp[1]; rg[2] = gp[2];
      }
    }
    if constexpr (PREP) {
#pragma unroll
      for (int r = 0; r < RP; ++r) {
        const int x = tid + r * kLaThreads, t = x / (DPAD / 4), i = 4 * (x - t * (DPAD / 4));
        fq[r] = fk[r] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t < n && i < D) {
          const float* row = prepared + (size_t)(row0 + c0 + t) * 2 * H * D + (size_t)head * D + i;
          fq[r] = *reinterpret_cast<const float4*>(row);
          fk[r] = *reinterpret_cast<const float4*>(row + (size_t)H * D);
        }
      }
    } else {
#pragma unroll
      for (int r = 0; r < RMAX; ++r) {
        const int x = tid + r * kLaThreads, t = x / DPAD, u = x - t * DPAD;
        rq0[r] = rq1[r] = rk0[r] = rk1[r] = from_float<T>(0.f);
        if (t < n && u < units) {
          const int i0 = u < half ? u : rot + (u - half);
          const T* row = src + (size_t)(row0 + c0 + t) * ld + (size_t)head * D;
          if (i0 < D) { rq0[r] = row[q_col0 + i0]; rk0[r] = row[k_col0 + i0]; }
          if (u < half) { rq1[r] = row[q_col0 + u + half]; rk1[r] = row[k_col0 + u + half]; }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < VMAX; ++r) {
      const int x = tid + r * kLaThreads, t = x / COLS, j = x - t * COLS;
      rv[r] = from_float<T>(0.f);
      if (t < n && col0 + j < V) rv[r] = src[(size_t)(row0 + c0 + t) * ld + v_col0 + (size_t)head * V + col0 + j];
    }
  };
  auto stage = [&](int c0, int n) {
    if constexpr (GATED) {
      if (tid < n) { sg[tid][0] = rg[0]; sg[tid][1] = rg[1]; sg[tid][2] = rg[2]; }
    }
    if constexpr (PREP) {
#pragma unroll
      for (int r = 0; r < RP; ++r) {
        const int x = tid + r * kLaThreads, t = x / (DPAD / 4), i = 4 * (x - t * (DPAD / 4));
        if (t < n) {                                       // (dimensions from D to DPAD get zeros)
          *reinterpret_cast<float4*>(&sq[t][at(i)]) = fq[r];
          *reinterpret_cast<float4*>(&sk[t][at(i)]) = fk[r];
        }
      }
    } else {
#pragma unroll
      for (int r = 0; r < RMAX; ++r) {
        const int x = tid + r * kLaThreads, t = x / DPAD, u = x - t * DPAD;
        if (t < n && u < units) {
          const int i0 = u < half ? u : rot + (u - half);   // (dimensions from D to DPAD hold zeros)
          if (u < half) {
            float a, b, c, d;
            la_turn(la_act(to_float(rq0[r]), use_silu), la_act(to_float(rq1[r]), use_silu), la_act(to_float(rk0[r]), use_silu),
                    la_act(to_float(rk1[r]), use_silu), (float)(pos0 + c0 + t) * inv_freq[u], k_scale, q_scale, a, b, c, d);
            sq[t][at(u)] = a; sq[t][at(u + half)] = b;
            sk[t][at(u)] = c; sk[t][at(u + half)] = d;
          } else {
            sq[t][at(i0)] = __fmul_rn(la_act(to_float(rq0[r]), use_silu), q_scale);
            sk[t][at(i0)] = __fmul_rn(la_act(to_float(rk0[r]), use_silu), k_scale);
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < VMAX; ++r) {
      const int x = tid + r * kLaThreads, t = x / COLS, j = x - t * COLS;
      if (t < n) sv[t][j] = la_act(to_float(rv[r]), use_silu);
    }
  };
  fetch(0, min(CH, rows));
  for (int c0 = 0; c0 < rows; c0 += CH) {
    const int n = min(CH, rows - c0);
    __syncthreads();                                       // the previous chunk has been read
    stage(c0, n);
    __syncthreads();
    if (c0 + CH < rows) fetch(c0 + CH, min(CH, rows - c0 - CH));      // in flight during the token loop
    const float* kq0 = &sk[0][lane * (EPL + PAD)];
    const float* qq0 = &sq[0][lane * (EPL + PAD)];
#pragma unroll 2
    for (int t = 0; t < n; ++t) {
      float v = sv[t][cidx];
      float g_t = g;
      if constexpr (GATED) { g_t = sg[t][0]; v *= sg[t][1]; }
      const float* kr = kq0 + t * DP;
      const float* qr = qq0 + t * DP;
      float o = 0.f;
      if (VEC) {
#pragma unroll
        for (int e = 0; e < EPL; e += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(kr + e);
          const float4 q4 = *reinterpret_cast<const float4*>(qr + e);
          s[e] = fmaf(g_t, s[e], k4.x * v);         o = fmaf(s[e], q4.x, o);
          s[e + 1] = fmaf(g_t, s[e + 1], k4.y * v); o = fmaf(s[e + 1], q4.y, o);
          s[e + 2] = fmaf(g_t, s[e + 2], k4.z * v); o = fmaf(s[e + 2], q4.z, o);
          s[e + 3] = fmaf(g_t, s[e + 3], k4.w * v); o = fmaf(s[e + 3], q4.w, o);
        }
      } else {
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
          s[e] = fmaf(g_t, s[e], kr[e] * v);
          o = fmaf(s[e], qr[e], o);
        }
      }
#pragma unroll
      for (int w = LANES / 2; w > 0; w >>= 1) o += __shfl_xor_sync(0xffffffffu, o, w);
      if constexpr (GATED) o *= sg[t][2];
      if (live && lane == 0) out[(size_t)(row0 + c0 + t) * H * V + (size_t)head * V + col] = o;
    }
  }
  if (live) {
    if (vec_state) {
#pragma unroll
      for (int e = 0; e < EPL; e += 4)
        if (lane * EPL + e < D) *reinterpret_cast<float4*>(sp + e) = make_float4(s[e], s[e + 1], s[e + 2], s[e + 3]);
    } else {
#pragma unroll
      for (int e = 0; e < EPL; ++e)
        if (lane * EPL + e < D) sp[e] = s[e];
    }
  }
}


// The gates of a matrix-memory recurrence (mLSTM) with exponential gating, stabilised by a running
// maximum, and its normaliser.  Per (request, head), from and into the request's state slot:
//
//   i_t = cap tanh((x_i + b_i) / cap)                     log input gate    (x_i, x_f: the row's gate projections)
//   f_t = logsigmoid(cap tanh((x_f + b_f) / cap))         log forget gate
//   m_t = max(f_t + m_{t-1}, i_t)                         (m starts at 0)
//   a_t = exp(f_t + m_{t-1} - m_t),  b_t = exp(i_t - m_t)
//   n_t = a_t n_{t-1} + b_t k_t                           (n starts at 0)
//   c_t = 1 / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)        q_t = q * q_scale
//
// and leaves (a_t, b_t, c_t) at gates[(t * H + head) * 3], with which the recurrence kernel above runs
// S_t = a_t S_{t-1} + b_t k_t v_t^T, o_t = c_t S_t^T q_t.  One warp a (request, head) walks the rows in
// order, 32 at a time: lane j works out row j's gates (the tanh, the logarithm and the exponentials of 32
// rows at once), the maximum then runs through the lanes by shuffles, and the normaliser through the rows
// with a few rows' q and k in flight at a time; n lies in the lanes' registers (dimension lane + 32 e), a
// row's n . q is added up from the lanes' shares in lane order.  Everything is float32; a row's numbers
// depend on earlier rows only through (n, m), and every sum runs in an order of its own row's making, so
// they hold the same bits however the request was cut.  cap <= 0: the gate projections enter uncapped.
template <typename T, int NE>               // D <= 32 NE
__global__ void __launch_bounds__(32)
mlstm_gates_kernel(const T* __restrict__ src, int ld, int q_col0, int k_col0, float q_scale,
                   const float* __restrict__ pre, int ldp, int i_col0, int f_col0, const float* __restrict__ bias_i,
                   const float* __restrict__ bias_f, float cap, float* __restrict__ state_n,
                   float* __restrict__ state_m, long slot_stride, const int* __restrict__ seg_row0,
                   const int* __restrict__ seg_slot, float* __restrict__ gates, int H, int D) {
  constexpr int GROUP = NE <= 2 ? 16 : (NE <= 4 ? 8 : 4);    // rows whose q and k are in flight together (two such groups)
  __shared__ float part[32][33];               // a lane's share of every token's n . q
  const int seg = blockIdx.x, head = blockIdx.y, lane = threadIdx.x;
  chain_release_if_small();
  chain_wait(src, pre, state_n, state_m);
  const int row0 = seg_row0[seg], rows = seg_row0[seg + 1] - row0;
  float* np = state_n + (size_t)seg_slot[seg] * slot_stride + (size_t)head * D;
  float* mp = state_m + (size_t)seg_slot[seg] * slot_stride + head;
  float n[NE];
#pragma unroll
  for (int j = 0; j < NE; ++j) n[j] = lane + 32 * j < D ? np[lane + 32 * j] : 0.f;
  float m = *mp;
  const float bi = bias_i ? bias_i[head] : 0.f, bf = bias_f ? bias_f[head] : 0.f;
  // 32 rows at a time: lane j has row c0 + j's gates; the maximum runs through the lanes in order, the
  // normaliser through the rows in order, and a row's n . q meets in shared memory.  Loads run ahead of their
  // use: the next 32 rows' gate projections during this chunk, the chunk's first two groups of q and k during the
  // gates' arithmetic (up to 64 dimensions a head that is the whole chunk), a later group's during the group before it.
  auto load_pre = [&](int c0, float& xi, float& xf) {
    const int cn = min(32, rows - c0);
    const size_t r = (size_t)(row0 + c0 + min(lane, cn - 1));
    xi = pre[r * ldp + i_col0 + head];
    xf = pre[r * ldp + f_col0 + head];
  };
  auto load_qk = [&](float (&kb)[GROUP][NE], float (&qb)[GROUP][NE], int c0, int cn, int j0) {
#pragma unroll
    for (int g = 0; g < GROUP; ++g) {
      const size_t rr = (size_t)(row0 + c0 + min(j0 + g, cn - 1));
      const T* qr = src + rr * ld + q_col0 + (size_t)head * D;
      const T* kr = src + rr * ld + k_col0 + (size_t)head * D;
#pragma unroll
      for (int e = 0; e < NE; ++e) {
        const int d = lane + 32 * e;
        kb[g][e] = d < D ? to_float(kr[d]) : 0.f;
        qb[g][e] = d < D ? __fmul_rn(to_float(qr[d]), q_scale) : 0.f;
      }
    }
  };
  float xi_next = 0.f, xf_next = 0.f;
  if (rows > 0) load_pre(0, xi_next, xf_next);
  for (int c0 = 0; c0 < rows; c0 += 32) {
    const int cn = min(32, rows - c0);
    float kA[GROUP][NE], qA[GROUP][NE], kB[GROUP][NE], qB[GROUP][NE];
    load_qk(kA, qA, c0, cn, 0);
    if (GROUP < cn) load_qk(kB, qB, c0, cn, GROUP);
    float xi = xi_next + bi, xf = xf_next + bf;
    if (c0 + 32 < rows) load_pre(c0 + 32, xi_next, xf_next);
    if (cap > 0.f) { xi = cap * tanhf(xi / cap); xf = cap * tanhf(xf / cap); }
    const float f = fminf(xf, 0.f) - log1pf(expf(-fabsf(xf)));
    float m_before = m, m_mine = m;
    for (int j = 0; j < cn; ++j) {
      const float fj = __shfl_sync(0xffffffffu, f, j), ij = __shfl_sync(0xffffffffu, xi, j);
      const float m_new = fmaxf(fj + m, ij);
      if (lane == j) { m_before = m; m_mine = m_new; }
      m = m_new;
    }
    const float a = expf(f + m_before - m_mine), b = expf(xi - m_mine);
    auto run_group = [&](float (&kb)[GROUP][NE], float (&qb)[GROUP][NE], int j0) {
#pragma unroll
      for (int g = 0; g < GROUP; ++g) {
        const int j = j0 + g;
        if (j < cn) {
          const float aj = __shfl_sync(0xffffffffu, a, j), bj = __shfl_sync(0xffffffffu, b, j);
          float dot = 0.f;
#pragma unroll
          for (int e = 0; e < NE; ++e) {
            n[e] = fmaf(aj, n[e], bj * kb[g][e]);
            dot = fmaf(n[e], qb[g][e], dot);
          }
          part[j][lane] = dot;
        }
      }
    };
    for (int j0 = 0; j0 < cn; j0 += 2 * GROUP) {
      run_group(kA, qA, j0);
      if (j0 + 2 * GROUP < cn) load_qk(kA, qA, c0, cn, j0 + 2 * GROUP);
      if (j0 + GROUP < cn) run_group(kB, qB, j0 + GROUP);
      if (j0 + 3 * GROUP < cn) load_qk(kB, qB, c0, cn, j0 + 3 * GROUP);
    }
    __syncwarp();
    if (lane < cn) {
      float dot = 0.f;
#pragma unroll 8
      for (int l = 0; l < 32; ++l) dot += part[lane][l];
      float* gp = gates + ((size_t)(row0 + c0 + lane) * H + head) * 3;
      gp[0] = a; gp[1] = b;
      gp[2] = 1.f / (fmaxf(fabsf(dot), expf(-m_mine)) + 1e-6f);
    }
    __syncwarp();
  }
#pragma unroll
  for (int j = 0; j < NE; ++j)
    if (lane + 32 * j < D) np[lane + 32 * j] = n[j];
  if (lane == 0) *mp = m;
}

template <typename T, int EPL, int LANES, int CH, bool PREP>
static void launch_la(const void* src, int ld, int q0, int k0, int v0, const float* decay, const float* inv_freq,
                      int rot, float k_scale, float q_scale, int use_silu, float* state, long long slot_stride,
                      const int* seg_row0, const int* seg_slot, const int* seg_pos0, float* out, int S, int H, int D,
                      int V, const float* prepared, const float* gates, cudaStream_t stream) {
  constexpr int COLS = kLaThreads / LANES;
  dim3 grid(S, H, (V + COLS - 1) / COLS);
  if (gates)
    launch_chained(decay_linear_attention_kernel<T, EPL, LANES, CH, PREP, true>, grid, dim3(kLaThreads), 0, stream, (const T*)src, ld,
                   q0, k0, v0, decay, inv_freq, rot, k_scale, q_scale, use_silu, state, (long)slot_stride, seg_row0, seg_slot,
                   seg_pos0, out, H, D, V, prepared, gates);
  else
    launch_chained(decay_linear_attention_kernel<T, EPL, LANES, CH, PREP, false>, grid, dim3(kLaThreads), 0, stream, (const T*)src, ld,
                   q0, k0, v0, decay, inv_freq, rot, k_scale, q_scale, use_silu, state, (long)slot_stride, seg_row0, seg_slot,
                   seg_pos0, out, H, D, V, prepared, gates);
}

template <typename T>
static int dispatch_la(const void* src, int ld, int q0, int k0, int v0, const float* decay, const float* inv_freq,
                       int rot, float k_scale, float q_scale, int use_silu, float* state, long long slot_stride,
                       const int* seg_row0, const int* seg_slot, const int* seg_pos0, float* out, int S, int H, int D,
                       int V, const float* prepared, const float* gates, int single, cudaStream_t stream) {
#define NF_LA(E, L, C, P)                                                                                          \
  launch_la<T, E, L, C, P>(src, ld, q0, k0, v0, decay, inv_freq, rot, k_scale, q_scale, use_silu, state, slot_stride, \
                           seg_row0, seg_slot, seg_pos0, out, S, H, D, V, prepared, gates, stream)
  // single: every segment brings one row (a decode step): one token staged at a time, few registers
  if (prepared) {
    if (D <= 32) NF_LA(4, 8, 16, true);
    else if (D <= 64) NF_LA(8, 8, 16, true);
    else if (D <= 128) NF_LA(8, 16, 16, true);
    else NF_LA(16, 16, 8, true);
  } else if (single) {
    if (D <= 8) NF_LA(1, 8, 1, false);
    else if (D <= 16) NF_LA(2, 8, 1, false);
    else if (D <= 32) NF_LA(4, 8, 1, false);
    else if (D <= 64) NF_LA(8, 8, 1, false);
    else if (D <= 128) NF_LA(8, 16, 1, false);
    else NF_LA(16, 16, 1, false);
  } else {
    if (D <= 8) NF_LA(1, 8, 16, false);
    else if (D <= 16) NF_LA(2, 8, 16, false);
    else if (D <= 32) NF_LA(4, 8, 16, false);
    else if (D <= 64) NF_LA(8, 8, 16, false);
    else if (D <= 128) NF_LA(8, 16, 16, false);
    else NF_LA(16, 16, 8, false);
  }
#undef NF_LA
  return check_launch("decay_linear_attention");
}

}  // namespace nf

using namespace nf;

extern "C" int nf_decay_linear_attention_max_dim() { return 256; }

// src [T, ld] holds q at q_col0 (H x D), k at k_col0 (H x D), v at v_col0 (H x V); decay float32 [H];
// inv_freq float32 [rot / 2] (rot 0: nothing is turned); state float32, slot s at state + s * slot_stride,
// [H][V][D]; out float32 [T, H * V].  prepared: null, or what nf_linear_attention_prepare made of the
// same rows (q and k are then taken from there as they are; D a multiple of 4 above 16).  single != 0:
// every segment brings one row.
// gates: null, or float32 [T, H, 3] of (decay, factor on k v^T, factor on the output) a (row, head), which
// then stand in for `decay` (which may be null).  q_scale multiplies q after the turn, as k_scale does k.
extern "C" int nf_decay_linear_attention(const void* src, int ld, int q_col0, int k_col0, int v_col0,
                                         const float* decay, const float* inv_freq, int rot, float k_scale,
                                         int use_silu, float* state, long long slot_stride, const int* seg_row0,
                                         const int* seg_slot, const int* seg_pos0, float* out, int S, int H, int D,
                                         int V, int dtype, const float* prepared, int single, float q_scale,
                                         const float* gates, cudaStream_t stream) {
  if (S == 0) return 0;
  NF_REQUIRE(decay || gates, "linear attention: neither a decay a head nor gates a row");
  NF_REQUIRE(S > 0 && H > 0 && D > 0 && V > 0 && D <= 256, "linear attention: bad sizes S=%d H=%d D=%d V=%d", S, H, D, V);
  NF_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= D && (rot == 0 || inv_freq), "linear attention: rot=%d with D=%d", rot, D);
  NF_REQUIRE(H <= 65535 && (V + 7) / 8 <= 65535, "linear attention: too many heads or columns");
  NF_REQUIRE(!prepared || (D % 4 == 0 && D > 16 && (uintptr_t)prepared % 16 == 0), "linear attention: prepared q and k need D a multiple of 4 above 16");
  if (dtype == kF32)
    return dispatch_la<float>(src, ld, q_col0, k_col0, v_col0, decay, inv_freq, rot, k_scale, q_scale, use_silu, state,
                              slot_stride, seg_row0, seg_slot, seg_pos0, out, S, H, D, V, prepared, gates, single, stream);
  return dispatch_la<__nv_bfloat16>(src, ld, q_col0, k_col0, v_col0, decay, inv_freq, rot, k_scale, q_scale, use_silu, state,
                                    slot_stride, seg_row0, seg_slot, seg_pos0, out, S, H, D, V, prepared, gates, single, stream);
}

// out float32 [T, 2 H D]: q then k of every row, activated, turned by positions[t] and (k) scaled.
extern "C" int nf_linear_attention_prepare(const void* src, int ld, int q_col0, int k_col0, const float* inv_freq, int rot,
                                           float k_scale, int use_silu, const int* positions, float* out, int T, int H,
                                           int D, int dtype, float q_scale, cudaStream_t stream) {
  if (T == 0) return 0;
  NF_REQUIRE(T > 0 && H > 0 && D > 0 && rot >= 0 && rot % 2 == 0 && rot <= D && (rot == 0 || inv_freq),
             "linear attention prepare: bad sizes T=%d H=%d D=%d rot=%d", T, H, D, rot);
  const int units = H * (rot / 2 + D - rot);
  const dim3 grid(T, (units + 1023) / 1024 < 1 ? 1 : (units + 1023) / 1024);
  if (dtype == kF32)
    launch_chained(linear_attention_prepare_kernel<float>, grid, dim3(256), 0, stream, (const float*)src, ld, q_col0, k_col0, inv_freq, rot, k_scale, q_scale, use_silu, positions, out, H, D);
  else
    launch_chained(linear_attention_prepare_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (const __nv_bfloat16*)src, ld, q_col0, k_col0, inv_freq, rot, k_scale, q_scale, use_silu, positions, out, H, D);
  return check_launch("linear_attention_prepare");
}

// src [T, ld] holds q at q_col0 and k at k_col0 (H x D each, as the recurrence reads them); pre float32
// [T, ldp] holds the gate projections of the H heads at i_col0 and f_col0; bias_i, bias_f float32 [H] or
// null; state_n (slot s at + s * slot_stride: [H][D]) and state_m ([H]) float32; gates float32 [T, H, 3].
extern "C" int nf_mlstm_gates(const void* src, int ld, int q_col0, int k_col0, float q_scale, const float* pre, int ldp,
                              int i_col0, int f_col0, const float* bias_i, const float* bias_f, float cap,
                              float* state_n, float* state_m, long long slot_stride, const int* seg_row0,
                              const int* seg_slot, float* gates, int S, int H, int D, int dtype, cudaStream_t stream) {
  if (S == 0) return 0;
  NF_REQUIRE(S > 0 && H > 0 && H <= 65535 && D > 0 && D <= 256, "mlstm gates: bad sizes S=%d H=%d D=%d", S, H, D);
  NF_REQUIRE(i_col0 >= 0 && f_col0 >= 0 && i_col0 + H <= ldp && f_col0 + H <= ldp, "mlstm gates: the gate columns leave their rows");
#define NF_MG(TT, NE_)                                                                                              \
  launch_chained(mlstm_gates_kernel<TT, NE_>, dim3(S, H), dim3(32), 0, stream, (const TT*)src, ld, q_col0, k_col0, q_scale, \
                 pre, ldp, i_col0, f_col0, bias_i, bias_f, cap, state_n, state_m, (long)slot_stride, seg_row0, seg_slot, \
                 gates, H, D)
#define NF_MG_D(TT)              \
  if (D <= 32) NF_MG(TT, 1);     \
  else if (D <= 64) NF_MG(TT, 2); \
  else if (D <= 128) NF_MG(TT, 4); \
  else NF_MG(TT, 8)
  if (dtype == kF32) { NF_MG_D(float); } else { NF_MG_D(__nv_bfloat16); }
#undef NF_MG_D
#undef NF_MG
  return check_launch("mlstm_gates");
}
