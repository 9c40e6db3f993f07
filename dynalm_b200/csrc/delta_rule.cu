// The gated delta rule: a matrix state per head that forgets, corrects and then is read, token by token.
//
// Per token and head h (query/key head j = h / (H / G), key size d, value size e), all in float32:
//
//   q = q_j / sqrt(sum(q_j^2) + 1e-6) * d^(-1/2),   k = k_j / sqrt(sum(k_j^2) + 1e-6)
//   beta = sigmoid(b_h),   g = exp(-exp(A_h) * softplus(a_h + dt_h))
//   S <- g S;   u = beta (v_h - S^T k);   S <- S + k u^T;   o_h = S^T q            (S is d x e, it starts at zero)
//
// q, k and v come from the short convolution's output (columns q | k | v of a row), b, a and the output gate from the
// projection's row. What a request keeps is S of every head, float32 [H][d][e], at the head of its state row.
//
// Block = (slice of the e columns, head, request), 256 threads: four warps that compute and four that fetch.
// A column of S lies over P neighbouring lanes of a computing warp, lane p holding the R rows p R .. p R + R - 1 in
// registers; the two dot products of a token are finished by shuffles among those lanes. A request's tokens are
// walked in tiles of 16 held twice in shared memory: while the computing warps run a tile's tokens over their
// registers, the fetching warps write the next tile (queries and keys made unit vectors, a warp per token; the
// values of the block's columns; the two gates; k . q) and ask for the one after it, whose numbers then have a whole
// tile's time to arrive in their registers: no token waits for global memory. Both dot products of a
// token run over the state it found (S'^T q = g S^T q + u (k . q)), so one round of shuffles a token is enough.
// A lane's rows are R + 4 floats apart in shared memory, so that the P lanes' 16-byte loads fall into different banks.
//
// dl_head_norm_gate: out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * w * silu(gate[t, h, :]).
#include "common.cuh"

namespace dl {

constexpr int DR_TT = 16;
constexpr int DR_COMPUTE = 128;
constexpr int DR_THREADS = 256;

__device__ __forceinline__ float dr_softplus(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

template <int R, int P>
struct DrTile {
  static constexpr int RS = R + 4;                      // floats between two lanes' rows
  static constexpr int TS = P * RS;                     // floats of one token's query (or key)
  static constexpr int COLS = DR_COMPUTE / P;
  static constexpr int FLOATS = 2 * DR_TT * TS + DR_TT * COLS + 4 * DR_TT;      // q | k | v | g | beta | k.q | spare
};

// What a fetching thread holds of one tile between asking for it and writing it to shared memory.
template <typename T, int R, int P>
struct DrRaw {
  static constexpr int NT = DR_TT / 4;                  // tokens of a warp
  static constexpr int NL = (R * P + 31) / 32;          // a lane's numbers of one query (or key)
  static constexpr int NV = DR_TT * DrTile<R, P>::COLS / (DR_THREADS - DR_COMPUTE);
  T q[NT][NL], k[NT][NL], v[NV], b, a;                  // as they lie in memory: nothing waits for a load before the tile is written
};

// The fetching warps ask for tile [first_row, first_row + tn) of the request's rows: every load is issued, none is
// waited for. The tile is asked for one tile's time before it is written, so its numbers are there by then.
template <typename T, int R, int P>
__device__ __forceinline__ void dr_ask(DrRaw<T, R, P>& raw, const T* __restrict__ u, int u_stride, int q_at, int k_at,
                                       int v_at, const T* __restrict__ proj, int proj_stride, int b_at, int a_at,
                                       int first_row, int tn, int d, int e, int col0, int lt) {
  using L = DrTile<R, P>;
  using W = DrRaw<T, R, P>;
  const int lane = lt & 31, warp = lt >> 5;
  const T zero = from_float<T>(0.0f);
#pragma unroll
  for (int s = 0; s < W::NT; ++s) {
    const int tt = warp + 4 * s;
    const T* urow = u + static_cast<size_t>(first_row + max(min(tt, tn - 1), 0)) * u_stride;
#pragma unroll
    for (int c = 0; c < W::NL; ++c) {
      const int i = lane + 32 * c;
      const bool ok = tt < tn && i < d;
      raw.q[s][c] = ok ? urow[q_at + i] : zero;
      raw.k[s][c] = ok ? urow[k_at + i] : zero;
    }
  }
#pragma unroll
  for (int c = 0; c < W::NV; ++c) {
    const int idx = lt + (DR_THREADS - DR_COMPUTE) * c;
    const int tt = idx / L::COLS, col = col0 + idx % L::COLS;
    raw.v[c] = (tt < tn && col < e) ? u[static_cast<size_t>(first_row + tt) * u_stride + v_at + col] : zero;
  }
  raw.b = zero;
  raw.a = zero;
  if (lt < tn) {
    const T* prow = proj + static_cast<size_t>(first_row + lt) * proj_stride;
    raw.b = prow[b_at];
    raw.a = prow[a_at];
  }
}

// ... and write it into one of the two buffers: queries and keys as unit vectors (a warp per token), k . q, the
// values of the block's columns, the two gates.
template <typename T, int R, int P>
__device__ __forceinline__ void dr_put(const DrRaw<T, R, P>& raw, float* buf, int tn, int d, float q_scale, float decay_rate,
                                       float bias, int lt) {
  using L = DrTile<R, P>;
  using W = DrRaw<T, R, P>;
  float* sq = buf;
  float* sk = sq + DR_TT * L::TS;
  float* sv = sk + DR_TT * L::TS;
  float* sg = sv + DR_TT * L::COLS;
  float* sbeta = sg + DR_TT;
  float* skq = sbeta + DR_TT;
  const int lane = lt & 31, warp = lt >> 5;
#pragma unroll
  for (int s = 0; s < W::NT; ++s) {
    const int tt = warp + 4 * s;
    float qq = 0.0f, kk = 0.0f, kq = 0.0f, qf[W::NL], kf[W::NL];
#pragma unroll
    for (int c = 0; c < W::NL; ++c) {
      qf[c] = to_float(raw.q[s][c]);
      kf[c] = to_float(raw.k[s][c]);
      qq = fmaf(qf[c], qf[c], qq);
      kk = fmaf(kf[c], kf[c], kk);
      kq = fmaf(kf[c], qf[c], kq);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {                  // three sums side by side
      qq += __shfl_xor_sync(0xffffffffu, qq, o);
      kk += __shfl_xor_sync(0xffffffffu, kk, o);
      kq += __shfl_xor_sync(0xffffffffu, kq, o);
    }
    const float fq = q_scale / sqrtf(qq + 1e-6f), fk = 1.0f / sqrtf(kk + 1e-6f);
    if (lane == 0 && tt < tn) skq[tt] = kq * fq * fk;   // the unit key times the scaled unit query
#pragma unroll
    for (int c = 0; c < W::NL; ++c) {
      const int i = lane + 32 * c;
      if (tt < tn && i < d) {
        const int at = tt * L::TS + (i / R) * L::RS + i % R;
        sq[at] = qf[c] * fq;
        sk[at] = kf[c] * fk;
      }
    }
  }
#pragma unroll
  for (int c = 0; c < W::NV; ++c) {
    const int idx = lt + (DR_THREADS - DR_COMPUTE) * c;
    if (idx < tn * L::COLS) sv[idx] = to_float(raw.v[c]);
  }
  if (lt < tn) {
    sbeta[lt] = 1.0f / (1.0f + expf(-to_float(raw.b)));
    sg[lt] = expf(-decay_rate * dr_softplus(to_float(raw.a) + bias));
  }
}

template <typename T, int R, int P>
__global__ void __launch_bounds__(DR_THREADS)
delta_rule_kernel(const T* __restrict__ u, int u_stride, int q_col, int k_col, int v_col,
                  const T* __restrict__ proj, int proj_stride, int b_col, int a_col,
                  const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                  float* __restrict__ state, size_t state_stride, const int* __restrict__ q_start,
                  const int* __restrict__ state_slots, float* __restrict__ out, int H, int G, int d, int e) {
  using L = DrTile<R, P>;
  extern __shared__ __align__(16) float sm[];   // two tiles
  const int h = blockIdx.y, r = blockIdx.z;
  const int j = h / (H / G);
  const int tid = threadIdx.x;
  const int col0 = blockIdx.x * L::COLS;
  const int row0 = q_start[r], n = q_start[r + 1] - row0;
  const float q_scale = rsqrtf(static_cast<float>(d));
  const float decay_rate = expf(a_log[h]), bias = dt_bias[h];
  const int q_at = q_col + j * d, k_at = k_col + j * d, v_at = v_col + h * e, b_at = b_col + h, a_at = a_col + h;

  // rows past d (a lane's share rounded up) stay zero in both tiles: the fetching warps never touch them
  if (R * P != d) {
    for (int idx = tid; idx < 2 * L::FLOATS; idx += DR_THREADS) sm[idx] = 0.0f;
    __syncthreads();
  }

  const bool computes = tid < DR_COMPUTE;
  const int col = col0 + tid / P, part = tid % P;
  const bool live = computes && col < e;
  float* S_g = state + static_cast<size_t>(ck_request(state_slots[r])) * state_stride + static_cast<size_t>(h) * d * e;
  float S[R];
  DrRaw<T, R, P> raw;
  const int lt = tid - DR_COMPUTE;
  if (computes) {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int row = part * R + i;
      S[i] = (live && row < d) ? S_g[static_cast<size_t>(row) * e + col] : 0.0f;
    }
  } else {
    dr_ask<T, R, P>(raw, u, u_stride, q_at, k_at, v_at, proj, proj_stride, b_at, a_at, row0, min(DR_TT, n), d, e, col0, lt);
    dr_put<T, R, P>(raw, sm, min(DR_TT, n), d, q_scale, decay_rate, bias, lt);
    if (n > DR_TT)
      dr_ask<T, R, P>(raw, u, u_stride, q_at, k_at, v_at, proj, proj_stride, b_at, a_at, row0 + DR_TT,
                      min(DR_TT, n - DR_TT), d, e, col0, lt);
  }
  __syncthreads();

  int which = 0;
  for (int t0 = 0; t0 < n; t0 += DR_TT, which ^= 1) {
    const int tn = min(DR_TT, n - t0);
    if (!computes) {
      // the tile after this one was asked for a tile ago: write it, then ask for the one after it
      if (t0 + DR_TT < n) {
        dr_put<T, R, P>(raw, sm + (which ^ 1) * L::FLOATS, min(DR_TT, n - t0 - DR_TT), d, q_scale, decay_rate, bias, lt);
        if (t0 + 2 * DR_TT < n)
          dr_ask<T, R, P>(raw, u, u_stride, q_at, k_at, v_at, proj, proj_stride, b_at, a_at, row0 + t0 + 2 * DR_TT,
                          min(DR_TT, n - t0 - 2 * DR_TT), d, e, col0, lt);
      }
    } else {
      const float* sq = sm + which * L::FLOATS;
      const float* sk = sq + DR_TT * L::TS;
      const float* sv = sk + DR_TT * L::TS;
      const float* sg = sv + DR_TT * L::COLS;
      const float* sbeta = sg + DR_TT;
      float* orow = out + static_cast<size_t>(row0 + t0) * (H * e) + h * e + col;
      const float* skq = sbeta + DR_TT;
      // Both dot products of a token run over the state the token found: with S' = g S + k u^T the read-out is
      // S'^T q = g (S^T q) + u (k . q), and k . q is the same for every column (the fetching warps leave it beside
      // the gates). So the path from token to token is one round of multiply-adds, one round of shuffles (both sums
      // at once) and the update; the products g S do not wait for the shuffles.
#pragma unroll 2
      for (int tt = 0; tt < tn; ++tt) {
        const float g = sg[tt], beta = sbeta[tt], kq = skq[tt], v = sv[tt * L::COLS + tid / P];
        const float4* k4 = reinterpret_cast<const float4*>(sk + tt * L::TS + part * L::RS);
        const float4* q4 = reinterpret_cast<const float4*>(sq + tt * L::TS + part * L::RS);
        float kr[R];
        float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f, o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
#pragma unroll
        for (int i = 0; i < R / 4; ++i) {
          const float4 kv = k4[i], qv = q4[i];
          kr[4 * i] = kv.x; kr[4 * i + 1] = kv.y; kr[4 * i + 2] = kv.z; kr[4 * i + 3] = kv.w;
          d0 = fmaf(S[4 * i], kv.x, d0);
          d1 = fmaf(S[4 * i + 1], kv.y, d1);
          d2 = fmaf(S[4 * i + 2], kv.z, d2);
          d3 = fmaf(S[4 * i + 3], kv.w, d3);
          o0 = fmaf(S[4 * i], qv.x, o0);
          o1 = fmaf(S[4 * i + 1], qv.y, o1);
          o2 = fmaf(S[4 * i + 2], qv.z, o2);
          o3 = fmaf(S[4 * i + 3], qv.w, o3);
        }
        float dot = (d0 + d1) + (d2 + d3), sq_dot = (o0 + o1) + (o2 + o3);
#pragma unroll
        for (int i = 0; i < R; ++i) S[i] *= g;
#pragma unroll
        for (int o = P >> 1; o > 0; o >>= 1) {
          dot += __shfl_xor_sync(0xffffffffu, dot, o);
          sq_dot += __shfl_xor_sync(0xffffffffu, sq_dot, o);
        }
        const float uval = beta * (v - g * dot);
#pragma unroll
        for (int i = 0; i < R; ++i) S[i] = fmaf(kr[i], uval, S[i]);
        if (live && part == 0) orow[static_cast<size_t>(tt) * (H * e)] = fmaf(uval, kq, g * sq_dot);
      }
    }
    __syncthreads();                            // the tile has been read, the next one is whole
  }
  if (computes) {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int row = part * R + i;
      if (live && row < d) S_g[static_cast<size_t>(row) * e + col] = S[i];
    }
  }
}

// Steps of single tokens (decoding): what counts is the state's trip through memory, H d e floats read and written a
// request. Block = (32 columns, head, request), 128 threads as 32 columns x 4 runs of rows, so that a warp reads 128
// bytes of a state row at once and many light blocks share an SM. The block's slice of S waits in shared memory
// between the two dot products and the update. A request that brought several tokens is walked token by token
// (correct, not fast: the host sends such steps to the tiled kernel above); one that brought none is left alone.
constexpr int DS_COLS = 32;
constexpr int DS_RUNS = 4;

template <typename T>
__global__ void __launch_bounds__(DS_COLS * DS_RUNS)
delta_rule_step_kernel(const T* __restrict__ u, int u_stride, int q_col, int k_col, int v_col,
                       const T* __restrict__ proj, int proj_stride, int b_col, int a_col,
                       const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                       float* __restrict__ state, size_t state_stride, const int* __restrict__ q_start,
                       const int* __restrict__ state_slots, float* __restrict__ out, int H, int G, int d, int e) {
  extern __shared__ __align__(16) float sm[];
  float* sS = sm;                               // [d][DS_COLS]
  float* sk = sS + static_cast<size_t>(d) * DS_COLS;      // [d]
  float* sq = sk + d;                           // [d]
  float* part = sq + d;                         // [2][DS_RUNS][DS_COLS]
  __shared__ float red[33];
  const int h = blockIdx.y, r = blockIdx.z;
  const int j = h / (H / G);
  const int tid = threadIdx.x, c = tid % DS_COLS, run = tid / DS_COLS;
  const int col = blockIdx.x * DS_COLS + c;
  const bool live = col < e;
  const int row0 = q_start[r], row1 = q_start[r + 1];
  if (row1 <= row0) return;
  float* S_g = state + static_cast<size_t>(ck_request(state_slots[r])) * state_stride + static_cast<size_t>(h) * d * e;
  const float q_scale = rsqrtf(static_cast<float>(d));
  const float decay_rate = expf(a_log[h]), bias = dt_bias[h];
  for (int row = row0; row < row1; ++row) {
    const T* urow = u + static_cast<size_t>(row) * u_stride;
    float qq = 0.0f, kk = 0.0f, kq = 0.0f;
    for (int i = tid; i < d; i += DS_COLS * DS_RUNS) {
      const float a = to_float(urow[q_col + j * d + i]), b = to_float(urow[k_col + j * d + i]);
      sq[i] = a;
      sk[i] = b;
      qq = fmaf(a, a, qq);
      kk = fmaf(b, b, kk);
      kq = fmaf(a, b, kq);
    }
    float dot = 0.0f, rd = 0.0f;
    if (row == row0) {                          // the state comes in under the three sums
#pragma unroll 8
      for (int i = run; i < d; i += DS_RUNS) sS[i * DS_COLS + c] = live ? S_g[static_cast<size_t>(i) * e + col] : 0.0f;
    }
    qq = block_sum(qq, red);
    kk = block_sum(kk, red);
    kq = block_sum(kq, red);
    const float fq = q_scale / sqrtf(qq + 1e-6f), fk = 1.0f / sqrtf(kk + 1e-6f);
    const T* prow = proj + static_cast<size_t>(row) * proj_stride;
    const float beta = 1.0f / (1.0f + expf(-to_float(prow[b_col + h])));
    const float g = expf(-decay_rate * dr_softplus(to_float(prow[a_col + h]) + bias));
    const float v = live ? to_float(urow[v_col + h * e + col]) : 0.0f;
#pragma unroll 8
    for (int i = run; i < d; i += DS_RUNS) {
      const float s = sS[i * DS_COLS + c];
      dot = fmaf(s, sk[i], dot);
      rd = fmaf(s, sq[i], rd);
    }
    part[run * DS_COLS + c] = dot;
    part[(DS_RUNS + run) * DS_COLS + c] = rd;
    __syncthreads();
    dot = 0.0f;
    rd = 0.0f;
#pragma unroll
    for (int w = 0; w < DS_RUNS; ++w) {
      dot += part[w * DS_COLS + c];
      rd += part[(DS_RUNS + w) * DS_COLS + c];
    }
    // with S' = g S + k u^T:  S'^T q = g S^T q + u (k . q)
    const float uval = beta * (v - g * fk * dot);
    if (live && run == 0) out[static_cast<size_t>(row) * (H * e) + h * e + col] = fmaf(uval, kq * fq * fk, g * fq * rd);
    const float ku = uval * fk;
    const bool last = row + 1 == row1;
#pragma unroll 8
    for (int i = run; i < d; i += DS_RUNS) {
      const float s = fmaf(sk[i], ku, g * sS[i * DS_COLS + c]);
      if (last) {
        if (live) S_g[static_cast<size_t>(i) * e + col] = s;
      } else {
        sS[i * DS_COLS + c] = s;
      }
    }
    __syncthreads();                            // sk, sq and the partial sums are free again
  }
}

// One warp per (row, head).
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const T* __restrict__ gate, int gate_stride, int gate_col,
                                      const float* __restrict__ w, float eps, T* __restrict__ out, int rows, int H, int e) {
  const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (unit >= rows * H) return;
  const int row = unit / H, h = unit % H;
  const float* orow = o + static_cast<size_t>(row) * H * e + h * e;
  float ss = 0.0f;
  for (int i = lane; i < e; i += 32) ss = fmaf(orow[i], orow[i], ss);
  const float rs = 1.0f / sqrtf(warp_sum(ss) / static_cast<float>(e) + eps);
  const T* grow = gate + static_cast<size_t>(row) * gate_stride + gate_col + h * e;
  T* dst = out + static_cast<size_t>(row) * H * e + h * e;
  for (int i = lane; i < e; i += 32) {
    const float z = to_float(grow[i]);
    dst[i] = from_float<T>(orow[i] * rs * w[i] * (z / (1.0f + expf(-z))));
  }
}

template <typename T, int R, int P>
int delta_rule_launch(const void* u, int u_stride, int q_col, int k_col, int v_col, const void* proj, int proj_stride,
                      int b_col, int a_col, const float* a_log, const float* dt_bias, float* state, long long state_stride,
                      const int* q_start, const int* state_slots, float* out, int requests, int H, int G, int d, int e,
                      cudaStream_t stream) {
  using L = DrTile<R, P>;
  const size_t smem = static_cast<size_t>(2 * L::FLOATS) * sizeof(float);
  auto kernel = delta_rule_kernel<T, R, P>;
  if (smem > 48 * 1024) {
    const cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err != cudaSuccess) return static_cast<int>(err);
  }
  dim3 grid((e + L::COLS - 1) / L::COLS, H, requests);
  kernel<<<grid, DR_THREADS, smem, stream>>>(static_cast<const T*>(u), u_stride, q_col, k_col, v_col,
                                             static_cast<const T*>(proj), proj_stride, b_col, a_col, a_log, dt_bias, state,
                                             static_cast<size_t>(state_stride), q_start, state_slots, out, H, G, d, e);
  return launch_status();
}

}  // namespace dl

// u: rows of u_stride elements with q of all G heads at q_col, k at k_col (G * d each) and v of all H heads at v_col
// (H * e); proj: rows of proj_stride elements with b at b_col and a at a_col (H each); state: float32 rows of
// state_stride floats, S of head h at h * d * e; out: float32 contiguous [rows, H * e]. d up to 512.
DL_EXPORT int dl_delta_rule(int dtype, const void* u, int u_stride, int q_col, int k_col, int v_col, const void* proj,
                            int proj_stride, int b_col, int a_col, const float* a_log, const float* dt_bias, float* state,
                            long long state_stride, const int* q_start, const int* state_slots, float* out, int requests,
                            int H, int G, int d, int e, cudaStream_t stream) {
  if (requests <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G != 0 || d <= 0 || e <= 0 || d > 512 || H > 65535 || requests > 65535 ||
      (dtype != 0 && dtype != 1))
    return DL_ERR_UNSUPPORTED;
  // lanes per column: the fewest (a power of two up to 16) that leave a lane at most 16 rows, or up to 32 from d = 257 on.
  // Short rows keep a token's chain of dependent multiply-adds short; the shuffles that finish a dot product grow
  // by one step with every doubling.
  int P = 1;
  while (P < 16 && (d + P - 1) / P > 16) P *= 2;
  const int need = (d + P - 1) / P;
  const int R = (need + 7) / 8 * 8;
#define DL_DR(RR, PP)                                                                                                      \
  if (R == RR && P == PP)                                                                                                  \
    return dtype == 0 ? dl::delta_rule_launch<float, RR, PP>(u, u_stride, q_col, k_col, v_col, proj, proj_stride, b_col,   \
                                                             a_col, a_log, dt_bias, state, state_stride, q_start,          \
                                                             state_slots, out, requests, H, G, d, e, stream)               \
                      : dl::delta_rule_launch<dl::bf16, RR, PP>(u, u_stride, q_col, k_col, v_col, proj, proj_stride,       \
                                                                b_col, a_col, a_log, dt_bias, state, state_stride,         \
                                                                q_start, state_slots, out, requests, H, G, d, e, stream)
  DL_DR(8, 1); DL_DR(16, 1);                                   // d up to 16
  DL_DR(16, 2); DL_DR(16, 4); DL_DR(16, 8); DL_DR(16, 16);     // 17 .. 32, .. 64, .. 128, .. 256
  DL_DR(24, 16); DL_DR(32, 16);                                // 257 .. 512
#undef DL_DR
  return DL_ERR_UNSUPPORTED;
}

// The same step for batches of single tokens: the same arguments, any d.
DL_EXPORT int dl_delta_rule_step(int dtype, const void* u, int u_stride, int q_col, int k_col, int v_col, const void* proj,
                                 int proj_stride, int b_col, int a_col, const float* a_log, const float* dt_bias,
                                 float* state, long long state_stride, const int* q_start, const int* state_slots,
                                 float* out, int requests, int H, int G, int d, int e, cudaStream_t stream) {
  if (requests <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G != 0 || d <= 0 || e <= 0 || H > 65535 || requests > 65535 || (dtype != 0 && dtype != 1))
    return DL_ERR_UNSUPPORTED;
  const size_t smem = (static_cast<size_t>(d) * dl::DS_COLS + 2 * d + 2 * dl::DS_RUNS * dl::DS_COLS) * sizeof(float);
  if (smem > 200 * 1024) return DL_ERR_UNSUPPORTED;
  dim3 grid((e + dl::DS_COLS - 1) / dl::DS_COLS, H, requests);
#define DL_DS(T)                                                                                                        \
  do {                                                                                                                  \
    auto kernel = dl::delta_rule_step_kernel<T>;                                                                        \
    if (smem > 48 * 1024) {                                                                                             \
      const cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)); \
      if (err != cudaSuccess) return static_cast<int>(err);                                                             \
    }                                                                                                                   \
    kernel<<<grid, dl::DS_COLS * dl::DS_RUNS, smem, stream>>>(static_cast<const T*>(u), u_stride, q_col, k_col, v_col,  \
                                                              static_cast<const T*>(proj), proj_stride, b_col, a_col,   \
                                                              a_log, dt_bias, state, static_cast<size_t>(state_stride), \
                                                              q_start, state_slots, out, H, G, d, e);                   \
  } while (0)
  if (dtype == 0) DL_DS(float);
  else DL_DS(dl::bf16);
#undef DL_DS
  return dl::launch_status();
}

// o: float32 contiguous [rows, H * e]; gate: rows of gate_stride elements, the gate of head h at gate_col + h * e;
// w: float32 [e]; out: contiguous [rows, H * e].
DL_EXPORT int dl_head_norm_gate(int dtype, const float* o, const void* gate, int gate_stride, int gate_col, const float* w,
                                float eps, void* out, int rows, int H, int e, cudaStream_t stream) {
  if (rows <= 0 || H <= 0 || e <= 0) return 0;
  const long long units = static_cast<long long>(rows) * H;
  const unsigned blocks = static_cast<unsigned>((units + 7) / 8);
  if (dtype == 0) dl::head_norm_gate_kernel<float><<<blocks, 256, 0, stream>>>(o, static_cast<const float*>(gate), gate_stride, gate_col, w, eps, static_cast<float*>(out), rows, H, e);
  else if (dtype == 1) dl::head_norm_gate_kernel<dl::bf16><<<blocks, 256, 0, stream>>>(o, static_cast<const dl::bf16*>(gate), gate_stride, gate_col, w, eps, static_cast<dl::bf16*>(out), rows, H, e);
  else return DL_ERR_UNSUPPORTED;
  return dl::launch_status();
}
