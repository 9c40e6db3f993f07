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
// registers, the fetching warps bring the next tile in (queries and keys made unit vectors, a warp per token; the
// values of the block's columns; the two gates), so no token waits for global memory. Within a token only
// g S . k, its shuffles and the rank-one update lie on the path to the next token; the read-out S . q does not.
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
  static constexpr int FLOATS = 2 * DR_TT * TS + DR_TT * COLS + 2 * DR_TT;      // q | k | v | g | beta
};

// The fetching warps: tile [t0, t0 + tn) of the request's rows into one of the two buffers.
template <typename T, int R, int P>
__device__ __forceinline__ void dr_fetch(float* buf, const T* __restrict__ u, int u_stride, int q_at, int k_at, int v_at,
                                         const T* __restrict__ proj, int proj_stride, int b_at, int a_at, int first_row,
                                         int tn, int d, int e, int col0, float q_scale, float decay_rate, float bias, int lt) {
  using L = DrTile<R, P>;
  float* sq = buf;
  float* sk = sq + DR_TT * L::TS;
  float* sv = sk + DR_TT * L::TS;
  float* sg = sv + DR_TT * L::COLS;
  float* sbeta = sg + DR_TT;
  const int lane = lt & 31, warp = lt >> 5;
  constexpr int NT = DR_TT / 4;                         // tokens of a warp
  constexpr int NL = (R * P + 31) / 32;                 // a lane's numbers of one query (or key)
  constexpr int NV = DR_TT * L::COLS / (DR_THREADS - DR_COMPUTE);
  // every load of the tile is issued before the first one is used
  float qv[NT][NL], kv[NT][NL], vv[NV], raw_b = 0.0f, raw_a = 0.0f;
#pragma unroll
  for (int s = 0; s < NT; ++s) {
    const int tt = warp + 4 * s;
    const T* urow = u + static_cast<size_t>(first_row + max(min(tt, tn - 1), 0)) * u_stride;
#pragma unroll
    for (int c = 0; c < NL; ++c) {
      const int i = lane + 32 * c;
      const bool ok = tt < tn && i < d;
      qv[s][c] = ok ? to_float(urow[q_at + i]) : 0.0f;
      kv[s][c] = ok ? to_float(urow[k_at + i]) : 0.0f;
    }
  }
#pragma unroll
  for (int c = 0; c < NV; ++c) {
    const int idx = lt + (DR_THREADS - DR_COMPUTE) * c;
    const int tt = idx / L::COLS, col = col0 + idx % L::COLS;
    vv[c] = (tt < tn && col < e) ? to_float(u[static_cast<size_t>(first_row + tt) * u_stride + v_at + col]) : 0.0f;
  }
  if (lt < tn) {
    const T* prow = proj + static_cast<size_t>(first_row + lt) * proj_stride;
    raw_b = to_float(prow[b_at]);
    raw_a = to_float(prow[a_at]);
  }
#pragma unroll
  for (int s = 0; s < NT; ++s) {
    const int tt = warp + 4 * s;
    float qq = 0.0f, kk = 0.0f;
#pragma unroll
    for (int c = 0; c < NL; ++c) {
      qq = fmaf(qv[s][c], qv[s][c], qq);
      kk = fmaf(kv[s][c], kv[s][c], kk);
    }
    const float fq = q_scale / sqrtf(warp_sum(qq) + 1e-6f), fk = 1.0f / sqrtf(warp_sum(kk) + 1e-6f);
#pragma unroll
    for (int c = 0; c < NL; ++c) {
      const int i = lane + 32 * c;
      if (tt < tn && i < d) {
        const int at = tt * L::TS + (i / R) * L::RS + i % R;
        sq[at] = qv[s][c] * fq;
        sk[at] = kv[s][c] * fk;
      }
    }
  }
#pragma unroll
  for (int c = 0; c < NV; ++c) {
    const int idx = lt + (DR_THREADS - DR_COMPUTE) * c;
    if (idx < tn * L::COLS) sv[idx] = vv[c];
  }
  if (lt < tn) {
    sbeta[lt] = 1.0f / (1.0f + expf(-raw_b));
    sg[lt] = expf(-decay_rate * dr_softplus(raw_a + bias));
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
  if (computes) {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int row = part * R + i;
      S[i] = (live && row < d) ? S_g[static_cast<size_t>(row) * e + col] : 0.0f;
    }
  } else {
    dr_fetch<T, R, P>(sm, u, u_stride, q_at, k_at, v_at, proj, proj_stride, b_at, a_at, row0, min(DR_TT, n), d, e, col0,
                      q_scale, decay_rate, bias, tid - DR_COMPUTE);
  }
  __syncthreads();

  int which = 0;
  for (int t0 = 0; t0 < n; t0 += DR_TT, which ^= 1) {
    const int tn = min(DR_TT, n - t0);
    if (!computes) {
      if (t0 + DR_TT < n)
        dr_fetch<T, R, P>(sm + (which ^ 1) * L::FLOATS, u, u_stride, q_at, k_at, v_at, proj, proj_stride, b_at, a_at,
                          row0 + t0 + DR_TT, min(DR_TT, n - t0 - DR_TT), d, e, col0, q_scale, decay_rate, bias,
                          tid - DR_COMPUTE);
    } else {
      const float* sq = sm + which * L::FLOATS;
      const float* sk = sq + DR_TT * L::TS;
      const float* sv = sk + DR_TT * L::TS;
      const float* sg = sv + DR_TT * L::COLS;
      const float* sbeta = sg + DR_TT;
      float* orow = out + static_cast<size_t>(row0 + t0) * (H * e) + h * e + col;
      // A token's key is in registers before its turn comes (fetched under the token before it), its query is
      // fetched under the shuffles of the first dot product.
      float kr[R];
      {
        const float4* k4 = reinterpret_cast<const float4*>(sk + part * L::RS);
#pragma unroll
        for (int i = 0; i < R / 4; ++i) {
          const float4 kv = k4[i];
          kr[4 * i] = kv.x; kr[4 * i + 1] = kv.y; kr[4 * i + 2] = kv.z; kr[4 * i + 3] = kv.w;
        }
      }
      float g = sg[0], beta = sbeta[0], v = sv[tid / P];
#pragma unroll 2
      for (int tt = 0; tt < tn; ++tt) {
        float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f;
#pragma unroll
        for (int i = 0; i < R / 4; ++i) {
          S[4 * i] *= g; S[4 * i + 1] *= g; S[4 * i + 2] *= g; S[4 * i + 3] *= g;
          d0 = fmaf(S[4 * i], kr[4 * i], d0);
          d1 = fmaf(S[4 * i + 1], kr[4 * i + 1], d1);
          d2 = fmaf(S[4 * i + 2], kr[4 * i + 2], d2);
          d3 = fmaf(S[4 * i + 3], kr[4 * i + 3], d3);
        }
        float dot = (d0 + d1) + (d2 + d3);
        const float4* q4 = reinterpret_cast<const float4*>(sq + tt * L::TS + part * L::RS);
        float qr[R];
#pragma unroll
        for (int i = 0; i < R / 4; ++i) {
          const float4 qv = q4[i];
          qr[4 * i] = qv.x; qr[4 * i + 1] = qv.y; qr[4 * i + 2] = qv.z; qr[4 * i + 3] = qv.w;
        }
#pragma unroll
        for (int o = P >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        const float uval = beta * (v - dot);
        const int nx = min(tt + 1, DR_TT - 1);            // the last token of a tile fetches its own key again
        const float4* k4 = reinterpret_cast<const float4*>(sk + nx * L::TS + part * L::RS);
        float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
#pragma unroll
        for (int i = 0; i < R / 4; ++i) {
          S[4 * i] = fmaf(kr[4 * i], uval, S[4 * i]);
          S[4 * i + 1] = fmaf(kr[4 * i + 1], uval, S[4 * i + 1]);
          S[4 * i + 2] = fmaf(kr[4 * i + 2], uval, S[4 * i + 2]);
          S[4 * i + 3] = fmaf(kr[4 * i + 3], uval, S[4 * i + 3]);
          const float4 kv = k4[i];
          kr[4 * i] = kv.x; kr[4 * i + 1] = kv.y; kr[4 * i + 2] = kv.z; kr[4 * i + 3] = kv.w;
          o0 = fmaf(S[4 * i], qr[4 * i], o0);
          o1 = fmaf(S[4 * i + 1], qr[4 * i + 1], o1);
          o2 = fmaf(S[4 * i + 2], qr[4 * i + 2], o2);
          o3 = fmaf(S[4 * i + 3], qr[4 * i + 3], o3);
        }
        g = sg[nx];
        beta = sbeta[nx];
        v = sv[nx * L::COLS + tid / P];
        float oq = (o0 + o1) + (o2 + o3);
#pragma unroll
        for (int o = P >> 1; o > 0; o >>= 1) oq += __shfl_xor_sync(0xffffffffu, oq, o);
        if (live && part == 0) orow[static_cast<size_t>(tt) * (H * e)] = oq;
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
  // lanes per column: the fewest (a power of two up to 8) that leave a lane at most 32 rows, or 64 from d = 257 on
  int P = 1;
  while (P < 8 && (d + P - 1) / P > 32) P *= 2;
  const int need = (d + P - 1) / P;
  const int R = need > 32 ? 64 : (need + 7) / 8 * 8;
#define DL_DR(RR, PP)                                                                                                      \
  if (R == RR && P == PP)                                                                                                  \
    return dtype == 0 ? dl::delta_rule_launch<float, RR, PP>(u, u_stride, q_col, k_col, v_col, proj, proj_stride, b_col,   \
                                                             a_col, a_log, dt_bias, state, state_stride, q_start,          \
                                                             state_slots, out, requests, H, G, d, e, stream)               \
                      : dl::delta_rule_launch<dl::bf16, RR, PP>(u, u_stride, q_col, k_col, v_col, proj, proj_stride,       \
                                                                b_col, a_col, a_log, dt_bias, state, state_stride,         \
                                                                q_start, state_slots, out, requests, H, G, d, e, stream)
  DL_DR(8, 1); DL_DR(16, 1); DL_DR(24, 1); DL_DR(32, 1);       // d up to 32
  DL_DR(24, 2); DL_DR(32, 2);                                  // 33 .. 64
  DL_DR(24, 4); DL_DR(32, 4);                                  // 65 .. 128
  DL_DR(24, 8); DL_DR(32, 8); DL_DR(64, 8);                    // 129 .. 512
#undef DL_DR
  return DL_ERR_UNSUPPORTED;
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
