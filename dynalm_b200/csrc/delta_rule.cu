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
// Block = (slice of the e columns, head, request). A column of S lies over P neighbouring lanes, lane p holding rows
// p, p + P, p + 2P, ... (R of them, in registers); the two dot products of a token are finished by shuffles among
// those lanes. A request's tokens are walked in tiles of 16: a tile's queries and keys are made unit vectors in
// shared memory, its gates worked out once, then every thread runs the tile's tokens over its registers.
//
// dl_head_norm_gate: out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * w * silu(gate[t, h, :]).
#include "common.cuh"

namespace dl {

constexpr int DR_TT = 16;
constexpr int DR_THREADS = 128;

__device__ __forceinline__ float dr_softplus(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

template <typename T, int R>
__global__ void __launch_bounds__(DR_THREADS)
delta_rule_kernel(const T* __restrict__ u, int u_stride, int q_col, int k_col, int v_col,
                  const T* __restrict__ proj, int proj_stride, int b_col, int a_col,
                  const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                  float* __restrict__ state, size_t state_stride, const int* __restrict__ q_start,
                  const int* __restrict__ state_slots, float* __restrict__ out, int H, int G, int d, int e, int P) {
  extern __shared__ float sm[];
  const int DP = R * P;                         // d rounded up: rows past d hold zeros
  float* sq = sm;                               // [TT][DP]
  float* sk = sq + DR_TT * DP;                  // [TT][DP]
  float* sv = sk + DR_TT * DP;                  // [TT][cols]
  const int cols = DR_THREADS / P;
  float* sg = sv + DR_TT * cols;                // [TT]
  float* sbeta = sg + DR_TT;                    // [TT]
  const int h = blockIdx.y, r = blockIdx.z;
  const int j = h / (H / G);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int col = blockIdx.x * cols + tid / P, part = tid % P;
  const bool live = col < e;
  const int row0 = q_start[r], n = q_start[r + 1] - row0;
  float* S_g = state + static_cast<size_t>(ck_request(state_slots[r])) * state_stride + static_cast<size_t>(h) * d * e;

  float S[R];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int row = i * P + part;
    S[i] = (live && row < d) ? S_g[static_cast<size_t>(row) * e + col] : 0.0f;
  }
  const float q_scale = rsqrtf(static_cast<float>(d));
  const float decay_rate = expf(a_log[h]), bias = dt_bias[h];

  for (int t0 = 0; t0 < n; t0 += DR_TT) {
    const int tn = min(DR_TT, n - t0);
    __syncthreads();                            // the previous tile has been read
    for (int idx = tid; idx < tn * DP; idx += DR_THREADS) {
      const int tt = idx / DP, i = idx % DP;
      const T* urow = u + static_cast<size_t>(row0 + t0 + tt) * u_stride;
      sq[idx] = i < d ? to_float(urow[q_col + j * d + i]) : 0.0f;
      sk[idx] = i < d ? to_float(urow[k_col + j * d + i]) : 0.0f;
    }
    for (int idx = tid; idx < tn * cols; idx += DR_THREADS) {
      const int tt = idx / cols, c = blockIdx.x * cols + idx % cols;
      sv[idx] = c < e ? to_float(u[static_cast<size_t>(row0 + t0 + tt) * u_stride + v_col + h * e + c]) : 0.0f;
    }
    if (tid < tn) {
      const T* prow = proj + static_cast<size_t>(row0 + t0 + tid) * proj_stride;
      sbeta[tid] = 1.0f / (1.0f + expf(-to_float(prow[b_col + h])));
      sg[tid] = expf(-decay_rate * dr_softplus(to_float(prow[a_col + h]) + bias));
    }
    __syncthreads();
    for (int tt = warp; tt < tn; tt += DR_THREADS / 32) {          // unit vectors, a warp per token
      float qq = 0.0f, kk = 0.0f;
      for (int i = lane; i < d; i += 32) {
        qq = fmaf(sq[tt * DP + i], sq[tt * DP + i], qq);
        kk = fmaf(sk[tt * DP + i], sk[tt * DP + i], kk);
      }
      qq = warp_sum(qq);
      kk = warp_sum(kk);
      const float fq = q_scale / sqrtf(qq + 1e-6f), fk = 1.0f / sqrtf(kk + 1e-6f);
      for (int i = lane; i < d; i += 32) {
        sq[tt * DP + i] *= fq;
        sk[tt * DP + i] *= fk;
      }
    }
    __syncthreads();
    for (int tt = 0; tt < tn; ++tt) {
      const float g = sg[tt], beta = sbeta[tt];
      const float* kt = sk + tt * DP + part;
      const float* qt = sq + tt * DP + part;
      float dot = 0.0f;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        S[i] *= g;
        dot = fmaf(S[i], kt[i * P], dot);
      }
      for (int o = P >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      const float uval = beta * (sv[tt * cols + tid / P] - dot);
      float oq = 0.0f;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        S[i] = fmaf(kt[i * P], uval, S[i]);
        oq = fmaf(S[i], qt[i * P], oq);
      }
      for (int o = P >> 1; o > 0; o >>= 1) oq += __shfl_xor_sync(0xffffffffu, oq, o);
      if (live && part == 0) out[static_cast<size_t>(row0 + t0 + tt) * (H * e) + h * e + col] = oq;
    }
  }
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int row = i * P + part;
    if (live && row < d) S_g[static_cast<size_t>(row) * e + col] = S[i];
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

template <typename T, int R>
int delta_rule_launch(const void* u, int u_stride, int q_col, int k_col, int v_col, const void* proj, int proj_stride,
                      int b_col, int a_col, const float* a_log, const float* dt_bias, float* state, long long state_stride,
                      const int* q_start, const int* state_slots, float* out, int requests, int H, int G, int d, int e, int P,
                      cudaStream_t stream) {
  const int cols = DR_THREADS / P;
  const size_t smem = (static_cast<size_t>(2 * DR_TT) * R * P + DR_TT * cols + 2 * DR_TT) * sizeof(float);
  auto kernel = delta_rule_kernel<T, R>;
  if (smem > 48 * 1024) {
    const cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err != cudaSuccess) return static_cast<int>(err);
  }
  dim3 grid((e + cols - 1) / cols, H, requests);
  kernel<<<grid, DR_THREADS, smem, stream>>>(static_cast<const T*>(u), u_stride, q_col, k_col, v_col,
                                             static_cast<const T*>(proj), proj_stride, b_col, a_col, a_log, dt_bias, state,
                                             static_cast<size_t>(state_stride), q_start, state_slots, out, H, G, d, e, P);
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
  // lanes per column: the fewest (a power of two up to 8) that leave a thread at most 32 rows, or 64 from d = 257 on
  int P = 1;
  while (P < 8 && (d + P - 1) / P > 32) P *= 2;
  const int need = (d + P - 1) / P;
  const int R = (need + 7) / 8 * 8;
#define DL_DR(RR)                                                                                                          \
  case RR:                                                                                                                 \
    return dtype == 0 ? dl::delta_rule_launch<float, RR>(u, u_stride, q_col, k_col, v_col, proj, proj_stride, b_col, a_col, \
                                                         a_log, dt_bias, state, state_stride, q_start, state_slots, out,   \
                                                         requests, H, G, d, e, P, stream)                                  \
                      : dl::delta_rule_launch<dl::bf16, RR>(u, u_stride, q_col, k_col, v_col, proj, proj_stride, b_col,    \
                                                            a_col, a_log, dt_bias, state, state_stride, q_start,           \
                                                            state_slots, out, requests, H, G, d, e, P, stream)
  switch (R) {
    DL_DR(8); DL_DR(16); DL_DR(24); DL_DR(32); DL_DR(40); DL_DR(48); DL_DR(56); DL_DR(64);
  }
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
