// A real-gated linear recurrent unit: per channel, S <- a S + sqrt(1 - a^2) * i * u, with the decay a and the input
// gate i functions of the token's own u through block-diagonal weights. All of it is float32.
//
//   r = sigmoid(Wa[b] u_b + ba[b]),  i = sigmoid(Wi[b] u_b + bi[b])        (b: one of `blocks` equal parts of the channels)
//   log a = -c * r * softplus(lam),  a = exp(log a),  m = sqrt(1 - a^2) * i * u       (c = 8)
//   S <- a S + m  (from S = 0, also for the first token),  out = S * gelu_tanh(y + by)
//
// dl_rglru_gates works out a and m for every row (rows side by side: a block takes 8 rows of one part and walks the
// part's two square matrices once for all of them; the matrices are given transposed, [part][in][out], so that
// neighbouring threads read neighbouring weights). dl_rglru_scan carries S along every request's rows, from and
// into the request's state row, several runs of tokens of a channel side by side.
#include "common.cuh"

namespace dl {

constexpr int LRU_ROWS = 8;

__device__ __forceinline__ float lru_softplus(float v) { return v > 20.0f ? v : log1pf(expf(v)); }
__device__ __forceinline__ float lru_sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float lru_gelu(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void __launch_bounds__(256)
rglru_gates_kernel(const T* __restrict__ u, const float* __restrict__ wa_t, const float* __restrict__ ba,
                   const float* __restrict__ wi_t, const float* __restrict__ bi, const float* __restrict__ lam,
                   float decay_scale, float* __restrict__ a_out, float* __restrict__ m_out, int rows, int width, int nb) {
  extern __shared__ float su[];                 // [LRU_ROWS][nb]
  const int b = blockIdx.y, row0 = blockIdx.x * LRU_ROWS;
  const int tn = min(LRU_ROWS, rows - row0);
  for (int idx = threadIdx.x; idx < LRU_ROWS * nb; idx += blockDim.x) {
    const int t = idx / nb, i = idx % nb;
    su[idx] = t < tn ? to_float(u[static_cast<size_t>(row0 + t) * width + b * nb + i]) : 0.0f;
  }
  __syncthreads();
  const float* wa = wa_t + static_cast<size_t>(b) * nb * nb;
  const float* wi = wi_t + static_cast<size_t>(b) * nb * nb;
  for (int o = threadIdx.x; o < nb; o += blockDim.x) {
    float ar[LRU_ROWS], ai[LRU_ROWS];
    const float b_a = ba[b * nb + o], b_i = bi[b * nb + o];
#pragma unroll
    for (int t = 0; t < LRU_ROWS; ++t) { ar[t] = b_a; ai[t] = b_i; }
    for (int i = 0; i < nb; ++i) {
      const float xa = wa[static_cast<size_t>(i) * nb + o], xi = wi[static_cast<size_t>(i) * nb + o];
#pragma unroll
      for (int t = 0; t < LRU_ROWS; ++t) {
        ar[t] = fmaf(xa, su[t * nb + i], ar[t]);
        ai[t] = fmaf(xi, su[t * nb + i], ai[t]);
      }
    }
    const int c = b * nb + o;
    const float sp = decay_scale * lru_softplus(lam[c]);
#pragma unroll
    for (int t = 0; t < LRU_ROWS; ++t) {
      if (t < tn) {
        const float log_a = -sp * lru_sigmoid(ar[t]);
        const float one_minus_a2 = -expm1f(2.0f * log_a);          // 1 - a^2 without the cancellation
        const size_t at = static_cast<size_t>(row0 + t) * width + c;
        a_out[at] = expf(log_a);
        m_out[at] = sqrtf(one_minus_a2) * lru_sigmoid(ai[t]) * su[t * nb + o];
      }
    }
  }
}

// A block carries 32 channels of one request, its tokens in tiles of SC_SEGS x SC_LEN: thread (lane, seg) first folds
// its SC_LEN tokens into one step (A, M) with S_after = A S_before + M, the block chains the SC_SEGS steps of a tile
// from the state the tile began with, and every thread then runs its tokens again from the state its segment begins
// with, writing the outputs. A tile costs one trip to global memory (every load is issued before the first use) and
// 2 SC_LEN + SC_SEGS dependent multiply-adds instead of SC_SEGS x SC_LEN. Places past the request's end are the step
// (1, 0), which changes nothing.
// A step of single tokens runs one run a block (SC_SEGS = 1): 32 threads, a channel each.
constexpr int SC_LEN = 16;

template <typename T, int SC_SEGS>
__global__ void __launch_bounds__(32 * SC_SEGS)
rglru_scan_kernel(const float* __restrict__ a, const float* __restrict__ m, const T* __restrict__ y,
                  int y_stride, int y_col, const float* __restrict__ y_bias, float* __restrict__ state,
                  size_t state_stride, const int* __restrict__ q_start, const int* __restrict__ state_slots,
                  T* __restrict__ out, int width) {
  __shared__ float sA[2][SC_SEGS][32], sM[2][SC_SEGS][32];
  const int lane = threadIdx.x, seg = threadIdx.y;
  const int c = blockIdx.x * 32 + lane, r = blockIdx.y;
  const bool live = c < width;
  const int row0 = q_start[r], row1 = q_start[r + 1];
  float* sp = state + static_cast<size_t>(ck_request(state_slots[r])) * state_stride + c;
  float S0 = live ? *sp : 0.0f;
  const float by = (y_bias && live) ? y_bias[c] : 0.0f;
  int which = 0;
  for (int base = row0; base < row1; base += SC_SEGS * SC_LEN, which ^= 1) {
    const int first = base + seg * SC_LEN;
    const int cnt = live ? max(0, min(SC_LEN, row1 - first)) : 0;
    float av[SC_LEN], mv[SC_LEN], yv[SC_LEN];
#pragma unroll
    for (int i = 0; i < SC_LEN; ++i) {
      av[i] = 1.0f;
      mv[i] = 0.0f;
      yv[i] = 0.0f;
      if (i < cnt) {
        const size_t at = static_cast<size_t>(first + i) * width + c;
        av[i] = a[at];
        mv[i] = m[at];
        yv[i] = to_float(y[static_cast<size_t>(first + i) * y_stride + y_col + c]);
      }
    }
    float A = 1.0f, M = 0.0f;
#pragma unroll
    for (int i = 0; i < SC_LEN; ++i) {
      M = fmaf(av[i], M, mv[i]);
      A *= av[i];
    }
    sA[which][seg][lane] = A;
    sM[which][seg][lane] = M;
    __syncthreads();                            // the other pair of tables is written next: one wait a tile is enough
    float S = S0, mine = S0;
#pragma unroll
    for (int s = 0; s < SC_SEGS; ++s) {
      if (s == seg) mine = S;
      S = fmaf(sA[which][s][lane], S, sM[which][s][lane]);
    }
    S0 = S;
#pragma unroll
    for (int i = 0; i < SC_LEN; ++i) {
      if (i < cnt) {
        mine = fmaf(av[i], mine, mv[i]);
        out[static_cast<size_t>(first + i) * width + c] = from_float<T>(mine * lru_gelu(yv[i] + by));
      }
    }
  }
  if (seg == 0 && live) *sp = S0;
}

}  // namespace dl

// u: contiguous [rows, width] (the convolution's output); wa_t, wi_t: float32 [blocks][in][out]; ba, bi, lam: float32
// [width]; a_out, m_out: float32 contiguous [rows, width].
DL_EXPORT int dl_rglru_gates(int dtype, const void* u, const float* wa_t, const float* ba, const float* wi_t, const float* bi,
                             const float* lam, float decay_scale, float* a_out, float* m_out, int rows, int width, int blocks,
                             cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (width <= 0 || blocks <= 0 || width % blocks != 0 || blocks > 65535 || (dtype != 0 && dtype != 1)) return DL_ERR_UNSUPPORTED;
  const int nb = width / blocks;
  const size_t smem = static_cast<size_t>(dl::LRU_ROWS) * nb * sizeof(float);
  if (smem > 160 * 1024) return DL_ERR_UNSUPPORTED;
  const int threads = nb >= 256 ? 256 : (nb + 31) / 32 * 32;
  dim3 grid((rows + dl::LRU_ROWS - 1) / dl::LRU_ROWS, blocks);
#define DL_LRU(T)                                                                                                       \
  do {                                                                                                                  \
    auto kernel = dl::rglru_gates_kernel<T>;                                                                            \
    if (smem > 48 * 1024) {                                                                                             \
      const cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)); \
      if (err != cudaSuccess) return static_cast<int>(err);                                                             \
    }                                                                                                                   \
    kernel<<<grid, threads, smem, stream>>>(static_cast<const T*>(u), wa_t, ba, wi_t, bi, lam, decay_scale, a_out, m_out, \
                                            rows, width, nb);                                                           \
  } while (0)
  if (dtype == 0) DL_LRU(float);
  else DL_LRU(dl::bf16);
#undef DL_LRU
  return dl::launch_status();
}

// a, m: float32 [rows, width]; y: rows of y_stride elements, the gate branch at y_col; state: float32 rows of
// state_stride floats with S at their head; out: contiguous [rows, width].
DL_EXPORT int dl_rglru_scan(int dtype, const float* a, const float* m, const void* y, int y_stride, int y_col,
                            const float* y_bias, float* state, long long state_stride, const int* q_start,
                            const int* state_slots, void* out, int requests, int width, int rows, cudaStream_t stream) {
  if (requests <= 0 || width <= 0) return 0;
  if (requests > 65535) return DL_ERR_UNSUPPORTED;
  dim3 grid((width + 31) / 32, requests);
#define DL_SCAN(T, SEGS)                                                                                                \
  dl::rglru_scan_kernel<T, SEGS><<<grid, dim3(32, SEGS), 0, stream>>>(a, m, static_cast<const T*>(y), y_stride, y_col,  \
                                                                      y_bias, state, static_cast<size_t>(state_stride), \
                                                                      q_start, state_slots, static_cast<T*>(out), width)
  const bool single = rows <= requests;         // no request brought more than a token or two
  if (dtype == 0) { if (single) DL_SCAN(float, 1); else DL_SCAN(float, 16); }
  else if (dtype == 1) { if (single) DL_SCAN(dl::bf16, 1); else DL_SCAN(dl::bf16, 16); }
  else return DL_ERR_UNSUPPORTED;
#undef DL_SCAN
  return dl::launch_status();
}
