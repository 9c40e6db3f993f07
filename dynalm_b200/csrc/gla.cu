// Gated linear attention: a matrix state per head with a decay per key channel.
//
// Per token and head (key size d, value size e), all float32:
//
//   alpha_i = sigmoid(z_i)^(1 / tau) = exp(-softplus(-z_i) / tau)          (z: the decay's projection, float32; dl_gla_decay,
//                                                                            once per token, in place)
//   S <- diag(alpha) S + k v^T                                              (S: d x e, row i belongs to key channel i)
//   o = S^T (q * q_scale)                                                   (read after the write)
//
// The columns of S are independent recurrences that share alpha, k and q, so the kernel deals columns over threads: a
// block is (a slice of columns, head, request); a column lies over P neighbouring lanes, each keeping R = Dp / P rows of
// it in registers (Dp: d rounded up to P * R, the rows past d idle). Tokens are walked in tiles of 16 whose q, k, alpha
// and v wait in shared memory; the outputs of a tile are written together. Nothing between one token and the next
// depends on a shuffle: the sum over a column's lanes only finishes o.
//
// A request's state row holds S of every head TRANSPOSED, [H, e, d], so that a lane's rows of a column are neighbours
// in memory. Steps of single tokens and portions of prompts run the same kernel.
#include "common.cuh"

namespace dl {

constexpr int GLA_TILE = 16;

// PRE: the next tile's numbers are asked for before the current tile is computed and wait in registers meanwhile (at most
// 8 of q, k and the decays each and 2 values a thread: Dp <= 128 with 256 threads), so that a tile's trip to memory hides
// behind the arithmetic of the tile in front of it.
template <typename T, int R, bool PRE>
__global__ void __launch_bounds__(256)
gla_scan_kernel(const T* __restrict__ proj, int stride, int q_col, int k_col, int v_col, const float* __restrict__ alpha,
                int a_stride, float q_scale, float* __restrict__ state, size_t state_stride,
                const int* __restrict__ q_start, const int* __restrict__ state_slots, float* __restrict__ o, int H, int d,
                int e, int P, int cols) {
  extern __shared__ __align__(16) float sm[];
  const int Dp = P * R;
  float* s_q = sm;                                // [TILE][Dp]
  float* s_k = s_q + GLA_TILE * Dp;
  float* s_a = s_k + GLA_TILE * Dp;
  float* s_v = s_a + GLA_TILE * Dp;               // [TILE][cols]
  float* s_o = s_v + GLA_TILE * cols;             // [TILE][cols]
  const int req = blockIdx.z, head = blockIdx.y, c0 = blockIdx.x * cols;
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int p = tid % P, cl = tid / P;            // lane within the column, column within the slice
  const int col = c0 + cl;
  const bool live = cl < cols && col < e;
  const int r0 = q_start[req], r1 = q_start[req + 1];
  if (r1 <= r0) return;
  float* srow = state + static_cast<size_t>(state_slots[req]) * state_stride + (static_cast<size_t>(head) * e + col) * d;

  // rows of this lane: i = 4 * (p + P * (j / 4)) + j % 4, so that at a given j the lanes of a column read neighbours
  float S[R];
#pragma unroll
  for (int j = 0; j < R; ++j) {
    const int i = 4 * (p + P * (j >> 2)) + (j & 3);
    S[j] = (live && i < d) ? srow[i] : 0.0f;
  }

  constexpr int MAXF = 8, MAXV = 2;
  // as they lie in memory: nothing here may depend on a number that is still on its way, or the warp would wait for it
  T pq[PRE ? MAXF : 1], pk[PRE ? MAXF : 1], pv[PRE ? MAXV : 1];
  float pa[PRE ? MAXF : 1];
  auto fetch = [&](int t0, int nt) {                // PRE only: a tile's numbers into registers
    int t = tid / Dp, i = tid % Dp;
    const int dt = 256 / Dp, di = 256 % Dp;
#pragma unroll
    for (int c = 0; c < MAXF; ++c) {
      pq[c] = pk[c] = from_float<T>(0.0f);
      pa[c] = 0.0f;
      if (t < nt && i < d) {
        const T* prow = proj + static_cast<size_t>(t0 + t) * stride;
        pq[c] = prow[q_col + head * d + i];
        pk[c] = prow[k_col + head * d + i];
        pa[c] = alpha[static_cast<size_t>(t0 + t) * a_stride + head * d + i];
      }
      t += dt;
      i += di;
      if (i >= Dp) { i -= Dp; ++t; }
    }
#pragma unroll
    for (int c = 0; c < MAXV; ++c) {
      const int x = tid + 256 * c, tt = x / cols, cc = x % cols;
      pv[c] = from_float<T>(0.0f);
      if (tt < nt && c0 + cc < e) pv[c] = proj[static_cast<size_t>(t0 + tt) * stride + v_col + head * e + c0 + cc];
    }
  };
  if (PRE) fetch(r0, min(GLA_TILE, r1 - r0));

  for (int t0 = r0; t0 < r1; t0 += GLA_TILE) {
    const int nt = min(GLA_TILE, r1 - t0);
    __syncthreads();                              // the tile before has been read
    if (PRE) {
#pragma unroll
      for (int c = 0; c < MAXF; ++c) {
        const int x = tid + 256 * c;
        if (x < GLA_TILE * Dp) { s_q[x] = to_float(pq[c]) * q_scale; s_k[x] = to_float(pk[c]); s_a[x] = pa[c]; }
      }
#pragma unroll
      for (int c = 0; c < MAXV; ++c) {
        const int x = tid + 256 * c;
        if (x < GLA_TILE * cols) s_v[x] = to_float(pv[c]);
      }
      __syncthreads();
      if (t0 + GLA_TILE < r1) fetch(t0 + GLA_TILE, min(GLA_TILE, r1 - t0 - GLA_TILE));
    } else {
      for (int x = tid; x < nt * Dp; x += nthr) {
        const int t = x / Dp, i = x % Dp;
        float qv = 0.0f, kv = 0.0f, av = 0.0f;
        if (i < d) {
          const T* prow = proj + static_cast<size_t>(t0 + t) * stride;
          qv = to_float(prow[q_col + head * d + i]) * q_scale;
          kv = to_float(prow[k_col + head * d + i]);
          av = alpha[static_cast<size_t>(t0 + t) * a_stride + head * d + i];
        }
        s_q[x] = qv;
        s_k[x] = kv;
        s_a[x] = av;
      }
      for (int x = tid; x < nt * cols; x += nthr) {
        const int t = x / cols, c = x % cols;
        s_v[x] = c0 + c < e ? to_float(proj[static_cast<size_t>(t0 + t) * stride + v_col + head * e + c0 + c]) : 0.0f;
      }
      __syncthreads();
    }
    if ((tid & ~31) / P < cols) {                 // warps that hold columns; all their lanes walk the tile (the shuffles
      const int clr = cl < cols ? cl : cols - 1;  // name the whole warp), the other warps of the block only fetch
#pragma unroll 4
      for (int t = 0; t < nt; ++t) {
        const float v = s_v[t * cols + clr];
        const float* qa = s_q + t * Dp;
        const float* ka = s_k + t * Dp;
        const float* aa = s_a + t * Dp;
        float acc = 0.0f;
#pragma unroll
        for (int j4 = 0; j4 < R / 4; ++j4) {
          const int i = 4 * (p + P * j4);
          const float4 q4 = *reinterpret_cast<const float4*>(qa + i);
          const float4 k4 = *reinterpret_cast<const float4*>(ka + i);
          const float4 a4 = *reinterpret_cast<const float4*>(aa + i);
          float* s = S + 4 * j4;
          s[0] = fmaf(a4.x, s[0], k4.x * v);
          s[1] = fmaf(a4.y, s[1], k4.y * v);
          s[2] = fmaf(a4.z, s[2], k4.z * v);
          s[3] = fmaf(a4.w, s[3], k4.w * v);
          acc = fmaf(s[0], q4.x, acc);
          acc = fmaf(s[1], q4.y, acc);
          acc = fmaf(s[2], q4.z, acc);
          acc = fmaf(s[3], q4.w, acc);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1)
          if (off < P) acc += __shfl_xor_sync(0xffffffffu, acc, off);
        if (p == 0 && cl < cols) s_o[t * cols + cl] = acc;
      }
    }
    __syncthreads();
    for (int x = tid; x < nt * cols; x += nthr) {
      const int t = x / cols, c = x % cols;
      if (c0 + c < e) o[static_cast<size_t>(t0 + t) * H * e + head * e + c0 + c] = s_o[x];
    }
  }
  if (live) {
#pragma unroll
    for (int j = 0; j < R; ++j) {
      const int i = 4 * (p + P * (j >> 2)) + (j & 3);
      if (i < d) srow[i] = S[j];
    }
  }
}

// z (+ bias) -> sigmoid(.)^(1 / tau), in place: exp(-softplus(-z) / tau), with softplus(x) = x for large x.
__global__ void gla_decay_kernel(float* __restrict__ z, int stride, int cols, const float* __restrict__ bias, float inv_tau,
                                 size_t total) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float* p = z + (i / cols) * stride + i % cols;
  const float x = -(*p + (bias != nullptr ? bias[i % cols] : 0.0f));
  const float sp = x > 20.0f ? x : log1pf(expf(x));
  *p = expf(-sp * inv_tau);
}

}  // namespace dl

DL_EXPORT int dl_gla_decay(float* z, int stride, int rows, int cols, const float* bias, float tau, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (!(tau > 0.0f)) return DL_ERR_UNSUPPORTED;
  const size_t total = static_cast<size_t>(rows) * cols;
  dl::gla_decay_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(z, stride, cols, bias, 1.0f / tau, total);
  return dl::launch_status();
}

// proj: rows of `stride` elements holding q (H * d numbers from column q_col), k (from k_col) and v (H * e from v_col).
// alpha: float32 rows of a_stride numbers, H * d of them used (the decays, from dl_gla_decay). state: float32, a request's row state_stride numbers from the
// next, the first H * e * d of it S transposed. q_start: requests + 1 row numbers. o: float32 [rows, H * e].
DL_EXPORT int dl_gla_scan(int dtype, const void* proj, int stride, int q_col, int k_col, int v_col, const float* alpha,
                          int a_stride, float q_scale, float* state, long long state_stride, const int* q_start,
                          const int* state_slots, float* o, int requests, int H, int d, int e, int sm_count,
                          cudaStream_t stream) {
  if (requests <= 0) return 0;
  if (H <= 0 || d <= 0 || d > 512 || e <= 0 || H > 65535 || requests > 65535 || (dtype != 0 && dtype != 1))
    return DL_ERR_UNSUPPORTED;
  int P = 1;
  while (P * 16 < d) P <<= 1;                      // lanes a column: the fewest that leave a lane at most 16 rows
  // A warp walks its tokens one after the other, each a short chain of dependent instructions, so what fills an SM is the
  // number of warps: while the step has fewer than four computing warps an SM (one long prompt), a column is laid over
  // more lanes (down to four rows a lane), which costs a shuffle a doubling.
  while (P < 32 && d >= 8 * P && static_cast<long long>(requests) * H * e * P / 32 < 4ll * sm_count) P <<= 1;
  const int R = ((d + P - 1) / P + 3) / 4 * 4;     // rows a lane, in fours
  int cols = 256 / P;                              // columns a block of 256 threads takes
  if (cols > e) cols = e;
  // fewer columns a block while the grid leaves SMs idle (a block keeps at least a warp's worth of lanes busy)
  while (cols > 1 && cols * P > 32 && static_cast<long long>((e + cols - 1) / cols) * H * requests < sm_count) cols = (cols + 1) / 2;
  // a block is 256 threads whatever its columns need: all of them fetch a tile's q, k, decays and values (the fetch of a
  // tile is a chain of dependent trips to memory, shorter the more threads share it), the first cols * P compute
  const int threads = 256;
  const int Dp = P * R;
  const size_t smem = static_cast<size_t>(dl::GLA_TILE) * (3 * Dp + 2 * cols) * sizeof(float);
  dim3 grid((e + cols - 1) / cols, H, requests);
  const bool pre = Dp <= 128 && cols <= 32;
#define DL_GLA(T, RR)                                                                                                    \
  do {                                                                                                                   \
    if (pre) DL_GLA_P(T, RR, true);                                                                                      \
    else DL_GLA_P(T, RR, false);                                                                                         \
  } while (0)
#define DL_GLA_P(T, RR, PP)                                                                                              \
  do {                                                                                                                   \
    cudaFuncSetAttribute(dl::gla_scan_kernel<T, RR, PP>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)); \
    dl::gla_scan_kernel<T, RR, PP><<<grid, threads, smem, stream>>>(static_cast<const T*>(proj), stride, q_col, k_col, v_col, alpha, \
                                                                a_stride, q_scale, state,                                \
                                                                static_cast<size_t>(state_stride), q_start, state_slots, o, \
                                                                H, d, e, P, cols);                                       \
  } while (0)
#define DL_GLA_R(T)              \
  do {                           \
    if (R == 4) DL_GLA(T, 4);    \
    else if (R == 8) DL_GLA(T, 8); \
    else if (R == 12) DL_GLA(T, 12); \
    else DL_GLA(T, 16);          \
  } while (0)
  if (dtype == 0) DL_GLA_R(float);
  else DL_GLA_R(dl::bf16);
#undef DL_GLA_R
#undef DL_GLA
#undef DL_GLA_P
  return dl::launch_status();
}
