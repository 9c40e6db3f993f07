// A state-space mixer's kernels: short causal convolution, the recurrence of every head, and the gated norm of
// its output. One projection of the layer's input gives a row [z: H*P | x: H*P | B: G*N | C: G*N | dt: H]
// (H heads of P channels, N state rows, G groups of heads that share B and C).
//
//   u    = silu(conv(x | B | C))        per channel, K taps, the last tap is the current token's, zeros before the start
//   dt_h = softplus(dt_h + bias_h)
//   S_h  = exp(-exp(a_h) dt_h) S_h + dt_h B x_h^T        (S_h is N x P, float32, carried from token to token)
//   y_h  = S_h^T C + D_h x_h
//   out  = norm_parts(y * silu(z)) * w                   (each of `parts` equal pieces by its own root mean square)
//
// What a request keeps between steps is one float32 row of a state array: H*N*P numbers of S, then the last K - 1
// inputs of the convolution, [K - 1][C], oldest first. A step may bring any number of consecutive tokens of a
// request; every kernel finds a row's request, position and slot in the step's arrays. Decays, step sizes, the
// state and the sums over it are float32 whatever the storage type of the projection.
#include "common.cuh"

namespace dl {

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

// ---- convolution --------------------------------------------------------------------------------------------
// One thread per (row, channel). The K - 1 inputs in front of a row come from the rows above it while those
// belong to the same step, and from the request's kept inputs otherwise.
template <typename T>
__global__ void ssm_conv_kernel(const T* __restrict__ proj, int proj_stride, int col0, int channels,
                                const float* __restrict__ taps, const float* __restrict__ bias, int K,
                                const float* __restrict__ state, size_t state_stride, size_t keep_off,
                                const int* __restrict__ positions, const int* __restrict__ row_request,
                                const int* __restrict__ row_slot, const int* __restrict__ pos_start,
                                T* __restrict__ out, int rows, int act, const float* __restrict__ in_bias) {
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<size_t>(rows) * channels) return;
  const int row = static_cast<int>(idx / channels), ch = static_cast<int>(idx % channels);
  const int pos = positions[row];
  const int first = pos_start[ck_request(row_request[row])];      // the position of the request's first row in this step
  const float* kept = state + static_cast<size_t>(ck_request(row_slot[row])) * state_stride + keep_off;
  float acc = bias ? bias[ch] : 0.0f;
  const float ib = in_bias ? in_bias[ch] : 0.0f;                   // joins every input that lies inside the sequence
  for (int k = K - 1; k >= 0; --k) {                               // oldest input first
    const int p = pos - k;
    float v;
    if (p >= first) v = to_float(proj[static_cast<size_t>(row - k) * proj_stride + col0 + ch]);
    else v = kept[static_cast<size_t>(K - 1 - (first - p)) * channels + ch];
    if (p >= 0) v += ib;
    acc = fmaf(taps[static_cast<size_t>(K - 1 - k) * channels + ch], v, acc);
  }
  out[idx] = from_float<T>(act ? silu_f(acc) : acc);
}

// The same with a thread on 8 (bfloat16) or 4 (float32) neighbouring channels of a row, 16 bytes a load: for channel
// counts, first columns and row pitches that are multiples of that.
template <typename T>
__global__ void ssm_conv_vec_kernel(const T* __restrict__ proj, int proj_stride, int col0, int channels,
                                    const float* __restrict__ taps, const float* __restrict__ bias, int K,
                                    const float* __restrict__ state, size_t state_stride, size_t keep_off,
                                    const int* __restrict__ positions, const int* __restrict__ row_request,
                                    const int* __restrict__ row_slot, const int* __restrict__ pos_start,
                                    T* __restrict__ out, int rows, int act, const float* __restrict__ in_bias) {
  constexpr int V = PerVec<T>::n;
  const int per_row = channels / V;
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<size_t>(rows) * per_row) return;
  const int row = static_cast<int>(idx / per_row), ch = static_cast<int>(idx % per_row) * V;
  const int pos = positions[row];
  const int first = pos_start[ck_request(row_request[row])];
  const float* kept = state + static_cast<size_t>(ck_request(row_slot[row])) * state_stride + keep_off;
  float acc[V];
#pragma unroll
  for (int j = 0; j < V; j += 4) {
    const float4 b4 = bias ? *reinterpret_cast<const float4*>(bias + ch + j) : make_float4(0.f, 0.f, 0.f, 0.f);
    acc[j] = b4.x; acc[j + 1] = b4.y; acc[j + 2] = b4.z; acc[j + 3] = b4.w;
  }
  for (int k = K - 1; k >= 0; --k) {                               // oldest input first
    const int p = pos - k;
    float v[V];
    if (p >= first) {
      unpack<T>(*reinterpret_cast<const Vec16*>(proj + static_cast<size_t>(row - k) * proj_stride + col0 + ch), v);
    } else {
      const float* kr = kept + static_cast<size_t>(K - 1 - (first - p)) * channels + ch;
#pragma unroll
      for (int j = 0; j < V; ++j) v[j] = kr[j];          // (kept inputs begin where the state's layout puts them: no wide loads)
    }
    if (in_bias != nullptr && p >= 0) {
#pragma unroll
      for (int j = 0; j < V; ++j) v[j] += in_bias[ch + j];
    }
    const float* tk = taps + static_cast<size_t>(K - 1 - k) * channels + ch;
#pragma unroll
    for (int j = 0; j < V; j += 4) {
      const float4 t4 = *reinterpret_cast<const float4*>(tk + j);
      acc[j] = fmaf(t4.x, v[j], acc[j]); acc[j + 1] = fmaf(t4.y, v[j + 1], acc[j + 1]);
      acc[j + 2] = fmaf(t4.z, v[j + 2], acc[j + 2]); acc[j + 3] = fmaf(t4.w, v[j + 3], acc[j + 3]);
    }
  }
  if (act) {
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = silu_f(acc[j]);
  }
  *reinterpret_cast<Vec16*>(out + static_cast<size_t>(row) * channels + ch) = pack<T>(acc);
}

// After the convolution of a step: the last K - 1 inputs of every request, oldest first. One thread per (request,
// channel); entries are written in ascending order, and entry j only ever needs an older entry at a higher index.
template <typename T>
__global__ void ssm_conv_keep_kernel(const T* __restrict__ proj, int proj_stride, int col0, int channels, int K,
                                     float* __restrict__ state, size_t state_stride, size_t keep_off,
                                     const int* __restrict__ q_start, const int* __restrict__ state_slots,
                                     int requests) {
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<size_t>(requests) * channels) return;
  const int r = static_cast<int>(idx / channels), ch = static_cast<int>(idx % channels);
  const int r0 = q_start[r], n = q_start[r + 1] - r0;
  float* kept = state + static_cast<size_t>(ck_request(state_slots[r])) * state_stride + keep_off;
  for (int j = 0; j < K - 1; ++j) {
    const int rel = n - (K - 1) + j;                               // which of the step's rows entry j is, if any
    kept[static_cast<size_t>(j) * channels + ch] =
        rel >= 0 ? to_float(proj[static_cast<size_t>(r0 + rel) * proj_stride + col0 + ch])
                 : kept[static_cast<size_t>(j + n) * channels + ch];
  }
}

// ---- recurrence ---------------------------------------------------------------------------------------------
// Block = (run of tokens, head, slice of PV channels). Thread (p, j) keeps rows n = j NR .. j NR + NR - 1 of column p
// of S in registers (FULL: N = NS NR, no row of a thread lies outside). The run's tokens are walked in tiles of TT: a tile's B, C, x, step sizes and
// decays go to shared memory, every thread then runs the tile's tokens over its registers and leaves its share of every
// y in shared memory, and the shares of a channel are added in a fixed order.
//
// A run is either all the tokens a request brings in this step (SCAN_WHOLE: from the request's state, back into it),
// or one SEGMENT of a long portion, so that the segments of a portion run side by side in three launches:
//   SCAN_LOCAL   every segment from a zero state: what it adds to the state, and the product of its decays, to scratch
//   (carry)      per request, over its segments in order: S_start[c] = the state before segment c (written over the
//                segment's scratch), S <- decay_c S + added_c; the last S is the request's new state
//   SCAN_FINISH  every segment again from S_start[c], now with its outputs
// The recurrence is linear in S, so this is the same arithmetic reordered; all of it is float32.
constexpr int SCAN_TT = 16;
constexpr int SCAN_WHOLE = 0, SCAN_LOCAL = 1, SCAN_FINISH = 2;

__device__ __forceinline__ void scan_cp16(void* smem, const void* gmem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}

// ASYNC: the next tile's x, B and C are copied, as stored, into a second set of shared-memory buffers (cp.async, 16 bytes
// a piece) while the current tile is computed, and its step sizes wait in registers; a tile then begins by widening
// what has arrived. For sizes that 16-byte pieces fit (see the launch).
template <typename T, int NR, int MODE, bool FULL, bool ASYNC>
__global__ void __launch_bounds__(256, 3) ssm_scan_kernel(const T* __restrict__ u, int u_stride,            // [rows, H*P + 2*G*N] after the convolution
                                const T* __restrict__ proj, int proj_stride, int dt_col,   // dt of head h at proj[row, dt_col + h]
                                const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                const float* __restrict__ d_skip, float* __restrict__ state, size_t state_stride,
                                const int* __restrict__ q_start, const int* __restrict__ state_slots,
                                const int* __restrict__ segments,                 // [n][4] = (slot, first row, rows, -)
                                float* __restrict__ scratch, float* __restrict__ seg_decay, int whole_up_to,
                                float* __restrict__ y, int H, int P, int N, int G, int PV, int NS) {
  extern __shared__ float sm[];
  float2* sBC = reinterpret_cast<float2*>(sm);  // [TT][N] (B, C)
  float* sX = sm + 2 * SCAN_TT * N;             // [TT][PV]
  float* sY = sX + SCAN_TT * PV;                // [TT][NS][PV]
  float* sDt = sY + SCAN_TT * NS * PV;          // [TT] step sizes, then [TT] decays
  float* sDa = sDt + SCAN_TT;
  const int h = blockIdx.y, p0 = blockIdx.z * PV;
  const int tid = threadIdx.x, pl = tid % PV, j = tid / PV;
  const int p = p0 + pl;
  const bool live = p < P;
  const int g = h / (H / G);
  const int inner = H * P;
  int r0, n_tok;
  float* S;
  if (MODE == SCAN_WHOLE) {
    const int r = blockIdx.x;
    r0 = q_start[r];
    n_tok = q_start[r + 1] - r0;
    if (n_tok > whole_up_to) return;            // a long portion: its segments are run by the other three launches
    S = state + static_cast<size_t>(ck_request(state_slots[r])) * state_stride + static_cast<size_t>(h) * N * P;
  } else {
    const int4 seg = reinterpret_cast<const int4*>(segments)[blockIdx.x];
    r0 = seg.y;
    n_tok = seg.z;
    S = scratch + (static_cast<size_t>(blockIdx.x) * H + h) * N * P;
  }
  const float rate = expf(a_log[h]), bias = dt_bias[h], skip = d_skip[h];
  const int n_first = j * NR;                    // this thread's rows of S: n_first + i
  float s[NR];
#pragma unroll
  for (int i = 0; i < NR; ++i)
    s[i] = (MODE != SCAN_LOCAL && live && (FULL || n_first + i < N)) ? S[static_cast<size_t>(n_first + i) * P + p] : 0.0f;
  float run_decay = 1.0f;
  // (ASYNC) raw copies of a tile: [2 stages][B: TT x N | C: TT x N | x: TT x PV] of T
  T* raw = reinterpret_cast<T*>(sDa + SCAN_TT);
  const int raw_stage = SCAN_TT * (2 * N + PV);
  float dt_raw = 0.0f;                          // this thread's token's step size of the tile at hand (threads < TT)
  auto prefetch = [&](int t0, int stage) {
    constexpr int V = PerVec<T>::n;
    const int tt = min(SCAN_TT, n_tok - t0);
    T* rs = raw + static_cast<size_t>(stage) * raw_stage;
    const int nb = N / V, per = 2 * nb + PV / V;
    for (int i = tid; i < tt * per; i += blockDim.x) {
      const int t = i / per, c = i % per;
      const T* row = u + static_cast<size_t>(r0 + t0 + t) * u_stride;
      if (c < nb) scan_cp16(rs + t * N + c * V, row + inner + g * N + c * V);
      else if (c < 2 * nb) scan_cp16(rs + (SCAN_TT + t) * N + (c - nb) * V, row + inner + (G + g) * N + (c - nb) * V);
      else scan_cp16(rs + 2 * SCAN_TT * N + t * PV + (c - 2 * nb) * V, row + h * P + p0 + (c - 2 * nb) * V);
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };
  if (ASYNC && n_tok > 0) {
    prefetch(0, 0);
    if (tid < min(SCAN_TT, n_tok)) dt_raw = to_float(proj[static_cast<size_t>(r0 + tid) * proj_stride + dt_col + h]);
  }
  for (int t0 = 0; t0 < n_tok; t0 += SCAN_TT) {
    const int tt = min(SCAN_TT, n_tok - t0);
    if (ASYNC) asm volatile("cp.async.wait_group 0;\n" ::);
    __syncthreads();                            // the tile before has been read (ASYNC: and this tile's copies are here)
    if (ASYNC) {
      const int stage = (t0 / SCAN_TT) & 1;
      float dt_next = 0.0f;
      if (t0 + SCAN_TT < n_tok) {
        prefetch(t0 + SCAN_TT, stage ^ 1);
        if (tid < min(SCAN_TT, n_tok - t0 - SCAN_TT))
          dt_next = to_float(proj[static_cast<size_t>(r0 + t0 + SCAN_TT + tid) * proj_stride + dt_col + h]);
      }
      const T* rs = raw + static_cast<size_t>(stage) * raw_stage;
      for (int i = tid; i < tt * N; i += blockDim.x) sBC[i] = make_float2(to_float(rs[i]), to_float(rs[SCAN_TT * N + i]));
      for (int i = tid; i < tt * PV; i += blockDim.x) sX[i] = to_float(rs[2 * SCAN_TT * N + i]);
      if (tid < tt) {
        const float dt = softplus_f(dt_raw + bias);
        sDt[tid] = dt;
        sDa[tid] = expf(-rate * dt);
      }
      dt_raw = dt_next;
    } else {
      for (int i = tid; i < tt * N; i += blockDim.x) {
        const int t = i / N, n = i % N;
        const T* ur = u + static_cast<size_t>(r0 + t0 + t) * u_stride + inner + g * N + n;
        sBC[i] = make_float2(to_float(ur[0]), to_float(ur[G * N]));
      }
      for (int i = tid; i < tt * PV; i += blockDim.x) {
        const int t = i / PV, q = p0 + i % PV;
        sX[i] = q < P ? to_float(u[static_cast<size_t>(r0 + t0 + t) * u_stride + h * P + q]) : 0.0f;
      }
      for (int t = tid; t < tt; t += blockDim.x) {
        const float rawv = to_float(proj[static_cast<size_t>(r0 + t0 + t) * proj_stride + dt_col + h]);
        const float dt = softplus_f(rawv + bias);
        sDt[t] = dt;
        sDa[t] = expf(-rate * dt);
      }
    }
    __syncthreads();
    for (int t = 0; t < tt; ++t) {
      const float dt = sDt[t], da = sDa[t];
      const float xv = sX[t * PV + pl] * dt;
      const float2* bc = sBC + t * N + n_first;
      if (MODE == SCAN_LOCAL) run_decay *= da;
      float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll
      for (int i = 0; i < NR; i += 2) {
        float2 v0, v1;
        if (FULL) {                              // two rows' (B, C) in one 16-byte load: N and NR are even
          const float4 q = *reinterpret_cast<const float4*>(bc + i);
          v0 = make_float2(q.x, q.y);
          v1 = make_float2(q.z, q.w);
        } else {
          v0 = n_first + i < N ? bc[i] : make_float2(0.f, 0.f);
          v1 = n_first + i + 1 < N ? bc[i + 1] : make_float2(0.f, 0.f);
        }
        s[i] = fmaf(da, s[i], v0.x * xv);
        s[i + 1] = fmaf(da, s[i + 1], v1.x * xv);
        if (MODE != SCAN_LOCAL) {
          acc0 = fmaf(s[i], v0.y, acc0);
          acc1 = fmaf(s[i + 1], v1.y, acc1);
        }
      }
      if (MODE != SCAN_LOCAL) sY[(t * NS + j) * PV + pl] = acc0 + acc1;
    }
    if (MODE != SCAN_LOCAL) {
      __syncthreads();
      for (int i = tid; i < tt * PV; i += blockDim.x) {
        const int t = i / PV, q = i % PV;
        if (p0 + q < P) {
          float sum = 0.0f;
          for (int k = 0; k < NS; ++k) sum += sY[(t * NS + k) * PV + q];
          y[static_cast<size_t>(r0 + t0 + t) * inner + h * P + p0 + q] = fmaf(skip, sX[t * PV + q], sum);
        }
      }
    }
  }
  if (MODE != SCAN_FINISH) {
#pragma unroll
    for (int i = 0; i < NR; ++i)
      if (live && (FULL || n_first + i < N)) S[static_cast<size_t>(n_first + i) * P + p] = s[i];
  }
  if (MODE == SCAN_LOCAL && tid == 0 && blockIdx.z == 0) seg_decay[static_cast<size_t>(blockIdx.x) * H + h] = run_decay;
}

// Between the two passes over the segments of long portions: per request of `long_requests` (first segment, segments,
// slot, -) and element of the state, the state before every segment in place of what the segment added, and the
// request's new state.
__global__ void ssm_carry_kernel(float* __restrict__ state, size_t state_stride, float* __restrict__ scratch,
                                 const float* __restrict__ seg_decay, const int* __restrict__ long_requests, int H,
                                 int per_head) {
  const int4 req = reinterpret_cast<const int4*>(long_requests)[blockIdx.y];
  const size_t per_seg = static_cast<size_t>(H) * per_head;
  const size_t e = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= per_seg) return;
  const int h = static_cast<int>(e / per_head);
  float* slot = state + static_cast<size_t>(ck_request(req.z)) * state_stride;
  float S = slot[e];
  for (int c = 0; c < req.y; ++c) {
    const size_t seg = static_cast<size_t>(req.x + c);
    const float added = scratch[seg * per_seg + e];
    scratch[seg * per_seg + e] = S;
    S = fmaf(seg_decay[seg * H + h], S, added);
  }
  slot[e] = S;
}

// ---- gated norm -----------------------------------------------------------------------------------------------
// Block = (row, part). v = y * silu(z) over the part's channels, out = v / sqrt(mean(v^2) + eps) * w.
template <typename T>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, const T* __restrict__ z, int z_stride,
                                        const float* __restrict__ w, float eps, T* __restrict__ out, int inner,
                                        int part_len) {
  __shared__ float red[33];
  const int row = blockIdx.x, c0 = blockIdx.y * part_len;
  const float* yr = y + static_cast<size_t>(row) * inner + c0;
  const T* zr = z + static_cast<size_t>(row) * z_stride + c0;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < part_len; i += blockDim.x) {
    const float v = yr[i] * silu_f(to_float(zr[i]));
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / static_cast<float>(part_len) + eps);
  T* orow = out + static_cast<size_t>(row) * inner + c0;
  for (int i = threadIdx.x; i < part_len; i += blockDim.x) {
    const float v = yr[i] * silu_f(to_float(zr[i]));
    orow[i] = from_float<T>(v * inv * w[c0 + i]);
  }
}

// The same with 8 channels a thread held in registers (one pass over memory, 16-byte accesses): for parts of a multiple of
// 8 channels, at most 8 * GN_CHUNKS * blockDim of them.
constexpr int GN_CHUNKS = 4;
template <typename T>
__global__ void gated_group_norm_vec_kernel(const float* __restrict__ y, const T* __restrict__ z, int z_stride,
                                            const float* __restrict__ w, float eps, T* __restrict__ out, int inner,
                                            int part_len) {
  __shared__ float red[33];
  const int row = blockIdx.x, c0 = blockIdx.y * part_len;
  const float* yr = y + static_cast<size_t>(row) * inner + c0;
  const T* zr = z + static_cast<size_t>(row) * z_stride + c0;
  float v[GN_CHUNKS][8];
  float ss = 0.0f;
#pragma unroll
  for (int k = 0; k < GN_CHUNKS; ++k) {
    const int i = (k * blockDim.x + threadIdx.x) * 8;
    if (i < part_len) {
      const float4 a = *reinterpret_cast<const float4*>(yr + i), b = *reinterpret_cast<const float4*>(yr + i + 4);
      float g[8];
      if (sizeof(T) == 2) {
        unpack<bf16>(*reinterpret_cast<const Vec16*>(zr + i), g);
      } else {
        unpack<float>(*reinterpret_cast<const Vec16*>(zr + i), g);
        unpack<float>(*reinterpret_cast<const Vec16*>(zr + i + 4), g + 4);
      }
      const float yv[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[k][j] = yv[j] * silu_f(g[j]);
        ss = fmaf(v[k][j], v[k][j], ss);
      }
    }
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / static_cast<float>(part_len) + eps);
  T* orow = out + static_cast<size_t>(row) * inner + c0;
#pragma unroll
  for (int k = 0; k < GN_CHUNKS; ++k) {
    const int i = (k * blockDim.x + threadIdx.x) * 8;
    if (i < part_len) {
      const float4 wa = *reinterpret_cast<const float4*>(w + c0 + i), wb = *reinterpret_cast<const float4*>(w + c0 + i + 4);
      float o[8] = {v[k][0] * inv * wa.x, v[k][1] * inv * wa.y, v[k][2] * inv * wa.z, v[k][3] * inv * wa.w,
                    v[k][4] * inv * wb.x, v[k][5] * inv * wb.y, v[k][6] * inv * wb.z, v[k][7] * inv * wb.w};
      if (sizeof(T) == 2) {
        *reinterpret_cast<Vec16*>(orow + i) = pack<bf16>(o);
      } else {
        *reinterpret_cast<Vec16*>(orow + i) = pack<float>(o);
        *reinterpret_cast<Vec16*>(orow + i + 4) = pack<float>(o + 4);
      }
    }
  }
}

}  // namespace dl

// out[row, ch] = silu(bias[ch] + sum_k taps[k, ch] * input(row's position - (K - 1 - k), ch)), the inputs being
// columns col0 .. col0 + channels of proj; taps: float32 [K, channels], tap by tap (the model file's [channels, K]
// transposed, so that neighbouring channels read neighbouring words). state: [slots, state_stride] float32, a slot's kept inputs at keep_off.
// The convolution with its options: act 1 = silu on the result, 0 = none; in_bias (float32 [channels], may be null) is
// added to every input that lies inside the sequence before the taps (the bias of the projection that made the
// inputs, where that product runs without it); kept inputs are stored without it.
DL_EXPORT int dl_short_conv(int dtype, const void* proj, int proj_stride, int col0, int channels, const float* taps,
                            const float* bias, int K, const float* state, long long state_stride, long long keep_off,
                            const int* positions, const int* row_request, const int* row_slot, const int* pos_start,
                            void* out, int rows, int act, const float* in_bias, cudaStream_t stream) {
  if (rows <= 0 || channels <= 0) return 0;
  if (K <= 0) return DL_ERR_UNSUPPORTED;
  const int threads = 256;
  if (dtype != 0 && dtype != 1) return DL_ERR_UNSUPPORTED;
  const int vec = dtype == 0 ? 4 : 8;
  const bool wide = channels % vec == 0 && col0 % vec == 0 && proj_stride % vec == 0 &&
                    (reinterpret_cast<uintptr_t>(proj) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
                    (reinterpret_cast<uintptr_t>(taps) & 15) == 0 && (bias == nullptr || (reinterpret_cast<uintptr_t>(bias) & 15) == 0);
  const size_t items = static_cast<size_t>(rows) * (wide ? channels / vec : channels);
  const unsigned blocks = static_cast<unsigned>((items + threads - 1) / threads);
#define DL_LAUNCH(KERNEL, T)                                                                                         \
  dl::KERNEL<T><<<blocks, threads, 0, stream>>>(static_cast<const T*>(proj), proj_stride, col0, channels, taps, bias, K, \
                                                state, static_cast<size_t>(state_stride), static_cast<size_t>(keep_off), \
                                                positions, row_request, row_slot, pos_start, static_cast<T*>(out), rows, \
                                                act, in_bias)
  if (dtype == 0 && wide) DL_LAUNCH(ssm_conv_vec_kernel, float);
  else if (dtype == 0) DL_LAUNCH(ssm_conv_kernel, float);
  else if (wide) DL_LAUNCH(ssm_conv_vec_kernel, dl::bf16);
  else DL_LAUNCH(ssm_conv_kernel, dl::bf16);
#undef DL_LAUNCH
  return dl::launch_status();
}

DL_EXPORT int dl_ssm_conv(int dtype, const void* proj, int proj_stride, int col0, int channels, const float* taps,
                          const float* bias, int K, const float* state, long long state_stride, long long keep_off,
                          const int* positions, const int* row_request, const int* row_slot, const int* pos_start,
                          void* out, int rows, cudaStream_t stream) {
  return dl_short_conv(dtype, proj, proj_stride, col0, channels, taps, bias, K, state, state_stride, keep_off, positions,
                       row_request, row_slot, pos_start, out, rows, 1, nullptr, stream);
}

DL_EXPORT int dl_ssm_conv_keep(int dtype, const void* proj, int proj_stride, int col0, int channels, int K, float* state,
                               long long state_stride, long long keep_off, const int* q_start, const int* state_slots,
                               int requests, cudaStream_t stream) {
  if (requests <= 0 || channels <= 0 || K <= 1) return 0;
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((static_cast<size_t>(requests) * channels + threads - 1) / threads);
  if (dtype == 0)
    dl::ssm_conv_keep_kernel<float><<<blocks, threads, 0, stream>>>(static_cast<const float*>(proj), proj_stride, col0, channels, K, state,
                                                                    static_cast<size_t>(state_stride), static_cast<size_t>(keep_off),
                                                                    q_start, state_slots, requests);
  else if (dtype == 1)
    dl::ssm_conv_keep_kernel<dl::bf16><<<blocks, threads, 0, stream>>>(static_cast<const dl::bf16*>(proj), proj_stride, col0, channels, K,
                                                                       state, static_cast<size_t>(state_stride),
                                                                       static_cast<size_t>(keep_off), q_start, state_slots, requests);
  else return DL_ERR_UNSUPPORTED;
  return dl::launch_status();
}

// u: the convolution's output [rows, H*P + 2*G*N]; proj: the projection (for dt); y: float32 [rows, H*P].
// Requests that bring at most `whole_up_to` tokens run from and into their state in one launch. The longer ones come cut
// into `n_segments` segments (segments: [n][4] = (slot, first row, rows, -), request by request and in order;
// long_requests: [n_long][4] = (first segment, segments, slot, -)) and run in three more launches through
// scratch (float32 [n_segments, H, N, P]) and seg_decay (float32 [n_segments, H]).
DL_EXPORT int dl_ssm_scan(int dtype, const void* u, int u_stride, const void* proj, int proj_stride, int dt_col,
                          const float* dt_bias, const float* a_log, const float* d_skip, float* state,
                          long long state_stride, const int* q_start, const int* state_slots, float* y, int requests, int H,
                          int P, int N, int G, int whole_up_to, const int* segments, int n_segments,
                          const int* long_requests, int n_long, float* scratch, float* seg_decay, cudaStream_t stream) {
  if (requests <= 0) return 0;
  if (H <= 0 || P <= 0 || N <= 0 || G <= 0 || H % G != 0 || H > 65535 || n_long > 65535) return DL_ERR_UNSUPPORTED;
  if (n_segments > 0 && (segments == nullptr || long_requests == nullptr || scratch == nullptr || seg_decay == nullptr))
    return DL_ERR_UNSUPPORTED;
  // rows of S per thread: 32 at most; NS threads share a channel
  const int NR = N <= 8 ? 8 : (N <= 64 ? 16 : 32);
  const int NS = (N + NR - 1) / NR;
  if (NS > 32) return DL_ERR_UNSUPPORTED;                          // N up to 1,024
  const bool full = NS * NR == N && N % 2 == 0;
  int PV = 256 / NS;                                               // channels to a block: at most 256 threads
  if (PV > P) PV = P;
  if (PV > 32) PV &= ~31;                                          // whole warps share a j
  const int slices = (P + PV - 1) / PV;
  if (slices > 65535) return DL_ERR_UNSUPPORTED;
  const int threads = PV * NS;
  // 16-byte pieces fit: the next tile is copied while this one is computed
  const int vec = dtype == 0 ? 4 : 8;
  const bool async = N % vec == 0 && PV % vec == 0 && P % PV == 0 && u_stride % vec == 0 && threads >= dl::SCAN_TT &&
                     (reinterpret_cast<uintptr_t>(u) & 15) == 0;
  const size_t smem = sizeof(float) * (static_cast<size_t>(dl::SCAN_TT) * (2 * N + PV + NS * PV) + 2 * dl::SCAN_TT) +
                      (async ? 2 * static_cast<size_t>(dl::SCAN_TT) * (2 * N + PV) * (dtype == 0 ? 4 : 2) : 0);
  if (smem > 200 * 1024) return DL_ERR_UNSUPPORTED;
#define DL_LAUNCH(T, R, MODE, F, BLOCKS)                                                                              \
  do {                                                                                                                \
    if (async) DL_LAUNCH2(T, R, MODE, F, true, BLOCKS);                                                               \
    else DL_LAUNCH2(T, R, MODE, F, false, BLOCKS);                                                                    \
  } while (0)
#define DL_LAUNCH2(T, R, MODE, F, A, BLOCKS)                                                                          \
  do {                                                                                                                \
    if (smem > 48 * 1024)                                                                                             \
      cudaFuncSetAttribute(dl::ssm_scan_kernel<T, R, MODE, F, A>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)); \
    dl::ssm_scan_kernel<T, R, MODE, F, A><<<dim3(BLOCKS, H, slices), threads, smem, stream>>>(                         \
        static_cast<const T*>(u), u_stride, static_cast<const T*>(proj), proj_stride, dt_col, dt_bias, a_log, d_skip,  \
        state, static_cast<size_t>(state_stride), q_start, state_slots, segments, scratch, seg_decay, whole_up_to, y,  \
        H, P, N, G, PV, NS);                                                                                           \
  } while (0)
#define DL_PICK(T, MODE, BLOCKS)                                                          \
  do {                                                                                    \
    if (NR == 8) { if (full) DL_LAUNCH(T, 8, MODE, true, BLOCKS); else DL_LAUNCH(T, 8, MODE, false, BLOCKS); }        \
    else if (NR == 16) { if (full) DL_LAUNCH(T, 16, MODE, true, BLOCKS); else DL_LAUNCH(T, 16, MODE, false, BLOCKS); } \
    else { if (full) DL_LAUNCH(T, 32, MODE, true, BLOCKS); else DL_LAUNCH(T, 32, MODE, false, BLOCKS); }              \
  } while (0)
#define DL_MODE(MODE, BLOCKS)                         \
  do {                                                \
    if (dtype == 0) DL_PICK(float, MODE, BLOCKS);     \
    else DL_PICK(dl::bf16, MODE, BLOCKS);             \
  } while (0)
  if (dtype != 0 && dtype != 1) return DL_ERR_UNSUPPORTED;
  DL_MODE(dl::SCAN_WHOLE, requests);
  if (n_segments > 0) {
    DL_MODE(dl::SCAN_LOCAL, n_segments);
    const int per_head = N * P;
    const size_t per_seg = static_cast<size_t>(H) * per_head;
    dl::ssm_carry_kernel<<<dim3(static_cast<unsigned>((per_seg + 255) / 256), n_long), 256, 0, stream>>>(
        state, static_cast<size_t>(state_stride), scratch, seg_decay, long_requests, H, per_head);
    DL_MODE(dl::SCAN_FINISH, n_segments);
  }
#undef DL_MODE
#undef DL_PICK
#undef DL_LAUNCH
#undef DL_LAUNCH2
  return dl::launch_status();
}

// y: float32 [rows, inner]; z: rows of z_stride elements (the gate's columns first); out: [rows, inner].
DL_EXPORT int dl_gated_group_norm(int dtype, const float* y, const void* z, int z_stride, const float* w, float eps,
                                  void* out, int rows, int inner, int parts, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (inner <= 0 || parts <= 0 || inner % parts != 0 || parts > 65535) return DL_ERR_UNSUPPORTED;
  const int part_len = inner / parts;
  dim3 grid(rows, parts);
  if ((dtype == 0 || dtype == 1) && part_len % 8 == 0 && part_len <= 8 * dl::GN_CHUNKS * 256 && inner % 8 == 0 && z_stride % 8 == 0 &&
      (reinterpret_cast<uintptr_t>(y) & 15) == 0 && (reinterpret_cast<uintptr_t>(z) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    int vt = (part_len / 8 + 31) / 32 * 32;                         // a thread per 8 channels, whole warps, 256 at most
    if (vt > 256) vt = 256;
    if (dtype == 0)
      dl::gated_group_norm_vec_kernel<float><<<grid, vt, 0, stream>>>(y, static_cast<const float*>(z), z_stride, w, eps,
                                                                      static_cast<float*>(out), inner, part_len);
    else
      dl::gated_group_norm_vec_kernel<dl::bf16><<<grid, vt, 0, stream>>>(y, static_cast<const dl::bf16*>(z), z_stride, w, eps,
                                                                         static_cast<dl::bf16*>(out), inner, part_len);
    return dl::launch_status();
  }
  const int threads = part_len >= 1024 ? 256 : (part_len >= 256 ? 128 : 64);
  if (dtype == 0)
    dl::gated_group_norm_kernel<float><<<grid, threads, 0, stream>>>(y, static_cast<const float*>(z), z_stride, w, eps,
                                                                     static_cast<float*>(out), inner, part_len);
  else if (dtype == 1)
    dl::gated_group_norm_kernel<dl::bf16><<<grid, threads, 0, stream>>>(y, static_cast<const dl::bf16*>(z), z_stride, w, eps,
                                                                        static_cast<dl::bf16*>(out), inner, part_len);
  else return DL_ERR_UNSUPPORTED;
  return dl::launch_status();
}
