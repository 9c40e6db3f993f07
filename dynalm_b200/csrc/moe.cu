// Mixture of experts: routing, the grouping of (token, expert) pairs by expert, the experts' products over those
// groups, and the weighted sum of a token's experts.
//
//   dl_moe_route     scores = softmax(router logits) over all experts, float32. Experts form `groups` equal groups of
//                    neighbours; a group's score is its largest score and only experts of the `keep` best groups can be
//                    chosen. The `top` allowed experts with the largest scores are chosen (equal scores: the lower
//                    index), their weights are their scores divided by their sum (+ 1e-20), times `scale`.
//   dl_moe_group     a counting sort of the tokens' pairs by expert: where every pair stands in that order, which pair
//                    stands at every place, and the list of row tiles (expert, first place, places) for the products.
//   dl_moe_linear    C[place] = act(A[row of place] W_e^T) for every place of every tile, W_e the matrix of the tile's
//                    expert: a plain tiled product with float32 accumulation in a fixed order of k (any dtype), and one on
//                    the tensor cores for bfloat16 (mma.sync m16n8k16, float32 accumulation), with tiles of 32 places for
//                    steps that bring an expert few and of 128 for steps that bring it many.
//   dl_moe_combine   y[t] = sum_k weight[t, k] * C[place of pair (t, k)], float32, in the order of k.
#include "common.cuh"

namespace dl {

constexpr int MOE_MAX_EXPERTS = 256;
constexpr int MOE_TM = 32;          // places a tile of the kernels for few places an expert
constexpr int MOE_TM_WIDE = 128;    // places a tile of the kernel for many

__global__ void moe_route_kernel(const float* __restrict__ logits, int stride, int tokens, int E, int top, int groups,
                                 int keep, float scale, int* __restrict__ ids, float* __restrict__ weights) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= tokens) return;
  float s[MOE_MAX_EXPERTS];
  const float* z = logits + static_cast<size_t>(t) * stride;
  float m = -INFINITY;
  for (int i = 0; i < E; ++i) m = fmaxf(m, z[i]);
  float sum = 0.0f;
  for (int i = 0; i < E; ++i) {
    s[i] = expf(z[i] - m);
    sum += s[i];
  }
  const float inv = 1.0f / sum;
  for (int i = 0; i < E; ++i) s[i] *= inv;
  const int per = E / groups;
  unsigned long long allowed_lo[MOE_MAX_EXPERTS / 64];      // bit g: group g is kept (groups <= experts <= 256)
  for (int w = 0; w < MOE_MAX_EXPERTS / 64; ++w) allowed_lo[w] = 0ull;
  if (keep >= groups) {
    for (int g = 0; g < groups; ++g) allowed_lo[g >> 6] |= 1ull << (g & 63);
  } else {
    for (int r = 0; r < keep; ++r) {
      int best = -1;
      float bs = -INFINITY;
      for (int g = 0; g < groups; ++g) {
        if (allowed_lo[g >> 6] >> (g & 63) & 1ull) continue;
        float gs = -INFINITY;
        for (int i = g * per; i < (g + 1) * per; ++i) gs = fmaxf(gs, s[i]);
        if (gs > bs) { bs = gs; best = g; }
      }
      if (best >= 0) allowed_lo[best >> 6] |= 1ull << (best & 63);
    }
  }
  float wsum = 0.0f;
  int* my_ids = ids + static_cast<size_t>(t) * top;
  float* my_w = weights + static_cast<size_t>(t) * top;
  for (int r = 0; r < top; ++r) {
    int best = -1;
    float bs = -INFINITY;
    for (int i = 0; i < E; ++i) {
      const int g = i / per;
      if (!(allowed_lo[g >> 6] >> (g & 63) & 1ull)) continue;
      bool taken = false;
      for (int q = 0; q < r; ++q) taken |= my_ids[q] == i;
      if (!taken && s[i] > bs) { bs = s[i]; best = i; }
    }
    if (best < 0) best = 0;                                  // (scores that are not numbers: some expert all the same)
    my_ids[r] = best;
    my_w[r] = s[best];
    wsum += s[best];
  }
  const float f = scale / (wsum + 1e-20f);
  for (int r = 0; r < top; ++r) my_w[r] *= f;
}

// One block. pairs = tokens * top. Outputs: place_of[pair], pair_at[place], tiles[3 * i] = (expert, first place,
// places) for i < n_tiles[0].
__global__ void __launch_bounds__(1024)
moe_group_kernel(const int* __restrict__ ids, int pairs, int E, int* __restrict__ place_of, int* __restrict__ pair_at,
                 int* __restrict__ tiles, int* __restrict__ n_tiles, int TM) {
  __shared__ int count[MOE_MAX_EXPERTS], first[MOE_MAX_EXPERTS + 1], cursor[MOE_MAX_EXPERTS], tile0[MOE_MAX_EXPERTS + 1];
  const int tid = threadIdx.x;
  for (int i = tid; i < E; i += blockDim.x) { count[i] = 0; cursor[i] = 0; }
  __syncthreads();
  for (int p = tid; p < pairs; p += blockDim.x) atomicAdd(&count[min(max(ids[p], 0), E - 1)], 1);
  __syncthreads();
  if (tid == 0) {
    int at = 0, tl = 0;
    for (int i = 0; i < E; ++i) {
      first[i] = at;
      tile0[i] = tl;
      at += count[i];
      tl += (count[i] + TM - 1) / TM;
    }
    first[E] = at;
    tile0[E] = tl;
    n_tiles[0] = tl;
  }
  __syncthreads();
  // Places inside an expert's run are dealt in the order in which the threads arrive: a run's order changes no
  // result (every place is a product of its own), only which places share a tile.
  for (int p = tid; p < pairs; p += blockDim.x) {
    const int ex = min(max(ids[p], 0), E - 1);
    const int place = first[ex] + atomicAdd(&cursor[ex], 1);
    place_of[p] = place;
    pair_at[place] = p;
  }
  for (int i = tid; i < E; i += blockDim.x) {
    const int nt = (count[i] + TM - 1) / TM;
    for (int j = 0; j < nt; ++j) {
      int* tl = tiles + 3 * (tile0[i] + j);
      tl[0] = i;
      tl[1] = first[i] + j * TM;
      tl[2] = min(TM, count[i] - j * TM);
    }
  }
}

template <typename T>
__device__ __forceinline__ float apply_act(float v, int act) {
  if (act == 1) { v = fmaxf(v, 0.0f); v = v * v; }
  return v;
}

// Plain tiled product: tile = 32 places x 64 features, 256 threads, 2 x 4 results a thread, k in steps of 16.
// A row of place p: a[(rows_of ? rows_of[pair_at[p]] / div : p) * lda]; W of expert x: w + x * N * K, [N, K].
template <typename T, typename TO>
__global__ void __launch_bounds__(256)
moe_linear_simt_kernel(const T* __restrict__ a, int lda, const int* __restrict__ pair_at, int top_div,
                       const T* __restrict__ w, int N, int K, TO* __restrict__ c, int ldc, const int* __restrict__ tiles,
                       const int* __restrict__ n_tiles, int act) {
  constexpr int TN = 64, TK = 16;
  __shared__ float As[TK][MOE_TM + 1], Bs[TK][TN + 1];
  __shared__ int src[MOE_TM];
  if (static_cast<int>(blockIdx.y) >= n_tiles[0]) return;
  const int* tl = tiles + 3 * blockIdx.y;
  const int ex = tl[0], p0 = tl[1], np = tl[2];
  const int n0 = blockIdx.x * TN;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  if (tid < MOE_TM) src[tid] = tid < np ? (pair_at != nullptr ? pair_at[p0 + tid] / top_div : p0 + tid) : -1;
  __syncthreads();
  const T* wx = w + static_cast<size_t>(ex) * N * K;
  float acc[2][4] = {};
  for (int k0 = 0; k0 < K; k0 += TK) {
    for (int x = tid; x < MOE_TM * TK; x += 256) {
      const int r = x / TK, k = x % TK;
      As[k][r] = (src[r] >= 0 && k0 + k < K) ? to_float(a[static_cast<size_t>(src[r]) * lda + k0 + k]) : 0.0f;
    }
    for (int x = tid; x < TN * TK; x += 256) {
      const int n = x / TK, k = x % TK;
      Bs[k][n] = (n0 + n < N && k0 + k < K) ? to_float(wx[static_cast<size_t>(n0 + n) * K + k0 + k]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TK; ++k) {
      const float a0 = As[k][ty * 2], a1 = As[k][ty * 2 + 1];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float b = Bs[k][tx * 4 + j];
        acc[0][j] = fmaf(a0, b, acc[0][j]);
        acc[1][j] = fmaf(a1, b, acc[1][j]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = ty * 2 + i;
    if (r >= np) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) c[static_cast<size_t>(p0 + r) * ldc + n] = from_float<TO>(apply_act<T>(acc[i][j], act));
    }
  }
}

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// bfloat16 on the tensor cores: tile = TM places x 128 features, 8 warps as WM x (8 / WM), k in steps of BK through a
// ring of STAGES cp.async buffers (the next steps' A and W are on their way while this one is multiplied, one block
// barrier a step), fragments by ldmatrix, rows padded by 16 bytes so that a fragment's rows fall on different banks.
//   TM = 128, WM = 2: a warp takes 64 places x 32 features; for steps that bring an expert many places, whose
//   matrix is then read once per 128 places.
//   TM = 32, WM = 1: a warp takes all 32 places x 16 features; for steps that bring an expert a few places (a
//   decode batch), which stream every touched expert's matrix once and are bound by that stream.
__device__ __forceinline__ void moe_cp16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const int bytes = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void moe_ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}

template <int TM, int WM, int BK, int STAGES, typename TO>
__global__ void __launch_bounds__(256)
moe_linear_tc_kernel(const bf16* __restrict__ a, int lda, const int* __restrict__ pair_at, int top_div,
                     const bf16* __restrict__ w, int N, int K, TO* __restrict__ c, int ldc, const int* __restrict__ tiles,
                     const int* __restrict__ n_tiles, int act) {
  constexpr int TN = 128, LD = BK + 8, WN = 8 / WM;
  constexpr int MI = TM / WM / 16;          // m16 fragments a warp
  constexpr int NI = TN / WN / 8;           // n8 fragments a warp (two per ldmatrix.x4)
  constexpr int CH = BK / 8;                // 16-byte pieces a row of a stage
  extern __shared__ __align__(16) unsigned char moe_smem[];
  bf16 (*As)[TM][LD] = reinterpret_cast<bf16 (*)[TM][LD]>(moe_smem);                                  // [STAGES][TM][LD]
  bf16 (*Bs)[TN][LD] = reinterpret_cast<bf16 (*)[TN][LD]>(moe_smem + sizeof(bf16) * STAGES * TM * LD);  // [STAGES][TN][LD]
  __shared__ int src[TM];
  if (static_cast<int>(blockIdx.y) >= n_tiles[0]) return;
  const int* tl = tiles + 3 * blockIdx.y;
  const int ex = tl[0], p0 = tl[1], np = tl[2];
  const int n0 = blockIdx.x * TN;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = warp / WN, wn = warp % WN;
  if (tid < TM) src[tid] = tid < np ? (pair_at != nullptr ? pair_at[p0 + tid] / top_div : p0 + tid) : -1;
  __syncthreads();
  const bf16* wx = w + static_cast<size_t>(ex) * N * K;
  auto load = [&](int stage, int k0) {
    for (int x = tid; x < TM * CH; x += 256) {
      const int r = x / CH, piece = x % CH;
      const bool ok = src[r] >= 0;
      moe_cp16(&As[stage][r][piece * 8], a + static_cast<size_t>(ok ? src[r] : 0) * lda + k0 + piece * 8, ok);
    }
    for (int x = tid; x < TN * CH; x += 256) {
      const int r = x / CH, piece = x % CH;
      const bool ok = n0 + r < N;
      moe_cp16(&Bs[stage][r][piece * 8], wx + static_cast<size_t>(ok ? n0 + r : 0) * K + k0 + piece * 8, ok);
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };
  float acc[MI][NI][4] = {};
  const int steps = K / BK;
  // STAGES - 1 steps are on their way at any time; a group is committed every round (an empty one past the end), so that
  // "all but the newest STAGES - 2 groups have landed" always names the step about to be multiplied
  for (int i = 0; i < STAGES - 1; ++i) {
    if (i < steps) load(i, i * BK);
    else asm volatile("cp.async.commit_group;\n" ::);
  }
  for (int s = 0; s < steps; ++s) {
    const int st = s % STAGES;
    asm volatile("cp.async.wait_group %0;\n" ::"n"(STAGES - 2));
    __syncthreads();                         // step s is in shared memory, and every warp is done with step s - 1
    if (s + STAGES - 1 < steps) load((s + STAGES - 1) % STAGES, (s + STAGES - 1) * BK);
    else asm volatile("cp.async.commit_group;\n" ::);
#pragma unroll
    for (int kk = 0; kk < BK; kk += 16) {
      uint32_t af[MI][4], bfr[NI / 2][4];
#pragma unroll
      for (int mi = 0; mi < MI; ++mi)
        moe_ldmatrix_x4(af[mi], &As[st][wm * (TM / WM) + mi * 16 + (lane & 7) + ((lane >> 3) & 1) * 8][kk + (lane >> 4) * 8]);
#pragma unroll
      for (int nj = 0; nj < NI / 2; ++nj)       // two n8 fragments per ldmatrix.x4
        moe_ldmatrix_x4(bfr[nj], &Bs[st][wn * (TN / WN) + nj * 16 + (lane & 7) + (lane >> 4) * 8][kk + ((lane >> 3) & 1) * 8]);
#pragma unroll
      for (int mi = 0; mi < MI; ++mi)
#pragma unroll
        for (int ni = 0; ni < NI; ++ni) {
          const uint32_t b2[2] = {bfr[ni >> 1][(ni & 1) * 2], bfr[ni >> 1][(ni & 1) * 2 + 1]};
          mma_bf16_16816(acc[mi][ni], af[mi], b2);
        }
    }
  }
  const int g = lane >> 2, q = lane & 3;
#pragma unroll
  for (int mi = 0; mi < MI; ++mi)
#pragma unroll
    for (int ni = 0; ni < NI; ++ni)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int r = wm * (TM / WM) + mi * 16 + g + 8 * h;
        const int n = n0 + wn * (TN / WN) + ni * 8 + q * 2;
        if (r >= np) continue;
        TO* dst = c + static_cast<size_t>(p0 + r) * ldc + n;
        if (n < N) dst[0] = from_float<TO>(apply_act<bf16>(acc[mi][ni][2 * h], act));
        if (n + 1 < N) dst[1] = from_float<TO>(apply_act<bf16>(acc[mi][ni][2 * h + 1], act));
      }
}

// out[place] = a[pair_at[place] / top_div]: the rows of a step in the order of their experts, 16 bytes a thread.
__global__ void moe_gather_kernel(const uint4* __restrict__ a, int lda16, const int* __restrict__ pair_at, int top_div,
                                  uint4* __restrict__ out, int row16, size_t total) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t place = i / row16;
  const int c = static_cast<int>(i % row16);
  out[i] = a[static_cast<size_t>(pair_at[place] / top_div) * lda16 + c];
}

template <typename TO>
__global__ void moe_combine_kernel(const float* __restrict__ c, int width, const int* __restrict__ place_of,
                                   const float* __restrict__ weights, int top, TO* __restrict__ y, size_t total) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t t = i / width;
  const int col = static_cast<int>(i % width);
  float sum = 0.0f;
  for (int k = 0; k < top; ++k)
    sum = fmaf(weights[t * top + k], c[static_cast<size_t>(place_of[t * top + k]) * width + col], sum);
  y[i] = from_float<TO>(sum);
}

}  // namespace dl

DL_EXPORT int dl_moe_route(const float* logits, int stride, int tokens, int E, int top, int groups, int keep, float scale,
                           int* ids, float* weights, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (E <= 0 || E > dl::MOE_MAX_EXPERTS || top <= 0 || top > E || groups <= 0 || E % groups || keep <= 0 || keep > groups ||
      top > keep * (E / groups))
    return DL_ERR_UNSUPPORTED;
  dl::moe_route_kernel<<<(tokens + 127) / 128, 128, 0, stream>>>(logits, stride, tokens, E, top, groups, keep, scale, ids, weights);
  return dl::launch_status();
}

DL_EXPORT int dl_moe_group(const int* ids, int pairs, int E, int* place_of, int* pair_at, int* tiles, int* n_tiles,
                           int tile_rows, cudaStream_t stream) {
  if (pairs <= 0) return 0;
  if (E <= 0 || E > dl::MOE_MAX_EXPERTS || (tile_rows != dl::MOE_TM && tile_rows != dl::MOE_TM_WIDE)) return DL_ERR_UNSUPPORTED;
  dl::moe_group_kernel<<<1, 1024, 0, stream>>>(ids, pairs, E, place_of, pair_at, tiles, n_tiles, tile_rows);
  return dl::launch_status();
}

// dtype of a and w: 0 float32, 1 bfloat16; out_dtype of c likewise. pair_at null: the rows of a are the places
// themselves; else the row of a place is pair_at[place] / top_div. act: 0 none, 1 squared ReLU. tensor_cores: use the
// mma.sync kernels where they apply (bfloat16, K a multiple of 64, rows of a and w on 16-byte boundaries).
// tile_rows: the places a tile as dl_moe_group was told: 32, or 128 for the wide tensor-core kernel (bfloat16 only).
DL_EXPORT int dl_moe_linear(int dtype, int out_dtype, const void* a, int lda, const int* pair_at, int top_div, const void* w,
                            int N, int K, void* c, int ldc, const int* tiles, const int* n_tiles, int max_tiles, int act,
                            int tensor_cores, int tile_rows, cudaStream_t stream) {
  if (max_tiles <= 0) return 0;
  if (N <= 0 || K <= 0 || top_div <= 0 || max_tiles > 65535) return DL_ERR_UNSUPPORTED;
  const bool wide = tile_rows == dl::MOE_TM_WIDE;
  if (!wide && tile_rows != dl::MOE_TM) return DL_ERR_UNSUPPORTED;
  const bool tc_ok = dtype == 1 && tensor_cores && K % 64 == 0 && lda % 8 == 0 && (reinterpret_cast<uintptr_t>(a) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(w) & 15) == 0;
  if (wide && !tc_ok) return DL_ERR_UNSUPPORTED;
  if (tc_ok) {
    dim3 grid((N + 127) / 128, max_tiles);
#define DL_MOE_TC_ONE(TM_, WM_, BK_, TO)                                                                                  \
  do {                                                                                                                    \
    constexpr int ST = 3;                                                                                                 \
    constexpr int smem = ST * (TM_ + 128) * (BK_ + 8) * 2;                                                                \
    static bool configured = false;                                                                                       \
    if (!configured) {                                                                                                    \
      cudaError_t e = cudaFuncSetAttribute(dl::moe_linear_tc_kernel<TM_, WM_, BK_, ST, TO>,                               \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, smem);                            \
      if (e != cudaSuccess) return static_cast<int>(e);                                                                   \
      configured = true;                                                                                                  \
    }                                                                                                                     \
    dl::moe_linear_tc_kernel<TM_, WM_, BK_, ST, TO><<<grid, 256, smem, stream>>>(                                         \
        static_cast<const dl::bf16*>(a), lda, pair_at, top_div, static_cast<const dl::bf16*>(w), N, K, static_cast<TO*>(c), \
        ldc, tiles, n_tiles, act);                                                                                        \
  } while (0)
#define DL_MOE_TC(TO)                                         \
  do {                                                        \
    if (wide) DL_MOE_TC_ONE(dl::MOE_TM_WIDE, 2, 64, TO);      \
    else DL_MOE_TC_ONE(dl::MOE_TM, 1, 64, TO);                \
  } while (0)
    if (out_dtype == 1) DL_MOE_TC(dl::bf16);
    else if (out_dtype == 0) DL_MOE_TC(float);
    else return DL_ERR_UNSUPPORTED;
#undef DL_MOE_TC
#undef DL_MOE_TC_ONE
    return dl::launch_status();
  }
  dim3 grid((N + 63) / 64, max_tiles);
#define DL_MOE(T, TO)                                                                                                      \
  dl::moe_linear_simt_kernel<T, TO><<<grid, 256, 0, stream>>>(static_cast<const T*>(a), lda, pair_at, top_div,              \
                                                              static_cast<const T*>(w), N, K, static_cast<TO*>(c), ldc, tiles, \
                                                              n_tiles, act)
  if (dtype == 0 && out_dtype == 0) DL_MOE(float, float);
  else if (dtype == 1 && out_dtype == 1) DL_MOE(dl::bf16, dl::bf16);
  else if (dtype == 1 && out_dtype == 0) DL_MOE(dl::bf16, float);
  else return DL_ERR_UNSUPPORTED;
#undef DL_MOE
  return dl::launch_status();
}

// out [pairs, K] = the rows of a (bf16, K a multiple of 8, lda a multiple of 8, both 16-byte aligned) in place order.
DL_EXPORT int dl_moe_gather(const void* a, int lda, const int* pair_at, int top_div, void* out, int pairs, int K,
                            cudaStream_t stream) {
  if (pairs <= 0) return 0;
  if (K <= 0 || (K & 7) || (lda & 7) || top_div <= 0 || (reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return DL_ERR_UNSUPPORTED;
  const size_t total = static_cast<size_t>(pairs) * (K / 8);
  dl::moe_gather_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
      static_cast<const uint4*>(a), lda / 8, pair_at, top_div, static_cast<uint4*>(out), K / 8, total);
  return dl::launch_status();
}

DL_EXPORT int dl_moe_combine(int out_dtype, const float* c, int width, const int* place_of, const float* weights, int top,
                             void* y, int tokens, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const size_t total = static_cast<size_t>(tokens) * width;
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
  if (out_dtype == 0) dl::moe_combine_kernel<float><<<blocks, 256, 0, stream>>>(c, width, place_of, weights, top, static_cast<float*>(y), total);
  else if (out_dtype == 1) dl::moe_combine_kernel<dl::bf16><<<blocks, 256, 0, stream>>>(c, width, place_of, weights, top, static_cast<dl::bf16*>(y), total);
  else return DL_ERR_UNSUPPORTED;
  return dl::launch_status();
}
