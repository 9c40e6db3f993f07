// Layer norm of the residual stream, fused with what the sublayer in front left to be added, for a stream of one
// part (a plain running sum) or of several (hyper-connections).
//
// A row of the stream holds S parts x_0 .. x_{S-1} of W numbers each, float32. Per row, in float32:
//
//   if `init` is given:   x_s = init for every s                      (the first layer: every part starts as the embedding)
//   if `delta` is given:  y = delta_scale * (sum over its partial sums);   x_t <- sum_s mix[s, t] x_s + outw[t] * y
//                         (mix absent: the identity; outw absent: ones), written back unless rows are gathered
//   u = sum_t inw[t] x_t  (inw absent: ones)
//   out = (u - mean(u)) / sqrt(mean((u - mean(u))^2) + eps) * w + b       (b may be absent)
//
// The mean and the variance are taken in two passes over u, which waits in shared memory. With `rows_idx` the kernel
// norms only those rows (the rows whose logits are wanted) and leaves the stream as it is.
#include "common.cuh"

namespace dl {

constexpr int LN_THREADS = 256;
constexpr int LN_MAX_PARTS = 16;      // the most parts a stream may have; a kernel instance holds 4, 8 or 16 of them (more
                                      // than 8: one number at a time, or the parts would not fit the registers)

// V numbers at a time: V = 4 when every row starts on a 16-byte boundary (W a multiple of 4), else 1.
template <typename T, int V> struct LnVec {
  static __device__ __forceinline__ void load(const T* p, float* out) {
#pragma unroll
    for (int i = 0; i < V; ++i) out[i] = to_float(p[i]);
  }
};
template <> struct LnVec<float, 4> {
  static __device__ __forceinline__ void load(const float* p, float* out) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
  }
};
template <> struct LnVec<bf16, 4> {
  static __device__ __forceinline__ void load(const bf16* p, float* out) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    out[0] = __uint_as_float(v.x << 16); out[1] = __uint_as_float(v.x & 0xffff0000u);
    out[2] = __uint_as_float(v.y << 16); out[3] = __uint_as_float(v.y & 0xffff0000u);
  }
};
template <int V> __device__ __forceinline__ void ln_store(float* p, const float* v) {
  if (V == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  else p[0] = v[0];
}
template <int V> __device__ __forceinline__ void ln_store(bf16* p, const float* v) {
  if (V == 4) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
  } else {
    p[0] = __float2bfloat16_rn(v[0]);
  }
}

template <typename TO, typename TD, int V, int MAXP>
__global__ void __launch_bounds__(LN_THREADS)
stream_layer_norm_kernel(float* __restrict__ streams, int S, int W, const float* __restrict__ init,
                         const TD* __restrict__ delta, int parts, size_t part_stride, float delta_scale,
                         const float* __restrict__ mix, const float* __restrict__ outw, const float* __restrict__ inw,
                         const float* __restrict__ w, const float* __restrict__ b, float eps, TO* __restrict__ out,
                         const int* __restrict__ rows_idx, int total_rows) {
  extern __shared__ __align__(16) float su[];   // u of the row, then 33 floats for the block sums
  float* red = su + ((W + 3) & ~3);
  __shared__ float s_mix[LN_MAX_PARTS * LN_MAX_PARTS], s_out[LN_MAX_PARTS], s_in[LN_MAX_PARTS];
  const int tid = threadIdx.x;
  const int row = rows_idx != nullptr ? ck_row(rows_idx[blockIdx.x], total_rows) : static_cast<int>(blockIdx.x);
  const bool write_back = rows_idx == nullptr;
  if (tid < S * S) s_mix[tid] = mix != nullptr ? mix[tid] : ((tid / S) == (tid % S) ? 1.0f : 0.0f);
  if (tid < S) {
    s_out[tid] = outw != nullptr ? outw[tid] : 1.0f;
    s_in[tid] = inw != nullptr ? inw[tid] : 1.0f;
  }
  __syncthreads();
  float* xrow = streams + static_cast<size_t>(row) * S * W;
  const bool update = delta != nullptr;
  float sum = 0.0f;
  for (int c = tid * V; c < W; c += LN_THREADS * V) {
    float x[MAXP][V];
    if (init != nullptr) {
      float v[V];
      LnVec<float, V>::load(init + static_cast<size_t>(row) * W + c, v);
#pragma unroll
      for (int s = 0; s < MAXP; ++s)
#pragma unroll
        for (int i = 0; i < V; ++i) x[s][i] = v[i];
    } else {
#pragma unroll
      for (int s = 0; s < MAXP; ++s) {
        if (s < S) {
          LnVec<float, V>::load(xrow + static_cast<size_t>(s) * W + c, x[s]);
        } else {
#pragma unroll
          for (int i = 0; i < V; ++i) x[s][i] = 0.0f;
        }
      }
    }
    float u[V];
#pragma unroll
    for (int i = 0; i < V; ++i) u[i] = 0.0f;
    if (update) {
      float y[V];
#pragma unroll
      for (int i = 0; i < V; ++i) y[i] = 0.0f;
      for (int p = 0; p < parts; ++p) {
        float d[V];
        LnVec<TD, V>::load(delta + p * part_stride + static_cast<size_t>(row) * W + c, d);
#pragma unroll
        for (int i = 0; i < V; ++i) y[i] += d[i];
      }
#pragma unroll
      for (int i = 0; i < V; ++i) y[i] *= delta_scale;
#pragma unroll
      for (int t = 0; t < MAXP; ++t) {
        if (t < S) {
          float v[V];
#pragma unroll
          for (int i = 0; i < V; ++i) {
            float a = 0.0f;
            if (mix != nullptr) {
#pragma unroll
              for (int s = 0; s < MAXP; ++s)
                if (s < S) a = fmaf(s_mix[s * S + t], x[s][i], a);
            } else {
              a = x[t][i];
            }
            v[i] = fmaf(s_out[t], y[i], a);
            u[i] = fmaf(s_in[t], v[i], u[i]);
          }
          if (write_back) ln_store<V>(xrow + static_cast<size_t>(t) * W + c, v);
        }
      }
    } else {
#pragma unroll
      for (int t = 0; t < MAXP; ++t) {
        if (t < S) {
          if (init != nullptr && write_back) ln_store<V>(xrow + static_cast<size_t>(t) * W + c, x[t]);
#pragma unroll
          for (int i = 0; i < V; ++i) u[i] = fmaf(s_in[t], x[t][i], u[i]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < V; ++i) {
      su[c + i] = u[i];
      sum += u[i];
    }
  }
  const float mean = block_sum(sum, red) / static_cast<float>(W);
  float sq = 0.0f;
  for (int c = tid; c < W; c += LN_THREADS) {
    const float dv = su[c] - mean;
    sq = fmaf(dv, dv, sq);
  }
  const float rstd = 1.0f / sqrtf(block_sum(sq, red) / static_cast<float>(W) + eps);
  if (out != nullptr) {
    TO* orow = out + static_cast<size_t>(blockIdx.x) * W;
    for (int c = tid * V; c < W; c += LN_THREADS * V) {
      float v[V], wv[V], bv[V];
      LnVec<float, V>::load(w + c, wv);
      if (b != nullptr) LnVec<float, V>::load(b + c, bv);
#pragma unroll
      for (int i = 0; i < V; ++i) v[i] = (su[c + i] - mean) * rstd * wv[i] + (b != nullptr ? bv[i] : 0.0f);
      ln_store<V>(orow + c, v);
    }
  }
}

// The sum of a stream's parts, out[row] = sum_s x_s (after the pending update, as above), float32: for a consumer that
// wants the stream as one row.
template <typename TD>
__global__ void __launch_bounds__(LN_THREADS)
stream_sum_kernel(const float* __restrict__ streams, int S, int W, const TD* __restrict__ delta, int parts,
                  size_t part_stride, float delta_scale, const float* __restrict__ mix, const float* __restrict__ outw,
                  float* __restrict__ out, size_t total) {
  const size_t i = static_cast<size_t>(blockIdx.x) * LN_THREADS + threadIdx.x;
  if (i >= total) return;
  const size_t row = i / W;
  const int c = static_cast<int>(i % W);
  float y = 0.0f;
  if (delta != nullptr) {
    for (int p = 0; p < parts; ++p) y += to_float(delta[p * part_stride + row * W + c]);
    y *= delta_scale;
  }
  float u = 0.0f;
  for (int t = 0; t < S; ++t) {
    float v = 0.0f;
    if (mix != nullptr) {
      for (int s = 0; s < S; ++s) v = fmaf(mix[s * S + t], streams[(row * S + s) * W + c], v);
    } else {
      v = streams[(row * S + t) * W + c];
    }
    if (delta != nullptr) v = fmaf(outw != nullptr ? outw[t] : 1.0f, y, v);
    u += v;
  }
  out[i] = u;
}

}  // namespace dl

// out_dtype / delta_dtype: 0 float32, 1 bfloat16. streams: float32 [total_rows, S, W]. delta: [parts][total_rows, W],
// part_stride elements apart, or null. rows_idx: n_out row numbers, or null for all total_rows rows in order.
DL_EXPORT int dl_stream_layer_norm(int out_dtype, int delta_dtype, float* streams, int S, int W, const float* init,
                                   const void* delta, int parts, long long part_stride, float delta_scale,
                                   const float* mix, const float* outw, const float* inw, const float* w, const float* b,
                                   float eps, void* out, const int* rows_idx, int n_out, int total_rows,
                                   cudaStream_t stream) {
  if (n_out <= 0) return 0;
  if (S <= 0 || S > dl::LN_MAX_PARTS || W <= 0 || W > 49152 / 4 - 64 || (delta != nullptr && parts <= 0)) return DL_ERR_UNSUPPORTED;
  const size_t smem = (static_cast<size_t>((W + 3) & ~3) + 33) * sizeof(float);
  // four numbers at a time when every row and every partial sum starts on a 16-byte boundary
  const bool wide = W % 4 == 0 && part_stride % 4 == 0 && ((reinterpret_cast<uintptr_t>(streams) | reinterpret_cast<uintptr_t>(init) |
                    reinterpret_cast<uintptr_t>(delta) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(b) |
                    reinterpret_cast<uintptr_t>(out)) & 15) == 0;
#define DL_LN_ONE(TO, TD, V, MAXP)                                                                                      \
  dl::stream_layer_norm_kernel<TO, TD, V, MAXP><<<n_out, dl::LN_THREADS, smem, stream>>>(                               \
      streams, S, W, init, static_cast<const TD*>(delta), parts, static_cast<size_t>(part_stride), delta_scale, mix,    \
      outw, inw, w, b, eps, static_cast<TO*>(out), rows_idx, total_rows)
#define DL_LN(TO, TD)                                                                                                   \
  do {                                                                                                                  \
    if (wide && S <= 4) DL_LN_ONE(TO, TD, 4, 4);                                                                        \
    else if (wide && S <= 8) DL_LN_ONE(TO, TD, 4, 8);                                                                   \
    else if (S <= 4) DL_LN_ONE(TO, TD, 1, 4);                                                                           \
    else DL_LN_ONE(TO, TD, 1, 16);                                                                                      \
  } while (0)
  if (out_dtype == 0 && delta_dtype == 0) DL_LN(float, float);
  else if (out_dtype == 1 && delta_dtype == 1) DL_LN(dl::bf16, dl::bf16);
  else if (out_dtype == 1 && delta_dtype == 0) DL_LN(dl::bf16, float);
  else if (out_dtype == 0 && delta_dtype == 1) DL_LN(float, dl::bf16);
  else return DL_ERR_UNSUPPORTED;
#undef DL_LN
#undef DL_LN_ONE
  return dl::launch_status();
}

DL_EXPORT int dl_stream_sum(int delta_dtype, const float* streams, int S, int W, const void* delta, int parts,
                            long long part_stride, float delta_scale, const float* mix, const float* outw, float* out,
                            int rows, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (S <= 0 || W <= 0) return DL_ERR_UNSUPPORTED;
  const size_t total = static_cast<size_t>(rows) * W;
  const unsigned blocks = static_cast<unsigned>((total + dl::LN_THREADS - 1) / dl::LN_THREADS);
  if (delta_dtype == 0)
    dl::stream_sum_kernel<float><<<blocks, dl::LN_THREADS, 0, stream>>>(streams, S, W, static_cast<const float*>(delta), parts,
                                                                        static_cast<size_t>(part_stride), delta_scale, mix, outw, out, total);
  else if (delta_dtype == 1)
    dl::stream_sum_kernel<dl::bf16><<<blocks, dl::LN_THREADS, 0, stream>>>(streams, S, W, static_cast<const dl::bf16*>(delta), parts,
                                                                           static_cast<size_t>(part_stride), delta_scale, mix, outw, out, total);
  else return DL_ERR_UNSUPPORTED;
  return dl::launch_status();
}
