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
constexpr int LN_MAX_PARTS = 8;

template <typename TO, typename TD>
__global__ void __launch_bounds__(LN_THREADS)
stream_layer_norm_kernel(float* __restrict__ streams, int S, int W, const float* __restrict__ init,
                         const TD* __restrict__ delta, int parts, size_t part_stride, float delta_scale,
                         const float* __restrict__ mix, const float* __restrict__ outw, const float* __restrict__ inw,
                         const float* __restrict__ w, const float* __restrict__ b, float eps, TO* __restrict__ out,
                         const int* __restrict__ rows_idx, int total_rows) {
  extern __shared__ float su[];                 // u of the row, then 33 floats for the block sums
  float* red = su + W;
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
  for (int c = tid; c < W; c += LN_THREADS) {
    float x[LN_MAX_PARTS];
    if (init != nullptr) {
      const float v = init[static_cast<size_t>(row) * W + c];
#pragma unroll
      for (int s = 0; s < LN_MAX_PARTS; ++s) x[s] = v;
    } else {
#pragma unroll
      for (int s = 0; s < LN_MAX_PARTS; ++s) x[s] = s < S ? xrow[static_cast<size_t>(s) * W + c] : 0.0f;
    }
    float u = 0.0f;
    if (update) {
      float y = 0.0f;
      for (int p = 0; p < parts; ++p) y += to_float(delta[p * part_stride + static_cast<size_t>(row) * W + c]);
      y *= delta_scale;
#pragma unroll
      for (int t = 0; t < LN_MAX_PARTS; ++t) {
        if (t < S) {
          float v = 0.0f;
          if (mix != nullptr) {
#pragma unroll
            for (int s = 0; s < LN_MAX_PARTS; ++s)
              if (s < S) v = fmaf(s_mix[s * S + t], x[s], v);
          } else {
            v = x[t];
          }
          v = fmaf(s_out[t], y, v);
          if (write_back) xrow[static_cast<size_t>(t) * W + c] = v;
          u = fmaf(s_in[t], v, u);
        }
      }
    } else {
#pragma unroll
      for (int t = 0; t < LN_MAX_PARTS; ++t) {
        if (t < S) {
          if (init != nullptr && write_back) xrow[static_cast<size_t>(t) * W + c] = x[t];
          u = fmaf(s_in[t], x[t], u);
        }
      }
    }
    su[c] = u;
    sum += u;
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
    for (int c = tid; c < W; c += LN_THREADS)
      orow[c] = from_float<TO>((su[c] - mean) * rstd * w[c] + (b != nullptr ? b[c] : 0.0f));
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
  const size_t smem = (static_cast<size_t>(W) + 33) * sizeof(float);
#define DL_LN(TO, TD)                                                                                                   \
  dl::stream_layer_norm_kernel<TO, TD><<<n_out, dl::LN_THREADS, smem, stream>>>(                                       \
      streams, S, W, init, static_cast<const TD*>(delta), parts, static_cast<size_t>(part_stride), delta_scale, mix, outw, \
      inw, w, b, eps, static_cast<TO*>(out), rows_idx, total_rows)
  if (out_dtype == 0 && delta_dtype == 0) DL_LN(float, float);
  else if (out_dtype == 1 && delta_dtype == 1) DL_LN(dl::bf16, dl::bf16);
  else if (out_dtype == 1 && delta_dtype == 0) DL_LN(dl::bf16, float);
  else if (out_dtype == 0 && delta_dtype == 1) DL_LN(float, dl::bf16);
  else return DL_ERR_UNSUPPORTED;
#undef DL_LN
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
