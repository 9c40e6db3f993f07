// The closing norm of a sublayer whose result is normed before it joins the stream, fused with the sum and with the
// opening norm of the sublayer that follows:
//
//   x   <- x + rmsnorm(delta) * w_post            rmsnorm(v) = v / sqrt(mean(v^2) + eps)
//   out  = rmsnorm(x) * w_pre                     (left out when w_pre is null)
//
// x is the float32 stream, updated in place; delta is the sublayer's result, [n, width] of either type or split-K
// partial sums [parts, n, width] that are added in order. One block per row; the row waits in shared memory between
// the two passes. Everything is float32.
#include "common.cuh"

namespace dl {

template <typename TD, typename TO>
__global__ void __launch_bounds__(256)
norm_add_norm_kernel(float* __restrict__ x, const TD* __restrict__ delta, int parts, size_t part_stride,
                     const float* __restrict__ w_post, float eps_post, const float* __restrict__ w_pre, float eps_pre,
                     TO* __restrict__ out, int width) {
  extern __shared__ float row_s[];
  __shared__ float red[33];
  const size_t base = static_cast<size_t>(blockIdx.x) * width;
  float ss = 0.0f;
  for (int j = threadIdx.x; j < width; j += blockDim.x) {
    float d = 0.0f;
    for (int p = 0; p < parts; ++p) d += to_float(delta[p * part_stride + base + j]);
    row_s[j] = d;
    ss = fmaf(d, d, ss);
  }
  const float rs = 1.0f / sqrtf(block_sum(ss, red) / static_cast<float>(width) + eps_post);
  float ss2 = 0.0f;
  for (int j = threadIdx.x; j < width; j += blockDim.x) {
    const float v = x[base + j] + row_s[j] * rs * w_post[j];
    x[base + j] = v;
    row_s[j] = v;
    ss2 = fmaf(v, v, ss2);
  }
  if (w_pre == nullptr) return;
  const float rs2 = 1.0f / sqrtf(block_sum(ss2, red) / static_cast<float>(width) + eps_pre);
  for (int j = threadIdx.x; j < width; j += blockDim.x) out[base + j] = from_float<TO>(row_s[j] * rs2 * w_pre[j]);
}

}  // namespace dl

// out_dtype / delta_dtype: 0 float32, 1 bfloat16. w_pre and out may be null (no opening norm behind the sum).
DL_EXPORT int dl_norm_add_norm(int out_dtype, int delta_dtype, float* x, const void* delta, int parts, long long part_stride,
                               const float* w_post, float eps_post, const float* w_pre, float eps_pre, void* out, int rows,
                               int width, cudaStream_t stream) {
  if (rows <= 0 || width <= 0) return 0;
  if (parts < 1 || width > 12000 || (out_dtype != 0 && out_dtype != 1) || (delta_dtype != 0 && delta_dtype != 1))
    return DL_ERR_UNSUPPORTED;
  const size_t smem = static_cast<size_t>(width) * sizeof(float);
#define DL_NAN(TD, TO)                                                                                                 \
  dl::norm_add_norm_kernel<TD, TO><<<rows, 256, smem, stream>>>(x, static_cast<const TD*>(delta), parts,               \
                                                                static_cast<size_t>(part_stride), w_post, eps_post,    \
                                                                w_pre, eps_pre, static_cast<TO*>(out), width)
  if (delta_dtype == 0 && out_dtype == 0) DL_NAN(float, float);
  else if (delta_dtype == 0) DL_NAN(float, dl::bf16);
  else if (out_dtype == 0) DL_NAN(dl::bf16, float);
  else DL_NAN(dl::bf16, dl::bf16);
#undef DL_NAN
  return dl::launch_status();
}
