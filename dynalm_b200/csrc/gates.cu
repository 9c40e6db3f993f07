// Small element-wise kernels around gates, sums and caps. All arithmetic is float32 whatever the storage type.
//
//   dl_gelu_mul       out[t, j] = gelu_tanh(gu[t, j]) * gu[t, inner + j]      (a gated feed-forward's activation)
//   dl_sigmoid_gate   x[t, j] <- x[t, j] * sigmoid(gate[t, j])                (an output gate on concatenated heads)
//   dl_scaled_sum     out[i] = sa * sum_p a[p][i] + sb * sum_p b[p][i]        (two mixers side by side; float32 out)
//   dl_softcap        x[i] <- cap * tanh(x[i] / cap)                          (float32 logits)
#include "common.cuh"

namespace dl {

__device__ __forceinline__ float gelu_tanh_full(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void gelu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int rows, int inner) {
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<size_t>(rows) * inner) return;
  const size_t t = idx / inner, j = idx % inner;
  const T* row = gu + t * 2 * inner;
  out[idx] = from_float<T>(gelu_tanh_full(to_float(row[j])) * to_float(row[inner + j]));
}

// 16 bytes per access: inner a multiple of the vector width.
template <typename T>
__global__ void gelu_mul_vec_kernel(const T* __restrict__ gu, T* __restrict__ out, int rows, int inner) {
  constexpr int V = PerVec<T>::n;
  const int per_row = inner / V;
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<size_t>(rows) * per_row) return;
  const size_t t = idx / per_row, j = idx % per_row;
  const Vec16* row = reinterpret_cast<const Vec16*>(gu + t * 2 * inner);
  float g[V], u[V];
  unpack<T>(row[j], g);
  unpack<T>(row[per_row + j], u);
#pragma unroll
  for (int k = 0; k < V; ++k) g[k] = gelu_tanh_full(g[k]) * u[k];
  reinterpret_cast<Vec16*>(out)[idx] = pack<T>(g);
}

template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ x, int x_stride, const T* __restrict__ gate, int gate_stride, int rows,
                                    int n) {
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<size_t>(rows) * n) return;
  const size_t t = idx / n, j = idx % n;
  const float g = to_float(gate[t * gate_stride + j]);
  T* p = x + t * x_stride + j;
  *p = from_float<T>(to_float(*p) / (1.0f + expf(-g)));
}

template <typename TA, typename TB>
__global__ void scaled_sum_kernel(const TA* __restrict__ a, int parts_a, size_t stride_a, float sa, const TB* __restrict__ b,
                                  int parts_b, size_t stride_b, float sb, float* __restrict__ out, size_t n) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float va = 0.0f, vb = 0.0f;
  for (int p = 0; p < parts_a; ++p) va += to_float(a[p * stride_a + i]);
  for (int p = 0; p < parts_b; ++p) vb += to_float(b[p * stride_b + i]);
  out[i] = sa * va + sb * vb;
}

__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap, float inv_cap) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) x[i] = cap * tanhf(x[i] * inv_cap);
}

inline unsigned blocks_for(size_t n) { return static_cast<unsigned>((n + 255) / 256); }

}  // namespace dl

// gu: contiguous [rows, 2 * inner] = [gate | up]; out: contiguous [rows, inner].
DL_EXPORT int dl_gelu_mul(int dtype, const void* gu, void* out, int rows, int inner, cudaStream_t stream) {
  if (rows <= 0 || inner <= 0) return 0;
  if (dtype != 0 && dtype != 1) return DL_ERR_UNSUPPORTED;
  const int vec = dtype == 0 ? 4 : 8;
  if (inner % vec == 0 && (reinterpret_cast<uintptr_t>(gu) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    const size_t n = static_cast<size_t>(rows) * (inner / vec);
    if (dtype == 0) dl::gelu_mul_vec_kernel<float><<<dl::blocks_for(n), 256, 0, stream>>>(static_cast<const float*>(gu), static_cast<float*>(out), rows, inner);
    else dl::gelu_mul_vec_kernel<dl::bf16><<<dl::blocks_for(n), 256, 0, stream>>>(static_cast<const dl::bf16*>(gu), static_cast<dl::bf16*>(out), rows, inner);
    return dl::launch_status();
  }
  const size_t n = static_cast<size_t>(rows) * inner;
  if (dtype == 0) dl::gelu_mul_kernel<float><<<dl::blocks_for(n), 256, 0, stream>>>(static_cast<const float*>(gu), static_cast<float*>(out), rows, inner);
  else dl::gelu_mul_kernel<dl::bf16><<<dl::blocks_for(n), 256, 0, stream>>>(static_cast<const dl::bf16*>(gu), static_cast<dl::bf16*>(out), rows, inner);
  return dl::launch_status();
}

// x: rows of x_stride elements, the first n of each are gated in place; gate: rows of gate_stride elements.
DL_EXPORT int dl_sigmoid_gate(int dtype, void* x, int x_stride, const void* gate, int gate_stride, int rows, int n,
                              cudaStream_t stream) {
  if (rows <= 0 || n <= 0) return 0;
  const size_t total = static_cast<size_t>(rows) * n;
  if (dtype == 0) dl::sigmoid_gate_kernel<float><<<dl::blocks_for(total), 256, 0, stream>>>(static_cast<float*>(x), x_stride, static_cast<const float*>(gate), gate_stride, rows, n);
  else if (dtype == 1) dl::sigmoid_gate_kernel<dl::bf16><<<dl::blocks_for(total), 256, 0, stream>>>(static_cast<dl::bf16*>(x), x_stride, static_cast<const dl::bf16*>(gate), gate_stride, rows, n);
  else return DL_ERR_UNSUPPORTED;
  return dl::launch_status();
}

// a, b: [parts, n] with `stride` elements between parts (parts 1: [n]), each float32 (0) or bfloat16 (1).
DL_EXPORT int dl_scaled_sum(int dtype_a, const void* a, int parts_a, long long stride_a, float sa, int dtype_b, const void* b,
                            int parts_b, long long stride_b, float sb, float* out, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((dtype_a != 0 && dtype_a != 1) || (dtype_b != 0 && dtype_b != 1) || parts_a < 1 || parts_b < 1) return DL_ERR_UNSUPPORTED;
#define DL_SS(TA, TB)                                                                                                   \
  dl::scaled_sum_kernel<TA, TB><<<dl::blocks_for(static_cast<size_t>(n)), 256, 0, stream>>>(                            \
      static_cast<const TA*>(a), parts_a, static_cast<size_t>(stride_a), sa, static_cast<const TB*>(b), parts_b,       \
      static_cast<size_t>(stride_b), sb, out, static_cast<size_t>(n))
  if (dtype_a == 0 && dtype_b == 0) DL_SS(float, float);
  else if (dtype_a == 0) DL_SS(float, dl::bf16);
  else if (dtype_b == 0) DL_SS(dl::bf16, float);
  else DL_SS(dl::bf16, dl::bf16);
#undef DL_SS
  return dl::launch_status();
}

DL_EXPORT int dl_softcap(float* x, long long n, float cap, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (!(cap > 0.0f)) return DL_ERR_UNSUPPORTED;
  dl::softcap_kernel<<<dl::blocks_for(static_cast<size_t>(n)), 256, 0, stream>>>(x, static_cast<size_t>(n), cap, 1.0f / cap);
  return dl::launch_status();
}

// x[r, c] += bias[c] over rows of ld elements (the bias of a projection whose product ran without one).
namespace dl {
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ x, long long ld, const float* __restrict__ bias, int n, size_t total) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t r = i / n;
  const int c = static_cast<int>(i % n);
  T* p = x + r * ld + c;
  *p = from_float<T>(to_float(*p) + bias[c]);
}
}  // namespace dl

DL_EXPORT int dl_add_bias(int dtype, void* x, long long ld, const float* bias, int rows, int n, cudaStream_t stream) {
  if (rows <= 0 || n <= 0) return 0;
  const size_t total = static_cast<size_t>(rows) * n;
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
  if (dtype == 0) dl::add_bias_kernel<float><<<blocks, 256, 0, stream>>>(static_cast<float*>(x), ld, bias, n, total);
  else if (dtype == 1) dl::add_bias_kernel<dl::bf16><<<blocks, 256, 0, stream>>>(static_cast<dl::bf16*>(x), ld, bias, n, total);
  else return DL_ERR_UNSUPPORTED;
  return dl::launch_status();
}
