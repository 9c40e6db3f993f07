// Queries and keys normed over their whole projection, turned by position, keys and values written into the cache.
//
// A row of the projection holds [q: H * d | k: G * d | v: G * e | ...]. Per row, in float32:
//
//   q <- q / sqrt(mean over all H * d numbers of q^2 + eps) * wq        (one statistic for the whole projection,
//   k <- k / sqrt(mean over all G * d numbers of k^2 + eps) * wk         not one per head; either weight may be absent)
//   the first `rot` numbers of every head of q and k: number i pairs with number i + rot / 2 and the pair (u, v) turns
//   to (u cos a - v sin a, v cos a + u sin a), a = position * pos_scale * inv_freq[i]
//
// q is written back in place; k and v go to the token's place in the request's pages. The two arrays of the cache may
// be one (a record [k | v] per token) or two: each is given by its base and the elements between two tokens.
#include "common.cuh"

namespace dl {

template <typename T>
__global__ void __launch_bounds__(256)
qk_proj_norm_kernel(T* __restrict__ proj, int stride, const float* __restrict__ wq, const float* __restrict__ wk, float eps,
                    int do_norm, const float* __restrict__ inv_freq, int rot, float pos_scale,
                    const int* __restrict__ positions, const int* __restrict__ row_slot,
                    const int* __restrict__ block_table, int max_blocks, T* __restrict__ k_cache, size_t k_row,
                    T* __restrict__ v_cache, size_t v_row, int H, int G, int d, int e, int page_size) {
  __shared__ float red[33];
  const int row = blockIdx.x, tid = threadIdx.x;
  T* q = proj + static_cast<size_t>(row) * stride;
  T* k = q + H * d;
  const T* v = k + G * d;
  const int nq = H * d, nk = G * d, nv = G * e;
  float rq = 1.0f, rk = 1.0f;
  if (do_norm) {
    float sq = 0.0f, sk = 0.0f;
    for (int i = tid; i < nq; i += blockDim.x) { const float x = to_float(q[i]); sq = fmaf(x, x, sq); }
    for (int i = tid; i < nk; i += blockDim.x) { const float x = to_float(k[i]); sk = fmaf(x, x, sk); }
    rq = 1.0f / sqrtf(block_sum(sq, red) / static_cast<float>(nq) + eps);
    rk = 1.0f / sqrtf(block_sum(sk, red) / static_cast<float>(nk) + eps);
  }
  const int pos = positions[row];
  const int* table = block_table + static_cast<size_t>(ck_request(row_slot[row])) * max_blocks;
  const int page = ck_page_store(table, pos / page_size, max_blocks);
  const size_t slot = static_cast<size_t>(page < 0 ? 0 : page) * page_size + pos % page_size;
  const int half = rot / 2;
  const float fpos = static_cast<float>(pos) * pos_scale;
  // queries and keys together: index n < nq is a query number, the rest are key numbers
  for (int n = tid; n < nq + nk; n += blockDim.x) {
    const bool is_q = n < nq;
    const int idx = is_q ? n : n - nq;
    const int i = idx % d;
    if (i >= half && i < rot) continue;                      // the second number of a pair: its first number's thread writes it
    T* src = is_q ? q : k;
    const float* w = is_q ? wq : wk;
    const float r = is_q ? rq : rk;
    float a = to_float(src[idx]) * r * (w ? w[idx] : 1.0f);
    float b = 0.0f;
    const bool pair = i < half;
    if (pair) {
      b = to_float(src[idx + half]) * r * (w ? w[idx + half] : 1.0f);
      float s, c;
      sincosf(fpos * inv_freq[i], &s, &c);
      const float a2 = a * c - b * s, b2 = b * c + a * s;
      a = a2;
      b = b2;
    }
    if (is_q) {
      q[idx] = from_float<T>(a);
      if (pair) q[idx + half] = from_float<T>(b);
    } else if (page >= 0) {
      T* dst = k_cache + slot * k_row;
      dst[idx] = from_float<T>(a);
      if (pair) dst[idx + half] = from_float<T>(b);
    }
  }
  if (page >= 0) {
    T* dst = v_cache + slot * v_row;
    for (int i = tid; i < nv; i += blockDim.x) dst[i] = v[i];
  }
}


// The other order: turn first, then make every head of q and k a unit-RMS vector by itself (no weight), or leave it
// as it is. One warp per unit, a unit being a query head, a key head or the values of a KV head. The pairs of the
// rotation are (i, i + rot / 2) or, interleaved, (2i, 2i + 1); a pair (u, v) turns to (u cos a - v sin a, v cos a + u
// sin a), a = position * inv_freq[i], in float32. A bias of the projection (q | k | v) may be added on the way in.
template <typename T>
__global__ void __launch_bounds__(256)
qk_rot_head_norm_kernel(T* __restrict__ proj, int stride, const float* __restrict__ bias, const float* __restrict__ inv_freq, int rot, int interleaved,
                        int unit_norm, float eps, const int* __restrict__ positions, const int* __restrict__ row_slot,
                        const int* __restrict__ block_table, int max_blocks, T* __restrict__ k_cache, size_t k_row,
                        T* __restrict__ v_cache, size_t v_row, int rows, int H, int G, int d, int e, int page_size) {
  constexpr int PER = 8;                                   // numbers a lane holds: heads of up to 256
  const int units = H + 2 * G;
  const long long unit = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (unit >= static_cast<long long>(rows) * units) return;
  const int row = static_cast<int>(unit / units), u = static_cast<int>(unit % units);
  const int pos = positions[row];
  const int* table = block_table + static_cast<size_t>(ck_request(row_slot[row])) * max_blocks;
  T* base = proj + static_cast<size_t>(row) * stride;
  size_t slot = 0;
  int page = 0;
  if (u >= H) {
    page = ck_page_store(table, pos / page_size, max_blocks);
    slot = static_cast<size_t>(page < 0 ? 0 : page) * page_size + pos % page_size;
  }
  if (u >= H + G) {                                         // values: a copy into the token's place
    if (page < 0) return;
    const int off = H * d + G * d + (u - H - G) * e;
    const T* v = base + off;
    T* dst = v_cache + slot * v_row + static_cast<size_t>(u - H - G) * e;
    if (bias != nullptr) {
      for (int i = lane; i < e; i += 32) dst[i] = from_float<T>(to_float(v[i]) + bias[off + i]);
    } else {
      for (int i = lane; i < e; i += 32) dst[i] = v[i];
    }
    return;
  }
  const int src_off = u < H ? u * d : H * d + (u - H) * d;
  T* src = base + src_off;
  const float* bsrc = bias != nullptr ? bias + src_off : nullptr;
  const int half = rot / 2;
  float x[PER], xp[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int i = lane + 32 * j;
    x[j] = i < d ? to_float(src[i]) + (bsrc != nullptr ? bsrc[i] : 0.0f) : 0.0f;
    xp[j] = 0.0f;
    if (i < rot) {
      const int partner = interleaved ? (i ^ 1) : (i < half ? i + half : i - half);
      xp[j] = to_float(src[partner]) + (bsrc != nullptr ? bsrc[partner] : 0.0f);
    }
  }
  __syncwarp();                                             // every lane has read before any lane writes in place
  const float fpos = static_cast<float>(pos);
  float ss = 0.0f;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int i = lane + 32 * j;
    if (i < rot) {
      const bool first = interleaved ? !(i & 1) : i < half;
      const int f = interleaved ? (i >> 1) : (first ? i : i - half);
      float sn, cs;
      sincosf(fpos * inv_freq[f], &sn, &cs);
      x[j] = first ? x[j] * cs - xp[j] * sn : x[j] * cs + xp[j] * sn;
    }
    ss = fmaf(x[j], x[j], ss);
  }
  float r = 1.0f;
  if (unit_norm) r = 1.0f / sqrtf(warp_sum(ss) / static_cast<float>(d) + eps);
  T* dst = src;
  if (u >= H) {
    if (page < 0) return;
    dst = k_cache + slot * k_row + static_cast<size_t>(u - H) * d;
  }
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int i = lane + 32 * j;
    if (i < d) dst[i] = from_float<T>(x[j] * r);
  }
}

}  // namespace dl

DL_EXPORT int dl_qk_proj_norm_cache(int dtype, void* proj, int stride, const float* wq, const float* wk, float eps, int do_norm,
                                    const float* inv_freq, int rot, float pos_scale, const int* positions,
                                    const int* row_slot, const int* block_table, int max_blocks, void* k_cache,
                                    long long k_row, void* v_cache, long long v_row, int rows, int H, int G, int d, int e,
                                    int page_size, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H <= 0 || G <= 0 || d <= 0 || e <= 0 || rot < 0 || rot > d || (rot & 1) || page_size <= 0 || (rot > 0 && inv_freq == nullptr))
    return DL_ERR_UNSUPPORTED;
#define DL_QK(T)                                                                                                          \
  dl::qk_proj_norm_kernel<T><<<rows, 256, 0, stream>>>(static_cast<T*>(proj), stride, wq, wk, eps, do_norm, inv_freq, rot, \
                                                       pos_scale, positions, row_slot, block_table, max_blocks,          \
                                                       static_cast<T*>(k_cache), static_cast<size_t>(k_row),              \
                                                       static_cast<T*>(v_cache), static_cast<size_t>(v_row), H, G, d, e,  \
                                                       page_size)
  if (dtype == 0) DL_QK(float);
  else if (dtype == 1) DL_QK(dl::bf16);
  else return DL_ERR_UNSUPPORTED;
#undef DL_QK
  return dl::launch_status();
}

// Rows [q: H*d | k: G*d | v: G*e | ...]: rotation first (rot numbers of every head, pairs by halves or interleaved),
// then every head of q and k divided by its own root mean square (unit_norm) or left; q in place, k and v into the
// pages. bias: float32 [H*d + G*d + G*e] added to q | k | v first, or null. d at most 256.
DL_EXPORT int dl_qk_rot_head_norm_cache(int dtype, void* proj, int stride, const float* bias, const float* inv_freq, int rot, int interleaved,
                                        int unit_norm, float eps, const int* positions, const int* row_slot,
                                        const int* block_table, int max_blocks, void* k_cache, long long k_row,
                                        void* v_cache, long long v_row, int rows, int H, int G, int d, int e, int page_size,
                                        cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H <= 0 || G <= 0 || d <= 0 || d > 256 || e <= 0 || rot < 0 || rot > d || (rot & 1) || page_size <= 0 ||
      (rot > 0 && inv_freq == nullptr))
    return DL_ERR_UNSUPPORTED;
  const long long units = static_cast<long long>(rows) * (H + 2 * G);
  const unsigned blocks = static_cast<unsigned>((units + 7) / 8);
#define DL_QK(T)                                                                                                          \
  dl::qk_rot_head_norm_kernel<T><<<blocks, 256, 0, stream>>>(static_cast<T*>(proj), stride, bias, inv_freq, rot, interleaved, \
                                                             unit_norm, eps, positions, row_slot, block_table, max_blocks, \
                                                             static_cast<T*>(k_cache), static_cast<size_t>(k_row),         \
                                                             static_cast<T*>(v_cache), static_cast<size_t>(v_row), rows, H, \
                                                             G, d, e, page_size)
  if (dtype == 0) DL_QK(float);
  else if (dtype == 1) DL_QK(dl::bf16);
  else return DL_ERR_UNSUPPORTED;
#undef DL_QK
  return dl::launch_status();
}
