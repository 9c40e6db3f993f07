// Paged flash attention with keys and values of two sizes, kept first tokens behind the window and an optional extra
// term in the softmax's denominator: bf16 tensor cores (mma.sync m16n8k16), fp32 softmax.
//
// The kernel of attention_prefill.cu made more general, for mixers whose mask or softmax the kernels of the plain
// attention do not know. One thread block per (query tile, head); a query tile is up to 128 consecutive rows of ONE
// request, a single decoded token a tile of one row, so prompt portions and decode rows share a launch. Differences:
//
//   * keys have KD numbers and values VD (both multiples of 16, at most 128); a token's keys lie k_row elements from
//     the next token's and its values v_row, so the cache may be two arrays or one array of records [k | v];
//   * a row at position p sees key j <= p if p - j < window (window 0: all) or j < keep_first: the key tiles that hold
//     kept tokens are walked first, then the tiles of the window;
//   * with `sink` the denominator of a row's softmax holds one more term exp(0), which carries no value;
//   * warps whose 16 rows lie past the end of the tile (a one-row tile leaves three of four) skip the arithmetic;
//   * in a step whose tiles are all single tokens the rows of a tile are the query heads that share a KV head, so the
//     keys and values of a token are read once for the group.
//
// Key tiles begin at multiples of 64 in absolute position, so the arithmetic of a row does not depend on where its
// portion was cut nor on its place inside a query tile.
#include "common.cuh"

namespace dl {

constexpr int MF_TILE = 128;    // rows of a query tile as the host cuts them
constexpr int MF_BN = 64;       // keys per tile
constexpr int MF_BM = 64;       // query rows per block (4 warps of 16)
constexpr int MF_THREADS = 128;

__device__ __forceinline__ void mf_cp_async16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const int bytes = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void mf_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void mf_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void mf_ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mf_ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mf_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float mf_exp2(float x) {      // 2^x by the special-function unit; 2^-inf = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t mf_pack(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}

// tiles[i] = (request, first row of the step, rows, first position)
template <int KD, int VD>
__global__ void __launch_bounds__(MF_THREADS)
masked_flash_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ k_cache, size_t k_row,
                    const bf16* __restrict__ v_cache, size_t v_row, const int* __restrict__ block_table, int max_blocks,
                    const int4* __restrict__ tiles, bf16* __restrict__ out, int out_stride, int n_heads, int n_kv_heads,
                    int page_shift, float scale_log2, int window, int keep_first, int sink, int grp, float* __restrict__ partial) {
  constexpr int SUB = MF_TILE / MF_BM;    // blocks per query tile
  constexpr int LDK = KD + 8;             // row strides in elements: 16 bytes of padding keep ldmatrix conflict-free
  constexpr int LDV = VD + 8;
  constexpr int CHK = KD / 8, CHV = VD / 8;      // 16-byte chunks per row
  constexpr int KS = KD / 16;             // k-steps of the Q K^T product
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);
  bf16* Ks = Qs + MF_BM * LDK;            // [2][MF_BN][LDK]
  bf16* Vs = Ks + 2 * MF_BN * LDK;        // [2][MF_BN][LDV]

  const int4 tile = ck_tile(tiles[blockIdx.x / SUB]);
  const int sub = blockIdx.x % SUB;
  const int req = tile.x, row0 = tile.y + sub * MF_BM, pos0 = tile.w + sub * MF_BM;
  int nrows = min(MF_BM, tile.z - sub * MF_BM);
  if (nrows <= 0) return;
  // grp > 0 (every tile one token): the block takes KV head blockIdx.y, and the rows of its tile are the grp query heads
  // of that KV head, all at the token's position, so the keys and values are read once for the group
  const int head = grp > 0 ? static_cast<int>(blockIdx.y) * grp : static_cast<int>(blockIdx.y);      // (the first head of the group)
  const int kvh = grp > 0 ? static_cast<int>(blockIdx.y) : head / (n_heads / n_kv_heads);
  if (grp > 0) nrows = grp;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int page_mask = (1 << page_shift) - 1;
  const int* table = block_table + static_cast<size_t>(req) * max_blocks;
  const bool warp_live = warp * 16 < nrows;

  const int pos_last = grp > 0 ? pos0 : pos0 + nrows - 1;
  const int lo_tile = window > 0 ? max(0, pos0 - window + 1) : 0;     // the first key of the window any row of the tile reads
  const int j_begin = lo_tile / MF_BN, j_end = pos_last / MF_BN;
  // key tiles in front of the window's that hold kept tokens: 0 .. n_kept - 1
  const int kept = lo_tile > 0 ? min(keep_first, lo_tile) : 0;
  const int n_kept = kept > 0 ? min((kept - 1) / MF_BN + 1, j_begin) : 0;
  const int n_iter = n_kept + (j_end - j_begin + 1);
  auto tile_of = [&](int it) { return it < n_kept ? it : j_begin + (it - n_kept); };
  // gridDim.z > 1 (single-token tiles of a step with few rows): the key tiles of a row are dealt over that many blocks,
  // each leaving its maximum, sum and unnormalised output in `partial` for masked_flash_merge_kernel
  const int n_parts = static_cast<int>(gridDim.z), part = static_cast<int>(blockIdx.z);
  const int per_part = (n_iter + n_parts - 1) / n_parts;
  const int it_begin = min(part * per_part, n_iter), it_end = min(it_begin + per_part, n_iter);

  for (int c = tid; c < MF_BM * CHK; c += MF_THREADS) {
    const int r = c / CHK, ch = c % CHK;
    const bool ok = r < nrows;
    const bf16* src = grp > 0 ? q + static_cast<size_t>(row0) * q_stride + static_cast<size_t>(head + (ok ? r : 0)) * KD + ch * 8
                              : q + static_cast<size_t>(row0 + (ok ? r : 0)) * q_stride + static_cast<size_t>(head) * KD + ch * 8;
    mf_cp_async16(Qs + r * LDK + ch * 8, src, ok);
  }
  auto load_kv = [&](int j, int stage) {
    bf16* ks = Ks + stage * MF_BN * LDK;
    bf16* vs = Vs + stage * MF_BN * LDV;
    for (int c = tid; c < MF_BN * (CHK + CHV); c += MF_THREADS) {
      const int r = c / (CHK + CHV), ch = c % (CHK + CHV);
      const int key = j * MF_BN + r;
      const bool ok = (key >= lo_tile || key < kept) && key <= pos_last;
      size_t slot = 0;
      if (ok) slot = (static_cast<size_t>(ck_page(table, key >> page_shift, max_blocks)) << page_shift) + (key & page_mask);
      if (ch < CHK) mf_cp_async16(ks + r * LDK + ch * 8, k_cache + slot * k_row + static_cast<size_t>(kvh) * KD + ch * 8, ok);
      else mf_cp_async16(vs + r * LDV + (ch - CHK) * 8, v_cache + slot * v_row + static_cast<size_t>(kvh) * VD + (ch - CHK) * 8, ok);
    }
  };
  if (it_begin < it_end) load_kv(tile_of(it_begin), 0);
  mf_commit();

  float o[VD / 8][4];
#pragma unroll
  for (int i = 0; i < VD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
  float m_run[2], l_run[2];
  int pos_r[2], lo_r[2];                  // position and first key of the window of the lane's rows
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    m_run[h] = -INFINITY;
    l_run[h] = 0.0f;
    pos_r[h] = grp > 0 ? pos0 : pos0 + warp * 16 + g + h * 8;
    lo_r[h] = window > 0 ? max(0, pos_r[h] - window + 1) : 0;
  }
  uint32_t qf[KS][4];

  for (int it = it_begin; it < it_end; ++it) {
    const int j = tile_of(it);
    const int stage = (it - it_begin) & 1;
    if (it + 1 < it_end) load_kv(tile_of(it + 1), stage ^ 1);
    mf_commit();
    mf_wait<1>();
    __syncthreads();
    if (warp_live) {
      if (it == it_begin) {
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          const int c = ks * 16 + (lane >> 4) * 8;
          mf_ldmatrix_x4(qf[ks], Qs + r * LDK + c);
        }
      }
      const bf16* kt = Ks + stage * MF_BN * LDK;
      const bf16* vt = Vs + stage * MF_BN * LDV;

      float s[MF_BN / 8][4];
#pragma unroll
      for (int i = 0; i < MF_BN / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f; }
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
        for (int np = 0; np < MF_BN / 16; ++np) {       // two key tiles of 8 per ldmatrix.x4
          uint32_t kb[4];
          const int key = np * 16 + (lane & 7) + (lane >> 4) * 8;
          const int c = ks * 16 + ((lane >> 3) & 1) * 8;
          mf_ldmatrix_x4(kb, kt + key * LDK + c);
          mf_mma(s[2 * np], qf[ks], kb[0], kb[1]);
          mf_mma(s[2 * np + 1], qf[ks], kb[2], kb[3]);
        }
      }
      // scale, mask by position, online softmax; P as bf16 A fragments
      const int key0 = j * MF_BN;
      uint32_t pf[MF_BN / 16][4];
      const bool edge = it < n_kept || key0 + MF_BN - 1 > (grp > 0 ? pos0 : pos0 + warp * 16) ||
                        (window > 0 && key0 < max(lo_r[0], lo_r[1]));
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < MF_BN / 8; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = s[i][e];
          if (edge) {
            const int key = key0 + i * 8 + 2 * t + (e & 1);
            if (key > pos_r[e >> 1] || (key < lo_r[e >> 1] && key >= keep_first)) v = -INFINITY;
            s[i][e] = v;
          }
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      }
      float corr[2], neg_m[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(m_run[h], mx[h] * scale_log2);     // the scale is positive
        corr[h] = m_new == -INFINITY ? 1.0f : mf_exp2(m_run[h] - m_new);
        m_run[h] = m_new;
        neg_m[h] = m_new == -INFINITY ? 0.0f : -m_new;
      }
      float ls[2] = {0.0f, 0.0f};
#pragma unroll
      for (int i = 0; i < MF_BN / 8; ++i) {
        const float p0 = mf_exp2(fmaf(s[i][0], scale_log2, neg_m[0])), p1 = mf_exp2(fmaf(s[i][1], scale_log2, neg_m[0]));
        const float p2 = mf_exp2(fmaf(s[i][2], scale_log2, neg_m[1])), p3 = mf_exp2(fmaf(s[i][3], scale_log2, neg_m[1]));
        ls[0] += p0 + p1;
        ls[1] += p2 + p3;
        pf[i >> 1][(i & 1) * 2] = mf_pack(p0, p1);
        pf[i >> 1][(i & 1) * 2 + 1] = mf_pack(p2, p3);
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        ls[h] += __shfl_xor_sync(0xffffffffu, ls[h], 1);
        ls[h] += __shfl_xor_sync(0xffffffffu, ls[h], 2);
        l_run[h] = l_run[h] * corr[h] + ls[h];
      }
      if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
        for (int i = 0; i < VD / 8; ++i) {
          o[i][0] *= corr[0]; o[i][1] *= corr[0];
          o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
      }
      // O += P V
#pragma unroll
      for (int kk = 0; kk < MF_BN / 16; ++kk) {
#pragma unroll
        for (int dp = 0; dp < VD / 16; ++dp) {           // two 8-wide slices of the value per ldmatrix.x4
          uint32_t vb[4];
          const int key = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          const int c = dp * 16 + (lane >> 4) * 8;
          mf_ldmatrix_x4_trans(vb, vt + key * LDV + c);
          mf_mma(o[2 * dp], pf[kk], vb[0], vb[1]);
          mf_mma(o[2 * dp + 1], pf[kk], vb[2], vb[3]);
        }
      }
    }
    __syncthreads();     // every warp is done with this stage before the next prefetch overwrites it
  }
  mf_wait<0>();
  if (!warp_live) return;

  const int r_a = warp * 16 + g, r_b = r_a + 8;
  if (partial != nullptr) {
    // records [row][head][part] of (maximum in base-2 units, sum, VD unnormalised outputs); a tile here is one token
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = h == 0 ? r_a : r_b;
      if (r >= nrows) continue;
      const int head_abs = grp > 0 ? head + r : head;
      float* rec = partial + ((static_cast<size_t>(row0) * n_heads + head_abs) * n_parts + part) * (VD + 2);
      if (t == 0) {
        rec[0] = m_run[h];
        rec[1] = l_run[h];
      }
#pragma unroll
      for (int i = 0; i < VD / 8; ++i) {
        rec[2 + i * 8 + 2 * t] = o[i][2 * h];
        rec[2 + i * 8 + 2 * t + 1] = o[i][2 * h + 1];
      }
    }
    return;
  }
  float inv[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float l = l_run[h], c = 1.0f;
    if (sink && m_run[h] != -INFINITY) {                 // one more term 2^0 in the denominator (m is in base-2 units)
      const float m_fin = fmaxf(m_run[h], 0.0f);
      c = mf_exp2(m_run[h] - m_fin);
      l = l * c + mf_exp2(-m_fin);
    }
    inv[h] = l > 0.0f ? c / l : 0.0f;
  }
#pragma unroll
  for (int i = 0; i < VD / 8; ++i) {
    const int col = head * VD + i * 8 + 2 * t;
    // row r of a tile is row row0 + r of the step, or (grp > 0) head `head + r` of row row0
    bf16* dst_a = grp > 0 ? out + static_cast<size_t>(row0) * out_stride + col + r_a * VD : out + static_cast<size_t>(row0 + r_a) * out_stride + col;
    bf16* dst_b = grp > 0 ? out + static_cast<size_t>(row0) * out_stride + col + r_b * VD : out + static_cast<size_t>(row0 + r_b) * out_stride + col;
    if (r_a < nrows) *reinterpret_cast<uint32_t*>(dst_a) = mf_pack(o[i][0] * inv[0], o[i][1] * inv[0]);
    if (r_b < nrows) *reinterpret_cast<uint32_t*>(dst_b) = mf_pack(o[i][2] * inv[1], o[i][3] * inv[1]);
  }
}

// out[row][head] = sum_p o_p 2^(m_p - M) / (sum_p l_p 2^(m_p - M) + [sink] 2^(-M)), M = max_p m_p (and 0 with the sink):
// the parts of a row and head that masked_flash_kernel left, in the order of the parts.
__global__ void masked_flash_merge_kernel(const float* __restrict__ partial, int n_parts, int VD, int n_heads, int sink,
                                          bf16* __restrict__ out, int out_stride) {
  const int row = blockIdx.x, head = blockIdx.y;
  const float* rec = partial + (static_cast<size_t>(row) * n_heads + head) * n_parts * (VD + 2);
  float M = sink ? 0.0f : -INFINITY;
  for (int p = 0; p < n_parts; ++p) M = fmaxf(M, rec[p * (VD + 2)]);
  float l = sink ? mf_exp2(-M) : 0.0f;
  for (int p = 0; p < n_parts; ++p) {
    const float m = rec[p * (VD + 2)];
    if (m != -INFINITY) l += rec[p * (VD + 2) + 1] * mf_exp2(m - M);
  }
  const float inv = l > 0.0f ? 1.0f / l : 0.0f;
  for (int v = threadIdx.x; v < VD; v += blockDim.x) {
    float acc = 0.0f;
    for (int p = 0; p < n_parts; ++p) {
      const float m = rec[p * (VD + 2)];
      if (m != -INFINITY) acc = fmaf(rec[p * (VD + 2) + 2 + v], mf_exp2(m - M), acc);
    }
    out[static_cast<size_t>(row) * out_stride + head * VD + v] = __float2bfloat16_rn(acc * inv);
  }
}

template <int KD, int VD>
int launch_masked_flash(const void* q, int q_stride, const void* kc, long long k_row, const void* vc, long long v_row,
                        const int* block_table, int max_blocks, const int* tiles, int n_tiles, void* out, int out_stride,
                        int n_heads, int n_kv_heads, int page_shift, float scale, int window, int keep_first, int sink,
                        int grp, int parts, float* partial, int rows, cudaStream_t stream) {
  constexpr size_t smem = (static_cast<size_t>(MF_BM + 2 * MF_BN) * (KD + 8) + static_cast<size_t>(2 * MF_BN) * (VD + 8)) * sizeof(bf16);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(masked_flash_kernel<KD, VD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  dim3 grid(n_tiles * (MF_TILE / MF_BM), grp > 0 ? n_kv_heads : n_heads, parts > 1 ? parts : 1);
  masked_flash_kernel<KD, VD><<<grid, MF_THREADS, smem, stream>>>(
      static_cast<const bf16*>(q), q_stride, static_cast<const bf16*>(kc), static_cast<size_t>(k_row),
      static_cast<const bf16*>(vc), static_cast<size_t>(v_row), block_table, max_blocks, reinterpret_cast<const int4*>(tiles),
      static_cast<bf16*>(out), out_stride, n_heads, n_kv_heads, page_shift, scale * 1.4426950408889634f, window, keep_first,
      sink, grp, parts > 1 ? partial : nullptr);
  if (parts > 1) {
    dim3 mgrid(rows, n_heads);
    masked_flash_merge_kernel<<<mgrid, VD < 64 ? 32 : 64, 0, stream>>>(partial, parts, VD, n_heads, sink, static_cast<bf16*>(out),
                                                                      out_stride);
  }
  return launch_status();
}

}  // namespace dl

// bfloat16 only. tiles: int32 [n_tiles, 4] = (request, first row, rows <= 128, first position), 16-byte aligned.
// q rows have head h at column h * key_dim, out rows at column h * value_dim. k_cache / v_cache point at the first
// token's keys / values (KV head j at j * key_dim / j * value_dim); k_row / v_row elements lie between two tokens.
// one_token_tiles: every tile is a single token, tile i being row i of the step; parts > 1 then deals a row's key tiles
// over that many blocks and merges them (partial: scratch). Sizes it takes: key_dim == value_dim in steps of 16 up to 128, and the pairs listed below; others are refused.
DL_EXPORT int dl_masked_flash_attention(const void* q, int q_stride, const void* k_cache, long long k_row, const void* v_cache,
                                        long long v_row, const int* block_table, int max_blocks, const int* tiles, int n_tiles,
                                        void* out, int out_stride, int n_heads, int n_kv_heads, int key_dim, int value_dim,
                                        int page_size, float scale, int window, int keep_first, int sink, int one_token_tiles,
                                        int parts, float* partial, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  if ((1 << page_shift) != page_size || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || n_heads > 65535 || (q_stride & 7) ||
      (out_stride & 1) || !(scale > 0.0f) || (k_row & 7) || (v_row & 7) || window < 0 || keep_first < 0 ||
      (reinterpret_cast<uintptr_t>(k_cache) & 15) || (reinterpret_cast<uintptr_t>(v_cache) & 15))
    return DL_ERR_UNSUPPORTED;
  // every tile one token (the caller says so) and heads that share keys: the heads of a KV head are the rows of a tile
  const int group = n_heads / n_kv_heads;
  const int grp = (one_token_tiles && group > 1 && group <= dl::MF_BM) ? group : 0;
  // parts > 1: every tile is one token, tile i is row i of the step, and `partial` holds n_tiles * n_heads * parts *
  // (value_dim + 2) floats
  if (parts > 1 && (!one_token_tiles || partial == nullptr || parts > 64)) return DL_ERR_UNSUPPORTED;
#define DL_CASE(K, V)                                                                                                   \
  if (key_dim == K && value_dim == V)                                                                                   \
    return dl::launch_masked_flash<K, V>(q, q_stride, k_cache, k_row, v_cache, v_row, block_table, max_blocks, tiles,   \
                                         n_tiles, out, out_stride, n_heads, n_kv_heads, page_shift, scale, window,      \
                                         keep_first, sink, grp, parts, partial, n_tiles, stream)
  DL_CASE(16, 16); DL_CASE(32, 32); DL_CASE(48, 48); DL_CASE(64, 64); DL_CASE(80, 80); DL_CASE(96, 96); DL_CASE(112, 112);
  DL_CASE(128, 128);
  DL_CASE(32, 16); DL_CASE(48, 32); DL_CASE(64, 32); DL_CASE(96, 48); DL_CASE(96, 64); DL_CASE(128, 64); DL_CASE(64, 128);
  DL_CASE(32, 64); DL_CASE(48, 16); DL_CASE(16, 32);
#undef DL_CASE
  return DL_ERR_UNSUPPORTED;
}
