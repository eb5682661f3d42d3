// Building blocks of the tensor-core (mma.sync) attention kernels: asynchronous 16-byte copies, ldmatrix
// and mma wrappers, swizzled tiles in shared memory, the loader of a key or value tile through a
// request's block table, one warp's Q K^T and P V products, and the online-softmax step.
#pragma once

#include "common.cuh"

namespace mlr {

constexpr int ATTN_WARPS = 4;
constexpr int ATTN_THREADS = ATTN_WARPS * 32;
constexpr int TILE_Q = 64;
constexpr int TILE_KV = 64;

__device__ __forceinline__ uint32_t shared_address(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;   // 0: the 16 destination bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(shared_address(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(shared_address(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t* r, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(shared_address(p)));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&pair);
}

// A tile in shared memory: rows of D bfloat16, the 16-byte chunks of a row XOR-swizzled by the row
// index so that ldmatrix (8 rows x 16 bytes) is free of bank conflicts.
// HALVES (head_dim 128 as the tensor memory accelerator delivers it): two sub-tiles of 64 columns,
// each with rows of 128 bytes and the same swizzle; for head_dim 64 both layouts coincide.
template <int D, bool HALVES = false, int TKV = TILE_KV>
__device__ __forceinline__ bf16* tile_at(bf16* tile, int row, int chunk) {
  if (HALVES && D > 64) return tile + (chunk >> 3) * (TKV * 64) + row * 64 + (((chunk & 7) ^ (row & 7)) << 3);
  return tile + row * D + ((chunk ^ (row & 7)) << 3);
}

// Fetch `rows` rows starting at key `key0` of one kv head into a swizzled tile.  Keys outside
// [key_lo, key_hi] and keys on pages the request does not hold become zeros.
// `page_shift` is log2(page_size) when the page size is a power of two (the usual case: address
// arithmetic by shifts), else -1 (division).
template <int D>
__device__ __forceinline__ void load_kv_tile(bf16* tile, const bf16* pool, const int* __restrict__ table,
                                             int key0, int rows, int key_lo, int key_hi, int kv_heads, int kv_head,
                                             int page_size, int page_shift) {
  constexpr int CHUNKS = D / 8;
  for (int item = threadIdx.x; item < rows * CHUNKS; item += ATTN_THREADS) {
    const int r = item / CHUNKS, c = item - r * CHUNKS;
    const int key = key0 + r;
    bool valid = key >= key_lo && key <= key_hi;
    const bf16* src = pool;
    if (valid) {
      const int logical = page_shift >= 0 ? key >> page_shift : key / page_size;
      const int offset = page_shift >= 0 ? key & (page_size - 1) : key - logical * page_size;
      const int page = table[logical];
      valid = page >= 0;
      if (valid) src = pool + (((size_t)page * kv_heads + kv_head) * page_size + offset) * D + c * 8;
    }
    cp_async_16(tile_at<D>(tile, r, c), src, valid);
  }
}

// One warp: S[16 x (8*NT)] = Q[16 x D] K^T for keys key_row0.. of a K tile.
template <int D, int NT, bool HALVES = false, int TKV = TILE_KV>
__device__ __forceinline__ void warp_qk(float (*s)[4], const uint32_t (*q_frag)[4], bf16* k_tile, int key_row0, int lane) {
#pragma unroll
  for (int j = 0; j < NT; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
    for (int jp = 0; jp < NT / 2; ++jp) {
      uint32_t b[4];
      const int key = key_row0 + jp * 16 + (lane & 7) + ((lane >> 4) << 3);
      const int chunk = ks * 2 + ((lane >> 3) & 1);
      ldmatrix_x4(b, tile_at<D, HALVES, TKV>(k_tile, key, chunk));
      mma_bf16(s[2 * jp], q_frag[ks], b[0], b[1]);
      mma_bf16(s[2 * jp + 1], q_frag[ks], b[2], b[3]);
    }
  }
}

// One warp: O[16 x D] += P[16 x (8*NT)] V for keys key_row0.. of a V tile; P comes from the score
// registers, rounded to bfloat16.
template <int D, int NT, bool HALVES = false, int TKV = TILE_KV>
__device__ __forceinline__ void warp_pv(float (*o)[4], const float (*p)[4], bf16* v_tile, int key_row0, int lane) {
#pragma unroll
  for (int kk = 0; kk < NT / 2; ++kk) {
    uint32_t a[4];
    a[0] = pack_bf16(p[2 * kk][0], p[2 * kk][1]);
    a[1] = pack_bf16(p[2 * kk][2], p[2 * kk][3]);
    a[2] = pack_bf16(p[2 * kk + 1][0], p[2 * kk + 1][1]);
    a[3] = pack_bf16(p[2 * kk + 1][2], p[2 * kk + 1][3]);
#pragma unroll
    for (int dp = 0; dp < D / 16; ++dp) {
      uint32_t b[4];
      const int key = key_row0 + kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
      const int chunk = dp * 2 + (lane >> 4);
      ldmatrix_x4_trans(b, tile_at<D, HALVES, TKV>(v_tile, key, chunk));
      mma_bf16(o[2 * dp], a, b[0], b[1]);
      mma_bf16(o[2 * dp + 1], a, b[2], b[3]);
    }
  }
}

// Online softmax step on one warp's score fragment.  Thread owns rows r0 = lane/4 and r0 + 8;
// limit_lo[i] <= key <= limit_hi[i] are visible for row i, and so are the first `keep_first` keys up to limit_hi[i].  Scores arrive unscaled; `scale_log2`
// = head_dim^-0.5 * log2(e).  Leaves probabilities in s and rescales o.
// MASKED = false: the caller knows that every key of the tile is visible to every row.
template <int NT, int OT, bool MASKED = true>
__device__ __forceinline__ void softmax_step(float (*s)[4], float (*o)[4], float* m, float* l, int key_base,
                                             const int* limit_lo, const int* limit_hi, float scale_log2, int lane,
                                             int keep_first = 0) {
  float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int j = 0; j < NT; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int key = key_base + j * 8 + (lane & 3) * 2 + (e & 1);
      const int i = e >> 1;
      const bool visible = !MASKED || ((key >= limit_lo[i] || key < keep_first) && key <= limit_hi[i]);
      s[j][e] = visible ? s[j][e] * scale_log2 : -INFINITY;
      tile_max[i] = fmaxf(tile_max[i], s[j][e]);
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    tile_max[i] = fmaxf(tile_max[i], __shfl_xor_sync(0xffffffffu, tile_max[i], 1));
    tile_max[i] = fmaxf(tile_max[i], __shfl_xor_sync(0xffffffffu, tile_max[i], 2));
  }
  float alpha[2], row_sum[2] = {0.f, 0.f}, base[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float m_new = fmaxf(m[i], tile_max[i]);
    base[i] = m_new == -INFINITY ? 0.f : m_new;       // nothing visible yet: keep everything at zero
    alpha[i] = exp2f(m[i] - base[i]);                  // m = -inf gives 0
    m[i] = m_new;
  }
#pragma unroll
  for (int j = 0; j < NT; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float prob = exp2f(s[j][e] - base[e >> 1]);   // -inf gives 0
      s[j][e] = prob;
      row_sum[e >> 1] += prob;
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    row_sum[i] += __shfl_xor_sync(0xffffffffu, row_sum[i], 1);
    row_sum[i] += __shfl_xor_sync(0xffffffffu, row_sum[i], 2);
    l[i] = l[i] * alpha[i] + row_sum[i];
  }
#pragma unroll
  for (int t = 0; t < OT; ++t) {
    o[t][0] *= alpha[0]; o[t][1] *= alpha[0];
    o[t][2] *= alpha[1]; o[t][3] *= alpha[1];
  }
}

}  // namespace mlr
