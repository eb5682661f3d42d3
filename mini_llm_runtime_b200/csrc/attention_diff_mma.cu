// Differential attention of prompt portions on the tensor cores (bfloat16, mma.sync m16n8k16).
//
// The two maps of a head are two ordinary attentions over the same values: work item (64 query rows,
// head, map) computes softmax(q_map K_map^T * scale) V with FlashAttention-2 arithmetic (scores and
// running statistics in float32, probabilities rounded to bfloat16 for the second product) and
// leaves its normalised rows as float32 in a scratch tensor [rows, heads, 2, vdim].  A second small
// kernel combines them: o = a1 - lambda * a2, o * rsqrt(mean(o^2) + eps) * out_scale.
//
// Keys are visible up to the row's own position if they lie inside its window or among the first
// `keep_first` positions; the tiles of 64 keys between the kept positions and the window are never
// fetched.  K tiles hold one map's half of the cached key rows (row stride 2 * dim), V tiles the
// whole value rows; both are double-buffered with asynchronous copies.
#include "mma_attention.cuh"

namespace mlr {

// Rows `key0 ..` of one kv head into a swizzled tile of DT columns; a key that is not visible to any
// row of the item (beyond `key_hi`, or below `key_lo` and not among the first `keep`), or on a page the
// request does not hold, becomes zeros.  `stride` and `column` select a column range of wider rows.
template <int DT>
__device__ __forceinline__ void load_tile_cols(bf16* tile, const bf16* pool, const int* __restrict__ table, int key0,
                                               int key_lo, int key_hi, int keep, int kv_heads, int kv_head,
                                               int page_size, int stride, int column) {
  constexpr int CHUNKS = DT / 8;
  for (int item = threadIdx.x; item < TILE_KV * CHUNKS; item += ATTN_THREADS) {
    const int r = item / CHUNKS, c = item - r * CHUNKS;
    const int key = key0 + r;
    bool valid = key <= key_hi && (key >= key_lo || key < keep);
    const bf16* src = pool;
    if (valid) {
      const int logical = key / page_size;
      const int page = table[logical];
      valid = page >= 0;
      if (valid)
        src = pool + (((size_t)page * kv_heads + kv_head) * page_size + (key - logical * page_size)) * stride + column + c * 8;
    }
    cp_async_16(tile_at<DT>(tile, r, c), src, valid);
  }
}

template <int DQ, int DV>
__global__ void __launch_bounds__(ATTN_THREADS)
diff_prefill_mma_kernel(const bf16* q, const bf16* k_pool, const bf16* v_pool, float* __restrict__ maps,
                        const int* __restrict__ tile_seg, const int* __restrict__ tile_row0,
                        const int* __restrict__ seg_q_start, const int* __restrict__ seg_q_len,
                        const int* __restrict__ seg_pos0, const int* __restrict__ block_table,
                        const int* __restrict__ seg_slot, int table_width, int heads, int kv_heads, int page_size,
                        int window, int keep_first, float scale_log2) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(128) uint8_t attn_shared[];
  bf16* q_tile = reinterpret_cast<bf16*>(attn_shared);         // [64][DQ]
  bf16* k_tiles = q_tile + TILE_Q * DQ;                         // 2 x [64][DQ]
  bf16* v_tiles = k_tiles + 2 * TILE_KV * DQ;                   // 2 x [64][DV]

  const int tile = blockIdx.x, head = blockIdx.y >> 1, map = blockIdx.y & 1;   // the list is heaviest first
  const int kv_head = head / (heads / kv_heads);
  const int seg = tile_seg[tile], row0 = tile_row0[tile];
  const int q_start = seg_q_start[seg], q_len = seg_q_len[seg], pos0 = seg_pos0[seg];
  const int rows = min(TILE_Q, q_len - row0);
  const int* table = block_table + (size_t)seg_slot[seg] * table_width;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int first_pos = pos0 + row0, last_pos = first_pos + rows - 1;
  const int lowest = window > 0 ? max(0, first_pos - window + 1) : 0;
  const int keep = window > 0 ? keep_first : 0;
  const int tile_begin = lowest / TILE_KV, tile_end = last_pos / TILE_KV;   // inclusive
  // key tiles in walking order: those of the kept positions that lie before the window's, then the window's
  const int before = min((keep + TILE_KV - 1) / TILE_KV, tile_begin);
  const int count = before + tile_end - tile_begin + 1;
  auto key_tile = [&](int n) { return n < before ? n : tile_begin + (n - before); };

  constexpr int CHUNKS = DQ / 8;
  for (int item = threadIdx.x; item < TILE_Q * CHUNKS; item += ATTN_THREADS) {
    const int r = item / CHUNKS, c = item - r * CHUNKS;
    const bool valid = r < rows;
    const bf16* src = valid ? q + (((size_t)(q_start + row0 + r) * heads + head) * 2 + map) * DQ + c * 8 : q;
    cp_async_16(tile_at<DQ>(q_tile, r, c), src, valid);
  }
  auto fetch = [&](int n, int buffer) {
    const int key0 = key_tile(n) * TILE_KV;
    load_tile_cols<DQ>(k_tiles + buffer * TILE_KV * DQ, k_pool, table, key0, lowest, last_pos, keep, kv_heads, kv_head,
                       page_size, 2 * DQ, map * DQ);
    load_tile_cols<DV>(v_tiles + buffer * TILE_KV * DV, v_pool, table, key0, lowest, last_pos, keep, kv_heads, kv_head,
                       page_size, DV, 0);
    cp_async_commit();
  };
  fetch(0, 0);

  int limit_lo[2], limit_hi[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = warp * 16 + (lane >> 2) + 8 * i;
    const int position = first_pos + r;
    limit_hi[i] = r < rows ? position : -1;                       // rows past the segment see nothing
    limit_lo[i] = window > 0 ? max(0, position - window + 1) : 0;
  }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[DV / 8][4];
#pragma unroll
  for (int t = 0; t < DV / 8; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;
  uint32_t q_frag[DQ / 16][4];

  for (int n = 0; n < count; ++n) {
    const int buffer = n & 1;
    if (n + 1 < count) {
      fetch(n + 1, buffer ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (n == 0) {
#pragma unroll
      for (int ks = 0; ks < DQ / 16; ++ks) {
        const int r = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
        ldmatrix_x4(q_frag[ks], tile_at<DQ>(q_tile, r, ks * 2 + (lane >> 4)));
      }
    }
    const int t = key_tile(n);
    const int warp_last = first_pos + min(rows - 1, warp * 16 + 15);
    if (warp * 16 < rows && t * TILE_KV <= warp_last) {
      float s[TILE_KV / 8][4];
      warp_qk<DQ, TILE_KV / 8>(s, q_frag, k_tiles + buffer * TILE_KV * DQ, 0, lane);
      softmax_step<TILE_KV / 8, DV / 8>(s, o, m, l, t * TILE_KV, limit_lo, limit_hi, scale_log2, lane, keep);
      warp_pv<DV, TILE_KV / 8>(o, s, v_tiles + buffer * TILE_KV * DV, 0, lane);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = warp * 16 + (lane >> 2) + 8 * i;
    if (r >= rows) continue;
    const float inv = 1.f / l[i];
    float* dst = maps + (((size_t)(q_start + row0 + r) * heads + head) * 2 + map) * DV + (lane & 3) * 2;
#pragma unroll
    for (int t = 0; t < DV / 8; ++t)
      *reinterpret_cast<float2*>(dst + t * 8) = make_float2(o[t][2 * i] * inv, o[t][2 * i + 1] * inv);
  }
}

// One warp per (row, head) of the listed segments: o = a1 - lambda * a2, o / rms(o) * out_scale.
__global__ void __launch_bounds__(128)
diff_combine_kernel(const float* maps, bf16* __restrict__ out, const int* __restrict__ tile_seg,
                    const int* __restrict__ tile_row0, const int* __restrict__ seg_q_start,
                    const int* __restrict__ seg_q_len, int heads, int vdim, float lambda, float eps, float out_scale) {
  pdl_trigger();
  pdl_wait();
  const int tile = blockIdx.x, seg = tile_seg[tile], row0 = tile_row0[tile];
  const int rows = min(TILE_Q, seg_q_len[seg] - row0);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int item = warp; item < rows * heads; item += 4) {
    const int r = item / heads, head = item - r * heads;
    const size_t row = (size_t)(seg_q_start[seg] + row0 + r);
    const float* a1 = maps + ((row * heads + head) * 2) * vdim;
    const float* a2 = a1 + vdim;
    float sq = 0.f;
    for (int c = lane; c < vdim; c += 32) {
      const float o = a1[c] - lambda * a2[c];
      sq = fmaf(o, o, sq);
    }
    sq = warp_sum(sq);
    const float factor = out_scale / sqrtf(sq / (float)vdim + eps);
    for (int c = lane; c < vdim; c += 32)
      out[(row * heads + head) * vdim + c] = __float2bfloat16_rn((a1[c] - lambda * a2[c]) * factor);
  }
}

template <int DQ, int DV>
int diff_prefill_launch(const void* q, const void* k_pool, const void* v_pool, float* maps, void* out,
                        const int* tile_seg, const int* tile_row0, const int* seg_q_start, const int* seg_q_len,
                        const int* seg_pos0, const int* block_table, const int* seg_slot, int table_width, int tiles,
                        int heads, int kv_heads, int page_size, int window, int keep_first, float scale, float lambda,
                        float eps, float out_scale, cudaStream_t stream) {
  const size_t shared = sizeof(bf16) * ((size_t)TILE_Q * DQ + 2 * TILE_KV * DQ + 2 * TILE_KV * DV);
  static bool configured = false;
  if (!configured && shared > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(diff_prefill_mma_kernel<DQ, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)shared);
    if (err != cudaSuccess) return (int)err;
    configured = true;
  }
  launch_kernel(diff_prefill_mma_kernel<DQ, DV>, dim3(tiles, heads * 2), dim3(ATTN_THREADS), shared, stream,
                (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, maps, tile_seg, tile_row0, seg_q_start,
                seg_q_len, seg_pos0, block_table, seg_slot, table_width, heads, kv_heads, page_size, window, keep_first,
                scale * 1.4426950408889634f);
  int status = launch_status();
  if (status != MLR_OK) return status;
  launch_kernel(diff_combine_kernel, dim3(tiles), dim3(128), 0, stream, (const float*)maps, (bf16*)out, tile_seg,
                tile_row0, seg_q_start, seg_q_len, heads, DV, lambda, eps, out_scale);
  return launch_status();
}

}  // namespace mlr

using namespace mlr;

MLR_DEFINE_PDL_SWITCH

// 1 if the tensor-core kernel takes these head sizes (the swizzled tiles want rows of 128 or 256 bytes).
MLR_EXPORT int mlr_attention_diff_mma_supports(int dim, int vdim) {
  return (dim == 64 || dim == 128) && (vdim == 64 || vdim == 128) ? 1 : 0;
}

// q: bfloat16 [rows, heads, 2, dim]; pools as the SIMT kernel's; maps: float32 scratch [rows, heads, 2, vdim];
// out: bfloat16 [rows, heads, vdim].  tile_seg/tile_row0: tiles of up to 64 rows of one segment, heaviest first.
MLR_EXPORT int mlr_attention_diff_mma(const void* q, const void* k_pool, const void* v_pool, float* maps, void* out,
                                      const int* tile_seg, const int* tile_row0, const int* seg_q_start,
                                      const int* seg_q_len, const int* seg_pos0, const int* block_table,
                                      const int* seg_slot, int table_width, int tiles, int heads, int kv_heads, int dim,
                                      int vdim, int page_size, int window, int keep_first, float scale, float lambda,
                                      float eps, float out_scale, cudaStream_t stream) {
  if (tiles == 0) return MLR_OK;
  if (tiles < 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || page_size <= 0 || table_width <= 0 ||
      keep_first < 0)
    return MLR_BAD_SIZE;
  if (2 * heads > 65535) return MLR_TOO_LARGE;
#define MLR_DIFF_CASE(DQ, DV)                                                                                      \
  if (dim == DQ && vdim == DV)                                                                                     \
    return diff_prefill_launch<DQ, DV>(q, k_pool, v_pool, maps, out, tile_seg, tile_row0, seg_q_start, seg_q_len,   \
                                       seg_pos0, block_table, seg_slot, table_width, tiles, heads, kv_heads,       \
                                       page_size, window, keep_first, scale, lambda, eps, out_scale, stream);
  MLR_DIFF_CASE(64, 64)
  MLR_DIFF_CASE(64, 128)
  MLR_DIFF_CASE(128, 64)
  MLR_DIFF_CASE(128, 128)
#undef MLR_DIFF_CASE
  return MLR_BAD_SIZE;
}
