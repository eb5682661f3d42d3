// Differential attention over the paged cache, with a sliding window that keeps the first positions.
//
// Every query head carries two attention maps over the same values.  A query row holds
// [map 1 | map 2] (2 * dim numbers) per head, a cached key likewise per kv head, a cached value vdim
// numbers.  With a1, a2 the two maps' softmax-weighted value sums:
//
//     o = a1 - lambda * a2;   out = o * rsqrt(mean(o^2) + eps) * out_scale       (per head, over vdim)
//
// Visibility of key j for the query at position i: j <= i and (i - j < window or j < keep_first);
// window <= 0 means every earlier key.  Scores, softmax, sums and the norm are float32.
//
// mlr_qk_norm_kv_write   RMS-normalises every (head, map) of q and k over dim with a weight shared by
//                        all heads and maps, stores k and v into the pages, returns q.
// mlr_attention_diff     ragged batch of prompt portions and decoded rows, 16 query rows per CTA;
//                        keys walked in tiles of 32 aligned to absolute positions, reductions in a fixed
//                        lane order: a row's result depends on its own request's cache only.
// mlr_attention_diff_decode   one CTA per (decoded row, head): its warps take the key tiles in turn and
//                        merge their running states in warp order.
#include "common.cuh"

namespace mlr {

constexpr int ROWS_PER_TILE = 16;
constexpr int KEYS_PER_TILE = 32;
constexpr int MAX_VDIM = 256;
constexpr int MAX_QK = 512;     // 2 * dim

// ------------------------------------------------------------------ q/k norm + cache write
// One warp per (row, unit): units 0 .. 2H-1 are q (head, map), then 2G of k, then G of v.
template <typename T>
__global__ void __launch_bounds__(128)
qk_norm_kv_write_kernel(const float* qkv, const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                        const long long* __restrict__ slots, T* __restrict__ q_out, T* __restrict__ k_pool,
                        T* __restrict__ v_pool, int rows, int heads, int kv_heads, int dim, int vdim, int page_size,
                        float eps, int write_kv) {
  pdl_trigger();
  pdl_wait();
  const int units = 2 * heads + 2 * kv_heads + kv_heads;
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= (long long)rows * units) return;
  const int row = (int)(item / units), unit = (int)(item - (long long)row * units);
  const int in_width = 2 * heads * dim + 2 * kv_heads * dim + kv_heads * vdim;
  const float* in = qkv + (size_t)row * in_width;
  if (unit < 2 * heads + 2 * kv_heads) {
    const bool is_q = unit < 2 * heads;
    const float* x = in + (size_t)unit * dim;       // q units then k units lie one after the other
    float sq = 0.f;
    for (int d = lane; d < dim; d += 32) sq = fmaf(x[d], x[d], sq);
    sq = warp_sum(sq);
    const float factor = 1.f / sqrtf(sq / (float)dim + eps);
    const float* w = is_q ? q_weight : k_weight;
    T* dst;
    if (is_q) {
      dst = q_out + (size_t)row * 2 * heads * dim + (size_t)unit * dim;
    } else {
      if (!write_kv) return;
      const int ku = unit - 2 * heads, g = ku >> 1, m = ku & 1;
      const long long slot = slots[row];
      const long long page = slot / page_size, offset = slot - page * page_size;
      dst = k_pool + (((size_t)page * kv_heads + g) * page_size + offset) * 2 * dim + (size_t)m * dim;
    }
    for (int d = lane; d < dim; d += 32) dst[d] = from_float<T>(x[d] * factor * w[d]);
  } else {
    if (!write_kv) return;
    const int g = unit - 2 * heads - 2 * kv_heads;
    const float* x = in + (size_t)(2 * heads + 2 * kv_heads) * dim + (size_t)g * vdim;
    const long long slot = slots[row];
    const long long page = slot / page_size, offset = slot - page * page_size;
    T* dst = v_pool + (((size_t)page * kv_heads + g) * page_size + offset) * vdim;
    for (int d = lane; d < vdim; d += 32) dst[d] = from_float<T>(x[d]);
  }
}

struct DiffArgs {
  const int *seg_q_start, *seg_q_len, *seg_pos0, *block_table, *seg_slot;
  int table_width, heads, kv_heads, dim, vdim, page_size, window, keep_first;
  float scale, lambda, eps, out_scale;
};

__device__ __forceinline__ bool key_visible(int key, int p, int window, int keep_first) {
  return key <= p && (window <= 0 || p - key < window || key < keep_first);
}

// The next key tile to visit after the tile starting at k0, skipping the tiles between the kept
// first positions and the lowest key the window of the tile's first row still sees.
__device__ __forceinline__ int next_key_tile(int k0, int lowest_tile, int keep_first) {
  int next = k0 + KEYS_PER_TILE;
  if (next >= keep_first && next < lowest_tile) next = lowest_tile;
  return next;
}

template <typename T>
__global__ void __launch_bounds__(128)
attention_diff_kernel(const T* q, const T* k_pool, const T* v_pool, T* __restrict__ out,
                      const int* __restrict__ tile_seg, const int* __restrict__ tile_row0, DiffArgs p) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float shared[];
  const int QK = 2 * p.dim, D = p.dim, V = p.vdim;
  float* q_rows = shared;                                  // [16][QK]
  float* k_tile = q_rows + ROWS_PER_TILE * QK;             // [32][QK + 1]
  float* v_tile = k_tile + KEYS_PER_TILE * (QK + 1);       // [32][V]
  float* p_tile = v_tile + KEYS_PER_TILE * V;              // [16 rows][2 maps][32]

  const int tile = blockIdx.x, head = blockIdx.y;
  const int kv_head = head / (p.heads / p.kv_heads);
  const int seg = tile_seg[tile], row0 = tile_row0[tile];
  const int q_start = p.seg_q_start[seg], q_len = p.seg_q_len[seg], pos0 = p.seg_pos0[seg];
  const int rows = min(ROWS_PER_TILE, q_len - row0);
  const int* table = p.block_table + (size_t)p.seg_slot[seg] * p.table_width;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  for (int idx = threadIdx.x; idx < ROWS_PER_TILE * QK; idx += blockDim.x) {
    const int r = idx / QK, d = idx - r * QK;
    q_rows[idx] = r < rows ? to_float(q[((size_t)(q_start + row0 + r) * p.heads + head) * QK + d]) : 0.f;
  }

  float m[4][2], l[4][2], acc[4][2][MAX_VDIM / 32];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      m[i][a] = -INFINITY;
      l[i][a] = 0.f;
#pragma unroll
      for (int c = 0; c < MAX_VDIM / 32; ++c) acc[i][a][c] = 0.f;
    }

  const int first_pos = pos0 + row0, last_pos = pos0 + row0 + rows - 1;
  const int lowest_key = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
  const int lowest_tile = (lowest_key / KEYS_PER_TILE) * KEYS_PER_TILE;
  const int keep = p.window > 0 ? p.keep_first : 0;
  for (int k0 = keep > 0 ? 0 : lowest_tile; k0 <= last_pos; k0 = next_key_tile(k0, lowest_tile, keep)) {
    __syncthreads();
    for (int idx = threadIdx.x; idx < KEYS_PER_TILE * QK; idx += blockDim.x) {
      const int j = idx / QK, d = idx - j * QK;
      const int key = k0 + j;
      float kv = 0.f;
      if (key <= last_pos) {
        const int page = table[key / p.page_size];
        if (page >= 0)
          kv = to_float(k_pool[(((size_t)page * p.kv_heads + kv_head) * p.page_size + key % p.page_size) * QK + d]);
      }
      k_tile[j * (QK + 1) + d] = kv;
    }
    for (int idx = threadIdx.x; idx < KEYS_PER_TILE * V; idx += blockDim.x) {
      const int j = idx / V, d = idx - j * V;
      const int key = k0 + j;
      float vv = 0.f;
      if (key <= last_pos) {
        const int page = table[key / p.page_size];
        if (page >= 0)
          vv = to_float(v_pool[(((size_t)page * p.kv_heads + kv_head) * p.page_size + key % p.page_size) * V + d]);
      }
      v_tile[j * V + d] = vv;
    }
    __syncthreads();

    const int key = k0 + lane;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = warp * 4 + i;
      if (r >= rows) continue;  // uniform per warp
      const int pos = first_pos + r;
      const bool visible = key_visible(key, pos, p.window, p.keep_first);
      const float* qr = q_rows + r * QK;
      const float* kr = k_tile + lane * (QK + 1);
      float alpha[2];
      bool any = false;
#pragma unroll
      for (int a = 0; a < 2; ++a) {
        float s = 0.f;
        for (int d = 0; d < D; ++d) s = fmaf(qr[a * D + d], kr[a * D + d], s);
        s = visible ? s * p.scale : -INFINITY;
        const float m_new = fmaxf(m[i][a], warp_max(s));
        float prob = 0.f;
        alpha[a] = 1.f;
        if (m_new != -INFINITY) {
          alpha[a] = expf(m[i][a] - m_new);      // m = -inf gives 0
          prob = visible ? expf(s - m_new) : 0.f;
          l[i][a] = l[i][a] * alpha[a] + warp_sum(prob);
          m[i][a] = m_new;
          any = true;
        }
        p_tile[(r * 2 + a) * KEYS_PER_TILE + lane] = prob;
      }
      if (!any) continue;       // no visible key yet for this row (uniform per warp)
      __syncwarp();
      const float* p1 = p_tile + (r * 2) * KEYS_PER_TILE;
      const float* p2 = p1 + KEYS_PER_TILE;
#pragma unroll
      for (int c = 0; c < MAX_VDIM / 32; ++c) {
        const int d = lane + 32 * c;
        if (d < V) {
          float a1 = acc[i][0][c] * alpha[0], a2 = acc[i][1][c] * alpha[1];
          for (int j = 0; j < KEYS_PER_TILE; ++j) {
            const float vv = v_tile[j * V + d];
            a1 = fmaf(p1[j], vv, a1);
            a2 = fmaf(p2[j], vv, a2);
          }
          acc[i][0][c] = a1;
          acc[i][1][c] = a2;
        }
      }
      __syncwarp();
    }
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = warp * 4 + i;
    if (r >= rows) continue;
    const float inv1 = 1.f / l[i][0], inv2 = 1.f / l[i][1];
    float o[MAX_VDIM / 32], sq = 0.f;
#pragma unroll
    for (int c = 0; c < MAX_VDIM / 32; ++c) {
      const int d = lane + 32 * c;
      o[c] = d < V ? acc[i][0][c] * inv1 - p.lambda * (acc[i][1][c] * inv2) : 0.f;
      sq = fmaf(o[c], o[c], sq);
    }
    sq = warp_sum(sq);
    const float factor = p.out_scale / sqrtf(sq / (float)V + p.eps);
    T* dst = out + ((size_t)(q_start + row0 + r) * p.heads + head) * V;
#pragma unroll
    for (int c = 0; c < MAX_VDIM / 32; ++c) {
      const int d = lane + 32 * c;
      if (d < V) dst[d] = from_float<T>(o[c] * factor);
    }
  }
}

// q . k over n entries, q in shared memory as floats, k a row of the pool: 16-byte loads where the
// row's start and length allow them.
__device__ __forceinline__ float dot_row(const float* q, const float* k, int n) {
  float s = 0.f;
  if ((n & 3) == 0 && (reinterpret_cast<uintptr_t>(k) & 15) == 0) {
    const float4* k4 = reinterpret_cast<const float4*>(k);
    for (int d = 0; d < n / 4; ++d) {
      const float4 kk = k4[d];
      s = fmaf(q[4 * d], kk.x, s); s = fmaf(q[4 * d + 1], kk.y, s);
      s = fmaf(q[4 * d + 2], kk.z, s); s = fmaf(q[4 * d + 3], kk.w, s);
    }
    return s;
  }
  for (int d = 0; d < n; ++d) s = fmaf(q[d], k[d], s);
  return s;
}
__device__ __forceinline__ float dot_row(const float* q, const bf16* k, int n) {
  float s = 0.f;
  if ((n & 7) == 0 && (reinterpret_cast<uintptr_t>(k) & 15) == 0) {
    const uint4* k8 = reinterpret_cast<const uint4*>(k);
    for (int d = 0; d < n / 8; ++d) {
      const uint4 kk = k8[d];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&kk);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        s = fmaf(q[8 * d + 2 * e], f.x, s);
        s = fmaf(q[8 * d + 2 * e + 1], f.y, s);
      }
    }
    return s;
  }
  for (int d = 0; d < n; ++d) s = fmaf(q[d], __bfloat162float(k[d]), s);
  return s;
}

// ------------------------------------------------------------------ decoded rows
// One CTA of DECODE_WARPS warps per (segment of one row, head).  Warp w takes the visible key tiles
// number w, w + DECODE_WARPS, ..; each lane scores one key of a tile.  The warps' running states
// (max, sum, value sums of both maps) are merged by warp 0 in warp order.
constexpr int DECODE_WARPS = 32;      // about one 32-key tile per warp at a window of a thousand keys

// WIDE (bfloat16 values, vdim a multiple of 8): a lane fetches eight adjacent value channels of one
// key with one 16-byte load, 32 / lanes-per-key keys per warp-wide load, and the lane groups' sums are
// added by shuffles after the last tile.
template <typename T, bool WIDE>
__global__ void __launch_bounds__(DECODE_WARPS * 32)
attention_diff_decode_kernel(const T* q, const T* k_pool, const T* v_pool, T* __restrict__ out,
                             const int* __restrict__ decode_seg, DiffArgs p) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) float shared[];
  const int QK = 2 * p.dim, D = p.dim, V = p.vdim;
  long long* places = reinterpret_cast<long long*>(shared);     // [warps][32]
  float* q_row = shared + 2 * DECODE_WARPS * KEYS_PER_TILE;     // [QK]
  float* probs = q_row + QK;                                    // [warps][2][32]
  float* merged = probs + DECODE_WARPS * 2 * KEYS_PER_TILE;     // [warps][2][V + 2]
  const int seg = decode_seg != nullptr ? decode_seg[blockIdx.x] : blockIdx.x, head = blockIdx.y;
  const int kv_head = head / (p.heads / p.kv_heads);
  const int row = p.seg_q_start[seg], pos = p.seg_pos0[seg];
  const int* table = p.block_table + (size_t)p.seg_slot[seg] * p.table_width;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  for (int d = threadIdx.x; d < QK; d += blockDim.x)
    q_row[d] = to_float(q[((size_t)row * p.heads + head) * QK + d]);
  __syncthreads();

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f}, acc[2][MAX_VDIM / 32];
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int c = 0; c < MAX_VDIM / 32; ++c) acc[a][c] = 0.f;

  // WIDE: lanes_per_key lanes cover a value row, eight channels each; `sub` is the lane's key within a load
  int lanes_per_key = 1;
  while (lanes_per_key * 8 < V) lanes_per_key *= 2;
  const int keys_per_load = 32 / lanes_per_key, sub = lane / lanes_per_key, d0 = (lane % lanes_per_key) * 8;
  float wide[2][8];
#pragma unroll
  for (int e = 0; e < 8; ++e) wide[0][e] = wide[1][e] = 0.f;

  // the visible keys: [0, kept) and [lowest, pos]; as one list of tiles of 32 consecutive list entries
  const int lowest = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  const int kept = p.window > 0 ? min(p.keep_first, lowest) : 0;      // kept positions below the window
  const int total = kept + (pos - lowest + 1);
  float* pw = probs + warp * 2 * KEYS_PER_TILE;
  long long* place = places + warp * KEYS_PER_TILE;       // row of each of the tile's keys in the pools, -1: none
  for (int t0 = warp * KEYS_PER_TILE; t0 < total; t0 += DECODE_WARPS * KEYS_PER_TILE) {
    const int entry = t0 + lane;
    long long at = -1;
    if (entry < total) {
      const int key = entry < kept ? entry : lowest + (entry - kept);
      const int page = table[key / p.page_size];
      if (page >= 0) at = ((long long)page * p.kv_heads + kv_head) * p.page_size + key % p.page_size;
    }
    place[lane] = at;
    float alpha[2];
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      float s = -INFINITY;
      if (at >= 0) {
        s = dot_row(q_row + a * D, k_pool + at * QK + a * D, D) * p.scale;
      }
      const float m_new = fmaxf(m[a], warp_max(s));
      float prob = 0.f;
      alpha[a] = 1.f;
      if (m_new != -INFINITY) {
        alpha[a] = expf(m[a] - m_new);
        prob = at >= 0 ? expf(s - m_new) : 0.f;
        l[a] = l[a] * alpha[a] + warp_sum(prob);
        m[a] = m_new;
      }
      pw[a * KEYS_PER_TILE + lane] = prob;
    }
    __syncwarp();
    const int count = min(KEYS_PER_TILE, total - t0);
    if (WIDE) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        wide[0][e] *= alpha[0];
        wide[1][e] *= alpha[1];
      }
      // a key without a page has probability 0: its load is pointed at row 0 and adds nothing, so
      // that the loads of a whole tile can be in flight at once
#pragma unroll 4
      for (int j0 = 0; j0 < KEYS_PER_TILE; j0 += keys_per_load) {
        const int j = j0 + sub;
        const bool live = j < count && d0 < V;
        const long long row_at = live ? max(place[j], 0LL) : 0LL;
        const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(v_pool) + row_at * V + (d0 < V ? d0 : 0));
        const float p1 = live ? pw[j] : 0.f, p2 = live ? pw[KEYS_PER_TILE + j] : 0.f;
        const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(pairs[e]);
          wide[0][2 * e] = fmaf(p1, f.x, wide[0][2 * e]);
          wide[0][2 * e + 1] = fmaf(p1, f.y, wide[0][2 * e + 1]);
          wide[1][2 * e] = fmaf(p2, f.x, wide[1][2 * e]);
          wide[1][2 * e + 1] = fmaf(p2, f.y, wide[1][2 * e + 1]);
        }
      }
    } else {
#pragma unroll
      for (int c = 0; c < MAX_VDIM / 32; ++c) {
        const int d = lane + 32 * c;
        if (d < V) {
          float a1 = acc[0][c] * alpha[0], a2 = acc[1][c] * alpha[1];
#pragma unroll 8
          for (int j = 0; j < KEYS_PER_TILE; ++j) {
            const long long row_at = j < count ? max(place[j], 0LL) : 0LL;
            const float vv = to_float(v_pool[row_at * V + d]);
            a1 = fmaf(j < count ? pw[j] : 0.f, vv, a1);
            a2 = fmaf(j < count ? pw[KEYS_PER_TILE + j] : 0.f, vv, a2);
          }
          acc[0][c] = a1;
          acc[1][c] = a2;
        }
      }
    }
    __syncwarp();
  }
  // hand the warp's state to warp 0
  if (WIDE) {
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
      for (int e = 0; e < 8; ++e)
        for (int offset = lanes_per_key; offset < 32; offset <<= 1)
          wide[a][e] += __shfl_xor_sync(0xffffffffu, wide[a][e], offset);
  }
#pragma unroll
  for (int a = 0; a < 2; ++a) {
    float* mine = merged + (size_t)(warp * 2 + a) * (V + 2);
    if (lane == 0) {
      mine[V] = m[a];
      mine[V + 1] = l[a];
    }
    if (WIDE) {
      if (sub == 0 && d0 < V) {
#pragma unroll
        for (int e = 0; e < 8; ++e) mine[d0 + e] = wide[a][e];
      }
    } else {
#pragma unroll
      for (int c = 0; c < MAX_VDIM / 32; ++c) {
        const int d = lane + 32 * c;
        if (d < V) mine[d] = acc[a][c];
      }
    }
  }
  __syncthreads();
  if (warp != 0) return;
  float o[MAX_VDIM / 32];
#pragma unroll
  for (int c = 0; c < MAX_VDIM / 32; ++c) o[c] = 0.f;
#pragma unroll
  for (int a = 0; a < 2; ++a) {
    float top = -INFINITY;
    for (int w = 0; w < DECODE_WARPS; ++w) top = fmaxf(top, merged[(size_t)(w * 2 + a) * (V + 2) + V]);
    float sum = 0.f, part[MAX_VDIM / 32];
#pragma unroll
    for (int c = 0; c < MAX_VDIM / 32; ++c) part[c] = 0.f;
    for (int w = 0; w < DECODE_WARPS; ++w) {
      const float* theirs = merged + (size_t)(w * 2 + a) * (V + 2);
      if (theirs[V] == -INFINITY) continue;
      const float f = expf(theirs[V] - top);
      sum = fmaf(theirs[V + 1], f, sum);
#pragma unroll
      for (int c = 0; c < MAX_VDIM / 32; ++c) {
        const int d = lane + 32 * c;
        if (d < V) part[c] = fmaf(theirs[d], f, part[c]);
      }
    }
    const float inv = 1.f / sum;
#pragma unroll
    for (int c = 0; c < MAX_VDIM / 32; ++c) o[c] = a == 0 ? part[c] * inv : o[c] - p.lambda * (part[c] * inv);
  }
  float sq = 0.f;
#pragma unroll
  for (int c = 0; c < MAX_VDIM / 32; ++c) {
    if (lane + 32 * c >= V) o[c] = 0.f;
    sq = fmaf(o[c], o[c], sq);
  }
  sq = warp_sum(sq);
  const float factor = p.out_scale / sqrtf(sq / (float)V + p.eps);
  T* dst = out + ((size_t)row * p.heads + head) * V;
#pragma unroll
  for (int c = 0; c < MAX_VDIM / 32; ++c) {
    const int d = lane + 32 * c;
    if (d < V) dst[d] = from_float<T>(o[c] * factor);
  }
}

template <typename T>
int attention_diff_launch(const void* q, const void* k_pool, const void* v_pool, void* out, const int* tile_seg,
                          const int* tile_row0, int tiles, const DiffArgs& args, cudaStream_t stream) {
  const int QK = 2 * args.dim;
  const size_t shared = sizeof(float) * ((size_t)ROWS_PER_TILE * QK + (size_t)KEYS_PER_TILE * (QK + 1) +
                                         (size_t)KEYS_PER_TILE * args.vdim + (size_t)ROWS_PER_TILE * 2 * KEYS_PER_TILE);
  if (shared > 200 * 1024) return MLR_TOO_LARGE;
  if (shared > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(attention_diff_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    if (err != cudaSuccess) return (int)err;
  }
  launch_kernel(attention_diff_kernel<T>, dim3(tiles, args.heads), dim3(128), shared, stream, (const T*)q,
                (const T*)k_pool, (const T*)v_pool, (T*)out, tile_seg, tile_row0, args);
  return launch_status();
}

template <typename T>
int attention_diff_decode_launch(const void* q, const void* k_pool, const void* v_pool, void* out,
                                 const int* decode_seg, int count, const DiffArgs& args, cudaStream_t stream) {
  const size_t shared = sizeof(float) * ((size_t)2 * args.dim + (size_t)DECODE_WARPS * 2 * KEYS_PER_TILE +
                                         (size_t)DECODE_WARPS * 2 * (args.vdim + 2)) +
                        sizeof(long long) * DECODE_WARPS * KEYS_PER_TILE;
  const bool wide = sizeof(T) == 2 && args.vdim % 8 == 0 && (reinterpret_cast<uintptr_t>(v_pool) & 15) == 0;
  auto kernel = wide ? attention_diff_decode_kernel<T, true> : attention_diff_decode_kernel<T, false>;
  if (shared > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    if (err != cudaSuccess) return (int)err;
  }
  launch_kernel(kernel, dim3(count, args.heads), dim3(DECODE_WARPS * 32), shared, stream,
                (const T*)q, (const T*)k_pool, (const T*)v_pool, (T*)out, decode_seg, args);
  return launch_status();
}

inline int fill_args(DiffArgs& a, const int* seg_q_start, const int* seg_q_len, const int* seg_pos0,
                     const int* block_table, const int* seg_slot, int table_width, int heads, int kv_heads, int dim,
                     int vdim, int page_size, int window, int keep_first, float scale, float lambda, float eps,
                     float out_scale) {
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || dim <= 0 || vdim <= 0 || page_size <= 0 ||
      table_width <= 0 || keep_first < 0)
    return MLR_BAD_SIZE;
  if (2 * dim > MAX_QK || vdim > MAX_VDIM || heads > 65535) return MLR_TOO_LARGE;
  a.seg_q_start = seg_q_start; a.seg_q_len = seg_q_len; a.seg_pos0 = seg_pos0; a.block_table = block_table;
  a.seg_slot = seg_slot; a.table_width = table_width; a.heads = heads; a.kv_heads = kv_heads; a.dim = dim;
  a.vdim = vdim; a.page_size = page_size; a.window = window; a.keep_first = keep_first; a.scale = scale;
  a.lambda = lambda; a.eps = eps; a.out_scale = out_scale;
  return MLR_OK;
}

}  // namespace mlr

using namespace mlr;

MLR_DEFINE_PDL_SWITCH

// qkv: float32 [rows, 2*heads*dim + 2*kv_heads*dim + kv_heads*vdim]; q_out: dtype [rows, 2*heads*dim];
// k_pool: dtype [pages, kv_heads, page_size, 2*dim]; v_pool: dtype [pages, kv_heads, page_size, vdim];
// slots: int64 [rows], page * page_size + offset of every row's key and value.
MLR_EXPORT int mlr_qk_norm_kv_write(const float* qkv, const float* q_weight, const float* k_weight,
                                    const long long* slots, void* q_out, void* k_pool, void* v_pool, int rows,
                                    int heads, int kv_heads, int dim, int vdim, int page_size, float eps,
                                    int write_kv, int dtype, cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || heads <= 0 || kv_heads <= 0 || dim <= 0 || vdim <= 0 || page_size <= 0) return MLR_BAD_SIZE;
  const long long items = (long long)rows * (2 * heads + 3 * kv_heads);
  const long long blocks = (items + 3) / 4;
  if (blocks > 0x7fffffffLL) return MLR_TOO_LARGE;
  if (dtype == MLR_F32)
    launch_kernel(qk_norm_kv_write_kernel<float>, dim3((unsigned)blocks), dim3(128), 0, stream, qkv, q_weight, k_weight,
                  slots, (float*)q_out, (float*)k_pool, (float*)v_pool, rows, heads, kv_heads, dim, vdim, page_size,
                  eps, write_kv);
  else if (dtype == MLR_BF16)
    launch_kernel(qk_norm_kv_write_kernel<bf16>, dim3((unsigned)blocks), dim3(128), 0, stream, qkv, q_weight, k_weight,
                  slots, (bf16*)q_out, (bf16*)k_pool, (bf16*)v_pool, rows, heads, kv_heads, dim, vdim, page_size, eps,
                  write_kv);
  else
    return MLR_BAD_DTYPE;
  return launch_status();
}

// q: [rows, heads, 2*dim]; out: [rows, heads, vdim]; tile_seg/tile_row0: one entry per CTA tile of up
// to 16 rows of one segment.
MLR_EXPORT int mlr_attention_diff(const void* q, const void* k_pool, const void* v_pool, void* out,
                                  const int* tile_seg, const int* tile_row0, const int* seg_q_start,
                                  const int* seg_q_len, const int* seg_pos0, const int* block_table,
                                  const int* seg_slot, int table_width, int tiles, int heads, int kv_heads, int dim,
                                  int vdim, int page_size, int window, int keep_first, float scale, float lambda,
                                  float eps, float out_scale, int dtype, cudaStream_t stream) {
  if (tiles == 0) return MLR_OK;
  if (tiles < 0) return MLR_BAD_SIZE;
  DiffArgs args;
  int status = fill_args(args, seg_q_start, seg_q_len, seg_pos0, block_table, seg_slot, table_width, heads, kv_heads,
                         dim, vdim, page_size, window, keep_first, scale, lambda, eps, out_scale);
  if (status != MLR_OK) return status;
  if (dtype == MLR_F32) return attention_diff_launch<float>(q, k_pool, v_pool, out, tile_seg, tile_row0, tiles, args, stream);
  if (dtype == MLR_BF16) return attention_diff_launch<bf16>(q, k_pool, v_pool, out, tile_seg, tile_row0, tiles, args, stream);
  return MLR_BAD_DTYPE;
}

// The same for segments of one row each: decode_seg lists them (null: segments 0 .. count-1).
MLR_EXPORT int mlr_attention_diff_decode(const void* q, const void* k_pool, const void* v_pool, void* out,
                                         const int* decode_seg, int count, const int* seg_q_start,
                                         const int* seg_pos0, const int* block_table, const int* seg_slot,
                                         int table_width, int heads, int kv_heads, int dim, int vdim, int page_size,
                                         int window, int keep_first, float scale, float lambda, float eps,
                                         float out_scale, int dtype, cudaStream_t stream) {
  if (count == 0) return MLR_OK;
  if (count < 0) return MLR_BAD_SIZE;
  DiffArgs args;
  int status = fill_args(args, seg_q_start, nullptr, seg_pos0, block_table, seg_slot, table_width, heads, kv_heads,
                         dim, vdim, page_size, window, keep_first, scale, lambda, eps, out_scale);
  if (status != MLR_OK) return status;
  if (dtype == MLR_F32) return attention_diff_decode_launch<float>(q, k_pool, v_pool, out, decode_seg, count, args, stream);
  if (dtype == MLR_BF16) return attention_diff_decode_launch<bf16>(q, k_pool, v_pool, out, decode_seg, count, args, stream);
  return MLR_BAD_DTYPE;
}
