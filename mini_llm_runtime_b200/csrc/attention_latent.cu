// Latent attention over the paged cache.
//
// Keys and values of all heads are made from one low-rank latent c [rank] per token, and the keys
// carry one more part r [rot] that is turned by the token's position and shared by all heads:
//
//     score(i, j, h) = (q_plain[i,h] . (Wuk[h] c_j)  +  q_turned[i,h] . r_j) * scale
//     value(j, h)    = Wuv[h] c_j
//
// Since q . (Wuk c) = (Wuk^T q) . c and sum_j p_j (Wuv c_j) = Wuv (sum_j p_j c_j), the cache holds
// one row [c | r] per token (a single "kv head" of rank + rot numbers), queries are carried into
// the latent space before the attention ("absorbed": a [rank + rot] vector per head), the attention
// sums latents, and the per-head value matrix is applied afterwards.  All heads read the same rows.
//
// mlr_latent_prepare     RMS norms of the query latent and of c, rotation of r, cache write.
// mlr_head_linear        per-head matrix products on float32 rows (absorbing queries, applying the
//                        value matrix), optionally with the rotation of the query's turned part
//                        appended or with a sigmoid gate multiplied in.
// mlr_latent_attention   ragged batch of prompt portions and decoded rows, 16 query rows of one head per
//                        CTA; keys walked in tiles of 32 aligned to absolute positions, reductions in
//                        a fixed lane order, so a row's result depends on its own request's cache only.
//                        Causal, optionally a sliding window (key j visible from i iff 0 <= i - j < window)
//                        and a per-head sink: exp(sink) joins the softmax denominator, unscaled, once.
// mlr_latent_attention_decode   one CTA per (decoded row, head): warps take the key tiles in turn and
//                        their running states are merged in warp order.
//
// Scores, softmax, norms, angles and all sums are float32.
#include "common.cuh"

namespace mlr {

constexpr int ROWS_PER_TILE = 16;
constexpr int KEYS_PER_TILE = 32;
constexpr int MAX_RANK = 512;       // latent size the attention kernels hold in registers
constexpr int MAX_KEY = 1024;       // rank + rot

// One pair (u, v) of a vector turned by `angle`: (u cos - v sin, v cos + u sin).  `pairs` pairs cover
// the first 2 * pairs entries: pair i is (i, i + pairs) or, interleaved, (2i, 2i + 1).
__device__ __forceinline__ void pair_places(int i, int pairs, int interleaved, int* a, int* b) {
  *a = interleaved ? 2 * i : i;
  *b = interleaved ? 2 * i + 1 : i + pairs;
}

// ------------------------------------------------------------------ norms, rotation, cache write
// One CTA per row.  down: float32 [rows, down_stride]; columns [q_at, q_at + q_rank) hold the query
// latent, [c_at, c_at + rank) the key/value latent, the next `rot` the shared key part.
template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const float* down, long long down_stride, int q_at, int q_rank, int c_at, int rank, int rot,
                      const float* __restrict__ q_weight, const float* __restrict__ c_weight,
                      const int* positions, const float* __restrict__ frequencies, int pairs, int interleaved,
                      const long long* slots, T* __restrict__ q_latent, T* __restrict__ pool, float eps, int write) {
  pdl_trigger();
  __shared__ float scratch[32];
  const int row = blockIdx.x;
  // what does not depend on the product is asked for before the wait: the row's place and position, and
  // (into the L2) the norms' weights and the frequencies; both sums of squares are then taken in one
  // sweep, so that the kernel waits for memory three times instead of six
  const long long slot = write ? slots[row] : -1;
  const float position = (float)positions[row];
  for (int d = threadIdx.x * 32; d < q_rank; d += blockDim.x * 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(q_weight + d));
  for (int d = threadIdx.x * 32; d < rank; d += blockDim.x * 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(c_weight + d));
  if (threadIdx.x * 32 < pairs) asm volatile("prefetch.global.L2 [%0];" ::"l"(frequencies + threadIdx.x * 32));
  pdl_wait();
  const float* in = down + (size_t)row * down_stride;
  const bool store = write && slot >= 0;
  float sq_q = 0.f, sq_c = 0.f;
  for (int d = threadIdx.x; d < q_rank; d += blockDim.x) sq_q = fmaf(in[q_at + d], in[q_at + d], sq_q);
  if (store)
    for (int d = threadIdx.x; d < rank; d += blockDim.x) sq_c = fmaf(in[c_at + d], in[c_at + d], sq_c);
  {
    const float factor = 1.f / sqrtf(block_sum(sq_q, scratch) / (float)q_rank + eps);
    T* dst = q_latent + (size_t)row * q_rank;
    for (int d = threadIdx.x; d < q_rank; d += blockDim.x) dst[d] = from_float<T>(in[q_at + d] * factor * q_weight[d]);
  }
  if (!store) return;
  T* dst = pool + (size_t)slot * (rank + rot);
  const float factor = 1.f / sqrtf(block_sum(sq_c, scratch) / (float)rank + eps);
  for (int d = threadIdx.x; d < rank; d += blockDim.x) dst[d] = from_float<T>(in[c_at + d] * factor * c_weight[d]);
  const float* r = in + c_at + rank;
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    int a, b;
    pair_places(i, pairs, interleaved, &a, &b);
    float sine, cosine, ya, yb;
    sincosf(position * frequencies[i], &sine, &cosine);
    rotate_pair(r[a], r[b], sine, cosine, &ya, &yb);
    dst[rank + a] = from_float<T>(ya);
    dst[rank + b] = from_float<T>(yb);
  }
  for (int d = 2 * pairs + threadIdx.x; d < rot; d += blockDim.x) dst[rank + d] = from_float<T>(r[d]);
}

// ------------------------------------------------------------------ per-head products
// y[r, h, n] = sum_k x[r, h, k] * W_h[n, k] for h < heads, n < N, k < K, with float32 x
// (x[r, h, k] at x + r * x_row + h * x_head + k), W in the compute dtype laid out [heads][N][K]
// (KN = 0) or [heads][K][N] (KN = 1), y in TO at y + r * y_row + h * y_head + n.  Sums run over k in
// ascending order in float32.  Then, depending on `mode`:
//   1  the `tail` numbers after x's K are copied behind y's N with their first 2 * pairs entries turned
//      by the row's position (the turned part of an absorbed query);
//   2  y is multiplied by sigmoid(g), g = gate[r * gate_row + (gate_per_head ? h : h * N + n)].
struct HeadLinearArgs {
  const float* x; long long x_row; int x_head;
  long long y_row; int y_head;
  int rows, heads, N, K, kn, mode;
  int tail, pairs, interleaved;
  const int* positions; const float* frequencies;
  const float* gate; long long gate_row; int gate_per_head;
};

constexpr int HL_BM = 32, HL_BN = 64, HL_BK = 16;

template <typename T, typename TO>
__global__ void __launch_bounds__(128)
head_linear_kernel(const T* __restrict__ w, TO* __restrict__ y, HeadLinearArgs p) {
  pdl_trigger();
  __shared__ float xs[HL_BK][HL_BM + 1];
  __shared__ float ws[HL_BK][HL_BN + 1];
  const int head = blockIdx.z, row0 = blockIdx.y * HL_BM, n0 = blockIdx.x * HL_BN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;       // 16 x 8 threads: 4 columns x 4 rows each
  const T* wh = w + (size_t)head * p.N * p.K;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  pdl_wait();
  for (int k0 = 0; k0 < p.K; k0 += HL_BK) {
    for (int idx = threadIdx.x; idx < HL_BM * HL_BK; idx += 128) {
      const int r = idx / HL_BK, k = idx - r * HL_BK;
      const int row = row0 + r;
      xs[k][r] = (row < p.rows && k0 + k < p.K)
                     ? p.x[(size_t)row * p.x_row + (size_t)head * p.x_head + k0 + k] : 0.f;
    }
    if (p.kn) {
      for (int idx = threadIdx.x; idx < HL_BN * HL_BK; idx += 128) {
        const int k = idx / HL_BN, n = idx - k * HL_BN;
        ws[k][n] = (n0 + n < p.N && k0 + k < p.K) ? to_float(wh[(size_t)(k0 + k) * p.N + n0 + n]) : 0.f;
      }
    } else {
      for (int idx = threadIdx.x; idx < HL_BN * HL_BK; idx += 128) {
        const int n = idx / HL_BK, k = idx - n * HL_BK;
        ws[k][n] = (n0 + n < p.N && k0 + k < p.K) ? to_float(wh[(size_t)(n0 + n) * p.K + k0 + k]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < HL_BK; ++k) {
      float xv[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) xv[i] = xs[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = ws[k][tx + 16 * j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = row0 + ty * 4 + i;
    if (row >= p.rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx + 16 * j;
      if (n >= p.N) continue;
      float v = acc[i][j];
      if (p.mode == 2) {
        const float g = p.gate[(size_t)row * p.gate_row + (p.gate_per_head ? head : head * p.N + n)];
        v = v / (1.f + expf(-g));
      }
      y[(size_t)row * p.y_row + (size_t)head * p.y_head + n] = from_float<TO>(v);
    }
  }
  if (p.mode == 1 && blockIdx.x == 0) {
    for (int idx = threadIdx.x; idx < HL_BM * p.tail; idx += 128) {
      const int r = idx / p.tail, d = idx - r * p.tail;
      const int row = row0 + r;
      if (row >= p.rows) continue;
      const float* src = p.x + (size_t)row * p.x_row + (size_t)head * p.x_head + p.K;
      TO* dst = y + (size_t)row * p.y_row + (size_t)head * p.y_head + p.N;
      if (d >= 2 * p.pairs) {
        dst[d] = from_float<TO>(src[d]);
      } else {
        // entry d belongs to pair i as its first or second member
        int i, second;
        if (p.interleaved) { i = d >> 1; second = d & 1; }
        else { second = d >= p.pairs; i = second ? d - p.pairs : d; }
        int a, b;
        pair_places(i, p.pairs, p.interleaved, &a, &b);
        float sine, cosine, ya, yb;
        sincosf((float)p.positions[row] * p.frequencies[i], &sine, &cosine);
        rotate_pair(src[a], src[b], sine, cosine, &ya, &yb);
        dst[d] = from_float<TO>(second ? yb : ya);
      }
    }
  }
}

// ------------------------------------------------------------------ attention
struct LatentArgs {
  const int *seg_q_start, *seg_q_len, *seg_pos0, *block_table, *seg_slot;
  int table_width, heads, rank, rot, page_size, window;
  float scale;
  const float* sink;      // [heads] or null
};

__device__ __forceinline__ bool key_visible(int key, int p, int window) {
  return key <= p && (window <= 0 || p - key < window);
}

// q: [rows, heads, rank + rot]; pool: [pages * page_size, rank + rot]; out: float32 [rows, heads, rank].
template <typename T>
__global__ void __launch_bounds__(128)
latent_attention_kernel(const T* q, const T* pool, float* __restrict__ out, const int* __restrict__ tile_seg,
                        const int* __restrict__ tile_row0, LatentArgs p) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float shared[];
  const int DK = p.rank + p.rot, R = p.rank;
  float* q_rows = shared;                                  // [16][DK]
  float* k_tile = q_rows + ROWS_PER_TILE * DK;             // [32][DK + 1]
  float* p_tile = k_tile + KEYS_PER_TILE * (DK + 1);       // [16][32]

  const int tile = blockIdx.x, head = blockIdx.y;
  const int seg = tile_seg[tile], row0 = tile_row0[tile];
  const int q_start = p.seg_q_start[seg], q_len = p.seg_q_len[seg], pos0 = p.seg_pos0[seg];
  const int rows = min(ROWS_PER_TILE, q_len - row0);
  const int* table = p.block_table + (size_t)p.seg_slot[seg] * p.table_width;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  for (int idx = threadIdx.x; idx < ROWS_PER_TILE * DK; idx += blockDim.x) {
    const int r = idx / DK, d = idx - r * DK;
    q_rows[idx] = r < rows ? to_float(q[((size_t)(q_start + row0 + r) * p.heads + head) * DK + d]) : 0.f;
  }

  float m[4], l[4], acc[4][MAX_RANK / 32];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int c = 0; c < MAX_RANK / 32; ++c) acc[i][c] = 0.f;
  }

  const int first_pos = pos0 + row0, last_pos = pos0 + row0 + rows - 1;
  const int lowest_key = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
  for (int k0 = (lowest_key / KEYS_PER_TILE) * KEYS_PER_TILE; k0 <= last_pos; k0 += KEYS_PER_TILE) {
    __syncthreads();
    for (int idx = threadIdx.x; idx < KEYS_PER_TILE * DK; idx += blockDim.x) {
      const int j = idx / DK, d = idx - j * DK;
      const int key = k0 + j;
      float kv = 0.f;
      if (key <= last_pos) {
        const int page = table[key / p.page_size];
        if (page >= 0) kv = to_float(pool[((size_t)page * p.page_size + key % p.page_size) * DK + d]);
      }
      k_tile[j * (DK + 1) + d] = kv;
    }
    __syncthreads();

    const int key = k0 + lane;
    const int r0 = warp * 4;
    if (r0 >= rows) continue;     // uniform per warp; the barriers above are reached by all
    // this lane's key against the warp's four rows
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    {
      const float* kr = k_tile + lane * (DK + 1);
      const float* qr = q_rows + r0 * DK;
      for (int d = 0; d < DK; ++d) {
        const float kv = kr[d];
#pragma unroll
        for (int i = 0; i < 4; ++i) s[i] = fmaf(qr[i * DK + d], kv, s[i]);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = r0 + i;
      if (r >= rows) continue;
      const bool visible = key_visible(key, first_pos + r, p.window);
      const float score = visible ? s[i] * p.scale : -INFINITY;
      const float m_new = fmaxf(m[i], warp_max(score));
      if (m_new == -INFINITY) continue;         // no visible key yet for this row (uniform per warp)
      const float alpha = expf(m[i] - m_new);   // m = -inf gives 0
      const float prob = visible ? expf(score - m_new) : 0.f;
      l[i] = l[i] * alpha + warp_sum(prob);
      m[i] = m_new;
      float* pr = p_tile + r * KEYS_PER_TILE;
      pr[lane] = prob;
      __syncwarp();
#pragma unroll
      for (int c = 0; c < MAX_RANK / 32; ++c) {
        const int d = lane + 32 * c;
        if (d < R) {
          float a = acc[i][c] * alpha;
          for (int j = 0; j < KEYS_PER_TILE; ++j) a = fmaf(pr[j], k_tile[j * (DK + 1) + d], a);
          acc[i][c] = a;
        }
      }
      __syncwarp();
    }
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = warp * 4 + i;
    if (r >= rows) continue;
    float scale_acc = 1.f, total = l[i];
    if (p.sink != nullptr) {
      const float sink = p.sink[head];
      const float top = fmaxf(m[i], sink);
      scale_acc = expf(m[i] - top);
      total = l[i] * scale_acc + expf(sink - top);
    }
    const float factor = scale_acc / total;
    float* dst = out + ((size_t)(q_start + row0 + r) * p.heads + head) * R;
#pragma unroll
    for (int c = 0; c < MAX_RANK / 32; ++c) {
      const int d = lane + 32 * c;
      if (d < R) dst[d] = acc[i][c] * factor;
    }
  }
}

// q . k over n entries, q in shared memory as floats, k a row of the pool.
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
// One CTA of DECODE_WARPS warps per (segment of one row, group of HEADS_PER_CTA heads).  Warp w takes
// the visible key tiles number w, w + DECODE_WARPS, ..; each lane scores one key of a tile against
// every head of the group (the key row is read once for all of them), then each lane sums its latent
// channels over the tile's keys.  The warps' running states are merged in warp order.
constexpr int DECODE_WARPS = 16;
constexpr int HEADS_PER_CTA = 4;
constexpr int DECODE_MAX_RANK = 512;

template <typename T>
__global__ void __launch_bounds__(DECODE_WARPS * 32)
latent_attention_decode_kernel(const T* q, const T* pool, float* __restrict__ out, const int* __restrict__ decode_seg,
                               LatentArgs p) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) float shared[];
  const int DK = p.rank + p.rot, R = p.rank;
  float* q_rows = shared;                                               // [HEADS_PER_CTA][DK]
  float* probs = q_rows + HEADS_PER_CTA * DK;                           // [warps][HEADS_PER_CTA][32]
  float* merged = probs + DECODE_WARPS * HEADS_PER_CTA * KEYS_PER_TILE; // [warps][HEADS_PER_CTA][R + 2]
  long long* places = reinterpret_cast<long long*>(merged + (size_t)DECODE_WARPS * HEADS_PER_CTA * (R + 2) + 2);
  places = reinterpret_cast<long long*>((reinterpret_cast<uintptr_t>(places) + 7) & ~(uintptr_t)7);   // [warps][32]
  const int seg = decode_seg != nullptr ? decode_seg[blockIdx.x] : blockIdx.x;
  const int head0 = blockIdx.y * HEADS_PER_CTA;
  const int group = min(HEADS_PER_CTA, p.heads - head0);
  const int row = p.seg_q_start[seg], pos = p.seg_pos0[seg];
  const int* table = p.block_table + (size_t)p.seg_slot[seg] * p.table_width;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  for (int idx = threadIdx.x; idx < HEADS_PER_CTA * DK; idx += blockDim.x) {
    const int g = idx / DK, d = idx - g * DK;
    q_rows[idx] = g < group ? to_float(q[((size_t)row * p.heads + head0 + g) * DK + d]) : 0.f;
  }
  __syncthreads();

  float m[HEADS_PER_CTA], l[HEADS_PER_CTA], acc[HEADS_PER_CTA][DECODE_MAX_RANK / 32];
#pragma unroll
  for (int g = 0; g < HEADS_PER_CTA; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int c = 0; c < DECODE_MAX_RANK / 32; ++c) acc[g][c] = 0.f;
  }
  const int lowest = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  const int total = pos - lowest + 1;
  float* pw = probs + warp * HEADS_PER_CTA * KEYS_PER_TILE;
  long long* place = places + warp * KEYS_PER_TILE;
  for (int t0 = warp * KEYS_PER_TILE; t0 < total; t0 += DECODE_WARPS * KEYS_PER_TILE) {
    const int entry = t0 + lane;
    long long at = -1;
    if (entry < total) {
      const int key = lowest + entry;
      const int page = table[key / p.page_size];
      if (page >= 0) at = (long long)page * p.page_size + key % p.page_size;
    }
    place[lane] = at;
    float alpha[HEADS_PER_CTA];
#pragma unroll
    for (int g = 0; g < HEADS_PER_CTA; ++g) {
      alpha[g] = 1.f;
      float prob = 0.f;
      if (g < group) {
        const float s = at >= 0 ? dot_row(q_rows + g * DK, pool + at * DK, DK) * p.scale : -INFINITY;
        const float m_new = fmaxf(m[g], warp_max(s));
        if (m_new != -INFINITY) {
          alpha[g] = expf(m[g] - m_new);
          prob = at >= 0 ? expf(s - m_new) : 0.f;
          l[g] = l[g] * alpha[g] + warp_sum(prob);
          m[g] = m_new;
        }
      }
      pw[g * KEYS_PER_TILE + lane] = prob;
    }
    __syncwarp();
    const int count = min(KEYS_PER_TILE, total - t0);
#pragma unroll
    for (int c = 0; c < DECODE_MAX_RANK / 32; ++c) {
      const int d = lane + 32 * c;
      if (d < R) {
        float a[HEADS_PER_CTA];
#pragma unroll
        for (int g = 0; g < HEADS_PER_CTA; ++g) a[g] = acc[g][c] * alpha[g];
#pragma unroll 8
        for (int j = 0; j < KEYS_PER_TILE; ++j) {
          // a key without a page (or beyond the tile's end) has probability 0: its load is pointed at
          // row 0 of the pool and adds nothing, so that the loads of a tile can be in flight at once
          const long long row_at = j < count ? max(place[j], 0LL) : 0LL;
          const float vv = to_float(pool[row_at * DK + d]);
#pragma unroll
          for (int g = 0; g < HEADS_PER_CTA; ++g) a[g] = fmaf(pw[g * KEYS_PER_TILE + j], vv, a[g]);
        }
#pragma unroll
        for (int g = 0; g < HEADS_PER_CTA; ++g) acc[g][c] = a[g];
      }
    }
    __syncwarp();
  }
#pragma unroll
  for (int g = 0; g < HEADS_PER_CTA; ++g) {
    float* mine = merged + (size_t)(warp * HEADS_PER_CTA + g) * (R + 2);
    if (lane == 0) {
      mine[R] = m[g];
      mine[R + 1] = l[g];
    }
#pragma unroll
    for (int c = 0; c < DECODE_MAX_RANK / 32; ++c) {
      const int d = lane + 32 * c;
      if (d < R) mine[d] = acc[g][c];
    }
  }
  __syncthreads();
  // warp g merges head g of the group, walking the warps' states in warp order
  if (warp >= group) return;
  const int g = warp, head = head0 + g;
  float top = -INFINITY;
  for (int w = 0; w < DECODE_WARPS; ++w) top = fmaxf(top, merged[(size_t)(w * HEADS_PER_CTA + g) * (R + 2) + R]);
  const bool has_sink = p.sink != nullptr;
  const float sink = has_sink ? p.sink[head] : 0.f;
  if (has_sink) top = fmaxf(top, sink);
  float sum = 0.f, part[DECODE_MAX_RANK / 32];
#pragma unroll
  for (int c = 0; c < DECODE_MAX_RANK / 32; ++c) part[c] = 0.f;
  for (int w = 0; w < DECODE_WARPS; ++w) {
    const float* theirs = merged + (size_t)(w * HEADS_PER_CTA + g) * (R + 2);
    if (theirs[R] == -INFINITY) continue;
    const float f = expf(theirs[R] - top);
    sum = fmaf(theirs[R + 1], f, sum);
#pragma unroll
    for (int c = 0; c < DECODE_MAX_RANK / 32; ++c) {
      const int d = lane + 32 * c;
      if (d < R) part[c] = fmaf(theirs[d], f, part[c]);
    }
  }
  if (has_sink) sum += expf(sink - top);
  const float inv = 1.f / sum;
  float* dst = out + ((size_t)row * p.heads + head) * R;
#pragma unroll
  for (int c = 0; c < DECODE_MAX_RANK / 32; ++c) {
    const int d = lane + 32 * c;
    if (d < R) dst[d] = part[c] * inv;
  }
}

inline int fill_args(LatentArgs& a, const int* seg_q_start, const int* seg_q_len, const int* seg_pos0,
                     const int* block_table, const int* seg_slot, int table_width, int heads, int rank, int rot,
                     int page_size, int window, float scale, const float* sink) {
  if (heads <= 0 || rank <= 0 || rot < 0 || page_size <= 0 || table_width <= 0) return MLR_BAD_SIZE;
  if (rank > MAX_RANK || rank + rot > MAX_KEY || heads > 65535) return MLR_TOO_LARGE;
  a.seg_q_start = seg_q_start; a.seg_q_len = seg_q_len; a.seg_pos0 = seg_pos0; a.block_table = block_table;
  a.seg_slot = seg_slot; a.table_width = table_width; a.heads = heads; a.rank = rank; a.rot = rot;
  a.page_size = page_size; a.window = window; a.scale = scale; a.sink = sink;
  return MLR_OK;
}

template <typename T>
int latent_attention_launch(const void* q, const void* pool, float* out, const int* tile_seg, const int* tile_row0,
                            int tiles, const LatentArgs& args, cudaStream_t stream) {
  const int DK = args.rank + args.rot;
  const size_t shared = sizeof(float) * ((size_t)ROWS_PER_TILE * DK + (size_t)KEYS_PER_TILE * (DK + 1) +
                                         (size_t)ROWS_PER_TILE * KEYS_PER_TILE);
  if (shared > 200 * 1024) return MLR_TOO_LARGE;
  if (shared > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(latent_attention_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    if (err != cudaSuccess) return (int)err;
  }
  launch_kernel(latent_attention_kernel<T>, dim3(tiles, args.heads), dim3(128), shared, stream, (const T*)q,
                (const T*)pool, out, tile_seg, tile_row0, args);
  return launch_status();
}

template <typename T>
int latent_decode_launch(const void* q, const void* pool, float* out, const int* decode_seg, int count,
                         const LatentArgs& args, cudaStream_t stream) {
  const int DK = args.rank + args.rot;
  const size_t shared = sizeof(float) * ((size_t)HEADS_PER_CTA * DK + (size_t)DECODE_WARPS * HEADS_PER_CTA * KEYS_PER_TILE +
                                         (size_t)DECODE_WARPS * HEADS_PER_CTA * (args.rank + 2) + 4) +
                        sizeof(long long) * DECODE_WARPS * KEYS_PER_TILE + 8;
  if (shared > 200 * 1024) return MLR_TOO_LARGE;
  if (shared > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(latent_attention_decode_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    if (err != cudaSuccess) return (int)err;
  }
  launch_kernel(latent_attention_decode_kernel<T>, dim3(count, (args.heads + HEADS_PER_CTA - 1) / HEADS_PER_CTA),
                dim3(DECODE_WARPS * 32), shared, stream, (const T*)q, (const T*)pool, out, decode_seg, args);
  return launch_status();
}

}  // namespace mlr

using namespace mlr;

MLR_DEFINE_PDL_SWITCH

// down: float32 [rows, down_stride] (a product's output; see the kernel for the column ranges);
// q_latent: dtype [rows, q_rank]; pool: dtype [pages, 1, page_size, rank + rot]; slots: int64 [rows],
// page * page_size + offset of every row's cache entry; frequencies: float32 [pairs].
MLR_EXPORT int mlr_latent_prepare(const float* down, long long down_stride, int q_at, int q_rank, int c_at, int rank,
                                  int rot, const float* q_weight, const float* c_weight, const int* positions,
                                  const float* frequencies, int pairs, int interleaved, const long long* slots,
                                  void* q_latent, void* pool, int rows, float eps, int write, int dtype,
                                  cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || q_rank <= 0 || rank <= 0 || rot < 0 || pairs < 0 || 2 * pairs > rot) return MLR_BAD_SIZE;
  if (dtype == MLR_F32)
    launch_kernel(latent_prepare_kernel<float>, dim3(rows), dim3(128), 0, stream, down, down_stride, q_at, q_rank, c_at,
                  rank, rot, q_weight, c_weight, positions, frequencies, pairs, interleaved, slots, (float*)q_latent,
                  (float*)pool, eps, write);
  else if (dtype == MLR_BF16)
    launch_kernel(latent_prepare_kernel<bf16>, dim3(rows), dim3(128), 0, stream, down, down_stride, q_at, q_rank, c_at,
                  rank, rot, q_weight, c_weight, positions, frequencies, pairs, interleaved, slots, (bf16*)q_latent,
                  (bf16*)pool, eps, write);
  else
    return MLR_BAD_DTYPE;
  return launch_status();
}

// See HeadLinearArgs.  w_dtype: dtype of w; y_dtype: dtype of y.
MLR_EXPORT int mlr_head_linear(const float* x, long long x_row, int x_head, const void* w, void* y, long long y_row,
                               int y_head, int rows, int heads, int N, int K, int kn, int mode, int tail, int pairs,
                               int interleaved, const int* positions, const float* frequencies, const float* gate,
                               long long gate_row, int gate_per_head, int w_dtype, int y_dtype, cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || heads <= 0 || N <= 0 || K <= 0 || tail < 0 || pairs < 0 || 2 * pairs > tail) return MLR_BAD_SIZE;
  if (heads > 65535 || (rows + HL_BM - 1) / HL_BM > 65535) return MLR_TOO_LARGE;
  if (mode == 1 && tail > 0 && pairs > 0 && (positions == nullptr || frequencies == nullptr)) return MLR_BAD_SIZE;
  if (mode == 2 && gate == nullptr) return MLR_BAD_SIZE;
  HeadLinearArgs p;
  p.x = x; p.x_row = x_row; p.x_head = x_head; p.y_row = y_row; p.y_head = y_head; p.rows = rows; p.heads = heads;
  p.N = N; p.K = K; p.kn = kn; p.mode = mode; p.tail = mode == 1 ? tail : 0; p.pairs = pairs; p.interleaved = interleaved;
  p.positions = positions; p.frequencies = frequencies; p.gate = gate; p.gate_row = gate_row; p.gate_per_head = gate_per_head;
  const dim3 grid((N + HL_BN - 1) / HL_BN, (rows + HL_BM - 1) / HL_BM, heads);
  if (w_dtype == MLR_F32 && y_dtype == MLR_F32)
    launch_kernel(head_linear_kernel<float, float>, grid, dim3(128), 0, stream, (const float*)w, (float*)y, p);
  else if (w_dtype == MLR_BF16 && y_dtype == MLR_BF16)
    launch_kernel(head_linear_kernel<bf16, bf16>, grid, dim3(128), 0, stream, (const bf16*)w, (bf16*)y, p);
  else if (w_dtype == MLR_BF16 && y_dtype == MLR_F32)
    launch_kernel(head_linear_kernel<bf16, float>, grid, dim3(128), 0, stream, (const bf16*)w, (float*)y, p);
  else
    return MLR_BAD_DTYPE;
  return launch_status();
}

// q: dtype [rows, heads, rank + rot]; pool: dtype [pages, 1, page_size, rank + rot]; out: float32
// [rows, heads, rank]; tile_seg/tile_row0: one entry per CTA tile of up to 16 rows of one segment;
// sink: float32 [heads] or null; window <= 0: every earlier key is visible.
MLR_EXPORT int mlr_latent_attention(const void* q, const void* pool, float* out, const int* tile_seg,
                                    const int* tile_row0, const int* seg_q_start, const int* seg_q_len,
                                    const int* seg_pos0, const int* block_table, const int* seg_slot, int table_width,
                                    int tiles, int heads, int rank, int rot, int page_size, int window, float scale,
                                    const float* sink, int dtype, cudaStream_t stream) {
  if (tiles == 0) return MLR_OK;
  if (tiles < 0) return MLR_BAD_SIZE;
  LatentArgs args;
  int status = fill_args(args, seg_q_start, seg_q_len, seg_pos0, block_table, seg_slot, table_width, heads, rank, rot,
                         page_size, window, scale, sink);
  if (status != MLR_OK) return status;
  if (dtype == MLR_F32) return latent_attention_launch<float>(q, pool, out, tile_seg, tile_row0, tiles, args, stream);
  if (dtype == MLR_BF16) return latent_attention_launch<bf16>(q, pool, out, tile_seg, tile_row0, tiles, args, stream);
  return MLR_BAD_DTYPE;
}

// The same for segments of one row each: decode_seg lists them (null: segments 0 .. count-1).
MLR_EXPORT int mlr_latent_attention_decode(const void* q, const void* pool, float* out, const int* decode_seg,
                                           int count, const int* seg_q_start, const int* seg_pos0,
                                           const int* block_table, const int* seg_slot, int table_width, int heads,
                                           int rank, int rot, int page_size, int window, float scale, const float* sink,
                                           int dtype, cudaStream_t stream) {
  if (count == 0) return MLR_OK;
  if (count < 0) return MLR_BAD_SIZE;
  LatentArgs args;
  int status = fill_args(args, seg_q_start, nullptr, seg_pos0, block_table, seg_slot, table_width, heads, rank, rot,
                         page_size, window, scale, sink);
  if (status != MLR_OK) return status;
  if (rank > DECODE_MAX_RANK) return MLR_TOO_LARGE;
  if (dtype == MLR_F32) return latent_decode_launch<float>(q, pool, out, decode_seg, count, args, stream);
  if (dtype == MLR_BF16) return latent_decode_launch<bf16>(q, pool, out, decode_seg, count, args, stream);
  return MLR_BAD_DTYPE;
}
