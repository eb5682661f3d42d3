// Latent attention of prompt portions on the tensor cores (bfloat16, mma.sync m16n8k16).
//
// Absorbed form: every query row is [rank + rot] numbers per head, every cached row [latent | turned key
// part] is key and (its first `rank` numbers) value at once, shared by all heads.  A CTA takes 16
// tokens of one request and two heads: 32 query rows over the same key tiles.  Eight warps: four per
// head.  For a tile of 32 keys, each of a head's four warps scores 8 of the keys against the 16 rows
// (Q K^T over rank + rot), the four exchange their row maxima and row sums through shared memory and
// leave their probabilities there (bfloat16); then each warp multiplies the whole 16 x 32 probability
// tile with its own quarter of the value columns, which stay in its registers over all key tiles
// (FlashAttention-2 arithmetic: statistics and sums in float32).  Key tiles are double-buffered with
// asynchronous copies through the request's block table.
//
// Decoded rows (segments of one token) run through the same kernel with the roles of tokens and heads
// exchanged: the 16 rows of a warp group are 16 heads of the one token (all heads read the same cache
// rows, so the whole head group rides on one pass over the keys), and the keys of a request are cut
// into chunks, one CTA each; a CTA leaves its un-normalised sums with its running maximum and
// denominator in a scratch buffer and a second small kernel merges the chunks in chunk order.
//
// Causal, optionally a sliding window (key j visible from i iff 0 <= i - j < window) and a per-head
// sink whose exponential joins the softmax denominator.  Output: float32 [rows, heads, rank].
#include "mma_attention.cuh"

namespace mlr {

constexpr int LM_TOKENS = 16;      // tokens per CTA
constexpr int LM_SPLIT = 4;        // warps per head
constexpr int LM_KEYS = 32;        // keys per tile, 8 per warp
constexpr int LM_MAX_NT = 16;      // value column blocks of 8 per warp: rank <= 4 * 16 * 8
constexpr int LM_P_STRIDE = LM_KEYS + 8;

struct LatentMmaArgs {
  const int *seg_q_start, *seg_q_len, *seg_pos0, *block_table, *seg_slot;
  int table_width, heads, rank, rot, page_size, window;
  float scale_log2;
  const float* sink;
  int stages;                // key tiles in shared memory (2 .. 4): stages - 1 of them are on their way while one is used
  const int* decode_seg;     // decoded rows: the segments to take (null: segments 0, 1, ..)
  float* partial;            // decoded rows in several chunks: [item][chunk][head][rank + 2]
};

// Keys key0 .. key0 + 31 into a tile.  Lane l of every warp looks up the page of key key0 + l (32 keys,
// 32 lanes: all lookups of a tile are in flight together; one lookup after the other cost eight
// round trips per tile and warp); then each warp takes rows in turn and its lanes copy the row's 16-byte
// pieces.  Keys outside [key_lo, key_hi] or on pages the request does not hold become zeros.
__device__ __forceinline__ void load_key_tile(bf16* tile, int stride, const bf16* pool, const int* __restrict__ table,
                                              int key0, int key_lo, int key_hi, int page_size, int dk) {
  const int chunks = dk >> 3, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  long long my_row = -1;       // row of the pool that holds key key0 + lane
  {
    const int key = key0 + lane;
    if (key >= key_lo && key <= key_hi) {
      const int logical = key / page_size;
      const int page = table[logical];
      if (page >= 0) my_row = (long long)page * page_size + (key - logical * page_size);
    }
  }
  for (int r = threadIdx.x >> 5; r < LM_KEYS; r += warps) {
    const long long row = __shfl_sync(0xffffffffu, my_row, r);
    const bool valid = row >= 0;
    const bf16* src = pool + (valid ? row : 0) * dk;
    for (int c = lane; c < chunks; c += 32) cp_async_16(tile + r * stride + c * 8, src + c * 8, valid);
  }
}

__device__ __forceinline__ void cp_async_wait_pending(int pending) {
  if (pending <= 0) cp_async_wait<0>();
  else if (pending == 1) cp_async_wait<1>();
  else cp_async_wait<2>();
}

template <int G, bool DECODE>
__global__ void __launch_bounds__(G * LM_SPLIT * 32)
latent_mma_kernel(const bf16* q, const bf16* pool, float* __restrict__ out, const int* __restrict__ tile_seg,
                  const int* __restrict__ tile_row0, LatentMmaArgs p) {
  constexpr int LM_THREADS = G * LM_SPLIT * 32;
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(128) uint8_t latent_shared[];
  const int DK = p.rank + p.rot, S = DK + 8;          // padded row stride: S / 8 is odd, ldmatrix is conflict-free
  bf16* q_tile = reinterpret_cast<bf16*>(latent_shared);                 // [G groups][16][S]
  bf16* k_tiles = q_tile + G * LM_TOKENS * S;                            // stages x [32][S]
  bf16* p_tile = k_tiles + p.stages * LM_KEYS * S;                       // [G][16][LM_P_STRIDE]
  float* stat_max = reinterpret_cast<float*>(p_tile + G * LM_TOKENS * LM_P_STRIDE);   // [G][4][16]
  float* stat_sum = stat_max + G * LM_SPLIT * LM_TOKENS;                              // [G][4][16]

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int group = warp / LM_SPLIT, split = warp % LM_SPLIT;
  // prompt tile: a group is one head, its rows 16 tokens; decoded row: a group is 16 heads of the one token
  // prompt tiles are taken from the end of the list: within a portion the later rows walk more keys, and the
  // CTAs that run longest should start first
  const int listed = DECODE ? blockIdx.x : gridDim.x - 1 - blockIdx.x;
  const int seg = DECODE ? (p.decode_seg != nullptr ? p.decode_seg[listed] : listed) : tile_seg[listed];
  const int row0 = DECODE ? 0 : tile_row0[listed];
  const int head = DECODE ? (blockIdx.y * G + group) * LM_TOKENS : blockIdx.y * G + group;    // the group's (first) head
  const bool live = head < p.heads;
  const int q_start = p.seg_q_start[seg], pos0 = p.seg_pos0[seg];
  const int rows = DECODE ? 1 : min(LM_TOKENS, p.seg_q_len[seg] - row0);
  const int* table = p.block_table + (size_t)p.seg_slot[seg] * p.table_width;
  const int first_pos = pos0 + row0, last_pos = first_pos + rows - 1;
  const int lowest_key = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
  int first_tile = (lowest_key / LM_KEYS) * LM_KEYS, last_key = last_pos;
  if (DECODE && gridDim.z > 1) {
    // this CTA's chunk of the key tiles
    const int tiles = (last_pos - first_tile) / LM_KEYS + 1;
    const int per_chunk = (tiles + gridDim.z - 1) / gridDim.z;
    first_tile += blockIdx.z * per_chunk * LM_KEYS;
    last_key = min(last_pos, first_tile + per_chunk * LM_KEYS - 1);
  }
  const int chunks = DK >> 3;

  // queries of all groups, and the first key tile
  for (int item = threadIdx.x; item < G * LM_TOKENS * chunks; item += LM_THREADS) {
    const int r = item / chunks, c = item - r * chunks;
    const int g = r / LM_TOKENS, t = r - g * LM_TOKENS;
    const int h = DECODE ? (blockIdx.y * G + g) * LM_TOKENS + t : blockIdx.y * G + g;
    const bool valid = (DECODE || t < rows) && h < p.heads;
    const bf16* src = valid ? q + ((size_t)(q_start + row0 + (DECODE ? 0 : t)) * p.heads + h) * DK + c * 8 : q;
    cp_async_16(q_tile + r * S + c * 8, src, valid);
  }
  // the first stages - 1 key tiles are asked for at once (the queries travel with the first)
  for (int i = 0; i < p.stages - 1; ++i) {
    if (first_tile + i * LM_KEYS <= last_key)
      load_key_tile(k_tiles + i * LM_KEYS * S, S, pool, table, first_tile + i * LM_KEYS, lowest_key, last_key, p.page_size, DK);
    cp_async_commit();
  }

  // this warp's value column blocks of 8: [nt_lo, nt_hi)
  const int nt_total = p.rank >> 3;
  const int nt_lo = split * nt_total / LM_SPLIT, nt_count = (split + 1) * nt_total / LM_SPLIT - nt_lo;
  float o[LM_MAX_NT][4];
#pragma unroll
  for (int t = 0; t < LM_MAX_NT; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  const int r_lo = lane >> 2;                         // this thread's rows: r_lo and r_lo + 8
  const int pos_row[2] = {DECODE ? first_pos : first_pos + r_lo, DECODE ? first_pos : first_pos + r_lo + 8};
  const bf16* q_mine = q_tile + group * LM_TOKENS * S;
  bf16* p_mine = p_tile + group * LM_TOKENS * LM_P_STRIDE;
  float* max_mine = stat_max + group * LM_SPLIT * LM_TOKENS;
  float* sum_mine = stat_sum + group * LM_SPLIT * LM_TOKENS;

  int buffer = 0;
  for (int k0 = first_tile; k0 <= last_key; k0 += LM_KEYS, buffer = buffer + 1 == p.stages ? 0 : buffer + 1) {
    cp_async_wait_pending(p.stages - 2);
    __syncthreads();
    {
      // the tile stages - 1 ahead goes where the tile before this one lay
      const int ahead = k0 + (p.stages - 1) * LM_KEYS;
      const int into = buffer == 0 ? p.stages - 1 : buffer - 1;
      if (ahead <= last_key)
        load_key_tile(k_tiles + into * LM_KEYS * S, S, pool, table, ahead, lowest_key, last_key, p.page_size, DK);
      cp_async_commit();
    }
    const bf16* k_tile = k_tiles + buffer * LM_KEYS * S;

    // scores of this warp's 8 keys; two chains of sums, over the even and the odd 16-channel steps
    float s[4] = {0.f, 0.f, 0.f, 0.f}, s_odd[4] = {0.f, 0.f, 0.f, 0.f};
    const bf16* q_lane = q_mine + ((lane & 7) + ((lane >> 3) & 1) * 8) * S + (lane >> 4) * 8;
    const bf16* k_lane = k_tile + (split * 8 + (lane & 7)) * S;
#pragma unroll 2
    for (int ks = 0; ks < DK / 16; ks += 2) {
      uint32_t b[4], a[4], a_next[4];
      // keys split*8 .. +7, channel chunks 2*ks .. 2*ks+3 (the last two may lie past DK when DK/16 is odd)
      const int chunk = min(ks * 2 + (lane >> 3), chunks - 1);
      ldmatrix_x4(b, k_lane + chunk * 8);
      ldmatrix_x4(a, q_lane + ks * 16);
      const bool pair = ks + 1 < DK / 16;
      if (pair) ldmatrix_x4(a_next, q_lane + ks * 16 + 16);
      mma_bf16(s, a, b[0], b[1]);
      if (pair) mma_bf16(s_odd, a_next, b[2], b[3]);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) s[e] += s_odd[e];
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int key = k0 + split * 8 + (lane & 3) * 2 + (e & 1);
      const int i = e >> 1;
      const bool visible = key <= min(pos_row[i], last_key) && (p.window <= 0 || pos_row[i] - key < p.window);
      s[e] = visible ? s[e] * p.scale_log2 : -INFINITY;
      tile_max[i] = fmaxf(tile_max[i], s[e]);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      tile_max[i] = fmaxf(tile_max[i], __shfl_xor_sync(0xffffffffu, tile_max[i], 1));
      tile_max[i] = fmaxf(tile_max[i], __shfl_xor_sync(0xffffffffu, tile_max[i], 2));
      if ((lane & 3) == 0) max_mine[split * LM_TOKENS + r_lo + 8 * i] = tile_max[i];
    }
    __syncthreads();
    float alpha[2], base[2], part[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float m_new = m[i];
#pragma unroll
      for (int w = 0; w < LM_SPLIT; ++w) m_new = fmaxf(m_new, max_mine[w * LM_TOKENS + r_lo + 8 * i]);
      base[i] = m_new == -INFINITY ? 0.f : m_new;
      alpha[i] = exp2f(m[i] - base[i]);
      m[i] = m_new;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      s[e] = exp2f(s[e] - base[e >> 1]);
      part[e >> 1] += s[e];
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      part[i] += __shfl_xor_sync(0xffffffffu, part[i], 1);
      part[i] += __shfl_xor_sync(0xffffffffu, part[i], 2);
      if ((lane & 3) == 0) sum_mine[split * LM_TOKENS + r_lo + 8 * i] = part[i];
      *reinterpret_cast<uint32_t*>(p_mine + (r_lo + 8 * i) * LM_P_STRIDE + split * 8 + (lane & 3) * 2) =
          pack_bf16(s[2 * i], s[2 * i + 1]);
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float total = 0.f;
#pragma unroll
      for (int w = 0; w < LM_SPLIT; ++w) total += sum_mine[w * LM_TOKENS + r_lo + 8 * i];
      l[i] = l[i] * alpha[i] + total;
    }
    if (!live) continue;
#pragma unroll
    for (int t = 0; t < LM_MAX_NT; ++t) {
      o[t][0] *= alpha[0]; o[t][1] *= alpha[0];
      o[t][2] *= alpha[1]; o[t][3] *= alpha[1];
    }
    // O += P V over this warp's value columns
#pragma unroll
    for (int kk = 0; kk < LM_KEYS / 16; ++kk) {
      uint32_t a[4];
      ldmatrix_x4(a, p_mine + ((lane & 7) + ((lane >> 3) & 1) * 8) * LM_P_STRIDE + (kk * 2 + (lane >> 4)) * 8);
#pragma unroll
      for (int dp = 0; dp < LM_MAX_NT / 2; ++dp) {
        if (2 * dp < nt_count) {
          uint32_t b[4];
          const int key = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
          const int chunk = nt_lo + dp * 2 + (lane >> 4);
          ldmatrix_x4_trans(b, k_tile + key * S + chunk * 8);
          mma_bf16(o[2 * dp], a, b[0], b[1]);
          if (2 * dp + 1 < nt_count) mma_bf16(o[2 * dp + 1], a, b[2], b[3]);
        }
      }
    }
  }
  cp_async_wait<0>();
  if (!live) return;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = r_lo + 8 * i;
    const int row_head = DECODE ? head + r : head;
    if (DECODE ? row_head >= p.heads : r >= rows) continue;
    const size_t token = (size_t)(q_start + row0 + (DECODE ? 0 : r));
    if (DECODE && gridDim.z > 1) {
      // un-normalised sums, running maximum (log2 domain) and denominator of this chunk
      float* dst = p.partial + (((size_t)blockIdx.x * gridDim.z + blockIdx.z) * p.heads + row_head) * (p.rank + 2);
      if (split == 0 && (lane & 3) == 0) {
        dst[p.rank] = m[i];
        dst[p.rank + 1] = l[i];
      }
#pragma unroll
      for (int t = 0; t < LM_MAX_NT; ++t) {
        if (t < nt_count) {
          dst[(nt_lo + t) * 8 + (lane & 3) * 2] = o[t][2 * i];
          dst[(nt_lo + t) * 8 + (lane & 3) * 2 + 1] = o[t][2 * i + 1];
        }
      }
      continue;
    }
    float factor = 1.f / l[i];
    if (p.sink != nullptr) {
      const float sink_log2 = p.sink[row_head] * 1.4426950408889634f;
      const float top = fmaxf(m[i], sink_log2);
      const float f = exp2f(m[i] - top);
      factor = f / (l[i] * f + exp2f(sink_log2 - top));
    }
    float* dst = out + (token * p.heads + row_head) * p.rank + nt_lo * 8 + (lane & 3) * 2;
#pragma unroll
    for (int t = 0; t < LM_MAX_NT; ++t) {
      if (t < nt_count) {
        dst[t * 8] = o[t][2 * i] * factor;
        dst[t * 8 + 1] = o[t][2 * i + 1] * factor;
      }
    }
  }
}

// Chunks of a decoded row merged: one CTA per (item, head).  Warp 0 turns the chunks' maxima and
// denominators into one factor per chunk; then every thread sums its four columns over the chunks in
// chunk order, eight chunks' loads in flight at a time.
__global__ void __launch_bounds__(128)
latent_merge_kernel(const float* partial, float* __restrict__ out, const int* __restrict__ decode_seg,
                    const int* __restrict__ seg_q_start, const float* __restrict__ sink, int items, int chunks, int heads,
                    int rank) {
  pdl_trigger();
  __shared__ float factor[32];
  const int item = blockIdx.x / heads, head = blockIdx.x - item * heads;
  const int seg = decode_seg != nullptr ? decode_seg[item] : item;
  const int lane = threadIdx.x & 31;
  pdl_wait();
  const float* mine = partial + ((size_t)item * chunks * heads + head) * (rank + 2);
  const size_t step = (size_t)heads * (rank + 2);
  if (threadIdx.x < 32) {
    const float sink_log2 = sink != nullptr ? sink[head] * 1.4426950408889634f : -INFINITY;
    const float my_max = lane < chunks ? __ldcg(mine + lane * step + rank) : -INFINITY;
    const float my_sum = lane < chunks ? __ldcg(mine + lane * step + rank + 1) : 0.f;
    const float top = fmaxf(warp_max(my_max), sink_log2);
    const float my_factor = my_max == -INFINITY ? 0.f : exp2f(my_max - top);
    float total = warp_sum(my_sum * my_factor);
    if (sink != nullptr) total += exp2f(sink_log2 - top);
    factor[lane] = my_factor / total;
  }
  __syncthreads();
  float* dst = out + ((size_t)seg_q_start[seg] * heads + head) * rank;
  for (int d = threadIdx.x * 2; d < rank; d += 256) {       // rank + 2 is even: pairs of columns are 8-byte aligned
    float2 sum = make_float2(0.f, 0.f);
#pragma unroll 8
    for (int c = 0; c < chunks; ++c) {
      const float2 v = __ldcg(reinterpret_cast<const float2*>(mine + c * step + d));
      sum.x = fmaf(v.x, factor[c], sum.x);
      sum.y = fmaf(v.y, factor[c], sum.y);
    }
    *reinterpret_cast<float2*>(dst + d) = sum;
  }
}

// ------------------------------------------------------------------ per-head products on the tensor cores
// y[r, h, n] = sum_k x[r, h, k] * W_h[n, k]: float32 x rounded to bfloat16 on its way into shared memory,
// bfloat16 W laid out [heads][N][K] (kn = 0) or [heads][K][N] (kn = 1), float32 sums.  A CTA of four
// warps takes 64 rows x 64 columns of one head, 32 of k at a time; each warp 16 rows.  mode 1 appends
// the `tail` numbers after x's K behind y's N with their first 2 * pairs entries turned by the row's
// position; mode 2 multiplies y by sigmoid(gate).  K and N multiples of 8, x 16-byte aligned pieces.
struct HeadMmaArgs {
  const float* x; long long x_row; int x_head;
  long long y_row; int y_head;
  int rows, heads, N, K, kn, mode;
  int tail, pairs, interleaved;
  const int* positions; const float* frequencies;
  const float* gate; long long gate_row; int gate_per_head;
};

constexpr int HM_COLS = 64;

// FEW: at most 16 rows per CTA (decode steps): the four warps share the rows and take 16 columns each,
// and k advances 128 at a time, so that a product over a latent of 512 is four rounds of loads instead
// of sixteen.
template <typename TO, bool FEW>
__global__ void __launch_bounds__(128)
head_linear_mma_kernel(const bf16* __restrict__ w, TO* __restrict__ y, HeadMmaArgs p) {
  pdl_trigger();
  constexpr int HM_ROWS = FEW ? 16 : 64, HM_K = FEW ? 128 : 32;
  constexpr int AS = HM_K + 8, BS_NK = HM_K + 8, BS_KN = HM_COLS + 8;
  __shared__ __align__(16) bf16 a_tile[HM_ROWS * AS];
  __shared__ __align__(16) bf16 b_tile[HM_COLS * BS_NK > HM_K * BS_KN ? HM_COLS * BS_NK : HM_K * BS_KN];
  const int head = blockIdx.z, row0 = blockIdx.y * HM_ROWS, n0 = blockIdx.x * HM_COLS;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warp_row = FEW ? 0 : warp * 16, warp_col = FEW ? warp * 16 : 0;
  constexpr int NT = FEW ? 2 : HM_COLS / 8;        // column blocks of 8 per warp
  const bf16* wh = w + (size_t)head * p.N * p.K;
  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  pdl_wait();
  // the pieces of the next k step are fetched into registers while the products of this one run
  constexpr int A_PIECES = HM_ROWS * HM_K / 4 / 128, B_PIECES = HM_COLS * HM_K / 8 / 128;
  float4 a_next[A_PIECES];
  uint4 b_next[B_PIECES];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int i = 0; i < A_PIECES; ++i) {
      const int item = threadIdx.x + 128 * i;
      const int r = item / (HM_K / 4), c = item - r * (HM_K / 4);
      const int row = row0 + r, k = k0 + 4 * c;
      a_next[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (row < p.rows && k < p.K)
        a_next[i] = __ldcg(reinterpret_cast<const float4*>(p.x + (size_t)row * p.x_row + (size_t)head * p.x_head + k));
    }
#pragma unroll
    for (int i = 0; i < B_PIECES; ++i) {
      const int item = threadIdx.x + 128 * i;
      b_next[i] = make_uint4(0, 0, 0, 0);
      if (p.kn) {
        const int k = item / (HM_COLS / 8), c = item - k * (HM_COLS / 8);
        if (k0 + k < p.K && n0 + 8 * c < p.N)
          b_next[i] = *reinterpret_cast<const uint4*>(wh + (size_t)(k0 + k) * p.N + n0 + 8 * c);
      } else {
        const int n = item / (HM_K / 8), c = item - n * (HM_K / 8);
        if (n0 + n < p.N && k0 + 8 * c < p.K)
          b_next[i] = *reinterpret_cast<const uint4*>(wh + (size_t)(n0 + n) * p.K + k0 + 8 * c);
      }
    }
  };
  fetch(0);
  for (int k0 = 0; k0 < p.K; k0 += HM_K) {
#pragma unroll
    for (int i = 0; i < A_PIECES; ++i) {
      const int item = threadIdx.x + 128 * i;
      const int r = item / (HM_K / 4), c = item - r * (HM_K / 4);
      uint2 packed;
      packed.x = pack_bf16(a_next[i].x, a_next[i].y);
      packed.y = pack_bf16(a_next[i].z, a_next[i].w);
      *reinterpret_cast<uint2*>(a_tile + r * AS + 4 * c) = packed;
    }
#pragma unroll
    for (int i = 0; i < B_PIECES; ++i) {
      const int item = threadIdx.x + 128 * i;
      if (p.kn) {
        const int k = item / (HM_COLS / 8), c = item - k * (HM_COLS / 8);
        *reinterpret_cast<uint4*>(b_tile + k * BS_KN + 8 * c) = b_next[i];
      } else {
        const int n = item / (HM_K / 8), c = item - n * (HM_K / 8);
        *reinterpret_cast<uint4*>(b_tile + n * BS_NK + 8 * c) = b_next[i];
      }
    }
    __syncthreads();
    if (k0 + HM_K < p.K) fetch(k0 + HM_K);
#pragma unroll
    for (int kk = 0; kk < HM_K / 16; ++kk) {
      uint32_t a[4];
      ldmatrix_x4(a, a_tile + (warp_row + (lane & 7) + ((lane >> 3) & 1) * 8) * AS + (kk * 2 + (lane >> 4)) * 8);
#pragma unroll
      for (int jp = 0; jp < NT / 2; ++jp) {
        uint32_t b[4];
        const int col = warp_col + jp * 16;
        if (p.kn)
          ldmatrix_x4_trans(b, b_tile + (kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3)) * BS_KN + col + (lane >> 4) * 8);
        else
          ldmatrix_x4(b, b_tile + (col + (lane & 7) + ((lane >> 4) << 3)) * BS_NK + (kk * 2 + ((lane >> 3) & 1)) * 8);
        mma_bf16(acc[2 * jp], a, b[0], b[1]);
        mma_bf16(acc[2 * jp + 1], a, b[2], b[3]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = row0 + warp_row + (lane >> 2) + 8 * i;
    if (row >= p.rows) continue;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int n = n0 + warp_col + j * 8 + (lane & 3) * 2 + e;
        if (n >= p.N) continue;
        float v = acc[j][2 * i + e];
        if (p.mode == 2) {
          const float g = p.gate[(size_t)row * p.gate_row + (p.gate_per_head ? head : head * p.N + n)];
          v = v / (1.f + expf(-g));
        }
        y[(size_t)row * p.y_row + (size_t)head * p.y_head + n] = from_float<TO>(v);
      }
    }
  }
  if (p.mode == 1 && blockIdx.x == 0) {
    for (int idx = threadIdx.x; idx < HM_ROWS * p.tail; idx += 128) {
      const int r = idx / p.tail, d = idx - r * p.tail;
      const int row = row0 + r;
      if (row >= p.rows) continue;
      const float* src = p.x + (size_t)row * p.x_row + (size_t)head * p.x_head + p.K;
      TO* dst = y + (size_t)row * p.y_row + (size_t)head * p.y_head + p.N;
      if (d >= 2 * p.pairs) {
        dst[d] = from_float<TO>(src[d]);
      } else {
        int i, second;
        if (p.interleaved) { i = d >> 1; second = d & 1; }
        else { second = d >= p.pairs; i = second ? d - p.pairs : d; }
        const int a = p.interleaved ? 2 * i : i, b = p.interleaved ? 2 * i + 1 : i + p.pairs;
        float sine, cosine, ya, yb;
        sincosf((float)p.positions[row] * p.frequencies[i], &sine, &cosine);
        rotate_pair(src[a], src[b], sine, cosine, &ya, &yb);
        dst[d] = from_float<TO>(second ? yb : ya);
      }
    }
  }
}

}  // namespace mlr

using namespace mlr;

MLR_DEFINE_PDL_SWITCH

static size_t latent_mma_shared(int groups, int dk, int stages = 2) {
  return sizeof(bf16) * ((size_t)(groups * LM_TOKENS + stages * LM_KEYS) * (dk + 8) + groups * LM_TOKENS * LM_P_STRIDE) +
         sizeof(float) * 2 * groups * LM_SPLIT * LM_TOKENS;
}

// Whether the kernels take these sizes (the caller falls back to the float32 kernels otherwise).
MLR_EXPORT int mlr_latent_attention_mma_fits(int rank, int rot) {
  const int dk = rank + rot;
  return rank > 0 && rank % 8 == 0 && rank <= LM_SPLIT * LM_MAX_NT * 8 && rot >= 8 && dk % 16 == 0 &&
         latent_mma_shared(2, dk) <= 200 * 1024;
}

template <int G, bool DECODE>
static int latent_mma_launch(const void* q, const void* pool, float* out, const int* tile_seg, const int* tile_row0,
                             dim3 grid, const LatentMmaArgs& args, cudaStream_t stream) {
  const size_t shared = latent_mma_shared(G, args.rank + args.rot, args.stages);
  if (shared > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(latent_mma_kernel<G, DECODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    if (err != cudaSuccess) return (int)err;
  }
  launch_kernel(latent_mma_kernel<G, DECODE>, grid, dim3(G * LM_SPLIT * 32), shared, stream, (const bf16*)q,
                (const bf16*)pool, out, tile_seg, tile_row0, args);
  return launch_status();
}

static int latent_mma_args(LatentMmaArgs& args, const void* q, const void* pool, const float* out, const int* seg_q_start,
                           const int* seg_q_len, const int* seg_pos0, const int* block_table, const int* seg_slot,
                           int table_width, int heads, int rank, int rot, int page_size, int window, float scale,
                           const float* sink) {
  if (heads <= 0 || page_size <= 0 || table_width <= 0) return MLR_BAD_SIZE;
  if (!mlr_latent_attention_mma_fits(rank, rot) || heads > 65535) return MLR_TOO_LARGE;
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(pool) & 15)) return MLR_BAD_ALIGNMENT;
  args.seg_q_start = seg_q_start; args.seg_q_len = seg_q_len; args.seg_pos0 = seg_pos0; args.block_table = block_table;
  args.seg_slot = seg_slot; args.table_width = table_width; args.heads = heads; args.rank = rank; args.rot = rot;
  args.page_size = page_size; args.window = window; args.scale_log2 = scale * 1.4426950408889634f; args.sink = sink;
  args.decode_seg = nullptr; args.partial = nullptr; args.stages = 2;
  return MLR_OK;
}

// q: bfloat16 [rows, heads, rank + rot]; pool: bfloat16 [pages, 1, page_size, rank + rot]; out: float32
// [rows, heads, rank]; tile_seg / tile_row0: one entry per tile of up to 16 rows of one segment.
MLR_EXPORT int mlr_latent_attention_mma(const void* q, const void* pool, float* out, const int* tile_seg,
                                        const int* tile_row0, const int* seg_q_start, const int* seg_q_len,
                                        const int* seg_pos0, const int* block_table, const int* seg_slot,
                                        int table_width, int tiles, int heads, int rank, int rot, int page_size,
                                        int window, float scale, const float* sink, cudaStream_t stream) {
  if (tiles == 0) return MLR_OK;
  if (tiles < 0) return MLR_BAD_SIZE;
  LatentMmaArgs args;
  const int status = latent_mma_args(args, q, pool, out, seg_q_start, seg_q_len, seg_pos0, block_table, seg_slot,
                                     table_width, heads, rank, rot, page_size, window, scale, sink);
  if (status != MLR_OK) return status;
  if (heads == 1)
    return latent_mma_launch<1, false>(q, pool, out, tile_seg, tile_row0, dim3(tiles, 1), args, stream);
  // four heads over one key tile where that many fit: the key tiles are fetched half as often and an SM
  // holds sixteen warps instead of eight
  if (heads > 2 && latent_mma_shared(4, rank + rot) <= 200 * 1024)
    return latent_mma_launch<4, false>(q, pool, out, tile_seg, tile_row0, dim3(tiles, (heads + 3) / 4), args, stream);
  return latent_mma_launch<2, false>(q, pool, out, tile_seg, tile_row0, dim3(tiles, (heads + 1) / 2), args, stream);
}

// Floats of scratch a decode call with `chunks` key chunks needs (0 for one chunk).
MLR_EXPORT long long mlr_latent_attention_mma_decode_scratch(int count, int chunks, int heads, int rank) {
  return chunks <= 1 ? 0 : (long long)count * chunks * heads * (rank + 2);
}

// Segments of one row each: decode_seg lists them (null: segments 0 .. count-1).  The keys of every
// row are cut into `chunks` chunks (>= 1); with more than one, `partial` holds
// mlr_latent_attention_mma_decode_scratch floats.
MLR_EXPORT int mlr_latent_attention_mma_decode(const void* q, const void* pool, float* out, const int* decode_seg,
                                               int count, int chunks, float* partial, const int* seg_q_start,
                                               const int* seg_pos0, const int* block_table, const int* seg_slot,
                                               int table_width, int heads, int rank, int rot, int page_size, int window,
                                               float scale, const float* sink, cudaStream_t stream) {
  if (count == 0) return MLR_OK;
  if (count < 0 || chunks < 1 || chunks > 32 || (chunks > 1 && partial == nullptr)) return MLR_BAD_SIZE;
  LatentMmaArgs args;
  int status = latent_mma_args(args, q, pool, out, seg_q_start, nullptr, seg_pos0, block_table, seg_slot, table_width,
                               heads, rank, rot, page_size, window, scale, sink);
  if (status != MLR_OK) return status;
  args.decode_seg = decode_seg;
  args.partial = partial;
  const int blocks16 = (heads + LM_TOKENS - 1) / LM_TOKENS;
  // a decoded row's CTAs are few and wait for memory: as many key tiles on their way as fit (up to three)
  while (args.stages < 4 && latent_mma_shared(blocks16 == 1 ? 1 : 2, rank + rot, args.stages + 1) <= 160 * 1024) ++args.stages;
  if (blocks16 == 1)
    status = latent_mma_launch<1, true>(q, pool, out, nullptr, nullptr, dim3(count, 1, chunks), args, stream);
  else
    status = latent_mma_launch<2, true>(q, pool, out, nullptr, nullptr, dim3(count, (blocks16 + 1) / 2, chunks), args, stream);
  if (status != MLR_OK || chunks == 1) return status;
  launch_kernel(latent_merge_kernel, dim3((unsigned)(count * heads)), dim3(128), 0, stream, (const float*)partial, out,
                decode_seg, seg_q_start, sink, count, chunks, heads, rank);
  return launch_status();
}

// The per-head product of mlr_head_linear on the tensor cores: bfloat16 w, float32 x; y_dtype MLR_BF16 or
// MLR_F32.  Refuses (MLR_BAD_ALIGNMENT) sizes whose pieces are not 16-byte aligned; the caller then
// takes the float32 kernel.
MLR_EXPORT int mlr_head_linear_mma(const float* x, long long x_row, int x_head, const void* w, void* y, long long y_row,
                                   int y_head, int rows, int heads, int N, int K, int kn, int mode, int tail, int pairs,
                                   int interleaved, const int* positions, const float* frequencies, const float* gate,
                                   long long gate_row, int gate_per_head, int y_dtype, cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || heads <= 0 || N <= 0 || K <= 0 || tail < 0 || pairs < 0 || 2 * pairs > tail) return MLR_BAD_SIZE;
  if (heads > 65535 || (rows + 63) / 64 > 65535) return MLR_TOO_LARGE;
  if (N % 8 || K % 8 || x_row % 4 || x_head % 4 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15))
    return MLR_BAD_ALIGNMENT;
  if (mode == 1 && tail > 0 && pairs > 0 && (positions == nullptr || frequencies == nullptr)) return MLR_BAD_SIZE;
  if (mode == 2 && gate == nullptr) return MLR_BAD_SIZE;
  HeadMmaArgs p;
  p.x = x; p.x_row = x_row; p.x_head = x_head; p.y_row = y_row; p.y_head = y_head; p.rows = rows; p.heads = heads;
  p.N = N; p.K = K; p.kn = kn; p.mode = mode; p.tail = mode == 1 ? tail : 0; p.pairs = pairs; p.interleaved = interleaved;
  p.positions = positions; p.frequencies = frequencies; p.gate = gate; p.gate_row = gate_row; p.gate_per_head = gate_per_head;
  const bool few = rows <= 16;
  const dim3 grid((N + HM_COLS - 1) / HM_COLS, few ? 1 : (rows + 63) / 64, heads);
  if (y_dtype == MLR_BF16) {
    if (few) launch_kernel(head_linear_mma_kernel<bf16, true>, grid, dim3(128), 0, stream, (const bf16*)w, (bf16*)y, p);
    else launch_kernel(head_linear_mma_kernel<bf16, false>, grid, dim3(128), 0, stream, (const bf16*)w, (bf16*)y, p);
  } else if (y_dtype == MLR_F32) {
    if (few) launch_kernel(head_linear_mma_kernel<float, true>, grid, dim3(128), 0, stream, (const bf16*)w, (float*)y, p);
    else launch_kernel(head_linear_mma_kernel<float, false>, grid, dim3(128), 0, stream, (const bf16*)w, (float*)y, p);
  } else {
    return MLR_BAD_DTYPE;
  }
  return launch_status();
}
