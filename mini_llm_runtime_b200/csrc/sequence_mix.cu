// Kernels of models that keep a 32-bit residual stream and mix along the sequence by recurrences:
//
//   embedding + learned position vector          -> float32 rows
//   RMS norm with one gain for the whole row     -> float32 and/or compute-dtype rows
//   token shift  y = a + (a_prev - a) * c        (a_prev: the row of the request's previous token,
//                                                 carried between steps in a per-request state)
//   gated linear recurrence over a [key, value] state per head (two read/write orders, see below)
//   residual += a (+ b), gate(z) * up on a stacked product, tanh
//
// The batch is ragged: segment s brings rows seg_q_start[s] .. +seg_q_len[s] of the request whose
// fixed-size state lives in slot seg_slot[s].  Every row's result depends only on its own request:
// reductions have a fixed order, recurrences run token by token, so a request's numbers do not
// change with how its tokens are cut into steps or what else is in the batch.
#include "common.cuh"

namespace mlr {

// ------------------------------------------------------------------ embedding + position vector
template <typename T>
__global__ void embedding_positions_kernel(const int* __restrict__ ids, const int* positions,
                                           const T* __restrict__ table, const T* __restrict__ pos_table,
                                           float* __restrict__ out, int width, int vocab, int max_positions) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  int id = ids[row], p = positions[row];
  id = min(max(id, 0), vocab - 1);
  p = min(max(p, 0), max_positions - 1);
  const T* e = table + (size_t)id * width;
  const T* q = pos_table + (size_t)p * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    out[(size_t)row * width + c] = to_float(e[c]) + to_float(q[c]);
}

// ------------------------------------------------------------------ scalar-gain RMS norm
// y = x * rsqrt(mean(x^2) + eps) * g.  One CTA of 256 threads per row; the sum of squares is taken in
// an order that depends on the width only.
template <typename T>
__global__ void __launch_bounds__(256)
scalar_rms_norm_kernel(const float* x, const float* __restrict__ gain, float* out32, T* out, int width, float eps) {
  pdl_trigger();
  pdl_wait();
  __shared__ float scratch[32];
  const float* row = x + (size_t)blockIdx.x * width;
  float sum = 0.f;
  for (int c = threadIdx.x; c < width; c += 256) {
    const float v = row[c];
    sum = fmaf(v, v, sum);
  }
  sum = block_sum(sum, scratch);
  const float factor = __fdiv_rn(gain[0], sqrtf(sum / (float)width + eps));
  for (int c = threadIdx.x; c < width; c += 256) {
    const float y = row[c] * factor;
    if (out32 != nullptr) out32[(size_t)blockIdx.x * width + c] = y;
    if (out != nullptr) out[(size_t)blockIdx.x * width + c] = from_float<T>(y);
  }
}

// ------------------------------------------------------------------ token shift
// out[i][row][c] = a[row][c] + (prev[c] - a[row][c]) * coef[i][c] for i < n, where prev is the row
// before in the same segment, or the request's carried row for the segment's first row.
// grid: (column blocks, row chunks of SHIFT_ROWS, segments).  With `save` (allowed only when every
// segment has one row, so that reader and writer of the state are the same thread) the carried row
// is replaced at once; otherwise save_last_rows_kernel runs afterwards.
constexpr int SHIFT_ROWS = 16;

template <typename T>
__global__ void __launch_bounds__(256)
token_shift_kernel(const float* a, const float* __restrict__ coef, float* state, T* __restrict__ out,
                   const int* __restrict__ seg_q_start, const int* __restrict__ seg_q_len,
                   const int* __restrict__ seg_slot, int width, int n, long long out_stride, int save) {
  pdl_trigger();
  pdl_wait();
  const int seg = blockIdx.z;
  const int length = seg_q_len[seg];
  const int r0 = blockIdx.y * SHIFT_ROWS;
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (r0 >= length || c >= width) return;
  const int first = seg_q_start[seg];
  float* carried = state + (size_t)seg_slot[seg] * width;
  float prev = r0 == 0 ? carried[c] : a[(size_t)(first + r0 - 1) * width + c];
  const int r1 = min(length, r0 + SHIFT_ROWS);
  for (int r = r0; r < r1; ++r) {
    const size_t at = (size_t)(first + r) * width + c;
    const float cur = a[at];
    for (int i = 0; i < n; ++i)
      out[(size_t)i * out_stride + at] = from_float<T>(fmaf(prev - cur, coef[(size_t)i * width + c], cur));
    prev = cur;
  }
  if (save && r1 == length) carried[c] = prev;
}

__global__ void __launch_bounds__(256)
save_last_rows_kernel(const float* a, float* state, const int* __restrict__ seg_q_start,
                      const int* __restrict__ seg_q_len, const int* __restrict__ seg_slot, int width) {
  pdl_trigger();
  pdl_wait();
  const int seg = blockIdx.y;
  const int c = blockIdx.x * 256 + threadIdx.x;
  const int length = seg_q_len[seg];
  if (c >= width || length <= 0) return;
  state[(size_t)seg_slot[seg] * width + c] = a[(size_t)(seg_q_start[seg] + length - 1) * width + c];
}

// ------------------------------------------------------------------ gated linear recurrence
// Per head a state S [dim, vdim] in 32-bit floats, carried per request.  Per token, with per-key-
// channel decay a_t, write strength b_t, read vector r_t and per-value v_t:
//
//   mode 0 (bonus):  o_t = (S + diag(c) b_t v_t^T)^T r_t ;  S <- diag(a_t) S + b_t v_t^T
//                    a = exp(-exp(raw + bias)), b = k, c a per-channel constant, r as given;
//                    out = o / rms(o) * weight[head, j] * silu(gate)
//   mode 1 (gate):   S <- diag(a_t) S + b_t v_t^T ;  o_t = S^T r_t
//                    a = lower + (1 - lower) * sigmoid(raw + bias), b = 1 - a, r = silu(raw r);
//                    out = o / rms(o) * weight[j]
//
// The bonus term is taken out of the sum over key channels: o_t[j] = sum_i r[i] S[i][j] +
// v[j] * sum_i r[i] c[i] b[i], one dot product per token instead of one more product per state entry.
//
// One CTA per (head, segment).  Thread (j, s) keeps rows s*KD .. s*KD+KD-1 of column j of S in
// registers.  Tokens are taken in chunks of REC_CHUNK: the chunk's inputs are transformed (the
// exponentials) by all threads at once into shared memory, the recurrence then runs token by token on
// registers with no barrier (inputs read four key channels per load, two running sums), the partial
// sums of the key slices are added in slice order, and the chunk's outputs are normalised one warp
// per token.
constexpr int REC_CHUNK = 32;

struct RecurrenceArgs {
  const float *r, *b, *v, *raw, *gate;           // row-major views, one row per token
  long long r_stride, b_stride, v_stride, raw_stride, gate_stride;
  const float *bias, *aux, *weight;              // aux: the bonus (mode 0) or the lower bound (mode 1)
  float eps;
  float* state;                                  // [slots, heads, dim, vdim]
  const int *seg_q_start, *seg_q_len, *seg_slot;
  int heads, dim, vdim, weight_per_head;
  int columns;        // value channels per CTA: vdim, or a part of it (blockIdx.z picks the part)
  float* raw_out;     // with parts: the un-normalised o [rows, heads*vdim]; recurrence_finish_kernel ends the job
};

template <typename T, int MODE, int KD>
__global__ void __launch_bounds__(512)
gated_recurrence_kernel(RecurrenceArgs p, T* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) float shared[];
  const int dim = p.dim, full = p.vdim, column0 = blockIdx.z * p.columns;
  const int vdim = min(p.columns, full - column0);      // this CTA's value channels (the last part may be short)
  const int slices = blockDim.y, dim_pad = slices * KD;
  float* s_r = shared;                              // [CHUNK][dim_pad]
  float* s_a = s_r + REC_CHUNK * dim_pad;
  float* s_b = s_a + REC_CHUNK * dim_pad;
  float* s_bonus = s_b + REC_CHUNK * dim_pad;       // [CHUNK] sum_i r c b (mode 0)
  float* s_v = s_bonus + REC_CHUNK;                 // [CHUNK][vdim]
  float* s_o = s_v + REC_CHUNK * vdim;              // [slices][CHUNK][vdim]

  const int head = blockIdx.x, seg = blockIdx.y;
  const int length = p.seg_q_len[seg], first = p.seg_q_start[seg];
  const int j = threadIdx.x, slice = threadIdx.y;
  const int tid = threadIdx.y * blockDim.x + threadIdx.x, threads = blockDim.x * blockDim.y;
  const int warp = tid >> 5, lane = tid & 31, warps = threads >> 5;
  const bool owner = j < vdim;
  float* state = p.state + ((size_t)p.seg_slot[seg] * p.heads + head) * dim * full + column0;

  float S[KD];
#pragma unroll
  for (int i = 0; i < KD; ++i) {
    const int row = slice * KD + i;
    S[i] = (owner && row < dim) ? state[(size_t)row * full + j] : 0.f;
  }

  for (int t0 = 0; t0 < length; t0 += REC_CHUNK) {
    const int count = min(REC_CHUNK, length - t0);
    __syncthreads();      // the chunk before has been written out
    for (int idx = tid; idx < count * dim_pad; idx += threads) {
      const int t = idx / dim_pad, i = idx - t * dim_pad;
      float r = 0.f, a = 0.f, b = 0.f;
      if (i < dim) {
        const size_t row = (size_t)(first + t0 + t);
        const int col = head * dim + i;
        r = p.r[row * p.r_stride + col];
        const float z = p.raw[row * p.raw_stride + col] + p.bias[col];
        if (MODE == 0) {
          a = expf(-expf(z));
          b = p.b[row * p.b_stride + col];
        } else {
          const float lower = p.aux[col];
          a = lower + (1.f - lower) * (1.f / (1.f + expf(-z)));
          b = 1.f - a;
          r = r / (1.f + expf(-r));
        }
      }
      s_r[idx] = r;
      s_a[idx] = a;
      s_b[idx] = b;
    }
    for (int idx = tid; idx < count * vdim; idx += threads) {
      const int t = idx / vdim, c = idx - t * vdim;
      s_v[idx] = p.v[(size_t)(first + t0 + t) * p.v_stride + head * full + column0 + c];
    }
    __syncthreads();
    if (MODE == 0) {
      for (int t = warp; t < count; t += warps) {
        float dot = 0.f;
        for (int i = lane; i < dim; i += 32)
          dot = fmaf(s_r[t * dim_pad + i] * p.aux[head * dim + i], s_b[t * dim_pad + i], dot);
        dot = warp_sum(dot);
        if (lane == 0) s_bonus[t] = dot;
      }
    }
    if (owner) {
      // one token: the thread's KD state rows against the token's r, a, b (four channels per load)
      auto one_token = [&](int t) {
        const float v = s_v[t * vdim + j];
        const float4* rr = reinterpret_cast<const float4*>(s_r + t * dim_pad + slice * KD);
        const float4* aa = reinterpret_cast<const float4*>(s_a + t * dim_pad + slice * KD);
        const float4* bb = reinterpret_cast<const float4*>(s_b + t * dim_pad + slice * KD);
        float o0 = 0.f, o1 = 0.f;
#pragma unroll
        for (int i4 = 0; i4 < KD / 4; ++i4) {
          const float4 r = rr[i4], a = aa[i4], b = bb[i4];
          float* s = S + 4 * i4;
          if (MODE == 0) {
            o0 = fmaf(r.x, s[0], o0); o1 = fmaf(r.y, s[1], o1);
            o0 = fmaf(r.z, s[2], o0); o1 = fmaf(r.w, s[3], o1);
            s[0] = fmaf(a.x, s[0], b.x * v); s[1] = fmaf(a.y, s[1], b.y * v);
            s[2] = fmaf(a.z, s[2], b.z * v); s[3] = fmaf(a.w, s[3], b.w * v);
          } else {
            s[0] = fmaf(a.x, s[0], b.x * v); s[1] = fmaf(a.y, s[1], b.y * v);
            s[2] = fmaf(a.z, s[2], b.z * v); s[3] = fmaf(a.w, s[3], b.w * v);
            o0 = fmaf(r.x, s[0], o0); o1 = fmaf(r.y, s[1], o1);
            o0 = fmaf(r.z, s[2], o0); o1 = fmaf(r.w, s[3], o1);
          }
        }
        s_o[(slice * REC_CHUNK + t) * vdim + j] = o0 + o1;
      };
      if (KD <= 8 && count == REC_CHUNK) {
        // a full chunk: eight tokens at a time, so that the next tokens' loads are issued under this token's arithmetic
#pragma unroll 8
        for (int t = 0; t < REC_CHUNK; ++t) one_token(t);
      } else if (KD <= 32 && count == REC_CHUNK) {
        // more rows per thread: two tokens at a time (more would not fit the registers)
#pragma unroll 2
        for (int t = 0; t < REC_CHUNK; ++t) one_token(t);
      } else {
        for (int t = 0; t < count; ++t) one_token(t);
      }
    }
    __syncthreads();
    // normalise and write: one warp per token, lanes over the value channels
    for (int t = warp; t < count; t += warps) {
      float sq = 0.f;
      const float bonus = MODE == 0 ? s_bonus[t] : 0.f;
      const size_t row = (size_t)(first + t0 + t);
      for (int c = lane; c < vdim; c += 32) {
        float o = 0.f;
        for (int s = 0; s < slices; ++s) o += s_o[(s * REC_CHUNK + t) * vdim + c];
        if (MODE == 0) o = fmaf(s_v[t * vdim + c], bonus, o);
        if (p.raw_out != nullptr) p.raw_out[(row * p.heads + head) * full + column0 + c] = o;
        s_o[t * vdim + c] = o;      // slice 0's place now holds the sum (same lane reads it below)
        sq = fmaf(o, o, sq);
      }
      if (p.raw_out != nullptr) continue;       // the value channels are spread over CTAs: finished elsewhere
      sq = warp_sum(sq);
      const float factor = 1.f / sqrtf(sq / (float)vdim + p.eps);
      for (int c = lane; c < vdim; c += 32) {
        float y = s_o[t * vdim + c] * factor * p.weight[p.weight_per_head ? head * vdim + c : c];
        if (MODE == 0) {
          const float g = p.gate[row * p.gate_stride + head * vdim + c];
          y *= g / (1.f + expf(-g));
        }
        out[(row * p.heads + head) * vdim + c] = from_float<T>(y);
      }
    }
  }
  if (owner && length > 0) {
#pragma unroll
    for (int i = 0; i < KD; ++i) {
      const int row = slice * KD + i;
      if (row < dim) state[(size_t)row * full + j] = S[i];
    }
  }
}

// The end of a recurrence whose value channels were spread over CTAs: one warp per (row, head) takes
// o / rms(o) * weight (* silu(gate)).
template <typename T>
__global__ void __launch_bounds__(128)
recurrence_finish_kernel(const float* raw, const float* gate, long long gate_stride, const float* __restrict__ weight,
                         int weight_per_head, T* __restrict__ out, long long items, int heads, int vdim, float eps) {
  pdl_trigger();
  pdl_wait();
  const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= items) return;
  const int lane = threadIdx.x & 31;
  const long long row = item / heads;
  const int head = (int)(item - row * heads);
  const float* o = raw + (row * heads + head) * vdim;
  float sq = 0.f;
  for (int c = lane; c < vdim; c += 32) sq = fmaf(o[c], o[c], sq);
  sq = warp_sum(sq);
  const float factor = 1.f / sqrtf(sq / (float)vdim + eps);
  for (int c = lane; c < vdim; c += 32) {
    float y = o[c] * factor * weight[weight_per_head ? head * vdim + c : c];
    if (gate != nullptr) {
      const float g = gate[row * gate_stride + head * vdim + c];
      y *= g / (1.f + expf(-g));
    }
    out[(row * heads + head) * vdim + c] = from_float<T>(y);
  }
}

// ------------------------------------------------------------------ small elementwise kernels
__global__ void add_residual_kernel(float* residual, const float* a, const float* b, long long count) {
  pdl_trigger();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  float delta = a[i];
  if (b != nullptr) delta += b[i];
  residual[i] += delta;
}

__device__ __forceinline__ float gelu_tanh(float z) {
  const float inner = 0.7978845608028654f * fmaf(0.044715f * z * z, z, z);
  return 0.5f * z * (1.f + tanhf(inner));
}

// out[row][c] = act(gate) * up on rows that hold blocks of `block` gate values followed by the
// `block` up values of the same outputs.  act: 0 silu, 1 gelu (tanh form).
template <typename T>
__global__ void gated_activation_kernel(const T* x, T* __restrict__ out, long long rows, int inner, int block, int act) {
  pdl_trigger();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * inner) return;
  const long long row = idx / inner;
  const int c = (int)(idx - row * inner);
  const int blk = c / block, within = c - blk * block;
  const T* base = x + row * 2 * inner + (long long)blk * 2 * block;
  const float gate = to_float(base[within]), up = to_float(base[block + within]);
  const float a = act == 1 ? gelu_tanh(gate) : gate / (1.f + expf(-gate));
  out[idx] = from_float<T>(a * up);
}

template <typename T>
__global__ void tanh_kernel(T* x, long long count) {
  pdl_trigger();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) x[i] = from_float<T>(tanhf(to_float(x[i])));
}

// `raw`: float32 scratch [rows, heads*vdim], or null.  With it, and value heads of several times 32
// channels, steps with long segments spread each head's value channels over CTAs of 32: more CTAs,
// and threads that each hold fewer state rows (the recurrence is bound by the latency of its
// per-token chain, not by throughput); the norm then runs as a second kernel.
template <typename T, int MODE>
int launch_recurrence(RecurrenceArgs args, void* out, float* raw, int segments, int rows, int max_q_len,
                      cudaStream_t stream) {
  // threads a CTA needs for `columns` value channels, with the fewest key channels per thread (8, 16, 32
  // or 64) that keep it within 512: more threads with shorter chains hide the latency of the
  // shared-memory loads that feed them
  auto plan = [&](int columns, int* kd_out) {
    const int lanes = (columns + 31) / 32 * 32;
    int kd = 8;
    while (kd < 64 && lanes * ((args.dim + kd - 1) / kd) > 512) kd *= 2;
    *kd_out = kd;
    return lanes * ((args.dim + kd - 1) / kd);
  };
  int kd = 8;
  const bool whole_fits = plan(args.vdim, &kd) <= 512;
  // parts of 32 channels: in steps with long segments, and whenever a whole head does not fit a CTA
  const bool spread = raw != nullptr && args.vdim > 32 && (max_q_len >= 64 || !whole_fits);
  args.columns = spread ? 32 : args.vdim;
  args.raw_out = spread ? raw : nullptr;
  const int vp = (args.columns + 31) / 32 * 32;
  if (plan(args.columns, &kd) > 512) return MLR_TOO_LARGE;
  const int slices = (args.dim + kd - 1) / kd;
  const int dim_pad = slices * kd;
  const size_t shared = sizeof(float) * ((size_t)3 * REC_CHUNK * dim_pad + REC_CHUNK + (size_t)REC_CHUNK * args.columns +
                                         (size_t)slices * REC_CHUNK * args.columns);
  auto kernel = kd == 8 ? gated_recurrence_kernel<T, MODE, 8> : kd == 16 ? gated_recurrence_kernel<T, MODE, 16>
                : kd == 32 ? gated_recurrence_kernel<T, MODE, 32> : gated_recurrence_kernel<T, MODE, 64>;
  if (shared > 200 * 1024) return MLR_TOO_LARGE;
  if (shared > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    if (err != cudaSuccess) return (int)err;
  }
  launch_kernel(kernel, dim3(args.heads, segments, (args.vdim + args.columns - 1) / args.columns), dim3(vp, slices), shared, stream, args,
                (T*)out);
  int status = launch_status();
  if (status != MLR_OK || !spread) return status;
  const long long items = (long long)rows * args.heads;
  launch_kernel(recurrence_finish_kernel<T>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, stream, (const float*)raw,
                MODE == 0 ? args.gate : (const float*)nullptr, args.gate_stride, args.weight, args.weight_per_head,
                (T*)out, items, args.heads, args.vdim, args.eps);
  return launch_status();
}

}  // namespace mlr

using namespace mlr;

MLR_DEFINE_PDL_SWITCH

MLR_EXPORT int mlr_embedding_positions(const int* ids, const int* positions, const void* table, const void* pos_table,
                                       float* out, int rows, int width, int vocab, int max_positions, int dtype,
                                       cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || width <= 0 || vocab <= 0 || max_positions <= 0) return MLR_BAD_SIZE;
  if (dtype == MLR_F32)
    launch_kernel(embedding_positions_kernel<float>, dim3(rows), dim3(256), 0, stream, ids, positions,
                  (const float*)table, (const float*)pos_table, out, width, vocab, max_positions);
  else if (dtype == MLR_BF16)
    launch_kernel(embedding_positions_kernel<bf16>, dim3(rows), dim3(256), 0, stream, ids, positions,
                  (const bf16*)table, (const bf16*)pos_table, out, width, vocab, max_positions);
  else
    return MLR_BAD_DTYPE;
  return launch_status();
}

// x: float32 [rows, width]; out32 (float32) and out (out_dtype) may each be null.
MLR_EXPORT int mlr_scalar_rms_norm(const float* x, const float* gain, float* out32, void* out, int rows, int width,
                                   float eps, int out_dtype, cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || width <= 0) return MLR_BAD_SIZE;
  if (out_dtype == MLR_F32)
    launch_kernel(scalar_rms_norm_kernel<float>, dim3(rows), dim3(256), 0, stream, x, gain, out32, (float*)out, width, eps);
  else if (out_dtype == MLR_BF16)
    launch_kernel(scalar_rms_norm_kernel<bf16>, dim3(rows), dim3(256), 0, stream, x, gain, out32, (bf16*)out, width, eps);
  else
    return MLR_BAD_DTYPE;
  return launch_status();
}

// a: float32 [rows, width]; coef: float32 [n, width]; state: float32 [slots, width];
// out: out_dtype [n, rows, width].  max_q_len: the longest segment of the step.
MLR_EXPORT int mlr_token_shift(const float* a, const float* coef, float* state, void* out, const int* seg_q_start,
                               const int* seg_q_len, const int* seg_slot, int segments, int max_q_len, int rows,
                               int width, int n, int out_dtype, cudaStream_t stream) {
  if (segments == 0 || rows == 0) return MLR_OK;
  if (segments < 0 || rows < 0 || width <= 0 || n <= 0 || max_q_len <= 0) return MLR_BAD_SIZE;
  if (segments > 65535) return MLR_TOO_LARGE;
  const int save = max_q_len == 1;
  dim3 grid((width + 255) / 256, (max_q_len + SHIFT_ROWS - 1) / SHIFT_ROWS, segments);
  if (grid.y > 65535) return MLR_TOO_LARGE;
  const long long stride = (long long)rows * width;
  if (out_dtype == MLR_F32)
    launch_kernel(token_shift_kernel<float>, grid, dim3(256), 0, stream, a, coef, state, (float*)out, seg_q_start,
                  seg_q_len, seg_slot, width, n, stride, save);
  else if (out_dtype == MLR_BF16)
    launch_kernel(token_shift_kernel<bf16>, grid, dim3(256), 0, stream, a, coef, state, (bf16*)out, seg_q_start,
                  seg_q_len, seg_slot, width, n, stride, save);
  else
    return MLR_BAD_DTYPE;
  int status = launch_status();
  if (status != MLR_OK || save) return status;
  launch_kernel(save_last_rows_kernel, dim3((width + 255) / 256, segments), dim3(256), 0, stream, a, state,
                seg_q_start, seg_q_len, seg_slot, width);
  return launch_status();
}

// mode 0: bonus recurrence (r, k = b, v, decay raw, gate raw; aux = bonus [heads*dim]; weight [heads*vdim]).
// mode 1: forget-gate recurrence (r = raw q, v, forget raw; aux = lower bound [heads*dim]; weight [vdim]).
// All inputs float32 views with a row stride (in elements); state float32 [slots, heads, dim, vdim];
// out: out_dtype [rows, heads*vdim]; scratch: float32 of the same shape or null; rows: the step's
// rows; max_q_len: its longest segment.
MLR_EXPORT int mlr_gated_recurrence(int mode, const float* r, long long r_stride, const float* b, long long b_stride,
                                    const float* v, long long v_stride, const float* raw, long long raw_stride,
                                    const float* gate, long long gate_stride, const float* bias, const float* aux,
                                    const float* weight, float eps, float* state, void* out, float* scratch,
                                    const int* seg_q_start, const int* seg_q_len, const int* seg_slot, int segments,
                                    int rows, int max_q_len, int heads, int dim, int vdim, int out_dtype,
                                    cudaStream_t stream) {
  if (segments == 0) return MLR_OK;
  if (segments < 0 || heads <= 0 || dim <= 0 || vdim <= 0) return MLR_BAD_SIZE;
  if (segments > 65535) return MLR_TOO_LARGE;
  RecurrenceArgs args;
  args.r = r; args.b = b; args.v = v; args.raw = raw; args.gate = gate;
  args.r_stride = r_stride; args.b_stride = b_stride; args.v_stride = v_stride;
  args.raw_stride = raw_stride; args.gate_stride = gate_stride;
  args.bias = bias; args.aux = aux; args.weight = weight; args.eps = eps; args.state = state;
  args.seg_q_start = seg_q_start; args.seg_q_len = seg_q_len; args.seg_slot = seg_slot;
  args.heads = heads; args.dim = dim; args.vdim = vdim; args.weight_per_head = mode == 0 ? 1 : 0;
  if (mode == 0 && out_dtype == MLR_F32) return launch_recurrence<float, 0>(args, out, scratch, segments, rows, max_q_len, stream);
  if (mode == 0 && out_dtype == MLR_BF16) return launch_recurrence<bf16, 0>(args, out, scratch, segments, rows, max_q_len, stream);
  if (mode == 1 && out_dtype == MLR_F32) return launch_recurrence<float, 1>(args, out, scratch, segments, rows, max_q_len, stream);
  if (mode == 1 && out_dtype == MLR_BF16) return launch_recurrence<bf16, 1>(args, out, scratch, segments, rows, max_q_len, stream);
  return mode == 0 || mode == 1 ? MLR_BAD_DTYPE : MLR_BAD_SIZE;
}

MLR_EXPORT int mlr_add_residual(float* residual, const float* a, const float* b, long long count, cudaStream_t stream) {
  if (count == 0) return MLR_OK;
  if (count < 0) return MLR_BAD_SIZE;
  launch_kernel(add_residual_kernel, dim3((unsigned)((count + 255) / 256)), dim3(256), 0, stream, residual, a, b, count);
  return launch_status();
}

MLR_EXPORT int mlr_gated_activation(const void* x, void* out, long long rows, int inner, int block, int act, int dtype,
                                    cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || inner <= 0 || block <= 0 || inner % block != 0 || act < 0 || act > 1) return MLR_BAD_SIZE;
  const long long count = rows * inner;
  dim3 grid((unsigned)((count + 255) / 256));
  if (dtype == MLR_F32)
    launch_kernel(gated_activation_kernel<float>, grid, dim3(256), 0, stream, (const float*)x, (float*)out, rows, inner, block, act);
  else if (dtype == MLR_BF16)
    launch_kernel(gated_activation_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)x, (bf16*)out, rows, inner, block, act);
  else
    return MLR_BAD_DTYPE;
  return launch_status();
}

MLR_EXPORT int mlr_tanh_inplace(void* x, long long count, int dtype, cudaStream_t stream) {
  if (count == 0) return MLR_OK;
  if (count < 0) return MLR_BAD_SIZE;
  dim3 grid((unsigned)((count + 255) / 256));
  if (dtype == MLR_F32)
    launch_kernel(tanh_kernel<float>, grid, dim3(256), 0, stream, (float*)x, count);
  else if (dtype == MLR_BF16)
    launch_kernel(tanh_kernel<bf16>, grid, dim3(256), 0, stream, (bf16*)x, count);
  else
    return MLR_BAD_DTYPE;
  return launch_status();
}
