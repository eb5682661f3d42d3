// Kernels of decoders whose residual stream is 32-bit floats and whose sublayers are wrapped in
// layer norms on both sides ("sandwich" arrangement).
//
// mlr_embedding_rows32     float32 rows table[ids] of a table in the compute dtype.
// mlr_layer_norm_step      one pass over each row of the stream x that does, in this order, whatever
//                          its arguments ask for:
//                            x += LN(delta; dw, db)      the sublayer output that was still to be added,
//                                                        normalised on its way into the stream
//                            x += offset                 one learned vector for all rows
//                            out = LN(x; w, b)           the input of the next sublayer, compute dtype
//                          LN(v; w, b) = (v - mean) / sqrt(var + eps) * w + b with var the mean of the
//                          squared deviations; all sums in float32 in an order fixed by the width.
// mlr_clamped_gate         y = g * sigmoid(slope * g) * (u + 1) with g = min(gate, limit) and
//                          u = clamp(up, -limit, limit), on rows of gate/up blocks.
// mlr_scale_inplace        x *= s for float32 x (logit scale).
#include "common.cuh"

namespace mlr {

template <typename T>
__global__ void __launch_bounds__(256)
embedding_rows32_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ out, int width,
                        int vocab) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  int id = ids[row];
  id = min(max(id, 0), vocab - 1);
  const T* src = table + (size_t)id * width;
  float* dst = out + (size_t)row * width;
  for (int d = threadIdx.x; d < width; d += blockDim.x) dst[d] = to_float(src[d]);
}

// mean and 1/sqrt(var + eps) of `width` floats in shared memory; every thread gets both.
__device__ __forceinline__ void row_statistics(const float* values, int width, float eps, float* scratch, float* mean_out,
                                               float* rstd_out) {
  float sum = 0.f;
  for (int d = threadIdx.x; d < width; d += blockDim.x) sum += values[d];
  const float mean = block_sum(sum, scratch) / (float)width;
  float sq = 0.f;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    const float c = values[d] - mean;
    sq = fmaf(c, c, sq);
  }
  const float variance = block_sum(sq, scratch) / (float)width;
  *mean_out = mean;
  *rstd_out = 1.f / sqrtf(variance + eps);
}

template <typename T>
__global__ void __launch_bounds__(256)
layer_norm_step_kernel(float* x, const float* delta, const float* __restrict__ dw, const float* __restrict__ db,
                       const float* __restrict__ offset, const float* __restrict__ w, const float* __restrict__ b,
                       T* __restrict__ out, int width, float eps) {
  pdl_trigger();
  extern __shared__ float staged[];      // [width] + 32
  float* scratch = staged + width;
  const size_t base = (size_t)blockIdx.x * width;
  pdl_wait();
  float mean, rstd;
  if (delta != nullptr) {
    for (int d = threadIdx.x; d < width; d += blockDim.x) staged[d] = delta[base + d];
    __syncthreads();
    row_statistics(staged, width, eps, scratch, &mean, &rstd);
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
      float v = x[base + d] + fmaf((staged[d] - mean) * rstd, dw[d], db[d]);
      if (offset != nullptr) v += offset[d];
      staged[d] = v;
      x[base + d] = v;
    }
  } else {
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
      float v = x[base + d];
      if (offset != nullptr) {
        v += offset[d];
        x[base + d] = v;
      }
      staged[d] = v;
    }
  }
  if (out == nullptr) return;
  __syncthreads();
  row_statistics(staged, width, eps, scratch, &mean, &rstd);
  for (int d = threadIdx.x; d < width; d += blockDim.x)
    out[base + d] = from_float<T>(fmaf((staged[d] - mean) * rstd, w[d], b[d]));
}

template <typename T>
__global__ void __launch_bounds__(256)
clamped_gate_kernel(const T* x, T* __restrict__ out, long long rows, int inner, int block, float limit, float slope) {
  pdl_trigger();
  pdl_wait();
  const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= rows * inner) return;
  const long long row = index / inner;
  const int column = (int)(index - row * inner);
  const int group = column / block, within = column - group * block;
  const T* source = x + row * 2 * inner + (size_t)group * 2 * block;
  const float g = fminf(to_float(source[within]), limit);
  const float u = fminf(fmaxf(to_float(source[block + within]), -limit), limit);
  out[index] = from_float<T>(g / (1.f + expf(-slope * g)) * (u + 1.f));
}

__global__ void __launch_bounds__(256) scale_inplace_kernel(float* x, long long count, float factor) {
  pdl_trigger();
  pdl_wait();
  const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (index < count) x[index] *= factor;
}

}  // namespace mlr

using namespace mlr;

MLR_DEFINE_PDL_SWITCH

MLR_EXPORT int mlr_embedding_rows32(const int* ids, const void* table, float* out, int rows, int width, int vocab,
                                    int dtype, cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || width <= 0 || vocab <= 0) return MLR_BAD_SIZE;
  if (dtype == MLR_F32)
    launch_kernel(embedding_rows32_kernel<float>, dim3(rows), dim3(256), 0, stream, ids, (const float*)table, out, width, vocab);
  else if (dtype == MLR_BF16)
    launch_kernel(embedding_rows32_kernel<bf16>, dim3(rows), dim3(256), 0, stream, ids, (const bf16*)table, out, width, vocab);
  else
    return MLR_BAD_DTYPE;
  return launch_status();
}

// x: float32 [rows, width], updated in place when delta or offset is given.  delta: float32
// [rows, width] or null (then dw, db are not read).  offset: float32 [width] or null.  out: compute
// dtype [rows, width] or null (then w, b are not read).
MLR_EXPORT int mlr_layer_norm_step(float* x, const float* delta, const float* dw, const float* db, const float* offset,
                                   const float* w, const float* b, void* out, int rows, int width, float eps,
                                   int out_dtype, cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || width <= 0) return MLR_BAD_SIZE;
  if ((delta != nullptr && (dw == nullptr || db == nullptr)) || (out != nullptr && (w == nullptr || b == nullptr)))
    return MLR_BAD_SIZE;
  const size_t shared = sizeof(float) * ((size_t)width + 32);
  if (shared > 200 * 1024) return MLR_TOO_LARGE;
  auto launch = [&](auto kernel, auto* typed_out) -> int {
    if (shared > 48 * 1024) {
      cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
      if (err != cudaSuccess) return (int)err;
    }
    launch_kernel(kernel, dim3(rows), dim3(256), shared, stream, x, delta, dw, db, offset, w, b, typed_out, width, eps);
    return launch_status();
  };
  if (out_dtype == MLR_F32) return launch(layer_norm_step_kernel<float>, (float*)out);
  if (out_dtype == MLR_BF16) return launch(layer_norm_step_kernel<bf16>, (bf16*)out);
  return MLR_BAD_DTYPE;
}

MLR_EXPORT int mlr_clamped_gate(const void* x, void* out, long long rows, int inner, int block, float limit, float slope,
                                int dtype, cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || inner <= 0 || block <= 0 || inner % block != 0) return MLR_BAD_SIZE;
  const long long blocks = (rows * inner + 255) / 256;
  if (blocks > 0x7fffffffLL) return MLR_TOO_LARGE;
  if (dtype == MLR_F32)
    launch_kernel(clamped_gate_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, stream, (const float*)x, (float*)out,
                  rows, inner, block, limit, slope);
  else if (dtype == MLR_BF16)
    launch_kernel(clamped_gate_kernel<bf16>, dim3((unsigned)blocks), dim3(256), 0, stream, (const bf16*)x, (bf16*)out,
                  rows, inner, block, limit, slope);
  else
    return MLR_BAD_DTYPE;
  return launch_status();
}

MLR_EXPORT int mlr_scale_inplace(float* x, long long count, float factor, cudaStream_t stream) {
  if (count == 0) return MLR_OK;
  if (count < 0) return MLR_BAD_SIZE;
  const long long blocks = (count + 255) / 256;
  if (blocks > 0x7fffffffLL) return MLR_TOO_LARGE;
  launch_kernel(scale_inplace_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, x, count, factor);
  return launch_status();
}
