// The seams of a sequential block (THA_BLOCK_SEQUENTIAL): x <- x + m mixer(norm1 x), x <- x + m ff(norm2 x), then the
// per-token side input.
//   hyb_add_norm_kernel     x += c_left * left + c_right * right (+ the embedding output) (+ a vector), then the next norm
//                           of the new x in the same pass: the mixer's residual add with norm2, or a pass's re-entry
//                           addends with norm1.
//   hyb_side_finish_kernel  x += m * ff; the side input y = W_proj (gelu_tanh(W_gate x) * e_token), x += m * y / rms(y) * w;
//                           the layer's tap.  One block per row: the gate's `dim` dot products over the width by warps,
//                           the projection's `width` dot products over `dim` by threads, the rms by the block.
// The residual stream, the norms, the gate's activation and the side norm are fp32 in both number formats; sums run in a
// fixed order per row, so a row's result does not depend on the rest of the step.
#include <cuda_bf16.h>

#include "common.cuh"
#include "hybrid_ops.cuh"
#include "tha_hybrid.h"

namespace tha {

template <typename T>
__global__ void hyb_add_norm_kernel(float* __restrict__ x, const float* __restrict__ left, float c_left, const float* __restrict__ right,
                                    float c_right, const float* __restrict__ embed_out, const float* __restrict__ vec, tha_norm_t n,
                                    int has_norm, float eps, T* __restrict__ out, int width) {
  __shared__ float red[33];
  const int r = blockIdx.x;
  float* xr = x + (size_t)r * width;
  float sum = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = xr[i];
    if (left) {
      float y = c_left * left[(size_t)r * width + i];
      if (right) y = fmaf(c_right, right[(size_t)r * width + i], y);
      v += y;
    }
    if (embed_out) v += embed_out[(size_t)r * width + i];
    if (vec) v += vec[i];
    xr[i] = v;
    sum += v;
  }
  if (!has_norm) return;
  // every thread reads back only what it wrote itself
  if (n.kind == THA_NORM_LAYER) {
    const float mean = block_sum(sum, red) / (float)width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) { const float d = xr[i] - mean; ss = fmaf(d, d, ss); }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) hyb_store(out + (size_t)r * width + i, fmaf((xr[i] - mean) * inv, n.w[i], n.b ? n.b[i] : 0.f));
  } else if (n.kind == THA_NORM_RMS) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) ss = fmaf(xr[i], xr[i], ss);
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) hyb_store(out + (size_t)r * width + i, xr[i] * inv * (n.w_offset + n.w[i]));
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) hyb_store(out + (size_t)r * width + i, fmaf(tanhf(n.alpha * xr[i]), n.w[i], n.b ? n.b[i] : 0.f));
  }
}

template <typename T>
__global__ void hyb_side_finish_kernel(float* __restrict__ x, const float* __restrict__ ff, float m, tha_side_t side, const T* __restrict__ table,
                                       int side_cols, const int* __restrict__ token, float eps, int width, float* __restrict__ tap) {
  extern __shared__ float sm[];   // x row [width] | g [dim]
  __shared__ float red[33];
  const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  float* xs = sm;
  float* g = sm + width;
  float* xr = x + (size_t)r * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) xs[i] = ff ? fmaf(m, ff[(size_t)r * width + i], xr[i]) : xr[i];
  __syncthreads();
  if (side.dim > 0) {
    const T* wg = (const T*)side.w_gate;
    const T* wp = (const T*)side.w_proj;
    const T* e = table + (size_t)token[r] * side_cols + side.col0;
    for (int j = warp; j < side.dim; j += nwarps) {
      float acc = 0.f;
      for (int i = lane; i < width; i += 32) acc = fmaf(hyb_load(wg + (size_t)j * width + i), xs[i], acc);
      acc = warp_sum(acc);
      if (lane == 0) g[j] = 0.5f * acc * (1.0f + tanhf(0.7978845608028654f * (acc + 0.044715f * acc * acc * acc))) * hyb_load(e + j);
    }
    __syncthreads();
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      float y = 0.f;
      for (int j = 0; j < side.dim; j++) y = fmaf(hyb_load(wp + (size_t)i * side.dim + j), g[j], y);
      ss = fmaf(y, y, ss);
      // parked in the output row until the rms is known (every thread reads back only what it wrote itself)
      xr[i] = y;
    }
    ss = block_sum(ss, red);
    const float inv = m / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      const float v = fmaf(xr[i] * inv, side.norm[i], xs[i]);
      xr[i] = v;
      if (tap) tap[(size_t)r * width + i] = v;
    }
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      xr[i] = xs[i];
      if (tap) tap[(size_t)r * width + i] = xs[i];
    }
  }
}

}  // namespace tha

using namespace tha;
typedef __nv_bfloat16 bf16;

static int block_threads(int width) {
  int t = 64;
  while (t < width / 4 && t < 256) t += 32;
  return t;
}

extern "C" int tha_hyb_add_norm(void* stream, int dtype, float* x, const float* left, float c_left, const float* right, float c_right,
                                const float* embed_out, const float* vec, const tha_norm_t* n, float eps, void* out, int n_rows, int width) {
  if (n_rows < 1) return THA_STATUS_SUCCESS;
  if (!x || (n && (!out || !n->w))) return THA_STATUS_INVALID_ARG;
  const tha_norm_t none = {};
  const int nt = block_threads(width);
  if (dtype == THA_DT_BF16)
    THA_CUDA_OK(launch(hyb_add_norm_kernel<bf16>, dim3(n_rows), dim3(nt), 0, (cudaStream_t)stream, false, x, left, c_left, right, c_right, embed_out, vec,
                       n ? *n : none, n ? 1 : 0, eps, (bf16*)out, width));
  else
    THA_CUDA_OK(launch(hyb_add_norm_kernel<float>, dim3(n_rows), dim3(nt), 0, (cudaStream_t)stream, false, x, left, c_left, right, c_right, embed_out,
                       vec, n ? *n : none, n ? 1 : 0, eps, (float*)out, width));
  return THA_STATUS_SUCCESS;
}

extern "C" int tha_hyb_side_finish(void* stream, int dtype, float* x, const float* ff, float m, const tha_side_t* side, const void* side_table,
                                   int side_cols, const int* token, float eps, int n_rows, int width, float* tap) {
  if (n_rows < 1) return THA_STATUS_SUCCESS;
  tha_side_t sd = {};
  if (side && side->dim > 0) {
    if (!side_table || !token || !side->w_gate || !side->w_proj || !side->norm || side->col0 + side->dim > side_cols) return THA_STATUS_INVALID_ARG;
    sd = *side;
  }
  const size_t smem = sizeof(float) * ((size_t)width + sd.dim);
  if (smem > 200 * 1024) return THA_STATUS_NOT_SUPPORTED;
  const int nt = block_threads(width);
  if (dtype == THA_DT_BF16) {
    if (smem > 48 * 1024) THA_CUDA_OK(cudaFuncSetAttribute(hyb_side_finish_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    THA_CUDA_OK(launch(hyb_side_finish_kernel<bf16>, dim3(n_rows), dim3(nt), smem, (cudaStream_t)stream, false, x, ff, m, sd, (const bf16*)side_table,
                       side_cols, token, eps, width, tap));
  } else {
    if (smem > 48 * 1024) THA_CUDA_OK(cudaFuncSetAttribute(hyb_side_finish_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    THA_CUDA_OK(launch(hyb_side_finish_kernel<float>, dim3(n_rows), dim3(nt), smem, (cudaStream_t)stream, false, x, ff, m, sd, (const float*)side_table,
                       side_cols, token, eps, width, tap));
  }
  return THA_STATUS_SUCCESS;
}
