// The seams of a sequential block (THA_BLOCK_SEQUENTIAL): x <- x + m mixer(norm1 x), x <- x + m ff(norm2 x), then the
// per-token side input.
//   hyb_add_norm_kernel     x += c_left * left + c_right * right (+ the embedding output) (+ a vector), then the next norm
//                           of the new x in the same pass: the mixer's residual add with norm2, or a pass's re-entry
//                           addends with norm1.
//                           THA_NORM_COPY hands x on in the product's number format (the input of the side gate).
//   hyb_side_gate_kernel    gelu_tanh of the side gate's product times the token's entries of the side table
//   hyb_block_finish_kernel x += m * ff, x += m * y / rms(y) * w for the side projection y, the layer's tap, then the addends
//                           and the first norm of the NEXT layer run: one pass over x at the end of a block.
// The two side products themselves are the framework's matrix products (tha_hyb_linear).
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
  } else if (n.kind == THA_NORM_DYT) {
    for (int i = threadIdx.x; i < width; i += blockDim.x) hyb_store(out + (size_t)r * width + i, fmaf(tanhf(n.alpha * xr[i]), n.w[i], n.b ? n.b[i] : 0.f));
  } else {   // THA_NORM_COPY
    for (int i = threadIdx.x; i < width; i += blockDim.x) hyb_store(out + (size_t)r * width + i, xr[i]);
  }
}

// g = gelu_tanh(gate product) * e_token, in the product's number format: the input of the side projection
template <typename T>
__global__ void hyb_side_gate_kernel(T* __restrict__ out, const float* __restrict__ gate_raw, long long ldg, const T* __restrict__ table, int side_cols,
                                     int col0, const int* __restrict__ token, int n_rows, int dim) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_rows * dim) return;
  const int r = i / dim, j = i - r * dim;
  const float z = gate_raw[(size_t)r * ldg + j];
  const float e = hyb_load(table + (size_t)token[r] * side_cols + col0 + j);
  hyb_store(out + i, 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))) * e);
}

// The last pass of a sequential block over a row: x += m * ff (ff nullable), x += m * y / rms(y) * w (y nullable: the side
// projection), the tap; then what comes ahead of the NEXT layer run -- the embedding output and the pass vector (nullable) --
// and its first norm, so that the next layer starts at its stacked product.
template <typename T>
__global__ void hyb_block_finish_kernel(float* __restrict__ x, const float* __restrict__ ff, const float* __restrict__ y, float m,
                                        const float* __restrict__ w, float eps, float* __restrict__ tap, const float* __restrict__ embed_out,
                                        const float* __restrict__ vec, tha_norm_t n, int has_norm, T* __restrict__ out, int width) {
  __shared__ float red[33];
  const int r = blockIdx.x;
  float* xr = x + (size_t)r * width;
  float inv = 0.f;
  if (y) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) { const float v = y[(size_t)r * width + i]; ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    inv = m / sqrtf(ss / (float)width + eps);
  }
  float sum = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = xr[i];
    if (ff) v = fmaf(m, ff[(size_t)r * width + i], v);
    if (y) v = fmaf(y[(size_t)r * width + i] * inv, w[i], v);
    if (tap) tap[(size_t)r * width + i] = v;
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
    const float iv = 1.0f / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) hyb_store(out + (size_t)r * width + i, fmaf((xr[i] - mean) * iv, n.w[i], n.b ? n.b[i] : 0.f));
  } else if (n.kind == THA_NORM_RMS) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) ss = fmaf(xr[i], xr[i], ss);
    ss = block_sum(ss, red);
    const float iv = 1.0f / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) hyb_store(out + (size_t)r * width + i, xr[i] * iv * (n.w_offset + n.w[i]));
  } else if (n.kind == THA_NORM_DYT) {
    for (int i = threadIdx.x; i < width; i += blockDim.x) hyb_store(out + (size_t)r * width + i, fmaf(tanhf(n.alpha * xr[i]), n.w[i], n.b ? n.b[i] : 0.f));
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) hyb_store(out + (size_t)r * width + i, xr[i]);
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
  if (!x || (n && (!out || (!n->w && n->kind != THA_NORM_COPY)))) return THA_STATUS_INVALID_ARG;
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

extern "C" int tha_hyb_side_gate(void* stream, int dtype, void* out, const float* gate_raw, long long ldg, const tha_side_t* side,
                                 const void* side_table, int side_cols, const int* token, int n_rows) {
  if (n_rows < 1 || !side || side->dim < 1) return THA_STATUS_SUCCESS;
  if (!out || !gate_raw || !side_table || !token || side->col0 < 0 || side->col0 + side->dim > side_cols) return THA_STATUS_INVALID_ARG;
  const dim3 grid(ceil_div(n_rows * side->dim, 256));
  if (dtype == THA_DT_BF16)
    THA_CUDA_OK(launch(hyb_side_gate_kernel<bf16>, grid, dim3(256), 0, (cudaStream_t)stream, false, (bf16*)out, gate_raw, ldg, (const bf16*)side_table,
                       side_cols, side->col0, token, n_rows, side->dim));
  else
    THA_CUDA_OK(launch(hyb_side_gate_kernel<float>, grid, dim3(256), 0, (cudaStream_t)stream, false, (float*)out, gate_raw, ldg,
                       (const float*)side_table, side_cols, side->col0, token, n_rows, side->dim));
  return THA_STATUS_SUCCESS;
}

extern "C" int tha_hyb_block_finish(void* stream, int dtype, float* x, const float* ff, const float* y, float m, const float* y_norm, float eps,
                                    float* tap, const float* embed_out, const float* vec, const tha_norm_t* next_norm, void* out, int n_rows,
                                    int width) {
  if (n_rows < 1) return THA_STATUS_SUCCESS;
  if (!x || (y && !y_norm) || (next_norm && (!out || (!next_norm->w && next_norm->kind != THA_NORM_COPY)))) return THA_STATUS_INVALID_ARG;
  const tha_norm_t none = {};
  const int nt = block_threads(width);
  if (dtype == THA_DT_BF16)
    THA_CUDA_OK(launch(hyb_block_finish_kernel<bf16>, dim3(n_rows), dim3(nt), 0, (cudaStream_t)stream, false, x, ff, y, m, y_norm, eps, tap, embed_out,
                       vec, next_norm ? *next_norm : none, next_norm ? 1 : 0, (bf16*)out, width));
  else
    THA_CUDA_OK(launch(hyb_block_finish_kernel<float>, dim3(n_rows), dim3(nt), 0, (cudaStream_t)stream, false, x, ff, y, m, y_norm, eps, tap, embed_out,
                       vec, next_norm ? *next_norm : none, next_norm ? 1 : 0, (float*)out, width));
  return THA_STATUS_SUCCESS;
}
