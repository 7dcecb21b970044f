// Residual streams, the PolyNorm activation and the combination of differential attention (include/tha_hybrid.h).
//
//   hyb_streams_kernel<NS>     one block per row, one pass over the row's n streams: the previous sublayer's write
//                              X'[t] = sum_s mix[s, t] X[s] + out[t] y (y = a dense result + bias, or a mixture's chosen experts by
//                              router weight), the tap sum_s X'[s], and the next sublayer's read u = sum_s in[s] X'[s] with its rms
//                              norm -- what would be three passes over n x width floats is one.  u waits in shared memory for
//                              the row's sum of squares.
//   hyb_polynorm_kernel        c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3 over a row z = up + bias, N(v) = v / sqrt(mean(v^2) + eps):
//                              one block per row, the three sums of squares (z^2, z^4, z^6) in one sweep, the result in a second.
//   hyb_diff_combine_kernel    a warp per (row, head): o = a1 - lambda a2, o / rms(o) * mult * sigmoid(gate).
// Everything here is fp32 arithmetic in both number formats; only results that feed a matrix product are rounded.
#include <cuda_bf16.h>

#include "common.cuh"
#include "hybrid_ops.cuh"
#include "tha_hybrid.h"

namespace tha {

struct StreamsArgs {
  float* X; int n;
  const float* init;
  const float* w_out; const float* w_mix;     // write (w_out NULL: none)
  const float* dense; const float* bias;
  int top; const float* weight; const int* inv; const float* down;
  float* tap; float* sum_out;
  const float* r_in;                          // read (NULL: none)
  int norm_kind; const float* norm_w; float norm_off; float eps;
  int width;
};

// V consecutive floats (V = 4: one 128-bit access; the callers check the alignment)
template <int V> __device__ __forceinline__ void ldv(const float* p, float* o) {
  if (V == 4) { const float4 t = *reinterpret_cast<const float4*>(p); o[0] = t.x; o[1] = t.y; o[2] = t.z; o[3] = t.w; }
  else o[0] = *p;
}
template <int V> __device__ __forceinline__ void stv(float* p, const float* o) {
  if (V == 4) *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]);
  else *p = o[0];
}
template <int V> __device__ __forceinline__ void stv(__nv_bfloat16* p, const float* o) {
  if (V == 4) {
    uint2 pk;
    const __nv_bfloat162 a = __floats2bfloat162_rn(o[0], o[1]), b = __floats2bfloat162_rn(o[2], o[3]);
    pk.x = *reinterpret_cast<const unsigned*>(&a); pk.y = *reinterpret_cast<const unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = pk;
  } else {
    *p = __float2bfloat16_rn(o[0]);
  }
}

template <int NS, typename T, int V>
__global__ void __launch_bounds__(512) hyb_streams_kernel(StreamsArgs a, T* __restrict__ out) {
  extern __shared__ __align__(16) float u_row[];   // [width] when a read follows
  __shared__ float red[33];
  __shared__ float c_mix[NS * NS], c_out[NS], c_in[NS];
  const int r = blockIdx.x, n = a.n, W = a.width;
  for (int k = threadIdx.x; k < NS * NS; k += blockDim.x) {
    const int s = k / NS, t = k % NS;
    c_mix[k] = (a.w_out && s < n && t < n) ? a.w_mix[s * n + t] : 0.f;
  }
  if (threadIdx.x < NS) {
    c_out[threadIdx.x] = (a.w_out && threadIdx.x < n) ? a.w_out[threadIdx.x] : 0.f;
    c_in[threadIdx.x] = (a.r_in && threadIdx.x < n) ? a.r_in[threadIdx.x] : 0.f;
  }
  __syncthreads();
  float* xr = a.X + (size_t)r * n * W;
  float ss = 0.f;
  for (int i = V * threadIdx.x; i < W; i += V * blockDim.x) {
    float x[NS][V];
#pragma unroll
    for (int s = 0; s < NS; s++) {
      if (s < n) ldv<V>(a.init ? a.init + (size_t)r * W + i : xr + (size_t)s * W + i, x[s]);
      else
#pragma unroll
        for (int v = 0; v < V; v++) x[s][v] = 0.f;
    }
    if (a.w_out) {
      float y[V], t4[V];
#pragma unroll
      for (int v = 0; v < V; v++) y[v] = 0.f;
      if (a.dense) ldv<V>(a.dense + (size_t)r * W + i, y);
      if (a.bias) {
        ldv<V>(a.bias + i, t4);
#pragma unroll
        for (int v = 0; v < V; v++) y[v] += t4[v];
      }
      for (int j = 0; j < a.top; j++) {
        const float wj = a.weight[(size_t)r * a.top + j];
        ldv<V>(a.down + (size_t)a.inv[(size_t)r * a.top + j] * W + i, t4);
#pragma unroll
        for (int v = 0; v < V; v++) y[v] = fmaf(wj, t4[v], y[v]);
      }
      float nx[NS][V];
#pragma unroll
      for (int t = 0; t < NS; t++)
#pragma unroll
        for (int v = 0; v < V; v++) {
          float acc = c_out[t] * y[v];
#pragma unroll
          for (int s = 0; s < NS; s++) acc = fmaf(c_mix[s * NS + t], x[s][v], acc);
          nx[t][v] = acc;
        }
#pragma unroll
      for (int t = 0; t < NS; t++)
#pragma unroll
        for (int v = 0; v < V; v++) x[t][v] = nx[t][v];
    }
    if (a.w_out || a.init) {
#pragma unroll
      for (int s = 0; s < NS; s++)
        if (s < n) stv<V>(xr + (size_t)s * W + i, x[s]);
    }
    if (a.tap || a.sum_out) {
      float sum[V];
#pragma unroll
      for (int v = 0; v < V; v++) {
        sum[v] = 0.f;
#pragma unroll
        for (int s = 0; s < NS; s++) sum[v] += x[s][v];
      }
      if (a.tap) stv<V>(a.tap + (size_t)r * W + i, sum);
      if (a.sum_out) stv<V>(a.sum_out + (size_t)r * W + i, sum);
    }
    if (a.r_in) {
      float u[V];
#pragma unroll
      for (int v = 0; v < V; v++) {
        u[v] = 0.f;
#pragma unroll
        for (int s = 0; s < NS; s++) u[v] = fmaf(c_in[s], x[s][v], u[v]);
        ss = fmaf(u[v], u[v], ss);
      }
      stv<V>(u_row + i, u);
    }
  }
  if (!a.r_in) return;
  float inv = 1.0f;
  if (a.norm_kind == THA_NORM_RMS) {
    ss = block_sum(ss, red);
    inv = 1.0f / sqrtf(ss / (float)W + a.eps);
  }
  for (int i = V * threadIdx.x; i < W; i += V * blockDim.x) {   // a thread reads back the entries it wrote
    float u[V], w[V];
    ldv<V>(u_row + i, u);
    if (a.norm_kind == THA_NORM_RMS) {
      ldv<V>(a.norm_w + i, w);
#pragma unroll
      for (int v = 0; v < V; v++) u[v] = u[v] * inv * (a.norm_off + w[v]);
    }
    stv<V>(out + (size_t)r * W + i, u);
  }
}

template <typename T, int V>
__global__ void __launch_bounds__(256) hyb_polynorm_kernel(T* __restrict__ y, const float* __restrict__ gu, long long ldg, int col_u,
                                                           const float* __restrict__ bias, float c0, float c1, float c2, float c3, float eps, int ff) {
  __shared__ float red[33];
  const size_t r = blockIdx.x;
  const float* z = gu + r * ldg + col_u;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int i = V * threadIdx.x; i < ff; i += V * blockDim.x) {
    float v[V], b[V];
    ldv<V>(z + i, v);
    if (bias) ldv<V>(bias + i, b);
#pragma unroll
    for (int k = 0; k < V; k++) {
      const float x = v[k] + (bias ? b[k] : 0.f), x2 = x * x;
      s2 += x2;
      s4 = fmaf(x2, x2, s4);
      s6 = fmaf(x2 * x, x2 * x, s6);
    }
  }
  s2 = block_sum(s2, red);
  s4 = block_sum(s4, red);
  s6 = block_sum(s6, red);
  const float i1 = c0 / sqrtf(s2 / (float)ff + eps), i2 = c1 / sqrtf(s4 / (float)ff + eps), i3 = c2 / sqrtf(s6 / (float)ff + eps);
  for (int i = V * threadIdx.x; i < ff; i += V * blockDim.x) {
    float v[V], b[V], o[V];
    ldv<V>(z + i, v);
    if (bias) ldv<V>(bias + i, b);
#pragma unroll
    for (int k = 0; k < V; k++) {
      const float x = v[k] + (bias ? b[k] : 0.f), x2 = x * x;
      o[k] = fmaf(i1, x, fmaf(i2, x2, fmaf(i3, x2 * x, c3)));
    }
    stv<V>(y + r * ff + i, o);
  }
}

// att [n_rows, 2 H E] in map order: per key/value group g the first maps of its gs heads, then their second maps
template <typename T>
__global__ void hyb_diff_combine_kernel(T* __restrict__ out, const float* __restrict__ att, int n_rows, int H, int gs, int E, float lambda,
                                        float mult, float eps, const float* __restrict__ gate, long long ldg) {
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (idx >= n_rows * H) return;
  const int r = idx / H, h = idx - r * H, g = h / gs, hh = h - g * gs;
  const float* a1 = att + (size_t)r * 2 * H * E + (size_t)((2 * g) * gs + hh) * E;
  const float* a2 = att + (size_t)r * 2 * H * E + (size_t)((2 * g + 1) * gs + hh) * E;
  float ss = 0.f;
  for (int e = lane; e < E; e += 32) { const float o = fmaf(-lambda, a2[e], a1[e]); ss = fmaf(o, o, ss); }
  ss = warp_sum(ss);
  float f = mult / sqrtf(ss / (float)E + eps);
  if (gate) f *= hyb_sigmoid(gate[(size_t)r * ldg + h]);
  for (int e = lane; e < E; e += 32) hyb_store(out + (size_t)r * H * E + (size_t)h * E + e, fmaf(-lambda, a2[e], a1[e]) * f);
}

template <int NS>
static int streams_launch(cudaStream_t s, const StreamsArgs& a, int out_kind, void* out, int n_rows) {
  const size_t smem = a.r_in ? (size_t)a.width * sizeof(float) : 0;
  // four columns per thread where every row starts on a 16-byte boundary
  constexpr int VV = NS <= 4 ? 4 : 1;   // more streams than four would not fit a thread's registers four columns at a time
  const bool vec = VV == 4 && a.width % 4 == 0 && aligned16(a.X) && aligned16(a.init) && aligned16(a.dense) && aligned16(a.bias) && aligned16(a.down) &&
                   aligned16(a.tap) && aligned16(a.sum_out) && aligned16(a.norm_w) && aligned16(out);
  const int per = vec ? 4 : 1;
  int nt = 64;
  while (nt < 512 && nt * per < a.width) nt *= 2;
#define STREAMS_GO(T, V)                                                                                                               \
  do {                                                                                                                                 \
    if (smem > 48 * 1024) THA_CUDA_OK(cudaFuncSetAttribute(hyb_streams_kernel<NS, T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    THA_CUDA_OK(launch(hyb_streams_kernel<NS, T, V>, dim3(n_rows), dim3(nt), smem, s, false, a, (T*)out));                             \
  } while (0)
  if (out_kind == 0) { if (vec) STREAMS_GO(float, VV); else STREAMS_GO(float, 1); }
  else { if (vec) STREAMS_GO(__nv_bfloat16, VV); else STREAMS_GO(__nv_bfloat16, 1); }
#undef STREAMS_GO
  return THA_STATUS_SUCCESS;
}

}  // namespace tha

using namespace tha;
typedef __nv_bfloat16 bf16;

extern "C" int tha_hyb_streams(void* stream, int dtype, float* X, int n, const float* init, const tha_streams_t* write, const float* dense,
                               const float* bias, int top, const float* weight, const int* inv, const float* down, float* tap,
                               float* sum_out, const tha_streams_t* read, const tha_norm_t* norm, float eps, int out_f32, void* out,
                               int n_rows, int width) {
  if (n_rows < 1) return THA_STATUS_SUCCESS;
  if (!X || n < 1 || n > 16 || width < 1 || (read && (!norm || !out))) return THA_STATUS_INVALID_ARG;
  if (read && norm->kind != THA_NORM_RMS && norm->kind != THA_NORM_COPY) return THA_STATUS_NOT_SUPPORTED;
  if ((size_t)width * sizeof(float) > 200 * 1024) return THA_STATUS_NOT_SUPPORTED;
  StreamsArgs a;
  a.X = X; a.n = n; a.init = init;
  a.w_out = write ? write->out : nullptr; a.w_mix = write ? write->mix : nullptr;
  a.dense = write ? dense : nullptr; a.bias = write ? bias : nullptr;
  a.top = write ? top : 0; a.weight = weight; a.inv = inv; a.down = down;
  a.tap = tap; a.sum_out = sum_out;
  a.r_in = read ? read->in : nullptr;
  a.norm_kind = read ? norm->kind : THA_NORM_COPY; a.norm_w = read ? norm->w : nullptr; a.norm_off = read ? norm->w_offset : 0.f; a.eps = eps;
  a.width = width;
  cudaStream_t s = (cudaStream_t)stream;
  const int out_kind = (out_f32 || dtype == THA_DT_F32) ? 0 : 1;
  if (n <= 1) return streams_launch<1>(s, a, out_kind, out, n_rows);
  if (n <= 2) return streams_launch<2>(s, a, out_kind, out, n_rows);
  if (n <= 3) return streams_launch<3>(s, a, out_kind, out, n_rows);
  if (n <= 4) return streams_launch<4>(s, a, out_kind, out, n_rows);
  if (n <= 8) return streams_launch<8>(s, a, out_kind, out, n_rows);
  return streams_launch<16>(s, a, out_kind, out, n_rows);
}

extern "C" int tha_hyb_polynorm(void* stream, int dtype, void* y, const float* gu, long long ldg, int col_u, const float* bias, const float* c,
                                float eps, int n, int ff) {
  if (n < 1 || ff < 1) return THA_STATUS_SUCCESS;
  cudaStream_t s = (cudaStream_t)stream;
  const bool vec = ff % 4 == 0 && ldg % 4 == 0 && col_u % 4 == 0 && aligned16(gu) && aligned16(bias) && aligned16(y);
  const int nt = ff >= (vec ? 4096 : 1024) ? 256 : 128;
#define POLY_GO(T, V) \
  THA_CUDA_OK(launch(hyb_polynorm_kernel<T, V>, dim3(n), dim3(nt), 0, s, false, (T*)y, gu, ldg, col_u, bias, c[0], c[1], c[2], c[3], eps, ff))
  if (dtype == THA_DT_BF16) { if (vec) POLY_GO(bf16, 4); else POLY_GO(bf16, 1); }
  else { if (vec) POLY_GO(float, 4); else POLY_GO(float, 1); }
#undef POLY_GO
  return THA_STATUS_SUCCESS;
}

extern "C" int tha_hyb_diff_combine(void* stream, int dtype, const tha_attn_t* a, const float* att, const float* proj, long long ldp, void* out,
                                    int n_rows) {
  if (n_rows < 1) return THA_STATUS_SUCCESS;
  if (!a->diff || (a->heads & 1) || (a->kv_heads & 1) || a->heads % a->kv_heads) return THA_STATUS_INVALID_ARG;
  const int H = a->heads / 2, gs = a->heads / a->kv_heads;
  const float* gate = (a->head_gate && proj) ? proj + a->o_g : nullptr;
  cudaStream_t s = (cudaStream_t)stream;
  const dim3 grid(ceil_div(n_rows * H, 4));
  if (dtype == THA_DT_BF16)
    THA_CUDA_OK(launch(hyb_diff_combine_kernel<bf16>, grid, dim3(128), 0, s, false, (bf16*)out, att, n_rows, H, gs, a->vdim, a->diff_lambda, a->diff_mult,
                       a->eps, gate, ldp));
  else
    THA_CUDA_OK(launch(hyb_diff_combine_kernel<float>, grid, dim3(128), 0, s, false, (float*)out, att, n_rows, H, gs, a->vdim, a->diff_lambda, a->diff_mult,
                       a->eps, gate, ldp));
  return THA_STATUS_SUCCESS;
}
