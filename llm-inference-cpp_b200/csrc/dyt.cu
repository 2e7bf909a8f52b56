// Dynamic Tanh: a norm that computes no statistics, y = tanh(alpha * x) * w + b, with a scalar alpha and
// vectors w, b.  All arithmetic is fp32; the result is stored in the compute type or added to the fp32
// residual stream.
//
// Two uses:
//   llmi_dyt       h[r] = dyt(x[rows ? rows[r] : r])                      (a norm ahead of a sublayer, or the last norm)
//   llmi_dyt_add   x += dyt_a(y)  and, optionally,  h = dyt_b(x)          (the norm BEHIND a sublayer, whose result
//                                                                          joins the residual stream, fused with the
//                                                                          norm ahead of the next sublayer)
// Elementwise, so every row is treated alone and a row's bits do not depend on its neighbours.
#include "common.cuh"

namespace llmi {

struct DytParams {
  const float* w;
  const float* b;
  float alpha;
};

__device__ __forceinline__ float dyt_one(float v, float alpha, float w, float b) { return fmaf(tanhf(alpha * v), w, b); }

template <typename T>
__global__ void __launch_bounds__(256)
dyt_kernel(const float* __restrict__ x, DytParams p, T* __restrict__ out, const int32_t* __restrict__ rows, int n_rows,
           int width) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = (size_t)n_rows * width;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / width), c = (int)(i - (size_t)r * width);
    const int src = rows ? rows[r] : r;
    out[i] = from_f32<T>(src < 0 ? 0.f : dyt_one(x[(size_t)src * width + c], p.alpha, p.w[c], p.b[c]));
  }
}

template <typename T, bool NEXT>
__global__ void __launch_bounds__(256)
dyt_add_kernel(const float* __restrict__ y, DytParams a, float* __restrict__ x, DytParams b, T* __restrict__ h,
               int n_rows, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = (size_t)n_rows * width;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % width);
    const float v = x[i] + dyt_one(y[i], a.alpha, a.w[c], a.b[c]);
    x[i] = v;
    if (NEXT) h[i] = from_f32<T>(dyt_one(v, b.alpha, b.w[c], b.b[c]));
  }
}

inline int dyt_blocks(size_t total) {
  const size_t most = (size_t)sm_count() * 16, need = (total + 255) / 256;
  return (int)(need < most ? need : most);
}

}  // namespace llmi

using namespace llmi;

LLMI_EXPORT int llmi_dyt(int out_dtype, const float* x, const float* w, const float* b, float alpha, void* out,
                         const int32_t* rows, int n_rows, int width, cudaStream_t stream) {
  if (n_rows <= 0 || width <= 0) return LLMI_ERR_BAD_SIZE;
  const DytParams p{w, b, alpha};
  const int blocks = dyt_blocks((size_t)n_rows * width);
  if (out_dtype == LLMI_DTYPE_F32)
    return launch_pdl(PDL_SMALL, dyt_kernel<float>, blocks, 256, 0, stream, x, p, (float*)out, rows, n_rows, width);
  if (out_dtype == LLMI_DTYPE_BF16)
    return launch_pdl(PDL_SMALL, dyt_kernel<__nv_bfloat16>, blocks, 256, 0, stream, x, p, (__nv_bfloat16*)out, rows, n_rows, width);
  return LLMI_ERR_BAD_DTYPE;
}

// x += tanh(alpha_a y) w_a + b_a; if h is given, h = tanh(alpha_b x) w_b + b_b of the updated x.
LLMI_EXPORT int llmi_dyt_add(const float* y, const float* w_a, const float* b_a, float alpha_a, float* x, int h_dtype,
                             void* h, const float* w_b, const float* b_b, float alpha_b, int n_rows, int width,
                             cudaStream_t stream) {
  if (n_rows <= 0 || width <= 0) return LLMI_ERR_BAD_SIZE;
  const DytParams a{w_a, b_a, alpha_a}, b{w_b, b_b, alpha_b};
  const int blocks = dyt_blocks((size_t)n_rows * width);
  if (!h)
    return launch_pdl(PDL_SMALL, dyt_add_kernel<float, false>, blocks, 256, 0, stream, y, a, x, b, (float*)nullptr, n_rows, width);
  if (h_dtype == LLMI_DTYPE_F32)
    return launch_pdl(PDL_SMALL, dyt_add_kernel<float, true>, blocks, 256, 0, stream, y, a, x, b, (float*)h, n_rows, width);
  if (h_dtype == LLMI_DTYPE_BF16)
    return launch_pdl(PDL_SMALL, dyt_add_kernel<__nv_bfloat16, true>, blocks, 256, 0, stream, y, a, x, b, (__nv_bfloat16*)h, n_rows, width);
  return LLMI_ERR_BAD_DTYPE;
}

// x[t] += add[t] (optional, same shape) + vec (optional, one row for all): what a pass of a looped span adds to the
// stream ahead of its first layer.  Rows alone; fp32.
namespace llmi {
__global__ void __launch_bounds__(256)
stream_add_kernel(float* __restrict__ x, const float* __restrict__ add, const float* __restrict__ vec, int n_rows, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = (size_t)n_rows * width;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    float v = x[i];
    if (add) v += add[i];
    if (vec) v += vec[i % width];
    x[i] = v;
  }
}
}  // namespace llmi

LLMI_EXPORT int llmi_stream_add(float* x, const float* add, const float* vec, int n_rows, int width, cudaStream_t stream) {
  if (n_rows <= 0 || width <= 0) return LLMI_ERR_BAD_SIZE;
  return launch_pdl(PDL_SMALL, stream_add_kernel, dyt_blocks((size_t)n_rows * width), 256, 0, stream, x, add, vec, n_rows, width);
}
