// Routed experts: each token runs `top` of E small gated feed-forwards, chosen by the largest router logits, and
// adds their outputs weighted by the softmax over the CHOSEN logits only.
//
//   llmi_moe_route    per token: the `top` largest of E fp32 logits (ties: the lower index), their softmax (fp32)
//   llmi_moe_up       per (token, choice): a = act(Wg_e h) * (Wu_e h)                      [T, top, F] fp32
//   llmi_moe_down     per token: y = sum over its choices, in the order of the choice, of weight * (Wd_e a)   [T, W] fp32
// The two product kernels stream an expert's rows once per (token, choice): the form for a handful of tokens (a
// decode step), where every chosen expert's weights are read once or a few times anyway.  Each output is one
// warp's sum in a fixed order, so a token's result does not depend on the batch it is in.
// Weights are stacked by expert: Wg, Wu [E, F, W], Wd [E, W, F], in the compute type; act: 0 silu, 1 tanh-GELU.
#include <math.h>

#include "common.cuh"

namespace llmi {

constexpr int MOE_MAX_PER_LANE = 8;      // experts per lane: E <= 256

// One warp per token.
__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, long ld, int E, int top, const int32_t* __restrict__ tok_seq,
                 int32_t* __restrict__ idx, float* __restrict__ wt, int n_tokens) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= n_tokens) return;
  if (tok_seq[t] < 0) {
    for (int j = lane; j < top; j += 32) { idx[(size_t)t * top + j] = -1; wt[(size_t)t * top + j] = 0.f; }
    return;
  }
  float v[MOE_MAX_PER_LANE];
#pragma unroll
  for (int i = 0; i < MOE_MAX_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? logits[(size_t)t * ld + e] : -INFINITY;
  }
  float first = 0.f, denom = 0.f, mine = 0.f;      // lane j keeps choice j's exp (top <= 32)
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < MOE_MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e < E && (v[i] > best || (v[i] == best && e < best_e))) { best = v[i]; best_e = e; }   // (a taken one is -inf: it never wins while a free one is left)
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    if (j == 0) first = best;                        // the largest logit: the softmax's shift
    const float ex = expf(best - first);
    denom += ex;
    if (lane == j) mine = ex;
    if (lane == 0) idx[(size_t)t * top + j] = best_e;
#pragma unroll
    for (int i = 0; i < MOE_MAX_PER_LANE; ++i)
      if (lane + 32 * i == best_e) v[i] = -INFINITY;   // taken
  }
  if (lane < top) wt[(size_t)t * top + lane] = mine / denom;
}

template <int ACT> __device__ __forceinline__ float moe_act(float g) {
  if (ACT == 0) return g / (1.0f + expf(-g));
  return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
}

// grid (T * top, ceil(F / rows per block)); 8 warps, one output f per warp at a time.
template <typename T, int ACT>
__global__ void __launch_bounds__(256)
moe_up_kernel(const T* __restrict__ h, long ldh, const T* __restrict__ wg, const T* __restrict__ wu, int W, int F, int top,
              const int32_t* __restrict__ idx, float* __restrict__ a, int f_per_block) {
  extern __shared__ float h_s[];
  pdl_launch_dependents();
  pdl_wait();
  const int item = blockIdx.x, t = item / top;
  const int e = idx[item];
  if (e < 0) return;
  for (int i = threadIdx.x; i < W; i += blockDim.x) h_s[i] = to_f32(h[(size_t)t * ldh + i]);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int f0 = blockIdx.y * f_per_block, f1 = min(F, f0 + f_per_block);
  for (int f = f0 + warp; f < f1; f += 8) {
    const T* g_row = wg + ((size_t)e * F + f) * W;
    const T* u_row = wu + ((size_t)e * F + f) * W;
    float g = 0.f, u = 0.f;
    for (int i = lane; i < W; i += 32) {
      g = fmaf(h_s[i], to_f32(g_row[i]), g);
      u = fmaf(h_s[i], to_f32(u_row[i]), u);
    }
    g = warp_sum(g);
    u = warp_sum(u);
    if (lane == 0) a[(size_t)item * F + f] = moe_act<ACT>(g) * u;
  }
}

// grid (T, ceil(W / rows per block)).
template <typename T>
__global__ void __launch_bounds__(256)
moe_down_kernel(const float* __restrict__ a, const T* __restrict__ wd, int W, int F, int top, const int32_t* __restrict__ idx,
                const float* __restrict__ wt, float* __restrict__ y, long ldy, int c_per_block) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c0 = blockIdx.y * c_per_block, c1 = min(W, c0 + c_per_block);
  for (int c = c0 + warp; c < c1; c += 8) {
    float total = 0.f;
    for (int j = 0; j < top; ++j) {
      const int e = idx[(size_t)t * top + j];
      if (e < 0) continue;
      const T* row = wd + ((size_t)e * W + c) * F;
      const float* aj = a + ((size_t)t * top + j) * F;
      float s = 0.f;
      for (int i = lane; i < F; i += 32) s = fmaf(aj[i], to_f32(row[i]), s);
      s = warp_sum(s);
      total = fmaf(wt[(size_t)t * top + j], s, total);
    }
    if (lane == 0) y[(size_t)t * ldy + c] = total;
  }
}

}  // namespace llmi

using namespace llmi;

LLMI_EXPORT int llmi_moe_route(const float* logits, long ld, int E, int top, const int32_t* tok_seq, int32_t* idx, float* wt,
                               int n_tokens, cudaStream_t stream) {
  if (n_tokens <= 0 || E <= 0 || top <= 0 || top > E || top > 32 || E > 32 * MOE_MAX_PER_LANE) return LLMI_ERR_BAD_SIZE;
  return launch_pdl(PDL_SMALL, moe_route_kernel, (n_tokens + 3) / 4, 128, 0, stream, logits, ld, E, top, tok_seq, idx, wt, n_tokens);
}

LLMI_EXPORT int llmi_moe_up(int dtype, const void* h, long ldh, const void* wg, const void* wu, int W, int F, int top,
                            const int32_t* idx, float* a, int act, int n_tokens, cudaStream_t stream) {
  if (n_tokens <= 0 || W <= 0 || F <= 0 || top <= 0 || (size_t)W * 4 > 160 * 1024) return LLMI_ERR_BAD_SIZE;
  if (act != 0 && act != 1) return LLMI_ERR_UNSUPPORTED;
  const int f_per_block = 64;
  dim3 grid(n_tokens * top, (F + f_per_block - 1) / f_per_block);
  if (grid.y > 65535) return LLMI_ERR_BAD_SIZE;
  const size_t smem = (size_t)W * 4;
#define LLMI_UP(T, ACT)                                                                                                   \
  do {                                                                                                                    \
    static PerDevice<size_t> allowed;                                                                                     \
    if (smem > 48 * 1024 && allowed.here() < smem) {                                                                      \
      if (cudaFuncSetAttribute(moe_up_kernel<T, ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
        return LLMI_ERR_BAD_SIZE;                                                                                         \
      allowed.here() = smem;                                                                                              \
    }                                                                                                                     \
    return launch_pdl(PDL_GEMM, moe_up_kernel<T, ACT>, grid, dim3(256), smem, stream, (const T*)h, ldh, (const T*)wg,     \
                      (const T*)wu, W, F, top, idx, a, f_per_block);                                                      \
  } while (0)
  if (dtype == LLMI_DTYPE_F32) { if (act == 0) LLMI_UP(float, 0); else LLMI_UP(float, 1); }
  if (dtype == LLMI_DTYPE_BF16) { if (act == 0) LLMI_UP(__nv_bfloat16, 0); else LLMI_UP(__nv_bfloat16, 1); }
#undef LLMI_UP
  return LLMI_ERR_BAD_DTYPE;
}

LLMI_EXPORT int llmi_moe_down(int dtype, const float* a, const void* wd, int W, int F, int top, const int32_t* idx,
                              const float* wt, float* y, long ldy, int n_tokens, cudaStream_t stream) {
  if (n_tokens <= 0 || W <= 0 || F <= 0 || top <= 0) return LLMI_ERR_BAD_SIZE;
  const int c_per_block = 64;
  dim3 grid(n_tokens, (W + c_per_block - 1) / c_per_block);
  if (grid.y > 65535) return LLMI_ERR_BAD_SIZE;
  if (dtype == LLMI_DTYPE_F32)
    return launch_pdl(PDL_GEMM, moe_down_kernel<float>, grid, dim3(256), 0, stream, a, (const float*)wd, W, F, top, idx, wt, y, ldy,
                      c_per_block);
  if (dtype == LLMI_DTYPE_BF16)
    return launch_pdl(PDL_GEMM, moe_down_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, a, (const __nv_bfloat16*)wd, W, F, top,
                      idx, wt, y, ldy, c_per_block);
  return LLMI_ERR_BAD_DTYPE;
}
