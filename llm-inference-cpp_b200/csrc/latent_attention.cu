// Attention through a low-rank latent ("latent attention"): every token leaves ONE row in the cache,
//     [ c (rank C, RMS-normed) | r (R dims, rotated by position) ],
// and all heads read it.  With the key and value expansions folded into the query and the output
// (q~_h = Uk_hᵀ q_h, out_h = Uv_h Σ p c), a head's score is the plain dot of its query row [q~_h | qrot_h] with the
// cache row, and its context is the weighted sum of the rows' first C entries: multi-query attention with one
// shared head of C + R key dims whose values are the first C of them.
//
// Kernels here:
//   llmi_latent_prepare     per token: RMS norm of the query latent and of c (fp32), rotation of r, append to the cache
//   llmi_latent_q_rotate    the rotated part of every head's query into its row [q~ | qrot]
//   llmi_attention_latent   scores, softmax and context of every (token, head), any sizes, fp32 arithmetic; serves
//                           prompts and single tokens, both types
// Rotation: neighbouring pairs (2i, 2i+1) by the angle float(pos) * inv_freq[i], computed in fp32 with sincosf;
// entries beyond rot_dims pass unchanged.
#include <math.h>

#include "common.cuh"
#include "step_meta.cuh"

namespace llmi {

// One block per token.  down: fp32 [T, ld]: columns [0, Q) query latent, [Q, Q+C) key/value latent, [Q+C, Q+C+R)
// the shared key part.  cq (type T) [T, Q] receives the normed query latent; the cache row of (sequence, position)
// receives [normed c | rotated r].
template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const float* __restrict__ down, long ld, int Q, int C, int R, const float* __restrict__ wq,
                      const float* __restrict__ wc, float eps, const float* __restrict__ inv_freq, int rot_dims,
                      const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ tok_pos, PagedKV kv,
                      T* __restrict__ cache, T* __restrict__ cq, int write_kv) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int seq = tok_seq[t];
  T* cq_row = cq + (size_t)t * Q;
  if (seq < 0) {
    for (int i = threadIdx.x; i < Q; i += blockDim.x) cq_row[i] = from_f32<T>(0.f);
    return;
  }
  const float* row = down + (size_t)t * ld;
  float ss = 0.f;
  for (int i = threadIdx.x; i < Q; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
  ss = block_sum(ss, scratch);
  const float sq = 1.0f / sqrtf(ss / (float)Q + eps);
  for (int i = threadIdx.x; i < Q; i += blockDim.x) cq_row[i] = from_f32<T>(wq[i] * (row[i] * sq));
  if (!write_kv) return;
  const float* c = row + Q;
  ss = 0.f;
  for (int i = threadIdx.x; i < C; i += blockDim.x) ss = fmaf(c[i], c[i], ss);
  ss = block_sum(ss, scratch);
  const float sc = 1.0f / sqrtf(ss / (float)C + eps);
  const int pos = tok_pos[t];
  T* dst = cache + kv_row_offset(kv, seq, pos, 0);
  for (int i = threadIdx.x; i < C; i += blockDim.x) dst[i] = from_f32<T>(wc[i] * (c[i] * sc));
  const float* r = c + C;
  for (int i = threadIdx.x; i < (R + 1) / 2; i += blockDim.x) {
    const int a = 2 * i, b = 2 * i + 1;
    if (b < rot_dims) {
      float s, co;
      sincosf((float)pos * inv_freq[i], &s, &co);
      dst[C + a] = from_f32<T>(rot_lo(r[a], r[b], co, s));
      dst[C + b] = from_f32<T>(rot_hi(r[a], r[b], co, s));
    } else {
      dst[C + a] = from_f32<T>(r[a]);
      if (b < R) dst[C + b] = from_f32<T>(r[b]);
    }
  }
}

// q (type T) [T, H, D + R] holds every head's plain part and its part to rotate; qa [T, H, C + R] receives the
// rotated part behind the C entries that the folded key expansion fills.
template <typename T>
__global__ void __launch_bounds__(256)
latent_q_rotate_kernel(const T* __restrict__ q, long ldq, int D, T* __restrict__ qa, long ldqa, int C, int R, int H,
                       const float* __restrict__ inv_freq, int rot_dims, const int32_t* __restrict__ tok_seq,
                       const int32_t* __restrict__ tok_pos, int n_tokens) {
  pdl_launch_dependents();
  pdl_wait();
  const int half = (R + 1) / 2;
  const size_t total = (size_t)n_tokens * H * half;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int i = (int)(idx % half);
    const int h = (int)((idx / half) % H);
    const int t = (int)(idx / ((size_t)half * H));
    const T* src = q + (size_t)t * ldq + (size_t)h * (D + R) + D;
    T* dst = qa + (size_t)t * ldqa + (size_t)h * (C + R) + C;
    const int a = 2 * i, b = 2 * i + 1;
    if (tok_seq[t] < 0) {
      dst[a] = from_f32<T>(0.f);
      if (b < R) dst[b] = from_f32<T>(0.f);
      continue;
    }
    if (b < rot_dims) {
      float s, co;
      sincosf((float)tok_pos[t] * inv_freq[i], &s, &co);
      const float u = to_f32(src[a]), v = to_f32(src[b]);
      dst[a] = from_f32<T>(rot_lo(u, v, co, s));
      dst[b] = from_f32<T>(rot_hi(u, v, co, s));
    } else {
      dst[a] = src[a];
      if (b < R) dst[b] = src[b];
    }
  }
}

constexpr int LAT_WARPS = 8;

// One block per (token, group of LAT_WARPS heads), one warp per head.  Keys are taken 32 at a time, in blocks anchored
// at positions 0, 32, 64, ..., staged once in shared memory (fp32) for all heads of the block: lane = key for the
// scores, lane = column for the context.  The order of every addition depends only on the key's position, so the
// result does not depend on how a prompt was cut or batched.  NJ = ceil(C / 32).
template <typename T, int NJ>
__global__ void __launch_bounds__(LAT_WARPS * 32)
attention_latent_kernel(const T* __restrict__ qa, long ldq, T* __restrict__ out, long ldo, const T* __restrict__ cache,
                        const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ tok_pos, PagedKV kv, int n_heads,
                        int C, float scale) {
  extern __shared__ float smem[];
  pdl_wait();
  pdl_launch_dependents();
  const int Dk = kv.head_dim;
  const int kstride = Dk | 1;                                 // odd: lanes on different keys hit different banks
  float* q_s = smem;                                          // [LAT_WARPS][Dk]
  float* k_s = smem + LAT_WARPS * Dk;                         // [32][kstride]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x, h = blockIdx.y * LAT_WARPS + warp;
  const bool head_ok = h < n_heads;
  const int seq = tok_seq[t];
  T* o = out + (size_t)t * ldo + (size_t)h * C;
  if (seq < 0) {
    if (head_ok)
      for (int d = lane; d < C; d += 32) o[d] = from_f32<T>(0.f);
    return;
  }
  const int pos = tok_pos[t];
  if (head_ok) {
    const T* qp = qa + (size_t)t * ldq + (size_t)h * Dk;
    for (int d = lane; d < Dk; d += 32) q_s[warp * Dk + d] = to_f32(qp[d]);
  }
  float m = -INFINITY, l = 0.f;
  float acc[NJ];
#pragma unroll
  for (int j = 0; j < NJ; ++j) acc[j] = 0.f;

  for (int c0 = 0; c0 <= pos; c0 += 32) {
    __syncthreads();                                          // the block before is read out (and q_s is written)
    const int n_rows = (pos - c0 + 1 < 32) ? pos - c0 + 1 : 32;
    for (int r = warp; r < n_rows; r += LAT_WARPS) {
      const T* kr = cache + kv_row_offset(kv, seq, c0 + r, 0);
      for (int d = lane; d < Dk; d += 32) k_s[r * kstride + d] = to_f32(kr[d]);
    }
    __syncthreads();
    if (!head_ok) continue;
    const bool valid = lane < n_rows;
    float score = -INFINITY;
    if (valid) {
      const float* kq = k_s + lane * kstride;
      const float* qq = q_s + warp * Dk;
      float a = 0.f;
      for (int d = 0; d < Dk; ++d) a = fmaf(qq[d], kq[d], a);
      score = a * scale;
    }
    const float m_new = fmaxf(m, warp_max(score));
    const float p = valid ? expf(score - m_new) : 0.f;
    const float corr = expf(m - m_new);                       // first block: exp(-inf) = 0
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int j = 0; j < NJ; ++j) acc[j] *= corr;
    for (int kk = 0; kk < n_rows; ++kk) {
      const float pk = __shfl_sync(0xffffffffu, p, kk);
      const float* vr = k_s + kk * kstride;
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const int d = lane + 32 * j;
        if (d < C) acc[j] = fmaf(pk, vr[d], acc[j]);
      }
    }
    m = m_new;
  }
  if (!head_ok) return;
  const float inv = 1.0f / l;
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    const int d = lane + 32 * j;
    if (d < C) o[d] = from_f32<T>(acc[j] * inv);
  }
}

template <typename T, int NJ>
int launch_attention_latent_nj(const void* qa, long ldq, void* out, long ldo, const void* cache, const int32_t* tok_seq,
                               const int32_t* tok_pos, PagedKV kv, int n_tokens, int n_heads, int C, float scale,
                               cudaStream_t stream) {
  const size_t smem = ((size_t)LAT_WARPS * kv.head_dim + 32 * (size_t)(kv.head_dim | 1)) * sizeof(float);
  static PerDevice<size_t> allowed;
  if (smem > 48 * 1024 && allowed.here() < smem) {
    if (cudaFuncSetAttribute(attention_latent_kernel<T, NJ>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return LLMI_ERR_BAD_SIZE;
    allowed.here() = smem;
  }
  dim3 grid(n_tokens, (n_heads + LAT_WARPS - 1) / LAT_WARPS);
  return launch_pdl(PDL_ATTENTION, attention_latent_kernel<T, NJ>, grid, dim3(LAT_WARPS * 32), smem, stream, (const T*)qa, ldq,
                    (T*)out, ldo, (const T*)cache, tok_seq, tok_pos, kv, n_heads, C, scale);
}

template <typename T>
int launch_attention_latent(const void* qa, long ldq, void* out, long ldo, const void* cache, const int32_t* tok_seq,
                            const int32_t* tok_pos, PagedKV kv, int n_tokens, int n_heads, int C, float scale,
                            cudaStream_t stream) {
  const int nj = (C + 31) / 32;
#define LLMI_LAT(NJ) \
  return launch_attention_latent_nj<T, NJ>(qa, ldq, out, ldo, cache, tok_seq, tok_pos, kv, n_tokens, n_heads, C, scale, stream)
  if (nj <= 1) LLMI_LAT(1);
  if (nj <= 2) LLMI_LAT(2);
  if (nj <= 4) LLMI_LAT(4);
  if (nj <= 8) LLMI_LAT(8);
  if (nj <= 16) LLMI_LAT(16);
  if (nj <= 32) LLMI_LAT(32);
#undef LLMI_LAT
  return LLMI_ERR_BAD_SIZE;
}

}  // namespace llmi

using namespace llmi;

LLMI_EXPORT int llmi_latent_prepare(int dtype, const float* down, long ld, int Q, int C, int R, const float* wq,
                                    const float* wc, float eps, const float* inv_freq, int rot_dims,
                                    const int32_t* tok_seq, const int32_t* tok_pos, const int32_t* seq_pages,
                                    int pages_stride, int page_size, void* cache, void* cq, int n_tokens, int write_kv,
                                    cudaStream_t stream) {
  if (n_tokens <= 0 || Q <= 0 || C <= 0 || R < 0 || rot_dims < 0 || rot_dims > R || (rot_dims & 1)) return LLMI_ERR_BAD_SIZE;
  PagedKV kv{seq_pages, pages_stride, page_size, 1, C + R};
  if (dtype == LLMI_DTYPE_F32)
    return launch_pdl(PDL_ROPE, latent_prepare_kernel<float>, n_tokens, 128, 0, stream, down, ld, Q, C, R, wq, wc, eps, inv_freq,
                      rot_dims, tok_seq, tok_pos, kv, (float*)cache, (float*)cq, write_kv);
  if (dtype == LLMI_DTYPE_BF16)
    return launch_pdl(PDL_ROPE, latent_prepare_kernel<__nv_bfloat16>, n_tokens, 128, 0, stream, down, ld, Q, C, R, wq, wc, eps,
                      inv_freq, rot_dims, tok_seq, tok_pos, kv, (__nv_bfloat16*)cache, (__nv_bfloat16*)cq, write_kv);
  return LLMI_ERR_BAD_DTYPE;
}

LLMI_EXPORT int llmi_latent_q_rotate(int dtype, const void* q, long ldq, int D, void* qa, long ldqa, int C, int R, int H,
                                     const float* inv_freq, int rot_dims, const int32_t* tok_seq, const int32_t* tok_pos,
                                     int n_tokens, cudaStream_t stream) {
  if (n_tokens <= 0 || H <= 0 || D < 0 || C <= 0 || R < 0 || rot_dims > R || (rot_dims & 1)) return LLMI_ERR_BAD_SIZE;
  if (R == 0) return LLMI_OK;
  const size_t total = (size_t)n_tokens * H * ((R + 1) / 2);
  const size_t most = (size_t)sm_count() * 16, need = (total + 255) / 256;
  const int blocks = (int)(need < most ? need : most);
  if (dtype == LLMI_DTYPE_F32)
    return launch_pdl(PDL_SMALL, latent_q_rotate_kernel<float>, blocks, 256, 0, stream, (const float*)q, ldq, D, (float*)qa, ldqa, C,
                      R, H, inv_freq, rot_dims, tok_seq, tok_pos, n_tokens);
  if (dtype == LLMI_DTYPE_BF16)
    return launch_pdl(PDL_SMALL, latent_q_rotate_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)q, ldq, D,
                      (__nv_bfloat16*)qa, ldqa, C, R, H, inv_freq, rot_dims, tok_seq, tok_pos, n_tokens);
  return LLMI_ERR_BAD_DTYPE;
}

// qa [T, H, C + R] (row pitch ldq), out [T, H, C] (row pitch ldo), cache: the layer's pages [page][1][page_size][C + R].
LLMI_EXPORT int llmi_attention_latent(int dtype, const void* qa, long ldq, void* out, long ldo, const void* cache,
                                      const int32_t* tok_seq, const int32_t* tok_pos, const int32_t* seq_pages,
                                      int pages_stride, int page_size, int n_tokens, int n_heads, int C, int R, float scale,
                                      cudaStream_t stream) {
  if (n_tokens <= 0 || n_heads <= 0 || C <= 0 || R < 0 || page_size <= 0) return LLMI_ERR_BAD_SIZE;
  if (n_tokens > 0x7fffffff || (n_heads + LAT_WARPS - 1) / LAT_WARPS > 65535) return LLMI_ERR_BAD_SIZE;
  PagedKV kv{seq_pages, pages_stride, page_size, 1, C + R};
  if (dtype == LLMI_DTYPE_F32)
    return launch_attention_latent<float>(qa, ldq, out, ldo, cache, tok_seq, tok_pos, kv, n_tokens, n_heads, C, scale, stream);
  if (dtype == LLMI_DTYPE_BF16)
    return launch_attention_latent<__nv_bfloat16>(qa, ldq, out, ldo, cache, tok_seq, tok_pos, kv, n_tokens, n_heads, C, scale, stream);
  return LLMI_ERR_BAD_DTYPE;
}
