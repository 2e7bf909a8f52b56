// A delta rule in its general form: a recurrent mixer whose per-head state S [D, Dv] changes per token by a diagonal
// decay plus a rank-one term, both read from the OLD state, and a write:
//     S <- diag(w) S + m (pᵀ S) + k vᵀ ;        o = Sᵀ r
// w, m, p, k, r are vectors over the D key channels, v over the Dv value channels.  With p = u (the unit key),
// m = -(a * u) and w a decay per channel this is the rule whose removal acts along the key's direction only
// (llmi_gdelta_prepare makes exactly these); other rules of the family differ in how w, m, p are made.
// Column j of S evolves alone:  s_j <- w * s_j + m (p . s_j) + k v_j,  o_j = s_j . r — so the state is kept column by
// column ([head][column][entry], fp32, one row of the cache's state slab per slot) and columns are spread over threads.
//
// Everything here is fp32 arithmetic.  Kernels, in the order of a step:
//   llmi_gdelta_prepare     per (token, head): the decay from a low-rank path, the removal rate, the unit key
//   llmi_dplr_recurrence    per (sequence, head, slice of columns): the recurrence over the step's tokens
//   (llmi_delta_finish of delta_rule.cu then norms and gates o)
// The recurrence treats a column alone and only continues what the slab holds: the result does not depend on how a
// prompt was cut or on what else is in the batch.
#include <math.h>

#include "common.cuh"

namespace llmi {

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }

// dst = tanh(src) row by row (the input of the low-rank path's second product).
template <typename T>
__global__ void __launch_bounds__(256)
tanh_rows_kernel(const float* __restrict__ src, long ld, T* __restrict__ dst, int R, long total) {
  pdl_launch_dependents();
  pdl_wait();
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long t = i / R;
    dst[i] = from_f32<T>(tanhf(src[t * ld + (i - t * R)]));
  }
}

// `proj`, one fp32 row per token:  [ r (H*D) | k (H*D) | v (H*Dv) | a (H*D) | gate (H*Dv) | low (R) ].
// `prep`, one fp32 row per token:  [ w (H*D) | p (H*D) | m (H*D) ]:
//   w = exp(-exp(-1/2) * sigmoid(w0 + W2 tanh(low)))   (W2 as w2t [R, H*D] fp32: neighbouring threads read neighbours)
//   p = k / sqrt(sum_head(k^2) + 1e-6),   m = -sigmoid(a + a_bias) * p
// With `z` (fp32 [T, ldz], the product W2 tanh(low) made by a matrix product beforehand: the way of a step of many
// tokens) the kernel adds w0 to it instead of walking the R entries itself.
__global__ void __launch_bounds__(128)
gdelta_prepare_kernel(const float* __restrict__ proj, long ld, int H, int D, int Dv, int R, const float* __restrict__ w2t,
                      const float* __restrict__ z_all, long ldz, const float* __restrict__ w0,
                      const float* __restrict__ a_bias, const int32_t* __restrict__ tok_seq, float* __restrict__ prep, long ldp) {
  extern __shared__ float low_s[];                       // tanh of the low-rank path's R entries
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  if (tok_seq[t] < 0) return;
  const int HD = H * D;
  const float* row = proj + (size_t)t * ld;
  const float* low = row + 3 * (size_t)HD + 2 * (size_t)H * Dv;
  if (!z_all)
    for (int j = threadIdx.x; j < R; j += blockDim.x) low_s[j] = tanhf(low[j]);
  const float* k = row + HD + (size_t)h * D;
  float ss = 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) ss = fmaf(k[d], k[d], ss);
  ss = block_sum(ss, scratch);                           // (its barriers also publish low_s)
  const float inv = 1.0f / sqrtf(ss + 1e-6f);
  float* out = prep + (size_t)t * ldp + (size_t)h * D;
  const float* a = row + 2 * (size_t)HD + (size_t)H * Dv + (size_t)h * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const int c = h * D + d;
    float z = w0[c];
    if (z_all) {
      z += z_all[(size_t)t * ldz + c];
    } else {
      for (int j = 0; j < R; ++j) z = fmaf(w2t[(size_t)j * HD + c], low_s[j], z);
    }
    const float u = k[d] * inv;
    out[d] = expf(-0.6065306597126334f * sigmoid_f(z));
    out[HD + d] = u;
    out[2 * (size_t)HD + d] = -sigmoid_f(a[d] + a_bias[c]) * u;
  }
}

// The general form: one block per (head, sequence), one thread per column j of S, the column in shared memory
// (S_s[d][cols]: no two threads share a bank); any D and Dv.  The vectors of the next token are fetched while the
// current one is computed (two buffers, one barrier per token).
__global__ void __launch_bounds__(1024)
dplr_recurrence_kernel(const float* __restrict__ proj, long ld, const float* __restrict__ prep, long ldp, int H, int D,
                       int Dv, float* __restrict__ state, long state_stride, const int32_t* __restrict__ seq_q_start,
                       const int32_t* __restrict__ seq_slot, float* __restrict__ o_raw, long ldo, int write_state) {
  extern __shared__ float sm[];
  pdl_wait();
  pdl_launch_dependents();
  const int h = blockIdx.x, seq = blockIdx.y;
  const int slot = seq_slot[seq];
  if (slot < 0) return;
  const int r0 = seq_q_start[seq], n = seq_q_start[seq + 1] - r0;
  if (n <= 0) return;
  const int cols = blockDim.x;                               // Dv rounded up to whole warps
  const int j = threadIdx.x;
  const bool live = j < Dv;
  float* vec = sm;                                           // [2][5*D]: w, p, m, k, r of a token
  float* S_s = sm + 10 * D;                                  // [D][cols]
  const int HD = H * D;
  float* S_g = state + (size_t)slot * state_stride + (size_t)h * D * Dv;
  if (live)
    for (int d = 0; d < D; ++d) S_s[(size_t)d * cols + j] = S_g[(size_t)j * D + d];
  auto fetch = [&](int i, int buf) {
    const float* pr = prep + (size_t)(r0 + i) * ldp + (size_t)h * D;
    const float* xr = proj + (size_t)(r0 + i) * ld + (size_t)h * D;
    float* dst = vec + buf * 5 * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
      dst[d] = pr[d];
      dst[D + d] = pr[HD + d];
      dst[2 * D + d] = pr[2 * (size_t)HD + d];
      dst[3 * D + d] = xr[HD + d];
      dst[4 * D + d] = xr[d];
    }
  };
  fetch(0, 0);
  for (int i = 0; i < n; ++i) {
    __syncthreads();                                         // buffer i&1 is filled; the other one is read out
    if (i + 1 < n) fetch(i + 1, (i + 1) & 1);
    if (!live) continue;
    const float v = proj[(size_t)(r0 + i) * ld + 2 * (size_t)HD + (size_t)h * Dv + j];
    const float* w = vec + (i & 1) * 5 * D;
    const float *p = w + D, *m = w + 2 * D, *k = w + 3 * D, *r = w + 4 * D;
    float dot = 0.f;
    for (int d = 0; d < D; ++d) dot = fmaf(S_s[(size_t)d * cols + j], p[d], dot);
    float o = 0.f;
    for (int d = 0; d < D; ++d) {
      const float s = fmaf(k[d], v, fmaf(m[d], dot, w[d] * S_s[(size_t)d * cols + j]));
      S_s[(size_t)d * cols + j] = s;
      o = fmaf(s, r[d], o);
    }
    o_raw[(size_t)(r0 + i) * ldo + (size_t)h * Dv + j] = o;
  }
  if (live && write_state)
    for (int d = 0; d < D; ++d) S_g[(size_t)j * D + d] = S_s[(size_t)d * cols + j];
}

// The form for D = 32, 64, 128 and Dv a multiple of 16.  A thread holds TWO neighbouring columns of S and a sixteenth
// of their entries (lane `sub` of sixteen: d = 64 i + 4 sub + 0..3, while d < D) in registers; partial sums over d are
// joined by four shuffles.  The recurrence is a chain over the tokens, so the work of a token is spread thin (16
// columns a warp), a head's columns are cut into slices of 32 (or 16), every slice a block of its own (blockIdx.z),
// and what a token needs — w, p, m, k, r of the head, the slice's v — is copied into a ring of DPLR_RING entries
// DPLR_RING - 1 tokens ahead (cp.async, 16 bytes a copy), so that no load's latency lies on the chain from token to
// token; one barrier per token.  (Two tokens per round — the second one's sum over the state follows from the state
// before the first, (p_B * w_A) . S + (p_B . m_A)(p_A . S) + (p_B . k_A) v_A, so one round of shuffles serves both — was
// measured slower, 1.10 against 0.96 ms for 2,048 tokens: the time of a token is its instructions, not the shuffles.)
constexpr int DPLR_RING = 8;

__device__ __forceinline__ void dplr_cp16(void* dst, const void* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}

template <int D>
__global__ void __launch_bounds__(256)
dplr_recurrence_quad_kernel(const float* __restrict__ proj, long ld, const float* __restrict__ prep, long ldp, int H, int Dv,
                            float* __restrict__ state, long state_stride, const int32_t* __restrict__ seq_q_start,
                            const int32_t* __restrict__ seq_slot, float* __restrict__ o_raw, long ldo, int write_state) {
  extern __shared__ __align__(16) float sm[];
  pdl_wait();
  pdl_launch_dependents();
  const int h = blockIdx.x, seq = blockIdx.y;
  const int slot = seq_slot[seq];
  if (slot < 0) return;
  const int r0 = seq_q_start[seq], n = seq_q_start[seq + 1] - r0;
  if (n <= 0) return;
  constexpr int NI = (D + 63) / 64;                          // chunks of four entries per lane (D = 32: lanes 8..15 hold none)
  const int CB = blockDim.x >> 3;                            // columns of this block's slice (the launcher gives 8 CB threads)
  const int cg = threadIdx.x >> 4, sub = threadIdx.x & 15;   // my columns: col0, col0 + 1
  const int col0 = blockIdx.z * CB + 2 * cg;
  const bool holds = 4 * sub < D;
  const int HD = H * D;
  float* S_g = state + (size_t)slot * state_stride + (size_t)h * D * Dv + (size_t)col0 * D;     // [column][entry]
  float2 S_r[NI][4];                                         // [chunk][entry of the chunk] . (x, y) = the two columns
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const float4 c0 = holds ? *reinterpret_cast<const float4*>(S_g + 64 * i + 4 * sub) : make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 c1 = holds ? *reinterpret_cast<const float4*>(S_g + D + 64 * i + 4 * sub) : make_float4(0.f, 0.f, 0.f, 0.f);
    S_r[i][0] = make_float2(c0.x, c1.x);
    S_r[i][1] = make_float2(c0.y, c1.y);
    S_r[i][2] = make_float2(c0.z, c1.z);
    S_r[i][3] = make_float2(c0.w, c1.w);
  }
  // ring entry: [w | p | m | k | r (D each) | v of the slice (CB)]; all parts are whole 16-byte pieces
  constexpr int Q = D / 4;                                   // 16-byte pieces of one vector
  const int n16 = 5 * Q + CB / 4, pitch = 5 * D + CB;
  const float* w_src = prep + (size_t)h * D;
  const float* x_src = proj + (size_t)h * D;
  const float* v_src = proj + 2 * (size_t)HD + (size_t)h * Dv + blockIdx.z * CB;
  auto issue = [&](int i) {
    float* dst = sm + (size_t)(i % DPLR_RING) * pitch;
    const size_t prow = (size_t)(r0 + i) * ldp, xrow = (size_t)(r0 + i) * ld;
    for (int e = threadIdx.x; e < n16; e += blockDim.x) {
      const int part = e / Q, off = 4 * (e - part * Q);
      if (part < 3) dplr_cp16(dst + 4 * e, w_src + prow + (size_t)part * HD + off);            // w, p, m
      else if (part == 3) dplr_cp16(dst + 4 * e, x_src + xrow + HD + off);                        // k
      else if (part == 4) dplr_cp16(dst + 4 * e, x_src + xrow + off);                             // r
      else dplr_cp16(dst + 4 * e, v_src + xrow + 4 * (e - 5 * Q));
    }
  };
#pragma unroll
  for (int s = 0; s < DPLR_RING - 1; ++s) {
    if (s < n) issue(s);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  float2 o_pend = make_float2(0.f, 0.f);                       // my part of the token before's S . r
  for (int i = 0; i < n; ++i) {
    asm volatile("cp.async.wait_group %0;" ::"n"(DPLR_RING - 2) : "memory");
    __syncthreads();                                         // token i's entry is there; token i-1's entry is read out
    if (i + DPLR_RING - 1 < n) issue(i + DPLR_RING - 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const float* in = sm + (size_t)(i % DPLR_RING) * pitch;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 pp[NI];
    float2 dot = make_float2(0.f, 0.f), dot2 = make_float2(0.f, 0.f);
#pragma unroll
    for (int c = 0; c < NI; ++c) {
      pp[c] = holds ? *reinterpret_cast<const float4*>(in + D + 64 * c + 4 * sub) : zero;
      dot.x = fmaf(S_r[c][0].x, pp[c].x, dot.x);
      dot.y = fmaf(S_r[c][0].y, pp[c].x, dot.y);
      dot2.x = fmaf(S_r[c][1].x, pp[c].y, dot2.x);
      dot2.y = fmaf(S_r[c][1].y, pp[c].y, dot2.y);
      dot.x = fmaf(S_r[c][2].x, pp[c].z, dot.x);
      dot.y = fmaf(S_r[c][2].y, pp[c].z, dot.y);
      dot2.x = fmaf(S_r[c][3].x, pp[c].w, dot2.x);
      dot2.y = fmaf(S_r[c][3].y, pp[c].w, dot2.y);
    }
    dot.x += dot2.x;
    dot.y += dot2.y;
    // the sums of this token's p . S and of the token BEFORE's S . r ride the same four rounds of shuffles: the latter
    // are not on the chain from token to token, and a round of their own per token would be
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) {
      dot.x += __shfl_xor_sync(0xffffffffu, dot.x, o);
      dot.y += __shfl_xor_sync(0xffffffffu, dot.y, o);
      o_pend.x += __shfl_xor_sync(0xffffffffu, o_pend.x, o);
      o_pend.y += __shfl_xor_sync(0xffffffffu, o_pend.y, o);
    }
    if (i > 0 && sub == 0) *reinterpret_cast<float2*>(o_raw + (size_t)(r0 + i - 1) * ldo + (size_t)h * Dv + col0) = o_pend;
    const float2 v = *reinterpret_cast<const float2*>(in + 5 * D + 2 * cg);
    float2 o2 = make_float2(0.f, 0.f), o3 = make_float2(0.f, 0.f);
#pragma unroll
    for (int c = 0; c < NI; ++c) {
      const float4 ww = holds ? *reinterpret_cast<const float4*>(in + 64 * c + 4 * sub) : zero;
      const float4 mm = holds ? *reinterpret_cast<const float4*>(in + 2 * D + 64 * c + 4 * sub) : zero;
      const float4 kk = holds ? *reinterpret_cast<const float4*>(in + 3 * D + 64 * c + 4 * sub) : zero;
      const float4 rr = holds ? *reinterpret_cast<const float4*>(in + 4 * D + 64 * c + 4 * sub) : zero;
      const float we[4] = {ww.x, ww.y, ww.z, ww.w}, me[4] = {mm.x, mm.y, mm.z, mm.w};
      const float ke[4] = {kk.x, kk.y, kk.z, kk.w}, re[4] = {rr.x, rr.y, rr.z, rr.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 s = S_r[c][e];
        s.x = fmaf(ke[e], v.x, fmaf(me[e], dot.x, we[e] * s.x));
        s.y = fmaf(ke[e], v.y, fmaf(me[e], dot.y, we[e] * s.y));
        S_r[c][e] = s;
        if (e & 1) {
          o3.x = fmaf(s.x, re[e], o3.x);
          o3.y = fmaf(s.y, re[e], o3.y);
        } else {
          o2.x = fmaf(s.x, re[e], o2.x);
          o2.y = fmaf(s.y, re[e], o2.y);
        }
      }
    }
    o_pend = make_float2(o2.x + o3.x, o2.y + o3.y);           // joined over the lanes in the next token's rounds
  }
#pragma unroll
  for (int o = 1; o < 16; o <<= 1) {                           // the last token's
    o_pend.x += __shfl_xor_sync(0xffffffffu, o_pend.x, o);
    o_pend.y += __shfl_xor_sync(0xffffffffu, o_pend.y, o);
  }
  if (sub == 0) *reinterpret_cast<float2*>(o_raw + (size_t)(r0 + n - 1) * ldo + (size_t)h * Dv + col0) = o_pend;
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  if (write_state && holds) {
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      *reinterpret_cast<float4*>(S_g + 64 * i + 4 * sub) = make_float4(S_r[i][0].x, S_r[i][1].x, S_r[i][2].x, S_r[i][3].x);
      *reinterpret_cast<float4*>(S_g + D + 64 * i + 4 * sub) = make_float4(S_r[i][0].y, S_r[i][1].y, S_r[i][2].y, S_r[i][3].y);
    }
  }
}

template <int D>
int launch_dplr_quad(const float* proj, long ld, const float* prep, long ldp, int H, int Dv, float* state, long state_stride,
                     const int32_t* seq_q_start, const int32_t* seq_slot, float* o_raw, long ldo, int n_seqs, int write_state,
                     cudaStream_t stream) {
  const int CB = Dv % 32 == 0 ? 32 : 16;                     // columns per block
  const size_t smem = (size_t)DPLR_RING * (5 * D + CB) * sizeof(float);
  return launch_pdl(PDL_ATTENTION, dplr_recurrence_quad_kernel<D>, dim3(H, n_seqs, Dv / CB), dim3(8 * CB), smem, stream, proj, ld,
                    prep, ldp, H, Dv, state, state_stride, seq_q_start, seq_slot, o_raw, ldo, write_state);
}

}  // namespace llmi

using namespace llmi;

// w2t: W2 transposed, fp32 [R, H*D]; z (optional): fp32 [T, ldz] = tanh(low) W2ᵀ made beforehand.
LLMI_EXPORT int llmi_gdelta_prepare(const float* proj, long ld, int H, int D, int Dv, int R, const float* w2t, const float* z,
                                    long ldz, const float* w0, const float* a_bias, const int32_t* tok_seq, float* prep, long ldp,
                                    int n_tokens, cudaStream_t stream) {
  if (n_tokens <= 0 || H <= 0 || H > 65535 || D <= 0 || Dv <= 0 || R <= 0 || R > 8192) return LLMI_ERR_BAD_SIZE;
  const int threads = D > 64 ? 128 : (D > 32 ? 64 : 32);
  return launch_pdl(PDL_SMALL, gdelta_prepare_kernel, dim3(n_tokens, H), dim3(threads), (size_t)R * sizeof(float), stream, proj, ld,
                    H, D, Dv, R, w2t, z, ldz, w0, a_bias, tok_seq, prep, ldp);
}

// dst [T, R] (type `dtype`, contiguous) = tanh(src[:, :R]); src fp32 rows of pitch ld.
LLMI_EXPORT int llmi_tanh_rows(int dtype, const float* src, long ld, void* dst, int n_rows, int R, cudaStream_t stream) {
  if (n_rows <= 0 || R <= 0) return LLMI_ERR_BAD_SIZE;
  const long total = (long)n_rows * R;
  const long want = (total + 255) / 256, most = (long)sm_count() * 16;
  const unsigned blocks = (unsigned)(want < most ? want : most);
  if (dtype == LLMI_DTYPE_F32)
    return launch_pdl(PDL_SMALL, tanh_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, src, ld, (float*)dst, R, total);
  if (dtype == LLMI_DTYPE_BF16)
    return launch_pdl(PDL_SMALL, tanh_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, src, ld, (__nv_bfloat16*)dst, R, total);
  return LLMI_ERR_BAD_DTYPE;
}

// proj fp32 [T, ld]: r at column 0, k at H*D, v at 2*H*D; prep fp32 [T, ldp]: w at 0, p at H*D, m at 2*H*D;
// state fp32 [slots, state_stride >= H*D*Dv]; o_raw fp32 [T, ldo] receives Sᵀ r.
LLMI_EXPORT int llmi_dplr_recurrence(const float* proj, long ld, const float* prep, long ldp, int H, int D, int Dv, float* state,
                                     long state_stride, const int32_t* seq_q_start, const int32_t* seq_slot, float* o_raw,
                                     long ldo, int n_seqs, int write_state, cudaStream_t stream) {
  if (n_seqs <= 0 || n_seqs > 65535 || H <= 0 || D <= 0 || Dv <= 0 || Dv > 1024) return LLMI_ERR_BAD_SIZE;
  if (Dv % 16 == 0 && ld % 4 == 0 && ldp % 4 == 0 && ldo % 4 == 0 && state_stride % 4 == 0 && !((uintptr_t)state & 15) &&
      !((uintptr_t)o_raw & 15) && !((uintptr_t)prep & 15) && !((uintptr_t)proj & 15)) {
#define LLMI_QUAD(DD)                                                                                                      \
  if (D == DD)                                                                                                             \
    return launch_dplr_quad<DD>(proj, ld, prep, ldp, H, Dv, state, state_stride, seq_q_start, seq_slot, o_raw, ldo, n_seqs, \
                                write_state, stream)
    LLMI_QUAD(32);
    LLMI_QUAD(64);
    LLMI_QUAD(128);
#undef LLMI_QUAD
  }
  const int cols = (Dv + 31) / 32 * 32;
  const size_t smem = ((size_t)10 * D + (size_t)D * cols) * sizeof(float);
  if (smem > 200 * 1024) return LLMI_ERR_BAD_SIZE;
  static PerDevice<size_t> allowed;
  if (smem > 48 * 1024 && allowed.here() < smem) {
    if (cudaFuncSetAttribute(dplr_recurrence_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return LLMI_ERR_BAD_SIZE;
    allowed.here() = smem;
  }
  return launch_pdl(PDL_ATTENTION, dplr_recurrence_kernel, dim3(H, n_seqs), dim3(cols), smem, stream, proj, ld, prep, ldp, H, D, Dv,
                    state, state_stride, seq_q_start, seq_slot, o_raw, ldo, write_state);
}
