// The gated delta rule: a recurrent mixer whose per-head state S [D, Dv] is a fast-weight matrix,
//     S <- g S;   u = beta (v - Sᵀ k);   S <- S + k uᵀ;   o = Sᵀ q        (in this order, per token)
// with q, k unit vectors (q also times D^-1/2), a decay g in (0, 1) and a write strength beta in (0, 1).
// q, k, v first pass a short causal convolution over time (per channel, no bias) and silu.  The state of a
// sequence is S (fp32) and the last taps-1 inputs of the convolution (fp32); both live in the cache's state slab,
// one row per slot:  [ S: H*D*Dv | conv: (taps-1) * Nc ],  Nc = 2*Hk*D + H*Dv channels.
//
// Everything here is fp32 arithmetic.  Kernels, in the order of a step:
//   llmi_delta_prepare      per token: convolution + silu, unit norms, beta, decay          (parallel over tokens)
//   llmi_delta_conv_carry   per sequence: the convolution's inputs that the next step needs (after prepare)
//   llmi_delta_recurrence   per (sequence, head): the recurrence over the step's tokens, one thread per column of S
//   llmi_delta_finish       per (token, head): o / rms(o) * w * silu(gate) in the compute type (parallel over tokens)
// The input `proj` is one fp32 row per token: [ q (Hk*D) | k (Hk*D) | v (H*Dv) | b (H) | a (H) | gate (H*Dv) ].
// The recurrence treats a column of S alone, and a step only continues what the slab holds: the result does not
// depend on how a prompt was cut or on what else is in the batch.
#include <math.h>

#include "common.cuh"

namespace llmi {

constexpr int DELTA_MAX_TAPS = 16;

struct DeltaDims {
  int H, Hk, D, Dv, taps;
  __host__ __device__ int n_qk() const { return 2 * Hk * D; }
  __host__ __device__ int n_conv() const { return 2 * Hk * D + H * Dv; }
  __host__ __device__ long state_floats() const { return (long)H * D * Dv + (long)(taps - 1) * n_conv(); }
  __host__ __device__ long conv_offset() const { return (long)H * D * Dv; }
};

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// One block per token.  prep: fp32 [T, Nc + 2H]: [ q^ | k^ | v (after convolution and silu) | beta | decay ].
__global__ void __launch_bounds__(128)
delta_prepare_kernel(const float* __restrict__ proj, long ld, DeltaDims m, const float* __restrict__ conv_w,
                     const float* __restrict__ a_log, const float* __restrict__ dt_bias, const float* __restrict__ state,
                     const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ tok_pos,
                     const int32_t* __restrict__ seq_q_start, const int32_t* __restrict__ seq_slot,
                     float* __restrict__ prep, long ldp) {
  extern __shared__ float qk_s[];                        // [2*Hk*D] convolved q and k of this token
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int seq = tok_seq[t];
  if (seq < 0) return;
  const int slot = seq_slot[seq];
  if (slot < 0) return;
  const int pos = tok_pos[t], r0 = seq_q_start[seq];
  const int p0 = pos - (t - r0);                         // position of the step's first token of this sequence
  const int K = m.taps, Nc = m.n_conv(), Nqk = m.n_qk();
  const float* carry = state + (size_t)slot * m.state_floats() + m.conv_offset();   // [K-1][Nc]: positions p0-(K-1) .. p0-1
  float* out = prep + (size_t)t * ldp;
  for (int ch = threadIdx.x; ch < Nc; ch += blockDim.x) {
    float acc = 0.f;
    for (int d = K - 1; d >= 0; --d) {                   // oldest tap first
      const int p = pos - d;
      if (p < 0) continue;
      const float x = p >= p0 ? proj[(size_t)(r0 + (p - p0)) * ld + ch] : carry[(size_t)(p - (p0 - (K - 1))) * Nc + ch];
      acc = fmaf(x, conv_w[(size_t)ch * K + (K - 1 - d)], acc);
    }
    const float y = silu_f(acc);
    if (ch < Nqk) qk_s[ch] = y; else out[ch] = y;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  for (int hh = warp; hh < 2 * m.Hk; hh += nwarp) {      // heads of q, then heads of k
    const float* src = qk_s + (size_t)hh * m.D;
    float ss = 0.f;
    for (int d = lane; d < m.D; d += 32) ss = fmaf(src[d], src[d], ss);
    ss = warp_sum(ss);
    float sc = 1.0f / sqrtf(ss + 1e-6f);
    if (hh < m.Hk) sc *= 1.0f / sqrtf((float)m.D);
    for (int d = lane; d < m.D; d += 32) out[(size_t)hh * m.D + d] = src[d] * sc;
  }
  const float* row = proj + (size_t)t * ld;
  for (int h = threadIdx.x; h < m.H; h += blockDim.x) {
    const float b = row[Nc + h], a = row[Nc + m.H + h];
    out[Nc + h] = 1.0f / (1.0f + expf(-b));
    out[Nc + m.H + h] = expf(-expf(a_log[h]) * softplus_f(a + dt_bias[h]));
  }
}

// One thread per (sequence, channel): the inputs of the last taps-1 positions after this step, from the step's own
// rows or, where the step brought fewer, from what the slab held.
__global__ void __launch_bounds__(128)
delta_conv_carry_kernel(const float* __restrict__ proj, long ld, DeltaDims m, float* __restrict__ state,
                        const int32_t* __restrict__ seq_q_start, const int32_t* __restrict__ seq_kv_len,
                        const int32_t* __restrict__ seq_slot, int n_seqs) {
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.y;
  const int slot = seq_slot[seq];
  if (slot < 0) return;
  const int ch = blockIdx.x * blockDim.x + threadIdx.x;
  const int Nc = m.n_conv(), K = m.taps;
  if (ch >= Nc || K <= 1) return;
  const int r0 = seq_q_start[seq], n = seq_q_start[seq + 1] - r0, L = seq_kv_len[seq];
  if (n <= 0) return;
  const int p0 = L - n;
  float* carry = state + (size_t)slot * m.state_floats() + m.conv_offset();
  float keep[DELTA_MAX_TAPS];
  for (int j = 0; j < K - 1; ++j) {
    const int p = L - (K - 1) + j;
    keep[j] = p < 0 ? 0.f : (p >= p0 ? proj[(size_t)(r0 + (p - p0)) * ld + ch] : carry[(size_t)(p - (p0 - (K - 1))) * Nc + ch]);
  }
  for (int j = 0; j < K - 1; ++j) carry[(size_t)j * Nc + ch] = keep[j];
}

// One block per (head, sequence), one thread per column j of S.  DREG > 0: the column (D = DREG entries) lives in
// registers; DREG == 0: any D, the column lives in shared memory (S_s[d][j]: no two threads share a bank).
// k and q of the next token are fetched while the current one is computed (two buffers, one barrier per token).
template <int DREG>
__global__ void __launch_bounds__(256)
delta_recurrence_kernel(const float* __restrict__ prep, long ldp, DeltaDims m, float* __restrict__ state,
                        const int32_t* __restrict__ seq_q_start, const int32_t* __restrict__ seq_slot,
                        float* __restrict__ o_raw, long ldo, int write_state) {
  extern __shared__ float sm[];
  pdl_wait();
  pdl_launch_dependents();
  const int h = blockIdx.x, seq = blockIdx.y;
  const int slot = seq_slot[seq];
  if (slot < 0) return;
  const int r0 = seq_q_start[seq], n = seq_q_start[seq + 1] - r0;
  if (n <= 0) return;
  const int D = DREG > 0 ? DREG : m.D, Dv = m.Dv;
  const int cols = blockDim.x;                               // Dv rounded up to whole warps
  const int j = threadIdx.x;
  const bool live = j < Dv;
  float* kq = sm;                                            // [2][2*D]: k then q of a token
  float* S_s = sm + 4 * D;                                   // [D][cols] (DREG == 0 only)
  const int kh = h / (m.H / m.Hk);
  float* S_g = state + (size_t)slot * m.state_floats() + (size_t)h * D * Dv;
  float S_r[DREG > 0 ? DREG : 1];
  if (live) {
    if (DREG > 0) {
#pragma unroll
      for (int d = 0; d < DREG; ++d) S_r[d] = S_g[(size_t)d * Dv + j];
    } else {
      for (int d = 0; d < D; ++d) S_s[(size_t)d * cols + j] = S_g[(size_t)d * Dv + j];
    }
  }
  const int Nc = m.n_conv();
  auto fetch = [&](int i, int buf) {
    const float* row = prep + (size_t)(r0 + i) * ldp;
    for (int d = threadIdx.x; d < 2 * D; d += blockDim.x)
      kq[buf * 2 * D + d] = d < D ? row[(size_t)m.Hk * D + (size_t)kh * D + d] : row[(size_t)kh * D + (d - D)];
  };
  fetch(0, 0);
  for (int i = 0; i < n; ++i) {
    __syncthreads();                                         // buffer i&1 is filled; the other one is read out
    if (i + 1 < n) fetch(i + 1, (i + 1) & 1);
    if (!live) continue;
    const float* row = prep + (size_t)(r0 + i) * ldp;
    const float v = row[(size_t)m.n_qk() + (size_t)h * Dv + j];
    const float beta = row[Nc + h], g = row[Nc + m.H + h];
    const float* k = kq + (i & 1) * 2 * D;
    const float* q = k + D;
    float sk = 0.f;
    if (DREG > 0) {
#pragma unroll
      for (int d = 0; d < DREG; ++d) sk = fmaf(S_r[d], k[d], sk);
    } else {
      for (int d = 0; d < D; ++d) sk = fmaf(S_s[(size_t)d * cols + j], k[d], sk);
    }
    const float u = beta * (v - g * sk);                     // (g S)ᵀ k = g (Sᵀ k)
    float o = 0.f;
    if (DREG > 0) {
#pragma unroll
      for (int d = 0; d < DREG; ++d) {
        const float s = fmaf(k[d], u, g * S_r[d]);
        S_r[d] = s;
        o = fmaf(s, q[d], o);
      }
    } else {
      for (int d = 0; d < D; ++d) {
        const float s = fmaf(k[d], u, g * S_s[(size_t)d * cols + j]);
        S_s[(size_t)d * cols + j] = s;
        o = fmaf(s, q[d], o);
      }
    }
    o_raw[(size_t)(r0 + i) * ldo + (size_t)h * Dv + j] = o;
  }
  if (live && write_state) {
    if (DREG > 0) {
#pragma unroll
      for (int d = 0; d < DREG; ++d) S_g[(size_t)d * Dv + j] = S_r[d];
    } else {
      for (int d = 0; d < D; ++d) S_g[(size_t)d * Dv + j] = S_s[(size_t)d * cols + j];
    }
  }
}

// The same with FOUR lanes per column of S (D = 4 * DQ, the column's entries d = sub, sub + 4, ... in registers of lane
// `sub`): a quarter of the serial work per token and of the registers, partial sums joined by two shuffles.  The
// recurrence is a chain over the tokens, so the time of a prompt is tokens x (time of one token): this form is what
// keeps that time short.
template <int DQ>
__global__ void __launch_bounds__(512)
delta_recurrence_quad_kernel(const float* __restrict__ prep, long ldp, DeltaDims m, float* __restrict__ state,
                             const int32_t* __restrict__ seq_q_start, const int32_t* __restrict__ seq_slot,
                             float* __restrict__ o_raw, long ldo, int write_state) {
  extern __shared__ float sm[];
  pdl_wait();
  pdl_launch_dependents();
  const int h = blockIdx.x, seq = blockIdx.y;
  const int slot = seq_slot[seq];
  if (slot < 0) return;
  const int r0 = seq_q_start[seq], n = seq_q_start[seq + 1] - r0;
  if (n <= 0) return;
  constexpr int D = 4 * DQ;
  const int Dv = m.Dv;
  const int col = threadIdx.x >> 2, sub = threadIdx.x & 3;
  const bool live = col < Dv;
  const int j = live ? col : Dv - 1;
  float* kq = sm;                                            // [2][2*D]: k then q of a token
  const int kh = h / (m.H / m.Hk);
  float* S_g = state + (size_t)slot * m.state_floats() + (size_t)h * D * Dv;
  float S_r[DQ];
#pragma unroll
  for (int i = 0; i < DQ; ++i) S_r[i] = S_g[(size_t)(sub + 4 * i) * Dv + j];
  const int Nc = m.n_conv();
  // What the NEXT token needs is asked for before the current token is computed and put down after it, so that
  // no load's latency lies on the chain from token to token: the entry of [k | q] this thread copies (the first 2*D
  // threads; 4 * Dv >= 2 * D is checked by the launcher), and v, beta, g.
  const bool copies = (int)threadIdx.x < 2 * D;
  const size_t kq_off = (int)threadIdx.x < D ? (size_t)m.Hk * D + (size_t)kh * D + threadIdx.x : (size_t)kh * D + (threadIdx.x - D);
  const size_t v_off = (size_t)m.n_qk() + (size_t)h * Dv + j;
  const float* row = prep + (size_t)r0 * ldp;
  if (copies) kq[threadIdx.x] = row[kq_off];
  float v = row[v_off], beta = row[Nc + h], g = row[Nc + m.H + h];
  for (int i = 0; i < n; ++i) {
    __syncthreads();                                         // buffer i&1 is filled; the other one is read out
    float n_kq = 0.f, n_v = 0.f, n_beta = 0.f, n_g = 0.f;
    if (i + 1 < n) {
      const float* nxt = prep + (size_t)(r0 + i + 1) * ldp;
      if (copies) n_kq = nxt[kq_off];
      n_v = nxt[v_off];
      n_beta = nxt[Nc + h];
      n_g = nxt[Nc + m.H + h];
    }
    const float* k = kq + (i & 1) * 2 * D + sub;
    const float* q = k + D;
    float p0 = 0.f, p1 = 0.f;
#pragma unroll
    for (int e = 0; e < DQ; e += 2) {
      p0 = fmaf(S_r[e], k[4 * e], p0);
      p1 = fmaf(S_r[e + 1], k[4 * e + 4], p1);
    }
    float sk = p0 + p1;
    sk += __shfl_xor_sync(0xffffffffu, sk, 1);
    sk += __shfl_xor_sync(0xffffffffu, sk, 2);
    const float u = beta * (v - g * sk);
    float o0 = 0.f, o1 = 0.f;
#pragma unroll
    for (int e = 0; e < DQ; e += 2) {
      const float s0 = fmaf(k[4 * e], u, g * S_r[e]), s1 = fmaf(k[4 * e + 4], u, g * S_r[e + 1]);
      S_r[e] = s0;
      S_r[e + 1] = s1;
      o0 = fmaf(s0, q[4 * e], o0);
      o1 = fmaf(s1, q[4 * e + 4], o1);
    }
    float o = o0 + o1;
    o += __shfl_xor_sync(0xffffffffu, o, 1);
    o += __shfl_xor_sync(0xffffffffu, o, 2);
    if (live && sub == 0) o_raw[(size_t)(r0 + i) * ldo + (size_t)h * Dv + j] = o;
    if (copies && i + 1 < n) kq[((i + 1) & 1) * 2 * D + threadIdx.x] = n_kq;
    v = n_v; beta = n_beta; g = n_g;
  }
  if (live && write_state) {
#pragma unroll
    for (int i = 0; i < DQ; ++i) S_g[(size_t)(sub + 4 * i) * Dv + j] = S_r[i];
  }
}

template <int DQ>
int launch_delta_recurrence_quad(const float* prep, long ldp, DeltaDims m, float* state, const int32_t* seq_q_start,
                                 const int32_t* seq_slot, float* o_raw, long ldo, int n_seqs, int write_state,
                                 cudaStream_t stream) {
  const int threads = (4 * m.Dv + 31) / 32 * 32;
  return launch_pdl(PDL_ATTENTION, delta_recurrence_quad_kernel<DQ>, dim3(m.H, n_seqs), dim3(threads), (size_t)16 * DQ * sizeof(float),
                    stream, prep, ldp, m, state, seq_q_start, seq_slot, o_raw, ldo, write_state);
}

// One warp per (token, head): out = o / sqrt(mean(o^2) + eps) * w * silu(gate).
template <typename T>
__global__ void __launch_bounds__(128)
delta_finish_kernel(const float* __restrict__ o_raw, long ldo, const float* __restrict__ gate, long ldg,
                    const float* __restrict__ w, float eps, int H, int Dv, const int32_t* __restrict__ tok_seq,
                    T* __restrict__ out, long ld_out, long n_items) {
  pdl_launch_dependents();
  pdl_wait();
  const long item = (long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= n_items) return;
  const int lane = threadIdx.x & 31;
  const int t = (int)(item / H), h = (int)(item - (long)t * H);
  T* dst = out + (size_t)t * ld_out + (size_t)h * Dv;
  if (tok_seq[t] < 0) {
    for (int d = lane; d < Dv; d += 32) dst[d] = from_f32<T>(0.f);
    return;
  }
  const float* o = o_raw + (size_t)t * ldo + (size_t)h * Dv;
  const float* g = gate + (size_t)t * ldg + (size_t)h * Dv;
  float ss = 0.f;
  for (int d = lane; d < Dv; d += 32) ss = fmaf(o[d], o[d], ss);
  ss = warp_sum(ss);
  const float sc = 1.0f / sqrtf(ss / (float)Dv + eps);
  for (int d = lane; d < Dv; d += 32) dst[d] = from_f32<T>(w[d] * (o[d] * sc) * silu_f(g[d]));
}

template <int DREG>
int launch_delta_recurrence(const float* prep, long ldp, DeltaDims m, float* state, const int32_t* seq_q_start,
                            const int32_t* seq_slot, float* o_raw, long ldo, int n_seqs, int write_state,
                            cudaStream_t stream) {
  const int cols = (m.Dv + 31) / 32 * 32;
  const size_t smem = ((size_t)4 * m.D + (DREG > 0 ? 0 : (size_t)m.D * cols)) * sizeof(float);
  static PerDevice<size_t> allowed;
  if (smem > 48 * 1024 && allowed.here() < smem) {
    if (cudaFuncSetAttribute(delta_recurrence_kernel<DREG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return LLMI_ERR_BAD_SIZE;
    allowed.here() = smem;
  }
  return launch_pdl(PDL_ATTENTION, delta_recurrence_kernel<DREG>, dim3(m.H, n_seqs), dim3(cols), smem, stream, prep, ldp, m, state,
                    seq_q_start, seq_slot, o_raw, ldo, write_state);
}

}  // namespace llmi

using namespace llmi;

static int delta_dims_ok(const DeltaDims& m) {
  return m.H > 0 && m.Hk > 0 && m.D > 0 && m.Dv > 0 && m.taps >= 1 && m.taps <= DELTA_MAX_TAPS && m.H % m.Hk == 0 && m.Dv <= 256;
}

LLMI_EXPORT long llmi_delta_state_floats(int H, int Hk, int D, int Dv, int taps) {
  return DeltaDims{H, Hk, D, Dv, taps}.state_floats();
}

LLMI_EXPORT int llmi_delta_prepare(const float* proj, long ld, int H, int Hk, int D, int Dv, int taps, const float* conv_w,
                                   const float* a_log, const float* dt_bias, const float* state, const int32_t* tok_seq,
                                   const int32_t* tok_pos, const int32_t* seq_q_start, const int32_t* seq_slot, float* prep,
                                   long ldp, int n_tokens, cudaStream_t stream) {
  const DeltaDims m{H, Hk, D, Dv, taps};
  if (n_tokens <= 0 || !delta_dims_ok(m)) return LLMI_ERR_BAD_SIZE;
  const size_t smem = (size_t)m.n_qk() * sizeof(float);
  if (smem > 48 * 1024) return LLMI_ERR_BAD_SIZE;
  return launch_pdl(PDL_SMALL, delta_prepare_kernel, n_tokens, 128, smem, stream, proj, ld, m, conv_w, a_log, dt_bias, state,
                    tok_seq, tok_pos, seq_q_start, seq_slot, prep, ldp);
}

LLMI_EXPORT int llmi_delta_conv_carry(const float* proj, long ld, int H, int Hk, int D, int Dv, int taps, float* state,
                                      const int32_t* seq_q_start, const int32_t* seq_kv_len, const int32_t* seq_slot,
                                      int n_seqs, cudaStream_t stream) {
  const DeltaDims m{H, Hk, D, Dv, taps};
  if (n_seqs <= 0 || n_seqs > 65535 || !delta_dims_ok(m)) return LLMI_ERR_BAD_SIZE;
  if (taps <= 1) return LLMI_OK;
  return launch_pdl(PDL_SMALL, delta_conv_carry_kernel, dim3((m.n_conv() + 127) / 128, n_seqs), dim3(128), 0, stream, proj, ld, m,
                    state, seq_q_start, seq_kv_len, seq_slot, n_seqs);
}

LLMI_EXPORT int llmi_delta_recurrence(const float* prep, long ldp, int H, int Hk, int D, int Dv, int taps, float* state,
                                      const int32_t* seq_q_start, const int32_t* seq_slot, float* o_raw, long ldo, int n_seqs,
                                      int write_state, cudaStream_t stream) {
  const DeltaDims m{H, Hk, D, Dv, taps};
  if (n_seqs <= 0 || n_seqs > 65535 || !delta_dims_ok(m)) return LLMI_ERR_BAD_SIZE;
  if (Dv <= 128 && 4 * ((Dv + 7) / 8 * 8) >= 2 * D) {          // (the block's threads also copy [k | q]: 2 * D entries)
    if (D == 32) return launch_delta_recurrence_quad<8>(prep, ldp, m, state, seq_q_start, seq_slot, o_raw, ldo, n_seqs, write_state, stream);
    if (D == 64) return launch_delta_recurrence_quad<16>(prep, ldp, m, state, seq_q_start, seq_slot, o_raw, ldo, n_seqs, write_state, stream);
    if (D == 128) return launch_delta_recurrence_quad<32>(prep, ldp, m, state, seq_q_start, seq_slot, o_raw, ldo, n_seqs, write_state, stream);
  }
  if ((size_t)D * ((Dv + 31) / 32 * 32) * 4 + 16 * (size_t)D > 200 * 1024) return LLMI_ERR_BAD_SIZE;
  return launch_delta_recurrence<0>(prep, ldp, m, state, seq_q_start, seq_slot, o_raw, ldo, n_seqs, write_state, stream);
}

LLMI_EXPORT int llmi_delta_finish(int dtype, const float* o_raw, long ldo, const float* gate, long ldg, const float* w,
                                  float eps, int H, int Dv, const int32_t* tok_seq, void* out, long ld_out, int n_tokens,
                                  cudaStream_t stream) {
  if (n_tokens <= 0 || H <= 0 || Dv <= 0) return LLMI_ERR_BAD_SIZE;
  const long items = (long)n_tokens * H;
  const unsigned blocks = (unsigned)((items + 3) / 4);
  if (dtype == LLMI_DTYPE_F32)
    return launch_pdl(PDL_SMALL, delta_finish_kernel<float>, blocks, 128, 0, stream, o_raw, ldo, gate, ldg, w, eps, H, Dv, tok_seq,
                      (float*)out, ld_out, items);
  if (dtype == LLMI_DTYPE_BF16)
    return launch_pdl(PDL_SMALL, delta_finish_kernel<__nv_bfloat16>, blocks, 128, 0, stream, o_raw, ldo, gate, ldg, w, eps, H, Dv,
                      tok_seq, (__nv_bfloat16*)out, ld_out, items);
  return LLMI_ERR_BAD_DTYPE;
}
