// Latent attention on the tensor cores (bf16): the kernel for prompts and for single tokens.
//
// All heads of a token read the same cached rows [c (C) | r (R)], so a block takes 16 query rows that share their
// keys — 16 heads of one token, or a few consecutive tokens of one sequence times all heads when there are fewer
// than 16 — and streams the sequence's rows ONCE for all of them, a page of 64 rows at a time:
//     S[16 x 64]  = Q[16 x (C+R)] · rowsᵀ        mma.sync m16n8k16 (bf16 in, fp32 out); warp w: keys 16w .. 16w+15
//     softmax     running maximum and sum per query row, fp32, shared by the four warps through shared memory
//     O[16 x C]  += P[16 x 64] · rows[:, :C]      warp w: columns wC/4 .. (w+1)C/4 - 1; the page serves as key AND value
// Pages arrive by cp.async into two buffers, the next one while the current one is multiplied; rows of a page beyond
// the block's newest position arrive as zeros.  With `splits` > 1 (single tokens over long caches) grid.z cuts the
// positions; every cut leaves (maximum, sum, unnormalised O) in a workspace and a second kernel joins them.
// Needs C % 64 == 0, (C + R) % 16 == 0, C <= 512, pages of 64 rows.
#include <math.h>

#include "common.cuh"
#include "mma_sync.cuh"
#include "step_meta.cuh"

namespace llmi {

constexpr int LM_ROWS = 16, LM_KEYS = 64, LM_WARPS = 4, LM_PAD = 8;

struct LatentMmaArgs {
  const __nv_bfloat16* qa;      // [T, H, C+R]
  long ldq;
  __nv_bfloat16* out;           // [T, H, C]
  long ldo;
  const __nv_bfloat16* cache;   // [page][1][64][C+R]
  const int32_t* tok_seq;
  const int32_t* tok_pos;
  const int32_t* seq_pages;
  int pages_stride;
  int n_tokens, n_heads, C, R;
  int heads_per_block, tokens_per_block;    // their product is 16
  int splits, pages_per_split;
  int page_buffers;             // 2: the next page arrives while the current one is multiplied; 1: half the shared memory,
                                // so that two blocks share an SM and overlap each other instead (steps of single tokens)
  float scale;
  float* ws_o;                  // [T, H, splits, C]   (splits > 1)
  float* ws_ml;                 // [T, H, splits, 2]
};

// NT = C / 32: the 8-column tiles of O that one warp owns.  RG: groups of 16 query rows (of four warps each) that share
// the block's pages — 1 for single tokens, 2 for prompts, where a page then feeds twice the rows per load.
template <int NT, int RG>
__global__ void __launch_bounds__(LM_WARPS * 32 * RG)
attention_latent_mma_kernel(const LatentMmaArgs a) {
  extern __shared__ __align__(16) unsigned char lm_smem[];
  pdl_wait();
  pdl_launch_dependents();
  const int Dk = a.C + a.R, ldk = Dk + LM_PAD;               // padded pitch: ldmatrix rows fall on different banks
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(lm_smem);                 // [RG * 16][ldk]
  __nv_bfloat16* k_s = q_s + RG * LM_ROWS * ldk;                                   // [page_buffers][64][ldk]
  const int rg = threadIdx.x >> 7;                                                 // my group of 16 rows
  const int nbuf = a.page_buffers;
  __nv_bfloat16* p_s = k_s + nbuf * LM_KEYS * ldk + rg * LM_ROWS * (LM_KEYS + LM_PAD);      // [RG][16][64 + 8]: my group's
  float* max_s = reinterpret_cast<float*>(k_s + nbuf * LM_KEYS * ldk + RG * LM_ROWS * (LM_KEYS + LM_PAD)) + rg * LM_WARPS * LM_ROWS;   // [RG][4][16]
  float* sum_s = max_s + RG * LM_WARPS * LM_ROWS;                                  // [RG][4][16]
  const int warp = (threadIdx.x >> 5) & 3, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  const int t0 = blockIdx.x * a.tokens_per_block, h0 = blockIdx.y * a.heads_per_block, split = blockIdx.z;
  const int t_last = min(t0 + a.tokens_per_block, a.n_tokens) - 1;

  // the block's tokens may belong to more than one sequence (they are flattened in sequence order): one pass each
  int seq_lo = 0x7fffffff, seq_hi = -1;
  for (int t = t0; t <= t_last; ++t) {
    const int s = a.tok_seq[t];
    if (s >= 0) { seq_lo = min(seq_lo, s); seq_hi = max(seq_hi, s); }
  }
  // my two rows: r = g and g + 8; row r is token t0 + r / heads_per_block, head h0 + r % heads_per_block
  int row_tok[2], row_head[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = rg * LM_ROWS + g + 8 * i;
    row_tok[i] = t0 + r / a.heads_per_block;
    row_head[i] = h0 + r % a.heads_per_block;
  }

  for (int seq = seq_lo; seq <= seq_hi; ++seq) {
    __syncthreads();                                           // the pass before has read q_s and k_s out
    // queries of this pass: rows of other sequences, of no token or of no head are zeros and see no key
    int newest = -1;
    for (int t = t0; t <= t_last; ++t)
      if (a.tok_seq[t] == seq) newest = max(newest, a.tok_pos[t]);
    int row_pos[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const bool ok = row_tok[i] <= t_last && row_head[i] < a.n_heads && a.tok_seq[row_tok[i]] == seq;
      row_pos[i] = ok ? a.tok_pos[row_tok[i]] : -1;
    }
    const int chunks = Dk / 8;
    for (int idx = threadIdx.x; idx < RG * LM_ROWS * chunks; idx += blockDim.x) {
      const int r = idx / chunks, c8 = idx - r * chunks;
      const int t = t0 + r / a.heads_per_block, h = h0 + r % a.heads_per_block;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (t <= t_last && h < a.n_heads && a.tok_seq[t] == seq)
        v = *reinterpret_cast<const uint4*>(a.qa + (size_t)t * a.ldq + (size_t)h * Dk + 8 * c8);
      *reinterpret_cast<uint4*>(q_s + r * ldk + 8 * c8) = v;
    }
    const int n_pages = newest / LM_KEYS + 1;
    const int pg_lo = split * a.pages_per_split, pg_hi = min(n_pages, pg_lo + a.pages_per_split);

    auto fetch = [&](int pg, int buf) {
      const int page = a.seq_pages[(size_t)seq * a.pages_stride + pg];
      const __nv_bfloat16* src = a.cache + (size_t)page * LM_KEYS * Dk;
      __nv_bfloat16* dst = k_s + (size_t)buf * LM_KEYS * ldk;
      for (int r = threadIdx.x >> 5; r < LM_KEYS; r += RG * LM_WARPS) {          // a warp copies whole rows
        const bool live = page >= 0 && pg * LM_KEYS + r <= newest;
        const __nv_bfloat16* from = live ? src + (size_t)r * Dk : a.cache;
        for (int c8 = lane; c8 < chunks; c8 += 32) cp_async16(dst + r * ldk + 8 * c8, live ? from + 8 * c8 : from, live ? 16 : 0);
      }
      cp_async_commit();
    };

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[j][e] = 0.f;

    if (pg_lo < pg_hi) fetch(pg_lo, 0);
    for (int pg = pg_lo; pg < pg_hi; ++pg) {
      const int buf = nbuf == 2 ? (pg - pg_lo) & 1 : 0;
      cp_async_wait_all();
      __syncthreads();                                         // this page is here; everyone is done with the page before
      if (nbuf == 2 && pg + 1 < pg_hi) fetch(pg + 1, buf ^ 1);
      const __nv_bfloat16* kt = k_s + (size_t)buf * LM_KEYS * ldk;

      // scores of my warp's 16 keys; the k steps go round four sets of accumulators, so that the chain of dependent
      // products is a quarter as long
      float s4[4][2][4];
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) s4[c][j][e] = 0.f;
      const __nv_bfloat16* a_ptr = q_s + (rg * LM_ROWS + (lane & 15)) * ldk + (lane >> 4) * 8;
      const __nv_bfloat16* b_ptr = kt + (16 * warp + (lane >> 4) * 8 + (lane & 7)) * ldk + ((lane >> 3) & 1) * 8;
      int k0 = 0;
      for (; k0 + 64 <= Dk; k0 += 64) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t af[4], bf[4];
          ldsm_x4(af, a_ptr + k0 + 16 * c);
          ldsm_x4(bf, b_ptr + k0 + 16 * c);
          mma_bf16(s4[c][0], af, bf[0], bf[1]);
          mma_bf16(s4[c][1], af, bf[2], bf[3]);
        }
      }
      for (; k0 < Dk; k0 += 16) {
        uint32_t af[4], bf[4];
        ldsm_x4(af, a_ptr + k0);
        ldsm_x4(bf, b_ptr + k0);
        mma_bf16(s4[0][0], af, bf[0], bf[1]);
        mma_bf16(s4[0][1], af, bf[2], bf[3]);
      }
      float s[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[j][e] = (s4[0][j][e] + s4[1][j][e]) + (s4[2][j][e] + s4[3][j][e]);
      // mask, and the maximum of each of my rows over my warp's keys
      const int key0 = pg * LM_KEYS + 16 * warp + 2 * tq;
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = key0 + 8 * j + (e & 1), i = e >> 1;
          const float v = key <= row_pos[i] ? s[j][e] * a.scale : -INFINITY;
          s[j][e] = v;
          mx[i] = fmaxf(mx[i], v);
        }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
        if (tq == 0) max_s[warp * LM_ROWS + g + 8 * i] = mx[i];
      }
      __syncthreads();
      float m_new[2], corr[2], ps[2] = {0.f, 0.f};
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        float m = m_run[i];
#pragma unroll
        for (int w = 0; w < LM_WARPS; ++w) m = fmaxf(m, max_s[w * LM_ROWS + g + 8 * i]);
        m_new[i] = m;
        corr[i] = m == -INFINITY ? 1.f : expf(m_run[i] - m);     // a row that has seen no key yet keeps its zeros
      }
      __nv_bfloat16* p_row0 = p_s + g * (LM_KEYS + LM_PAD) + 16 * warp + 2 * tq;
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const float shift = m_new[i] == -INFINITY ? 0.f : m_new[i];
          const __nv_bfloat162 pp = __floats2bfloat162_rn(expf(s[j][2 * i] - shift), expf(s[j][2 * i + 1] - shift));
          // the sum runs over the rounded weights, the ones the context is made of
          ps[i] += __low2float(pp) + __high2float(pp);
          *reinterpret_cast<__nv_bfloat162*>(p_row0 + 8 * i * (LM_KEYS + LM_PAD) + 8 * j) = pp;
        }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        ps[i] += __shfl_xor_sync(0xffffffffu, ps[i], 1);
        ps[i] += __shfl_xor_sync(0xffffffffu, ps[i], 2);
        if (tq == 0) sum_s[warp * LM_ROWS + g + 8 * i] = ps[i];
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        float add = 0.f;
#pragma unroll
        for (int w = 0; w < LM_WARPS; ++w) add += sum_s[w * LM_ROWS + g + 8 * i];
        l_run[i] = l_run[i] * corr[i] + add;
        m_run[i] = m_new[i];
      }
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        o[j][0] *= corr[0]; o[j][1] *= corr[0];
        o[j][2] *= corr[1]; o[j][3] *= corr[1];
      }
      // context: my warp's columns, all 64 keys of the page
      const int col0 = warp * (NT * 8);
      const __nv_bfloat16* pa_ptr = p_s + (lane & 15) * (LM_KEYS + LM_PAD) + (lane >> 4) * 8;
      const __nv_bfloat16* v_ptr = kt + (((lane >> 3) & 1) * 8 + (lane & 7)) * ldk + col0 + (lane >> 4) * 8;
#pragma unroll
      for (int kk = 0; kk < LM_KEYS; kk += 16) {
        uint32_t af[4];
        ldsm_x4(af, pa_ptr + kk);
#pragma unroll
        for (int j = 0; j < NT; j += 2) {
          uint32_t bf[4];
          ldsm_x4_t(bf, v_ptr + (size_t)kk * ldk + 8 * j);
          mma_bf16(o[j], af, bf[0], bf[1]);
          mma_bf16(o[j + 1], af, bf[2], bf[3]);
        }
      }
      if (nbuf == 1 && pg + 1 < pg_hi) {
        __syncthreads();                                       // everyone has read this page out
        fetch(pg + 1, 0);
      }
    }
    cp_async_wait_all();

    // out
    const int col0 = warp * (NT * 8) + 2 * tq;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if (row_pos[i] < 0) continue;
      const int t = row_tok[i], h = row_head[i];
      if (a.splits == 1) {
        const float inv = 1.0f / l_run[i];
        __nv_bfloat16* dst = a.out + (size_t)t * a.ldo + (size_t)h * a.C + col0;
#pragma unroll
        for (int j = 0; j < NT; ++j)
          *reinterpret_cast<__nv_bfloat162*>(dst + 8 * j) = __floats2bfloat162_rn(o[j][2 * i] * inv, o[j][2 * i + 1] * inv);
      } else {
        const size_t item = ((size_t)t * a.n_heads + h) * a.splits + split;
        float* dst = a.ws_o + item * a.C + col0;
#pragma unroll
        for (int j = 0; j < NT; ++j) *reinterpret_cast<float2*>(dst + 8 * j) = make_float2(o[j][2 * i], o[j][2 * i + 1]);
        if (warp == 0 && tq == 0) {
          a.ws_ml[2 * item] = m_run[i];
          a.ws_ml[2 * item + 1] = l_run[i];
        }
      }
    }
  }
  // token rows of no sequence: zeros (one thread group per row)
  if (blockIdx.z == 0)
    for (int t = t0; t <= t_last; ++t)
      if (a.tok_seq[t] < 0)
        for (int hh = h0; hh < min(a.n_heads, h0 + a.heads_per_block); ++hh)
          for (int c = threadIdx.x; c < a.C; c += blockDim.x) a.out[(size_t)t * a.ldo + (size_t)hh * a.C + c] = __float2bfloat16_rn(0.f);
}

// One block per (token, head): joins the cuts.  out = sum_s e^(m_s - M) O_s / sum_s e^(m_s - M) l_s.  The weights
// e^(m_s - M) / denominator are made once, in shared memory; every thread then adds its columns over the cuts with
// independent loads.
constexpr int LM_MAX_SPLITS = 512;
__global__ void __launch_bounds__(128)
attention_latent_join_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_ml, __nv_bfloat16* __restrict__ out,
                             long ldo, const int32_t* __restrict__ tok_seq, int n_heads, int C, int splits) {
  __shared__ float w_s[LM_MAX_SPLITS];
  __shared__ float red[32];
  pdl_wait();
  pdl_launch_dependents();
  const long item = blockIdx.x;
  const int t = (int)(item / n_heads), h = (int)(item - (long)t * n_heads);
  if (tok_seq[t] < 0) return;                                 // (zeros were written by the first kernel)
  const float* ml = ws_ml + (size_t)item * splits * 2;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, ml[2 * s]);   // (the same few words for every thread: served by the cache)
  float part = 0.f;
  for (int s = threadIdx.x; s < splits; s += blockDim.x) {
    const float m = ml[2 * s];
    const float w = m == -INFINITY ? 0.f : expf(m - M);
    w_s[s] = w;
    part += w * ml[2 * s + 1];
  }
  const float denom = block_sum(part, red);
  const float inv = 1.0f / denom;
  const float* o = ws_o + (size_t)item * splits * C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    int s = 0;
    for (; s + 4 <= splits; s += 4) {
      a0 = fmaf(w_s[s], o[(size_t)s * C + c], a0);
      a1 = fmaf(w_s[s + 1], o[(size_t)(s + 1) * C + c], a1);
      a2 = fmaf(w_s[s + 2], o[(size_t)(s + 2) * C + c], a2);
      a3 = fmaf(w_s[s + 3], o[(size_t)(s + 3) * C + c], a3);
    }
    for (; s < splits; ++s) a0 = fmaf(w_s[s], o[(size_t)s * C + c], a0);
    out[(size_t)t * ldo + (size_t)h * C + c] = __float2bfloat16_rn(((a0 + a1) + (a2 + a3)) * inv);
  }
}

template <int NT, int RG>
int launch_latent_mma_rg(const LatentMmaArgs& a, dim3 grid, size_t smem, cudaStream_t stream) {
  static PerDevice<size_t> allowed;
  if (smem > 48 * 1024 && allowed.here() < smem) {
    if (cudaFuncSetAttribute(attention_latent_mma_kernel<NT, RG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return LLMI_ERR_BAD_SIZE;
    allowed.here() = smem;
  }
  return launch_pdl(PDL_ATTENTION, attention_latent_mma_kernel<NT, RG>, grid, dim3(LM_WARPS * 32 * RG), smem, stream, a);
}
template <int NT>
int launch_latent_mma(const LatentMmaArgs& a, dim3 grid, size_t smem, int row_groups, cudaStream_t stream) {
  return row_groups == 2 ? launch_latent_mma_rg<NT, 2>(a, grid, smem, stream) : launch_latent_mma_rg<NT, 1>(a, grid, smem, stream);
}

}  // namespace llmi

using namespace llmi;

LLMI_EXPORT int llmi_attention_latent_mma_supported(int C, int R, int page_size) {
  return C > 0 && R >= 0 && C % 64 == 0 && C <= 512 && (C + R) % 16 == 0 && page_size == LM_KEYS && (C / 32 <= 8 || C / 32 == 12 || C / 32 == 16);
}

// floats of workspace for `splits` cuts: O parts and (maximum, sum) pairs
LLMI_EXPORT long llmi_attention_latent_mma_workspace(int n_tokens, int n_heads, int C, int splits) {
  return splits <= 1 ? 0 : (long)n_tokens * n_heads * splits * (C + 2);
}

LLMI_EXPORT int llmi_attention_latent_mma(const void* qa, long ldq, void* out, long ldo, const void* cache,
                                          const int32_t* tok_seq, const int32_t* tok_pos, const int32_t* seq_pages,
                                          int pages_stride, int page_size, int n_tokens, int n_heads, int C, int R, float scale,
                                          int splits, int pages_per_split, int row_groups, float* workspace,
                                          long workspace_floats, cudaStream_t stream) {
  if (n_tokens <= 0 || n_heads <= 0 || !llmi_attention_latent_mma_supported(C, R, page_size)) return LLMI_ERR_UNSUPPORTED;
  if (splits < 1 || splits > LM_MAX_SPLITS || pages_per_split < 1 || (row_groups != 1 && row_groups != 2)) return LLMI_ERR_BAD_SIZE;
  if (((uintptr_t)qa & 15) || ((uintptr_t)cache & 15) || (ldq % 8) || ((uintptr_t)out & 3) || (ldo % 2)) return LLMI_ERR_ALIGN;
  if (splits > 1 && (!workspace || workspace_floats < llmi_attention_latent_mma_workspace(n_tokens, n_heads, C, splits)))
    return LLMI_ERR_BAD_SIZE;
  int hpb = 1;
  while (hpb < n_heads && hpb < LM_ROWS) hpb *= 2;
  LatentMmaArgs a;
  a.qa = (const __nv_bfloat16*)qa; a.ldq = ldq; a.out = (__nv_bfloat16*)out; a.ldo = ldo; a.cache = (const __nv_bfloat16*)cache;
  a.tok_seq = tok_seq; a.tok_pos = tok_pos; a.seq_pages = seq_pages; a.pages_stride = pages_stride;
  a.n_tokens = n_tokens; a.n_heads = n_heads; a.C = C; a.R = R;
  a.heads_per_block = hpb; a.tokens_per_block = row_groups * LM_ROWS / hpb;
  a.splits = splits; a.pages_per_split = pages_per_split; a.scale = scale;
  a.page_buffers = row_groups == 1 ? 1 : 2;
  a.ws_o = workspace;
  a.ws_ml = workspace ? workspace + (size_t)n_tokens * n_heads * splits * C : nullptr;
  dim3 grid((n_tokens + a.tokens_per_block - 1) / a.tokens_per_block, (n_heads + hpb - 1) / hpb, splits);
  if (grid.y > 65535) return LLMI_ERR_BAD_SIZE;
  const int ldk = C + R + LM_PAD;
  const size_t smem = (size_t)(row_groups * LM_ROWS + a.page_buffers * LM_KEYS) * ldk * 2 +
                      (size_t)row_groups * (LM_ROWS * (LM_KEYS + LM_PAD) * 2 + 2 * LM_WARPS * LM_ROWS * 4);
  int rc;
  switch (C / 32) {
    case 2: rc = launch_latent_mma<2>(a, grid, smem, row_groups, stream); break;
    case 4: rc = launch_latent_mma<4>(a, grid, smem, row_groups, stream); break;
    case 6: rc = launch_latent_mma<6>(a, grid, smem, row_groups, stream); break;
    case 8: rc = launch_latent_mma<8>(a, grid, smem, row_groups, stream); break;
    case 12: rc = launch_latent_mma<12>(a, grid, smem, row_groups, stream); break;
    case 16: rc = launch_latent_mma<16>(a, grid, smem, row_groups, stream); break;
    default: return LLMI_ERR_UNSUPPORTED;
  }
  if (rc != LLMI_OK || splits == 1) return rc;
  const long items = (long)n_tokens * n_heads;
  return launch_pdl(PDL_SMALL, attention_latent_join_kernel, dim3((unsigned)items), dim3(128), 0, stream, (const float*)a.ws_o,
                    (const float*)a.ws_ml, (__nv_bfloat16*)out, ldo, tok_seq, n_heads, C, splits);
}
