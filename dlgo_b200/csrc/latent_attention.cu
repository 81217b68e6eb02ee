// Attention over a cache of latents (one vector of `rank` numbers per position, shared by all heads).
//
// Per position the cache holds c = rms(Wd h) * g.  A head's keys and values are k = Wk c and v = Wv c, so
//   score(i, j) = q_i . (Wk c_j) * scale = (Wk^T q_i) . c_j * scale
//   out_i       = Wv (sum_j p_ij c_j)
// and neither keys nor values are ever materialised: the query is carried into the latent space once, the
// softmax runs over the latents themselves, and the weighted latent is carried out through Wv at the end.
// Causal; `window` > 0 keeps keys with 0 <= i - j < window; `sink` (one number per head) adds exp(sink) to the
// softmax's denominator and nothing else.  No positions are encoded.
//
// latent_norm_append: the RMS norms of the down-projections (fp32), the kv latent appended to the paged
// cache, the query latent (if the queries go through one) handed on in the activation type.
// latent_attention:   one block per (token, head), all arithmetic in fp32; T is the type of the cache, the
//                     weights and the output.  Keys are spread over the block's warps in a fixed pattern, so a
//                     token's result does not depend on what else is in the batch.
#include "common.cuh"

namespace dlgo {

template <typename T>
__global__ void latent_norm_append_kernel(const float* __restrict__ proj, int ld, int kv_off, int kv_rank,
                                          const float* __restrict__ w_kv, int q_off, int q_rank,
                                          const float* __restrict__ w_q, T* __restrict__ cq, float eps,
                                          const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                                          const int* __restrict__ seq_slot, const int* __restrict__ page_table,
                                          int max_pages, T* __restrict__ pages, int page_size, int write_cache) {
  pdl_launch_dependents();
  __shared__ float scratch[32];
  __shared__ float scale_s;
  const int t = blockIdx.x;
  const bool is_q = blockIdx.y == 1;
  const int n = is_q ? q_rank : kv_rank;
  const float* w = is_q ? w_q : w_kv;
  T* dst = nullptr;
  if (is_q) {
    dst = cq + (size_t)t * q_rank;
  } else if (write_cache) {
    const int pos = token_pos[t];
    const int slot = seq_slot[token_seq[t]];
    const int page = page_table[(size_t)slot * max_pages + pos / page_size];
    if (page >= 0) dst = pages + ((size_t)page * page_size + pos % page_size) * kv_rank;
  }
  pdl_wait();
  if (dst == nullptr) return;
  const float* x = proj + (size_t)t * ld + (is_q ? q_off : kv_off);
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) ss = fmaf(x[i], x[i], ss);
  ss = block_sum(ss, scratch);
  if (threadIdx.x == 0) scale_s = 1.0f / sqrtf(ss / (float)n + eps);
  __syncthreads();
  const float sc = scale_s;
  for (int i = threadIdx.x; i < n; i += blockDim.x) dst[i] = from_float<T>(x[i] * sc * w[i]);
}

// Latents of the pages a prompt step attends, gathered into rows [n_tmp * page_size, rank] (row = temporary page
// * page_size + place in the page) for the contraction that makes the step's keys and values.  `tmp_pages`
// [n_tmp, 3]: (sequence of the step, its page index, rows of the page that are written); other rows are zero.
template <typename T>
__global__ void latent_gather_kernel(const T* __restrict__ pages, const int* __restrict__ page_table, int max_pages,
                                     int page_size, const int* __restrict__ tmp_pages,
                                     const int* __restrict__ seq_slot, T* __restrict__ out, int rank) {
  pdl_launch_dependents();
  const int tp = blockIdx.x;
  const int seq = tmp_pages[tp * 3], lp = tmp_pages[tp * 3 + 1], valid = tmp_pages[tp * 3 + 2];
  const int page = page_table[(size_t)seq_slot[seq] * max_pages + lp];
  pdl_wait();
  const T* src = pages + (size_t)(page < 0 ? 0 : page) * page_size * rank;
  T* dst = out + (size_t)tp * page_size * rank;
  const int n_valid = page < 0 ? 0 : valid * rank;
  for (int i = threadIdx.x; i < page_size * rank; i += blockDim.x) dst[i] = i < n_valid ? src[i] : from_float<T>(0.f);
}

__device__ __forceinline__ float2 load_pair(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load_pair(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}

constexpr int LA_WARPS = 8;

// NP: pairs of latent dimensions a lane holds (rank <= 64 * NP, rank even)
template <typename T, int NP>
__global__ void __launch_bounds__(LA_WARPS * 32)
latent_attention_kernel(const void* __restrict__ q, int q_is_f32, int ldq, const T* __restrict__ w_k,
                        const T* __restrict__ w_v, const float* __restrict__ sink, const T* __restrict__ pages,
                        const int* __restrict__ page_table, int max_pages, int page_size,
                        const int* __restrict__ seq_slot, const int* __restrict__ token_seq,
                        const int* __restrict__ token_pos, T* __restrict__ out, int ldo, int dk, int dv, int rank,
                        float scale, int window) {
  pdl_launch_dependents();
  extern __shared__ float smem[];
  float* s_q = smem;                         // [dk] the head's query
  float* s_lat = s_q + dk;                   // [rank] the query in latent space, later the weighted latent
  float* s_acc = s_lat + rank;               // [LA_WARPS][rank]
  __shared__ float s_m[LA_WARPS], s_l[LA_WARPS];
  const int t = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pos = token_pos[t];
  const int slot = seq_slot[token_seq[t]];
  const int* table = page_table + (size_t)slot * max_pages;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  pdl_wait();
  for (int i = threadIdx.x; i < dk; i += blockDim.x)
    s_q[i] = q_is_f32 ? reinterpret_cast<const float*>(q)[(size_t)t * ldq + h * dk + i]
                      : to_float(reinterpret_cast<const __nv_bfloat16*>(q)[(size_t)t * ldq + h * dk + i]);
  __syncthreads();
  // the query in latent space: (Wk_h)^T q
  const T* wk = w_k + (size_t)h * dk * rank;
  for (int r = threadIdx.x; r < rank; r += blockDim.x) {
    float a = 0.f;
    for (int i = 0; i < dk; ++i) a = fmaf(s_q[i], to_float(wk[(size_t)i * rank + r]), a);
    s_lat[r] = a;
  }
  __syncthreads();
  float2 ql[NP], acc[NP];
#pragma unroll
  for (int i = 0; i < NP; ++i) {
    const int r = (i * 32 + lane) * 2;
    ql[i] = r < rank ? make_float2(s_lat[r], s_lat[r + 1]) : make_float2(0.f, 0.f);
    acc[i] = make_float2(0.f, 0.f);
  }
  float m = -INFINITY, l = 0.f;
  for (int j = lo + warp; j <= pos; j += LA_WARPS) {
    const int page = table[j / page_size];
    const T* c = pages + ((size_t)page * page_size + j % page_size) * rank;
    float2 cv[NP];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NP; ++i) {
      const int r = (i * 32 + lane) * 2;
      cv[i] = r < rank ? load_pair(c + r) : make_float2(0.f, 0.f);
      s = fmaf(ql[i].x, cv[i].x, s);
      s = fmaf(ql[i].y, cv[i].y, s);
    }
    s = warp_sum(s) * scale;
    const float m_new = fmaxf(m, s);
    const float corr = expf(m - m_new);        // 0 for the first key (m = -inf)
    const float p = expf(s - m_new);
    l = fmaf(l, corr, p);
#pragma unroll
    for (int i = 0; i < NP; ++i) {
      acc[i].x = fmaf(acc[i].x, corr, p * cv[i].x);
      acc[i].y = fmaf(acc[i].y, corr, p * cv[i].y);
    }
    m = m_new;
  }
  if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
  for (int i = 0; i < NP; ++i) {
    const int r = (i * 32 + lane) * 2;
    if (r < rank) { s_acc[warp * rank + r] = acc[i].x; s_acc[warp * rank + r + 1] = acc[i].y; }
  }
  __syncthreads();
  // the warps' parts meet in warp order; the sink joins the denominator only
  const float sk = sink ? sink[h] : -INFINITY;
  float M = sk;
  for (int w = 0; w < LA_WARPS; ++w) M = fmaxf(M, s_m[w]);
  float L = sink ? expf(sk - M) : 0.f;
  float f[LA_WARPS];
#pragma unroll
  for (int w = 0; w < LA_WARPS; ++w) {
    f[w] = s_m[w] == -INFINITY ? 0.f : expf(s_m[w] - M);
    L = fmaf(s_l[w], f[w], L);
  }
  const float inv = 1.0f / L;
  for (int r = threadIdx.x; r < rank; r += blockDim.x) {
    float a = 0.f;
#pragma unroll
    for (int w = 0; w < LA_WARPS; ++w) a = fmaf(s_acc[w * rank + r], f[w], a);
    s_lat[r] = a * inv;
  }
  __syncthreads();
  // out through Wv_h: a warp per output column
  const T* wv = w_v + (size_t)h * dv * rank;
  for (int e = warp; e < dv; e += LA_WARPS) {
    const T* row = wv + (size_t)e * rank;
    float a = 0.f;
    for (int r = lane * 2; r < rank; r += 64) {
      const float2 wv2 = load_pair(row + r);
      a = fmaf(wv2.x, s_lat[r], a);
      a = fmaf(wv2.y, s_lat[r + 1], a);
    }
    a = warp_sum(a);
    if (lane == 0) out[(size_t)t * ldo + h * dv + e] = from_float<T>(a);
  }
}

template <typename T, int NP>
static int launch_latent(const void* q, int q_is_f32, int ldq, const void* w_k, const void* w_v, const float* sink,
                         const void* pages, const int* page_table, int max_pages, int page_size, const int* seq_slot,
                         const int* token_seq, const int* token_pos, void* out, int ldo, int T_tokens, int H, int dk,
                         int dv, int rank, float scale, int window, cudaStream_t stream) {
  const size_t smem = (size_t)(dk + rank + LA_WARPS * rank) * sizeof(float);
  if (smem > 200 * 1024) return DLGO_ERR_SIZE;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(latent_attention_kernel<T, NP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  launch_kernel(latent_attention_kernel<T, NP>, dim3(T_tokens, H), dim3(LA_WARPS * 32), smem, stream, q, q_is_f32, ldq,
                (const T*)w_k, (const T*)w_v, sink, (const T*)pages, page_table, max_pages, page_size, seq_slot,
                token_seq, token_pos, (T*)out, ldo, dk, dv, rank, scale, window);
  return launch_status();
}

}  // namespace dlgo

using namespace dlgo;

DLGO_EXPORT int dlgo_latent_norm_append(const float* proj, int ld, int T_tokens, int kv_off, int kv_rank,
                                        const float* w_kv, int q_off, int q_rank, const float* w_q, void* cq,
                                        float eps, const int* token_pos, const int* token_seq, const int* seq_slot,
                                        const int* page_table, int max_pages, void* pages, int dtype, int page_size,
                                        int write_cache, cudaStream_t stream) {
  if (T_tokens <= 0) return DLGO_OK;
  if (kv_rank <= 0 || q_rank < 0 || page_size <= 0) return DLGO_ERR_SIZE;
  const dim3 grid(T_tokens, q_rank > 0 ? 2 : 1);
  const int n = kv_rank > q_rank ? kv_rank : q_rank;
  const int threads = n >= 1024 ? 256 : 128;
  if (dtype == DLGO_F32)
    launch_kernel(latent_norm_append_kernel<float>, grid, dim3(threads), 0, stream, proj, ld, kv_off, kv_rank, w_kv,
                  q_off, q_rank, w_q, (float*)cq, eps, token_pos, token_seq, seq_slot, page_table, max_pages,
                  (float*)pages, page_size, write_cache);
  else if (dtype == DLGO_BF16)
    launch_kernel(latent_norm_append_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, proj, ld, kv_off, kv_rank,
                  w_kv, q_off, q_rank, w_q, (__nv_bfloat16*)cq, eps, token_pos, token_seq, seq_slot, page_table,
                  max_pages, (__nv_bfloat16*)pages, page_size, write_cache);
  else
    return DLGO_ERR_DTYPE;
  return launch_status();
}

DLGO_EXPORT int dlgo_latent_gather(const void* pages, int dtype, const int* page_table, int max_pages, int page_size,
                                   const int* tmp_pages, int n_tmp, const int* seq_slot, void* out, int rank,
                                   cudaStream_t stream) {
  if (n_tmp <= 0) return DLGO_OK;
  if (rank <= 0 || page_size <= 0) return DLGO_ERR_SIZE;
  if (dtype == DLGO_F32)
    launch_kernel(latent_gather_kernel<float>, dim3(n_tmp), dim3(256), 0, stream, (const float*)pages, page_table,
                  max_pages, page_size, tmp_pages, seq_slot, (float*)out, rank);
  else if (dtype == DLGO_BF16)
    launch_kernel(latent_gather_kernel<__nv_bfloat16>, dim3(n_tmp), dim3(256), 0, stream, (const __nv_bfloat16*)pages,
                  page_table, max_pages, page_size, tmp_pages, seq_slot, (__nv_bfloat16*)out, rank);
  else
    return DLGO_ERR_DTYPE;
  return launch_status();
}

#define LATENT_ARGS q, q_is_f32, ldq, w_k, w_v, sink, pages, page_table, max_pages, page_size, seq_slot, token_seq, \
                    token_pos, out, ldo, T_tokens, H, dk, dv, rank, scale, window, stream

template <typename T>
static int latent_by_rank(const void* q, int q_is_f32, int ldq, const void* w_k, const void* w_v, const float* sink,
                          const void* pages, const int* page_table, int max_pages, int page_size, const int* seq_slot,
                          const int* token_seq, const int* token_pos, void* out, int ldo, int T_tokens, int H, int dk,
                          int dv, int rank, float scale, int window, cudaStream_t stream) {
  if (rank <= 64) return launch_latent<T, 1>(LATENT_ARGS);
  if (rank <= 128) return launch_latent<T, 2>(LATENT_ARGS);
  if (rank <= 256) return launch_latent<T, 4>(LATENT_ARGS);
  if (rank <= 512) return launch_latent<T, 8>(LATENT_ARGS);
  if (rank <= 1024) return launch_latent<T, 16>(LATENT_ARGS);
  return DLGO_ERR_SIZE;
}

// q [T, >= H*dk] (fp32 or the cache's type), w_k [H*dk, rank], w_v [H*dv, rank], pages [n, page_size, rank],
// out [T, >= H*dv]; sink [H] fp32 or null; window 0: every earlier key
DLGO_EXPORT int dlgo_latent_attention(const void* q, int q_is_f32, int ldq, const void* w_k, const void* w_v,
                                      const float* sink, const void* pages, int dtype, const int* page_table,
                                      int max_pages, int page_size, const int* seq_slot, const int* token_seq,
                                      const int* token_pos, void* out, int ldo, int T_tokens, int H, int dk, int dv,
                                      int rank, float scale, int window, cudaStream_t stream) {
  if (T_tokens <= 0) return DLGO_OK;
  if (H <= 0 || dk <= 0 || dv <= 0 || rank <= 0 || (rank & 1) || page_size <= 0 || window < 0) return DLGO_ERR_SIZE;
  if (dtype == DLGO_F32) return latent_by_rank<float>(LATENT_ARGS);
  if (dtype == DLGO_BF16) {
    if (((uintptr_t)pages & 3) || ((uintptr_t)w_v & 3)) return DLGO_ERR_ALIGN;
    return latent_by_rank<__nv_bfloat16>(LATENT_ARGS);
  }
  return DLGO_ERR_DTYPE;
}
