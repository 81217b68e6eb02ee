// Per-head RMS norm of queries and keys, rotary positions computed from the position itself, and the
// append of this step's keys and values to the paged cache, in one pass over the fp32 result of the
// q|k (or q|k|v) projection.
//
// proj[T, ld] (fp32): Hq query heads, then Hkv key heads, then (unless `v_from_k`) Hkv value heads, hd
// numbers each; `bias` (fp32, one number per column, may be null) is added first.  With `v_from_k` the
// value of a position is its key as projected (with the bias, before norm and rotation).
//
//   head norm (w_q / w_k not null):  u <- u / sqrt(mean(u^2) + eps) * w      (plain weight, per head; the mean runs
//   over the first `norm_dim` numbers of a head: a head may be laid out with trailing zeros)
//   rotation of the first `rot` numbers of a head: (u_i, u_{i + rot/2}) turns by a = pos * freq[i],
//   with a = float(pos) * freq[i] in fp32 and cos / sin of that fp32 angle.
//
// q goes to q_out[T, Hq * hd] in the run's type; k and v go to the page of the token's position:
// pages[page_table[slot][pos / PS]][kv_head][pos % PS][:].  `clear`: zeros are left in proj (a sum that
// the projection's K-slices add themselves into and that must be zero again for the next step).
// Everything is fp32 until the final store.
#include "common.cuh"

namespace dlgo {

// Set when a token's position had no page in the table (-1): the append is skipped.
__device__ int g_headnorm_rope_error = 0;

constexpr int HR_WARPS = 4;

template <typename T>
__global__ void __launch_bounds__(HR_WARPS * 32)
headnorm_rope_append_kernel(float* __restrict__ proj, int ld, const float* __restrict__ bias,
                            const float* __restrict__ w_q, const float* __restrict__ w_k, float eps,
                            const float* __restrict__ freq, int rot, const int* __restrict__ token_pos,
                            const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
                            const int* __restrict__ page_table, int max_pages, T* __restrict__ kpages,
                            T* __restrict__ vpages, T* __restrict__ q_out, int T_tokens, int Hq, int Hkv, int hd,
                            int page_size, int v_from_k, int write_cache, int clear, int norm_dim) {
  extern __shared__ float hr_smem[];
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int heads = Hq + Hkv + (v_from_k ? 0 : Hkv);
  const long long item = (long long)blockIdx.x * HR_WARPS + warp;
  if (item >= (long long)T_tokens * heads) return;
  const int t = (int)(item / heads), head = (int)(item - (long long)t * heads);
  float* u = hr_smem + (size_t)warp * hd;
  // the step's own inputs: in place before the step's first kernel starts
  const int pos = token_pos[t];
  const bool is_q = head < Hq, is_k = !is_q && head < Hq + Hkv;
  T* kdst = nullptr;
  T* vdst = nullptr;
  if (!is_q && write_cache) {
    const int slot = seq_slot[token_seq[t]];
    const int page = page_table[(size_t)slot * max_pages + pos / page_size];
    if (page < 0) {
      if (lane == 0) atomicExch(&g_headnorm_rope_error, 1);
    } else {
      const int kvh = is_k ? head - Hq : head - Hq - Hkv;
      const size_t base = (((size_t)page * Hkv + kvh) * page_size + (size_t)(pos % page_size)) * hd;
      kdst = kpages + base;
      vdst = vpages + base;
    }
  }
  const float* w = is_q ? w_q : (is_k ? w_k : nullptr);
  pdl_wait();
  float* src = proj + (size_t)t * ld + (size_t)head * hd;
  float ss = 0.f;
  for (int i = lane; i < hd; i += 32) {
    float x = src[i];
    if (bias != nullptr) x += bias[(size_t)head * hd + i];
    u[i] = x;
    ss += x * x;
    if (is_k && v_from_k && vdst != nullptr) vdst[i] = from_float<T>(x);
  }
  if (clear)                     // (after every load of the row has been issued: a store right behind a load holds the loads up)
    for (int i = lane; i < hd; i += 32) src[i] = 0.f;
  if (!is_q && !is_k) {          // a value head of its own: stored as projected
    if (vdst != nullptr)
      for (int i = lane; i < hd; i += 32) vdst[i] = from_float<T>(u[i]);
    return;
  }
  ss = warp_sum(ss);
  const float r = (w != nullptr) ? 1.0f / sqrtf(ss / (float)norm_dim + eps) : 1.0f;
  __syncwarp();
  T* dst = is_q ? q_out + (size_t)t * Hq * hd + (size_t)head * hd : kdst;
  if (dst == nullptr) return;
  const int rh = rot / 2;
  const float p = (float)pos;
  for (int i = lane; i < rh; i += 32) {
    float a = u[i] * r, b = u[i + rh] * r;
    if (w != nullptr) { a *= w[i]; b *= w[i + rh]; }
    float sn, cs;
    sincosf(p * freq[i], &sn, &cs);
    dst[i] = from_float<T>(a * cs - b * sn);
    dst[i + rh] = from_float<T>(b * cs + a * sn);
  }
  for (int i = rot + lane; i < hd; i += 32) {
    float a = u[i] * r;
    if (w != nullptr) a *= w[i];
    dst[i] = from_float<T>(a);
  }
}

template <typename T>
int launch_headnorm_rope(float* proj, int ld, const float* bias, const float* w_q, const float* w_k, float eps,
                         const float* freq, int rot, const int* token_pos, const int* token_seq, const int* seq_slot,
                         const int* page_table, int max_pages, void* kpages, void* vpages, void* q_out, int T_tokens,
                         int Hq, int Hkv, int hd, int page_size, int v_from_k, int write_cache, int clear, int norm_dim,
                         cudaStream_t stream) {
  const int heads = Hq + Hkv + (v_from_k ? 0 : Hkv);
  const long long items = (long long)T_tokens * heads;
  const long long blocks = (items + HR_WARPS - 1) / HR_WARPS;
  if (blocks > 0x7fffffffLL) return DLGO_ERR_SIZE;
  const size_t smem = (size_t)HR_WARPS * hd * sizeof(float);
  if (smem > 48 * 1024) return DLGO_ERR_SIZE;
  launch_kernel(headnorm_rope_append_kernel<T>, dim3((unsigned)blocks), dim3(HR_WARPS * 32), smem, stream, proj, ld,
                bias, w_q, w_k, eps, freq, rot, token_pos, token_seq, seq_slot, page_table, max_pages, (T*)kpages,
                (T*)vpages, (T*)q_out, T_tokens, Hq, Hkv, hd, page_size, v_from_k, write_cache, clear, norm_dim);
  return launch_status();
}

}  // namespace dlgo

DLGO_EXPORT int dlgo_headnorm_rope_append(float* proj, int ld, const float* bias, const float* w_q, const float* w_k,
                                          float eps, const float* freq, int rot, const int* token_pos,
                                          const int* token_seq, const int* seq_slot, const int* page_table,
                                          int max_pages, void* kpages, void* vpages, void* q_out, int dtype, int T,
                                          int Hq, int Hkv, int hd, int page_size, int v_from_k, int write_cache,
                                          int clear, int norm_dim, cudaStream_t stream) {
  if (T <= 0) return DLGO_OK;
  if (Hq <= 0 || Hkv <= 0 || hd <= 0 || rot < 0 || rot > hd || rot % 2) return DLGO_ERR_SIZE;
  if (rot > 0 && freq == nullptr) return DLGO_ERR_SIZE;
  if (norm_dim <= 0 || norm_dim > hd) return DLGO_ERR_SIZE;
  if (ld < (Hq + Hkv + (v_from_k ? 0 : Hkv)) * hd) return DLGO_ERR_SIZE;
  if (dtype == DLGO_F32)
    return dlgo::launch_headnorm_rope<float>(proj, ld, bias, w_q, w_k, eps, freq, rot, token_pos, token_seq, seq_slot,
                                             page_table, max_pages, kpages, vpages, q_out, T, Hq, Hkv, hd, page_size,
                                             v_from_k, write_cache, clear, norm_dim, stream);
  if (dtype == DLGO_BF16)
    return dlgo::launch_headnorm_rope<__nv_bfloat16>(proj, ld, bias, w_q, w_k, eps, freq, rot, token_pos, token_seq,
                                                     seq_slot, page_table, max_pages, kpages, vpages, q_out, T, Hq,
                                                     Hkv, hd, page_size, v_from_k, write_cache, clear, norm_dim, stream);
  return DLGO_ERR_DTYPE;
}

// The error word (1: a position had no page), cleared by the read.
DLGO_EXPORT int dlgo_headnorm_rope_error() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, dlgo::g_headnorm_rope_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(dlgo::g_headnorm_rope_error, &zero, sizeof(int));
  return v;
}
