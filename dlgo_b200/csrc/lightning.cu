// Linear attention with a per-head decay ("lightning attention"), as a recurrence over a fixed-size state.
//
// Per head, with q_t = silu(Wq h_t), k_t = silu(Wk h_t) (dk numbers) and v_t = silu(Wv h_t) (dv numbers):
//   S_t = lambda * S_(t-1) + k_t v_t^T          S is [dk, dv], fp32, zero at a sequence's start
//   o_t = S_t^T q_t
// The state of a sequence lives in its slot of the state area between steps, so a prompt may arrive in any
// number of portions and decoding continues where the prompt stopped.
//
// lightning_scan: one block per (sequence, head); the state sits in shared memory while the block walks the
// sequence's tokens of this step in order.  The projections arrive as fp32 rows [q | k | v | ...]; silu,
// decay, state and output are fp32.
#include "common.cuh"

namespace dlgo {

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

__global__ void lightning_scan_kernel(const float* __restrict__ proj, int ld, int q_off, int k_off, int v_off,
                                      const int* __restrict__ tiles, const int* __restrict__ seq_slot,
                                      const float* __restrict__ decay, float* __restrict__ state,
                                      float* __restrict__ out, int ldo, int H, int dk, int dv) {
  pdl_launch_dependents();
  extern __shared__ float smem[];
  float* S = smem;                       // [dk][dv]
  float* qk = S + (size_t)dk * dv;       // two buffers of [q (dk) | k (dk) | v (dv)]
  const int per = 2 * dk + dv;
  const int h = blockIdx.y;
  const int seq = tiles[blockIdx.x * 3 + 0], first = tiles[blockIdx.x * 3 + 1], count = tiles[blockIdx.x * 3 + 2];
  const int slot = seq_slot[seq];
  const float lam = decay[h];
  float* st = state + ((size_t)slot * H + h) * dk * dv;
  pdl_wait();
  for (int i = threadIdx.x; i < dk * dv; i += blockDim.x) S[i] = st[i];
  auto fetch = [&](int tok, float* buf) {
    const float* row = proj + (size_t)tok * ld;
    for (int i = threadIdx.x; i < per; i += blockDim.x) {
      const int col = i < dk ? q_off + h * dk + i : (i < 2 * dk ? k_off + h * dk + (i - dk) : v_off + h * dv + (i - 2 * dk));
      buf[i] = silu_f(row[col]);
    }
  };
  fetch(first, qk);
  __syncthreads();
  for (int n = 0; n < count; ++n) {
    float* cur = qk + (n & 1) * per;
    if (n + 1 < count) fetch(first + n + 1, qk + ((n + 1) & 1) * per);
    const float* sq = cur;
    const float* sk = cur + dk;
    const float* sv = cur + 2 * dk;
    // a thread owns columns e of the state: no two threads touch the same element
    for (int e = threadIdx.x; e < dv; e += blockDim.x) {
      const float v = sv[e];
      float o = 0.f;
      for (int i = 0; i < dk; ++i) {
        const float s = fmaf(lam, S[i * dv + e], sk[i] * v);
        S[i * dv + e] = s;
        o = fmaf(s, sq[i], o);
      }
      out[(size_t)(first + n) * ldo + h * dv + e] = o;
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < dk * dv; i += blockDim.x) st[i] = S[i];
}

}  // namespace dlgo

using namespace dlgo;

// proj [T, ld] fp32; tiles [n_seqs, 3] (sequence, first packed token, count): one row per sequence of the step;
// state [slots, H, dk, dv] fp32; out [T, ldo] fp32 (heads side by side, dv each)
DLGO_EXPORT int dlgo_lightning_scan(const float* proj, int ld, int q_off, int k_off, int v_off, const int* tiles,
                                    int n_seqs, const int* seq_slot, const float* decay, float* state, float* out,
                                    int ldo, int H, int dk, int dv, cudaStream_t stream) {
  if (n_seqs <= 0) return DLGO_OK;
  if (H <= 0 || dk <= 0 || dv <= 0) return DLGO_ERR_SIZE;
  const size_t smem = ((size_t)dk * dv + 2 * (2 * dk + dv)) * sizeof(float);
  if (smem > 200 * 1024) return DLGO_ERR_SIZE;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(lightning_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  int threads = ((dv + 31) / 32) * 32;
  if (threads > 256) threads = 256;
  if (threads < 64) threads = 64;
  launch_kernel(lightning_scan_kernel, dim3(n_seqs, H), dim3(threads), smem, stream, proj, ld, q_off, k_off, v_off,
                tiles, seq_slot, decay, state, out, ldo, H, dk, dv);
  return launch_status();
}
