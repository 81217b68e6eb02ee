// The hand-over of a layer that norms AFTER the residual sum:
//
//   u = skip * x + ls * y          (skip a constant, ls one number per channel or absent, y a sublayer's result)
//   x <- u / sqrt(mean(u^2) + eps) * w
//
// x [T, d] is the fp32 residual stream, rewritten in place; y [T, d] is fp32 and, with `clear_y`, left zero
// for the next sublayer to add into; the new x is also written in the run's type (`act`) for the
// contractions that read it next.  Sum, statistics and norm are fp32.  With y == nullptr and w == nullptr
// the kernel only makes the copy in the run's type (the first layer's input).
//
// Few rows: a block per row.  Many rows: a warp per row.  Either way a row's result depends on nothing
// else in the launch.
#include "common.cuh"

namespace dlgo {

template <typename T, bool WARP_ROW>
__global__ void __launch_bounds__(256)
scaled_add_rmsnorm_kernel(float* __restrict__ x, float* __restrict__ y, const float* __restrict__ ls,
                          const float* __restrict__ w, T* __restrict__ act, int rows, int d, float skip, float eps,
                          int clear_y) {
  __shared__ float red[32];
  pdl_launch_dependents();
  const int row = WARP_ROW ? blockIdx.x * 8 + (threadIdx.x >> 5) : blockIdx.x;
  const int tid = WARP_ROW ? (threadIdx.x & 31) : threadIdx.x;
  const int step = WARP_ROW ? 32 : blockDim.x;
  pdl_wait();
  if (WARP_ROW && row >= rows) return;
  float* xr = x + (size_t)row * d;
  float* yr = y == nullptr ? nullptr : y + (size_t)row * d;
  T* ar = act == nullptr ? nullptr : act + (size_t)row * d;
  if (w == nullptr) {            // copy only
    for (int i = tid; i < d; i += step) ar[i] = from_float<T>(xr[i]);
    return;
  }
  float ss = 0.f;
  for (int i = tid; i < d; i += step) {
    float u = skip * xr[i];
    if (yr != nullptr) {
      const float v = yr[i];
      u += (ls != nullptr ? ls[i] : 1.0f) * v;
      if (clear_y) yr[i] = 0.f;
    }
    xr[i] = u;                   // each thread reads back only what it wrote itself
    ss += u * u;
  }
  ss = WARP_ROW ? warp_sum(ss) : block_sum(ss, red);
  const float r = 1.0f / sqrtf(ss / (float)d + eps);
  for (int i = tid; i < d; i += step) {
    const float v = xr[i] * r * w[i];
    xr[i] = v;
    if (ar != nullptr) ar[i] = from_float<T>(v);
  }
}

template <typename T>
int launch_scaled_add_rmsnorm(float* x, float* y, const float* ls, const float* w, void* act, int rows, int d,
                              float skip, float eps, int clear_y, cudaStream_t stream) {
  if (rows > 64) {
    launch_kernel(scaled_add_rmsnorm_kernel<T, true>, dim3((rows + 7) / 8), dim3(256), 0, stream, x, y, ls, w, (T*)act,
                  rows, d, skip, eps, clear_y);
  } else {
    const int threads = d >= 2048 ? 256 : (d >= 512 ? 128 : 64);
    launch_kernel(scaled_add_rmsnorm_kernel<T, false>, dim3(rows), dim3(threads), 0, stream, x, y, ls, w, (T*)act, rows,
                  d, skip, eps, clear_y);
  }
  return launch_status();
}

}  // namespace dlgo

DLGO_EXPORT int dlgo_scaled_add_rmsnorm(float* x, float* y, const float* ls, const float* w, void* act, int dtype,
                                        int rows, int d, float skip, float eps, int clear_y, cudaStream_t stream) {
  if (rows <= 0) return DLGO_OK;
  if (d <= 0) return DLGO_ERR_SIZE;
  if (w == nullptr && (act == nullptr || y != nullptr)) return DLGO_ERR_SIZE;
  if (dtype == DLGO_F32)
    return dlgo::launch_scaled_add_rmsnorm<float>(x, y, ls, w, act, rows, d, skip, eps, clear_y, stream);
  if (dtype == DLGO_BF16)
    return dlgo::launch_scaled_add_rmsnorm<__nv_bfloat16>(x, y, ls, w, act, rows, d, skip, eps, clear_y, stream);
  return DLGO_ERR_DTYPE;
}
