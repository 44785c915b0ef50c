// Row softmax forward / backward over the last dimension (fp32, fp16 or bf16 rows).
//
// One warp per row.  Rows whose length and alignment allow it are read with 128-bit
// loads and kept in registers between the max, sum and write passes; every other row
// takes the scalar kernel, which re-reads the row from cache.
#include "common.cuh"

namespace tfb {

template <typename T> struct Vec16 { static constexpr int N = 8; };
template <> struct Vec16<float> { static constexpr int N = 4; };

template <typename T>
__device__ __forceinline__ void load_vec(const T* p, float* f) {
  if constexpr (sizeof(T) == 4) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  } else {
    float t[8];
    unpack8<T>(*reinterpret_cast<const uint4*>(p), t);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = t[i];
  }
}
template <typename T>
__device__ __forceinline__ void store_vec(T* p, const float* f) {
  if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  } else {
    float t[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) t[i] = f[i];
    *reinterpret_cast<uint4*>(p) = pack8<T>(t);
  }
}

constexpr float kLog2e = 1.4426950408889634f;

template <typename T, int NV>
__global__ void __launch_bounds__(128) softmax_fwd_vec_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                              int64_t rows, int cols, int64_t x_ld,
                                                              int64_t y_ld) {
  grid_dependency_wait();
  allow_dependents();
  constexpr int W = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nvec = cols / W;
  const T* xr = x + row * x_ld;
  float v[NV][W];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = i * 32 + lane;
    if (c < nvec) {
      load_vec<T>(xr + (int64_t)c * W, v[i]);
#pragma unroll
      for (int j = 0; j < W; ++j) m = fmaxf(m, v[i][j]);
    }
  }
  m = warp_max(m);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (i * 32 + lane < nvec) {
#pragma unroll
      for (int j = 0; j < W; ++j) {
        v[i][j] = exp2f((v[i][j] - m) * kLog2e);
        s += v[i][j];
      }
    }
  }
  const float inv = 1.f / warp_sum(s);
  T* yr = y + row * y_ld;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = i * 32 + lane;
    if (c < nvec) {
#pragma unroll
      for (int j = 0; j < W; ++j) v[i][j] *= inv;
      store_vec<T>(yr + (int64_t)c * W, v[i]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128) softmax_fwd_generic_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                                  int64_t rows, int cols, int64_t x_ld,
                                                                  int64_t y_ld) {
  grid_dependency_wait();
  allow_dependents();
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* xr = x + row * x_ld;
  float m = -INFINITY;
  for (int c = lane; c < cols; c += 32) m = fmaxf(m, Num<T>::to_f(xr[c]));
  m = warp_max(m);
  float s = 0.f;
  for (int c = lane; c < cols; c += 32) s += exp2f((Num<T>::to_f(xr[c]) - m) * kLog2e);
  const float inv = 1.f / warp_sum(s);
  T* yr = y + row * y_ld;
  for (int c = lane; c < cols; c += 32)
    yr[c] = Num<T>::from_f(exp2f((Num<T>::to_f(xr[c]) - m) * kLog2e) * inv);
}

// dx = y * (dy - sum_j y_j dy_j)
template <typename T, int NV>
__global__ void __launch_bounds__(128) softmax_bwd_vec_kernel(const T* __restrict__ dy, const T* __restrict__ y,
                                                              T* __restrict__ dx, int64_t rows, int cols,
                                                              int64_t dy_ld, int64_t y_ld, int64_t dx_ld) {
  grid_dependency_wait();
  allow_dependents();
  constexpr int W = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nvec = cols / W;
  float g[NV][W], p[NV][W];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = i * 32 + lane;
    if (c < nvec) {
      load_vec<T>(dy + row * dy_ld + (int64_t)c * W, g[i]);
      load_vec<T>(y + row * y_ld + (int64_t)c * W, p[i]);
#pragma unroll
      for (int j = 0; j < W; ++j) s += g[i][j] * p[i][j];
    }
  }
  s = warp_sum(s);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = i * 32 + lane;
    if (c < nvec) {
#pragma unroll
      for (int j = 0; j < W; ++j) g[i][j] = p[i][j] * (g[i][j] - s);
      store_vec<T>(dx + row * dx_ld + (int64_t)c * W, g[i]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128) softmax_bwd_generic_kernel(const T* __restrict__ dy,
                                                                  const T* __restrict__ y, T* __restrict__ dx,
                                                                  int64_t rows, int cols, int64_t dy_ld,
                                                                  int64_t y_ld, int64_t dx_ld) {
  grid_dependency_wait();
  allow_dependents();
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* gr = dy + row * dy_ld;
  const T* pr = y + row * y_ld;
  float s = 0.f;
  for (int c = lane; c < cols; c += 32) s += Num<T>::to_f(gr[c]) * Num<T>::to_f(pr[c]);
  s = warp_sum(s);
  T* o = dx + row * dx_ld;
  for (int c = lane; c < cols; c += 32)
    o[c] = Num<T>::from_f(Num<T>::to_f(pr[c]) * (Num<T>::to_f(gr[c]) - s));
}

template <typename T>
static int softmax_fwd_launch(const void* x, void* y, int64_t rows, int64_t cols, int64_t x_ld,
                              int64_t y_ld, cudaStream_t st) {
  constexpr int W = Vec16<T>::N;
  const unsigned grid = (unsigned)ceil_div(rows, 4);
  const bool vec = cols % W == 0 && x_ld % W == 0 && y_ld % W == 0 && aligned16(x) && aligned16(y) &&
                   cols <= 8 * 32 * W;
  const T* xp = (const T*)x;
  T* yp = (T*)y;
  const int nv = (int)ceil_div(cols, 32 * W);
  if (!vec) launch_overlapped(softmax_fwd_generic_kernel<T>, dim3(grid), dim3(128), 0, st, xp, yp, rows, (int)cols, x_ld, y_ld);
  else if (nv <= 1) launch_overlapped(softmax_fwd_vec_kernel<T, 1>, dim3(grid), dim3(128), 0, st, xp, yp, rows, (int)cols, x_ld, y_ld);
  else if (nv <= 2) launch_overlapped(softmax_fwd_vec_kernel<T, 2>, dim3(grid), dim3(128), 0, st, xp, yp, rows, (int)cols, x_ld, y_ld);
  else if (nv <= 4) launch_overlapped(softmax_fwd_vec_kernel<T, 4>, dim3(grid), dim3(128), 0, st, xp, yp, rows, (int)cols, x_ld, y_ld);
  else launch_overlapped(softmax_fwd_vec_kernel<T, 8>, dim3(grid), dim3(128), 0, st, xp, yp, rows, (int)cols, x_ld, y_ld);
  return launched("softmax_fwd");
}

template <typename T>
static int softmax_bwd_launch(const void* dy, const void* y, void* dx, int64_t rows, int64_t cols,
                              int64_t dy_ld, int64_t y_ld, int64_t dx_ld, cudaStream_t st) {
  constexpr int W = Vec16<T>::N;
  const unsigned grid = (unsigned)ceil_div(rows, 4);
  const bool vec = cols % W == 0 && dy_ld % W == 0 && y_ld % W == 0 && dx_ld % W == 0 &&
                   aligned16(dy) && aligned16(y) && aligned16(dx) && cols <= 8 * 32 * W;
  const T *gp = (const T*)dy, *pp = (const T*)y;
  T* op = (T*)dx;
  const int nv = (int)ceil_div(cols, 32 * W);
  if (!vec) launch_overlapped(softmax_bwd_generic_kernel<T>, dim3(grid), dim3(128), 0, st, gp, pp, op, rows, (int)cols, dy_ld, y_ld, dx_ld);
  else if (nv <= 1) launch_overlapped(softmax_bwd_vec_kernel<T, 1>, dim3(grid), dim3(128), 0, st, gp, pp, op, rows, (int)cols, dy_ld, y_ld, dx_ld);
  else if (nv <= 2) launch_overlapped(softmax_bwd_vec_kernel<T, 2>, dim3(grid), dim3(128), 0, st, gp, pp, op, rows, (int)cols, dy_ld, y_ld, dx_ld);
  else if (nv <= 4) launch_overlapped(softmax_bwd_vec_kernel<T, 4>, dim3(grid), dim3(128), 0, st, gp, pp, op, rows, (int)cols, dy_ld, y_ld, dx_ld);
  else launch_overlapped(softmax_bwd_vec_kernel<T, 8>, dim3(grid), dim3(128), 0, st, gp, pp, op, rows, (int)cols, dy_ld, y_ld, dx_ld);
  return launched("softmax_bwd");
}

}  // namespace tfb

using namespace tfb;

extern "C" int tfb_softmax_fwd(const void* x, void* y, int64_t rows, int64_t cols, int64_t x_ld,
                               int64_t y_ld, int dtype, void* stream) {
  TFB_REQUIRE(rows >= 0 && cols > 0 && cols < (1 << 30), "softmax_fwd: bad shape");
  TFB_REQUIRE(x_ld >= cols && y_ld >= cols, "softmax_fwd: row stride smaller than cols");
  if (rows == 0) return TFB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == TFB_F32) return softmax_fwd_launch<float>(x, y, rows, cols, x_ld, y_ld, st);
  if (dtype == TFB_F16) return softmax_fwd_launch<__half>(x, y, rows, cols, x_ld, y_ld, st);
  if (dtype == TFB_BF16) return softmax_fwd_launch<__nv_bfloat16>(x, y, rows, cols, x_ld, y_ld, st);
  return fail(TFB_ERR_ARG, "softmax_fwd: dtype %d", dtype);
}

extern "C" int tfb_softmax_bwd(const void* dy, const void* y, void* dx, int64_t rows, int64_t cols,
                               int64_t dy_ld, int64_t y_ld, int64_t dx_ld, int dtype, void* stream) {
  TFB_REQUIRE(rows >= 0 && cols > 0 && cols < (1 << 30), "softmax_bwd: bad shape");
  TFB_REQUIRE(dy_ld >= cols && y_ld >= cols && dx_ld >= cols, "softmax_bwd: row stride smaller than cols");
  if (rows == 0) return TFB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == TFB_F32) return softmax_bwd_launch<float>(dy, y, dx, rows, cols, dy_ld, y_ld, dx_ld, st);
  if (dtype == TFB_F16) return softmax_bwd_launch<__half>(dy, y, dx, rows, cols, dy_ld, y_ld, dx_ld, st);
  if (dtype == TFB_BF16)
    return softmax_bwd_launch<__nv_bfloat16>(dy, y, dx, rows, cols, dy_ld, y_ld, dx_ld, st);
  return fail(TFB_ERR_ARG, "softmax_bwd: dtype %d", dtype);
}
