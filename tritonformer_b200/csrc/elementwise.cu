// ReLU gradient mask and column sums (bias gradient) for sm_100a: HBM-bound,
// 128-bit accesses, fp32 accumulation.
#include "common.cuh"

namespace tfb {

template <typename T> int finalize_partials(const float*, int64_t, int, int, void*, void*, cudaStream_t, int);

template <typename T>
__global__ void __launch_bounds__(256) relu_bwd_vec_kernel(const uint4* __restrict__ dy,
                                                           const uint4* __restrict__ act,
                                                           uint4* __restrict__ dz, int64_t nvec) {
  grid_dependency_wait();
  allow_dependents();
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float g[8], a[8];
    unpack8<T>(ld_stream16(dy + i), g);
    unpack8<T>(ld_stream16(act + i), a);
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] = a[j] > 0.f ? g[j] : 0.f;
    st_stream16(dz + i, pack8<T>(g));
  }
}

template <typename T>
__global__ void __launch_bounds__(256) relu_bwd_scalar_kernel(const T* __restrict__ dy, const T* __restrict__ act,
                                                              T* __restrict__ dz, int64_t n) {
  grid_dependency_wait();
  allow_dependents();
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    dz[i] = Num<T>::to_f(act[i]) > 0.f ? dy[i] : Num<T>::from_f(0.f);
}

// grid (ceil(cols/256), n_partials); block 256 = 32 column lanes (8 columns each) x 8 row lanes.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) colsum_kernel(const T* __restrict__ x, float* __restrict__ partials,
                                                     int64_t rows, int cols, int64_t ld) {
  grid_dependency_wait();
  allow_dependents();
  __shared__ float sm[8][32][9];
  const int cl = threadIdx.x & 31, rl = threadIdx.x >> 5;
  const int c0 = (blockIdx.x * 32 + cl) * 8;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  if (c0 < cols) {
    const int ncol = min(8, cols - c0);
    for (int64_t r = (int64_t)blockIdx.y * 8 + rl; r < rows; r += (int64_t)gridDim.y * 8) {
      if (VEC) {
        float f[8];
        unpack8<T>(ld_stream16(x + r * ld + c0), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += f[j];
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j < ncol) acc[j] += Num<T>::to_f(x[r * ld + c0 + j]);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) sm[rl][cl][j] = acc[j];
  __syncthreads();
  // 256 threads fold 8 row lanes for 32*8 columns
  const int cc = threadIdx.x;  // column within the CTA's 256
  const int col = blockIdx.x * 256 + cc;
  if (col < cols) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += sm[i][cc >> 3][cc & 7];
    partials[(int64_t)blockIdx.y * cols + col] = s;
  }
}

}  // namespace tfb

using namespace tfb;

extern "C" int tfb_relu_bwd(const void* dy, const void* act, void* dz, int64_t n, int dtype,
                            void* stream) {
  TFB_REQUIRE(n >= 0, "relu_bwd: negative size");
  if (n == 0) return TFB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = n % 8 == 0 && aligned16(dy) && aligned16(act) && aligned16(dz);
  TFB_DISPATCH_16(dtype, T, {
    if (vec) {
      const int64_t nvec = n / 8;
      const unsigned grid = (unsigned)(ceil_div(nvec, 256) < 148 * 16 ? ceil_div(nvec, 256) : 148 * 16);
      launch_overlapped(relu_bwd_vec_kernel<T>, dim3(grid), dim3(256), 0, st, (const uint4*)dy, (const uint4*)act, (uint4*)dz, nvec);
    } else {
      const unsigned grid = (unsigned)(ceil_div(n, 256) < 148 * 16 ? ceil_div(n, 256) : 148 * 16);
      launch_overlapped(relu_bwd_scalar_kernel<T>, dim3(grid), dim3(256), 0, st, (const T*)dy, (const T*)act, (T*)dz, n);
    }
  })
  return launched("relu_bwd");
}

extern "C" int64_t tfb_colsum_partials(int64_t rows, int64_t cols) {
  // enough row slices to fill the machine given ceil(cols/256) column CTAs
  const int64_t col_ctas = ceil_div(cols, 256);
  int64_t n = ceil_div(148 * 4, col_ctas);
  const int64_t max_n = ceil_div(rows, 8);
  if (n > max_n) n = max_n;
  return n < 1 ? 1 : n;
}

extern "C" int tfb_colsum(const void* x, void* out, float* partials, int64_t n_partials,
                          int64_t rows, int64_t cols, int64_t x_ld, int dtype, void* stream) {
  TFB_REQUIRE(rows > 0 && cols > 0 && cols < (1 << 30), "colsum: bad shape");
  TFB_REQUIRE(x_ld >= cols, "colsum: row stride smaller than cols");
  TFB_REQUIRE(n_partials == tfb_colsum_partials(rows, cols),
              "colsum: scratch must hold tfb_colsum_partials() rows");
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = cols % 8 == 0 && x_ld % 8 == 0 && aligned16(x);
  dim3 grid((unsigned)ceil_div(cols, 256), (unsigned)n_partials);
  TFB_DISPATCH_16(dtype, T, {
    if (vec) launch_overlapped(colsum_kernel<T, true>, dim3(grid), dim3(256), 0, st, (const T*)x, partials, rows, (int)cols, x_ld);
    else launch_overlapped(colsum_kernel<T, false>, dim3(grid), dim3(256), 0, st, (const T*)x, partials, rows, (int)cols, x_ld);
    int rc = launched("colsum");
    if (rc) return rc;
    return finalize_partials<T>(partials, n_partials, (int)cols, (int)cols, out, out, st, 0);
  })
}
