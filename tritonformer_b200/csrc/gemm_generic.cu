// Generic-stride tensor-core GEMM (mma.sync m16n8k16) for operands the TMA path cannot
// take: row pitches that are not multiples of 16 bytes, unaligned bases, tiny shapes.
// Element-wise predicated loads, 128x128x32 CTA tile, 8 warps of 64x32, fp32 accumulate.
#include "common.cuh"

namespace tfb {

template <typename T> struct MmaOp;
template <> struct MmaOp<__half> {
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  }
};
template <> struct MmaOp<__nv_bfloat16> {
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  }
};

constexpr int GB_M = 128, GB_N = 128, GB_K = 32, GB_PAD = 8, GB_THREADS = 256;
constexpr int GB_PER_THREAD = GB_M * GB_K / GB_THREADS;  // 16 elements of A and of B per thread

template <typename T>
__global__ void __launch_bounds__(GB_THREADS) gemm_generic_kernel(
    const T* __restrict__ A, const T* __restrict__ Bm, T* C, const T* __restrict__ bias, const T* addend,
    int64_t ld_addend, const T* mask, int64_t ld_mask, int M, int N, int K, int64_t a_sm, int64_t a_sk,
    int64_t b_sk, int64_t b_sn, int64_t ldc, int relu) {
  __shared__ __align__(16) T As[GB_M][GB_K + GB_PAD];
  __shared__ __align__(16) T Bs[GB_N][GB_K + GB_PAD];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = (warp >> 2) * 64, wn = (warp & 3) * 32;
  const int g = lane >> 2, t = lane & 3;
  const int m0 = blockIdx.y * GB_M, n0 = blockIdx.x * GB_N;
  const bool a_kfast = (a_sk == 1), b_kfast = (b_sk == 1);

  float acc[4][4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

  T ra[GB_PER_THREAD], rb[GB_PER_THREAD];
  const T zero = Num<T>::from_f(0.f);
  auto fetch = [&](int k0) {
#pragma unroll
    for (int i = 0; i < GB_PER_THREAD; ++i) {
      const int idx = tid + i * GB_THREADS;
      const int am = a_kfast ? idx / GB_K : idx % GB_M;
      const int ak = a_kfast ? idx % GB_K : idx / GB_M;
      const int gm = m0 + am, gk = k0 + ak;
      ra[i] = (gm < M && gk < K) ? A[(int64_t)gm * a_sm + (int64_t)gk * a_sk] : zero;
      const int bn = b_kfast ? idx / GB_K : idx % GB_N;
      const int bk = b_kfast ? idx % GB_K : idx / GB_N;
      const int gn = n0 + bn, gk2 = k0 + bk;
      rb[i] = (gn < N && gk2 < K) ? Bm[(int64_t)gk2 * b_sk + (int64_t)gn * b_sn] : zero;
    }
  };
  auto stash = [&]() {
#pragma unroll
    for (int i = 0; i < GB_PER_THREAD; ++i) {
      const int idx = tid + i * GB_THREADS;
      const int am = a_kfast ? idx / GB_K : idx % GB_M;
      const int ak = a_kfast ? idx % GB_K : idx / GB_M;
      As[am][ak] = ra[i];
      const int bn = b_kfast ? idx / GB_K : idx % GB_N;
      const int bk = b_kfast ? idx % GB_K : idx / GB_N;
      Bs[bn][bk] = rb[i];
    }
  };

  fetch(0);
  for (int k0 = 0; k0 < K; k0 += GB_K) {
    __syncthreads();  // previous tile fully consumed
    stash();
    __syncthreads();
    if (k0 + GB_K < K) fetch(k0 + GB_K);
#pragma unroll
    for (int kk = 0; kk < GB_K; kk += 16) {
      uint32_t af[4][4], bf[4][2];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = wm + i * 16 + g;
        af[i][0] = *reinterpret_cast<const uint32_t*>(&As[r][kk + 2 * t]);
        af[i][1] = *reinterpret_cast<const uint32_t*>(&As[r + 8][kk + 2 * t]);
        af[i][2] = *reinterpret_cast<const uint32_t*>(&As[r][kk + 2 * t + 8]);
        af[i][3] = *reinterpret_cast<const uint32_t*>(&As[r + 8][kk + 2 * t + 8]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = wn + j * 8 + g;
        bf[j][0] = *reinterpret_cast<const uint32_t*>(&Bs[c][kk + 2 * t]);
        bf[j][1] = *reinterpret_cast<const uint32_t*>(&Bs[c][kk + 2 * t + 8]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) MmaOp<T>::mma(acc[i][j], af[i], bf[j]);
    }
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int m = m0 + wm + i * 16 + g + ((e >> 1) ? 8 : 0);
        const int n = n0 + wn + j * 8 + 2 * t + (e & 1);
        if (m < M && n < N) {
          float v = acc[i][j][e];
          if (bias) v += Num<T>::to_f(bias[n]);
          if (relu) v = fmaxf(v, 0.f);
          if (addend) v += Num<T>::to_f(addend[(int64_t)m * ld_addend + n]);
          if (mask && !(Num<T>::to_f(mask[(int64_t)m * ld_mask + n]) > 0.f)) v = 0.f;
          C[(int64_t)m * ldc + n] = Num<T>::from_f(v);
        }
      }
    }
  }
}

int gemm_generic(const void* a, const void* b, void* c, const void* bias, const void* addend, int64_t ld_addend,
                 const void* mask, int64_t ld_mask, int64_t M, int64_t N, int64_t K, int64_t a_sm, int64_t a_sk,
                 int64_t b_sk, int64_t b_sn, int64_t ldc, int relu, int dtype, cudaStream_t st) {
  dim3 grid((unsigned)ceil_div(N, GB_N), (unsigned)ceil_div(M, GB_M));
  if (grid.y > 65535) return fail(TFB_ERR_UNSUPPORTED, "gemm(generic): M=%lld too large", (long long)M);
  TFB_DISPATCH_16(dtype, T, {
    gemm_generic_kernel<T><<<grid, GB_THREADS, 0, st>>>((const T*)a, (const T*)b, (T*)c, (const T*)bias,
                                                        (const T*)addend, ld_addend, (const T*)mask, ld_mask,
                                                        (int)M, (int)N, (int)K, a_sm, a_sk, b_sk, b_sn, ldc, relu);
  })
  return launched("gemm_generic");
}

}  // namespace tfb
