// Fused softmax cross-entropy forward / backward for sm_100a (HBM-bound).
//
// Forward reads each logit once: every thread keeps an online (max, sum) pair in the
// log2 domain over 128-bit chunks of its row, the CTA merges the pairs, and only the
// per-row loss and log-sum-exp leave the chip.  Backward reads the logits and the saved
// log-sum-exp and writes (softmax - onehot) * grad in one pass.
#include "common.cuh"

namespace tfb {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr int CE_THREADS = 256;

__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
  const float mm = fmaxf(m, m2);
  // (-inf) - (-inf) would be NaN: an empty partner contributes nothing.
  const float a = (m == -INFINITY) ? 0.f : s * exp2f(m - mm);
  const float b = (m2 == -INFINITY) ? 0.f : s2 * exp2f(m2 - mm);
  m = mm;
  s = a + b;
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(CE_THREADS) ce_fwd_kernel(
    const T* __restrict__ logits, const int64_t* __restrict__ labels, T* __restrict__ loss,
    float* __restrict__ loss_f32, float* __restrict__ lse, int vocab, int64_t ld) {
  grid_dependency_wait();
  allow_dependents();
  __shared__ float sm_m[CE_THREADS / 32], sm_s[CE_THREADS / 32];
  const int64_t row = blockIdx.x;
  const T* xr = logits + row * ld;
  float m = -INFINITY, s = 0.f;  // log2 domain: sum of 2^(x*log2e - m)
  if (VEC) {
    const int nvec = vocab >> 3;
    for (int c = threadIdx.x; c < nvec; c += CE_THREADS) {
      float f[8];
      unpack8<T>(ld_stream16(xr + (int64_t)c * 8), f);
      float vm = f[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) vm = fmaxf(vm, f[j]);
      vm *= kLog2e;
      if (vm > m) {
        s *= exp2f(m - vm);  // m == -inf gives 0 * 0
        m = vm;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) s += exp2f(fmaf(f[j], kLog2e, -m));
    }
  } else {
    for (int c = threadIdx.x; c < vocab; c += CE_THREADS) {
      const float t = Num<T>::to_f(xr[c]) * kLog2e;
      if (t > m) {
        s *= exp2f(m - t);
        m = t;
      }
      s += exp2f(t - m);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
    online_merge(m, s, m2, s2);
  }
  if ((threadIdx.x & 31) == 0) {
    sm_m[threadIdx.x >> 5] = m;
    sm_s[threadIdx.x >> 5] = s;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    m = sm_m[0];
    s = sm_s[0];
    for (int w = 1; w < CE_THREADS / 32; ++w) online_merge(m, s, sm_m[w], sm_s[w]);
    const float l = (m + log2f(s)) * kLn2;
    lse[row] = l;
    const int64_t lab = labels[row];
    float v = 0.f;
    if (lab >= 0 && lab < vocab) v = l - Num<T>::to_f(xr[lab]);
    loss[row] = Num<T>::from_f(v);
    if (loss_f32) loss_f32[row] = v;
  }
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(CE_THREADS) ce_bwd_kernel(
    const T* __restrict__ logits, const int64_t* __restrict__ labels, const float* __restrict__ lse,
    const T* __restrict__ grad, int64_t grad_stride, T* __restrict__ dlogits, int vocab, int64_t ld,
    int64_t dld) {
  grid_dependency_wait();
  allow_dependents();
  const int64_t row = blockIdx.x;
  const T* xr = logits + row * ld;
  T* dr = dlogits + row * dld;
  const int64_t lab64 = labels[row];
  const bool valid = lab64 >= 0 && lab64 < vocab;
  const int lab = valid ? (int)lab64 : -1;
  const float g = valid ? Num<T>::to_f(grad[row * grad_stride]) : 0.f;
  const float l2 = lse[row] * kLog2e;
  if (VEC) {
    const int nvec = vocab >> 3;
    for (int c = threadIdx.x; c < nvec; c += CE_THREADS) {
      float f[8];
      unpack8<T>(ld_stream16(xr + (int64_t)c * 8), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = exp2f(fmaf(f[j], kLog2e, -l2));
      const int k = lab - c * 8;
      if (k >= 0 && k < 8) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j == k) f[j] -= 1.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] *= g;
      st_stream16(dr + (int64_t)c * 8, pack8<T>(f));
    }
  } else {
    for (int c = threadIdx.x; c < vocab; c += CE_THREADS) {
      float p = exp2f(fmaf(Num<T>::to_f(xr[c]), kLog2e, -l2));
      if (c == lab) p -= 1.f;
      dr[c] = Num<T>::from_f(p * g);
    }
  }
}

}  // namespace tfb

using namespace tfb;

extern "C" int tfb_cross_entropy_fwd(const void* logits, const int64_t* labels, void* loss,
                                     float* loss_f32, float* lse, int64_t rows, int64_t vocab,
                                     int64_t logits_ld, int dtype, void* stream) {
  TFB_REQUIRE(rows >= 0 && vocab > 0 && vocab < (1LL << 31) - 8, "cross_entropy_fwd: bad shape");
  TFB_REQUIRE(logits_ld >= vocab, "cross_entropy_fwd: row stride smaller than vocab");
  if (rows == 0) return TFB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = vocab % 8 == 0 && logits_ld % 8 == 0 && aligned16(logits);
  TFB_DISPATCH_16(dtype, T, {
    if (vec)
      launch_overlapped(ce_fwd_kernel<T, true>, dim3((unsigned)rows), dim3(CE_THREADS), 0, st, (const T*)logits, labels, (T*)loss, loss_f32, lse, (int)vocab, logits_ld);
    else
      launch_overlapped(ce_fwd_kernel<T, false>, dim3((unsigned)rows), dim3(CE_THREADS), 0, st, (const T*)logits, labels, (T*)loss, loss_f32, lse, (int)vocab, logits_ld);
  })
  return launched("cross_entropy_fwd");
}

extern "C" int tfb_cross_entropy_bwd(const void* logits, const int64_t* labels, const float* lse,
                                     const void* grad, int64_t grad_stride, void* dlogits,
                                     int64_t rows, int64_t vocab, int64_t logits_ld,
                                     int64_t dlogits_ld, int dtype, void* stream) {
  TFB_REQUIRE(rows >= 0 && vocab > 0 && vocab < (1LL << 31) - 8, "cross_entropy_bwd: bad shape");
  TFB_REQUIRE(logits_ld >= vocab && dlogits_ld >= vocab, "cross_entropy_bwd: row stride smaller than vocab");
  if (rows == 0) return TFB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = vocab % 8 == 0 && logits_ld % 8 == 0 && dlogits_ld % 8 == 0 && aligned16(logits) &&
                   aligned16(dlogits);
  TFB_DISPATCH_16(dtype, T, {
    if (vec)
      launch_overlapped(ce_bwd_kernel<T, true>, dim3((unsigned)rows), dim3(CE_THREADS), 0, st, (const T*)logits, labels, lse, (const T*)grad, grad_stride, (T*)dlogits, (int)vocab,
          logits_ld, dlogits_ld);
    else
      launch_overlapped(ce_bwd_kernel<T, false>, dim3((unsigned)rows), dim3(CE_THREADS), 0, st, (const T*)logits, labels, lse, (const T*)grad, grad_stride, (T*)dlogits, (int)vocab,
          logits_ld, dlogits_ld);
  })
  return launched("cross_entropy_bwd");
}
