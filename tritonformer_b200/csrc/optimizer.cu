// Optimizer step on the flat gradient buckets for sm_100a: loss-scale handling and AdamW with fp32 master
// weights, entirely on the device (no host read decides anything), HBM-bound.
//
//   grad_check      one pass over a bucket of 16-bit gradients: raises *found_inf if any value is not finite
//   adamw_step      per element: g = grad * inv_scale; decoupled weight decay on the fp32 master weight;
//                   m, v moment updates; bias-corrected step; the 16-bit parameter is the rounded master weight.
//                   The whole launch does nothing while *found_inf is set (the step is skipped as a whole).
//   scale_update    one thread: dynamic loss scale (back off after a skipped step, grow after `interval` good
//                   ones), the step counter (advances only when the step was taken), and clears found_inf.
// The arithmetic follows torch.optim.AdamW's single-tensor form operation by operation (decay, lerp of the
// first moment, mul + addcmul of the second, sqrt / sqrt(bias_correction2) + eps, addcdiv) with the bias
// corrections evaluated in double like the Python floats there, so the fp32 state tracks a CPU run of
// torch.optim.AdamW to the last bit or one unit beside it.
// Algorithmic bytes per element (e = 2): check e; step e (grad) + 12 read + 12 written (master, m, v) + e (param).
#include "common.cuh"

namespace tfb {

template <typename T>
__global__ void __launch_bounds__(256) grad_check_kernel(const T* __restrict__ grad, int64_t n, int* __restrict__ found_inf) {
  grid_dependency_wait();
  allow_dependents();
  bool bad = false;
  const int64_t nvec = n / 8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    const uint4 raw = ld_stream16(grad + i * 8);
    float f[8];
    unpack8<T>(raw, f);
#pragma unroll
    for (int k = 0; k < 8; ++k) bad |= !isfinite(f[k]);
  }
  for (int64_t i = nvec * 8 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    bad |= !isfinite(Num<T>::to_f(grad[i]));
  if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicExch(found_inf, 1);
}

// Scalars worked out on the host in double and rounded once, as torch does with its Python floats.
struct AdamArgs {
  double lr, beta1, beta2d;  // enter the bias corrections, which are evaluated in double
  float beta2, eps;
  float decay;    // 1 - lr * weight_decay
  float om_beta1; // 1 - beta1
  float om_beta2; // 1 - beta2
};

__device__ __forceinline__ void adamw_one(float g, float& w, float& m, float& v, const AdamArgs& a, float step_size,
                                          float bc2_sqrt) {
  // the forms a CPU run of torch.optim.AdamW takes (found by comparing bit patterns over several steps): the
  // lerp of the first moment and the addcmul of the second are fused multiply-adds, the addcdiv is
  // value * exp_avg / denom with the product first
  w = __fmul_rn(w, a.decay);
  m = __fmaf_rn(a.om_beta1, __fsub_rn(g, m), m);
  v = __fmaf_rn(__fmul_rn(a.om_beta2, g), g, __fmul_rn(v, a.beta2));
  const float denom = __fadd_rn(__fdiv_rn(__fsqrt_rn(v), bc2_sqrt), a.eps);
  w = __fadd_rn(w, __fdiv_rn(__fmul_rn(-step_size, m), denom));
}

template <typename T>
__global__ void __launch_bounds__(256) adamw_step_kernel(const T* __restrict__ grad, T* __restrict__ param,
                                                         float* __restrict__ master, float* __restrict__ m_,
                                                         float* __restrict__ v_, int64_t n,
                                                         const float* __restrict__ inv_scale,
                                                         const int* __restrict__ found_inf,
                                                         const float* __restrict__ steps_taken, AdamArgs a) {
  grid_dependency_wait();
  allow_dependents();
  if (found_inf && *found_inf) return;  // the whole step is skipped
  const float unscale = inv_scale ? *inv_scale : 1.f;
  const double t = (double)(steps_taken ? *steps_taken : 0.f) + 1.0;
  const float step_size = (float)(a.lr / (1.0 - pow(a.beta1, t)));
  const float bc2_sqrt = (float)sqrt(1.0 - pow(a.beta2d, t));
  const int64_t nvec = n / 8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    const uint4 raw = ld_stream16(grad + i * 8);
    float g[8], w[8], m[8], v[8];
    unpack8<T>(raw, g);
    *reinterpret_cast<float4*>(w) = *reinterpret_cast<const float4*>(master + i * 8);
    *reinterpret_cast<float4*>(w + 4) = *reinterpret_cast<const float4*>(master + i * 8 + 4);
    *reinterpret_cast<float4*>(m) = *reinterpret_cast<const float4*>(m_ + i * 8);
    *reinterpret_cast<float4*>(m + 4) = *reinterpret_cast<const float4*>(m_ + i * 8 + 4);
    *reinterpret_cast<float4*>(v) = *reinterpret_cast<const float4*>(v_ + i * 8);
    *reinterpret_cast<float4*>(v + 4) = *reinterpret_cast<const float4*>(v_ + i * 8 + 4);
#pragma unroll
    for (int k = 0; k < 8; ++k) adamw_one(g[k] * unscale, w[k], m[k], v[k], a, step_size, bc2_sqrt);
    *reinterpret_cast<float4*>(master + i * 8) = *reinterpret_cast<const float4*>(w);
    *reinterpret_cast<float4*>(master + i * 8 + 4) = *reinterpret_cast<const float4*>(w + 4);
    *reinterpret_cast<float4*>(m_ + i * 8) = *reinterpret_cast<const float4*>(m);
    *reinterpret_cast<float4*>(m_ + i * 8 + 4) = *reinterpret_cast<const float4*>(m + 4);
    *reinterpret_cast<float4*>(v_ + i * 8) = *reinterpret_cast<const float4*>(v);
    *reinterpret_cast<float4*>(v_ + i * 8 + 4) = *reinterpret_cast<const float4*>(v + 4);
    *reinterpret_cast<uint4*>(param + i * 8) = pack8<T>(w);
  }
  for (int64_t i = nvec * 8 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float w = master[i], m = m_[i], v = v_[i];
    adamw_one(Num<T>::to_f(grad[i]) * unscale, w, m, v, a, step_size, bc2_sqrt);
    master[i] = w;
    m_[i] = m;
    v_[i] = v;
    param[i] = Num<T>::from_f(w);
  }
}

// state[0] = loss scale, state[1] = 1 / scale, state[2] = good steps since the last change of the scale,
// state[3] = optimizer steps taken
__global__ void scale_update_kernel(float* __restrict__ state, int* __restrict__ found_inf, float growth, float backoff,
                                    int interval) {
  grid_dependency_wait();
  allow_dependents();
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  if (*found_inf) {
    state[0] *= backoff;
    state[2] = 0.f;
  } else {
    state[3] += 1.f;
    const float good = state[2] + 1.f;
    if (good >= (float)interval) {
      state[0] *= growth;
      state[2] = 0.f;
    } else {
      state[2] = good;
    }
  }
  state[1] = 1.f / state[0];
  *found_inf = 0;
}

static unsigned flat_grid(int64_t n) {
  const int64_t want = ceil_div(ceil_div(n, 8), 256);
  const int64_t cap = (int64_t)sm_count() * 8;
  return (unsigned)(want < cap ? (want > 0 ? want : 1) : cap);
}

}  // namespace tfb

using namespace tfb;

extern "C" int tfb_grad_check(const void* grad, int64_t n, int dtype, int* found_inf, void* stream) {
  TFB_REQUIRE(n >= 0 && found_inf != nullptr, "grad_check: bad arguments");
  if (n == 0) return TFB_OK;
  TFB_REQUIRE(grad != nullptr && aligned16(grad), "grad_check: the gradient buffer must be 16-byte aligned");
  TFB_DISPATCH_16(dtype, T, {
    launch_overlapped(grad_check_kernel<T>, dim3(flat_grid(n)), dim3(256), 0, (cudaStream_t)stream, (const T*)grad, n,
                      found_inf);
  })
  return launched("grad_check");
}

extern "C" int tfb_adamw_step(const void* grad, void* param, float* master, float* exp_avg, float* exp_avg_sq,
                              int64_t n, int dtype, const float* inv_scale, const int* found_inf,
                              const float* steps_taken, double lr, double beta1, double beta2, double eps,
                              double weight_decay, void* stream) {
  TFB_REQUIRE(n >= 0, "adamw_step: negative size");
  if (n == 0) return TFB_OK;
  TFB_REQUIRE(grad && param && master && exp_avg && exp_avg_sq, "adamw_step: null buffer");
  TFB_REQUIRE(aligned16(grad) && aligned16(param) && aligned16(master) && aligned16(exp_avg) && aligned16(exp_avg_sq),
              "adamw_step: buffers must be 16-byte aligned");
  TFB_REQUIRE(lr >= 0.0 && beta1 >= 0.0 && beta1 < 1.0 && beta2 >= 0.0 && beta2 < 1.0 && eps >= 0.0,
              "adamw_step: bad hyper-parameter");
  TFB_REQUIRE(1.0 - beta1 < 0.5, "adamw_step: beta1 must exceed 0.5 (the first-moment update is written for that case)");
  // hyper-parameters arrive as doubles (Python floats) and every derived scalar is rounded to fp32 once
  AdamArgs a{lr, beta1, beta2, (float)beta2, (float)eps, (float)(1.0 - lr * weight_decay), (float)(1.0 - beta1),
             (float)(1.0 - beta2)};
  TFB_DISPATCH_16(dtype, T, {
    launch_overlapped(adamw_step_kernel<T>, dim3(flat_grid(n)), dim3(256), 0, (cudaStream_t)stream, (const T*)grad,
                      (T*)param, master, exp_avg, exp_avg_sq, n, inv_scale, found_inf, steps_taken, a);
  })
  return launched("adamw_step");
}

extern "C" int tfb_loss_scale_update(float* state4, int* found_inf, float growth, float backoff, int interval,
                                     void* stream) {
  TFB_REQUIRE(state4 != nullptr && found_inf != nullptr, "loss_scale_update: null state");
  TFB_REQUIRE(growth >= 1.f && backoff > 0.f && backoff <= 1.f && interval > 0, "loss_scale_update: bad factors");
  launch_overlapped(scale_update_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, state4, found_inf, growth, backoff,
                    interval);
  return launched("loss_scale_update");
}
