// Shared host/device helpers for the tritonformer_b200 kernel library (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <atomic>

#include "../../include/tritonformer_b200.h"

namespace tfb {

// ---- host-side error plumbing -------------------------------------------------------
extern thread_local char g_err[512];
extern std::atomic<int64_t> g_launches;

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

// Call after a <<<>>> launch: counts it and converts a launch error into a status.
inline int launched(const char* what) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(TFB_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
  return TFB_OK;
}

// Raises a kernel's dynamic shared-memory limit once per device (the attribute is per device; `done`
// holds one bit per device ordinal).  Idempotent, so a race between two threads is harmless.
template <typename F>
inline int ensure_dynamic_smem(F func, int bytes, std::atomic<uint64_t>& done, const char* what) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  const uint64_t bit = 1ull << dev;
  if (done.load(std::memory_order_acquire) & bit) return TFB_OK;
  cudaError_t e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return fail(TFB_ERR_LAUNCH, "%s: shared-memory attribute: %s", what, cudaGetErrorString(e));
  done.fetch_or(bit, std::memory_order_release);
  return TFB_OK;
}

// ---- programmatic dependent launch ----------------------------------------------------
// Kernels launched through launch_overlapped() may become resident while the previous kernel of
// the stream is still draining: their set-up (barrier init, TMEM allocation, tensor-map prefetch)
// overlaps its tail.  Every such kernel calls grid_dependency_wait() before its first access to
// global memory (the wait returns once the previous grid has completed and its writes are visible)
// and then allow_dependents(), which lets the following kernel do the same with respect to it.
// A kernel launched the plain way treats both calls as no-ops.  tfb_debug_set(3, 1) turns the
// launch attribute off.
extern std::atomic<int> g_plain_launch;

template <typename... KArgs, typename... Args>
inline void launch_overlapped(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_plain_launch.load(std::memory_order_relaxed) ? 0 : 1;
  (void)cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);  // error read by launched()
}

#ifdef __CUDACC__
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void allow_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

#define TFB_REQUIRE(cond, ...)                         \
  do {                                                 \
    if (!(cond)) return ::tfb::fail(TFB_ERR_ARG, __VA_ARGS__); \
  } while (0)

// SMs of the device the library first ran on (every GPU of a node is the same part).
inline int sm_count() {
  static int n = []() {
    int dev = 0, v = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v > 0 ? v : 148;
  }();
  return n;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- device-side numeric helpers ------------------------------------------------------
template <typename T> struct Num;
template <> struct Num<__half> {
  using T2 = __half2;
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
  static __device__ __forceinline__ float2 to_f2(__half2 v) { return __half22float2(v); }
  static __device__ __forceinline__ __half2 from_f2(float a, float b) { return __floats2half2_rn(a, b); }
};
template <> struct Num<__nv_bfloat16> {
  using T2 = __nv_bfloat162;
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float2 to_f2(__nv_bfloat162 v) { return __bfloat1622float2(v); }
  static __device__ __forceinline__ __nv_bfloat162 from_f2(float a, float b) { return __floats2bfloat162_rn(a, b); }
};
template <> struct Num<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};

// 16-byte vector of 8 sixteen-bit values, unpacked to / packed from fp32.
template <typename T>
__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
  using T2 = typename Num<T>::T2;
  const T2* p = reinterpret_cast<const T2*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = Num<T>::to_f2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  using T2 = typename Num<T>::T2;
  uint4 raw;
  T2* p = reinterpret_cast<T2*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = Num<T>::from_f2(f[2 * i], f[2 * i + 1]);
  return raw;
}

// Two fp32 values in one 64-bit register pair and the packed fused multiply-add that works on both (sm_100): one
// issue slot for two FMAs.
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Streaming (evict-first) 16-byte global accesses for data touched once.
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 r;
  asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}
__device__ __forceinline__ void st_stream16(void* p, const uint4& v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// Dispatch a 16-bit dtype code to a template instantiation.
#define TFB_DISPATCH_16(dtype, T, ...)                                   \
  if ((dtype) == TFB_F16) { using T = __half; __VA_ARGS__ }              \
  else if ((dtype) == TFB_BF16) { using T = __nv_bfloat16; __VA_ARGS__ } \
  else return ::tfb::fail(TFB_ERR_ARG, "dtype %d: expected fp16 or bf16", (int)(dtype));

}  // namespace tfb
