// Argument block shared by the attention kernels and their entry points.
#pragma once
#include "common.cuh"

namespace tfb {

struct AttnStrides { int64_t b, h, t; };

struct AttnArgs {
  const void *q, *k, *v, *o, *d_o;
  void *out, *dq, *dk, *dv;
  float* lse;          // (B,H,T) natural log-sum-exp
  float* delta;        // (B,H,T)
  float* dq_acc;       // (B,H,T,hd) fp32 accumulator of the tcgen05 backward
  AttnStrides sq, sk, sv, so, sdo, sdq, sdk, sdv;
  int B, H, T;
  float scale;         // 1/sqrt(hd)
  int bias_mode;       // 0 none, 1 ALiBi fp32, 2 / 4 ALiBi rounded like an fp16 / bf16 reference table, 3 dense table
  const float* slopes;
  const void* bias;
  int64_t bias_sh, bias_si;
};


// The tcgen05 kernels order their CTAs longest walk first ACROSS batch*head slices.  The slices walked
// together keep their K and V (forward) or Q, K, V, dO (backward) live in the L2 at the same time; this
// is how many slices share 64 MB at four 16-bit tensors each, in groups of equal size.
inline int attn_slices_per_group(int bh, int T, int hd) {
  const int64_t per_slice = (int64_t)4 * T * hd * 2;
  int64_t g = (64ll << 20) / per_slice;
  if (g < 1) g = 1;
  if (g >= bh) return bh;
  const int64_t groups = (bh + g - 1) / g;
  return (int)((bh + groups - 1) / groups);
}

// delta[b,h,i] = sum_d dO[i,d] * O[i,d] (fp32), shared by both backward paths
// `clear`: optional fp32 (B,H,T,hd) buffer that the same pass sets to zero (the dQ accumulator).
int attn_delta(const AttnArgs& a, int hd, int dtype, cudaStream_t st, float* clear = nullptr);
int attn_generic_fwd(const AttnArgs& a, int hd, int dtype, cudaStream_t st);
int attn_generic_bwd(const AttnArgs& a, int hd, int dtype, cudaStream_t st);

// ALiBi bias -(i - j) * slope as the reference's 16-bit table holds it (mode 2: fp16, mode 4: bf16):
// distance, slope and product each rounded to nearest-even at 11 or 8 significant bits; mode 1: exact
// fp32.  The rounding is integer arithmetic on the ALU pipe rather than three conversions per score on
// the pipe the exponentials need.  Exact while the values stay in the 16-bit type's normal range
// (slopes >= 2^-8 times distances below 2^23 do).
__device__ __forceinline__ float round_significand(float x, int drop) {  // drop the low `drop` mantissa bits
  uint32_t t = __float_as_uint(x);
  t += ((1u << (drop - 1)) - 1u) + ((t >> drop) & 1u);
  return __uint_as_float(t & ~((1u << drop) - 1u));
}
__device__ __forceinline__ float alibi_table_value(int mode, float slope, int dist) {
  const float d = __uint_as_float(0x4B000000u | (uint32_t)dist) - 8388608.f;  // exact int -> float
  if (mode == 1) return -slope * d;
  const int drop = (mode == 2) ? 13 : 16;
  const float s16 = (mode == 2) ? __half2float(__float2half_rn(slope)) : __bfloat162float(__float2bfloat16_rn(slope));
  return -round_significand(round_significand(d, drop) * s16, drop);
}

// The same penalty for the tcgen05 kernels, in log2 units, with the mode a compile-time constant (0 none, 1 exact
// fp32, 2 / 4 rounded like an fp16 / bf16 table) and everything that depends only on the head worked out once:
// with the mode a run-time value the compiler evaluated both forms for every score, and the 16-bit rounding of
// the slope - a conversion on the pipe the exponentials need - ran once per score as well.
template <int MODE>
struct AlibiLog2 {
  float k;  // MODE 1: slope * log2(e); MODE 2 / 4: the slope rounded to the table's type
  static constexpr int DROP = (MODE == 2) ? 13 : 16;
  __device__ __forceinline__ explicit AlibiLog2(float slope) {
    k = (MODE == 1) ? slope * 1.4426950408889634f
                    : (MODE == 2 ? __half2float(__float2half_rn(slope))
                                 : (MODE == 4 ? __bfloat162float(__float2bfloat16_rn(slope)) : 0.f));
  }
  static __device__ __forceinline__ float round_sig(float x) {
    uint32_t t = __float_as_uint(x);
    t += ((1u << (DROP - 1)) - 1u) + ((t >> DROP) & 1u);
    return __uint_as_float(t & ~((1u << DROP) - 1u));
  }
  // x - penalty(distance d), d >= 0 given as an exactly converted float
  __device__ __forceinline__ float sub_from(float x, float d) const {
    if (MODE == 0) return x;
    if (MODE == 1) return fmaf(-k, d, x);
    return fmaf(-round_sig(round_sig(d) * k), 1.4426950408889634f, x);
  }
};

}  // namespace tfb
