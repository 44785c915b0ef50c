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


// delta[b,h,i] = sum_d dO[i,d] * O[i,d] (fp32), shared by both backward paths
int attn_delta(const AttnArgs& a, int hd, int dtype, cudaStream_t st);
int attn_generic_fwd(const AttnArgs& a, int hd, int dtype, cudaStream_t st);
int attn_generic_bwd(const AttnArgs& a, int hd, int dtype, cudaStream_t st);

}  // namespace tfb
