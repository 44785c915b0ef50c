// Causal flash attention forward / backward on mma.sync tensor cores, any {b,h,t} strides.
// This is the kernel family for head sizes and bias forms the tcgen05 kernels do not take
// (head_dim 32, dense bias tables) and the cross-check for them in the tests.
//
// 64-row tiles, 4 warps of 16 rows.  Scores live in the log2 domain:
//   s2(i,j) = (q_i . k_j) * scale * log2e + bias(i,j) * log2e,  p = 2^(s2 - lse2)
// Forward keeps a running (max, sum) per row (FA2 style: one division at the end) and
// stores the natural log-sum-exp.  Backward is two kernels without atomics: one CTA per
// key/value tile for dK, dV and one CTA per query tile for dQ; delta = rowsum(dO*O) comes
// from a small pre-pass.
#include "attn.cuh"
#include <type_traits>

namespace tfb {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr int AT = 64;         // tile rows (queries) and columns (keys)
constexpr int AT_THREADS = 128;

template <typename T> struct Mma16816;
template <> struct Mma16816<__half> {
  static __device__ __forceinline__ void run(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ uint32_t pack(float x, float y) {
    __half2 h = __floats2half2_rn(x, y);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) { return __half22float2(*reinterpret_cast<__half2*>(&u)); }
};
template <> struct Mma16816<__nv_bfloat16> {
  static __device__ __forceinline__ void run(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ uint32_t pack(float x, float y) {
    __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
  }
};

// additive bias (natural units) for query i, key j (j <= i)
// modes 2 / 4 rebuild the reference ALiBi table entry: the (negative) distance and the slope are
// rounded to fp16 (2) or bf16 (4) and multiplied in that type.
template <typename T>
__device__ __forceinline__ float bias_at(int mode, float slope, const T* table_h, int64_t si, int i, int j) {
  if (mode == 1) return -slope * (float)(i - j);
  if (mode == 2) return __half2float(__hmul(__float2half_rn(-(float)(i - j)), __float2half_rn(slope)));
  if (mode == 4) return __bfloat162float(__hmul(__float2bfloat16_rn(-(float)(i - j)), __float2bfloat16_rn(slope)));
  if (mode == 3) return Num<T>::to_f(table_h[(int64_t)i * si + j]);
  return 0.f;
}

// 64 x HD tile, row-major in smem with pitch HD+8
template <typename T, int HD>
__device__ __forceinline__ void load_rows(T (*dst)[HD + 8], const T* src, int64_t row_stride) {
  constexpr int VPR = HD / 8;
#pragma unroll
  for (int i = 0; i < AT * VPR / AT_THREADS; ++i) {
    const int idx = threadIdx.x + i * AT_THREADS;
    const int r = idx / VPR, c = idx % VPR;
    *reinterpret_cast<uint4*>(&dst[r][c * 8]) = *reinterpret_cast<const uint4*>(src + (int64_t)r * row_stride + c * 8);
  }
}
// the same tile transposed: dst[HD][64+8]
template <typename T, int HD>
__device__ __forceinline__ void load_transposed(T (*dst)[AT + 8], const T* src, int64_t row_stride) {
  constexpr int VPR = HD / 8;
#pragma unroll
  for (int i = 0; i < AT * VPR / AT_THREADS; ++i) {
    const int idx = threadIdx.x + i * AT_THREADS;
    const int r = idx % AT, c = idx / AT;  // consecutive threads -> consecutive rows: conflict-free stores
    const uint4 raw = *reinterpret_cast<const uint4*>(src + (int64_t)r * row_stride + c * 8);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int j = 0; j < 8; ++j) dst[c * 8 + j][r] = e[j];
  }
}

template <typename T, int P>
__device__ __forceinline__ void frag_a(uint32_t (&a)[4], const T (*x)[P], int r0, int k0, int g, int t) {
  a[0] = *reinterpret_cast<const uint32_t*>(&x[r0 + g][k0 + 2 * t]);
  a[1] = *reinterpret_cast<const uint32_t*>(&x[r0 + g + 8][k0 + 2 * t]);
  a[2] = *reinterpret_cast<const uint32_t*>(&x[r0 + g][k0 + 2 * t + 8]);
  a[3] = *reinterpret_cast<const uint32_t*>(&x[r0 + g + 8][k0 + 2 * t + 8]);
}
template <typename T, int P>
__device__ __forceinline__ void frag_b(uint32_t& b0, uint32_t& b1, const T (*y)[P], int n0, int k0, int g, int t) {
  b0 = *reinterpret_cast<const uint32_t*>(&y[n0 + g][k0 + 2 * t]);
  b1 = *reinterpret_cast<const uint32_t*>(&y[n0 + g][k0 + 2 * t + 8]);
}

// ----------------------------------------------------------------------------------- forward
template <typename T, int HD>
__global__ void __launch_bounds__(AT_THREADS) attn_fwd_kernel(const AttnArgs a) {
  __shared__ __align__(16) T Ks[AT][HD + 8];   // also stages Q once
  __shared__ __align__(16) T Vt[HD][AT + 8];
  using M = Mma16816<T>;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int qt = gridDim.x - 1 - blockIdx.x;  // heaviest tiles first
  const int bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const int q0 = qt * AT;
  const T* qp = (const T*)a.q + b * a.sq.b + h * a.sq.h + (int64_t)q0 * a.sq.t;
  const T* kp = (const T*)a.k + b * a.sk.b + h * a.sk.h;
  const T* vp = (const T*)a.v + b * a.sv.b + h * a.sv.h;
  const float slope = (a.bias_mode != 0 && a.bias_mode != 3) ? a.slopes[h] : 0.f;
  const T* table_h = a.bias_mode == 3 ? (const T*)a.bias + h * a.bias_sh : nullptr;
  const float c2 = a.scale * kLog2e;

  load_rows<T, HD>(Ks, qp, a.sq.t);
  __syncthreads();
  uint32_t qf[HD / 16][4];
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks) frag_a<T, HD + 8>(qf[ks], Ks, warp * 16, ks * 16, g, t);
  __syncthreads();

  float o[HD / 8][4];
#pragma unroll
  for (int n = 0; n < HD / 8; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int row0 = q0 + warp * 16 + g;  // rows row0 and row0+8

  for (int j0 = 0; j0 <= q0; j0 += AT) {
    load_rows<T, HD>(Ks, kp + (int64_t)j0 * a.sk.t, a.sk.t);
    load_transposed<T, HD>(Vt, vp + (int64_t)j0 * a.sv.t, a.sv.t);
    __syncthreads();
    float s[AT / 8][4];
#pragma unroll
    for (int n = 0; n < AT / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        uint32_t b0, b1;
        frag_b<T, HD + 8>(b0, b1, Ks, n * 8, ks * 16, g, t);
        M::run(s[n], qf[ks], b0, b1);
      }
    }
    const bool diag = (j0 == q0);
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < AT / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = row0 + ((e >> 1) ? 8 : 0);
        const int j = j0 + n * 8 + 2 * t + (e & 1);
        float v = s[n][e] * c2;
        if (a.bias_mode && j <= i) v += bias_at<T>(a.bias_mode, slope, table_h, a.bias_si, i, j) * kLog2e;
        if (diag && j > i) v = -INFINITY;
        s[n][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float mn = fmaxf(m_run[r], mx[r]);  // finite: column j0 <= i is never masked
      corr[r] = exp2f(m_run[r] - mn);
      m_run[r] = mn;
      l_run[r] *= corr[r];
    }
    float ls[2] = {0.f, 0.f};
#pragma unroll
    for (int n = 0; n < AT / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = exp2f(s[n][e] - m_run[e >> 1]);
        s[n][e] = p;
        ls[e >> 1] += p;
      }
    }
    l_run[0] += ls[0];
    l_run[1] += ls[1];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
      o[n][0] *= corr[0]; o[n][1] *= corr[0];
      o[n][2] *= corr[1]; o[n][3] *= corr[1];
    }
#pragma unroll
    for (int ks = 0; ks < AT / 16; ++ks) {
      uint32_t pf[4];
      pf[0] = M::pack(s[2 * ks][0], s[2 * ks][1]);
      pf[1] = M::pack(s[2 * ks][2], s[2 * ks][3]);
      pf[2] = M::pack(s[2 * ks + 1][0], s[2 * ks + 1][1]);
      pf[3] = M::pack(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
      for (int n = 0; n < HD / 8; ++n) {
        uint32_t b0, b1;
        frag_b<T, AT + 8>(b0, b1, Vt, n * 8, ks * 16, g, t);
        M::run(o[n], pf, b0, b1);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  T* op = (T*)a.out + b * a.so.b + h * a.so.h;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int i = row0 + r * 8;
    const float inv = 1.f / l_run[r];
    T* orow = op + (int64_t)i * a.so.t;
#pragma unroll
    for (int n = 0; n < HD / 8; ++n)
      *reinterpret_cast<uint32_t*>(orow + n * 8 + 2 * t) = M::pack(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
    if (t == 0) a.lse[((int64_t)bh) * a.T + i] = (m_run[r] + log2f(l_run[r])) * kLn2;
  }
}

// delta[b,h,i] = sum_d dO[i,d] * O[i,d]; hd/8 lanes per row, one 16-byte load of each operand per lane.
// `clear` (may be null): contiguous fp32 (B,H,T,HD) buffer; each lane zeroes the eight floats under its chunk.
template <typename T, int HD>
__global__ void __launch_bounds__(256) attn_delta_kernel(const AttnArgs a, float* __restrict__ clear) {
  grid_dependency_wait();
  allow_dependents();
  constexpr int LPR = HD / 8;          // lanes per row
  constexpr int RPW = 32 / LPR;        // rows per warp
  const int lane = threadIdx.x & 31;
  const int sub = lane % LPR;
  const int64_t row = ((int64_t)blockIdx.x * 8 + (threadIdx.x >> 5)) * RPW + lane / LPR;
  const int64_t total = (int64_t)a.B * a.H * a.T;
  float s = 0.f;
  if (row < total) {
    const int i = (int)(row % a.T);
    const int64_t bh = row / a.T;
    const int b = (int)(bh / a.H), h = (int)(bh % a.H);
    const T* op = (const T*)a.o + b * a.so.b + h * a.so.h + (int64_t)i * a.so.t + sub * 8;
    const T* gp = (const T*)a.d_o + b * a.sdo.b + h * a.sdo.h + (int64_t)i * a.sdo.t + sub * 8;
    float x[8], y[8];
    unpack8<T>(ld_stream16(op), x);
    unpack8<T>(ld_stream16(gp), y);
#pragma unroll
    for (int j = 0; j < 8; ++j) s += x[j] * y[j];
    if (clear) {
      float4* z = reinterpret_cast<float4*>(clear + row * HD + sub * 8);
      z[0] = make_float4(0.f, 0.f, 0.f, 0.f);
      z[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (row < total && sub == 0) a.delta[row] = s;
}

// --------------------------------------------------------------------------- backward: dK, dV
template <typename T, int HD>
struct BwdKvSmem {
  T Ks[AT][HD + 8], Vs[AT][HD + 8], Qs[AT][HD + 8], Gs[AT][HD + 8];
  T Qt[HD][AT + 8], Gt[HD][AT + 8];
  float lse2[AT], delta[AT];
};

template <typename T, int HD>
__global__ void __launch_bounds__(AT_THREADS) attn_bwd_kv_kernel(const AttnArgs a) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  BwdKvSmem<T, HD>& sm = *reinterpret_cast<BwdKvSmem<T, HD>*>(smem_raw);
  using M = Mma16816<T>;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int kt = blockIdx.x;  // tile 0 has the most query tiles to visit
  const int bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const int j0 = kt * AT;
  const T* qp = (const T*)a.q + b * a.sq.b + h * a.sq.h;
  const T* gp = (const T*)a.d_o + b * a.sdo.b + h * a.sdo.h;
  const float slope = (a.bias_mode != 0 && a.bias_mode != 3) ? a.slopes[h] : 0.f;
  const T* table_h = a.bias_mode == 3 ? (const T*)a.bias + h * a.bias_sh : nullptr;
  const float c2 = a.scale * kLog2e;

  load_rows<T, HD>(sm.Ks, (const T*)a.k + b * a.sk.b + h * a.sk.h + (int64_t)j0 * a.sk.t, a.sk.t);
  load_rows<T, HD>(sm.Vs, (const T*)a.v + b * a.sv.b + h * a.sv.h + (int64_t)j0 * a.sv.t, a.sv.t);

  float dk[HD / 8][4], dv[HD / 8][4];
#pragma unroll
  for (int n = 0; n < HD / 8; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) dk[n][e] = dv[n][e] = 0.f;
  const int jrow = j0 + warp * 16 + g;  // key rows jrow, jrow+8

  for (int i0 = j0; i0 < a.T; i0 += AT) {
    __syncthreads();  // previous iteration done with the query-side tiles
    load_rows<T, HD>(sm.Qs, qp + (int64_t)i0 * a.sq.t, a.sq.t);
    load_rows<T, HD>(sm.Gs, gp + (int64_t)i0 * a.sdo.t, a.sdo.t);
    load_transposed<T, HD>(sm.Qt, qp + (int64_t)i0 * a.sq.t, a.sq.t);
    load_transposed<T, HD>(sm.Gt, gp + (int64_t)i0 * a.sdo.t, a.sdo.t);
    if (threadIdx.x < AT) {
      sm.lse2[threadIdx.x] = a.lse[(int64_t)bh * a.T + i0 + threadIdx.x] * kLog2e;
      sm.delta[threadIdx.x] = a.delta[(int64_t)bh * a.T + i0 + threadIdx.x];
    }
    __syncthreads();
    // S^T (16 keys x 64 queries) = K Q^T
    float s[AT / 8][4];
#pragma unroll
    for (int n = 0; n < AT / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      uint32_t af[4];
      frag_a<T, HD + 8>(af, sm.Ks, warp * 16, ks * 16, g, t);
#pragma unroll
      for (int n = 0; n < AT / 8; ++n) {
        uint32_t b0, b1;
        frag_b<T, HD + 8>(b0, b1, sm.Qs, n * 8, ks * 16, g, t);
        M::run(s[n], af, b0, b1);
      }
    }
    const bool diag = (i0 == j0);
    uint32_t pf[AT / 16][4];  // P^T as A fragments (rounded to the element type)
#pragma unroll
    for (int n = 0; n < AT / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = jrow + ((e >> 1) ? 8 : 0);
        const int il = n * 8 + 2 * t + (e & 1);
        const int i = i0 + il;
        float v = s[n][e] * c2;
        if (a.bias_mode && j <= i) v += bias_at<T>(a.bias_mode, slope, table_h, a.bias_si, i, j) * kLog2e;
        float p = exp2f(v - sm.lse2[il]);
        if (diag && j > i) p = 0.f;
        s[n][e] = p;
      }
    }
#pragma unroll
    for (int ks = 0; ks < AT / 16; ++ks) {
      pf[ks][0] = M::pack(s[2 * ks][0], s[2 * ks][1]);
      pf[ks][1] = M::pack(s[2 * ks][2], s[2 * ks][3]);
      pf[ks][2] = M::pack(s[2 * ks + 1][0], s[2 * ks + 1][1]);
      pf[ks][3] = M::pack(s[2 * ks + 1][2], s[2 * ks + 1][3]);
    }
    // dV += P^T dO
#pragma unroll
    for (int ks = 0; ks < AT / 16; ++ks) {
#pragma unroll
      for (int n = 0; n < HD / 8; ++n) {
        uint32_t b0, b1;
        frag_b<T, AT + 8>(b0, b1, sm.Gt, n * 8, ks * 16, g, t);
        M::run(dv[n], pf[ks], b0, b1);
      }
    }
    // dP^T = V dO^T
#pragma unroll
    for (int n = 0; n < AT / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      uint32_t af[4];
      frag_a<T, HD + 8>(af, sm.Vs, warp * 16, ks * 16, g, t);
#pragma unroll
      for (int n = 0; n < AT / 8; ++n) {
        uint32_t b0, b1;
        frag_b<T, HD + 8>(b0, b1, sm.Gs, n * 8, ks * 16, g, t);
        M::run(s[n], af, b0, b1);
      }
    }
    // dS^T = P^T * (dP^T - delta), reusing pf
#pragma unroll
    for (int ks = 0; ks < AT / 16; ++ks) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int n = 2 * ks + half;
        const float d0 = sm.delta[n * 8 + 2 * t], d1 = sm.delta[n * 8 + 2 * t + 1];
        const float2 p01 = M::unpack(pf[ks][2 * half]);      // row g
        const float2 p23 = M::unpack(pf[ks][2 * half + 1]);  // row g+8
        pf[ks][2 * half] = M::pack(p01.x * (s[n][0] - d0), p01.y * (s[n][1] - d1));
        pf[ks][2 * half + 1] = M::pack(p23.x * (s[n][2] - d0), p23.y * (s[n][3] - d1));
      }
    }
    // dK += dS^T Q
#pragma unroll
    for (int ks = 0; ks < AT / 16; ++ks) {
#pragma unroll
      for (int n = 0; n < HD / 8; ++n) {
        uint32_t b0, b1;
        frag_b<T, AT + 8>(b0, b1, sm.Qt, n * 8, ks * 16, g, t);
        M::run(dk[n], pf[ks], b0, b1);
      }
    }
  }
  T* dkp = (T*)a.dk + b * a.sdk.b + h * a.sdk.h;
  T* dvp = (T*)a.dv + b * a.sdv.b + h * a.sdv.h;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int j = jrow + r * 8;
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
      *reinterpret_cast<uint32_t*>(dkp + (int64_t)j * a.sdk.t + n * 8 + 2 * t) =
          M::pack(dk[n][2 * r] * a.scale, dk[n][2 * r + 1] * a.scale);
      *reinterpret_cast<uint32_t*>(dvp + (int64_t)j * a.sdv.t + n * 8 + 2 * t) =
          M::pack(dv[n][2 * r], dv[n][2 * r + 1]);
    }
  }
}

// -------------------------------------------------------------------------------- backward: dQ
template <typename T, int HD>
struct BwdQSmem {
  T Qs[AT][HD + 8], Gs[AT][HD + 8], Ks[AT][HD + 8], Vs[AT][HD + 8];
  T Kt[HD][AT + 8];
};

template <typename T, int HD>
__global__ void __launch_bounds__(AT_THREADS) attn_bwd_q_kernel(const AttnArgs a) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  BwdQSmem<T, HD>& sm = *reinterpret_cast<BwdQSmem<T, HD>*>(smem_raw);
  using M = Mma16816<T>;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const int i0 = qt * AT;
  const T* kp = (const T*)a.k + b * a.sk.b + h * a.sk.h;
  const T* vp = (const T*)a.v + b * a.sv.b + h * a.sv.h;
  const float slope = (a.bias_mode != 0 && a.bias_mode != 3) ? a.slopes[h] : 0.f;
  const T* table_h = a.bias_mode == 3 ? (const T*)a.bias + h * a.bias_sh : nullptr;
  const float c2 = a.scale * kLog2e;

  load_rows<T, HD>(sm.Qs, (const T*)a.q + b * a.sq.b + h * a.sq.h + (int64_t)i0 * a.sq.t, a.sq.t);
  load_rows<T, HD>(sm.Gs, (const T*)a.d_o + b * a.sdo.b + h * a.sdo.h + (int64_t)i0 * a.sdo.t, a.sdo.t);
  const int irow = i0 + warp * 16 + g;
  float lse2[2], dl[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    lse2[r] = a.lse[(int64_t)bh * a.T + irow + r * 8] * kLog2e;
    dl[r] = a.delta[(int64_t)bh * a.T + irow + r * 8];
  }
  float dq[HD / 8][4];
#pragma unroll
  for (int n = 0; n < HD / 8; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) dq[n][e] = 0.f;

  for (int j0 = 0; j0 <= i0; j0 += AT) {
    __syncthreads();
    load_rows<T, HD>(sm.Ks, kp + (int64_t)j0 * a.sk.t, a.sk.t);
    load_rows<T, HD>(sm.Vs, vp + (int64_t)j0 * a.sv.t, a.sv.t);
    load_transposed<T, HD>(sm.Kt, kp + (int64_t)j0 * a.sk.t, a.sk.t);
    __syncthreads();
    float s[AT / 8][4], dp[AT / 8][4];
#pragma unroll
    for (int n = 0; n < AT / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[n][e] = dp[n][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      uint32_t aq[4], ag[4];
      frag_a<T, HD + 8>(aq, sm.Qs, warp * 16, ks * 16, g, t);
      frag_a<T, HD + 8>(ag, sm.Gs, warp * 16, ks * 16, g, t);
#pragma unroll
      for (int n = 0; n < AT / 8; ++n) {
        uint32_t b0, b1;
        frag_b<T, HD + 8>(b0, b1, sm.Ks, n * 8, ks * 16, g, t);
        M::run(s[n], aq, b0, b1);
        frag_b<T, HD + 8>(b0, b1, sm.Vs, n * 8, ks * 16, g, t);
        M::run(dp[n], ag, b0, b1);
      }
    }
    const bool diag = (j0 == i0);
#pragma unroll
    for (int n = 0; n < AT / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;
        const int i = irow + r * 8;
        const int j = j0 + n * 8 + 2 * t + (e & 1);
        float v = s[n][e] * c2;
        if (a.bias_mode && j <= i) v += bias_at<T>(a.bias_mode, slope, table_h, a.bias_si, i, j) * kLog2e;
        float p = exp2f(v - lse2[r]);
        if (diag && j > i) p = 0.f;
        // P is rounded to the element type before it meets dP, as in the dK/dV kernel
        const float pr = M::unpack(M::pack(p, 0.f)).x;
        s[n][e] = pr * (dp[n][e] - dl[r]);
      }
    }
#pragma unroll
    for (int ks = 0; ks < AT / 16; ++ks) {
      uint32_t df[4];
      df[0] = M::pack(s[2 * ks][0], s[2 * ks][1]);
      df[1] = M::pack(s[2 * ks][2], s[2 * ks][3]);
      df[2] = M::pack(s[2 * ks + 1][0], s[2 * ks + 1][1]);
      df[3] = M::pack(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
      for (int n = 0; n < HD / 8; ++n) {
        uint32_t b0, b1;
        frag_b<T, AT + 8>(b0, b1, sm.Kt, n * 8, ks * 16, g, t);
        M::run(dq[n], df, b0, b1);
      }
    }
  }
  T* dqp = (T*)a.dq + b * a.sdq.b + h * a.sdq.h;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int i = irow + r * 8;
#pragma unroll
    for (int n = 0; n < HD / 8; ++n)
      *reinterpret_cast<uint32_t*>(dqp + (int64_t)i * a.sdq.t + n * 8 + 2 * t) =
          M::pack(dq[n][2 * r] * a.scale, dq[n][2 * r + 1] * a.scale);
  }
}

// ---------------------------------------------------------------------------------- launchers
template <typename T, int HD>
static int fwd_launch(const AttnArgs& a, cudaStream_t st) {
  dim3 grid(a.T / AT, a.B * a.H);
  attn_fwd_kernel<T, HD><<<grid, AT_THREADS, 0, st>>>(a);
  return launched("attention_fwd(generic)");
}

template <typename T, int HD>
static int bwd_launch(const AttnArgs& a, cudaStream_t st) {
  int rc = attn_delta(a, HD, sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? TFB_BF16 : TFB_F16, st);
  if (rc) return rc;
  dim3 grid(a.T / AT, a.B * a.H);
  {
    auto kern = attn_bwd_kv_kernel<T, HD>;
    const int bytes = (int)sizeof(BwdKvSmem<T, HD>);
    static std::atomic<uint64_t> attr_done{0};
    if ((rc = ensure_dynamic_smem(kern, bytes, attr_done, "attention_bwd"))) return rc;
    kern<<<grid, AT_THREADS, bytes, st>>>(a);
    if ((rc = launched("attention_bwd_kv(generic)"))) return rc;
  }
  {
    auto kern = attn_bwd_q_kernel<T, HD>;
    const int bytes = (int)sizeof(BwdQSmem<T, HD>);
    static std::atomic<uint64_t> attr_done{0};
    if ((rc = ensure_dynamic_smem(kern, bytes, attr_done, "attention_bwd"))) return rc;
    kern<<<grid, AT_THREADS, bytes, st>>>(a);
    if ((rc = launched("attention_bwd_q(generic)"))) return rc;
  }
  return TFB_OK;
}

int attn_delta(const AttnArgs& a, int hd, int dtype, cudaStream_t st, float* clear) {
  const int64_t rows = (int64_t)a.B * a.H * a.T;
  TFB_DISPATCH_16(dtype, T, {
    if (hd == 32) launch_overlapped(attn_delta_kernel<T, 32>, dim3((unsigned)ceil_div(rows, 8 * 8)), dim3(256), 0, st, a, clear);
    else if (hd == 64) launch_overlapped(attn_delta_kernel<T, 64>, dim3((unsigned)ceil_div(rows, 8 * 4)), dim3(256), 0, st, a, clear);
    else launch_overlapped(attn_delta_kernel<T, 128>, dim3((unsigned)ceil_div(rows, 8 * 2)), dim3(256), 0, st, a, clear);
  })
  return launched("attention_delta");
}

int attn_generic_fwd(const AttnArgs& a, int hd, int dtype, cudaStream_t st) {
  TFB_DISPATCH_16(dtype, T, {
    if (hd == 32) return fwd_launch<T, 32>(a, st);
    if (hd == 64) return fwd_launch<T, 64>(a, st);
    if (hd == 128) return fwd_launch<T, 128>(a, st);
  })
  return fail(TFB_ERR_UNSUPPORTED, "Only head_dims of [32,64,128] are supported.");
}

int attn_generic_bwd(const AttnArgs& a, int hd, int dtype, cudaStream_t st) {
  TFB_DISPATCH_16(dtype, T, {
    if (hd == 32) return bwd_launch<T, 32>(a, st);
    if (hd == 64) return bwd_launch<T, 64>(a, st);
    if (hd == 128) return bwd_launch<T, 128>(a, st);
  })
  return fail(TFB_ERR_UNSUPPORTED, "Only head_dims of [32,64,128] are supported.");
}

}  // namespace tfb
