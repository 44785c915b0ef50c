// LayerNorm forward / backward for sm_100a: HBM-bound, 128-bit accesses, fp32 math.
//
// Forward : one warp per row, the row held in registers between the mean, variance and
//           write passes, so x is read once and y written once (4 bytes / element).
// Backward: a CTA owns all columns (8 per thread) and walks groups of rows; it writes dx
//           and keeps the per-column sums for dalpha / dbeta in registers, which leave the
//           CTA once as fp32 partial rows.  finalize_partials() folds those rows.
#include "common.cuh"

namespace tfb {

// ------------------------------------------------------------------------------ forward
template <typename T, int NV>
__global__ void __launch_bounds__(128) ln_fwd_vec_kernel(
    const T* __restrict__ x, const T* __restrict__ alpha, const T* __restrict__ beta,
    T* __restrict__ y, float* __restrict__ mean, float* __restrict__ rstd,
    int64_t rows, int d, int64_t x_ld, int64_t y_ld, float eps) {
  grid_dependency_wait();
  allow_dependents();
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nvec = d >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * x_ld);
  float v[NV][8];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = i * 32 + lane;
    if (c < nvec) {
      unpack8<T>(ld_stream16(xr + c), v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) s += v[i][j];
    }
  }
  const float mu = warp_sum(s) / (float)d;
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (i * 32 + lane < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float t = v[i][j] - mu;
        q += t * t;
      }
    }
  }
  const float rs = rsqrtf(warp_sum(q) / (float)d + eps);
  if (lane == 0) {
    mean[row] = mu;
    rstd[row] = rs;
  }
  uint4* yr = reinterpret_cast<uint4*>(y + row * y_ld);
  const uint4* av = reinterpret_cast<const uint4*>(alpha);
  const uint4* bv = reinterpret_cast<const uint4*>(beta);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = i * 32 + lane;
    if (c < nvec) {
      float a[8], b[8], o[8];
      unpack8<T>(__ldg(av + c), a);
      unpack8<T>(__ldg(bv + c), b);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = a[j] * ((v[i][j] - mu) * rs) + b[j];
      st_stream16(yr + c, pack8<T>(o));
    }
  }
}

// Any d, any alignment: the row is re-read (from L1/L2) for each pass.
template <typename T>
__global__ void __launch_bounds__(128) ln_fwd_generic_kernel(
    const T* __restrict__ x, const T* __restrict__ alpha, const T* __restrict__ beta,
    T* __restrict__ y, float* __restrict__ mean, float* __restrict__ rstd,
    int64_t rows, int d, int64_t x_ld, int64_t y_ld, float eps) {
  grid_dependency_wait();
  allow_dependents();
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* xr = x + row * x_ld;
  float s = 0.f;
  for (int c = lane; c < d; c += 32) s += Num<T>::to_f(xr[c]);
  const float mu = warp_sum(s) / (float)d;
  float q = 0.f;
  for (int c = lane; c < d; c += 32) {
    const float t = Num<T>::to_f(xr[c]) - mu;
    q += t * t;
  }
  const float rs = rsqrtf(warp_sum(q) / (float)d + eps);
  if (lane == 0) {
    mean[row] = mu;
    rstd[row] = rs;
  }
  T* yr = y + row * y_ld;
  for (int c = lane; c < d; c += 32)
    yr[c] = Num<T>::from_f(Num<T>::to_f(alpha[c]) * ((Num<T>::to_f(xr[c]) - mu) * rs) +
                           Num<T>::to_f(beta[c]));
}

// ----------------------------------------------------------------------------- backward
constexpr int LN_RB = 4;  // rows per CTA iteration

template <typename T, bool VEC, int MAXT>
__global__ void __launch_bounds__(MAXT) ln_bwd_kernel(
    const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ alpha,
    const float* __restrict__ mean, const float* __restrict__ rstd, T* __restrict__ dx,
    float* __restrict__ partials, int64_t rows, int d, int64_t dy_ld, int64_t x_ld,
    int64_t dx_ld, const T* __restrict__ dres, int64_t dres_ld) {
  grid_dependency_wait();
  allow_dependents();
  __shared__ float red[2][32][2 * LN_RB];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nwarp = blockDim.x >> 5;
  const int c0 = tid * 8;
  const bool active = c0 < d;
  const int ncol = active ? min(8, d - c0) : 0;  // < 8 only on the scalar path

  float a[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) a[j] = (j < ncol) ? Num<T>::to_f(alpha[c0 + j]) : 0.f;
  float acc_a[8], acc_b[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc_a[j] = acc_b[j] = 0.f;

  const float inv_d = 1.f / (float)d;
  int buf = 0;
  const int64_t stride = (int64_t)gridDim.x * LN_RB;
  // raw 16-byte vectors of the row group being processed and of the next one (loads for the next
  // group are in flight while this one goes through its reduction, barrier and stores)
  uint4 cx[LN_RB], cg[LN_RB], nx[LN_RB], ng[LN_RB];
  auto fetch = [&](int64_t r0, uint4 (&vx)[LN_RB], uint4 (&vg)[LN_RB]) {
    if (!VEC) return;
#pragma unroll
    for (int r = 0; r < LN_RB; ++r) {
      const int64_t row = r0 + r;
      if (row < rows && active) {
        vx[r] = ld_stream16(x + row * x_ld + c0);
        vg[r] = ld_stream16(dy + row * dy_ld + c0);
      }
    }
  };
  fetch((int64_t)blockIdx.x * LN_RB, cx, cg);
  for (int64_t r0 = (int64_t)blockIdx.x * LN_RB; r0 < rows; r0 += stride) {
    if (r0 + stride < rows) fetch(r0 + stride, nx, ng);
    uint4 rv[LN_RB];  // residual-branch gradient, needed only after the reduction
    if (VEC && dres) {
#pragma unroll
      for (int r = 0; r < LN_RB; ++r)
        if (r0 + r < rows && active) rv[r] = ld_stream16(dres + (r0 + r) * dres_ld + c0);
    }
    float xh[LN_RB][8], g[LN_RB][8];
    float s[2 * LN_RB];
#pragma unroll
    for (int r = 0; r < LN_RB; ++r) {
      const int64_t row = r0 + r;
      s[2 * r] = s[2 * r + 1] = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) xh[r][j] = g[r][j] = 0.f;
      if (row < rows && active) {
        float xv[8], dv[8];
        if (VEC) {
          unpack8<T>(cx[r], xv);
          unpack8<T>(cg[r], dv);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            xv[j] = (j < ncol) ? Num<T>::to_f(x[row * x_ld + c0 + j]) : 0.f;
            dv[j] = (j < ncol) ? Num<T>::to_f(dy[row * dy_ld + c0 + j]) : 0.f;
          }
        }
        const float mu = __ldg(mean + row), rs = __ldg(rstd + row);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float h = (j < ncol) ? (xv[j] - mu) * rs : 0.f;
          xh[r][j] = h;
          g[r][j] = dv[j] * a[j];
          acc_a[j] += dv[j] * h;
          acc_b[j] += dv[j];
          s[2 * r] += g[r][j] * h;
          s[2 * r + 1] += g[r][j];
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 2 * LN_RB; ++i) s[i] = warp_sum(s[i]);
    if (lane == 0) {
#pragma unroll
      for (int i = 0; i < 2 * LN_RB; ++i) red[buf][warp][i] = s[i];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 2 * LN_RB; ++i) {
      float t = 0.f;
      for (int w = 0; w < nwarp; ++w) t += red[buf][w][i];
      s[i] = t * inv_d;
    }
    buf ^= 1;
#pragma unroll
    for (int r = 0; r < LN_RB; ++r) {
      const int64_t row = r0 + r;
      if (row < rows && active) {
        const float rs = __ldg(rstd + row);
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rs * (g[r][j] - xh[r][j] * s[2 * r] - s[2 * r + 1]);
        if (VEC) {
          if (dres) {  // gradient arriving through the residual branch that forked at this LayerNorm's input
            float e[8];
            unpack8<T>(rv[r], e);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] += e[j];
          }
          st_stream16(dx + row * dx_ld + c0, pack8<T>(o));
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (j < ncol)
              dx[row * dx_ld + c0 + j] =
                  Num<T>::from_f(o[j] + (dres ? Num<T>::to_f(dres[row * dres_ld + c0 + j]) : 0.f));
        }
      }
    }
#pragma unroll
    for (int r = 0; r < LN_RB; ++r) {
      cx[r] = nx[r];
      cg[r] = ng[r];
    }
  }
  if (active) {
    float* pa = partials + (int64_t)blockIdx.x * 2 * d;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (j < ncol) {
        pa[c0 + j] = acc_a[j];
        pa[d + c0 + j] = acc_b[j];
      }
    }
  }
}

// Backward for vectorisable rows of at most 2048 elements: G warps share a row, a lane owns ONE
// 16-byte vector of it, so a thread keeps only 8 columns of alpha and of the dalpha / dbeta sums in
// registers.  Each step handles two rows of the row group.  The vectors of the following steps are
// already on their way: every lane copies its own 16-byte pieces into a private slot of a
// shared-memory ring with cp.async (LN_DEPTH steps deep, no registers held, no barrier needed since
// a lane reads back only what it copied itself), which keeps about 100 KB per SM in flight - what
// the HBM latency needs at this bandwidth.  The two row sums are reduced by warp shuffles and
// exchanged between the G warps through shared memory behind a named barrier (double-buffered).
constexpr int LN_DEPTH = 4;
constexpr int LN_RING_BYTES = 8 * LN_DEPTH * 2 * 3 * 32 * 16;  // warps x steps x rows x tensors x lanes x 16 B

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)),
               "l"(gsrc)
               : "memory");
}

template <typename T, int G>
__global__ void __launch_bounds__(256, 2) ln_bwd_split_kernel(
    const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ alpha,
    const float* __restrict__ mean, const float* __restrict__ rstd, T* __restrict__ dx,
    float* __restrict__ partials, int64_t rows, int d, int64_t dy_ld, int64_t x_ld, int64_t dx_ld,
    const T* __restrict__ dres, int64_t dres_ld) {
  grid_dependency_wait();
  allow_dependents();
  constexpr int RG = 8 / G;  // row groups per CTA
  extern __shared__ __align__(16) uint8_t ln_smem[];
  uint4* ring = reinterpret_cast<uint4*>(ln_smem);                  // [warp][step][row][tensor][lane]
  float* fold = reinterpret_cast<float*>(ln_smem + LN_RING_BYTES);  // [2][d]
  __shared__ float4 xch[RG][2][G];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int part = warp % G, rg = warp / G;
  const int nvec = d >> 3;
  const int per = (nvec + G - 1) / G;  // vectors per warp, at most 32
  const int c = part * per + lane;
  const bool has = lane < per && c < nvec;
  for (int i = threadIdx.x; i < 2 * d; i += blockDim.x) fold[i] = 0.f;
  __syncthreads();

  float a[8], acc_a[8], acc_b[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) a[j] = acc_a[j] = acc_b[j] = 0.f;
  if (has) unpack8<T>(__ldg(reinterpret_cast<const uint4*>(alpha) + c), a);
  const float inv_d = 1.f / (float)d;
  const int64_t stride = (int64_t)gridDim.x * RG;  // rows between the two rows of a step
  const int64_t step_rows = 2 * stride;
  int64_t row = (int64_t)blockIdx.x * RG + rg;
  uint4* mine = ring + (size_t)warp * LN_DEPTH * 2 * 3 * 32 + lane;

  // One commit group per step, issued by every lane (empty groups keep the count uniform).  The source pointers
  // of the step being issued walk down the tensors (one 64-bit add per tensor and step; the row strides are
  // multiples of eight elements on this path); `ileft` counts the rows from the first row of that step to the end.
  const uint4* ix = reinterpret_cast<const uint4*>(x + row * x_ld) + c;
  const uint4* idy = reinterpret_cast<const uint4*>(dy + row * dy_ld) + c;
  const uint4* idr = dres ? reinterpret_cast<const uint4*>(dres + row * dres_ld) + c : nullptr;
  const int64_t x_k = stride * (x_ld >> 3), dy_k = stride * (dy_ld >> 3), dr_k = stride * (dres_ld >> 3);  // second row
  int64_t ileft = rows - row;
  auto issue = [&](int slot) {
    uint4* dst = mine + (slot * 2 * 3) * 32;
    if (has && ileft > 0) {
      cp_async16(dst, ix);
      cp_async16(dst + 32, idy);
      if (dres) cp_async16(dst + 64, idr);
    }
    if (has && ileft > stride) {
      cp_async16(dst + 96, ix + x_k);
      cp_async16(dst + 128, idy + dy_k);
      if (dres) cp_async16(dst + 160, idr + dr_k);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    ix += 2 * x_k;
    idy += 2 * dy_k;
    if (dres) idr += 2 * dr_k;
    ileft -= step_rows;
  };
#pragma unroll
  for (int s = 0; s < LN_DEPTH - 1; ++s) issue(s);
  // the row statistics travel one step ahead in registers (a dependent load per step otherwise)
  float mu_next[2], rs_next[2];
  auto fetch_stats = [&](int64_t r0) {
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int64_t r = r0 + k * stride;
      mu_next[k] = r < rows ? __ldg(mean + r) : 0.f;
      rs_next[k] = r < rows ? __ldg(rstd + r) : 0.f;
    }
  };
  fetch_stats(row);
  int slot = 0, parity = 0;
  for (; row < rows; row += step_rows) {
    issue((slot + LN_DEPTH - 1) % LN_DEPTH);
    const float mu_cur[2] = {mu_next[0], mu_next[1]}, rs_cur[2] = {rs_next[0], rs_next[1]};
    fetch_stats(row + step_rows);
    asm volatile("cp.async.wait_group %0;" ::"n"(LN_DEPTH - 1) : "memory");  // this step's copies have landed
    uint4 cr[2];
    float rs[2], s1[2], s2[2];
    float h[2][8], gg[2][8];  // normalised input and alpha-scaled gradient, kept for the second pass
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int64_t r = row + k * stride;
      const bool live = r < rows;
      const float mu = mu_cur[k];
      rs[k] = rs_cur[k];
      const float shift = -mu * rs[k];
      s1[k] = s2[k] = 0.f;
      if (has && live) {
        const uint4* src = mine + ((slot * 2 + k) * 3) * 32;
        float xv[8], dv[8];
        unpack8<T>(src[0], xv);
        unpack8<T>(src[32], dv);
        if (dres) cr[k] = src[64];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          h[k][j] = fmaf(xv[j], rs[k], shift);
          gg[k][j] = dv[j] * a[j];
          acc_a[j] = fmaf(dv[j], h[k][j], acc_a[j]);
          acc_b[j] += dv[j];
          s1[k] = fmaf(gg[k][j], h[k][j], s1[k]);
          s2[k] += gg[k][j];
        }
      }
    }
    // The four sums of the step are reduced together: after the exchanges over 16 and over 8 lanes each lane
    // carries ONE of them (which one: bits 4 and 3 of its lane number), so three more exchanges finish all four -
    // six shuffles instead of twenty.  Lanes 0, 8, 16, 24 end up with s1[0], s2[0], s1[1], s2[1].
    float red;
    {
      const bool hi = lane & 16, mid = lane & 8;
      float k0 = hi ? s1[1] : s1[0], k1 = hi ? s2[1] : s2[0];
      k0 += __shfl_xor_sync(0xffffffffu, hi ? s1[0] : s1[1], 16);
      k1 += __shfl_xor_sync(0xffffffffu, hi ? s2[0] : s2[1], 16);
      red = (mid ? k1 : k0) + __shfl_xor_sync(0xffffffffu, mid ? k0 : k1, 8);
      red += __shfl_xor_sync(0xffffffffu, red, 4);
      red += __shfl_xor_sync(0xffffffffu, red, 2);
      red += __shfl_xor_sync(0xffffffffu, red, 1);
    }
    if (G == 1) {
      s1[0] = __shfl_sync(0xffffffffu, red, 0);
      s2[0] = __shfl_sync(0xffffffffu, red, 8);
      s1[1] = __shfl_sync(0xffffffffu, red, 16);
      s2[1] = __shfl_sync(0xffffffffu, red, 24);
    }
    if (G > 1) {
      // all G warps of the row group run the same number of steps, so the barrier counts match
      if ((lane & 7) == 0) reinterpret_cast<float*>(&xch[rg][parity][part])[lane >> 3] = red;
      asm volatile("bar.sync %0, %1;" ::"r"(1 + rg), "r"(32 * G) : "memory");
      float4 t = xch[rg][parity][0];
#pragma unroll
      for (int g = 1; g < G; ++g) {
        const float4 u = xch[rg][parity][g];
        t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
      }
      s1[0] = t.x; s2[0] = t.y; s1[1] = t.z; s2[1] = t.w;
      parity ^= 1;
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int64_t r = row + k * stride;
      if (has && r < rows) {
        // dx = rstd * (g - h * mean(g h) - mean(g)) as two fused multiply-adds per element
        const float k1 = -rs[k] * s1[k] * inv_d, k2 = -rs[k] * s2[k] * inv_d;
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = fmaf(rs[k], gg[k][j], fmaf(k1, h[k][j], k2));
        if (dres) {
          float e[8];
          unpack8<T>(cr[k], e);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += e[j];
        }
        st_stream16(reinterpret_cast<uint4*>(dx + r * dx_ld) + c, pack8<T>(o));
      }
    }
    slot = (slot + 1) % LN_DEPTH;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  if (has) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (RG > 1) {
        atomicAdd(&fold[c * 8 + j], acc_a[j]);
        atomicAdd(&fold[d + c * 8 + j], acc_b[j]);
      } else {
        fold[c * 8 + j] = acc_a[j];
        fold[d + c * 8 + j] = acc_b[j];
      }
    }
  }
  __syncthreads();
  float* pa = partials + (int64_t)blockIdx.x * 2 * d;
  for (int i = threadIdx.x; i < 2 * d; i += blockDim.x) pa[i] = fold[i];
}

// 32 columns per CTA; the rows are spread over the CTA's warps (32 for many partial rows, 8 otherwise), so
// that each thread has only a few dependent-free loads to wait for.
template <typename T>
__global__ void __launch_bounds__(1024) finalize_partials_kernel(
    const float* __restrict__ partials, int64_t n, int ncols, int split, T* __restrict__ out0,
    T* __restrict__ out1, int accumulate) {
  grid_dependency_wait();
  allow_dependents();
  __shared__ float sm[32][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5, nry = blockDim.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float s = 0.f;
  if (c < ncols)
    for (int64_t r = ry; r < n; r += nry) s += partials[r * ncols + c];
  sm[ry][cx] = s;
  __syncthreads();
  if (ry == 0 && c < ncols) {
    for (int i = 1; i < nry; ++i) s += sm[i][cx];
    T* dst = c < split ? out0 + c : out1 + (c - split);
    if (accumulate) s += Num<T>::to_f(*dst);  // the sums are added to what the output already holds
    *dst = Num<T>::from_f(s);
  }
}

template <typename T>
int finalize_partials(const float* partials, int64_t n, int ncols, int split, void* out0,
                      void* out1, cudaStream_t st, int accumulate) {
  launch_overlapped(finalize_partials_kernel<T>, dim3((unsigned)ceil_div(ncols, 32)), dim3(n > 64 ? 1024 : 256), 0, st,
                    partials, n, ncols, split, (T*)out0, (T*)out1, accumulate);
  return launched("finalize_partials");
}
template int finalize_partials<__half>(const float*, int64_t, int, int, void*, void*, cudaStream_t, int);
template int finalize_partials<__nv_bfloat16>(const float*, int64_t, int, int, void*, void*, cudaStream_t, int);

static int ln_bwd_threads(int64_t d) { return (int)(ceil_div(ceil_div(d, 8), 32) * 32); }

template <typename T>
static int ln_bwd_launch(const void* dy, const void* x, const void* alpha, const float* mean,
                         const float* rstd, void* dx, void* dalpha, void* dbeta, float* partials,
                         int64_t n_partials, int64_t rows, int d, int64_t dy_ld, int64_t x_ld,
                         int64_t dx_ld, bool vec, int threads, cudaStream_t st, const void* dres = nullptr,
                         int64_t dres_ld = 0, int accumulate = 0) {
#define TFB_LN_BWD(V, MT)                                                                     \
  launch_overlapped(ln_bwd_kernel<T, V, MT>, dim3((unsigned)n_partials), dim3(threads), 0, st, \
      (const T*)dy, (const T*)x, (const T*)alpha, mean, rstd, (T*)dx, partials, rows, d, dy_ld, \
      x_ld, dx_ld, (const T*)dres, dres_ld)
  if (vec && d <= 2048 && aligned16(alpha)) {
    const size_t sm = (size_t)LN_RING_BYTES + (size_t)2 * d * sizeof(float);
    const T *gp = (const T*)dy, *xp = (const T*)x, *ap = (const T*)alpha, *rp = (const T*)dres;
    T* op = (T*)dx;
    const dim3 grid((unsigned)n_partials), block(256);
#define TFB_LN_SPLIT(G)                                                                                         \
  do {                                                                                                          \
    static std::atomic<uint64_t> attr_done{0};                                                                  \
    if (int rc0 = ensure_dynamic_smem(ln_bwd_split_kernel<T, G>, (int)(LN_RING_BYTES + 2 * 2048 * sizeof(float)), \
                                      attr_done, "layernorm_bwd"))                                              \
      return rc0;                                                                                               \
    launch_overlapped(ln_bwd_split_kernel<T, G>, grid, block, sm, st, gp, xp, ap, mean, rstd, op, partials, rows, d, \
                      dy_ld, x_ld, dx_ld, rp, dres_ld);                                                         \
  } while (0)
    if (d <= 256) TFB_LN_SPLIT(1);
    else if (d <= 512) TFB_LN_SPLIT(2);
    else if (d <= 1024) TFB_LN_SPLIT(4);
    else TFB_LN_SPLIT(8);
#undef TFB_LN_SPLIT
  } else if (vec && threads <= 256) TFB_LN_BWD(true, 256);
  else if (vec) TFB_LN_BWD(true, 1024);
  else if (threads <= 256) TFB_LN_BWD(false, 256);
  else TFB_LN_BWD(false, 1024);
#undef TFB_LN_BWD
  int rc = launched("layernorm_bwd");
  if (rc) return rc;
  return finalize_partials<T>(partials, n_partials, 2 * d, d, dalpha, dbeta, st, accumulate);
}

}  // namespace tfb

using namespace tfb;

extern "C" int tfb_layernorm_fwd(const void* x, const void* alpha, const void* beta, void* y,
                                 float* mean, float* rstd, int64_t rows, int64_t d, int64_t x_ld,
                                 int64_t y_ld, float eps, int dtype, void* stream) {
  TFB_REQUIRE(rows >= 0 && d > 0 && d < (1 << 30), "layernorm_fwd: bad shape rows=%lld d=%lld",
              (long long)rows, (long long)d);
  TFB_REQUIRE(x_ld >= d && y_ld >= d, "layernorm_fwd: row stride smaller than d");
  if (rows == 0) return TFB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned grid = (unsigned)ceil_div(rows, 4);
  const bool vec = (d % 8 == 0) && (x_ld % 8 == 0) && (y_ld % 8 == 0) && aligned16(x) &&
                   aligned16(y) && aligned16(alpha) && aligned16(beta) && d <= 2048;
  TFB_DISPATCH_16(dtype, T, {
    const T *xp = (const T*)x, *ap = (const T*)alpha, *bp = (const T*)beta;
    T* yp = (T*)y;
    if (!vec) {
      launch_overlapped(ln_fwd_generic_kernel<T>, dim3(grid), dim3(128), 0, st, xp, ap, bp, yp, mean, rstd, rows, (int)d, x_ld, y_ld, eps);
    } else if (d <= 256) {
      launch_overlapped(ln_fwd_vec_kernel<T, 1>, dim3(grid), dim3(128), 0, st, xp, ap, bp, yp, mean, rstd, rows, (int)d, x_ld, y_ld, eps);
    } else if (d <= 512) {
      launch_overlapped(ln_fwd_vec_kernel<T, 2>, dim3(grid), dim3(128), 0, st, xp, ap, bp, yp, mean, rstd, rows, (int)d, x_ld, y_ld, eps);
    } else if (d <= 1024) {
      launch_overlapped(ln_fwd_vec_kernel<T, 4>, dim3(grid), dim3(128), 0, st, xp, ap, bp, yp, mean, rstd, rows, (int)d, x_ld, y_ld, eps);
    } else {
      launch_overlapped(ln_fwd_vec_kernel<T, 8>, dim3(grid), dim3(128), 0, st, xp, ap, bp, yp, mean, rstd, rows, (int)d, x_ld, y_ld, eps);
    }
  })
  return launched("layernorm_fwd");
}

extern "C" int64_t tfb_layernorm_bwd_partials(int64_t rows, int64_t d) {
  (void)d;
  int64_t n = ceil_div(rows, 16);
  const int64_t cap = 148 * 2;  // two CTAs per SM
  if (n > cap) n = cap;
  return n < 1 ? 1 : n;
}

extern "C" int tfb_layernorm_bwd_acc(const void* dy, const void* x, const void* alpha, const float* mean,
                                     const float* rstd, const void* dres, void* dx, void* dalpha, void* dbeta,
                                     float* partials, int64_t n_partials, int64_t rows, int64_t d, int64_t dy_ld,
                                     int64_t x_ld, int64_t dres_ld, int64_t dx_ld, int accumulate, int dtype,
                                     void* stream) {
  TFB_REQUIRE(rows > 0 && d > 0, "layernorm_bwd: bad shape rows=%lld d=%lld", (long long)rows,
              (long long)d);
  if (d > 8192) return fail(TFB_ERR_UNSUPPORTED, "layernorm_bwd: d=%lld > 8192", (long long)d);
  TFB_REQUIRE(n_partials == tfb_layernorm_bwd_partials(rows, d),
              "layernorm_bwd: scratch must hold tfb_layernorm_bwd_partials() rows");
  TFB_REQUIRE(dy_ld >= d && x_ld >= d && dx_ld >= d && (!dres || dres_ld >= d),
              "layernorm_bwd: row stride smaller than d");
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = (d % 8 == 0) && (x_ld % 8 == 0) && (dy_ld % 8 == 0) && (dx_ld % 8 == 0) &&
                   aligned16(x) && aligned16(dy) && aligned16(dx) &&
                   (!dres || (aligned16(dres) && dres_ld % 8 == 0));
  const int threads = ln_bwd_threads(d);
  TFB_DISPATCH_16(dtype, T, {
    return ln_bwd_launch<T>(dy, x, alpha, mean, rstd, dx, dalpha, dbeta, partials, n_partials, rows,
                            (int)d, dy_ld, x_ld, dx_ld, vec, threads, st, dres, dres_ld, accumulate ? 1 : 0);
  })
}

extern "C" int tfb_layernorm_bwd_res(const void* dy, const void* x, const void* alpha, const float* mean,
                                     const float* rstd, const void* dres, void* dx, void* dalpha, void* dbeta,
                                     float* partials, int64_t n_partials, int64_t rows, int64_t d, int64_t dy_ld,
                                     int64_t x_ld, int64_t dres_ld, int64_t dx_ld, int dtype, void* stream) {
  return tfb_layernorm_bwd_acc(dy, x, alpha, mean, rstd, dres, dx, dalpha, dbeta, partials, n_partials, rows, d,
                               dy_ld, x_ld, dres_ld, dx_ld, 0, dtype, stream);
}

extern "C" int tfb_layernorm_bwd(const void* dy, const void* x, const void* alpha,
                                 const float* mean, const float* rstd, void* dx, void* dalpha,
                                 void* dbeta, float* partials, int64_t n_partials, int64_t rows,
                                 int64_t d, int64_t dy_ld, int64_t x_ld, int64_t dx_ld, int dtype,
                                 void* stream) {
  return tfb_layernorm_bwd_res(dy, x, alpha, mean, rstd, nullptr, dx, dalpha, dbeta, partials, n_partials, rows,
                               d, dy_ld, x_ld, 0, dx_ld, dtype, stream);
}

// ------------------------------------------------------------------------------------------
// LayerNorm backward without caller-provided scratch.
//
// Some hosts of this library cannot hand it scratch memory: a binding that marshals only the
// operator's own inputs and outputs, or a service whose device memory is carved up once at
// start-up and which keeps cudaMalloc / cudaFree (device-wide synchronising calls) off its
// request path.  For them the fp32 partial column sums live in the fixed device array below
// instead of a buffer the caller allocates.  The array belongs to the library image: every
// GPU that loads the library carries it (kStaticRows * 2 * kStaticMaxD floats) until exit.
constexpr int kStaticRows = 296;    // partial rows (two CTAs per SM)
constexpr int kStaticMaxD = 4096;   // widest supported row
static __device__ __align__(256) float g_ln_static_scratch[(size_t)kStaticRows * 2 * kStaticMaxD];

namespace {
struct StaticScratch {
  std::atomic<float*> ptr[64];
};
StaticScratch g_static_scratch;

// Device address of the array on the current device.  `g_ln_static_scratch` named in host code
// is only a handle for the runtime, not something a kernel may dereference; the address has
// to be asked for once per device, with that device current.
int static_scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64)
    return tfb::fail(TFB_ERR_LAUNCH, "layernorm_bwd_static: cudaGetDevice: %s", cudaGetErrorString(e));
  float* p = g_static_scratch.ptr[dev].load(std::memory_order_acquire);
  if (!p) {
    void* sym = nullptr;
    e = cudaGetSymbolAddress(&sym, g_ln_static_scratch);
    if (e != cudaSuccess || !sym)
      return tfb::fail(TFB_ERR_LAUNCH, "layernorm_bwd_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    p = static_cast<float*>(sym);
    g_static_scratch.ptr[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return TFB_OK;
}
}  // namespace

extern "C" int tfb_layernorm_bwd_static(const void* dy, const void* x, const void* alpha, const float* mean,
                                        const float* rstd, void* dx, void* dalpha, void* dbeta, int64_t rows,
                                        int64_t d, int64_t dy_ld, int64_t x_ld, int64_t dx_ld, int dtype,
                                        void* stream) {
  TFB_REQUIRE(rows > 0 && d > 0, "layernorm_bwd_static: bad shape rows=%lld d=%lld", (long long)rows, (long long)d);
  if (d > kStaticMaxD)
    return fail(TFB_ERR_UNSUPPORTED,
                "layernorm_bwd_static: d=%lld exceeds the built-in scratch (rows of at most %d elements); "
                "use tfb_layernorm_bwd with caller-provided scratch",
                (long long)d, kStaticMaxD);
  TFB_REQUIRE(dy_ld >= d && x_ld >= d && dx_ld >= d, "layernorm_bwd_static: row stride smaller than d");
  float* scratch = nullptr;
  int rc = static_scratch_for_current_device(&scratch);
  if (rc) return rc;
  int64_t n = ceil_div(rows, 16);
  if (n > kStaticRows) n = kStaticRows;
  // Every one of the n partial rows is rewritten in full by the first kernel before the second
  // reads it, so nothing in the array has to be cleared between calls.
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = (d % 8 == 0) && (x_ld % 8 == 0) && (dy_ld % 8 == 0) && (dx_ld % 8 == 0) && aligned16(x) &&
                   aligned16(dy) && aligned16(dx);
  const int threads = ln_bwd_threads(d);
  TFB_DISPATCH_16(dtype, T, {
    return ln_bwd_launch<T>(dy, x, alpha, mean, rstd, dx, dalpha, dbeta, scratch, n, rows, (int)d, dy_ld, x_ld,
                            dx_ld, vec, threads, st);
  })
}
