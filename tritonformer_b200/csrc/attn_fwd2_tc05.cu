// Causal flash attention forward on tcgen05 / TMEM, two query tiles per CTA (head_dim 64, T % 128 == 0).
//
// One CTA owns 256 consecutive queries of one (batch, head) as two 128-row tiles A and B, each with
// its own score buffer and output accumulator in TMEM and its own four softmax warps.  The tensor
// core alternates between the tiles: while the warps of one tile turn scores into probabilities, it
// multiplies the other tile's probabilities with V and computes that tile's next scores, so the
// exponential unit and the tensor core both stay busy.  K_j / V_j tiles (128 keys) are loaded once
// per CTA through 2-stage TMA rings and serve both query tiles.
//   warp 0      TMA producer
//   warp 1      MMA issuer (one elected lane)
//   warps 2-5   softmax of tile A        warps 6-9   softmax of tile B
// A softmax thread owns one query row (= TMEM lane): it reads its 128 scores into registers once,
// applies scale / ALiBi / causal mask in the log2 domain, and updates the running maximum lazily
// (the accumulator row is rescaled only when the maximum grew by more than 2^8; P stays below 2^8,
// inside fp16/bf16 range), so in the steady state no TMEM round trip of O is needed.
// For tiles below the diagonal the softmax is a single pass against the maximum of the earlier tiles
// (redone in two passes if the tile's maximum exceeds it by more than the threshold), with one
// exponential in four evaluated on the FMA pipe.  P never touches shared memory: the softmax warps
// store it (16-bit, two keys per 32-bit column) into tensor memory and the product with V takes it
// from there as its A operand, so the tensor core reads only V from shared memory for it.  The tensor
// core is given a tile's NEXT scores before the product of its current P with V.
// TMEM columns: [0,128) S_A, [128,256) S_B, [256,320) O_A, [320,384) O_B, [384,448) P_A, [448,512) P_B.
#include "attn.cuh"
#include "tc05.cuh"
#include <type_traits>

namespace tfb {

extern std::atomic<int> g_attn_debug;

namespace {

constexpr float kLog2e2 = 1.4426950408889634f;
constexpr float kLn2_2 = 0.6931471805599453f;
constexpr int F2_HD = 64;
constexpr int F2_TILE = 128;
constexpr int F2_THREADS = 320;
constexpr int F2_TILE_BYTES = 16384;  // 128 rows x 64 x 2 B
constexpr int F2_OFF_Q = 0;                        // [2]
constexpr int F2_OFF_K = 2 * F2_TILE_BYTES;        // [2]
constexpr int F2_OFF_V = 4 * F2_TILE_BYTES;        // [2]
constexpr int F2_OFF_BAR = 6 * F2_TILE_BYTES;
constexpr int F2_SMEM_BYTES = F2_OFF_BAR + 256 + 1024;
constexpr int F2_COL_S = 0, F2_COL_O = 256, F2_COL_P = 384;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct F2Params {
  int debug;  // bit 1: cycle counters of one softmax warp and the MMA thread (tfb_debug_set key 2)
  void* out;
  float* lse;
  int64_t so_b, so_h, so_t;
  int H, T;
  float scale;
  int bias_mode;
  const float* slopes;
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float alibi_term2(int mode, float slope, int dist) {
  if (mode == 1) return -slope * (float)dist;
  if (mode == 2) return __half2float(__hmul(__float2half_rn(-(float)dist), __float2half_rn(slope)));
  return __bfloat162float(__hmul(__float2bfloat16_rn(-(float)dist), __float2bfloat16_rn(slope)));
}

}  // namespace

static __device__ unsigned long long g_prof_f2[16];
#define F2_PROF(idx, t0, t1) do { if (prof) atomicAdd(&g_prof_f2[idx], (unsigned long long)((t1) - (t0))); } while (0)

// 2^x on the FMA pipe, for a share of the exponentials (the exponential unit gives 16 results per
// clock and SM and is the busiest pipe of this kernel).  x is split into a rounded integer and a
// fraction in [-0.5, 0.5] with the 1.5 * 2^23 constant; a cubic fitted to 2^f (relative error 7.5e-5,
// far below the 16-bit rounding of P) is scaled by adding the integer to the exponent field.
__device__ __forceinline__ float ex2_fma(float x) {
  x = fmaxf(x, -125.f);
  const float xr = x + 12582912.f;
  const float f = x - (xr - 12582912.f);
  float q = fmaf(f, 0.0551716685f, 0.2426111251f);
  q = fmaf(q, f, 0.6932609677f);
  q = fmaf(q, f, 0.9999280572f);
  return __int_as_float(__float_as_int(q) + (__float_as_int(xr) << 23));
}

template <typename T, bool BIAS>
__global__ void __launch_bounds__(F2_THREADS, 1) attn_fwd2_tc05_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                                       const __grid_constant__ CUtensorMap tmK,
                                                                       const __grid_constant__ CUtensorMap tmV,
                                                                       const F2Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + F2_OFF_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2 tiles] scores of the tile are in TMEM
  uint64_t* p_full = bars + 11;   // [2 tiles] probabilities in smem, accumulator rescaled
  uint64_t* pv_done = bars + 13;  // [2 tiles] P·V of the tile retired
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = p.T / F2_TILE;                      // query tiles in the sequence
  const int pair = (gridDim.x - 1) - blockIdx.x;     // longest rows first
  const int bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  const int tile_a = 2 * pair, tile_b = 2 * pair + 1;
  const bool has_b = tile_b < nq;
  const int last_a = tile_a;                         // last key tile each query tile attends to
  const int last_b = tile_b;
  const int jmax = has_b ? last_b : last_a;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);
      mbar_init(&pv_done[i], 1);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc(tmem_holder, 512);
  }
  // set-up above is CTA-local and may overlap the previous kernel's tail; global memory comes after
  grid_dependency_wait();
  allow_dependents();
  if (threadIdx.x == 0) *abort_flag = (*(volatile int*)&g_dev_status != 0) ? 1 : 0;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const bool dead = *abort_flag != 0;

  if (warp == 0) {
    // --------------------------------------------------------------------- TMA producer
    if (lane == 0 && !dead) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, (has_b ? 2 : 1) * F2_TILE_BYTES);
      tma_load_4d(smem + F2_OFF_Q, &tmQ, 0, tile_a * F2_TILE, h, b, q_full);
      if (has_b) tma_load_4d(smem + F2_OFF_Q + F2_TILE_BYTES, &tmQ, 0, tile_b * F2_TILE, h, b, q_full);
      for (int j = 0; j <= jmax; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_empty[st], ph ^ 1, 0x3100 | st, abort_flag)) break;
        mbar_expect_tx(&k_full[st], F2_TILE_BYTES);
        tma_load_4d(smem + F2_OFF_K + st * F2_TILE_BYTES, &tmK, 0, j * F2_TILE, h, b, &k_full[st]);
        if (!mbar_wait(&v_empty[st], ph ^ 1, 0x3200 | st, abort_flag)) break;
        mbar_expect_tx(&v_full[st], F2_TILE_BYTES);
        tma_load_4d(smem + F2_OFF_V + st * F2_TILE_BYTES, &tmV, 0, j * F2_TILE, h, b, &v_full[st]);
      }
    }
  } else if (warp == 1) {
    // ----------------------------------------------------------------------- MMA issuer
    if (lane == 0 && !dead) {
      constexpr int fmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t idesc_s = instr_desc_f16(128, 128, fmt, 0, 0);
      constexpr uint32_t idesc_o = instr_desc_f16(128, F2_HD, fmt, 0, 1);
      bool ok = mbar_wait(q_full, 0, 0x3300, abort_flag);
      const bool prof = (p.debug & 2) != 0;
      auto last = [&](int x) { return x == 0 ? last_a : last_b; };
      // query tiles that attend to key tile j (its K / V stage is released by the last of them)
      auto users = [&](int j) { return (j <= last_a ? 1 : 0) + ((has_b && j <= last_b) ? 1 : 0); };
      int s_cnt[2] = {0, 0}, pv_cnt[2] = {0, 0};  // per ring stage: products issued against the resident tile
      // operand descriptors are built once; the issuing thread shares its scheduler with two softmax
      // warps, so every instruction it saves per MMA shortens the tensor core's idle gaps
      uint64_t dq[2], dk[2], dv[2];
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        dq[t] = smem_desc_sw128(smem_u32(smem + F2_OFF_Q + t * F2_TILE_BYTES), 16, 1024);
        dk[t] = smem_desc_sw128(smem_u32(smem + F2_OFF_K + t * F2_TILE_BYTES), 16, 1024);
        dv[t] = smem_desc_sw128(smem_u32(smem + F2_OFF_V + t * F2_TILE_BYTES), 16384, 1024);
      }
      // S_x(j) = Q_x K_jᵀ
      auto issue_s = [&](int x, int j) {
        const int st = j & 1;
        tc_fence_after();
        const long long i0 = clock64();
#pragma unroll
        for (int s = 0; s < F2_HD / 16; ++s)
          tc_mma_ss(tmem_base + F2_COL_S + x * 128, desc_advance(dq[x], s * 32), desc_advance(dk[st], s * 32), idesc_s,
                    s ? 1u : 0u);
        tc_commit(&s_full[x]);
        if (++s_cnt[st] == users(j)) {  // K_j is free once every query tile that attends to it has been multiplied
          tc_commit(&k_empty[st]);
          s_cnt[st] = 0;
        }
        F2_PROF(10, i0, clock64());
      };
      // O_x += P_x(j) V_j
      auto issue_pv = [&](int x, int j) {
        const int st = j & 1;
        tc_fence_after();
        const long long i1 = clock64();
        // A = P_x from tensor memory (a lane is a query row, a 32-bit column holds two consecutive keys),
        // B = V_j from shared memory
        const uint32_t tp = tmem_base + F2_COL_P + x * 64;
#pragma unroll
        for (int s = 0; s < F2_TILE / 16; ++s)
          tc_mma_ts(tmem_base + F2_COL_O + x * F2_HD, tp + s * 8, desc_advance(dv[st], s * 2048), idesc_o,
                    (j | s) ? 1u : 0u);
        tc_commit(&pv_done[x]);
        if (++pv_cnt[st] == users(j)) {
          tc_commit(&v_empty[st]);
          pv_cnt[st] = 0;
        }
        F2_PROF(11, i1, clock64());
        if (prof) atomicAdd(&g_prof_f2[9], 1ull);
      };
      if (ok) ok = mbar_wait(&k_full[0], 0, 0x3400, abort_flag);
      if (ok) {
        issue_s(0, 0);
        if (has_b) issue_s(1, 0);
      }
      // Event loop: whichever tile has its probabilities ready is served, its NEXT scores first (the
      // tile's softmax warps wait for nothing else) and the product with V behind them.  Every
      // condition is probed without blocking, so a tile never waits for the other one's turn.
      int js[2] = {1, 1};  // next scores to issue per tile
      int jp[2] = {0, 0};  // next P·V to issue per tile
      uint64_t t_idle = global_ns();
      while (ok) {
        bool pending = false, progress = false;
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          if (x == 1 && !has_b) continue;
          const int L = last(x);
          if (js[x] <= L) {
            pending = true;
            const int j = js[x];  // needs P_x(j-1) complete (every read of S_x(j-1) made) and K_j resident
            if (mbar_test(&p_full[x], (j - 1) & 1) && mbar_test(&k_full[j & 1], (j >> 1) & 1)) {
              issue_s(x, j);
              js[x] = j + 1;
              progress = true;
            }
          }
          if (jp[x] <= L) {
            pending = true;
            const int j = jp[x];  // behind the tile's next scores; needs P_x(j) and V_j
            if ((js[x] > j + 1 || j == L) && mbar_test(&p_full[x], j & 1) && mbar_test(&v_full[j & 1], (j >> 1) & 1)) {
              issue_pv(x, j);
              jp[x] = j + 1;
              progress = true;
            }
          }
        }
        if (!pending) break;
        if (progress) {
          t_idle = global_ns();
        } else if (*abort_flag) {
          ok = false;
        } else if (global_ns() - t_idle > kWaitLimitNs) {
          *abort_flag = 1;
          atomicCAS(&g_dev_status, 0, 0x3500);
          ok = false;
        } else {
          __nanosleep(20);
        }
      }
    }
  } else if (!dead) {
    // -------------------------------------------------------------------------- softmax
    const int x = (warp - 2) >> 2;     // query tile of this warp: 0 = A, 1 = B
    const int qd = warp & 3;           // TMEM lane quarter
    if (x == 0 || has_b) {
      const int r = qd * 32 + lane;    // row within the tile == TMEM lane
      const int my_tile = x == 0 ? tile_a : tile_b;
      const int i = my_tile * F2_TILE + r;
      const int jlast = x == 0 ? last_a : last_b;
      const uint32_t lane_addr = tmem_base + ((uint32_t)(qd * 32) << 16);
      const uint32_t s_addr = lane_addr + F2_COL_S + x * 128;
      const uint32_t o_addr = lane_addr + F2_COL_O + x * F2_HD;
      const float c2 = p.scale * kLog2e2;
      const float slope = p.bias_mode ? p.slopes[h] : 0.f;
      const uint32_t p_addr = lane_addr + F2_COL_P + x * 64;
      float m_run = -INFINITY;   // true running maximum
      float m_used = -INFINITY;  // maximum the accumulator and the running sum are expressed against
      float l_run = 0.f;
      bool ok = true;
      for (int j = 0; j <= jlast && ok; ++j) {
        const int j0 = j * F2_TILE;
        const bool diag = (j == jlast);
        const bool plain = !BIAS && !diag;  // scores need only the common scale
        const bool prof = (p.debug & 2) && warp == 2 && lane == 0;
        const long long w0 = clock64();
        if (!mbar_wait(&s_full[x], j & 1, 0x3700 | x, abort_flag)) { ok = false; break; }
        const long long w1 = clock64();
        const long long w1b = clock64();
        F2_PROF(12, w1, w1b);
        F2_PROF(1, w0, w1);
        if (prof) atomicAdd(&g_prof_f2[0], 1ull);
        tc_fence_after();
        // ---- single pass for tiles below the diagonal once a maximum is known: p = 2^(s - m_used)
        // with the maximum of the EARLIER tiles, the row maximum of this tile tracked alongside.  If
        // that exceeds m_used by more than the rescale threshold (rare after the first tiles) the
        // tile is redone by the two passes below; otherwise O and the running sum keep their scale.
        // The scores of this tile were issued after the previous P·V of the tile, so P's buffer is
        // free as soon as they have landed.
        bool done = false;
        if (plain && j > 0) {
          float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
          float ls4[4] = {0.f, 0.f, 0.f, 0.f};
          const float neg_m = -m_used;
          uint32_t buf[2][32];
          tmem_ld32(s_addr, buf[0]);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            tc_wait_ld();
            if (c < 3) tmem_ld32(s_addr + (c + 1) * 32, buf[(c + 1) & 1]);
            const uint32_t* v = buf[c & 1];
            float g[32];
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const float sv = __uint_as_float(v[e]);
              mx4[e & 3] = fmaxf(mx4[e & 3], sv);
              const float t = fmaf(sv, c2, neg_m);
              g[e] = (e & 3) == 3 ? ex2_fma(t) : ex2_approx(t);  // one exponential in four on the FMA pipe
            }
#pragma unroll
            for (int e = 0; e < 32; ++e) ls4[e & 3] += g[e];
            uint32_t pk[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const typename Num<T>::T2 h2 = Num<T>::from_f2(g[2 * e], g[2 * e + 1]);
              pk[e] = *reinterpret_cast<const uint32_t*>(&h2);
            }
            // P of the previous step is read by its product with V until that has retired; the first
            // chunk's exponentials above overlap its tail
            if (c == 0 && !mbar_wait(&pv_done[x], (j - 1) & 1, 0x3a00 | x, abort_flag)) { ok = false; break; }
            tmem_st16(p_addr + c * 16, pk);
          }
          if (!ok) break;
          const float m_tile = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * c2;
          if (!__any_sync(0xffffffffu, (m_tile - m_used) > kRescaleThreshold)) {
            m_run = fmaxf(m_run, m_tile);
            l_run += (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
            done = true;
          }
          F2_PROF(2, w1b, clock64());
          if (prof && done) atomicAdd(&g_prof_f2[3], 1ull);
        }
        if (!done) {
        // ---- pass 1: row maximum (four independent chains; the next chunk is in flight meanwhile)
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        {
          uint32_t buf[2][32];
          tmem_ld32(s_addr, buf[0]);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            tc_wait_ld();
            if (c < 3) tmem_ld32(s_addr + (c + 1) * 32, buf[(c + 1) & 1]);
            const uint32_t* v = buf[c & 1];
            if (plain) {
#pragma unroll
              for (int e = 0; e < 32; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(v[e]));
            } else {
#pragma unroll
              for (int e = 0; e < 32; ++e) {
                const int jj = j0 + c * 32 + e;
                float t = __uint_as_float(v[e]) * c2;
                if (BIAS) t += alibi_term2(p.bias_mode, slope, max(i - jj, 0)) * kLog2e2;
                if (jj > i) t = -INFINITY;
                mx4[e & 3] = fmaxf(mx4[e & 3], t);
              }
            }
          }
        }
        float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        if (plain) mx *= c2;  // c2 > 0: scaling commutes with the maximum
        m_run = fmaxf(m_run, mx);
        // the previous P·V of this tile must have retired before P's buffer or O is touched
        if (j > 0 && !mbar_wait(&pv_done[x], (j - 1) & 1, 0x3800 | x, abort_flag)) { ok = false; break; }
        if (j == 0) {
          m_used = m_run;
        } else {
          const bool grow = (m_run - m_used) > kRescaleThreshold;
          if (__any_sync(0xffffffffu, grow)) {
            tc_fence_after();
            const float f = grow ? ex2_approx(m_used - m_run) : 1.f;
#pragma unroll
            for (int c = 0; c < F2_HD / 32; ++c) {
              uint32_t v[32];
              tmem_ld32(o_addr + c * 32, v);
              tc_wait_ld();
#pragma unroll
              for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * f);
              tmem_st32(o_addr + c * 32, v);
            }
            tc_wait_st();
            l_run *= f;
            if (grow) m_used = m_run;
          }
        }
        // ---- pass 2: p = 2^(s - m_used), partial row sums, P into swizzled smem
        float ls4[4] = {0.f, 0.f, 0.f, 0.f};
        {
          uint32_t buf[2][32];
          tmem_ld32(s_addr, buf[0]);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            tc_wait_ld();
            if (c < 3) tmem_ld32(s_addr + (c + 1) * 32, buf[(c + 1) & 1]);
            const uint32_t* v = buf[c & 1];
            float g[32];
            if (plain) {
              const float neg_m = -m_used;
#pragma unroll
              for (int e = 0; e < 32; ++e) g[e] = ex2_approx(fmaf(__uint_as_float(v[e]), c2, neg_m));
            } else {
#pragma unroll
              for (int e = 0; e < 32; ++e) {
                const int jj = j0 + c * 32 + e;
                float t = __uint_as_float(v[e]) * c2;
                if (BIAS) t += alibi_term2(p.bias_mode, slope, max(i - jj, 0)) * kLog2e2;
                g[e] = (jj > i) ? 0.f : ex2_approx(t - m_used);
              }
            }
#pragma unroll
            for (int e = 0; e < 32; ++e) ls4[e & 3] += g[e];
            uint32_t pk[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const typename Num<T>::T2 h2 = Num<T>::from_f2(g[2 * e], g[2 * e + 1]);
              pk[e] = *reinterpret_cast<const uint32_t*>(&h2);
            }
            tmem_st16(p_addr + c * 16, pk);
          }
        }
        l_run += (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
        }  // two-pass path
        const long long w2 = clock64();
        tc_wait_st();  // P is in tensor memory
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[x]);
        F2_PROF(4, w1b, w2);
        F2_PROF(5, w2, clock64());
      }
      if (ok && mbar_wait(&pv_done[x], jlast & 1, 0x3900 | x, abort_flag)) {
        tc_fence_after();
        const float inv = 1.f / l_run;
        T* orow = reinterpret_cast<T*>(p.out) + b * p.so_b + h * p.so_h + (int64_t)i * p.so_t;
#pragma unroll
        for (int c = 0; c < F2_HD / 32; ++c) {
          uint32_t v[32];
          tmem_ld32(o_addr + c * 32, v);
          tc_wait_ld();
#pragma unroll
          for (int v4 = 0; v4 < 4; ++v4) {
            float g[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) g[e] = __uint_as_float(v[v4 * 8 + e]) * inv;
            *reinterpret_cast<uint4*>(orow + c * 32 + v4 * 8) = pack8<T>(g);
          }
        }
        p.lse[(int64_t)bh * p.T + i] = (m_used + log2f(l_run)) * kLn2_2;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int k = 0; k < 64; ++k) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------- host side

// Copies the 16 cycle counters to the host and clears them.
int attn_fwd2_tc05_counters(unsigned long long* out) {
  cudaDeviceSynchronize();
  if (cudaMemcpyFromSymbol(out, g_prof_f2, sizeof(unsigned long long) * 16) != cudaSuccess) return -1;
  unsigned long long z[16] = {0};
  cudaMemcpyToSymbol(g_prof_f2, z, sizeof(z));
  return 0;
}

template <typename T>
static int fwd2_launch(const AttnArgs& a, int dtype, cudaStream_t st) {
  CUtensorMap tq, tk, tv;
  int rc;
  const uint32_t box[4] = {64, 128, 1, 1};
  const uint64_t dims[4] = {(uint64_t)F2_HD, (uint64_t)a.T, (uint64_t)a.H, (uint64_t)a.B};
  {
    const uint64_t s[3] = {(uint64_t)a.sq.t * 2, (uint64_t)a.sq.h * 2, (uint64_t)a.sq.b * 2};
    if ((rc = encode_tmap_sw128(&tq, a.q, dtype, 4, dims, s, box))) return rc;
  }
  {
    const uint64_t s[3] = {(uint64_t)a.sk.t * 2, (uint64_t)a.sk.h * 2, (uint64_t)a.sk.b * 2};
    if ((rc = encode_tmap_sw128(&tk, a.k, dtype, 4, dims, s, box))) return rc;
  }
  {
    const uint64_t s[3] = {(uint64_t)a.sv.t * 2, (uint64_t)a.sv.h * 2, (uint64_t)a.sv.b * 2};
    if ((rc = encode_tmap_sw128(&tv, a.v, dtype, 4, dims, s, box))) return rc;
  }
  F2Params p;
  p.out = a.out; p.lse = a.lse; p.so_b = a.so.b; p.so_h = a.so.h; p.so_t = a.so.t;
  p.H = a.H; p.T = a.T; p.scale = a.scale; p.bias_mode = a.bias_mode; p.slopes = a.slopes;
  p.debug = g_attn_debug.load();
  static std::atomic<uint64_t> done_plain{0}, done_bias{0};
  if ((rc = ensure_dynamic_smem(attn_fwd2_tc05_kernel<T, false>, F2_SMEM_BYTES, done_plain, "attention_fwd(tcgen05)")))
    return rc;
  if ((rc = ensure_dynamic_smem(attn_fwd2_tc05_kernel<T, true>, F2_SMEM_BYTES, done_bias, "attention_fwd(tcgen05)")))
    return rc;
  const int nq = a.T / F2_TILE;
  dim3 grid((nq + 1) / 2, a.B * a.H);
  if (a.bias_mode) launch_overlapped(attn_fwd2_tc05_kernel<T, true>, grid, dim3(F2_THREADS), F2_SMEM_BYTES, st, tq, tk, tv, p);
  else launch_overlapped(attn_fwd2_tc05_kernel<T, false>, grid, dim3(F2_THREADS), F2_SMEM_BYTES, st, tq, tk, tv, p);
  return launched("attention_fwd(tcgen05, two tiles)");
}

int attn_fwd2_tc05(const AttnArgs& a, int dtype, cudaStream_t st) {
  TFB_DISPATCH_16(dtype, T, { return fwd2_launch<T>(a, dtype, st); })
}

}  // namespace tfb
