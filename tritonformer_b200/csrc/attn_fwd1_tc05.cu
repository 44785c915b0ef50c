// Causal flash attention forward on tcgen05 / TMEM, one 128-query tile per CTA with its score and P
// buffers doubled and eight softmax warps (head_dim 64 or 128, T % 128 == 0).
//
//   warp 0      TMA producer (Q once, K_j / V_j tiles of 128 keys through 3-stage rings)
//   warp 1      MMA issuer (one elected lane, an event loop over non-blocking barrier probes)
//   warps 2-9   softmax: two warps per TMEM lane quarter, each taking 64 of the 128 keys of a step
//               (F1_NW; four per quarter measured slower: the pass is bound by issue slots and the
//               exponential unit of a scheduler, not by latency)
// The scores of step j+1 are computed into the other score buffer while the softmax warps work on
// step j, so they go from step to step without waiting for the tensor core (with one buffer per tile
// the round trip "probabilities ready -> next scores issued -> scores landed" is a fixed 1.5 k cycles
// per step that nothing hides).  A thread owns 64 keys of one query row; the two warps of a row
// exchange one value per step through shared memory (an mbarrier with one arrival per warp and lane
// quarter, so the wait is bounded), keep separate partial row sums and add them at the end.
// Below the diagonal the softmax is a single pass against the maximum of the EARLIER steps (redone in
// two passes if the new maximum exceeds it by more than 2^8, which also bounds P inside fp16/bf16
// range; the accumulator row is rescaled only then), with one exponential in four on the FMA pipe.
// P is stored 16-bit, two keys per 32-bit column, into tensor memory and is the A operand of P·V.
// TMEM columns: [0,128) S0, [128,256) S1, [256,320) P0, [320,384) P1, [384,384+head_dim) O.
#include "attn.cuh"
#include "tc05.cuh"
#include <type_traits>

namespace tfb {

extern std::atomic<int> g_attn_debug;

namespace {

constexpr float kLog2e1 = 1.4426950408889634f;
constexpr float kLn2_1 = 0.6931471805599453f;
constexpr int F1_TILE = 128;
constexpr int F1_NW = 2;                       // softmax warps per TMEM lane quarter (per query row)
constexpr int F1_KW = F1_TILE / F1_NW;         // keys of a step per softmax warp
constexpr int F1_NC = F1_KW / 32;              // 32-key chunks per warp and step
constexpr int F1_THREADS = 64 + 128 * F1_NW;
constexpr int F1_COL_S = 0, F1_COL_P = 256, F1_COL_O = 384;

template <int HD> struct F1Cfg {
  static constexpr int PANELS = HD / 64;                 // 64-element (128-byte) panels along head_dim
  static constexpr int TILE_BYTES = PANELS * 16384;      // 128 rows x HD x 2 B
  static constexpr int STAGES = (HD == 64) ? 3 : 2;      // K / V ring depth (shared memory bound at 128)
  static constexpr int OW = HD / F1_NW;                  // accumulator columns per warp (rescale, output)
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = TILE_BYTES;                         // [STAGES]
  static constexpr int OFF_V = OFF_K + STAGES * TILE_BYTES;        // [STAGES]
  static constexpr int OFF_X = OFF_V + STAGES * TILE_BYTES;        // row exchange: [2 parities][warps per row][128 rows] floats
  static constexpr int OFF_BAR = OFF_X + 2 * F1_NW * 128 * 4;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  static_assert(OW % 32 == 0, "a softmax warp handles whole 32-column chunks of the accumulator");
  static_assert(F1_COL_O + HD <= 512, "tensor memory");
};
constexpr float kRescale1 = 8.0f;  // log2 units

struct F1Params {
  int debug;  // bit 1: cycle counters of one softmax warp (tfb_debug_set key 2)
  void* out;
  float* lse;
  int64_t so_b, so_h, so_t;
  int H, T;
  float scale;
  int bias_mode;
  const float* slopes;
};

__device__ __forceinline__ float ex2_mufu(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 2^x on the FMA pipe (cubic fitted to 2^f on [-0.5, 0.5], relative error 7.5e-5, far below the 16-bit
// rounding of P; the integer part goes into the exponent field).
__device__ __forceinline__ float ex2_fma1(float x) {
  x = fmaxf(x, -125.f);
  const float xr = x + 12582912.f;
  const float f = x - (xr - 12582912.f);
  float q = fmaf(f, 0.0551716685f, 0.2426111251f);
  q = fmaf(q, f, 0.6932609677f);
  q = fmaf(q, f, 0.9999280572f);
  return __int_as_float(__float_as_int(q) + (__float_as_int(xr) << 23));
}

}  // namespace

// [0] steps, [1] wait for scores, [2] pass, [3] row-pair exchange, [4] store fence + arrive (warp 2, lane 0)
static __device__ unsigned long long g_prof_f1[16];
#define F1_PROF(idx, t0, t1) do { if (prof) atomicAdd(&g_prof_f1[idx], (unsigned long long)((t1) - (t0))); } while (0)

template <typename T, int HD, bool BIAS>
__global__ void __launch_bounds__(F1_THREADS, 1) attn_fwd1_tc05_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                                       const __grid_constant__ CUtensorMap tmK,
                                                                       const __grid_constant__ CUtensorMap tmV,
                                                                       const F1Params p) {
  using Cfg = F1Cfg<HD>;
  constexpr int F1_STAGES = Cfg::STAGES, F1_TILE_BYTES = Cfg::TILE_BYTES, F1_OW = Cfg::OW;
  constexpr int F1_OFF_Q = Cfg::OFF_Q, F1_OFF_K = Cfg::OFF_K, F1_OFF_V = Cfg::OFF_V, F1_OFF_X = Cfg::OFF_X;
  constexpr int F1_OFF_BAR = Cfg::OFF_BAR;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + F1_OFF_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;                   // [STAGES]
  uint64_t* k_empty = k_full + F1_STAGES;        // [STAGES]
  uint64_t* v_full = k_empty + F1_STAGES;        // [STAGES]
  uint64_t* v_empty = v_full + F1_STAGES;        // [STAGES]
  uint64_t* s_full = v_empty + F1_STAGES;        // [2 buffers] scores of a step are in TMEM
  uint64_t* p_full = s_full + 2;                 // [2 buffers] probabilities stored, score buffer read (8 warps)
  uint64_t* pv_done = p_full + 2;                // [2 buffers] the P·V that read the P buffer has retired
  uint64_t* pair_bar = pv_done + 2;              // [4 lane quarters] both warps of the row pair have published
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(pair_bar + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  float* xch = reinterpret_cast<float*>(smem + F1_OFF_X);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = (gridDim.x - 1) - blockIdx.x;  // longest rows first
  const int bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  const int jlast = qt;                          // last key tile this query tile attends to

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < F1_STAGES; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4 * F1_NW);
      mbar_init(&pv_done[i], 1);
    }
    for (int i = 0; i < 4; ++i) mbar_init(&pair_bar[i], F1_NW);
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
      mbar_expect_tx(q_full, F1_TILE_BYTES);
#pragma unroll
      for (int c = 0; c < Cfg::PANELS; ++c) tma_load_4d(smem + F1_OFF_Q + c * 16384, &tmQ, c * 64, qt * F1_TILE, h, b, q_full);
      int st = 0;
      uint32_t ph = 0;
      for (int j = 0; j <= jlast; ++j) {
        if (!mbar_wait(&k_empty[st], ph ^ 1, 0x5100 | st, abort_flag)) break;
        mbar_expect_tx(&k_full[st], F1_TILE_BYTES);
#pragma unroll
        for (int c = 0; c < Cfg::PANELS; ++c)
          tma_load_4d(smem + F1_OFF_K + st * F1_TILE_BYTES + c * 16384, &tmK, c * 64, j * F1_TILE, h, b, &k_full[st]);
        if (!mbar_wait(&v_empty[st], ph ^ 1, 0x5200 | st, abort_flag)) break;
        mbar_expect_tx(&v_full[st], F1_TILE_BYTES);
#pragma unroll
        for (int c = 0; c < Cfg::PANELS; ++c)
          tma_load_4d(smem + F1_OFF_V + st * F1_TILE_BYTES + c * 16384, &tmV, c * 64, j * F1_TILE, h, b, &v_full[st]);
        if (++st == F1_STAGES) { st = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ----------------------------------------------------------------------- MMA issuer
    if (lane == 0 && !dead) {
      constexpr int fmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t idesc_s = instr_desc_f16(128, 128, fmt, 0, 0);
      constexpr uint32_t idesc_o = instr_desc_f16(128, HD, fmt, 0, 1);
      bool ok = mbar_wait(q_full, 0, 0x5300, abort_flag);
      const uint64_t dq = smem_desc_sw128(smem_u32(smem + F1_OFF_Q), 16, 1024);
      // Event loop: the next scores go out as soon as their buffer has been read (two steps back) and
      // K has landed; the product with V as soon as P is stored and V has landed.
      int us = 0, up = 0;            // next scores / next P·V to issue
      int ks = 0, vs = 0;            // ring stage of that step's K / V
      uint32_t kph = 0, vph = 0;     // ring phase of that step's K / V
      uint64_t t_idle = global_ns();
      while (ok && up <= jlast) {
        bool progress = false;
        if (us <= jlast && (us < 2 || mbar_test(&p_full[us & 1], ((us - 2) >> 1) & 1)) && mbar_test(&k_full[ks], kph)) {
          tc_fence_after();
          const uint64_t dk = smem_desc_sw128(smem_u32(smem + F1_OFF_K + ks * F1_TILE_BYTES), 16, 1024);
#pragma unroll
          for (int s = 0; s < HD / 16; ++s) {
            const uint32_t off = (s / 4) * 16384 + (s % 4) * 32;  // 64-element panel, then 32 bytes per k-step
            tc_mma_ss(tmem_base + F1_COL_S + (us & 1) * 128, desc_advance(dq, off), desc_advance(dk, off), idesc_s,
                      s ? 1u : 0u);
          }
          tc_commit(&s_full[us & 1]);
          tc_commit(&k_empty[ks]);
          if (++ks == F1_STAGES) { ks = 0; kph ^= 1; }
          ++us;
          progress = true;
        }
        if (mbar_test(&p_full[up & 1], (up >> 1) & 1) && mbar_test(&v_full[vs], vph)) {
          tc_fence_after();
          // A = P from tensor memory (a lane is a query row, a 32-bit column holds two consecutive
          // keys), B = V_j from shared memory
          const uint64_t dv = smem_desc_sw128(smem_u32(smem + F1_OFF_V + vs * F1_TILE_BYTES), 16384, 1024);
          const uint32_t tp = tmem_base + F1_COL_P + (up & 1) * 64;
#pragma unroll
          for (int s = 0; s < F1_TILE / 16; ++s)
            tc_mma_ts(tmem_base + F1_COL_O, tp + s * 8, desc_advance(dv, s * 2048), idesc_o, (up | s) ? 1u : 0u);
          tc_commit(&pv_done[up & 1]);
          tc_commit(&v_empty[vs]);
          if (++vs == F1_STAGES) { vs = 0; vph ^= 1; }
          ++up;
          progress = true;
        }
        if (progress) {
          t_idle = global_ns();
        } else if (*abort_flag) {
          ok = false;
        } else if (global_ns() - t_idle > kWaitLimitNs) {
          *abort_flag = 1;
          atomicCAS(&g_dev_status, 0, 0x5500);
          ok = false;
        } else {
          __nanosleep(20);
        }
      }
    }
  } else if (!dead) {
    // -------------------------------------------------------------------------- softmax
    const int qd = warp & 3;            // TMEM lane quarter
    const int ch = (warp - 2) >> 2;     // which F1_KW of the step's 128 keys
    const int r = qd * 32 + lane;       // row within the tile == TMEM lane
    const int i = qt * F1_TILE + r;     // query
    const uint32_t lane_addr = tmem_base + ((uint32_t)(qd * 32) << 16);
    const uint32_t o_addr = lane_addr + F1_COL_O;
    const float c2 = p.scale * kLog2e1;
    const float slope = p.bias_mode ? p.slopes[h] : 0.f;
    float m_run = -INFINITY;   // true running maximum of the row (both halves)
    float m_used = -INFINITY;  // maximum the accumulator and the running sums are expressed against
    float l_run = 0.f;         // this thread's partial row sum (its 64 keys of every step)
    uint32_t pair_phase = 0;
    int xpar = 0;
    bool ok = true;
    // Row-pair exchange: publish a value for this row, learn the partner's (the warp that handles the
    // other 64 keys of the same rows).  Both warps of a pair take the same path through a step, so
    // they make the same number of exchanges.  Bounded wait; double-buffered by exchange parity.
    long long xw_total = 0;
    // Row exchange: publish a value for this row and combine the values of the other warps that share
    // the row (maximum, or sum when `add`).  All warps of a row take the same path through a step, so
    // they make the same number of exchanges.  Bounded wait; double-buffered by exchange parity.
    auto exchange = [&](float mine, bool& fine, bool add) -> float {
      const long long x0 = clock64();
      float* slot = xch + xpar * (F1_NW * 128);
      slot[ch * 128 + r] = mine;
      __syncwarp();
      if (lane == 0) mbar_arrive(&pair_bar[qd]);
      if (fine) fine = mbar_wait(&pair_bar[qd], pair_phase, 0x5c00 | qd, abort_flag);
      pair_phase ^= 1;
      float acc = mine;
#pragma unroll
      for (int w = 1; w < F1_NW; ++w) {
        const float other = slot[((ch + w) % F1_NW) * 128 + r];
        acc = add ? acc + other : fmaxf(acc, other);
      }
      xpar ^= 1;
      xw_total += clock64() - x0;
      return acc;
    };
    for (int j = 0; j <= jlast; ++j) {
      const int bsel = j & 1;
      const int j0 = j * F1_TILE + ch * F1_KW;  // first key of this thread's share
      const bool diag = (j == jlast);
      const bool plain = !BIAS && !diag;      // scores need only the common scale
      const uint32_t s_addr = lane_addr + F1_COL_S + bsel * 128 + ch * F1_KW;
      const uint32_t p_addr = lane_addr + F1_COL_P + bsel * 64 + ch * (F1_KW / 2);
      const bool prof = (p.debug & 2) && warp == 2 && lane == 0;
      const long long w0 = clock64();
      if (ok) ok = mbar_wait(&s_full[bsel], (j >> 1) & 1, 0x5700 | bsel, abort_flag);
      const long long w1 = clock64();
      F1_PROF(1, w0, w1);
      if (prof) atomicAdd(&g_prof_f1[0], 1ull);
      const long long xw = xw_total;  // exchange cycles before this step
      tc_fence_after();
      bool done = false;
      if (plain && j > 0) {
        // ---- single pass against the maximum of the earlier steps.  No maximum is tracked here: a
        // probability is at most this thread's partial row sum, so while that stays below 2^8 the
        // 16-bit range holds; otherwise (rare after the first steps) the step is redone in two passes
        // with a fresh maximum.  The two warps of a row pair exchange the verdict.
        float ls4[4] = {0.f, 0.f, 0.f, 0.f};
        const float neg_m = -m_used;
        uint32_t buf[2][32];
        tmem_ld32(s_addr, buf[0]);
#pragma unroll
        for (int c = 0; c < F1_NC; ++c) {
          tc_wait_ld();
          if (c + 1 < F1_NC) tmem_ld32(s_addr + (c + 1) * 32, buf[(c + 1) & 1]);
          const uint32_t* v = buf[c & 1];
          float g[32];
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const float t = fmaf(__uint_as_float(v[e]), c2, neg_m);
            g[e] = (e & 3) == 3 ? ex2_fma1(t) : ex2_mufu(t);  // one exponential in four on the FMA pipe
          }
#pragma unroll
          for (int e = 0; e < 32; ++e) ls4[e & 3] += g[e];
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const typename Num<T>::T2 h2 = Num<T>::from_f2(g[2 * e], g[2 * e + 1]);
            pk[e] = *reinterpret_cast<const uint32_t*>(&h2);
          }
          // this P buffer is read by the P·V of step j - 2 until that has retired (long ago, normally)
          if (c == 0 && j >= 2 && ok) ok = mbar_wait(&pv_done[bsel], ((j - 2) >> 1) & 1, 0x5a00 | bsel, abort_flag);
          tmem_st16(p_addr + c * 16, pk);
        }
        const float part = (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
        float bad = __any_sync(0xffffffffu, !(part <= 256.f)) ? 1.f : 0.f;  // also true for inf / nan
        bad = exchange(bad, ok, false);
        if (bad == 0.f) {
          l_run += part;
          done = true;
        }
      }
      if (!done) {
        // ---- pass 1: maximum of this thread's 64 keys, then of the row
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        {
          uint32_t buf[2][32];
          tmem_ld32(s_addr, buf[0]);
#pragma unroll
          for (int c = 0; c < F1_NC; ++c) {
            tc_wait_ld();
            if (c + 1 < F1_NC) tmem_ld32(s_addr + (c + 1) * 32, buf[(c + 1) & 1]);
            const uint32_t* v = buf[c & 1];
            if (plain) {
#pragma unroll
              for (int e = 0; e < 32; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(v[e]));
            } else {
#pragma unroll
              for (int e = 0; e < 32; ++e) {
                const int jj = j0 + c * 32 + e;
                float t = __uint_as_float(v[e]) * c2;
                if (BIAS) t += alibi_table_value(p.bias_mode, slope, max(i - jj, 0)) * kLog2e1;
                if (jj > i) t = -INFINITY;
                mx4[e & 3] = fmaxf(mx4[e & 3], t);
              }
            }
          }
        }
        float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        if (plain) mx *= c2;  // c2 > 0: scaling commutes with the maximum
        mx = exchange(mx, ok, false);  // finite: every row sees key 0 .. i within its first steps
        m_run = fmaxf(m_run, mx);
        // every earlier P·V must have retired before O is rescaled or this P buffer rewritten (the
        // tensor core retires them in order, so the latest one covers the rest)
        if (j > 0 && ok) ok = mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, 0x5800, abort_flag);
        if (j == 0) {
          m_used = m_run;
        } else {
          // same values in both warps of the pair (m_run and m_used are row-wide), so the same decision
          const bool grow = (m_run - m_used) > kRescale1;
          if (__any_sync(0xffffffffu, grow)) {
            tc_fence_after();
            const float f = grow ? ex2_mufu(m_used - m_run) : 1.f;
            // each warp of the row rescales its share of the accumulator columns
#pragma unroll
            for (int cc = 0; cc < F1_OW / 32; ++cc) {
              uint32_t v[32];
              tmem_ld32(o_addr + ch * F1_OW + cc * 32, v);
              tc_wait_ld();
#pragma unroll
              for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * f);
              tmem_st32(o_addr + ch * F1_OW + cc * 32, v);
            }
            tc_wait_st();
            l_run *= f;
            if (grow) m_used = m_run;
          }
        }
        // ---- pass 2: p = 2^(s - m_used), partial row sum, P into tensor memory
        float ls4[4] = {0.f, 0.f, 0.f, 0.f};
        {
          uint32_t buf[2][32];
          tmem_ld32(s_addr, buf[0]);
#pragma unroll
          for (int c = 0; c < F1_NC; ++c) {
            tc_wait_ld();
            if (c + 1 < F1_NC) tmem_ld32(s_addr + (c + 1) * 32, buf[(c + 1) & 1]);
            const uint32_t* v = buf[c & 1];
            float g[32];
            if (plain) {
              const float neg_m = -m_used;
#pragma unroll
              for (int e = 0; e < 32; ++e) g[e] = ex2_mufu(fmaf(__uint_as_float(v[e]), c2, neg_m));
            } else {
#pragma unroll
              for (int e = 0; e < 32; ++e) {
                const int jj = j0 + c * 32 + e;
                float t = __uint_as_float(v[e]) * c2;
                if (BIAS) t += alibi_table_value(p.bias_mode, slope, max(i - jj, 0)) * kLog2e1;
                g[e] = (jj > i) ? 0.f : ex2_mufu(t - m_used);
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
      }
      const long long w2 = clock64();
      tc_wait_st();  // P is in tensor memory, the score buffer has been read
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[bsel]);
      F1_PROF(2, w1, w2);
      F1_PROF(4, w2, clock64());
      if (prof) { atomicAdd(&g_prof_f1[3], (unsigned long long)(xw_total - xw)); }
    }
    // the row sum is the sum of the pair's partial sums
    const float l_tot = exchange(l_run, ok, true);
    if (ok && mbar_wait(&pv_done[jlast & 1], (jlast >> 1) & 1, 0x5900, abort_flag)) {
      tc_fence_after();
      const float inv = 1.f / l_tot;
      T* orow = reinterpret_cast<T*>(p.out) + b * p.so_b + h * p.so_h + (int64_t)i * p.so_t + ch * F1_OW;
#pragma unroll
      for (int cc = 0; cc < F1_OW / 32; ++cc) {  // each warp of the row writes its share of the columns
        uint32_t v[32];
        tmem_ld32(o_addr + ch * F1_OW + cc * 32, v);
        tc_wait_ld();
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          float g[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) g[e] = __uint_as_float(v[v4 * 8 + e]) * inv;
          *reinterpret_cast<uint4*>(orow + cc * 32 + v4 * 8) = pack8<T>(g);
        }
      }
      if (ch == 0) p.lse[(int64_t)bh * p.T + i] = (m_used + log2f(l_tot)) * kLn2_1;
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
int attn_fwd1_tc05_status(int reset) { return read_dev_status(reset); }

// Copies the 16 cycle counters to the host and clears them.
int attn_fwd1_tc05_counters(unsigned long long* out) {
  cudaDeviceSynchronize();
  if (cudaMemcpyFromSymbol(out, g_prof_f1, sizeof(unsigned long long) * 16) != cudaSuccess) return -1;
  unsigned long long z[16] = {0};
  cudaMemcpyToSymbol(g_prof_f1, z, sizeof(z));
  return 0;
}

int encode_tmap_sw128(CUtensorMap* out, const void* base, int dtype, int rank, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box);

template <typename T, int HD>
static int fwd1_launch(const AttnArgs& a, int dtype, cudaStream_t st) {
  using Cfg = F1Cfg<HD>;
  CUtensorMap tq, tk, tv;
  int rc;
  const uint32_t box[4] = {64, 128, 1, 1};
  const uint64_t dims[4] = {(uint64_t)HD, (uint64_t)a.T, (uint64_t)a.H, (uint64_t)a.B};
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
  F1Params p;
  p.out = a.out; p.lse = a.lse; p.so_b = a.so.b; p.so_h = a.so.h; p.so_t = a.so.t;
  p.H = a.H; p.T = a.T; p.scale = a.scale; p.bias_mode = a.bias_mode; p.slopes = a.slopes;
  p.debug = g_attn_debug.load();
  static std::atomic<uint64_t> done_plain{0}, done_bias{0};
  if ((rc = ensure_dynamic_smem(attn_fwd1_tc05_kernel<T, HD, false>, Cfg::SMEM_BYTES, done_plain, "attention_fwd(tcgen05)")))
    return rc;
  if ((rc = ensure_dynamic_smem(attn_fwd1_tc05_kernel<T, HD, true>, Cfg::SMEM_BYTES, done_bias, "attention_fwd(tcgen05)")))
    return rc;
  dim3 grid(a.T / F1_TILE, a.B * a.H);
  if (a.bias_mode) launch_overlapped(attn_fwd1_tc05_kernel<T, HD, true>, grid, dim3(F1_THREADS), Cfg::SMEM_BYTES, st, tq, tk, tv, p);
  else launch_overlapped(attn_fwd1_tc05_kernel<T, HD, false>, grid, dim3(F1_THREADS), Cfg::SMEM_BYTES, st, tq, tk, tv, p);
  return launched("attention_fwd(tcgen05, doubled score buffers)");
}

int attn_fwd1_tc05(const AttnArgs& a, int hd, int dtype, cudaStream_t st) {
  TFB_DISPATCH_16(dtype, T, {
    if (hd == 64) return fwd1_launch<T, 64>(a, dtype, st);
    return fwd1_launch<T, 128>(a, dtype, st);
  })
}

}  // namespace tfb
