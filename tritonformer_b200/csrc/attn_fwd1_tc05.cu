// Causal flash attention forward on tcgen05 / TMEM: persistent CTAs, one 128-query tile at a time with its
// score buffers doubled and eight softmax warps (head_dim 64 or 128, T % 128 == 0).
//
//   warp 0      TMA producer (Q of each tile into one of two buffers, K_j / V_j tiles of 128 keys through rings)
//   warp 1      MMA issuer (one elected lane, an event loop over non-blocking barrier probes)
//   warps 2-    softmax: NW warps per TMEM lane quarter (four at head_dim 64, two at 128), each taking 128 / NW
//               of the 128 keys of a step
// One CTA per SM walks a static list of (query tile, batch*head) items: the items are ordered longest walk
// first over ALL slices and dealt to the CTAs in serpentine order, which balances the CTAs like a greedy
// longest-first schedule.  Nothing is torn down between items: the producer runs ahead into the next item's
// Q, K and V while the current item's last steps are computed, the MMA thread issues the next item's first
// scores as soon as a score buffer is free, and a finished tile is normalised and stored one step late, behind
// the first step of the next item.  (One CTA per tile, the
// earlier form, paid 1.6 k cycles of set-up, 1.8 k of waiting for the first scores and the launch gap on
// every tile: a third of the kernel at T 2048.)
// The scores of step j+1 are computed into the other score buffer while the softmax warps work on
// step j, so they go from step to step without waiting for the tensor core (with one buffer per tile
// the round trip "probabilities ready -> next scores issued -> scores landed" is a fixed 1.5 k cycles
// per step that nothing hides).  A thread owns 64 keys of one query row; the two warps of a row each keep
// an accumulator, a reference maximum and a row sum for THEIR keys and meet only twice per item, through
// shared memory (an mbarrier with one arrival per warp and lane quarter, so the wait is bounded): for the
// row maximum of the diagonal step and when the accumulators are merged.
// An item walks its key tiles from the diagonal outwards.  The diagonal tile takes two passes (row maximum,
// then probabilities) with the causal mask applied per 32-key chunk, which for a whole warp is either
// untouched, cut by the diagonal or fully masked (then nothing is computed).  Every later tile is a single
// pass against the maximum found so far (redone in two passes if a partial row sum exceeds 2^15, which also
// bounds P inside fp16/bf16 range; the accumulator row is rescaled only then), with one exponential in four
// on the FMA pipe.  With ALiBi the penalty only grows along this walk, so the first maximum holds; walking
// towards the diagonal instead, the maximum rose at every step and every step needed both passes.
// P is stored 16-bit, two keys per 32-bit column, into tensor memory, over the first half of the score columns
// it was computed from, and is the A operand of P·V.
// TMEM columns: [0,128) S0 / P0, [128,256) S1 / P1, [256, 256 + 2 head_dim) the two accumulators.
// Barrier phases run on counters that continue across items: `g` counts the steps of the CTA (score and P
// buffers alternate with g), `n` counts its items (Q buffers and accumulators alternate with n).
#include "attn.cuh"
#include "tc05.cuh"
#include <type_traits>

namespace tfb {

extern std::atomic<int> g_attn_debug;

namespace {

constexpr float kLog2e1 = 1.4426950408889634f;
constexpr float kLn2_1 = 0.6931471805599453f;
constexpr int F1_TILE = 128;
constexpr int F1_COL_S = 0;

template <int HD> struct F1Cfg {
  static constexpr int PANELS = HD / 64;                 // 64-element (128-byte) panels along head_dim
  static constexpr int TILE_BYTES = PANELS * 16384;      // 128 rows x HD x 2 B
  static constexpr int STAGES = (HD == 64) ? 3 : 2;      // K / V ring depth (shared memory bound at 128)
  // softmax warps per TMEM lane quarter, i.e. per query row: each takes KW of the 128 keys of a step
  static constexpr int NW = 2;
  static constexpr int KW = F1_TILE / NW;
  static constexpr int NC = KW / 32;                     // 32-key chunks per warp and step
  static constexpr int THREADS = 64 + 128 * NW;
  static constexpr int OW = HD / NW;                     // output columns per warp when a tile is stored
  // The NW softmax warps of a row each own an accumulator for THEIR keys of every step (column 256 + w * HD), with
  // their own reference maximum and row sum; the accumulators are merged when the tile is stored, so the warps
  // exchange values once per item instead of once per step and drift apart freely.  P (16-bit) is written over the
  // first half of the score columns it was computed from, which is what leaves tensor memory for NW accumulators.
  static constexpr int COL_O = 256;
  static constexpr int OFF_Q = 0;                                  // [2]
  static constexpr int OFF_K = 2 * TILE_BYTES;                     // [STAGES]
  static constexpr int OFF_V = OFF_K + STAGES * TILE_BYTES;        // [STAGES]
  static constexpr int OFF_X = OFF_V + STAGES * TILE_BYTES;        // row exchange: [2 parities][warps per row][128 rows] floats
  static constexpr int OFF_BAR = OFF_X + 2 * NW * 128 * 4;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  static_assert(OW % 16 == 0, "a softmax warp handles whole 16-column chunks of the accumulator");
  static_assert(COL_O + NW * HD <= 512, "tensor memory");
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory");
};
constexpr float kRescale1 = 8.0f;  // log2 units
// A single pass stands while the thread's partial row sum (an upper bound of every probability it stored)
// stays below this: inside fp16 range (65504) with room to spare.  The first maximum of a row comes from its
// share of the diagonal tile - a single key for the first row of a tile - so later tiles routinely exceed it
// by a few units; a tighter limit sent most second steps through the two-pass path.
constexpr float kSinglePassLimit = 32768.f;

struct F1Params {
  int debug;  // bit 1: cycle counters of one softmax warp (tfb_debug_set key 2); bit 5: per-slice item order
  void* out;
  float* lse;
  int64_t so_b, so_h, so_t;
  int H, T;
  int BH, group;  // batch*heads; how many of them are walked together (their K and V share the L2)
  int total;      // items: query tiles x batch*heads
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

// (f2_pack / f2_unpack / f2_fma, the packed fp32 pair arithmetic, live in common.cuh: half the instructions for the
// scale-and-shift of the scores, the polynomial of the FMA-pipe exponentials and the row sums.)
// 2^x for a pair on the FMA pipe (the polynomial of ex2_fma1, packed)
__device__ __forceinline__ void ex2_fma2(uint64_t xp, float& r0, float& r1) {
  float x0, x1;
  f2_unpack(xp, x0, x1);
  const uint64_t x = f2_pack(fmaxf(x0, -125.f), fmaxf(x1, -125.f));
  const uint64_t one = f2_pack(1.f, 1.f);
  const uint64_t xr = f2_fma(x, one, f2_pack(12582912.f, 12582912.f));
  const uint64_t fr = f2_fma(xr, one, f2_pack(-12582912.f, -12582912.f));
  const uint64_t f = f2_fma(fr, f2_pack(-1.f, -1.f), x);
  uint64_t q = f2_fma(f, f2_pack(0.0551716685f, 0.0551716685f), f2_pack(0.2426111251f, 0.2426111251f));
  q = f2_fma(q, f, f2_pack(0.6932609677f, 0.6932609677f));
  q = f2_fma(q, f, f2_pack(0.9999280572f, 0.9999280572f));
  float q0, q1, xr0, xr1;
  f2_unpack(q, q0, q1);
  f2_unpack(xr, xr0, xr1);
  r0 = __int_as_float(__float_as_int(q0) + (__float_as_int(xr0) << 23));
  r1 = __int_as_float(__float_as_int(q1) + (__float_as_int(xr1) << 23));
}

// The n-th item of this CTA: query tile and batch*head slice.  Items are numbered longest walk first across
// the slices of a group (groups keep the K and V that are live at one time within the L2); round n of the
// deal goes over the CTAs forwards when n is even and backwards when it is odd.  False past the last item
// (and then for every later n as well).
__device__ __forceinline__ bool f1_item(const F1Params& p, int n, int& qt, int& bh) {
  const int G = (int)gridDim.x, c = (int)blockIdx.x;
  const int v = n * G + ((n & 1) ? (G - 1 - c) : c);
  if (v >= p.total) return false;
  const int nt = p.T / F1_TILE;
  if (p.debug & 32) {  // per-slice order (test switch)
    qt = (nt - 1) - v % nt;
    bh = v / nt;
  } else {
    const int g = v / (nt * p.group), r = v % (nt * p.group);
    const int gsz = min(p.group, p.BH - g * p.group);
    qt = (nt - 1) - r / gsz;
    bh = g * p.group + r % gsz;
  }
  return true;
}

}  // namespace

// [0] steps, [1] wait for scores, [2] pass, [3] row-pair exchange, [4] store fence + arrive (warp 2, lane 0);
// per CTA: [5] items, [6] lifetime of the CTA, [7] entry -> set-up done, [8] first (diagonal) step of an item,
// [9] its second step, [10] single passes that had to be redone, [11] normalisation and store of an item, [12] lifetime in ns
static __device__ unsigned long long g_prof_f1[16];
#define F1_PROF(idx, t0, t1) do { if (prof) atomicAdd(&g_prof_f1[idx], (unsigned long long)((t1) - (t0))); } while (0)

template <typename T, int HD, int BIAS>
__global__ void __launch_bounds__(F1Cfg<HD>::THREADS, 1) attn_fwd1_tc05_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                                       const __grid_constant__ CUtensorMap tmK,
                                                                       const __grid_constant__ CUtensorMap tmV,
                                                                       const F1Params p) {
  using Cfg = F1Cfg<HD>;
  constexpr int F1_STAGES = Cfg::STAGES, F1_TILE_BYTES = Cfg::TILE_BYTES, F1_OW = Cfg::OW;
  constexpr int F1_NW = Cfg::NW, F1_KW = Cfg::KW, F1_NC = Cfg::NC, F1_COL_O = Cfg::COL_O;
  constexpr int KSTEPS = (F1_TILE / 16) / F1_NW;  // P.V instructions per softmax warp's share of the keys
  constexpr int F1_OFF_Q = Cfg::OFF_Q, F1_OFF_K = Cfg::OFF_K, F1_OFF_V = Cfg::OFF_V, F1_OFF_X = Cfg::OFF_X;
  constexpr int F1_OFF_BAR = Cfg::OFF_BAR;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + F1_OFF_BAR);
  uint64_t* q_full = bars + 0;                   // [2 buffers] Q of an item has landed
  uint64_t* q_empty = q_full + 2;                // [2 buffers] the item's last score product has retired
  uint64_t* k_full = q_empty + 2;                // [STAGES]
  uint64_t* k_empty = k_full + F1_STAGES;        // [STAGES]
  uint64_t* v_full = k_empty + F1_STAGES;        // [STAGES]
  uint64_t* v_empty = v_full + F1_STAGES;        // [STAGES]
  uint64_t* s_full = v_empty + F1_STAGES;        // [2 buffers] scores of a step are in TMEM
  uint64_t* p_full = s_full + 2;                 // [2 buffers] probabilities stored, score buffer read (8 warps)
  uint64_t* pv_done = p_full + 2;                // [2 buffers] the P·V that read the P buffer has retired
  uint64_t* o_free = pv_done + 2;                // [2 accumulators] the finished tile has been read out (8 warps)
  uint64_t* pair_bar = o_free + 2;               // [4 lane quarters] both warps of the row pair have published
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(pair_bar + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  float* xch = reinterpret_cast<float*>(smem + F1_OFF_X);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long t_entry = clock64();
  const uint64_t ns_entry = global_ns();

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4 * F1_NW);
      mbar_init(&pv_done[i], 1);
      mbar_init(&o_free[i], 4 * F1_NW);
    }
    for (int i = 0; i < F1_STAGES; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
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
      int st = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int n = 0; ok; ++n) {
        int qt, bh;
        if (!f1_item(p, n, qt, bh)) break;
        const int b = bh / p.H, h = bh % p.H;
        const int qb = n & 1;
        // the Q buffer was read by the score products of item n - 2
        if (n >= 2 && !mbar_wait(&q_empty[qb], ((n - 2) >> 1) & 1, 0x5000 | qb, abort_flag)) break;
        mbar_expect_tx(&q_full[qb], F1_TILE_BYTES);
#pragma unroll
        for (int c = 0; c < Cfg::PANELS; ++c)
          tma_load_4d(smem + F1_OFF_Q + qb * F1_TILE_BYTES + c * 16384, &tmQ, c * 64, qt * F1_TILE, h, b, &q_full[qb]);
        for (int j = qt; j >= 0; --j) {  // key tiles from the diagonal outwards
          if (!mbar_wait(&k_empty[st], ph ^ 1, 0x5100 | st, abort_flag)) { ok = false; break; }
          mbar_expect_tx(&k_full[st], F1_TILE_BYTES);
#pragma unroll
          for (int c = 0; c < Cfg::PANELS; ++c)
            tma_load_4d(smem + F1_OFF_K + st * F1_TILE_BYTES + c * 16384, &tmK, c * 64, j * F1_TILE, h, b, &k_full[st]);
          if (!mbar_wait(&v_empty[st], ph ^ 1, 0x5200 | st, abort_flag)) { ok = false; break; }
          mbar_expect_tx(&v_full[st], F1_TILE_BYTES);
#pragma unroll
          for (int c = 0; c < Cfg::PANELS; ++c)
            tma_load_4d(smem + F1_OFF_V + st * F1_TILE_BYTES + c * 16384, &tmV, c * 64, j * F1_TILE, h, b, &v_full[st]);
          if (++st == F1_STAGES) { st = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ----------------------------------------------------------------------- MMA issuer
    // The whole warp runs the loop and one elected lane issues each tcgen05 instruction: warp-uniform code keeps
    // the operand descriptors in uniform registers, where the tensor core reads them; with the loop in a single
    // lane every instruction paid for moving them there (63 against 49 cycles per M128 N64 K16 instruction).
    if (!dead) {
      constexpr int fmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t idesc_s = instr_desc_f16(128, 128, fmt, 0, 0);
      constexpr uint32_t idesc_o = instr_desc_f16(128, HD, fmt, 0, 1);
      const uint32_t tb = __shfl_sync(0xffffffffu, tmem_base, 0);  // read from shared memory: tell the compiler it is uniform
      const uint32_t s0 = smem_u32(smem);
      auto ready = [&](uint64_t* bar, uint32_t parity) -> bool { return __all_sync(0xffffffffu, mbar_test(bar, parity)) != 0; };
      // Event loop over two cursors: the next scores go out as soon as their buffer has been read (two
      // steps back), K has landed and, for the first step of an item, its Q; the product with V as soon
      // as P is stored, V has landed and, for the first step of an item, its accumulator has been read out.
      int sn = 0, sj = 0, sg = 0, s_last = 0, s_bh;   // scores: item, step, step count of the CTA, last step
      int pn = 0, pj = 0, pg = 0, p_last = 0, p_bh;   // P·V
      bool s_valid = f1_item(p, 0, s_last, s_bh);
      bool p_valid = s_valid;
      p_last = s_last;
      int ks = 0, vs = 0;            // ring stage of that step's K / V
      uint32_t kph = 0, vph = 0;     // ring phase of that step's K / V
      bool ok = true;
      uint64_t t_idle = global_ns();
      while (ok && p_valid) {
        bool progress = false;
        // (P in the score columns: the product that reads P of two steps ago must be in the pipe before these
        // scores, which overwrite it; the tensor core runs them in the order of issue)
        if (s_valid && (sg < 2 || (pg > sg - 2 && ready(&p_full[sg & 1], ((sg - 2) >> 1) & 1))) &&
            ready(&k_full[ks], kph) &&
            (sj > 0 || ready(&q_full[sn & 1], (sn >> 1) & 1))) {
          tc_fence_after();
          const uint64_t dq = smem_desc_sw128(s0 + F1_OFF_Q + (sn & 1) * F1_TILE_BYTES, 16, 1024);
          const uint64_t dk = smem_desc_sw128(s0 + F1_OFF_K + ks * F1_TILE_BYTES, 16, 1024);
#pragma unroll
          for (int s = 0; s < HD / 16; ++s) {
            const uint32_t off = (s / 4) * 16384 + (s % 4) * 32;  // 64-element panel, then 32 bytes per k-step
            if (elect_one())
              tc_mma_ss(tb + F1_COL_S + (sg & 1) * 128, desc_advance(dq, off), desc_advance(dk, off), idesc_s, s ? 1u : 0u);
          }
          if (elect_one()) {
            tc_commit(&s_full[sg & 1]);
            tc_commit(&k_empty[ks]);
            if (sj == s_last) tc_commit(&q_empty[sn & 1]);
          }
          if (++ks == F1_STAGES) { ks = 0; kph ^= 1; }
          ++sg;
          if (sj == s_last) {
            ++sn;
            sj = 0;
            s_valid = f1_item(p, sn, s_last, s_bh);
          } else {
            ++sj;
          }
          progress = true;
        }
        if (ready(&p_full[pg & 1], (pg >> 1) & 1) && ready(&v_full[vs], vph) &&
            (pj > 0 || pn < 1 || ready(&o_free[0], (pn - 1) & 1))) {
          tc_fence_after();
          // A = P from tensor memory (a lane is a query row, a 32-bit column holds two consecutive
          // keys), B = V_j from shared memory
          const uint64_t dv = smem_desc_sw128(s0 + F1_OFF_V + vs * F1_TILE_BYTES, 16384, 1024);
          const uint32_t tp = tb + F1_COL_S + (pg & 1) * 128;
          const uint32_t to = tb + F1_COL_O;
#pragma unroll
          for (int s = 0; s < F1_TILE / 16; ++s) {
            // split accumulators: each softmax warp's share of the keys (KSTEPS instructions) has its own
            const uint32_t acc = to + (s / KSTEPS) * HD;
            const uint32_t add = (pj | (s % KSTEPS)) ? 1u : 0u;
            const uint32_t pa = tp + (s / KSTEPS) * F1_KW + (s % KSTEPS) * 8;  // P sits at the head of its warp's score columns
            if (elect_one()) tc_mma_ts(acc, pa, desc_advance(dv, s * 2048), idesc_o, add);
          }
          if (elect_one()) {
            tc_commit(&pv_done[pg & 1]);
            tc_commit(&v_empty[vs]);
          }
          if (++vs == F1_STAGES) { vs = 0; vph ^= 1; }
          ++pg;
          if (pj == p_last) {
            ++pn;
            pj = 0;
            p_valid = f1_item(p, pn, p_last, p_bh);
          } else {
            ++pj;
          }
          progress = true;
        }
        if (progress) {
          t_idle = global_ns();
        } else if (__any_sync(0xffffffffu, *abort_flag != 0)) {
          ok = false;
        } else if (__any_sync(0xffffffffu, global_ns() - t_idle > kWaitLimitNs)) {
          if (lane == 0) {
            *abort_flag = 1;
            atomicCAS(&g_dev_status, 0, 0x5500);
          }
          ok = false;
        } else {
          __nanosleep(20);
        }
      }
      __syncwarp();
    }
  } else if (!dead) {
    // -------------------------------------------------------------------------- softmax
    const int qd = warp & 3;            // TMEM lane quarter
    const int ch = (warp - 2) >> 2;     // which F1_KW of the step's 128 keys
    const int r = qd * 32 + lane;       // row within the tile == TMEM lane
    const uint32_t lane_addr = tmem_base + ((uint32_t)(qd * 32) << 16);
    const float c2 = p.scale * kLog2e1;
    uint32_t pair_phase = 0;
    int xpar = 0;
    bool ok = true;
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
    // the same hand-shake, returning the value of every warp of the row, in warp order
    auto gather = [&](float mine, bool& fine, float (&all)[F1_NW]) {
      float* slot = xch + xpar * (F1_NW * 128);
      slot[ch * 128 + r] = mine;
      __syncwarp();
      if (lane == 0) mbar_arrive(&pair_bar[qd]);
      if (fine) fine = mbar_wait(&pair_bar[qd], pair_phase, 0x5d00 | qd, abort_flag);
      pair_phase ^= 1;
#pragma unroll
      for (int w = 0; w < F1_NW; ++w) all[w] = slot[w * 128 + r];
      xpar ^= 1;
    };
    const bool prof = (p.debug & 2) && warp == 2 + ((p.debug >> 8) & 15) && lane == 0;  // bits 8-11: which softmax warp
    if (prof) atomicAdd(&g_prof_f1[7], (unsigned long long)(clock64() - t_entry));
    int g0 = 0;  // steps of the CTA before this item
    long long last_w3 = clock64();
    // Normalisation and store of a finished tile, run one step late: after the first (diagonal) step of the NEXT
    // item, whose scores are already there, so that the wait for the tile's last P·V is hidden behind that step.
    bool pend = false;
    int pend_glast = 0;
    float pend_l = 1.f, pend_m = 0.f;
    float pend_w[F1_NW];  // (split accumulators: their weights)
#pragma unroll
    for (int w = 0; w < F1_NW; ++w) pend_w[w] = 1.f;
    T* pend_row = nullptr;
    float* pend_lse = nullptr;
    auto finish_pending = [&]() {
      if (!pend) return;
      pend = false;
      const long long f0 = clock64();
      if (ok) ok = mbar_wait(&pv_done[pend_glast & 1], (pend_glast >> 1) & 1, 0x5900, abort_flag);
      if (ok) {
        tc_fence_after();
        const float inv = 1.f / pend_l;
        const uint32_t o_addr = lane_addr + F1_COL_O;
        {
          // this warp's OW output columns of every accumulator, each weighted back to the common maximum
          float acc[F1_OW];
#pragma unroll
          for (int e = 0; e < F1_OW; ++e) acc[e] = 0.f;
#pragma unroll
          for (int w = 0; w < F1_NW; ++w) {
            uint32_t v[F1_OW / 16][16];
#pragma unroll
            for (int cc = 0; cc < F1_OW / 16; ++cc) tmem_ld16(o_addr + w * HD + ch * F1_OW + cc * 16, v[cc]);
            tc_wait_ld();
#pragma unroll
            for (int e = 0; e < F1_OW; ++e) acc[e] = fmaf(__uint_as_float(v[e / 16][e % 16]), pend_w[w], acc[e]);
          }
          // the accumulators have been read out: the first product of a later item may overwrite them
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&o_free[0]);
#pragma unroll
          for (int v8 = 0; v8 < F1_OW / 8; ++v8) {
            float o8[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) o8[e] = acc[v8 * 8 + e] * inv;
            *reinterpret_cast<uint4*>(pend_row + v8 * 8) = pack8<T>(o8);
          }
        }
        if (ch == 0) *pend_lse = (pend_m + log2f(pend_l)) * kLn2_1;
      }
      if (prof) atomicAdd(&g_prof_f1[11], (unsigned long long)(clock64() - f0));
    };
    for (int n = 0; ok; ++n) {
      int qt, bh;
      if (!f1_item(p, n, qt, bh)) break;
      const int b = bh / p.H, h = bh % p.H;
      const int jlast = qt;               // last key tile this query tile attends to
      const int i = qt * F1_TILE + r;     // query
      // the accumulator this warp rescales: its own (split) or its share of the columns of the common one
      const uint32_t o_addr = lane_addr + F1_COL_O + ch * HD;
      constexpr int RESCALE_COLS = HD;
      const AlibiLog2<BIAS> alibi(BIAS ? p.slopes[h] : 0.f);
      float m_run = -INFINITY;   // true running maximum of the row (both halves)
      float m_used = -INFINITY;  // maximum the accumulator and the running sums are expressed against
      float l_run = 0.f;         // this thread's partial row sum (its 64 keys of every step)
      for (int t = 0; t <= jlast; ++t) {
        const int j = jlast - t;                  // key tile: the diagonal first, then outwards
        const int g = g0 + t;
        const int bsel = g & 1;
        const int kbase = j * F1_TILE + ch * F1_KW;  // first key of this thread's share
        const bool diag = (t == 0);
        const uint32_t s_addr = lane_addr + F1_COL_S + bsel * 128 + ch * F1_KW;
        // P of a 32-key chunk: 16 columns, at head_dim 64 the first 16 of this warp's own score columns
        const uint32_t p_addr = s_addr;
        const long long w0 = clock64();
        F1_PROF(14, last_w3, w0);
        if (ok) ok = mbar_wait(&s_full[bsel], (g >> 1) & 1, 0x5700 | bsel, abort_flag);
        const long long w1 = clock64();
        F1_PROF(1, w0, w1);
        if (prof) atomicAdd(&g_prof_f1[0], 1ull);
        const long long xw = xw_total;  // exchange cycles before this step
        tc_fence_after();
        bool done = false;
        if (!diag) {
          // ---- single pass against the maximum of the earlier steps (the diagonal tile and, with ALiBi,
          // the tiles with the smallest penalty came first).  No maximum is tracked here: a probability is
          // at most this thread's partial row sum, so while that stays below 2^8 the 16-bit range holds;
          // otherwise (rare) the step is redone in two passes with a fresh maximum.  The two warps of a
          // row pair exchange the verdict.
          uint64_t ls2[2] = {0ull, 0ull};  // four partial row sums in two register pairs
          const float neg_m = -m_used;
          const uint64_t c2p = f2_pack(c2, c2), negmp = f2_pack(neg_m, neg_m), onep = f2_pack(1.f, 1.f);
          uint32_t buf[2][32];
          uint32_t pk_all[F1_NC][16];  // P goes over the scores: stored once the pass is known to stand
          tmem_ld32(s_addr, buf[0]);
#pragma unroll
          for (int c = 0; c < F1_NC; ++c) {
            tc_wait_ld();
            if (c + 1 < F1_NC) tmem_ld32(s_addr + (c + 1) * 32, buf[(c + 1) & 1]);
            const uint32_t* v = buf[c & 1];
            const float d0 = (float)(i - (kbase + c * 32));  // distance of the chunk's first key
            uint32_t (&pk)[16] = pk_all[c];
#pragma unroll
            for (int e2 = 0; e2 < 16; ++e2) {  // pairs of keys
              uint64_t xp = f2_fma(f2_pack(__uint_as_float(v[2 * e2]), __uint_as_float(v[2 * e2 + 1])), c2p, negmp);
              float p0, p1;
              if (BIAS) {
                float x0, x1;
                f2_unpack(xp, x0, x1);
                xp = f2_pack(alibi.sub_from(x0, d0 - (float)(2 * e2)), alibi.sub_from(x1, d0 - (float)(2 * e2 + 1)));
              }
              if ((e2 & 3) == 3) {  // one pair in four on the FMA pipe
                ex2_fma2(xp, p0, p1);
              } else {
                float x0, x1;
                f2_unpack(xp, x0, x1);
                p0 = ex2_mufu(x0);
                p1 = ex2_mufu(x1);
              }
              ls2[e2 & 1] = f2_fma(f2_pack(p0, p1), onep, ls2[e2 & 1]);
              const typename Num<T>::T2 h2 = Num<T>::from_f2(p0, p1);
              pk[e2] = *reinterpret_cast<const uint32_t*>(&h2);
            }
          }
          float ls4[4];
          f2_unpack(ls2[0], ls4[0], ls4[1]);
          f2_unpack(ls2[1], ls4[2], ls4[3]);
          const float part = (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
          float bad = __any_sync(0xffffffffu, !(part <= kSinglePassLimit)) ? 1.f : 0.f;  // also true for inf / nan
          if (bad == 0.f) {
#pragma unroll
            for (int c = 0; c < F1_NC; ++c) tmem_st16(p_addr + c * 16, pk_all[c]);
            l_run += part;
            done = true;
          } else if (prof) {
            atomicAdd(&g_prof_f1[10], 1ull);
          }
        }
        if (!done) {
          // ---- two passes with a fresh maximum: the diagonal tile of every item, and a step whose single
          // pass overflowed.  On the diagonal a 32-key chunk is, for the whole warp, either fully allowed,
          // fully masked (nothing to compute: P = 0) or cut by the diagonal (per-element mask).
          int cls[F1_NC];  // 0 full, 1 cut, 2 masked
          int cnt[F1_NC];  // allowed keys of this row in the chunk (may be <= 0 or >= 32)
#pragma unroll
          for (int c = 0; c < F1_NC; ++c) {
            cnt[c] = i - (kbase + c * 32) + 1;
            const int lo = __shfl_sync(0xffffffffu, cnt[c], 0), hi = __shfl_sync(0xffffffffu, cnt[c], 31);
            cls[c] = !diag ? 0 : (hi <= 0 ? 2 : (lo >= 32 ? 0 : 1));
          }
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
              if (cls[c] == 2) continue;
              if (!BIAS && cls[c] == 0) {
#pragma unroll
                for (int e = 0; e < 32; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(v[e]) * c2);
              } else {
                const float d0 = (float)(i - (kbase + c * 32));
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                  float x = alibi.sub_from(__uint_as_float(v[e]) * c2, d0 - (float)e);  // masked keys: overwritten
                  if (e >= cnt[c]) x = -INFINITY;
                  mx4[e & 3] = fmaxf(mx4[e & 3], x);
                }
              }
            }
          }
          float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
          // finite after the exchange: the diagonal tile holds key i of every row.  Split accumulators: only the
          // diagonal step needs the partner (a warp whose share of the diagonal tile is masked has no maximum of
          // its own yet); a redone step further out concerns this warp's accumulator alone.
          if (t == 0) mx = exchange(mx, ok, false);
          m_run = fmaxf(m_run, mx);
          // every earlier P·V must have retired before O is rescaled or this P buffer rewritten (the
          // tensor core retires them in order, so the latest one covers the rest; at the first step of an
          // item that is the previous item's last product, which this warp has already waited for)
          // (the first step of an item rescales nothing and only rewrites the P buffer, which the product of two
          // steps ago read: it does not wait for the previous item's last product, whose tile is still pending)
          if (t == 0) {
            if (g >= 2 && ok) ok = mbar_wait(&pv_done[bsel], ((g - 2) >> 1) & 1, 0x5a80 | bsel, abort_flag);
          } else if (ok) {
            ok = mbar_wait(&pv_done[(g - 1) & 1], ((g - 1) >> 1) & 1, 0x5800, abort_flag);
          }
          if (t == 0) {
            m_used = m_run;
          } else {
            // same values in both warps of the pair (m_run and m_used are row-wide), so the same decision
            const bool grow = (m_run - m_used) > kRescale1;
            if (__any_sync(0xffffffffu, grow)) {
              tc_fence_after();
              const float f = grow ? ex2_mufu(m_used - m_run) : 1.f;
              // each warp of the row rescales its share of the accumulator columns
#pragma unroll
              for (int cc = 0; cc < RESCALE_COLS / 32; ++cc) {
                uint32_t v[32];
                tmem_ld32(o_addr + cc * 32, v);
                tc_wait_ld();
#pragma unroll
                for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * f);
                tmem_st32(o_addr + cc * 32, v);
              }
              tc_wait_st();
              l_run *= f;
              if (grow) m_used = m_run;
            }
          }
          // ---- pass 2: p = 2^(s - m_used), partial row sum, P into tensor memory
          float ls4[4] = {0.f, 0.f, 0.f, 0.f};
          {
            const float neg_m = -m_used;
            uint32_t buf[2][32];
            tmem_ld32(s_addr, buf[0]);
#pragma unroll
            for (int c = 0; c < F1_NC; ++c) {
              tc_wait_ld();
              if (c + 1 < F1_NC) tmem_ld32(s_addr + (c + 1) * 32, buf[(c + 1) & 1]);
              const uint32_t* v = buf[c & 1];
              uint32_t pk[16];
              if (cls[c] == 2) {
#pragma unroll
                for (int e = 0; e < 16; ++e) pk[e] = 0u;
              } else {
                float e_[32];
                if (!BIAS && cls[c] == 0) {
#pragma unroll
                  for (int e = 0; e < 32; ++e) e_[e] = ex2_mufu(fmaf(__uint_as_float(v[e]), c2, neg_m));
                } else {
                  const float d0 = (float)(i - (kbase + c * 32));
#pragma unroll
                  for (int e = 0; e < 32; ++e) {
                    const float x = alibi.sub_from(fmaf(__uint_as_float(v[e]), c2, neg_m), d0 - (float)e);
                    e_[e] = (e >= cnt[c]) ? 0.f : ex2_mufu(x);
                  }
                }
#pragma unroll
                for (int e = 0; e < 32; ++e) ls4[e & 3] += e_[e];
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                  const typename Num<T>::T2 h2 = Num<T>::from_f2(e_[2 * e], e_[2 * e + 1]);
                  pk[e] = *reinterpret_cast<const uint32_t*>(&h2);
                }
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
        const long long w3 = clock64();
        F1_PROF(4, w2, w3);
        last_w3 = w3;
        if (prof) {
          atomicAdd(&g_prof_f1[3], (unsigned long long)(xw_total - xw));
          if (t == 0) atomicAdd(&g_prof_f1[8], (unsigned long long)(w3 - w0));
          if (t == 1) atomicAdd(&g_prof_f1[9], (unsigned long long)(w3 - w0));
        }
        if (t == 0) finish_pending();  // the previous item's tile
      }
      // the row sum is the sum of the pair's partial sums; the tile itself is finished one step later
      {
        // merge the two streams: common maximum, each stream's weight against it, common row sum
        float m_w[F1_NW], l_w[F1_NW];
        const long long g0_ = clock64();
        gather(m_used, ok, m_w);
        gather(l_run, ok, l_w);
        if (prof) atomicAdd(&g_prof_f1[13], (unsigned long long)(clock64() - g0_));
        float m_all = m_w[0];
#pragma unroll
        for (int w = 1; w < F1_NW; ++w) m_all = fmaxf(m_all, m_w[w]);
        pend_l = 0.f;
#pragma unroll
        for (int w = 0; w < F1_NW; ++w) {
          pend_w[w] = ex2_mufu(m_w[w] - m_all);
          pend_l = fmaf(l_w[w], pend_w[w], pend_l);
        }
        pend_m = m_all;
      }
      pend_glast = g0 + jlast;
      pend_row = reinterpret_cast<T*>(p.out) + b * p.so_b + h * p.so_h + (int64_t)i * p.so_t + ch * F1_OW;
      pend_lse = p.lse + (int64_t)bh * p.T + i;
      pend = true;
      g0 += jlast + 1;
      if (prof) atomicAdd(&g_prof_f1[5], 1ull);
    }
    finish_pending();  // the CTA's last tile
    if (prof) {
      atomicAdd(&g_prof_f1[6], (unsigned long long)(clock64() - t_entry));
      atomicAdd(&g_prof_f1[12], (unsigned long long)(global_ns() - ns_entry));
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
  p.BH = a.B * a.H;
  p.group = attn_slices_per_group(a.B * a.H, a.T, HD);
  p.total = (a.T / F1_TILE) * a.B * a.H;
  const int sms = sm_count();
  if (sms <= 0) return fail(TFB_ERR_LAUNCH, "attention_fwd(tcgen05): cannot read the SM count");
  dim3 grid(p.total < sms ? p.total : sms);  // one persistent CTA per SM
  static std::atomic<uint64_t> done[4] = {{0}, {0}, {0}, {0}};
#define F1_LAUNCH(MODE, SLOT)                                                                                        \
  {                                                                                                                  \
    if ((rc = ensure_dynamic_smem(attn_fwd1_tc05_kernel<T, HD, MODE>, Cfg::SMEM_BYTES, done[SLOT],                   \
                                  "attention_fwd(tcgen05)")))                                                        \
      return rc;                                                                                                     \
    launch_overlapped(attn_fwd1_tc05_kernel<T, HD, MODE>, grid, dim3(Cfg::THREADS), Cfg::SMEM_BYTES, st, tq, tk, tv, p); \
  }
  if (a.bias_mode == 0) F1_LAUNCH(0, 0)
  else if (a.bias_mode == 1) F1_LAUNCH(1, 1)
  else if (a.bias_mode == 2) F1_LAUNCH(2, 2)
  else F1_LAUNCH(4, 3)
#undef F1_LAUNCH
  return launched("attention_fwd(tcgen05, persistent)");
}

// The tcgen05 forward takes head_dim 64 / 128, whole 128-query tiles and no dense bias table.
bool attn_tc05_fwd_eligible(const AttnArgs& a, int hd) {
  return (hd == 64 || hd == 128) && a.T % 128 == 0 && a.bias_mode != 3;
}

int attn_fwd1_tc05(const AttnArgs& a, int hd, int dtype, cudaStream_t st) {
  TFB_DISPATCH_16(dtype, T, {
    if (hd == 64) return fwd1_launch<T, 64>(a, dtype, st);
    return fwd1_launch<T, 128>(a, dtype, st);
  })
}

}  // namespace tfb
