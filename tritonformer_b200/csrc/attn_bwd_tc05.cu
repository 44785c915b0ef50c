// Causal flash attention backward on tcgen05 / TMEM for sm_100a (head_dim 64 or 128, T % 128 == 0).
//
// One CTA per (128-key tile, batch*head); it walks the query tiles at or below the diagonal.
// Everything is computed transposed (rows = keys) so that the per-query statistics (log-sum-exp,
// delta) are per-column constants and no row reductions are needed:
//   Sᵀ  = K Q_iᵀ                 dPᵀ = V dO_iᵀ                      (tensor cores -> TMEM)
//   Pᵀ  = 2^(Sᵀ·c + bias - lse)  dSᵀ = Pᵀ ∘ (dPᵀ - delta)            (compute warps -> smem, 16 bit)
//   dV += Pᵀ dO_i     dK += dSᵀ Q_i     dQ_i = dS K                  (tensor cores -> TMEM)
// dV and dK stay in TMEM for the whole walk; dQ_i is added to an fp32 global accumulator (TMA
// reduce-add) because every key tile contributes to it; a small kernel scales and rounds the
// accumulator afterwards.
// A 128 x 64 swizzled panel of 16-bit values is at the same time a K-major operand with 128 rows
// and an MN-major operand with 128 contraction rows, so each of K, V, Q_i, dO_i, dSᵀ sits in
// shared memory once and serves two products.
//
// Roles: warp 0 TMA producer, warp 1 MMA issuer, warps 2-17 compute (thread = TMEM lane, four
// warps per lane quarter, each taking a quarter of the columns), warps 18-21 drain dQ_i.
// At head_dim 64, Pᵀ goes into the 64 TMEM columns that are left instead of shared memory and is
// the A operand of the dV product.
// At head_dim 64 the scores of tile i+1 are issued as soon as the compute warps hold the scores of tile i in
// registers, ahead of the gradient products of tile i, so the compute warps find them ready and work on tile
// i+1 while the tensor core finishes tile i.
// TMEM columns: [0,128) Sᵀ; [128,256) dPᵀ; [256,256+hd) dV; then dK; then dQ_i (at head_dim 128
// dQ_i reuses the Sᵀ columns).
#include "attn.cuh"
#include "tc05.cuh"
#include <type_traits>

namespace tfb {

extern std::atomic<int> g_attn_debug;

constexpr float kLog2eB = 1.4426950408889634f;
constexpr int FB_T = 128;           // tile edge (keys and queries)
constexpr int FB_CWARPS = 16;        // compute warps: 4 TMEM lane quarters x 4 column quarters
constexpr int FB_THREADS = 64 + 32 * FB_CWARPS + 128;  // TMA, MMA, compute warps, 4 dQ-drain warps
constexpr int FB_COMPUTE = 256;     // threads in the compute warps

template <int HD> struct FbCfg {
  static constexpr int PANELS = HD / 64;
  static constexpr int TILE_BYTES = PANELS * 16384;   // 128 rows x HD x 2 B
  // Query-side ring depth.  head_dim 64 needs three stages: the gradient products of tile i-1 still read their
  // Q / dO while the scores of tile i+1 are issued (with two, the load of tile i+1 could only start when tile
  // i-1 had retired, and its latency showed up as a wait for scores on every tile).  Pᵀ lives in tensor memory
  // there, so its shared-memory buffer is not allocated and the third stage takes its place.  One stage at
  // head_dim 128 (shared memory).
  static constexpr int QSTAGES = (HD == 64) ? 3 : 1;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = TILE_BYTES;
  static constexpr int OFF_Q = 2 * TILE_BYTES;                       // [QSTAGES]
  static constexpr int OFF_DO = OFF_Q + QSTAGES * TILE_BYTES;        // [QSTAGES]
  static constexpr int OFF_P = OFF_DO + QSTAGES * TILE_BYTES;        // Pᵀ  128 x 128 x 2 B (head_dim 128 only)
  static constexpr int OFF_DS = OFF_P + ((256 + 3 * HD + 64 <= 512) ? 0 : 32768);  // dSᵀ 128 x 128 x 2 B
  static constexpr int OFF_STAT = OFF_DS + 32768;                    // [2 parities][16 compute warps][lse2[32], delta[32]] fp32
  // dQ_i staging for the TMA reduction: boxes of 32 rows x 128 B, one per drain warp and 32-column chunk.  At
  // head_dim 64 they have shared memory of their own (two per warp).  At head_dim 128 there is none left, and the
  // sixteen boxes are the Pᵀ / dSᵀ buffers themselves: between the last gradient product of a tile and the
  // compute warps' next write nothing else uses them.
  static constexpr bool DQ_TMA = true;
  static constexpr bool DQ_IN_PDS = (HD == 128);
  static constexpr int DQ_BOXES = (HD == 64) ? 2 : 0;
  static constexpr int OFF_DQ = OFF_STAT + 8192;
  static constexpr int OFF_BAR = OFF_DQ + 4 * DQ_BOXES * 4096;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory");
  static constexpr int COL_S = 0, COL_DP = 128, COL_DV = 256, COL_DK = 256 + HD;
  // dQ_i has columns of its own when they fit (hd 64); otherwise it reuses the Sᵀ columns
  static constexpr bool DQ_ALIASED = (256 + 3 * HD > 512);
  static constexpr int COL_DQ = DQ_ALIASED ? 0 : 256 + 2 * HD;
  // Pᵀ (16-bit, two queries per column) lives in tensor memory when 64 columns are left for it (hd 64):
  // it is the A operand of the dV product, which then reads only dO from shared memory
  static constexpr bool P_TMEM = (256 + 3 * HD + 64 <= 512);
  static constexpr int COL_PT = 256 + 3 * HD;
};

struct FbParams {
  const float* lse;
  const float* delta;
  float* dq_acc;  // (B,H,T,HD) fp32, zero on entry
  void *dk, *dv;
  int64_t sdk_b, sdk_h, sdk_t, sdv_b, sdv_h, sdv_t;
  int H, T;
  int BH, group;  // batch*heads; how many of them are walked together (their tiles share the L2)
  float scale;
  int bias_mode;
  const float* slopes;
  int debug;  // test switch: bit 0 skips the dQ accumulation (timing experiments only)
};

// Cycle counters for the timing switch (debug bit 1): [0] CTA iterations, [1..5] compute warp 2:
// wait scores, math, wait previous products, smem write, barrier+stats; [6..9] MMA thread: wait P/dS,
// wait Q/dO, wait dQ drain, total; [10,11] drain warp: wait, drain; [12] / [15] MMA thread: time to issue the
// score products / the gradient products of a tile.
static __device__ unsigned long long g_prof[16];
#define PROF_T(var) long long var = prof ? clock64() : 0
#define PROF_ADD(idx, t0, t1) do { if (prof) atomicAdd(&g_prof[idx], (unsigned long long)((t1) - (t0))); } while (0)

__device__ __forceinline__ float ex2_approx_b(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  typename Num<T>::T2 h = Num<T>::from_f2(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <typename T, int HD, int BIAS>
__global__ void __launch_bounds__(FB_THREADS, 1) attn_bwd_tc05_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                                      const __grid_constant__ CUtensorMap tmK,
                                                                      const __grid_constant__ CUtensorMap tmV,
                                                                      const __grid_constant__ CUtensorMap tmDO,
                                                                      const __grid_constant__ CUtensorMap tmDQ,
                                                                      const FbParams p) {
  using Cfg = FbCfg<HD>;
  constexpr int QS = Cfg::QSTAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* s_stat = reinterpret_cast<float*>(smem + Cfg::OFF_STAT);  // [2 parities][16 warps][lse2[32], delta[32]]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* kv_full = bars + 0;
  uint64_t* q_full = bars + 1;    // [3] Q_i and dO_i landed
  uint64_t* q_empty = bars + 4;   // [3] products reading them retired
  uint64_t* s_full = bars + 7;    // Sᵀ and dPᵀ in TMEM
  uint64_t* pds_full = bars + 8;  // Pᵀ and dSᵀ in smem (and Sᵀ, dPᵀ consumed)
  uint64_t* dq_full = bars + 9;   // dV, dK, dQ_i products retired
  uint64_t* dq_free = bars + 10;  // dQ_i read out of TMEM
  uint64_t* s_free = bars + 11;   // Sᵀ and dPᵀ read out of TMEM (head_dim 64: the next scores may overwrite them)
  uint64_t* stage_free = bars + 12;  // head_dim 128: the TMA unit has read dQ_i out of the Pᵀ / dSᵀ buffers
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // CTAs are dispatched in block order: within a group of batch*head slices the key tiles with the
  // longest walk (tile 0) of EVERY slice come first, so the tail of the kernel is made of short CTAs
  const int nq = p.T / FB_T;
  int kt, bh;
  if (p.debug & 32) {  // per-slice order (test switch)
    kt = blockIdx.x % nq;
    bh = blockIdx.x / nq;
  } else {
    const int g = blockIdx.x / (nq * p.group), r = blockIdx.x % (nq * p.group);
    const int gsz = min(p.group, p.BH - g * p.group);
    kt = r / gsz;
    bh = g * p.group + r % gsz;
  }
  const int b = bh / p.H, h = bh % p.H;
  const int j0 = kt * FB_T;
  const int iters = nq - kt;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 3; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(pds_full, FB_CWARPS);
    mbar_init(dq_full, 1);
    mbar_init(dq_free, 4);
    mbar_init(s_free, FB_CWARPS);
    mbar_init(stage_free, 4);
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
      tma_prefetch_desc(&tmDO);
      mbar_expect_tx(kv_full, 2 * Cfg::TILE_BYTES);
#pragma unroll
      for (int c = 0; c < Cfg::PANELS; ++c) {
        tma_load_4d(smem + Cfg::OFF_K + c * 16384, &tmK, c * 64, j0, h, b, kv_full);
        tma_load_4d(smem + Cfg::OFF_V + c * 16384, &tmV, c * 64, j0, h, b, kv_full);
      }
      for (int it = 0; it < iters; ++it) {
        const int st = it % QS;
        const uint32_t ph = (it / QS) & 1;
        if (!mbar_wait(&q_empty[st], ph ^ 1, 0x2100 | st, abort_flag)) break;
        mbar_expect_tx(&q_full[st], 2 * Cfg::TILE_BYTES);
        const int i0 = (kt + it) * FB_T;
#pragma unroll
        for (int c = 0; c < Cfg::PANELS; ++c) {
          tma_load_4d(smem + Cfg::OFF_Q + st * Cfg::TILE_BYTES + c * 16384, &tmQ, c * 64, i0, h, b, &q_full[st]);
          tma_load_4d(smem + Cfg::OFF_DO + st * Cfg::TILE_BYTES + c * 16384, &tmDO, c * 64, i0, h, b, &q_full[st]);
        }
      }
    }
  } else if (warp == 1) {
    // ----------------------------------------------------------------------- MMA issuer
    // The whole warp runs this code and one elected lane issues each tcgen05 instruction.  With the loop in a
    // single lane the operand descriptors live in ordinary registers and every instruction pays for moving
    // them to the uniform registers the tensor core reads (measured: 63 cycles per M128 N64 K16 instruction
    // against 49 with warp-uniform code, and 80-120 in this kernel, where it made the issue of a tile's 32
    // instructions the longest item of the step).
    // At head_dim 128 every instruction is 64 cycles of tensor work, the single lane keeps up, and the faster
    // bursts only took tensor-memory bandwidth from the compute warps (373 against 349 us at T 4096): there the
    // loop stays in lane 0.
    constexpr bool WHOLE_WARP = (HD == 64);
    if (!dead && (WHOLE_WARP || lane == 0)) {
      constexpr int fmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t idesc_s = instr_desc_f16(128, 128, fmt, 0, 0);   // Sᵀ, dPᵀ : both K-major
      constexpr uint32_t idesc_kv = instr_desc_f16(128, HD, fmt, 0, 1);   // dV, dK  : A K-major, B MN-major
      constexpr uint32_t idesc_q = instr_desc_f16(128, HD, fmt, 1, 1);    // dQ      : both MN-major
      // read from shared memory: tell the compiler it is uniform
      const uint32_t tb = WHOLE_WARP ? __shfl_sync(0xffffffffu, tmem_base, 0) : tmem_base;
      auto leader = [&]() -> bool { return WHOLE_WARP ? elect_one() : true; };
      // operand descriptors of every buffer in both roles; each MMA only advances the start address
      // (K-major: lbo unused, 8-row groups 1024 B apart; MN-major: 64-element chunks one 16 KB panel apart,
      // 8-row groups 1024 B apart)
      const uint32_t s0 = smem_u32(smem);
      const uint64_t dk_k = smem_desc_sw128(s0 + Cfg::OFF_K, 16, 1024);
      const uint64_t dk_mn = smem_desc_sw128(s0 + Cfg::OFF_K, 16384, 1024);
      const uint64_t dv_k = smem_desc_sw128(s0 + Cfg::OFF_V, 16, 1024);
      const uint64_t dp_k = smem_desc_sw128(s0 + Cfg::OFF_P, 16, 1024);
      const uint64_t dds_k = smem_desc_sw128(s0 + Cfg::OFF_DS, 16, 1024);
      const uint64_t dds_mn = smem_desc_sw128(s0 + Cfg::OFF_DS, 16384, 1024);
      const bool prof = (p.debug & 2) && lane == 0;
      PROF_T(tm_start);
      // every lane waits; the verdict is made uniform so that the warp stays converged
      auto wait = [&](uint64_t* bar, uint32_t parity, int code) -> bool {
        const bool r = mbar_wait(bar, parity, code, abort_flag);
        return WHOLE_WARP ? (__all_sync(0xffffffffu, r) != 0) : r;
      };
      bool ok = wait(kv_full, 0, 0x2200);
      // Sᵀ = K Q_iᵀ and dPᵀ = V dO_iᵀ of query tile `it`
      auto issue_scores = [&](int it) -> bool {
        const int st = it % QS;
        PROF_T(a0);
        if (!wait(&q_full[st], (it / QS) & 1, 0x2300 | st)) return false;
        PROF_T(a1);
        PROF_ADD(7, a0, a1);
        tc_fence_after();
        PROF_T(i0_);
        const uint64_t q_k = smem_desc_sw128(s0 + Cfg::OFF_Q + st * Cfg::TILE_BYTES, 16, 1024);
        const uint64_t do_k = smem_desc_sw128(s0 + Cfg::OFF_DO + st * Cfg::TILE_BYTES, 16, 1024);
#pragma unroll
        for (int s = 0; s < HD / 16; ++s) {
          const uint32_t off = (s / 4) * 16384 + (s % 4) * 32;
          if (leader()) tc_mma_ss(tb + Cfg::COL_S, desc_advance(dk_k, off), desc_advance(q_k, off), idesc_s, s ? 1u : 0u);
        }
#pragma unroll
        for (int s = 0; s < HD / 16; ++s) {
          const uint32_t off = (s / 4) * 16384 + (s % 4) * 32;
          if (leader()) tc_mma_ss(tb + Cfg::COL_DP, desc_advance(dv_k, off), desc_advance(do_k, off), idesc_s, s ? 1u : 0u);
        }
        if (leader()) tc_commit(s_full);
        PROF_T(i1_);
        PROF_ADD(12, i0_, i1_);
        return true;
      };
      // dV += Pᵀ dO_i, dK += dSᵀ Q_i, dQ_i = dS K
      auto issue_grads = [&](int it) -> bool {
        const int st = it % QS;
        const uint64_t q_mn = smem_desc_sw128(s0 + Cfg::OFF_Q + st * Cfg::TILE_BYTES, 16384, 1024);
        const uint64_t do_mn = smem_desc_sw128(s0 + Cfg::OFF_DO + st * Cfg::TILE_BYTES, 16384, 1024);
        // the dQ columns still hold the previous tile's dQ until the drain warps are done with it
        PROF_T(a0);
        if (it > 0 && !wait(dq_free, (it - 1) & 1, 0x2400)) return false;
        PROF_T(a1);
        PROF_ADD(8, a0, a1);
        tc_fence_after();
        PROF_T(i0_);
        const uint32_t acc = it ? 1u : 0u;
#pragma unroll
        for (int s = 0; s < FB_T / 16; ++s) {  // contraction over the 128 queries of this tile
          const uint32_t koff = (s / 4) * 16384 + (s % 4) * 32;  // K-major A: 16 queries = 32 B along the row
          const uint32_t moff = s * 2048;                         // MN-major B: 16 query rows of 128 B
          if (leader()) {
            if (Cfg::P_TMEM)
              tc_mma_ts(tb + Cfg::COL_DV, tb + Cfg::COL_PT + s * 8, desc_advance(do_mn, moff), idesc_kv, s ? 1u : acc);
            else
              tc_mma_ss(tb + Cfg::COL_DV, desc_advance(dp_k, koff), desc_advance(do_mn, moff), idesc_kv, s ? 1u : acc);
            tc_mma_ss(tb + Cfg::COL_DK, desc_advance(dds_k, koff), desc_advance(q_mn, moff), idesc_kv, s ? 1u : acc);
          }
        }
#pragma unroll
        for (int s = 0; s < FB_T / 16; ++s) {  // contraction over the 128 keys of this CTA
          const uint32_t moff = s * 2048;      // 16 key rows of 128 B in dSᵀ and in K
          if (leader()) tc_mma_ss(tb + Cfg::COL_DQ, desc_advance(dds_mn, moff), desc_advance(dk_mn, moff), idesc_q, s ? 1u : 0u);
        }
        if (leader()) {
          tc_commit(&q_empty[st]);
          tc_commit(dq_full);
        }
        PROF_T(i1_);
        PROF_ADD(15, i0_, i1_);
        return true;
      };
      if (ok) ok = issue_scores(0);
      for (int it = 0; it < iters && ok; ++it) {
        if (!Cfg::DQ_ALIASED && it + 1 < iters) {
          // The compute warps hand Sᵀ / dPᵀ back as soon as they hold them in registers, about half-way through
          // their work on the tile: the next tile's scores are issued then and have landed when the warps come
          // back for them.  (Issued only once Pᵀ / dSᵀ were ready, they cost a round trip of 1.5 k cycles per
          // tile that nothing hid: the score buffers cannot be doubled, tensor memory is full.)
          if (!wait(s_free, it & 1, 0x2550)) { ok = false; break; }
          if (!issue_scores(it + 1)) { ok = false; break; }
        }
        PROF_T(a0);
        if (!wait(pds_full, it & 1, 0x2500)) { ok = false; break; }
        PROF_T(a1);
        PROF_ADD(6, a0, a1);
        if (!Cfg::DQ_ALIASED) {
          ok = issue_grads(it);
        } else {
          // dQ_i reuses the Sᵀ columns: the next scores may only follow once dQ_i has been drained
          ok = issue_grads(it);
          if (ok && it + 1 < iters) {
            PROF_T(b0);
            ok = wait(dq_free, it & 1, 0x2450);
            PROF_T(b1);
            PROF_ADD(8, b0, b1);
            if (ok) ok = issue_scores(it + 1);
          }
        }
      }
      PROF_T(tm_end);
      PROF_ADD(9, tm_start, tm_end);
    }
    __syncwarp();
  } else if (warp < 2 + FB_CWARPS) {
    // -------------------------------------------------------------------------- compute
    if (!dead) {
      const int cw = warp - 2;           // 0..15
      const int qd = warp & 3;           // TMEM lane quarter
      const int cq = cw >> 2;            // which quarter (32) of the 128 query columns
      const int r = qd * 32 + lane;      // TMEM lane = key row
      const int ct = threadIdx.x - 64;   // 0..255 within the compute group
      const uint32_t lane_addr = tmem_base + ((uint32_t)(qd * 32) << 16);
      const float c2 = p.scale * kLog2eB;
      const AlibiLog2<BIAS> alibi(BIAS ? p.slopes[h] : 0.f);
      const int j = j0 + r;              // this thread's key
      uint8_t* sp = smem + Cfg::OFF_P;
      uint8_t* sds = smem + Cfg::OFF_DS;
      bool ok = true;
      const bool prof = (p.debug & 2) && threadIdx.x == 64;
      // Per-query statistics of the warp's 32 query columns: lane l carries lse and delta of
      // column l, fetched one tile ahead (so the global-memory latency is not part of the tile) and handed to the
      // other lanes through a slice of shared memory that belongs to this warp: no barrier across the warps.
      auto load_stat = [&](int it, float& l2, float& dl) {
        const int64_t at = (int64_t)bh * p.T + (kt + it) * FB_T + cq * 32 + lane;
        l2 = p.lse[at];  // converted to log2 units where it is used: nothing here may wait for the load
        dl = p.delta[at];
      };
      float lse_next, delta_next;
      load_stat(0, lse_next, delta_next);
      for (int it = 0; it < iters; ++it) {
        const int i0 = (kt + it) * FB_T;
        const bool diag = (it == 0);
        PROF_T(t0);
        // this tile's statistics, double buffered by iteration parity: a lane that is already here may share
        // the warp with one that still reads the previous tile's slice
        float* s_lse2 = s_stat + ((it & 1) * FB_CWARPS + cw) * 64;
        float* s_delta = s_lse2 + 32;
        s_lse2[lane] = lse_next * kLog2eB;
        s_delta[lane] = delta_next;
        __syncwarp();
        PROF_T(t1);
        if (it + 1 < iters) load_stat(it + 1, lse_next, delta_next);  // after the warp barrier, which would wait for it
        if (ok) ok = mbar_wait(s_full, it & 1, 0x2600, abort_flag);
        PROF_T(t2);
        PROF_ADD(5, t0, t1);
        PROF_ADD(1, t1, t2);
        if (prof) atomicAdd(&g_prof[0], 1ull);
        uint32_t pk[16], dk_[16];  // this thread's 32 columns of Pᵀ and dSᵀ, packed 16-bit pairs
        long long t3 = 0, t4 = 0;
        const bool quiet = (p.debug & 128) != 0;  // timing experiment: the compute warps only keep the barriers going
        if (quiet) {
#pragma unroll
          for (int e = 0; e < 16; ++e) pk[e] = dk_[e] = 0u;
          if (!Cfg::DQ_ALIASED && lane == 0) mbar_arrive(s_free);
          if (it > 0 && ok) ok = mbar_wait(dq_full, (it - 1) & 1, 0x2650, abort_flag);
        }
        if (ok && !quiet) {
          tc_fence_after();
          const bool plain = !BIAS && !diag;  // no bias and not the diagonal tile: scale, subtract, 2^x
          // Four chunks of 8 query columns; the tensor-memory loads of a chunk are issued before the chunk ahead of
          // it is worked on (two register sets of 8 + 8 values), so only the first load's latency is exposed.
          // (Requesting a tile's first chunk at the end of the tile before it, ahead of the gradient products whose
          // burst makes the load wait 850 cycles, was tried: the wait for the next scores at that point cost more
          // than it saved, 230 against 210 us.)
          uint32_t sv_[2][8], dv_[2][8];
          PROF_T(tl0);
          tmem_ld8(lane_addr + Cfg::COL_S + cq * 32, sv_[0]);
          tmem_ld8(lane_addr + Cfg::COL_DP + cq * 32, dv_[0]);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int col0 = cq * 32 + c * 8;
            const float d0 = (float)(i0 + col0 - j);  // distance of the chunk's first query to this thread's key
            tc_wait_ld();
            if (c + 1 < 4) {
              tmem_ld8(lane_addr + Cfg::COL_S + col0 + 8, sv_[(c + 1) & 1]);
              tmem_ld8(lane_addr + Cfg::COL_DP + col0 + 8, dv_[(c + 1) & 1]);
            } else if (!Cfg::DQ_ALIASED) {  // this warp's share of Sᵀ and dPᵀ is in registers
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(s_free);
            }
            if (c == 0) {
              PROF_T(tl1);
              PROF_ADD(14, tl0, tl1);
            }
#pragma unroll
            for (int e4 = 0; e4 < 2; ++e4) {
              const float4 l4 = *reinterpret_cast<const float4*>(s_lse2 + c * 8 + e4 * 4);
              const float4 d4 = *reinterpret_cast<const float4*>(s_delta + c * 8 + e4 * 4);
              const float lv[4] = {l4.x, l4.y, l4.z, l4.w};
              const float dl[4] = {d4.x, d4.y, d4.z, d4.w};
              float pe[4], de[4];
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const int e = e4 * 4 + k;
                float x = fmaf(__uint_as_float(sv_[c & 1][e]), c2, -lv[k]);
                if (plain) {
                  pe[k] = ex2_approx_b(x);  // (one exponential in four on the FMA pipe, as in the forward, changed nothing here)
                } else {
                  const int i = i0 + col0 + e;
                  x = alibi.sub_from(x, d0 + (float)e);  // a key above the diagonal (negative distance) is masked below
                  pe[k] = (j > i) ? 0.f : ex2_approx_b(x);
                }
                de[k] = pe[k] * (__uint_as_float(dv_[c & 1][e]) - dl[k]);
              }
              pk[c * 4 + e4 * 2] = pack2<T>(pe[0], pe[1]);
              pk[c * 4 + e4 * 2 + 1] = pack2<T>(pe[2], pe[3]);
              dk_[c * 4 + e4 * 2] = pack2<T>(de[0], de[1]);
              dk_[c * 4 + e4 * 2 + 1] = pack2<T>(de[2], de[3]);
            }
          }
          // Pᵀ / dSᵀ of the previous tile are still being read by its gradient products
          if (prof) t3 = clock64();
          if (it > 0) ok = mbar_wait(dq_full, (it - 1) & 1, 0x2650, abort_flag);
          // ... and, at head_dim 128, by the TMA reduction of its dQ, which was staged in them
          if (Cfg::DQ_IN_PDS && it > 0 && ok) ok = mbar_wait(stage_free, (it - 1) & 1, 0x2660, abort_flag);
          if (prof) t4 = clock64();
          PROF_ADD(2, t2, t3);
          PROF_ADD(3, t3, t4);
        }
        if (ok && quiet) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(pds_full);
        }
        if (ok && !quiet) {
          if (Cfg::P_TMEM) tmem_st16(lane_addr + Cfg::COL_PT + cq * 16, pk);  // this thread's 32 queries of Pᵀ
#pragma unroll
          for (int v4 = 0; v4 < 4; ++v4) {
            const int cc = cq * 4 + v4;  // 16-byte chunk index along the 128 queries
            const uint32_t off = (cc >> 3) * 16384 + r * 128 + (((cc & 7) ^ (r & 7)) << 4);
            if (!Cfg::P_TMEM)
              *reinterpret_cast<uint4*>(sp + off) = make_uint4(pk[v4 * 4], pk[v4 * 4 + 1], pk[v4 * 4 + 2], pk[v4 * 4 + 3]);
            *reinterpret_cast<uint4*>(sds + off) = make_uint4(dk_[v4 * 4], dk_[v4 * 4 + 1], dk_[v4 * 4 + 2], dk_[v4 * 4 + 3]);
          }
          if (Cfg::P_TMEM) tc_wait_st();
          PROF_T(t45);
          tc_fence_before();
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(pds_full);
          PROF_T(t5);
          PROF_ADD(4, t4, t5);
          PROF_ADD(13, t45, t5);
        }
      }
      if (ok && mbar_wait(dq_full, (iters - 1) & 1, 0x2680, abort_flag)) {
        // dV and dK are complete
        tc_fence_after();
        T* dvp = reinterpret_cast<T*>(p.dv) + b * p.sdv_b + h * p.sdv_h + (int64_t)j * p.sdv_t;
        T* dkp = reinterpret_cast<T*>(p.dk) + b * p.sdk_b + h * p.sdk_h + (int64_t)j * p.sdk_t;
#pragma unroll 1
        for (int c = 0; c < HD / 64; ++c) {  // this warp's HD / 4 columns in steps of 16
          const int col0 = cq * (HD / 4) + c * 16;
          uint32_t v[16], w[16];
          tmem_ld16(lane_addr + Cfg::COL_DV + col0, v);
          tmem_ld16(lane_addr + Cfg::COL_DK + col0, w);
          tc_wait_ld();
#pragma unroll
          for (int v4 = 0; v4 < 2; ++v4) {
            float g[8], d[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              g[e] = __uint_as_float(v[v4 * 8 + e]);
              d[e] = __uint_as_float(w[v4 * 8 + e]) * p.scale;
            }
            *reinterpret_cast<uint4*>(dvp + col0 + v4 * 8) = pack8<T>(g);
            *reinterpret_cast<uint4*>(dkp + col0 + v4 * 8) = pack8<T>(d);
          }
        }
      }
    }
  } else if (!dead) {
    // ---------------------------------------------------------------------------- dQ drain
    // the last four warps: lanes are query rows here; each warp adds its 32 rows of dQ_i to the fp32 accumulator.
    // head_dim 64: the rows go through swizzled shared-memory boxes and the TMA unit performs the
    // reduction (cp.reduce.async.bulk.tensor), which keeps the load/store path free for the compute
    // warps; head_dim 128: vector red.global.add.
    const int qd = warp & 3;
    const int r = qd * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(qd * 32) << 16);
    const bool prof = (p.debug & 2) && warp == 2 + FB_CWARPS && lane == 0;
    uint8_t* stage = smem + Cfg::OFF_DQ + (warp - 2 - FB_CWARPS) * Cfg::DQ_BOXES * 4096;
    if (Cfg::DQ_TMA && lane == 0) tma_prefetch_desc(&tmDQ);
    for (int it = 0; it < iters; ++it) {
      const int i0 = (kt + it) * FB_T;
      PROF_T(a0);
      if (!mbar_wait(dq_full, it & 1, 0x2700, abort_flag)) break;
      PROF_T(a1);
      PROF_ADD(10, a0, a1);
      tc_fence_after();
      if (HD == 128 && !(p.debug & 64)) {
        // The warp's four chunks of 32 columns go into four boxes inside the Pᵀ / dSᵀ buffers (idle until the
        // compute warps write the next tile's Pᵀ / dSᵀ), so tensor memory is free after four loads and the next
        // scores - dQ reuses their columns - start while the TMA unit adds the boxes to the accumulator.  (Through
        // one box per warp with a wait between chunks the drain took 4.3 k cycles per tile, all of it ahead of the
        // next scores; vector atomics from registers 4.9 k.)
        const int row0 = (int)((int64_t)bh * p.T) + i0 + qd * 32;
        uint8_t* boxes = smem + Cfg::OFF_P + (warp - 2 - FB_CWARPS) * 4 * 4096;
        // two loads in flight at a time; the columns are handed back as soon as the last load has landed, before
        // the last stores and the proxy fence
        auto store_box = [&](int c, const uint32_t (&v)[32]) {
          if (p.debug & 1) return;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const uint32_t off = lane * 128 + ((q ^ (lane & 7)) << 4);
            *reinterpret_cast<uint4*>(boxes + c * 4096 + off) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
          }
        };
        {
          uint32_t va[32], vb[32];
          tmem_ld32(lane_addr + Cfg::COL_DQ, va);
          tmem_ld32(lane_addr + Cfg::COL_DQ + 32, vb);
          tc_wait_ld();
          store_box(0, va);
          store_box(1, vb);
          tmem_ld32(lane_addr + Cfg::COL_DQ + 64, va);
          tmem_ld32(lane_addr + Cfg::COL_DQ + 96, vb);
          tc_wait_ld();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(dq_free);  // tensor memory is drained: the next scores may overwrite the columns
          store_box(2, va);
          store_box(3, vb);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (!(p.debug & 1)) {
#pragma unroll
            for (int c = 0; c < HD / 32; ++c) tma_reduce_add_2d(&tmDQ, boxes + c * 4096, c * 32, row0);
            tma_store_commit();
            tma_store_wait_read();  // the boxes have been read: Pᵀ / dSᵀ may be written again
          }
          mbar_arrive(stage_free);
        }
      } else if (HD == 64 && !(p.debug & 64)) {
        uint32_t v0[32], v1[32];
        tmem_ld32(lane_addr + Cfg::COL_DQ, v0);
        tmem_ld32(lane_addr + Cfg::COL_DQ + 32, v1);
        tc_wait_ld();
        // TMEM is drained: the tensor core may overwrite dQ while the rows travel on
        tc_fence_before();
        if (lane == 0) tma_store_wait_read();  // previous boxes have been read by the TMA unit
        __syncwarp();
        if (lane == 0) mbar_arrive(dq_free);
        if (!(p.debug & 1)) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {  // 16-byte chunks (4 floats) of this row in each of the two boxes
            const uint32_t off = lane * 128 + ((j ^ (lane & 7)) << 4);
            *reinterpret_cast<uint4*>(stage + off) = make_uint4(v0[4 * j], v0[4 * j + 1], v0[4 * j + 2], v0[4 * j + 3]);
            *reinterpret_cast<uint4*>(stage + 4096 + off) =
                make_uint4(v1[4 * j], v1[4 * j + 1], v1[4 * j + 2], v1[4 * j + 3]);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const int row0 = (int)((int64_t)bh * p.T) + i0 + qd * 32;
            tma_reduce_add_2d(&tmDQ, stage, 0, row0);
            tma_reduce_add_2d(&tmDQ, stage + 4096, 32, row0);
            tma_store_commit();
          }
        }
      } else {
        float* dq_row = p.dq_acc + ((int64_t)bh * p.T + i0 + r) * HD;
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t v[32];
          tmem_ld32(lane_addr + Cfg::COL_DQ + c * 32, v);
          tc_wait_ld();
          if (!(p.debug & 1))
#pragma unroll
            for (int e = 0; e < 32; e += 4)
              asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dq_row + c * 32 + e),
                           "f"(__uint_as_float(v[e])), "f"(__uint_as_float(v[e + 1])),
                           "f"(__uint_as_float(v[e + 2])), "f"(__uint_as_float(v[e + 3]))
                           : "memory");
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(dq_free);
      }
      PROF_T(a2);
      PROF_ADD(11, a1, a2);
    }
    if (Cfg::DQ_TMA && lane == 0) tma_store_wait_all();  // every reduction has reached global memory
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

// dq = round(scale * dq_acc), written with the caller's strides
template <typename T>
__global__ void __launch_bounds__(256) attn_dq_convert_kernel(const float* __restrict__ acc, T* __restrict__ dq,
                                                              int64_t sb, int64_t sh, int64_t st, int H, int T_,
                                                              int hd, float scale, int64_t nvec) {
  grid_dependency_wait();
  allow_dependents();
  const int vpr = hd / 8;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < nvec;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(idx % vpr);
    const int64_t row = idx / vpr;
    const int i = (int)(row % T_);
    const int64_t bh = row / T_;
    const int b = (int)(bh / H), h = (int)(bh % H);
    const float4 x = *reinterpret_cast<const float4*>(acc + idx * 8);
    const float4 y = *reinterpret_cast<const float4*>(acc + idx * 8 + 4);
    float f[8] = {x.x * scale, x.y * scale, x.z * scale, x.w * scale, y.x * scale, y.y * scale, y.z * scale, y.w * scale};
    *reinterpret_cast<uint4*>(dq + b * sb + h * sh + (int64_t)i * st + c * 8) = pack8<T>(f);
  }
}

// ------------------------------------------------------------------------------- host side

// Copies the timing counters to `out` (16 values) and clears them.  Synchronises the device.
int attn_bwd_tc05_counters(unsigned long long* out) {
  cudaDeviceSynchronize();
  if (cudaMemcpyFromSymbol(out, g_prof, sizeof(unsigned long long) * 16) != cudaSuccess) return -1;
  unsigned long long z[16] = {0};
  cudaMemcpyToSymbol(g_prof, z, sizeof(z));
  return 0;
}

static int encode_bhtd(CUtensorMap* m, const void* ptr, const AttnStrides& s, int B, int H, int T, int hd, int dtype) {
  const uint64_t dims[4] = {(uint64_t)hd, (uint64_t)T, (uint64_t)H, (uint64_t)B};
  const uint64_t str[3] = {(uint64_t)s.t * 2, (uint64_t)s.h * 2, (uint64_t)s.b * 2};
  const uint32_t box[4] = {64, 128, 1, 1};
  return encode_tmap_sw128(m, ptr, dtype, 4, dims, str, box);
}

bool attn_tc05_bwd_eligible(const AttnArgs& a, int hd) {
  return (hd == 64 || hd == 128) && a.T % 128 == 0 && a.bias_mode != 3;
}

template <typename T, int HD>
static int bwd_tc05_launch(const AttnArgs& a, int dtype, cudaStream_t st) {
  using Cfg = FbCfg<HD>;
  int rc;
  // the delta pass also clears the fp32 dQ accumulator (contiguous (B,H,T,HD), 16-byte aligned: checked by the
  // caller), so no fill sits between the kernels in the stream
  if ((rc = attn_delta(a, HD, dtype, st, a.dq_acc))) return rc;
  CUtensorMap tq, tk, tv, tdo, tdq;
  {
    // fp32 dQ accumulator as a (HD, B*H*T) matrix, boxes of 32 floats x 32 rows
    const uint64_t dims[2] = {(uint64_t)HD, (uint64_t)a.B * a.H * a.T};
    const uint64_t str[1] = {(uint64_t)HD * 4};
    const uint32_t box[2] = {32, 32};
    if ((rc = encode_tmap_sw128(&tdq, a.dq_acc, TFB_F32, 2, dims, str, box))) return rc;
  }
  if ((rc = encode_bhtd(&tq, a.q, a.sq, a.B, a.H, a.T, HD, dtype))) return rc;
  if ((rc = encode_bhtd(&tk, a.k, a.sk, a.B, a.H, a.T, HD, dtype))) return rc;
  if ((rc = encode_bhtd(&tv, a.v, a.sv, a.B, a.H, a.T, HD, dtype))) return rc;
  if ((rc = encode_bhtd(&tdo, a.d_o, a.sdo, a.B, a.H, a.T, HD, dtype))) return rc;
  FbParams p;
  p.lse = a.lse; p.delta = a.delta; p.dq_acc = a.dq_acc; p.dk = a.dk; p.dv = a.dv;
  p.sdk_b = a.sdk.b; p.sdk_h = a.sdk.h; p.sdk_t = a.sdk.t;
  p.sdv_b = a.sdv.b; p.sdv_h = a.sdv.h; p.sdv_t = a.sdv.t;
  p.H = a.H; p.T = a.T; p.scale = a.scale; p.bias_mode = a.bias_mode; p.slopes = a.slopes;
  p.debug = g_attn_debug.load();
  p.BH = a.B * a.H;
  p.group = attn_slices_per_group(a.B * a.H, a.T, HD);
  dim3 grid((a.T / FB_T) * a.B * a.H);
  static std::atomic<uint64_t> done[4] = {{0}, {0}, {0}, {0}};
#define FB_LAUNCH(MODE, SLOT)                                                                                       \
  {                                                                                                                 \
    if ((rc = ensure_dynamic_smem(attn_bwd_tc05_kernel<T, HD, MODE>, Cfg::SMEM_BYTES, done[SLOT],                   \
                                  "attention_bwd(tcgen05)")))                                                       \
      return rc;                                                                                                    \
    launch_overlapped(attn_bwd_tc05_kernel<T, HD, MODE>, grid, dim3(FB_THREADS), Cfg::SMEM_BYTES, st, tq, tk, tv, tdo, \
                      tdq, p);                                                                                      \
  }
  if (a.bias_mode == 0) FB_LAUNCH(0, 0)
  else if (a.bias_mode == 1) FB_LAUNCH(1, 1)
  else if (a.bias_mode == 2) FB_LAUNCH(2, 2)
  else FB_LAUNCH(4, 3)
#undef FB_LAUNCH
  if ((rc = launched("attention_bwd(tcgen05)"))) return rc;
  const int64_t nvec = (int64_t)a.B * a.H * a.T * HD / 8;
  const unsigned blocks = (unsigned)(ceil_div(nvec, 256) < 148 * 8 ? ceil_div(nvec, 256) : 148 * 8);
  launch_overlapped(attn_dq_convert_kernel<T>, dim3(blocks), dim3(256), 0, st, a.dq_acc, (T*)a.dq, a.sdq.b, a.sdq.h,
                    a.sdq.t, a.H, a.T, HD, a.scale, nvec);
  return launched("attention_dq_convert");
}

int attn_tc05_bwd(const AttnArgs& a, int hd, int dtype, cudaStream_t st) {
  TFB_DISPATCH_16(dtype, T, {
    if (hd == 64) return bwd_tc05_launch<T, 64>(a, dtype, st);
    return bwd_tc05_launch<T, 128>(a, dtype, st);
  })
}

}  // namespace tfb
