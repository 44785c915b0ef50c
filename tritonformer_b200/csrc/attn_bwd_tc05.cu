// Causal flash attention backward on tcgen05 / TMEM for sm_100a (head_dim 64 or 128, T % 128 == 0).
//
// One CTA per (128-key tile, batch*head); it walks the query tiles at or below the diagonal.
// Everything is computed transposed (rows = keys) so that the per-query statistics (log-sum-exp,
// delta) are per-column constants and no row reductions are needed:
//   Sᵀ  = K Q_iᵀ                 dPᵀ = V dO_iᵀ                      (tensor cores -> TMEM)
//   Pᵀ  = 2^(Sᵀ·c + bias - lse)  dSᵀ = Pᵀ ∘ (dPᵀ - delta)            (compute warps -> smem, 16 bit)
//   dV += Pᵀ dO_i     dK += dSᵀ Q_i     dQ_i = dS K                  (tensor cores -> TMEM)
// dV and dK stay in TMEM for the whole walk; dQ_i is added to an fp32 global accumulator
// (red.global.add.f32) because every key tile contributes to it; a small kernel scales and
// rounds the accumulator afterwards.
// A 128 x 64 swizzled panel of 16-bit values is at the same time a K-major operand with 128 rows
// and an MN-major operand with 128 contraction rows, so each of K, V, Q_i, dO_i, dSᵀ sits in
// shared memory once and serves two products.
//
// Roles: warp 0 TMA producer, warp 1 MMA issuer, warps 2-17 compute (thread = TMEM lane, four
// warps per lane quarter, each taking a quarter of the columns), warps 18-21 drain dQ_i.
// At head_dim 64, Pᵀ goes into the 64 TMEM columns that are left instead of shared memory and is
// the A operand of the dV product.
// At head_dim 64 the scores of tile i+1 are issued before the gradient products of tile i, so the
// compute warps work on tile i+1 while the tensor core finishes tile i.
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
  static constexpr int QSTAGES = (HD == 64) ? 2 : 1;  // query-side ring depth (smem bound at hd 128)
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = TILE_BYTES;
  static constexpr int OFF_Q = 2 * TILE_BYTES;                       // [QSTAGES]
  static constexpr int OFF_DO = OFF_Q + QSTAGES * TILE_BYTES;        // [QSTAGES]
  static constexpr int OFF_P = OFF_DO + QSTAGES * TILE_BYTES;        // Pᵀ  128 x 128 x 2 B
  static constexpr int OFF_DS = OFF_P + 32768;                       // dSᵀ 128 x 128 x 2 B
  static constexpr int OFF_STAT = OFF_DS + 32768;                    // 2 x (lse2[128], delta[128]) fp32
  // dQ_i staging for the TMA reduction (head_dim 64 only: it does not fit next to 128-wide tiles)
  static constexpr bool DQ_TMA = (HD == 64);
  static constexpr int OFF_DQ = OFF_STAT + 2048;                     // 4 drain warps x 2 boxes of 32 rows x 128 B
  static constexpr int OFF_BAR = OFF_DQ + (DQ_TMA ? 32768 : 0);
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
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
  float scale;
  int bias_mode;
  const float* slopes;
  int debug;  // test switch: bit 0 skips the dQ accumulation (timing experiments only)
};

__device__ __forceinline__ float alibi_term_b(int mode, float slope, int dist) {
  return alibi_table_value(mode, slope, dist);
}

// Cycle counters for the timing switch (debug bit 1): [0] CTA iterations, [1..5] compute warp 2:
// wait scores, math, wait previous products, smem write, barrier+stats; [6..9] MMA thread: wait P/dS,
// wait Q/dO, wait dQ drain, total; [10,11] drain warp: wait, drain; [12] CTA lifetime.
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

__device__ __forceinline__ void compute_bar_sync() { asm volatile("bar.sync 1, %0;" ::"n"(32 * FB_CWARPS) : "memory"); }

template <typename T, int HD, bool BIAS>
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
  float* s_stat = reinterpret_cast<float*>(smem + Cfg::OFF_STAT);  // [2 parities][lse2[128], delta[128]]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* kv_full = bars + 0;
  uint64_t* q_full = bars + 1;    // [2] Q_i and dO_i landed
  uint64_t* q_empty = bars + 3;   // [2] products reading them retired
  uint64_t* s_full = bars + 5;    // Sᵀ and dPᵀ in TMEM
  uint64_t* pds_full = bars + 6;  // Pᵀ and dSᵀ in smem (and Sᵀ, dPᵀ consumed)
  uint64_t* dq_full = bars + 7;   // dV, dK, dQ_i products retired
  uint64_t* dq_free = bars + 8;   // dQ_i read out of TMEM
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.x;  // key tile; tile 0 has the longest walk and starts first
  const int bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  const int j0 = kt * FB_T;
  const int nq = p.T / FB_T;
  const int iters = nq - kt;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(pds_full, FB_CWARPS);
    mbar_init(dq_full, 1);
    mbar_init(dq_free, 4);
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
    if (lane == 0 && !dead) {
      constexpr int fmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t idesc_s = instr_desc_f16(128, 128, fmt, 0, 0);   // Sᵀ, dPᵀ : both K-major
      constexpr uint32_t idesc_kv = instr_desc_f16(128, HD, fmt, 0, 1);   // dV, dK  : A K-major, B MN-major
      constexpr uint32_t idesc_q = instr_desc_f16(128, HD, fmt, 1, 1);    // dQ      : both MN-major
      // operand descriptors of every buffer in both roles, built once; each MMA only advances the
      // start address (K-major: lbo unused, 8-row groups 1024 B apart; MN-major: 64-element chunks
      // one 16 KB panel apart, 8-row groups 1024 B apart)
      const uint64_t dk_k = smem_desc_sw128(smem_u32(smem + Cfg::OFF_K), 16, 1024);
      const uint64_t dk_mn = smem_desc_sw128(smem_u32(smem + Cfg::OFF_K), 16384, 1024);
      const uint64_t dv_k = smem_desc_sw128(smem_u32(smem + Cfg::OFF_V), 16, 1024);
      const uint64_t dp_k = smem_desc_sw128(smem_u32(smem + Cfg::OFF_P), 16, 1024);
      const uint64_t dds_k = smem_desc_sw128(smem_u32(smem + Cfg::OFF_DS), 16, 1024);
      const uint64_t dds_mn = smem_desc_sw128(smem_u32(smem + Cfg::OFF_DS), 16384, 1024);
      uint64_t dq_k[QS], dq_mn[QS], ddo_k[QS], ddo_mn[QS];
#pragma unroll
      for (int i = 0; i < QS; ++i) {
        dq_k[i] = smem_desc_sw128(smem_u32(smem + Cfg::OFF_Q + i * Cfg::TILE_BYTES), 16, 1024);
        dq_mn[i] = smem_desc_sw128(smem_u32(smem + Cfg::OFF_Q + i * Cfg::TILE_BYTES), 16384, 1024);
        ddo_k[i] = smem_desc_sw128(smem_u32(smem + Cfg::OFF_DO + i * Cfg::TILE_BYTES), 16, 1024);
        ddo_mn[i] = smem_desc_sw128(smem_u32(smem + Cfg::OFF_DO + i * Cfg::TILE_BYTES), 16384, 1024);
      }
      const bool prof = (p.debug & 2) != 0;
      PROF_T(tm_start);
      bool ok = mbar_wait(kv_full, 0, 0x2200, abort_flag);
      // Sᵀ = K Q_iᵀ and dPᵀ = V dO_iᵀ of query tile `it`
      auto issue_scores = [&](int it) -> bool {
        const int st = it % QS;
        PROF_T(a0);
        if (!mbar_wait(&q_full[st], (it / QS) & 1, 0x2300 | st, abort_flag)) return false;
        PROF_T(a1);
        PROF_ADD(7, a0, a1);
        tc_fence_after();
        const uint64_t q_k = dq_k[st], do_k = ddo_k[st];
#pragma unroll
        for (int s = 0; s < HD / 16; ++s) {
          const uint32_t off = (s / 4) * 16384 + (s % 4) * 32;
          tc_mma_ss(tmem_base + Cfg::COL_S, desc_advance(dk_k, off), desc_advance(q_k, off), idesc_s, s ? 1u : 0u);
        }
#pragma unroll
        for (int s = 0; s < HD / 16; ++s) {
          const uint32_t off = (s / 4) * 16384 + (s % 4) * 32;
          tc_mma_ss(tmem_base + Cfg::COL_DP, desc_advance(dv_k, off), desc_advance(do_k, off), idesc_s, s ? 1u : 0u);
        }
        tc_commit(s_full);
        return true;
      };
      // dV += Pᵀ dO_i, dK += dSᵀ Q_i, dQ_i = dS K
      auto issue_grads = [&](int it) -> bool {
        const int st = it % QS;
        const uint64_t q_mn = dq_mn[st], do_mn = ddo_mn[st];
        // the dQ columns still hold the previous tile's dQ until the drain warps are done with it
        PROF_T(a0);
        if (it > 0 && !mbar_wait(dq_free, (it - 1) & 1, 0x2400, abort_flag)) return false;
        PROF_T(a1);
        PROF_ADD(8, a0, a1);
        tc_fence_after();
#pragma unroll
        for (int s = 0; s < FB_T / 16; ++s) {  // contraction over the 128 queries of this tile
          const uint32_t koff = (s / 4) * 16384 + (s % 4) * 32;  // K-major A: 16 queries = 32 B along the row
          const uint32_t moff = s * 2048;                         // MN-major B: 16 query rows of 128 B
          if (Cfg::P_TMEM)
            tc_mma_ts(tmem_base + Cfg::COL_DV, tmem_base + Cfg::COL_PT + s * 8, desc_advance(do_mn, moff), idesc_kv,
                      (it | s) ? 1u : 0u);
          else
            tc_mma_ss(tmem_base + Cfg::COL_DV, desc_advance(dp_k, koff), desc_advance(do_mn, moff), idesc_kv,
                      (it | s) ? 1u : 0u);
          tc_mma_ss(tmem_base + Cfg::COL_DK, desc_advance(dds_k, koff), desc_advance(q_mn, moff), idesc_kv,
                    (it | s) ? 1u : 0u);
        }
#pragma unroll
        for (int s = 0; s < FB_T / 16; ++s) {  // contraction over the 128 keys of this CTA
          const uint32_t moff = s * 2048;      // 16 key rows of 128 B in dSᵀ and in K
          tc_mma_ss(tmem_base + Cfg::COL_DQ, desc_advance(dds_mn, moff), desc_advance(dk_mn, moff), idesc_q,
                    s ? 1u : 0u);
        }
        tc_commit(&q_empty[st]);
        tc_commit(dq_full);
        return true;
      };
      if (ok) ok = issue_scores(0);
      for (int it = 0; it < iters && ok; ++it) {
        PROF_T(a0);
        if (!mbar_wait(pds_full, it & 1, 0x2500, abort_flag)) { ok = false; break; }
        PROF_T(a1);
        PROF_ADD(6, a0, a1);
        if (!Cfg::DQ_ALIASED) {
          // Sᵀ/dPᵀ of this tile are consumed: the next tile's scores go first, so the compute warps
          // can start on them while the three gradient products of this tile run
          if (it + 1 < iters) ok = issue_scores(it + 1);
          if (ok) ok = issue_grads(it);
        } else {
          // dQ_i reuses the Sᵀ columns: the next scores may only follow once dQ_i has been drained
          ok = issue_grads(it);
          if (ok && it + 1 < iters) {
            ok = mbar_wait(dq_free, it & 1, 0x2450, abort_flag);
            if (ok) ok = issue_scores(it + 1);
          }
        }
      }
      PROF_T(tm_end);
      PROF_ADD(9, tm_start, tm_end);
    }
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
      const float slope = BIAS ? p.slopes[h] : 0.f;
      const int j = j0 + r;              // this thread's key
      uint8_t* sp = smem + Cfg::OFF_P;
      uint8_t* sds = smem + Cfg::OFF_DS;
      bool ok = true;
      const bool prof = (p.debug & 2) && threadIdx.x == 64;
      // Every compute thread runs every iteration up to the named barrier, also after a wait gave
      // up (the remaining waits then return at once), so nobody is left alone at the barrier.
      for (int it = 0; it < iters; ++it) {
        const int i0 = (kt + it) * FB_T;
        const bool diag = (it == 0);
        PROF_T(t0);
        // per-query statistics of this tile, double buffered by iteration parity: a thread that is
        // already here may share the CTA with one still computing the previous tile
        float* s_lse2 = s_stat + (it & 1) * 256;
        float* s_delta = s_lse2 + FB_T;
        if (ct < FB_T) s_lse2[ct] = p.lse[(int64_t)bh * p.T + i0 + ct] * kLog2eB;
        else if (ct < 2 * FB_T) s_delta[ct - FB_T] = p.delta[(int64_t)bh * p.T + i0 + ct - FB_T];
        compute_bar_sync();
        PROF_T(t1);
        if (ok) ok = mbar_wait(s_full, it & 1, 0x2600, abort_flag);
        PROF_T(t2);
        PROF_ADD(5, t0, t1);
        PROF_ADD(1, t1, t2);
        if (prof) atomicAdd(&g_prof[0], 1ull);
        uint32_t pk[16], dk_[16];  // this thread's 32 columns of Pᵀ and dSᵀ, packed 16-bit pairs
        long long t3 = 0, t4 = 0;
        if (ok) {
          tc_fence_after();
          const bool plain = !BIAS && !diag;  // no bias and not the diagonal tile: scale, subtract, 2^x
#pragma unroll
          for (int c = 0; c < 2; ++c) {         // 16-column steps keep the live register set small
            const int col0 = cq * 32 + c * 16;
            uint32_t sv_[16], dv_[16];
            PROF_T(tl0);
            tmem_ld16(lane_addr + Cfg::COL_S + col0, sv_);
            tmem_ld16(lane_addr + Cfg::COL_DP + col0, dv_);
            tc_wait_ld();
            PROF_T(tl1);
            PROF_ADD(14, tl0, tl1);
#pragma unroll
            for (int e4 = 0; e4 < 4; ++e4) {
              const float4 l4 = *reinterpret_cast<const float4*>(s_lse2 + col0 + e4 * 4);
              const float4 d4 = *reinterpret_cast<const float4*>(s_delta + col0 + e4 * 4);
              const float lv[4] = {l4.x, l4.y, l4.z, l4.w};
              const float dl[4] = {d4.x, d4.y, d4.z, d4.w};
              float pe[4], de[4];
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const int e = e4 * 4 + k;
                float x = fmaf(__uint_as_float(sv_[e]), c2, -lv[k]);
                if (plain) {
                  pe[k] = ex2_approx_b(x);
                } else {
                  const int i = i0 + col0 + e;
                  if (BIAS) x += alibi_term_b(p.bias_mode, slope, max(i - j, 0)) * kLog2eB;
                  pe[k] = (j > i) ? 0.f : ex2_approx_b(x);
                }
                de[k] = pe[k] * (__uint_as_float(dv_[e]) - dl[k]);
              }
              pk[c * 8 + e4 * 2] = pack2<T>(pe[0], pe[1]);
              pk[c * 8 + e4 * 2 + 1] = pack2<T>(pe[2], pe[3]);
              dk_[c * 8 + e4 * 2] = pack2<T>(de[0], de[1]);
              dk_[c * 8 + e4 * 2 + 1] = pack2<T>(de[2], de[3]);
            }
          }
          // Pᵀ / dSᵀ of the previous tile are still being read by its gradient products
          if (prof) t3 = clock64();
          if (it > 0) ok = mbar_wait(dq_full, (it - 1) & 1, 0x2650, abort_flag);
          if (prof) t4 = clock64();
          PROF_ADD(2, t2, t3);
          PROF_ADD(3, t3, t4);
        }
        if (ok) {
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
    uint8_t* stage = smem + Cfg::OFF_DQ + (warp - 2 - FB_CWARPS) * 8192;
    if (Cfg::DQ_TMA && lane == 0) tma_prefetch_desc(&tmDQ);
    for (int it = 0; it < iters; ++it) {
      const int i0 = (kt + it) * FB_T;
      PROF_T(a0);
      if (!mbar_wait(dq_full, it & 1, 0x2700, abort_flag)) break;
      PROF_T(a1);
      PROF_ADD(10, a0, a1);
      tc_fence_after();
      if (Cfg::DQ_TMA) {
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
int attn_bwd_tc05_status(int reset) { return read_dev_status(reset); }

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
  static std::atomic<uint64_t> done_plain{0}, done_bias{0};
  if ((rc = ensure_dynamic_smem(attn_bwd_tc05_kernel<T, HD, false>, Cfg::SMEM_BYTES, done_plain, "attention_bwd(tcgen05)")))
    return rc;
  if ((rc = ensure_dynamic_smem(attn_bwd_tc05_kernel<T, HD, true>, Cfg::SMEM_BYTES, done_bias, "attention_bwd(tcgen05)")))
    return rc;
  dim3 grid(a.T / FB_T, a.B * a.H);
  if (a.bias_mode)
    launch_overlapped(attn_bwd_tc05_kernel<T, HD, true>, grid, dim3(FB_THREADS), Cfg::SMEM_BYTES, st, tq, tk, tv, tdo, tdq, p);
  else
    launch_overlapped(attn_bwd_tc05_kernel<T, HD, false>, grid, dim3(FB_THREADS), Cfg::SMEM_BYTES, st, tq, tk, tv, tdo, tdq, p);
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
