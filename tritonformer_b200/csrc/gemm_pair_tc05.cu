// tcgen05 GEMM on CTA pairs (cta_group::2) for sm_100a: one 256 x 256 output tile per pair of SMs.
//
// Same contract as gemm_tc05.cu (C = mask(act(A·B + bias) + addend), either operand K- or MN-major),
// for outputs large enough to give every pair of SMs tiles.  Why a second kernel: the one-CTA kernel
// moves 48 KB of operands from L2 to shared memory per 128 x 256 x 64 block of work and is bound by
// that traffic; here the two CTAs of a cluster each load their own 128 rows of A and HALF of the B
// tile (32 KB per CTA for the same work), and the pair's tensor cores read B from both halves.
//
// Per CTA (both CTAs of the pair run the same code; "leader" = cluster rank 0):
//   warp 0   : TMA producer - its A rows and its half of B into a 6-stage ring; the copies signal the
//              LEADER's full barrier (cp.async.bulk.tensor with .cta_group::2, no multicast)
//   warp 1   : leader only: issues tcgen05.mma.cta_group::2 (M 256 over the pair, N 256, K 16) and
//              commits ring slots / finished accumulators to the barriers of BOTH CTAs
//   warps 2-5: epilogue of this CTA's 128 rows from its own TMEM (two accumulator buffers), as in the
//              one-CTA kernel; the buffer is handed back by an arrival on the leader's barrier
// Every wait is bounded (mbar_wait); the two cluster-wide barriers (after set-up, before exit) are
// reached unconditionally by both CTAs.
#include "gemm_sched.cuh"
#include <type_traits>

namespace tfb {

extern std::atomic<int> g_gemm_debug;

constexpr int GP_M = 128;    // rows per CTA
constexpr int GP_N = 256;    // columns per pair tile
constexpr int GP_NH = 128;   // B rows loaded per CTA
constexpr int GP_K = 64;
constexpr int GP_EPI_WARPS = 8;  // 4, or 8 (two warps per TMEM lane quarter, half of the columns each)
constexpr int GP_THREADS = 64 + 32 * GP_EPI_WARPS;
constexpr int GP_STAGES = GP_EPI_WARPS == 8 ? 5 : 6;  // the staging boxes of eight warps take a ring slot's room
constexpr int GP_A_BYTES = GP_M * GP_K * 2;
constexpr int GP_B_BYTES = GP_NH * GP_K * 2;
constexpr int GP_STAGE_BYTES = GP_A_BYTES + GP_B_BYTES;
constexpr int GP_EPI_BYTES = GP_EPI_WARPS * 4096;  // one staging box per epilogue warp
constexpr int GP_OFF_EPI_C = GP_STAGES * GP_STAGE_BYTES;
constexpr int GP_OFF_EPI_X = GP_OFF_EPI_C + GP_EPI_BYTES;
constexpr int GP_OFF_BAR = GP_OFF_EPI_X + GP_EPI_BYTES;
constexpr int GP_SMEM_BYTES = GP_OFF_BAR + 1024 + 256;
constexpr int GP_TMEM_COLS = 512;

struct PairParams {
  void* C;
  const void* bias;
  const void* addend;
  const void* mask;
  int M, N, K;
  int64_t ldc, ld_addend, ld_mask;
  int relu;
  int tiles_m, tiles_n;  // in 256 x 256 pair tiles
  int sk_tiles;          // pair tiles [0, sk_tiles) are split along K over all pairs; 0 = whole tiles only
  int* flags;            // per split tile: one arrival counter per (CTA of the pair, epilogue warp)
  float* partials;       // one fp32 128 x 256 slot per CTA
  int debug;             // bit 6 (64): per-CTA timeline into g_pair_prof (tfb_debug_set key 4)
};

// Timeline of each CTA for tuning (cycle stamps and wait sums), read through tfb_debug_counters.
static __device__ unsigned long long g_pair_prof[148][16];

// ---- cluster / pair primitives ------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* holder, uint32_t ncols) {  // one warp in each CTA
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(holder)),
               "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Tile load into this CTA's shared memory whose completion is counted on a barrier that may live in
// the peer CTA (bar_cluster_addr is a shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, int c0, int c1,
                                                 uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(m), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tc_mma_ss_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One arrival on the barrier at this shared-memory offset in BOTH CTAs of the pair once every MMA
// issued so far by this thread has retired.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"((uint16_t)3)
      : "memory");
}

template <typename T, bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GP_THREADS, 1)
    gemm_pair_tc05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                          const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmX,
                          const PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + GP_OFF_BAR);
  uint64_t* full = bars;                       // [STAGES] both producers -> leader's MMA (leader's copy is used)
  uint64_t* empty = bars + GP_STAGES;          // [STAGES] leader's MMA -> each CTA's producer
  uint64_t* acc_full = bars + 2 * GP_STAGES;   // [2] leader's MMA -> each CTA's epilogue
  uint64_t* acc_empty = acc_full + 2;          // [2] both epilogues -> leader's MMA (leader's copy is used)
  uint64_t* x_full = acc_empty + 2;            // [4] addend / mask box of an epilogue warp landed
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(x_full + GP_EPI_WARPS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const bool prof = (p.debug & 64) && blockIdx.x < 148;
  unsigned long long* pr = g_pair_prof[blockIdx.x < 148 ? blockIdx.x : 0];
  const long long t_entry = clock64();
  if (prof && threadIdx.x == 0) { pr[0] = global_ns(); }
  if (threadIdx.x == 0) {
    for (int i = 0; i < GP_STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 2 * GP_EPI_WARPS);  // the epilogue warps of both CTAs
    }
    for (int i = 0; i < GP_EPI_WARPS; ++i) mbar_init(&x_full[i], 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc_pair(tmem_holder, GP_TMEM_COLS);
  }
  // set-up above is CTA-local and may overlap the previous kernel's tail; global memory comes after
  grid_dependency_wait();
  allow_dependents();
  if (threadIdx.x == 0) *abort_flag = (*(volatile int*)&g_dev_status != 0) ? 1 : 0;
  tc_fence_before();
  __syncthreads();
  // the peer's barriers and tensor memory are ready before anything is signalled across the pair
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const bool dead = *abort_flag != 0;
  if (prof && threadIdx.x == 0) pr[1] = (unsigned long long)(clock64() - t_entry);  // set-up

  const int num_tiles = dead ? 0 : p.tiles_m * p.tiles_n;
  const int kblocks = (p.K + GP_K - 1) / GP_K;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      Segments segs(kblocks, num_tiles, p.sk_tiles, num_pairs, pair, dead);
      int tile, kb0, kb1;
      while (ok && segs.next(tile, kb0, kb1)) {
        const int m0 = (tile % p.tiles_m) * (2 * GP_M) + (int)rank * GP_M;  // this CTA's rows
        const int n0 = (tile / p.tiles_m) * GP_N + (int)rank * GP_NH;       // this CTA's half of B
        for (int kb = kb0; kb < kb1; ++kb) {
          const long long w0 = clock64();
          if (!mbar_wait(&empty[stage], phase ^ 1, 0x700 | stage, abort_flag)) { ok = false; break; }
          if (prof) pr[2] += (unsigned long long)(clock64() - w0);  // producer waiting for a free slot
          uint8_t* sa = smem + stage * GP_STAGE_BYTES;
          uint8_t* sb = sa + GP_A_BYTES;
          // the leader's barrier counts the bytes of both CTAs
          if (leader) mbar_expect_tx(&full[stage], 2 * GP_STAGE_BYTES);
          const uint32_t bar = map_to_cta(smem_u32(&full[stage]), 0);
          const int k0 = kb * GP_K;
          if (A_MN) {
#pragma unroll
            for (int i = 0; i < GP_M / 64; ++i) tma_load_2d_pair(sa + i * 8192, &tmA, m0 + i * 64, k0, bar);
          } else {
            tma_load_2d_pair(sa, &tmA, k0, m0, bar);
          }
          if (B_MN) {
#pragma unroll
            for (int i = 0; i < GP_NH / 64; ++i) tma_load_2d_pair(sb + i * 8192, &tmB, n0 + i * 64, k0, bar);
          } else {
            tma_load_2d_pair(sb, &tmB, k0, n0, bar);
          }
          if (++stage == GP_STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (prof) pr[3] = (unsigned long long)(clock64() - t_entry);  // last load issued
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------------- MMA issuer (leader only)
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = instr_desc_f16(2 * GP_M, GP_N, std::is_same<T, __nv_bfloat16>::value ? 1 : 0,
                                                A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      Segments segs(kblocks, num_tiles, p.sk_tiles, num_pairs, pair, dead);
      int tile, kb0, kb1;
      while (ok && segs.next(tile, kb0, kb1)) {
        const long long a0 = clock64();
        if (!mbar_wait(&acc_empty[buf], acc_phase ^ 1, 0x800 | buf, abort_flag)) { ok = false; break; }
        if (prof) pr[4] += (unsigned long long)(clock64() - a0);  // MMA waiting for a free accumulator
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * GP_N;
        for (int kb = kb0; kb < kb1; ++kb) {
          const long long f0 = clock64();
          if (!mbar_wait(&full[stage], phase, 0x900 | stage, abort_flag)) { ok = false; break; }
          if (prof) {
            const long long f1 = clock64();
            pr[5] += (unsigned long long)(f1 - f0);  // MMA waiting for operands
            if (pr[6] == 0) pr[6] = (unsigned long long)(f1 - t_entry);  // first operands landed
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * GP_STAGE_BYTES);
          const uint32_t sb = sa + GP_A_BYTES;
#pragma unroll
          for (int k = 0; k < GP_K / 16; ++k) {
            const uint64_t ad = A_MN ? smem_desc_sw128(sa + k * 2048, 8192, 1024)
                                     : smem_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t bd = B_MN ? smem_desc_sw128(sb + k * 2048, 8192, 1024)
                                     : smem_desc_sw128(sb + k * 32, 16, 1024);
            tc_mma_ss_pair(d_tmem, ad, bd, idesc, ((kb - kb0) | k) ? 1u : 0u);
          }
          tc_commit_pair(&empty[stage]);  // both producers may refill the slot once these MMAs have read it
          if (++stage == GP_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit_pair(&acc_full[buf]);  // both epilogues
        buf ^= 1;
        if (buf == 0) acc_phase ^= 1;
      }
      if (prof) pr[7] = (unsigned long long)(clock64() - t_entry);  // last MMA issued
    }
  } else {
    // ---------------------------------------------------------------------- epilogue (both CTAs)
    const int q = warp & 3;   // TMEM lane quarter this warp may read
    const int ew = warp - 2;  // 0 .. EPI_WARPS-1
    const int half = ew >> 2; // with eight epilogue warps: which half of the tile's columns
    const T* bias = reinterpret_cast<const T*>(p.bias);
    uint8_t* stage_c = smem + GP_OFF_EPI_C + ew * 4096;
    uint8_t* stage_x = smem + GP_OFF_EPI_X + ew * 4096;
    const bool x_is_addend = p.addend != nullptr;
    const bool use_x = (p.addend != nullptr || p.mask != nullptr);
    const T* mask_direct = (p.addend != nullptr && p.mask != nullptr) ? reinterpret_cast<const T*>(p.mask) : nullptr;
    constexpr int STEPS = GP_N / 64 / (GP_EPI_WARPS / 4);  // 64-column steps per warp
    int buf = 0;
    uint32_t acc_phase = 0, x_phase = 0;
    bool ok = true;
    if (lane == 0) {
      tma_prefetch_desc(&tmC);
      if (use_x) tma_prefetch_desc(&tmX);
    }
    Segments segs(kblocks, num_tiles, p.sk_tiles, num_pairs, pair, dead);
    int tile, kb0, kb1;
    while (ok && segs.next(tile, kb0, kb1)) {
      const int m0 = (tile % p.tiles_m) * (2 * GP_M) + (int)rank * GP_M;
      const int n0 = (tile / p.tiles_m) * GP_N + half * STEPS * 64;  // first column of this warp's share
      const int row0 = m0 + q * 32;
      const int row = row0 + lane;
      const bool contributes = kb0 > 0;                  // a later part of a split tile
      const bool finishes = kb0 == 0 && kb1 < kblocks;   // first part of a split tile: owns its epilogue
      if (use_x && !contributes && lane == 0) {  // box of step 0, in flight while the main loop still runs
        mbar_expect_tx(&x_full[ew], 4096);
        tma_load_2d(stage_x, &tmX, n0, row0, &x_full[ew]);
      }
      const long long e0 = clock64();
      if (!mbar_wait(&acc_full[buf], acc_phase, 0xa00 | buf, abort_flag)) { ok = false; break; }
      const long long e1 = clock64();
      if (prof && ew == 0 && lane == 0) pr[8] += (unsigned long long)(e1 - e0);  // epilogue waiting for an accumulator
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * GP_N + half * STEPS * 64;
      // partial tiles: slot layout [group of 4 columns][row], so the 32 lanes of a warp touch 512
      // contiguous bytes; this warp's share starts at column group half * STEPS * 16
      const int64_t slot_f4 = (int64_t)GP_M * GP_N / 4;  // float4 per slot
      const int my_f4 = half * STEPS * 16 * GP_M + q * 32 + lane;
      if (contributes) {
        float4* slot = reinterpret_cast<float4*>(p.partials) + (int64_t)blockIdx.x * slot_f4 + my_f4;
#pragma unroll 1
        for (int st = 0; st < STEPS; ++st) {
          uint32_t r0[32], r1[32];
          tmem_ld32(taddr + st * 64, r0);
          tmem_ld32(taddr + st * 64 + 32, r1);
          tc_wait_ld();
          float4* dst = slot + st * 16 * GP_M;
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            __stcg(dst + e * GP_M, make_float4(__uint_as_float(r0[4 * e]), __uint_as_float(r0[4 * e + 1]),
                                               __uint_as_float(r0[4 * e + 2]), __uint_as_float(r0[4 * e + 3])));
            __stcg(dst + (8 + e) * GP_M, make_float4(__uint_as_float(r1[4 * e]), __uint_as_float(r1[4 * e + 1]),
                                                     __uint_as_float(r1[4 * e + 2]), __uint_as_float(r1[4 * e + 3])));
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          __threadfence();  // the warp's partial rows are visible before the arrival
          atomicAdd(p.flags + (tile * 2 + (int)rank) * GP_EPI_WARPS + ew, 1);
          mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[buf]), 0));
        }
        buf ^= 1;
        if (buf == 0) acc_phase ^= 1;
        continue;
      }
      int n_parts = 0;  // partial tiles to add: the pairs after this one whose ranges reach into the tile
      if (finishes) {
        n_parts = partials_expected(tile, kblocks, p.sk_tiles, num_pairs, pair);
        int* flag = p.flags + (tile * 2 + (int)rank) * GP_EPI_WARPS + ew;
        int fine = 1;
        if (lane == 0) {
          fine = flag_wait(flag, n_parts, 0xc00 | ew, abort_flag) ? 1 : 0;
          if (fine) *flag = 0;  // this warp is the counter's only reader: hand it back cleared
        }
        fine = __shfl_sync(0xffffffffu, fine, 0);
        __syncwarp();  // lane 0's acquire orders the whole warp's reads of the partial tiles
        if (!fine) { ok = false; break; }
      }
#pragma unroll 1
      for (int st = 0; st < STEPS && ok; ++st) {
        const int col0 = n0 + st * 64;
        uint32_t r0[32], r1[32];
        tmem_ld32(taddr + st * 64, r0);
        tmem_ld32(taddr + st * 64 + 32, r1);
        tc_wait_ld();
        for (int c = 1; c <= n_parts; ++c) {
          // the same CTA rank of pair + c wrote this slot
          const float4* src = reinterpret_cast<const float4*>(p.partials) + (int64_t)(blockIdx.x + 2 * c) * slot_f4 +
                              my_f4 + st * 16 * GP_M;
          float4 v[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) v[e] = __ldcg(src + e * GP_M);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            r0[4 * e] = __float_as_uint(__uint_as_float(r0[4 * e]) + v[e].x);
            r0[4 * e + 1] = __float_as_uint(__uint_as_float(r0[4 * e + 1]) + v[e].y);
            r0[4 * e + 2] = __float_as_uint(__uint_as_float(r0[4 * e + 2]) + v[e].z);
            r0[4 * e + 3] = __float_as_uint(__uint_as_float(r0[4 * e + 3]) + v[e].w);
            r1[4 * e] = __float_as_uint(__uint_as_float(r1[4 * e]) + v[8 + e].x);
            r1[4 * e + 1] = __float_as_uint(__uint_as_float(r1[4 * e + 1]) + v[8 + e].y);
            r1[4 * e + 2] = __float_as_uint(__uint_as_float(r1[4 * e + 2]) + v[8 + e].z);
            r1[4 * e + 3] = __float_as_uint(__uint_as_float(r1[4 * e + 3]) + v[8 + e].w);
          }
        }
        if (use_x) {
          if (!mbar_wait(&x_full[ew], x_phase, 0xb00 | ew, abort_flag)) { ok = false; break; }
          x_phase ^= 1;
        }
        // the staging box of the previous step must have been read by the TMA unit
        if (lane == 0) tma_store_wait_read();
        __syncwarp();
#pragma unroll
        for (int v = 0; v < 8; ++v) {  // 16-byte chunks (8 columns) of this thread's row
          const int col = col0 + v * 8;
          float f[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v < 4 ? r0[v * 8 + j] : r1[(v - 4) * 8 + j]);
          if (bias && col < p.N) {
            if (col + 8 <= p.N) {
              float b[8];
              unpack8<T>(__ldg(reinterpret_cast<const uint4*>(bias + col)), b);
#pragma unroll
              for (int j = 0; j < 8; ++j) f[j] += b[j];
            } else {
              for (int j = 0; j < 8 && col + j < p.N; ++j) f[j] += Num<T>::to_f(bias[col + j]);
            }
          }
          if (p.relu) {
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = fmaxf(f[j], 0.f);
          }
          const uint32_t soff = lane * 128 + ((v ^ (lane & 7)) << 4);
          if (use_x) {
            float o[8];
            unpack8<T>(*reinterpret_cast<const uint4*>(stage_x + soff), o);
            if (x_is_addend) {
#pragma unroll
              for (int j = 0; j < 8; ++j) f[j] += o[j];
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j) f[j] = o[j] > 0.f ? f[j] : 0.f;
            }
          }
          if (mask_direct && row < p.M) {
            for (int j = 0; j < 8 && col + j < p.N; ++j)
              if (!(Num<T>::to_f(mask_direct[(int64_t)row * p.ld_mask + col + j]) > 0.f)) f[j] = 0.f;
          }
          *reinterpret_cast<uint4*>(stage_c + soff) = pack8<T>(f);
        }
        fence_proxy_async_smem();  // staged output visible to the TMA unit; addend box reads are done
        __syncwarp();
        if (lane == 0) {
          if (col0 < p.N && row0 < p.M) tma_store_2d(&tmC, stage_c, col0, row0);
          tma_store_commit();
          if (use_x && st + 1 < STEPS) {
            mbar_expect_tx(&x_full[ew], 4096);
            tma_load_2d(stage_x, &tmX, col0 + 64, row0, &x_full[ew]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[buf]), 0));
      if (prof && ew == 0 && lane == 0) { pr[9] += (unsigned long long)(clock64() - e1); pr[10] += 1; }  // epilogue busy, tiles
      buf ^= 1;
      if (buf == 0) acc_phase ^= 1;
    }
    if (lane == 0) tma_store_wait_all();
    if (prof && ew == 0 && lane == 0) pr[11] = (unsigned long long)(clock64() - t_entry);  // epilogue done
  }

  // Unwind: every role has left its loop (normally or through a bounded wait).
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  // neither CTA leaves (or frees tensor memory) while the other may still signal its barriers or
  // have MMAs reading its shared memory
  cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, GP_TMEM_COLS);
  }
  if (prof && threadIdx.x == 0) { pr[12] = (unsigned long long)(clock64() - t_entry); pr[13] = global_ns(); }
}

// Copies the timeline of CTA `cta` (16 words) to the host and clears it.
int gemm_pair_counters(int cta, unsigned long long* out) {
  if (cta < 0 || cta >= 148) return -1;
  cudaDeviceSynchronize();
  if (cudaMemcpyFromSymbol(out, g_pair_prof, sizeof(unsigned long long) * 16, sizeof(unsigned long long) * 16 * cta) !=
      cudaSuccess)
    return -1;
  unsigned long long z[16] = {0};
  cudaMemcpyToSymbol(g_pair_prof, z, sizeof(z), sizeof(unsigned long long) * 16 * cta);
  return 0;
}


int encode_tmap_sw128(CUtensorMap* out, const void* base, int dtype, int rank, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box);

template <typename T, bool A_MN, bool B_MN>
static int launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const CUtensorMap& tmX,
                       const PairParams& p, int grid, cudaStream_t st) {
  auto kern = gemm_pair_tc05_kernel<T, A_MN, B_MN>;
  static std::atomic<uint64_t> attr_done{0};
  if (int rc0 = ensure_dynamic_smem(kern, GP_SMEM_BYTES, attr_done, "gemm_pair_tc05")) return rc0;
  launch_overlapped(kern, dim3(grid), dim3(GP_THREADS), GP_SMEM_BYTES, st, tmA, tmB, tmC, tmX, p);
  return launched("gemm_pair_tc05");
}

// Pair tiles the output offers; the caller takes this kernel when they fill the pairs of SMs.
int64_t gemm_pair_tiles(int64_t M, int64_t N) { return ceil_div(M, 2 * GP_M) * ceil_div(N, GP_N); }

// Work split of the pair kernel.  `workspace` may be null (whole tiles only).  Returns the number of
// pairs to launch and sets *sk_tiles.
static int64_t pair_schedule(int64_t tiles, int64_t kblocks, int64_t pairs, bool can_split, int64_t* sk_tiles) {
  *sk_tiles = 0;
  if (!can_split) return tiles < pairs ? tiles : pairs;
  // With at least one tile per pair the tiles are handed out whole: cutting the tiles of a partial
  // last wave along K (tried, also with the cut tiles done first) balances the pairs but does not
  // shorten the kernel - with fewer pairs busy in the last wave each runs its k-blocks faster, and
  // the partial tiles add traffic.
  if (tiles >= pairs) return pairs;
  // fewer tiles than pairs: as many pairs as leave each at least 8 k-blocks and each tile about 8 parts
  int64_t g = tiles * kblocks / 8;
  if (g > pairs) g = pairs;
  if (g > tiles * 8) g = tiles * 8;
  if (g * 4 >= tiles * 5 && tiles * 16 * 4 <= kFlagBytes) { *sk_tiles = tiles; return g; }
  return tiles;
}

int gemm_pair_tc05(const void* a, const void* b, void* c, const void* bias, const void* addend, int64_t ld_addend,
                   const void* mask, int64_t ld_mask, int64_t M, int64_t N, int64_t K, int64_t a_sm, int64_t a_sk,
                   int64_t b_sk, int64_t b_sn, int64_t ldc, int relu, int dtype, int sms, void* workspace,
                   cudaStream_t st) {
  const bool a_mn = (a_sk != 1), b_mn = (b_sk != 1);
  CUtensorMap tmA, tmB, tmC, tmX;
  int rc;
  {
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)M}, str[1] = {(uint64_t)ldc * 2};
    uint32_t box[2] = {64, 32};
    if ((rc = encode_tmap_sw128(&tmC, c, dtype, 2, dims, str, box))) return rc;
    const void* xp = addend ? addend : mask;
    str[0] = (uint64_t)(addend ? ld_addend : ld_mask) * 2;
    if (xp) { if ((rc = encode_tmap_sw128(&tmX, xp, dtype, 2, dims, str, box))) return rc; }
    else tmX = tmC;
  }
  {
    uint64_t dims[2], str[1];
    uint32_t box[2];
    if (a_mn) { dims[0] = (uint64_t)M; dims[1] = (uint64_t)K; str[0] = (uint64_t)a_sk * 2; box[0] = 64; box[1] = GP_K; }
    else      { dims[0] = (uint64_t)K; dims[1] = (uint64_t)M; str[0] = (uint64_t)a_sm * 2; box[0] = GP_K; box[1] = GP_M; }
    if ((rc = encode_tmap_sw128(&tmA, a, dtype, 2, dims, str, box))) return rc;
    if (b_mn) { dims[0] = (uint64_t)N; dims[1] = (uint64_t)K; str[0] = (uint64_t)b_sk * 2; box[0] = 64; box[1] = GP_K; }
    else      { dims[0] = (uint64_t)K; dims[1] = (uint64_t)N; str[0] = (uint64_t)b_sn * 2; box[0] = GP_K; box[1] = GP_NH; }
    if ((rc = encode_tmap_sw128(&tmB, b, dtype, 2, dims, str, box))) return rc;
  }
  PairParams p;
  p.C = c; p.bias = bias; p.addend = addend; p.mask = mask;
  p.M = (int)M; p.N = (int)N; p.K = (int)K; p.ldc = ldc; p.ld_addend = ld_addend; p.ld_mask = ld_mask;
  p.relu = relu; p.debug = g_gemm_debug.load();
  p.tiles_m = (int)ceil_div(M, 2 * GP_M); p.tiles_n = (int)ceil_div(N, GP_N);
  const int64_t tiles = (int64_t)p.tiles_m * p.tiles_n;
  int64_t sk_tiles = 0;
  const int64_t pairs = pair_schedule(tiles, ceil_div(K, GP_K), sms / 2, workspace != nullptr && !(p.debug & 1), &sk_tiles);
  p.sk_tiles = (int)sk_tiles;
  p.flags = reinterpret_cast<int*>(workspace);
  p.partials = workspace ? reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + kFlagBytes) : nullptr;
  const int grid = (int)(2 * pairs);
  TFB_DISPATCH_16(dtype, T, {
    if (a_mn && b_mn) return launch_pair<T, true, true>(tmA, tmB, tmC, tmX, p, grid, st);
    if (a_mn) return launch_pair<T, true, false>(tmA, tmB, tmC, tmX, p, grid, st);
    if (b_mn) return launch_pair<T, false, true>(tmA, tmB, tmC, tmX, p, grid, st);
    return launch_pair<T, false, false>(tmA, tmB, tmC, tmX, p, grid, st);
  })
}

}  // namespace tfb
