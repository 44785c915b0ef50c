// tcgen05 / TMEM GEMM for sm_100a.
//
//   C[M,N] = act(A·B + bias) (+ C), fp16/bf16 operands, fp32 accumulation in tensor memory.
//
// Persistent CTAs (one per SM) walk 128 x BN output tiles.  Per CTA:
//   warp 0  : TMA producer  - 128-byte-swizzled operand tiles into a STAGES-deep smem ring
//   warp 1  : MMA issuer    - one elected lane issues tcgen05.mma (M=128, N=BN, K=16) into one
//                             of two TMEM accumulator buffers, commits ring slots back
//   warps 2-5: epilogue     - tcgen05.ld the finished accumulator (each warp its 32 lanes),
//                             bias / ReLU / addend / mask in fp32, round once into a swizzled smem
//                             box, TMA store (the addend / mask box arrives by TMA load); overlaps
//                             the next tile's main loop through the second accumulator buffer
// Work split ("stream-K"): when there are fewer tiles than SMs, the tiles are cut along K into one
// equal, contiguous range of k-blocks per CTA (the scheduler also handles a split region followed by
// whole tiles).  A CTA whose range starts inside a tile writes that fp32 partial tile to its
// own workspace slot and raises the tile's flags; the CTA that owns the tile's first k-blocks (its
// last piece of the range, so the others are long done) adds the partials in CTA order and runs the
// epilogue.  The sum order is fixed, so results do not depend on timing.
// Either operand may be K-major (contraction index contiguous) or MN-major, so the forward
// product X·W, the input gradient dY·Wᵀ and the weight gradient Xᵀ·dY (contraction over every
// token of the batch, i.e. the batch reduction fused into the product) are the same kernel.
#include "gemm_sched.cuh"
#include <type_traits>

namespace tfb {

extern std::atomic<int> g_gemm_debug;
extern std::atomic<int> g_gemm_free_sms;
int64_t gemm_pair_tiles(int64_t M, int64_t N);
int gemm_pair_tc05(const void* a, const void* b, void* c, const void* bias, const void* addend, int64_t ld_addend,
                   const void* mask, int64_t ld_mask, int64_t M, int64_t N, int64_t K, int64_t a_sm, int64_t a_sk,
                   int64_t b_sk, int64_t b_sn, int64_t ldc, int relu, int dtype, int sms, void* workspace,
                   cudaStream_t st);

constexpr int TB_M = 128;
constexpr int TB_K = 64;  // 64 sixteen-bit elements = one 128-byte swizzle row
constexpr int TB_THREADS = 192;

template <int BN> struct GemmCfg {
  static constexpr int A_BYTES = TB_M * TB_K * 2;
  static constexpr int B_BYTES = BN * TB_K * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int EPI_BYTES = 4 * 4096;  // per epilogue warp: one 32-row x 64-column 16-bit box
  static constexpr int OFF_EPI_C = STAGES * STAGE_BYTES;       // output staging for the TMA store
  static constexpr int OFF_EPI_X = OFF_EPI_C + EPI_BYTES;      // addend / mask staging filled by TMA
  static constexpr int OFF_BAR = OFF_EPI_X + EPI_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 1024 /*align slack*/ + 256 /*barriers*/;
  static constexpr int TMEM_COLS = 2 * BN;
};

struct GemmParams {
  void* C;
  const void* bias;
  const void* addend;  // added after bias/ReLU (the residual stream, or C itself to accumulate); may be null
  const void* mask;    // result is zeroed where mask <= 0 (a saved ReLU output); may be null
  int* flags;          // stream-K: 4 arrival counters per split tile (one per epilogue warp), zero between kernels
  float* partials;     // stream-K: one fp32 128 x BN slot per CTA
  int M, N, K;
  int64_t ldc, ld_addend, ld_mask;
  int relu;
  int tiles_m, tiles_n;
  int sk_tiles;        // tiles [0, sk_tiles) are split along K over all CTAs; 0 = whole tiles only
};

template <typename T, int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(TB_THREADS, 1) gemm_tc05_kernel(const __grid_constant__ CUtensorMap tmA,
                                                                  const __grid_constant__ CUtensorMap tmB,
                                                                  const __grid_constant__ CUtensorMap tmC,
                                                                  const __grid_constant__ CUtensorMap tmX,
                                                                  const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the swizzle pattern is a function of the shared-memory address
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* full = bars;                    // [STAGES] TMA -> MMA
  uint64_t* empty = bars + STAGES;          // [STAGES] MMA -> TMA
  uint64_t* acc_full = bars + 2 * STAGES;   // [2] MMA -> epilogue
  uint64_t* acc_empty = acc_full + 2;       // [2] epilogue -> MMA
  uint64_t* x_full = acc_empty + 2;         // [4] addend / mask box of an epilogue warp landed
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(x_full + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 4);  // one arrival per epilogue warp
    }
    for (int i = 0; i < 4; ++i) mbar_init(&x_full[i], 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc(tmem_holder, Cfg::TMEM_COLS);
  }
  // everything above touches only this CTA's shared memory, TMEM and kernel parameters, so it may
  // run while the previous kernel of the stream is still finishing; global memory comes after this
  grid_dependency_wait();
  allow_dependents();
  // an earlier kernel that gave up leaves the status set: then this one does nothing
  if (threadIdx.x == 0) *abort_flag = (*(volatile int*)&g_dev_status != 0) ? 1 : 0;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  const int kblocks_all = (p.K + TB_K - 1) / TB_K;
  const bool dead = *abort_flag != 0;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      Segments segs(kblocks_all, p.tiles_m * p.tiles_n, p.sk_tiles, (int)gridDim.x, (int)blockIdx.x, dead);
      int tile, kb0, kb1;
      while (ok && segs.next(tile, kb0, kb1)) {
        const int m0 = (tile % p.tiles_m) * TB_M;
        const int n0 = (tile / p.tiles_m) * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, 0x100 | stage, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          mbar_expect_tx(&full[stage], Cfg::STAGE_BYTES);
          const int k0 = kb * TB_K;
          if (A_MN) {
#pragma unroll
            for (int i = 0; i < TB_M / 64; ++i) tma_load_2d(sa + i * 8192, &tmA, m0 + i * 64, k0, &full[stage]);
          } else {
            tma_load_2d(sa, &tmA, k0, m0, &full[stage]);
          }
          if (B_MN) {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i) tma_load_2d(sb + i * 8192, &tmB, n0 + i * 64, k0, &full[stage]);
          } else {
            tma_load_2d(sb, &tmB, k0, n0, &full[stage]);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc_f16(TB_M, BN, sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1 : 0,
                                                A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      Segments segs(kblocks_all, p.tiles_m * p.tiles_n, p.sk_tiles, (int)gridDim.x, (int)blockIdx.x, dead);
      int tile, kb0, kb1;
      while (ok && segs.next(tile, kb0, kb1)) {
        if (!mbar_wait(&acc_empty[buf], acc_phase ^ 1, 0x300 | buf, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full[stage], phase, 0x200 | stage, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < TB_K / 16; ++k) {
            // K-major: 16 elements = 32 bytes along the swizzled row; MN-major: 16 k-rows of 128 B
            const uint64_t ad = A_MN ? smem_desc_sw128(sa + k * 2048, 8192, 1024)
                                     : smem_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t bd = B_MN ? smem_desc_sw128(sb + k * 2048, 8192, 1024)
                                     : smem_desc_sw128(sb + k * 32, 16, 1024);
            tc_mma_ss(d_tmem, ad, bd, idesc, ((kb - kb0) | k) ? 1u : 0u);
          }
          tc_commit(&empty[stage]);  // slot reusable once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit(&acc_full[buf]);  // accumulator complete
        buf ^= 1;
        if (buf == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ---------------------------------------------------------------------- epilogue
    // Each warp owns 32 accumulator rows.  Per 64-column step it reads its TMEM slice, applies
    // bias / ReLU / addend / mask in fp32, rounds once into a swizzled 32 x 64 box in shared memory
    // and hands the box to the TMA unit, which writes full 128-byte rows and clips at the matrix
    // edges.  The addend or mask box of the next step is fetched by TMA while this one is computed.
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int ew = warp - 2; // 0..3: index of this warp's staging boxes and barrier
    const T* bias = reinterpret_cast<const T*>(p.bias);
    uint8_t* stage_c = smem + Cfg::OFF_EPI_C + ew * 4096;
    uint8_t* stage_x = smem + Cfg::OFF_EPI_X + ew * 4096;
    // at most one of addend / mask travels through the TMA box; a second one is read directly
    const bool x_is_addend = p.addend != nullptr;
    const bool use_x = (p.addend != nullptr || p.mask != nullptr);
    const T* mask_direct = (p.addend != nullptr && p.mask != nullptr) ? reinterpret_cast<const T*>(p.mask) : nullptr;
    constexpr int STEPS = BN / 64;
    int buf = 0;
    uint32_t acc_phase = 0, x_phase = 0;
    bool ok = true;
    if (lane == 0) {
      tma_prefetch_desc(&tmC);
      if (use_x) tma_prefetch_desc(&tmX);
    }
    Segments segs(kblocks_all, p.tiles_m * p.tiles_n, p.sk_tiles, (int)gridDim.x, (int)blockIdx.x, dead);
    int tile, kb0, kb1;
    while (ok && segs.next(tile, kb0, kb1)) {
      const int m0 = (tile % p.tiles_m) * TB_M;
      const int n0 = (tile / p.tiles_m) * BN;
      const int row0 = m0 + q * 32;       // first row of this warp's slice
      const int row = row0 + lane;
      const bool contributes = kb0 > 0;                      // a later part of a split tile
      const bool finishes = kb0 == 0 && kb1 < kblocks_all;   // first part of a split tile: owns its epilogue
      if (use_x && !contributes && lane == 0) {  // box of step 0, in flight while the main loop still runs
        mbar_expect_tx(&x_full[ew], 4096);
        tma_load_2d(stage_x, &tmX, n0, row0, &x_full[ew]);
      }
      if (!mbar_wait(&acc_full[buf], acc_phase, 0x400 | buf, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
      if (contributes) {
        // fp32 partial of this warp's 32 rows into this CTA's slot, then one arrival on the tile's counter
        // slot layout [column group of 4][row]: the 32 lanes of a warp touch 512 contiguous bytes
        float4* slot = reinterpret_cast<float4*>(p.partials + (int64_t)blockIdx.x * TB_M * BN) + q * 32 + lane;
#pragma unroll 1
        for (int st = 0; st < STEPS; ++st) {
          uint32_t r0[32], r1[32];
          tmem_ld32(taddr + st * 64, r0);
          tmem_ld32(taddr + st * 64 + 32, r1);
          tc_wait_ld();
          float4* dst = slot + st * 16 * TB_M;
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            __stcg(dst + e * TB_M, make_float4(__uint_as_float(r0[4 * e]), __uint_as_float(r0[4 * e + 1]),
                                        __uint_as_float(r0[4 * e + 2]), __uint_as_float(r0[4 * e + 3])));
            __stcg(dst + (8 + e) * TB_M, make_float4(__uint_as_float(r1[4 * e]), __uint_as_float(r1[4 * e + 1]),
                                            __uint_as_float(r1[4 * e + 2]), __uint_as_float(r1[4 * e + 3])));
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          __threadfence();  // the warp's partial rows are visible before the arrival
          atomicAdd(p.flags + tile * 4 + q, 1);
          mbar_arrive(&acc_empty[buf]);
        }
        buf ^= 1;
        if (buf == 0) acc_phase ^= 1;
        continue;
      }
      int n_parts = 0;  // partial tiles to add: the CTAs after this one whose ranges reach into the tile
      if (finishes) {
        n_parts = partials_expected(tile, kblocks_all, p.sk_tiles, (int)gridDim.x, (int)blockIdx.x);
        int* flag = p.flags + tile * 4 + q;
        int fine = 1;
        if (lane == 0) {
          fine = flag_wait(flag, n_parts, 0x600 | q, abort_flag) ? 1 : 0;
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
          // all sixteen loads of this thread's 64 columns are issued before the first add
          const float4* src = reinterpret_cast<const float4*>(p.partials + (int64_t)(blockIdx.x + c) * TB_M * BN) +
                              st * 16 * TB_M + q * 32 + lane;
          float4 v[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) v[e] = __ldcg(src + e * TB_M);
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
          if (!mbar_wait(&x_full[ew], x_phase, 0x500 | ew, abort_flag)) { ok = false; break; }
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
          if (use_x) {  // next box: the next step of this tile, or nothing (step 0 of the next tile is issued above)
            if (st + 1 < STEPS) {
              mbar_expect_tx(&x_full[ew], 4096);
              tma_load_2d(stage_x, &tmX, col0 + 64, row0, &x_full[ew]);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
      buf ^= 1;
      if (buf == 0) acc_phase ^= 1;
    }
    if (lane == 0) tma_store_wait_all();  // global writes of this warp are complete before the CTA exits
  }

  // Unwind: every role has left its loop (normally or through a bounded wait).
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // give copies that may still be in flight time to land before the CTA's smem goes away
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                             const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                             CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn get_encoder() {
  static EncodeFn fn = []() -> EncodeFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
    if (q != cudaDriverEntryPointSuccess) return nullptr;
    return reinterpret_cast<EncodeFn>(p);
  }();
  return fn;
}

static int encode_tmap(CUtensorMap* out, const void* base, int dtype, int rank, const uint64_t* dims,
                       const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle) {
  EncodeFn enc = get_encoder();
  if (!enc) return fail(TFB_ERR_DRIVER, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[5], gstr[5];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i + 1 < rank) gstr[i] = strides_bytes[i];
  }
  const CUtensorMapDataType dt = dtype == TFB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                 : dtype == TFB_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                                    : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = enc(out, dt, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bx, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TFB_ERR_DRIVER, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return TFB_OK;
}

// Boxes whose rows are 128 bytes in shared memory, 16-byte chunks swizzled over eight rows.
int encode_tmap_sw128(CUtensorMap* out, const void* base, int dtype, int rank, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box) {
  return encode_tmap(out, base, dtype, rank, dims, strides_bytes, box, CU_TENSOR_MAP_SWIZZLE_128B);
}


// Arrival counters plus one fp32 128 x 256 partial tile per SM.
int64_t gemm_tc05_workspace_bytes() { return kFlagBytes + (int64_t)sm_count() * TB_M * 256 * (int64_t)sizeof(float); }

template <typename T, int BN, bool A_MN, bool B_MN>
static int launch_tc05(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const CUtensorMap& tmX,
                       const GemmParams& p, int grid, cudaStream_t st) {
  using Cfg = GemmCfg<BN>;
  auto kern = gemm_tc05_kernel<T, BN, A_MN, B_MN>;
  static std::atomic<uint64_t> attr_done{0};
  if (int rc0 = ensure_dynamic_smem(kern, Cfg::SMEM_BYTES, attr_done, "gemm_tc05")) return rc0;
  launch_overlapped(kern, dim3(grid), dim3(TB_THREADS), Cfg::SMEM_BYTES, st, tmA, tmB, tmC, tmX, p);
  return launched("gemm_tc05");
}

template <typename T, int BN>
static int dispatch_major(bool a_mn, bool b_mn, const CUtensorMap& tmA, const CUtensorMap& tmB,
                          const CUtensorMap& tmC, const CUtensorMap& tmX, const GemmParams& p, int grid,
                          cudaStream_t st) {
  if (a_mn && b_mn) return launch_tc05<T, BN, true, true>(tmA, tmB, tmC, tmX, p, grid, st);
  if (a_mn) return launch_tc05<T, BN, true, false>(tmA, tmB, tmC, tmX, p, grid, st);
  if (b_mn) return launch_tc05<T, BN, false, true>(tmA, tmB, tmC, tmX, p, grid, st);
  return launch_tc05<T, BN, false, false>(tmA, tmB, tmC, tmX, p, grid, st);
}

// Whether (ptr, strides) can be described by a TMA tensor map of 16-bit elements.
static bool tma_ok(const void* ptr, int64_t s_outer) { return aligned16(ptr) && s_outer % 8 == 0 && s_outer > 0; }

bool gemm_tc05_eligible(const void* a, const void* b, const void* c, const void* bias, const void* addend,
                        int64_t ld_addend, const void* mask, int64_t ld_mask, int64_t M, int64_t N, int64_t K,
                        int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn, int64_t ldc) {
  if (addend && !(aligned16(addend) && ld_addend % 8 == 0)) return false;
  if (mask && !(aligned16(mask) && ld_mask % 8 == 0)) return false;
  if (M < 1 || N < 1 || K < 1) return false;
  if (M >= (1LL << 31) || N >= (1LL << 31) || K >= (1LL << 31)) return false;
  const bool a_ok = (a_sk == 1) ? tma_ok(a, a_sm) : (a_sm == 1 && tma_ok(a, a_sk));
  const bool b_ok = (b_sk == 1) ? tma_ok(b, b_sn) : (b_sn == 1 && tma_ok(b, b_sk));
  // A tensor of extent 1 along its strided dim still needs a legal stride; callers pass real strides.
  return a_ok && b_ok && aligned16(c) && ldc % 8 == 0 && (bias == nullptr || aligned16(bias));
}

int gemm_tc05(const void* a, const void* b, void* c, const void* bias, const void* addend, int64_t ld_addend,
              const void* mask, int64_t ld_mask, int64_t M, int64_t N, int64_t K, int64_t a_sm, int64_t a_sk,
              int64_t b_sk, int64_t b_sn, int64_t ldc, int relu, int dtype, void* workspace,
              int64_t workspace_bytes, cudaStream_t st) {
  const bool a_mn = (a_sk != 1);  // M contiguous
  const bool b_mn = (b_sk != 1);  // N contiguous
  const int64_t tm = ceil_div(M, TB_M);
  // SMs left to a collective that runs beside the GEMMs: a persistent grid sized for every SM would have its
  // last CTAs wait for one the collective holds, and the whole product would take two rounds
  int sms = sm_count() - g_gemm_free_sms.load();
  sms = sms < 2 ? 2 : sms & ~1;
  const int64_t kblocks = ceil_div(K, TB_K);
  const int dbg = g_gemm_debug.load();
  const bool can_split = !(dbg & 1) && workspace != nullptr && aligned16(workspace) &&
                         workspace_bytes >= gemm_tc05_workspace_bytes();
  // Outputs of at least 256 x 256 that can occupy the pairs of SMs run on CTA pairs (a third less
  // operand traffic per flop): either a 256 x 256 tile for every pair, or a tile for at least every
  // second pair and enough k-blocks to share.
  {
    const int64_t pt = gemm_pair_tiles(M, N);
    if (!(dbg & 32) && M >= 256 && N >= 256 &&
        (pt >= sms / 2 || (can_split && pt * 2 >= sms / 2 && pt * kblocks >= (int64_t)(sms / 2) * 8)))
      return gemm_pair_tc05(a, b, c, bias, addend, ld_addend, mask, ld_mask, M, N, K, a_sm, a_sk, b_sk, b_sn, ldc,
                            relu, dtype, sms, can_split ? workspace : nullptr, st);
  }
  // Tile width: fewest "waves x tile cost" over the SMs; the wide tile moves fewer operand bytes per
  // flop, so the narrow one has to win by a clear margin.
  const int64_t cost256 = ceil_div(tm * ceil_div(N, 256), sms) * 256;
  const int64_t cost128 = ceil_div(tm * ceil_div(N, 128), sms) * 128;
  int BN = (N <= 128 || cost128 * 10 < cost256 * 9) ? 128 : 256;
  // Outputs with fewer tiles than SMs (weight gradients: small M x N, contraction over every token)
  // share the K range of each tile between CTAs.  This pays only here: with more tiles than SMs the
  // kernel is bound by operand traffic rather than by idle SMs in the last wave (measured), and the
  // partial tiles would add to that traffic.  Very small outputs take the narrow tile so that a tile
  // has fewer partials to add.
  if (can_split && N > 128 && tm * ceil_div(N, 256) < sms) BN = (tm * ceil_div(N, 256) * 3 <= sms) ? 128 : 256;
  const int64_t tiles = tm * ceil_div(N, BN);
  int64_t grid = tiles < sms ? tiles : sms;
  int64_t sk_tiles = 0;
  if (can_split && tiles < sms) {
    // as many CTAs as leave each at least 8 k-blocks and each tile at most about 8 parts
    int64_t g = tiles * kblocks / 8;
    if (g > sms) g = sms;
    if (g > tiles * 8) g = tiles * 8;
    if (g * 4 >= tiles * 5 && tiles * 16 <= kFlagBytes) { grid = g; sk_tiles = tiles; }
  }

  CUtensorMap tmA, tmB, tmC, tmX;
  int rc;
  {
    // output and addend/mask: (N inner, M outer), boxes of 64 columns x 32 rows
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
    if (a_mn) { dims[0] = (uint64_t)M; dims[1] = (uint64_t)K; str[0] = (uint64_t)a_sk * 2; box[0] = 64; box[1] = TB_K; }
    else      { dims[0] = (uint64_t)K; dims[1] = (uint64_t)M; str[0] = (uint64_t)a_sm * 2; box[0] = TB_K; box[1] = TB_M; }
    if ((rc = encode_tmap_sw128(&tmA, a, dtype, 2, dims, str, box))) return rc;
    if (b_mn) { dims[0] = (uint64_t)N; dims[1] = (uint64_t)K; str[0] = (uint64_t)b_sk * 2; box[0] = 64; box[1] = TB_K; }
    else      { dims[0] = (uint64_t)K; dims[1] = (uint64_t)N; str[0] = (uint64_t)b_sn * 2; box[0] = TB_K; box[1] = (uint32_t)BN; }
    if ((rc = encode_tmap_sw128(&tmB, b, dtype, 2, dims, str, box))) return rc;
  }
  GemmParams p;
  p.C = c; p.bias = bias; p.addend = addend; p.mask = mask;
  p.flags = sk_tiles ? reinterpret_cast<int*>(workspace) : nullptr;
  p.partials = sk_tiles ? reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + kFlagBytes) : nullptr;
  p.M = (int)M; p.N = (int)N; p.K = (int)K; p.ldc = ldc; p.ld_addend = ld_addend; p.ld_mask = ld_mask;
  p.relu = relu;
  p.tiles_m = (int)tm; p.tiles_n = (int)ceil_div(N, BN); p.sk_tiles = (int)sk_tiles;
  TFB_DISPATCH_16(dtype, T, {
    if (BN == 256) return dispatch_major<T, 256>(a_mn, b_mn, tmA, tmB, tmC, tmX, p, (int)grid, st);
    return dispatch_major<T, 128>(a_mn, b_mn, tmA, tmB, tmC, tmX, p, (int)grid, st);
  })
}

}  // namespace tfb
