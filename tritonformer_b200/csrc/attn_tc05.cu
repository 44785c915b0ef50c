// Causal flash attention forward on tcgen05 / TMEM for sm_100a (head_dim 64 or 128, T % 128 == 0).
//
// One CTA per (128-query tile, batch*head).  Roles:
//   warp 0    : TMA producer - Q once, then K_j / V_j tiles (128 keys) through 2-stage rings;
//               4-D tensor maps over the caller's (hd, T, H, B) strides, 128-byte swizzle
//   warp 1    : MMA issuer   - S_j = Q K_jᵀ into one of two TMEM score buffers (so the next
//               tile's scores are computed while this tile's softmax runs), then O += P_j V_j
//   warps 2-5 : softmax      - thread == query row == TMEM lane: reads its score row, applies
//               scale / ALiBi / causal mask in the log2 domain, keeps the running max and sum,
//               rescales its O row in TMEM, writes P_j (16-bit) into swizzled shared memory for
//               the second product; at the end normalises O and stores it with the row's
//               log-sum-exp
// TMEM columns: [0,128) S even tiles, [128,256) S odd tiles, [256,256+hd) O.
#include "attn.cuh"
#include "tc05.cuh"
#include <type_traits>

namespace tfb {

constexpr float kLog2e_ = 1.4426950408889634f;
constexpr float kLn2_ = 0.6931471805599453f;
constexpr int FA_M = 128, FA_N = 128, FA_THREADS = 192;

template <int HD> struct FaCfg {
  static constexpr int PANELS = HD / 64;             // 64-element (128-byte) panels along head_dim
  static constexpr int TILE_BYTES = PANELS * 16384;  // 128 rows x HD x 2 bytes
  static constexpr int P_BYTES = 2 * 16384;          // 128 x 128 x 2 bytes
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = TILE_BYTES;
  static constexpr int OFF_V = OFF_K + 2 * TILE_BYTES;
  static constexpr int OFF_P = OFF_V + 2 * TILE_BYTES;
  static constexpr int OFF_BAR = OFF_P + P_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  static constexpr int TMEM_COLS = 512;
  static constexpr int COL_O = 256;
};

struct FaParams {
  void* out;
  float* lse;
  int64_t so_b, so_h, so_t;
  int H, T;
  float scale;
  int bias_mode;  // 0 none, 1 ALiBi fp32, 2 / 4 ALiBi rounded like an fp16 / bf16 table
  const float* slopes;
};

__device__ __forceinline__ float alibi_term(int mode, float slope, int dist) {
  // this kernel has conversion-pipe slack: the 16-bit multiply measured faster here than the integer rounding
  if (mode == 1) return -slope * (float)dist;
  if (mode == 2) return __half2float(__hmul(__float2half_rn(-(float)dist), __float2half_rn(slope)));
  return __bfloat162float(__hmul(__float2bfloat16_rn(-(float)dist), __float2bfloat16_rn(slope)));
}

template <typename T, int HD>
__global__ void __launch_bounds__(FA_THREADS, 1) attn_fwd_tc05_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                                      const __grid_constant__ CUtensorMap tmK,
                                                                      const __grid_constant__ CUtensorMap tmV,
                                                                      const FaParams p) {
  using Cfg = FaCfg<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2] MMA -> softmax
  uint64_t* s_free = bars + 11;   // [2] softmax -> MMA (score buffer read)
  uint64_t* p_full = bars + 13;   // softmax -> MMA (P in smem, O rescaled)
  uint64_t* pv_done = bars + 14;  // MMA -> softmax (P buffer and O may be touched again)
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;  // longest rows first
  const int bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  const int q0 = qt * FA_M;
  const int ntiles = qt + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 4);
    }
    mbar_init(p_full, 4);
    mbar_init(pv_done, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc(tmem_holder, Cfg::TMEM_COLS);
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
      mbar_expect_tx(q_full, Cfg::TILE_BYTES);
#pragma unroll
      for (int c = 0; c < Cfg::PANELS; ++c) tma_load_4d(smem + Cfg::OFF_Q + c * 16384, &tmQ, c * 64, q0, h, b, q_full);
      for (int j = 0; j < ntiles; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_empty[st], ph ^ 1, 0x1100 | st, abort_flag)) break;
        mbar_expect_tx(&k_full[st], Cfg::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < Cfg::PANELS; ++c)
          tma_load_4d(smem + Cfg::OFF_K + st * Cfg::TILE_BYTES + c * 16384, &tmK, c * 64, j * FA_N, h, b, &k_full[st]);
        if (!mbar_wait(&v_empty[st], ph ^ 1, 0x1200 | st, abort_flag)) break;
        mbar_expect_tx(&v_full[st], Cfg::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < Cfg::PANELS; ++c)
          tma_load_4d(smem + Cfg::OFF_V + st * Cfg::TILE_BYTES + c * 16384, &tmV, c * 64, j * FA_N, h, b, &v_full[st]);
      }
    }
  } else if (warp == 1) {
    // ----------------------------------------------------------------------- MMA issuer
    if (lane == 0 && !dead) {
      constexpr int fmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t idesc_s = instr_desc_f16(FA_M, FA_N, fmt, 0, 0);
      constexpr uint32_t idesc_o = instr_desc_f16(FA_M, HD, fmt, 0, 1);
      const uint32_t sq = smem_u32(smem + Cfg::OFF_Q);
      const uint32_t sp = smem_u32(smem + Cfg::OFF_P);
      bool ok = mbar_wait(q_full, 0, 0x1300, abort_flag);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_full[st], ph, 0x1400 | st, abort_flag)) return false;
        if (!mbar_wait(&s_free[st], ph ^ 1, 0x1500 | st, abort_flag)) return false;
        tc_fence_after();
        const uint32_t sk = smem_u32(smem + Cfg::OFF_K + st * Cfg::TILE_BYTES);
#pragma unroll
        for (int s = 0; s < HD / 16; ++s) {
          const uint32_t off = (s / 4) * 16384 + (s % 4) * 32;
          tc_mma_ss(tmem_base + st * FA_N, smem_desc_sw128(sq + off, 16, 1024), smem_desc_sw128(sk + off, 16, 1024),
                    idesc_s, s ? 1u : 0u);
        }
        tc_commit(&k_empty[st]);
        tc_commit(&s_full[st]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < ntiles && ok; ++j) {
        if (j + 1 < ntiles && !issue_s(j + 1)) { ok = false; break; }
        const int st = j & 1;
        if (!mbar_wait(p_full, j & 1, 0x1600, abort_flag)) { ok = false; break; }
        if (!mbar_wait(&v_full[st], (j >> 1) & 1, 0x1700 | st, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sv = smem_u32(smem + Cfg::OFF_V + st * Cfg::TILE_BYTES);
#pragma unroll
        for (int s = 0; s < FA_N / 16; ++s) {
          const uint64_t ad = smem_desc_sw128(sp + (s / 4) * 16384 + (s % 4) * 32, 16, 1024);
          const uint64_t bd = smem_desc_sw128(sv + s * 2048, 16384, 1024);  // MN-major: 16 key rows per step
          tc_mma_ss(tmem_base + Cfg::COL_O, ad, bd, idesc_o, (j | s) ? 1u : 0u);
        }
        tc_commit(&v_empty[st]);
        tc_commit(pv_done);
      }
    }
  } else if (!dead) {
    // -------------------------------------------------------------------------- softmax
    const int qd = warp & 3;
    const int r = qd * 32 + lane;      // query row within the tile == TMEM lane
    const int i = q0 + r;              // global query index
    const uint32_t lane_addr = tmem_base + ((uint32_t)(qd * 32) << 16);
    const float c2 = p.scale * kLog2e_;
    const float slope = p.bias_mode ? p.slopes[h] : 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    uint8_t* sp = smem + Cfg::OFF_P;
    bool ok = true;
    for (int j = 0; j < ntiles && ok; ++j) {
      const int st = j & 1;
      const int j0 = j * FA_N;
      const bool diag = (j == ntiles - 1);
      if (!mbar_wait(&s_full[st], (j >> 1) & 1, 0x1800 | st, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint32_t s_addr = lane_addr + st * FA_N;
      // pass 1: row maximum of the scaled, biased, masked scores
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < FA_N / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(s_addr + c * 32, v);
        tc_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const int jj = j0 + c * 32 + e;
          float x = __uint_as_float(v[e]) * c2;
          if (p.bias_mode) x += alibi_term(p.bias_mode, slope, max(i - jj, 0)) * kLog2e_;
          if (diag && jj > i) x = -INFINITY;
          mx = fmaxf(mx, x);
        }
      }
      const float m_new = fmaxf(m_run, mx);
      const float corr = exp2f(m_run - m_new);  // 0 on the first tile
      // the previous P·V must have retired before P's buffer and O are touched
      if (j > 0 && !mbar_wait(pv_done, (j - 1) & 1, 0x1900, abort_flag)) { ok = false; break; }
      tc_fence_after();
      if (j > 0) {
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t v[32];
          tmem_ld32(lane_addr + Cfg::COL_O + c * 32, v);
          tc_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * corr);
          tmem_st32(lane_addr + Cfg::COL_O + c * 32, v);
        }
      }
      // pass 2: p = 2^(s - m), row sum, P to swizzled smem (K-major A operand of P·V)
      float ls = 0.f;
#pragma unroll 1
      for (int c = 0; c < FA_N / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(s_addr + c * 32, v);
        tc_wait_ld();
        float f[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const int jj = j0 + c * 32 + e;
          float x = __uint_as_float(v[e]) * c2;
          if (p.bias_mode) x += alibi_term(p.bias_mode, slope, max(i - jj, 0)) * kLog2e_;
          float pe = exp2f(x - m_new);
          if (diag && jj > i) pe = 0.f;
          f[e] = pe;
          ls += pe;
        }
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          float g[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) g[e] = f[v4 * 8 + e];
          const int cc = c * 4 + v4;  // 16-byte chunk index along the 128 keys
          uint8_t* dst = sp + (cc >> 3) * 16384 + r * 128 + (((cc & 7) ^ (r & 7)) << 4);
          *reinterpret_cast<uint4*>(dst) = pack8<T>(g);
        }
      }
      m_run = m_new;
      l_run = l_run * corr + ls;
      // score buffer fully read; P and O writes visible to the tensor core before it is told
      tc_wait_st();
      tc_fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s_free[st]);
        mbar_arrive(p_full);
      }
    }
    if (ok && mbar_wait(pv_done, (ntiles - 1) & 1, 0x1A00, abort_flag)) {
      tc_fence_after();
      const float inv = 1.f / l_run;
      T* orow = reinterpret_cast<T*>(p.out) + b * p.so_b + h * p.so_h + (int64_t)i * p.so_t;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(lane_addr + Cfg::COL_O + c * 32, v);
        tc_wait_ld();
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          float g[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) g[e] = __uint_as_float(v[v4 * 8 + e]) * inv;
          *reinterpret_cast<uint4*>(orow + c * 32 + v4 * 8) = pack8<T>(g);
        }
      }
      p.lse[(int64_t)bh * p.T + i] = (m_run + log2f(l_run)) * kLn2_;
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
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------- host side

static int encode_qkv(CUtensorMap* m, const void* ptr, const AttnStrides& s, int B, int H, int T, int hd, int dtype) {
  const uint64_t dims[4] = {(uint64_t)hd, (uint64_t)T, (uint64_t)H, (uint64_t)B};
  const uint64_t str[3] = {(uint64_t)s.t * 2, (uint64_t)s.h * 2, (uint64_t)s.b * 2};
  const uint32_t box[4] = {64, 128, 1, 1};
  return encode_tmap_sw128(m, ptr, dtype, 4, dims, str, box);
}

bool attn_tc05_fwd_eligible(const AttnArgs& a, int hd) {
  return (hd == 64 || hd == 128) && a.T % 128 == 0 && a.bias_mode != 3;
}

template <typename T, int HD>
static int fwd_tc05_launch(const AttnArgs& a, int dtype, cudaStream_t st) {
  using Cfg = FaCfg<HD>;
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = encode_qkv(&tq, a.q, a.sq, a.B, a.H, a.T, HD, dtype))) return rc;
  if ((rc = encode_qkv(&tk, a.k, a.sk, a.B, a.H, a.T, HD, dtype))) return rc;
  if ((rc = encode_qkv(&tv, a.v, a.sv, a.B, a.H, a.T, HD, dtype))) return rc;
  FaParams p;
  p.out = a.out; p.lse = a.lse; p.so_b = a.so.b; p.so_h = a.so.h; p.so_t = a.so.t;
  p.H = a.H; p.T = a.T; p.scale = a.scale; p.bias_mode = a.bias_mode; p.slopes = a.slopes;
  auto kern = attn_fwd_tc05_kernel<T, HD>;
  static std::atomic<uint64_t> attr_done{0};
  if ((rc = ensure_dynamic_smem(kern, Cfg::SMEM_BYTES, attr_done, "attention_fwd(tcgen05)"))) return rc;
  dim3 grid(a.T / FA_M, a.B * a.H);
  launch_overlapped(kern, grid, dim3(FA_THREADS), Cfg::SMEM_BYTES, st, tq, tk, tv, p);
  return launched("attention_fwd(tcgen05)");
}

int attn_tc05_fwd(const AttnArgs& a, int hd, int dtype, cudaStream_t st) {
  TFB_DISPATCH_16(dtype, T, {
    if (hd == 64) return fwd_tc05_launch<T, 64>(a, dtype, st);
    return fwd_tc05_launch<T, 128>(a, dtype, st);
  })
}

}  // namespace tfb
