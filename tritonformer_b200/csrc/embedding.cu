// Token (+ learned position) embedding lookup and its gradient for sm_100a.  Row gathers and
// scatters with 128-bit accesses; every sum is taken in fp32 and rounded once.
//
// Gradient of the token table without a sort: a first kernel records, per vocabulary row, the
// smallest position that holds it and how many positions hold it.  Rows held once (nearly all of
// them) are added to the table gradient directly; rows held several times are summed with fp32
// vector atomics into the scratch row of their first position, and a last kernel folds those
// scratch rows into the table gradient.
#include "common.cuh"

namespace tfb {

extern __device__ int g_dev_status;  // the library's status word (status.cu)
constexpr int kBadToken = 0x7100;       // a token id outside [0, vocab)
constexpr int kTableFill = 0x7f7f7f7f;  // what a byte fill of 0x7f leaves in every int32
constexpr int kTestLanes = 32;          // threads per row in the kernels that mostly test and skip rows

// How many positions hold token `id` (the count half of the table starts at kTableFill).
__device__ __forceinline__ unsigned held(const int* table, int64_t vocab, int64_t id) {
  return (unsigned)table[vocab + id] - (unsigned)kTableFill;
}

template <typename T, int W>
__device__ __forceinline__ void load_w(const T* p, float (&f)[W]) {
  if constexpr (W == 8) unpack8<T>(*reinterpret_cast<const uint4*>(p), f);
  else f[0] = Num<T>::to_f(*p);
}
template <typename T, int W>
__device__ __forceinline__ void store_w(T* p, const float (&f)[W]) {
  if constexpr (W == 8) *reinterpret_cast<uint4*>(p) = pack8<T>(f);
  else *p = Num<T>::from_f(f[0]);
}

// 256 threads = (256 / lanes) rows x lanes column chunks of W elements; lanes is a power of two.
template <typename T, int W>
__global__ void __launch_bounds__(256) embed_fwd_kernel(const int64_t* __restrict__ ids, const T* __restrict__ tok,
                                                        const T* __restrict__ pos, T* __restrict__ out,
                                                        int64_t n, int64_t seq, int d, int64_t vocab, int lanes) {
  grid_dependency_wait();
  allow_dependents();
  const int sub = threadIdx.x / lanes, l = threadIdx.x % lanes, per = 256 / lanes;
  const int chunks = d / W;
  for (int64_t row = (int64_t)blockIdx.x * per + sub; row < n; row += (int64_t)gridDim.x * per) {
    const int64_t id = ids[row];
    const bool ok = id >= 0 && id < vocab;
    if (!ok && l == 0) atomicCAS(&g_dev_status, 0, kBadToken);
    const T* prow = pos ? pos + (row % seq) * d : nullptr;
    for (int c = l; c < chunks; c += lanes) {
      float a[W];
#pragma unroll
      for (int j = 0; j < W; ++j) a[j] = 0.f;
      if (ok) {
        load_w<T, W>(tok + id * d + c * W, a);
        if (prow) {
          float b[W];
          load_w<T, W>(prow + c * W, b);
#pragma unroll
          for (int j = 0; j < W; ++j) a[j] += b[j];
        }
      }
      store_w<T, W>(out + row * d + c * W, a);
    }
  }
}

// table[v] = smallest position holding token v, table[vocab + v] = kTableFill + how many hold it
// (both start as kTableFill).
__global__ void __launch_bounds__(256) embed_index_kernel(const int64_t* __restrict__ ids, int* __restrict__ table,
                                                          int64_t n, int64_t vocab) {
  const int64_t stride = (int64_t)gridDim.x * 256;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) {
    const int64_t id = ids[i];
    if (id >= 0 && id < vocab) {
      atomicMin(table + id, (int)i);
      atomicAdd(table + vocab + id, 1);
    } else {
      atomicCAS(&g_dev_status, 0, kBadToken);
    }
  }
}

// Clears the fp32 scratch row of every position that is the first holder of a token held several
// times: the only rows the scatter kernel adds into.
__global__ void __launch_bounds__(256) embed_clear_kernel(const int64_t* __restrict__ ids,
                                                          const int* __restrict__ table, float* __restrict__ scratch,
                                                          int64_t n, int d, int64_t vocab, int lanes) {
  grid_dependency_wait();
  allow_dependents();
  const int sub = threadIdx.x / lanes, l = threadIdx.x % lanes, per = 256 / lanes;
  for (int64_t row = (int64_t)blockIdx.x * per + sub; row < n; row += (int64_t)gridDim.x * per) {
    const int64_t id = ids[row];
    if (id < 0 || id >= vocab) continue;
    if (held(table, vocab, id) < 2u || table[id] != (int)row) continue;
    for (int c = l; c < d; c += lanes) scratch[row * d + c] = 0.f;
  }
}

// One sub-group of `lanes` threads per time step t: reads the gradient rows of every sequence at
// t, adds their sum to the position-table gradient and routes each row to the token-table
// gradient (directly when its token occurs once, through the fp32 scratch otherwise).
template <typename T, int W>
__global__ void __launch_bounds__(256) embed_bwd_scatter_kernel(const int64_t* __restrict__ ids,
                                                                const T* __restrict__ dout, T* __restrict__ dtok,
                                                                T* __restrict__ dpos, const int* __restrict__ table,
                                                                float* __restrict__ scratch, int64_t batch,
                                                                int64_t seq, int d, int64_t vocab, int lanes) {
  grid_dependency_wait();
  allow_dependents();
  const int sub = threadIdx.x / lanes, l = threadIdx.x % lanes, per = 256 / lanes;
  const int chunks = d / W;
  for (int64_t t = (int64_t)blockIdx.x * per + sub; t < seq; t += (int64_t)gridDim.x * per) {
    for (int c = l; c < chunks; c += lanes) {
      float psum[W];
#pragma unroll
      for (int j = 0; j < W; ++j) psum[j] = 0.f;
      // four sequences at a time, so that their loads are in flight together; rows that take the
      // direct path within one group belong to different tokens (a token held twice goes through
      // the scratch), so their read-modify-writes do not overlap
      for (int64_t b0 = 0; b0 < batch; b0 += 4) {
        float g[4][W], w[4][W];
        int64_t id[4];
        bool direct[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          id[u] = -1;
          direct[u] = false;
          if (b0 + u < batch) {
            const int64_t row = (b0 + u) * seq + t;
            load_w<T, W>(dout + row * d + c * W, g[u]);
            const int64_t v = dtok ? ids[row] : -1;  // no token-table gradient wanted: position sums only
            if (v >= 0 && v < vocab) {
              id[u] = v;
              direct[u] = held(table, vocab, v) == 1u;
            }
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (direct[u]) load_w<T, W>(dtok + id[u] * d + c * W, w[u]);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (b0 + u < batch) {
#pragma unroll
            for (int j = 0; j < W; ++j) psum[j] += g[u][j];
          }
          if (direct[u]) {
#pragma unroll
            for (int j = 0; j < W; ++j) w[u][j] += g[u][j];
            store_w<T, W>(dtok + id[u] * d + c * W, w[u]);
          } else if (id[u] >= 0) {
            float* dst = scratch + (int64_t)table[id[u]] * d + c * W;
            if constexpr (W == 8) {
              atomicAdd(reinterpret_cast<float4*>(dst), make_float4(g[u][0], g[u][1], g[u][2], g[u][3]));
              atomicAdd(reinterpret_cast<float4*>(dst) + 1, make_float4(g[u][4], g[u][5], g[u][6], g[u][7]));
            } else {
              atomicAdd(dst, g[u][0]);
            }
          }
        }
      }
      if (dpos) {
        float w[W];
        load_w<T, W>(dpos + t * d + c * W, w);
#pragma unroll
        for (int j = 0; j < W; ++j) w[j] += psum[j];
        store_w<T, W>(dpos + t * d + c * W, w);
      }
    }
  }
}

// Rows that are the first position of a token held several times carry that token's fp32 sum.
template <typename T, int W>
__global__ void __launch_bounds__(256) embed_bwd_fold_kernel(const int64_t* __restrict__ ids, T* __restrict__ dtok,
                                                             const int* __restrict__ table,
                                                             const float* __restrict__ scratch, int64_t n, int d,
                                                             int64_t vocab, int lanes) {
  grid_dependency_wait();
  allow_dependents();
  const int sub = threadIdx.x / lanes, l = threadIdx.x % lanes, per = 256 / lanes;
  const int chunks = d / W;
  for (int64_t row = (int64_t)blockIdx.x * per + sub; row < n; row += (int64_t)gridDim.x * per) {
    const int64_t id = ids[row];
    if (id < 0 || id >= vocab) continue;
    if (held(table, vocab, id) < 2u || table[id] != (int)row) continue;
    for (int c = l; c < chunks; c += lanes) {
      float w[W];
      load_w<T, W>(dtok + id * d + c * W, w);
      const float* src = scratch + row * d + c * W;
#pragma unroll
      for (int j = 0; j < W; ++j) w[j] += src[j];
      store_w<T, W>(dtok + id * d + c * W, w);
    }
  }
}

// Threads per row: the smallest power of two that covers the row's chunks, at most 256.
static int lanes_for(int64_t chunks) {
  int lanes = 1;
  while (lanes < chunks && lanes < 256) lanes *= 2;
  return lanes;
}

static unsigned grid_for(int64_t units, int per) {
  const int64_t want = ceil_div(units, per);
  return (unsigned)(want < 148 * 8 ? (want < 1 ? 1 : want) : 148 * 8);
}

}  // namespace tfb

using namespace tfb;

extern "C" int tfb_embedding_fwd(const int64_t* ids, const void* tok, const void* pos, void* out, int64_t batch,
                                 int64_t seq, int64_t d, int64_t vocab, int64_t pos_rows, int dtype, void* stream) {
  TFB_REQUIRE(batch >= 0 && seq >= 0 && d > 0 && d < (1 << 30) && vocab > 0, "embedding_fwd: bad shape");
  TFB_REQUIRE(pos == nullptr || seq <= pos_rows, "embedding_fwd: sequence of %lld longer than the position table (%lld rows)",
              (long long)seq, (long long)pos_rows);
  const int64_t n = batch * seq;
  if (n == 0) return TFB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = d % 8 == 0 && aligned16(tok) && aligned16(out) && (pos == nullptr || aligned16(pos));
  TFB_DISPATCH_16(dtype, T, {
    if (vec) {
      const int lanes = lanes_for(d / 8);
      launch_overlapped(embed_fwd_kernel<T, 8>, dim3(grid_for(n, 256 / lanes)), dim3(256), 0, st, ids, (const T*)tok,
                        (const T*)pos, (T*)out, n, seq, (int)d, vocab, lanes);
    } else {
      const int lanes = lanes_for(d);
      launch_overlapped(embed_fwd_kernel<T, 1>, dim3(grid_for(n, 256 / lanes)), dim3(256), 0, st, ids, (const T*)tok,
                        (const T*)pos, (T*)out, n, seq, (int)d, vocab, lanes);
    }
  })
  return launched("embedding_fwd");
}

extern "C" int64_t tfb_embedding_bwd_scratch_bytes(int64_t batch, int64_t seq, int64_t d, int64_t vocab) {
  if (batch < 0 || seq < 0 || d <= 0 || vocab <= 0) return 0;
  const int64_t table = ceil_div(2 * vocab * (int64_t)sizeof(int), 16) * 16;
  return table + batch * seq * d * (int64_t)sizeof(float);
}

extern "C" int tfb_embedding_bwd(const int64_t* ids, const void* dout, void* dtok, void* dpos, void* scratch,
                                 int64_t scratch_bytes, int64_t batch, int64_t seq, int64_t d, int64_t vocab,
                                 int64_t pos_rows, int dtype, void* stream) {
  TFB_REQUIRE(batch >= 0 && seq >= 0 && d > 0 && d < (1 << 30) && vocab > 0, "embedding_bwd: bad shape");
  TFB_REQUIRE(dpos == nullptr || seq <= pos_rows, "embedding_bwd: sequence of %lld longer than the position table (%lld rows)",
              (long long)seq, (long long)pos_rows);
  const int64_t n = batch * seq;
  TFB_REQUIRE(n < (1 << 30), "embedding_bwd: more than 2^30 positions");
  if (n == 0 || (dtok == nullptr && dpos == nullptr)) return TFB_OK;
  TFB_REQUIRE(scratch != nullptr && aligned16(scratch) &&
                  scratch_bytes >= tfb_embedding_bwd_scratch_bytes(batch, seq, d, vocab),
              "embedding_bwd: scratch must hold tfb_embedding_bwd_scratch_bytes() bytes, 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  int* table = (int*)scratch;
  const int64_t table_bytes = ceil_div(2 * vocab * (int64_t)sizeof(int), 16) * 16;
  float* sums = (float*)((char*)scratch + table_bytes);
  int rc = TFB_OK;
  if (dtok) {  // a frozen token table (dtok == NULL) needs neither the index nor the fp32 scratch rows
    TFB_REQUIRE(cudaMemsetAsync(table, 0x7f, (size_t)table_bytes, st) == cudaSuccess, "embedding_bwd: table fill failed");
    embed_index_kernel<<<grid_for(n, 256), 256, 0, st>>>(ids, table, n, vocab);
    rc = launched("embedding_bwd index");
    if (rc) return rc;
  }
  if (dtok) {
    // most rows are only tested (few tokens are held twice): a warp per row keeps eight tests in flight per CTA
    const int lanes = kTestLanes;
    launch_overlapped(embed_clear_kernel, dim3(grid_for(n, 256 / lanes)), dim3(256), 0, st, ids, (const int*)table, sums,
                      n, (int)d, vocab, lanes);
    rc = launched("embedding_bwd clear");
    if (rc) return rc;
  }
  const bool vec = d % 8 == 0 && aligned16(dout) && aligned16(dtok) && (dpos == nullptr || aligned16(dpos));
  TFB_DISPATCH_16(dtype, T, {
    if (vec) {
      const int lanes = lanes_for(d / 8);
      launch_overlapped(embed_bwd_scatter_kernel<T, 8>, dim3(grid_for(seq, 256 / lanes)), dim3(256), 0, st, ids,
                        (const T*)dout, (T*)dtok, (T*)dpos, (const int*)table, sums, batch, seq, (int)d, vocab, lanes);
      rc = launched("embedding_bwd scatter");
      if (rc || !dtok) return rc;
      launch_overlapped(embed_bwd_fold_kernel<T, 8>, dim3(grid_for(n, 256 / kTestLanes)), dim3(256), 0, st, ids,
                        (T*)dtok, (const int*)table, (const float*)sums, n, (int)d, vocab, kTestLanes);
    } else {
      const int lanes = lanes_for(d);
      launch_overlapped(embed_bwd_scatter_kernel<T, 1>, dim3(grid_for(seq, 256 / lanes)), dim3(256), 0, st, ids,
                        (const T*)dout, (T*)dtok, (T*)dpos, (const int*)table, sums, batch, seq, (int)d, vocab, lanes);
      rc = launched("embedding_bwd scatter");
      if (rc || !dtok) return rc;
      launch_overlapped(embed_bwd_fold_kernel<T, 1>, dim3(grid_for(n, 256 / kTestLanes)), dim3(256), 0, st, ids,
                        (T*)dtok, (const int*)table, (const float*)sums, n, (int)d, vocab, kTestLanes);
    }
  })
  return launched("embedding_bwd fold");
}
