// Library-wide state of the tritonformer_b200 C ABI: version, last error, launch counter,
// test switches, and the GEMM entry point that picks between the two GEMM kernels.
#include "common.cuh"
#include "../../include/tritonformer_b200_debug.h"

namespace tfb {
thread_local char g_err[512] = {0};
std::atomic<int64_t> g_launches{0};
std::atomic<int> g_force_generic_gemm{0};
std::atomic<int> g_force_fallback_attn{0};
std::atomic<int> g_attn_debug{0};
std::atomic<int> g_plain_launch{0};
std::atomic<int> g_gemm_debug{0};
std::atomic<int> g_gemm_free_sms{0};

int gemm_generic(const void* a, const void* b, void* c, const void* bias, const void* addend, int64_t ld_addend,
                 const void* mask, int64_t ld_mask, int64_t M, int64_t N, int64_t K, int64_t a_sm, int64_t a_sk,
                 int64_t b_sk, int64_t b_sn, int64_t ldc, int relu, int dtype, cudaStream_t st);
int gemm_tc05(const void* a, const void* b, void* c, const void* bias, const void* addend, int64_t ld_addend,
              const void* mask, int64_t ld_mask, int64_t M, int64_t N, int64_t K, int64_t a_sm, int64_t a_sk,
              int64_t b_sk, int64_t b_sn, int64_t ldc, int relu, int dtype, void* workspace,
              int64_t workspace_bytes, cudaStream_t st);
bool gemm_tc05_eligible(const void* a, const void* b, const void* c, const void* bias, const void* addend,
                        int64_t ld_addend, const void* mask, int64_t ld_mask, int64_t M, int64_t N, int64_t K,
                        int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn, int64_t ldc);
int64_t gemm_tc05_workspace_bytes();
int read_dev_status(int reset);
int launch_wait_probe(unsigned long long limit_ns, int* waited_ok, cudaStream_t st);
int attn_bwd_tc05_counters(unsigned long long* out);
int gemm_pair_counters(int cta, unsigned long long* out);
int attn_fwd1_tc05_counters(unsigned long long* out);
std::atomic<int> g_counter_select{-1};
}  // namespace tfb

using namespace tfb;

extern "C" int tfb_version(void) { return 1; }
extern "C" const char* tfb_last_error(void) { return g_err; }
extern "C" int64_t tfb_launch_count(void) { return g_launches.load(); }

extern "C" int tfb_device_status(int reset) {
  cudaDeviceSynchronize();
  return read_dev_status(reset);
}

extern "C" int tfb_debug_wait_probe(unsigned long long limit_ns, int* waited_ok, void* stream) {
  TFB_REQUIRE(limit_ns <= 100000000ull, "wait_probe: limit above 100 ms");
  return launch_wait_probe(limit_ns, waited_ok, (cudaStream_t)stream);
}

extern "C" int tfb_debug_counters(unsigned long long* out16) {
  const int sel = g_counter_select.load();
  if (sel == -3) return attn_fwd1_tc05_counters(out16);
  return sel >= 0 ? gemm_pair_counters(sel, out16) : attn_bwd_tc05_counters(out16);
}

extern "C" void tfb_debug_set(int key, int value) {
  if (key == 0) g_force_generic_gemm.store(value);
  if (key == 1) g_force_fallback_attn.store(value);
  if (key == 2) g_attn_debug.store(value);
  if (key == 3) g_plain_launch.store(value);
  if (key == 4) g_gemm_debug.store(value);
  if (key == 6) g_gemm_free_sms.store(value < 0 ? 0 : value);
  if (key == 5) g_counter_select.store(value);
}

extern "C" int64_t tfb_gemm_workspace_bytes(void) { return gemm_tc05_workspace_bytes(); }

extern "C" int tfb_gemm_fused(const void* a, const void* b, void* c, const void* bias, const void* addend,
                              int64_t ld_addend, const void* mask, int64_t ld_mask, int64_t M, int64_t N, int64_t K,
                              int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn, int64_t ldc, int relu,
                              int dtype, void* workspace, int64_t workspace_bytes, void* stream, int* path) {
  TFB_REQUIRE(M >= 0 && N >= 0 && K >= 0, "gemm: negative dimension");
  TFB_REQUIRE(M < (1LL << 31) && N < (1LL << 31) && K < (1LL << 31), "gemm: dimension exceeds 2^31");
  TFB_REQUIRE(a_sm == 1 || a_sk == 1, "gemm: A needs a unit stride (a_sm=%lld a_sk=%lld)", (long long)a_sm,
              (long long)a_sk);
  TFB_REQUIRE(b_sk == 1 || b_sn == 1, "gemm: B needs a unit stride (b_sk=%lld b_sn=%lld)", (long long)b_sk,
              (long long)b_sn);
  TFB_REQUIRE(ldc >= N, "gemm: ldc=%lld smaller than N=%lld", (long long)ldc, (long long)N);
  TFB_REQUIRE(!addend || ld_addend >= N, "gemm: addend leading dimension smaller than N");
  TFB_REQUIRE(!mask || ld_mask >= N, "gemm: mask leading dimension smaller than N");
  TFB_REQUIRE(dtype == TFB_F16 || dtype == TFB_BF16, "gemm: dtype %d: expected fp16 or bf16", dtype);
  if (M == 0 || N == 0) return TFB_OK;
  TFB_REQUIRE(K > 0, "gemm: empty contraction");
  cudaStream_t st = (cudaStream_t)stream;
  const bool fast = !g_force_generic_gemm.load() &&
                    gemm_tc05_eligible(a, b, c, bias, addend, ld_addend, mask, ld_mask, M, N, K, a_sm, a_sk, b_sk,
                                       b_sn, ldc);
  if (path) *path = fast ? 1 : 0;
  if (fast)
    return gemm_tc05(a, b, c, bias, addend, ld_addend, mask, ld_mask, M, N, K, a_sm, a_sk, b_sk, b_sn, ldc, relu,
                     dtype, workspace, workspace_bytes, st);
  return gemm_generic(a, b, c, bias, addend, ld_addend, mask, ld_mask, M, N, K, a_sm, a_sk, b_sk, b_sn, ldc, relu,
                      dtype, st);
}

extern "C" int tfb_gemm(const void* a, const void* b, void* c, const void* bias, int64_t M, int64_t N,
                        int64_t K, int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn, int64_t ldc,
                        int relu, int accumulate, int dtype, void* stream, int* path) {
  return tfb_gemm_fused(a, b, c, bias, accumulate ? c : nullptr, ldc, nullptr, 0, M, N, K, a_sm, a_sk, b_sk, b_sn,
                        ldc, relu, dtype, nullptr, 0, stream, path);
}
