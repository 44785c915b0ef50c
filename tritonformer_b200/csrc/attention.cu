// Entry points of the attention family: argument checks, scratch layout, kernel choice.
#include "attn.cuh"

namespace tfb {
extern std::atomic<int> g_force_fallback_attn;
extern std::atomic<int> g_attn_debug;
bool attn_tc05_fwd_eligible(const AttnArgs& a, int hd);
int attn_fwd1_tc05(const AttnArgs& a, int hd, int dtype, cudaStream_t st);
bool attn_tc05_bwd_eligible(const AttnArgs& a, int hd);
int attn_tc05_bwd(const AttnArgs& a, int hd, int dtype, cudaStream_t st);
}  // namespace tfb

using namespace tfb;

static AttnStrides mk(const int64_t* s) { return AttnStrides{s[0], s[1], s[2]}; }

static int check_tensor(const char* name, const void* p, const int64_t* s) {
  TFB_REQUIRE(p != nullptr, "attention: %s is null", name);
  TFB_REQUIRE(aligned16(p) && s[0] % 8 == 0 && s[1] % 8 == 0 && s[2] % 8 == 0,
              "attention: %s needs a 16-byte aligned base and strides that are multiples of 8 elements", name);
  return TFB_OK;
}

static int check_common(int64_t B, int64_t H, int64_t T, int64_t hd, const float* slopes, const void* bias) {
  TFB_REQUIRE(B > 0 && H > 0 && T > 0 && B * H < 65536, "attention: bad shape B=%lld H=%lld T=%lld", (long long)B,
              (long long)H, (long long)T);
  if (hd != 32 && hd != 64 && hd != 128)
    return fail(TFB_ERR_UNSUPPORTED, "Only head_dims of [32,64,128] are supported.");
  TFB_REQUIRE(T % 64 == 0, "Number of elements in sequence must be a multiple of 64");
  TFB_REQUIRE(!(slopes && bias), "attention: pass ALiBi slopes or a dense bias, not both");
  return TFB_OK;
}

extern "C" int tfb_attention_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int64_t B,
                                 int64_t H, int64_t T, int64_t hd, const int64_t* q_strides,
                                 const int64_t* k_strides, const int64_t* v_strides, const int64_t* o_strides,
                                 const float* slopes, int alibi_round, const void* bias, int64_t bias_sh,
                                 int64_t bias_si, int dtype, void* stream, int* path) {
  int rc;
  if ((rc = check_common(B, H, T, hd, slopes, bias))) return rc;
  if ((rc = check_tensor("q", q, q_strides)) || (rc = check_tensor("k", k, k_strides)) ||
      (rc = check_tensor("v", v, v_strides)) || (rc = check_tensor("out", o, o_strides)))
    return rc;
  TFB_REQUIRE(lse != nullptr, "attention: lse is null");
  AttnArgs a{};
  a.q = q; a.k = k; a.v = v; a.out = o; a.lse = lse;
  a.sq = mk(q_strides); a.sk = mk(k_strides); a.sv = mk(v_strides); a.so = mk(o_strides);
  a.B = (int)B; a.H = (int)H; a.T = (int)T;
  a.scale = 1.0f / sqrtf((float)hd);
  a.bias_mode = slopes ? (alibi_round == 1 ? 2 : alibi_round == 2 ? 4 : 1) : (bias ? 3 : 0);
  a.slopes = slopes; a.bias = bias; a.bias_sh = bias_sh; a.bias_si = bias_si;
  const bool fast = !g_force_fallback_attn.load() && attn_tc05_fwd_eligible(a, (int)hd);
  if (path) *path = fast ? 1 : 0;
  if (fast) return attn_fwd1_tc05(a, (int)hd, dtype, (cudaStream_t)stream);
  return attn_generic_fwd(a, (int)hd, dtype, (cudaStream_t)stream);
}

extern "C" int64_t tfb_attention_bwd_scratch_bytes(int64_t B, int64_t H, int64_t T, int64_t hd) {
  // delta (B,H,T) fp32, then the fp32 dQ accumulator (B,H,T,hd) of the tcgen05 path
  return ((B * H * T * 4 + 255) / 256) * 256 + B * H * T * hd * 4;
}

extern "C" int tfb_attention_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                 const float* lse, void* dq, void* dk, void* dv, int64_t B, int64_t H, int64_t T,
                                 int64_t hd, const int64_t* q_strides, const int64_t* k_strides,
                                 const int64_t* v_strides, const int64_t* o_strides, const int64_t* do_strides,
                                 const int64_t* dq_strides, const int64_t* dk_strides, const int64_t* dv_strides,
                                 const float* slopes, int alibi_round, const void* bias, int64_t bias_sh,
                                 int64_t bias_si, void* scratch, int64_t scratch_bytes, int dtype, void* stream,
                                 int* path) {
  int rc;
  if ((rc = check_common(B, H, T, hd, slopes, bias))) return rc;
  if ((rc = check_tensor("q", q, q_strides)) || (rc = check_tensor("k", k, k_strides)) ||
      (rc = check_tensor("v", v, v_strides)) || (rc = check_tensor("out", o, o_strides)) ||
      (rc = check_tensor("grad_out", d_o, do_strides)) || (rc = check_tensor("grad_q", dq, dq_strides)) ||
      (rc = check_tensor("grad_k", dk, dk_strides)) || (rc = check_tensor("grad_v", dv, dv_strides)))
    return rc;
  TFB_REQUIRE(lse != nullptr && scratch != nullptr && aligned16(scratch), "attention_bwd: lse/scratch missing");
  TFB_REQUIRE(scratch_bytes >= tfb_attention_bwd_scratch_bytes(B, H, T, hd),
              "attention_bwd: scratch smaller than tfb_attention_bwd_scratch_bytes()");
  AttnArgs a{};
  a.q = q; a.k = k; a.v = v; a.o = o; a.d_o = d_o; a.lse = const_cast<float*>(lse);
  a.dq = dq; a.dk = dk; a.dv = dv;
  a.delta = reinterpret_cast<float*>(scratch);
  a.sq = mk(q_strides); a.sk = mk(k_strides); a.sv = mk(v_strides); a.so = mk(o_strides);
  a.sdo = mk(do_strides); a.sdq = mk(dq_strides); a.sdk = mk(dk_strides); a.sdv = mk(dv_strides);
  a.B = (int)B; a.H = (int)H; a.T = (int)T;
  a.scale = 1.0f / sqrtf((float)hd);
  a.bias_mode = slopes ? (alibi_round == 1 ? 2 : alibi_round == 2 ? 4 : 1) : (bias ? 3 : 0);
  a.slopes = slopes; a.bias = bias; a.bias_sh = bias_sh; a.bias_si = bias_si;
  a.dq_acc = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(scratch) + ((B * H * T * 4 + 255) / 256) * 256);
  const bool fast = !g_force_fallback_attn.load() && attn_tc05_bwd_eligible(a, (int)hd);
  if (path) *path = fast ? 1 : 0;
  if (fast) return attn_tc05_bwd(a, (int)hd, dtype, (cudaStream_t)stream);
  return attn_generic_bwd(a, (int)hd, dtype, (cudaStream_t)stream);
}
