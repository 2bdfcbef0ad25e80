// Attention entry points: argument checks and routing between the tcgen05
// kernels (bf16 / fp16, D = 64 / 128, with or without an additive mask) and the CUDA-core kernels (the rest).
#include "attn.cuh"
#include "common.cuh"

using namespace mgb;

namespace {

int check_attn(const char* who, int64_t B, int64_t S, int64_t H, int64_t D, int causal, int has_bias, int dtype) {
  MGB_REQUIRE(B > 0 && S > 0 && H > 0, MGB_EINVAL, "%s: B=%lld S=%lld H=%lld must be positive", who, (long long)B,
              (long long)S, (long long)H);
  MGB_REQUIRE(D >= 1 && D <= 512, MGB_EUNSUPPORTED, "%s: head dim %lld outside [1, 512]", who, (long long)D);
  MGB_REQUIRE(!(causal && has_bias), MGB_EINVAL, "%s: causal and has_bias cannot both be set", who);
  MGB_REQUIRE(dtype == MGB_BF16 || dtype == MGB_F32 || dtype == MGB_F16, MGB_EDTYPE, "%s: unsupported dtype code %d",
              who, dtype);
  MGB_REQUIRE(B * H * S < (1LL << 31) && S < (1 << 30), MGB_EUNSUPPORTED, "%s: B*H*S exceeds 2^31", who);
  return MGB_OK;
}

size_t delta_bytes(int64_t B, int64_t S, int64_t H) { return round_up(static_cast<size_t>(B * H * S) * sizeof(float), 256); }
size_t dq_acc_bytes(int64_t B, int64_t S, int64_t H, int64_t D) {
  return round_up(static_cast<size_t>(B * S * H * D) * sizeof(float), 256);
}

}  // namespace

int check_layouts(const char* who, int64_t H, int64_t D, int64_t ld_qkv, int64_t ld_dqkv, int o_layout) {
  MGB_REQUIRE(ld_qkv >= H * D && ld_dqkv >= H * D, MGB_EINVAL, "%s: token stride smaller than H*D", who);
  MGB_REQUIRE(o_layout == 0 || o_layout == 1, MGB_EINVAL, "%s: o_layout=%d (0 = BHSD, 1 = BSHD)", who, o_layout);
  return MGB_OK;
}

MGB_EXPORT int mograd_b200_flash_attn_fwd_ex(const void* q, const void* k, const void* v, const void* mask, void* dst,
                                             float* lse, int64_t B, int64_t S, int64_t H, int64_t D, float scale,
                                             int causal, int has_bias, int64_t ld_qkv, int o_layout, int dtype,
                                             void* stream) {
  MGB_REQUIRE(q && k && v && dst && lse, MGB_EINVAL, "flash_attn_fwd: NULL argument");
  MGB_REQUIRE(!has_bias || mask, MGB_EINVAL, "flash_attn_fwd: has_bias set but mask is NULL");
  int rc = check_attn("flash_attn_fwd", B, S, H, D, causal, has_bias, dtype);
  if (rc != MGB_OK) return rc;
  rc = check_layouts("flash_attn_fwd", H, D, ld_qkv, ld_qkv, o_layout);
  if (rc != MGB_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int b = static_cast<int>(B), s = static_cast<int>(S), h = static_cast<int>(H), d = static_cast<int>(D);
  const attn::Layouts lay{ld_qkv, ld_qkv, o_layout};
  if (dtype == MGB_F32)
    return attn::generic_fwd<float>(q, k, v, mask, dst, lse, b, s, h, d, scale, causal, has_bias, lay, st);
  const void* ptrs[] = {q, k, v, dst};
  if (attn::tc_supported(d, lay, ptrs, 4))
    return attn::tc_fwd(q, k, v, dst, lse, b, s, h, d, scale, causal, dtype == MGB_F16, has_bias ? mask : nullptr, lay, st);
  if (dtype == MGB_F16)
    return attn::generic_fwd<__half>(q, k, v, mask, dst, lse, b, s, h, d, scale, causal, has_bias, lay, st);
  return attn::generic_fwd<__nv_bfloat16>(q, k, v, mask, dst, lse, b, s, h, d, scale, causal, has_bias, lay, st);
}

MGB_EXPORT int mograd_b200_flash_attn_fwd(const void* q, const void* k, const void* v, const void* mask, void* dst,
                                          float* lse, int64_t B, int64_t S, int64_t H, int64_t D, float scale,
                                          int causal, int has_bias, int dtype, void* stream) {
  return mograd_b200_flash_attn_fwd_ex(q, k, v, mask, dst, lse, B, S, H, D, scale, causal, has_bias, H * D, 0, dtype,
                                       stream);
}

MGB_EXPORT size_t mograd_b200_flash_attn_bwd_workspace_bytes(int64_t B, int64_t S, int64_t H, int64_t D, int dtype) {
  if (B <= 0 || S <= 0 || H <= 0 || D <= 0) return 0;
  size_t n = delta_bytes(B, S, H);
  if (dtype != MGB_F32 && (D == 64 || D == 128)) n += dq_acc_bytes(B, S, H, D);
  return n;
}

MGB_EXPORT int mograd_b200_flash_attn_bwd_ex(const void* dy, const void* o, const void* q, const void* k,
                                             const void* v, const void* mask, const float* lse, void* dq, void* dk,
                                             void* dv, int64_t B, int64_t S, int64_t H, int64_t D, float scale,
                                             int causal, int has_bias, int64_t ld_qkv, int64_t ld_dqkv, int o_layout,
                                             int dtype, void* workspace, size_t workspace_bytes, void* stream) {
  MGB_REQUIRE(dy && o && q && k && v && lse && dq && dk && dv, MGB_EINVAL, "flash_attn_bwd: NULL argument");
  MGB_REQUIRE(!has_bias || mask, MGB_EINVAL, "flash_attn_bwd: has_bias set but mask is NULL");
  int rc = check_attn("flash_attn_bwd", B, S, H, D, causal, has_bias, dtype);
  if (rc != MGB_OK) return rc;
  rc = check_layouts("flash_attn_bwd", H, D, ld_qkv, ld_dqkv, o_layout);
  if (rc != MGB_OK) return rc;
  const size_t need = mograd_b200_flash_attn_bwd_workspace_bytes(B, S, H, D, dtype);
  MGB_REQUIRE(workspace && workspace_bytes >= need, MGB_EWORKSPACE,
              "flash_attn_bwd: workspace of %zu bytes needed, %zu given", need, workspace ? workspace_bytes : (size_t)0);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int b = static_cast<int>(B), s = static_cast<int>(S), h = static_cast<int>(H), d = static_cast<int>(D);
  const attn::Layouts lay{ld_qkv, ld_dqkv, o_layout};
  float* delta = static_cast<float*>(workspace);
  if (dtype == MGB_F32) {
    rc = attn::launch_delta<float>(o, dy, delta, b, s, h, d, o_layout, nullptr, nullptr, st);
    if (rc != MGB_OK) return rc;
    return attn::generic_bwd<float>(dy, q, k, v, mask, lse, delta, dq, dk, dv, b, s, h, d, scale, causal, has_bias, lay,
                                    st);
  }
  const void* ptrs[] = {dy, q, k, v, dq, dk, dv};
  const bool tc = attn::tc_supported(d, lay, ptrs, 7);
  float* dq_acc = reinterpret_cast<float*>(static_cast<char*>(workspace) + delta_bytes(B, S, H));
  bool acc_zeroed = false;
  const bool f16 = dtype == MGB_F16;
  rc = f16 ? attn::launch_delta<__half>(o, dy, delta, b, s, h, d, o_layout, tc ? dq_acc : nullptr, &acc_zeroed, st)
           : attn::launch_delta<__nv_bfloat16>(o, dy, delta, b, s, h, d, o_layout, tc ? dq_acc : nullptr, &acc_zeroed, st);
  if (rc != MGB_OK) return rc;
  if (tc)
    return attn::tc_bwd(dy, q, k, v, lse, delta, dq_acc, acc_zeroed, dq, dk, dv, b, s, h, d, scale, causal, f16,
                        has_bias ? mask : nullptr, lay, st);
  if (f16)
    return attn::generic_bwd<__half>(dy, q, k, v, mask, lse, delta, dq, dk, dv, b, s, h, d, scale, causal, has_bias, lay,
                                     st);
  return attn::generic_bwd<__nv_bfloat16>(dy, q, k, v, mask, lse, delta, dq, dk, dv, b, s, h, d, scale, causal,
                                          has_bias, lay, st);
}

MGB_EXPORT int mograd_b200_flash_attn_bwd(const void* dy, const void* o, const void* q, const void* k, const void* v,
                                          const void* mask, const float* lse, void* dq, void* dk, void* dv, int64_t B,
                                          int64_t S, int64_t H, int64_t D, float scale, int causal, int has_bias,
                                          int dtype, void* workspace, size_t workspace_bytes, void* stream) {
  return mograd_b200_flash_attn_bwd_ex(dy, o, q, k, v, mask, lse, dq, dk, dv, B, S, H, D, scale, causal, has_bias,
                                       H * D, H * D, 0, dtype, workspace, workspace_bytes, stream);
}
