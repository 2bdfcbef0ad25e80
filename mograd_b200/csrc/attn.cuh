// Internal interface between the attention entry points and their kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace mgb {
namespace attn {

// How the tensors lie in memory beyond the reference's packed defaults.
struct Layouts {
  int64_t ld_qkv;   // elements between consecutive tokens of Q / K / V (H*D when each is packed BSHD)
  int64_t ld_dqkv;  // same for dQ / dK / dV
  int o_bshd;       // 0: O and dO are (B,H,S,D) as in the reference; 1: (B,S,H,D)
};

// delta[(b,h,s)] = sum_d O[.,d] * dO[.,d].
template <typename T>
// zero (optional): fp32 array of B*S*H*D elements cleared by the same kernel when it can; *zeroed says whether it was
int launch_delta(const void* o, const void* dy, float* delta, int B, int S, int H, int D, int o_bshd, float* zero,
                 bool* zeroed, cudaStream_t st);

// CUDA-core kernels (any D <= 512, optional additive bias).
template <typename T>
int generic_fwd(const void* q, const void* k, const void* v, const void* mask, void* dst, float* lse, int B, int S,
                int H, int D, float scale, int causal, int has_bias, const Layouts& lay, cudaStream_t st);
template <typename T>
int generic_bwd(const void* dy, const void* q, const void* k, const void* v, const void* mask, const float* lse,
                const float* delta, void* dq, void* dk, void* dv, int B, int S, int H, int D, float scale, int causal,
                int has_bias, const Layouts& lay, cudaStream_t st);

// tcgen05 kernels: bf16 or fp16 storage (f16 != 0), D in {64, 128}, 16-byte aligned tensors; bias: the additive
// (B, H, S, S) mask in the storage type, or nullptr.
bool tc_supported(int D, const Layouts& lay, const void* const* ptrs, int nptrs);
int tc_fwd(const void* q, const void* k, const void* v, void* dst, float* lse, int B, int S, int H, int D, float scale,
           int causal, int f16, const void* bias, const Layouts& lay, cudaStream_t st);
// dq_acc: fp32 (B,S,H,D) accumulator; zero-filled by the callee unless acc_zeroed says an earlier kernel on the
// stream has done it.
int tc_bwd(const void* dy, const void* q, const void* k, const void* v, const float* lse, const float* delta,
           float* dq_acc, bool acc_zeroed, void* dq, void* dk, void* dv, int B, int S, int H, int D, float scale,
           int causal, int f16, const void* bias, const Layouts& lay, cudaStream_t st);

}  // namespace attn
}  // namespace mgb
