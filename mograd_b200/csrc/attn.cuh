// Internal interface between the attention entry points and their kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace mgb {
namespace attn {

// delta[row] = sum_d O[row,d] * dO[row,d] over BHSD rows.
template <typename T>
int launch_delta(const void* o, const void* dy, float* delta, int64_t rows, int D, cudaStream_t st);

// CUDA-core kernels (any D <= 512, optional additive bias).
template <typename T>
int generic_fwd(const void* q, const void* k, const void* v, const void* mask, void* dst, float* lse, int B, int S,
                int H, int D, float scale, int causal, int has_bias, cudaStream_t st);
template <typename T>
int generic_bwd(const void* dy, const void* q, const void* k, const void* v, const void* mask, const float* lse,
                const float* delta, void* dq, void* dk, void* dv, int B, int S, int H, int D, float scale, int causal,
                int has_bias, cudaStream_t st);

// tcgen05 kernels: bf16, D in {64, 128}, no bias, 16-byte aligned tensors.
bool tc_supported(int D, int has_bias, const void* const* ptrs, int nptrs);
int tc_fwd(const void* q, const void* k, const void* v, void* dst, float* lse, int B, int S, int H, int D, float scale,
           int causal, cudaStream_t st);
// dq_acc: fp32 (B,S,H,D) accumulator, zero-filled by the callee.
int tc_bwd(const void* dy, const void* q, const void* k, const void* v, const float* lse, const float* delta,
           float* dq_acc, void* dq, void* dk, void* dv, int B, int S, int H, int D, float scale, int causal,
           cudaStream_t st);

}  // namespace attn
}  // namespace mgb
