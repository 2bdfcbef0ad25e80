// CUDA-core attention kernels: any head dim 1..512, float32 or bf16 storage,
// causal or additive-bias masking.  They serve every request the tensor-core
// kernels do not take (fp32, D not in {64,128}, bias).  All arithmetic is
// fp32.  Structure: one warp owns one query row (forward, dQ) or one key row
// (dK/dV) and walks the other sequence in chunks of 32, one lane per
// counterpart row, so the dot products need no shuffles; the rank-1 updates
// broadcast the 32 weights with shuffles and read V / K / dO rows coalesced.
// Nothing is accumulated with atomics: results are bitwise reproducible.
#include <math.h>

#include "attn.cuh"
#include "common.cuh"

namespace mgb {
namespace attn {
namespace {

constexpr int kWarps = 4;
constexpr int kMaxDPerLane = 16;  // D <= 512

template <typename T>
struct GArgs {
  const T *q, *k, *v, *mask, *o, *dy;
  const float *lse, *delta;
  T *out, *dq, *dk, *dv;
  float* lse_out;
  int B, S, H, D;
  float scale;
  int causal, has_bias;
  int64_t ld_qkv;   // elements between consecutive tokens of q / k / v (H*D when packed)
  int64_t ld_dqkv;  // same for dq / dk / dv
  int o_bshd;       // 0: O and dO are (B,H,S,D); 1: (B,S,H,D)
};

template <typename T>
__device__ __forceinline__ const T* row_bshd(const T* p, int b, int s, int h, int S, int64_t ld, int D) {
  return p + (static_cast<int64_t>(b) * S + s) * ld + static_cast<int64_t>(h) * D;
}
// element offset of row (b, h, s) of O / dO
__device__ __forceinline__ int64_t o_row_off(int o_bshd, int b, int h, int s, int S, int H, int D) {
  return o_bshd ? ((static_cast<int64_t>(b) * S + s) * H + h) * D : ((static_cast<int64_t>(b) * H + h) * S + s) * D;
}

// dot(q_row (shared, fp32), k_row (global))
template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ qs, const T* __restrict__ kr, int D) {
  float acc = 0.f;
  for (int d = 0; d < D; ++d) acc = fmaf(qs[d], to_f32(kr[d]), acc);
  return acc;
}

// ---- forward: warp per query row
template <typename T>
__global__ void __launch_bounds__(kWarps * 32) generic_fwd_kernel(const GArgs<T> a) {
  extern __shared__ float smem[];  // kWarps x D query rows
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarps + warp;
  const int64_t total = static_cast<int64_t>(a.B) * a.H * a.S;
  if (row >= total) return;
  const int i = static_cast<int>(row % a.S);
  const int bh = static_cast<int>(row / a.S);
  const int b = bh / a.H, h = bh % a.H;
  float* qs = smem + warp * a.D;
  const T* qr = row_bshd(a.q, b, i, h, a.S, a.ld_qkv, a.D);
  for (int d = lane; d < a.D; d += 32) qs[d] = to_f32(qr[d]);
  __syncwarp();
  float acc[kMaxDPerLane];
#pragma unroll
  for (int u = 0; u < kMaxDPerLane; ++u) acc[u] = 0.f;
  float m = -INFINITY, l = 0.f;
  const int j_end = a.causal ? i + 1 : a.S;
  for (int j0 = 0; j0 < j_end; j0 += 32) {
    const int j = j0 + lane;
    float s = -INFINITY;
    if (j < j_end) {
      s = dot_row(qs, row_bshd(a.k, b, j, h, a.S, a.ld_qkv, a.D), a.D) * a.scale;
      if (a.has_bias) s += to_f32(a.mask[(static_cast<int64_t>(bh) * a.S + i) * a.S + j]);
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    const float p = (j < j_end && m_new != -INFINITY) ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(p);
    m = m_new;
    const int cnt = min(32, j_end - j0);
#pragma unroll
    for (int u = 0; u < kMaxDPerLane; ++u) acc[u] *= corr;
    for (int jj = 0; jj < cnt; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const T* vr = row_bshd(a.v, b, j0 + jj, h, a.S, a.ld_qkv, a.D);
#pragma unroll
      for (int u = 0; u < kMaxDPerLane; ++u) {
        const int d = lane + 32 * u;
        if (d < a.D) acc[u] = fmaf(pj, to_f32(vr[d]), acc[u]);
      }
    }
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  T* orow = a.out + o_row_off(a.o_bshd, b, h, i, a.S, a.H, a.D);
#pragma unroll
  for (int u = 0; u < kMaxDPerLane; ++u) {
    const int d = lane + 32 * u;
    if (d < a.D) orow[d] = from_f32<T>(acc[u] * inv);
  }
  if (lane == 0 && a.lse_out) a.lse_out[row] = m + logf(l);
}

// ---- dQ: warp per query row; dq_i = sum_j ds_ij k_j, ds = p (dp - delta) scale
template <typename T>
__global__ void __launch_bounds__(kWarps * 32) generic_dq_kernel(const GArgs<T> a) {
  extern __shared__ float smem[];  // kWarps x 2D: q row, dO row
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarps + warp;
  const int64_t total = static_cast<int64_t>(a.B) * a.H * a.S;
  if (row >= total) return;
  const int i = static_cast<int>(row % a.S);
  const int bh = static_cast<int>(row / a.S);
  const int b = bh / a.H, h = bh % a.H;
  float* qs = smem + warp * 2 * a.D;
  float* dos = qs + a.D;
  const T* qr = row_bshd(a.q, b, i, h, a.S, a.ld_qkv, a.D);
  const T* dor = a.dy + o_row_off(a.o_bshd, b, h, i, a.S, a.H, a.D);
  for (int d = lane; d < a.D; d += 32) {
    qs[d] = to_f32(qr[d]);
    dos[d] = to_f32(dor[d]);
  }
  __syncwarp();
  const float lse = a.lse[row], delta = a.delta[row];
  float acc[kMaxDPerLane];
#pragma unroll
  for (int u = 0; u < kMaxDPerLane; ++u) acc[u] = 0.f;
  const int j_end = a.causal ? i + 1 : a.S;
  for (int j0 = 0; j0 < j_end; j0 += 32) {
    const int j = j0 + lane;
    float ds = 0.f;
    if (j < j_end) {
      float s = dot_row(qs, row_bshd(a.k, b, j, h, a.S, a.ld_qkv, a.D), a.D) * a.scale;
      if (a.has_bias) s += to_f32(a.mask[(static_cast<int64_t>(bh) * a.S + i) * a.S + j]);
      const float p = expf(s - lse);
      const float dp = dot_row(dos, row_bshd(a.v, b, j, h, a.S, a.ld_qkv, a.D), a.D);
      ds = p * (dp - delta) * a.scale;
    }
    const int cnt = min(32, j_end - j0);
    for (int jj = 0; jj < cnt; ++jj) {
      const float w = __shfl_sync(0xffffffffu, ds, jj);
      const T* kr = row_bshd(a.k, b, j0 + jj, h, a.S, a.ld_qkv, a.D);
#pragma unroll
      for (int u = 0; u < kMaxDPerLane; ++u) {
        const int d = lane + 32 * u;
        if (d < a.D) acc[u] = fmaf(w, to_f32(kr[d]), acc[u]);
      }
    }
  }
  T* dqr = a.dq + (static_cast<int64_t>(b) * a.S + i) * a.ld_dqkv + static_cast<int64_t>(h) * a.D;
#pragma unroll
  for (int u = 0; u < kMaxDPerLane; ++u) {
    const int d = lane + 32 * u;
    if (d < a.D) dqr[d] = from_f32<T>(acc[u]);
  }
}

// ---- dK/dV: warp per key row j; walks query rows i (>= j when causal)
template <typename T>
__global__ void __launch_bounds__(kWarps * 32) generic_dkdv_kernel(const GArgs<T> a) {
  extern __shared__ float smem[];  // kWarps x 2D: k row, v row
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarps + warp;
  const int64_t total = static_cast<int64_t>(a.B) * a.H * a.S;
  if (row >= total) return;
  const int j = static_cast<int>(row % a.S);
  const int bh = static_cast<int>(row / a.S);
  const int b = bh / a.H, h = bh % a.H;
  float* ks = smem + warp * 2 * a.D;
  float* vs = ks + a.D;
  const T* kr = row_bshd(a.k, b, j, h, a.S, a.ld_qkv, a.D);
  const T* vr = row_bshd(a.v, b, j, h, a.S, a.ld_qkv, a.D);
  for (int d = lane; d < a.D; d += 32) {
    ks[d] = to_f32(kr[d]);
    vs[d] = to_f32(vr[d]);
  }
  __syncwarp();
  float dk[kMaxDPerLane], dv[kMaxDPerLane];
#pragma unroll
  for (int u = 0; u < kMaxDPerLane; ++u) dk[u] = dv[u] = 0.f;
  const int i_begin = a.causal ? j : 0;
  for (int i0 = i_begin; i0 < a.S; i0 += 32) {
    const int i = i0 + lane;
    float p = 0.f, ds = 0.f;
    if (i < a.S) {
      const int64_t qrow = static_cast<int64_t>(bh) * a.S + i;
      float s = dot_row(ks, row_bshd(a.q, b, i, h, a.S, a.ld_qkv, a.D), a.D) * a.scale;
      if (a.has_bias) s += to_f32(a.mask[qrow * a.S + j]);
      p = expf(s - a.lse[qrow]);
      const float dp = dot_row(vs, a.dy + o_row_off(a.o_bshd, b, h, i, a.S, a.H, a.D), a.D);
      ds = p * (dp - a.delta[qrow]) * a.scale;
    }
    const int cnt = min(32, a.S - i0);
    for (int ii = 0; ii < cnt; ++ii) {
      const float pw = __shfl_sync(0xffffffffu, p, ii);
      const float dw = __shfl_sync(0xffffffffu, ds, ii);
      const T* qr = row_bshd(a.q, b, i0 + ii, h, a.S, a.ld_qkv, a.D);
      const T* dor = a.dy + o_row_off(a.o_bshd, b, h, i0 + ii, a.S, a.H, a.D);
#pragma unroll
      for (int u = 0; u < kMaxDPerLane; ++u) {
        const int d = lane + 32 * u;
        if (d < a.D) {
          dv[u] = fmaf(pw, to_f32(dor[d]), dv[u]);
          dk[u] = fmaf(dw, to_f32(qr[d]), dk[u]);
        }
      }
    }
  }
  T* dkr = a.dk + (static_cast<int64_t>(b) * a.S + j) * a.ld_dqkv + static_cast<int64_t>(h) * a.D;
  T* dvr = a.dv + (static_cast<int64_t>(b) * a.S + j) * a.ld_dqkv + static_cast<int64_t>(h) * a.D;
#pragma unroll
  for (int u = 0; u < kMaxDPerLane; ++u) {
    const int d = lane + 32 * u;
    if (d < a.D) {
      dkr[d] = from_f32<T>(dk[u]);
      dvr[d] = from_f32<T>(dv[u]);
    }
  }
}

// ---- delta[row] = sum_d O[row,d] * dO[row,d]   (both BHSD); warp per row
template <typename T>
__global__ void __launch_bounds__(256) delta_kernel(const T* __restrict__ o, const T* __restrict__ dy,
                                                    float* __restrict__ delta, int64_t rows, int S, int H, int D,
                                                    int o_bshd) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);  // (b, h, s) order
  if (row >= rows) return;
  const int s = static_cast<int>(row % S);
  const int bh = static_cast<int>(row / S);
  const int64_t off = o_row_off(o_bshd, bh / H, bh % H, s, S, H, D);
  const T* orow = o + off;
  const T* drow = dy + off;
  float acc = 0.f;
  for (int d = lane; d < D; d += 32) acc = fmaf(to_f32(orow[d]), to_f32(drow[d]), acc);
  acc = warp_sum(acc);
  if (lane == 0) delta[row] = acc;
}

}  // namespace

// Same reduction for packed 16-byte-aligned rows whose length is a power of two between 8 and 256 elements
// (bf16) : each thread takes one 16-byte slice, D/V lanes cover a row, a warp covers 32*V/D rows per step.
template <typename T>
__global__ void __launch_bounds__(256) delta_vec_kernel(const T* __restrict__ o, const T* __restrict__ dy,
                                                        float* __restrict__ delta, int64_t rows, int S, int H, int D,
                                                        int o_bshd, float* __restrict__ zero) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int V = Vec<T>::N;
  const int lanes_per_row = D / V;
  const int rows_per_warp = 32 / lanes_per_row;
  const int lane = threadIdx.x & 31;
  const int sub = lane / lanes_per_row, part = lane % lanes_per_row;
  const int64_t warp_global = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int64_t row = warp_global * rows_per_warp + sub;
  float acc = 0.f;
  if (row < rows) {
    const int s = static_cast<int>(row % S);
    const int bh = static_cast<int>(row / S);
    const int64_t off = o_row_off(o_bshd, bh / H, bh % H, s, S, H, D) + part * V;
    float a[V], b[V];
    load_vec(o + off, a);
    load_vec(dy + off, b);
#pragma unroll
    for (int e = 0; e < V; ++e) acc = fmaf(a[e], b[e], acc);
  }
  for (int ofs = lanes_per_row >> 1; ofs > 0; ofs >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, ofs);
  if (row < rows && part == 0) delta[row] = acc;
  // optional: clear an fp32 array with one element per element of O (the dQ accumulator of the tensor-core
  // backward), V floats per thread, instead of a separate fill pass
  if (zero != nullptr && row < rows) {
    float4* z = reinterpret_cast<float4*>(zero + (warp_global * 32 + lane) * V);
#pragma unroll
    for (int e = 0; e < V / 4; ++e) z[e] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

template <typename T>
int launch_delta(const void* o, const void* dy, float* delta, int B, int S, int H, int D, int o_bshd, float* zero,
                 bool* zeroed, cudaStream_t st) {
  if (zeroed) *zeroed = false;
  const int64_t rows = static_cast<int64_t>(B) * H * S;
  constexpr int V = Vec<T>::N;
  const int lpr = D / V;
  if (D % V == 0 && lpr >= 1 && lpr <= 32 && (lpr & (lpr - 1)) == 0 && aligned16(o) && aligned16(dy)) {
    const int rows_per_block = 8 * (32 / lpr);
    launch_pdl(delta_vec_kernel<T>, dim3(static_cast<unsigned>((rows + rows_per_block - 1) / rows_per_block)), dim3(256), 0, st,
               static_cast<const T*>(o), static_cast<const T*>(dy), delta, static_cast<int64_t>(rows), S, H, D, o_bshd,
               aligned16(zero) ? zero : static_cast<float*>(nullptr));
    if (zeroed) *zeroed = zero != nullptr && aligned16(zero);
    return check_launch("delta_vec_kernel");
  }
  delta_kernel<T><<<static_cast<unsigned>((rows + 7) / 8), 256, 0, st>>>(static_cast<const T*>(o),
                                                                       static_cast<const T*>(dy), delta, rows, S, H, D,
                                                                       o_bshd);
  return check_launch("delta_kernel");
}
template int launch_delta<float>(const void*, const void*, float*, int, int, int, int, int, float*, bool*, cudaStream_t);
template int launch_delta<__nv_bfloat16>(const void*, const void*, float*, int, int, int, int, int, float*, bool*, cudaStream_t);
template int launch_delta<__half>(const void*, const void*, float*, int, int, int, int, int, float*, bool*, cudaStream_t);

template <typename T>
int generic_fwd(const void* q, const void* k, const void* v, const void* mask, void* dst, float* lse, int B, int S,
                int H, int D, float scale, int causal, int has_bias, const Layouts& lay, cudaStream_t st) {
  GArgs<T> a{};
  a.q = static_cast<const T*>(q);
  a.k = static_cast<const T*>(k);
  a.v = static_cast<const T*>(v);
  a.mask = static_cast<const T*>(mask);
  a.out = static_cast<T*>(dst);
  a.lse_out = lse;
  a.B = B, a.S = S, a.H = H, a.D = D, a.scale = scale, a.causal = causal, a.has_bias = has_bias;
  a.ld_qkv = lay.ld_qkv, a.ld_dqkv = lay.ld_dqkv, a.o_bshd = lay.o_bshd;
  const int64_t rows = static_cast<int64_t>(B) * H * S;
  generic_fwd_kernel<T><<<static_cast<unsigned>((rows + kWarps - 1) / kWarps), kWarps * 32,
                          kWarps * D * sizeof(float), st>>>(a);
  return check_launch("generic_fwd_kernel");
}
template int generic_fwd<float>(const void*, const void*, const void*, const void*, void*, float*, int, int, int, int,
                                float, int, int, const Layouts&, cudaStream_t);
template int generic_fwd<__nv_bfloat16>(const void*, const void*, const void*, const void*, void*, float*, int, int,
                                        int, int, float, int, int, const Layouts&, cudaStream_t);
template int generic_fwd<__half>(const void*, const void*, const void*, const void*, void*, float*, int, int, int, int,
                                 float, int, int, const Layouts&, cudaStream_t);

template <typename T>
int generic_bwd(const void* dy, const void* q, const void* k, const void* v, const void* mask, const float* lse,
                const float* delta, void* dq, void* dk, void* dv, int B, int S, int H, int D, float scale, int causal,
                int has_bias, const Layouts& lay, cudaStream_t st) {
  GArgs<T> a{};
  a.q = static_cast<const T*>(q);
  a.k = static_cast<const T*>(k);
  a.v = static_cast<const T*>(v);
  a.mask = static_cast<const T*>(mask);
  a.dy = static_cast<const T*>(dy);
  a.lse = lse;
  a.delta = delta;
  a.dq = static_cast<T*>(dq);
  a.dk = static_cast<T*>(dk);
  a.dv = static_cast<T*>(dv);
  a.B = B, a.S = S, a.H = H, a.D = D, a.scale = scale, a.causal = causal, a.has_bias = has_bias;
  a.ld_qkv = lay.ld_qkv, a.ld_dqkv = lay.ld_dqkv, a.o_bshd = lay.o_bshd;
  const int64_t rows = static_cast<int64_t>(B) * H * S;
  const unsigned grid = static_cast<unsigned>((rows + kWarps - 1) / kWarps);
  const size_t smem = kWarps * 2 * D * sizeof(float);
  generic_dq_kernel<T><<<grid, kWarps * 32, smem, st>>>(a);
  int rc = check_launch("generic_dq_kernel");
  if (rc != MGB_OK) return rc;
  generic_dkdv_kernel<T><<<grid, kWarps * 32, smem, st>>>(a);
  return check_launch("generic_dkdv_kernel");
}
template int generic_bwd<float>(const void*, const void*, const void*, const void*, const void*, const float*,
                                const float*, void*, void*, void*, int, int, int, int, float, int, int, const Layouts&,
                                cudaStream_t);
template int generic_bwd<__nv_bfloat16>(const void*, const void*, const void*, const void*, const void*, const float*,
                                        const float*, void*, void*, void*, int, int, int, int, float, int, int,
                                        const Layouts&, cudaStream_t);
template int generic_bwd<__half>(const void*, const void*, const void*, const void*, const void*, const float*,
                                 const float*, void*, void*, void*, int, int, int, int, float, int, int, const Layouts&,
                                 cudaStream_t);

}  // namespace attn
}  // namespace mgb
