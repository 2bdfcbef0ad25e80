// Softmax cross-entropy: fused forward+backward with index labels, and the
// reference-shaped dense-label forward / backward entry points.
//
// Bandwidth-bound design: one CTA owns one row.  Pass 1 streams the row from
// HBM with 16-byte loads (four in flight per thread), keeps a copy in shared
// memory and folds it into an online (max, sum-exp) pair; pass 2 re-reads the
// row from shared memory and writes (softmax - label) * g with 16-byte
// stores.  The logits therefore cross HBM exactly once in each direction and
// the probabilities never exist in memory.  Rows too large for shared memory
// are re-read through L2 instead.  Short rows (a few KB) use one warp per row.
// Row losses go to a workspace and are summed by a single block in a fixed
// order, so the loss is bitwise reproducible.
#include <math.h>

#include "common.cuh"
#include "sm100.cuh"

namespace mgb {
namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr int kRowThreads = 512;
constexpr int kSmallThreads = 256;  // 8 warps, one row each
constexpr int kSumThreads = 1024;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// (m, s): running maximum and sum of exp(x - m).
__device__ __forceinline__ void ms_merge(float& m, float& s, float m2, float s2) {
  const float nm = fmaxf(m, m2);
  const float a = (m == -INFINITY) ? 0.f : s * ex2((m - nm) * kLog2e);
  const float b = (m2 == -INFINITY) ? 0.f : s2 * ex2((m2 - nm) * kLog2e);
  m = nm;
  s = a + b;
}

template <typename T>
struct XentParams {
  const T* logits;
  const T* dense;         // dense labels (N x C) or nullptr
  const int64_t* index;   // class index per row or nullptr
  T* dlogits;             // nullptr: forward only
  float* row_loss;        // nullptr: backward only
  const T* upstream_dev;  // one element, or nullptr -> upstream_host
  float upstream_host;
  int64_t N, C, ldx, ldl, lddx;
  int staged;                    // row copy kept in shared memory
  int vec_in, vec_lbl, vec_out;  // 16-byte access allowed for logits / labels / dlogits
};

template <int V>
__device__ __forceinline__ void fold_vec(const float (&v)[V], float& m, float& s) {
  float vm = v[0];
#pragma unroll
  for (int j = 1; j < V; ++j) vm = fmaxf(vm, v[j]);
  if (vm > m) {
    s *= ex2((m - vm) * kLog2e);  // first vector: m = -inf, s = 0 -> 0
    m = vm;
  }
  if (m != -INFINITY) {
    const float mb = m * kLog2e;
#pragma unroll
    for (int j = 0; j < V; ++j) s += ex2(fmaf(v[j], kLog2e, -mb));
  }
}

template <typename T>
__device__ __forceinline__ void load_labels(const T* lbl, int64_t i, bool vec, float (&l)[Vec<T>::N]) {
  constexpr int V = Vec<T>::N;
  if (vec) {
    load_vec(lbl + i * V, l);
  } else {
#pragma unroll
    for (int j = 0; j < V; ++j) l[j] = to_f32(lbl[i * V + j]);
  }
}

template <typename T, bool DENSE>
__global__ void __launch_bounds__(kRowThreads) xent_row_kernel(const XentParams<T> p) {
  constexpr int V = Vec<T>::N;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* row_s = reinterpret_cast<T*>(smem_raw);
  __shared__ float red[4][kRowThreads / 32];
  __shared__ float bcast[4];

  const int64_t row = blockIdx.x;
  const int tid = threadIdx.x;
  const T* x = p.logits + row * p.ldx;
  const T* lbl = DENSE ? p.dense + row * p.ldl : nullptr;
  const int nvec = p.vec_in ? static_cast<int>(p.C / V) : 0;

  float m = -INFINITY, s = 0.f, slx = 0.f, sl = 0.f;

  // ---- pass 1: HBM -> registers (-> shared), online max / sum-exp
  for (int i0 = 0; i0 < nvec; i0 += 4 * kRowThreads) {
    uint4 raw[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = i0 + u * kRowThreads + tid;
      if (i < nvec) raw[u] = __ldcs(reinterpret_cast<const uint4*>(x) + i);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = i0 + u * kRowThreads + tid;
      if (i < nvec) {
        if (p.staged) reinterpret_cast<uint4*>(row_s)[i] = raw[u];
        float v[V];
        load_vec(reinterpret_cast<const T*>(&raw[u]), v);
        fold_vec<V>(v, m, s);
        if (DENSE) {
          float l[V];
          load_labels<T>(lbl, i, p.vec_lbl, l);
#pragma unroll
          for (int j = 0; j < V; ++j) {
            slx = fmaf(l[j], v[j], slx);
            sl += l[j];
          }
        }
      }
    }
  }
  for (int c = nvec * V + tid; c < static_cast<int>(p.C); c += kRowThreads) {  // scalar tail / unaligned rows
    const T raw = x[c];
    if (p.staged) row_s[c] = raw;
    const float v = to_f32(raw);
    ms_merge(m, s, v, 1.f);
    if (DENSE) {
      const float l = to_f32(lbl[c]);
      slx = fmaf(l, v, slx);
      sl += l;
    }
  }

  // ---- block reduction of (m, s) and the label sums
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
    ms_merge(m, s, m2, s2);
  }
  if (DENSE) {
    slx = warp_sum(slx);
    sl = warp_sum(sl);
  }
  const int warp = tid >> 5, lane = tid & 31;
  if (lane == 0) {
    red[0][warp] = m;
    red[1][warp] = s;
    red[2][warp] = slx;
    red[3][warp] = sl;
  }
  __syncthreads();  // also publishes row_s
  if (warp == 0) {
    constexpr int W = kRowThreads / 32;
    float mm = lane < W ? red[0][lane] : -INFINITY;
    float ss = lane < W ? red[1][lane] : 0.f;
    float a = lane < W ? red[2][lane] : 0.f;
    float b = lane < W ? red[3][lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, mm, o);
      const float s2 = __shfl_xor_sync(0xffffffffu, ss, o);
      ms_merge(mm, ss, m2, s2);
    }
    a = warp_sum(a);
    b = warp_sum(b);
    if (lane == 0) {
      bcast[0] = mm;
      bcast[1] = ss;
      bcast[2] = a;
      bcast[3] = b;
    }
  }
  __syncthreads();
  m = bcast[0];
  s = bcast[1];

  int64_t t = -1;
  if (!DENSE) t = p.index[row];
  if (tid == 0 && p.row_loss) {
    const float lse = m + logf(s);
    float l;
    if (DENSE) {
      l = -(bcast[2] - lse * bcast[3]);
    } else {
      const float xt = (t >= 0 && t < p.C) ? to_f32(p.staged ? row_s[t] : x[t]) : lse;
      l = -(xt - lse);
    }
    p.row_loss[row] = l / static_cast<float>(p.N);
  }
  if (!p.dlogits) return;

  // ---- pass 2: shared (or L2) -> (softmax - label) * g -> HBM
  const float up = p.upstream_dev ? to_f32(p.upstream_dev[0]) : p.upstream_host;
  const float g = up / static_cast<float>(p.N);
  const float k = g / s;
  const float mb = m * kLog2e;
  T* out = p.dlogits + row * p.lddx;
  const T* src = p.staged ? row_s : x;
  const int C = static_cast<int>(p.C);
  const int nvec2 = (p.vec_out && (p.staged || p.vec_in)) ? C / V : 0;
  const int ti = (t >= 0 && t < p.C) ? static_cast<int>(t) : -1;
  // index labels with the row in shared memory: plain softmax * g in the loop, the target element is
  // rewritten afterwards by the thread that stored it (no per-element compare)
  const bool fixup = !DENSE && p.staged;
  for (int i = tid; i < nvec2; i += kRowThreads) {
    float v[V], o[V];
    load_vec(src + i * V, v);
    if (DENSE) {
      float l[V];
      load_labels<T>(lbl, i, p.vec_lbl, l);
#pragma unroll
      for (int j = 0; j < V; ++j) o[j] = fmaf(ex2(fmaf(v[j], kLog2e, -mb)), k, -l[j] * g);
    } else if (fixup) {
#pragma unroll
      for (int j = 0; j < V; ++j) o[j] = ex2(fmaf(v[j], kLog2e, -mb)) * k;
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j) o[j] = fmaf(ex2(fmaf(v[j], kLog2e, -mb)), k, (i * V + j == ti) ? -g : 0.f);
    }
    store_vec(out + i * V, o);
  }
  for (int c = nvec2 * V + tid; c < C; c += kRowThreads) {
    const float v = to_f32(src[c]);
    const float l = DENSE ? to_f32(lbl[c]) : ((c == ti && !fixup) ? 1.f : 0.f);
    out[c] = from_f32<T>(fmaf(ex2(fmaf(v, kLog2e, -mb)), k, -l * g));
  }
  if (fixup && ti >= 0) {
    const int owner = (ti < nvec2 * V) ? ((ti / V) % kRowThreads) : ((ti - nvec2 * V) % kRowThreads);
    if (tid == owner) out[ti] = from_f32<T>(fmaf(ex2(fmaf(to_f32(row_s[ti]), kLog2e, -mb)), k, -g));
  }
}

// One warp per row for short rows; the row is re-read from L1/L2 in pass 2.
template <typename T, bool DENSE>
__global__ void __launch_bounds__(kSmallThreads) xent_small_kernel(const XentParams<T> p) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (kSmallThreads / 32) + (threadIdx.x >> 5);
  if (row >= p.N) return;
  const T* x = p.logits + row * p.ldx;
  const T* lbl = DENSE ? p.dense + row * p.ldl : nullptr;
  float m = -INFINITY, s = 0.f, slx = 0.f, sl = 0.f;
  for (int64_t c = lane; c < p.C; c += 32) {
    const float v = to_f32(x[c]);
    ms_merge(m, s, v, 1.f);
    if (DENSE) {
      const float l = to_f32(lbl[c]);
      slx = fmaf(l, v, slx);
      sl += l;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
    ms_merge(m, s, m2, s2);
  }
  if (DENSE) {
    slx = warp_sum(slx);
    sl = warp_sum(sl);
  }
  int64_t t = -1;
  if (!DENSE) t = p.index[row];
  if (lane == 0 && p.row_loss) {
    const float lse = m + logf(s);
    float l;
    if (DENSE) {
      l = -(slx - lse * sl);
    } else {
      const float xt = (t >= 0 && t < p.C) ? to_f32(x[t]) : lse;
      l = -(xt - lse);
    }
    p.row_loss[row] = l / static_cast<float>(p.N);
  }
  if (!p.dlogits) return;
  const float up = p.upstream_dev ? to_f32(p.upstream_dev[0]) : p.upstream_host;
  const float g = up / static_cast<float>(p.N);
  const float inv_s = 1.f / s;
  const float mb = m * kLog2e;
  T* out = p.dlogits + row * p.lddx;
  for (int64_t c = lane; c < p.C; c += 32) {
    const float v = to_f32(x[c]);
    const float l = DENSE ? to_f32(lbl[c]) : (c == t ? 1.f : 0.f);
    out[c] = from_f32<T>((ex2(fmaf(v, kLog2e, -mb)) * inv_s - l) * g);
  }
}

// ---------------------------------------------------------------------------------------------------------
// Index-label fused forward+backward for long rows, fed by the bulk-copy engine.
// A persistent CTA (one per SM) owns every gridDim.x-th row.  A producer thread streams whole rows from HBM
// into one of two shared-memory row buffers with bulk copies; 16 compute warps turn the buffer into
// (softmax - onehot) * g in place; the producer sends the buffer back to HBM with bulk stores and refills
// it with the row after next once the stores have read it.  No logit passes through a register on its way in
// or out, so the compute warps only ever wait on shared memory, and the loads, exponentials and stores of
// neighbouring rows overlap.
constexpr int kBulkComputeThreads = 512;
constexpr int kBulkThreads = kBulkComputeThreads + 32;
constexpr uint32_t kBulkChunk = 32768;  // bytes per bulk copy
enum : int { kErrXentProducer = 301, kErrXentCompute = 302 };

template <typename T>
__global__ void __launch_bounds__(kBulkThreads, 1) xent_bulk_kernel(XentParams<T> p, int* status) {
  using namespace sm100;
  constexpr int V = Vec<T>::N;
  constexpr int W = kBulkComputeThreads / 32;
  extern __shared__ __align__(128) unsigned char xent_bulk_smem[];
  const uint32_t row_bytes = static_cast<uint32_t>(p.C) * sizeof(T);
  const uint32_t buf_stride = (row_bytes + 127u) & ~127u;
  unsigned char* base = xent_bulk_smem;
  const uint32_t base_s = smem_u32(base);
  const uint32_t bar_s = base_s + 2 * buf_stride;  // full[0], full[1], done[0], done[1]
  float* red = reinterpret_cast<float*>(base + 2 * buf_stride + 64);  // [2][W], then the two broadcast slots
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    mbar_init(bar_s + 0, 1);
    mbar_init(bar_s + 8, 1);
    mbar_init(bar_s + 16, W);
    mbar_init(bar_s + 24, W);
    mbar_fence_init();
  }
  __syncthreads();
  const int64_t first = blockIdx.x, step = gridDim.x;

  if (warp == W) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      auto load_row = [&](int64_t row, int b) {
        mbar_expect_tx(bar_s + 8 * b, row_bytes);
        const unsigned char* src = reinterpret_cast<const unsigned char*>(p.logits + row * p.ldx);
        for (uint32_t off = 0; off < row_bytes; off += kBulkChunk) {
          const uint32_t n = row_bytes - off < kBulkChunk ? row_bytes - off : kBulkChunk;
          bulk_load_1d(base_s + b * buf_stride + off, src + off, n, bar_s + 8 * b);
        }
      };
      for (int i = 0; i < 2; ++i)
        if (first + i * step < p.N) load_row(first + i * step, i);
      int i = 0;
      for (int64_t row = first; row < p.N; row += step, ++i) {
        const int b = i & 1;
        if (!mbar_wait(bar_s + 16 + 8 * b, (i >> 1) & 1u)) {
          atomicExch(status, kErrXentProducer);
          break;
        }
        if (p.dlogits) {
          unsigned char* dst = reinterpret_cast<unsigned char*>(p.dlogits + row * p.lddx);
          for (uint32_t off = 0; off < row_bytes; off += kBulkChunk) {
            const uint32_t n = row_bytes - off < kBulkChunk ? row_bytes - off : kBulkChunk;
            bulk_store_1d(dst + off, base_s + b * buf_stride + off, n);
          }
          bulk_commit();
        }
        if (row + 2 * step < p.N) {
          if (p.dlogits) bulk_wait_read0();  // the stores have left the buffer
          load_row(row + 2 * step, b);
        }
      }
      bulk_wait0();  // every row is in memory before the CTA retires
    }
    return;
  }

  // ------------------------------------------------------------------ compute warps
  const float up = p.upstream_dev ? to_f32(p.upstream_dev[0]) : p.upstream_host;
  const float g = up / static_cast<float>(p.N);
  const int C = static_cast<int>(p.C);
  const int nvec = C / V;  // the launcher guarantees C % V == 0
  int i = 0;
  for (int64_t row = first; row < p.N; row += step, ++i) {
    const int b = i & 1;
    T* row_s = reinterpret_cast<T*>(base + b * buf_stride);
    const int64_t t = p.index[row];
    const int ti = (t >= 0 && t < p.C) ? static_cast<int>(t) : -1;
    if (!mbar_wait(bar_s + 8 * b, (i >> 1) & 1u)) {
      if (lane == 0) atomicExch(status, kErrXentCompute);
      break;
    }
    const float xt = ti >= 0 ? to_f32(row_s[ti]) : 0.f;  // read before anyone overwrites the row
    // ---- pass 1: online (max, sum exp)
    float m = -INFINITY, s = 0.f;
#pragma unroll 2
    for (int v0 = tid; v0 < nvec; v0 += kBulkComputeThreads) {
      float v[V];
      load_vec(row_s + v0 * V, v);
      fold_vec<V>(v, m, s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
      const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
      ms_merge(m, s, m2, s2);
    }
    if (lane == 0) {
      red[warp] = m;
      red[W + warp] = s;
    }
    named_barrier(1, kBulkComputeThreads);
    if (warp == 0) {
      float mm = lane < W ? red[lane] : -INFINITY;
      float ss = lane < W ? red[W + lane] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, mm, o);
        const float s2 = __shfl_xor_sync(0xffffffffu, ss, o);
        ms_merge(mm, ss, m2, s2);
      }
      if (lane == 0) {
        red[2 * W] = mm;
        red[2 * W + 1] = ss;
      }
    }
    named_barrier(1, kBulkComputeThreads);
    m = red[2 * W];
    s = red[2 * W + 1];
    if (tid == 0 && p.row_loss) {
      const float lse = m + logf(s);
      p.row_loss[row] = (ti >= 0 ? lse - xt : 0.f) / static_cast<float>(p.N);
    }
    if (p.dlogits) {
      // ---- pass 2: (softmax - onehot) * g, in place
      const float k = g / s;
      const float mb = m * kLog2e;
#pragma unroll 2
      for (int v0 = tid; v0 < nvec; v0 += kBulkComputeThreads) {
        float v[V], o[V];
        load_vec(row_s + v0 * V, v);
#pragma unroll
        for (int j = 0; j < V; ++j) o[j] = ex2(fmaf(v[j], kLog2e, -mb)) * k;
        store_vec(row_s + v0 * V, o);
      }
      // the thread that wrote the target's vector rewrites that one element
      if (ti >= 0 && (ti / V) % kBulkComputeThreads == tid)
        row_s[ti] = from_f32<T>(ex2(fmaf(xt, kLog2e, -mb)) * k - g);
      fence_async_smem();  // the bulk stores read these writes through the async proxy
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_s + 16 + 8 * b);
    // red[] is rewritten only after the next row's first barrier, which every thread reaches after reading m, s
  }
}

// Fixed-order sum of the per-row losses (already divided by N).
template <typename TOut>
__global__ void __launch_bounds__(kSumThreads) xent_sum_rows_kernel(const float* row_loss, int64_t N, TOut* loss) {
  __shared__ float red[kSumThreads / 32];
  float acc = 0.f;
  for (int64_t i = threadIdx.x; i < N; i += kSumThreads) acc += row_loss[i];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < kSumThreads / 32 ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) loss[0] = from_f32<TOut>(v);
  }
}

template <typename T, bool DENSE>
int launch_xent(XentParams<T> p, cudaStream_t st) {
  constexpr int V = Vec<T>::N;
  p.vec_in = aligned16(p.logits) && (p.ldx % V == 0);
  p.vec_lbl = DENSE && aligned16(p.dense) && (p.ldl % V == 0);
  p.vec_out = p.dlogits && aligned16(p.dlogits) && (p.lddx % V == 0);
  const size_t row_bytes = static_cast<size_t>(p.C) * sizeof(T);
  if (row_bytes <= 4096) {
    p.staged = 0;
    const int rows_per_block = kSmallThreads / 32;
    const unsigned grid = static_cast<unsigned>((p.N + rows_per_block - 1) / rows_per_block);
    xent_small_kernel<T, DENSE><<<grid, kSmallThreads, 0, st>>>(p);
    return check_launch("xent_small_kernel");
  }
  const size_t smem_cap = static_cast<size_t>(max_smem_optin()) - 1024;  // static reductions live there too
  if (!DENSE) {
    // long rows of index-label problems go through the bulk-copy kernel when two row buffers fit
    const size_t need = 2 * round_up(row_bytes, 128) + 64 + (2 * (kBulkComputeThreads / 32) + 2) * sizeof(float);
    const bool aligned = row_bytes % 16 == 0 && p.vec_in && (!p.dlogits || p.vec_out) && (p.C % V == 0);
    if (row_bytes >= 32 * 1024 && aligned && need <= smem_cap) {
      int* status = device_status_ptr();
      if (!status) return fail(MGB_ECUDA, "xent: device status word unavailable");
      auto kern = xent_bulk_kernel<T>;
      const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(need));
      if (e != cudaSuccess) return fail(MGB_ECUDA, "xent smem opt-in (%zu B): %s", need, cudaGetErrorString(e));
      const int64_t grid = p.N < sm_count() ? p.N : sm_count();
      kern<<<static_cast<unsigned>(grid), kBulkThreads, need, st>>>(p, status);
      return check_launch("xent_bulk_kernel");
    }
  }
  const size_t smem = round_up(row_bytes, 16);
  p.staged = smem <= smem_cap;
  const size_t dyn = p.staged ? smem : 0;
  auto kern = xent_row_kernel<T, DENSE>;
  if (dyn > 48 * 1024) {
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(dyn));
    if (e != cudaSuccess) return fail(MGB_ECUDA, "xent smem opt-in (%zu B): %s", dyn, cudaGetErrorString(e));
  }
  kern<<<static_cast<unsigned>(p.N), kRowThreads, dyn, st>>>(p);
  return check_launch("xent_row_kernel");
}

template <typename T>
int xent_index(const void* logits, const int64_t* labels, float* loss, void* dlogits, int64_t N, int64_t C,
               int64_t ldx, int64_t lddx, float upstream, void* ws, cudaStream_t st) {
  XentParams<T> p{};
  p.logits = static_cast<const T*>(logits);
  p.index = labels;
  p.dlogits = static_cast<T*>(dlogits);
  p.row_loss = loss ? static_cast<float*>(ws) : nullptr;
  p.upstream_host = upstream;
  p.N = N;
  p.C = C;
  p.ldx = ldx;
  p.lddx = lddx;
  int rc = launch_xent<T, false>(p, st);
  if (rc != MGB_OK) return rc;
  if (loss) {
    xent_sum_rows_kernel<float><<<1, kSumThreads, 0, st>>>(p.row_loss, N, loss);
    rc = check_launch("xent_sum_rows_kernel");
  }
  return rc;
}

template <typename T>
int xent_dense_fwd(const void* logits, const void* labels, void* loss, int64_t N, int64_t C, int64_t ldx,
                   int64_t ldl, void* ws, cudaStream_t st) {
  XentParams<T> p{};
  p.logits = static_cast<const T*>(logits);
  p.dense = static_cast<const T*>(labels);
  p.row_loss = static_cast<float*>(ws);
  p.N = N;
  p.C = C;
  p.ldx = ldx;
  p.ldl = ldl;
  int rc = launch_xent<T, true>(p, st);
  if (rc != MGB_OK) return rc;
  xent_sum_rows_kernel<T><<<1, kSumThreads, 0, st>>>(p.row_loss, N, static_cast<T*>(loss));
  return check_launch("xent_sum_rows_kernel");
}

template <typename T>
int xent_dense_bwd(const void* upstream, const void* logits, const void* labels, void* dst, int64_t N, int64_t C,
                   int64_t ldx, int64_t ldl, int64_t lddst, cudaStream_t st) {
  XentParams<T> p{};
  p.logits = static_cast<const T*>(logits);
  p.dense = static_cast<const T*>(labels);
  p.dlogits = static_cast<T*>(dst);
  p.upstream_dev = static_cast<const T*>(upstream);
  p.N = N;
  p.C = C;
  p.ldx = ldx;
  p.ldl = ldl;
  p.lddx = lddst;
  return launch_xent<T, true>(p, st);
}

int check_shape(int64_t N, int64_t C, int64_t ldx) {
  MGB_REQUIRE(N > 0 && C > 0, MGB_EINVAL, "cross_entropy: N=%lld C=%lld must be positive", (long long)N, (long long)C);
  MGB_REQUIRE(N <= 0x7fffffffLL, MGB_EUNSUPPORTED, "cross_entropy: N=%lld exceeds the grid limit", (long long)N);
  MGB_REQUIRE(ldx >= C, MGB_EINVAL, "cross_entropy: row stride %lld < C=%lld", (long long)ldx, (long long)C);
  return MGB_OK;
}

}  // namespace
}  // namespace mgb

using namespace mgb;

MGB_EXPORT size_t mograd_b200_softmax_xent_workspace_bytes(int64_t N, int64_t, int) {
  return N > 0 ? round_up(static_cast<size_t>(N) * sizeof(float), 256) : 0;
}
MGB_EXPORT size_t mograd_b200_cross_entropy_workspace_bytes(int64_t N, int64_t C, int dtype) {
  return mograd_b200_softmax_xent_workspace_bytes(N, C, dtype);
}

MGB_EXPORT int mograd_b200_softmax_xent_fwd_bwd(const void* logits, const int64_t* labels, float* loss,
                                                void* dlogits, int64_t N, int64_t C, int64_t ldx, int64_t lddx,
                                                float upstream, int dtype, void* workspace,
                                                size_t workspace_bytes, void* stream) {
  MGB_REQUIRE(logits && labels, MGB_EINVAL, "softmax_xent_fwd_bwd: logits / labels is NULL");
  MGB_REQUIRE(loss || dlogits, MGB_EINVAL, "softmax_xent_fwd_bwd: both outputs are NULL");
  int rc = check_shape(N, C, ldx);
  if (rc != MGB_OK) return rc;
  MGB_REQUIRE(!dlogits || lddx >= C, MGB_EINVAL, "softmax_xent_fwd_bwd: lddx %lld < C", (long long)lddx);
  if (loss)
    MGB_REQUIRE(workspace && workspace_bytes >= mograd_b200_softmax_xent_workspace_bytes(N, C, dtype),
                MGB_EWORKSPACE, "softmax_xent_fwd_bwd: workspace of %zu bytes needed, %zu given",
                mograd_b200_softmax_xent_workspace_bytes(N, C, dtype), workspace ? workspace_bytes : (size_t)0);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case MGB_BF16:
      return xent_index<__nv_bfloat16>(logits, labels, loss, dlogits, N, C, ldx, lddx, upstream, workspace, st);
    case MGB_F32:
      return xent_index<float>(logits, labels, loss, dlogits, N, C, ldx, lddx, upstream, workspace, st);
    case MGB_F16:
      return xent_index<__half>(logits, labels, loss, dlogits, N, C, ldx, lddx, upstream, workspace, st);
    default:
      return fail(MGB_EDTYPE, "softmax_xent_fwd_bwd: unsupported dtype code %d", dtype);
  }
}

MGB_EXPORT int mograd_b200_cross_entropy(const void* logits, const void* labels, void* loss, int64_t N, int64_t C,
                                         int64_t ldx, int64_t ldl, int dtype, void* workspace,
                                         size_t workspace_bytes, void* stream) {
  MGB_REQUIRE(logits && labels && loss, MGB_EINVAL, "cross_entropy: NULL argument");
  int rc = check_shape(N, C, ldx);
  if (rc != MGB_OK) return rc;
  MGB_REQUIRE(ldl >= C, MGB_EINVAL, "cross_entropy: label row stride %lld < C", (long long)ldl);
  MGB_REQUIRE(workspace && workspace_bytes >= mograd_b200_cross_entropy_workspace_bytes(N, C, dtype),
              MGB_EWORKSPACE, "cross_entropy: workspace of %zu bytes needed, %zu given",
              mograd_b200_cross_entropy_workspace_bytes(N, C, dtype), workspace ? workspace_bytes : (size_t)0);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case MGB_BF16:
      return xent_dense_fwd<__nv_bfloat16>(logits, labels, loss, N, C, ldx, ldl, workspace, st);
    case MGB_F32:
      return xent_dense_fwd<float>(logits, labels, loss, N, C, ldx, ldl, workspace, st);
    case MGB_F16:
      return xent_dense_fwd<__half>(logits, labels, loss, N, C, ldx, ldl, workspace, st);
    default:
      return fail(MGB_EDTYPE, "cross_entropy: unsupported dtype code %d", dtype);
  }
}

MGB_EXPORT int mograd_b200_cross_entropy_grad(const void* upstream, const void* logits, const void* labels,
                                              void* dst, int64_t N, int64_t C, int64_t ldx, int64_t ldl,
                                              int64_t lddst, int dtype, void* stream) {
  MGB_REQUIRE(upstream && logits && labels && dst, MGB_EINVAL, "cross_entropy_grad: NULL argument");
  int rc = check_shape(N, C, ldx);
  if (rc != MGB_OK) return rc;
  MGB_REQUIRE(ldl >= C && lddst >= C, MGB_EINVAL, "cross_entropy_grad: row stride < C");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case MGB_BF16:
      return xent_dense_bwd<__nv_bfloat16>(upstream, logits, labels, dst, N, C, ldx, ldl, lddst, st);
    case MGB_F32:
      return xent_dense_bwd<float>(upstream, logits, labels, dst, N, C, ldx, ldl, lddst, st);
    case MGB_F16:
      return xent_dense_bwd<__half>(upstream, logits, labels, dst, N, C, ldx, ldl, lddst, st);
    default:
      return fail(MGB_EDTYPE, "cross_entropy_grad: unsupported dtype code %d", dtype);
  }
}
