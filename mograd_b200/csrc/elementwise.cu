// Callers of the hot path inside a train step: ReLU backward, residual add,
// embedding gather / scatter-add and the AdamW update.  All are one pass over
// their operands with 16-byte accesses where the pointers allow it.
#include "common.cuh"

namespace mgb {
namespace {

constexpr int kEwThreads = 256;

inline int ew_grid(int64_t work_items) {
  int64_t g = (work_items + kEwThreads - 1) / kEwThreads;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  if (g > cap) g = cap;
  return g < 1 ? 1 : static_cast<int>(g);
}

// dx = dy where y > 0 else 0 (y is the ReLU output).  dx may alias dy: no __restrict__ on either.
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
    relu_grad_kernel(const T* __restrict__ y, const T* dy, T* dx, int64_t n, int vec) {
  constexpr int V = Vec<T>::N;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kEwThreads;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * kEwThreads + threadIdx.x;
  const int64_t nv = vec ? n / V : 0;
  for (int64_t i = tid; i < nv; i += stride) {
    float a[V], b[V], o[V];
    load_vec(y + i * V, a);
    load_vec(dy + i * V, b);
#pragma unroll
    for (int j = 0; j < V; ++j) o[j] = a[j] > 0.f ? b[j] : 0.f;
    store_vec(dx + i * V, o);
  }
  for (int64_t i = nv * V + tid; i < n; i += stride) dx[i] = to_f32(y[i]) > 0.f ? dy[i] : from_f32<T>(0.f);
}

// dst may alias a or b: no __restrict__.
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
    add_kernel(const T* a, const T* b, T* dst, int64_t n, int vec) {
  constexpr int V = Vec<T>::N;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kEwThreads;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * kEwThreads + threadIdx.x;
  const int64_t nv = vec ? n / V : 0;
  for (int64_t i = tid; i < nv; i += stride) {
    float x[V], y[V], o[V];
    load_vec(a + i * V, x);
    load_vec(b + i * V, y);
#pragma unroll
    for (int j = 0; j < V; ++j) o[j] = x[j] + y[j];
    store_vec(dst + i * V, o);
  }
  for (int64_t i = nv * V + tid; i < n; i += stride) dst[i] = from_f32<T>(to_f32(a[i]) + to_f32(b[i]));
}

// out[t, :] = table[idx[t], :]; one warp per row chunk
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
    gather_rows_kernel(const T* __restrict__ table, const int64_t* __restrict__ idx, T* __restrict__ out, int64_t rows,
                       int64_t vocab, int64_t d, int vec) {
  constexpr int V = Vec<T>::N;
  const int64_t per_row = vec ? d / V : d;
  const int64_t total = rows * per_row;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kEwThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kEwThreads + threadIdx.x; i < total; i += stride) {
    const int64_t t = i / per_row, c = i - t * per_row;
    int64_t r = idx[t];
    r = r < 0 ? 0 : (r >= vocab ? vocab - 1 : r);
    if (vec)
      reinterpret_cast<uint4*>(out + t * d)[c] = reinterpret_cast<const uint4*>(table + r * d)[c];
    else
      out[t * d + c] = table[r * d + c];
  }
}

// acc[idx[t], :] += dout[t, :] in fp32
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
    scatter_add_rows_kernel(const T* __restrict__ dout, const int64_t* __restrict__ idx, float* __restrict__ acc,
                            int64_t rows, int64_t vocab, int64_t d) {
  const int64_t total = rows * d;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kEwThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kEwThreads + threadIdx.x; i < total; i += stride) {
    const int64_t t = i / d, c = i - t * d;
    const int64_t r = idx[t];
    if (r >= 0 && r < vocab) atomicAdd(acc + r * d + c, to_f32(dout[i]));
  }
}

template <typename T>
__global__ void __launch_bounds__(kEwThreads) cast_from_f32_kernel(const float* __restrict__ src, T* __restrict__ dst, int64_t n) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kEwThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kEwThreads + threadIdx.x; i < n; i += stride)
    dst[i] = from_f32<T>(src[i]);
}

// AdamW with bias correction and decoupled weight decay:
//   m = b1 m + (1-b1) g;  v = b2 v + (1-b2) g^2
//   w = w (1 - lr wd) - lr (m / bc1) / (sqrt(v / bc2) + eps)
// (mograd/nn/optim/adam.mojo:6-58, decoupled_wd = True).  m, v and the master
// copy are fp32; w is rewritten in its storage dtype from the master copy.
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
    adamw_kernel(T* __restrict__ w, const T* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                 float* __restrict__ master, int64_t n, float lr, float b1, float b2, float eps, float wd, float inv_bc1,
                 float inv_bc2, float grad_scale, int vec, const int* __restrict__ step_dev) {
  constexpr int V = Vec<T>::N;  // elements per 16-byte access of the parameter type
  if (step_dev) {  // step number kept on the device (a captured launch cannot carry a new scalar per replay)
    const float t = static_cast<float>(*step_dev);
    inv_bc1 = 1.f / (1.f - powf(b1, t));
    inv_bc2 = 1.f / (1.f - powf(b2, t));
  }
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kEwThreads;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * kEwThreads + threadIdx.x;
  const float decay = wd > 0.f ? 1.f - lr * wd : 1.f;
  auto update = [&](float gi, float& mi, float& vi, float& wi) {
    gi *= grad_scale;
    mi = b1 * mi + (1.f - b1) * gi;
    vi = b2 * vi + (1.f - b2) * gi * gi;
    // sqrt.approx and the reciprocal-multiply division are within 2 ulp each; their error enters w scaled by lr,
    // far below the rounding of w itself, and they take a third of the instructions of the IEEE forms: under the
    // step's power cap this kernel is bound by instruction issue, not by DRAM
    float root, inv;
    asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(root) : "f"(vi * inv_bc2));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(inv) : "f"(root + eps));
    wi = fmaf(-lr * (mi * inv_bc1), inv, wi * decay);
  };
  const int64_t nv = vec ? n / V : 0;
  for (int64_t i = tid; i < nv; i += stride) {
    // every stream is read with 16-byte loads issued before any arithmetic
    float gf[V], wf[V];
    float4 mq[V / 4], vq[V / 4], wq[V / 4];
    load_vec(g + i * V, gf);
#pragma unroll
    for (int q = 0; q < V / 4; ++q) {
      mq[q] = reinterpret_cast<const float4*>(m)[i * (V / 4) + q];
      vq[q] = reinterpret_cast<const float4*>(v)[i * (V / 4) + q];
      if (master) wq[q] = reinterpret_cast<const float4*>(master)[i * (V / 4) + q];
    }
    if (master) {
#pragma unroll
      for (int q = 0; q < V / 4; ++q) {
        wf[4 * q] = wq[q].x;
        wf[4 * q + 1] = wq[q].y;
        wf[4 * q + 2] = wq[q].z;
        wf[4 * q + 3] = wq[q].w;
      }
    } else {
      load_vec(w + i * V, wf);
    }
#pragma unroll
    for (int q = 0; q < V / 4; ++q) {
      update(gf[4 * q], mq[q].x, vq[q].x, wf[4 * q]);
      update(gf[4 * q + 1], mq[q].y, vq[q].y, wf[4 * q + 1]);
      update(gf[4 * q + 2], mq[q].z, vq[q].z, wf[4 * q + 2]);
      update(gf[4 * q + 3], mq[q].w, vq[q].w, wf[4 * q + 3]);
      reinterpret_cast<float4*>(m)[i * (V / 4) + q] = mq[q];
      reinterpret_cast<float4*>(v)[i * (V / 4) + q] = vq[q];
      if (master)
        reinterpret_cast<float4*>(master)[i * (V / 4) + q] = make_float4(wf[4 * q], wf[4 * q + 1], wf[4 * q + 2], wf[4 * q + 3]);
    }
    store_vec(w + i * V, wf);
  }
  for (int64_t i = nv * V + tid; i < n; i += stride) {
    float mi = m[i], vi = v[i];
    float wi = master ? master[i] : to_f32(w[i]);
    update(to_f32(g[i]), mi, vi, wi);
    m[i] = mi;
    v[i] = vi;
    if (master) master[i] = wi;
    w[i] = from_f32<T>(wi);
  }
}

template <typename T>
bool vec_ok3(const void* a, const void* b, const void* c) {
  return aligned16(a) && aligned16(b) && aligned16(c);
}

}  // namespace
}  // namespace mgb

using namespace mgb;

#define MGB_DTYPE_SWITCH(dtype, who, ...)                                   \
  switch (dtype) {                                                          \
    case MGB_BF16: {                                                        \
      using T = __nv_bfloat16;                                              \
      __VA_ARGS__;                                                          \
    } break;                                                                \
    case MGB_F32: {                                                         \
      using T = float;                                                      \
      __VA_ARGS__;                                                          \
    } break;                                                                \
    case MGB_F16: {                                                         \
      using T = __half;                                                     \
      __VA_ARGS__;                                                          \
    } break;                                                                \
    default:                                                                \
      return fail(MGB_EDTYPE, who ": unsupported dtype code %d", dtype);    \
  }

MGB_EXPORT int mograd_b200_relu_grad(const void* y, const void* dy, void* dx, int64_t numel, int dtype, void* stream) {
  MGB_REQUIRE(y && dy && dx, MGB_EINVAL, "relu_grad: NULL argument");
  MGB_REQUIRE(numel > 0, MGB_EINVAL, "relu_grad: numel=%lld", (long long)numel);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MGB_DTYPE_SWITCH(dtype, "relu_grad", {
    const int vec = vec_ok3<T>(y, dy, dx);
    relu_grad_kernel<T><<<ew_grid(numel / Vec<T>::N + 1), kEwThreads, 0, st>>>(
        static_cast<const T*>(y), static_cast<const T*>(dy), static_cast<T*>(dx), numel, vec);
  })
  return check_launch("relu_grad_kernel");
}

MGB_EXPORT int mograd_b200_add(const void* a, const void* b, void* dst, int64_t numel, int dtype, void* stream) {
  MGB_REQUIRE(a && b && dst, MGB_EINVAL, "add: NULL argument");
  MGB_REQUIRE(numel > 0, MGB_EINVAL, "add: numel=%lld", (long long)numel);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MGB_DTYPE_SWITCH(dtype, "add", {
    const int vec = vec_ok3<T>(a, b, dst);
    add_kernel<T><<<ew_grid(numel / Vec<T>::N + 1), kEwThreads, 0, st>>>(static_cast<const T*>(a), static_cast<const T*>(b),
                                                                      static_cast<T*>(dst), numel, vec);
  })
  return check_launch("add_kernel");
}

MGB_EXPORT int mograd_b200_gather_rows(const void* table, const int64_t* idx, void* out, int64_t rows, int64_t vocab,
                                       int64_t d, int dtype, void* stream) {
  MGB_REQUIRE(table && idx && out, MGB_EINVAL, "gather_rows: NULL argument");
  MGB_REQUIRE(rows > 0 && vocab > 0 && d > 0, MGB_EINVAL, "gather_rows: non-positive dimension");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MGB_DTYPE_SWITCH(dtype, "gather_rows", {
    const int vec = aligned16(table) && aligned16(out) && (d % Vec<T>::N == 0);
    gather_rows_kernel<T><<<ew_grid(rows * (vec ? d / Vec<T>::N : d)), kEwThreads, 0, st>>>(
        static_cast<const T*>(table), idx, static_cast<T*>(out), rows, vocab, d, vec);
  })
  return check_launch("gather_rows_kernel");
}

MGB_EXPORT size_t mograd_b200_scatter_add_rows_workspace_bytes(int64_t vocab, int64_t d, int dtype) {
  if (vocab <= 0 || d <= 0) return 0;
  return dtype == MGB_F32 ? 0 : round_up(static_cast<size_t>(vocab) * d * sizeof(float), 256);
}

MGB_EXPORT int mograd_b200_scatter_add_rows(const void* dout, const int64_t* idx, void* dtable, int64_t rows,
                                            int64_t vocab, int64_t d, int dtype, void* workspace,
                                            size_t workspace_bytes, void* stream) {
  MGB_REQUIRE(dout && idx && dtable, MGB_EINVAL, "scatter_add_rows: NULL argument");
  MGB_REQUIRE(rows > 0 && vocab > 0 && d > 0, MGB_EINVAL, "scatter_add_rows: non-positive dimension");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t need = mograd_b200_scatter_add_rows_workspace_bytes(vocab, d, dtype);
  MGB_REQUIRE(need == 0 || (workspace && workspace_bytes >= need), MGB_EWORKSPACE,
              "scatter_add_rows: workspace of %zu bytes needed", need);
  const int64_t n = vocab * d;
  if (dtype == MGB_F32) {
    float* acc = static_cast<float*>(dtable);
    if (cudaMemsetAsync(acc, 0, n * sizeof(float), st) != cudaSuccess) return fail(MGB_ECUDA, "scatter_add_rows: memset failed");
    scatter_add_rows_kernel<float><<<ew_grid(rows * d), kEwThreads, 0, st>>>(static_cast<const float*>(dout), idx, acc,
                                                                           rows, vocab, d);
    return check_launch("scatter_add_rows_kernel");
  }
  MGB_REQUIRE(dtype == MGB_BF16 || dtype == MGB_F16, MGB_EDTYPE, "scatter_add_rows: unsupported dtype code %d", dtype);
  float* acc = static_cast<float*>(workspace);
  if (cudaMemsetAsync(acc, 0, n * sizeof(float), st) != cudaSuccess) return fail(MGB_ECUDA, "scatter_add_rows: memset failed");
  if (dtype == MGB_BF16)
    scatter_add_rows_kernel<__nv_bfloat16><<<ew_grid(rows * d), kEwThreads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(dout), idx, acc, rows, vocab, d);
  else
    scatter_add_rows_kernel<__half><<<ew_grid(rows * d), kEwThreads, 0, st>>>(static_cast<const __half*>(dout), idx, acc,
                                                                            rows, vocab, d);
  int rc = check_launch("scatter_add_rows_kernel");
  if (rc != MGB_OK) return rc;
  if (dtype == MGB_BF16)
    cast_from_f32_kernel<__nv_bfloat16><<<ew_grid(n), kEwThreads, 0, st>>>(acc, static_cast<__nv_bfloat16*>(dtable), n);
  else
    cast_from_f32_kernel<__half><<<ew_grid(n), kEwThreads, 0, st>>>(acc, static_cast<__half*>(dtable), n);
  return check_launch("cast_from_f32_kernel");
}

MGB_EXPORT int mograd_b200_adamw_step(void* w, const void* g, float* m, float* v, float* master, int64_t numel, float lr,
                                      float beta1, float beta2, float eps, float weight_decay, int step,
                                      float grad_scale, int dtype, void* stream) {
  MGB_REQUIRE(w && g && m && v, MGB_EINVAL, "adamw_step: NULL argument");
  MGB_REQUIRE(numel > 0 && step >= 1, MGB_EINVAL, "adamw_step: numel=%lld step=%d", (long long)numel, step);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const float inv_bc1 = 1.f / (1.f - powf(beta1, static_cast<float>(step)));
  const float inv_bc2 = 1.f / (1.f - powf(beta2, static_cast<float>(step)));
  MGB_DTYPE_SWITCH(dtype, "adamw_step", {
    const int vec = aligned16(w) && aligned16(g) && aligned16(m) && aligned16(v) && (!master || aligned16(master));
    adamw_kernel<T><<<ew_grid(numel / Vec<T>::N + 1), kEwThreads, 0, st>>>(
        static_cast<T*>(w), static_cast<const T*>(g), m, v, master, numel, lr, beta1, beta2, eps, weight_decay, inv_bc1,
        inv_bc2, grad_scale, vec, nullptr);
  })
  return check_launch("adamw_kernel");
}

namespace mgb {
namespace {
__global__ void bump_counter_kernel(int* c) { *c += 1; }
}  // namespace
}  // namespace mgb

MGB_EXPORT int mograd_b200_adamw_step_dev(void* w, const void* g, float* m, float* v, float* master, int64_t numel,
                                          float lr, float beta1, float beta2, float eps, float weight_decay,
                                          int* step_dev, int advance, float grad_scale, int dtype, void* stream) {
  MGB_REQUIRE(w && g && m && v && step_dev, MGB_EINVAL, "adamw_step_dev: NULL argument");
  MGB_REQUIRE(numel > 0, MGB_EINVAL, "adamw_step_dev: numel=%lld", (long long)numel);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (advance) {
    mgb::bump_counter_kernel<<<1, 1, 0, st>>>(step_dev);
    int rc = check_launch("bump_counter_kernel");
    if (rc != MGB_OK) return rc;
  }
  MGB_DTYPE_SWITCH(dtype, "adamw_step_dev", {
    const int vec = aligned16(w) && aligned16(g) && aligned16(m) && aligned16(v) && (!master || aligned16(master));
    adamw_kernel<T><<<ew_grid(numel / Vec<T>::N + 1), kEwThreads, 0, st>>>(
        static_cast<T*>(w), static_cast<const T*>(g), m, v, master, numel, lr, beta1, beta2, eps, weight_decay, 1.f, 1.f,
        grad_scale, vec, step_dev);
  })
  return check_launch("adamw_kernel");
}
