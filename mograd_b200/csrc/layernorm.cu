// LayerNorm forward and fused backward (dx, dgamma, dbeta).
//
// Bandwidth-bound design.  A "team" of WPR warps owns one row at a time; each
// lane keeps its CHUNKS 16-byte slices of x and dy in registers, so every
// element of x and dy is read from HBM exactly once and dx written once
// (the reference makes three passes over x and two over dy per row,
// mograd/runtime/gpu/kernels/normalization.mojo:126-170).  Row statistics use
// warp shuffles (plus one shared-memory hop when WPR > 1).  The grid is
// persistent (a multiple of the SM count); every lane accumulates its columns'
// dgamma / dbeta contributions in fp32 registers across all rows its team
// visits, teams are folded inside the CTA, each CTA writes one partial row to
// the workspace and a second small kernel sums the partial rows in a fixed
// order (folding them inside the first launch was measured: whichever CTAs
// finish last have too few loads in flight, 20 -> 42 us at 16384 x 768).
// Both statistics and partials are fp32 (the reference accumulates the
// partials in the I/O dtype, normalization.mojo:114-115).  The row arithmetic
// uses the packed fp32 pair instructions of sm_100 (two lanes per issue
// slot): the kernel is bound by instruction issue, not by DRAM latency.
#include <mutex>

#include "common.cuh"

namespace mgb {
namespace {

constexpr int kMinWarps = 8;
constexpr int kFinCols = 16;   // finalize kernel: columns per block
constexpr int kFinLanes = 16;  // finalize kernel: partial-row lanes per column

template <typename T>
__device__ __forceinline__ void unpack(const uint4& r, float (&v)[Vec<T>::N]) {
  load_vec(reinterpret_cast<const T*>(&r), v);
}
template <typename T>
__device__ __forceinline__ uint4 pack(const float (&v)[Vec<T>::N]) {
  uint4 r;
  store_vec(reinterpret_cast<T*>(&r), v);
  return r;
}

// The same 16 bytes as fp32 pairs (element 2i in .x, 2i+1 in .y), the operand shape of the packed fp32 instructions.
__device__ __forceinline__ void unpack2(const uint4& r, float2 (&v)[4], const __nv_bfloat16*) {
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
}
__device__ __forceinline__ void unpack2(const uint4& r, float2 (&v)[4], const __half*) {
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
}
__device__ __forceinline__ void unpack2(const uint4& r, float2 (&v)[2], const float*) {
  v[0] = make_float2(__uint_as_float(r.x), __uint_as_float(r.y));
  v[1] = make_float2(__uint_as_float(r.z), __uint_as_float(r.w));
}
__device__ __forceinline__ uint4 pack2(const float2 (&v)[4], const __nv_bfloat16*) {
  return make_uint4(pack_bf16x2(v[0].x, v[0].y), pack_bf16x2(v[1].x, v[1].y), pack_bf16x2(v[2].x, v[2].y),
                    pack_bf16x2(v[3].x, v[3].y));
}
__device__ __forceinline__ uint4 pack2(const float2 (&v)[4], const __half*) {
  return make_uint4(pack_f16x2(v[0].x, v[0].y), pack_f16x2(v[1].x, v[1].y), pack_f16x2(v[2].x, v[2].y),
                    pack_f16x2(v[3].x, v[3].y));
}
__device__ __forceinline__ uint4 pack2(const float2 (&v)[2], const float*) {
  return make_uint4(__float_as_uint(v[0].x), __float_as_uint(v[0].y), __float_as_uint(v[1].x), __float_as_uint(v[1].y));
}

// Loads Vec<T>::N elements starting at column `col` of a row; out-of-range
// columns read as zero.
template <typename T, bool VEC>
__device__ __forceinline__ uint4 load_chunk(const T* row, int64_t col, int64_t cols) {
  constexpr int V = Vec<T>::N;
  if (VEC) {
    if (col < cols) return *reinterpret_cast<const uint4*>(row + col);
    return make_uint4(0, 0, 0, 0);
  } else {
    union {
      uint4 u;
      T e[V];
    } t;
    t.u = make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int j = 0; j < V; ++j)
      if (col + j < cols) t.e[j] = row[col + j];
    return t.u;
  }
}

template <typename T, bool VEC>
__device__ __forceinline__ void store_chunk(T* row, int64_t col, int64_t cols, const uint4& r) {
  constexpr int V = Vec<T>::N;
  if (VEC) {
    if (col < cols) *reinterpret_cast<uint4*>(row + col) = r;
  } else {
    const T* e = reinterpret_cast<const T*>(&r);
#pragma unroll
    for (int j = 0; j < V; ++j)
      if (col + j < cols) row[col + j] = e[j];
  }
}

// Sums (a, b) over the team's WPR warps.  `red` holds 2 floats per warp.
template <int WPR>
__device__ __forceinline__ void team_sum2(float& a, float& b, float* red, int warp, int team, int lane) {
  a = warp_sum(a);
  b = warp_sum(b);
  if (WPR > 1) {
    if (lane == 0) {
      red[2 * warp] = a;
      red[2 * warp + 1] = b;
    }
    __syncthreads();
    a = 0.f;
    b = 0.f;
#pragma unroll
    for (int w = 0; w < WPR; ++w) {
      a += red[2 * (team * WPR + w)];
      b += red[2 * (team * WPR + w) + 1];
    }
  }
}

template <int WPR>
struct Shape {
  static constexpr int WARPS = WPR > kMinWarps ? WPR : kMinWarps;
  static constexpr int TEAMS = WARPS / WPR;
  static constexpr int THREADS = WARPS * 32;
  static constexpr int MIN_CTAS = THREADS <= 256 ? 2 : 1;  // register cap: 128 per thread at 256 threads
};

template <typename T, int WPR, int CHUNKS, bool VEC>
__global__ void __launch_bounds__(Shape<WPR>::THREADS, Shape<WPR>::MIN_CTAS)
    ln_fwd_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
                  T* __restrict__ y, float* __restrict__ mean, float* __restrict__ rstd, int64_t rows,
                  int64_t cols, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int V = Vec<T>::N;
  using S = Shape<WPR>;
  __shared__ float redA[2 * S::WARPS];
  __shared__ float redB[2 * S::WARPS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int team = warp / WPR;
  const int lt = (warp % WPR) * 32 + lane;
  const float inv_n = 1.f / static_cast<float>(cols);

  uint4 g_raw[CHUNKS], b_raw[CHUNKS];
#pragma unroll
  for (int j = 0; j < CHUNKS; ++j) {
    const int64_t col = (static_cast<int64_t>(j) * WPR * 32 + lt) * V;
    g_raw[j] = load_chunk<T, VEC>(gamma, col, cols);
    b_raw[j] = load_chunk<T, VEC>(beta, col, cols);
  }

  // the next row of this team is requested before the current one is reduced: one row is always in flight
  const int64_t r_step = static_cast<int64_t>(gridDim.x) * S::TEAMS;
  uint4 x_next[CHUNKS];
  auto fetch = [&](int64_t row) {
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
      const int64_t col = (static_cast<int64_t>(j) * WPR * 32 + lt) * V;
      x_next[j] = row < rows ? load_chunk<T, VEC>(x + row * cols, col, cols) : make_uint4(0, 0, 0, 0);
    }
  };
  fetch(static_cast<int64_t>(blockIdx.x) * S::TEAMS + team);
  for (int64_t r0 = static_cast<int64_t>(blockIdx.x) * S::TEAMS; r0 < rows; r0 += r_step) {
    const int64_t row = r0 + team;
    const bool live = row < rows;
    uint4 x_raw[CHUNKS];
    float sx = 0.f;
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) x_raw[j] = x_next[j];
    fetch(row + r_step);
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
      float v[V];
      unpack<T>(x_raw[j], v);
#pragma unroll
      for (int e = 0; e < V; ++e) sx += v[e];
    }
    float dummy = 0.f;
    team_sum2<WPR>(sx, dummy, redA, warp, team, lane);
    const float mu = sx * inv_n;
    // second moment about the mean; out-of-range columns hold 0 and must not count
    float sq = 0.f;
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
      const int64_t col = (static_cast<int64_t>(j) * WPR * 32 + lt) * V;
      float v[V];
      unpack<T>(x_raw[j], v);
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const float d = (col + e < cols) ? v[e] - mu : 0.f;
        sq = fmaf(d, d, sq);
      }
    }
    dummy = 0.f;
    team_sum2<WPR>(sq, dummy, redB, warp, team, lane);
    const float rs = rsqrtf(sq * inv_n + eps);
    if (live) {
      T* yr = y + row * cols;
#pragma unroll
      for (int j = 0; j < CHUNKS; ++j) {
        const int64_t col = (static_cast<int64_t>(j) * WPR * 32 + lt) * V;
        float v[V], g[V], b[V], o[V];
        unpack<T>(x_raw[j], v);
        unpack<T>(g_raw[j], g);
        unpack<T>(b_raw[j], b);
#pragma unroll
        for (int e = 0; e < V; ++e) o[e] = fmaf((v[e] - mu) * rs, g[e], b[e]);
        store_chunk<T, VEC>(yr, col, cols, pack<T>(o));
      }
      if (lt == 0) {
        if (mean) mean[row] = mu;
        if (rstd) rstd[row] = rs;
      }
    }
  }
}

template <typename T, int WPR, int CHUNKS, bool VEC>
__global__ void __launch_bounds__(Shape<WPR>::THREADS, Shape<WPR>::MIN_CTAS)
    ln_bwd_kernel(const T* dy, const T* __restrict__ x, const T* __restrict__ gamma, const T* resid, T* dx,
                  float* __restrict__ part, int64_t rows, int64_t cols, float eps) {
  constexpr int V = Vec<T>::N;
  using S = Shape<WPR>;
  extern __shared__ float fold[];  // [2][cols]: dgamma then dbeta, folded over the CTA's teams
  __shared__ float redA[2 * S::WARPS];
  __shared__ float redB[2 * S::WARPS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int team = warp / WPR;
  const int lt = (warp % WPR) * 32 + lane;
  const float inv_n = 1.f / static_cast<float>(cols);

  uint4 g_raw[CHUNKS];
  float dg[CHUNKS][V], db[CHUNKS][V];
#pragma unroll
  for (int j = 0; j < CHUNKS; ++j) {
    const int64_t col = (static_cast<int64_t>(j) * WPR * 32 + lt) * V;
    g_raw[j] = load_chunk<T, VEC>(gamma, col, cols);
#pragma unroll
    for (int e = 0; e < V; ++e) {
      dg[j][e] = 0.f;
      db[j][e] = 0.f;
    }
  }

  for (int64_t r0 = static_cast<int64_t>(blockIdx.x) * S::TEAMS; r0 < rows;
       r0 += static_cast<int64_t>(gridDim.x) * S::TEAMS) {
    const int64_t row = r0 + team;
    const bool live = row < rows;
    const T* xr = x + (live ? row : 0) * cols;
    const T* dyr = dy + (live ? row : 0) * cols;
    uint4 x_raw[CHUNKS], dy_raw[CHUNKS];
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
      const int64_t col = (static_cast<int64_t>(j) * WPR * 32 + lt) * V;
      x_raw[j] = live ? load_chunk<T, VEC>(xr, col, cols) : make_uint4(0, 0, 0, 0);
      dy_raw[j] = live ? load_chunk<T, VEC>(dyr, col, cols) : make_uint4(0, 0, 0, 0);
    }
    // mean and E[x^2] (the reference's statistic: var = E[x^2] - mu^2 clamped at 0)
    float sx = 0.f, sx2 = 0.f;
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
      float v[V];
      unpack<T>(x_raw[j], v);
#pragma unroll
      for (int e = 0; e < V; ++e) {
        sx += v[e];
        sx2 = fmaf(v[e], v[e], sx2);
      }
    }
    team_sum2<WPR>(sx, sx2, redA, warp, team, lane);
    const float mu = sx * inv_n;
    const float rs = rsqrtf(fmaxf(sx2 * inv_n - mu * mu, 0.f) + eps);
    // c1 = mean(dy * gamma), c2 = mean(dy * gamma * xhat); padded columns hold dy = 0
    float c1 = 0.f, c2 = 0.f;
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
      float v[V], d[V], g[V];
      unpack<T>(x_raw[j], v);
      unpack<T>(dy_raw[j], d);
      unpack<T>(g_raw[j], g);
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const float dyg = d[e] * g[e];
        c1 += dyg;
        c2 = fmaf(dyg, (v[e] - mu) * rs, c2);
      }
    }
    team_sum2<WPR>(c1, c2, redB, warp, team, lane);
    c1 *= inv_n;
    c2 *= inv_n;
    if (live) {
      T* dxr = dx + row * cols;
#pragma unroll
      for (int j = 0; j < CHUNKS; ++j) {
        const int64_t col = (static_cast<int64_t>(j) * WPR * 32 + lt) * V;
        float v[V], d[V], g[V], o[V];
        unpack<T>(x_raw[j], v);
        unpack<T>(dy_raw[j], d);
        unpack<T>(g_raw[j], g);
#pragma unroll
        for (int e = 0; e < V; ++e) {
          const float xhat = (v[e] - mu) * rs;
          o[e] = rs * (d[e] * g[e] - c1 - xhat * c2);
          dg[j][e] = fmaf(d[e], xhat, dg[j][e]);
          db[j][e] += d[e];
        }
        if (resid) {
          float rv[V];
          unpack<T>(load_chunk<T, VEC>(resid + row * cols, col, cols), rv);
#pragma unroll
          for (int e = 0; e < V; ++e) o[e] += rv[e];
        }
        store_chunk<T, VEC>(dxr, col, cols, pack<T>(o));
      }
    }
  }

  // fold the teams' column partials inside the CTA, one team per round
  for (int t = 0; t < S::TEAMS; ++t) {
    if (team == t) {
#pragma unroll
      for (int j = 0; j < CHUNKS; ++j) {
        const int64_t col = (static_cast<int64_t>(j) * WPR * 32 + lt) * V;
#pragma unroll
        for (int e = 0; e < V; ++e) {
          if (col + e < cols) {
            if (t == 0) {
              fold[col + e] = dg[j][e];
              fold[cols + col + e] = db[j][e];
            } else {
              fold[col + e] += dg[j][e];
              fold[cols + col + e] += db[j][e];
            }
          }
        }
      }
    }
    __syncthreads();
  }
  float* prow = part + static_cast<int64_t>(blockIdx.x) * 2 * cols;
  for (int64_t c = threadIdx.x; c < 2 * cols; c += S::THREADS) prow[c] = fold[c];
}

// ---- pipelined variant for 16-byte-aligned rows --------------------------
// Each warp keeps a ring of kLnStages row slots in shared memory and fills it
// with cp.async (global -> shared without passing through registers), so up
// to kLnStages - 1 rows of x and dy per warp are in flight while the current
// row is being reduced.  A lane only ever reads back the 16-byte chunks it
// copied itself, so the ring needs no barrier.  Registers hold just gamma and
// the fp32 dgamma / dbeta partials.
// Row slots per warp: three for narrow slices; two when a slice is 4 chunks wide, so that two CTAs still fit per SM.
template <int CHUNKS>
struct LnStages {
  static constexpr int N = CHUNKS >= 4 ? 2 : 3;
};

__device__ __forceinline__ void cp_async16(uint32_t saddr, const void* gptr) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(saddr), "l"(gptr) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Sums four values over the team's WPR warps with one block barrier per call;
// `red` holds two parity buffers of 4 floats per warp, alternated by the caller.
template <int WPR>
__device__ __forceinline__ void team_sum4(float (&v)[4], float* red, int parity, int warps, int warp, int team,
                                          int lane) {
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = warp_sum(v[i]);
  if (WPR > 1) {
    float* buf = red + parity * warps * 4;
    if (lane == 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) buf[warp * 4 + i] = v[i];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = 0.f;
#pragma unroll
    for (int w = 0; w < WPR; ++w) {
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] += buf[(team * WPR + w) * 4 + i];
    }
  }
}

// Instruction issue is what bounds this kernel once the loads are asynchronous, so the row is visited twice, not
// three times, and all row arithmetic is done on fp32 pairs (fma.rn.f32x2 and friends: two elements per issue
// slot; a 32-bit word of two bf16 values unpacks straight into one pair).  Pass A forms sum x, sum x^2, sum dy*g
// and sum dy*g*x together; c2 = mean(dy*g*xhat) then follows as rstd*(sum dy*g*x - mu*sum dy*g)/n.  Pass B writes
// dx = dy*g*rstd - rstd*c1 - xhat*rstd*c2 with two FMAs and accumulates dgamma / dbeta.  When a lane's slice is
// small (KEEP) the unpacked x and dy stay in registers between the passes.
// RESID: a residual gradient is added to dx (compiled out otherwise: the wide-row instantiations have no
// registers to spare).  dy may alias dx (a row's dy is in shared memory before its dx is written).
template <typename T, int WPR, int CHUNKS, bool RESID>
__global__ void __launch_bounds__(Shape<WPR>::THREADS, Shape<WPR>::MIN_CTAS)
    ln_bwd_pipe_kernel(const T* dy, const T* __restrict__ x, const T* __restrict__ gamma, const T* resid, T* dx,
                       float* __restrict__ part, int64_t rows, int64_t cols, float eps) {
  constexpr int V = Vec<T>::N;
  constexpr int P = V / 2;  // fp32 pairs per 16-byte chunk
  using S = Shape<WPR>;
  constexpr int SLOT = CHUNKS * 512;  // bytes of one array (x or dy) of one row slot of one warp
  constexpr int kLnStages = LnStages<CHUNKS>::N;
  constexpr bool KEEP = CHUNKS * V <= 16;
  const T* const tag = nullptr;
  extern __shared__ __align__(16) unsigned char dsm[];
  unsigned char* ring_base = dsm;
  __shared__ float red[2 * S::WARPS * 4];
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int team = warp / WPR;
  const int lt = (warp % WPR) * 32 + lane;
  const float inv_n = 1.f / static_cast<float>(cols);
  unsigned char* ring = ring_base + static_cast<size_t>(warp) * kLnStages * 2 * SLOT;
  const uint32_t ring_s = static_cast<uint32_t>(__cvta_generic_to_shared(ring));

  uint4 g_raw[CHUNKS];
  float2 dg[CHUNKS][P], db[CHUNKS][P];
  int64_t colj[CHUNKS];
#pragma unroll
  for (int j = 0; j < CHUNKS; ++j) {
    colj[j] = (static_cast<int64_t>(j) * WPR * 32 + lt) * V;
    g_raw[j] = load_chunk<T, true>(gamma, colj[j], cols);
#pragma unroll
    for (int e = 0; e < P; ++e) {
      dg[j][e] = make_float2(0.f, 0.f);
      db[j][e] = make_float2(0.f, 0.f);
    }
  }

  const int64_t r_first = static_cast<int64_t>(blockIdx.x) * S::TEAMS + team;
  const int64_t r_step = static_cast<int64_t>(gridDim.x) * S::TEAMS;
  auto issue = [&](int64_t row, int slot) {
    if (row < rows) {
#pragma unroll
      for (int j = 0; j < CHUNKS; ++j) {
        if (colj[j] < cols) {
          const uint32_t so = ring_s + slot * 2 * SLOT + (j * 32 + lane) * 16;
          cp_async16(so, x + row * cols + colj[j]);
          cp_async16(so + SLOT, dy + row * cols + colj[j]);
        }
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int s = 0; s < kLnStages - 1; ++s) issue(r_first + s * r_step, s);

  int slot = 0, parity = 0;
  for (int64_t r0 = static_cast<int64_t>(blockIdx.x) * S::TEAMS; r0 < rows; r0 += r_step) {
    const int64_t row = r0 + team;
    const bool live = row < rows;
    issue(row + (kLnStages - 1) * r_step, (slot + kLnStages - 1) % kLnStages);
    cp_async_wait<kLnStages - 1>();
    const uint4* xs = reinterpret_cast<const uint4*>(ring + slot * 2 * SLOT);
    const uint4* ds = reinterpret_cast<const uint4*>(ring + slot * 2 * SLOT + SLOT);
    // the residual gradient of this row is requested now and consumed in the second pass: its latency hides behind
    // the first pass and the row reduction
    constexpr bool EARLY = RESID && CHUNKS <= 3;  // wider rows fetch it where it is used instead
    uint4 r_raw[EARLY ? CHUNKS : 1];
    if (EARLY && live) {
#pragma unroll
      for (int j = 0; j < CHUNKS; ++j)
        if (colj[j] < cols) r_raw[j] = *reinterpret_cast<const uint4*>(resid + row * cols + colj[j]);
    }
    float2 xk[KEEP ? CHUNKS : 1][P], dk[KEEP ? CHUNKS : 1][P];
    float2 s0 = make_float2(0.f, 0.f), s1 = s0, s2 = s0, s3 = s0;  // sum x, sum x^2, sum dy*g, sum dy*g*x
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
      float2 v[P], d[P], g[P];
      const bool in = live && colj[j] < cols;
      unpack2(in ? xs[j * 32 + lane] : make_uint4(0, 0, 0, 0), v, tag);
      unpack2(in ? ds[j * 32 + lane] : make_uint4(0, 0, 0, 0), d, tag);
      unpack2(g_raw[j], g, tag);
#pragma unroll
      for (int e = 0; e < P; ++e) {
        const float2 dyg = __fmul2_rn(d[e], g[e]);
        s0 = __fadd2_rn(s0, v[e]);
        s1 = __ffma2_rn(v[e], v[e], s1);
        s2 = __fadd2_rn(s2, dyg);
        s3 = __ffma2_rn(dyg, v[e], s3);
        if (KEEP) {
          xk[j][e] = v[e];
          dk[j][e] = d[e];
        }
      }
    }
    float sums[4] = {s0.x + s0.y, s1.x + s1.y, s2.x + s2.y, s3.x + s3.y};
    team_sum4<WPR>(sums, red, parity, S::WARPS, warp, team, lane);
    parity ^= 1;
    const float mu = sums[0] * inv_n;
    const float rs = rsqrtf(fmaxf(sums[1] * inv_n - mu * mu, 0.f) + eps);
    const float c1 = sums[2] * inv_n;
    const float c2 = rs * (sums[3] - mu * sums[2]) * inv_n;
    const float2 rs2 = make_float2(rs, rs), nmr2 = make_float2(-mu * rs, -mu * rs);
    const float2 k12 = make_float2(-rs * c1, -rs * c1), k22 = make_float2(-rs * c2, -rs * c2);
    if (live) {
      T* dxr = dx + row * cols;
#pragma unroll
      for (int j = 0; j < CHUNKS; ++j) {
        if (colj[j] < cols) {
          float2 v[P], d[P], g[P], o[P];
          if (KEEP) {
#pragma unroll
            for (int e = 0; e < P; ++e) {
              v[e] = xk[j][e];
              d[e] = dk[j][e];
            }
          } else {
            unpack2(xs[j * 32 + lane], v, tag);
            unpack2(ds[j * 32 + lane], d, tag);
          }
          unpack2(g_raw[j], g, tag);
#pragma unroll
          for (int e = 0; e < P; ++e) {
            const float2 xhat = __ffma2_rn(v[e], rs2, nmr2);
            o[e] = __ffma2_rn(xhat, k22, __ffma2_rn(__fmul2_rn(d[e], g[e]), rs2, k12));
            dg[j][e] = __ffma2_rn(d[e], xhat, dg[j][e]);
            db[j][e] = __fadd2_rn(db[j][e], d[e]);
          }
          if (RESID) {
            float2 rv[P];
            unpack2(EARLY ? r_raw[EARLY ? j : 0] : *reinterpret_cast<const uint4*>(resid + row * cols + colj[j]), rv, tag);
#pragma unroll
            for (int e = 0; e < P; ++e) o[e] = __fadd2_rn(o[e], rv[e]);
          }
          *reinterpret_cast<uint4*>(dxr + colj[j]) = pack2(o, tag);
        }
      }
    }
    slot = (slot + 1) % kLnStages;
  }
  cp_async_wait<0>();
  __syncthreads();  // every warp is done with its ring: the rings become [TEAMS][2][cols] floats

  // Column partials of the CTA: every warp parks its own columns in its team's row with 16-byte stores, then
  // each thread adds up a few columns over the teams in a fixed order and writes them out.  (The ring always
  // has room: it holds at least two rows of x and dy per warp, four bytes of partials replace two or four
  // bytes of input per column.)
  float* stage = reinterpret_cast<float*>(ring_base);
  float* mine = stage + static_cast<size_t>(team) * 2 * cols;
#pragma unroll
  for (int j = 0; j < CHUNKS; ++j) {
    if (colj[j] + V <= cols) {
#pragma unroll
      for (int e = 0; e < P; e += 2) {
        *reinterpret_cast<float4*>(mine + colj[j] + 2 * e) = make_float4(dg[j][e].x, dg[j][e].y, dg[j][e + 1].x, dg[j][e + 1].y);
        *reinterpret_cast<float4*>(mine + cols + colj[j] + 2 * e) = make_float4(db[j][e].x, db[j][e].y, db[j][e + 1].x, db[j][e + 1].y);
      }
    } else {
#pragma unroll
      for (int e = 0; e < P; ++e) {
        if (colj[j] + 2 * e < cols) {
          mine[colj[j] + 2 * e] = dg[j][e].x;
          mine[cols + colj[j] + 2 * e] = db[j][e].x;
        }
        if (colj[j] + 2 * e + 1 < cols) {
          mine[colj[j] + 2 * e + 1] = dg[j][e].y;
          mine[cols + colj[j] + 2 * e + 1] = db[j][e].y;
        }
      }
    }
  }
  __syncthreads();
  float* prow = part + static_cast<int64_t>(blockIdx.x) * 2 * cols;
  for (int64_t c = threadIdx.x; c < 2 * cols; c += S::THREADS) {
    float acc = stage[c];
#pragma unroll
    for (int t = 1; t < S::TEAMS; ++t) acc += stage[static_cast<size_t>(t) * 2 * cols + c];
    prow[c] = acc;
  }
}

// dgamma[c] = sum_p part[p][0][c], dbeta[c] = sum_p part[p][1][c], fixed order.
template <typename T>
__global__ void __launch_bounds__(kFinCols* kFinLanes)
    ln_bwd_finalize_kernel(const float* __restrict__ part, int nparts, int64_t cols, T* __restrict__ dgamma,
                           T* __restrict__ dbeta) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[kFinLanes][kFinCols + 1];
  const int cx = threadIdx.x % kFinCols, ry = threadIdx.x / kFinCols;
  const int64_t c2 = static_cast<int64_t>(blockIdx.x) * kFinCols + cx;  // index into [2*cols]
  float acc = 0.f;
  if (c2 < 2 * cols)
    for (int p = ry; p < nparts; p += kFinLanes) acc += part[static_cast<int64_t>(p) * 2 * cols + c2];
  red[ry][cx] = acc;
  __syncthreads();
  if (ry == 0 && c2 < 2 * cols) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kFinLanes; ++i) s += red[i][cx];
    if (c2 < cols)
      dgamma[c2] = from_f32<T>(s);
    else
      dbeta[c2 - cols] = from_f32<T>(s);
  }
}

// The same sums with 16-byte loads: a block owns 32 consecutive entries of the [2*cols] partial row (8 threads of
// float4) and 32 lanes stride over the partial rows with four loads in flight each; the 32 lane sums of a column are
// then added in lane order, so the result does not depend on timing.  Needs 2*cols % 4 == 0 and a 16-byte aligned
// workspace.
constexpr int kFin4Lanes = 32;
template <typename T>
__global__ void __launch_bounds__(8 * kFin4Lanes)
    ln_bwd_finalize4_kernel(const float* __restrict__ part, int nparts, int64_t cols, T* __restrict__ dgamma,
                            T* __restrict__ dbeta) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[kFin4Lanes][33];
  const int cx = threadIdx.x & 7, ry = threadIdx.x >> 3;
  const int64_t c4 = static_cast<int64_t>(blockIdx.x) * 32 + cx * 4;  // index into [2*cols]
  float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0, a2 = a0, a3 = a0;
  if (c4 < 2 * cols) {
    const float* col = part + c4;
    const int64_t ld = 2 * cols;
    int q = ry;
    for (; q + 3 * kFin4Lanes < nparts; q += 4 * kFin4Lanes) {
      const float4 v0 = *reinterpret_cast<const float4*>(col + static_cast<int64_t>(q) * ld);
      const float4 v1 = *reinterpret_cast<const float4*>(col + static_cast<int64_t>(q + kFin4Lanes) * ld);
      const float4 v2 = *reinterpret_cast<const float4*>(col + static_cast<int64_t>(q + 2 * kFin4Lanes) * ld);
      const float4 v3 = *reinterpret_cast<const float4*>(col + static_cast<int64_t>(q + 3 * kFin4Lanes) * ld);
      a0.x += v0.x, a0.y += v0.y, a0.z += v0.z, a0.w += v0.w;
      a1.x += v1.x, a1.y += v1.y, a1.z += v1.z, a1.w += v1.w;
      a2.x += v2.x, a2.y += v2.y, a2.z += v2.z, a2.w += v2.w;
      a3.x += v3.x, a3.y += v3.y, a3.z += v3.z, a3.w += v3.w;
    }
    for (; q < nparts; q += kFin4Lanes) {
      const float4 v0 = *reinterpret_cast<const float4*>(col + static_cast<int64_t>(q) * ld);
      a0.x += v0.x, a0.y += v0.y, a0.z += v0.z, a0.w += v0.w;
    }
  }
  red[ry][cx * 4 + 0] = (a0.x + a1.x) + (a2.x + a3.x);
  red[ry][cx * 4 + 1] = (a0.y + a1.y) + (a2.y + a3.y);
  red[ry][cx * 4 + 2] = (a0.z + a1.z) + (a2.z + a3.z);
  red[ry][cx * 4 + 3] = (a0.w + a1.w) + (a2.w + a3.w);
  __syncthreads();
  const int64_t c = static_cast<int64_t>(blockIdx.x) * 32 + threadIdx.x;
  if (threadIdx.x < 32 && c < 2 * cols) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < kFin4Lanes; ++i) t += red[i][threadIdx.x];
    if (c < cols)
      dgamma[c] = from_f32<T>(t);
    else
      dbeta[c - cols] = from_f32<T>(t);
  }
}

struct Plan {
  int wpr, chunks, grid;
};

template <typename T>
bool make_plan(int64_t rows, int64_t cols, Plan& pl) {
  constexpr int V = Vec<T>::N;
  int wpr = 1;
  while (wpr <= 32 && static_cast<int64_t>(V) * 32 * wpr * 4 < cols) wpr *= 2;
  if (wpr > 32) return false;
  pl.wpr = wpr;
  pl.chunks = static_cast<int>((cols + static_cast<int64_t>(V) * 32 * wpr - 1) / (static_cast<int64_t>(V) * 32 * wpr));
  const int warps = wpr > kMinWarps ? wpr : kMinWarps;
  const int teams = warps / wpr;
  const int ctas_per_sm = warps >= 32 ? 1 : 2;
  int64_t grid = static_cast<int64_t>(sm_count()) * ctas_per_sm;
  const int64_t need = (rows + teams - 1) / teams;
  if (grid > need) grid = need;
  pl.grid = static_cast<int>(grid);
  return true;
}

template <typename T, int WPR, int CHUNKS>
int launch_fwd(const T* x, const T* g, const T* b, T* y, float* mean, float* rstd, int64_t rows, int64_t cols,
               float eps, bool vec, int grid, cudaStream_t st) {
  constexpr int TH = Shape<WPR>::THREADS;
  if (vec)
    launch_pdl(ln_fwd_kernel<T, WPR, CHUNKS, true>, dim3(grid), dim3(TH), 0, st, x, g, b, y, mean, rstd, rows, cols, eps);
  else
    launch_pdl(ln_fwd_kernel<T, WPR, CHUNKS, false>, dim3(grid), dim3(TH), 0, st, x, g, b, y, mean, rstd, rows, cols, eps);
  return check_launch("ln_fwd_kernel");
}

template <typename T, int WPR, int CHUNKS>
int launch_bwd(const T* dy, const T* x, const T* g, const T* resid, T* dx, float* part, int64_t rows, int64_t cols,
               float eps, bool vec, int grid, cudaStream_t st) {
  constexpr int TH = Shape<WPR>::THREADS;
  const size_t fold_bytes = round_up(static_cast<size_t>(2 * cols) * sizeof(float), 16);
  const size_t pipe_smem = static_cast<size_t>(Shape<WPR>::WARPS) * LnStages<CHUNKS>::N * 2 * CHUNKS * 512;
  if (vec && pipe_smem + 1024 <= static_cast<size_t>(max_smem_optin())) {
    const size_t smem = pipe_smem;
    auto k = resid ? ln_bwd_pipe_kernel<T, WPR, CHUNKS, true> : ln_bwd_pipe_kernel<T, WPR, CHUNKS, false>;
    // static shared memory (reduction buffers) counts against the 48 KB default too: opt in well below it
    if (smem > 40 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    launch_pdl(k, dim3(grid), dim3(TH), smem, st, dy, x, g, resid, dx, part, rows, cols, eps);
    return check_launch("ln_bwd_pipe_kernel");
  }
  if (vec) {  // very wide rows: the ring does not fit next to the fold buffer, keep the row in registers instead
    auto k = ln_bwd_kernel<T, WPR, CHUNKS, true>;
    if (fold_bytes > 40 * 1024)
      cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(fold_bytes));
    k<<<grid, TH, fold_bytes, st>>>(dy, x, g, resid, dx, part, rows, cols, eps);
  } else {
    auto k = ln_bwd_kernel<T, WPR, CHUNKS, false>;
    if (fold_bytes > 40 * 1024)
      cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(fold_bytes));
    k<<<grid, TH, fold_bytes, st>>>(dy, x, g, resid, dx, part, rows, cols, eps);
  }
  return check_launch("ln_bwd_kernel");
}

#define MGB_LN_DISPATCH(FN, ...)                                            \
  switch (pl.wpr * 8 + pl.chunks) {                                         \
    case 1 * 8 + 1: return FN<T, 1, 1>(__VA_ARGS__);                        \
    case 1 * 8 + 2: return FN<T, 1, 2>(__VA_ARGS__);                        \
    case 1 * 8 + 3: return FN<T, 1, 3>(__VA_ARGS__);                        \
    case 1 * 8 + 4: return FN<T, 1, 4>(__VA_ARGS__);                        \
    case 2 * 8 + 3: return FN<T, 2, 3>(__VA_ARGS__);                        \
    case 2 * 8 + 4: return FN<T, 2, 4>(__VA_ARGS__);                        \
    case 4 * 8 + 3: return FN<T, 4, 3>(__VA_ARGS__);                        \
    case 4 * 8 + 4: return FN<T, 4, 4>(__VA_ARGS__);                        \
    case 8 * 8 + 3: return FN<T, 8, 3>(__VA_ARGS__);                        \
    case 8 * 8 + 4: return FN<T, 8, 4>(__VA_ARGS__);                        \
    case 16 * 8 + 3: return FN<T, 16, 3>(__VA_ARGS__);                      \
    case 16 * 8 + 4: return FN<T, 16, 4>(__VA_ARGS__);                      \
    case 32 * 8 + 3: return FN<T, 32, 3>(__VA_ARGS__);                      \
    case 32 * 8 + 4: return FN<T, 32, 4>(__VA_ARGS__);                      \
    default: return fail(MGB_EUNSUPPORTED, "layer_norm: no kernel for wpr=%d chunks=%d", pl.wpr, pl.chunks); \
  }

template <typename T>
int ln_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd, int64_t rows,
           int64_t cols, float eps, cudaStream_t st) {
  Plan pl;
  if (!make_plan<T>(rows, cols, pl))
    return fail(MGB_EUNSUPPORTED, "layer_norm_fwd: cols=%lld exceeds 16384", (long long)cols);
  const bool vec = (cols % Vec<T>::N == 0) && aligned16(x) && aligned16(gamma) && aligned16(beta) && aligned16(y);
  MGB_LN_DISPATCH(launch_fwd, static_cast<const T*>(x), static_cast<const T*>(gamma), static_cast<const T*>(beta),
                  static_cast<T*>(y), mean, rstd, rows, cols, eps, vec, pl.grid, st)
}

template <typename T>
int ln_bwd_main(const void* dy, const void* x, const void* gamma, const void* resid, void* dx, float* part,
                int64_t rows, int64_t cols, float eps, const Plan& pl, cudaStream_t st) {
  const bool vec = (cols % Vec<T>::N == 0) && aligned16(x) && aligned16(gamma) && aligned16(dy) && aligned16(dx) &&
                   aligned16(resid);
  MGB_LN_DISPATCH(launch_bwd, static_cast<const T*>(dy), static_cast<const T*>(x), static_cast<const T*>(gamma),
                  static_cast<const T*>(resid), static_cast<T*>(dx), part, rows, cols, eps, vec, pl.grid, st)
}

template <typename T>
int ln_bwd_finalize(const float* part, int nparts, int64_t cols, void* dgamma, void* dbeta, cudaStream_t st) {
  if (cols % 2 == 0 && aligned16(part)) {
    const unsigned fgrid = static_cast<unsigned>((2 * cols + 31) / 32);
    launch_pdl(ln_bwd_finalize4_kernel<T>, dim3(fgrid), dim3(8 * kFin4Lanes), 0, st, part, nparts, cols,
               static_cast<T*>(dgamma), static_cast<T*>(dbeta));
    return check_launch("ln_bwd_finalize4_kernel");
  }
  const unsigned fgrid = static_cast<unsigned>((2 * cols + kFinCols - 1) / kFinCols);
  launch_pdl(ln_bwd_finalize_kernel<T>, dim3(fgrid), dim3(kFinCols * kFinLanes), 0, st, part, nparts, cols,
             static_cast<T*>(dgamma), static_cast<T*>(dbeta));
  return check_launch("ln_bwd_finalize_kernel");
}

template <typename T>
int ln_bwd(const void* dy, const void* x, const void* gamma, const void* resid, void* dx, void* dgamma, void* dbeta,
           int64_t rows, int64_t cols, float eps, void* ws, size_t ws_bytes, cudaStream_t st) {
  Plan pl;
  if (!make_plan<T>(rows, cols, pl))
    return fail(MGB_EUNSUPPORTED, "layer_norm_bwd: cols=%lld exceeds 16384", (long long)cols);
  const size_t need = static_cast<size_t>(pl.grid) * 2 * cols * sizeof(float);
  MGB_REQUIRE(ws && ws_bytes >= need, MGB_EWORKSPACE, "layer_norm_bwd: workspace of %zu bytes needed, %zu given", need,
              ws ? ws_bytes : (size_t)0);
  float* part = static_cast<float*>(ws);
  int rc = ln_bwd_main<T>(dy, x, gamma, resid, dx, part, rows, cols, eps, pl, st);
  if (rc != MGB_OK) return rc;
  return ln_bwd_finalize<T>(part, pl.grid, cols, dgamma, dbeta, st);
}

// Scratch for mograd_b200_layer_norm_bwd_static: room for the per-CTA dgamma /
// dbeta partial rows of a launch of up to 296 CTAs at cols <= 4096
// (296 * 2 * 4096 floats, 9.25 MiB).  It lives in every CUDA context that loads
// this library, from load until the process exits.
constexpr size_t kStaticScratchFloats = static_cast<size_t>(296) * 2 * 4096;
static __device__ __align__(256) float g_ln_bwd_static_scratch[kStaticScratchFloats];

// Device address of the array on the current device.  The array's name is only
// a host-side handle here, so it is resolved once per device through the
// runtime and cached; the resolved pointer is what the kernels receive.
int static_scratch_ptr(float** out) {
  constexpr int kDevs = 64;
  struct Slot {
    std::once_flag once;
    float* ptr = nullptr;
    cudaError_t err = cudaSuccess;
  };
  static Slot slots[kDevs];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(MGB_ECUDA, "layer_norm_bwd_static: cudaGetDevice: %s", cudaGetErrorString(e));
  MGB_REQUIRE(dev >= 0 && dev < kDevs, MGB_EUNSUPPORTED, "layer_norm_bwd_static: device ordinal %d out of range", dev);
  Slot& sl = slots[dev];
  std::call_once(sl.once, [&] {  // once per device, with that device current; safe when two host threads call first
    float* p = nullptr;
    sl.err = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_ln_bwd_static_scratch);
    sl.ptr = p;
  });
  if (sl.err != cudaSuccess || !sl.ptr)
    return fail(MGB_ECUDA, "layer_norm_bwd_static: cudaGetSymbolAddress: %s", cudaGetErrorString(sl.err));
  *out = sl.ptr;
  return MGB_OK;
}

int check_ln(const char* who, int64_t rows, int64_t cols) {
  MGB_REQUIRE(rows > 0 && cols > 0, MGB_EINVAL, "%s: rows=%lld cols=%lld must be positive", who, (long long)rows,
              (long long)cols);
  MGB_REQUIRE(cols <= 16384, MGB_EUNSUPPORTED, "%s: cols=%lld exceeds 16384", who, (long long)cols);
  return MGB_OK;
}

}  // namespace
}  // namespace mgb

using namespace mgb;

MGB_EXPORT int mograd_b200_layer_norm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean,
                                          float* rstd, int64_t rows, int64_t cols, float eps, int dtype,
                                          void* stream) {
  MGB_REQUIRE(x && gamma && beta && y, MGB_EINVAL, "layer_norm_fwd: NULL argument");
  int rc = check_ln("layer_norm_fwd", rows, cols);
  if (rc != MGB_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case MGB_BF16:
      return ln_fwd<__nv_bfloat16>(x, gamma, beta, y, mean, rstd, rows, cols, eps, st);
    case MGB_F32:
      return ln_fwd<float>(x, gamma, beta, y, mean, rstd, rows, cols, eps, st);
    case MGB_F16:
      return ln_fwd<__half>(x, gamma, beta, y, mean, rstd, rows, cols, eps, st);
    default:
      return fail(MGB_EDTYPE, "layer_norm_fwd: unsupported dtype code %d", dtype);
  }
}

MGB_EXPORT size_t mograd_b200_layer_norm_bwd_workspace_bytes(int64_t rows, int64_t cols, int dtype) {
  if (rows <= 0 || cols <= 0 || cols > 16384) return 0;
  Plan pl;
  const bool ok = dtype == MGB_F32 ? make_plan<float>(rows, cols, pl) : make_plan<__nv_bfloat16>(rows, cols, pl);
  if (!ok) return 0;
  return round_up(static_cast<size_t>(pl.grid) * 2 * cols * sizeof(float), 256);
}

MGB_EXPORT int mograd_b200_layer_norm_bwd_ex(const void* dy, const void* x, const void* gamma,
                                             const void* dx_residual, void* dx, void* dgamma, void* dbeta,
                                             int64_t rows, int64_t cols, float eps, int dtype, void* workspace,
                                             size_t workspace_bytes, void* stream);

MGB_EXPORT int mograd_b200_layer_norm_bwd(const void* dy, const void* x, const void* gamma, void* dx, void* dgamma,
                                          void* dbeta, int64_t rows, int64_t cols, float eps, int dtype,
                                          void* workspace, size_t workspace_bytes, void* stream) {
  return mograd_b200_layer_norm_bwd_ex(dy, x, gamma, nullptr, dx, dgamma, dbeta, rows, cols, eps, dtype, workspace,
                                       workspace_bytes, stream);
}

MGB_EXPORT int mograd_b200_layer_norm_bwd_ex(const void* dy, const void* x, const void* gamma,
                                             const void* dx_residual, void* dx, void* dgamma, void* dbeta,
                                             int64_t rows, int64_t cols, float eps, int dtype, void* workspace,
                                             size_t workspace_bytes, void* stream) {
  const void* resid = dx_residual;
  MGB_REQUIRE(dy && x && gamma && dx && dgamma && dbeta, MGB_EINVAL, "layer_norm_bwd: NULL argument");
  int rc = check_ln("layer_norm_bwd", rows, cols);
  if (rc != MGB_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case MGB_BF16:
      return ln_bwd<__nv_bfloat16>(dy, x, gamma, resid, dx, dgamma, dbeta, rows, cols, eps, workspace, workspace_bytes,
                                   st);
    case MGB_F32:
      return ln_bwd<float>(dy, x, gamma, resid, dx, dgamma, dbeta, rows, cols, eps, workspace, workspace_bytes, st);
    case MGB_F16:
      return ln_bwd<__half>(dy, x, gamma, resid, dx, dgamma, dbeta, rows, cols, eps, workspace, workspace_bytes, st);
    default:
      return fail(MGB_EDTYPE, "layer_norm_bwd: unsupported dtype code %d", dtype);
  }
}

// Same computation and kernels as mograd_b200_layer_norm_bwd, for callers that
// have no allocator to take a workspace from: the partial rows go to the
// library's own statically allocated device array instead.
MGB_EXPORT int mograd_b200_layer_norm_bwd_static(const void* dy, const void* x, const void* gamma, void* dx,
                                                 void* dgamma, void* dbeta, int64_t rows, int64_t cols, float eps,
                                                 int dtype, void* stream) {
  MGB_REQUIRE(dy && x && gamma && dx && dgamma && dbeta, MGB_EINVAL, "layer_norm_bwd_static: NULL argument");
  int rc = check_ln("layer_norm_bwd_static", rows, cols);
  if (rc != MGB_OK) return rc;
  MGB_REQUIRE(dtype == MGB_BF16 || dtype == MGB_F32 || dtype == MGB_F16, MGB_EDTYPE,
              "layer_norm_bwd_static: unsupported dtype code %d", dtype);
  const size_t need = mograd_b200_layer_norm_bwd_workspace_bytes(rows, cols, dtype);
  const size_t have = kStaticScratchFloats * sizeof(float);
  MGB_REQUIRE(need > 0 && need <= have, MGB_EUNSUPPORTED,
              "layer_norm_bwd_static: rows=%lld cols=%lld needs %zu bytes of scratch, the built-in array holds %zu "
              "(cols <= 4096 always fits); use layer_norm_bwd with a caller workspace",
              (long long)rows, (long long)cols, need, have);
  float* scratch = nullptr;
  rc = static_scratch_ptr(&scratch);
  if (rc != MGB_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == MGB_BF16)
    return ln_bwd<__nv_bfloat16>(dy, x, gamma, nullptr, dx, dgamma, dbeta, rows, cols, eps, scratch, have, st);
  if (dtype == MGB_F16)
    return ln_bwd<__half>(dy, x, gamma, nullptr, dx, dgamma, dbeta, rows, cols, eps, scratch, have, st);
  return ln_bwd<float>(dy, x, gamma, nullptr, dx, dgamma, dbeta, rows, cols, eps, scratch, have, st);
}
