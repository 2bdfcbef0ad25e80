// Flash-attention forward and backward on the tcgen05 tensor cores
// (bf16 or fp16 storage, a template parameter that only selects the operand
// format of the MMAs and the packing of P, dS and the outputs; fp32
// accumulation in TMEM, D = 64 or 128, causal or full).  Pointers to 16-bit
// tensors are typed bf16* throughout: they are only used for addressing.
//
// Tiles are 128 query rows x 128 key rows.  Q / K / V / dO tiles are brought
// in by TMA as [128 rows][D] bf16 with the 128-byte swizzle (one 16 KB box per
// 64 columns); the same shared-memory tile serves as a K-major operand
// (contraction over D) and as an MN-major operand (contraction over rows), so
// nothing is transposed.  The TMEM accumulator puts score row r in lane r, so
// the thread that owns lane r sees a whole row: softmax statistics need no
// shuffles.
//
// Backward, per CTA = one key tile j of one (batch, head), looping over query
// tiles i (i >= j when causal; tiles above the diagonal are skipped):
//     S  = Q_i K_j^T          dP = dO_i V_j^T              (tensor cores -> TMEM)
//     P  = exp2(S*scale*log2e - lse*log2e),  dS' = P*(dP - delta)
//                                                          (16 warps, TMEM -> bf16 in shared)
//     dV += P^T dO_i          dK' += dS'^T Q_i             (accumulate in TMEM over i)
//     dQ'_i partial = dS' K_j -> staged in shared memory, added into the fp32 dQ
//                                accumulator by one TMA tensor reduce per tile
// The softmax scale is left out of dS' and applied once: to dK when it leaves
// TMEM, to dQ when the last kernel converts the accumulator to bf16.
// dK / dV leave TMEM once per CTA.
// TMEM columns: S 128 | dP 128 | dV D | dK D, then dQ: its own D columns for
// D = 64 (drained one tile late, behind the next tile's MMAs); for D = 128 the
// 512 columns are full, so dQ is accumulated over the dP columns once dP is read.
//
// Forward: a softmax thread owns one query row (all 128 scores of a tile in registers: one TMEM read, no exchange
// of row maxima); P goes to shared memory as bf16, O += P V_j accumulates in TMEM and is rescaled in place only
// when the row maximum has grown by more than 2^8.  D = 128: one CTA owns two adjacent query tiles and walks the
// key tiles once for both (the tensor pipe works for one tile while the other is in its exp phase); D = 64: small
// six-warp CTAs, two per SM, run out of phase.
#include <math.h>

#include "attn.cuh"
#include "common.cuh"
#include "sm100.cuh"

namespace mgb {
namespace attn {
namespace {

using namespace sm100;
using bf16 = __nv_bfloat16;

constexpr float kLog2e = 1.4426950408889634f;
constexpr int kHalfBytes = 128 * 128;  // [128 rows][64 bf16] box
constexpr int kPsBytes = 128 * 128 * 2;

enum : int { kErrBwdTma = 201, kErrBwdMma = 202, kErrBwdCompute = 203, kErrFwdTma = 211, kErrFwdMma = 212, kErrFwdSoftmax = 213 };

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Descriptors are built once per tile; the slice for contraction step k is the base plus a constant in the
// 16-byte-granular start-address field (the field cannot carry: shared addresses stay below 256 KB).
// K-major slice k (16 contraction elements) of a [128][cols] swizzled tile.
__device__ __forceinline__ uint64_t base_k(uint32_t tile) { return smem_desc_sw128(tile, 16, 1024); }
__device__ __forceinline__ uint64_t desc_k(uint64_t base, int k) {
  return base + static_cast<uint64_t>(((k >> 2) * kHalfBytes + (k & 3) * 32) >> 4);
}
// MN-major slice k (16 contraction rows) of a [128 rows][cols] swizzled tile.
__device__ __forceinline__ uint64_t base_mn(uint32_t tile) { return smem_desc_sw128(tile, kHalfBytes, 1024); }
__device__ __forceinline__ uint64_t desc_mn(uint64_t base, int k) {
  return base + static_cast<uint64_t>((k * 2048) >> 4);
}
// Byte offset of the 16-byte chunk holding columns [c8*8, c8*8+8) of row r in a [128][128] bf16 swizzled tile.
__device__ __forceinline__ uint32_t ps_chunk_off(int r, int c8) {
  return (c8 >> 3) * kHalfBytes + r * 128 + (((c8 & 7) ^ (r & 7)) << 4);
}

struct AttnParams {
  const float* lse;
  const float* delta;
  float* dq_acc;
  bf16* dk;
  bf16* dv;
  bf16* out;
  float* lse_out;
  int B, S, H;
  float scale;
  int causal;
  int64_t ld_dqkv;  // elements between consecutive tokens of dK / dV
  int o_bshd;       // layout of O (forward output)
  const bf16* bias;  // additive mask (B, H, S, S) in the storage type, or nullptr
  float inv_scale;   // 1 / scale: the mask is folded into the raw scores as bias / scale
  int bias_vec;      // mask rows take 16-byte loads (S a multiple of 8, aligned base)
  int* status;
};

// Additive mask: v[e] += bias[row][col0 + e] / scale for the N raw scores (Q K^T, before the softmax scale) of one
// query row held by this thread, so that everything downstream (scale, running maximum, exponentials) stays as in
// the unmasked kernels.  bias_row points at the first element of this thread's row of the (B, H, S, S) mask.
template <typename T, int N>
__device__ __forceinline__ void add_bias_row(uint32_t (&v)[N], const bf16* bias_row, int col0, int S, bool row_ok,
                                             float inv_scale, int vec) {
  if (!row_ok) return;
  if (vec) {
#pragma unroll
    for (int e = 0; e < N; e += 8) {
      if (col0 + e < S) {  // S is a multiple of 8 here: the whole chunk is inside the row
        float b[8];
        load_vec(reinterpret_cast<const T*>(bias_row + col0 + e), b);
#pragma unroll
        for (int u = 0; u < 8; ++u) v[e + u] = __float_as_uint(fmaf(b[u], inv_scale, __uint_as_float(v[e + u])));
      }
    }
  } else {
#pragma unroll
    for (int e = 0; e < N; ++e)
      if (col0 + e < S)
        v[e] = __float_as_uint(fmaf(to_f32(*reinterpret_cast<const T*>(bias_row + col0 + e)), inv_scale, __uint_as_float(v[e])));
  }
}

// ============================================================== backward
// Schedule of one CTA (key tile j), steady state of query tile i:
//   tensor cores : dP_i | S_{i+1} (as soon as S_i, dP_i sit in registers) | dV_i, dK_i, dQ_i
//   16 warps     : S_i, dP_i -> registers | exp / dS math -> P, dS in shared | dQ_i -> registers -> reductions
//   TMA          : Q two tiles ahead (two slots), dO one tile ahead (D = 64: two slots; D = 128: one)
// dQ_i is written over the dP columns, which are free once dP_i is in registers; the next dP waits for the
// 16 warps to have read dQ_i out of TMEM (the reductions themselves are issued afterwards and do not block).
template <int D>
struct BwdCfg {
  static constexpr int HALVES = D / 64;
  static constexpr int TILE_BYTES = 128 * D * 2;
  static constexpr int QST = 2;
  static constexpr int DOST = (D == 64) ? 2 : 1;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = TILE_BYTES;
  static constexpr int OFF_Q = 2 * TILE_BYTES;
  static constexpr int OFF_DO = OFF_Q + QST * TILE_BYTES;
  static constexpr int OFF_P = OFF_DO + DOST * TILE_BYTES;
  static constexpr int OFF_DS = OFF_P + kPsBytes;
  // D = 64 leaves room in TMEM and shared memory: dQ gets its own columns and its own fp32 staging tile, so the
  // next tile's dP can start early and the dQ drain runs one tile behind the exp phase (LATE).  D = 128 fills
  // TMEM: dQ overwrites the dP columns, is staged in the P | dS tiles and drained right away.
  static constexpr bool LATE = (D == 64);
  static constexpr int STG_BYTES = LATE ? 128 * D * 4 : 0;
  static constexpr int OFF_STG = LATE ? OFF_DS + kPsBytes : OFF_P;
  static constexpr int OFF_BAR = OFF_DS + kPsBytes + STG_BYTES;
  static constexpr int SMEM = OFF_BAR + 256 + 1024;
  static constexpr int COL_S = 0, COL_DP = 128, COL_DV = 256, COL_DK = 256 + D;
  static constexpr int COL_DQ = LATE ? 384 : COL_DP;
  // D = 64 also has 64 columns left for dS as a bf16 TMEM operand: dQ = dS K then reads its A operand from TMEM
  // instead of shared memory (one operand stream less on the shared-memory port)
  static constexpr bool DS_TMEM = LATE;
  static constexpr int COL_DSA = 448;
  static constexpr int TMEM_COLS = 512;
  static constexpr int THREADS = 608;  // TMA warp, MMA warp, 16 compute warps, dQ reduction warp
};

template <int D, typename T, bool BIAS>
__global__ void __launch_bounds__(BwdCfg<D>::THREADS, 1)
    attn_bwd_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                       const __grid_constant__ CUtensorMap tm_dq, const __grid_constant__ CUtensorMap tm_dk,
                       const __grid_constant__ CUtensorMap tm_dv, const AttnParams p) {
  using C = BwdCfg<D>;
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  unsigned char* gen = smem_dyn + (base - smem_u32(smem_dyn));
  const uint32_t bar = base + C::OFF_BAR;
  const uint32_t bar_kv = bar, bar_sdp = bar + 8, bar_sfree = bar + 16, bar_pds = bar + 24, bar_dqf = bar + 32,
                 bar_dqd = bar + 40;
  auto bar_qf = [&](int s) { return bar + 48 + 8u * s; };
  auto bar_qe = [&](int s) { return bar + 64 + 8u * s; };
  auto bar_dof = [&](int s) { return bar + 80 + 8u * s; };
  auto bar_doe = [&](int s) { return bar + 96 + 8u * s; };
  const uint32_t bar_stg = bar + 112;   // dQ staging area (the P | dS tiles) has been read by the TMA unit
  const uint32_t bar_stgf = bar + 120;  // dQ staging area holds this tile's fp32 dQ
  const uint32_t tmem_slot = bar + 128;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(gen + C::OFF_BAR + 128);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // D = 128: (batch, head) runs fastest in launch order, the key tile slowest: with a causal mask the CTAs of key
  // tile 0 (the most query tiles) all start first and the single-tile CTAs last, so the grid ends on short CTAs
  // (3% at B4 H16 S4096).  D = 64 keeps the key tile fastest: there the same order measured 1-2% slower.
  const int j = (D == 128) ? blockIdx.y : blockIdx.x;  // key tile
  const int bh = (D == 128) ? blockIdx.x : blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int nq = (p.S + 127) / 128;
  const int i0 = p.causal ? j : 0;
  const int iters = nq - i0;

  if (threadIdx.x == 0) {
    mbar_init(bar_kv, 1);
    mbar_init(bar_sdp, 1);
    mbar_init(bar_sfree, 16);
    mbar_init(bar_pds, 16);
    mbar_init(bar_dqf, 1);
    mbar_init(bar_dqd, 16);
    mbar_init(bar_stg, 1);
    mbar_init(bar_stgf, 16);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_qf(s), 1);
      mbar_init(bar_qe(s), 1);
      mbar_init(bar_dof(s), 1);
      mbar_init(bar_doe(s), 1);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_gen;
  pdl_launch_dependents();  // after the TMEM allocation: a successor takes the columns over only once they are freed
  pdl_wait();

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      tma_prefetch_desc(&tm_do);
      tma_prefetch_desc(&tm_dq);
      mbar_expect_tx(bar_kv, 2 * C::TILE_BYTES);
#pragma unroll
      for (int c = 0; c < C::HALVES; ++c) {
        tma_load_4d(base + C::OFF_K + c * kHalfBytes, &tm_k, bar_kv, c * 64, h, j * 128, b);
        tma_load_4d(base + C::OFF_V + c * kHalfBytes, &tm_v, bar_kv, c * 64, h, j * 128, b);
      }
      bool ok = true;
      auto load_q = [&](int it) {
        const int s = it % C::QST;
        if (!mbar_wait(bar_qe(s), ((it / C::QST) & 1u) ^ 1u)) return false;
        mbar_expect_tx(bar_qf(s), C::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < C::HALVES; ++c)
          tma_load_4d(base + C::OFF_Q + s * C::TILE_BYTES + c * kHalfBytes, &tm_q, bar_qf(s), c * 64, h,
                      (i0 + it) * 128, b);
        return true;
      };
      auto load_do = [&](int it) {
        const int s = it % C::DOST;
        if (!mbar_wait(bar_doe(s), ((it / C::DOST) & 1u) ^ 1u)) return false;
        mbar_expect_tx(bar_dof(s), C::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < C::HALVES; ++c) {
          const uint32_t dst = base + C::OFF_DO + s * C::TILE_BYTES + c * kHalfBytes;
          if (p.o_bshd)
            tma_load_4d(dst, &tm_do, bar_dof(s), c * 64, h, (i0 + it) * 128, b);
          else
            tma_load_3d(dst, &tm_do, bar_dof(s), c * 64, (i0 + it) * 128, bh);
        }
        return true;
      };
      ok = load_q(0) && load_do(0);
      for (int it = 0; it < iters && ok; ++it) {
        if (it + 1 < iters) ok = load_q(it + 1);
        if (ok && it + 1 < iters) ok = load_do(it + 1);
      }
      if (!ok) atomicExch(p.status, kErrBwdTma);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA
    if (lane == 0) {
      constexpr uint32_t id_ss = umma_idesc_16<T>(128, 128, 0, 0);
      constexpr uint32_t id_mm = umma_idesc_16<T>(128, D, 1, 1);
      constexpr uint32_t id_km = umma_idesc_16<T>(128, D, 0, 1);
      const uint32_t sK = base + C::OFF_K, sV = base + C::OFF_V, sP = base + C::OFF_P, sDS = base + C::OFF_DS;
      auto q_tile = [&](int it) { return base + C::OFF_Q + (it % C::QST) * C::TILE_BYTES; };
      auto do_tile = [&](int it) { return base + C::OFF_DO + (it % C::DOST) * C::TILE_BYTES; };
      const uint64_t dK_k = base_k(sK), dK_mn = base_mn(sK), dV_k = base_k(sV);
      const uint64_t dP_mn = base_mn(sP), dDS_mn = base_mn(sDS), dDS_k = base_k(sDS);
      auto issue_s = [&](int it) {
        const uint64_t dQ_k = base_k(q_tile(it));
#pragma unroll
        for (int k = 0; k < D / 16; ++k) umma_ss(tmem + C::COL_S, desc_k(dQ_k, k), desc_k(dK_k, k), id_ss, k > 0);
      };
      auto issue_dp = [&](int it) {
        const uint64_t dDO_k = base_k(do_tile(it));
#pragma unroll
        for (int k = 0; k < D / 16; ++k) umma_ss(tmem + C::COL_DP, desc_k(dDO_k, k), desc_k(dV_k, k), id_ss, k > 0);
      };
      auto issue_grads = [&](int it) {  // dV, dK (accumulating over tiles) and this tile's dQ
        const uint64_t dQ_mn = base_mn(q_tile(it)), dDO_mn = base_mn(do_tile(it));
        const uint32_t acc = it > 0 ? 1u : 0u;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ss(tmem + C::COL_DV, desc_mn(dP_mn, k), desc_mn(dDO_mn, k), id_mm, k > 0 ? 1u : acc);
        umma_commit(bar_doe(it % C::DOST));
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ss(tmem + C::COL_DK, desc_mn(dDS_mn, k), desc_mn(dQ_mn, k), id_mm, k > 0 ? 1u : acc);
        umma_commit(bar_qe(it % C::QST));
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          if (C::DS_TMEM)
            umma_ts(tmem + C::COL_DQ, tmem + C::COL_DSA + k * 8, desc_mn(dK_mn, k), id_km, k > 0);
          else
            umma_ss(tmem + C::COL_DQ, desc_k(dDS_k, k), desc_mn(dK_mn, k), id_km, k > 0);
        }
        umma_commit(bar_dqf);
      };
      auto wait_q = [&](int it) { return mbar_wait(bar_qf(it % C::QST), (it / C::QST) & 1u); };
      auto wait_do = [&](int it) { return mbar_wait(bar_dof(it % C::DOST), (it / C::DOST) & 1u); };
      bool ok = iters > 0 && mbar_wait(bar_kv, 0) && wait_q(0);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      if (C::LATE) {
        if (ok && (ok = wait_do(0))) {
          tc_fence_after();
          issue_dp(0);
          umma_commit(bar_sdp);
        }
        for (int it = 0; it < iters && ok; ++it) {
          ok = mbar_wait(bar_sfree, it & 1u);  // S_it, dP_it are in registers
          if (ok && it + 1 < iters) {
            ok = wait_q(it + 1) && wait_do(it + 1);
            if (!ok) break;
            tc_fence_after();
            issue_s(it + 1);
            issue_dp(it + 1);
            umma_commit(bar_sdp);
          }
          ok = ok && mbar_wait(bar_pds, it & 1u);
          if (ok && it > 0) ok = mbar_wait(bar_dqd, (it - 1) & 1u);  // dQ_{it-1} has left its columns
          if (!ok) break;
          tc_fence_after();
          issue_grads(it);
        }
      } else {
        for (int it = 0; it < iters && ok; ++it) {
          ok = wait_do(it);
          if (ok && it > 0) ok = mbar_wait(bar_dqd, (it - 1) & 1u);  // dQ_{it-1} has left the dP columns
          if (!ok) break;
          tc_fence_after();
          issue_dp(it);
          umma_commit(bar_sdp);  // also covers S_it, issued one iteration earlier
          if (!mbar_wait(bar_sfree, it & 1u)) {
            ok = false;
            break;
          }
          if (it + 1 < iters) {
            if (!wait_q(it + 1)) {
              ok = false;
              break;
            }
            tc_fence_after();
            issue_s(it + 1);  // runs while the 16 warps work on tile it
          }
          if (!mbar_wait(bar_pds, it & 1u)) {
            ok = false;
            break;
          }
          tc_fence_after();
          issue_grads(it);
        }
      }
      if (!ok && iters > 0) atomicExch(p.status, kErrBwdMma);
    }
    __syncwarp();
  } else if (warp == 18) {
    // ------------------------------------------------- dQ reduction (TMA)
    if (lane == 0) {
      for (int it = 0; it < iters; ++it) {
        if (!mbar_wait(bar_stgf, it & 1u)) {
          atomicExch(p.status, kErrBwdCompute);
          break;
        }
#pragma unroll
        for (int c = 0; c < D / 32; ++c)
          tma_reduce_add_4d(&tm_dq, base + C::OFF_STG + c * kHalfBytes, c * 32, h, (i0 + it) * 128, b);
        bulk_commit();
        bulk_wait_read0();
        mbar_arrive(bar_stg);
      }
      // every reduction has been read out of shared memory (wait_group.read above); the adds themselves complete
      // before the grid does, which is what the kernel after this one waits for
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ compute
    // 16 warps: TMEM lane quarter = warp % 4 (hardware rule), column group cg = 32 of the 128 S / dP columns.
    // The softmax scale is left out of dS here and applied once to dK (epilogue) and dQ (final cast).
    const int cw = warp - 2;
    const int quarter = warp & 3;
    const int cg = cw >> 2;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const float scale_log2 = p.scale * kLog2e;
    constexpr int DC = D / 4;  // dQ / dK / dV columns per warp
    bool ok = true;
    // dQ of tile t: TMEM -> registers (frees the columns) -> fp32 staging tile in shared memory as
    // [128 rows][32 floats] boxes with the 128-byte swizzle -> the reduction warp lets the TMA unit add it into
    // the accumulator (whole 128-byte lines per request; rows past S are clipped by the tensor map).
    auto drain = [&](int t, bool wait_ready) -> bool {
      if (wait_ready && !mbar_wait(bar_dqf, t & 1u)) return false;  // never wait twice on one phase
      tc_fence_after();
      uint32_t v[DC];
      if constexpr (DC == 32) {
        tmem_ld32(tmem + lane_base + C::COL_DQ + cg * DC, v);
      } else {
        tmem_ld16(tmem + lane_base + C::COL_DQ + cg * DC, v);
      }
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_dqd);
      if (C::LATE && t > 0 && !mbar_wait(bar_stg, (t - 1) & 1u)) return false;  // staging tile read by the TMA unit
      constexpr int CH = DC / 4;             // 16-byte chunks this thread owns
      const int box = (cg * DC) / 32;        // which [128][32] box
      const int ch0 = ((cg * DC) % 32) / 4;  // first chunk inside the 128-byte row
      unsigned char* stg = gen + C::OFF_STG + box * kHalfBytes + r * 128;
#pragma unroll
      for (int t4 = 0; t4 < CH; ++t4)
        *reinterpret_cast<uint4*>(stg + (((ch0 + t4) ^ (r & 7)) << 4)) =
            make_uint4(v[4 * t4], v[4 * t4 + 1], v[4 * t4 + 2], v[4 * t4 + 3]);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_stgf);
      return true;
    };
    for (int it = 0; it < iters && ok; ++it) {
      const int i = i0 + it;
      const int qrow = i * 128 + r;
      const bool vq = qrow < p.S;
      const float lse2 = vq ? p.lse[static_cast<int64_t>(bh) * p.S + qrow] * kLog2e : 0.f;
      const float dlt = vq ? p.delta[static_cast<int64_t>(bh) * p.S + qrow] : 0.f;
      if (!mbar_wait(bar_sdp, it & 1u)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const bool diag = p.causal && (i == j);
      const bool masked = diag || (j * 128 + 128 > p.S) || (i * 128 + 128 > p.S);  // uniform over the CTA
      const int col0 = cg * 32;
      uint32_t sv[32], dpv[32];
      tmem_ld32(tmem + lane_base + C::COL_S + col0, sv);
      tmem_ld32(tmem + lane_base + C::COL_DP + col0, dpv);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_sfree);  // S and dP columns may be overwritten
      if constexpr (BIAS)
        add_bias_row<T, 32>(sv, p.bias + (static_cast<int64_t>(bh) * p.S + (vq ? qrow : 0)) * p.S, j * 128 + col0, p.S, vq,
                            p.inv_scale, p.bias_vec);
      uint32_t pk[16], dk[16];
      if (!masked) {
        // packed fp32 pairs: one FMA / ADD / MUL instruction per two elements
        const float2 c2 = make_float2(scale_log2, scale_log2), nl2 = make_float2(-lse2, -lse2), nd2 = make_float2(-dlt, -dlt);
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const float2 x = __ffma2_rn(make_float2(__uint_as_float(sv[e]), __uint_as_float(sv[e + 1])), c2, nl2);
          const float2 pp = make_float2(ex2(x.x), ex2(x.y));
          const float2 ds =
              __fmul2_rn(pp, __fadd2_rn(make_float2(__uint_as_float(dpv[e]), __uint_as_float(dpv[e + 1])), nd2));
          pk[e >> 1] = pack_pair<T>(pp.x, pp.y);
          dk[e >> 1] = pack_pair<T>(ds.x, ds.y);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float pv[2], dv[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int kvrow = j * 128 + col0 + e + u;
            const bool keep = vq && kvrow < p.S && (!diag || kvrow <= qrow);
            const float pe = keep ? ex2(fmaf(__uint_as_float(sv[e + u]), scale_log2, -lse2)) : 0.f;
            pv[u] = pe;
            dv[u] = pe * (__uint_as_float(dpv[e + u]) - dlt);
          }
          pk[e >> 1] = pack_pair<T>(pv[0], pv[1]);
          dk[e >> 1] = pack_pair<T>(dv[0], dv[1]);
        }
      }
      // P | dS may be rewritten once the previous tile's MMAs have read them (LATE: bar_dqf of that tile;
      // otherwise: the TMA unit has read the dQ tile that was staged there)
      if (it > 0) {
        ok = C::LATE ? mbar_wait(bar_dqf, (it - 1) & 1u) : mbar_wait(bar_stg, (it - 1) & 1u);
        if (!ok) break;
      }
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const uint32_t off = ps_chunk_off(r, (col0 >> 3) + t);
        *reinterpret_cast<uint4*>(gen + C::OFF_P + off) = make_uint4(pk[4 * t], pk[4 * t + 1], pk[4 * t + 2], pk[4 * t + 3]);
        *reinterpret_cast<uint4*>(gen + C::OFF_DS + off) = make_uint4(dk[4 * t], dk[4 * t + 1], dk[4 * t + 2], dk[4 * t + 3]);
      }
      if (C::DS_TMEM) {  // dS once more as packed bf16 pairs: 16 TMEM columns per 32 key columns
        tmem_st16(tmem + lane_base + C::COL_DSA + cg * 16, dk);
        tmem_st_wait();
      }
      fence_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pds);
      if (C::LATE) {
        if (it > 0) ok = drain(it - 1, false);  // bar_dqf of tile it-1 was waited for above
      } else {
        ok = drain(it, true);
      }
    }
    if (C::LATE && ok && iters > 0) ok = drain(iters - 1, true);
    if (!ok && lane == 0) atomicExch(p.status, kErrBwdCompute);
    // dK / dV: every MMA was complete when the last bar_dqf fired, so the K and V tiles in shared memory are free:
    // each thread parks its slice of the two accumulators there (16-bit, same swizzled [128][64] boxes the loads
    // used) and one thread lets the TMA unit write both tiles out, whole 128-byte lines per request, rows past S
    // clipped by the tensor map.  (Per-thread 16-byte stores to rows 4.6 KB apart cost 9% of the kernel.)
    if (ok && iters > 0) {
      const float sc = p.scale;
#pragma unroll 1
      for (int c0 = 0; c0 < DC; c0 += 16) {
        uint32_t a[16], c[16];
        tmem_ld16(tmem + lane_base + C::COL_DK + cg * DC + c0, a);
        tmem_ld16(tmem + lane_base + C::COL_DV + cg * DC + c0, c);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 16; e += 8) {
          uint4 o1, o2;
          o1.x = pack_pair<T>(__uint_as_float(a[e]) * sc, __uint_as_float(a[e + 1]) * sc);
          o1.y = pack_pair<T>(__uint_as_float(a[e + 2]) * sc, __uint_as_float(a[e + 3]) * sc);
          o1.z = pack_pair<T>(__uint_as_float(a[e + 4]) * sc, __uint_as_float(a[e + 5]) * sc);
          o1.w = pack_pair<T>(__uint_as_float(a[e + 6]) * sc, __uint_as_float(a[e + 7]) * sc);
          o2.x = pack_pair<T>(__uint_as_float(c[e]), __uint_as_float(c[e + 1]));
          o2.y = pack_pair<T>(__uint_as_float(c[e + 2]), __uint_as_float(c[e + 3]));
          o2.z = pack_pair<T>(__uint_as_float(c[e + 4]), __uint_as_float(c[e + 5]));
          o2.w = pack_pair<T>(__uint_as_float(c[e + 6]), __uint_as_float(c[e + 7]));
          const uint32_t off = ps_chunk_off(r, (cg * DC + c0 + e) >> 3);
          *reinterpret_cast<uint4*>(gen + C::OFF_K + off) = o1;
          *reinterpret_cast<uint4*>(gen + C::OFF_V + off) = o2;
        }
      }
      fence_async_smem();
    }
    named_barrier(1, 16 * 32);  // the 16 compute warps (all of them get here, also after a failed wait)
    if (ok && iters > 0 && warp == 2 && lane == 0) {
#pragma unroll
      for (int c = 0; c < C::HALVES; ++c) {
        tma_store_4d(&tm_dk, base + C::OFF_K + c * kHalfBytes, c * 64, h, j * 128, b);
        tma_store_4d(&tm_dv, base + C::OFF_V + c * kHalfBytes, c * 64, h, j * 128, b);
      }
      bulk_commit();
      bulk_wait_read0();  // the tiles have been read; the writes themselves complete before the grid does
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, C::TMEM_COLS);
  }
}

// acc is packed (tokens x HD) fp32; dq rows are ld elements apart.
template <typename T>
__global__ void __launch_bounds__(256) cast_dq_kernel(const float* __restrict__ acc, bf16* __restrict__ dq, int64_t n8,
                                                      int hd8, int64_t ld, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t stride = static_cast<int64_t>(gridDim.x) * 256;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < n8; i += stride) {
    const int64_t tok = i / hd8;
    const int c8 = static_cast<int>(i - tok * hd8);
    const float4 a = reinterpret_cast<const float4*>(acc)[2 * i];
    const float4 c = reinterpret_cast<const float4*>(acc)[2 * i + 1];
    uint4 o;
    o.x = pack_pair<T>(a.x * scale, a.y * scale);
    o.y = pack_pair<T>(a.z * scale, a.w * scale);
    o.z = pack_pair<T>(c.x * scale, c.y * scale);
    o.w = pack_pair<T>(c.z * scale, c.w * scale);
    *reinterpret_cast<uint4*>(dq + tok * ld + c8 * 8) = o;
  }
}

// =============================================================== forward
// ------------------------------------------------- forward, D = 64: persistent, two CTAs per SM
// A launch of one CTA per query tile spends 4 to 5 us per CTA outside the tile loop (launch gap, TMEM allocation,
// first loads from cold, output epilogue) against 0.8 us per 64 keys inside it, so the kernel is persistent: two
// CTAs per SM, each walking a static list of (batch, head, query tile) items, heavy tiles first and dealt out in
// alternating direction so that the lists weigh about the same.  The pipelines run across item boundaries: Q has
// two slots (the next item's Q arrives while this one computes; the finished item's output is parked in its own Q
// slot and leaves by a TMA store that the next item does not wait for), and the first scores of the next item are
// formed while the softmax warps are still in this item's epilogue.
// A CTA is 6 warps (TMA, MMA, 4 softmax warps; a softmax thread owns a query row).  K and V arrive in 128-key
// chunks (two stages each) but the products run on 64-key tiles, so that everything between the tensor pipe and
// the softmax warps has two buffers inside 256 TMEM columns: S0 S1 (64 fp32 columns each), O (64), and P0 P1 as
// packed 16-bit pairs (32 columns each; the P V product reads its A operand from TMEM).  With two buffers the
// exponentials of tile t + 1 never wait for the product P_t V_t: the only dependence of a softmax thread on that
// product is the rescale of O, which the lazy reference maximum makes rare.
struct Fwd64Cfg {
  static constexpr int D = 64;
  static constexpr int KT = 64;                   // keys per tile
  static constexpr int TILE_BYTES = 128 * D * 2;  // 16 KB: a 128-row chunk of Q, K or V
  static constexpr int OFF_Q = 0;                 // 2 slots
  static constexpr int OFF_K = 2 * TILE_BYTES;    // 2 stages
  static constexpr int OFF_V = 4 * TILE_BYTES;    // 2 stages
  static constexpr int OFF_BAR = 6 * TILE_BYTES;
  static constexpr int SMEM = OFF_BAR + 256 + 1024;
  static constexpr int COL_S = 0, COL_O = 128, COL_P = 192;
  static constexpr int TMEM_COLS = 256;
  static constexpr int THREADS = 192;
};

// The n-th work item of this CTA.  Items are numbered heavy first (all heads of the last query tile, then of the
// one before, ...); round n of the deal hands items n*G .. n*G + G - 1 to the G CTAs, in reversed order on odd rounds.
struct Fwd64Item {
  int i, bh, b, h;  // query tile, (batch, head)
  int nt, nch;      // 64-key tiles, 128-key chunks
};
__device__ __forceinline__ bool fwd64_item(const AttnParams& p, int n, Fwd64Item& it) {
  const int G = static_cast<int>(gridDim.x), c = static_cast<int>(blockIdx.x);
  const int BH = p.B * p.H, nq = (p.S + 127) / 128;
  // 32-bit arithmetic: the host refuses launches with more than 2^30 items
  const unsigned w = static_cast<unsigned>(n) * G + ((n & 1) ? G - 1 - c : c);
  if (w >= static_cast<unsigned>(BH) * nq) return false;
  const int level = static_cast<int>(w / static_cast<unsigned>(BH));
  it.bh = static_cast<int>(w - static_cast<unsigned>(level) * BH);
  it.i = nq - 1 - level;
  it.b = it.bh / p.H;
  it.h = it.bh - it.b * p.H;
  const int nt_all = (p.S + Fwd64Cfg::KT - 1) / Fwd64Cfg::KT;
  it.nt = p.causal ? min(2 * (it.i + 1), nt_all) : nt_all;
  it.nch = (it.nt + 1) >> 1;
  return true;
}

template <typename T, bool BIAS>
__global__ void __launch_bounds__(Fwd64Cfg::THREADS, 2)
    attn_fwd_tc64_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                         const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                         const AttnParams p) {
  using C = Fwd64Cfg;
  constexpr int D = C::D;
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  unsigned char* gen = smem_dyn + (base - smem_u32(smem_dyn));
  const uint32_t bar = base + C::OFF_BAR;
  auto bar_qf = [&](int s) { return bar + 0 + 8u * s; };    // Q slot s loaded
  auto bar_qe = [&](int s) { return bar + 16 + 8u * s; };   // ... free again (its parked output has left)
  auto bar_kf = [&](int s) { return bar + 32 + 8u * s; };
  auto bar_ke = [&](int s) { return bar + 48 + 8u * s; };
  auto bar_vf = [&](int s) { return bar + 64 + 8u * s; };
  auto bar_ve = [&](int s) { return bar + 80 + 8u * s; };
  auto bar_sf = [&](int u) { return bar + 96 + 8u * u; };   // scores of a tile complete in TMEM buffer u
  auto bar_sr = [&](int u) { return bar + 112 + 8u * u; };  // ... are in registers: the buffer is free
  auto bar_pr = [&](int u) { return bar + 128 + 8u * u; };  // P written into buffer u (and O rescaled)
  auto bar_pv = [&](int u) { return bar + 144 + 8u * u; };  // O += P V complete for buffer u
  const uint32_t tmem_slot = bar + 160;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(gen + C::OFF_BAR + 160);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_qf(s), 1);
      mbar_init(bar_qe(s), 1);
      mbar_init(bar_kf(s), 1);
      mbar_init(bar_ke(s), 1);
      mbar_init(bar_vf(s), 1);
      mbar_init(bar_ve(s), 1);
      mbar_init(bar_sf(s), 1);
      mbar_init(bar_sr(s), 4);
      mbar_init(bar_pr(s), 4);
      mbar_init(bar_pv(s), 1);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_gen;
  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      tma_prefetch_desc(&tm_o);
      auto load_q = [&](int n, const Fwd64Item& it) -> bool {
        const int s = n & 1;
        if (!mbar_wait(bar_qe(s), ((n >> 1) & 1u) ^ 1u)) return false;
        mbar_expect_tx(bar_qf(s), C::TILE_BYTES);
        tma_load_4d(base + C::OFF_Q + s * C::TILE_BYTES, &tm_q, bar_qf(s), 0, it.h, it.i * 128, it.b);
        return true;
      };
      Fwd64Item it, nx;
      bool ok = true;
      bool have = fwd64_item(p, 0, it);
      if (have) ok = load_q(0, it);
      int g = 0;  // chunks loaded so far, over all items: stage and phase of the K / V rings
      for (int n = 0; have && ok; ++n) {
        const bool has_next = fwd64_item(p, n + 1, nx);
        const int c_q = it.nch > 1 ? 1 : 0;  // the next Q is asked for once this item's first chunks are on their way
        for (int c = 0; c < it.nch && ok; ++c, ++g) {
          const int s = g & 1;
          const uint32_t par = ((g >> 1) & 1u) ^ 1u;
          if (!mbar_wait(bar_ke(s), par)) {
            ok = false;
            break;
          }
          mbar_expect_tx(bar_kf(s), C::TILE_BYTES);
          tma_load_4d(base + C::OFF_K + s * C::TILE_BYTES, &tm_k, bar_kf(s), 0, it.h, c * 128, it.b);
          if (!mbar_wait(bar_ve(s), par)) {
            ok = false;
            break;
          }
          mbar_expect_tx(bar_vf(s), C::TILE_BYTES);
          tma_load_4d(base + C::OFF_V + s * C::TILE_BYTES, &tm_v, bar_vf(s), 0, it.h, c * 128, it.b);
          if (c == c_q && has_next) ok = load_q(n + 1, nx);
        }
        it = nx;
        have = has_next;
      }
      if (!ok) atomicExch(p.status, kErrFwdTma);
    }
    __syncwarp();
  } else if (warp == 1) {
    // All 32 lanes walk the same control flow (waits included, their outcome made uniform by a vote) and one
    // elected lane issues: descriptors and cursors then live in uniform registers.
    {
      constexpr uint32_t id_s = umma_idesc_16<T>(128, C::KT, 0, 0);
      constexpr uint32_t id_o = umma_idesc_16<T>(128, D, 0, 1);
      const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
      auto wait_all = [&](uint32_t bar_addr, uint32_t parity) -> bool {
        return __all_sync(0xffffffffu, mbar_wait(bar_addr, parity));
      };
      // Two cursors over the CTA's tiles (item n, tile t of it, g0 = chunks of earlier items): the scores run two
      // tiles ahead of the P V products, across item boundaries.
      struct Cursor {
        int n, t, g0;
        bool valid;
        Fwd64Item it;
      };
      auto advance = [&](Cursor& c) {
        if (++c.t == c.it.nt) {
          c.g0 += c.it.nch;
          c.t = 0;
          c.valid = fwd64_item(p, ++c.n, c.it);
        }
      };
      Cursor cs{0, 0, 0, false, {}}, cp{0, 0, 0, false, {}};
      cs.valid = fwd64_item(p, 0, cs.it);
      cp = cs;
      int ts = 0, tp = 0;  // tiles issued so far: buffer and phase of the S / P rings
      // operand descriptors of every buffer, built once
      const uint64_t dQs[2] = {base_k(base + C::OFF_Q), base_k(base + C::OFF_Q + C::TILE_BYTES)};
      const uint64_t dKs[2] = {base_k(base + C::OFF_K), base_k(base + C::OFF_K + C::TILE_BYTES)};
      const uint64_t dVs[2] = {base_mn(base + C::OFF_V), base_mn(base + C::OFF_V + C::TILE_BYTES)};
      auto issue_s = [&]() -> bool {
        const int t = cs.t, g = cs.g0 + (t >> 1), s = g & 1, u = ts & 1, qs = cs.n & 1;
        if (t == 0 && !wait_all(bar_qf(qs), (cs.n >> 1) & 1u)) return false;
        if ((t & 1) == 0 && !wait_all(bar_kf(s), (g >> 1) & 1u)) return false;
        if (ts >= 2 && !wait_all(bar_sr(u), ((ts - 2) >> 1) & 1u)) return false;  // tile ts - 2 is in registers
        tc_fence_after();
        const uint64_t dQ = qs ? dQs[1] : dQs[0];
        const uint64_t dK = (s ? dKs[1] : dKs[0]) + static_cast<uint64_t>(((t & 1) * (C::KT * 128)) >> 4);
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < D / 16; ++k)
            umma_ss(tm + C::COL_S + u * C::KT, desc_k(dQ, k), desc_k(dK, k), id_s, k > 0);
          if ((t & 1) || t == cs.it.nt - 1) umma_commit(bar_ke(s));  // last product that reads this K chunk
          umma_commit(bar_sf(u));
        }
        __syncwarp();
        ++ts;
        advance(cs);
        return true;
      };
      bool ok = true;
      if (cs.valid) ok = issue_s();
      if (ok && cs.valid) ok = issue_s();
      while (ok && cp.valid) {
        // scores first: tile tp + 2 only needs tile tp in registers, which comes before P of tile tp
        if (cs.valid && ts < tp + 3) ok = issue_s();
        if (!ok) break;
        const int t = cp.t, g = cp.g0 + (t >> 1), s = g & 1, u = tp & 1;
        ok = wait_all(bar_pr(u), (tp >> 1) & 1u);
        if (ok && (t & 1) == 0) ok = wait_all(bar_vf(s), (g >> 1) & 1u);
        if (!ok) break;
        tc_fence_after();
        const uint64_t dV = desc_mn(s ? dVs[1] : dVs[0], (t & 1) * 4);
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < C::KT / 16; ++k)  // P is a TMEM operand: 8 packed columns per 16 keys
            umma_ts(tm + C::COL_O, tm + C::COL_P + u * (C::KT / 2) + k * 8, desc_mn(dV, k), id_o,
                    (t > 0 || k > 0) ? 1u : 0u);
          if ((t & 1) || t == cp.it.nt - 1) umma_commit(bar_ve(s));
          umma_commit(bar_pv(u));
        }
        __syncwarp();
        ++tp;
        advance(cp);
      }
      if (!ok && lane == 0) atomicExch(p.status, kErrFwdMma);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ softmax: one thread per query row
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const float scale_log2 = p.scale * kLog2e;
    const bool storer = (warp == 2 && lane == 0);
    int tt = 0;          // tiles done so far, over all items
    int parked = -1;     // Q slot whose parked output is still leaving (storer only)
    bool ok = true;
    Fwd64Item it;
    // After a failed wait a warp stops touching TMEM and mbarriers but still walks its items for the named
    // barrier of the epilogue, so that the other softmax warps are never left waiting on it.
    for (int n = 0; fwd64_item(p, n, it); ++n) {
      const int i = it.i, bh = it.bh;
      const int qrow = i * 128 + r;
      float m = -INFINITY, l = 0.f;
      for (int t = 0; t < it.nt && ok; ++t, ++tt) {
        const int u = tt & 1;
        if (!mbar_wait(bar_sf(u), (tt >> 1) & 1u)) {
          ok = false;
          break;
        }
        tc_fence_after();
        uint32_t v[C::KT];
#pragma unroll
        for (int c = 0; c < C::KT / 32; ++c)
          tmem_ld32(tmem + lane_base + C::COL_S + u * C::KT + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[c * 32]));
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_sr(u));
        const int key0 = t * C::KT;
        if constexpr (BIAS)
          add_bias_row<T, C::KT>(v, p.bias + (static_cast<int64_t>(bh) * p.S + (qrow < p.S ? qrow : 0)) * p.S, key0, p.S,
                                 qrow < p.S, p.inv_scale, p.bias_vec);
        const bool diag = p.causal && (key0 + C::KT - 1 > i * 128);
        if (diag || (key0 + C::KT > p.S)) {
#pragma unroll
          for (int e = 0; e < C::KT; ++e) {
            const int kvrow = key0 + e;
            const bool keep = kvrow < p.S && (!diag || kvrow <= qrow);
            if (!keep) v[e] = __float_as_uint(-INFINITY);
          }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int e = 0; e < C::KT; e += 4) {
          mx0 = fmaxf(mx0, __uint_as_float(v[e]));
          mx1 = fmaxf(mx1, __uint_as_float(v[e + 1]));
          mx2 = fmaxf(mx2, __uint_as_float(v[e + 2]));
          mx3 = fmaxf(mx3, __uint_as_float(v[e + 3]));
        }
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        // lazy reference maximum, as in the D = 128 kernel
        const float m_cand = fmaxf(m, mx * scale_log2);
        const float m_new = (t == 0 || m_cand - m > 8.f) ? m_cand : m;
        const float corr = (t == 0) ? 0.f : ex2(m - m_new);
        // P buffer u is free once the product of tile tt - 2 is complete (every phase of bar_pv(u) is waited for
        // here, in order)
        if (tt >= 2 && !mbar_wait(bar_pv(u), ((tt - 2) >> 1) & 1u)) {
          ok = false;
          break;
        }
        if (t > 0 && __any_sync(0xffffffffu, m_new != m)) {
          // O must be stable: the product of tile tt - 1 (the other buffer; this phase is waited for again, as the
          // "buffer free" wait of tile tt + 1, which is harmless)
          if (!mbar_wait(bar_pv(u ^ 1), ((tt - 1) >> 1) & 1u)) {
            ok = false;
            break;
          }
          tc_fence_after();
#pragma unroll 1
          for (int c0 = 0; c0 < D; c0 += 16) {
            uint32_t o[16];
            tmem_ld16(tmem + lane_base + C::COL_O + c0, o);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 16; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * corr);
            tmem_st16(tmem + lane_base + C::COL_O + c0, o);
          }
          tmem_st_wait();
        }
        tc_fence_after();
        float rs0 = 0.f, rs1 = 0.f;
        const float neg_m = (m_new == -INFINITY) ? 0.f : -m_new;
#pragma unroll
        for (int c32 = 0; c32 < C::KT / 32; ++c32) {
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const float p0 = ex2(fmaf(__uint_as_float(v[c32 * 32 + 2 * e]), scale_log2, neg_m));
            const float p1 = ex2(fmaf(__uint_as_float(v[c32 * 32 + 2 * e + 1]), scale_log2, neg_m));
            rs0 += p0;
            rs1 += p1;
            pk[e] = pack_pair<T>(p0, p1);
          }
          tmem_st16(tmem + lane_base + C::COL_P + u * (C::KT / 2) + c32 * 16, pk);
        }
        tmem_st_wait();
        l = l * corr + (rs0 + rs1);
        m = m_new;
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_pr(u));
        if (t == 0 && storer && parked >= 0) {  // the previous item's output has had a tile's time to leave
          bulk_wait_read0();
          mbar_arrive(bar_qe(parked));
          parked = -1;
        }
      }
      // the item's last product; the tensor pipe completes a thread's products in order, so every earlier one is
      // done too
      if (ok && !mbar_wait(bar_pv((tt - 1) & 1), ((tt - 1) >> 1) & 1u)) ok = false;
      // The normalised output leaves through the TMA unit: every thread parks its row in the item's Q slot (free
      // once the last scores were formed; same swizzled box) and one thread stores the tile, whole 128-byte lines
      // per request, rows past S clipped by the tensor map.
      const uint32_t q_off = C::OFF_Q + (n & 1) * C::TILE_BYTES;
      if (ok) {
        tc_fence_after();
        const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 16) {
          uint32_t o[16];
          tmem_ld16(tmem + lane_base + C::COL_O + c0, o);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 16; e += 8) {
            uint4 w;
            w.x = pack_pair<T>(__uint_as_float(o[e]) * inv, __uint_as_float(o[e + 1]) * inv);
            w.y = pack_pair<T>(__uint_as_float(o[e + 2]) * inv, __uint_as_float(o[e + 3]) * inv);
            w.z = pack_pair<T>(__uint_as_float(o[e + 4]) * inv, __uint_as_float(o[e + 5]) * inv);
            w.w = pack_pair<T>(__uint_as_float(o[e + 6]) * inv, __uint_as_float(o[e + 7]) * inv);
            *reinterpret_cast<uint4*>(gen + q_off + ps_chunk_off(r, (c0 + e) >> 3)) = w;
          }
        }
        tc_fence_before();
        fence_async_smem();
        if (qrow < p.S) p.lse_out[static_cast<int64_t>(bh) * p.S + qrow] = (m + log2f(l)) / kLog2e;
      }
      named_barrier(1, 4 * 32);  // the four softmax warps
      if (ok && storer) {
        if (p.o_bshd)
          tma_store_4d(&tm_o, base + q_off, 0, it.h, i * 128, it.b);
        else
          tma_store_3d(&tm_o, base + q_off, 0, i * 128, bh);
        bulk_commit();
        parked = n & 1;
      }
    }
    if (storer && parked >= 0) bulk_wait_read0();  // shared memory must outlive the last store's reads
    if (!ok && lane == 0) atomicExch(p.status, kErrFwdSoftmax);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, C::TMEM_COLS);
  }
}

// ------------------------------------------- forward, D = 128: two query tiles per CTA
// One CTA owns two adjacent 128-row query tiles (A = 2c, B = 2c + 1) and walks the key tiles once for both: every
// K / V tile is loaded once and used twice, and while the four softmax warps of one tile are in their exp phase the
// tensor pipe works for the other tile.  A softmax thread owns a whole row (128 scores in registers, one TMEM read,
// no exchange of row maxima).  TMEM: S_A | S_B | O_A | O_B, 128 columns each; shared memory: Q_A, Q_B, two K
// stages, one V stage, P_A, P_B (224 KB).  With a causal mask tile B has one key tile more than tile A.
struct Fwd128Cfg {
  static constexpr int D = 128;
  static constexpr int TILE_BYTES = 128 * D * 2;  // 32 KB
  static constexpr int OFF_Q = 0;                 // A, B
  static constexpr int OFF_K = 2 * TILE_BYTES;    // 2 stages
  static constexpr int OFF_V = 4 * TILE_BYTES;    // 1 stage
  static constexpr int OFF_P = 5 * TILE_BYTES;    // A, B
  static constexpr int OFF_BAR = 7 * TILE_BYTES;
  static constexpr int SMEM = OFF_BAR + 256 + 1024;
  static constexpr int TMEM_COLS = 512;
  static constexpr int THREADS = 320;  // TMA, MMA, 4 softmax warps per query tile
};

template <typename T, bool BIAS>
__global__ void __launch_bounds__(Fwd128Cfg::THREADS, 1)
    attn_fwd_tc128x2_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                            const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                            const AttnParams p) {
  using C = Fwd128Cfg;
  constexpr int D = C::D;
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  unsigned char* gen = smem_dyn + (base - smem_u32(smem_dyn));
  const uint32_t bar = base + C::OFF_BAR;
  const uint32_t bar_q = bar;
  auto bar_kf = [&](int s) { return bar + 8 + 8u * s; };
  auto bar_ke = [&](int s) { return bar + 24 + 8u * s; };
  const uint32_t bar_vf = bar + 40, bar_ve = bar + 48;
  auto bar_sf = [&](int t) { return bar + 56 + 8u * t; };   // scores of tile t complete in TMEM
  auto bar_sr = [&](int t) { return bar + 72 + 8u * t; };   // scores of tile t are in registers
  auto bar_pr = [&](int t) { return bar + 88 + 8u * t; };   // P of tile t written (and O rescaled)
  auto bar_pv = [&](int t) { return bar + 104 + 8u * t; };  // O_t += P_t V complete
  const uint32_t tmem_slot = bar + 120;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(gen + C::OFF_BAR + 120);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = (p.S + 127) / 128;
  const int npair = (nq + 1) / 2;
  const int c = npair - 1 - static_cast<int>(blockIdx.x);  // heavy (late) pairs first
  const int bh = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int qt[2] = {2 * c, 2 * c + 1};
  int nkv[2];
  nkv[0] = p.causal ? qt[0] + 1 : nq;
  nkv[1] = qt[1] < nq ? (p.causal ? qt[1] + 1 : nq) : 0;
  const int nmax = nkv[0] > nkv[1] ? nkv[0] : nkv[1];

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_kf(s), 1);
      mbar_init(bar_ke(s), 1);
      mbar_init(bar_sf(s), 1);
      mbar_init(bar_sr(s), 4);
      mbar_init(bar_pr(s), 4);
      mbar_init(bar_pv(s), 1);
    }
    mbar_init(bar_vf, 1);
    mbar_init(bar_ve, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_gen;
  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      mbar_expect_tx(bar_q, 2 * C::TILE_BYTES);  // rows past the sequence arrive as zeros
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf)
          tma_load_4d(base + C::OFF_Q + t * C::TILE_BYTES + hf * kHalfBytes, &tm_q, bar_q, hf * 64, h, qt[t] * 128, b);
      bool ok = true;
      auto load_k = [&](int jt) {
        const int s = jt & 1;
        if (!mbar_wait(bar_ke(s), ((jt >> 1) & 1u) ^ 1u)) return false;
        mbar_expect_tx(bar_kf(s), C::TILE_BYTES);
#pragma unroll
        for (int hf = 0; hf < 2; ++hf)
          tma_load_4d(base + C::OFF_K + s * C::TILE_BYTES + hf * kHalfBytes, &tm_k, bar_kf(s), hf * 64, h, jt * 128, b);
        return true;
      };
      ok = load_k(0);
      for (int jt = 0; jt < nmax && ok; ++jt) {
        if (jt + 1 < nmax) ok = load_k(jt + 1);  // K runs a tile ahead of V
        if (!ok || !mbar_wait(bar_ve, (jt & 1u) ^ 1u)) {
          ok = false;
          break;
        }
        mbar_expect_tx(bar_vf, C::TILE_BYTES);
#pragma unroll
        for (int hf = 0; hf < 2; ++hf)
          tma_load_4d(base + C::OFF_V + hf * kHalfBytes, &tm_v, bar_vf, hf * 64, h, jt * 128, b);
      }
      if (!ok) atomicExch(p.status, kErrFwdTma);
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t id_s = umma_idesc_16<T>(128, 128, 0, 0);
      constexpr uint32_t id_o = umma_idesc_16<T>(128, D, 0, 1);
      const uint64_t dV = base_mn(base + C::OFF_V);
      // scores of key tile jt for every query tile that still has work there
      auto issue_s = [&](int jt) -> bool {
        const int s = jt & 1;
        if (!mbar_wait(bar_kf(s), (jt >> 1) & 1u)) return false;
        const uint64_t dK = base_k(base + C::OFF_K + s * C::TILE_BYTES);
        for (int t = 0; t < 2; ++t) {
          if (jt >= nkv[t]) continue;
          if (jt >= 1 && !mbar_wait(bar_sr(t), (jt - 1) & 1u)) return false;  // previous scores are in registers
          tc_fence_after();
          const uint64_t dQ = base_k(base + C::OFF_Q + t * C::TILE_BYTES);
#pragma unroll
          for (int k = 0; k < D / 16; ++k) umma_ss(tmem + t * 128, desc_k(dQ, k), desc_k(dK, k), id_s, k > 0);
          umma_commit(bar_sf(t));
        }
        umma_commit(bar_ke(s));
        return true;
      };
      bool ok = mbar_wait(bar_q, 0) && issue_s(0);
      for (int jt = 0; jt < nmax && ok; ++jt) {
        if (jt + 1 < nmax) ok = issue_s(jt + 1);
        ok = ok && mbar_wait(bar_vf, jt & 1u);
        for (int t = 0; t < 2 && ok; ++t) {
          if (jt >= nkv[t]) continue;
          if (!mbar_wait(bar_pr(t), jt & 1u)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t dP = base_k(base + C::OFF_P + t * kPsBytes);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            umma_ss(tmem + 256 + t * 128, desc_k(dP, k), desc_mn(dV, k), id_o, (jt > 0 || k > 0) ? 1u : 0u);
          umma_commit(bar_pv(t));
        }
        if (ok) umma_commit(bar_ve);  // after the last product that reads this V tile
      }
      if (!ok) atomicExch(p.status, kErrFwdMma);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ softmax: one thread per query row
    const int t = (warp - 2) >> 2;  // query tile of this warp
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t col_s = t * 128, col_o = 256 + t * 128;
    unsigned char* ps = gen + C::OFF_P + t * kPsBytes;
    const int i = qt[t];
    const int qrow = i * 128 + r;
    const int my_nkv = nkv[t];
    const float scale_log2 = p.scale * kLog2e;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int jt = 0; jt < my_nkv && ok; ++jt) {
      if (!mbar_wait(bar_sf(t), jt & 1u)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t v[128];
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) tmem_ld32(tmem + lane_base + col_s + cc * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[cc * 32]));
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_sr(t));
      if constexpr (BIAS)
        add_bias_row<T, 128>(v, p.bias + (static_cast<int64_t>(bh) * p.S + (qrow < p.S ? qrow : 0)) * p.S, jt * 128, p.S,
                             qrow < p.S, p.inv_scale, p.bias_vec);
      const bool diag = p.causal && (jt == i);
      if (diag || (jt * 128 + 128 > p.S)) {
#pragma unroll
        for (int e = 0; e < 128; ++e) {
          const int kvrow = jt * 128 + e;
          const bool keep = kvrow < p.S && (!diag || kvrow <= qrow);
          if (!keep) v[e] = __float_as_uint(-INFINITY);
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int e = 0; e < 128; e += 4) {
        mx0 = fmaxf(mx0, __uint_as_float(v[e]));
        mx1 = fmaxf(mx1, __uint_as_float(v[e + 1]));
        mx2 = fmaxf(mx2, __uint_as_float(v[e + 2]));
        mx3 = fmaxf(mx3, __uint_as_float(v[e + 3]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      const float m_cand = fmaxf(m, mx * scale_log2);
      const float m_new = (jt == 0 || m_cand - m > 8.f) ? m_cand : m;  // lazy reference maximum
      const float corr = (jt == 0) ? 0.f : ex2(m - m_new);
      if (jt > 0 && !mbar_wait(bar_pv(t), (jt - 1) & 1u)) {  // P may be overwritten, O is stable
        ok = false;
        break;
      }
      tc_fence_after();
      if (jt > 0 && __any_sync(0xffffffffu, m_new != m)) {
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 16) {
          uint32_t o[16];
          tmem_ld16(tmem + lane_base + col_o + c0, o);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 16; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * corr);
          tmem_st16(tmem + lane_base + col_o + c0, o);
        }
        tmem_st_wait();
      }
      float rs0 = 0.f, rs1 = 0.f;
      const float neg_m = (m_new == -INFINITY) ? 0.f : -m_new;
#pragma unroll
      for (int c8 = 0; c8 < 16; ++c8) {
        uint32_t pk[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p0 = ex2(fmaf(__uint_as_float(v[c8 * 8 + 2 * e]), scale_log2, neg_m));
          const float p1 = ex2(fmaf(__uint_as_float(v[c8 * 8 + 2 * e + 1]), scale_log2, neg_m));
          rs0 += p0;
          rs1 += p1;
          pk[e] = pack_pair<T>(p0, p1);
        }
        *reinterpret_cast<uint4*>(ps + ps_chunk_off(r, c8)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
      l = l * corr + (rs0 + rs1);
      m = m_new;
      fence_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pr(t));
    }
    if (ok && my_nkv > 0 && !mbar_wait(bar_pv(t), (my_nkv - 1) & 1u)) ok = false;
    // The normalised output leaves through the TMA unit: every thread parks its row in its query tile's Q buffer
    // (free once the tile's last scores were formed) and one thread per tile stores it.
    if (!ok) {
      if (lane == 0) atomicExch(p.status, kErrFwdSoftmax);
    } else if (my_nkv > 0) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 16) {
        uint32_t o[16];
        tmem_ld16(tmem + lane_base + col_o + c0, o);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 16; e += 8) {
          uint4 w;
          w.x = pack_pair<T>(__uint_as_float(o[e]) * inv, __uint_as_float(o[e + 1]) * inv);
          w.y = pack_pair<T>(__uint_as_float(o[e + 2]) * inv, __uint_as_float(o[e + 3]) * inv);
          w.z = pack_pair<T>(__uint_as_float(o[e + 4]) * inv, __uint_as_float(o[e + 5]) * inv);
          w.w = pack_pair<T>(__uint_as_float(o[e + 6]) * inv, __uint_as_float(o[e + 7]) * inv);
          *reinterpret_cast<uint4*>(gen + C::OFF_Q + t * C::TILE_BYTES + ps_chunk_off(r, (c0 + e) >> 3)) = w;
        }
      }
      fence_async_smem();
      if (qrow < p.S) p.lse_out[static_cast<int64_t>(bh) * p.S + qrow] = (m + log2f(l)) / kLog2e;
    }
    named_barrier(1 + t, 4 * 32);  // the four softmax warps of this query tile
    if (ok && my_nkv > 0 && (warp & 3) == 2 && lane == 0) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const uint32_t src = base + C::OFF_Q + t * C::TILE_BYTES + c * kHalfBytes;
        if (p.o_bshd)
          tma_store_4d(&tm_o, src, c * 64, h, i * 128, b);
        else
          tma_store_3d(&tm_o, src, c * 64, i * 128, bh);
      }
      bulk_commit();
      bulk_wait_read0();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, C::TMEM_COLS);
  }
}

// ------------------------------------------------------------------ host
bool map_bshd(CUtensorMap* m, const void* ptr, int B, int S, int H, int D, int64_t ld) {
  const uint64_t dims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(H), static_cast<uint64_t>(S),
                            static_cast<uint64_t>(B)};
  const uint64_t strides[3] = {static_cast<uint64_t>(D) * 2, static_cast<uint64_t>(ld) * 2,
                               static_cast<uint64_t>(S) * ld * 2};
  const uint32_t box[4] = {64, 1, 128, 1};
  return encode_tmap_bf16(m, ptr, 4, dims, strides, box);
}
bool map_bhsd(CUtensorMap* m, const void* ptr, int B, int S, int H, int D) {
  const uint64_t dims[3] = {static_cast<uint64_t>(D), static_cast<uint64_t>(S), static_cast<uint64_t>(B) * H};
  const uint64_t strides[2] = {static_cast<uint64_t>(D) * 2, static_cast<uint64_t>(S) * D * 2};
  const uint32_t box[3] = {64, 128, 1};
  return encode_tmap_bf16(m, ptr, 3, dims, strides, box);
}

template <typename K>
int set_smem(K kern, int bytes) {
  const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return fail(MGB_ECUDA, "attention smem opt-in (%d B): %s", bytes, cudaGetErrorString(e));
  // the largest shared-memory carveout, so that two CTAs of the D = 64 forward kernel fit on an SM
  cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  return MGB_OK;
}

template <int D, typename T>
int run_bwd(const void* dy, const void* q, const void* k, const void* v, AttnParams p, int64_t ld_qkv,
            cudaStream_t st) {
  using C = BwdCfg<D>;
  CUtensorMap mq, mk, mv, mdo;
  if (!map_bshd(&mq, q, p.B, p.S, p.H, D, ld_qkv) || !map_bshd(&mk, k, p.B, p.S, p.H, D, ld_qkv) ||
      !map_bshd(&mv, v, p.B, p.S, p.H, D, ld_qkv))
    return MGB_ECUDA;
  if (!(p.o_bshd ? map_bshd(&mdo, dy, p.B, p.S, p.H, D, static_cast<int64_t>(p.H) * D)
                 : map_bhsd(&mdo, dy, p.B, p.S, p.H, D)))
    return MGB_ECUDA;
  CUtensorMap mdq;  // fp32 (B,S,H,D) accumulator, boxes of [128 rows][32 floats]
  {
    const uint64_t dims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(p.H), static_cast<uint64_t>(p.S),
                              static_cast<uint64_t>(p.B)};
    const uint64_t strides[3] = {static_cast<uint64_t>(D) * 4, static_cast<uint64_t>(p.H) * D * 4,
                                 static_cast<uint64_t>(p.S) * p.H * D * 4};
    const uint32_t box[4] = {32, 1, 128, 1};
    if (!encode_tmap_f32(&mdq, p.dq_acc, 4, dims, strides, box)) return MGB_ECUDA;
  }
  CUtensorMap mdk, mdv;  // dK / dV leave through the TMA unit too
  if (!map_bshd(&mdk, p.dk, p.B, p.S, p.H, D, p.ld_dqkv) || !map_bshd(&mdv, p.dv, p.B, p.S, p.H, D, p.ld_dqkv))
    return MGB_ECUDA;
  auto kern = p.bias ? attn_bwd_tc_kernel<D, T, true> : attn_bwd_tc_kernel<D, T, false>;
  int rc = set_smem(kern, C::SMEM);
  if (rc != MGB_OK) return rc;
  const unsigned nkt = static_cast<unsigned>((p.S + 127) / 128), nbh = static_cast<unsigned>(p.B * p.H);
  dim3 grid(D == 128 ? nbh : nkt, D == 128 ? nkt : nbh);
  launch_pdl(kern, grid, dim3(C::THREADS), C::SMEM, st, mq, mk, mv, mdo, mdq, mdk, mdv, p);
  return check_launch("attn_bwd_tc_kernel");
}

template <typename T>
int run_fwd128x2(const void* q, const void* k, const void* v, AttnParams p, int64_t ld_qkv, cudaStream_t st) {
  using C = Fwd128Cfg;
  CUtensorMap mq, mk, mv;
  if (!map_bshd(&mq, q, p.B, p.S, p.H, 128, ld_qkv) || !map_bshd(&mk, k, p.B, p.S, p.H, 128, ld_qkv) ||
      !map_bshd(&mv, v, p.B, p.S, p.H, 128, ld_qkv))
    return MGB_ECUDA;
  CUtensorMap mo;
  if (!(p.o_bshd ? map_bshd(&mo, p.out, p.B, p.S, p.H, 128, static_cast<int64_t>(p.H) * 128)
                 : map_bhsd(&mo, p.out, p.B, p.S, p.H, 128)))
    return MGB_ECUDA;
  auto kern = p.bias ? attn_fwd_tc128x2_kernel<T, true> : attn_fwd_tc128x2_kernel<T, false>;
  int rc = set_smem(kern, C::SMEM);
  if (rc != MGB_OK) return rc;
  const int nq = (p.S + 127) / 128;
  dim3 grid(static_cast<unsigned>((nq + 1) / 2), static_cast<unsigned>(p.B * p.H));
  launch_pdl(kern, grid, dim3(C::THREADS), C::SMEM, st, mq, mk, mv, mo, p);
  return check_launch("attn_fwd_tc128x2_kernel");
}

template <typename T>
int run_fwd64(const void* q, const void* k, const void* v, AttnParams p, int64_t ld_qkv, cudaStream_t st) {
  using C = Fwd64Cfg;
  CUtensorMap mq, mk, mv;
  if (!map_bshd(&mq, q, p.B, p.S, p.H, 64, ld_qkv) || !map_bshd(&mk, k, p.B, p.S, p.H, 64, ld_qkv) ||
      !map_bshd(&mv, v, p.B, p.S, p.H, 64, ld_qkv))
    return MGB_ECUDA;
  CUtensorMap mo;
  if (!(p.o_bshd ? map_bshd(&mo, p.out, p.B, p.S, p.H, 64, static_cast<int64_t>(p.H) * 64)
                 : map_bhsd(&mo, p.out, p.B, p.S, p.H, 64)))
    return MGB_ECUDA;
  auto kern = p.bias ? attn_fwd_tc64_kernel<T, true> : attn_fwd_tc64_kernel<T, false>;
  int rc = set_smem(kern, C::SMEM);
  if (rc != MGB_OK) return rc;
  const int64_t items = static_cast<int64_t>((p.S + 127) / 128) * p.B * p.H;
  MGB_REQUIRE(items <= (int64_t{1} << 30), MGB_EUNSUPPORTED, "flash_attn_fwd: %lld query tiles exceed 2^30",
              static_cast<long long>(items));
  const int ctas = static_cast<int>(std::min<int64_t>(items, 2 * static_cast<int64_t>(sm_count())));
  launch_pdl(kern, dim3(static_cast<unsigned>(ctas)), dim3(C::THREADS), C::SMEM, st, mq, mk, mv, mo, p);
  return check_launch("attn_fwd_tc64_kernel");
}

void set_bias(AttnParams& p, const void* bias, int S, float scale) {
  p.bias = static_cast<const bf16*>(bias);
  p.inv_scale = scale != 0.f ? 1.f / scale : 0.f;
  p.bias_vec = (S % 8 == 0) && aligned16(bias);
}

}  // namespace

bool tc_supported(int D, const Layouts& lay, const void* const* ptrs, int nptrs) {
  if (D != 64 && D != 128) return false;
  if (lay.ld_qkv % 8 != 0 || lay.ld_dqkv % 8 != 0) return false;
  for (int i = 0; i < nptrs; ++i)
    if (!aligned16(ptrs[i])) return false;
  return true;
}

int tc_fwd(const void* q, const void* k, const void* v, void* dst, float* lse, int B, int S, int H, int D, float scale,
           int causal, int f16, const void* bias, const Layouts& lay, cudaStream_t st) {
  AttnParams p{};
  set_bias(p, bias, S, scale);
  p.out = static_cast<bf16*>(dst);
  p.lse_out = lse;
  p.B = B, p.S = S, p.H = H, p.scale = scale, p.causal = causal;
  p.o_bshd = lay.o_bshd;
  p.status = device_status_ptr();
  if (!p.status) return fail(MGB_ECUDA, "flash_attn_fwd: device status word unavailable");
  MGB_REQUIRE(static_cast<int64_t>(B) * H <= 65535, MGB_EUNSUPPORTED, "flash_attn_fwd: B*H=%d exceeds 65535", B * H);
  if (f16) return D == 64 ? run_fwd64<__half>(q, k, v, p, lay.ld_qkv, st) : run_fwd128x2<__half>(q, k, v, p, lay.ld_qkv, st);
  return D == 64 ? run_fwd64<bf16>(q, k, v, p, lay.ld_qkv, st) : run_fwd128x2<bf16>(q, k, v, p, lay.ld_qkv, st);
}

int tc_bwd(const void* dy, const void* q, const void* k, const void* v, const float* lse, const float* delta,
           float* dq_acc, bool acc_zeroed, void* dq, void* dk, void* dv, int B, int S, int H, int D, float scale,
           int causal, int f16, const void* bias, const Layouts& lay, cudaStream_t st) {
  AttnParams p{};
  set_bias(p, bias, S, scale);
  p.lse = lse;
  p.delta = delta;
  p.dq_acc = dq_acc;
  p.dk = static_cast<bf16*>(dk);
  p.dv = static_cast<bf16*>(dv);
  p.B = B, p.S = S, p.H = H, p.scale = scale, p.causal = causal;
  p.ld_dqkv = lay.ld_dqkv;
  p.o_bshd = lay.o_bshd;
  p.status = device_status_ptr();
  if (!p.status) return fail(MGB_ECUDA, "flash_attn_bwd: device status word unavailable");
  MGB_REQUIRE(static_cast<int64_t>(B) * H <= 65535, MGB_EUNSUPPORTED, "flash_attn_bwd: B*H=%d exceeds 65535", B * H);
  const int64_t n = static_cast<int64_t>(B) * S * H * D;
  if (!acc_zeroed) {
    const cudaError_t e = cudaMemsetAsync(dq_acc, 0, static_cast<size_t>(n) * sizeof(float), st);
    if (e != cudaSuccess) return fail(MGB_ECUDA, "flash_attn_bwd: memset of the dQ accumulator: %s", cudaGetErrorString(e));
  }
  int rc;
  if (f16)
    rc = D == 64 ? run_bwd<64, __half>(dy, q, k, v, p, lay.ld_qkv, st) : run_bwd<128, __half>(dy, q, k, v, p, lay.ld_qkv, st);
  else
    rc = D == 64 ? run_bwd<64, bf16>(dy, q, k, v, p, lay.ld_qkv, st) : run_bwd<128, bf16>(dy, q, k, v, p, lay.ld_qkv, st);
  if (rc != MGB_OK) return rc;
  const int64_t n8 = n / 8;
  int grid = static_cast<int>((n8 + 255) / 256);
  if (grid > sm_count() * 8) grid = sm_count() * 8;
  if (f16)
    launch_pdl(cast_dq_kernel<__half>, dim3(grid), dim3(256), 0, st, dq_acc, static_cast<bf16*>(dq), n8, H * D / 8,
               lay.ld_dqkv, scale);
  else
    launch_pdl(cast_dq_kernel<bf16>, dim3(grid), dim3(256), 0, st, dq_acc, static_cast<bf16*>(dq), n8, H * D / 8,
               lay.ld_dqkv, scale);
  return check_launch("cast_dq_kernel");
}

}  // namespace attn
}  // namespace mgb
