// matmul_bias_bt forward and its backward (dX, dW, db).
//
// 16-bit path (bf16 or fp16 storage: a template parameter T that selects the
// operand format of the MMAs and the conversions in the epilogue; pointers to
// 16-bit tensors are typed bf16* throughout, they are only used for
// addressing): one persistent, warp-specialised tcgen05 kernel computes
//     D[i,j] = sum_l A(i,l) * B(j,l)      (fp32 accumulation in TMEM)
// for the three products of a Linear layer, which differ only in which
// operand is K-major (contraction index contiguous in memory) or MN-major:
//     Y  = X  . W^T : A = X  (K-major),  B = W (K-major)
//     dX = dY . W   : A = dY (K-major),  B = W viewed [k][n] (MN-major)
//     dW = dY^T . X : A = dY viewed [n][m] (MN-major), B = X viewed [k][m] (MN-major)
// so no operand is ever transposed in memory.  Per CTA: warp 0 issues TMA
// loads of 128-byte-swizzled tiles into a shared-memory ring, warp 1 issues
// UMMA 128xBNx16 instructions into one of two TMEM accumulators, warps 2-9
// drain the other accumulator (tcgen05.ld -> bias / ReLU -> bf16 -> global),
// so the epilogue of tile t overlaps the main loop of tile t+1.  Tiles whose
// output is small next to the contraction length (dW) are split along the
// contraction; the fp32 partial tiles go to the workspace and a finalize
// kernel adds them in a fixed order.
//
// f32 path and bf16 operands that TMA cannot address (leading dimension not a
// multiple of 8 elements, unaligned base): a shared-memory tiled CUDA-core
// kernel with fp32 accumulation.
#include "common.cuh"
#include "sm100.cuh"

namespace mgb {
namespace {

using namespace sm100;
using bf16 = __nv_bfloat16;

constexpr int BM = 128;
constexpr int BK = 64;     // bf16 elements per stage along the contraction = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int kGemmThreads = 448;  // warp 0 TMA, 1 MMA, 2-9 epilogue, 10-13 column sums of A (db)
constexpr int kMaxSplits = 16;

enum : int { kErrTmaWait = 101, kErrMmaWait = 102, kErrEpiWait = 103 };

// One element of a 16-bit tensor of storage type T, addressed through the untyped bf16* the parameters carry.
template <typename T>
__device__ __forceinline__ float ld16(const bf16* p) {
  return to_f32(*reinterpret_cast<const T*>(p));
}
template <typename T>
__device__ __forceinline__ void st16(bf16* p, float v) {
  *reinterpret_cast<T*>(p) = from_f32<T>(v);
}

template <int BN>
struct Tile {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int STG_BYTES = 2 * 128 * 128;  // two [128][64] bf16 output boxes, one per column half
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STG_BYTES + BAR_BYTES + 1024;  // + alignment slack
  static constexpr int TMEM_COLS = 2 * BN;
};

struct GemmParams {
  int M, N, K;                 // D is M x N, contraction length K
  int num_m, num_n, num_kb;    // tile counts
  int splits, kb_per_split;
  bf16* d;                     // output when splits == 1
  int64_t ldd;
  float* partial;              // [splits][M][N] when splits > 1
  const bf16* bias;            // length N or nullptr (splits == 1 only)
  int act;                     // 1 = ReLU
  const bf16* relu_mask;       // optional M x N: output zeroed where mask <= 0 (ReLU backward), splits == 1 only
  int64_t ldm;
  const bf16* residual;        // optional M x N added last (may alias d), splits == 1 only
  int64_t ldr;
  uint32_t* bits_out;          // optional [M][ldbits]: bit c%32 of word c/32 = (value after bias and ReLU) > 0
  const uint32_t* bits_in;     // optional, same layout: the output is zeroed where the bit is clear (ReLU backward)
  int64_t ldbits;
  float* rowsum_partial;       // optional [splits][M]: sum over the contraction of A(i, :) (db inside the dW GEMM)
  int d_vec;                   // output (or fp32 partial) rows take aligned 16-byte stores: staged epilogue
  int stream_out;              // the output is larger than L2 can keep for its consumer
  int n_fastest;               // tile order: consecutive tiles walk the N blocks of one M block (else the M blocks of one N block)
  int* status;
};

// Tile index -> block coordinates.  CTAs that run at the same time hold consecutive tile indices, so the order
// decides which operand panels they share through L2: walking M first shares one B panel among all CTAs and
// streams A; walking N first shares each A panel among the CTAs of its row of tiles and keeps all of B hot.
__device__ __forceinline__ void tile_coords(const GemmParams& p, int rem, int& m_blk, int& n_blk) {
  if (p.n_fastest) {
    m_blk = rem / p.num_n;
    n_blk = rem - m_blk * p.num_n;
  } else {
    n_blk = rem / p.num_m;
    m_blk = rem - n_blk * p.num_m;
  }
}

// Where one epilogue warp puts its part of the output tile.
struct EpilogueOut {
  bool vec;            // staged path: rows leave as whole 128-byte lines
  unsigned char* stg;  // this column-half's [128 rows][128 bytes] staging box; a warp only touches its own 32 rows
  int m0;              // first output row of this CTA's 128-row tile
  int lane;
  uint64_t policy;
};

// Drains one half (chalf) of a 128 x BN fp32 accumulator: TMEM -> registers -> (+ bias, ReLU, ReLU-backward
// mask, + residual) -> bf16.  TMEM gives each thread one row, which is the worst shape for global stores, so on
// the staged path every warp writes its 32 rows of a 64-column box into its own 4 KB slice of shared memory
// (128-byte swizzle, conflict-free) and reads it back four rows per instruction: each global store instruction
// then covers four whole 128-byte lines.  Only the warp itself touches its slice, so __syncwarp is the only
// synchronisation and nothing waits on an asynchronous copy.  fp32 partial tiles of a split contraction take the
// same route.  Otherwise (unaligned output) each thread stores its own row.  `row` is the output row of this
// thread, t_row the TMEM address of its lane at the accumulator's first column.
// FUSED = false compiles the elementwise epilogue (bias, ReLU, mask, residual) out: plain products keep the
// shortest possible drain loop.
template <int BN, bool FUSED, typename T>
__device__ __forceinline__ void drain_accumulator(const GemmParams& p, uint32_t t_row, int row, int n_blk, int split,
                                                  int chalf, const EpilogueOut& eo, int lane_row) {
  const bf16* const e_bias = FUSED ? p.bias : nullptr;
  const int e_act = FUSED ? p.act : 0;
  const bf16* const e_mask = FUSED ? p.relu_mask : nullptr;
  const bf16* const e_res = FUSED ? p.residual : nullptr;
  uint32_t* const e_bits_out = FUSED ? p.bits_out : nullptr;
  const uint32_t* const e_bits_in = FUSED ? p.bits_in : nullptr;
  const bool bias_vec = (reinterpret_cast<uintptr_t>(p.bias) & 15u) == 0;
  const bool mask_vec = (p.ldm & 7) == 0 && (reinterpret_cast<uintptr_t>(p.relu_mask) & 15u) == 0;
  const bool res_vec = (p.ldr & 7) == 0 && (reinterpret_cast<uintptr_t>(p.residual) & 15u) == 0;
  const bool staged = eo.vec && p.splits == 1;  // bf16 output boxes; fp32 partial boxes are handled apart
#pragma unroll 1
  for (int c0 = chalf * (BN / 2); c0 < (chalf + 1) * (BN / 2); c0 += 32) {
    const int col0 = n_blk * BN + c0;
    if (col0 >= p.N) break;  // uniform over the four warps of this half
    const int sub = (c0 >> 5) & 1;  // which 32-column half of the 64-column box
    uint32_t r[32];
    tmem_ld32(t_row + c0, r);
    // epilogue operands of this chunk are fetched while the TMEM load is in flight: 16-byte loads, the
    // bias slice is the same for every lane (one broadcast transaction)
    const bool full = col0 + 32 <= p.N;
    uint4 ep_bias[4], ep_mask[4], ep_res[4];
    if (p.splits == 1 && full && row < p.M) {
      if (e_bias && bias_vec) {
#pragma unroll
        for (int q = 0; q < 4; ++q) ep_bias[q] = __ldg(reinterpret_cast<const uint4*>(e_bias + col0) + q);
      }
      if (e_mask && mask_vec) {
        const uint4* src = reinterpret_cast<const uint4*>(e_mask + static_cast<int64_t>(row) * p.ldm + col0);
#pragma unroll
        for (int q = 0; q < 4; ++q) ep_mask[q] = __ldg(src + q);
      }
      if (e_res && res_vec) {
        const uint4* src = reinterpret_cast<const uint4*>(e_res + static_cast<int64_t>(row) * p.ldr + col0);
#pragma unroll
        for (int q = 0; q < 4; ++q) ep_res[q] = src[q];  // may alias the output: plain load
      }
    }
    uint32_t keep_bits = 0xffffffffu;
    if (e_bits_in && p.splits == 1 && row < p.M) keep_bits = __ldg(e_bits_in + static_cast<int64_t>(row) * p.ldbits + (col0 >> 5));
    tmem_ld_wait();
    if (p.splits > 1 && eo.vec) {
      // fp32 partial tile of a split contraction: this warp's [32 rows][32 floats] box goes through its own
      // shared-memory slice so that the global stores are whole 128-byte lines
      unsigned char* brow = eo.stg + lane_row * 128;
#pragma unroll
      for (int t = 0; t < 8; ++t)
        *reinterpret_cast<uint4*>(brow + ((t ^ (lane_row & 7)) << 4)) = make_uint4(r[4 * t], r[4 * t + 1], r[4 * t + 2], r[4 * t + 3]);
      __syncwarp();
      const int c = eo.lane & 7;
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int rr = (lane_row & ~31) + it * 4 + (eo.lane >> 3);
        const uint4 val = *reinterpret_cast<const uint4*>(eo.stg + rr * 128 + ((c ^ (rr & 7)) << 4));
        const int grow = eo.m0 + rr;
        if (grow < p.M && col0 + c * 4 < p.N)
          *reinterpret_cast<uint4*>(p.partial + (static_cast<int64_t>(split) * p.M + grow) * p.N + col0 + c * 4) = val;
      }
      __syncwarp();
      continue;
    }
    if (p.splits > 1) {
      if (row < p.M) {
        float* dst = p.partial + (static_cast<int64_t>(split) * p.M + row) * p.N + col0;
        if (col0 + 32 <= p.N && (p.N & 3) == 0) {
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(dst + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                              __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) dst[j] = __uint_as_float(r[j]);
        }
      }
      continue;
    }
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
    if (row < p.M) {
      if (e_bias) {
        if (full && bias_vec) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            float bv[8];
            load_vec(reinterpret_cast<const T*>(&ep_bias[j >> 3]), bv);
#pragma unroll
            for (int e = 0; e < 8; ++e) v[j + e] += bv[e];
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) v[j] += ld16<T>(e_bias + col0 + j);
        }
      }
      if (e_act == 1) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
      }
      if (e_bits_out) {
        // v >= 0 here (the entry point fixes act = ReLU), so v > 0 <=> its bit pattern is a positive integer:
        // adding 0x7fffffff carries into bit 31 exactly then, and a funnel shift appends that bit to the word
        uint32_t word = 0;
#pragma unroll
        for (int j = 0; j < 32; ++j) word = __funnelshift_l(__float_as_uint(v[j]) + 0x7fffffffu, word, 1);
        word = __brev(word);  // element j -> bit j
        if (col0 + 32 > p.N) word &= (1u << (p.N - col0)) - 1u;
        e_bits_out[static_cast<int64_t>(row) * p.ldbits + (col0 >> 5)] = word;
      }
      if (e_bits_in) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = ((keep_bits >> j) & 1u) ? v[j] : 0.f;
      }
      if (e_mask) {
        if (full && mask_vec) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            float mv[8];
            load_vec(reinterpret_cast<const T*>(&ep_mask[j >> 3]), mv);
#pragma unroll
            for (int e = 0; e < 8; ++e) v[j + e] = mv[e] > 0.f ? v[j + e] : 0.f;
          }
        } else {
          const bf16* mk = e_mask + static_cast<int64_t>(row) * p.ldm + col0;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) v[j] = ld16<T>(mk + j) > 0.f ? v[j] : 0.f;
        }
      }
      if (e_res) {
        if (full && res_vec) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            float rv[8];
            load_vec(reinterpret_cast<const T*>(&ep_res[j >> 3]), rv);
#pragma unroll
            for (int e = 0; e < 8; ++e) v[j + e] += rv[e];
          }
        } else {
          const bf16* rs = e_res + static_cast<int64_t>(row) * p.ldr + col0;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) v[j] += ld16<T>(rs + j);
        }
      }
    }
    if (staged) {
      // row lane_row of the box, 16-byte chunks (sub * 4 + t) ^ (row & 7)
      unsigned char* brow = eo.stg + lane_row * 128;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        uint4 o;
        o.x = pack_pair<T>(v[8 * t], v[8 * t + 1]);
        o.y = pack_pair<T>(v[8 * t + 2], v[8 * t + 3]);
        o.z = pack_pair<T>(v[8 * t + 4], v[8 * t + 5]);
        o.w = pack_pair<T>(v[8 * t + 6], v[8 * t + 7]);
        *reinterpret_cast<uint4*>(brow + (((sub * 4 + t) ^ (lane_row & 7)) << 4)) = o;
      }
      const bool last_of_box = sub == 1 || col0 + 32 >= p.N;
      if (last_of_box) {
        // read the warp's 32 x 64 box back four rows per instruction: every global store is a whole 128-byte line
        __syncwarp();
        const int box_col0 = col0 - sub * 32;
        const int c = eo.lane & 7;
        const bool col_ok = box_col0 + c * 8 < p.N;  // N is a multiple of 8 on this path
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int rr = (lane_row & ~31) + it * 4 + (eo.lane >> 3);
          const uint4 val = *reinterpret_cast<const uint4*>(eo.stg + rr * 128 + ((c ^ (rr & 7)) << 4));
          const int grow = eo.m0 + rr;
          if (grow < p.M && col_ok) {
            bf16* dst = p.d + static_cast<int64_t>(grow) * p.ldd + box_col0 + c * 8;
            if (p.stream_out)
              st_global_v4_hint(dst, val, eo.policy);  // larger than L2: leave first, keep the operands resident
            else
              *reinterpret_cast<uint4*>(dst) = val;
          }
        }
        __syncwarp();  // the slice may be rewritten
      }
    } else if (row < p.M) {
      bf16* dst = p.d + static_cast<int64_t>(row) * p.ldd + col0;
      if (col0 + 32 <= p.N && (p.ldd & 7) == 0 && (reinterpret_cast<uintptr_t>(p.d) & 15u) == 0) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 o;
          o.x = pack_pair<T>(v[j], v[j + 1]);
          o.y = pack_pair<T>(v[j + 2], v[j + 3]);
          o.z = pack_pair<T>(v[j + 4], v[j + 5]);
          o.w = pack_pair<T>(v[j + 6], v[j + 7]);
          *reinterpret_cast<uint4*>(dst + j) = o;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j < p.N) st16<T>(dst + j, v[j]);
      }
    }
  }
}

template <int BN, bool A_MN, bool B_MN, bool FUSED, typename T>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_tc_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                   const GemmParams p) {
  using TL = Tile<BN>;
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  const uint32_t stg_base = smem_base + TL::STAGES * TL::STAGE_BYTES;
  const uint32_t bar_base = stg_base + TL::STG_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (TL::STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * TL::STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * TL::STAGES + 2 + a); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * TL::STAGES + 4);
  unsigned char* smem_gen = smem_dyn + (smem_base - smem_u32(smem_dyn));
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + TL::STAGES * TL::STAGE_BYTES +
                                                                          TL::STG_BYTES + 8 * (2 * TL::STAGES + 4));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TL::STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), (A_MN && p.rowsum_partial) ? 5 : 1);  // MMA commit (+ the four row-sum warps)
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TL::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_gen;
  pdl_launch_dependents();  // TMEM is held: a successor can only take it over when this CTA has freed it
  pdl_wait();               // operands and outputs of earlier kernels are settled from here on

  const int tiles_mn = p.num_m * p.num_n;
  const int total = tiles_mn * p.splits;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        const int split = tile / tiles_mn;
        const int rem = tile - split * tiles_mn;
        int m_blk, n_blk;
        tile_coords(p, rem, m_blk, n_blk);
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(kb0 + p.kb_per_split, p.num_kb);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u)) {
            atomicExch(p.status, kErrTmaWait);
            ok = false;
            break;
          }
          const uint32_t sa = smem_base + stage * TL::STAGE_BYTES;
          const uint32_t sb = sa + TL::A_BYTES;
          mbar_expect_tx(full_bar(stage), TL::STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i)
              tma_load_2d(sa + i * (64 * BK * 2), &tma_a, full_bar(stage), m_blk * BM + i * 64, kb * BK);
          } else {
            tma_load_2d(sa, &tma_a, full_bar(stage), kb * BK, m_blk * BM);
          }
          if (B_MN) {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i)
              tma_load_2d(sb + i * (64 * BK * 2), &tma_b, full_bar(stage), n_blk * BN + i * 64, kb * BK);
          } else {
            tma_load_2d(sb, &tma_b, full_bar(stage), kb * BK, n_blk * BN);
          }
          if (++stage == TL::STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_16<T>(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x, ++local) {
        const int split = tile / tiles_mn;
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(kb0 + p.kb_per_split, p.num_kb);
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1u;
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u)) {
          atomicExch(p.status, kErrMmaWait);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(full_bar(stage), phase)) {
            atomicExch(p.status, kErrMmaWait);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * TL::STAGE_BYTES;
          const uint32_t sb = sa + TL::A_BYTES;
          // one descriptor per operand and stage; contraction step k adds a constant to the start-address field
          const uint64_t a0 = A_MN ? smem_desc_sw128(sa, 64 * BK * 2, 1024) : smem_desc_sw128(sa, 16, 1024);
          const uint64_t b0 = B_MN ? smem_desc_sw128(sb, 64 * BK * 2, 1024) : smem_desc_sw128(sb, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t adesc = a0 + static_cast<uint64_t>((k * (A_MN ? UMMA_K * 128 : UMMA_K * 2)) >> 4);
            const uint64_t bdesc = b0 + static_cast<uint64_t>((k * (B_MN ? UMMA_K * 128 : UMMA_K * 2)) >> 4);
            umma_ss(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));  // stage reusable once these MMAs have read it
          if (++stage == TL::STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) umma_commit(tfull_bar(acc));  // accumulator complete
      }
    }
    __syncwarp();
  } else if (warp >= 10) {
    // ------------------------------------------- row sums of A (bias gradient)
    // Only used with an MN-major A (dW = dY^T X, A = dY): every stage's A tile
    // is [BK rows of the contraction][128 output rows], so the sum over the
    // contraction of output row t is a column sum of the tile in shared memory.
    if (A_MN && p.rowsum_partial) {
      // A stage's A tile is two [BK rows][64 columns] boxes (128-byte rows, swizzled).  Lane (c << 3 | g) of warp w
      // takes the 16-byte chunk 4w + c of the eight rows g, g+8, ... (the swizzle spreads the eight rows of a
      // quarter-warp over all banks), keeps eight column sums in registers for the whole tile and folds the eight
      // row groups with three shuffles at the end: eight 16-byte loads per thread and stage, no dependent chain.
      const int wq = warp - 10;
      const int g = lane & 7;
      const int chunk16 = 4 * wq + (lane >> 3);  // 0..15 across the two boxes
      const uint32_t lane_off = (chunk16 >> 3) * (64 * BK * 2) + g * 128 + (((chunk16 & 7) ^ g) << 4);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        const int split = tile / tiles_mn;
        const int rem = tile - split * tiles_mn;
        int m_blk, n_blk;
        tile_coords(p, rem, m_blk, n_blk);
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(kb0 + p.kb_per_split, p.num_kb);
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.f;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(full_bar(stage), phase)) {
            atomicExch(p.status, kErrEpiWait);
            ok = false;
            break;
          }
          if (n_blk == 0) {
            const unsigned char* src = smem_gen + stage * TL::STAGE_BYTES + lane_off;
#pragma unroll
            for (int rr = 0; rr < BK / 8; ++rr) {
              float v[8];
              load_vec(reinterpret_cast<const T*>(src + rr * 8 * 128), v);
#pragma unroll
              for (int e = 0; e < 8; ++e) acc[e] += v[e];
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(empty_bar(stage));
          if (++stage == TL::STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok && n_blk == 0) {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 1);
            acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 2);
            acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 4);
          }
          const int row0 = m_blk * BM + chunk16 * 8;  // chunk16 * 8 = box * 64 + chunk * 8
          if (g == 0) {
            float* dst = p.rowsum_partial + static_cast<int64_t>(split) * p.M + row0;
#pragma unroll
            for (int e = 0; e < 8; ++e)
              if (row0 + e < p.M) dst[e] = acc[e];
          }
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;  // TMEM lanes this warp may read: 32*quarter .. +31
    const int chalf = (warp - 2) >> 2;  // the two warps of a lane quarter split the tile's columns
    EpilogueOut eo;
    eo.vec = p.d_vec != 0;
    eo.stg = smem_gen + TL::STAGES * TL::STAGE_BYTES + chalf * (128 * 128);
    eo.m0 = 0;
    eo.lane = lane;
    eo.policy = l2_policy_evict_first();
    int local = 0;
    for (int tile = blockIdx.x; tile < total; tile += gridDim.x, ++local) {
      const int split = tile / tiles_mn;
      const int rem = tile - split * tiles_mn;
      int m_blk, n_blk;
        tile_coords(p, rem, m_blk, n_blk);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1u;
      if (!mbar_wait(tfull_bar(acc), acc_phase)) {
        if (lane == 0) atomicExch(p.status, kErrEpiWait);
        break;
      }
      tc_fence_after();
      const int row = m_blk * BM + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      eo.m0 = m_blk * BM;
      drain_accumulator<BN, FUSED, T>(p, t_row, row, n_blk, split, chalf, eo, quarter * 32 + lane);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TL::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------------------
// CTA-pair variant for large products: a cluster of two CTAs computes a 256 x 256 tile with one
// tcgen05.mma.cta_group::2 per 16 contraction elements.  Each CTA loads only its own 128 rows of A and 128 of the
// 256 B rows per stage (32 KB instead of 48 KB for the same flops: the L2 -> SM traffic per flop drops by a
// third, which is what bounds the single-CTA kernel), keeps 128 accumulator rows in its own TMEM and drains
// them with its own 8 epilogue warps.  Rank 0 issues the MMAs; barriers: full[s] lives in rank 0 and counts the
// bytes of both CTAs' loads; empty[s] and tfull[a] exist in both CTAs and get one commit each; tempty[a] lives
// in rank 0 and collects the 16 epilogue warps of the pair.
struct Tile2 {
  static constexpr int BN = 256;
  static constexpr int A_BYTES = 128 * BK * 2;
  static constexpr int B_BYTES = 128 * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = 6;
  static constexpr int STG_BYTES = 2 * 128 * 128;
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STG_BYTES + BAR_BYTES + 1024;
  static constexpr int TMEM_COLS = 2 * BN;
};

template <bool A_MN, bool B_MN, bool FUSED, typename T>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
    gemm_tc2_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    const GemmParams p) {
  using TL = Tile2;
  constexpr int BN = TL::BN;
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  const uint32_t stg_base = smem_base + TL::STAGES * TL::STAGE_BYTES;
  const uint32_t bar_base = stg_base + TL::STG_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (TL::STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * TL::STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * TL::STAGES + 2 + a); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * TL::STAGES + 4);
  unsigned char* smem_gen = smem_dyn + (smem_base - smem_u32(smem_dyn));
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + TL::STAGES * TL::STAGE_BYTES +
                                                                          TL::STG_BYTES + 8 * (2 * TL::STAGES + 4));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();

  if (threadIdx.x == 0) {
    for (int s = 0; s < TL::STAGES; ++s) {
      mbar_init(full_bar(s), 1);   // rank 0: its producer's arrive.expect_tx (bytes of both CTAs)
      mbar_init(empty_bar(s), 1);  // one MMA commit
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 16);              // rank 0: 8 epilogue warps of each CTA
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_2cta(tmem_slot, TL::TMEM_COLS);
    tmem_relinquish_2cta();
  }
  tc_fence_before();
  cluster_sync_all();  // barriers of both CTAs are initialised before any remote arrival
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_gen;
  pdl_launch_dependents();
  pdl_wait();

  const int tiles_mn = p.num_m * p.num_n;  // num_m counts 256-row blocks here
  const int total = tiles_mn * p.splits;
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < total && ok; tile += num_clusters) {
        const int split = tile / tiles_mn;
        const int rem = tile - split * tiles_mn;
        int m_blk, n_blk;
        tile_coords(p, rem, m_blk, n_blk);
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(kb0 + p.kb_per_split, p.num_kb);
        const int m0 = m_blk * 256 + static_cast<int>(rank) * 128;
        const int n0 = n_blk * 256 + static_cast<int>(rank) * 128;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u)) {
            atomicExch(p.status, kErrTmaWait);
            ok = false;
            break;
          }
          const uint32_t sa = smem_base + stage * TL::STAGE_BYTES;
          const uint32_t sb = sa + TL::A_BYTES;
          const uint32_t full0 = map_to_cta(full_bar(stage), 0);
          if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * TL::STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int i = 0; i < 2; ++i) tma_load_2d_2cta(sa + i * (64 * BK * 2), &tma_a, full0, m0 + i * 64, kb * BK);
          } else {
            tma_load_2d_2cta(sa, &tma_a, full0, kb * BK, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int i = 0; i < 2; ++i) tma_load_2d_2cta(sb + i * (64 * BK * 2), &tma_b, full0, n0 + i * 64, kb * BK);
          } else {
            tma_load_2d_2cta(sb, &tma_b, full0, kb * BK, n0);
          }
          if (++stage == TL::STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer (rank 0 only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma_idesc_16<T>(256, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < total && ok; tile += num_clusters, ++local) {
        const int split = tile / tiles_mn;
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(kb0 + p.kb_per_split, p.num_kb);
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1u;
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u)) {
          atomicExch(p.status, kErrMmaWait);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(full_bar(stage), phase)) {
            atomicExch(p.status, kErrMmaWait);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * TL::STAGE_BYTES;
          const uint32_t sb = sa + TL::A_BYTES;
          const uint64_t a0 = A_MN ? smem_desc_sw128(sa, 64 * BK * 2, 1024) : smem_desc_sw128(sa, 16, 1024);
          const uint64_t b0 = B_MN ? smem_desc_sw128(sb, 64 * BK * 2, 1024) : smem_desc_sw128(sb, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t adesc = a0 + static_cast<uint64_t>((k * (A_MN ? UMMA_K * 128 : UMMA_K * 2)) >> 4);
            const uint64_t bdesc = b0 + static_cast<uint64_t>((k * (B_MN ? UMMA_K * 128 : UMMA_K * 2)) >> 4);
            umma_ss_2cta(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit_2cta(map_to_cta(empty_bar(stage), 0));  // both CTAs may refill this stage
          umma_commit_2cta(map_to_cta(empty_bar(stage), 1));
          if (++stage == TL::STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) {
          umma_commit_2cta(map_to_cta(tfull_bar(acc), 0));  // accumulator complete in both CTAs
          umma_commit_2cta(map_to_cta(tfull_bar(acc), 1));
        }
      }
    }
    __syncwarp();
  } else if (warp >= 10) {
    // the bias-gradient row sums are only fused into the single-CTA kernel: a CTA of rank 1 cannot poll the
    // full barrier, which lives in rank 0
  } else {
    // ---------------------------------------------------------------- epilogue (both CTAs)
    const int quarter = warp & 3;
    const int chalf = (warp - 2) >> 2;
    EpilogueOut eo;
    eo.vec = p.d_vec != 0;
    eo.stg = smem_gen + TL::STAGES * TL::STAGE_BYTES + chalf * (128 * 128);
    eo.m0 = 0;
    eo.lane = lane;
    eo.policy = l2_policy_evict_first();
    int local = 0;
    for (int tile = cluster_id; tile < total; tile += num_clusters, ++local) {
      const int split = tile / tiles_mn;
      const int rem = tile - split * tiles_mn;
      int m_blk, n_blk;
        tile_coords(p, rem, m_blk, n_blk);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1u;
      if (!mbar_wait(tfull_bar(acc), acc_phase)) {
        if (lane == 0) atomicExch(p.status, kErrEpiWait);
        break;
      }
      tc_fence_after();
      const int row = m_blk * 256 + static_cast<int>(rank) * 128 + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      eo.m0 = m_blk * 256 + static_cast<int>(rank) * 128;
      drain_accumulator<BN, FUSED, T>(p, t_row, row, n_blk, split, chalf, eo, quarter * 32 + lane);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  cluster_sync_all();  // no CTA retires while its peer may still signal its barriers or read its shared memory
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_2cta(tmem_base, TL::TMEM_COLS);
  }
}

// out[r][c] = T(sum_s partial[s][r][c]) (+ bias[c], ReLU); fixed summation order.
// VEC: four columns per thread (N, ldd multiples of 4, 8-byte aligned output), 32-bit indices.
template <bool VEC, typename T>
__global__ void __launch_bounds__(256)
    splitk_finalize_kernel(const float* __restrict__ partial, int splits, int M, int N, bf16* __restrict__ out,
                           int64_t ldd, const bf16* __restrict__ bias, int act) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t total = static_cast<int64_t>(M) * N;
  if (VEC) {
    const int n4 = N >> 2;
    const int total4 = static_cast<int>(total >> 2);
    const float4* src = reinterpret_cast<const float4*>(partial);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += gridDim.x * blockDim.x) {
      float4 acc = src[i];
      for (int s = 1; s < splits; ++s) {
        const float4 t = src[static_cast<int64_t>(s) * total4 + i];
        acc.x += t.x;
        acc.y += t.y;
        acc.z += t.z;
        acc.w += t.w;
      }
      const int r = i / n4, c = (i - r * n4) << 2;
      if (bias) {
        acc.x += ld16<T>(bias + c);
        acc.y += ld16<T>(bias + c + 1);
        acc.z += ld16<T>(bias + c + 2);
        acc.w += ld16<T>(bias + c + 3);
      }
      if (act == 1) {
        acc.x = fmaxf(acc.x, 0.f);
        acc.y = fmaxf(acc.y, 0.f);
        acc.z = fmaxf(acc.z, 0.f);
        acc.w = fmaxf(acc.w, 0.f);
      }
      uint2 o;
      o.x = pack_pair<T>(acc.x, acc.y);
      o.y = pack_pair<T>(acc.z, acc.w);
      *reinterpret_cast<uint2*>(out + static_cast<int64_t>(r) * ldd + c) = o;
    }
    return;
  }
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += partial[s * total + i];
    const int64_t r = i / N, c = i - r * N;
    if (bias) acc += ld16<T>(bias + c);
    if (act == 1) acc = fmaxf(acc, 0.f);
    st16<T>(out + r * ldd + c, acc);
  }
}

// db[i] = sum_s rowsum_partial[s][i], fixed order.
template <typename T>
__global__ void __launch_bounds__(256)
    rowsum_finalize_kernel(const float* __restrict__ partial, int splits, int M, bf16* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i >= M) return;
  float acc = 0.f;
  for (int s = 0; s < splits; ++s) acc += partial[static_cast<int64_t>(s) * M + i];
  st16<T>(out + i, acc);
}

// ------------------------------------------------------- CUDA-core fallback
// D[i,j] = sum_l A[i*sai + l*sal] * B[j*sbj + l*sbl] (+ bias[j], ReLU), fp32 accumulation.
template <typename T>
__global__ void __launch_bounds__(256)
    gemm_simt_kernel(const T* __restrict__ a, const T* __restrict__ b, const T* __restrict__ bias, T* d, int M, int N,
                     int K, int64_t sai, int64_t sal, int64_t sbj, int64_t sbl, int64_t ldd, int act,
                     const T* __restrict__ relu_mask, int64_t ldm, const T* residual, int64_t ldr) {
  constexpr int TM = 64, TN = 64, TK = 16;
  __shared__ float As[TK][TM + 1];
  __shared__ float Bs[TK][TN + 1];
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int i0 = blockIdx.y * TM, j0 = blockIdx.x * TN;
  float acc[4][4] = {};
  for (int l0 = 0; l0 < K; l0 += TK) {
    for (int e = threadIdx.x; e < TM * TK; e += 256) {
      // consecutive threads walk whichever index is contiguous in memory
      int i, l;
      if (sal == 1) {
        l = e % TK;
        i = e / TK;
      } else {
        i = e % TM;
        l = e / TM;
      }
      const int gi = i0 + i, gl = l0 + l;
      As[l][i] = (gi < M && gl < K) ? to_f32(a[gi * sai + gl * sal]) : 0.f;
    }
    for (int e = threadIdx.x; e < TN * TK; e += 256) {
      int j, l;
      if (sbl == 1) {
        l = e % TK;
        j = e / TK;
      } else {
        j = e % TN;
        l = e / TN;
      }
      const int gj = j0 + j, gl = l0 + l;
      Bs[l][j] = (gj < N && gl < K) ? to_f32(b[gj * sbj + gl * sbl]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int l = 0; l < TK; ++l) {
      float av[4], bv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        av[u] = As[l][ty * 4 + u];
        bv[u] = Bs[l][tx * 4 + u];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int v = 0; v < 4; ++v) acc[u][v] = fmaf(av[u], bv[v], acc[u][v]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int gi = i0 + ty * 4 + u;
    if (gi >= M) continue;
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const int gj = j0 + tx * 4 + v;
      if (gj >= N) continue;
      float r = acc[u][v];
      if (bias) r += to_f32(bias[gj]);
      if (act == 1) r = fmaxf(r, 0.f);
      if (relu_mask && !(to_f32(relu_mask[static_cast<int64_t>(gi) * ldm + gj]) > 0.f)) r = 0.f;
      if (residual) r += to_f32(residual[static_cast<int64_t>(gi) * ldr + gj]);
      d[static_cast<int64_t>(gi) * ldd + gj] = from_f32<T>(r);
    }
  }
}

// db[n] = sum_m dY[m][n]: each block owns 32 columns and all rows; fixed order.
template <typename T>
__global__ void __launch_bounds__(256)
    colsum_kernel(const T* __restrict__ dy, T* __restrict__ db, int M, int N, int64_t ld) {
  __shared__ float red[8][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + cx;
  float acc = 0.f;
  if (col < N)
    for (int m = ry; m < M; m += 8) acc += to_f32(dy[static_cast<int64_t>(m) * ld + col]);
  red[ry][cx] = acc;
  __syncthreads();
  if (ry == 0 && col < N) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += red[i][cx];
    db[col] = from_f32<T>(s);
  }
}

// ------------------------------------------------------------------- host
struct Operand {
  const void* ptr;
  int64_t rows;   // number of rows in memory
  int64_t cols;   // contiguous extent
  int64_t ld;     // row stride in elements
};

// What happens to the accumulator on its way out: (+ bias) -> ReLU -> ReLU-backward mask -> + residual.
struct Epilogue {
  const void* bias = nullptr;
  int act = 0;
  const void* relu_mask = nullptr;
  int64_t ldm = 0;
  const void* residual = nullptr;
  int64_t ldr = 0;
  uint32_t* bits_out = nullptr;
  const uint32_t* bits_in = nullptr;
  int64_t ldbits = 0;
};

bool tma_ok(const Operand& o) { return aligned16(o.ptr) && (o.ld % 8 == 0) && o.ld >= o.cols; }

// Map over a row-major bf16 matrix; box = box_cols x box_rows.
bool make_map(CUtensorMap* m, const Operand& o, uint32_t box_cols, uint32_t box_rows) {
  const uint64_t dims[2] = {static_cast<uint64_t>(o.cols), static_cast<uint64_t>(o.rows)};
  const uint64_t strides[1] = {static_cast<uint64_t>(o.ld) * 2};
  const uint32_t box[2] = {box_cols, box_rows};
  return encode_tmap_bf16(m, o.ptr, 2, dims, strides, box);
}

size_t splitk_bytes(int64_t M, int64_t N, int splits) {
  return splits > 1 ? round_up(static_cast<size_t>(splits) * M * N * sizeof(float), 256) : 0;
}
size_t rowsum_bytes(int64_t M) { return round_up(static_cast<size_t>(kMaxSplits) * M * sizeof(float), 256); }

// Split the contraction when the output has too few tiles to fill the GPU.
// Splits of the contraction for an output of `tiles` tiles on `slots` concurrent CTAs (or CTA pairs).
int choose_splits(int64_t tiles, int64_t K, int slots) {
  const int64_t num_kb = (K + BK - 1) / BK;
  if (tiles * 2 > slots || num_kb < 16) return 1;
  int64_t s = slots / tiles;
  if (s > num_kb / 8) s = num_kb / 8;
  if (s > kMaxSplits) s = kMaxSplits;
  return s < 1 ? 1 : static_cast<int>(s);
}

int choose_bn(int64_t N) { return N > 128 ? 256 : 128; }

template <int BN, bool A_MN, bool B_MN, bool FUSED, typename T>
int launch_tc(const Operand& a, const Operand& b, GemmParams p, cudaStream_t st) {
  using TL = Tile<BN>;
  CUtensorMap ma, mb;
  if (!make_map(&ma, a, 64, A_MN ? BK : BM)) return MGB_ECUDA;
  if (!make_map(&mb, b, 64, B_MN ? BK : BN)) return MGB_ECUDA;
  auto kern = gemm_tc_kernel<BN, A_MN, B_MN, FUSED, T>;
  static bool attr_done = false;  // per instantiation; the attribute is per function and device
  static int attr_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done || attr_dev != dev) {
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TL::SMEM_BYTES);
    if (e != cudaSuccess) return fail(MGB_ECUDA, "gemm smem opt-in (%d B): %s", TL::SMEM_BYTES, cudaGetErrorString(e));
    attr_done = true;
    attr_dev = dev;
  }
  const int total = p.num_m * p.num_n * p.splits;
  const int grid = total < sm_count() ? total : sm_count();
  launch_pdl(kern, dim3(grid), dim3(kGemmThreads), TL::SMEM_BYTES, st, ma, mb, p);
  return check_launch("gemm_tc_kernel");
}

template <bool A_MN, bool B_MN, bool FUSED, typename T>
int launch_tc2(const Operand& a, const Operand& b, GemmParams p, cudaStream_t st) {
  using TL = Tile2;
  CUtensorMap ma, mb;
  if (!make_map(&ma, a, 64, A_MN ? BK : 128)) return MGB_ECUDA;
  if (!make_map(&mb, b, 64, B_MN ? BK : 128)) return MGB_ECUDA;
  auto kern = gemm_tc2_kernel<A_MN, B_MN, FUSED, T>;
  static bool attr_done = false;
  static int attr_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done || attr_dev != dev) {
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TL::SMEM_BYTES);
    if (e != cudaSuccess) return fail(MGB_ECUDA, "gemm smem opt-in (%d B): %s", TL::SMEM_BYTES, cudaGetErrorString(e));
    attr_done = true;
    attr_dev = dev;
  }
  const int total = p.num_m * p.num_n * p.splits;
  // CTA pairs that can be resident at once: pairs need two SMs of one GPC, so this can be fewer than half the SMs,
  // and a pair that starts late would hold its round-robin share of the tiles back
  static int resident_by_dev[64] = {};
  int& resident = resident_by_dev[dev & 63];
  if (resident == 0) {
    cudaLaunchConfig_t occ = {};
    occ.gridDim = dim3(sm_count() / 2 * 2);
    occ.blockDim = dim3(kGemmThreads);
    occ.dynamicSmemBytes = TL::SMEM_BYTES;
    cudaLaunchAttribute ca[1];
    ca[0].id = cudaLaunchAttributeClusterDimension;
    ca[0].val.clusterDim.x = 2;
    ca[0].val.clusterDim.y = 1;
    ca[0].val.clusterDim.z = 1;
    occ.attrs = ca;
    occ.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &occ) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = sm_count() / 2;
    }
    resident = n < sm_count() / 2 ? n : sm_count() / 2;
  }
  const int max_clusters = resident;
  const int clusters = total < max_clusters ? total : max_clusters;
  launch_pdl(kern, dim3(2 * clusters), dim3(kGemmThreads), TL::SMEM_BYTES, st, ma, mb, p);
  return check_launch("gemm_tc2_kernel");
}

// D[M,N] = A . B^T style product on tensor cores; operands described as they lie in memory.
// rowsum_out (A_MN only): bf16[M] = sum over the contraction of A(i, :), produced inside the same kernel.
template <bool A_MN, bool B_MN, typename T>
int gemm_tc(const Operand& a, const Operand& b, bf16* d, int64_t ldd, const Epilogue& ep, bf16* rowsum_out, int64_t M,
            int64_t N, int64_t K, void* ws, size_t ws_bytes, bool allow_split, cudaStream_t st) {
  const int BN = choose_bn(N);
  // CTA pairs (256 x 256 tiles) for products large enough to fill the GPU with them.  Measured at 12 k-blocks per
  // tile: plain products are 2-5% faster on pairs (less L2 traffic per flop), products with an elementwise
  // epilogue 3-7% slower (the longer drain meets the cluster-wide accumulator hand-off); from 32 k-blocks on the
  // pair always wins.  db is fused only in the single-CTA kernel.
  const bool plain = !ep.relu_mask && !ep.residual && !ep.bits_out && !ep.bits_in;
  const bool may_split = allow_split && plain;
  const int64_t tiles1 = ((M + BM - 1) / BM) * ((N + BN - 1) / BN), tiles2 = ((M + 255) / 256) * ((N + 255) / 256);
  const int splits1 = may_split ? choose_splits(tiles1, K, sm_count()) : 1;
  const int splits2 = may_split ? choose_splits(tiles2, K, sm_count() / 2) : 1;
  const bool fused_ep = ep.bias || ep.act || ep.relu_mask || ep.residual || ep.bits_out || ep.bits_in;
  const bool pair = !rowsum_out && BN == 256 && M >= 512 && K >= (fused_ep ? 32 : 8) * BK &&
                    tiles2 * splits2 >= sm_count() / 4;
  const int bm = pair ? 256 : BM;
  GemmParams p{};
  p.M = static_cast<int>(M);
  p.N = static_cast<int>(N);
  p.K = static_cast<int>(K);
  p.num_m = static_cast<int>((M + bm - 1) / bm);
  p.num_n = static_cast<int>((N + BN - 1) / BN);
  p.num_kb = static_cast<int>((K + BK - 1) / BK);
  p.splits = pair ? splits2 : splits1;
  size_t ws_used = 0;
  if (rowsum_out) {  // the row-sum partials sit at the start of the workspace
    if (!ws || ws_bytes < rowsum_bytes(M)) return fail(MGB_EWORKSPACE, "gemm: workspace too small for the bias gradient");
    p.rowsum_partial = static_cast<float*>(ws);
    ws_used = rowsum_bytes(M);
  }
  if (p.splits > 1 && (!ws || ws_bytes < ws_used + splitk_bytes(M, N, p.splits))) p.splits = 1;
  p.kb_per_split = (p.num_kb + p.splits - 1) / p.splits;
  p.splits = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;  // no empty split
  {
    // DRAM bytes of the two tile orders: an operand that does not stay in L2 is re-read once per pass over it
    const double l2 = 64e6, bytes_a = 2.0 * M * K, bytes_b = 2.0 * N * K;
    const double passes_b = static_cast<double>(p.num_m) * p.num_n / (pair ? sm_count() / 2 : sm_count());
    const double m_first = bytes_b + (bytes_a <= l2 ? bytes_a : bytes_a * p.num_n);
    const double n_first = bytes_a + (bytes_b <= l2 ? bytes_b : bytes_b * (passes_b < 1 ? 1 : passes_b));
    p.n_fastest = n_first < m_first ? 1 : 0;
  }
  p.stream_out = 2.0 * M * N > 96e6 ? 1 : 0;
  p.d = d;
  p.ldd = ldd;
  p.partial = reinterpret_cast<float*>(static_cast<char*>(ws) + ws_used);
  const bf16* bias = static_cast<const bf16*>(ep.bias);
  p.bias = p.splits > 1 ? nullptr : bias;
  p.act = p.splits > 1 ? 0 : ep.act;
  p.relu_mask = static_cast<const bf16*>(ep.relu_mask);
  p.ldm = ep.ldm;
  p.residual = static_cast<const bf16*>(ep.residual);
  p.bits_out = ep.bits_out;
  p.bits_in = ep.bits_in;
  p.ldbits = ep.ldbits;
  p.ldr = ep.ldr;
  p.d_vec = p.splits == 1 ? (aligned16(d) && (ldd % 8 == 0) && (N % 8 == 0)) : (aligned16(p.partial) && (N % 4 == 0));
  p.status = device_status_ptr();
  if (!p.status) return fail(MGB_ECUDA, "gemm: device status word unavailable");
  const bool fused = p.bias || p.act || p.relu_mask || p.residual || p.bits_out || p.bits_in;
  int rc;
  if (fused)
    rc = pair ? launch_tc2<A_MN, B_MN, true, T>(a, b, p, st)
              : (BN == 256 ? launch_tc<256, A_MN, B_MN, true, T>(a, b, p, st)
                           : launch_tc<128, A_MN, B_MN, true, T>(a, b, p, st));
  else
    rc = pair ? launch_tc2<A_MN, B_MN, false, T>(a, b, p, st)
              : (BN == 256 ? launch_tc<256, A_MN, B_MN, false, T>(a, b, p, st)
                           : launch_tc<128, A_MN, B_MN, false, T>(a, b, p, st));
  if (rc != MGB_OK) return rc;
  if (p.splits > 1) {
    const int64_t total = M * N;
    const bool vec = (N % 4 == 0) && (ldd % 4 == 0) && (reinterpret_cast<uintptr_t>(d) % 8 == 0) && aligned16(p.partial) &&
                     total < (int64_t{1} << 31);
    int grid = static_cast<int>(((vec ? total / 4 : total) + 255) / 256);
    if (grid > sm_count() * 8) grid = sm_count() * 8;
    if (vec)
      launch_pdl(splitk_finalize_kernel<true, T>, dim3(grid), dim3(256), 0, st, p.partial, p.splits, p.M, p.N, d, ldd, bias, ep.act);
    else
      launch_pdl(splitk_finalize_kernel<false, T>, dim3(grid), dim3(256), 0, st, p.partial, p.splits, p.M, p.N, d, ldd, bias, ep.act);
    rc = check_launch("splitk_finalize_kernel");
    if (rc != MGB_OK) return rc;
  }
  if (rowsum_out) {
    launch_pdl(rowsum_finalize_kernel<T>, dim3((p.M + 255) / 256), dim3(256), 0, st, p.rowsum_partial, p.splits, p.M, rowsum_out);
    rc = check_launch("rowsum_finalize_kernel");
  }
  return rc;
}

template <typename T>
int gemm_simt(const T* a, const T* b, T* d, int64_t M, int64_t N, int64_t K, int64_t sai, int64_t sal, int64_t sbj,
              int64_t sbl, int64_t ldd, const Epilogue& ep, cudaStream_t st) {
  dim3 grid(static_cast<unsigned>((N + 63) / 64), static_cast<unsigned>((M + 63) / 64));
  MGB_REQUIRE(grid.y <= 65535, MGB_EUNSUPPORTED, "matmul: M=%lld too large for the CUDA-core kernel", (long long)M);
  gemm_simt_kernel<T><<<grid, 256, 0, st>>>(a, b, static_cast<const T*>(ep.bias), d, static_cast<int>(M),
                                            static_cast<int>(N), static_cast<int>(K), sai, sal, sbj, sbl, ldd, ep.act,
                                            static_cast<const T*>(ep.relu_mask), ep.ldm,
                                            static_cast<const T*>(ep.residual), ep.ldr);
  return check_launch("gemm_simt_kernel");
}

int check_dims(const char* who, int64_t M, int64_t N, int64_t K) {
  MGB_REQUIRE(M > 0 && N > 0 && K > 0, MGB_EINVAL, "%s: M=%lld N=%lld K=%lld must be positive", who, (long long)M,
              (long long)N, (long long)K);
  MGB_REQUIRE(M < (1LL << 31) && N < (1LL << 31) && K < (1LL << 31), MGB_EUNSUPPORTED, "%s: dimension exceeds 2^31",
              who);
  return MGB_OK;
}

template <typename T>
int colsum(const void* dy, void* db, int64_t M, int64_t N, int64_t ld, cudaStream_t st) {
  colsum_kernel<T><<<static_cast<unsigned>((N + 31) / 32), 256, 0, st>>>(static_cast<const T*>(dy), static_cast<T*>(db),
                                                                       static_cast<int>(M), static_cast<int>(N), ld);
  return check_launch("colsum_kernel");
}

}  // namespace
}  // namespace mgb

using namespace mgb;

namespace {
int matmul_fwd_impl(const void* a, const void* w, const void* bias, const void* residual, void* y, void* relu_bits,
                    int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldw, int64_t ldr, int64_t ldy, int64_t ld_bits,
                    int act, int dtype, void* stream) {
  MGB_REQUIRE(a && w && y, MGB_EINVAL, "matmul_bias_bt: NULL argument");
  int rc = check_dims("matmul_bias_bt", M, N, K);
  if (rc != MGB_OK) return rc;
  MGB_REQUIRE(lda >= K && ldw >= K && ldy >= N && (!residual || ldr >= N), MGB_EINVAL,
              "matmul_bias_bt: leading dimension too small");
  MGB_REQUIRE(act == 0 || act == 1, MGB_EINVAL, "matmul_bias_bt: act=%d (0 none, 1 relu)", act);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Epilogue ep;
  ep.bias = bias;
  ep.act = act;
  ep.residual = residual;
  ep.ldr = ldr;
  ep.bits_out = static_cast<uint32_t*>(relu_bits);
  ep.ldbits = ld_bits;
  const Operand oa{a, M, K, lda}, ow{w, N, K, ldw};
  const bool half16 = dtype == MGB_BF16 || dtype == MGB_F16;
  const bool tc = half16 && tma_ok(oa) && tma_ok(ow);
  MGB_REQUIRE(!relu_bits || tc, MGB_EUNSUPPORTED,
              "matmul_bias_bt_relu_bits: needs 16-bit operands with 16-byte-aligned rows (the tensor-core path)");
  if (dtype == MGB_F32)
    return gemm_simt<float>(static_cast<const float*>(a), static_cast<const float*>(w), static_cast<float*>(y), M, N, K,
                            lda, 1, ldw, 1, ldy, ep, st);
  MGB_REQUIRE(half16, MGB_EDTYPE, "matmul_bias_bt: unsupported dtype code %d", dtype);
  if (dtype == MGB_F16) {
    if (tc)
      return gemm_tc<false, false, __half>(oa, ow, static_cast<bf16*>(y), ldy, ep, nullptr, M, N, K, nullptr, 0, false, st);
    return gemm_simt<__half>(static_cast<const __half*>(a), static_cast<const __half*>(w), static_cast<__half*>(y), M, N,
                             K, lda, 1, ldw, 1, ldy, ep, st);
  }
  if (tc) return gemm_tc<false, false, bf16>(oa, ow, static_cast<bf16*>(y), ldy, ep, nullptr, M, N, K, nullptr, 0, false, st);
  return gemm_simt<bf16>(static_cast<const bf16*>(a), static_cast<const bf16*>(w), static_cast<bf16*>(y), M, N, K, lda,
                         1, ldw, 1, ldy, ep, st);
}
}  // namespace

MGB_EXPORT int mograd_b200_matmul_bias_bt_ex(const void* a, const void* w, const void* bias, const void* residual,
                                             void* y, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldw,
                                             int64_t ldr, int64_t ldy, int act, int dtype, void* stream) {
  return matmul_fwd_impl(a, w, bias, residual, y, nullptr, M, N, K, lda, ldw, ldr, ldy, 0, act, dtype, stream);
}

MGB_EXPORT int mograd_b200_matmul_bias_bt_relu_bits(const void* a, const void* w, const void* bias, void* y,
                                                    void* relu_bits, int64_t M, int64_t N, int64_t K, int64_t lda,
                                                    int64_t ldw, int64_t ldy, int64_t ld_bits, int dtype, void* stream) {
  MGB_REQUIRE(relu_bits, MGB_EINVAL, "matmul_bias_bt_relu_bits: relu_bits is NULL");
  MGB_REQUIRE(ld_bits >= (N + 31) / 32, MGB_EINVAL, "matmul_bias_bt_relu_bits: ld_bits=%lld < ceil(N/32)", (long long)ld_bits);
  return matmul_fwd_impl(a, w, bias, nullptr, y, relu_bits, M, N, K, lda, ldw, 0, ldy, ld_bits, 1, dtype, stream);
}

MGB_EXPORT int mograd_b200_matmul_bias_bt(const void* a, const void* w, const void* bias, void* y, int64_t M,
                                          int64_t N, int64_t K, int64_t lda, int64_t ldw, int64_t ldy, int act,
                                          int dtype, void* stream) {
  return mograd_b200_matmul_bias_bt_ex(a, w, bias, nullptr, y, M, N, K, lda, ldw, 0, ldy, act, dtype, stream);
}

MGB_EXPORT size_t mograd_b200_matmul_bias_bt_bwd_workspace_bytes(int64_t M, int64_t N, int64_t K, int dtype) {
  if ((dtype != MGB_BF16 && dtype != MGB_F16) || M <= 0 || N <= 0 || K <= 0) return 0;
  // dW is N x K with contraction M (may be split); db partials ride along.  dX (contraction N) is never split.
  return rowsum_bytes(N) + splitk_bytes(N, K, kMaxSplits);
}

namespace {
// dX, dW, db of a 16-bit (bf16 / fp16) Linear layer: tensor cores where TMA can address the operands, the CUDA-core
// kernel otherwise.
template <typename T>
int matmul_bwd_16(const void* dy, const void* x, const void* w, const Epilogue& epx, void* dx, void* dw, void* db,
                  int64_t M, int64_t N, int64_t K, int64_t lddy, int64_t ldx, int64_t ldw, int64_t lddx, int64_t lddw,
                  void* workspace, size_t workspace_bytes, cudaStream_t st) {
  int rc = MGB_OK;
  const Epilogue none;
  const T* dyb = static_cast<const T*>(dy);
  const Operand ody{dy, M, N, lddy};
  if (dx) {
    const Operand ow{w, N, K, ldw};
    if (tma_ok(ody) && tma_ok(ow))
      rc = gemm_tc<false, true, T>(ody, ow, static_cast<bf16*>(dx), lddx, epx, nullptr, M, K, N, nullptr, 0, false, st);
    else
      rc = gemm_simt<T>(dyb, static_cast<const T*>(w), static_cast<T*>(dx), M, K, N, lddy, 1, 1, ldw, lddx, epx, st);
    if (rc != MGB_OK) return rc;
  }
  bool db_done = false;
  if (dw) {
    const Operand ox{x, M, K, ldx};
    if (tma_ok(ody) && tma_ok(ox)) {
      // db comes out of the same kernel when the workspace has room for its partial sums
      bf16* db_fused = (db && workspace && workspace_bytes >= rowsum_bytes(N)) ? static_cast<bf16*>(db) : nullptr;
      rc = gemm_tc<true, true, T>(ody, ox, static_cast<bf16*>(dw), lddw, none, db_fused, N, K, M, workspace,
                                  workspace_bytes, true, st);
      db_done = db_fused != nullptr;
    } else {
      rc = gemm_simt<T>(dyb, static_cast<const T*>(x), static_cast<T*>(dw), N, K, M, 1, lddy, 1, ldx, lddw, none, st);
    }
    if (rc != MGB_OK) return rc;
  }
  if (db && !db_done) rc = colsum<T>(dy, db, M, N, lddy, st);
  return rc;
}

int matmul_bwd_impl(const void* dy, const void* x, const void* w, const void* relu_y, const void* relu_bits,
                    const void* dx_residual, void* dx, void* dw, void* db, int64_t M, int64_t N, int64_t K, int64_t lddy,
                    int64_t ldx, int64_t ldw, int64_t ld_relu_y, int64_t ld_bits, int64_t ld_dx_residual, int64_t lddx,
                    int64_t lddw, int dtype, void* workspace, size_t workspace_bytes, void* stream) {
  MGB_REQUIRE(dy, MGB_EINVAL, "matmul_bias_bt_bwd: dy is NULL");
  MGB_REQUIRE(dx || dw || db, MGB_EINVAL, "matmul_bias_bt_bwd: no output requested");
  MGB_REQUIRE(!dx || w, MGB_EINVAL, "matmul_bias_bt_bwd: dX needs W");
  MGB_REQUIRE(!dw || x, MGB_EINVAL, "matmul_bias_bt_bwd: dW needs X");
  int rc = check_dims("matmul_bias_bt_bwd", M, N, K);
  if (rc != MGB_OK) return rc;
  MGB_REQUIRE(lddy >= N && (!dx || (ldw >= K && lddx >= K)) && (!dw || (ldx >= K && lddw >= K)) &&
                  (!relu_y || ld_relu_y >= K) && (!dx_residual || ld_dx_residual >= K),
              MGB_EINVAL, "matmul_bias_bt_bwd: leading dimension too small");
  MGB_REQUIRE(dtype == MGB_BF16 || dtype == MGB_F32 || dtype == MGB_F16, MGB_EDTYPE,
              "matmul_bias_bt_bwd: unsupported dtype code %d", dtype);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Epilogue epx;  // dX = (dY W) masked by relu_y > 0, plus dx_residual
  epx.relu_mask = relu_y;
  epx.ldm = ld_relu_y;
  epx.residual = dx_residual;
  epx.ldr = ld_dx_residual;
  epx.bits_in = static_cast<const uint32_t*>(relu_bits);
  epx.ldbits = ld_bits;
  if (relu_bits && dx) {
    const Operand ody0{dy, M, N, lddy}, ow0{w, N, K, ldw};
    MGB_REQUIRE(dtype != MGB_F32 && tma_ok(ody0) && tma_ok(ow0), MGB_EUNSUPPORTED,
                "matmul_bias_bt_bwd_relu_bits: needs 16-bit operands with 16-byte-aligned rows (the tensor-core path)");
  }
  const Epilogue none;
  if (dtype == MGB_F32) {
    const float* dyf = static_cast<const float*>(dy);
    if (dx) {
      // dX[m,k] = sum_n dY[m,n] W[n,k]: A = dY (i=m, l=n), B(j=k, l=n) = W[n*ldw + k]
      rc = gemm_simt<float>(dyf, static_cast<const float*>(w), static_cast<float*>(dx), M, K, N, lddy, 1, 1, ldw, lddx,
                            epx, st);
      if (rc != MGB_OK) return rc;
    }
    if (dw) {
      // dW[n,k] = sum_m dY[m,n] X[m,k]: A(i=n, l=m) = dY[m*lddy + n], B(j=k, l=m) = X[m*ldx + k]
      rc = gemm_simt<float>(dyf, static_cast<const float*>(x), static_cast<float*>(dw), N, K, M, 1, lddy, 1, ldx, lddw,
                            none, st);
      if (rc != MGB_OK) return rc;
    }
    if (db) rc = colsum<float>(dy, db, M, N, lddy, st);
    return rc;
  }
  if (dtype == MGB_F16)
    return matmul_bwd_16<__half>(dy, x, w, epx, dx, dw, db, M, N, K, lddy, ldx, ldw, lddx, lddw, workspace,
                                 workspace_bytes, st);
  return matmul_bwd_16<bf16>(dy, x, w, epx, dx, dw, db, M, N, K, lddy, ldx, ldw, lddx, lddw, workspace, workspace_bytes,
                             st);
}
}  // namespace

MGB_EXPORT int mograd_b200_matmul_bias_bt_bwd_ex(const void* dy, const void* x, const void* w, const void* relu_y,
                                                 const void* dx_residual, void* dx, void* dw, void* db, int64_t M,
                                                 int64_t N, int64_t K, int64_t lddy, int64_t ldx, int64_t ldw,
                                                 int64_t ld_relu_y, int64_t ld_dx_residual, int64_t lddx,
                                                 int64_t lddw, int dtype, void* workspace, size_t workspace_bytes,
                                                 void* stream) {
  return matmul_bwd_impl(dy, x, w, relu_y, nullptr, dx_residual, dx, dw, db, M, N, K, lddy, ldx, ldw, ld_relu_y, 0,
                         ld_dx_residual, lddx, lddw, dtype, workspace, workspace_bytes, stream);
}

MGB_EXPORT int mograd_b200_matmul_bias_bt_bwd_relu_bits(const void* dy, const void* x, const void* w,
                                                        const void* relu_bits, const void* dx_residual, void* dx,
                                                        void* dw, void* db, int64_t M, int64_t N, int64_t K,
                                                        int64_t lddy, int64_t ldx, int64_t ldw, int64_t ld_bits,
                                                        int64_t ld_dx_residual, int64_t lddx, int64_t lddw, int dtype,
                                                        void* workspace, size_t workspace_bytes, void* stream) {
  MGB_REQUIRE(relu_bits, MGB_EINVAL, "matmul_bias_bt_bwd_relu_bits: relu_bits is NULL");
  MGB_REQUIRE(ld_bits >= (K + 31) / 32, MGB_EINVAL, "matmul_bias_bt_bwd_relu_bits: ld_bits=%lld < ceil(K/32)", (long long)ld_bits);
  return matmul_bwd_impl(dy, x, w, nullptr, relu_bits, dx_residual, dx, dw, db, M, N, K, lddy, ldx, ldw, 0, ld_bits,
                         ld_dx_residual, lddx, lddw, dtype, workspace, workspace_bytes, stream);
}

MGB_EXPORT int mograd_b200_matmul_bias_bt_bwd(const void* dy, const void* x, const void* w, void* dx, void* dw,
                                              void* db, int64_t M, int64_t N, int64_t K, int64_t lddy, int64_t ldx,
                                              int64_t ldw, int64_t lddx, int64_t lddw, int dtype, void* workspace,
                                              size_t workspace_bytes, void* stream) {
  return mograd_b200_matmul_bias_bt_bwd_ex(dy, x, w, nullptr, nullptr, dx, dw, db, M, N, K, lddy, ldx, ldw, 0, 0, lddx,
                                           lddw, dtype, workspace, workspace_bytes, stream);
}
