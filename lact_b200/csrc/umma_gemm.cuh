// Batched bf16 GEMM engine for sm_100a: TMA-fed shared-memory tiles, tcgen05.mma into tensor
// memory, warp-specialised (1 TMA warp, 1 MMA warp, 4 epilogue warps), pluggable fp32 epilogue.
//
// One CTA computes one 128 x BN output tile of one batch entry of one problem:
//     acc[c] (+)= A[term_a] * B[term_b]^T          for every term of the op
// where A operands are (M x K) and B operands are (N x K), each either K-major (k contiguous
// in global memory) or MN-major (m / n contiguous).  Several terms may share operands (SwiGLU
// gate + up projection share the activations) or accumulators (split-precision products).
// Out-of-range parts of a tile are zero-filled by TMA, so ragged M, N and K need no masks in
// the main loop; the epilogue clips its stores.
#pragma once
#include "ptx.cuh"

namespace lact {

constexpr int kBM = 128;   // UMMA M (rows of the accumulator = TMEM lanes)
constexpr int kBK = 64;    // k-block: 64 bf16 = 128 bytes = one swizzle row
constexpr int kUmmaK = 16; // K of one tcgen05.mma for 16-bit operands
constexpr int kGemmThreads = 192;
constexpr uint32_t kATileBytes = kBM * kBK * 2;
constexpr uint32_t kAtomBytes = 64 * kBK * 2;  // one 64(mn) x 64(k) MN-major atom column

struct OperandInfo {
  int32_t mn_major;   // 0: global [mn][k] (k contiguous); 1: global [k][mn] (mn contiguous)
  int32_t mn_off;     // added to the mn coordinate
  int32_t k_off;      // added to the k coordinate
  int32_t batch_off;  // added to the batch coordinate
};

template <class Op>
struct GemmProblem {
  CUtensorMap a[Op::NA];
  CUtensorMap b[Op::NB];
  OperandInfo ai[Op::NA];
  OperandInfo bi[Op::NB];
  int32_t M, N, K, batch;
  typename Op::Epi ep;
};

template <class Op, int NPROB>
struct GemmArgs {
  GemmProblem<Op> prob[NPROB];
  int32_t* status;  // device status word (0 = ok)
};

__host__ __device__ constexpr uint32_t tmem_cols_pow2(uint32_t n) {
  return n <= 32 ? 32 : n <= 64 ? 64 : n <= 128 ? 128 : n <= 256 ? 256 : 512;
}

template <class Op>
__host__ __device__ constexpr uint32_t gemm_smem_bytes() {
  return Op::STAGES * (Op::NA * kATileBytes + Op::NB * Op::BN * kBK * 2) + 1024 /*alignment slack*/ + 256;
}

template <int ROWS>
__device__ __forceinline__ void load_operand_tile(uint32_t dst, const CUtensorMap* map, const OperandInfo& oi,
                                                  int mn0, int kc, int batch, uint64_t* bar) {
  if (!oi.mn_major) {
    tma_load_3d(dst, map, bar, oi.k_off + kc, oi.mn_off + mn0, oi.batch_off + batch);
  } else {
#pragma unroll
    for (int j = 0; j < ROWS / 64; ++j)
      tma_load_3d(dst + j * kAtomBytes, map, bar, oi.mn_off + mn0 + 64 * j, oi.k_off + kc, oi.batch_off + batch);
  }
}

__device__ __forceinline__ uint64_t operand_desc(uint32_t tile, int mn_major, int k4) {
  // K-major: advance 16 elements (32 bytes) inside the swizzled 128-byte row.
  // MN-major: advance 16 k-rows (2 groups of 8 rows x 128 bytes).
  return mn_major ? make_smem_desc(tile + k4 * 2048, kAtomBytes, 1024) : make_smem_desc(tile + k4 * 32, 0, 1024);
}

template <class Op, int NPROB>
__global__ void __launch_bounds__(kGemmThreads, 1)
umma_gemm_kernel(const __grid_constant__ GemmArgs<Op, NPROB> args) {
  constexpr int BN = Op::BN, NA = Op::NA, NB = Op::NB, NACC = Op::NACC, STAGES = Op::STAGES;
  constexpr uint32_t kBTileBytes = BN * kBK * 2;
  constexpr uint32_t kStageBytes = NA * kATileBytes + NB * kBTileBytes;
  constexpr uint32_t kTmemCols = tmem_cols_pow2(NACC * BN);
  static_assert(NACC * BN <= 512, "accumulators exceed tensor memory");
  static_assert(BN % 64 == 0 && BN <= 256, "BN must be 64, 128, 192 or 256");

  const GemmProblem<Op>& P = args.prob[blockIdx.z];
  const int tiles_n = (P.N + BN - 1) / BN;
  const int tiles_m = (P.M + kBM - 1) / kBM;
  if (static_cast<int>(blockIdx.x) >= tiles_m * tiles_n || static_cast<int>(blockIdx.y) >= P.batch) return;
  if (*reinterpret_cast<volatile int32_t*>(args.status) != kStatusOk) return;  // an earlier CTA gave up
  const int m0 = (blockIdx.x / tiles_n) * kBM;
  const int n0 = (blockIdx.x % tiles_n) * BN;
  const int batch = blockIdx.y;
  const int num_kb = (P.K + kBK - 1) / kBK;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t smem_base = (raw_addr + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (smem_base - raw_addr);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(aligned + STAGES * kStageBytes);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full_bar = empty_bar + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full_bar + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tmem_full_bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
#pragma unroll
    for (int i = 0; i < NA; ++i) tma_prefetch_desc(&P.a[i]);
#pragma unroll
    for (int i = 0; i < NB; ++i) tma_prefetch_desc(&P.b[i]);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  bool failed = false;
  if (warp == 0) {
    // ---------------- TMA producer
    if (lane == 0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % STAGES;
        const uint32_t ph = (kb / STAGES) & 1;
        if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag)) { failed = true; break; }
        mbar_expect_tx(&full_bar[s], kStageBytes);
        const uint32_t st = smem_base + s * kStageBytes;
        const int kc = kb * kBK;
#pragma unroll
        for (int i = 0; i < NA; ++i)
          load_operand_tile<kBM>(st + i * kATileBytes, &P.a[i], P.ai[i], m0, kc, batch, &full_bar[s]);
#pragma unroll
        for (int i = 0; i < NB; ++i)
          load_operand_tile<BN>(st + NA * kATileBytes + i * kBTileBytes, &P.b[i], P.bi[i], n0, kc, batch,
                                &full_bar[s]);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (single thread)
    if (lane == 0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % STAGES;
        const uint32_t ph = (kb / STAGES) & 1;
        if (!mbar_wait(&full_bar[s], ph, abort_flag)) { failed = true; break; }
        tc_fence_after();
        const uint32_t st = smem_base + s * kStageBytes;
#pragma unroll
        for (int t = 0; t < Op::NTERMS; ++t) {
          const int ia = Op::term_a(t), ib = Op::term_b(t), ic = Op::term_acc(t);
          const int a_mn = P.ai[ia].mn_major, b_mn = P.bi[ib].mn_major;
          const uint32_t idesc = make_idesc_bf16(kBM, BN, a_mn, b_mn);
          const uint32_t a_tile = st + ia * kATileBytes;
          const uint32_t b_tile = st + NA * kATileBytes + ib * kBTileBytes;
#pragma unroll
          for (int k4 = 0; k4 < kBK / kUmmaK; ++k4) {
            const uint32_t acc = (kb > 0 || k4 > 0 || !Op::term_first(t)) ? 1u : 0u;
            umma_bf16(tmem_base + ic * BN, operand_desc(a_tile, a_mn, k4), operand_desc(b_tile, b_mn, k4), idesc,
                      acc);
          }
        }
        umma_commit(&empty_bar[s]);  // frees the stage once these MMAs have read it
      }
      if (!failed) umma_commit(tmem_full_bar);
    }
  } else {
    // ---------------- epilogue: warp w may only touch TMEM lanes [32*(w%4), 32*(w%4)+32)
    const int quarter = warp & 3;
    const int row = m0 + quarter * 32 + lane;
    bool ok = true;
    if (num_kb > 0) {
      ok = mbar_wait(tmem_full_bar, 0, abort_flag);
      tc_fence_after();
    }
    if (ok) {
      for (int c = 0; c < BN; c += 32) {
        if (n0 + c >= P.N) break;  // warp-uniform
        float v[NACC][32];
        if (num_kb > 0) {
#pragma unroll
          for (int a = 0; a < NACC; ++a) {
            uint32_t bits[32];
            tmem_ld32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + a * BN + c, bits);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) v[a][j] = __uint_as_float(bits[j]);
          }
        } else {
#pragma unroll
          for (int a = 0; a < NACC; ++a)
#pragma unroll
            for (int j = 0; j < 32; ++j) v[a][j] = 0.f;
        }
        Op::epilogue(P.ep, batch, row, n0 + c, P.M, P.N, v);
      }
    } else {
      failed = true;
    }
  }
  if (failed) {
    *abort_flag = 1;
    atomicCAS(args.status, kStatusOk, kStatusWaitTimeout);
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    // let bulk copies still in flight land before shared memory is released
    for (int i = 0; i < 256; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace lact
