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
constexpr uint32_t kATileBytes = kBM * kBK * 2;
constexpr uint32_t kAtomBytes = 64 * kBK * 2;  // one 64(mn) x 64(k) MN-major atom column

struct OperandInfo {
  int32_t mn_major;   // 0: global [mn][k] (k contiguous); 1: global [k][mn] (mn contiguous)
  int32_t k4d;        // K-major only: the map is 4-D (64 k, rows, k-blocks, batch) and one box spans the stage's k-blocks
  int32_t mn_off;     // added to the mn coordinate
  int32_t k_off;      // added to the k coordinate
  int32_t batch_off;  // added to the batch coordinate
};

// Where a staged (TMA-stored) output tile lands: tile (m0, n0) of batch entry b is stored at
// coordinates (col_off + n0, row_off + m0, batch_off + b) of the output map, whose extents clip it.
struct OutInfo {
  int32_t row_off, col_off, batch_off, enabled;
};

template <class Op>
struct GemmProblem {
  CUtensorMap a[Op::NA];
  CUtensorMap b[Op::NB];
  CUtensorMap out[Op::NOUT > 0 ? Op::NOUT : 1];  // bf16 outputs written by TMA store (NOUT == 0: none)
  OperandInfo ai[Op::NA];
  OperandInfo bi[Op::NB];
  OutInfo oi[Op::NOUT > 0 ? Op::NOUT : 1];
  int32_t M, N, K, batch;
  typename Op::Epi ep;
};

template <class Op, int NPROB>
struct GemmArgs {
  using OpType = Op;
  GemmProblem<Op> prob[NPROB];
  int32_t* status;  // device status word (0 = ok)
};

__host__ __device__ constexpr uint32_t tmem_cols_pow2(uint32_t n) {
  return n <= 32 ? 32 : n <= 64 ? 64 : n <= 128 ? 128 : n <= 256 ? 256 : 512;
}

// An op describes the wiring of one GEMM kernel:
//   NA, NB        operand tiles loaded per pipeline stage (A tiles: 128 rows; B tiles: BT rows)
//   BT            width of the output tile in logical columns (= rows of every B operand tile)
//   NACC          accumulators handed to the epilogue, accumulator a at TMEM columns [a*BT, (a+1)*BT)
//   terms         each term issues MMAs  acc[cols term_col .. term_col + term_n) (+)= A[term_a] * B[term_b..]^T;
//                 term_n may span several consecutive B tiles (they are adjacent in shared memory)
//   STAGES        depth of the shared-memory ring
// Accumulators are double-buffered in tensor memory (2 * NACC * BT <= 512 columns), so the epilogue
// of tile i overlaps the main loop of tile i + 1.
template <class Op>
__host__ __device__ constexpr uint32_t gemm_stage_bytes() {
  return Op::KB * (Op::NA * kATileBytes + Op::NB * Op::BT * kBK * 2);
}
// bf16 staging tiles for TMA-stored outputs: NOUT x [128 rows][BT columns], 128-byte swizzled in
// 64-column panels (the layout the output tensor maps expect)
template <class Op>
__host__ __device__ constexpr uint32_t gemm_staging_bytes();
template <class Op>
__host__ __device__ constexpr uint32_t gemm_smem_bytes() {
  return Op::STAGES * gemm_stage_bytes<Op>() + gemm_staging_bytes<Op>() + 1024 /*alignment slack*/ + 256 /*barriers*/;
}

constexpr int kEpiWarps = 8;
constexpr int kGemmThreadsV2 = 64 + 32 * kEpiWarps;  // producer warp + MMA warp + epilogue warps
// dataflow kernels add a scout warp that walks the tile sequence ahead of the producer and checks
// every tile's dependency, so that the global-memory latency of that check never stalls the loads
constexpr int kGemmThreadsFlow = kGemmThreadsV2 + 64;  // + dependency scout warp + storing warp

// One operand tile of a ring stage: ROWS (mn) x KB k-blocks.  Shared-memory layout:
//   K-major:  [k-block][ROWS rows][64 k] (KB tiles of ROWS x 128 bytes back to back);
//   MN-major: per 64-wide mn atom [KB * 64 k rows][64 mn] (atoms KB * 8 KB apart).
// With KB = 2 a K-major tile arrives as one box of a 4-D map when the operand allows it (k4d), an
// MN-major tile as one 128-k-row box per atom.
template <int ROWS, int KB>
__device__ __forceinline__ void load_operand_tile(uint32_t dst, const CUtensorMap* map, const OperandInfo& oi,
                                                  int mn0, int kc, int batch, uint64_t* bar) {
  if (!oi.mn_major) {
    if (KB == 2 && oi.k4d) {
      tma_load_4d(dst, map, bar, 0, oi.mn_off + mn0, (oi.k_off + kc) / kBK, oi.batch_off + batch);
    } else {
#pragma unroll
      for (int kk = 0; kk < KB; ++kk)
        tma_load_3d(dst + kk * (ROWS * kBK * 2), map, bar, oi.k_off + kc + kk * kBK, oi.mn_off + mn0, oi.batch_off + batch);
    }
  } else {
#pragma unroll
    for (int j = 0; j < ROWS / 64; ++j)
      tma_load_3d(dst + j * (KB * kAtomBytes), map, bar, oi.mn_off + mn0 + 64 * j, oi.k_off + kc, oi.batch_off + batch);
  }
}

// Descriptor of the k-block `kk`, 16-element k-slice `k4`, of an operand tile of ROWS_BYTES = rows * 128.
template <int KB>
__device__ __forceinline__ uint64_t operand_desc(uint32_t tile, int mn_major, uint32_t rows_bytes, int kk, int k4) {
  // K-major: advance 16 elements (32 bytes) inside the swizzled 128-byte row.
  // MN-major: advance 16 k-rows (2 groups of 8 rows x 128 bytes); atoms are KB * 8 KB apart.
  return mn_major ? make_smem_desc(tile + kk * kAtomBytes + k4 * 2048, KB * kAtomBytes, 1024)
                  : make_smem_desc(tile + kk * rows_bytes + k4 * 32, 0, 1024);
}

struct TileCoord {
  int prob, batch, m0, n0;
};

// Ops whose output is a symmetric M x M matrix (both operands the same rows) may declare `kSymmetric`: only the
// 128 x 128 tiles on and above the diagonal are computed, and every off-diagonal tile is stored twice, as it is and
// transposed (from a second staging tile the epilogue fills).  Needs BT = 128, one staged output, dataflow mode.
template <class Op, class = void>
struct op_symmetric { static constexpr bool value = false; };
template <class Op>
struct op_symmetric<Op, decltype(void(Op::kSymmetric))> { static constexpr bool value = Op::kSymmetric; };

template <class Op>
__host__ __device__ constexpr uint32_t gemm_staging_bytes() {
  return (Op::NOUT + (op_symmetric<Op>::value ? 1 : 0)) * kBM * Op::BT * 2 + Op::kEpiScratch;
}

// Per-thread view of the CTA's pipeline resources and of this thread's progress counters.  The
// producer thread advances `it`, the MMA thread `it` and `tcount`, epilogue threads `tcount`;
// all three walk the same tile sequence, so their private copies stay consistent.  The counters
// run on across phases of a multi-phase kernel.
struct GemmCtx {
  uint32_t smem_base;     // 1024-byte aligned start of the stage ring
  uint32_t stage_stride;  // bytes between ring stages (>= the op's stage bytes)
  uint32_t staging;       // 1024-byte aligned start of the output staging tiles
  uint64_t *full_bar, *empty_bar, *acc_full_bar, *acc_empty_bar;
  uint64_t *stg_full_bar, *stg_empty_bar;  // dataflow kernels: staging tile handed to / returned by the storing warp
  volatile uint32_t* abort_flag;
  uint32_t tmem_base;
  uint32_t it = 0, tcount = 0;
  // dataflow mode (multi-phase kernels whose phases are ordered by completion counters, see FlowDeps)
  uint32_t rot = 0;              // tiles handed out by earlier phases, modulo the grid size
  uint32_t ptile = 0;            // tiles whose dependency has been verified (scout) / consumed (producer)
  uint32_t sround = 0;           // staging hand-overs so far (epilogue threads and the storing thread count alike)
  uint32_t* dep_ok = nullptr;    // shared-memory word: tiles verified by the scout warp, read by the producer thread
};

struct NoPatch {
  template <class Epi>
  __device__ __forceinline__ void operator()(Epi&, int) const {}
};

// Phase ordering of a multi-phase kernel without grid-wide barriers.  Every (problem, batch entry)
// owns a completion counter in global memory; a tile's stores are followed (once they have landed)
// by one increment of its batch entry's counter, and a tile of a later phase may load only after the
// counter of its batch entry has reached `need` = the number of tiles all earlier phases produce for
// that entry.  The phases of a batch entry must form a chain (each phase reads only what earlier
// phases of the same entry wrote, and overwrites only what earlier phases of the same entry read).
// All CTAs walk the phases in the same order and must be co-resident; every wait is bounded.
struct NoDeps {
  static constexpr bool kOn = false;
};
struct FlowDeps {
  static constexpr bool kOn = true;
  uint32_t* counter[2];  // per problem: [batch] counters
  uint32_t need[2];      // per problem: value required before a tile of this phase loads
};

__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_cta_shared_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_cta_shared_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}
// Bounded spin until *ctr >= need (global memory, written by other CTAs).
__device__ __forceinline__ bool dep_wait(const uint32_t* ctr, uint32_t need, volatile uint32_t* abort_flag) {
  if (need == 0 || ld_acquire_gpu_u32(ctr) >= need) return true;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t i = 1;; ++i) {
    if (ld_acquire_gpu_u32(ctr) >= need) return true;
    if ((i & 31u) == 0 && (*abort_flag != 0 || globaltimer_ns() - t0 > wait_limit_ns())) return false;
  }
}
// Storing thread: once all its stores have landed, publish the completion of a tile.
__device__ __forceinline__ void flow_publish(uint32_t* counter) {
  bulk_wait_all();
  asm volatile("fence.proxy.async;" ::: "memory");
  __threadfence();
  atomicAdd(counter, 1u);
}
// Producer thread: bounded wait until the scout warp has verified the dependency of the tile with
// running number `seq` (0-based).
__device__ __forceinline__ bool flow_wait_verified(const GemmCtx& cx, uint32_t seq) {
  if (ld_acquire_cta_shared_u32(cx.dep_ok) > seq) return true;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t i = 1;; ++i) {
    if (ld_acquire_cta_shared_u32(cx.dep_ok) > seq) return true;
    if ((i & 63u) == 0 && (*cx.abort_flag != 0 || globaltimer_ns() - t0 > wait_limit_ns())) return false;
  }
}

// Round r of the persistent loop hands CTA c tile r*G + c in even rounds and r*G + (G-1-c) in odd
// rounds ("snake"): with the problems listed heaviest first, a CTA that drew an expensive tile in
// one round draws a cheap one (or none) in the next.
__device__ __forceinline__ int snake_tile(int round, int grid, int cta) {
  return round * grid + ((round & 1) ? (grid - 1 - cta) : cta);
}

// One GEMM phase: CTA c processes its snake sequence of tiles of the concatenated tile lists of
// `nprob` problems.  Tiles of one batch entry are consecutive (n fastest), so CTAs that run at
// the same time share operand tiles in L2.  Warp 0 = TMA producer, warp 1 = MMA issuer, warps
// 2.. = epilogue.  Returns true if a bounded wait ran out.  No CTA-wide sync inside.
// With Deps = FlowDeps tiles are dealt round-robin continuing from the previous phase (no snake) and
// ordered by the completion counters described above.
template <class Op, int RING, class EpiPatch, class Deps = NoDeps>
__device__ __forceinline__ bool gemm_phase(GemmCtx& cx, const GemmProblem<Op>* probs, const int nprob,
                                           EpiPatch patch, Deps deps = Deps{}) {
  constexpr int BT = Op::BT, NA = Op::NA, NB = Op::NB, NACC = Op::NACC, KB = Op::KB;
  constexpr uint32_t kBTileBytes = BT * kBK * 2;  // one k-block of a B tile
  constexpr uint32_t kStageBytes = gemm_stage_bytes<Op>();
  constexpr uint32_t kAccCols = NACC * BT;
  constexpr int kMaxProb = 2;
  static_assert(2 * kAccCols <= 512, "double-buffered accumulators exceed tensor memory");
  // Multi-phase (dataflow) kernels run ops of different tile widths back to back without draining the pipeline: the two
  // accumulator buffers sit at fixed halves of the 512 allocated columns there, so that buffer 0 of one op can never
  // overlap buffer 1 of the previous op while its epilogue is still reading it.
  constexpr uint32_t kAccStride = Deps::kOn ? 256u : kAccCols;
  static_assert(BT % 64 == 0 && BT <= 256, "BT must be 64, 128, 192 or 256");

  constexpr bool SYM = op_symmetric<Op>::value;
  static_assert(!SYM || (BT == kBM && Op::NOUT == 1 && Deps::kOn), "symmetric ops: 128-wide tiles, one staged output, dataflow");
  int tiles_of[kMaxProb], tn_of[kMaxProb], tm_of[kMaxProb], per_batch_of[kMaxProb];
  int total_tiles = 0;
#pragma unroll
  for (int p = 0; p < kMaxProb; ++p) {
    if (p < nprob) {
      tn_of[p] = (probs[p].N + BT - 1) / BT;
      tm_of[p] = (probs[p].M + kBM - 1) / kBM;
      per_batch_of[p] = SYM ? tm_of[p] * (tm_of[p] + 1) / 2 : tn_of[p] * tm_of[p];
      tiles_of[p] = per_batch_of[p] * probs[p].batch;
    } else {
      tn_of[p] = tm_of[p] = per_batch_of[p] = 1;
      tiles_of[p] = 0;
    }
    total_tiles += tiles_of[p];
  }
  auto coord = [&](int tile) {
    TileCoord c;
    c.prob = 0;
    if (tile >= tiles_of[0]) { tile -= tiles_of[0]; c.prob = 1; }
    const int per_batch = per_batch_of[c.prob];
    c.batch = tile / per_batch;
    int r = tile - c.batch * per_batch;
    // a consumer of large intermediates walks the batch entries backwards: the entries its producer wrote last
    // are the ones still in L2
    if constexpr (Op::kReverseBatch) c.batch = probs[c.prob].batch - 1 - c.batch;
    if constexpr (SYM) {
      // tiles on and above the diagonal, row by row: row i holds the tiles (i, i) .. (i, T - 1)
      int i = 0, len = tm_of[c.prob];
      while (r >= len) { r -= len; ++i; --len; }
      c.m0 = i * kBM;
      c.n0 = (i + r) * BT;
    } else {
      c.m0 = (r / tn_of[c.prob]) * kBM;
      c.n0 = (r % tn_of[c.prob]) * BT;
    }
    return c;
  };

  const int rounds = (total_tiles + gridDim.x - 1) / gridDim.x;
  const uint32_t rot0 = cx.rot;
  auto tile_at = [&](int r) {
    if constexpr (Deps::kOn) return r * static_cast<int>(gridDim.x) + static_cast<int>((blockIdx.x + gridDim.x - rot0) % gridDim.x);
    else return snake_tile(r, gridDim.x, blockIdx.x);
  };
  if constexpr (Deps::kOn) cx.rot = (cx.rot + static_cast<uint32_t>(total_tiles)) % gridDim.x;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  bool failed = false;
  if (warp == 0) {
    // ---------------- TMA producer (one thread); the ring keeps running across tiles
    if (lane == 0) {
      for (int tile_i = 0; tile_i < rounds && !failed; ++tile_i) {
        const int tile = tile_at(tile_i);
        if (tile >= total_tiles) continue;
        const TileCoord tc = coord(tile);
        const GemmProblem<Op>& P = probs[tc.prob];
        const int num_kb = (P.K + kBK - 1) / kBK;
        if constexpr (Deps::kOn) {
          if (!flow_wait_verified(cx, cx.ptile++)) { failed = true; break; }  // the scout warp checked this tile
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        const int num_sb = (num_kb + KB - 1) / KB;  // ring stages of KB k-blocks
        for (int sb = 0; sb < num_sb; ++sb, ++cx.it) {
          const int s = cx.it % RING;
          const uint32_t ph = (cx.it / RING) & 1;
          if (!mbar_wait(&cx.empty_bar[s], ph ^ 1, cx.abort_flag)) { failed = true; break; }
          mbar_expect_tx(&cx.full_bar[s], kStageBytes);
          const uint32_t st = cx.smem_base + s * cx.stage_stride;
          const int kc = sb * KB * kBK;
#pragma unroll
          for (int i = 0; i < NA; ++i)
            load_operand_tile<kBM, KB>(st + i * (KB * kATileBytes), &P.a[i], P.ai[i], tc.m0, kc, tc.batch, &cx.full_bar[s]);
#pragma unroll
          for (int i = 0; i < NB; ++i)
            load_operand_tile<BT, KB>(st + NA * (KB * kATileBytes) + i * (KB * kBTileBytes), &P.b[i], P.bi[i], tc.n0, kc,
                                      tc.batch, &cx.full_bar[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (one thread)
    if (lane == 0) {
      for (int tile_i = 0; tile_i < rounds && !failed; ++tile_i) {
        const int tile = tile_at(tile_i);
        if (tile >= total_tiles) continue;
        const TileCoord tc = coord(tile);
        const GemmProblem<Op>& P = probs[tc.prob];
        const int num_kb = (P.K + kBK - 1) / kBK;
        const uint32_t as = cx.tcount & 1, aph = (cx.tcount >> 1) & 1;
        if (!mbar_wait(&cx.acc_empty_bar[as], aph ^ 1, cx.abort_flag)) { failed = true; break; }
        tc_fence_after();
        const uint32_t acc_base = cx.tmem_base + as * kAccStride;
        const int num_sb = (num_kb + KB - 1) / KB;
        for (int sb = 0; sb < num_sb; ++sb, ++cx.it) {
          const int s = cx.it % RING;
          const uint32_t ph = (cx.it / RING) & 1;
          if (!mbar_wait(&cx.full_bar[s], ph, cx.abort_flag)) { failed = true; break; }
          tc_fence_after();
          const uint32_t st = cx.smem_base + s * cx.stage_stride;
#pragma unroll
          for (int kk = 0; kk < KB; ++kk) {
            if (sb * KB + kk >= num_kb) break;  // a trailing half-empty stage
#pragma unroll
            for (int t = 0; t < Op::NTERMS; ++t) {
              const int ia = Op::term_a(t), ib = Op::term_b(t);
              const int a_mn = P.ai[ia].mn_major, b_mn = P.bi[ib].mn_major;
              const uint32_t idesc = make_idesc_bf16(kBM, Op::term_n(t), a_mn, b_mn);
              const uint32_t a_tile = st + ia * (KB * kATileBytes);
              const uint32_t b_tile = st + NA * (KB * kATileBytes) + ib * (KB * kBTileBytes);
#pragma unroll
              for (int k4 = 0; k4 < kBK / kUmmaK; ++k4) {
                const uint32_t acc = (sb > 0 || kk > 0 || k4 > 0 || !Op::term_first(t)) ? 1u : 0u;
                umma_bf16(acc_base + Op::term_col(t), operand_desc<KB>(a_tile, a_mn, kATileBytes, kk, k4),
                          operand_desc<KB>(b_tile, b_mn, kBTileBytes, kk, k4), idesc, acc);
              }
            }
          }
          umma_commit(&cx.empty_bar[s]);  // frees the stage once these MMAs have read it
        }
        if (!failed) umma_commit(&cx.acc_full_bar[as]);
        ++cx.tcount;
      }
    }
  } else if (warp == 2 + kEpiWarps) {
    // ---------------- dependency scout (dataflow kernels only): one thread verifies, in tile order,
    // that every tile's inputs are complete and publishes the count of verified tiles
    if constexpr (Deps::kOn) {
      if (lane == 0) {
        for (int tile_i = 0; tile_i < rounds && !failed; ++tile_i) {
          const int tile = tile_at(tile_i);
          if (tile >= total_tiles) continue;
          const TileCoord tc = coord(tile);
          if (!dep_wait(deps.counter[tc.prob] + tc.batch, deps.need[tc.prob], cx.abort_flag)) { failed = true; break; }
          st_release_cta_shared_u32(cx.dep_ok, ++cx.ptile);
        }
      }
    }
  } else if (warp > 2 + kEpiWarps) {
    // ---------------- storing thread (dataflow kernels only): takes each staged tile from the epilogue
    // warps, issues its TMA stores, returns the staging tile as soon as the stores have read it, and
    // publishes the tile's completion as soon as they have landed -- the epilogue warps never wait for
    // global memory, and no CTA can wait on a tile it has not yet published itself
    if constexpr (Deps::kOn && Op::NOUT > 0) {
      if (lane == 0) {
        for (int tile_i = 0; tile_i < rounds && !failed; ++tile_i) {
          const int tile = tile_at(tile_i);
          if (tile >= total_tiles) continue;
          const TileCoord tc = coord(tile);
          const GemmProblem<Op>& P = probs[tc.prob];
          typename Op::Epi ep = P.ep;
          patch(ep, tc.prob);
          const uint32_t stg = cx.staging;
          if (!mbar_wait(&cx.stg_full_bar[0], cx.sround & 1, cx.abort_flag)) { failed = true; break; }
#pragma unroll
          for (int o = 0; o < Op::NOUT; ++o) {
            if (!P.oi[o].enabled || Op::skip_store(ep, o)) continue;
            for (int pnl = 0; pnl < BT / 64; ++pnl) {
              if (tc.n0 + pnl * 64 >= P.N) break;
              tma_store_3d(&P.out[o], stg + o * (kBM * BT * 2) + pnl * (kBM * 128), P.oi[o].col_off + tc.n0 + pnl * 64,
                           P.oi[o].row_off + tc.m0, P.oi[o].batch_off + tc.batch);
            }
          }
          if constexpr (SYM) {
            // the transposed tile (second staging tile) goes below the diagonal
            if (tc.m0 != tc.n0) {
              for (int pnl = 0; pnl < BT / 64; ++pnl) {
                if (tc.m0 + pnl * 64 >= P.N) break;
                tma_store_3d(&P.out[0], stg + kBM * BT * 2 + pnl * (kBM * 128), P.oi[0].col_off + tc.m0 + pnl * 64,
                             P.oi[0].row_off + tc.n0, P.oi[0].batch_off + tc.batch);
              }
            }
          }
          bulk_commit_group();
          bulk_wait_read_all();
          mbar_arrive(&cx.stg_empty_bar[0]);
          ++cx.sround;
          flow_publish(deps.counter[tc.prob] + tc.batch);
        }
      }
    }
  } else {
    // ---------------- epilogue: warp w may only touch TMEM lanes [32*(w%4), 32*(w%4)+32); the two
    // warps of a lane quarter take alternate 32-column chunks.  Ops with NOUT > 0 round their
    // results to bf16 into swizzled shared-memory tiles that one thread hands to TMA stores
    // (full-line writes, clipped by the output map); other ops store from registers.
    constexpr int NOUT = Op::NOUT;
    constexpr int NSTG = NOUT;  // staging tiles
    constexpr int kEpiThreads = kEpiWarps * 32;
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const bool elected = threadIdx.x == 64;
    const int row_local = quarter * 32 + lane;
    auto tile_of_round = [&](int r) {
      if (r >= rounds) return -1;
      const int t = tile_at(r);
      return t < total_tiles ? t : -1;
    };
    for (int tile_i = 0; tile_i < rounds; ++tile_i) {
      const int tile = tile_of_round(tile_i);
      if (tile < 0) continue;
      const TileCoord tc = coord(tile);
      const GemmProblem<Op>& P = probs[tc.prob];
      typename Op::Epi ep = P.ep;
      patch(ep, tc.prob);
      const uint32_t stg = cx.staging;
      const uint32_t as = cx.tcount & 1, aph = (cx.tcount >> 1) & 1;
      const int row = tc.m0 + row_local;
      // global operands of the epilogue are fetched while the tile's MMAs are still running
      typename Op::Prefetch pf;
      Op::prefetch(ep, tc.batch, row, tc.n0, half, P.M, P.N, pf);
      bool got = mbar_wait(&cx.acc_full_bar[as], aph, cx.abort_flag);
      tc_fence_after();
      const uint32_t acc_base = cx.tmem_base + as * kAccStride + (static_cast<uint32_t>(quarter * 32) << 16);
      if constexpr (NOUT > 0) {
        // A warp whose wait ran out must not leave the others stuck at a named barrier: it raises
        // a flag that only epilogue warps write, and every warp decides after the barrier.
        if (!got) cx.abort_flag[1] = 1;
        // the previous tile's stores must have finished reading the staging tile
        if (elected) {
          if constexpr (Deps::kOn) {
            // the storing warp returns the staging tile once its stores have read it
            if (cx.sround > 0 && !mbar_wait(&cx.stg_empty_bar[0], (cx.sround - 1) & 1, cx.abort_flag)) cx.abort_flag[1] = 1;
          } else {
            bulk_wait_read_all();
          }
        }
        named_barrier_sync(1, kEpiThreads);
        if (cx.abort_flag[1] != 0) { failed = true; break; }
      } else {
        if (!got) { failed = true; break; }
      }
      for (int c = half * 32; c < BT; c += 64) {
        if (tc.n0 + c >= P.N) break;  // warp-uniform
        float v[NACC][32];
        {
          uint32_t bits[NACC][32];
#pragma unroll
          for (int a = 0; a < NACC; ++a) tmem_ld32(acc_base + a * BT + c, bits[a]);
          tmem_ld_wait();  // one wait for the loads of all accumulators
#pragma unroll
          for (int a = 0; a < NACC; ++a)
#pragma unroll
            for (int j = 0; j < 32; ++j) v[a][j] = __uint_as_float(bits[a][j]);
        }
        if constexpr (NOUT > 0) {
          float ov[NSTG > 0 ? NSTG : 1][32];
          const uint32_t rowaddr = (c >> 6) * (kBM * 128) + row_local * 128;
          const uint32_t unit0 = (c & 63) >> 3;
          Op::epilogue_staged(ep, tc.batch, row, tc.n0 + c, P.M, P.N, v, ov, pf);
#pragma unroll
          for (int o = 0; o < NSTG; ++o) {
            const uint32_t base = stg + o * (kBM * BT * 2) + rowaddr;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const uint32_t addr = base + (((unit0 + g) ^ (row_local & 7)) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr),
                           "r"(pack_bf16x2(ov[o][g * 8 + 0], ov[o][g * 8 + 1])),
                           "r"(pack_bf16x2(ov[o][g * 8 + 2], ov[o][g * 8 + 3])),
                           "r"(pack_bf16x2(ov[o][g * 8 + 4], ov[o][g * 8 + 5])),
                           "r"(pack_bf16x2(ov[o][g * 8 + 6], ov[o][g * 8 + 7]))
                           : "memory");
            }
          }
          if constexpr (SYM) {
            if (tc.m0 != tc.n0) {
              // element (row_local, c + j) lands at (c + j, row_local) of the second staging tile: the 32 lanes of a
              // warp write 32 consecutive columns of one row (64 contiguous bytes)
              const uint32_t tbase = stg + kBM * BT * 2 + (row_local >> 6) * (kBM * 128) + (row_local & 7) * 2;
              const uint32_t tunit = (row_local & 63) >> 3;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const uint32_t rt = c + j;
                const uint32_t addr = tbase + rt * 128 + ((tunit ^ (rt & 7)) << 4);
                const __nv_bfloat16 hv = __float2bfloat16_rn(ov[0][j]);
                asm volatile("st.shared.b16 [%0], %1;" ::"r"(addr), "h"(*reinterpret_cast<const uint16_t*>(&hv)) : "memory");
              }
            }
          }
        } else {
          if constexpr (Op::kWarpTranspose)
            Op::epilogue_warp(ep, tc.batch, tc.m0 + quarter * 32, tc.n0 + c, P.M, P.N, v, pf,
                              cx.staging + (warp - 2) * (32 * 144), lane);
          else
            Op::epilogue(ep, tc.batch, row, tc.n0 + c, P.M, P.N, v, pf, c >> 6);
        }
      }
      // all TMEM reads of this warp are complete (wait::ld above): hand the buffer back
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&cx.acc_empty_bar[as]);
      if constexpr (Op::kTileReduce) {
        // per-tile, per-warp reduction of a per-thread value (no cross-warp synchronisation: the
        // consumer adds the eight warp partials of every tile in a fixed order)
        float tv = Op::tile_value(pf);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) tv += __shfl_xor_sync(0xFFFFFFFFu, tv, o);
        if (lane == 0) Op::tile_store(ep, tc.batch, tc.m0 / kBM, tc.n0 / BT, warp - 2, tv);
      }
      if constexpr (NOUT > 0) {
        fence_async_proxy();
        named_barrier_sync(2, kEpiThreads);
        if constexpr (Deps::kOn) {
          if (elected) mbar_arrive(&cx.stg_full_bar[0]);  // the storing warp issues the stores and publishes the tile
          ++cx.sround;
        } else if (elected) {
#pragma unroll
          for (int o = 0; o < NOUT; ++o) {
            if (!P.oi[o].enabled || Op::skip_store(ep, o)) continue;
            for (int pnl = 0; pnl < BT / 64; ++pnl) {
              if (tc.n0 + pnl * 64 >= P.N) break;
              tma_store_3d(&P.out[o], stg + o * (kBM * BT * 2) + pnl * (kBM * 128),
                           P.oi[o].col_off + tc.n0 + pnl * 64, P.oi[o].row_off + tc.m0, P.oi[o].batch_off + tc.batch);
            }
          }
          bulk_commit_group();
        }
      }
      ++cx.tcount;
    }
    if constexpr (NOUT > 0 && !Deps::kOn) {
      if (elected) bulk_wait_all();  // this CTA's output tiles are in global memory
    }
  }
  return failed;
}

// Carves barriers out of shared memory behind a ring of `ring` stages of `stage_stride` bytes,
// initialises them and allocates `tmem_cols` columns of tensor memory.  Ends with a CTA-wide sync.
__device__ __forceinline__ void gemm_setup(GemmCtx& cx, uint8_t* smem_raw, int ring, uint32_t stage_stride,
                                           uint32_t staging_bytes, uint32_t tmem_cols) {
  const uint32_t raw_addr = smem_u32(smem_raw);
  cx.smem_base = (raw_addr + 1023u) & ~1023u;
  cx.stage_stride = stage_stride;
  cx.staging = cx.smem_base + ring * stage_stride;
  uint8_t* aligned = smem_raw + (cx.smem_base - raw_addr);
  cx.full_bar = reinterpret_cast<uint64_t*>(aligned + ring * stage_stride + staging_bytes);
  cx.empty_bar = cx.full_bar + ring;
  cx.acc_full_bar = cx.empty_bar + ring;    // [2]
  cx.acc_empty_bar = cx.acc_full_bar + 2;   // [2]
  cx.stg_full_bar = cx.acc_empty_bar + 2;   // [1]
  cx.stg_empty_bar = cx.stg_full_bar + 1;   // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(cx.stg_empty_bar + 1);
  cx.abort_flag = tmem_slot + 1;  // [2]
  cx.dep_ok = tmem_slot + 3;
  if (threadIdx.x == 0) {
    for (int s = 0; s < ring; ++s) {
      mbar_init(&cx.full_bar[s], 1);
      mbar_init(&cx.empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&cx.acc_full_bar[s], 1);
      mbar_init(&cx.acc_empty_bar[s], kEpiWarps);
    }
    mbar_init(&cx.stg_full_bar[0], 1);
    mbar_init(&cx.stg_empty_bar[0], 1);
    cx.abort_flag[0] = 0;
    cx.abort_flag[1] = 0;
    *cx.dep_ok = 0;
    fence_mbar_init();
  }
  if ((threadIdx.x >> 5) == 1) {
    tmem_alloc(tmem_slot, tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  cx.tmem_base = *tmem_slot;
}

__device__ __forceinline__ void gemm_teardown(GemmCtx& cx, bool failed, int32_t* status, uint32_t tmem_cols) {
  if (failed) {
    *cx.abort_flag = 1;
    atomicCAS(status, kStatusOk, kStatusWaitTimeout);
  }
  tc_fence_before();
  __syncthreads();
  if (*cx.abort_flag && threadIdx.x == 0) {
    // let bulk copies still in flight land before shared memory is released
    for (int i = 0; i < 256; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if ((threadIdx.x >> 5) == 1) tmem_dealloc(cx.tmem_base, tmem_cols);
}

// Persistent single-phase kernel.  The prologue (barriers, tensor memory, descriptor prefetch)
// touches no global memory and may overlap the tail of the previous kernel in the stream.
template <class Op, int NPROB>
__global__ void __launch_bounds__(kGemmThreadsV2, 1)
umma_gemm_kernel(const __grid_constant__ GemmArgs<Op, NPROB> args, const int nprob) {
  static_assert(NPROB <= 2, "at most two problems per launch");
  extern __shared__ uint8_t smem_raw[];
  constexpr uint32_t kTmemCols = tmem_cols_pow2(2 * Op::NACC * Op::BT);
  GemmCtx cx;
  gemm_setup(cx, smem_raw, Op::STAGES, gemm_stage_bytes<Op>(), gemm_staging_bytes<Op>(), kTmemCols);
  if (threadIdx.x == 32) {
    for (int p = 0; p < nprob; ++p) {
#pragma unroll
      for (int i = 0; i < Op::NA; ++i) tma_prefetch_desc(&args.prob[p].a[i]);
#pragma unroll
      for (int i = 0; i < Op::NB; ++i) tma_prefetch_desc(&args.prob[p].b[i]);
#pragma unroll
      for (int i = 0; i < Op::NOUT; ++i) tma_prefetch_desc(&args.prob[p].out[i]);
    }
  }
  griddep_launch_dependents();
  griddep_wait();
  bool failed = false;
  // an earlier launch gave up: do nothing but release the resources
  if (*reinterpret_cast<volatile int32_t*>(args.status) == kStatusOk)
    failed = gemm_phase<Op, Op::STAGES>(cx, args.prob, nprob, NoPatch{});
  gemm_teardown(cx, failed, args.status, kTmemCols);
}

}  // namespace lact
