// All Newton-Schulz iterations of a Muon update in ONE persistent kernel: `steps` x (gram, poly,
// update) GEMM phases on the tcgen05 engine.  The phases of one matrix form a dependency chain, but
// different matrices are independent: instead of a grid-wide barrier between phases, every matrix
// owns a completion counter in global memory (see FlowDeps) and a tile waits (bounded spin) only for
// the previous phase of its own matrix.  Tiles are dealt round-robin across phase boundaries, so
// the shared-memory ring and the tensor-memory pipeline of a CTA keep running from the first tile
// of the first phase to the last tile of the last one.  All CTAs must be co-resident: the kernel
// is launched cooperatively with at most one CTA per SM.
#pragma once
#include "ops.cuh"

namespace lact {

// NITER sets of problems are held, iteration `it` uses set it % NITER: two sets for the plain iteration (the iterates
// ping-pong between two buffers), one set per iteration when every iterate, shifted Gram matrix and polynomial is
// kept for the backward pass (steps <= NITER then).
// SYM: the Gram and polynomial phases compute only the tiles on and above the diagonal (BT_MM = 128).
template <int BT_MM, int BT_MN, int NITER = 2, bool SYM = false>
struct NsFusedArgs {
  GemmProblem<OpNsT<BT_MM, SYM>> gram[NITER][2];  // [iteration % NITER][group]
  GemmProblem<OpNsT<BT_MM, SYM>> poly[NITER][2];
  GemmProblem<OpNs<BT_MN>> upd[NITER][2];
  const float* scale[2];                // per group: [matrix] 1 / (||G|| + 1e-7) when the first iterate is unscaled
  float coef[16][3];                    // (a, b, c) per iteration
  int32_t steps, ngroups;
  int32_t* status;
  uint32_t* done[2];  // per group: [matrix] completion counters, zero at launch
};

constexpr int kNsFusedMaxSteps = 16;

struct NsPatch {
  float diag, acc_scale;
  int32_t scale_pow;
  const float* scale[2];
  __device__ __forceinline__ void operator()(EpiNs& ep, int prob) const {
    ep.diag = diag;
    ep.acc_scale = acc_scale;
    ep.scale = scale[prob];
    ep.scale_pow = scale_pow;
  }
};

template <int BT_MM, int BT_MN, bool SYM = false>
__host__ __device__ constexpr uint32_t ns_fused_stage_stride() {
  return gemm_stage_bytes<OpNsT<BT_MM, SYM>>() > gemm_stage_bytes<OpNs<BT_MN>>() ? gemm_stage_bytes<OpNsT<BT_MM, SYM>>()
                                                                                : gemm_stage_bytes<OpNs<BT_MN>>();
}
template <int BT_MM, int BT_MN, bool SYM = false>
__host__ __device__ constexpr uint32_t ns_fused_staging() {
  return gemm_staging_bytes<OpNsT<BT_MM, SYM>>() > gemm_staging_bytes<OpNs<BT_MN>>() ? gemm_staging_bytes<OpNsT<BT_MM, SYM>>()
                                                                                    : gemm_staging_bytes<OpNs<BT_MN>>();
}
template <int BT_MM, int BT_MN, bool SYM = false>
__host__ __device__ constexpr int ns_fused_ring() {
  return static_cast<int>((232448u - 1024u - 256u - ns_fused_staging<BT_MM, BT_MN, SYM>()) /
                          ns_fused_stage_stride<BT_MM, BT_MN, SYM>());
}
template <int BT_MM, int BT_MN, bool SYM = false>
__host__ __device__ constexpr uint32_t ns_fused_smem_bytes() {
  return ns_fused_ring<BT_MM, BT_MN, SYM>() * ns_fused_stage_stride<BT_MM, BT_MN, SYM>() +
         ns_fused_staging<BT_MM, BT_MN, SYM>() + 1024 + 256;
}

template <int BT_MM, int BT_MN, int NITER, bool SYM = false>
__global__ void __launch_bounds__(kGemmThreadsFlow, 1)
ns_fused_kernel(const __grid_constant__ NsFusedArgs<BT_MM, BT_MN, NITER, SYM> args) {
  static_assert(!SYM || BT_MM == kBM, "symmetric phases use square 128 x 128 tiles");
  using OpMM = OpNsT<BT_MM, SYM>;
  using OpMN = OpNs<BT_MN>;
  constexpr int RING = ns_fused_ring<BT_MM, BT_MN, SYM>();
  constexpr uint32_t kStride = ns_fused_stage_stride<BT_MM, BT_MN, SYM>();
  constexpr uint32_t kTmemCols = 512;
  griddep_launch_dependents();  // the next kernel may run its prologue while this one works
  if (*reinterpret_cast<volatile int32_t*>(args.status) != kStatusOk) return;  // uniform over the grid
  extern __shared__ uint8_t smem_raw[];
  GemmCtx cx;
  gemm_setup(cx, smem_raw, RING, kStride, ns_fused_staging<BT_MM, BT_MN, SYM>(), kTmemCols);
  if (threadIdx.x == 32) {
    for (int par = 0; par < (NITER < 2 ? NITER : 2); ++par)
      for (int g = 0; g < args.ngroups; ++g) {
        tma_prefetch_desc(&args.gram[par][g].a[0]);
        tma_prefetch_desc(&args.gram[par][g].b[0]);
        tma_prefetch_desc(&args.upd[par][g].a[0]);
        tma_prefetch_desc(&args.upd[par][g].b[0]);
        tma_prefetch_desc(&args.gram[par][g].out[0]);
        tma_prefetch_desc(&args.upd[par][g].out[0]);
        tma_prefetch_desc(&args.poly[par][g].a[0]);
        tma_prefetch_desc(&args.poly[par][g].b[0]);
        tma_prefetch_desc(&args.poly[par][g].out[0]);
      }
  }
  bool failed = false;

  // ---------------- Newton-Schulz iterations
  NsPatch patch;
  FlowDeps deps;
  uint32_t tiles_mm[2], tiles_mn[2];  // tiles one matrix contributes to a gram / poly phase, an update phase
  for (int g = 0; g < 2; ++g) {
    patch.scale[g] = args.scale[g];
    deps.counter[g] = args.done[g];
    deps.need[g] = 0;
    const auto& A = args.poly[0][g];
    const auto& U = args.upd[0][g];
    const uint32_t tm = (A.M + kBM - 1) / kBM;
    tiles_mm[g] = SYM ? tm * (tm + 1) / 2 : tm * ((A.N + BT_MM - 1) / BT_MM);
    tiles_mn[g] = ((U.M + kBM - 1) / kBM) * ((U.N + BT_MN - 1) / BT_MN);
  }
  for (int it = 0; it < args.steps && !failed; ++it) {
    const int par = it % NITER;
    const float a = args.coef[it][0], b = args.coef[it][1], c = args.coef[it][2];
    patch.scale_pow = it == 0 ? 2 : 0;
    patch.diag = b / (2.f * c);       // gram: S = X X^T + (b / 2c) I
    patch.acc_scale = 1.f;
    failed = gemm_phase<OpMM, RING>(cx, args.gram[par], args.ngroups, patch, deps);
    if (failed) break;
    for (int g = 0; g < 2; ++g) deps.need[g] += tiles_mm[g];
    patch.diag = a - b * b / (4.f * c);  // poly: P = c S S + (a - b^2 / 4c) I
    patch.acc_scale = c;
    patch.scale_pow = 0;
    failed = gemm_phase<OpMM, RING>(cx, args.poly[par], args.ngroups, patch, deps);
    if (failed) break;
    for (int g = 0; g < 2; ++g) deps.need[g] += tiles_mm[g];
    patch.diag = 0.f;                 // update: X' = P X
    patch.acc_scale = 1.f;
    patch.scale_pow = it == 0 ? 1 : 0;
    failed = gemm_phase<OpMN, RING>(cx, args.upd[par], args.ngroups, patch, deps);
    for (int g = 0; g < 2; ++g) deps.need[g] += tiles_mn[g];
  }
  if (failed) *cx.abort_flag = 1;
  // (the storing thread published every tile of this CTA after its stores had landed)

  gemm_teardown(cx, failed, args.status, kTmemCols);
}

}  // namespace lact
