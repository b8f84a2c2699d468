// Backward of all Newton-Schulz iterations of a Muon update in ONE persistent kernel.  With the forward's
// iterates X_i, shifted Gram matrices S_i = X_i X_i^T + (b/2c) I and polynomials P_i kept, the gradient
// dX_{i+1} -> dX_i of X_{i+1} = P_i X_i is three two-product contractions (roundings treated as identities):
//   Q  = dX_{i+1} X_i^T + X_i dX_{i+1}^T                      (m x m, contraction over the long side)
//   T  = c (S_i Q + Q S_i)                                    (m x m)
//   dX_i = P_i dX_{i+1} + T X_i                               (the iterate's own shape)
// which form, per matrix, the same kind of dependency chain as the forward (see ns_fused.cuh): the phases are
// ordered by per-matrix completion counters, tiles are dealt round-robin across phase boundaries, every wait is
// bounded, and the kernel is launched cooperatively with at most one CTA per SM.
#pragma once
#include "ns_fused.cuh"

namespace lact {

// SYM: Q and T (both symmetric) are computed on and above the diagonal only, in 128 x 128 tiles (BT_MM = 128).
template <int BT_MM, int BT, int NITER, bool SYM>
struct NsBwdFusedArgs {
  GemmProblem<OpNs2T<BT_MM, SYM>> q[NITER][2];    // [iteration][group]
  GemmProblem<OpNs2T<BT_MM, SYM>> t[NITER][2];
  GemmProblem<OpNs2<BT>> dx[NITER][2];
  float coef_c[NITER];                   // c of (a, b, c) per iteration
  int32_t steps, ngroups;
  int32_t* status;
  uint32_t* done[2];  // per group: [matrix] completion counters, zero at launch
};

template <int BT_MM, int BT, bool SYM>
__host__ __device__ constexpr uint32_t ns_bwd_stride() {
  return gemm_stage_bytes<OpNs2T<BT_MM, SYM>>() > gemm_stage_bytes<OpNs2<BT>>() ? gemm_stage_bytes<OpNs2T<BT_MM, SYM>>()
                                                                               : gemm_stage_bytes<OpNs2<BT>>();
}
template <int BT_MM, int BT, bool SYM>
__host__ __device__ constexpr uint32_t ns_bwd_staging() {
  return gemm_staging_bytes<OpNs2T<BT_MM, SYM>>() > gemm_staging_bytes<OpNs2<BT>>() ? gemm_staging_bytes<OpNs2T<BT_MM, SYM>>()
                                                                                   : gemm_staging_bytes<OpNs2<BT>>();
}
template <int BT_MM, int BT, bool SYM>
__host__ __device__ constexpr int ns_bwd_ring() {
  return static_cast<int>((232448u - 1024u - 256u - ns_bwd_staging<BT_MM, BT, SYM>()) / ns_bwd_stride<BT_MM, BT, SYM>());
}
template <int BT_MM, int BT, bool SYM>
__host__ __device__ constexpr uint32_t ns_bwd_smem_bytes() {
  return ns_bwd_ring<BT_MM, BT, SYM>() * ns_bwd_stride<BT_MM, BT, SYM>() + ns_bwd_staging<BT_MM, BT, SYM>() + 1024 + 256;
}

template <int BT_MM, int BT, int NITER, bool SYM>
__global__ void __launch_bounds__(kGemmThreadsFlow, 1)
ns_bwd_fused_kernel(const __grid_constant__ NsBwdFusedArgs<BT_MM, BT, NITER, SYM> args) {
  static_assert(!SYM || BT_MM == kBM, "symmetric phases use square 128 x 128 tiles");
  using OpMM = OpNs2T<BT_MM, SYM>;
  using Op = OpNs2<BT>;
  constexpr int RING = ns_bwd_ring<BT_MM, BT, SYM>();
  constexpr uint32_t kTmemCols = 512;
  griddep_launch_dependents();
  if (*reinterpret_cast<volatile int32_t*>(args.status) != kStatusOk) return;  // uniform over the grid
  extern __shared__ uint8_t smem_raw[];
  GemmCtx cx;
  gemm_setup(cx, smem_raw, RING, ns_bwd_stride<BT_MM, BT, SYM>(), ns_bwd_staging<BT_MM, BT, SYM>(), kTmemCols);
  bool failed = false;
  NsPatch patch;
  FlowDeps deps;
  uint32_t tiles_mm[2], tiles_mn[2];
  for (int g = 0; g < 2; ++g) {
    patch.scale[g] = nullptr;
    deps.counter[g] = args.done[g];
    deps.need[g] = 0;
    const auto& A = args.q[0][g];
    const auto& U = args.dx[0][g];
    const uint32_t tm = (A.M + kBM - 1) / kBM;
    tiles_mm[g] = SYM ? tm * (tm + 1) / 2 : tm * ((A.N + BT_MM - 1) / BT_MM);
    tiles_mn[g] = ((U.M + kBM - 1) / kBM) * ((U.N + BT - 1) / BT);
  }
  patch.diag = 0.f;
  patch.scale_pow = 0;
  for (int it = args.steps - 1; it >= 0 && !failed; --it) {
    patch.acc_scale = 1.f;
    failed = gemm_phase<OpMM, RING>(cx, args.q[it], args.ngroups, patch, deps);
    if (failed) break;
    for (int g = 0; g < 2; ++g) deps.need[g] += tiles_mm[g];
    patch.acc_scale = args.coef_c[it];
    failed = gemm_phase<OpMM, RING>(cx, args.t[it], args.ngroups, patch, deps);
    if (failed) break;
    for (int g = 0; g < 2; ++g) deps.need[g] += tiles_mm[g];
    patch.acc_scale = 1.f;
    failed = gemm_phase<Op, RING>(cx, args.dx[it], args.ngroups, patch, deps);
    for (int g = 0; g < 2; ++g) deps.need[g] += tiles_mn[g];
  }
  if (failed) *cx.abort_flag = 1;
  gemm_teardown(cx, failed, args.status, kTmemCols);
}

}  // namespace lact
