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

template <int BT, int NITER>
struct NsBwdFusedArgs {
  GemmProblem<OpNs2<BT>> q[NITER][2];    // [iteration][group]
  GemmProblem<OpNs2<BT>> t[NITER][2];
  GemmProblem<OpNs2<BT>> dx[NITER][2];
  float coef_c[NITER];                   // c of (a, b, c) per iteration
  int32_t steps, ngroups;
  int32_t* status;
  uint32_t* done[2];  // per group: [matrix] completion counters, zero at launch
};

template <int BT>
__host__ __device__ constexpr int ns_bwd_ring() {
  return static_cast<int>((232448u - 1024u - 256u - kBM * BT * 2) / gemm_stage_bytes<OpNs2<BT>>());
}
template <int BT>
__host__ __device__ constexpr uint32_t ns_bwd_smem_bytes() {
  return ns_bwd_ring<BT>() * gemm_stage_bytes<OpNs2<BT>>() + kBM * BT * 2 + 1024 + 256;
}

template <int BT, int NITER>
__global__ void __launch_bounds__(kGemmThreadsFlow, 1)
ns_bwd_fused_kernel(const __grid_constant__ NsBwdFusedArgs<BT, NITER> args) {
  using Op = OpNs2<BT>;
  constexpr int RING = ns_bwd_ring<BT>();
  constexpr uint32_t kTmemCols = 512;
  griddep_launch_dependents();
  if (*reinterpret_cast<volatile int32_t*>(args.status) != kStatusOk) return;  // uniform over the grid
  extern __shared__ uint8_t smem_raw[];
  GemmCtx cx;
  gemm_setup(cx, smem_raw, RING, gemm_stage_bytes<Op>(), kBM * BT * 2, kTmemCols);
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
    tiles_mm[g] = ((A.M + kBM - 1) / kBM) * ((A.N + BT - 1) / BT);
    tiles_mn[g] = ((U.M + kBM - 1) / kBM) * ((U.N + BT - 1) / BT);
  }
  patch.diag = 0.f;
  patch.scale_pow = 0;
  for (int it = args.steps - 1; it >= 0 && !failed; --it) {
    patch.acc_scale = 1.f;
    failed = gemm_phase<Op, RING>(cx, args.q[it], args.ngroups, patch, deps);
    if (failed) break;
    for (int g = 0; g < 2; ++g) deps.need[g] += tiles_mm[g];
    patch.acc_scale = args.coef_c[it];
    failed = gemm_phase<Op, RING>(cx, args.t[it], args.ngroups, patch, deps);
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
