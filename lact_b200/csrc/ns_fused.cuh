// All Newton-Schulz iterations of a Muon update in ONE persistent kernel: `steps` x (gram, poly,
// update) GEMM phases on the tcgen05 engine, separated by a grid-wide barrier (an atomic counter in
// global memory, bounded spin), so the 3*steps dependent stages cost no kernel launches and the
// shared-memory ring / tensor-memory pipeline never has to be rebuilt.  All CTAs must be
// co-resident: the kernel is launched cooperatively with at most one CTA per SM.
#pragma once
#include "ops.cuh"

namespace lact {

template <int BT_MM, int BT_MN>
struct NsFusedArgs {
  GemmProblem<OpNs<BT_MM>> gram[2][2];  // [iteration parity][group]
  GemmProblem<OpNs<BT_MM>> poly[2];     // [group]
  GemmProblem<OpNs<BT_MN>> upd[2][2];   // [iteration parity][group]
  int32_t transposed[2], m[2];          // per group: iterate is the gradient's transpose; rows of the iterate
  float coef[16][3];                    // (a, b, c) per iteration
  int32_t steps, ngroups;
  int32_t* status;
  uint32_t* barrier;  // grid barrier counter, zero at launch
  uint64_t* trace;    // optional [2 * phases + 2] globaltimer stamps of CTA 0 (diagnostics), or nullptr
};

constexpr int kNsFusedMaxSteps = 16;

__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Grid-wide barrier for a co-resident grid; every thread of every CTA calls it.  Orders the
// generic-proxy global writes made before it with the generic and async-proxy (TMA) reads made
// after it.  Returns false if the wait ran out (the CTA's abort flag is then set).
__device__ __forceinline__ bool grid_sync(uint32_t* counter, uint32_t& epoch, volatile uint32_t* abort_flag,
                                          uint64_t* trace = nullptr) {
  asm volatile("fence.proxy.async;" ::: "memory");
  __threadfence();
  __syncthreads();
  epoch += 1;
  if (threadIdx.x == 0) {
    if (trace != nullptr && blockIdx.x == 0) trace[2 * epoch - 1] = globaltimer_ns();  // CTA 0 finished the phase
    atomicAdd(counter, 1u);
    const uint32_t target = epoch * gridDim.x;
    const uint64_t t0 = globaltimer_ns();
    uint32_t i = 0;
    while (ld_acquire_u32(counter) < target) {
      if ((++i & 63u) == 0 && (*abort_flag != 0 || globaltimer_ns() - t0 > kWaitLimitNs)) {
        *abort_flag = 1;
        break;
      }
    }
    __threadfence();
    if (trace != nullptr && blockIdx.x == 0) trace[2 * epoch] = globaltimer_ns();  // every CTA finished it
  }
  __syncthreads();
  asm volatile("fence.proxy.async;" ::: "memory");
  return *abort_flag == 0;
}

struct NsPatch {
  float alpha, gamma;
  int32_t last;
  int32_t transposed[2];
  int32_t m[2];
  __device__ __forceinline__ void operator()(EpiNs& ep, int prob) const {
    ep.alpha = alpha;
    ep.gamma = gamma;
    ep.out_transposed = (last && transposed[prob]) ? 1 : 0;
    ep.out_ld_t = m[prob];
  }
};

template <int BT_MM, int BT_MN>
__host__ __device__ constexpr uint32_t ns_fused_stage_stride() {
  return gemm_stage_bytes<OpNs<BT_MM>>() > gemm_stage_bytes<OpNs<BT_MN>>() ? gemm_stage_bytes<OpNs<BT_MM>>()
                                                                         : gemm_stage_bytes<OpNs<BT_MN>>();
}
template <int BT_MM, int BT_MN>
__host__ __device__ constexpr uint32_t ns_fused_staging() {
  return 2 * kBM * (BT_MM > BT_MN ? BT_MM : BT_MN) * 2;  // double-buffered (OpNs::kStagingBuffers)
}
template <int BT_MM, int BT_MN>
__host__ __device__ constexpr int ns_fused_ring() {
  return static_cast<int>((232448u - 1024u - 256u - ns_fused_staging<BT_MM, BT_MN>()) /
                          ns_fused_stage_stride<BT_MM, BT_MN>());
}
template <int BT_MM, int BT_MN>
__host__ __device__ constexpr uint32_t ns_fused_smem_bytes() {
  return ns_fused_ring<BT_MM, BT_MN>() * ns_fused_stage_stride<BT_MM, BT_MN>() + ns_fused_staging<BT_MM, BT_MN>() +
         1024 + 256;
}

template <int BT_MM, int BT_MN>
__global__ void __launch_bounds__(kGemmThreadsV2, 1)
ns_fused_kernel(const __grid_constant__ NsFusedArgs<BT_MM, BT_MN> args) {
  using OpMM = OpNs<BT_MM>;
  using OpMN = OpNs<BT_MN>;
  constexpr int RING = ns_fused_ring<BT_MM, BT_MN>();
  constexpr uint32_t kStride = ns_fused_stage_stride<BT_MM, BT_MN>();
  constexpr uint32_t kTmemCols = 512;
  griddep_launch_dependents();  // the next kernel may run its prologue while this one works
  if (*reinterpret_cast<volatile int32_t*>(args.status) != kStatusOk) return;  // uniform over the grid
  extern __shared__ uint8_t smem_raw[];
  GemmCtx cx;
  gemm_setup(cx, smem_raw, RING, kStride, ns_fused_staging<BT_MM, BT_MN>(), kTmemCols);
  if (threadIdx.x == 32) {
    for (int par = 0; par < 2; ++par)
      for (int g = 0; g < args.ngroups; ++g) {
        tma_prefetch_desc(&args.gram[par][g].a[0]);
        tma_prefetch_desc(&args.gram[par][g].b[0]);
        tma_prefetch_desc(&args.upd[par][g].a[0]);
        tma_prefetch_desc(&args.upd[par][g].b[0]);
        tma_prefetch_desc(&args.gram[par][g].out[0]);
        tma_prefetch_desc(&args.gram[par][g].out[1]);
        tma_prefetch_desc(&args.upd[par][g].out[0]);
      }
    for (int g = 0; g < args.ngroups; ++g) {
      tma_prefetch_desc(&args.poly[g].a[0]);
      tma_prefetch_desc(&args.poly[g].b[0]);
      tma_prefetch_desc(&args.poly[g].out[0]);
    }
  }
  cx.trace = args.trace;
  uint32_t epoch = 0;
  bool ok = true;
  bool failed = false;
  if (args.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0) args.trace[0] = globaltimer_ns();

  // ---------------- Newton-Schulz iterations
  NsPatch patch;
  for (int g = 0; g < 2; ++g) {
    patch.transposed[g] = args.transposed[g];
    patch.m[g] = args.m[g];
  }
  for (int it = 0; it < args.steps && ok; ++it) {
    const int par = it & 1;
    patch.last = 0;
    patch.alpha = 0.f;
    patch.gamma = args.coef[it][2];
    failed = gemm_phase<OpMM, RING>(cx, args.gram[par], args.ngroups, patch);
    ++cx.phase;
    if (failed) *cx.abort_flag = 1;
    ok = grid_sync(args.barrier, epoch, cx.abort_flag, args.trace);
    if (!ok) break;
    patch.alpha = args.coef[it][1];
    patch.gamma = 0.f;
    failed = gemm_phase<OpMM, RING>(cx, args.poly, args.ngroups, patch);
    ++cx.phase;
    if (failed) *cx.abort_flag = 1;
    ok = grid_sync(args.barrier, epoch, cx.abort_flag, args.trace);
    if (!ok) break;
    patch.alpha = args.coef[it][0];
    patch.last = (it == args.steps - 1);
    failed = gemm_phase<OpMN, RING>(cx, args.upd[par], args.ngroups, patch);
    ++cx.phase;
    if (failed) *cx.abort_flag = 1;
    ok = grid_sync(args.barrier, epoch, cx.abort_flag, args.trace);
  }

  gemm_teardown(cx, !ok, args.status, kTmemCols);
}

}  // namespace lact
