// Host side of liblact_b200: argument validation, TMA tensor-map construction, workspace
// planning, the chunk-recurrence driver and the extern "C" entry points declared in
// include/lact_b200.h.  No device memory is allocated here: all scratch is carved out of the
// caller's workspace.
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "../../include/lact_b200.h"
#include "ns_bwd_fused.cuh"
#include "swa_bwd.cuh"

namespace lact {
namespace {

// ------------------------------------------------------------------------------------------
// tensor maps
// ------------------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode_fn() {
  static EncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
    return reinterpret_cast<EncodeFn>(p);
  }();
  return fn;
}

// A batched row-major bf16 matrix in global memory: [batch][rows][cols], cols contiguous.
struct Mat {
  const void* ptr;
  int64_t rows, cols, ld, batch, bs;  // ld / bs: row / batch stride in elements
};

// Encodes a 3-D map (cols, rows, batch) with a {64, box_rows, 1} box and 128-byte swizzle.
int encode_map(CUtensorMap* map, const Mat& m, uint32_t box_rows) {
  EncodeFn fn = get_encode_fn();
  if (fn == nullptr) return LACT_ERR_CUDA;
  if ((reinterpret_cast<uintptr_t>(m.ptr) & 15) != 0 || (m.ld % 8) != 0 || (m.batch > 1 && (m.bs % 8) != 0))
    return LACT_ERR_SHAPE;
  if (m.rows < 1 || m.cols < 1 || m.batch < 1 || box_rows > 256) return LACT_ERR_SHAPE;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(m.cols), static_cast<cuuint64_t>(m.rows),
                        static_cast<cuuint64_t>(m.batch)};
  const int64_t bs = m.batch > 1 ? m.bs : m.ld * m.rows;
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(m.ld) * 2, static_cast<cuuint64_t>(bs) * 2};
  cuuint32_t box[3] = {64, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(m.ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? LACT_OK : LACT_ERR_CUDA;
}

// Encodes a 4-D map (64 cols of a k-block, rows, k-blocks, batch) of a matrix whose column count is a
// multiple of 64, with a {64, box_rows, kb, 1} box: one load brings `kb` consecutive k-blocks of a row
// block, laid out in shared memory k-block after k-block.
int encode_map_kblocks(CUtensorMap* map, const Mat& m, uint32_t box_rows, uint32_t kb) {
  EncodeFn fn = get_encode_fn();
  if (fn == nullptr) return LACT_ERR_CUDA;
  if ((reinterpret_cast<uintptr_t>(m.ptr) & 15) != 0 || (m.ld % 8) != 0 || (m.batch > 1 && (m.bs % 8) != 0))
    return LACT_ERR_SHAPE;
  if (m.rows < 1 || m.cols < 64 || (m.cols % 64) != 0 || m.batch < 1 || box_rows > 256) return LACT_ERR_SHAPE;
  cuuint64_t dims[4] = {64, static_cast<cuuint64_t>(m.rows), static_cast<cuuint64_t>(m.cols / 64),
                        static_cast<cuuint64_t>(m.batch)};
  const int64_t bs = m.batch > 1 ? m.bs : m.ld * m.rows;
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(m.ld) * 2, 128, static_cast<cuuint64_t>(bs) * 2};
  cuuint32_t box[4] = {64, box_rows, kb, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(m.ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? LACT_OK : LACT_ERR_CUDA;
}

template <class Op>
constexpr int kb_of(const GemmProblem<Op>&) { return Op::KB; }

// Operand of a GEMM: `m` used K-major (mn = rows, k = cols) or MN-major (k = rows, mn = cols); `kb` =
// k-blocks per ring stage of the op that reads it.  With two k-blocks per stage a K-major operand
// whose k extent is whole k-blocks gets the 4-D map (one box per stage), an MN-major operand a box of
// 128 k rows per 64-wide atom.
int make_operand(int kb, CUtensorMap* map, OperandInfo* info, const Mat& m, int mn_major, int tile_rows, int mn_off,
                 int k_off, int batch_off = 0) {
  info->mn_major = mn_major;
  info->k4d = 0;
  info->mn_off = mn_off;
  info->k_off = k_off;
  info->batch_off = batch_off;
  if (((mn_major ? mn_off : k_off) % 8) != 0) return LACT_ERR_SHAPE;  // innermost TMA coordinate: 16-byte rule
  if (mn_major) return encode_map(map, m, static_cast<uint32_t>(64 * kb));
  if (kb == 2 && (m.cols % 64) == 0 && (k_off % 64) == 0) {
    info->k4d = 1;
    return encode_map_kblocks(map, m, static_cast<uint32_t>(tile_rows), 2);
  }
  return encode_map(map, m, static_cast<uint32_t>(tile_rows));
}

// Output of a staged epilogue: bf16 matrix `m` whose extents clip the stored tiles.
int make_output(CUtensorMap* map, OutInfo* info, const Mat& m, int row_off, int col_off, int batch_off = 0) {
  info->row_off = row_off;
  info->col_off = col_off;
  info->batch_off = batch_off;
  info->enabled = 1;
  if ((col_off % 8) != 0 || row_off < 0 || col_off < 0) return LACT_ERR_SHAPE;
  return encode_map(map, m, kBM);
}

// ------------------------------------------------------------------------------------------
// launch accounting and optional per-kernel-class timing
// ------------------------------------------------------------------------------------------
enum KernelClass : int {
  kClsPrepare = 0, kClsGate, kClsDown, kClsGradPointwise, kClsGradContract, kClsMomentumMean, kClsNsPrepare,
  kClsNsGram, kClsNsPoly, kClsNsUpdate, kClsRenorm, kClsNsFused, kClsOther, kNumClasses
};
const char* const kClassNames[kNumClasses] = {
    "prepare_weights", "gemm_swiglu_gate", "gemm_down_proj", "gemm_fwgrad_pointwise", "gemm_fwgrad_contract",
    "momentum_mean", "ns_prepare", "gemm_ns_gram", "gemm_ns_poly", "gemm_ns_update", "add_renorm", "ns_fused", "other"};

struct Profiler {
  std::mutex mu;
  std::atomic<bool> enabled{false};
  std::atomic<int64_t> launches{0};
  struct Rec { cudaEvent_t a, b; int cls; };
  std::vector<Rec> recs;
  std::vector<cudaEvent_t> pool;
  cudaEvent_t get() {
    std::lock_guard<std::mutex> lock(mu);
    if (!pool.empty()) { cudaEvent_t e = pool.back(); pool.pop_back(); return e; }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
  }
};
Profiler g_prof;
std::atomic<int64_t> g_stream_syncs{0};  // cudaStreamSynchronize calls made by the library

// Counts one kernel launch; when timing is enabled, brackets it with two events on its stream.
std::atomic<bool> g_nvtx{false};  // NVTX range around every launch, named after its kernel class

struct KernelScope {
  int cls;
  cudaStream_t stream;
  cudaEvent_t a = nullptr, b = nullptr;
  bool range = false;
  KernelScope(int cls_, cudaStream_t s) : cls(cls_), stream(s) {
    g_prof.launches.fetch_add(1, std::memory_order_relaxed);
    if (g_nvtx.load(std::memory_order_relaxed)) {
      nvtxRangePushA(kClassNames[cls]);
      range = true;
    }
    if (g_prof.enabled.load(std::memory_order_relaxed)) {
      a = g_prof.get();
      b = g_prof.get();
      if (a) cudaEventRecord(a, stream);
    }
  }
  ~KernelScope() {
    if (a && b) {
      cudaEventRecord(b, stream);
      std::lock_guard<std::mutex> lock(g_prof.mu);
      g_prof.recs.push_back({a, b, cls});
    }
    if (range) nvtxRangePop();
  }
};

// ------------------------------------------------------------------------------------------
// launch helpers
// ------------------------------------------------------------------------------------------
#define LACT_TRY(expr)                   \
  do {                                   \
    int _rc = (expr);                    \
    if (_rc != LACT_OK) return _rc;      \
  } while (0)

#define LACT_CUDA(expr)                               \
  do {                                                \
    if ((expr) != cudaSuccess) return LACT_ERR_CUDA;  \
  } while (0)

int check_device() {
  static std::mutex mu;
  static int ok_dev[64] = {0};
  int dev = 0;
  LACT_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(mu);
  if (dev < 64 && ok_dev[dev] == 1) return LACT_OK;
  int major = 0;
  LACT_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10) return LACT_ERR_DEVICE;
  if (dev < 64) ok_dev[dev] = 1;
  return LACT_OK;
}

// Launch with programmatic stream serialization: the kernel's prologue may overlap the tail of the
// previous kernel in the stream; every kernel waits (griddepcontrol.wait) before it touches global memory.
template <class... KArgs, class... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                       Args&&... args) {
  cudaLaunchConfig_t cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  // Measured (10 forward steps of the benchmark shape, same GPU, back to back): 8.16 -> 8.05 ms at 32 (batch x head)
  // units, 3.58 -> 3.39 ms at 8 units, 2.94 -> 2.74 ms at 4 units: the fewer units, the larger the share of the
  // launch gaps that the overlap hides.
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// Launches the first `nprob` problems of `args` as one persistent grid (one CTA per SM at most).
template <class Op, int NPROB>
int launch_gemm(const GemmArgs<Op, NPROB>& args, cudaStream_t stream, int cls, int nprob = NPROB) {
  auto kernel = umma_gemm_kernel<Op, NPROB>;
  constexpr uint32_t smem = gemm_smem_bytes<Op>();
  static_assert(smem <= 232448, "shared memory budget exceeded");
  static std::mutex mu;
  static bool configured[64] = {false};
  int dev = 0;
  LACT_CUDA(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 64 || !configured[dev]) {
      LACT_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      if (dev < 64) configured[dev] = true;
    }
  }
  int64_t tiles = 0;
  for (int p = 0; p < nprob; ++p) {
    const auto& P = args.prob[p];
    if (P.M < 1 || P.N < 1 || P.batch < 1 || P.K < 1) return LACT_ERR_SHAPE;
    tiles += static_cast<int64_t>((P.M + kBM - 1) / kBM) * ((P.N + Op::BT - 1) / Op::BT) * P.batch;
  }
  if (tiles > (1ll << 30)) return LACT_ERR_SHAPE;
  const int grid = static_cast<int>(std::min<int64_t>(tiles, sm_count()));
  KernelScope scope(cls, stream);
  LACT_CUDA(launch_pdl(kernel, dim3(grid), dim3(kGemmThreadsV2), smem, stream, args, nprob));
  return LACT_OK;
}

inline int ceil_div(int64_t a, int64_t b) { return static_cast<int>((a + b - 1) / b); }

// Output-tile width for a single-accumulator GEMM: the candidate with the least padded work over
// the problems of the launch (ties go to the wider tile, whose MMA shape is more efficient).
struct NW { int64_t n, weight; };
int choose_bt(std::initializer_list<NW> probs) {
  const int cands[4] = {256, 192, 128, 64};
  int best = 128;
  int64_t best_cost = -1;
  for (int bt : cands) {
    int64_t cost = 0;
    for (const NW& q : probs) cost += ((q.n + bt - 1) / bt) * bt * q.weight;
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bt; }
  }
  return best;
}

// Instantiates OpT<BT> for the chosen tile width; `fill(args, bt)` populates the problems.
template <template <int> class OpT, int NPROB, class Fill>
int launch_op(int bt, Fill&& fill, cudaStream_t stream, int cls, int nprob) {
#define LACT_OP_CASE(BTV)                                    \
  case BTV: {                                                \
    GemmArgs<OpT<BTV>, NPROB> g;                             \
    std::memset(&g, 0, sizeof(g));                           \
    LACT_TRY(fill(g, BTV));                                  \
    return launch_gemm(g, stream, cls, nprob);               \
  }
  switch (bt) {
    LACT_OP_CASE(64)
    LACT_OP_CASE(128)
    LACT_OP_CASE(192)
    LACT_OP_CASE(256)
    default: return LACT_ERR_CONFIG;
  }
#undef LACT_OP_CASE
}
template <int BT> using OpStoreDirectT = OpBmm<EpiStore, BT>;
template <int BT> using OpStore2T = OpBmm2<EpiStore, BT>;

// ------------------------------------------------------------------------------------------
// building blocks (device pointers in, kernels enqueued)
// ------------------------------------------------------------------------------------------
struct ApplyArgs {
  const bf16* w02b;  // [B][2H][D]
  const bf16* w1b;   // [B][D][H]
  const void* x;     // activations [B][*][D], bf16
  int64_t x_bs, x_ts;
  int64_t start, end;  // token range
  void* out;           // [B][*][D] bf16
  int64_t o_bs, o_ts;
  int64_t out_start;
  bf16* hidden;  // scratch [B][end-start][H]
  int64_t B, D, H;
};

template <int BT>
int launch_gate(const ApplyArgs& a, const Mat& x, const Mat& w02, int64_t len, int32_t* status, cudaStream_t stream) {
  GemmArgs<OpSwigluGate<BT>, 1> g;
  std::memset(&g, 0, sizeof(g));
  auto& P = g.prob[0];
  LACT_TRY(make_operand(kb_of(P), &P.a[0], &P.ai[0], x, 0, kBM, static_cast<int>(a.start), 0));
  LACT_TRY(make_operand(kb_of(P), &P.b[0], &P.bi[0], w02, 0, BT, 0, 0));
  LACT_TRY(make_operand(kb_of(P), &P.b[1], &P.bi[1], w02, 0, BT, static_cast<int>(a.H), 0));
  const Mat hid{a.hidden, len, a.H, a.H, a.B, len * a.H};
  LACT_TRY(make_output(&P.out[0], &P.oi[0], hid, 0, 0));
  P.M = static_cast<int>(len); P.N = static_cast<int>(a.H); P.K = static_cast<int>(a.D);
  P.batch = static_cast<int>(a.B);
  g.status = status;
  return launch_gemm(g, stream, kClsGate);
}

int run_apply(const ApplyArgs& a, int32_t* status, cudaStream_t stream) {
  const int64_t len = a.end - a.start;
  if (len <= 0) return LACT_OK;
  const Mat w02{a.w02b, 2 * a.H, a.D, a.D, a.B, 2 * a.H * a.D};
  const Mat w1{a.w1b, a.D, a.H, a.H, a.B, a.D * a.H};
  const Mat x{a.x, a.end, a.D, a.x_ts, a.B, a.x_bs};
  const Mat hid{a.hidden, len, a.H, a.H, a.B, len * a.H};
  if (a.H % 128 == 0) LACT_TRY(launch_gate<128>(a, x, w02, len, status, stream));
  else LACT_TRY(launch_gate<64>(a, x, w02, len, status, stream));
  const int bt = choose_bt({{a.D, 1}});
  auto fill = [&](auto& g, int btv) -> int {
    auto& P = g.prob[0];
    LACT_TRY(make_operand(kb_of(P), &P.a[0], &P.ai[0], hid, 0, kBM, 0, 0));
    LACT_TRY(make_operand(kb_of(P), &P.b[0], &P.bi[0], w1, 0, btv, 0, 0));
    // rows beyond the range's end must not be written: the map ends at out_start + len
    const Mat om{a.out, a.out_start + len, a.D, a.o_ts, a.B, a.o_bs};
    LACT_TRY(make_output(&P.out[0], &P.oi[0], om, static_cast<int>(a.out_start), 0));
    P.M = static_cast<int>(len); P.N = static_cast<int>(a.D); P.K = static_cast<int>(a.H);
    P.batch = static_cast<int>(a.B);
    g.status = status;
    return LACT_OK;
  };
  return launch_op<OpBmmStore, 1>(bt, fill, stream, kClsDown, 1);
}

struct GradArgs {
  const bf16* w02b;
  const bf16* w1b;
  const void *k, *v;
  int64_t k_bs, k_ts, v_bs, v_ts;
  int64_t start, end;
  const void *lr0, *lr1, *lr2;
  int32_t lr_f32;
  int64_t lr_bs;
  float w_scale;
  bf16* dy02;  // scratch [B][len][2H]
  bf16* hid;   // scratch [B][len][H]
  void* g02;   // [B][2H][D] fp32 (state) or bf16
  void* g1;    // [B][D][H]
  int32_t g_f32;
  const float* beta;  // [B] or nullptr
  int64_t B, D, H;
  float* partial02 = nullptr;  // optional per-tile sums of squares of the two outputs
  float* partial1 = nullptr;
  bf16* gb02 = nullptr;        // optional bf16 copies of the two outputs (Newton-Schulz input)
  bf16* gb1 = nullptr;
  const float* g02_prev = nullptr;  // optional: momentum state read from here instead of g02 / g1 (fp32)
  const float* g1_prev = nullptr;
};

inline int contract_bt(int64_t D, int64_t H) { return choose_bt({{D, 2 * H}, {H, D}}); }

// Pointwise stage: dy02 = [dy0 | dy2] ([B][len][2H]) and hid = hidden * lr1 ([B][len][H]) for tokens [start, end).
int run_grad_pointwise(const GradArgs& a, int32_t* status, cudaStream_t stream) {
  const int64_t len = a.end - a.start;
  if (len <= 0) return LACT_ERR_STEPS;
  const Mat w02{a.w02b, 2 * a.H, a.D, a.D, a.B, 2 * a.H * a.D};
  const Mat w1{a.w1b, a.D, a.H, a.H, a.B, a.D * a.H};
  const Mat km{a.k, a.end, a.D, a.k_ts, a.B, a.k_bs};
  const Mat vm{a.v, a.end, a.D, a.v_ts, a.B, a.v_bs};
  const Mat hid{a.hid, len, a.H, a.H, a.B, len * a.H};
  GemmArgs<OpFwGradPointwise, 1> g;
  std::memset(&g, 0, sizeof(g));
  auto& P = g.prob[0];
  constexpr int BT = OpFwGradPointwise::BT;
  LACT_TRY(make_operand(kb_of(P), &P.a[0], &P.ai[0], km, 0, kBM, static_cast<int>(a.start), 0));
  LACT_TRY(make_operand(kb_of(P), &P.a[1], &P.ai[1], vm, 0, kBM, static_cast<int>(a.start), 0));
  LACT_TRY(make_operand(kb_of(P), &P.b[0], &P.bi[0], w02, 0, BT, 0, 0));
  LACT_TRY(make_operand(kb_of(P), &P.b[1], &P.bi[1], w02, 0, BT, static_cast<int>(a.H), 0));
  // dh = v w1: w1 is [D][H], i.e. k (= D) rows with the n (= H) axis contiguous
  LACT_TRY(make_operand(kb_of(P), &P.b[2], &P.bi[2], w1, 1, BT, 0, 0));
  P.M = static_cast<int>(len); P.N = static_cast<int>(a.H); P.K = static_cast<int>(a.D);
  P.batch = static_cast<int>(a.B);
  P.ep = EpiFwGrad{a.lr0, a.lr1, a.lr2, a.lr_f32, static_cast<int32_t>(a.start), a.lr_bs, a.w_scale};
  // dy0 and dy2 share the [len][2H] plane: two maps of H columns each, so neither can spill
  const Mat dy0m{a.dy02, len, a.H, 2 * a.H, a.B, len * 2 * a.H};
  const Mat dy2m{a.dy02 + a.H, len, a.H, 2 * a.H, a.B, len * 2 * a.H};
  LACT_TRY(make_output(&P.out[0], &P.oi[0], dy0m, 0, 0));
  LACT_TRY(make_output(&P.out[1], &P.oi[1], dy2m, 0, 0));
  LACT_TRY(make_output(&P.out[2], &P.oi[2], hid, 0, 0));
  g.status = status;
  return launch_gemm(g, stream, kClsGradPointwise);
}

int run_grad(const GradArgs& a, int32_t* status, cudaStream_t stream) {
  const int64_t len = a.end - a.start;
  LACT_TRY(run_grad_pointwise(a, status, stream));
  const Mat km{a.k, a.end, a.D, a.k_ts, a.B, a.k_bs};
  const Mat vm{a.v, a.end, a.D, a.v_ts, a.B, a.v_bs};
  const Mat dy{a.dy02, len, 2 * a.H, 2 * a.H, a.B, len * 2 * a.H};
  const Mat hid{a.hid, len, a.H, a.H, a.B, len * a.H};
  // token contraction: [dw0; dw2] = dy02^T k  and  dw1 = v^T hidden
  const int bt = contract_bt(a.D, a.H);
  auto fill = [&](auto& g, int btv) -> int {
    auto& P0 = g.prob[0];
    LACT_TRY(make_operand(kb_of(P0), &P0.a[0], &P0.ai[0], dy, 1, kBM, 0, 0));
    LACT_TRY(make_operand(kb_of(P0), &P0.b[0], &P0.bi[0], km, 1, btv, 0, static_cast<int>(a.start)));
    P0.M = static_cast<int>(2 * a.H); P0.N = static_cast<int>(a.D); P0.K = static_cast<int>(len);
    P0.batch = static_cast<int>(a.B);
    P0.ep = EpiDW{a.g02, 2 * a.H * a.D, a.D, a.beta, 1, a.g_f32, a.partial02, ceil_div(2 * a.H, kBM),
                  ceil_div(a.D, btv), a.gb02, a.g02_prev};
    auto& P1 = g.prob[1];
    LACT_TRY(make_operand(kb_of(P1), &P1.a[0], &P1.ai[0], vm, 1, kBM, 0, static_cast<int>(a.start)));
    LACT_TRY(make_operand(kb_of(P1), &P1.b[0], &P1.bi[0], hid, 1, btv, 0, 0));
    P1.M = static_cast<int>(a.D); P1.N = static_cast<int>(a.H); P1.K = static_cast<int>(len);
    P1.batch = static_cast<int>(a.B);
    P1.ep = EpiDW{a.g1, a.D * a.H, a.H, a.beta, 1, a.g_f32, a.partial1, ceil_div(a.D, kBM), ceil_div(a.H, btv),
                  a.gb1, a.g1_prev};
    g.status = status;
    return LACT_OK;
  };
  return launch_op<OpDW, 2>(bt, fill, stream, kClsGradContract, 2);
}

// Newton-Schulz coefficient schedules.
const float kNsTuned[5][3] = {{4.0848f, -6.8946f, 2.9270f},
                              {3.9505f, -6.3029f, 2.6377f},
                              {3.7418f, -5.5913f, 2.3037f},
                              {2.8769f, -3.1427f, 1.2046f},
                              {2.8366f, -3.0525f, 1.2012f}};
const float kNsConst[3] = {3.4445f, -4.7750f, 2.0315f};

constexpr int kNsMaxParts = 512;

// One group of equally shaped gradient matrices [R][C] under iteration.  The iterate X keeps the
// gradient's own [R][C] layout.  With m = min(R, C), n = max(R, C) the Gram matrix is m x m:
//   wide (R <= C):               A = X X^T   (operands K-major),       X' = P X    (X read MN-major)
//   tall (R > C, `transposed`):  A = X^T X   (operands MN-major),      X' = X P^T  (P's rows as K-major B operand)
// which is the reference's "transpose, iterate, transpose back" without moving data.
struct NsGroup {
  int32_t nmat, R, C, m, n, transposed;
  bf16 *xa, *xb;              // ping-pong iterates, nmat * R * C each
  bf16 *gram, *poly;  // [nmat][m][m]: shifted Gram matrix S = A + (b / 2c) I and polynomial P
  float* partial;             // [nmat][<= kNsMaxParts] partial sums of squares
  float* scale;               // [nmat] 1 / (||G||_F + 1e-7) when the first iterate is the unscaled bf16(G)
  uint32_t* done;             // [nmat] tile completion counters of the fused kernel
};

inline size_t ns_group_bytes(int64_t nmat, int64_t m, int64_t n) {
  return static_cast<size_t>(nmat) * (2 * m * n + 3 * m * m) * 2 + static_cast<size_t>(nmat) * kNsMaxParts * 4 +
         static_cast<size_t>(nmat) * 8 + 8 * 256;
}

void ns_group_init(NsGroup& g, int64_t nmat, int64_t R, int64_t C, int gram_right) {
  g.nmat = static_cast<int32_t>(nmat);
  g.R = static_cast<int32_t>(R);
  g.C = static_cast<int32_t>(C);
  g.m = static_cast<int32_t>(std::min(R, C));
  g.n = static_cast<int32_t>(std::max(R, C));
  g.transposed = (R > C) || (R == C && gram_right);
}

// columns of the update product's output: X' is [R][C] = [m][n] (wide) or [n][m] (tall)
inline int ns_upd_cols(const NsGroup& g) { return g.transposed ? g.m : g.n; }
inline int ns_upd_rows(const NsGroup& g) { return g.transposed ? g.n : g.m; }

// Start of the iteration for one or two groups (src[g]: [nmat][R][C], contiguous).
//   scaled = 1: the first iterate X0 = bf16(bf16(G) / (||G|| + 1e-7)) is written to grp[g].xa
//               (norm partials from `fused_parts`, or computed here);
//   scaled = 0: the first iterate is bf16(G), already in grp[g].xa with `fused_parts` partial sums
//               per matrix; only the scale factors 1 / (||G|| + 1e-7) are computed.
int launch_ns_prepare(const NsGroup* grp, int ngroups, const void* const* src, int src_f32, int scaled,
                      cudaStream_t stream, const int* fused_parts = nullptr) {
  NsPrepArgs pa;
  std::memset(&pa, 0, sizeof(pa));
  pa.ngroups = ngroups;
  int nmat = 0, tiles = 0;
  bool need_sumsq = false;
  for (int g = 0; g < ngroups; ++g) {
    const NsGroup& G = grp[g];
    const int parts = (fused_parts != nullptr && fused_parts[g] > 0) ? fused_parts[g] : kNsSlabs;
    if (fused_parts == nullptr || fused_parts[g] <= 0) need_sumsq = true;
    pa.grp[g] = NsPrepGroup{src[g], src_f32, G.nmat, G.R, G.C, G.xa, G.partial, parts, G.scale, G.done};
    nmat += G.nmat;
    tiles = std::max(tiles, ceil_div(G.R, 64) * ceil_div(G.C, 64));
  }
  if (need_sumsq) {
    if (fused_parts != nullptr) return LACT_ERR_CONFIG;  // all groups or none
    KernelScope scope(kClsNsPrepare, stream);
    LACT_CUDA(launch_pdl(ns_sumsq_kernel, dim3(nmat, kNsSlabs), dim3(256), 0, stream, pa));
  }
  KernelScope scope(kClsNsPrepare, stream);
  if (scaled) LACT_CUDA(launch_pdl(ns_scale_kernel, dim3(nmat, tiles), dim3(256), 0, stream, pa));
  else LACT_CUDA(launch_pdl(ns_den_kernel, dim3(ceil_div(nmat, 4)), dim3(128), 0, stream, pa));
  return LACT_OK;
}

// Fills the three contractions of one iteration of group G, reading the iterate `cur` and writing
// `nxt` (both [nmat][R][C]).  PG / PP / PU: GemmProblem<OpNs<..>> of the gram, poly and update phase.
template <class PG, class PP, class PU>
int wire_ns_group(const NsGroup& G, bf16* cur, bf16* nxt, int bt_mm, int bt_mn, PG& gram, PP& poly, PU& upd) {
  const int64_t mm = static_cast<int64_t>(G.m) * G.m, rc = static_cast<int64_t>(G.R) * G.C;
  const Mat X{cur, G.R, G.C, G.C, G.nmat, rc};
  const Mat XN{nxt, G.R, G.C, G.C, G.nmat, rc};
  const Mat S{G.gram, G.m, G.m, G.m, G.nmat, mm};
  const Mat PB{G.poly, G.m, G.m, G.m, G.nmat, mm};
  const int tall = G.transposed;
  // gram: S = X X^T (wide) / X^T X (tall) + (b / 2c) I
  LACT_TRY(make_operand(kb_of(gram), &gram.a[0], &gram.ai[0], X, tall, kBM, 0, 0));
  LACT_TRY(make_operand(kb_of(gram), &gram.b[0], &gram.bi[0], X, tall, bt_mm, 0, 0));
  gram.M = G.m; gram.N = G.m; gram.K = G.n; gram.batch = G.nmat;
  LACT_TRY(make_output(&gram.out[0], &gram.oi[0], S, 0, 0));
  // poly: P = c S S + (a - b^2 / 4c) I   (S is exactly symmetric: its rows serve as the K-major B operand too)
  LACT_TRY(make_operand(kb_of(poly), &poly.a[0], &poly.ai[0], S, 0, kBM, 0, 0));
  LACT_TRY(make_operand(kb_of(poly), &poly.b[0], &poly.bi[0], S, 0, bt_mm, 0, 0));
  poly.M = G.m; poly.N = G.m; poly.K = G.m; poly.batch = G.nmat;
  LACT_TRY(make_output(&poly.out[0], &poly.oi[0], PB, 0, 0));
  // update: X' = poly X (wide; X is [k][n]: MN-major B operand) / X' = X poly^T (tall)
  if (!tall) {
    LACT_TRY(make_operand(kb_of(upd), &upd.a[0], &upd.ai[0], PB, 0, kBM, 0, 0));
    LACT_TRY(make_operand(kb_of(upd), &upd.b[0], &upd.bi[0], X, 1, bt_mn, 0, 0));
  } else {
    LACT_TRY(make_operand(kb_of(upd), &upd.a[0], &upd.ai[0], X, 0, kBM, 0, 0));
    LACT_TRY(make_operand(kb_of(upd), &upd.b[0], &upd.bi[0], PB, 0, bt_mn, 0, 0));
  }
  upd.M = ns_upd_rows(G); upd.N = ns_upd_cols(G); upd.K = G.m; upd.batch = G.nmat;
  LACT_TRY(make_output(&upd.out[0], &upd.oi[0], XN, 0, 0));
  return LACT_OK;
}

inline void ns_tile_widths(const NsGroup* grp, int ngroups, int* bt_mm, int* bt_mn) {
  const NsGroup& G0 = grp[0];
  const NsGroup& G1 = grp[ngroups - 1];
  *bt_mm = choose_bt({{G0.m, static_cast<int64_t>(G0.nmat) * G0.m}, {G1.m, static_cast<int64_t>(G1.nmat) * G1.m}});
  *bt_mn = choose_bt({{ns_upd_cols(G0), static_cast<int64_t>(G0.nmat) * ns_upd_rows(G0)},
                      {ns_upd_cols(G1), static_cast<int64_t>(G1.nmat) * ns_upd_rows(G1)}});
}

// Runs `steps` iterations on one or two groups, one launch per contraction (every launch covers
// all groups).  The first iterate is grp[g].xa (scaled unless `unscaled_first`, in which case the
// scale factors grp[g].scale are folded into the first iteration).
// result[g] = buffer holding the final iterate of group g.
int run_ns_iterations(const NsGroup* grp, int ngroups, int steps, int const_coeffs, const bf16** result,
                      int32_t* status, cudaStream_t stream, int unscaled_first = 0, int coef_offset = 0) {
  // `steps` iterations of the schedule starting at iteration `coef_offset` (the tuned table has five
  // entries; the public entry points insist on all five)
  if (ngroups < 1 || ngroups > 2) return LACT_ERR_CONFIG;
  if (!const_coeffs && steps + coef_offset > 5) return LACT_ERR_CONFIG;
  bf16* cur[2];
  bf16* nxt[2];
  for (int g = 0; g < ngroups; ++g) { cur[g] = grp[g].xa; nxt[g] = grp[g].xb; }
  int bt_mm = 0, bt_mn = 0;
  ns_tile_widths(grp, ngroups, &bt_mm, &bt_mn);
  for (int it = 0; it < steps; ++it) {
    const float* co = const_coeffs ? kNsConst : kNsTuned[it + coef_offset];
    const int fold = (it == 0 && unscaled_first) ? 1 : 0;
    // which = 0 gram, 1 poly, 2 update: every fill wires all three and keeps the one it launches
    auto fill = [&](auto& ga, int btv, int which) -> int {
      using Prob = std::remove_reference_t<decltype(ga.prob[0])>;
      for (int g = 0; g < ngroups; ++g) {
        Prob pg, pp, pu;
        std::memset(&pg, 0, sizeof(Prob)); std::memset(&pp, 0, sizeof(Prob)); std::memset(&pu, 0, sizeof(Prob));
        LACT_TRY(wire_ns_group(grp[g], cur[g], nxt[g], btv, btv, pg, pp, pu));
        const float* sc = fold ? grp[g].scale : nullptr;
        if (which == 0) { ga.prob[g] = pg; ga.prob[g].ep = EpiNs{co[1] / (2.f * co[2]), 1.f, sc, fold ? 2 : 0}; }
        if (which == 1) {
          ga.prob[g] = pp;
          ga.prob[g].ep = EpiNs{co[0] - co[1] * co[1] / (4.f * co[2]), co[2], nullptr, 0};
        }
        if (which == 2) { ga.prob[g] = pu; ga.prob[g].ep = EpiNs{0.f, 1.f, sc, fold ? 1 : 0}; }
      }
      ga.status = status;
      return LACT_OK;
    };
    LACT_TRY((launch_op<OpNs, 2>(bt_mm, [&](auto& ga, int btv) { return fill(ga, btv, 0); }, stream, kClsNsGram, ngroups)));
    LACT_TRY((launch_op<OpNs, 2>(bt_mm, [&](auto& ga, int btv) { return fill(ga, btv, 1); }, stream, kClsNsPoly, ngroups)));
    LACT_TRY((launch_op<OpNs, 2>(bt_mn, [&](auto& ga, int btv) { return fill(ga, btv, 2); }, stream, kClsNsUpdate, ngroups)));
    for (int g = 0; g < ngroups; ++g) std::swap(cur[g], nxt[g]);
  }
  for (int g = 0; g < ngroups; ++g) result[g] = cur[g];
  return LACT_OK;
}

// Fused path: all iterations in one cooperative launch.  launch_ns_prepare must have run on the same groups
// just before: it leaves the first iterates in grp[g].xa and clears the completion counters grp[g].done.
// NITER = 2: iterates ping-pong between grp[g].xa / xb, one Gram / polynomial buffer.  NITER > 2 (steps <= NITER):
// every iteration has its own buffers, `keep[g]` = {iterates (steps + 1) x [nmat][R][C] starting with the first
// iterate, shifted Gram matrices steps x [nmat][m][m], polynomials likewise}.
struct NsKeep {
  bf16 *X, *A, *P;
};
template <int BT_MM, int BT_MN, int NITER, bool SYM = false>
int launch_ns_fused(const NsGroup* grp, int ngroups, int steps, int const_coeffs, int32_t* status,
                    cudaStream_t stream, int unscaled_first, const NsKeep* keep = nullptr, int coef_offset = 0) {
  using Args = NsFusedArgs<BT_MM, BT_MN, NITER, SYM>;
  auto kernel = ns_fused_kernel<BT_MM, BT_MN, NITER, SYM>;
  constexpr uint32_t smem = ns_fused_smem_bytes<BT_MM, BT_MN, SYM>();
  static_assert(smem <= 232448, "shared memory budget exceeded");
  static_assert(ns_fused_ring<BT_MM, BT_MN, SYM>() >= 2, "ring too shallow");
  static std::mutex mu;
  static bool configured[64] = {false};
  int dev = 0;
  LACT_CUDA(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 64 || !configured[dev]) {
      LACT_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      if (dev < 64) configured[dev] = true;
    }
  }
  if (NITER > 2 && (keep == nullptr || steps > NITER)) return LACT_ERR_CONFIG;
  // the argument block (a few KB per problem set) lives on the heap: it is copied at launch
  std::vector<uint8_t> storage(sizeof(Args));
  Args& args = *reinterpret_cast<Args*>(storage.data());
  std::memset(&args, 0, sizeof(args));
  int64_t max_tiles = 1;
  for (int g = 0; g < ngroups; ++g) {
    const NsGroup& G = grp[g];
    const int64_t rc = static_cast<int64_t>(G.nmat) * G.R * G.C, mm = static_cast<int64_t>(G.nmat) * G.m * G.m;
    for (int par = 0; par < NITER; ++par) {
      NsGroup Gi = G;
      bf16 *cur, *nxt;
      if (NITER == 2) {
        cur = par == 0 ? G.xa : G.xb;
        nxt = par == 0 ? G.xb : G.xa;
      } else {
        cur = keep[g].X + rc * par;
        nxt = keep[g].X + rc * (par + 1);
        Gi.gram = keep[g].A + mm * par;
        Gi.poly = keep[g].P + mm * par;
      }
      LACT_TRY(wire_ns_group(Gi, cur, nxt, BT_MM, BT_MN, args.gram[par][g], args.poly[par][g], args.upd[par][g]));
    }
    args.scale[g] = unscaled_first ? G.scale : nullptr;
    max_tiles = std::max<int64_t>(max_tiles, static_cast<int64_t>(G.nmat) * ceil_div(ns_upd_rows(G), kBM) *
                                                 ceil_div(ns_upd_cols(G), BT_MN) * ngroups);
  }
  for (int it = 0; it < steps; ++it) {
    const float* co = const_coeffs ? kNsConst : kNsTuned[it + coef_offset];
    args.coef[it][0] = co[0]; args.coef[it][1] = co[1]; args.coef[it][2] = co[2];
  }
  args.steps = steps;
  args.ngroups = ngroups;
  args.status = status;
  for (int g = 0; g < ngroups; ++g) args.done[g] = grp[g].done;  // cleared by launch_ns_prepare
  const int grid = static_cast<int>(std::min<int64_t>(sm_count(), std::max<int64_t>(max_tiles, 8)));
  void* kargs[] = {&args};
  KernelScope scope(kClsNsFused, stream);
  LACT_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kernel), dim3(grid), dim3(kGemmThreadsFlow), kargs, smem,
                                        stream));
  return LACT_OK;
}

// Picks the fused kernel instantiated for the tile widths this problem wants; returns
// LACT_ERR_CONFIG when there is none (the caller then runs the multi-launch path).
int try_ns_fused(const NsGroup* grp, int ngroups, int steps, int const_coeffs, int32_t* status,
                 cudaStream_t stream, const bf16** result, int unscaled_first = 0, const NsKeep* keep = nullptr) {
  if (steps < 1 || steps > kNsFusedMaxSteps) return LACT_ERR_CONFIG;
  if (!const_coeffs && steps != 5) return LACT_ERR_CONFIG;
  if (keep != nullptr && steps > 5) return LACT_ERR_CONFIG;
  int bt_mm = 0, bt_mn = 0;
  ns_tile_widths(grp, ngroups, &bt_mm, &bt_mn);
  for (int g = 0; g < ngroups; ++g) {
    if (keep != nullptr) result[g] = keep[g].X + static_cast<int64_t>(grp[g].nmat) * grp[g].R * grp[g].C * steps;
    else result[g] = (steps % 2 == 0) ? grp[g].xa : grp[g].xb;
  }
  // Few matrices per launch (a small (batch x head) shard): the kernel is bound by the 15-phase chain of each
  // matrix, not by throughput, so narrower tiles that spread every phase over more SMs (and shorten the serial
  // work per tile) win.  Tiles of the Gram phase at width bt over all groups:
  auto gram_tiles = [&](int bt) {
    int64_t t = 0;
    for (int g = 0; g < ngroups; ++g) t += static_cast<int64_t>(grp[g].nmat) * ceil_div(grp[g].m, kBM) * ceil_div(grp[g].m, bt);
    return t;
  };
  // keep == nullptr: iterates ping-pong (two problem sets); else every iteration keeps its buffers (five sets)
#define LACT_NS_FUSED(BTV)                                                                                          \
  (keep == nullptr ? launch_ns_fused<BTV, BTV, 2>(grp, ngroups, steps, const_coeffs, status, stream, unscaled_first) \
                   : launch_ns_fused<BTV, BTV, 5>(grp, ngroups, steps, const_coeffs, status, stream, unscaled_first, keep))
  const int64_t want = static_cast<int64_t>(sm_count()) * 3 / 4;
  // Gram side a multiple of 128 in every group and plenty of matrices: the symmetric phases (Gram matrix, polynomial)
  // run on 128 x 128 tiles on and above the diagonal only, the update keeps its 192-wide tiles.  With fewer matrices
  // (measured at D = H = 384: 16 and 12 units, i.e. under 1.5 Gram tiles of width 192 per SM) the symmetric phases
  // leave a second, nearly empty round of tiles and plain 128-wide tiles are 4-5 % faster; from 20 units up the
  // symmetric variant wins.
  const bool wide = bt_mm == 192 && bt_mn == 192;
  bool symmable = wide;
  for (int g = 0; g < ngroups; ++g) symmable = symmable && grp[g].m % kBM == 0 && grp[g].m >= 2 * kBM;
  if (symmable && gram_tiles(192) >= static_cast<int64_t>(sm_count()) * 3 / 2)
    return keep == nullptr
               ? launch_ns_fused<128, 192, 2, true>(grp, ngroups, steps, const_coeffs, status, stream, unscaled_first)
               : launch_ns_fused<128, 192, 5, true>(grp, ngroups, steps, const_coeffs, status, stream, unscaled_first, keep);
  if (wide && !symmable && gram_tiles(192) >= want) return LACT_NS_FUSED(192);
  // (a 256-wide update tile leaves no room for a useful ring next to two staging tiles: 128 is used)
  const bool ok128 = (bt_mm == 192 && bt_mn == 192) || (bt_mm == 128 && (bt_mn == 128 || bt_mn == 256));
  if (ok128 && (gram_tiles(128) >= want || gram_tiles(64) == gram_tiles(128))) return LACT_NS_FUSED(128);
  if (ok128 || (bt_mm == 64 && bt_mn == 64)) return LACT_NS_FUSED(64);
#undef LACT_NS_FUSED
  return LACT_ERR_CONFIG;
}

// ------------------------------------------------------------------------------------------
// workspace planning
// ------------------------------------------------------------------------------------------
struct Carver {
  uint8_t* base;
  size_t off = 0;
  explicit Carver(void* b) : base(static_cast<uint8_t*>(b)) {}
  template <class T>
  T* take(size_t count) {
    off = (off + 255) & ~static_cast<size_t>(255);
    T* p = base ? reinterpret_cast<T*>(base + off) : nullptr;
    off += count * sizeof(T);
    return p;
  }
};

struct NsPlan {
  int ngroups;
  NsGroup grp[2];
};

void carve_ns_group(Carver& c, NsGroup& g) {
  const size_t mn = static_cast<size_t>(g.nmat) * g.m * g.n, mm = static_cast<size_t>(g.nmat) * g.m * g.m;
  g.xa = c.take<bf16>(mn);
  g.xb = c.take<bf16>(mn);
  g.gram = c.take<bf16>(mm);
  g.poly = c.take<bf16>(mm);
  g.partial = c.take<float>(static_cast<size_t>(g.nmat) * kNsMaxParts);
  g.scale = c.take<float>(static_cast<size_t>(g.nmat));
  g.done = c.take<uint32_t>(static_cast<size_t>(g.nmat));
}

// Group 0 orthogonalises the [w0; w2] gradient (concat: B matrices [2H][D]; separate: 2B matrices
// [H][D], w0 and w2 of batch b at 2b, 2b+1), group 1 the w1 gradient (B matrices [D][H]).
void plan_ns(Carver& c, int64_t B, int64_t D, int64_t H, int concat, int gram_right, NsPlan* plan) {
  plan->ngroups = 2;
  if (concat) ns_group_init(plan->grp[0], B, 2 * H, D, gram_right);
  else ns_group_init(plan->grp[0], 2 * B, H, D, gram_right);
  ns_group_init(plan->grp[1], B, D, H, gram_right);
  carve_ns_group(c, plan->grp[0]);
  carve_ns_group(c, plan->grp[1]);
}

// Trace layout in the caller's buffer (bf16 unless noted): group scratch (norm partials,
// scale factors); X[0..steps] ([B][R][C] each); shifted Gram matrix A + (b/2c) I and polynomial P per iteration
// ([B][m][m]); then the backward's temporaries: c A + (b/2) I, Q, S ([B][m][m]) and two [B][R][C] gradient buffers.
struct NsTrace {
  NsGroup grp;
  bf16* X;   // (steps + 1) iterates
  bf16 *A, *P;  // steps matrices each (A: the shifted Gram matrix)
  bf16 *CB, *Q, *S, *dXa, *dXb;
  size_t bytes;
};

int plan_ns_trace(void* base, int64_t B, int64_t R, int64_t C, int steps, int gram_right, NsTrace* t) {
  if (B < 1 || B > 65535 || R < 8 || C < 8 || (R % 8) || (C % 8) || steps < 1 || steps > 16) return LACT_ERR_SHAPE;
  Carver cv(base);
  ns_group_init(t->grp, B, R, C, gram_right);
  const size_t rc = static_cast<size_t>(B) * R * C, mm = static_cast<size_t>(B) * t->grp.m * t->grp.m;
  t->grp.partial = cv.take<float>(static_cast<size_t>(B) * kNsMaxParts);
  t->grp.scale = cv.take<float>(B);
  t->grp.done = cv.take<uint32_t>(static_cast<size_t>(B) + 64);
  t->X = cv.take<bf16>(rc * (steps + 1));
  t->A = cv.take<bf16>(mm * steps);
  t->P = cv.take<bf16>(mm * steps);
  t->CB = cv.take<bf16>(mm);
  t->Q = cv.take<bf16>(mm);
  t->S = cv.take<bf16>(mm);
  t->dXa = cv.take<bf16>(rc);
  t->dXb = cv.take<bf16>(rc);
  t->bytes = cv.off + 256;
  return LACT_OK;
}


static int ns_norm_bwd_launch(const float* g, const void* dx0, int dx_bf16, float* dg, float* partials, int64_t nmat,
                              int64_t elems, cudaStream_t s) {
  if (nmat < 1 || nmat > 65535 * 16 || elems < 4 || (elems % 4) != 0) return LACT_ERR_SHAPE;
  if (((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(dx0) | reinterpret_cast<uintptr_t>(dg)) & 15) != 0)
    return LACT_ERR_SHAPE;
  const dim3 grid(static_cast<unsigned>(nmat), kNormBwdSlices);
  {
    KernelScope scope(kClsOther, s);
    ns_norm_bwd_partial_kernel<<<grid, 512, 0, s>>>(g, dx0, dx_bf16, partials, elems);
    LACT_CUDA(cudaGetLastError());
  }
  KernelScope scope(kClsOther, s);
  ns_norm_bwd_apply_kernel<<<grid, 512, 0, s>>>(g, dx0, dx_bf16, dg, partials, elems);
  LACT_CUDA(cudaGetLastError());
  return LACT_OK;
}

// ---- all iterations of the Newton-Schulz backward of one or two groups in one cooperative launch
template <int BT_MM, int BT, bool SYM>
static int launch_ns_bwd_fused(const NsTrace* tr, const bf16* const* du, int ngroups, int steps, int const_coeffs,
                               int32_t* status, cudaStream_t stream) {
  constexpr int NITER = 5;
  using Args = NsBwdFusedArgs<BT_MM, BT, NITER, SYM>;
  auto kernel = ns_bwd_fused_kernel<BT_MM, BT, NITER, SYM>;
  constexpr uint32_t smem = ns_bwd_smem_bytes<BT_MM, BT, SYM>();
  static_assert(smem <= 232448, "shared memory budget exceeded");
  static_assert(ns_bwd_ring<BT_MM, BT, SYM>() >= 2, "ring too shallow");
  static_assert(sizeof(Args) <= 32000, "kernel parameter block too large");
  static std::mutex mu;
  static bool configured[64] = {false};
  int dev = 0;
  LACT_CUDA(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 64 || !configured[dev]) {
      LACT_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      if (dev < 64) configured[dev] = true;
    }
  }
  std::vector<uint8_t> storage(sizeof(Args));
  Args& args = *reinterpret_cast<Args*>(storage.data());
  std::memset(&args, 0, sizeof(args));
  int64_t max_tiles = 1;
  for (int g = 0; g < ngroups; ++g) {
    const NsTrace& t = tr[g];
    const NsGroup& G = t.grp;
    const int64_t rc1 = static_cast<int64_t>(G.R) * G.C, mm1 = static_cast<int64_t>(G.m) * G.m;
    const int64_t rc = rc1 * G.nmat, mm = mm1 * G.nmat;
    const int tall = G.transposed;
    const Mat Q{t.Q, G.m, G.m, G.m, G.nmat, mm1};
    const Mat T{t.S, G.m, G.m, G.m, G.nmat, mm1};
    const bf16* dX = du[g];
    for (int it = steps - 1; it >= 0; --it) {
      bf16* out = (it & 1) ? t.dXa : t.dXb;
      const Mat X{t.X + rc * it, G.R, G.C, G.C, G.nmat, rc1};
      const Mat D{dX, G.R, G.C, G.C, G.nmat, rc1};
      const Mat O{out, G.R, G.C, G.C, G.nmat, rc1};
      const Mat S{t.A + mm * it, G.m, G.m, G.m, G.nmat, mm1};
      const Mat PB{t.P + mm * it, G.m, G.m, G.m, G.nmat, mm1};
      auto& pq = args.q[it][g];
      auto& pt = args.t[it][g];
      auto& px = args.dx[it][g];
      // Q = dX X^T + X dX^T (wide; the iterate's rows are K-major operands) / dX^T X + X^T dX (tall; MN-major)
      LACT_TRY(make_operand(1, &pq.a[0], &pq.ai[0], D, tall, kBM, 0, 0));
      LACT_TRY(make_operand(1, &pq.b[0], &pq.bi[0], X, tall, BT_MM, 0, 0));
      LACT_TRY(make_operand(1, &pq.a[1], &pq.ai[1], X, tall, kBM, 0, 0));
      LACT_TRY(make_operand(1, &pq.b[1], &pq.bi[1], D, tall, BT_MM, 0, 0));
      pq.M = G.m; pq.N = G.m; pq.K = G.n; pq.batch = G.nmat;
      LACT_TRY(make_output(&pq.out[0], &pq.oi[0], Q, 0, 0));
      // T = c (S Q + Q S): all three symmetric, rows serve as K-major operands on either side
      LACT_TRY(make_operand(1, &pt.a[0], &pt.ai[0], S, 0, kBM, 0, 0));
      LACT_TRY(make_operand(1, &pt.b[0], &pt.bi[0], Q, 0, BT_MM, 0, 0));
      LACT_TRY(make_operand(1, &pt.a[1], &pt.ai[1], Q, 0, kBM, 0, 0));
      LACT_TRY(make_operand(1, &pt.b[1], &pt.bi[1], S, 0, BT_MM, 0, 0));
      pt.M = G.m; pt.N = G.m; pt.K = G.m; pt.batch = G.nmat;
      LACT_TRY(make_output(&pt.out[0], &pt.oi[0], T, 0, 0));
      // dX_i = P dX + T X (wide: the [k][n] iterates are MN-major B operands) / dX P + X T (tall)
      if (!tall) {
        LACT_TRY(make_operand(1, &px.a[0], &px.ai[0], PB, 0, kBM, 0, 0));
        LACT_TRY(make_operand(1, &px.b[0], &px.bi[0], D, 1, BT, 0, 0));
        LACT_TRY(make_operand(1, &px.a[1], &px.ai[1], T, 0, kBM, 0, 0));
        LACT_TRY(make_operand(1, &px.b[1], &px.bi[1], X, 1, BT, 0, 0));
      } else {
        LACT_TRY(make_operand(1, &px.a[0], &px.ai[0], D, 0, kBM, 0, 0));
        LACT_TRY(make_operand(1, &px.b[0], &px.bi[0], PB, 0, BT, 0, 0));
        LACT_TRY(make_operand(1, &px.a[1], &px.ai[1], X, 0, kBM, 0, 0));
        LACT_TRY(make_operand(1, &px.b[1], &px.bi[1], T, 0, BT, 0, 0));
      }
      px.M = ns_upd_rows(G); px.N = ns_upd_cols(G); px.K = G.m; px.batch = G.nmat;
      LACT_TRY(make_output(&px.out[0], &px.oi[0], O, 0, 0));
      dX = out;
    }
    args.done[g] = G.done;
    LACT_CUDA(cudaMemsetAsync(G.done, 0, sizeof(uint32_t) * G.nmat, stream));
    max_tiles = std::max<int64_t>(max_tiles, static_cast<int64_t>(G.nmat) * ceil_div(ns_upd_rows(G), kBM) *
                                                 ceil_div(ns_upd_cols(G), BT) * ngroups);
  }
  for (int it = 0; it < steps; ++it) args.coef_c[it] = (const_coeffs ? kNsConst : kNsTuned[it])[2];
  args.steps = steps;
  args.ngroups = ngroups;
  args.status = status;
  const int grid = static_cast<int>(std::min<int64_t>(sm_count(), std::max<int64_t>(max_tiles, 8)));
  void* kargs[] = {&args};
  KernelScope scope(kClsOther, stream);
  LACT_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kernel), dim3(grid), dim3(kGemmThreadsFlow), kargs, smem,
                                        stream));
  return LACT_OK;
}


// 4-D map (feature, token, head, batch) of a [b][l][h][d] bf16 activation whose token / batch strides are free
// (views of a fused projection) and whose heads are adjacent; box {64, 128, 1, 1}, 128-byte swizzle.
int encode_map_heads(CUtensorMap* map, const void* ptr, int64_t b, int64_t l, int64_t h, int64_t d, int64_t ts,
                     int64_t bs, uint32_t box_rows = 128) {
  EncodeFn fn = get_encode_fn();
  if (fn == nullptr) return LACT_ERR_CUDA;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || (ts % 8) != 0 || (bs % 8) != 0 || ts < h * d) return LACT_ERR_SHAPE;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(l), static_cast<cuuint64_t>(h),
                        static_cast<cuuint64_t>(b)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(ts) * 2, static_cast<cuuint64_t>(d) * 2,
                           static_cast<cuuint64_t>(b > 1 ? bs : ts * l) * 2};
  cuuint32_t box[4] = {64, box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? LACT_OK : LACT_ERR_CUDA;
}

template <int HD>
int launch_swa(const SwaArgs& a, int64_t ctas, cudaStream_t stream) {
  auto kernel = swa_fwd_kernel<HD>;
  constexpr uint32_t smem = SwaSmem<HD>::kBytes;
  static_assert(smem <= 232448, "shared memory budget exceeded");
  static std::mutex mu;
  static bool configured[64] = {false};
  int dev = 0;
  LACT_CUDA(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 64 || !configured[dev]) {
      LACT_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      if (dev < 64) configured[dev] = true;
    }
  }
  KernelScope scope(kClsOther, stream);
  kernel<<<static_cast<unsigned>(ctas), 320, smem, stream>>>(a);
  LACT_CUDA(cudaGetLastError());
  return LACT_OK;
}

template <int HD, int MODE>
int launch_swa_bwd(const SwaBwdArgs& a, int64_t ctas, cudaStream_t stream) {
  auto kernel = swa_bwd_kernel<HD, MODE>;
  constexpr uint32_t smem = SwaBwdSmem<HD>::kBytes;
  static_assert(smem <= 232448, "shared memory budget exceeded");
  static std::mutex mu;
  static bool configured[64] = {false};
  int dev = 0;
  LACT_CUDA(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 64 || !configured[dev]) {
      LACT_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      if (dev < 64) configured[dev] = true;
    }
  }
  KernelScope scope(kClsOther, stream);
  kernel<<<static_cast<unsigned>(ctas), 320, smem, stream>>>(a);
  LACT_CUDA(cudaGetLastError());
  return LACT_OK;
}

struct ScanPlan {
  int32_t* status;
  float *W02, *W1, *W02c, *W1c, *n02, *n1, *G02, *G1, *beta;
  bf16 *W02b, *W1b, *hidden, *dy02, *hid;
  NsPlan ns;
  size_t bytes;
};

int plan_scan(const lact_scan_config& c, int32_t n_steps, const int32_t* kind, const int64_t* start,
              const int64_t* end, void* base, ScanPlan* p) {
  int64_t max_apply = 0, max_update = 0;
  for (int i = 0; i < n_steps; ++i) {
    if (start[i] < 0 || end[i] > c.L || end[i] < start[i]) return LACT_ERR_STEPS;
    const int64_t len = end[i] - start[i];
    if (kind[i] == LACT_STEP_APPLY) max_apply = std::max(max_apply, len);
    else if (kind[i] == LACT_STEP_UPDATE) {
      if (len <= 0) return LACT_ERR_STEPS;
      max_update = std::max(max_update, len);
    } else return LACT_ERR_STEPS;
  }
  Carver cv(base);
  const size_t B = c.B, D = c.D, H = c.H;
  p->status = cv.take<int32_t>(64);  // device status word
  p->W02 = cv.take<float>(B * 2 * H * D);
  p->W1 = cv.take<float>(B * D * H);
  p->W02c = cv.take<float>(B * 2 * H * D);
  p->W1c = cv.take<float>(B * D * H);
  p->n02 = cv.take<float>(B * 2 * H);
  p->n1 = cv.take<float>(B * D);
  p->G02 = cv.take<float>(B * 2 * H * D);
  p->G1 = cv.take<float>(B * D * H);
  p->beta = cv.take<float>(B * static_cast<size_t>(std::max(1, n_steps)));
  p->W02b = cv.take<bf16>(B * 2 * H * D);
  p->W1b = cv.take<bf16>(B * D * H);
  p->hidden = cv.take<bf16>(B * static_cast<size_t>(max_apply) * H);
  p->dy02 = cv.take<bf16>(B * static_cast<size_t>(max_update) * 2 * H);
  p->hid = cv.take<bf16>(B * static_cast<size_t>(max_update) * H);
  p->ns.ngroups = 0;
  if (c.use_muon && max_update > 0) plan_ns(cv, c.B, c.D, c.H, c.ns_concat, c.ns_gram_right, &p->ns);
  p->bytes = cv.off + 256;
  return LACT_OK;
}

// add + renormalise of one or two weight arrays (a1.B = 0: one); rows of up to 1024 elements
int launch_add_renorm(const RenormArgs& a0, const RenormArgs& a1, cudaStream_t stream) {
  const int64_t rows = static_cast<int64_t>(a0.B) * a0.R + static_cast<int64_t>(a1.B) * a1.R;
  const int nv = ceil_div(std::max(a0.C, a1.B > 0 ? a1.C : 0), 128);
  if (rows < 1 || nv > 8) return LACT_ERR_SHAPE;
  const dim3 grid(ceil_div(rows, 8)), block(256);
  KernelScope scope(kClsRenorm, stream);
  switch (nv) {
    case 1: LACT_CUDA(launch_pdl(add_renorm_kernel<1>, grid, block, 0, stream, a0, a1)); break;
    case 2: LACT_CUDA(launch_pdl(add_renorm_kernel<2>, grid, block, 0, stream, a0, a1)); break;
    case 3: LACT_CUDA(launch_pdl(add_renorm_kernel<3>, grid, block, 0, stream, a0, a1)); break;
    case 4: LACT_CUDA(launch_pdl(add_renorm_kernel<4>, grid, block, 0, stream, a0, a1)); break;
    default: LACT_CUDA(launch_pdl(add_renorm_kernel<8>, grid, block, 0, stream, a0, a1)); break;
  }
  return LACT_OK;
}

int validate_scan_config(const lact_scan_config& c) {
  if (c.B < 1 || c.L < 1 || c.D < 16 || c.H < 16 || c.out_len < 0) return LACT_ERR_SHAPE;
  if ((c.D % 16) != 0 || (c.H % 16) != 0) return LACT_ERR_SHAPE;
  if (c.B > 65535 / 3 || c.L > (1ll << 30)) return LACT_ERR_SHAPE;
  if (c.act_dtype != LACT_BF16) return LACT_ERR_DTYPE;
  if (c.use_muon) {
    if (c.ns_steps < 0 || c.ns_steps > 64) return LACT_ERR_CONFIG;
    if (!c.ns_const_coeffs && c.ns_steps != 5) return LACT_ERR_CONFIG;
  }
  if (c.renorm < 0 || c.renorm > 2) return LACT_ERR_CONFIG;
  if (c.prenorm && c.overwrite_quirk) return LACT_ERR_CONFIG;
  return LACT_OK;
}

// True if an UPDATE step follows step i (then the fp32 copy of the normalised weights, which only
// the final export reads in post-norm mode, need not be written).
bool has_later_update(const int32_t* kind, int n_steps, int i) {
  for (int j = i + 1; j < n_steps; ++j)
    if (kind[j] == LACT_STEP_UPDATE) return true;
  return false;
}

// Bytes of Newton-Schulz trace one UPDATE step keeps in training (both groups, 256-byte aligned), and the offset of
// the second group's trace; LACT_ERR_CONFIG if this configuration keeps none (Muon off, more than five steps).
int scan_ns_trace_layout(const lact_scan_config& c, size_t* stride, size_t* g0_bytes) {
  if (!c.use_muon || c.ns_steps < 1 || c.ns_steps > 5) return LACT_ERR_CONFIG;
  NsGroup g0, g1;
  if (c.ns_concat) ns_group_init(g0, c.B, 2 * c.H, c.D, c.ns_gram_right);
  else ns_group_init(g0, 2 * c.B, c.H, c.D, c.ns_gram_right);
  ns_group_init(g1, c.B, c.D, c.H, c.ns_gram_right);
  NsTrace t0, t1;
  LACT_TRY(plan_ns_trace(nullptr, g0.nmat, g0.R, g0.C, c.ns_steps, c.ns_gram_right, &t0));
  LACT_TRY(plan_ns_trace(nullptr, g1.nmat, g1.R, g1.C, c.ns_steps, c.ns_gram_right, &t1));
  const size_t a = (t0.bytes + 255) & ~static_cast<size_t>(255), b = (t1.bytes + 255) & ~static_cast<size_t>(255);
  *g0_bytes = a;
  *stride = a + b;
  return LACT_OK;
}

int scan_fwd(const lact_scan_config& c, const lact_scan_io& io, int32_t n_steps, const int32_t* kind,
             const int64_t* start, const int64_t* end, const int64_t* out_start, void* workspace, size_t ws_bytes,
             cudaStream_t stream) {
  LACT_TRY(check_device());
  LACT_TRY(validate_scan_config(c));
  if (!io.w0 || !io.w1 || !io.w2 || !io.q || !io.k || !io.v || !io.lr0 || !io.lr1 || !io.lr2 || !io.o)
    return LACT_ERR_NULL;
  if (c.use_momentum && !io.momentum) return LACT_ERR_NULL;
  if (!workspace) return LACT_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0) return LACT_ERR_WORKSPACE;
  ScanPlan p;
  LACT_TRY(plan_scan(c, n_steps, kind, start, end, workspace, &p));
  if (p.bytes > ws_bytes) return LACT_ERR_WORKSPACE;
  for (int i = 0; i < n_steps; ++i)
    if (kind[i] == LACT_STEP_APPLY && (out_start[i] < 0 || out_start[i] + (end[i] - start[i]) > c.out_len))
      return LACT_ERR_STEPS;

  const int64_t B = c.B, D = c.D, H = c.H;
  LACT_CUDA(cudaMemsetAsync(p.status, 0, 256, stream));
  // Training (post-norm): the per-update state the backward needs is not copied out, it LIVES in the caller's dump:
  // update u reads its master weights from slot u and writes the new ones into slot u + 1 (the last update into the
  // workspace), and the gradient / momentum state of update u is written into slot u while slot u - 1 is read.
  const size_t n02 = static_cast<size_t>(B) * 2 * H * D, n1 = static_cast<size_t>(B) * D * H;
  int n_updates = 0;
  for (int i = 0; i < n_steps; ++i) n_updates += kind[i] == LACT_STEP_UPDATE;
  const bool dump_in_place = io.state_dump != nullptr && !c.prenorm && n_updates > 0;
  auto slot = [&](int u) { return static_cast<float*>(io.state_dump) + static_cast<size_t>(u) * 2 * (n02 + n1); };
  float* W02cur = dump_in_place ? slot(0) : p.W02;   // master weights in force
  float* W1cur = dump_in_place ? slot(0) + n02 : p.W1;
  float* G02cur = p.G02;                              // gradient / momentum state after the latest update
  float* G1cur = p.G1;
  {
    const int64_t rows = B * (2 * H + D);
    KernelScope scope(kClsPrepare, stream);
    prepare_weights_kernel<<<ceil_div(rows, 8), 256, 0, stream>>>(io.w0, io.w1, io.w2, c.w_dtype == LACT_F32,
                                                                  static_cast<int>(B), static_cast<int>(H),
                                                                  static_cast<int>(D), W02cur, W1cur, p.W02c, p.W1c,
                                                                  p.n02, p.n1, p.W02b, p.W1b);
    LACT_CUDA(cudaGetLastError());
  }
  // gradient / momentum state
  if (io.m0_in && io.m1_in && io.m2_in) {
    LACT_CUDA(cudaMemcpy2DAsync(p.G02, 2 * H * D * 4, io.m0_in, H * D * 4, H * D * 4, B, cudaMemcpyDeviceToDevice,
                                stream));
    LACT_CUDA(cudaMemcpy2DAsync(p.G02 + H * D, 2 * H * D * 4, io.m2_in, H * D * 4, H * D * 4, B,
                                cudaMemcpyDeviceToDevice, stream));
    LACT_CUDA(cudaMemcpyAsync(p.G1, io.m1_in, B * D * H * 4, cudaMemcpyDeviceToDevice, stream));
  } else {
    LACT_CUDA(cudaMemsetAsync(p.G02, 0, B * 2 * H * D * 4, stream));
    LACT_CUDA(cudaMemsetAsync(p.G1, 0, B * D * H * 4, stream));
  }

  // per-update momentum factors, all steps at once
  if (c.use_momentum) {
    MeanArgs ma;
    std::memset(&ma, 0, sizeof(ma));
    int u = 0;
    auto flush = [&](int first_u) -> int {
      if (ma.n == 0) return LACT_OK;
      KernelScope scope(kClsMomentumMean, stream);
      momentum_mean_kernel<<<dim3(static_cast<unsigned>(B), ma.n), 256, 0, stream>>>(
          io.momentum, c.mom_dtype == LACT_F32, c.L, ma, p.beta + static_cast<int64_t>(first_u) * B,
          static_cast<int>(B));
      LACT_CUDA(cudaGetLastError());
      return LACT_OK;
    };
    ma.n = 0;
    int first_u = 0;
    for (int i = 0; i < n_steps; ++i) {
      if (kind[i] != LACT_STEP_UPDATE) continue;
      ma.s[ma.n] = static_cast<int32_t>(start[i]);
      ma.e[ma.n] = static_cast<int32_t>(end[i]);
      ++ma.n; ++u;
      if (ma.n == kMeanBatch) { LACT_TRY(flush(first_u)); first_u = u; ma.n = 0; }
    }
    LACT_TRY(flush(first_u));
  }

  // training with Muon: per-update Newton-Schulz traces in the caller's buffer (see lact_scan_ns_trace_bytes)
  size_t ns_trace_stride = 0, ns_trace_g0 = 0;
  const bool ns_keep = io.ns_trace != nullptr && c.use_muon && scan_ns_trace_layout(c, &ns_trace_stride, &ns_trace_g0) == LACT_OK;
  if (io.ns_trace != nullptr && !ns_keep) return LACT_ERR_CONFIG;
  if (ns_keep && (reinterpret_cast<uintptr_t>(io.ns_trace) & 255) != 0) return LACT_ERR_WORKSPACE;

  int update_idx = 0;
  for (int i = 0; i < n_steps; ++i) {
    if (kind[i] == LACT_STEP_APPLY) {
      ApplyArgs a{p.W02b, p.W1b, io.q, c.q_bs, c.q_ts, start[i], end[i], io.o, c.o_bs, c.o_ts, out_start[i],
                  p.hidden, B, D, H};
      LACT_TRY(run_apply(a, p.status, stream));
      continue;
    }
    const float* beta = c.use_momentum ? p.beta + static_cast<int64_t>(update_idx) * B : nullptr;
    float* dump = nullptr;
    if (io.state_dump != nullptr && !dump_in_place) {
      // training (pre-norm): the weights this update computed with and (below) its gradient after momentum are copied
      dump = slot(update_idx);
      LACT_CUDA(cudaMemcpyAsync(dump, c.prenorm ? p.W02c : p.W02, n02 * 4, cudaMemcpyDeviceToDevice, stream));
      LACT_CUDA(cudaMemcpyAsync(dump + n02, c.prenorm ? p.W1c : p.W1, n1 * 4, cudaMemcpyDeviceToDevice, stream));
    }
    const float* G02prev = nullptr;
    const float* G1prev = nullptr;
    if (dump_in_place) {
      G02prev = G02cur;
      G1prev = G1cur;
      G02cur = slot(update_idx) + n02 + n1;
      G1cur = slot(update_idx) + 2 * n02 + n1;
    }
    ++update_idx;
    GradArgs g{p.W02b, p.W1b, io.k, io.v, c.k_bs, c.k_ts, c.v_bs, c.v_ts, start[i], end[i], io.lr0, io.lr1, io.lr2,
               c.lr_dtype == LACT_F32, c.L, c.w_scale, p.dy02, p.hid, G02cur, G1cur, 1, beta, B, D, H};
    g.g02_prev = G02prev;
    g.g1_prev = G1prev;
    // The Frobenius norms Newton-Schulz needs are gathered per output tile by the contraction when a
    // tile never straddles two matrices (concatenated [2H, D], or H a multiple of the 128-row tile).
    int fused_parts[2] = {0, 0};
    if (c.use_muon && (c.ns_concat || H % kBM == 0)) {
      const int bt = contract_bt(D, H);
      const int tn0 = ceil_div(D, bt), tn1 = ceil_div(H, bt);
      fused_parts[0] = (c.ns_concat ? ceil_div(2 * H, kBM) : static_cast<int>(H / kBM)) * tn0 * kEpiWarps;
      fused_parts[1] = ceil_div(D, kBM) * tn1 * kEpiWarps;
      if (fused_parts[0] <= kNsMaxParts && fused_parts[1] <= kNsMaxParts) {
        g.partial02 = p.ns.grp[0].partial;
        g.partial1 = p.ns.grp[1].partial;
        if (c.ns_steps > 0 && !ns_keep) {  // the iteration starts from bf16(G) itself, normalisation folded in
          g.gb02 = p.ns.grp[0].xa;
          g.gb1 = p.ns.grp[1].xa;
        }
      } else {
        fused_parts[0] = fused_parts[1] = 0;
      }
    }
    LACT_TRY(run_grad(g, p.status, stream));
    if (dump != nullptr) {
      LACT_CUDA(cudaMemcpyAsync(dump + n02 + n1, p.G02, n02 * 4, cudaMemcpyDeviceToDevice, stream));
      LACT_CUDA(cudaMemcpyAsync(dump + 2 * n02 + n1, p.G1, n1 * 4, cudaMemcpyDeviceToDevice, stream));
    }

    // add + renormalise arguments (the update is the Newton-Schulz result when Muon is on)
    const bool want_compute = c.prenorm || !has_later_update(kind, n_steps, i);
    RenormArgs rn[2];
    for (int w = 0; w < 2; ++w) {
      RenormArgs& r = rn[w];
      std::memset(&r, 0, sizeof(r));
      const int R = static_cast<int>(w == 0 ? 2 * H : D), C = static_cast<int>(w == 0 ? D : H);
      if (C > kRenormMaxCols) return LACT_ERR_SHAPE;
      r.master = w == 0 ? p.W02 : p.W1;
      if (dump_in_place) {  // read slot u, write slot u + 1 (the last update writes the workspace copy)
        r.master_in = w == 0 ? W02cur : W1cur;
        if (update_idx < n_updates) r.master = w == 0 ? slot(update_idx) : slot(update_idx) + n02;
      }
      r.compute = want_compute ? (w == 0 ? p.W02c : p.W1c) : nullptr;
      r.shadow = w == 0 ? p.W02b : p.W1b;
      r.n0 = w == 0 ? p.n02 : p.n1;
      r.g = w == 0 ? G02cur : G1cur;
      r.x = nullptr;
      r.x_bs = static_cast<int64_t>(R) * C;
      r.B = static_cast<int>(B); r.R = R; r.C = C;
      r.mode = c.renorm; r.prenorm = c.prenorm; r.prenorm_bf16 = c.prenorm_bf16; r.quirk = c.overwrite_quirk;
    }
    if (c.use_muon && ns_keep) {
      // training: every iterate, shifted Gram matrix and polynomial of this update stays in the caller's trace
      // buffers (the layout lact_ns_trace_bwd reads); the first iterate is the explicitly normalised gradient
      NsPlan& ns = p.ns;
      const bf16* xres[2] = {nullptr, nullptr};
      const void* srcs[2] = {G02cur, G1cur};
      NsGroup tg[2];
      NsKeep keep[2];
      uint8_t* tb = static_cast<uint8_t*>(io.ns_trace) + static_cast<size_t>(update_idx - 1) * ns_trace_stride;
      for (int gi = 0; gi < 2; ++gi) {
        NsTrace t;
        LACT_TRY(plan_ns_trace(tb + (gi == 0 ? 0 : ns_trace_g0), ns.grp[gi].nmat, ns.grp[gi].R, ns.grp[gi].C, c.ns_steps,
                               c.ns_gram_right, &t));
        tg[gi] = ns.grp[gi];
        tg[gi].xa = t.X;
        keep[gi] = NsKeep{t.X, t.A, t.P};
      }
      LACT_TRY(launch_ns_prepare(tg, 2, srcs, 1, 1, stream, fused_parts[0] > 0 ? fused_parts : nullptr));
      LACT_TRY(try_ns_fused(tg, 2, c.ns_steps, c.ns_const_coeffs, p.status, stream, xres, 0, keep));
      rn[0].x = xres[0];
      rn[1].x = xres[1];
    } else if (c.use_muon) {
      NsPlan& ns = p.ns;
      const bf16* xres[2] = {nullptr, nullptr};
      const void* srcs[2] = {G02cur, G1cur};
      const int unscaled = g.gb02 != nullptr ? 1 : 0;
      LACT_TRY(launch_ns_prepare(ns.grp, ns.ngroups, srcs, 1, !unscaled, stream,
                                 fused_parts[0] > 0 ? fused_parts : nullptr));
      int rc = try_ns_fused(ns.grp, ns.ngroups, c.ns_steps, c.ns_const_coeffs, p.status, stream, xres, unscaled);
      if (rc == LACT_ERR_CONFIG)
        rc = run_ns_iterations(ns.grp, ns.ngroups, c.ns_steps, c.ns_const_coeffs, xres, p.status, stream, unscaled);
      LACT_TRY(rc);
      rn[0].x = xres[0];
      rn[1].x = xres[1];
    }
    LACT_TRY(launch_add_renorm(rn[0], rn[1], stream));
    if (dump_in_place) {
      W02cur = rn[0].master;
      W1cur = rn[1].master;
    }
  }
  // final state out
  if (io.w0_out) LACT_CUDA(cudaMemcpy2DAsync(io.w0_out, H * D * 4, p.W02c, 2 * H * D * 4, H * D * 4, B,
                                             cudaMemcpyDeviceToDevice, stream));
  if (io.w2_out) LACT_CUDA(cudaMemcpy2DAsync(io.w2_out, H * D * 4, p.W02c + H * D, 2 * H * D * 4, H * D * 4, B,
                                             cudaMemcpyDeviceToDevice, stream));
  if (io.w1_out) LACT_CUDA(cudaMemcpyAsync(io.w1_out, p.W1c, B * D * H * 4, cudaMemcpyDeviceToDevice, stream));
  if (io.m0_out) LACT_CUDA(cudaMemcpy2DAsync(io.m0_out, H * D * 4, G02cur, 2 * H * D * 4, H * D * 4, B,
                                             cudaMemcpyDeviceToDevice, stream));
  if (io.m2_out) LACT_CUDA(cudaMemcpy2DAsync(io.m2_out, H * D * 4, G02cur + H * D, 2 * H * D * 4, H * D * 4, B,
                                             cudaMemcpyDeviceToDevice, stream));
  if (io.m1_out) LACT_CUDA(cudaMemcpyAsync(io.m1_out, G1cur, B * D * H * 4, cudaMemcpyDeviceToDevice, stream));
  return LACT_OK;
}

}  // namespace
}  // namespace lact

// ==========================================================================================
// extern "C" entry points
// ==========================================================================================
using namespace lact;

extern "C" {

int lact_version(void) { return 1000; }

const char* lact_error_string(int code) {
  switch (code) {
    case LACT_OK: return "ok";
    case LACT_ERR_NULL: return "a required pointer is NULL";
    case LACT_ERR_SHAPE: return "unsupported or inconsistent sizes, strides or alignment";
    case LACT_ERR_DTYPE: return "unsupported dtype combination";
    case LACT_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case LACT_ERR_CONFIG: return "inconsistent configuration flags";
    case LACT_ERR_STEPS: return "malformed step list";
    case LACT_ERR_CUDA: return "a CUDA runtime or driver call failed";
    case LACT_ERR_DEVICE: return "device is not compute capability 10.x (B200)";
    case LACT_ERR_STATIC_LIMIT:
      return "problem needs more scratch than the library's built-in static buffer holds (16 MiB): "
             "use the workspace variant or a smaller B * N * H";
    case kStatusWaitTimeout: return "device: a bounded barrier wait timed out";
    default: return "unknown code";
  }
}

int64_t lact_launch_count(void) { return g_prof.launches.load(); }

int lact_profile_enable(int enable) {
  g_prof.enabled.store(enable != 0);
  return LACT_OK;
}

int lact_nvtx_enable(int enable) {
  g_nvtx.store(enable != 0);
  return LACT_OK;
}

int lact_profile_num_classes(void) { return kNumClasses; }

const char* lact_profile_class_name(int cls) { return (cls >= 0 && cls < kNumClasses) ? kClassNames[cls] : "?"; }

int lact_profile_read(double* ms, int64_t* launches) {
  if (!ms || !launches) return LACT_ERR_NULL;
  std::vector<Profiler::Rec> recs;
  {
    std::lock_guard<std::mutex> lock(g_prof.mu);
    recs.swap(g_prof.recs);
  }
  for (int i = 0; i < kNumClasses; ++i) { ms[i] = 0.0; launches[i] = 0; }
  int rc = LACT_OK;
  for (auto& r : recs) {
    float t = 0.f;
    if (cudaEventSynchronize(r.b) != cudaSuccess || cudaEventElapsedTime(&t, r.a, r.b) != cudaSuccess) rc = LACT_ERR_CUDA;
    ms[r.cls] += t;
    launches[r.cls] += 1;
  }
  std::lock_guard<std::mutex> lock(g_prof.mu);
  for (auto& r : recs) { g_prof.pool.push_back(r.a); g_prof.pool.push_back(r.b); }
  return rc;
}

// Copies one status word to the host; the only place where the library waits for a stream.
static int read_status_word(const void* device_word, cudaStream_t stream) {
  int32_t st = 0;
  g_stream_syncs.fetch_add(1, std::memory_order_relaxed);
  if (cudaMemcpyAsync(&st, device_word, 4, cudaMemcpyDeviceToHost, stream) != cudaSuccess) return LACT_ERR_CUDA;
  if (cudaStreamSynchronize(stream) != cudaSuccess) return LACT_ERR_CUDA;
  return st;
}

int lact_read_status(const void* workspace, void* stream) {
  if (!workspace) return LACT_ERR_NULL;
  return read_status_word(workspace, static_cast<cudaStream_t>(stream));
}

int64_t lact_stream_sync_count(void) { return g_stream_syncs.load(); }

int lact_set_wait_limit_ns(uint64_t limit_ns) {
  if (limit_ns == 0) limit_ns = kDefaultWaitLimitNs;
  LACT_CUDA(cudaMemcpyToSymbol(g_wait_limit_ns, &limit_ns, sizeof(limit_ns)));
  return LACT_OK;
}

// One CTA whose single waiting thread sits on an mbarrier that nobody arrives on: the bounded
// wait runs out and the kernel records kStatusWaitTimeout, exactly as the GEMM kernels do.
__global__ void wait_timeout_probe_kernel(int32_t* status) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
    if (!mbar_wait(&bar, 0)) atomicCAS(status, kStatusOk, kStatusWaitTimeout);
  }
}

int lact_debug_wait_timeout(int32_t* status_word, void* stream) {
  if (!status_word) return LACT_ERR_NULL;
  LACT_TRY(check_device());
  wait_timeout_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status_word);
  LACT_CUDA(cudaGetLastError());
  return LACT_OK;
}

int lact_scan_workspace_bytes(const lact_scan_config* cfg, int32_t n_steps, const int32_t* kind,
                              const int64_t* start, const int64_t* end, size_t* bytes_out) {
  if (!cfg || !bytes_out || (n_steps > 0 && (!kind || !start || !end))) return LACT_ERR_NULL;
  LACT_TRY(validate_scan_config(*cfg));
  ScanPlan p;
  LACT_TRY(plan_scan(*cfg, n_steps, kind, start, end, nullptr, &p));
  *bytes_out = p.bytes;
  return LACT_OK;
}

int lact_scan_ns_trace_bytes(const lact_scan_config* cfg, size_t* bytes_per_update, size_t* second_group_offset) {
  if (!cfg || !bytes_per_update || !second_group_offset) return LACT_ERR_NULL;
  LACT_TRY(validate_scan_config(*cfg));
  return scan_ns_trace_layout(*cfg, bytes_per_update, second_group_offset);
}

int lact_scan_fwd(const lact_scan_config* cfg, const lact_scan_io* io, int32_t n_steps, const int32_t* kind,
                  const int64_t* start, const int64_t* end, const int64_t* out_start, void* workspace,
                  size_t workspace_bytes, void* stream) {
  if (!cfg || !io || (n_steps > 0 && (!kind || !start || !end || !out_start))) return LACT_ERR_NULL;
  return scan_fwd(*cfg, *io, n_steps, kind, start, end, out_start, workspace, workspace_bytes,
                  static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------- sub-ops
static int check_dims(int64_t B, int64_t N, int64_t D, int64_t H) {
  if (B < 1 || N < 1 || D < 16 || H < 16 || (D % 16) || (H % 16) || B > 65535 || N > (1ll << 30))
    return LACT_ERR_SHAPE;
  return LACT_OK;
}

int lact_swiglu_ffn_workspace_bytes(int64_t B, int64_t N, int64_t D, int64_t H, size_t* bytes_out) {
  if (!bytes_out) return LACT_ERR_NULL;
  LACT_TRY(check_dims(B, N, D, H));
  *bytes_out = 512 + static_cast<size_t>(B) * N * H * 2;
  return LACT_OK;
}

int lact_swiglu_ffn_fwd(const void* w0w2, const void* w1, const void* x, void* out, int64_t B, int64_t N, int64_t D,
                        int64_t H, void* workspace, size_t workspace_bytes, void* stream) {
  if (!w0w2 || !w1 || !x || !out) return LACT_ERR_NULL;
  LACT_TRY(check_device());
  size_t need = 0;
  LACT_TRY(lact_swiglu_ffn_workspace_bytes(B, N, D, H, &need));
  if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255)) return LACT_ERR_WORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  LACT_CUDA(cudaMemsetAsync(workspace, 0, 256, s));
  ApplyArgs a{static_cast<const bf16*>(w0w2), static_cast<const bf16*>(w1), x, N * D, D, 0, N, out, N * D, D, 0,
              reinterpret_cast<bf16*>(static_cast<uint8_t*>(workspace) + 256), B, D, H};
  return run_apply(a, static_cast<int32_t*>(workspace), s);
}

// ---------------------------------------------------------------- allocation-free variant
// Scratch for lact_swiglu_ffn_fwd_static.  It lives in the library image: every GPU that loads
// the library holds these bytes until the process exits.
#define LACT_STATIC_SCRATCH_BYTES (16u << 20)
static __device__ __align__(256) unsigned char g_static_scratch[LACT_STATIC_SCRATCH_BYTES];

// Device address of g_static_scratch on the current device, resolved once per device.  In host
// code the array's name is only a handle for the runtime, never a pointer a kernel may use, so
// the address is asked for with cudaGetSymbolAddress and that result is what kernels receive.
static int static_scratch_address(void** out) {
  static std::mutex mu;
  static void* addr[64] = {nullptr};
  int dev = 0;
  LACT_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return LACT_ERR_DEVICE;
  std::lock_guard<std::mutex> lock(mu);
  if (addr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_scratch) != cudaSuccess || p == nullptr)
      return LACT_ERR_CUDA;
    addr[dev] = p;
  }
  *out = addr[dev];
  return LACT_OK;
}

size_t lact_static_scratch_bytes(void) { return LACT_STATIC_SCRATCH_BYTES; }

int lact_swiglu_ffn_fwd_static(const void* w0w2, const void* w1, const void* x, void* out, int64_t B, int64_t N,
                               int64_t D, int64_t H, void* stream) {
  if (!w0w2 || !w1 || !x || !out) return LACT_ERR_NULL;
  LACT_TRY(check_device());
  LACT_TRY(check_dims(B, N, D, H));
  // status word (256 bytes reserved) + hidden activations [B, N, H] bf16
  const unsigned long long hidden_bytes = static_cast<unsigned long long>(B) * static_cast<unsigned long long>(N) *
                                          static_cast<unsigned long long>(H) * 2ull;
  if (hidden_bytes > LACT_STATIC_SCRATCH_BYTES - 256ull) return LACT_ERR_STATIC_LIMIT;
  void* scratch = nullptr;
  LACT_TRY(static_scratch_address(&scratch));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // the array keeps whatever the previous call left: the status word must start at zero; the
  // hidden activations behind it are fully overwritten before they are read
  LACT_CUDA(cudaMemsetAsync(scratch, 0, 256, s));
  ApplyArgs a{static_cast<const bf16*>(w0w2), static_cast<const bf16*>(w1), x, N * D, D, 0, N, out, N * D, D, 0,
              reinterpret_cast<bf16*>(static_cast<uint8_t*>(scratch) + 256), B, D, H};
  return run_apply(a, static_cast<int32_t*>(scratch), s);
}

int lact_static_status(void* stream) {
  LACT_TRY(check_device());
  void* scratch = nullptr;
  LACT_TRY(static_scratch_address(&scratch));
  return read_status_word(scratch, static_cast<cudaStream_t>(stream));
}

int lact_fw_grad_workspace_bytes(int64_t B, int64_t N, int64_t D, int64_t H, size_t* bytes_out) {
  if (!bytes_out) return LACT_ERR_NULL;
  LACT_TRY(check_dims(B, N, D, H));
  *bytes_out = 1024 + static_cast<size_t>(B) * N * 3 * H * 2;
  return LACT_OK;
}

int lact_fw_grad(const void* w0w2, const void* w1, const void* k, const void* v, const void* lr0, const void* lr1,
                 const void* lr2, int32_t lr_dtype, void* dw0w2, void* dw1, int64_t B, int64_t N, int64_t D, int64_t H,
                 void* workspace, size_t workspace_bytes, void* stream) {
  if (!w0w2 || !w1 || !k || !v || !lr0 || !lr1 || !lr2 || !dw0w2 || !dw1) return LACT_ERR_NULL;
  LACT_TRY(check_device());
  size_t need = 0;
  LACT_TRY(lact_fw_grad_workspace_bytes(B, N, D, H, &need));
  if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255)) return LACT_ERR_WORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  LACT_CUDA(cudaMemsetAsync(workspace, 0, 256, s));
  Carver cv(workspace);
  int32_t* status = cv.take<int32_t>(64);
  bf16* dy02 = cv.take<bf16>(static_cast<size_t>(B) * N * 2 * H);
  bf16* hid = cv.take<bf16>(static_cast<size_t>(B) * N * H);
  GradArgs g{static_cast<const bf16*>(w0w2), static_cast<const bf16*>(w1), k, v, N * D, D, N * D, D, 0, N, lr0, lr1,
             lr2, lr_dtype == LACT_F32, N, 1.0f, dy02, hid, dw0w2, dw1, 0, nullptr, B, D, H};
  return run_grad(g, status, s);
}

int lact_newton_schulz_workspace_bytes(int64_t B, int64_t R, int64_t C, size_t* bytes_out) {
  if (!bytes_out) return LACT_ERR_NULL;
  if (B < 1 || B > 65535 || R < 8 || C < 8 || (R % 8) || (C % 8)) return LACT_ERR_SHAPE;
  *bytes_out = 2048 + ns_group_bytes(B, std::min(R, C), std::max(R, C));
  return LACT_OK;
}

int lact_newton_schulz(const void* g, int32_t g_dtype, void* x, int64_t B, int64_t R, int64_t C, int32_t steps,
                       int32_t const_coeffs, void* workspace, size_t workspace_bytes, void* stream) {
  if (!g || !x) return LACT_ERR_NULL;
  LACT_TRY(check_device());
  size_t need = 0;
  LACT_TRY(lact_newton_schulz_workspace_bytes(B, R, C, &need));
  if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255)) return LACT_ERR_WORKSPACE;
  if (steps < 0 || steps > 64 || (!const_coeffs && steps != 5)) return LACT_ERR_CONFIG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  LACT_CUDA(cudaMemsetAsync(workspace, 0, 256, s));
  Carver cv(workspace);
  int32_t* status = cv.take<int32_t>(64);
  NsGroup grp;
  ns_group_init(grp, B, R, C, 0);
  carve_ns_group(cv, grp);
  const bf16* res = nullptr;
  const void* srcs[2] = {g, g};
  LACT_TRY(launch_ns_prepare(&grp, 1, srcs, g_dtype == LACT_F32, 1, s));
  int rc = try_ns_fused(&grp, 1, steps, const_coeffs, status, s, &res);
  if (rc == LACT_ERR_CONFIG) rc = run_ns_iterations(&grp, 1, steps, const_coeffs, &res, status, s);
  LACT_TRY(rc);
  LACT_CUDA(cudaMemcpyAsync(x, res, static_cast<size_t>(B) * R * C * 2, cudaMemcpyDeviceToDevice, s));
  return LACT_OK;
}

// ---------------------------------------------------------------- Newton-Schulz with saved iterates, and its backward
int lact_ns_trace_bytes(int64_t B, int64_t R, int64_t C, int32_t steps, size_t* bytes_out) {
  if (!bytes_out) return LACT_ERR_NULL;
  NsTrace t;
  LACT_TRY(plan_ns_trace(nullptr, B, R, C, steps, 0, &t));
  *bytes_out = t.bytes;
  return LACT_OK;
}

int lact_ns_trace_result_offset(int64_t B, int64_t R, int64_t C, int32_t steps, size_t* offset_out) {
  if (!offset_out) return LACT_ERR_NULL;
  NsTrace t;
  // carve from a fake, never dereferenced base (a null base yields null pointers) and subtract it again
  uint8_t* const fake = reinterpret_cast<uint8_t*>(static_cast<uintptr_t>(1) << 40);
  LACT_TRY(plan_ns_trace(fake, B, R, C, steps, 0, &t));
  *offset_out = static_cast<size_t>(reinterpret_cast<uint8_t*>(t.X) - fake) +
                static_cast<size_t>(B) * R * C * steps * sizeof(bf16);
  return LACT_OK;
}

int lact_ns_trace_fwd(const void* g, int32_t g_dtype, void* x_out, int64_t B, int64_t R, int64_t C, int32_t steps,
                      int32_t const_coeffs, int32_t gram_right, void* trace, size_t trace_bytes, int32_t* status_word,
                      void* stream) {
  if (!g || !x_out || !trace || !status_word) return LACT_ERR_NULL;
  LACT_TRY(check_device());
  if ((reinterpret_cast<uintptr_t>(trace) & 255) != 0) return LACT_ERR_WORKSPACE;
  if (!const_coeffs && steps != 5) return LACT_ERR_CONFIG;
  NsTrace t;
  LACT_TRY(plan_ns_trace(trace, B, R, C, steps, gram_right, &t));
  if (t.bytes > trace_bytes) return LACT_ERR_WORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t rc = static_cast<size_t>(B) * R * C, mm = static_cast<size_t>(B) * t.grp.m * t.grp.m;
  t.grp.xa = t.X;
  const void* srcs[2] = {g, g};
  LACT_TRY(launch_ns_prepare(&t.grp, 1, srcs, g_dtype == LACT_F32, 1, s));  // X[0] = normalised bf16(g)
  // all iterations in one dataflow launch that keeps every iterate (up to five: both coefficient schedules of the
  // reference's drivers); longer constant-coefficient runs go iteration by iteration
  int rc_f = LACT_ERR_CONFIG;
  if (steps <= 5) {
    const NsKeep keep{t.X, t.A, t.P};
    const bf16* res = nullptr;
    rc_f = try_ns_fused(&t.grp, 1, steps, const_coeffs, status_word, s, &res, 0, &keep);
  }
  if (rc_f == LACT_ERR_CONFIG) {
    for (int it = 0; it < steps; ++it) {
      NsGroup gi = t.grp;
      gi.xa = t.X + rc * it;
      gi.xb = t.X + rc * (it + 1);
      gi.gram = t.A + mm * it;
      gi.poly = t.P + mm * it;
      const bf16* res = nullptr;
      LACT_TRY(run_ns_iterations(&gi, 1, 1, const_coeffs, &res, status_word, s, 0, const_coeffs ? 0 : it));
    }
  } else {
    LACT_TRY(rc_f);
  }
  LACT_CUDA(cudaMemcpyAsync(x_out, t.X + rc * steps, rc * 2, cudaMemcpyDeviceToDevice, s));
  return LACT_OK;
}

static int bmm2_scaled(const void* a0, int32_t a0_mn, const void* b0, int32_t b0_mn, const void* a1, int32_t a1_mn,
                       const void* b1, int32_t b1_mn, void* c, int32_t c_dtype, int64_t batch, int64_t M, int64_t N,
                       int64_t K, int32_t* status_word, void* stream, float alpha);

// dx0 (fp32) = gradient w.r.t. the normalised first iterate X[0], given du = bf16 gradient w.r.t. the
// result X[steps]; roundings are treated as identities and every operand is bf16 (the reference
// differentiates its bf16 iteration the same way).  With Q = dP + dP^T (dP = dX' X^T) and
// CB = c A + (b/2) I the three products per iteration are, for a wide iterate ([m][n], A = X X^T):
//   Q = dX' X^T + X dX'^T,   S = CB Q + Q CB,   dX = P dX' + S X,
// and for a tall one ([n][m], A = X^T X, X' = X P^T):  Q = dX'^T X + X^T dX',  dX = dX' P + X S.
int lact_ns_trace_bwd(const void* du, void* dx0, int64_t B, int64_t R, int64_t C, int32_t steps, int32_t const_coeffs,
                      int32_t gram_right, void* trace, size_t trace_bytes, int32_t* status_word, void* stream) {
  if (!du || !dx0 || !trace || !status_word) return LACT_ERR_NULL;
  LACT_TRY(check_device());
  NsTrace t;
  LACT_TRY(plan_ns_trace(trace, B, R, C, steps, gram_right, &t));
  if (t.bytes > trace_bytes) return LACT_ERR_WORKSPACE;
  const int64_t m = t.grp.m, n = t.grp.n;
  const size_t rc = static_cast<size_t>(B) * R * C, mm = static_cast<size_t>(B) * m * m;
  const int tall = t.grp.transposed;
  const bf16* dX = static_cast<const bf16*>(du);
  for (int it = steps - 1; it >= 0; --it) {
    const float* co = const_coeffs ? kNsConst : kNsTuned[it];
    const bf16* X = t.X + rc * it;
    const bf16* P = t.P + mm * it;
    // Q [m][m]: contraction over the long side n
    LACT_TRY(lact_bmm2_bf16(dX, tall, X, tall, X, tall, dX, tall, t.Q, LACT_BF16, 0, B, m, m, n, status_word, stream));
    // S = CB Q + Q CB with CB = c A + (b/2) I = c (A + (b/2c) I): the kept shifted Gram matrix, scaled in the epilogue
    const bf16* As = t.A + mm * it;
    LACT_TRY(bmm2_scaled(As, 0, t.Q, 0, t.Q, 0, As, 0, t.S, LACT_BF16, B, m, m, m, status_word, stream, co[2]));
    void* out = it == 0 ? dx0 : static_cast<void*>((it & 1) ? t.dXa : t.dXb);
    const int out_dt = it == 0 ? LACT_F32 : LACT_BF16;
    if (!tall) LACT_TRY(lact_bmm2_bf16(P, 0, dX, 1, t.S, 0, X, 1, out, out_dt, 0, B, m, n, m, status_word, stream));
    else LACT_TRY(lact_bmm2_bf16(dX, 0, P, 1, X, 0, t.S, 0, out, out_dt, 0, B, n, m, m, status_word, stream));
    dX = static_cast<const bf16*>(out);
  }
  return LACT_OK;
}

static int qkv_prologue_impl(const void* xq, const void* xk, const void* xv, int64_t ld_q, int64_t ld_k, int64_t ld_v,
                             int64_t bs_q, int64_t bs_k, int64_t bs_v, void* q, void* k, void* v, int64_t b, int64_t s,
                             int64_t n_heads, int64_t d, int32_t qkv_silu, int32_t v_silu, const void* cos,
                             const void* sin, int64_t rope_head_dim, int64_t n_positions, int64_t seqlen_offset,
                             const int32_t* seq_start, void* stream) {
  if (!xq || !xk || !xv || !q || !k || !v) return LACT_ERR_NULL;
  if (seq_start != nullptr && (b != 1 || rope_head_dim == 0)) return LACT_ERR_CONFIG;
  LACT_TRY(check_device());
  if (b < 1 || s < 1 || n_heads < 1 || d < 8 || d > 1024 || (d % 8) != 0) return LACT_ERR_SHAPE;
  if (b * s * n_heads > (1ll << 40) || b > 65535 || s > (1ll << 30)) return LACT_ERR_SHAPE;
  const void* xs[3] = {xq, xk, xv};
  void* outs[3] = {q, k, v};
  const int64_t lds[3] = {ld_q, ld_k, ld_v}, bss[3] = {bs_q, bs_k, bs_v};
  PrologueArgs a;
  std::memset(&a, 0, sizeof(a));
  for (int t = 0; t < 3; ++t) {
    // rows move as 16-byte vectors
    if ((reinterpret_cast<uintptr_t>(xs[t]) & 15) != 0 || (reinterpret_cast<uintptr_t>(outs[t]) & 15) != 0 ||
        lds[t] < n_heads * d || (lds[t] % 8) != 0 || (bss[t] % 8) != 0)
      return LACT_ERR_SHAPE;
    a.x[t] = static_cast<const bf16*>(xs[t]);
    a.out[t] = static_cast<bf16*>(outs[t]);
    a.ld[t] = lds[t];
    a.bs[t] = bss[t];
  }
  a.b = static_cast<int32_t>(b); a.s = static_cast<int32_t>(s);
  a.n_h = static_cast<int32_t>(n_heads); a.d = static_cast<int32_t>(d);
  a.silu[0] = a.silu[1] = qkv_silu ? 1 : 0;
  a.silu[2] = (qkv_silu && v_silu) ? 1 : 0;
  a.l2norm[0] = a.l2norm[1] = 1;
  a.l2norm[2] = 0;
  if (rope_head_dim != 0) {
    if (!cos || !sin) return LACT_ERR_NULL;
    // attention heads of a power-of-two size that tile every fast-weight head; positions inside the tables
    if (rope_head_dim < 32 || rope_head_dim > 1024 || (rope_head_dim & (rope_head_dim - 1)) != 0 ||
        (d % rope_head_dim) != 0 || seqlen_offset < 0 || seqlen_offset + s > n_positions)
      return LACT_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(cos) & 15) != 0 || (reinterpret_cast<uintptr_t>(sin) & 15) != 0) return LACT_ERR_SHAPE;
    a.cos = static_cast<const bf16*>(cos);
    a.sin = static_cast<const bf16*>(sin);
    a.rope_hd = static_cast<int32_t>(rope_head_dim);
    a.pos0 = static_cast<int32_t>(seqlen_offset);
    a.seq_start = seq_start;
  }
  const int64_t rows = b * s * n_heads;
  KernelScope scope(kClsOther, static_cast<cudaStream_t>(stream));
  const unsigned grid = static_cast<unsigned>(ceil_div(rows, 8));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (a.rope_hd != 0) {
    switch (ceil_div(d, 256)) {
      case 1: qkv_prologue_kernel<1, true><<<grid, 256, 0, st>>>(a); break;
      case 2: qkv_prologue_kernel<2, true><<<grid, 256, 0, st>>>(a); break;
      case 3: qkv_prologue_kernel<3, true><<<grid, 256, 0, st>>>(a); break;
      default: qkv_prologue_kernel<4, true><<<grid, 256, 0, st>>>(a); break;
    }
  } else {
    switch (ceil_div(d, 256)) {
      case 1: qkv_prologue_kernel<1, false><<<grid, 256, 0, st>>>(a); break;
      case 2: qkv_prologue_kernel<2, false><<<grid, 256, 0, st>>>(a); break;
      case 3: qkv_prologue_kernel<3, false><<<grid, 256, 0, st>>>(a); break;
      default: qkv_prologue_kernel<4, false><<<grid, 256, 0, st>>>(a); break;
    }
  }
  LACT_CUDA(cudaGetLastError());
  return LACT_OK;
}

int lact_qkv_prologue_bwd(const void* xq, const void* xk, const void* xv, int64_t ld_q, int64_t ld_k, int64_t ld_v,
                          int64_t bs_q, int64_t bs_k, int64_t bs_v, const void* dq, const void* dk, const void* dv,
                          void* dxq, void* dxk, void* dxv, int64_t b, int64_t s, int64_t n_heads, int64_t d,
                          int32_t qkv_silu, int32_t v_silu, const void* cos, const void* sin, int64_t rope_head_dim,
                          int64_t n_positions, int64_t seqlen_offset, const int32_t* seq_start, void* stream) {
  if (!xq || !xk || !xv || !dxq || !dxk || !dxv) return LACT_ERR_NULL;
  if (seq_start != nullptr && (b != 1 || rope_head_dim == 0)) return LACT_ERR_CONFIG;
  LACT_TRY(check_device());
  if (b < 1 || s < 1 || n_heads < 1 || d < 8 || d > 1024 || (d % 8) != 0) return LACT_ERR_SHAPE;
  if (b * s * n_heads > (1ll << 40) || b > 65535 || s > (1ll << 30)) return LACT_ERR_SHAPE;
  const void* xs[3] = {xq, xk, xv};
  const void* dzs[3] = {dq, dk, dv};
  void* outs[3] = {dxq, dxk, dxv};
  const int64_t lds[3] = {ld_q, ld_k, ld_v}, bss[3] = {bs_q, bs_k, bs_v};
  PrologueBwdArgs a;
  std::memset(&a, 0, sizeof(a));
  for (int t = 0; t < 3; ++t) {
    if ((reinterpret_cast<uintptr_t>(xs[t]) & 15) != 0 || (reinterpret_cast<uintptr_t>(outs[t]) & 15) != 0 ||
        (reinterpret_cast<uintptr_t>(dzs[t]) & 15) != 0 || lds[t] < n_heads * d || (lds[t] % 8) != 0 || (bss[t] % 8) != 0)
      return LACT_ERR_SHAPE;
    a.x[t] = static_cast<const bf16*>(xs[t]);
    a.dz[t] = static_cast<const bf16*>(dzs[t]);
    a.dx[t] = static_cast<bf16*>(outs[t]);
    a.ld[t] = lds[t];
    a.bs[t] = bss[t];
  }
  a.b = static_cast<int32_t>(b); a.s = static_cast<int32_t>(s);
  a.n_h = static_cast<int32_t>(n_heads); a.d = static_cast<int32_t>(d);
  a.silu[0] = a.silu[1] = qkv_silu ? 1 : 0;
  a.silu[2] = (qkv_silu && v_silu) ? 1 : 0;
  a.l2norm[0] = a.l2norm[1] = 1;
  a.l2norm[2] = 0;
  if (rope_head_dim != 0) {
    if (!cos || !sin) return LACT_ERR_NULL;
    if (rope_head_dim < 32 || rope_head_dim > 1024 || (rope_head_dim & (rope_head_dim - 1)) != 0 ||
        (d % rope_head_dim) != 0 || seqlen_offset < 0 || seqlen_offset + s > n_positions)
      return LACT_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(cos) & 15) != 0 || (reinterpret_cast<uintptr_t>(sin) & 15) != 0) return LACT_ERR_SHAPE;
    a.cos = static_cast<const bf16*>(cos);
    a.sin = static_cast<const bf16*>(sin);
    a.rope_hd = static_cast<int32_t>(rope_head_dim);
    a.pos0 = static_cast<int32_t>(seqlen_offset);
    a.seq_start = seq_start;
  }
  const int64_t rows = b * s * n_heads;
  KernelScope scope(kClsOther, static_cast<cudaStream_t>(stream));
  const unsigned grid = static_cast<unsigned>(ceil_div(rows, 8));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (a.rope_hd != 0) {
    switch (ceil_div(d, 256)) {
      case 1: qkv_prologue_bwd_kernel<1, true><<<grid, 256, 0, st>>>(a); break;
      case 2: qkv_prologue_bwd_kernel<2, true><<<grid, 256, 0, st>>>(a); break;
      case 3: qkv_prologue_bwd_kernel<3, true><<<grid, 256, 0, st>>>(a); break;
      default: qkv_prologue_bwd_kernel<4, true><<<grid, 256, 0, st>>>(a); break;
    }
  } else {
    switch (ceil_div(d, 256)) {
      case 1: qkv_prologue_bwd_kernel<1, false><<<grid, 256, 0, st>>>(a); break;
      case 2: qkv_prologue_bwd_kernel<2, false><<<grid, 256, 0, st>>>(a); break;
      case 3: qkv_prologue_bwd_kernel<3, false><<<grid, 256, 0, st>>>(a); break;
      default: qkv_prologue_bwd_kernel<4, false><<<grid, 256, 0, st>>>(a); break;
    }
  }
  LACT_CUDA(cudaGetLastError());
  return LACT_OK;
}

int lact_out_epilogue_bwd_blocks(void) { return sm_count() * 4; }

int lact_out_epilogue_bwd(const void* fw_x, const void* weight, const void* gate_proj, int64_t gate_ld, const void* dout,
                          int64_t dout_ld, void* dx, void* dgate, void* dw_partial, int64_t b, int64_t s, int64_t n_heads,
                          int64_t d, float eps, void* stream) {
  if (!fw_x || !weight || !dout || !dx || !dw_partial) return LACT_ERR_NULL;
  if ((gate_proj == nullptr) != (dgate == nullptr)) return LACT_ERR_NULL;
  LACT_TRY(check_device());
  if (b < 1 || s < 1 || n_heads < 1 || d < 8 || d > 1024 || (d % 8) != 0 || b > 65535 || s > (1ll << 30))
    return LACT_ERR_SHAPE;
  auto bad = [&](const void* p, int64_t ld) {
    return p != nullptr && ((reinterpret_cast<uintptr_t>(p) & 15) != 0 || ld < n_heads * d || (ld % 8) != 0);
  };
  if ((reinterpret_cast<uintptr_t>(fw_x) & 15) != 0 || (reinterpret_cast<uintptr_t>(weight) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(dx) & 15) != 0 || (reinterpret_cast<uintptr_t>(dgate) & 15) != 0 ||
      bad(gate_proj, gate_ld) || bad(dout, dout_ld))
    return LACT_ERR_SHAPE;
  EpilogueBwdArgs a;
  std::memset(&a, 0, sizeof(a));
  a.x = static_cast<const bf16*>(fw_x);
  a.weight = static_cast<const float*>(weight);
  a.gate = static_cast<const bf16*>(gate_proj);
  a.dout = static_cast<const bf16*>(dout);
  a.gate_ld = gate_ld; a.dout_ld = dout_ld;
  a.dx = static_cast<bf16*>(dx);
  a.dgate = static_cast<bf16*>(dgate);
  a.dw_partial = static_cast<float*>(dw_partial);
  a.b = static_cast<int32_t>(b); a.s = static_cast<int32_t>(s);
  a.n_h = static_cast<int32_t>(n_heads); a.d = static_cast<int32_t>(d);
  a.eps = eps;
  KernelScope scope(kClsOther, static_cast<cudaStream_t>(stream));
  const unsigned grid = static_cast<unsigned>(lact_out_epilogue_bwd_blocks());
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (ceil_div(d, 256)) {
    case 1: out_epilogue_bwd_kernel<1><<<grid, 256, 0, st>>>(a); break;
    case 2: out_epilogue_bwd_kernel<2><<<grid, 256, 0, st>>>(a); break;
    case 3: out_epilogue_bwd_kernel<3><<<grid, 256, 0, st>>>(a); break;
    default: out_epilogue_bwd_kernel<4><<<grid, 256, 0, st>>>(a); break;
  }
  LACT_CUDA(cudaGetLastError());
  return LACT_OK;
}

int lact_qkv_prologue(const void* xq, const void* xk, const void* xv, int64_t ld_q, int64_t ld_k, int64_t ld_v,
                      int64_t bs_q, int64_t bs_k, int64_t bs_v, void* q, void* k, void* v, int64_t b, int64_t s,
                      int64_t n_heads, int64_t d, int32_t qkv_silu, int32_t v_silu, void* stream) {
  return qkv_prologue_impl(xq, xk, xv, ld_q, ld_k, ld_v, bs_q, bs_k, bs_v, q, k, v, b, s, n_heads, d, qkv_silu, v_silu,
                           nullptr, nullptr, 0, 0, 0, nullptr, stream);
}

int lact_qkv_prologue_rope(const void* xq, const void* xk, const void* xv, int64_t ld_q, int64_t ld_k, int64_t ld_v,
                           int64_t bs_q, int64_t bs_k, int64_t bs_v, void* q, void* k, void* v, int64_t b, int64_t s,
                           int64_t n_heads, int64_t d, int32_t qkv_silu, int32_t v_silu, const void* cos, const void* sin,
                           int64_t rope_head_dim, int64_t n_positions, int64_t seqlen_offset, const int32_t* seq_start,
                           void* stream) {
  if (rope_head_dim == 0) return LACT_ERR_SHAPE;
  return qkv_prologue_impl(xq, xk, xv, ld_q, ld_k, ld_v, bs_q, bs_k, bs_v, q, k, v, b, s, n_heads, d, qkv_silu, v_silu,
                           cos, sin, rope_head_dim, n_positions, seqlen_offset, seq_start, stream);
}

int lact_lr_prologue(const void* lr_proj, int32_t proj_dtype, int64_t proj_ld, float base_lr_inv, const void* mom_logits,
                     int32_t logits_dtype, int64_t logits_ld, void* lr0, void* lr1, void* lr2, void* momentum, int64_t b,
                     int64_t s, int64_t n_heads, void* stream) {
  if (!lr_proj || !lr0 || !lr1 || !lr2 || ((mom_logits == nullptr) != (momentum == nullptr))) return LACT_ERR_NULL;
  LACT_TRY(check_device());
  if (b < 1 || s < 1 || n_heads < 1 || b > 65535 || s > (1ll << 30) || n_heads > 4096) return LACT_ERR_SHAPE;
  if (proj_ld < 3 * n_heads || (mom_logits && logits_ld < n_heads)) return LACT_ERR_SHAPE;
  if ((proj_dtype != LACT_F32 && proj_dtype != LACT_BF16) ||
      (mom_logits && logits_dtype != LACT_F32 && logits_dtype != LACT_BF16))
    return LACT_ERR_DTYPE;
  LrPrologueArgs a;
  std::memset(&a, 0, sizeof(a));
  a.proj = lr_proj; a.logits = mom_logits;
  a.proj_f32 = proj_dtype == LACT_F32; a.logits_f32 = logits_dtype == LACT_F32;
  a.proj_ld = proj_ld; a.logits_ld = logits_ld;
  a.base_lr_inv = base_lr_inv;
  a.lr[0] = static_cast<float*>(lr0); a.lr[1] = static_cast<float*>(lr1); a.lr[2] = static_cast<float*>(lr2);
  a.mom = static_cast<float*>(momentum);
  a.b = static_cast<int32_t>(b); a.s = static_cast<int32_t>(s); a.n_h = static_cast<int32_t>(n_heads);
  const int64_t total = b * s * n_heads;
  KernelScope scope(kClsOther, static_cast<cudaStream_t>(stream));
  lr_prologue_kernel<<<static_cast<unsigned>(ceil_div(total, 256)), 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  LACT_CUDA(cudaGetLastError());
  return LACT_OK;
}

int lact_out_epilogue(const void* fw_x, const void* weight, const void* gate_proj, int64_t gate_ld, const void* resid,
                      int64_t resid_ld, void* out, int64_t out_ld, int64_t b, int64_t s, int64_t n_heads, int64_t d,
                      float eps, void* stream) {
  if (!fw_x || !weight || !out) return LACT_ERR_NULL;
  LACT_TRY(check_device());
  if (b < 1 || s < 1 || n_heads < 1 || d < 8 || d > 1024 || (d % 8) != 0 || b > 65535 || s > (1ll << 30))
    return LACT_ERR_SHAPE;
  auto bad = [&](const void* p, int64_t ld) {
    return p != nullptr && ((reinterpret_cast<uintptr_t>(p) & 15) != 0 || ld < n_heads * d || (ld % 8) != 0);
  };
  if ((reinterpret_cast<uintptr_t>(fw_x) & 15) != 0 || (reinterpret_cast<uintptr_t>(weight) & 15) != 0 ||
      bad(gate_proj, gate_ld) || bad(resid, resid_ld) || bad(out, out_ld))
    return LACT_ERR_SHAPE;
  EpilogueArgs a;
  std::memset(&a, 0, sizeof(a));
  a.x = static_cast<const bf16*>(fw_x);
  a.weight = static_cast<const float*>(weight);
  a.gate = static_cast<const bf16*>(gate_proj);
  a.resid = static_cast<const bf16*>(resid);
  a.out = static_cast<bf16*>(out);
  a.gate_ld = gate_ld; a.resid_ld = resid_ld; a.out_ld = out_ld;
  a.b = static_cast<int32_t>(b); a.s = static_cast<int32_t>(s);
  a.n_h = static_cast<int32_t>(n_heads); a.d = static_cast<int32_t>(d);
  a.eps = eps;
  const int64_t rows = b * s * n_heads;
  KernelScope scope(kClsOther, static_cast<cudaStream_t>(stream));
  const unsigned grid = static_cast<unsigned>(ceil_div(rows, 8));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (ceil_div(d, 256)) {
    case 1: out_epilogue_kernel<1><<<grid, 256, 0, st>>>(a); break;
    case 2: out_epilogue_kernel<2><<<grid, 256, 0, st>>>(a); break;
    case 3: out_epilogue_kernel<3><<<grid, 256, 0, st>>>(a); break;
    default: out_epilogue_kernel<4><<<grid, 256, 0, st>>>(a); break;
  }
  LACT_CUDA(cudaGetLastError());
  return LACT_OK;
}

int lact_swa_fwd(const void* q, const void* k, const void* v, void* o, int64_t b, int64_t l, int64_t lk, int64_t n_heads,
                 int64_t d, int64_t q_ts, int64_t q_bs, int64_t k_ts, int64_t k_bs, int64_t v_ts, int64_t v_bs, int64_t o_ts,
                 int64_t o_bs, int64_t window, float softmax_scale, const int32_t* seq_start, void* lse, int32_t* status_word,
                 void* stream) {
  if (!q || !k || !v || !o || !status_word) return LACT_ERR_NULL;
  if (seq_start != nullptr && b != 1) return LACT_ERR_CONFIG;   // packed sequences live in one batch entry
  const bool causal = window >= 0;
  if (lk <= 0) lk = l;
  if (causal ? lk != l : seq_start != nullptr) return LACT_ERR_CONFIG;   // causal: keys = queries; block: no packing
  LACT_TRY(check_device());
  if (d != 64 && d != 128) return LACT_ERR_SHAPE;
  if (b < 1 || l < 1 || n_heads < 1 || b > 65535 || n_heads > 65535 || l > (1ll << 30) || lk > (1ll << 30)) return LACT_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(o) & 15) != 0 || o_ts < n_heads * d || (o_ts % 8) != 0 || (o_bs % 8) != 0)
    return LACT_ERR_SHAPE;
  if (!(softmax_scale > 0.f)) return LACT_ERR_CONFIG;
  SwaArgs a;
  std::memset(&a, 0, sizeof(a));
  LACT_TRY(encode_map_heads(&a.q, q, b, l, n_heads, d, q_ts, q_bs));
  LACT_TRY(encode_map_heads(&a.k, k, b, lk, n_heads, d, k_ts, k_bs));
  LACT_TRY(encode_map_heads(&a.v, v, b, lk, n_heads, d, v_ts, v_bs));
  a.Lk = static_cast<int32_t>(lk);
  a.causal = causal ? 1 : 0;
  a.o = static_cast<bf16*>(o);
  a.o_bs = o_bs; a.o_ts = o_ts; a.o_hs = d;
  a.L = static_cast<int32_t>(l);
  a.window = window > 0 && window < l ? static_cast<int32_t>(window) : 0;
  a.heads = static_cast<int32_t>(n_heads);
  a.q_tiles = ceil_div(l, 128);
  a.scale_log2 = softmax_scale * 1.4426950408889634f;
  a.lse = static_cast<float*>(lse);
  a.seq_start = seq_start;
  a.status = status_word;
  const int64_t ctas = b * n_heads * a.q_tiles;
  if (ctas > 0x7FFFFFFFll) return LACT_ERR_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return d == 64 ? launch_swa<64>(a, ctas, st) : launch_swa<128>(a, ctas, st);
}

int lact_swa_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, const void* lse, void* dq,
                 void* dk, void* dv, void* delta, int64_t b, int64_t l, int64_t lk, int64_t n_heads, int64_t d, int64_t q_ts,
                 int64_t q_bs, int64_t k_ts, int64_t k_bs, int64_t v_ts, int64_t v_bs, int64_t o_ts, int64_t o_bs,
                 int64_t do_ts, int64_t do_bs, int64_t window, float softmax_scale, const int32_t* seq_start,
                 int32_t* status_word, void* stream) {
  if (!q || !k || !v || !o || !dout || !lse || !dq || !dk || !dv || !delta || !status_word) return LACT_ERR_NULL;
  if (seq_start != nullptr && b != 1) return LACT_ERR_CONFIG;
  const bool causal = window >= 0;
  if (lk <= 0) lk = l;
  if (causal ? lk != l : seq_start != nullptr) return LACT_ERR_CONFIG;
  LACT_TRY(check_device());
  if (d != 64 && d != 128) return LACT_ERR_SHAPE;
  if (b < 1 || l < 1 || n_heads < 1 || b > 65535 || n_heads > 65535 || l > (1ll << 30) || lk > (1ll << 30)) return LACT_ERR_SHAPE;
  if (!(softmax_scale > 0.f)) return LACT_ERR_CONFIG;
  for (const void* p : {static_cast<const void*>(dq), static_cast<const void*>(dk), static_cast<const void*>(dv), o, dout})
    if ((reinterpret_cast<uintptr_t>(p) & 15) != 0) return LACT_ERR_SHAPE;
  if (o_ts < n_heads * d || do_ts < n_heads * d || (o_ts % 8) || (o_bs % 8) || (do_ts % 8) || (do_bs % 8)) return LACT_ERR_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  {
    SwaDeltaArgs da;
    std::memset(&da, 0, sizeof(da));
    da.o = static_cast<const bf16*>(o);
    da.dout = static_cast<const bf16*>(dout);
    da.o_ts = o_ts; da.o_bs = o_bs; da.d_ts = do_ts; da.d_bs = do_bs;
    da.delta = static_cast<float*>(delta);
    da.b = static_cast<int32_t>(b); da.L = static_cast<int32_t>(l);
    da.heads = static_cast<int32_t>(n_heads); da.d = static_cast<int32_t>(d);
    const int64_t rows = b * l * n_heads;
    KernelScope scope(kClsOther, st);
    swa_delta_kernel<<<static_cast<unsigned>(ceil_div(rows, 8)), 256, 0, st>>>(da);
    LACT_CUDA(cudaGetLastError());
  }
  SwaBwdArgs a;
  std::memset(&a, 0, sizeof(a));
  LACT_TRY(encode_map_heads(&a.q, q, b, l, n_heads, d, q_ts, q_bs));
  LACT_TRY(encode_map_heads(&a.k, k, b, lk, n_heads, d, k_ts, k_bs));
  LACT_TRY(encode_map_heads(&a.v, v, b, lk, n_heads, d, v_ts, v_bs));
  LACT_TRY(encode_map_heads(&a.dout, dout, b, l, n_heads, d, do_ts, do_bs));
  LACT_TRY(encode_map_heads(&a.q64, q, b, l, n_heads, d, q_ts, q_bs, 64));
  LACT_TRY(encode_map_heads(&a.k64, k, b, lk, n_heads, d, k_ts, k_bs, 64));
  LACT_TRY(encode_map_heads(&a.v64, v, b, lk, n_heads, d, v_ts, v_bs, 64));
  LACT_TRY(encode_map_heads(&a.dout64, dout, b, l, n_heads, d, do_ts, do_bs, 64));
  a.lse = static_cast<const float*>(lse);
  a.delta = static_cast<const float*>(delta);
  a.seq_start = seq_start;
  a.o_ts = n_heads * d; a.o_hs = d;   // gradients are written contiguous [b][l or lk][h][d]
  a.L = static_cast<int32_t>(l);
  a.Lk = static_cast<int32_t>(lk);
  a.causal = causal ? 1 : 0;
  a.window = window > 0 && window < l ? static_cast<int32_t>(window) : 0;
  a.heads = static_cast<int32_t>(n_heads);
  a.scale_log2 = softmax_scale * 1.4426950408889634f;
  a.scale = softmax_scale;
  a.status = status_word;
  const int64_t k_tiles = ceil_div(lk, 128), q_tiles = ceil_div(l, 128);
  if (b * n_heads * std::max(k_tiles, q_tiles) > 0x7FFFFFFFll) return LACT_ERR_SHAPE;
  // keys' side (dK, dV): one CTA per key tile; then queries' side (dQ): one CTA per query tile
  a.out0 = static_cast<bf16*>(dk);
  a.out1 = static_cast<bf16*>(dv);
  a.tiles = static_cast<int32_t>(k_tiles);
  a.o_bs = lk * n_heads * d;
  LACT_TRY((d == 64 ? launch_swa_bwd<64, 0>(a, b * n_heads * k_tiles, st) : launch_swa_bwd<128, 0>(a, b * n_heads * k_tiles, st)));
  a.out0 = static_cast<bf16*>(dq);
  a.out1 = nullptr;
  a.tiles = static_cast<int32_t>(q_tiles);
  a.o_bs = l * n_heads * d;
  const int64_t ctas = b * n_heads * q_tiles;
  return d == 64 ? launch_swa_bwd<64, 1>(a, ctas, st) : launch_swa_bwd<128, 1>(a, ctas, st);
}

int lact_l2_norm_add(const void* x, int32_t x_dtype, const void* x_add, int32_t add_dtype, const void* scale, void* y,
                     int32_t y_dtype, int64_t B, int64_t T, int64_t D, float eps, void* stream) {
  if (!x || !x_add || !scale || !y) return LACT_ERR_NULL;
  if (B < 1 || T < 1 || D < 1) return LACT_ERR_SHAPE;
  const int64_t rows = B * T;
  KernelScope scope(kClsOther, static_cast<cudaStream_t>(stream));
  l2_norm_add_kernel<<<ceil_div(rows, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      x, x_dtype == LACT_F32, x_add, add_dtype == LACT_F32, static_cast<const float*>(scale), y, y_dtype == LACT_F32,
      rows, static_cast<int>(D), eps);
  LACT_CUDA(cudaGetLastError());
  return LACT_OK;
}

int lact_prenorm_momentum_l2norm(const void* x, const void* dx, const void* m, const void* mu, const void* scale,
                                 void* x_out, void* m_out, void* y_out, int64_t B, int64_t T, int64_t D, float eps,
                                 void* stream) {
  if (!x || !dx || !m || !mu || !scale || !x_out || !m_out || !y_out) return LACT_ERR_NULL;
  if (B < 1 || T < 1 || D < 1) return LACT_ERR_SHAPE;
  const int64_t rows = B * T;
  KernelScope scope(kClsOther, static_cast<cudaStream_t>(stream));
  prenorm_momentum_kernel<<<ceil_div(rows, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(x), static_cast<const bf16*>(dx), static_cast<const float*>(m),
      static_cast<const float*>(mu), static_cast<const float*>(scale), static_cast<float*>(x_out),
      static_cast<float*>(m_out), static_cast<bf16*>(y_out), rows, static_cast<int>(T), static_cast<int>(D), eps);
  LACT_CUDA(cudaGetLastError());
  return LACT_OK;
}

// One or two independent problems c (+)= alpha (a0 b0^T [+ a1 b1^T]) in one persistent launch (both single-product
// or both two-product; one tile width for the launch).
static int bmm_group(const lact_bmm_desc* d, int n, int32_t* status_word, void* stream, float alpha) {
  if (!d || !status_word) return LACT_ERR_NULL;
  if (n < 1 || n > 2) return LACT_ERR_CONFIG;
  LACT_TRY(check_device());
  const bool two = d[0].a1 != nullptr;
  for (int p = 0; p < n; ++p) {
    const lact_bmm_desc& q = d[p];
    if (!q.a0 || !q.b0 || !q.c || ((q.a1 == nullptr) != (q.b1 == nullptr))) return LACT_ERR_NULL;
    if ((q.a1 != nullptr) != two) return LACT_ERR_CONFIG;
    if (q.batch < 1 || q.batch > 65535 || q.M < 1 || q.N < 8 || q.K < 1 || (q.N % 8)) return LACT_ERR_SHAPE;
    // the contiguous axis of every operand must be a multiple of 8 elements (16-byte TMA strides)
    if (((q.a0_mn || (q.a1 && q.a1_mn)) && (q.M % 8)) ||
        ((!q.a0_mn || (q.a1 && !q.a1_mn) || !q.b0_mn || (q.b1 && !q.b1_mn)) && (q.K % 8)))
      return LACT_ERR_SHAPE;
    if (q.accumulate && q.c_dtype != LACT_F32) return LACT_ERR_DTYPE;
    // c is written in 16-byte (fp32) / 8-byte (bf16) units
    if ((reinterpret_cast<uintptr_t>(q.c) & 15) != 0 || q.c_ld < q.N || (q.c_ld % 8) != 0 ||
        (q.batch > 1 && (q.c_bs % 8) != 0))
      return LACT_ERR_SHAPE;
    auto bad = [&](int mn, int64_t rows, int64_t ld) { return ld < (mn ? rows : q.K); };
    if (bad(q.a0_mn, q.M, q.a0_ld) || bad(q.b0_mn, q.N, q.b0_ld) ||
        (q.a1 && (bad(q.a1_mn, q.M, q.a1_ld) || bad(q.b1_mn, q.N, q.b1_ld))))
      return LACT_ERR_SHAPE;
  }
  // operand as a matrix of `rows` = M or N: [rows][K] with row stride ld, or (MN-major) [K][rows]
  auto mat = [](const lact_bmm_desc& q, const void* ptr, int mn, int64_t rows, int64_t ld, int64_t bs) {
    return mn ? Mat{ptr, q.K, rows, ld, q.batch, bs} : Mat{ptr, rows, q.K, ld, q.batch, bs};
  };
  const lact_bmm_desc& l = d[n - 1];
  int bt = choose_bt({{d[0].N, d[0].M * d[0].batch}, {l.N, n > 1 ? l.M * l.batch : 0}});
  if (two) bt = std::min(bt, 192);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  auto fill = [&](auto& g, int btv) -> int {
    for (int p = 0; p < n; ++p) {
      const lact_bmm_desc& q = d[p];
      auto& P = g.prob[p];
      LACT_TRY(make_operand(kb_of(P), &P.a[0], &P.ai[0], mat(q, q.a0, q.a0_mn, q.M, q.a0_ld, q.a0_bs), q.a0_mn, kBM, 0, 0));
      LACT_TRY(make_operand(kb_of(P), &P.b[0], &P.bi[0], mat(q, q.b0, q.b0_mn, q.N, q.b0_ld, q.b0_bs), q.b0_mn, btv, 0, 0));
      if constexpr (std::remove_reference_t<decltype(g)>::OpType::NA == 2) {
        LACT_TRY(make_operand(kb_of(P), &P.a[1], &P.ai[1], mat(q, q.a1, q.a1_mn, q.M, q.a1_ld, q.a1_bs), q.a1_mn, kBM, 0, 0));
        LACT_TRY(make_operand(kb_of(P), &P.b[1], &P.bi[1], mat(q, q.b1, q.b1_mn, q.N, q.b1_ld, q.b1_bs), q.b1_mn, btv, 0, 0));
      }
      P.M = static_cast<int>(q.M); P.N = static_cast<int>(q.N); P.K = static_cast<int>(q.K);
      P.batch = static_cast<int>(q.batch);
      P.ep = EpiStore{q.c, q.c_bs, q.c_ld, 0, q.c_dtype == LACT_F32, q.accumulate, alpha};
    }
    g.status = status_word;
    return LACT_OK;
  };
  if (n == 1) return two ? launch_op<OpStore2T, 1>(bt, fill, s, kClsOther, 1) : launch_op<OpStoreDirectT, 1>(bt, fill, s, kClsOther, 1);
  return two ? launch_op<OpStore2T, 2>(bt, fill, s, kClsOther, 2) : launch_op<OpStoreDirectT, 2>(bt, fill, s, kClsOther, 2);
}

int lact_bmm_group_bf16(const lact_bmm_desc* problems, int32_t n, int32_t* status_word, void* stream) {
  return bmm_group(problems, n, status_word, stream, 1.0f);
}

static int bmm2_strided(const void* a0, int32_t a0_mn, int64_t a0_ld, int64_t a0_bs, const void* b0, int32_t b0_mn,
                        int64_t b0_ld, int64_t b0_bs, const void* a1, int32_t a1_mn, int64_t a1_ld, int64_t a1_bs,
                        const void* b1, int32_t b1_mn, int64_t b1_ld, int64_t b1_bs, void* c, int32_t c_dtype,
                        int64_t c_ld, int64_t c_bs, int32_t accumulate, int64_t batch, int64_t M, int64_t N, int64_t K,
                        int32_t* status_word, void* stream, float alpha) {
  if (!a0 || !b0 || !c) return LACT_ERR_NULL;
  lact_bmm_desc q;
  std::memset(&q, 0, sizeof(q));
  q.a0 = a0; q.b0 = b0; q.a1 = a1; q.b1 = b1; q.c = c;
  q.a0_ld = a0_ld; q.a0_bs = a0_bs; q.b0_ld = b0_ld; q.b0_bs = b0_bs;
  q.a1_ld = a1_ld; q.a1_bs = a1_bs; q.b1_ld = b1_ld; q.b1_bs = b1_bs;
  q.c_ld = c_ld; q.c_bs = c_bs;
  q.batch = batch; q.M = M; q.N = N; q.K = K;
  q.a0_mn = a0_mn; q.b0_mn = b0_mn; q.a1_mn = a1_mn; q.b1_mn = b1_mn;
  q.c_dtype = c_dtype; q.accumulate = accumulate;
  return bmm_group(&q, 1, status_word, stream, alpha);
}

// Pointwise stage of the fast-weight gradient on its own (see lact_fw_grad): also the backward of apply's
// pre-activations with (k, v) = (q, dO) and unit learning rates.
int lact_fw_grad_pointwise(const void* w0w2, const void* w1, const void* k, int64_t k_ts, int64_t k_bs, const void* v,
                           int64_t v_ts, int64_t v_bs, const void* lr0, const void* lr1, const void* lr2, int32_t lr_dtype,
                           int64_t lr_bs, float w_scale, void* dy02, void* hid, int64_t B, int64_t N, int64_t D, int64_t H,
                           int32_t* status_word, void* stream) {
  if (!w0w2 || !w1 || !k || !v || !dy02 || !hid || !status_word) return LACT_ERR_NULL;
  LACT_TRY(check_device());
  if (B < 1 || B > 65535 || N < 1 || D < 8 || H < 8 || (D % 8) || (H % 8)) return LACT_ERR_SHAPE;
  if (k_ts < D || v_ts < D || (k_ts % 8) || (v_ts % 8) || (k_bs % 8) || (v_bs % 8)) return LACT_ERR_SHAPE;
  if (lr_dtype != LACT_F32 && lr_dtype != LACT_BF16) return LACT_ERR_DTYPE;
  GradArgs a{};
  a.w02b = static_cast<const bf16*>(w0w2);
  a.w1b = static_cast<const bf16*>(w1);
  a.k = k; a.v = v;
  a.k_ts = k_ts; a.k_bs = k_bs; a.v_ts = v_ts; a.v_bs = v_bs;
  a.start = 0; a.end = N;
  a.lr0 = lr0; a.lr1 = lr1; a.lr2 = lr2;
  a.lr_f32 = lr_dtype == LACT_F32;
  a.lr_bs = lr_bs;
  a.w_scale = w_scale;
  a.dy02 = static_cast<bf16*>(dy02);
  a.hid = static_cast<bf16*>(hid);
  a.B = B; a.D = D; a.H = H;
  return run_grad_pointwise(a, status_word, static_cast<cudaStream_t>(stream));
}

int lact_bmm2_strided_bf16(const void* a0, int32_t a0_mn, int64_t a0_ld, int64_t a0_bs, const void* b0, int32_t b0_mn,
                           int64_t b0_ld, int64_t b0_bs, const void* a1, int32_t a1_mn, int64_t a1_ld, int64_t a1_bs,
                           const void* b1, int32_t b1_mn, int64_t b1_ld, int64_t b1_bs, void* c, int32_t c_dtype,
                           int64_t c_ld, int64_t c_bs, int32_t accumulate, int64_t batch, int64_t M, int64_t N, int64_t K,
                           int32_t* status_word, void* stream) {
  return bmm2_strided(a0, a0_mn, a0_ld, a0_bs, b0, b0_mn, b0_ld, b0_bs, a1, a1_mn, a1_ld, a1_bs, b1, b1_mn, b1_ld, b1_bs, c,
                      c_dtype, c_ld, c_bs, accumulate, batch, M, N, K, status_word, stream, 1.0f);
}

// contiguous two-product with the accumulator scaled by alpha before the store (internal)
static int bmm2_scaled(const void* a0, int32_t a0_mn, const void* b0, int32_t b0_mn, const void* a1, int32_t a1_mn,
                       const void* b1, int32_t b1_mn, void* c, int32_t c_dtype, int64_t batch, int64_t M, int64_t N,
                       int64_t K, int32_t* status_word, void* stream, float alpha) {
  auto ld = [&](int mn, int64_t rows) { return mn ? rows : K; };
  return bmm2_strided(a0, a0_mn, ld(a0_mn, M), M * K, b0, b0_mn, ld(b0_mn, N), N * K, a1, a1_mn, ld(a1_mn, M), M * K, b1,
                      b1_mn, ld(b1_mn, N), N * K, c, c_dtype, N, M * N, 0, batch, M, N, K, status_word, stream, alpha);
}

int lact_bmm2_bf16(const void* a0, int32_t a0_mn, const void* b0, int32_t b0_mn, const void* a1, int32_t a1_mn,
                   const void* b1, int32_t b1_mn, void* c, int32_t c_dtype, int32_t accumulate, int64_t batch,
                   int64_t M, int64_t N, int64_t K, int32_t* status_word, void* stream) {
  // contiguous operands: [batch][rows][K] or (MN-major) [batch][K][rows]
  auto ld = [&](int mn, int64_t rows) { return mn ? rows : K; };
  return lact_bmm2_strided_bf16(a0, a0_mn, ld(a0_mn, M), M * K, b0, b0_mn, ld(b0_mn, N), N * K, a1, a1_mn, ld(a1_mn, M),
                                M * K, b1, b1_mn, ld(b1_mn, N), N * K, c, c_dtype, N, M * N, accumulate, batch, M, N, K,
                                status_word, stream);
}

static PlaneArgs make_plane_args(const void* y02, const void* dh, const void* g_dy02, const void* g_hid,
                                 const void* lr0, const void* lr1, const void* lr2, int32_t lr_dtype, float w_scale,
                                 void* dy02, void* hid, void* g_y02, void* g_dh, void* g_lr0, void* g_lr1, void* g_lr2,
                                 int64_t rows, int64_t H) {
  PlaneArgs a;
  std::memset(&a, 0, sizeof(a));
  a.y02 = static_cast<const bf16*>(y02); a.dh = static_cast<const bf16*>(dh);
  a.g_dy02 = static_cast<const bf16*>(g_dy02); a.g_hid = static_cast<const bf16*>(g_hid);
  a.lr0 = lr0; a.lr1 = lr1; a.lr2 = lr2; a.lr_f32 = lr_dtype == LACT_F32; a.w_scale = w_scale;
  a.dy02 = static_cast<bf16*>(dy02); a.hid = static_cast<bf16*>(hid);
  a.g_y02 = static_cast<bf16*>(g_y02); a.g_dh = static_cast<bf16*>(g_dh);
  a.g_lr0 = static_cast<float*>(g_lr0); a.g_lr1 = static_cast<float*>(g_lr1); a.g_lr2 = static_cast<float*>(g_lr2);
  a.rows = rows; a.H = static_cast<int32_t>(H);
  return a;
}

int lact_swiglu_bwd_planes(const void* y02, const void* dh, const void* lr0, const void* lr1, const void* lr2,
                           int32_t lr_dtype, float w_scale, void* dy02, void* hid, int64_t rows, int64_t H,
                           void* stream) {
  if (!y02 || !dh || !dy02 || !hid) return LACT_ERR_NULL;
  if (rows < 1 || H < 8 || (H % 8) != 0) return LACT_ERR_SHAPE;  // planes move as 16-byte vectors
  const PlaneArgs a = make_plane_args(y02, dh, nullptr, nullptr, lr0, lr1, lr2, lr_dtype, w_scale, dy02, hid, nullptr,
                                      nullptr, nullptr, nullptr, nullptr, rows, H);
  KernelScope scope(kClsOther, static_cast<cudaStream_t>(stream));
  swiglu_bwd_planes_kernel<<<ceil_div(rows, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  LACT_CUDA(cudaGetLastError());
  return LACT_OK;
}

int lact_fw_grad_bwd_pointwise(const void* y02, const void* dh, const void* g_dy02, const void* g_hid, const void* lr0,
                               const void* lr1, const void* lr2, int32_t lr_dtype, float w_scale, void* g_y02,
                               void* g_dh, void* dy02, void* hid, void* g_lr0, void* g_lr1, void* g_lr2, int64_t rows,
                               int64_t H, void* stream) {
  if (!y02 || !dh || !g_dy02 || !g_hid || !lr0 || !lr1 || !lr2 || !g_y02 || !g_dh || !dy02 || !hid || !g_lr0 ||
      !g_lr1 || !g_lr2)
    return LACT_ERR_NULL;
  if (rows < 1 || H < 8 || (H % 8) != 0) return LACT_ERR_SHAPE;  // planes move as 16-byte vectors
  const PlaneArgs a = make_plane_args(y02, dh, g_dy02, g_hid, lr0, lr1, lr2, lr_dtype, w_scale, dy02, hid, g_y02, g_dh,
                                      g_lr0, g_lr1, g_lr2, rows, H);
  KernelScope scope(kClsOther, static_cast<cudaStream_t>(stream));
  fw_grad_bwd_pointwise_kernel<<<ceil_div(rows, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  LACT_CUDA(cudaGetLastError());
  return LACT_OK;
}

int lact_renorm_bwd(const void* base, const void* upd, int32_t upd_dtype, const void* n0, const void* dy, void* dw,
                    void* dw_bf16, void* dn0, int64_t rows, int64_t C, int32_t mode, void* stream) {
  if (!base || !upd || !n0 || !dy || !dw) return LACT_ERR_NULL;
  if (rows < 1 || C < 1 || mode < 0 || mode > 2) return LACT_ERR_SHAPE;
  RenormBwdArgs a{static_cast<const float*>(base), upd, upd_dtype == LACT_F32, static_cast<const float*>(n0),
                  static_cast<const float*>(dy), static_cast<float*>(dw), static_cast<bf16*>(dw_bf16),
                  static_cast<float*>(dn0), rows, static_cast<int32_t>(C), mode};
  KernelScope scope(kClsOther, static_cast<cudaStream_t>(stream));
  renorm_bwd_kernel<<<ceil_div(rows, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  LACT_CUDA(cudaGetLastError());
  return LACT_OK;
}

int lact_ns_norm_bwd(const void* g, void* dx0, void* partials, int64_t nmat, int64_t elems_per_matrix, void* stream) {
  if (!g || !dx0 || !partials) return LACT_ERR_NULL;
  return ns_norm_bwd_launch(static_cast<const float*>(g), dx0, 0, static_cast<float*>(dx0), static_cast<float*>(partials),
                            nmat, elems_per_matrix, static_cast<cudaStream_t>(stream));
}

int lact_ns_trace_bwd_fused(const lact_ns_bwd_group* groups, int32_t ngroups, int32_t steps, int32_t const_coeffs,
                            int32_t gram_right, int32_t* status_word, void* stream) {
  if (!groups || !status_word) return LACT_ERR_NULL;
  if (ngroups < 1 || ngroups > 2 || steps < 1 || steps > 5) return LACT_ERR_CONFIG;
  LACT_TRY(check_device());
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  NsTrace tr[2];
  NsGroup grp[2];
  const bf16* du[2] = {nullptr, nullptr};
  for (int g = 0; g < ngroups; ++g) {
    const lact_ns_bwd_group& G = groups[g];
    if (!G.du || !G.g || !G.dg || !G.trace || !G.partials) return LACT_ERR_NULL;
    LACT_TRY(plan_ns_trace(G.trace, G.nmat, G.rows, G.cols, steps, gram_right, &tr[g]));
    if (tr[g].bytes > G.trace_bytes) return LACT_ERR_WORKSPACE;
    grp[g] = tr[g].grp;
    du[g] = static_cast<const bf16*>(G.du);
  }
  // Tile width (one for all phases).  Among the widths that give the m x m phases enough tiles to occupy most SMs,
  // the one with the least padded work (wider on a tie); with few matrices the kernel is bound by each matrix's
  // chain of phases, so the width with the most tiles (again wider on a tie).
  auto mm_tiles = [&](int bt) {
    int64_t t = 0;
    for (int g = 0; g < ngroups; ++g) t += static_cast<int64_t>(grp[g].nmat) * ceil_div(grp[g].m, kBM) * ceil_div(grp[g].m, bt);
    return t;
  };
  auto padded_work = [&](int bt) {
    int64_t w = 0;
    for (int g = 0; g < ngroups; ++g)
      w += static_cast<int64_t>(grp[g].nmat) * bt *
           (2 * ceil_div(grp[g].m, kBM) * ceil_div(grp[g].m, bt) * static_cast<int64_t>(grp[g].m + grp[g].n) / 2 +
            ceil_div(ns_upd_rows(grp[g]), kBM) * ceil_div(ns_upd_cols(grp[g]), bt) * static_cast<int64_t>(grp[g].m));
    return w;
  };
  const int64_t want = static_cast<int64_t>(sm_count()) * 3 / 4;
  int bt = 0;
  for (int cand : {192, 128, 64})
    if (mm_tiles(cand) >= want && (bt == 0 || padded_work(cand) < padded_work(bt))) bt = cand;
  if (bt == 0) bt = mm_tiles(64) > mm_tiles(128) ? 64 : (mm_tiles(128) > mm_tiles(192) ? 128 : 192);
  // Q and T are symmetric: with Gram sides that are multiples of 128 their phases run on the 128 x 128 tiles on and
  // above the diagonal only
  bool sym_ok = bt == 192;
  for (int g = 0; g < ngroups; ++g) sym_ok = sym_ok && grp[g].m % kBM == 0 && grp[g].m >= 2 * kBM;
  int rc = LACT_ERR_CONFIG;
  if (sym_ok) rc = launch_ns_bwd_fused<128, 192, true>(tr, du, ngroups, steps, const_coeffs, status_word, s);
  else if (bt == 192) rc = launch_ns_bwd_fused<192, 192, false>(tr, du, ngroups, steps, const_coeffs, status_word, s);
  else if (bt == 128) rc = launch_ns_bwd_fused<128, 128, false>(tr, du, ngroups, steps, const_coeffs, status_word, s);
  else rc = launch_ns_bwd_fused<64, 64, false>(tr, du, ngroups, steps, const_coeffs, status_word, s);
  if (rc != LACT_OK) return rc;
  // the gradient w.r.t. the first iterate is the bf16 buffer the last phase wrote; the Frobenius normalisation
  // X0 = bf16(G) / (||G|| + 1e-7) is differentiated into the caller's fp32 dG
  for (int g = 0; g < ngroups; ++g) {
    const lact_ns_bwd_group& G = groups[g];
    LACT_TRY(ns_norm_bwd_launch(static_cast<const float*>(G.g), tr[g].dXb, 1, static_cast<float*>(G.dg),
                                static_cast<float*>(G.partials), G.nmat, G.rows * G.cols, s));
  }
  return LACT_OK;
}

int lact_momentum_bwd_slices(void) { return kNormBwdSlices; }

int lact_momentum_bwd(void* dg0, void* dg1, void* carry0, void* carry1, const void* mprev0, const void* mprev1,
                      void* dgb0, void* dgb1, const void* beta, void* dbeta, int64_t B, int64_t n0, int64_t n1,
                      int32_t add_carry, void* stream) {
  if (!dg0 || !dg1 || !dgb0 || !dgb1) return LACT_ERR_NULL;
  if ((carry0 == nullptr) != (carry1 == nullptr) || (mprev0 == nullptr) != (mprev1 == nullptr)) return LACT_ERR_NULL;
  if (B < 1 || B > 65535 * 16 || n0 < 4 || n1 < 4 || (n0 % 4) != 0 || (n1 % 4) != 0) return LACT_ERR_SHAPE;
  MomentumBwdArgs a;
  std::memset(&a, 0, sizeof(a));
  a.dg[0] = static_cast<float*>(dg0); a.dg[1] = static_cast<float*>(dg1);
  a.carry[0] = static_cast<float*>(carry0); a.carry[1] = static_cast<float*>(carry1);
  a.mprev[0] = static_cast<const float*>(mprev0); a.mprev[1] = static_cast<const float*>(mprev1);
  a.dgb[0] = static_cast<bf16*>(dgb0); a.dgb[1] = static_cast<bf16*>(dgb1);
  a.beta = static_cast<const float*>(beta);
  a.dbeta = static_cast<float*>(dbeta);
  a.n[0] = n0; a.n[1] = n1;
  a.add_carry = add_carry;
  KernelScope scope(kClsOther, static_cast<cudaStream_t>(stream));
  momentum_bwd_kernel<<<dim3(static_cast<unsigned>(B), kNormBwdSlices), 512, 0, static_cast<cudaStream_t>(stream)>>>(a);
  LACT_CUDA(cudaGetLastError());
  return LACT_OK;
}

// ---------------------------------------------------------------- fp32 mode building blocks
int lact_sgemm_f32(const void* a, int32_t a_t, const void* b, int32_t b_t, void* c, int32_t accumulate,
                   const void* beta, int64_t batch, int64_t M, int64_t N, int64_t K, void* stream) {
  if (!a || !b || !c) return LACT_ERR_NULL;
  if (batch < 1 || batch > 65535 || M < 1 || N < 1 || K < 1) return LACT_ERR_SHAPE;
  dim3 grid(ceil_div(N, 64), ceil_div(M, 64), static_cast<unsigned>(batch));
  if (grid.y > 65535) return LACT_ERR_SHAPE;
  KernelScope scope(kClsOther, static_cast<cudaStream_t>(stream));
  sgemm_f32_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(a), a_t, static_cast<const float*>(b), b_t, static_cast<float*>(c), accumulate,
      static_cast<const float*>(beta), static_cast<int>(M), static_cast<int>(N), static_cast<int>(K));
  LACT_CUDA(cudaGetLastError());
  return LACT_OK;
}

int lact_swiglu_planes_f32(const void* y02, const void* dh, const void* lr0, const void* lr1, const void* lr2,
                           int32_t lr_dtype, float w_scale, void* dy02, void* hid, int64_t rows, int64_t H,
                           void* stream) {
  if (!y02 || !hid || (dh != nullptr && !dy02)) return LACT_ERR_NULL;
  if (rows < 1 || H < 8 || (H % 8) != 0) return LACT_ERR_SHAPE;  // planes move as 16-byte vectors
  KernelScope scope(kClsOther, static_cast<cudaStream_t>(stream));
  swiglu_planes_f32_kernel<<<ceil_div(rows, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(y02), static_cast<const float*>(dh), lr0, lr1, lr2, lr_dtype == LACT_F32, w_scale,
      static_cast<float*>(dy02), static_cast<float*>(hid), rows, static_cast<int>(H));
  LACT_CUDA(cudaGetLastError());
  return LACT_OK;
}

int lact_add_renorm(void* master, void* compute, void* shadow, const void* n0, const void* g, const void* x,
                    int64_t B, int64_t R, int64_t C, int32_t mode, int32_t prenorm, int32_t prenorm_bf16,
                    int32_t quirk, void* stream) {
  if (!master || !shadow || !n0 || !g) return LACT_ERR_NULL;
  if (B < 1 || R < 1 || C < 4 || (C % 4) || C > kRenormMaxCols || mode < 0 || mode > 2) return LACT_ERR_SHAPE;
  RenormArgs r;
  std::memset(&r, 0, sizeof(r));
  r.master = static_cast<float*>(master);
  r.compute = static_cast<float*>(compute);
  r.shadow = static_cast<bf16*>(shadow);
  r.n0 = static_cast<const float*>(n0);
  r.g = static_cast<const float*>(g);
  r.x = static_cast<const bf16*>(x);
  r.x_bs = R * C;
  r.B = static_cast<int>(B); r.R = static_cast<int>(R); r.C = static_cast<int>(C);
  r.mode = mode; r.prenorm = prenorm; r.prenorm_bf16 = prenorm_bf16; r.quirk = quirk;
  RenormArgs none = r;
  none.B = 0;
  return launch_add_renorm(r, none, static_cast<cudaStream_t>(stream));
}

int lact_bmm_bf16(const void* a, int32_t a_mn_major, const void* b, int32_t b_mn_major, void* c, int32_t c_dtype,
                  int64_t batch, int64_t M, int64_t N, int64_t K, int32_t* status_word, void* stream) {
  if (!a || !b || !c || !status_word) return LACT_ERR_NULL;
  LACT_TRY(check_device());
  if (batch < 1 || batch > 65535 || M < 1 || N < 8 || K < 1 || (M % 8) || (N % 8) || (K % 8)) return LACT_ERR_SHAPE;
  const Mat A = a_mn_major ? Mat{a, K, M, M, batch, K * M} : Mat{a, M, K, K, batch, M * K};
  const Mat Bm = b_mn_major ? Mat{b, K, N, N, batch, K * N} : Mat{b, N, K, K, batch, N * K};
  auto fill = [&](auto& g, int btv) -> int {
    auto& P = g.prob[0];
    LACT_TRY(make_operand(kb_of(P), &P.a[0], &P.ai[0], A, a_mn_major, kBM, 0, 0));
    LACT_TRY(make_operand(kb_of(P), &P.b[0], &P.bi[0], Bm, b_mn_major, btv, 0, 0));
    P.M = static_cast<int>(M); P.N = static_cast<int>(N); P.K = static_cast<int>(K);
    P.batch = static_cast<int>(batch);
    P.ep = EpiStore{c, M * N, N, 0, 1, 0};
    g.status = status_word;
    return LACT_OK;
  };
  auto fill_bf16 = [&](auto& g, int btv) -> int {
    auto& P = g.prob[0];
    LACT_TRY(make_operand(kb_of(P), &P.a[0], &P.ai[0], A, a_mn_major, kBM, 0, 0));
    LACT_TRY(make_operand(kb_of(P), &P.b[0], &P.bi[0], Bm, b_mn_major, btv, 0, 0));
    LACT_TRY(make_output(&P.out[0], &P.oi[0], Mat{c, M, N, N, batch, M * N}, 0, 0));
    P.M = static_cast<int>(M); P.N = static_cast<int>(N); P.K = static_cast<int>(K);
    P.batch = static_cast<int>(batch);
    g.status = status_word;
    return LACT_OK;
  };
  const int bt = choose_bt({{N, 1}});
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (c_dtype == LACT_F32) return launch_op<OpStoreDirectT, 1>(bt, fill, s, kClsOther, 1);
  return launch_op<OpBmmStore, 1>(bt, fill_bf16, s, kClsOther, 1);
}

}  // extern "C"
