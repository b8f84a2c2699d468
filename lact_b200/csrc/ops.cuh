// GEMM ops (operand/accumulator wiring + fp32 epilogues) built on the tcgen05 engine, and the
// small row-wise kernels of the fast-weight update (norms, momentum mean, Newton-Schulz
// normalisation, add + renormalise).
#pragma once
#include "umma_gemm.cuh"

namespace lact {

using bf16 = __nv_bfloat16;

// one value of an fp32 or bf16 vector
__device__ __forceinline__ float load_scalar(const void* p, int is_f32, int64_t idx) {
  return is_f32 ? reinterpret_cast<const float*>(p)[idx] : __bfloat162float(reinterpret_cast<const bf16*>(p)[idx]);
}

// ------------------------------------------------------------------------------------------
// epilogues
// ------------------------------------------------------------------------------------------
// Plain store of one accumulator (bf16 or fp32), rows shifted by row_off.
struct EpiStore {
  void* out;
  int64_t bs, ld;
  int32_t row_off;
  int32_t f32;
  int32_t accumulate;  // fp32 only: out += acc (each element is owned by exactly one lane)
  float alpha = 1.0f;  // the accumulator is multiplied by alpha before it is stored / added
  static constexpr uint32_t kScratch = kEpiWarps * 32 * 144;
  // One warp's 32 x 32 block of results, thread `lane` holding row `row0 + lane` in v[0..31]: the block goes through
  // `scratch` (this warp's 32 x 144 bytes of shared memory) so that eight lanes cover a 128-byte row segment and every
  // global access of the warp touches four full lines instead of 32.
  __device__ __forceinline__ void warp_block(int batch, int row0, int col, int M, int N, const float* v, uint32_t scratch,
                                             int lane) const {
#pragma unroll
    for (int gq = 0; gq < 8; ++gq)
      asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(scratch + lane * 144 + gq * 16), "f"(v[gq * 4] * alpha),
                   "f"(v[gq * 4 + 1] * alpha), "f"(v[gq * 4 + 2] * alpha), "f"(v[gq * 4 + 3] * alpha)
                   : "memory");
    __syncwarp();
    const int u = lane & 7, rsub = lane >> 3;
    const bool col_ok = col + u * 4 + 4 <= N;
    const bool rmw = f32 && accumulate;
    const int64_t base = batch * bs + col + u * 4;
    float4 old[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int row = row0 + i * 4 + rsub;
      old[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (rmw && col_ok && row < M)
        old[i] = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(out) + base +
                                                  static_cast<int64_t>(row + row_off) * ld);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int rr = i * 4 + rsub, row = row0 + rr;
      if (!col_ok || row >= M) continue;
      float4 x;
      asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                   : "=f"(x.x), "=f"(x.y), "=f"(x.z), "=f"(x.w)
                   : "r"(scratch + rr * 144 + u * 16)
                   : "memory");
      x.x += old[i].x; x.y += old[i].y; x.z += old[i].z; x.w += old[i].w;
      const int64_t idx = base + static_cast<int64_t>(row + row_off) * ld;
      if (f32) *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + idx) = x;
      else *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(out) + idx) = make_uint2(pack_bf16x2(x.x, x.y), pack_bf16x2(x.z, x.w));
    }
    __syncwarp();  // the scratch block is rewritten by the next call
  }
};

// Fast-weight gradient accumulation: g = round_bf16(acc) [+ beta[batch] * g_old]; g is stored in
// fp32 (state / momentum buffer) or bf16 (sub-op output).
struct EpiDW {
  void* g;
  int64_t bs, ld;
  const float* beta;  // per-batch momentum factor, or nullptr
  int32_t round_bf16;
  int32_t out_f32;
  // optional: partial sums of squares of bf16(g), one per output tile and epilogue warp (the
  // Frobenius norm that Newton-Schulz needs, gathered while the gradient is still in registers);
  // index = ((batch * tiles_m + tile_m) * tiles_n + tile_n) * 8 + warp
  float* partial;
  int32_t tiles_m, tiles_n;
  // optional: bf16 copy of g with the same strides (the first Newton-Schulz iterate before scaling)
  bf16* gb;
  // optional: the momentum state is read from here instead of `g` (same layout, fp32): training keeps every update's
  // state in its own slot, so the previous one is read and the next one written without a copy in between
  const float* g_prev = nullptr;
  // One warp's 32 x 32 block of results, thread `lane` holding row `row0 + lane` in v[0..31].  The block goes
  // through `scratch` (this warp's 32 x 144 bytes of shared memory) so that the read-modify-write of the fp32
  // state is issued with eight lanes per 128-byte row segment (four full lines per instruction) instead of one
  // row per lane.  Returns this lane's share of the sum of squares of the bf16-rounded results if `want_ss`.
  __device__ __forceinline__ float warp_block(int batch, int row0, int col, int M, int N, const float* v,
                                              uint32_t scratch, int lane, bool want_ss) const {
#pragma unroll
    for (int gq = 0; gq < 8; ++gq) {
      float r[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) r[j] = round_bf16 ? bf16_round(v[gq * 4 + j]) : v[gq * 4 + j];
      asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(scratch + lane * 144 + gq * 16), "f"(r[0]), "f"(r[1]),
                   "f"(r[2]), "f"(r[3])
                   : "memory");
    }
    __syncwarp();
    const int u = lane & 7, rsub = lane >> 3;
    const bool col_ok = col + u * 4 + 4 <= N;
    const bool rmw = out_f32 && beta != nullptr;
    const float bt = rmw ? beta[batch] : 0.f;
    const int64_t base = batch * bs + col + u * 4;
    float4 old[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int row = row0 + i * 4 + rsub;
      old[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (rmw && col_ok && row < M)
        old[i] = *reinterpret_cast<const float4*>((g_prev != nullptr ? g_prev : reinterpret_cast<const float*>(g)) + base +
                                                  static_cast<int64_t>(row) * ld);
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int rr = i * 4 + rsub, row = row0 + rr;
      if (!col_ok || row >= M) continue;
      float4 x;
      asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                   : "=f"(x.x), "=f"(x.y), "=f"(x.z), "=f"(x.w)
                   : "r"(scratch + rr * 144 + u * 16)
                   : "memory");
      x.x += old[i].x * bt; x.y += old[i].y * bt; x.z += old[i].z * bt; x.w += old[i].w * bt;
      const int64_t idx = base + static_cast<int64_t>(row) * ld;
      const uint2 xb = make_uint2(pack_bf16x2(x.x, x.y), pack_bf16x2(x.z, x.w));
      if (out_f32) *reinterpret_cast<float4*>(reinterpret_cast<float*>(g) + idx) = x;
      else *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(g) + idx) = xb;
      if (gb != nullptr) *reinterpret_cast<uint2*>(gb + idx) = xb;
      if (want_ss) {
        const float a = bf16_round(x.x), b = bf16_round(x.y), c = bf16_round(x.z), d = bf16_round(x.w);
        ss += a * a + b * b + c * c + d * d;
      }
    }
    __syncwarp();  // the scratch block is rewritten by the next call
    return ss;
  }
};

// Newton-Schulz epilogue: out = bf16(acc * acc_scale * s^scale_pow + diag * I), s = scale[matrix].
struct EpiNs {
  float diag;
  float acc_scale;
  const float* scale;  // per-matrix 1 / (||G||_F + 1e-7), or nullptr
  int32_t scale_pow;   // 0: no per-matrix scaling, 1: s, 2: s * s
};

// Fast-weight-gradient pointwise stage: from y0 = k w0^T, y2 = k w2^T, dh = v w1 and the three
// per-token learning rates produce (fp32 math, one rounding to bf16 at the store)
//   hidden*lr1, dy0 = dh*y2*sigma*(1 + y0*(1 - sigma))*lr0, dy2 = dh*silu(y0)*lr2.
struct EpiFwGrad {
  const void *lr0, *lr1, *lr2;
  int32_t lr_f32;
  int32_t tok_off;  // global token index of row 0
  int64_t lr_bs;    // batch stride of the lr tensors (token stride is 1)
  float w_scale;
};

// ------------------------------------------------------------------------------------------
// ops
// ------------------------------------------------------------------------------------------
// Ops without global epilogue operands prefetch nothing.
struct NoPrefetch {};

// k-blocks per ring stage: two when two such stages fit next to `staging` bytes (each operand tile of a
// stage then arrives as ONE TMA box spanning both k-blocks: the load path is bound by the number of
// boxes, not by bytes), else one
__host__ __device__ constexpr int kb_per_stage(uint32_t kblock_bytes, uint32_t staging) {
  return (232448u - 1024u - 256u - staging) / (2 * kblock_bytes) >= 2 ? 2 : 1;
}
// ring depth that fits 227 KB next to `staging` bytes of output tiles
__host__ __device__ constexpr int ring_depth(uint32_t stage_bytes, uint32_t staging) {
  return static_cast<int>((232448u - 1024u - 256u - staging) / stage_bytes) > 8
             ? 8
             : static_cast<int>((232448u - 1024u - 256u - staging) / stage_bytes);
}

// c = a b^T, one accumulator, direct (register) epilogue `EpiT`; output tile 128 x BT.
template <class EpiT, int BT_>
struct OpBmm {
  static constexpr int NA = 1, NB = 1, NACC = 1, BT = BT_, NTERMS = 1, NOUT = 0;
  static constexpr bool kTileReduce = false;
  static constexpr bool kWarpTranspose = true, kReverseBatch = false;
  static constexpr uint32_t kEpiScratch = EpiT::kScratch;
  static constexpr int KB = 1;  // measured: two-k-block stages slow the training backward's products by 7 %
  static constexpr int STAGES = ring_depth(KB * (kATileBytes + BT_ * kBK * 2), kEpiScratch);
  using Epi = EpiT;
  __host__ __device__ static constexpr int term_a(int) { return 0; }
  __host__ __device__ static constexpr int term_b(int) { return 0; }
  __host__ __device__ static constexpr int term_col(int) { return 0; }
  __host__ __device__ static constexpr int term_n(int) { return BT_; }
  __host__ __device__ static constexpr bool term_first(int) { return true; }
  using Prefetch = NoPrefetch;
  __device__ static __forceinline__ void prefetch(const Epi&, int, int, int, int, int, int, Prefetch&) {}
  __device__ static __forceinline__ void epilogue_warp(const Epi& ep, int batch, int row0, int col, int M, int N,
                                                       const float (&v)[1][32], Prefetch&, uint32_t scratch, int lane) {
    ep.warp_block(batch, row0, col, M, N, v[0], scratch, lane);
  }
};

// Token contraction of the fast-weight gradient: c = a b^T with the momentum epilogue; each tile
// also leaves the sums of squares of its bf16-rounded results, one per epilogue warp (per-thread,
// then warp shuffle; the consumer adds them in a fixed order, so the norm is deterministic).
template <int BT_>
struct OpDW {
  static constexpr int NA = 1, NB = 1, NACC = 1, BT = BT_, NTERMS = 1, NOUT = 0;
  static constexpr bool kTileReduce = true;
  static constexpr bool kWarpTranspose = true;                   // results reach global memory through `EpiDW::warp_block`
  static constexpr bool kReverseBatch = true;                    // reads the planes the pointwise kernel has just written
  static constexpr uint32_t kEpiScratch = kEpiWarps * 32 * 144;  // one 32 x 32 fp32 block (rows padded to 144 bytes) per epilogue warp
  static constexpr int KB = kb_per_stage(kATileBytes + BT_ * kBK * 2, kEpiScratch);
  static constexpr int STAGES = ring_depth(KB * (kATileBytes + BT_ * kBK * 2), kEpiScratch);
  using Epi = EpiDW;
  __host__ __device__ static constexpr int term_a(int) { return 0; }
  __host__ __device__ static constexpr int term_b(int) { return 0; }
  __host__ __device__ static constexpr int term_col(int) { return 0; }
  __host__ __device__ static constexpr int term_n(int) { return BT_; }
  __host__ __device__ static constexpr bool term_first(int) { return true; }
  struct Prefetch {
    float acc;
  };
  __device__ static __forceinline__ void prefetch(const Epi&, int, int, int, int, int, int, Prefetch& pf) {
    pf.acc = 0.f;
  }
  __device__ static __forceinline__ void epilogue_warp(const Epi& ep, int batch, int row0, int col, int M, int N,
                                                       const float (&v)[1][32], Prefetch& pf, uint32_t scratch,
                                                       int lane) {
    pf.acc += ep.warp_block(batch, row0, col, M, N, v[0], scratch, lane, ep.partial != nullptr);
  }
  __device__ static __forceinline__ float tile_value(const Prefetch& pf) { return pf.acc; }
  __device__ static __forceinline__ void tile_store(const Epi& ep, int batch, int tile_m, int tile_n, int warp_slot,
                                                    float value) {
    if (ep.partial != nullptr)
      ep.partial[((static_cast<int64_t>(batch) * ep.tiles_m + tile_m) * ep.tiles_n + tile_n) * kEpiWarps + warp_slot] =
          value;
  }
};

// c = bf16(a b^T) written through the staged TMA-store epilogue.
struct EpiNone {};
template <int BT_>
struct OpBmmStore {
  static constexpr int NA = 1, NB = 1, NACC = 1, BT = BT_, NTERMS = 1, NOUT = 1;
  static constexpr bool kTileReduce = false;
  static constexpr bool kWarpTranspose = false, kReverseBatch = true;
  static constexpr uint32_t kEpiScratch = 0;
  static constexpr int KB = 1;  // measured: two-k-block stages are 5 % slower for this op (K-major operands, short K)
  static constexpr int STAGES = ring_depth(KB * (kATileBytes + BT_ * kBK * 2), kBM * BT_ * 2);
  using Epi = EpiNone;
  __host__ __device__ static constexpr int term_a(int) { return 0; }
  __host__ __device__ static constexpr int term_b(int) { return 0; }
  __host__ __device__ static constexpr int term_col(int) { return 0; }
  __host__ __device__ static constexpr int term_n(int) { return BT_; }
  __host__ __device__ static constexpr bool term_first(int) { return true; }
  using Prefetch = NoPrefetch;
  __device__ static __forceinline__ void prefetch(const Epi&, int, int, int, int, int, int, Prefetch&) {}
  __device__ static __forceinline__ bool skip_store(const Epi&, int) { return false; }
  __device__ static __forceinline__ void epilogue_staged(const Epi&, int, int, int, int, int, const float (&v)[1][32],
                                                         float (&o)[1][32], Prefetch&) {
#pragma unroll
    for (int j = 0; j < 32; ++j) o[0][j] = v[0][j];
  }
};

// c = a0 b0^T + a1 b1^T (both products accumulate into one accumulator; equal K), direct epilogue.
template <class EpiT, int BT_>
struct OpBmm2 {
  static constexpr int NA = 2, NB = 2, NACC = 1, BT = BT_, NTERMS = 2, NOUT = 0;
  static constexpr bool kTileReduce = false;
  static constexpr bool kWarpTranspose = true, kReverseBatch = false;
  static constexpr uint32_t kEpiScratch = EpiT::kScratch;
  static constexpr int KB = 1;
  static constexpr int STAGES = ring_depth(KB * (2 * kATileBytes + 2 * BT_ * kBK * 2), kEpiScratch);
  using Epi = EpiT;
  __host__ __device__ static constexpr int term_a(int t) { return t; }
  __host__ __device__ static constexpr int term_b(int t) { return t; }
  __host__ __device__ static constexpr int term_col(int) { return 0; }
  __host__ __device__ static constexpr int term_n(int) { return BT_; }
  __host__ __device__ static constexpr bool term_first(int t) { return t == 0; }
  using Prefetch = NoPrefetch;
  __device__ static __forceinline__ void prefetch(const Epi&, int, int, int, int, int, int, Prefetch&) {}
  __device__ static __forceinline__ void epilogue_warp(const Epi& ep, int batch, int row0, int col, int M, int N,
                                                       const float (&v)[1][32], Prefetch&, uint32_t scratch, int lane) {
    ep.warp_block(batch, row0, col, M, N, v[0], scratch, lane);
  }
};

// Newton-Schulz GEMM.  One iteration X' = a X + (b A + c A A) X, A = X X^T, runs as three plain products with
// the polynomial's residual terms folded in as multiples of the identity (completing the square):
//   gram:    S = A + (b / 2c) I                         (diagonal add in the epilogue)
//   poly:    P = c S S + (a - b^2 / 4c) I = a I + b A + c A A   (S is symmetric: its rows serve as both operands)
//   update:  X' = P X
// so no phase reads a residual tile or writes a second output.  All stored values are bf16 with fp32
// accumulation, as in the reference; the folding moves its rounding points (one rounding per stored matrix),
// which against an fp64 iteration is about twice as accurate as the reference's eager bf16 arithmetic.
// The Frobenius normalisation X0 = G / (||G|| + 1e-7) can be folded in as well: the first iteration then runs
// on bf16(G) itself and its gram / update epilogues multiply the fp32 accumulator by s^2 / s,
// s = 1 / (||G|| + 1e-7) (per matrix, `scale`).
// SYM_: the output is symmetric (Gram matrix, polynomial): only tiles on and above the diagonal are computed and the
// others are stored as transposes (see op_symmetric in the engine); identical values, a third fewer products at m = 384.
template <int BT_, bool SYM_>
struct OpNsT {
  static constexpr int NA = 1, NB = 1, NACC = 1, BT = BT_, NTERMS = 1, NOUT = 1;
  static constexpr bool kTileReduce = false;
  static constexpr bool kWarpTranspose = false, kReverseBatch = false;
  static constexpr bool kSymmetric = SYM_;
  static constexpr uint32_t kEpiScratch = 0;
  static constexpr uint32_t kStagingTiles = (SYM_ ? 2 : 1) * kBM * BT_ * 2;
  static constexpr int KB = kb_per_stage(kATileBytes + BT_ * kBK * 2, kStagingTiles);
  static constexpr int STAGES = ring_depth(KB * (kATileBytes + BT_ * kBK * 2), kStagingTiles);
  using Epi = EpiNs;
  __host__ __device__ static constexpr int term_a(int) { return 0; }
  __host__ __device__ static constexpr int term_b(int) { return 0; }
  __host__ __device__ static constexpr int term_col(int) { return 0; }
  __host__ __device__ static constexpr int term_n(int) { return BT_; }
  __host__ __device__ static constexpr bool term_first(int) { return true; }
  __device__ static __forceinline__ bool skip_store(const Epi&, int) { return false; }
  struct Prefetch {
    float sc;
  };
  __device__ static __forceinline__ void prefetch(const Epi& ep, int batch, int, int, int, int, int, Prefetch& pf) {
    pf.sc = ep.acc_scale;
    if (ep.scale_pow != 0 && ep.scale != nullptr) {
      const float s1 = ep.scale[batch];
      pf.sc *= ep.scale_pow == 2 ? s1 * s1 : s1;
    }
  }
  __device__ static __forceinline__ void epilogue_staged(const Epi& ep, int, int row, int col, int, int,
                                                         const float (&v)[1][32], float (&o)[1][32], Prefetch& pf) {
#pragma unroll
    for (int j = 0; j < 32; ++j) o[0][j] = bf16_round(v[0][j] * pf.sc + (row == col + j ? ep.diag : 0.f));
  }
};

template <int BT_>
using OpNs = OpNsT<BT_, false>;

// Two-product Newton-Schulz GEMM for the backward pass: out = bf16(acc_scale * (a0 b0^T + a1 b1^T)), both products
// into one accumulator (equal K), one k-block of both products per ring stage, staged (TMA-stored) output.
template <int BT_, bool SYM_>
struct OpNs2T {
  static constexpr int NA = 2, NB = 2, NACC = 1, BT = BT_, NTERMS = 2, NOUT = 1;
  static constexpr bool kTileReduce = false;
  static constexpr bool kWarpTranspose = false, kReverseBatch = false;
  static constexpr bool kSymmetric = SYM_;
  static constexpr uint32_t kEpiScratch = 0;
  static constexpr int KB = 1;
  static constexpr int STAGES = ring_depth(2 * (kATileBytes + BT_ * kBK * 2), (SYM_ ? 2 : 1) * kBM * BT_ * 2);
  using Epi = EpiNs;
  __host__ __device__ static constexpr int term_a(int t) { return t; }
  __host__ __device__ static constexpr int term_b(int t) { return t; }
  __host__ __device__ static constexpr int term_col(int) { return 0; }
  __host__ __device__ static constexpr int term_n(int) { return BT_; }
  __host__ __device__ static constexpr bool term_first(int t) { return t == 0; }
  __device__ static __forceinline__ bool skip_store(const Epi&, int) { return false; }
  struct Prefetch {
    float sc;
  };
  __device__ static __forceinline__ void prefetch(const Epi& ep, int, int, int, int, int, int, Prefetch& pf) {
    pf.sc = ep.acc_scale;
  }
  __device__ static __forceinline__ void epilogue_staged(const Epi&, int, int, int, int, int, const float (&v)[1][32],
                                                         float (&o)[1][32], Prefetch& pf) {
#pragma unroll
    for (int j = 0; j < 32; ++j) o[0][j] = v[0][j] * pf.sc;
  }
};

template <int BT_>
using OpNs2 = OpNs2T<BT_, false>;

// [y0 | y2] = x [w0 slice ; w2 slice]^T; epilogue = SwiGLU gate, staged.  With one k-block per stage
// the two weight tiles are adjacent in shared memory and one 128 x 2BT MMA covers both; with two
// k-blocks per stage each tile holds its k-blocks back to back, so the product is two 128 x BT MMAs
// into adjacent accumulator columns.
template <int BT_>
struct OpSwigluGate {
  static constexpr int KB = 1;  // measured: two-k-block stages (a 2-deep ring here) are 7 % slower for this op
  static constexpr int NA = 1, NB = 2, NACC = 2, BT = BT_, NTERMS = KB, NOUT = 1;
  static constexpr bool kTileReduce = false;
  static constexpr bool kWarpTranspose = false, kReverseBatch = false;
  static constexpr uint32_t kEpiScratch = 0;
  static constexpr int STAGES = ring_depth(KB * (kATileBytes + 2 * BT_ * kBK * 2), kBM * BT_ * 2);
  using Epi = EpiNone;
  __host__ __device__ static constexpr int term_a(int) { return 0; }
  __host__ __device__ static constexpr int term_b(int t) { return t; }
  __host__ __device__ static constexpr int term_col(int t) { return t * BT_; }
  __host__ __device__ static constexpr int term_n(int) { return KB == 2 ? BT_ : 2 * BT_; }
  __host__ __device__ static constexpr bool term_first(int) { return true; }
  using Prefetch = NoPrefetch;
  __device__ static __forceinline__ void prefetch(const Epi&, int, int, int, int, int, int, Prefetch&) {}
  __device__ static __forceinline__ bool skip_store(const Epi&, int) { return false; }
  __device__ static __forceinline__ void epilogue_staged(const Epi&, int, int, int, int, int, const float (&v)[2][32],
                                                         float (&o)[1][32], Prefetch&) {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float y0 = v[0][j];
      o[0][j] = v[1][j] * (y0 * sigmoidf_fast(y0));
    }
  }
};

// [y0 | y2] = k [w0 slice ; w2 slice]^T (one 128 x 128 MMA) and dh = v w1 slice (128 x 64 MMA):
// three accumulators of 64 hidden columns, two activation tiles, three weight tiles; three staged
// outputs (dy0, dy2, hidden * lr1).
struct OpFwGradPointwise {
  static constexpr int NA = 2, NB = 3, NACC = 3, BT = 64, NTERMS = 2, NOUT = 3;
  static constexpr bool kTileReduce = false;
  static constexpr bool kWarpTranspose = false, kReverseBatch = false;
  static constexpr uint32_t kEpiScratch = 0;
  static constexpr int KB = 1;  // two k-blocks of this op's five tiles would leave a one-stage ring
  static constexpr int STAGES = ring_depth(KB * (2 * kATileBytes + 3 * 64 * kBK * 2), 3 * kBM * 64 * 2);
  using Epi = EpiFwGrad;
  __host__ __device__ static constexpr int term_a(int t) { return t; }
  __host__ __device__ static constexpr int term_b(int t) { return t == 0 ? 0 : 2; }
  __host__ __device__ static constexpr int term_col(int t) { return t == 0 ? 0 : 128; }
  __host__ __device__ static constexpr int term_n(int t) { return t == 0 ? 128 : 64; }
  __host__ __device__ static constexpr bool term_first(int) { return true; }
  struct Prefetch {
    float l0, l1, l2;
  };
  __device__ static __forceinline__ void prefetch(const Epi& ep, int batch, int row, int, int, int M, int,
                                                  Prefetch& pf) {
    pf.l0 = pf.l1 = pf.l2 = 0.f;
    if (row < M) {
      const int64_t li = batch * ep.lr_bs + ep.tok_off + row;
      // (a null learning rate stands for 1: the backward of apply is this same pointwise stage on (q, dO))
      pf.l0 = (ep.lr0 ? load_scalar(ep.lr0, ep.lr_f32, li) : 1.f) * ep.w_scale;
      pf.l1 = (ep.lr1 ? load_scalar(ep.lr1, ep.lr_f32, li) : 1.f) * ep.w_scale;
      pf.l2 = (ep.lr2 ? load_scalar(ep.lr2, ep.lr_f32, li) : 1.f) * ep.w_scale;
    }
  }
  __device__ static __forceinline__ bool skip_store(const Epi&, int) { return false; }
  __device__ static __forceinline__ void epilogue_staged(const Epi&, int, int, int, int, int,
                                                         const float (&v)[3][32], float (&o)[3][32],
                                                         Prefetch& pf) {
    const float l0 = pf.l0, l1 = pf.l1, l2 = pf.l2;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float y0 = v[0][j], y2 = v[1][j], dh = v[2][j];
      const float sg = sigmoidf_fast(y0);
      const float sw = sg * y0;
      o[0][j] = sg * y2 * dh * (1.0f + y0 * (1.0f - sg)) * l0;  // dy0
      o[1][j] = sw * dh * l2;                                     // dy2
      o[2][j] = sw * y2 * l1;                                     // hidden * lr1
    }
  }
};

// ------------------------------------------------------------------------------------------
// row-wise kernels
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xFFFFFFFFu, x, o);
  return x;
}

// Splits the caller's w0, w1, w2 into the internal state: fp32 masters W02 = [w0; w2] ([B,2H,D])
// and W1 ([B,D,H]), their row norms n0, the fp32 compute copies and the bf16 shadows.
// One warp per weight row.
__global__ void prepare_weights_kernel(const void* w0, const void* w1, const void* w2, int w_f32, int B, int H, int D,
                                       float* W02, float* W1, float* W02c, float* W1c, float* n02, float* n1,
                                       bf16* W02b, bf16* W1b) {
  griddep_launch_dependents();
  griddep_wait();
  const int rows_per_b = 2 * H + D;
  const int64_t r = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= static_cast<int64_t>(B) * rows_per_b) return;
  const int lane = threadIdx.x & 31;
  const int b = static_cast<int>(r / rows_per_b), rr = static_cast<int>(r % rows_per_b);
  const void* src;
  int64_t soff, doff;
  int len;
  float *dm, *dc, *dn;
  bf16* db;
  if (rr < 2 * H) {
    len = D;
    src = rr < H ? w0 : w2;
    soff = (static_cast<int64_t>(b) * H + (rr < H ? rr : rr - H)) * D;
    doff = (static_cast<int64_t>(b) * 2 * H + rr) * D;
    dm = W02; dc = W02c; db = W02b;
    dn = n02 + static_cast<int64_t>(b) * 2 * H + rr;
  } else {
    len = H;
    src = w1;
    soff = (static_cast<int64_t>(b) * D + (rr - 2 * H)) * H;
    doff = soff;
    dm = W1; dc = W1c; db = W1b;
    dn = n1 + static_cast<int64_t>(b) * D + (rr - 2 * H);
  }
  float ss = 0.f;
  for (int c = lane; c < len; c += 32) {
    const float x = load_scalar(src, w_f32, soff + c);
    ss += x * x;
    dm[doff + c] = x;
    dc[doff + c] = x;
    db[doff + c] = __float2bfloat16_rn(x);
  }
  ss = warp_sum(ss);
  if (lane == 0) *dn = sqrtf(ss);
}

// beta[u][b] = mean over tokens [s_u, e_u) of momentum[b, t] for up to kMeanBatch update steps per
// launch; grid (batch entries, steps).
constexpr int kMeanBatch = 64;
struct MeanArgs {
  int32_t n;
  int32_t s[kMeanBatch], e[kMeanBatch];
};
__global__ void momentum_mean_kernel(const void* mom, int mom_f32, int64_t bs, const MeanArgs ma, float* beta, int B) {
  griddep_launch_dependents();
  griddep_wait();
  __shared__ float part[32];
  const int b = blockIdx.x, u = blockIdx.y;
  const int s = ma.s[u], e = ma.e[u];
  float acc = 0.f;
  for (int t = s + threadIdx.x; t < e; t += blockDim.x) acc += load_scalar(mom, mom_f32, b * bs + t);
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float x = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0.f;
    x = warp_sum(x);
    if (threadIdx.x == 0) {
      const float m = x / static_cast<float>(e - s);
      beta[static_cast<int64_t>(u) * B + b] = mom_f32 ? m : bf16_round(m);
    }
  }
}

// Newton-Schulz start for up to two groups of gradient matrices.
struct NsPrepGroup {
  const void* src;  // gradient matrices [nmat][R][C], contiguous
  int32_t src_f32;
  int32_t nmat, R, C;
  bf16* x0;           // first iterate
  float* partial;     // [nmat][nparts] partial sums of squares, added in index order
  int32_t nparts;
  float* scale;       // [nmat] out of ns_den_kernel
  uint32_t* done;     // [nmat] completion counters of the fused iteration kernel, cleared here (or nullptr)
};
struct NsPrepArgs {
  NsPrepGroup grp[2];
  int32_t ngroups;
};
constexpr int kNsSlabs = 16;

// Part 1: partial sums of squares of bf16(G).  Grid (matrices of all groups, slabs): CTA (mat,
// slab) reduces rows [slab * rows_per_slab, ...) and writes one float; part 2 adds the partials in
// a fixed order, so the norm does not depend on scheduling.
__global__ void __launch_bounds__(256) ns_sumsq_kernel(const NsPrepArgs args) {
  griddep_launch_dependents();
  griddep_wait();
  __shared__ float part[32];
  int mat = blockIdx.x;
  const int gi = (args.ngroups > 1 && mat >= args.grp[0].nmat) ? 1 : 0;
  if (gi == 1) mat -= args.grp[0].nmat;
  const NsPrepGroup& G = args.grp[gi];
  const int slab = blockIdx.y;
  const int rows_per_slab = (G.R + kNsSlabs - 1) / kNsSlabs;
  const int r0 = slab * rows_per_slab, r1 = min(G.R, r0 + rows_per_slab);
  const int64_t base = static_cast<int64_t>(mat) * G.R * G.C;
  float ss = 0.f;
  for (int r = r0 + (threadIdx.x >> 5); r < r1; r += (blockDim.x >> 5)) {
    const int64_t rb = base + static_cast<int64_t>(r) * G.C;
    for (int c0 = threadIdx.x & 31; c0 < G.C; c0 += 256) {
      float xv[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) xv[i] = (c0 + 32 * i < G.C) ? load_scalar(G.src, G.src_f32, rb + c0 + 32 * i) : 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float x = bf16_round(xv[i]);
        ss += x * x;
      }
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float x = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0.f;
    x = warp_sum(x);
    if (threadIdx.x == 0) G.partial[mat * kNsSlabs + slab] = x;
  }
}

// Scale factors for the folded normalisation: scale[mat] = 1 / (bf16(bf16(||bf16(G)||_F) + 1e-7)).
// One warp per matrix: lane l adds partials l, l + 32, ... in order, then a fixed butterfly adds the
// 32 lane sums, so the result does not depend on scheduling.
__global__ void __launch_bounds__(128) ns_den_kernel(const NsPrepArgs args) {
  griddep_launch_dependents();
  griddep_wait();
  int mat = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int total = args.grp[0].nmat + (args.ngroups > 1 ? args.grp[1].nmat : 0);
  if (mat >= total) return;
  const int gi = (args.ngroups > 1 && mat >= args.grp[0].nmat) ? 1 : 0;
  if (gi == 1) mat -= args.grp[0].nmat;
  const NsPrepGroup& G = args.grp[gi];
  float tot = 0.f;
  for (int i = lane; i < G.nparts; i += 32) tot += G.partial[static_cast<int64_t>(mat) * G.nparts + i];
  tot = warp_sum(tot);
  if (lane == 0) {
    G.scale[mat] = 1.0f / bf16_round(bf16_round(sqrtf(tot)) + 1e-7f);
    if (G.done != nullptr) G.done[mat] = 0;
  }
}

// Part 2: X = bf16(bf16(G) / (bf16(||bf16(G)||_F) + 1e-7)), every operation rounded to bf16 as in
// the reference, in the gradient's own layout.  Grid (matrices of all groups, 64x64 tiles); rows
// whose length allows it move as 16-byte vectors.
__global__ void __launch_bounds__(256) ns_scale_kernel(const NsPrepArgs args) {
  griddep_launch_dependents();
  griddep_wait();
  int mat = blockIdx.x;
  const int gi = (args.ngroups > 1 && mat >= args.grp[0].nmat) ? 1 : 0;
  if (gi == 1) mat -= args.grp[0].nmat;
  const NsPrepGroup& G = args.grp[gi];
  const int tiles_c = (G.C + 63) / 64, tiles_r = (G.R + 63) / 64;
  if (static_cast<int>(blockIdx.y) >= tiles_c * tiles_r) return;
  if (blockIdx.y == 0 && threadIdx.x == 0 && G.done != nullptr) G.done[mat] = 0;
  const int tr = (blockIdx.y / tiles_c) * 64, tcx = (blockIdx.y % tiles_c) * 64;
  __shared__ float parts[512];
  __shared__ float den_s;
  for (int i = threadIdx.x; i < G.nparts; i += blockDim.x) parts[i] = G.partial[static_cast<int64_t>(mat) * G.nparts + i];
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int i = 0; i < G.nparts; ++i) tot += parts[i];  // same order in every CTA
    den_s = bf16_round(bf16_round(sqrtf(tot)) + 1e-7f);
  }
  __syncthreads();
  const float den = den_s;
  const int64_t base = static_cast<int64_t>(mat) * G.R * G.C;
  bf16* xo = G.x0 + base;
  if ((G.C % 4) == 0) {
    const int lx = (threadIdx.x & 15) * 4, ly = threadIdx.x >> 4;  // 16 x 16 threads, 4 columns each
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = tr + ly + 16 * i, c = tcx + lx;
      if (r >= G.R || c >= G.C) continue;
      const int64_t off = base + static_cast<int64_t>(r) * G.C + c;
      float x0, x1, x2, x3;
      if (G.src_f32) {
        const float4 t = *reinterpret_cast<const float4*>(static_cast<const float*>(G.src) + off);
        x0 = t.x; x1 = t.y; x2 = t.z; x3 = t.w;
      } else {
        const uint2 t = *reinterpret_cast<const uint2*>(static_cast<const bf16*>(G.src) + off);
        x0 = __uint_as_float(t.x << 16); x1 = __uint_as_float(t.x & 0xFFFF0000u);
        x2 = __uint_as_float(t.y << 16); x3 = __uint_as_float(t.y & 0xFFFF0000u);
      }
      *reinterpret_cast<uint2*>(xo + static_cast<int64_t>(r) * G.C + c) =
          make_uint2(pack_bf16x2(bf16_round(x0) / den, bf16_round(x1) / den),
                     pack_bf16x2(bf16_round(x2) / den, bf16_round(x3) / den));
    }
    return;
  }
  const int lx = threadIdx.x & 63, ly = threadIdx.x >> 6;  // 64 x 4
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int r = tr + ly + 4 * i, c = tcx + lx;
    if (r < G.R && c < G.C) {
      const int64_t off = static_cast<int64_t>(r) * G.C + c;
      xo[off] = __float2bfloat16_rn(bf16_round(load_scalar(G.src, G.src_f32, base + off)) / den);
    }
  }
}

struct RenormArgs {
  float* master;     // [B][R][C] fp32, in/out
  const float* master_in;  // nullptr, or where the current master is read from (`master` is then written only)
  float* compute;    // [B][R][C] fp32 out (may be nullptr): the weights the next step computes with
  bf16* shadow;      // [B][R][C] bf16 out
  const float* n0;   // [B][R]
  const float* g;    // [B][R][C] fp32 gradient (after momentum)
  const bf16* x;     // Newton-Schulz result in the weight's own orientation, or nullptr (update = g)
  int64_t x_bs;      // stride of x between batch entries
  int32_t B, R, C;
  int32_t mode;      // LACT_RENORM_*
  int32_t prenorm, prenorm_bf16, quirk;
};

constexpr int kRenormMaxCols = 1024;

// One weight row: w_new = (quirk ? g : master) + update; normalise.  Lane l owns columns
// 4l .. 4l+3 of every 128-column group (NV groups, row kept in registers).  The Newton-Schulz
// result is read with L2-only loads (another SM may have written it earlier in the same kernel).
template <int NV>
__device__ __forceinline__ void renorm_row(const RenormArgs& a, int64_t row, int lane) {
  const int b = static_cast<int>(row / a.R), r = static_cast<int>(row % a.R);
  const int64_t off = row * a.C;
  const bf16* xr = a.x != nullptr ? a.x + b * a.x_bs + static_cast<int64_t>(r) * a.C : nullptr;
  const bool use_g_base = a.quirk && xr != nullptr;
  const float n0 = a.n0[row];
  float4 w[NV];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = 4 * lane + 128 * i;
    w[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < a.C) {
      float4 upd;
      if (xr != nullptr) {
        const uint2 u = __ldcg(reinterpret_cast<const uint2*>(xr + c));
        upd = make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xFFFF0000u),
                          __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xFFFF0000u));
      } else {
        upd = *reinterpret_cast<const float4*>(a.g + off + c);
      }
      const float4 base = use_g_base ? *reinterpret_cast<const float4*>(a.g + off + c)
                                     : *reinterpret_cast<const float4*>((a.master_in != nullptr ? a.master_in : a.master) + off + c);
      w[i] = make_float4(base.x + upd.x, base.y + upd.y, base.z + upd.z, base.w + upd.w);
      ss += w[i].x * w[i].x + w[i].y * w[i].y + w[i].z * w[i].z + w[i].w * w[i].w;
    }
  }
  ss = warp_sum(ss);
  const float den = sqrtf(ss) + 1e-5f;
  const float rstd = 1.0f / sqrtf(ss + 1e-5f);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = 4 * lane + 128 * i;
    if (c < a.C) {
      float y[4] = {w[i].x, w[i].y, w[i].z, w[i].w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (a.mode == 1) y[q] = y[q] / den * n0;
        else if (a.mode == 2) y[q] = y[q] * rstd * n0;
        if (a.prenorm && a.prenorm_bf16) y[q] = bf16_round(y[q]);
      }
      const float4 yv = make_float4(y[0], y[1], y[2], y[3]);
      *reinterpret_cast<float4*>(a.master + off + c) = a.prenorm ? w[i] : yv;
      if (a.compute != nullptr) *reinterpret_cast<float4*>(a.compute + off + c) = yv;
      *reinterpret_cast<uint2*>(a.shadow + off + c) = make_uint2(pack_bf16x2(y[0], y[1]), pack_bf16x2(y[2], y[3]));
    }
  }
}

// Both weight arrays in one launch; one warp per row; NV = float4 per lane (row length <= 128 * NV).  The register
// footprint follows the row length, so short rows run at higher occupancy.
template <int NV>
__global__ void __launch_bounds__(256, NV <= 3 ? 6 : (NV <= 4 ? 4 : 2)) add_renorm_kernel(const RenormArgs a0, const RenormArgs a1) {
  griddep_launch_dependents();
  griddep_wait();
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t rows0 = static_cast<int64_t>(a0.B) * a0.R, rows1 = static_cast<int64_t>(a1.B) * a1.R;
  if (row < rows0) renorm_row<NV>(a0, row, threadIdx.x & 31);
  else if (row < rows0 + rows1) renorm_row<NV>(a1, row - rows0, threadIdx.x & 31);
}

// ------------------------------------------------------------------------------------------
// pointwise kernels of the training backward (planes are [B*N rows][H or 2H columns], bf16)
// ------------------------------------------------------------------------------------------
struct PlaneArgs {
  const bf16* y02;    // [rows][2H]: y0 | y2
  const bf16* dh;     // [rows][H]
  const bf16* g_dy02; // [rows][2H] upstream grads of dy0 | dy2 (second-order kernel only)
  const bf16* g_hid;  // [rows][H]  upstream grad of hidden*lr1 (second-order kernel only)
  const void *lr0, *lr1, *lr2;  // [rows] or nullptr (= 1)
  int32_t lr_f32;
  float w_scale;
  bf16* dy02;   // out [rows][2H]: dy0*lr0 | dy2*lr2
  bf16* hid;    // out [rows][H]: hidden*lr1
  bf16* g_y02;  // out [rows][2H] (second-order only)
  bf16* g_dh;   // out [rows][H]  (second-order only)
  float *g_lr0, *g_lr1, *g_lr2;  // out [rows] (second-order only)
  int64_t rows;
  int32_t H;
};

// eight consecutive bf16 values as floats / back (16-byte accesses; column counts here are multiples of 8)
__device__ __forceinline__ void load8_bf16(const bf16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ void store8_bf16(bf16* p, const float (&v)[8]) {
  uint4 u;
  u.x = pack_bf16x2(v[0], v[1]); u.y = pack_bf16x2(v[2], v[3]);
  u.z = pack_bf16x2(v[4], v[5]); u.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// First-order planes: hidden*lr1, dy0*lr0, dy2*lr2 from (bf16-rounded) y0, y2, dh.  Used by the
// backward of apply (lr = 1; lact_swiglu_ffn.py:46-76).  One warp per token row.
__global__ void __launch_bounds__(256) swiglu_bwd_planes_kernel(const PlaneArgs a) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= a.rows) return;
  const int lane = threadIdx.x & 31;
  const float l0 = (a.lr0 ? load_scalar(a.lr0, a.lr_f32, row) : 1.f) * a.w_scale;
  const float l1 = (a.lr1 ? load_scalar(a.lr1, a.lr_f32, row) : 1.f) * a.w_scale;
  const float l2 = (a.lr2 ? load_scalar(a.lr2, a.lr_f32, row) : 1.f) * a.w_scale;
  const int H = a.H;
  for (int c = lane * 8; c < H; c += 256) {
    float y0[8], y2[8], dh[8], oh[8], o0[8], o2[8];
    load8_bf16(a.y02 + row * 2 * H + c, y0);
    load8_bf16(a.y02 + row * 2 * H + H + c, y2);
    load8_bf16(a.dh + row * H + c, dh);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = sigmoidf_fast(y0[j]), sw = sg * y0[j];
      oh[j] = sw * y2[j] * l1;
      o0[j] = sg * y2[j] * dh[j] * (1.0f + y0[j] * (1.0f - sg)) * l0;
      o2[j] = sw * dh[j] * l2;
    }
    store8_bf16(a.hid + row * H + c, oh);
    store8_bf16(a.dy02 + row * 2 * H + c, o0);
    store8_bf16(a.dy02 + row * 2 * H + H + c, o2);
  }
}

// Second-order pointwise stage of the fast-weight-gradient backward
// (lact_llm/lact_model/lact_triton_kernels/lact_fw_grad.py:178-260): with A = d silu / dy0,
//   g_y0 = g_hid*A*y2*l1 + g_dy0*A'*y2*dh*l0 + g_dy2*A*dh*l2,   g_y2 = g_hid*sw*l1 + g_dy0*A*dh*l0,
//   g_dh = g_dy0*A*y2*l0 + g_dy2*sw*l2,   g_lr = row sums (deterministic: one warp per row).
__global__ void __launch_bounds__(256, 4) fw_grad_bwd_pointwise_kernel(const PlaneArgs a) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= a.rows) return;
  const int lane = threadIdx.x & 31;
  const float l0 = load_scalar(a.lr0, a.lr_f32, row) * a.w_scale;
  const float l1 = load_scalar(a.lr1, a.lr_f32, row) * a.w_scale;
  const float l2 = load_scalar(a.lr2, a.lr_f32, row) * a.w_scale;
  const int H = a.H;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f;
  for (int c = lane * 8; c < H; c += 256) {
    float y0[8], y2[8], dh[8], gd0[8], gd2[8], gh[8];
    load8_bf16(a.y02 + row * 2 * H + c, y0);
    load8_bf16(a.y02 + row * 2 * H + H + c, y2);
    load8_bf16(a.dh + row * H + c, dh);
    load8_bf16(a.g_dy02 + row * 2 * H + c, gd0);
    load8_bf16(a.g_dy02 + row * 2 * H + H + c, gd2);
    load8_bf16(a.g_hid + row * H + c, gh);
    float gy0[8], gy2[8], gdh[8], oh[8], o0[8], o2[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = sigmoidf_fast(y0[j]), sw = sg * y0[j];
      const float A = sg * (1.0f + y0[j] * (1.0f - sg));
      const float Ap = sg * (1.0f - sg) * (2.0f + y0[j] * (1.0f - 2.0f * sg));
      gy0[j] = gh[j] * A * y2[j] * l1 + gd0[j] * Ap * y2[j] * dh[j] * l0 + gd2[j] * A * dh[j] * l2;
      gy2[j] = gh[j] * sw * l1 + gd0[j] * A * dh[j] * l0;
      gdh[j] = gd0[j] * A * y2[j] * l0 + gd2[j] * sw * l2;
      oh[j] = sw * y2[j] * l1;
      o0[j] = A * y2[j] * dh[j] * l0;
      o2[j] = sw * dh[j] * l2;
      s0 += gd0[j] * A * y2[j] * dh[j];
      s1 += gh[j] * sw * y2[j];
      s2 += gd2[j] * sw * dh[j];
    }
    store8_bf16(a.g_y02 + row * 2 * H + c, gy0);
    store8_bf16(a.g_y02 + row * 2 * H + H + c, gy2);
    store8_bf16(a.g_dh + row * H + c, gdh);
    store8_bf16(a.hid + row * H + c, oh);
    store8_bf16(a.dy02 + row * 2 * H + c, o0);
    store8_bf16(a.dy02 + row * 2 * H + H + c, o2);
  }
  s0 = warp_sum(s0); s1 = warp_sum(s1); s2 = warp_sum(s2);
  if (lane == 0) {
    a.g_lr0[row] = s0 * a.w_scale;
    a.g_lr1[row] = s1 * a.w_scale;
    a.g_lr2[row] = s2 * a.w_scale;
  }
}

// Backward of w -> y = renorm(w) for rows of w = base + upd (recomputed here):
//   mode 1 (eps outside): y = w / (r + eps) * n0;   mode 2: y = w * rsqrt(r^2 + eps) * n0;   mode 0: y = w.
// Writes dw (fp32) and ADDS <dy, w> * scale into dn0[row]; one warp per row.
struct RenormBwdArgs {
  const float* base;  // [rows][C]
  const void* upd;    // [rows][C] fp32 or bf16
  int32_t upd_f32;
  const float* n0;    // [rows]
  const float* dy;    // [rows][C]
  float* dw;          // [rows][C] out
  bf16* dw_b;         // optional bf16 copy of dw (operand of the Newton-Schulz backward), or nullptr
  float* dn0;         // [rows] accumulated
  int64_t rows;
  int32_t C, mode;
};
__global__ void __launch_bounds__(256) renorm_bwd_kernel(const RenormBwdArgs a) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= a.rows) return;
  const int lane = threadIdx.x & 31;
  const int64_t off = row * a.C;
  float ss = 0.f, dot = 0.f;
  for (int c = lane; c < a.C; c += 32) {
    const float w = a.base[off + c] + load_scalar(a.upd, a.upd_f32, off + c);
    ss += w * w;
    dot += w * a.dy[off + c];
  }
  ss = warp_sum(ss);
  dot = warp_sum(dot);
  const float n0 = a.n0[row];
  float s, k;  // dw = s * dy - k * w ; dn0 += dot * t
  float t;
  if (a.mode == 1) {
    const float r = sqrtf(ss), den = r + 1e-5f;
    s = n0 / den;
    k = r > 0.f ? n0 * dot / (den * den * r) : 0.f;
    t = 1.0f / den;
  } else if (a.mode == 2) {
    const float rs = 1.0f / sqrtf(ss + 1e-5f);
    s = n0 * rs;
    k = n0 * dot * rs * rs * rs;
    t = rs;
  } else {
    s = 1.f; k = 0.f; t = 0.f;
  }
  for (int c = lane; c < a.C; c += 32) {
    const float w = a.base[off + c] + load_scalar(a.upd, a.upd_f32, off + c);
    const float d = s * a.dy[off + c] - k * w;
    a.dw[off + c] = d;
    if (a.dw_b != nullptr) a.dw_b[off + c] = __float2bfloat16_rn(d);
  }
  if (lane == 0 && a.dn0 != nullptr) a.dn0[row] += dot * t;
}

// block-wide sum of two values (blockDim.x a multiple of 32, at most 1024); every thread gets the totals
__device__ __forceinline__ void block_sum2(float& a, float& b, float* scratch /* [66] */) {
  a = warp_sum(a);
  b = warp_sum(b);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (l == 0) { scratch[w] = a; scratch[32 + w] = b; }
  __syncthreads();
  if (w == 0) {
    float x = l < nw ? scratch[l] : 0.f, y = l < nw ? scratch[32 + l] : 0.f;
    x = warp_sum(x);
    y = warp_sum(y);
    if (l == 0) { scratch[64] = x; scratch[65] = y; }
  }
  __syncthreads();
  a = scratch[64];
  b = scratch[65];
}

// Backward of the Frobenius normalisation in front of Newton-Schulz, X0 = bf16(G) / den with nrm = bf16(||bf16(G)||),
// den = bf16(nrm + 1e-7):  dG = dX0 / den - bf16(G) <dX0, bf16(G)> / (den^2 nrm), written in place over dX0.
// Two launches over (matrices x slices) blocks: partial sums, then the rewrite (`n` elements per matrix).
constexpr int kNormBwdSlices = 16;
// four consecutive gradient values, fp32 or bf16 storage
__device__ __forceinline__ float4 load4_f32_or_bf16(const void* p, int is_bf16, int64_t i) {
  if (!is_bf16) return *reinterpret_cast<const float4*>(static_cast<const float*>(p) + i);
  const uint2 u = *reinterpret_cast<const uint2*>(static_cast<const bf16*>(p) + i);
  return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xFFFF0000u), __uint_as_float(u.y << 16),
                     __uint_as_float(u.y & 0xFFFF0000u));
}
// part 1: per (matrix, slice) partial sums of bf16(G)^2 and dX0 * bf16(G) into part[(mat * slices + s) * 2 + {0, 1}]
__global__ void __launch_bounds__(512) ns_norm_bwd_partial_kernel(const float* g, const void* dx0, int dx_bf16, float* part,
                                                                  int64_t n) {
  __shared__ float scratch[66];
  const float* G = g + static_cast<int64_t>(blockIdx.x) * n;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * n;
  const int64_t per = ((n / 4 + gridDim.y - 1) / gridDim.y) * 4;
  const int64_t lo = static_cast<int64_t>(blockIdx.y) * per, hi = lo + per < n ? lo + per : n;
  float ss = 0.f, dot = 0.f;
  for (int64_t i = lo + threadIdx.x * 4; i < hi; i += blockDim.x * 4) {
    const float4 gv = *reinterpret_cast<const float4*>(G + i), dv = load4_f32_or_bf16(dx0, dx_bf16, base + i);
    const float a = bf16_round(gv.x), b = bf16_round(gv.y), c = bf16_round(gv.z), d = bf16_round(gv.w);
    ss += a * a + b * b + c * c + d * d;
    dot += a * dv.x + b * dv.y + c * dv.z + d * dv.w;
  }
  block_sum2(ss, dot, scratch);
  if (threadIdx.x == 0) {
    part[(static_cast<int64_t>(blockIdx.x) * gridDim.y + blockIdx.y) * 2] = ss;
    part[(static_cast<int64_t>(blockIdx.x) * gridDim.y + blockIdx.y) * 2 + 1] = dot;
  }
}
// part 2: the partials are added in slice order (same result in every block), then the slice of dG is written
// (`dg` may be `dx0` itself when that is fp32)
__global__ void __launch_bounds__(512) ns_norm_bwd_apply_kernel(const float* g, const void* dx0, int dx_bf16, float* dg,
                                                                const float* part, int64_t n) {
  const float* G = g + static_cast<int64_t>(blockIdx.x) * n;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * n;
  float ss = 0.f, dot = 0.f;
  for (int s = 0; s < static_cast<int>(gridDim.y); ++s) {
    ss += part[(static_cast<int64_t>(blockIdx.x) * gridDim.y + s) * 2];
    dot += part[(static_cast<int64_t>(blockIdx.x) * gridDim.y + s) * 2 + 1];
  }
  const float nrm = bf16_round(sqrtf(ss)), den = bf16_round(nrm + 1e-7f);
  const float inv = 1.0f / den, coef = dot / (den * den * fmaxf(nrm, 1e-30f));
  const int64_t per = ((n / 4 + gridDim.y - 1) / gridDim.y) * 4;
  const int64_t lo = static_cast<int64_t>(blockIdx.y) * per, hi = lo + per < n ? lo + per : n;
  for (int64_t i = lo + threadIdx.x * 4; i < hi; i += blockDim.x * 4) {
    const float4 gv = *reinterpret_cast<const float4*>(G + i);
    float4 dv = load4_f32_or_bf16(dx0, dx_bf16, base + i);
    dv.x = dv.x * inv - bf16_round(gv.x) * coef;
    dv.y = dv.y * inv - bf16_round(gv.y) * coef;
    dv.z = dv.z * inv - bf16_round(gv.z) * coef;
    dv.w = dv.w * inv - bf16_round(gv.w) * coef;
    *reinterpret_cast<float4*>(dg + base + i) = dv;
  }
}

// Momentum step of the reverse sweep for one batch entry per block, over the two gradient arrays (n0 and n1 elements
// per entry):  dG += carry (the gradient that reaches this update's momentum state from the NEXT update, if any);
// dbeta[b] = <dG, Mprev> (Mprev: momentum state before this update, or nullptr at the first update);
// carry <- dG * beta[b] (what reaches the previous update's state); and a bf16 copy of dG for the contractions of
// the fast-weight-gradient backward.  beta == nullptr: no momentum (only dG += 0 and the bf16 copy).
struct MomentumBwdArgs {
  float* dg[2];          // in/out
  float* carry[2];       // in/out, or nullptr when there is no momentum
  const float* mprev[2]; // or nullptr
  bf16* dgb[2];          // out
  const float* beta;     // [B] or nullptr
  float* dbeta;          // [B] out (written, not accumulated), or nullptr
  int64_t n[2];
  int32_t add_carry;     // 0 at the last update of the program (nothing arrives from a later one)
};
__global__ void __launch_bounds__(1024) momentum_bwd_kernel(const MomentumBwdArgs a) {
  // grid (batch entries, slices): block (b, s) owns the s-th of gridDim.y equal slices of both arrays of entry b and
  // leaves its share of <dG, Mprev> in dbeta[b * gridDim.y + s] (the host adds the slices)
  __shared__ float scratch[66];
  const int b = blockIdx.x;
  const float bt = a.beta != nullptr ? a.beta[b] : 0.f;
  float dot = 0.f, unused = 0.f;
#pragma unroll
  for (int w = 0; w < 2; ++w) {
    const int64_t off = static_cast<int64_t>(b) * a.n[w];
    const int64_t per = ((a.n[w] / 4 + gridDim.y - 1) / gridDim.y) * 4;
    const int64_t lo = static_cast<int64_t>(blockIdx.y) * per, hi = lo + per < a.n[w] ? lo + per : a.n[w];
    for (int64_t i = lo + threadIdx.x * 4; i < hi; i += blockDim.x * 4) {
      float4 d = *reinterpret_cast<const float4*>(a.dg[w] + off + i);
      if (a.carry[w] != nullptr && a.add_carry) {
        const float4 c = *reinterpret_cast<const float4*>(a.carry[w] + off + i);
        d.x += c.x; d.y += c.y; d.z += c.z; d.w += c.w;
        *reinterpret_cast<float4*>(a.dg[w] + off + i) = d;
      }
      if (a.mprev[w] != nullptr) {
        const float4 m = *reinterpret_cast<const float4*>(a.mprev[w] + off + i);
        dot += d.x * m.x + d.y * m.y + d.z * m.z + d.w * m.w;
      }
      if (a.carry[w] != nullptr)
        *reinterpret_cast<float4*>(a.carry[w] + off + i) = make_float4(d.x * bt, d.y * bt, d.z * bt, d.w * bt);
      *reinterpret_cast<uint2*>(a.dgb[w] + off + i) = make_uint2(pack_bf16x2(d.x, d.y), pack_bf16x2(d.z, d.w));
    }
  }
  block_sum2(dot, unused, scratch);
  if (threadIdx.x == 0 && a.dbeta != nullptr) a.dbeta[b * gridDim.y + blockIdx.y] = dot;
}

// ------------------------------------------------------------------------------------------
// fp32 mode (parity path for fp32 activations): plain FFMA kernels, no tensor cores.
// tcgen05 has no fp32 x fp32 MMA; this path exists for accuracy (max relative error ~1e-6 when
// Muon is off), not for throughput.
// ------------------------------------------------------------------------------------------
// c[b][m][n] = sum_k A(b, m, k) * B(b, n, k) (+ beta[b] * c[b][m][n] when accumulating; beta = 1
// without a beta vector); A stored [M][K] (a_t = 0) or [K][M] (a_t = 1), B stored [N][K] (b_t = 0)
// or [K][N] (b_t = 1); all contiguous.  64 x 64 tile, 256 threads, 4 x 4 per thread.
__global__ void __launch_bounds__(256) sgemm_f32_kernel(const float* A, int a_t, const float* B, int b_t, float* C,
                                                        int accumulate, const float* beta, int M, int N, int K) {
  __shared__ float As[16][65];
  __shared__ float Bs[16][65];
  const int b = blockIdx.z;
  A += static_cast<int64_t>(b) * M * K;
  B += static_cast<int64_t>(b) * N * K;
  C += static_cast<int64_t>(b) * M * N;
  const float cb = beta != nullptr ? beta[b] : 1.f;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int i = threadIdx.x; i < 16 * 64; i += 256) {
      const int kk = a_t ? i / 64 : i % 16, mm = a_t ? i % 64 : i / 16;
      const int gm = m0 + mm, gk = k0 + kk;
      As[kk][mm] = (gm < M && gk < K) ? (a_t ? A[static_cast<int64_t>(gk) * M + gm] : A[static_cast<int64_t>(gm) * K + gk]) : 0.f;
      const int kb = b_t ? i / 64 : i % 16, nn = b_t ? i % 64 : i / 16;
      const int gn = n0 + nn, gkb = k0 + kb;
      Bs[kb][nn] = (gn < N && gkb < K) ? (b_t ? B[static_cast<int64_t>(gkb) * N + gn] : B[static_cast<int64_t>(gn) * K + gkb]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float a[4], bb[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = As[kk][ty * 4 + i]; bb[i] = Bs[kk][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gm = m0 + ty * 4 + i, gn = n0 + tx * 4 + j;
      if (gm < M && gn < N) {
        float* o = C + static_cast<int64_t>(gm) * N + gn;
        *o = accumulate ? fmaf(*o, cb, acc[i][j]) : acc[i][j];
      }
    }
}

// fp32 planes: hidden = silu(y0) * y2 (lr pointers null and dh null), or the lr-weighted gradient
// planes (hidden*lr1, dy0*lr0, dy2*lr2).  Exact expf / division.  One warp per token row.
__global__ void __launch_bounds__(256) swiglu_planes_f32_kernel(const float* y02, const float* dh, const void* lr0,
                                                                const void* lr1, const void* lr2, int lr_f32,
                                                                float w_scale, float* dy02, float* hid, int64_t rows,
                                                                int H) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const float l0 = (lr0 ? load_scalar(lr0, lr_f32, row) : 1.f) * w_scale;
  const float l1 = (lr1 ? load_scalar(lr1, lr_f32, row) : 1.f) * w_scale;
  const float l2 = (lr2 ? load_scalar(lr2, lr_f32, row) : 1.f) * w_scale;
  for (int c = lane; c < H; c += 32) {
    const float y0 = y02[row * 2 * H + c], y2 = y02[row * 2 * H + H + c];
    const float sg = 1.0f / (1.0f + expf(-y0)), sw = sg * y0;
    hid[row * H + c] = sw * y2 * l1;
    if (dh != nullptr) {
      const float d = dh[row * H + c];
      dy02[row * 2 * H + c] = sg * y2 * d * (1.0f + y0 * (1.0f - sg)) * l0;
      dy02[row * 2 * H + H + c] = sw * d * l2;
    }
  }
}

// y = (x + x_add) * rsqrt(sum (x + x_add)^2 + eps) * scale[row]; one warp per row.
__global__ void l2_norm_add_kernel(const void* x, int x_f32, const void* xa, int xa_f32, const float* scale, void* y,
                                   int y_f32, int64_t rows, int D, float eps) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int64_t off = row * D;
  float ss = 0.f;
  for (int c = lane; c < D; c += 32) {
    const float w = load_scalar(x, x_f32, off + c) + load_scalar(xa, xa_f32, off + c);
    ss += w * w;
  }
  ss = warp_sum(ss);
  const float rstd = 1.0f / sqrtf(ss + eps);
  const float sc = scale[row];
  for (int c = lane; c < D; c += 32) {
    const float w = load_scalar(x, x_f32, off + c) + load_scalar(xa, xa_f32, off + c);
    const float v = w * rstd * sc;
    if (y_f32) reinterpret_cast<float*>(y)[off + c] = v;
    else reinterpret_cast<bf16*>(y)[off + c] = __float2bfloat16_rn(v);
  }
}

// m' = dx + mu[b]*m; x' = x + m'; y = bf16(x' / sqrt(sum x'^2 + eps) * scale[row]); one warp per row.
__global__ void prenorm_momentum_kernel(const float* x, const bf16* dx, const float* m, const float* mu,
                                        const float* scale, float* xo, float* mo, bf16* yo, int64_t rows, int T, int D,
                                        float eps) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int64_t off = row * D;
  const float mub = mu[row / T];
  float ss = 0.f;
  for (int c = lane; c < D; c += 32) {
    const float mn = __bfloat162float(dx[off + c]) + m[off + c] * mub;
    const float xn = x[off + c] + mn;
    mo[off + c] = mn;
    xo[off + c] = xn;
    ss += xn * xn;
  }
  ss = warp_sum(ss);
  const float den = sqrtf(ss + eps);
  const float sc = scale[row];
  __syncwarp();
  for (int c = lane; c < D; c += 32) yo[off + c] = __float2bfloat16_rn(xo[off + c] / den * sc);
}

// ------------------------------------------------------------------------------------------
// layer prologue: fast-weight inputs from the projected activations
// ------------------------------------------------------------------------------------------
struct PrologueArgs {
  const bf16* x[3];      // q, k, v projections: [b][s][n_h * d], row stride ld[i], batch stride bs[i] (elements)
  int64_t ld[3], bs[3];
  bf16* out[3];          // [(b n_h)][s][d] contiguous
  int32_t b, s, n_h, d;
  int32_t silu[3];       // apply SiLU to q / k / v
  int32_t l2norm[3];     // per-head l2 norm (q and k in the reference layer)
  // rotary position embedding on q and k after the l2 norm (layer_lact_swiglu.py:417-446), or rope_hd = 0 for none.
  // The merged feature axis (n_h * d) is cut into attention heads of rope_hd features (a power of two, 32..1024,
  // dividing d); within each, feature j < rope_hd / 2 pairs with j + rope_hd / 2 (non-interleaved layout):
  //   y[j] = x[j] cos[p][j] - x[j + hd/2] sin[p][j],   y[j + hd/2] = x[j] sin[p][j] + x[j + hd/2] cos[p][j]
  // in fp32 from the bf16 inputs, rounded once (the arithmetic of the rotary kernel the reference calls).
  const bf16 *cos, *sin;  // [positions][rope_hd / 2], bf16 (the reference caches them in the activations' dtype)
  int32_t rope_hd, pos0;  // position of token 0
  const int32_t* seq_start;  // optional [s] (b = 1): packed sequences, token t sits at position pos0 + t - seq_start[t]
};

// One warp per (batch, token, head): y = silu(x) rounded to bf16, then y / (bf16(||y||) + 1e-5) with the norm, the
// sum and the quotient rounded to bf16 one after the other, as the reference's bf16 eager arithmetic does
// (layer_lact_swiglu.py:404-414, ttt_operation.py:19-26); rows are written head-major, so the head split costs no
// extra pass.  d <= 1024, a multiple of 8.
// NCH = ceil(d / 256): 16-byte chunks per lane (the register footprint, hence the occupancy, follows the head size).
// ROPE: the rotary variant (more registers: compiled separately so that the plain pass keeps its occupancy).
template <int NCH, bool ROPE>
__global__ void __launch_bounds__(256, ROPE ? (NCH <= 2 ? 4 : 2) : (NCH <= 2 ? 8 : 4)) qkv_prologue_kernel(const PrologueArgs a) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t rows = static_cast<int64_t>(a.b) * a.s * a.n_h;
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int h = static_cast<int>(row % a.n_h);
  const int64_t bs_idx = row / a.n_h;
  const int tok = static_cast<int>(bs_idx % a.s), bi = static_cast<int>(bs_idx / a.s);
  const int64_t out_off = ((static_cast<int64_t>(bi) * a.n_h + h) * a.s + tok) * a.d;
#pragma unroll
  for (int t = 0; t < 3; ++t) {
    const bf16* src = a.x[t] + bi * a.bs[t] + tok * a.ld[t] + static_cast<int64_t>(h) * a.d;
    float y[NCH][8];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int col = (c * 32 + lane) * 8;
#pragma unroll
      for (int i = 0; i < 8; ++i) y[c][i] = 0.f;
      if (col < a.d) {
        const uint4 u = *reinterpret_cast<const uint4*>(src + col);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float lo = __uint_as_float(w[i] << 16), hi = __uint_as_float(w[i] & 0xFFFF0000u);
          if (a.silu[t]) {
            // fast exponential and divide: their fp32 error (a few ulp) moves the bf16 rounding of about one value
            // in ten thousand by one ulp
            lo = bf16_round(__fdividef(lo, 1.f + __expf(-lo)));
            hi = bf16_round(__fdividef(hi, 1.f + __expf(-hi)));
          }
          y[c][2 * i] = lo;
          y[c][2 * i + 1] = hi;
          ss += lo * lo + hi * hi;
        }
      }
    }
    float inv_den = 1.f;
    if (a.l2norm[t]) {
      ss = warp_sum(ss);
      inv_den = 1.f / bf16_round(bf16_round(sqrtf(ss)) + 1e-5f);
    }
    if (ROPE && t < 2) {
      // the normalised row, rounded to bf16 as the reference's l2_norm returns it, is rotated in registers: the
      // partner of a feature sits rope_hd / 2 columns away, i.e. rope_hd / 16 lanes away (same 16-byte chunk index)
      // or, from rope_hd = 512 up, rope_hd / 512 chunks away in the same lane
      const int half = a.rope_hd >> 1;
      const int64_t trow = static_cast<int64_t>(a.pos0 + tok - (a.seq_start != nullptr ? a.seq_start[tok] : 0)) * half;
#pragma unroll
      for (int c = 0; c < NCH; ++c)
#pragma unroll
        for (int i = 0; i < 8; ++i) y[c][i] = bf16_round(y[c][i] * inv_den);
      float other[NCH][8];
#pragma unroll
      for (int c = 0; c < NCH; ++c)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (half < 256) other[c][i] = __shfl_xor_sync(0xFFFFFFFFu, y[c][i], half >> 3);
          else other[c][i] = y[(c ^ (half >> 8)) < NCH ? (c ^ (half >> 8)) : c][i];
        }
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        const int col = (c * 32 + lane) * 8;
        if (col < a.d) {
          const int j = (static_cast<int>(h) * a.d + col) % a.rope_hd;  // column inside its attention head
          const bool first = j < half;
          const uint4 cu = *reinterpret_cast<const uint4*>(a.cos + trow + (first ? j : j - half));
          const uint4 su = *reinterpret_cast<const uint4*>(a.sin + trow + (first ? j : j - half));
          const uint32_t cw[4] = {cu.x, cu.y, cu.z, cu.w}, sw[4] = {su.x, su.y, su.z, su.w};
          uint4 u;
          uint32_t* w = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float c0 = __uint_as_float(cw[i] << 16), c1 = __uint_as_float(cw[i] & 0xFFFF0000u);
            const float s0 = __uint_as_float(sw[i] << 16), s1 = __uint_as_float(sw[i] & 0xFFFF0000u);
            const float x0 = y[c][2 * i], x1 = y[c][2 * i + 1], p0 = other[c][2 * i], p1 = other[c][2 * i + 1];
            // first half: x cos - partner sin; second half: partner sin + x cos
            const float r0 = first ? __fsub_rn(__fmul_rn(x0, c0), __fmul_rn(p0, s0)) : __fadd_rn(__fmul_rn(p0, s0), __fmul_rn(x0, c0));
            const float r1 = first ? __fsub_rn(__fmul_rn(x1, c1), __fmul_rn(p1, s1)) : __fadd_rn(__fmul_rn(p1, s1), __fmul_rn(x1, c1));
            w[i] = pack_bf16x2(r0, r1);
          }
          *reinterpret_cast<uint4*>(a.out[t] + out_off + col) = u;
        }
      }
      continue;
    }
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int col = (c * 32 + lane) * 8;
      if (col < a.d) {
        uint4 u;
        uint32_t* w = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          w[i] = pack_bf16x2(y[c][2 * i] * inv_den, y[c][2 * i + 1] * inv_den);
        }
        *reinterpret_cast<uint4*>(a.out[t] + out_off + col) = u;
      }
    }
  }
}

// Learning rates and momentum of the layer: lr = softplus(proj + base_lr_inv) in fp32 (torch's threshold of 20),
// proj [b][s][n_h * 3] -> three [(b n_h)][s] fp32 vectors; momentum = float(round_to_input_dtype(sigmoid(logit))),
// logits [b][s][n_h] -> [(b n_h)][s] (layer_lact_swiglu.py:463-480, 245-249).  One thread per (batch, token, head).
struct LrPrologueArgs {
  const void* proj;    // bf16 or fp32
  const void* logits;  // bf16 or fp32, or nullptr
  int32_t proj_f32, logits_f32;
  int64_t proj_ld, logits_ld;  // row strides in elements (rows = b * s)
  float base_lr_inv;
  float* lr[3];
  float* mom;          // or nullptr
  int32_t b, s, n_h;
};
__global__ void __launch_bounds__(256) lr_prologue_kernel(const LrPrologueArgs a) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t total = static_cast<int64_t>(a.b) * a.s * a.n_h;
  if (i >= total) return;
  // consecutive threads walk the tokens of one (batch, head): coalesced stores, strided (small) loads
  const int tok = static_cast<int>(i % a.s);
  const int64_t bh = i / a.s;
  const int h = static_cast<int>(bh % a.n_h), bi = static_cast<int>(bh / a.n_h);
  const int64_t row = static_cast<int64_t>(bi) * a.s + tok;
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    const float x = load_scalar(a.proj, a.proj_f32, row * a.proj_ld + h * 3 + j) + a.base_lr_inv;
    a.lr[j][i] = x > 20.f ? x : log1pf(expf(x));
  }
  if (a.mom != nullptr) {
    const float x = load_scalar(a.logits, a.logits_f32, row * a.logits_ld + h);
    const float sg = 1.f / (1.f + expf(-x));
    a.mom[i] = a.logits_f32 ? sg : bf16_round(sg);
  }
}

// Output side of the layer: y = bf16(x * rsqrt(mean(x^2) + eps) * weight) per head row (fp32 arithmetic, as the
// RMSNorm kernel the reference calls), times bf16(silu(gate projection)) rounded to bf16, heads merged back to
// [b][s][n_h * d], plus the attention output (layer_lact_swiglu.py:556-568).  One warp per (batch, token, head).
struct EpilogueArgs {
  const bf16* x;        // [(b n_h)][s][d] contiguous: output of the recurrence
  const float* weight;  // [d]
  const bf16* gate;     // [b][s][n_h * d] gate projection before its SiLU, or nullptr
  const bf16* resid;    // [b][s][n_h * d] tensor the result is added to, or nullptr
  bf16* out;            // [b][s][n_h * d]
  int64_t gate_ld, resid_ld, out_ld;  // row strides in elements (rows = b * s)
  int32_t b, s, n_h, d;
  float eps;
};
template <int NCH>
__global__ void __launch_bounds__(256, NCH <= 2 ? 8 : 4) out_epilogue_kernel(const EpilogueArgs a) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t rows = static_cast<int64_t>(a.b) * a.s * a.n_h;
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int h = static_cast<int>(row % a.n_h);
  const int64_t bs_idx = row / a.n_h;  // batch * s + token
  const int tok = static_cast<int>(bs_idx % a.s), bi = static_cast<int>(bs_idx / a.s);
  const bf16* src = a.x + ((static_cast<int64_t>(bi) * a.n_h + h) * a.s + tok) * a.d;
  float v[NCH][8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int col = (c * 32 + lane) * 8;
    if (col < a.d) {
      load8_bf16(src + col, v[c]);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[c][j] * v[c][j];
    }
  }
  ss = warp_sum(ss);
  const float rstd = 1.f / sqrtf(ss / static_cast<float>(a.d) + a.eps);
  const int64_t off = static_cast<int64_t>(h) * a.d;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int col = (c * 32 + lane) * 8;
    if (col >= a.d) continue;
    float y[8];
    const float4 w0 = *reinterpret_cast<const float4*>(a.weight + col), w1 = *reinterpret_cast<const float4*>(a.weight + col + 4);
    const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) y[j] = bf16_round(v[c][j] * rstd * w[j]);
    if (a.gate != nullptr) {
      float gt[8];
      load8_bf16(a.gate + bs_idx * a.gate_ld + off + col, gt);
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = bf16_round(y[j] * bf16_round(__fdividef(gt[j], 1.f + __expf(-gt[j]))));
    }
    if (a.resid != nullptr) {
      float r[8];
      load8_bf16(a.resid + bs_idx * a.resid_ld + off + col, r);
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] += r[j];
    }
    store8_bf16(a.out + bs_idx * a.out_ld + off + col, y);
  }
}

// ------------------------------------------------------------------------------------------
// backward of the layer passes (roundings of the forward treated as identities, fp32 arithmetic on the saved inputs)
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float silu_grad(float x) {
  const float sg = sigmoidf_fast(x);
  return sg * (1.f + x * (1.f - sg));
}

// Backward of qkv_prologue_kernel: one warp per (batch, token, head) and tensor.  Given dz (gradient of the head-major
// output) it undoes the rotation (dy = R^T dz), the per-head l2 norm (y = u / (||u|| + 1e-5)) and the SiLU, and writes
// dx [b][s][n_h * d] (contiguous).
struct PrologueBwdArgs {
  const bf16* x[3];      // saved projections, strides as in the forward
  int64_t ld[3], bs[3];
  const bf16* dz[3];     // [(b n_h)][s][d] contiguous, or nullptr (no gradient for that tensor: zeros are written)
  bf16* dx[3];           // [b][s][n_h * d] contiguous
  int32_t b, s, n_h, d;
  int32_t silu[3], l2norm[3];
  const bf16 *cos, *sin;
  int32_t rope_hd, pos0;
  const int32_t* seq_start;  // as in the forward
};
template <int NCH, bool ROPE>
__global__ void __launch_bounds__(256, (ROPE || NCH > 1) ? 2 : 4) qkv_prologue_bwd_kernel(const PrologueBwdArgs a) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t rows = static_cast<int64_t>(a.b) * a.s * a.n_h;
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int h = static_cast<int>(row % a.n_h);
  const int64_t bs_idx = row / a.n_h;
  const int tok = static_cast<int>(bs_idx % a.s), bi = static_cast<int>(bs_idx / a.s);
  const int64_t z_off = ((static_cast<int64_t>(bi) * a.n_h + h) * a.s + tok) * a.d;
  const int64_t x_out = bs_idx * (static_cast<int64_t>(a.n_h) * a.d) + static_cast<int64_t>(h) * a.d;
#pragma unroll
  for (int t = 0; t < 3; ++t) {
    const bf16* src = a.x[t] + bi * a.bs[t] + tok * a.ld[t] + static_cast<int64_t>(h) * a.d;
    float xv[NCH][8], u[NCH][8], g[NCH][8];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int col = (c * 32 + lane) * 8;
#pragma unroll
      for (int i = 0; i < 8; ++i) { xv[c][i] = 0.f; u[c][i] = 0.f; g[c][i] = 0.f; }
      if (col < a.d) {
        load8_bf16(src + col, xv[c]);
        if (a.dz[t] != nullptr) load8_bf16(a.dz[t] + z_off + col, g[c]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          u[c][i] = a.silu[t] ? bf16_round(__fdividef(xv[c][i], 1.f + __expf(-xv[c][i]))) : xv[c][i];
          ss += u[c][i] * u[c][i];
        }
      }
    }
    if (ROPE && t < 2) {
      // dy = R^T dz: first half dz cos + partner sin, second half dz cos - partner sin (partner as in the forward)
      const int half = a.rope_hd >> 1;
      const int64_t trow = static_cast<int64_t>(a.pos0 + tok - (a.seq_start != nullptr ? a.seq_start[tok] : 0)) * half;
      float other[NCH][8];
#pragma unroll
      for (int c = 0; c < NCH; ++c)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (half < 256) other[c][i] = __shfl_xor_sync(0xFFFFFFFFu, g[c][i], half >> 3);
          else other[c][i] = g[(c ^ (half >> 8)) < NCH ? (c ^ (half >> 8)) : c][i];
        }
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        const int col = (c * 32 + lane) * 8;
        if (col < a.d) {
          const int j = (static_cast<int>(h) * a.d + col) % a.rope_hd;
          const bool first = j < half;
          float cs[8], sn[8];
          load8_bf16(a.cos + trow + (first ? j : j - half), cs);
          load8_bf16(a.sin + trow + (first ? j : j - half), sn);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            g[c][i] = first ? g[c][i] * cs[i] + other[c][i] * sn[i] : g[c][i] * cs[i] - other[c][i] * sn[i];
        }
      }
    }
    if (a.l2norm[t]) {
      float dot = 0.f;
#pragma unroll
      for (int c = 0; c < NCH; ++c)
#pragma unroll
        for (int i = 0; i < 8; ++i) dot += g[c][i] * u[c][i];
      ss = warp_sum(ss);
      dot = warp_sum(dot);
      const float nrm = sqrtf(ss), den = nrm + 1e-5f;
      const float inv = 1.f / den, coef = dot / (den * den * fmaxf(nrm, 1e-30f));
#pragma unroll
      for (int c = 0; c < NCH; ++c)
#pragma unroll
        for (int i = 0; i < 8; ++i) g[c][i] = g[c][i] * inv - u[c][i] * coef;
    }
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int col = (c * 32 + lane) * 8;
      if (col < a.d) {
        if (a.silu[t]) {
#pragma unroll
          for (int i = 0; i < 8; ++i) g[c][i] *= silu_grad(xv[c][i]);
        }
        store8_bf16(a.dx[t] + x_out + col, g[c]);
      }
    }
  }
}

// Backward of out_epilogue_kernel.  Persistent grid: warp w of the grid walks rows w, w + W, ... (a fixed order), writes
// dx and dgate per row and keeps its share of the norm weight's gradient in registers; the block's eight shares are
// added in shared memory and stored as one partial row [gridDim.x][d] (the caller adds the partials: deterministic).
struct EpilogueBwdArgs {
  const bf16* x;        // [(b n_h)][s][d]
  const float* weight;  // [d]
  const bf16* gate;     // [b][s][n_h * d] or nullptr
  const bf16* dout;     // [b][s][n_h * d]
  int64_t gate_ld, dout_ld;
  bf16* dx;             // [(b n_h)][s][d]
  bf16* dgate;          // [b][s][n_h * d] contiguous, or nullptr
  float* dw_partial;    // [gridDim.x][d]
  int32_t b, s, n_h, d;
  float eps;
};
template <int NCH>
__global__ void __launch_bounds__(256, 2) out_epilogue_bwd_kernel(const EpilogueBwdArgs a) {
  __shared__ float red[8][32 * 8 + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t rows = static_cast<int64_t>(a.b) * a.s * a.n_h;
  const int64_t nwarps = static_cast<int64_t>(gridDim.x) * 8;
  float dw[NCH][8];
  float w[NCH][8];
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int col = (c * 32 + lane) * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) { dw[c][j] = 0.f; w[c][j] = col + j < a.d ? a.weight[col + j] : 0.f; }
  }
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + warp; row < rows; row += nwarps) {
    const int h = static_cast<int>(row % a.n_h);
    const int64_t bs_idx = row / a.n_h;
    const int tok = static_cast<int>(bs_idx % a.s), bi = static_cast<int>(bs_idx / a.s);
    const int64_t x_off = ((static_cast<int64_t>(bi) * a.n_h + h) * a.s + tok) * a.d;
    const int64_t off = static_cast<int64_t>(h) * a.d;
    float v[NCH][8], dn[NCH][8];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int col = (c * 32 + lane) * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) { v[c][j] = 0.f; dn[c][j] = 0.f; }
      if (col < a.d) {
        load8_bf16(a.x + x_off + col, v[c]);
        load8_bf16(a.dout + bs_idx * a.dout_ld + off + col, dn[c]);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += v[c][j] * v[c][j];
      }
    }
    ss = warp_sum(ss);
    const float rstd = 1.f / sqrtf(ss / static_cast<float>(a.d) + a.eps);
    float dot = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int col = (c * 32 + lane) * 8;
      if (col >= a.d) continue;
      if (a.gate != nullptr) {
        float gt[8], dg[8];
        load8_bf16(a.gate + bs_idx * a.gate_ld + off + col, gt);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float n = v[c][j] * rstd * w[c][j];
          dg[j] = dn[c][j] * n * silu_grad(gt[j]);
          dn[c][j] *= __fdividef(gt[j], 1.f + __expf(-gt[j]));
        }
        if (a.dgate != nullptr) store8_bf16(a.dgate + bs_idx * (static_cast<int64_t>(a.n_h) * a.d) + off + col, dg);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        dw[c][j] += dn[c][j] * v[c][j] * rstd;
        dot += dn[c][j] * w[c][j] * v[c][j];
      }
    }
    dot = warp_sum(dot);
    const float k3 = rstd * rstd * rstd * dot / static_cast<float>(a.d);
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int col = (c * 32 + lane) * 8;
      if (col >= a.d) continue;
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = rstd * w[c][j] * dn[c][j] - v[c][j] * k3;
      store8_bf16(a.dx + x_off + col, o);
    }
  }
  // block partial of the weight gradient: warp shares added in a fixed order
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 8; ++j) red[warp][lane * 8 + j] = dw[c][j];
    __syncthreads();
    if (warp == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int col = (c * 32 + lane) * 8 + j;
        float tot = 0.f;
        for (int ww = 0; ww < 8; ++ww) tot += red[ww][lane * 8 + j];
        if (col < a.d) a.dw_partial[static_cast<int64_t>(blockIdx.x) * a.d + col] = tot;
      }
    }
  }
}

}  // namespace lact
