// GEMM ops (operand/accumulator wiring + fp32 epilogues) built on the tcgen05 engine, and the
// small row-wise kernels of the fast-weight update (norms, momentum mean, Newton-Schulz
// normalisation, add + renormalise).
#pragma once
#include "umma_gemm.cuh"

namespace lact {

using bf16 = __nv_bfloat16;

// ------------------------------------------------------------------------------------------
// epilogue store helpers: each epilogue thread owns one accumulator row and 32 columns
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void store_row32_bf16(bf16* dst, const float* v, int valid) {
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    if (g * 8 < valid) {
      uint4 u;
      u.x = pack_bf16x2(v[g * 8 + 0], v[g * 8 + 1]);
      u.y = pack_bf16x2(v[g * 8 + 2], v[g * 8 + 3]);
      u.z = pack_bf16x2(v[g * 8 + 4], v[g * 8 + 5]);
      u.w = pack_bf16x2(v[g * 8 + 6], v[g * 8 + 7]);
      *reinterpret_cast<uint4*>(dst + g * 8) = u;
    }
  }
}
__device__ __forceinline__ void store_row32_f32(float* dst, const float* v, int valid) {
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    if (g * 4 < valid) {
      *reinterpret_cast<float4*>(dst + g * 4) = make_float4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
    }
  }
}
__device__ __forceinline__ void load_row32_bf16(const bf16* src, float* v, int valid) {
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    if (g * 8 < valid) {
      const uint4 u = *reinterpret_cast<const uint4*>(src + g * 8);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[g * 8 + 2 * i] = __uint_as_float(w[i] << 16);
        v[g * 8 + 2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[g * 8 + i] = 0.f;
    }
  }
}
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
  __device__ __forceinline__ void operator()(int batch, int row, int col, int M, int N, const float* v) const {
    if (row >= M) return;
    const int valid = min(32, N - col);
    const int64_t idx = batch * bs + static_cast<int64_t>(row + row_off) * ld + col;
    if (f32) store_row32_f32(reinterpret_cast<float*>(out) + idx, v, valid);
    else store_row32_bf16(reinterpret_cast<bf16*>(out) + idx, v, valid);
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
  __device__ __forceinline__ void operator()(int batch, int row, int col, int M, int N, const float* v) const {
    if (row >= M) return;
    const int valid = min(32, N - col);
    const int64_t idx = batch * bs + static_cast<int64_t>(row) * ld + col;
    float r[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) r[j] = round_bf16 ? bf16_round(v[j]) : v[j];
    if (out_f32) {
      float* gp = reinterpret_cast<float*>(g) + idx;
      if (beta != nullptr) {
        const float bt = beta[batch];
#pragma unroll
        for (int gq = 0; gq < 8; ++gq) {
          if (gq * 4 < valid) {
            const float4 old = *reinterpret_cast<const float4*>(gp + gq * 4);
            r[gq * 4 + 0] += old.x * bt;
            r[gq * 4 + 1] += old.y * bt;
            r[gq * 4 + 2] += old.z * bt;
            r[gq * 4 + 3] += old.w * bt;
          }
        }
      }
      store_row32_f32(gp, r, valid);
    } else {
      store_row32_bf16(reinterpret_cast<bf16*>(g) + idx, r, valid);
    }
  }
};

// Newton-Schulz epilogue, bf16 rounding after every elementwise op (the reference's eager
// arithmetic): t = bf16(acc); if res: t = bf16(bf16(alpha * res) + t); out = t;
// if out2: out2 = bf16(gamma * t).
struct EpiNs {
  bf16* out;
  bf16* out2;
  const bf16* res;
  float alpha, gamma;
  int64_t bs, ld;  // shared by out, out2 and res
  __device__ __forceinline__ void operator()(int batch, int row, int col, int M, int N, const float* v) const {
    if (row >= M) return;
    const int valid = min(32, N - col);
    const int64_t idx = batch * bs + static_cast<int64_t>(row) * ld + col;
    float t[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) t[j] = bf16_round(v[j]);
    if (res != nullptr) {
      float r[32];
      load_row32_bf16(res + idx, r, valid);
#pragma unroll
      for (int j = 0; j < 32; ++j) t[j] = bf16_round(bf16_round(alpha * r[j]) + t[j]);
    }
    store_row32_bf16(out + idx, t, valid);
    if (out2 != nullptr) {
      float u[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) u[j] = gamma * t[j];
      store_row32_bf16(out2 + idx, u, valid);
    }
  }
};

// SwiGLU gate: hidden = silu(y0) * y2 (fp32), stored as bf16 [batch][row][col].
struct EpiSwiglu {
  bf16* out;
  int64_t bs, ld;
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
  bf16* dy02;  // [batch][row][2H]: dy0 at column c, dy2 at column H + c
  int64_t dy_bs, dy_ld;
  int32_t H;
  bf16* hid;  // [batch][row][H]
  int64_t hid_bs, hid_ld;
};

// ------------------------------------------------------------------------------------------
// ops
// ------------------------------------------------------------------------------------------
template <class EpiT, int BN_, int STAGES_>
struct OpBmm {
  static constexpr int NA = 1, NB = 1, NACC = 1, BN = BN_, STAGES = STAGES_, NTERMS = 1;
  using Epi = EpiT;
  __host__ __device__ static constexpr int term_a(int) { return 0; }
  __host__ __device__ static constexpr int term_b(int) { return 0; }
  __host__ __device__ static constexpr int term_acc(int) { return 0; }
  __host__ __device__ static constexpr bool term_first(int) { return true; }
  __device__ static __forceinline__ void epilogue(const Epi& ep, int batch, int row, int col, int M, int N,
                                                  const float (&v)[1][32]) {
    ep(batch, row, col, M, N, v[0]);
  }
};

// y0 = x w0^T, y2 = x w2^T share the activation tile; epilogue = SwiGLU gate.
struct OpSwigluGate {
  static constexpr int NA = 1, NB = 2, NACC = 2, BN = 128, STAGES = 2, NTERMS = 2;
  using Epi = EpiSwiglu;
  __host__ __device__ static constexpr int term_a(int) { return 0; }
  __host__ __device__ static constexpr int term_b(int t) { return t; }
  __host__ __device__ static constexpr int term_acc(int t) { return t; }
  __host__ __device__ static constexpr bool term_first(int) { return true; }
  __device__ static __forceinline__ void epilogue(const Epi& ep, int batch, int row, int col, int M, int N,
                                                  const float (&v)[2][32]) {
    if (row >= M) return;
    float h[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float y0 = v[0][j];
      h[j] = v[1][j] * (y0 * sigmoidf_fast(y0));
    }
    store_row32_bf16(ep.out + batch * ep.bs + static_cast<int64_t>(row) * ep.ld + col, h, min(32, N - col));
  }
};

// y0 = k w0^T, y2 = k w2^T, dh = v w1: three accumulators, two activation tiles, three weights.
struct OpFwGradPointwise {
  static constexpr int NA = 2, NB = 3, NACC = 3, BN = 128, STAGES = 2, NTERMS = 3;
  using Epi = EpiFwGrad;
  __host__ __device__ static constexpr int term_a(int t) { return t == 2 ? 1 : 0; }
  __host__ __device__ static constexpr int term_b(int t) { return t; }
  __host__ __device__ static constexpr int term_acc(int t) { return t; }
  __host__ __device__ static constexpr bool term_first(int) { return true; }
  __device__ static __forceinline__ void epilogue(const Epi& ep, int batch, int row, int col, int M, int N,
                                                  const float (&v)[3][32]) {
    if (row >= M) return;
    const int64_t li = batch * ep.lr_bs + ep.tok_off + row;
    const float l0 = load_scalar(ep.lr0, ep.lr_f32, li) * ep.w_scale;
    const float l1 = load_scalar(ep.lr1, ep.lr_f32, li) * ep.w_scale;
    const float l2 = load_scalar(ep.lr2, ep.lr_f32, li) * ep.w_scale;
    float hid[32], dy0[32], dy2[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float y0 = v[0][j], y2 = v[1][j], dh = v[2][j];
      const float sg = sigmoidf_fast(y0);
      const float sw = sg * y0;
      hid[j] = sw * y2 * l1;
      dy0[j] = sg * y2 * dh * (1.0f + y0 * (1.0f - sg)) * l0;
      dy2[j] = sw * dh * l2;
    }
    const int valid = min(32, N - col);
    bf16* d = ep.dy02 + batch * ep.dy_bs + static_cast<int64_t>(row) * ep.dy_ld + col;
    store_row32_bf16(d, dy0, valid);
    store_row32_bf16(d + ep.H, dy2, valid);
    store_row32_bf16(ep.hid + batch * ep.hid_bs + static_cast<int64_t>(row) * ep.hid_ld + col, hid, valid);
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

// beta[b] = mean over tokens [s, e) of momentum[b, t]; one CTA per batch entry.
__global__ void momentum_mean_kernel(const void* mom, int mom_f32, int64_t bs, int s, int e, float* beta) {
  __shared__ float part[32];
  const int b = blockIdx.x;
  float acc = 0.f;
  for (int t = s + threadIdx.x; t < e; t += blockDim.x) acc += load_scalar(mom, mom_f32, b * bs + t);
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float x = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0.f;
    x = warp_sum(x);
    if (threadIdx.x == 0) {
      float m = x / static_cast<float>(e - s);
      beta[b] = mom_f32 ? m : bf16_round(m);
    }
  }
}

// Newton-Schulz start: X = bf16(G); X = X / (||X||_F + 1e-7) with bf16 rounding of the norm, of
// the sum and of the quotient; written transposed when `transpose` (the iteration always runs
// on the wide orientation).  One CTA per matrix; src is fp32 or bf16, [R][C] with row stride ld.
__global__ void ns_prepare_kernel(const void* src, int src_f32, int64_t src_ms, int ld, int R, int C, int transpose,
                                  bf16* X, int64_t x_ms) {
  __shared__ float part[32];
  __shared__ float den_s;
  const int mat = blockIdx.x;
  const int64_t base = mat * src_ms;
  const int total = R * C;
  float ss = 0.f;
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    const int r = i / C, c = i - r * C;
    const float x = bf16_round(load_scalar(src, src_f32, base + static_cast<int64_t>(r) * ld + c));
    ss += x * x;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float x = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0.f;
    x = warp_sum(x);
    if (threadIdx.x == 0) den_s = bf16_round(bf16_round(sqrtf(x)) + 1e-7f);
  }
  __syncthreads();
  const float den = den_s;
  bf16* xo = X + mat * x_ms;
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    const int r = i / C, c = i - r * C;
    const float x = bf16_round(load_scalar(src, src_f32, base + static_cast<int64_t>(r) * ld + c));
    const bf16 y = __float2bfloat16_rn(x / den);
    if (transpose) xo[static_cast<int64_t>(c) * R + r] = y;
    else xo[static_cast<int64_t>(r) * C + c] = y;
  }
}

// Copies a bf16 Newton-Schulz result back to the caller's [R][C] orientation.
__global__ void ns_export_kernel(const bf16* X, int64_t x_ms, int R, int C, int transposed, bf16* out, int64_t o_ms) {
  const int mat = blockIdx.x;
  const int total = R * C;
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    const int r = i / C, c = i - r * C;
    out[mat * o_ms + i] = transposed ? X[mat * x_ms + static_cast<int64_t>(c) * R + r] : X[mat * x_ms + i];
  }
}

struct RenormArgs {
  float* master;     // [B][R][C] fp32, in/out
  float* compute;    // [B][R][C] fp32 out: the weights the next step computes with
  bf16* shadow;      // [B][R][C] bf16 out
  const float* n0;   // [B][R]
  const float* g;    // [B][R][C] fp32 gradient (after momentum)
  const bf16* x;     // Newton-Schulz result or nullptr (then the update is g)
  int64_t x_ms;      // matrix stride of x
  int32_t x_mats_per_b, x_rows_per_mat;  // W rows [j*rows_per_mat, (j+1)*rows_per_mat) belong to matrix b*mats_per_b + j
  int32_t x_mat_off;                     // index of this weight's first matrix in x
  int32_t x_transposed, x_ld;            // x is stored [C][rows_per_mat] (transposed) or [rows_per_mat][C]
  int32_t B, R, C;
  int32_t mode;      // LACT_RENORM_*
  int32_t prenorm, prenorm_bf16, quirk;
};

// w_new = (quirk ? g : master) + update; normalise rows; one warp per row.
__global__ void add_renorm_kernel(const RenormArgs a) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= static_cast<int64_t>(a.B) * a.R) return;
  const int lane = threadIdx.x & 31;
  const int b = static_cast<int>(row / a.R), r = static_cast<int>(row % a.R);
  const int64_t off = row * a.C;
  const bf16* xm = nullptr;
  int lr = 0;
  if (a.x != nullptr) {
    const int j = r / a.x_rows_per_mat;
    lr = r - j * a.x_rows_per_mat;
    xm = a.x + static_cast<int64_t>(a.x_mat_off + b * a.x_mats_per_b + j) * a.x_ms;
  }
  float ss = 0.f;
  for (int c = lane; c < a.C; c += 32) {
    const float g = a.g[off + c];
    float upd = g;
    if (xm != nullptr)
      upd = __bfloat162float(a.x_transposed ? xm[static_cast<int64_t>(c) * a.x_ld + lr]
                                            : xm[static_cast<int64_t>(lr) * a.x_ld + c]);
    const float base = (a.quirk && xm != nullptr) ? g : a.master[off + c];
    const float w = base + upd;
    a.compute[off + c] = w;  // staged; normalised below
    ss += w * w;
  }
  ss = warp_sum(ss);
  const float n0 = a.n0[row];
  const float den = sqrtf(ss) + 1e-5f;
  const float rstd = 1.0f / sqrtf(ss + 1e-5f);
  __syncwarp();
  for (int c = lane; c < a.C; c += 32) {
    const float w = a.compute[off + c];
    float y = w;
    if (a.mode == 1) y = w / den * n0;
    else if (a.mode == 2) y = w * rstd * n0;
    if (a.prenorm && a.prenorm_bf16) y = bf16_round(y);
    a.master[off + c] = a.prenorm ? w : y;
    a.compute[off + c] = y;
    a.shadow[off + c] = __float2bfloat16_rn(y);
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

}  // namespace lact
