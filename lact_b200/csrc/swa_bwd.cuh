// Backward of the causal sliding-window attention (swa.cuh) for sm_100a.  With P = softmax(q k^T * scale) restricted
// to the band, recomputed from the forward's log-sum-exp L, and Delta_i = sum_d dO_i O_i:
//   dV_j = sum_i P_ij dO_i,   dS_ij = P_ij (dO_i . v_j - Delta_i) * scale,   dK_j = sum_i dS_ij q_i,   dQ_i = sum_j dS_ij k_j.
// One kernel, two modes (a CTA owns a 128-row OUTER tile and walks the INNER tiles of its band):
//   MODE 0  outer = key tile j, inner = query tiles i:  dV_j += P^T dO_i,  dK_j += dS^T Q_i   (two accumulators)
//   MODE 1  outer = query tile i, inner = key tiles j:  dQ_i += dS K_j                        (one accumulator)
// Per inner tile: S = Q K^T and dP = dO V^T into tensor memory (128 columns each), the softmax threads (two per query
// row, 64 keys each; a row is a tensor-memory lane) turn them into bf16 P and dS tiles in shared memory
// ([queries][keys], 128-byte swizzled panels), and the second group of products reads those tiles K-major (dS K) or
// MN-major (P^T dO, dS^T Q: the same bytes seen as [k = queries][m = keys]).  Every tile in shared memory is a set of
// [128 rows][64 columns] TMA boxes, so q / k / v / dO tiles serve as K-major (features = k) or MN-major (rows = k)
// operands as needed.  The stages run strictly one after the other (load, first products, softmax, second products):
// single-buffered, simple, every wait bounded.
#pragma once
#include "swa.cuh"

namespace lact {

struct SwaBwdArgs {
  CUtensorMap q, k, v, dout;   // 4-D maps (feature, token, head, batch), box {64, 128, 1, 1}
  const float* lse;            // [b][h][l]: log2-domain log-sum-exp of the forward (m + log2(l))
  const float* delta;          // [b][h][l]: sum_d dO O
  const int32_t* seq_start;    // optional [l], as in the forward
  bf16* out0;                  // MODE 0: dK, MODE 1: dQ   ([b][l][h][d], strides below)
  bf16* out1;                  // MODE 0: dV
  int64_t o_bs, o_ts, o_hs;
  int32_t L, window, heads, tiles;
  float scale_log2, scale;
  int32_t* status;
};

template <int HD>
struct SwaBwdSmem {
  static constexpr uint32_t kTile = 128 * HD * 2;
  static constexpr uint32_t kPTile = 128 * 128 * 2;
  // outer pair, inner pair, P, dS
  static constexpr uint32_t kOuter = 0, kInner = 2 * kTile, kP = 4 * kTile, kDS = 4 * kTile + kPTile, kBars = 4 * kTile + 2 * kPTile;
  static constexpr uint32_t kBytes = kBars + 256 + 1024;
};

template <int HD, int MODE>
__global__ void __launch_bounds__(320, 1) swa_bwd_kernel(const __grid_constant__ SwaBwdArgs a) {
  static_assert(HD == 64 || HD == 128, "head dimensions 64 and 128");
  using SM = SwaBwdSmem<HD>;
  constexpr int KBD = HD / 64;
  constexpr uint32_t kBox = 128 * 128;
  constexpr uint32_t kTmemCols = 512;   // S 128, dP 128, accumulators 2 x HD
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + SM::kBars);
  uint64_t* outer_full = bars;        // the CTA's own two tiles have landed
  uint64_t* inner_full = bars + 1;    // the inner pair of this iteration has landed
  uint64_t* inner_empty = bars + 2;   // second products done: inner tiles, P / dS tiles and S / dP columns reusable
  uint64_t* sdp_full = bars + 3;      // S and dP are in tensor memory
  uint64_t* pds_full = bars + 4;      // 8 arrivals: P and dS are in shared memory
  uint64_t* acc_full = bars + 5;      // all products of this CTA done
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(outer_full, 1);
    mbar_init(inner_full, 1);
    mbar_init(inner_empty, 1);
    mbar_init(sdp_full, 1);
    mbar_init(pds_full, 8);
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  const int ot = blockIdx.x % a.tiles;
  const int head = (blockIdx.x / a.tiles) % a.heads;
  const int batch = blockIdx.x / (a.tiles * a.heads);
  const int o0 = ot * 128;   // first row of the outer tile (keys in mode 0, queries in mode 1)
  const int window = a.window > 0 ? a.window : a.L;
  // inner tiles [t_lo, t_hi]
  int t_lo, t_hi;
  if (MODE == 0) {   // queries that see any key of this tile: q >= key, q <= key + window - 1
    t_lo = ot;
    const int q_max = o0 + 127 + window - 1;
    t_hi = (q_max < a.L - 1 ? q_max : a.L - 1) / 128;
  } else {           // keys this query tile sees
    const int lo = o0 - (window - 1);
    t_lo = lo < 0 ? 0 : lo / 128;
    t_hi = ot;
  }
  const int T = t_hi - t_lo + 1;
  bool failed = *reinterpret_cast<volatile int32_t*>(a.status) != kStatusOk;
  const CUtensorMap* outer_a = MODE == 0 ? &a.k : &a.q;      // outer pair: (K, V) or (Q, dO)
  const CUtensorMap* outer_b = MODE == 0 ? &a.v : &a.dout;
  const CUtensorMap* inner_a = MODE == 0 ? &a.q : &a.k;      // inner pair: (Q, dO) or (K, V)
  const CUtensorMap* inner_b = MODE == 0 ? &a.dout : &a.v;

  if (warp == 0) {
    if (lane == 0 && !failed) {
      mbar_expect_tx(outer_full, 2 * SM::kTile);
      for (int j = 0; j < KBD; ++j) {
        tma_load_4d(base + SM::kOuter + j * kBox, outer_a, outer_full, 64 * j, o0, head, batch);
        tma_load_4d(base + SM::kOuter + SM::kTile + j * kBox, outer_b, outer_full, 64 * j, o0, head, batch);
      }
      for (int t = 0; t < T && !failed; ++t) {
        if (t >= 1 && !mbar_wait(inner_empty, (t - 1) & 1, abort_flag)) { failed = true; break; }
        mbar_expect_tx(inner_full, 2 * SM::kTile);
        for (int j = 0; j < KBD; ++j) {
          tma_load_4d(base + SM::kInner + j * kBox, inner_a, inner_full, 64 * j, (t_lo + t) * 128, head, batch);
          tma_load_4d(base + SM::kInner + SM::kTile + j * kBox, inner_b, inner_full, 64 * j, (t_lo + t) * 128, head, batch);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && !failed) {
      const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      // MODE 0: [keys x HD] = (P or dS)^T [keys x queries] (A MN-major) * (dO or Q) [queries x HD] (B MN-major)
      // MODE 1: [queries x HD] = dS [queries x keys] (A K-major) * K [keys x HD] (B MN-major)
      const uint32_t idesc_acc = make_idesc_bf16(128, HD, MODE == 0 ? 1 : 0, 1);
      // tiles by role: Q, dO hold the queries; K, V the keys
      const uint32_t t_q = base + (MODE == 0 ? SM::kInner : SM::kOuter), t_do = t_q + SM::kTile;
      const uint32_t t_k = base + (MODE == 0 ? SM::kOuter : SM::kInner), t_v = t_k + SM::kTile;
      if (!mbar_wait(outer_full, 0, abort_flag)) failed = true;
      for (int t = 0; t < T && !failed; ++t) {
        if (!mbar_wait(inner_full, t & 1, abort_flag)) { failed = true; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < KBD; ++kk)
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4)
            umma_bf16(tmem, make_smem_desc(t_q + kk * kBox + k4 * 32, 0, 1024),
                      make_smem_desc(t_k + kk * kBox + k4 * 32, 0, 1024), idesc_s, (kk | k4) != 0);
#pragma unroll
        for (int kk = 0; kk < KBD; ++kk)
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4)
            umma_bf16(tmem + 128, make_smem_desc(t_do + kk * kBox + k4 * 32, 0, 1024),
                      make_smem_desc(t_v + kk * kBox + k4 * 32, 0, 1024), idesc_s, (kk | k4) != 0);
        umma_commit(sdp_full);
        if (!mbar_wait(pds_full, t & 1, abort_flag)) { failed = true; break; }
        tc_fence_after();
        const uint32_t t_p = base + SM::kP, t_ds = base + SM::kDS;
        if (MODE == 0) {
          // contraction over the 128 queries: two 64-query k-blocks, four 16-query steps each; A atoms = 64-key panels
#pragma unroll
          for (int kk = 0; kk < 2; ++kk)
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
              const uint32_t step = kk * kAtomBytes + k4 * 2048;
              umma_bf16(tmem + 256, make_smem_desc(t_p + step, kBox, 1024), make_smem_desc(t_do + step, kBox, 1024),
                        idesc_acc, (t | kk | k4) != 0);            // dV += P^T dO
              umma_bf16(tmem + 256 + HD, make_smem_desc(t_ds + step, kBox, 1024), make_smem_desc(t_q + step, kBox, 1024),
                        idesc_acc, (t | kk | k4) != 0);            // dK += dS^T Q
            }
        } else {
          // contraction over the 128 keys: A = dS K-major (two 64-key panels), B = K tile MN-major
#pragma unroll
          for (int kk = 0; kk < 2; ++kk)
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4)
              umma_bf16(tmem + 256, make_smem_desc(t_ds + kk * kBox + k4 * 32, 0, 1024),
                        make_smem_desc(t_k + kk * kAtomBytes + k4 * 2048, kBox, 1024), idesc_acc, (t | kk | k4) != 0);
        }
        umma_commit(inner_empty);
      }
      if (!failed) umma_commit(acc_full);
    }
  } else {
    // ---------------- softmax / epilogue: two threads per tensor-memory lane (row), 64 columns each
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const int64_t stat_base = (static_cast<int64_t>(batch) * a.heads + head) * a.L;
    float lse_r = INFINITY, delta_r = 0.f;
    if (MODE == 1 && o0 + r < a.L) {
      lse_r = a.lse[stat_base + o0 + r];
      delta_r = a.delta[stat_base + o0 + r];
    }
    for (int t = 0; t < T && !failed; ++t) {
      const int i0 = (t_lo + t) * 128;
      const int q0 = MODE == 0 ? i0 : o0, kv0 = MODE == 0 ? o0 : i0;
      const int qi = q0 + r;
      if (MODE == 0) {   // the rows are this iteration's queries
        lse_r = qi < a.L ? a.lse[stat_base + qi] : INFINITY;
        delta_r = qi < a.L ? a.delta[stat_base + qi] : 0.f;
      }
      if (!mbar_wait(sdp_full, t & 1, abort_flag)) { failed = true; break; }
      tc_fence_after();
      // (packed sequences: the last query row of the tile has the latest sequence start)
      const int tile_start = a.seq_start != nullptr ? a.seq_start[q0 + 127 < a.L ? q0 + 127 : a.L - 1] : 0;
      const int row_start = (a.seq_start != nullptr && qi < a.L) ? a.seq_start[qi] : 0;
      const bool interior = kv0 + 127 <= q0 && kv0 >= q0 + 127 - (window - 1) && kv0 + 127 < a.L && q0 + 127 < a.L &&
                            kv0 >= tile_start;
      const int c0 = half * 64;
      const int j_hi = (qi < a.L ? qi : -1) - kv0;   // last / first key column of the tile this query may see
      const int j_lo = (qi - (window - 1) > row_start ? qi - (window - 1) : row_start) - kv0;
      const int j_end = a.L - kv0;                     // keys beyond the sequence
      const uint32_t s_addr = tmem + lane_off + c0, dp_addr = tmem + lane_off + 128 + c0;
      const uint32_t p_row = base + SM::kP + half * kBox + r * 128, ds_row = base + SM::kDS + half * kBox + r * 128;
#pragma unroll
      for (int c = 0; c < 64; c += 32) {
        uint32_t sb[32], db[32];
        tmem_ld32(s_addr + c, sb);
        tmem_ld32(dp_addr + c, db);
        tmem_ld_wait();
        float p[32], ds[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int col = c0 + c + j;
          const bool ok = interior || (col >= j_lo && col <= j_hi && col < j_end);
          p[j] = ok ? fast_exp2(fmaf(__uint_as_float(sb[j]), a.scale_log2, -lse_r)) : 0.f;
          ds[j] = p[j] * (__uint_as_float(db[j]) - delta_r) * a.scale;
        }
        const uint32_t unit0 = (c & 63) >> 3;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const uint32_t sw = ((unit0 + g) ^ (r & 7)) << 4;
          if (MODE == 0)
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(p_row + sw), "r"(pack_bf16x2(p[g * 8 + 0], p[g * 8 + 1])),
                         "r"(pack_bf16x2(p[g * 8 + 2], p[g * 8 + 3])), "r"(pack_bf16x2(p[g * 8 + 4], p[g * 8 + 5])),
                         "r"(pack_bf16x2(p[g * 8 + 6], p[g * 8 + 7]))
                         : "memory");
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(ds_row + sw), "r"(pack_bf16x2(ds[g * 8 + 0], ds[g * 8 + 1])),
                       "r"(pack_bf16x2(ds[g * 8 + 2], ds[g * 8 + 3])), "r"(pack_bf16x2(ds[g * 8 + 4], ds[g * 8 + 5])),
                       "r"(pack_bf16x2(ds[g * 8 + 6], ds[g * 8 + 7]))
                       : "memory");
        }
      }
      tc_fence_before();
      fence_async_proxy();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
    }
    // accumulators: row = outer-tile row (key in mode 0, query in mode 1); this thread stores HD / 2 features of it
    if (!failed && !mbar_wait(acc_full, 0, abort_flag)) failed = true;
    if (!failed) {
      tc_fence_after();
      constexpr int OC = HD / 2;
      const int row = o0 + r;
#pragma unroll
      for (int acc = 0; acc < (MODE == 0 ? 2 : 1); ++acc) {
        // mode 0: accumulator 0 = dV, accumulator 1 = dK; mode 1: dQ
        bf16* dst_base = MODE == 0 ? (acc == 0 ? a.out1 : a.out0) : a.out0;
        bf16* dst = dst_base + batch * a.o_bs + static_cast<int64_t>(row) * a.o_ts + head * a.o_hs + half * OC;
#pragma unroll
        for (int c = 0; c < OC; c += 32) {
          uint32_t bits[32];
          tmem_ld32(tmem + lane_off + 256 + acc * HD + half * OC + c, bits);
          tmem_ld_wait();
          if (row < a.L) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 u;
              u.x = pack_bf16x2(__uint_as_float(bits[g * 8 + 0]), __uint_as_float(bits[g * 8 + 1]));
              u.y = pack_bf16x2(__uint_as_float(bits[g * 8 + 2]), __uint_as_float(bits[g * 8 + 3]));
              u.z = pack_bf16x2(__uint_as_float(bits[g * 8 + 4]), __uint_as_float(bits[g * 8 + 5]));
              u.w = pack_bf16x2(__uint_as_float(bits[g * 8 + 6]), __uint_as_float(bits[g * 8 + 7]));
              *reinterpret_cast<uint4*>(dst + c + g * 8) = u;
            }
          }
        }
      }
    }
  }
  if (failed && *reinterpret_cast<volatile int32_t*>(a.status) == kStatusOk) {
    *abort_flag = 1;
    atomicCAS(a.status, kStatusOk, kStatusWaitTimeout);
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    for (int i = 0; i < 256; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

// Delta[b][h][i] = sum_d dO[b][i][h][d] * O[b][i][h][d]: one warp per (batch, token, head) row.
struct SwaDeltaArgs {
  const bf16 *o, *dout;      // [b][l][h][d], token / batch strides below, head stride d
  int64_t o_ts, o_bs, d_ts, d_bs;
  float* delta;              // [b][h][l]
  int32_t b, L, heads, d;
};
__global__ void __launch_bounds__(256) swa_delta_kernel(const SwaDeltaArgs a) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int64_t rows = static_cast<int64_t>(a.b) * a.L * a.heads;
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int h = static_cast<int>(row % a.heads);
  const int64_t bl = row / a.heads;
  const int tok = static_cast<int>(bl % a.L), bi = static_cast<int>(bl / a.L);
  const bf16* po = a.o + bi * a.o_bs + tok * a.o_ts + static_cast<int64_t>(h) * a.d;
  const bf16* pd = a.dout + bi * a.d_bs + tok * a.d_ts + static_cast<int64_t>(h) * a.d;
  float acc = 0.f;
  for (int c = lane * 4; c < a.d; c += 128) {
    const uint2 uo = *reinterpret_cast<const uint2*>(po + c), ud = *reinterpret_cast<const uint2*>(pd + c);
    acc += __uint_as_float(uo.x << 16) * __uint_as_float(ud.x << 16) +
           __uint_as_float(uo.x & 0xFFFF0000u) * __uint_as_float(ud.x & 0xFFFF0000u) +
           __uint_as_float(uo.y << 16) * __uint_as_float(ud.y << 16) +
           __uint_as_float(uo.y & 0xFFFF0000u) * __uint_as_float(ud.y & 0xFFFF0000u);
  }
  acc = warp_sum(acc);
  if (lane == 0) a.delta[(static_cast<int64_t>(bi) * a.heads + h) * a.L + tok] = acc;
}

}  // namespace lact
