// Backward of the attention kernel of swa.cuh (causal sliding window, or - causal = 0 - every key of the batch entry
// visible to every query) for sm_100a.  With P = softmax(q k^T * scale) restricted to the visible keys, recomputed from
// the forward's log-sum-exp L, and Delta_i = sum_d dO_i O_i:
//   dV_j = sum_i P_ij dO_i,   dS_ij = P_ij (dO_i . v_j - Delta_i) * scale,   dK_j = sum_i dS_ij q_i,   dQ_i = sum_j dS_ij k_j.
// One kernel, two modes (a CTA owns a 128-row OUTER tile and walks 64-row INNER tiles of its band):
//   MODE 0  outer = key tile j, inner = query tiles i:  dV_j += P^T dO_i,  dK_j += dS^T Q_i   (two accumulators)
//   MODE 1  outer = query tile i, inner = key tiles j:  dQ_i += dS K_j                        (one accumulator)
// The OUTER rows are the tensor-memory lanes in both modes: per inner tile the first products are
// [128 outer x 64 inner] (mode 0: S^T = K Q^T and dP^T = V dO^T; mode 1: S = Q K^T and dP = dO V^T), two softmax
// threads per lane (32 columns each) turn them into bf16 tiles [128 outer][64 inner] in shared memory (one 128-byte
// swizzled row per lane: the K-major A operand of the second products), and the inner tiles, [64 rows][64 columns] TMA
// boxes, serve as K-major B operands of the first products and as MN-major B operands (rows = k) of the second.
// Pipeline over the inner tiles: the inner tiles go through a three-stage ring (a stage is held from its load to the end
// of its second products, so two stages would put the load latency on the critical path), S / dP columns and the
// P / dS tiles are double-buffered; the issuing thread queues the first products of tile t + 1 BEFORE the second
// products of tile t, so the tensor pipe works on one tile while the softmax threads work on the other.  Every
// mbarrier wait is bounded; the one named barrier (mode 0, per-query values staged a tile ahead) is reached by every
// softmax thread in every iteration, whatever its waits returned.
#pragma once
#include "swa.cuh"

namespace lact {

struct SwaBwdArgs {
  CUtensorMap q, k, v, dout;           // 4-D maps (feature, token, head, batch), box {64, 128, 1, 1}: outer tiles
  CUtensorMap q64, k64, v64, dout64;   // the same tensors with box {64, 64, 1, 1}: inner tiles
  const float* lse;            // [b][h][l]: log2-domain log-sum-exp of the forward (m + log2(l))
  const float* delta;          // [b][h][l]: sum_d dO O
  const int32_t* seq_start;    // optional [l], as in the forward
  bf16* out0;                  // MODE 0: dK, MODE 1: dQ   ([b][l][h][d], strides below)
  bf16* out1;                  // MODE 0: dV
  int64_t o_bs, o_ts, o_hs;
  int32_t L, window, heads, tiles;   // L: queries per batch entry; tiles: outer tiles per (batch, head) of this launch
  int32_t Lk, causal;                // keys per batch entry (= L when causal); causal = 0: every query sees every key
  float scale_log2, scale;
  int32_t* status;
};

template <int HD>
struct SwaBwdSmem {
  static constexpr uint32_t kOTile = 128 * HD * 2;   // outer tile
  static constexpr uint32_t kITile = 64 * HD * 2;    // inner tile
  static constexpr uint32_t kWTile = 128 * 64 * 2;   // P or dS tile written by the softmax threads
  static constexpr int kInnerStages = 3;
  // outer pair | 3 stages x inner pair | 2 stages x (P, dS) | 2 stages x 3 x 64 per-query words (mode 0) | barriers
  static constexpr uint32_t kOuter = 0, kInner = 2 * kOTile, kW = kInner + kInnerStages * 2 * kITile,
                            kStats = kW + 4 * kWTile, kBars = kStats + 2 * 3 * 64 * 4;
  static constexpr uint32_t kBytes = kBars + 256 + 1024;
};

template <int HD, int MODE>
__global__ void __launch_bounds__(320, 1) swa_bwd_kernel(const __grid_constant__ SwaBwdArgs a) {
  static_assert(HD == 64 || HD == 128, "head dimensions 64 and 128");
  using SM = SwaBwdSmem<HD>;
  constexpr int KBD = HD / 64;
  constexpr uint32_t kBox = 128 * 128;    // [128 rows][64 features] box of an outer tile
  constexpr uint32_t kIBox = 64 * 128;    // [64 rows][64 features] box of an inner tile
  constexpr uint32_t kTmemCols = 512;     // 2 stages x (S 64, dP 64) at columns 0 / 128, accumulators from column 256
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + SM::kBars);
  uint64_t* outer_full = bars;        // the CTA's own two tiles have landed
  constexpr int NI = SM::kInnerStages;
  uint64_t* inner_full = bars + 1;    // [3] the inner pair of a ring stage has landed
  uint64_t* inner_empty = bars + 4;   // [3] second products that read a ring stage are done
  uint64_t* sdp_full = bars + 7;      // [2] S and dP of a stage are in tensor memory
  uint64_t* pds_full = bars + 9;      // [2] 8 arrivals: P and dS of a stage are in shared memory (S / dP columns read)
  uint64_t* w_empty = bars + 11;      // [2] second products that read a stage's P / dS tiles are done
  uint64_t* acc_full = bars + 13;     // all products of this CTA done
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(outer_full, 1);
    for (int s = 0; s < NI; ++s) {
      mbar_init(&inner_full[s], 1);
      mbar_init(&inner_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sdp_full[s], 1);
      mbar_init(&pds_full[s], 8);
      mbar_init(&w_empty[s], 1);
    }
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
  // inner 64-row tiles [t_lo, t_hi]
  int t_lo, t_hi;
  if (MODE == 0) {   // queries that see any key of this tile: q >= key, q <= key + window - 1
    t_lo = o0 / 64;
    const int q_max = o0 + 127 + window - 1;
    t_hi = (q_max < a.L - 1 ? q_max : a.L - 1) / 64;
    if (!a.causal) t_lo = 0, t_hi = (a.L - 1) / 64;   // block attention: every query tile
  } else {           // keys this query tile sees: not before the window of its first query, nor before that query's sequence
    int lo = o0 - (window - 1);
    if (lo < 0) lo = 0;
    if (a.seq_start != nullptr && a.seq_start[o0] > lo) lo = a.seq_start[o0];
    t_lo = lo / 64;
    t_hi = (o0 + 127 < a.L - 1 ? o0 + 127 : a.L - 1) / 64;
    if (!a.causal) t_lo = 0, t_hi = (a.Lk - 1) / 64;  // every key tile
  }
  const int T = t_hi - t_lo + 1;
  bool failed = *reinterpret_cast<volatile int32_t*>(a.status) != kStatusOk;
  const CUtensorMap* outer_a = MODE == 0 ? &a.k : &a.q;          // outer pair: (K, V) or (Q, dO)
  const CUtensorMap* outer_b = MODE == 0 ? &a.v : &a.dout;
  const CUtensorMap* inner_a = MODE == 0 ? &a.q64 : &a.k64;      // inner pair: (Q, dO) or (K, V)
  const CUtensorMap* inner_b = MODE == 0 ? &a.dout64 : &a.v64;

  if (warp == 0) {
    if (lane == 0 && !failed) {
      mbar_expect_tx(outer_full, 2 * SM::kOTile);
      for (int j = 0; j < KBD; ++j) {
        tma_load_4d(base + SM::kOuter + j * kBox, outer_a, outer_full, 64 * j, o0, head, batch);
        tma_load_4d(base + SM::kOuter + SM::kOTile + j * kBox, outer_b, outer_full, 64 * j, o0, head, batch);
      }
      for (int t = 0; t < T && !failed; ++t) {
        const int s = t % NI;
        if (t >= NI && !mbar_wait(&inner_empty[s], (t / NI - 1) & 1, abort_flag)) { failed = true; break; }
        mbar_expect_tx(&inner_full[s], 2 * SM::kITile);
        const uint32_t dst = base + SM::kInner + s * 2 * SM::kITile;
        for (int j = 0; j < KBD; ++j) {
          tma_load_4d(dst + j * kIBox, inner_a, &inner_full[s], 64 * j, (t_lo + t) * 64, head, batch);
          tma_load_4d(dst + SM::kITile + j * kIBox, inner_b, &inner_full[s], 64 * j, (t_lo + t) * 64, head, batch);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && !failed) {
      const uint32_t idesc_first = make_idesc_bf16(128, 64, 0, 0);   // [outer x inner], both operands K-major (features)
      const uint32_t idesc_acc = make_idesc_bf16(128, HD, 0, 1);     // [outer x HD]: A = P / dS tile K-major, B = inner tile MN-major
      const uint32_t o_a = base + SM::kOuter, o_b = o_a + SM::kOTile;
      // first products of inner tile t into its stage's columns
      auto first = [&](int t) -> bool {
        const int s = t & 1, si = t % NI;
        if (!mbar_wait(&inner_full[si], (t / NI) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t i_a = base + SM::kInner + si * 2 * SM::kITile, i_b = i_a + SM::kITile;
        const uint32_t col = tmem + s * 128;
#pragma unroll
        for (int kk = 0; kk < KBD; ++kk)
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4)
            umma_bf16(col, make_smem_desc(o_a + kk * kBox + k4 * 32, 0, 1024),
                      make_smem_desc(i_a + kk * kIBox + k4 * 32, 0, 1024), idesc_first, (kk | k4) != 0);
#pragma unroll
        for (int kk = 0; kk < KBD; ++kk)
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4)
            umma_bf16(col + 64, make_smem_desc(o_b + kk * kBox + k4 * 32, 0, 1024),
                      make_smem_desc(i_b + kk * kIBox + k4 * 32, 0, 1024), idesc_first, (kk | k4) != 0);
        umma_commit(&sdp_full[s]);
        return true;
      };
      if (!mbar_wait(outer_full, 0, abort_flag)) failed = true;
      if (!failed && !first(0)) failed = true;
      for (int t = 0; t < T && !failed; ++t) {
        const int s = t & 1;
        // (the other stage's columns were read by the softmax threads of tile t - 1: awaited one iteration ago)
        if (t + 1 < T && !first(t + 1)) { failed = true; break; }
        if (!mbar_wait(&pds_full[s], (t >> 1) & 1, abort_flag)) { failed = true; break; }
        tc_fence_after();
        const int si = t % NI;
        const uint32_t i_a = base + SM::kInner + si * 2 * SM::kITile, i_b = i_a + SM::kITile;
        const uint32_t w_p = base + SM::kW + s * 2 * SM::kWTile, w_ds = w_p + SM::kWTile;
        // contraction over the 64 inner rows: four 16-row steps
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
          if (MODE == 0) {
            umma_bf16(tmem + 256, make_smem_desc(w_p + k4 * 32, 0, 1024), make_smem_desc(i_b + k4 * 2048, kIBox, 1024),
                      idesc_acc, (t | k4) != 0);            // dV += P^T dO
            umma_bf16(tmem + 256 + HD, make_smem_desc(w_ds + k4 * 32, 0, 1024), make_smem_desc(i_a + k4 * 2048, kIBox, 1024),
                      idesc_acc, (t | k4) != 0);            // dK += dS^T Q
          } else {
            umma_bf16(tmem + 256, make_smem_desc(w_ds + k4 * 32, 0, 1024), make_smem_desc(i_a + k4 * 2048, kIBox, 1024),
                      idesc_acc, (t | k4) != 0);            // dQ += dS K
          }
        }
        umma_commit(&inner_empty[si]);
        umma_commit(&w_empty[s]);
      }
      if (!failed) umma_commit(acc_full);
    }
  } else {
    // ---------------- softmax / epilogue: two threads per tensor-memory lane (outer row), 32 inner columns each
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const int sid = threadIdx.x - 64;   // 0 .. 255
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const int64_t stat_base = (static_cast<int64_t>(batch) * a.heads + head) * a.L;
    const int row = o0 + r;             // this thread's key (mode 0) or query (mode 1)
    float* stats = reinterpret_cast<float*>(aligned + SM::kStats);   // [stage][lse | delta * scale | sequence start][64]
    // mode 0: per-query values of an inner tile, one word per thread 0 .. 191, staged one tile ahead
    auto stat_load = [&](int t) -> uint32_t {
      const int arr = sid >> 6, qi = (t_lo + t) * 64 + (sid & 63);
      if (arr == 0) return __float_as_uint(qi < a.L ? a.lse[stat_base + qi] : INFINITY);
      if (arr == 1) return __float_as_uint(qi < a.L ? a.delta[stat_base + qi] * a.scale : 0.f);
      return (a.seq_start != nullptr && qi < a.L) ? static_cast<uint32_t>(a.seq_start[qi]) : 0u;
    };
    float lse_r = INFINITY, delta_r = 0.f;
    int row_start = 0;
    if (MODE == 1 && row < a.L) {
      lse_r = a.lse[stat_base + row];
      delta_r = a.delta[stat_base + row] * a.scale;
      if (a.seq_start != nullptr) row_start = a.seq_start[row];
    }
    if (MODE == 0 && sid < 192) reinterpret_cast<uint32_t*>(stats)[sid] = stat_load(0);
    for (int t = 0; t < T; ++t) {
      const int s = t & 1;
      // every thread runs every iteration (the named barrier counts all 256), failed or not
      if (MODE == 0) named_barrier_sync(1, 256);   // stage s of the per-query words is written, stage s ^ 1 no longer read
      uint32_t next_stat = 0;
      if (MODE == 0 && sid < 192 && t + 1 < T) next_stat = stat_load(t + 1);
      if (!failed) {
        const int i0 = (t_lo + t) * 64;
        if (!mbar_wait(&sdp_full[s], (t >> 1) & 1, abort_flag) ||
            (t >= 2 && !mbar_wait(&w_empty[s], ((t >> 1) - 1) & 1, abort_flag))) {
          failed = true;
          *abort_flag = 1;
        }
        if (!failed) {
          tc_fence_after();
          const int c0 = half * 32;
          uint32_t sb[32], db[32];
          tmem_ld32(tmem + lane_off + s * 128 + c0, sb);
          tmem_ld32(tmem + lane_off + s * 128 + 64 + c0, db);
          tmem_ld_wait();
          // p = 2^(s c - lse),  dS = p (dP scale - Delta scale); tiles wholly inside the band skip the masks
          float p[32], ds[32];
          if (MODE == 0) {
            // rows = keys, columns = queries i0 + c
            const int last_q = i0 + 63 < a.L ? i0 + 63 : a.L - 1;
            const int tile_start = a.seq_start != nullptr ? a.seq_start[last_q] : 0;
            const bool interior = a.causal ? (o0 + 127 <= i0 && o0 >= i0 + 63 - (window - 1) && i0 + 63 < a.L && o0 >= tile_start)
                                           : (i0 + 63 < a.L && o0 + 127 < a.Lk);
            const float* st = stats + s * 192 + c0;
            if (interior) {
#pragma unroll
              for (int g = 0; g < 8; ++g) {
                const float4 l4 = *reinterpret_cast<const float4*>(st + g * 4);
                const float4 d4 = *reinterpret_cast<const float4*>(st + 64 + g * 4);
                const float lv[4] = {l4.x, l4.y, l4.z, l4.w}, dv[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const int j = g * 4 + e;
                  p[j] = fast_exp2(fmaf(__uint_as_float(sb[j]), a.scale_log2, -lv[e]));
                  ds[j] = p[j] * fmaf(__uint_as_float(db[j]), a.scale, -dv[e]);
                }
              }
            } else {
#pragma unroll
              for (int g = 0; g < 8; ++g) {
                const float4 l4 = *reinterpret_cast<const float4*>(st + g * 4);
                const float4 d4 = *reinterpret_cast<const float4*>(st + 64 + g * 4);
                const int4 s4 = *reinterpret_cast<const int4*>(st + 128 + g * 4);
                const float lv[4] = {l4.x, l4.y, l4.z, l4.w}, dv[4] = {d4.x, d4.y, d4.z, d4.w};
                const int sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const int j = g * 4 + e, qi = i0 + c0 + j;
                  const bool ok = (!a.causal || (row <= qi && row >= qi - (window - 1) && row >= sv[e])) && qi < a.L && row < a.Lk;
                  p[j] = ok ? fast_exp2(fmaf(__uint_as_float(sb[j]), a.scale_log2, -lv[e])) : 0.f;
                  ds[j] = p[j] * fmaf(__uint_as_float(db[j]), a.scale, -dv[e]);
                }
              }
            }
          } else {
            // rows = queries, columns = keys i0 + c
            const int last_q = o0 + 127 < a.L ? o0 + 127 : a.L - 1;
            const int tile_start = a.seq_start != nullptr ? a.seq_start[last_q] : 0;
            const bool interior = a.causal ? (i0 + 63 <= o0 && i0 >= o0 + 127 - (window - 1) && o0 + 127 < a.L && i0 >= tile_start)
                                           : (i0 + 63 < a.Lk && o0 + 127 < a.L);
            if (interior) {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                p[j] = fast_exp2(fmaf(__uint_as_float(sb[j]), a.scale_log2, -lse_r));
                ds[j] = p[j] * fmaf(__uint_as_float(db[j]), a.scale, -delta_r);
              }
            } else {
              const int k_hi = row < a.L ? (a.causal ? row : a.Lk - 1) : -1;   // last / first key this query may see
              const int k_lo = a.causal ? (row - (window - 1) > row_start ? row - (window - 1) : row_start) : 0;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const int kv = i0 + c0 + j;
                const bool ok = kv >= k_lo && kv <= k_hi;
                p[j] = ok ? fast_exp2(fmaf(__uint_as_float(sb[j]), a.scale_log2, -lse_r)) : 0.f;
                ds[j] = p[j] * fmaf(__uint_as_float(db[j]), a.scale, -delta_r);
              }
            }
          }
          const uint32_t p_row = base + SM::kW + s * 2 * SM::kWTile + r * 128, ds_row = p_row + SM::kWTile;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const uint32_t sw = ((half * 4 + g) ^ (r & 7)) << 4;
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
          tc_fence_before();
          fence_async_proxy();
          __syncwarp();
          if (lane == 0) mbar_arrive(&pds_full[s]);
        }
      }
      if (MODE == 0 && sid < 192 && t + 1 < T) reinterpret_cast<uint32_t*>(stats)[(s ^ 1) * 192 + sid] = next_stat;
    }
    // accumulators: row = outer-tile row (key in mode 0, query in mode 1); this thread stores HD / 2 features of it
    if (!failed && !mbar_wait(acc_full, 0, abort_flag)) failed = true;
    if (!failed) {
      tc_fence_after();
      constexpr int OC = HD / 2;
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
          if (row < (MODE == 0 ? a.Lk : a.L)) {
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
