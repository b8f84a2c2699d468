// Causal sliding-window attention forward for sm_100a: o_i = softmax_j(q_i . k_j / sqrt(d)) v_j over the keys
// i - window < j <= i of the same (batch, head); with causal = 0, over all Lk keys of the batch entry (block
// attention).  One CTA per (batch, head, 128-query tile):
//   warp 0     TMA producer: the query tile once, then key and value tiles of 128 rows through two-stage rings;
//   warp 1     MMA issuer:   S = Q K^T (128 x 128, fp32, tensor memory, double-buffered) and O_t = P V per key tile
//                            (128 x d, tensor memory, double-buffered; NOT accumulated across tiles);
//   warps 2-9  softmax:      two threads per query row (a row is a tensor-memory lane; the two warps that may read a
//                            lane quarter split the row: 64 keys of S and half of the output features each, and
//                            swap their row maxima through shared memory at a named barrier): the 64 scores are read
//                            once into registers (max, then exp2 / sum), the bf16 probabilities go to shared memory in the swizzled K-major layout
//                            the second product reads as its A operand, and the running output row lives in
//                            registers: O <- O * exp2(m_old - m_new) + O_t, folded one tile behind so that the
//                            products of tile t + 1 overlap the softmax of tile t.  Two warps per scheduler hide the
//                            fixed latencies one warp alone sits out.
// Key and value tiles share one shared-memory layout ([128 rows][64 features] boxes, 128-byte swizzle): the first
// product reads it K-major (features = k), the second MN-major (keys = k).  Every mbarrier wait is bounded; the named
// barriers of the row pairs are reached by every softmax thread in every iteration, whatever its waits returned.
#pragma once
#include "umma_gemm.cuh"

namespace lact {

struct SwaArgs {
  CUtensorMap q, k, v;   // 4-D maps (feature, token, head, batch), box {64, 128, 1, 1}
  bf16* o;               // [b][l][h][d], strides below (elements); feature stride 1
  int64_t o_bs, o_ts, o_hs;
  int32_t L, window;     // queries per batch entry; window <= 0: unbounded (plain causal attention)
  int32_t Lk, causal;    // keys per batch entry (= L when causal); causal = 0: every query sees every key of its entry
  int32_t heads, q_tiles;
  float scale_log2;      // log2(e) / sqrt(d)
  const int32_t* seq_start;  // optional [l]: first token of the packed sequence every token belongs to (nondecreasing;
                             // keys before it are invisible), or nullptr: one sequence per batch entry
  float* lse;            // optional [b][h][l]: log2-domain log-sum-exp of every row (the backward's input), or nullptr
  int32_t* status;
};

// 2^x by the hardware approximation (2^-inf = 0)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int HD>
struct SwaSmem {
  static constexpr uint32_t kTile = 128 * HD * 2;          // one Q / K / V tile
  static constexpr uint32_t kPTile = 128 * 128 * 2;        // probabilities of one key tile
  static constexpr uint32_t kQ = 0, kK = kTile, kV = 3 * kTile, kP = 5 * kTile, kBars = 5 * kTile + 2 * kPTile;
  static constexpr uint32_t kBytes = kBars + 256 + 1024 + 1024;   // + barriers + row-pair exchange + alignment slack
};

template <int HD>
__global__ void __launch_bounds__(320, 1) swa_fwd_kernel(const __grid_constant__ SwaArgs a) {
  static_assert(HD == 64 || HD == 128, "head dimensions 64 and 128");
  using SM = SwaSmem<HD>;
  constexpr int KBD = HD / 64;                // 64-feature blocks of a tile
  constexpr uint32_t kBox = 128 * 128;        // bytes of one [128][64] box
  constexpr uint32_t kTmemCols = 512;         // S: 2 x 128, O: 2 x HD
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + SM::kBars);
  uint64_t* q_full = bars;            // [1]
  uint64_t* k_full = bars + 1;        // [2]
  uint64_t* k_empty = bars + 3;       // [2]
  uint64_t* v_full = bars + 5;        // [2]
  uint64_t* s_full = bars + 7;        // [2]
  uint64_t* s_empty = bars + 9;       // [2]  8 arrivals (one per softmax warp)
  uint64_t* p_full = bars + 11;       // [2]  8 arrivals
  uint64_t* pv_done = bars + 13;      // [2]  frees the value stage and the probability buffer, publishes O_t
  uint64_t* o_empty = bars + 15;      // [2]  8 arrivals
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  float* xch = reinterpret_cast<float*>(aligned + SM::kBars + 256);   // [2 halves][128 rows]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], 8);
      mbar_init(&p_full[s], 8);
      mbar_init(&pv_done[s], 1);
      mbar_init(&o_empty[s], 8);
    }
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

  // this CTA's query tile and the key tiles its window touches
  const int qt = blockIdx.x % a.q_tiles;
  const int head = (blockIdx.x / a.q_tiles) % a.heads;
  const int batch = blockIdx.x / (a.q_tiles * a.heads);
  const int q0 = qt * 128;
  const int window = a.window > 0 ? a.window : a.L;
  int kv_lo = q0 - (window - 1);
  kv_lo = kv_lo < 0 ? 0 : (kv_lo / 128) * 128;
  // packed sequences: no row of this tile sees a key before the first row's sequence start
  if (a.seq_start != nullptr && a.seq_start[q0] > kv_lo) kv_lo = (a.seq_start[q0] / 128) * 128;
  const int tile_start = a.seq_start != nullptr ? a.seq_start[q0 + 127 < a.L ? q0 + 127 : a.L - 1] : 0;  // last row's
  int kv_hi = q0 + 128 < a.L ? q0 + 128 : a.L;
  if (!a.causal) {   // block attention: all keys of the entry
    kv_lo = 0;
    kv_hi = a.Lk;
  }
  const int T = (kv_hi - kv_lo + 127) / 128;
  bool failed = *reinterpret_cast<volatile int32_t*>(a.status) != kStatusOk;

  if (warp == 0) {
    if (lane == 0 && !failed) {
      mbar_expect_tx(q_full, SM::kTile);
      for (int j = 0; j < KBD; ++j) tma_load_4d(base + SM::kQ + j * kBox, &a.q, q_full, 64 * j, q0, head, batch);
      for (int t = 0; t < T && !failed; ++t) {
        const int sb = t & 1;
        if (t >= 2 && !mbar_wait(&k_empty[sb], ((t - 2) >> 1) & 1, abort_flag)) { failed = true; break; }
        mbar_expect_tx(&k_full[sb], SM::kTile);
        for (int j = 0; j < KBD; ++j)
          tma_load_4d(base + SM::kK + sb * SM::kTile + j * kBox, &a.k, &k_full[sb], 64 * j, kv_lo + t * 128, head, batch);
        if (t >= 2 && !mbar_wait(&pv_done[sb], ((t - 2) >> 1) & 1, abort_flag)) { failed = true; break; }
        mbar_expect_tx(&v_full[sb], SM::kTile);
        for (int j = 0; j < KBD; ++j)
          tma_load_4d(base + SM::kV + sb * SM::kTile + j * kBox, &a.v, &v_full[sb], 64 * j, kv_lo + t * 128, head, batch);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && !failed) {
      const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_o = make_idesc_bf16(128, HD, 0, 1);
      auto issue_s = [&](int u) -> bool {
        const int sb = u & 1;
        if (!mbar_wait(&k_full[sb], (u >> 1) & 1, abort_flag)) return false;
        if (u >= 2 && !mbar_wait(&s_empty[sb], ((u - 2) >> 1) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t qa = base + SM::kQ, kb = base + SM::kK + sb * SM::kTile;
#pragma unroll
        for (int kk = 0; kk < KBD; ++kk)
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4)
            umma_bf16(tmem + sb * 128, make_smem_desc(qa + kk * kBox + k4 * 32, 0, 1024),
                      make_smem_desc(kb + kk * kBox + k4 * 32, 0, 1024), idesc_s, (kk | k4) != 0);
        umma_commit(&s_full[sb]);
        umma_commit(&k_empty[sb]);
        return true;
      };
      if (!mbar_wait(q_full, 0, abort_flag)) failed = true;
      for (int t = 0; t < T && !failed; ++t) {
        const int sb = t & 1;
        if (t == 0 && !issue_s(0)) { failed = true; break; }
        if (t + 1 < T && !issue_s(t + 1)) { failed = true; break; }
        if (!mbar_wait(&p_full[sb], (t >> 1) & 1, abort_flag) || !mbar_wait(&v_full[sb], (t >> 1) & 1, abort_flag) ||
            (t >= 2 && !mbar_wait(&o_empty[sb], ((t - 2) >> 1) & 1, abort_flag))) {
          failed = true;
          break;
        }
        tc_fence_after();
        const uint32_t pa = base + SM::kP + sb * SM::kPTile, vb = base + SM::kV + sb * SM::kTile;
        // A = probabilities, K-major over the 128 keys (two 64-key panels); B = values, MN-major: atoms of 64
        // features, each [128 key rows][64] (one box), 16 key rows = 2048 bytes per MMA step
#pragma unroll
        for (int kk = 0; kk < 2; ++kk)
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4)
            umma_bf16(tmem + 256 + sb * HD, make_smem_desc(pa + kk * kBox + k4 * 32, 0, 1024),
                      make_smem_desc(vb + kk * kAtomBytes + k4 * 2048, kBox, 1024), idesc_o, (kk | k4) != 0);
        umma_commit(&pv_done[sb]);
      }
    }
  } else {
    // ---------------- softmax: two threads per query row (warps w and w + 4 share a tensor-memory lane quarter):
    // thread `half` owns keys [64 half, 64 half + 64) of every S tile and output features [HD/2 half, HD/2 (half + 1))
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const int qi = q0 + r;
    const int row_start = (a.seq_start != nullptr && qi < a.L) ? a.seq_start[qi] : 0;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    constexpr int OC = HD / 2;   // output features per thread
    float m = -INFINITY, l = 0.f, a_prev = 1.f;
    float O[OC];
#pragma unroll
    for (int j = 0; j < OC; ++j) O[j] = 0.f;
    // the two threads of a row swap a value through shared memory; the two warps of a lane quarter meet at a named
    // barrier of their own.  A named barrier has no time limit, so EVERY softmax thread runs every exchange of every
    // iteration, also after one of its bounded waits has run out (it then skips the work, never the barriers).
    auto exchange = [&](float mine) -> float {
      xch[half * 128 + r] = mine;
      named_barrier_sync(1 + quarter, 64);
      const float other = xch[(half ^ 1) * 128 + r];
      named_barrier_sync(1 + quarter, 64);
      return other;
    };
    auto fold = [&](int u, float alpha) -> bool {   // O <- O * alpha + O_u (this thread's features)
      const int ob = u & 1;
      if (!mbar_wait(&pv_done[ob], (u >> 1) & 1, abort_flag)) return false;
      tc_fence_after();
      const uint32_t o_addr = tmem + lane_off + 256 + ob * HD + half * OC;
      uint32_t ba[32];
#pragma unroll
      for (int c = 0; c < OC; c += 32) {
        tmem_ld32(o_addr + c, ba);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) O[c + j] = fmaf(O[c + j], alpha, __uint_as_float(ba[j]));
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&o_empty[ob]);
      return true;
    };
    for (int t = 0; t < T; ++t) {
      const int sb = t & 1;
      const int kv0 = kv_lo + t * 128;
      if (!failed && !mbar_wait(&s_full[sb], (t >> 1) & 1, abort_flag)) {
        failed = true;
        *abort_flag = 1;
      }
      // every (row, key) pair of the tile inside the band and the sequence: no masks
      const bool interior = a.causal ? (kv0 + 127 <= q0 && kv0 >= q0 + 127 - (window - 1) && kv0 + 127 < a.L && kv0 >= tile_start)
                                     : kv0 + 127 < a.Lk;
      const int c0 = half * 64;                                // this thread's first key column of the tile
      // last / first column of the tile this row may see
      const int j_hi = (a.causal ? (qi < a.L - 1 ? qi : a.L - 1) : a.Lk - 1) - kv0;
      const int j_lo = (a.causal ? (qi - (window - 1) > row_start ? qi - (window - 1) : row_start) : 0) - kv0;
      const uint32_t s_addr = tmem + lane_off + sb * 128 + c0;
      uint32_t ba[32], bb[32];   // this thread's 64 scores: read once, kept across the exchange of the row maximum
      float mx = -INFINITY;
      if (!failed) {
        tc_fence_after();
        tmem_ld32(s_addr, ba);
        tmem_ld32(s_addr + 32, bb);
        tmem_ld_wait();
        if (interior) {
#pragma unroll
          for (int j = 0; j < 32; ++j) mx = fmaxf(mx, fmaxf(__uint_as_float(ba[j]), __uint_as_float(bb[j])));
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (c0 + j >= j_lo && c0 + j <= j_hi) mx = fmaxf(mx, __uint_as_float(ba[j]));
            if (c0 + 32 + j >= j_lo && c0 + 32 + j <= j_hi) mx = fmaxf(mx, __uint_as_float(bb[j]));
          }
        }
      }
      mx = fmaxf(mx, exchange(mx));
      if (failed) continue;
      const float m_new = fmaxf(m, mx * a.scale_log2);
      const float alpha = m_new == -INFINITY ? 1.f : fast_exp2(m - m_new);
      const float shift = m_new == -INFINITY ? 0.f : m_new;
      float sum = 0.f;
      const uint32_t p_row = base + SM::kP + sb * SM::kPTile + half * kBox + r * 128;   // this thread's 64-key panel
      auto exp_chunk = [&](const uint32_t (&bits)[32], int c, const bool masked) {
        const uint32_t unit0 = (c & 63) >> 3;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float p[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int j = g * 8 + e;
            const float x = fast_exp2(fmaf(__uint_as_float(bits[j]), a.scale_log2, -shift));
            p[e] = (!masked || (c + j >= j_lo && c + j <= j_hi)) ? x : 0.f;
            sum += p[e];
          }
          const uint32_t addr = p_row + (((unit0 + g) ^ (r & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pack_bf16x2(p[0], p[1])),
                       "r"(pack_bf16x2(p[2], p[3])), "r"(pack_bf16x2(p[4], p[5])), "r"(pack_bf16x2(p[6], p[7]))
                       : "memory");
        }
      };
      if (interior) {   // (two copies of the loop: the mask tests vanish from this one)
        exp_chunk(ba, c0, false);
        exp_chunk(bb, c0 + 32, false);
      } else {
        exp_chunk(ba, c0, true);
        exp_chunk(bb, c0 + 32, true);
      }
      // S has been read and is free; the probabilities are visible to the tensor core
      tc_fence_before();
      fence_async_proxy();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s_empty[sb]);
        mbar_arrive(&p_full[sb]);
      }
      l = l * alpha + sum;   // this thread's share of the row sum (both shares see the same alphas)
      m = m_new;
      if (t >= 1 && !fold(t - 1, a_prev)) {
        failed = true;
        *abort_flag = 1;
      }
      a_prev = alpha;
    }
    if (!failed && T > 0 && !fold(T - 1, a_prev)) failed = true;
    const float l_other = exchange(l);
    if (!failed && qi < a.L) {
      const float tot = l + l_other;
      const float inv = tot > 0.f ? 1.0f / tot : 0.f;
      if (a.lse != nullptr && half == 0) a.lse[(static_cast<int64_t>(batch) * a.heads + head) * a.L + qi] = m + log2f(tot);
      bf16* dst = a.o + batch * a.o_bs + static_cast<int64_t>(qi) * a.o_ts + head * a.o_hs + half * OC;
#pragma unroll
      for (int c = 0; c < OC; c += 8) {
        uint4 u;
        u.x = pack_bf16x2(O[c] * inv, O[c + 1] * inv);
        u.y = pack_bf16x2(O[c + 2] * inv, O[c + 3] * inv);
        u.z = pack_bf16x2(O[c + 4] * inv, O[c + 5] * inv);
        u.w = pack_bf16x2(O[c + 6] * inv, O[c + 7] * inv);
        *reinterpret_cast<uint4*>(dst + c) = u;
      }
    }
  }
  // a wait that ran out: raise the flag so the other roles stop, record the status
  if (failed && *reinterpret_cast<volatile int32_t*>(a.status) == kStatusOk) {
    *abort_flag = 1;
    atomicCAS(a.status, kStatusOk, kStatusWaitTimeout);
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    for (int i = 0; i < 256; ++i) __nanosleep(1000);  // bulk copies still in flight land before shared memory goes
  }
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace lact
