// Flash-style attention backward for head dimension 64, pipelined over the two halves of a query
// tile.  One CTA owns one (batch, head, 128-row K/V tile) and streams the 128-row query tiles
// that attend to it, in the transposed orientation (K/V rows on the tensor-memory lanes):
//   S^T  = K_j . Q_i^T          dP^T = V_j . dO_i^T
//   P^T  = exp2(S^T * c - LSE_i)       dS^T = P^T o (dP^T - delta_i)
//   dV_j += P^T . dO_i          dK_j += dS^T . Q_i          dQ_i = dS . K_j
// What distinguishes it from the generic kernel (attention_bwd.cu):
//  * a query tile is handled as two halves of 64 query columns, each with its own S^T / dP^T
//    columns in tensor memory and its own softmax warpgroup; while one half's products and next
//    scores run on the tensor cores the other half's softmax runs, so neither side idles for the
//    whole length of the other;
//  * P^T and dS^T are written back as packed bf16 over their own score columns in tensor memory
//    and feed dV and dK as tensor-memory A operands: no shared-memory round trip for P^T at all,
//    dS^T goes to shared memory only for dQ (where it is the transposed operand);
//  * dQ is double-buffered in tensor memory, so its drain (bulk reduce-adds into the fp32
//    accumulation buffer shared by all K/V tiles) overlaps the next tile;
//  * the tensor pipe executes one thread's MMAs in issue order, which is what lets the scores of
//    tile i+1 overwrite the columns P^T / dS^T of tile i were read from without a barrier.
//   warp 0        TMA producer (K_j, V_j once; Q_i, dO_i through a 3-stage ring)
//   warp 1        MMA issuer          (warps 2, 3 idle: register donors)
//   warps 4..7    softmax / dS of the first half; afterwards the dV epilogue
//   warps 8..11   softmax / dS of the second half; afterwards the dK epilogue
//   warps 12..15  dQ drain (TMEM -> shared memory -> bulk reduce-add into the fp32 accumulator)
// delta_i = rowsum(dO_i o O_i) comes from a pre-kernel, a post-kernel scales and casts dQ (both in
// attention_bwd.cu).  The reference (plugins/model-transformer/src/lib.rs:300-372) computes the
// attention gradient on the CPU in fp32 with materialised probabilities.
#include <climits>

#include "attention_bwd.cuh"
#include "common.cuh"
#include "ptx.cuh"

namespace cb {
namespace {

struct B64 {
  static constexpr int DH = 64, BQ = 128, BKV = 128, HQ = 64;
  static constexpr int THREADS = 512;
  static constexpr int NST = 3;                           // Q_i / dO_i stages
  static constexpr int KV_BYTES = BKV * DH * 2;           // K_j or V_j
  static constexpr int Q_BYTES = BQ * DH * 2;             // Q_i or dO_i
  static constexpr int ST_BYTES = 2 * Q_BYTES;            // one stage: Q_i | dO_i
  static constexpr int DST_BYTES = BKV * BQ * 2;          // dS^T of one tile
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = KV_BYTES;
  static constexpr int OFF_Q = 2 * KV_BYTES;
  static constexpr int OFF_DST = OFF_Q + NST * ST_BYTES;  // two buffers (tile parity)
  static constexpr int OFF_DQS = OFF_DST + 2 * DST_BYTES;   // dQ staging: per drain warp two boxes
                                                            // of [32 rows][32 floats], swizzled
  static constexpr int DQS_BYTES = BQ * DH * 4;
  static constexpr int OFF_STAT = OFF_DQS + DQS_BYTES;      // [2 parities][lse | delta][BQ] floats
  static constexpr int OFF_BAR = OFF_STAT + 2 * 2 * BQ * 4;
  static constexpr int SMEM_BYTES = OFF_BAR + 256;
  static_assert(SMEM_BYTES <= 232448, "attention backward: shared memory budget");
  // tensor-memory columns: per half h, S^T at 128 h (P^T over its first 32 columns) and dP^T at
  // 128 h + 64 (dS^T over its first 32); then dV, dK and two dQ buffers
  static constexpr int DV_COL = 256, DK_COL = 320, DQ_COL = 384;
  static constexpr int TMEM_COLS = 512;
  enum {
    B_KV = 0,
    B_QF = 1,                // + stage: Q_i / dO_i landed
    B_QE = B_QF + NST,       // + stage: stage free
    B_SF = B_QE + NST,       // + half: S^T / dP^T of the half complete
    B_PF = B_SF + 2,         // + half: P^T / dS^T of the half written (4 warps)
    B_STF = B_PF + 2,        // + half: the half's lse / delta in shared memory (4 warps)
    B_DF = B_STF + 2,        // + parity: dS^T buffer free (its dQ product completed)
    B_DQF = B_DF + 2,        // + parity: dQ complete in tensor memory
    B_DQE = B_DQF + 2,       // + parity: dQ drained (4 warps)
    B_DONE = B_DQE + 2,
    N_BARS
  };
  static_assert(N_BARS * 8 + 8 <= 256, "barrier block");
};

// One 32-column chunk of a half: p = exp2(s c - lse), ds = p (dp - delta), both packed to bf16.
// `lim` > query index hides the element (causal mask and rows beyond the sequence).
template <bool MASK>
__device__ __forceinline__ void bwd_chunk(const uint32_t* sv, const uint32_t* dv,
                                          const float* s_lse, const float* s_dl, float c, int lim,
                                          int q_first, uint32_t* pk, uint32_t* dk) {
#pragma unroll
  for (int e = 0; e < 32; e += 4) {
    const float4 L = *reinterpret_cast<const float4*>(s_lse + e);
    const float4 D = *reinterpret_cast<const float4*>(s_dl + e);
    float p0 = fast_exp2(fmaf(__uint_as_float(sv[e]), c, -L.x));
    float p1 = fast_exp2(fmaf(__uint_as_float(sv[e + 1]), c, -L.y));
    float p2 = fast_exp2(fmaf(__uint_as_float(sv[e + 2]), c, -L.z));
    float p3 = fast_exp2(fmaf(__uint_as_float(sv[e + 3]), c, -L.w));
    if (MASK) {
      if (lim > q_first + e) p0 = 0.f;
      if (lim > q_first + e + 1) p1 = 0.f;
      if (lim > q_first + e + 2) p2 = 0.f;
      if (lim > q_first + e + 3) p3 = 0.f;
    }
    const float d0 = p0 * (__uint_as_float(dv[e]) - D.x);
    const float d1 = p1 * (__uint_as_float(dv[e + 1]) - D.y);
    const float d2 = p2 * (__uint_as_float(dv[e + 2]) - D.z);
    const float d3 = p3 * (__uint_as_float(dv[e + 3]) - D.w);
    pk[e >> 1] = pack_bf16x2(p0, p1);
    pk[(e >> 1) + 1] = pack_bf16x2(p2, p3);
    dk[e >> 1] = pack_bf16x2(d0, d1);
    dk[(e >> 1) + 1] = pack_bf16x2(d2, d3);
  }
}

__global__ void __launch_bounds__(B64::THREADS, 1)
attn_bwd_dh64_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                     const __grid_constant__ CUtensorMap tmDQ, const AttnBwdArgs p) {
  using C = B64;
  constexpr int DH = C::DH, BQ = C::BQ, BKV = C::BKV, HQ = C::HQ, NST = C::NST;
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + C::N_BARS);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  auto bar = [&](int i) { return smem_u32(bars + i); };
  float* s_stat = reinterpret_cast<float*>(smem + C::OFF_STAT);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if ((sbase & 1023u) != 0u) {
    if (threadIdx.x == 0) record_status(p.status, ST_BAD_ARG, 1100);
    return;
  }
  const int bh = blockIdx.x % (p.B * p.nh);
  const int j = blockIdx.x / (p.B * p.nh);  // early K/V tiles see the most queries: first
  const int b = bh / p.nh, h = bh % p.nh;
  const int kv0 = j * BKV;
  const int n_q_tiles = (p.S + BQ - 1) / BQ;
  const int i_start = p.causal ? j : 0;      // BQ == BKV
  const int n_it = n_q_tiles - i_start;

  if (threadIdx.x == 0) {
    mbar_init(bar(C::B_KV), 1);
    for (int s = 0; s < NST; ++s) {
      mbar_init(bar(C::B_QF + s), 1);
      mbar_init(bar(C::B_QE + s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(C::B_SF + s), 1);
      mbar_init(bar(C::B_PF + s), 4);      // one arrival per softmax warp of the half
      mbar_init(bar(C::B_STF + s), 4);
      mbar_init(bar(C::B_DF + s), 1);
      mbar_init(bar(C::B_DQF + s), 1);
      mbar_init(bar(C::B_DQE + s), 4);     // one arrival per dQ-drain warp
    }
    mbar_init(bar(C::B_DONE), 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmdO);
    tma_prefetch_desc(&tmDQ);
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t sK = sbase + C::OFF_K, sV = sbase + C::OFF_V;
  auto sDST = [&](int buf) { return sbase + C::OFF_DST + buf * C::DST_BYTES; };
  auto sQ = [&](int st) { return sbase + C::OFF_Q + st * C::ST_BYTES; };
  auto sDO = [&](int st) { return sQ(st) + C::Q_BYTES; };
  const int row0 = b * p.S;

  // 512 threads start with 128 registers each.  The first warpgroup (producer, MMA issue) and the
  // dQ-drain warpgroup hand registers to the two softmax warpgroups, which keep both chunks of a
  // half (S^T and dP^T, 128 values) in flight: 128 * (56 + 88 + 184 + 184) = 65536.
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;" ::: "memory");
    if (warp == 0) {
      // -------------------------------------------------------------- producer
      if (lane == 0) {
        mbar_arrive_expect_tx(bar(C::B_KV), 2 * C::KV_BYTES);
        tma_load_2d(sK, &tmK, bar(C::B_KV), h * DH, row0 + kv0);
        tma_load_2d(sV, &tmV, bar(C::B_KV), h * DH, row0 + kv0);
        int issued = 0;
        for (int it = 0; it < n_it; ++it) {
          const int st = it % NST;
          if (!mbar_wait(bar(C::B_QE + st), ((it / NST) & 1u) ^ 1u, abort_flag)) {
            record_status(p.status, ST_WAIT_TIMEOUT, 1110);
            break;
          }
          const int qrow = row0 + (i_start + it) * BQ;
          mbar_arrive_expect_tx(bar(C::B_QF + st), C::ST_BYTES);
          tma_load_2d(sQ(st), &tmQ, bar(C::B_QF + st), h * DH, qrow);
          tma_load_2d(sDO(st), &tmdO, bar(C::B_QF + st), h * DH, qrow);
          ++issued;
        }
        if (*abort_flag) {
          // let the copies already in flight land before shared memory is released
          const uint64_t t0 = globaltimer_ns();
          for (int i = max(0, issued - NST); i < issued; ++i) {
            while (!mbar_try_wait(bar(C::B_QF + i % NST), (i / NST) & 1u)) {
              if (globaltimer_ns() - t0 > 200000000ull) break;
            }
          }
          while (!mbar_try_wait(bar(C::B_KV), 0)) {
            if (globaltimer_ns() - t0 > 200000000ull) break;
          }
        }
      }
      __syncwarp();
    } else if (warp == 1) {
      // -------------------------------------------------------------- MMA issuer
      // The whole warp runs the control flow (addresses and descriptors stay warp-uniform); one
      // elected lane issues.  Descriptors are built once; a product only adds constants to their
      // address field.
      constexpr uint32_t idesc_sc = umma_idesc_bf16(BKV, HQ, 0, 0);   // S^T, dP^T of a half
      constexpr uint32_t idesc_pv = umma_idesc_bf16(BKV, DH, 0, 1);   // dV, dK (A in tensor memory)
      constexpr uint32_t idesc_dq = umma_idesc_bf16(BQ, DH, 1, 1);    // dQ
      const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
      const uint64_t dK_k = umma_desc_sw128(sK, 16, 1024), dV_k = umma_desc_sw128(sV, 16, 1024);
      const uint64_t dK_mn = umma_desc_sw128(sK, BKV * 128, 1024);
      const uint64_t dQ_k0 = umma_desc_sw128(sQ(0), 16, 1024);
      const uint64_t dDO_k0 = umma_desc_sw128(sDO(0), 16, 1024);
      const uint64_t dQ_mn0 = umma_desc_sw128(sQ(0), BQ * 128, 1024);
      const uint64_t dDO_mn0 = umma_desc_sw128(sDO(0), BQ * 128, 1024);
      const uint64_t dDST_mn0 = umma_desc_sw128(sDST(0), BKV * 128, 1024);
      constexpr uint64_t ST_STEP = C::ST_BYTES >> 4;       // stage pitch
      constexpr uint64_t BUF_STEP = C::DST_BYTES >> 4;     // dS^T buffer pitch
      constexpr uint64_t HALF_STEP = (HQ * 128) >> 4;      // 64 query rows further in a Q / dO tile
      auto wait_all = [&](int b_idx, uint32_t parity, int where) {
        const bool got = mbar_wait(bar(b_idx), parity, abort_flag);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0) record_status(p.status, ST_WAIT_TIMEOUT, where);
          return false;
        }
        return true;
      };
      // S^T and dP^T of half hf of the tile in stage st (K-major operands, contraction over dh)
      auto scores = [&](int hf, int st) {
        const uint64_t bq = dQ_k0 + st * ST_STEP + hf * HALF_STEP;
        const uint64_t bdo = dDO_k0 + st * ST_STEP + hf * HALF_STEP;
        const uint32_t s_col = tmem_u + hf * 128, d_col = s_col + 64;
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
          umma_bf16_ss(s_col, dK_k + 2 * kk, bq + 2 * kk, idesc_sc, kk > 0 ? 1u : 0u);
          umma_bf16_ss(d_col, dV_k + 2 * kk, bdo + 2 * kk, idesc_sc, kk > 0 ? 1u : 0u);
        }
        umma_commit(bar(C::B_SF + hf));
      };
      // dV += P^T . dO and dK += dS^T . Q over the 64 query rows of half hf
      auto products = [&](int hf, int st, uint32_t acc0) {
        const uint64_t bdo = dDO_mn0 + st * ST_STEP + hf * HALF_STEP;
        const uint64_t bq = dQ_mn0 + st * ST_STEP + hf * HALF_STEP;
        const uint32_t pt = tmem_u + hf * 128, dst = pt + 64;
#pragma unroll
        for (int kk = 0; kk < HQ / 16; ++kk) {
          umma_bf16_ts(tmem_u + C::DV_COL, pt + kk * 8, bdo + 128 * kk, idesc_pv, kk > 0 ? 1u : acc0);
          umma_bf16_ts(tmem_u + C::DK_COL, dst + kk * 8, bq + 128 * kk, idesc_pv, kk > 0 ? 1u : acc0);
        }
      };
      long long* trace = (blockIdx.x == 0 && lane == 0) ? p.trace : nullptr;
      bool ok = wait_all(C::B_KV, 0, 1120);
      if (ok) ok = wait_all(C::B_QF, 0, 1121);
      if (ok) {
        tc_fence_after();
        if (elect_one()) {
          scores(0, 0);
          scores(1, 0);
        }
        __syncwarp();
      }
      for (int it = 0; it < n_it && ok; ++it) {
        const int st = it % NST, buf = it & 1;
        const int nst = (it + 1) % NST;
        const bool more = it + 1 < n_it;
        // ---- first half: its products, then the next tile's scores over the same columns
        if (!wait_all(C::B_PF + 0, it & 1u, 1122)) { ok = false; break; }
        if (more && !wait_all(C::B_QF + nst, ((it + 1) / NST) & 1u, 1123)) { ok = false; break; }
        tc_fence_after();
        if (trace && it < 16) trace[it * 16 + 6] = clock64();
        if (elect_one()) {
          products(0, st, it > 0 ? 1u : 0u);
          if (more) scores(0, nst);
        }
        __syncwarp();
        if (trace && it < 16) trace[it * 16 + 7] = clock64();
        // ---- second half
        if (!wait_all(C::B_PF + 1, it & 1u, 1124)) { ok = false; break; }
        tc_fence_after();
        if (trace && it < 16) trace[it * 16 + 8] = clock64();
        if (elect_one()) {
          products(1, st, 1u);
          umma_commit(bar(C::B_QE + st));        // Q_i / dO_i stage free
          if (more) scores(1, nst);
        }
        __syncwarp();
        if (trace && it < 16) trace[it * 16 + 9] = clock64();
        // ---- dQ_i = dS . K_j over the whole tile, into the dQ buffer of this parity
        if (it >= 2) {
          if (!wait_all(C::B_DQE + buf, ((it >> 1) - 1) & 1u, 1125)) { ok = false; break; }
          tc_fence_after();
        }
        if (trace && it < 16) trace[it * 16 + 10] = clock64();
        if (elect_one()) {
          const uint64_t a = dDST_mn0 + buf * BUF_STEP;
          const uint32_t d = tmem_u + C::DQ_COL + buf * DH;
#pragma unroll
          for (int kk = 0; kk < BKV / 16; ++kk)
            umma_bf16_ss(d, a + 128 * kk, dK_mn + 128 * kk, idesc_dq, kk > 0 ? 1u : 0u);
          umma_commit(bar(C::B_DQF + buf));
          umma_commit(bar(C::B_DF + buf));
        }
        __syncwarp();
        if (trace && it < 16) trace[it * 16 + 11] = clock64();
      }
      if (ok && elect_one()) umma_commit(bar(C::B_DONE));
      __syncwarp();
    }
  } else if (warp < 12) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 184;" ::: "memory");
    // ---------------------------------------------------------------- softmax / dS of one half
    const int hf = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;        // K/V row within the tile = tensor-memory lane
    const int kv_idx = kv0 + r;
    const int gt = threadIdx.x - 128 - hf * 128;   // 0..127 within the half's warpgroup
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t s_addr = lane_addr + hf * 128, d_addr = s_addr + 64;
    const size_t stat_base = (static_cast<size_t>(b) * p.nh + h) * p.S;
    const float c = p.scale_log2;
    // the thread's share of a tile's statistics: lse (times log2 e) of one query column for the
    // first 64 threads, delta of one column for the others
    auto load_stat = [&](int it) {
      const int qi = (i_start + it) * BQ + hf * HQ + (gt & 63);
      if (gt < 64) return qi < p.S ? p.lse[stat_base + qi] * 1.4426950408889634f : INFINITY;
      return qi < p.S ? p.delta[stat_base + qi] : 0.f;
    };
    float stat_next = load_stat(0);
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int q0 = (i_start + it) * BQ;
      float* s_lse = s_stat + (it & 1) * 2 * BQ + hf * HQ;
      float* s_dl = s_lse + BQ;
      (gt < 64 ? s_lse : s_dl)[gt & 63] = stat_next;
      if (it + 1 < n_it) stat_next = load_stat(it + 1);   // lands during this tile's work
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(C::B_STF + hf));
      bool got = mbar_wait(bar(C::B_STF + hf), it & 1u, abort_flag);
      if (got) got = mbar_wait(bar(C::B_SF + hf), it & 1u, abort_flag);
      // the dS^T buffer of this parity was last read by the dQ product of tile it - 2
      if (got && it > 1) got = mbar_wait(bar(C::B_DF + (it & 1)), ((it >> 1) - 1) & 1u, abort_flag);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) record_status(p.status, ST_WAIT_TIMEOUT, 1130);
        ok = false;
        break;
      }
      tc_fence_after();
      long long* tr = (blockIdx.x == 0 && it < 16 && quarter == 0 && lane == 0) ? p.trace : nullptr;
      if (tr) tr[it * 16 + hf * 3] = clock64();
      const bool mask = (p.causal && kv0 + BKV - 1 > q0) || (kv0 + BKV > p.S);
      const int lim = kv_idx >= p.S ? INT_MAX : (p.causal ? kv_idx : INT_MIN);
      // dS^T in shared memory: two groups of 64 query columns, each [128 K/V rows][128 bytes],
      // 128-byte swizzled (the layout the dQ product reads as a transposed A operand)
      const uint32_t srow = sDST(it & 1) + hf * (BKV * 128) + r * 128;
      uint32_t s0[32], d0[32], s1[32], d1[32];
      tmem_ld_32x32b_x32(s_addr, s0);
      tmem_ld_32x32b_x32(d_addr, d0);
      tmem_ld_wait();
      tmem_ld_32x32b_x32(s_addr + 32, s1);     // in flight during the first chunk's arithmetic
      tmem_ld_32x32b_x32(d_addr + 32, d1);
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        uint32_t pk[16], dk[16];
        const uint32_t* sv = ch ? s1 : s0;
        const uint32_t* dv = ch ? d1 : d0;
        if (ch) tmem_ld_wait();
        if (mask)
          bwd_chunk<true>(sv, dv, s_lse + ch * 32, s_dl + ch * 32, c, lim, q0 + hf * HQ + ch * 32, pk, dk);
        else
          bwd_chunk<false>(sv, dv, s_lse + ch * 32, s_dl + ch * 32, c, lim, 0, pk, dk);
        tmem_st_32x32b_x16(s_addr + ch * 16, pk);
        tmem_st_32x32b_x16(d_addr + ch * 16, dk);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const uint32_t sw = static_cast<uint32_t>((ch * 4 + g) ^ (r & 7)) << 4;
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(srow + sw),
                       "r"(dk[4 * g]), "r"(dk[4 * g + 1]), "r"(dk[4 * g + 2]), "r"(dk[4 * g + 3])
                       : "memory");
        }
      }
      if (tr) tr[it * 16 + hf * 3 + 1] = clock64();
      tmem_st_wait();
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(C::B_PF + hf));
      if (tr) tr[it * 16 + hf * 3 + 2] = clock64();
    }
    // ---- epilogue: dV (first half's warps) and dK (second half's) of this K/V tile
    if (ok) {
      const bool got = mbar_wait(bar(C::B_DONE), 0, abort_flag);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) record_status(p.status, ST_WAIT_TIMEOUT, 1131);
        ok = false;
      }
    }
    if (ok) {
      tc_fence_after();
      const bool row_ok = kv_idx < p.S;
      const size_t orow = (static_cast<size_t>(row0) + kv_idx) * p.ldd + static_cast<size_t>(h) * DH;
      __nv_bfloat16* dst = (hf == 0 ? p.dv : p.dk) + orow;
      const float mul = hf == 0 ? 1.0f : p.scale;
      const int col = hf == 0 ? C::DV_COL : C::DK_COL;
#pragma unroll 1
      for (int ch = 0; ch < DH / 32; ++ch) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(lane_addr + col + ch * 32, o);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(o[8 * g + 0]) * mul, __uint_as_float(o[8 * g + 1]) * mul);
            w.y = pack_bf16x2(__uint_as_float(o[8 * g + 2]) * mul, __uint_as_float(o[8 * g + 3]) * mul);
            w.z = pack_bf16x2(__uint_as_float(o[8 * g + 4]) * mul, __uint_as_float(o[8 * g + 5]) * mul);
            w.w = pack_bf16x2(__uint_as_float(o[8 * g + 6]) * mul, __uint_as_float(o[8 * g + 7]) * mul);
            *reinterpret_cast<uint4*>(dst + ch * 32 + g * 8) = w;
          }
        }
      }
    }
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 88;" ::: "memory");
    // ---------------------------------------------------------------- dQ drain
    // Each warp moves its 32 query rows on its own: tensor memory -> registers -> a swizzled
    // staging tile in shared memory -> bulk reduce-add into the fp32 accumulator (whole 128-byte
    // lines added in L2, against 32 separate 16-byte atomics per instruction from registers,
    // which kept the load/store pipe busy a third of the time).  Rows beyond the sequence are
    // dropped by the tensor map's bounds.
    const int quarter = warp & 3;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t stage = sbase + C::OFF_DQS + quarter * (C::DQS_BYTES / 4);
    const uint32_t srow = stage + lane * 128;
    bool pending = false;
    for (int it = 0; it < n_it; ++it) {
      const int buf = it & 1;
      const bool got = mbar_wait(bar(C::B_DQF + buf), (it >> 1) & 1u, abort_flag);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) record_status(p.status, ST_WAIT_TIMEOUT, 1140);
        break;
      }
      tc_fence_after();
      long long* trq = (blockIdx.x == 0 && it < 16 && quarter == 0 && lane == 0) ? p.trace : nullptr;
      if (trq) trq[it * 16 + 12] = clock64();
      uint32_t o0[32], o1[32];
      tmem_ld_32x32b_x32(lane_addr + C::DQ_COL + buf * DH, o0);
      tmem_ld_32x32b_x32(lane_addr + C::DQ_COL + buf * DH + 32, o1);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bar(C::B_DQE + buf));               // the tensor-memory buffer is free again
        if (pending) tma_store_wait_read_all();         // ... and so is the staging tile
      }
      __syncwarp();
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        const uint32_t sw = static_cast<uint32_t>(g ^ (lane & 7)) << 4;
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(srow + sw), "r"(o0[4 * g]),
                     "r"(o0[4 * g + 1]), "r"(o0[4 * g + 2]), "r"(o0[4 * g + 3]) : "memory");
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(srow + 4096 + sw),
                     "r"(o1[4 * g]), "r"(o1[4 * g + 1]), "r"(o1[4 * g + 2]), "r"(o1[4 * g + 3])
                     : "memory");
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        const int qrow = (i_start + it) * BQ + quarter * 32;
        if (qrow < p.S) {
          tma_reduce_add_3d(&tmDQ, stage, h * DH, qrow, b);
          tma_reduce_add_3d(&tmDQ, stage + 4096, h * DH + 32, qrow, b);
          tma_store_commit();
          pending = true;
        }
      }
      if (trq) trq[it * 16 + 13] = clock64();
    }
    if (lane == 0 && pending) tma_store_wait_all();
    __syncwarp();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

}  // namespace

int launch_attn_bwd_dh64(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                         const CUtensorMap& tdo, const CUtensorMap& tdq, const AttnBwdArgs& a,
                         cudaStream_t st) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_bwd_dh64_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             B64::SMEM_BYTES) != cudaSuccess)
      return -10;
    configured = true;
  }
  const int n_kv_tiles = (a.S + B64::BKV - 1) / B64::BKV;
  attn_bwd_dh64_kernel<<<n_kv_tiles * a.B * a.nh, B64::THREADS, B64::SMEM_BYTES, st>>>(
      tq, tk, tv, tdo, tdq, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace cb
