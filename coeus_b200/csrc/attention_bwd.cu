// Flash-style attention backward on tcgen05.  One CTA owns one (batch, head, 128-row K/V tile)
// and streams the query tiles that attend to it; all five products run on the tensor cores
// with accumulators in tensor memory, in the transposed orientation (K/V rows on the TMEM lanes)
// so that P^T and dS^T are produced row-per-thread and feed the next MMAs from shared memory:
//   S^T  = K_j . Q_i^T          dP^T = V_j . dO_i^T
//   P^T  = exp2(S^T * c - LSE_i)       dS^T = P^T o (dP^T - delta_i)
//   dV_j += P^T . dO_i          dK_j += dS^T . Q_i
//   dQ_i  = dS . K_j  (dh = 64; for dh = 128 the transposed dQ_i^T = K_j^T . dS^T), drained from
//           TMEM with fp32 atomic adds into an accumulation buffer shared by all K/V tiles.
// delta_i = rowsum(dO_i o O_i) comes from a small pre-kernel; a post-kernel scales and casts dQ.
//   warp 0      TMA producer (K_j, V_j once; Q_i, dO_i through a 2-stage ring)
//   warp 1      MMA issuer
//   warps 2..9   softmax / dS: two threads per K/V row, each taking half of the query columns
//                (warps 2..5 the first half, 6..9 the second); afterwards the dV (first group)
//                and dK (second group) epilogue
//   warps 10..13 dQ drain (TMEM -> red.global.add)
#include <algorithm>

#include "attention_bwd.cuh"
#include "common.cuh"
#include "ptx.cuh"

namespace cb {

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                      uint64_t ld, uint32_t box_inner, uint32_t box_outer);
int make_tmap_f32_3d(CUtensorMap* out, void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                     uint64_t ld1, uint64_t ld2, uint32_t box1);
int make_tmap_bf16_3d(CUtensorMap* out, void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                      uint64_t ld1, uint64_t ld2, uint32_t box1);
int sm_count();

constexpr int ATB_BKV = 128;
constexpr int ATB_THREADS = 448;

// Optional timeline of block 0 (a debugging aid; off unless a trace buffer is registered):
// [it][0..11] = clock64 at: softmax S^T/dP^T ready, after the first TMEM load, after the maths of
// both chunks, after the fence+arrive; MMA thread: stage ready, S^T/dP^T issued, P^T ready,
// dV/dK/dQ issued; dQ drain: start, end; MMA thread: previous dQ drained.
static long long* g_attn_bwd_trace_host = nullptr;

template <int DH>
struct AttnBwdCfg {
  static constexpr int BQ = (DH == 64) ? 128 : 64;
  static constexpr int KV_BYTES = ATB_BKV * DH * 2;     // K_j or V_j
  static constexpr int Q_BYTES = BQ * DH * 2;           // Q_i or dO_i
  static constexpr int PT_BYTES = ATB_BKV * BQ * 2;     // P^T or dS^T
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = KV_BYTES;
  static constexpr int OFF_Q = 2 * KV_BYTES;                    // 2 stages of (Q_i | dO_i)
  static constexpr int OFF_PT = OFF_Q + 2 * 2 * Q_BYTES;        // two buffers of P^T ...
  static constexpr int OFF_DST = OFF_PT + 2 * PT_BYTES;         // ... and of dS^T: the softmax of
                                                                // tile i+1 writes one pair while
                                                                // the MMAs of tile i read the other
  static constexpr int OFF_STAT = OFF_DST + 2 * PT_BYTES;       // [2 stages][2][BQ] floats
  static constexpr int OFF_BAR = OFF_STAT + 2 * 2 * BQ * 4;
  static constexpr int SMEM_BYTES = OFF_BAR + 256;
  static_assert(SMEM_BYTES <= 232448, "attention backward: shared memory budget");
  static constexpr int ST_COL = 0;
  static constexpr int DPT_COL = BQ;
  static constexpr int DV_COL = 2 * BQ;
  static constexpr int DK_COL = 2 * BQ + DH;
  static constexpr int DQ_COL = 2 * BQ + 2 * DH;
  static constexpr int TMEM_COLS = 512;
};

// delta[b,h,s] = sum_d dO[s, h*dh + d] * O[s, h*dh + d]
// A warp takes one token at a time: its nh * dh / 8 vectors of eight columns go round the lanes,
// four vectors a lane and round with their loads issued together (eight 16-byte loads in flight
// a lane); the dh / 8 lanes of a head add up with shuffles.  All index arithmetic is 32-bit and
// per token, not per vector.
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ dO,
                                  const __nv_bfloat16* __restrict__ O, float* __restrict__ delta,
                                  int rows, int S, int nh, int dh, int lddo, int ldo) {
  constexpr int UNR = 4;
  const int lane = threadIdx.x & 31;
  const int tpg = dh >> 3;              // lanes per head: 8 (dh 64) or 16 (dh 128)
  const int nvec = nh * tpg;            // vectors per token
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int GW = (gridDim.x * blockDim.x) >> 5;
  for (int tok = gw; tok < rows; tok += GW) {
    const int bb = tok / S, ss = tok - bb * S;
    const __nv_bfloat16* pa = dO + static_cast<size_t>(tok) * lddo;
    const __nv_bfloat16* pb = O + static_cast<size_t>(tok) * ldo;
    float* out = delta + static_cast<size_t>(bb) * nh * S + ss;
    for (int c0 = 0; c0 < nvec; c0 += 32 * UNR) {
      uint4 a[UNR], b[UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int c = c0 + u * 32 + lane;
        a[u] = make_uint4(0u, 0u, 0u, 0u);
        b[u] = make_uint4(0u, 0u, 0u, 0u);
        if (c < nvec) {
          a[u] = *reinterpret_cast<const uint4*>(pa + c * 8);
          b[u] = *reinterpret_cast<const uint4*>(pb + c * 8);
        }
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int c = c0 + u * 32 + lane;
        const uint32_t aw[4] = {a[u].x, a[u].y, a[u].z, a[u].w};
        const uint32_t bw[4] = {b[u].x, b[u].y, b[u].z, b[u].w};
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 fa = unpack_bf16x2(aw[e]), fb = unpack_bf16x2(bw[e]);
          s += fa.x * fb.x + fa.y * fb.y;
        }
        for (int o = tpg >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (c < nvec && (lane & (tpg - 1)) == 0) out[static_cast<size_t>(c / tpg) * S] = s;
      }
    }
  }
}

// dq[t, c] = bf16(dq_acc[t, c] * scale)
__global__ void attn_dq_finalize_kernel(const float* __restrict__ acc,
                                        __nv_bfloat16* __restrict__ dq, size_t T, int H, int ldd,
                                        float scale) {
  const int nv = H / 8;
  const size_t total = T * nv;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t t = i / nv;
    const int vec = static_cast<int>(i % nv);
    const float4 a = *reinterpret_cast<const float4*>(acc + t * H + vec * 8);
    const float4 b = *reinterpret_cast<const float4*>(acc + t * H + vec * 8 + 4);
    const float v[8] = {a.x * scale, a.y * scale, a.z * scale, a.w * scale,
                        b.x * scale, b.y * scale, b.z * scale, b.w * scale};
    store8(dq + t * ldd + vec * 8, v);
  }
}

template <int DH, bool DROP>
__global__ void __launch_bounds__(ATB_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                const AttnBwdArgs p) {
  using Cfg = AttnBwdCfg<DH>;
  constexpr int BQ = Cfg::BQ;
  constexpr int BKV = ATB_BKV;
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  // 0 kv_full | 1,2 q_full | 3,4 q_empty | 5 s_full | 6 pds_full | 7 pds_empty (even tiles) |
  // 8 dq_full | 9 dq_empty | 10 done | 11 stat_full | 12 pds_empty (odd tiles)
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 13);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  auto bar = [&](int i) { return smem_u32(bars + i); };
  float* s_stat = reinterpret_cast<float*>(smem + Cfg::OFF_STAT);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if ((sbase & 1023u) != 0u) {
    if (threadIdx.x == 0) record_status(p.status, ST_BAD_ARG, 1000);
    return;
  }
  const int n_kv_tiles = (p.S + BKV - 1) / BKV;
  const int bh = blockIdx.x % (p.B * p.nh);
  const int j = blockIdx.x / (p.B * p.nh);  // early K/V tiles see the most queries: first
  const int b = bh / p.nh, h = bh % p.nh;
  const int kv0 = j * BKV;
  const int n_q_tiles = (p.S + BQ - 1) / BQ;
  const int i_start = p.causal ? kv0 / BQ : 0;
  const int n_it = n_q_tiles - i_start;
  (void)n_kv_tiles;

  if (threadIdx.x == 0) {
    mbar_init(bar(0), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(1 + s), 1);
      mbar_init(bar(3 + s), 1);
    }
    mbar_init(bar(5), 1);
    mbar_init(bar(6), 8);      // one arrival per softmax warp
    mbar_init(bar(7), 1);
    mbar_init(bar(8), 1);
    mbar_init(bar(9), 4);      // one arrival per dQ-drain warp
    mbar_init(bar(10), 1);
    mbar_init(bar(11), 8);
    mbar_init(bar(12), 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmdO);
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t sK = sbase + Cfg::OFF_K, sV = sbase + Cfg::OFF_V;
  auto sPTb = [&](int buf) { return sbase + Cfg::OFF_PT + buf * Cfg::PT_BYTES; };
  auto sDSTb = [&](int buf) { return sbase + Cfg::OFF_DST + buf * Cfg::PT_BYTES; };
  auto sQ = [&](int st) { return sbase + Cfg::OFF_Q + st * 2 * Cfg::Q_BYTES; };
  auto sDO = [&](int st) { return sQ(st) + Cfg::Q_BYTES; };
  const int row0 = b * p.S;

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      mbar_arrive_expect_tx(bar(0), 2 * Cfg::KV_BYTES);
#pragma unroll
      for (int c = 0; c < DH / 64; ++c) {
        tma_load_2d(sK + c * (BKV * 128), &tmK, bar(0), h * DH + c * 64, row0 + kv0);
        tma_load_2d(sV + c * (BKV * 128), &tmV, bar(0), h * DH + c * 64, row0 + kv0);
      }
      int issued = 0;
      for (int it = 0; it < n_it; ++it) {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1u;
        if (!mbar_wait(bar(3 + st), ph ^ 1u, abort_flag)) {
          record_status(p.status, ST_WAIT_TIMEOUT, 1010);
          break;
        }
        const int qrow = row0 + (i_start + it) * BQ;
        mbar_arrive_expect_tx(bar(1 + st), 2 * Cfg::Q_BYTES);
#pragma unroll
        for (int c = 0; c < DH / 64; ++c) {
          tma_load_2d(sQ(st) + c * (BQ * 128), &tmQ, bar(1 + st), h * DH + c * 64, qrow);
          tma_load_2d(sDO(st) + c * (BQ * 128), &tmdO, bar(1 + st), h * DH + c * 64, qrow);
        }
        ++issued;
      }
      if (*abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        for (int i = max(0, issued - 2); i < issued; ++i) {
          while (!mbar_try_wait(bar(1 + (i & 1)), (i >> 1) & 1u)) {
            if (globaltimer_ns() - t0 > 200000000ull) break;
          }
        }
        while (!mbar_try_wait(bar(0), 0)) {
          if (globaltimer_ns() - t0 > 200000000ull) break;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    // The whole warp runs the control flow (addresses and descriptors stay warp-uniform, which
    // keeps the issue of one MMA near 35 clocks instead of ~100 from a divergent single lane);
    // one elected lane issues.  Descriptors are built once; a product only adds constants to
    // their address field.
    {
      constexpr uint32_t idesc_st = umma_idesc_bf16(BKV, BQ, 0, 0);   // S^T, dP^T
      constexpr uint32_t idesc_dv = umma_idesc_bf16(BKV, DH, 0, 1);   // dV, dK
      constexpr uint32_t idesc_dq =
          (DH == 64) ? umma_idesc_bf16(BQ, DH, 1, 1) : umma_idesc_bf16(DH, BQ, 1, 1);
      const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
      // K-major forms (rows of 64 contraction elements) and MN-major forms (one row per
      // contraction index, 64-element column groups lbo bytes apart)
      const uint64_t dK_k = umma_desc_sw128(sK, 16, 1024), dV_k = umma_desc_sw128(sV, 16, 1024);
      const uint64_t dK_mn = umma_desc_sw128(sK, BKV * 128, 1024);
      const uint64_t dQ_k0 = umma_desc_sw128(sQ(0), 16, 1024), dDO_k0 = umma_desc_sw128(sDO(0), 16, 1024);
      const uint64_t dQ_mn0 = umma_desc_sw128(sQ(0), BQ * 128, 1024);
      const uint64_t dDO_mn0 = umma_desc_sw128(sDO(0), BQ * 128, 1024);
      const uint64_t dPT_k0 = umma_desc_sw128(sPTb(0), 16, 1024);
      const uint64_t dDST_k0 = umma_desc_sw128(sDSTb(0), 16, 1024);
      const uint64_t dDST_mn0 = umma_desc_sw128(sDSTb(0), BKV * 128, 1024);
      constexpr uint64_t ST_STEP = (2 * Cfg::Q_BYTES) >> 4;     // Q/dO stage pitch
      constexpr uint64_t BUF_STEP = Cfg::PT_BYTES >> 4;         // P^T / dS^T buffer pitch
      auto wait_all = [&](int b_idx, uint32_t parity, int where) {
        const bool got = mbar_wait(bar(b_idx), parity, abort_flag);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0) record_status(p.status, ST_WAIT_TIMEOUT, where);
          return false;
        }
        return true;
      };
      bool ok = wait_all(0, 0, 1020);
      long long* trace = (blockIdx.x == 0 && lane == 0) ? p.trace : nullptr;
      // S^T and dP^T of query tile `it` (needs its Q/dO stage and the S^T/dP^T columns free)
      auto issue_scores = [&](int it) {
        const int st = it & 1;
        if (!wait_all(1 + st, (it >> 1) & 1u, 1021)) return false;
        tc_fence_after();
        if (trace && it < 32) trace[it * 12 + 4] = clock64();
        const uint64_t bq = dQ_k0 + st * ST_STEP, bdo = dDO_k0 + st * ST_STEP;
        if (elect_one()) {
          // the two products are independent: alternating them keeps two accumulation chains
          // in flight
#pragma unroll
          for (int kk = 0; kk < DH / 16; ++kk) {
            constexpr int dummy = 0;
            (void)dummy;
            const uint64_t ko = static_cast<uint64_t>(((kk / 4) * (BKV * 128) + (kk % 4) * 32) >> 4);
            const uint64_t qo = static_cast<uint64_t>(((kk / 4) * (BQ * 128) + (kk % 4) * 32) >> 4);
            umma_bf16_ss(tmem_u + Cfg::ST_COL, dK_k + ko, bq + qo, idesc_st, kk > 0 ? 1u : 0u);
            umma_bf16_ss(tmem_u + Cfg::DPT_COL, dV_k + ko, bdo + qo, idesc_st, kk > 0 ? 1u : 0u);
          }
          umma_commit(bar(5));
        }
        __syncwarp();
        if (trace && it < 32) trace[it * 12 + 5] = clock64();
        return true;
      };
      if (ok && n_it > 0) ok = issue_scores(0);
      for (int it = 0; it < n_it && ok; ++it) {
        const int st = it & 1, buf = it & 1;
        // P^T / dS^T of this tile are in shared memory and its S^T / dP^T columns have been read
        if (!wait_all(6, it & 1u, 1022)) { ok = false; break; }
        tc_fence_after();
        if (trace && it < 32) trace[it * 12 + 6] = clock64();
        // The next tile's scores go first: its softmax then runs while the three products below
        // execute (they read the other P^T / dS^T buffer).
        if (it + 1 < n_it && !issue_scores(it + 1)) { ok = false; break; }
        if (it > 0) {     // the previous tile's dQ must have left tensor memory
          if (!wait_all(9, (it - 1) & 1u, 1023)) { ok = false; break; }
          tc_fence_after();
        }
        if (trace && it < 32) trace[it * 12 + 10] = clock64();
        // dV += P^T . dO_i, dK += dS^T . Q_i (contraction over the BQ query rows) and
        // dQ_i = dS . K_j (contraction over the 128 K/V rows): three independent accumulation
        // chains, issued round-robin
        const uint64_t aPT = dPT_k0 + buf * BUF_STEP, aDST = dDST_k0 + buf * BUF_STEP;
        const uint64_t mDST = dDST_mn0 + buf * BUF_STEP;
        const uint64_t bDO = dDO_mn0 + st * ST_STEP, bQ = dQ_mn0 + st * ST_STEP;
        const uint32_t acc0 = it > 0 ? 1u : 0u;
        if (elect_one()) {
          constexpr int NK = (BQ > BKV ? BQ : BKV) / 16;
#pragma unroll
          for (int kk = 0; kk < NK; ++kk) {
            const uint64_t ko = static_cast<uint64_t>(((kk / 4) * (BKV * 128) + (kk % 4) * 32) >> 4);
            const uint64_t mo = static_cast<uint64_t>((kk * 2048) >> 4);
            if (kk < BQ / 16) {
              umma_bf16_ss(tmem_u + Cfg::DV_COL, aPT + ko, bDO + mo, idesc_dv, kk > 0 ? 1u : acc0);
              umma_bf16_ss(tmem_u + Cfg::DK_COL, aDST + ko, bQ + mo, idesc_dv, kk > 0 ? 1u : acc0);
            }
            if (kk < BKV / 16) {
              if constexpr (DH == 64) {
                // dQ_i[q, d] = sum_kv dS^T[kv, q] K_j[kv, d]
                umma_bf16_ss(tmem_u + Cfg::DQ_COL, mDST + mo, dK_mn + mo, idesc_dq, kk > 0 ? 1u : 0u);
              } else {
                // dQ_i^T[d, q] = sum_kv K_j[kv, d] dS^T[kv, q]
                umma_bf16_ss(tmem_u + Cfg::DQ_COL, dK_mn + mo, mDST + mo, idesc_dq, kk > 0 ? 1u : 0u);
              }
            }
          }
          umma_commit(bar(8));                 // dQ ready to drain
          umma_commit(bar(3 + st));            // Q_i / dO_i stage free
          umma_commit(bar(buf ? 12 : 7));      // this P^T / dS^T buffer free
        }
        __syncwarp();
        if (trace && it < 32) trace[it * 12 + 7] = clock64();
      }
      if (ok && elect_one()) umma_commit(bar(10));
      __syncwarp();
    }
  } else if (warp < 10) {
    // ---------------------------------------------------------------- softmax / dS
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;   // which half of the query columns this thread covers
    const int r = quarter * 32 + lane;  // K/V row within the tile
    const int kv_idx = kv0 + r;
    const int tid = threadIdx.x - 64;   // 0..255
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const size_t stat_base = (static_cast<size_t>(b) * p.nh + h) * p.S;
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int q0 = (i_start + it) * BQ;
      float* s_lse = s_stat + (it & 1) * 2 * BQ;
      float* s_dl = s_lse + BQ;
      if (tid < BQ) {
        const int qi = q0 + tid;
        s_lse[tid] = qi < p.S ? p.lse[stat_base + qi] * 1.4426950408889634f : INFINITY;
        s_dl[tid] = qi < p.S ? p.delta[stat_base + qi] : 0.f;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(11));
      bool got = mbar_wait(bar(11), it & 1u, abort_flag);
      if (got) got = mbar_wait(bar(5), it & 1u, abort_flag);
      // the buffer pair of this parity was last read by the products of tile it - 2
      if (got && it > 1) got = mbar_wait(bar((it & 1) ? 12 : 7), ((it >> 1) - 1) & 1u, abort_flag);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) record_status(p.status, ST_WAIT_TIMEOUT, 1030);
        ok = false;
        break;
      }
      tc_fence_after();
      long long* tr = (blockIdx.x == 0 && it < 32 && warp == 2 && lane == 0) ? p.trace : nullptr;
      if (tr) tr[it * 12 + 0] = clock64();
      const uint32_t sPT = sPTb(it & 1), sDST = sDSTb(it & 1);
      const bool diag = p.causal && (kv0 + BKV - 1 > q0);
      const bool row_dead = kv_idx >= p.S;
#pragma unroll 1
      for (int c = half * (BQ / 64); c < (half + 1) * (BQ / 64); ++c) {
        uint32_t sv[32], dv[32];
        tmem_ld_32x32b_x32(lane_addr + Cfg::ST_COL + c * 32, sv);
        tmem_ld_32x32b_x32(lane_addr + Cfg::DPT_COL + c * 32, dv);
        tmem_ld_wait();
        if (tr && c == half * (BQ / 64)) tr[it * 12 + 1] = clock64();
        uint32_t pk[16], dk[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const int qc = c * 32 + e;
          float p0 = fast_exp2(__uint_as_float(sv[e]) * p.scale_log2 - s_lse[qc]);
          float p1 = fast_exp2(__uint_as_float(sv[e + 1]) * p.scale_log2 - s_lse[qc + 1]);
          if (row_dead || (diag && kv_idx > q0 + qc)) p0 = 0.f;
          if (row_dead || (diag && kv_idx > q0 + qc + 1)) p1 = 0.f;
          float m0 = 1.f, m1 = 1.f;
          if constexpr (DROP) {
            // the forward pass's mask: element (query, key) of the [B nh S, S] probability matrix
            const unsigned long long gq =
                ((static_cast<unsigned long long>(b) * p.nh + h) * p.S + (q0 + qc)) *
                    static_cast<unsigned long long>(p.S >> 2) + static_cast<unsigned long long>(kv_idx >> 2);
            m0 = dropout_factor(dropout_bits(gq, p.drop_key), kv_idx & 3, p.drop_thr, p.drop_scale);
            m1 = dropout_factor(dropout_bits(gq + (p.S >> 2), p.drop_key), kv_idx & 3, p.drop_thr,
                                p.drop_scale);
          }
          const float d0 = p0 * (__uint_as_float(dv[e]) * m0 - s_dl[qc]);
          const float d1 = p1 * (__uint_as_float(dv[e + 1]) * m1 - s_dl[qc + 1]);
          pk[e >> 1] = pack_bf16x2(p0 * m0, p1 * m1);
          dk[e >> 1] = pack_bf16x2(d0, d1);
        }
        const uint32_t off = ((c * 32) / 64) * (BKV * 128) + r * 128;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const uint32_t chunk = static_cast<uint32_t>(((c * 4) & 7) + g);
          const uint32_t sw = (chunk ^ (r & 7)) << 4;
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sPT + off + sw),
                       "r"(pk[4 * g]), "r"(pk[4 * g + 1]), "r"(pk[4 * g + 2]), "r"(pk[4 * g + 3])
                       : "memory");
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sDST + off + sw),
                       "r"(dk[4 * g]), "r"(dk[4 * g + 1]), "r"(dk[4 * g + 2]), "r"(dk[4 * g + 3])
                       : "memory");
        }
      }
      if (tr) tr[it * 12 + 2] = clock64();
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(6));
      if (tr) tr[it * 12 + 3] = clock64();
    }
    // ---- epilogue: dV and dK of this K/V tile
    if (ok) {
      const bool got = mbar_wait(bar(10), 0, abort_flag);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) record_status(p.status, ST_WAIT_TIMEOUT, 1031);
        ok = false;
      }
    }
    if (ok) {
      tc_fence_after();
      const bool row_ok = kv_idx < p.S;
      const size_t orow = (static_cast<size_t>(row0) + kv_idx) * p.ldd + static_cast<size_t>(h) * DH;
      {
        const int which = half;   // first group writes dV, second group dK
        __nv_bfloat16* dst = (which == 0 ? p.dv : p.dk) + orow;
        const float mul = which == 0 ? 1.0f : p.scale;
        const int col = which == 0 ? Cfg::DV_COL : Cfg::DK_COL;
#pragma unroll 1
        for (int c = 0; c < DH / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(lane_addr + col + c * 32, o);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 w;
              w.x = pack_bf16x2(__uint_as_float(o[8 * g + 0]) * mul, __uint_as_float(o[8 * g + 1]) * mul);
              w.y = pack_bf16x2(__uint_as_float(o[8 * g + 2]) * mul, __uint_as_float(o[8 * g + 3]) * mul);
              w.z = pack_bf16x2(__uint_as_float(o[8 * g + 4]) * mul, __uint_as_float(o[8 * g + 5]) * mul);
              w.w = pack_bf16x2(__uint_as_float(o[8 * g + 6]) * mul, __uint_as_float(o[8 * g + 7]) * mul);
              *reinterpret_cast<uint4*>(dst + c * 32 + g * 8) = w;
            }
          }
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- dQ drain
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const int Hd = p.nh * DH;
    for (int it = 0; it < n_it; ++it) {
      const bool got = mbar_wait(bar(8), it & 1u, abort_flag);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) record_status(p.status, ST_WAIT_TIMEOUT, 1040);
        break;
      }
      tc_fence_after();
      long long* trq = (blockIdx.x == 0 && it < 32 && warp == 10 && lane == 0) ? p.trace : nullptr;
      if (trq) trq[it * 12 + 8] = clock64();
      const int q0 = (i_start + it) * BQ;
      if constexpr (DH == 64) {
        const int qi = q0 + r;
        float* dst = p.dq_acc + (static_cast<size_t>(row0) + qi) * Hd + static_cast<size_t>(h) * DH;
#pragma unroll 1
        for (int c = 0; c < DH / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(lane_addr + Cfg::DQ_COL + c * 32, o);
          tmem_ld_wait();
          if (qi < p.S) {
#pragma unroll
            for (int g = 0; g < 8; ++g)
              asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                           ::"l"(dst + c * 32 + g * 4), "f"(__uint_as_float(o[4 * g])),
                             "f"(__uint_as_float(o[4 * g + 1])), "f"(__uint_as_float(o[4 * g + 2])),
                             "f"(__uint_as_float(o[4 * g + 3]))
                           : "memory");
          }
        }
      } else {
        // lanes hold the head dimension, columns the BQ queries
        float* dst = p.dq_acc + static_cast<size_t>(row0) * Hd + static_cast<size_t>(h) * DH + r;
#pragma unroll 1
        for (int c = 0; c < BQ / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(lane_addr + Cfg::DQ_COL + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int qi = q0 + c * 32 + e;
            if (qi < p.S) atomicAdd(dst + static_cast<size_t>(qi) * Hd, __uint_as_float(o[e]));
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (trq) trq[it * 12 + 9] = clock64();
      if (lane == 0) mbar_arrive(bar(9));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

template <int DH, bool DROP>
static int launch_attn_bwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                           const CUtensorMap& tdo, const AttnBwdArgs& a, cudaStream_t st) {
  using Cfg = AttnBwdCfg<DH>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_bwd_kernel<DH, DROP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg::SMEM_BYTES) != cudaSuccess)
      return -10;
    configured = true;
  }
  const int n_kv_tiles = (a.S + ATB_BKV - 1) / ATB_BKV;
  attn_bwd_kernel<DH, DROP><<<n_kv_tiles * a.B * a.nh, ATB_THREADS, Cfg::SMEM_BYTES, st>>>(
      tq, tk, tv, tdo, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace cb

// dqkv: bf16 [B*S, 3*nh*dh] (pitch ldd) receiving dQ | dK | dV.  dq_acc: zeroed fp32
// [B*S, nh*dh] scratch; delta: fp32 [B, nh, S] scratch.
extern "C" int cb_attn_bwd_set_trace(long long* device_buffer) {
  cb::g_attn_bwd_trace_host = device_buffer;
  return 0;
}

// drop_thr in [0, 255] and drop_key: the dropout of the forward pass (0: none; else S % 4 == 0).
extern "C" int cb_attn_bwd_dropout(const void* dO, const void* q, const void* k, const void* v,
                                   const void* o, const float* lse, float* delta, float* dq_acc,
                                   void* dqkv, int B, int S, int nh, int dh, int lddo, int ldq,
                                   int ldk, int ldv, int ldo, int ldd, float scale, int causal,
                                   int drop_thr, unsigned int drop_key, int* status, void* stream) {
  using namespace cb;
  if (dh != 64 && dh != 128) return -1;
  if (B <= 0 || S <= 0 || nh <= 0 || (ldd % 8) != 0) return -2;
  if (drop_thr < 0 || drop_thr > 255 || (drop_thr > 0 && (S % 4) != 0)) return -13;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int H = nh * dh;
  const uint64_t rows = static_cast<uint64_t>(B) * S;
  // every argument check (the tensor maps included) comes before the first launch, so that a
  // refused call has enqueued nothing
  const uint32_t bq = 64;   // rows per query / dO box: a tile (dh 128) or half a tile (dh 64)
  CUtensorMap tq, tk, tv, tdo;
  if (make_tmap_bf16_2d(&tq, q, H, rows, ldq, 64, bq) != 0) return -3;
  if (make_tmap_bf16_2d(&tk, k, H, rows, ldk, 64, ATB_BKV) != 0) return -4;
  if (make_tmap_bf16_2d(&tv, v, H, rows, ldv, 64, ATB_BKV) != 0) return -5;
  if (make_tmap_bf16_2d(&tdo, dO, H, rows, lddo, 64, bq) != 0) return -6;
  CUtensorMap tdq, tdk, tdv;
  if (dh == 64) {
    __nv_bfloat16* out = static_cast<__nv_bfloat16*>(dqkv);
    const uint64_t slab = static_cast<uint64_t>(S) * ldd;
    if (make_tmap_f32_3d(&tdq, dq_acc, H, S, B, H, static_cast<uint64_t>(S) * H, 32) != 0) return -7;
    if (make_tmap_bf16_3d(&tdk, out + H, H, S, B, ldd, slab, 128) != 0) return -8;
    if (make_tmap_bf16_3d(&tdv, out + 2 * H, H, S, B, ldd, slab, 128) != 0) return -9;
  }
  {
    // a warp per token, eight warps a block
    const int blocks = static_cast<int>(std::min<size_t>((rows + 7) / 8, sm_count() * 16));
    attn_delta_kernel<<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(dO),
                                              static_cast<const __nv_bfloat16*>(o), delta,
                                              static_cast<int>(rows), S, nh, dh, lddo, ldo);
  }
  AttnBwdArgs a;
  a.B = B; a.S = S; a.nh = nh;
  a.lse = lse; a.delta = delta; a.dq_acc = dq_acc;
  a.dk = static_cast<__nv_bfloat16*>(dqkv) + H;
  a.dv = static_cast<__nv_bfloat16*>(dqkv) + 2 * H;
  a.ldd = ldd;
  a.scale = scale;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.causal = causal;
  a.status = status;
  a.trace = g_attn_bwd_trace_host;
  a.drop_thr = drop_thr;
  a.drop_key = drop_key;
  a.drop_scale = 256.0f / static_cast<float>(256 - drop_thr);
  int rc = dh == 64 ? launch_attn_bwd_dh64(tq, tk, tv, tdo, tdq, tdk, tdv, a, st)
           : drop_thr > 0 ? launch_attn_bwd<128, true>(tq, tk, tv, tdo, a, st)
                          : launch_attn_bwd<128, false>(tq, tk, tv, tdo, a, st);
  if (rc != 0) return rc;
  {
    const size_t work = rows * (H / 8);
    const int blocks = static_cast<int>(std::min<size_t>((work + 255) / 256, sm_count() * 16));
    attn_dq_finalize_kernel<<<blocks, 256, 0, st>>>(dq_acc, static_cast<__nv_bfloat16*>(dqkv),
                                                    rows, H, ldd, scale);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -12;
}

extern "C" int cb_attn_bwd(const void* dO, const void* q, const void* k, const void* v,
                           const void* o, const float* lse, float* delta, float* dq_acc,
                           void* dqkv, int B, int S, int nh, int dh, int lddo, int ldq, int ldk,
                           int ldv, int ldo, int ldd, float scale, int causal, int* status,
                           void* stream) {
  return cb_attn_bwd_dropout(dO, q, k, v, o, lse, delta, dq_acc, dqkv, B, S, nh, dh, lddo, ldq, ldk,
                             ldv, ldo, ldd, scale, causal, 0, 0u, status, stream);
}

// ------------------------------------------------------------------------------------------
// Allocation-free variant (declared and documented in no_alloc.h): the dQ accumulator and the
// delta rows come from a fixed array inside the library image instead of from the caller.
#include "no_alloc.h"

static __device__ __align__(256) float g_noalloc_scratch[CB_NOALLOC_SCRATCH_FLOATS];

#include <mutex>

namespace {
constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {nullptr};
std::mutex g_noalloc_mutex;   // guards the one-time fill of g_noalloc_ptr

// Device address of the scratch array on the current device.  In host code the array's name is
// only a handle for the runtime, not an address a kernel could use, so the address is asked for
// once per device (with that device current) and cached.
int noalloc_scratch(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return CB_NOALLOC_ERR_SYMBOL;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_ptr[dev] == nullptr) {
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch) != cudaSuccess ||
        p == nullptr)
      return CB_NOALLOC_ERR_SYMBOL;
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return 0;
}
}  // namespace

extern "C" int cb_attn_bwd_noalloc(const void* dO, const void* q, const void* k, const void* v,
                                   const void* o, const float* lse, void* dqkv, int B, int S,
                                   int nh, int dh, int lddo, int ldq, int ldk, int ldv, int ldo,
                                   int ldd, float scale, int causal, int* status, void* stream) {
  // the checks cb_attn_bwd() would make on these arguments, made here before anything (the
  // clearing of the scratch included) is enqueued
  if (dh != 64 && dh != 128) return -1;
  if (B <= 0 || S <= 0 || nh <= 0 || (ldd % 8) != 0) return -2;
  const size_t dq_floats = static_cast<size_t>(B) * S * nh * dh;
  const size_t delta_floats = static_cast<size_t>(B) * nh * S;
  if (dq_floats + delta_floats > CB_NOALLOC_SCRATCH_FLOATS) return CB_NOALLOC_ERR_TOO_LARGE;
  float* scratch = nullptr;
  const int rc = noalloc_scratch(&scratch);
  if (rc != 0) return rc;
  // The accumulator must start at zero; delta is fully overwritten by its producer kernel.
  if (cudaMemsetAsync(scratch, 0, dq_floats * sizeof(float),
                      static_cast<cudaStream_t>(stream)) != cudaSuccess)
    return -102;
  return cb_attn_bwd(dO, q, k, v, o, lse, scratch + dq_floats, scratch, dqkv, B, S, nh, dh, lddo,
                     ldq, ldk, ldv, ldo, ldd, scale, causal, status, stream);
}

extern "C" const char* cb_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case CB_NOALLOC_ERR_TOO_LARGE:
      return "problem too large for the built-in scratch: B*S*nh*dh + B*nh*S exceeds the maximum "
             "of CB_NOALLOC_SCRATCH_FLOATS (4 Mi floats, 16 MiB)";
    case CB_NOALLOC_ERR_SYMBOL:
      return "could not obtain the device address of the built-in scratch array";
    case -1: return "unsupported head dimension (the kernels cover dh = 64 and dh = 128)";
    case -2: return "bad sizes: B, S and nh must be positive and ldd a multiple of 8";
    case -102: return "clearing the scratch failed";
    default: return "attention backward failed (see cb_attn_bwd return codes)";
  }
}
