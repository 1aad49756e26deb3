// Flash-style attention backward for head dimension 64: persistent CTAs, pipelined over the two
// halves of a query tile.  A work item is one (batch, head, 128-row K/V tile); a CTA takes items
// from the list sorted by length (heavy and light ends alternate, see BwdWalk) and streams the
// 128-row query tiles that attend to the item's K/V tile, in the transposed orientation (K/V rows
// on the tensor-memory lanes):
//   S^T  = K_j . Q_i^T          dP^T = V_j . dO_i^T
//   P^T  = exp2(S^T * c - LSE_i)       dS^T = P^T o (dP^T - delta_i)
//   dV_j += P^T . dO_i          dK_j += dS^T . Q_i          dQ_i = dS . K_j
// What distinguishes it from the generic kernel (attention_bwd.cu):
//  * a query tile is handled as two halves of 64 query columns, each with its own S^T / dP^T
//    columns in tensor memory, its own softmax warpgroup and its own query / dO ring slots; while
//    one half's products and next scores run on the tensor cores the other half's softmax runs;
//  * P^T and dS^T are written back as packed bf16 over their own score columns in tensor memory
//    and feed dV and dK as tensor-memory A operands: no shared-memory round trip for P^T at all,
//    dS^T goes to shared memory only for dQ (where it is the transposed operand);
//  * dQ is double-buffered in tensor memory and leaves through a swizzled staging tile and bulk
//    reduce-adds into the fp32 accumulation buffer shared by all K/V tiles;
//  * the tensor pipe executes one thread's MMAs in issue order, which is what lets the scores of
//    the next step overwrite the columns P^T / dS^T of this step were read from without a barrier;
//  * the steps of consecutive items form one stream: the next item's K/V tile is loaded (second
//    buffer) and its first scores are issued while the current item finishes, and the dV / dK
//    epilogue of an item runs after the softmax of the next item's first step.
//   warp 0        TMA producer (K_j, V_j per item, two buffers; Q_i, dO_i by halves through a ring
//                 of five slots)
//   warp 1        MMA issuer: products, scores, dQ     warp 2   idle (the dQ issuer if DQ_OWN_WARP)
//   warp 3        stores the staged dV / dK tiles (bulk stores)
//   warps 4..11   softmax / dS of the first half (two threads per K/V row, 32 query columns each);
//                 warps 4..7 also the dV epilogue (staged in the item's K tile)
//   warps 12..19  softmax / dS of the second half; warps 12..15 also the dK epilogue (V tile)
//   warps 20..23  dQ drain (TMEM -> shared memory -> bulk reduce-add into the fp32 accumulator)
// delta_i = rowsum(dO_i o O_i) comes from a pre-kernel, a post-kernel scales and casts dQ (both in
// attention_bwd.cu).  The reference (plugins/model-transformer/src/lib.rs:300-372) computes the
// attention gradient on the CPU in fp32 with materialised probabilities.
#include <climits>

#include "attention_bwd.cuh"
#include "common.cuh"
#include "ptx.cuh"

namespace cb {

int sm_count();

namespace {

struct B64 {
  static constexpr int DH = 64, BQ = 128, BKV = 128, HQ = 64;
  static constexpr int NSUB = 2;                          // softmax threads per K/V row and half
  static constexpr int THREADS = 32 * (4 + 2 * NSUB * 4 + 4);
  static constexpr bool DQ_OWN_WARP = false;   // dQ issued by warp 2 (else by warp 1, after a
                                               // step's second half: measured 3 % faster)
  static constexpr int NSLOT = 5;                         // ring of half-tile slots (2.5 steps)
  static constexpr int KV_BYTES = BKV * DH * 2;           // K_j or V_j
  static constexpr int HALF_BYTES = HQ * DH * 2;          // 64 query rows of Q_i or dO_i
  static constexpr int SLOT_BYTES = 2 * HALF_BYTES;       // one slot: half of Q_i | half of dO_i
  static constexpr int DST_BYTES = BKV * BQ * 2;          // dS^T of one tile
  static constexpr int OFF_K = 0;                         // two buffers of (K_j | V_j)
  static constexpr int OFF_Q = 2 * 2 * KV_BYTES;
  static constexpr int OFF_DST = OFF_Q + NSLOT * SLOT_BYTES;  // two buffers (step parity)
  static constexpr int OFF_DQS = OFF_DST + 2 * DST_BYTES;   // dQ staging: per drain warp one box
                                                            // of [32 rows][32 floats], swizzled
  static constexpr int DQS_BYTES = BQ * 32 * 4;
  static constexpr int OFF_STAT = OFF_DQS + DQS_BYTES;      // [2 parities][lse | delta][BQ] floats
  static constexpr int OFF_BAR = OFF_STAT + 2 * 2 * BQ * 4;
  static constexpr int SMEM_BYTES = OFF_BAR + 256;
  static_assert(SMEM_BYTES <= 232448, "attention backward: shared memory budget");
  // tensor-memory columns: per half h, S^T at 128 h (P^T over its first 32 columns) and dP^T at
  // 128 h + 64 (dS^T over its first 32); then dV, dK and two dQ buffers
  static constexpr int DV_COL = 256, DK_COL = 320, DQ_COL = 384;
  static constexpr int TMEM_COLS = 512;
  enum {
    B_KVF = 0,               // + buffer: K_j / V_j landed
    B_KVE = 2,               // + buffer: buffer free (issuers and epilogue through with the item)
    B_QF = 4,                // + slot: a half's Q_i / dO_i rows landed
    B_QE = B_QF + NSLOT,     // + slot: slot free
    B_SF = B_QE + NSLOT,     // + half: S^T / dP^T of the half complete
    B_PF = B_SF + 2,         // + half: P^T / dS^T of the half written (4 warps)
    B_STF = B_PF + 2,        // + half: the half's lse / delta in shared memory (4 warps)
    B_DF = B_STF + 2,        // + parity: dS^T buffer free (its dQ product completed)
    B_DQF = B_DF + 2,        // + parity: dQ complete in tensor memory
    B_DQE = B_DQF + 2,       // + parity: dQ drained (4 warps)
    B_DONE = B_DQE + 2,      // the item's dV / dK are complete and its K/V buffer is not read any more
    B_EPI,                   // dV / dK of the item have left tensor memory (8 warps)
    B_STG,                   // dV / dK of the item are staged in shared memory (8 warps)
    N_BARS
  };
  static_assert(N_BARS * 8 + 8 <= 256, "barrier block");
};

// The items of one CTA in the order every role walks them.  Items are sorted by the number of
// query tiles (K/V tile 0 sees all of them under a causal mask); CTA c takes one item of every
// wave of gridDim.x items, counted from the front of even waves and from the back of odd ones.
struct BwdWalk {
  int wave;
  int b, h, j, n_it;
  bool valid;
  __device__ int i_start(const AttnBwdArgs& p) const { return p.causal ? j : 0; }   // BQ == BKV
  __device__ void init(const AttnBwdArgs& p) {
    wave = -1;
    valid = true;
    next(p);
  }
  __device__ void next(const AttnBwdArgs& p) {
    const int n_bh = p.B * p.nh;
    const int n_items = n_bh * ((p.S + B64::BKV - 1) / B64::BKV);
    while (true) {
      ++wave;
      if (wave * static_cast<int>(gridDim.x) >= n_items) { valid = false; return; }
      const int c = (wave & 1) ? static_cast<int>(gridDim.x - 1 - blockIdx.x)
                               : static_cast<int>(blockIdx.x);
      const int i = wave * static_cast<int>(gridDim.x) + c;
      if (i >= n_items) continue;
      const int bh = i % n_bh;
      j = i / n_bh;
      b = bh / p.nh;
      h = bh % p.nh;
      n_it = (p.S + B64::BQ - 1) / B64::BQ - (p.causal ? j : 0);
      return;
    }
  }
  // the item after this one (a temporary: only the roles' last step of an item looks ahead)
  __device__ BwdWalk peek(const AttnBwdArgs& p) const {
    BwdWalk t = *this;
    t.next(p);
    return t;
  }
};

// One 16-column chunk of a half: p = exp2(s c - lse), ds = p (dp - delta), both packed to bf16.
// `lim` > query index hides the element (causal mask and rows beyond the sequence).  With DROP
// the forward pass's dropout is applied: P^T holds the dropped probabilities (the dV operand),
// dS = p (m dp - delta) with m = 0 or the keep scale; `g0` is the hash group of the chunk's first
// query column for this thread's key (consecutive queries are `gstep` groups apart), `lane4` the
// key's byte within its group.
template <bool MASK, bool DROP>
__device__ __forceinline__ void bwd_chunk(const uint32_t* sv, const uint32_t* dv,
                                          const float* s_lse, const float* s_dl, float c, int lim,
                                          int q_first, uint32_t* pk, uint32_t* dk,
                                          unsigned long long g0 = 0, unsigned long long gstep = 0,
                                          int lane4 = 0, int thr = 0, uint32_t key = 0,
                                          float dscale = 1.f) {
#pragma unroll
  for (int e = 0; e < 16; e += 4) {
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
    float m0 = 1.f, m1 = 1.f, m2 = 1.f, m3 = 1.f;
    if (DROP) {
      m0 = dropout_factor(dropout_bits(g0 + (e + 0) * gstep, key), lane4, thr, dscale);
      m1 = dropout_factor(dropout_bits(g0 + (e + 1) * gstep, key), lane4, thr, dscale);
      m2 = dropout_factor(dropout_bits(g0 + (e + 2) * gstep, key), lane4, thr, dscale);
      m3 = dropout_factor(dropout_bits(g0 + (e + 3) * gstep, key), lane4, thr, dscale);
    }
    const float d0 = p0 * (__uint_as_float(dv[e]) * m0 - D.x);
    const float d1 = p1 * (__uint_as_float(dv[e + 1]) * m1 - D.y);
    const float d2 = p2 * (__uint_as_float(dv[e + 2]) * m2 - D.z);
    const float d3 = p3 * (__uint_as_float(dv[e + 3]) * m3 - D.w);
    pk[e >> 1] = pack_bf16x2(p0 * m0, p1 * m1);
    pk[(e >> 1) + 1] = pack_bf16x2(p2 * m2, p3 * m3);
    dk[e >> 1] = pack_bf16x2(d0, d1);
    dk[(e >> 1) + 1] = pack_bf16x2(d2, d3);
  }
}

// tmQ / tmdO: boxes of 64 rows (one half of a query tile); tmK / tmV: boxes of 128 rows.
template <bool DROP>
__global__ void __launch_bounds__(B64::THREADS, 1)
attn_bwd_dh64_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                     const __grid_constant__ CUtensorMap tmDQ, const __grid_constant__ CUtensorMap tmDK,
                     const __grid_constant__ CUtensorMap tmDV, const AttnBwdArgs p) {
  using C = B64;
  constexpr int DH = C::DH, BQ = C::BQ, BKV = C::BKV, HQ = C::HQ, NSLOT = C::NSLOT;
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + C::N_BARS);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  auto bar = [&](int i) { return smem_u32(bars + i); };
  float* s_stat = reinterpret_cast<float*>(smem + C::OFF_STAT);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (blockIdx.x == 0 && threadIdx.x == 0 && p.trace) p.trace[1088] = clock64();
  if ((sbase & 1023u) != 0u) {
    if (threadIdx.x == 0) record_status(p.status, ST_BAD_ARG, 1100);
    return;
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(C::B_KVF + s), 1);
      // the MMA issuer(s), and warp 3 once the dV / dK staged in the finished item's K/V buffer
      // have been stored
      mbar_init(bar(C::B_KVE + s), C::DQ_OWN_WARP ? 3 : 2);
      mbar_init(bar(C::B_SF + s), 1);
      mbar_init(bar(C::B_PF + s), 4 * C::NSUB);      // one arrival per softmax warp of the half
      mbar_init(bar(C::B_STF + s), 4 * C::NSUB);
      mbar_init(bar(C::B_DF + s), 1);
      mbar_init(bar(C::B_DQF + s), 1);
      mbar_init(bar(C::B_DQE + s), 4);     // one arrival per dQ-drain warp
    }
    for (int s = 0; s < NSLOT; ++s) {
      mbar_init(bar(C::B_QF + s), 1);
      mbar_init(bar(C::B_QE + s), 1);
    }
    mbar_init(bar(C::B_DONE), C::DQ_OWN_WARP ? 2 : 1);   // the MMA issuer(s)
    mbar_init(bar(C::B_EPI), 8);           // one arrival per softmax warp
    mbar_init(bar(C::B_STG), 8);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmdO);
    tma_prefetch_desc(&tmDQ);
    tma_prefetch_desc(&tmDK);
    tma_prefetch_desc(&tmDV);
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  auto sK = [&](int kb) { return sbase + C::OFF_K + kb * 2 * C::KV_BYTES; };
  auto sV = [&](int kb) { return sK(kb) + C::KV_BYTES; };
  auto sDST = [&](int buf) { return sbase + C::OFF_DST + buf * C::DST_BYTES; };
  auto sQ = [&](int slot) { return sbase + C::OFF_Q + slot * C::SLOT_BYTES; };   // half of Q_i
  auto sDO = [&](int slot) { return sQ(slot) + C::HALF_BYTES; };                  // half of dO_i

  // 768 threads at 80 registers each: the softmax threads hold one 16-column chunk of S^T and dP^T
  // at a time, so no role needs registers moved to it.
  if (warp < 4) {
    if (warp == 0) {
      // -------------------------------------------------------------- producer
      if (lane == 0) {
        uint32_t n = 0;               // items so far
        uint32_t q_issued = 0;        // half-tile loads issued (two per step): the ring position
        uint32_t kv_issued = 0;
        bool ok = true;
        BwdWalk w;
        for (w.init(p); w.valid && ok; w.next(p), ++n) {
          const int kb = n & 1;
          const int row0 = w.b * p.S;
          if (!mbar_wait(bar(C::B_KVE + kb), ((n >> 1) & 1u) ^ 1u, abort_flag)) {
            record_status(p.status, ST_WAIT_TIMEOUT, 1110);
            break;
          }
          mbar_arrive_expect_tx(bar(C::B_KVF + kb), 2 * C::KV_BYTES);
          tma_load_2d(sK(kb), &tmK, bar(C::B_KVF + kb), w.h * DH, row0 + w.j * BKV);
          tma_load_2d(sV(kb), &tmV, bar(C::B_KVF + kb), w.h * DH, row0 + w.j * BKV);
          ++kv_issued;
          for (int it = 0; it < w.n_it && ok; ++it) {
            const int qrow = row0 + (w.i_start(p) + it) * BQ;
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
              const int slot = q_issued % NSLOT;
              if (!mbar_wait(bar(C::B_QE + slot), ((q_issued / NSLOT) & 1u) ^ 1u, abort_flag)) {
                record_status(p.status, ST_WAIT_TIMEOUT, 1111);
                ok = false;
                break;
              }
              if (blockIdx.x == 0 && p.trace && q_issued < 64) p.trace[1024 + q_issued] = clock64();
              mbar_arrive_expect_tx(bar(C::B_QF + slot), C::SLOT_BYTES);
              tma_load_2d(sQ(slot), &tmQ, bar(C::B_QF + slot), w.h * DH, qrow + hf * HQ);
              tma_load_2d(sDO(slot), &tmdO, bar(C::B_QF + slot), w.h * DH, qrow + hf * HQ);
              ++q_issued;
            }
          }
        }
        if (*abort_flag) {
          // let the copies already in flight land before shared memory is released: the last use
          // of every ring slot and of both K/V buffers
          const uint64_t t0 = globaltimer_ns();
          auto settle = [&](int b_idx, uint32_t parity) {
            while (!mbar_try_wait(bar(b_idx), parity)) {
              if (globaltimer_ns() - t0 > 200000000ull) return;
            }
          };
          const uint32_t q_first = q_issued > NSLOT ? q_issued - NSLOT : 0u;
          for (uint32_t u = q_first; u < q_issued; ++u)
            settle(C::B_QF + u % NSLOT, (u / NSLOT) & 1u);
          for (uint32_t u = kv_issued > 2u ? kv_issued - 2u : 0u; u < kv_issued; ++u)
            settle(C::B_KVF + (u & 1u), (u >> 1) & 1u);
        }
      }
      __syncwarp();
    } else if (warp == 1) {
      // -------------------------------------------------------------- MMA issuer: products, scores
      // The whole warp runs the control flow (addresses and descriptors stay warp-uniform); one
      // elected lane issues.  Every operand descriptor is one base plus compile-time constants
      // (offset in the address field; the leading-dimension field switched from the K-major to
      // the MN-major value).  (Polling waits here were tried and cost more than they saved: the
      // spinning warp takes issue slots from the softmax warps of its scheduler.)
      // dQ has an issuer of its own (warp 2): it shares no accumulator with these products.
      constexpr uint32_t idesc_sc = umma_idesc_bf16(BKV, HQ, 0, 0);   // S^T, dP^T of a half
      constexpr uint32_t idesc_pv = umma_idesc_bf16(BKV, DH, 0, 1);   // dV, dK (A in tensor memory)
      const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
      const uint64_t d_base = umma_desc_sw128(sbase, 16, 1024);
      constexpr uint64_t MN = static_cast<uint64_t>(((BKV * 128) >> 4) - 1) << 16;
      const uint64_t dK_k0 = d_base + (C::OFF_K >> 4);
      const uint64_t dV_k0 = d_base + ((C::OFF_K + C::KV_BYTES) >> 4);
      const uint64_t dQ_k0 = d_base + (C::OFF_Q >> 4);
      constexpr uint64_t KB_STEP = (2 * C::KV_BYTES) >> 4;  // K/V buffer pitch
      constexpr uint64_t SLOT_STEP = C::SLOT_BYTES >> 4;    // ring slot pitch
      constexpr uint64_t DO_STEP = C::HALF_BYTES >> 4;      // dO half after the Q half of a slot
      auto wait_all = [&](int b_idx, uint32_t parity, int where) {
        const bool got = mbar_wait_poll(bar(b_idx), parity, abort_flag);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0) record_status(p.status, ST_WAIT_TIMEOUT, where);
          return false;
        }
        return true;
      };
      // S^T and dP^T of half hf from ring slot `slot` against K/V buffer kb (K-major operands,
      // contraction over dh)
      auto scores = [&](int hf, uint32_t slot, int kb) {
        const uint64_t bq = dQ_k0 + slot * SLOT_STEP, bdo = bq + DO_STEP;
        const uint64_t ak = dK_k0 + kb * KB_STEP, av = dV_k0 + kb * KB_STEP;
        const uint32_t s_col = tmem_u + hf * 128, d_col = s_col + 64;
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
          umma_bf16_ss(s_col, ak + 2 * kk, bq + 2 * kk, idesc_sc, kk > 0 ? 1u : 0u);
          umma_bf16_ss(d_col, av + 2 * kk, bdo + 2 * kk, idesc_sc, kk > 0 ? 1u : 0u);
        }
        umma_commit(bar(C::B_SF + hf));
      };
      // dV += P^T . dO and dK += dS^T . Q over the 64 query rows of half hf (ring slot `slot`)
      auto products = [&](int hf, uint32_t slot, uint32_t acc0) {
        const uint64_t bq = dQ_k0 + slot * SLOT_STEP + MN, bdo = bq + DO_STEP;
        const uint32_t pt = tmem_u + hf * 128, dst = pt + 64;
#pragma unroll
        for (int kk = 0; kk < HQ / 16; ++kk) {
          // the packed P^T / dS^T of query columns [32 s, 32 s + 32) sit at columns 32 s .. 32 s + 15
          // of the half's S^T / dP^T (each softmax thread writes over columns it has read itself)
          const uint32_t ao = static_cast<uint32_t>((kk >> 1) * 32 + (kk & 1) * 8);
          umma_bf16_ts(tmem_u + C::DV_COL, pt + ao, bdo + 128 * kk, idesc_pv, kk > 0 ? 1u : acc0);
          umma_bf16_ts(tmem_u + C::DK_COL, dst + ao, bq + 128 * kk, idesc_pv, kk > 0 ? 1u : acc0);
        }
        umma_commit(bar(C::B_QE + slot));       // the slot may be refilled
      };
      long long* trace = (blockIdx.x == 0 && lane == 0) ? p.trace : nullptr;
      uint32_t n = 0, g = 0;
      BwdWalk w;
      // A wait on an mbarrier costs a few hundred clocks even when its phase completed long ago,
      // so the ring slots are waited for ahead of their use, while this warp has nothing to
      // issue: qf_waited half-slots (in ring order) have been seen to land, of qf_total in all.
      uint32_t qf_total = 0;
      for (w.init(p); w.valid; w.next(p)) qf_total += 2u * static_cast<uint32_t>(w.n_it);
      uint32_t qf_waited = 0;
      auto wait_slots = [&](uint32_t upto) {     // ... until half-slots [0, upto) have landed
        upto = min(upto, qf_total);
        while (qf_waited < upto) {
          if (!wait_all(C::B_QF + qf_waited % NSLOT, (qf_waited / NSLOT) & 1u, 1123)) return false;
          ++qf_waited;
        }
        return true;
      };
      w.init(p);
      bool ok = w.valid;
      if (ok) ok = wait_all(C::B_KVF, 0, 1120);
      if (ok) ok = wait_slots(2);
      if (ok) {
        tc_fence_after();
        if (trace) trace[1090] = clock64();
        if (elect_one()) {
          scores(0, 0, 0);
          scores(1, 1, 0);
        }
        __syncwarp();
        ok = wait_slots(4);
      }
      while (ok && w.valid) {
        const bool has_next = w.peek(p).valid;
        const int kb = n & 1;
        for (int it = 0; it < w.n_it && ok; ++it, ++g) {
          const bool last = it + 1 == w.n_it;
          const bool more = !last || has_next;
          const int nkb = last ? (n + 1) & 1 : kb;
          const uint32_t u = 2 * g, un = u + 2;            // ring positions of this / the next step
          const uint32_t slot0 = u % NSLOT, slot1 = (u + 1) % NSLOT;
          const uint32_t nslot0 = un % NSLOT, nslot1 = (un + 1) % NSLOT;
          // ---- first half: its products, then the next step's scores over the same columns
          if (!wait_all(C::B_PF + 0, g & 1u, 1122)) { ok = false; break; }
          if (trace && g < 32) trace[512 + g * 8 + 0] = clock64();
          // the first products of an item overwrite dV / dK: the previous item's must have left
          if (it == 0 && n > 0 && !wait_all(C::B_EPI, (n - 1) & 1u, 1126)) { ok = false; break; }
          if (more) {
            if (last && !wait_all(C::B_KVF + nkb, ((n + 1) >> 1) & 1u, 1127)) { ok = false; break; }
            if (!wait_slots(un + 1)) { ok = false; break; }      // normally seen already
          }
          tc_fence_after();
          if (trace && g < 32) trace[g * 16 + 6] = clock64();
          if (elect_one()) {
            products(0, slot0, it > 0 ? 1u : 0u);
            if (more) scores(0, nslot0, nkb);
          }
          __syncwarp();
          if (trace && g < 32) trace[g * 16 + 7] = clock64();
          if (more && !wait_slots(un + 2)) { ok = false; break; }   // ahead of its use just below
          // ---- second half
          if (!wait_all(C::B_PF + 1, g & 1u, 1124)) { ok = false; break; }
          if (trace && g < 32) trace[512 + g * 8 + 1] = clock64();
          if (more && !wait_slots(un + 2)) { ok = false; break; }
          tc_fence_after();
          if (trace && g < 32) trace[g * 16 + 8] = clock64();
          if (elect_one()) {
            products(1, slot1, 1u);
            if (C::DQ_OWN_WARP && last) {
              umma_commit(bar(C::B_KVE + kb));   // no score product reads this K/V buffer any more
              umma_commit(bar(C::B_DONE));       // dV / dK of the item are complete
            }
            if (more) scores(1, nslot1, nkb);
          }
          __syncwarp();
          if (trace && g < 32) trace[g * 16 + 9] = clock64();
          if constexpr (!C::DQ_OWN_WARP) {
            // ---- dQ_i = dS . K_j over the whole tile, into the dQ buffer of this parity
            const int buf = g & 1;
            if (g >= 2) {
              if (!wait_all(C::B_DQE + buf, ((g >> 1) - 1) & 1u, 1125)) { ok = false; break; }
              tc_fence_after();
            }
            if (trace && g < 32) trace[g * 16 + 10] = clock64();
            if (elect_one()) {
              const uint64_t a = d_base + MN + (C::OFF_DST >> 4) + buf * (C::DST_BYTES >> 4);
              const uint64_t bk = dK_k0 + MN + kb * KB_STEP;
              const uint32_t d = tmem_u + C::DQ_COL + buf * DH;
              constexpr uint32_t idesc_dq = umma_idesc_bf16(BQ, DH, 1, 1);
#pragma unroll
              for (int kk = 0; kk < BKV / 16; ++kk)
                umma_bf16_ss(d, a + 128 * kk, bk + 128 * kk, idesc_dq, kk > 0 ? 1u : 0u);
              umma_commit(bar(C::B_DQF + buf));
              umma_commit(bar(C::B_DF + buf));
              if (last) {
                umma_commit(bar(C::B_KVE + kb));
                umma_commit(bar(C::B_DONE));
              }
            }
            __syncwarp();
            if (trace && g < 32) trace[g * 16 + 11] = clock64();
          }
          // nothing to issue until the softmax of the next step is through: the first slot of the
          // step after it (the second one was freed just now and is still being refilled)
          if (!wait_slots(un + 3)) { ok = false; break; }
        }
        w.next(p);
        ++n;
      }
    } else if (warp == 3) {
      // -------------------------------------------------------------- dV / dK store
      // The softmax warps stage an item's dV / dK in its K / V tiles; this warp (which has nothing
      // else to do and whose waits hold nobody up) stores the two tiles in bulk and hands the
      // K/V buffer back to the producer once the stores have read it.
      if (lane == 0) {
        uint32_t n = 0;
        bool stored = false;
        BwdWalk w;
        for (w.init(p); w.valid; w.next(p), ++n) {
          if (!mbar_wait(bar(C::B_STG), n & 1u, abort_flag)) {
            record_status(p.status, ST_WAIT_TIMEOUT, 1160);
            break;
          }
          const int kb = n & 1;
          tma_store_3d(&tmDV, sK(kb), w.h * DH, w.j * BKV, w.b);
          tma_store_3d(&tmDK, sV(kb), w.h * DH, w.j * BKV, w.b);
          tma_store_commit();
          tma_store_wait_read_all();
          mbar_arrive(bar(C::B_KVE + kb));
          stored = true;
        }
        if (stored) tma_store_wait_all();
      }
      __syncwarp();
    } else if (warp == 2 && C::DQ_OWN_WARP) {
      // -------------------------------------------------------------- MMA issuer: dQ
      // dQ_i = dS . K_j over the whole tile (dS^T from shared memory as the transposed operand),
      // into the dQ buffer of the step's parity, once both halves' dS^T are written.
      constexpr uint32_t idesc_dq = umma_idesc_bf16(BQ, DH, 1, 1);
      const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
      constexpr uint64_t MN = static_cast<uint64_t>(((BKV * 128) >> 4) - 1) << 16;
      const uint64_t d_base = umma_desc_sw128(sbase, 16, 1024) + MN;
      const uint64_t dK_mn0 = d_base + (C::OFF_K >> 4);
      const uint64_t dDST_mn0 = d_base + (C::OFF_DST >> 4);
      constexpr uint64_t KB_STEP = (2 * C::KV_BYTES) >> 4;
      constexpr uint64_t BUF_STEP = C::DST_BYTES >> 4;
      auto wait_all = [&](int b_idx, uint32_t parity, int where) {
        const bool got = mbar_wait_poll(bar(b_idx), parity, abort_flag);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0) record_status(p.status, ST_WAIT_TIMEOUT, where);
          return false;
        }
        return true;
      };
      long long* trace = (blockIdx.x == 0 && lane == 0) ? p.trace : nullptr;
      uint32_t n = 0, g = 0;
      bool ok = true;
      BwdWalk w;
      for (w.init(p); w.valid && ok; w.next(p), ++n) {
        const int kb = n & 1;
        for (int it = 0; it < w.n_it; ++it, ++g) {
          const int buf = g & 1;
          ok = wait_all(C::B_PF + 0, g & 1u, 1150) && wait_all(C::B_PF + 1, g & 1u, 1151);
          // the dQ of step g - 2 must have left this tensor-memory buffer
          if (ok && g >= 2) ok = wait_all(C::B_DQE + buf, ((g >> 1) - 1) & 1u, 1152);
          if (!ok) break;
          tc_fence_after();
          if (trace && g < 32) trace[g * 16 + 10] = clock64();
          if (elect_one()) {
            const uint64_t a = dDST_mn0 + buf * BUF_STEP;
            const uint64_t bk = dK_mn0 + kb * KB_STEP;
            const uint32_t d = tmem_u + C::DQ_COL + buf * DH;
#pragma unroll
            for (int kk = 0; kk < BKV / 16; ++kk)
              umma_bf16_ss(d, a + 128 * kk, bk + 128 * kk, idesc_dq, kk > 0 ? 1u : 0u);
            umma_commit(bar(C::B_DQF + buf));
            umma_commit(bar(C::B_DF + buf));
            if (it + 1 == w.n_it) {
              umma_commit(bar(C::B_KVE + kb));   // K_j is not read any more
              umma_commit(bar(C::B_DONE));
            }
          }
          __syncwarp();
          if (trace && g < 32) trace[g * 16 + 11] = clock64();
        }
      }
    }
  } else if (warp < 4 + 8 * C::NSUB) {
    // ---------------------------------------------------------------- softmax / dS of one half
    // Two threads per K/V row and half, 32 query columns each: four softmax warps per scheduler
    // hide the tensor-memory and shared-memory latencies of a step by multithreading, where two
    // threads with 64 columns each could not by instruction-level parallelism alone.
    const int sw_id = warp - 4;
    const int hf = sw_id / (4 * C::NSUB);
    const int sub = (sw_id >> 2) % C::NSUB;   // which 32 of the half's 64 query columns
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;        // K/V row within the tile = tensor-memory lane
    const int gt = (sw_id % (4 * C::NSUB)) * 32 + lane;   // index within the half's warps
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t s_addr = lane_addr + hf * 128 + sub * 32, d_addr = s_addr + 64;
    const float c = p.scale_log2;
    // the thread's share of a tile's statistics: lse (times log2 e) of one query column for the
    // first 64 threads, delta of one column for the others
    auto load_stat = [&](const BwdWalk& w, int it) {
      const size_t stat_base = (static_cast<size_t>(w.b) * p.nh + w.h) * p.S;
      const int qi = (w.i_start(p) + it) * BQ + hf * HQ + (gt & 63);
      if (gt >= 128) return 0.f;
      if (gt < 64) return qi < p.S ? p.lse[stat_base + qi] * 1.4426950408889634f : INFINITY;
      return qi < p.S ? p.delta[stat_base + qi] : 0.f;
    };
    // dV (first half's warps) or dK (second half's) of a finished item: tensor memory -> bf16 ->
    // the finished item's K (for dV) or V (for dK) tile in shared memory, which nothing reads any
    // more and which has the very layout of a 64-column swizzled store tile; warp 3 stores it in
    // bulk (a row per thread straight to global memory takes 32 separate 16-byte segments per
    // instruction and kept the load/store pipe busy for ~2000 clocks per item).
    auto epilogue = [&](uint32_t n_done) {
      const bool got = mbar_wait(bar(C::B_DONE), n_done & 1u, abort_flag);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) record_status(p.status, ST_WAIT_TIMEOUT, 1131);
        return false;
      }
      tc_fence_after();
      const float mul = hf == 0 ? 1.0f : p.scale;
      const int col = hf == 0 ? C::DV_COL : C::DK_COL;
      const uint32_t tile = (hf == 0 ? sK(n_done & 1) : sV(n_done & 1)) + quarter * 4096;
      const uint32_t trow = tile + lane * 128;
      uint32_t o0[32], o1[32];
      tmem_ld_32x32b_x32(lane_addr + col, o0);
      tmem_ld_32x32b_x32(lane_addr + col + 32, o1);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(C::B_EPI));       // dV / dK may be overwritten
#pragma unroll
      for (int gq = 0; gq < 8; ++gq) {
        const uint32_t* o = gq < 4 ? o0 + 8 * gq : o1 + 8 * (gq - 4);
        const uint32_t v0 = pack_bf16x2(__uint_as_float(o[0]) * mul, __uint_as_float(o[1]) * mul);
        const uint32_t v1 = pack_bf16x2(__uint_as_float(o[2]) * mul, __uint_as_float(o[3]) * mul);
        const uint32_t v2 = pack_bf16x2(__uint_as_float(o[4]) * mul, __uint_as_float(o[5]) * mul);
        const uint32_t v3 = pack_bf16x2(__uint_as_float(o[6]) * mul, __uint_as_float(o[7]) * mul);
        const uint32_t sw = static_cast<uint32_t>(gq ^ (lane & 7)) << 4;
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(trow + sw), "r"(v0), "r"(v1),
                     "r"(v2), "r"(v3) : "memory");
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(C::B_STG));       // warp 3 stores the tile
      return true;
    };
    uint32_t n = 0, g = 0;
    bool ok = true;
    BwdWalk w;
    w.init(p);
    float stat_next = w.valid ? load_stat(w, 0) : 0.f;
    while (ok && w.valid) {
      const int kv0 = w.j * BKV;
      const int kv_idx = kv0 + r;
      const int lim = kv_idx >= p.S ? INT_MAX : (p.causal ? kv_idx : INT_MIN);
      for (int it = 0; it < w.n_it; ++it, ++g) {
        const int q0 = (w.i_start(p) + it) * BQ;
        float* s_lse = s_stat + (g & 1) * 2 * BQ + hf * HQ;
        float* s_dl = s_lse + BQ;
        if (gt < 128) (gt < 64 ? s_lse : s_dl)[gt & 63] = stat_next;
        // the next step's statistics land during this step's work
        if (it + 1 < w.n_it) {
          stat_next = load_stat(w, it + 1);
        } else {
          const BwdWalk t = w.peek(p);
          if (t.valid) stat_next = load_stat(t, 0);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(C::B_STF + hf));
        bool got = mbar_wait(bar(C::B_STF + hf), g & 1u, abort_flag);
        // The dS^T buffer of this parity was last read by the dQ product of step g - 2.  When one
        // warp issues all MMAs that product was issued before this step's scores and has completed
        // before them (a thread's MMAs complete in issue order): no wait of its own.
        if (C::DQ_OWN_WARP && got && g > 1)
          got = mbar_wait(bar(C::B_DF + (g & 1)), ((g >> 1) - 1) & 1u, abort_flag);
        // the scores last: they are what this step is really waiting for, and every wait costs a
        // few hundred clocks even when its phase completed long ago
        if (got) got = mbar_wait_poll(bar(C::B_SF + hf), g & 1u, abort_flag);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0) record_status(p.status, ST_WAIT_TIMEOUT, 1130);
          ok = false;
          break;
        }
        tc_fence_after();
        long long* tr = (blockIdx.x == 0 && g < 32 && quarter == 0 && sub == 0 && lane == 0) ? p.trace : nullptr;
        if (tr) tr[g * 16 + hf * 3] = clock64();
        const bool mask = (p.causal && kv0 + BKV - 1 > q0) || (kv0 + BKV > p.S);
        // dS^T in shared memory: two groups of 64 query columns, each [128 K/V rows][128 bytes],
        // 128-byte swizzled (the layout the dQ product reads as a transposed A operand)
        const uint32_t srow = sDST(g & 1) + hf * (BKV * 128) + r * 128;
        // two chunks of 16 query columns.  P^T / dS^T (packed, 8 columns a chunk) go over columns
        // this thread has read before.
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
          uint32_t sv[16], dv[16], pk[8], dk[8];
          tmem_ld_32x32b_x16(s_addr + ch * 16, sv);
          tmem_ld_32x32b_x16(d_addr + ch * 16, dv);
          tmem_ld_wait();
          const int cq = sub * 32 + ch * 16;     // first query column of the chunk within the half
          if constexpr (DROP) {
            // hash group of (query q0 + hf HQ + cq, key kv_idx) in the [B nh S, S] matrix
            const unsigned long long gq =
                ((static_cast<unsigned long long>(w.b) * p.nh + w.h) * p.S + (q0 + hf * HQ + cq)) *
                    static_cast<unsigned long long>(p.S >> 2) + static_cast<unsigned long long>(kv_idx >> 2);
            bwd_chunk<true, true>(sv, dv, s_lse + cq, s_dl + cq, c, mask ? lim : INT_MIN,
                                  q0 + hf * HQ + cq, pk, dk, gq, static_cast<unsigned long long>(p.S >> 2),
                                  kv_idx & 3, p.drop_thr, p.drop_key, p.drop_scale);
          } else if (mask) {
            bwd_chunk<true, false>(sv, dv, s_lse + cq, s_dl + cq, c, lim, q0 + hf * HQ + cq, pk, dk);
          } else {
            bwd_chunk<false, false>(sv, dv, s_lse + cq, s_dl + cq, c, lim, 0, pk, dk);
          }
          tmem_st_32x32b_x8(s_addr + ch * 8, pk);
          tmem_st_32x32b_x8(d_addr + ch * 8, dk);
#pragma unroll
          for (int gq = 0; gq < 2; ++gq) {
            const uint32_t sw = static_cast<uint32_t>((sub * 4 + ch * 2 + gq) ^ (r & 7)) << 4;
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(srow + sw),
                         "r"(dk[4 * gq]), "r"(dk[4 * gq + 1]), "r"(dk[4 * gq + 2]), "r"(dk[4 * gq + 3])
                         : "memory");
          }
        }
        if (tr) tr[g * 16 + hf * 3 + 1] = clock64();
        tmem_st_wait();
        fence_proxy_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(C::B_PF + hf));
        if (tr) tr[g * 16 + hf * 3 + 2] = clock64();
        if (blockIdx.x == 0 && g < 32 && lane == 0 && sub == 0 && p.trace)
          p.trace[512 + 256 * hf + g * 8 + 2 + quarter] = clock64();
        // the previous item's dV / dK leave after this item's first softmax, whose scores were
        // issued while that item was finishing
        if (sub == 0 && it == 0 && n > 0 && !epilogue(n - 1)) { ok = false; break; }
      }
      w.next(p);
      ++n;
    }
    if (sub == 0 && ok && n > 0) epilogue(n - 1);
  } else {
    // ---------------------------------------------------------------- dQ drain
    // Each warp moves its 32 query rows on its own: tensor memory -> registers -> a swizzled
    // staging tile in shared memory -> bulk reduce-add into the fp32 accumulator (whole 128-byte
    // lines added in L2, against 32 separate 16-byte atomics per instruction from registers,
    // which kept the load/store pipe busy a third of the time).  Rows beyond the sequence are
    // dropped by the tensor map's bounds.
    const int quarter = warp & 3;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t stage = sbase + C::OFF_DQS + quarter * (C::DQS_BYTES / 4);   // 4 KB
    const uint32_t srow = stage + lane * 128;
    bool pending = false, ok = true;
    uint32_t g = 0;
    BwdWalk w;
    for (w.init(p); w.valid && ok; w.next(p)) {
      for (int it = 0; it < w.n_it; ++it, ++g) {
        const int buf = g & 1;
        const bool got = mbar_wait(bar(C::B_DQF + buf), (g >> 1) & 1u, abort_flag);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0) record_status(p.status, ST_WAIT_TIMEOUT, 1140);
          ok = false;
          break;
        }
        tc_fence_after();
        long long* trq = (blockIdx.x == 0 && g < 32 && quarter == 0 && lane == 0) ? p.trace : nullptr;
        if (trq) trq[g * 16 + 12] = clock64();
        const int qrow = (w.i_start(p) + it) * BQ + quarter * 32;
#pragma unroll 1
        for (int ch = 0; ch < 2; ++ch) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(lane_addr + C::DQ_COL + buf * DH + ch * 32, o);
          tmem_ld_wait();
          if (ch == 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(C::B_DQE + buf));   // the tensor-memory buffer is free
          }
          if (pending) {
            if (lane == 0) tma_store_wait_read_all();          // ... and so is the staging tile
            __syncwarp();
          }
#pragma unroll
          for (int gq = 0; gq < 8; ++gq) {
            const uint32_t sw = static_cast<uint32_t>(gq ^ (lane & 7)) << 4;
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(srow + sw), "r"(o[4 * gq]),
                         "r"(o[4 * gq + 1]), "r"(o[4 * gq + 2]), "r"(o[4 * gq + 3]) : "memory");
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (qrow < p.S) {
            if (lane == 0) {
              tma_reduce_add_3d(&tmDQ, stage, w.h * DH + ch * 32, qrow, w.b);
              tma_store_commit();
            }
            pending = true;
          }
        }
        if (trq) trq[g * 16 + 13] = clock64();
      }
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
  if (blockIdx.x == 0 && threadIdx.x == 0 && p.trace) p.trace[1089] = clock64();
}

}  // namespace

int launch_attn_bwd_dh64(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                         const CUtensorMap& tdo, const CUtensorMap& tdq, const CUtensorMap& tdk,
                         const CUtensorMap& tdv, const AttnBwdArgs& a, cudaStream_t st) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_bwd_dh64_kernel<false>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             B64::SMEM_BYTES) != cudaSuccess ||
        cudaFuncSetAttribute(attn_bwd_dh64_kernel<true>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             B64::SMEM_BYTES) != cudaSuccess)
      return -10;
    configured = true;
  }
  const int n_items = ((a.S + B64::BKV - 1) / B64::BKV) * a.B * a.nh;
  const int grid = n_items < sm_count() ? n_items : sm_count();
  if (a.drop_thr > 0)
    attn_bwd_dh64_kernel<true><<<grid, B64::THREADS, B64::SMEM_BYTES, st>>>(tq, tk, tv, tdo, tdq,
                                                                            tdk, tdv, a);
  else
    attn_bwd_dh64_kernel<false><<<grid, B64::THREADS, B64::SMEM_BYTES, st>>>(tq, tk, tv, tdo, tdq,
                                                                             tdk, tdv, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace cb
