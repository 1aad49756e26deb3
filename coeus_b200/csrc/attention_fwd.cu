// Flash-style attention forward on tcgen05: S = Q.K^T and O += P.V run on the tensor cores with
// S and O in tensor memory; the S x S score matrix of the reference
// (plugins/model-transformer/src/lib.rs:237-277) is never materialised.  Causal masking is
// implicit (lower triangle incl. diagonal, lib.rs:746-756) and fully-masked K/V tiles are skipped.
//
// One CTA handles one (batch, head, 128-row query tile):
//   warp 0      TMA producer: Q once, then K_j / V_j tiles through a 2-stage ring
//   warp 1      MMA issuer:  S = Q.K_j^T  (SS, fp32 in TMEM), O += P_j.V_j (P from shared memory)
//   warps 2..5  softmax: one thread per query row; online softmax in the exp2 domain with lazy
//               rescaling of O (only when the running max grew by more than 2^8), P written as
//               bf16 into 128-byte-swizzled shared memory, final O / l and LSE written out.
// Two CTAs are resident per SM (256 TMEM columns and ~112 KB shared memory each), so one CTA's
// softmax overlaps the other's MMAs.
#include "common.cuh"
#include "ptx.cuh"

namespace cb {

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                      uint64_t ld, uint32_t box_inner, uint32_t box_outer);

constexpr int ATT_BM = 128;      // query rows per CTA
constexpr int ATT_THREADS = 192;

struct AttnFwdArgs {
  int B, S, nh;
  __nv_bfloat16* O;
  int ldo;
  float* lse;          // [B, nh, S] natural-log LSE of the scaled scores
  float scale_log2;    // softmax scale * log2(e)
  int causal;
  int* status;
};

template <int DH>
struct AttnCfg {
  static constexpr int BKV = (DH == 64) ? 128 : 64;
  static constexpr int Q_BYTES = ATT_BM * DH * 2;
  static constexpr int KV_BYTES = BKV * DH * 2;      // one of K or V
  static constexpr int P_BYTES = ATT_BM * BKV * 2;
  static constexpr int STAGES = 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_KV = Q_BYTES;
  static constexpr int OFF_P = OFF_KV + STAGES * 2 * KV_BYTES;
  static constexpr int OFF_BAR = OFF_P + P_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 128;
  static constexpr int TMEM_COLS = 256;
  static constexpr int S_COL = 0;
  static constexpr int O_COL = 128;
};

template <int DH>
__global__ void __launch_bounds__(ATT_THREADS, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnFwdArgs p) {
  using Cfg = AttnCfg<DH>;
  constexpr int BKV = Cfg::BKV;
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  // 0 q_full | 1,2 k_full | 3,4 v_full | 5,6 kv_empty | 7 s_full | 8 p_full | 9 pv_done
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 10);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  auto bar = [&](int i) { return smem_u32(bars + i); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if ((sbase & 1023u) != 0u) {  // swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) record_status(p.status, ST_BAD_ARG, 900);
    return;
  }

  const int n_q_tiles = (p.S + ATT_BM - 1) / ATT_BM;
  const int bh = blockIdx.x % (p.B * p.nh);
  const int q_tile = n_q_tiles - 1 - blockIdx.x / (p.B * p.nh);  // heavy (late) tiles first
  const int b = bh / p.nh, h = bh % p.nh;
  const int q0 = q_tile * ATT_BM;
  const int kv_end = p.causal ? min(p.S, q0 + ATT_BM) : p.S;
  const int n_kv = (kv_end + BKV - 1) / BKV;

  if (threadIdx.x == 0) {
    mbar_init(bar(0), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(1 + s), 1);
      mbar_init(bar(3 + s), 1);
      mbar_init(bar(5 + s), 1);
    }
    mbar_init(bar(7), 1);
    mbar_init(bar(8), 128);
    mbar_init(bar(9), 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t sQ = sbase + Cfg::OFF_Q;
  const uint32_t sP = sbase + Cfg::OFF_P;
  auto sK = [&](int st) { return sbase + Cfg::OFF_KV + st * 2 * Cfg::KV_BYTES; };
  auto sV = [&](int st) { return sK(st) + Cfg::KV_BYTES; };

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      const int row0 = b * p.S;
      mbar_arrive_expect_tx(bar(0), Cfg::Q_BYTES);
#pragma unroll
      for (int c = 0; c < DH / 64; ++c)
        tma_load_2d(sQ + c * (ATT_BM * 128), &tmQ, bar(0), h * DH + c * 64, row0 + q0);
      int issued = 0;
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1u;
        if (!mbar_wait(bar(5 + st), ph ^ 1u, abort_flag)) {
          record_status(p.status, ST_WAIT_TIMEOUT, 910);
          break;
        }
        mbar_arrive_expect_tx(bar(1 + st), Cfg::KV_BYTES);
#pragma unroll
        for (int c = 0; c < DH / 64; ++c)
          tma_load_2d(sK(st) + c * (BKV * 128), &tmK, bar(1 + st), h * DH + c * 64,
                      row0 + j * BKV);
        mbar_arrive_expect_tx(bar(3 + st), Cfg::KV_BYTES);
#pragma unroll
        for (int c = 0; c < DH / 64; ++c)
          tma_load_2d(sV(st) + c * (BKV * 128), &tmV, bar(3 + st), h * DH + c * 64,
                      row0 + j * BKV);
        ++issued;
      }
      if (*abort_flag) {
        // let the copies already in flight land before shared memory is released
        const uint64_t t0 = globaltimer_ns();
        for (int i = max(0, issued - 2); i < issued; ++i) {
          const int st = i & 1;
          const uint32_t ph = (i >> 1) & 1u;
          while (!(mbar_try_wait(bar(1 + st), ph) && mbar_try_wait(bar(3 + st), ph))) {
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
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(ATT_BM, BKV, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc_bf16(ATT_BM, DH, 0, 1);
      bool ok = mbar_wait(bar(0), 0, abort_flag);
      if (!ok) record_status(p.status, ST_WAIT_TIMEOUT, 920);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1u;
        if (!mbar_wait(bar(1 + st), ph, abort_flag)) {
          record_status(p.status, ST_WAIT_TIMEOUT, 921);
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
          const uint64_t ad =
              umma_desc_sw128(sQ + (kk / 4) * (ATT_BM * 128) + (kk % 4) * 32, 16, 1024);
          const uint64_t bd =
              umma_desc_sw128(sK(st) + (kk / 4) * (BKV * 128) + (kk % 4) * 32, 16, 1024);
          umma_bf16_ss(tmem_base + Cfg::S_COL, ad, bd, idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(bar(7));
        if (!mbar_wait(bar(8), j & 1u, abort_flag)) {
          record_status(p.status, ST_WAIT_TIMEOUT, 922);
          break;
        }
        if (!mbar_wait(bar(3 + st), ph, abort_flag)) {
          record_status(p.status, ST_WAIT_TIMEOUT, 923);
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          const uint64_t ad =
              umma_desc_sw128(sP + (kk / 4) * (ATT_BM * 128) + (kk % 4) * 32, 16, 1024);
          const uint64_t bd = umma_desc_sw128(sV(st) + kk * 2048, BKV * 128, 1024);
          umma_bf16_ss(tmem_base + Cfg::O_COL, ad, bd, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(bar(5 + st));
        umma_commit(bar(9));
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- softmax + epilogue
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;       // query row within the tile
    const int q_idx = q0 + r;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    float m_used = -INFINITY, l = 0.f, l1 = 0.f;   // the row sum is kept as two partial sums
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const bool got = mbar_wait(bar(7), j & 1u, abort_flag);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) record_status(p.status, ST_WAIT_TIMEOUT, 930);
        ok = false;
        break;
      }
      tc_fence_after();
      const int kv0 = j * BKV;
      const bool need_mask = (p.causal && kv0 + BKV - 1 > q0) || (kv0 + BKV > p.S);
      const int kv_limit = p.causal ? min(q_idx, p.S - 1) : (p.S - 1);  // last visible kv index
      // The whole score row goes to registers with back-to-back TMEM loads and one wait, so the
      // load latency is paid once per tile and S is read from tensor memory only once.
      uint32_t v[BKV];
#pragma unroll
      for (int c = 0; c < BKV / 32; ++c) tmem_ld_32x32b_x32(lane_addr + Cfg::S_COL + c * 32, v + c * 32);
      tmem_ld_wait();
      float mx = -INFINITY;
      if (need_mask) {
#pragma unroll
        for (int e = 0; e < BKV; ++e)
          if (kv0 + e <= kv_limit) mx = fmaxf(mx, __uint_as_float(v[e]));
      } else {
        float mx1 = -INFINITY;      // two chains of three-input maxima
#pragma unroll
        for (int e = 0; e < BKV; e += 4) {
          mx = max3(mx, __uint_as_float(v[e]), __uint_as_float(v[e + 1]));
          mx1 = max3(mx1, __uint_as_float(v[e + 2]), __uint_as_float(v[e + 3]));
        }
        mx = fmaxf(mx, mx1);
      }
      mx *= p.scale_log2;  // scale > 0, so max commutes with it
      const float m_new = fmaxf(m_used, mx);
      const bool grow = (m_new - m_used) > 8.0f;  // also true for the first tile (m_used = -inf)
      // P's shared-memory buffer and O are free once the previous P.V finished
      if (j > 0) {
        const bool got2 = mbar_wait(bar(9), (j - 1) & 1u, abort_flag);
        if (!__all_sync(0xffffffffu, got2)) {
          if (lane == 0) record_status(p.status, ST_WAIT_TIMEOUT, 931);
          ok = false;
          break;
        }
        tc_fence_after();
        if (__any_sync(0xffffffffu, grow)) {
          const float f = grow ? fast_exp2(m_used - m_new) : 1.0f;
#pragma unroll 1
          for (int c = 0; c < DH / 16; ++c) {
            uint32_t o[16];
            tmem_ld_32x32b_x16(lane_addr + Cfg::O_COL + c * 16, o);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 16; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * f);
            tmem_st_32x32b_x16(lane_addr + Cfg::O_COL + c * 16, o);
          }
          tmem_st_wait();
          l *= f;
          l1 *= f;
        }
      }
      if (grow) m_used = (m_new == -INFINITY) ? 0.f : m_new;
      // P = exp2(s * scale - m), row sum, bf16 P into swizzled shared memory
#pragma unroll
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float t0, t1;
          fma2(t0, t1, __uint_as_float(v[c * 32 + e]), __uint_as_float(v[c * 32 + e + 1]),
               p.scale_log2, p.scale_log2, -m_used, -m_used);
          float p0 = fast_exp2(t0);
          float p1 = fast_exp2(t1);
          if (need_mask) {
            if (kv0 + c * 32 + e > kv_limit) p0 = 0.f;
            if (kv0 + c * 32 + e + 1 > kv_limit) p1 = 0.f;
          }
          add2(l, l1, l, l1, p0, p1);
          pk[e >> 1] = pack_bf16x2(p0, p1);
        }
        // columns [c*32, c*32+32) of row r: half = (c*32)/64, 16-byte chunks (c*4 % 8)..+3
        const uint32_t row_base = sP + ((c * 32) / 64) * (ATT_BM * 128) + r * 128;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const uint32_t chunk = static_cast<uint32_t>(((c * 4) & 7) + g);
          const uint32_t addr = row_base + ((chunk ^ (r & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk[4 * g]),
                       "r"(pk[4 * g + 1]), "r"(pk[4 * g + 2]), "r"(pk[4 * g + 3])
                       : "memory");
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(bar(8));
    }
    if (ok) {
      const bool got = mbar_wait(bar(9), (n_kv - 1) & 1u, abort_flag);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) record_status(p.status, ST_WAIT_TIMEOUT, 932);
        ok = false;
      }
    }
    if (ok) {
      tc_fence_after();
      l += l1;
      const float inv_l = l > 0.f ? 1.0f / l : 0.f;
      const bool row_ok = q_idx < p.S;
      __nv_bfloat16* orow =
          p.O + (static_cast<size_t>(b) * p.S + q_idx) * p.ldo + static_cast<size_t>(h) * DH;
#pragma unroll 1
      for (int c = 0; c < DH / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(lane_addr + Cfg::O_COL + c * 32, o);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(o[8 * g + 0]) * inv_l, __uint_as_float(o[8 * g + 1]) * inv_l);
            w.y = pack_bf16x2(__uint_as_float(o[8 * g + 2]) * inv_l, __uint_as_float(o[8 * g + 3]) * inv_l);
            w.z = pack_bf16x2(__uint_as_float(o[8 * g + 4]) * inv_l, __uint_as_float(o[8 * g + 5]) * inv_l);
            w.w = pack_bf16x2(__uint_as_float(o[8 * g + 6]) * inv_l, __uint_as_float(o[8 * g + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = w;
          }
        }
      }
      if (row_ok && p.lse != nullptr)
        p.lse[(static_cast<size_t>(b) * p.nh + h) * p.S + q_idx] =
            (m_used + log2f(l)) * 0.6931471805599453f;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

template <int DH>
static int launch_attn_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                           const AttnFwdArgs& a, cudaStream_t st) {
  using Cfg = AttnCfg<DH>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_fwd_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg::SMEM_BYTES) != cudaSuccess)
      return -10;
    configured = true;
  }
  const int n_q_tiles = (a.S + ATT_BM - 1) / ATT_BM;
  const int grid = n_q_tiles * a.B * a.nh;
  attn_fwd_kernel<DH><<<grid, ATT_THREADS, Cfg::SMEM_BYTES, st>>>(tq, tk, tv, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace cb

// q, k, v: bf16, token-major [B*S, nh*dh] views with row pitches ldq / ldk / ldv (elements); they
// may alias one fused [B*S, 3*nh*dh] buffer.  o: [B*S, nh*dh] pitch ldo.  lse: fp32 [B, nh, S].
extern "C" int cb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                           int B, int S, int nh, int dh, int ldq, int ldk, int ldv, int ldo,
                           float scale, int causal, int* status, void* stream) {
  using namespace cb;
  if (dh != 64 && dh != 128) return -1;
  if (B <= 0 || S <= 0 || nh <= 0 || (ldo % 8) != 0) return -2;
  CUtensorMap tq, tk, tv;
  const uint64_t rows = static_cast<uint64_t>(B) * S;
  const uint32_t bkv = dh == 64 ? 128 : 64;
  if (make_tmap_bf16_2d(&tq, q, static_cast<uint64_t>(nh) * dh, rows, ldq, 64, ATT_BM) != 0) return -3;
  if (make_tmap_bf16_2d(&tk, k, static_cast<uint64_t>(nh) * dh, rows, ldk, 64, bkv) != 0) return -4;
  if (make_tmap_bf16_2d(&tv, v, static_cast<uint64_t>(nh) * dh, rows, ldv, 64, bkv) != 0) return -5;
  AttnFwdArgs a;
  a.B = B; a.S = S; a.nh = nh;
  a.O = static_cast<__nv_bfloat16*>(o);
  a.ldo = ldo;
  a.lse = lse;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.causal = causal;
  a.status = status;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dh == 64 ? launch_attn_fwd<64>(tq, tk, tv, a, st) : launch_attn_fwd<128>(tq, tk, tv, a, st);
}
