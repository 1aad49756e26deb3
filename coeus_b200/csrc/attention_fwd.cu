// Flash-style attention forward on tcgen05 with the probabilities kept in tensor memory.
//
// Every CTA works on TWO 128-row query tiles of one (batch, head) at a time.  The work of an item
// is a stream of steps (query tile t, key tile j); step g uses score buffer g % NBUF of tensor
// memory, and the scores of step g + NBUF are issued as soon as P.V of step g has completed, so
// that (with three buffers) a softmax warpgroup finds its next scores computed when it finishes:
//   S  = Q_t . K_j^T      tcgen05.mma, operands in 128-byte-swizzled shared memory, S in TMEM
//   P  = exp2(S - m)      one thread per query row; P overwrites S in TMEM as packed bf16
//   O_t += P . V_j        tcgen05.mma with the A operand read from TMEM (no shared-memory trip)
// The S x S score matrix of the reference (plugins/model-transformer/src/lib.rs:237-277) is never
// materialised; causal masking is implicit (lib.rs:746-756) and fully-masked key tiles are skipped.
//
// Roles (384 threads, one CTA per SM, persistent over a heavy-first list of work items):
//   warp 0        TMA producer: Q_A, Q_B once per item, K_j / V_j through two rings
//   warp 1        MMA issue of O_t += P . V (warp-uniform control flow, one elected lane issues)
//   warp 2        MMA issue of the scores, NBUF steps ahead (same form)
//   warps 4..7    softmax of tile A (row r = 32 * (warp % 4) + lane, the TMEM lane it may read)
//   warps 8..11   softmax of tile B
// Online softmax in the exp2 domain with lazy rescaling of O (only when the running maximum grew
// by more than 2^8); optionally a quarter of the exponentials is evaluated as a cubic polynomial
// on the FMA pipe, because the exponential unit (16 results per clock per SM) bounds dh = 64.
// Grouped-query attention: query head h reads K/V head h / (nh / nkv).
// Every wait is bounded; a wait that runs out records a status code and the CTA leaves.
#include "common.cuh"
#include "ptx.cuh"

namespace cb {

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                      uint64_t ld, uint32_t box_inner, uint32_t box_outer);
int sm_count();

constexpr int AF_BM = 128;        // rows of one query tile
constexpr int AF_THREADS = 384;

struct AttnFwdArgs {
  int B, S, nh, nkv;
  __nv_bfloat16* O;
  int ldo;
  float* lse;          // [B, nh, S] natural-log LSE of the scaled scores
  float scale_log2;    // softmax scale * log2(e)
  int causal;
  int* status;
  // dropout on the probabilities (training only; drop_thr = 0: none): P is dropped before P.V,
  // the row sums and the LSE are those of the full softmax.  The mask is the one of
  // dropout_bits() over the [B*nh*S, S] probability matrix in row-major order (S % 4 == 0).
  int drop_thr;
  uint32_t drop_key;
  float drop_scale;
};

// Optional device timeline of CTA 0 (clock64 stamps; see cb_attn_fwd_set_trace): softmax warp 0
// of tile t writes five stamps per step at [t * 1024 + n * 8 + 0..4] (scores ready, scores in
// registers, maximum known, exponentials done, P handed over), the MMA warp two per step at
// [2048 + n * 8 + 0..1] (P ready, P.V issued and committed), the score warp at [.. + 2..3].
__device__ long long* g_attn_fwd_trace = nullptr;
__device__ int g_attn_fwd_trace_cta = 0;   // which CTA writes the step timeline

template <int DH>
struct AFCfg {
  static constexpr int BKV = 128;                       // keys per step
  static constexpr int NBUF = (DH == 64) ? 3 : 2;       // score buffers in tensor memory
  static constexpr int Q_BYTES = AF_BM * DH * 2;        // one query tile
  static constexpr int KV_BYTES = BKV * DH * 2;         // one K (or V) tile
  static constexpr int KST = (DH == 64) ? 3 : 2;        // ring depth of K and of V
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = 2 * Q_BYTES;
  static constexpr int OFF_V = OFF_K + KST * KV_BYTES;
  static constexpr int OFF_BAR = OFF_V + KST * KV_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 512;
  static constexpr int TMEM_COLS = 512;
  static constexpr int O_COL0 = 0;            // O_t (fp32, DH columns each)
  static constexpr int S_COL0 = 2 * DH;       // NBUF score buffers of BKV fp32 columns; P (bf16)
                                              // takes the first BKV / 2 columns of its buffer
  static_assert(S_COL0 + NBUF * BKV <= TMEM_COLS, "tensor memory budget");
  // barrier indices
  static constexpr int B_QF = 0, B_QE = 2, B_SF = 4, B_PR = B_SF + NBUF, B_BF = B_PR + NBUF,
                       B_KF = B_BF + NBUF, B_KE = B_KF + KST, B_VF = B_KE + KST,
                       B_VE = B_VF + KST, N_BARS = B_VE + KST;
};

// 2^x for x <= ~8 without the special-function unit and without conversion instructions (which
// share that unit): adding 1.5 * 2^23 rounded down leaves floor(x) in the low mantissa bits, so
// n = floor(x) and f = x - n come from three additions; 2^f is a cubic (relative error 8.6e-5,
// below bf16 resolution) and 2^n is added to the exponent field with a shift and an integer add.
__device__ __forceinline__ float exp2_poly(float x) {
  x = fmaxf(x, -120.0f);
  const float magic = 12582912.0f;
  const float fi = __fadd_rd(x, magic);
  const float f = x - (fi - magic);
  float p = 0.07710139f;
  p = fmaf(p, f, 0.22760755f);
  p = fmaf(p, f, 0.69512522f);
  p = fmaf(p, f, 1.0f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(fi) << 23));
}

// The steps of one CTA in the order every role walks them: items wave by wave (CTA c takes one
// item of every wave of gridDim.x items, counted from the front of even waves and from the back
// of odd ones, so that the heavy and the light ends of the sorted list meet in one CTA), within
// an item key tile by key tile, tile A before tile B.
struct AFWalk {
  // problem
  int n_items, n_bh, n_pairs, n_q_tiles, n_kv_tiles, nh, causal, bkv, n_waves;
  // position
  int wave, j, t;
  int b, h, qa;          // batch, head, first query tile of the pair
  int n0, n1, nmax;      // key tiles of tile A / B (0: the tile does not exist)
  int kv_seq;            // how many (item, j) groups came before this one: the K/V ring position
  bool valid;

  __device__ void init(const AttnFwdArgs& p, int bkv_) {
    bkv = bkv_;
    n_q_tiles = (p.S + AF_BM - 1) / AF_BM;
    n_kv_tiles = (p.S + bkv - 1) / bkv;
    n_pairs = (n_q_tiles + 1) / 2;
    nh = p.nh;
    n_bh = p.B * p.nh;
    n_items = n_pairs * n_bh;
    causal = p.causal;
    n_waves = (n_items + gridDim.x - 1) / gridDim.x;
    wave = -1;
    kv_seq = -1;
    valid = true;
    next_item();
  }
  __device__ void next_item() {
    while (true) {
      ++wave;
      if (wave >= n_waves) { valid = false; return; }
      const int c = (wave & 1) ? static_cast<int>(gridDim.x - 1 - blockIdx.x)
                               : static_cast<int>(blockIdx.x);
      const int i = wave * static_cast<int>(gridDim.x) + c;
      if (i >= n_items) continue;
      const int bh = i % n_bh;
      const int pair = n_pairs - 1 - i / n_bh;     // pairs with the most key tiles first
      b = bh / nh;
      h = bh % nh;
      qa = 2 * pair;
      n0 = causal ? min(n_kv_tiles, ((qa + 1) * AF_BM + bkv - 1) / bkv) : n_kv_tiles;
      n1 = qa + 1 >= n_q_tiles ? 0
           : (causal ? min(n_kv_tiles, ((qa + 2) * AF_BM + bkv - 1) / bkv) : n_kv_tiles);
      nmax = max(n0, n1);
      j = 0;
      t = 0;
      ++kv_seq;
      return;
    }
  }
  __device__ void advance() {
    if (t == 0 && j < n1) { t = 1; return; }
    ++j;
    if (j < nmax) {
      ++kv_seq;
      t = j < n0 ? 0 : 1;
      return;
    }
    next_item();
  }
  __device__ bool last_of_kv() const { return t == 1 || j >= n1; }   // last tile using K_j / V_j
  __device__ bool last_of_tile() const { return j == (t ? n1 : n0) - 1; }
};

template <int DH, bool POLY, bool DROP>
__global__ void __launch_bounds__(AF_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const AttnFwdArgs p) {
  using Cfg = AFCfg<DH>;
  constexpr int KST = Cfg::KST, NBUF = Cfg::NBUF, BKV = Cfg::BKV;
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + Cfg::N_BARS);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile uint32_t* seen = tmem_slot + 2;   // [t]: 1 + the last step whose scores tile t's warps saw
  auto bar = [&](int i) { return smem_u32(bars + i); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if ((sbase & 1023u) != 0u) {  // swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) record_status(p.status, ST_BAD_ARG, 950);
    return;
  }
  const int group = p.nh / p.nkv;

  if (threadIdx.x == 0) {
    for (int t = 0; t < 2; ++t) {
      mbar_init(bar(Cfg::B_QF + t), 1);
      mbar_init(bar(Cfg::B_QE + t), 1);
    }
    for (int s = 0; s < NBUF; ++s) {
      mbar_init(bar(Cfg::B_BF + s), 1);
      mbar_init(bar(Cfg::B_SF + s), 1);
      mbar_init(bar(Cfg::B_PR + s), 4);      // one arrival per softmax warp
    }
    for (int s = 0; s < KST; ++s) {
      mbar_init(bar(Cfg::B_KF + s), 1);
      mbar_init(bar(Cfg::B_KE + s), 1);
      mbar_init(bar(Cfg::B_VF + s), 1);
      mbar_init(bar(Cfg::B_VE + s), 1);
    }
    *abort_flag = 0;
    seen[0] = 0;
    seen[1] = 0;
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
  auto sQ = [&](int t) { return sbase + Cfg::OFF_Q + t * Cfg::Q_BYTES; };
  auto sK = [&](int s) { return sbase + Cfg::OFF_K + s * Cfg::KV_BYTES; };
  auto sV = [&](int s) { return sbase + Cfg::OFF_V + s * Cfg::KV_BYTES; };

  // The kernel starts with 168 registers per thread (384 threads); the first warpgroup (producer
  // and MMA issue: little state) hands registers to the two softmax warpgroups, whose step keeps a
  // whole score row plus the walk state in registers: 128 * (88 + 208 + 208) = 64512.
  if (threadIdx.x == 0 && g_attn_fwd_trace != nullptr)
    g_attn_fwd_trace[3072 + 2 * blockIdx.x] = static_cast<long long>(globaltimer_ns());
  if (warp < 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 88;" ::: "memory");
  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      uint32_t qcnt[2] = {0u, 0u};     // uses of each query buffer so far
      uint32_t kcnt = 0, vcnt = 0;     // K / V tiles loaded so far
      bool ok = true;
      AFWalk w;
      w.init(p, BKV);
      while (w.valid && ok) {
        const int row0 = w.b * p.S;
        const int h = w.h, hk = w.h / group, qa = w.qa;
        const int n0 = w.n0, n1 = w.n1, nmax = w.nmax;
        auto load_q = [&](int t) {
          if ((t == 0 ? n0 : n1) == 0) return;
          if (!mbar_wait(bar(Cfg::B_QE + t), (qcnt[t] & 1u) ^ 1u, abort_flag)) {
            record_status(p.status, ST_WAIT_TIMEOUT, 951);
            ok = false;
            return;
          }
          mbar_arrive_expect_tx(bar(Cfg::B_QF + t), Cfg::Q_BYTES);
#pragma unroll
          for (int c = 0; c < DH / 64; ++c)
            tma_load_2d(sQ(t) + c * (AF_BM * 128), &tmQ, bar(Cfg::B_QF + t), h * DH + c * 64,
                        row0 + (qa + t) * AF_BM);
          ++qcnt[t];
        };
        auto load_k = [&](int j) {
          const int s = kcnt % KST;
          if (!mbar_wait(bar(Cfg::B_KE + s), ((kcnt / KST) & 1u) ^ 1u, abort_flag)) {
            record_status(p.status, ST_WAIT_TIMEOUT, 952);
            ok = false;
            return;
          }
          mbar_arrive_expect_tx(bar(Cfg::B_KF + s), Cfg::KV_BYTES);
#pragma unroll
          for (int c = 0; c < DH / 64; ++c)
            tma_load_2d(sK(s) + c * (BKV * 128), &tmK, bar(Cfg::B_KF + s), hk * DH + c * 64,
                        row0 + j * BKV);
          ++kcnt;
        };
        auto load_v = [&](int j) {
          const int s = vcnt % KST;
          if (!mbar_wait(bar(Cfg::B_VE + s), ((vcnt / KST) & 1u) ^ 1u, abort_flag)) {
            record_status(p.status, ST_WAIT_TIMEOUT, 953);
            ok = false;
            return;
          }
          mbar_arrive_expect_tx(bar(Cfg::B_VF + s), Cfg::KV_BYTES);
#pragma unroll
          for (int c = 0; c < DH / 64; ++c)
            tma_load_2d(sV(s) + c * (BKV * 128), &tmV, bar(Cfg::B_VF + s), hk * DH + c * 64,
                        row0 + j * BKV);
          ++vcnt;
        };
        load_q(0);
        if (ok) load_k(0);
        if (ok) load_q(1);
        if (ok) load_v(0);
        for (int j = 1; j < nmax && ok; ++j) {
          load_k(j);
          if (ok) load_v(j);
        }
        w.next_item();
      }
      if (*abort_flag) {
        // let the copies already in flight land before shared memory is released
        const uint64_t t0 = globaltimer_ns();
        auto drain = [&](int full0, uint32_t cnt, int depth) {
          const uint32_t first = cnt > static_cast<uint32_t>(depth) ? cnt - depth : 0u;
          for (uint32_t u = first; u < cnt; ++u) {
            while (!mbar_try_wait(bar(full0 + u % depth), (u / depth) & 1u)) {
              if (globaltimer_ns() - t0 > 200000000ull) return;
            }
          }
        };
        drain(Cfg::B_KF, kcnt, KST);
        drain(Cfg::B_VF, vcnt, KST);
        for (int t = 0; t < 2; ++t)
          if (qcnt[t] > 0) drain(Cfg::B_QF + t, qcnt[t], 1);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issue: P.V
    // Two warps issue the tensor-core work because the issue cost of an MMA is of the order of
    // its run time at these tile sizes: this warp issues O_t += P.V for every step in order, warp
    // 2 the scores NBUF steps ahead.  Both run warp-uniform control flow with one elected lane
    // issuing (measured ~35 clocks per MMA against ~60-100 from a divergent single lane), and
    // build their descriptors once; a step only adds constants to the address field.
    {
      constexpr uint32_t idesc_o = umma_idesc_bf16(AF_BM, DH, 0, 1);
      const uint64_t dV0 = umma_desc_sw128(sV(0), BKV * 128, 1024);
      const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
      bool ok = true;
      int v_waited = -1;
      AFWalk wp;
      wp.init(p, BKV);
      for (uint32_t gp = 0; wp.valid && ok; wp.advance(), ++gp) {
        const uint32_t buf = gp % NBUF;
        const int t = wp.t;
        const int vs = wp.kv_seq % KST;
        if (v_waited != wp.kv_seq) {
          if (!mbar_wait(bar(Cfg::B_VF + vs), (wp.kv_seq / KST) & 1u, abort_flag)) {
            record_status(p.status, ST_WAIT_TIMEOUT, 962);
            break;
          }
          v_waited = wp.kv_seq;
        }
        if (!mbar_wait(bar(Cfg::B_PR + buf), (gp / NBUF) & 1u, abort_flag)) {
          record_status(p.status, ST_WAIT_TIMEOUT, 964);
          break;
        }
        long long* tr = (blockIdx.x == g_attn_fwd_trace_cta && gp < 120 && lane == 0) ? g_attn_fwd_trace : nullptr;
        if (tr) tr[2048 + gp * 8] = clock64();
        tc_fence_after();
        const uint64_t bd0 = dV0 + static_cast<uint64_t>((vs * Cfg::KV_BYTES) >> 4);
        const uint32_t d_addr = tmem_u + Cfg::O_COL0 + t * DH;
        const uint32_t a_addr = tmem_u + Cfg::S_COL0 + buf * BKV;
        const uint32_t acc0 = wp.j > 0 ? 1u : 0u;
        const bool last_kv = wp.last_of_kv();
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < BKV / 16; ++kk)
            umma_bf16_ts(d_addr, a_addr + kk * 8, bd0 + static_cast<uint64_t>((kk * 2048) >> 4),
                         idesc_o, kk > 0 ? 1u : acc0);
          umma_commit(bar(Cfg::B_BF + buf));     // P consumed, O_t updated
          if (last_kv) umma_commit(bar(Cfg::B_VE + vs));
        }
        __syncwarp();
        if (tr) tr[2048 + gp * 8 + 1] = clock64();
      }
    }
    __syncwarp();
  } else if (warp == 2) {
    // ---------------------------------------------------------------- MMA issue: scores
    {
      constexpr uint32_t idesc_s = umma_idesc_bf16(AF_BM, BKV, 0, 0);
      const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
      const uint64_t dQ0 = umma_desc_sw128(sQ(0), 16, 1024);
      const uint64_t dK0 = umma_desc_sw128(sK(0), 16, 1024);
      uint32_t qc0 = 0u, qc1 = 0u;
      int k_waited = -1;
      bool ok = true;
      auto wait1 = [&](int b_idx, uint32_t parity, int where) {
        if (!mbar_wait(bar(b_idx), parity, abort_flag)) {
          record_status(p.status, ST_WAIT_TIMEOUT, where);
          ok = false;
        }
        return ok;
      };
      AFWalk ws;
      ws.init(p, BKV);
      for (uint32_t gs = 0; ws.valid && ok; ws.advance(), ++gs) {
        const int t = ws.t;
        const uint32_t buf = gs % NBUF;
        // the buffer is free once P.V of the step that used it last has completed
        if (gs >= NBUF && !wait1(Cfg::B_BF + buf, ((gs / NBUF) - 1u) & 1u, 963)) break;
        if (ws.j == 0) {
          if (!wait1(Cfg::B_QF + t, (t ? qc1 : qc0) & 1u, 960)) break;
          if (t) ++qc1; else ++qc0;
        }
        const int ks = ws.kv_seq % KST;
        if (k_waited != ws.kv_seq) {
          if (!wait1(Cfg::B_KF + ks, (ws.kv_seq / KST) & 1u, 961)) break;
          k_waited = ws.kv_seq;
        }
        long long* tr = (blockIdx.x == g_attn_fwd_trace_cta && gs < 120 && lane == 0) ? g_attn_fwd_trace : nullptr;
        if (tr) tr[2048 + gs * 8 + 2] = clock64();
        tc_fence_after();
        const uint64_t ad0 = dQ0 + static_cast<uint64_t>((t * Cfg::Q_BYTES) >> 4);
        const uint64_t bd0 = dK0 + static_cast<uint64_t>((ks * Cfg::KV_BYTES) >> 4);
        const uint32_t d_addr = tmem_u + Cfg::S_COL0 + buf * BKV;
        const bool last_tile = ws.last_of_tile(), last_kv = ws.last_of_kv();
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < DH / 16; ++kk) {
            const uint64_t a_off = static_cast<uint64_t>(((kk / 4) * (AF_BM * 128) + (kk % 4) * 32) >> 4);
            const uint64_t b_off = static_cast<uint64_t>(((kk / 4) * (BKV * 128) + (kk % 4) * 32) >> 4);
            umma_bf16_ss(d_addr, ad0 + a_off, bd0 + b_off, idesc_s, kk > 0 ? 1u : 0u);
          }
          umma_commit(bar(Cfg::B_SF + buf));
          if (last_tile) umma_commit(bar(Cfg::B_QE + t));   // Q_t's buffer may be refilled
          if (last_kv) umma_commit(bar(Cfg::B_KE + ks));
        }
        __syncwarp();
        if (tr) tr[2048 + gs * 8 + 3] = clock64();
      }
    }
    __syncwarp();
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;" ::: "memory");
    // ---------------------------------------------------------------- softmax + epilogue
    const int t = (warp - 4) >> 2;             // which query tile of the pair
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;         // query row within the tile = TMEM lane
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t o_addr = lane_addr + Cfg::O_COL0 + t * DH;
    uint32_t g = 0, g_prev = 0, mine = 0, own_seen = 0;
    bool ok = true;
    float m_used = -INFINITY;
    float l[4] = {0.f, 0.f, 0.f, 0.f};           // the row sum is kept as four partial sums
    AFWalk w;
    w.init(p, BKV);
    for (; w.valid && ok; w.advance(), ++g) {
      if (w.t != t) continue;
      const int j = w.j;
      const int q0 = (w.qa + t) * AF_BM;
      const int q_idx = q0 + r;
      if (j == 0) {
        m_used = -INFINITY;
        l[0] = l[1] = l[2] = l[3] = 0.f;
      }
      const uint32_t buf = g % NBUF;
      const uint32_t s_addr = lane_addr + Cfg::S_COL0 + buf * BKV;
      // The parity wait below is only meaningful once the scores of step g - NBUF (the previous
      // use of this barrier) are known to be complete: with that phase still open, the wait for
      // the opposite parity would return at once.  A warpgroup's own recent steps imply it; after
      // sitting out several steps (an item with a single query tile; key tiles that only tile B
      // sees under a causal mask) the other warpgroup's published progress does: it owned all the
      // steps in between, none of which depends on this warpgroup.
      {
        const uint32_t need = g >= NBUF ? g - NBUF + 1u : 0u;
        if (own_seen < need) {
          bool got = true;
          if (seen[1 - t] < need) {
            const uint64_t t0 = globaltimer_ns();
            uint32_t n = 0;
            while (seen[1 - t] < need) {
              if ((++n & 63u) == 0u) {
                if (*abort_flag) { got = false; break; }
                if (globaltimer_ns() - t0 > CB_WAIT_LIMIT_NS) {
                  *abort_flag = 1u;
                  got = false;
                  break;
                }
              }
            }
          }
          if (!__all_sync(0xffffffffu, got)) {
            if (lane == 0) record_status(p.status, ST_WAIT_TIMEOUT, 973);
            ok = false;
            break;
          }
        }
      }
      {
        const bool got = mbar_wait(bar(Cfg::B_SF + buf), (g / NBUF) & 1u, abort_flag);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0) record_status(p.status, ST_WAIT_TIMEOUT, 970);
          ok = false;
          break;
        }
      }
      own_seen = g + 1u;
      if (quarter == 0 && lane == 0) seen[t] = g + 1u;   // one writer per tile: monotonic
      long long* tr = (blockIdx.x == g_attn_fwd_trace_cta && mine < 120 && quarter == 0 && lane == 0)
                          ? g_attn_fwd_trace : nullptr;
      const uint32_t tri = t * 1024 + mine * 8;
      ++mine;
      if (tr) tr[tri] = clock64();
      tc_fence_after();
      const int kv0 = j * BKV;
      const bool need_mask = (p.causal && kv0 + BKV - 1 > q0) || (kv0 + BKV > p.S);
      const int kv_limit = p.causal ? min(q_idx, p.S - 1) : (p.S - 1);  // last visible key
      uint32_t v[BKV];
#pragma unroll
      for (int c = 0; c < BKV / 32; ++c) tmem_ld_32x32b_x32(s_addr + c * 32, v + c * 32);
      tmem_ld_wait();
      if (tr) tr[tri + 1] = clock64();
      if (need_mask) {
        // hidden keys get a score of -inf, after which the step takes the common path (their
        // exponential is an exact zero); with causal masking every row sees at least key 0
#pragma unroll
        for (int e = 0; e < BKV; ++e)
          if (kv0 + e > kv_limit) v[e] = 0xff800000u;
      }
      float mx;
      {
        float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
        for (int e = 0; e < BKV; e += 8) {     // four chains of three-input maxima
          m0 = max3(m0, __uint_as_float(v[e]), __uint_as_float(v[e + 1]));
          m1 = max3(m1, __uint_as_float(v[e + 2]), __uint_as_float(v[e + 3]));
          m2 = max3(m2, __uint_as_float(v[e + 4]), __uint_as_float(v[e + 5]));
          m3 = max3(m3, __uint_as_float(v[e + 6]), __uint_as_float(v[e + 7]));
        }
        mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
      }
      mx *= p.scale_log2;  // scale > 0, so max commutes with it
      const float m_new = fmaxf(m_used, mx);
      const bool grow = (m_new - m_used) > 8.0f;  // also true for the first step (m_used = -inf)
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        // O_t may be rescaled once P.V of the previous step of this tile has completed.  (The
        // wait is skipped when no row needs rescaling: the barrier of that buffer cannot advance
        // a second time before this step hands over its P, so no phase is missed.)
        const bool got = mbar_wait(bar(Cfg::B_BF + g_prev % NBUF), (g_prev / NBUF) & 1u, abort_flag);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0) record_status(p.status, ST_WAIT_TIMEOUT, 972);
          ok = false;
          break;
        }
        tc_fence_after();
        const float f = grow ? fast_exp2(m_used - m_new) : 1.0f;
#pragma unroll 1
        for (int c = 0; c < DH / 16; ++c) {
          uint32_t o[16];
          tmem_ld_32x32b_x16(o_addr + c * 16, o);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 16; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * f);
          tmem_st_32x32b_x16(o_addr + c * 16, o);
        }
#pragma unroll
        for (int a = 0; a < 4; ++a) l[a] *= f;
      }
      g_prev = g;
      if (grow) m_used = (m_new == -INFINITY) ? 0.f : m_new;
      // P = exp2(s * scale - m) as packed bf16 over the first half of the score buffer; row sum
      const float sc = p.scale_log2, nm = -m_used;
      if (tr) tr[tri + 2] = clock64();
      if constexpr (DROP) {
        // four consecutive keys share one hash; the index of this row's first key of the tile is
        // a multiple of four (S and the tile width are)
        const unsigned long long g0 =
            ((static_cast<unsigned long long>(w.b) * p.nh + w.h) * p.S + q_idx) *
                static_cast<unsigned long long>(p.S >> 2) + static_cast<unsigned long long>(kv0 >> 2);
#pragma unroll
        for (int c = 0; c < BKV / 32; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 32; e += 4) {
            const uint32_t bits = dropout_bits(g0 + (c * 32 + e) / 4, p.drop_key);
            float pe[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              pe[j] = fast_exp2(fmaf(__uint_as_float(v[c * 32 + e + j]), sc, nm));
              l[j] += pe[j];
              pe[j] *= dropout_factor(bits, j, p.drop_thr, p.drop_scale);
            }
            pk[e >> 1] = pack_bf16x2(pe[0], pe[1]);
            pk[(e >> 1) + 1] = pack_bf16x2(pe[2], pe[3]);
          }
          tmem_st_32x32b_x16(s_addr + c * 16, pk);
        }
      } else {
#pragma unroll
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const float t0 = fmaf(__uint_as_float(v[c * 32 + e]), sc, nm);
          const float t1 = fmaf(__uint_as_float(v[c * 32 + e + 1]), sc, nm);
          float p0, p1;
          if (POLY && (e & 6) == 6) {       // columns 6, 7 of every 8: a quarter of the row
            p0 = exp2_poly(t0);
            p1 = exp2_poly(t1);
          } else {
            p0 = fast_exp2(t0);
            p1 = fast_exp2(t1);
          }
          l[(e >> 1) & 3] += p0 + p1;
          pk[e >> 1] = pack_bf16x2(p0, p1);
        }
        tmem_st_32x32b_x16(s_addr + c * 16, pk);
      }
      }
      if (tr) tr[tri + 3] = clock64();
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(Cfg::B_PR + buf));
      if (tr) tr[tri + 4] = clock64();
      if (!w.last_of_tile()) continue;
      // ---- last step of this tile: O_t / l and the LSE leave once its P.V has completed
      {
        const bool got = mbar_wait(bar(Cfg::B_BF + buf), (g / NBUF) & 1u, abort_flag);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0) record_status(p.status, ST_WAIT_TIMEOUT, 971);
          ok = false;
          break;
        }
      }
      tc_fence_after();
      const float lsum = (l[0] + l[1]) + (l[2] + l[3]);
      const float inv_l = lsum > 0.f ? 1.0f / lsum : 0.f;
      const bool row_ok = q_idx < p.S;
      __nv_bfloat16* orow =
          p.O + (static_cast<size_t>(w.b) * p.S + q_idx) * p.ldo + static_cast<size_t>(w.h) * DH;
#pragma unroll 1
      for (int c = 0; c < DH / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(o_addr + c * 32, o);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int gq = 0; gq < 4; ++gq) {
            uint4 wv;
            wv.x = pack_bf16x2(__uint_as_float(o[8 * gq + 0]) * inv_l, __uint_as_float(o[8 * gq + 1]) * inv_l);
            wv.y = pack_bf16x2(__uint_as_float(o[8 * gq + 2]) * inv_l, __uint_as_float(o[8 * gq + 3]) * inv_l);
            wv.z = pack_bf16x2(__uint_as_float(o[8 * gq + 4]) * inv_l, __uint_as_float(o[8 * gq + 5]) * inv_l);
            wv.w = pack_bf16x2(__uint_as_float(o[8 * gq + 6]) * inv_l, __uint_as_float(o[8 * gq + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + c * 32 + gq * 8) = wv;
          }
        }
      }
      if (row_ok && p.lse != nullptr)
        p.lse[(static_cast<size_t>(w.b) * p.nh + w.h) * p.S + q_idx] =
            (m_used + log2f(lsum)) * 0.6931471805599453f;
      tc_fence_before();   // these reads of O_t precede the next item's first P.V (ordered by B_PR)
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && g_attn_fwd_trace != nullptr)
    g_attn_fwd_trace[3072 + 2 * blockIdx.x + 1] = static_cast<long long>(globaltimer_ns());
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

template <int DH, bool POLY, bool DROP = false>
static int launch_attn_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                              const AttnFwdArgs& a, int max_ctas, cudaStream_t st) {
  using Cfg = AFCfg<DH>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_fwd_kernel<DH, POLY, DROP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg::SMEM_BYTES) != cudaSuccess)
      return -10;
    configured = true;
  }
  const int n_q_tiles = (a.S + AF_BM - 1) / AF_BM;
  const int items = ((n_q_tiles + 1) / 2) * a.B * a.nh;
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (items < grid) grid = items;
  attn_fwd_kernel<DH, POLY, DROP><<<grid, AF_THREADS, Cfg::SMEM_BYTES, st>>>(tq, tk, tv, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace cb

// Device buffer of at least 3072 + 2 * (number of CTAs) int64 for the timeline of CTA `cta` and
// the start / end times (globaltimer) of every CTA at [3072 + 2 * c]; nullptr switches it off.
extern "C" int cb_attn_fwd_set_trace(long long* device_buffer, int cta) {
  if (cudaMemcpyToSymbol(cb::g_attn_fwd_trace_cta, &cta, sizeof(cta)) != cudaSuccess) return -1;
  return cudaMemcpyToSymbol(cb::g_attn_fwd_trace, &device_buffer, sizeof(device_buffer)) == cudaSuccess ? 0 : -1;
}

// q: bf16 [B*S, nh*dh] view (row pitch ldq); k, v: bf16 [B*S, nkv*dh] views (pitches ldk, ldv;
// nkv divides nh, query head h reads K/V head h / (nh / nkv)); they may be column slices of one
// fused projection output.  o: [B*S, nh*dh] pitch ldo.  lse: fp32 [B, nh, S].
// poly != 0 evaluates a quarter of the exponentials as a polynomial on the FMA pipe.
// drop_thr in [0, 255] (0: no dropout; needs S % 4 == 0 otherwise), drop_key: see AttnFwdArgs.
extern "C" int cb_attn_fwd_dropout(const void* q, const void* k, const void* v, void* o, float* lse,
                                   int B, int S, int nh, int nkv, int dh, int ldq, int ldk,
                                   int ldv, int ldo, float scale, int causal, int poly,
                                   int drop_thr, unsigned int drop_key, int* status, int max_ctas,
                                   void* stream) {
  using namespace cb;
  if (dh != 64 && dh != 128) return -1;
  if (B <= 0 || S <= 0 || nh <= 0 || nkv <= 0 || (nh % nkv) != 0 || (ldo % 8) != 0) return -2;
  if (drop_thr < 0 || drop_thr > 255 || (drop_thr > 0 && (S % 4) != 0)) return -6;
  CUtensorMap tq, tk, tv;
  const uint64_t rows = static_cast<uint64_t>(B) * S;
  const uint32_t bkv = dh == 64 ? AFCfg<64>::BKV : AFCfg<128>::BKV;
  if (make_tmap_bf16_2d(&tq, q, static_cast<uint64_t>(nh) * dh, rows, ldq, 64, AF_BM) != 0) return -3;
  if (make_tmap_bf16_2d(&tk, k, static_cast<uint64_t>(nkv) * dh, rows, ldk, 64, bkv) != 0) return -4;
  if (make_tmap_bf16_2d(&tv, v, static_cast<uint64_t>(nkv) * dh, rows, ldv, 64, bkv) != 0) return -5;
  AttnFwdArgs a;
  a.B = B; a.S = S; a.nh = nh; a.nkv = nkv;
  a.O = static_cast<__nv_bfloat16*>(o);
  a.ldo = ldo;
  a.lse = lse;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.causal = causal;
  a.status = status;
  a.drop_thr = drop_thr;
  a.drop_key = drop_key;
  a.drop_scale = 256.0f / static_cast<float>(256 - drop_thr);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (drop_thr > 0)
    return dh == 64 ? launch_attn_fwd<64, false, true>(tq, tk, tv, a, max_ctas, st)
                    : launch_attn_fwd<128, false, true>(tq, tk, tv, a, max_ctas, st);
  if (poly)
    return dh == 64 ? launch_attn_fwd<64, true>(tq, tk, tv, a, max_ctas, st)
                    : launch_attn_fwd<128, true>(tq, tk, tv, a, max_ctas, st);
  return dh == 64 ? launch_attn_fwd<64, false>(tq, tk, tv, a, max_ctas, st)
                  : launch_attn_fwd<128, false>(tq, tk, tv, a, max_ctas, st);
}

extern "C" int cb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                           int B, int S, int nh, int nkv, int dh, int ldq, int ldk, int ldv,
                           int ldo, float scale, int causal, int poly, int* status, int max_ctas,
                           void* stream) {
  return cb_attn_fwd_dropout(q, k, v, o, lse, B, S, nh, nkv, dh, ldq, ldk, ldv, ldo, scale, causal,
                             poly, 0, 0u, status, max_ctas, stream);
}
