// bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM, operands
// staged by TMA into 128-byte-swizzled shared memory), persistent and warp-specialised:
//   warp 0      TMA producer (one lane)
//   warp 1      MMA issuer   (one lane)
//   warps 2..5  epilogue: TMEM -> registers -> fused epilogue -> swizzled shared memory -> TMA
//               store (bf16 outputs; fp32 and atomic outputs are stored directly)
// The accumulator is double-buffered in TMEM so the epilogue of tile i overlaps the main
// loop of tile i+1.  Both operands may be K-major or MN-major, which covers the three GEMMs
// of a linear layer whose weight is stored [in, out] row-major (the layout of math::matmul in
// the reference, plugins/model-transformer/src/lib.rs:50-74):
//   forward  Y[M,N]  = X[M,K]   . W[K,N]      A K-major,  B MN-major
//   dgrad    dX[M,K] = dY[M,N]  . W[K,N]^T    A K-major,  B K-major
//   wgrad    dW[K,N] = X[M,K]^T . dY[M,N]     A MN-major, B MN-major (split along tokens,
//                                             fp32 atomic accumulation)
// Fused epilogues: alpha scale, +bias[N], GELU(tanh) with the pre-activation kept, dGELU,
// +residual, bf16 / fp32 / fp32-atomic-add output.
#include <cudaTypedefs.h>

#include <cstring>

#include "common.cuh"
#include "ptx.cuh"

namespace cb {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_THREADS = 192;
constexpr int AG_PARTS = 8;   // row groups a pulled tile is split into
constexpr int MAX_TP = 8;
enum : int { COMM_NONE = 0, COMM_AG = 1, COMM_RS = 2 };

enum : int { EPI_NONE = 0, EPI_GELU = 1, EPI_DGELU = 2, EPI_SWIGLU_BWD = 3 };
enum : int { OUT_BF16 = 0, OUT_F32 = 1, OUT_F32_ATOMIC = 2, OUT_DISCARD = 3 };

struct GemmArgs {
  int M, N, K;
  void* D;
  int ldd;
  const __nv_bfloat16* bias;    // [N] or null
  const __nv_bfloat16* resid;   // [M, N] (ldr) or null
  int ldr;
  const __nv_bfloat16* aux_in;  // [M, N] (ldaux): pre-activation for EPI_DGELU
  __nv_bfloat16* aux_out;       // [M, N] (ldaux): pre-activation written by EPI_GELU
  int ldaux;
  int epi;
  int out_mode;
  float alpha;
  int ksplit;
  int tma_store;                // bf16 outputs leave through shared memory and TMA stores
  int drop_thr;                 // dropout on the value before the residual is added: bytes below
  uint32_t drop_key;            // drop_thr (= round(p * 256)) drop the element; 0 = off
  float drop_scale;             // 256 / (256 - drop_thr)
  int* status;
  // ---- grouped GEMM (experts stacked along the row dimension of every operand's memory)
  int group_m;                  // output rows per group; 0 = one group.  Group g of a tile adds
  int g_am, g_ak;               // g * g_am to A's m coordinate, g * g_ak to its k coordinate,
  int g_bn, g_bk;               // g * g_bn to B's n coordinate, g * g_bk to its k coordinate
  // ---- fused collectives over peer memory (COMM template parameter)
  int tp, rank;                 // ranks of the tensor-parallel group, this rank
  int tiles_per_shard;          // 128-row tiles per rank's sequence shard
  const void* ag_src[MAX_TP];   // COMM_AG: every rank's copy of the gathered operand (peer mapped)
  __nv_bfloat16* ag_dst;        //          this rank's copy (the A operand of the GEMM)
  int ag_ld;                    //          its row pitch (elements)
  uint32_t* ag_flags;           //          local per-tile arrival counters: AG_PARTS per epoch,
                                //          zero before the first use and never reset
  uint32_t ag_epoch;
  const uint64_t* peer_flags;   //          local signal pad: peer_flags[s] >= peer_expect once
  uint64_t peer_expect;         //          rank s has written its shard
  uint64_t wait_limit_ns;
  void* rs_dst[MAX_TP];         // COMM_RS: rank s's receive slot for this rank's partial rows
  int rs_ld;
};

constexpr int GEMM_STAGING_BYTES = 32768;   // two [128 rows x 64 bf16] swizzled store tiles

constexpr int PULL_SLOT_BYTES = 16384;      // one bulk copy of the all-gather pull ring

// The all-gather variant gives up one pipeline stage for a ring of bulk-copy slots through which
// one thread streams the peers' rows (peer memory -> shared memory -> the local gather buffer).
// CTA2: two CTAs of a cluster share one 256 x BN tile; each stages its 128 rows of A and half of
// the B rows, so a stage is 32 KB and six stages fit.
// AUX2 (CTA pairs only): the epilogue that stores two tensors per step (the activation and the
// kept pre-activation of the fused GELU) gets two pairs of store tiles, paid for with one pipeline
// stage, so that it no longer waits for its own stores after every 64 columns.
template <int BN, int COMM = 0, bool CTA2 = false, bool AUX2 = false>
struct GemmCfg {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = (CTA2 ? BN / 2 : BN) * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES =
      CTA2 ? (AUX2 ? 5 : 6) : ((BN == 256) ? 4 : 6) - (COMM == 1 ? 1 : 0);
  static constexpr int PULL_SLOTS = COMM == 1 ? STAGE_BYTES / PULL_SLOT_BYTES : 0;
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int STAGING_BYTES = AUX2 ? 2 * GEMM_STAGING_BYTES : GEMM_STAGING_BYTES;
  static constexpr int OFF_STAGING = STAGES * STAGE_BYTES;
  static constexpr int OFF_PULL = OFF_STAGING + STAGING_BYTES;
  static constexpr int OFF_BAR = OFF_PULL + PULL_SLOTS * PULL_SLOT_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 1024 /*align*/ + 256 /*barriers*/;
};

// Fused epilogue math on 32 consecutive columns of one output row.  `u` receives the
// pre-activation when EPI_GELU keeps it.
__device__ __forceinline__ void epilogue_math(const GemmArgs& p, float* v, float* u, int row,
                                              int col0, int ncols, bool row_ok) {
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] *= p.alpha;
  if (p.bias != nullptr) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      if (g * 8 < ncols) {
        const uint4 b = *reinterpret_cast<const uint4*>(p.bias + col0 + g * 8);
        const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(bw[j]);
          v[g * 8 + 2 * j] += f.x;
          v[g * 8 + 2 * j + 1] += f.y;
        }
      }
    }
  }
  if (p.epi == EPI_GELU) {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      u[j] = v[j];
      v[j] = gelu_tanh(v[j]);
    }
  } else if (p.epi == EPI_DGELU && row_ok) {
    const __nv_bfloat16* ap = p.aux_in + static_cast<size_t>(row) * p.ldaux + col0;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      if (g * 8 < ncols) {
        const uint4 a = *reinterpret_cast<const uint4*>(ap + g * 8);
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(aw[j]);
          v[g * 8 + 2 * j] *= gelu_tanh_grad(f.x);
          v[g * 8 + 2 * j + 1] *= gelu_tanh_grad(f.y);
        }
      }
    }
  }
  if (p.drop_thr > 0) {
    // the 32 columns start on a multiple of 32: eight hash groups of four elements
    const unsigned long long g0 =
        (static_cast<unsigned long long>(row) * static_cast<unsigned long long>(p.N) + col0) >> 2;
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      const uint32_t h = dropout_bits(g0 + g, p.drop_key);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        v[g * 4 + j] = static_cast<int>((h >> (8 * j)) & 255u) < p.drop_thr ? 0.f
                                                                             : v[g * 4 + j] * p.drop_scale;
    }
  }
  if (p.resid != nullptr && row_ok) {
    const __nv_bfloat16* rp = p.resid + static_cast<size_t>(row) * p.ldr + col0;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      if (g * 8 < ncols) {
        const uint4 a = *reinterpret_cast<const uint4*>(rp + g * 8);
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(aw[j]);
          v[g * 8 + 2 * j] += f.x;
          v[g * 8 + 2 * j + 1] += f.y;
        }
      }
    }
  }
}

__device__ __forceinline__ uint4 pack8(const float* v) {
  uint4 o;
  o.x = pack_bf16x2(v[0], v[1]);
  o.y = pack_bf16x2(v[2], v[3]);
  o.z = pack_bf16x2(v[4], v[5]);
  o.w = pack_bf16x2(v[6], v[7]);
  return o;
}

// 32 bf16 columns of row r into a 128-byte-swizzled [128 x 64] store tile; `half` selects
// columns 0..31 or 32..63 of the tile.
__device__ __forceinline__ void stage_row(uint32_t tile, int r, int half, const float* v) {
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const uint4 o = pack8(v + g * 8);
    const uint32_t chunk = static_cast<uint32_t>(half * 4 + g);
    const uint32_t addr = tile + r * 128 + ((chunk ^ (r & 7)) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(o.x), "r"(o.y),
                 "r"(o.z), "r"(o.w) : "memory");
  }
}

__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t ld_acquire_sys_u64_g(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// COMM_AG: the A operand is the all-gather of per-rank row shards.  Two extra warps of every
// CTA pull the other ranks' shards over NVLink (plain peer loads) into this GPU's own copy, 128
// rows at a time, and publish a per-tile flag; the TMA producer waits for the flag of a remote
// tile and then loads it from LOCAL memory.  Tiles are visited local shard first, then the
// peers in ring order, which is also the order of the pulls.
// COMM_RS: the result is reduce-scattered by rows.  The epilogue pushes each tile of partial
// sums straight into the owner rank's receive slot (coalesced peer stores from the staging
// tile); the owner adds the slots in its next kernel.
template <int BN, bool A_MN, bool B_MN, int COMM, bool CTA2 = false, bool AUX2 = false>
__global__ void __launch_bounds__(COMM == COMM_AG ? GEMM_THREADS + 32 : GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmD, const __grid_constant__ CUtensorMap tmAux,
                 const GemmArgs p) {
  static_assert(!CTA2 || (COMM == COMM_NONE && BN == 256), "CTA pairs: plain 256-wide GEMM only");
  static_assert(!AUX2 || CTA2, "the doubled store tiles exist for CTA pairs");
  using Cfg = GemmCfg<BN, COMM, CTA2, AUX2>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int TILE_M = CTA2 ? 2 * GEMM_BM : GEMM_BM;     // rows of one (cluster) tile
  const uint32_t cta_rank = CTA2 ? cluster_ctarank() : 0u;  // 0 = the CTA that issues the MMAs
  const int first_tile = CTA2 ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int tile_step = CTA2 ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_aligned + Cfg::OFF_BAR);
  // bars[0..S) full, [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2 * STAGES + 4);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile int* epi_ok = reinterpret_cast<volatile int*>(tmem_slot + 2);
  const uint32_t s_staging = smem_base + Cfg::OFF_STAGING;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  auto full_bar = [&](int s) { return smem_u32(bars + s); };
  auto empty_bar = [&](int s) { return smem_u32(bars + STAGES + s); };
  auto tfull_bar = [&](int a) { return smem_u32(bars + 2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return smem_u32(bars + 2 * STAGES + 2 + a); };
  auto pull_bar = [&](int s) { return smem_u32(bars + 2 * STAGES + 6 + s); };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), CTA2 ? 256 : 128);   // pair: both CTAs' epilogues report to rank 0
    }
    for (int s = 0; s < Cfg::PULL_SLOTS; ++s) mbar_init(pull_bar(s), 1);
    *abort_flag = 0;
    *epi_ok = 1;
    *(epi_ok + 1) = 1;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (p.tma_store) tma_prefetch_desc(&tmD);
  }
  if (warp == 0) {
    if constexpr (CTA2) {
      tmem_alloc_cg2(smem_u32(const_cast<uint32_t*>(tmem_slot)), Cfg::TMEM_COLS);
      tmem_relinquish_cg2();
    } else {
      tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), Cfg::TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (CTA2) cluster_sync_all();   // the peer's barriers exist before anything targets them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_m = (p.M + TILE_M - 1) / TILE_M;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int kblocks = (p.K + GEMM_BK - 1) / GEMM_BK;
  const int kb_per = (kblocks + p.ksplit - 1) / p.ksplit;
  const int total = tiles_m * tiles_n * p.ksplit;
  // With a fused collective the m-blocks are visited starting at this rank's own shard.
  auto m_block_of = [&](int tile) {
    const int mi = tile / tiles_n;
    if constexpr (COMM == COMM_NONE) return mi;
    else return (mi + p.rank * p.tiles_per_shard) % tiles_m;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t armed = 0;  // number of stage fills issued
      bool ok = true;
      for (int w = first_tile; w < total && ok; w += tile_step) {
        const int split = w % p.ksplit;
        const int tile = w / p.ksplit;
        const int m_blk = m_block_of(tile);
        const int m0 = m_blk * TILE_M + static_cast<int>(cta_rank) * GEMM_BM;
        const int n0 = (tile % tiles_n) * BN;
        const int kb0 = split * kb_per;
        const int kb1 = min(kblocks, kb0 + kb_per);
        // grouped GEMM: the tile's group shifts where its operands start
        const int grp = p.group_m > 0 ? (m_blk * TILE_M) / p.group_m : 0;
        const int am0 = m0 + grp * p.g_am, ak0 = grp * p.g_ak;
        const int bn_off = grp * p.g_bn, bk0 = grp * p.g_bk;
        if constexpr (COMM == COMM_AG) {
          if (m_blk / p.tiles_per_shard != p.rank) {  // rows that come from a peer
            const uint64_t t0 = globaltimer_ns();
            uint32_t n = 0;
            // the tile arrives in AG_PARTS row groups, each adding one to the tile's counter
            while (ld_acquire_gpu_u32(p.ag_flags + m_blk) < p.ag_epoch * AG_PARTS) {
              if ((++n & 15u) == 0u &&
                  (*abort_flag || globaltimer_ns() - t0 > p.wait_limit_ns)) {
                *abort_flag = 1u;
                record_status(p.status, ST_COMM_TIMEOUT, m_blk);
                ok = false;
                break;
              }
            }
            if (!ok) break;
            asm volatile("fence.proxy.async.global;" ::: "memory");  // generic writes -> TMA reads
          }
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
            record_status(p.status, ST_WAIT_TIMEOUT, 100);
            ok = false;
            break;
          }
          const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES;
          const uint32_t sB = sA + Cfg::A_BYTES;
          if constexpr (CTA2) {
            // both CTAs fill their own stage; all bytes are counted on rank 0's barrier, which
            // rank 0 arms for the pair
            const uint32_t fb = mapa_shared(full_bar(stage), 0u);
            if (cta_rank == 0u) mbar_arrive_expect_tx(full_bar(stage), 2 * Cfg::STAGE_BYTES);
            // this CTA's half of B
            const int nb = n0 + bn_off + static_cast<int>(cta_rank) * (BN / 2);
            if constexpr (!A_MN) {
              tma_load_2d_cg2(sA, &tmA, fb, kb * GEMM_BK + ak0, am0);
            } else {
#pragma unroll
              for (int c = 0; c < GEMM_BM / 64; ++c)
                tma_load_2d_cg2(sA + c * 8192, &tmA, fb, am0 + c * 64, kb * GEMM_BK + ak0);
            }
            if constexpr (!B_MN) {
              tma_load_2d_cg2(sB, &tmB, fb, kb * GEMM_BK + bk0, nb);
            } else {
#pragma unroll
              for (int c = 0; c < BN / 128; ++c)
                tma_load_2d_cg2(sB + c * 8192, &tmB, fb, nb + c * 64, kb * GEMM_BK + bk0);
            }
          } else {
          const uint32_t fb = full_bar(stage);
          mbar_arrive_expect_tx(fb, Cfg::STAGE_BYTES);
          if constexpr (!A_MN) {
            tma_load_2d(sA, &tmA, fb, kb * GEMM_BK + ak0, am0);
          } else {
#pragma unroll
            for (int c = 0; c < GEMM_BM / 64; ++c)
              tma_load_2d(sA + c * 8192, &tmA, fb, am0 + c * 64, kb * GEMM_BK + ak0);
          }
          if constexpr (!B_MN) {
            tma_load_2d(sB, &tmB, fb, kb * GEMM_BK + bk0, n0 + bn_off);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sB + c * 8192, &tmB, fb, n0 + bn_off + c * 64, kb * GEMM_BK + bk0);
          }
          }
          ++armed;
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok && cta_rank == 0u) {
        // Let copies that were already issued land before the CTA's shared memory goes away
        // (rank 0's barriers also count the peer's bytes; both CTAs stay until the final
        // cluster barrier).
        const uint32_t n_wait = armed < (uint32_t)STAGES ? armed : (uint32_t)STAGES;
        for (uint32_t i = 0; i < n_wait; ++i) {
          const uint32_t idx = armed - 1 - i;  // fill index
          const int s = idx % STAGES;
          const uint32_t par = (idx / STAGES) & 1u;
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(full_bar(s), par)) {
            if (globaltimer_ns() - t0 > 200000000ull) break;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp runs the control flow (addresses and descriptors stay warp-uniform, which
    // makes the issue of an MMA markedly cheaper than from a divergent single lane); one elected
    // lane issues.  The descriptors of stage 0 are built once; a k-step adds constants to them.
    if (cta_rank == 0u) {
      constexpr uint32_t idesc = umma_idesc_bf16(TILE_M, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
      const uint64_t dA0 = A_MN ? umma_desc_sw128(smem_base, 8192, 1024)
                                : umma_desc_sw128(smem_base, 16, 1024);
      const uint64_t dB0 = B_MN ? umma_desc_sw128(smem_base + Cfg::A_BYTES, 8192, 1024)
                                : umma_desc_sw128(smem_base + Cfg::A_BYTES, 16, 1024);
      constexpr uint64_t STAGE_STEP = Cfg::STAGE_BYTES >> 4;
      constexpr uint64_t A_K_STEP = (A_MN ? 2048 : 32) >> 4, B_K_STEP = (B_MN ? 2048 : 32) >> 4;
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      auto wait_all = [&](uint32_t b_addr, uint32_t parity, int where) {
        const bool got = mbar_wait(b_addr, parity, abort_flag);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0) record_status(p.status, ST_WAIT_TIMEOUT, where);
          ok = false;
        }
        return ok;
      };
      for (int w = first_tile; w < total && ok; w += tile_step, ++it) {
        const int split = w % p.ksplit;
        const int kb0 = split * kb_per;
        const int kb1 = min(kblocks, kb0 + kb_per);
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1u;
        if (!wait_all(tempty_bar(acc), acc_phase ^ 1u, 200)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_u + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!wait_all(full_bar(stage), phase, 201)) break;
          tc_fence_after();
          const uint64_t ad0 = dA0 + stage * STAGE_STEP, bd0 = dB0 + stage * STAGE_STEP;
          const uint32_t acc_first = kb > kb0 ? 1u : 0u;
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < GEMM_BK / 16; ++k) {
              if constexpr (CTA2)
                umma_bf16_ss_cg2(tmem_d, ad0 + k * A_K_STEP, bd0 + k * B_K_STEP, idesc,
                                 k > 0 ? 1u : acc_first);
              else
                umma_bf16_ss(tmem_d, ad0 + k * A_K_STEP, bd0 + k * B_K_STEP, idesc,
                             k > 0 ? 1u : acc_first);
            }
            if constexpr (CTA2) umma_commit_cg2(empty_bar(stage), 3);   // frees the stage in both CTAs
            else umma_commit(empty_bar(stage));
          }
          __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) {
          if (elect_one()) {
            if constexpr (CTA2) umma_commit_cg2(tfull_bar(acc), 3);     // both epilogues may drain
            else umma_commit(tfull_bar(acc));
          }
          __syncwarp();
        }
      }
    }
    __syncwarp();
  } else if (COMM == COMM_AG && warp >= 6) {
    // ------------------------------------------------------------------ all-gather pull
    // One thread streams this CTA's share of the peers' rows through a ring of shared-memory
    // slots with bulk copies: peer memory -> slot (completion on the slot's mbarrier), slot ->
    // local gather buffer (bulk group).  No registers hold data, PULL_SLOTS - 1 loads are in
    // flight per SM at all times, and nothing drains between row groups: a group's arrival
    // counter is raised when the bulk group of its last chunk has completed.
    if constexpr (COMM == COMM_AG) {
      if (lane == 0) {
        constexpr int NS = Cfg::PULL_SLOTS;
        constexpr int PART_ROWS = GEMM_BM / AG_PARTS;
        const uint32_t s_pull = smem_base + Cfg::OFF_PULL;
        const int n_units = (p.tp - 1) * p.tiles_per_shard * AG_PARTS;
        const size_t row_bytes = static_cast<size_t>(p.K) * 2;
        const bool contig = p.ag_ld == p.K;           // a row group is one contiguous run
        const int runs = contig ? 1 : PART_ROWS;
        const size_t run_bytes = contig ? PART_ROWS * row_bytes : row_bytes;
        const int chunks_per_run = static_cast<int>((run_bytes + PULL_SLOT_BYTES - 1) / PULL_SLOT_BYTES);
        const int chunks_per_unit = runs * chunks_per_run;
        const int my_units = n_units > static_cast<int>(blockIdx.x)
                                 ? (n_units - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
        const long total = static_cast<long>(my_units) * chunks_per_unit;
        uint32_t ready = 1u << p.rank;                // peers whose buffers may be read
        bool ok = true;
        struct Chunk { const char* src; char* dst; uint32_t bytes; int m_blk; bool last; };
        auto chunk_of = [&](long j) {
          const int ui = static_cast<int>(j / chunks_per_unit), rem = static_cast<int>(j % chunks_per_unit);
          const int c = blockIdx.x + ui * gridDim.x;
          const int tile_c = c / AG_PARTS, part = c % AG_PARTS;
          const int src = (p.rank + tile_c / p.tiles_per_shard + 1) % p.tp;
          const int m_blk = src * p.tiles_per_shard + tile_c % p.tiles_per_shard;
          const int run = rem / chunks_per_run, ch = rem % chunks_per_run;
          const size_t row = static_cast<size_t>(m_blk) * GEMM_BM + part * PART_ROWS + (contig ? 0 : run);
          const size_t off = row * p.ag_ld * 2 + static_cast<size_t>(ch) * PULL_SLOT_BYTES;
          const size_t left = run_bytes - static_cast<size_t>(ch) * PULL_SLOT_BYTES;
          Chunk k;
          k.src = static_cast<const char*>(p.ag_src[src]) + off;
          k.dst = reinterpret_cast<char*>(p.ag_dst) + off;
          k.bytes = static_cast<uint32_t>(left < PULL_SLOT_BYTES ? left : PULL_SLOT_BYTES);
          k.m_blk = m_blk;
          k.last = rem == chunks_per_unit - 1;
          if (!(ready >> src & 1u)) {                 // first touch of this peer: is its shard written?
            const uint64_t t0 = globaltimer_ns();
            uint32_t n = 0;
            while (ld_acquire_sys_u64_g(p.peer_flags + src) < p.peer_expect) {
              if ((++n & 15u) == 0u && (*abort_flag || globaltimer_ns() - t0 > p.wait_limit_ns)) {
                *abort_flag = 1u;
                record_status(p.status, ST_COMM_TIMEOUT, src);
                ok = false;
                break;
              }
            }
            ready |= 1u << src;
          }
          return k;
        };
        auto issue_load = [&](long j) {
          const Chunk k = chunk_of(j);
          if (!ok) return;
          const int slot = static_cast<int>(j % NS);
          mbar_arrive_expect_tx(pull_bar(slot), k.bytes);
          bulk_load_g2s(s_pull + slot * PULL_SLOT_BYTES, k.src, k.bytes, pull_bar(slot));
        };
        int pend_blk[2] = {-1, -1};                    // counters to raise once older groups finish
        auto raise = [&](int m_blk) {
          asm volatile("fence.proxy.async.global;" ::: "memory");
          asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.ag_flags + m_blk) : "memory");
        };
        long loads = 0, done_j = 0;               // loads issued / loads waited for
        for (; loads < total && loads < NS && ok; ++loads) issue_load(loads);
        if (!ok && loads > 0) --loads;               // the load that found its peer missing was not issued
        for (long j = 0; j < total && ok; ++j) {
          const int slot = static_cast<int>(j % NS);
          if (!mbar_wait(pull_bar(slot), static_cast<uint32_t>(j / NS) & 1u, abort_flag)) {
            record_status(p.status, ST_WAIT_TIMEOUT, 600);
            ok = false;
            break;
          }
          done_j = j + 1;
          const Chunk k = chunk_of(j);
          fence_proxy_async_smem();
          bulk_store_s2g(k.dst, s_pull + slot * PULL_SLOT_BYTES, k.bytes);
          tma_store_commit();
          // groups older than the two most recent have completed: their rows are in place
          asm volatile("cp.async.bulk.wait_group 2;" ::: "memory");
          if (pend_blk[0] >= 0) raise(pend_blk[0]);
          pend_blk[0] = pend_blk[1];
          pend_blk[1] = k.last ? k.m_blk : -1;
          // the store before this one has read its slot: refill it
          asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          if (j >= 1 && loads < total) {
            issue_load(loads);
            if (ok) ++loads;
          }
        }
        tma_store_wait_all();
        if (!ok) {
          // let the loads that were issued but not consumed land before the shared memory goes away
          for (long i2 = done_j; i2 < loads; ++i2) {
            const uint64_t t0 = globaltimer_ns();
            while (!mbar_try_wait(pull_bar(static_cast<int>(i2 % NS)),
                                  static_cast<uint32_t>(i2 / NS) & 1u)) {
              if (globaltimer_ns() - t0 > 200000000ull) break;
            }
          }
        }
        if (ok) {
          if (pend_blk[0] >= 0) raise(pend_blk[0]);
          if (pend_blk[1] >= 0) raise(pend_blk[1]);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const bool leader = (warp == 2 && lane == 0);
    const bool aux_staged = p.tma_store && p.epi == EPI_GELU && p.aux_out != nullptr;
    int it = 0;
    uint32_t step = 0;  // running count of staged 64-column steps (selects the store tile)
    for (int w = first_tile; w < total; w += tile_step, ++it) {
      const int tile = w / p.ksplit;
      const int m_blk = m_block_of(tile);
      const int m0 = m_blk * TILE_M + static_cast<int>(cta_rank) * GEMM_BM;
      const int n0 = (tile % tiles_n) * BN;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      const bool got = mbar_wait(tfull_bar(acc), acc_phase, abort_flag);
      // The four epilogue warps must take the same decision: they meet at named barriers below.
      if (!__all_sync(0xffffffffu, got) && lane == 0) {
        *epi_ok = 0;
        record_status(p.status, ST_WAIT_TIMEOUT, 300);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*epi_ok == 0) break;
      tc_fence_after();
      const int r_in_tile = q * 32 + lane;
      const int row = m0 + r_in_tile;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      if (p.tma_store) {
#pragma unroll 1
        for (int qs = 0; qs < BN / 64; ++qs) {
          const int colq = n0 + qs * 64;
          if (colq >= p.N) break;
          const uint32_t buf = AUX2 ? (step & 1u) : (aux_staged ? 0u : (step & 1u));
          const uint32_t s_out = s_staging + buf * (AUX2 ? 32768 : 16384);
          const uint32_t s_aux = AUX2 ? s_out + 16384 : s_staging + 16384;
          // the store that last read this tile must be done with it
          if constexpr (COMM != COMM_RS) {
            if (leader) {
              if (aux_staged && !AUX2) tma_store_wait_read_all();
              else asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            }
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int col0 = colq + h * 32;
            uint32_t r[32];
            tmem_ld_32x32b_x32(taddr + qs * 64 + h * 32, r);
            tmem_ld_wait();
            float v[32], u[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
            const int ncols = max(0, min(32, p.N - col0));
            epilogue_math(p, v, u, row, col0, ncols, row_ok);
            stage_row(s_out, r_in_tile, h, v);
            if (aux_staged) stage_row(s_aux, r_in_tile, h, u);
          }
          if constexpr (COMM == COMM_RS) {
            // push the [128 x 64] tile of partial sums into the owner's receive slot: eight
            // lanes write one 128-byte row segment, so every peer store is a full line
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const int owner = m_blk / p.tiles_per_shard;
            const int lrow0 = (m_blk % p.tiles_per_shard) * GEMM_BM;
            __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.rs_dst[owner]);
            const int t = threadIdx.x - 64;          // 0..127 over the epilogue warps
            const int chunk = t & 7;
            const int col = colq + chunk * 8;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rr = i * 16 + (t >> 3);
              uint4 val;
              const uint32_t addr = s_out + rr * 128 + ((static_cast<uint32_t>(chunk) ^ (rr & 7)) << 4);
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w) : "r"(addr));
              if (m0 + rr < p.M && col < p.N)
                *reinterpret_cast<uint4*>(dst + static_cast<size_t>(lrow0 + rr) * p.rs_ld + col) = val;
            }
          } else {
            fence_proxy_async_smem();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (leader && m0 < p.M) {     // a pair's second CTA may lie entirely below the matrix
              tma_store_2d(&tmD, s_out, colq, m0);
              if (aux_staged) tma_store_2d(&tmAux, s_aux, colq, m0);
              tma_store_commit();
            }
          }
          ++step;
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col0 = n0 + c * 32;
          if (col0 >= p.N) break;
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c * 32, r);
          tmem_ld_wait();
          if (!row_ok) continue;
          float v[32], u[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          const int ncols = min(32, p.N - col0);  // multiple of 8 (N % 8 == 0)
          epilogue_math(p, v, u, row, col0, ncols, true);
          if (p.epi == EPI_GELU && p.aux_out != nullptr) {
            __nv_bfloat16* ap = p.aux_out + static_cast<size_t>(row) * p.ldaux + col0;
#pragma unroll
            for (int g = 0; g < 4; ++g)
              if (g * 8 < ncols) *reinterpret_cast<uint4*>(ap + g * 8) = pack8(u + g * 8);
          }
          if (p.out_mode == OUT_BF16) {
            __nv_bfloat16* dp =
                reinterpret_cast<__nv_bfloat16*>(p.D) + static_cast<size_t>(row) * p.ldd + col0;
#pragma unroll
            for (int g = 0; g < 4; ++g)
              if (g * 8 < ncols) *reinterpret_cast<uint4*>(dp + g * 8) = pack8(v + g * 8);
          } else if (p.out_mode == OUT_F32) {
            float* dp = reinterpret_cast<float*>(p.D) + static_cast<size_t>(row) * p.ldd + col0;
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              if (g * 4 < ncols)
                *reinterpret_cast<float4*>(dp + g * 4) =
                    make_float4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
            }
          } else if (p.out_mode == OUT_F32_ATOMIC) {
            float* dp = reinterpret_cast<float*>(p.D) + static_cast<size_t>(row) * p.ldd + col0;
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              if (g * 4 < ncols) {
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                             ::"l"(dp + g * 4), "f"(v[g * 4]), "f"(v[g * 4 + 1]),
                               "f"(v[g * 4 + 2]), "f"(v[g * 4 + 3])
                             : "memory");
              }
            }
          }
        }
      }
      tc_fence_before();
      if constexpr (CTA2) mbar_arrive_cluster(mapa_shared(tempty_bar(acc), 0u));
      else mbar_arrive(tempty_bar(acc));
    }
    // every bulk store must have finished (reading shared memory and writing global memory)
    if (leader && p.tma_store) tma_store_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  if constexpr (CTA2) cluster_sync_all();   // nothing of the peer targets this CTA any more
  if (warp == 0) {
    tc_fence_after();
    if constexpr (CTA2) tmem_dealloc_cg2(tmem_base, Cfg::TMEM_COLS);
    else tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------- host side
static PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }
  return fn;
}

// 2-D bf16 tensor map: `inner` contiguous elements per row, `outer` rows, row pitch ld
// elements, 128-byte swizzle.  Returns 0 on success.
int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                      uint64_t ld, uint32_t box_inner, uint32_t box_outer) {
  auto fn = get_encode_fn();
  if (fn == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (ld * 2) % 16 != 0) return -2;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

// 3-D fp32 tensor map (inner `d0` contiguous floats, then `d1` rows of pitch ld1 floats, then `d2`
// slabs of pitch ld2 floats) with a box of 32 floats x box1 rows x 1 slab, 128-byte swizzle: the
// target of bulk reduce-add stores of an fp32 tile.
int make_tmap_f32_3d(CUtensorMap* out, void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                     uint64_t ld1, uint64_t ld2, uint32_t box1) {
  auto fn = get_encode_fn();
  if (fn == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (ld1 * 4) % 16 != 0 || (ld2 * 4) % 16 != 0)
    return -2;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {ld1 * 4, ld2 * 4};
  cuuint32_t box[3] = {32, box1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, base, dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

// 3-D bf16 tensor map (inner `d0` contiguous elements, then `d1` rows of pitch ld1 elements, then
// `d2` slabs of pitch ld2 elements) with a box of 64 x box1 x 1, 128-byte swizzle: tiles of one
// sequence that must not run into the next one.
int make_tmap_bf16_3d(CUtensorMap* out, void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                      uint64_t ld1, uint64_t ld2, uint32_t box1) {
  auto fn = get_encode_fn();
  if (fn == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (ld1 * 2) % 16 != 0 || (ld2 * 2) % 16 != 0)
    return -2;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {ld1 * 2, ld2 * 2};
  cuuint32_t box[3] = {64, box1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

template <int BN, bool A_MN, bool B_MN, int COMM = COMM_NONE>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td,
                       const CUtensorMap& taux, const GemmArgs& args, int max_ctas,
                       cudaStream_t stream) {
  using Cfg = GemmCfg<BN, COMM>;
  static bool configured = false;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, COMM>;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg::SMEM_BYTES) != cudaSuccess)
      return -10;
    configured = true;
  }
  const int tiles = ((args.M + GEMM_BM - 1) / GEMM_BM) * ((args.N + BN - 1) / BN) * args.ksplit;
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (tiles < grid) grid = tiles;
  kern<<<grid, COMM == COMM_AG ? GEMM_THREADS + 32 : GEMM_THREADS, Cfg::SMEM_BYTES, stream>>>(
      ta, tb, td, taux, args);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// CTA-pair variant: clusters of two CTAs, 256 x 256 tiles.
template <bool A_MN, bool B_MN, bool AUX2 = false>
static int launch_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td,
                            const CUtensorMap& taux, const GemmArgs& args, int max_ctas,
                            cudaStream_t stream) {
  using Cfg = GemmCfg<256, COMM_NONE, true, AUX2>;
  static bool configured = false;
  auto kern = gemm_bf16_kernel<256, A_MN, B_MN, COMM_NONE, true, AUX2>;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg::SMEM_BYTES) != cudaSuccess)
      return -10;
    configured = true;
  }
  const int tiles = ((args.M + 255) / 256) * ((args.N + 255) / 256) * args.ksplit;
  int pairs = sm_count() / 2;
  if (max_ctas > 0 && max_ctas / 2 < pairs) pairs = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
  if (tiles < pairs) pairs = tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, ta, tb, td, taux, args) == cudaSuccess ? 0 : -11;
}

static int g_use_pairs = 0;   // 1: plain 256-wide GEMMs run on CTA pairs

}  // namespace cb

extern "C" void cb_gemm_use_pairs(int on) { cb::g_use_pairs = on; }

// D[M,N] = epilogue(alpha * A . B^T)
//   A: logical [M,K]; a_mn == 0: memory [M,K] row-major (pitch lda); a_mn == 1: memory [K,M].
//   B: logical [N,K]; b_mn == 0: memory [N,K] row-major (pitch ldb); b_mn == 1: memory [K,N].
// Requirements: N a multiple of 8; K a multiple of 8 unless both operands are
// MN-major (there K is the outer, strided dimension of both tensor maps and any length works: the
// last k-block reads zero fill past the end); 16-byte aligned pointers and pitches.
//
// groups > 1 (grouped GEMM, e.g. the experts of a mixture-of-experts layer): M, N and K are the
// sizes of ONE group and every operand holds the groups stacked along the row dimension of its
// memory: A is [groups*M, K] (a_mn == 0) or [groups*K, M] (a_mn == 1); B is [groups*N, K]
// (b_mn == 0) or [groups*K, N] (b_mn == 1); D, resid and aux are [groups*M, N].  Group g's output
// rows are produced from group g's slices.  Needs M a multiple of the tile height (128; CTA pairs
// are used when it is a multiple of 256) and K a multiple of 64, so that no tile or k-block
// straddles two groups.
static int gemm_bf16_impl(const void* A, const void* B, void* D, int M, int N, int K, int lda,
                          int ldb, int ldd, int a_mn, int b_mn, const void* bias,
                          const void* resid, int ldr, const void* aux_in, void* aux_out,
                          int ldaux, int epi, int out_mode, float alpha, int ksplit, int bn,
                          int* status, int max_ctas, void* stream, int groups, int drop_thr = 0,
                          unsigned int drop_key = 0) {
  using namespace cb;
  if (drop_thr < 0 || drop_thr > 255 || (drop_thr > 0 && (N % 32) != 0)) return -25;
  if (M <= 0 || N <= 0 || K <= 0 || groups < 1) return -20;
  if ((N % 8) != 0 || (ldd % 4) != 0) return -21;
  if ((K % 8) != 0 && !(a_mn && b_mn)) return -21;
  if (out_mode == OUT_BF16 && (ldd % 8) != 0) return -21;
  // bn = 512 selects the 256-wide tile on CTA pairs
  bool pairs = bn == 512 || (bn == 256 && cb::g_use_pairs);
  if (bn == 512) bn = 256;
  if (bn != 128 && bn != 256) return -22;
  const int Mg = M, Kg = K;       // per-group sizes; M becomes the stacked row count below
  if (groups > 1) {
    if ((Mg % GEMM_BM) != 0 || (Kg % GEMM_BK) != 0) return -24;
    if ((Mg % (2 * GEMM_BM)) != 0) pairs = false;
    if (static_cast<long long>(Mg) * groups > 0x7fffffffLL) return -24;
    M = Mg * groups;
  }
  const int kblocks = (K + GEMM_BK - 1) / GEMM_BK;
  if (ksplit < 1) ksplit = 1;
  if (ksplit > kblocks) ksplit = kblocks;
  // every split must own at least one k-block
  {
    const int per = (kblocks + ksplit - 1) / ksplit;
    ksplit = (kblocks + per - 1) / per;
  }
  if (ksplit > 1 && out_mode != OUT_F32_ATOMIC) return -23;
  CUtensorMap ta, tb;
  int rc;
  const uint64_t G64 = static_cast<uint64_t>(groups);
  if (a_mn == 0)
    rc = make_tmap_bf16_2d(&ta, A, K, M, lda, 64, GEMM_BM);
  else
    rc = make_tmap_bf16_2d(&ta, A, Mg, G64 * Kg, lda, 64, 64);
  if (rc != 0) return rc - 30;
  if (b_mn == 0)
    rc = make_tmap_bf16_2d(&tb, B, K, G64 * N, ldb, 64, (bn == 256 && pairs) ? 128 : bn);
  else
    rc = make_tmap_bf16_2d(&tb, B, N, G64 * Kg, ldb, 64, 64);
  if (rc != 0) return rc - 40;
  // bf16 results (and the kept pre-activation) go out through swizzled shared memory and TMA
  // stores whenever the output rows are 16-byte aligned; fp32 / atomic outputs are stored directly
  CUtensorMap td = ta, taux = ta;
  int tma_store = 0;
  if (out_mode == OUT_BF16 && (reinterpret_cast<uintptr_t>(D) & 15u) == 0 && (ldd % 8) == 0) {
    tma_store = make_tmap_bf16_2d(&td, D, N, M, ldd, 64, GEMM_BM) == 0 ? 1 : 0;
    if (tma_store && epi == EPI_GELU && aux_out != nullptr) {
      if ((reinterpret_cast<uintptr_t>(aux_out) & 15u) != 0 || (ldaux % 8) != 0 ||
          make_tmap_bf16_2d(&taux, aux_out, N, M, ldaux, 64, GEMM_BM) != 0)
        tma_store = 0;
    }
  }
  GemmArgs g;
  std::memset(&g, 0, sizeof(g));
  g.tma_store = tma_store;
  g.tp = 1;
  g.tiles_per_shard = 1;
  g.M = M; g.N = N; g.K = K;
  g.D = D; g.ldd = ldd;
  g.bias = static_cast<const __nv_bfloat16*>(bias);
  g.resid = static_cast<const __nv_bfloat16*>(resid);
  g.ldr = ldr;
  g.aux_in = static_cast<const __nv_bfloat16*>(aux_in);
  g.aux_out = static_cast<__nv_bfloat16*>(aux_out);
  g.ldaux = ldaux;
  g.epi = epi; g.out_mode = out_mode; g.alpha = alpha; g.ksplit = ksplit; g.status = status;
  g.drop_thr = drop_thr;
  g.drop_key = drop_key;
  g.drop_scale = 256.0f / static_cast<float>(256 - drop_thr);
  if (groups > 1) {
    g.group_m = Mg;
    g.g_am = a_mn ? -Mg : 0;
    g.g_ak = a_mn ? Kg : 0;
    g.g_bn = b_mn ? 0 : N;
    g.g_bk = b_mn ? Kg : 0;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define CB_DISPATCH(BN_)                                                            \
  do {                                                                              \
    if (!a_mn && !b_mn) return launch_gemm<BN_, false, false>(ta, tb, td, taux, g, max_ctas, st); \
    if (!a_mn && b_mn) return launch_gemm<BN_, false, true>(ta, tb, td, taux, g, max_ctas, st);   \
    if (a_mn && !b_mn) return launch_gemm<BN_, true, false>(ta, tb, td, taux, g, max_ctas, st);   \
    return launch_gemm<BN_, true, true>(ta, tb, td, taux, g, max_ctas, st);                       \
  } while (0)
  if (bn == 256 && pairs) {
    if (!a_mn && b_mn && tma_store && epi == EPI_GELU && aux_out != nullptr)
      return launch_gemm_pair<false, true, true>(ta, tb, td, taux, g, max_ctas, st);
    if (!a_mn && !b_mn) return launch_gemm_pair<false, false>(ta, tb, td, taux, g, max_ctas, st);
    if (!a_mn && b_mn) return launch_gemm_pair<false, true>(ta, tb, td, taux, g, max_ctas, st);
    if (a_mn && !b_mn) return launch_gemm_pair<true, false>(ta, tb, td, taux, g, max_ctas, st);
    return launch_gemm_pair<true, true>(ta, tb, td, taux, g, max_ctas, st);
  }
  if (bn == 256) CB_DISPATCH(256);
  CB_DISPATCH(128);
#undef CB_DISPATCH
}

extern "C" int cb_gemm_bf16(const void* A, const void* B, void* D, int M, int N, int K, int lda,
                            int ldb, int ldd, int a_mn, int b_mn, const void* bias,
                            const void* resid, int ldr, const void* aux_in, void* aux_out,
                            int ldaux, int epi, int out_mode, float alpha, int ksplit, int bn,
                            int* status, int max_ctas, void* stream) {
  return gemm_bf16_impl(A, B, D, M, N, K, lda, ldb, ldd, a_mn, b_mn, bias, resid, ldr, aux_in,
                        aux_out, ldaux, epi, out_mode, alpha, ksplit, bn, status, max_ctas, stream,
                        1);
}

// cb_gemm_bf16 with dropout on the epilogue value (after bias / activation, before the residual):
// drop_thr = round(p * 256) in 1..255, drop_key selects the mask (see dropout_bits); N % 32 == 0.
extern "C" int cb_gemm_bf16_dropout(const void* A, const void* B, void* D, int M, int N, int K,
                                    int lda, int ldb, int ldd, int a_mn, int b_mn,
                                    const void* bias, const void* resid, int ldr, int epi,
                                    float alpha, int bn, int drop_thr, unsigned int drop_key,
                                    int* status, int max_ctas, void* stream) {
  return gemm_bf16_impl(A, B, D, M, N, K, lda, ldb, ldd, a_mn, b_mn, bias, resid, ldr, nullptr,
                        nullptr, 0, epi, cb::OUT_BF16, alpha, 1, bn, status, max_ctas, stream, 1,
                        drop_thr, drop_key);
}

extern "C" int cb_gemm_bf16_grouped(const void* A, const void* B, void* D, int groups, int M, int N,
                                    int K, int lda, int ldb, int ldd, int a_mn, int b_mn,
                                    int out_mode, float alpha, int ksplit, int bn, int* status,
                                    int max_ctas, void* stream) {
  return gemm_bf16_impl(A, B, D, M, N, K, lda, ldb, ldd, a_mn, b_mn, nullptr, nullptr, 0, nullptr,
                        nullptr, 0, cb::EPI_NONE, out_mode, alpha, ksplit, bn, status, max_ctas,
                        stream, groups);
}

// ------------------------------------------------------------------------------------------
// Fused tensor-parallel GEMMs.  `comm` selects:
//   1 (all-gather -> GEMM): A is this rank's [tp * rows_per_shard, K] gathered operand, of which
//     only rows [rank * rows_per_shard, ...) are valid on entry; ag_src[s] is rank s's copy of the
//     same buffer (peer mapped).  Weights: B as in cb_gemm_bf16.  Output: plain D[M, N].
//   2 (GEMM -> reduce-scatter): D is not written locally; rs_dst[s] is the receive slot on rank
//     s (already offset to this rank's slot), [rows_per_shard, N] with pitch rs_ld.
struct CbCommArgs {
  int comm, tp, rank, rows_per_shard;
  const void* ag_src[8];
  void* ag_flags;
  unsigned int ag_epoch;
  const void* peer_flags;
  unsigned long long peer_expect;
  unsigned long long wait_limit_ns;
  void* rs_dst[8];
  int rs_ld;
};

extern "C" int cb_gemm_bf16_fused(const void* A, const void* B, void* D, int M, int N, int K,
                                  int lda, int ldb, int ldd, int b_mn, const void* bias, int bn,
                                  const CbCommArgs* c, int* status, int max_ctas, void* stream) {
  using namespace cb;
  if (c == nullptr || (c->comm != COMM_AG && c->comm != COMM_RS)) return -50;
  if (c->tp < 1 || c->tp > MAX_TP || c->rows_per_shard % GEMM_BM != 0) return -51;
  if (M != c->tp * c->rows_per_shard) return -52;
  if ((N % 8) != 0 || (K % 8) != 0) return -21;
  if (bn != 128 && bn != 256) return -22;
  CUtensorMap ta, tb, td;
  if (make_tmap_bf16_2d(&ta, A, K, M, lda, 64, GEMM_BM) != 0) return -31;
  int rc = b_mn == 0 ? make_tmap_bf16_2d(&tb, B, K, N, ldb, 64, bn)
                     : make_tmap_bf16_2d(&tb, B, N, K, ldb, 64, 64);
  if (rc != 0) return rc - 40;
  td = ta;
  GemmArgs g;
  std::memset(&g, 0, sizeof(g));
  g.M = M; g.N = N; g.K = K;
  g.D = D; g.ldd = ldd;
  g.bias = static_cast<const __nv_bfloat16*>(bias);
  g.epi = EPI_NONE; g.out_mode = OUT_BF16; g.alpha = 1.0f; g.ksplit = 1; g.status = status;
  g.tp = c->tp; g.rank = c->rank; g.tiles_per_shard = c->rows_per_shard / GEMM_BM;
  g.wait_limit_ns = c->wait_limit_ns;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (c->comm == COMM_AG) {
    if (make_tmap_bf16_2d(&td, D, N, M, ldd, 64, GEMM_BM) != 0) return -32;
    g.tma_store = 1;
    for (int i = 0; i < c->tp; ++i) g.ag_src[i] = c->ag_src[i];
    g.ag_dst = static_cast<__nv_bfloat16*>(const_cast<void*>(A));
    g.ag_ld = lda;
    g.ag_flags = static_cast<uint32_t*>(c->ag_flags);
    g.ag_epoch = c->ag_epoch;
    g.peer_flags = static_cast<const uint64_t*>(c->peer_flags);
    g.peer_expect = c->peer_expect;
    if (bn == 256)
      return b_mn ? launch_gemm<256, false, true, COMM_AG>(ta, tb, td, td, g, max_ctas, st)
                  : launch_gemm<256, false, false, COMM_AG>(ta, tb, td, td, g, max_ctas, st);
    return b_mn ? launch_gemm<128, false, true, COMM_AG>(ta, tb, td, td, g, max_ctas, st)
                : launch_gemm<128, false, false, COMM_AG>(ta, tb, td, td, g, max_ctas, st);
  }
  g.tma_store = 1;   // staged epilogue; the tile leaves through peer stores instead of TMA
  for (int i = 0; i < c->tp; ++i) g.rs_dst[i] = c->rs_dst[i];
  g.rs_ld = c->rs_ld;
  if (bn == 256)
    return b_mn ? launch_gemm<256, false, true, COMM_RS>(ta, tb, td, td, g, max_ctas, st)
                : launch_gemm<256, false, false, COMM_RS>(ta, tb, td, td, g, max_ctas, st);
  return b_mn ? launch_gemm<128, false, true, COMM_RS>(ta, tb, td, td, g, max_ctas, st)
              : launch_gemm<128, false, false, COMM_RS>(ta, tb, td, td, g, max_ctas, st);
}
