// One-shot all-reduce over NVLink peer memory fused with the residual add and the following
// normalisation -- the collective of tensor-parallel decoding, where the message is a few
// hundred KB and latency is everything.
//
// Every rank has written its partial result [rows, H] (bf16) into a buffer that all peers have
// mapped.  One kernel per rank then
//   1. tells every peer "my partial of call e is ready" (st.release.sys into the peer's flags),
//   2. waits (bounded) until all peers have said the same,
//   3. loads the row from every rank's buffer, sums in rank order in fp32 (so all ranks get the
//      same bits), adds the residual, stores x_out, and
//   4. optionally normalises the row (RMSNorm or LayerNorm) into n_out.
// The call counter e lives in device memory and is advanced by the last block, so the launch
// parameters never change and the kernel can sit in a CUDA graph.  Callers alternate between two
// partial buffers: a rank can only be one call ahead of a peer (step 2), so the buffer of call e
// is not rewritten before every peer has finished reading it.
#include "common.cuh"
#include "ptx.cuh"

namespace cb {
int sm_count();

constexpr int AR_MAX_RANKS = 8;
constexpr int AR_THREADS = 256;
constexpr int AR_MAX_VEC = 4;   // 8-element vectors per thread: H <= 256 * 4 * 8 = 8192

struct ArArgs {
  const __nv_bfloat16* parts[AR_MAX_RANKS];
  unsigned long long* peer_flags[AR_MAX_RANKS];   // rank s's flag array (this rank writes [rank])
  const unsigned long long* my_flags;
  unsigned long long* epoch;                      // completed calls on this flag array
  unsigned int* done;                             // blocks that have finished this call
  const __nv_bfloat16* resid;
  __nv_bfloat16* x_out;
  const __nv_bfloat16* scale;
  const __nv_bfloat16* bias;
  __nv_bfloat16* n_out;
  int tp, rank, rows, H, rms;
  float eps;
  unsigned long long limit_ns;
  int* status;
};

__global__ void __launch_bounds__(AR_THREADS) ar_resid_norm_kernel(ArArgs a) {
  __shared__ float red[32];
  __shared__ int s_ok;
  const unsigned long long e = *reinterpret_cast<volatile unsigned long long*>(a.epoch) + 1ull;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x < a.tp) {
    __threadfence_system();
    asm volatile("st.release.sys.global.u64 [%0], %1;"
                 :: "l"(a.peer_flags[threadIdx.x] + a.rank), "l"(e) : "memory");
  }
  if (threadIdx.x < a.tp) {
    const unsigned long long* f = a.my_flags + threadIdx.x;
    const uint64_t t0 = globaltimer_ns();
    uint32_t it = 0;
    unsigned long long v;
    while (true) {
      asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(f) : "memory");
      if (v >= e) break;
      if ((++it & 63u) == 0u && globaltimer_ns() - t0 > a.limit_ns) {
        record_status(a.status, ST_COMM_TIMEOUT, threadIdx.x);
        s_ok = 0;
        break;
      }
    }
  }
  __syncthreads();
  if (s_ok != 0) {
    const int nv = a.H >> 3;
    for (int row = blockIdx.x; row < a.rows; row += gridDim.x) {
      float x[AR_MAX_VEC][8];
      float sum = 0.f, sq = 0.f;
#pragma unroll
      for (int j = 0; j < AR_MAX_VEC; ++j) {
        const int v = threadIdx.x + j * AR_THREADS;
        if (v < nv) {
          const size_t off = static_cast<size_t>(row) * a.H + v * 8;
          float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          for (int s = 0; s < a.tp; ++s) {
            uint4 raw;
            asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w)
                         : "l"(a.parts[s] + off) : "memory");
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float2 f = __bfloat1622float2(h[q]);
              acc[2 * q] += f.x;
              acc[2 * q + 1] += f.y;
            }
          }
          if (a.resid != nullptr) {
            float r[8];
            load8(a.resid + off, r);
#pragma unroll
            for (int q = 0; q < 8; ++q) acc[q] += r[q];
          }
          store8(a.x_out + off, acc);
#pragma unroll
          for (int q = 0; q < 8; ++q) {   // normalise what was stored (bf16-rounded values)
            x[j][q] = __bfloat162float(__float2bfloat16(acc[q]));
            sum += x[j][q];
            sq += x[j][q] * x[j][q];
          }
        }
      }
      if (a.n_out != nullptr) {
        float mean = 0.f, rstd;
        if (a.rms) {
          sq = block_sum(sq, red);
          rstd = rsqrtf(sq / a.H + a.eps);
        } else {
          sum = block_sum(sum, red);
          mean = sum / a.H;
          float var = 0.f;
#pragma unroll
          for (int j = 0; j < AR_MAX_VEC; ++j)
            if (threadIdx.x + j * AR_THREADS < nv)
#pragma unroll
              for (int q = 0; q < 8; ++q) var += (x[j][q] - mean) * (x[j][q] - mean);
          var = block_sum(var, red);
          rstd = rsqrtf(var / a.H + a.eps);
        }
#pragma unroll
        for (int j = 0; j < AR_MAX_VEC; ++j) {
          const int v = threadIdx.x + j * AR_THREADS;
          if (v < nv) {
            float g[8], b[8], y[8];
            load8(a.scale + v * 8, g);
            if (a.bias != nullptr) load8(a.bias + v * 8, b);
#pragma unroll
            for (int q = 0; q < 8; ++q)
              y[q] = (x[j][q] - mean) * rstd * g[q] + (a.bias != nullptr ? b[q] : 0.f);
            store8(a.n_out + static_cast<size_t>(row) * a.H + v * 8, y);
          }
        }
      }
    }
  }
  // the last block to finish closes the call
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int prev = atomicAdd(a.done, 1u);
    if (prev == gridDim.x - 1) {
      *a.done = 0u;
      *reinterpret_cast<volatile unsigned long long*>(a.epoch) = e;
      __threadfence();
    }
  }
}
}  // namespace cb

// state: [0] = epoch (u64), [1] = done counter (u32 in the low half); zero before the first call
extern "C" int cb_ar_resid_norm(void* const* parts, void* const* peer_flags, const void* my_flags,
                                void* state, const void* resid, void* x_out, const void* scale,
                                const void* bias, void* n_out, int tp, int rank, int rows, int H,
                                int rms, float eps, unsigned long long limit_ns, int* status,
                                void* stream) {
  using namespace cb;
  if (tp < 1 || tp > AR_MAX_RANKS || H % 8 != 0 || H > AR_THREADS * AR_MAX_VEC * 8) return -1;
  if (rows <= 0) return 0;
  ArArgs a;
  for (int i = 0; i < tp; ++i) {
    a.parts[i] = static_cast<const __nv_bfloat16*>(parts[i]);
    a.peer_flags[i] = static_cast<unsigned long long*>(peer_flags[i]);
  }
  a.my_flags = static_cast<const unsigned long long*>(my_flags);
  a.epoch = static_cast<unsigned long long*>(state);
  a.done = reinterpret_cast<unsigned int*>(static_cast<unsigned long long*>(state) + 1);
  a.resid = static_cast<const __nv_bfloat16*>(resid);
  a.x_out = static_cast<__nv_bfloat16*>(x_out);
  a.scale = static_cast<const __nv_bfloat16*>(scale);
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.n_out = static_cast<__nv_bfloat16*>(n_out);
  a.tp = tp; a.rank = rank; a.rows = rows; a.H = H; a.rms = rms; a.eps = eps;
  a.limit_ns = limit_ns; a.status = status;
  const int grid = rows < sm_count() * 2 ? rows : sm_count() * 2;
  ar_resid_norm_kernel<<<grid, AR_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// ------------------------------------------------------------------------------------------
// The same collective through NVLink multicast (NVLS): every buffer below is symmetric memory
// bound to one multicast object, so `mc + offset` names that offset on ALL ranks at once.
//   1. arrive: one multimem.red adds 1 to the arrival counter on every rank; wait (bounded) until
//      the local counter shows all ranks of this call,
//   2. each rank takes the rows r with r % tp == rank: multimem.ld_reduce returns the sum of the
//      row over all ranks' partial buffers (reduced in the switch, fp32 accumulation), the
//      residual is added, the row is normalised, and x / n are written to EVERY rank's output
//      buffers with multimem.st -- so all ranks hold bit-identical results,
//   3. leave: a second counter (multimem.red by the last block of every rank) tells each rank
//      that all rows have arrived before its kernel completes.
// A rank moves 1/tp of the rows in and out instead of reading every rank's copy of all of them.
// Outputs and partials alternate between two buffers (a rank can be at most one call ahead of a
// peer), the call counter lives on the device, launch parameters never change (graph replay).
namespace cb {

struct ArMmArgs {
  const __nv_bfloat16* part_mc;     // multicast address of the partial buffer of this call
  __nv_bfloat16* x_mc;              // multicast addresses of the outputs of this call
  __nv_bfloat16* n_mc;
  const __nv_bfloat16* resid;       // local [rows, H] or null
  unsigned int* flags_mc;           // multicast address of {arrive, leave} counters
  const unsigned int* flags_local;  // the same counters through this rank's own mapping
  unsigned long long* epoch;
  unsigned int* done;
  const __nv_bfloat16* scale;
  const __nv_bfloat16* bias;
  int tp, rank, rows, H, rms;
  int one_shot;                     // 1: every rank reduces all rows for itself (x / n are local
                                    // addresses, plain stores, no second counter)
  float eps;
  unsigned long long limit_ns;
  int* status;
};

__device__ __forceinline__ void st_out(__nv_bfloat16* dst, const uint4& v, bool multicast) {
  if (multicast) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 :: "l"(dst), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)),
                    "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w)) : "memory");
  } else {
    *reinterpret_cast<uint4*>(dst) = v;
  }
}

__device__ __forceinline__ bool wait_counter(const unsigned int* p, unsigned int target,
                                             unsigned long long limit_ns, int* status, int where) {
  const uint64_t t0 = globaltimer_ns();
  uint32_t it = 0;
  while (true) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    // counters only grow; the comparison survives wrap-around of the 32-bit value
    if (static_cast<int>(v - target) >= 0) return true;
    if ((++it & 63u) == 0u && globaltimer_ns() - t0 > limit_ns) {
      record_status(status, ST_COMM_TIMEOUT, where);
      return false;
    }
  }
}

__global__ void __launch_bounds__(AR_THREADS) ar_multimem_kernel(ArMmArgs a) {
  __shared__ float red[32];
  __shared__ int s_ok;
  const unsigned long long e = *reinterpret_cast<volatile unsigned long long*>(a.epoch) + 1ull;
  const unsigned int target = static_cast<unsigned int>(e) * static_cast<unsigned int>(a.tp);
  if (threadIdx.x == 0) {
    s_ok = 1;
    if (blockIdx.x == 0) {
      __threadfence_system();      // this rank's partial (written by the kernel before) is visible
      asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;"
                   :: "l"(a.flags_mc), "r"(1u) : "memory");
    }
    if (!wait_counter(a.flags_local, target, a.limit_ns, a.status, 0)) s_ok = 0;
  }
  __syncthreads();
  const int row = a.one_shot ? static_cast<int>(blockIdx.x)
                             : a.rank + static_cast<int>(blockIdx.x) * a.tp;
  const bool mcast = a.one_shot == 0;
  if (s_ok != 0 && row < a.rows) {
    const int nv = a.H >> 3;
    float x[AR_MAX_VEC][8];
    float sum = 0.f, sq = 0.f;
#pragma unroll
    for (int j = 0; j < AR_MAX_VEC; ++j) {
      const int v = threadIdx.x + j * AR_THREADS;
      if (v < nv) {
        const size_t off = static_cast<size_t>(row) * a.H + v * 8;
        uint4 raw;
        asm volatile(
            "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
            : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w)
            : "l"(a.part_mc + off) : "memory");
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
        float acc[8];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = __bfloat1622float2(h[q]);
          acc[2 * q] = f.x;
          acc[2 * q + 1] = f.y;
        }
        if (a.resid != nullptr) {
          float r[8];
          load8(a.resid + off, r);
#pragma unroll
          for (int q = 0; q < 8; ++q) acc[q] += r[q];
        }
        uint4 out;
        out.x = pack_bf16x2(acc[0], acc[1]);
        out.y = pack_bf16x2(acc[2], acc[3]);
        out.z = pack_bf16x2(acc[4], acc[5]);
        out.w = pack_bf16x2(acc[6], acc[7]);
        st_out(a.x_mc + off, out, mcast);
#pragma unroll
        for (int q = 0; q < 8; ++q) {   // normalise what was stored (bf16-rounded values)
          x[j][q] = __bfloat162float(__float2bfloat16(acc[q]));
          sum += x[j][q];
          sq += x[j][q] * x[j][q];
        }
      }
    }
    if (a.n_mc != nullptr) {
      float mean = 0.f, rstd;
      if (a.rms) {
        sq = block_sum(sq, red);
        rstd = rsqrtf(sq / a.H + a.eps);
      } else {
        sum = block_sum(sum, red);
        mean = sum / a.H;
        float var = 0.f;
#pragma unroll
        for (int j = 0; j < AR_MAX_VEC; ++j)
          if (threadIdx.x + j * AR_THREADS < nv)
#pragma unroll
            for (int q = 0; q < 8; ++q) var += (x[j][q] - mean) * (x[j][q] - mean);
        var = block_sum(var, red);
        rstd = rsqrtf(var / a.H + a.eps);
      }
#pragma unroll
      for (int j = 0; j < AR_MAX_VEC; ++j) {
        const int v = threadIdx.x + j * AR_THREADS;
        if (v < nv) {
          float g[8], b[8], y[8];
          load8(a.scale + v * 8, g);
          if (a.bias != nullptr) load8(a.bias + v * 8, b);
#pragma unroll
          for (int q = 0; q < 8; ++q)
            y[q] = (x[j][q] - mean) * rstd * g[q] + (a.bias != nullptr ? b[q] : 0.f);
          uint4 yo;
          yo.x = pack_bf16x2(y[0], y[1]);
          yo.y = pack_bf16x2(y[2], y[3]);
          yo.z = pack_bf16x2(y[4], y[5]);
          yo.w = pack_bf16x2(y[6], y[7]);
          st_out(a.n_mc + static_cast<size_t>(row) * a.H + v * 8, yo, mcast);
        }
      }
    }
  }
  // the last block of this rank announces its rows everywhere and waits for everybody's
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int prev = atomicAdd(a.done, 1u);
    if (prev == gridDim.x - 1) {
      if (mcast) {
        asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;"
                     :: "l"(a.flags_mc + 1), "r"(1u) : "memory");
        if (s_ok != 0) wait_counter(a.flags_local + 1, target, a.limit_ns, a.status, 1);
      }
      *a.done = 0u;
      *reinterpret_cast<volatile unsigned long long*>(a.epoch) = e;
      __threadfence();
    }
  }
}
}  // namespace cb

// part_mc: multicast address of the [rows, H] bf16 partial buffer; x_mc / n_mc: multicast
// addresses of the outputs (n_mc may be null) -- or, with one_shot != 0, local addresses: every
// rank then reduces all rows for itself and nothing is broadcast;
// flags_mc / flags_local: two 32-bit counters (arrive, leave), zero before the first call;
// state as in cb_ar_resid_norm.
extern "C" int cb_ar_multimem(const void* part_mc, void* x_mc, void* n_mc, const void* resid,
                              void* flags_mc, const void* flags_local, void* state,
                              const void* scale, const void* bias, int tp, int rank, int rows,
                              int H, int rms, float eps, unsigned long long limit_ns, int* status,
                              int one_shot, void* stream) {
  using namespace cb;
  if (tp < 1 || tp > AR_MAX_RANKS || H % 8 != 0 || H > AR_THREADS * AR_MAX_VEC * 8) return -1;
  if (rows <= 0) return 0;
  ArMmArgs a;
  a.part_mc = static_cast<const __nv_bfloat16*>(part_mc);
  a.x_mc = static_cast<__nv_bfloat16*>(x_mc);
  a.n_mc = static_cast<__nv_bfloat16*>(n_mc);
  a.resid = static_cast<const __nv_bfloat16*>(resid);
  a.flags_mc = static_cast<unsigned int*>(flags_mc);
  a.flags_local = static_cast<const unsigned int*>(flags_local);
  a.epoch = static_cast<unsigned long long*>(state);
  a.done = reinterpret_cast<unsigned int*>(static_cast<unsigned long long*>(state) + 1);
  a.scale = static_cast<const __nv_bfloat16*>(scale);
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.tp = tp; a.rank = rank; a.rows = rows; a.H = H; a.rms = rms; a.eps = eps;
  a.one_shot = one_shot;
  a.limit_ns = limit_ns; a.status = status;
  const int grid = one_shot ? rows : (rows + tp - 1) / tp;   // the same on every rank
  ar_multimem_kernel<<<grid, AR_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// ------------------------------------------------------------------------------------------
// Greedy token selection over a vocabulary that is split across ranks, without a library
// collective: block b finds the arg-max of row b of this rank's logits slice, stores the pair
// (value, global index) into slot [rank][b] of EVERY rank's pair table, raises the slot's flag,
// waits (bounded) for the slots of all ranks and keeps the best pair (lowest rank wins ties,
// which is the first index, as one arg-max over the whole row would give).  Same call counter
// scheme as the all-reduce above.
namespace cb {

struct GreedyArgs {
  const __nv_bfloat16* logits;   // [B, ld]
  int ld, valid, col0;           // columns that compete; global index of column 0
  unsigned long long* pairs[AR_MAX_RANKS];   // rank s's table: [tp][B] packed (value bits << 32 | index)
  unsigned long long* flags[AR_MAX_RANKS];   // rank s's flags: [tp][B] call numbers
  unsigned long long* epoch;
  unsigned int* done;
  long long* out;                // [B] chosen token ids
  int tp, rank, B;
  unsigned long long limit_ns;
  int* status;
};

__global__ void __launch_bounds__(AR_THREADS) greedy_select_kernel(GreedyArgs a) {
  __shared__ float s_val[AR_THREADS / 32];
  __shared__ int s_idx[AR_THREADS / 32];
  __shared__ unsigned long long s_pair[AR_MAX_RANKS];
  __shared__ int s_ok;
  const unsigned long long e = *reinterpret_cast<volatile unsigned long long*>(a.epoch) + 1ull;
  const int b = blockIdx.x;
  if (threadIdx.x == 0) s_ok = 1;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  const __nv_bfloat16* row = a.logits + static_cast<size_t>(b) * a.ld;
  for (int c = threadIdx.x; c < a.valid; c += AR_THREADS) {
    const float v = __bfloat162float(row[c]);
    if (v > best || (v == best && c < bi)) { best = v; bi = c; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { s_val[threadIdx.x >> 5] = best; s_idx[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < AR_THREADS / 32; ++w)
      if (s_val[w] > best || (s_val[w] == best && s_idx[w] < bi)) { best = s_val[w]; bi = s_idx[w]; }
    const unsigned long long packed =
        (static_cast<unsigned long long>(__float_as_uint(best)) << 32) |
        static_cast<unsigned int>(a.valid > 0 ? bi + a.col0 : 0x7fffffff);
    s_pair[0] = packed;
  }
  __syncthreads();
  if (threadIdx.x < a.tp) {      // one thread per destination rank
    const size_t slot = static_cast<size_t>(a.rank) * a.B + b;
    unsigned long long* dp = a.pairs[threadIdx.x] + slot;
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" :: "l"(dp), "l"(s_pair[0]) : "memory");
    asm volatile("st.release.sys.global.u64 [%0], %1;"
                 :: "l"(a.flags[threadIdx.x] + slot), "l"(e) : "memory");
  }
  __syncthreads();
  if (threadIdx.x < a.tp) {      // one thread per source rank
    const size_t slot = static_cast<size_t>(threadIdx.x) * a.B + b;
    const unsigned long long* f = a.flags[a.rank] + slot;
    const uint64_t t0 = globaltimer_ns();
    uint32_t it = 0;
    unsigned long long v;
    bool ok = true;
    while (true) {
      asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(f) : "memory");
      if (v >= e) break;
      if ((++it & 63u) == 0u && globaltimer_ns() - t0 > a.limit_ns) {
        record_status(a.status, ST_COMM_TIMEOUT, threadIdx.x);
        s_ok = 0;
        ok = false;
        break;
      }
    }
    unsigned long long p = 0;
    if (ok) asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(p) : "l"(a.pairs[a.rank] + slot) : "memory");
    s_pair[threadIdx.x] = p;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (s_ok != 0) {
      float bv = -INFINITY;
      long long bidx = 0;
      for (int s = 0; s < a.tp; ++s) {
        const float v = __uint_as_float(static_cast<unsigned int>(s_pair[s] >> 32));
        const unsigned int idx = static_cast<unsigned int>(s_pair[s] & 0xffffffffull);
        if (idx != 0x7fffffffu && (s == 0 || v > bv)) { bv = v; bidx = idx; }
      }
      a.out[b] = bidx;
    }
    __threadfence();
    const unsigned int prev = atomicAdd(a.done, 1u);
    if (prev == gridDim.x - 1) {
      *a.done = 0u;
      *reinterpret_cast<volatile unsigned long long*>(a.epoch) = e;
      __threadfence();
    }
  }
}
}  // namespace cb

extern "C" int cb_greedy_select(const void* logits, int ld, int valid, int col0,
                                void* const* pairs, void* const* flags, void* state, void* out,
                                int tp, int rank, int B, unsigned long long limit_ns, int* status,
                                void* stream) {
  using namespace cb;
  if (tp < 1 || tp > AR_MAX_RANKS || B <= 0) return -1;
  GreedyArgs a;
  a.logits = static_cast<const __nv_bfloat16*>(logits);
  a.ld = ld; a.valid = valid; a.col0 = col0;
  for (int i = 0; i < tp; ++i) {
    a.pairs[i] = static_cast<unsigned long long*>(pairs[i]);
    a.flags[i] = static_cast<unsigned long long*>(flags[i]);
  }
  a.epoch = static_cast<unsigned long long*>(state);
  a.done = reinterpret_cast<unsigned int*>(static_cast<unsigned long long*>(state) + 1);
  a.out = static_cast<long long*>(out);
  a.tp = tp; a.rank = rank; a.B = B; a.limit_ns = limit_ns; a.status = status;
  greedy_select_kernel<<<B, AR_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
