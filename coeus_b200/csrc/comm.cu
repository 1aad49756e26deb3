// Communication substrate over NVLink peer memory and the fused data-parallel kernel.
//
//  * symmetric buffers: cudaMalloc'ed by each rank, exported with CUDA IPC and mapped by every
//    peer, so a kernel on one GPU can load from / store to the same offset on any other GPU;
//  * signal flags: 64-bit epochs in a symmetric buffer, written with st.release.sys by the
//    producer and polled with ld.acquire.sys by the consumer -- every poll loop is bounded by a
//    time limit after which the kernel records ST_COMM_TIMEOUT and returns;
//  * rs_adamw_ag_kernel: the data-parallel step in ONE kernel.  The owner of a shard loads that
//    shard of the fp32 gradients from every rank over NVLink (reduce-scatter, summed in rank
//    order so all ranks agree bit for bit), scales, applies AdamW to its fp32 master shard and
//    moments, and stores the updated bf16 weights into every rank's working copy (all-gather).
//
// Nothing here uses TMA multicast or any other cluster-multicast load.
#include "common.cuh"
#include "ptx.cuh"

namespace cb {
int sm_count();

constexpr int MAX_RANKS = 16;

__device__ __forceinline__ uint64_t ld_acquire_sys_u64(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys_u64(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ float4 ld_relaxed_sys_f4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_relaxed_sys_u4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

struct PeerPtrs {
  void* p[MAX_RANKS];
};

// Every rank runs this with one thread per peer: flags_of_peer[p][slot * n + my_rank] = value.
__global__ void signal_peers_kernel(PeerPtrs flags, int slot, int n, int my_rank, uint64_t value) {
  __threadfence_system();  // order all earlier writes of this GPU before the signal
  const int p = threadIdx.x;
  if (p < n) st_release_sys_u64(static_cast<uint64_t*>(flags.p[p]) + slot * n + my_rank, value);
}

// Wait until local flags[slot * n + p] >= value for every p.  Returns false after the limit.
__device__ __forceinline__ bool wait_flags(const uint64_t* flags, int slot, int n, uint64_t value,
                                           uint64_t limit_ns, int* status) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < n) {
    const uint64_t* f = flags + slot * n + threadIdx.x;
    const uint64_t t0 = globaltimer_ns();
    uint32_t it = 0;
    while (ld_acquire_sys_u64(f) < value) {
      if ((++it & 63u) == 0u && globaltimer_ns() - t0 > limit_ns) {
        record_status(status, ST_COMM_TIMEOUT, threadIdx.x);
        s_ok = 0;
        break;
      }
    }
  }
  __syncthreads();
  return s_ok != 0;
}

__global__ void wait_flags_kernel(const uint64_t* flags, int slot, int n, uint64_t value,
                                  uint64_t limit_ns, int* status) {
  wait_flags(flags, slot, n, value, limit_ns, status);
}

struct AdamArgs {
  float lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale;
};

// Owner-side fused reduce-scatter + AdamW + all-gather for global elements [gstart, gend)
// (multiples of 8).  grads.p[r] / params.p[r] are rank r's fp32 gradient and bf16 weight flat
// buffers; p32 is this rank's flat master buffer (only its own shards are kept current), m / v
// are its moment shards with element `gstart` at index `moff`.
//
// MODE 0 does all three steps.  With gradient clipping the global norm is known only after the
// last bucket, so the step is split: MODE 1 reduces the shard over the ranks, leaves the sums in
// this rank's own gradient buffer (only the owner reads that range) and writes the block's sum
// of squares to partials[blockIdx.x] (fixed summation order, no atomics); MODE 2 reads the sums
// back, multiplies them by *clip_coef and does AdamW + all-gather.
// The kernel runs beside the backward pass and must share SMs with the persistent compute
// kernels: a GEMM CTA takes about 42K of an SM's 64K registers and nearly all of its shared
// memory, so a block here is small (128 threads, ~12-16K registers, no dynamic shared memory) and
// the launch spreads about one block per SM.  Blocks of 256 threads, two of which can land on one
// SM, kept the GEMM's CTA off that SM for the duration of the bucket (measured: the bucket time
// was then added to the step instead of hidden).
constexpr int RS_THREADS = 128;
template <int MODE, bool NVLS>
__global__ void __launch_bounds__(RS_THREADS)
rs_adamw_ag_kernel(PeerPtrs grads, PeerPtrs params, float* __restrict__ p32,
                   float* __restrict__ m, float* __restrict__ v, size_t gstart, size_t gend,
                   size_t moff, size_t decay_end, AdamArgs a, int n, const uint64_t* flags,
                   int slot, uint64_t expect, uint64_t limit_ns, int* status, int my_rank,
                   float* __restrict__ partials, const float* __restrict__ clip_coef,
                   const float* __restrict__ grads_mc, __nv_bfloat16* __restrict__ params_mc) {
  // grads_mc / params_mc (both or neither): NVLink multicast mappings of the gradient and weight
  // buffers.  With them the shard is read with multimem.ld_reduce (one load returns the sum over
  // all ranks, added in the switch) and the new weights leave with one multimem.st instead of a
  // store per rank.
  __shared__ float red[32];
  if (MODE != 2 && flags != nullptr && !wait_flags(flags, slot, n, expect, limit_ns, status)) {
    if (MODE == 1 && threadIdx.x == 0) partials[blockIdx.x] = 0.f;
    return;
  }
  if (MODE == 2) a.grad_scale *= *clip_coef;
  float sq = 0.f;
  const size_t nvec = (gend - gstart) >> 3;
  // what happens to one vector of eight summed gradients: AdamW on the owner's master weights and
  // moments and the broadcast of the new bf16 weights (MODE 0 / 2), or the store of the sums (1)
  auto update = [&](size_t i, float (&acc)[8]) {
    const size_t g0 = gstart + (i << 3);
    if (MODE == 1) {
      float* own = static_cast<float*>(grads.p[my_rank]) + g0;
      *reinterpret_cast<float4*>(own) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      *reinterpret_cast<float4*>(own + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
#pragma unroll
      for (int e = 0; e < 8; ++e) sq = fmaf(acc[e], acc[e], sq);
      return;
    }
    const size_t mi = moff + (i << 3);
    float pw[8], mm[8], vv[8];
    {
      const float4 p0 = *reinterpret_cast<const float4*>(p32 + g0);
      const float4 p1 = *reinterpret_cast<const float4*>(p32 + g0 + 4);
      const float4 m0 = *reinterpret_cast<const float4*>(m + mi);
      const float4 m1 = *reinterpret_cast<const float4*>(m + mi + 4);
      const float4 v0 = *reinterpret_cast<const float4*>(v + mi);
      const float4 v1 = *reinterpret_cast<const float4*>(v + mi + 4);
      pw[0] = p0.x; pw[1] = p0.y; pw[2] = p0.z; pw[3] = p0.w;
      pw[4] = p1.x; pw[5] = p1.y; pw[6] = p1.z; pw[7] = p1.w;
      mm[0] = m0.x; mm[1] = m0.y; mm[2] = m0.z; mm[3] = m0.w;
      mm[4] = m1.x; mm[5] = m1.y; mm[6] = m1.z; mm[7] = m1.w;
      vv[0] = v0.x; vv[1] = v0.y; vv[2] = v0.z; vv[3] = v0.w;
      vv[4] = v1.x; vv[5] = v1.y; vv[6] = v1.z; vv[7] = v1.w;
    }
    const float wd = g0 < decay_end ? a.wd : 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float g = acc[e] * a.grad_scale;
      mm[e] = a.beta1 * mm[e] + (1.f - a.beta1) * g;
      vv[e] = a.beta2 * vv[e] + (1.f - a.beta2) * g * g;
      pw[e] = pw[e] * (1.f - a.lr * wd) - a.lr * (mm[e] / a.bc1) / (sqrtf(vv[e] / a.bc2) + a.eps);
    }
    *reinterpret_cast<float4*>(p32 + g0) = make_float4(pw[0], pw[1], pw[2], pw[3]);
    *reinterpret_cast<float4*>(p32 + g0 + 4) = make_float4(pw[4], pw[5], pw[6], pw[7]);
    *reinterpret_cast<float4*>(m + mi) = make_float4(mm[0], mm[1], mm[2], mm[3]);
    *reinterpret_cast<float4*>(m + mi + 4) = make_float4(mm[4], mm[5], mm[6], mm[7]);
    *reinterpret_cast<float4*>(v + mi) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    *reinterpret_cast<float4*>(v + mi + 4) = make_float4(vv[4], vv[5], vv[6], vv[7]);
    uint4 o;
    o.x = pack_bf16x2(pw[0], pw[1]);
    o.y = pack_bf16x2(pw[2], pw[3]);
    o.z = pack_bf16x2(pw[4], pw[5]);
    o.w = pack_bf16x2(pw[6], pw[7]);
    if (NVLS) {
      asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                   :: "l"(params_mc + g0), "f"(__uint_as_float(o.x)), "f"(__uint_as_float(o.y)),
                      "f"(__uint_as_float(o.z)), "f"(__uint_as_float(o.w)) : "memory");
    } else {
#pragma unroll
      for (int r = 0; r < MAX_RANKS; ++r)
        if (r < n) *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(params.p[r]) + g0) = o;
    }
  };
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  const size_t first = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (NVLS && MODE != 2) {
    // D vectors per thread are requested before the first is used: with few blocks beside the
    // backward pass the loop lives on the bytes it keeps in flight through the switch
    constexpr int D = 4;
    for (size_t i0 = first; i0 < nvec; i0 += D * stride) {
      float4 qx[D], qy[D];
#pragma unroll
      for (int d = 0; d < D; ++d) {
        const size_t i = i0 + d * stride;
        if (i < nvec) {
          const float* gp = grads_mc + gstart + (i << 3);
          asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                       : "=f"(qx[d].x), "=f"(qx[d].y), "=f"(qx[d].z), "=f"(qx[d].w) : "l"(gp) : "memory");
          asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                       : "=f"(qy[d].x), "=f"(qy[d].y), "=f"(qy[d].z), "=f"(qy[d].w) : "l"(gp + 4) : "memory");
        }
      }
#pragma unroll
      for (int d = 0; d < D; ++d) {
        const size_t i = i0 + d * stride;
        if (i < nvec) {
          float acc[8] = {qx[d].x, qx[d].y, qx[d].z, qx[d].w, qy[d].x, qy[d].y, qy[d].z, qy[d].w};
          update(i, acc);
        }
      }
    }
  } else {
  for (size_t i = first; i < nvec; i += stride) {
    const size_t g0 = gstart + (i << 3);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (MODE == 2) {
      const float* gp = static_cast<const float*>(grads.p[my_rank]) + g0;
      const float4 x = *reinterpret_cast<const float4*>(gp);
      const float4 y = *reinterpret_cast<const float4*>(gp + 4);
      acc[0] = x.x; acc[1] = x.y; acc[2] = x.z; acc[3] = x.w;
      acc[4] = y.x; acc[5] = y.y; acc[6] = y.z; acc[7] = y.w;
    } else {
      // every rank's vector of a group of four is requested before the first one is used
      constexpr int U = 4;
      for (int r0 = 0; r0 < n; r0 += U) {
        float4 x[U], y[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (r0 + u < n) {
            const float* gp = static_cast<const float*>(grads.p[r0 + u]) + g0;
            x[u] = ld_relaxed_sys_f4(gp);
            y[u] = ld_relaxed_sys_f4(gp + 4);
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (r0 + u < n) {
            acc[0] += x[u].x; acc[1] += x[u].y; acc[2] += x[u].z; acc[3] += x[u].w;
            acc[4] += y[u].x; acc[5] += y[u].y; acc[6] += y[u].z; acc[7] += y[u].w;
          }
        }
      }
    }
    update(i, acc);
  }
  }
  if (MODE == 1) {
    const float tot = block_sum(sq, red);
    if (threadIdx.x == 0) partials[blockIdx.x] = tot;
  }
}

// out[r, c] = sum_s slots[s][r, c] (+ resid[r, c]) : the owner side of the reduce-scatter that
// the GEMM epilogues push into (bf16 slots, fp32 accumulation in slot order, so every run adds
// in the same order).  slots is one buffer of `tp` consecutive [rows, ld] matrices.
__global__ void reduce_slots_kernel(const __nv_bfloat16* __restrict__ slots, int tp, int rows,
                                    int cols, int ld, const __nv_bfloat16* __restrict__ resid,
                                    int ldr, __nv_bfloat16* __restrict__ out, int ldo) {
  const int nv = cols >> 3;
  const size_t total = static_cast<size_t>(rows) * nv;
  const size_t slot_stride = static_cast<size_t>(rows) * ld;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t r = i / nv;
    const int vec = static_cast<int>(i % nv);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int s = 0; s < tp; ++s) {
      float v[8];
      load8(slots + s * slot_stride + r * ld + vec * 8, v);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += v[e];
    }
    if (resid != nullptr) {
      float v[8];
      load8(resid + r * ldr + vec * 8, v);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += v[e];
    }
    store8(out + r * ldo + vec * 8, acc);
  }
}

// Plain peer copy kernel: dst[i] = src[i] for 16-byte vectors (src may be a peer pointer).
__global__ void peer_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                 size_t nvec) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * blockDim.x)
    dst[i] = ld_relaxed_sys_u4(src + i);
}

}  // namespace cb

using namespace cb;

// ---------------------------------------------------------------------- symmetric buffers
extern "C" int cb_symm_alloc(size_t bytes, void** out) {
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return -1;
  if (cudaMemset(p, 0, bytes) != cudaSuccess) return -2;
  *out = p;
  return 0;
}
extern "C" int cb_symm_free(void* p) { return cudaFree(p) == cudaSuccess ? 0 : -1; }
extern "C" int cb_ipc_get_handle(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) return -1;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
extern "C" int cb_ipc_open(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return -static_cast<int>(e);
  *out = p;
  return 0;
}
extern "C" int cb_ipc_close(void* p) { return cudaIpcCloseMemHandle(p) == cudaSuccess ? 0 : -1; }

// ---------------------------------------------------------------------- signals
extern "C" int cb_signal_peers(void* const* flag_ptrs, int slot, int n, int my_rank,
                               unsigned long long value, void* stream) {
  if (n < 1 || n > MAX_RANKS) return -1;
  PeerPtrs f;
  for (int i = 0; i < n; ++i) f.p[i] = flag_ptrs[i];
  signal_peers_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(f, slot, n, my_rank, value);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
extern "C" int cb_wait_flags(const void* flags, int slot, int n, unsigned long long value,
                             unsigned long long limit_ns, int* status, void* stream) {
  if (n < 1 || n > MAX_RANKS) return -1;
  wait_flags_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint64_t*>(flags), slot, n, value, limit_ns, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// ---------------------------------------------------------------------- fused DP step
// mode 0: fused reduce-scatter + AdamW + all-gather; mode 1: reduce-scatter into this rank's own
// gradient buffer plus per-block sums of squares in partials[0 .. blocks) (entries of blocks that
// are not launched are set to zero); mode 2: AdamW + all-gather from the reduced gradients,
// scaled by grad_scale * *clip_coef.
extern "C" int cb_rs_adamw_ag(void* const* grad_ptrs, void* const* param_ptrs, float* p32,
                              float* m, float* v, size_t gstart, size_t gend, size_t moff,
                              size_t decay_end, float lr, float beta1, float beta2, float eps,
                              float wd, int step, float grad_scale, int n, const void* flags,
                              int slot, unsigned long long expect, unsigned long long limit_ns,
                              int blocks, int* status, void* stream, int mode, int my_rank,
                              float* partials, const float* clip_coef, const void* grads_mc,
                              void* params_mc) {
  if (n < 1 || n > MAX_RANKS || mode < 0 || mode > 2 || my_rank < 0 || my_rank >= n) return -1;
  if (mode == 1 && partials == nullptr) return -1;
  if (mode == 2 && clip_coef == nullptr) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (blocks <= 0) blocks = 64;
  const int slots = blocks;
  if (gend <= gstart) {
    if (mode == 1) cudaMemsetAsync(partials, 0, sizeof(float) * slots, st);
    return 0;
  }
  if (((gend - gstart) & 7) != 0 || (gstart & 7) != 0 || (moff & 3) != 0) return -3;
  PeerPtrs g, p;
  for (int i = 0; i < n; ++i) { g.p[i] = grad_ptrs[i]; p.p[i] = param_ptrs[i]; }
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.wd = wd;
  a.bc1 = 1.0f - powf(beta1, static_cast<float>(step));
  a.bc2 = 1.0f - powf(beta2, static_cast<float>(step));
  a.grad_scale = grad_scale;
  const size_t need = ((gend - gstart) / 8 + RS_THREADS - 1) / RS_THREADS;
  if (static_cast<size_t>(blocks) > need) blocks = static_cast<int>(need);
  if (mode == 1 && blocks < slots)
    cudaMemsetAsync(partials + blocks, 0, sizeof(float) * (slots - blocks), st);
  const uint64_t* f = static_cast<const uint64_t*>(flags);
  const bool nvls = grads_mc != nullptr && params_mc != nullptr;
#define CB_RS_LAUNCH(MODE_)                                                                    \
  if (nvls)                                                                                    \
    rs_adamw_ag_kernel<MODE_, true><<<blocks, RS_THREADS, 0, st>>>(g, p, p32, m, v, gstart, gend, moff, \
                                                    decay_end, a, n, f, slot, expect, limit_ns, \
                                                    status, my_rank, partials, clip_coef,     \
                                                    static_cast<const float*>(grads_mc),      \
                                                    static_cast<__nv_bfloat16*>(params_mc));  \
  else                                                                                         \
  rs_adamw_ag_kernel<MODE_, false><<<blocks, RS_THREADS, 0, st>>>(g, p, p32, m, v, gstart, gend, moff,       \
                                                    decay_end, a, n, f, slot, expect, limit_ns, \
                                                    status, my_rank, partials, clip_coef,     \
                                                    static_cast<const float*>(grads_mc),      \
                                                    static_cast<__nv_bfloat16*>(params_mc))
  if (mode == 0) CB_RS_LAUNCH(0);
  else if (mode == 1) CB_RS_LAUNCH(1);
  else CB_RS_LAUNCH(2);
#undef CB_RS_LAUNCH
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int cb_reduce_slots(const void* slots, int tp, int rows, int cols, int ld,
                               const void* resid, int ldr, void* out, int ldo, void* stream) {
  if (cols % 8 != 0 || ld % 8 != 0 || ldo % 8 != 0) return -1;
  const size_t work = static_cast<size_t>(rows) * (cols / 8);
  const int blocks = static_cast<int>(min(static_cast<size_t>(sm_count()) * 8, (work + 255) / 256));
  reduce_slots_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(slots), tp, rows, cols, ld,
      static_cast<const __nv_bfloat16*>(resid), ldr, static_cast<__nv_bfloat16*>(out), ldo);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int cb_peer_copy(const void* src, void* dst, size_t bytes, int blocks, void* stream) {
  if (bytes % 16 != 0) return -1;
  if (blocks <= 0) blocks = 64;
  peer_copy_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), bytes / 16);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
