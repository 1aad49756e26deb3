// LayerNorm and RMSNorm, forward and backward, per token (row) statistics in fp32.
// The reference's math::layer_norm (plugins/model-transformer/src/lib.rs:105-128) takes its
// statistics over the whole [S*H] buffer it is handed; these kernels implement the standard
// per-token operator, which coincides with the reference at S = 1.
//
// Two families of kernels.  Rows of up to 2048 columns go through the row-pipelined kernels in
// the second half of this file (per-warp rings of row buffers in shared memory filled by bulk
// copies).  Wider rows use the kernels below: one row is handled by WPR warps of a 128-thread
// block (WPR = 4 up to 8192 columns) and lives in registers between the statistics pass and the
// normalisation pass, so x is read from HBM once; backward accumulates dgamma/dbeta per thread
// over a grid-stride loop of rows and finishes with one fp32 atomic add per column per block.
#include "common.cuh"
#include "ptx.cuh"

namespace cb {

constexpr int NORM_THREADS = 128;

template <int WPR>
__device__ __forceinline__ float group_sum(float v, float* red, int row_in_block, int wir) {
  v = warp_sum(v);
  if constexpr (WPR == 1) {
    return v;
  } else {
    const int lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) red[row_in_block * WPR + wir] = v;
    __syncthreads();
    float r = 0.f;
#pragma unroll
    for (int i = 0; i < WPR; ++i) r += red[row_in_block * WPR + i];
    return r;
  }
}

// y = (x - mean) * rstd * gamma + beta      (RMS: y = x * rstd * gamma)
template <int WPR, int NORM_NV, bool RMS>
__global__ void __launch_bounds__(NORM_THREADS)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                const __nv_bfloat16* __restrict__ beta, __nv_bfloat16* __restrict__ y,
                float* __restrict__ mean_out, float* __restrict__ rstd_out, int T, int H,
                float eps) {
  __shared__ float red[8];
  constexpr int RPB = (NORM_THREADS / 32) / WPR;  // rows per block
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_in_block = warp / WPR, wir = warp % WPR;
  const int tid_in_row = wir * 32 + lane;
  const int nv = H >> 3;
  const int nblocks_rows = (T + RPB - 1) / RPB;
  for (int rb = blockIdx.x; rb < nblocks_rows; rb += gridDim.x) {
    const int row = rb * RPB + row_in_block;
    const bool live = row < T;
    float v[NORM_NV][8];
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < NORM_NV; ++j) {
      const int vec = tid_in_row + j * 32 * WPR;
      if (live && vec < nv) {
        load8(x + static_cast<size_t>(row) * H + vec * 8, v[j]);
#pragma unroll
        for (int e = 0; e < 8; ++e) s += RMS ? v[j][e] * v[j][e] : v[j][e];
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[j][e] = 0.f;
      }
    }
    s = group_sum<WPR>(s, red, row_in_block, wir);
    float mean = 0.f, rstd;
    if constexpr (RMS) {
      rstd = rsqrtf(s / H + eps);
    } else {
      mean = s / H;
      float q = 0.f;
#pragma unroll
      for (int j = 0; j < NORM_NV; ++j) {
        const int vec = tid_in_row + j * 32 * WPR;
        if (live && vec < nv) {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float d = v[j][e] - mean;
            q += d * d;
          }
        }
      }
      q = group_sum<WPR>(q, red, row_in_block, wir);
      rstd = rsqrtf(q / H + eps);
    }
    if (live && tid_in_row == 0) {
      if (mean_out != nullptr) mean_out[row] = mean;
      rstd_out[row] = rstd;
    }
#pragma unroll
    for (int j = 0; j < NORM_NV; ++j) {
      const int vec = tid_in_row + j * 32 * WPR;
      if (live && vec < nv) {
        float g[8], b[8], o[8];
        load8(gamma + vec * 8, g);
        if (!RMS && beta != nullptr) {
          load8(beta + vec * 8, b);
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) b[e] = 0.f;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = (v[j][e] - mean) * rstd * g[e] + b[e];
        store8(y + static_cast<size_t>(row) * H + vec * 8, o);
      }
    }
  }
}

// dx = rstd * (dy*g - mean(dy*g) - xhat * mean(dy*g*xhat))  (+ dres)      [LayerNorm]
// dx = rstd * (dy*g - xhat * mean(dy*g*xhat))               (+ dres)      [RMSNorm]
// dgamma += sum_t dy*xhat ; dbeta += sum_t dy   (fp32, atomically accumulated)
template <int WPR, int NORM_NV, bool RMS>
__global__ void __launch_bounds__(NORM_THREADS)
norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres,
                __nv_bfloat16* __restrict__ dx, float* __restrict__ dgamma,
                float* __restrict__ dbeta, int T, int H) {
  __shared__ float red[8];
  extern __shared__ float colred[];  // [2][RPB][H] only used when RPB > 1
  constexpr int RPB = (NORM_THREADS / 32) / WPR;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_in_block = warp / WPR, wir = warp % WPR;
  const int tid_in_row = wir * 32 + lane;
  const int nv = H >> 3;
  const int nblocks_rows = (T + RPB - 1) / RPB;
  float accg[NORM_NV][8], accb[NORM_NV][8];
  float g[NORM_NV][8];
#pragma unroll
  for (int j = 0; j < NORM_NV; ++j) {
    const int vec = tid_in_row + j * 32 * WPR;
#pragma unroll
    for (int e = 0; e < 8; ++e) { accg[j][e] = 0.f; accb[j][e] = 0.f; g[j][e] = 0.f; }
    if (vec < nv) load8(gamma + vec * 8, g[j]);
  }
  for (int rb = blockIdx.x; rb < nblocks_rows; rb += gridDim.x) {
    const int row = rb * RPB + row_in_block;
    const bool live = row < T;
    const float mean = (live && !RMS) ? mean_in[row] : 0.f;
    const float rstd = live ? rstd_in[row] : 0.f;
    float xh[NORM_NV][8], dyv[NORM_NV][8];
    uint4 rres[NORM_NV];  // residual gradient, fetched up front so it overlaps the reductions
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int j = 0; j < NORM_NV; ++j) {
      const int vec = tid_in_row + j * 32 * WPR;
      rres[j] = make_uint4(0u, 0u, 0u, 0u);
      if (live && vec < nv) {
        load8(x + static_cast<size_t>(row) * H + vec * 8, xh[j]);
        load8(dy + static_cast<size_t>(row) * H + vec * 8, dyv[j]);
        if (dres != nullptr)
          rres[j] = *reinterpret_cast<const uint4*>(dres + static_cast<size_t>(row) * H + vec * 8);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          xh[j][e] = (xh[j][e] - mean) * rstd;
          const float dg = dyv[j][e] * g[j][e];
          s1 += dg;
          s2 += dg * xh[j][e];
          accg[j][e] += dyv[j][e] * xh[j][e];
          accb[j][e] += dyv[j][e];
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) { xh[j][e] = 0.f; dyv[j][e] = 0.f; }
      }
    }
    if constexpr (!RMS) s1 = group_sum<WPR>(s1, red, row_in_block, wir);
    s2 = group_sum<WPR>(s2, red, row_in_block, wir);
    const float m1 = RMS ? 0.f : s1 / H, m2 = s2 / H;
#pragma unroll
    for (int j = 0; j < NORM_NV; ++j) {
      const int vec = tid_in_row + j * 32 * WPR;
      if (live && vec < nv) {
        float o[8];
        const uint32_t rw[4] = {rres[j].x, rres[j].y, rres[j].z, rres[j].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 r2 = unpack_bf16x2(rw[e]);
          o[2 * e] = rstd * (dyv[j][2 * e] * g[j][2 * e] - m1 - xh[j][2 * e] * m2) + r2.x;
          o[2 * e + 1] =
              rstd * (dyv[j][2 * e + 1] * g[j][2 * e + 1] - m1 - xh[j][2 * e + 1] * m2) + r2.y;
        }
        store8(dx + static_cast<size_t>(row) * H + vec * 8, o);
      }
    }
  }
  // column sums: combine the RPB rows of the block in shared memory, then one atomic per column
  if constexpr (RPB > 1) {
    float* sg = colred;
    float* sb = colred + RPB * H;
    __syncthreads();
#pragma unroll
    for (int j = 0; j < NORM_NV; ++j) {
      const int vec = tid_in_row + j * 32 * WPR;
      if (vec < nv) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          sg[row_in_block * H + vec * 8 + e] = accg[j][e];
          sb[row_in_block * H + vec * 8 + e] = accb[j][e];
        }
      }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < H; c += NORM_THREADS) {
      float a = 0.f, b = 0.f;
#pragma unroll
      for (int r = 0; r < RPB; ++r) { a += sg[r * H + c]; b += sb[r * H + c]; }
      atomicAdd(dgamma + c, a);
      if (!RMS && dbeta != nullptr) atomicAdd(dbeta + c, b);
    }
  } else {
#pragma unroll
    for (int j = 0; j < NORM_NV; ++j) {
      const int vec = tid_in_row + j * 32 * WPR;
      if (vec < nv) {
#pragma unroll
        for (int e = 0; e < 8; e += 4) {   // four columns per reduction instruction
          asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                       ::"l"(dgamma + vec * 8 + e), "f"(accg[j][e]), "f"(accg[j][e + 1]),
                         "f"(accg[j][e + 2]), "f"(accg[j][e + 3]) : "memory");
          if (!RMS && dbeta != nullptr)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                         ::"l"(dbeta + vec * 8 + e), "f"(accb[j][e]), "f"(accb[j][e + 1]),
                           "f"(accb[j][e + 2]), "f"(accb[j][e + 3]) : "memory");
        }
      }
    }
  }
}


// ----------------------------------------------------------------------------------------------
// Row-pipelined variants for H <= 2048.  Every warp owns a ring of row buffers in shared memory
// that one lane fills with untiled bulk copies (completion on one mbarrier per stage) a few rows
// ahead of the row the warp is working on, so the bytes in flight do not depend on how many
// registers or warps an SM can hold (the plain kernels above keep a row in registers and have
// nothing in flight while they reduce and store: 0.45 / 0.37 of the copy bandwidth at
// 16384 x 1024).  With the loads out of the way the kernels are bound by instruction issue, so
// the arithmetic runs on pairs (fma.rn.f32x2), gamma / beta sit in shared memory as fp32 and the
// backward pass reads the row twice from shared memory instead of keeping it in registers.
// Results are stored straight from registers.
constexpr int PIPE_WARPS = 4;        // forward, and backward of rows wider than 1024
constexpr int PIPE_WARPS_BWD = 6;    // backward up to 1024 columns: two blocks of six warps fill an SM's shared memory

struct RowPipe {
  unsigned char* ring;        // this warp's stages
  uint32_t bars;              // shared-memory address of this warp's first mbarrier
  volatile uint32_t* abort_flag;
  uint32_t stage_bytes;
  int stages;
  int cur, parity;            // stage and phase of the row being worked on
  int fill;                   // stage that the next copy goes to

  // Shared memory: [head_bytes of the caller][warps x stages x stage_bytes][mbarriers][flag]
  __device__ __forceinline__ void init(unsigned char* smem, uint32_t head_bytes, int nstages,
                                       uint32_t sbytes) {
    const int warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    stages = nstages;
    stage_bytes = sbytes;
    cur = 0;
    parity = 0;
    fill = 0;
    unsigned char* base = smem + head_bytes;
    ring = base + static_cast<size_t>(warp) * nstages * sbytes;
    uint64_t* b = reinterpret_cast<uint64_t*>(base + static_cast<size_t>(nwarps) * nstages * sbytes);
    abort_flag = reinterpret_cast<volatile uint32_t*>(b + nwarps * nstages);
    bars = smem_u32(b + warp * nstages);
    if (threadIdx.x == 0) {
      for (int i = 0; i < nwarps * nstages; ++i) mbar_init(smem_u32(b + i), 1);
      *abort_flag = 0u;
      mbar_fence_init();
    }
  }
  __device__ __forceinline__ unsigned char* fill_ptr() const {
    return ring + static_cast<size_t>(fill) * stage_bytes;
  }
  __device__ __forceinline__ uint32_t fill_bar() const { return bars + 8u * fill; }
  __device__ __forceinline__ void filled() { fill = fill + 1 == stages ? 0 : fill + 1; }
  __device__ __forceinline__ const unsigned char* cur_ptr() const {
    return ring + static_cast<size_t>(cur) * stage_bytes;
  }
  // All lanes call this; false (for the whole warp) when the wait ran out of time.
  __device__ __forceinline__ bool wait() const {
    const bool ok = mbar_wait(bars + 8u * cur, static_cast<uint32_t>(parity), abort_flag);
    return __all_sync(0xffffffffu, ok);
  }
  __device__ __forceinline__ void advance() {
    if (++cur == stages) {
      cur = 0;
      parity ^= 1;
    }
  }
  // After a failed wait: give the copies that are still on their way (at most one per stage) a
  // bounded time to land before the block's shared memory goes away.
  __device__ __forceinline__ void drain(int outstanding) {
    for (int k = 0; k < outstanding; ++k) {
      for (int n = 0; n < (1 << 20) && !mbar_test_wait(bars + 8u * cur, static_cast<uint32_t>(parity)); ++n) {}
      advance();
    }
  }
};

__device__ __forceinline__ void mul2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
  asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "mul.rn.f32x2 rd, ra, rb;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
// The two bf16 halves of a word as floats: a shift and a mask.
__device__ __forceinline__ void unpack2(uint32_t w, float& lo, float& hi) {
  lo = __uint_as_float(w << 16);
  hi = __uint_as_float(w & 0xffff0000u);
}
__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  unpack2(u.x, f[0], f[1]);
  unpack2(u.y, f[2], f[3]);
  unpack2(u.z, f[4], f[5]);
  unpack2(u.w, f[6], f[7]);
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]);
  u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]);
  u.w = pack_bf16x2(f[6], f[7]);
  return u;
}
// fp32 copies of a bf16 vector (zeros when the pointer is null) in shared memory, by the block:
// eight columns a thread.
__device__ __forceinline__ void stage_vector(float* dst, const __nv_bfloat16* src, int H) {
  for (int vec = threadIdx.x; vec < (H >> 3); vec += blockDim.x) {
    float f[8];
    if (src != nullptr) {
      unpack8(*reinterpret_cast<const uint4*>(src + vec * 8), f);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = 0.f;
    }
    *reinterpret_cast<float4*>(dst + vec * 8) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(dst + vec * 8 + 4) = make_float4(f[4], f[5], f[6], f[7]);
  }
}

template <int NORM_NV, bool RMS>
__global__ void __launch_bounds__(PIPE_WARPS * 32, NORM_NV <= 4 ? 5 : 3)
norm_fwd_pipe_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                     const __nv_bfloat16* __restrict__ beta, __nv_bfloat16* __restrict__ y,
                     float* __restrict__ mean_out, float* __restrict__ rstd_out, int T, int H,
                     float eps, int stages, int* status) {
  extern __shared__ __align__(128) unsigned char pipe_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nv = H >> 3;
  const uint32_t row_bytes = static_cast<uint32_t>(H) * 2u;
  float* gs = reinterpret_cast<float*>(pipe_smem);   // gamma [H], then beta [H] (LayerNorm)
  float* bs = gs + H;
  RowPipe pipe;
  pipe.init(pipe_smem, (RMS ? 1u : 2u) * static_cast<uint32_t>(H) * 4u, stages, row_bytes);
  __syncthreads();      // the mbarriers are initialised
  const int gw = blockIdx.x * PIPE_WARPS + warp, GW = gridDim.x * PIPE_WARPS;
  int next_row = gw;          // the row that the next copy fetches
  auto issue = [&]() {
    if (lane == 0 && next_row < T) {
      mbar_arrive_expect_tx(pipe.fill_bar(), row_bytes);
      bulk_load_g2s(smem_u32(pipe.fill_ptr()), x + static_cast<size_t>(next_row) * H, row_bytes,
                    pipe.fill_bar());
    }
    pipe.filled();
    next_row += GW;
  };
  for (int i = 0; i < stages - 1; ++i) issue();     // every lane keeps the counters, lane 0 copies
  stage_vector(gs, gamma, H);                       // while the first rows are on their way
  if constexpr (!RMS) stage_vector(bs, beta, H);
  __syncthreads();
  const float inv_h = 1.0f / H;
  for (int row = gw; row < T; row += GW) {
    // refills the stage that was read in the previous round (all lanes passed its __syncwarp)
    issue();
    if (!pipe.wait()) {
      if (lane == 0) record_status(status, ST_WAIT_TIMEOUT, 940);
      pipe.drain(stages);
      break;
    }
    const uint4* src = reinterpret_cast<const uint4*>(pipe.cur_ptr());
    float v[NORM_NV][8];
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int j = 0; j < NORM_NV; ++j) {
      const int vec = lane + j * 32;
      if (vec < nv) {
        unpack8(src[vec], v[j]);
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          if constexpr (RMS) fma2(s0, s1, v[j][e], v[j][e + 1], v[j][e], v[j][e + 1], s0, s1);
          else add2(s0, s1, s0, s1, v[j][e], v[j][e + 1]);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[j][e] = 0.f;
      }
    }
    __syncwarp();     // the row is in registers: its stage may be refilled in the next round
    pipe.advance();
    const float s = warp_sum(s0 + s1);
    float mean = 0.f, rstd;
    if constexpr (RMS) {
      rstd = rsqrtf(s * inv_h + eps);
    } else {
      mean = s * inv_h;
      float q0 = 0.f, q1 = 0.f;
#pragma unroll
      for (int j = 0; j < NORM_NV; ++j) {
        if (lane + j * 32 < nv) {
#pragma unroll
          for (int e = 0; e < 8; e += 2) {   // v becomes x - mean
            add2(v[j][e], v[j][e + 1], v[j][e], v[j][e + 1], -mean, -mean);
            fma2(q0, q1, v[j][e], v[j][e + 1], v[j][e], v[j][e + 1], q0, q1);
          }
        }
      }
      rstd = rsqrtf(warp_sum(q0 + q1) * inv_h + eps);
    }
    if (lane == 0) {
      if (mean_out != nullptr) mean_out[row] = mean;
      rstd_out[row] = rstd;
    }
#pragma unroll
    for (int j = 0; j < NORM_NV; ++j) {
      const int vec = lane + j * 32;
      if (vec < nv) {
        float o[8];
        const float4 ga = *reinterpret_cast<const float4*>(gs + vec * 8);
        const float4 gb = *reinterpret_cast<const float4*>(gs + vec * 8 + 4);
        const float g[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
        if constexpr (RMS) {
#pragma unroll
          for (int e = 0; e < 8; e += 2) {
            float t0, t1;
            mul2(t0, t1, g[e], g[e + 1], rstd, rstd);
            mul2(o[e], o[e + 1], v[j][e], v[j][e + 1], t0, t1);
          }
        } else {
          const float4 ba = *reinterpret_cast<const float4*>(bs + vec * 8);
          const float4 bb = *reinterpret_cast<const float4*>(bs + vec * 8 + 4);
          const float b[8] = {ba.x, ba.y, ba.z, ba.w, bb.x, bb.y, bb.z, bb.w};
#pragma unroll
          for (int e = 0; e < 8; e += 2) {
            float t0, t1;
            mul2(t0, t1, g[e], g[e + 1], rstd, rstd);
            fma2(o[e], o[e + 1], v[j][e], v[j][e + 1], t0, t1, b[e], b[e + 1]);
          }
        }
        *reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * H + vec * 8) = pack8(o);
      }
    }
  }
}

// Backward: a stage holds the row of x, of dy and (when given) of the residual gradient.  With
// COLS the column sums of the result dx are accumulated too (the bias gradient of the linear
// layer whose output this residual stream is), which saves a separate pass over dx.
//   dx = dy * (rstd * g) + x * A + B (+ dres),  A = -rstd^2 * m2,  B = -rstd * m1 - mean * A,
//   m1 = mean_c(dy * g) (0 for RMSNorm), m2 = mean_c(dy * g * xhat), xhat = x * rstd - mean * rstd
template <int NORM_NV, bool RMS, bool COLS>
__global__ void __launch_bounds__((NORM_NV <= 4 ? PIPE_WARPS_BWD : PIPE_WARPS) * 32, 2)
norm_bwd_pipe_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                     const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                     const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres,
                     __nv_bfloat16* __restrict__ dx, float* __restrict__ dgamma,
                     float* __restrict__ dbeta, float* __restrict__ dcol, int T, int H,
                     int stages, int* status) {
  extern __shared__ __align__(128) unsigned char pipe_smem[];
  constexpr int NW = NORM_NV <= 4 ? PIPE_WARPS_BWD : PIPE_WARPS;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nv = H >> 3;
  const uint32_t row_bytes = static_cast<uint32_t>(H) * 2u;
  const uint32_t nin = dres != nullptr ? 3u : 2u;
  float* gs = reinterpret_cast<float*>(pipe_smem);   // gamma [H] as fp32
  RowPipe pipe;
  pipe.init(pipe_smem, static_cast<uint32_t>(H) * 4u, stages, nin * row_bytes);
  __syncthreads();      // the mbarriers are initialised
  const int gw = blockIdx.x * NW + warp, GW = gridDim.x * NW;
  int next_row = gw;
  auto issue = [&]() {
    if (lane == 0 && next_row < T) {
      const uint32_t dst = smem_u32(pipe.fill_ptr()), bar = pipe.fill_bar();
      const size_t off = static_cast<size_t>(next_row) * H;
      mbar_arrive_expect_tx(bar, nin * row_bytes);
      bulk_load_g2s(dst, x + off, row_bytes, bar);
      bulk_load_g2s(dst + row_bytes, dy + off, row_bytes, bar);
      if (dres != nullptr) bulk_load_g2s(dst + 2u * row_bytes, dres + off, row_bytes, bar);
    }
    pipe.filled();
    next_row += GW;
  };
  for (int i = 0; i < stages - 1; ++i) issue();
  stage_vector(gs, gamma, H);   // while the first rows are on their way
  __syncthreads();
  float accg[NORM_NV][8], accb[RMS ? 1 : NORM_NV][8], accc[COLS ? NORM_NV : 1][8];
#pragma unroll
  for (int j = 0; j < NORM_NV; ++j) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      accg[j][e] = 0.f;
      if constexpr (!RMS) accb[j][e] = 0.f;
      if constexpr (COLS) accc[j][e] = 0.f;
    }
  }
  const float inv_h = 1.0f / H;
  for (int row = gw; row < T; row += GW) {
    issue();
    const float mean = RMS ? 0.f : mean_in[row];
    const float rstd = rstd_in[row];
    if (!pipe.wait()) {
      if (lane == 0) record_status(status, ST_WAIT_TIMEOUT, 941);
      pipe.drain(stages);
      break;
    }
    const uint4* sx = reinterpret_cast<const uint4*>(pipe.cur_ptr());
    const uint4* sdy = sx + nv;
    const uint4* sdr = sx + 2 * nv;
    const float c = -mean * rstd;            // xhat = x * rstd + c
    // first pass over the row (in shared memory): the two row sums and the column accumulators
    float s10 = 0.f, s11 = 0.f, s20 = 0.f, s21 = 0.f;
#pragma unroll
    for (int j = 0; j < NORM_NV; ++j) {
      const int vec = lane + j * 32;
      if (vec < nv) {
        float xh[8], dyv[8];
        unpack8(sx[vec], xh);
        unpack8(sdy[vec], dyv);
        const float4 ga = *reinterpret_cast<const float4*>(gs + vec * 8);
        const float4 gb = *reinterpret_cast<const float4*>(gs + vec * 8 + 4);
        const float g[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          float d0, d1;
          fma2(xh[e], xh[e + 1], xh[e], xh[e + 1], rstd, rstd, c, c);
          mul2(d0, d1, dyv[e], dyv[e + 1], g[e], g[e + 1]);
          if constexpr (!RMS) add2(s10, s11, s10, s11, d0, d1);
          fma2(s20, s21, d0, d1, xh[e], xh[e + 1], s20, s21);
          fma2(accg[j][e], accg[j][e + 1], dyv[e], dyv[e + 1], xh[e], xh[e + 1], accg[j][e],
               accg[j][e + 1]);
          if constexpr (!RMS)
            add2(accb[j][e], accb[j][e + 1], accb[j][e], accb[j][e + 1], dyv[e], dyv[e + 1]);
        }
      }
    }
    const float m1 = RMS ? 0.f : warp_sum(s10 + s11) * inv_h;
    const float m2 = warp_sum(s20 + s21) * inv_h;
    const float A = -rstd * rstd * m2;
    const float Bc = -rstd * m1 - mean * A;
    // second pass: the row is read again from shared memory instead of being kept in registers
#pragma unroll
    for (int j = 0; j < NORM_NV; ++j) {
      const int vec = lane + j * 32;
      if (vec < nv) {
        float xv[8], dyv[8], o[8];
        unpack8(sx[vec], xv);
        unpack8(sdy[vec], dyv);
        if (dres != nullptr) {
          unpack8(sdr[vec], o);
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = 0.f;
        }
        const float4 ga = *reinterpret_cast<const float4*>(gs + vec * 8);
        const float4 gb = *reinterpret_cast<const float4*>(gs + vec * 8 + 4);
        const float g[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          float t0, t1;
          add2(o[e], o[e + 1], o[e], o[e + 1], Bc, Bc);
          mul2(t0, t1, g[e], g[e + 1], rstd, rstd);
          fma2(o[e], o[e + 1], dyv[e], dyv[e + 1], t0, t1, o[e], o[e + 1]);
          fma2(o[e], o[e + 1], xv[e], xv[e + 1], A, A, o[e], o[e + 1]);
          if constexpr (COLS)
            add2(accc[j][e], accc[j][e + 1], accc[j][e], accc[j][e + 1], o[e], o[e + 1]);
        }
        *reinterpret_cast<uint4*>(dx + static_cast<size_t>(row) * H + vec * 8) = pack8(o);
      }
    }
    __syncwarp();   // every lane is done with the stage: the next round's copy may refill it
    pipe.advance();
  }
  // Column sums: the warps of the block are combined in shared memory (the ring is idle
  // now: every copy that was issued has been waited for), then one reduction per four columns.
  __syncthreads();
  if (*pipe.abort_flag) return;   // a wait ran out of time: the status word says so
  float* sg = reinterpret_cast<float*>(pipe_smem);
  auto combine = [&](float (*acc)[8], float* out) {
#pragma unroll
    for (int j = 0; j < NORM_NV; ++j) {
      const int vec = lane + j * 32;
      if (vec < nv) {
        *reinterpret_cast<float4*>(sg + warp * H + vec * 8) =
            make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
        *reinterpret_cast<float4*>(sg + warp * H + vec * 8 + 4) =
            make_float4(acc[j][4], acc[j][5], acc[j][6], acc[j][7]);
      }
    }
    __syncthreads();
    for (int c4 = threadIdx.x * 4; c4 < H; c4 += NW * 32 * 4) {
      float4 a = *reinterpret_cast<const float4*>(sg + c4);
#pragma unroll
      for (int w = 1; w < NW; ++w) {
        const float4 t = *reinterpret_cast<const float4*>(sg + w * H + c4);
        a.x += t.x; a.y += t.y; a.z += t.z; a.w += t.w;
      }
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                   ::"l"(out + c4), "f"(a.x), "f"(a.y), "f"(a.z), "f"(a.w) : "memory");
    }
    __syncthreads();
  };
  combine(accg, dgamma);
  if constexpr (!RMS) {
    if (dbeta != nullptr) combine(accb, dbeta);
  }
  if constexpr (COLS) combine(accc, dcol);
}

int sm_count();

}  // namespace cb

using namespace cb;

namespace {
template <int WPR, int NV>
int launch_fwd(const __nv_bfloat16* X, const __nv_bfloat16* G, const __nv_bfloat16* B,
               __nv_bfloat16* Y, float* mean, float* rstd, int T, int H, float eps, int rms,
               cudaStream_t st) {
  constexpr int RPB = 4 / WPR;
  const int blocks = min((T + RPB - 1) / RPB, sm_count() * 16);
  if (rms)
    norm_fwd_kernel<WPR, NV, true><<<blocks, NORM_THREADS, 0, st>>>(X, G, B, Y, mean, rstd, T, H, eps);
  else
    norm_fwd_kernel<WPR, NV, false><<<blocks, NORM_THREADS, 0, st>>>(X, G, B, Y, mean, rstd, T, H, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
template <int WPR, int NV, bool RMS>
int launch_bwd(const __nv_bfloat16* DY, const __nv_bfloat16* X, const __nv_bfloat16* G,
               const float* mean, const float* rstd, const __nv_bfloat16* DR,
               __nv_bfloat16* DX, float* dgamma, float* dbeta, int T, int H, cudaStream_t st) {
  constexpr int RPB = 4 / WPR;
  // persistent blocks: as many as can be resident (the register count falls with the share of a
  // row that one thread holds)
  const int per_sm = WPR == 1 ? 3 : (WPR == 2 ? 4 : 3);   // every block ends with H column reductions
  const int blocks = min((T + RPB - 1) / RPB, sm_count() * per_sm);
  const size_t sh = RPB > 1 ? 2 * RPB * static_cast<size_t>(H) * sizeof(float) : 0;
  static bool configured = false;
  if (!configured && sh > 0) {
    cudaFuncSetAttribute(norm_bwd_kernel<WPR, NV, RMS>,
                         cudaFuncAttributeMaxDynamicSharedMemorySize, 65536);
    configured = true;
  }
  norm_bwd_kernel<WPR, NV, RMS><<<blocks, NORM_THREADS, sh, st>>>(DY, X, G, mean, rstd, DR, DX,
                                                                 dgamma, dbeta, T, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

constexpr size_t PIPE_SMEM_MAX = 113 * 1024;
inline size_t pipe_smem_bytes(size_t head_bytes, int warps, int stages, size_t stage_bytes) {
  return head_bytes + warps * stages * stage_bytes + warps * stages * 8 + 16;
}
inline int pipe_blocks(int T, int warps, size_t sh, int reg_limit) {
  const int by_smem = static_cast<int>((228 * 1024) / (sh + 1024));
  const int per_sm = max(1, min(reg_limit, by_smem));
  return min((T + warps - 1) / warps, sm_count() * per_sm);
}
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <int NV, bool RMS>
int launch_fwd_pipe(const __nv_bfloat16* X, const __nv_bfloat16* G, const __nv_bfloat16* B,
                    __nv_bfloat16* Y, float* mean, float* rstd, int T, int H, float eps,
                    int* status, cudaStream_t st) {
  const size_t row_bytes = static_cast<size_t>(H) * 2;
  const int stages = row_bytes <= 2048 ? 4 : 3;
  const size_t sh = pipe_smem_bytes((RMS ? 1 : 2) * static_cast<size_t>(H) * 4, PIPE_WARPS, stages, row_bytes);
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(norm_fwd_pipe_kernel<NV, RMS>,
                         cudaFuncAttributeMaxDynamicSharedMemorySize, PIPE_SMEM_MAX);
    configured = true;
  }
  norm_fwd_pipe_kernel<NV, RMS><<<pipe_blocks(T, PIPE_WARPS, sh, NV <= 4 ? 5 : 3), PIPE_WARPS * 32, sh, st>>>(
      X, G, B, Y, mean, rstd, T, H, eps, stages, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

template <int NV, bool RMS, bool COLS>
int launch_bwd_pipe(const __nv_bfloat16* DY, const __nv_bfloat16* X, const __nv_bfloat16* G,
                    const float* mean, const float* rstd, const __nv_bfloat16* DR,
                    __nv_bfloat16* DX, float* dgamma, float* dbeta, float* dcol, int T, int H,
                    int* status, cudaStream_t st) {
  const size_t stage_bytes = static_cast<size_t>(H) * 2 * (DR != nullptr ? 3 : 2);
  const int stages = stage_bytes <= 8192 ? 3 : 2;
  constexpr int NW = NV <= 4 ? PIPE_WARPS_BWD : PIPE_WARPS;
  const size_t sh = pipe_smem_bytes(static_cast<size_t>(H) * 4, NW, stages, stage_bytes);
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(norm_bwd_pipe_kernel<NV, RMS, COLS>,
                         cudaFuncAttributeMaxDynamicSharedMemorySize, PIPE_SMEM_MAX);
    configured = true;
  }
  norm_bwd_pipe_kernel<NV, RMS, COLS><<<pipe_blocks(T, NW, sh, 2), NW * 32, sh, st>>>(
      DY, X, G, mean, rstd, DR, DX, dgamma, dbeta, dcol, T, H, stages, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
}  // namespace

// 3: row-pipelined kernel (H <= 2048); 0, 1, 2: a row / half a row / a quarter of a row per warp
// in registers.
static int g_norm_bwd_variant = 3;
static int g_norm_fwd_variant = 1;   // 1: row-pipelined kernel (H <= 2048); 0: row in registers
extern "C" void cb_norm_bwd_variant(int v) { g_norm_bwd_variant = v; }
extern "C" void cb_norm_fwd_variant(int v) { g_norm_fwd_variant = v; }

// rms == 0: LayerNorm (beta may be null); rms == 1: RMSNorm (mean may be null).  status: the
// per-device status word (may be null).
extern "C" int cb_norm_fwd(const void* x, const void* gamma, const void* beta, void* y,
                           float* mean, float* rstd, int T, int H, float eps, int rms,
                           int* status, void* stream) {
  if (H % 8 != 0 || H > 8192 || T <= 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto G = static_cast<const __nv_bfloat16*>(gamma);
  auto B = static_cast<const __nv_bfloat16*>(beta);
  auto Y = static_cast<__nv_bfloat16*>(y);
  if (g_norm_fwd_variant == 1 && H <= 2048 && aligned16(x) && aligned16(y) && aligned16(gamma) &&
      aligned16(beta)) {
    if (H <= 1024)
      return rms ? launch_fwd_pipe<4, true>(X, G, B, Y, mean, rstd, T, H, eps, status, st)
                 : launch_fwd_pipe<4, false>(X, G, B, Y, mean, rstd, T, H, eps, status, st);
    return rms ? launch_fwd_pipe<8, true>(X, G, B, Y, mean, rstd, T, H, eps, status, st)
               : launch_fwd_pipe<8, false>(X, G, B, Y, mean, rstd, T, H, eps, status, st);
  }
  if (H <= 1024) return launch_fwd<1, 4>(X, G, B, Y, mean, rstd, T, H, eps, rms, st);
  if (H <= 2048) return launch_fwd<1, 8>(X, G, B, Y, mean, rstd, T, H, eps, rms, st);
  return launch_fwd<4, 8>(X, G, B, Y, mean, rstd, T, H, eps, rms, st);
}

// dgamma / dbeta are fp32 and are accumulated into (zero them before the first call).  dcol
// (fp32 [H], may be null) receives the column sums of dx, accumulated as well: only the
// row-pipelined kernel computes them, so -3 is returned when dcol is given and that kernel does
// not apply (the caller then sums the columns of dx itself).
extern "C" int cb_norm_bwd(const void* dy, const void* x, const void* gamma, const float* mean,
                           const float* rstd, const void* dres, void* dx, float* dgamma,
                           float* dbeta, float* dcol, int T, int H, int rms, int* status,
                           void* stream) {
  if (H % 8 != 0 || H > 8192 || T <= 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto DY = static_cast<const __nv_bfloat16*>(dy);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto G = static_cast<const __nv_bfloat16*>(gamma);
  auto DR = static_cast<const __nv_bfloat16*>(dres);
  auto DX = static_cast<__nv_bfloat16*>(dx);
  const bool pipe_ok = g_norm_bwd_variant == 3 && H <= 2048 && aligned16(dy) && aligned16(x) &&
                       aligned16(gamma) && aligned16(dres) && aligned16(dx) && aligned16(dgamma) &&
                       aligned16(dbeta) && aligned16(dcol);
  if (pipe_ok) {
#define CB_PIPE(NV, RMS)                                                                          \
  return dcol != nullptr                                                                          \
             ? launch_bwd_pipe<NV, RMS, true>(DY, X, G, mean, rstd, DR, DX, dgamma, dbeta, dcol,  \
                                              T, H, status, st)                                   \
             : launch_bwd_pipe<NV, RMS, false>(DY, X, G, mean, rstd, DR, DX, dgamma, dbeta,       \
                                               nullptr, T, H, status, st)
    if (H <= 1024) {
      if (rms) { CB_PIPE(4, true); }
      CB_PIPE(4, false);
    }
    if (rms) { CB_PIPE(8, true); }
    CB_PIPE(8, false);
#undef CB_PIPE
  }
  if (dcol != nullptr) return -3;
#define CB_BWD(WPR, NV)                                                                        \
  return rms ? launch_bwd<WPR, NV, true>(DY, X, G, mean, rstd, DR, DX, dgamma, dbeta, T, H, st) \
             : launch_bwd<WPR, NV, false>(DY, X, G, mean, rstd, DR, DX, dgamma, dbeta, T, H, st)
  if (H <= 1024) {
    if (g_norm_bwd_variant == 1 || g_norm_bwd_variant == 3) { CB_BWD(2, 2); }
    if (g_norm_bwd_variant == 2) { CB_BWD(4, 1); }
    CB_BWD(1, 4);
  }
  if (H <= 4096) { CB_BWD(4, 4); }
  CB_BWD(4, 8);
#undef CB_BWD
}
