// LayerNorm and RMSNorm, forward and backward, per token (row) statistics in fp32.
// The reference's math::layer_norm (plugins/model-transformer/src/lib.rs:105-128) takes its
// statistics over the whole [S*H] buffer it is handed; these kernels implement the standard
// per-token operator, which coincides with the reference at S = 1.
//
// One row is handled by WPR warps of a 128-thread block (WPR = 1 for H <= 2048, 4 up to 8192);
// a row lives in registers between the statistics pass and the normalisation pass, so x is
// read from HBM once.  Backward accumulates dgamma/dbeta per thread over a grid-stride loop of
// rows and finishes with one fp32 atomic add per column per block.
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
}  // namespace

static int g_norm_bwd_variant = 1;   // half a row per warp: 123 registers, four blocks per SM
extern "C" void cb_norm_bwd_variant(int v) { g_norm_bwd_variant = v; }

// rms == 0: LayerNorm (beta may be null); rms == 1: RMSNorm (mean may be null).
extern "C" int cb_norm_fwd(const void* x, const void* gamma, const void* beta, void* y,
                           float* mean, float* rstd, int T, int H, float eps, int rms,
                           void* stream) {
  if (H % 8 != 0 || H > 8192 || T <= 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto G = static_cast<const __nv_bfloat16*>(gamma);
  auto B = static_cast<const __nv_bfloat16*>(beta);
  auto Y = static_cast<__nv_bfloat16*>(y);
  if (H <= 1024) return launch_fwd<1, 4>(X, G, B, Y, mean, rstd, T, H, eps, rms, st);
  if (H <= 2048) return launch_fwd<1, 8>(X, G, B, Y, mean, rstd, T, H, eps, rms, st);
  return launch_fwd<4, 8>(X, G, B, Y, mean, rstd, T, H, eps, rms, st);
}

// dgamma / dbeta are fp32 and are accumulated into (zero them before the first call).
extern "C" int cb_norm_bwd(const void* dy, const void* x, const void* gamma, const float* mean,
                           const float* rstd, const void* dres, void* dx, float* dgamma,
                           float* dbeta, int T, int H, int rms, void* stream) {
  if (H % 8 != 0 || H > 8192 || T <= 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto DY = static_cast<const __nv_bfloat16*>(dy);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto G = static_cast<const __nv_bfloat16*>(gamma);
  auto DR = static_cast<const __nv_bfloat16*>(dres);
  auto DX = static_cast<__nv_bfloat16*>(dx);
#define CB_BWD(WPR, NV)                                                                        \
  return rms ? launch_bwd<WPR, NV, true>(DY, X, G, mean, rstd, DR, DX, dgamma, dbeta, T, H, st) \
             : launch_bwd<WPR, NV, false>(DY, X, G, mean, rstd, DR, DX, dgamma, dbeta, T, H, st)
  if (H <= 1024) {
    if (g_norm_bwd_variant == 1) { CB_BWD(2, 2); }
    if (g_norm_bwd_variant == 2) { CB_BWD(4, 1); }
    CB_BWD(1, 4);
  }
  if (H <= 4096) { CB_BWD(4, 4); }
  CB_BWD(4, 8);
#undef CB_BWD
}
