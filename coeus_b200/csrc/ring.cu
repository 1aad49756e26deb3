// Helpers of context-parallel (ring) attention.
//   attn_merge      running (O, lse) of a query chunk absorbs the partial (O_p, lse_p) computed
//                   against one more key/value chunk:  lse' = log(exp(lse) + exp(lse_p)),
//                   O' = O * exp(lse - lse') + O_p * exp(lse_p - lse')   (O kept in fp32)
//   accum_rows      acc_f32[t, :] += x_bf16[t, :]  (strided source rows: dq/dk/dv slices)
//   peer_add_f32    dst[i] += src[i] with system-scope reductions; dst may be another GPU's
//                   memory (key/value gradients go home to the rank that owns the chunk)
//   cast_rows       bf16 <- fp32 rows with an optional scale
#include "common.cuh"
#include "ptx.cuh"

namespace cb {
int sm_count();

__global__ void attn_merge_kernel(float* __restrict__ o_acc, float* __restrict__ lse_acc,
                                  const __nv_bfloat16* __restrict__ o_p, int ld_p,
                                  const float* __restrict__ lse_p, int B, int S, int nh, int dh,
                                  int first) {
  // one warp per (row, head)
  const int lane = threadIdx.x & 31;
  const size_t warp_id = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) >> 5;
  const size_t n_warps = (static_cast<size_t>(gridDim.x) * blockDim.x) >> 5;
  const size_t total = static_cast<size_t>(B) * S * nh;
  const int H = nh * dh;
  for (size_t w = warp_id; w < total; w += n_warps) {
    const int h = static_cast<int>(w % nh);
    const size_t row = w / nh;             // b * S + s
    const size_t b = row / S, s = row % S;
    const size_t li = (b * nh + h) * S + s;
    const float lp = lse_p[li];
    float wa = 0.f, wp = 1.f, ln = lp;
    if (!first) {
      const float la = lse_acc[li];
      const float mx = fmaxf(la, lp);
      if (mx == -INFINITY) { wa = 0.f; wp = 0.f; ln = -INFINITY; }
      else {
        const float ea = __expf(la - mx), ep = __expf(lp - mx);
        ln = mx + __logf(ea + ep);
        wa = ea / (ea + ep);
        wp = ep / (ea + ep);
      }
    }
    float* oa = o_acc + row * H + h * dh;
    const __nv_bfloat16* op = o_p + row * ld_p + h * dh;
    for (int d = lane; d < dh; d += 32) {
      const float prev = first ? 0.f : oa[d];
      oa[d] = prev * wa + __bfloat162float(op[d]) * wp;
    }
    if (lane == 0) lse_acc[li] = ln;
  }
}

__global__ void accum_rows_kernel(float* __restrict__ acc, int ld_acc,
                                  const __nv_bfloat16* __restrict__ x, int ld_x, int T, int W) {
  const int nv = W >> 3;
  const size_t total = static_cast<size_t>(T) * nv;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t t = i / nv;
    const int vec = static_cast<int>(i % nv);
    float v[8];
    load8(x + t * ld_x + vec * 8, v);
    float4* a = reinterpret_cast<float4*>(acc + t * ld_acc + vec * 8);
    float4 a0 = a[0], a1 = a[1];
    a0.x += v[0]; a0.y += v[1]; a0.z += v[2]; a0.w += v[3];
    a1.x += v[4]; a1.y += v[5]; a1.z += v[6]; a1.w += v[7];
    a[0] = a0; a[1] = a1;
  }
}

__global__ void peer_add_f32_kernel(float* __restrict__ dst, const float* __restrict__ src, size_t n4) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(src)[i];
    asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                 :: "l"(dst + i * 4), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
  }
}

__global__ void cast_rows_kernel(const float* __restrict__ src, int ld_src,
                                 __nv_bfloat16* __restrict__ dst, int ld_dst, int T, int W,
                                 float scale) {
  const int nv = W >> 3;
  const size_t total = static_cast<size_t>(T) * nv;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t t = i / nv;
    const int vec = static_cast<int>(i % nv);
    const float4* s = reinterpret_cast<const float4*>(src + t * ld_src + vec * 8);
    const float4 a = s[0], b = s[1];
    float v[8] = {a.x * scale, a.y * scale, a.z * scale, a.w * scale,
                  b.x * scale, b.y * scale, b.z * scale, b.w * scale};
    store8(dst + t * ld_dst + vec * 8, v);
  }
}

static inline int ring_grid(size_t work) {
  const size_t b = (work + 255) / 256, cap = static_cast<size_t>(sm_count()) * 8;
  return static_cast<int>(b < cap ? (b ? b : 1) : cap);
}
}  // namespace cb

using namespace cb;
#define CB_ST(s) static_cast<cudaStream_t>(s)

extern "C" int cb_attn_merge(float* o_acc, float* lse_acc, const void* o_p, int ld_p,
                             const float* lse_p, int B, int S, int nh, int dh, int first,
                             void* stream) {
  attn_merge_kernel<<<ring_grid(static_cast<size_t>(B) * S * nh * 32), 256, 0, CB_ST(stream)>>>(
      o_acc, lse_acc, static_cast<const __nv_bfloat16*>(o_p), ld_p, lse_p, B, S, nh, dh, first);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int cb_accum_rows(float* acc, int ld_acc, const void* x, int ld_x, int T, int W,
                             void* stream) {
  if (W % 8 != 0 || ld_acc % 4 != 0) return -1;
  accum_rows_kernel<<<ring_grid(static_cast<size_t>(T) * (W / 8)), 256, 0, CB_ST(stream)>>>(
      acc, ld_acc, static_cast<const __nv_bfloat16*>(x), ld_x, T, W);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int cb_peer_add_f32(float* dst, const float* src, size_t n, void* stream) {
  if (n % 4 != 0) return -1;
  peer_add_f32_kernel<<<ring_grid(n / 4), 256, 0, CB_ST(stream)>>>(dst, src, n / 4);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int cb_cast_rows(const float* src, int ld_src, void* dst, int ld_dst, int T, int W,
                            float scale, void* stream) {
  if (W % 8 != 0 || ld_src % 4 != 0) return -1;
  cast_rows_kernel<<<ring_grid(static_cast<size_t>(T) * (W / 8)), 256, 0, CB_ST(stream)>>>(
      src, ld_src, static_cast<__nv_bfloat16*>(dst), ld_dst, T, W, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
