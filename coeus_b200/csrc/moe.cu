// Mixture-of-experts routing and token permutation kernels.
//   router_topk   softmax over the expert logits, top-k experts per token, weights renormalised
//   router_slots  deterministic slot of every (token, k) inside its expert's capacity-bounded
//                 region: one block per expert walks the tokens in order with a block scan, so
//                 the assignment does not depend on scheduling (tokens beyond capacity are dropped)
//   gather_rows   expert-major send buffer: row (e * C + slot) <- x[token] (optionally scaled)
//   combine_rows  out[token] = resid[token] + sum_k w[token,k] * ret[e_k * C + slot_k]
//   pair_dot      d w[token,k] = <dy[token], ret[e_k * C + slot_k]>
// The all-to-all itself is not here: the expert GEMMs pull the send buffers of the other ranks
// and push their results back from inside the GEMM kernel (csrc/gemm.cu, COMM_AG / COMM_RS).
#include "common.cuh"
#include "ptx.cuh"

namespace cb {
int sm_count();

constexpr int MOE_MAX_E = 64;
constexpr int MOE_MAX_K = 4;

__global__ void router_topk_kernel(const float* __restrict__ logits, int T, int E, int K,
                                   int* __restrict__ expert, float* __restrict__ weight,
                                   float* __restrict__ probs) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  float p[MOE_MAX_E];
  float mx = -INFINITY;
  for (int e = 0; e < E; ++e) { p[e] = logits[static_cast<size_t>(t) * E + e]; mx = fmaxf(mx, p[e]); }
  float sum = 0.f;
  for (int e = 0; e < E; ++e) { p[e] = expf(p[e] - mx); sum += p[e]; }
  for (int e = 0; e < E; ++e) {
    p[e] /= sum;
    if (probs != nullptr) probs[static_cast<size_t>(t) * E + e] = p[e];
  }
  float wsum = 0.f;
  int chosen[MOE_MAX_K];
  float wv[MOE_MAX_K];
  for (int k = 0; k < K; ++k) {
    int best = -1;
    float bv = -1.f;
    for (int e = 0; e < E; ++e) {
      bool used = false;
      for (int j = 0; j < k; ++j) used = used || (chosen[j] == e);
      if (!used && p[e] > bv) { bv = p[e]; best = e; }   // ties: lowest expert index
    }
    chosen[k] = best;
    wv[k] = bv;
    wsum += bv;
  }
  for (int k = 0; k < K; ++k) {
    expert[static_cast<size_t>(t) * K + k] = chosen[k];
    weight[static_cast<size_t>(t) * K + k] = wv[k] / wsum;
  }
}

constexpr int SLOT_THREADS = 256;
__global__ void __launch_bounds__(SLOT_THREADS)
router_slots_kernel(const int* __restrict__ expert, int T, int K, int capacity,
                    int* __restrict__ slot, int* __restrict__ counts) {
  __shared__ int warp_tot[SLOT_THREADS / 32];
  __shared__ int base;
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) base = 0;
  __syncthreads();
  const int n = T * K;
  for (int i0 = 0; i0 < n; i0 += SLOT_THREADS) {
    const int i = i0 + threadIdx.x;
    const int mine = (i < n && expert[i] == e) ? 1 : 0;
    int incl = mine;
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    int before = 0;
    for (int w = 0; w < warp; ++w) before += warp_tot[w];
    const int pos = base + before + incl - mine;
    if (mine) slot[i] = pos < capacity ? pos : -1;
    __syncthreads();
    if (threadIdx.x == SLOT_THREADS - 1) base = pos + mine;
    __syncthreads();
  }
  if (threadIdx.x == 0) counts[e] = base < capacity ? base : capacity;
}

// dst[(expert * C + slot), :] = src[token, :] * (scale ? scale[token, k] : 1)
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ src, int ld_src,
                                   const int* __restrict__ expert, const int* __restrict__ slot,
                                   const float* __restrict__ scale, __nv_bfloat16* __restrict__ dst,
                                   int T, int K, int H, int capacity) {
  const int nv = H >> 3;
  const size_t total = static_cast<size_t>(T) * K * nv;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int vec = static_cast<int>(i % nv);
    const size_t pair = i / nv;
    const int s = slot[pair];
    if (s < 0) continue;
    const size_t t = pair / K;
    float v[8];
    load8(src + t * ld_src + vec * 8, v);
    if (scale != nullptr) {
      const float sc = scale[pair];
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] *= sc;
    }
    store8(dst + (static_cast<size_t>(expert[pair]) * capacity + s) * H + vec * 8, v);
  }
}

// out[t, :] = (resid ? resid[t, :] : 0) + sum_k (w ? w[t,k] : 1) * ret[(expert * C + slot), :]
__global__ void combine_rows_kernel(const __nv_bfloat16* __restrict__ ret,
                                    const int* __restrict__ expert, const int* __restrict__ slot,
                                    const float* __restrict__ w,
                                    const __nv_bfloat16* __restrict__ resid,
                                    __nv_bfloat16* __restrict__ out, int T, int K, int H,
                                    int capacity) {
  const int nv = H >> 3;
  const size_t total = static_cast<size_t>(T) * nv;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t t = i / nv;
    const int vec = static_cast<int>(i % nv);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (resid != nullptr) load8(resid + t * H + vec * 8, acc);
    for (int k = 0; k < K; ++k) {
      const size_t pair = t * K + k;
      const int s = slot[pair];
      if (s < 0) continue;
      float v[8];
      load8(ret + (static_cast<size_t>(expert[pair]) * capacity + s) * H + vec * 8, v);
      const float wk = w != nullptr ? w[pair] : 1.0f;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += wk * v[e];
    }
    store8(out + t * H + vec * 8, acc);
  }
}

// dots[t, k] = <a[t, :], ret[(expert * C + slot), :]>   (0 for dropped pairs); one warp per pair
__global__ void pair_dot_kernel(const __nv_bfloat16* __restrict__ a,
                                const __nv_bfloat16* __restrict__ ret,
                                const int* __restrict__ expert, const int* __restrict__ slot,
                                float* __restrict__ dots, int T, int K, int H, int capacity) {
  const int lane = threadIdx.x & 31;
  const size_t warp_id = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) >> 5;
  const size_t n_warps = (static_cast<size_t>(gridDim.x) * blockDim.x) >> 5;
  const size_t total = static_cast<size_t>(T) * K;
  for (size_t pair = warp_id; pair < total; pair += n_warps) {
    const int s = slot[pair];
    float acc = 0.f;
    if (s >= 0) {
      const size_t t = pair / K;
      const __nv_bfloat16* r = ret + (static_cast<size_t>(expert[pair]) * capacity + s) * H;
      for (int vec = lane; vec < (H >> 3); vec += 32) {
        float x[8], y[8];
        load8(a + t * H + vec * 8, x);
        load8(r + vec * 8, y);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc += x[e] * y[e];
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) dots[pair] = acc;
  }
}

}  // namespace cb

using namespace cb;
#define CB_ST(s) static_cast<cudaStream_t>(s)

extern "C" int cb_moe_route(const float* logits, int T, int E, int K, int capacity, int* expert,
                            float* weight, float* probs, int* slot, int* counts, void* stream) {
  if (E > MOE_MAX_E || K > MOE_MAX_K || K > E || T <= 0) return -1;
  router_topk_kernel<<<(T + 127) / 128, 128, 0, CB_ST(stream)>>>(logits, T, E, K, expert, weight, probs);
  router_slots_kernel<<<E, SLOT_THREADS, 0, CB_ST(stream)>>>(expert, T, K, capacity, slot, counts);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

static inline int moe_grid(size_t work) {
  const size_t b = (work + 255) / 256, cap = static_cast<size_t>(sm_count()) * 8;
  return static_cast<int>(b < cap ? (b ? b : 1) : cap);
}

extern "C" int cb_moe_gather_rows(const void* src, int ld_src, const int* expert, const int* slot,
                                  const float* scale, void* dst, int T, int K, int H,
                                  int capacity, void* stream) {
  if (H % 8 != 0) return -1;
  gather_rows_kernel<<<moe_grid(static_cast<size_t>(T) * K * (H / 8)), 256, 0, CB_ST(stream)>>>(
      static_cast<const __nv_bfloat16*>(src), ld_src, expert, slot, scale,
      static_cast<__nv_bfloat16*>(dst), T, K, H, capacity);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int cb_moe_combine_rows(const void* ret, const int* expert, const int* slot,
                                   const float* w, const void* resid, void* out, int T, int K,
                                   int H, int capacity, void* stream) {
  if (H % 8 != 0) return -1;
  combine_rows_kernel<<<moe_grid(static_cast<size_t>(T) * (H / 8)), 256, 0, CB_ST(stream)>>>(
      static_cast<const __nv_bfloat16*>(ret), expert, slot, w,
      static_cast<const __nv_bfloat16*>(resid), static_cast<__nv_bfloat16*>(out), T, K, H, capacity);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int cb_moe_pair_dot(const void* a, const void* ret, const int* expert, const int* slot,
                               float* dots, int T, int K, int H, int capacity, void* stream) {
  if (H % 8 != 0) return -1;
  pair_dot_kernel<<<moe_grid(static_cast<size_t>(T) * K * 32), 256, 0, CB_ST(stream)>>>(
      static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(ret), expert, slot,
      dots, T, K, H, capacity);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
