// Decode-time attention over a paged KV cache, and the kernel that appends K/V to the pages.
//
// Cache layout: k_cache / v_cache are [num_pages, PAGE, nkv, dh] bf16 with PAGE = 64 tokens
// (nkv key/value heads; with grouped-query attention query head h reads head h / (nh / nkv), so
// the cache and the bytes streamed per step shrink by the group factor);
// page_table[b, i] is the physical page of logical page i of sequence b.  One query token per
// sequence attends to ctx_len[b] cached tokens.  The kernel is bandwidth bound (it streams the
// whole K and V of the sequence once): one CTA per (head, sequence), 16-byte loads, 8 (dh = 64)
// or 16 (dh = 128) lanes per token, online softmax per lane group, and one merge of the groups'
// (max, sum, acc) through shared memory at the end.  With `splits` > 1 the context is cut into
// ranges handled by different CTAs whose partial results are merged by a second tiny kernel.
// The reference has no KV cache (it recomputes the whole sequence per token,
// plugins/model-transformer/src/lib.rs:788-789); this is what `generate` runs on.
#include "common.cuh"
#include "ptx.cuh"

namespace cb {
int sm_count();

constexpr int KV_PAGE = 64;
constexpr int DEC_THREADS = 128;

template <int DH>
__global__ void __launch_bounds__(DEC_THREADS)
decode_attn_kernel(const __nv_bfloat16* __restrict__ q, int ldq,
                   const __nv_bfloat16* __restrict__ k_cache,
                   const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ page_table,
                   int max_pages, const int* __restrict__ ctx_len, __nv_bfloat16* __restrict__ out,
                   int ldo, float* __restrict__ part_o, float* __restrict__ part_ml, int nh,
                   int nkv, int splits, float scale_log2) {
  constexpr int LPT = DH / 8;                 // lanes per token
  constexpr int GROUPS = DEC_THREADS / LPT;   // token groups per CTA
  const int h = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int hk = h / (nh / nkv);              // the key/value head this query head reads
  const int g = threadIdx.x / LPT, part = threadIdx.x % LPT;
  const int n_ctx = ctx_len[b];
  const int per = (n_ctx + splits - 1) / splits;
  const int t0 = split * per, t1 = min(n_ctx, t0 + per);
  float qv[8];
  load8(q + static_cast<size_t>(b) * ldq + h * DH + part * 8, qv);
#pragma unroll
  for (int e = 0; e < 8; ++e) qv[e] *= scale_log2;
  float m = -INFINITY, l = 0.f, acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const int* pt = page_table + static_cast<size_t>(b) * max_pages;
  // U tokens per thread group and iteration: all their K and V loads are issued before any of
  // them is used (the kernel lives on bytes in flight), one running-max update per chunk.
  constexpr int U = 8;
  for (int tb = t0; tb < t1; tb += GROUPS * U) {  // same trip count for every lane of a warp
    uint4 kr[U], vr[U];
    bool act[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int t = tb + g + u * GROUPS;
      act[u] = t < t1;
      kr[u] = make_uint4(0u, 0u, 0u, 0u);
      vr[u] = kr[u];
      if (act[u]) {
        const int page = pt[t / KV_PAGE];
        const size_t off =
            ((static_cast<size_t>(page) * KV_PAGE + (t % KV_PAGE)) * nkv + hk) * DH + part * 8;
        kr[u] = __ldg(reinterpret_cast<const uint4*>(k_cache + off));
        vr[u] = __ldg(reinterpret_cast<const uint4*>(v_cache + off));
      }
    }
    float s[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const __nv_bfloat162* kh = reinterpret_cast<const __nv_bfloat162*>(&kr[u]);
      float d = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(kh[e]);
        d += qv[2 * e] * f.x + qv[2 * e + 1] * f.y;
      }
      s[u] = d;
    }
#pragma unroll
    for (int o = LPT / 2; o > 0; o >>= 1)
#pragma unroll
      for (int u = 0; u < U; ++u) s[u] += __shfl_xor_sync(0xffffffffu, s[u], o);
    float mx = -INFINITY;
#pragma unroll
    for (int u = 0; u < U; ++u) if (act[u]) mx = fmaxf(mx, s[u]);
    const float mn = fmaxf(m, mx);
    if (mn != -INFINITY) {
      const float c = fast_exp2(m - mn);     // m = -inf on the first chunk: c = 0
      l *= c;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] *= c;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (act[u]) {
          const float p = fast_exp2(s[u] - mn);
          l += p;
          const __nv_bfloat162* vh = reinterpret_cast<const __nv_bfloat162*>(&vr[u]);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(vh[e]);
            acc[2 * e] += p * f.x;
            acc[2 * e + 1] += p * f.y;
          }
        }
      }
      m = mn;
    }
  }
  __shared__ float s_m[GROUPS], s_l[GROUPS];
  __shared__ float s_acc[GROUPS][DH];
  if (part == 0) { s_m[g] = m; s_l[g] = l; }
#pragma unroll
  for (int e = 0; e < 8; ++e) s_acc[g][part * 8 + e] = acc[e];
  __syncthreads();
  if (threadIdx.x < DH) {
    const int d = threadIdx.x;
    float gm = -INFINITY;
    for (int i = 0; i < GROUPS; ++i) gm = fmaxf(gm, s_m[i]);
    float gl = 0.f, o = 0.f;
    for (int i = 0; i < GROUPS; ++i) {
      const float c = s_m[i] == -INFINITY ? 0.f : fast_exp2(s_m[i] - gm);
      gl += s_l[i] * c;
      o += s_acc[i][d] * c;
    }
    if (splits == 1) {
      out[static_cast<size_t>(b) * ldo + h * DH + d] = __float2bfloat16(gl > 0.f ? o / gl : 0.f);
    } else {
      const size_t idx = (static_cast<size_t>(b) * nh + h) * splits + split;
      part_o[idx * DH + d] = o;
      if (d == 0) { part_ml[idx * 2] = gm; part_ml[idx * 2 + 1] = gl; }
    }
  }
}

template <int DH>
__global__ void decode_merge_kernel(const float* __restrict__ part_o,
                                    const float* __restrict__ part_ml,
                                    __nv_bfloat16* __restrict__ out, int ldo, int nh, int splits) {
  const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const size_t base = (static_cast<size_t>(b) * nh + h) * splits;
  float gm = -INFINITY;
  for (int i = 0; i < splits; ++i) gm = fmaxf(gm, part_ml[(base + i) * 2]);
  float gl = 0.f, o = 0.f;
  for (int i = 0; i < splits; ++i) {
    const float mi = part_ml[(base + i) * 2];
    const float c = mi == -INFINITY ? 0.f : fast_exp2(mi - gm);
    gl += part_ml[(base + i) * 2 + 1] * c;
    o += part_o[(base + i) * DH + d] * c;
  }
  out[static_cast<size_t>(b) * ldo + h * DH + d] = __float2bfloat16(gl > 0.f ? o / gl : 0.f);
}

// Append: token t of sequence b = t / tokens_per_seq sits at position pos0[b] + t % tokens_per_seq.
__global__ void kv_write_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                int ldk, int ldv, __nv_bfloat16* __restrict__ k_cache,
                                __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ page_table,
                                int max_pages, const int* __restrict__ pos0, int T, int tokens_per_seq,
                                int nh, int dh, int* status) {
  const int row = nh * dh / 8;  // 16-byte vectors per token
  const size_t total = static_cast<size_t>(T) * row;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / row), vec = static_cast<int>(i % row);
    const int b = t / tokens_per_seq;
    const int pos = pos0[b] + t % tokens_per_seq;
    const int lp = pos / KV_PAGE;
    if (lp >= max_pages) {
      record_status(status, ST_BOUNDS, t);
      continue;
    }
    const int page = page_table[static_cast<size_t>(b) * max_pages + lp];
    const size_t dst = (static_cast<size_t>(page) * KV_PAGE + pos % KV_PAGE) * nh * dh + vec * 8;
    *reinterpret_cast<uint4*>(k_cache + dst) =
        *reinterpret_cast<const uint4*>(k + static_cast<size_t>(t) * ldk + vec * 8);
    *reinterpret_cast<uint4*>(v_cache + dst) =
        *reinterpret_cast<const uint4*>(v + static_cast<size_t>(t) * ldv + vec * 8);
  }
}

// argmax over the last dimension of bf16 logits [B, V] -> int64 ids
__global__ void argmax_kernel(const __nv_bfloat16* __restrict__ logits, int ld, int V,
                              int64_t* __restrict__ out) {
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  const int b = blockIdx.x;
  const __nv_bfloat16* row = logits + static_cast<size_t>(b) * ld;
  float best = -INFINITY;
  int bi = 0;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = __bfloat162float(row[i]);
    if (v > best) { best = v; bi = i; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { s_val[warp] = best; s_idx[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    best = lane < nw ? s_val[lane] : -INFINITY;
    bi = lane < nw ? s_idx[lane] : 0x7fffffff;
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) out[b] = bi;
  }
}

}  // namespace cb

using namespace cb;

// part_o: fp32 [B, nh, splits, dh] and part_ml: fp32 [B, nh, splits, 2] scratch, used when
// splits > 1.  nh query heads, nkv key/value heads in the cache (nkv divides nh).
extern "C" int cb_decode_attn(const void* q, int ldq, const void* k_cache, const void* v_cache,
                              const int* page_table, int max_pages, const int* ctx_len, void* out,
                              int ldo, float* part_o, float* part_ml, int B, int nh, int nkv,
                              int dh, int splits, float scale, void* stream) {
  if (dh != 64 && dh != 128) return -1;
  if (nkv < 1 || nh % nkv != 0) return -1;
  if (splits < 1) splits = 1;
  if (splits > 1 && (part_o == nullptr || part_ml == nullptr)) return -2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid(nh, B, splits);
  const float sl2 = scale * 1.4426950408889634f;
  auto Q = static_cast<const __nv_bfloat16*>(q);
  auto K = static_cast<const __nv_bfloat16*>(k_cache);
  auto V = static_cast<const __nv_bfloat16*>(v_cache);
  auto O = static_cast<__nv_bfloat16*>(out);
  if (dh == 64)
    decode_attn_kernel<64><<<grid, DEC_THREADS, 0, st>>>(Q, ldq, K, V, page_table, max_pages, ctx_len, O, ldo, part_o, part_ml, nh, nkv, splits, sl2);
  else
    decode_attn_kernel<128><<<grid, DEC_THREADS, 0, st>>>(Q, ldq, K, V, page_table, max_pages, ctx_len, O, ldo, part_o, part_ml, nh, nkv, splits, sl2);
  if (splits > 1) {
    dim3 g2(nh, B);
    if (dh == 64) decode_merge_kernel<64><<<g2, 64, 0, st>>>(part_o, part_ml, O, ldo, nh, splits);
    else decode_merge_kernel<128><<<g2, 128, 0, st>>>(part_o, part_ml, O, ldo, nh, splits);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int cb_kv_write(const void* k, const void* v, int ldk, int ldv, void* k_cache,
                           void* v_cache, const int* page_table, int max_pages, const int* pos0,
                           int T, int tokens_per_seq, int nh, int dh, int* status, void* stream) {
  if ((nh * dh) % 8 != 0 || T <= 0) return -1;
  const size_t work = static_cast<size_t>(T) * (nh * dh / 8);
  const int blocks = static_cast<int>(min(static_cast<size_t>(sm_count()) * 8, (work + 255) / 256));
  kv_write_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), ldk, ldv,
      static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), page_table,
      max_pages, pos0, T, tokens_per_seq, nh, dh, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int cb_argmax(const void* logits, int ld, int B, int V, int64_t* out, void* stream) {
  argmax_kernel<<<B, 1024, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(logits), ld, V, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
