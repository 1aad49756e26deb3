// Memory-bound kernels of the model and the optimizer: embedding (+ positional encoding)
// forward/backward, fused softmax-cross-entropy forward+backward, AdamW, GELU / SwiGLU,
// row softmax, RoPE, column sums (bias gradients), parameter init and casts.
// All of them move 16 bytes per thread per access and keep statistics in fp32.
#include "common.cuh"
#include "ptx.cuh"

namespace cb {
int sm_count();

// ------------------------------------------------------------------------------ embedding
// out[t,:] = E[ids[t],:] + PE[t % S,:]   (reference: plugins/model-transformer/src/lib.rs:815-835)
// A token id outside [0,V) records ST_BOUNDS in the status word and yields a zero row; the
// reference raises invalid_input for the same condition.
__global__ void embed_fwd_kernel(const int64_t* __restrict__ ids,
                                 const __nv_bfloat16* __restrict__ E,
                                 const float* __restrict__ pe, __nv_bfloat16* __restrict__ out,
                                 int T, int H, int V, int S, int pos_offset, int* status) {
  const int nv = H >> 3;
  const size_t total = static_cast<size_t>(T) * nv;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / nv), vec = static_cast<int>(i % nv);
    const int64_t id = ids[t];
    float v[8];
    if (id < 0 || id >= V) {
      record_status(status, ST_BOUNDS, t);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = 0.f;
    } else {
      load8(E + static_cast<size_t>(id) * H + vec * 8, v);
    }
    if (pe != nullptr) {
      const int p = (t % S) + pos_offset;
      const float4 a = *reinterpret_cast<const float4*>(pe + static_cast<size_t>(p) * H + vec * 8);
      const float4 b =
          *reinterpret_cast<const float4*>(pe + static_cast<size_t>(p) * H + vec * 8 + 4);
      v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w;
      v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
    }
    store8(out + static_cast<size_t>(t) * H + vec * 8, v);
  }
}

// dE[ids[t],:] += dy[t,:]   (fp32 atomics)
__global__ void embed_bwd_kernel(const int64_t* __restrict__ ids,
                                 const __nv_bfloat16* __restrict__ dy, float* __restrict__ dE,
                                 int T, int H, int V) {
  const int nv = H >> 3;
  const size_t total = static_cast<size_t>(T) * nv;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / nv), vec = static_cast<int>(i % nv);
    const int64_t id = ids[t];
    if (id < 0 || id >= V) continue;
    float v[8];
    load8(dy + static_cast<size_t>(t) * H + vec * 8, v);
    float* dst = dE + static_cast<size_t>(id) * H + vec * 8;
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(v[0]),
                 "f"(v[1]), "f"(v[2]), "f"(v[3]) : "memory");
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 4), "f"(v[4]),
                 "f"(v[5]), "f"(v[6]), "f"(v[7]) : "memory");
  }
}

// PE[p,2i] = sin(p / 10000^(2i/H)), PE[p,2i+1] = cos(same)   (lib.rs:398-414)
__global__ void sinusoid_pe_kernel(float* __restrict__ pe, int S, int H) {
  const size_t total = static_cast<size_t>(S) * (H / 2);
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int p = static_cast<int>(i / (H / 2)), k = static_cast<int>(i % (H / 2));
    const float div = powf(10000.0f, static_cast<float>(2 * k) / static_cast<float>(H));
    const float a = static_cast<float>(p) / div;
    pe[static_cast<size_t>(p) * H + 2 * k] = sinf(a);
    pe[static_cast<size_t>(p) * H + 2 * k + 1] = cosf(a);
  }
}

// ------------------------------------------------------------------------------ cross-entropy
// One block per row of logits[T, V] (bf16, row pitch ld).  Pass 1: online max / sum-exp.
// Pass 2 (the row is L2-resident by then): dlogits = (softmax - onehot) * grad_scale written in
// place of the logits.  loss[t] = lse - logit[target]; target < 0 (ignore) gives loss 0, d = 0.
// With vocab-parallel shards (vocab_start, partial stats) the fwd/bwd halves are split:
//   mode 0: fused fwd+bwd;  mode 1: stats only (max, sumexp, target logit);  mode 2: bwd from lse.
constexpr int CE_THREADS = 512;
__global__ void __launch_bounds__(CE_THREADS, 4)
ce_kernel(__nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ targets,
          float* __restrict__ loss, float* __restrict__ stats, const float* __restrict__ lse_in,
          int T, int V, int ld, int vocab_start, float grad_scale, int mode) {
  __shared__ float red[32];
  const int nv = (V + 7) >> 3;  // the row buffer is padded to a multiple of 8 columns
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    __nv_bfloat16* row = logits + static_cast<size_t>(t) * ld;
    const int64_t tgt = targets[t];
    const int local_tgt = (tgt >= vocab_start && tgt < vocab_start + V)
                              ? static_cast<int>(tgt - vocab_start) : -1;
    // exponentials run as ex2(v * log2(e) - c * log2(e)): one FMA and one special-function op
    constexpr float L2E = 1.4426950408889634f;
    float lse;
    if (mode != 2) {
      float m = -INFINITY, s = 0.f;
      for (int vec = threadIdx.x; vec < nv; vec += CE_THREADS) {
        float v[8];
        load8(row + vec * 8, v);
        if (vec * 8 + 8 > V) {
#pragma unroll
          for (int e = 0; e < 8; ++e)
            if (vec * 8 + e >= V) v[e] = -INFINITY;
        }
        const float lm = fmaxf(max3(v[0], v[1], v[2]), fmaxf(max3(v[3], v[4], v[5]),
                                                              fmaxf(v[6], v[7])));
        const float nm = fmaxf(m, lm);
        const float nb = -nm * L2E;
        float add0 = 0.f, add1 = 0.f;
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          add0 += fast_exp2(fmaf(v[e], L2E, nb));
          add1 += fast_exp2(fmaf(v[e + 1], L2E, nb));
        }
        s = s * fast_exp2((m - nm) * L2E) + (add0 + add1);
        m = nm;
      }
      const float gm = block_max(m, red);
      s = (m == -INFINITY) ? 0.f : s * fast_exp2((m - gm) * L2E);
      const float gs = block_sum(s, red);
      lse = gm + __logf(gs);
      const float tl = local_tgt >= 0 ? __bfloat162float(row[local_tgt]) : 0.f;
      if (threadIdx.x == 0) {
        if (mode == 1) {
          stats[3 * t + 0] = gm;
          stats[3 * t + 1] = gs;
          stats[3 * t + 2] = tl;
        } else {
          loss[t] = tgt < 0 ? 0.f : (lse - tl);
        }
      }
      if (mode == 1) continue;
    } else {
      lse = lse_in[t];
    }
    // d logit = (softmax - onehot) * scale; exp(v - lse) * scale = ex2(v * log2(e) + c) with the
    // scale folded into the exponent would lose the exact zero of an ignored token, so the
    // product stays a separate multiply
    const float scale = tgt < 0 ? 0.f : grad_scale;
    const float nl = -lse * L2E;
    const int tvec = local_tgt >> 3;          // -1 when the target lies in another shard
    for (int vec = threadIdx.x; vec < nv; vec += CE_THREADS) {
      float v[8];
      load8(row + vec * 8, v);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = fast_exp2(fmaf(v[e], L2E, nl)) * scale;
      if (vec == tvec) {                       // one vector per row
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if (e == (local_tgt & 7)) v[e] -= scale;
      }
      if (vec * 8 + 8 > V) {                   // padding columns of the last vector
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if (vec * 8 + e >= V) v[e] = 0.f;
      }
      store8(row + vec * 8, v);
    }
  }
}

// ------------------------------------------------------------------------------ AdamW
// Decoupled weight decay AdamW on an fp32 master copy; writes the bf16 working copy.
// grad is fp32 (the accumulation buffer of the weight-gradient GEMMs) and is scaled by
// grad_scale (1/world, 1/accumulation steps, clip coefficient).  wd_mask selects per element
// range is handled by the caller launching per parameter group.
__global__ void adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                             const float* __restrict__ g, __nv_bfloat16* __restrict__ p_bf16,
                             size_t n, float lr, float beta1, float beta2, float eps, float wd,
                             float bc1, float bc2, float grad_scale,
                             const float* __restrict__ clip_coef) {
  const float gs = grad_scale * (clip_coef != nullptr ? *clip_coef : 1.0f);
  const size_t nv = n >> 2;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float4 P = reinterpret_cast<float4*>(p)[i];
    float4 M = reinterpret_cast<float4*>(m)[i];
    float4 Vv = reinterpret_cast<float4*>(v)[i];
    const float4 G = reinterpret_cast<const float4*>(g)[i];
    float pp[4] = {P.x, P.y, P.z, P.w}, mm[4] = {M.x, M.y, M.z, M.w},
          vv[4] = {Vv.x, Vv.y, Vv.z, Vv.w};
    const float gg[4] = {G.x * gs, G.y * gs, G.z * gs, G.w * gs};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      mm[e] = beta1 * mm[e] + (1.f - beta1) * gg[e];
      vv[e] = beta2 * vv[e] + (1.f - beta2) * gg[e] * gg[e];
      const float mh = mm[e] / bc1, vh = vv[e] / bc2;
      pp[e] = pp[e] * (1.f - lr * wd) - lr * mh / (sqrtf(vh) + eps);
    }
    reinterpret_cast<float4*>(p)[i] = make_float4(pp[0], pp[1], pp[2], pp[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (p_bf16 != nullptr) {
      uint2 o;
      o.x = pack_bf16x2(pp[0], pp[1]);
      o.y = pack_bf16x2(pp[2], pp[3]);
      reinterpret_cast<uint2*>(p_bf16)[i] = o;
    }
  }
  // tail (n not a multiple of 4)
  for (size_t i = (nv << 2) + blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const float gi = g[i] * gs;
    const float mi = beta1 * m[i] + (1.f - beta1) * gi;
    const float vi = beta2 * v[i] + (1.f - beta2) * gi * gi;
    const float pi = p[i] * (1.f - lr * wd) - lr * (mi / bc1) / (sqrtf(vi / bc2) + eps);
    m[i] = mi; v[i] = vi; p[i] = pi;
    if (p_bf16 != nullptr) p_bf16[i] = __float2bfloat16(pi);
  }
}

// *out += scale * sum(g) (square == 0) or scale * sum(g*g) (square == 1) of an fp32 buffer:
// the mean loss and the global gradient norm.
__global__ void sumsq_kernel(const float* __restrict__ g, size_t n, float* __restrict__ out,
                             int square, float scale) {
  __shared__ float red[32];
  float s = 0.f;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x)
    s += square ? g[i] * g[i] : g[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) atomicAdd(out, s * scale);
}
// coef = min(1, max_norm / (sqrt(sumsq * scale^2) + 1e-6))
__global__ void clip_coef_kernel(const float* sumsq, float scale, float max_norm, float* coef,
                                 float* norm_out) {
  const float norm = sqrtf(*sumsq) * scale;
  if (norm_out != nullptr) *norm_out = norm;
  *coef = fminf(1.0f, max_norm / (norm + 1e-6f));
}

// ------------------------------------------------------------------------------ activations
__global__ void gelu_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                size_t n8) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float v[8];
    load8(x + i * 8, v);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = gelu_tanh(v[e]);
    store8(y + i * 8, v);
  }
}
__global__ void gelu_bwd_kernel(const __nv_bfloat16* __restrict__ x,
                                const __nv_bfloat16* __restrict__ dy,
                                __nv_bfloat16* __restrict__ dx, size_t n8) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float v[8], d[8];
    load8(x + i * 8, v);
    load8(dy + i * 8, d);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = d[e] * gelu_tanh_grad(v[e]);
    store8(dx + i * 8, v);
  }
}
// gu is [T, 2I] with the gate in columns [0,I) and up in [I,2I); y[T,I] = silu(gate) * up
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ y, int T, int I) {
  const int nv = I >> 3;
  const size_t total = static_cast<size_t>(T) * nv;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t t = i / nv;
    const int vec = static_cast<int>(i % nv);
    float g[8], u[8];
    load8(gu + t * 2 * I + vec * 8, g);
    load8(gu + t * 2 * I + I + vec * 8, u);
#pragma unroll
    for (int e = 0; e < 8; ++e) g[e] = silu(g[e]) * u[e];
    store8(y + t * I + vec * 8, g);
  }
}
// dgu[T,2I] from dy[T,I]
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu,
                                  const __nv_bfloat16* __restrict__ dy,
                                  __nv_bfloat16* __restrict__ dgu, int T, int I) {
  const int nv = I >> 3;
  const size_t total = static_cast<size_t>(T) * nv;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t t = i / nv;
    const int vec = static_cast<int>(i % nv);
    float g[8], u[8], d[8], dg[8], du[8];
    load8(gu + t * 2 * I + vec * 8, g);
    load8(gu + t * 2 * I + I + vec * 8, u);
    load8(dy + t * I + vec * 8, d);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float sg = 1.0f / (1.0f + __expf(-g[e]));
      const float sl = g[e] * sg;
      du[e] = d[e] * sl;
      dg[e] = d[e] * u[e] * (sg + sl * (1.0f - sg));
    }
    store8(dgu + t * 2 * I + vec * 8, dg);
    store8(dgu + t * 2 * I + I + vec * 8, du);
  }
}

// ------------------------------------------------------------------------------ softmax
// Row softmax, fp32 in/out (API parity with math::softmax, lib.rs:80-88; router probabilities).
__global__ void softmax_rows_kernel(const float* __restrict__ x, float* __restrict__ y, int R,
                                    int C) {
  __shared__ float red[32];
  for (int r = blockIdx.x; r < R; r += gridDim.x) {
    const float* xr = x + static_cast<size_t>(r) * C;
    float* yr = y + static_cast<size_t>(r) * C;
    float m = -INFINITY;
    for (int c = threadIdx.x; c < C; c += blockDim.x) m = fmaxf(m, xr[c]);
    m = block_max(m, red);
    float s = 0.f;
    for (int c = threadIdx.x; c < C; c += blockDim.x) s += expf(xr[c] - m);
    s = block_sum(s, red);
    for (int c = threadIdx.x; c < C; c += blockDim.x) yr[c] = expf(xr[c] - m) / s;
  }
}

// ------------------------------------------------------------------------------ RoPE
// In-place rotary embedding on x[T, nheads, dh] (row pitch ld elements between tokens), the
// half-split convention: (x[i], x[i+dh/2]) rotated by pos * theta^(-2i/dh).  inverse = 1
// applies the transposed rotation (the backward pass).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, int T, int nheads, int dh, int ld,
                            int S, int pos_offset, const int* __restrict__ pos_dev, float theta,
                            int inverse) {
  // pos_dev (optional): first position of every sequence, read on the device so that a captured
  // graph can be replayed while the positions advance
  const int half = dh >> 1;
  const size_t total = static_cast<size_t>(T) * nheads * half;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int k = static_cast<int>(i % half);
    const int h = static_cast<int>((i / half) % nheads);
    const size_t t = i / (static_cast<size_t>(half) * nheads);
    const int pos = static_cast<int>(t % S) + (pos_dev != nullptr ? pos_dev[t / S] : pos_offset);
    const float inv_freq = __powf(theta, -2.0f * k / dh);
    float sn, cs;
    sincosf(pos * inv_freq, &sn, &cs);
    if (inverse) sn = -sn;
    __nv_bfloat16* p = x + t * ld + static_cast<size_t>(h) * dh;
    const float a = __bfloat162float(p[k]), b = __bfloat162float(p[k + half]);
    p[k] = __float2bfloat16(a * cs - b * sn);
    p[k + half] = __float2bfloat16(a * sn + b * cs);
  }
}

// Same rotation with the trigonometry hoisted out of the head loop: one thread owns eight
// adjacent frequencies of one token, computes their sines and cosines once and applies them to
// every head with 16-byte loads and stores (the head count no longer multiplies the sincos work,
// which made the element-per-thread kernel compute-bound).  Needs dh % 16 == 0 and ld % 8 == 0.
__global__ void rope_vec_kernel(__nv_bfloat16* __restrict__ x, int T, int nheads, int dh, int ld,
                                int S, int pos_offset, const int* __restrict__ pos_dev,
                                float theta, int inverse) {
  const int half = dh >> 1;
  const int vecs = half >> 3;
  const float l2t = __log2f(theta);
  const size_t total = static_cast<size_t>(T) * vecs;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(i % vecs);
    const size_t t = i / vecs;
    const int pos = static_cast<int>(t % S) + (pos_dev != nullptr ? pos_dev[t / S] : pos_offset);
    float sn[8], cs[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float inv_freq = exp2f(-2.0f * (v * 8 + e) / dh * l2t);
      sincosf(pos * inv_freq, &sn[e], &cs[e]);
      if (inverse) sn[e] = -sn[e];
    }
    __nv_bfloat16* p = x + t * ld + v * 8;
    for (int h = 0; h < nheads; ++h, p += dh) {
      float a[8], b[8], oa[8], ob[8];
      load8(p, a);
      load8(p + half, b);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        oa[e] = a[e] * cs[e] - b[e] * sn[e];
        ob[e] = a[e] * sn[e] + b[e] * cs[e];
      }
      store8(p, oa);
      store8(p + half, ob);
    }
  }
}

// ------------------------------------------------------------------------------ column sums
// out[c] += sum_t x[t, c]   (x bf16 [T, C] with pitch ld; out fp32) — bias gradients.
constexpr int COLSUM_THREADS = 256;
__global__ void __launch_bounds__(COLSUM_THREADS)
colsum_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out, int T, int C, int ld,
              int rows_per_block) {
  // blockIdx.x: group of 32*8 = 256 columns; blockIdx.y: row chunk.  8 warps split the rows.
  __shared__ float red[8][256];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.x * 256 + lane * 8;
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(T, r0 + rows_per_block);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (col < C) {
    // four rows per warp and trip: four 16-byte loads in flight per thread
    for (int r = r0 + warp; r < r1; r += 32) {
      bf16x8 xv[4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (r + 8 * k < r1)
          xv[k] = *reinterpret_cast<const bf16x8*>(x + static_cast<size_t>(r + 8 * k) * ld + col);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (r + 8 * k < r1) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 q = __bfloat1622float2(xv[k].v[e]);
            acc[2 * e] += q.x;
            acc[2 * e + 1] += q.y;
          }
        }
      }
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) red[warp][lane * 8 + e] = acc[e];
  __syncthreads();
  const int c = threadIdx.x;
  float s = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) s += red[w][c];
  if (blockIdx.x * 256 + c < C) atomicAdd(out + blockIdx.x * 256 + c, s);
}

// dx = dy * gelu'(x) and out[c] += sum_t dx[t, c] (the bf16 values that are stored) in one pass:
// the bias gradient of the layer that produced x needs no second read of dx.  x, dy, dx are
// [T, C] contiguous.  A block covers 2048 adjacent columns of one row at a time (4 KB per
// operand, in address order across the block) and strides over the rows, four rows per trip;
// each thread keeps the sums of its eight columns and adds them to `out` at the end.
__global__ void __launch_bounds__(COLSUM_THREADS)
gelu_bwd_colsum_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                       __nv_bfloat16* __restrict__ dx, float* __restrict__ out, int T, int C) {
  const int col = (blockIdx.x * COLSUM_THREADS + threadIdx.x) * 8;
  if (col >= C) return;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const int stride = gridDim.y;
  for (int r = blockIdx.y; r < T; r += 4 * stride) {
    bf16x8 xv[4], dv[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int rr = r + k * stride;
      if (rr < T) {
        const size_t off = static_cast<size_t>(rr) * C + col;
        xv[k] = *reinterpret_cast<const bf16x8*>(x + off);
        dv[k] = *reinterpret_cast<const bf16x8*>(dy + off);
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int rr = r + k * stride;
      if (rr < T) {
        bf16x8 o;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 a = __bfloat1622float2(xv[k].v[e]);
          const float2 b = __bfloat1622float2(dv[k].v[e]);
          o.v[e] = __floats2bfloat162_rn(b.x * gelu_tanh_grad(a.x), b.y * gelu_tanh_grad(a.y));
          const float2 q = __bfloat1622float2(o.v[e]);
          acc[2 * e] += q.x;
          acc[2 * e + 1] += q.y;
        }
        *reinterpret_cast<bf16x8*>(dx + static_cast<size_t>(rr) * C + col) = o;
      }
    }
  }
#pragma unroll
  for (int e = 0; e < 8; e += 4)
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                 ::"l"(out + col + e), "f"(acc[e]), "f"(acc[e + 1]), "f"(acc[e + 2]), "f"(acc[e + 3])
                 : "memory");
}

// ------------------------------------------------------------------------------ init / casts
// p[i] = clamp(sin(float(i) * 0.1234567) * sqrt(2/H), -0.1, 0.1)   (lib.rs:604-611); the index
// is converted to fp32 first, exactly like the reference's `i as f32`.
__global__ void sin_init_kernel(float* __restrict__ p, size_t n, size_t index_offset,
                                float scale) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const float fi = static_cast<float>(i + index_offset);
    const float v = sinf(fi * 0.1234567f) * scale;
    p[i] = fminf(0.1f, fmaxf(-0.1f, v));
  }
}
// Counter-based normal init: Philox4x32-10 keyed by the seed, counter = group index; each group
// of four consecutive elements takes the four outputs of one block through two Box-Muller pairs.
// The value of element i depends on (seed, i + index_offset) only, so any shard of a tensor can
// be drawn by itself.
__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
  const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
  const uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
  c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
}
__device__ __forceinline__ float u01(uint32_t x) {   // (0, 1), exact in fp32
  return static_cast<float>(x >> 8) * 5.9604644775390625e-8f + 2.98023223876953125e-8f;
}
__global__ void normal_init_kernel(float* __restrict__ p, size_t n, size_t index_offset,
                                   uint32_t seed_lo, uint32_t seed_hi, float mean, float std) {
  const size_t g_first = index_offset / 4, g_last = (index_offset + n + 3) / 4;
  for (size_t g = g_first + blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
       g < g_last; g += static_cast<size_t>(gridDim.x) * blockDim.x) {
    uint32_t c[4] = {static_cast<uint32_t>(g), static_cast<uint32_t>(g >> 32), 0u, 0u};
    uint32_t k0 = seed_lo, k1 = seed_hi;
#pragma unroll
    for (int r = 0; r < 10; ++r) {
      philox_round(c, k0, k1);
      k0 += 0x9E3779B9u;
      k1 += 0xBB67AE85u;
    }
    float z[4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float r = sqrtf(-2.0f * logf(u01(c[2 * h])));
      float sn, cs;
      sincosf(6.283185307179586f * u01(c[2 * h + 1]), &sn, &cs);
      z[2 * h] = r * cs;
      z[2 * h + 1] = r * sn;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const size_t i = g * 4 + j;
      if (i >= index_offset && i < index_offset + n) p[i - index_offset] = mean + std * z[j];
    }
  }
}
__global__ void f32_to_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                   size_t n) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x)
    y[i] = __float2bfloat16(x[i]);
}

static inline int grid_for(size_t work_items, int threads) {
  const size_t blocks = (work_items + threads - 1) / threads;
  const size_t cap = static_cast<size_t>(sm_count()) * 16;
  return static_cast<int>(blocks < cap ? (blocks == 0 ? 1 : blocks) : cap);
}

}  // namespace cb

using namespace cb;
#define CB_ST(s) static_cast<cudaStream_t>(s)
#define CB_RET() return cudaGetLastError() == cudaSuccess ? 0 : -2

extern "C" int cb_embed_fwd(const int64_t* ids, const void* E, const float* pe, void* out, int T,
                            int H, int V, int S, int pos_offset, int* status, void* stream) {
  if (H % 8 != 0 || T <= 0) return -1;
  embed_fwd_kernel<<<grid_for(static_cast<size_t>(T) * (H / 8), 256), 256, 0, CB_ST(stream)>>>(
      ids, static_cast<const __nv_bfloat16*>(E), pe, static_cast<__nv_bfloat16*>(out), T, H, V, S,
      pos_offset, status);
  CB_RET();
}
extern "C" int cb_embed_bwd(const int64_t* ids, const void* dy, float* dE, int T, int H, int V,
                            void* stream) {
  if (H % 8 != 0 || T <= 0) return -1;
  embed_bwd_kernel<<<grid_for(static_cast<size_t>(T) * (H / 8), 256), 256, 0, CB_ST(stream)>>>(
      ids, static_cast<const __nv_bfloat16*>(dy), dE, T, H, V);
  CB_RET();
}
extern "C" int cb_sinusoid_pe(float* pe, int S, int H, void* stream) {
  if (H % 2 != 0) return -1;
  sinusoid_pe_kernel<<<grid_for(static_cast<size_t>(S) * (H / 2), 256), 256, 0, CB_ST(stream)>>>(
      pe, S, H);
  CB_RET();
}
extern "C" int cb_cross_entropy(void* logits, const int64_t* targets, float* loss, float* stats,
                                const float* lse_in, int T, int V, int ld, int vocab_start,
                                float grad_scale, int mode, void* stream) {
  if (ld % 8 != 0 || ld < ((V + 7) / 8) * 8 || T <= 0) return -1;
  const int blocks = min(T, sm_count() * 4);
  ce_kernel<<<blocks, CE_THREADS, 0, CB_ST(stream)>>>(static_cast<__nv_bfloat16*>(logits),
                                                     targets, loss, stats, lse_in, T, V, ld,
                                                     vocab_start, grad_scale, mode);
  CB_RET();
}
extern "C" int cb_adamw(float* p, float* m, float* v, const float* g, void* p_bf16, size_t n,
                        float lr, float beta1, float beta2, float eps, float wd, int step,
                        float grad_scale, const float* clip_coef, void* stream) {
  if (n == 0) return 0;
  const float bc1 = 1.0f - powf(beta1, static_cast<float>(step));
  const float bc2 = 1.0f - powf(beta2, static_cast<float>(step));
  adamw_kernel<<<grid_for(n / 4 + 1, 256), 256, 0, CB_ST(stream)>>>(
      p, m, v, g, static_cast<__nv_bfloat16*>(p_bf16), n, lr, beta1, beta2, eps, wd, bc1, bc2,
      grad_scale, clip_coef);
  CB_RET();
}
extern "C" int cb_sumsq(const float* g, size_t n, float* out, void* stream) {
  if (n == 0) return 0;
  sumsq_kernel<<<grid_for(n, 1024) > 1184 ? 1184 : grid_for(n, 1024), 1024, 0, CB_ST(stream)>>>(
      g, n, out, 1, 1.0f);
  CB_RET();
}
extern "C" int cb_sum_scaled(const float* g, size_t n, float* out, float scale, void* stream) {
  if (n == 0) return 0;
  sumsq_kernel<<<grid_for(n, 1024) > 1184 ? 1184 : grid_for(n, 1024), 1024, 0, CB_ST(stream)>>>(
      g, n, out, 0, scale);
  CB_RET();
}
extern "C" int cb_clip_coef(const float* sumsq, float scale, float max_norm, float* coef,
                            float* norm_out, void* stream) {
  clip_coef_kernel<<<1, 1, 0, CB_ST(stream)>>>(sumsq, scale, max_norm, coef, norm_out);
  CB_RET();
}
extern "C" int cb_gelu_fwd(const void* x, void* y, size_t n, void* stream) {
  if (n % 8 != 0) return -1;
  gelu_fwd_kernel<<<grid_for(n / 8, 256), 256, 0, CB_ST(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), n / 8);
  CB_RET();
}
extern "C" int cb_gelu_bwd(const void* x, const void* dy, void* dx, size_t n, void* stream) {
  if (n % 8 != 0) return -1;
  gelu_bwd_kernel<<<grid_for(n / 8, 256), 256, 0, CB_ST(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy),
      static_cast<__nv_bfloat16*>(dx), n / 8);
  CB_RET();
}
extern "C" int cb_swiglu_fwd(const void* gu, void* y, int T, int I, void* stream) {
  if (I % 8 != 0) return -1;
  swiglu_fwd_kernel<<<grid_for(static_cast<size_t>(T) * (I / 8), 256), 256, 0, CB_ST(stream)>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(y), T, I);
  CB_RET();
}
extern "C" int cb_swiglu_bwd(const void* gu, const void* dy, void* dgu, int T, int I,
                             void* stream) {
  if (I % 8 != 0) return -1;
  swiglu_bwd_kernel<<<grid_for(static_cast<size_t>(T) * (I / 8), 256), 256, 0, CB_ST(stream)>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<const __nv_bfloat16*>(dy),
      static_cast<__nv_bfloat16*>(dgu), T, I);
  CB_RET();
}
extern "C" int cb_softmax_rows(const float* x, float* y, int R, int C, void* stream) {
  const int threads = C >= 1024 ? 256 : (C >= 128 ? 128 : 32);
  softmax_rows_kernel<<<min(R, sm_count() * 8), threads, 0, CB_ST(stream)>>>(x, y, R, C);
  CB_RET();
}
extern "C" int cb_rope(void* x, int T, int nheads, int dh, int ld, int S, int pos_offset,
                       float theta, int inverse, void* stream) {
  if (dh % 2 != 0) return -1;
  if (dh % 16 == 0 && ld % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0) {
    rope_vec_kernel<<<grid_for(static_cast<size_t>(T) * (dh / 16), 128), 128, 0, CB_ST(stream)>>>(
        static_cast<__nv_bfloat16*>(x), T, nheads, dh, ld, S, pos_offset, nullptr, theta, inverse);
    CB_RET();
  }
  rope_kernel<<<grid_for(static_cast<size_t>(T) * nheads * (dh / 2), 256), 256, 0,
                CB_ST(stream)>>>(static_cast<__nv_bfloat16*>(x), T, nheads, dh, ld, S,
                                 pos_offset, nullptr, theta, inverse);
  CB_RET();
}
extern "C" int cb_rope_dev(void* x, int T, int nheads, int dh, int ld, int S, const int* pos_dev,
                           float theta, int inverse, void* stream) {
  if (dh % 2 != 0 || pos_dev == nullptr) return -1;
  if (dh % 16 == 0 && ld % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0) {
    rope_vec_kernel<<<grid_for(static_cast<size_t>(T) * (dh / 16), 128), 128, 0, CB_ST(stream)>>>(
        static_cast<__nv_bfloat16*>(x), T, nheads, dh, ld, S, 0, pos_dev, theta, inverse);
    CB_RET();
  }
  rope_kernel<<<grid_for(static_cast<size_t>(T) * nheads * (dh / 2), 256), 256, 0,
                CB_ST(stream)>>>(static_cast<__nv_bfloat16*>(x), T, nheads, dh, ld, S, 0, pos_dev,
                                 theta, inverse);
  CB_RET();
}
extern "C" int cb_gelu_bwd_colsum(const void* x, const void* dy, void* dx, float* out, int T, int C,
                                  void* stream) {
  if (C % 8 != 0 || T <= 0) return -1;
  const int col_groups = (C / 8 + COLSUM_THREADS - 1) / COLSUM_THREADS;
  // two blocks per SM: enough loads in flight for the memory system, and few enough blocks that
  // their atomic adds on the same `out` entries (one per block and column) do not queue up
  int row_blocks = (sm_count() * 2 + col_groups - 1) / col_groups;
  if (row_blocks > T) row_blocks = T;
  dim3 grid(col_groups, row_blocks);
  gelu_bwd_colsum_kernel<<<grid, COLSUM_THREADS, 0, CB_ST(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy),
      static_cast<__nv_bfloat16*>(dx), out, T, C);
  CB_RET();
}
extern "C" int cb_colsum(const void* x, float* out, int T, int C, int ld, void* stream) {
  if (C % 8 != 0 || ld % 8 != 0) return -1;
  const int col_groups = (C + 255) / 256;
  int row_chunks = (sm_count() * 4 + col_groups - 1) / col_groups;
  if (row_chunks > (T + 63) / 64) row_chunks = (T + 63) / 64;
  if (row_chunks < 1) row_chunks = 1;
  const int rpb = (T + row_chunks - 1) / row_chunks;
  dim3 grid(col_groups, (T + rpb - 1) / rpb);
  colsum_kernel<<<grid, COLSUM_THREADS, 0, CB_ST(stream)>>>(static_cast<const __nv_bfloat16*>(x),
                                                            out, T, C, ld, rpb);
  CB_RET();
}
extern "C" int cb_sin_init(float* p, size_t n, size_t index_offset, float scale, void* stream) {
  sin_init_kernel<<<grid_for(n, 256), 256, 0, CB_ST(stream)>>>(p, n, index_offset, scale);
  CB_RET();
}
extern "C" int cb_normal_init(float* p, size_t n, size_t index_offset, unsigned long long seed,
                              float mean, float std, void* stream) {
  normal_init_kernel<<<grid_for((n + 3) / 4 + 1, 256), 256, 0, CB_ST(stream)>>>(
      p, n, index_offset, static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32), mean, std);
  CB_RET();
}
extern "C" int cb_f32_to_bf16(const float* x, void* y, size_t n, void* stream) {
  f32_to_bf16_kernel<<<grid_for(n, 256), 256, 0, CB_ST(stream)>>>(
      x, static_cast<__nv_bfloat16*>(y), n);
  CB_RET();
}

// ------------------------------------------------------------------------------------------
// Dropout applied to a [rows, cols] bf16 tensor (cols % 8 == 0): y = x * mask * scale with the
// mask of common.cuh (dropout_bits) over the element index row * cols + col.  The forward pass
// of the decoder applies it inside GEMM epilogues; this kernel recomputes the same mask on the
// gradient in the backward pass and serves the stand-alone nn module.
namespace cb {
__global__ void dropout_apply_kernel(const __nv_bfloat16* __restrict__ x, int ldx,
                                     __nv_bfloat16* __restrict__ y, int ldy, size_t rows, int cols,
                                     int thr, uint32_t key, float scale) {
  const int nv = cols / 8;
  const size_t total = rows * nv;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t r = i / nv;
    const int c = static_cast<int>(i % nv) * 8;
    float v[8];
    load8(x + r * ldx + c, v);
    const unsigned long long g0 = (static_cast<unsigned long long>(r) * cols + c) >> 2;
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      const uint32_t h = dropout_bits(g0 + g, key);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        v[g * 4 + j] = static_cast<int>((h >> (8 * j)) & 255u) < thr ? 0.f : v[g * 4 + j] * scale;
    }
    store8(y + r * ldy + c, v);
  }
}
}  // namespace cb

extern "C" int cb_dropout_apply(const void* x, int ldx, void* y, int ldy, size_t rows, int cols,
                                int thr, unsigned int key, void* stream) {
  if (cols % 8 != 0 || ldx % 8 != 0 || ldy % 8 != 0 || thr < 0 || thr > 255) return -1;
  if (rows == 0) return 0;
  const size_t work = rows * (cols / 8);
  const int blocks = static_cast<int>(std::min<size_t>((work + 255) / 256, cb::sm_count() * 16));
  cb::dropout_apply_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), ldx, static_cast<__nv_bfloat16*>(y), ldy, rows, cols,
      thr, key, 256.0f / static_cast<float>(256 - thr));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
