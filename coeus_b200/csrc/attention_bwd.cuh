// Launch arguments shared by the attention-backward kernels (attention_bwd.cu: the generic
// kernel; attention_bwd_dh64.cu: the pipelined kernel for head dimension 64).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace cb {

struct AttnBwdArgs {
  int B, S, nh;
  const float* lse;     // [B, nh, S]
  const float* delta;   // [B, nh, S]
  float* dq_acc;        // fp32 [B*S, nh*dh], zero-initialised
  __nv_bfloat16* dk;    // [B*S, ...] pitch ldd, already offset to the K slice
  __nv_bfloat16* dv;
  int ldd;
  float scale;
  float scale_log2;
  int causal;
  int* status;
  long long* trace;     // optional timeline of block 0 (a debugging aid), else nullptr
  // dropout on the probabilities (drop_thr = 0: none), the mask of the forward pass: element
  // (query q, key kv) of head (b, h) has index ((b nh + h) S + q) S + kv, S % 4 == 0
  int drop_thr;
  uint32_t drop_key;
  float drop_scale;
};

// Head dimension 64 (attention_bwd_dh64.cu).
// `tdq`: fp32 map of the dQ accumulator as (nh*64, S, B), box 32 x 32 x 1; `tdk`, `tdv`: bf16 maps
// of the dK / dV output slices as (nh*64, S, B), box 64 x 128 x 1.
int launch_attn_bwd_dh64(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                         const CUtensorMap& tdo, const CUtensorMap& tdq, const CUtensorMap& tdk,
                         const CUtensorMap& tdv, const AttnBwdArgs& a, cudaStream_t st);
// (with a.drop_thr > 0 the kernels apply the forward pass's dropout mask)

}  // namespace cb
