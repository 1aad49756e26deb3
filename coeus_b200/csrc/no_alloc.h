/* Attention backward for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference (which has no GPU code and no backward
 * pass); it is an addition of this library.
 *
 * Who needs it: a process whose device memory was budgeted once at start-up -- for instance a
 * serving or fine-tuning host that handed the rest of HBM to its own KV-cache or activation
 * pool, so that a late cudaMalloc can fail outright -- and latency-sensitive loops in which
 * cudaMalloc / cudaFree are unwelcome because they synchronise the whole device.  Such callers
 * cannot provide the two scratch buffers that cb_attn_bwd() asks for (the fp32 dQ accumulator
 * and the per-row delta), and cannot let a framework allocator create them either.
 *
 * cb_attn_bwd_noalloc() computes exactly what cb_attn_bwd() computes, but takes its scratch from
 * a fixed array that lives in the library image itself (a file-scope __device__ array of
 * CB_NOALLOC_SCRATCH_FLOATS floats = 16 MiB).  Every GPU whose context loads the library holds
 * that array until the process exits.  The function calls no cudaMalloc, cudaFree or any other
 * allocating routine; the caller still passes all inputs and the output.
 *
 * Limit: B*S*nh*dh + B*nh*S <= CB_NOALLOC_SCRATCH_FLOATS, otherwise the call returns
 * CB_NOALLOC_ERR_TOO_LARGE and launches nothing.
 *
 * First call on a device: the address of the array is looked up once per device (with that
 * device current) and cached.  Make that first call outside of any stream capture.
 *
 * Sharing: all calls on a device use the same array and it keeps the previous call's contents;
 * the function clears the part that must start at zero on the given stream before using it.
 * Two calls whose kernels can overlap on the GPU (different streams without an ordering between
 * them, or different host threads on the same device) race on the scratch and give wrong
 * results; order them.
 */
#ifndef COEUS_B200_NO_ALLOC_H_
#define COEUS_B200_NO_ALLOC_H_

#ifdef __cplusplus
extern "C" {
#endif

#define CB_NOALLOC_SCRATCH_FLOATS (4u * 1024u * 1024u)
#define CB_NOALLOC_ERR_TOO_LARGE (-100)
#define CB_NOALLOC_ERR_SYMBOL (-101)

/* Same arguments and meaning as cb_attn_bwd() without `delta` and `dq_acc`:
 *   dO, q, k, v, o : bf16 [B*S, nh*dh] views with row pitches lddo, ldq, ldk, ldv, ldo (elements)
 *   lse            : fp32 [B, nh, S] from the forward pass
 *   dqkv           : bf16 [B*S, 3*nh*dh] (pitch ldd) receiving dQ | dK | dV
 * Returns 0 on success, a negative code otherwise (see cb_noalloc_strerror). */
int cb_attn_bwd_noalloc(const void* dO, const void* q, const void* k, const void* v,
                        const void* o, const float* lse, void* dqkv, int B, int S, int nh, int dh,
                        int lddo, int ldq, int ldk, int ldv, int ldo, int ldd, float scale,
                        int causal, int* status, void* stream);

/* Human-readable text for a return code of cb_attn_bwd_noalloc. */
const char* cb_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
#endif
