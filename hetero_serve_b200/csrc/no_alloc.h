// An entry point that allocates nothing.  It has no counterpart in the reference
// (mneha05/hetero-serve): the reference's kernels take scratch tensors that PyTorch allocates.
//
// Who needs it.  Some hosts of this library may not call cudaMalloc while they run: a
// real-time loop whose memory was fixed at start-up, a process that shares its GPU memory
// budget with another allocator and has promised it every byte, code that runs where an
// allocation would synchronise the device or could fail.  Such a caller brings its inputs
// and outputs and wants the kernel's working memory to exist already.
//
// hs_attention_decode_noalloc is hs_attention_decode (split-context paged attention for
// single-query tokens, attention_decode.cu) with its scratch memory — partial sums, their
// (max, sum) pairs and the arrival counters — taken from one static device array of
// HS_NOALLOC_SCRATCH_FLOATS floats (8 MiB) that every GPU which loads the library holds
// until the process exits.  The caller still passes every input and output.  It calls no
// cudaMalloc, cudaFree or allocating library routine.
//
// Limits and rules:
//  * token_cap * n_heads * splits * (head_dim + 2) + token_cap * n_heads must not exceed
//    HS_NOALLOC_SCRATCH_FLOATS; larger launches return HS_ERR_TOO_LARGE (-3) and do nothing.
//    hs_attention_decode_noalloc_capacity() returns the limit.
//  * The first call on each device looks the array's device address up
//    (cudaGetSymbolAddress, with that device current).  That look-up is not a stream
//    operation: make the first call on a device outside any stream capture.
//  * All calls share the array, and it keeps what the last call left.  The counters are
//    cleared (cudaMemsetAsync on the caller's stream) before each launch; the rest is
//    overwritten before it is read.  Two calls that overlap on the GPU — on different
//    streams, or from different threads — race on it: serialise them.
#pragma once

#define HS_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define HS_NOALLOC_MAX_DEVICES 64

#ifdef __cplusplus
extern "C" {
#endif

// Largest scratch, in floats, a launch may need (see the rule above).
long long hs_attention_decode_noalloc_capacity(void);

// Arguments as hs_attention_decode without the three scratch pointers.  Returns 0, a negative
// HS_ERR_* code (-1 unsupported size, -2 bad argument, -3 beyond the static capacity) or a
// positive cudaError_t.
int hs_attention_decode_noalloc(void* out, const void* qkv, const void* pool, const int* table,
                                const int* tok_pos, const int* tok_req, const int* dec_info,
                                const int* plan_head, int token_cap, int n_heads, int n_kv_heads,
                                int head_dim, int page_size, int num_pages, int max_pages,
                                int q_off, int qkv_stride, int window, float scale, int splits,
                                int* status, void* stream);

#ifdef __cplusplus
}
#endif
