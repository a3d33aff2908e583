// Allocation-free entry point of libmaester_b200.  It has no counterpart in the reference project.
//
// Who needs it: hosts that must not (or cannot) create device allocations while they run — a
// process that handed the whole GPU to its own memory pool at start-up, a C or C++ caller that
// links this library without PyTorch's caching allocator, a service whose memory plan is fixed
// before the first request.  For those, the regular attention backward is awkward because it
// wants a caller-allocated fp32 work buffer of B*H*S elements.
//
// mb_attn_bwd_noalloc() is the same computation as mb_attn_bwd() (gradients of q, k, v of masked
// GQA attention into one packed buffer) but keeps that work buffer in a fixed array inside the
// library's device image:
//   * capacity: MB_NOALLOC_MAX_ROWS = 1,048,576 fp32 values (4 MiB) -> B*H*S must not exceed it;
//     larger problems are refused with return code MB_NOALLOC_TOO_LARGE and a message on stderr;
//   * every GPU that loads the library carries these 4 MiB until the process exits;
//   * the function calls no cudaMalloc / cudaFree / cudaHostAlloc nor any allocating library
//     routine; inputs, outputs and the optional status word are the caller's memory.  (A host
//     thread that has no CUDA context bound yet gets the device's primary context bound with
//     cudaSetDevice before the TMA descriptors are encoded.)
//   * the first call on each device looks up the device address of the array
//     (cudaGetSymbolAddress, with that device current); the first call of each head size on each
//     device raises that kernel's shared-memory limit.  Make those first calls outside of any
//     stream capture, and do not race two first calls on one device from different host threads;
//   * all calls on one device share the array.  The array keeps whatever the previous call left;
//     this is harmless because each call first rewrites the B*H*S entries it will read, but two
//     calls that overlap on the GPU (different streams, no dependency) race on it — serialise them.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MB_NOALLOC_MAX_ROWS (1 << 20)
#define MB_NOALLOC_TOO_LARGE (-20)
#define MB_NOALLOC_SETUP_FAILED (-21)

// Arguments as mb_attn_bwd without the work buffer:
//   q, k: [B,S,H|KV,hd] bf16 after norm/rope, v: [B,S,KV,hd]; token strides in elements, head stride hd
//   out, dout: [B,S,H,hd] contiguous bf16;  lse: [B,H,S] fp32 from the forward pass
//   dqkv: [B*S, >= (H+2KV)*hd] bf16 with row pitch g_stride, receives dq | dk | dv
//   doc, kv_lo_blk, q_hi_blk: optional int32 mask helpers (may be null)
//   status_out: optional device int (the caller clears it); a kernel whose bounded wait expires stores a
//     non-zero code there.  If null, the code goes to a word inside the library instead: read and clear it
//     with mb_noalloc_status() once the stream has finished.
// Returns 0 on success, a negative code otherwise.
int mb_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* out, const void* dout,
                        const float* lse, void* dqkv, const int* doc, const int* kv_lo_blk, const int* q_hi_blk,
                        int B, int S, int H, int KV, int hd, long long q_tok_stride, long long k_tok_stride,
                        long long v_tok_stride, long long g_stride, int causal, int window, float scale,
                        int* status_out, cudaStream_t stream);


// Reads and clears the built-in status word of the current device (used by calls with status_out == null).
// Synchronises the device (it copies one int back).  Returns the code (0: no wait expired), or
// MB_NOALLOC_SETUP_FAILED if the word cannot be read.
int mb_noalloc_status(void);

#ifdef __cplusplus
}
#endif
