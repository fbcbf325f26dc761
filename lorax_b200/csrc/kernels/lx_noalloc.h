/* C declarations of the GEMM entry point that never allocates.
 *
 * This entry point has no counterpart in the reference (predibase/lorax): there every GEMM goes through
 * cuBLAS, which manages its own workspace.  It exists for callers of this library that are not allowed to
 * allocate device memory when they call it -- a host program that pre-allocates everything at start-up and
 * bans cudaMalloc afterwards, or a plugin inside another framework's process that must stay out of that
 * framework's allocator -- and that therefore cannot hand the split-K kernel the scratch buffer the regular
 * entry point (lx_gemm_bf16) asks for.  The scratch is a fixed array inside the library image instead.
 *
 * Cost and limits: lx_gemm_bf16_noalloc_scratch_bytes() bytes (8 MiB + 4 KiB + 16 B) are held on every GPU
 * that loads the library, until the process exits.  T <= 256 tokens, N <= 131072.  A split_k whose partial tiles
 * exceed 8 MiB is rejected; split_k = 0 picks one that fits.  Calls share the array: calls that overlap on the
 * GPU race.  The first call on each device performs a one-time set-up (resolves the array's device address and
 * sets a kernel attribute) and should be made before any stream capture.
 */
#ifndef LX_NOALLOC_H_
#define LX_NOALLOC_H_

#ifdef __cplusplus
extern "C" {
#endif

/* out[T, N] (bf16) = x[T, K] @ w[N, K]^T (+ bias[N]); row strides ldx / ldw / ldo in elements; `stream` is a
 * cudaStream_t.  Returns 0, or a negative code that lx_gemm_bf16_noalloc_strerror() explains. */
int lx_gemm_bf16_noalloc(const void* x, const void* w, void* out, const void* bias, int T, int N, int K,
                         long long ldx, long long ldw, long long ldo, int split_k, void* stream);

/* Device-side status of the last launch on the current device: out2[0] == 0 means ok.  The read is queued on `stream`
 * (a cudaStream_t: the one the GEMM ran on, which may be a non-blocking stream) and the call waits for it. */
int lx_gemm_bf16_noalloc_status(int* out2, void* stream);

const char* lx_gemm_bf16_noalloc_strerror(int code);
long long lx_gemm_bf16_noalloc_scratch_bytes(void);
int lx_gemm_bf16_noalloc_max_tokens(void);

#ifdef __cplusplus
}
#endif
#endif /* LX_NOALLOC_H_ */
