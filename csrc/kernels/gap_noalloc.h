/* Global average pooling for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference (FastDeploy); it exists for users of
 * this library's C ABI who cannot call cudaMalloc themselves and cannot let a library do it
 * for them:
 *   - plugin or callback code hosted by another application (a media pipeline element, an
 *     inference-server execute hook) whose device-memory budget was handed out at start-up,
 *     so that a late cudaMalloc may fail or is simply forbidden by the host;
 *   - latency-critical loops: cudaMalloc / cudaFree synchronise the whole device, which
 *     stalls every other stream of the process for the duration of the call;
 *   - plain C programs that link this library without PyTorch and therefore have no caching
 *     allocator to hand the regular entry point a scratch tensor from.
 *
 * The regular path (fdb_simple_create with kind 0 and 1) takes a caller-allocated scratch
 * buffer for the per-split partial sums. Here that scratch lives in one array of
 * FDB_GAP_NOALLOC_MAX_SCRATCH_FLOATS floats (4 MiB) that is part of the library image: every
 * GPU that loads the library holds those 4 MiB until the process exits.
 *
 * Rules of use
 *   - n * splits * c must not exceed FDB_GAP_NOALLOC_MAX_SCRATCH_FLOATS; larger problems are
 *     rejected with FDB_GAP_NOALLOC_TOO_LARGE and nothing is launched.
 *   - The first call on each device looks up the device address of the array (with that device
 *     current). Make this first call during start-up, before any stream capture begins.
 *   - All calls on one device share the one array. It keeps whatever the previous call left in
 *     it; this operation overwrites every element it later reads, so nothing has to be cleared
 *     between calls. Two calls whose kernels can overlap on the GPU (different streams without
 *     an ordering between them) race on the array: serialise them.
 *   - x must be 16-byte aligned, and c, x_ld and x_n_stride multiples of 8 elements (the kernel reads
 *     16 bytes at a time from every pixel of every image); x_ld and out_ld must be at least c; a non-zero
 *     x_n_stride must span one whole image ((hw - 1) * x_ld + c elements). Anything else is rejected
 *     with FDB_GAP_NOALLOC_BAD_ARGUMENT before a kernel is launched.
 *   - If the CUDA runtime already holds an error from earlier work when the call comes in, the call
 *     launches nothing and returns FDB_GAP_NOALLOC_CUDA_ERROR; it never clears that error.
 *   - No cudaMalloc, cudaFree or other allocating routine is called, on any path.
 */
#ifndef FDB_GAP_NOALLOC_H_
#define FDB_GAP_NOALLOC_H_

#ifdef __cplusplus
extern "C" {
#endif

#define FDB_GAP_NOALLOC_MAX_SCRATCH_FLOATS (1 << 20)

enum {
  FDB_GAP_NOALLOC_OK = 0,
  FDB_GAP_NOALLOC_BAD_ARGUMENT = 1, /* null / misaligned pointer, non-positive size, c, x_ld or x_n_stride not a
                                       multiple of 8, strides too short, out_dtype outside 0..2 */
  FDB_GAP_NOALLOC_TOO_LARGE = 2,    /* n * splits * c exceeds the built-in scratch */
  FDB_GAP_NOALLOC_CUDA_ERROR = 3    /* device query, symbol lookup or launch failed */
};

/* out[i][ch] = mean over p of x[i][p][ch] for an NHWC tensor of 16-bit floats.
 *   x          device pointer, fp16 (is_bf16 = 0) or bf16 (is_bf16 = 1), 16-byte aligned
 *   out        device pointer, [n][out_ld] of out_dtype (0 fp16, 1 bf16, 2 fp32), out_ld >= c
 *   n, hw, c   images, pixels per image, channels (c a multiple of 8)
 *   x_ld       elements between consecutive pixels (>= c, multiple of 8)
 *   x_n_stride elements between consecutive images (0 means hw * x_ld; otherwise a multiple of 8 that
 *              spans at least one image)
 *   splits     pixel ranges summed by separate thread blocks (>= 1)
 *   stream     cudaStream_t
 * Returns one of the codes above. */
int fdb_global_avgpool_noalloc(const void* x, void* out, int n, int hw, int c, int x_ld,
                               long long x_n_stride, int splits, int is_bf16, int out_dtype,
                               int out_ld, void* stream);

/* Constant, human-readable text for a return code (never allocates). */
const char* fdb_global_avgpool_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
#endif /* FDB_GAP_NOALLOC_H_ */
