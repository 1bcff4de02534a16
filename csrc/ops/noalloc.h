/* Column-sum entry point for callers that must not allocate.
 *
 * This entry point has no counterpart in the reference project; it exists for
 * embedders of this library.
 *
 * Who needs it: code that runs where a device allocation is forbidden or
 * impossible -- a host callback or a plugin invoked inside someone else's
 * stream-ordered region, a real-time loop with a no-allocation rule, a runtime
 * whose memory is handed out once at start-up and whose allocator the library
 * is not allowed to touch.  The regular path, mccl::ops::colsum_bf16, needs a
 * scratch buffer of colsum_slabs(rows) * dim floats from its caller, and the
 * Python binding gets that buffer from torch's allocator on every call.
 *
 * What it does: out[c] = sum over r of in[r * dim + c] for a row-major bf16
 * matrix, same two-stage, fixed-order reduction as the regular path, with the
 * partial sums kept in a fixed array that is part of the library image
 * (MCCL_NOALLOC_SCRATCH_FLOATS floats, 4 MiB).  Every GPU that loads the
 * library carries that array until the process exits.
 *
 * Rules for callers
 *  - `in` (bf16, 16-byte aligned) and `out` (fp32) are device pointers the
 *    caller owns; dim must be a multiple of 8.
 *  - ceil(rows / 64) * dim must not exceed MCCL_NOALLOC_SCRATCH_FLOATS and
 *    ceil(rows / 64) must not exceed MCCL_NOALLOC_MAX_SLABS (a grid-dimension
 *    limit that very long, narrow matrices reach first); larger problems are
 *    refused with MCCL_NOALLOC_TOO_LARGE and nothing is launched.
 *  - `in`, `out` and `stream` must belong to the device that is current when
 *    the call is made: the scratch array used is the current device's copy,
 *    and a kernel given another device's pointers would read or write the
 *    wrong memory.  Pointers that CUDA reports as another device's (or as
 *    host memory) are refused with MCCL_NOALLOC_BAD_ARGUMENT.
 *  - The first call on a device looks up the device address of the array (no
 *    allocation, but a runtime query): make that first call before any stream
 *    capture begins on that device.
 *  - All calls in the process share the one array per device.  Nothing in it
 *    has to be cleared between calls (every cell that is read is written first
 *    by the same call), but two calls whose kernels overlap on the GPU -- two
 *    streams, or two threads -- would overwrite each other's partial sums:
 *    keep calls on one device ordered.
 *  - No cudaMalloc, cudaFree or allocating library routine is called.
 */
#ifndef MCCL_OPS_NOALLOC_H_
#define MCCL_OPS_NOALLOC_H_

#ifdef __cplusplus
extern "C" {
#endif

#define MCCL_NOALLOC_SCRATCH_FLOATS (1 << 20)
#define MCCL_NOALLOC_MAX_SLABS 65535

enum {
  MCCL_NOALLOC_OK = 0,
  MCCL_NOALLOC_BAD_ARGUMENT = -1,  /* null pointer, dim not a multiple of 8, misaligned input, memory of another device */
  MCCL_NOALLOC_TOO_LARGE = -2,     /* partial sums would not fit the fixed array */
  MCCL_NOALLOC_CUDA_ERROR = -3     /* a CUDA call failed; see mccl_noalloc_last_error() */
};

/* stream is a cudaStream_t passed as void* (NULL = the default stream).
 * Returns one of the codes above. */
int mccl_colsum_bf16_noalloc(const void* in_bf16, float* out, int rows, int dim, void* stream);

/* Human-readable reason for the last non-zero return on this thread. */
const char* mccl_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif

#endif  /* MCCL_OPS_NOALLOC_H_ */
