/* Fused softmax cross-entropy, mean loss, for callers that cannot allocate.
 *
 * This entry point has no counterpart in the reference library.
 *
 * Who needs it: some callers of this library are not in a position to obtain
 * device memory when they want a loss value.  Examples are a serving or
 * training process that has already handed every byte of the GPU to its own
 * pool (a fresh cudaMalloc would fail, or would fragment the pool), and code
 * that runs on a latency-critical path where the implicit device-wide
 * synchronisation of cudaMalloc / cudaFree is not acceptable.  The regular
 * path (cclx_softmax_xent) writes one loss per row into a buffer that the
 * caller has to provide and then average; here the per-row losses live in a
 * fixed array inside the library, and a second small kernel averages them into
 * the single float the caller passes.
 *
 * What it does: same math as cclx_softmax_xent.  `logits` is [rows, ld] bf16
 * with `vocab` classes per row followed by `pad_cols` alignment columns; on
 * return every row holds (softmax - onehot) * grad_scale (padding columns
 * zero) and *mean_loss = sum_rows(logsumexp - logit[target]) / rows.  Rows with
 * a target outside [0, vocab) contribute zero loss and zero gradient.
 *
 * Limits and rules:
 *  - rows <= CCLX_XENT_NOALLOC_MAX_ROWS (65536).  More rows are rejected with
 *    return code -1 and a message from cclx_last_error(); nothing is launched.
 *  - The scratch array is CCLX_XENT_NOALLOC_MAX_ROWS floats (256 KiB).  Every GPU
 *    on which the library is loaded holds it until the process exits.
 *  - The call makes no cudaMalloc / cudaFree and calls no allocating routine.
 *    The first call on each device looks up the device address of the scratch
 *    array (cudaGetSymbolAddress, with that device current) and caches it; make
 *    that first call before starting any stream capture.
 *  - All calls on one device share the scratch array and it keeps the last
 *    call's values.  Nothing in it has to start at zero: each call overwrites
 *    the first `rows` entries before reading them.  Two calls that overlap on
 *    the GPU (different streams, no dependency) race on it; order them.
 *  - `mean_loss` is device memory owned by the caller (one float, written, not
 *    accumulated).  `stream` is a cudaStream_t; the device of the pointers must
 *    be the current device of the calling thread.
 *
 * Returns 0 on success, -1 on error.
 */
#ifndef CCLX_XENT_NOALLOC_H
#define CCLX_XENT_NOALLOC_H

#include <stddef.h>

#define CCLX_XENT_NOALLOC_MAX_ROWS 65536

#ifdef __cplusplus
extern "C" {
#endif

int cclx_softmax_xent_mean_noalloc(void* logits_bf16, const long long* targets, float* mean_loss, size_t rows,
                                   int vocab, size_t ld, float grad_scale, int pad_cols, void* stream);

#ifdef __cplusplus
}
#endif

#endif
