/* Decode attention without any allocation.  This entry point has no counterpart in the
 * reference (neuralboot/trapetum allocates every buffer when a model is loaded).
 *
 * Who needs it: a caller that cannot allocate device memory at the time of the call.  Examples:
 * a C program or a plugin inside another runtime that received a fixed slice of device memory at
 * start-up and is not allowed to call cudaMalloc later; a control loop with a latency bound, for
 * which the device-wide synchronisation inside cudaMalloc/cudaFree is not acceptable.  The
 * ordinary entry point, tb_attn_decode, needs scratch for the partial results of its key splits
 * and leaves its allocation to the caller; this one keeps that scratch inside the library.
 *
 *   int tb_attn_decode_noalloc(const DecodeArgs* args, int dtype, int batch, cudaStream_t stream);
 *
 * The argument block is defined in decode_args.h, which this header includes, so a C caller can fill it.
 * Same arguments, same result and same return convention as tb_attn_decode (0 = launched,
 * > 0 = a cudaError_t, < 0 = refused, tb_error() tells why).  `args->partial` is ignored.  The
 * caller still owns the query, the cache pools, the page table, the lengths and the output.
 *
 * - The scratch is a fixed array in device memory, TB_ATTN_DECODE_NOALLOC_MAX_FLOATS floats
 *   (4 MiB), part of the library image: every GPU that loads the library holds it until the
 *   process ends.  A call that needs more, batch * n_heads * n_splits * (head_dim + 2) floats when
 *   n_splits > 1, is refused with a message that names both numbers.  With n_splits == 1 no
 *   scratch is used and any batch goes through.
 * - The first call on a device looks up the array's device address (once per device, with that
 *   device current) and keeps it.  Make that first call in ordinary stream order, before any
 *   stream capture is begun on the device.
 * - It calls neither cudaMalloc nor cudaFree nor any routine that allocates, torch's included.
 * - All calls share the one array, and it keeps whatever the last call left.  Nothing in it has
 *   to start at zero: each call writes every partial slot it later reads (empty splits write a
 *   "nothing here" marker), so stale contents are never read.  Two calls that overlap on the GPU
 *   (different streams without an ordering between them) race on the array; order them.
 */
#ifndef TB_ATTENTION_DECODE_NOALLOC_H
#define TB_ATTENTION_DECODE_NOALLOC_H

#include <cuda_runtime_api.h>
#include "decode_args.h"         /* the argument block, with a comment on every field */

#define TB_ATTN_DECODE_NOALLOC_MAX_FLOATS (1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

int tb_attn_decode_noalloc(const DecodeArgs* args, int dtype, int batch, cudaStream_t stream);

#ifdef __cplusplus
}
#endif

#endif
