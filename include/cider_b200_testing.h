/*
 * cider_b200 - testing aids of the C ABI.  Not part of the drop-in boundary: a
 * binding of the reference has no use for these.  They only choose WHICH of the
 * library's equivalent kernels runs, so that the test-suite can put every kernel
 * under the oracle on shapes the automatic choice would not give it; every
 * choice computes the same results.  Process-wide; 0 restores the automatic
 * choice.
 */
#ifndef CIDER_B200_TESTING_H_
#define CIDER_B200_TESTING_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Integer-GEMM kernel family: 0 = automatic (tensor-core kernel whenever the shape
 * allows, streaming kernel for a handful of rows), 1 = always the plain CUDA-core
 * kernel, 2 = tensor-core kernel or CIDER_E_SHAPE. */
int cider_set_gemm_backend(int backend);

/* Tile shape of the tensor-core GEMM: tile 128 = single-CTA 128-row kernel, 2 =
 * CTA-pair (256 x 256) kernel, 0 = automatic; bn = N tile of the single-CTA kernel
 * (64, 128, 192, 256; 0 = automatic); for the per-group linear on int8 weights bn 128 is
 * the 128 x 128-tile kernel and bn 256 the 128 x 256-tile one.  Other values return
 * CIDER_E_INVALID. */
int cider_testing_set_tile(int tile, int bn);

/* Decode-attention kernel: 0 = automatic, 1 = the CUDA-core form, 2 = the tensor-core form
 * (mma.sync; grouped queries of 128 dims with 2, 4 or 8 query heads per KV head - other
 * shapes keep the CUDA-core form). */
int cider_testing_set_sdpa_kernel(int mode);

/* Name of the tensor-core GEMM kernel the calling thread launched last ("" if none): lets a
 * report name the kernel a timed figure belongs to from the dispatch itself. */
const char *cider_testing_last_gemm_kernel(void);

/* cider_allreduce_f16 with all `world` ranks emulated on ONE GPU as a single cooperative
 * launch (rank = blockIdx.y; a cooperative launch guarantees that the CTAs that wait for
 * one another are resident together - separate launches on one GPU would not be).  ins /
 * outs / inboxes are host arrays of `world` device pointers on the current device, the
 * inboxes zeroed before first use.  absent_rank >= 0 makes that rank skip the call, so
 * that the others' bounded wait runs out: CIDER_STATUS_PEER_TIMEOUT is recorded and the
 * kernel returns without writing results. */
int cider_testing_allreduce_emulated(const void *const *ins, void *const *outs, int64_t count, int world,
                                     void *const *inboxes, size_t inbox_bytes, int64_t wait_cycles,
                                     int absent_rank, void *stream);

/* cider_allreduce_add_rmsnorm_quant with its ranks emulated on one GPU the same way; the ranks
 * share norm_w; partials / xs / ys / qs / scales are host arrays of `world` device pointers. */
int cider_testing_allreduce_norm_emulated(const void *const *partials, void *const *xs, const void *norm_w,
                                          float eps, int64_t M, int64_t K, void *const *ys, void *const *qs,
                                          float *const *scales, int world, void *const *inboxes,
                                          size_t inbox_bytes, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* CIDER_B200_TESTING_H_ */
