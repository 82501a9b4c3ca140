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

#ifdef __cplusplus
extern "C" {
#endif

/* Integer-GEMM kernel family: 0 = automatic (tensor-core kernel whenever the shape
 * allows, streaming kernel for a handful of rows), 1 = always the plain CUDA-core
 * kernel, 2 = tensor-core kernel or CIDER_E_SHAPE. */
int cider_set_gemm_backend(int backend);

/* Tile shape of the tensor-core GEMM: tile 128 = single-CTA 128-row kernel, 2 =
 * CTA-pair (256 x 256) kernel, 0 = automatic; bn = N tile of the single-CTA kernel
 * (64, 128, 192, 256; 0 = automatic).  Other values return CIDER_E_INVALID. */
int cider_testing_set_tile(int tile, int bn);

#ifdef __cplusplus
}
#endif
#endif /* CIDER_B200_TESTING_H_ */
