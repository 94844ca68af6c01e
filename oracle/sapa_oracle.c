/* sapa_oracle.c — CPU oracle for the SAPA upsampling hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  Only the tests, the smoke check and the benchmark's CPU-baseline leg may
 * load this library; the product never does (it fails loudly when its CUDA library is missing).
 *
 * It restates, as plain scalar C, the eight CUDA kernels of the reference:
 *   sapa/sapa/src/cuda/qk_cuda_kernel.cu        QKForward :29-68,  QKBackward :101-137
 *   sapa/sapa/src/cuda/av_cuda_kernel.cu        AVForward :29-75,  AVBackward :103-148
 *   deformsapa/deformsapa/src/cuda/deform_qk_cuda_kernel.cu   helpers :23-137, DeformQKForward :139-197,
 *                                                             DeformQKBackward :233-296
 *   deformsapa/deformsapa/src/cuda/deform_av_cuda_kernel.cu   DeformAVForward :139-195, DeformAVBackward :230-292
 * plus the softmax that the modules put between them (sapa_base.py:39, sapa_deform.py:52).
 *
 * Parity is PINNED: tests/golden holds vectors produced by the reference's own PyTorch check functions
 * (sapa/sapa/forward_check.py:9-24, deformsapa/deformsapa/forward_check.py:6-40, gradients by autograd
 * through them) and by the reference's compiled CUDA extensions run on a B200; tests/test_oracle.py
 * checks this file against both sets.
 *
 * Exported as <name>_f32 and <name>_f64.
 */
#include <math.h>
#include <stddef.h>
#include <string.h>

#define REAL float
#define FN(name) name##_f32
#include "sapa_oracle_impl.inc"
#undef REAL
#undef FN

#define REAL double
#define FN(name) name##_f64
#include "sapa_oracle_impl.inc"
#undef REAL
#undef FN

#ifdef _OPENMP
#include <omp.h>
int oracle_num_threads(void) { return omp_get_max_threads(); }
void oracle_set_num_threads(int n) { omp_set_num_threads(n); }
#else
int oracle_num_threads(void) { return 1; }
void oracle_set_num_threads(int n) { (void)n; }
#endif
