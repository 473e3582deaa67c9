/* CPU oracle for the deformable-kernel operator path -- TEST INFRASTRUCTURE ONLY.
 * Builds the fp32 and fp64 instantiations of dk_oracle_impl.inc and a few helpers.
 * Compile:  gcc -O2 -fopenmp -shared -fPIC oracle/dk_oracle.c -o oracle/_build/libdk_oracle.so -lm
 */
#include <math.h>
#include <stdlib.h>
#include "dk_oracle.h"

#define REAL float
#define SUF _f32
#include "dk_oracle_impl.inc"
#undef REAL
#undef SUF

#define REAL double
#define SUF _f64
#include "dk_oracle_impl.inc"
#undef REAL
#undef SUF

#ifdef _OPENMP
#include <omp.h>
int dk_oracle_max_threads(void) { return omp_get_max_threads(); }
void dk_oracle_set_threads(int n) { omp_set_num_threads(n); }
#else
int dk_oracle_max_threads(void) { return 1; }
void dk_oracle_set_threads(int n) { (void)n; }
#endif

/* Output extent, csrc/filter_sample_depthwise_cuda.cpp:42-43 (integer division). */
void dk_oracle_fill_out_size(dk_oracle_geom *g) {
  g->out_h = (g->in_h + 2 * g->pad_h - (g->dil_h * (g->k_h - 1) + 1)) / g->stride_h + 1;
  g->out_w = (g->in_w + 2 * g->pad_w - (g->dil_w * (g->k_w - 1) + 1)) / g->stride_w + 1;
}
