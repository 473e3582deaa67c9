/* CPU oracle for the deformable-kernel operator path -- TEST INFRASTRUCTURE ONLY.
 * Only tests/, the smoke check and bench.py's CPU-baseline legs may link or load
 * this; the product library never does.  Parity is pinned by outputs of the
 * reference's own CUDA build run on a B200 (tests/golden/), see oracle/build_ref.py.
 */
#ifndef DK_ORACLE_H
#define DK_ORACLE_H

#define DK_ORACLE_MAX_CELLS 1024 /* largest scope_h * scope_w the oracle accepts */

/* Geometry of one call: the fields of the reference's SampleDepthwiseArgs
 * (csrc/filter_sample_depthwise_cuda.h:1-28) under shorter names. */
typedef struct {
  int batch, channel, in_h, in_w;
  int k_h, k_w, stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
  int out_h, out_w;
  int scope_h, scope_w, groups;
} dk_oracle_geom;

#endif
