/* gatzk_b200_tuning.h — measurement aids kept OUT of libgatzk_b200.so, in
 * libgatzk_b200_tuning.so: nothing here is on the proving path. */
#ifndef GATZK_B200_TUNING_H
#define GATZK_B200_TUNING_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Integer-pipe ceiling for the roofline of the inner-product kernels: 8x8-limb
 * multiply-accumulates per second over the whole GPU on register operands, with
 * 1 or 2 independent accumulators per lane.  No reference counterpart.
 * Returns 0 on success, a cudaError_t value otherwise. */
int gzk_tuning_mac_peak(int device, int chains, uint32_t iters, double* products_per_second);

#ifdef __cplusplus
}
#endif
#endif
