/* pam_b200 -- hooks for the test suite.  NOT part of the product ABI: nothing in the package's
 * hot path calls these, and a host application should not either. */
#ifndef PAM_B200_TESTING_H
#define PAM_B200_TESTING_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Forces the CTA tile of the matrix-product kernels so that tests can run every tile shape on the
 * same problem and check that results do not depend on the tile (the library normally picks a
 * 128x128, a 64x64 or, for small or ragged-edged products, a 32x32 tile per problem from a cost
 * model).  0 = by cost model (default), 1 = always 128x128, 2 = always 64x64, 3 = always
 * 32x32 (products that have no 32x32 kernel use 64x64).  Process-wide and not thread-safe, which is
 * why it is kept out of pam_b200.h.  No counterpart in the reference. */
int pamk_test_set_tile_policy(int policy);

/* The tile edge (128, 64 or 32) the cost model gives the PAM product of these dimensions under the
 * current policy, with the automatic split: lets a test pin the measured-best choices without a GPU.
 * Negative (PAMK_ERR_ARG) for an empty problem.  No counterpart in the reference. */
int pamk_test_planned_tile(int64_t batch, int64_t M, int64_t N, int64_t K);

#ifdef __cplusplus
}
#endif
#endif
