/* pam_b200 -- hooks for the test suite.  NOT part of the product ABI: nothing in the package's
 * hot path calls these, and a host application should not either. */
#ifndef PAM_B200_TESTING_H
#define PAM_B200_TESTING_H

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

#ifdef __cplusplus
}
#endif
#endif
