/*
 * TEST INFRASTRUCTURE — builds liboracle: the C restatement of the PAM scalar semantics
 * (pam_scalar_oracle.h) wrapped in the array / matrix loops of array_loops.inc.
 * See those two files for the reference lines each function follows.
 * Build: python oracle/build.py   (gcc -O2 -fopenmp, no fast-math, no flush-to-zero)
 */
#include "pam_scalar_oracle.h"
#include "array_loops.inc"
