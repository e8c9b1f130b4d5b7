/*
 * TEST INFRASTRUCTURE — host-side prelude that lets the reference's scalar device functions
 * (epfml/pam pam/cuda_kernels.cu:15-136) compile as ordinary C++ without CUDA or torch.
 * nvcc resolves the unqualified calls in those functions as floor(float)->float,
 * log2(float)->float and pow(int,float)->double; "using namespace std" with <cmath> gives
 * g++ the same overload set, so the host build evaluates each expression in the same types.
 */
#include <cmath>
#include <math.h>
#include <cstdint>
using namespace std;
#define __device__
#define __host__
#define __forceinline__ inline
