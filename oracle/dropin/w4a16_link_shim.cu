// Link-level drop-in: external definitions of the reference's W4 launchers (include/kernels.cuh:39-153 of
// the reference) on top of libw4a16_b200.so.  Built together with the reference's OWN, unmodified
// tests/test_kernels.cu, src/engine.cu, src/tokenizer.cpp and the kernel files that are not part of the W4
// projection path, it takes the place of src/kernels/gemv_w4a16.cu and src/kernels/gemm_prefill.cu; the two
// Q8_1 quantiser launchers of src/kernels/rmsnorm_rope.cu are renamed away on that file's command line
// (see the Makefile) so that the ones defined here are the ones the engine and the tests call.
// Test infrastructure: nothing here is part of the product library.
#include "kernels.cuh"   // the reference's declarations (with their default arguments)

#define W4A16_COMPAT_OUT_OF_LINE
#include "w4a16_kernels_compat.hpp"
