// C entry point around the UNMODIFIED reference CPU SDPA.  TEST INFRASTRUCTURE ONLY.
//
// oracle/Makefile compiles this file together with the reference's own
// csrc/cpu/tensor_cpu.cpp, taken from the reference checkout where it lies
// (nothing of the reference is copied into this repository), into
// oracle/_ref/libtensorax_ref_cpu.so.  The only thing added here is an
// unmangled name for tensorax::sdpa_cpu (csrc/tensor_ops.h:132-134).
#include "tensor_ops.h"

extern "C" __attribute__((visibility("default"))) void ref_sdpa_cpu(
    const float *Q, const float *K, const float *V, const float *mask, float *out,
    int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t d_k, int64_t d_v)
{
    tensorax::sdpa_cpu(Q, K, V, mask, out, B, H, Sq, Sk, d_k, d_v);
}

// tensorax::matmul_cpu (csrc/tensor_ops.h, csrc/cpu/tensor_cpu.cpp:131-156): a [batch, m, k] x b [batch, k, n]
extern "C" __attribute__((visibility("default"))) void ref_matmul_cpu(
    const float *a, const float *b, float *out, int64_t batch, int64_t m, int64_t n, int64_t k)
{
    tensorax::matmul_cpu(a, b, out, batch, m, n, k);
}
