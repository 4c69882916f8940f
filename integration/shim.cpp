// Reference-side binding: the launcher layer of tensorax (csrc/tensor_ops.h:170-240), implemented
// on libtensorax_b200.so instead of csrc/cuda/kernels/attn.cu and csrc/cuda/tensor_cuda.cu.
//
// integration/Makefile compiles the reference's own, unmodified csrc/tensor_ops.cpp (the pybind11
// module `_C` and its dispatchers), csrc/cpu/tensor_cpu.cpp and its non-attention CUDA files from the
// reference checkout where they lie, and links them with THIS file in place of attn.cu and
// tensor_cuda.cu.  Every function below keeps the reference's name and argument list; a non-zero
// status of the library becomes the std::runtime_error the dispatchers already let through to Python
// (the reference's own launchers print and exit() instead, csrc/cuda/cuda_utils.cuh:6-14).
#include <stdexcept>
#include <vector>

#include "tensor_ops.h"          // the reference's header, found through -I<reference>/csrc
#include "tensorax_b200.h"

namespace tensorax {

static inline void tx_check(int rc)
{
    if (rc != TX_OK) throw std::runtime_error(tx_last_error());
}

// ---- csrc/tensor_ops.h:170-194, defined in the reference by csrc/cuda/kernels/attn.cu:962-1111,1564-1615
void sdpa_naive_cuda(const float *Q, const float *K, const float *V, const float *mask, float *out,
                     int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t dk, int64_t dv)
{
    tx_check(tx_sdpa_naive_cuda(Q, K, V, mask, out, B, H, Sq, Sk, dk, dv));
}
void sdpa_tiled_cuda(const float *Q, const float *K, const float *V, const float *mask, float *out,
                     int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t dk, int64_t dv)
{
    tx_check(tx_sdpa_tiled_cuda(Q, K, V, mask, out, B, H, Sq, Sk, dk, dv));
}
void sdpa_flash_cuda(const float *Q, const float *K, const float *V, const float *mask, float *out,
                     int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t dk, int64_t dv)
{
    tx_check(tx_sdpa_flash_cuda(Q, K, V, mask, out, B, H, Sq, Sk, dk, dv));
}
void sdpa_optimized_flash_cuda(const float *Q, const float *K, const float *V, const float *mask, float *out,
                               int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t dk, int64_t dv)
{
    tx_check(tx_sdpa_optimized_flash_cuda(Q, K, V, mask, out, B, H, Sq, Sk, dk, dv));
}
void sdpa_mma_cuda(const float *Q, const float *K, const float *V, const float *mask, float *out,
                   int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t dk, int64_t dv)
{
    tx_check(tx_sdpa_mma_cuda(Q, K, V, mask, out, B, H, Sq, Sk, dk, dv));
}
// attn.cu:1462-1521
void sdpa_mma_fp16_cuda(const void *Qh, const void *Kh, const void *Vh, float *out,
                        int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t dk, int64_t dv)
{
    tx_check(tx_sdpa_mma_fp16_cuda(Qh, Kh, Vh, out, B, H, Sq, Sk, dk, dv));
}
// attn.cu:1523-1562
void cast_f32_to_f16_cuda(const float *in, void *out, int64_t n)
{
    tx_check(tx_cast_f32_to_f16_cuda(in, out, n));
}

// ---- csrc/tensor_ops.h:214-233, attn.cu:1113-1140,1617-1722: 32 clock64 stamps per call
#define TX_PROFILE_SHIM(ref_name, lib_name)                                                              \
    std::vector<long long> ref_name(const float *Q, const float *K, const float *V, const float *mask,    \
                                    float *out, int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t dk, \
                                    int64_t dv)                                                           \
    {                                                                                                     \
        std::vector<long long> ticks(32, 0);                                                              \
        tx_check(lib_name(Q, K, V, mask, out, B, H, Sq, Sk, dk, dv, ticks.data()));                       \
        return ticks;                                                                                     \
    }
TX_PROFILE_SHIM(sdpa_naive_profile_sections_cuda, tx_sdpa_naive_profile_sections_cuda)
TX_PROFILE_SHIM(sdpa_tiled_profile_sections_cuda, tx_sdpa_tiled_profile_sections_cuda)
TX_PROFILE_SHIM(sdpa_flash_profile_sections_cuda, tx_sdpa_flash_profile_sections_cuda)
TX_PROFILE_SHIM(sdpa_mma_profile_sections_cuda, tx_sdpa_mma_profile_sections_cuda)
TX_PROFILE_SHIM(sdpa_optimized_flash_profile_sections_cuda, tx_sdpa_optimized_flash_profile_sections_cuda)
#undef TX_PROFILE_SHIM

// ---- csrc/cuda/tensor_cuda.cu:7-29
bool cuda_is_available() { return tx_cuda_is_available() != 0; }
void *cuda_malloc(size_t n)
{
    void *p = tx_cuda_malloc(n);
    if (!p) throw std::runtime_error(tx_last_error());
    return p;
}
void cuda_free(void *p) { tx_check(tx_cuda_free(p)); }
void cuda_memcpy_h2d(void *d, const void *s, size_t n) { tx_check(tx_cuda_memcpy_h2d(d, s, n)); }
void cuda_memcpy_d2h(void *d, const void *s, size_t n) { tx_check(tx_cuda_memcpy_d2h(d, s, n)); }

}  // namespace tensorax
