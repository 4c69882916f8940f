// Exact-fp32 linear layer on CUDA cores: out = x @ W^T + bias, with the head
// split / merge of multi-head attention folded into the addressing.
//
// This is the step either side of SDPA in the reference's MultiHeadAttention.forward
// (tensorax/nn/attention/layers.py:112-128): F.linear (tensorax/functional.py:105-110
// = matmul, csrc/tensor_ops.cpp:295-329 / csrc/cpu/tensor_cpu.cpp:131-156, then a
// broadcast add of the bias) followed by reshape + transpose(1, 2), which in the
// reference are copies (and the transpose is not even bound).  Here the projection
// writes [B, heads, S, d_head] directly, and the output projection reads it back as
// [B, S, heads*d_head]: no intermediate tensor, no transpose kernel.
//
// fp32 FMAs, k ascending per output element, so results stay within 1e-5 of the
// reference CPU matmul; tensor cores are not used on purpose (TF32 products would
// not meet that bound).
#pragma once
#include <cstdint>

namespace txb {

struct LinearParams {
    const float *x;      // [B, S, K], or [B, heads_in, S, K/heads_in] when heads_in > 0
    const float *w;      // [N, K] row-major (the layer's weight; the product uses its transpose)
    const float *bias;   // optional [N]
    float *out;          // [B, S, N], or [B, heads_out, S, N/heads_out] when heads_out > 0
    int64_t B, S, K, N;
    int heads_in, heads_out;
};

constexpr int LIN_BM = 64, LIN_BN = 64, LIN_BK = 16, LIN_THREADS = 256;

__device__ __forceinline__ int64_t lin_index(int64_t m, int64_t c, int64_t S, int64_t width, int heads)
{
    if (heads <= 0) return m * width + c;
    const int64_t b = m / S, s = m % S, dh = width / heads;
    return ((b * heads + c / dh) * S + s) * dh + c % dh;
}

__global__ void __launch_bounds__(LIN_THREADS) linear_simt_kernel(const LinearParams p)
{
    __shared__ float a_s[LIN_BK][LIN_BM + 4];
    __shared__ float w_s[LIN_BK][LIN_BN + 4];
    const int tid = threadIdx.x;
    const int64_t M = p.B * p.S;
    const int64_t m0 = (int64_t)blockIdx.y * LIN_BM, n0 = (int64_t)blockIdx.x * LIN_BN;
    const int tx = tid & 15, ty = tid >> 4;          // 16 x 16 threads, 4 x 4 outputs each
    float acc[4][4] = {};
    for (int64_t k0 = 0; k0 < p.K; k0 += LIN_BK) {
        // tile loads: thread -> (row = tid / 4, four consecutive k)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int row = tid >> 2, kk = (tid & 3) * 4 + i;
            const int64_t m = m0 + row, n = n0 + row, k = k0 + kk;
            a_s[kk][row] = (m < M && k < p.K) ? __ldg(p.x + lin_index(m, k, p.S, p.K, p.heads_in)) : 0.f;
            w_s[kk][row] = (n < p.N && k < p.K) ? __ldg(p.w + n * p.K + k) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < LIN_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = a_s[kk][ty * 4 + i]; b[i] = w_s[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t n = n0 + tx * 4 + j;
            if (n >= p.N) continue;
            const float v = p.bias ? acc[i][j] + __ldg(p.bias + n) : acc[i][j];
            p.out[lin_index(m, n, p.S, p.N, p.heads_out)] = v;
        }
    }
}

}  // namespace txb
