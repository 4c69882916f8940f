// Exact-fp32 flash-attention forward on CUDA cores (no tensor cores).
//
// This kernel backs the fp32 entry points (tensorax csrc/tensor_ops.h:170-194:
// sdpa_naive_cuda / sdpa_tiled_cuda / sdpa_flash_cuda / sdpa_optimized_flash_cuda /
// sdpa_mma_cuda when a mask or an unaligned shape is given) and every shape or
// mask form the tcgen05 kernel does not take (dense additive masks, ragged head
// dims, d_k != d_v).  All products and sums are fp32 FMAs and the exponential is
// expf, so results stay within 1e-5 of the reference CPU path
// (csrc/cpu/tensor_cpu.cpp:464-529), which the fp16-operand tensor-core variants
// of the reference cannot do.
//
// Semantics kept from the reference:
//   score = dot(q,k) * (1/sqrt(d_k)) + mask[b,h,i,j]        (tensor_cpu.cpp:491-496)
//   running max starts at -FLT_MAX, so a row whose every key is masked with -inf
//   ends with 0/0 = NaN                                      (tensor_cpu.cpp:489-515)
// Added (no reference counterpart; the dense mask forms cannot exist at
// S = 8192): implicit causal mask (key j visible to query i iff j <= i),
// per-batch key lengths, and grouped K/V heads (query head h reads K/V head
// h / (Hq/Hkv), as csrc/tensor_ops.cpp:145-154 replicates them).
//
// Tiling: one CTA = 32 query rows x one slice of up to 32*DVC value columns;
// keys are walked in tiles of 64, d_k in chunks of 64.  HBM traffic is K and V
// once per 32 query rows, served from L2 after the first touch.
#pragma once
#include <cuda_fp16.h>
#include <cfloat>
#include <cstdint>

namespace txb {

struct SimtParams {
    const void *q, *k, *v;   // [B,Hq,Sq,dk], [B,Hkv,Sk,dk], [B,Hkv,Sk,dv]
    const float *mask;       // optional dense additive [B,Hq,Sq,Sk]
    const int32_t *kv_lens;  // optional [B]
    void *out;               // [B,Hq,Sq,dv] fp32, or fp16 when out_f16
    int64_t B, Hq, Hkv, Sq, Sk, dk, dv;
    int causal;
    int out_f16;
    float scale;
    long long *prof;         // optional [32]: clock64 stamps of CTA (0,0,0), thread 0 (PROF instantiation only)
    const int *only_if = nullptr;   // optional device word: the launch does nothing while it is 0 (this kernel as the
                                    // stand-in behind a faster one that found it could not take the call)
};

// Stamps of the section profile (the counterpart of TX_TICK, tensorax csrc/cuda/profiling.cuh:20-51):
// consecutive differences are the time thread 0 of CTA (0,0,0) spent in a section.
enum SimtStamp : int {
    SIMT_T_START = 0,        // kernel entry
    SIMT_T_LOADED = 1,       // first Q / K chunk in shared memory
    SIMT_T_SCORES = 2,       // first key tile: Q K^T accumulated
    SIMT_T_PARKED = 3,       // first key tile: scaled, masked, written to shared memory
    SIMT_T_SOFTMAX = 4,      // first key tile: online softmax done
    SIMT_T_PV = 5,           // first key tile: O updated
    SIMT_T_LOOP_END = 6,     // all key tiles done
    SIMT_T_STORED = 7,       // output written
};

constexpr int SIMT_BR = 32;    // query rows per CTA
constexpr int SIMT_BC = 64;    // keys per tile
constexpr int SIMT_DKC = 64;   // d_k chunk held in shared memory
constexpr int SIMT_THREADS = 256;

__device__ __forceinline__ float simt_load(const float *p) { return __ldg(p); }
__device__ __forceinline__ float simt_load(const __half *p) { return __half2float(__ldg(p)); }

template <typename T, int DVC, bool PROF = false>
__global__ void __launch_bounds__(SIMT_THREADS)
sdpa_simt_kernel(const SimtParams p)
{
    auto stamp = [&](int i, bool when = true) {
        if constexpr (PROF) {
            if (when && p.prof && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0)
                p.prof[i] = clock64();
        }
    };
    if (p.only_if && *reinterpret_cast<const volatile int *>(p.only_if) == 0) return;
    stamp(SIMT_T_START);
    __shared__ float q_s[SIMT_BR][SIMT_DKC + 1];
    __shared__ float k_s[SIMT_BC][SIMT_DKC + 1];
    __shared__ float s_s[SIMT_BR][SIMT_BC + 1];
    __shared__ float alpha_s[SIMT_BR];
    __shared__ float l_s[SIMT_BR];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int64_t bh = blockIdx.z;                 // b*Hq + h
    const int64_t b = bh / p.Hq;
    const int64_t h = bh % p.Hq;
    const int64_t kvh = b * p.Hkv + h / (p.Hq / p.Hkv);
    const int64_t q0 = (int64_t)blockIdx.y * SIMT_BR;
    const int64_t dv0 = (int64_t)blockIdx.x * (32 * DVC);

    const T *Q = static_cast<const T *>(p.q) + bh * p.Sq * p.dk;
    const T *K = static_cast<const T *>(p.k) + kvh * p.Sk * p.dk;
    const T *V = static_cast<const T *>(p.v) + kvh * p.Sk * p.dv;
    const float *M = p.mask ? p.mask + bh * p.Sq * p.Sk : nullptr;

    int64_t key_end = p.Sk;
    if (p.kv_lens) key_end = min(key_end, (int64_t)max(p.kv_lens[b], 0));
    const int64_t len_b = key_end;
    if (p.causal) key_end = min(key_end, q0 + SIMT_BR);   // keys past the last row's diagonal

    // score phase mapping: 2 rows x 4 keys per thread
    const int sx = tid & 15, sy = tid >> 4;
    // output phase mapping: warp -> 4 rows, lane -> columns lane + 32c
    float o[4][DVC];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < DVC; ++c) o[r][c] = 0.f;

    float m_run[4], l_run[4];   // softmax state of the 4 rows this warp owns (kept by every lane)
#pragma unroll
    for (int r = 0; r < 4; ++r) { m_run[r] = -FLT_MAX; l_run[r] = 0.f; }

    for (int64_t k0 = 0; k0 < key_end; k0 += SIMT_BC) {
        float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        for (int64_t d0 = 0; d0 < p.dk; d0 += SIMT_DKC) {
            __syncthreads();   // previous users of q_s / k_s / s_s are done
            for (int i = tid; i < SIMT_BR * SIMT_DKC; i += SIMT_THREADS) {
                const int r = i / SIMT_DKC, d = i % SIMT_DKC;
                const int64_t row = q0 + r, col = d0 + d;
                q_s[r][d] = (row < p.Sq && col < p.dk) ? simt_load(Q + row * p.dk + col) : 0.f;
            }
            for (int i = tid; i < SIMT_BC * SIMT_DKC; i += SIMT_THREADS) {
                const int r = i / SIMT_DKC, d = i % SIMT_DKC;
                const int64_t key = k0 + r, col = d0 + d;
                k_s[r][d] = (key < p.Sk && col < p.dk) ? simt_load(K + key * p.dk + col) : 0.f;
            }
            __syncthreads();
            stamp(SIMT_T_LOADED, k0 == 0 && d0 == 0);
            const int dmax = (int)min((int64_t)SIMT_DKC, p.dk - d0);
            for (int d = 0; d < dmax; ++d) {
                const float qa = q_s[sy * 2][d], qb = q_s[sy * 2 + 1][d];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float kk = k_s[sx + 16 * c][d];
                    acc[0][c] = fmaf(qa, kk, acc[0][c]);
                    acc[1][c] = fmaf(qb, kk, acc[1][c]);
                }
            }
        }
        stamp(SIMT_T_SCORES, k0 == 0);
        // scale, add masks, park the scores
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row_l = sy * 2 + r;
            const int64_t row = q0 + row_l;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int key_l = sx + 16 * c;
                const int64_t key = k0 + key_l;
                float s = acc[r][c] * p.scale;
                if (M && row < p.Sq && key < p.Sk) s += M[row * p.Sk + key];
                const bool visible = key < len_b && (!p.causal || key <= row);
                s_s[row_l][key_l] = visible ? s : -INFINITY;
            }
        }
        __syncthreads();
        stamp(SIMT_T_PARKED, k0 == 0);
        // online softmax: warp w owns rows 4w..4w+3, lane covers keys lane, lane+32
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int row_l = warp * 4 + r;
            const float v0 = s_s[row_l][lane], v1 = s_s[row_l][lane + 32];
            float mx = fmaxf(v0, v1);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            const float m_new = fmaxf(m_run[r], mx);
            const float p0 = expf(v0 - m_new), p1 = expf(v1 - m_new);
            float sum = p0 + p1;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
            const float alpha = expf(m_run[r] - m_new);
            l_run[r] = l_run[r] * alpha + sum;
            m_run[r] = m_new;
            s_s[row_l][lane] = p0;
            s_s[row_l][lane + 32] = p1;
            if (lane == 0) alpha_s[row_l] = alpha;
        }
        __syncwarp();
        stamp(SIMT_T_SOFTMAX, k0 == 0);
        // O <- O*alpha + P V for the warp's own 4 rows (only this warp wrote them)
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const float a = alpha_s[warp * 4 + r];
#pragma unroll
            for (int c = 0; c < DVC; ++c) o[r][c] *= a;
        }
        const int kmax = (int)min((int64_t)SIMT_BC, p.Sk - k0);
        for (int j = 0; j < kmax; ++j) {
            float vv[DVC];
#pragma unroll
            for (int c = 0; c < DVC; ++c) {
                const int64_t col = dv0 + lane + 32 * c;
                vv[c] = col < p.dv ? simt_load(V + (k0 + j) * p.dv + col) : 0.f;
            }
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float pj = s_s[warp * 4 + r][j];
#pragma unroll
                for (int c = 0; c < DVC; ++c) o[r][c] = fmaf(pj, vv[c], o[r][c]);
            }
        }
        stamp(SIMT_T_PV, k0 == 0);
    }
    stamp(SIMT_T_LOOP_END);
    if (lane == 0)
#pragma unroll
        for (int r = 0; r < 4; ++r) l_s[warp * 4 + r] = l_run[r];
    __syncwarp();
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int64_t row = q0 + warp * 4 + r;
        if (row >= p.Sq) continue;
        const float l = l_s[warp * 4 + r];
#pragma unroll
        for (int c = 0; c < DVC; ++c) {
            const int64_t col = dv0 + lane + 32 * c;
            if (col < p.dv) {
                const float val = o[r][c] / l;                                    // l == 0 -> NaN, as the reference
                const int64_t idx = (bh * p.Sq + row) * p.dv + col;
                if (p.out_f16) static_cast<__half *>(p.out)[idx] = __float2half_rn(val);
                else static_cast<float *>(p.out)[idx] = val;
            }
        }
    }
    stamp(SIMT_T_STORED);
}

}  // namespace txb
