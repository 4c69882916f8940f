// fp32 linear layer on the tcgen05 tensor cores: out = x @ W^T + bias with fp32-grade accuracy
// from TF32 instructions (split-TF32), head split / merge folded into the TMA tensor maps.
//
// Same contract as linear_simt.cuh (reference: F.linear, tensorax/functional.py:105-110, with
// MultiHeadAttention's reshape + transpose, tensorax/nn/attention/layers.py:112-128); this is
// the tensor-core form for shapes whose dims are multiples of 32.
//
// A TF32 operand keeps 10 mantissa bits, so one TF32 product is only good to ~1e-3.  Every fp32
// value is therefore split once, in shared memory, into hi = its top 19 bits (exactly what the
// tensor core reads) and lo = x - hi (exact in fp32, |lo| < 2^-10 |x|), and the product is
// accumulated as hi*hi + hi*lo + lo*hi in the fp32 accumulator: the dropped lo*lo term and the
// rounding of lo are of order 2^-21 relative, which keeps the result within 1e-5 of the
// reference's fp32 matmul.
//
// The tensor core adds into its fp32 accumulator with truncation, so a long chain of
// accumulations drifts by about one ulp per step, always downwards in magnitude (measured:
// 2.3e-5 at K = 512 with every MMA on one accumulator).  The chain is therefore kept short: the
// two correction products go to an accumulator of their own (they are 2^-10 of the result, their
// drift does not matter) and the main product rotates over three accumulators; the epilogue adds
// the four partial sums with ordinary round-to-nearest fp32 adds.  4 x 128 columns = all of
// tensor memory, one CTA per SM.
//
// One CTA = 128 rows of one batch element x 128 output features.  Six warps:
//   warp 0     TMA producer: x tile [128 rows][32 k] and W tile [128 features][32 k] per stage
//              (fp32, 128-byte rows, 128-byte swizzle); x is addressed through a 4-D map
//              (d_head, S, heads, B), so reading a head-split tensor as [B, S, E] costs nothing
//   warps 2-5  split each landed stage element-wise into hi (in place) and lo (second copy);
//              afterwards the epilogue: accumulator -> registers, + bias, fp32 stores straight
//              into [B, S, N] or head-split [B, heads, S, N/heads]
//   warp 1     issues 3 MMAs (128x128x8, kind::tf32) per 8-wide k step and commits the stage back
// All waits are bounded as in the attention kernel.
#pragma once
#include "ptx.cuh"

namespace txb {

struct LinearTcParams {
    const float *bias;   // optional [N]
    float *out;
    int *status;
    int S, N, K;
    int dh_in;           // K / heads_in (K when the input is not head-split)
    int heads_out;       // 0 = [B, S, N]
};

constexpr int LTC_BM = 128, LTC_BN = 128, LTC_BK = 32, LTC_STAGES = 3, LTC_THREADS = 192;
constexpr uint32_t LTC_TILE = LTC_BM * LTC_BK * 4;                 // 16 KB: one x or W tile
constexpr uint32_t LTC_STAGE = 4 * LTC_TILE;                       // x, W, x_lo, W_lo
constexpr uint32_t LTC_OFF_BAR = LTC_STAGES * LTC_STAGE;           // full[], split[], empty[], acc_done
constexpr uint32_t LTC_OFF_TMEM = LTC_OFF_BAR + (3 * LTC_STAGES + 1) * 8;
constexpr uint32_t LTC_OFF_ABORT = LTC_OFF_TMEM + 4;
constexpr uint32_t LTC_SMEM = ((LTC_OFF_ABORT + 4 + 127) / 128) * 128;
enum : int { LTC_ERR_PRODUCER = 12, LTC_ERR_MMA = 13, LTC_ERR_SPLIT = 14 };

__global__ void __launch_bounds__(LTC_THREADS, 1)
linear_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                 const LinearTcParams p)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = ptx::smem_u32(smem);
    const uint32_t bar0 = sbase + LTC_OFF_BAR;
    const uint32_t full = bar0, split = bar0 + 8 * LTC_STAGES, empty = bar0 + 16 * LTC_STAGES,
                   acc_done = bar0 + 24 * LTC_STAGES;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + LTC_OFF_TMEM);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + LTC_OFF_ABORT);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * LTC_BN, s0 = blockIdx.y * LTC_BM, b = blockIdx.z;
    const int k_tiles = p.K / LTC_BK;

    if (tid == 0) {
        *abort_flag = 0;
        for (int s = 0; s < LTC_STAGES; ++s) {
            ptx::mbar_init(full + 8 * s, 1);
            ptx::mbar_init(split + 8 * s, 4);
            ptx::mbar_init(empty + 8 * s, 1);
        }
        ptx::mbar_init(acc_done, 1);
        ptx::fence_mbar_init();
        if ((sbase & 1023u) || *reinterpret_cast<volatile int *>(p.status) != 0) *abort_flag = 1;
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t *>(tmem_slot)), 512);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const bool run = *abort_flag == 0;

    if (warp == 0) {
        if (run) {
            const bool leader = ptx::elect_one();
            if (leader) { ptx::prefetch_tmap(&tm_x); ptx::prefetch_tmap(&tm_w); }
            bool ok = true;
            for (int kt = 0; kt < k_tiles && ok; ++kt) {
                const int s = kt % LTC_STAGES;
                const uint32_t ph = (uint32_t)(kt / LTC_STAGES) & 1u;
                ok = ptx::mbar_wait(empty + 8 * s, ph ^ 1u, abort_flag);
                if (!ok) break;
                if (leader) {
                    const int k = kt * LTC_BK;
                    ptx::mbar_arrive_expect_tx(full + 8 * s, 2 * LTC_TILE);
                    ptx::tma_load_4d(sbase + s * LTC_STAGE, &tm_x, full + 8 * s, k % p.dh_in, s0, k / p.dh_in, b);
                    ptx::tma_load_3d(sbase + s * LTC_STAGE + LTC_TILE, &tm_w, full + 8 * s, k, n0, 0);
                }
                __syncwarp();
            }
            if (!ok && leader) { *abort_flag = 1; atomicCAS(p.status, 0, LTC_ERR_PRODUCER); }
        }
    } else if (warp == 1) {
        if (run) {
            const bool leader = ptx::elect_one();
            constexpr uint32_t idesc = ptx::idesc_tf32(LTC_BM, LTC_BN);
            constexpr uint32_t desc_hi = ptx::smem_desc_sw128_hi(1024);
            const uint32_t base_lo = ptx::smem_desc_sw128_lo(sbase, 16);
            bool ok = true;
            for (int kt = 0; kt < k_tiles && ok; ++kt) {
                const int s = kt % LTC_STAGES;
                const uint32_t ph = (uint32_t)(kt / LTC_STAGES) & 1u;
                ok = ptx::mbar_wait(split + 8 * s, ph, abort_flag);
                if (!ok) break;
                ptx::tc_fence_after_sync();
                if (leader) {
                    const uint32_t st_lo = base_lo + (uint32_t)s * (LTC_STAGE >> 4);
#pragma unroll
                    for (int k8 = 0; k8 < LTC_BK / 8; ++k8) {
                        const uint32_t x_hi = st_lo + ((k8 * 32) >> 4), w_hi = x_hi + (LTC_TILE >> 4);
                        const uint32_t x_lo = x_hi + (2 * LTC_TILE >> 4), w_lo = x_hi + (3 * LTC_TILE >> 4);
                        // columns [0,384): three main accumulators used in rotation; [384,512): corrections
                        const uint32_t d_main = tmem + (uint32_t)(kt % 3) * 128, d_corr = tmem + 384;
                        ptx::mma_ss_tf32(d_corr, ptx::make_desc(x_lo, desc_hi), ptx::make_desc(w_hi, desc_hi), idesc,
                                         (kt > 0 || k8 > 0) ? 1u : 0u);
                        ptx::mma_ss_tf32(d_corr, ptx::make_desc(x_hi, desc_hi), ptx::make_desc(w_lo, desc_hi), idesc, 1u);
                        ptx::mma_ss_tf32(d_main, ptx::make_desc(x_hi, desc_hi), ptx::make_desc(w_hi, desc_hi), idesc,
                                         (kt >= 3 || k8 > 0) ? 1u : 0u);
                    }
                    ptx::mma_commit(empty + 8 * s);
                    if (kt == k_tiles - 1) ptx::mma_commit(acc_done);
                }
                __syncwarp();
            }
            if (!ok && leader) { *abort_flag = 1; atomicCAS(p.status, 0, LTC_ERR_MMA); }
        }
    } else {
        const int t = tid - 64;                       // 0..127
        bool ok = run;
        for (int kt = 0; kt < k_tiles && ok; ++kt) {
            const int s = kt % LTC_STAGES;
            const uint32_t ph = (uint32_t)(kt / LTC_STAGES) & 1u;
            ok = ptx::mbar_wait(full + 8 * s, ph, abort_flag);
            if (!ok) break;
            // element-wise, so the swizzled placement does not matter: hi in place, lo 32 KB further
            uint4 *tile = reinterpret_cast<uint4 *>(smem + s * LTC_STAGE);
#pragma unroll 4
            for (int i = t; i < (int)(2 * LTC_TILE / 16); i += 128) {
                uint4 x = tile[i], hi, lo;
                hi.x = x.x & 0xFFFFE000u; hi.y = x.y & 0xFFFFE000u; hi.z = x.z & 0xFFFFE000u; hi.w = x.w & 0xFFFFE000u;
                lo.x = __float_as_uint(__uint_as_float(x.x) - __uint_as_float(hi.x));
                lo.y = __float_as_uint(__uint_as_float(x.y) - __uint_as_float(hi.y));
                lo.z = __float_as_uint(__uint_as_float(x.z) - __uint_as_float(hi.z));
                lo.w = __float_as_uint(__uint_as_float(x.w) - __uint_as_float(hi.w));
                tile[i] = hi;
                tile[i + (2 * LTC_TILE / 16)] = lo;
            }
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(split + 8 * s);
        }
        if (ok && run) {
            ok = ptx::mbar_wait(acc_done, 0, abort_flag);
            if (ok) {
                ptx::tc_fence_after_sync();
                const int quarter = warp & 3;
                const int row = s0 + quarter * 32 + lane;
                const uint32_t t_acc = tmem + ((uint32_t)(quarter * 32) << 16);
                const int n_main = k_tiles < 3 ? k_tiles : 3;      // main accumulators that were written
#pragma unroll 1
                for (int c = 0; c < LTC_BN / 32; ++c) {
                    uint32_t v[32];
                    ptx::tmem_ld32(t_acc + 384 + c * 32, v);            // corrections first, then the main sums
                    ptx::tmem_wait_ld();
                    ptx::reg_fence32(v);
                    for (int a = 0; a < n_main; ++a) {
                        uint32_t u[32];
                        ptx::tmem_ld32(t_acc + a * 128 + c * 32, u);
                        ptx::tmem_wait_ld();
                        ptx::reg_fence32(u);
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) + __uint_as_float(u[i]));
                    }
                    const int n = n0 + c * 32;
                    if (row < p.S && n < p.N) {
                        float *dst;
                        if (p.heads_out > 0) {
                            const int dho = p.N / p.heads_out;
                            dst = p.out + (((size_t)b * p.heads_out + n / dho) * p.S + row) * dho + n % dho;
                        } else {
                            dst = p.out + ((size_t)b * p.S + row) * p.N + n;
                        }
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            float4 f = make_float4(__uint_as_float(v[i]), __uint_as_float(v[i + 1]),
                                                   __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
                            if (p.bias) {
                                const float4 bb = __ldg(reinterpret_cast<const float4 *>(p.bias + n + i));
                                f.x += bb.x; f.y += bb.y; f.z += bb.z; f.w += bb.w;
                            }
                            *reinterpret_cast<float4 *>(dst + i) = f;
                        }
                    }
                }
            }
        }
        if (run && !ok) { *abort_flag = 1; atomicCAS(p.status, 0, LTC_ERR_SPLIT); }
    }

    ptx::tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
        __syncthreads();
    }
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem, 512);
    }
}

}  // namespace txb
