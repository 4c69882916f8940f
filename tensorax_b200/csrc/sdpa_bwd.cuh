// SDPA backward on sm_100a: dQ, dK, dV from Q, K, V (fp16), dO and the forward's row statistics.
//
// The math is the reference's autograd rule for 'scaled_dot_product_attention'
// (tensorax/tensor.py:806-827):
//     P  = softmax(Q K^T * scale [+ mask])          dV = P^T dO
//     dP = dO V^T                                   D  = rowsum(dP o P)  (= rowsum(dO o O))
//     dS = P o (dP - D) * scale                     dQ = dS K,   dK = dS^T Q
// done flash-style: P is rebuilt tile by tile from the forward's per-row log-sum-exp, nothing of
// size Sq x Sk ever reaches global memory.  Two kernels, so that no gradient needs atomics and the
// result is bitwise reproducible:
//
//   sdpa_bwd_dq_kernel   one CTA = one 128-row query tile; loops over key tiles:
//                        S = Q K^T, dP = dO V^T (SS MMAs) -> registers -> dS (fp16, TMEM) ->
//                        dQ += dS K (TS MMA, K read MN-major from the same stage)
//   sdpa_bwd_dkv_kernel  one CTA = one 128-row key tile of one K/V head; loops over the query heads
//                        of its group and their query tiles: S^T = K Q^T, dP^T = V dO^T ->
//                        registers -> P^T, dS^T (fp16, TMEM) -> dV += P^T dO, dK += dS^T Q
//
// Roles per CTA as in the forward kernel: warp 0 TMA producer, warp 1 MMA issuer and TMEM owner,
// then one or two row warpgroups (4 warps each, one thread per TMEM lane; two warpgroups split a
// tile's columns).  Head dims 64, 128 and 256 (at 256 the dK/dV kernel runs two CTAs per key tile,
// each accumulating half of the gradient columns).  Every wait is bounded (ptx::mbar_wait); a wait that runs out
// sets the CTA's abort flag and a code in the device status word.
#pragma once

#include "ptx.cuh"
#include "sdpa_tc.cuh"

namespace txb {

enum : int { BWD_ERR_PRODUCER = 22, BWD_ERR_MMA = 23, BWD_ERR_ROWS = 24 };

struct BwdParams {
    const float *lse;         // [B,Hq,Sq] log2-domain row statistic written by the forward
    const float *delta;       // [B,Hq,Sq] rowsum(dO o O)
    const int32_t *kv_lens;   // optional [B]
    float *dq, *dk, *dv;      // [B,Hq,Sq,D], [B,Hkv,Sk,D], [B,Hkv,Sk,D] fp32
    int *status;
    int Hq, Hkv, Sq, Sk;
    int causal;
    float scale;              // 1/sqrt(d)
    float scale_log2;         // scale * log2(e)
    // Launch order of the 1-D grids (as in the forward's two-tile kernel): slabs are walked in groups, inside a
    // group every slab's longest items first.  *_q: the dQ kernel (slab = (batch, query head), item = query tile);
    // *_k: the dK/dV kernel (slab = (batch, K/V head), item = key tile; its ZS column parts stay side by side).
    int group_q, items_q, slabs_q;
    int group_k, items_k, slabs_k;
};

// ------------------------------------------------------------------ preprocess
// dO fp32 -> fp16 (MMA operand) and delta = rowsum(dO o O); one warp per row.
template <typename OT>
__global__ void sdpa_bwd_prep_kernel(const float *__restrict__ dout, const OT *__restrict__ out,
                                     __half *__restrict__ dout_h, float *__restrict__ delta, int64_t rows, int d)
{
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float *g = dout + row * d;
    const OT *o = out + row * d;
    __half *gh = dout_h + row * d;
    float acc = 0.f;
    for (int c = lane * 2; c < d; c += 64) {
        const float2 gv = *reinterpret_cast<const float2 *>(g + c);
        float ox, oy;
        if constexpr (sizeof(OT) == 2) {
            const __half2 hv = *reinterpret_cast<const __half2 *>(o + c);
            ox = __low2float(hv); oy = __high2float(hv);
        } else {
            const float2 ov = *reinterpret_cast<const float2 *>(o + c);
            ox = ov.x; oy = ov.y;
        }
        acc = fmaf(gv.x, ox, acc);
        acc = fmaf(gv.y, oy, acc);
        *reinterpret_cast<__half2 *>(gh + c) = __floats2half2_rn(gv.x, gv.y);
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
    if (lane == 0) delta[row] = acc;
}

// ------------------------------------------------------------------ dQ
// WGS: row warpgroups (4 warps, one thread per TMEM lane each); with 2, each takes half of a tile's columns.
// NS / NSV: depth of the K / V ring.  A K stage is read twice (S = Q K^T, later dQ += dS K) and only
// then freed, so its ring is one deeper than V's, whose stage goes back right after dP = dO V^T.
template <int D_, int BN_, int NS_, int WGS_ = 1, int NSV_ = 2>
struct BwdDqCfg {
    static constexpr int D = D_, BN = BN_, NS = NS_, NSV = NSV_, BM = 128, WGS = WGS_;
    static constexpr int CW = BN / WGS;                      // tile columns per warpgroup
    static constexpr int THREADS = 64 + 128 * WGS;
    static constexpr int KP = D / 64;
    static constexpr uint32_t Q_BYTES = BM * D * 2;          // Q tile, dO tile
    static constexpr uint32_t KV_BYTES = BN * D * 2;         // one K or V stage
    static constexpr uint32_t KV_PANEL = BN * 128;
    static constexpr uint32_t OFF_Q = 0, OFF_DO = Q_BYTES, OFF_K = 2 * Q_BYTES, OFF_V = OFF_K + NS * KV_BYTES;
    static constexpr uint32_t OFF_BAR = OFF_V + NSV * KV_BYTES;
    // barriers: qdo_full, s_full, dp_full, s_free, ds_full, dq_done, k_full/k_empty[NS], v_full/v_empty[NSV]
    static constexpr int N_BARS = 6 + 2 * NS + 2 * NSV;
    static constexpr uint32_t OFF_TMEM = OFF_BAR + N_BARS * 8;
    static constexpr uint32_t OFF_ABORT = OFF_TMEM + 4;
    static constexpr uint32_t SMEM_BYTES = ((OFF_ABORT + 4 + 127) / 128) * 128;
    // tensor memory: S [BN] | dP [BN] | dQ [D] | dS fp16 pairs [BN/2]
    static constexpr uint32_t COL_S = 0, COL_DP = BN, COL_DQ = 2 * BN, COL_DS = 2 * BN + D;
    static constexpr uint32_t COLS_USED = 2 * BN + D + BN / 2;
    static constexpr uint32_t TMEM_COLS = COLS_USED <= 256 ? 256 : 512;
    static constexpr int CTAS_PER_SM = (SMEM_BYTES <= 115712 && TMEM_COLS <= 256) ? 2 : 1;
    static_assert(D % 64 == 0 && CW % 32 == 0 && (D / 32) % WGS == 0 && COLS_USED <= 512 && SMEM_BYTES <= 232448,
                  "tile shape");
};

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, Cfg::CTAS_PER_SM)
sdpa_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                   const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                   const BwdParams p)
{
    constexpr int D = Cfg::D, BN = Cfg::BN, NS = Cfg::NS, NSV = Cfg::NSV, BM = Cfg::BM;
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = ptx::smem_u32(smem);
    const uint32_t q_s = sbase + Cfg::OFF_Q, do_s = sbase + Cfg::OFF_DO, k_s = sbase + Cfg::OFF_K,
                   v_s = sbase + Cfg::OFF_V;
    const uint32_t bar0 = sbase + Cfg::OFF_BAR;
    const uint32_t qdo_full = bar0, s_full = bar0 + 8, dp_full = bar0 + 16, s_free = bar0 + 24,
                   ds_full = bar0 + 32, dq_done = bar0 + 40;
    const uint32_t k_full = bar0 + 48, k_empty = k_full + 8 * NS, v_full = k_empty + 8 * NS,
                   v_empty = v_full + 8 * NSV;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + Cfg::OFF_TMEM);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + Cfg::OFF_ABORT);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // work item: group-major, then longest first over all slabs of the group (late causal query tiles walk most keys)
    const int span = p.group_q * p.items_q;
    const int grp = (int)blockIdx.x / span, rem = (int)blockIdx.x % span;
    const int in_grp = min(p.group_q, p.slabs_q - grp * p.group_q);
    const int q_tile = p.items_q - 1 - rem / in_grp;
    const int q0 = q_tile * BM;
    const int bh = grp * p.group_q + rem % in_grp;
    const int b = bh / p.Hq, h = bh % p.Hq;
    const int kvh = b * p.Hkv + h / (p.Hq / p.Hkv);
    int kv_limit = p.Sk;
    if (p.kv_lens) kv_limit = min(kv_limit, max(p.kv_lens[b], 0));
    int kv_end = kv_limit;
    if (p.causal) kv_end = min(kv_end, q0 + BM);
    const int n_tiles = (kv_end + BN - 1) / BN;

    if (tid == 0) {
        *abort_flag = 0;
        ptx::mbar_init(qdo_full, 1);
        ptx::mbar_init(s_full, 1);
        ptx::mbar_init(dp_full, 1);
        ptx::mbar_init(s_free, 4 * Cfg::WGS);
        ptx::mbar_init(ds_full, 4 * Cfg::WGS);
        ptx::mbar_init(dq_done, 1);
        for (int s = 0; s < NS; ++s) {
            ptx::mbar_init(k_full + 8 * s, 1);
            ptx::mbar_init(k_empty + 8 * s, 1);
        }
        for (int s = 0; s < NSV; ++s) {
            ptx::mbar_init(v_full + 8 * s, 1);
            ptx::mbar_init(v_empty + 8 * s, 1);
        }
        ptx::fence_mbar_init();
        if (sbase & 1023u) { *abort_flag = 1; atomicCAS(p.status, 0, TC_ERR_ALIGN); }
        if (*reinterpret_cast<volatile int *>(p.status) != 0) *abort_flag = 1;
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t *>(tmem_slot)), Cfg::TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const bool run = (*abort_flag == 0) && n_tiles > 0;

    if (warp == 0) {
        if (run) {
            const bool leader = ptx::elect_one();
            if (leader) {
                ptx::prefetch_tmap(&tm_q);
                ptx::prefetch_tmap(&tm_do);
                ptx::prefetch_tmap(&tm_k);
                ptx::prefetch_tmap(&tm_v);
                ptx::mbar_arrive_expect_tx(qdo_full, 2 * Cfg::Q_BYTES);
#pragma unroll
                for (int pn = 0; pn < Cfg::KP; ++pn) {
                    ptx::tma_load_3d(q_s + pn * (BM * 128), &tm_q, qdo_full, pn * 64, q0, bh);
                    ptx::tma_load_3d(do_s + pn * (BM * 128), &tm_do, qdo_full, pn * 64, q0, bh);
                }
            }
            __syncwarp();
            bool ok = true;
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int s = j % NS;
                const uint32_t ph = (uint32_t)(j / NS) & 1u;
                ok = ptx::mbar_wait(k_empty + 8 * s, ph ^ 1u, abort_flag);
                if (!ok) break;
                if (leader) {
                    ptx::mbar_arrive_expect_tx(k_full + 8 * s, Cfg::KV_BYTES);
#pragma unroll
                    for (int pn = 0; pn < Cfg::KP; ++pn)
                        ptx::tma_load_3d(k_s + s * Cfg::KV_BYTES + pn * Cfg::KV_PANEL, &tm_k, k_full + 8 * s,
                                         pn * 64, j * BN, kvh);
                }
                __syncwarp();
                const int sv_ = j % NSV;
                const uint32_t phv = (uint32_t)(j / NSV) & 1u;
                ok = ptx::mbar_wait(v_empty + 8 * sv_, phv ^ 1u, abort_flag);
                if (!ok) break;
                if (leader) {
                    ptx::mbar_arrive_expect_tx(v_full + 8 * sv_, Cfg::KV_BYTES);
#pragma unroll
                    for (int pn = 0; pn < Cfg::KP; ++pn)
                        ptx::tma_load_3d(v_s + sv_ * Cfg::KV_BYTES + pn * Cfg::KV_PANEL, &tm_v, v_full + 8 * sv_,
                                         pn * 64, j * BN, kvh);
                }
                __syncwarp();
            }
            if (!ok && leader) { *abort_flag = 1; atomicCAS(p.status, 0, BWD_ERR_PRODUCER); }
        }
    } else if (warp == 1) {
        if (run) {
            const bool leader = ptx::elect_one();
            constexpr uint32_t idesc_s = ptx::idesc_f16(BM, BN, false);     // S, dP: both operands K-major
            constexpr uint32_t idesc_dq = ptx::idesc_f16(BM, D, true);      // dQ: B = K tile read MN-major
            constexpr uint32_t desc_hi = ptx::smem_desc_sw128_hi(1024);
            const uint32_t q_lo = ptx::smem_desc_sw128_lo(q_s, 16);
            const uint32_t do_lo = ptx::smem_desc_sw128_lo(do_s, 16);
            const uint32_t k_lo = ptx::smem_desc_sw128_lo(k_s, 16);
            const uint32_t v_lo = ptx::smem_desc_sw128_lo(v_s, 16);
            const uint32_t kmn_lo = ptx::smem_desc_sw128_lo(k_s, Cfg::KV_PANEL);
            const uint32_t t_s = tmem + Cfg::COL_S, t_dp = tmem + Cfg::COL_DP, t_dq = tmem + Cfg::COL_DQ,
                           t_ds = tmem + Cfg::COL_DS;
            bool ok = ptx::mbar_wait(qdo_full, 0, abort_flag);
            auto issue_s_dp = [&](int j) -> bool {
                const int s = j % NS;
                const uint32_t ph = (uint32_t)(j / NS) & 1u;
                if (!ptx::mbar_wait(k_full + 8 * s, ph, abort_flag)) return false;
                ptx::tc_fence_after_sync();
                const uint32_t st_off = (uint32_t)s * (Cfg::KV_BYTES >> 4);
                if (leader) {
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        const uint32_t a = ((kk >> 2) * (BM * 128) + (kk & 3) * 32) >> 4;
                        const uint32_t bb = ((kk >> 2) * Cfg::KV_PANEL + (kk & 3) * 32) >> 4;
                        ptx::mma_ss(t_s, ptx::make_desc(q_lo + a, desc_hi), ptx::make_desc(k_lo + st_off + bb, desc_hi),
                                    idesc_s, kk > 0);
                    }
                    ptx::mma_commit(s_full);
                }
                __syncwarp();
                const int sv_ = j % NSV;
                const uint32_t phv = (uint32_t)(j / NSV) & 1u;
                const uint32_t sv_off = (uint32_t)sv_ * (Cfg::KV_BYTES >> 4);
                if (!ptx::mbar_wait(v_full + 8 * sv_, phv, abort_flag)) return false;
                ptx::tc_fence_after_sync();
                if (leader) {
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        const uint32_t a = ((kk >> 2) * (BM * 128) + (kk & 3) * 32) >> 4;
                        const uint32_t bb = ((kk >> 2) * Cfg::KV_PANEL + (kk & 3) * 32) >> 4;
                        ptx::mma_ss(t_dp, ptx::make_desc(do_lo + a, desc_hi), ptx::make_desc(v_lo + sv_off + bb, desc_hi),
                                    idesc_s, kk > 0);
                    }
                    ptx::mma_commit(v_empty + 8 * sv_);
                    ptx::mma_commit(dp_full);
                }
                __syncwarp();
                return true;
            };
            if (ok) ok = issue_s_dp(0);
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (j + 1 < n_tiles) {
                    ok = ptx::mbar_wait(s_free, (uint32_t)j & 1u, abort_flag);
                    if (!ok) break;
                    ptx::tc_fence_after_sync();
                    ok = issue_s_dp(j + 1);
                    if (!ok) break;
                }
                ok = ptx::mbar_wait(ds_full, (uint32_t)j & 1u, abort_flag);
                if (!ok) break;
                ptx::tc_fence_after_sync();
                const int s = j % NS;
                const uint32_t ks = kmn_lo + (uint32_t)s * (Cfg::KV_BYTES >> 4);
                if (leader) {
#pragma unroll
                    for (int kk = 0; kk < BN / 16; ++kk)
                        ptx::mma_ts(t_dq, t_ds + kk * 8, ptx::make_desc(ks + kk * ((16 * 128) >> 4), desc_hi), idesc_dq,
                                    (j > 0 || kk > 0) ? 1u : 0u);
                    ptx::mma_commit(k_empty + 8 * s);
                    ptx::mma_commit(dq_done);
                }
                __syncwarp();
            }
            if (!ok && leader) { *abort_flag = 1; atomicCAS(p.status, 0, BWD_ERR_MMA); }
        }
    } else {
        constexpr int CW = Cfg::CW;
        const int quarter = warp & 3;
        const int wg = (warp - 2) >> 2;
        const int c0 = wg * CW;                     // this warpgroup's first column of every tile
        const int r = quarter * 32 + lane;
        const int row = q0 + r;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const uint32_t t_s = tmem + lane_base + Cfg::COL_S + c0, t_dp = tmem + lane_base + Cfg::COL_DP + c0,
                       t_dq = tmem + lane_base + Cfg::COL_DQ, t_ds = tmem + lane_base + Cfg::COL_DS + c0 / 2;
        const bool row_ok = row < p.Sq;
        // a row outside the problem gets lse = +inf: every P of it is 2^(-inf) = 0
        const float lse = row_ok ? p.lse[(size_t)bh * p.Sq + row] : INFINITY;
        const float delta = row_ok ? p.delta[(size_t)bh * p.Sq + row] : 0.f;
        bool ok = run;
        auto arrive_warp = [&](uint32_t bar) {
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar);
        };
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int kv0 = j * BN + c0;
            ok = ptx::mbar_wait(s_full, (uint32_t)j & 1u, abort_flag);
            if (!ok) break;
            ptx::tc_fence_after_sync();
            uint32_t sv[CW], dpv[CW];
            ptx::tmem_ld_cols<CW>(t_s, sv);
            ok = ptx::mbar_wait(dp_full, (uint32_t)j & 1u, abort_flag);
            if (!ok) break;
            ptx::tc_fence_after_sync();
            ptx::tmem_ld_cols<CW>(t_dp, dpv);
            ptx::tmem_wait_ld();
            ptx::reg_fence_cols<CW>(sv);
            ptx::reg_fence_cols<CW>(dpv);
            arrive_warp(s_free);
            const bool need_mask = (kv0 + CW > kv_limit) || (p.causal && (kv0 + CW - 1 > q0));
            const int lim = min(kv_limit - kv0, p.causal ? row - kv0 + 1 : CW);
            uint32_t pk[CW / 2];
            // packed fp32 pairs: x = s*c - lse, t = dP*scale - D*scale, dS = P*t
            const float2 c2 = make_float2(p.scale_log2, p.scale_log2), nl2 = make_float2(-lse, -lse);
            const float2 s2 = make_float2(p.scale, p.scale), nd2 = make_float2(-delta * p.scale, -delta * p.scale);
#pragma unroll
            for (int i = 0; i < CW; i += 2) {
                const float2 x = __ffma2_rn(make_float2(__uint_as_float(sv[i]), __uint_as_float(sv[i + 1])), c2, nl2);
                float2 pr = make_float2(ptx::ex2_approx(x.x), ptx::ex2_approx(x.y));
                if (need_mask) {                 // visible keys of this row are a prefix of the tile: [0, lim)
                    pr.x = ptx::zero_unless_lt(pr.x, i, lim);
                    pr.y = ptx::zero_unless_lt(pr.y, i + 1, lim);
                }
                const float2 tt = __ffma2_rn(make_float2(__uint_as_float(dpv[i]), __uint_as_float(dpv[i + 1])), s2, nd2);
                const float2 ds = __fmul2_rn(pr, tt);
                pk[i / 2] = ptx::pack_half2(ds.x, ds.y);
            }
            if (j > 0) {
                ok = ptx::mbar_wait(dq_done, (uint32_t)(j - 1) & 1u, abort_flag);   // dS of tile j-1 consumed
                if (!ok) break;
                ptx::tc_fence_after_sync();
            }
            ptx::tmem_st_cols<CW / 2>(t_ds, pk);
            ptx::tmem_wait_st();
            arrive_warp(ds_full);
        }
        if (run && ok) {
            ok = ptx::mbar_wait(dq_done, (uint32_t)(n_tiles - 1) & 1u, abort_flag);
            if (ok) {
                ptx::tc_fence_after_sync();
                float *grow = p.dq + ((size_t)bh * p.Sq + row) * D;
#pragma unroll
                for (int cc = 0; cc < D / 32 / Cfg::WGS; ++cc) {
                    const int c = cc * Cfg::WGS + wg;          // the warpgroups share the row's chunks
                    uint32_t o[32];
                    ptx::tmem_ld32(t_dq + c * 32, o);
                    ptx::tmem_wait_ld();
                    ptx::reg_fence32(o);
                    if (row_ok) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            *reinterpret_cast<float4 *>(grow + c * 32 + i) =
                                make_float4(__uint_as_float(o[i]), __uint_as_float(o[i + 1]), __uint_as_float(o[i + 2]),
                                            __uint_as_float(o[i + 3]));
                    }
                }
            }
        }
        if (run && !ok) { *abort_flag = 1; atomicCAS(p.status, 0, BWD_ERR_ROWS); }
        if (!run && *abort_flag == 0 && row_ok) {
            // no visible key: the forward row is 0/0, and so is its gradient
            float *grow = p.dq + ((size_t)bh * p.Sq + row) * D;
            for (int i = 0; i < D; ++i) grow[i] = __int_as_float(0x7fc00000);
        }
    }

    ptx::tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
        __syncthreads();
    }
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem, Cfg::TMEM_COLS);
    }
}

// ------------------------------------------------------------------ dK, dV
// PS_SMEM: P^T and dS^T are staged in shared memory (SS-form MMAs) instead of tensor memory, which
// brings the CTA down to 256 tensor-memory columns at d = 64 so that two CTAs share an SM.
// NS / NSD: depth of the Q / dO ring; both stages are read twice (K-major for S^T / dP^T, MN-major for
// dK / dV) and stay occupied until the second read is done.
// ZS: CTAs (side by side in the 1-D grid) that share one key tile, each accumulating D/ZS columns of dK and dV (both form the whole
// S^T and dP^T): at d = 256 the two accumulators of one CTA would need all 512 tensor-memory columns.
template <int D_, int BQ_, int NS_, int WGS_ = 1, bool PS_SMEM_ = false, int NSD_ = NS_, int ZS_ = 1>
struct BwdDkvCfg {
    static constexpr int D = D_, BQ = BQ_, NS = NS_, NSD = NSD_, BMK = 128, WGS = WGS_, ZS = ZS_;
    static constexpr int DA = D / ZS;                        // gradient columns this CTA accumulates
    static constexpr bool PS_SMEM = PS_SMEM_;
    static constexpr int CW = BQ / WGS;                      // tile columns (queries) per warpgroup
    static constexpr int THREADS = 64 + 128 * WGS;
    static constexpr int KP = D / 64;
    static constexpr uint32_t KV_BYTES = BMK * D * 2;        // resident K tile, V tile
    static constexpr uint32_t Q_BYTES = BQ * D * 2;          // one Q or dO stage
    static constexpr uint32_t Q_PANEL = BQ * 128;
    static constexpr uint32_t OFF_K = 0, OFF_V = KV_BYTES, OFF_Q = 2 * KV_BYTES, OFF_DO = OFF_Q + NS * Q_BYTES;
    static constexpr uint32_t PS_BYTES = PS_SMEM ? BMK * BQ * 2 : 0;  // P^T / dS^T tile when staged in shared memory
    static constexpr uint32_t OFF_PS = OFF_DO + NSD * Q_BYTES, OFF_DSS = OFF_PS + PS_BYTES;
    static constexpr uint32_t OFF_STAT = OFF_DSS + PS_BYTES;          // float lse[2][BQ], delta[2][BQ]
    static constexpr uint32_t OFF_BAR = OFF_STAT + 4 * BQ * 4;
    // barriers: kv_full, s_full, dp_full, s_free, pds_full, pds_done, q_full/q_empty[NS], do_full/do_empty[NSD]
    static constexpr int N_BARS = 6 + 2 * NS + 2 * NSD;
    static constexpr uint32_t OFF_TMEM = OFF_BAR + N_BARS * 8;
    static constexpr uint32_t OFF_ABORT = OFF_TMEM + 4;
    static constexpr uint32_t SMEM_BYTES = ((OFF_ABORT + 4 + 127) / 128) * 128;
    // tensor memory: S^T [BQ] | dP^T [BQ] | dK [D] | dV [D] | P^T fp16 [BQ/2] | dS^T fp16 [BQ/2]
    static constexpr uint32_t COL_S = 0, COL_DP = BQ, COL_DK = 2 * BQ, COL_DV = 2 * BQ + DA, COL_P = 2 * BQ + 2 * DA,
                              COL_DS = 2 * BQ + 2 * DA + BQ / 2;
    static constexpr uint32_t COLS_USED = (PS_SMEM ? 2 : 3) * BQ + 2 * DA;
    static constexpr uint32_t TMEM_COLS = COLS_USED <= 256 ? 256 : 512;
    static constexpr int CTAS_PER_SM = (SMEM_BYTES <= 115712 && TMEM_COLS <= 256) ? 2 : 1;
    static_assert(D % 64 == 0 && DA % 64 == 0 && CW % 32 == 0 && (DA / 32) % WGS == 0 && 2 * BQ <= 128 * WGS &&
                      COLS_USED <= 512 && SMEM_BYTES <= 232448 && (!PS_SMEM || BQ == 64), "tile shape");
    static_assert(NS >= 2 && NSD >= 2, "Q and dO stages are held from their first read to their second");
};

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, Cfg::CTAS_PER_SM)
sdpa_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                    const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                    const BwdParams p)
{
    constexpr int D = Cfg::D, DA = Cfg::DA, BQ = Cfg::BQ, NS = Cfg::NS, NSD = Cfg::NSD, BMK = Cfg::BMK;
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = ptx::smem_u32(smem);
    const uint32_t k_s = sbase + Cfg::OFF_K, v_s = sbase + Cfg::OFF_V, q_s = sbase + Cfg::OFF_Q,
                   do_s = sbase + Cfg::OFF_DO;
    float *stat = reinterpret_cast<float *>(smem + Cfg::OFF_STAT);   // [stage][0: -lse, 1: -delta*scale][BQ]
    const uint32_t bar0 = sbase + Cfg::OFF_BAR;
    const uint32_t kv_full = bar0, s_full = bar0 + 8, dp_full = bar0 + 16, s_free = bar0 + 24,
                   pds_full = bar0 + 32, pds_done = bar0 + 40;
    const uint32_t q_full = bar0 + 48, q_empty = q_full + 8 * NS, do_full = q_empty + 8 * NS,
                   do_empty = do_full + 8 * NSD;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + Cfg::OFF_TMEM);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + Cfg::OFF_ABORT);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // work item: column part fastest, then group-major and longest first over the group's slabs (with a causal
    // mask the FIRST key tiles are seen by most queries)
    const int item = (int)blockIdx.x / Cfg::ZS;
    const int span = p.group_k * p.items_k;
    const int grp = item / span, rem = item % span;
    const int in_grp = min(p.group_k, p.slabs_k - grp * p.group_k);
    const int key0 = (rem / in_grp) * BMK;
    const int col0 = ((int)blockIdx.x % Cfg::ZS) * DA;          // first dK / dV column of this CTA
    const int kvh = grp * p.group_k + rem % in_grp;             // b * Hkv + kv head
    const int b = kvh / p.Hkv;
    const int group = p.Hq / p.Hkv;
    const int bh0 = b * p.Hq + (kvh % p.Hkv) * group;           // first query head of the group
    int kv_limit = p.Sk;
    if (p.kv_lens) kv_limit = min(kv_limit, max(p.kv_lens[b], 0));
    const int nq = (p.Sq + BQ - 1) / BQ;
    // causal: query rows below the tile's first key see none of its keys
    const int i_start = p.causal ? min(key0 / BQ, nq) : 0;
    const int per_head = (key0 < kv_limit) ? nq - i_start : 0;  // a tile beyond the valid keys gets zero gradients
    const int n_it = per_head * group;

    if (tid == 0) {
        *abort_flag = 0;
        ptx::mbar_init(kv_full, 1);
        ptx::mbar_init(s_full, 1);
        ptx::mbar_init(dp_full, 1);
        ptx::mbar_init(s_free, 4 * Cfg::WGS);
        ptx::mbar_init(pds_full, 4 * Cfg::WGS);
        ptx::mbar_init(pds_done, 1);
        for (int s = 0; s < NS; ++s) {
            ptx::mbar_init(q_full + 8 * s, 1);
            ptx::mbar_init(q_empty + 8 * s, 1);
        }
        for (int s = 0; s < NSD; ++s) {
            ptx::mbar_init(do_full + 8 * s, 1);
            ptx::mbar_init(do_empty + 8 * s, 1);
        }
        ptx::fence_mbar_init();
        if (sbase & 1023u) { *abort_flag = 1; atomicCAS(p.status, 0, TC_ERR_ALIGN); }
        if (*reinterpret_cast<volatile int *>(p.status) != 0) *abort_flag = 1;
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t *>(tmem_slot)), Cfg::TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const bool run = (*abort_flag == 0) && n_it > 0;

    if (warp == 0) {
        if (run) {
            const bool leader = ptx::elect_one();
            if (leader) {
                ptx::prefetch_tmap(&tm_q);
                ptx::prefetch_tmap(&tm_do);
                ptx::prefetch_tmap(&tm_k);
                ptx::prefetch_tmap(&tm_v);
                ptx::mbar_arrive_expect_tx(kv_full, 2 * Cfg::KV_BYTES);
#pragma unroll
                for (int pn = 0; pn < Cfg::KP; ++pn) {
                    ptx::tma_load_3d(k_s + pn * (BMK * 128), &tm_k, kv_full, pn * 64, key0, kvh);
                    ptx::tma_load_3d(v_s + pn * (BMK * 128), &tm_v, kv_full, pn * 64, key0, kvh);
                }
            }
            __syncwarp();
            bool ok = true;
            for (int t = 0; t < n_it && ok; ++t) {
                const int bhq = bh0 + t / per_head;
                const int qr0 = (i_start + t % per_head) * BQ;
                const int s = t % NS;
                const uint32_t ph = (uint32_t)(t / NS) & 1u;
                ok = ptx::mbar_wait(q_empty + 8 * s, ph ^ 1u, abort_flag);
                if (!ok) break;
                if (leader) {
                    ptx::mbar_arrive_expect_tx(q_full + 8 * s, Cfg::Q_BYTES);
#pragma unroll
                    for (int pn = 0; pn < Cfg::KP; ++pn)
                        ptx::tma_load_3d(q_s + s * Cfg::Q_BYTES + pn * Cfg::Q_PANEL, &tm_q, q_full + 8 * s, pn * 64, qr0, bhq);
                }
                __syncwarp();
                const int sd = t % NSD;
                const uint32_t phd = (uint32_t)(t / NSD) & 1u;
                ok = ptx::mbar_wait(do_empty + 8 * sd, phd ^ 1u, abort_flag);
                if (!ok) break;
                if (leader) {
                    ptx::mbar_arrive_expect_tx(do_full + 8 * sd, Cfg::Q_BYTES);
#pragma unroll
                    for (int pn = 0; pn < Cfg::KP; ++pn)
                        ptx::tma_load_3d(do_s + sd * Cfg::Q_BYTES + pn * Cfg::Q_PANEL, &tm_do, do_full + 8 * sd, pn * 64, qr0,
                                         bhq);
                }
                __syncwarp();
            }
            if (!ok && leader) { *abort_flag = 1; atomicCAS(p.status, 0, BWD_ERR_PRODUCER); }
        }
    } else if (warp == 1) {
        if (run) {
            const bool leader = ptx::elect_one();
            constexpr uint32_t idesc_s = ptx::idesc_f16(BMK, BQ, false);    // S^T, dP^T: both operands K-major
            constexpr uint32_t idesc_g = ptx::idesc_f16(BMK, DA, true);     // dV, dK: B = dO / Q tile read MN-major
            constexpr uint32_t desc_hi = ptx::smem_desc_sw128_hi(1024);
            const uint32_t k_lo = ptx::smem_desc_sw128_lo(k_s, 16);
            const uint32_t v_lo = ptx::smem_desc_sw128_lo(v_s, 16);
            const uint32_t q_lo = ptx::smem_desc_sw128_lo(q_s, 16);
            const uint32_t do_lo = ptx::smem_desc_sw128_lo(do_s, 16);
            // MN-major reads start at this CTA's first 64-column panel
            const uint32_t pan0 = (uint32_t)(col0 / 64) * Cfg::Q_PANEL;
            const uint32_t qmn_lo = ptx::smem_desc_sw128_lo(q_s + pan0, Cfg::Q_PANEL);
            const uint32_t domn_lo = ptx::smem_desc_sw128_lo(do_s + pan0, Cfg::Q_PANEL);
            const uint32_t ps_lo = ptx::smem_desc_sw128_lo(sbase + Cfg::OFF_PS, 16);
            const uint32_t dss_lo = ptx::smem_desc_sw128_lo(sbase + Cfg::OFF_DSS, 16);
            const uint32_t t_s = tmem + Cfg::COL_S, t_dp = tmem + Cfg::COL_DP, t_dk = tmem + Cfg::COL_DK,
                           t_dv = tmem + Cfg::COL_DV, t_p = tmem + Cfg::COL_P, t_ds = tmem + Cfg::COL_DS;
            bool ok = ptx::mbar_wait(kv_full, 0, abort_flag);
            auto issue_s_dp = [&](int t) -> bool {
                const int s = t % NS;
                const uint32_t ph = (uint32_t)(t / NS) & 1u;
                const uint32_t st_off = (uint32_t)s * (Cfg::Q_BYTES >> 4);
                if (!ptx::mbar_wait(q_full + 8 * s, ph, abort_flag)) return false;
                ptx::tc_fence_after_sync();
                if (leader) {
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        const uint32_t a = ((kk >> 2) * (BMK * 128) + (kk & 3) * 32) >> 4;
                        const uint32_t bb = ((kk >> 2) * Cfg::Q_PANEL + (kk & 3) * 32) >> 4;
                        ptx::mma_ss(t_s, ptx::make_desc(k_lo + a, desc_hi), ptx::make_desc(q_lo + st_off + bb, desc_hi),
                                    idesc_s, kk > 0);
                    }
                    ptx::mma_commit(s_full);
                }
                __syncwarp();
                const int sd = t % NSD;
                const uint32_t phd = (uint32_t)(t / NSD) & 1u;
                const uint32_t sd_off = (uint32_t)sd * (Cfg::Q_BYTES >> 4);
                if (!ptx::mbar_wait(do_full + 8 * sd, phd, abort_flag)) return false;
                ptx::tc_fence_after_sync();
                if (leader) {
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        const uint32_t a = ((kk >> 2) * (BMK * 128) + (kk & 3) * 32) >> 4;
                        const uint32_t bb = ((kk >> 2) * Cfg::Q_PANEL + (kk & 3) * 32) >> 4;
                        ptx::mma_ss(t_dp, ptx::make_desc(v_lo + a, desc_hi), ptx::make_desc(do_lo + sd_off + bb, desc_hi),
                                    idesc_s, kk > 0);
                    }
                    ptx::mma_commit(dp_full);
                }
                __syncwarp();
                return true;
            };
            if (ok) ok = issue_s_dp(0);
            for (int t = 0; t < n_it && ok; ++t) {
                if (t + 1 < n_it) {
                    ok = ptx::mbar_wait(s_free, (uint32_t)t & 1u, abort_flag);
                    if (!ok) break;
                    ptx::tc_fence_after_sync();
                    ok = issue_s_dp(t + 1);
                    if (!ok) break;
                }
                ok = ptx::mbar_wait(pds_full, (uint32_t)t & 1u, abort_flag);
                if (!ok) break;
                ptx::tc_fence_after_sync();
                const int s = t % NS, sd = t % NSD;
                const uint32_t st_off = (uint32_t)s * (Cfg::Q_BYTES >> 4), sd_off = (uint32_t)sd * (Cfg::Q_BYTES >> 4);
                if (leader) {
#pragma unroll
                    for (int kk = 0; kk < BQ / 16; ++kk) {
                        const uint64_t bdesc = ptx::make_desc(domn_lo + sd_off + kk * ((16 * 128) >> 4), desc_hi);
                        const uint32_t acc = (t > 0 || kk > 0) ? 1u : 0u;
                        if constexpr (Cfg::PS_SMEM)
                            ptx::mma_ss(t_dv, ptx::make_desc(ps_lo + ((kk * 32) >> 4), desc_hi), bdesc, idesc_g, acc);
                        else
                            ptx::mma_ts(t_dv, t_p + kk * 8, bdesc, idesc_g, acc);
                    }
                    ptx::mma_commit(do_empty + 8 * sd);
#pragma unroll
                    for (int kk = 0; kk < BQ / 16; ++kk) {
                        const uint64_t bdesc = ptx::make_desc(qmn_lo + st_off + kk * ((16 * 128) >> 4), desc_hi);
                        const uint32_t acc = (t > 0 || kk > 0) ? 1u : 0u;
                        if constexpr (Cfg::PS_SMEM)
                            ptx::mma_ss(t_dk, ptx::make_desc(dss_lo + ((kk * 32) >> 4), desc_hi), bdesc, idesc_g, acc);
                        else
                            ptx::mma_ts(t_dk, t_ds + kk * 8, bdesc, idesc_g, acc);
                    }
                    ptx::mma_commit(q_empty + 8 * s);
                    ptx::mma_commit(pds_done);
                }
                __syncwarp();
            }
            if (!ok && leader) { *abort_flag = 1; atomicCAS(p.status, 0, BWD_ERR_MMA); }
        }
    } else {
        constexpr int CW = Cfg::CW;
        const int quarter = warp & 3;
        const int wg = (warp - 2) >> 2;
        const int c0 = wg * CW;                     // this warpgroup's first query column of every tile
        const int r = quarter * 32 + lane;          // key row inside the tile = TMEM lane
        const int key = key0 + r;
        const int st = tid - 64;                    // 0 .. 128*WGS-1 among the row warps
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const uint32_t t_s = tmem + lane_base + Cfg::COL_S + c0, t_dp = tmem + lane_base + Cfg::COL_DP + c0,
                       t_dk = tmem + lane_base + Cfg::COL_DK, t_dv = tmem + lane_base + Cfg::COL_DV,
                       t_p = tmem + lane_base + Cfg::COL_P + c0 / 2, t_ds = tmem + lane_base + Cfg::COL_DS + c0 / 2;
        const bool key_ok = key < kv_limit;
        bool ok = run;
        auto arrive_warp = [&](uint32_t bar) {
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar);
        };
        for (int t = 0; t < n_it; ++t) {
            // All row warps take every iteration's named barrier, also after a failed wait, so
            // that none of them is left behind at it.
            const int bhq = bh0 + t / per_head;
            const int qr0 = (i_start + t % per_head) * BQ;
            float *st_lse = stat + (t & 1) * 2 * BQ, *st_delta = st_lse + BQ;
            if (st < BQ) {
                const int qrow = qr0 + st;
                st_lse[st] = qrow < p.Sq ? -p.lse[(size_t)bhq * p.Sq + qrow] : -INFINITY;   // -lse; -inf: P = 0
            } else if (st < 2 * BQ) {
                const int qrow = qr0 + st - BQ;
                st_delta[st - BQ] = qrow < p.Sq ? -p.scale * p.delta[(size_t)bhq * p.Sq + qrow] : 0.f;   // -D*scale
            }
            if constexpr (Cfg::WGS == 1) asm volatile("bar.sync 1, 128;" ::: "memory");
            else asm volatile("bar.sync 1, 256;" ::: "memory");
            if (!ok) continue;
            ok = ptx::mbar_wait(s_full, (uint32_t)t & 1u, abort_flag);
            if (!ok) continue;
            ptx::tc_fence_after_sync();
            uint32_t sv[CW], dpv[CW];
            ptx::tmem_ld_cols<CW>(t_s, sv);
            ok = ptx::mbar_wait(dp_full, (uint32_t)t & 1u, abort_flag);
            if (!ok) continue;
            ptx::tc_fence_after_sync();
            ptx::tmem_ld_cols<CW>(t_dp, dpv);
            ptx::tmem_wait_ld();
            ptx::reg_fence_cols<CW>(sv);
            ptx::reg_fence_cols<CW>(dpv);
            arrive_warp(s_free);
            const int qc0 = qr0 + c0;               // first query of this warpgroup's columns
            const bool need_mask = p.causal && (key0 + BMK - 1 > qc0);
            const int key_lo = key - qc0 - 1;
            uint32_t pp[CW / 2], pd[CW / 2];
            const float2 c2 = make_float2(p.scale_log2, p.scale_log2), s2 = make_float2(p.scale, p.scale);
#pragma unroll
            for (int i = 0; i < CW; i += 2) {
                // packed fp32 pairs; the two queries' statistics sit side by side in shared memory
                const float2 l2 = *reinterpret_cast<const float2 *>(st_lse + c0 + i);
                const float2 dl = *reinterpret_cast<const float2 *>(st_delta + c0 + i);
                const float2 x = __ffma2_rn(make_float2(__uint_as_float(sv[i]), __uint_as_float(sv[i + 1])), c2, l2);
                float2 pr = make_float2(ptx::ex2_approx(x.x), ptx::ex2_approx(x.y));
                if (!key_ok) pr = make_float2(0.f, 0.f);
                if (need_mask) {                 // query qc0 + i sees this key when key <= qc0 + i
                    pr.x = ptx::zero_unless_lt(pr.x, key_lo, i);
                    pr.y = ptx::zero_unless_lt(pr.y, key_lo, i + 1);
                }
                const float2 tt = __ffma2_rn(make_float2(__uint_as_float(dpv[i]), __uint_as_float(dpv[i + 1])), s2,
                                             dl);
                const float2 ds = __fmul2_rn(pr, tt);
                pp[i / 2] = ptx::pack_half2(pr.x, pr.y);
                pd[i / 2] = ptx::pack_half2(ds.x, ds.y);
            }
            if (t > 0) {
                ok = ptx::mbar_wait(pds_done, (uint32_t)(t - 1) & 1u, abort_flag);
                if (!ok) continue;
                ptx::tc_fence_after_sync();
            }
            if constexpr (Cfg::PS_SMEM) {
                // row r of the [128 keys][64 queries] tile: 128 bytes = 8 chunks of 8 halves, chunk ^= r % 8
                const uint32_t prow = sbase + Cfg::OFF_PS + (uint32_t)r * 128, drow = sbase + Cfg::OFF_DSS + (uint32_t)r * 128;
#pragma unroll
                for (int ch = 0; ch < 8; ++ch) {
                    const uint32_t sw = ((uint32_t)ch ^ (uint32_t)(r & 7)) << 4;
                    ptx::st_shared_v4(prow + sw, pp[ch * 4], pp[ch * 4 + 1], pp[ch * 4 + 2], pp[ch * 4 + 3]);
                    ptx::st_shared_v4(drow + sw, pd[ch * 4], pd[ch * 4 + 1], pd[ch * 4 + 2], pd[ch * 4 + 3]);
                }
                ptx::fence_proxy_async_smem();
            } else {
                ptx::tmem_st_cols<CW / 2>(t_p, pp);
                ptx::tmem_st_cols<CW / 2>(t_ds, pd);
                ptx::tmem_wait_st();
            }
            arrive_warp(pds_full);
        }
        const size_t gbase = ((size_t)kvh * p.Sk + key) * D + col0;
        if (run && ok) {
            ok = ptx::mbar_wait(pds_done, (uint32_t)(n_it - 1) & 1u, abort_flag);
            if (ok) {
                ptx::tc_fence_after_sync();
#pragma unroll
                for (int cc = 0; cc < DA / 32 / Cfg::WGS; ++cc) {
                    const int c = cc * Cfg::WGS + wg;          // the warpgroups share the row's chunks
                    uint32_t o[32];
                    ptx::tmem_ld32(t_dk + c * 32, o);
                    ptx::tmem_wait_ld();
                    ptx::reg_fence32(o);
                    if (key < p.Sk) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            *reinterpret_cast<float4 *>(p.dk + gbase + c * 32 + i) =
                                make_float4(__uint_as_float(o[i]), __uint_as_float(o[i + 1]), __uint_as_float(o[i + 2]),
                                            __uint_as_float(o[i + 3]));
                    }
                    ptx::tmem_ld32(t_dv + c * 32, o);
                    ptx::tmem_wait_ld();
                    ptx::reg_fence32(o);
                    if (key < p.Sk) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            *reinterpret_cast<float4 *>(p.dv + gbase + c * 32 + i) =
                                make_float4(__uint_as_float(o[i]), __uint_as_float(o[i + 1]), __uint_as_float(o[i + 2]),
                                            __uint_as_float(o[i + 3]));
                    }
                }
            }
        }
        if (run && !ok) { *abort_flag = 1; atomicCAS(p.status, 0, BWD_ERR_ROWS); }
        if (!run && *abort_flag == 0 && key < p.Sk) {
            // no query sees these keys: zero gradients -- unless the batch element has no valid key at
            // all, where the forward rows are 0/0 and the reference's rule propagates NaN to every gradient
            const float fill = kv_limit == 0 ? __int_as_float(0x7fc00000) : 0.f;
            for (int i = 0; i < DA; i += 4) {
                *reinterpret_cast<float4 *>(p.dk + gbase + i) = make_float4(fill, fill, fill, fill);
                *reinterpret_cast<float4 *>(p.dv + gbase + i) = make_float4(fill, fill, fill, fill);
            }
        }
    }

    ptx::tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
        __syncthreads();
    }
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem, Cfg::TMEM_COLS);
    }
}

}  // namespace txb
