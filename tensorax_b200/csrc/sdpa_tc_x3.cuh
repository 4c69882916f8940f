// fp32 flash-attention forward on the fp16 tensor cores of sm_100a: every fp32 operand is carried as the sum of
// two fp16 numbers (hi = rn(x), lo = rn(x - hi): 22 significand bits) and every product is three tcgen05 MMAs,
//     S  = Qhi Klo^T + Qlo Khi^T + Qhi Khi^T          O += Phi Vlo + Plo Vhi + Phi Vhi
// accumulated in fp32 in tensor memory (the lo*lo term is below fp32's own rounding).  It stands where the
// reference's fp32 kernels do (tensorax csrc/cuda/kernels/attn.cu:296-656 sdpa_kernel_mma and the naive / tiled /
// flash forms before it) for the calls that fit it: no dense mask, d_k = d_v in {64, 128}, |x| < 2^15 everywhere.
// The split pass that writes the hi / lo copies also checks the range and raises a device flag when a value does
// not fit; this kernel then returns at once and the exact CUDA-core kernel, launched behind it, does the work.
//
// One CTA per SM and 128-row query tile, 64 keys per tile:
//   warp 0        TMA producer: Q hi / lo once, then K hi / lo and V hi / lo of every key tile through an NS-deep ring
//   warp 1        issues the MMAs: QK^T of tile j+1 as soon as the softmax warps have S_j in registers, then PV of tile j
//   warps 2-3     idle
//   warps 4-7     softmax, thread = row = tensor-memory lane: fp32 online softmax with the exact running max
//                 (full-precision `ex2.approx`, no polynomial), P split into hi / lo in registers and stored to
//                 tensor memory as two fp16 operands; the row's rescale factor of the tile goes to shared memory
//   warps 8-11    accumulators, thread = row: O lives in REGISTERS.  Each tile's P V is a fresh tensor-memory
//                 accumulator (12 MMAs) that these warps fold in with O = O * alpha + PV, rounded to nearest.  The
//                 tensor core's own fp32 accumulation truncates, and carried over hundreds of key tiles that bias
//                 grows with the sequence length; twelve steps of it stay below fp32's rounding of the result.
//                 They also write the result (staged bulk tensor stores).
// Tensor memory: S 64 | Phi 32 | Plo 32 | PV_0 D | PV_1 D columns.
// Every mbarrier wait is bounded, as in the fp16 kernels.
#pragma once
#include "ptx.cuh"
#include "sdpa_tc.cuh"

namespace txb {

template <int D_, int NS_>
struct X3Cfg {
    static constexpr int D = D_, NS = NS_;
    static constexpr int BM = 128, BN = 64;
    static constexpr int THREADS = 384;
    // registers: producer / MMA warpgroup, softmax warpgroup, accumulator warpgroup (128 * (56 + 192 + 248) <= 384 * 168)
    static constexpr int REGS_LIGHT = 56, REGS_SOFTMAX = 192, REGS_ACC = 248;
    static constexpr int KP = D / 64;                      // 64-column panels per row
    static constexpr uint32_t Q_BYTES = BM * D * 2;        // one of hi / lo
    static constexpr uint32_t KV_BYTES = BN * D * 2;       // one of K hi, K lo, V hi, V lo
    static constexpr uint32_t KV_PANEL = BN * 128;
    static constexpr uint32_t OFF_QH = 0, OFF_QL = Q_BYTES;
    static constexpr uint32_t OFF_K = 2 * Q_BYTES;         // per stage: K hi | K lo
    static constexpr uint32_t OFF_V = OFF_K + NS * 2 * KV_BYTES;
    static constexpr uint32_t OFF_BAR = OFF_V + NS * 2 * KV_BYTES;
    // q_full s_full s_free p_full l_full pv_done[2] pv_free[2] alpha_full[4] k_full[NS] k_empty[NS] v_full[NS] v_empty[NS]
    static constexpr int N_BARS = 13 + 4 * NS;
    static constexpr uint32_t OFF_ALPHA = OFF_BAR + ((N_BARS * 8 + 15) / 16) * 16;   // [4][BM] rescale factors, then [BM] row sums
    static constexpr uint32_t OFF_TMEM = OFF_ALPHA + 5 * BM * 4;
    static constexpr uint32_t OFF_ABORT = OFF_TMEM + 4;
    static constexpr uint32_t SMEM_BYTES = ((OFF_ABORT + 4 + 127) / 128) * 128;
    static constexpr uint32_t COL_S = 0, COL_PH = BN, COL_PL = BN + BN / 2, COL_PV0 = 2 * BN, COL_PV1 = 2 * BN + D;
    static constexpr uint32_t TMEM_COLS = 512;
    static_assert(D == 64 || D == 128, "head dim");
    static_assert(2 * BN + 2 * D <= TMEM_COLS, "tensor memory");
    static_assert(SMEM_BYTES <= 232448, "more than the 227 KB a CTA may have");
    static_assert(Q_BYTES / 4 >= 4096, "a softmax warp stages its results in its quarter of the Q buffers");
};

struct X3Params {
    float *out;               // [B,Hq,Sq,D] fp32
    const int32_t *kv_lens;   // optional [B]
    const int *out_of_range;  // device word the split pass sets: nonzero = this kernel does nothing
    int *status;              // device word: 0 = ok, else first failing wait's code
    int Hq, Hkv, Sq, Sk;
    int causal;
    float scale_log2;         // (1/sqrt(d_k)) * log2(e)
    int group, n_tiles_q, BH; // work-item order, as in sdpa_tc_pair_kernel (query tiles in place of pairs)
};

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
sdpa_tc_x3_kernel(const __grid_constant__ CUtensorMap tm_qh, const __grid_constant__ CUtensorMap tm_ql,
                  const __grid_constant__ CUtensorMap tm_kh, const __grid_constant__ CUtensorMap tm_kl,
                  const __grid_constant__ CUtensorMap tm_vh, const __grid_constant__ CUtensorMap tm_vl,
                  const __grid_constant__ CUtensorMap tm_o, const X3Params p)
{
    constexpr int D = Cfg::D, BN = Cfg::BN, NS = Cfg::NS, BM = Cfg::BM;
    if (*reinterpret_cast<const volatile int *>(p.out_of_range) != 0) return;   // the exact kernel takes this call

    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = ptx::smem_u32(smem);
    const uint32_t qh_s = sbase + Cfg::OFF_QH, ql_s = sbase + Cfg::OFF_QL, k_s = sbase + Cfg::OFF_K, v_s = sbase + Cfg::OFF_V;
    const uint32_t bar0 = sbase + Cfg::OFF_BAR;
    const uint32_t q_full = bar0, s_full = bar0 + 8, s_free = bar0 + 16, p_full = bar0 + 24, l_full = bar0 + 32;
    const uint32_t pv_done = bar0 + 40, pv_free = bar0 + 56;     // one pair each: PV accumulator j & 1
    float *alpha_s = reinterpret_cast<float *>(smem + Cfg::OFF_ALPHA);       // [4][BM]: tile j's factors in slot j & 3
    float *l_s = alpha_s + 4 * BM;
    // Four slots and four barriers for the factors: the softmax warps reach tile j + 4 only after PV_{j+2} was
    // issued, which waited for the accumulator warps to be done with tile j -- so a slot is never rewritten, and
    // its barrier never a phase ahead, while its reader still needs it.
    const uint32_t alpha_full = bar0 + 72;
    const uint32_t k_full = bar0 + 104, k_empty = k_full + 8 * NS, v_full = k_empty + 8 * NS, v_empty = v_full + 8 * NS;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + Cfg::OFF_TMEM);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + Cfg::OFF_ABORT);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // work item: groups of slabs, each group's longest items first (see sdpa_tc_pair_kernel)
    const int span = p.group * p.n_tiles_q;
    const int grp = (int)blockIdx.x / span, rem = (int)blockIdx.x % span;
    const int slabs = min(p.group, p.BH - grp * p.group);
    const int q_tile = p.n_tiles_q - 1 - rem / slabs;
    const int q0 = q_tile * BM;
    const int bh = grp * p.group + rem % slabs;
    const int b = bh / p.Hq, h = bh % p.Hq;
    const int kvh = b * p.Hkv + h / (p.Hq / p.Hkv);

    int kv_limit = p.Sk;                                         // keys any row of this batch may see
    if (p.kv_lens) kv_limit = min(kv_limit, max(p.kv_lens[b], 0));
    const int kv_end = p.causal ? min(kv_limit, q0 + BM) : kv_limit;
    const int nt = (kv_end + BN - 1) / BN;

    auto load_kv = [&](uint32_t dst, const CUtensorMap *hi, const CUtensorMap *lo, uint32_t bar, int j) {
        ptx::mbar_arrive_expect_tx(bar, 2 * Cfg::KV_BYTES);
#pragma unroll
        for (int pn = 0; pn < Cfg::KP; ++pn) {
            ptx::tma_load_3d(dst + pn * Cfg::KV_PANEL, hi, bar, pn * 64, j * BN, kvh);
            ptx::tma_load_3d(dst + Cfg::KV_BYTES + pn * Cfg::KV_PANEL, lo, bar, pn * 64, j * BN, kvh);
        }
    };

    // warp 0 sets the barriers up and sends Q and the first key tile on their way before the CTA meets
    if (warp == 0) {
        if (lane == 0) {
            *abort_flag = 0;
            ptx::mbar_init(q_full, 1);
            ptx::mbar_init(s_full, 1);
            ptx::mbar_init(s_free, 4);                           // one arrival per softmax warp
            ptx::mbar_init(p_full, 4);
            ptx::mbar_init(l_full, 4);
            for (int t = 0; t < 2; ++t) {
                ptx::mbar_init(pv_done + 8 * t, 1);
                ptx::mbar_init(pv_free + 8 * t, 4);              // one arrival per accumulator warp
            }
            for (int t = 0; t < 4; ++t) ptx::mbar_init(alpha_full + 8 * t, 4);
            for (int s = 0; s < NS; ++s) {
                ptx::mbar_init(k_full + 8 * s, 1);
                ptx::mbar_init(k_empty + 8 * s, 1);
                ptx::mbar_init(v_full + 8 * s, 1);
                ptx::mbar_init(v_empty + 8 * s, 1);
            }
            ptx::fence_mbar_init();
            if (sbase & 1023u) {
                *abort_flag = 1;
                atomicCAS(p.status, 0, TC_ERR_ALIGN);
            } else if (nt > 0) {
                ptx::prefetch_tmap(&tm_qh);
                ptx::prefetch_tmap(&tm_kh);
                ptx::mbar_arrive_expect_tx(q_full, 2 * Cfg::Q_BYTES);
#pragma unroll
                for (int pn = 0; pn < Cfg::KP; ++pn) {
                    ptx::tma_load_3d(qh_s + pn * (BM * 128), &tm_qh, q_full, pn * 64, q0, bh);
                    ptx::tma_load_3d(ql_s + pn * (BM * 128), &tm_ql, q_full, pn * 64, q0, bh);
                }
                load_kv(k_s, &tm_kh, &tm_kl, k_full, 0);
                load_kv(v_s, &tm_vh, &tm_vl, v_full, 0);
            }
            if (*reinterpret_cast<volatile int *>(p.status) != 0) *abort_flag = 1;   // an earlier CTA gave up
        }
        __syncwarp();
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t *>(tmem_slot)), Cfg::TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const bool run = (*abort_flag == 0) && nt > 0;

    if (warp < 4) {
    ptx::setmaxnreg_dec<Cfg::REGS_LIGHT>();
    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (run) {
            const bool leader = ptx::elect_one();
            bool ok = true;
            for (int j = 1; j < nt && ok; ++j) {                 // key tile 0 went out before the meeting
                const int s = j % NS;
                const uint32_t ph = (uint32_t)(j / NS) & 1u;
                ok = ptx::mbar_wait(k_empty + 8 * s, ph ^ 1u, abort_flag);
                if (!ok) break;
                if (leader) load_kv(k_s + s * 2 * Cfg::KV_BYTES, &tm_kh, &tm_kl, k_full + 8 * s, j);
                __syncwarp();
                ok = ptx::mbar_wait(v_empty + 8 * s, ph ^ 1u, abort_flag);
                if (!ok) break;
                if (leader) load_kv(v_s + s * 2 * Cfg::KV_BYTES, &tm_vh, &tm_vl, v_full + 8 * s, j);
                __syncwarp();
            }
            if (!ok && leader) { *abort_flag = 1; atomicCAS(p.status, 0, TC_ERR_PRODUCER); }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // Three products per GEMM, the small ones first; the tensor pipe runs them in issue order.
        if (run) {
            const bool leader = ptx::elect_one();
            constexpr uint32_t idesc_qk = ptx::idesc_f16(BM, BN, false);
            constexpr uint32_t idesc_pv = ptx::idesc_f16(BM, D, true);
            constexpr uint32_t desc_hi = ptx::smem_desc_sw128_hi(1024);
            const uint32_t qh_lo = ptx::smem_desc_sw128_lo(qh_s, 16), ql_lo = ptx::smem_desc_sw128_lo(ql_s, 16);
            const uint32_t k_lo = ptx::smem_desc_sw128_lo(k_s, 16);
            const uint32_t v_lo = ptx::smem_desc_sw128_lo(v_s, Cfg::KV_PANEL);
            const uint32_t t_s = tmem + Cfg::COL_S;
            const uint32_t t_ph = tmem + Cfg::COL_PH, t_pl = tmem + Cfg::COL_PL;
            bool ok = true;
            auto issue_qk = [&](int j) -> bool {
                const int s = j % NS;
                const uint32_t ph = (uint32_t)(j / NS) & 1u;
                if (!ptx::mbar_wait(k_full + 8 * s, ph, abort_flag)) return false;
                ptx::tc_fence_after_sync();
                const uint32_t kh = k_lo + (uint32_t)s * ((2 * Cfg::KV_BYTES) >> 4), kl = kh + (Cfg::KV_BYTES >> 4);
                if (leader) {
#pragma unroll
                    for (int c = 0; c < 3; ++c) {
                        const uint32_t qa0 = c == 1 ? ql_lo : qh_lo;         // Qhi Klo, Qlo Khi, Qhi Khi
                        const uint32_t kb0 = c == 0 ? kl : kh;
#pragma unroll
                        for (int kk = 0; kk < D / 16; ++kk) {
                            const uint32_t qa = ((kk >> 2) * (BM * 128) + (kk & 3) * 32) >> 4;
                            const uint32_t kb = ((kk >> 2) * Cfg::KV_PANEL + (kk & 3) * 32) >> 4;
                            ptx::mma_ss(t_s, ptx::make_desc(qa0 + qa, desc_hi), ptx::make_desc(kb0 + kb, desc_hi),
                                        idesc_qk, (c > 0 || kk > 0) ? 1u : 0u);
                        }
                    }
                    ptx::mma_commit(k_empty + 8 * s);
                    ptx::mma_commit(s_full);
                }
                __syncwarp();
                return true;
            };
            // PV_j = P_j V_j into the fresh accumulator j & 1, once the accumulator warps have taken PV_{j-2} out of it
            auto issue_pv = [&](int j) -> bool {
                const int s = j % NS;
                const uint32_t ph = (uint32_t)(j / NS) & 1u;
                const int a = j & 1;
                if (!ptx::mbar_wait(v_full + 8 * s, ph, abort_flag)) return false;
                if (j >= 2 && !ptx::mbar_wait(pv_free + 8 * a, (uint32_t)((j - 2) >> 1) & 1u, abort_flag)) return false;
                if (!ptx::mbar_wait(p_full, (uint32_t)j & 1u, abort_flag)) return false;
                ptx::tc_fence_after_sync();
                const uint32_t vh = v_lo + (uint32_t)s * ((2 * Cfg::KV_BYTES) >> 4), vl = vh + (Cfg::KV_BYTES >> 4);
                const uint32_t t_pv = tmem + (a ? Cfg::COL_PV1 : Cfg::COL_PV0);
                if (leader) {
#pragma unroll
                    for (int c = 0; c < 3; ++c) {
                        const uint32_t pa0 = c == 1 ? t_pl : t_ph;           // Phi Vlo, Plo Vhi, Phi Vhi
                        const uint32_t vb0 = c == 0 ? vl : vh;
#pragma unroll
                        for (int kk = 0; kk < BN / 16; ++kk) {
                            const uint64_t bdesc = ptx::make_desc(vb0 + kk * ((16 * 128) >> 4), desc_hi);
                            ptx::mma_ts(t_pv, pa0 + kk * 8, bdesc, idesc_pv, (c > 0 || kk > 0) ? 1u : 0u);
                        }
                    }
                    ptx::mma_commit(v_empty + 8 * s);
                    ptx::mma_commit(pv_done + 8 * a);
                }
                __syncwarp();
                return true;
            };
            ok = ptx::mbar_wait(q_full, 0, abort_flag);
            if (ok) ok = issue_qk(0);
            for (int j = 0; j < nt && ok; ++j) {
                if (j + 1 < nt) {
                    ok = ptx::mbar_wait(s_free, (uint32_t)j & 1u, abort_flag);
                    if (ok) { ptx::tc_fence_after_sync(); ok = issue_qk(j + 1); }
                }
                if (ok) ok = issue_pv(j);
            }
            if (!ok && leader) { *abort_flag = 1; atomicCAS(p.status, 0, TC_ERR_MMA); }
        }
    }
    } else if (warp < 8) {
        ptx::setmaxnreg_inc<Cfg::REGS_SOFTMAX>();
        // ------------------------------------------------------------ softmax
        const int quarter = warp & 3;                    // tensor-memory lanes this warp may touch
        const int r = quarter * 32 + lane;               // row inside the tile
        const int row = q0 + r;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const uint32_t t_s = tmem + lane_base + Cfg::COL_S;
        const uint32_t t_ph = tmem + lane_base + Cfg::COL_PH, t_pl = tmem + lane_base + Cfg::COL_PL;
        const float scale = p.scale_log2;
        float m_run = -1.0e30f;    // finite stand-in for "no key seen yet"
        float l = 0.f;
        bool ok = run;
        auto arrive_warp = [&](uint32_t bar) {
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar);
        };
        for (int j = 0; j < nt && ok; ++j) {
            const int kv0 = j * BN;
            ok = ptx::mbar_wait(s_full, (uint32_t)j & 1u, abort_flag);
            if (!ok) break;
            ptx::tc_fence_after_sync();
            uint32_t sv[BN];
            ptx::tmem_ld_cols<BN>(t_s, sv);
            ptx::tmem_wait_ld();
            ptx::reg_fence_cols<BN>(sv);
            arrive_warp(s_free);                         // S belongs to the MMA warp again
            const bool need_mask = (kv0 + BN > kv_limit) || (p.causal && (kv0 + BN - 1 > q0));
            if (need_mask) {
                // visible keys of this row are a prefix of the tile: columns [0, lim)
                const int lim = min(kv_limit - kv0, p.causal ? row - kv0 + 1 : BN);
#pragma unroll
                for (int i = 0; i < BN; ++i) sv[i] = ptx::keep_if_below(sv[i], i, lim);
            }
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
            for (int i = 0; i < BN; i += 8) {
                mx0 = ptx::max3(mx0, __uint_as_float(sv[i]), __uint_as_float(sv[i + 1]));
                mx1 = ptx::max3(mx1, __uint_as_float(sv[i + 2]), __uint_as_float(sv[i + 3]));
                mx2 = ptx::max3(mx2, __uint_as_float(sv[i + 4]), __uint_as_float(sv[i + 5]));
                mx3 = ptx::max3(mx3, __uint_as_float(sv[i + 6]), __uint_as_float(sv[i + 7]));
            }
            const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
            const float m_next = fmaxf(m_run, mx * scale);          // exact running max: every p <= 1
            const float alpha = ptx::ex2_approx(m_run - m_next);
            m_run = m_next;
            alpha_s[(j & 3) * BM + r] = alpha;                      // for the accumulator thread of this row
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(alpha_full + 8 * (j & 3));
            // p = 2^(s*scale - m): a masked score is -inf and gives exactly 0
            const float2 scale2 = make_float2(scale, scale), negm2 = make_float2(-m_next, -m_next);
            float2 sum_a = make_float2(0.f, 0.f), sum_b = make_float2(0.f, 0.f);
            uint32_t pkh[BN / 2], pkl[BN / 2];
#pragma unroll
            for (int i = 0; i < BN; i += 4) {
                const float2 xa = __ffma2_rn(make_float2(__uint_as_float(sv[i]), __uint_as_float(sv[i + 1])), scale2, negm2);
                const float2 xb = __ffma2_rn(make_float2(__uint_as_float(sv[i + 2]), __uint_as_float(sv[i + 3])), scale2, negm2);
                const float2 ea = make_float2(ptx::ex2_approx(xa.x), ptx::ex2_approx(xa.y));
                const float2 eb = make_float2(ptx::ex2_approx(xb.x), ptx::ex2_approx(xb.y));
                sum_a = __fadd2_rn(sum_a, ea);
                sum_b = __fadd2_rn(sum_b, eb);
                const __half2 ha = __floats2half2_rn(ea.x, ea.y), hb = __floats2half2_rn(eb.x, eb.y);
                const float2 ba = __half22float2(ha), bb = __half22float2(hb);
                const __half2 la = __floats2half2_rn(ea.x - ba.x, ea.y - ba.y), lb = __floats2half2_rn(eb.x - bb.x, eb.y - bb.y);
                pkh[i / 2] = *reinterpret_cast<const uint32_t *>(&ha);
                pkh[i / 2 + 1] = *reinterpret_cast<const uint32_t *>(&hb);
                pkl[i / 2] = *reinterpret_cast<const uint32_t *>(&la);
                pkl[i / 2 + 1] = *reinterpret_cast<const uint32_t *>(&lb);
            }
            l = l * alpha + ((sum_a.x + sum_a.y) + (sum_b.x + sum_b.y));
            if (j > 0) {
                // PV of the previous tile must have read P before it is overwritten
                ok = ptx::mbar_wait(pv_done + 8 * ((j - 1) & 1), (uint32_t)((j - 1) >> 1) & 1u, abort_flag);
                if (!ok) break;
                ptx::tc_fence_after_sync();
            }
            ptx::tmem_st_cols<BN / 2>(t_ph, pkh);
            ptx::tmem_st_cols<BN / 2>(t_pl, pkl);
            ptx::tmem_wait_st();
            arrive_warp(p_full);
        }
        if (run && ok) {
            l_s[r] = l;
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(l_full);
        }
        if (run && !ok) { *abort_flag = 1; atomicCAS(p.status, 0, TC_ERR_SOFTMAX); }
        if (nt == 0 && *abort_flag == 0 && row < p.Sq) {
            // no visible key at all for this tile: the reference's 0/0
            float *orow = p.out + ((size_t)bh * p.Sq + row) * D;
            for (int i = 0; i < D; ++i) orow[i] = __int_as_float(0x7fc00000);
        }
    } else {
        ptx::setmaxnreg_inc<Cfg::REGS_ACC>();
        // ------------------------------------------------------------ accumulators + epilogue
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        float o[D];
#pragma unroll
        for (int i = 0; i < D; ++i) o[i] = 0.f;
        bool ok = run;
        for (int j = 0; j < nt && ok; ++j) {
            const int a = j & 1;
            ok = ptx::mbar_wait(alpha_full + 8 * (j & 3), (uint32_t)(j >> 2) & 1u, abort_flag);
            if (!ok) break;
            const float alpha = alpha_s[(j & 3) * BM + r];
            ok = ptx::mbar_wait(pv_done + 8 * a, (uint32_t)(j >> 1) & 1u, abort_flag);
            if (!ok) break;
            ptx::tc_fence_after_sync();
            const uint32_t t_pv = tmem + lane_base + (a ? Cfg::COL_PV1 : Cfg::COL_PV0);
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                uint32_t t[32];
                ptx::tmem_ld32(t_pv + c * 32, t);
                ptx::tmem_wait_ld();
                ptx::reg_fence32(t);
#pragma unroll
                for (int i = 0; i < 32; ++i) o[c * 32 + i] = fmaf(o[c * 32 + i], alpha, __uint_as_float(t[i]));
            }
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(pv_free + 8 * a);
        }
        if (run && ok) {
            ok = ptx::mbar_wait(l_full, 0, abort_flag);
            if (ok) {
                const float inv_l = 1.0f / l_s[r];   // l == 0 (no visible key) -> inf -> NaN rows, as the reference
                // staging: two 4 KB chunk buffers in this warp's quarter of the Q buffers (all QK^T have completed)
                constexpr uint32_t CHUNK_BYTES = 32 * 128;
                const uint32_t buf_a = qh_s + (uint32_t)quarter * (Cfg::Q_BYTES / 4);
                const uint32_t buf_b = ql_s + (uint32_t)quarter * (Cfg::Q_BYTES / 4);
                static_assert(CHUNK_BYTES <= Cfg::Q_BYTES / 4, "chunk buffer");
                const int row0 = q0 + quarter * 32;
                const uint32_t my_line = (uint32_t)lane * 128u;
                const uint32_t sw = (uint32_t)(lane & 7);
                auto put = [&](uint32_t buf, int piece, float x, float y, float z, float w) {
                    ptx::st_shared_v4(buf + my_line + (((uint32_t)piece ^ sw) << 4), __float_as_uint(x * inv_l),
                                      __float_as_uint(y * inv_l), __float_as_uint(z * inv_l), __float_as_uint(w * inv_l));
                };
                auto send = [&](uint32_t buf, int col) {
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0 && row0 < p.Sq) {
                        ptx::tma_store_3d(&tm_o, buf, col, row0, bh);
                        ptx::tma_store_commit();
                    }
                };
#pragma unroll
                for (int c = 0; c < D / 64; ++c) {
                    if (c > 0) {                                        // both buffers were sent in the step before
                        if (lane == 0) ptx::tma_store_wait_read<0>();
                        __syncwarp();
                    }
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        put(buf_a, i / 4, o[c * 64 + i], o[c * 64 + i + 1], o[c * 64 + i + 2], o[c * 64 + i + 3]);
                    send(buf_a, c * 64);
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        put(buf_b, i / 4, o[c * 64 + 32 + i], o[c * 64 + 33 + i], o[c * 64 + 34 + i], o[c * 64 + 35 + i]);
                    send(buf_b, c * 64 + 32);
                }
                if (lane == 0) ptx::tma_store_wait_read<0>();   // shared memory must outlive the stores' reads
                __syncwarp();
            }
        }
        if (run && !ok) { *abort_flag = 1; atomicCAS(p.status, 0, TC_ERR_SOFTMAX); }
    }

    // ---------------------------------------------------------------- teardown
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        // a wait ran out in this CTA (or in an earlier one of the launch): its rows are not valid and say so
        if (warp >= 4 && warp < 8) {
            const int row_a = q0 + (warp & 3) * 32 + lane;
            if (row_a < p.Sq) {
                float *orow = p.out + ((size_t)bh * p.Sq + row_a) * D;
                for (int i = 0; i < D; ++i) orow[i] = __int_as_float(0x7fc00000);
            }
        }
        for (int i = 0; i < 64; ++i) __nanosleep(2000);   // let copies in flight land
        __syncthreads();
    }
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem, Cfg::TMEM_COLS);
    }
}

// The split pass: hi = rn_fp16(x), lo = rn_fp16(x - hi) for up to three tensors in one launch, and the range
// check that decides between the tensor-core kernel above and the exact one (any |x| >= 2^15, or a value that is
// not finite, raises *flag).
struct SplitSeg {
    const float *x;
    __half *hi, *lo;
    long long n;              // elements, a multiple of 4
};
struct SplitParams {
    SplitSeg seg[3];
    int *flag;
};

__global__ void __launch_bounds__(256) split_f32_hi_lo_kernel(const SplitParams sp)
{
    bool bad = false;
    const long long stride = (long long)gridDim.x * blockDim.x;
#pragma unroll
    for (int t = 0; t < 3; ++t) {
        const SplitSeg s = sp.seg[t];
        const long long n4 = s.n >> 2;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
            const float4 v = reinterpret_cast<const float4 *>(s.x)[i];
            const __half2 h01 = __floats2half2_rn(v.x, v.y), h23 = __floats2half2_rn(v.z, v.w);
            const float2 b01 = __half22float2(h01), b23 = __half22float2(h23);
            const __half2 l01 = __floats2half2_rn(v.x - b01.x, v.y - b01.y), l23 = __floats2half2_rn(v.z - b23.x, v.w - b23.y);
            uint2 hh, ll;
            hh.x = *reinterpret_cast<const uint32_t *>(&h01);
            hh.y = *reinterpret_cast<const uint32_t *>(&h23);
            ll.x = *reinterpret_cast<const uint32_t *>(&l01);
            ll.y = *reinterpret_cast<const uint32_t *>(&l23);
            reinterpret_cast<uint2 *>(s.hi)[i] = hh;
            reinterpret_cast<uint2 *>(s.lo)[i] = ll;
            // !(|x| < 2^15) is also true for NaN
            bad |= !(fabsf(v.x) < 32768.f) || !(fabsf(v.y) < 32768.f) || !(fabsf(v.z) < 32768.f) || !(fabsf(v.w) < 32768.f);
        }
    }
    if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicOr(sp.flag, 1);
}

}  // namespace txb
