// fp16 flash-attention forward for sm_100a, two query tiles per CTA, one CTA per SM.
//
// Same arithmetic and the same operand flow as sdpa_tc_kernel (TMA-staged tiles, QK^T and
// PV as tcgen05 MMAs into tensor memory, fp32 online softmax with one thread per query row),
// replacing the reference's fp16 tensor-core path (tensorax csrc/cuda/kernels/attn.cu:1143-1521).
// ONE CTA owns the SM and works on two 128-row query tiles of the same head:
//   warp 0        TMA producer: both Q tiles once, then every K / V tile ONCE for both query
//                 tiles through an NS-deep ring (half the L2 -> shared-memory traffic of one
//                 CTA per query tile)
//   warp 1        issues every MMA in the fixed order QK0, PV0, QK1, PV1 and parks on the
//                 barrier of the next one
//   warps 2-3     idle (they only give their registers away)
//   warps 4-7     softmax of query tile 0 (thread = row = tensor-memory lane)
//   warps 8-11    softmax of query tile 1
// The producer / MMA warpgroup keeps 56 registers per thread and the softmax warpgroups take
// 224 (setmaxnreg), so a 128-wide score row, its packed P and the exponent pipeline stay in
// registers without spills.
//
// Tensor memory (512 columns):
//   P_ALIAS = false   S0 | S1 | O0 | O1 | P0 | P1   QK^T of the next key tile is issued once the
//                                                   softmax warps have pulled S into registers (d = 64)
//   P_ALIAS = true    S0/P0 | S1/P1 | O0 | O1       P overwrites the first half of the S columns it
//                                                   came from; the next QK^T of that tile follows its
//                                                   PV in program order (d = 128, where O takes 256 columns)
// Every mbarrier wait is bounded; a wait that runs out records a code in `status` and the
// whole CTA drains and frees its tensor memory.
#pragma once
#include "ptx.cuh"
#include "sdpa_tc.cuh"

namespace txb {

// Section profile of this kernel: cycles per step, summed over key tiles, for one softmax lane of either
// query tile ([0..15] tile 0, [32..47] tile 1) and the MMA lane ([16..31]).
enum PairSection : int {
    PSEC_SM_TOTAL = 0, PSEC_SM_WAIT_S = 1, PSEC_SM_LOAD_S = 2, PSEC_SM_MASK = 3, PSEC_SM_EXP = 5,
    PSEC_SM_WAIT_PV = 6, PSEC_SM_STORE_P = 7, PSEC_SM_EPILOGUE = 9, PSEC_SM_TILES = 10,
    PSEC_MMA_TOTAL = 16, PSEC_MMA_WAIT_S = 17, PSEC_MMA_WAIT_K = 18, PSEC_MMA_WAIT_P = 19, PSEC_MMA_WAIT_V = 20,
    PSEC_MMA_ISSUE = 21,
    // from the CTA's first instruction: to the softmax lane's first score tile, to the end of its loop and of its
    // epilogue; to the MMA lane's start (barriers and tensor memory set up), its Q tile and its first K tile
    PSEC_SM_FIRST_S = 11, PSEC_SM_LOOP_END = 12, PSEC_SM_END = 13,
    // inside the epilogue, from the end of the loop: the last PV has finished; the last result store is issued
    PSEC_SM_EPI_PV = 14, PSEC_SM_EPI_SENT = 15,
    PSEC_MMA_START = 22, PSEC_MMA_Q = 23, PSEC_MMA_K0 = 24,
};

// POLY: bit e set = element e of every group of 16 exponentials is evaluated on the FMA pipe
//       (bits come in pairs 2k, 2k+1: the polynomial works on two-wide fp32 vectors).
// FAULT_TEST: the instantiation behind tx_selftest_wait_timeout -- every wait gives up after 2 ms instead of 2 s and
//       the producer leaves out the K tile TcParams::skip_k_tile names, so that the give-up path can be exercised
//       on a GPU without faulting or hanging anything.
template <int D_, int BN_, int NS_, int POLY_, bool P_ALIAS_, bool PROF_ = false, bool FAULT_TEST_ = false>
struct PairCfg {
    static constexpr int D = D_, BN = BN_, NS = NS_, POLY = POLY_;
    static constexpr bool P_ALIAS = P_ALIAS_, PROF = PROF_, FAULT_TEST = FAULT_TEST_;
    static constexpr uint64_t WAIT_NS = FAULT_TEST_ ? 2000000ull : kWaitLimitNs;
    static constexpr int BM = 128;
    static constexpr int THREADS = 384;
    static constexpr int REGS_LIGHT = 64, REGS_SOFTMAX = 216;   // 128 * 64 + 256 * 216 = 63488 <= 384 * 168 = 64512
    static constexpr int KP = D / 64;                      // 64-column panels per row
    static constexpr uint32_t Q_TILE_BYTES = BM * D * 2;
    static constexpr uint32_t K_BYTES = BN * D * 2;
    static constexpr uint32_t V_BYTES = BN * D * 2;
    static constexpr uint32_t KV_PANEL = BN * 128;
    static constexpr uint32_t OFF_Q = 0;
    static constexpr uint32_t OFF_K = 2 * Q_TILE_BYTES;
    static constexpr uint32_t OFF_V = OFF_K + NS * K_BYTES;
    // result staging of the epilogue: two 4 KB chunk buffers per softmax warp.  They live in the warp's quarter of
    // its query tile's Q buffer; at D = 64 that quarter holds one, the other comes from here.
    static constexpr uint32_t OFF_STAGE = OFF_V + NS * V_BYTES;
    static constexpr uint32_t STAGE_BYTES = (Q_TILE_BYTES / 4 >= 8192) ? 0 : 8 * 4096;
    static constexpr uint32_t OFF_BAR = OFF_STAGE + STAGE_BYTES;
    // q_full[2] s_full[2] s_free[2] p_full[2] pv_done[2] k_full[NS] k_empty[NS] v_full[NS] v_empty[NS]
    static constexpr int N_BARS = 10 + 4 * NS;
    static constexpr uint32_t OFF_TMEM = OFF_BAR + N_BARS * 8;
    static constexpr uint32_t OFF_ABORT = OFF_TMEM + 4;
    static constexpr uint32_t SMEM_BYTES = ((OFF_ABORT + 4 + 127) / 128) * 128;
    static constexpr uint32_t COL_S0 = 0, COL_S1 = BN;
    static constexpr uint32_t COL_O0 = 2 * BN, COL_O1 = 2 * BN + D;
    static constexpr uint32_t COL_P0 = P_ALIAS ? COL_S0 : 2 * BN + 2 * D;
    static constexpr uint32_t COL_P1 = P_ALIAS ? COL_S1 : 2 * BN + 2 * D + BN / 2;
    static constexpr uint32_t COLS_USED = P_ALIAS ? 2 * BN + 2 * D : 3 * BN + 2 * D;
    static constexpr uint32_t TMEM_COLS = 512;
    static_assert(D % 64 == 0 && BN % 64 == 0 && BN <= 256 && D <= 256, "tile shape");
    static_assert(COLS_USED <= 512, "tensor memory has 512 columns");
    static_assert(SMEM_BYTES <= 232448, "more than the 227 KB a CTA may have");
};

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
sdpa_tc_pair_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                    const TcParams p)
{
    constexpr int D = Cfg::D, BN = Cfg::BN, NS = Cfg::NS, BM = Cfg::BM;
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = ptx::smem_u32(smem);
    const uint32_t q_s = sbase + Cfg::OFF_Q, k_s = sbase + Cfg::OFF_K, v_s = sbase + Cfg::OFF_V;
    const uint32_t bar0 = sbase + Cfg::OFF_BAR;
    // per-tile barriers: index t = 0, 1
    const uint32_t q_full = bar0, s_full = bar0 + 16, s_free = bar0 + 32, p_full = bar0 + 48, pv_done = bar0 + 64;
    const uint32_t k_full = bar0 + 80, k_empty = k_full + 8 * NS, v_full = k_empty + 8 * NS, v_empty = v_full + 8 * NS;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + Cfg::OFF_TMEM);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + Cfg::OFF_ABORT);

    const long long t_entry = Cfg::PROF ? clock64() : 0;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool prof_on = Cfg::PROF && p.prof != nullptr && blockIdx.x == 0;
    long long prof_last = 0;
    long long prof_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    auto tick = [&](int i) {
        if constexpr (Cfg::PROF) {
            if (prof_on) {
                const long long now = clock64();
                prof_acc[i] += now - prof_last;
                prof_last = now;
            }
        }
    };
    auto tick_start = [&]() {
        if constexpr (Cfg::PROF) {
            if (prof_on) prof_last = clock64();
        }
    };

    // Work item of this CTA.  CTAs start in blockIdx order, so inside a group of `p.group` slabs the items are
    // laid out longest first over ALL the group's slabs (late causal query pairs walk the most keys): the
    // launch's last wave is then made of the shortest items.  A group is small enough for its K/V to stay in L2
    // while the slabs' CTAs that share them run side by side.
    const int span = p.group * p.n_pairs;
    const int grp = (int)blockIdx.x / span, rem = (int)blockIdx.x % span;
    const int slabs = min(p.group, p.BH - grp * p.group);
    const int q_pair = p.n_pairs - 1 - rem / slabs;
    const int q0 = q_pair * (2 * BM);                            // first row of tile 0; tile 1 starts at q0 + BM
    const int bh = grp * p.group + rem % slabs;
    const int b = bh / p.Hq, h = bh % p.Hq;
    const int kvh = b * p.Hkv + h / (p.Hq / p.Hkv);

    int kv_limit = p.Sk;                                         // keys any row of this batch may see
    if (p.kv_lens) kv_limit = min(kv_limit, max(p.kv_lens[b], 0));
    // key tiles each query tile walks; tile 1 does not exist when the sequence ends inside tile 0
    const bool live1 = q0 + BM < p.Sq;
    const int kv_end0 = p.causal ? min(kv_limit, q0 + BM) : kv_limit;
    const int kv_end1 = live1 ? (p.causal ? min(kv_limit, q0 + 2 * BM) : kv_limit) : 0;
    const int n0 = (kv_end0 + BN - 1) / BN, n1 = (kv_end1 + BN - 1) / BN;
    const int n_max = max(n0, n1);

    // Warp 0 sets the barriers up and sends the first loads (both Q tiles, K and V of key tile 0) on their way
    // before the CTA meets: the tensor-memory allocation, the meeting and the register hand-over then run
    // under the loads' latency instead of in front of it.
    const bool first_k_left_out = Cfg::FAULT_TEST && p.skip_k_tile == 0;
    if (warp == 0) {
        if (lane == 0) {
            *abort_flag = 0;
            for (int t = 0; t < 2; ++t) {
                ptx::mbar_init(q_full + 8 * t, 1);
                ptx::mbar_init(s_full + 8 * t, 1);
                ptx::mbar_init(s_free + 8 * t, 4);          // one arrival per softmax warp of the tile
                ptx::mbar_init(p_full + 8 * t, 4);
                ptx::mbar_init(pv_done + 8 * t, 1);
            }
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
            } else if (n_max > 0) {
                ptx::prefetch_tmap(&tm_q);
                ptx::prefetch_tmap(&tm_k);
                ptx::prefetch_tmap(&tm_v);
                if (n0 > 0) {
                    ptx::mbar_arrive_expect_tx(q_full, Cfg::Q_TILE_BYTES);
#pragma unroll
                    for (int pn = 0; pn < Cfg::KP; ++pn)
                        ptx::tma_load_3d(q_s + pn * (BM * 128), &tm_q, q_full, pn * 64, q0, bh);
                }
                if (!first_k_left_out) {
                    ptx::mbar_arrive_expect_tx(k_full, Cfg::K_BYTES);
#pragma unroll
                    for (int pn = 0; pn < Cfg::KP; ++pn)
                        ptx::tma_load_3d(k_s + pn * Cfg::KV_PANEL, &tm_k, k_full, pn * 64, 0, kvh);
                }
                if (n1 > 0) {
                    ptx::mbar_arrive_expect_tx(q_full + 8, Cfg::Q_TILE_BYTES);
#pragma unroll
                    for (int pn = 0; pn < Cfg::KP; ++pn)
                        ptx::tma_load_3d(q_s + Cfg::Q_TILE_BYTES + pn * (BM * 128), &tm_q, q_full + 8, pn * 64,
                                         q0 + BM, bh);
                }
                ptx::mbar_arrive_expect_tx(v_full, Cfg::V_BYTES);
#pragma unroll
                for (int pn = 0; pn < Cfg::KP; ++pn)
                    ptx::tma_load_3d(v_s + pn * Cfg::KV_PANEL, &tm_v, v_full, pn * 64, 0, kvh);
            }
            // an earlier CTA of the launch may already have given up (asked after the loads are out: the answer
            // takes a trip to global memory; the loads land during the teardown's grace period)
            if (*reinterpret_cast<volatile int *>(p.status) != 0) *abort_flag = 1;
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
    const bool run = (*abort_flag == 0) && n_max > 0;
    // The launch gives every thread 168 registers (65536 / 384); the producer / MMA warpgroup needs
    // few and hands the rest to the softmax warpgroups, whose score rows then stay in registers.

    if (warp < 4) {
    ptx::setmaxnreg_dec<Cfg::REGS_LIGHT>();
    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (run) {
            const bool leader = ptx::elect_one();
            bool ok = true;
            for (int j = 0; j < n_max && ok; ++j) {
                const int s = j % NS;
                const uint32_t ph = (uint32_t)(j / NS) & 1u;
                ok = ptx::mbar_wait(k_empty + 8 * s, ph ^ 1u, abort_flag, Cfg::WAIT_NS);
                if (!ok) break;
                const bool left_out = Cfg::FAULT_TEST && j == p.skip_k_tile;     // self-test: this tile never arrives
                if (leader && j > 0) {                                           // key tile 0 went out before the meeting
                    if (!left_out) {
                        ptx::mbar_arrive_expect_tx(k_full + 8 * s, Cfg::K_BYTES);
#pragma unroll
                        for (int pn = 0; pn < Cfg::KP; ++pn)
                            ptx::tma_load_3d(k_s + s * Cfg::K_BYTES + pn * Cfg::KV_PANEL, &tm_k, k_full + 8 * s,
                                             pn * 64, j * BN, kvh);
                    }
                }
                __syncwarp();
                ok = ptx::mbar_wait(v_empty + 8 * s, ph ^ 1u, abort_flag, Cfg::WAIT_NS);
                if (!ok) break;
                if (leader && j > 0) {
                    ptx::mbar_arrive_expect_tx(v_full + 8 * s, Cfg::V_BYTES);
#pragma unroll
                    for (int pn = 0; pn < Cfg::KP; ++pn)
                        ptx::tma_load_3d(v_s + s * Cfg::V_BYTES + pn * Cfg::KV_PANEL, &tm_v, v_full + 8 * s,
                                         pn * 64, j * BN, kvh);
                }
                __syncwarp();
            }
            if (!ok && leader) { *abort_flag = 1; atomicCAS(p.status, 0, TC_ERR_PRODUCER); }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // Warp-uniform control flow; one elected lane, the same one every time, issues the MMAs and
        // the commits that track them.  The tensor pipe runs them in issue order, which is what
        // P_ALIAS relies on (the QK^T that overwrites S/P follows the PV that read P).
        if (run) {
            const bool leader = ptx::elect_one();
            constexpr uint32_t idesc_qk = ptx::idesc_f16(BM, BN, false);
            constexpr uint32_t idesc_pv = ptx::idesc_f16(BM, D, true);
            constexpr uint32_t desc_hi = ptx::smem_desc_sw128_hi(1024);
            const uint32_t q_lo = ptx::smem_desc_sw128_lo(q_s, 16);
            const uint32_t k_lo = ptx::smem_desc_sw128_lo(k_s, 16);
            const uint32_t v_lo = ptx::smem_desc_sw128_lo(v_s, Cfg::KV_PANEL);
            bool ok = true;
            tick_start();
            const long long t_begin = Cfg::PROF ? clock64() : 0;
            long long t_q = 0, t_k0 = 0;
            // S_t = Q_t K_j^T; the K stage is released by whichever tile reads it last
            auto issue_qk = [&](int t, int j) -> bool {
                const int s = j % NS;
                const uint32_t ph = (uint32_t)(j / NS) & 1u;
                tick(0);
                if (!ptx::mbar_wait(k_full + 8 * s, ph, abort_flag, Cfg::WAIT_NS)) return false;
                if constexpr (Cfg::PROF) { if (t_k0 == 0) t_k0 = clock64(); }
                tick(2);
                ptx::tc_fence_after_sync();
                const uint32_t ks_lo = k_lo + (uint32_t)s * (Cfg::K_BYTES >> 4);
                const uint32_t qt_lo = q_lo + (uint32_t)t * (Cfg::Q_TILE_BYTES >> 4);
                const uint32_t t_s = tmem + (t ? Cfg::COL_S1 : Cfg::COL_S0);
                const bool last_reader = t == 1 ? true : (j >= n1);
                if (leader) {
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        const uint32_t qa = ((kk >> 2) * (BM * 128) + (kk & 3) * 32) >> 4;
                        const uint32_t kb = ((kk >> 2) * Cfg::KV_PANEL + (kk & 3) * 32) >> 4;
                        ptx::mma_ss(t_s, ptx::make_desc(qt_lo + qa, desc_hi), ptx::make_desc(ks_lo + kb, desc_hi),
                                    idesc_qk, kk > 0);
                    }
                    if (last_reader) ptx::mma_commit(k_empty + 8 * s);
                    ptx::mma_commit(s_full + 8 * t);
                }
                __syncwarp();
                tick(5);
                return true;
            };
            // O_t += P_t V_j
            auto issue_pv = [&](int t, int j) -> bool {
                const int s = j % NS;
                const uint32_t ph = (uint32_t)(j / NS) & 1u;
                tick(0);
                if (!ptx::mbar_wait(v_full + 8 * s, ph, abort_flag, Cfg::WAIT_NS)) return false;
                tick(4);
                if (!ptx::mbar_wait(p_full + 8 * t, (uint32_t)j & 1u, abort_flag, Cfg::WAIT_NS)) return false;
                tick(3);
                ptx::tc_fence_after_sync();
                const uint32_t vs_lo = v_lo + (uint32_t)s * (Cfg::V_BYTES >> 4);
                const uint32_t t_o = tmem + (t ? Cfg::COL_O1 : Cfg::COL_O0);
                const uint32_t t_p = tmem + (t ? Cfg::COL_P1 : Cfg::COL_P0);
                const bool last_reader = t == 1 ? true : (j >= n1);
                if (leader) {
#pragma unroll
                    for (int kk = 0; kk < BN / 16; ++kk) {
                        const uint64_t bdesc = ptx::make_desc(vs_lo + kk * ((16 * 128) >> 4), desc_hi);
                        ptx::mma_ts(t_o, t_p + kk * 8, bdesc, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
                    }
                    if (last_reader) ptx::mma_commit(v_empty + 8 * s);
                    ptx::mma_commit(pv_done + 8 * t);
                }
                __syncwarp();
                tick(5);
                return true;
            };
            if (n0 > 0) {
                ok = ptx::mbar_wait(q_full, 0, abort_flag, Cfg::WAIT_NS);
                if constexpr (Cfg::PROF) t_q = clock64();
                if (ok) ok = issue_qk(0, 0);
            }
            if (ok && n1 > 0) {
                ok = ptx::mbar_wait(q_full + 8, 0, abort_flag, Cfg::WAIT_NS);
                if (ok) ok = issue_qk(1, 0);
            }
            for (int j = 0; j < n_max && ok; ++j) {
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    const int nt = t ? n1 : n0;
                    if constexpr (!Cfg::P_ALIAS) {
                        if (j + 1 < nt && ok) {
                            tick(0);
                            ok = ptx::mbar_wait(s_free + 8 * t, (uint32_t)j & 1u, abort_flag, Cfg::WAIT_NS);
                            tick(1);
                            if (ok) { ptx::tc_fence_after_sync(); ok = issue_qk(t, j + 1); }
                        }
                        if (j < nt && ok) ok = issue_pv(t, j);
                    } else {
                        // P_t lives in S_t's columns: the next QK^T of this tile follows its PV in program order
                        if (j < nt && ok) ok = issue_pv(t, j);
                        if (j + 1 < nt && ok) ok = issue_qk(t, j + 1);
                    }
                }
            }
            if (!ok && leader) { *abort_flag = 1; atomicCAS(p.status, 0, TC_ERR_MMA); }
            if constexpr (Cfg::PROF) {
                if (prof_on && leader) {
                    p.prof[PSEC_MMA_TOTAL] = clock64() - t_begin;
                    p.prof[PSEC_MMA_WAIT_S] = prof_acc[1];
                    p.prof[PSEC_MMA_WAIT_K] = prof_acc[2];
                    p.prof[PSEC_MMA_WAIT_P] = prof_acc[3];
                    p.prof[PSEC_MMA_WAIT_V] = prof_acc[4];
                    p.prof[PSEC_MMA_ISSUE] = prof_acc[5];
                    p.prof[PSEC_MMA_START] = t_begin - t_entry;
                    p.prof[PSEC_MMA_Q] = t_q - t_entry;
                    p.prof[PSEC_MMA_K0] = t_k0 - t_entry;
                }
            }
        }
    }
    } else {
        ptx::setmaxnreg_inc<Cfg::REGS_SOFTMAX>();
        // ------------------------------------------------------------ softmax + epilogue
        const int t = (warp - 4) >> 2;                   // query tile of this warp
        const int quarter = warp & 3;                    // tensor-memory lanes this warp may touch
        const int r = quarter * 32 + lane;               // row inside the tile
        const int q0t = q0 + t * BM;
        const int row = q0t + r;
        const int nt = t ? n1 : n0;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const uint32_t t_s = tmem + lane_base + (t ? Cfg::COL_S1 : Cfg::COL_S0);
        const uint32_t t_o = tmem + lane_base + (t ? Cfg::COL_O1 : Cfg::COL_O0);
        const uint32_t t_p = tmem + lane_base + (t ? Cfg::COL_P1 : Cfg::COL_P0);
        const uint32_t my_s_full = s_full + 8 * t, my_s_free = s_free + 8 * t, my_p_full = p_full + 8 * t,
                       my_pv_done = pv_done + 8 * t;
        const float scale = p.scale_log2;
        float m_used = -1.0e30f;   // finite stand-in for "no key seen yet"
        float l = 0.f;
        bool ok = run && nt > 0;
        auto arrive_warp = [&](uint32_t bar) {
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar);
        };
        const bool prof_lane = prof_on && quarter == 0 && lane == 0;
        tick_start();
        const long long t_begin = Cfg::PROF ? clock64() : 0;
        for (int j = 0; j < nt && ok; ++j) {
            const int kv0 = j * BN;
            tick(0);
            ok = ptx::mbar_wait(my_s_full, (uint32_t)j & 1u, abort_flag, Cfg::WAIT_NS);
            tick(PSEC_SM_WAIT_S);
            if constexpr (Cfg::PROF) { if (j == 0 && prof_lane) p.prof[(t ? 32 : 0) + PSEC_SM_FIRST_S] = clock64() - t_entry; }
            if (!ok) break;
            ptx::tc_fence_after_sync();
            // The whole score row goes to registers with one wait.  The array is defined here, inside the
            // loop, by this one load: a row kept alive across the loop edge (loaded at the bottom for the
            // next iteration) cost a register shuffle per tile and 20 % of the kernel's speed.
            uint32_t sv[BN];
            ptx::tmem_ld_cols<BN>(t_s, sv);
            ptx::tmem_wait_ld();
            ptx::reg_fence_cols<BN>(sv);
            if constexpr (!Cfg::P_ALIAS) arrive_warp(my_s_free);   // S belongs to the MMA warp again
            tick(PSEC_SM_LOAD_S);
            const bool need_mask = (kv0 + BN > kv_limit) || (p.causal && (kv0 + BN - 1 > q0t));
            if (need_mask) {
                // visible keys of this row are a prefix of the tile: columns [0, lim)
                const int lim = min(kv_limit - kv0, p.causal ? row - kv0 + 1 : BN);
#pragma unroll
                for (int i = 0; i < BN; ++i) sv[i] = ptx::keep_if_below(sv[i], i, lim);
            }
            tick(PSEC_SM_MASK);
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
            for (int i = 0; i < BN; i += 8) {
                mx0 = ptx::max3(mx0, __uint_as_float(sv[i]), __uint_as_float(sv[i + 1]));
                mx1 = ptx::max3(mx1, __uint_as_float(sv[i + 2]), __uint_as_float(sv[i + 3]));
                mx2 = ptx::max3(mx2, __uint_as_float(sv[i + 4]), __uint_as_float(sv[i + 5]));
                mx3 = ptx::max3(mx3, __uint_as_float(sv[i + 6]), __uint_as_float(sv[i + 7]));
            }
            const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
            const float m_new = fmaxf(m_used, mx * scale);
            const float m_next = (m_new > m_used + kLazyRescaleLog2) ? m_new : m_used;
            const float alpha = ptx::ex2_approx(m_used - m_next);   // 1 when the max is kept
            m_used = m_next;
            // p = 2^(s*scale - m): a masked score is -inf and gives exactly 0
            const float2 scale2 = make_float2(scale, scale), negm2 = make_float2(-m_next, -m_next);
            float2 sum_a = make_float2(0.f, 0.f), sum_b = make_float2(0.f, 0.f);
            uint32_t pk[BN / 2];
#pragma unroll
            for (int i = 0; i < BN; i += 4) {
                const float2 xa = __ffma2_rn(make_float2(__uint_as_float(sv[i]), __uint_as_float(sv[i + 1])), scale2, negm2);
                const float2 xb = __ffma2_rn(make_float2(__uint_as_float(sv[i + 2]), __uint_as_float(sv[i + 3])), scale2, negm2);
                const int e0 = i & 15;
                const bool poly_a = (Cfg::POLY >> e0) & 1, poly_b = (Cfg::POLY >> (e0 + 2)) & 1;
                const float2 ea = poly_a ? ptx::ex2_poly2(xa) : make_float2(ptx::ex2_approx(xa.x), ptx::ex2_approx(xa.y));
                const float2 eb = poly_b ? ptx::ex2_poly2(xb) : make_float2(ptx::ex2_approx(xb.x), ptx::ex2_approx(xb.y));
                sum_a = __fadd2_rn(sum_a, ea);
                sum_b = __fadd2_rn(sum_b, eb);
                pk[i / 2] = ptx::pack_half2(ea.x, ea.y);
                pk[i / 2 + 1] = ptx::pack_half2(eb.x, eb.y);
            }
            l = l * alpha + ((sum_a.x + sum_a.y) + (sum_b.x + sum_b.y));
            tick(PSEC_SM_EXP);
            if (j > 0) {
                // PV of the previous tile must be finished before P is overwritten or O rescaled (with P in
                // S's columns the scores themselves came after it, so this wait returns at once)
                ok = ptx::mbar_wait(my_pv_done, (uint32_t)(j - 1) & 1u, abort_flag, Cfg::WAIT_NS);
                if (!ok) break;
                ptx::tc_fence_after_sync();
                if (__any_sync(0xffffffffu, alpha != 1.0f)) {
                    // rare after the first tiles; 16 columns at a time
#pragma unroll 1
                    for (int c = 0; c < D / 16; ++c) {
                        uint32_t o[16];
                        ptx::tmem_ld16(t_o + c * 16, o);
                        ptx::tmem_wait_ld();
                        ptx::reg_fence16(o);
#pragma unroll
                        for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        ptx::tmem_st16(t_o + c * 16, o);
                    }
                }
            }
            tick(PSEC_SM_WAIT_PV);
            ptx::tmem_st_cols<BN / 2>(t_p, pk);
            ptx::tmem_wait_st();
            arrive_warp(my_p_full);
            tick(PSEC_SM_STORE_P);
        }
        const long long t_loop_end = Cfg::PROF ? clock64() : 0;
        if (run && nt > 0 && ok) {
            ok = ptx::mbar_wait(my_pv_done, (uint32_t)(nt - 1) & 1u, abort_flag, Cfg::WAIT_NS);
            if constexpr (Cfg::PROF) { if (prof_lane) p.prof[(t ? 32 : 0) + PSEC_SM_EPI_PV] = clock64() - t_loop_end; }
            if (ok) {
                ptx::tc_fence_after_sync();
                const float inv_l = 1.0f / l;    // l == 0 (no visible key) -> inf -> NaN rows, as the reference
                if (p.lse && row < p.Sq) p.lse[(size_t)bh * p.Sq + row] = m_used + __log2f(l);
                // O leaves through shared memory and one bulk tensor store per 128-byte-wide chunk of this warp's
                // 32 rows: a thread owns a row, so direct stores would put 32 rows' 16-byte pieces into every
                // store instruction.  The staging space is this warp's quarter of its own query tile's Q buffer
                // (every QK^T of the tile has completed: the last s_full said so), written in the 128-byte
                // swizzle the tensor map expects, which also keeps the 32 lanes on distinct banks.
                constexpr uint32_t CHUNK_BYTES = 32 * 128;
                const uint32_t buf_a = q_s + (uint32_t)t * Cfg::Q_TILE_BYTES + (uint32_t)quarter * (Cfg::Q_TILE_BYTES / 4);
                const uint32_t buf_b = Cfg::STAGE_BYTES ? sbase + Cfg::OFF_STAGE + (uint32_t)(warp - 4) * CHUNK_BYTES
                                                        : buf_a + CHUNK_BYTES;
                const int row0 = q0t + quarter * 32;
                const uint32_t my_line = (uint32_t)lane * 128u;
                const uint32_t sw = (uint32_t)(lane & 7);
                auto put = [&](uint32_t buf, int piece, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
                    ptx::st_shared_v4(buf + my_line + (((uint32_t)piece ^ sw) << 4), x, y, z, w);
                };
                auto send = [&](uint32_t buf, int col) {
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0 && row0 < p.Sq) {
                        ptx::tma_store_3d(&tm_o, buf, col, row0, bh);
                        ptx::tma_store_commit();
                    }
                };
                // 64 columns of O per step: both loads first, then one chunk buffer each
#pragma unroll
                for (int c = 0; c < D / 64; ++c) {
                    uint32_t o[32], o2[32];
                    ptx::tmem_ld32(t_o + c * 64, o);
                    ptx::tmem_ld32(t_o + c * 64 + 32, o2);
                    ptx::tmem_wait_ld();
                    ptx::reg_fence32(o);
                    ptx::reg_fence32(o2);
                    if (p.out_f16) {
                        const uint32_t buf = (c & 1) ? buf_b : buf_a;      // D / 64 <= 2 chunks: no buffer is used twice
                        auto h2 = [&](uint32_t a, uint32_t b2) {
                            return ptx::pack_half2(__uint_as_float(a) * inv_l, __uint_as_float(b2) * inv_l);
                        };
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            put(buf, i / 8, h2(o[i], o[i + 1]), h2(o[i + 2], o[i + 3]), h2(o[i + 4], o[i + 5]),
                                h2(o[i + 6], o[i + 7]));
                            put(buf, 4 + i / 8, h2(o2[i], o2[i + 1]), h2(o2[i + 2], o2[i + 3]), h2(o2[i + 4], o2[i + 5]),
                                h2(o2[i + 6], o2[i + 7]));
                        }
                        send(buf, c * 64);
                    } else {
                        if (c > 0) {                                        // both buffers were sent in the step before
                            if (lane == 0) ptx::tma_store_wait_read<0>();
                            __syncwarp();
                        }
                        auto f = [&](uint32_t a) { return __float_as_uint(__uint_as_float(a) * inv_l); };
#pragma unroll
                        for (int i = 0; i < 32; i += 4) put(buf_a, i / 4, f(o[i]), f(o[i + 1]), f(o[i + 2]), f(o[i + 3]));
                        send(buf_a, c * 64);
#pragma unroll
                        for (int i = 0; i < 32; i += 4) put(buf_b, i / 4, f(o2[i]), f(o2[i + 1]), f(o2[i + 2]), f(o2[i + 3]));
                        send(buf_b, c * 64 + 32);
                    }
                }
                if constexpr (Cfg::PROF) { if (prof_lane) p.prof[(t ? 32 : 0) + PSEC_SM_EPI_SENT] = clock64() - t_loop_end; }
                if (lane == 0) ptx::tma_store_wait_read<0>();   // shared memory must outlive the stores' reads
                __syncwarp();
            }
        }
        if (run && nt > 0 && !ok) { *abort_flag = 1; atomicCAS(p.status, 0, TC_ERR_SOFTMAX); }
        if constexpr (Cfg::PROF) {
            if (prof_lane) {
                long long *dst = p.prof + (t ? 32 : 0);
                dst[PSEC_SM_TOTAL] = t_loop_end - t_begin;
                for (int i = 1; i <= 7; ++i) dst[i] = prof_acc[i];
                dst[PSEC_SM_EPILOGUE] = clock64() - t_loop_end;
                dst[PSEC_SM_LOOP_END] = t_loop_end - t_entry;
                dst[PSEC_SM_END] = clock64() - t_entry;
                dst[PSEC_SM_TILES] = nt;
            }
        }
        if (nt == 0 && *abort_flag == 0 && row < p.Sq && (t == 0 || live1)) {
            // no visible key at all for this tile: the reference's 0/0
            const size_t obase = ((size_t)bh * p.Sq + row) * p.dv_total;
            if (p.out_f16) {
                __half *orow_h = static_cast<__half *>(p.out) + obase;
                for (int i = 0; i < D; ++i) orow_h[i] = __ushort_as_half((unsigned short)0x7e00);
            } else {
                float *orow = static_cast<float *>(p.out) + obase;
                for (int i = 0; i < D; ++i) orow[i] = __int_as_float(0x7fc00000);
            }
            if (p.lse) p.lse[(size_t)bh * p.Sq + row] = __int_as_float(0x7fc00000);
        }
    }

    // ---------------------------------------------------------------- teardown
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        // A wait ran out somewhere in this CTA (or in an earlier one of the launch): its rows are not valid.
        // They are overwritten with NaN so that the failure is visible in the data, not only in the status word.
        if (warp >= 4) {
            const int ta = (warp - 4) >> 2, row_a = q0 + ta * BM + (warp & 3) * 32 + lane;
            if (row_a < p.Sq) {
                const size_t ob = ((size_t)bh * p.Sq + row_a) * p.dv_total;
                for (int i = 0; i < D; ++i) {
                    if (p.out_f16) static_cast<__half *>(p.out)[ob + i] = __ushort_as_half((unsigned short)0x7e00);
                    else static_cast<float *>(p.out)[ob + i] = __int_as_float(0x7fc00000);
                }
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

}  // namespace txb
