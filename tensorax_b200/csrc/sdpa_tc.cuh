// fp16 flash-attention forward for sm_100a: TMA-staged Q/K/V tiles, QK^T and PV
// as tcgen05 MMAs accumulating in tensor memory, fp32 online softmax.
//
// Replaces the reference's fp16 tensor-core path (tensorax
// csrc/cuda/kernels/attn.cu:1143-1521, sdpa_kernel_mma_fp16 + sdpa_mma_fp16_cuda):
// fp16 Q/K/V [B,H,S,d] -> fp32 O, fp32 accumulation, P rounded to fp16 before PV
// (attn.cu:1357-1360).  Differences on purpose: the softmax scale is applied in
// fp32 inside the exponent instead of pre-multiplying Q in fp16 (attn.cu:1218-1232),
// and causal / key-length masks and grouped K/V heads are applied in-kernel,
// which the reference path cannot do at all.
//
// One CTA = one 128-row query tile of one (batch, query head) and one slice of DV
// value columns (the slice is the whole head except for d = 512, where two CTAs
// each recompute S and own 256 output columns, as the reference's D_V_PASSES does
// in sequence, attn.cu:1239-1241).  Six warps:
//   warp 0      TMA producer: Q once, then K/V tiles through an NS-deep ring of
//               shared-memory stages, 128-byte swizzled
//   warp 1      owns tensor memory (alloc/dealloc) and issues every MMA:
//               S = Q K^T (M=128, N=BN, K=16 per instruction) and
//               O += P V  (M=128, N=DV, K=16 per instruction, V read MN-major)
//               Both warps keep their control flow warp-uniform and elect one lane
//               only for the issue instructions, so descriptors, coordinates and
//               barrier handles stay in uniform registers (issuing from a divergent
//               single lane cost ~75 extra cycles per MMA).
//   warps 2-5   softmax: thread t owns query row 32*(warp%4)+lane, the tensor
//               memory lane it is allowed to read.  The whole S row is pulled into
//               registers with one wait and S is handed back to the MMA warp at
//               once; then masks in registers, row max, exp2 (two-wide fp32 FMAs
//               form the exponents), fp16 pack, P written to tensor memory (or
//               swizzled shared memory).  O is rescaled in tensor memory only when
//               the running max grew by more than 2^8; the epilogue writes O/l as
//               fp32.
// For d <= 128 two such CTAs fit one SM (shared memory <= 113 KB, 256
// tensor-memory columns), so one CTA's softmax overlaps the other's MMAs.
//
// Every mbarrier wait is bounded; a wait that runs out records a code in
// `status` and the whole CTA drains and frees its tensor memory.
#pragma once
#include "ptx.cuh"

namespace txb {

struct TcParams {
    void *out;                // [B,Hq,Sq,dv_total] fp32, or fp16 when out_f16
    float *lse;               // optional [B,Hq,Sq]: log2 of the row's sum of 2^(score*scale_log2)
    const int32_t *kv_lens;   // optional [B]
    int *status;              // device word: 0 = ok, else first failing wait's code
    int Hq, Hkv, Sq, Sk;
    int dv_total;             // row length of `out` (= DV * the CTAs per query tile)
    int causal;
    int out_f16;
    float scale_log2;         // (1/sqrt(d_k)) * log2(e)
    long long *prof;          // optional [64] cycle counters written by CTA (0,0,0) (section profile)
    int skip_k_tile;          // failure-path self-test instantiation only: the producer leaves this K tile out (-1 = none)
    // sdpa_tc_pair_kernel only: the 1-D grid walks groups of `group` (batch, head) slabs; inside a group all
    // slabs' longest work items come first (n_pairs = 256-row query pairs per slab, BH = slabs)
    int group, n_pairs, BH;
};

// Section profile (the counterpart of the reference's TX_TICK clock64 sections,
// csrc/cuda/profiling.cuh:20-51): cycles one softmax lane, the MMA lane and the
// producer lane of CTA (0,0,0) spend in each step of their loops, summed over tiles.
enum TcSection : int {
    SEC_SM_TOTAL = 0, SEC_SM_WAIT_S = 1, SEC_SM_LOAD_S = 2, SEC_SM_MAX = 3, SEC_SM_EXP = 5,
    SEC_SM_WAIT_PV = 6, SEC_SM_RESCALE = 7, SEC_SM_STORE_P = 8, SEC_SM_EPILOGUE = 9, SEC_SM_TILES = 10,
    SEC_MMA_TOTAL = 16, SEC_MMA_WAIT_SFREE = 17, SEC_MMA_QK = 18, SEC_MMA_WAIT_V = 19, SEC_MMA_WAIT_P = 20,
    SEC_MMA_PV = 21,
    SEC_LD_TOTAL = 24, SEC_LD_WAIT_K = 25, SEC_LD_WAIT_V = 26,
};

enum TcStatus : int {
    TC_OK = 0,
    TC_ERR_ALIGN = 1,
    TC_ERR_PRODUCER = 2,
    TC_ERR_MMA = 3,
    TC_ERR_SOFTMAX = 4,
};

template <int DK_, int DV_, int BN_, int NS_, bool P_TMEM_, bool PROF_ = false, int POLY_ = 0, int NSV_ = NS_,
          bool LD_SPLIT_ = false, int QT_ = 0, bool Q_ALIAS_ = false>
struct TcCfg {
    // Q_ALIAS: the Q panels that move to tensor memory are staged in the (still empty) K/V ring instead of
    // a region of their own; the producer starts the ring only after the copy.  Shared memory then holds
    // just the tail panels of Q, which is what lets d = 512 use 64-key tiles.
    static constexpr bool Q_ALIAS = Q_ALIAS_;
    // QT: tensor-memory columns that hold the first 2*QT elements of every Q row (fp16 pairs).
    // The QK^T MMAs over that part take A from tensor memory, so they read only the K tile from
    // shared memory; with narrow key tiles the A read is what the shared-memory port runs out of.
    static constexpr int QT = QT_;
    static constexpr bool PROF = PROF_;   // collect the section profile
    // LD_SPLIT: the producer serves the K ring and the V ring as two independent queues (a K
    // tile never waits behind a V stage that is still being read, nor the reverse).
    static constexpr bool LD_SPLIT = LD_SPLIT_;
    // POLY: bit e set = element e of every group of 16 exponentials is evaluated by a polynomial
    // on the FMA pipe instead of the special-function unit (16 results per clock and SM), which
    // is the busiest pipe of this kernel at small head dims.
    static constexpr int POLY = POLY_;
    static constexpr int DK = DK_;        // head dim of Q and K
    static constexpr int DV = DV_;        // value columns this CTA owns
    static constexpr int BN = BN_;        // keys per tile
    static constexpr int NS = NS_;        // K ring depth
    static constexpr int NSV = NSV_;      // V ring depth
    static constexpr bool P_TMEM = P_TMEM_;
    static constexpr int BM = 128;        // query rows per CTA
    static constexpr int SOFTMAX_WARPS = 4;
    static constexpr int THREADS = 64 + 32 * SOFTMAX_WARPS;
    static constexpr int KP = DK / 64;    // 64-column (128-byte) panels per row of Q / K
    static constexpr int VP = DV / 64;    // panels per row of this CTA's V slice
    static constexpr uint32_t Q_BYTES = BM * DK * 2;          // all of the Q tile (what the TMA loads bring in)
    static constexpr int QP_TMEM = QT_ / 32;                   // 64-element panels of Q held in tensor memory
    static constexpr int QP_SKIP = Q_ALIAS_ ? QP_TMEM : 0;     // ... of which this many have no place in the Q region
    static constexpr uint32_t Q_REGION = (DK / 64 - QP_SKIP) * BM * 128;
    static constexpr uint32_t K_BYTES = BN * DK * 2;       // one K stage
    static constexpr uint32_t V_BYTES = BN * DV * 2;       // one V stage
    static constexpr uint32_t KV_PANEL = BN * 128;         // one 64-column panel of a stage
    static constexpr uint32_t P_BYTES = P_TMEM ? 0 : BM * BN * 2;
    static constexpr uint32_t OFF_Q = 0;
    static constexpr uint32_t OFF_K = OFF_Q + Q_REGION;
    static constexpr uint32_t OFF_V = OFF_K + NS * K_BYTES;
    static constexpr uint32_t OFF_P = OFF_V + NSV * V_BYTES;
    static constexpr uint32_t OFF_BAR = OFF_P + P_BYTES;
    // barriers: q_full, s_full, s_free, p_full, pv_done, q_tmem, then k_full/k_empty[NS], v_full/v_empty[NSV]
    static constexpr int N_BARS = 6 + 2 * NS + 2 * NSV;
    static constexpr uint32_t OFF_TMEM = OFF_BAR + N_BARS * 8;
    static constexpr uint32_t OFF_ABORT = OFF_TMEM + 4;
    static constexpr uint32_t SMEM_BYTES = ((OFF_ABORT + 4 + 127) / 128) * 128;
    // tensor memory columns: S fp32 [BN] | O fp32 [DV] | P fp16 pairs [BN/2] (only if P_TMEM)
    static constexpr uint32_t COL_S = 0;
    static constexpr uint32_t COL_O = BN;
    static constexpr uint32_t COL_P = BN + DV;
    static constexpr uint32_t COL_Q = BN + DV + (P_TMEM ? BN / 2 : 0);
    static constexpr uint32_t COLS_USED = COL_Q + QT;
    static_assert(QT % 32 == 0 && 2 * QT <= DK, "Q columns in tensor memory come in whole 64-element panels");
    static_assert(!Q_ALIAS || (QT > 0 && (uint32_t)QP_TMEM * BM * 128 <= NS * K_BYTES + NSV * V_BYTES),
                  "the staged Q panels must fit in the K/V ring");
    static constexpr uint32_t TMEM_COLS = COLS_USED <= 32 ? 32 : COLS_USED <= 64 ? 64
                                        : COLS_USED <= 128 ? 128 : COLS_USED <= 256 ? 256 : 512;
    static constexpr int CTAS_PER_SM = (SMEM_BYTES <= 115712 && TMEM_COLS <= 256) ? 2 : 1;
    static_assert(DK % 64 == 0 && DV % 64 == 0, "panels are 64 columns wide");
    static_assert(BN % 32 == 0 && (P_TMEM || BN % 64 == 0), "P in shared memory needs 64-column panels");
    static_assert(COLS_USED <= 512, "tensor memory has 512 columns");
    static_assert(BN <= 256 && DV <= 256, "one MMA instruction covers N <= 256");
    static_assert(SMEM_BYTES <= 232448, "more than the 227 KB a CTA may have");
};

// Running-max growth (in log2 units) tolerated before O and l are rescaled.
// P then stays below 2^8, far inside fp16 range, and the final O/l is exact.
constexpr float kLazyRescaleLog2 = 8.0f;

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, Cfg::CTAS_PER_SM)
sdpa_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o, const TcParams p)
{
    constexpr int DK = Cfg::DK, DV = Cfg::DV, BN = Cfg::BN, NS = Cfg::NS, NSV = Cfg::NSV, BM = Cfg::BM;
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = ptx::smem_u32(smem);
    const uint32_t q_s = sbase + Cfg::OFF_Q, k_s = sbase + Cfg::OFF_K, v_s = sbase + Cfg::OFF_V;
    const uint32_t p_s = sbase + Cfg::OFF_P;
    const uint32_t bar0 = sbase + Cfg::OFF_BAR;
    const uint32_t q_full = bar0, s_full = bar0 + 8, s_free = bar0 + 16, p_full = bar0 + 24,
                   pv_done = bar0 + 32, q_tmem = bar0 + 40;
    const uint32_t k_full = bar0 + 48, k_empty = k_full + 8 * NS, v_full = k_empty + 8 * NS,
                   v_empty = v_full + 8 * NSV;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + Cfg::OFF_TMEM);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + Cfg::OFF_ABORT);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // section profile: `tick(i)` adds the cycles since the previous tick to counter i
    const bool prof_on = Cfg::PROF && p.prof != nullptr && blockIdx.x == 0;
    long long prof_last = 0;
    long long prof_acc[12] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
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
    // Work item of this CTA (1-D grid): the value-column parts of a query tile side by side, then slabs in groups
    // with every slab's longest items first inside a group (late causal query tiles walk most keys), as in
    // sdpa_tc_pair_kernel; p.n_pairs counts this kernel's query tiles per slab.
    const int zparts = p.dv_total / DV;
    const int item = (int)blockIdx.x / zparts;
    const int span = p.group * p.n_pairs;
    const int grp = item / span, rem = item % span;
    const int in_grp = min(p.group, p.BH - grp * p.group);
    const int q_tile = p.n_pairs - 1 - rem / in_grp;
    const int q0 = q_tile * BM;
    const int bh = grp * p.group + rem % in_grp;
    const int dv0 = ((int)blockIdx.x % zparts) * DV;           // first value column of this CTA
    const int b = bh / p.Hq, h = bh % p.Hq;
    const int kvh = b * p.Hkv + h / (p.Hq / p.Hkv);

    int kv_limit = p.Sk;                                   // keys any row of this batch may see
    if (p.kv_lens) kv_limit = min(kv_limit, max(p.kv_lens[b], 0));
    int kv_end = kv_limit;                                 // keys this query tile may see
    if (p.causal) kv_end = min(kv_end, q0 + BM);
    const int n_tiles = (kv_end + BN - 1) / BN;

    if (tid == 0) {
        *abort_flag = 0;
        ptx::mbar_init(q_full, 1);
        ptx::mbar_init(q_tmem, Cfg::SOFTMAX_WARPS);
        ptx::mbar_init(s_full, 1);
        ptx::mbar_init(s_free, Cfg::SOFTMAX_WARPS);     // one arrival per softmax warp
        ptx::mbar_init(p_full, Cfg::SOFTMAX_WARPS);
        ptx::mbar_init(pv_done, 1);
        for (int s = 0; s < NS; ++s) {
            ptx::mbar_init(k_full + 8 * s, 1);
            ptx::mbar_init(k_empty + 8 * s, 1);
        }
        for (int s = 0; s < NSV; ++s) {
            ptx::mbar_init(v_full + 8 * s, 1);
            ptx::mbar_init(v_empty + 8 * s, 1);
        }
        ptx::fence_mbar_init();
        if (sbase & 1023u) {
            *abort_flag = 1;
            atomicCAS(p.status, 0, TC_ERR_ALIGN);
        } else if (n_tiles > 0) {
            // The Q tile is requested before the CTA meets: the tensor-memory allocation and the meeting then
            // run under the load's latency instead of in front of it.
            ptx::prefetch_tmap(&tm_q);
            ptx::prefetch_tmap(&tm_k);
            ptx::prefetch_tmap(&tm_v);
            ptx::mbar_arrive_expect_tx(q_full, Cfg::Q_BYTES);
#pragma unroll
            for (int pn = 0; pn < Cfg::KP; ++pn) {
                const uint32_t dst = (Cfg::Q_ALIAS && pn < Cfg::QP_TMEM)
                                         ? k_s + pn * (BM * 128)                           // staged in the ring
                                         : q_s + (pn - Cfg::QP_SKIP) * (BM * 128);
                ptx::tma_load_3d(dst, &tm_q, q_full, pn * 64, q0, bh);
            }
        }
        // another CTA of this (or an earlier, unchecked) launch already gave up: do not start (asked after the
        // load is out: the answer takes a trip to global memory; the load lands during the teardown's grace period)
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
    const uint32_t tmem_p = tmem + Cfg::COL_P;
    const bool run = (*abort_flag == 0) && n_tiles > 0;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        // The whole warp walks the loop with identical values (so addresses, coordinates and
        // barrier handles stay in uniform registers); one elected lane issues the copies.
        if (run) {
            const bool leader = ptx::elect_one();
            bool ok = true;
            if constexpr (Cfg::Q_ALIAS) ok = ptx::mbar_wait(q_tmem, 0, abort_flag);   // the ring is free once Q has been copied out
            tick_start();
            const long long t_begin = Cfg::PROF ? clock64() : 0;
            if constexpr (Cfg::LD_SPLIT) {
                // Two queues polled in turn; neither blocks the other.  A stage's "empty" phase
                // cannot flip again before this warp re-arms it, so any lane seeing it is enough.
                int jk = 0, jv = 0;
                uint64_t t_idle = 0;
                uint32_t spins = 0;
                while ((jk < n_tiles || jv < n_tiles) && ok) {
                    bool moved = false;
                    if (jk < n_tiles) {
                        const int s = jk % NS;
                        const uint32_t ph = (uint32_t)(jk / NS) & 1u;
                        if (__any_sync(0xffffffffu, ptx::mbar_test_wait(k_empty + 8 * s, ph ^ 1u))) {
                            if (leader) {
                                ptx::mbar_arrive_expect_tx(k_full + 8 * s, Cfg::K_BYTES);
#pragma unroll
                                for (int pn = 0; pn < Cfg::KP; ++pn)
                                    ptx::tma_load_3d(k_s + s * Cfg::K_BYTES + pn * Cfg::KV_PANEL, &tm_k,
                                                     k_full + 8 * s, pn * 64, jk * BN, kvh);
                            }
                            __syncwarp();
                            ++jk;
                            moved = true;
                        }
                    }
                    if (jv < n_tiles) {
                        const int sv_ = jv % NSV;
                        const uint32_t phv = (uint32_t)(jv / NSV) & 1u;
                        if (__any_sync(0xffffffffu, ptx::mbar_test_wait(v_empty + 8 * sv_, phv ^ 1u))) {
                            if (leader) {
                                ptx::mbar_arrive_expect_tx(v_full + 8 * sv_, Cfg::V_BYTES);
#pragma unroll
                                for (int pn = 0; pn < Cfg::VP; ++pn)
                                    ptx::tma_load_3d(v_s + sv_ * Cfg::V_BYTES + pn * Cfg::KV_PANEL, &tm_v,
                                                     v_full + 8 * sv_, dv0 + pn * 64, jv * BN, kvh);
                            }
                            __syncwarp();
                            ++jv;
                            moved = true;
                        }
                    }
                    if (moved) { spins = 0; t_idle = 0; }
                    else if ((++spins & 127u) == 0u) {
                        if (*abort_flag) ok = false;
                        const uint64_t now = ptx::global_timer_ns();
                        if (t_idle == 0) t_idle = now;
                        else if (now - t_idle > kWaitLimitNs) ok = false;
                    }
                }
            } else {
                for (int j = 0; j < n_tiles && ok; ++j) {
                    const int s = j % NS;
                    const uint32_t ph = (uint32_t)(j / NS) & 1u;
                    tick(0);
                    ok = ptx::mbar_wait(k_empty + 8 * s, ph ^ 1u, abort_flag);
                    tick(1);
                    if (!ok) break;
                    if (leader) {
                        ptx::mbar_arrive_expect_tx(k_full + 8 * s, Cfg::K_BYTES);
#pragma unroll
                        for (int pn = 0; pn < Cfg::KP; ++pn)
                            ptx::tma_load_3d(k_s + s * Cfg::K_BYTES + pn * Cfg::KV_PANEL, &tm_k,
                                             k_full + 8 * s, pn * 64, j * BN, kvh);
                    }
                    __syncwarp();
                    const int sv_ = j % NSV;
                    const uint32_t phv = (uint32_t)(j / NSV) & 1u;
                    tick(0);
                    ok = ptx::mbar_wait(v_empty + 8 * sv_, phv ^ 1u, abort_flag);
                    tick(2);
                    if (!ok) break;
                    if (leader) {
                        ptx::mbar_arrive_expect_tx(v_full + 8 * sv_, Cfg::V_BYTES);
#pragma unroll
                        for (int pn = 0; pn < Cfg::VP; ++pn)
                            ptx::tma_load_3d(v_s + sv_ * Cfg::V_BYTES + pn * Cfg::KV_PANEL, &tm_v,
                                             v_full + 8 * sv_, dv0 + pn * 64, j * BN, kvh);
                    }
                    __syncwarp();
                }
            }
            if (!ok && leader) { *abort_flag = 1; atomicCAS(p.status, 0, TC_ERR_PRODUCER); }
            if constexpr (Cfg::PROF) {
                if (prof_on && leader) {
                    p.prof[SEC_LD_TOTAL] = clock64() - t_begin;
                    p.prof[SEC_LD_WAIT_K] = prof_acc[1];
                    p.prof[SEC_LD_WAIT_V] = prof_acc[2];
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // Warp-uniform control flow (descriptors live in uniform registers); one elected lane,
        // the same one every time, issues the MMAs and the commits that track them.
        if (run) {
            const bool leader = ptx::elect_one();
            constexpr uint32_t idesc_qk = ptx::idesc_f16(BM, BN, false);
            constexpr uint32_t idesc_pv = ptx::idesc_f16(BM, DV, true);
            const uint32_t t_s = tmem + Cfg::COL_S, t_o = tmem + Cfg::COL_O, t_p = tmem_p;
            // Descriptors are formed once; inside the loops a descriptor is one 32-bit add away.
            constexpr uint32_t desc_hi = ptx::smem_desc_sw128_hi(1024);
            const uint32_t q_lo = ptx::smem_desc_sw128_lo(q_s, 16);
            const uint32_t k_lo = ptx::smem_desc_sw128_lo(k_s, 16);
            const uint32_t v_lo = ptx::smem_desc_sw128_lo(v_s, Cfg::KV_PANEL);
            const uint32_t p_lo = ptx::smem_desc_sw128_lo(p_s, 16);
            bool ok = ptx::mbar_wait(q_full, 0, abort_flag);
            if constexpr (Cfg::QT > 0) {
                if (ok) ok = ptx::mbar_wait(q_tmem, 0, abort_flag);
                ptx::tc_fence_after_sync();
            }
            const uint32_t t_q = tmem + Cfg::COL_Q;
            auto issue_qk = [&](int j) -> bool {
                const int s = j % NS;
                const uint32_t ph = (uint32_t)(j / NS) & 1u;
                if (!ptx::mbar_wait(k_full + 8 * s, ph, abort_flag)) return false;
                ptx::tc_fence_after_sync();
                const uint32_t ks_lo = k_lo + (uint32_t)s * (Cfg::K_BYTES >> 4);
                if (leader) {
#pragma unroll
                    for (int kk = 0; kk < DK / 16; ++kk) {
                        const uint32_t qa = (((kk >> 2) - (kk * 8 < Cfg::QT ? 0 : Cfg::QP_SKIP)) * (BM * 128) + (kk & 3) * 32) >> 4;
                        const uint32_t kb = ((kk >> 2) * Cfg::KV_PANEL + (kk & 3) * 32) >> 4;
                        if (kk * 8 < Cfg::QT)
                            ptx::mma_ts(t_s, t_q + kk * 8, ptx::make_desc(ks_lo + kb, desc_hi), idesc_qk, kk > 0);
                        else
                            ptx::mma_ss(t_s, ptx::make_desc(q_lo + qa, desc_hi), ptx::make_desc(ks_lo + kb, desc_hi),
                                        idesc_qk, kk > 0);
                    }
                    ptx::mma_commit(k_empty + 8 * s);
                    ptx::mma_commit(s_full);
                }
                __syncwarp();
                return true;
            };
            if (ok) ok = issue_qk(0);
            tick_start();
            const long long t_begin = Cfg::PROF ? clock64() : 0;
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (j + 1 < n_tiles) {
                    tick(0);
                    ok = ptx::mbar_wait(s_free, (uint32_t)j & 1u, abort_flag);
                    tick(1);
                    if (!ok) break;
                    ptx::tc_fence_after_sync();
                    ok = issue_qk(j + 1);
                    tick(2);
                    if (!ok) break;
                }
                const int s = j % NSV;
                const uint32_t ph = (uint32_t)(j / NSV) & 1u;
                tick(0);
                ok = ptx::mbar_wait(v_full + 8 * s, ph, abort_flag);
                tick(3);
                if (!ok) break;
                ok = ptx::mbar_wait(p_full, (uint32_t)j & 1u, abort_flag);
                tick(4);
                if (!ok) break;
                ptx::tc_fence_after_sync();
                const uint32_t vs_lo = v_lo + (uint32_t)s * (Cfg::V_BYTES >> 4);
                if (leader) {
#pragma unroll
                    for (int kk = 0; kk < BN / 16; ++kk) {
                        // V stage: DV/64 panels of [BN keys][64 cols]; 16 keys = 2 KB further down
                        const uint64_t bdesc = ptx::make_desc(vs_lo + kk * ((16 * 128) >> 4), desc_hi);
                        const uint32_t acc = (j > 0 || kk > 0) ? 1u : 0u;
                        if constexpr (Cfg::P_TMEM) {
                            ptx::mma_ts(t_o, t_p + kk * 8, bdesc, idesc_pv, acc);
                        } else {
                            const uint32_t pa = ((kk >> 2) * (BM * 128) + (kk & 3) * 32) >> 4;
                            ptx::mma_ss(t_o, ptx::make_desc(p_lo + pa, desc_hi), bdesc, idesc_pv, acc);
                        }
                    }
                    ptx::mma_commit(v_empty + 8 * s);
                    ptx::mma_commit(pv_done);
                }
                __syncwarp();
                tick(5);
            }
            if (!ok && leader) { *abort_flag = 1; atomicCAS(p.status, 0, TC_ERR_MMA); }
            if constexpr (Cfg::PROF) {
                if (prof_on && leader) {
                    p.prof[SEC_MMA_TOTAL] = clock64() - t_begin;
                    p.prof[SEC_MMA_WAIT_SFREE] = prof_acc[1];
                    p.prof[SEC_MMA_QK] = prof_acc[2];
                    p.prof[SEC_MMA_WAIT_V] = prof_acc[3];
                    p.prof[SEC_MMA_WAIT_P] = prof_acc[4];
                    p.prof[SEC_MMA_PV] = prof_acc[5];
                }
            }
        }
    } else {
        // ------------------------------------------------------------ softmax + epilogue
        const int quarter = warp & 3;                    // tensor-memory lanes this warp may touch
        const int r = quarter * 32 + lane;               // row inside the tile
        const int row = q0 + r;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const uint32_t t_s = tmem + lane_base + Cfg::COL_S;
        const uint32_t t_o = tmem + lane_base + Cfg::COL_O;
        const uint32_t t_p = tmem_p + lane_base;
        const float scale = p.scale_log2;
        float m_used = -1.0e30f;   // finite stand-in for "no key seen yet"
        float l = 0.f;
        bool ok = run;
        // Every lane polls the same barrier with the same instruction, so the answer is the same
        // for the whole warp and the .sync.aligned tensor-memory instructions that follow are
        // executed by all of it (polling from one lane and broadcasting cost more than it saved).
        auto wait_all = [&](uint32_t bar, uint32_t parity) -> bool {
            return ptx::mbar_wait(bar, parity, abort_flag);
        };
        // Every lane has fenced its own tensor-memory / shared-memory writes; one lane
        // then arrives for the warp.
        auto arrive_warp = [&](uint32_t bar) {
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar);
        };
        if constexpr (Cfg::QT > 0) {
            // Copy this thread's Q row (its first 2*QT elements) from the swizzled panels in shared
            // memory into tensor memory, where the QK^T MMAs read it as their A operand.
            if (ok) ok = wait_all(q_full, 0);
            if (ok) {
#pragma unroll 1
                for (int pn = 0; pn < Cfg::QT / 32; ++pn) {
                    uint32_t qv[32];
                    const uint32_t rowaddr = (Cfg::Q_ALIAS ? k_s : q_s) + (uint32_t)pn * (BM * 128) + (uint32_t)r * 128;
#pragma unroll
                    for (int c = 0; c < 8; ++c)
                        ptx::ld_shared_v4(rowaddr + (uint32_t)((c ^ (r & 7)) << 4), qv[4 * c], qv[4 * c + 1],
                                          qv[4 * c + 2], qv[4 * c + 3]);
                    ptx::tmem_st_cols<32>(tmem + lane_base + Cfg::COL_Q + (uint32_t)pn * 32, qv);
                }
                ptx::tmem_wait_st();
            }
            arrive_warp(q_tmem);
        }
        tick_start();
        const long long t_begin = Cfg::PROF ? clock64() : 0;
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int kv0 = j * BN;
            tick(0);
            ok = wait_all(s_full, (uint32_t)j & 1u);
            tick(SEC_SM_WAIT_S);
            if (!ok) break;
            ptx::tc_fence_after_sync();
            // this thread's part of the S row in registers, one wait; then S belongs to the MMA warp again
            uint32_t sv[BN];
            ptx::tmem_ld_cols<BN>(t_s, sv);
            ptx::tmem_wait_ld();
            ptx::reg_fence_cols<BN>(sv);
            arrive_warp(s_free);
            tick(SEC_SM_LOAD_S);

            const bool need_mask = (j * BN + BN > kv_limit) || (p.causal && (j * BN + BN - 1 > q0));
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
            tick(SEC_SM_MAX);
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
                const float2 xa = __ffma2_rn(make_float2(__uint_as_float(sv[i]), __uint_as_float(sv[i + 1])),
                                             scale2, negm2);
                const float2 xb = __ffma2_rn(make_float2(__uint_as_float(sv[i + 2]), __uint_as_float(sv[i + 3])),
                                             scale2, negm2);
                // which elements of a group of 16 go to the polynomial is fixed at compile time
                const int e0 = i & 15;
                const bool pa_x = (Cfg::POLY >> e0) & 1, pa_y = (Cfg::POLY >> (e0 + 1)) & 1;
                const bool pb_x = (Cfg::POLY >> (e0 + 2)) & 1, pb_y = (Cfg::POLY >> (e0 + 3)) & 1;
                // a pair that goes to the polynomial as a whole is evaluated two-wide
                const float2 ea = (pa_x && pa_y) ? ptx::ex2_poly2(xa)
                                  : make_float2(pa_x ? ptx::ex2_poly(xa.x) : ptx::ex2_approx(xa.x),
                                                pa_y ? ptx::ex2_poly(xa.y) : ptx::ex2_approx(xa.y));
                const float2 eb = (pb_x && pb_y) ? ptx::ex2_poly2(xb)
                                  : make_float2(pb_x ? ptx::ex2_poly(xb.x) : ptx::ex2_approx(xb.x),
                                                pb_y ? ptx::ex2_poly(xb.y) : ptx::ex2_approx(xb.y));
                sum_a = __fadd2_rn(sum_a, ea);
                sum_b = __fadd2_rn(sum_b, eb);
                pk[i / 2] = ptx::pack_half2(ea.x, ea.y);
                pk[i / 2 + 1] = ptx::pack_half2(eb.x, eb.y);
            }
            l = l * alpha + ((sum_a.x + sum_a.y) + (sum_b.x + sum_b.y));
            tick(SEC_SM_EXP);
            if (j > 0) {
                // PV of the previous tile must be finished before P is overwritten or O rescaled
                ok = wait_all(pv_done, (uint32_t)(j - 1) & 1u);
                tick(SEC_SM_WAIT_PV);
                if (!ok) break;
                ptx::tc_fence_after_sync();
                if (__any_sync(0xffffffffu, alpha != 1.0f)) {
                    // rare after the first tiles; 16 columns at a time so the score row stays in registers
#pragma unroll 1
                    for (int c = 0; c < DV / 16; ++c) {
                        uint32_t o[16];
                        ptx::tmem_ld16(t_o + c * 16, o);
                        ptx::tmem_wait_ld();
                        ptx::reg_fence16(o);
#pragma unroll
                        for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        ptx::tmem_st16(t_o + c * 16, o);
                    }
                    ptx::tmem_wait_st();
                }
                tick(SEC_SM_RESCALE);
            }
            if constexpr (Cfg::P_TMEM) {
                ptx::tmem_st_cols<BN / 2>(t_p, pk);
                ptx::tmem_wait_st();
            } else {
                // row r of P: 64-column panels, each row 128 bytes = 8 chunks of 8 halves, chunk ^= r%8
#pragma unroll
                for (int q = 0; q < BN / 8; ++q) {
                    const int ch = q;
                    const uint32_t addr = p_s + (ch >> 3) * (BM * 128) + r * 128 +
                                          (((uint32_t)(ch & 7) ^ (uint32_t)(r & 7)) << 4);
                    ptx::st_shared_v4(addr, pk[q * 4], pk[q * 4 + 1], pk[q * 4 + 2], pk[q * 4 + 3]);
                }
                ptx::fence_proxy_async_smem();
            }
            arrive_warp(p_full);
            tick(SEC_SM_STORE_P);
        }
        const long long t_loop_end = Cfg::PROF ? clock64() : 0;
        if (run && ok) {
            ok = wait_all(pv_done, (uint32_t)(n_tiles - 1) & 1u);
            if (ok) {
                ptx::tc_fence_after_sync();
                const float inv_l = 1.0f / l;    // l == 0 (no visible key) -> inf -> NaN rows, as the reference
                if (p.lse && dv0 == 0 && row < p.Sq) p.lse[(size_t)bh * p.Sq + row] = m_used + __log2f(l);
                // O leaves through shared memory and one bulk tensor store per 128-byte-wide chunk of this warp's
                // 32 rows (a thread owns a row: direct stores would put 32 rows' 16-byte pieces into every store
                // instruction).  Staging: two 4 KB chunk buffers per warp in the K ring, which nothing uses any
                // more (the last pv_done says every MMA has completed), written in the tensor map's 128-byte swizzle.
                constexpr uint32_t CHUNK_BYTES = 32 * 128;
                static_assert(NS * Cfg::K_BYTES >= 8 * CHUNK_BYTES, "staging space");
                const int quarter = warp & 3;
                const uint32_t buf_a = k_s + (uint32_t)quarter * (2 * CHUNK_BYTES), buf_b = buf_a + CHUNK_BYTES;
                const int row0 = q0 + quarter * 32;
                const uint32_t my_line = (uint32_t)lane * 128u;
                const uint32_t sw = (uint32_t)(lane & 7);
                auto put = [&](uint32_t buf, int piece, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
                    ptx::st_shared_v4(buf + my_line + (((uint32_t)piece ^ sw) << 4), x, y, z, w);
                };
                auto send = [&](uint32_t buf, int col) {
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0 && row0 < p.Sq) {
                        ptx::tma_store_3d(&tm_o, buf, dv0 + col, row0, bh);
                        ptx::tma_store_commit();
                    }
                };
                auto reuse = [&](int step) {                        // both buffers were sent in the step before
                    if (step > 0) {
                        if (lane == 0) ptx::tma_store_wait_read<0>();
                        __syncwarp();
                    }
                };
#pragma unroll
                for (int c = 0; c < DV / 64; ++c) {
                    uint32_t o[32], o2[32];
                    ptx::tmem_ld32(t_o + c * 64, o);
                    ptx::tmem_ld32(t_o + c * 64 + 32, o2);
                    ptx::tmem_wait_ld();
                    ptx::reg_fence32(o);
                    ptx::reg_fence32(o2);
                    if (p.out_f16) {
                        const uint32_t buf = (c & 1) ? buf_b : buf_a;
                        if ((c & 1) == 0) reuse(c);
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
                        reuse(c);
                        auto f = [&](uint32_t a) { return __float_as_uint(__uint_as_float(a) * inv_l); };
#pragma unroll
                        for (int i = 0; i < 32; i += 4) put(buf_a, i / 4, f(o[i]), f(o[i + 1]), f(o[i + 2]), f(o[i + 3]));
                        send(buf_a, c * 64);
#pragma unroll
                        for (int i = 0; i < 32; i += 4) put(buf_b, i / 4, f(o2[i]), f(o2[i + 1]), f(o2[i + 2]), f(o2[i + 3]));
                        send(buf_b, c * 64 + 32);
                    }
                }
                if (lane == 0) ptx::tma_store_wait_read<0>();   // shared memory must outlive the stores' reads
                __syncwarp();
            }
        }
        if (run && !ok) { *abort_flag = 1; atomicCAS(p.status, 0, TC_ERR_SOFTMAX); }
        if constexpr (Cfg::PROF) {
            if (prof_on && warp == 2 && lane == 0) {
                p.prof[SEC_SM_TOTAL] = t_loop_end - t_begin;
                for (int i = 1; i <= 8; ++i) p.prof[i] = prof_acc[i];
                p.prof[SEC_SM_EPILOGUE] = clock64() - t_loop_end;
                p.prof[SEC_SM_TILES] = n_tiles;
            }
        }
        if (!run && *abort_flag == 0 && row < p.Sq) {
            // no visible key at all for this tile: the reference's 0/0
            const size_t obase = ((size_t)bh * p.Sq + row) * p.dv_total + dv0;
            if (p.out_f16) {
                __half *orow_h = static_cast<__half *>(p.out) + obase;
                for (int i = 0; i < DV; ++i) orow_h[i] = __ushort_as_half((unsigned short)0x7e00);
            } else {
                float *orow = static_cast<float *>(p.out) + obase;
                for (int i = 0; i < DV; ++i) orow[i] = __int_as_float(0x7fc00000);
            }
            if (p.lse && dv0 == 0) p.lse[(size_t)bh * p.Sq + row] = __int_as_float(0x7fc00000);
        }
    }

    // ---------------------------------------------------------------- teardown
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        // A wait ran out somewhere in this CTA (or in an earlier one of the launch): its rows are not valid.
        // They are overwritten with NaN so that the failure is visible in the data, not only in the status word.
        if (warp >= 2) {
            const int row_a = q0 + (warp & 3) * 32 + lane;
            if (row_a < p.Sq) {
                const size_t ob = ((size_t)bh * p.Sq + row_a) * p.dv_total + dv0;
                for (int i = 0; i < DV; ++i) {
                    if (p.out_f16) static_cast<__half *>(p.out)[ob + i] = __ushort_as_half((unsigned short)0x7e00);
                    else static_cast<float *>(p.out)[ob + i] = __int_as_float(0x7fc00000);
                }
            }
        }
        // give copies that may still be in flight time to land before the CTA's memory goes away
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
        __syncthreads();
    }
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem, Cfg::TMEM_COLS);
    }
}

}  // namespace txb
