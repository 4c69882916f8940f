// C ABI of the B200 SDPA forward path: validation, kernel selection, launch.
// Declarations and the reference interfaces they replace: include/tensorax_b200.h.
#include "../../include/tensorax_b200.h"

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

// NVTX ranges around the entry points, as the reference's launchers have them
// (csrc/cuda/profiling.cuh:7-18: scoped ranges when the NVTX header is present, nothing otherwise).
#if defined(__has_include)
#if __has_include(<nvtx3/nvtx3.hpp>)
#include <nvtx3/nvtx3.hpp>
#define TX_NVTX_RANGE(name) ::nvtx3::scoped_range tx_nvtx_range_{(name)}
#endif
#endif
#ifndef TX_NVTX_RANGE
#define TX_NVTX_RANGE(name) ((void)0)
#endif

#include "linear_simt.cuh"
#include "linear_tc.cuh"
#include "sdpa_simt.cuh"
#include "sdpa_tc.cuh"
#include "sdpa_tc_pair.cuh"
#include "sdpa_tc_x3.cuh"
#include "sdpa_bwd.cuh"

namespace {

thread_local std::string g_err;
std::atomic<int64_t> g_launches{0};

int fail(int code, const char *fmt, ...)
{
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_err = buf;
    return code;
}

#define TX_CUDA(call)                                                                     \
    do {                                                                                  \
        cudaError_t e_ = (call);                                                          \
        if (e_ != cudaSuccess)                                                            \
            return fail(TX_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e_));     \
    } while (0)

int ensure_device()
{
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0) {
        (void)cudaGetLastError();
        return fail(TX_ERR_NO_DEVICE, "no CUDA device available (%s)",
                    e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
    }
    return TX_OK;
}

constexpr int kMaxDevices = 64;
int pool_ready();

// Workspace of one call from the device's stream-ordered pool.  pool_ready() first: with the pool's default release
// threshold of zero every synchronisation hands the freed workspace back to the driver, and the next call pays for
// mapping it again (2.5 ms for 400 MB).
int pool_alloc(char **p, size_t bytes, cudaStream_t st)
{
    if (int rc = pool_ready()) return rc;
    TX_CUDA(cudaMallocAsync(reinterpret_cast<void **>(p), bytes, st));
    return TX_OK;
}

// One status word per device, written by kernels whose bounded waits run out.
int *g_status[kMaxDevices] = {};
std::mutex g_status_mu;

int status_word(int **out)
{
    int dev = 0;
    TX_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(TX_ERR_INVALID, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lk(g_status_mu);
    if (!g_status[dev]) {
        int *w = nullptr;
        TX_CUDA(cudaMalloc(&w, 256));
        TX_CUDA(cudaMemset(w, 0, 256));
        g_status[dev] = w;
    }
    *out = g_status[dev];
    return TX_OK;
}

// ------------------------------------------------------------------ TMA descriptors
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                   const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                   const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int get_encode_fn(EncodeTiledFn *fn)
{
    static EncodeTiledFn cached = nullptr;
    if (!cached) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        TX_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q));
        if (!sym || q != cudaDriverEntryPointSuccess)
            return fail(TX_ERR_CUDA, "driver does not provide cuTensorMapEncodeTiled");
        cached = reinterpret_cast<EncodeTiledFn>(sym);
    }
    *fn = cached;
    return TX_OK;
}

// fp16 (or fp32: elem_bytes 4) tensor [slabs, rows, d] -> 3-D map (d, rows, slabs); box = 128 bytes of a row x
// box_rows, 128B swizzle.
// A map is a pure function of (base, slabs, rows, d, box_rows): the last few are kept per host thread, so a
// caller that runs the same buffers again (a decoding loop, a benchmark) does not pay the driver's encode
// call three times per launch.
struct MapKey {
    const void *base;
    int64_t slabs, rows, d;
    int box_rows, elem_bytes;
    bool operator==(const MapKey &o) const
    {
        return base == o.base && slabs == o.slabs && rows == o.rows && d == o.d && box_rows == o.box_rows &&
               elem_bytes == o.elem_bytes;
    }
};
constexpr int kMapCache = 16;
struct MapCache {
    MapKey key[kMapCache] = {};
    CUtensorMap map[kMapCache];
    bool used[kMapCache] = {};
    int next = 0;
};
thread_local MapCache g_map_cache;

int make_map(CUtensorMap *m, const void *base, int64_t slabs, int64_t rows, int64_t d, int box_rows, int elem_bytes = 2)
{
    const MapKey key{base, slabs, rows, d, box_rows, elem_bytes};
    MapCache &mc = g_map_cache;
    for (int i = 0; i < kMapCache; ++i)
        if (mc.used[i] && mc.key[i] == key) {
            *m = mc.map[i];
            return TX_OK;
        }
    EncodeTiledFn enc;
    if (int rc = get_encode_fn(&enc)) return rc;
    cuuint64_t dims[3] = {(cuuint64_t)d, (cuuint64_t)rows, (cuuint64_t)slabs};
    const cuuint64_t eb = (cuuint64_t)elem_bytes;
    cuuint64_t strides[2] = {(cuuint64_t)d * eb, (cuuint64_t)rows * (cuuint64_t)d * eb};
    cuuint32_t box[3] = {(cuuint32_t)(128 / elem_bytes), (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(m, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                     const_cast<void *>(base), dims, strides,
                     box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(TX_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    mc.key[mc.next] = key;
    mc.map[mc.next] = *m;
    mc.used[mc.next] = true;
    mc.next = (mc.next + 1) % kMapCache;
    return TX_OK;
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per kernel (by entry address) and device.
std::mutex g_smem_mu;
std::vector<std::pair<const void *, int>> g_smem_done;
template <class Kernel>
int allow_smem(Kernel kernel, int bytes)
{
    int dev = 0;
    TX_CUDA(cudaGetDevice(&dev));
    const std::pair<const void *, int> key(reinterpret_cast<const void *>(kernel), dev);
    std::lock_guard<std::mutex> lk(g_smem_mu);
    if (std::find(g_smem_done.begin(), g_smem_done.end(), key) != g_smem_done.end()) return TX_OK;
    TX_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    g_smem_done.push_back(key);
    return TX_OK;
}

// Multiprocessors of the current device (asked once per device).
int sm_count(int *n)
{
    static std::mutex mu;
    static std::vector<std::pair<int, int>> seen;
    int dev = 0;
    TX_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(mu);
    for (const auto &e : seen)
        if (e.first == dev) { *n = e.second; return TX_OK; }
    int v = 0;
    TX_CUDA(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev));
    seen.emplace_back(dev, v);
    *n = v;
    return TX_OK;
}

// fp32 tensor maps of the linear layer: 128-byte-swizzled boxes of 32 floats x `box_rows` rows.
int make_map_f32(CUtensorMap *m, const void *base, int rank, const cuuint64_t *dims, const cuuint64_t *strides,
                 int box_rows)
{
    EncodeTiledFn enc;
    if (int rc = get_encode_fn(&enc)) return rc;
    cuuint32_t box[4] = {32, (cuuint32_t)box_rows, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank, const_cast<void *>(base), dims, strides,
                     box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(TX_ERR_CUDA, "cuTensorMapEncodeTiled (fp32) failed with code %d", (int)r);
    return TX_OK;
}

// ------------------------------------------------------------------ validation
bool tc_eligible(const tx_sdpa_desc *d);

int validate(const tx_sdpa_desc *d)
{
    if (!d) return fail(TX_ERR_INVALID, "SDPA: null descriptor");
    if (!d->q || !d->k || !d->v || !d->out)
        return fail(TX_ERR_INVALID, "SDPA: Query, Key, Value and output pointers must not be null");
    if (d->batch <= 0 || d->q_heads <= 0 || d->kv_heads <= 0 || d->seq_q <= 0 || d->seq_k <= 0 ||
        d->d_k <= 0 || d->d_v <= 0)
        return fail(TX_ERR_INVALID, "SDPA: every dimension must be positive");
    if (d->q_heads % d->kv_heads != 0)
        return fail(TX_ERR_INVALID, "SDPA: Key dimensions don't match Query (q_heads %lld not a multiple of kv_heads %lld)",
                    (long long)d->q_heads, (long long)d->kv_heads);
    if (d->dtype != TX_DTYPE_F32 && d->dtype != TX_DTYPE_F16)
        return fail(TX_ERR_INVALID, "SDPA: dtype must be float32 or float16");
    if (d->batch * d->q_heads > 0x7fffffffLL / 2 || d->seq_q > 0x3fffffffLL || d->seq_k > 0x3fffffffLL)
        return fail(TX_ERR_UNSUPPORTED, "SDPA: dimension too large");
    if (d->lse && !tc_eligible(d))
        return fail(TX_ERR_UNSUPPORTED, "SDPA: the log-sum-exp output is written by the tensor-core kernel only "
                                        "(fp16, no dense mask, d_k == d_v in {64,128,256,512})");
    return TX_OK;
}

bool tc_eligible(const tx_sdpa_desc *d)
{
    if (d->flags & TX_SDPA_FORCE_SIMT) return false;
    if (d->dtype != TX_DTYPE_F16 || d->mask) return false;
    if (d->d_k != d->d_v) return false;
    if (d->d_k != 64 && d->d_k != 128 && d->d_k != 256 && d->d_k != 512) return false;
    auto al = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    if (!al(d->q) || !al(d->k) || !al(d->v) || !al(d->out)) return false;
    if (d->batch * d->q_heads > 65535) return false;   // grid.y
    return true;
}

// ------------------------------------------------------------------ launches
template <typename T, int DVC, bool PROF>
int launch_simt_t(const txb::SimtParams &p, cudaStream_t st)
{
    dim3 grid((unsigned)((p.dv + 32 * DVC - 1) / (32 * DVC)),
              (unsigned)((p.Sq + txb::SIMT_BR - 1) / txb::SIMT_BR), (unsigned)(p.B * p.Hq));
    txb::sdpa_simt_kernel<T, DVC, PROF><<<grid, txb::SIMT_THREADS, 0, st>>>(p);
    g_launches++;
    TX_CUDA(cudaGetLastError());
    return TX_OK;
}

template <typename T, bool PROF = false>
int launch_simt(const txb::SimtParams &p, cudaStream_t st)
{
    if (p.B * p.Hq > 65535) return fail(TX_ERR_UNSUPPORTED, "SDPA: batch*heads > 65535");
    if ((p.Sq + txb::SIMT_BR - 1) / txb::SIMT_BR > 65535) return fail(TX_ERR_UNSUPPORTED, "SDPA: seq_len_q too large");
    if (p.dv <= 32) return launch_simt_t<T, 1, PROF>(p, st);
    if (p.dv <= 64) return launch_simt_t<T, 2, PROF>(p, st);
    if (p.dv <= 128) return launch_simt_t<T, 4, PROF>(p, st);
    return launch_simt_t<T, 8, PROF>(p, st);   // wider heads: one CTA column per 256 value columns
}

// Elements (bit e = element e of each group of 16) whose exponential is evaluated by the FMA-pipe
// polynomial at d = 64: two whole pairs of 16 (the polynomial is evaluated two-wide); measured round-robin
// against 0, 1, 3 and 4 pairs of 8.
constexpr int kPolyPairsD64 = 0x0303;
// d = 128: one pair of 16 (0.896 -> 0.880 ms at B4 H8 S8192 against none, 0.884 with two pairs; the medians of
// back-to-back runs move by 4-5 %: fewer special-function instructions also means a cooler part)
constexpr int kPolyPairsD128 = 0x0003;

int causal_group(const tx_sdpa_desc *d, int64_t items_per_slab, int64_t *group);

template <class Cfg>
int launch_tc_t(const tx_sdpa_desc *d, cudaStream_t st, int *status, long long *prof = nullptr)
{
    CUtensorMap tq, tk, tv, to;
    const bool out_f16 = (d->flags & TX_SDPA_OUT_F16) != 0;
    if (int rc = make_map(&tq, d->q, d->batch * d->q_heads, d->seq_q, d->d_k, Cfg::BM)) return rc;
    if (int rc = make_map(&tk, d->k, d->batch * d->kv_heads, d->seq_k, d->d_k, Cfg::BN)) return rc;
    if (int rc = make_map(&tv, d->v, d->batch * d->kv_heads, d->seq_k, d->d_v, Cfg::BN)) return rc;
    // the result leaves in boxes of one softmax warp's 32 rows x 128 bytes
    if (int rc = make_map(&to, d->out, d->batch * d->q_heads, d->seq_q, d->d_v, 32, out_f16 ? 2 : 4)) return rc;
    txb::TcParams p;
    p.out = d->out;
    p.out_f16 = out_f16 ? 1 : 0;
    p.lse = d->lse;
    p.kv_lens = d->kv_lens;
    p.status = status;
    p.Hq = (int)d->q_heads;
    p.Hkv = (int)d->kv_heads;
    p.Sq = (int)d->seq_q;
    p.Sk = (int)d->seq_k;
    p.dv_total = (int)d->d_v;
    p.causal = d->causal ? 1 : 0;
    p.scale_log2 = (1.0f / std::sqrt((float)d->d_k)) * 1.4426950408889634f;
    p.prof = prof;
    p.skip_k_tile = -1;
    const int64_t n_tiles = (d->seq_q + Cfg::BM - 1) / Cfg::BM, slabs = d->batch * d->q_heads, zparts = d->d_v / Cfg::DV;
    int64_t group = 1;
    if (int rc = causal_group(d, n_tiles * zparts, &group)) return rc;
    p.group = (int)group; p.n_pairs = (int)n_tiles; p.BH = (int)slabs;
    if (n_tiles * slabs * zparts > 0x7fffffffLL) return fail(TX_ERR_UNSUPPORTED, "SDPA: more than 2^31 work items");
    if (int rc = allow_smem(txb::sdpa_tc_kernel<Cfg>, (int)Cfg::SMEM_BYTES)) return rc;
    dim3 grid((unsigned)(n_tiles * slabs * zparts), 1, 1);
    txb::sdpa_tc_kernel<Cfg><<<grid, Cfg::THREADS, Cfg::SMEM_BYTES, st>>>(tq, tk, tv, to, p);
    g_launches++;
    TX_CUDA(cudaGetLastError());
    return TX_OK;
}

// Slabs per group of the launch order of a causal call (see launch_two_tiles); 1 = slab-major.  `bytes_per_slab`: what
// the CTAs of one slab stream through L2; `multiple`: slabs that share those bytes and should stay together.
std::atomic<long long> g_group_l2_bytes{48ll << 20};

int launch_group(bool causal, int64_t slabs, int64_t items_per_slab, double bytes_per_slab, int64_t multiple, int64_t *group,
                 int64_t max_waves = 0)
{
    *group = 1;
    int sms = 0;
    if (int rc = sm_count(&sms)) return rc;
    if (!causal || slabs <= 1) return TX_OK;
    if (max_waves > 0 && items_per_slab * slabs > max_waves * sms) return TX_OK;   // a long launch: its tail is small anyway
    const int64_t by_l2 = std::max<int64_t>(1, (int64_t)((double)g_group_l2_bytes.load() / bytes_per_slab));
    const int64_t two_waves = (2 * sms + items_per_slab - 1) / items_per_slab;
    const int64_t want = std::min<int64_t>(slabs, std::max(by_l2, two_waves));
    const int64_t n_groups = (slabs + want - 1) / want;
    const int64_t g = (slabs + n_groups - 1) / n_groups;          // equal groups, none left small at the end
    *group = std::min<int64_t>(slabs, (g + multiple - 1) / multiple * multiple);
    return TX_OK;
}

int causal_group(const tx_sdpa_desc *d, int64_t items_per_slab, int64_t *group)
{
    const int64_t ratio = d->q_heads / d->kv_heads;
    return launch_group(d->causal != 0, d->batch * d->q_heads, items_per_slab,
                        2.0 * (double)d->seq_k * (double)(d->d_k + d->d_v) / (double)ratio, ratio, group);
}

template <class Cfg>
int launch_pair_t(const tx_sdpa_desc *d, cudaStream_t st, int *status, long long *prof = nullptr, int skip_k_tile = -1)
{
    CUtensorMap tq, tk, tv, to;
    const bool out_f16 = (d->flags & TX_SDPA_OUT_F16) != 0;
    if (int rc = make_map(&tq, d->q, d->batch * d->q_heads, d->seq_q, d->d_k, Cfg::BM)) return rc;
    if (int rc = make_map(&tk, d->k, d->batch * d->kv_heads, d->seq_k, d->d_k, Cfg::BN)) return rc;
    if (int rc = make_map(&tv, d->v, d->batch * d->kv_heads, d->seq_k, d->d_v, Cfg::BN)) return rc;
    // the result leaves in boxes of one softmax warp's 32 rows x 128 bytes
    if (int rc = make_map(&to, d->out, d->batch * d->q_heads, d->seq_q, d->d_v, 32, out_f16 ? 2 : 4)) return rc;
    txb::TcParams p;
    p.out = d->out;
    p.out_f16 = out_f16 ? 1 : 0;
    p.lse = d->lse;
    p.kv_lens = d->kv_lens;
    p.status = status;
    p.Hq = (int)d->q_heads;
    p.Hkv = (int)d->kv_heads;
    p.Sq = (int)d->seq_q;
    p.Sk = (int)d->seq_k;
    p.dv_total = (int)d->d_v;
    p.causal = d->causal ? 1 : 0;
    p.scale_log2 = (1.0f / std::sqrt((float)d->d_k)) * 1.4426950408889634f;
    p.prof = prof;
    p.skip_k_tile = skip_k_tile;
    // Work items in launch order.  Slab-major (group = 1: a slab's CTAs, which share its K/V, start side by side)
    // unless the mask is causal: then the slabs are taken in groups, and inside a group every slab's longest items
    // come before any shorter one, so that the SMs do not end on a late slab's long items.  A group is as large as
    // its K/V may be while staying in L2 (48 MB; K/V heads shared by several query heads count once), at least two
    // waves of CTAs, a whole number of K/V heads, and the groups are equal (a small last group is the same tail
    // again: 32 slabs as 10 + 10 + 10 + 2 were slower than slab-major, as 4 x 8 or as one group 12-24 % faster).
    // Measured on B200, causal, slab-major -> grouped: d = 128 B1 Hq32 Hkv8 S8192 0.514 -> 0.468 ms, B1 H16 S8192
    // 0.333 -> 0.253, d = 64 B4 H8 S8192 0.388 -> 0.342, B4 H16 S4096 d = 128 0.286 -> 0.268, d = 64 0.220 -> 0.199,
    // B8 H16 S2048 0.170 -> 0.162; long launches gain less but gain (B8 Hq32 Hkv8 S8192, 55 waves: 3.80 -> 3.73 ms).
    const int64_t n_pairs = (d->seq_q + 2 * Cfg::BM - 1) / (2 * Cfg::BM);
    const int64_t slabs = d->batch * d->q_heads;
    int64_t group = 1;
    if (int rc = causal_group(d, n_pairs, &group)) return rc;
    p.group = (int)group;
    p.n_pairs = (int)n_pairs;
    p.BH = (int)slabs;
    if (n_pairs * slabs > 0x7fffffffLL) return fail(TX_ERR_UNSUPPORTED, "SDPA: more than 2^31 work items");
    if (int rc = allow_smem(txb::sdpa_tc_pair_kernel<Cfg>, (int)Cfg::SMEM_BYTES)) return rc;
    dim3 grid((unsigned)(n_pairs * slabs), 1, 1);
    txb::sdpa_tc_pair_kernel<Cfg><<<grid, Cfg::THREADS, Cfg::SMEM_BYTES, st>>>(tq, tk, tv, to, p);
    g_launches++;
    TX_CUDA(cudaGetLastError());
    return TX_OK;
}

// Kernel and tile shape per head dim.
//   d = 64, 128   sdpa_tc_pair_kernel: one CTA per SM, two 128-row query tiles, 128 keys per tile
//                 (d = 64: four-deep K/V ring, P in its own tensor-memory columns, a quarter of the
//                 exponentials on the FMA pipe; d = 128: two-deep ring, P over S)
//   d = 256       sdpa_tc_kernel, 64 keys per tile, one CTA per SM, Q in tensor memory
//   d = 512       sdpa_tc_kernel, 64 keys per tile, two CTAs split the value columns
// `prof` (section profile) selects the instrumented instantiation of the same shape.
using PairD64 = txb::PairCfg<64, 128, 4, kPolyPairsD64, false>;
using PairD64Prof = txb::PairCfg<64, 128, 4, kPolyPairsD64, false, true>;
using PairD128 = txb::PairCfg<128, 128, 2, kPolyPairsD128, true>;
using PairD128Prof = txb::PairCfg<128, 128, 2, kPolyPairsD128, true, true>;

int launch_tc(const tx_sdpa_desc *d, cudaStream_t st, int *status, long long *prof = nullptr)
{
    const bool p_smem = (d->flags & TX_SDPA_P_IN_SMEM) != 0;
    switch (d->d_k) {
    case 64:
        if (p_smem) return launch_tc_t<txb::TcCfg<64, 64, 128, 2, false>>(d, st, status);
        return prof ? launch_pair_t<PairD64Prof>(d, st, status, prof) : launch_pair_t<PairD64>(d, st, status);
    case 128:
        if (p_smem) return launch_tc_t<txb::TcCfg<128, 128, 64, 2, false>>(d, st, status);
        return prof ? launch_pair_t<PairD128Prof>(d, st, status, prof) : launch_pair_t<PairD128>(d, st, status);
    case 256:
        if (p_smem) return launch_tc_t<txb::TcCfg<256, 256, 64, 2, false>>(d, st, status);
        // Narrow key tiles make the A (Q) read the busiest user of the shared-memory port: Q lives
        // in tensor memory instead, and K / V are fetched as two independent queues.
        if (prof) return launch_tc_t<txb::TcCfg<256, 256, 64, 2, true, true, 0, 2, true, 128>>(d, st, status, prof);
        return launch_tc_t<txb::TcCfg<256, 256, 64, 2, true, false, 0, 2, true, 128>>(d, st, status);
    case 512:
        // All 512 tensor-memory columns: S 64 | O 256 | P 32 | first 320 elements of Q 160.  Those five Q panels
        // are staged in the empty K/V ring, so shared memory holds only Q's last three panels (48 KB) beside
        // two 64-key K stages (128 KB) and one V stage (32 KB): 64-key tiles where 32 fitted before.
        if (prof) return launch_tc_t<txb::TcCfg<512, 256, 64, 2, true, true, 0, 1, true, 160, true>>(d, st, status, prof);
        return launch_tc_t<txb::TcCfg<512, 256, 64, 2, true, false, 0, 1, true, 160, true>>(d, st, status);
    }
    return fail(TX_ERR_UNSUPPORTED, "SDPA: no tensor-core tile shape for d = %lld", (long long)d->d_k);
}

template <int D, class DqCfg, class DkvCfg>
int launch_bwd(const tx_sdpa_bwd_desc *d, cudaStream_t st, int *status, const __half *dout_h, const float *delta)
{
    txb::BwdParams p;
    p.lse = d->lse; p.delta = delta; p.kv_lens = d->kv_lens;
    p.dq = d->dq; p.dk = d->dk; p.dv = d->dv;
    p.status = status;
    p.Hq = (int)d->q_heads; p.Hkv = (int)d->kv_heads; p.Sq = (int)d->seq_q; p.Sk = (int)d->seq_k;
    p.causal = d->causal ? 1 : 0;
    p.scale = 1.0f / std::sqrt((float)D);
    p.scale_log2 = p.scale * 1.4426950408889634f;
    p.group_q = p.group_k = 1;
    p.items_q = p.items_k = p.slabs_q = p.slabs_k = 1;
    {
        CUtensorMap tq, tdo, tk, tv;
        if (int rc = make_map(&tq, d->q, d->batch * d->q_heads, d->seq_q, D, DqCfg::BM)) return rc;
        if (int rc = make_map(&tdo, dout_h, d->batch * d->q_heads, d->seq_q, D, DqCfg::BM)) return rc;
        if (int rc = make_map(&tk, d->k, d->batch * d->kv_heads, d->seq_k, D, DqCfg::BN)) return rc;
        if (int rc = make_map(&tv, d->v, d->batch * d->kv_heads, d->seq_k, D, DqCfg::BN)) return rc;
        TX_CUDA(cudaFuncSetAttribute(txb::sdpa_bwd_dq_kernel<DqCfg>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)DqCfg::SMEM_BYTES));
        // 1-D grid, grouped longest-first order for causal calls (a slab's CTAs stream its K and V)
        const int64_t items = (d->seq_q + DqCfg::BM - 1) / DqCfg::BM, slabs = d->batch * d->q_heads;
        const int64_t ratio = d->q_heads / d->kv_heads;
        int64_t group = 1;
        // (beyond 32 waves the slab-major order was the better one here: B8 Hq32 Hkv8 S4096 d128 4.24 against 4.35 ms)
        if (int rc = launch_group(d->causal != 0, slabs, items, 4.0 * (double)d->seq_k * (double)D / (double)ratio, ratio, &group, 32))
            return rc;
        p.group_q = (int)group; p.items_q = (int)items; p.slabs_q = (int)slabs;
        if (items * slabs > 0x7fffffffLL) return fail(TX_ERR_UNSUPPORTED, "SDPA backward: more than 2^31 work items");
        dim3 grid((unsigned)(items * slabs));
        txb::sdpa_bwd_dq_kernel<DqCfg><<<grid, DqCfg::THREADS, DqCfg::SMEM_BYTES, st>>>(tq, tdo, tk, tv, p);
        g_launches++;
        TX_CUDA(cudaGetLastError());
    }
    {
        CUtensorMap tq, tdo, tk, tv;
        if (int rc = make_map(&tq, d->q, d->batch * d->q_heads, d->seq_q, D, DkvCfg::BQ)) return rc;
        if (int rc = make_map(&tdo, dout_h, d->batch * d->q_heads, d->seq_q, D, DkvCfg::BQ)) return rc;
        if (int rc = make_map(&tk, d->k, d->batch * d->kv_heads, d->seq_k, D, DkvCfg::BMK)) return rc;
        if (int rc = make_map(&tv, d->v, d->batch * d->kv_heads, d->seq_k, D, DkvCfg::BMK)) return rc;
        TX_CUDA(cudaFuncSetAttribute(txb::sdpa_bwd_dkv_kernel<DkvCfg>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)DkvCfg::SMEM_BYTES));
        // 1-D grid: (slab of (batch, K/V head)) x key tile x column part; a slab's CTAs stream the Q and dO of its
        // query heads
        const int64_t items = (d->seq_k + DkvCfg::BMK - 1) / DkvCfg::BMK, slabs = d->batch * d->kv_heads;
        const int64_t ratio = d->q_heads / d->kv_heads;
        int64_t group = 1;
        if (int rc = launch_group(d->causal != 0, slabs, items * DkvCfg::ZS, 4.0 * (double)ratio * (double)d->seq_q * (double)D, 1, &group, 32))
            return rc;
        p.group_k = (int)group; p.items_k = (int)items; p.slabs_k = (int)slabs;
        if (items * slabs * DkvCfg::ZS > 0x7fffffffLL) return fail(TX_ERR_UNSUPPORTED, "SDPA backward: more than 2^31 work items");
        dim3 grid((unsigned)(items * slabs * DkvCfg::ZS));
        txb::sdpa_bwd_dkv_kernel<DkvCfg><<<grid, DkvCfg::THREADS, DkvCfg::SMEM_BYTES, st>>>(tq, tdo, tk, tv, p);
        g_launches++;
        TX_CUDA(cudaGetLastError());
    }
    return TX_OK;
}

__global__ void cast_f32_to_f16_kernel(const float *__restrict__ in, __half *__restrict__ out, int64_t n);
__global__ void copy_out_kernel(const uint4 *__restrict__ src, uint4 *__restrict__ dst, size_t n16);
size_t align_up(size_t x, size_t a);

// fp32 inputs through the tensor-core kernel: fp16 copies of Q, K, V in stream-ordered pool memory.
int forward_f32_via_f16(const tx_sdpa_desc *d, cudaStream_t st)
{
    const int64_t nq = d->batch * d->q_heads * d->seq_q * d->d_k, nk = d->batch * d->kv_heads * d->seq_k * d->d_k,
                  nv = d->batch * d->kv_heads * d->seq_k * d->d_v;
    const size_t oq = 0, ok = align_up((size_t)nq * 2, 256), ov = ok + align_up((size_t)nk * 2, 256);
    char *ws = nullptr;
    if (int rc = pool_alloc(&ws, ov + (size_t)nv * 2, st)) return rc;
    const void *src[3] = {d->q, d->k, d->v};
    const int64_t n[3] = {nq, nk, nv};
    const size_t off[3] = {oq, ok, ov};
    int rc = TX_OK;
    for (int i = 0; i < 3 && rc == TX_OK; ++i) {
        const int64_t blocks = (n[i] + 1023) / 1024;
        if (blocks > 0x7fffffffLL) { rc = fail(TX_ERR_UNSUPPORTED, "SDPA: tensor too large"); break; }
        cast_f32_to_f16_kernel<<<(unsigned)blocks, 256, 0, st>>>(static_cast<const float *>(src[i]),
                                                               reinterpret_cast<__half *>(ws + off[i]), n[i]);
        g_launches++;
        if (cudaGetLastError() != cudaSuccess) rc = fail(TX_ERR_CUDA, "SDPA: cast launch failed");
    }
    if (rc == TX_OK) {
        tx_sdpa_desc h = *d;
        h.q = ws + oq; h.k = ws + ok; h.v = ws + ov;
        h.dtype = TX_DTYPE_F16;
        int *status = nullptr;
        rc = status_word(&status);
        if (rc == TX_OK) rc = launch_tc(&h, st, status);
    }
    (void)cudaFreeAsync(ws, st);
    return rc;
}

// fp32 in, fp32 out on the fp16 tensor cores (three products per GEMM, sdpa_tc_x3.cuh) for the calls that fit it.
bool x3_eligible(const tx_sdpa_desc *d)
{
    if (d->dtype != TX_DTYPE_F32 || d->mask || d->lse) return false;
    if (d->flags & (TX_SDPA_FORCE_SIMT | TX_SDPA_OUT_F16 | TX_SDPA_P_IN_SMEM)) return false;
    if (d->d_k != d->d_v || (d->d_k != 64 && d->d_k != 128)) return false;
    auto al = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    if (!al(d->q) || !al(d->k) || !al(d->v) || !al(d->out)) return false;
    // the exact kernel stands behind it and must be launchable for the same call
    if (d->batch * d->q_heads > 65535 || (d->seq_q + txb::SIMT_BR - 1) / txb::SIMT_BR > 65535) return false;
    return true;
}

void fill_simt_params(txb::SimtParams *p, const tx_sdpa_desc *d)
{
    p->q = d->q; p->k = d->k; p->v = d->v;
    p->mask = d->mask;
    p->kv_lens = d->kv_lens;
    p->out = d->out;
    p->out_f16 = (d->flags & TX_SDPA_OUT_F16) ? 1 : 0;
    p->B = d->batch; p->Hq = d->q_heads; p->Hkv = d->kv_heads;
    p->Sq = d->seq_q; p->Sk = d->seq_k; p->dk = d->d_k; p->dv = d->d_v;
    p->causal = d->causal ? 1 : 0;
    p->scale = 1.0f / std::sqrt((float)d->d_k);
    p->prof = nullptr;
}

template <class Cfg>
int launch_x3_t(const tx_sdpa_desc *d, cudaStream_t st, int *status)
{
    const int64_t nq = d->batch * d->q_heads * d->seq_q * d->d_k, nk = d->batch * d->kv_heads * d->seq_k * d->d_k;
    // workspace: hi and lo fp16 copies of Q, K, V and the range flag, stream-ordered pool memory
    const size_t bq = align_up((size_t)nq * 2, 256), bk = align_up((size_t)nk * 2, 256);
    const size_t o_qh = 0, o_ql = bq, o_kh = 2 * bq, o_kl = o_kh + bk, o_vh = o_kl + bk, o_vl = o_vh + bk, o_flag = o_vl + bk;
    char *ws = nullptr;
    if (int rc = pool_alloc(&ws, o_flag + 256, st)) return rc;
    int rc = TX_OK;
    auto body = [&]() -> int {
        int *flag = reinterpret_cast<int *>(ws + o_flag);
        TX_CUDA(cudaMemsetAsync(flag, 0, sizeof(int), st));
        txb::SplitParams sp;
        sp.seg[0] = {static_cast<const float *>(d->q), reinterpret_cast<__half *>(ws + o_qh), reinterpret_cast<__half *>(ws + o_ql), nq};
        sp.seg[1] = {static_cast<const float *>(d->k), reinterpret_cast<__half *>(ws + o_kh), reinterpret_cast<__half *>(ws + o_kl), nk};
        sp.seg[2] = {static_cast<const float *>(d->v), reinterpret_cast<__half *>(ws + o_vh), reinterpret_cast<__half *>(ws + o_vl), nk};
        sp.flag = flag;
        int sms = 0;
        if (int r = sm_count(&sms)) return r;
        const int64_t want = (std::max(nq, nk) / 4 + 255) / 256;
        txb::split_f32_hi_lo_kernel<<<(unsigned)std::max<int64_t>(1, std::min<int64_t>(want, 16 * sms)), 256, 0, st>>>(sp);
        g_launches++;
        TX_CUDA(cudaGetLastError());

        CUtensorMap qh, ql, kh, kl, vh, vl, to;
        const int64_t sq = d->batch * d->q_heads, sk = d->batch * d->kv_heads;
        if (int r = make_map(&qh, ws + o_qh, sq, d->seq_q, d->d_k, Cfg::BM)) return r;
        if (int r = make_map(&ql, ws + o_ql, sq, d->seq_q, d->d_k, Cfg::BM)) return r;
        if (int r = make_map(&kh, ws + o_kh, sk, d->seq_k, d->d_k, Cfg::BN)) return r;
        if (int r = make_map(&kl, ws + o_kl, sk, d->seq_k, d->d_k, Cfg::BN)) return r;
        if (int r = make_map(&vh, ws + o_vh, sk, d->seq_k, d->d_v, Cfg::BN)) return r;
        if (int r = make_map(&vl, ws + o_vl, sk, d->seq_k, d->d_v, Cfg::BN)) return r;
        if (int r = make_map(&to, d->out, sq, d->seq_q, d->d_v, 32, 4)) return r;
        txb::X3Params p;
        p.out = static_cast<float *>(d->out);
        p.kv_lens = d->kv_lens;
        p.out_of_range = flag;
        p.status = status;
        p.Hq = (int)d->q_heads; p.Hkv = (int)d->kv_heads; p.Sq = (int)d->seq_q; p.Sk = (int)d->seq_k;
        p.causal = d->causal ? 1 : 0;
        p.scale_log2 = (1.0f / std::sqrt((float)d->d_k)) * 1.4426950408889634f;
        const int64_t n_tiles = (d->seq_q + Cfg::BM - 1) / Cfg::BM;
        int64_t group = 1;
        if (int r = causal_group(d, n_tiles, &group)) return r;
        p.group = (int)group; p.n_tiles_q = (int)n_tiles; p.BH = (int)sq;
        if (n_tiles * sq > 0x7fffffffLL) return fail(TX_ERR_UNSUPPORTED, "SDPA: more than 2^31 work items");
        if (int r = allow_smem(txb::sdpa_tc_x3_kernel<Cfg>, (int)Cfg::SMEM_BYTES)) return r;
        txb::sdpa_tc_x3_kernel<Cfg><<<(unsigned)(n_tiles * sq), Cfg::THREADS, Cfg::SMEM_BYTES, st>>>(qh, ql, kh, kl, vh, vl, to, p);
        g_launches++;
        TX_CUDA(cudaGetLastError());
        // the exact kernel behind it: works only when the split pass found a value the fp16 pairs cannot carry
        txb::SimtParams sp2;
        fill_simt_params(&sp2, d);
        sp2.only_if = flag;
        return launch_simt<float>(sp2, st);
    };
    rc = body();
    (void)cudaFreeAsync(ws, st);
    return rc;
}

int launch_x3(const tx_sdpa_desc *d, cudaStream_t st, int *status)
{
    if (d->d_k == 64) return launch_x3_t<txb::X3Cfg<64, 4>>(d, st, status);
    return launch_x3_t<txb::X3Cfg<128, 2>>(d, st, status);
}

int forward(const tx_sdpa_desc *d)
{
    if (int rc = validate(d)) return rc;
    if (int rc = ensure_device()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(d->stream);
    if (d->dtype == TX_DTYPE_F32 && (d->flags & TX_SDPA_F32_VIA_F16)) {
        tx_sdpa_desc probe = *d;
        probe.dtype = TX_DTYPE_F16;                 // would the fp16 form of this call run on the tensor cores?
        if (tc_eligible(&probe)) return forward_f32_via_f16(d, st);
    }
    if (tc_eligible(d)) {
        int *status = nullptr;
        if (int rc = status_word(&status)) return rc;
        return launch_tc(d, st, status);
    }
    if (x3_eligible(d)) {
        int *status = nullptr;
        if (int rc = status_word(&status)) return rc;
        return launch_x3(d, st, status);
    }
    txb::SimtParams p;
    fill_simt_params(&p, d);
    return d->dtype == TX_DTYPE_F16 ? launch_simt<__half>(p, st) : launch_simt<float>(p, st);
}

int finish(cudaStream_t st)
{
    TX_CUDA(cudaStreamSynchronize(st));
    int dev = 0;
    TX_CUDA(cudaGetDevice(&dev));
    int *w = (dev >= 0 && dev < kMaxDevices) ? g_status[dev] : nullptr;
    if (w) {
        int code = 0;
        TX_CUDA(cudaMemcpy(&code, w, sizeof code, cudaMemcpyDeviceToHost));
        if (code != 0) {
            (void)cudaMemset(w, 0, sizeof code);
            return fail(TX_ERR_KERNEL, "SDPA kernel gave up on a bounded wait (stage code %d); output is not valid", code);
        }
    }
    return TX_OK;
}

int sync_f32(const float *Q, const float *K, const float *V, const float *mask, float *out,
             int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t dk, int64_t dv)
{
    tx_sdpa_desc d;
    std::memset(&d, 0, sizeof d);
    d.q = Q; d.k = K; d.v = V; d.mask = mask; d.out = out;
    d.batch = B; d.q_heads = H; d.kv_heads = H; d.seq_q = Sq; d.seq_k = Sk; d.d_k = dk; d.d_v = dv;
    d.dtype = TX_DTYPE_F32;
    if (int rc = forward(&d)) return rc;
    return finish(nullptr);
}

// The fp32 launchers' section profile: one instrumented launch of the exact-fp32 kernel, 32 clock64
// stamps of thread 0 of CTA (0,0,0) (txb::SimtStamp; unused entries stay 0), as the reference's
// sdpa_*_profile_sections_cuda return them (csrc/cuda/kernels/attn.cu:1113-1140,1617-1722).
int profile_f32(const float *Q, const float *K, const float *V, const float *mask, float *out,
                int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t dk, int64_t dv, long long *ticks32)
{
    if (!ticks32) return fail(TX_ERR_INVALID, "profile_sections: null output");
    tx_sdpa_desc d;
    std::memset(&d, 0, sizeof d);
    d.q = Q; d.k = K; d.v = V; d.mask = mask; d.out = out;
    d.batch = B; d.q_heads = H; d.kv_heads = H; d.seq_q = Sq; d.seq_k = Sk; d.d_k = dk; d.d_v = dv;
    d.dtype = TX_DTYPE_F32;
    if (int rc = validate(&d)) return rc;
    if (int rc = ensure_device()) return rc;
    long long *dev = nullptr;
    TX_CUDA(cudaMalloc(&dev, 32 * sizeof(long long)));
    int rc = cudaMemset(dev, 0, 32 * sizeof(long long)) == cudaSuccess ? TX_OK : fail(TX_ERR_CUDA, "cudaMemset failed");
    if (rc == TX_OK) {
        txb::SimtParams p;
        p.q = Q; p.k = K; p.v = V; p.mask = mask; p.kv_lens = nullptr; p.out = out; p.out_f16 = 0;
        p.B = B; p.Hq = H; p.Hkv = H; p.Sq = Sq; p.Sk = Sk; p.dk = dk; p.dv = dv;
        p.causal = 0;
        p.scale = 1.0f / std::sqrt((float)dk);
        p.prof = dev;
        rc = launch_simt<float, true>(p, nullptr);
    }
    if (rc == TX_OK) rc = finish(nullptr);
    if (rc == TX_OK && cudaMemcpy(ticks32, dev, 32 * sizeof(long long), cudaMemcpyDeviceToHost) != cudaSuccess)
        rc = fail(TX_ERR_CUDA, "cudaMemcpy of the section profile failed");
    (void)cudaFree(dev);
    return rc;
}

__global__ void cast_f32_to_f16_kernel(const float *__restrict__ in, __half *__restrict__ out, int64_t n)
{
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i + 3 < n && ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0) {
        const float4 f = *reinterpret_cast<const float4 *>(in + i);
        __half2 a = __floats2half2_rn(f.x, f.y), b = __floats2half2_rn(f.z, f.w);
        uint2 u;
        u.x = *reinterpret_cast<uint32_t *>(&a);
        u.y = *reinterpret_cast<uint32_t *>(&b);
        *reinterpret_cast<uint2 *>(out + i) = u;
    } else {
        for (int64_t j = i; j < n && j < i + 4; ++j) out[j] = __float2half_rn(in[j]);
    }
}

// Result slab of one chunk of the host form, written by a few CTAs straight into the caller's pinned (device-mapped)
// buffer: 16 bytes per thread, a warp's 512 bytes contiguous.
__global__ void __launch_bounds__(1024) copy_out_kernel(const uint4 *__restrict__ src, uint4 *__restrict__ dst, size_t n16)
{
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) dst[i] = src[i];
}

template <typename T>
__global__ void repeat_interleave_kernel(const T *__restrict__ in, T *__restrict__ out, int64_t total,
                                         int64_t dim_size, int64_t inner, int64_t repeats)
{
    for (int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; o < total;
         o += (int64_t)gridDim.x * blockDim.x) {
        const int64_t k = o % inner;
        const int64_t jr = (o / inner) % (dim_size * repeats);
        const int64_t i = o / (inner * dim_size * repeats);
        out[o] = in[(i * dim_size + jr / repeats) * inner + k];
    }
}

// ------------------------------------------------------------------ host-buffer form
struct Workspace {
    void *ptr = nullptr;
    size_t bytes = 0;
};
Workspace g_ws[kMaxDevices];
std::mutex g_ws_mu;

int workspace(size_t bytes, void **out)
{
    int dev = 0;
    TX_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(TX_ERR_INVALID, "device index %d out of range", dev);
    Workspace &w = g_ws[dev];
    if (w.bytes < bytes) {
        if (w.ptr) TX_CUDA(cudaFree(w.ptr));
        w.ptr = nullptr;
        w.bytes = 0;
        TX_CUDA(cudaMalloc(&w.ptr, bytes));
        w.bytes = bytes;
    }
    *out = w.ptr;
    return TX_OK;
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

std::atomic<int> g_linear_force_simt{0};
bool flags_linear_force_simt() { return g_linear_force_simt.load() != 0; }

// Streams and events of the host-buffer form, created once per device.
constexpr int kHostChunks = 16;
struct HostPipe {
    bool ready = false;
    cudaStream_t in = nullptr, out = nullptr;
    cudaEvent_t start = nullptr, out_done = nullptr, in_done[kHostChunks] = {}, k_done[kHostChunks] = {};
};
HostPipe g_pipe[kMaxDevices];

int host_pipe(HostPipe **out)
{
    int dev = 0;
    TX_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(TX_ERR_INVALID, "device index %d out of range", dev);
    HostPipe &p = g_pipe[dev];
    if (!p.ready) {
        TX_CUDA(cudaStreamCreateWithFlags(&p.in, cudaStreamNonBlocking));
        TX_CUDA(cudaStreamCreateWithFlags(&p.out, cudaStreamNonBlocking));
        TX_CUDA(cudaEventCreateWithFlags(&p.start, cudaEventDisableTiming));
        TX_CUDA(cudaEventCreateWithFlags(&p.out_done, cudaEventDisableTiming));
        for (int i = 0; i < kHostChunks; ++i) {
            TX_CUDA(cudaEventCreateWithFlags(&p.in_done[i], cudaEventDisableTiming));
            TX_CUDA(cudaEventCreateWithFlags(&p.k_done[i], cudaEventDisableTiming));
        }
        p.ready = true;
    }
    *out = &p;
    return TX_OK;
}

// ------------------------------------------------------------------ allocation-free form
// Scratch of tx_sdpa_fp16_static_scratch: [0,256) status word (+ padding), then up to
// TX_STATIC_SCRATCH_MAX_BATCH key lengths.  It is part of the module image on every GPU that
// loads the library.  In host code the name below is only a handle for
// cudaGetSymbolAddress; kernels are given the address that call returns.
static __device__ __align__(256) unsigned char g_static_scratch[TX_STATIC_SCRATCH_BYTES];
unsigned char *g_static_scratch_addr[kMaxDevices] = {};
std::mutex g_static_mu;

// Device address of the array on the current device, looked up once per device.
int static_scratch(unsigned char **out)
{
    int dev = 0;
    TX_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(TX_ERR_INVALID, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (!g_static_scratch_addr[dev]) {
        unsigned char *ptr = nullptr;
        TX_CUDA(cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_static_scratch));
        if (!ptr) return fail(TX_ERR_CUDA, "cudaGetSymbolAddress returned a null address for the static scratch");
        g_static_scratch_addr[dev] = ptr;
    }
    *out = g_static_scratch_addr[dev];
    return TX_OK;
}

// Output tensors are allocated per call by the dispatchers (csrc/tensor_ops.cpp:901-907), and in the
// reference every one of them is a cudaMalloc / cudaFree pair -- device-wide synchronisations that
// dominate short calls (docs/profiling/RESULTS.md:149-152).  Here the pair goes through the device's
// stream-ordered memory pool with a release threshold that keeps freed blocks cached, so a steady
// sequence of calls stops touching the driver's allocator after the first one.
int pool_ready()
{
    int dev = 0;
    TX_CUDA(cudaGetDevice(&dev));
    static bool ready[kMaxDevices] = {};
    if (dev < 0 || dev >= kMaxDevices) return fail(TX_ERR_INVALID, "device index %d out of range", dev);
    if (!ready[dev]) {
        cudaMemPool_t pool;
        TX_CUDA(cudaDeviceGetDefaultMemPool(&pool, dev));
        // Freed blocks stay cached up to this much; beyond it the pool gives memory back to the driver at the
        // next synchronisation, so a process on a shared GPU does not sit on everything it ever touched.
        unsigned long long keep = 4ull << 30;
        TX_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
        ready[dev] = true;
    }
    return TX_OK;
}

}  // namespace

extern "C" {

const char *tx_last_error(void) { return g_err.c_str(); }
int tx_version(void) { return 100; }

int tx_cuda_is_available(void)
{
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return n > 0 ? 1 : 0;
}

int tx_cuda_device_count(void)
{
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return n;
}

int tx_cuda_set_device(int device)
{
    TX_CUDA(cudaSetDevice(device));
    return TX_OK;
}

void *tx_cuda_malloc(size_t bytes)
{
    void *p = nullptr;
    if (pool_ready() != TX_OK) return nullptr;
    cudaError_t e = cudaMallocAsync(&p, bytes ? bytes : 1, (cudaStream_t)0);
    if (e != cudaSuccess) {
        fail(TX_ERR_CUDA, "cudaMallocAsync(%zu) failed: %s", bytes, cudaGetErrorString(e));
        (void)cudaGetLastError();
        return nullptr;
    }
    return p;
}

int tx_cuda_free(void *ptr)
{
    if (!ptr) return TX_OK;
    TX_CUDA(cudaFreeAsync(ptr, (cudaStream_t)0));
    return TX_OK;
}

int tx_cuda_free_on(void *ptr, void *stream)
{
    if (!ptr) return TX_OK;
    TX_CUDA(cudaFreeAsync(ptr, static_cast<cudaStream_t>(stream)));
    return TX_OK;
}

int tx_cuda_pool_trim(void)
{
    int dev = 0;
    TX_CUDA(cudaGetDevice(&dev));
    cudaMemPool_t pool;
    TX_CUDA(cudaDeviceGetDefaultMemPool(&pool, dev));
    TX_CUDA(cudaDeviceSynchronize());
    TX_CUDA(cudaMemPoolTrimTo(pool, 0));
    return TX_OK;
}

int tx_cuda_memcpy_h2d(void *dst, const void *src, size_t bytes)
{
    TX_CUDA(cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice));
    return TX_OK;
}

int tx_cuda_memcpy_d2h(void *dst, const void *src, size_t bytes)
{
    TX_CUDA(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost));
    return TX_OK;
}

int tx_cuda_memcpy_d2d(void *dst, const void *src, size_t bytes)
{
    TX_CUDA(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToDevice));
    return TX_OK;
}

int tx_cuda_synchronize(void)
{
    TX_CUDA(cudaDeviceSynchronize());
    return TX_OK;
}

void *tx_host_alloc_pinned(size_t bytes)
{
    void *p = nullptr;
    cudaError_t e = cudaHostAlloc(&p, bytes ? bytes : 1, cudaHostAllocDefault);
    if (e != cudaSuccess) {
        fail(TX_ERR_CUDA, "cudaHostAlloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
        (void)cudaGetLastError();
        return nullptr;
    }
    return p;
}

int tx_host_free_pinned(void *ptr)
{
    if (!ptr) return TX_OK;
    TX_CUDA(cudaFreeHost(ptr));
    return TX_OK;
}

int tx_sdpa_naive_cuda(const float *Q, const float *K, const float *V, const float *mask, float *out,
                       int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t dk, int64_t dv)
{
    TX_NVTX_RANGE("sdpa.naive");
    return sync_f32(Q, K, V, mask, out, B, H, Sq, Sk, dk, dv);
}
int tx_sdpa_tiled_cuda(const float *Q, const float *K, const float *V, const float *mask, float *out,
                       int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t dk, int64_t dv)
{
    TX_NVTX_RANGE("sdpa.tiled");
    return sync_f32(Q, K, V, mask, out, B, H, Sq, Sk, dk, dv);
}
int tx_sdpa_flash_cuda(const float *Q, const float *K, const float *V, const float *mask, float *out,
                       int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t dk, int64_t dv)
{
    TX_NVTX_RANGE("sdpa.flash");
    return sync_f32(Q, K, V, mask, out, B, H, Sq, Sk, dk, dv);
}
int tx_sdpa_optimized_flash_cuda(const float *Q, const float *K, const float *V, const float *mask,
                                 float *out, int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t dk,
                                 int64_t dv)
{
    TX_NVTX_RANGE("sdpa.flash_optimized");
    return sync_f32(Q, K, V, mask, out, B, H, Sq, Sk, dk, dv);
}
int tx_sdpa_mma_cuda(const float *Q, const float *K, const float *V, const float *mask, float *out,
                     int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t dk, int64_t dv)
{
    TX_NVTX_RANGE("sdpa.mma");
    // The reference computes this variant with fp16 operands; the exact-fp32 kernel
    // is used here, which is strictly closer to the CPU path.
    return sync_f32(Q, K, V, mask, out, B, H, Sq, Sk, dk, dv);
}

int tx_sdpa_mma_fp16_cuda(const void *Q_h, const void *K_h, const void *V_h, float *out, int64_t B,
                          int64_t H, int64_t Sq, int64_t Sk, int64_t dk, int64_t dv)
{
    TX_NVTX_RANGE("sdpa.mma.fp16");
    tx_sdpa_desc d;
    std::memset(&d, 0, sizeof d);
    d.q = Q_h; d.k = K_h; d.v = V_h; d.out = out;
    d.batch = B; d.q_heads = H; d.kv_heads = H; d.seq_q = Sq; d.seq_k = Sk; d.d_k = dk; d.d_v = dv;
    d.dtype = TX_DTYPE_F16;
    if (int rc = forward(&d)) return rc;
    return finish(nullptr);
}

int tx_sdpa_naive_profile_sections_cuda(const float *Q, const float *K, const float *V, const float *mask, float *out,
        int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t dk, int64_t dv, long long *ticks32)
{
    TX_NVTX_RANGE("sdpa.naive.profile");
    return profile_f32(Q, K, V, mask, out, B, H, Sq, Sk, dk, dv, ticks32);
}
int tx_sdpa_tiled_profile_sections_cuda(const float *Q, const float *K, const float *V, const float *mask, float *out,
        int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t dk, int64_t dv, long long *ticks32)
{
    TX_NVTX_RANGE("sdpa.tiled.profile");
    return profile_f32(Q, K, V, mask, out, B, H, Sq, Sk, dk, dv, ticks32);
}
int tx_sdpa_flash_profile_sections_cuda(const float *Q, const float *K, const float *V, const float *mask, float *out,
        int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t dk, int64_t dv, long long *ticks32)
{
    TX_NVTX_RANGE("sdpa.flash.profile");
    return profile_f32(Q, K, V, mask, out, B, H, Sq, Sk, dk, dv, ticks32);
}
int tx_sdpa_optimized_flash_profile_sections_cuda(const float *Q, const float *K, const float *V, const float *mask, float *out,
        int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t dk, int64_t dv, long long *ticks32)
{
    TX_NVTX_RANGE("sdpa.flash_optimized.profile");
    return profile_f32(Q, K, V, mask, out, B, H, Sq, Sk, dk, dv, ticks32);
}
int tx_sdpa_mma_profile_sections_cuda(const float *Q, const float *K, const float *V, const float *mask, float *out,
        int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t dk, int64_t dv, long long *ticks32)
{
    TX_NVTX_RANGE("sdpa.mma.profile");
    return profile_f32(Q, K, V, mask, out, B, H, Sq, Sk, dk, dv, ticks32);
}

int tx_cast_f32_to_f16_cuda(const float *in, void *out, int64_t size)
{
    if (size < 0 || (size > 0 && (!in || !out))) return fail(TX_ERR_INVALID, "cast_to_fp16: bad arguments");
    if (int rc = ensure_device()) return rc;
    if (size == 0) return TX_OK;
    const int threads = 256;
    const int64_t blocks = (size + threads * 4 - 1) / (threads * 4);
    if (blocks > 0x7fffffffLL) return fail(TX_ERR_UNSUPPORTED, "cast_to_fp16: tensor too large");
    cast_f32_to_f16_kernel<<<(unsigned)blocks, threads>>>(in, static_cast<__half *>(out), size);
    g_launches++;
    TX_CUDA(cudaGetLastError());
    return TX_OK;
}

int tx_repeat_interleave_cuda(const void *in, void *out, int64_t outer, int64_t dim_size,
                              int64_t inner, int64_t repeats, int32_t elem_bytes)
{
    if (!in || !out || outer <= 0 || dim_size <= 0 || inner <= 0 || repeats <= 0)
        return fail(TX_ERR_INVALID, "repeat_interleave: bad arguments");
    if (elem_bytes != 2 && elem_bytes != 4) return fail(TX_ERR_INVALID, "repeat_interleave: element size must be 2 or 4");
    if (int rc = ensure_device()) return rc;
    const int64_t total = outer * dim_size * repeats * inner;
    const int threads = 256;
    const unsigned blocks = (unsigned)std::min<int64_t>((total + threads - 1) / threads, 148 * 16);
    if (elem_bytes == 2)
        repeat_interleave_kernel<uint16_t><<<blocks, threads>>>(static_cast<const uint16_t *>(in),
                                                               static_cast<uint16_t *>(out), total, dim_size, inner, repeats);
    else
        repeat_interleave_kernel<uint32_t><<<blocks, threads>>>(static_cast<const uint32_t *>(in),
                                                               static_cast<uint32_t *>(out), total, dim_size, inner, repeats);
    g_launches++;
    TX_CUDA(cudaGetLastError());
    return TX_OK;
}

int tx_sdpa_set_group_l2_bytes(int64_t bytes)
{
    g_group_l2_bytes.store(bytes > 0 ? (long long)bytes : (48ll << 20));
    return TX_OK;
}

int tx_linear_set_cuda_cores_only(int on)
{
    g_linear_force_simt.store(on ? 1 : 0);
    return TX_OK;
}

int tx_linear_f32_cuda(const float *x, const float *w, const float *bias, float *out, int64_t batch,
                       int64_t seq, int64_t in_features, int64_t out_features, int32_t heads_in,
                       int32_t heads_out)
{
    if (!x || !w || !out || batch <= 0 || seq <= 0 || in_features <= 0 || out_features <= 0)
        return fail(TX_ERR_INVALID, "linear: bad arguments");
    if (heads_in < 0 || heads_out < 0 || (heads_in > 0 && in_features % heads_in) ||
        (heads_out > 0 && out_features % heads_out))
        return fail(TX_ERR_INVALID, "linear: feature count must be a multiple of the head count");
    if (int rc = ensure_device()) return rc;
    const int64_t dh_in = heads_in > 0 ? in_features / heads_in : in_features;
    const int64_t dh_out = heads_out > 0 ? out_features / heads_out : out_features;
    auto al = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    const bool tensor_cores = !(flags_linear_force_simt()) && in_features % 32 == 0 && dh_in % 32 == 0 &&
                              out_features % 32 == 0 && dh_out % 32 == 0 && al(x) && al(w) && al(out) &&
                              (!bias || al(bias)) && batch <= 65535 && (seq + 127) / 128 <= 65535;
    if (tensor_cores) {
        int *status = nullptr;
        if (int rc = status_word(&status)) return rc;
        CUtensorMap tx_map, tw_map;
        const int64_t hin = heads_in > 0 ? heads_in : 1;
        cuuint64_t xd[4] = {(cuuint64_t)dh_in, (cuuint64_t)seq, (cuuint64_t)hin, (cuuint64_t)batch};
        cuuint64_t xs[3];
        if (heads_in > 0) {        // [B, H, S, dh]
            xs[0] = (cuuint64_t)dh_in * 4; xs[1] = (cuuint64_t)seq * dh_in * 4; xs[2] = (cuuint64_t)hin * seq * dh_in * 4;
        } else {                   // [B, S, K] seen as one head
            xs[0] = (cuuint64_t)in_features * 4; xs[1] = (cuuint64_t)seq * in_features * 4; xs[2] = (cuuint64_t)seq * in_features * 4;
        }
        if (int rc = make_map_f32(&tx_map, x, 4, xd, xs, txb::LTC_BM)) return rc;
        cuuint64_t wd[3] = {(cuuint64_t)in_features, (cuuint64_t)out_features, 1};
        cuuint64_t ws[2] = {(cuuint64_t)in_features * 4, (cuuint64_t)in_features * out_features * 4};
        if (int rc = make_map_f32(&tw_map, w, 3, wd, ws, txb::LTC_BN)) return rc;
        txb::LinearTcParams lp;
        lp.bias = bias; lp.out = out; lp.status = status;
        lp.S = (int)seq; lp.N = (int)out_features; lp.K = (int)in_features;
        lp.dh_in = (int)dh_in; lp.heads_out = heads_out;
        TX_CUDA(cudaFuncSetAttribute(txb::linear_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)txb::LTC_SMEM));
        dim3 grid((unsigned)((out_features + txb::LTC_BN - 1) / txb::LTC_BN), (unsigned)((seq + txb::LTC_BM - 1) / txb::LTC_BM),
                  (unsigned)batch);
        txb::linear_tc_kernel<<<grid, txb::LTC_THREADS, txb::LTC_SMEM>>>(tx_map, tw_map, lp);
        g_launches++;
        TX_CUDA(cudaGetLastError());
        return TX_OK;
    }
    txb::LinearParams p;
    p.x = x; p.w = w; p.bias = bias; p.out = out;
    p.B = batch; p.S = seq; p.K = in_features; p.N = out_features;
    p.heads_in = heads_in; p.heads_out = heads_out;
    const int64_t gy = (batch * seq + txb::LIN_BM - 1) / txb::LIN_BM, gx = (out_features + txb::LIN_BN - 1) / txb::LIN_BN;
    if (gy > 65535 || gx > 0x7fffffffLL) return fail(TX_ERR_UNSUPPORTED, "linear: too many rows for one launch");
    txb::linear_simt_kernel<<<dim3((unsigned)gx, (unsigned)gy), txb::LIN_THREADS>>>(p);
    g_launches++;
    TX_CUDA(cudaGetLastError());
    return TX_OK;
}

int tx_sdpa_forward(const tx_sdpa_desc *desc)
{
    TX_NVTX_RANGE("sdpa.forward");
    return forward(desc);
}

int tx_profile_sections_sdpa(const tx_sdpa_desc *d, long long *ticks64)
{
    TX_NVTX_RANGE("sdpa.mma.fp16.profile");
    if (!ticks64) return fail(TX_ERR_INVALID, "profile_sections: null output");
    if (int rc = validate(d)) return rc;
    if (!tc_eligible(d))
        return fail(TX_ERR_UNSUPPORTED, "profile_sections: built for the tensor-core kernel only");
    if (d->flags & TX_SDPA_P_IN_SMEM)
        return fail(TX_ERR_UNSUPPORTED, "profile_sections: not built for the P-in-shared-memory variant");
    if (int rc = ensure_device()) return rc;
    int *status = nullptr;
    if (int rc = status_word(&status)) return rc;
    long long *dev = nullptr;
    TX_CUDA(cudaMalloc(&dev, 64 * sizeof(long long)));
    cudaStream_t st = static_cast<cudaStream_t>(d->stream);
    int rc = TX_OK;
    if (cudaMemsetAsync(dev, 0, 64 * sizeof(long long), st) != cudaSuccess) rc = fail(TX_ERR_CUDA, "cudaMemsetAsync failed");
    if (rc == TX_OK) rc = launch_tc(d, st, status, dev);
    if (rc == TX_OK) rc = finish(st);
    if (rc == TX_OK && cudaMemcpy(ticks64, dev, 64 * sizeof(long long), cudaMemcpyDeviceToHost) != cudaSuccess)
        rc = fail(TX_ERR_CUDA, "cudaMemcpy of the section profile failed");
    (void)cudaFree(dev);
    return rc;
}

int tx_selftest_wait_timeout(const tx_sdpa_desc *d, int32_t skip_k_tile)
{
    if (int rc = validate(d)) return rc;
    if (!tc_eligible(d) || d->d_k != 64 || (d->flags & TX_SDPA_P_IN_SMEM))
        return fail(TX_ERR_UNSUPPORTED, "wait-timeout self-test: built for the fp16 d = 64 tensor-core kernel");
    if (int rc = ensure_device()) return rc;
    int *status = nullptr;
    if (int rc = status_word(&status)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(d->stream);
    if (int rc = launch_pair_t<txb::PairCfg<64, 128, 4, kPolyPairsD64, false, false, true>>(d, st, status, nullptr, skip_k_tile))
        return rc;
    return finish(st);
}

int tx_sdpa_backward(const tx_sdpa_bwd_desc *d)
{
    if (!d) return fail(TX_ERR_INVALID, "SDPA backward: null descriptor");
    if (!d->q || !d->k || !d->v || !d->out || !d->dout || !d->lse || !d->dq || !d->dk || !d->dv)
        return fail(TX_ERR_INVALID, "SDPA backward: q, k, v, out, dout, lse, dq, dk, dv must not be null");
    if (d->batch <= 0 || d->q_heads <= 0 || d->kv_heads <= 0 || d->seq_q <= 0 || d->seq_k <= 0)
        return fail(TX_ERR_INVALID, "SDPA backward: every dimension must be positive");
    if (d->q_heads % d->kv_heads != 0)
        return fail(TX_ERR_INVALID, "SDPA backward: q_heads %lld not a multiple of kv_heads %lld",
                    (long long)d->q_heads, (long long)d->kv_heads);
    if (d->d != 64 && d->d != 128 && d->d != 256)
        return fail(TX_ERR_UNSUPPORTED, "SDPA backward: built for d in {64, 128, 256}, got %lld", (long long)d->d);
    if (d->batch * d->q_heads > 65535 || d->seq_q > 0x3fffffffLL || d->seq_k > 0x3fffffffLL)
        return fail(TX_ERR_UNSUPPORTED, "SDPA backward: dimension too large");
    auto al = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    if (!al(d->q) || !al(d->k) || !al(d->v) || !al(d->out) || !al(d->dout) || !al(d->dq) || !al(d->dk) || !al(d->dv))
        return fail(TX_ERR_INVALID, "SDPA backward: pointers must be 16-byte aligned");
    if (int rc = ensure_device()) return rc;
    int *status = nullptr;
    if (int rc = status_word(&status)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(d->stream);
    const int64_t rows = d->batch * d->q_heads * d->seq_q;
    const size_t h_bytes = align_up((size_t)rows * (size_t)d->d * 2, 256);
    char *ws = nullptr;
    if (int rc = pool_alloc(&ws, h_bytes + (size_t)rows * 4, st)) return rc;
    __half *dout_h = reinterpret_cast<__half *>(ws);
    float *delta = reinterpret_cast<float *>(ws + h_bytes);
    const int warps = 8;
    const unsigned blocks = (unsigned)((rows + warps - 1) / warps);
    if (d->flags & TX_SDPA_OUT_F16)
        txb::sdpa_bwd_prep_kernel<__half><<<blocks, warps * 32, 0, st>>>(d->dout, static_cast<const __half *>(d->out),
                                                                       dout_h, delta, rows, (int)d->d);
    else
        txb::sdpa_bwd_prep_kernel<float><<<blocks, warps * 32, 0, st>>>(d->dout, static_cast<const float *>(d->out),
                                                                      dout_h, delta, rows, (int)d->d);
    g_launches++;
    int rc = (cudaGetLastError() == cudaSuccess) ? TX_OK : fail(TX_ERR_CUDA, "SDPA backward: preprocess launch failed");
    if (rc == TX_OK) {
        // d = 64: two CTAs per SM for both kernels (64-key / 64-query tiles; dK/dV stages P^T and dS^T in shared
        // memory to stay inside 256 tensor-memory columns: 3.23 ms against 3.51 ms with 128-query tiles, one CTA
        // per SM and two row warpgroups, config-2 size).
        // d = 128: one CTA per SM for both, two row warpgroups, 128-key / 64-query tiles (all of tensor memory).
        if (d->d == 64)
            rc = launch_bwd<64, txb::BwdDqCfg<64, 64, 3, 1, 2>, txb::BwdDkvCfg<64, 64, 3, 1, true, 2>>(d, st, status, dout_h, delta);
        else if (d->d == 128)
            rc = launch_bwd<128, txb::BwdDqCfg<128, 128, 3, 2, 2>, txb::BwdDkvCfg<128, 64, 3, 2, false, 3>>(d, st, status, dout_h, delta);
        else
            // d = 256: dQ alone takes 256 tensor-memory columns (64-key tiles, single V stage: 224 KB of shared
            // memory); two CTAs per key tile each own 128 columns of dK and dV, with 32-query tiles so that two
            // stages each of Q and dO fit beside the resident K and V (a stage stays occupied from its first
            // read to its second, so one stage per ring would deadlock the MMA warp).
            rc = launch_bwd<256, txb::BwdDqCfg<256, 64, 2, 1, 1>, txb::BwdDkvCfg<256, 32, 2, 1, false, 2, 2>>(d, st, status, dout_h, delta);
    }
    (void)cudaFreeAsync(ws, st);        // ordered after the kernels on `st`
    return rc;
}

int tx_sdpa_finish(void *stream) { return finish(static_cast<cudaStream_t>(stream)); }

int tx_sdpa_uses_tensor_cores(const tx_sdpa_desc *desc)
{
    if (validate(desc) != TX_OK) return 0;
    if (desc->dtype == TX_DTYPE_F32 && (desc->flags & TX_SDPA_F32_VIA_F16)) {
        tx_sdpa_desc probe = *desc;
        probe.dtype = TX_DTYPE_F16;
        return tc_eligible(&probe) ? 1 : 0;
    }
    return (tc_eligible(desc) || x3_eligible(desc)) ? 1 : 0;
}

int64_t tx_kernel_launch_count(void) { return g_launches.load(); }

// Host-buffer form.  `with_kernel == false` runs the same copy schedule with the kernels left out: what the
// host <-> device path alone takes (the benchmark reports it beside the full call).
static int forward_host(const tx_sdpa_desc *h, bool with_kernel)
{
    if (int rc = validate(h)) return rc;
    if (h->mask) return fail(TX_ERR_UNSUPPORTED, "SDPA host form: dense masks are not taken; use causal / kv_lens");
    if (h->lse) return fail(TX_ERR_UNSUPPORTED, "SDPA host form: no log-sum-exp output");
    if (int rc = ensure_device()) return rc;
    // The call is cut into chunks of whole (batch, K/V head) units -- contiguous slabs of Q, K, V and
    // O -- so that the upload of chunk i+1, the kernel of chunk i and the download of chunk i-1 run
    // at the same time on three streams (PCIe is full duplex; with pinned host buffers the copies
    // are asynchronous).  Chunks are about an eighth of the call: smaller ones start the first kernel and
    // the first download earlier but pay the fixed cost of a copy (some microseconds) more often.
    const int64_t units = h->batch * h->kv_heads, group = h->q_heads / h->kv_heads;
    const size_t es = h->dtype == TX_DTYPE_F16 ? 2 : 4;
    const size_t uq = (size_t)(group * h->seq_q * h->d_k) * es;       // bytes of one unit
    const size_t uk = (size_t)(h->seq_k * h->d_k) * es;
    const size_t uv = (size_t)(h->seq_k * h->d_v) * es;
    const size_t uo = (size_t)(group * h->seq_q * h->d_v) * ((h->flags & TX_SDPA_OUT_F16) ? 2 : 4);
    const size_t nl = h->kv_lens ? (size_t)units * 4 : 0;
    const size_t oq = 0, ok = align_up(oq + uq * units, 256), ov = align_up(ok + uk * units, 256),
                 oo = align_up(ov + uv * units, 256), ol = align_up(oo + uo * units, 256);
    const size_t total = align_up(ol + nl, 256);
    std::lock_guard<std::mutex> lk(g_ws_mu);
    void *base = nullptr;
    if (int rc = workspace(total, &base)) return rc;
    char *w = static_cast<char *>(base);
    HostPipe *hp = nullptr;
    if (int rc = host_pipe(&hp)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(h->stream);

    // chunk boundaries in units
    int64_t bounds[kHostChunks + 1];
    int n_chunks = 0;
    bounds[0] = 0;
    const size_t bytes_total = (uq + uk + uv + uo) * (size_t)units;
    if (bytes_total < (8u << 20) || units < 2) {                       // too small to be worth cutting
        bounds[1] = units;
        n_chunks = 1;
    } else {
        // A small first chunk (the first kernel and the first download start early), large middle chunks (every
        // copy costs about 10 us of set-up and small opposite copies disturb each other), a small last chunk (its
        // kernel and its download are the tail nothing overlaps).  Measured on B200 + PCIe 5 with the copies alone
        // (96 MiB in, 64 MiB out; units 4 8 8 6 4 2 of 32): 2.35 ms; eight eighths 2.49, 4 6 4 4 4 4 4 2 2.44,
        // quarters 2.39, sixteenths 2.81, one chunk 3.00; two big opposite copies 1.93, the upload alone 1.82.
        static const double cum[] = {0.125, 0.375, 0.625, 0.8125, 0.9375, 1.0};
        int64_t u = 0;
        for (double f : cum) {
            const int64_t to = std::min<int64_t>(units, std::max<int64_t>(u + 1, (int64_t)std::llround(f * (double)units)));
            if (to > u) { u = to; bounds[++n_chunks] = u; }
            if (u >= units) break;
        }
        if (u < units) bounds[n_chunks] = units;
    }
    // The result goes back either by the copy engine or, when the caller's buffer is pinned memory the device can
    // address (what tx_host_alloc_pinned returns), by a small kernel that writes it there: next to the uploads the
    // copy engine's many small downloads disturbed them more (copies alone, 96 MiB in and 64 MiB out in eight chunks:
    // 2.19 ms with the kernel, 2.44 ms with download copies; two big opposite copies 1.93 ms).
    uint4 *out_mapped = nullptr;
    {
        cudaPointerAttributes at;
        if (cudaPointerGetAttributes(&at, h->out) == cudaSuccess && at.type == cudaMemoryTypeHost && at.devicePointer &&
            (reinterpret_cast<uintptr_t>(at.devicePointer) & 15u) == 0 && (uo & 15u) == 0)
            out_mapped = static_cast<uint4 *>(at.devicePointer);
        else
            (void)cudaGetLastError();
    }
    // everything below is ordered after what the caller already put on its stream
    TX_CUDA(cudaEventRecord(hp->start, st));
    TX_CUDA(cudaStreamWaitEvent(hp->in, hp->start, 0));
    TX_CUDA(cudaStreamWaitEvent(hp->out, hp->start, 0));
    std::vector<int32_t> unit_lens;
    if (nl) {
        unit_lens.resize((size_t)units);
        for (int64_t u = 0; u < units; ++u) unit_lens[(size_t)u] = h->kv_lens[u / h->kv_heads];
        TX_CUDA(cudaMemcpyAsync(w + ol, unit_lens.data(), nl, cudaMemcpyHostToDevice, hp->in));
    }
    for (int c = 0; c < n_chunks; ++c) {
        const int64_t u0 = bounds[c], u1 = bounds[c + 1], nu = u1 - u0;
        if (nu <= 0) continue;
        TX_CUDA(cudaMemcpyAsync(w + oq + uq * u0, static_cast<const char *>(h->q) + uq * u0, uq * nu, cudaMemcpyHostToDevice, hp->in));
        TX_CUDA(cudaMemcpyAsync(w + ok + uk * u0, static_cast<const char *>(h->k) + uk * u0, uk * nu, cudaMemcpyHostToDevice, hp->in));
        TX_CUDA(cudaMemcpyAsync(w + ov + uv * u0, static_cast<const char *>(h->v) + uv * u0, uv * nu, cudaMemcpyHostToDevice, hp->in));
        TX_CUDA(cudaEventRecord(hp->in_done[c], hp->in));
        TX_CUDA(cudaStreamWaitEvent(st, hp->in_done[c], 0));
        if (with_kernel) {
            tx_sdpa_desc d = *h;                   // the chunk as a problem of its own: one K/V head per "batch"
            d.q = w + oq + uq * u0; d.k = w + ok + uk * u0; d.v = w + ov + uv * u0;
            d.out = w + oo + uo * u0;
            d.kv_lens = nl ? reinterpret_cast<const int32_t *>(w + ol) + u0 : nullptr;
            d.batch = nu; d.q_heads = group; d.kv_heads = 1;
            if (int rc = forward(&d)) return rc;
        }
        TX_CUDA(cudaEventRecord(hp->k_done[c], st));
        TX_CUDA(cudaStreamWaitEvent(hp->out, hp->k_done[c], 0));
        if (out_mapped) {
            copy_out_kernel<<<8, 1024, 0, hp->out>>>(reinterpret_cast<const uint4 *>(w + oo + uo * u0),
                                                     out_mapped + (uo * u0) / 16, (uo * (size_t)nu) / 16);
            g_launches++;
            TX_CUDA(cudaGetLastError());
        } else {
            TX_CUDA(cudaMemcpyAsync(reinterpret_cast<char *>(h->out) + uo * u0, w + oo + uo * u0, uo * nu, cudaMemcpyDeviceToHost, hp->out));
        }
    }
    TX_CUDA(cudaEventRecord(hp->out_done, hp->out));
    TX_CUDA(cudaStreamWaitEvent(st, hp->out_done, 0));      // the caller's stream ends after the last download
    return finish(st);
}

int tx_sdpa_forward_host(const tx_sdpa_desc *h)
{
    TX_NVTX_RANGE("sdpa.forward_host");
    return forward_host(h, true);
}

int tx_sdpa_forward_host_copies_only(const tx_sdpa_desc *h) { return forward_host(h, false); }

int tx_sdpa_fp16_static_scratch(const void *Q_h, const void *K_h, const void *V_h, float *out,
                                int64_t batch, int64_t q_heads, int64_t kv_heads, int64_t seq_q,
                                int64_t seq_k, int64_t d, int32_t causal, const int32_t *kv_lens_host,
                                void *stream)
{
    tx_sdpa_desc desc;
    std::memset(&desc, 0, sizeof desc);
    desc.q = Q_h; desc.k = K_h; desc.v = V_h; desc.out = out;
    desc.batch = batch; desc.q_heads = q_heads; desc.kv_heads = kv_heads;
    desc.seq_q = seq_q; desc.seq_k = seq_k; desc.d_k = d; desc.d_v = d;
    desc.dtype = TX_DTYPE_F16;
    desc.causal = causal;
    desc.stream = stream;
    if (int rc = validate(&desc)) return rc;
    if (kv_lens_host && batch > TX_STATIC_SCRATCH_MAX_BATCH)
        return fail(TX_ERR_INVALID, "static-scratch SDPA: batch %lld exceeds the %d key lengths the fixed scratch holds",
                    (long long)batch, TX_STATIC_SCRATCH_MAX_BATCH);
    if (!tc_eligible(&desc))
        return fail(TX_ERR_UNSUPPORTED,
                    "static-scratch SDPA: only the tensor-core shapes are taken (fp16, d_k == d_v in {64,128,256,512}, "
                    "16-byte aligned pointers, batch*heads <= 65535)");
    if (int rc = ensure_device()) return rc;
    unsigned char *scratch = nullptr;
    if (int rc = static_scratch(&scratch)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int *status = reinterpret_cast<int *>(scratch);
    TX_CUDA(cudaMemsetAsync(status, 0, 256, st));            // the array keeps the last call's contents
    if (kv_lens_host) {
        TX_CUDA(cudaMemcpyAsync(scratch + 256, kv_lens_host, (size_t)batch * 4, cudaMemcpyHostToDevice, st));
        desc.kv_lens = reinterpret_cast<const int32_t *>(scratch + 256);
    }
    if (int rc = launch_tc(&desc, st, status)) return rc;
    int code = 0;
    TX_CUDA(cudaMemcpyAsync(&code, status, sizeof code, cudaMemcpyDeviceToHost, st));
    TX_CUDA(cudaStreamSynchronize(st));
    if (code != 0)
        return fail(TX_ERR_KERNEL, "SDPA kernel gave up on a bounded wait (stage code %d); output is not valid", code);
    return TX_OK;
}

}  // extern "C"
