/*
 * tensorax_b200 -- C ABI of the B200 (sm_100a) scaled-dot-product-attention forward path.
 *
 * The library is a drop-in for the raw-pointer launcher layer that tensorax's
 * pybind11 dispatchers call (tensorax csrc/tensor_ops.h:170-194 and :234-237).
 * Each entry point below names the reference declaration it replaces.  Argument
 * order and meaning are the reference's; the differences are
 *   - names carry a `tx_` prefix and have C linkage,
 *   - every function returns 0 on success or a TX_ERR_* code instead of printing
 *     and calling exit() (csrc/cuda/cuda_utils.cuh:6-14); tx_last_error() gives the
 *     message of the calling thread's last failure,
 *   - pointers are device pointers unless the name ends in `_host`.
 * Tensors are contiguous row-major [batch, heads, seq, dim].  There is no CPU
 * fallback: without a CUDA device every compute entry point fails with
 * TX_ERR_NO_DEVICE.
 */
#ifndef TENSORAX_B200_H
#define TENSORAX_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define TX_API __attribute__((visibility("default")))
#else
#define TX_API
#endif

enum {
    TX_OK = 0,
    TX_ERR_INVALID = 1,    /* bad shape / pointer / dtype combination (reference: std::runtime_error) */
    TX_ERR_NO_DEVICE = 2,  /* no usable CUDA device */
    TX_ERR_CUDA = 3,       /* a CUDA runtime or driver call failed */
    TX_ERR_KERNEL = 4,     /* a kernel gave up on a bounded wait (2 s) and reported it; tx_last_error() names the
                              stage: 1 misaligned shared memory, 2/3/4 forward producer / MMA / softmax warp,
                              12/13/14 linear-kernel producer / MMA / split warps, 22/23/24 backward
                              producer / MMA / row warps */
    TX_ERR_UNSUPPORTED = 5
};

enum { TX_DTYPE_F32 = 0, TX_DTYPE_F16 = 1 };

/* flags of tx_sdpa_desc */
enum {
    TX_SDPA_FORCE_SIMT = 1,  /* use the exact CUDA-core kernel even where a tensor-core kernel applies (fp16 or fp32) */
    TX_SDPA_OUT_F16 = 4,     /* `out` is fp16 [batch, q_heads, seq_q, d_v] instead of fp32 (the reference only has fp32
                                output, csrc/tensor_ops.cpp:1062; halves the result's bytes) */
    TX_SDPA_F32_VIA_F16 = 8, /* fp32 q/k/v: round them to fp16 on the device (pool temporaries, stream-ordered) and run the
                                tensor-core kernel where its shapes apply -- what the reference's `_mma` variant does inside
                                its kernel (fp32 in/out, fp16 MMA operands, csrc/cuda/kernels/attn.cu:441-603); fp16
                                tolerances then apply.  Without the flag fp32 inputs always get exact fp32 arithmetic. */
    TX_SDPA_P_IN_SMEM = 2    /* tensor-core kernel: stage P in shared memory instead of tensor memory
                                (ignored for d = 512, where shared memory has no room for it) */
};

/* Message of the last failure on the calling thread ("" if none). */
TX_API const char *tx_last_error(void);
TX_API int tx_version(void);

/* ---- device memory helpers: reference csrc/cuda/tensor_cuda.cu:7-29
 *      (cuda_is_available, cuda_malloc, cuda_free, cuda_memcpy_h2d, cuda_memcpy_d2h) */
TX_API int tx_cuda_is_available(void);
/* one process drives one GPU: select it before anything else (no reference counterpart;
 * the reference never leaves device 0) */
TX_API int tx_cuda_device_count(void);
TX_API int tx_cuda_set_device(int device);
/* allocations come from the device's stream-ordered pool on the default stream; freed blocks stay
 * cached in the pool (the reference pays a cudaMalloc/cudaFree pair per output tensor) */
TX_API void *tx_cuda_malloc(size_t bytes);            /* NULL on failure */
TX_API int tx_cuda_free(void *ptr);
/* tx_cuda_malloc / tx_cuda_free are ordered on the legacy default stream: safe with work on stream NULL and on
 * ordinary (blocking) streams, which synchronise with it.  A buffer last used by a kernel on a cudaStreamNonBlocking
 * stream must be freed with tx_cuda_free_on(ptr, that_stream) (or after synchronising that stream): the block then
 * returns to the pool in that stream's order.  No reference counterpart (its cuda_free is a synchronous cudaFree). */
TX_API int tx_cuda_free_on(void *ptr, void *stream);
TX_API int tx_cuda_pool_trim(void);                   /* give cached blocks back to the driver */
TX_API int tx_cuda_memcpy_h2d(void *dst, const void *src, size_t bytes);
TX_API int tx_cuda_memcpy_d2h(void *dst, const void *src, size_t bytes);
TX_API int tx_cuda_memcpy_d2d(void *dst, const void *src, size_t bytes);
TX_API int tx_cuda_synchronize(void);
/* pinned host memory for callers that stream inputs (no reference counterpart) */
TX_API void *tx_host_alloc_pinned(size_t bytes);
TX_API int tx_host_free_pinned(void *ptr);

/* ---- fp32 SDPA launchers: reference csrc/tensor_ops.h:170-188 and :192-194
 *      (sdpa_naive_cuda, sdpa_tiled_cuda, sdpa_flash_cuda, sdpa_mma_cuda,
 *       sdpa_optimized_flash_cuda; kernels csrc/cuda/kernels/attn.cu:135-1111,1564-1615).
 *      Q [B,H,Sq,d_k], K [B,H,Sk,d_k], V [B,H,Sk,d_v], optional dense additive
 *      mask [B,H,Sq,Sk] (NULL = none), out [B,H,Sq,d_v], all fp32 on the device.
 *      Like the reference they return after the result is complete.
 *      Two kernels stand behind the five names.  Calls without a dense mask and with d_k = d_v in {64, 128} run on
 *      the tensor cores: every fp32 operand is carried as two fp16 numbers (hi + lo, 22 significand bits), every
 *      product is three tcgen05 MMAs, tiles are summed in fp32 registers, the softmax is fp32 (within 2e-6 of the
 *      reference's sdpa_cpu on unit-variance inputs, the figure of the exact kernel; 3e-5 at scores of +-100, where
 *      the exact kernel itself is at 1e-5).  A device-side range check sends a call with |x| >= 2^15 or a
 *      non-finite input to the exact CUDA-core kernel, which also takes every other shape and every dense mask. */
TX_API int tx_sdpa_naive_cuda(const float *Q, const float *K, const float *V, const float *mask,
                              float *out, int64_t batch_size, int64_t num_heads,
                              int64_t seq_len_q, int64_t seq_len_k, int64_t d_k, int64_t d_v);
TX_API int tx_sdpa_tiled_cuda(const float *Q, const float *K, const float *V, const float *mask,
                              float *out, int64_t batch_size, int64_t num_heads,
                              int64_t seq_len_q, int64_t seq_len_k, int64_t d_k, int64_t d_v);
TX_API int tx_sdpa_flash_cuda(const float *Q, const float *K, const float *V, const float *mask,
                              float *out, int64_t batch_size, int64_t num_heads,
                              int64_t seq_len_q, int64_t seq_len_k, int64_t d_k, int64_t d_v);
TX_API int tx_sdpa_optimized_flash_cuda(const float *Q, const float *K, const float *V,
                                        const float *mask, float *out, int64_t batch_size,
                                        int64_t num_heads, int64_t seq_len_q, int64_t seq_len_k,
                                        int64_t d_k, int64_t d_v);
TX_API int tx_sdpa_mma_cuda(const float *Q, const float *K, const float *V, const float *mask,
                            float *out, int64_t batch_size, int64_t num_heads,
                            int64_t seq_len_q, int64_t seq_len_k, int64_t d_k, int64_t d_v);

/* ---- fp16 tensor-core SDPA: reference csrc/tensor_ops.h:186-188 (sdpa_mma_fp16_cuda;
 *      kernel csrc/cuda/kernels/attn.cu:1143-1521).  fp16 Q/K/V, fp32 out, no mask. */
TX_API int tx_sdpa_mma_fp16_cuda(const void *Q_h, const void *K_h, const void *V_h, float *out,
                                 int64_t batch_size, int64_t num_heads, int64_t seq_len_q,
                                 int64_t seq_len_k, int64_t d_k, int64_t d_v);

/* ---- fp32 -> fp16 cast: reference csrc/tensor_ops.h:190 (cast_f32_to_f16_cuda;
 *      csrc/cuda/kernels/attn.cu:1523-1562).  Round-to-nearest-even; like the
 *      reference it does not synchronise (stream order is enough). */
TX_API int tx_cast_f32_to_f16_cuda(const float *in, void *out, int64_t size);

/* ---- K/V head replication: reference csrc/tensor_ops.cpp:121-162 (repeat_interleave),
 *      which round-trips through host memory.  Here it is one device gather:
 *      out[i, j*repeats + r, k] = in[i, j, k] for i < outer, j < dim_size, k < inner.
 *      elem_bytes is 2 or 4.  Does not synchronise. */
TX_API int tx_repeat_interleave_cuda(const void *in, void *out, int64_t outer, int64_t dim_size,
                                     int64_t inner, int64_t repeats, int32_t elem_bytes);

/* ---- linear layer either side of SDPA in MultiHeadAttention.forward: reference F.linear
 *      (tensorax/functional.py:105-110) = matmul (csrc/tensor_ops.cpp:295-329, matmul_cpu
 *      csrc/cpu/tensor_cpu.cpp:131-156) + bias, then reshape/transpose to heads
 *      (tensorax/nn/attention/layers.py:112-128).  out = x @ W^T + bias in exact fp32;
 *      x is [batch, seq, in_features], or [batch, heads_in, seq, in_features/heads_in] when
 *      heads_in > 0; out is [batch, seq, out_features], or head-split
 *      [batch, heads_out, seq, out_features/heads_out] when heads_out > 0; W is [out_features,
 *      in_features]; bias may be NULL.  Does not synchronise (tx_sdpa_finish / tx_cuda_synchronize
 *      also report a kernel-side failure of this launch).  Shapes whose feature counts (per head,
 *      where split) are multiples of 32 run on the tensor cores as split-TF32 (three TF32 MMAs per
 *      product keep fp32-grade accuracy); everything else runs on CUDA cores in exact fp32.
 *      tx_linear_set_cuda_cores_only(1) forces the latter (testing). */
TX_API int tx_linear_f32_cuda(const float *x, const float *w, const float *bias, float *out,
                              int64_t batch, int64_t seq, int64_t in_features, int64_t out_features,
                              int32_t heads_in, int32_t heads_out);
TX_API int tx_linear_set_cuda_cores_only(int on);

/* ---- general form (no reference counterpart: the reference has no fp16+mask,
 *      no implicit causal / key-length mask and no grouped K/V heads; its dense
 *      mask forms cannot exist at S = 8192).  Asynchronous on `stream`. */
typedef struct tx_sdpa_desc {
    const void *q;            /* [batch, q_heads,  seq_q, d_k]  dtype */
    const void *k;            /* [batch, kv_heads, seq_k, d_k]  dtype */
    const void *v;            /* [batch, kv_heads, seq_k, d_v]  dtype */
    const float *mask;        /* optional dense additive fp32 [batch, q_heads, seq_q, seq_k] */
    const int32_t *kv_lens;   /* optional [batch] on the device: keys j >= kv_lens[b] are masked */
    void *out;                /* [batch, q_heads, seq_q, d_v] fp32 (fp16 with TX_SDPA_OUT_F16) */
    int64_t batch, q_heads, kv_heads, seq_q, seq_k, d_k, d_v;
    int32_t dtype;            /* TX_DTYPE_* of q, k, v */
    int32_t causal;           /* nonzero: key j visible to query i iff j <= i */
    int32_t flags;            /* TX_SDPA_* */
    int32_t reserved;
    void *stream;             /* cudaStream_t; NULL = default stream */
    float *lse;               /* optional [batch, q_heads, seq_q] fp32: log2 of sum_j 2^(score_ij * log2(e)/sqrt(d_k)),
                                 what tx_sdpa_backward needs; tensor-core shapes only, else must be NULL */
} tx_sdpa_desc;

/* Enqueue one forward pass.  Query head h reads K/V head h / (q_heads/kv_heads). */
TX_API int tx_sdpa_forward(const tx_sdpa_desc *desc);
/* Wait for `stream` and report a kernel-side failure (bounded wait ran out), if any.  This is THE completion
 * check of the asynchronous entry points (tx_sdpa_forward, tx_sdpa_backward, tx_linear_f32_cuda): a caller that
 * synchronises some other way does not learn that a kernel gave up (its rows then read NaN).  The status word is one
 * per device and stays set until a tx_sdpa_finish call on that device reports and clears it; launches issued in
 * between return at once and write NaN. */
TX_API int tx_sdpa_finish(void *stream);
/* 1 if tx_sdpa_forward would run `desc` on a tcgen05 kernel (fp16, or fp32 as hi/lo fp16 pairs), 0 if on CUDA cores.
 * (For fp32 the answer is about the shape: a value outside the pairs' range still sends the call to CUDA cores.) */
TX_API int tx_sdpa_uses_tensor_cores(const tx_sdpa_desc *desc);
/* How many kernels of this library have been launched by this process so far. */
TX_API int64_t tx_kernel_launch_count(void);
/* Launch order of causal calls (forward and backward): the (batch, head) slabs are walked in equal groups and inside
 * a group every slab's longest work items come first; a group holds as many slabs as stream `bytes` of K/V (or, in
 * the dK/dV kernel, Q and dO) through L2 together, at least two waves of CTAs.  Default 48 MiB (bytes <= 0 restores
 * it).  The order changes when a CTA runs, never what it computes: results are bitwise the same for every value. */
TX_API int tx_sdpa_set_group_l2_bytes(int64_t bytes);

/* ---- section profiles of the fp32 launchers: reference csrc/tensor_ops.h:214-233
 *      (sdpa_{naive,tiled,flash,mma,optimized_flash}_profile_sections_cuda, bound to Python as
 *      profile_sections_sdpa_{naive,tiled,flash,mma,flash_optimized}, csrc/tensor_ops.cpp:1434-1507,1622-1636).
 *      Same pointers and sizes as the launcher of the same name; `ticks32` receives 32 clock64 stamps of
 *      thread 0 of CTA (0,0,0) of one instrumented launch (consecutive differences = section times, as with
 *      TX_TICK, csrc/cuda/profiling.cuh:20-51): [0] kernel entry, [1] first Q/K chunk staged, and for the
 *      first key tile [2] QK^T accumulated, [3] scores scaled/masked/parked, [4] online softmax done,
 *      [5] O updated; [6] all key tiles done, [7] output written; the rest stay 0.  All five names profile the
 *      one exact-fp32 CUDA-core kernel, so they report the same sections -- also for a shape the launcher of
 *      the same name would send to the fp32 tensor-core kernel (whose stages are those of the fp16 kernels:
 *      tx_profile_sections_sdpa on an fp16 copy of the call shows them).  Each call is also an NVTX range
 *      ("sdpa.naive.profile", ...; the launchers themselves are "sdpa.naive", ..., "sdpa.mma.fp16"), as in
 *      the reference (csrc/cuda/profiling.cuh:7-18, csrc/cuda/kernels/attn.cu:973-1701). */
TX_API int tx_sdpa_naive_profile_sections_cuda(const float *Q, const float *K, const float *V, const float *mask,
                                               float *out, int64_t batch_size, int64_t num_heads, int64_t seq_len_q,
                                               int64_t seq_len_k, int64_t d_k, int64_t d_v, long long *ticks32);
TX_API int tx_sdpa_tiled_profile_sections_cuda(const float *Q, const float *K, const float *V, const float *mask,
                                               float *out, int64_t batch_size, int64_t num_heads, int64_t seq_len_q,
                                               int64_t seq_len_k, int64_t d_k, int64_t d_v, long long *ticks32);
TX_API int tx_sdpa_flash_profile_sections_cuda(const float *Q, const float *K, const float *V, const float *mask,
                                               float *out, int64_t batch_size, int64_t num_heads, int64_t seq_len_q,
                                               int64_t seq_len_k, int64_t d_k, int64_t d_v, long long *ticks32);
TX_API int tx_sdpa_mma_profile_sections_cuda(const float *Q, const float *K, const float *V, const float *mask,
                                             float *out, int64_t batch_size, int64_t num_heads, int64_t seq_len_q,
                                             int64_t seq_len_k, int64_t d_k, int64_t d_v, long long *ticks32);
TX_API int tx_sdpa_optimized_flash_profile_sections_cuda(const float *Q, const float *K, const float *V,
                                                         const float *mask, float *out, int64_t batch_size,
                                                         int64_t num_heads, int64_t seq_len_q, int64_t seq_len_k,
                                                         int64_t d_k, int64_t d_v, long long *ticks32);

/* ---- section profile of the tensor-core kernels: the counterpart, for the fp16 path, of the reference's
 *      profile_sections_sdpa_* (csrc/tensor_ops.cpp:1434-1507) over the TX_TICK clock64 sections of
 *      csrc/cuda/profiling.cuh:20-51.  Runs `desc` (fp16, d in {64,128,256,512}) once on an instrumented build of
 *      the kernel that serves that shape and returns 64 cycle counters of CTA (0,0,0), summed over its key tiles.
 *      d = 64, 128 (two query tiles per CTA): softmax lane of query tile 0 in [0..10], of query tile 1 in [32..42]:
 *        [+0] loop total, [+1] wait for S, [+2] S -> registers, [+3] mask, [+5] row max + exponentials + pack + sum,
 *        [+6] wait for the previous PV (+ O rescale), [+7] P store + hand-over, [+9] epilogue, [+10] key tiles;
 *        MMA lane: [16] loop total, [17] wait for S to be consumed, [18] wait for K, [19] wait for P,
 *        [20] wait for V, [21] MMA issue (blocks while the tensor pipe's queue is full).
 *        The CTA's start and end, in cycles from its first instruction: softmax lane [+11] first score tile in hand,
 *        [+12] end of the loop, [+13] end of the epilogue; from the end of the loop [+14] last PV finished,
 *        [+15] last result store issued; MMA lane [22] started (barriers, tensor memory and the CTA-wide meeting
 *        done), [23] Q tile 0 in shared memory, [24] first K tile in shared memory.
 *      d = 256, 512 (one query tile per CTA): softmax lane [0] loop total, [1] wait for S, [2] S -> registers,
 *        [3] mask + row max, [5] exponentials + pack + sum, [6] wait for the previous PV, [7] O rescale,
 *        [8] P store + hand-over, [9] epilogue, [10] key tiles; MMA lane [16] total, [17] wait for S to be consumed,
 *        [18] K wait + QK^T issue, [19] wait for V, [20] wait for P, [21] PV issue; producer lane [24] total,
 *        [25] wait for a free K stage, [26] wait for a free V stage.  Entries not listed stay 0. */
TX_API int tx_profile_sections_sdpa(const tx_sdpa_desc *desc, long long *ticks64);

/* ---- failure-path self-test (no reference counterpart: the reference's device code cannot fail softly, its host
 *      code prints and exits, csrc/cuda/cuda_utils.cuh:6-14).  Runs `desc` (fp16, d = 64) on an instantiation of the
 *      production kernel whose bounded waits give up after 2 ms instead of 2 s and whose TMA producer leaves out K
 *      tile `skip_k_tile` of every CTA (-1: none, the call is then an ordinary forward pass).  With a tile left out
 *      the MMA warp's wait for it runs out: the CTA records stage code 3 in the device status word, overwrites its
 *      output rows with NaN, drains, frees its tensor memory and returns; the call waits for the stream and returns
 *      TX_ERR_KERNEL, as tx_sdpa_finish does after any kernel that gave up.  Nothing faults, traps or spins without
 *      bound, and the context stays usable: the next ordinary launch is unaffected. */
TX_API int tx_selftest_wait_timeout(const tx_sdpa_desc *desc, int32_t skip_k_tile);

/* ---- backward: the reference's autograd rule for 'scaled_dot_product_attention'
 *      (tensorax/tensor.py:806-827: dV = P^T dO, dP = dO V^T, dS = P o (dP - rowsum(dP o P)) / sqrt(d),
 *      dQ = dS K, dK = dS^T Q), which the reference evaluates with dense [Sq,Sk] temporaries through
 *      Tensor.transpose/matmul.  Here: flash-style on the tensor cores, P rebuilt from the forward's `lse`,
 *      gradients of grouped K/V heads summed over their query heads, no atomics (bitwise reproducible).
 *      fp16 q/k/v with d in {64,128,256}, implicit masks only (causal / kv_lens); asynchronous on `stream`
 *      (tx_sdpa_finish reports kernel-side failures).  Takes 2*batch*q_heads*seq_q*(d+2) bytes from the
 *      device's stream-ordered pool for the fp16 copy of `dout` and the row sums, and returns them. */
typedef struct tx_sdpa_bwd_desc {
    const void *q, *k, *v;    /* fp16, exactly what the forward got */
    const void *out;          /* the forward's result: fp32, or fp16 with TX_SDPA_OUT_F16 in flags */
    const float *dout;        /* gradient of the result, fp32 [batch, q_heads, seq_q, d] */
    const float *lse;         /* [batch, q_heads, seq_q], written by tx_sdpa_forward through desc.lse */
    const int32_t *kv_lens;   /* optional [batch], as in the forward */
    float *dq, *dk, *dv;      /* fp32 [batch, q_heads, seq_q, d], [batch, kv_heads, seq_k, d] x 2 */
    int64_t batch, q_heads, kv_heads, seq_q, seq_k, d;
    int32_t causal;
    int32_t flags;            /* TX_SDPA_OUT_F16: dtype of `out` */
    void *stream;
} tx_sdpa_bwd_desc;
TX_API int tx_sdpa_backward(const tx_sdpa_bwd_desc *desc);

/* ---- host-buffer form (no reference counterpart): `desc` holds HOST pointers
 *      (q, k, v, kv_lens, out; mask must be NULL).  Copies in, runs, copies out,
 *      and returns when `out` is complete.  Device staging buffers are cached in
 *      the library and reused between calls.  With pinned buffers (tx_host_alloc_pinned) uploads, kernels and
 *      the way back overlap in chunks of whole (batch, head) units, and the results are written into `out` by a
 *      small kernel (the device addresses pinned memory directly); pageable buffers work too, through staged copies. */
TX_API int tx_sdpa_forward_host(const tx_sdpa_desc *desc);
/* The copy schedule of tx_sdpa_forward_host with the kernels left out (no reference counterpart): same chunks, same
 * three streams, same bytes in both directions, `out` on the host receives whatever the device staging buffer holds.
 * The benchmark times it beside the full call to show how much of the end-to-end time is the host <-> device path. */
TX_API int tx_sdpa_forward_host_copies_only(const tx_sdpa_desc *desc);

/* ---- allocation-free form (no counterpart in the reference).
 *
 * For callers that must not, or cannot, allocate device memory while they run
 * attention: a host program whose device memory is handed out once, up front, by
 * its own arena or memory planner and that forbids libraries from calling
 * cudaMalloc behind its back; a serving loop that cannot afford the device-wide
 * synchronisation an allocation implies; a process already at its memory limit.
 * Every other entry point of this library may allocate (a status word per
 * device on first use, staging buffers in the _host form).
 *
 * This one allocates nothing, ever.  The tensor-core kernel's scratch -- the
 * status word its bounded waits report through and the device copy of the
 * per-batch key lengths -- lives in a fixed array that is part of the loaded
 * library image on every GPU (TX_STATIC_SCRATCH_BYTES, held until the process
 * exits).  The caller passes inputs and outputs as usual; `kv_lens_host` is a
 * HOST array of `batch` lengths, or NULL.
 *
 * Limits: fp16 inputs, d_k == d_v in {64, 128, 256, 512}, 16-byte aligned pointers (the
 * shapes the tensor-core kernel takes -- others are refused with
 * TX_ERR_UNSUPPORTED, never routed elsewhere), and batch <=
 * TX_STATIC_SCRATCH_MAX_BATCH when key lengths are given (TX_ERR_INVALID beyond).
 *
 * The first call on a device looks up the array's device address once; make
 * that first call before any stream capture begins.  All calls on one GPU share
 * the array: the entry point clears the status word and overwrites the lengths
 * itself, but two calls whose kernels may overlap on the GPU (different
 * streams, or different host threads) race on it -- serialise them.
 * Returns after `out` is complete, like the reference launchers. */
#define TX_STATIC_SCRATCH_MAX_BATCH 4096
#define TX_STATIC_SCRATCH_BYTES (256 + 4 * TX_STATIC_SCRATCH_MAX_BATCH)
TX_API int tx_sdpa_fp16_static_scratch(const void *Q_h, const void *K_h, const void *V_h, float *out,
                                       int64_t batch, int64_t q_heads, int64_t kv_heads,
                                       int64_t seq_q, int64_t seq_k, int64_t d, int32_t causal,
                                       const int32_t *kv_lens_host, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* TENSORAX_B200_H */
