/*
 * CPU oracle for scaled-dot-product-attention forward.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference's CPU SDPA
 * (tensorax csrc/cpu/tensor_cpu.cpp:464-529, `sdpa_cpu`).  It is the checker the
 * CUDA path is compared against; it is never linked into, imported by or called
 * from the product library.  Only tests, the smoke check and the benchmark's
 * cpu_baseline / reference legs may load it.
 *
 * Parity status: PINNED.  The restatement is compared bit-for-bit with the
 * reference's own `sdpa_cpu`, compiled from the reference sources by
 * oracle/Makefile into oracle/_ref/, and with golden vectors that build wrote
 * under tests/golden/ (see tests/test_oracle.py).
 *
 * Arithmetic contract kept identical to the reference (file:line of the step):
 *   scale = 1/sqrtf((float)d_k)                              tensor_cpu.cpp:477
 *   score_j = (sum_d q_d*k_jd, fp32, d ascending) * scale    tensor_cpu.cpp:491-495
 *   score_j += mask_ij   when a mask is given                tensor_cpu.cpp:496
 *   row max starts at -FLT_MAX, strict '>' update            tensor_cpu.cpp:489,497
 *   a_j = expf(score_j - max); sum in j-ascending order      tensor_cpu.cpp:502-511
 *   a_j /= sum   (normalise BEFORE the value product)        tensor_cpu.cpp:513-515
 *   o_d = sum_j a_j*v_jd, fp32, j ascending                  tensor_cpu.cpp:517-523
 * A fully masked row therefore yields 0/0 = NaN, as in the reference.
 * The reference evaluates every score twice; the values are identical both
 * times, so this file keeps them in a row buffer instead.
 *
 * Build without value-changing options (no -ffast-math, no FMA contraction):
 *   gcc -O2 -ffp-contract=off -fPIC -shared oracle/sdpa_oracle.c -lm
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

#if defined(__GNUC__)
#define ORACLE_API __attribute__((visibility("default")))
#else
#define ORACLE_API
#endif

/* One query row: q[d_k] against n_keys keys; `mrow` may be NULL. */
static void oracle_row(const float *q, const float *k, const float *v, const float *mrow,
                       float *o, float *attn, int64_t n_keys, int64_t d_k, int64_t d_v,
                       float scale)
{
    float row_max = -FLT_MAX;
    for (int64_t j = 0; j < n_keys; ++j) {
        const float *kj = k + j * d_k;
        float s = 0.0f;
        for (int64_t d = 0; d < d_k; ++d) s += q[d] * kj[d];
        s *= scale;
        if (mrow) s += mrow[j];
        attn[j] = s;
        if (s > row_max) row_max = s;
    }
    float denom = 0.0f;
    for (int64_t j = 0; j < n_keys; ++j) {
        attn[j] = expf(attn[j] - row_max);
        denom += attn[j];
    }
    for (int64_t j = 0; j < n_keys; ++j) attn[j] /= denom;
    for (int64_t d = 0; d < d_v; ++d) {
        float acc = 0.0f;
        for (int64_t j = 0; j < n_keys; ++j) acc += attn[j] * v[j * d_v + d];
        o[d] = acc;
    }
}

/* Same argument list and meaning as the reference's sdpa_cpu
 * (csrc/tensor_ops.h:132-134): contiguous [B,H,S,d] fp32, optional dense
 * additive mask [B,H,Sq,Sk]. */
ORACLE_API void oracle_sdpa_f32(const float *Q, const float *K, const float *V, const float *mask,
                                float *out, int64_t B, int64_t H, int64_t Sq, int64_t Sk,
                                int64_t d_k, int64_t d_v)
{
    const float scale = 1.0f / sqrtf((float)d_k);
    float *attn = (float *)malloc(sizeof(float) * (size_t)(Sk > 0 ? Sk : 1));
    for (int64_t bh = 0; bh < B * H; ++bh) {
        const float *q = Q + bh * Sq * d_k;
        const float *k = K + bh * Sk * d_k;
        const float *v = V + bh * Sk * d_v;
        const float *m = mask ? mask + bh * Sq * Sk : NULL;
        float *o = out + bh * Sq * d_v;
        for (int64_t i = 0; i < Sq; ++i)
            oracle_row(q + i * d_k, k, v, m ? m + i * Sk : NULL, o + i * d_v, attn, Sk, d_k, d_v,
                       scale);
    }
    free(attn);
}

/*
 * Structured-mask / grouped-head form used for the large configurations, where
 * the dense [B,H,Sq,Sk] mask the reference API would need cannot be materialised.
 * It is the same per-row arithmetic with the mask row built on the fly:
 *   mask_ij = 0      if (j < kv_lens[b] or kv_lens == NULL) and (!causal or j <= i)
 *           = -inf   otherwise
 * which is exactly what the reference's create_causal_mask / create_padding_mask
 * (tensorax/nn/attention/utils.py:4-21) put in a dense mask.  Query head h reads
 * K/V head h / (Hq/Hkv), the mapping of the reference's repeat_interleave
 * (csrc/tensor_ops.cpp:145-154: output index j*r+t <- input j).
 * Only query heads [bh_begin, bh_end) (flattened b*Hq+h) and rows
 * [row_begin, row_end) are evaluated and written; `out` has the full
 * [B,Hq,Sq,d_v] layout.
 */
ORACLE_API void oracle_sdpa_structured(const float *Q, const float *K, const float *V, float *out,
                                       int64_t B, int64_t Hq, int64_t Hkv, int64_t Sq, int64_t Sk,
                                       int64_t d_k, int64_t d_v, int causal,
                                       const int32_t *kv_lens, int64_t bh_begin, int64_t bh_end,
                                       int64_t row_begin, int64_t row_end)
{
    const float scale = 1.0f / sqrtf((float)d_k);
    const int64_t group = Hq / Hkv;
    float *attn = (float *)malloc(sizeof(float) * (size_t)(Sk > 0 ? Sk : 1));
    float *mrow = (float *)malloc(sizeof(float) * (size_t)(Sk > 0 ? Sk : 1));
    (void)B;
    for (int64_t bh = bh_begin; bh < bh_end; ++bh) {
        const int64_t b = bh / Hq, h = bh % Hq;
        const int64_t kvh = b * Hkv + h / group;
        const float *q = Q + bh * Sq * d_k;
        const float *k = K + kvh * Sk * d_k;
        const float *v = V + kvh * Sk * d_v;
        float *o = out + bh * Sq * d_v;
        const int64_t len = kv_lens ? (int64_t)kv_lens[b] : Sk;
        for (int64_t i = row_begin; i < row_end; ++i) {
            const int use_mask = causal || kv_lens;
            if (use_mask)
                for (int64_t j = 0; j < Sk; ++j)
                    mrow[j] = (j < len && (!causal || j <= i)) ? 0.0f : -INFINITY;
            oracle_row(q + i * d_k, k, v, use_mask ? mrow : NULL, o + i * d_v, attn, Sk, d_k,
                       d_v, scale);
        }
    }
    free(attn);
    free(mrow);
}

/*
 * Linear layer of the reference: F.linear (tensorax/functional.py:105-110) is
 * `x @ weight.T` through matmul_cpu (csrc/cpu/tensor_cpu.cpp:131-156: the output
 * element starts at 0.0f and accumulates a[i,p]*b[p,j] for p ascending) followed by
 * a broadcast add of the bias.  x [rows, K], w [N, K], bias [N] or NULL, out [rows, N].
 */
ORACLE_API void oracle_linear_f32(const float *x, const float *w, const float *bias, float *out,
                                  int64_t rows, int64_t K, int64_t N)
{
    for (int64_t i = 0; i < rows; ++i)
        for (int64_t j = 0; j < N; ++j) {
            float acc = 0.0f;
            for (int64_t p = 0; p < K; ++p) acc += x[i * K + p] * w[j * K + p];
            out[i * N + j] = bias ? acc + bias[j] : acc;
        }
}
