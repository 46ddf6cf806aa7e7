/*
 * CPU oracle for the attention forward path.  TEST INFRASTRUCTURE ONLY: nothing
 * in the shipped library links, loads or calls this file; it is the checker the
 * tests, the smoke test and the benchmark's CPU-baseline leg compare against.
 *
 * It restates, loop for loop, the reference project's naive fp32 attention
 * (src/demo.cu:28-70, `cpu_attention`; the same arithmetic is inlined in
 * src/bench.cu:192-236):
 *
 *   S[i][j] = (sum_k Q[i][k]*K[j][k]) * scale          src/demo.cu:36-40
 *   causal: j > i  ->  S[i][j] = -1e9f                  src/demo.cu:41-42
 *   m_i = max_j S[i][j], starting from -1e30f           src/demo.cu:48-50
 *   P[i][j] = expf(S[i][j]-m_i); sum_i += P[i][j]       src/demo.cu:52-56
 *   P[i][j] /= sum_i                                    src/demo.cu:57-58
 *   O[i][k] = sum_j P[i][j]*V[j][k]                     src/demo.cu:62-69
 *
 * all in fp32 and in the same summation order, so on square inputs the result
 * is bit-identical to the reference function compiled with the same flags.
 *
 * Additions the reference's oracle does not have (the kernel under test needs
 * them checked): the log-sum-exp  LSE_i = m_i + logf(sum_i)  in natural-log
 * units (the quantity kernels/flash_attention.cu:498-505 writes to L),
 * rectangular problems (n_q query rows against n_kv keys, with the causal
 * diagonal shifted by `causal_shift` so that key j is masked iff
 * j > i + causal_shift), and evaluating only a chosen subset of query rows so
 * that long sequences can be spot-checked in seconds.
 *
 * Build: see oracle/build_oracle.py (plain gcc, no fast-math, no FMA
 * contraction, so the summation order above is what the machine executes).
 */
#include <math.h>
#include <stddef.h>
#include <stdlib.h>

#ifdef __cplusplus
extern "C" {
#endif

/*
 * One head.  q: [n_q_total, d] (rows addressed by absolute index), k, v:
 * [n_kv, d].  rows: indices of the query rows to evaluate, or NULL for
 * 0..n_rows-1.  o: [n_rows, d], lse: [n_rows] or NULL, p_out: [n_rows, n_kv]
 * or NULL (normalised probabilities, as the reference returns them).
 * Returns 0, or -1 if scratch allocation failed.
 */
int fa_oracle_rows(const float* q, const float* k, const float* v,
                   float* o, float* lse, float* p_out,
                   const int* rows, int n_rows, int n_kv, int d,
                   float scale, int causal, int causal_shift)
{
    float* s = (float*)malloc((size_t)n_kv * sizeof(float));
    if (!s) return -1;
    for (int r = 0; r < n_rows; r++) {
        const int i = rows ? rows[r] : r;
        const float* qi = q + (size_t)i * d;
        for (int j = 0; j < n_kv; j++) {
            const float* kj = k + (size_t)j * d;
            float dot = 0.0f;
            for (int c = 0; c < d; c++) dot += qi[c] * kj[c];
            s[j] = dot * scale;
            if (causal && j > i + causal_shift) s[j] = -1e9f;
        }
        float max_val = -1e30f;
        for (int j = 0; j < n_kv; j++) max_val = s[j] > max_val ? s[j] : max_val;
        float sum = 0.0f;
        for (int j = 0; j < n_kv; j++) {
            s[j] = expf(s[j] - max_val);
            sum += s[j];
        }
        for (int j = 0; j < n_kv; j++) s[j] /= sum;
        float* oi = o + (size_t)r * d;
        for (int c = 0; c < d; c++) {
            float val = 0.0f;
            for (int j = 0; j < n_kv; j++) val += s[j] * v[(size_t)j * d + c];
            oi[c] = val;
        }
        if (lse) lse[r] = max_val + logf(sum);
        if (p_out) {
            float* pr = p_out + (size_t)r * n_kv;
            for (int j = 0; j < n_kv; j++) pr[j] = s[j];
        }
    }
    free(s);
    return 0;
}

/*
 * Square self-attention for one head, every row: the exact call shape of the
 * reference's cpu_attention(Q,K,V,O,P,seq_len,d_head,scale,causal), plus LSE.
 */
int fa_oracle_head(const float* q, const float* k, const float* v,
                   float* o, float* lse, float* p_out,
                   int seq_len, int d, float scale, int causal)
{
    return fa_oracle_rows(q, k, v, o, lse, p_out, NULL, seq_len, seq_len, d,
                          scale, causal, 0);
}

/*
 * Merge of per-slice partial results, the arithmetic of split-KV decode and of
 * the cross-GPU merge: given n_parts normalised partial outputs o_part[p][d]
 * with their natural-log LSEs,
 *   m = max_p lse_p;  w_p = expf(lse_p - m);  O = sum_p w_p*o_p / sum_p w_p;
 *   LSE = m + logf(sum_p w_p).
 * The reference has no counterpart (it has no split path); this restates the
 * standard log-sum-exp merge so the combine kernel has an independent checker.
 * A part with lse = -INFINITY (empty slice) contributes nothing.
 */
void fa_oracle_merge(const float* o_part, const float* lse_part, int n_parts,
                     int d, float* o, float* lse)
{
    float m = -INFINITY;
    for (int p = 0; p < n_parts; p++) m = lse_part[p] > m ? lse_part[p] : m;
    float wsum = 0.0f;
    for (int c = 0; c < d; c++) o[c] = 0.0f;
    for (int p = 0; p < n_parts; p++) {
        if (lse_part[p] == -INFINITY) continue;
        const float w = expf(lse_part[p] - m);
        wsum += w;
        for (int c = 0; c < d; c++) o[c] += w * o_part[(size_t)p * d + c];
    }
    for (int c = 0; c < d; c++) o[c] = wsum > 0.0f ? o[c] / wsum : 0.0f;
    if (lse) *lse = wsum > 0.0f ? m + logf(wsum) : -INFINITY;
}

#ifdef __cplusplus
}
#endif
