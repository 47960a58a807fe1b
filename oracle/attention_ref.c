/* TEST INFRASTRUCTURE ONLY: a plain-C, double-precision restatement of the attention the
 * hot path computes. Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline /
 * reference legs may load it; the product never does.
 *
 * What it restates. The reference checks its flash kernels against
 * F.scaled_dot_product_attention on float64 tensors with K/V repeat_interleave'd for
 * grouped heads (tests/hardware/ops/test_flash.py:57-63), float64 autograd for
 * gradients (:197-215), a per-sequence loop with the causal rule
 * arange(m) < arange(n) + 1 + m - n for packed batches
 * (tests/hardware/ops/test_flash_varlen.py:62-73) and a bool mask key < length for key
 * lengths (tests/hardware/ops/test_attention_lengths.py:37-52). The arithmetic itself
 * lives in PyTorch (the reference pins torch 2.11 to 2.15, README.md:99-100), which is
 * not part of the reference tree, so this file writes the published definition out:
 *
 *   s_ij = scale * q_i . k_j + mask_ij          (mask clamped below at -5e5,
 *                                                ktt_flash/varlen_plan.hpp:12-17)
 *   visible(i, j) = j < len  and  (not causal or j <= i + shift)
 *       shift = 0 for dense calls (top-left, aten_attention.cpp:431-436),
 *       shift = Lk - Lq for packed calls (bottom-right, varlen_plan.hpp:69-70)
 *   p_ij = softmax_j over visible j,  o_i = sum_j p_ij v_j,  lse_i = log sum_j exp s_ij
 *   backward: delta_i = do_i . o_i, ds_ij = p_ij (do_i . v_j - delta_i),
 *             dq_i = scale sum_j ds_ij k_j, dk_j = scale sum_i ds_ij q_i,
 *             dv_j = sum_i p_ij do_i     (dk, dv summed over the query heads of a group)
 *
 * Pinned by tests/test_oracle.py against torch's float64 SDPA and float64 autograd on
 * the reference's own test shapes, and against tests/golden/*.
 */
#include <math.h>
#include <stdlib.h>

#define MASKED_LOGIT (-5e5)

/* Scores of one (b, h, i) row into s[0..Sk); returns the row maximum over visible keys. */
static double row_scores(
    const double* q, const double* k, const double* mask, int len, int i, int Sk, int D,
    int causal, int shift, double scale, double* s) {
    double mx = -INFINITY;
    for (int j = 0; j < Sk; ++j) {
        if (j >= len || (causal && j > i + shift)) {
            s[j] = -INFINITY;
            continue;
        }
        double acc = 0.0;
        for (int c = 0; c < D; ++c) acc += q[c] * k[(long)j * D + c];
        acc *= scale;
        if (mask) {
            double m = mask[j];
            acc += (m > MASKED_LOGIT) ? m : MASKED_LOGIT;
        }
        s[j] = acc;
        if (acc > mx) mx = acc;
    }
    return mx;
}

/* q [B,H,Sq,D], k [B,Hk,Sk,D], v [B,Hk,Sk,Dv], mask [B,H,Sq,Sk] additive or NULL,
 * key_lengths [B] or NULL, out [B,H,Sq,Dv], lse [B,H,Sq]; all contiguous.
 * causal: 0 none, 1 top-left, 2 bottom-right. */
int attn_ref_forward(
    const double* q, const double* k, const double* v, const double* mask,
    const int* key_lengths, int B, int H, int Hk, int Sq, int Sk, int D, int Dv, int causal,
    double scale, double* out, double* lse) {
    if (H % Hk) return -1;
    const int group = H / Hk;
    const int shift = causal == 2 ? Sk - Sq : 0;
    double* s = (double*)malloc(sizeof(double) * (size_t)Sk);
    if (!s) return -2;
    for (int b = 0; b < B; ++b) {
        int len = Sk;
        if (key_lengths) {
            len = key_lengths[b] < 1 ? 1 : key_lengths[b];
            if (len > Sk) len = Sk;
        }
        for (int h = 0; h < H; ++h) {
            const double* kb = k + ((long)b * Hk + h / group) * Sk * D;
            const double* vb = v + ((long)b * Hk + h / group) * Sk * Dv;
            for (int i = 0; i < Sq; ++i) {
                const long row = ((long)b * H + h) * Sq + i;
                const double* mrow = mask ? mask + row * Sk : 0;
                const double mx = row_scores(q + row * D, kb, mrow, len, i, Sk, D, causal, shift, scale, s);
                double* o = out + row * Dv;
                for (int c = 0; c < Dv; ++c) o[c] = 0.0;
                if (mx == -INFINITY) {
                    if (lse) lse[row] = -INFINITY;
                    continue;
                }
                double sum = 0.0;
                for (int j = 0; j < Sk; ++j) {
                    s[j] = (s[j] == -INFINITY) ? 0.0 : exp(s[j] - mx);
                    sum += s[j];
                }
                for (int j = 0; j < Sk; ++j) {
                    const double p = s[j] / sum;
                    if (p == 0.0) continue;
                    for (int c = 0; c < Dv; ++c) o[c] += p * vb[(long)j * Dv + c];
                }
                if (lse) lse[row] = mx + log(sum);
            }
        }
    }
    free(s);
    return 0;
}

/* Gradients for the same operands; dq [B,H,Sq,D], dk [B,Hk,Sk,D], dv [B,Hk,Sk,Dv]. */
int attn_ref_backward(
    const double* q, const double* k, const double* v, const double* mask,
    const int* key_lengths, const double* dout, int B, int H, int Hk, int Sq, int Sk, int D,
    int Dv, int causal, double scale, double* dq, double* dk, double* dv) {
    if (H % Hk) return -1;
    const int group = H / Hk;
    const int shift = causal == 2 ? Sk - Sq : 0;
    double* s = (double*)malloc(sizeof(double) * (size_t)Sk);
    double* o = (double*)malloc(sizeof(double) * (size_t)Dv);
    if (!s || !o) return -2;
    for (long n = 0; n < (long)B * H * Sq * D; ++n) dq[n] = 0.0;
    for (long n = 0; n < (long)B * Hk * Sk * D; ++n) dk[n] = 0.0;
    for (long n = 0; n < (long)B * Hk * Sk * Dv; ++n) dv[n] = 0.0;
    for (int b = 0; b < B; ++b) {
        int len = Sk;
        if (key_lengths) {
            len = key_lengths[b] < 1 ? 1 : key_lengths[b];
            if (len > Sk) len = Sk;
        }
        for (int h = 0; h < H; ++h) {
            const long kv = ((long)b * Hk + h / group) * Sk;
            const double* kb = k + kv * D;
            const double* vb = v + kv * Dv;
            for (int i = 0; i < Sq; ++i) {
                const long row = ((long)b * H + h) * Sq + i;
                const double* mrow = mask ? mask + row * Sk : 0;
                const double* qi = q + row * D;
                const double* doi = dout + row * Dv;
                const double mx = row_scores(qi, kb, mrow, len, i, Sk, D, causal, shift, scale, s);
                if (mx == -INFINITY) continue;
                double sum = 0.0;
                for (int j = 0; j < Sk; ++j) {
                    s[j] = (s[j] == -INFINITY) ? 0.0 : exp(s[j] - mx);
                    sum += s[j];
                }
                for (int c = 0; c < Dv; ++c) o[c] = 0.0;
                for (int j = 0; j < Sk; ++j) {
                    s[j] /= sum;
                    for (int c = 0; c < Dv; ++c) o[c] += s[j] * vb[(long)j * Dv + c];
                }
                double delta = 0.0;
                for (int c = 0; c < Dv; ++c) delta += doi[c] * o[c];
                for (int j = 0; j < Sk; ++j) {
                    const double p = s[j];
                    if (p == 0.0) continue;
                    double dp = 0.0;
                    for (int c = 0; c < Dv; ++c) dp += doi[c] * vb[(long)j * Dv + c];
                    const double ds = p * (dp - delta) * scale;
                    for (int c = 0; c < D; ++c) {
                        dq[row * D + c] += ds * kb[(long)j * D + c];
                        dk[(kv + j) * D + c] += ds * qi[c];
                    }
                    for (int c = 0; c < Dv; ++c) dv[(kv + j) * Dv + c] += p * doi[c];
                }
            }
        }
    }
    free(s);
    free(o);
    return 0;
}
