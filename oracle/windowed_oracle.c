/*
 * CPU oracle, plain C.  TEST INFRASTRUCTURE ONLY — never linked into, loaded by
 * or called from the shipped library.
 *
 * A second, independent restatement of the attention core of the reference's
 * titans_core/attn/windowed_attention.py, written as scalar loops with double
 * accumulation so that it shares nothing with either PyTorch's fused attention
 * or the CUDA kernels.  Parity status: pinned through the golden fixtures (this
 * file is checked against them in the CPU test-suite).
 *
 * Mask rule (windowed_attention.py:113-150), for query position p and key
 * position g, both counted over the whole length L = Np + T:
 *   g <  Np                          -> visible            (:118)
 *   p <  Np and g >= Np              -> hidden             (:115, :122-132)
 *   p >= Np and g >= Np              -> g <= p and p - g <= w   (:136-150)
 * Scores are scaled by 1/sqrt(dh) unless a scale is given (:318-323 uses the
 * library default) and soft-maxed over the visible keys.
 *
 * Build: make -C oracle   (produces oracle/liboracle_c.so)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

static int key_visible(long p, long g, long w, long np) {
    if (g < np) return 1;
    if (p < np) return 0;
    return g <= p && p - g <= w;
}

/* Number of visible keys of query position p in a length-L problem. */
long tmw_oracle_row_count(long p, long L, long w, long np) {
    long n = 0;
    for (long g = 0; g < L; ++g) n += key_visible(p, g, w, np);
    return n;
}

/*
 * q: [B, H, q_rows, dh], k/v: [B, H, k_rows, dh], o: [B, H, q_rows, dh], all
 * contiguous float32.  Query row r sits at position q_pos0 + r.  Key rows
 * [0, Np) are the persistent keys (positions 0..Np-1); key row Np + i sits at
 * position k_pos0 + i.  For the unsharded problem q_pos0 = 0 and k_pos0 = Np.
 * Returns 0, or -1 on bad arguments.
 */
int tmw_oracle_attention_f32(const float* q, const float* k, const float* v, float* o,
                             int B, int H, int q_rows, int k_rows, int dh,
                             int w, int np, long q_pos0, long k_pos0, float scale) {
    if (B < 0 || H < 0 || q_rows < 0 || k_rows < np || dh <= 0 || w < 0 || np < 0 || k_pos0 < np)
        return -1;
    if (scale == 0.0f) scale = (float)(1.0 / sqrt((double)dh));
    const long n_bh = (long)B * H;
    for (long bh = 0; bh < n_bh; ++bh) {
        for (int r = 0; r < q_rows; ++r) {
            const float* qr = q + (bh * q_rows + r) * (long)dh;
            const float* kb = k + bh * (long)k_rows * dh;
            const float* vb = v + bh * (long)k_rows * dh;
            float* orow = o + (bh * q_rows + r) * (long)dh;
            const long p = q_pos0 + r;
            double* acc = (double*)calloc((size_t)dh, sizeof(double));
            double m = -INFINITY, l = 0.0;
            for (int pass = 0; pass < 2; ++pass) {
                for (int kr = 0; kr < k_rows; ++kr) {
                    const long g = kr < np ? kr : k_pos0 + (kr - np);
                    if (!key_visible(p, g, w, np)) continue;
                    double s = 0.0;
                    for (int d = 0; d < dh; ++d) s += (double)qr[d] * (double)kb[(long)kr * dh + d];
                    s *= (double)scale;
                    if (pass == 0) {
                        if (s > m) m = s;
                    } else {
                        const double e = exp(s - m);
                        l += e;
                        for (int d = 0; d < dh; ++d) acc[d] += e * (double)vb[(long)kr * dh + d];
                    }
                }
            }
            for (int d = 0; d < dh; ++d) orow[d] = l > 0.0 ? (float)(acc[d] / l) : 0.0f;
            free(acc);
        }
    }
    return 0;
}
