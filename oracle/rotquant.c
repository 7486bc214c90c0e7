/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the ODM-KV Lloyd-Max quantiser.
 *
 * Restates TurboQuantMSE.quantize / .dequantize of the reference
 * (kvquant/tq_backend.py:185-203) and the nearest-centroid rule its comment at
 * kvquant/tq_backend.py:191-196 describes (searchsorted, clamp, two distances, where).
 *
 * The reference's "x_unit @ pi.T" is a library SGEMM whose summation order is not
 * specified.  This restatement fixes one order: a single fp32 fused-multiply-add
 * chain over the contraction index in ascending order, starting from +0.  The CUDA
 * kernels use the same chain, so codes can be compared bit for bit.  Coordinates that
 * fall within rounding distance of a Voronoi midpoint may differ from a run of the
 * reference itself; the golden fixtures record how many do.
 *
 * Nothing outside tests/, the smoke check and the bench's CPU-baseline leg may load
 * this file's shared object.
 */
#include <math.h>
#include <stdint.h>
#include <stddef.h>

/* fp32 L2 norm as one ascending FMA chain of squares, then an IEEE square root. */
static float chain_norm(const float *x, int d) {
    float acc = 0.0f;
    for (int i = 0; i < d; ++i) acc = fmaf(x[i], x[i], acc);
    return sqrtf(acc);
}

/* searchsorted(left) + neighbour pick; the lower index wins an exact tie. */
static int nearest_centroid(float y, const float *c, int k) {
    int lo = 0, hi = k; /* first index with c[idx] >= y */
    while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (c[mid] < y) lo = mid + 1; else hi = mid;
    }
    int idx = lo;
    int a = idx - 1 < 0 ? 0 : idx - 1;
    int b = idx > k - 1 ? k - 1 : idx;
    float da = fabsf(y - c[a]);
    float db = fabsf(y - c[b]);
    return (da <= db) ? a : b;
}

/*
 * x      [n, d] fp32 (already upcast from the cache dtype)
 * pi     [d, d] fp32 row-major; y_j = sum_i x_unit[i] * pi[j, i]   (x_unit @ pi.T)
 * cent   [k]    fp32 ascending
 * idx    [n, d] uint8 out, norms [n] fp32 out, y [n, d] fp32 out (may be NULL)
 * Follows kvquant/tq_backend.py:185-197.
 */
void oracle_quantize(const float *x, int64_t n, int d, const float *pi,
                     const float *cent, int k, uint8_t *idx, float *norms, float *y_out) {
    float unit[1024];
    for (int64_t r = 0; r < n; ++r) {
        const float *xr = x + r * d;
        float nrm = chain_norm(xr, d);
        norms[r] = nrm;
        float den = nrm + 1e-10f;
        for (int i = 0; i < d; ++i) unit[i] = xr[i] / den;
        for (int j = 0; j < d; ++j) {
            const float *pj = pi + (size_t)j * d;
            float acc = 0.0f;
            for (int i = 0; i < d; ++i) acc = fmaf(unit[i], pj[i], acc);
            if (y_out) y_out[r * d + j] = acc;
            idx[r * d + j] = (uint8_t)nearest_centroid(acc, cent, k);
        }
    }
}

/* Encode-only stage: nearest centroid of already-rotated coordinates. */
void oracle_encode(const float *y, int64_t count, const float *cent, int k, uint8_t *idx) {
    for (int64_t r = 0; r < count; ++r) idx[r] = (uint8_t)nearest_centroid(y[r], cent, k);
}

/*
 * x_hat_j = (sum_i cent[idx_i] * pi[i, j]) * norm      (y_hat @ pi, then scale)
 * Follows kvquant/tq_backend.py:199-203.  Same ascending FMA chain.
 */
void oracle_dequantize(const uint8_t *idx, const float *norms, int64_t n, int d,
                       const float *pi, const float *cent, float *x_hat) {
    for (int64_t r = 0; r < n; ++r) {
        const uint8_t *ir = idx + r * d;
        for (int j = 0; j < d; ++j) {
            float acc = 0.0f;
            for (int i = 0; i < d; ++i) acc = fmaf(cent[ir[i]], pi[(size_t)i * d + j], acc);
            x_hat[r * d + j] = acc * norms[r];
        }
    }
}
