/* CPU oracle for the SS2D core of VMamba, C restatement -- TEST INFRASTRUCTURE.
 *
 * Same algorithm as oracle/ss2d_oracle.py (which is the readable statement and is
 * pinned against the reference's golden outputs); this file exists so that the
 * oracle finishes full-size workloads in seconds and can serve as the timed CPU
 * baseline on all host cores.  It is compiled by oracle/Makefile into
 * oracle/libss2d_oracle.so and is only ever loaded by tests, the smoke check and
 * the benchmark's CPU-baseline legs.
 *
 * Reference anchors (paths inside MzeroMiko/VMamba):
 *   orc_cross_scan      vmamba.py:41-84     cross_scan_fwd, channel-first
 *   orc_cross_merge     vmamba.py:87-130    cross_merge_fwd, channel-first
 *   orc_selective_scan  vmamba.py:791-834   selective_scan_torch
 *   orc_layer_norm_cf   vmamba.py:1078-1093 LayerNorm(channel_first=True)
 * All tensors are dense float32, C order.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

/* position in the (H, W) map visited at step l of route k (scans mode `scans`) */
static inline int64_t route_pos(int scans, int k, int64_t l, int64_t H, int64_t W)
{
    const int64_t L = H * W;
    if (scans == 0) {
        int64_t t = (k >= 2) ? (L - 1 - l) : l;      /* routes 2,3 = routes 0,1 reversed */
        if ((k & 1) == 0) return t;                 /* row-major */
        return (t % H) * W + (t / H);               /* column-major: t = w*H + h */
    }
    if (scans == 1) return l;
    if (scans == 2) return (k >= 2) ? (L - 1 - l) : l;
    /* scans == 3: row-major walk over rot90(x, k) */
    switch (k) {
    case 0: return l;
    case 1: { int64_t i = l / H, j = l % H; return j * W + (W - 1 - i); }   /* out (W,H): x[j, W-1-i] */
    case 2: return L - 1 - l;
    default: { int64_t i = l / H, j = l % H; return (H - 1 - j) * W + i; }  /* x[H-1-j, i] */
    }
}

void orc_cross_scan(const float *x, float *y, int64_t B, int64_t C, int64_t H, int64_t W, int scans)
{
    const int64_t L = H * W;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t b = 0; b < B; ++b)
        for (int64_t kc = 0; kc < 4 * C; ++kc) {
            const int k = (int)(kc / C);
            const int64_t c = kc % C;
            const float *src = x + (b * C + c) * L;
            float *dst = y + ((b * 4 + k) * C + c) * L;
            for (int64_t l = 0; l < L; ++l) dst[l] = src[route_pos(scans, k, l, H, W)];
        }
}

/* y[b,c,p] = sum over routes of ys[b,k,c,l] with route_pos(k,l) == p.
 * Association order of the reference: scans 0 -> (y0 + y2) + (y1 + y3);
 * scans 1 -> ((y0+y1)+y2)+y3; scans 2 -> (y0+y2) + (y1+y3); scans 3 -> ((y0+y1)+y2)+y3. */
void orc_cross_merge(const float *ys, float *y, int64_t B, int64_t C, int64_t H, int64_t W, int scans)
{
    const int64_t L = H * W;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t b = 0; b < B; ++b)
        for (int64_t c = 0; c < C; ++c) {
            const float *s0 = ys + ((b * 4 + 0) * C + c) * L;
            const float *s1 = ys + ((b * 4 + 1) * C + c) * L;
            const float *s2 = ys + ((b * 4 + 2) * C + c) * L;
            const float *s3 = ys + ((b * 4 + 3) * C + c) * L;
            float *dst = y + (b * C + c) * L;
            if (scans == 0) {
                for (int64_t h = 0; h < H; ++h)
                    for (int64_t w = 0; w < W; ++w) {
                        const int64_t p = h * W + w, q = w * H + h;
                        dst[p] = (s0[p] + s2[L - 1 - p]) + (s1[q] + s3[L - 1 - q]);
                    }
            } else if (scans == 1) {
                for (int64_t p = 0; p < L; ++p) dst[p] = ((s0[p] + s1[p]) + s2[p]) + s3[p];
            } else if (scans == 2) {
                for (int64_t p = 0; p < L; ++p) dst[p] = (s0[p] + s2[L - 1 - p]) + (s1[p] + s3[L - 1 - p]);
            } else {
                memset(dst, 0, sizeof(float) * (size_t)L);
                for (int64_t l = 0; l < L; ++l) dst[l] = s0[l];
                for (int64_t l = 0; l < L; ++l) dst[route_pos(3, 1, l, H, W)] += s1[l];
                for (int64_t l = 0; l < L; ++l) dst[route_pos(3, 2, l, H, W)] += s2[l];
                for (int64_t l = 0; l < L; ++l) dst[route_pos(3, 3, l, H, W)] += s3[l];
            }
        }
}

static inline float softplus_f(float x)
{
    return (x > 20.0f) ? x : log1pf(expf(x));       /* F.softplus, threshold 20 */
}

/* u, delta, out: (Bt, K*Cd, L); A: (K*Cd, N); Bm, Cm: (Bt, K, N, L); D, bias: (K*Cd) or NULL.
 * `h` scratch is on the stack for N <= 256 (the reference's own limit). */
int orc_selective_scan(const float *u, const float *delta, const float *A, const float *Bm,
                       const float *Cm, const float *D, const float *bias, float *out,
                       int64_t Bt, int64_t K, int64_t Cd, int64_t N, int64_t L, int delta_softplus)
{
    if (N > 256 || N < 1) return -1;
    const int64_t KC = K * Cd;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t b = 0; b < Bt; ++b)
        for (int64_t r = 0; r < KC; ++r) {
            const int64_t k = r / Cd;
            const float *ur = u + (b * KC + r) * L;
            const float *dr = delta + (b * KC + r) * L;
            const float *Br = Bm + (b * K + k) * N * L;
            const float *Cr = Cm + (b * K + k) * N * L;
            float *orow = out + (b * KC + r) * L;
            const float bi = bias ? bias[r] : 0.0f;
            const float Dv = D ? D[r] : 0.0f;
            float h[256];
            for (int64_t n = 0; n < N; ++n) h[n] = 0.0f;
            for (int64_t l = 0; l < L; ++l) {
                float dl = dr[l] + bi;
                if (delta_softplus) dl = softplus_f(dl);
                const float uu = ur[l];
                float acc = 0.0f;
                for (int64_t n = 0; n < N; ++n) {
                    h[n] = expf(dl * A[r * N + n]) * h[n] + dl * Br[n * L + l] * uu;
                    acc += h[n] * Cr[n * L + l];
                }
                orow[l] = D ? (acc + uu * Dv) : acc;
            }
        }
    return 0;
}

/* LayerNorm over D for each (b, p) of a (B, D, L) array; weight/bias may be NULL */
void orc_layer_norm_cf(const float *y, const float *w, const float *bvec, float *out,
                       int64_t B, int64_t D, int64_t L, float eps)
{
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t b = 0; b < B; ++b)
        for (int64_t p = 0; p < L; ++p) {
            const float *src = y + b * D * L + p;
            float *dst = out + b * D * L + p;
            double s = 0.0;
            for (int64_t d = 0; d < D; ++d) s += src[d * L];
            const float mean = (float)(s / (double)D);
            double v = 0.0;
            for (int64_t d = 0; d < D; ++d) { const float t = src[d * L] - mean; v += (double)t * t; }
            const float rstd = 1.0f / sqrtf((float)(v / (double)D) + eps);
            for (int64_t d = 0; d < D; ++d) {
                float t = (src[d * L] - mean) * rstd;
                if (w) t *= w[d];
                if (bvec) t += bvec[d];
                dst[d * L] = t;
            }
        }
}
