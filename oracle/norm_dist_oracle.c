/*
 * CPU oracle for the norm-distance neuron path of SortNet (G = 1, HW = 1 shapes).
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the arithmetic of the
 * reference CUDA kernels so that the sm_100a kernels can be checked against it.  It is
 * linked/loaded only by the test-suite, by the smoke check and by the CPU-baseline leg of
 * the benchmark; the product library never calls it and has no CPU fallback.
 *
 * Every function cites the reference kernel it follows (paths inside zbh2047/SortNet).
 * All fp32 arithmetic is done with single IEEE operations (compile with
 * -ffp-contract=off, no fast-math) so the bit-exact items (l-inf outputs, IBP bounds,
 * argmax words) can be compared with memcmp.
 *
 * Index-mask layout (core/models/norm_dist.py:14-17, inf_dist_cuda.cu:123,166-169):
 * rows are grouped in sub-batches of 32; sub-batch s uses column list ci[s*CI .. +CI) and
 * row list co[s*CO .. +CO) of the full weight matrix W[W_CO][W_CI].  A NULL list means
 * identity.  CI / CO below are the compact widths seen by x / y.
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_EPS 1e-10f
#define SUB_BATCH 32
#define SIGN_BIT 0x80000000u
#define NO_GRAD_ID 0xffffffffu

static inline const float *w_row(const float *w, const int *co, int s, int CO, int W_CI, int j) {
    int row = co ? co[(size_t)s * CO + j] : j;
    return w + (size_t)row * W_CI;
}

static inline int w_col(const int *ci, int s, int CI, int c) {
    return ci ? ci[(size_t)s * CI + c] : c;
}

/* l-inf forward with argmax word.  inf_dist_cuda.cu:135-211 (strict '>' scan in ascending
 * c from acc = EPS, pos = c | sign bit of (x - w)); :17-107 gives the same y without pos
 * (pos may be NULL here). */
void oracle_inf_dist_forward(const float *x, const float *w, int B, int CO, int CI,
                             float *y, int32_t *pos, const int *ci, const int *co, int W_CI) {
    if (!ci) W_CI = W_CI > 0 ? W_CI : CI;
#pragma omp parallel for schedule(static)
    for (int b = 0; b < B; b++) {
        int s = b / SUB_BATCH;
        const float *xb = x + (size_t)b * CI;
        for (int j = 0; j < CO; j++) {
            const float *wj = w_row(w, co, s, CO, W_CI, j);
            float acc = ORACLE_EPS;
            uint32_t p = 0;
            if (ci) {
                const int *cis = ci + (size_t)s * CI;
                for (int c = 0; c < CI; c++) {
                    float t = xb[c] - wj[cis[c]];
                    float a = fabsf(t);
                    if (a > acc) { acc = a; p = (uint32_t)c | (t >= 0 ? 0u : SIGN_BIT); }
                }
            } else {
                for (int c = 0; c < CI; c++) {
                    float t = xb[c] - wj[c];
                    float a = fabsf(t);
                    if (a > acc) { acc = a; p = (uint32_t)c | (t >= 0 ? 0u : SIGN_BIT); }
                }
            }
            y[(size_t)b * CO + j] = acc;
            if (pos) pos[(size_t)b * CO + j] = (int32_t)p;
        }
    }
}

/* l-inf sparse backward.  inf_dist_cuda.cu:214-271 (value = pos >= 0 ? g : -g, added to
 * grad_x[b, idx]; -value added to grad_w[co[s][j], ci[s][idx]]); launchers :325-354 zero
 * both gradients first.  Sums are taken in double and rounded once, so the result is the
 * correctly rounded sum that any fp32 atomic order approximates.  grad_w may be NULL. */
void oracle_inf_dist_backward(const float *g, const int32_t *pos, int B, int CO, int CI,
                              float *gx, float *gw, const int *ci, const int *co,
                              int W_CO, int W_CI) {
    double *ax = (double *)calloc((size_t)B * CI, sizeof(double));
    double *aw = gw ? (double *)calloc((size_t)W_CO * W_CI, sizeof(double)) : NULL;
    for (int b = 0; b < B; b++) {
        int s = b / SUB_BATCH;
        for (int j = 0; j < CO; j++) {
            uint32_t p = (uint32_t)pos[(size_t)b * CO + j];
            float gv = g[(size_t)b * CO + j];
            int idx = (int)(p & ~SIGN_BIT);
            float v = (p & SIGN_BIT) ? -gv : gv;
            ax[(size_t)b * CI + idx] += v;
            if (aw) {
                int row = co ? co[(size_t)s * CO + j] : j;
                int col = w_col(ci, s, CI, idx);
                aw[(size_t)row * W_CI + col] -= v;
            }
        }
    }
    for (size_t i = 0; i < (size_t)B * CI; i++) gx[i] = (float)ax[i];
    if (aw) for (size_t i = 0; i < (size_t)W_CO * W_CI; i++) gw[i] = (float)aw[i];
    free(ax);
    free(aw);
}

/* Interval-bound forward.  bound_inf_dist_cuda.cu:35-117 (no pos) and :141-237 (pos):
 * midpoint repair when xL > xU (:63), t1 = w - xL, t2 = xU - w, accL from -EPS by strict
 * '<' on min(t1,t2), accU from EPS by strict '>' on max(t1,t2), shared word
 * c | (t1 <= t2 ? 0 : sign bit); posL defaults to 0xffffffff, posU to 0. */
void oracle_bound_inf_dist_forward(const float *xl, const float *xu, const float *w,
                                   int B, int CO, int CI, float *yl, float *yu,
                                   int32_t *posl, int32_t *posu) {
#pragma omp parallel
    {
        float *l = (float *)malloc(sizeof(float) * CI);
        float *u = (float *)malloc(sizeof(float) * CI);
#pragma omp for schedule(static)
        for (int b = 0; b < B; b++) {
            for (int c = 0; c < CI; c++) {
                float a = xl[(size_t)b * CI + c], d = xu[(size_t)b * CI + c];
                if (a > d) { float m = (a + d) * 0.5f; a = m; d = m; }
                l[c] = a; u[c] = d;
            }
            for (int j = 0; j < CO; j++) {
                const float *wj = w + (size_t)j * CI;
                float accl = -ORACLE_EPS, accu = ORACLE_EPS;
                uint32_t pl = NO_GRAD_ID, pu = 0;
                for (int c = 0; c < CI; c++) {
                    float t1 = wj[c] - l[c], t2 = u[c] - wj[c];
                    float lo = fminf(t1, t2), hi = fmaxf(t1, t2);
                    uint32_t p = (uint32_t)c | (t1 <= t2 ? 0u : SIGN_BIT);
                    if (lo < accl) { accl = lo; pl = p; }
                    if (hi > accu) { accu = hi; pu = p; }
                }
                yl[(size_t)b * CO + j] = -accl;
                yu[(size_t)b * CO + j] = accu;
                if (posl) posl[(size_t)b * CO + j] = (int32_t)pl;
                if (posu) posu[(size_t)b * CO + j] = (int32_t)pu;
            }
        }
        free(l);
        free(u);
    }
}

/* Interval-bound sparse backward.  bound_inf_dist_cuda.cu:240-299: the lower-bound
 * gradient goes to grad_xL (+g) when the sign bit is clear, else to grad_xU (-g), and is
 * skipped when posL == 0xffffffff; the upper-bound gradient goes to grad_xU (+g) when
 * clear, else to grad_xL (-g); grad_w receives the negated values.  gw may be NULL. */
void oracle_bound_inf_dist_backward(const float *gl, const float *gu, const int32_t *posl,
                                    const int32_t *posu, int B, int CO, int CI,
                                    float *gxl, float *gxu, float *gw) {
    double *al = (double *)calloc((size_t)B * CI, sizeof(double));
    double *au = (double *)calloc((size_t)B * CI, sizeof(double));
    double *aw = gw ? (double *)calloc((size_t)CO * CI, sizeof(double)) : NULL;
    for (int b = 0; b < B; b++) {
        for (int j = 0; j < CO; j++) {
            size_t o = (size_t)b * CO + j;
            uint32_t pl = (uint32_t)posl[o], pu = (uint32_t)posu[o];
            int il = (int)(pl & ~SIGN_BIT), iu = (int)(pu & ~SIGN_BIT);
            float vl = (pl & SIGN_BIT) ? -gl[o] : gl[o];
            float vu = (pu & SIGN_BIT) ? -gu[o] : gu[o];
            if (pl != NO_GRAD_ID) {
                ((pl & SIGN_BIT) ? au : al)[(size_t)b * CI + il] += vl;
                if (aw) aw[(size_t)j * CI + il] -= vl;
            }
            ((pu & SIGN_BIT) ? al : au)[(size_t)b * CI + iu] += vu;
            if (aw) aw[(size_t)j * CI + iu] -= vu;
        }
    }
    for (size_t i = 0; i < (size_t)B * CI; i++) { gxl[i] = (float)al[i]; gxu[i] = (float)au[i]; }
    if (aw) for (size_t i = 0; i < (size_t)CO * CI; i++) gw[i] = (float)aw[i];
    free(al);
    free(au);
    free(aw);
}

/* l-p forward in exact (double) math on the fp32 differences.
 * p <= 10 (norm_dist.cpp:51-55, norm_dist_cuda.cu:238,253): y = max(sum |t|^p, FLT_MIN)^(1/p).
 * p  > 10 (norm_dist.cpp:56-60, norm_dist_cuda.cu:61-71,119-129,154):
 *   y = M * (sum (|t|/M)^p + (EPS/M)^p)^(1/p),  M = max(EPS, max |t|)
 * (the reference reaches this with an online running max; this is its exact-math value). */
void oracle_norm_dist_forward(const float *x, const float *w, int B, int CO, int CI,
                              double p, double *y, const int *ci, const int *co, int W_CI) {
#pragma omp parallel for schedule(static)
    for (int b = 0; b < B; b++) {
        int s = b / SUB_BATCH;
        const float *xb = x + (size_t)b * CI;
        for (int j = 0; j < CO; j++) {
            const float *wj = w_row(w, co, s, CO, W_CI, j);
            double res;
            if (p <= 10.0) {
                double acc = 0;
                for (int c = 0; c < CI; c++) {
                    float t = xb[c] - wj[w_col(ci, s, CI, c)];
                    acc += pow(fabs((double)t), p);
                }
                if (acc < (double)FLT_MIN) acc = (double)FLT_MIN;
                res = pow(acc, 1.0 / p);
            } else {
                double m = (double)ORACLE_EPS;
                for (int c = 0; c < CI; c++) {
                    float t = xb[c] - wj[w_col(ci, s, CI, c)];
                    double a = fabs((double)t);
                    if (a > m) m = a;
                }
                double acc = pow((double)ORACLE_EPS / m, p);
                for (int c = 0; c < CI; c++) {
                    float t = xb[c] - wj[w_col(ci, s, CI, c)];
                    acc += pow(fabs((double)t) / m, p);
                }
                res = m * pow(acc, 1.0 / p);
            }
            y[(size_t)b * CO + j] = res;
        }
    }
}

/* l-p dense backward in double.  norm_dist_cuda.cu:261-266,295,349:
 * term = g[b,j] * sgn(t) * (|t| / y[b,j])^(p-1); grad_x[b,c] = sum_j term;
 * grad_w[co[s][j], ci[s][c]] = -sum_b term.  y is the forward output handed back by the
 * caller (fp32 in the product, promoted here).  gw may be NULL. */
void oracle_norm_dist_backward(const float *g, const float *x, const float *w, const float *y,
                               int B, int CO, int CI, double p, double *gx, double *gw,
                               const int *ci, const int *co, int W_CO, int W_CI) {
    memset(gx, 0, sizeof(double) * (size_t)B * CI);
    if (gw) memset(gw, 0, sizeof(double) * (size_t)W_CO * W_CI);
    /* Sub-batches one after the other; inside one, threads take different outputs j.  The kept
     * rows of a sub-batch are distinct, so no two threads touch the same row of gw; grad_x is
     * summed per thread and merged at the end of the sub-batch. */
    int S = (B + SUB_BATCH - 1) / SUB_BATCH;
    for (int s = 0; s < S; s++) {
        int b0 = s * SUB_BATCH, b1 = b0 + SUB_BATCH < B ? b0 + SUB_BATCH : B;
#pragma omp parallel
        {
            double *loc = (double *)calloc((size_t)(b1 - b0) * CI, sizeof(double));
#pragma omp for schedule(static)
            for (int j = 0; j < CO; j++) {
                int row = co ? co[(size_t)s * CO + j] : j;
                const float *wj = w + (size_t)row * W_CI;
                for (int b = b0; b < b1; b++) {
                    const float *xb = x + (size_t)b * CI;
                    double gv = g[(size_t)b * CO + j];
                    double ry = 1.0 / (double)y[(size_t)b * CO + j];
                    double *lb = loc + (size_t)(b - b0) * CI;
                    for (int c = 0; c < CI; c++) {
                        int col = w_col(ci, s, CI, c);
                        float t = xb[c] - wj[col];
                        double term = gv * pow(fabs((double)t) * ry, p - 1.0);
                        if (t < 0) term = -term;
                        lb[c] += term;
                        if (gw) gw[(size_t)row * W_CI + col] -= term;
                    }
                }
            }
#pragma omp critical
            for (size_t i = 0; i < (size_t)(b1 - b0) * CI; i++) gx[(size_t)b0 * CI + i] += loc[i];
            free(loc);
        }
    }
}

/* Geometric weights of the sort neuron: rank r (0 = largest) gets q (1-q)^r, the sum is divided
 * by 1 - (1-q)^K.  sort_neuron.cu:91-97 evaluates it in fp32 as below (no contraction here). */
static float sort_combine(const float *res /* ascending, res[K-1] largest */, int K, float q, float eps0) {
    float ans = eps0, c = 1.0f;
    for (int k = K - 1; k >= 0; k--) {
        ans += res[k] * c * q;
        c *= 1 - q;
    }
    return ans / (1 - c);
}

/* Sort neuron forward.  sort_neuron.cu:16-102 (values: K-slot min/max insertion chain from
 * zeros) and :115-214 (positions: a value enters only if it exceeds the smallest slot; it
 * moves up past every slot it is >= to, so of equal values the later index ranks higher; slots
 * never filled keep value 0 / word 0).  pos is [K][B][CO], rank 0 = largest; may be NULL. */
void oracle_sort_forward(const float *x, const float *w, int B, int CO, int CI, float q, int K,
                         float *y, int32_t *pos) {
#pragma omp parallel for schedule(static)
    for (int b = 0; b < B; b++) {
        float res[32];
        uint32_t idx[32];
        for (int j = 0; j < CO; j++) {
            for (int k = 0; k < K; k++) { res[k] = 0.f; idx[k] = 0; }
            for (int c = 0; c < CI; c++) {
                float t = x[(size_t)b * CI + c] - w[(size_t)j * CI + c];
                float v = fabsf(t);
                if (v > res[0]) {
                    uint32_t word = (uint32_t)c | (t >= 0 ? 0u : SIGN_BIT);
                    int k = 0;
                    for (; k < K - 1; k++) {
                        if (v < res[k + 1]) { res[k] = v; idx[k] = word; break; }
                        res[k] = res[k + 1];
                        idx[k] = idx[k + 1];
                    }
                    if (k == K - 1) { res[k] = v; idx[k] = word; }
                }
            }
            y[(size_t)b * CO + j] = sort_combine(res, K, q, ORACLE_EPS);
            if (pos)
                for (int k = K - 1; k >= 0; k--)
                    pos[(size_t)(K - 1 - k) * B * CO + (size_t)b * CO + j] = (int32_t)idx[k];
        }
    }
}

/* Interval bounds of the sort neuron.  sort_neuron.cu:216-314: bottom-K of min(t1, t2) and top-K of
 * max(t1, t2) (t1 = w - xL, t2 = xU - w, inverted intervals repaired to the midpoint), both
 * chains from zeros; yL = -(-EPS + sum)/(1 - (1-q)^K), yU = (EPS + sum)/(1 - (1-q)^K). */
void oracle_sort_bound_forward(const float *xl, const float *xu, const float *w, int B, int CO,
                               int CI, float q, int K, float *yl, float *yu) {
#pragma omp parallel for schedule(static)
    for (int b = 0; b < B; b++) {
        float rl[32], ru[32];
        for (int j = 0; j < CO; j++) {
            for (int k = 0; k < K; k++) { rl[k] = 0.f; ru[k] = 0.f; }
            for (int c = 0; c < CI; c++) {
                float a = xl[(size_t)b * CI + c], d = xu[(size_t)b * CI + c];
                if (a > d) { float m = (a + d) * 0.5f; a = m; d = m; }
                float t1 = w[(size_t)j * CI + c] - a, t2 = d - w[(size_t)j * CI + c];
                float vl = fminf(t1, t2), vu = fmaxf(t1, t2);
                for (int k = 0; k < K - 1; k++) {
                    rl[k] = fminf(rl[k], fmaxf(rl[k + 1], vl));
                    ru[k] = fmaxf(ru[k], fminf(ru[k + 1], vu));
                }
                rl[K - 1] = fminf(rl[K - 1], vl);
                ru[K - 1] = fmaxf(ru[K - 1], vu);
            }
            yl[(size_t)b * CO + j] = -sort_combine(rl, K, q, -ORACLE_EPS);
            yu[(size_t)b * CO + j] = sort_combine(ru, K, q, ORACLE_EPS);
        }
    }
}

/* Sort neuron sparse backward.  sort_neuron.cu:316-375: rank r contributes
 * (+/-) g * q (1-q)^r / (1 - (1-q)^K) to grad_x[b, idx_r] and its negation to grad_w[j, idx_r].
 * Sums in double, rounded once.  gw may be NULL. */
void oracle_sort_backward(const float *g, const int32_t *pos, int B, int CO, int CI, float q, int K,
                          float *gx, float *gw) {
    double *ax = (double *)calloc((size_t)B * CI, sizeof(double));
    double *aw = gw ? (double *)calloc((size_t)CO * CI, sizeof(double)) : NULL;
    float n = powf(1 - q, (float)K);
    n = 1.0f + n / (1.0f - n);
    for (int b = 0; b < B; b++)
        for (int j = 0; j < CO; j++) {
            float grad = g[(size_t)b * CO + j], c = n;
            for (int k = 0; k < K; k++) {
                uint32_t p = (uint32_t)pos[(size_t)k * B * CO + (size_t)b * CO + j];
                int idx = (int)(p & ~SIGN_BIT);
                float v = ((p & SIGN_BIT) ? -grad : grad) * c * q;
                ax[(size_t)b * CI + idx] += v;
                if (aw) aw[(size_t)j * CI + idx] -= v;
                c *= 1 - q;
            }
        }
    for (size_t i = 0; i < (size_t)B * CI; i++) gx[i] = (float)ax[i];
    if (aw) for (size_t i = 0; i < (size_t)CO * CI; i++) gw[i] = (float)aw[i];
    free(ax);
    free(aw);
}
