/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the L_p-distance operator family of
 * zbh2047/L_inf-dist-net-v2.  It is the checker for the CUDA kernels of this repository
 * (tests, the smoke check, and the CPU-baseline leg of the benchmark) and is never part of
 * the product path.
 *
 * Parity status: pinned.  tests/golden/ holds vectors produced by the reference's own
 * pure-torch implementation (core/norm_dist.py:99-103 and :112-120) and this file is
 * checked against them by tests/test_oracle_golden.py.
 *
 * Layouts (all contiguous, fp32 unless noted), as in core/cuda/norm_dist_cuda.cu:72,84,143:
 *   x[B, CI, HW]   element ((b*G + g)*CIg + c)*HW + hw
 *   w[CO, CIg]     element (g*COg + o)*CIg + c
 *   y[B, CO, HW]   element ((b*G + g)*COg + o)*HW + hw
 * with CIg = CI/G, COg = CO/G.  pos arrays are int32 with the layout of y: bit 31 is a
 * flag, bits 0..30 a channel index inside the group.
 *
 * Arithmetic: the difference t = x - w is taken in fp32 exactly as every implementation
 * does; sums and powers are carried in double so that the result is the correctly rounded
 * target the fp32 kernels are compared against with a tolerance.  The p = inf and bound
 * functions use only fp32 subtract / min / max, which are exact, so they are bit-exact
 * targets (values and indices).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define LDN_EPS 1e-10f                 /* core/cuda/norm_dist_cuda.cu:13, inf_dist_cuda.cu:11 */
#define LDN_UNDERFLOW 1.175494351e-38f /* core/cuda/norm_dist_cuda.cu:15 */
#define LDN_MIN_NORMALIZED_P 10.0f     /* core/cuda/norm_dist.cpp:4 */
#define LDN_NO_GRAD_ID ((int32_t)0xffffffff) /* core/cuda/bound_inf_dist_cuda.cu:12 */
#define LDN_SIGN ((int32_t)0x80000000)

static inline size_t x_off(int b, int g, int c, int hw, int G, int CIg, int HW) {
    return (((size_t)b * G + g) * CIg + c) * HW + hw;
}
static inline size_t w_off(int g, int o, int c, int COg, int CIg) {
    return ((size_t)g * COg + o) * CIg + c;
}
static inline size_t y_off(int b, int g, int o, int hw, int G, int COg, int HW) {
    return (((size_t)b * G + g) * COg + o) * HW + hw;
}

/* |t|^p for t given in fp32; integer p by repeated multiplication (core/cuda/fast_pow.cuh:4-12). */
static inline double abs_pow(float t, double p, int ip) {
    double a = fabs((double)t);
    if (ip >= 0) {
        double r = 1.0;
        for (int k = 0; k < ip; k++) r *= a;
        return r;
    }
    return pow(a, p);
}

/* integer template value used by the reference dispatch (core/cuda/norm_dist.cpp:17-35) */
static inline int int_power_or_neg1(float p) {
    if (p == (float)(int)p && (int)p >= 0 && (int)p <= 8) return (int)p;
    return -1;
}

/*
 * Finite-p forward.  core/cuda/norm_dist.cpp:40-53 picks the algorithm:
 *   p <= 10: y = (max(sum_i |t|^p, 1.175494351e-38))^(1/p)        norm_dist_cuda.cu:151-236 (has_max = false)
 *   p  > 10: y = M * (sum_i (|t|/M)^p + (1e-10/M)^p)^(1/p), M = max(1e-10, max_i |t|)
 *            (the closed form of the online rescaling of norm_dist_cuda.cu:35-148)
 */
void ldn_oracle_norm_dist_forward(const float* x, const float* w, float* y,
                                  int B, int CO, int CI, int G, int HW, float p) {
    const int CIg = CI / G, COg = CO / G;
    const int ip = int_power_or_neg1(p);
    const long long rows = (long long)B * G * COg;
#pragma omp parallel for schedule(static)
    for (long long r = 0; r < rows; r++) {
        int o = (int)(r % COg);
        int g = (int)((r / COg) % G);
        int b = (int)(r / ((long long)COg * G));
        for (int hw = 0; hw < HW; hw++) {
            double res;
            if (p <= LDN_MIN_NORMALIZED_P) {
                double s = 0.0;
                for (int c = 0; c < CIg; c++) {
                    float t = x[x_off(b, g, c, hw, G, CIg, HW)] - w[w_off(g, o, c, COg, CIg)];
                    s += abs_pow(t, p, ip);
                }
                if (s < (double)LDN_UNDERFLOW) s = (double)LDN_UNDERFLOW;
                res = pow(s, 1.0 / (double)p);
            } else {
                float M = LDN_EPS;
                for (int c = 0; c < CIg; c++) {
                    float t = x[x_off(b, g, c, hw, G, CIg, HW)] - w[w_off(g, o, c, COg, CIg)];
                    float a = fabsf(t);
                    if (a > M) M = a;
                }
                double s = pow((double)LDN_EPS / (double)M, (double)p);
                for (int c = 0; c < CIg; c++) {
                    float t = x[x_off(b, g, c, hw, G, CIg, HW)] - w[w_off(g, o, c, COg, CIg)];
                    s += pow(fabs((double)t) / (double)M, (double)p);
                }
                res = (double)M * pow(s, 1.0 / (double)p);
            }
            y[y_off(b, g, o, hw, G, COg, HW)] = (float)res;
        }
    }
}

/*
 * Forward normalised by a caller-supplied per-output maximum (core/cuda/norm_dist.cpp:55-64,
 * norm_dist_cuda.cu:151-236 with has_max = true):
 *   r = 1/max;  y = (sum_i (|t| r)^p + (1e-10 r)^p)^(1/p) / r
 */
void ldn_oracle_norm_dist_forward_with_max(const float* x, const float* w, const float* mx, float* y,
                                           int B, int CO, int CI, int G, int HW, float p) {
    const int CIg = CI / G, COg = CO / G;
    const long long rows = (long long)B * G * COg;
#pragma omp parallel for schedule(static)
    for (long long r = 0; r < rows; r++) {
        int o = (int)(r % COg);
        int g = (int)((r / COg) % G);
        int b = (int)(r / ((long long)COg * G));
        for (int hw = 0; hw < HW; hw++) {
            size_t yo = y_off(b, g, o, hw, G, COg, HW);
            double rm = 1.0 / (double)mx[yo];
            double s = pow((double)LDN_EPS * rm, (double)p);
            for (int c = 0; c < CIg; c++) {
                float t = x[x_off(b, g, c, hw, G, CIg, HW)] - w[w_off(g, o, c, COg, CIg)];
                s += pow(fabs((double)t) * rm, (double)p);
            }
            y[yo] = (float)(pow(s, 1.0 / (double)p) / rm);
        }
    }
}

/*
 * One backward term (core/cuda/norm_dist_cuda.cu:238-243), q = p - 1:
 *   term = g * sgn(t) * (|t| / y)^q,  sgn(t) = +1 for t >= 0 else -1
 */
static inline double bwd_term(float t, double rinv, double gval, double q, int iq) {
    double a = fabs((double)t) * rinv;
    double pw;
    if (iq >= 0) {
        pw = 1.0;
        for (int k = 0; k < iq; k++) pw *= a;
    } else {
        pw = pow(a, q);
    }
    return (t >= 0.0f ? gval : -gval) * pw;
}

/*
 * Finite-p backward (core/cuda/norm_dist.cpp:66-91):
 *   gx[b,c] = sum_o term,  gw[o,c] = -sum_b,hw term.
 * Either output pointer may be NULL.  The template integer of the reference is p - 1
 * (norm_dist.cpp:74,88).
 */
void ldn_oracle_norm_dist_backward(const float* go, const float* x, const float* w, const float* y,
                                   float* gx, float* gw,
                                   int B, int CO, int CI, int G, int HW, float p) {
    const int CIg = CI / G, COg = CO / G;
    const double q = (double)p - 1.0;
    const float qf = p - 1.0f;
    const int iq = int_power_or_neg1(qf);
    if (gx) {
        const long long rows = (long long)B * G;
#pragma omp parallel
        {
            double* acc = (double*)malloc(sizeof(double) * (size_t)CIg);
#pragma omp for schedule(static)
            for (long long r = 0; r < rows; r++) {
                int g = (int)(r % G);
                int b = (int)(r / G);
                for (int hw = 0; hw < HW; hw++) {
                    memset(acc, 0, sizeof(double) * (size_t)CIg);
                    for (int o = 0; o < COg; o++) {
                        size_t yo = y_off(b, g, o, hw, G, COg, HW);
                        double rinv = 1.0 / (double)y[yo];
                        double gval = (double)go[yo];
                        const float* wr = w + w_off(g, o, 0, COg, CIg);
                        for (int c = 0; c < CIg; c++) {
                            float t = x[x_off(b, g, c, hw, G, CIg, HW)] - wr[c];
                            acc[c] += bwd_term(t, rinv, gval, q, iq);
                        }
                    }
                    for (int c = 0; c < CIg; c++) gx[x_off(b, g, c, hw, G, CIg, HW)] = (float)acc[c];
                }
            }
            free(acc);
        }
    }
    if (gw) {
        const long long rows = (long long)G * COg;
#pragma omp parallel
        {
            double* acc = (double*)malloc(sizeof(double) * (size_t)CIg);
#pragma omp for schedule(static)
            for (long long r = 0; r < rows; r++) {
                int o = (int)(r % COg);
                int g = (int)(r / COg);
                memset(acc, 0, sizeof(double) * (size_t)CIg);
                const float* wr = w + w_off(g, o, 0, COg, CIg);
                for (int b = 0; b < B; b++) {
                    for (int hw = 0; hw < HW; hw++) {
                        size_t yo = y_off(b, g, o, hw, G, COg, HW);
                        double rinv = 1.0 / (double)y[yo];
                        double gval = (double)go[yo];
                        for (int c = 0; c < CIg; c++) {
                            float t = x[x_off(b, g, c, hw, G, CIg, HW)] - wr[c];
                            acc[c] -= bwd_term(t, rinv, gval, q, iq);
                        }
                    }
                }
                for (int c = 0; c < CIg; c++) gw[w_off(g, o, c, COg, CIg)] = (float)acc[c];
            }
            free(acc);
        }
    }
}

/*
 * p = inf forward (core/cuda/inf_dist_cuda.cu:106-198; no-grad variant :14-103 gives the same value):
 *   y = max(1e-10, max_i |t|);  pos = first index whose |t| strictly exceeds the running
 *   maximum (scan in ascending channel order, start value 1e-10, start pos 0), with bit 31
 *   set when t < 0.  pos may be NULL.
 */
void ldn_oracle_inf_dist_forward(const float* x, const float* w, float* y, int32_t* pos,
                                 int B, int CO, int CI, int G, int HW) {
    const int CIg = CI / G, COg = CO / G;
    const long long rows = (long long)B * G * COg;
#pragma omp parallel for schedule(static)
    for (long long r = 0; r < rows; r++) {
        int o = (int)(r % COg);
        int g = (int)((r / COg) % G);
        int b = (int)(r / ((long long)COg * G));
        for (int hw = 0; hw < HW; hw++) {
            float m = LDN_EPS;
            int32_t ps = 0;
            for (int c = 0; c < CIg; c++) {
                float t = x[x_off(b, g, c, hw, G, CIg, HW)] - w[w_off(g, o, c, COg, CIg)];
                float a = fabsf(t);
                if (a > m) {
                    m = a;
                    ps = (int32_t)c | (t >= 0.0f ? 0 : LDN_SIGN);
                }
            }
            size_t yo = y_off(b, g, o, hw, G, COg, HW);
            y[yo] = m;
            if (pos) pos[yo] = ps;
        }
    }
}

/*
 * p = inf backward (core/cuda/inf_dist_cuda.cu:200-246): v = pos >= 0 ? g : -g, idx = pos & 0x7fffffff;
 *   gx[b, idx] += v;  gw[o, idx] -= v.   Sums are carried in double, in a fixed order; gw may be NULL.
 */
void ldn_oracle_inf_dist_backward(const float* go, const int32_t* pos, float* gx, float* gw,
                                  int B, int CO, int CI, int G, int HW) {
    const int CIg = CI / G, COg = CO / G;
    size_t nx = (size_t)B * CI * HW, nw = (size_t)CO * CIg;
    double* ax = (double*)calloc(nx, sizeof(double));
    double* aw = gw ? (double*)calloc(nw, sizeof(double)) : NULL;
    for (int b = 0; b < B; b++)
        for (int g = 0; g < G; g++)
            for (int o = 0; o < COg; o++)
                for (int hw = 0; hw < HW; hw++) {
                    size_t yo = y_off(b, g, o, hw, G, COg, HW);
                    int32_t ps = pos[yo];
                    int idx = (int)(ps & 0x7fffffff);
                    double v = ps >= 0 ? (double)go[yo] : -(double)go[yo];
                    ax[x_off(b, g, idx, hw, G, CIg, HW)] += v;
                    if (aw) aw[w_off(g, o, idx, COg, CIg)] -= v;
                }
    for (size_t i = 0; i < nx; i++) gx[i] = (float)ax[i];
    if (gw) for (size_t i = 0; i < nw; i++) gw[i] = (float)aw[i];
    free(ax);
    free(aw);
}

/*
 * Interval bound forward for p = inf (core/cuda/bound_inf_dist_cuda.cu:15-118 and :121-238).
 * With t1 = w - xL, t2 = xU - w (inputs with xL > xU first collapsed to their midpoint, :63,172):
 *   yL = -min(-1e-10, min_i min(t1,t2)),  yU = max(1e-10, max_i max(t1,t2)).
 * posL starts at 0xffffffff ("no gradient") and posU at 0; both take index | flag on a strict
 * improvement, flag = (t1 <= t2 ? 0 : bit 31).  posL/posU may be NULL.
 */
void ldn_oracle_bound_inf_dist_forward(const float* xL, const float* xU, const float* w,
                                       float* yL, float* yU, int32_t* posL, int32_t* posU,
                                       int B, int CO, int CI, int G, int HW) {
    const int CIg = CI / G, COg = CO / G;
    const long long rows = (long long)B * G * COg;
#pragma omp parallel for schedule(static)
    for (long long r = 0; r < rows; r++) {
        int o = (int)(r % COg);
        int g = (int)((r / COg) % G);
        int b = (int)(r / ((long long)COg * G));
        for (int hw = 0; hw < HW; hw++) {
            float mn = -LDN_EPS, mx = LDN_EPS;
            int32_t pl = LDN_NO_GRAD_ID, pu = 0;
            for (int c = 0; c < CIg; c++) {
                size_t xo = x_off(b, g, c, hw, G, CIg, HW);
                float lo = xL[xo], up = xU[xo];
                if (lo > up) lo = up = (lo + up) * 0.5f;
                float wv = w[w_off(g, o, c, COg, CIg)];
                float t1 = wv - lo, t2 = up - wv;
                float a = fminf(t1, t2), bb = fmaxf(t1, t2);
                int32_t ps = (int32_t)c | (t1 <= t2 ? 0 : LDN_SIGN);
                if (a < mn) { mn = a; pl = ps; }
                if (bb > mx) { mx = bb; pu = ps; }
            }
            size_t yo = y_off(b, g, o, hw, G, COg, HW);
            yL[yo] = -mn;
            yU[yo] = mx;
            if (posL) posL[yo] = pl;
            if (posU) posU[yo] = pu;
        }
    }
}

/*
 * Interval bound backward (core/cuda/bound_inf_dist_cuda.cu:240-299).  For the lower bound
 * (skipped when posL is 0xffffffff): flag clear -> gxL[idx] += gL else gxU[idx] -= gL; the weight
 * receives the negated value.  For the upper bound: flag clear -> gxU[idx] += gU else
 * gxL[idx] -= gU; weight again negated.  gw may be NULL.
 */
void ldn_oracle_bound_inf_dist_backward(const float* goL, const float* goU,
                                        const int32_t* posL, const int32_t* posU,
                                        float* gxL, float* gxU, float* gw,
                                        int B, int CO, int CI, int G, int HW) {
    const int CIg = CI / G, COg = CO / G;
    size_t nx = (size_t)B * CI * HW, nw = (size_t)CO * CIg;
    double* aL = (double*)calloc(nx, sizeof(double));
    double* aU = (double*)calloc(nx, sizeof(double));
    double* aw = gw ? (double*)calloc(nw, sizeof(double)) : NULL;
    for (int b = 0; b < B; b++)
        for (int g = 0; g < G; g++)
            for (int o = 0; o < COg; o++)
                for (int hw = 0; hw < HW; hw++) {
                    size_t yo = y_off(b, g, o, hw, G, COg, HW);
                    int32_t pl = posL[yo], pu = posU[yo];
                    int il = (int)(pl & 0x7fffffff), iu = (int)(pu & 0x7fffffff);
                    double vl = pl >= 0 ? (double)goL[yo] : -(double)goL[yo];
                    double vu = pu >= 0 ? (double)goU[yo] : -(double)goU[yo];
                    if (pl != LDN_NO_GRAD_ID) {
                        double* dst = pl >= 0 ? aL : aU;
                        dst[x_off(b, g, il, hw, G, CIg, HW)] += vl;
                        if (aw) aw[w_off(g, o, il, COg, CIg)] -= vl;
                    }
                    double* dst = pu >= 0 ? aU : aL;
                    dst[x_off(b, g, iu, hw, G, CIg, HW)] += vu;
                    if (aw) aw[w_off(g, o, iu, COg, CIg)] -= vu;
                }
    for (size_t i = 0; i < nx; i++) { gxL[i] = (float)aL[i]; gxU[i] = (float)aU[i]; }
    if (gw) for (size_t i = 0; i < nw; i++) gw[i] = (float)aw[i];
    free(aL);
    free(aU);
    free(aw);
}

int ldn_oracle_num_threads(void) {
    int n = 1;
#ifdef _OPENMP
#pragma omp parallel
    {
#pragma omp single
        n = omp_get_num_threads();
    }
#endif
    return n;
}
