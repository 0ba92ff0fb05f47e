/*
 * CPU oracle of the multi-head Flow-Lenia neural-CA step and of its fitness reduction.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared with; nothing in the
 * product library calls, links or loads it.  It is compiled twice by the Makefile beside it:
 *   libca_oracle_f64.so  (-DORACLE_REAL=double)  every intermediate in fp64: the truth used by tests;
 *   libca_oracle_f32.so  (-DORACLE_REAL=float)   fp32 intermediates, fp64 reductions: the timed CPU
 *                                                transcription of the step (multithreaded, OpenMP).
 *
 * PARITY UNPINNED BY THE REFERENCE: J0pari/Slime ships no golden vector, known-answer test or fixture
 * for this path, has no CPU implementation, and its live CUDA step is racy and mis-indexed
 * (slime/core/organism.cu:617-688 launches the child sequence from 128 threads at once;
 * slime/core/pseudopod.cu:54 visits only the diagonal tiles), so it cannot produce reference outputs.
 * The oracle is pinned instead against an independently written numpy restatement
 * (tests/golden/make_golden.py) and against the invariants the reference's own documents state
 * (per-channel mass, buildplan.md:179; rank range, effective_rank tests recorded in .test_checkpoints).
 *
 * The step, stage by stage, with the reference lines each stage follows (paths inside J0pari/Slime):
 *   1 projections   P_h = X Wp_h, I_h = X Wi_h, V_h = X Wv_h   weight order [head][c_in][d_out]
 *                   slime/core/pseudopod.cu:78-120 (index order :86-87), buildplan.md:572-592
 *   2 stencil       U_h(y,x,d) = sum_t K_h[t] P_h(y+dy,x+dx,d), t=(dy+1)*3+(dx+1), torus
 *                   slime/core/pseudopod.cu:153,172-180 (tap order), slime/kernels/warp_ca.cu:305-306 (wrap)
 *   3 growth        G = 2 exp(-(U-mu)^2 / (2 sigma^2)) - 1
 *                   failed_attempts/warp_ca.cu:49-56, failed_attempts/pseudopod.cu:46-48
 *   4 activation    A = clamp(G * I, -80, 80)                  README.md:42-45; the clamp is this step's
 *                   domain limit: stages 5-6 are also evaluated in their closed form exp(A) / box3(exp(A)),
 *                   which has no max-subtraction, and exp(80) keeps nine-term sums finite in fp32.  Inside
 *                   |G I| <= 80 the clamp does nothing.  ORACLE_ACT_CLAMP below; oracle_set_activation_clamp().
 *   5 flow weights  source s sends to n in N(s) the share softmax_n(A(n)), max-subtracted
 *                   failed_attempts/pseudopod.cu:234-251, buildplan.md:608-622
 *   6 propagation   V'(n) = sum_{s in N(n)} w(s->n) V(s)        README.md:45-47 (sum out = sum in)
 *   7 output proj   Y = concat_h(V'_h) Wo                      slime/core/pseudopod.cu:217-253
 *   8 residual      X+ = X + dt Y, dt = 0.1                    slime/core/pseudopod.cu:186-187, organism.cu:659
 *   9 renorm        X+[:,:,c] *= M_c / sum_cells X+[:,:,c]     failed_attempts/warp_ca.cu:401-450
 * Fitness: Gram of each head's V' (64x64 over cells), cyclic two-sided Jacobi, exp-entropy rank, Pearson
 * coherence of V' between the last two steps, fitness = rank x coherence, hunger = 1 - coherence
 *   failed_attempts/pseudopod.cu:366-432, slime/kernels/warp_ca.cu:51-63,107-144,219,238.
 */
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifndef ORACLE_REAL
#define ORACLE_REAL double
#endif
typedef ORACLE_REAL real;

#define NH 8   /* heads            slime/core/pseudopod.cu:15 */
#define HD 64  /* head dim         slime/core/pseudopod.cu:16 */
#define NC 64  /* state channels                              */
#define HC (NH * HD)

/* Bound on |A| (stage 4).  Part of the step's definition; the CUDA kernels use the same constant. */
static double g_act_clamp = 80.0;
double oracle_set_activation_clamp(double c) { const double old = g_act_clamp; if (c > 0) g_act_clamp = c; return old; }

static inline real r_exp(real x) { return sizeof(real) == 4 ? (real)expf((float)x) : (real)exp((double)x); }

static inline int wrap(int i, int n) { i %= n; return i < 0 ? i + n : i; }

/* One weight set, host fp32, in the reference's index order. */
typedef struct {
    const float* Wp;    /* [8][64][64]  [head][c_in][d_out] */
    const float* Wi;    /* [8][64][64] */
    const float* Wv;    /* [8][64][64] */
    const float* Wo;    /* [512][64]    [head*64+d][c_out]  */
    const float* K;     /* [8][9]       taps t=(dy+1)*3+(dx+1), already softmax-normalised */
    const float* mu;    /* [8] */
    const float* sigma; /* [8] */
} weight_set;

int oracle_real_bytes(void) { return (int)sizeof(real); }

/* ---- stage 1: projections for one head over one grid (cells x 64 -> cells x 64, three times) ---- */
static void project_head(const float* X, int cells, const weight_set* w, int h, real* P, real* I, real* V) {
    const float* wp = w->Wp + (size_t)h * NC * HD;
    const float* wi = w->Wi + (size_t)h * NC * HD;
    const float* wv = w->Wv + (size_t)h * NC * HD;
#pragma omp parallel for schedule(static)
    for (int s = 0; s < cells; ++s) {
        real ap[HD], ai[HD], av[HD];
        for (int d = 0; d < HD; ++d) ap[d] = ai[d] = av[d] = 0;
        const float* x = X + (size_t)s * NC;
        for (int c = 0; c < NC; ++c) {
            real xc = (real)x[c];
            const float* rp = wp + c * HD;
            const float* ri = wi + c * HD;
            const float* rv = wv + c * HD;
            for (int d = 0; d < HD; ++d) {
                ap[d] += xc * (real)rp[d];
                ai[d] += xc * (real)ri[d];
                av[d] += xc * (real)rv[d];
            }
        }
        memcpy(P + (size_t)s * HD, ap, sizeof ap);
        memcpy(I + (size_t)s * HD, ai, sizeof ai);
        memcpy(V + (size_t)s * HD, av, sizeof av);
    }
}

/* ---- stages 2-4: stencil on P, growth, activation; result A (overwrites nothing it reads) ---- */
static void activation_head(const real* P, const real* I, int H, int W, const weight_set* w, int h, real* A) {
    const float* k = w->K + h * 9;
    const real mu = (real)w->mu[h];
    const real sg = (real)w->sigma[h];
    const real inv2s2 = (real)1 / ((real)2 * sg * sg);
    const real clampv = (real)g_act_clamp;
#pragma omp parallel for schedule(static)
    for (int y = 0; y < H; ++y) {
        for (int x = 0; x < W; ++x) {
            real u[HD];
            for (int d = 0; d < HD; ++d) u[d] = 0;
            for (int dy = -1; dy <= 1; ++dy)
                for (int dx = -1; dx <= 1; ++dx) {
                    const real kt = (real)k[(dy + 1) * 3 + (dx + 1)];
                    const real* p = P + ((size_t)wrap(y + dy, H) * W + wrap(x + dx, W)) * HD;
                    for (int d = 0; d < HD; ++d) u[d] += kt * p[d];
                }
            const size_t o = ((size_t)y * W + x) * HD;
            for (int d = 0; d < HD; ++d) {
                const real z = u[d] - mu;
                const real g = (real)2 * r_exp(-(z * z) * inv2s2) - (real)1;
                real a = g * I[o + d];
                if (a > clampv) a = clampv;
                if (a < -clampv) a = -clampv;
                A[o + d] = a;
            }
        }
    }
}

/* ---- stages 5-6, literal form: per-source max-subtracted softmax over its 3x3 targets, then gather ---- */
static void redistribute_literal(const real* A, const real* V, int H, int W, real* mx, real* den, real* Vp) {
#pragma omp parallel for schedule(static)
    for (int y = 0; y < H; ++y)
        for (int x = 0; x < W; ++x) {
            const size_t o = ((size_t)y * W + x) * HD;
            for (int d = 0; d < HD; ++d) {
                real m = -INFINITY;
                for (int dy = -1; dy <= 1; ++dy)
                    for (int dx = -1; dx <= 1; ++dx) {
                        const real a = A[((size_t)wrap(y + dy, H) * W + wrap(x + dx, W)) * HD + d];
                        if (a > m) m = a;
                    }
                real sden = 0;
                for (int dy = -1; dy <= 1; ++dy)
                    for (int dx = -1; dx <= 1; ++dx)
                        sden += r_exp(A[((size_t)wrap(y + dy, H) * W + wrap(x + dx, W)) * HD + d] - m);
                mx[o + d] = m;
                den[o + d] = sden;
            }
        }
#pragma omp parallel for schedule(static)
    for (int y = 0; y < H; ++y)
        for (int x = 0; x < W; ++x) {
            const size_t o = ((size_t)y * W + x) * HD;
            for (int d = 0; d < HD; ++d) {
                const real an = A[o + d];
                real acc = 0;
                for (int dy = -1; dy <= 1; ++dy)
                    for (int dx = -1; dx <= 1; ++dx) {
                        const size_t s = ((size_t)wrap(y + dy, H) * W + wrap(x + dx, W)) * HD + d;
                        acc += r_exp(an - mx[s]) / den[s] * V[s];
                    }
                Vp[o + d] = acc;
            }
        }
}

/* ---- stages 5-6, closed form: E = exp(A), Z = box3(E), R = V/Z, V' = E * box3(R).  Same function as the
 * literal form (the softmax's max cancels); used by the timed CPU baseline and checked against it. ---- */
static void redistribute_boxsum(const real* A, const real* V, int H, int W, real* E, real* R, real* Vp) {
    const size_t n = (size_t)H * W * HD;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) E[i] = r_exp(A[i]);
#pragma omp parallel for schedule(static)
    for (int y = 0; y < H; ++y)
        for (int x = 0; x < W; ++x) {
            const size_t o = ((size_t)y * W + x) * HD;
            real z[HD];
            for (int d = 0; d < HD; ++d) z[d] = 0;
            for (int dy = -1; dy <= 1; ++dy)
                for (int dx = -1; dx <= 1; ++dx) {
                    const real* e = E + ((size_t)wrap(y + dy, H) * W + wrap(x + dx, W)) * HD;
                    for (int d = 0; d < HD; ++d) z[d] += e[d];
                }
            for (int d = 0; d < HD; ++d) R[o + d] = V[o + d] / z[d];
        }
#pragma omp parallel for schedule(static)
    for (int y = 0; y < H; ++y)
        for (int x = 0; x < W; ++x) {
            const size_t o = ((size_t)y * W + x) * HD;
            real b[HD];
            for (int d = 0; d < HD; ++d) b[d] = 0;
            for (int dy = -1; dy <= 1; ++dy)
                for (int dx = -1; dx <= 1; ++dx) {
                    const real* r = R + ((size_t)wrap(y + dy, H) * W + wrap(x + dx, W)) * HD;
                    for (int d = 0; d < HD; ++d) b[d] += r[d];
                }
            for (int d = 0; d < HD; ++d) Vp[o + d] = E[o + d] * b[d];
        }
}

/* ---- stage 7 for one head: Y += V'_h Wo_h ---- */
static void output_head(const real* Vp, int cells, const weight_set* w, int h, real* Y) {
    const float* wo = w->Wo + (size_t)h * HD * NC;
#pragma omp parallel for schedule(static)
    for (int s = 0; s < cells; ++s) {
        real acc[NC];
        real* y = Y + (size_t)s * NC;
        for (int c = 0; c < NC; ++c) acc[c] = y[c];
        const real* v = Vp + (size_t)s * HD;
        for (int d = 0; d < HD; ++d) {
            const real vd = v[d];
            const float* r = wo + d * NC;
            for (int c = 0; c < NC; ++c) acc[c] += vd * (real)r[c];
        }
        for (int c = 0; c < NC; ++c) y[c] = acc[c];
    }
}

/* Per-channel sums of one grid, fp64, fixed order (row by row). */
static void channel_sums(const float* X, int cells, double* out) {
    for (int c = 0; c < NC; ++c) out[c] = 0;
    for (int s = 0; s < cells; ++s)
        for (int c = 0; c < NC; ++c) out[c] += (double)X[(size_t)s * NC + c];
}

/*
 * Per-channel masses of every grid: mass[b][c] = sum over cells of X[b,:,:,c]  (fp64).
 */
void oracle_channel_mass(const float* X, int B, int H, int W, double* mass) {
    for (int b = 0; b < B; ++b) channel_sums(X + (size_t)b * H * W * NC, H * W, mass + (size_t)b * NC);
}

/*
 * Run n_steps of the contract step on B independent grids, in place.
 *   X        [B][H][W][64] fp32, in/out
 *   mass     [B][64] target per-channel masses (M_c); NULL = take them from X at entry
 *   sets     n_sets weight sets given as seven arrays, each the concatenation over sets
 *            grid b uses set b / (B / n_sets)
 *   literal  1 = stages 5-6 as the per-source softmax scatter; 0 = closed box-sum form
 *   renorm   1 = apply stage 9 after every step
 *   vp_prev, vp_last  optional [B][H][W][512] fp32: V' (index h*64+d) of steps n_steps-1 and n_steps
 * Returns 0, or -1 on bad arguments / allocation failure.
 */
int oracle_ca_steps(float* X, const double* mass, int B, int H, int W,
                    const float* Wp, const float* Wi, const float* Wv, const float* Wo,
                    const float* K, const float* mu, const float* sigma, int n_sets,
                    int n_steps, float dt, int literal, int renorm,
                    float* vp_prev, float* vp_last) {
    if (!X || B <= 0 || H <= 0 || W <= 0 || n_sets <= 0 || B % n_sets != 0 || n_steps < 0) return -1;
    const int cells = H * W;
    const size_t n = (size_t)cells * HD;
    real* P = (real*)malloc(n * sizeof(real));
    real* I = (real*)malloc(n * sizeof(real));
    real* V = (real*)malloc(n * sizeof(real));
    real* A = (real*)malloc(n * sizeof(real));
    real* T0 = (real*)malloc(n * sizeof(real));
    real* T1 = (real*)malloc(n * sizeof(real));
    real* Vp = (real*)malloc(n * sizeof(real));
    real* Y = (real*)malloc((size_t)cells * NC * sizeof(real));
    double* M = (double*)malloc((size_t)B * NC * sizeof(double));
    if (!P || !I || !V || !A || !T0 || !T1 || !Vp || !Y || !M) {
        free(P); free(I); free(V); free(A); free(T0); free(T1); free(Vp); free(Y); free(M);
        return -1;
    }
    if (mass) memcpy(M, mass, (size_t)B * NC * sizeof(double));
    else oracle_channel_mass(X, B, H, W, M);
    const int per_set = B / n_sets;

    for (int b = 0; b < B; ++b) {
        const int si = b / per_set;
        weight_set w = { Wp + (size_t)si * NH * NC * HD, Wi + (size_t)si * NH * NC * HD,
                         Wv + (size_t)si * NH * NC * HD, Wo + (size_t)si * HC * NC,
                         K + (size_t)si * NH * 9, mu + (size_t)si * NH, sigma + (size_t)si * NH };
        float* Xb = X + (size_t)b * cells * NC;
        for (int step = 0; step < n_steps; ++step) {
            memset(Y, 0, (size_t)cells * NC * sizeof(real));
            for (int h = 0; h < NH; ++h) {
                project_head(Xb, cells, &w, h, P, I, V);
                activation_head(P, I, H, W, &w, h, A);
                if (literal) redistribute_literal(A, V, H, W, T0, T1, Vp);
                else redistribute_boxsum(A, V, H, W, T0, T1, Vp);
                output_head(Vp, cells, &w, h, Y);
                float* dst = NULL;
                if (step == n_steps - 1 && vp_last) dst = vp_last;
                if (step == n_steps - 2 && vp_prev) dst = vp_prev;
                if (dst) {
                    dst += (size_t)b * cells * HC;
                    for (int s = 0; s < cells; ++s)
                        for (int d = 0; d < HD; ++d) dst[(size_t)s * HC + h * HD + d] = (float)Vp[(size_t)s * HD + d];
                }
            }
            /* stage 8 */
            for (size_t i = 0; i < (size_t)cells * NC; ++i) Xb[i] = (float)((real)Xb[i] + (real)dt * Y[i]);
            /* stage 9 */
            if (renorm) {
                double s[NC];
                channel_sums(Xb, cells, s);
                for (int c = 0; c < NC; ++c) s[c] = M[(size_t)b * NC + c] / s[c];
                for (int q = 0; q < cells; ++q)
                    for (int c = 0; c < NC; ++c) Xb[(size_t)q * NC + c] = (float)((double)Xb[(size_t)q * NC + c] * s[c]);
            }
        }
    }
    free(P); free(I); free(V); free(A); free(T0); free(T1); free(Vp); free(Y); free(M);
    return 0;
}

/* ------------------------------------------------------------------------------------------------ */
/* Fitness                                                                                           */
/* ------------------------------------------------------------------------------------------------ */

/*
 * Eigenvalues of a symmetric n x n matrix by cyclic two-sided Jacobi (in place; fp64).
 * Rotation: tau = (aqq-app)/(2 apq), t = sign(tau)/(|tau|+sqrt(1+tau^2)), c = 1/sqrt(1+t^2), s = t c
 * (slime/kernels/warp_ca.cu:51-63).  At most 30 sweeps (warp_ca.cu:20), stopping once the
 * off-diagonal Frobenius norm is <= 1e-6 x the matrix Frobenius norm (tolerance of
 * failed_attempts/pseudopod.cu:367, made scale-free).  Returns the number of sweeps done.
 */
int oracle_jacobi_eigenvalues(double* A, int n, double* eig) {
    double fro = 0;
    for (int i = 0; i < n * n; ++i) fro += A[i] * A[i];
    fro = sqrt(fro);
    int sweep = 0;
    for (; sweep < 30; ++sweep) {
        double off = 0;
        for (int p = 0; p < n; ++p)
            for (int q = 0; q < n; ++q)
                if (p != q) off += A[p * n + q] * A[p * n + q];
        if (sqrt(off) <= 1e-6 * fro) break;
        for (int p = 0; p < n - 1; ++p)
            for (int q = p + 1; q < n; ++q) {
                const double apq = A[p * n + q];
                if (apq == 0.0) continue;
                const double app = A[p * n + p], aqq = A[q * n + q];
                const double tau = (aqq - app) / (2.0 * apq);
                const double t = (tau >= 0 ? 1.0 : -1.0) / (fabs(tau) + sqrt(1.0 + tau * tau));
                const double c = 1.0 / sqrt(1.0 + t * t), s = t * c;
                for (int k = 0; k < n; ++k) { /* columns p,q */
                    const double akp = A[k * n + p], akq = A[k * n + q];
                    A[k * n + p] = c * akp - s * akq;
                    A[k * n + q] = s * akp + c * akq;
                }
                for (int k = 0; k < n; ++k) { /* rows p,q */
                    const double apk = A[p * n + k], aqk = A[q * n + k];
                    A[p * n + k] = c * apk - s * aqk;
                    A[q * n + k] = s * apk + c * aqk;
                }
            }
    }
    for (int i = 0; i < n; ++i) eig[i] = A[i * n + i];
    return sweep;
}

/*
 * exp-entropy rank of a spectrum: clamp to >= 0, p = l/(sum l + 1e-7), rank = exp(-sum p ln(p + 1e-7))
 * (slime/kernels/warp_ca.cu:107-144, epsilon :21).
 */
double oracle_entropy_rank(const double* eig, int n) {
    double sum = 0;
    for (int i = 0; i < n; ++i) sum += eig[i] > 0 ? eig[i] : 0;
    double ent = 0;
    for (int i = 0; i < n; ++i) {
        const double p = (eig[i] > 0 ? eig[i] : 0) / (sum + 1e-7);
        ent -= p * log(p + 1e-7);
    }
    return exp(ent);
}

/* Gram matrices of one grid's V' : gram[h][i][j] = sum_cells F[s][h*64+i] F[s][h*64+j]  (fp64). */
void oracle_gram(const float* vp, int cells, double* gram) {
#pragma omp parallel for schedule(static)
    for (int h = 0; h < NH; ++h) {
        double* g = gram + (size_t)h * HD * HD;
        for (int i = 0; i < HD * HD; ++i) g[i] = 0;
        for (int s = 0; s < cells; ++s) {
            const float* f = vp + (size_t)s * HC + h * HD;
            for (int i = 0; i < HD; ++i) {
                const double fi = f[i];
                for (int j = 0; j < HD; ++j) g[i * HD + j] += fi * (double)f[j];
            }
        }
    }
}

/*
 * Fitness of B grids from V' at the last two steps ([B][cells][512] fp32 each).
 * out_rank[b]  = mean over heads of the exp-entropy rank of that head's Gram spectrum
 * out_coh[b]   = Pearson r between all cells x 512 elements of vp_prev and vp_last (BLUEPRINT.md:362,428)
 * out_fit[b]   = rank x coherence (slime/kernels/warp_ca.cu:219); out_hunger[b] = 1 - coherence (:238)
 * out_head_rank optional [B][8].
 */
int oracle_fitness(const float* vp_prev, const float* vp_last, int B, int cells,
                   float* out_rank, float* out_coh, float* out_fit, float* out_hunger, float* out_head_rank) {
    if (!vp_prev || !vp_last || B <= 0 || cells <= 0) return -1;
    double* gram = (double*)malloc((size_t)NH * HD * HD * sizeof(double));
    if (!gram) return -1;
    for (int b = 0; b < B; ++b) {
        const float* a = vp_prev + (size_t)b * cells * HC;
        const float* c = vp_last + (size_t)b * cells * HC;
        oracle_gram(c, cells, gram);
        double rk = 0;
        for (int h = 0; h < NH; ++h) {
            double eig[HD];
            oracle_jacobi_eigenvalues(gram + (size_t)h * HD * HD, HD, eig);
            const double r = oracle_entropy_rank(eig, HD);
            if (out_head_rank) out_head_rank[(size_t)b * NH + h] = (float)r;
            rk += r;
        }
        rk /= NH;
        const size_t n = (size_t)cells * HC;
        double sa = 0, sb = 0;
        for (size_t i = 0; i < n; ++i) { sa += a[i]; sb += c[i]; }
        const double ma = sa / (double)n, mb = sb / (double)n;
        double saa = 0, sbb = 0, sab = 0;
        for (size_t i = 0; i < n; ++i) {
            const double da = a[i] - ma, db = c[i] - mb;
            saa += da * da; sbb += db * db; sab += da * db;
        }
        const double coh = sab / sqrt(saa * sbb);
        if (out_rank) out_rank[b] = (float)rk;
        if (out_coh) out_coh[b] = (float)coh;
        if (out_fit) out_fit[b] = (float)(rk * coh);
        if (out_hunger) out_hunger[b] = (float)(1.0 - coh);
    }
    free(gram);
    return 0;
}

/* ------------------------------------------------------------------------------------------------ */
/* Field <-> CA coupling (the step's two neighbours in the reference driver)                         */
/* ------------------------------------------------------------------------------------------------ */

/*
 * Lift a one-channel field into the 64-channel CA state: X[b,y,x,c] = img[b,y,x] * L[c], after zero-padding
 * the image by `pad` pixels on every side.  Mirrors slime/core/organism.cu:691-720, which lifts the chemical
 * field with a fixed per-channel factor.
 */
void oracle_lift(const float* img, int B, int h, int w, int pad, const float* L, float* X) {
    const int H = h + 2 * pad, W = w + 2 * pad;
    memset(X, 0, (size_t)B * H * W * NC * sizeof(float));
    for (int b = 0; b < B; ++b)
        for (int y = 0; y < h; ++y)
            for (int x = 0; x < w; ++x) {
                const float v = img[((size_t)b * h + y) * w + x];
                float* o = X + (((size_t)b * H + y + pad) * W + x + pad) * NC;
                for (int c = 0; c < NC; ++c) o[c] = v * L[c];
            }
}

/*
 * Mean-pool the state over space and apply a 64 -> n_out linear readout:
 * logits[b][o] = sum_c mean_cells(X[b,:,:,c]) Wr[c][o] + br[o].  The pooling mirrors
 * slime/core/organism.cu:723-743 (mean write-back of the CA into the field).
 */
void oracle_pool_readout(const float* X, int B, int cells, const float* Wr, const float* br, int n_out, float* logits) {
    for (int b = 0; b < B; ++b) {
        double m[NC];
        channel_sums(X + (size_t)b * cells * NC, cells, m);
        for (int o = 0; o < n_out; ++o) {
            double acc = br ? br[o] : 0.0;
            for (int c = 0; c < NC; ++c) acc += m[c] / cells * (double)Wr[c * n_out + o];
            logits[(size_t)b * n_out + o] = (float)acc;
        }
    }
}

/*
 * Write the CA back into a one-channel field: field[b][cell] = mean over the 64 channels of X[b][cell][:].
 * Follows slime/core/organism.cu:723-743 (update_field_from_ca_kernel: sum over the cell's channels / CHANNELS).
 */
void oracle_field_from_state(const float* X, int B, int cells, float* field) {
    for (size_t i = 0; i < (size_t)B * cells; ++i) {
        double acc = 0.0;
        for (int c = 0; c < NC; ++c) acc += (double)X[i * NC + c];
        field[i] = (float)(acc / NC);
    }
}

/*
 * The contract's weight set taken out of the reference's weight bundle (struct MultiHeadCAState,
 * slime/core/pseudopod.cu:29-38), as the reference's kernels index it:
 *   Wp[h][c][d] = perception [h][c][d]  of [8][512][256]   (slime/core/pseudopod.cu:86-87; only c, d < 64 are read)
 *   Wi[h][c][d] = interaction[h][c][d]  of [8][512][256]   (slime/core/pseudopod.cu:102-103)
 *   Wv[h][c][d] = sum over r < 4 of value[h][c + 64 r][d] of [8][256][512]: the reference sums j < 256 of
 *                 interaction[j % 64] * value[h][j][d] (slime/core/pseudopod.cu:114-119)
 *   K[h][t]     = flow_kernels[h][t]                        (slime/core/pseudopod.cu:153)
 *   Wo[(h, d)][c] = (d == c) * mean over out-heads o of mixing[o][h]: the 8 x 8 head mixing
 *                 (slime/core/pseudopod.cu:231-249) followed by the mean of the 8 output heads, which is what a
 *                 64-channel state can take from a bundle that has no 512 -> 64 projection.
 */
void oracle_weights_from_reference_layout(const float* perception, const float* interaction, const float* value,
                                          const float* mixing, const float* flow, float* Wp, float* Wi, float* Wv,
                                          float* Wo, float* K) {
    for (int h = 0; h < NH; ++h) {
        double m = 0.0;
        for (int o = 0; o < NH; ++o) m += (double)mixing[o * NH + h];
        for (int c = 0; c < NC; ++c)
            for (int d = 0; d < HD; ++d) {
                const size_t dst = ((size_t)h * NC + c) * HD + d;
                Wp[dst] = perception[((size_t)h * 512 + c) * 256 + d];
                Wi[dst] = interaction[((size_t)h * 512 + c) * 256 + d];
                float acc = 0.f;
                for (int r = 0; r < 4; ++r) acc += value[((size_t)h * 256 + c + 64 * r) * 512 + d];
                Wv[dst] = acc;
                Wo[((size_t)h * HD + d) * NC + c] = d == c ? (float)(m / NH) : 0.f;
            }
        for (int t = 0; t < 9; ++t) K[h * 9 + t] = flow[h * 9 + t];
    }
}

/*
 * The population step over weight sets (culling, best, refill by mutated copies of the best).  Rules:
 * culling thresholds slime/core/organism.cu:594-611; best = arg max fitness, slime/core/organism.cu:442-470;
 * refill = parent's values, each perturbed with probability `rate` by sigma * N(0,1), slime/memory/pool.cu:84-93.
 * fit: [n_sets * per_set][4] = {rank, coherence, fitness, hunger} per grid.  Wp, Wi, Wv: [n_sets][8*64*64],
 * Wo: [n_sets][512*64], updated in place.  parent[s] = s for survivors, else the best; returns the number of
 * replaced sets and stores the best index (or -1).  The perturbation stream is a counter hash of
 * (seed, generation, set, value index, draw).
 */
static uint64_t evolve_mix(uint64_t z) {
    z += 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}
static uint32_t evolve_bits(uint64_t seed, int generation, int s, int i, int k) {
    const uint64_t key = evolve_mix(evolve_mix(seed ^ ((uint64_t)(uint32_t)generation << 32)) ^ (uint64_t)(uint32_t)s);
    return (uint32_t)(evolve_mix(key ^ ((uint64_t)(uint32_t)i * 4u + (uint32_t)k)) >> 40);
}
int oracle_evolve(const float* fit, int n_sets, int per_set, float fitness_threshold, float hunger_threshold,
                  float rate, float sigma, unsigned long long seed, int generation, float* Wp, float* Wi, float* Wv,
                  float* Wo, int* parent, int* best_out) {
    const int NM = NH * NC * HD;
    float* mf = (float*)malloc(sizeof(float) * (size_t)n_sets);
    int best = -1, replaced = 0;
    for (int s = 0; s < n_sets; ++s) {
        double f = 0.0, q = 0.0;
        for (int j = 0; j < per_set; ++j) {
            f += (double)fit[(size_t)(s * per_set + j) * 4 + 2];
            q += (double)fit[(size_t)(s * per_set + j) * 4 + 3];
        }
        mf[s] = (float)(f / per_set);
        const float mq = (float)(q / per_set);
        const int alive = isfinite(mf[s]) && isfinite(mq) && !(mf[s] < 0.1f * fitness_threshold) && !(mq > hunger_threshold);
        parent[s] = alive ? s : -1;
        if (!alive) { ++replaced; continue; }
        if (best < 0 || mf[s] > mf[best]) best = s;
    }
    free(mf);
    *best_out = best;
    if (best < 0) {
        for (int s = 0; s < n_sets; ++s) parent[s] = s;
        return 0;
    }
    float r = rate < 0.f ? 0.f : (rate > 1.f ? 1.f : rate);
    const uint32_t rate24 = (uint32_t)(r * 16777216.0f);
    float* arrays[4] = { Wp, Wi, Wv, Wo };
    for (int s = 0; s < n_sets; ++s) {
        if (parent[s] >= 0) continue;
        parent[s] = best;
        for (int a = 0; a < 4; ++a)
            for (int j = 0; j < NM; ++j) {
                const int i = a * NM + j;       /* index in the set's concatenated Wp | Wi | Wv | Wo */
                double v = (double)arrays[a][(size_t)best * NM + j];
                if (evolve_bits(seed, generation, s, i, 0) < rate24) {
                    const double u1 = ((double)evolve_bits(seed, generation, s, i, 1) + 1.0) / 16777216.0;
                    const double u2 = (double)evolve_bits(seed, generation, s, i, 2) / 16777216.0;
                    v = (double)(float)v + (double)sigma * sqrt(-2.0 * log(u1)) * cos(6.283185307179586 * u2);
                }
                arrays[a][(size_t)s * NM + j] = (float)v;
            }
    }
    return replaced;
}

/* Threads the OpenMP loops above use from now on (n <= 0: leave as is); returns the count in force.  Launchers
 * that start one process per GPU export OMP_NUM_THREADS=1, which is not what a timed CPU baseline wants. */
int oracle_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}

/*
 * The reference's genome hash of an elite record (gpu_sha256, slime/memory/archive.cu:41-60; the name
 * notwithstanding, a 64-bit shift-add-xor mix taken over the fp32 bit patterns in order).  Per value:
 *   h ^= (bits + 0x9e3779b9 mod 2^32) + (h << 6) + (h >> 2);  h += h << 3;  h ^= h >> 11;  h += h << 15;
 *   h *= 0xc4ceb9fe1a85ec53;  h ^= h >> 33;          starting from h = 0x9e3779b97f4a7c15.
 * Pinned by tests/golden/ref_elite.json, which the reference's own create_elite_kernel wrote.
 */
unsigned long long oracle_genome_hash(const float* genome, unsigned long long n) {
    uint64_t h = UINT64_C(0x9e3779b97f4a7c15);
    for (unsigned long long i = 0; i < n; ++i) {
        uint32_t bits;
        memcpy(&bits, genome + i, 4);
        h ^= (uint64_t)(uint32_t)(bits + UINT32_C(0x9e3779b9)) + (h << 6) + (h >> 2);   /* the 32-bit sum wraps, as in the reference's expression */
        h += h << 3;
        h ^= h >> 11;
        h += h << 15;
        h *= UINT64_C(0xc4ceb9fe1a85ec53);
        h ^= h >> 33;
    }
    return (unsigned long long)h;
}
