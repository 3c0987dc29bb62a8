/*
 * CPU oracle for the three scan operators.  TEST INFRASTRUCTURE ONLY: nothing
 * in the shipped package may link, import or call this file; it exists so the
 * CUDA kernels can be checked against an independent evaluation of the same
 * mathematics.
 *
 * Each function restates one of the reference's pure-PyTorch definitions:
 *   oracle_selective_scan     <- mamba_ssm/ops/selective_scan_interface.py:127-193
 *   oracle_selective_scan_bwd <- the gradient autograd derives from the same lines (checked against the CUDA
 *                                backward at tests/ops/test_selective_scan.py:119-147)
 *   oracle_state_update       <- mamba_ssm/ops/triton/selective_state_update.py:224-285
 *   oracle_causal_conv1d      <- the depthwise nn.Conv1d with left padding that the mixers fall back to,
 *                                mamba_ssm/modules/mamba2.py:232-234 (mamba_simple.py:166-171), with the packed-
 *                                sequence and carried-state options of the causal-conv1d package it stands in for
 *   oracle_conv1d_update      <- the single-token roll / multiply / sum at mamba_ssm/modules/mamba2.py:309-315
 *   oracle_rmsnorm_gated      <- rms_norm_ref, mamba_ssm/ops/triton/layernorm_gated.py:18-41
 *   oracle_ssd_chunk_scan     <- mamba_ssm/ops/triton/ssd_combined.py:687-725, built from
 *                                ssd_chunk_state.py:1094-1122 (chunk states),
 *                                ssd_state_passing.py:327-350 (inter-chunk recurrence) and
 *                                ssd_chunk_scan.py:1846-1887 (chunk output)
 *
 * The arithmetic is carried in double so the oracle sits closer to the exact
 * result than either fp32 implementation (the reference's or the GPU's); the
 * pin against the reference (tests/golden) therefore holds to fp32 round-off,
 * not bit-exactly.  All arrays are dense row-major float32; callers upcast
 * bf16/fp16 inputs first, as the reference's selective_scan_ref does.
 *
 * Parity pin: tests/test_oracle.py checks every function here against golden
 * outputs produced by importing the reference itself (tests/golden/make_golden.py).
 */
#include <math.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* torch.nn.functional.softplus with its default threshold of 20. */
static inline double softplus20(double x) { return x > 20.0 ? x : log1p(exp(x)); }
static inline double silu(double z) { return z / (1.0 + exp(-z)); }

int oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/*
 * Mamba-1 selective scan.
 *   u, delta, z, out : (batch, dim, L)
 *   A                : (dim, N)
 *   B, C             : variable -> (batch, ngroups, N, L); constant -> (dim, N)
 *   D, delta_bias    : (dim) or NULL
 *   last_state       : (batch, dim, N) or NULL
 * Recurrence per (b, d, n):  h_t = exp(dt_t A) h_{t-1} + dt_t B_t u_t,
 *   y_t = sum_n C_t h_t + D u_t, then y_t * silu(z_t) when z is given.
 */
void oracle_selective_scan(const float *u, const float *delta, const float *A,
                           const float *B, const float *C, const float *D,
                           const float *z, const float *delta_bias,
                           int delta_softplus, int batch, int dim, int L, int N,
                           int ngroups, int B_variable, int C_variable,
                           float *out, float *last_state)
{
    const int per_group = dim / (ngroups > 0 ? ngroups : 1);
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < batch; ++b) {
        for (int d = 0; d < dim; ++d) {
            double h[256];
            for (int n = 0; n < N; ++n) h[n] = 0.0;
            const size_t row = ((size_t)b * dim + d) * (size_t)L;
            const int g = B_variable || C_variable ? d / per_group : 0;
            const float *Bv = B_variable ? B + ((size_t)b * ngroups + g) * (size_t)N * L : B + (size_t)d * N;
            const float *Cv = C_variable ? C + ((size_t)b * ngroups + g) * (size_t)N * L : C + (size_t)d * N;
            for (int t = 0; t < L; ++t) {
                double dt = delta[row + t];
                if (delta_bias) dt += delta_bias[d];
                if (delta_softplus) dt = softplus20(dt);
                const double uu = u[row + t];
                double y = 0.0;
                for (int n = 0; n < N; ++n) {
                    const double a = exp(dt * (double)A[(size_t)d * N + n]);
                    const double bn = B_variable ? Bv[(size_t)n * L + t] : Bv[n];
                    const double cn = C_variable ? Cv[(size_t)n * L + t] : Cv[n];
                    h[n] = a * h[n] + dt * bn * uu;
                    y += h[n] * cn;
                }
                if (D) y += uu * (double)D[d];
                if (z) y *= silu(z[row + t]);
                out[row + t] = (float)y;
            }
            if (last_state)
                for (int n = 0; n < N; ++n)
                    last_state[((size_t)b * dim + d) * N + n] = (float)h[n];
        }
    }
}

/*
 * Gradient of the Mamba-1 selective scan with respect to every differentiable input, given dout = dL/d(out).
 * The reference defines it only through autograd on selective_scan_ref (the check that
 * tests/ops/test_selective_scan.py:119-147 makes against the CUDA backward); this is the adjoint of the
 * recurrence above, written out:
 *   dy_t = dout_t silu(z_t)            dz_t = dout_t y_t silu'(z_t)            (dy_t = dout_t without z)
 *   g_t  = C_t dy_t + a_{t+1} g_{t+1}                                          (a_t = exp(dt_t A), g_L = 0)
 *   du_t = D dy_t + dt_t sum_n g_t B_t          dD = sum u_t dy_t
 *   d(dt_t) = sum_n g_t (A a_t h_{t-1} + B_t u_t)        dA = sum_t g_t dt_t a_t h_{t-1}
 *   dB_t = sum_d g_t dt_t u_t   dC_t = sum_d dy_t h_t    (sums over the channels of the group; over batch and
 *                                                          time for constant B, C)
 *   d(delta_t) = d(dt_t) softplus'(delta_t + bias)        d(delta_bias) = sum_{b,t} d(delta_t)
 * Shapes as in oracle_selective_scan; dB, dC have the shape of B, C.  dD, ddelta_bias, dz may be NULL.
 */
void oracle_selective_scan_bwd(const float *u, const float *delta, const float *A,
                               const float *B, const float *C, const float *D,
                               const float *z, const float *delta_bias, const float *dout,
                               int delta_softplus, int batch, int dim, int L, int N,
                               int ngroups, int B_variable, int C_variable,
                               float *du, float *ddelta, float *dA, float *dB, float *dC,
                               float *dD, float *ddelta_bias, float *dz)
{
    const int G = ngroups > 0 ? ngroups : 1;
    const int per_group = dim / G;
    double *accA = (double *)calloc((size_t)dim * N, sizeof(double));
    double *accBc = (double *)calloc((size_t)dim * N, sizeof(double));      /* constant B, C */
    double *accCc = (double *)calloc((size_t)dim * N, sizeof(double));
    double *accD = (double *)calloc((size_t)dim, sizeof(double));
    double *accb = (double *)calloc((size_t)dim, sizeof(double));
    /* one (batch row, group) per iteration: its channels are walked one after the other, so the sums over the
     * channels of a group stay inside one thread; the per-channel parameter gradients, which sum over batch rows,
     * are accumulated with atomic updates */
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (int b = 0; b < batch; ++b) {
        for (int g = 0; g < G; ++g) {
            double *hist = (double *)malloc(sizeof(double) * (size_t)(L + 1) * N);     /* h_0 .. h_L */
            double *dts = (double *)malloc(sizeof(double) * (size_t)L);
            double *sBv = B_variable ? (double *)calloc((size_t)N * L, sizeof(double)) : NULL;
            double *sCv = C_variable ? (double *)calloc((size_t)N * L, sizeof(double)) : NULL;
            double gv[256];
            const float *Bg = B_variable ? B + ((size_t)b * G + g) * (size_t)N * L : NULL;
            const float *Cg = C_variable ? C + ((size_t)b * G + g) * (size_t)N * L : NULL;
            for (int d = g * per_group; d < (g + 1) * per_group; ++d) {
                const size_t row = ((size_t)b * dim + d) * (size_t)L;
                const float *Ad = A + (size_t)d * N;
                for (int n = 0; n < N; ++n) hist[n] = 0.0;
                for (int t = 0; t < L; ++t) {
                    double dt = delta[row + t];
                    if (delta_bias) dt += delta_bias[d];
                    if (delta_softplus) dt = softplus20(dt);
                    dts[t] = dt;
                    for (int n = 0; n < N; ++n) {
                        const double bn = B_variable ? Bg[(size_t)n * L + t] : B[(size_t)d * N + n];
                        hist[(size_t)(t + 1) * N + n] = exp(dt * (double)Ad[n]) * hist[(size_t)t * N + n] + dt * bn * (double)u[row + t];
                    }
                }
                for (int n = 0; n < N; ++n) gv[n] = 0.0;       /* a_{t+1} g_{t+1}, carried backwards */
                double sumD = 0.0, sumb = 0.0;
                for (int t = L - 1; t >= 0; --t) {
                    const double dt = dts[t], uu = u[row + t];
                    double dy = dout[row + t];
                    if (z) {
                        const double zz = z[row + t], sg = 1.0 / (1.0 + exp(-zz));
                        double y = D ? uu * (double)D[d] : 0.0;
                        for (int n = 0; n < N; ++n) {
                            const double cn = C_variable ? Cg[(size_t)n * L + t] : C[(size_t)d * N + n];
                            y += hist[(size_t)(t + 1) * N + n] * cn;
                        }
                        if (dz) dz[row + t] = (float)(dy * y * sg * (1.0 + zz * (1.0 - sg)));
                        dy *= zz * sg;
                    }
                    double s_gb = 0.0, ddt = 0.0;
                    for (int n = 0; n < N; ++n) {
                        const double bn = B_variable ? Bg[(size_t)n * L + t] : B[(size_t)d * N + n];
                        const double cn = C_variable ? Cg[(size_t)n * L + t] : C[(size_t)d * N + n];
                        const double a = exp(dt * (double)Ad[n]);
                        const double hprev = hist[(size_t)t * N + n], hcur = hist[(size_t)(t + 1) * N + n];
                        const double gt = cn * dy + gv[n];
                        s_gb += gt * bn;
                        ddt += gt * ((double)Ad[n] * a * hprev + bn * uu);
#pragma omp atomic
                        accA[(size_t)d * N + n] += gt * dt * a * hprev;
                        if (B_variable) sBv[(size_t)n * L + t] += gt * dt * uu;
                        else {
#pragma omp atomic
                            accBc[(size_t)d * N + n] += gt * dt * uu;
                        }
                        if (C_variable) sCv[(size_t)n * L + t] += dy * hcur;
                        else {
#pragma omp atomic
                            accCc[(size_t)d * N + n] += dy * hcur;
                        }
                        gv[n] = a * gt;
                    }
                    du[row + t] = (float)((D ? (double)D[d] * dy : 0.0) + dt * s_gb);
                    sumD += uu * dy;
                    double dd = ddt;
                    if (delta_softplus) {
                        const double x = (double)delta[row + t] + (delta_bias ? (double)delta_bias[d] : 0.0);
                        if (x <= 20.0) dd *= 1.0 / (1.0 + exp(-x));
                    }
                    ddelta[row + t] = (float)dd;
                    sumb += dd;
                }
#pragma omp atomic
                accD[d] += sumD;
#pragma omp atomic
                accb[d] += sumb;
            }
            if (B_variable)
                for (size_t i = 0; i < (size_t)N * L; ++i) dB[((size_t)b * G + g) * (size_t)N * L + i] = (float)sBv[i];
            if (C_variable)
                for (size_t i = 0; i < (size_t)N * L; ++i) dC[((size_t)b * G + g) * (size_t)N * L + i] = (float)sCv[i];
            free(hist); free(dts); free(sBv); free(sCv);
        }
    }
    for (size_t i = 0; i < (size_t)dim * N; ++i) {
        dA[i] = (float)accA[i];
        if (!B_variable) dB[i] = (float)accBc[i];
        if (!C_variable) dC[i] = (float)accCc[i];
    }
    for (int d = 0; d < dim; ++d) {
        if (dD) dD[d] = (float)accD[d];
        if (ddelta_bias) ddelta_bias[d] = (float)accb[d];
    }
    free(accA); free(accBc); free(accCc); free(accD); free(accb);
}

/*
 * Single-token decode update (heads form; the no-heads form is nheads == 1).
 *   state : (batch, nheads, dim, N) updated in place
 *   x, dt, z, out : (batch, nheads, dim)
 *   A : (nheads, dim, N);  B, C : (batch, ngroups, N);  D, dt_bias : (nheads, dim) or NULL
 */
void oracle_state_update(float *state, const float *x, const float *dt,
                         const float *A, const float *B, const float *C,
                         const float *D, const float *z, const float *dt_bias,
                         int dt_softplus, int batch, int nheads, int dim, int N,
                         int ngroups, float *out)
{
    const int hpg = nheads / ngroups;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < batch; ++b) {
        for (int h = 0; h < nheads; ++h) {
            const int g = h / hpg;
            const float *Bv = B + ((size_t)b * ngroups + g) * N;
            const float *Cv = C + ((size_t)b * ngroups + g) * N;
            for (int p = 0; p < dim; ++p) {
                const size_t i = ((size_t)b * nheads + h) * dim + p;
                double t = dt[i];
                if (dt_bias) t += dt_bias[(size_t)h * dim + p];
                if (dt_softplus) t = softplus20(t);
                const double xx = x[i];
                float *s = state + i * N;
                const float *Ap = A + ((size_t)h * dim + p) * N;
                double y = 0.0;
                for (int n = 0; n < N; ++n) {
                    const double sn = (double)s[n] * exp(t * (double)Ap[n]) + t * (double)Bv[n] * xx;
                    s[n] = (float)sn;
                    y += sn * (double)Cv[n];
                }
                if (D) y += xx * (double)D[(size_t)h * dim + p];
                if (z) y *= silu(z[i]);
                out[i] = (float)y;
            }
        }
    }
}

/*
 * Mamba-2 SSD chunked forward.
 *   x, z, out : (batch, L, nheads, P);  dt : (batch, L, nheads)
 *   A, dt_bias : (nheads);  B, C : (batch, L, ngroups, N)
 *   D : (nheads) or (nheads, P) per D_has_hdim;  initial_states, final_states : (batch, nheads, P, N)
 * dt is biased, soft-plussed, clamped to [dt_min, dt_max] and treated as zero past L
 * (the padding rule of ssd_chunk_state.py:81).  Per chunk of Q steps:
 *   cum_k   = inclusive cumsum of dt_k A over the chunk
 *   S_c     = sum_k exp(cum_last - cum_k) dt_k x_k (outer) B_k          (chunk state)
 *   H_{c+1} = exp(cum_last) H_c + S_c                                      (state passing)
 *   y_m     = exp(cum_m) C_m.H_c + sum_{k<=m} (C_m.B_k) exp(cum_m - cum_k) dt_k x_k + D x_m
 */
void oracle_ssd_chunk_scan(const float *x, const float *dt, const float *A,
                           const float *B, const float *C, const float *D,
                           const float *z, const float *dt_bias,
                           const float *initial_states, int dt_softplus,
                           float dt_min, float dt_max, int D_has_hdim, int batch,
                           int L, int nheads, int P, int ngroups, int N, int Q,
                           float *out, float *final_states)
{
    const int nchunks = (L + Q - 1) / Q;
    const int hpg = nheads / ngroups;
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (int b = 0; b < batch; ++b) {
        for (int h = 0; h < nheads; ++h) {
            const int g = h / hpg;
            double *H = (double *)malloc(sizeof(double) * (size_t)P * N);
            double *S = (double *)malloc(sizeof(double) * (size_t)P * N);
            double *dtv = (double *)malloc(sizeof(double) * Q);
            double *cum = (double *)malloc(sizeof(double) * Q);
            double *cb = (double *)malloc(sizeof(double) * Q);
            double *acc = (double *)malloc(sizeof(double) * P);
            for (size_t i = 0; i < (size_t)P * N; ++i)
                H[i] = initial_states ? (double)initial_states[((size_t)b * nheads + h) * P * N + i] : 0.0;
            for (int c = 0; c < nchunks; ++c) {
                const int t0 = c * Q;
                const int len = (L - t0 < Q) ? L - t0 : Q;
                double run = 0.0;
                for (int k = 0; k < Q; ++k) {
                    double v = 0.0;
                    if (k < len) {
                        v = dt[((size_t)b * L + t0 + k) * nheads + h];
                        if (dt_bias) v += dt_bias[h];
                        if (dt_softplus) v = softplus20(v);
                        if (v < dt_min) v = dt_min;
                        if (v > dt_max) v = dt_max;
                    }
                    dtv[k] = v;
                    run += v * (double)A[h];
                    cum[k] = run;
                }
                /* outputs of this chunk from the incoming state H and the intra-chunk terms */
                for (int m = 0; m < len; ++m) {
                    const float *Cm = C + (((size_t)b * L + t0 + m) * ngroups + g) * N;
                    for (int k = 0; k <= m; ++k) {
                        const float *Bk = B + (((size_t)b * L + t0 + k) * ngroups + g) * N;
                        double s = 0.0;
                        for (int n = 0; n < N; ++n) s += (double)Cm[n] * (double)Bk[n];
                        cb[k] = s * exp(cum[m] - cum[k]) * dtv[k];
                    }
                    const double dec = exp(cum[m]);
                    for (int p = 0; p < P; ++p) {
                        double s = 0.0;
                        for (int n = 0; n < N; ++n) s += (double)Cm[n] * H[(size_t)p * N + n];
                        acc[p] = s * dec;
                    }
                    for (int k = 0; k <= m; ++k) {
                        const float *xk = x + (((size_t)b * L + t0 + k) * nheads + h) * P;
                        const double w = cb[k];
                        for (int p = 0; p < P; ++p) acc[p] += w * (double)xk[p];
                    }
                    const size_t o = (((size_t)b * L + t0 + m) * nheads + h) * P;
                    for (int p = 0; p < P; ++p) {
                        double y = acc[p];
                        if (D) y += (double)x[o + p] * (double)(D_has_hdim ? D[(size_t)h * P + p] : D[h]);
                        if (z) y *= silu(z[o + p]);
                        out[o + p] = (float)y;
                    }
                }
                /* chunk state and the recurrence to the next chunk */
                memset(S, 0, sizeof(double) * (size_t)P * N);
                for (int k = 0; k < len; ++k) {
                    const float *Bk = B + (((size_t)b * L + t0 + k) * ngroups + g) * N;
                    const float *xk = x + (((size_t)b * L + t0 + k) * nheads + h) * P;
                    const double w = exp(cum[Q - 1] - cum[k]) * dtv[k];
                    for (int p = 0; p < P; ++p) {
                        const double xw = w * (double)xk[p];
                        for (int n = 0; n < N; ++n) S[(size_t)p * N + n] += xw * (double)Bk[n];
                    }
                }
                const double carry = exp(cum[Q - 1]);
                for (size_t i = 0; i < (size_t)P * N; ++i) H[i] = carry * H[i] + S[i];
            }
            if (final_states)
                for (size_t i = 0; i < (size_t)P * N; ++i)
                    final_states[((size_t)b * nheads + h) * P * N + i] = (float)H[i];
            free(H); free(S); free(dtv); free(cum); free(cb); free(acc);
        }
    }
}


/* ---- causal depthwise conv1d ------------------------------------------------------------------
 * x, out (batch, dim, seqlen) dense; weight (dim, width); bias (dim) or NULL; seq_idx (batch, seqlen) or NULL;
 * init (batch, dim, width-1) or NULL; fin (batch, dim, width-1) or NULL. */
void oracle_causal_conv1d(const float *x, const float *weight, const float *bias, const int *seq_idx, const float *init,
                          int silu_act, int batch, int dim, int L, int W, float *out, float *fin)
{
#pragma omp parallel for collapse(2)
    for (int b = 0; b < batch; ++b)
        for (int c = 0; c < dim; ++c) {
            const float *xr = x + ((size_t)b * dim + c) * L;
            const float *ir = init ? init + ((size_t)b * dim + c) * (W - 1) : NULL;
            for (int t = 0; t < L; ++t) {
                double s = bias ? bias[c] : 0.0;
                for (int k = 0; k < W; ++k) {
                    const int tk = t - (W - 1) + k;
                    double v;
                    if (tk >= 0) {
                        if (seq_idx && seq_idx[(size_t)b * L + tk] != seq_idx[(size_t)b * L + t]) continue;
                        v = xr[tk];
                    } else {
                        v = ir ? ir[W - 1 + tk] : 0.0;
                    }
                    s += (double)weight[(size_t)c * W + k] * v;
                }
                out[((size_t)b * dim + c) * L + t] = (float)(silu_act ? silu(s) : s);
            }
            if (fin)
                for (int j = 0; j < W - 1; ++j) {
                    const int t = L - (W - 1) + j;
                    fin[((size_t)b * dim + c) * (W - 1) + j] = t >= 0 ? xr[t] : (ir ? ir[W - 1 + t] : 0.f);
                }
        }
}

/* state (batch, dim, S) updated in place; x, out (batch, dim). */
void oracle_conv1d_update(float *state, const float *x, const float *weight, const float *bias, int silu_act, int batch,
                          int dim, int W, int S, float *out)
{
    for (int b = 0; b < batch; ++b)
        for (int c = 0; c < dim; ++c) {
            float *st = state + ((size_t)b * dim + c) * S;
            for (int j = 0; j + 1 < S; ++j) st[j] = st[j + 1];
            st[S - 1] = x[(size_t)b * dim + c];
            double s = bias ? bias[c] : 0.0;
            for (int k = 0; k < W; ++k) s += (double)weight[(size_t)c * W + k] * st[S - W + k];
            out[(size_t)b * dim + c] = (float)(silu_act ? silu(s) : s);
        }
}

/* x, z, out (rows, cols) dense; weight, bias (cols). */
void oracle_rmsnorm_gated(const float *x, const float *z, const float *weight, const float *bias, double eps, int group,
                          int norm_before_gate, long rows, int cols, float *out)
{
#pragma omp parallel for
    for (long r = 0; r < rows; ++r)
        for (int g0 = 0; g0 < cols; g0 += group) {
            double ss = 0.0;
            for (int e = g0; e < g0 + group; ++e) {
                double v = x[(size_t)r * cols + e];
                if (z && !norm_before_gate) v *= silu(z[(size_t)r * cols + e]);
                ss += v * v;
            }
            const double rstd = 1.0 / sqrt(ss / group + eps);
            for (int e = g0; e < g0 + group; ++e) {
                double v = x[(size_t)r * cols + e];
                if (z && !norm_before_gate) v *= silu(z[(size_t)r * cols + e]);
                double y = v * rstd * weight[e] + (bias ? bias[e] : 0.0);
                if (z && norm_before_gate) y *= silu(z[(size_t)r * cols + e]);
                out[(size_t)r * cols + e] = (float)y;
            }
        }
}
