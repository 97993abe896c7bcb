/*
 * CPU oracle for the mgpt Mixture-of-Experts layer: a plain-C restatement of
 * the arithmetic the reference performs with Device::CPU tensors.
 *
 * TEST INFRASTRUCTURE ONLY (see moe_oracle.h). Parity status: PINNED against
 * the reference's own code (oracle/_ref) and tests/golden/.
 *
 * Build with -O2 -ffp-contract=off and no -march/-ffast-math: the reference's
 * loops use a separate float multiply and add per term and the restatement
 * must round the same way.  Every function cites the reference lines it
 * follows (paths are relative to the reference's src/main/).
 */
#include "moe_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

/* Minimal row-parallel helper (POSIX threads): calls fn(lo, hi, arg) on
 * disjoint row ranges.  Only whole output rows are split, never a sum. */
typedef void (*range_fn)(int lo, int hi, void* arg);
typedef struct {
    range_fn fn;
    void* arg;
    int lo, hi;
} range_job;

static void* range_thread(void* p)
{
    range_job* j = (range_job*)p;
    j->fn(j->lo, j->hi, j->arg);
    return NULL;
}

static void parallel_rows(int n, int nt, range_fn fn, void* arg)
{
    if (nt > n) nt = n;
    if (nt <= 1) {
        fn(0, n, arg);
        return;
    }
    pthread_t* th = (pthread_t*)malloc((size_t)nt * sizeof(pthread_t));
    range_job* jobs = (range_job*)malloc((size_t)nt * sizeof(range_job));
    int started = 0;
    for (int t = 0; t < nt; ++t) {
        jobs[t].fn = fn;
        jobs[t].arg = arg;
        jobs[t].lo = (int)((long long)n * t / nt);
        jobs[t].hi = (int)((long long)n * (t + 1) / nt);
        if (pthread_create(&th[t], NULL, range_thread, &jobs[t]) != 0) {
            fn(jobs[t].lo, jobs[t].hi, arg); /* could not spawn: run inline */
            th[t] = 0;
        } else {
            started++;
        }
    }
    (void)started;
    for (int t = 0; t < nt; ++t)
        if (th[t]) pthread_join(th[t], NULL);
    free(th);
    free(jobs);
}

/* C[M,N] = A[M,K] * B[K,N], i-k-j order, C zeroed first.
 * utils/Tensor.cpp:567-577 (matmul2d_raw). Rows are independent, so they may
 * be split across threads without changing any sum. */
typedef struct {
    const float *A, *B;
    float* C;
    int K, N;
} mm_args;

static void mm_rows(int lo, int hi, void* p)
{
    const mm_args* a = (const mm_args*)p;
    const int K = a->K, N = a->N;
    for (int i = lo; i < hi; ++i) {
        float* c = a->C + (size_t)i * N;
        for (int j = 0; j < N; ++j) c[j] = 0.0f;
        for (int k = 0; k < K; ++k) {
            const float av = a->A[(size_t)i * K + k];
            const float* b = a->B + (size_t)k * N;
            for (int j = 0; j < N; ++j) c[j] += av * b[j];
        }
    }
}

static void mm(const float* A, const float* B, float* C, int M, int K, int N, int nt)
{
    mm_args a = {A, B, C, K, N};
    parallel_rows(M, nt, mm_rows, &a);
}

/* out[cols,rows] = in[rows,cols]^T  (utils/Tensor.cpp transpose; value copy only) */
static void transpose(const float* in, float* out, int rows, int cols, int nt)
{
    (void)nt;
    for (int c = 0; c < cols; ++c)
        for (int r = 0; r < rows; ++r) out[(size_t)c * rows + r] = in[(size_t)r * cols + c];
}

/* Y = X*W + b.  layers/LinearLayer.cpp:23-28; bias added after the full product
 * (utils/Tensor.cpp:1499-1507, CPU arm = elementwise a+b with b broadcast). */
static void linear_fwd(const float* X, const float* W, const float* b, float* Y,
                       int rows, int in, int out, int nt)
{
    mm(X, W, Y, rows, in, out, nt);
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < out; ++c) Y[(size_t)r * out + c] = Y[(size_t)r * out + c] + b[c];
}

/* layers/LinearLayer.cpp:36-80: db += column sums (row order, from zero,
 * utils/Tensor.cpp:1610-1616), dW += X^T * dOut, dX = dOut * W^T.  The
 * reference materialises both transposes and calls the same i-k-j product. */
static void linear_bwd(const float* X, const float* W, const float* dOut,
                       float* gW, float* gb, float* dX, int rows, int in, int out, int nt)
{
    if (gb) {
        float* s = (float*)calloc((size_t)out, sizeof(float));
        for (int r = 0; r < rows; ++r)
            for (int c = 0; c < out; ++c) s[c] += dOut[(size_t)r * out + c];
        for (int c = 0; c < out; ++c) gb[c] += s[c];
        free(s);
    }
    if (gW) {
        float* XT = (float*)malloc((size_t)in * rows * sizeof(float));
        float* dW = (float*)malloc((size_t)in * out * sizeof(float));
        transpose(X, XT, rows, in, nt);
        mm(XT, dOut, dW, in, rows, out, nt);
        for (size_t i = 0; i < (size_t)in * out; ++i) gW[i] += dW[i];
        free(XT);
        free(dW);
    }
    if (dX) {
        float* WT = (float*)malloc((size_t)in * out * sizeof(float));
        transpose(W, WT, in, out, nt);
        mm(dOut, WT, dX, rows, out, in, nt);
        free(WT);
    }
}

/* utils/Tensor.cpp:850-883: max-subtracted softmax, inv = 1/max(sum,1e-15),
 * then clamp to [1e-7, 1]. */
static void softmax_clamped(const float* logits, float* probs, int rows, int V)
{
    for (int i = 0; i < rows; ++i) {
        const float* l = logits + (size_t)i * V;
        float* p = probs + (size_t)i * V;
        float mx = l[0];
        for (int v = 1; v < V; ++v)
            if (l[v] > mx) mx = l[v];
        float sum = 0.0f;
        for (int v = 0; v < V; ++v) {
            float e = expf(l[v] - mx);
            p[v] = e;
            sum += e;
        }
        float inv = 1.0f / fmaxf(sum, 1e-15f);
        for (int v = 0; v < V; ++v) p[v] = fminf(fmaxf(p[v] * inv, 1e-7f), 1.0f);
    }
}

/* utils/Tensor.cpp:1296-1334: insertion top-k, strict '>' so that equal values
 * keep the lower expert index first; values are not renormalised. */
static void top_k(const float* probs, int32_t* idx, float* val, int rows, int E, int k)
{
    for (int t = 0; t < rows; ++t) {
        const float* p = probs + (size_t)t * E;
        float* v = val + (size_t)t * k;
        int32_t* ix = idx + (size_t)t * k;
        for (int i = 0; i < k; ++i) {
            v[i] = -1e9f;
            ix[i] = -1;
        }
        for (int e = 0; e < E; ++e) {
            float x = p[e];
            if (x > v[k - 1]) {
                int pos = k - 1;
                while (pos > 0 && x > v[pos - 1]) {
                    v[pos] = v[pos - 1];
                    ix[pos] = ix[pos - 1];
                    pos--;
                }
                v[pos] = x;
                ix[pos] = e;
            }
        }
    }
}

typedef struct {
    float *logits, *probs, *top_p;
    int32_t *top_idx, *counts, *offsets, *map;
} route_bufs;

/* layers/MoELayer.cpp:52-83: router linear, softmax, top-k, histogram
 * (utils/Tensor.cpp:1336-1352), exclusive prefix sum (MoELayer.cpp:70-75) and
 * the stable slot assignment of moe_gather (utils/Tensor.cpp:1368-1381). */
static void route(const moe_oracle_dims* d, const moe_oracle_inputs* in, route_bufs* rb, int nt)
{
    const int N = d->n_tokens, C = d->C, E = d->E, k = d->k, R = N * k;
    linear_fwd(in->x, in->params[0], in->params[1], rb->logits, N, C, E, nt);
    softmax_clamped(rb->logits, rb->probs, N, E);
    top_k(rb->probs, rb->top_idx, rb->top_p, N, E, k);
    for (int e = 0; e < E; ++e) rb->counts[e] = 0;
    for (int i = 0; i < R; ++i) {
        int e = rb->top_idx[i];
        if (e >= 0 && e < E) rb->counts[e] += 1;
    }
    int run = 0;
    for (int e = 0; e < E; ++e) {
        rb->offsets[e] = run;
        run += rb->counts[e];
    }
    int32_t* cur = (int32_t*)malloc((size_t)E * sizeof(int32_t));
    memcpy(cur, rb->offsets, (size_t)E * sizeof(int32_t));
    for (int i = 0; i < R; ++i) {
        int e = rb->top_idx[i];
        if (e >= 0) rb->map[cur[e]++] = i;
    }
    free(cur);
}

static route_bufs route_alloc(const moe_oracle_dims* d)
{
    const size_t N = d->n_tokens, E = d->E, k = d->k;
    route_bufs rb;
    rb.logits = (float*)malloc(N * E * sizeof(float));
    rb.probs = (float*)malloc(N * E * sizeof(float));
    rb.top_p = (float*)malloc(N * k * sizeof(float));
    rb.top_idx = (int32_t*)malloc(N * k * sizeof(int32_t));
    rb.counts = (int32_t*)malloc(E * sizeof(int32_t));
    rb.offsets = (int32_t*)malloc(E * sizeof(int32_t));
    rb.map = (int32_t*)malloc(N * k * sizeof(int32_t));
    return rb;
}

static void route_export(const moe_oracle_dims* d, const route_bufs* rb, moe_oracle_outputs* out)
{
    const size_t N = d->n_tokens, E = d->E, k = d->k;
    if (out->logits) memcpy(out->logits, rb->logits, N * E * sizeof(float));
    if (out->probs) memcpy(out->probs, rb->probs, N * E * sizeof(float));
    if (out->top_p) memcpy(out->top_p, rb->top_p, N * k * sizeof(float));
    if (out->top_idx) memcpy(out->top_idx, rb->top_idx, N * k * sizeof(int32_t));
    if (out->counts) memcpy(out->counts, rb->counts, E * sizeof(int32_t));
    if (out->offsets) memcpy(out->offsets, rb->offsets, E * sizeof(int32_t));
    if (out->map) memcpy(out->map, rb->map, N * k * sizeof(int32_t));
}

static void route_free(route_bufs* rb)
{
    free(rb->logits);
    free(rb->probs);
    free(rb->top_p);
    free(rb->top_idx);
    free(rb->counts);
    free(rb->offsets);
    free(rb->map);
}

int moe_oracle_route(const moe_oracle_dims* d, const moe_oracle_inputs* in,
                     moe_oracle_outputs* out, int n_threads)
{
    if (!d || !in || !out || d->k > d->E || d->k < 1) return 1;
    route_bufs rb = route_alloc(d);
    route(d, in, &rb, n_threads < 1 ? 1 : n_threads);
    route_export(d, &rb, out);
    route_free(&rb);
    return 0;
}

int moe_oracle_run(const moe_oracle_dims* d, const moe_oracle_inputs* in,
                   moe_oracle_outputs* out, int n_threads)
{
    if (!d || !in || !out || d->k > d->E || d->k < 1) return 1;
    const int nt = n_threads < 1 ? 1 : n_threads;
    const int N = d->n_tokens, C = d->C, H = d->H, E = d->E, k = d->k, R = N * k;
    const float* const* P = in->params;

    route_bufs rb = route_alloc(d);
    route(d, in, &rb, nt);
    route_export(d, &rb, out);

    /* moe_gather row copies, utils/Tensor.cpp:1376-1379 */
    float* Xg = (float*)malloc((size_t)R * C * sizeof(float));
    for (int s = 0; s < R; ++s)
        memcpy(Xg + (size_t)s * C, in->x + (size_t)(rb.map[s] / k) * C, (size_t)C * sizeof(float));

    /* Expert loop, layers/MoELayer.cpp:94-118 -> layers/SwiGLU.cpp:23-50.
     * G and U are kept for backward (SwiGLU.cpp:32-33). */
    float* G = (float*)malloc((size_t)R * H * sizeof(float));
    float* U = (float*)malloc((size_t)R * H * sizeof(float));
    float* Hh = (float*)malloc((size_t)R * H * sizeof(float));
    float* Yg = (float*)malloc((size_t)R * C * sizeof(float));
    for (int e = 0; e < E; ++e) {
        const int cnt = rb.counts[e], off = rb.offsets[e];
        if (cnt == 0) continue;
        const float *Wg = P[2 + 6 * e], *bg = P[3 + 6 * e], *Wu = P[4 + 6 * e], *bu = P[5 + 6 * e],
                    *Wd = P[6 + 6 * e], *bd = P[7 + 6 * e];
        float *g = G + (size_t)off * H, *u = U + (size_t)off * H, *h = Hh + (size_t)off * H;
        linear_fwd(Xg + (size_t)off * C, Wg, bg, g, cnt, C, H, nt);
        linear_fwd(Xg + (size_t)off * C, Wu, bu, u, cnt, C, H, nt);
        /* utils/Tensor.cpp:1997-2002 */
        for (size_t i = 0; i < (size_t)cnt * H; ++i) {
            float gs = g[i] / (1.0f + expf(-g[i]));
            h[i] = gs * u[i];
        }
        linear_fwd(h, Wd, bd, Yg + (size_t)off * C, cnt, H, C, nt);
    }
    if (out->gathered_out) memcpy(out->gathered_out, Yg, (size_t)R * C * sizeof(float));

    /* Combine: zero-fill then slot-order scatter-add, layers/MoELayer.cpp:121-123,
     * utils/Tensor.cpp:1398-1406. */
    float* y = (float*)calloc((size_t)N * C, sizeof(float));
    for (int s = 0; s < R; ++s) {
        const int flat = rb.map[s], tok = flat / k;
        const float p = rb.top_p[flat];
        for (int c = 0; c < C; ++c) y[(size_t)tok * C + c] += Yg[(size_t)s * C + c] * p;
    }
    if (out->y) memcpy(out->y, y, (size_t)N * C * sizeof(float));
    free(y);

    if (in->dy) {
        const float* dy = in->dy;
        /* utils/Tensor.cpp:1424-1436 */
        float* dYg = (float*)malloc((size_t)R * C * sizeof(float));
        float* dtp = (float*)calloc((size_t)N * k, sizeof(float));
        for (int s = 0; s < R; ++s) {
            const int flat = rb.map[s], tok = flat / k;
            const float p = rb.top_p[flat];
            float dot = 0.0f;
            for (int c = 0; c < C; ++c) {
                dYg[(size_t)s * C + c] = dy[(size_t)tok * C + c] * p;
                dot += Yg[(size_t)s * C + c] * dy[(size_t)tok * C + c];
            }
            dtp[flat] = dot;
        }
        if (out->d_top_p) memcpy(out->d_top_p, dtp, (size_t)N * k * sizeof(float));

        /* Expert backward, layers/MoELayer.cpp:159-181 -> layers/SwiGLU.cpp:57-96 */
        float* dXg = (float*)malloc((size_t)R * C * sizeof(float));
        float* dH = (float*)malloc((size_t)R * H * sizeof(float));
        float* dU = (float*)malloc((size_t)R * H * sizeof(float));
        float* dG = (float*)malloc((size_t)R * H * sizeof(float));
        float* dXa = (float*)malloc((size_t)R * C * sizeof(float));
        float* dXb = (float*)malloc((size_t)R * C * sizeof(float));
        for (int e = 0; e < E; ++e) {
            const int cnt = rb.counts[e], off = rb.offsets[e];
            if (cnt == 0) continue;
            const float *Wg = P[2 + 6 * e], *Wu = P[4 + 6 * e], *Wd = P[6 + 6 * e];
            float* const* gr = out->grads;
            float *g = G + (size_t)off * H, *u = U + (size_t)off * H, *h = Hh + (size_t)off * H;
            float *dh = dH + (size_t)off * H, *du = dU + (size_t)off * H, *dg = dG + (size_t)off * H;
            const float* dyg = dYg + (size_t)off * C;
            linear_bwd(h, Wd, dyg, gr ? gr[6 + 6 * e] : NULL, gr ? gr[7 + 6 * e] : NULL, dh, cnt, H, C, nt);
            /* utils/Tensor.cpp:2020-2027 */
            for (size_t i = 0; i < (size_t)cnt * H; ++i) {
                float dd = dh[i], uu = u[i], gg = g[i];
                float sig = 1.0f / (1.0f + expf(-gg));
                du[i] = dd * (gg * sig);
                dg[i] = (dd * uu) * (sig * (1.0f + gg * (1.0f - sig)));
            }
            const float* xg = Xg + (size_t)off * C;
            float *da = dXa + (size_t)off * C, *db = dXb + (size_t)off * C;
            linear_bwd(xg, Wg, dg, gr ? gr[2 + 6 * e] : NULL, gr ? gr[3 + 6 * e] : NULL, da, cnt, C, H, nt);
            linear_bwd(xg, Wu, du, gr ? gr[4 + 6 * e] : NULL, gr ? gr[5 + 6 * e] : NULL, db, cnt, C, H, nt);
            /* layers/SwiGLU.cpp:90 */
            for (size_t i = 0; i < (size_t)cnt * C; ++i) dXg[(size_t)off * C + i] = da[i] + db[i];
        }
        free(dH);
        free(dU);
        free(dG);
        free(dXa);
        free(dXb);

        /* layers/MoELayer.cpp:184-186, utils/Tensor.cpp:1451-1458 */
        float* dx = (float*)calloc((size_t)N * C, sizeof(float));
        for (int s = 0; s < R; ++s) {
            const int tok = rb.map[s] / k;
            for (int c = 0; c < C; ++c) dx[(size_t)tok * C + c] += dXg[(size_t)s * C + c];
        }
        free(dXg);
        free(dYg);

        /* layers/MoELayer.cpp:189-204: scatter d_top_p into [N,E], then add the
         * load-balance term alpha*E*f_e/N to every token. */
        float* dP = (float*)calloc((size_t)N * E, sizeof(float));
        for (int i = 0; i < R; ++i) dP[(size_t)(i / k) * E + rb.top_idx[i]] = dtp[i];
        for (int e = 0; e < E; ++e) {
            float f = (float)rb.counts[e] / (float)N;
            float lb = (d->alpha * E * f) / (float)N;
            for (int t = 0; t < N; ++t) dP[(size_t)t * E + e] = dP[(size_t)t * E + e] + lb;
        }
        free(dtp);
        /* utils/Tensor.cpp:890-907 */
        float* dL = (float*)malloc((size_t)N * E * sizeof(float));
        for (int t = 0; t < N; ++t) {
            const float* p = rb.probs + (size_t)t * E;
            const float* dp = dP + (size_t)t * E;
            float dot = 0.0f;
            for (int e = 0; e < E; ++e) dot += dp[e] * p[e];
            for (int e = 0; e < E; ++e) dL[(size_t)t * E + e] = p[e] * (dp[e] - dot);
        }
        free(dP);
        if (out->dlogits) memcpy(out->dlogits, dL, (size_t)N * E * sizeof(float));
        /* layers/MoELayer.cpp:212-218 */
        float* rdx = (float*)malloc((size_t)N * C * sizeof(float));
        linear_bwd(in->x, P[0], dL, out->grads ? out->grads[0] : NULL, out->grads ? out->grads[1] : NULL,
                   rdx, N, C, E, nt);
        for (size_t i = 0; i < (size_t)N * C; ++i) dx[i] = dx[i] + rdx[i];
        free(rdx);
        free(dL);
        if (out->dx) memcpy(out->dx, dx, (size_t)N * C * sizeof(float));
        free(dx);
    }

    free(Xg);
    free(G);
    free(U);
    free(Hh);
    free(Yg);
    route_free(&rb);
    return 0;
}

/* Timed CPU baseline of the restatement: `iters` runs of forward (+ backward
 * when dy is given); seconds[i] receives run i.  Gradients are accumulated
 * into scratch buffers that are cleared, untimed, before each run. */
int moe_oracle_bench(const moe_oracle_dims* d, const moe_oracle_inputs* in, int iters, double* seconds,
                     int n_threads)
{
    const int np = 2 + 6 * d->E;
    float** grads = (float**)calloc((size_t)np, sizeof(float*));
    size_t* sizes = (size_t*)calloc((size_t)np, sizeof(size_t));
    for (int i = 0; i < np; ++i) {
        size_t n;
        if (i == 0) n = (size_t)d->C * d->E;
        else if (i == 1) n = (size_t)d->E;
        else {
            int r = (i - 2) % 6;
            n = (r == 0 || r == 2 || r == 4) ? (size_t)d->C * d->H : (r == 5 ? (size_t)d->C : (size_t)d->H);
        }
        sizes[i] = n;
        grads[i] = (float*)malloc(n * sizeof(float));
    }
    float* y = (float*)malloc((size_t)d->n_tokens * d->C * sizeof(float));
    float* dx = (float*)malloc((size_t)d->n_tokens * d->C * sizeof(float));
    int rc = 0;
    for (int it = 0; it < iters && rc == 0; ++it) {
        for (int i = 0; i < np; ++i) memset(grads[i], 0, sizes[i] * sizeof(float));
        moe_oracle_outputs out;
        memset(&out, 0, sizeof(out));
        out.y = y;
        out.dx = dx;
        out.grads = grads;
        struct timespec t0, t1;
        clock_gettime(CLOCK_MONOTONIC, &t0);
        rc = moe_oracle_run(d, in, &out, n_threads);
        clock_gettime(CLOCK_MONOTONIC, &t1);
        seconds[it] = (double)(t1.tv_sec - t0.tv_sec) + 1e-9 * (double)(t1.tv_nsec - t0.tv_nsec);
    }
    for (int i = 0; i < np; ++i) free(grads[i]);
    free(grads);
    free(sizes);
    free(y);
    free(dx);
    return rc;
}

/* utils/Tensor.cpp:683-699: bias-correction scales from powf once per step, then per element
 * m = b1*m + (1-b1)*g;  v = b2*v + (1-b2)*g*g;  w -= lr*wd*w;  w -= lr*(m*ms) / (sqrt(v*vs) + eps),
 * every operation a separate FP32 rounding (the oracle is built with -ffp-contract=off). */
int moe_oracle_adamw(float* w, const float* g, float* m, float* v, long n, float lr, float beta1, float beta2,
                     float eps, float weight_decay, int t)
{
    if (!w || !g || !m || !v || n < 0 || t < 1) return 1;
    const float ms = 1.0f / (1.0f - powf(beta1, (float)t));
    const float vs = 1.0f / (1.0f - powf(beta2, (float)t));
    for (long i = 0; i < n; ++i) {
        const float gi = g[i];
        m[i] = beta1 * m[i] + (1.0f - beta1) * gi;
        v[i] = beta2 * v[i] + (1.0f - beta2) * gi * gi;
        const float m_hat = m[i] * ms;
        const float v_hat = v[i] * vs;
        w[i] -= lr * weight_decay * w[i];
        w[i] -= lr * m_hat / (sqrtf(v_hat) + eps);
    }
    return 0;
}
