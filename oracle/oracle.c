/* CPU oracle for the token-loop hot path.  TEST INFRASTRUCTURE ONLY: nothing in
 * the shipped library links, loads or calls this file (see oracle.h).
 *
 * Arithmetic contract restated from the reference CPU build: tensors are fp32,
 * every dot product / norm statistic / softmax accumulates in fp64 in index
 * order and rounds once to fp32, element-wise fp32 expressions are evaluated
 * without fused multiply-add (build with -ffp-contract=off), ties go to the
 * lowest index.  Where a loop is parallelised or blocked here, every output
 * element still sees exactly the reference's sequence of operations, so results
 * are bit-identical to the reference build.
 */
#define _POSIX_C_SOURCE 200809L
#include "oracle.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static void *xmalloc(size_t n) {
    void *p = malloc(n ? n : 1);
    if (!p) { fprintf(stderr, "oracle: out of memory (%zu bytes)\n", n); exit(1); }
    return p;
}
static void *xcalloc(size_t n, size_t s) {
    void *p = calloc(n ? n : 1, s ? s : 1);
    if (!p) { fprintf(stderr, "oracle: out of memory\n"); exit(1); }
    return p;
}
static float *falloc(size_t n) { return (float *)xmalloc(n * sizeof(float)); }

/* ====================================================================== */
/* layer kernels                                                          */
/* ====================================================================== */

/* y = x W^T + b, W:[M][K].  reference src/kernels.c:38-54.  Eight outputs are
 * carried at once for instruction-level parallelism; each keeps its own fp64
 * accumulator and its own k order. */
void orc_linear(const float *x, const float *W, const float *b, float *y,
                int64_t batch, int M, int K) {
#pragma omp parallel for schedule(static) if (batch * M > 512)
    for (int64_t r = 0; r < batch; r++) {
        const float *xr = x + r * K;
        float *yr = y + r * M;
        int m0 = 0;
        for (; m0 + 8 <= M; m0 += 8) {
            double a0, a1, a2, a3, a4, a5, a6, a7;
            if (b) { a0 = b[m0]; a1 = b[m0 + 1]; a2 = b[m0 + 2]; a3 = b[m0 + 3];
                     a4 = b[m0 + 4]; a5 = b[m0 + 5]; a6 = b[m0 + 6]; a7 = b[m0 + 7]; }
            else a0 = a1 = a2 = a3 = a4 = a5 = a6 = a7 = 0.0;
            const float *w0 = W + (int64_t)m0 * K;
            for (int k = 0; k < K; k++) {
                double xv = (double)xr[k];
                a0 += xv * w0[k];
                a1 += xv * w0[(int64_t)K + k];
                a2 += xv * w0[(int64_t)2 * K + k];
                a3 += xv * w0[(int64_t)3 * K + k];
                a4 += xv * w0[(int64_t)4 * K + k];
                a5 += xv * w0[(int64_t)5 * K + k];
                a6 += xv * w0[(int64_t)6 * K + k];
                a7 += xv * w0[(int64_t)7 * K + k];
            }
            yr[m0] = (float)a0; yr[m0 + 1] = (float)a1; yr[m0 + 2] = (float)a2;
            yr[m0 + 3] = (float)a3; yr[m0 + 4] = (float)a4; yr[m0 + 5] = (float)a5;
            yr[m0 + 6] = (float)a6; yr[m0 + 7] = (float)a7;
        }
        for (; m0 < M; m0++) {
            double acc = b ? b[m0] : 0.0;
            const float *wr = W + (int64_t)m0 * K;
            for (int k = 0; k < K; k++) acc += (double)xr[k] * wr[k];
            yr[m0] = (float)acc;
        }
    }
}

/* reference src/kernels.c:101-148 (eps 1e-6 default, 1e-5 for GPT-2) */
void orc_layernorm(const float *x, const float *w, const float *b, float *y,
                   int64_t rows, int C, double eps) {
#pragma omp parallel for schedule(static) if (rows > 4)
    for (int64_t r = 0; r < rows; r++) {
        const float *xr = x + r * C;
        float *yr = y + r * C;
        double mean = 0;
        for (int c = 0; c < C; c++) mean += xr[c];
        mean /= C;
        double var = 0;
        for (int c = 0; c < C; c++) { double d = xr[c] - mean; var += d * d; }
        var /= C;
        double inv = 1.0 / sqrt(var + eps);
        for (int c = 0; c < C; c++) {
            float n = (float)((xr[c] - mean) * inv);
            yr[c] = n * (w ? w[c] : 1.0f) + (b ? b[c] : 0.0f);
        }
    }
}

/* reference src/kernels.c:150-162 (eps fixed at 1e-6) */
void orc_rmsnorm(const float *x, const float *w, float *y, int64_t rows, int C) {
#pragma omp parallel for schedule(static) if (rows > 4)
    for (int64_t r = 0; r < rows; r++) {
        const float *xr = x + r * C;
        float *yr = y + r * C;
        double ms = 0;
        for (int c = 0; c < C; c++) ms += (double)xr[c] * xr[c];
        ms /= C;
        float s = (float)(1.0 / sqrt(ms + 1e-6));
        for (int c = 0; c < C; c++) yr[c] = xr[c] * s * (w ? w[c] : 1.0f);
    }
}

/* reference src/kernels.c:185-194 */
void orc_gelu(const float *x, float *y, int64_t n) {
    for (int64_t i = 0; i < n; i++) {
        float v = x[i];
        y[i] = 0.5f * v * (1.0f + erff(v * 0.7071067811865475f));
    }
}
/* reference src/kernels.c:207-218 (the CPU build evaluates gelu_new in fp64) */
void orc_gelu_tanh(const float *x, float *y, int64_t n) {
    for (int64_t i = 0; i < n; i++) {
        double v = x[i];
        double t = 0.7978845608028654 * (v + 0.044715 * v * v * v);
        y[i] = (float)(0.5 * v * (1.0 + tanh(t)));
    }
}
/* reference src/kernels.c:220-226 */
void orc_silu(const float *x, float *y, int64_t n) {
    for (int64_t i = 0; i < n; i++) { float v = x[i]; y[i] = v / (1.0f + expf(-v)); }
}
/* reference src/kernels.c:228-240 */
void orc_softmax(const float *x, float *y, int64_t rows, int C) {
    for (int64_t r = 0; r < rows; r++) {
        const float *xr = x + r * C; float *yr = y + r * C;
        float mx = xr[0];
        for (int c = 1; c < C; c++) if (xr[c] > mx) mx = xr[c];
        double s = 0;
        for (int c = 0; c < C; c++) s += exp((double)xr[c] - mx);
        for (int c = 0; c < C; c++) yr[c] = (float)(exp((double)xr[c] - mx) / s);
    }
}

/* Half-split rotation with pair-duplicated tables [T][hd], in place; row r uses
 * table row r % T.  reference src/kernels.c:249-264. */
void orc_rope(float *x, const float *cs, const float *sn, int64_t rows, int T, int hd) {
    int h = hd / 2;
    for (int64_t r = 0; r < rows; r++) {
        int t = (int)(r % T);
        float *xr = x + r * hd;
        const float *co = cs + (int64_t)t * hd, *si = sn + (int64_t)t * hd;
        for (int d = 0; d < h; d++) {
            float a = xr[d], b = xr[d + h];
            xr[d] = a * co[d] + (-b) * si[d];
            xr[d + h] = b * co[d + h] + a * si[d + h];
        }
    }
}

/* softmax(q k^T * scale + mask) v with an additive [Tq][Tkv] mask; q:[B][Hq][Tq][hd],
 * k,v:[B][Hkv][Tkv][hd].  Two passes over the keys (max, then accumulate), the
 * output accumulated in fp32 and normalised at the end.
 * reference src/kernels.c:423-507. */
void orc_sdpa(const float *q, const float *k, const float *v, const float *mask,
              float *out, int B, int Hq, int Hkv, int Tq, int Tkv, int hd) {
    float scale = 1.0f / sqrtf((float)hd);
    int rep = Hq / Hkv;
#pragma omp parallel for collapse(2) schedule(static) if ((int64_t)B * Hq * Tq > 4)
    for (int b = 0; b < B; b++) for (int h = 0; h < Hq; h++) {
        int kvh = h / rep;
        const float *kb = k + ((int64_t)b * Hkv + kvh) * Tkv * hd;
        const float *vb = v + ((int64_t)b * Hkv + kvh) * Tkv * hd;
        for (int tq = 0; tq < Tq; tq++) {
            const float *qr = q + (((int64_t)b * Hq + h) * Tq + tq) * hd;
            float *o = out + (((int64_t)b * Hq + h) * Tq + tq) * hd;
            double mx = -1e300, den = 0;
            for (int tk = 0; tk < Tkv; tk++) {
                const float *kr = kb + (int64_t)tk * hd;
                double s = 0;
                for (int d = 0; d < hd; d++) s += (double)qr[d] * kr[d];
                s *= scale;
                if (mask) s += mask[(int64_t)tq * Tkv + tk];
                if (s > mx) mx = s;
            }
            for (int d = 0; d < hd; d++) o[d] = 0;
            for (int tk = 0; tk < Tkv; tk++) {
                const float *kr = kb + (int64_t)tk * hd;
                double s = 0;
                for (int d = 0; d < hd; d++) s += (double)qr[d] * kr[d];
                s *= scale;
                if (mask) s += mask[(int64_t)tq * Tkv + tk];
                double p = exp(s - mx);
                den += p;
                const float *vr = vb + (int64_t)tk * hd;
                float pf = (float)p;
                for (int d = 0; d < hd; d++) o[d] += pf * vr[d];
            }
            double inv = 1.0 / den;
            for (int d = 0; d < hd; d++) o[d] = (float)(o[d] * inv);
        }
    }
}

/* NCL convolution. reference src/kernels.c:546-566 */
void orc_conv1d(const float *x, const float *W, const float *b, float *y,
                int N, int Cin, int Cout, int T, int K, int stride, int pad) {
    int64_t Tout = (T + 2 * pad - K) / stride + 1;
#pragma omp parallel for collapse(2) schedule(static) if ((int64_t)N * Cout > 2)
    for (int n = 0; n < N; n++) for (int co = 0; co < Cout; co++)
        for (int64_t t = 0; t < Tout; t++) {
            double acc = b ? b[co] : 0.0;
            for (int ci = 0; ci < Cin; ci++) for (int kk = 0; kk < K; kk++) {
                int ti = (int)(t * stride + kk - pad);
                if (ti < 0 || ti >= T) continue;
                acc += (double)x[((int64_t)n * Cin + ci) * T + ti] *
                       W[((int64_t)co * Cin + ci) * K + kk];
            }
            y[((int64_t)n * Cout + co) * Tout + t] = (float)acc;
        }
}

/* Transposed convolution, weight [Cin][Cout][K], no padding.
 * reference src/kernels.c:568-591 */
void orc_convT1d(const float *x, const float *W, const float *b, float *y,
                 int N, int Cin, int Cout, int T, int K, int stride) {
    int64_t Tout = (int64_t)(T - 1) * stride + K;
#pragma omp parallel for collapse(2) schedule(static) if ((int64_t)N * Cout > 2)
    for (int n = 0; n < N; n++) for (int co = 0; co < Cout; co++)
        for (int64_t t = 0; t < Tout; t++) {
            double acc = b ? b[co] : 0.0;
            for (int ci = 0; ci < Cin; ci++) for (int kk = 0; kk < K; kk++) {
                int num = (int)(t - kk);
                if (num < 0 || num % stride != 0) continue;
                int ti = num / stride;
                if (ti >= T) continue;
                acc += (double)x[((int64_t)n * Cin + ci) * T + ti] *
                       W[((int64_t)ci * Cout + co) * K + kk];
            }
            y[((int64_t)n * Cout + co) * Tout + t] = (float)acc;
        }
}

/* affine-free GroupNorm on NCL, eps 1e-5. reference src/kernels.c:618-641 */
void orc_groupnorm(const float *x, float *y, int N, int G, int C, int T) {
    int Cg = C / G;
    for (int n = 0; n < N; n++) for (int g = 0; g < G; g++) {
        const float *xb = x + ((int64_t)n * C + (int64_t)g * Cg) * T;
        float *yb = y + ((int64_t)n * C + (int64_t)g * Cg) * T;
        int64_t cnt = (int64_t)Cg * T;
        double mean = 0;
        for (int64_t i = 0; i < cnt; i++) mean += xb[i];
        mean /= cnt;
        double var = 0;
        for (int64_t i = 0; i < cnt; i++) { double d = xb[i] - mean; var += d * d; }
        var /= cnt;
        double inv = 1.0 / sqrt(var + 1e-5);
        for (int64_t i = 0; i < cnt; i++) yb[i] = (float)((xb[i] - mean) * inv);
    }
}

/* ATen "area" resampling on NCL. reference src/kernels.c:681-700 */
void orc_interp_area(const float *x, float *y, int N, int C, int Tin, int Tout) {
    for (int64_t nc = 0; nc < (int64_t)N * C; nc++) {
        const float *xr = x + nc * Tin;
        float *yr = y + nc * Tout;
        for (int t = 0; t < Tout; t++) {
            int64_t s = (int64_t)((double)t * Tin / Tout);
            int64_t e = (int64_t)ceil((double)(t + 1) * Tin / Tout);
            if (e <= s) e = s + 1;
            if (s < 0) s = 0;
            if (e > Tin) e = Tin;
            double acc = 0;
            for (int64_t k = s; k < e; k++) acc += xr[k];
            yr[t] = (float)(acc / (e - s));
        }
    }
}

/* ATen "linear", align_corners=False, with a mean fallback when either length
 * is 1. reference src/kernels.c:702-727 */
void orc_interp_linear(const float *x, float *y, int N, int C, int Tin, int Tout) {
    for (int64_t nc = 0; nc < (int64_t)N * C; nc++) {
        const float *xr = x + nc * Tin;
        float *yr = y + nc * Tout;
        if (Tout == 1 || Tin == 1) {
            double acc = 0;
            for (int k = 0; k < Tin; k++) acc += xr[k];
            for (int t = 0; t < Tout; t++) yr[t] = (float)(acc / Tin);
            continue;
        }
        double scale = (double)Tin / Tout;
        for (int t = 0; t < Tout; t++) {
            double src = (t + 0.5) * scale - 0.5;
            int64_t s0 = (int64_t)floor(src);
            double w1 = src - s0, w0 = 1.0 - w1;
            double v0 = xr[s0 < 0 ? 0 : (s0 >= Tin ? Tin - 1 : s0)];
            int64_t s1 = s0 + 1;
            double v1 = xr[s1 < 0 ? 0 : (s1 >= Tin ? Tin - 1 : s1)];
            yr[t] = (float)(w0 * v0 + w1 * v1);
        }
    }
}

/* d2[i][j] = |a_i - b_j|^2. reference src/kernels.c:753-770 */
void orc_l2sq(const float *a, const float *b, float *d2, int64_t rows, int64_t cols, int C) {
#pragma omp parallel for schedule(static) if (rows * cols > 4096)
    for (int64_t i = 0; i < rows; i++)
        for (int64_t j = 0; j < cols; j++) {
            double s = 0;
            for (int c = 0; c < C; c++) {
                double d = (double)a[i * C + c] - b[j * C + c];
                s += d * d;
            }
            d2[i * cols + j] = (float)s;
        }
}

/* first maximum wins. reference src/kernels.c:731-735 */
int orc_argmax(const float *x, int n) {
    int bi = 0; float bv = x[0];
    for (int i = 1; i < n; i++) if (x[i] > bv) { bv = x[i]; bi = i; }
    return bi;
}

/* xorshift64*. reference src/kernels.c:774-784 */
uint64_t orc_rng_next(uint64_t *state) {
    uint64_t x = *state;
    x ^= x >> 12; x ^= x << 25; x ^= x >> 27;
    *state = x;
    return x * 0x2545F4914F6CDD1DULL;
}
static double rng_unit(uint64_t *rng) {
    return (double)(orc_rng_next(rng) >> 11) * (1.0 / 9007199254740992.0);
}

static const float *g_sort_vals;   /* sampling is serial: one global stream */
static int by_value_desc(const void *a, const void *b) {
    float va = g_sort_vals[*(const int *)a], vb = g_sort_vals[*(const int *)b];
    return (va < vb) - (va > vb);
}

/* temperature / top-k / nucleus sampling, one uniform draw per call when
 * temp > 0, none when greedy. reference src/kernels.c:794-825 */
int orc_sample_topkp(const float *logits, int V, float temp, int top_k, float top_p,
                     uint64_t *rng) {
    if (!(temp > 0)) return orc_argmax(logits, V);
    float *work = falloc(V);
    int *ord = (int *)xmalloc((size_t)V * sizeof(int));
    double *probs = (double *)xmalloc((size_t)V * sizeof(double));
    for (int i = 0; i < V; i++) { work[i] = logits[i] / temp; ord[i] = i; }
    g_sort_vals = work;
    qsort(ord, V, sizeof(int), by_value_desc);
    int keep = (top_k > 0) ? (top_k < V ? top_k : V) : V;
    for (int r = keep; r < V; r++) work[ord[r]] = -INFINITY;
    double mx = work[ord[0]], den = 0;
    for (int r = 0; r < keep; r++) { probs[r] = exp((double)work[ord[r]] - mx); den += probs[r]; }
    for (int r = 0; r < keep; r++) probs[r] /= den;
    double cum = 0;
    int nkeep = keep;
    for (int r = 0; r < keep; r++) {
        if (cum - probs[r] > top_p) { nkeep = r; break; }
        cum += probs[r];
    }
    den = 0;
    for (int r = 0; r < nkeep; r++) den += probs[r];
    double u = rng_unit(rng) * den, acc = 0;
    int pick = ord[nkeep - 1];
    for (int r = 0; r < nkeep; r++) { acc += probs[r]; if (u <= acc) { pick = ord[r]; break; } }
    free(work); free(ord); free(probs);
    return pick;
}

/* ====================================================================== */
/* weight store + config                                                  */
/* ====================================================================== */

typedef struct { char name[256]; float *data; int64_t shape[4]; int ndim; int64_t n; } OT;
typedef struct { OT *items; int count; } Store;

/* NCM1 container. reference src/tensor.c:70-128 */
static int store_load(Store *s, const char *path) {
    FILE *f = fopen(path, "rb");
    if (!f) { fprintf(stderr, "oracle: cannot open %s\n", path); return -1; }
    char magic[4];
    uint32_t count = 0;
    if (fread(magic, 1, 4, f) != 4 || memcmp(magic, "NCM1", 4) != 0 ||
        fread(&count, 4, 1, f) != 1) { fclose(f); return -1; }
    s->items = (OT *)xcalloc(count, sizeof(OT));
    s->count = 0;
    for (uint32_t i = 0; i < count; i++) {
        OT *t = &s->items[i];
        unsigned char nl = 0, nd = 0;
        if (fread(&nl, 1, 1, f) != 1 || fread(t->name, 1, nl, f) != nl) goto bad;
        t->name[nl] = 0;
        if (fread(&nd, 1, 1, f) != 1 || nd > 4) goto bad;
        t->ndim = nd; t->n = 1;
        for (int d = 0; d < nd; d++) {
            uint32_t v;
            if (fread(&v, 4, 1, f) != 1) goto bad;
            t->shape[d] = v; t->n *= v;
        }
        uint64_t nbytes = 0;
        if (fread(&nbytes, 8, 1, f) != 1 || nbytes != (uint64_t)t->n * 4) goto bad;
        t->data = falloc((size_t)t->n);
        if (fread(t->data, 1, nbytes, f) != nbytes) goto bad;
        s->count++;
    }
    fclose(f);
    return 0;
bad:
    fclose(f);
    fprintf(stderr, "oracle: %s: malformed NCM1 file\n", path);
    return -1;
}
static void store_free(Store *s) {
    for (int i = 0; i < s->count; i++) free(s->items[i].data);
    free(s->items);
    s->items = NULL; s->count = 0;
}
static OT *store_get(const Store *s, const char *name) {
    for (int i = 0; i < s->count; i++)
        if (strcmp(s->items[i].name, name) == 0) return &s->items[i];
    return NULL;
}
static OT *store_getf(const Store *s, const char *fmt, ...) __attribute__((format(printf, 2, 3)));
#include <stdarg.h>
static OT *store_getf(const Store *s, const char *fmt, ...) {
    char key[320];
    va_list ap; va_start(ap, fmt); vsnprintf(key, sizeof key, fmt, ap); va_end(ap);
    return store_get(s, key);
}
static OT *store_need(const Store *s, const char *fmt, ...) __attribute__((format(printf, 2, 3)));
static OT *store_need(const Store *s, const char *fmt, ...) {
    char key[320];
    va_list ap; va_start(ap, fmt); vsnprintf(key, sizeof key, fmt, ap); va_end(ap);
    OT *t = store_get(s, key);
    if (!t) { fprintf(stderr, "oracle: missing weight %s\n", key); exit(1); }
    return t;
}
#define DATA(t) ((t) ? (t)->data : NULL)

#define MAXLV 64
typedef struct {
    int n_layer, n_head, n_embd, n_kv_heads, context_length, prefix_len;
    int prefix_pad, query_level0, block_diag, use_rope, rope_base, use_qk_norm;
    double rope_theta;
    int puc_enabled, puc_kernel;
    int shared_head, shared_head_lvl_bias, untied_head_bias, tie_heads;
    int swiglu, geglu, relu2;
    int vocab_size[MAXLV], n_vocab;
    int vq_D, vq_in_vocab, vq_ctx, vq_heads, vq_compression;
    int levels[MAXLV], n_levels, vq_vocab[MAXLV];
    int qr_enabled, qr_share; float qr_ratio;
    int l1_sampling, l1_norm, l1_norm_final, all_sampling, pre_quant_gn, vq_qk_norm;
    int enc_layers, enc_window, enc_convs, enc_conv_kernel, enc_positional;
    int dec_layers, dec_positional;
    int eos_id, pad_id;
} Cfg;

/* booleans may be spelled True/False. reference src/tensor.c:151-156 */
static int conf_int(const char *v) {
    while (*v == ' ') v++;
    if (*v == 'T' || *v == 't') return 1;
    if (*v == 'F' || *v == 'f') return 0;
    return atoi(v);
}
static int conf_list(const char *v, int *out, int cap) {
    int k = 0;
    const char *p = v;
    while (*p && k < cap) {
        while (*p == ' ' || *p == ',') p++;
        if (!*p) break;
        out[k++] = atoi(p);
        while (*p && *p != ',') p++;
    }
    return k;
}

/* flat key=value file, unknown keys ignored. reference src/tensor.c:170-266 */
static int cfg_load(Cfg *c, const char *path) {
    memset(c, 0, sizeof *c);
    c->rope_base = 10000; c->rope_theta = 10000.0; c->n_kv_heads = -1;
    c->prefix_pad = -1; c->eos_id = -1; c->pad_id = -1; c->block_diag = 1;
    FILE *f = fopen(path, "r");
    if (!f) { fprintf(stderr, "oracle: cannot open %s\n", path); return -1; }
    char line[1024];
    struct { const char *key; int *dst; int boolish; } ints[] = {
        {"model.n_layer", &c->n_layer, 1}, {"model.n_head", &c->n_head, 1},
        {"model.n_embd", &c->n_embd, 1}, {"model.context_length", &c->context_length, 1},
        {"model.prefix_len", &c->prefix_len, 1}, {"model.prefix_pad_token_id", &c->prefix_pad, 1},
        {"model.query_level0", &c->query_level0, 1}, {"model.use_rope", &c->use_rope, 1},
        {"model.rope_base", &c->rope_base, 1}, {"model.use_qk_norm", &c->use_qk_norm, 1},
        {"model.n_kv_heads", &c->n_kv_heads, 1}, {"model.puc_enabled", &c->puc_enabled, 1},
        {"model.puc_kernel", &c->puc_kernel, 1}, {"model.shared_output_head", &c->shared_head, 1},
        {"model.shared_head_per_level_bias", &c->shared_head_lvl_bias, 1},
        {"model.untied_head_bias", &c->untied_head_bias, 1},
        {"model.tie_heads_to_codebook", &c->tie_heads, 1},
        {"model.use_swiglu", &c->swiglu, 1}, {"model.use_geglu", &c->geglu, 1},
        {"model.use_relu2", &c->relu2, 1},
        {"vq.embed_dim", &c->vq_D, 0}, {"vq.in_vocab", &c->vq_in_vocab, 0},
        {"vq.context_length", &c->vq_ctx, 0}, {"vq.n_layers", &c->vq_heads, 0},
        {"vq.compression", &c->vq_compression, 0}, {"vq.qr_enabled", &c->qr_enabled, 0},
        {"vq.qr_share", &c->qr_share, 0}, {"vq.l1_sampling", &c->l1_sampling, 0},
        {"vq.l1_norm", &c->l1_norm, 1}, {"vq.l1_norm_final", &c->l1_norm_final, 1},
        {"vq.all_sampling", &c->all_sampling, 0}, {"vq.pre_quant_gn", &c->pre_quant_gn, 0},
        {"vq.qk_norm", &c->vq_qk_norm, 1}, {"vq.enc_layers", &c->enc_layers, 0},
        {"vq.enc_window", &c->enc_window, 0}, {"vq.enc_convs", &c->enc_convs, 0},
        {"vq.enc_conv_kernel", &c->enc_conv_kernel, 0},
        {"vq.enc_positional", &c->enc_positional, 0}, {"vq.dec_layers", &c->dec_layers, 0},
        {"vq.dec_positional", &c->dec_positional, 0},
        {"tok.eos_id", &c->eos_id, 1}, {"tok.pad_id", &c->pad_id, 1},
    };
    while (fgets(line, sizeof line, f)) {
        char *eq = strchr(line, '=');
        if (!eq) continue;
        *eq = 0;
        char *k = line, *v = eq + 1;
        v[strcspn(v, "\r\n")] = 0;
        int done = 0;
        for (size_t i = 0; i < sizeof ints / sizeof ints[0]; i++)
            if (strcmp(k, ints[i].key) == 0) {
                *ints[i].dst = ints[i].boolish ? conf_int(v) : atoi(v);
                done = 1; break;
            }
        if (done) continue;
        if (!strcmp(k, "model.rope_theta")) c->rope_theta = atof(v);
        else if (!strcmp(k, "model.attn_pattern")) c->block_diag = (strcmp(v, "block_diagonal") == 0);
        else if (!strcmp(k, "model.vocab_size")) c->n_vocab = conf_list(v, c->vocab_size, MAXLV);
        else if (!strcmp(k, "vq.levels")) c->n_levels = conf_list(v, c->levels, MAXLV);
        else if (!strcmp(k, "vq.vocab")) conf_list(v, c->vq_vocab, MAXLV);
        else if (!strcmp(k, "vq.qr_ratio")) c->qr_ratio = (float)atof(v);
    }
    fclose(f);
    if (c->n_kv_heads < 0) c->n_kv_heads = c->n_head;
    return 0;
}

/* ====================================================================== */
/* quantizer                                                              */
/* ====================================================================== */

typedef struct {
    int n_levels, *levels, *vocabs, D, L;
    float *E[MAXLV];
    int resi; float resi_ratio; int n_phi;
    float *phiW[MAXLV], *phiB[MAXLV]; double ticks[MAXLV];
    int has_l1, n_down, n_up, l1_norm, l1_norm_final;
    float *downW[16], *downB[16], *upW[16], *upB[16]; int downK[16], upK[16];
    int has_all;
    float *drefW[MAXLV], *drefB[MAXLV], *urefW[MAXLV], *urefB[MAXLV];
} VQ;

struct OrcModel {
    Cfg c;
    Store ws;
    VQ vq;
    /* NCP */
    int P, L, T, lvl_first, n_tgt;
    float **gcos, **gsin;        /* per target level: [P+l][hd] */
    float *rope_cos, *rope_sin;  /* full sequence [P+T][hd] */
    float *lvl_pos;              /* [T][C] */
};

/* binds codebooks, Phi convs, cascade stages and refine convs by name.
 * reference src/vq.c:75-192 */
static void vq_bind(VQ *v, const Cfg *c, const Store *ws) {
    const char *pre = "tok.vq.";
    memset(v, 0, sizeof *v);
    v->n_levels = c->n_levels;
    v->levels = (int *)c->levels; v->vocabs = (int *)c->vq_vocab;
    v->D = c->vq_D; v->L = c->levels[c->n_levels - 1];
    for (int i = 0; i < v->n_levels; i++) v->E[i] = store_need(ws, "%sembeddings.%d.weight", pre, i)->data;
    v->resi = c->qr_enabled && fabsf(c->qr_ratio) > 1e-6f;
    v->resi_ratio = c->qr_ratio;
    if (v->resi) {
        v->n_phi = c->qr_share == 0 ? v->n_levels : (c->qr_share == 1 ? 1 : c->qr_share);
        for (int i = 0; i < v->n_phi; i++) {
            OT *w = store_getf(ws, "%squant_resi.%d.weight", pre, i);
            OT *b = store_getf(ws, "%squant_resi.%d.bias", pre, i);
            if (!w && v->n_phi == 1) w = store_getf(ws, "%squant_resi.weight", pre);
            if (!b && v->n_phi == 1) b = store_getf(ws, "%squant_resi.bias", pre);
            if (!w || !b) { fprintf(stderr, "oracle: missing quant_resi.%d\n", i); exit(1); }
            v->phiW[i] = w->data; v->phiB[i] = b->data;
            v->ticks[i] = (v->n_phi == 4) ? (i + 1.0 / 3.0) / v->n_phi : (i + 0.5) / v->n_phi;
        }
    }
    if (c->l1_sampling) {
        v->has_l1 = 1; v->l1_norm = c->l1_norm; v->l1_norm_final = c->l1_norm_final;
        for (int s = 0; s < 16; s++) {
            OT *t = store_getf(ws, "%slearned_down_l1.%d.weight", pre, s);
            if (t) {
                v->downW[v->n_down] = t->data; v->downK[v->n_down] = (int)t->shape[2];
                v->downB[v->n_down] = store_need(ws, "%slearned_down_l1.%d.bias", pre, s)->data;
                v->n_down++;
            }
            t = store_getf(ws, "%slearned_up_l1.%d.weight", pre, s);
            if (t) {
                v->upW[v->n_up] = t->data; v->upK[v->n_up] = (int)t->shape[2];
                v->upB[v->n_up] = store_need(ws, "%slearned_up_l1.%d.bias", pre, s)->data;
                v->n_up++;
            }
        }
        if (!v->n_down) { fprintf(stderr, "oracle: learned_l1 weights missing\n"); exit(1); }
    }
    if (c->all_sampling) {
        v->has_all = 1;
        for (int i = 1; i <= v->n_levels - 2; i++) {
            OT *t = store_getf(ws, "%slearned_down_refine.%d.weight", pre, i);
            if (t) { v->drefW[i] = t->data; v->drefB[i] = store_need(ws, "%slearned_down_refine.%d.bias", pre, i)->data; }
            t = store_getf(ws, "%slearned_up_refine.%d.weight", pre, i);
            if (t) { v->urefW[i] = t->data; v->urefB[i] = store_need(ws, "%slearned_up_refine.%d.bias", pre, i)->data; }
        }
    }
}

static int vq_total(const VQ *v) {
    int s = 0;
    for (int i = 0; i < v->n_levels; i++) s += v->levels[i];
    return s;
}

/* reference src/vq.c:212-221 */
static int phi_index(const VQ *v, int level) {
    if (v->n_phi == 1) return 0;
    double at = (double)level / (v->n_levels - 1);
    int best = 0; double bd = 1e300;
    for (int j = 0; j < v->n_phi; j++) {
        double d = fabs(v->ticks[j] - at);
        if (d < bd) { bd = d; best = j; }
    }
    return best;
}

/* [B][L][D] <-> [B][D][L] */
static void tr_bld(float *y, const float *x, int B, int L, int D) {
    for (int b = 0; b < B; b++) for (int l = 0; l < L; l++) for (int d = 0; d < D; d++)
        y[((int64_t)b * D + d) * L + l] = x[((int64_t)b * L + l) * D + d];
}

/* y = x + conv3(x) on a [B][L][D] tensor (used by refine convs and post-upsample) */
static void add_conv_bld(float *h, const float *W, const float *bias, int B, int L, int D,
                         int K, int pad) {
    size_t n = (size_t)B * L * D;
    float *bcl = falloc(n), *cv = falloc(n), *back = falloc(n);
    tr_bld(bcl, h, B, L, D);
    orc_conv1d(bcl, W, bias, cv, B, D, D, L, K, 1, pad);
    tr_bld(back, cv, B, D, L);
    for (size_t i = 0; i < n; i++) h[i] += back[i];
    free(bcl); free(cv); free(back);
}

/* h = (1-r) h + r conv3(h). reference src/vq.c:244-268 */
static void apply_phi(const VQ *v, float *h, int B, int L, int level) {
    if (!v->resi) return;
    int j = phi_index(v, level), D = v->D;
    size_t n = (size_t)B * L * D;
    float *bcl = falloc(n), *cv = falloc(n), *back = falloc(n);
    tr_bld(bcl, h, B, L, D);
    orc_conv1d(bcl, v->phiW[j], v->phiB[j], cv, B, D, D, L, 3, 1, 1);
    tr_bld(back, cv, B, D, L);
    float r = v->resi_ratio;
    for (size_t i = 0; i < n; i++) h[i] = (1 - r) * h[i] + r * back[i];
    free(bcl); free(cv); free(back);
}

/* z_rest [B][L][D] -> [B][levels[level]][D]. reference src/vq.c:271-324 */
static void down_for_quant(const VQ *v, const float *z, int B, int Lin, int level, float *out) {
    int D = v->D, tlen = v->levels[level];
    if (level == 0 && v->has_l1) {
        float *cur = falloc((size_t)B * Lin * D);
        tr_bld(cur, z, B, Lin, D);
        int Tc = Lin;
        for (int i = 0; i < v->n_down; i++) {
            int s = v->downK[i], To = Tc / s;
            if (v->l1_norm && i > 0) {
                float *gn = falloc((size_t)B * Tc * D);
                orc_groupnorm(cur, gn, B, 8, D, Tc);
                free(cur); cur = gn;
            }
            float *nx = falloc((size_t)B * To * D);
            orc_conv1d(cur, v->downW[i], v->downB[i], nx, B, D, D, Tc, s, s, 0);
            free(cur); cur = nx; Tc = To;
        }
        if (v->l1_norm_final) {
            float *gn = falloc((size_t)B * Tc * D);
            orc_groupnorm(cur, gn, B, 8, D, Tc);
            free(cur); cur = gn;
        }
        tr_bld(out, cur, B, D, Tc);
        free(cur);
    } else {
        float *bcl = falloc((size_t)B * Lin * D), *cv = falloc((size_t)B * tlen * D);
        tr_bld(bcl, z, B, Lin, D);
        orc_interp_area(bcl, cv, B, D, Lin, tlen);
        tr_bld(out, cv, B, D, tlen);
        free(bcl); free(cv);
    }
    if (v->has_all && level >= 1 && level <= v->n_levels - 2 && v->drefW[level])
        add_conv_bld(out, v->drefW[level], v->drefB[level], B, tlen, D, 3, 1);
}

/* q [B][tlen][D] -> [B][L][D]. reference src/vq.c:327-376 */
static void up_to_full(const VQ *v, const float *q, int B, int tlen, int level, float *out) {
    int D = v->D, L = v->L;
    if (level == 0 && v->has_l1) {
        float *cur = falloc((size_t)B * tlen * D);
        tr_bld(cur, q, B, tlen, D);
        int Tc = tlen;
        for (int i = 0; i < v->n_up; i++) {
            int s = v->upK[i], To = (Tc - 1) * s + s;
            if (v->l1_norm && i > 0) {
                float *gn = falloc((size_t)B * Tc * D);
                orc_groupnorm(cur, gn, B, 8, D, Tc);
                free(cur); cur = gn;
            }
            float *nx = falloc((size_t)B * To * D);
            orc_convT1d(cur, v->upW[i], v->upB[i], nx, B, D, D, Tc, s, s);
            free(cur); cur = nx; Tc = To;
        }
        if (v->l1_norm_final) {
            float *gn = falloc((size_t)B * Tc * D);
            orc_groupnorm(cur, gn, B, 8, D, Tc);
            free(cur); cur = gn;
        }
        tr_bld(out, cur, B, D, Tc);
        free(cur);
    } else {
        float *bcl = falloc((size_t)B * tlen * D), *cv = falloc((size_t)B * L * D);
        tr_bld(bcl, q, B, tlen, D);
        orc_interp_linear(bcl, cv, B, D, tlen, L);
        tr_bld(out, cv, B, D, L);
        free(bcl); free(cv);
    }
    if (v->has_all && level >= 1 && level <= v->n_levels - 2 && v->urefW[level])
        add_conv_bld(out, v->urefW[level], v->urefB[level], B, L, D, 3, 1);
}

/* gather one level's code vectors, upsample, Phi: the increment added to z_hat */
static void level_increment(const VQ *v, const int *codes, int stride, int level, int B, float *up) {
    int D = v->D, tlen = v->levels[level];
    float *q = falloc((size_t)B * tlen * D);
    for (int b = 0; b < B; b++) for (int t = 0; t < tlen; t++)
        memcpy(q + ((size_t)b * tlen + t) * D, v->E[level] + (size_t)codes[(size_t)b * stride + t] * D,
               (size_t)D * sizeof(float));
    up_to_full(v, q, B, tlen, level, up);
    apply_phi(v, up, B, v->L, level);
    free(q);
}

static void area_bld(const float *z, float *out, int B, int L, int D, int Lout) {
    float *bcl = falloc((size_t)B * L * D), *cv = falloc((size_t)B * Lout * D);
    tr_bld(bcl, z, B, L, D);
    orc_interp_area(bcl, cv, B, D, L, Lout);
    tr_bld(out, cv, B, D, Lout);
    free(bcl); free(cv);
}

/* residual quantizer encode, strict-< argmin. reference src/vq.c:388-500 (argmin path) */
void orc_vq_z_to_idx(OrcModel *m, const float *z, int B, int *idx) {
    VQ *v = &m->vq;
    int D = v->D, L = v->L, total = vq_total(v);
    size_t n = (size_t)B * L * D;
    float *z_rest = falloc(n), *z_hat = (float *)xcalloc(n, sizeof(float));
    float *down = falloc(n), *up = falloc(n);
    memcpy(z_rest, z, n * sizeof(float));
    int off = 0;
    for (int lv = 0; lv < v->n_levels; lv++) {
        int tlen = v->levels[lv], V = v->vocabs[lv];
        float *dd = falloc((size_t)B * tlen * V);
        down_for_quant(v, z_rest, B, L, lv, down);
        orc_l2sq(down, v->E[lv], dd, (int64_t)B * tlen, V, D);
        for (int r = 0; r < B * tlen; r++) {
            const float *row = dd + (size_t)r * V;
            int bi = 0; float bv = row[0];
            for (int j = 1; j < V; j++) if (row[j] < bv) { bv = row[j]; bi = j; }
            idx[(r / tlen) * total + off + (r % tlen)] = bi;
        }
        free(dd);
        level_increment(v, idx + off, total, lv, B, up);
        for (size_t i = 0; i < n; i++) z_hat[i] += up[i];
        for (size_t i = 0; i < n; i++) z_rest[i] -= up[i];
        off += tlen;
    }
    free(z_rest); free(z_hat); free(down); free(up);
}

/* reference src/vq.c:502-553 */
void orc_vq_idx_to_zhats(OrcModel *m, const int *idx, int B, float **zhats) {
    VQ *v = &m->vq;
    int total = vq_total(v);
    size_t n = (size_t)B * v->L * v->D;
    float *z_hat = (float *)xcalloc(n, sizeof(float)), *up = falloc(n);
    int base = 0;
    for (int lv = 0; lv < v->n_levels; lv++) {
        level_increment(v, idx + base, total, lv, B, up);
        for (size_t i = 0; i < n; i++) z_hat[i] += up[i];
        memcpy(zhats[lv], z_hat, n * sizeof(float));
        base += v->levels[lv];
    }
    free(z_hat); free(up);
}

/* reference src/vq.c:555-597 */
void orc_vq_next_input(OrcModel *m, const int *codes, int level, float *z_hat, float *x_out, int B) {
    VQ *v = &m->vq;
    size_t n = (size_t)B * v->L * v->D;
    float *up = falloc(n);
    level_increment(v, codes, v->levels[level], level, B, up);
    for (size_t i = 0; i < n; i++) z_hat[i] += up[i];
    area_bld(z_hat, x_out, B, v->L, v->D, v->levels[level + 1]);
    free(up);
}

/* reference src/vq.c:601-674 */
void orc_vq_idx_to_ncm_input(OrcModel *m, const int *idx, int B, float *x_out) {
    VQ *v = &m->vq;
    int D = v->D, total = vq_total(v), T = total - v->levels[0];
    size_t n = (size_t)B * v->L * D;
    float *z_hat = (float *)xcalloc(n, sizeof(float)), *up = falloc(n);
    int base = 0, off = 0;
    for (int li = 0; li < v->n_levels - 1; li++) {
        int nlen = v->levels[li + 1];
        level_increment(v, idx + base, total, li, B, up);
        for (size_t i = 0; i < n; i++) z_hat[i] += up[i];
        float *chunk = falloc((size_t)B * nlen * D);
        area_bld(z_hat, chunk, B, v->L, D, nlen);
        for (int b = 0; b < B; b++)
            memcpy(x_out + ((size_t)b * T + off) * D, chunk + (size_t)b * nlen * D,
                   (size_t)nlen * D * sizeof(float));
        free(chunk);
        base += v->levels[li]; off += nlen;
    }
    free(z_hat); free(up);
}

/* ====================================================================== */
/* attention blocks                                                       */
/* ====================================================================== */

/* [B][T][W] row-major fused projections -> head-major [B][H][T][hd]; GQA heads
 * are replicated. reference src/ncp.c:213-236, src/vqvae.c:76-110 */
static void split_heads(const float *qkv, float *q, float *k, float *v, int B, int T, int C,
                        int H, int nkv, int hd) {
    int W = C + 2 * nkv * hd, rep = H / nkv;
    for (int b = 0; b < B; b++) for (int s = 0; s < T; s++) {
        const float *row = qkv + ((size_t)b * T + s) * W;
        for (int h = 0; h < H; h++) {
            size_t o = (((size_t)b * H + h) * T + s) * hd;
            int kvh = h / rep;
            memcpy(q + o, row + h * hd, (size_t)hd * sizeof(float));
            memcpy(k + o, row + C + kvh * hd, (size_t)hd * sizeof(float));
            memcpy(v + o, row + C + nkv * hd + kvh * hd, (size_t)hd * sizeof(float));
        }
    }
}
static void merge_heads(const float *ctx, float *out, int B, int T, int C, int H, int hd) {
    for (int b = 0; b < B; b++) for (int s = 0; s < T; s++) for (int h = 0; h < H; h++)
        memcpy(out + ((size_t)b * T + s) * C + h * hd, ctx + (((size_t)b * H + h) * T + s) * hd,
               (size_t)hd * sizeof(float));
}

/* One VQ-VAE transformer block, in place on x [B][T][C].
 * reference src/vqvae.c:44-225 */
static void vae_block(const Store *ws, const char *pre, float *x, int B, int T, int C,
                      int H, int qk_norm, int window) {
    size_t n = (size_t)B * T * C;
    int hd = C / H;
    float *ln = falloc(n), *qkv = falloc(3 * n);
    float *q = falloc(n), *k = falloc(n), *v = falloc(n), *ctx = falloc(n), *o = falloc(n), *po = falloc(n);
    orc_layernorm(x, store_need(ws, "%sln_1.weight", pre)->data, DATA(store_getf(ws, "%sln_1.bias", pre)),
                  ln, (int64_t)B * T, C, 1e-6);
    orc_linear(ln, store_need(ws, "%sattn.c_attn.weight", pre)->data,
               DATA(store_getf(ws, "%sattn.c_attn.bias", pre)), qkv, (int64_t)B * T, 3 * C, C);
    split_heads(qkv, q, k, v, B, T, C, H, H, hd);
    if (qk_norm) {
        orc_rmsnorm(q, store_need(ws, "%sattn.q_norm.weight", pre)->data, q, (int64_t)B * H * T, hd);
        orc_rmsnorm(k, store_need(ws, "%sattn.k_norm.weight", pre)->data, k, (int64_t)B * H * T, hd);
    }
    float *mask = NULL;
    if (window > 0) {
        mask = falloc((size_t)T * T);
        for (int i = 0; i < T; i++) for (int j = 0; j < T; j++)
            mask[i * T + j] = (abs(i - j) <= window) ? 0.0f : -INFINITY;
    }
    orc_sdpa(q, k, v, mask, ctx, B, H, H, T, T, hd);
    free(mask);
    merge_heads(ctx, o, B, T, C, H, hd);
    orc_linear(o, store_need(ws, "%sattn.c_proj.weight", pre)->data,
               DATA(store_getf(ws, "%sattn.c_proj.bias", pre)), po, (int64_t)B * T, C, C);
    for (size_t i = 0; i < n; i++) x[i] += po[i];
    orc_layernorm(x, store_need(ws, "%sln_2.weight", pre)->data, DATA(store_getf(ws, "%sln_2.bias", pre)),
                  ln, (int64_t)B * T, C, 1e-6);
    OT *fc = store_need(ws, "%smlp.c_fc.weight", pre);
    int H4 = (int)fc->shape[0];
    float *mm = falloc((size_t)B * T * H4);
    orc_linear(ln, fc->data, DATA(store_getf(ws, "%smlp.c_fc.bias", pre)), mm, (int64_t)B * T, H4, C);
    orc_gelu(mm, mm, (int64_t)B * T * H4);
    orc_linear(mm, store_need(ws, "%smlp.c_proj.weight", pre)->data,
               DATA(store_getf(ws, "%smlp.c_proj.bias", pre)), po, (int64_t)B * T, C, H4);
    for (size_t i = 0; i < n; i++) x[i] += po[i];
    free(ln); free(qkv); free(q); free(k); free(v); free(ctx); free(o); free(po); free(mm);
}

/* reference src/vqvae.c:228-420 */
void orc_vqvae_encode(OrcModel *m, const int *ids, float *z, int B) {
    const Cfg *c = &m->c; const Store *ws = &m->ws;
    int T = c->vq_ctx, D = c->vq_D;
    size_t n = (size_t)B * T * D;
    float *x = falloc(n);
    const float *wte = store_need(ws, "tok.encoder.wte.weight")->data;
    for (size_t i = 0; i < (size_t)B * T; i++) memcpy(x + i * D, wte + (size_t)ids[i] * D, (size_t)D * sizeof(float));
    if (c->enc_positional) {
        const float *wpe = store_need(ws, "tok.encoder.wpe.weight")->data;
        for (int b = 0; b < B; b++) for (int i = 0; i < T * D; i++) x[(size_t)b * T * D + i] += wpe[i];
    }
    for (int i = 0; i < c->enc_convs; i++) {
        char pre[96];
        snprintf(pre, sizeof pre, "tok.encoder.conv_blocks.%d.", i);
        float *ln = falloc(n), *bcl = falloc(n), *c1 = falloc(n), *c2 = falloc(n), *back = falloc(n);
        orc_layernorm(x, store_need(ws, "%sln.weight", pre)->data, NULL, ln, (int64_t)B * T, D, 1e-6);
        tr_bld(bcl, ln, B, T, D);
        int K = c->enc_conv_kernel;
        orc_conv1d(bcl, store_need(ws, "%sc1.weight", pre)->data, store_need(ws, "%sc1.bias", pre)->data,
                   c1, B, D, D, T, K, 1, K / 2);
        orc_gelu(c1, c1, (int64_t)n);
        orc_conv1d(c1, store_need(ws, "%sc2.weight", pre)->data, store_need(ws, "%sc2.bias", pre)->data,
                   c2, B, D, D, T, K, 1, K / 2);
        tr_bld(back, c2, B, D, T);
        for (size_t j = 0; j < n; j++) x[j] += back[j];
        free(ln); free(bcl); free(c1); free(c2); free(back);
    }
    for (int i = 0; i < c->enc_layers; i++) {
        char pre[96];
        snprintf(pre, sizeof pre, "tok.encoder.blocks.%d.", i);
        vae_block(ws, pre, x, B, T, D, c->vq_heads, c->vq_qk_norm, c->enc_window);
    }
    if (c->enc_layers > 0 || c->enc_convs > 0) {
        float *ln = falloc(n);
        orc_layernorm(x, store_need(ws, "tok.encoder.ln_e.weight")->data, NULL, ln, (int64_t)B * T, D, 1e-6);
        free(x); x = ln;
    }
    if (c->vq_compression > 1) {
        int f = c->vq_compression, T2 = T / f;
        float *bcl = falloc(n), *cv = falloc((size_t)B * T2 * D);
        tr_bld(bcl, x, B, T, D);
        orc_conv1d(bcl, store_need(ws, "tok.encoder.down.weight")->data,
                   store_need(ws, "tok.encoder.down.bias")->data, cv, B, D, D, T, f, f, 0);
        tr_bld(z, cv, B, D, T2);
        free(bcl); free(cv); free(x);
        return;
    }
    if (c->pre_quant_gn > 0) {
        float *bcl = falloc(n), *gn = falloc(n);
        tr_bld(bcl, x, B, T, D);
        orc_groupnorm(bcl, gn, B, c->pre_quant_gn, D, T);
        tr_bld(z, gn, B, D, T);
        free(bcl); free(gn);
    } else {
        memcpy(z, x, n * sizeof(float));
    }
    free(x);
}

/* reference src/vqvae.c:422-470 */
void orc_vqvae_decode(OrcModel *m, const float *zhat, float *logits, int B) {
    const Cfg *c = &m->c; const Store *ws = &m->ws;
    int T = c->vq_ctx, D = c->vq_D, V = c->vq_in_vocab;
    size_t n = (size_t)B * T * D;
    if (c->vq_compression > 1) { fprintf(stderr, "oracle: decoder upsampling not defined by the reference\n"); exit(1); }
    float *x = falloc(n);
    memcpy(x, zhat, n * sizeof(float));
    if (c->dec_positional) {
        const float *wpe = store_need(ws, "tok.decoder.wpe.weight")->data;
        for (int b = 0; b < B; b++) for (int i = 0; i < T * D; i++) x[(size_t)b * T * D + i] += wpe[i];
    }
    vae_block(ws, "tok.decoder.middle_block.", x, B, T, D, c->vq_heads, c->vq_qk_norm, 0);
    for (int i = 0; i < c->dec_layers - 1; i++) {
        char pre[96];
        snprintf(pre, sizeof pre, "tok.decoder.extra_blocks.%d.", i);
        vae_block(ws, pre, x, B, T, D, c->vq_heads, c->vq_qk_norm, 0);
    }
    float *ln = falloc(n);
    orc_layernorm(x, store_need(ws, "tok.decoder.ln_f.weight")->data, NULL, ln, (int64_t)B * T, D, 1e-6);
    orc_linear(ln, store_need(ws, "tok.decoder.output_layer.weight")->data, NULL, logits, (int64_t)B * T, V, D);
    free(ln); free(x);
}

/* reference src/main.c:863-879 */
void orc_decode_tokens(OrcModel *m, const int *codes, int B, int *tokens) {
    VQ *v = &m->vq;
    int L = v->L, D = v->D, Vp = m->c.vq_in_vocab;
    float **zh = (float **)xmalloc((size_t)v->n_levels * sizeof(float *));
    for (int i = 0; i < v->n_levels; i++) zh[i] = falloc((size_t)B * L * D);
    orc_vq_idx_to_zhats(m, codes, B, zh);
    float *lg = falloc((size_t)B * L * Vp);
    orc_vqvae_decode(m, zh[v->n_levels - 1], lg, B);
    for (int i = 0; i < B * L; i++) tokens[i] = orc_argmax(lg + (size_t)i * Vp, Vp);
    for (int i = 0; i < v->n_levels; i++) free(zh[i]);
    free(zh); free(lg);
}

/* ====================================================================== */
/* NCP transformer                                                        */
/* ====================================================================== */

/* cos/sin of pos * base^(-d/half), duplicated over both halves.
 * reference src/ncp.c:80-92 */
static void rope_table(float *cs, float *sn, const int *pos, int S, int hd, int base) {
    int half = hd / 2;
    for (int t = 0; t < S; t++) for (int d = 0; d < half; d++) {
        double inv = 1.0 / pow((double)base, (double)d / half);
        double f = pos[t] * inv;
        float co = (float)cos(f), si = (float)sin(f);
        cs[t * hd + d] = co; cs[t * hd + half + d] = co;
        sn[t * hd + d] = si; sn[t * hd + half + d] = si;
    }
}

/* reference src/ncp.c:94-175 */
static void ncp_bind(OrcModel *m) {
    const Cfg *c = &m->c;
    m->P = c->prefix_len;
    m->lvl_first = c->query_level0 ? 0 : 1;
    m->L = 0;
    for (int i = 0; i < c->n_levels; i++) m->L += c->levels[i];
    m->T = m->L - (c->query_level0 ? 0 : c->levels[0]);
    m->n_tgt = c->n_levels - m->lvl_first;
    int hd = c->n_embd / c->n_head, S = m->P + m->T, C = c->n_embd;
    int *pos = (int *)xmalloc((size_t)S * sizeof(int));
    for (int i = 0; i < m->P; i++) pos[i] = i;
    int o = m->P;
    for (int k = m->lvl_first; k < c->n_levels; k++)
        for (int t = 0; t < c->levels[k]; t++) pos[o++] = t;
    m->rope_cos = falloc((size_t)S * hd); m->rope_sin = falloc((size_t)S * hd);
    rope_table(m->rope_cos, m->rope_sin, pos, S, hd, c->rope_base);
    m->gcos = (float **)xmalloc((size_t)m->n_tgt * sizeof(float *));
    m->gsin = (float **)xmalloc((size_t)m->n_tgt * sizeof(float *));
    for (int k = 0; k < m->n_tgt; k++) {
        int lk = c->levels[k + m->lvl_first], Sk = m->P + lk;
        for (int i = 0; i < m->P; i++) pos[i] = i;
        for (int t = 0; t < lk; t++) pos[m->P + t] = t;
        m->gcos[k] = falloc((size_t)Sk * hd); m->gsin[k] = falloc((size_t)Sk * hd);
        rope_table(m->gcos[k], m->gsin[k], pos, Sk, hd, c->rope_base);
    }
    free(pos);
    m->lvl_pos = falloc((size_t)m->T * C);
    const float *wle = store_need(&m->ws, "gen.transformer.wle.weight")->data;
    int tt = 0;
    for (int k = 0; k < m->n_tgt; k++)
        for (int t = 0; t < c->levels[k + m->lvl_first]; t++, tt++)
            memcpy(m->lvl_pos + (size_t)tt * C, wle + (size_t)k * C, (size_t)C * sizeof(float));
    if (!c->use_rope) {
        const float *wpe = store_need(&m->ws, "gen.transformer.wpe.weight")->data;
        tt = 0;
        for (int k = 0; k < m->n_tgt; k++)
            for (int t = 0; t < c->levels[k + m->lvl_first]; t++, tt++)
                for (int d = 0; d < C; d++) m->lvl_pos[(size_t)tt * C + d] += wpe[(size_t)t * C + d];
    }
}

/* One pre-LN block, in place on x [B][S][C]. reference src/ncp.c:184-344 */
static void ncp_block(const OrcModel *m, int li, float *x, int B, int S, const float *mask,
                      const float *cs, const float *sn) {
    const Cfg *c = &m->c; const Store *ws = &m->ws;
    int C = c->n_embd, H = c->n_head, hd = C / H, nkv = c->n_kv_heads;
    int Wq = C + 2 * nkv * hd;
    size_t n = (size_t)B * S * C;
    char pre[64];
    snprintf(pre, sizeof pre, "gen.transformer.blocks.%d.", li);
    float *ln = falloc(n), *qkv = falloc((size_t)B * S * Wq);
    float *q = falloc(n), *k = falloc(n), *v = falloc(n), *ctx = falloc(n), *mo = falloc(n), *ao = falloc(n);
    orc_layernorm(x, store_need(ws, "%sln_1.weight", pre)->data, DATA(store_getf(ws, "%sln_1.bias", pre)),
                  ln, (int64_t)B * S, C, 1e-6);
    orc_linear(ln, store_need(ws, "%sattn.c_attn.weight", pre)->data,
               DATA(store_getf(ws, "%sattn.c_attn.bias", pre)), qkv, (int64_t)B * S, Wq, C);
    split_heads(qkv, q, k, v, B, S, C, H, nkv, hd);
    if (c->use_qk_norm) {
        orc_rmsnorm(q, store_need(ws, "%sattn.q_norm.weight", pre)->data, q, (int64_t)B * H * S, hd);
        orc_rmsnorm(k, store_need(ws, "%sattn.k_norm.weight", pre)->data, k, (int64_t)B * H * S, hd);
    }
    if (c->use_rope) {
        orc_rope(q, cs, sn, (int64_t)B * H * S, S, hd);
        orc_rope(k, cs, sn, (int64_t)B * H * S, S, hd);
    }
    orc_sdpa(q, k, v, mask, ctx, B, H, H, S, S, hd);
    merge_heads(ctx, mo, B, S, C, H, hd);
    orc_linear(mo, store_need(ws, "%sattn.c_proj.weight", pre)->data,
               DATA(store_getf(ws, "%sattn.c_proj.bias", pre)), ao, (int64_t)B * S, C, C);
    for (size_t i = 0; i < n; i++) x[i] += ao[i];
    orc_layernorm(x, store_need(ws, "%sln_2.weight", pre)->data, DATA(store_getf(ws, "%sln_2.bias", pre)),
                  ln, (int64_t)B * S, C, 1e-6);
    float *mlpo = falloc(n);
    if (c->swiglu || c->geglu) {
        OT *tg = store_need(ws, "%smlp.w_gate.weight", pre);
        int Hh = (int)tg->shape[0];
        size_t nh = (size_t)B * S * Hh;
        float *g = falloc(nh), *u = falloc(nh);
        orc_linear(ln, tg->data, DATA(store_getf(ws, "%smlp.w_gate.bias", pre)), g, (int64_t)B * S, Hh, C);
        orc_linear(ln, store_need(ws, "%smlp.w_up.weight", pre)->data,
                   DATA(store_getf(ws, "%smlp.w_up.bias", pre)), u, (int64_t)B * S, Hh, C);
        if (c->swiglu) orc_silu(g, g, (int64_t)nh); else orc_gelu(g, g, (int64_t)nh);
        for (size_t i = 0; i < nh; i++) g[i] *= u[i];
        orc_linear(g, store_need(ws, "%smlp.c_proj.weight", pre)->data,
                   DATA(store_getf(ws, "%smlp.c_proj.bias", pre)), mlpo, (int64_t)B * S, C, Hh);
        free(g); free(u);
    } else {
        OT *tf = store_need(ws, "%smlp.c_fc.weight", pre);
        int Hh = (int)tf->shape[0];
        size_t nh = (size_t)B * S * Hh;
        float *h = falloc(nh);
        orc_linear(ln, tf->data, DATA(store_getf(ws, "%smlp.c_fc.bias", pre)), h, (int64_t)B * S, Hh, C);
        if (c->relu2) for (size_t i = 0; i < nh; i++) { float r = h[i] > 0 ? h[i] : 0; h[i] = r * r; }
        else orc_gelu(h, h, (int64_t)nh);
        orc_linear(h, store_need(ws, "%smlp.c_proj.weight", pre)->data,
                   DATA(store_getf(ws, "%smlp.c_proj.bias", pre)), mlpo, (int64_t)B * S, C, Hh);
        free(h);
    }
    for (size_t i = 0; i < n; i++) x[i] += mlpo[i];
    free(ln); free(qkv); free(q); free(k); free(v); free(ctx); free(mo); free(ao); free(mlpo);
}

/* all blocks then the final LayerNorm, in place. reference src/ncp.c:347-358 */
static void run_stack(const OrcModel *m, float *h, int B, int S, const float *mask,
                      const float *cs, const float *sn) {
    int C = m->c.n_embd;
    for (int li = 0; li < m->c.n_layer; li++) ncp_block(m, li, h, B, S, mask, cs, sn);
    size_t n = (size_t)B * S * C;
    float *t = falloc(n);
    orc_layernorm(h, store_need(&m->ws, "gen.transformer.ln_f.weight")->data,
                  DATA(store_getf(&m->ws, "gen.transformer.ln_f.bias")), t, (int64_t)B * S, C, 1e-6);
    memcpy(h, t, n * sizeof(float));
    free(t);
}

/* per-level output head: untied, shared (+ per-level bias), or tied to the
 * level's codebook. reference src/ncp.c:406-477 */
static void head_logits(const OrcModel *m, int k, const float *slice, float *lg, int rows) {
    const Cfg *c = &m->c; const Store *ws = &m->ws;
    int V = c->vocab_size[k], C = c->n_embd;
    if (c->shared_head) {
        const float *bias = NULL;
        if (c->shared_head_lvl_bias) bias = store_need(ws, "gen.lm_heads.biases.%d", k)->data;
        else if (c->untied_head_bias) bias = store_need(ws, "gen.lm_heads.head.bias")->data;
        orc_linear(slice, store_need(ws, "gen.lm_heads.head.weight")->data, bias, lg, rows, V, C);
    } else if (c->tie_heads) {
        OT *tp = store_need(ws, "gen.lm_heads.%d.proj.weight", k);
        int Dd = (int)tp->shape[0];
        float *z = falloc((size_t)rows * Dd);
        orc_linear(slice, tp->data, DATA(store_getf(ws, "gen.lm_heads.%d.proj.bias", k)), z, rows, Dd, C);
        const float *E = store_need(ws, "tok.vq.embeddings.%d.weight", k + m->lvl_first)->data;
        double *Esq = (double *)xmalloc((size_t)V * sizeof(double)), ds = 0;
        for (int v = 0; v < V; v++) {
            double s = 0;
            for (int d = 0; d < Dd; d++) s += (double)E[(size_t)v * Dd + d] * E[(size_t)v * Dd + d];
            Esq[v] = s; ds += s;
        }
        ds /= V;
        float invT = expf(store_need(ws, "gen.lm_heads.%d.log_inv_T", k)->data[0]);
        const float *hb = DATA(store_getf(ws, "gen.lm_heads.%d.bias", k));
#pragma omp parallel for schedule(static) if ((int64_t)rows * V > 4096)
        for (int r = 0; r < rows; r++) for (int v = 0; v < V; v++) {
            double dot = 0;
            for (int d = 0; d < Dd; d++) dot += (double)z[(size_t)r * Dd + d] * E[(size_t)v * Dd + d];
            double o = (2 * dot - Esq[v]) / ds * invT;
            if (hb) o += hb[v];
            lg[(size_t)r * V + v] = (float)o;
        }
        free(z); free(Esq);
    } else {
        orc_linear(slice, store_need(ws, "gen.lm_heads.%d.weight", k)->data,
                   DATA(store_getf(ws, "gen.lm_heads.%d.bias", k)), lg, rows, V, C);
    }
}

/* Sequential per-row, per-position sampling with frequency / deficit / adjacency
 * penalties; counts and history persist across levels. reference src/ncp.c:654-705 */
static void sample_rows(const float *logits, int *out, int B, int Lc, int V, float temp, int top_k,
                        float top_p, float freq, float mu, float adj_a, int adj_w, float adj_d,
                        const double *allow, uint64_t *rng, double **cnt_s, int **hist_s, int *hist_n) {
    float *adj = falloc(V);
    for (int b = 0; b < B; b++) {
        double *cnt = cnt_s[b];
        int *hist = hist_s[b], hl = hist_n[b];
        for (int t = 0; t < Lc; t++) {
            const float *row = logits + ((size_t)b * Lc + t) * V;
            int pick;
            if (freq <= 0 && adj_a == 0) {
                pick = orc_sample_topkp(row, V, temp, top_k, top_p, rng);
            } else {
                for (int v = 0; v < V; v++) {
                    double lg = row[v];
                    if (freq > 0) {
                        double al = allow ? allow[v] * Lc : 0.0;
                        double excess = cnt[v] - al;
                        if (excess < 0) excess = 0;
                        lg -= freq * excess;
                        if (mu > 0 && allow) {
                            double def = al - cnt[v];
                            if (def < 0) def = 0;
                            lg += mu * ((Lc - t) / (double)Lc) * def;
                        }
                    }
                    adj[v] = (float)lg;
                }
                if (adj_a != 0) {
                    int w = adj_w > 0 ? adj_w : 1;
                    int start = hl - w; if (start < 0) start = 0;
                    for (int h = start; h < hl; h++) {
                        double pen = adj_a * pow(adj_d, hl - 1 - h);
                        adj[hist[h]] -= (float)pen;
                    }
                }
                pick = orc_sample_topkp(adj, V, temp, top_k, top_p, rng);
            }
            out[b * Lc + t] = pick;
            cnt[pick] += 1.0;
            hist[hl++] = pick;
        }
        hist_n[b] = hl;
    }
    free(adj);
}

/* Post-upsample conv residual of the teacher-forced forward: x += conv_k(x) on
 * [B][L][D], with the conv output transposed back. reference src/ncp.c:503-532 */
static void puc_apply(const OrcModel *m, int idx, float *x, int B, int L, int K) {
    int D = m->c.vq_D;
    add_conv_bld(x, store_need(&m->ws, "gen.post_upsample_convs.%d.weight", idx)->data,
                 store_need(&m->ws, "gen.post_upsample_convs.%d.bias", idx)->data, B, L, D, K, K / 2);
}

/* Post-upsample conv residual as the GENERATE path applies it: the conv output
 * stays in [B][D][L] order and is added flat, element i to element i, onto the
 * [B][L][D] tensor (reference src/ncp.c:863-869 for level 0, :1040-1045 for the
 * refinement levels).  For L > 1 this is not a transposed add; it is restated as
 * is because generated codes must equal the reference's. */
static void puc_apply_gen(const OrcModel *m, int idx, float *x, int B, int L, int K) {
    int D = m->c.vq_D;
    size_t n = (size_t)B * L * D;
    float *bcl = falloc(n), *cv = falloc(n);
    tr_bld(bcl, x, B, L, D);
    orc_conv1d(bcl, store_need(&m->ws, "gen.post_upsample_convs.%d.weight", idx)->data,
               store_need(&m->ws, "gen.post_upsample_convs.%d.bias", idx)->data, cv, B, D, D, L, K, 1, K / 2);
    for (size_t i = 0; i < n; i++) x[i] += cv[i];
    free(bcl); free(cv);
}

/* Runs the stack for every model row on [prefix ; level] with that row's pad
 * mask and returns head logits [Bm][Lcur][V]. Rows are independent, so they run
 * in parallel; each row's arithmetic is the reference's single-board call.
 * reference src/ncp.c:1070-1104 (and :893-932 for level 0) */
static void level_logits(const OrcModel *m, const float *pemb, const float *xe, const int *padcol,
                         int Bm, int Lcur, int head, float *logits) {
    int P = m->P, C = m->c.n_embd, S = P + Lcur, V = m->c.vocab_size[head];
#pragma omp parallel for schedule(dynamic, 1)
    for (int b = 0; b < Bm; b++) {
        float *mask = falloc((size_t)S * S);
        for (int i = 0; i < S; i++) for (int j = 0; j < S; j++)
            mask[i * S + j] = (i < P && j >= P) ? -INFINITY : 0.0f;
        if (padcol) for (int i = 0; i < S; i++) for (int j = 0; j < P; j++)
            if (padcol[b * P + j]) mask[i * S + j] = -INFINITY;
        float *h = falloc((size_t)S * C);
        memcpy(h, pemb + (size_t)b * P * C, (size_t)P * C * sizeof(float));
        memcpy(h + (size_t)P * C, xe + (size_t)b * Lcur * C, (size_t)Lcur * C * sizeof(float));
        run_stack(m, h, 1, S, mask, m->gcos[head], m->gsin[head]);
        head_logits(m, head, h + (size_t)P * C, logits + (size_t)b * Lcur * V, Lcur);
        free(mask); free(h);
    }
}

/* reference src/ncp.c:730-1208 (gen_setup, gen_l0, gen_level, teardown) */
void orc_ncp_generate(OrcModel *m, const int *l0, const int *prefix, int B,
                      float temp, int top_k, float top_p, float cfg_scale,
                      float freq, float mu, float adj_a, int adj_w, float adj_d,
                      const double *allow, uint64_t seed, int *codes_out, float *logits_cap) {
    const Cfg *c = &m->c; const Store *ws = &m->ws;
    int P = m->P, C = c->n_embd, D = c->vq_D, nlev = c->n_levels;
    int use_cfg = cfg_scale > 0, Bm = use_cfg ? 2 * B : B;
    int total = vq_total(&m->vq), l0len = c->levels[0];
    const float *wteW = store_need(ws, "gen.transformer.wte.weight")->data;
    const float *wteB = DATA(store_getf(ws, "gen.transformer.wte.bias"));
    /* model prefix with the null branch */
    int *mprefix = (int *)xmalloc((size_t)Bm * P * sizeof(int));
    memcpy(mprefix, prefix, (size_t)B * P * sizeof(int));
    if (use_cfg) {
        int null_first = c->eos_id >= 0 ? c->eos_id : c->prefix_pad;
        for (int b = B; b < Bm; b++) {
            for (int s = 0; s < P; s++) mprefix[(size_t)b * P + s] = c->prefix_pad;
            if (P > 0) mprefix[(size_t)b * P] = null_first;
        }
    }
    float *zpre = falloc((size_t)Bm * P * D), *pemb = falloc((size_t)Bm * P * C);
    const float *ewte = store_need(ws, "tok.encoder.wte.weight")->data;
    for (size_t i = 0; i < (size_t)Bm * P; i++)
        memcpy(zpre + i * D, ewte + (size_t)mprefix[i] * D, (size_t)D * sizeof(float));
    orc_linear(zpre, wteW, wteB, pemb, (int64_t)Bm * P, C, D);
    if (!c->use_rope) {
        const float *wpe = store_need(ws, "gen.transformer.wpe.weight")->data;
        for (int b = 0; b < Bm; b++) for (int i = 0; i < P * C; i++) pemb[(size_t)b * P * C + i] += wpe[i];
    }
    int *padcol = NULL;
    if (c->prefix_pad >= 0) {
        padcol = (int *)xmalloc((size_t)Bm * P * sizeof(int));
        for (size_t i = 0; i < (size_t)Bm * P; i++) padcol[i] = (mprefix[i] == c->prefix_pad);
    }
    uint64_t rng = seed ? seed : 0x9E3779B97F4A7C15ULL;
    float *z_hat = (float *)xcalloc((size_t)Bm * m->vq.L * D, sizeof(float));
    int *cur = NULL;      /* current level's codes; B rows under CFG after a step, else Bm */
    size_t cap_row = 0;   /* per-row floats in logits_cap */
    if (logits_cap) {
        if (!l0 && c->query_level0) cap_row += (size_t)l0len * c->vocab_size[0];
        for (int li = 0; li < nlev - 1; li++)
            cap_row += (size_t)c->levels[li + 1] * c->vocab_size[li + (1 - m->lvl_first)];
    }
    size_t cap_off = 0;

    /* ---- level 0 ---- */
    if (l0) {
        cur = (int *)xmalloc((size_t)B * l0len * sizeof(int));
        memcpy(cur, l0, (size_t)B * l0len * sizeof(int));
        for (int b = 0; b < B; b++) memcpy(codes_out + (size_t)b * total, l0 + (size_t)b * l0len, (size_t)l0len * sizeof(int));
    } else if (c->query_level0) {
        int V0 = c->vocab_size[0];
        float *q0 = falloc((size_t)Bm * l0len * D), *qe = falloc((size_t)Bm * l0len * C);
        const float *lq = store_need(ws, "gen.l0_queries")->data;
        for (int b = 0; b < Bm; b++) memcpy(q0 + (size_t)b * l0len * D, lq, (size_t)l0len * D * sizeof(float));
        if (c->puc_enabled) puc_apply_gen(m, 0, q0, Bm, l0len, 3);
        orc_linear(q0, wteW, wteB, qe, (int64_t)Bm * l0len, C, D);
        const float *wle = store_need(ws, "gen.transformer.wle.weight")->data;
        for (size_t r = 0; r < (size_t)Bm * l0len; r++) for (int d = 0; d < C; d++) qe[r * C + d] += wle[d];
        float *lg = falloc((size_t)Bm * l0len * V0);
        level_logits(m, pemb, qe, padcol, Bm, l0len, 0, lg);
        int *all0 = (int *)xmalloc((size_t)Bm * l0len * sizeof(int));
        for (int b = 0; b < Bm; b++) {       /* fresh penalty state per row; every model row draws */
            double *cnt = (double *)xcalloc(V0, sizeof(double));
            int *hist = (int *)xmalloc((size_t)(l0len * 8 + 64) * sizeof(int)), hn = 0;
            sample_rows(lg + (size_t)b * l0len * V0, all0 + (size_t)b * l0len, 1, l0len, V0, temp, top_k, top_p,
                        freq, mu, adj_a, adj_w, adj_d, allow, &rng, &cnt, &hist, &hn);
            free(cnt); free(hist);
        }
        if (logits_cap) {
            for (int b = 0; b < B; b++)
                memcpy(logits_cap + (size_t)b * cap_row, lg + (size_t)b * l0len * V0, (size_t)l0len * V0 * sizeof(float));
            cap_off += (size_t)l0len * V0;
        }
        cur = (int *)xmalloc((size_t)B * l0len * sizeof(int));
        memcpy(cur, all0, (size_t)B * l0len * sizeof(int));
        for (int b = 0; b < B; b++) memcpy(codes_out + (size_t)b * total, all0 + (size_t)b * l0len, (size_t)l0len * sizeof(int));
        free(q0); free(qe); free(lg); free(all0);
    } else {
        fprintf(stderr, "oracle: generate without l0 needs query_level0\n"); exit(1);
    }

    int Vmax = 0;
    for (int k = 0; k < m->n_tgt; k++) if (c->vocab_size[k] > Vmax) Vmax = c->vocab_size[k];
    double **cntS = (double **)xmalloc((size_t)Bm * sizeof(double *));
    int **histS = (int **)xmalloc((size_t)Bm * sizeof(int *));
    int *histN = (int *)xcalloc(Bm, sizeof(int));
    for (int b = 0; b < Bm; b++) {
        cntS[b] = (double *)xcalloc(Vmax, sizeof(double));
        histS[b] = (int *)xmalloc((size_t)(total + 64) * sizeof(int));
    }
    int level_accum = (m->lvl_first == 0) ? c->levels[0] : 0, out_off = l0len;

    /* ---- refinement levels ---- */
    for (int li = 0; li < nlev - 1; li++) {
        int hi = li + (1 - m->lvl_first), Lprev = c->levels[li], Lcur = c->levels[li + 1];
        int V = c->vocab_size[hi];
        int *codes = (int *)xmalloc((size_t)Bm * Lprev * sizeof(int));
        memcpy(codes, cur, (size_t)B * Lprev * sizeof(int));
        if (use_cfg) memcpy(codes + (size_t)B * Lprev, cur, (size_t)B * Lprev * sizeof(int));
        free(cur); cur = NULL;
        float *x_out = falloc((size_t)Bm * Lcur * D), *xe = falloc((size_t)Bm * Lcur * C);
        orc_vq_next_input(m, codes, li, z_hat, x_out, Bm);
        free(codes);
        if (c->puc_enabled) puc_apply_gen(m, hi, x_out, Bm, Lcur, c->puc_kernel);
        orc_linear(x_out, wteW, wteB, xe, (int64_t)Bm * Lcur, C, D);
        for (int b = 0; b < Bm; b++) for (int t = 0; t < Lcur; t++) for (int d = 0; d < C; d++)
            xe[((size_t)b * Lcur + t) * C + d] += m->lvl_pos[(size_t)(level_accum + t) * C + d];
        float *lg = falloc((size_t)Bm * Lcur * V);
        level_logits(m, pemb, xe, padcol, Bm, Lcur, hi, lg);
        float *use = lg, *blend = NULL;
        if (use_cfg) {
            blend = falloc((size_t)B * Lcur * V);
            double tw = cfg_scale * ((li + 1) / (double)(nlev - 1));
            for (size_t i = 0; i < (size_t)B * Lcur * V; i++) {
                double a = lg[i], u = lg[(size_t)B * Lcur * V + i];
                blend[i] = (float)((1 + tw) * a - tw * u);
            }
            use = blend;
        }
        int Bn = use_cfg ? B : Bm;
        if (logits_cap) {
            for (int b = 0; b < B; b++)
                memcpy(logits_cap + (size_t)b * cap_row + cap_off, use + (size_t)b * Lcur * V, (size_t)Lcur * V * sizeof(float));
            cap_off += (size_t)Lcur * V;
        }
        int *next = (int *)xmalloc((size_t)Bn * Lcur * sizeof(int));
        sample_rows(use, next, Bn, Lcur, V, temp, top_k, top_p, freq, mu, adj_a, adj_w, adj_d,
                    allow, &rng, cntS, histS, histN);
        for (int b = 0; b < B; b++)
            memcpy(codes_out + (size_t)b * total + out_off, next + (size_t)b * Lcur, (size_t)Lcur * sizeof(int));
        out_off += Lcur; level_accum += Lcur;
        cur = next;
        free(x_out); free(xe); free(lg); free(blend);
    }
    for (int b = 0; b < Bm; b++) { free(cntS[b]); free(histS[b]); }
    free(cntS); free(histS); free(histN); free(cur);
    free(mprefix); free(zpre); free(pemb); free(padcol); free(z_hat);
}

int orc_ncp_T(const OrcModel *m) { return m->T; }
int orc_ncp_maxV(const OrcModel *m) {
    int mv = 0;
    for (int k = 0; k < m->n_tgt; k++) if (m->c.vocab_size[k] > mv) mv = m->c.vocab_size[k];
    return mv;
}

/* Teacher-forced forward over [prefix ; all target levels] with the level mask
 * (block-diagonal or block-causal) and, when pads occur, a per-row pad mask.
 * reference src/ncp.c:361-403, 480-647 */
void orc_ncp_forward(OrcModel *m, const float *x, const int *prefix, float *logits, int B) {
    const Cfg *c = &m->c; const Store *ws = &m->ws;
    int P = m->P, T = m->T, S = P + T, C = c->n_embd, D = c->vq_D;
    const float *wteW = store_need(ws, "gen.transformer.wte.weight")->data;
    const float *wteB = DATA(store_getf(ws, "gen.transformer.wte.bias"));
    float *zpre = falloc((size_t)B * P * D), *xt = falloc((size_t)B * T * D);
    for (int b = 0; b < B; b++) {
        memcpy(zpre + (size_t)b * P * D, x + (size_t)b * S * D, (size_t)P * D * sizeof(float));
        memcpy(xt + (size_t)b * T * D, x + ((size_t)b * S + P) * D, (size_t)T * D * sizeof(float));
    }
    if (c->puc_enabled) {
        int off = 0;
        for (int k = 0; k < m->n_tgt; k++) {
            int lk = c->levels[k + m->lvl_first];
            float *chunk = falloc((size_t)B * lk * D);
            for (int b = 0; b < B; b++) memcpy(chunk + (size_t)b * lk * D, xt + ((size_t)b * T + off) * D, (size_t)lk * D * sizeof(float));
            puc_apply(m, k, chunk, B, lk, c->puc_kernel);
            for (int b = 0; b < B; b++) memcpy(xt + ((size_t)b * T + off) * D, chunk + (size_t)b * lk * D, (size_t)lk * D * sizeof(float));
            free(chunk);
            off += lk;
        }
    }
    float *h = falloc((size_t)B * S * C);
    float *pemb = falloc((size_t)B * P * C), *xe = falloc((size_t)B * T * C);
    orc_linear(zpre, wteW, wteB, pemb, (int64_t)B * P, C, D);
    orc_linear(xt, wteW, wteB, xe, (int64_t)B * T, C, D);
    for (int b = 0; b < B; b++) for (int i = 0; i < T * C; i++) xe[(size_t)b * T * C + i] += m->lvl_pos[i];
    if (!c->use_rope) {
        const float *wpe = store_need(ws, "gen.transformer.wpe.weight")->data;
        for (int b = 0; b < B; b++) for (int i = 0; i < P * C; i++) pemb[(size_t)b * P * C + i] += wpe[i];
    }
    for (int b = 0; b < B; b++) {
        memcpy(h + (size_t)b * S * C, pemb + (size_t)b * P * C, (size_t)P * C * sizeof(float));
        memcpy(h + ((size_t)b * S + P) * C, xe + (size_t)b * T * C, (size_t)T * C * sizeof(float));
    }
    int *lvl_of = (int *)xmalloc((size_t)T * sizeof(int));
    { int o = 0; for (int k = m->lvl_first; k < c->n_levels; k++) for (int t = 0; t < c->levels[k]; t++) lvl_of[o++] = k; }
    float *mask = falloc((size_t)S * S);
    for (int i = 0; i < S; i++) for (int j = 0; j < S; j++) {
        float v = 0;
        if (i < P && j >= P) v = -INFINITY;
        else if (i >= P && j >= P) {
            int li = lvl_of[i - P], lj = lvl_of[j - P];
            v = c->block_diag ? (li == lj ? 0.0f : -INFINITY) : (li >= lj ? 0.0f : -INFINITY);
        }
        mask[i * S + j] = v;
    }
    int any_pad = 0;
    if (c->prefix_pad >= 0 && prefix)
        for (int i = 0; i < B * P; i++) if (prefix[i] == c->prefix_pad) any_pad = 1;
    if (any_pad) {
#pragma omp parallel for schedule(dynamic, 1)
        for (int b = 0; b < B; b++) {
            float *bm = falloc((size_t)S * S);
            memcpy(bm, mask, (size_t)S * S * sizeof(float));
            for (int i = 0; i < S; i++) for (int j = 0; j < P; j++)
                if (prefix[b * P + j] == c->prefix_pad) bm[(size_t)i * S + j] = -INFINITY;
            run_stack(m, h + (size_t)b * S * C, 1, S, bm, m->rope_cos, m->rope_sin);
            free(bm);
        }
    } else {
        run_stack(m, h, B, S, mask, m->rope_cos, m->rope_sin);
    }
    int maxV = orc_ncp_maxV(m), off = 0;
    for (size_t i = 0; i < (size_t)B * T * maxV; i++) logits[i] = -INFINITY;
    for (int k = 0; k < m->n_tgt; k++) {
        int lk = c->levels[k + m->lvl_first], V = c->vocab_size[k];
        float *slice = falloc((size_t)B * lk * C), *lg = falloc((size_t)B * lk * V);
        for (int b = 0; b < B; b++)
            memcpy(slice + (size_t)b * lk * C, h + ((size_t)b * S + P + off) * C, (size_t)lk * C * sizeof(float));
        head_logits(m, k, slice, lg, B * lk);
        for (int b = 0; b < B; b++) for (int t = 0; t < lk; t++)
            memcpy(logits + ((size_t)b * T + off + t) * maxV, lg + ((size_t)b * lk + t) * V, (size_t)V * sizeof(float));
        free(slice); free(lg);
        off += lk;
    }
    free(zpre); free(xt); free(h); free(pemb); free(xe); free(lvl_of); free(mask);
}

OrcModel *orc_model_load(const char *conf_path, const char *weights_path) {
    OrcModel *m = (OrcModel *)xcalloc(1, sizeof *m);
    if (cfg_load(&m->c, conf_path) || store_load(&m->ws, weights_path)) { free(m); return NULL; }
    vq_bind(&m->vq, &m->c, &m->ws);
    ncp_bind(m);
    return m;
}
void orc_model_free(OrcModel *m) {
    if (!m) return;
    for (int k = 0; k < m->n_tgt; k++) { free(m->gcos[k]); free(m->gsin[k]); }
    free(m->gcos); free(m->gsin); free(m->rope_cos); free(m->rope_sin); free(m->lvl_pos);
    store_free(&m->ws);
    free(m);
}
int orc_total_codes(const OrcModel *m) { return vq_total(&m->vq); }
int orc_L(const OrcModel *m) { return m->vq.L; }
int orc_D(const OrcModel *m) { return m->vq.D; }
int orc_in_vocab(const OrcModel *m) { return m->c.vq_in_vocab; }

/* ====================================================================== */
/* GPT-2 / Qwen2                                                          */
/* ====================================================================== */

struct OrcLM {
    Cfg c; Store ws; int is_qwen;
    int n_layer, n_head, n_kv, C, I, n_ctx, V;
    float *cosb, *sinb;
};

/* reference src/gpt2.c:43-80, src/qwen.c:44-112 */
OrcLM *orc_lm_load(const char *conf_path, const char *weights_path, int is_qwen) {
    OrcLM *m = (OrcLM *)xcalloc(1, sizeof *m);
    if (cfg_load(&m->c, conf_path) || store_load(&m->ws, weights_path)) { free(m); return NULL; }
    m->is_qwen = is_qwen;
    m->n_layer = m->c.n_layer; m->n_head = m->c.n_head; m->C = m->c.n_embd;
    m->n_kv = m->c.n_kv_heads > 0 ? m->c.n_kv_heads : m->c.n_head;
    if (!is_qwen) {
        m->n_ctx = m->c.context_length > 0 ? m->c.context_length : 1024;
        m->V = (int)store_need(&m->ws, "wte.weight")->shape[0];
        m->I = 4 * m->C;
    } else {
        m->n_ctx = m->c.context_length > 0 ? m->c.context_length : 4096;
        double theta = m->c.rope_theta > 0 ? m->c.rope_theta : 1000000.0;
        m->V = (int)store_need(&m->ws, "model.embed_tokens.weight")->shape[0];
        m->I = (int)store_need(&m->ws, "model.layers.0.mlp.gate_proj.weight")->shape[0];
        int hd = m->C / m->n_head, h = hd / 2, T = m->n_ctx;
        m->cosb = falloc((size_t)T * hd); m->sinb = falloc((size_t)T * hd);
        for (int t = 0; t < T; t++) for (int d = 0; d < h; d++) {
            double a = (double)t * pow(theta, -(double)(2 * d) / (double)hd);
            float co = (float)cos(a), si = (float)sin(a);
            m->cosb[(size_t)t * hd + d] = co; m->cosb[(size_t)t * hd + d + h] = co;
            m->sinb[(size_t)t * hd + d] = si; m->sinb[(size_t)t * hd + d + h] = si;
        }
    }
    return m;
}
void orc_lm_free(OrcLM *m) {
    if (!m) return;
    free(m->cosb); free(m->sinb); store_free(&m->ws); free(m);
}
int orc_lm_vocab(const OrcLM *m) { return m->V; }

static float *causal_mask(int T) {
    float *mk = falloc((size_t)T * T);
    for (int i = 0; i < T; i++) for (int j = 0; j < T; j++) mk[(size_t)i * T + j] = (j <= i) ? 0.0f : -1e9f;
    return mk;
}

/* [T][H*hd] -> [H][T][hd] */
static void heads_first(const float *in, float *out, int T, int H, int hd) {
    for (int t = 0; t < T; t++) for (int h = 0; h < H; h++)
        memcpy(out + ((size_t)h * T + t) * hd, in + ((size_t)t * H + h) * hd, (size_t)hd * sizeof(float));
}

/* reference src/gpt2.c:92-157 */
static void gpt2_logits(OrcLM *m, const int *ids, int T, int last_only, float *out) {
    const Store *ws = &m->ws;
    int C = m->C, H = m->n_head, hd = C / H, V = m->V, I = m->I;
    size_t n = (size_t)T * C;
    const float *wte = store_need(ws, "wte.weight")->data, *wpe = store_need(ws, "wpe.weight")->data;
    float *h = falloc(n);
    for (int t = 0; t < T; t++) for (int d = 0; d < C; d++)
        h[(size_t)t * C + d] = wte[(size_t)ids[t] * C + d] + wpe[(size_t)t * C + d];
    float *mask = causal_mask(T);
    float *ln = falloc(n), *qkv = falloc(3 * n), *q = falloc(n), *k = falloc(n), *v = falloc(n);
    float *ctx = falloc(n), *mo = falloc(n), *ao = falloc(n), *mm = falloc((size_t)T * I), *mlpo = falloc(n);
    for (int li = 0; li < m->n_layer; li++) {
        char pre[32];
        snprintf(pre, sizeof pre, "h.%d.", li);
        orc_layernorm(h, store_need(ws, "%sln_1.weight", pre)->data, store_need(ws, "%sln_1.bias", pre)->data, ln, T, C, (double)1e-5f);
        orc_linear(ln, store_need(ws, "%sattn.c_attn.weight", pre)->data, DATA(store_getf(ws, "%sattn.c_attn.bias", pre)), qkv, T, 3 * C, C);
        split_heads(qkv, q, k, v, 1, T, C, H, H, hd);
        orc_sdpa(q, k, v, mask, ctx, 1, H, H, T, T, hd);
        merge_heads(ctx, mo, 1, T, C, H, hd);
        orc_linear(mo, store_need(ws, "%sattn.c_proj.weight", pre)->data, DATA(store_getf(ws, "%sattn.c_proj.bias", pre)), ao, T, C, C);
        for (size_t i = 0; i < n; i++) h[i] = h[i] + ao[i];
        orc_layernorm(h, store_need(ws, "%sln_2.weight", pre)->data, store_need(ws, "%sln_2.bias", pre)->data, ln, T, C, (double)1e-5f);
        orc_linear(ln, store_need(ws, "%smlp.c_fc.weight", pre)->data, DATA(store_getf(ws, "%smlp.c_fc.bias", pre)), mm, T, I, C);
        orc_gelu_tanh(mm, mm, (int64_t)T * I);
        orc_linear(mm, store_need(ws, "%smlp.c_proj.weight", pre)->data, DATA(store_getf(ws, "%smlp.c_proj.bias", pre)), mlpo, T, C, I);
        for (size_t i = 0; i < n; i++) h[i] = h[i] + mlpo[i];
    }
    orc_layernorm(h, store_need(ws, "ln_f.weight")->data, store_need(ws, "ln_f.bias")->data, ln, T, C, (double)1e-5f);
    if (last_only) orc_linear(ln + (size_t)(T - 1) * C, wte, NULL, out, 1, V, C);
    else orc_linear(ln, wte, NULL, out, T, V, C);
    free(h); free(mask); free(ln); free(qkv); free(q); free(k); free(v); free(ctx); free(mo); free(ao); free(mm); free(mlpo);
}

/* reference src/qwen.c:121-190 */
static void qwen_logits(OrcLM *m, const int *ids, int T, int last_only, float *out) {
    const Store *ws = &m->ws;
    int C = m->C, H = m->n_head, K = m->n_kv, hd = C / H, I = m->I, V = m->V;
    size_t n = (size_t)T * C, nk = (size_t)T * K * hd;
    const float *wte = store_need(ws, "model.embed_tokens.weight")->data;
    float *h = falloc(n);
    for (int t = 0; t < T; t++) memcpy(h + (size_t)t * C, wte + (size_t)ids[t] * C, (size_t)C * sizeof(float));
    float *mask = causal_mask(T);
    float *h1 = falloc(n), *ql = falloc(n), *kl = falloc(nk), *vl = falloc(nk);
    float *q = falloc(n), *k = falloc(nk), *v = falloc(nk), *ctx = falloc(n), *mo = falloc(n), *ao = falloc(n);
    float *gt = falloc((size_t)T * I), *up = falloc((size_t)T * I), *mlpo = falloc(n);
    for (int li = 0; li < m->n_layer; li++) {
        char pre[48];
        snprintf(pre, sizeof pre, "model.layers.%d.", li);
        orc_rmsnorm(h, store_need(ws, "%sinput_layernorm.weight", pre)->data, h1, T, C);
        orc_linear(h1, store_need(ws, "%sself_attn.q_proj.weight", pre)->data, store_need(ws, "%sself_attn.q_proj.bias", pre)->data, ql, T, C, C);
        orc_linear(h1, store_need(ws, "%sself_attn.k_proj.weight", pre)->data, store_need(ws, "%sself_attn.k_proj.bias", pre)->data, kl, T, K * hd, C);
        orc_linear(h1, store_need(ws, "%sself_attn.v_proj.weight", pre)->data, store_need(ws, "%sself_attn.v_proj.bias", pre)->data, vl, T, K * hd, C);
        heads_first(ql, q, T, H, hd); heads_first(kl, k, T, K, hd); heads_first(vl, v, T, K, hd);
        orc_rope(q, m->cosb, m->sinb, (int64_t)H * T, T, hd);
        orc_rope(k, m->cosb, m->sinb, (int64_t)K * T, T, hd);
        orc_sdpa(q, k, v, mask, ctx, 1, H, K, T, T, hd);
        merge_heads(ctx, mo, 1, T, C, H, hd);
        orc_linear(mo, store_need(ws, "%sself_attn.o_proj.weight", pre)->data, NULL, ao, T, C, C);
        for (size_t i = 0; i < n; i++) h[i] = h[i] + ao[i];
        orc_rmsnorm(h, store_need(ws, "%spost_attention_layernorm.weight", pre)->data, h1, T, C);
        orc_linear(h1, store_need(ws, "%smlp.gate_proj.weight", pre)->data, NULL, gt, T, I, C);
        orc_linear(h1, store_need(ws, "%smlp.up_proj.weight", pre)->data, NULL, up, T, I, C);
        orc_silu(gt, gt, (int64_t)T * I);
        for (size_t i = 0; i < (size_t)T * I; i++) gt[i] = gt[i] * up[i];
        orc_linear(gt, store_need(ws, "%smlp.down_proj.weight", pre)->data, NULL, mlpo, T, C, I);
        for (size_t i = 0; i < n; i++) h[i] = h[i] + mlpo[i];
    }
    orc_rmsnorm(h, store_need(ws, "model.norm.weight")->data, h1, T, C);
    if (last_only) orc_linear(h1 + (size_t)(T - 1) * C, wte, NULL, out, 1, V, C);
    else orc_linear(h1, wte, NULL, out, T, V, C);
    free(h); free(mask); free(h1); free(ql); free(kl); free(vl); free(q); free(k); free(v);
    free(ctx); free(mo); free(ao); free(gt); free(up); free(mlpo);
}

void orc_lm_logits(OrcLM *m, const int *ids, int T, int last_only, float *out) {
    if (m->is_qwen) qwen_logits(m, ids, T, last_only, out);
    else gpt2_logits(m, ids, T, last_only, out);
}

/* reference gpt2_nll src/gpt2.c:160-176 = qwen_nll src/qwen.c:192-208: mean over the T-1 shifted positions of
 * -log(exp(l[next] - max) / sum_v exp(l[v] - max) + 1e-30), all in fp64, v in index order */
double orc_lm_nll(OrcLM *m, const int *ids, int T) {
    float *lg = falloc((size_t)T * m->V);
    orc_lm_logits(m, ids, T, 0, lg);
    double tot = 0;
    for (int t = 0; t + 1 < T; t++) {
        const float *row = lg + (size_t)t * m->V;
        double mx = row[0];
        for (int v = 1; v < m->V; v++) if (row[v] > mx) mx = row[v];
        double den = 0;
        for (int v = 0; v < m->V; v++) den += exp(row[v] - mx);
        tot += -log(exp(row[ids[t + 1]] - mx) / den + 1e-30);
    }
    free(lg);
    return tot / (T - 1);
}

/* reference src/gpt2.c:179-202, src/qwen.c:209-231 */
int orc_lm_generate(OrcLM *m, const int *prompt, int np, int n_new, float temp,
                    int top_k, float top_p, uint64_t seed, int eos, int *out) {
    int *ids = (int *)xmalloc((size_t)(np + n_new) * sizeof(int));
    float *row = falloc(m->V);
    memcpy(ids, prompt, (size_t)np * sizeof(int));
    uint64_t rng = seed ? seed : 0x12345678ULL;
    int n = np;
    for (int s = 0; s < n_new; s++) {
        if (n > m->n_ctx) break;
        orc_lm_logits(m, ids, n, 1, row);
        int nx = !(temp > 0) ? orc_argmax(row, m->V) : orc_sample_topkp(row, m->V, temp, top_k, top_p, &rng);
        ids[n++] = nx;
        if (nx == eos) break;
    }
    memcpy(out, ids + np, (size_t)(n - np) * sizeof(int));
    free(ids); free(row);
    return n - np;
}
