// Bandwidth-bound layer kernels: LayerNorm / RMSNorm (one warp per row, 128-bit
// loads, shuffle reductions), activations, gathers and element-wise ops, plus the
// C entry points of the reference's kernel API that map onto them
// (src/ncm.h:148-158, 163-165, 184-190).
#include "common.cuh"
#include "split.cuh"

namespace ncmb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float act_apply(float v, int act) {
    switch (act) {
        case ACT_GELU: return 0.5f * v * (1.0f + erff(v * 0.7071067811865475f));
        case ACT_GELU_TANH: return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
        case ACT_SILU: return v / (1.0f + expf(-v));
        case ACT_RELU2: { float r = v > 0.f ? v : 0.f; return r * r; }
        default: return v;
    }
}

__device__ __forceinline__ float tf32_hi(float v) {
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v));
    return __uint_as_float(u);
}

// ---- LayerNorm: y = (x - mean) * rstd * w + b, statistics over C in two passes ----
// One warp per row; the row (<= a few KB) is re-read from L1 for the second and third
// pass. The affine step is evaluated unfused (mul then add) like the CPU definition.
template <bool VEC4>
__global__ void __launch_bounds__(256) k_layernorm(const float *__restrict__ x, const float *__restrict__ w,
                                                  const float *__restrict__ b, float *__restrict__ y,
                                                  float *__restrict__ ylo, int64_t rows, int C, float eps, int fmt) {
    pdl_launch_dependents();          // programmatic dependent launch: see launch_pdl()
    pdl_wait();
    int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float *xr = x + row * C;
    float *yr = y + row * C;
    float *lr = ylo ? ylo + row * C : nullptr;
    float s = 0.f;
    if (VEC4) {
        for (int c = lane * 4; c < C; c += 128) { float4 v = *(const float4 *)(xr + c); s += (v.x + v.y) + (v.z + v.w); }
    } else {
        for (int c = lane; c < C; c += 32) s += xr[c];
    }
    float mean = warp_sum(s) / (float)C;
    float q = 0.f;
    if (VEC4) {
        for (int c = lane * 4; c < C; c += 128) {
            float4 v = *(const float4 *)(xr + c);
            float a0 = v.x - mean, a1 = v.y - mean, a2 = v.z - mean, a3 = v.w - mean;
            q += (a0 * a0 + a1 * a1) + (a2 * a2 + a3 * a3);
        }
    } else {
        for (int c = lane; c < C; c += 32) { float a = xr[c] - mean; q += a * a; }
    }
    float var = warp_sum(q) / (float)C;
    float inv = 1.0f / sqrtf(var + eps);
    if (VEC4) {
        for (int c = lane * 4; c < C; c += 128) {
            float4 v = *(const float4 *)(xr + c);
            float4 ww = w ? *(const float4 *)(w + c) : make_float4(1.f, 1.f, 1.f, 1.f);
            float4 bb = b ? *(const float4 *)(b + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            float4 o;
            o.x = __fadd_rn(__fmul_rn(__fmul_rn(v.x - mean, inv), ww.x), bb.x);
            o.y = __fadd_rn(__fmul_rn(__fmul_rn(v.y - mean, inv), ww.y), bb.y);
            o.z = __fadd_rn(__fmul_rn(__fmul_rn(v.z - mean, inv), ww.z), bb.z);
            o.w = __fadd_rn(__fmul_rn(__fmul_rn(v.w - mean, inv), ww.w), bb.w);
            if (lr) store_split4(y, ylo, row * C + c, o, fmt);
            else *(float4 *)(yr + c) = o;
        }
    } else {
        for (int c = lane; c < C; c += 32) {
            float o = __fadd_rn(__fmul_rn(__fmul_rn(xr[c] - mean, inv), w ? w[c] : 1.f), b ? b[c] : 0.f);
            if (lr) store_split1(y, ylo, row * C + c, o, fmt);
            else yr[c] = o;
        }
    }
}

static inline bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

void layernorm_split(const float *x, const float *w, const float *b, float *y, float *y_lo, int64_t rows, int C, float eps, int fmt) {
    if (rows <= 0) return;
    ProfScope ps(NCMB_K_NORM, 0, (double)rows * C * (y_lo ? 12 : 8));
    bool v4 = (C % 4 == 0) && aligned16(x) && aligned16(y) && (!y_lo || aligned16(y_lo)) && (!w || aligned16(w)) && (!b || aligned16(b));
    unsigned g = grid1d(rows, 8);
    if (v4) LAUNCH_PDL_IF(pdl_small(g), (k_layernorm<true>), g, 256, 0, x, w, b, y, y_lo, rows, C, eps, fmt);
    else LAUNCH_PDL_IF(pdl_small(g), (k_layernorm<false>), g, 256, 0, x, w, b, y, y_lo, rows, C, eps, fmt);
}
void layernorm(const float *x, const float *w, const float *b, float *y, int64_t rows, int C, float eps) {
    layernorm_split(x, w, b, y, nullptr, rows, C, eps, SPLIT_NONE);
}

// ---- RMSNorm: y = x * rsqrt(mean(x^2) + 1e-6) * w ----
__global__ void __launch_bounds__(256) k_rmsnorm(const float *__restrict__ x, const float *__restrict__ w,
                                                float *__restrict__ y, float *__restrict__ ylo, int64_t rows, int C,
                                                int64_t ldx, int64_t ldy, int fmt) {
    pdl_launch_dependents();          // programmatic dependent launch: see launch_pdl()
    pdl_wait();
    int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float *xr = x + row * ldx;
    float *yr = y + row * ldy;
    float s = 0.f;
    for (int c = lane; c < C; c += 32) { float v = xr[c]; s += v * v; }
    float ms = warp_sum(s) / (float)C;
    float r = 1.0f / sqrtf(ms + 1e-6f);
    float *lr = ylo ? ylo + row * ldy : nullptr;
    for (int c = lane; c < C; c += 32) {
        float o = __fmul_rn(__fmul_rn(xr[c], r), w ? w[c] : 1.f);
        if (lr) store_split1(y, ylo, row * ldy + c, o, fmt);
        else yr[c] = o;
    }
}

void rmsnorm(const float *x, const float *w, float *y, int64_t rows, int C, int64_t ldx, int64_t ldy) {
    if (rows <= 0) return;
    ProfScope ps(NCMB_K_NORM, 0, (double)rows * C * 8);
    LAUNCH_PDL_IF(pdl_small(rows / 8), k_rmsnorm, grid1d(rows, 8), 256, 0, x, w, y, (float *)nullptr, rows, C, ldx, ldy, (int)SPLIT_NONE);
}
void rmsnorm_split(const float *x, const float *w, float *y, float *y_lo, int64_t rows, int C, int fmt) {
    if (rows <= 0) return;
    ProfScope ps(NCMB_K_NORM, 0, (double)rows * C * 12);
    LAUNCH_PDL_IF(pdl_small(rows / 8), k_rmsnorm, grid1d(rows, 8), 256, 0, x, w, y, y_lo, rows, C, (int64_t)C, (int64_t)C, fmt);
}

// ---- element-wise ----
__global__ void k_add_inplace(float *__restrict__ y, const float *__restrict__ x, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) y[i] += x[i];
}
__global__ void k_add(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ y, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) y[i] = a[i] + b[i];
}
__global__ void k_mul(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ y, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) y[i] = a[i] * b[i];
}
__global__ void k_scale(const float *__restrict__ x, float s, float *__restrict__ y, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) y[i] = x[i] * s;
}
__global__ void k_act(const float *__restrict__ x, float *__restrict__ y, int64_t n, int act) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) y[i] = act_apply(x[i], act);
}
__global__ void k_fill(float *p, float v, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) p[i] = v;
}
__global__ void k_add_rows_bcast(float *__restrict__ y, const float *__restrict__ v, int64_t rows, int C) {
    int64_t n = rows * C;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) y[i] += v[i % C];
}
__global__ void k_embed(const float *__restrict__ W, const int *__restrict__ idx, float *__restrict__ y, int64_t n, int D) {
    int64_t tot = n * D;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < tot; i += (int64_t)gridDim.x * blockDim.x)
        y[i] = W[(int64_t)idx[i / D] * D + (i % D)];
}
// gu: [rows][2*Hh] with the gate in the first Hh columns and the up projection in the last Hh
__global__ void k_glu(const float *__restrict__ gu, float *__restrict__ y, int64_t rows, int Hh, int act) {
    int64_t n = rows * Hh;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t r = i / Hh; int c = (int)(i % Hh);
        float g = gu[r * 2 * Hh + c], u = gu[r * 2 * Hh + Hh + c];
        y[i] = __fmul_rn(act_apply(g, act), u);
    }
}

__global__ void k_interleave_rows(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ y, int64_t rows, int64_t cols) {
    int64_t n = 2 * rows * cols;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t r = i / cols, c = i % cols;
        const float *src = (r & 1) ? b : a;
        y[i] = src ? src[(r >> 1) * cols + c] : 0.f;
    }
}

static unsigned ew_grid(int64_t n) {
    int64_t g = cdiv(n, 256);
    int64_t cap = (int64_t)ctx().sm_count * 16;
    if (g > cap) g = cap;
    return (unsigned)(g < 1 ? 1 : g);
}

float *dev_interleave_rows(const float *a, const float *b, int64_t rows, int64_t cols) {
    float *d = (float *)dev_alloc((size_t)(2 * rows * cols) * sizeof(float));
    LAUNCH(k_interleave_rows, ew_grid(2 * rows * cols), 256, 0, a, b, d, rows, cols);
    return d;
}

void add_inplace(float *y, const float *x, int64_t n) {
    if (n <= 0) return;
    ProfScope ps(NCMB_K_ELEM, 0, (double)n * 12);
    LAUNCH(k_add_inplace, ew_grid(n), 256, 0, y, x, n);
}
void add_rows_bcast(float *y, const float *v, int64_t rows, int C) {
    if (rows <= 0) return;
    ProfScope ps(NCMB_K_ELEM, 0, (double)rows * C * 8);
    LAUNCH(k_add_rows_bcast, ew_grid(rows * C), 256, 0, y, v, rows, C);
}
void embed_rows(const float *W, const int *idx, float *y, int64_t n, int D) {
    if (n <= 0) return;
    ProfScope ps(NCMB_K_ELEM, 0, (double)n * D * 8);
    LAUNCH(k_embed, ew_grid(n * D), 256, 0, W, idx, y, n, D);
}
void glu_combine(const float *gu, float *y, int64_t rows, int Hh, int act) {
    if (rows <= 0) return;
    ProfScope ps(NCMB_K_ELEM, 0, (double)rows * Hh * 12);
    LAUNCH(k_glu, ew_grid(rows * Hh), 256, 0, gu, y, rows, Hh, act);
}
void act_inplace(float *x, int64_t n, int act) {
    if (n <= 0) return;
    ProfScope ps(NCMB_K_ELEM, 0, (double)n * 8);
    LAUNCH(k_act, ew_grid(n), 256, 0, x, x, n, act);
}
void fill_f32(float *p, float v, int64_t n) {
    if (n <= 0) return;
    LAUNCH(k_fill, ew_grid(n), 256, 0, p, v, n);
}

// ---- per-row argmax, lowest index wins ties (reference argmax_row, kernels.c:731) ----
__global__ void __launch_bounds__(256) k_argmax_rows(const float *__restrict__ x, int64_t rows, int V, int *__restrict__ out) {
    int64_t r = blockIdx.x;
    if (r >= rows) return;
    const float *xr = x + r * V;
    float bv = -INFINITY; int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {     // ascending i: strict > keeps the first maximum
        float v = xr[i];
        if (bi == 0x7fffffff || v > bv) { bv = v; bi = i; }
    }
    __shared__ float sv[256];
    __shared__ int si[256];
    sv[threadIdx.x] = bv; si[threadIdx.x] = bi;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if ((int)threadIdx.x < s) {
            float ov = sv[threadIdx.x + s]; int oi = si[threadIdx.x + s];
            if (oi != 0x7fffffff && (si[threadIdx.x] == 0x7fffffff || ov > sv[threadIdx.x] || (ov == sv[threadIdx.x] && oi < si[threadIdx.x]))) {
                sv[threadIdx.x] = ov; si[threadIdx.x] = oi;
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) out[r] = si[0] == 0x7fffffff ? 0 : si[0];
}
void argmax_rows(const float *x, int64_t rows, int V, int *out) {
    if (rows <= 0) return;
    ProfScope ps(NCMB_K_SAMPLE, 0, (double)rows * V * 4);
    LAUNCH(k_argmax_rows, (unsigned)rows, 256, 0, x, rows, V, out);
}

// ---- layout shuffles of the reference kernel API ----
__global__ void k_heads_transpose_b(const float *__restrict__ in, float *__restrict__ out, int64_t B, int64_t T, int H, int hd) {
    int64_t n = B * T * H * hd;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int d = (int)(i % hd); int64_t r = i / hd; int h = (int)(r % H); r /= H; int64_t t = r % T; int64_t b = r / T;
        out[((b * H + h) * T + t) * hd + d] = in[i];
    }
}
__global__ void k_qkvsplit(const float *__restrict__ in, float *__restrict__ qq, float *__restrict__ kk, float *__restrict__ vv,
                           int B, int T, int C, int H, int hd, int K, int rep) {
    int64_t n = (int64_t)B * H * T * hd;
    int64_t W = (int64_t)C + 2 * K * hd;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int d = (int)(i % hd); int t = (int)((i / hd) % T); int h = (int)((i / ((int64_t)hd * T)) % H); int b = (int)(i / ((int64_t)H * T * hd));
        int kvh = h / rep;
        const float *row = in + ((int64_t)b * T + t) * W;
        qq[i] = row[h * hd + d];
        kk[i] = row[C + kvh * hd + d];
        vv[i] = row[C + K * hd + kvh * hd + d];
    }
}
__global__ void k_headmerge(const float *__restrict__ ctxp, float *__restrict__ out, int B, int T, int C, int H, int hd) {
    int64_t n = (int64_t)B * T * C;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int d = (int)(i % C); int hh = d / hd, dd = d % hd; int t = (int)((i / C) % T); int b = (int)(i / ((int64_t)T * C));
        out[i] = ctxp[(((int64_t)b * H + hh) * T + t) * hd + dd];
    }
}
// row softmax, one warp per row (reference kernel API; not on the generate path)
__global__ void k_softmax(const float *__restrict__ x, float *__restrict__ y, int64_t rows, int C) {
    int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float *xr = x + row * C; float *yr = y + row * C;
    float mx = -INFINITY;
    for (int c = lane; c < C; c += 32) mx = fmaxf(mx, xr[c]);
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float s = 0.f;
    for (int c = lane; c < C; c += 32) s += expf(xr[c] - mx);
    s = warp_sum(s);
    for (int c = lane; c < C; c += 32) yr[c] = expf(xr[c] - mx) / s;
}

} // namespace ncmb

using namespace ncmb;

extern "C" {

void embedding_fwd(const float *W, const int *idx, float *y, int64_t n, int D) { ensure_device(); embed_rows(W, idx, y, n, D); }
void layernorm_fwd(const float *x, const float *w, const float *b, float *y, int64_t rows, int C) { ensure_device(); layernorm(x, w, b, y, rows, C, 1e-6f); }
void layernorm_eps_fwd(const float *x, const float *w, const float *b, float *y, int64_t rows, int C, float eps) { ensure_device(); layernorm(x, w, b, y, rows, C, eps); }
void rmsnorm_fwd(const float *x, const float *w, float *y, int64_t rows, int C) { ensure_device(); rmsnorm(x, w, y, rows, C, C, C); }
static void act_api(const float *x, float *y, int64_t n, int act) {
    ensure_device();
    if (n <= 0) return;
    LAUNCH(k_act, ew_grid(n), 256, 0, x, y, n, act);
}
void gelu_fwd(const float *x, float *y, int64_t n) { act_api(x, y, n, ACT_GELU); }
void gelu_tanh_fwd(const float *x, float *y, int64_t n) { act_api(x, y, n, ACT_GELU_TANH); }
void silu_fwd(const float *x, float *y, int64_t n) { act_api(x, y, n, ACT_SILU); }
void softmax_fwd(const float *x, float *y, int64_t rows, int C) {
    ensure_device();
    if (rows > 0) LAUNCH(k_softmax, grid1d(rows, 8), 256, 0, x, y, rows, C);
}
void add_fwd(const float *a, const float *b, float *y, int64_t n) { ensure_device(); if (n > 0) LAUNCH(k_add, ew_grid(n), 256, 0, a, b, y, n); }
void mul_fwd(const float *a, const float *b, float *y, int64_t n) { ensure_device(); if (n > 0) LAUNCH(k_mul, ew_grid(n), 256, 0, a, b, y, n); }
void scale_fwd(const float *x, float s, float *y, int64_t n) { ensure_device(); if (n > 0) LAUNCH(k_scale, ew_grid(n), 256, 0, x, s, y, n); }
void add_inplace_fwd(float *y, const float *x, int64_t n) { ensure_device(); add_inplace(y, x, n); }
void heads_transpose_fwd_b(const float *in, float *out, int B, int64_t T, int H, int hd) {
    ensure_device();
    int64_t n = (int64_t)B * T * H * hd;
    if (n > 0) LAUNCH(k_heads_transpose_b, ew_grid(n), 256, 0, in, out, (int64_t)B, T, H, hd);
}
void heads_transpose_fwd(const float *in, float *out, int64_t T, int H, int hd) { heads_transpose_fwd_b(in, out, 1, T, H, hd); }
void qkv_split_fwd(const float *in, float *qq, float *kk, float *vv, int B, int T, int C, int H, int hd, int K, int rep) {
    ensure_device();
    int64_t n = (int64_t)B * H * T * hd;
    if (n > 0) LAUNCH(k_qkvsplit, ew_grid(n), 256, 0, in, qq, kk, vv, B, T, C, H, hd, K, rep);
}
void head_merge_fwd(const float *ctxp, float *out, int B, int T, int C, int H, int hd) {
    ensure_device();
    int64_t n = (int64_t)B * T * C;
    if (n > 0) LAUNCH(k_headmerge, ew_grid(n), 256, 0, ctxp, out, B, T, C, H, hd);
}

// Host-side helpers of the kernel API: they take HOST rows in the reference too
// (argmax over a downloaded logits row, src/main.c:854; sampling, src/gpt2.c:193-194).
int argmax_row(const float *x, int n) {
    int bi = 0; float bv = x[0];
    for (int i = 1; i < n; i++) if (x[i] > bv) { bv = x[i]; bi = i; }
    return bi;
}
unsigned long long rng_next(unsigned long long *state) {
    unsigned long long x = *state;
    x ^= x >> 12; x ^= x << 25; x ^= x >> 27;
    *state = x;
    return x * 0x2545F4914F6CDD1DULL;
}

} // extern "C"
