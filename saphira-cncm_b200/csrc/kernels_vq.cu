// Small strided kernels behind the quantizer's resampling path: conv1d /
// conv-transpose1d / GroupNorm / area and linear resampling. Every kernel takes
// explicit (batch, channel, time) strides, so the same code serves the reference
// kernel API's channel-major [N][C][T] tensors (src/ncm.h:172-180) and the
// token-major [N][T][C] tensors the generate path keeps (no transposes on the path).
#include "common.cuh"

namespace ncmb {

// mode 0: y = conv; 1: y = add + conv; 2: y = (1-r)*add + r*conv (r = alpha), add read with y's strides
__global__ void k_conv1d(const float *__restrict__ x, NCT xs, const float *__restrict__ W,
                         const float *__restrict__ b, float *__restrict__ y, NCT ys,
                         int N, int Cin, int Cout, int T, int Tout, int K, int stride, int pad,
                         const float *__restrict__ add, float alpha, int mode) {
    int64_t total = (int64_t)N * Cout * Tout;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int co = (int)(i % Cout); int t = (int)((i / Cout) % Tout); int n = (int)(i / ((int64_t)Cout * Tout));
        float acc = b ? b[co] : 0.f;
        const float *wr = W + (int64_t)co * Cin * K;
        for (int ci = 0; ci < Cin; ci++) {
            const float *xc = x + n * xs.sn + ci * xs.sc;
            for (int kk = 0; kk < K; kk++) {
                int ti = t * stride + kk - pad;
                if (ti < 0 || ti >= T) continue;
                acc = fmaf(xc[ti * xs.st], wr[ci * K + kk], acc);
            }
        }
        int64_t o = n * ys.sn + co * ys.sc + t * ys.st;
        if (mode == 1) acc = __fadd_rn(add[o], acc);
        else if (mode == 2) acc = __fadd_rn(__fmul_rn(1.0f - alpha, add[o]), __fmul_rn(alpha, acc));
        y[o] = acc;
    }
}

// weight layout [Cin][Cout][K] (torch ConvTranspose1d), no padding
__global__ void k_convT1d(const float *__restrict__ x, NCT xs, const float *__restrict__ W,
                          const float *__restrict__ b, float *__restrict__ y, NCT ys,
                          int N, int Cin, int Cout, int T, int Tout, int K, int stride) {
    int64_t total = (int64_t)N * Cout * Tout;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int co = (int)(i % Cout); int t = (int)((i / Cout) % Tout); int n = (int)(i / ((int64_t)Cout * Tout));
        float acc = b ? b[co] : 0.f;
        if (K == stride) {                    // non-overlapping taps (the up-cascade): exactly one (input step, tap) per output step
            const int ti = t / stride, kk = t - ti * stride;
            if (ti < T) {
                const float *xc = x + n * xs.sn + ti * xs.st;
                const float *wc = W + (int64_t)co * K + kk;
                for (int ci = 0; ci < Cin; ci++) acc = fmaf(xc[ci * xs.sc], wc[(int64_t)ci * Cout * K], acc);
            }
            y[n * ys.sn + co * ys.sc + t * ys.st] = acc;
            continue;
        }
        for (int ci = 0; ci < Cin; ci++) {
            const float *xc = x + n * xs.sn + ci * xs.sc;
            for (int kk = 0; kk < K; kk++) {
                int num = t - kk;
                if (num < 0 || num % stride != 0) continue;
                int ti = num / stride;
                if (ti >= T) continue;
                acc = fmaf(xc[ti * xs.st], W[((int64_t)ci * Cout + co) * K + kk], acc);
            }
        }
        y[n * ys.sn + co * ys.sc + t * ys.st] = acc;
    }
}

// affine-free GroupNorm, eps 1e-5: one CTA per (n, group), statistics over Cg x T
__global__ void __launch_bounds__(128) k_groupnorm(const float *__restrict__ x, NCT xs, float *__restrict__ y, NCT ys,
                                                   int G, int C, int T) {
    int n = blockIdx.x / G, g = blockIdx.x % G;
    int Cg = C / G, cnt = Cg * T;
    __shared__ float red[128];
    __shared__ float stat[2];
    float s = 0.f;
    for (int i = threadIdx.x; i < cnt; i += 128) {
        int c = g * Cg + i / T, t = i % T;
        s += x[n * xs.sn + c * xs.sc + t * xs.st];
    }
    red[threadIdx.x] = s; __syncthreads();
    for (int o = 64; o > 0; o >>= 1) { if ((int)threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o]; __syncthreads(); }
    if (threadIdx.x == 0) stat[0] = red[0] / (float)cnt;
    __syncthreads();
    float mean = stat[0], q = 0.f;
    for (int i = threadIdx.x; i < cnt; i += 128) {
        int c = g * Cg + i / T, t = i % T;
        float d = x[n * xs.sn + c * xs.sc + t * xs.st] - mean;
        q += d * d;
    }
    __syncthreads();
    red[threadIdx.x] = q; __syncthreads();
    for (int o = 64; o > 0; o >>= 1) { if ((int)threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o]; __syncthreads(); }
    if (threadIdx.x == 0) stat[1] = 1.0f / sqrtf(red[0] / (float)cnt + 1e-5f);
    __syncthreads();
    float inv = stat[1];
    for (int i = threadIdx.x; i < cnt; i += 128) {
        int c = g * Cg + i / T, t = i % T;
        y[n * ys.sn + c * ys.sc + t * ys.st] = (x[n * xs.sn + c * xs.sc + t * xs.st] - mean) * inv;
    }
}

// ATen "area": equal-weight mean over [floor(t*Tin/Tout), ceil((t+1)*Tin/Tout))
__global__ void k_interp_area(const float *__restrict__ x, NCT xs, float *__restrict__ y, NCT ys,
                              int N, int C, int Tin, int Tout) {
    int64_t total = (int64_t)N * C * Tout;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int c = (int)(i % C); int t = (int)((i / C) % Tout); int n = (int)(i / ((int64_t)C * Tout));
        int s = (int)(((int64_t)t * Tin) / Tout);
        int e = (int)(((int64_t)(t + 1) * Tin + Tout - 1) / Tout);
        if (e <= s) e = s + 1;
        if (e > Tin) e = Tin;
        const float *xc = x + n * xs.sn + c * xs.sc;
        float acc = 0.f;
        for (int k = s; k < e; k++) acc += xc[k * xs.st];
        y[n * ys.sn + c * ys.sc + t * ys.st] = acc / (float)(e - s);
    }
}

// ATen "linear", align_corners=False; mean when either length is 1
__global__ void k_interp_linear(const float *__restrict__ x, NCT xs, float *__restrict__ y, NCT ys,
                                int N, int C, int Tin, int Tout) {
    int64_t total = (int64_t)N * C * Tout;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int c = (int)(i % C); int t = (int)((i / C) % Tout); int n = (int)(i / ((int64_t)C * Tout));
        const float *xc = x + n * xs.sn + c * xs.sc;
        float out;
        if (Tout == 1 || Tin == 1) {
            float acc = 0.f;
            for (int k = 0; k < Tin; k++) acc += xc[k * xs.st];
            out = acc / (float)Tin;
        } else {
            double scale = (double)Tin / Tout;
            double src = (t + 0.5) * scale - 0.5;
            int s0 = (int)floor(src);
            double w1 = src - s0, w0 = 1.0 - w1;
            int i0 = s0 < 0 ? 0 : (s0 >= Tin ? Tin - 1 : s0);
            int s1 = s0 + 1;
            int i1 = s1 < 0 ? 0 : (s1 >= Tin ? Tin - 1 : s1);
            out = (float)(w0 * (double)xc[i0 * xs.st] + w1 * (double)xc[i1 * xs.st]);
        }
        y[n * ys.sn + c * ys.sc + t * ys.st] = out;
    }
}

__global__ void k_l2sq(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ d2,
                       int64_t rows, int64_t cols, int C) {
    int64_t total = rows * cols;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t r = i / cols, j = i % cols;
        float s = 0.f;
        for (int c = 0; c < C; c++) { float d = a[r * C + c] - b[j * C + c]; s = fmaf(d, d, s); }
        d2[i] = s;
    }
}

static unsigned vq_grid(int64_t n) {
    int64_t g = cdiv(n, 128);
    int64_t cap = (int64_t)ctx().sm_count * 32;
    if (g > cap) g = cap;
    return (unsigned)(g < 1 ? 1 : g);
}

void conv1d(const float *x, NCT xs, const float *W, const float *b, float *y, NCT ys,
            int N, int Cin, int Cout, int T, int K, int stride, int pad, const float *add, float alpha) {
    int Tout = (T + 2 * pad - K) / stride + 1;
    int64_t n = (int64_t)N * Cout * Tout;
    if (n <= 0) return;
    int mode = !add ? 0 : (alpha == 0.f ? 1 : 2);
    ProfScope ps(NCMB_K_VQ, 2.0 * n * Cin * K, 0);
    LAUNCH(k_conv1d, vq_grid(n), 128, 0, x, xs, W, b, y, ys, N, Cin, Cout, T, Tout, K, stride, pad, add, alpha, mode);
}
void convT1d(const float *x, NCT xs, const float *W, const float *b, float *y, NCT ys,
             int N, int Cin, int Cout, int T, int K, int stride) {
    int Tout = (T - 1) * stride + K;
    int64_t n = (int64_t)N * Cout * Tout;
    if (n <= 0) return;
    ProfScope ps(NCMB_K_VQ, 2.0 * n * Cin, 0);
    LAUNCH(k_convT1d, vq_grid(n), 128, 0, x, xs, W, b, y, ys, N, Cin, Cout, T, Tout, K, stride);
}
void groupnorm(const float *x, NCT xs, float *y, NCT ys, int N, int G, int C, int T) {
    if (N <= 0) return;
    ProfScope ps(NCMB_K_VQ);
    LAUNCH(k_groupnorm, (unsigned)(N * G), 128, 0, x, xs, y, ys, G, C, T);
}
void interp_area(const float *x, NCT xs, float *y, NCT ys, int N, int C, int Tin, int Tout) {
    int64_t n = (int64_t)N * C * Tout;
    if (n <= 0) return;
    ProfScope ps(NCMB_K_VQ);
    LAUNCH(k_interp_area, vq_grid(n), 128, 0, x, xs, y, ys, N, C, Tin, Tout);
}
void interp_linear(const float *x, NCT xs, float *y, NCT ys, int N, int C, int Tin, int Tout) {
    int64_t n = (int64_t)N * C * Tout;
    if (n <= 0) return;
    ProfScope ps(NCMB_K_VQ);
    LAUNCH(k_interp_linear, vq_grid(n), 128, 0, x, xs, y, ys, N, C, Tin, Tout);
}

} // namespace ncmb

using namespace ncmb;

extern "C" {

void conv1d_fwd(const float *x, const float *W, const float *b, float *y, int N, int Cin, int Cout, int T, int K, int stride, int pad) {
    ensure_device();
    int Tout = (T + 2 * pad - K) / stride + 1;
    conv1d(x, ncl(Cin, T), W, b, y, ncl(Cout, Tout), N, Cin, Cout, T, K, stride, pad, nullptr, 0.f);
}
void convtranspose1d_fwd(const float *x, const float *W, const float *b, float *y, int N, int Cin, int Cout, int T, int K, int stride) {
    ensure_device();
    int Tout = (T - 1) * stride + K;
    convT1d(x, ncl(Cin, T), W, b, y, ncl(Cout, Tout), N, Cin, Cout, T, K, stride);
}
void groupnorm_fwd(const float *x, float *y, int N, int G, int C, int T) {
    ensure_device();
    groupnorm(x, ncl(C, T), y, ncl(C, T), N, G, C, T);
}
void interpolate_area_fwd(const float *x, float *y, int N, int C, int Tin, int Tout) {
    ensure_device();
    interp_area(x, ncl(C, Tin), y, ncl(C, Tout), N, C, Tin, Tout);
}
void interpolate_linear_fwd(const float *x, float *y, int N, int C, int Tin, int Tout) {
    ensure_device();
    interp_linear(x, ncl(C, Tin), y, ncl(C, Tout), N, C, Tin, Tout);
}
void rowwise_l2sq(const float *a, const float *b, float *d2, int64_t rows, int64_t colsA, int C) {
    ensure_device();
    int64_t n = rows * colsA;
    if (n <= 0) return;
    ProfScope ps(NCMB_K_VQ, 3.0 * n * C, 4.0 * n);
    LAUNCH(k_l2sq, vq_grid(n), 128, 0, a, b, d2, rows, colsA, C);
}

} // extern "C"
