// fp32 CUDA-core GEMM: y = act(x W^T + bias) (+ res), both operands K-major.
// This is the exact-arithmetic engine (fp32 FMA accumulation): it serves shapes the
// tensor-core engine does not take (tiny M, odd K) and gemm mode 0, and it is what
// linear_fwd of the reference kernel API (src/ncm.h:146) maps to in that mode.
#include "common.cuh"

namespace ncmb {

__device__ __forceinline__ float act_fn(float v, int act) {
    switch (act) {
        case ACT_GELU: return 0.5f * v * (1.0f + erff(v * 0.7071067811865475f));
        case ACT_GELU_TANH: return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
        case ACT_SILU: return v / (1.0f + expf(-v));
        case ACT_RELU2: { float r = v > 0.f ? v : 0.f; return r * r; }
        default: return v;
    }
}

struct GemmDev {
    const float *x; int64_t ldx;
    const float *W;
    const float *bias;
    const float *res; int64_t ldres;
    float *y; int64_t ldy;
    int64_t M; int N, K;
    int act;
    int vec;        // 1: K % 4 == 0 and x / W rows are 16-byte aligned
    int ln_kind; const float *ln_w, *ln_b; float ln_eps;
    float *y2; int y2_col0; int64_t ldy2; const int *y2_step_d; int64_t y2_step;
    const unsigned short *W16;      // optional exact bf16 copy of W (GEMV kernel only): half the bytes to stream
};

// ---- tiled kernel: BM x BN output tile per CTA, BK-deep stages, TMxTN per thread ----
// Each thread owns two 4-wide column groups (tx*4 and BN/2 + tx*4) and two 4-high row
// groups, so shared-memory reads are conflict-free float4s.
template <int BM, int BN, int BK>
__global__ void __launch_bounds__((BM / 8) * (BN / 8)) k_gemm_tiled(GemmDev a) {
    constexpr int NT = (BM / 8) * (BN / 8);
    constexpr int LDA = BM + 4, LDB = BN + 4;
    __shared__ __align__(16) float As[2][BK][LDA];
    __shared__ __align__(16) float Bs[2][BK][LDB];
    const int tid = threadIdx.x;
    const int tx = tid % (BN / 8), ty = tid / (BN / 8);
    const int64_t m0 = (int64_t)blockIdx.y * BM;
    const int n0 = blockIdx.x * BN;
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = 0.f;

    constexpr int KQ = BK / 4;                    // float4 per tile row
    constexpr int A_ITERS = (BM * KQ + NT - 1) / NT;
    constexpr int B_ITERS = (BN * KQ + NT - 1) / NT;
    float4 ra[A_ITERS], rb[B_ITERS];

    auto gload = [&](int k0) {
#pragma unroll
        for (int it = 0; it < A_ITERS; it++) {
            int i = tid + it * NT;
            int row = i / KQ, kq = i % KQ;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            int64_t m = m0 + row;
            int k = k0 + kq * 4;
            if (i < BM * KQ && m < a.M) {
                const float *p = a.x + m * a.ldx + k;
                if (a.vec && k + 3 < a.K) v = *(const float4 *)p;
                else {
                    if (k < a.K) v.x = p[0];
                    if (k + 1 < a.K) v.y = p[1];
                    if (k + 2 < a.K) v.z = p[2];
                    if (k + 3 < a.K) v.w = p[3];
                }
            }
            ra[it] = v;
        }
#pragma unroll
        for (int it = 0; it < B_ITERS; it++) {
            int i = tid + it * NT;
            int row = i / KQ, kq = i % KQ;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            int n = n0 + row;
            int k = k0 + kq * 4;
            if (i < BN * KQ && n < a.N) {
                const float *p = a.W + (int64_t)n * a.K + k;
                if (a.vec && k + 3 < a.K) v = *(const float4 *)p;
                else {
                    if (k < a.K) v.x = p[0];
                    if (k + 1 < a.K) v.y = p[1];
                    if (k + 2 < a.K) v.z = p[2];
                    if (k + 3 < a.K) v.w = p[3];
                }
            }
            rb[it] = v;
        }
    };
    auto sstore = [&](int buf) {
#pragma unroll
        for (int it = 0; it < A_ITERS; it++) {
            int i = tid + it * NT;
            if (i < BM * KQ) {
                int row = i / KQ, kq = i % KQ;
                As[buf][kq * 4 + 0][row] = ra[it].x; As[buf][kq * 4 + 1][row] = ra[it].y;
                As[buf][kq * 4 + 2][row] = ra[it].z; As[buf][kq * 4 + 3][row] = ra[it].w;
            }
        }
#pragma unroll
        for (int it = 0; it < B_ITERS; it++) {
            int i = tid + it * NT;
            if (i < BN * KQ) {
                int row = i / KQ, kq = i % KQ;
                Bs[buf][kq * 4 + 0][row] = rb[it].x; Bs[buf][kq * 4 + 1][row] = rb[it].y;
                Bs[buf][kq * 4 + 2][row] = rb[it].z; Bs[buf][kq * 4 + 3][row] = rb[it].w;
            }
        }
    };

    const int nk = (a.K + BK - 1) / BK;
    gload(0);
    sstore(0);
    __syncthreads();
    for (int kt = 0; kt < nk; kt++) {
        int buf = kt & 1;
        if (kt + 1 < nk) gload((kt + 1) * BK);
#pragma unroll
        for (int k = 0; k < BK; k++) {
            float4 a0 = *(const float4 *)&As[buf][k][ty * 4];
            float4 a1 = *(const float4 *)&As[buf][k][BM / 2 + ty * 4];
            float4 b0 = *(const float4 *)&Bs[buf][k][tx * 4];
            float4 b1 = *(const float4 *)&Bs[buf][k][BN / 2 + tx * 4];
            float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < 8; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        if (kt + 1 < nk) sstore(buf ^ 1);
        __syncthreads();
    }
    // epilogue
#pragma unroll
    for (int i = 0; i < 8; i++) {
        int64_t m = m0 + (i < 4 ? ty * 4 + i : BM / 2 + ty * 4 + (i - 4));
        if (m >= a.M) continue;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            int n = n0 + (j < 4 ? tx * 4 + j : BN / 2 + tx * 4 + (j - 4));
            if (n >= a.N) continue;
            float v = acc[i][j];
            if (a.bias) v += a.bias[n];
            v = act_fn(v, a.act);
            if (a.res) v += a.res[m * a.ldres + n];
            a.y[m * a.ldy + n] = v;
        }
    }
}

// ---- skinny kernel (M small): one warp per output column, the weight row is streamed
// once with 128-bit loads and reused for up to MT activation rows held in registers. ----
template <int MT>
__global__ void __launch_bounds__(256) k_gemm_skinny(GemmDev a) {
    int warp = (int)(((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
    int lane = threadIdx.x & 31;
    if (warp >= a.N) return;
    const float *wr = a.W + (int64_t)warp * a.K;
    for (int64_t mb = 0; mb < a.M; mb += MT) {
        float acc[MT];
#pragma unroll
        for (int i = 0; i < MT; i++) acc[i] = 0.f;
        if (a.vec) {
            for (int k = lane * 4; k < a.K; k += 128) {
                float4 w = *(const float4 *)(wr + k);
#pragma unroll
                for (int i = 0; i < MT; i++) {
                    if (mb + i < a.M) {
                        float4 xv = *(const float4 *)(a.x + (mb + i) * a.ldx + k);
                        acc[i] = fmaf(xv.x, w.x, acc[i]); acc[i] = fmaf(xv.y, w.y, acc[i]);
                        acc[i] = fmaf(xv.z, w.z, acc[i]); acc[i] = fmaf(xv.w, w.w, acc[i]);
                    }
                }
            }
        } else {
            for (int k = lane; k < a.K; k += 32) {
                float w = wr[k];
#pragma unroll
                for (int i = 0; i < MT; i++)
                    if (mb + i < a.M) acc[i] = fmaf(a.x[(mb + i) * a.ldx + k], w, acc[i]);
            }
        }
#pragma unroll
        for (int i = 0; i < MT; i++) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
        }
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < MT; i++) {
                int64_t m = mb + i;
                if (m < a.M) {
                    float v = acc[i];
                    if (a.bias) v += a.bias[warp];
                    v = act_fn(v, a.act);
                    if (a.res) v += a.res[m * a.ldres + warp];
                    a.y[m * a.ldy + warp] = v;
                }
            }
        }
    }
}

// ---- GEMV-like kernel (M <= 8 rows per pass, vector path): one CTA per GV_NC output columns, all 256 threads
// stride over K together, so every thread has its 128-bit weight loads of all columns in flight at once
// (the weights are read exactly once, coalesced 512 bytes per warp and column); partial dot products are
// reduced by warp shuffles and one shared-memory pass. Decode steps (one token per sequence) live here: they
// are bound by streaming the weights, not by arithmetic.
// The kernel is launched with programmatic stream serialization: it lets its successor start at once
// (griddepcontrol.launch_dependents), requests the weights of its first GV_PF k-steps -- which no kernel of a
// decode step writes -- and only then waits for its predecessor (griddepcontrol.wait) before touching x. So
// the launch latency and the DRAM latency of the weight stream run under the previous kernel. ----
// four consecutive weights of row `row` at column k: fp32, or bf16 widened exactly (bits << 16)
__device__ __forceinline__ float4 gv_w4(const GemmDev &a, int64_t row, int k) {
    if (a.W16) {
        const uint2 u = __ldg((const uint2 *)(a.W16 + row * a.K + k));
        return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u),
                           __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
    }
    return __ldg((const float4 *)(a.W + row * a.K + k));
}

template <int MT, int GV_NC, int GV_PF>
__global__ void __launch_bounds__(256) k_gemv(GemmDev a) {
    __shared__ float red[8][MT][GV_NC];
    __shared__ float stat[8][MT], s_mean[MT], s_rstd[MT];
    const int n0 = blockIdx.x * GV_NC;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_launch_dependents();
    int64_t wr[GV_NC];                                   // weight rows of this CTA's columns
#pragma unroll
    for (int c = 0; c < GV_NC; c++) wr[c] = min(n0 + c, a.N - 1);
    float4 wpre[GV_PF][GV_NC];
#pragma unroll
    for (int p = 0; p < GV_PF; p++) {
        const int k = tid * 4 + p * 1024;
        if (k < a.K) {
#pragma unroll
            for (int c = 0; c < GV_NC; c++) wpre[p][c] = gv_w4(a, wr[c], k);
        }
    }
    pdl_wait();
    for (int64_t mb = 0; mb < a.M; mb += MT) {
        float acc[MT][GV_NC];
#pragma unroll
        for (int i = 0; i < MT; i++)
#pragma unroll
            for (int c = 0; c < GV_NC; c++) acc[i][c] = 0.f;
        if (a.ln_kind) {
            // row statistics of the MT input rows (every CTA repeats them: a row is a few KB out of L2)
            float mean[MT];
            for (int pass = 0; pass < 2; pass++) {
                if (pass == 0 && a.ln_kind == 2) {
#pragma unroll
                    for (int i = 0; i < MT; i++) mean[i] = 0.f;
                    continue;                                   // RMSNorm: no mean
                }
                float part[MT];
#pragma unroll
                for (int i = 0; i < MT; i++) part[i] = 0.f;
                for (int k = tid * 4; k < a.K; k += 1024) {
#pragma unroll
                    for (int i = 0; i < MT; i++) {
                        if (mb + i < a.M) {
                            const float4 v = *(const float4 *)(a.x + (mb + i) * a.ldx + k);
                            if (pass == 0) part[i] += (v.x + v.y) + (v.z + v.w);
                            else {
                                float d0 = v.x - mean[i], d1 = v.y - mean[i], d2 = v.z - mean[i], d3 = v.w - mean[i];
                                part[i] += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
                            }
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < MT; i++) {
                    float v = part[i];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                    if (lane == 0) stat[warp][i] = v;
                }
                __syncthreads();
                if (tid < MT) {
                    float v = 0.f;
#pragma unroll
                    for (int w8 = 0; w8 < 8; w8++) v += stat[w8][tid];
                    v /= (float)a.K;
                    if (pass == 0) s_mean[tid] = v; else s_rstd[tid] = 1.0f / sqrtf(v + a.ln_eps);
                }
                __syncthreads();
                if (pass == 0) {
#pragma unroll
                    for (int i = 0; i < MT; i++) mean[i] = s_mean[i];
                }
            }
        }
        auto kstep = [&](int k, const float4 *w) {
            float4 lw = make_float4(1.f, 1.f, 1.f, 1.f), lb = make_float4(0.f, 0.f, 0.f, 0.f);
            if (a.ln_kind) {
                if (a.ln_w) lw = __ldg((const float4 *)(a.ln_w + k));
                if (a.ln_b) lb = __ldg((const float4 *)(a.ln_b + k));
            }
#pragma unroll
            for (int i = 0; i < MT; i++) {
                if (mb + i < a.M) {
                    float4 xv = *(const float4 *)(a.x + (mb + i) * a.ldx + k);
                    if (a.ln_kind) {   // unfused mul / mul / add like the stand-alone norm kernels
                        const float mu = a.ln_kind == 1 ? s_mean[i] : 0.f, rs = s_rstd[i];
                        xv.x = __fadd_rn(__fmul_rn(__fmul_rn(xv.x - mu, rs), lw.x), lb.x);
                        xv.y = __fadd_rn(__fmul_rn(__fmul_rn(xv.y - mu, rs), lw.y), lb.y);
                        xv.z = __fadd_rn(__fmul_rn(__fmul_rn(xv.z - mu, rs), lw.z), lb.z);
                        xv.w = __fadd_rn(__fmul_rn(__fmul_rn(xv.w - mu, rs), lw.w), lb.w);
                    }
#pragma unroll
                    for (int c = 0; c < GV_NC; c++) {
                        acc[i][c] = fmaf(xv.x, w[c].x, acc[i][c]); acc[i][c] = fmaf(xv.y, w[c].y, acc[i][c]);
                        acc[i][c] = fmaf(xv.z, w[c].z, acc[i][c]); acc[i][c] = fmaf(xv.w, w[c].w, acc[i][c]);
                    }
                }
            }
        };
#pragma unroll
        for (int p = 0; p < GV_PF; p++) {
            const int k = tid * 4 + p * 1024;
            if (k < a.K) kstep(k, wpre[p]);
        }
        for (int k = tid * 4 + GV_PF * 1024; k < a.K; k += 1024) {
            float4 w[GV_NC];
#pragma unroll
            for (int c = 0; c < GV_NC; c++) w[c] = gv_w4(a, wr[c], k);
            kstep(k, w);
        }
#pragma unroll
        for (int i = 0; i < MT; i++)
#pragma unroll
            for (int c = 0; c < GV_NC; c++) {
                float v = acc[i][c];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0) red[warp][i][c] = v;
            }
        __syncthreads();
        if (tid < MT * GV_NC) {
            const int i = tid / GV_NC, c = tid % GV_NC;
            const int64_t m = mb + i; const int n = n0 + c;
            if (m < a.M && n < a.N) {
                float v = 0.f;
#pragma unroll
                for (int w8 = 0; w8 < 8; w8++) v += red[w8][i][c];
                if (a.bias) v += a.bias[n];
                v = act_fn(v, a.act);
                if (a.res) v += a.res[m * a.ldres + n];
                a.y[m * a.ldy + n] = v;
                if (a.y2 && n >= a.y2_col0)
                    a.y2[m * a.ldy2 + (a.y2_step_d ? (int64_t)(*a.y2_step_d) * a.y2_step : 0) + (n - a.y2_col0)] = v;
            }
        }
        __syncthreads();
    }
}

void gemm_simt(const GemmArgs &g) {
    if (g.M <= 0 || g.N <= 0) return;
    if (g.glu) fatal("gemm_simt: fused gated epilogue is a tensor-core engine feature");
    GemmDev d;
    d.x = g.x; d.ldx = g.ldx ? g.ldx : g.K;
    d.W = g.W; d.bias = g.bias;
    d.res = g.res; d.ldres = g.ldres ? g.ldres : g.N;
    d.y = g.y; d.ldy = g.ldy ? g.ldy : g.N;
    d.M = g.M; d.N = g.N; d.K = g.K; d.act = g.act;
    d.vec = (g.K % 4 == 0) && (d.ldx % 4 == 0) && (((uintptr_t)g.x & 15) == 0) && (((uintptr_t)g.W & 15) == 0);
    d.W16 = (g.M <= 16 && d.vec) ? g.W16 : nullptr;
    d.ln_kind = g.ln_kind; d.ln_w = g.ln_w; d.ln_b = g.ln_b; d.ln_eps = g.ln_eps;
    d.y2 = g.y2; d.y2_col0 = g.y2_col0; d.ldy2 = g.ldy2; d.y2_step_d = g.y2_step_d; d.y2_step = g.y2_step;
    if ((g.ln_kind || g.y2) && !(g.M <= 16 && d.vec)) fatal("gemm_simt: fused norm / second output on a call the GEMV kernel does not take");
    ProfScope ps(NCMB_K_GEMM, 2.0 * (double)g.M * g.N * g.K,
                 4.0 * ((double)g.M * g.K + (double)g.N * g.K + (double)g.M * g.N));
    // Few rows: the weights dominate the traffic and a 64x64 / 128x128 tiling would leave most
    // SMs idle, so stream each weight row once through one warp (decode-time GEMV / skinny GEMM).
    if (g.M <= 16 && d.vec) {
        // columns per CTA: more of them when there are many, so a CTA moves tens of KB per launch-and-reduce
        // cycle and a few waves cover the matrix (N = vocabulary: 16 columns; MLP widths: 8)
        const int nc = (g.M <= 2 && g.N >= 32768) ? 16 : (g.M <= 4 && g.N >= 2048) ? 8 : 4;
        unsigned grid = (unsigned)cdiv(g.N, nc);
        if (nc == 16) {
            if (g.M <= 1) LAUNCH_PDL((k_gemv<1, 16, 1>), grid, 256, 0, d);
            else LAUNCH_PDL((k_gemv<2, 16, 1>), grid, 256, 0, d);
        } else if (nc == 8) {
            if (g.M <= 1) LAUNCH_PDL((k_gemv<1, 8, 2>), grid, 256, 0, d);
            else if (g.M <= 2) LAUNCH_PDL((k_gemv<2, 8, 1>), grid, 256, 0, d);
            else LAUNCH_PDL((k_gemv<4, 8, 1>), grid, 256, 0, d);
        } else {
            if (g.M <= 1) LAUNCH_PDL((k_gemv<1, 4, 3>), grid, 256, 0, d);
            else if (g.M <= 2) LAUNCH_PDL((k_gemv<2, 4, 3>), grid, 256, 0, d);
            else if (g.M <= 4) LAUNCH_PDL((k_gemv<4, 4, 3>), grid, 256, 0, d);
            else LAUNCH_PDL((k_gemv<8, 4, 2>), grid, 256, 0, d);
        }
        return;
    }
    if (g.M <= 16) {
        unsigned grid = grid1d((int64_t)g.N * 32, 256);
        if (g.M <= 1) LAUNCH(k_gemm_skinny<1>, grid, 256, 0, d);
        else if (g.M <= 4) LAUNCH(k_gemm_skinny<4>, grid, 256, 0, d);
        else LAUNCH(k_gemm_skinny<8>, grid, 256, 0, d);
        return;
    }
    int64_t big = cdiv(g.M, 128) * cdiv(g.N, 128);
    if (big >= ctx().sm_count) {
        dim3 grid((unsigned)cdiv(g.N, 128), (unsigned)cdiv(g.M, 128));
        LAUNCH((k_gemm_tiled<128, 128, 16>), grid, 256, 0, d);
    } else {
        dim3 grid((unsigned)cdiv(g.N, 64), (unsigned)cdiv(g.M, 64));
        LAUNCH((k_gemm_tiled<64, 64, 16>), grid, 64, 0, d);
    }
}

bool gemv_fusable(const GemmArgs &g) {
    int64_t ldx = g.ldx ? g.ldx : g.K;
    return g.M <= 16 && g.M > 0 && !g.glu && !g.x_lo && !g.y_lo && (g.K % 4 == 0) && (ldx % 4 == 0) &&
           (((uintptr_t)g.x & 15) == 0) && (((uintptr_t)g.W & 15) == 0) &&
           (!g.ln_w || ((uintptr_t)g.ln_w & 15) == 0) && (!g.ln_b || ((uintptr_t)g.ln_b & 15) == 0);
}

void gemm(const GemmArgs &a) {
    const int mode = ctx().gemm_mode;
    // a pre-split input names its engine; otherwise mode 3 prefers the fp16-pair kernel
    if (a.x_lo && a.x_fmt == SPLIT_H16) {
        if (!gemm_h3_supported(a)) fatal("gemm: fp16-pair operands for a shape the fp16-pair kernel does not take (M=%lld N=%d K=%d)", (long long)a.M, a.N, a.K);
        gemm_h3(a); return;
    }
    if (mode >= 3 && !a.x_lo && gemm_h3_supported(a)) { gemm_h3(a); return; }
    if (mode >= 1 && gemm_tc_supported(a)) { gemm_tc(a); return; }
    if (a.x_lo || a.y_lo) fatal("gemm: split operands reached the CUDA-core engine (M=%lld N=%d K=%d)", (long long)a.M, a.N, a.K);
    gemm_simt(a);
}

} // namespace ncmb

extern "C" void linear_fwd(const float *x, const float *W, const float *b, float *y, int64_t batch, int M, int K) {
    ncmb::ensure_device();
    ncmb::GemmArgs a;
    a.x = x; a.ldx = K; a.W = W; a.bias = b; a.y = y; a.ldy = M;
    a.M = batch; a.N = M; a.K = K;
    ncmb::gemm(a);
}
