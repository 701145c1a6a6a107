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
    ProfScope ps(NCMB_K_GEMM, 2.0 * (double)g.M * g.N * g.K,
                 4.0 * ((double)g.M * g.K + (double)g.N * g.K + (double)g.M * g.N));
    // Few rows: the weights dominate the traffic and a 64x64 / 128x128 tiling would leave most
    // SMs idle, so stream each weight row once through one warp (decode-time GEMV / skinny GEMM).
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
