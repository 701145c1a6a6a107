// Attention kernels.
//
//  * attention(): token-major fused SDPA for the generate / decode paths. Queries,
//    keys and values are read straight out of the fused projection buffers
//    ([token][heads*hd]) and the context is written token-major, so no head
//    split / merge pass exists. Each row (sequence) attends to up to two key
//    segments (a cached prefix and the tokens of the current pass); masked keys
//    are never visited instead of being added as -inf (exp(-inf) contributes
//    exactly 0 in the reference, src/kernels.c:484-503, so skipping is exact).
//    Streaming (online) softmax over 64-key tiles staged in shared memory: no
//    [Tq][Tkv] score scratch, unlike the reference's k_sdpa (src/kernels.c:364-389).
//  * sdpa_masked(): the reference kernel API (head-major tensors, additive mask).
//  * qk_post(): per-head RMSNorm (optional) + rotary embedding, in place.
#include "common.cuh"
#include "split.cuh"

namespace ncmb {

constexpr int AT_KT = 64;      // keys per shared-memory tile
constexpr int AT_WARPS = 4;
constexpr int AT_QW = 8;       // queries per warp
constexpr int AT_QT = AT_WARPS * AT_QW;

struct AttnDev {
    const float *q; int64_t ldq;
    const float *k1, *v1; int64_t ldk1;
    const float *k2, *v2; int64_t ldk2;
    float *out; float *out_lo; int64_t ldo; int out_fmt;
    const int *q_start, *k1_start, *k2_start, *k1_len;
    int H, Hkv, hd;
    int causal, causal_off, window;
    float scale;
};

template <int HD>
__global__ void __launch_bounds__(AT_WARPS * 32) k_attention(AttnDev a) {
    constexpr int LDK = HD + 4;
    constexpr int DPL = (HD + 31) / 32;          // output dims per lane
    extern __shared__ __align__(16) float smem[];
    float *Ks = smem;                             // [AT_KT][LDK]
    float *Vs = Ks + AT_KT * LDK;                 // [AT_KT][HD]
    float *Qs = Vs + AT_KT * HD;                  // [AT_QT][HD]
    float *Ps = Qs + AT_QT * HD;                  // [AT_WARPS][AT_QW][AT_KT]

    const int row = blockIdx.z, h = blockIdx.y, qt = blockIdx.x;
    const int q0 = a.q_start[row], nq = a.q_start[row + 1] - q0;
    if (qt * AT_QT >= nq) return;
    const int k10 = a.k1_start[row], n1 = a.k1_len ? a.k1_len[row] : a.k1_start[row + 1] - k10;
    const int k20 = a.k2_start ? a.k2_start[row] : 0;
    const int n2 = a.k2_start ? a.k2_start[row + 1] - k20 : 0;
    const int nk = n1 + n2;
    const int kvh = h / (a.H / a.Hkv);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // stage this block's queries (pre-scaled by nothing; the scale is applied to the score)
    for (int i = tid; i < AT_QT * (HD / 4); i += AT_WARPS * 32) {
        int t = i / (HD / 4), d4 = i % (HD / 4);
        int qi = qt * AT_QT + t;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (qi < nq) v = *(const float4 *)(a.q + (int64_t)(q0 + qi) * a.ldq + h * HD + d4 * 4);
        *(float4 *)(Qs + t * HD + d4 * 4) = v;
    }
    float m[AT_QW], l[AT_QW], o[AT_QW][DPL];
#pragma unroll
    for (int t = 0; t < AT_QW; t++) {
        m[t] = -INFINITY; l[t] = 0.f;
#pragma unroll
        for (int i = 0; i < DPL; i++) o[t][i] = 0.f;
    }
    float *Pw = Ps + warp * AT_QW * AT_KT;

    for (int kt0 = 0; kt0 < nk; kt0 += AT_KT) {
        __syncthreads();                           // previous tile fully consumed (and Qs visible)
        for (int i = tid; i < AT_KT * (HD / 4); i += AT_WARPS * 32) {
            int r = i / (HD / 4), d4 = i % (HD / 4);
            int j = kt0 + r;
            float4 kv = make_float4(0.f, 0.f, 0.f, 0.f), vv = kv;
            if (j < nk) {
                const float *kp, *vp;
                if (j < n1) { int64_t tok = k10 + j; kp = a.k1 + tok * a.ldk1; vp = a.v1 + tok * a.ldk1; }
                else { int64_t tok = k20 + (j - n1); kp = a.k2 + tok * a.ldk2; vp = a.v2 + tok * a.ldk2; }
                kv = *(const float4 *)(kp + kvh * HD + d4 * 4);
                vv = *(const float4 *)(vp + kvh * HD + d4 * 4);
            }
            *(float4 *)(Ks + r * LDK + d4 * 4) = kv;
            *(float4 *)(Vs + r * HD + d4 * 4) = vv;
        }
        __syncthreads();
        // scores: lane owns keys (lane, lane + 32) of the tile, for the warp's AT_QW queries
        float s0[AT_QW], s1[AT_QW];
#pragma unroll
        for (int t = 0; t < AT_QW; t++) { s0[t] = 0.f; s1[t] = 0.f; }
#pragma unroll 4
        for (int d4 = 0; d4 < HD / 4; d4++) {
            float4 ka = *(const float4 *)(Ks + lane * LDK + d4 * 4);
            float4 kb = *(const float4 *)(Ks + (lane + 32) * LDK + d4 * 4);
#pragma unroll
            for (int t = 0; t < AT_QW; t++) {
                float4 qv = *(const float4 *)(Qs + (warp * AT_QW + t) * HD + d4 * 4);
                s0[t] = fmaf(qv.x, ka.x, s0[t]); s0[t] = fmaf(qv.y, ka.y, s0[t]);
                s0[t] = fmaf(qv.z, ka.z, s0[t]); s0[t] = fmaf(qv.w, ka.w, s0[t]);
                s1[t] = fmaf(qv.x, kb.x, s1[t]); s1[t] = fmaf(qv.y, kb.y, s1[t]);
                s1[t] = fmaf(qv.z, kb.z, s1[t]); s1[t] = fmaf(qv.w, kb.w, s1[t]);
            }
        }
        const int ja = kt0 + lane, jb = kt0 + lane + 32;
#pragma unroll
        for (int t = 0; t < AT_QW; t++) {
            int qi = qt * AT_QT + warp * AT_QW + t;
            bool va = ja < nk, vb = jb < nk;
            if (a.causal) {                        // applies to segment-1 keys only
                if (ja < n1 && ja > qi + a.causal_off) va = false;
                if (jb < n1 && jb > qi + a.causal_off) vb = false;
            }
            if (a.window > 0) {
                int da = ja - qi, db = jb - qi;
                if (da < 0) da = -da;
                if (db < 0) db = -db;
                if (da > a.window) va = false;
                if (db > a.window) vb = false;
            }
            float x0 = va ? s0[t] * a.scale : -INFINITY;
            float x1 = vb ? s1[t] * a.scale : -INFINITY;
            float mx = fmaxf(x0, x1);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            float mnew = fmaxf(m[t], mx);
            float p0 = 0.f, p1 = 0.f, alpha = 1.f;
            if (mnew != -INFINITY) {
                p0 = va ? expf(x0 - mnew) : 0.f;
                p1 = vb ? expf(x1 - mnew) : 0.f;
                alpha = (m[t] == -INFINITY) ? 0.f : expf(m[t] - mnew);
            }
            float ps = p0 + p1;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
            l[t] = l[t] * alpha + ps;
            m[t] = mnew;
#pragma unroll
            for (int i = 0; i < DPL; i++) o[t][i] *= alpha;
            Pw[t * AT_KT + lane] = p0;
            Pw[t * AT_KT + lane + 32] = p1;
        }
        __syncwarp();
        // o += P V: lane owns output dims lane + 32*i
        const int jmax = (nk - kt0) < AT_KT ? (nk - kt0) : AT_KT;
        for (int j4 = 0; j4 < jmax; j4 += 4) {
            float vv[4][DPL];
#pragma unroll
            for (int jj = 0; jj < 4; jj++)
#pragma unroll
                for (int i = 0; i < DPL; i++) {
                    int d = lane + 32 * i;
                    vv[jj][i] = (d < HD) ? Vs[(j4 + jj) * HD + d] : 0.f;   // rows beyond nk hold zeros
                }
#pragma unroll
            for (int t = 0; t < AT_QW; t++) {
                float4 p = *(const float4 *)(Pw + t * AT_KT + j4);
#pragma unroll
                for (int i = 0; i < DPL; i++) {
                    o[t][i] = fmaf(p.x, vv[0][i], o[t][i]); o[t][i] = fmaf(p.y, vv[1][i], o[t][i]);
                    o[t][i] = fmaf(p.z, vv[2][i], o[t][i]); o[t][i] = fmaf(p.w, vv[3][i], o[t][i]);
                }
            }
        }
        __syncwarp();
    }
#pragma unroll
    for (int t = 0; t < AT_QW; t++) {
        int qi = qt * AT_QT + warp * AT_QW + t;
        if (qi >= nq) continue;
        float inv = l[t] > 0.f ? 1.0f / l[t] : 0.f;
#pragma unroll
        for (int i = 0; i < DPL; i++) {
            int d = lane + 32 * i;
            if (d < HD) {
                float v = o[t][i] * inv;
                int64_t at = (int64_t)(q0 + qi) * a.ldo + h * HD + d;
                if (a.out_lo) store_split1(a.out, a.out_lo, at, v, a.out_fmt);
                else a.out[at] = v;
            }
        }
    }
}

template <int HD>
static void launch_attention(const AttnDev &d, dim3 grid) {
    size_t smem = sizeof(float) * ((size_t)AT_KT * (HD + 4) + (size_t)AT_KT * HD + (size_t)AT_QT * HD +
                                   (size_t)AT_WARPS * AT_QW * AT_KT);
    static bool set = false;
    if (!set) {
        CUDA_CHECK(cudaFuncSetAttribute(k_attention<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        set = true;
    }
    LAUNCH(k_attention<HD>, grid, AT_WARPS * 32, smem, d);
}

void attention(const AttnArgs &a) {
    if (a.rows <= 0 || a.max_q <= 0) return;
    if (attention_decode_supported(a)) { attention_decode(a); return; }
    if (ctx().gemm_mode >= 1 && attention_tc_supported(a)) { attention_tc(a); return; }
    if (ctx().gemm_mode >= 1 && attention_tc_long_supported(a)) { attention_tc_long(a); return; }
    if (a.step_d) fatal("attention: a step-indexed plan reached a kernel that does not read the step counter");
    AttnDev d;
    d.q = a.q; d.ldq = a.ldq; d.k1 = a.k1; d.v1 = a.v1; d.ldk1 = a.ldk1;
    d.k2 = a.k2; d.v2 = a.v2; d.ldk2 = a.ldk2; d.out = a.out; d.out_lo = a.out_lo; d.ldo = a.ldo; d.out_fmt = a.out_fmt;
    d.q_start = a.q_start; d.k1_start = a.k1_start; d.k2_start = a.k2_start; d.k1_len = a.k1_len;
    d.H = a.H; d.Hkv = a.Hkv; d.hd = a.hd;
    d.causal = a.causal; d.causal_off = a.causal_off; d.window = a.window;
    d.scale = 1.0f / sqrtf((float)a.hd);
    if ((a.ldq | a.ldk1 | a.ldk2 | a.ldo) % 4) fatal("attention: row strides must be multiples of 4 floats");
    dim3 grid((unsigned)cdiv(a.max_q, AT_QT), (unsigned)a.H, (unsigned)a.rows);
    ProfScope ps(NCMB_K_ATTN, 4.0 * (double)a.total_q * a.avg_keys * a.H * a.hd, 0);
    switch (a.hd) {
        case 8: launch_attention<8>(d, grid); break;
        case 16: launch_attention<16>(d, grid); break;
        case 32: launch_attention<32>(d, grid); break;
        case 64: launch_attention<64>(d, grid); break;
        case 128: launch_attention<128>(d, grid); break;
        default: fatal("attention: head dim %d not supported (8, 16, 32, 64, 128)", a.hd);
    }
}

// ---- reference-layout SDPA with additive mask: one warp per (b, h, tq), 32-key chunks ----
template <int DPL>
__global__ void __launch_bounds__(128) k_sdpa_masked(const float *__restrict__ q, const float *__restrict__ k,
                                                    const float *__restrict__ v, const float *__restrict__ mask,
                                                    float *__restrict__ out, int B, int Hq, int Hkv, int Tq, int Tkv,
                                                    int hd, float scale) {
    int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (w >= (int64_t)B * Hq * Tq) return;
    int tq = (int)(w % Tq); int h = (int)((w / Tq) % Hq); int b = (int)(w / ((int64_t)Tq * Hq));
    int kvh = h / (Hq / Hkv);
    const float *qr = q + (((int64_t)b * Hq + h) * Tq + tq) * hd;
    const float *kb = k + ((int64_t)b * Hkv + kvh) * Tkv * hd;
    const float *vb = v + ((int64_t)b * Hkv + kvh) * Tkv * hd;
    float m = -INFINITY, l = 0.f, o[DPL];
#pragma unroll
    for (int i = 0; i < DPL; i++) o[i] = 0.f;
    for (int j0 = 0; j0 < Tkv; j0 += 32) {
        int j = j0 + lane;
        float s = -INFINITY;
        if (j < Tkv) {
            float acc = 0.f;
            const float *kr = kb + (int64_t)j * hd;
            for (int d = 0; d < hd; d++) acc = fmaf(qr[d], kr[d], acc);
            s = acc * scale;
            if (mask) s += mask[(int64_t)tq * Tkv + j];
        }
        float mx = s;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        float mnew = fmaxf(m, mx);
        float p = 0.f, alpha = 1.f;
        if (mnew != -INFINITY) {
            p = (s == -INFINITY) ? 0.f : expf(s - mnew);
            alpha = (m == -INFINITY) ? 0.f : expf(m - mnew);
        }
        float ps = p;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
        l = l * alpha + ps; m = mnew;
#pragma unroll
        for (int i = 0; i < DPL; i++) o[i] *= alpha;
        int jn = (Tkv - j0) < 32 ? (Tkv - j0) : 32;
        for (int jj = 0; jj < jn; jj++) {
            float pj = __shfl_sync(0xffffffffu, p, jj);
            const float *vr = vb + (int64_t)(j0 + jj) * hd;
#pragma unroll
            for (int i = 0; i < DPL; i++) { int d = lane + 32 * i; if (d < hd) o[i] = fmaf(pj, vr[d], o[i]); }
        }
    }
    float inv = l > 0.f ? 1.0f / l : 0.f;
    float *orow = out + (((int64_t)b * Hq + h) * Tq + tq) * hd;
#pragma unroll
    for (int i = 0; i < DPL; i++) { int d = lane + 32 * i; if (d < hd) orow[d] = o[i] * inv; }
}

void sdpa_masked(const float *q, const float *k, const float *v, const float *mask, float *out,
                 int B, int Hq, int Hkv, int Tq, int Tkv, int hd) {
    int64_t warps = (int64_t)B * Hq * Tq;
    if (warps <= 0) return;
    if (hd > 256) fatal("sdpa: head dim %d > 256", hd);
    float scale = 1.0f / sqrtf((float)hd);
    ProfScope ps(NCMB_K_ATTN, 4.0 * (double)warps * Tkv * hd, 0);
    unsigned grid = grid1d(warps * 32, 128);
    if (hd <= 32) LAUNCH(k_sdpa_masked<1>, grid, 128, 0, q, k, v, mask, out, B, Hq, Hkv, Tq, Tkv, hd, scale);
    else if (hd <= 64) LAUNCH(k_sdpa_masked<2>, grid, 128, 0, q, k, v, mask, out, B, Hq, Hkv, Tq, Tkv, hd, scale);
    else if (hd <= 128) LAUNCH(k_sdpa_masked<4>, grid, 128, 0, q, k, v, mask, out, B, Hq, Hkv, Tq, Tkv, hd, scale);
    else LAUNCH(k_sdpa_masked<8>, grid, 128, 0, q, k, v, mask, out, B, Hq, Hkv, Tq, Tkv, hd, scale);
}

// ---- per-head RMSNorm (optional) + rotary embedding, in place; one warp per (token, head) ----
// Rotation with pair-duplicated tables [pos][hd]: y[d] = x[d] c[d] - x[d+h] s[d],
// y[d+h] = x[d+h] c[d+h] + x[d] s[d+h] (reference src/kernels.c:249-264), unfused.
__global__ void __launch_bounds__(256) k_qk_post(float *q, int64_t ldq, int H, float *k, int64_t ldk, int Hkv, int hd,
                                                int64_t ntok, const float *__restrict__ qw, const float *__restrict__ kw,
                                                const float *__restrict__ cs, const float *__restrict__ sn,
                                                const int *__restrict__ pos, const int *__restrict__ step_d, int64_t pos_step) {
    if (step_d) pos += (int64_t)(*step_d) * pos_step;          // decode steps replayed from one graph
    int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    int HT = H + Hkv;
    if (w >= ntok * HT) return;
    int64_t tok = w / HT; int hh = (int)(w % HT);
    float *x; const float *nw;
    if (hh < H) { x = q + tok * ldq + hh * hd; nw = qw; }
    else { x = k + tok * ldk + (hh - H) * hd; nw = kw; }
    int half = hd / 2;
    float r = 1.f;
    if (nw) {
        float s = 0.f;
        for (int d = lane; d < hd; d += 32) { float v = x[d]; s += v * v; }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        r = 1.0f / sqrtf(s / (float)hd + 1e-6f);
    }
    const float *co = cs ? cs + (int64_t)pos[tok] * hd : nullptr;
    const float *si = sn ? sn + (int64_t)pos[tok] * hd : nullptr;
    for (int d = lane; d < half; d += 32) {
        float a = x[d], b = x[d + half];
        if (nw) { a = __fmul_rn(__fmul_rn(a, r), nw[d]); b = __fmul_rn(__fmul_rn(b, r), nw[d + half]); }
        if (co) {
            float ya = __fadd_rn(__fmul_rn(a, co[d]), __fmul_rn(-b, si[d]));
            float yb = __fadd_rn(__fmul_rn(b, co[d + half]), __fmul_rn(a, si[d + half]));
            a = ya; b = yb;
        }
        x[d] = a; x[d + half] = b;
    }
}

// Same operation, one warp per TOKEN (head dim <= 64): the lane owns the pair (d, d + hd/2) of every head, so the
// position and the four table values are fetched once per token instead of once per head, and the loads of
// eight heads are in flight together.
constexpr int QKP_HG = 8;
__global__ void __launch_bounds__(256) k_qk_post_tok(float *q, int64_t ldq, int H, float *k, int64_t ldk, int Hkv, int hd,
                                                    int64_t ntok, const float *__restrict__ qw, const float *__restrict__ kw,
                                                    const float *__restrict__ cs, const float *__restrict__ sn,
                                                    const int *__restrict__ pos, const int *__restrict__ step_d, int64_t pos_step) {
    pdl_launch_dependents();          // programmatic dependent launch: see launch_pdl()
    pdl_wait();
    if (step_d) pos += (int64_t)(*step_d) * pos_step;
    const int64_t tok = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31, half = hd / 2, HT = H + Hkv;
    if (tok >= ntok) return;
    const bool on = lane < half;
    float c0 = 1.f, c1 = 1.f, s0 = 0.f, s1 = 0.f;
    if (cs && on) {
        const int64_t p = (int64_t)pos[tok] * hd;
        c0 = cs[p + lane]; c1 = cs[p + lane + half]; s0 = sn[p + lane]; s1 = sn[p + lane + half];
    }
    for (int h0 = 0; h0 < HT; h0 += QKP_HG) {
        float a[QKP_HG], b[QKP_HG];
        float *xp[QKP_HG];
#pragma unroll
        for (int i = 0; i < QKP_HG; i++) {
            const int hh = h0 + i;
            xp[i] = hh < H ? q + tok * ldq + hh * hd : k + tok * ldk + (hh - H) * hd;
            a[i] = (hh < HT && on) ? xp[i][lane] : 0.f;
            b[i] = (hh < HT && on) ? xp[i][lane + half] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < QKP_HG; i++) {
            const int hh = h0 + i;
            if (hh >= HT) break;
            const float *nw = hh < H ? qw : kw;
            float x0 = a[i], x1 = b[i];
            if (nw) {
                float ss = x0 * x0 + x1 * x1;
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
                const float r = 1.0f / sqrtf(ss / (float)hd + 1e-6f);
                if (on) { x0 = __fmul_rn(__fmul_rn(x0, r), nw[lane]); x1 = __fmul_rn(__fmul_rn(x1, r), nw[lane + half]); }
            }
            if (cs) {
                const float y0 = __fadd_rn(__fmul_rn(x0, c0), __fmul_rn(-x1, s0));
                const float y1 = __fadd_rn(__fmul_rn(x1, c1), __fmul_rn(x0, s1));
                x0 = y0; x1 = y1;
            }
            if (on) { xp[i][lane] = x0; xp[i][lane + half] = x1; }
        }
    }
}

void qk_post(float *q, int64_t ldq, int H, float *k, int64_t ldk, int Hkv, int hd, int64_t ntok,
             const float *qnorm_w, const float *knorm_w, const float *cos_t, const float *sin_t, const int *pos_dev, const int *step_d, int64_t pos_step) {
    if (ntok <= 0 || (!qnorm_w && !cos_t)) return;
    ProfScope ps(NCMB_K_ELEM, 0, (double)ntok * (H + Hkv) * hd * 8);
    if (hd <= 64 && (hd & 1) == 0) {
        LAUNCH_PDL_IF(pdl_small(ntok / 8), k_qk_post_tok, grid1d(ntok * 32, 256), 256, 0, q, ldq, H, k, ldk, Hkv, hd, ntok,
               qnorm_w, knorm_w, cos_t, sin_t, pos_dev, step_d, pos_step);
        return;
    }
    LAUNCH(k_qk_post, grid1d(ntok * (H + Hkv) * 32, 256), 256, 0, q, ldq, H, k, ldk, Hkv, hd, ntok,
           qnorm_w, knorm_w, cos_t, sin_t, pos_dev, step_d, pos_step);
}

// table row = index within each group of T rows (reference rope_apply semantics)
__global__ void k_rope_rows(float *x, const float *__restrict__ cs, const float *__restrict__ sn, int64_t rows, int T, int hd) {
    int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (w >= rows) return;
    int t = (int)(w % T), half = hd / 2;
    float *xr = x + w * hd;
    const float *co = cs + (int64_t)t * hd, *si = sn + (int64_t)t * hd;
    for (int d = lane; d < half; d += 32) {
        float a = xr[d], b = xr[d + half];
        xr[d] = __fadd_rn(__fmul_rn(a, co[d]), __fmul_rn(-b, si[d]));
        xr[d + half] = __fadd_rn(__fmul_rn(b, co[d + half]), __fmul_rn(a, si[d + half]));
    }
}

} // namespace ncmb

using namespace ncmb;

extern "C" {

void sdpa_fwd(const float *q, const float *k, const float *v, const float *mask, float *out, int B, int H, int Tq, int Tkv, int hd) {
    ensure_device();
    sdpa_masked(q, k, v, mask, out, B, H, H, Tq, Tkv, hd);
}
void sdpa_fwd_gqa(const float *q, const float *k, const float *v, const float *mask, float *out, int B, int Hq, int Hkv, int Tq, int Tkv, int hd) {
    ensure_device();
    sdpa_masked(q, k, v, mask, out, B, Hq, Hkv, Tq, Tkv, hd);
}
void rope_apply_gqa(float *q, float *k, const float *cs, const float *sn, int B, int H, int K, int T, int hd) {
    ensure_device();
    if (q) { int64_t rows = (int64_t)B * H * T; LAUNCH(k_rope_rows, grid1d(rows * 32, 256), 256, 0, q, cs, sn, rows, T, hd); }
    if (k) { int64_t rows = (int64_t)B * K * T; LAUNCH(k_rope_rows, grid1d(rows * 32, 256), 256, 0, k, cs, sn, rows, T, hd); }
}
void rope_apply(float *q, float *k, const float *cs, const float *sn, int B, int H, int T, int hd) {
    rope_apply_gqa(q, k, cs, sn, B, H, H, T, hd);
}

} // extern "C"
