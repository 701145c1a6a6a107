// One pre-norm transformer block on a token-major activation matrix, shared by the
// NCP stack (reference ncp_block, src/ncp.c:184-344), the VQ-VAE blocks
// (vae_block, src/vqvae.c:44-225) and the GPT-2 / Qwen2 layers (src/gpt2.c:123-151,
// src/qwen.c:139-176). The reference shuffles heads through host memory around its
// SDPA; here the fused QKV projection is consumed in place by the attention kernel
// and the residual adds ride in the GEMM epilogues.
#include "common.cuh"

#include <stdarg.h>

namespace ncmb {

void apply_norm_split(const float *x, const float *w, const float *b, float *y, float *y_lo, int64_t rows, int C, int kind, float eps, int fmt) {
    if (kind == NORM_RMS) { if (y_lo) rmsnorm_split(x, w, y, y_lo, rows, C, fmt); else rmsnorm(x, w, y, rows, C, C, C); }
    else layernorm_split(x, w, b, y, y_lo, rows, C, eps, fmt);
}

void make_gated_interleaved(BlockWeights &w, int C, std::vector<void *> &owned) {
    if (!w.gated) return;
    const float *gate = w.fcw, *up = w.fcw + (size_t)w.Hh * C;
    float *il = dev_interleave_rows(gate, up, w.Hh, C);
    owned.push_back(il);
    w.fcw_il = il;
    if (w.fcb) {
        float *bil = dev_interleave_rows(w.fcb, w.fcb + w.Hh, w.Hh, 1);
        owned.push_back(bil);
        w.fcb_il = bil;
    }
}

void apply_norm(const float *x, const float *w, const float *b, float *y, int64_t rows, int C, int kind, float eps) {
    if (kind == NORM_RMS) rmsnorm(x, w, y, rows, C, C, C);
    else layernorm(x, w, b, y, rows, C, eps);
}

__global__ void k_kv_store(const float *__restrict__ src, int64_t ldsrc, float *__restrict__ dst, int64_t pitch,
                           int rows_per_seq, int64_t seq_pitch, int64_t ntok, int width4,
                           const int *__restrict__ step_d, int64_t step_stride) {
    pdl_launch_dependents();          // programmatic dependent launch: see launch_pdl()
    pdl_wait();
    if (step_d) dst += (int64_t)(*step_d) * step_stride;       // decode steps replayed from one graph
    int64_t total = ntok * width4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t tok = i / width4; int c = (int)(i % width4);
        int64_t s = rows_per_seq > 0 ? tok / rows_per_seq : 0;
        int64_t t = rows_per_seq > 0 ? tok % rows_per_seq : tok;
        float4 v = *(const float4 *)(src + tok * ldsrc + c * 4);
        *(float4 *)(dst + s * seq_pitch + t * pitch + c * 4) = v;
    }
}

__global__ void k_to_bf16_exact(const float *__restrict__ w, unsigned short *__restrict__ o, int64_t n, int *bad) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        unsigned u = __float_as_uint(w[i]);
        if (u & 0xffffu) *bad = 1;                     // low mantissa bits set: not a bf16 value
        o[i] = (unsigned short)(u >> 16);
    }
}
unsigned short *dev_bf16_exact(const float *w, int64_t n) {
    if (!w || n <= 0) return nullptr;
    unsigned short *o = (unsigned short *)dev_alloc((size_t)n * 2);
    int *bad = (int *)dev_alloc(4);
    CUDA_CHECK(cudaMemsetAsync(bad, 0, 4, stream()));
    int64_t g = cdiv(n, 256), cap = (int64_t)ctx().sm_count * 16;
    LAUNCH(k_to_bf16_exact, (unsigned)(g > cap ? cap : g), 256, 0, w, o, n, bad);
    int h = 0;
    CUDA_CHECK(cudaMemcpyAsync(&h, bad, 4, cudaMemcpyDeviceToHost, stream()));
    CUDA_CHECK(cudaStreamSynchronize(stream()));
    dev_free(bad);
    if (h) { dev_free(o); return nullptr; }
    return o;
}

// Scratch for the lo halves of the block's GEMM inputs in three-pass mode (ln, ctx, hidden).
static Workspace &block_lo_ws() { static Workspace w; return w; }

void run_block(float *x, int64_t ntok, int C, int H, int nkv, const BlockWeights &w, const BlockBufs &b, const AttnPlan &p) {
    if (ntok <= 0) return;
    const int hd = C / H, kvd = nkv * hd, Wq = C + 2 * kvd;
    // In three-pass mode the producers of GEMM inputs (norms, attention, MLP activation) write
    // TF32 hi / lo pairs directly, so no separate split pass runs between kernels.
    GemmArgs probe;
    probe.x = b.ln; probe.ldx = C; probe.W = w.qkvw; probe.y = b.qkv; probe.ldy = Wq; probe.M = ntok; probe.N = Wq; probe.K = C;
    static const bool fuse_split = !getenv("NCM_B200_NO_SPLIT_FUSE");
    bool split = fuse_split && ctx().gemm_mode >= 2 && gemm_tc_supported(probe) && (C % 4 == 0) && (w.Hh % 4 == 0) && C >= 32 && w.Hh >= 32;
    // mode 3: fp16 pairs for the fp16-pair kernel (rows of C and Hh halfs must keep 16-byte strides)
    int fmt = split ? SPLIT_TF32 : SPLIT_NONE;
    if (split && ctx().gemm_mode >= 3 && gemm_h3_supported(probe) && (C % 8 == 0) && (w.Hh % 8 == 0)) fmt = SPLIT_H16;
    auto tc_ok = [&](const GemmArgs &q) { return fmt == SPLIT_H16 ? gemm_h3_supported(q) : (ctx().gemm_mode >= 1 && gemm_tc_supported(q)); };
    float *ln_lo = nullptr, *ctx_lo = nullptr, *h_lo = nullptr;
    if (split) {
        Workspace &lw = block_lo_ws();
        size_t need = (size_t)ntok * (2 * (size_t)C + w.Hh) * 4 + 4096;
        if (need > lw.cap) lw.reserve(need + need / 4);
        lw.reset();
        ln_lo = lw.get<float>((size_t)ntok * C); ctx_lo = lw.get<float>((size_t)ntok * C); h_lo = lw.get<float>((size_t)ntok * w.Hh);
    }
    // Few rows (decode steps): the projections run on the GEMV kernel, which normalises its input rows on the
    // fly and can write the K|V columns straight into the cache -- three launches fewer per block.
    GemmArgs g;
    g.x = x; g.ldx = C; g.W = w.qkvw; g.bias = w.qkvb; g.y = b.qkv; g.ldy = Wq; g.M = ntok; g.N = Wq; g.K = C;
    g.ln_kind = w.norm == NORM_RMS ? 2 : 1; g.ln_w = w.ln1w; g.ln_b = w.ln1b; g.ln_eps = w.norm == NORM_RMS ? 1e-6f : w.eps;
    static const bool fuse_small = !getenv("NCM_B200_NO_GEMV_FUSE");
    const bool small = fuse_small && !split && gemv_fusable(g);
    bool kv_written = false, qk_done = false;
    g.W16 = w.qkvw16;
    // decode steps: every weight-streaming kernel asks L2 for the matrix the next one reads (2- or 4-byte form)
    auto next_is = [&](GemmArgs &q, const float *W, const unsigned short *W16, int64_t n) {
        q.pf_next = small ? (W16 ? (const void *)W16 : (const void *)W) : nullptr;
        q.pf_next_bytes = (size_t)n * (W16 ? 2 : 4);
    };
    if (small) {
        next_is(g, w.ow, w.ow16, (int64_t)C * C);
        // up to four rows: the warp-per-row-pair GEMV also rotates the query / key heads in its epilogue, so the
        // rotation pass and the cache copy of a decode step disappear (per-head norms keep their own pass)
        if (p.cos_t && !w.qnw && !w.knw && (hd & 1) == 0 && gemv_warp_takes(g)) {
            g.gv_rope_cos = p.cos_t; g.gv_rope_sin = p.sin_t; g.gv_rope_pos = p.pos; g.gv_rope_step_d = p.step_d;
            g.gv_rope_pos_step = p.pos_step; g.gv_rope_cols = C + kvd; g.gv_hd = hd;
            qk_done = true;
        }
        if (p.kv_store && !w.qnw && !w.knw && (!p.cos_t || qk_done) && p.kv_rows_per_seq == 1) {
            g.y2 = p.kv_store; g.y2_col0 = C; g.ldy2 = p.kv_seq_pitch; g.y2_step_d = p.step_d; g.y2_step = p.kv_store_step;
            kv_written = true;
        }
    } else {
        apply_norm_split(x, w.ln1w, w.ln1b, b.ln, ln_lo, ntok, C, w.norm, w.eps, fmt);
        g.ln_kind = 0;
        g.x_fmt = fmt;
        g.x = b.ln; g.x_lo = ln_lo;
    }
    // head dim 64: the GEMM's epilogue can apply the per-head norm and the rotation itself (it says whether it did)
    if (hd == 64 && !small && !p.step_d && (w.qnw || w.knw || p.cos_t)) {
        g.qk_heads = H + nkv; g.qk_H = H; g.qk_qw = w.qnw; g.qk_kw = w.knw; g.qk_cos = p.cos_t; g.qk_sin = p.sin_t; g.qk_pos = p.pos;
        g.qk_applied = &qk_done;
    }
    gemm(g);
    float *qp = b.qkv, *kp = b.qkv + C, *vp = b.qkv + C + kvd;
    if (!qk_done) qk_post(qp, Wq, H, kp, Wq, nkv, hd, ntok, w.qnw, w.knw, p.cos_t, p.sin_t, p.pos, p.step_d, p.pos_step);
    if (p.kv_store && !kv_written) {
        int width4 = 2 * kvd / 4;
        int64_t n = ntok * width4;
        int64_t gsz = cdiv(n, 256), cap = (int64_t)ctx().sm_count * 16;
        ProfScope ps(NCMB_K_ELEM, 0, (double)ntok * 2 * kvd * 8);
        LAUNCH_PDL_IF(pdl_small(gsz), k_kv_store, (unsigned)(gsz > cap ? cap : gsz), 256, 0, kp, (int64_t)Wq, p.kv_store, p.kv_pitch,
               p.kv_rows_per_seq, p.kv_seq_pitch, ntok, width4, p.step_d, p.kv_store_step);
    }
    if (p.kv_only) return;
    AttnArgs a;
    a.q = qp; a.ldq = Wq;
    if (p.k1) { a.k1 = p.k1; a.v1 = p.v1; a.ldk1 = p.ldk1; }
    else { a.k1 = kp; a.v1 = vp; a.ldk1 = Wq; }
    a.k1_start = p.k1_start; a.k1_len = p.k1_len;
    if (p.self_is_k2) { a.k2 = kp; a.v2 = vp; a.ldk2 = Wq; a.k2_start = p.k2_start ? p.k2_start : p.q_start; }
    else if (p.k2) { a.k2 = p.k2; a.v2 = p.v2; a.ldk2 = p.ldk2; a.k2_start = p.k2_start; }
    a.out = b.ctx; a.out_lo = ctx_lo; a.out_fmt = fmt; a.ldo = C;
    a.q_start = p.q_start;
    a.rows = p.rows; a.H = H; a.Hkv = nkv; a.hd = hd; a.max_q = p.max_q;
    a.causal = p.causal; a.causal_off = p.causal_off; a.window = p.window;
    a.total_q = p.total_q; a.avg_keys = p.avg_keys;
    a.max_k1 = p.max_k1; a.max_k2 = p.self_is_k2 ? p.max_q : (p.k2 ? p.max_k2 : 0);
    a.step_d = p.step_d; a.k1_len_step = p.k1_len_step;
    a.q_total = ntok; a.k1_total = p.k1 ? p.k1_total : ntok; a.k2_total = p.self_is_k2 ? ntok : (p.k2 ? p.k2_total : 0);
    attention(a);
    // x += ctx Wo^T + bo
    g = GemmArgs();
    g.x_fmt = fmt;
    g.x = b.ctx; g.x_lo = ctx_lo; g.ldx = C; g.W = w.ow; g.W16 = w.ow16; g.bias = w.ob; g.res = x; g.ldres = C; g.y = x; g.ldy = C; g.M = ntok; g.N = C; g.K = C;
    next_is(g, w.fcw, w.fcw16, (int64_t)(w.gated ? 2 : 1) * w.Hh * C);
    gemm(g);
    g = GemmArgs();
    g.ldx = C; g.M = ntok; g.K = C;
    if (small) {
        g.x = x;
        g.ln_kind = w.norm == NORM_RMS ? 2 : 1; g.ln_w = w.ln2w; g.ln_b = w.ln2b; g.ln_eps = w.norm == NORM_RMS ? 1e-6f : w.eps;
    } else {
        apply_norm_split(x, w.ln2w, w.ln2b, b.ln, ln_lo, ntok, C, w.norm, w.eps, fmt);
        g.x_fmt = fmt; g.y_fmt = fmt;
        g.x = b.ln; g.x_lo = ln_lo;
    }
    next_is(g, w.pw, w.pw16, (int64_t)C * w.Hh);                       // the up-projection is followed by the down-projection
    if (w.gated && small && w.fcw && gemv_warp_takes(g)) {
        // up to four rows: gate and up rows are paired inside the GEMV, the gated product leaves from its epilogue
        g.W = w.fcw; g.W16 = w.fcw16; g.bias = w.fcb; g.N = 2 * w.Hh; g.gv_pair_half = w.Hh; g.act = w.act; g.y = b.h; g.ldy = w.Hh;
        gemm(g);
        h_lo = nullptr;
    } else if (w.gated) {
        GemmArgs t = g;
        t.W = w.fcw_il; t.bias = w.fcb_il; t.N = 2 * w.Hh; t.glu = 1; t.act = w.act; t.y = b.h; t.ldy = w.Hh;
        static const bool fuse_glu = !getenv("NCM_B200_NO_GLU_FUSE");
        if (fuse_glu && w.fcw_il && tc_ok(t)) {
            t.y_lo = h_lo;                       // gated product fused into the epilogue (interleaved gate/up rows)
            gemm(t);
        } else {
            g.x_lo = ln_lo;
            g.W = w.fcw; g.W16 = w.fcw16; g.bias = w.fcb; g.y = b.mlp; g.N = 2 * w.Hh; g.ldy = 2 * w.Hh;
            gemm(g);
            glu_combine(b.mlp, b.h, ntok, w.Hh, w.act);
            h_lo = nullptr;
        }
    } else {
        g.W = w.fcw; g.W16 = w.fcw16; g.bias = w.fcb; g.y = b.h; g.y_lo = h_lo; g.N = w.Hh; g.ldy = w.Hh; g.act = w.act;
        if (!tc_ok(g)) { g.y_lo = nullptr; h_lo = nullptr; }
        gemm(g);
    }
    g = GemmArgs();
    g.x_fmt = fmt;
    g.x = b.h; g.x_lo = h_lo; g.ldx = w.Hh; g.W = w.pw; g.W16 = w.pw16; g.bias = w.pb; g.res = x; g.ldres = C; g.y = x; g.ldy = C; g.M = ntok; g.N = C; g.K = w.Hh;
    if (small) { g.pf_next = w.next_w; g.pf_next_bytes = w.next_w_bytes; }
    gemm(g);
}

// ---- small host helpers ----
Tensor *wget(WeightStore *ws, const char *fmt, ...) {
    char key[320];
    va_list ap; va_start(ap, fmt); vsnprintf(key, sizeof key, fmt, ap); va_end(ap);
    return weights_get(ws, key);
}
Tensor *wneed(WeightStore *ws, const char *fmt, ...) {
    char key[320];
    va_list ap; va_start(ap, fmt); vsnprintf(key, sizeof key, fmt, ap); va_end(ap);
    Tensor *t = weights_get(ws, key);
    if (!t) { fprintf(stderr, "missing weight %s\n", key); exit(1); }
    return t;
}
void *dev_alloc(size_t bytes) {
    ensure_device();
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes ? bytes : 256);
    if (e != cudaSuccess) fatal("device allocation of %.1f MB failed: %s", bytes / 1048576.0, cudaGetErrorString(e));
    return p;
}
void dev_free(void *p) { if (p) { cudaStreamSynchronize(stream()); cudaFree(p); } }
void upload(void *dev, const void *host, size_t bytes) {
    if (!bytes) return;
    CUDA_CHECK(cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, stream()));
    CUDA_CHECK(cudaStreamSynchronize(stream()));
    ctx().h2d_bytes += bytes;
}
float *dev_concat_rows(const float *a, int64_t na, const float *b, int64_t nb) {
    float *d = (float *)dev_alloc((size_t)(na + nb) * sizeof(float));
    if (a) CUDA_CHECK(cudaMemcpyAsync(d, a, (size_t)na * 4, cudaMemcpyDeviceToDevice, stream()));
    else CUDA_CHECK(cudaMemsetAsync(d, 0, (size_t)na * 4, stream()));
    if (b) CUDA_CHECK(cudaMemcpyAsync(d + na, b, (size_t)nb * 4, cudaMemcpyDeviceToDevice, stream()));
    else CUDA_CHECK(cudaMemsetAsync(d + na, 0, (size_t)nb * 4, stream()));
    return d;
}

} // namespace ncmb
