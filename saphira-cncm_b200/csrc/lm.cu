// GPT-2 and Qwen2 decoders with a KV cache, batched over independent prompts
// (reference src/gpt2.c, src/qwen.c). The reference recomputes the whole context for
// every new token at batch 1 (gpt2.c:187-198, qwen.c:217-227); causal attention makes
// a cached, batched run produce the same logits, so each row here equals one
// reference run. Layers reuse the transformer block of the NCP stack.
#include "common.cuh"
#include "lm_mega.cuh"
#include "tc_common.cuh"

#include <algorithm>
#include <string>
#include <vector>

using namespace ncmb;

typedef struct TokState TokState;
extern "C" {
// host tokenizer of the reference (src/ncm.h:294-303); optional at link time
TokState *tok_load(const NCMConfig *c, const char *asset_dir) __attribute__((weak));
void tok_free(TokState *t) __attribute__((weak));
int tok_encode(TokState *t, const char *text, int *out, int cap) __attribute__((weak));
int tok_decode(TokState *t, const int *ids, int n, char *out, int cap, int skip_special) __attribute__((weak));
}

extern "C" int ncmb_weights_import_safetensors(WeightStore *ws, const char *path, int conv1d_transpose);

struct NcmbLM {
    NCMConfig cfg;
    WeightStore ws{};
    int is_qwen = 0;
    int NL = 0, H = 0, nkv = 0, C = 0, hd = 0, I = 0, n_ctx = 0, V = 0, eos = -1;
    const float *wte = nullptr, *wpe = nullptr, *lnfw = nullptr, *lnfb = nullptr;
    const unsigned short *wte16 = nullptr;      // exact bf16 copy of the embedding / head matrix (bf16 weight files)
    float *cosb = nullptr, *sinb = nullptr;
    std::vector<BlockWeights> blocks;
    std::vector<void *> owned;
    Workspace work;
};

static const float *need(WeightStore *ws, const char *who, const char *fmt, int li, const char *leaf) {
    char key[192];
    snprintf(key, sizeof key, fmt, li, leaf);
    Tensor *t = weights_get(ws, key);
    if (!t) { fprintf(stderr, "%s: missing tensor %s\n", who, key); exit(1); }
    return t->data;
}
static const float *maybe(WeightStore *ws, const char *fmt, int li, const char *leaf) {
    char key[192];
    snprintf(key, sizeof key, fmt, li, leaf);
    Tensor *t = weights_get(ws, key);
    return t ? t->data : nullptr;
}

extern "C" NcmbLM *ncmb_lm_open(const NCMConfig *c, const char *weights, int is_qwen, int bf16_weights) {
    ensure_device();
    NcmbLM *m = new NcmbLM();
    m->cfg = *c; m->is_qwen = is_qwen;
    {   // a Hugging Face checkpoint is read directly (the reference converts it to NCM1 offline first)
        const size_t wl = strlen(weights);
        const bool st = wl > 12 && strcmp(weights + wl - 12, ".safetensors") == 0;
        const int rc = st ? ncmb_weights_import_safetensors(&m->ws, weights, is_qwen ? 0 : 1) : weights_load(&m->ws, weights);
        if (rc) { delete m; return nullptr; }
    }
    WeightStore *ws = &m->ws;
    m->NL = c->n_layer; m->H = c->n_head; m->C = c->n_embd; m->hd = m->C / m->H;
    m->nkv = (is_qwen && c->n_kv_heads > 0) ? c->n_kv_heads : c->n_head;
    m->eos = c->eos_token_id;
    if (m->hd != 8 && m->hd != 16 && m->hd != 32 && m->hd != 64 && m->hd != 128) fatal("head dim %d not supported", m->hd);
    int C = m->C, kvd = m->nkv * m->hd;
    if (!is_qwen) {
        m->n_ctx = c->context_length > 0 ? c->context_length : 1024;
        Tensor *wte = weights_get(ws, "wte.weight");
        if (!wte) { fprintf(stderr, "gpt2: missing tensor wte.weight\n"); exit(1); }
        m->V = (int)wte->shape[0]; m->wte = wte->data;
        m->wpe = need(ws, "gpt2", "%.0dwpe.%s", 0, "weight");
        m->lnfw = need(ws, "gpt2", "%.0dln_f.%s", 0, "weight");
        m->lnfb = need(ws, "gpt2", "%.0dln_f.%s", 0, "bias");
        m->I = 4 * C;
        for (int li = 0; li < m->NL; li++) {
            BlockWeights w;
            w.norm = NORM_LAYER; w.eps = 1e-5f;
            w.ln1w = need(ws, "gpt2", "h.%d.ln_1.%s", li, "weight"); w.ln1b = need(ws, "gpt2", "h.%d.ln_1.%s", li, "bias");
            w.qkvw = need(ws, "gpt2", "h.%d.attn.c_attn.%s", li, "weight"); w.qkvb = maybe(ws, "h.%d.attn.c_attn.%s", li, "bias");
            w.ow = need(ws, "gpt2", "h.%d.attn.c_proj.%s", li, "weight"); w.ob = maybe(ws, "h.%d.attn.c_proj.%s", li, "bias");
            w.ln2w = need(ws, "gpt2", "h.%d.ln_2.%s", li, "weight"); w.ln2b = need(ws, "gpt2", "h.%d.ln_2.%s", li, "bias");
            w.fcw = need(ws, "gpt2", "h.%d.mlp.c_fc.%s", li, "weight"); w.fcb = maybe(ws, "h.%d.mlp.c_fc.%s", li, "bias");
            w.pw = need(ws, "gpt2", "h.%d.mlp.c_proj.%s", li, "weight"); w.pb = maybe(ws, "h.%d.mlp.c_proj.%s", li, "bias");
            w.Hh = m->I; w.gated = 0; w.act = ACT_GELU_TANH;
            m->blocks.push_back(w);
        }
    } else {
        m->n_ctx = c->context_length > 0 ? c->context_length : 4096;
        double theta = c->rope_theta > 0 ? c->rope_theta : 1000000.0;
        Tensor *te = weights_get(ws, "model.embed_tokens.weight");
        if (!te) { fprintf(stderr, "qwen: missing tensor model.embed_tokens.weight\n"); exit(1); }
        m->V = (int)te->shape[0]; m->wte = te->data;
        m->lnfw = need(ws, "qwen", "%.0dmodel.norm.%s", 0, "weight");
        Tensor *tg = weights_get(ws, "model.layers.0.mlp.gate_proj.weight");
        if (!tg) { fprintf(stderr, "qwen: missing tensor model.layers.0.mlp.gate_proj.weight\n"); exit(1); }
        m->I = (int)tg->shape[0];
        for (int li = 0; li < m->NL; li++) {
            BlockWeights w;
            w.norm = NORM_RMS; w.eps = 1e-6f;
            w.ln1w = need(ws, "qwen", "model.layers.%d.input_layernorm.%s", li, "weight");
            const float *qw = need(ws, "qwen", "model.layers.%d.self_attn.q_proj.%s", li, "weight");
            const float *qb = need(ws, "qwen", "model.layers.%d.self_attn.q_proj.%s", li, "bias");
            const float *kw = need(ws, "qwen", "model.layers.%d.self_attn.k_proj.%s", li, "weight");
            const float *kb = need(ws, "qwen", "model.layers.%d.self_attn.k_proj.%s", li, "bias");
            const float *vw = need(ws, "qwen", "model.layers.%d.self_attn.v_proj.%s", li, "weight");
            const float *vb = need(ws, "qwen", "model.layers.%d.self_attn.v_proj.%s", li, "bias");
            // fused [C + 2*kvd][C] projection: q rows, then k rows, then v rows
            float *kvw = dev_concat_rows(kw, (int64_t)kvd * C, vw, (int64_t)kvd * C);
            float *qkvw = dev_concat_rows(qw, (int64_t)C * C, kvw, (int64_t)2 * kvd * C);
            float *kvb = dev_concat_rows(kb, kvd, vb, kvd);
            float *qkvb = dev_concat_rows(qb, C, kvb, 2 * kvd);
            CUDA_CHECK(cudaStreamSynchronize(stream()));
            dev_free(kvw); dev_free(kvb);
            m->owned.push_back(qkvw); m->owned.push_back(qkvb);
            w.qkvw = qkvw; w.qkvb = qkvb;
            w.ow = need(ws, "qwen", "model.layers.%d.self_attn.o_proj.%s", li, "weight");
            w.ln2w = need(ws, "qwen", "model.layers.%d.post_attention_layernorm.%s", li, "weight");
            const float *gw = need(ws, "qwen", "model.layers.%d.mlp.gate_proj.%s", li, "weight");
            const float *uw = need(ws, "qwen", "model.layers.%d.mlp.up_proj.%s", li, "weight");
            float *gu = dev_concat_rows(gw, (int64_t)m->I * C, uw, (int64_t)m->I * C);
            m->owned.push_back(gu);
            w.fcw = gu;
            w.pw = need(ws, "qwen", "model.layers.%d.mlp.down_proj.%s", li, "weight");
            w.Hh = m->I; w.gated = 1; w.act = ACT_SILU;
            make_gated_interleaved(w, C, m->owned);
            m->blocks.push_back(w);
        }
        // rotary tables [n_ctx][hd], angle t * theta^(-2d/hd), pair-duplicated (qwen.c:85-110)
        int hd = m->hd, h = hd / 2, T = m->n_ctx;
        std::vector<float> hc((size_t)T * hd), hs((size_t)T * hd);
        for (int t = 0; t < T; t++) for (int d = 0; d < h; d++) {
            double a = (double)t * pow(theta, -(double)(2 * d) / (double)hd);
            float co = (float)cos(a), si = (float)sin(a);
            hc[(size_t)t * hd + d] = co; hc[(size_t)t * hd + d + h] = co;
            hs[(size_t)t * hd + d] = si; hs[(size_t)t * hd + d + h] = si;
        }
        m->cosb = (float *)dev_alloc(hc.size() * 4); m->sinb = (float *)dev_alloc(hs.size() * 4);
        upload(m->cosb, hc.data(), hc.size() * 4); upload(m->sinb, hs.data(), hs.size() * 4);
        m->owned.push_back(m->cosb); m->owned.push_back(m->sinb);
    }
    // bf16 weight files (values already rounded to bf16, stored as fp32): decode steps are bound by streaming the
    // weights, so the matrices get an exact 2-byte copy that the GEMV kernel reads instead -- same values, half
    // the bytes. A matrix with any element that is not a bf16 value keeps its fp32 path.
    if (bf16_weights || ncmb_weights_are_bf16(&m->ws)) {
        const int kvd2 = m->nkv * m->hd;
        auto shadow = [&](const float *w, int64_t n) -> const unsigned short * {
            unsigned short *p = dev_bf16_exact(w, n);
            if (p) m->owned.push_back(p);
            return p;
        };
        for (auto &bw : m->blocks) {
            bw.qkvw16 = shadow(bw.qkvw, (int64_t)(m->C + 2 * kvd2) * m->C);
            bw.ow16 = shadow(bw.ow, (int64_t)m->C * m->C);
            bw.fcw16 = shadow(bw.fcw, (int64_t)(bw.gated ? 2 : 1) * bw.Hh * m->C);
            bw.pw16 = shadow(bw.pw, (int64_t)m->C * bw.Hh);
        }
        m->wte16 = shadow(m->wte, (int64_t)m->V * m->C);
    }
    // what a decode step's weight-streaming kernels read after each block's last one: the next block's QKV matrix,
    // after the last block the first 32 MB of the vocabulary projection (the whole of it would evict what L2 holds)
    for (size_t li = 0; li < m->blocks.size(); li++) {
        BlockWeights &bw = m->blocks[li];
        if (li + 1 < m->blocks.size()) {
            const BlockWeights &nx = m->blocks[li + 1];
            const int64_t n = (int64_t)(m->C + 2 * m->nkv * m->hd) * m->C;
            bw.next_w = nx.qkvw16 ? (const void *)nx.qkvw16 : (const void *)nx.qkvw;
            bw.next_w_bytes = (size_t)n * (nx.qkvw16 ? 2 : 4);
        } else {
            const size_t bytes = (size_t)m->V * m->C * (m->wte16 ? 2 : 4);
            bw.next_w = m->wte16 ? (const void *)m->wte16 : (const void *)m->wte;
            bw.next_w_bytes = bytes < ((size_t)32 << 20) ? bytes : ((size_t)32 << 20);
        }
    }
    CUDA_CHECK(cudaStreamSynchronize(stream()));
    return m;
}

extern "C" void ncmb_lm_close(NcmbLM *m) {
    if (!m) return;
    for (void *p : m->owned) dev_free(p);
    m->work.release();
    weights_free(&m->ws);
    delete m;
}
extern "C" int ncmb_lm_vocab(const NcmbLM *m) { return m->V; }
extern "C" void ncmb_set_lm_persistent(int on) { lm_mega_enable(on); }

namespace {

struct LMRun {
    NcmbLM *m;
    int B, np, cap;
    std::vector<float *> kv;      // per layer [B][cap][2*kvd]
    BlockBufs bufs{};
    float *x = nullptr, *last = nullptr, *logits = nullptr, *samp_scr = nullptr;
    int *ids_d = nullptr, *pos_d = nullptr, *start_np = nullptr, *start_1 = nullptr, *kstart = nullptr;
    int *posmat = nullptr, *lenmat = nullptr, *out_d = nullptr, *last_rows = nullptr;
    double *uni_d = nullptr;
    // decode loop state on the device: absolute position of the step, this step's picks / packed argmax / uniforms
    int *step_d = nullptr, *pick_d = nullptr;
    long long graph_launches = 0;
    // persistent decode kernel (up to four rows, head dim 64)
    float *mg_part = nullptr; unsigned *mg_count = nullptr, *mg_bar = nullptr; MegaLayer *mg_layers = nullptr;                      // kernel launches one replay of the captured step stands for
    unsigned long long *amax_d = nullptr;
    double *uni_cur = nullptr;
    // likelihood runs: next-token target and result per token row
    int64_t nll_rows = 0; int *tgt_d = nullptr; double *nll_d = nullptr;
};

void lm_layout(LMRun &r, Workspace &w, int n_new, int64_t logit_rows) {
    NcmbLM *m = r.m;
    int C = m->C, kvd = m->nkv * m->hd, Wq = C + 2 * kvd;
    int64_t nmax = (int64_t)r.B * r.np;
    r.kv.clear();
    for (int li = 0; li < m->NL; li++) r.kv.push_back(w.get<float>((size_t)r.B * r.cap * 2 * kvd));
    r.x = w.get<float>((size_t)nmax * C);
    r.bufs.ln = w.get<float>((size_t)nmax * C);
    r.bufs.qkv = w.get<float>((size_t)nmax * Wq);
    r.bufs.ctx = w.get<float>((size_t)nmax * C);
    r.bufs.mlp = m->is_qwen ? w.get<float>((size_t)nmax * 2 * m->I) : nullptr;
    r.bufs.h = w.get<float>((size_t)nmax * m->I);
    r.last = w.get<float>((size_t)r.B * C);
    r.logits = w.get<float>((size_t)(logit_rows > r.B ? logit_rows : r.B) * m->V);
    size_t ss = sample_scratch_floats(r.B, m->V);
    r.samp_scr = ss ? w.get<float>(ss) : nullptr;
    r.ids_d = w.get<int>((size_t)nmax);
    r.pos_d = w.get<int>((size_t)nmax);
    r.start_np = w.get<int>(r.B + 1);
    r.start_1 = w.get<int>(r.B + 1);
    r.kstart = w.get<int>(r.B + 1);
    r.posmat = w.get<int>((size_t)r.cap * r.B);
    r.lenmat = w.get<int>((size_t)r.cap * r.B);
    r.out_d = w.get<int>((size_t)r.B * (n_new > 0 ? n_new : 1));
    r.last_rows = w.get<int>(r.B);
    r.uni_d = w.get<double>((size_t)(n_new > 0 ? n_new : 1) * r.B);
    r.uni_cur = w.get<double>(r.B);
    r.amax_d = w.get<unsigned long long>(r.B);
    r.pick_d = w.get<int>(r.B);
    r.step_d = w.get<int>(4);
    const int max_split = (r.cap + 31) / 32;
    r.mg_part = w.get<float>((size_t)r.B * m->H * max_split * 66);
    r.mg_count = w.get<unsigned>((size_t)r.B * m->nkv + 4);
    r.mg_bar = w.get<unsigned>(4);
    r.mg_layers = (MegaLayer *)w.get<unsigned char>(sizeof(MegaLayer) * (size_t)m->NL);
    if (r.nll_rows > 0) { r.tgt_d = w.get<int>((size_t)r.nll_rows); r.nll_d = w.get<double>((size_t)r.nll_rows); }
}

void lm_embed(LMRun &r, const int *ids_d, const int *pos_d, int64_t n) {
    NcmbLM *m = r.m;
    embed_rows(m->wte, ids_d, r.x, n, m->C);
    if (!m->is_qwen) {
        embed_rows(m->wpe, pos_d, r.bufs.ctx, n, m->C);
        add_inplace(r.x, r.bufs.ctx, n * m->C);
    }
}

void lm_head(LMRun &r, const float *h, int64_t rows, float *logits) {
    NcmbLM *m = r.m;
    GemmArgs g;
    g.x = h; g.ldx = m->C; g.W = m->wte; g.W16 = m->wte16; g.y = logits; g.ldy = m->V; g.M = rows; g.N = m->V; g.K = m->C;
    g.ln_kind = m->is_qwen ? 2 : 1; g.ln_w = m->lnfw; g.ln_b = m->lnfb; g.ln_eps = m->is_qwen ? 1e-6f : 1e-5f;
    if (!gemv_fusable(g)) {        // many rows: stand-alone norm, tensor-core GEMM
        apply_norm(h, m->lnfw, m->lnfb, r.bufs.ln, rows, m->C, m->is_qwen ? NORM_RMS : NORM_LAYER, m->is_qwen ? 1e-6f : 1e-5f);
        g.x = r.bufs.ln; g.ln_kind = 0;
    }
    gemm(g);
}

// prompt tokens of all rows through every layer, K/V into the cache
void lm_prefill(LMRun &r) {
    NcmbLM *m = r.m;
    int kvd = m->nkv * m->hd;
    int64_t n = (int64_t)r.B * r.np;
    lm_embed(r, r.ids_d, r.pos_d, n);
    AttnPlan p;
    p.q_start = p.k1_start = r.start_np;
    p.rows = r.B; p.max_q = r.np; p.max_k1 = r.np; p.causal = 1;
    p.pos = r.pos_d;
    if (m->is_qwen) { p.cos_t = m->cosb; p.sin_t = m->sinb; }
    p.total_q = n; p.avg_keys = (r.np + 1) / 2.0;
    p.kv_pitch = 2 * kvd; p.kv_rows_per_seq = r.np; p.kv_seq_pitch = (int64_t)r.cap * 2 * kvd;
    for (int li = 0; li < m->NL; li++) {
        p.kv_store = r.kv[li];
        run_block(r.x, n, m->C, m->H, m->nkv, m->blocks[li], r.bufs, p);
    }
}

// token + position embedding of the decode step whose absolute position sits in *step_d
__global__ void k_lm_embed_dec(const float *__restrict__ wte, const float *__restrict__ wpe, const int *__restrict__ ids,
                               const int *__restrict__ posmat, const int *__restrict__ step_d, int pos_base, int B, int C,
                               float *__restrict__ x) {
    pdl_launch_dependents();
    pdl_wait();
    const int *pos = posmat + (int64_t)(*step_d + pos_base) * B;
    int64_t n = (int64_t)B * C;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int b = (int)(i / C), c = (int)(i % C);
        float v = wte[(int64_t)ids[b] * C + c];
        if (wpe) v = __fadd_rn(v, wpe[(int64_t)pos[b] * C + c]);
        x[i] = v;
    }
}

// One new token per row. *r.step_d = v counts the tokens finalised so far (k_lm_finish_step advances it); this
// step's token sits at absolute position np + v - 1, and every per-step array is indexed through the
// counter (bases shifted by np - 1 steps), so the same launches -- eagerly or replayed from one captured
// CUDA graph -- serve every step.
void lm_decode_step(LMRun &r, const int *ids_d) {
    NcmbLM *m = r.m;
    int kvd = m->nkv * m->hd;
    {
        int64_t n = (int64_t)r.B * m->C, g = cdiv(n, 256), cap = (int64_t)ctx().sm_count * 8;
        ProfScope ps(NCMB_K_ELEM, 0, (double)n * 8);
        LAUNCH_PDL(k_lm_embed_dec, (unsigned)(g > cap ? cap : g), 256, 0, m->wte, m->is_qwen ? (const float *)nullptr : m->wpe, ids_d,
               r.posmat, r.step_d, r.np - 1, r.B, m->C, r.x);
    }
    AttnPlan p;
    p.step_d = r.step_d;
    p.q_start = r.start_1; p.k1_start = r.kstart;
    const int64_t sh = r.np - 1;                               // counter value v <-> absolute position np - 1 + v
    p.k1_len = r.lenmat + sh * r.B; p.k1_len_step = r.B;
    p.ldk1 = 2 * kvd;
    p.rows = r.B; p.max_q = 1; p.max_k1 = r.cap; p.k1_total = (int64_t)r.B * r.cap;
    p.pos = r.posmat + sh * r.B; p.pos_step = r.B;
    if (m->is_qwen) { p.cos_t = m->cosb; p.sin_t = m->sinb; }
    p.total_q = r.B; p.avg_keys = (r.np + r.cap) / 2.0;
    p.kv_pitch = 2 * kvd; p.kv_rows_per_seq = 1; p.kv_seq_pitch = (int64_t)r.cap * 2 * kvd;
    p.kv_store_step = 2 * kvd;
    for (int li = 0; li < m->NL; li++) {
        p.k1 = r.kv[li]; p.v1 = r.kv[li] + kvd;
        p.kv_store = r.kv[li] + sh * 2 * kvd;
        run_block(r.x, r.B, m->C, m->H, m->nkv, m->blocks[li], r.bufs, p);
    }
}

void lm_setup(LMRun &r, const int *prompts, int n_new, int64_t logit_rows) {
    NcmbLM *m = r.m;
    int B = r.B, np = r.np, cap = r.cap;
    Workspace sizing;
    sizing.measuring = true;
    lm_layout(r, sizing, n_new, logit_rows);
    m->work.reserve(sizing.off + 4096);
    m->work.reset();
    lm_layout(r, m->work, n_new, logit_rows);
    std::vector<int> pos((size_t)B * np), st(B + 1), s1(B + 1), ks(B + 1), pm((size_t)cap * B), lm((size_t)cap * B), lr(B);
    for (int b = 0; b < B; b++) for (int t = 0; t < np; t++) pos[(size_t)b * np + t] = t;
    for (int b = 0; b <= B; b++) { st[b] = b * np; s1[b] = b; ks[b] = b * cap; }
    for (int s = 0; s < cap; s++) for (int b = 0; b < B; b++) { pm[(size_t)s * B + b] = s; lm[(size_t)s * B + b] = s + 1; }
    for (int b = 0; b < B; b++) lr[b] = b * np + np - 1;
    upload(r.ids_d, prompts, (size_t)B * np * 4);
    upload(r.pos_d, pos.data(), pos.size() * 4);
    upload(r.start_np, st.data(), st.size() * 4);
    upload(r.start_1, s1.data(), s1.size() * 4);
    upload(r.kstart, ks.data(), ks.size() * 4);
    upload(r.posmat, pm.data(), pm.size() * 4);
    upload(r.lenmat, lm.data(), lm.size() * 4);
    upload(r.last_rows, lr.data(), lr.size() * 4);
}

// greedy pick over a long vocabulary row on many CTAs: block-local first-index argmax, then one atomicMax per
// block on (order-preserving value bits << 32 | ~index), so equal values resolve to the smallest index
__global__ void __launch_bounds__(256) k_argmax_packed(const float *__restrict__ logits, int V, int chunk,
                                                      unsigned long long *__restrict__ amax) {
    __shared__ unsigned long long red[256];
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y, v0 = blockIdx.x * chunk, v1 = min(V, v0 + chunk);
    const float *row = logits + (size_t)b * V;
    unsigned long long best = 0;
    for (int v = v0 + threadIdx.x; v < v1; v += 256) {
        unsigned u = __float_as_uint(row[v]);
        u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
        unsigned long long p = ((unsigned long long)u << 32) | (0xffffffffu - (unsigned)v);
        if (p > best) best = p;
    }
    red[threadIdx.x] = best;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if (threadIdx.x < s && red[threadIdx.x + s] > red[threadIdx.x]) red[threadIdx.x] = red[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0 && red[0]) atomicMax(amax + b, red[0]);
}

// closes a step: token s = *step_d of every row goes to out[b][s] and to ids[b] (the next step's input), the
// next step's uniforms are staged, the packed argmax is cleared, and the counter advances
__global__ void k_lm_finish_step(const int *__restrict__ pick, unsigned long long *__restrict__ amax, int greedy, int B, int n_new,
                                 int *__restrict__ out, int *__restrict__ ids, const double *__restrict__ uni, double *__restrict__ uni_cur,
                                 int *__restrict__ step_d) {
    pdl_launch_dependents();
    pdl_wait();
    const int s = *step_d;
    for (int b = threadIdx.x; b < B; b += blockDim.x) {
        int t = greedy ? (int)(0xffffffffu - (unsigned)(amax[b] & 0xffffffffull)) : pick[b];
        out[(size_t)b * n_new + s] = t;
        ids[b] = t;
        if (greedy) amax[b] = 0;
        else if (s + 1 < n_new) uni_cur[b] = uni[(size_t)(s + 1) * B + b];
    }
    __syncthreads();
    if (threadIdx.x == 0) *step_d = s + 1;
}

void lm_sample(LMRun &r, float temp, int top_k, float top_p, int n_new) {
    NcmbLM *m = r.m;
    const int greedy = !(temp > 0.f);
    if (greedy) {
        const int chunk = 2048;
        dim3 grid((unsigned)cdiv(m->V, chunk), (unsigned)r.B);
        ProfScope ps(NCMB_K_SAMPLE, 0, (double)r.B * m->V * 4);
        LAUNCH_PDL(k_argmax_packed, grid, 256, 0, r.logits, m->V, chunk, r.amax_d);
    } else {
        SampleArgs s{};
        s.logits = r.logits; s.Bn = r.B; s.Lc = 1; s.V = m->V; s.uncond_off = 0; s.cfg_w = 0;
        s.temp = temp; s.top_k = top_k; s.top_p = top_p;
        s.freq = 0; s.mu = 0; s.adj_a = 0; s.adj_w = 0; s.adj_d = 1;
        s.uniforms = r.uni_cur;
        s.out = r.pick_d; s.out_stride = 1; s.out_off = 0;
        s.scratch = r.samp_scr;
        sample_rows(s);
    }
    ProfScope ps(NCMB_K_SAMPLE, 0, 0);
    LAUNCH_PDL(k_lm_finish_step, 1, 256, 0, r.pick_d, r.amax_d, greedy, r.B, n_new, r.out_d, r.ids_d, r.uni_d, r.uni_cur, r.step_d);
}

} // namespace

extern "C" int ncmb_lm_generate(NcmbLM *m, const int *prompts, int B, int np, int n_new,
                                float temp, int top_k, float top_p, unsigned long long seed, int eos, int *out) {
    ensure_device();
    if (B <= 0 || np <= 0 || n_new <= 0) return 0;
    StaticWeights sw;
    if (np + n_new - 1 > m->n_ctx) fatal("%s: context overflow (%d + %d > %d)", m->is_qwen ? "qwen" : "gpt2", np, n_new, m->n_ctx);
    LMRun r;
    r.m = m; r.B = B; r.np = np; r.cap = np + n_new;
    lm_setup(r, prompts, n_new, 0);
    if (temp > 0) {
        // every row replays the reference's stream for this seed: one draw per generated token
        std::vector<double> u((size_t)n_new * B);
        unsigned long long st = seed ? seed : 0x12345678ULL;
        for (int s = 0; s < n_new; s++) {
            double v = (double)(rng_next(&st) >> 11) * (1.0 / 9007199254740992.0);
            for (int b = 0; b < B; b++) u[(size_t)s * B + b] = v;
        }
        upload(r.uni_d, u.data(), u.size() * 8);
    }
    CUDA_CHECK(cudaMemsetAsync(r.step_d, 0, 4 * sizeof(int), stream()));
    CUDA_CHECK(cudaMemsetAsync(r.amax_d, 0, (size_t)B * 8, stream()));
    if (temp > 0) CUDA_CHECK(cudaMemcpyAsync(r.uni_cur, r.uni_d, (size_t)B * 8, cudaMemcpyDeviceToDevice, stream()));
    lm_prefill(r);
    embed_rows(r.x, r.last_rows, r.last, B, m->C);           // hidden state of each row's last prompt token
    lm_head(r, r.last, B, r.logits);
    std::vector<int> col(B);
    std::vector<char> done(B, 0);
    int produced = 0;
    // Steps without a host decision (no EOS to watch) are replayed from one CUDA graph: the first decode step
    // runs eagerly (it sizes every workspace), the second is captured, the rest are graph launches. The work
    // moves to a stream of its own for that, because the caller's stream may be the legacy default stream,
    // which cannot be captured.
    // Up to four rows (head dim 64): the whole decode step is one persistent cooperative kernel; nothing to replay.
    bool qk_norm = false;
    for (auto &bw : m->blocks) qk_norm = qk_norm || bw.qnw || bw.knw;
    const bool mega = lm_mega_eligible(B, m->hd, m->C, m->I, qk_norm) && r.cap <= 2048 && n_new >= 2;
    MegaArgs mg{};
    if (mega) {
        std::vector<MegaLayer> hl(m->NL);
        for (int li = 0; li < m->NL; li++) {
            const BlockWeights &bw = m->blocks[li];
            hl[li] = MegaLayer{bw.ln1w, bw.ln1b, bw.qkvw, bw.qkvb, bw.ow, bw.ob, bw.ln2w, bw.ln2b, bw.fcw, bw.fcb, bw.pw, bw.pb, r.kv[li]};
        }
        upload(r.mg_layers, hl.data(), sizeof(MegaLayer) * hl.size());
        CUDA_CHECK(cudaMemsetAsync(r.mg_count, 0, ((size_t)B * m->nkv + 4) * 4, stream()));
        CUDA_CHECK(cudaMemsetAsync(r.mg_bar, 0, 16, stream()));
        CUDA_CHECK(cudaStreamSynchronize(stream()));             // hl goes out of scope
        const BlockWeights &b0 = m->blocks[0];
        mg.B = B; mg.C = m->C; mg.H = m->H; mg.nkv = m->nkv; mg.I = m->I; mg.NL = m->NL; mg.V = m->V;
        mg.norm = b0.norm == NORM_RMS ? 2 : 1; mg.gated = b0.gated; mg.act = b0.act; mg.rope = m->is_qwen ? 1 : 0;
        mg.eps = b0.norm == NORM_RMS ? 1e-6f : b0.eps; mg.eps_f = m->is_qwen ? 1e-6f : 1e-5f;
        mg.layers = r.mg_layers; mg.wte = m->wte; mg.wpe = m->is_qwen ? nullptr : m->wpe; mg.lnfw = m->lnfw; mg.lnfb = m->lnfb;
        mg.cosb = m->cosb; mg.sinb = m->sinb;
        mg.x = r.x; mg.qkv = r.bufs.qkv; mg.ctx = r.bufs.ctx; mg.h = r.bufs.h; mg.logits = r.logits;
        mg.part = r.mg_part; mg.count = r.mg_count;
        mg.ids = r.ids_d; mg.posmat = r.posmat; mg.lenmat = r.lenmat; mg.step_d = r.step_d;
        mg.np = np; mg.cap = r.cap; mg.n_new = n_new; mg.max_split = (r.cap + 31) / 32;
        mg.kv_seq_pitch = (int64_t)r.cap * 2 * m->nkv * m->hd;
        mg.bar = r.mg_bar; mg.bar_base = r.mg_bar + 1; mg.err = tc_err_flag();
        mg.greedy = !(temp > 0.f); mg.amax = r.amax_d; mg.out = r.out_d; mg.ids_out = r.ids_d;
    }
    static const bool graphs_ok = !getenv("NCM_B200_NO_GRAPH");
    const bool use_graph = !mega && graphs_ok && eos < 0 && n_new >= 4 && !prof_enabled();
    cudaStream_t user = stream(), gs = nullptr;
    cudaEvent_t ev = nullptr;
    cudaGraph_t graph = nullptr; cudaGraphExec_t gexec = nullptr;
    if (use_graph) {
        CUDA_CHECK(cudaStreamCreateWithFlags(&gs, cudaStreamNonBlocking));
        CUDA_CHECK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        CUDA_CHECK(cudaEventRecord(ev, user));
        CUDA_CHECK(cudaStreamWaitEvent(gs, ev, 0));
        ctx().stream = gs;
    }
    for (int s = 0; s < n_new; s++) {
        // (the sample + finish of a step is inside the graph for replayed steps, inside the kernel for greedy persistent steps)
        if (s == 0 || (!gexec && !(mega && mg.greedy))) lm_sample(r, temp, top_k, top_p, n_new);
        produced = s + 1;
        if (eos >= 0) {
            mem_d2h(col.data(), r.ids_d, (size_t)B * 4);
            bool all = true;
            for (int b = 0; b < B; b++) { if (col[b] == eos) done[b] = 1; all = all && done[b]; }
            if (all) break;
        }
        if (s + 1 == n_new) break;
        if (mega) { lm_mega_launch(mg); continue; }
        if (gexec) { CUDA_CHECK(cudaGraphLaunch(gexec, gs)); ctx().launches += r.graph_launches; continue; }
        const bool capture = use_graph && s == 1;
        long long l0 = ctx().launches;
        if (capture) CUDA_CHECK(cudaStreamBeginCapture(gs, cudaStreamCaptureModeThreadLocal));
        lm_decode_step(r, r.ids_d);
        lm_head(r, r.x, B, r.logits);
        if (capture) {
            lm_sample(r, temp, top_k, top_p, n_new);
            CUDA_CHECK(cudaStreamEndCapture(gs, &graph));
            CUDA_CHECK(cudaGraphInstantiate(&gexec, graph, 0));
            r.graph_launches = ctx().launches - l0;
            CUDA_CHECK(cudaGraphLaunch(gexec, gs));                      // capturing did not run the step: run it now
        }
    }
    if (use_graph) {
        CUDA_CHECK(cudaEventRecord(ev, gs));
        CUDA_CHECK(cudaStreamWaitEvent(user, ev, 0));
        ctx().stream = user;
        CUDA_CHECK(cudaStreamSynchronize(user));
        if (gexec) CUDA_CHECK(cudaGraphExecDestroy(gexec));
        if (graph) CUDA_CHECK(cudaGraphDestroy(graph));
        CUDA_CHECK(cudaEventDestroy(ev));
        CUDA_CHECK(cudaStreamDestroy(gs));
    }
    std::vector<int> tmp((size_t)B * n_new);
    mem_d2h(tmp.data(), r.out_d, tmp.size() * 4);
    for (int b = 0; b < B; b++) {
        bool ended = false;
        for (int s = 0; s < n_new; s++) {
            int v = (s < produced && !ended) ? tmp[(size_t)b * n_new + s] : -1;
            out[(size_t)b * n_new + s] = v;
            if (eos >= 0 && v == eos) ended = true;
        }
    }
    return produced;
}

extern "C" void ncmb_lm_logits(NcmbLM *m, const int *ids, int T, int last_only, float *out_host) {
    ensure_device();
    if (T <= 0) return;
    StaticWeights sw;
    if (T > m->n_ctx) fatal("%s: context overflow", m->is_qwen ? "qwen" : "gpt2");
    LMRun r;
    r.m = m; r.B = 1; r.np = T; r.cap = T;
    lm_setup(r, ids, 0, last_only ? 1 : T);
    lm_prefill(r);
    if (last_only) {
        lm_head(r, r.x + (size_t)(T - 1) * m->C, 1, r.logits);
        mem_d2h(out_host, r.logits, (size_t)m->V * 4);
    } else {
        // ln buffer holds T rows; head over all positions
        lm_head(r, r.x, T, r.logits);
        mem_d2h(out_host, r.logits, (size_t)T * m->V * 4);
    }
}

// ---------------------------------------------------------------------------------------------
// Next-token negative log-likelihood (reference gpt2_nll src/gpt2.c:160-176, qwen_nll src/qwen.c:192-208): the
// reference brings the [T][V] logits to the host and takes, per position, -log(exp(l[target] - max) / sum + 1e-30)
// in fp64. Here the logits stay on the device: one CTA per token row takes the row maximum and the fp64 sum of
// exponentials, and one double per position goes back to the host, which adds them in position order as the
// reference does.
__global__ void __launch_bounds__(256) k_nll_rows(const float *__restrict__ logits, const int *__restrict__ target, int V,
                                                  double *__restrict__ out) {
    __shared__ double red[256];
    const int64_t r = blockIdx.x;
    const int tg = target[r];
    if (tg < 0) { if (threadIdx.x == 0) out[r] = 0.0; return; }      // block-uniform: position without a successor
    const float *row = logits + r * V;
    float mxf = -INFINITY;
    for (int v = threadIdx.x; v < V; v += 256) mxf = fmaxf(mxf, row[v]);
    red[threadIdx.x] = (double)mxf;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if (threadIdx.x < s) red[threadIdx.x] = fmax(red[threadIdx.x], red[threadIdx.x + s]);
        __syncthreads();
    }
    const double mx = red[0];
    __syncthreads();
    double den = 0.0;
    for (int v = threadIdx.x; v < V; v += 256) den += exp((double)row[v] - mx);
    red[threadIdx.x] = den;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0) out[r] = -log(exp((double)row[tg] - mx) / red[0] + 1e-30);
}

// B windows of up to T ids each (row pitch T, lens[b] ids used; lens == NULL means T everywhere); nll_out[b] = mean
// over the lens[b] - 1 shifted positions. Padding sits behind the used ids, where causal attention cannot see it.
extern "C" void ncmb_lm_nll(NcmbLM *m, const int *ids, int B, int T, const int *lens, double *nll_out) {
    ensure_device();
    if (B <= 0 || T <= 0) return;
    StaticWeights sw;
    if (T > m->n_ctx) fatal("%s: context overflow", m->is_qwen ? "qwen" : "gpt2");
    const int64_t n = (int64_t)B * T;
    int64_t chunk = ((int64_t)512 << 20) / ((int64_t)m->V * 4);          // head rows per pass: at most 512 MB of logits
    if (chunk < 1) chunk = 1;
    if (chunk > n) chunk = n;
    std::vector<int> clean((size_t)n), tgt((size_t)n);
    for (int b = 0; b < B; b++) {
        const int len = lens ? lens[b] : T;
        if (len < 0 || len > T) fatal("ncmb_lm_nll: window %d has length %d outside 0..%d", b, len, T);
        for (int t = 0; t < T; t++) {
            const int id = t < len ? ids[(size_t)b * T + t] : 0;
            if (id < 0 || id >= m->V) fatal("ncmb_lm_nll: id %d out of range", id);
            clean[(size_t)b * T + t] = id;
            tgt[(size_t)b * T + t] = t + 1 < len ? ids[(size_t)b * T + t + 1] : -1;
        }
    }
    LMRun r;
    r.m = m; r.B = B; r.np = T; r.cap = T; r.nll_rows = n;
    lm_setup(r, clean.data(), 0, chunk);
    int *tgt_d = r.tgt_d;
    double *nll_d = r.nll_d;
    upload(tgt_d, tgt.data(), (size_t)n * 4);
    lm_prefill(r);
    for (int64_t r0 = 0; r0 < n; r0 += chunk) {
        const int64_t rows = n - r0 < chunk ? n - r0 : chunk;
        lm_head(r, r.x + r0 * m->C, rows, r.logits);
        ProfScope ps(NCMB_K_SAMPLE, 0, (double)rows * m->V * 4);
        k_nll_rows<<<(unsigned)rows, 256, 0, stream()>>>(r.logits, tgt_d + r0, m->V, nll_d + r0);
        CUDA_CHECK(cudaGetLastError());
    }
    std::vector<double> h((size_t)n);
    mem_d2h(h.data(), nll_d, (size_t)n * 8);
    for (int b = 0; b < B; b++) {
        const int len = lens ? lens[b] : T;
        double tot = 0;
        for (int t = 0; t + 1 < len; t++) tot += h[(size_t)b * T + t];
        nll_out[b] = len > 1 ? tot / (len - 1) : 0.0;
    }
}

static int lm_cmd_gen(const NCMConfig *c, const char *weights, const char *adir, const char *prompt, const char *ids_csv,
                      int n_new, float temp, int top_k, float top_p, unsigned long long seed, int is_qwen) {
    const char *who = is_qwen ? "qwen-gen" : "gpt2-gen";
    NcmbLM *m = ncmb_lm_open(c, weights, is_qwen, 0);
    if (!m) return 1;
    TokState *tok = tok_load ? tok_load(c, adir) : nullptr;
    const int cap = is_qwen ? 8192 : 4096;
    std::vector<int> ids(cap);
    int n = 0;
    if (ids_csv) {
        const char *p = ids_csv;
        while (*p && n < cap) { ids[n++] = atoi(p); while (*p && *p != ',') p++; if (*p) p++; }
    } else if (prompt) {
        if (!tok || !tok_encode) { fprintf(stderr, "%s: text prompts need the host tokenizer linked in; pass --ids\n", who); return 2; }
        n = tok_encode(tok, prompt, ids.data(), cap);
    } else {
        fprintf(stderr, is_qwen ? "qwen-gen needs --prompt TEXT | --ids CSV\n" : "gpt2-gen needs --prompt TEXT or --ids CSV\n");
        return 2;
    }
    if (n == 0) { fprintf(stderr, "%s: empty prompt\n", who); return 2; }
    int room = m->n_ctx - n + 1;
    if (n_new > room) { fprintf(stderr, "%s: context overflow\n", is_qwen ? "qwen" : "gpt2"); n_new = room > 0 ? room : 0; }
    std::vector<int> gen(n_new > 0 ? n_new : 1);
    int ngen = 0;
    if (n_new > 0) {
        ncmb_lm_generate(m, ids.data(), 1, n, n_new, temp, top_k, top_p, seed, m->eos, gen.data());
        while (ngen < n_new && gen[ngen] >= 0) ngen++;
    }
    printf("ids:");
    for (int i = 0; i < ngen; i++) printf(" %d", gen[i]);
    printf("\n");
    if (tok && tok_decode) {
        char *text = (char *)malloc(65536);
        tok_decode(tok, gen.data(), ngen, text, 65536, 1);
        printf("%s\n", text);
        free(text);
    }
    if (tok && tok_free) tok_free(tok);
    ncmb_lm_close(m);
    return 0;
}

extern "C" int gpt2_cmd_gen(const NCMConfig *c, const char *weights, const char *adir, const char *prompt, const char *ids_csv,
                            int n_new, float temp, int top_k, float top_p, unsigned long long seed) {
    return lm_cmd_gen(c, weights, adir, prompt, ids_csv, n_new, temp, top_k, top_p, seed, 0);
}
extern "C" int qwen_cmd_gen(const NCMConfig *c, const char *weights, const char *adir, const char *prompt, const char *ids_csv,
                            int n_new, float temp, int top_k, float top_p, unsigned long long seed) {
    return lm_cmd_gen(c, weights, adir, prompt, ids_csv, n_new, temp, top_k, top_p, seed, 1);
}

// ---------------------------------------------------------------------------------------------
// gpt2-ppl / qwen-ppl / gpt2-verify / qwen-verify (reference src/gpt2.c:237-270, 330-485; src/qwen.c:266-297,
// 323-478): same files in, same lines out. Windows of a document are batched onto the device instead of being run
// one by one. Text needs the reference's host tokenizer linked in (the weak tok_* symbols); without it a line of
// the texts file is read as white-space separated token ids, and the fixture checks that need text are skipped.

static int lm_line_ids(TokState *tok, const char *line, int *out, int cap) {
    if (tok && tok_encode) return tok_encode(tok, line, out, cap);
    int n = 0;
    const char *p = line;
    while (*p && n < cap) {
        while (*p == ' ' || *p == '\t' || *p == ',') p++;
        if (!*p) break;
        char *end = nullptr;
        long v = strtol(p, &end, 10);
        if (end == p) return -1;                      // not a list of ids
        out[n++] = (int)v;
        p = end;
    }
    return n;
}

namespace {
struct NllWindow { std::vector<int> ids; };

// mean NLL per window, windows batched by a token budget; results in the order given
std::vector<double> lm_nll_windows(NcmbLM *m, const std::vector<NllWindow> &ws) {
    std::vector<double> out(ws.size());
    const size_t budget = 16384;
    size_t i = 0;
    while (i < ws.size()) {
        size_t j = i, T = 0;
        while (j < ws.size()) {
            size_t t2 = std::max(T, ws[j].ids.size());
            if (j > i && t2 * (j - i + 1) > budget) break;
            T = t2; j++;
        }
        const int B = (int)(j - i);
        std::vector<int> ids((size_t)B * T, 0), lens(B);
        for (int b = 0; b < B; b++) {
            lens[b] = (int)ws[i + b].ids.size();
            std::copy(ws[i + b].ids.begin(), ws[i + b].ids.end(), ids.begin() + (size_t)b * T);
        }
        ncmb_lm_nll(m, ids.data(), B, (int)T, lens.data(), out.data() + i);
        i = j;
    }
    return out;
}
} // namespace

static int lm_cmd_ppl(const NCMConfig *c, const char *weights, const char *adir, const char *texts_path, int is_qwen) {
    NcmbLM *m = ncmb_lm_open(c, weights, is_qwen, 0);
    if (!m) return 1;
    TokState *tok = tok_load ? tok_load(c, adir) : nullptr;
    FILE *f = fopen(texts_path, "r");
    if (!f) { fprintf(stderr, "cannot open %s\n", texts_path); return 1; }
    const int window = is_qwen ? 512 : m->n_ctx;        // qwen.c:284, gpt2.c:255
    char *line = nullptr;
    size_t cap = 0;
    ssize_t len;
    int ndoc = 0;
    std::vector<int> ids(8192);
    std::vector<NllWindow> ws;
    while ((len = getline(&line, &cap, f)) >= 0) {
        while (len > 0 && (line[len - 1] == '\n' || line[len - 1] == '\r')) line[--len] = 0;
        if (!len) continue;
        int n = lm_line_ids(tok, line, ids.data(), 8192);
        if (n < 0) { fprintf(stderr, "%s: text lines need the host tokenizer linked in; give token ids\n", is_qwen ? "qwen-ppl" : "gpt2-ppl"); return 2; }
        if (n < 2) continue;
        for (int o = 0; o + 1 < n; o += window) {
            int T = n - o > window ? window : n - o;
            if (T < 2) break;
            NllWindow w;
            w.ids.assign(ids.begin() + o, ids.begin() + o + T);
            ws.push_back(std::move(w));
        }
        ndoc++;
    }
    free(line);
    fclose(f);
    std::vector<double> nw = lm_nll_windows(m, ws);
    double tot = 0;
    long ntok = 0;
    for (size_t i = 0; i < ws.size(); i++) {
        const int T = (int)ws[i].ids.size();
        tot += nw[i] * (T - 1);
        ntok += T - 1;
    }
    double nll = tot / ntok;
    printf("docs=%d tokens=%ld nll=%.6f ppl=%.6f\n", ndoc, ntok, nll, exp(nll));
    if (tok && tok_free) tok_free(tok);
    ncmb_lm_close(m);
    return 0;
}

extern "C" int gpt2_cmd_ppl(const NCMConfig *c, const char *weights, const char *adir, const char *texts_path) {
    return lm_cmd_ppl(c, weights, adir, texts_path, 0);
}
extern "C" int qwen_cmd_ppl(const NCMConfig *c, const char *weights, const char *adir, const char *texts_path) {
    return lm_cmd_ppl(c, weights, adir, texts_path, 1);
}

namespace {
int hex_nibble(char ch) {
    if (ch >= '0' && ch <= '9') return ch - '0';
    if (ch >= 'a' && ch <= 'f') return ch - 'a' + 10;
    if (ch >= 'A' && ch <= 'F') return ch - 'A' + 10;
    return -1;
}
bool hex_to_text(const char *h, std::string &out) {
    size_t n = strlen(h);
    if (n % 2) return false;
    out.clear();
    for (size_t i = 0; i < n; i += 2) {
        int a = hex_nibble(h[i]), b = hex_nibble(h[i + 1]);
        if (a < 0 || b < 0) return false;
        out.push_back((char)((a << 4) | b));
    }
    return true;
}
std::vector<int> ids_of(const char *s, size_t cap) {
    std::vector<int> v;
    while (*s && v.size() < cap) {
        while (*s == ' ') s++;
        if (!*s || *s == '\n' || *s == '\r') break;
        v.push_back(atoi(s));
        while (*s && *s != ' ' && *s != '\n' && *s != '\r') s++;
    }
    return v;
}
// splits "a\tb\tc" in place; false when a tab is missing
bool three_fields(char *line, char **b, char **c) {
    char *t1 = strchr(line, '\t');
    if (!t1) return false;
    *t1 = 0;
    char *t2 = strchr(t1 + 1, '\t');
    if (!t2) return false;
    *t2 = 0;
    *b = t1 + 1; *c = t2 + 1;
    return true;
}
} // namespace

static int lm_cmd_verify(const NCMConfig *c, const char *weights, const char *adir, const char *dir, int is_qwen) {
    const char *stem = is_qwen ? "qwen" : "gpt2";
    NcmbLM *m = ncmb_lm_open(c, weights, is_qwen, 0);
    if (!m) return 1;
    TokState *tok = tok_load ? tok_load(c, adir) : nullptr;
    const bool have_tok = tok && tok_encode;
    int fails = 0, checked = 0;
    char path[1024];
    std::vector<char> line(65536);
    const int V = m->V;
    // 1 + 2: tokenisation and all-position logits
    snprintf(path, sizeof(path), "%s/%s_tok.txt", dir, stem);
    FILE *f = fopen(path, "r");
    if (!f) { fprintf(stderr, "missing %s\n", path); return 1; }
    while (fgets(line.data(), (int)line.size(), f)) {
        char *hex, *idtxt;
        if (!three_fields(line.data(), &hex, &idtxt)) continue;
        const char *name = line.data();
        std::string text;
        if (!hex_to_text(hex, text)) { printf("FAIL tok %s: bad hex\n", name); fails++; checked++; continue; }
        std::vector<int> want = ids_of(idtxt, 8192);
        if (have_tok) {
            std::vector<int> got(8192);
            int n = tok_encode(tok, text.c_str(), got.data(), 8192);
            int bad = -1;
            if (n != (int)want.size()) { printf("FAIL tok %s: len %d vs %d\n", name, n, (int)want.size()); fails++; }
            else {
                for (int i = 0; i < n && bad < 0; i++) if (got[i] != want[i]) bad = i;
                if (bad >= 0) { printf("FAIL tok %s: pos %d got %d want %d\n", name, bad, got[bad], want[bad]); fails++; }
                else printf("ok   tok %s (%d ids exact)\n", name, n);
            }
        } else {
            printf("skip tok %s (host tokenizer not linked)\n", name);
        }
        checked++;
        const int T = (int)want.size();
        snprintf(path, sizeof(path), "%s/%s_logits_%s.f32", dir, stem, name);
        FILE *lf = fopen(path, "rb");
        checked++;
        if (!lf) { printf("FAIL logits %s: missing %s\n", name, path); fails++; continue; }
        std::vector<float> ref((size_t)T * V), got((size_t)T * V);
        size_t rd = fread(ref.data(), sizeof(float), ref.size(), lf);
        fclose(lf);
        if (rd != ref.size()) { printf("FAIL logits %s: short read\n", name); fails++; continue; }
        ncmb_lm_logits(m, want.data(), T, 0, got.data());
        double maxabs = 0, maxrel = 0;
        for (size_t i = 0; i < ref.size(); i++) {
            double a = got[i], b = ref[i], d = fabs(a - b);
            if (d > maxabs) maxabs = d;
            double r = d / (fabs(b) + 1.0);
            if (r > maxrel) maxrel = r;
        }
        const bool ok = is_qwen ? (maxrel < 5e-4 && maxabs < 1e-3) : (maxrel < 1e-4 && maxabs < 1e-2);   // qwen.c:379, gpt2.c:385
        printf("%s logits %s: maxabs=%.3g maxrel=%.3g\n", ok ? "ok  " : "FAIL", name, maxabs, maxrel);
        if (!ok) fails++;
    }
    fclose(f);
    // 3: greedy continuations
    snprintf(path, sizeof(path), "%s/%s_gen.txt", dir, stem);
    f = fopen(path, "r");
    if (!f) { fprintf(stderr, "missing %s\n", path); return 1; }
    while (fgets(line.data(), (int)line.size(), f)) {
        char *hex, *idtxt;
        if (!three_fields(line.data(), &hex, &idtxt)) continue;
        const char *name = line.data();
        std::string text;
        if (!hex_to_text(hex, text)) continue;
        std::vector<int> want = ids_of(idtxt, 256);
        const int ne = (int)want.size();
        if (!have_tok) { printf("skip gen %s (host tokenizer not linked)\n", name); checked++; continue; }
        std::vector<int> prompt(8192);
        int np = tok_encode(tok, text.c_str(), prompt.data(), 8192);
        std::vector<int> gen(ne > 0 ? ne : 1, -1);
        int ng = 0;
        if (ne > 0 && np > 0) {
            ncmb_lm_generate(m, prompt.data(), 1, np, ne, 0.0f, 0, 1.0f, 0, m->eos, gen.data());
            while (ng < ne && gen[ng] >= 0) ng++;
        }
        bool ok = ng == ne;
        for (int i = 0; ok && i < ne; i++) if (gen[i] != want[i]) ok = false;
        if (ok) printf("ok   gen %s (%d tokens exact)\n", name, ne);
        else { printf("FAIL gen %s: got %d tokens, want %d\n", name, ng, ne); fails++; }
        checked++;
    }
    fclose(f);
    // 4: likelihood of one text
    snprintf(path, sizeof(path), "%s/%s_ppl.txt", dir, stem);
    f = fopen(path, "r");
    if (f && fgets(line.data(), (int)line.size(), f)) {
        char *a, *b;
        if (three_fields(line.data(), &a, &b)) {
            std::string text;
            const double want_nll = atof(a), want_ppl = atof(b);
            if (hex_to_text(line.data(), text)) {
                if (!have_tok) { printf("skip ppl (host tokenizer not linked)\n"); }
                else {
                    std::vector<int> ids(8192);
                    int n = tok_encode(tok, text.c_str(), ids.data(), 8192);
                    double nll = 0;
                    ncmb_lm_nll(m, ids.data(), 1, n, nullptr, &nll);
                    if (fabs(nll - want_nll) < 1e-4) printf("ok   ppl nll=%.6f (want %.6f) ppl=%.4f (want %.4f)\n", nll, want_nll, exp(nll), want_ppl);
                    else { printf("FAIL ppl nll=%.6f want %.6f\n", nll, want_nll); fails++; }
                }
                checked++;
            }
        }
    }
    if (f) fclose(f);
    printf("%s-VERIFY %s (%d checked)\n", is_qwen ? "QWEN" : "GPT2", fails ? "FAIL" : "PASS", checked);
    if (tok && tok_free) tok_free(tok);
    ncmb_lm_close(m);
    return fails != 0;
}

extern "C" int gpt2_cmd_verify(const NCMConfig *c, const char *weights, const char *adir, const char *dir) {
    return lm_cmd_verify(c, weights, adir, dir, 0);
}
extern "C" int qwen_cmd_verify(const NCMConfig *c, const char *weights, const char *adir, const char *dir) {
    return lm_cmd_verify(c, weights, adir, dir, 1);
}
