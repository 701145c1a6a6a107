// NCP transformer: load, coarse-to-fine generate (monolithic and stepper) and the
// teacher-forced forward (reference src/ncp.c).
//
// What is different from the reference, with results kept identical:
//  * The reference re-runs the whole [prefix ; level] stack for every level, one
//    board at a time (src/ncp.c:1082-1104). Prefix rows never attend to level rows
//    (mask at :1078-1079) and their rotary positions do not depend on the level
//    (:126-131), so their hidden states, keys and values are the same at every
//    level. They are computed ONCE, batched over all rows, and each layer's K/V is
//    kept in an HBM cache; a level pass then runs only the level's tokens.
//  * Pad columns carry an additive -inf in the reference (:1084-1085): they
//    contribute exactly zero to every softmax and nothing reads their rows, so pad
//    positions are dropped from the batch altogether (per-row variable-length
//    prefixes; the unconditional CFG rows shrink to their single non-pad token).
//    A row whose prefix is ALL pad is NaN in the reference; here it is finite.
//  * Logits never leave the device: CFG blend, penalties and sampling run in one
//    kernel per level; the reference's RNG stream is pre-drawn on the host in its
//    (level, row, position) order so sampled codes match it draw for draw.
#include "common.cuh"
#include "vq.cuh"
#include "vqvae.cuh"

#include <vector>

using namespace ncmb;

struct HeadW {
    const float *W = nullptr, *b = nullptr;        // untied / shared: [V][C]
    const float *proj = nullptr, *projb = nullptr; // tied: [Dd][C]
    const float *E2 = nullptr, *b2 = nullptr;      // tied: scaled codebook [V][Dd] and folded bias [V]
    int V = 0, Dd = 0;
};

struct NCPState {
    NCMConfig cfg;
    WeightStore *ws = nullptr;
    VQVAEState *vqvae = nullptr;
    VQState *vq = nullptr;
    int L = 0, T = 0, P = 0, lvl_first = 0, n_tgt = 0;
    int one_pass_rows = 0; size_t one_pass_cap = 0;       // largest model batch that ran in one pass, on a workspace of this size
    int C = 0, H = 0, nkv = 0, hd = 0, D = 0, Hh = 0, NL = 0;
    float *rope_cos = nullptr, *rope_sin = nullptr;
    std::vector<float *> gcos, gsin;
    float *lvl_pos = nullptr;                      // [T][C]
    std::vector<BlockWeights> blocks;
    const float *lnfw = nullptr, *lnfb = nullptr, *wteW = nullptr, *wteB = nullptr, *wle = nullptr, *wpe = nullptr;
    const float *l0q = nullptr, *enc_wte = nullptr;
    std::vector<HeadW> heads;
    std::vector<const float *> pucW, pucB;
    std::vector<void *> owned;
    Workspace work, small;
};

struct NCPGen {
    NCPState *m = nullptr;
    int B = 0, Bm = 0, use_cfg = 0;
    float temp = 0, top_p = 1, cfg_scale = 0, freq = 0, mu = 0, adj_a = 0, adj_d = 1;
    int top_k = 0, adj_w = 0;
    int have_l0 = 0;
    int total = 0, Vmax = 0, Lmax = 0;
    // prefix compaction
    int ntok = 0, max_row = 0;
    int *row_start_d = nullptr, *tok_pos_d = nullptr, *tok_src_d = nullptr;
    // device state
    std::vector<float *> kv;                       // per layer [ntok][2*kvd]
    float *xpre = nullptr;                         // [ntok][C]
    BlockBufs bufs{};
    float *xlev = nullptr, *xout = nullptr, *xtmp = nullptr, *logits = nullptr, *z_hat = nullptr, *vqscr = nullptr;
    float *blend = nullptr, *samp_scr = nullptr;
    int *codes_d = nullptr, *l0tmp_d = nullptr, *hist_d = nullptr, *hist_len_d = nullptr;
    const int *lev_start_d[NCM_MAX_LEVELS] = {nullptr};
    int *lev_pos_d[NCM_MAX_LEVELS] = {nullptr};
    double *cnt_d = nullptr, *cnt0_d = nullptr, *uni_d = nullptr, *allow_d = nullptr;
    size_t uni_off = 0;
    unsigned long long seed = 0;
    const std::vector<double> *uni_given = nullptr;    // wave of a larger batch: this wave's slice of the batch's RNG stream
    int prefix_done = 0;
    int phase = 0, li = 0, level_accum = 0, out_off = 0, last_n = 0;
    float *cap_host = nullptr; size_t cap_row = 0, cap_off = 0;
    int *all_host = nullptr;
};

// ------------------------------------------------------------------ load

// cos/sin of pos * base^(-d/half) in fp64, duplicated over both halves (src/ncp.c:80-92)
static void rope_table(std::vector<float> &cs, std::vector<float> &sn, const std::vector<int> &pos, int hd, int base) {
    int half = hd / 2, S = (int)pos.size();
    cs.assign((size_t)S * hd, 0.f); sn.assign((size_t)S * hd, 0.f);
    for (int t = 0; t < S; t++) for (int d = 0; d < half; d++) {
        double inv = 1.0 / pow((double)base, (double)d / half);
        double f = pos[t] * inv;
        float co = (float)cos(f), si = (float)sin(f);
        cs[(size_t)t * hd + d] = co; cs[(size_t)t * hd + half + d] = co;
        sn[(size_t)t * hd + d] = si; sn[(size_t)t * hd + half + d] = si;
    }
}

static const float *opt_data(Tensor *t) { return t ? t->data : nullptr; }

extern "C" NCPState *ncp_load(const NCMConfig *c, WeightStore *ws, VQVAEState *vqvae) {
    ensure_device();
    NCPState *m = new NCPState();
    m->cfg = *c; m->ws = ws; m->vqvae = vqvae; m->vq = vqvae_vq(vqvae);
    m->P = c->prefix_len;
    m->lvl_first = c->query_level0 ? 0 : 1;
    for (int i = 0; i < c->n_qlevels; i++) m->L += c->levels[i];
    m->T = m->L - (c->query_level0 ? 0 : c->levels[0]);
    m->n_tgt = c->n_qlevels - m->lvl_first;
    m->C = c->n_embd; m->H = c->n_head; m->nkv = c->n_kv_heads; m->hd = m->C / m->H;
    m->D = c->vq_embed_dim; m->NL = c->n_layer;
    if (m->hd != 8 && m->hd != 16 && m->hd != 32 && m->hd != 64 && m->hd != 128)
        fatal("NCP head dim %d not supported (16, 32, 64, 128)", m->hd);
    int hd = m->hd, C = m->C, S = m->P + m->T;
    // rotary tables: the full-sequence one (API accessors) and one per target level
    parena_init(1ULL << 28);
    {
        std::vector<int> pos(S);
        for (int i = 0; i < m->P; i++) pos[i] = i;
        int o = m->P;
        for (int k = m->lvl_first; k < c->n_qlevels; k++) for (int t = 0; t < c->levels[k]; t++) pos[o++] = t;
        std::vector<float> cs, sn;
        rope_table(cs, sn, pos, hd, c->rope_base);
        m->rope_cos = parena_alloc((size_t)S * hd); m->rope_sin = parena_alloc((size_t)S * hd);
        upload(m->rope_cos, cs.data(), cs.size() * 4); upload(m->rope_sin, sn.data(), sn.size() * 4);
    }
    for (int k = 0; k < m->n_tgt; k++) {
        int lk = c->levels[k + m->lvl_first];
        std::vector<int> pos(m->P + lk);
        for (int i = 0; i < m->P; i++) pos[i] = i;
        for (int t = 0; t < lk; t++) pos[m->P + t] = t;
        std::vector<float> cs, sn;
        rope_table(cs, sn, pos, hd, c->rope_base);
        float *dc = parena_alloc(cs.size()), *ds = parena_alloc(sn.size());
        upload(dc, cs.data(), cs.size() * 4); upload(ds, sn.data(), sn.size() * 4);
        m->gcos.push_back(dc); m->gsin.push_back(ds);
    }
    m->wle = wneed(ws, "gen.transformer.wle.weight")->data;
    if (!c->use_rope) m->wpe = wneed(ws, "gen.transformer.wpe.weight")->data;
    // level_pos_embed: wle[level] per target position (+ wpe[t] without rope), src/ncp.c:143-173
    {
        std::vector<float> hwle((size_t)m->n_tgt * C), hlp((size_t)m->T * C);
        mem_d2h(hwle.data(), m->wle, hwle.size() * 4);
        int Tmax = m->P;
        for (int k = m->lvl_first; k < c->n_qlevels; k++) if (c->levels[k] > Tmax) Tmax = c->levels[k];
        std::vector<float> hwpe;
        if (!c->use_rope) { hwpe.resize((size_t)Tmax * C); mem_d2h(hwpe.data(), m->wpe, hwpe.size() * 4); }
        int tt = 0;
        for (int k = 0; k < m->n_tgt; k++)
            for (int t = 0; t < c->levels[k + m->lvl_first]; t++, tt++)
                for (int d = 0; d < C; d++) {
                    float v = hwle[(size_t)k * C + d];
                    if (!c->use_rope) v += hwpe[(size_t)t * C + d];
                    hlp[(size_t)tt * C + d] = v;
                }
        m->lvl_pos = parena_alloc(hlp.size());
        upload(m->lvl_pos, hlp.data(), hlp.size() * 4);
    }
    m->wteW = wneed(ws, "gen.transformer.wte.weight")->data;
    m->wteB = opt_data(wget(ws, "gen.transformer.wte.bias"));
    m->l0q = opt_data(wget(ws, "gen.l0_queries"));
    m->enc_wte = opt_data(wget(ws, "tok.encoder.wte.weight"));
    m->lnfw = wneed(ws, "gen.transformer.ln_f.weight")->data;
    m->lnfb = opt_data(wget(ws, "gen.transformer.ln_f.bias"));
    int gated = c->use_swiglu || c->use_geglu;
    for (int li = 0; li < c->n_layer; li++) {
        char pre[64];
        snprintf(pre, sizeof pre, "gen.transformer.blocks.%d.", li);
        BlockWeights w;
        w.norm = NORM_LAYER; w.eps = 1e-6f;
        w.ln1w = wneed(ws, "%sln_1.weight", pre)->data; w.ln1b = opt_data(wget(ws, "%sln_1.bias", pre));
        w.qkvw = wneed(ws, "%sattn.c_attn.weight", pre)->data; w.qkvb = opt_data(wget(ws, "%sattn.c_attn.bias", pre));
        w.ow = wneed(ws, "%sattn.c_proj.weight", pre)->data; w.ob = opt_data(wget(ws, "%sattn.c_proj.bias", pre));
        if (c->use_qk_norm) {
            w.qnw = wneed(ws, "%sattn.q_norm.weight", pre)->data;
            w.knw = wneed(ws, "%sattn.k_norm.weight", pre)->data;
        }
        w.ln2w = wneed(ws, "%sln_2.weight", pre)->data; w.ln2b = opt_data(wget(ws, "%sln_2.bias", pre));
        if (gated) {
            Tensor *tg = wneed(ws, "%smlp.w_gate.weight", pre), *tu = wneed(ws, "%smlp.w_up.weight", pre);
            int Hh = (int)tg->shape[0];
            Tensor *bg = wget(ws, "%smlp.w_gate.bias", pre), *bu = wget(ws, "%smlp.w_up.bias", pre);
            float *wcat = dev_concat_rows(tg->data, (int64_t)Hh * C, tu->data, (int64_t)Hh * C);
            m->owned.push_back(wcat);
            w.fcw = wcat;
            if (bg || bu) {
                float *bcat = dev_concat_rows(opt_data(bg), Hh, opt_data(bu), Hh);
                m->owned.push_back(bcat);
                w.fcb = bcat;
            }
            w.Hh = Hh; w.gated = 1; w.act = c->use_swiglu ? ACT_SILU : ACT_GELU;
        } else {
            Tensor *tf = wneed(ws, "%smlp.c_fc.weight", pre);
            w.fcw = tf->data; w.fcb = opt_data(wget(ws, "%smlp.c_fc.bias", pre));
            w.Hh = (int)tf->shape[0]; w.gated = 0; w.act = c->use_relu2 ? ACT_RELU2 : ACT_GELU;
        }
        w.pw = wneed(ws, "%smlp.c_proj.weight", pre)->data; w.pb = opt_data(wget(ws, "%smlp.c_proj.bias", pre));
        if (w.Hh > m->Hh) m->Hh = w.Hh;
        make_gated_interleaved(w, C, m->owned);
        m->blocks.push_back(w);
    }
    // output heads (src/ncp.c:406-477)
    for (int k = 0; k < m->n_tgt; k++) {
        HeadW h;
        h.V = c->vocab_size[k];
        if (c->shared_output_head) {
            h.W = wneed(ws, "gen.lm_heads.head.weight")->data;
            if (c->shared_head_per_level_bias) h.b = wneed(ws, "gen.lm_heads.biases.%d", k)->data;
            else if (c->untied_head_bias) h.b = wneed(ws, "gen.lm_heads.head.bias")->data;
        } else if (c->tie_heads_to_codebook) {
            Tensor *tp = wneed(ws, "gen.lm_heads.%d.proj.weight", k);
            h.proj = tp->data; h.Dd = (int)tp->shape[0];
            h.projb = opt_data(wget(ws, "gen.lm_heads.%d.proj.bias", k));
            Tensor *te = wneed(ws, "tok.vq.embeddings.%d.weight", k + m->lvl_first);
            int V = h.V, Dd = h.Dd;
            std::vector<float> hE((size_t)V * Dd), e2((size_t)V * Dd), b2(V), hb;
            mem_d2h(hE.data(), te->data, hE.size() * 4);
            std::vector<double> esq(V);
            double ds = 0;
            for (int v = 0; v < V; v++) {
                double s = 0;
                for (int d = 0; d < Dd; d++) s += (double)hE[(size_t)v * Dd + d] * hE[(size_t)v * Dd + d];
                esq[v] = s; ds += s;
            }
            ds /= V;
            float lit = 0;
            mem_d2h(&lit, wneed(ws, "gen.lm_heads.%d.log_inv_T", k)->data, 4);
            double invT = (double)expf(lit);
            Tensor *tb = wget(ws, "gen.lm_heads.%d.bias", k);
            if (tb) { hb.resize(V); mem_d2h(hb.data(), tb->data, (size_t)V * 4); }
            // logits = (2 z.E - |E|^2) / mean|E|^2 * invT + bias  ==  z.(2 invT/ds E) + (bias - |E|^2 invT/ds)
            for (size_t i = 0; i < hE.size(); i++) e2[i] = (float)(2.0 * invT / ds * (double)hE[i]);
            for (int v = 0; v < V; v++) b2[v] = (float)(-esq[v] * invT / ds + (tb ? (double)hb[v] : 0.0));
            float *dE2 = (float *)dev_alloc(e2.size() * 4), *db2 = (float *)dev_alloc((size_t)V * 4);
            upload(dE2, e2.data(), e2.size() * 4); upload(db2, b2.data(), (size_t)V * 4);
            m->owned.push_back(dE2); m->owned.push_back(db2);
            h.E2 = dE2; h.b2 = db2;
        } else {
            h.W = wneed(ws, "gen.lm_heads.%d.weight", k)->data;
            h.b = opt_data(wget(ws, "gen.lm_heads.%d.bias", k));
        }
        m->heads.push_back(h);
    }
    if (c->puc_enabled)
        for (int k = 0; k < m->n_tgt; k++) {
            m->pucW.push_back(wneed(ws, "gen.post_upsample_convs.%d.weight", k)->data);
            m->pucB.push_back(wneed(ws, "gen.post_upsample_convs.%d.bias", k)->data);
        }
    CUDA_CHECK(cudaStreamSynchronize(stream()));
    return m;
}

extern "C" void ncp_free(NCPState *m) {
    if (!m) return;
    for (void *p : m->owned) dev_free(p);
    m->work.release(); m->small.release();
    delete m;
}
extern "C" int ncp_P(NCPState *m) { return m->P; }
extern "C" int ncp_T(NCPState *m) { return m->T; }
extern "C" int ncp_ntgt(NCPState *m) { return m->n_tgt; }
extern "C" int ncp_lvlfirst(NCPState *m) { return m->lvl_first; }
extern "C" float *ncp_rope_cos(NCPState *m) { return m->rope_cos; }
extern "C" float *ncp_rope_sin(NCPState *m) { return m->rope_sin; }
extern "C" float *ncp_rope_gen_cos(NCPState *m, int k) { return m->gcos[k]; }
extern "C" float *ncp_rope_gen_sin(NCPState *m, int k) { return m->gsin[k]; }
extern "C" VQState *ncp_vq(NCPState *m) { return m->vq; }

// ------------------------------------------------------------------ shared pieces

static void head_logits(NCPState *m, int k, const float *x, int64_t rows, float *lg, float *tmp) {
    const HeadW &h = m->heads[k];
    GemmArgs g;
    if (h.proj) {
        g.x = x; g.ldx = m->C; g.W = h.proj; g.bias = h.projb; g.y = tmp; g.ldy = h.Dd; g.M = rows; g.N = h.Dd; g.K = m->C;
        gemm(g);
        g = GemmArgs();
        g.x = tmp; g.ldx = h.Dd; g.W = h.E2; g.bias = h.b2; g.y = lg; g.ldy = h.V; g.M = rows; g.N = h.V; g.K = h.Dd;
        gemm(g);
    } else {
        g.x = x; g.ldx = m->C; g.W = h.W; g.bias = h.b; g.y = lg; g.ldy = h.V; g.M = rows; g.N = h.V; g.K = m->C;
        gemm(g);
    }
}

// Fills the per-layer K/V cache from the compacted prefix tokens in g->xpre.
static void prefix_pass(NCPGen *g) {
    NCPState *m = g->m;
    AttnPlan p;
    p.q_start = p.k1_start = g->row_start_d;
    p.rows = g->Bm; p.max_q = g->max_row; p.max_k1 = g->max_row;
    p.pos = g->tok_pos_d;
    if (m->cfg.use_rope) { p.cos_t = m->gcos[0]; p.sin_t = m->gsin[0]; }
    p.total_q = g->ntok; p.avg_keys = g->Bm ? (double)g->ntok / g->Bm : 0;
    p.kv_pitch = 2 * m->nkv * m->hd;
    for (int li = 0; li < m->NL; li++) {
        p.kv_store = g->kv[li];
        p.kv_only = (li == m->NL - 1);            // the last layer's prefix outputs are never read
        run_block(g->xpre, g->ntok, m->C, m->H, m->nkv, m->blocks[li], g->bufs, p);
    }
    g->prefix_done = 1;
}

// One pass of the stack over `Lc` level tokens per model row (x: [Bm*Lc][C]), then
// ln_f and head `hi` into g->logits [Bm*Lc][V].
static void level_pass(NCPGen *g, float *x, int Lc, int hi, int lev_slot) {
    NCPState *m = g->m;
    int kvd = m->nkv * m->hd;
    int64_t n = (int64_t)g->Bm * Lc;
    AttnPlan p;
    p.q_start = g->lev_start_d[lev_slot];
    p.k1_start = g->row_start_d;
    p.ldk1 = 2 * kvd;
    p.self_is_k2 = 1;
    p.rows = g->Bm; p.max_q = Lc; p.max_k1 = g->max_row; p.k1_total = g->ntok;
    p.pos = g->lev_pos_d[lev_slot];
    if (m->cfg.use_rope) { p.cos_t = m->gcos[hi]; p.sin_t = m->gsin[hi]; }
    p.total_q = n; p.avg_keys = (g->Bm ? (double)g->ntok / g->Bm : 0) + Lc;
    for (int li = 0; li < m->NL; li++) {
        p.k1 = g->kv[li]; p.v1 = g->kv[li] + kvd;
        run_block(x, n, m->C, m->H, m->nkv, m->blocks[li], g->bufs, p);
    }
    layernorm(x, m->lnfw, m->lnfb, g->bufs.ln, n, m->C, 1e-6f);
    head_logits(m, hi, g->bufs.ln, n, g->logits, g->bufs.ctx);
}

// The same for the teacher-forced forward with the block-causal pattern (reference src/ncp.c:361-404: a target
// token sees the prefix and every target token of its own and of earlier levels). Levels are passed in order;
// each layer keeps the levels' final K|V in a cache of its own (`lvlkv[li]`, [B][T][2*kvd]), so a level's keys are
// that cache up to and including itself (segment 1, per-row length `len_d`) plus the cached prefix (segment 2).
static void level_pass_causal(NCPGen *g, float *x, int Lc, int hi, int lev_slot, int off, std::vector<float *> &lvlkv,
                              const int *seq_start_d, const int *len_d) {
    NCPState *m = g->m;
    int kvd = m->nkv * m->hd;
    int64_t n = (int64_t)g->Bm * Lc;
    AttnPlan p;
    p.q_start = g->lev_start_d[lev_slot];
    p.k1_start = seq_start_d; p.k1_len = len_d; p.ldk1 = 2 * kvd;
    p.max_k1 = off + Lc; p.k1_total = (int64_t)g->Bm * m->T;
    p.k2_start = g->row_start_d; p.ldk2 = 2 * kvd; p.max_k2 = g->max_row; p.k2_total = g->ntok;
    p.rows = g->Bm; p.max_q = Lc;
    p.pos = g->lev_pos_d[lev_slot];
    if (m->cfg.use_rope) { p.cos_t = m->gcos[hi]; p.sin_t = m->gsin[hi]; }
    p.total_q = n; p.avg_keys = (g->Bm ? (double)g->ntok / g->Bm : 0) + off + Lc;
    p.kv_pitch = 2 * kvd; p.kv_rows_per_seq = Lc; p.kv_seq_pitch = (int64_t)m->T * 2 * kvd;
    for (int li = 0; li < m->NL; li++) {
        p.k1 = lvlkv[li]; p.v1 = lvlkv[li] + kvd;
        p.k2 = g->kv[li]; p.v2 = g->kv[li] + kvd;
        p.kv_store = lvlkv[li] + (size_t)off * 2 * kvd;
        run_block(x, n, m->C, m->H, m->nkv, m->blocks[li], g->bufs, p);
    }
    layernorm(x, m->lnfw, m->lnfb, g->bufs.ln, n, m->C, 1e-6f);
    head_logits(m, hi, g->bufs.ln, n, g->logits, g->bufs.ctx);
}

// x += conv(x) as the reference's GENERATE path computes it: the conv output stays in
// [B][D][L] order and is added element i to element i onto the [B][L][D] tensor
// (src/ncp.c:863-869, 1040-1045). Kept bit-compatible on purpose.
static void puc_generate(NCPState *m, int idx, float *x, float *tmp, int Bm, int Lc, int K) {
    int D = m->D;
    conv1d(x, nlc(D, Lc), m->pucW[idx], m->pucB[idx], tmp, ncl(D, Lc), Bm, D, D, Lc, K, 1, K / 2, x, 0.f);
    CUDA_CHECK(cudaMemcpyAsync(x, tmp, (size_t)Bm * Lc * D * 4, cudaMemcpyDeviceToDevice, stream()));
}

// ------------------------------------------------------------------ generate

static void gen_plan(NCPGen *g, const int *l0, const int *prefix_ids, const double *allow) {
    NCPState *m = g->m;
    const NCMConfig *c = &m->cfg;
    int B = g->B, Bm = g->Bm, P = m->P, C = m->C, D = m->D, nlev = c->n_qlevels;
    int kvd = m->nkv * m->hd, Wq = C + 2 * kvd;
    g->total = vq_total_codes(m->vq);
    for (int k = 0; k < m->n_tgt; k++) if (c->vocab_size[k] > g->Vmax) g->Vmax = c->vocab_size[k];
    for (int k = 0; k < nlev; k++) if (c->levels[k] > g->Lmax) g->Lmax = c->levels[k];
    // ---- host planning: model prefix, pad flags, compaction ----
    std::vector<int> mp((size_t)Bm * P);
    memcpy(mp.data(), prefix_ids, (size_t)B * P * sizeof(int));
    if (g->use_cfg) {
        int null_first = c->eos_token_id >= 0 ? c->eos_token_id : c->prefix_pad_token_id;
        for (int b = B; b < Bm; b++) {
            for (int s = 0; s < P; s++) mp[(size_t)b * P + s] = c->prefix_pad_token_id;
            if (P > 0) mp[(size_t)b * P] = null_first;
        }
    }
    std::vector<int> row_start(Bm + 1, 0), tok_pos, tok_id;
    tok_pos.reserve((size_t)Bm * P); tok_id.reserve((size_t)Bm * P);
    for (int b = 0; b < Bm; b++) {
        for (int s = 0; s < P; s++) {
            int id = mp[(size_t)b * P + s];
            if (c->prefix_pad_token_id >= 0 && id == c->prefix_pad_token_id) continue;
            tok_pos.push_back(s); tok_id.push_back(id);
        }
        row_start[b + 1] = (int)tok_pos.size();
        int len = row_start[b + 1] - row_start[b];
        if (len > g->max_row) g->max_row = len;
    }
    g->ntok = (int)tok_pos.size();
    // ---- RNG stream (reference order): level 0 draws for every model row, then B rows per level ----
    int l0len = c->levels[0];
    bool sample_l0 = !l0 && c->query_level0;
    size_t ndraw = 0;
    if (g->temp > 0) {
        if (sample_l0) ndraw += (size_t)Bm * l0len;
        for (int k = 1; k < nlev; k++) ndraw += (size_t)B * c->levels[k];
    }
    std::vector<double> uni;
    if (ndraw && ctx().rng_mode == 0) {
        if (g->uni_given) {
            if (g->uni_given->size() != ndraw) fatal("ncp_generate: wave RNG slice has %zu draws, expected %zu", g->uni_given->size(), ndraw);
            uni = *g->uni_given;
        } else {
            uni.resize(ndraw);
            unsigned long long st = g->seed ? g->seed : 0x9E3779B97F4A7C15ULL;
            for (size_t i = 0; i < ndraw; i++) uni[i] = (double)(rng_next(&st) >> 11) * (1.0 / 9007199254740992.0);
        }
    }
    // ---- workspace: one sizing pass over the layout, then the real one ----
    int64_t nmax = g->ntok > (int64_t)Bm * g->Lmax ? g->ntok : (int64_t)Bm * g->Lmax;
    if (nmax < 1) nmax = 1;
    int Hh = m->Hh;
    bool any_gated = false;
    for (auto &bw : m->blocks) any_gated |= (bw.gated != 0);
    size_t nzl = (size_t)Bm * m->vq->L * D;
    bool penal = (g->freq > 0) || (g->adj_a != 0);
    auto layout = [&](Workspace &w) {
        g->kv.clear();
        g->row_start_d = w.get<int>(Bm + 1);
        g->tok_pos_d = w.get<int>(g->ntok + 1);
        g->tok_src_d = w.get<int>(g->ntok + 1);
        g->xpre = w.get<float>((size_t)(g->ntok + 1) * C);
        g->bufs.ln = w.get<float>((size_t)nmax * C);
        g->bufs.qkv = w.get<float>((size_t)nmax * Wq);
        g->bufs.ctx = w.get<float>((size_t)nmax * C);
        g->bufs.mlp = any_gated ? w.get<float>((size_t)nmax * 2 * Hh) : nullptr;
        g->bufs.h = w.get<float>((size_t)nmax * Hh);
        for (int li = 0; li < m->NL; li++) g->kv.push_back(w.get<float>((size_t)g->ntok * 2 * kvd + 4));
        g->xlev = w.get<float>((size_t)Bm * g->Lmax * C);
        g->xout = w.get<float>((size_t)Bm * g->Lmax * D);
        g->xtmp = w.get<float>((size_t)Bm * g->Lmax * D);
        g->logits = w.get<float>((size_t)Bm * g->Lmax * g->Vmax);
        g->z_hat = w.get<float>(nzl);
        g->vqscr = w.get<float>(5 * nzl);
        size_t ss = sample_scratch_floats(Bm, g->Vmax);
        g->samp_scr = ss ? w.get<float>(ss) : nullptr;
        g->blend = g->cap_host ? w.get<float>((size_t)Bm * g->Lmax * g->Vmax) : nullptr;
        g->cnt_d = w.get<double>((size_t)Bm * g->Vmax);
        g->cnt0_d = w.get<double>((size_t)Bm * g->Vmax);
        g->uni_d = uni.empty() ? nullptr : w.get<double>(ndraw);
        g->allow_d = (allow && penal) ? w.get<double>(g->Vmax) : nullptr;
        g->hist_d = w.get<int>((size_t)Bm * (g->total + 64));
        g->hist_len_d = w.get<int>(2 * (size_t)Bm);
        g->codes_d = w.get<int>((size_t)B * g->total);
        g->l0tmp_d = w.get<int>((size_t)Bm * g->Lmax);
        for (int k = 0; k < nlev; k++) {
            g->lev_start_d[k] = w.get<int>(Bm + 1);
            g->lev_pos_d[k] = w.get<int>((size_t)Bm * c->levels[k]);
        }
    };
    {
        Workspace sizing;
        sizing.measuring = true;
        layout(sizing);
        m->work.reserve(sizing.off + 4096);
        m->work.reset();
        layout(m->work);
    }
    upload(g->row_start_d, row_start.data(), (size_t)(Bm + 1) * 4);
    upload(g->tok_pos_d, tok_pos.data(), (size_t)g->ntok * 4);
    upload(g->tok_src_d, tok_id.data(), (size_t)g->ntok * 4);
    // per-level uniform row starts and rotary positions (P + t)
    for (int k = 0; k < nlev; k++) {
        int Lk = c->levels[k];
        std::vector<int> st(Bm + 1), ps((size_t)Bm * Lk);
        for (int b = 0; b <= Bm; b++) st[b] = b * Lk;
        for (int b = 0; b < Bm; b++) for (int t = 0; t < Lk; t++) ps[(size_t)b * Lk + t] = P + t;
        upload((void *)g->lev_start_d[k], st.data(), st.size() * 4);
        upload(g->lev_pos_d[k], ps.data(), ps.size() * 4);
    }
    if (g->uni_d) upload(g->uni_d, uni.data(), ndraw * 8);
    if (g->allow_d) upload(g->allow_d, allow, (size_t)g->Vmax * 8);
    CUDA_CHECK(cudaMemsetAsync(g->z_hat, 0, nzl * 4, stream()));
    CUDA_CHECK(cudaMemsetAsync(g->cnt_d, 0, (size_t)Bm * g->Vmax * 8, stream()));
    CUDA_CHECK(cudaMemsetAsync(g->hist_len_d, 0, 2 * (size_t)Bm * 4, stream()));
    CUDA_CHECK(cudaMemsetAsync(g->codes_d, 0, (size_t)B * g->total * 4, stream()));
    if (l0) {
        g->have_l0 = 1;
        std::vector<int> tmp((size_t)B * g->total, 0);
        for (int b = 0; b < B; b++) memcpy(&tmp[(size_t)b * g->total], l0 + (size_t)b * l0len, (size_t)l0len * 4);
        upload(g->codes_d, tmp.data(), tmp.size() * 4);
    }
    if (g->cap_host) {
        g->cap_row = 0;
        if (sample_l0) g->cap_row += (size_t)l0len * c->vocab_size[0];
        for (int li = 0; li < nlev - 1; li++) g->cap_row += (size_t)c->levels[li + 1] * c->vocab_size[li + (1 - m->lvl_first)];
    }
}

// prefix embeddings of the compacted tokens: wte(E_enc[id]) (+ wpe[pos] without rope), src/ncp.c:768-792
static void prefix_embed(NCPGen *g) {
    NCPState *m = g->m;
    if (g->ntok == 0) return;
    if (!m->enc_wte) { fprintf(stderr, "missing weight tok.encoder.wte.weight\n"); exit(1); }
    float *zpre = g->bufs.ln;                       // [ntok][D] scratch (C >= D is not required: ln holds nmax*C >= ntok*? )
    if ((size_t)m->D > (size_t)m->C) zpre = g->bufs.h;
    embed_rows(m->enc_wte, g->tok_src_d, zpre, g->ntok, m->D);
    GemmArgs a;
    a.x = zpre; a.ldx = m->D; a.W = m->wteW; a.bias = m->wteB; a.y = g->xpre; a.ldy = m->C; a.M = g->ntok; a.N = m->C; a.K = m->D;
    gemm(a);
    if (!m->cfg.use_rope) {
        // xpre[i] += wpe[pos[i]]: gather the rows then add
        embed_rows(m->wpe, g->tok_pos_d, g->bufs.ctx, g->ntok, m->C);
        add_inplace(g->xpre, g->bufs.ctx, (int64_t)g->ntok * m->C);
    }
}

static void capture_level(NCPGen *g, int Lc, int V) {
    if (!g->cap_host) return;
    CUDA_CHECK(cudaStreamSynchronize(stream()));
    CUDA_CHECK(cudaMemcpy2D(g->cap_host + g->cap_off, g->cap_row * 4, g->blend, (size_t)Lc * V * 4, (size_t)Lc * V * 4,
                            g->B, cudaMemcpyDeviceToHost));
    g->cap_off += (size_t)Lc * V;
    ctx().d2h_bytes += (unsigned long long)g->B * Lc * V * 4;
}

static void gen_l0(NCPGen *g) {
    NCPState *m = g->m;
    const NCMConfig *c = &m->cfg;
    int Bm = g->Bm, B = g->B, C = m->C, D = m->D, l0len = c->levels[0];
    if (!g->prefix_done) { prefix_embed(g); prefix_pass(g); }
    if (!g->have_l0) {
        if (!c->query_level0) { fprintf(stderr, "generate(idx=None) requires query_level0 or predict_level0\n"); exit(1); }
        if (!m->l0q) { fprintf(stderr, "missing weight gen.l0_queries\n"); exit(1); }
        // q0 = l0_queries broadcast over rows
        for (int b = 0; b < Bm; b++)
            CUDA_CHECK(cudaMemcpyAsync(g->xout + (size_t)b * l0len * D, m->l0q, (size_t)l0len * D * 4, cudaMemcpyDeviceToDevice, stream()));
        if (c->puc_enabled) puc_generate(m, 0, g->xout, g->xtmp, Bm, l0len, 3);
        GemmArgs a;
        a.x = g->xout; a.ldx = D; a.W = m->wteW; a.bias = m->wteB; a.y = g->xlev; a.ldy = C; a.M = (int64_t)Bm * l0len; a.N = C; a.K = D;
        gemm(a);
        add_rows_bcast(g->xlev, m->wle, (int64_t)Bm * l0len, C);          // + wle[0] on every position
        level_pass(g, g->xlev, l0len, 0, 0);
        // every model row samples level 0 on its own, fresh penalty state (src/ncp.c:933-944)
        int V0 = c->vocab_size[0];
        bool penal = (g->freq > 0) || (g->adj_a != 0);
        if (penal) CUDA_CHECK(cudaMemsetAsync(g->cnt0_d, 0, (size_t)Bm * g->Vmax * 8, stream()));
        SampleArgs s{};
        s.logits = g->logits; s.Bn = Bm; s.Lc = l0len; s.V = V0; s.uncond_off = 0; s.cfg_w = 0;
        s.temp = g->temp; s.top_k = g->top_k; s.top_p = g->top_p;
        s.freq = g->freq; s.mu = g->mu; s.adj_a = g->adj_a; s.adj_w = g->adj_w; s.adj_d = g->adj_d;
        s.allow_dev = g->allow_d; s.cnt = penal ? g->cnt0_d : nullptr; s.cnt_stride = g->Vmax;
        s.hist = penal ? g->hist_d : nullptr; s.hist_len = penal ? g->hist_len_d + Bm : nullptr; s.hist_stride = g->total + 64;
        s.uniforms = g->uni_d ? g->uni_d + g->uni_off : nullptr;
        s.rng_seed = g->seed; s.rng_row0 = ctx().row_offset; s.rng_level = 0; s.rng_wrap = Bm > B ? B : 0;
        s.out = g->l0tmp_d; s.out_stride = l0len; s.out_off = 0;
        s.blend_out = g->blend; s.scratch = g->samp_scr; s.picks_bound = g->total;
        sample_rows(s);
        if (g->temp > 0) g->uni_off += (size_t)Bm * l0len;
        CUDA_CHECK(cudaMemcpy2DAsync(g->codes_d, (size_t)g->total * 4, g->l0tmp_d, (size_t)l0len * 4, (size_t)l0len * 4, B,
                                     cudaMemcpyDeviceToDevice, stream()));
        capture_level(g, l0len, V0);
        if (penal) CUDA_CHECK(cudaMemsetAsync(g->hist_len_d, 0, 2 * (size_t)Bm * 4, stream()));
    }
    g->level_accum = (m->lvl_first == 0) ? c->levels[0] : 0;
    g->out_off = l0len;
    g->last_n = l0len;
    g->phase = 1; g->li = 0;
}

static void gen_level(NCPGen *g, int li) {
    NCPState *m = g->m;
    const NCMConfig *c = &m->cfg;
    int Bm = g->Bm, B = g->B, C = m->C, D = m->D, nlev = c->n_qlevels;
    int hi = li + (1 - m->lvl_first), Lcur = c->levels[li + 1], V = c->vocab_size[hi];
    int prev_off = g->out_off - c->levels[li];
    // autoregressive input from the previous level's codes (the CFG half reuses them)
    vq_next_input_dev(m->vq, g->codes_d + prev_off, g->total, g->use_cfg ? B : 0, li, g->z_hat, g->xout, Bm, g->vqscr);
    if (c->puc_enabled) puc_generate(m, hi, g->xout, g->xtmp, Bm, Lcur, c->puc_kernel);
    GemmArgs a;
    a.x = g->xout; a.ldx = D; a.W = m->wteW; a.bias = m->wteB; a.y = g->xlev; a.ldy = C; a.M = (int64_t)Bm * Lcur; a.N = C; a.K = D;
    gemm(a);
    add_rows_bcast(g->xlev, m->lvl_pos + (size_t)g->level_accum * C, Bm, Lcur * C);
    level_pass(g, g->xlev, Lcur, hi, li + 1);
    bool penal = (g->freq > 0) || (g->adj_a != 0);
    SampleArgs s{};
    s.logits = g->logits; s.Bn = B; s.Lc = Lcur; s.V = V;
    s.uncond_off = g->use_cfg ? B : 0;
    s.cfg_w = g->use_cfg ? (double)g->cfg_scale * ((li + 1) / (double)(nlev - 1)) : 0.0;
    s.temp = g->temp; s.top_k = g->top_k; s.top_p = g->top_p;
    s.freq = g->freq; s.mu = g->mu; s.adj_a = g->adj_a; s.adj_w = g->adj_w; s.adj_d = g->adj_d;
    s.allow_dev = g->allow_d; s.cnt = penal ? g->cnt_d : nullptr; s.cnt_stride = g->Vmax;
    s.hist = penal ? g->hist_d : nullptr; s.hist_len = penal ? g->hist_len_d : nullptr; s.hist_stride = g->total + 64;
    s.uniforms = g->uni_d ? g->uni_d + g->uni_off : nullptr;
    s.rng_seed = g->seed; s.rng_row0 = ctx().row_offset; s.rng_level = li + 1;
    s.out = g->codes_d; s.out_stride = g->total; s.out_off = g->out_off;
    s.blend_out = g->blend; s.scratch = g->samp_scr; s.picks_bound = g->total;
    sample_rows(s);
    if (g->temp > 0) g->uni_off += (size_t)B * Lcur;
    capture_level(g, Lcur, V);
    g->out_off += Lcur;
    g->last_n = Lcur;
    g->level_accum += Lcur;
}

extern "C" {

NCPGen *ncp_gen_begin(NCPState *m, const int *l0, const int *prefix_ids, int B,
                      float temp, int top_k, float top_p, float cfg_scale,
                      float freq, float mu, float adj_a, int adj_w, float adj_d,
                      const double *allow, unsigned long long seed) {
    ensure_device();
    if (B <= 0) fatal("ncp_gen_begin: batch %d", B);
    NCPGen *g = new NCPGen();
    g->m = m; g->B = B;
    g->temp = temp; g->top_k = top_k; g->top_p = top_p; g->cfg_scale = cfg_scale;
    g->freq = freq; g->mu = mu; g->adj_a = adj_a; g->adj_w = adj_w; g->adj_d = adj_d;
    g->seed = seed;
    g->use_cfg = cfg_scale > 0;
    g->Bm = g->use_cfg ? 2 * B : B;
    if (g->use_cfg && m->cfg.prefix_pad_token_id < 0)
        fatal("classifier-free guidance needs model.prefix_pad_token_id >= 0 (the null prefix is built from it)");
    gen_plan(g, l0, prefix_ids, allow);
    return g;
}

int ncp_gen_nsteps(NCPGen *g) { return g->m->cfg.n_qlevels; }
int ncp_gen_step_size(NCPGen *g, int s) {
    if (s < 0 || s >= g->m->cfg.n_qlevels) return -1;
    return g->m->cfg.levels[s];
}

int ncp_gen_step(NCPGen *g, int *codes_out, int *n_out) {
    if (g->phase == 2) return 1;
    StaticWeights sw;
    if (g->phase == 0) {
        gen_l0(g);
        if (g->m->cfg.n_qlevels <= 1) g->phase = 2;
    } else {
        if (g->li >= g->m->cfg.n_qlevels - 1) { g->phase = 2; return 1; }
        gen_level(g, g->li);
        g->li++;
        if (g->li >= g->m->cfg.n_qlevels - 1) g->phase = 2;
    }
    if (codes_out) mem_d2h(codes_out, g->codes_d + (g->out_off - g->last_n), (size_t)g->last_n * sizeof(int));
    if (n_out) *n_out = g->last_n;
    return 0;
}

const int *ncmb_gen_codes_dev(NCPGen *g) { return g->codes_d; }

int *ncp_gen_finish(NCPGen *g) {
    int *all = (int *)malloc((size_t)g->B * g->total * sizeof(int));
    if (!all) fatal("oom codes");
    mem_d2h(all, g->codes_d, (size_t)g->B * g->total * sizeof(int));
    delete g;
    return all;
}

void ncp_gen_abort(NCPGen *g) {
    CUDA_CHECK(cudaStreamSynchronize(stream()));
    delete g;
}

// Device bytes one generate over B sequences needs (upper bound: every prefix position kept), following the
// workspace layout of gen_plan plus the split-pair scratch of the blocks.
static double gen_bytes_bound(NCPState *m, int B, bool use_cfg, bool capture) {
    const NCMConfig *c = &m->cfg;
    const int nlev = c->n_qlevels, C = m->C, D = m->D, kvd = m->nkv * m->hd, Wq = C + 2 * kvd, Hh = m->Hh;
    int Lmax = 0, Vmax = 0, total = 0;
    for (int k = 0; k < nlev; k++) { Lmax = std::max(Lmax, c->levels[k]); total += c->levels[k]; }
    for (int k = 0; k < m->n_tgt; k++) Vmax = std::max(Vmax, c->vocab_size[k]);
    const double Bm = use_cfg ? 2.0 * B : B;
    const double ntok = (double)B * m->P + (use_cfg ? B : 0), nmax = std::max(ntok, Bm * Lmax);
    bool gated = false;
    for (auto &bw : m->blocks) gated |= (bw.gated != 0);
    double fl = ntok * C + nmax * (2.0 * C + Wq + (gated ? 2.0 * Hh : 0.0) + Hh) + m->NL * ntok * 2.0 * kvd
              + Bm * Lmax * (C + 2.0 * D + (capture ? 2.0 : 1.0) * Vmax) + 6.0 * Bm * m->vq->L * D
              + nmax * (2.0 * C + Hh)                                   /* split-pair scratch of the blocks */
              + 2.0 * ntok + Bm * (total + 70.0) + B * (double)total;   /* index arrays */
    double db = 2.0 * Bm * Vmax + Bm * total;
    return 4.0 * fl + 8.0 * db + (64 << 20);
}

static int *gen_one(NCPState *m, const int *l0, const int *prefix_ids, int B,
                    float temp, int top_k, float top_p, float cfg_scale,
                    float freq, float mu, float adj_a, int adj_w, float adj_d,
                    const double *allow, unsigned long long seed, float *logits_host, const std::vector<double> *uni) {
    NCPGen *g = new NCPGen();
    g->m = m; g->B = B;
    g->temp = temp; g->top_k = top_k; g->top_p = top_p; g->cfg_scale = cfg_scale;
    g->freq = freq; g->mu = mu; g->adj_a = adj_a; g->adj_w = adj_w; g->adj_d = adj_d;
    g->seed = seed;
    g->use_cfg = cfg_scale > 0;
    g->Bm = g->use_cfg ? 2 * B : B;
    g->cap_host = logits_host;
    g->uni_given = uni;
    gen_plan(g, l0, prefix_ids, allow);
    while (!ncp_gen_step(g, nullptr, nullptr)) { }
    return ncp_gen_finish(g);
}

// A batch that does not fit the GPU's free memory runs as waves of rows. Rows are independent, so the result is
// the same as one pass; in the reference-stream RNG mode every wave gets exactly the draws its rows would have
// consumed in the full batch (the stream is laid out level by level, row by row), in the counter mode the
// row offset does it. NCM_B200_WAVE_MB overrides the memory budget, NCM_B200_WAVE_ROWS caps the wave size (testing).
int *ncmb_ncp_generate_ex(NCPState *m, const int *l0, const int *prefix_ids, int B,
                          float temp, int top_k, float top_p, float cfg_scale,
                          float freq, float mu, float adj_a, int adj_w, float adj_d,
                          const double *allow, unsigned long long seed, float *logits_host) {
    ensure_device();
    if (B <= 0) fatal("ncp_generate: batch %d", B);
    const NCMConfig *c = &m->cfg;
    const bool use_cfg = cfg_scale > 0;
    if (use_cfg && c->prefix_pad_token_id < 0)
        fatal("classifier-free guidance needs model.prefix_pad_token_id >= 0 (the null prefix is built from it)");
    // A batch no larger than one that already ran in a single pass on the workspace this state still holds fits
    // again: the free-memory query (about a millisecond on this device) is skipped for it.
    const bool known_fit = !getenv("NCM_B200_WAVE_MB") && m->one_pass_rows >= (use_cfg ? 2 * B : B) && m->work.cap >= m->one_pass_cap &&
                           m->one_pass_cap > 0;
    size_t free_b = 0, total_b = 0;
    if (!known_fit) CUDA_CHECK(cudaMemGetInfo(&free_b, &total_b));
    double budget = 0.6 * ((double)free_b + (double)m->work.cap);      // head room for the engines' own scratch and the caller
    if (const char *e = getenv("NCM_B200_WAVE_MB")) budget = atof(e) * 1048576.0;
    int Bw = B;
    if (!known_fit && gen_bytes_bound(m, B, use_cfg, logits_host != nullptr) > budget) {
        int lo = 1, hi = B;                                  // largest wave that fits
        while (lo < hi) { int mid = (lo + hi + 1) / 2; if (gen_bytes_bound(m, mid, use_cfg, logits_host != nullptr) <= budget) lo = mid; else hi = mid - 1; }
        Bw = lo;
    }
    if (const char *e = getenv("NCM_B200_WAVE_ROWS")) { int v = atoi(e); if (v >= 1 && v < Bw) Bw = v; }   // testing: force waves
    if (Bw >= B) {
        int *codes = gen_one(m, l0, prefix_ids, B, temp, top_k, top_p, cfg_scale, freq, mu, adj_a, adj_w, adj_d, allow, seed, logits_host, nullptr);
        if (!logits_host) { m->one_pass_rows = use_cfg ? 2 * B : B; m->one_pass_cap = m->work.cap; }
        return codes;
    }
    if (logits_host) fatal("ncp_generate_ex: logits capture needs the batch in one wave (%d rows fit, %d asked)", Bw, B);

    const int nlev = c->n_qlevels, P = m->P, l0len = c->levels[0];
    int total = 0;
    for (int k = 0; k < nlev; k++) total += c->levels[k];
    const int Bm = use_cfg ? 2 * B : B;
    const bool sample_l0 = !l0 && c->query_level0;
    // the whole batch's stream, then one slice per wave
    std::vector<double> all;
    if (temp > 0 && ctx().rng_mode == 0) {
        size_t nd = (sample_l0 ? (size_t)Bm * l0len : 0);
        for (int k = 1; k < nlev; k++) nd += (size_t)B * c->levels[k];
        all.resize(nd);
        unsigned long long st = seed ? seed : 0x9E3779B97F4A7C15ULL;
        for (size_t i = 0; i < nd; i++) all[i] = (double)(rng_next(&st) >> 11) * (1.0 / 9007199254740992.0);
    }
    int *out = (int *)malloc((size_t)B * total * sizeof(int));
    if (!out) fatal("oom codes");
    const long long row_off0 = ctx().row_offset;
    for (int r0 = 0; r0 < B; r0 += Bw) {
        const int nb = std::min(Bw, B - r0);
        std::vector<double> uni;
        if (!all.empty()) {
            size_t base = 0;
            if (sample_l0) {                                  // level 0: rows 0..Bm-1 of the batch (conditional rows, then unconditional)
                for (int b = 0; b < nb; b++) uni.insert(uni.end(), all.begin() + (size_t)(r0 + b) * l0len, all.begin() + (size_t)(r0 + b + 1) * l0len);
                if (use_cfg)
                    for (int b = 0; b < nb; b++) uni.insert(uni.end(), all.begin() + (size_t)(B + r0 + b) * l0len, all.begin() + (size_t)(B + r0 + b + 1) * l0len);
                base = (size_t)Bm * l0len;
            }
            for (int k = 1; k < nlev; k++) {
                const size_t Lk = c->levels[k];
                uni.insert(uni.end(), all.begin() + base + (size_t)r0 * Lk, all.begin() + base + (size_t)(r0 + nb) * Lk);
                base += (size_t)B * Lk;
            }
        }
        ctx().row_offset = row_off0 + r0;
        int *part = gen_one(m, l0 ? l0 + (size_t)r0 * l0len : nullptr, prefix_ids ? prefix_ids + (size_t)r0 * P : nullptr, nb,
                            temp, top_k, top_p, cfg_scale, freq, mu, adj_a, adj_w, adj_d, allow, seed, nullptr, all.empty() ? nullptr : &uni);
        memcpy(out + (size_t)r0 * total, part, (size_t)nb * total * sizeof(int));
        free(part);
    }
    ctx().row_offset = row_off0;
    return out;
}

int *ncp_generate(NCPState *m, const int *l0, const int *prefix_ids, int B,
                  float temp, int top_k, float top_p, float cfg_scale,
                  float freq, float mu, float adj_a, int adj_w, float adj_d,
                  const double *allow, unsigned long long seed) {
    return ncmb_ncp_generate_ex(m, l0, prefix_ids, B, temp, top_k, top_p, cfg_scale, freq, mu, adj_a, adj_w, adj_d,
                                allow, seed, nullptr);
}

// ------------------------------------------------------------------ teacher-forced forward
// x: [B][P+T][D] (device), logits: [B][T][maxV] (device), unused vocabulary slots -inf
// (reference src/ncp.c:480-647). Block-diagonal pattern: each target level attends to the prefix and to itself,
// one level pass per level over the shared prefix cache. Block-causal pattern: also to every earlier level,
// whose keys and values each layer keeps as the levels are passed in order.
__global__ void k_scatter_logits(const float *__restrict__ lg, float *__restrict__ out, int B, int lk, int V, int T, int off, int maxV) {
    int64_t n = (int64_t)B * lk * V;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int v = (int)(i % V); int t = (int)((i / V) % lk); int b = (int)(i / ((int64_t)V * lk));
        out[((int64_t)b * T + off + t) * maxV + v] = lg[i];
    }
}

void ncp_forward(NCPState *m, const float *x, const int *prefix_ids, float *logits, int B) {
    ensure_device();
    StaticWeights sw;
    const NCMConfig *c = &m->cfg;
    int P = m->P, T = m->T, S = P + T, C = m->C, D = m->D;
    NCPGen *g = new NCPGen();
    g->m = m; g->B = B; g->Bm = B;
    std::vector<int> ids((size_t)B * P, 1);
    if (c->prefix_pad_token_id >= 0 && prefix_ids) memcpy(ids.data(), prefix_ids, ids.size() * 4);
    else if (c->prefix_pad_token_id == 1) for (auto &v : ids) v = 2;
    gen_plan(g, nullptr, ids.data(), nullptr);
    // prefix rows come from x, not from an embedding lookup: token i of row b at position s -> row b*S + s
    {
        std::vector<int> rs(B + 1), pos(g->ntok), src(g->ntok);
        mem_d2h(rs.data(), g->row_start_d, rs.size() * 4);
        mem_d2h(pos.data(), g->tok_pos_d, pos.size() * 4);
        for (int b = 0; b < B; b++) for (int i = rs[b]; i < rs[b + 1]; i++) src[i] = b * S + pos[i];
        upload(g->tok_src_d, src.data(), src.size() * 4);
        float *zpre = g->bufs.h;
        embed_rows(x, g->tok_src_d, zpre, g->ntok, D);
        GemmArgs a;
        a.x = zpre; a.ldx = D; a.W = m->wteW; a.bias = m->wteB; a.y = g->xpre; a.ldy = C; a.M = g->ntok; a.N = C; a.K = D;
        gemm(a);
        if (!c->use_rope) {
            embed_rows(m->wpe, g->tok_pos_d, g->bufs.ctx, g->ntok, C);
            add_inplace(g->xpre, g->bufs.ctx, (int64_t)g->ntok * C);
        }
    }
    prefix_pass(g);
    // block-causal pattern: per-layer K|V of the target tokens, per-row starts and (per level) visible lengths
    const bool causal = !c->attn_pattern_block_diag;
    std::vector<float *> lvlkv;
    int *seq_start_d = nullptr, *len_d = nullptr;
    if (causal) {
        const int kvd = m->nkv * m->hd;
        for (int li = 0; li < m->NL; li++) lvlkv.push_back((float *)dev_alloc((size_t)B * T * 2 * kvd * 4 + 64));
        std::vector<int> st(B + 1);
        for (int b = 0; b <= B; b++) st[b] = b * T;
        seq_start_d = (int *)dev_alloc((size_t)(B + 1) * 4);
        len_d = (int *)dev_alloc((size_t)B * 4 * (m->n_tgt > 0 ? m->n_tgt : 1));
        upload(seq_start_d, st.data(), st.size() * 4);
        std::vector<int> ln((size_t)B * m->n_tgt);
        int o = 0;
        for (int k = 0; k < m->n_tgt; k++) { o += c->levels[k + m->lvl_first]; for (int b = 0; b < B; b++) ln[(size_t)k * B + b] = o; }
        upload(len_d, ln.data(), ln.size() * 4);
        CUDA_CHECK(cudaStreamSynchronize(stream()));
    }
    int maxV = 0;
    for (int k = 0; k < m->n_tgt; k++) if (c->vocab_size[k] > maxV) maxV = c->vocab_size[k];
    fill_f32(logits, -INFINITY, (int64_t)B * T * maxV);
    int off = 0;
    for (int k = 0; k < m->n_tgt; k++) {
        int lk = c->levels[k + m->lvl_first], V = c->vocab_size[k];
        // chunk of x for this level: rows b*S + P + off + t
        NCT xs{(int64_t)S * D, 1, (int64_t)D};
        const float *xc = x + (size_t)(P + off) * D;
        if (c->puc_enabled) {
            int K = c->puc_kernel;
            conv1d(xc, xs, m->pucW[k], m->pucB[k], g->xout, nlc(D, lk), B, D, D, lk, K, 1, K / 2, nullptr, 0.f);
            // xout += chunk (proper, transposed-back residual: src/ncp.c:525-526)
            CUDA_CHECK(cudaMemcpy2DAsync(g->xtmp, (size_t)lk * D * 4, xc, (size_t)S * D * 4, (size_t)lk * D * 4, B, cudaMemcpyDeviceToDevice, stream()));
            add_inplace(g->xtmp, g->xout, (int64_t)B * lk * D);
            CUDA_CHECK(cudaMemcpyAsync(g->xout, g->xtmp, (size_t)B * lk * D * 4, cudaMemcpyDeviceToDevice, stream()));
        } else {
            CUDA_CHECK(cudaMemcpy2DAsync(g->xout, (size_t)lk * D * 4, xc, (size_t)S * D * 4, (size_t)lk * D * 4, B, cudaMemcpyDeviceToDevice, stream()));
        }
        GemmArgs a;
        a.x = g->xout; a.ldx = D; a.W = m->wteW; a.bias = m->wteB; a.y = g->xlev; a.ldy = C; a.M = (int64_t)B * lk; a.N = C; a.K = D;
        gemm(a);
        add_rows_bcast(g->xlev, m->lvl_pos + (size_t)off * C, B, lk * C);
        if (causal) level_pass_causal(g, g->xlev, lk, k, k + m->lvl_first, off, lvlkv, seq_start_d, len_d + (size_t)k * B);
        else level_pass(g, g->xlev, lk, k, k + m->lvl_first);
        int64_t n = (int64_t)B * lk * V;
        int64_t gsz = cdiv(n, 256);
        LAUNCH(k_scatter_logits, (unsigned)(gsz > 4096 ? 4096 : gsz), 256, 0, g->logits, logits, B, lk, V, T, off, maxV);
        off += lk;
    }
    CUDA_CHECK(cudaStreamSynchronize(stream()));
    for (float *p : lvlkv) dev_free(p);
    if (seq_start_d) dev_free(seq_start_d);
    if (len_d) dev_free(len_d);
    delete g;
}

} // extern "C"
