// VQ-VAE encoder / decoder on the device (reference src/vqvae.c) and the device
// form of the reference CLI's decode step (codes -> z_hat -> decoder -> argmax,
// src/main.c:863-879).
#include "common.cuh"
#include "vq.cuh"
#include "vqvae.cuh"

namespace ncmb {

BlockWeights vae_block_weights(WeightStore *ws, const char *pre, int qk_norm) {
    BlockWeights w;
    w.norm = NORM_LAYER; w.eps = 1e-6f;
    Tensor *t;
    w.ln1w = wneed(ws, "%sln_1.weight", pre)->data;
    w.ln1b = (t = wget(ws, "%sln_1.bias", pre)) ? t->data : nullptr;
    w.qkvw = wneed(ws, "%sattn.c_attn.weight", pre)->data;
    w.qkvb = (t = wget(ws, "%sattn.c_attn.bias", pre)) ? t->data : nullptr;
    w.ow = wneed(ws, "%sattn.c_proj.weight", pre)->data;
    w.ob = (t = wget(ws, "%sattn.c_proj.bias", pre)) ? t->data : nullptr;
    if (qk_norm) {
        w.qnw = wneed(ws, "%sattn.q_norm.weight", pre)->data;
        w.knw = wneed(ws, "%sattn.k_norm.weight", pre)->data;
    }
    w.ln2w = wneed(ws, "%sln_2.weight", pre)->data;
    w.ln2b = (t = wget(ws, "%sln_2.bias", pre)) ? t->data : nullptr;
    Tensor *fc = wneed(ws, "%smlp.c_fc.weight", pre);
    w.fcw = fc->data; w.Hh = (int)fc->shape[0];
    w.fcb = (t = wget(ws, "%smlp.c_fc.bias", pre)) ? t->data : nullptr;
    w.pw = wneed(ws, "%smlp.c_proj.weight", pre)->data;
    w.pb = (t = wget(ws, "%smlp.c_proj.bias", pre)) ? t->data : nullptr;
    w.gated = 0; w.act = ACT_GELU;
    return w;
}

// row starts 0, T, 2T, ... for B uniform sequences (device, cached per (B, T))
const int *uniform_starts(VQVAEState *v, int B, int T) {
    if (v->starts_B != B || v->starts_T != T) {
        v->starts_ws.reserve((size_t)(B + 1) * sizeof(int) + 256);
        v->starts_ws.reset();
        int *d = v->starts_ws.get<int>(B + 1);
        int *h = (int *)malloc((size_t)(B + 1) * sizeof(int));
        for (int i = 0; i <= B; i++) h[i] = i * T;
        upload(d, h, (size_t)(B + 1) * sizeof(int));
        free(h);
        v->starts = d; v->starts_B = B; v->starts_T = T;
    }
    return v->starts;
}

static BlockBufs vae_bufs(Workspace &w, int64_t ntok, int C, int Hh) {
    BlockBufs b;
    b.ln = w.get<float>(ntok * C);
    b.qkv = w.get<float>(ntok * 3 * C);
    b.ctx = w.get<float>(ntok * C);
    b.mlp = nullptr;
    b.h = w.get<float>(ntok * Hh);
    return b;
}

static void vae_run_block(VQVAEState *v, const BlockWeights &w, float *x, int B, int T, int window, const BlockBufs &bufs) {
    int D = v->cfg.vq_embed_dim, H = v->cfg.vq_n_layers;      // vq.n_layers is the head count (vqvae.c:321)
    AttnPlan p;
    p.q_start = p.k1_start = uniform_starts(v, B, T);
    p.rows = B; p.max_q = T; p.window = window;
    p.total_q = (int64_t)B * T; p.avg_keys = T;
    run_block(x, (int64_t)B * T, D, H, H, w, bufs, p);
}

// zhat [B][T][D] (device) -> logits [B][T][V] (device). reference src/vqvae.c:422-470
void vqvae_decode_dev(VQVAEState *v, const float *zhat, float *logits, int B) {
    StaticWeights sw;
    const NCMConfig *c = &v->cfg;
    int T = c->vq_context_length, D = c->vq_embed_dim, V = c->vq_in_vocab;
    if (c->vq_compression > 1) { fprintf(stderr, "decoder upsampling (compression>1) not wired\n"); exit(1); }
    int64_t n = (int64_t)B * T;
    int Hh = v->dec.empty() ? 4 * D : v->dec[0].Hh;
    v->work.reserve((size_t)(n * D * 6 + n * Hh + 4096) * sizeof(float));
    v->work.reset();
    float *x = v->work.get<float>(n * D);
    BlockBufs bufs = vae_bufs(v->work, n, D, Hh);
    CUDA_CHECK(cudaMemcpyAsync(x, zhat, (size_t)n * D * 4, cudaMemcpyDeviceToDevice, stream()));
    if (c->dec_positional) add_rows_bcast(x, v->dec_wpe, B, T * D);
    for (auto &w : v->dec) vae_run_block(v, w, x, B, T, 0, bufs);
    layernorm(x, v->dec_lnf, nullptr, bufs.ln, n, D, 1e-6f);
    GemmArgs g;
    g.x = bufs.ln; g.ldx = D; g.W = v->dec_out; g.y = logits; g.ldy = V; g.M = n; g.N = V; g.K = D;
    gemm(g);
}

// codes (device) -> tokens (device)
void decode_tokens_dev(VQVAEState *v, const int *codes_dev, int B, int *tokens_dev) {
    VQState *vq = v->vq;
    int L = vq->L, D = vq->D, Vp = v->cfg.vq_in_vocab;
    size_t n = (size_t)B * L * D;
    v->dec_ws.reserve((6 * n + (size_t)B * L * Vp + 4096) * sizeof(float));
    v->dec_ws.reset();
    float *scr = v->dec_ws.get<float>(5 * n);
    float *zh = v->dec_ws.get<float>(n);
    float *lg = v->dec_ws.get<float>((size_t)B * L * Vp);
    vq_zhat_final_dev(vq, codes_dev, B, zh, nullptr, scr);
    vqvae_decode_dev(v, zh, lg, B);
    argmax_rows(lg, (int64_t)B * L, Vp, tokens_dev);
}

} // namespace ncmb

using namespace ncmb;

extern "C" {

VQVAEState *vqvae_load(const NCMConfig *c, WeightStore *ws) {
    ensure_device();
    VQVAEState *v = new VQVAEState();
    v->cfg = *c;
    v->ws = ws;
    v->vq = vq_load(c, ws, "tok.vq.");
    // decoder (always needed on the generate path)
    if (wget(ws, "tok.decoder.middle_block.ln_1.weight")) {
        v->dec.push_back(vae_block_weights(ws, "tok.decoder.middle_block.", c->vq_qk_norm));
        for (int i = 0; i < c->dec_layers - 1; i++) {
            char pre[96];
            snprintf(pre, sizeof pre, "tok.decoder.extra_blocks.%d.", i);
            v->dec.push_back(vae_block_weights(ws, pre, c->vq_qk_norm));
        }
        v->dec_lnf = wneed(ws, "tok.decoder.ln_f.weight")->data;
        v->dec_out = wneed(ws, "tok.decoder.output_layer.weight")->data;
        if (c->dec_positional) v->dec_wpe = wneed(ws, "tok.decoder.wpe.weight")->data;
    }
    // encoder (optional: absent from generate-only weight files)
    Tensor *t = wget(ws, "tok.encoder.wte.weight");
    v->enc_wte = t ? t->data : nullptr;
    if (c->enc_positional && (t = wget(ws, "tok.encoder.wpe.weight"))) v->enc_wpe = t->data;
    bool enc_ok = true;
    for (int i = 0; i < c->enc_layers && enc_ok; i++) {
        char pre[96];
        snprintf(pre, sizeof pre, "tok.encoder.blocks.%d.", i);
        if (!wget(ws, "%sln_1.weight", pre)) { enc_ok = false; break; }
        v->enc.push_back(vae_block_weights(ws, pre, c->vq_qk_norm));
    }
    v->enc_ready = enc_ok && v->enc_wte;
    return v;
}

void vqvae_free(VQVAEState *v) {
    if (!v) return;
    vq_free(v->vq);
    v->work.release(); v->dec_ws.release(); v->starts_ws.release();
    delete v;
}

VQState *vqvae_vq(VQVAEState *v) { return v->vq; }

void vqvae_decode(VQVAEState *v, const float *zhat, float *logits, int B) {
    if (v->dec.empty()) { fprintf(stderr, "missing weight tok.decoder.middle_block.ln_1.weight\n"); exit(1); }
    vqvae_decode_dev(v, zhat, logits, B);
}

// ids (host) -> z [B][T][D] (device). reference src/vqvae.c:228-420
void vqvae_encode_z(VQVAEState *v, const int *ids, float *z, int B) {
    const NCMConfig *c = &v->cfg;
    WeightStore *ws = v->ws;
    if (!v->enc_ready) { fprintf(stderr, "missing weight tok.encoder.*\n"); exit(1); }
    StaticWeights sw;
    int T = c->vq_context_length, D = c->vq_embed_dim;
    int64_t n = (int64_t)B * T;
    int Hh = v->enc.empty() ? 4 * D : v->enc[0].Hh;
    v->work.reserve((size_t)(n * D * 9 + n * Hh + n + 4096) * sizeof(float));
    v->work.reset();
    int *ids_dev = v->work.get<int>(n);
    float *x = v->work.get<float>(n * D);
    float *t1 = v->work.get<float>(n * D), *t2 = v->work.get<float>(n * D);
    BlockBufs bufs = vae_bufs(v->work, n, D, Hh);
    upload(ids_dev, ids, (size_t)n * sizeof(int));
    embed_rows(v->enc_wte, ids_dev, x, n, D);
    if (c->enc_positional) add_rows_bcast(x, v->enc_wpe, B, T * D);
    for (int i = 0; i < c->enc_conv_layers; i++) {
        char pre[96];
        snprintf(pre, sizeof pre, "tok.encoder.conv_blocks.%d.", i);
        int K = c->enc_conv_kernel;
        layernorm(x, wneed(ws, "%sln.weight", pre)->data, nullptr, bufs.ln, n, D, 1e-6f);
        conv1d(bufs.ln, nlc(D, T), wneed(ws, "%sc1.weight", pre)->data, wneed(ws, "%sc1.bias", pre)->data,
               t1, nlc(D, T), B, D, D, T, K, 1, K / 2, nullptr, 0.f);
        act_inplace(t1, n * D, ACT_GELU);
        conv1d(t1, nlc(D, T), wneed(ws, "%sc2.weight", pre)->data, wneed(ws, "%sc2.bias", pre)->data,
               t2, nlc(D, T), B, D, D, T, K, 1, K / 2, x, 0.f);          // t2 = x + conv
        CUDA_CHECK(cudaMemcpyAsync(x, t2, (size_t)n * D * 4, cudaMemcpyDeviceToDevice, stream()));
    }
    for (auto &w : v->enc) vae_run_block(v, w, x, B, T, c->enc_attn_window, bufs);
    const float *cur = x;
    if (c->enc_layers > 0 || c->enc_conv_layers > 0) {
        layernorm(x, wneed(ws, "tok.encoder.ln_e.weight")->data, nullptr, t1, n, D, 1e-6f);
        cur = t1;
    }
    if (c->vq_compression > 1) {
        int f = c->vq_compression, T2 = T / f;
        conv1d(cur, nlc(D, T), wneed(ws, "tok.encoder.down.weight")->data, wneed(ws, "tok.encoder.down.bias")->data,
               z, nlc(D, T2), B, D, D, T, f, f, 0, nullptr, 0.f);
        return;
    }
    if (c->pre_quant_groupnorm > 0) groupnorm(cur, nlc(D, T), z, nlc(D, T), B, c->pre_quant_groupnorm, D, T);
    else CUDA_CHECK(cudaMemcpyAsync(z, cur, (size_t)n * D * 4, cudaMemcpyDeviceToDevice, stream()));
}

void ncmb_decode_tokens_dev(VQVAEState *v, const int *codes_dev, int B, int *tokens_dev) {
    decode_tokens_dev(v, codes_dev, B, tokens_dev);
}

void ncmb_decode_tokens(VQVAEState *v, const int *codes, int B, int *tokens) {
    VQState *vq = v->vq;
    int total = vq_total_codes(vq), L = vq->L;
    int *cd = vq_codes_to_dev(vq, codes, (size_t)B * total);
    v->tok_ws.reserve((size_t)B * L * sizeof(int) + 256);
    v->tok_ws.reset();
    int *td = v->tok_ws.get<int>((size_t)B * L);
    decode_tokens_dev(v, cd, B, td);
    mem_d2h(tokens, td, (size_t)B * L * sizeof(int));
}

} // extern "C"
