/* CPU oracle for the token-loop hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the reference's CPU algorithm (fp32 storage, fp64
 * accumulation, first-index-wins ties) for: the layer kernels, the multiscale
 * residual quantizer, the VQ-VAE encoder/decoder, the NCP coarse-to-fine
 * generate and the GPT-2 / Qwen2 decode loops.  It exists so that parity tests
 * and the benchmark's CPU-baseline leg have a checker that travels with the
 * repository.  The shipped library never links, loads or calls it.
 *
 * Parity pin: tests/test_oracle_pin.py checks every function here bit-for-bit
 * against the reference's own CPU build (oracle/_ref, built by `make ref`) when
 * that build is present, and against golden vectors generated from it
 * (tests/golden/, generator script beside them) everywhere else.
 *
 * All pointers are host memory.  Each function names the reference file:line it
 * follows in oracle.c.
 */
#ifndef ORACLE_H
#define ORACLE_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- layer kernels (reference src/kernels.c) ---- */
void orc_linear(const float *x, const float *W, const float *b, float *y,
                int64_t batch, int M, int K);
void orc_layernorm(const float *x, const float *w, const float *b, float *y,
                   int64_t rows, int C, double eps);
void orc_rmsnorm(const float *x, const float *w, float *y, int64_t rows, int C);
void orc_gelu(const float *x, float *y, int64_t n);
void orc_gelu_tanh(const float *x, float *y, int64_t n);
void orc_silu(const float *x, float *y, int64_t n);
void orc_softmax(const float *x, float *y, int64_t rows, int C);
void orc_rope(float *x, const float *cs, const float *sn, int64_t rows, int T, int hd);
void orc_sdpa(const float *q, const float *k, const float *v, const float *mask,
              float *out, int B, int Hq, int Hkv, int Tq, int Tkv, int hd);
void orc_conv1d(const float *x, const float *W, const float *b, float *y,
                int N, int Cin, int Cout, int T, int K, int stride, int pad);
void orc_convT1d(const float *x, const float *W, const float *b, float *y,
                 int N, int Cin, int Cout, int T, int K, int stride);
void orc_groupnorm(const float *x, float *y, int N, int G, int C, int T);
void orc_interp_area(const float *x, float *y, int N, int C, int Tin, int Tout);
void orc_interp_linear(const float *x, float *y, int N, int C, int Tin, int Tout);
void orc_l2sq(const float *a, const float *b, float *d2, int64_t rows, int64_t cols, int C);
int  orc_argmax(const float *x, int n);
uint64_t orc_rng_next(uint64_t *state);
int  orc_sample_topkp(const float *logits, int V, float temp, int top_k, float top_p,
                      uint64_t *rng);

/* ---- NCP + VQ-VAE model ---- */
typedef struct OrcModel OrcModel;
OrcModel *orc_model_load(const char *conf_path, const char *weights_path);
void orc_model_free(OrcModel *m);
int  orc_total_codes(const OrcModel *m);
int  orc_L(const OrcModel *m);
int  orc_D(const OrcModel *m);
int  orc_in_vocab(const OrcModel *m);

/* Quantizer (reference src/vq.c).  z, zhat: [B][L][D]; idx: [B][sum levels]. */
void orc_vq_z_to_idx(OrcModel *m, const float *z, int B, int *idx);
/* zhats: n_levels arrays of [B][L][D] (cumulative reconstruction per level) */
void orc_vq_idx_to_zhats(OrcModel *m, const int *idx, int B, float **zhats);
void orc_vq_next_input(OrcModel *m, const int *codes, int level, float *z_hat,
                       float *x_out, int B);
void orc_vq_idx_to_ncm_input(OrcModel *m, const int *idx, int B, float *x_out);
/* VQ-VAE (reference src/vqvae.c).  ids: [B][L]; logits: [B][L][in_vocab]. */
void orc_vqvae_encode(OrcModel *m, const int *ids, float *z, int B);
void orc_vqvae_decode(OrcModel *m, const float *zhat, float *logits, int B);
/* codes -> final z_hat -> decoder -> per-position argmax (reference
 * src/main.c:863-879, without the text step). tokens: [B][L]. */
void orc_decode_tokens(OrcModel *m, const int *codes, int B, int *tokens);

/* Coarse-to-fine generate (reference src/ncp.c:730-1208).  codes: [B][sum levels].
 * logits_cap, when not NULL, receives the logits each sampled position was
 * drawn from (after the CFG blend, before penalties), level-major per row:
 * row b at offset b*sum_k(L_k*V_k) — only the first B (sampled) rows; level 0 is
 * included when the model generates it. */
void orc_ncp_generate(OrcModel *m, const int *l0, const int *prefix, int B,
                      float temp, int top_k, float top_p, float cfg_scale,
                      float freq, float mu, float adj_a, int adj_w, float adj_d,
                      const double *allow, uint64_t seed, int *codes, float *logits_cap);
/* Teacher-forced forward (reference src/ncp.c:480-647). x: [B][P+T][D];
 * logits: [B][T][maxV], unused vocabulary slots -inf. */
void orc_ncp_forward(OrcModel *m, const float *x, const int *prefix, float *logits, int B);
int  orc_ncp_T(const OrcModel *m);
int  orc_ncp_maxV(const OrcModel *m);

/* ---- GPT-2 / Qwen2 decoders (reference src/gpt2.c, src/qwen.c) ---- */
typedef struct OrcLM OrcLM;
OrcLM *orc_lm_load(const char *conf_path, const char *weights_path, int is_qwen);
void orc_lm_free(OrcLM *m);
int  orc_lm_vocab(const OrcLM *m);
/* Full recompute over ids[0..T): logits of every position ([T][V]) or, with
 * last_only, of the last one ([V]). */
void orc_lm_logits(OrcLM *m, const int *ids, int T, int last_only, float *out);
/* Token loop without a KV cache, exactly as the reference runs it. Returns the
 * number of ids written to out. eos < 0 disables the stop test. */
int  orc_lm_generate(OrcLM *m, const int *prompt, int np, int n_new, float temp,
                     int top_k, float top_p, uint64_t seed, int eos, int *out);

#ifdef __cplusplus
}
#endif
#endif
