/* ncm_b200.h -- C interface of libncm_b200.so, the B200 (sm_100a) implementation of
 * the cncm token loop.
 *
 * The reference has no plugin or FFI layer: its boundary is the set of C symbols
 * declared in its src/ncm.h.  This header re-declares the inference part of that
 * boundary with identical names, argument order, struct layouts and error
 * behaviour, so a host program written against the reference (its CLI, a cgo or
 * ctypes binding) links against this library unchanged.  Each declaration cites
 * the reference line it replaces.  Entry points that the reference does not have
 * are grouped at the end and prefixed `ncmb_`.
 *
 * Conventions kept from the reference:
 *   - `float *` / `int *` arguments of kernels and model functions are BACKEND
 *     pointers: device memory here (the reference documents Tensor.data as "host
 *     ptr (CPU) or device ptr (CUDA build)", src/ncm.h:30).  ids / codes /
 *     prefixes passed to the model-level functions are host pointers, exactly
 *     where the reference takes host pointers.
 *   - loaders return 0 / -1; everything else prints one line to stderr and
 *     exit(1)s on a fatal error (src/tensor.c:10-12, src/ncp.c:28-32).
 *   - ncp_generate / ncp_gen_finish return malloc'ed int[B][sum(levels)] that the
 *     caller frees.
 *   - not re-entrant: one process-wide scratch arena, one CUDA stream.
 * There is no CPU fallback: every entry point fails loudly without a CUDA device.
 */
#ifndef NCM_B200_H
#define NCM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---------------------------------------------------------------- runtime types
 * Layout-identical to src/ncm.h:27-34, 58-66, 76-137. */
#define NCM_MAX_DIMS 4
#define NCM_MAX_LEVELS 64
#define NCM_MAX_VOCAB_LIST 64

typedef struct {
    float  *data;                    /* device pointer */
    int64_t shape[NCM_MAX_DIMS];
    int     ndim;
    int64_t n;
} Tensor;

typedef struct { char name[256]; Tensor *t; } NamedTensor;
typedef struct { NamedTensor *items; int count; } WeightStore;

typedef struct {
    char task[64];
    int  n_layer, n_head, n_embd, context_length, prefix_len;
    int  bias;
    int  raw_token_prefix, contextual_prefix;
    int  prefix_pad_token_id;
    int  vocab_size[NCM_MAX_VOCAB_LIST];
    int  n_levels_out;
    int  predict_level0, query_level0, l0_autoregressive;
    int  attn_pattern_block_diag;
    int  use_positional_encoding, use_level_encoding;
    int  use_rope, rope_base, use_qk_norm, use_flex_attention;
    double rope_theta;
    int  n_kv_heads;
    int  ctx_enabled, ctx_n_layer, ctx_vocab;
    int  puc_enabled, puc_kernel;
    int  shared_output_head, shared_head_per_level_bias, untied_head_bias;
    int  tie_heads_to_codebook, tie_heads_learn_scale, tie_heads_trainable;
    int  tie_heads_bias;
    int  use_swiglu, use_geglu, use_relu2, parallel_block, normformer;
    int  use_layerscale, use_rezero;
    float layerscale_init;
    float dropout;
    int  vq_embed_dim, vq_in_vocab, vq_context_length, vq_n_layers;
    int  vq_compression;
    int  vq_soft_levels;
    double vq_soft_tau;
    int  levels[NCM_MAX_LEVELS];
    int  n_qlevels;
    int  vq_vocab[NCM_MAX_LEVELS];
    float quant_resi_ratio;
    int   quant_resi_enabled;
    int   quant_resi_share_mode;
    int   learned_l1_sampling, learned_l1_cascade;
    int   learned_l1_cascade_base;
    int   learned_l1_norm, learned_l1_norm_final;
    int   learned_all_sampling;
    int   pre_quant_groupnorm;
    int   vq_qk_norm;
    int   enc_layers, enc_attn_window, enc_conv_layers, enc_conv_kernel;
    int   enc_positional;
    int   dec_layers, dec_positional;
    char pre_tok[16];
    int  sudoku_size;
    char hf_model_id[128];
    int  eos_token_id, pad_token_id;
    float gen_temperature;
    int   gen_top_k;
    float gen_top_p, gen_cfg_scale;
    float gen_freq, gen_mu;
    float gen_adj_a; int gen_adj_w; float gen_adj_d;
} NCMConfig;

/* ---------------------------------------------------------------- runtime
 * src/ncm.h:37-55 (tensor.c:15-62, 274-367) */
Tensor *tensor_alloc(int ndim, const int64_t *shape);
void    tensor_free(Tensor *t);
int64_t tensor_numel(int ndim, const int64_t *shape);
void tensor_to_host(const Tensor *t, float *out);
void tensor_to_backend(Tensor *t, const float *in);
void mem_d2h(void *h, const void *d, size_t n);
void mem_h2d(void *d, const void *h, size_t n);
void mem_d2d(void *d, const void *s, size_t n);
void  arena_init(size_t bytes);
void  arena_init_default(void);              /* NCM_ARENA_MB, else 4096 MB (tensor.c:290) */
float *arena_alloc(size_t n_floats);
void  arena_reset(void);
void  arena_free(void);
void  parena_init(size_t bytes);
float *parena_alloc(size_t n_floats);
/* src/ncm.h:68-70, 139, 261 (tensor.c:70-143, 170-266, 369-373) */
int  weights_load(WeightStore *ws, const char *path);     /* NCM1 / NCM2 weights or NCK1 checkpoints; 0 / -1 */
/* "NCM2" is this library's 2-byte variant of the NCM1 file (the reference's loader, tensor.c:70-128, is fp32-only):
 * same header and records with one byte of element type (0 = fp32, 1 = bf16) in front of each record's u64 byte
 * count. bf16 payloads cross PCIe as 2 bytes per element and are widened on the device, so every tensor is fp32 to
 * its consumers -- exactly what the reference computes from the same values stored as fp32. */
/* src/ncm.h:441, 465 (ckpt.c:67-77, 549-625): which of the two a file is (1 = NCK1 training checkpoint,
 * 0 = NCM1, -1 = neither), and the checkpoint's tensor records alone -- checksum verified first, run state and
 * optimizer section ignored -- so that every inference command accepts a training checkpoint. 0 / -1 with the
 * reason in err. Saving and resuming checkpoints belong to training and are not part of this library. */
int  ckpt_probe(const char *path);
int  ckpt_load_weights_only(const char *path, WeightStore *ws, char *err, size_t errcap);
void weights_free(WeightStore *ws);
Tensor *weights_get(WeightStore *ws, const char *name);   /* NULL if missing */
int  config_load(NCMConfig *c, const char *path);         /* 0 / -1 */
void *backend_to_host(const float *d, size_t nbytes);     /* malloc'ed host copy */
/* src/ncm.h:262-264 (tensor.c:375-397): rows of token ids in an "NCMT" file (magic, u64 row count, u64 row
 * length, int32 ids) -- what the data-preparation commands vq-encode / vq-recon read before they call
 * vqvae_encode_z and vq_z_to_idx. Host memory; max_rows > 0 keeps the first max_rows rows. NULL with a message
 * on a missing file, a wrong magic or a short file. */
typedef struct { int *rows; int n_rows, row_len; } TrainData;
TrainData *train_data_load(const char *path, int max_rows);
void train_data_free(TrainData *d);

/* ---------------------------------------------------------------- layer kernels
 * src/ncm.h:146-199 (kernels.c). fp32 in, fp32 out, out-parameter last. */
void linear_fwd(const float *x, const float *W, const float *b, float *y, int64_t batch, int M, int K);
void embedding_fwd(const float *W, const int *idx, float *y, int64_t n, int D);
void layernorm_fwd(const float *x, const float *w, const float *b, float *y, int64_t rows, int C);
void layernorm_eps_fwd(const float *x, const float *w, const float *b, float *y, int64_t rows, int C, float eps);
void gelu_tanh_fwd(const float *x, float *y, int64_t n);
void rmsnorm_fwd(const float *x, const float *w, float *y, int64_t rows, int C);
void gelu_fwd(const float *x, float *y, int64_t n);
void silu_fwd(const float *x, float *y, int64_t n);
void softmax_fwd(const float *x, float *y, int64_t rows, int C);
void rope_apply(float *q, float *k, const float *cos, const float *sin, int B, int H, int T, int hd);
void rope_apply_gqa(float *q, float *k, const float *cos, const float *sin, int B, int H, int K, int T, int hd);
void heads_transpose_fwd(const float *in, float *out, int64_t T, int H, int hd);
void heads_transpose_fwd_b(const float *in, float *out, int B, int64_t T, int H, int hd);
void sdpa_fwd(const float *q, const float *k, const float *v, const float *mask, float *out,
              int B, int H, int Tq, int Tkv, int hd);
void sdpa_fwd_gqa(const float *q, const float *k, const float *v, const float *mask, float *out,
                  int B, int Hq, int Hkv, int Tq, int Tkv, int hd);
void conv1d_fwd(const float *x, const float *W, const float *b, float *y,
                int N, int Cin, int Cout, int T, int K, int stride, int pad);
void convtranspose1d_fwd(const float *x, const float *W, const float *b, float *y,
                         int N, int Cin, int Cout, int T, int K, int stride);
void groupnorm_fwd(const float *x, float *y, int N, int G, int C, int T);
void interpolate_area_fwd(const float *x, float *y, int N, int C, int Tin, int Tout);
void interpolate_linear_fwd(const float *x, float *y, int N, int C, int Tin, int Tout);
int  argmax_row(const float *x, int n);                   /* x is a HOST row (main.c:854) */
void rowwise_l2sq(const float *a, const float *b, float *d2, int64_t rows, int64_t colsA, int C);
void add_fwd(const float *a, const float *b, float *y, int64_t n);
void scale_fwd(const float *x, float s, float *y, int64_t n);
void mul_fwd(const float *a, const float *b, float *y, int64_t n);
void add_inplace_fwd(float *y, const float *x, int64_t n);
void qkv_split_fwd(const float *in, float *qq, float *kk, float *vv,
                   int B, int T, int C, int H, int hd, int K, int rep);
void head_merge_fwd(const float *ctx, float *out, int B, int T, int C, int H, int hd);
/* host-side sampling helpers, src/ncm.h:197-199 (kernels.c:774-825); logits is a HOST row */
int  sample_topkp(const float *logits, int V, float temp, int top_k, float top_p, unsigned long long *rng);
unsigned long long rng_next(unsigned long long *state);

/* ---------------------------------------------------------------- quantizer
 * src/ncm.h:205-239 (vq.c) */
typedef struct VQState VQState;
VQState *vq_load(const NCMConfig *c, WeightStore *ws, const char *prefix);
void     vq_free(VQState *vq);
int      vq_total_codes(const VQState *vq);
void vq_z_to_idx(VQState *vq, const float *z, int B, int *idx);            /* idx: host */
void vq_idx_to_zhats(VQState *vq, const int *idx, int B, float **zhats);   /* idx: host */
void vq_next_input(VQState *vq, const int *codes, int level_idx, float *z_hat, float *x_out, int B);
void vq_idx_to_ncm_input(VQState *vq, const int *idx, int B, float *x_out);
int vq_nlevels(const VQState *vq);
int vq_level_len(const VQState *vq, int k);
int vq_level_V(const VQState *vq, int k);
int vq_Ltotal(const VQState *vq);
int vq_Ddim(const VQState *vq);

/* ---------------------------------------------------------------- VQ-VAE
 * src/ncm.h:224-247 (vqvae.c) */
typedef struct VQVAEState VQVAEState;
VQVAEState *vqvae_load(const NCMConfig *c, WeightStore *ws);
void        vqvae_free(VQVAEState *v);
VQState    *vqvae_vq(VQVAEState *v);
void vqvae_encode_z(VQVAEState *v, const int *ids, float *z, int B);       /* ids: host */
void vqvae_decode(VQVAEState *v, const float *zhat, float *logits, int B);

/* ---------------------------------------------------------------- NCP
 * src/ncm.h:249-287 (ncp.c) */
typedef struct NCPState NCPState;
NCPState *ncp_load(const NCMConfig *c, WeightStore *ws, VQVAEState *vqvae);
void      ncp_free(NCPState *m);
int   ncp_P(NCPState *m);
int   ncp_T(NCPState *m);
int   ncp_ntgt(NCPState *m);
int   ncp_lvlfirst(NCPState *m);
float *ncp_rope_cos(NCPState *m);
float *ncp_rope_sin(NCPState *m);
float *ncp_rope_gen_cos(NCPState *m, int k);
float *ncp_rope_gen_sin(NCPState *m, int k);
VQState *ncp_vq(NCPState *m);
void ncp_forward(NCPState *m, const float *x, const int *prefix_ids, float *logits, int B);
int *ncp_generate(NCPState *m, const int *l0, const int *prefix_ids, int B,
                  float temp, int top_k, float top_p, float cfg_scale,
                  float freq, float mu, float adj_a, int adj_w, float adj_d,
                  const double *allow, unsigned long long seed);
typedef struct NCPGen NCPGen;
NCPGen *ncp_gen_begin(NCPState *m, const int *l0, const int *prefix_ids, int B,
                      float temp, int top_k, float top_p, float cfg_scale,
                      float freq, float mu, float adj_a, int adj_w, float adj_d,
                      const double *allow, unsigned long long seed);
int ncp_gen_step(NCPGen *g, int *codes_out, int *n_out);   /* 0 = ran a level, 1 = done */
int *ncp_gen_finish(NCPGen *g);
void ncp_gen_abort(NCPGen *g);
int ncp_gen_nsteps(NCPGen *g);
int ncp_gen_step_size(NCPGen *g, int s);

/* ---------------------------------------------------------------- decoder LMs
 * src/ncm.h:315-317, 326-328 (gpt2.c:204-235, qwen.c:233-264): load, generate,
 * print "ids: ..." then the decoded text. Text needs the host tokenizer
 * (tok_load / tok_decode, src/ncm.h:294-303); when those symbols are not linked
 * in, only the ids line is printed. */
int gpt2_cmd_gen(const NCMConfig *c, const char *weights, const char *adir,
                 const char *prompt, const char *ids_csv, int n_new,
                 float temp, int top_k, float top_p, unsigned long long seed);
int qwen_cmd_gen(const NCMConfig *c, const char *weights, const char *adir,
                 const char *prompt, const char *ids_csv, int n_new,
                 float temp, int top_k, float top_p, unsigned long long seed);
/* src/ncm.h:318-321, 329-332. *_cmd_ppl (gpt2.c:237-270, qwen.c:266-297): one document per line of texts_path,
 * non-overlapping windows (n_ctx ids for GPT-2, 512 for Qwen2), prints
 * "docs=%d tokens=%ld nll=%.6f ppl=%.6f". *_cmd_verify (gpt2.c:417-485, qwen.c:386-478): checks
 * <stem>_tok.txt / <stem>_logits_<name>.f32 / <stem>_gen.txt / <stem>_ppl.txt of fixtures_dir with the
 * reference's bounds and prints its "ok" / "FAIL" lines and "<STEM>-VERIFY PASS|FAIL (n checked)"; returns 1 on a
 * failure. Without the host tokenizer linked in, a texts line is read as white-space separated token ids and
 * the fixture checks that need text print "skip ..." (the logits check uses the fixture's ids and always runs). */
int gpt2_cmd_ppl(const NCMConfig *c, const char *weights, const char *adir, const char *texts_path);
int gpt2_cmd_verify(const NCMConfig *c, const char *weights, const char *adir, const char *fixtures_dir);
int qwen_cmd_ppl(const NCMConfig *c, const char *weights, const char *adir, const char *texts_path);
int qwen_cmd_verify(const NCMConfig *c, const char *weights, const char *adir, const char *fixtures_dir);

/* ================================================================ additions
 * Entry points with no counterpart in the reference. */

/* Library / device control. ncmb_set_stream makes every later launch and copy
 * use the given cudaStream_t (default: the legacy default stream). */
const char *ncmb_version(void);
void  ncmb_set_stream(void *cuda_stream);
void *ncmb_get_stream(void);
void  ncmb_sync(void);
/* GEMM engine: 0 = fp32 CUDA cores, 1 = tcgen05 TF32 single pass,
 * 2 = tcgen05 3xTF32 (fp32-grade), 3 = tcgen05 fp16 pairs: every operand is carried as
 * v1 + v2 in fp16 behind a power-of-two factor and the product takes three fp16 MMAs into
 * one fp32 accumulator (fp32-grade, twice the MMA rate of 2; activations beyond +-4094
 * saturate). Default from NCM_B200_GEMM, else 3. */
void  ncmb_set_gemm_mode(int mode);
int   ncmb_get_gemm_mode(void);
/* The tensor-core kernels bound every barrier wait; when one runs out they record a
 * code and drain. Returns and clears that code (0 = never happened); synchronises. */
int   ncmb_gemm_tc_check(void);
/* Entries the TMA descriptor caches keep before they start over (default 4096; diagnostic: tests
 * set 1 so that every lookup evicts the one before it). No counterpart in the reference. */
void  ncmb_set_map_cache_limit(int entries);
/* Diagnostic: the transformer blocks' token-major attention (head dim 64) on caller-supplied DEVICE
 * buffers, with engine 0 (CUDA-core kernel), 1 (tcgen05 kernel) or 2 (split-key decode kernel, one query
 * per row, one key segment), so they can be compared on the same
 * inputs. q [q_total][H*64]; kv1 / kv2 [tokens][2*Hkv*64] (keys, then values); *_start are HOST
 * int[rows+1] prefix offsets, k2_start NULL for one key segment. Returns 0, -1 when the tensor-core
 * engine does not take the shape, else the timeout code. No counterpart in the reference. */
int   ncmb_attention_check(const float *q, const float *kv1, const float *kv2, float *out,
                           const int *q_start, const int *k1_start, const int *k2_start,
                           int rows, int H, int Hkv, int causal, int window, int engine);
/* Sampling stream: 0 = the reference's single xorshift64* stream consumed in
 * (level, row, position) order (src/ncp.c:660-705) -- sampled codes equal the
 * reference's; 1 = counter-based, keyed by (seed, row_offset + row, level,
 * position), independent of batch size and sharding. Default 0. */
void  ncmb_set_rng_mode(int mode);
/* Global index of row 0 of the next generate call (counter-based stream only);
 * lets a batch be sharded over processes without changing any row's draws. */
void  ncmb_set_row_offset(long long row_offset);
/* Kernel-class timing with CUDA events on the launch stream. ncmb_prof_enable(1)
 * starts collecting; ncmb_prof_read synchronises and returns, per class, the
 * launch count, total milliseconds and algorithmic FLOPs and bytes. */
enum { NCMB_K_GEMM = 0, NCMB_K_ATTN = 1, NCMB_K_NORM = 2, NCMB_K_SAMPLE = 3,
       NCMB_K_ELEM = 4, NCMB_K_VQ = 5, NCMB_K_COUNT = 6 };
void  ncmb_prof_enable(int on);
void  ncmb_prof_reset(void);
/* The profiler also keeps one entry per distinct call shape (class, flops, bytes of one call).
 * ncmb_prof_top_shape: the shape of class `klass` with the largest total time since the last reset
 * (launch count, total ms, flops and bytes of ONE call); -1 when the class recorded nothing.
 * ncmb_prof_dump_shapes: prints the whole table to stderr, largest total first, and clears it. */
int   ncmb_prof_top_shape(int klass, long long *launches, double *ms, double *flops, double *bytes);
void  ncmb_prof_dump_shapes(void);
int   ncmb_prof_read(int klass, long long *launches, double *ms, double *flops, double *bytes);
long long ncmb_launch_count(void);            /* kernels launched since load */
/* The GEMM engines keep converted copies (fp16 pairs, TF32 hi/lo) of weight matrices, keyed by the matrix's device
 * address. weights_free, tensor_free, mem_h2d, mem_d2d and tensor_to_backend drop the copies of the memory they touch;
 * a caller that rewrites weight memory by other means (its own kernels, cudaMemcpy) calls this before the next
 * forward. No counterpart in the reference. */
void  ncmb_forget_weight_copies(void);
/* 1 when the store came from an "NCM2" file whose matrices are all 2-byte (bf16) records: ncmb_lm_open then streams
 * exact 2-byte copies in its decode steps without being told. No counterpart in the reference. */
int   ncmb_weights_are_bf16(const WeightStore *ws);
/* free and total bytes of the current device's memory (cudaMemGetInfo) */
void  ncmb_mem_info(unsigned long long *free_bytes, unsigned long long *total_bytes);
/* bytes this library has copied host->device and device->host since load */
void  ncmb_copy_bytes(unsigned long long *h2d, unsigned long long *d2h);

/* linear_fwd (three-pass TF32) that allocates no memory at all -- no counterpart in the
 * reference. For callers that may not allocate on the device: loops with a memory budget
 * fixed at start-up, host callbacks and stream-capture regions (where cudaMalloc is not
 * legal), or steady-state serving code that must not stall or fail on an allocation. Scratch
 * for the split operands (2*batch*K + 2*M*K floats) comes from a 32 MiB array built into the
 * library; larger problems, or shapes outside batch > 16, M >= 32, K >= 32, K % 4 == 0 with
 * 16-byte aligned pointers, return -1 with a message (0 = kernels queued). The first call on a
 * device resolves the array's address: make it before any stream capture. Calls share the
 * array, so calls that overlap on one GPU race; keep them ordered on one stream. A call made
 * with a device current other than the one the library first ran on is refused (-1).
 * The kernels bound every barrier wait; whether one ran out is known only after
 * ncmb_linear_fwd_noalloc_check(): it synchronises the stream, then returns and clears this
 * entry point's own status word (0 = all calls completed, -1 = never set up on this device).
 * It allocates nothing either. */
int ncmb_linear_fwd_noalloc(const float *x, const float *W, const float *b, float *y,
                            int64_t batch, int M, int K);
int ncmb_linear_fwd_noalloc_check(void);

/* Diagnostic: the device sampler on caller-supplied DEVICE rows (one position per row, no CFG, no penalties):
 * sample_topkp's rule (src/kernels.c:794-825) with row b's uniform taken from uniforms[b] (device doubles in
 * [0, 1)); picks is a device int[B]. Lets tests feed crafted rows (ties, constant rows) to the selection-based and
 * the sort-based nucleus paths. Synchronises. No counterpart in the reference. */
void ncmb_sample_rows_dev(const float *logits, int B, int V, float temp, int top_k, float top_p,
                          const double *uniforms, int *picks);

/* NCP generate, extended: same as ncp_generate, and when logits_host is not NULL
 * it receives the logits each sampled position was drawn from (after the CFG
 * blend, before penalties), per sampled row, level-major. */
int *ncmb_ncp_generate_ex(NCPState *m, const int *l0, const int *prefix_ids, int B,
                          float temp, int top_k, float top_p, float cfg_scale,
                          float freq, float mu, float adj_a, int adj_w, float adj_d,
                          const double *allow, unsigned long long seed, float *logits_host);
/* codes[B][sum levels] (host) -> token ids[B][L] (host): cumulative z_hat, VQ-VAE
 * decoder, per-position argmax on the device (the device form of the reference
 * CLI's decode_boards, src/main.c:863-879, without the text step). */
void ncmb_decode_tokens(VQVAEState *v, const int *codes, int B, int *tokens);
/* Device-resident variants for callers whose data already lives in HBM: the codes
 * of a running generate (valid after the last ncp_gen_step, until finish / abort),
 * and decoding from device codes to device token ids; nothing crosses PCIe. */
const int *ncmb_gen_codes_dev(NCPGen *g);
void ncmb_decode_tokens_dev(VQVAEState *v, const int *codes_dev, int B, int *tokens_dev);
/* Standalone residual-quantizer encode on device-resident vectors, argmin fused
 * into the distance computation: z [B][L][D] (device) -> idx [B][sum levels] (device). */
void ncmb_vq_encode_dev(VQState *vq, const float *z_dev, int B, int *idx_dev);
/* Flat nearest-code search: x [n][D] against codebook level k -> idx [n] (device). */
void ncmb_vq_nearest_dev(VQState *vq, int level, const float *x_dev, long long n, int *idx_dev);

/* Batched GPT-2 / Qwen2 decoding with a KV cache. The reference decodes one
 * prompt per process and recomputes the whole context per token
 * (gpt2.c:179-202, qwen.c:209-231); results here equal B independent runs of it.
 * bf16_weights != 0: the file holds values already rounded to bf16 (stored as fp32, which is how the
 * fp32-only reference consumes them); every projection matrix whose elements all are bf16 values gets an
 * exact 2-byte copy that decode steps stream instead of the fp32 one -- same results, half the bytes. */
typedef struct NcmbLM NcmbLM;
NcmbLM *ncmb_lm_open(const NCMConfig *c, const char *weights, int is_qwen, int bf16_weights);   /* weights: .ncm, .nckpt or .safetensors */
void   ncmb_lm_close(NcmbLM *m);
int    ncmb_lm_vocab(const NcmbLM *m);
/* Decode steps of up to four sequences (head dim 64) can run as ONE persistent cooperative kernel with grid
 * barriers between the phases of a layer instead of a replayed chain of kernels. Off by default (it is the
 * slower of the two today); results are the same either way. No counterpart in the reference. */
void  ncmb_set_lm_persistent(int on);
/* prompts: host int[B][np]; out: host int[B][n_new]; eos < 0 disables stopping.
 * Returns the number of ids generated per row (n_new unless every row hit eos). */
int    ncmb_lm_generate(NcmbLM *m, const int *prompts, int B, int np, int n_new,
                        float temp, int top_k, float top_p, unsigned long long seed,
                        int eos, int *out);
/* logits of one sequence: all positions ([T][V]) or the last one ([V]) to host */
void   ncmb_lm_logits(NcmbLM *m, const int *ids, int T, int last_only, float *out_host);
/* A Hugging Face .safetensors file straight into a WeightStore on the device, with the tensor rules of the
 * reference's offline converters (tools/gpt2import.c:385-417, tools/qwenimport.c:383-420, which write an NCM1
 * file instead): F16 / BF16 widened to fp32, "*.attn.bias" mask buffers dropped, names and order kept, and with
 * conv1d_transpose != 0 (GPT-2) the 2-D c_attn / c_proj / c_fc weights transposed from [in][out] to [out][in].
 * 0 / -1. ncmb_lm_open takes such a path too. Tokenizer assets stay with the reference's tools (host text). */
int    ncmb_weights_import_safetensors(WeightStore *ws, const char *path, int conv1d_transpose);
/* Mean next-token negative log-likelihood of B windows (gpt2_nll gpt2.c:160-176, qwen_nll qwen.c:192-208, which
 * take one window and read the [T][V] logits on the host). ids: host int[B][T]; lens: host int[B] ids used per
 * window (NULL = T); nll_out: host double[B], the mean over lens[b] - 1 positions of
 * -log(exp(l[next] - max) / sum exp(l - max) + 1e-30) in fp64. Logits never leave the device. */
void   ncmb_lm_nll(NcmbLM *m, const int *ids, int B, int T, const int *lens, double *nll_out);

#ifdef __cplusplus
}
#endif
#endif /* NCM_B200_H */
