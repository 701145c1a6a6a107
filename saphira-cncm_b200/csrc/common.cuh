// Internal declarations shared by the translation units of libncm_b200.so.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>
#include <vector>

#include "../../include/ncm_b200.h"

namespace ncmb {

[[noreturn]] void fatal(const char *fmt, ...);

#define CUDA_CHECK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) \
    ::ncmb::fatal("cuda: %s:%d %s", __FILE__, __LINE__, cudaGetErrorString(e_)); } while (0)

// ---- process-wide context: one stream, launch counter, kernel-class timers ----
struct Ctx {
    cudaStream_t stream = 0;
    long long launches = 0;
    int gemm_mode = 3;                  // 0 fp32 CUDA cores | 1 TF32 | 2 3xTF32 | 3 fp16 pairs, three fp16 MMAs (default)
    int rng_mode = 0;
    long long row_offset = 0;
    int sm_count = 148;
    int device = -1;                  // the device ensure_device() found current; the library's caches belong to it
    int w_static = 0;                 // > 0: GEMM weights are model weights that do not change (split copies may be cached)
    unsigned long long h2d_bytes = 0, d2h_bytes = 0;   // bytes moved across PCIe by this library
    bool inited = false;
};
Ctx &ctx();
void ensure_device();            // fails loudly when no CUDA device is present
inline cudaStream_t stream() { return ctx().stream; }

void prof_begin(int klass, double flops, double bytes);
void prof_end();
bool prof_enabled();
struct ProfScope {
    ProfScope(int klass, double flops = 0, double bytes = 0) { prof_begin(klass, flops, bytes); }
    ~ProfScope() { prof_end(); }
};

// every kernel launch goes through this: counts it and surfaces launch errors
#define LAUNCH(kernel, grid, block, smem, ...) do { \
    kernel<<<(grid), (block), (smem), ::ncmb::stream()>>>(__VA_ARGS__); \
    ::ncmb::ctx().launches++; \
    cudaError_t le_ = cudaGetLastError(); \
    if (le_ != cudaSuccess) ::ncmb::fatal("launch %s failed: %s (%s:%d)", #kernel, \
        cudaGetErrorString(le_), __FILE__, __LINE__); } while (0)

// Programmatic dependent launch (decode-step kernels): the kernel may begin while its predecessor on the
// stream is still running; it must not read anything the predecessor writes before pdl_wait(). A kernel
// calls pdl_launch_dependents() early so that its own successor may begin the same way.
// `early` = false launches the same kernel in plain stream order: worth it for the large launches, where starting
// early buys nothing and the successor's CTAs waiting on the SMs measured about 2% slower on the 12-layer generate.
template <typename... KArgs, typename... Args>
static inline void launch_pdl_if(bool early, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args... args) {
    static const bool off = getenv("NCM_B200_NO_PDL") != nullptr;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = ::ncmb::stream();
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = (off || !early) ? 0 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    if (e != cudaSuccess) ::ncmb::fatal("launch failed: %s", cudaGetErrorString(e));
}
template <typename... KArgs, typename... Args>
static inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args... args) {
    static const bool off = getenv("NCM_B200_NO_PDL") != nullptr;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = ::ncmb::stream();
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = off ? 0 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    if (e != cudaSuccess) ::ncmb::fatal("launch failed: %s", cudaGetErrorString(e));
}
#define LAUNCH_PDL(kernel, grid, block, smem, ...) do { \
    ::ncmb::launch_pdl(kernel, dim3(grid), dim3(block), (size_t)(smem), __VA_ARGS__); \
    ::ncmb::ctx().launches++; \
    cudaError_t le_ = cudaGetLastError(); \
    if (le_ != cudaSuccess) ::ncmb::fatal("launch %s failed: %s (%s:%d)", #kernel, \
        cudaGetErrorString(le_), __FILE__, __LINE__); } while (0)
#define LAUNCH_PDL_IF(early, kernel, grid, block, smem, ...) do { \
    ::ncmb::launch_pdl_if((early), kernel, dim3(grid), dim3(block), (size_t)(smem), __VA_ARGS__); \
    ::ncmb::ctx().launches++; \
    cudaError_t le_ = cudaGetLastError(); \
    if (le_ != cudaSuccess) ::ncmb::fatal("launch %s failed: %s (%s:%d)", #kernel, \
        cudaGetErrorString(le_), __FILE__, __LINE__); } while (0)
// launches of at most this many CTAs (or GEMM tiles) start early
static inline bool pdl_small(int64_t ctas) { return ctas <= (int64_t)::ncmb::ctx().sm_count * 8; }
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

static inline int64_t cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }
static inline unsigned grid1d(int64_t n, int block) {
    int64_t g = cdiv(n, block);
    if (g < 1) g = 1;
    if (g > 0x7fffffff) fatal("grid too large");
    return (unsigned)g;
}

// ---- device workspace: bump allocator over one cudaMalloc'ed slab, grown on demand ----
struct Workspace {
    char *base = nullptr;
    size_t cap = 0, off = 0;
    bool measuring = false;              // alloc() only advances `off` (sizing pass before reserve)
    void reserve(size_t bytes);          // frees and reallocates when too small (contents lost)
    void reset() { off = 0; }
    void *alloc(size_t bytes);           // 256-byte aligned; fatal on overflow
    template <class T> T *get(size_t n) { return (T *)alloc(n * sizeof(T)); }
    void release();
};

// ---- activation codes for fused epilogues ----
enum Act { ACT_NONE = 0, ACT_GELU = 1, ACT_GELU_TANH = 2, ACT_SILU = 3, ACT_RELU2 = 4 };

// Format of a GEMM input that its producer already wrote as a split pair (x, x_lo):
//   SPLIT_TF32: float arrays, x = rn_tf32(v), x_lo = v - x
//   SPLIT_H16:  both buffers read as __half arrays with the same element stride,
//               x = rn_f16(16 v), x_lo = rn_f16(16 v - x)
enum SplitFmt { SPLIT_NONE = 0, SPLIT_TF32 = 1, SPLIT_H16 = 2 };

// y[M,N] = act(x[M,K] W[N,K]^T + bias[N]) (+ res[M,N]); res may alias y. ldx/ldy: row strides.
struct GemmArgs {
    const float *x = nullptr; int64_t ldx = 0;
    const float *W = nullptr;            // [N][K] row-major
    const float *bias = nullptr;
    const float *res = nullptr; int64_t ldres = 0;
    float *y = nullptr; int64_t ldy = 0;
    int64_t M = 0; int N = 0, K = 0;
    int act = ACT_NONE;
    // gated MLP: y[m, j] = act(acc[m, 2j]) * acc[m, 2j+1] with W holding interleaved
    // gate/up rows (N = 2 * hidden); y has N/2 columns.
    int glu = 0;
    const void *wshadow = nullptr;       // engine-specific preprocessed copy of W (or null)
    // three-pass mode: x may arrive already split (x = hi part, x_lo = lo part, both [M][K] with stride ldx),
    // and the result may be written split (y = hi, y_lo = lo, same stride) for the next GEMM to consume.
    const float *x_lo = nullptr;
    float *y_lo = nullptr;
    int x_fmt = SPLIT_TF32, y_fmt = SPLIT_TF32;   // formats of (x, x_lo) and (y, y_lo) when the lo pointer is set
    // few-row (decode) calls only: bytes the NEXT weight-streaming kernel of the step will read; the GEMV asks L2 for
    // them while it runs (a 2 - 20 MB matrix is about one memory latency's worth of bandwidth, so a chain of such
    // kernels is paced by latency unless each one's weights are on their way before it starts)
    const void *pf_next = nullptr; size_t pf_next_bytes = 0;
    // few-row (decode) calls only, honoured by the GEMV kernel (see gemv_fusable()):
    //  * the input rows are normalised on the fly: x <- norm(x) * ln_w (+ ln_b), ln_kind 1 LayerNorm, 2 RMSNorm
    //  * output columns >= y2_col0 are also written to y2[m*ldy2 + (*y2_step_d)*y2_step + (n - y2_col0)]
    //    (the K|V part of a fused QKV projection going straight into the cache)
    int ln_kind = 0; const float *ln_w = nullptr, *ln_b = nullptr; float ln_eps = 0.f;
    float *y2 = nullptr; int y2_col0 = 0; int64_t ldy2 = 0; const int *y2_step_d = nullptr; int64_t y2_step = 0;
    //  * W16: an exact bf16 copy of W ([N][K]); the GEMV kernel streams it instead of W (other engines ignore it)
    const unsigned short *W16 = nullptr;
    // up to four rows on the warp-per-row-pair GEMV only (gemv_warp_takes()):
    //  * gv_pair_half > 0: W holds gate rows [0, half) then up rows [half, 2*half) (N = 2*half); the result is
    //    y[m][j] = act(x.W_j + b_j) * (x.W_{half+j} + b_{half+j}), `half` columns wide
    //  * gv_rope_cos set: columns [0, gv_rope_cols) are heads of width gv_hd whose halves (d, d + gv_hd/2) are
    //    rotated with table row gv_rope_pos[(*gv_rope_step_d) * gv_rope_pos_step + m] before anything is stored
    int gv_pair_half = 0;
    const float *gv_rope_cos = nullptr, *gv_rope_sin = nullptr;
    const int *gv_rope_pos = nullptr, *gv_rope_step_d = nullptr; int64_t gv_rope_pos_step = 0;
    int gv_rope_cols = 0, gv_hd = 0;
    // nearest-row search instead of a stored product (tensor-core engine only): for every x row, the
    // W row n minimising colnorm[n] - 2 x.W_n, kept as min over packed (ordered distance << 32 | n).
    const float *argmin_colnorm = nullptr;
    unsigned long long *argmin_best = nullptr;
    // fused QKV projection, head dim 64 (fp16-pair engine with 128-column tiles only): the per-head RMSNorm and
    // the rotary embedding of the query / key heads (what qk_post() does in a pass of its own) are applied in the
    // epilogue, where a thread holds the 64 columns of one head of its row. Columns [0, qk_heads * 64) are heads
    // (the first qk_H of them queries); qk_pos[m] selects the table row. *qk_applied tells the caller whether the
    // engine did it (otherwise the caller runs qk_post()).
    int qk_heads = 0, qk_H = 0;
    const float *qk_qw = nullptr, *qk_kw = nullptr, *qk_cos = nullptr, *qk_sin = nullptr;
    const int *qk_pos = nullptr;
    bool *qk_applied = nullptr;
};
void gemm(const GemmArgs &a);            // dispatches on ctx().gemm_mode and shape
void gemm_simt(const GemmArgs &a);
bool gemv_fusable(const GemmArgs &a);    // true when the call will run on the GEMV kernel (M <= 16, 16-byte rows)
bool gemv_warp_takes(const GemmArgs &a); // ... on the warp-per-row-pair GEMV, which also takes the gv_* epilogues (M <= 4)
bool gemm_tc_supported(const GemmArgs &a);
void gemm_tc(const GemmArgs &a);
// gemm mode 3: fp16 split pairs, three kind::f16 MMAs per k-step into one accumulator (gemm_h3.cu)
bool gemm_h3_supported(const GemmArgs &a);
void gemm_h3(const GemmArgs &a);
void gemm_h3_forget_weights();
void gemm_tc_forget_weights();
void gemm_h3_forget_range(const void *p, size_t bytes);     // cached copies of matrices overlapping the range only
void gemm_tc_forget_range(const void *p, size_t bytes);
struct StaticWeights { StaticWeights() { ctx().w_static++; } ~StaticWeights() { ctx().w_static--; } };
int gemm_tc_check();                    // reads + clears the tensor-core engine's timeout word

// ---- normalisation / elementwise (kernels_elem.cu) ----
void layernorm(const float *x, const float *w, const float *b, float *y, int64_t rows, int C, float eps);
// y_lo != null: the result is written as a split pair in format fmt (SplitFmt)
void layernorm_split(const float *x, const float *w, const float *b, float *y, float *y_lo, int64_t rows, int C, float eps, int fmt);
void rmsnorm_split(const float *x, const float *w, float *y, float *y_lo, int64_t rows, int C, int fmt);
float *dev_interleave_rows(const float *a, const float *b, int64_t rows, int64_t cols);   // new [2*rows][cols]: a0,b0,a1,b1,...
void rmsnorm(const float *x, const float *w, float *y, int64_t rows, int C, int64_t ldx, int64_t ldy);
void add_inplace(float *y, const float *x, int64_t n);
void add_rows_bcast(float *y, const float *rowvec, int64_t rows, int C);             // y[r,:] += v[:]
void embed_rows(const float *W, const int *idx_dev, float *y, int64_t n, int D);
void glu_combine(const float *gu, float *y, int64_t rows, int Hh, int act);          // [rows][2Hh] halves
void act_inplace(float *x, int64_t n, int act);
void fill_f32(float *p, float v, int64_t n);
void argmax_rows(const float *x, int64_t rows, int V, int *out);                    // first max wins

// ---- generic strided conv / norm / resampling (kernels_vq.cu); layouts via strides ----
struct NCT { int64_t sn, sc, st; };     // element strides of (batch, channel, time)
static inline NCT ncl(int C, int T) { return NCT{(int64_t)C * T, (int64_t)T, 1}; }
static inline NCT nlc(int C, int T) { return NCT{(int64_t)C * T, 1, (int64_t)C}; }
void conv1d(const float *x, NCT xs, const float *W, const float *b, float *y, NCT ys,
            int N, int Cin, int Cout, int T, int K, int stride, int pad, const float *add, float add_scale);
void convT1d(const float *x, NCT xs, const float *W, const float *b, float *y, NCT ys,
             int N, int Cin, int Cout, int T, int K, int stride);
void groupnorm(const float *x, NCT xs, float *y, NCT ys, int N, int G, int C, int T);
void interp_area(const float *x, NCT xs, float *y, NCT ys, int N, int C, int Tin, int Tout);
void interp_linear(const float *x, NCT xs, float *y, NCT ys, int N, int C, int Tin, int Tout);

// ---- attention (attention.cu) ----
// Token-major fused attention. Row r owns query tokens [q_start[r], q_start[r+1]) and
// attends to key segment 1 tokens [k1_start[r], k1_start[r+1]) plus (optionally) key
// segment 2 tokens [k2_start[r], k2_start[r+1]); all keys of a row are visible to all of
// its queries (bidirectional). With causal != 0 segment-1 key j (0-based inside the row)
// is visible to query i only when j <= i + causal_off.
struct AttnArgs {
    const float *q; int64_t ldq;                 // q[token][h*hd + d]
    const float *k1, *v1; int64_t ldk1;          // [token][kvh*hd + d]
    const float *k2 = nullptr, *v2 = nullptr; int64_t ldk2 = 0;
    float *out; int64_t ldo;                     // out[token][h*hd + d]
    float *out_lo = nullptr;                     // optional: write the context as a split pair ...
    int out_fmt = SPLIT_TF32;                    // ... in this format
    const int *q_start, *k1_start, *k2_start = nullptr;   // device int[rows+1]
    const int *k1_len = nullptr;                 // optional device int[rows]: segment-1 lengths (strided caches)
    int rows, H, Hkv, hd;
    int max_q = 0;                                 // max queries of any row (grid sizing)
    int causal = 0, causal_off = 0;
    int window = 0;                              // > 0: key j visible to query i only if |i - j| <= window
    int64_t total_q = 0; double avg_keys = 0;    // for the profiler only
    // tensor-core path only (0 = unknown, which keeps the call on the CUDA-core kernel):
    int max_k1 = 0, max_k2 = 0;                  // longest key segment of any row
    int64_t q_total = 0, k1_total = 0, k2_total = 0;   // token rows the q / k1 / k2 buffers hold (TMA bounds)
    // decode steps replayed from one CUDA graph: lengths are read from k1_len + (*step_d) * k1_len_step
    const int *step_d = nullptr; int64_t k1_len_step = 0;
};
void attention(const AttnArgs &a);
bool attention_decode_supported(const AttnArgs &a);   // attention_decode.cu: one query per row, keys split over CTAs
void attention_decode(const AttnArgs &a);
bool attention_tc_supported(const AttnArgs &a);  // attention_tc.cu: head dim 64, <= 288 padded keys per row
void attention_tc(const AttnArgs &a);
bool attention_tc_long_supported(const AttnArgs &a);   // more keys: 256-key blocks through the same kernel + a merge
void attention_tc_long(const AttnArgs &a);
// reference-layout SDPA with an additive [Tq][Tkv] mask (ncm.h API)
void sdpa_masked(const float *q, const float *k, const float *v, const float *mask, float *out,
                 int B, int Hq, int Hkv, int Tq, int Tkv, int hd);
// in place on the q / k slices of a token-major fused projection: optional per-head
// RMSNorm (eps 1e-6) then half-split rotary embedding with table row pos[token].
void qk_post(float *q, int64_t ldq, int H, float *k, int64_t ldk, int Hkv, int hd, int64_t ntok,
             const float *qnorm_w, const float *knorm_w, const float *cos_t, const float *sin_t,
             const int *pos_dev, const int *step_d = nullptr, int64_t pos_step = 0);

// ---- sampling (sampling.cu) ----
struct SampleArgs {
    const float *logits;       // [rows_model][Lc][V]; cond rows first, uncond rows at +uncond_off rows
    int Bn, Lc, V;
    int64_t uncond_off;        // in rows; 0 = no CFG
    double cfg_w;              // blend weight tw: (1+tw)*cond - tw*uncond
    float temp; int top_k; float top_p;
    float freq, mu, adj_a; int adj_w; float adj_d;
    const double *allow_dev;   // [V] or null
    double *cnt;               // [Bn][cnt_stride] persistent counts (null when penalties are off)
    int cnt_stride;
    int *hist; int *hist_len; int hist_stride;   // [Bn][hist_stride], [Bn]
    const double *uniforms;    // [Bn][Lc] pre-drawn uniforms in [0,1) (temp > 0); null = counter-based
    unsigned long long rng_seed = 0; long long rng_row0 = 0; int rng_level = 0;   // counter-based stream key
    int rng_wrap = 0;          // > 0: rows b >= rng_wrap are the unconditional twins of rows b - rng_wrap (level 0 under CFG);
                               // they draw on their sequence's key with a level of their own, so a sequence's draws do
                               // not depend on how many sequences share the call
    int *out;                  // [Bn][out_stride] picks written at out_off + t
    int out_stride, out_off;
    float *blend_out;          // optional [Bn][Lc][V] copy of the logits actually sampled from
    float *scratch;            // [Bn][V] when V does not fit shared memory, else null
    int picks_bound = 0;       // upper bound on the tokens a row has picked before and during this call (0 = unknown)
};
void sample_rows(const SampleArgs &a);
size_t sample_scratch_floats(int Bn, int V);

// ---- transformer block shared by the NCP stack, the VQ-VAE blocks and the decoder LMs ----
enum NormKind { NORM_LAYER = 0, NORM_RMS = 1 };
struct BlockWeights {
    int norm = NORM_LAYER; float eps = 1e-6f;
    const float *ln1w = nullptr, *ln1b = nullptr, *ln2w = nullptr, *ln2b = nullptr;
    const float *qkvw = nullptr, *qkvb = nullptr;      // [C + 2*nkv*hd][C]
    const float *ow = nullptr, *ob = nullptr;          // [C][C]
    const float *qnw = nullptr, *knw = nullptr;        // per-head RMSNorm gains or null
    const float *fcw = nullptr, *fcb = nullptr;        // ungated [Hh][C]; gated [2*Hh][C] (gate rows, then up rows)
    const float *fcw_il = nullptr, *fcb_il = nullptr;  // gated only: gate/up rows interleaved (fused gated epilogue)
    const float *pw = nullptr, *pb = nullptr;          // [C][Hh]
    // exact bf16 copies of the four matrices (decode steps stream these), or null
    const unsigned short *qkvw16 = nullptr, *ow16 = nullptr, *fcw16 = nullptr, *pw16 = nullptr;
    // decode steps: the matrix the step's next weight-streaming kernel will read after this block's last one (the
    // next block's QKV matrix, or the start of the vocabulary projection), for that kernel's L2 prefetch
    const void *next_w = nullptr; size_t next_w_bytes = 0;
    int Hh = 0, gated = 0, act = ACT_GELU;
};
struct BlockBufs { float *ln, *qkv, *ctx, *mlp, *h; };   // [n][C], [n][C+2kvd], [n][C], [n][Hh or 2Hh], [n][Hh]
struct AttnPlan {
    const int *q_start = nullptr, *k1_start = nullptr, *k1_len = nullptr, *k2_start = nullptr;
    const float *k1 = nullptr, *v1 = nullptr; int64_t ldk1 = 0;   // null: segment 1 is this pass's own K/V
    int self_is_k2 = 0;                  // segment 2 = this pass's own K/V (k2_start = q_start)
    const float *k2 = nullptr, *v2 = nullptr; int64_t ldk2 = 0;   // or an explicit second segment (k2_start required)
    int max_k2 = 0; int64_t k2_total = 0;
    int rows = 0, max_q = 0, causal = 0, causal_off = 0, window = 0;
    const int *pos = nullptr; const float *cos_t = nullptr, *sin_t = nullptr;
    int64_t total_q = 0; double avg_keys = 0;
    int max_k1 = 0; int64_t k1_total = 0;  // longest segment-1 key run; token rows behind k1 (0 = not stated)
    // one captured graph for every decode step: per-step arrays are indexed by the device counter *step_d
    const int *step_d = nullptr;
    int64_t k1_len_step = 0, pos_step = 0, kv_store_step = 0;   // strides (elements) of k1_len / pos / kv_store per step
    // after the K/V of this pass are final (norm + rope applied) they are stored here:
    float *kv_store = nullptr; int64_t kv_pitch = 0;   // row pitch in floats; rows = tokens, width 2*kvd
    int kv_rows_per_seq = 0; int64_t kv_seq_pitch = 0; // > 0: token t of sequence s goes to s*kv_seq_pitch + t*kv_pitch
    int kv_only = 0;                     // stop after the K/V of this pass are stored (last layer of a cache fill)
};
void run_block(float *x, int64_t ntok, int C, int H, int nkv, const BlockWeights &w, const BlockBufs &b, const AttnPlan &p);
void apply_norm(const float *x, const float *w, const float *b, float *y, int64_t rows, int C, int kind, float eps);
void apply_norm_split(const float *x, const float *w, const float *b, float *y, float *y_lo, int64_t rows, int C, int kind, float eps, int fmt);
// [rows][cols] fp32 -> bf16 copy when every element is exactly representable in bf16, else null (new device buffer)
unsigned short *dev_bf16_exact(const float *w, int64_t n);
void make_gated_interleaved(BlockWeights &w, int C, std::vector<void *> &owned);   // fills fcw_il / fcb_il from fcw / fcb

// weight lookup helpers
Tensor *wget(WeightStore *ws, const char *fmt, ...);      // null when missing
Tensor *wneed(WeightStore *ws, const char *fmt, ...);     // fatal when missing
float *dev_concat_rows(const float *a, int64_t na, const float *b, int64_t nb);   // new buffer [na+nb]; null parts -> zeros
void upload(void *dev, const void *host, size_t bytes);
void *dev_alloc(size_t bytes);
void dev_free(void *p);

} // namespace ncmb
