// Multiscale residual quantizer on the device (reference src/vq.c).
//
// The reference walks every level through host memory (code gather, z_hat += up,
// Phi blend, argmin over a materialised [rows][V] distance matrix). Here every
// tensor stays token-major [B][L][D] in HBM: the resampling kernels take strides,
// so no [B][L][D] <-> [B][D][L] transposes are issued, and the nearest-code search
// keeps a running (distance, index) minimum instead of writing distances out.
#include "common.cuh"
#include "vq.cuh"

namespace ncmb {

// rowmod > 0: row b reads the codes of row b % rowmod (the CFG half shares the sampled codes)
__global__ void k_gather_codes(const float *__restrict__ E, const int *__restrict__ codes, int stride, int rowmod, int tlen,
                               int D, int V, int64_t n, float *__restrict__ out) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int d = (int)(i % D); int64_t r = i / D; int t = (int)(r % tlen); int64_t b = r / tlen;
        if (rowmod > 0) b %= rowmod;
        int code = codes[b * stride + t];
        code = code < 0 ? 0 : (code >= V ? V - 1 : code);
        out[i] = E[(int64_t)code * D + d];
    }
}
__global__ void k_sub_inplace(float *__restrict__ y, const float *__restrict__ x, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) y[i] -= x[i];
}

// ---- nearest code: argmin_j |x_r - E_j|^2, strict < so the lowest index wins ties
// (reference src/vq.c:440-441). 16 rows per CTA; the codebook streams through shared
// memory in 128-code tiles; thread j of a tile owns code j for all 16 rows. ----
constexpr int NR_ROWS = 16, NR_TILE = 128;
__global__ void __launch_bounds__(NR_TILE) k_nearest(const float *__restrict__ x, const float *__restrict__ E,
                                                     int64_t rows, int V, int D, int *__restrict__ idx_out,
                                                     int out_tlen, int out_stride, int out_off) {
    extern __shared__ float sm[];
    float *xs = sm;                         // [NR_ROWS][D]
    float *es = xs + NR_ROWS * D;           // [NR_TILE][D + 1]
    const int tid = threadIdx.x;
    const int64_t r0 = (int64_t)blockIdx.x * NR_ROWS;
    for (int i = tid; i < NR_ROWS * D; i += NR_TILE) {
        int64_t r = r0 + i / D;
        xs[i] = r < rows ? x[r * D + (i % D)] : 0.f;
    }
    float best[NR_ROWS]; int bi[NR_ROWS];
#pragma unroll
    for (int r = 0; r < NR_ROWS; r++) { best[r] = INFINITY; bi[r] = 0x7fffffff; }
    for (int j0 = 0; j0 < V; j0 += NR_TILE) {
        __syncthreads();
        for (int i = tid; i < NR_TILE * D; i += NR_TILE) {
            int j = i / D, c = i % D;
            es[j * (D + 1) + c] = (j0 + j < V) ? E[(int64_t)(j0 + j) * D + c] : 0.f;
        }
        __syncthreads();
        int j = j0 + tid;
        if (j < V) {
            float acc[NR_ROWS];
#pragma unroll
            for (int r = 0; r < NR_ROWS; r++) acc[r] = 0.f;
            const float *er = es + tid * (D + 1);
            for (int c = 0; c < D; c++) {
                float e = er[c];
#pragma unroll
                for (int r = 0; r < NR_ROWS; r++) { float d = xs[r * D + c] - e; acc[r] = fmaf(d, d, acc[r]); }
            }
#pragma unroll
            for (int r = 0; r < NR_ROWS; r++) if (acc[r] < best[r]) { best[r] = acc[r]; bi[r] = j; }
        }
    }
    __syncthreads();                         // the code tile is dead: reuse it for the cross-thread reduction
    float *bval = es;                        // [NR_ROWS][NR_TILE]
    int *bidx = (int *)(es + NR_ROWS * NR_TILE);
#pragma unroll
    for (int r = 0; r < NR_ROWS; r++) { bval[r * NR_TILE + tid] = best[r]; bidx[r * NR_TILE + tid] = bi[r]; }
    __syncthreads();
    if (tid < NR_ROWS) {
        int64_t r = r0 + tid;
        if (r < rows) {
            float bv = INFINITY; int bj = 0x7fffffff;
            for (int t = 0; t < NR_TILE; t++) {
                float v = bval[tid * NR_TILE + t]; int j = bidx[tid * NR_TILE + t];
                if (v < bv || (v == bv && j < bj)) { bv = v; bj = j; }
            }
            if (bj == 0x7fffffff) bj = 0;
            int64_t b = r / out_tlen; int t = (int)(r % out_tlen);
            idx_out[b * out_stride + out_off + t] = bj;
        }
    }
}

// ---- tensor-core route: |x - e|^2 = |x|^2 - 2 x.e + |e|^2, and |x|^2 does not change the argmin, so
// the search is a [rows x V x D] GEMM whose epilogue keeps min_n(|e_n|^2 - 2 x.e_n) per row and never
// writes the products. Three-pass TF32 keeps the dot products fp32-grade. ----
__global__ void k_row_sqnorm(const float *__restrict__ E, int V, int D, float *__restrict__ out) {
    int v = blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= V) return;
    float s = 0.f;
    for (int c = 0; c < D; c++) { float e = E[(int64_t)v * D + c]; s = fmaf(e, e, s); }
    out[v] = s;
}
__global__ void k_unpack_best(const unsigned long long *__restrict__ best, int64_t rows, int *__restrict__ idx_out,
                              int out_tlen, int out_stride, int out_off) {
    int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    int64_t b = r / out_tlen; int t = (int)(r % out_tlen);
    idx_out[b * out_stride + out_off + t] = (int)(best[r] & 0xffffffffull);
}

static bool vq_nearest_tc(const float *x, const float *E, int64_t rows, int V, int D, int *idx_out, int out_tlen, int out_stride, int out_off) {
    static Workspace ws;
    GemmArgs g;
    g.x = x; g.ldx = D; g.W = E; g.M = rows; g.N = V; g.K = D;
    size_t need = (size_t)rows * 8 + (size_t)V * 4 + 1024;
    if (need > ws.cap) ws.reserve(need + need / 4);
    ws.reset();
    unsigned long long *best = ws.get<unsigned long long>(rows);
    float *cn = ws.get<float>(V);
    g.argmin_best = best; g.argmin_colnorm = cn;
    if (ctx().gemm_mode < 1 || !gemm_tc_supported(g)) return false;
    CUDA_CHECK(cudaMemsetAsync(best, 0xff, (size_t)rows * 8, stream()));
    LAUNCH(k_row_sqnorm, (unsigned)cdiv(V, 128), 128, 0, E, V, D, cn);
    {
        StaticWeights sw;                       // codebooks are model weights: cache their hi / lo split
        gemm_tc(g);
    }
    LAUNCH(k_unpack_best, (unsigned)cdiv(rows, 256), 256, 0, best, rows, idx_out, out_tlen, out_stride, out_off);
    return true;
}

void vq_nearest(const float *x, const float *E, int64_t rows, int V, int D, int *idx_out, int out_tlen, int out_stride, int out_off) {
    if (rows <= 0) return;
    if (rows >= 1024 && vq_nearest_tc(x, E, rows, V, D, idx_out, out_tlen, out_stride, out_off)) return;
    size_t es_fl = (size_t)NR_TILE * (D + 1);
    if (es_fl < 2 * (size_t)NR_ROWS * NR_TILE) es_fl = 2 * (size_t)NR_ROWS * NR_TILE;
    size_t smem = sizeof(float) * ((size_t)NR_ROWS * D + es_fl);
    if (smem > 48 * 1024) fatal("vq_nearest: D=%d too large for this kernel", D);
    ProfScope ps(NCMB_K_VQ, 3.0 * (double)rows * V * D, 4.0 * (double)rows * (D + 1));
    LAUNCH(k_nearest, grid1d(rows, NR_ROWS), NR_TILE, smem, x, E, rows, V, D, idx_out, out_tlen, out_stride, out_off);
}

static unsigned ew(int64_t n) {
    int64_t g = cdiv(n, 256), cap = (int64_t)ctx().sm_count * 16;
    return (unsigned)(g < 1 ? 1 : (g > cap ? cap : g));
}

// q [B][tlen][D] -> out [B][L][D]  (reference up_to_full, src/vq.c:327-376). tmp1/tmp2: [B][L][D] scratch.
static void up_to_full_dev(VQState *v, const float *q, int B, int tlen, int level, float *out, float *tmp1, float *tmp2) {
    int D = v->D, L = v->L;
    if (level == 0 && v->has_l1) {
        const float *cur = q;
        int Tc = tlen;
        float *bufs[2] = {tmp1, tmp2};
        int flip = 0;
        for (int i = 0; i < v->n_up; i++) {
            int s = v->upK[i], To = (Tc - 1) * s + s;
            if (v->l1_norm && i > 0) {
                float *gn = bufs[flip]; flip ^= 1;
                groupnorm(cur, nlc(D, Tc), gn, nlc(D, Tc), B, 8, D, Tc);
                cur = gn;
            }
            bool last = (i == v->n_up - 1) && !v->l1_norm_final;
            float *nx = last ? out : bufs[flip];
            if (!last) flip ^= 1;
            convT1d(cur, nlc(D, Tc), v->upW[i], v->upB[i], nx, nlc(D, To), B, D, D, Tc, s, s);
            cur = nx; Tc = To;
        }
        if (Tc != L) fatal("learned up cascade yields length %d, expected %d", Tc, L);
        if (v->l1_norm_final) groupnorm(cur, nlc(D, Tc), out, nlc(D, Tc), B, 8, D, Tc);
        else if (cur != out) CUDA_CHECK(cudaMemcpyAsync(out, cur, (size_t)B * L * D * 4, cudaMemcpyDeviceToDevice, stream()));
    } else {
        interp_linear(q, nlc(D, tlen), out, nlc(D, L), B, D, tlen, L);
    }
    if (v->has_all && level >= 1 && level <= v->n_levels - 2 && v->urefW[level]) {
        conv1d(out, nlc(D, L), v->urefW[level], v->urefB[level], tmp1, nlc(D, L), B, D, D, L, 3, 1, 1, out, 0.f);
        CUDA_CHECK(cudaMemcpyAsync(out, tmp1, (size_t)B * L * D * 4, cudaMemcpyDeviceToDevice, stream()));
    }
}

// z [B][Lin][D] -> out [B][levels[level]][D]  (reference down_for_quant, src/vq.c:271-324)
static void down_for_quant_dev(VQState *v, const float *z, int B, int Lin, int level, float *out, float *tmp1, float *tmp2) {
    int D = v->D, tlen = v->levels[level];
    if (level == 0 && v->has_l1) {
        const float *cur = z;
        int Tc = Lin;
        float *bufs[2] = {tmp1, tmp2};
        int flip = 0;
        for (int i = 0; i < v->n_down; i++) {
            int s = v->downK[i], To = Tc / s;
            if (v->l1_norm && i > 0) {
                float *gn = bufs[flip]; flip ^= 1;
                groupnorm(cur, nlc(D, Tc), gn, nlc(D, Tc), B, 8, D, Tc);
                cur = gn;
            }
            bool last = (i == v->n_down - 1) && !v->l1_norm_final;
            float *nx = last ? out : bufs[flip];
            if (!last) flip ^= 1;
            conv1d(cur, nlc(D, Tc), v->downW[i], v->downB[i], nx, nlc(D, To), B, D, D, Tc, s, s, 0, nullptr, 0.f);
            cur = nx; Tc = To;
        }
        if (v->l1_norm_final) groupnorm(cur, nlc(D, Tc), out, nlc(D, Tc), B, 8, D, Tc);
        else if (cur != out) CUDA_CHECK(cudaMemcpyAsync(out, cur, (size_t)B * Tc * D * 4, cudaMemcpyDeviceToDevice, stream()));
    } else {
        interp_area(z, nlc(D, Lin), out, nlc(D, tlen), B, D, Lin, tlen);
    }
    if (v->has_all && level >= 1 && level <= v->n_levels - 2 && v->drefW[level]) {
        conv1d(out, nlc(D, tlen), v->drefW[level], v->drefB[level], tmp1, nlc(D, tlen), B, D, D, tlen, 3, 1, 1, out, 0.f);
        CUDA_CHECK(cudaMemcpyAsync(out, tmp1, (size_t)B * tlen * D * 4, cudaMemcpyDeviceToDevice, stream()));
    }
}

static int phi_index(const VQState *v, int level) {       // reference src/vq.c:212-221
    if (v->n_phi == 1) return 0;
    double at = (double)level / (v->n_levels - 1);
    int best = 0; double bd = 1e300;
    for (int j = 0; j < v->n_phi; j++) {
        double d = fabs(v->ticks[j] - at);
        if (d < bd) { bd = d; best = j; }
    }
    return best;
}

void vq_increment_dev(VQState *v, const int *codes_dev, int stride, int rowmod, int level, int B, float *up, float *scratch) {
    int D = v->D, L = v->L, tlen = v->levels[level];
    size_t n = (size_t)B * L * D;
    float *q = scratch, *t1 = scratch + n, *t2 = scratch + 2 * n, *t3 = scratch + 3 * n;
    {
        int64_t ng = (int64_t)B * tlen * D;
        ProfScope ps(NCMB_K_VQ);
        LAUNCH(k_gather_codes, ew(ng), 256, 0, v->E[level], codes_dev, stride, rowmod, tlen, D, v->vocabs[level], ng, q);
    }
    if (v->resi) {
        up_to_full_dev(v, q, B, tlen, level, t3, t1, t2);
        int j = phi_index(v, level);
        conv1d(t3, nlc(D, L), v->phiW[j], v->phiB[j], up, nlc(D, L), B, D, D, L, 3, 1, 1, t3, v->resi_ratio);
    } else {
        up_to_full_dev(v, q, B, tlen, level, up, t1, t2);
    }
}

size_t vq_scratch_floats(const VQState *v, int B) { return 4 * (size_t)B * v->L * v->D + 64; }

void vq_next_input_dev(VQState *v, const int *codes_dev, int stride, int rowmod, int level, float *z_hat, float *x_out, int B, float *scratch) {
    size_t n = (size_t)B * v->L * v->D;
    float *up = scratch + 4 * n;           // caller provides 5n floats
    vq_increment_dev(v, codes_dev, stride, rowmod, level, B, up, scratch);
    add_inplace(z_hat, up, (int64_t)n);
    interp_area(z_hat, nlc(v->D, v->L), x_out, nlc(v->D, v->levels[level + 1]), B, v->D, v->L, v->levels[level + 1]);
}

void vq_encode_dev(VQState *v, const float *z, int B, int *idx_dev, float *scratch) {
    int D = v->D, L = v->L, total = vq_total_codes(v);
    size_t n = (size_t)B * L * D;
    float *z_rest = scratch + 5 * n, *down = scratch + 6 * n, *up = scratch + 4 * n;   // caller provides 7n floats
    CUDA_CHECK(cudaMemcpyAsync(z_rest, z, n * 4, cudaMemcpyDeviceToDevice, stream()));
    int off = 0;
    for (int lv = 0; lv < v->n_levels; lv++) {
        int tlen = v->levels[lv];
        down_for_quant_dev(v, z_rest, B, L, lv, down, scratch, scratch + n);
        vq_nearest(down, v->E[lv], (int64_t)B * tlen, v->vocabs[lv], D, idx_dev, tlen, total, off);
        if (lv + 1 < v->n_levels) {
            vq_increment_dev(v, idx_dev + off, total, 0, lv, B, up, scratch);
            ProfScope ps(NCMB_K_VQ);
            LAUNCH(k_sub_inplace, ew((int64_t)n), 256, 0, z_rest, up, (int64_t)n);
        }
        off += tlen;
    }
}

void vq_zhat_final_dev(VQState *v, const int *idx_dev, int B, float *z_hat, float **snapshots, float *scratch) {
    int total = vq_total_codes(v);
    size_t n = (size_t)B * v->L * v->D;
    float *up = scratch + 4 * n;
    CUDA_CHECK(cudaMemsetAsync(z_hat, 0, n * 4, stream()));
    int base = 0;
    for (int lv = 0; lv < v->n_levels; lv++) {
        vq_increment_dev(v, idx_dev + base, total, 0, lv, B, up, scratch);
        add_inplace(z_hat, up, (int64_t)n);
        if (snapshots && snapshots[lv] && snapshots[lv] != z_hat)
            CUDA_CHECK(cudaMemcpyAsync(snapshots[lv], z_hat, n * 4, cudaMemcpyDeviceToDevice, stream()));
        base += v->levels[lv];
    }
}

int *vq_codes_to_dev(VQState *v, const int *host, size_t n) {
    v->codes_ws.reserve(n * sizeof(int) + 256);
    v->codes_ws.reset();
    int *d = v->codes_ws.get<int>(n);
    upload(d, host, n * sizeof(int));
    return d;
}

} // namespace ncmb

using namespace ncmb;

extern "C" {

// binds codebooks, Phi convs, cascade stages and refine convs by name (reference src/vq.c:75-192)
VQState *vq_load(const NCMConfig *c, WeightStore *ws, const char *prefix) {
    ensure_device();
    VQState *v = new VQState();
    v->n_levels = c->n_qlevels;
    for (int i = 0; i < v->n_levels; i++) { v->levels[i] = c->levels[i]; v->vocabs[i] = c->vq_vocab[i]; }
    v->D = c->vq_embed_dim;
    v->L = c->levels[c->n_qlevels - 1];
    for (int i = 0; i < v->n_levels; i++) v->E[i] = wneed(ws, "%sembeddings.%d.weight", prefix, i)->data;
    v->resi = c->quant_resi_enabled && fabsf(c->quant_resi_ratio) > 1e-6f;
    v->resi_ratio = c->quant_resi_ratio;
    if (v->resi) {
        int sm = c->quant_resi_share_mode;
        v->n_phi = sm == 0 ? v->n_levels : (sm == 1 ? 1 : sm);
        for (int i = 0; i < v->n_phi; i++) {
            Tensor *w = wget(ws, "%squant_resi.%d.weight", prefix, i), *b = wget(ws, "%squant_resi.%d.bias", prefix, i);
            if (!w && v->n_phi == 1) w = wget(ws, "%squant_resi.weight", prefix);
            if (!b && v->n_phi == 1) b = wget(ws, "%squant_resi.bias", prefix);
            if (!w || !b) { fprintf(stderr, "missing weight %squant_resi.%d\n", prefix, i); exit(1); }
            v->phiW[i] = w->data; v->phiB[i] = b->data;
            v->ticks[i] = (v->n_phi == 4) ? (i + 1.0 / 3.0) / v->n_phi : (i + 0.5) / v->n_phi;
        }
    }
    if (c->learned_l1_sampling) {
        v->has_l1 = 1; v->l1_norm = c->learned_l1_norm; v->l1_norm_final = c->learned_l1_norm_final;
        for (int s = 0; s < 16; s++) {
            Tensor *t = wget(ws, "%slearned_down_l1.%d.weight", prefix, s);
            if (t) {
                v->downW[v->n_down] = t->data; v->downK[v->n_down] = (int)t->shape[2];
                v->downB[v->n_down] = wneed(ws, "%slearned_down_l1.%d.bias", prefix, s)->data;
                v->n_down++;
            }
            t = wget(ws, "%slearned_up_l1.%d.weight", prefix, s);
            if (t) {
                v->upW[v->n_up] = t->data; v->upK[v->n_up] = (int)t->shape[2];
                v->upB[v->n_up] = wneed(ws, "%slearned_up_l1.%d.bias", prefix, s)->data;
                v->n_up++;
            }
        }
        if (!v->n_down) { fprintf(stderr, "learned_l1 weights missing\n"); exit(1); }
    }
    if (c->learned_all_sampling) {
        v->has_all = 1;
        for (int i = 1; i <= v->n_levels - 2; i++) {
            Tensor *t = wget(ws, "%slearned_down_refine.%d.weight", prefix, i);
            if (t) { v->drefW[i] = t->data; v->drefB[i] = wneed(ws, "%slearned_down_refine.%d.bias", prefix, i)->data; }
            t = wget(ws, "%slearned_up_refine.%d.weight", prefix, i);
            if (t) { v->urefW[i] = t->data; v->urefB[i] = wneed(ws, "%slearned_up_refine.%d.bias", prefix, i)->data; }
        }
    }
    return v;
}

void vq_free(VQState *vq) {
    if (!vq) return;
    vq->work.release(); vq->codes_ws.release();
    delete vq;
}
int vq_total_codes(const VQState *vq) { int s = 0; for (int i = 0; i < vq->n_levels; i++) s += vq->levels[i]; return s; }
int vq_nlevels(const VQState *vq) { return vq->n_levels; }
int vq_level_len(const VQState *vq, int k) { return vq->levels[k]; }
int vq_level_V(const VQState *vq, int k) { return vq->vocabs[k]; }
int vq_Ltotal(const VQState *vq) { return vq->L; }
int vq_Ddim(const VQState *vq) { return vq->D; }

static float *vq_scratch(VQState *vq, int B, int mult) {
    size_t n = (size_t)B * vq->L * vq->D;
    vq->work.reserve((mult * n + 1024) * sizeof(float));
    vq->work.reset();
    return vq->work.get<float>(mult * n);
}

void vq_next_input(VQState *vq, const int *codes, int level_idx, float *z_hat, float *x_out, int B) {
    int *cd = vq_codes_to_dev(vq, codes, (size_t)B * vq->levels[level_idx]);
    vq_next_input_dev(vq, cd, vq->levels[level_idx], 0, level_idx, z_hat, x_out, B, vq_scratch(vq, B, 5));
}

void vq_idx_to_zhats(VQState *vq, const int *idx, int B, float **zhats) {
    int *cd = vq_codes_to_dev(vq, idx, (size_t)B * vq_total_codes(vq));
    float *scr = vq_scratch(vq, B, 6);
    float *zh = scr + 5 * (size_t)B * vq->L * vq->D;
    vq_zhat_final_dev(vq, cd, B, zh, zhats, scr);
}

void vq_z_to_idx(VQState *vq, const float *z, int B, int *idx) {
    int total = vq_total_codes(vq);
    vq->codes_ws.reserve((size_t)B * total * sizeof(int) + 256);
    vq->codes_ws.reset();
    int *idx_dev = vq->codes_ws.get<int>((size_t)B * total);
    vq_encode_dev(vq, z, B, idx_dev, vq_scratch(vq, B, 7));
    mem_d2h(idx, idx_dev, (size_t)B * total * sizeof(int));
}

// idx [B][total] -> teacher-forcing input [B][T][D] (reference src/vq.c:601-674)
void vq_idx_to_ncm_input(VQState *vq, const int *idx, int B, float *x_out) {
    int D = vq->D, L = vq->L, total = vq_total_codes(vq), T = total - vq->levels[0];
    size_t n = (size_t)B * L * D;
    int *cd = vq_codes_to_dev(vq, idx, (size_t)B * total);
    float *scr = vq_scratch(vq, B, 7);
    float *up = scr + 4 * n, *z_hat = scr + 5 * n, *chunk = scr + 6 * n;
    CUDA_CHECK(cudaMemsetAsync(z_hat, 0, n * 4, stream()));
    int base = 0, off = 0;
    for (int li = 0; li < vq->n_levels - 1; li++) {
        int nlen = vq->levels[li + 1];
        vq_increment_dev(vq, cd + base, total, 0, li, B, up, scr);
        add_inplace(z_hat, up, (int64_t)n);
        interp_area(z_hat, nlc(D, L), chunk, nlc(D, nlen), B, D, L, nlen);
        CUDA_CHECK(cudaMemcpy2DAsync(x_out + (size_t)off * D, (size_t)T * D * 4, chunk, (size_t)nlen * D * 4,
                                     (size_t)nlen * D * 4, B, cudaMemcpyDeviceToDevice, stream()));
        base += vq->levels[li]; off += nlen;
    }
}

void ncmb_vq_encode_dev(VQState *vq, const float *z_dev, int B, int *idx_dev) {
    vq_encode_dev(vq, z_dev, B, idx_dev, vq_scratch(vq, B, 7));
}
void ncmb_vq_nearest_dev(VQState *vq, int level, const float *x_dev, long long n, int *idx_dev) {
    ensure_device();
    vq_nearest(x_dev, vq->E[level], n, vq->vocabs[level], vq->D, idx_dev, 1, 1, 0);
}

} // extern "C"
