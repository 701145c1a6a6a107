// One decode step of a decoder LM (up to four sequences, head dim 64) as ONE persistent cooperative kernel.
//
// A decode step is a chain of small dependent matrix-vector products: launched one by one, each costs a
// launch, a first DRAM round trip and a reduction (~6 us) for ~1.5 us of weight streaming. Here one CTA per SM
// walks the whole step -- embed, then per layer [norm + QKV (+RoPE, K|V to the cache)] [split-key attention]
// [output projection + residual] [norm + MLP up (+ gated product)] [MLP down + residual], then the final norm,
// the vocabulary projection and the greedy pick -- with a grid-wide barrier between phases. Before it arrives
// at a barrier a CTA issues L2 prefetches for the weight rows it will read in the next phase, so the DRAM
// latency of the weight stream runs under the barrier instead of after it.
//
// Work split inside a GEMV phase: one warp per output column (or per pair of columns that belong together: a
// rotary pair (d, d+32) of a head, so RoPE is applied by the warp that produced both halves; a gate column and
// its up column of a gated MLP). The lanes stride over K with 128-bit loads; normalised input rows sit in
// shared memory (once per CTA), un-normalised ones are read from L2. No block-level synchronisation happens
// inside a phase.
//
// Every barrier wait is bounded (2 s): on a timeout the CTA records a code and keeps going, so the kernel always
// ends; the host reads the code and discards the step. The launch is cooperative (all CTAs co-resident).
#include "common.cuh"
#include "lm_mega.cuh"

namespace ncmb {

constexpr int MG_THREADS = 512;
constexpr int MG_KEYS = 32, MG_TEAMS = 4, MG_TEAM = MG_THREADS / MG_TEAMS, MG_MAXG = 8, MG_MAXSPLIT = 64;

__device__ __forceinline__ float mg_act(float v, int act) {
    switch (act) {
        case ACT_GELU: return 0.5f * v * (1.0f + erff(v * 0.7071067811865475f));
        case ACT_GELU_TANH: return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
        case ACT_SILU: return v / (1.0f + expf(-v));
        case ACT_RELU2: { float r = v > 0.f ? v : 0.f; return r * r; }
        default: return v;
    }
}
__device__ __forceinline__ unsigned long long mg_time() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// grid-wide barrier on a counter that only grows: the k-th barrier of this launch is passed when the counter
// reaches base + k * gridDim.x
__device__ __forceinline__ void mg_barrier(const MegaArgs &a, unsigned base, unsigned &k) {
    k++;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned target = base + k * gridDim.x;
        atomicAdd(a.bar, 1u);
        unsigned long long t0 = 0;
        for (unsigned it = 0;; it++) {
            unsigned v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(a.bar) : "memory");
            if ((int)(v - target) >= 0) break;
            if ((it & 1023u) == 1023u) {
                if (*(volatile int *)a.err) break;               // some CTA already gave up: do not wait out every barrier
                unsigned long long now = mg_time();
                if (t0 == 0) t0 = now;
                else if (now - t0 > 2000000000ull) { atomicExch(a.err, 31); break; }
            }
        }
        __threadfence();
    }
    __syncthreads();
}

// block-wide sum of one value per thread (16 warps); red needs 16 floats; every thread gets the result
__device__ __forceinline__ float mg_block_sum(float v, float *red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < MG_THREADS / 32; w++) s += red[w];
    return s;
}

// input rows -> shared memory, optionally normalised (1 LayerNorm, 2 RMSNorm) exactly like the stand-alone kernels
__device__ void mg_stage(const MegaArgs &a, const float *src, int64_t ld, int K, int norm, const float *w, const float *b,
                         float eps, float *xs, float *red) {
    for (int r = 0; r < a.B; r++) {
        const float *xr = src + r * ld;
        float mean = 0.f, rstd = 1.f;
        if (norm) {
            if (norm == 1) {
                float p = 0.f;
                for (int k = threadIdx.x * 4; k < K; k += MG_THREADS * 4) { float4 v = *(const float4 *)(xr + k); p += (v.x + v.y) + (v.z + v.w); }
                mean = mg_block_sum(p, red) / (float)K;
            }
            float q = 0.f;
            for (int k = threadIdx.x * 4; k < K; k += MG_THREADS * 4) {
                float4 v = *(const float4 *)(xr + k);
                float d0 = v.x - mean, d1 = v.y - mean, d2 = v.z - mean, d3 = v.w - mean;
                q += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
            }
            rstd = 1.0f / sqrtf(mg_block_sum(q, red) / (float)K + eps);
        }
        for (int k = threadIdx.x * 4; k < K; k += MG_THREADS * 4) {
            float4 v = *(const float4 *)(xr + k);
            if (norm) {
                float4 lw = w ? *(const float4 *)(w + k) : make_float4(1.f, 1.f, 1.f, 1.f);
                float4 lb = b ? *(const float4 *)(b + k) : make_float4(0.f, 0.f, 0.f, 0.f);
                v.x = __fadd_rn(__fmul_rn(__fmul_rn(v.x - mean, rstd), lw.x), lb.x);
                v.y = __fadd_rn(__fmul_rn(__fmul_rn(v.y - mean, rstd), lw.y), lb.y);
                v.z = __fadd_rn(__fmul_rn(__fmul_rn(v.z - mean, rstd), lw.z), lb.z);
                v.w = __fadd_rn(__fmul_rn(__fmul_rn(v.w - mean, rstd), lw.w), lb.w);
            }
            *(float4 *)(xs + (size_t)r * K + k) = v;
        }
    }
    __syncthreads();
}

// ---- GEMV phases: one warp per item, no block-level synchronisation inside a phase ----
// An item is one output column, or the two columns that belong together: a rotary pair (c, c + 32) of a q / k
// head, or a gate column j and its up column half + j. The lanes stride over K with 128-bit loads (all of a
// column's loads in flight), the B input rows come from shared memory (normalised) or straight from L2, and a
// shuffle reduction leaves the dot products in every lane.
//   layout 0: item = column        1: rotary pair p -> (p/32)*64 + p%32, +32        2: gated j -> j, half + j
__device__ __forceinline__ void mg_item_cols(int layout, int it, int half, int &c0, int &c1) {
    if (layout == 1) { c0 = (it >> 5) * 64 + (it & 31); c1 = c0 + 32; }
    else if (layout == 2) { c0 = it; c1 = half + it; }
    else { c0 = it; c1 = -1; }
}

// L2 prefetch of the weight rows of this warp's first item of the next phase
__device__ __forceinline__ void mg_prefetch(const float *W, int K, int layout, int half, int nitems) {
    const int wg = blockIdx.x * (MG_THREADS / 32) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (wg >= nitems) return;
    int c0, c1;
    mg_item_cols(layout, wg, half, c0, c1);
    const int lines = (K * 4 + 127) / 128;
    for (int l = lane; l < lines; l += 32) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(W + (size_t)c0 * K + l * 32));
        if (c1 >= 0) asm volatile("prefetch.global.L2 [%0];" ::"l"(W + (size_t)c1 * K + l * 32));
    }
}

// d0[r], d1[r] = W[c0] . x[r], W[c1] . x[r] (c1 < 0: one column); x rows are K floats apart at xrow (shared or global)
template <bool TWO>
__device__ __forceinline__ void mg_item_dot(const MegaArgs &a, const float *W, int K, int c0, int c1, const float *xrow, int64_t ldx,
                                            float *d0, float *d1) {
    const int lane = threadIdx.x & 31, K4 = K >> 2;
    const float4 *w0 = (const float4 *)(W + (size_t)c0 * K), *w1 = (const float4 *)(W + (size_t)(TWO ? c1 : c0) * K);
#pragma unroll
    for (int r = 0; r < MG_MAXB; r++) { d0[r] = 0.f; d1[r] = 0.f; }
#pragma unroll 4
    for (int k4 = lane; k4 < K4; k4 += 32) {
        const float4 p = __ldg(w0 + k4);
        float4 q = p;
        if (TWO) q = __ldg(w1 + k4);
#pragma unroll
        for (int r = 0; r < MG_MAXB; r++) {
            if (r < a.B) {
                const float4 xv = *((const float4 *)(xrow + (size_t)r * ldx) + k4);
                d0[r] = fmaf(xv.x, p.x, d0[r]); d0[r] = fmaf(xv.y, p.y, d0[r]); d0[r] = fmaf(xv.z, p.z, d0[r]); d0[r] = fmaf(xv.w, p.w, d0[r]);
                if (TWO) { d1[r] = fmaf(xv.x, q.x, d1[r]); d1[r] = fmaf(xv.y, q.y, d1[r]); d1[r] = fmaf(xv.z, q.z, d1[r]); d1[r] = fmaf(xv.w, q.w, d1[r]); }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < MG_MAXB; r++) {
        if (r < a.B) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                d0[r] += __shfl_xor_sync(0xffffffffu, d0[r], o);
                if (TWO) d1[r] += __shfl_xor_sync(0xffffffffu, d1[r], o);
            }
        }
    }
}

// ---- split-key attention of one (row, kv head, 32-key chunk) by a team of 128 threads; the last chunk of a
// (row, kv head) to finish merges the partials (same scheme as attention_decode.cu) ----
struct MgAttnSmem {
    float qs[MG_MAXG][64];
    float sc[MG_MAXG][MG_KEYS];
    float red[2][MG_MAXG][64];
    float mg[MG_MAXG], lg[MG_MAXG];
    float wsm[MG_MAXSPLIT][MG_MAXG], lsm[MG_MAXSPLIT][MG_MAXG], Lg[MG_MAXG];
    int last;
};
__device__ __forceinline__ void mg_team_sync(int team) { asm volatile("bar.sync %0, %1;" ::"r"(team + 1), "n"(MG_TEAM) : "memory"); }

__device__ void mg_attn_unit(const MegaArgs &a, const MegaLayer &L, int row, int kvh, int sp, int n1, MgAttnSmem &sm, int team, int t) {
    constexpr int HD = 64, DP = 16, GROUPS = 2, KPG = 16;
    const int G = a.H / a.nkv, kvd = a.nkv * HD, Wq = a.C + 2 * kvd;
    const int warp = t >> 5, lane = t & 31;
    const int nsplit = (n1 + MG_KEYS - 1) / MG_KEYS, k0 = sp * MG_KEYS;
    const float *kbase = L.kv + (size_t)row * a.kv_seq_pitch;
    const int64_t ldk = 2 * kvd;
    const float scale = 0.125f;
    for (int i = t; i < G * HD; i += MG_TEAM) { int g = i / HD, d = i % HD; sm.qs[g][d] = a.qkv[(size_t)row * Wq + (kvh * G + g) * HD + d]; }
    mg_team_sync(team);
    {
        const int j = t >> 2, part = t & 3;
        const bool valid = k0 + j < n1;
        float kr[DP];
        if (valid) {
            const float4 *kp = (const float4 *)(kbase + (int64_t)(k0 + j) * ldk + kvh * HD + part * DP);
#pragma unroll
            for (int i = 0; i < DP / 4; i++) { float4 v = kp[i]; kr[4 * i] = v.x; kr[4 * i + 1] = v.y; kr[4 * i + 2] = v.z; kr[4 * i + 3] = v.w; }
        } else {
#pragma unroll
            for (int i = 0; i < DP; i++) kr[i] = 0.f;
        }
        for (int g = 0; g < G; g++) {
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < DP; i++) dot = fmaf(kr[i], sm.qs[g][part * DP + i], dot);
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            if (part == 0) sm.sc[g][j] = valid ? dot * scale : -INFINITY;
        }
    }
    mg_team_sync(team);
    for (int g = warp; g < G; g += MG_TEAM / 32) {
        float s = sm.sc[g][lane], m = s;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float p = (s == -INFINITY) ? 0.f : expf(s - m), l = p;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
        sm.sc[g][lane] = p;
        if (lane == 0) { sm.mg[g] = m; sm.lg[g] = l; }
    }
    mg_team_sync(team);
    {
        const int grp = t / HD, d = t % HD;
        float acc[MG_MAXG], vr[KPG];
#pragma unroll
        for (int g = 0; g < MG_MAXG; g++) acc[g] = 0.f;
#pragma unroll
        for (int jj = 0; jj < KPG; jj++) {
            const int j = grp * KPG + jj;
            vr[jj] = (k0 + j < n1) ? kbase[(int64_t)(k0 + j) * ldk + kvd + kvh * HD + d] : 0.f;
        }
#pragma unroll
        for (int jj = 0; jj < KPG; jj++) {
            const int j = grp * KPG + jj;
#pragma unroll
            for (int g = 0; g < MG_MAXG; g++) if (g < G) acc[g] = fmaf(sm.sc[g][j], vr[jj], acc[g]);
        }
#pragma unroll
        for (int g = 0; g < MG_MAXG; g++) if (g < G) sm.red[grp][g][d] = acc[g];
    }
    mg_team_sync(team);
    float *mine = a.part + ((int64_t)(row * a.nkv + kvh) * a.max_split + sp) * G * (HD + 2);
    for (int i = t; i < G * HD; i += MG_TEAM) {
        int g = i / HD, d = i % HD;
        mine[g * (HD + 2) + 2 + d] = sm.red[0][g][d] + sm.red[1][g][d];
        if (d == 0) { mine[g * (HD + 2)] = sm.mg[g]; mine[g * (HD + 2) + 1] = sm.lg[g]; }
    }
    __threadfence();
    mg_team_sync(team);
    if (t == 0) {
        unsigned old = atomicAdd(a.count + row * a.nkv + kvh, 1u);
        sm.last = (old == (unsigned)(nsplit - 1));
    }
    mg_team_sync(team);
    if (!sm.last) return;
    __threadfence();
    const float *base = a.part + (int64_t)(row * a.nkv + kvh) * a.max_split * G * (HD + 2);
    for (int i = t; i < nsplit * G; i += MG_TEAM) {
        int s = i / G, g = i % G;
        const float *ps = base + ((int64_t)s * G + g) * (HD + 2);
        sm.wsm[s][g] = __ldcg(ps); sm.lsm[s][g] = __ldcg(ps + 1);
    }
    mg_team_sync(team);
    if (t < G) {
        float M = -INFINITY, Ls = 0.f;
        for (int s = 0; s < nsplit; s++) M = fmaxf(M, sm.wsm[s][t]);
        for (int s = 0; s < nsplit; s++) { float w = expf(sm.wsm[s][t] - M); sm.wsm[s][t] = w; Ls = fmaf(sm.lsm[s][t], w, Ls); }
        sm.Lg[t] = Ls;
    }
    mg_team_sync(team);
    for (int i = t; i < G * HD; i += MG_TEAM) {
        int g = i / HD, d = i % HD;
        float O = 0.f;
        int s = 0;
        for (; s + 4 <= nsplit; s += 4) {
            float o0 = __ldcg(base + ((int64_t)(s + 0) * G + g) * (HD + 2) + 2 + d);
            float o1 = __ldcg(base + ((int64_t)(s + 1) * G + g) * (HD + 2) + 2 + d);
            float o2 = __ldcg(base + ((int64_t)(s + 2) * G + g) * (HD + 2) + 2 + d);
            float o3 = __ldcg(base + ((int64_t)(s + 3) * G + g) * (HD + 2) + 2 + d);
            O = fmaf(o0, sm.wsm[s][g], O); O = fmaf(o1, sm.wsm[s + 1][g], O); O = fmaf(o2, sm.wsm[s + 2][g], O); O = fmaf(o3, sm.wsm[s + 3][g], O);
        }
        for (; s < nsplit; s++) O = fmaf(__ldcg(base + ((int64_t)s * G + g) * (HD + 2) + 2 + d), sm.wsm[s][g], O);
        const float Ls = sm.Lg[g];
        a.ctx[(size_t)row * a.C + (kvh * G + g) * HD + d] = Ls > 0.f ? O / Ls : 0.f;
    }
    if (t == 0) a.count[row * a.nkv + kvh] = 0;
}

// ---- the step ----
__global__ void __launch_bounds__(MG_THREADS, 1) k_lm_decode_mega(MegaArgs a) {
    extern __shared__ __align__(16) unsigned char mg_smem[];
    float *xs = (float *)mg_smem;                               // staged input rows [B][K] (GEMV phases)
    MgAttnSmem *asmem = (MgAttnSmem *)mg_smem;                  // four team scratch areas (attention phase)
    __shared__ float bred[MG_THREADS / 32];
    __shared__ unsigned long long s_best[MG_MAXB];
    const int tid = threadIdx.x;
    if (*(volatile int *)a.err) return;                         // an earlier launch timed out: the host will discard the run
    const unsigned base = *a.bar_base;
    unsigned nb = 0;
    const int v = *a.step_d;                                    // tokens finalised so far
    const int pos = a.np - 1 + v;                               // absolute position of this step's token
    const int C = a.C, HD = 64, kvd = a.nkv * HD, Wq = C + 2 * kvd, I = a.I;
    const int warp = tid >> 5, lane = tid & 31;
    const int wg = blockIdx.x * (MG_THREADS / 32) + warp, TW = gridDim.x * (MG_THREADS / 32);
    const int n_qkv = a.rope ? Wq / 2 : Wq, l_qkv = a.rope ? 1 : 0;      // items of the QKV phase
    // gated MLP: item j = (gate j, up j); plain MLP: item j = columns (j, I/2 + j), two per warp so one round covers it
    const int n_fc = a.gated ? I : I / 2, l_fc = 2, h_fc = a.gated ? I : I / 2;

    // embed: x[r] = wte[id] (+ wpe[pos])
    for (int i = blockIdx.x * MG_THREADS + tid; i < a.B * C; i += gridDim.x * MG_THREADS) {
        int r = i / C, c = i % C;
        float e = a.wte[(size_t)a.ids[r] * C + c];
        if (a.wpe) e = __fadd_rn(e, a.wpe[(size_t)a.posmat[(size_t)pos * a.B + r] * C + c]);
        a.x[i] = e;
    }
    mg_prefetch(a.layers[0].qkvw, C, l_qkv, 0, n_qkv);
    mg_barrier(a, base, nb);

    for (int li = 0; li < a.NL; li++) {
        const MegaLayer L = a.layers[li];
        // ---- norm + QKV, rotary pairs, K|V into the cache ----
        mg_stage(a, a.x, C, C, a.norm, L.ln1w, L.ln1b, a.eps, xs, bred);
        for (int it = wg; it < n_qkv; it += TW) {
            int c0, c1;
            mg_item_cols(l_qkv, it, 0, c0, c1);
            float d0[MG_MAXB], d1[MG_MAXB];
            if (a.rope) mg_item_dot<true>(a, L.qkvw, C, c0, c1, xs, C, d0, d1);
            else mg_item_dot<false>(a, L.qkvw, C, c0, c1, xs, C, d0, d1);
            if (lane < a.B) {
                const int r = lane;
                float y0 = 0.f, y1 = 0.f;
#pragma unroll
                for (int q = 0; q < MG_MAXB; q++) if (q == r) { y0 = d0[q]; y1 = d1[q]; }
                if (L.qkvb) { y0 += L.qkvb[c0]; if (a.rope) y1 += L.qkvb[c1]; }
                if (a.rope && c0 < C + kvd) {                    // q and k heads rotate, v does not
                    const int d = c0 & 63;
                    const size_t tp = (size_t)a.posmat[(size_t)pos * a.B + r] * HD;
                    const float z0 = __fadd_rn(__fmul_rn(y0, a.cosb[tp + d]), __fmul_rn(-y1, a.sinb[tp + d]));
                    const float z1 = __fadd_rn(__fmul_rn(y1, a.cosb[tp + d + 32]), __fmul_rn(y0, a.sinb[tp + d + 32]));
                    y0 = z0; y1 = z1;
                }
                float *dst = L.kv + (size_t)r * a.kv_seq_pitch + (size_t)pos * 2 * kvd;
                a.qkv[(size_t)r * Wq + c0] = y0;
                if (c0 >= C) dst[c0 - C] = y0;
                if (a.rope) { a.qkv[(size_t)r * Wq + c1] = y1; if (c1 >= C) dst[c1 - C] = y1; }
            }
        }
        mg_prefetch(L.ow, C, 0, 0, C);
        {   // the cached K|V rows of this CTA's attention units: one 128-byte line per thread of the team
            const int team = tid / MG_TEAM, t = tid % MG_TEAM, u = blockIdx.x * MG_TEAMS + team;
            if (u < a.B * a.nkv * a.max_split) {
                const int sp = u % a.max_split, kvh = (u / a.max_split) % a.nkv, row = u / (a.max_split * a.nkv);
                const int key = sp * MG_KEYS + (t >> 2);
                if (key < pos)                                      // rows of earlier steps only: this step's row is being written
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(L.kv + (size_t)row * a.kv_seq_pitch + (size_t)key * 2 * kvd +
                                                                      ((t >> 1) & 1) * kvd + kvh * HD + (t & 1) * 32));
            }
        }
        mg_barrier(a, base, nb);
        // ---- attention over the cache (this step's key included) ----
        {
            const int team = tid / MG_TEAM, t = tid % MG_TEAM;
            const int nunits = a.B * a.nkv * a.max_split;
            for (int u = blockIdx.x * MG_TEAMS + team; u < nunits; u += gridDim.x * MG_TEAMS) {
                const int sp = u % a.max_split, kvh = (u / a.max_split) % a.nkv, row = u / (a.max_split * a.nkv);
                const int n1 = a.lenmat[(size_t)pos * a.B + row];
                if (sp * MG_KEYS < n1) mg_attn_unit(a, L, row, kvh, sp, n1, asmem[team], team, t);
            }
        }
        mg_barrier(a, base, nb);
        // ---- output projection + residual (input rows straight from L2) ----
        for (int it = wg; it < C; it += TW) {
            float d0[MG_MAXB], d1[MG_MAXB];
            mg_item_dot<false>(a, L.ow, C, it, -1, a.ctx, C, d0, d1);
            if (lane < a.B) {
                float y = 0.f;
#pragma unroll
                for (int q = 0; q < MG_MAXB; q++) if (q == lane) y = d0[q];
                if (L.ob) y += L.ob[it];
                a.x[(size_t)lane * C + it] = y + a.x[(size_t)lane * C + it];
            }
        }
        mg_prefetch(L.fcw, C, l_fc, h_fc, n_fc);
        mg_barrier(a, base, nb);
        // ---- norm + MLP up (+ gated product) ----
        mg_stage(a, a.x, C, C, a.norm, L.ln2w, L.ln2b, a.eps, xs, bred);
        for (int it = wg; it < n_fc; it += TW) {
            float d0[MG_MAXB], d1[MG_MAXB];
            mg_item_dot<true>(a, L.fcw, C, it, h_fc + it, xs, C, d0, d1);
            if (lane < a.B) {
                float g = 0.f, up = 0.f;
#pragma unroll
                for (int q = 0; q < MG_MAXB; q++) if (q == lane) { g = d0[q]; up = d1[q]; }
                if (L.fcb) { g += L.fcb[it]; up += L.fcb[h_fc + it]; }
                if (a.gated) a.h[(size_t)lane * I + it] = __fmul_rn(mg_act(g, a.act), up);
                else { a.h[(size_t)lane * I + it] = mg_act(g, a.act); a.h[(size_t)lane * I + h_fc + it] = mg_act(up, a.act); }
            }
        }
        mg_prefetch(L.pw, I, 0, 0, C);
        mg_barrier(a, base, nb);
        // ---- MLP down + residual ----
        for (int it = wg; it < C; it += TW) {
            float d0[MG_MAXB], d1[MG_MAXB];
            mg_item_dot<false>(a, L.pw, I, it, -1, a.h, I, d0, d1);
            if (lane < a.B) {
                float y = 0.f;
#pragma unroll
                for (int q = 0; q < MG_MAXB; q++) if (q == lane) y = d0[q];
                if (L.pb) y += L.pb[it];
                a.x[(size_t)lane * C + it] = y + a.x[(size_t)lane * C + it];
            }
        }
        if (li + 1 < a.NL) mg_prefetch(a.layers[li + 1].qkvw, C, l_qkv, 0, n_qkv);
        else mg_prefetch(a.wte, C, 0, 0, a.V);
        mg_barrier(a, base, nb);
    }
    // ---- final norm, vocabulary projection, greedy pick ----
    mg_stage(a, a.x, C, C, a.norm, a.lnfw, a.lnfb, a.eps_f, xs, bred);
    if (tid < MG_MAXB) s_best[tid] = 0;
    __syncthreads();
    {
        unsigned long long best = 0;
        for (int it = wg; it < a.V; it += TW) {
            float d0[MG_MAXB], d1[MG_MAXB];
            mg_item_dot<false>(a, a.wte, C, it, -1, xs, C, d0, d1);
            if (lane < a.B) {
                float y = 0.f;
#pragma unroll
                for (int q = 0; q < MG_MAXB; q++) if (q == lane) y = d0[q];
                a.logits[(size_t)lane * a.V + it] = y;
                unsigned ub = __float_as_uint(y);
                ub = (ub & 0x80000000u) ? ~ub : (ub | 0x80000000u);
                const unsigned long long pk = ((unsigned long long)ub << 32) | (0xffffffffu - (unsigned)it);
                if (pk > best) best = pk;
            }
        }
        if (a.greedy && lane < a.B && best) atomicMax(&s_best[lane], best);
    }
    __syncthreads();
    if (a.greedy && tid < a.B && s_best[tid]) atomicMax(a.amax + tid, s_best[tid]);
    mg_barrier(a, base, nb);
    if (blockIdx.x == 0) {
        if (a.greedy && tid < a.B) {                             // close the step: token v of every row
            const int tkn = (int)(0xffffffffu - (unsigned)(a.amax[tid] & 0xffffffffull));
            a.out[(size_t)tid * a.n_new + v] = tkn;
            a.ids_out[tid] = tkn;
            a.amax[tid] = 0;
        }
        __syncthreads();
        if (tid == 0) {
            if (a.greedy) *a.step_d = v + 1;
            *a.bar_base = base + nb * gridDim.x;                 // where the counter stands for the next launch
        }
    }
}

// Off unless asked for (ncmb_set_lm_persistent(1) or NCM_B200_LM_PERSISTENT=1): measured on GPT-2 124M, batch 1,
// the persistent kernel takes 0.51 ms per token against 0.47 ms for the graph-replayed kernel chain -- its 62
// grid barriers cost 2-4 us each, as much as the launches they replace.
static int g_lm_persistent = -1;
void lm_mega_enable(int on) { g_lm_persistent = on ? 1 : 0; }
bool lm_mega_eligible(int B, int hd, int C, int I, bool qk_norm) {
    if (g_lm_persistent < 0) g_lm_persistent = getenv("NCM_B200_LM_PERSISTENT") ? 1 : 0;
    return g_lm_persistent == 1 && B >= 1 && B <= MG_MAXB && hd == 64 && (C % 64) == 0 && (I % 8) == 0 && !qk_norm;
}

size_t lm_mega_smem(const MegaArgs &a) {
    size_t rows = (size_t)a.B * (a.C > a.I ? a.C : a.I) * 4;
    size_t attn = sizeof(MgAttnSmem) * MG_TEAMS;
    return (rows > attn ? rows : attn) + 16;
}

void lm_mega_launch(const MegaArgs &a) {
    const size_t smem = lm_mega_smem(a);
    static size_t attr = 0;
    if (smem > attr) {
        CUDA_CHECK(cudaFuncSetAttribute(k_lm_decode_mega, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr = smem;
    }
    int per_sm = 0;
    CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_lm_decode_mega, MG_THREADS, smem));
    if (per_sm < 1) fatal("lm_mega: the persistent decode kernel does not fit an SM (%zu bytes of shared memory)", smem);
    MegaArgs arg = a;
    void *params[] = {&arg};
    ProfScope ps(NCMB_K_GEMM, 0, 0);
    cudaError_t e = cudaLaunchCooperativeKernel((const void *)k_lm_decode_mega, dim3(ctx().sm_count), dim3(MG_THREADS), params, smem, stream());
    if (e != cudaSuccess) fatal("lm_mega: cooperative launch failed: %s", cudaGetErrorString(e));
    ctx().launches++;
}

} // namespace ncmb
