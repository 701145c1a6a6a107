// Few-query attention: ONE query per sequence row against that row's K/V cache (the decoder-LM token loop,
// reference src/gpt2.c:92 / src/qwen.c:121 run with a KV cache instead of recomputing), or up to four queries
// per row against the cached prefix plus the row's own new tokens (the first levels of the NCP generate,
// reference src/ncp.c:990: level sizes 1 and 4).
//
// With one query there is nothing to tile over queries, so the keys are split instead: one CTA per
// (32-key chunk, kv head, row) computes the chunk's scores for every query head that shares the kv
// head (K and V are read once per group), a local softmax and the partial context, and writes
// (max, sum, context[hd]) per head to scratch. The last CTA of a (row, kv head) to finish -- an
// atomic counter tells it -- merges the partials with the usual log-sum-exp rescaling and writes the
// context row. A batch-1, 12-head step with 300 cached keys thus runs on ~120 CTAs instead of 12. With many
// rows a CTA takes several consecutive chunks (running maximum and sum), and a CTA that sees all keys of its
// row writes the context directly.
//
// step_d: optional device counter. When set, row lengths are read from k1_len + (*step_d) * len_step,
// so one captured CUDA graph serves every decode step.
#include "common.cuh"
#include "split.cuh"

#include <algorithm>

namespace ncmb {

constexpr int AD_KEYS = 32, AD_THREADS = 128, AD_MAXSPLIT = 64;   // up to 2048 keys per row
constexpr int AD_MAXG = 16;        // (query, head) pairs of one kv group handled together: G * queries per row <= 16

struct AttnDecDev {
    const float *q; int64_t ldq;
    const float *k, *v; int64_t ldk;
    const float *k2, *v2; int64_t ldk2; const int *k2_start;      // optional second key segment (this pass's own tokens)
    float *out; float *out_lo; int out_fmt; int64_t ldo;
    const int *q_start, *k_start, *k_len;
    const int *step_d; int64_t len_step;
    int H, Hkv, max_split, cps;
    int hs;                            // warp-per-chunk kernel: warps that share a chunk's (query, head) pairs
    float scale;
    float *part; unsigned *count;
};

// GM: compile-time bound on the (query, head) pairs of a kv group (1, 4, 8 or 16). Every loop over them is unrolled
// to GM, so a one-head-per-kv-head model (GPT-2) does not issue the 16-wide context step of a grouped one.
template <int HD, int GM>
__global__ void __launch_bounds__(AD_THREADS) k_attention_decode(AttnDecDev a) {
    constexpr int DP = HD / 4;                         // dims per thread in the score step (4 threads per key)
    constexpr int QP = DP + 4;                         // pitch of a quarter in qs: the four quarters land in distinct banks
    constexpr int GROUPS = AD_THREADS / HD > 0 ? AD_THREADS / HD : 1;   // key groups in the PV step
    constexpr int KPG = AD_KEYS / GROUPS;
    __shared__ __align__(16) float qs[GM][4 * QP];
    __shared__ __align__(16) float sc[AD_KEYS][GM];    // scores, then probabilities, of the chunk: [key][head]
    __shared__ float red[GROUPS][GM][HD];
    __shared__ float mg[GM], lg[GM], alpha[GM];
    __shared__ int s_last;
    const int row = blockIdx.z, kvh = blockIdx.y, sp = blockIdx.x;
    const int Gh = a.H / a.Hkv;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_launch_dependents();          // programmatic dependent launch: the successor may start launching now,
    pdl_wait();                       // and nothing the predecessor wrote is read before this point
    const int *lens = a.k_len ? a.k_len + (a.step_d ? (int64_t)(*a.step_d) * a.len_step : 0) : nullptr;
    const int k00 = a.k_start[row], n1s = lens ? lens[row] : a.k_start[row + 1] - k00;
    const int k20 = a.k2_start ? a.k2_start[row] : 0, n2s = a.k2_start ? a.k2_start[row + 1] - k20 : 0;
    const int n1 = n1s + n2s;                          // keys of both segments, segment 1 first
    const int nchunks = (n1 + AD_KEYS - 1) / AD_KEYS;
    const int nsplit = (nchunks + a.cps - 1) / a.cps;   // CTAs that share the row's keys, cps 32-key chunks each
    if (sp >= nsplit) return;
    const int k0 = sp * a.cps * AD_KEYS;
    const int nch = min(a.cps, nchunks - sp * a.cps);
    const int q0 = a.q_start[row], nq = a.q_start[row + 1] - q0;
    const int G = Gh * nq;                             // virtual heads: vh = g * nq + qi
    // row pointer of key j of the row (either segment)
    auto krow = [&](int j) -> const float * {
        return j < n1s ? a.k + (int64_t)(k00 + j) * a.ldk : a.k2 + (int64_t)(k20 + j - n1s) * a.ldk2;
    };
    auto vrow = [&](int j) -> const float * {
        return j < n1s ? a.v + (int64_t)(k00 + j) * a.ldk : a.v2 + (int64_t)(k20 + j - n1s) * a.ldk2;
    };

    for (int i = tid; i < G * HD; i += AD_THREADS) {
        int vh = i / HD, d = i % HD;
        qs[vh][(d / DP) * QP + d % DP] = a.q[(int64_t)(q0 + vh % nq) * a.ldq + (kvh * Gh + vh / nq) * HD + d];
    }
    if (tid < GM) { mg[tid] = -INFINITY; lg[tid] = 0.f; alpha[tid] = 0.f; }
    for (int i = tid; i < AD_KEYS * GM; i += AD_THREADS) (&sc[0][0])[i] = 0.f;     // heads past G stay 0 in the context step
    // The CTA walks its cps chunks with a running maximum / sum per head (the usual rescaling when the maximum
    // grows). Loads run ahead of the arithmetic: the V elements of a chunk are requested before its scores are
    // formed, the K rows of the next chunk before the softmax of this one.
    const int sj = tid >> 2, spart = tid & 3;             // score step: four threads per key, a quarter of the head dim each
    const int grp = tid / HD, d = tid % HD;               // context step: thread = (key group, dim)
    float kr[DP];
    auto load_k = [&](int kbase) {
        if (kbase + sj < n1) {
            const float4 *kp = (const float4 *)(krow(kbase + sj) + kvh * HD + spart * DP);
#pragma unroll
            for (int i = 0; i < DP / 4; i++) { float4 t = kp[i]; kr[4 * i] = t.x; kr[4 * i + 1] = t.y; kr[4 * i + 2] = t.z; kr[4 * i + 3] = t.w; }
        } else {
#pragma unroll
            for (int i = 0; i < DP; i++) kr[i] = 0.f;
        }
    };
    float acc[GM];
#pragma unroll
    for (int g = 0; g < GM; g++) acc[g] = 0.f;
    load_k(k0);
    __syncthreads();
    for (int c = 0; c < nch; c++) {
        const int kb = k0 + c * AD_KEYS;
        float vr[KPG];                                   // all V loads of this thread in flight together
        if (grp < GROUPS) {
            if (kb + AD_KEYS <= n1s) {                    // the whole chunk lies in the first segment: one base, fixed strides
                const float *vb = a.v + (int64_t)(k00 + kb + grp * KPG) * a.ldk + kvh * HD + d;
#pragma unroll
                for (int jj = 0; jj < KPG; jj++) vr[jj] = vb[(int64_t)jj * a.ldk];
            } else {
#pragma unroll
                for (int jj = 0; jj < KPG; jj++) {
                    const int j = grp * KPG + jj;
                    vr[jj] = (kb + j < n1) ? vrow(kb + j)[kvh * HD + d] : 0.f;
                }
            }
        }
        {   // scores of the chunk
            const bool valid = kb + sj < n1;
#pragma unroll
            for (int g = 0; g < GM; g++) {
                if (g < G) {                              // warp-uniform
                    const float4 *qp = (const float4 *)&qs[g][spart * QP];
                    float dot = 0.f;
#pragma unroll
                    for (int i = 0; i < DP / 4; i++) {
                        const float4 t = qp[i];
                        dot = fmaf(kr[4 * i], t.x, dot); dot = fmaf(kr[4 * i + 1], t.y, dot);
                        dot = fmaf(kr[4 * i + 2], t.z, dot); dot = fmaf(kr[4 * i + 3], t.w, dot);
                    }
                    dot += __shfl_xor_sync(0xffffffffu, dot, 1);
                    dot += __shfl_xor_sync(0xffffffffu, dot, 2);
                    if (spart == 0) sc[sj][g] = valid ? dot * a.scale : -INFINITY;
                }
            }
        }
        if (c + 1 < nch) load_k(kb + AD_KEYS);
        __syncthreads();
        for (int g = warp; g < G; g += AD_THREADS / 32) {   // chunk softmax against the running maximum, one warp per head
            float s = sc[lane][g];
            float m = s;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            const float mold = mg[g];
            m = fmaxf(m, mold);
            float p = (s == -INFINITY) ? 0.f : expf(s - m);
            float l = p;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
            sc[lane][g] = p;
            __syncwarp();
            if (lane == 0) {
                const float al = (mold == -INFINITY) ? 0.f : expf(mold - m);
                alpha[g] = al; mg[g] = m; lg[g] = fmaf(lg[g], al, l);
            }
        }
        __syncthreads();
        if (grp < GROUPS) {
#pragma unroll
            for (int g = 0; g < GM; g++) acc[g] *= alpha[g];
#pragma unroll
            for (int jj = 0; jj < KPG; jj++) {
                const int j = grp * KPG + jj;
                if constexpr (GM % 4 == 0) {
#pragma unroll
                    for (int g4 = 0; g4 < GM / 4; g4++) {
                        const float4 pr = *(const float4 *)&sc[j][4 * g4];     // the same address for the whole warp: a broadcast
                        acc[4 * g4] = fmaf(pr.x, vr[jj], acc[4 * g4]); acc[4 * g4 + 1] = fmaf(pr.y, vr[jj], acc[4 * g4 + 1]);
                        acc[4 * g4 + 2] = fmaf(pr.z, vr[jj], acc[4 * g4 + 2]); acc[4 * g4 + 3] = fmaf(pr.w, vr[jj], acc[4 * g4 + 3]);
                    }
                } else {
#pragma unroll
                    for (int g = 0; g < GM; g++) acc[g] = fmaf(sc[j][g], vr[jj], acc[g]);
                }
            }
        }
        __syncthreads();                                  // sc and alpha are rewritten by the next chunk
    }
    if (grp < GROUPS) {
#pragma unroll
        for (int g = 0; g < GM; g++) red[grp][g][d] = acc[g];
    }
    __syncthreads();
    if (nsplit == 1) {                                    // the CTA saw every key of the row: no partials, no merge
        for (int i = tid; i < G * HD; i += AD_THREADS) {
            int g = i / HD, dd = i % HD;
            float o = 0.f;
#pragma unroll
            for (int r = 0; r < GROUPS; r++) o += red[r][g][dd];
            const float L = lg[g];
            const float r = L > 0.f ? o / L : 0.f;
            const int64_t at = (int64_t)(q0 + g % nq) * a.ldo + (kvh * Gh + g / nq) * HD + dd;
            if (a.out_lo) store_split1(a.out, a.out_lo, at, r, a.out_fmt);
            else a.out[at] = r;
        }
        return;
    }
    float *mine = a.part + ((int64_t)(row * a.Hkv + kvh) * a.max_split + sp) * AD_MAXG * (HD + 2);
    for (int i = tid; i < G * HD; i += AD_THREADS) {
        int g = i / HD, d = i % HD;
        float o = 0.f;
#pragma unroll
        for (int r = 0; r < GROUPS; r++) o += red[r][g][d];
        mine[g * (HD + 2) + 2 + d] = o;
        if (d == 0) { mine[g * (HD + 2)] = mg[g]; mine[g * (HD + 2) + 1] = lg[g]; }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        unsigned old = atomicAdd(a.count + row * a.Hkv + kvh, 1u);
        s_last = (old == (unsigned)(nsplit - 1));
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // merge: the chunk partials of this (row, kv head), read through L2. Maxima and sums first (one load per
    // thread, all in flight together), then the rescaling weights once per head, then the context columns
    // with independent loads -- a chain of dependent L2 round trips per split would dominate the kernel.
    __shared__ float wsm[AD_MAXSPLIT][GM], lsm[AD_MAXSPLIT][GM], Lg[GM];
    const float *base = a.part + (int64_t)(row * a.Hkv + kvh) * a.max_split * AD_MAXG * (HD + 2);
    for (int i = tid; i < nsplit * G; i += AD_THREADS) {
        int s = i / G, g = i % G;
        const float *ps = base + ((int64_t)s * AD_MAXG + g) * (HD + 2);
        wsm[s][g] = __ldcg(ps); lsm[s][g] = __ldcg(ps + 1);
    }
    __syncthreads();
    if (tid < G) {
        float M = -INFINITY, L = 0.f;
        for (int s = 0; s < nsplit; s++) M = fmaxf(M, wsm[s][tid]);
        for (int s = 0; s < nsplit; s++) { float w = expf(wsm[s][tid] - M); wsm[s][tid] = w; L = fmaf(lsm[s][tid], w, L); }
        Lg[tid] = L;
    }
    __syncthreads();
    for (int i = tid; i < G * HD; i += AD_THREADS) {
        int g = i / HD, d = i % HD;
        float O = 0.f;
        int s = 0;
        for (; s + 4 <= nsplit; s += 4) {
            float o0 = __ldcg(base + ((int64_t)(s + 0) * AD_MAXG + g) * (HD + 2) + 2 + d);
            float o1 = __ldcg(base + ((int64_t)(s + 1) * AD_MAXG + g) * (HD + 2) + 2 + d);
            float o2 = __ldcg(base + ((int64_t)(s + 2) * AD_MAXG + g) * (HD + 2) + 2 + d);
            float o3 = __ldcg(base + ((int64_t)(s + 3) * AD_MAXG + g) * (HD + 2) + 2 + d);
            O = fmaf(o0, wsm[s][g], O); O = fmaf(o1, wsm[s + 1][g], O); O = fmaf(o2, wsm[s + 2][g], O); O = fmaf(o3, wsm[s + 3][g], O);
        }
        for (; s < nsplit; s++) O = fmaf(__ldcg(base + ((int64_t)s * AD_MAXG + g) * (HD + 2) + 2 + d), wsm[s][g], O);
        const float L = Lg[g];
        const float r = L > 0.f ? O / L : 0.f;
        const int64_t at = (int64_t)(q0 + g % nq) * a.ldo + (kvh * Gh + g / nq) * HD + d;
        if (a.out_lo) store_split1(a.out, a.out_lo, at, r, a.out_fmt);
        else a.out[at] = r;
    }
    if (tid == 0) a.count[row * a.Hkv + kvh] = 0;          // ready for the next launch
}

// ---- head dim 64: one WARP per (32-key chunk, group of heads) ----
// The kernel above gives every 32-key chunk a CTA, three block-wide barriers per chunk, and merges all chunk
// partials of a row through global memory; at one sequence that chain of barriers and L2 round trips is the kernel
// (16 us per layer for 800 cached keys of the 14-query-head / 2-kv-head shape). Here a warp works alone on 32 keys
// and up to GMW of the kv group's (query, head) pairs: the lane holding key j forms that key's scores (q broadcast
// from shared memory), the softmax statistics of the chunk are warp shuffles, and for O += P V the lanes switch to
// owning two output dimensions each while the probabilities travel by shuffle -- K and V rows are requested
// before anything is computed and no barrier is needed until the warps' partials (maximum, sum, context) meet in
// shared memory. A kv group with more pairs than one warp takes is shared out over `hs` warps per chunk (they read
// the same K and V rows, out of L1), so a warp's arithmetic stays short. A CTA covers `blockDim / 32 / hs` chunks;
// one partial per CTA goes to global memory, and only when the row needs more than one CTA.
constexpr int ADW_MAXC = 8;            // chunks per CTA at most

template <int GMW>
__global__ void __launch_bounds__(256) k_attention_dec_warp(AttnDecDev a) {
    constexpr int HD = 64, GA = AD_MAXG;
    __shared__ __align__(16) float qs[GA][HD];
    __shared__ float pm[ADW_MAXC][GA], pl[ADW_MAXC][GA], wg[ADW_MAXC][GA];
    __shared__ __align__(8) float po[ADW_MAXC][GA][HD];
    __shared__ float Mg[GA], Lg[GA];
    __shared__ int s_last;
    const int row = blockIdx.z, kvh = blockIdx.y, sp = blockIdx.x;
    const int Gh = a.H / a.Hkv;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hs = a.hs, cpc = (blockDim.x >> 5) / hs;        // warps per chunk, chunks per CTA
    const int cw = warp / hs, hg = warp - cw * hs;
    pdl_launch_dependents();
    pdl_wait();
    const int *lens = a.k_len ? a.k_len + (a.step_d ? (int64_t)(*a.step_d) * a.len_step : 0) : nullptr;
    const int k00 = a.k_start[row], n1s = lens ? lens[row] : a.k_start[row + 1] - k00;
    const int k20 = a.k2_start ? a.k2_start[row] : 0, n2s = a.k2_start ? a.k2_start[row + 1] - k20 : 0;
    const int n1 = n1s + n2s;
    const int per_cta = cpc * 32;
    const int nsplit = (n1 + per_cta - 1) / per_cta;
    if (sp >= nsplit) return;
    const int kw = sp * per_cta + cw * 32;                    // first key of this warp's chunk
    const int q0 = a.q_start[row], nq = a.q_start[row + 1] - q0;
    const int G = Gh * nq;                                    // virtual heads: vh = g * nq + qi
    const int g0 = hg * GMW;                                  // this warp's heads: [g0, g0 + GMW) below G
    auto krow = [&](int j) -> const float * {
        return j < n1s ? a.k + (int64_t)(k00 + j) * a.ldk : a.k2 + (int64_t)(k20 + j - n1s) * a.ldk2;
    };
    auto vrow = [&](int j) -> const float * {
        return j < n1s ? a.v + (int64_t)(k00 + j) * a.ldk : a.v2 + (int64_t)(k20 + j - n1s) * a.ldk2;
    };
    for (int i = tid; i < G * HD; i += blockDim.x) {
        const int vh = i / HD, d = i % HD;
        qs[vh][d] = a.q[(int64_t)(q0 + vh % nq) * a.ldq + (kvh * Gh + vh / nq) * HD + d];
    }
    // every load of the chunk is requested now: the lane's key row, and for the context step the two dimensions
    // (2 lane, 2 lane + 1) of all 32 value rows
    const bool valid = kw + lane < n1;
    float4 kr[HD / 4];
    {
        const float4 *kp = (const float4 *)(krow(valid ? kw + lane : 0) + kvh * HD);
#pragma unroll
        for (int i = 0; i < HD / 4; i++) kr[i] = valid ? kp[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float2 vv[32];
#pragma unroll
    for (int jj = 0; jj < 32; jj++)
        vv[jj] = (kw + jj < n1) ? *(const float2 *)(vrow(kw + jj) + kvh * HD + 2 * lane) : make_float2(0.f, 0.f);
    __syncthreads();
    float s[GMW];
#pragma unroll
    for (int gi = 0; gi < GMW; gi++) {
        s[gi] = 0.f;
        const int g = g0 + gi;
        if (g < G) {                                          // warp-uniform
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < HD / 4; i++) {
                const float4 t = *(const float4 *)&qs[g][4 * i];   // one address for the whole warp: a broadcast
                dot = fmaf(kr[i].x, t.x, dot); dot = fmaf(kr[i].y, t.y, dot); dot = fmaf(kr[i].z, t.z, dot); dot = fmaf(kr[i].w, t.w, dot);
            }
            const float sc = valid ? dot * a.scale : -INFINITY;
            float m = sc;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            const float p = (sc == -INFINITY) ? 0.f : expf(sc - m);
            float l = p;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
            s[gi] = p;
            if (lane == 0) { pm[cw][g] = m; pl[cw][g] = l; }
        }
    }
    float2 acc[GMW];
#pragma unroll
    for (int gi = 0; gi < GMW; gi++) acc[gi] = make_float2(0.f, 0.f);
#pragma unroll
    for (int jj = 0; jj < 32; jj++) {
#pragma unroll
        for (int gi = 0; gi < GMW; gi++) {
            const float pj = __shfl_sync(0xffffffffu, s[gi], jj);
            acc[gi].x = fmaf(pj, vv[jj].x, acc[gi].x); acc[gi].y = fmaf(pj, vv[jj].y, acc[gi].y);
        }
    }
#pragma unroll
    for (int gi = 0; gi < GMW; gi++)
        if (g0 + gi < G) *(float2 *)&po[cw][g0 + gi][2 * lane] = acc[gi];
    __syncthreads();
    // ---- the chunks' partials meet: maximum and weights per head, then the context columns ----
    if (tid < G) {
        float M = -INFINITY, L = 0.f;
        for (int w = 0; w < cpc; w++) M = fmaxf(M, pm[w][tid]);
        for (int w = 0; w < cpc; w++) {
            const float e = (pm[w][tid] == -INFINITY) ? 0.f : expf(pm[w][tid] - M);
            wg[w][tid] = e; L = fmaf(pl[w][tid], e, L);
        }
        Mg[tid] = M; Lg[tid] = L;
    }
    __syncthreads();
    float *mine = a.part + ((int64_t)(row * a.Hkv + kvh) * a.max_split + sp) * AD_MAXG * (HD + 2);
    for (int i = tid; i < G * HD; i += blockDim.x) {
        const int g = i / HD, d = i % HD;
        float O = 0.f;
        for (int w = 0; w < cpc; w++) O = fmaf(po[w][g][d], wg[w][g], O);
        if (nsplit == 1) {
            const float L = Lg[g];
            const float r = L > 0.f ? O / L : 0.f;
            const int64_t at = (int64_t)(q0 + g % nq) * a.ldo + (kvh * Gh + g / nq) * HD + d;
            if (a.out_lo) store_split1(a.out, a.out_lo, at, r, a.out_fmt);
            else a.out[at] = r;
        } else {
            mine[g * (HD + 2) + 2 + d] = O;
            if (d == 0) { mine[g * (HD + 2)] = Mg[g]; mine[g * (HD + 2) + 1] = Lg[g]; }
        }
    }
    if (nsplit == 1) return;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        unsigned old = atomicAdd(a.count + row * a.Hkv + kvh, 1u);
        s_last = (old == (unsigned)(nsplit - 1));
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // the last CTA of the (row, kv head) merges the CTAs' partials (a handful: 64 to 256 keys each); the weights of a
    // partial are recomputed where they are used (an exponential per load) rather than staged
    const float *base = a.part + (int64_t)(row * a.Hkv + kvh) * a.max_split * AD_MAXG * (HD + 2);
    if (tid < G) {
        float M = -INFINITY, L = 0.f;
        for (int x = 0; x < nsplit; x++) M = fmaxf(M, __ldcg(base + ((int64_t)x * AD_MAXG + tid) * (HD + 2)));
        for (int x = 0; x < nsplit; x++) {
            const float *ps = base + ((int64_t)x * AD_MAXG + tid) * (HD + 2);
            L = fmaf(__ldcg(ps + 1), expf(__ldcg(ps) - M), L);
        }
        Mg[tid] = M; Lg[tid] = L;
    }
    __syncthreads();
    for (int i = tid; i < G * HD; i += blockDim.x) {
        const int g = i / HD, d = i % HD;
        const float M = Mg[g];
        float O = 0.f;
        for (int x = 0; x < nsplit; x++) {
            const float *ps = base + ((int64_t)x * AD_MAXG + g) * (HD + 2);
            O = fmaf(__ldcg(ps + 2 + d), expf(__ldcg(ps) - M), O);
        }
        const float L = Lg[g];
        const float r = L > 0.f ? O / L : 0.f;
        const int64_t at = (int64_t)(q0 + g % nq) * a.ldo + (kvh * Gh + g / nq) * HD + d;
        if (a.out_lo) store_split1(a.out, a.out_lo, at, r, a.out_fmt);
        else a.out[at] = r;
    }
    if (tid == 0) a.count[row * a.Hkv + kvh] = 0;
}

// ---- head dim 64, many (query, head) pairs per kv group: one WARP per run of 32-key chunks, products on mma.sync ----
// With 7 to 16 (query, head) pairs per kv group (grouped-query decode steps of many sequences, the 4-token NCP
// level) the kernels above spend their time re-reading q and the probabilities from shared memory, one load per four
// multiply-adds. Here the pairs are the 16 rows of an m16n8k8 tensor-core tile: S[16 x 32] = Q[16 x 64] K^T and
// O[16 x 64] += P[16 x 32] V per 32-key chunk, each product as three TF32 MMAs over hi/lo splits (fp32-grade, as
// the three-pass GEMM engine). Every K and V element of a chunk is loaded from global memory exactly once, straight
// into the lane that needs it as a B fragment, sixteen bytes at a time: which head dimension sits at which k position
// of a score MMA, and which at which column of an output tile, is free as long as both operands agree, so the
// positions are chosen to make a lane's elements contiguous (k-step 2 m + h holds dims 16 m + 4 tig + 2 h and + 1 at
// positions tig and tig + 4; column gid of output tile j is dim 8 gid + j). The hi / lo halves of Q sit in shared
// memory (a lane's A fragments of two k-steps are four 16-byte reads); the
// probabilities cross from the accumulator layout to the A-fragment layout through 2 KB of shared memory per warp.
// Loads run a phase ahead of the arithmetic (the next chunk's keys are requested when the score MMAs are done with
// their registers, the chunk's values before its score MMAs).
// A warp walks `cps` chunks with a running maximum and sum per row; the four warps of a CTA take every fourth chunk
// of the CTA's stretch of the (row, kv head)'s keys and their partials meet in shared memory; one partial per CTA goes to
// global memory, and only when the row needs more than one CTA (last CTA merges, as above). The tcgen05 path needs
// 64 rows at least: for 16 it would idle three quarters of the tile.
constexpr int ADM_WARPS = 4;
#ifndef ADM_MINB
#define ADM_MINB 2
#endif
__device__ __forceinline__ void adm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void adm_split(float v, uint32_t &hi, uint32_t &lo) {
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hi) : "f"(v));
    const float r = v - __uint_as_float(hi);
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lo) : "f"(r));
}
__device__ __forceinline__ float adm_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(ADM_WARPS * 32, ADM_MINB) k_attention_dec_mma(AttnDecDev a) {
    constexpr int HD = 64, GA = AD_MAXG;
    __shared__ __align__(8) float ps[ADM_WARPS][GA][36];      // a warp's probabilities of a chunk, [row][key] (padded rows)
    __shared__ __align__(16) uint32_t qsh[GA][68], qsl[GA][68];   // TF32 hi / lo halves of the query tile (padded rows)
    __shared__ float pm[ADM_WARPS][GA], pl[ADM_WARPS][GA], wg[ADM_WARPS][GA];
    __shared__ __align__(8) float po[ADM_WARPS][GA][HD];
    __shared__ float Mg[GA], Lg[GA];
    __shared__ int s_last;
    const int row = blockIdx.z, kvh = blockIdx.y, sp = blockIdx.x;
    const int Gh = a.H / a.Hkv;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gid = lane >> 2, tig = lane & 3;                // fragment coordinates of the lane
    pdl_launch_dependents();
    pdl_wait();
    const int *lens = a.k_len ? a.k_len + (a.step_d ? (int64_t)(*a.step_d) * a.len_step : 0) : nullptr;
    const int k00 = a.k_start[row], n1s = lens ? lens[row] : a.k_start[row + 1] - k00;
    const int k20 = a.k2_start ? a.k2_start[row] : 0, n2s = a.k2_start ? a.k2_start[row + 1] - k20 : 0;
    const int n1 = n1s + n2s;
    const int per_warp = a.cps * 32, per_cta = ADM_WARPS * per_warp;
    const int nsplit = (n1 + per_cta - 1) / per_cta;
    if (sp >= nsplit) return;
    // the CTA's chunks are dealt to its warps in turn (warp w takes chunks w, w + 4, ...): rows shorter than the
    // longest the launch was sized for -- early steps of a graph-replayed decode loop -- still occupy all four warps
    const int kbeg = sp * per_cta + warp * 32;                // first key of this warp's first chunk
    constexpr int KSTEP = ADM_WARPS * 32;                     // keys from one of its chunks to the next
    const int q0 = a.q_start[row], nq = a.q_start[row + 1] - q0;
    const int G = Gh * nq;                                    // virtual heads (tile rows): vh = g * nq + qi
    auto krow = [&](int j) -> const float * {
        return j < n1s ? a.k + (int64_t)(k00 + j) * a.ldk : a.k2 + (int64_t)(k20 + j - n1s) * a.ldk2;
    };
    auto vrow = [&](int j) -> const float * {
        return j < n1s ? a.v + (int64_t)(k00 + j) * a.ldk : a.v2 + (int64_t)(k20 + j - n1s) * a.ldk2;
    };
    // Q as A fragments (16 x 8 per k-step: a0 (row gid, k tig), a1 (gid + 8, tig), a2 (gid, tig + 4), a3 (gid + 8, tig + 4)),
    // k positions mapped to head dims as described above. The hi / lo halves of the 16 x 64 tile are formed once per CTA
    // and kept in shared memory; a lane fetches its fragments of two k-steps with four 16-byte reads.
    {
        const int r = tid >> 3, d0 = (tid & 7) * 8;                  // 128 threads: row, eight dims
        const float *p = r < G ? a.q + (int64_t)(q0 + r % nq) * a.ldq + (kvh * Gh + r / nq) * HD + d0 : nullptr;
        const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 f0 = p ? *(const float4 *)p : z4, f1 = p ? *(const float4 *)(p + 4) : z4;
        uint4 h0, l0, h1, l1;
        adm_split(f0.x, h0.x, l0.x); adm_split(f0.y, h0.y, l0.y); adm_split(f0.z, h0.z, l0.z); adm_split(f0.w, h0.w, l0.w);
        adm_split(f1.x, h1.x, l1.x); adm_split(f1.y, h1.y, l1.y); adm_split(f1.z, h1.z, l1.z); adm_split(f1.w, h1.w, l1.w);
        *(uint4 *)&qsh[r][d0] = h0; *(uint4 *)&qsh[r][d0 + 4] = h1;
        *(uint4 *)&qsl[r][d0] = l0; *(uint4 *)&qsl[r][d0 + 4] = l1;
    }
    __syncthreads();
    const float sl2 = a.scale * 1.4426950408889634f;          // scores in the log2 domain
    float oacc[8][4];                                         // O[16 x 64]: tile j column n is dim 8 n + j, rows gid / gid + 8
#pragma unroll
    for (int j = 0; j < 8; j++) { oacc[j][0] = oacc[j][1] = oacc[j][2] = oacc[j][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f; // running maximum (log2 domain) and sum of rows gid, gid + 8
    const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
    // Loads run a phase ahead of the arithmetic: the keys of chunk c + 1 are requested when the score MMAs of chunk c
    // are done with their registers (they arrive under the softmax and the P V MMAs), the values of chunk c before its
    // score MMAs.
    float4 kf[4][4];                                          // n-tile j = keys kc + 8 j + gid; the lane's sixteen dims, 16 m + 4 tig ..
    auto load_k = [&](int kc) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int key = kc + 8 * j + gid;
            const float *kp = key < n1 ? krow(key) + kvh * HD + 4 * tig : nullptr;
#pragma unroll
            for (int m = 0; m < 4; m++) kf[j][m] = kp ? *(const float4 *)(kp + 16 * m) : z4;
        }
    };
    if (kbeg < n1) load_k(kbeg);
    for (int c = 0; c < a.cps; c++) {
        const int kc = kbeg + c * KSTEP;
        if (kc >= n1) break;                                  // warp-uniform
        // the chunk's values: k-step s takes keys kc + 8 s + tig (b0) and + 4 (b1); column gid of output tile j is dim
        // 8 gid + j, so the lane's eight dims of a value row are two 16-byte loads
        float4 vf[4][4];
#pragma unroll
        for (int s = 0; s < 4; s++) {
            const int ka = kc + 8 * s + tig, kb = ka + 4;
            const float *va = ka < n1 ? vrow(ka) + kvh * HD + 8 * gid : nullptr, *vb = kb < n1 ? vrow(kb) + kvh * HD + 8 * gid : nullptr;
            vf[s][0] = va ? *(const float4 *)va : z4; vf[s][1] = va ? *(const float4 *)(va + 4) : z4;
            vf[s][2] = vb ? *(const float4 *)vb : z4; vf[s][3] = vb ? *(const float4 *)(vb + 4) : z4;
        }
        // ---- S = Q K^T ----
        float sacc[4][4];
#pragma unroll
        for (int j = 0; j < 4; j++) { sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = 0.f; }
#pragma unroll
        for (int m = 0; m < 4; m++) {
            const uint4 h0 = *(const uint4 *)&qsh[gid][16 * m + 4 * tig], h1 = *(const uint4 *)&qsh[gid + 8][16 * m + 4 * tig];
            const uint4 q0l = *(const uint4 *)&qsl[gid][16 * m + 4 * tig], q1l = *(const uint4 *)&qsl[gid + 8][16 * m + 4 * tig];
            const uint32_t ah0[4] = {h0.x, h1.x, h0.y, h1.y}, al0[4] = {q0l.x, q1l.x, q0l.y, q1l.y};      // k-step 2 m
            const uint32_t ah1[4] = {h0.z, h1.z, h0.w, h1.w}, al1[4] = {q0l.z, q1l.z, q0l.w, q1l.w};      // k-step 2 m + 1
#pragma unroll
            for (int j = 0; j < 4; j++) {
                uint32_t bh0, bl0, bh1, bl1;
                adm_split(kf[j][m].x, bh0, bl0); adm_split(kf[j][m].y, bh1, bl1);
                adm_mma(sacc[j], al0, bh0, bh1);
                adm_mma(sacc[j], ah0, bl0, bl1);
                adm_mma(sacc[j], ah0, bh0, bh1);
                adm_split(kf[j][m].z, bh0, bl0); adm_split(kf[j][m].w, bh1, bl1);
                adm_mma(sacc[j], al1, bh0, bh1);
                adm_mma(sacc[j], ah1, bl0, bl1);
                adm_mma(sacc[j], ah1, bh0, bh1);
            }
        }
        if (c + 1 < a.cps && kc + KSTEP < n1) load_k(kc + KSTEP);   // the next chunk's keys, under the rest of this chunk
        // ---- softmax of the chunk, rows gid (c0, c1) and gid + 8 (c2, c3); columns 8 j + 2 tig, + 1 ----
        float cm0 = -INFINITY, cm1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 4; j++) {
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const bool ok = kc + 8 * j + 2 * tig + e < n1;
                sacc[j][e] = ok ? sacc[j][e] * sl2 : -INFINITY;
                sacc[j][2 + e] = ok ? sacc[j][2 + e] * sl2 : -INFINITY;
                cm0 = fmaxf(cm0, sacc[j][e]); cm1 = fmaxf(cm1, sacc[j][2 + e]);
            }
        }
        cm0 = fmaxf(cm0, __shfl_xor_sync(0xffffffffu, cm0, 1)); cm0 = fmaxf(cm0, __shfl_xor_sync(0xffffffffu, cm0, 2));
        cm1 = fmaxf(cm1, __shfl_xor_sync(0xffffffffu, cm1, 1)); cm1 = fmaxf(cm1, __shfl_xor_sync(0xffffffffu, cm1, 2));
        const float nm0 = fmaxf(m0, cm0), nm1 = fmaxf(m1, cm1);   // finite: the chunk has at least one key
        const float al0 = m0 == -INFINITY ? 0.f : adm_ex2(m0 - nm0), al1 = m1 == -INFINITY ? 0.f : adm_ex2(m1 - nm1);
        m0 = nm0; m1 = nm1;
        float cs0 = 0.f, cs1 = 0.f;
        __syncwarp();                                         // the previous chunk's reads of ps are done
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float p00 = adm_ex2(sacc[j][0] - nm0), p01 = adm_ex2(sacc[j][1] - nm0);
            const float p10 = adm_ex2(sacc[j][2] - nm1), p11 = adm_ex2(sacc[j][3] - nm1);
            cs0 += p00 + p01; cs1 += p10 + p11;
            *(float2 *)&ps[warp][gid][8 * j + 2 * tig] = make_float2(p00, p01);
            *(float2 *)&ps[warp][gid + 8][8 * j + 2 * tig] = make_float2(p10, p11);
        }
        cs0 += __shfl_xor_sync(0xffffffffu, cs0, 1); cs0 += __shfl_xor_sync(0xffffffffu, cs0, 2);
        cs1 += __shfl_xor_sync(0xffffffffu, cs1, 1); cs1 += __shfl_xor_sync(0xffffffffu, cs1, 2);
        l0 = fmaf(l0, al0, cs0); l1 = fmaf(l1, al1, cs1);
#pragma unroll
        for (int j = 0; j < 8; j++) { oacc[j][0] *= al0; oacc[j][1] *= al0; oacc[j][2] *= al1; oacc[j][3] *= al1; }
        __syncwarp();
        // ---- O += P V: A fragment of k-step s (keys kc + 8 s + tig, + 4) from ps ----
#pragma unroll
        for (int s = 0; s < 4; s++) {
            uint32_t ph[4], pl_[4];
            adm_split(ps[warp][gid][8 * s + tig], ph[0], pl_[0]);
            adm_split(ps[warp][gid + 8][8 * s + tig], ph[1], pl_[1]);
            adm_split(ps[warp][gid][8 * s + tig + 4], ph[2], pl_[2]);
            adm_split(ps[warp][gid + 8][8 * s + tig + 4], ph[3], pl_[3]);
            const float vb0[8] = {vf[s][0].x, vf[s][0].y, vf[s][0].z, vf[s][0].w, vf[s][1].x, vf[s][1].y, vf[s][1].z, vf[s][1].w};
            const float vb1[8] = {vf[s][2].x, vf[s][2].y, vf[s][2].z, vf[s][2].w, vf[s][3].x, vf[s][3].y, vf[s][3].z, vf[s][3].w};
#pragma unroll
            for (int j = 0; j < 8; j++) {
                uint32_t bh0, bl0, bh1, bl1;
                adm_split(vb0[j], bh0, bl0); adm_split(vb1[j], bh1, bl1);
                adm_mma(oacc[j], pl_, bh0, bh1);
                adm_mma(oacc[j], ph, bl0, bl1);
                adm_mma(oacc[j], ph, bh0, bh1);
            }
        }
    }
    // ---- the warps' partials meet in shared memory ----
    if (tig == 0) { pm[warp][gid] = m0; pm[warp][gid + 8] = m1; pl[warp][gid] = l0; pl[warp][gid + 8] = l1; }
#pragma unroll
    for (int j = 0; j < 8; j++) {                             // columns 2 tig, 2 tig + 1 of tile j are dims 16 tig + j, + 8
        po[warp][gid][16 * tig + j] = oacc[j][0]; po[warp][gid][16 * tig + 8 + j] = oacc[j][1];
        po[warp][gid + 8][16 * tig + j] = oacc[j][2]; po[warp][gid + 8][16 * tig + 8 + j] = oacc[j][3];
    }
    __syncthreads();
    if (tid < G) {
        float M = -INFINITY, L = 0.f;
        for (int w = 0; w < ADM_WARPS; w++) M = fmaxf(M, pm[w][tid]);
        for (int w = 0; w < ADM_WARPS; w++) {
            const float e = (pm[w][tid] == -INFINITY) ? 0.f : adm_ex2(pm[w][tid] - M);
            wg[w][tid] = e; L = fmaf(pl[w][tid], e, L);
        }
        Mg[tid] = M; Lg[tid] = L;
    }
    __syncthreads();
    float *mine = a.part + ((int64_t)(row * a.Hkv + kvh) * a.max_split + sp) * AD_MAXG * (HD + 2);
    for (int i = tid; i < G * HD; i += blockDim.x) {
        const int g = i / HD, d = i % HD;
        float O = 0.f;
        for (int w = 0; w < ADM_WARPS; w++) O = fmaf(po[w][g][d], wg[w][g], O);
        if (nsplit == 1) {
            const float L = Lg[g];
            const float r = L > 0.f ? O / L : 0.f;
            const int64_t at = (int64_t)(q0 + g % nq) * a.ldo + (kvh * Gh + g / nq) * HD + d;
            if (a.out_lo) store_split1(a.out, a.out_lo, at, r, a.out_fmt);
            else a.out[at] = r;
        } else {
            mine[g * (HD + 2) + 2 + d] = O;
            if (d == 0) { mine[g * (HD + 2)] = Mg[g]; mine[g * (HD + 2) + 1] = Lg[g]; }
        }
    }
    if (nsplit == 1) return;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        unsigned old = atomicAdd(a.count + row * a.Hkv + kvh, 1u);
        s_last = (old == (unsigned)(nsplit - 1));
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // the last CTA of the (row, kv head) merges the CTAs' partials (maxima in the log2 domain here)
    const float *base = a.part + (int64_t)(row * a.Hkv + kvh) * a.max_split * AD_MAXG * (HD + 2);
    if (tid < G) {
        float M = -INFINITY, L = 0.f;
        for (int x = 0; x < nsplit; x++) M = fmaxf(M, __ldcg(base + ((int64_t)x * AD_MAXG + tid) * (HD + 2)));
        for (int x = 0; x < nsplit; x++) {
            const float *pp = base + ((int64_t)x * AD_MAXG + tid) * (HD + 2);
            const float mx = __ldcg(pp);
            L = fmaf(__ldcg(pp + 1), mx == -INFINITY ? 0.f : adm_ex2(mx - M), L);
        }
        Mg[tid] = M; Lg[tid] = L;
    }
    __syncthreads();
    for (int i = tid; i < G * HD; i += blockDim.x) {
        const int g = i / HD, d = i % HD;
        const float M = Mg[g];
        float O = 0.f;
        for (int x = 0; x < nsplit; x++) {
            const float *pp = base + ((int64_t)x * AD_MAXG + g) * (HD + 2);
            const float mx = __ldcg(pp);
            O = fmaf(__ldcg(pp + 2 + d), mx == -INFINITY ? 0.f : adm_ex2(mx - M), O);
        }
        const float L = Lg[g];
        const float r = L > 0.f ? O / L : 0.f;
        const int64_t at = (int64_t)(q0 + g % nq) * a.ldo + (kvh * Gh + g / nq) * HD + d;
        if (a.out_lo) store_split1(a.out, a.out_lo, at, r, a.out_fmt);
        else a.out[at] = r;
    }
    if (tid == 0) a.count[row * a.Hkv + kvh] = 0;
}

bool attention_decode_supported(const AttnArgs &a) {
    if (a.max_q < 1 || a.max_q > 4 || a.causal || a.window > 0) return false;      // a few queries per row, no mask
    if (a.hd != 16 && a.hd != 32 && a.hd != 64 && a.hd != 128) return false;
    if (a.Hkv <= 0 || a.H % a.Hkv || (a.H / a.Hkv) * a.max_q > AD_MAXG) return false;
    if (a.max_k1 <= 0 || a.max_k1 + a.max_k2 > AD_KEYS * AD_MAXSPLIT) return false;
    if ((a.ldk1 & 3) || ((uintptr_t)a.k1 & 15)) return false;
    if (a.k2 && ((a.ldk2 & 3) || ((uintptr_t)a.k2 & 15) || a.step_d)) return false;
    return true;
}

void attention_decode(const AttnArgs &a) {
    static float *part = nullptr; static size_t part_cap = 0;
    static unsigned *count = nullptr; static size_t count_cap = 0;
    // Keys of a row are shared out in 32-key chunks. With few (row, kv head) pairs every chunk gets a CTA of its own
    // (a batch-1 decode step has nothing else to fill the GPU with); with many pairs a CTA walks several chunks,
    // so that the fixed cost per CTA (query load, partials through L2, the merge) is paid about 8 x SMs times
    // and not once per chunk.
    const int max_chunks = (int)cdiv(a.max_k1 + a.max_k2, AD_KEYS);
    const int64_t pairs = (int64_t)a.rows * a.Hkv;
    static const bool warp_kernel = !getenv("NCM_B200_OLD_ATTN_DEC");
    const bool warp_always = getenv("NCM_B200_ATTN_DEC_WARP") != nullptr;       // read per call: tests run both kernels on the same inputs
    // The warp-per-chunk kernel for few (row, kv head) pairs, where the older kernel is a chain of barriers and a long
    // merge: a warp takes up to two (query, head) pairs (more make its serial arithmetic the kernel: seven per warp
    // measured 1.10 -> 1.16 ms per token on the Qwen2 shape), two or four chunks per CTA, and all CTAs must be resident at
    // once. With hundreds of pairs the older kernel's higher occupancy wins (GPT-2 at 64 sequences: 1.44 against
    // 1.94 ms per step).
    const int gq_w = (a.H / a.Hkv) * a.max_q;
    // many (query, head) pairs per kv group and enough (row, kv head) pairs to fill the GPU with warps: the
    // tensor-core kernel (read per call: the tests run every kernel on the same inputs)
    const char *mma_s = getenv("NCM_B200_ATTN_DEC_MMA");
    const int mma_env = mma_s ? atoi(mma_s) : -1;
    auto al16 = [](const void *q) { return ((uintptr_t)q & 15) == 0; };
    const bool mma_takes = a.hd == 64 && gq_w <= AD_MAXG && ((a.ldk1 & 3) == 0) && (!a.k2 || (a.ldk2 & 3) == 0) && ((a.ldq & 3) == 0) &&
                           al16(a.q) && al16(a.k1) && al16(a.v1) && (!a.k2 || (al16(a.k2) && al16(a.v2)));
    // (measured: the 4-token level of config 2 -- 16 pairs per group, 9 chunks -- 2.99 -> 2.44 ms over its 12 layers; the
    // Qwen2 batched-decode shape -- 7 pairs, 16 - 32 chunks -- at 256 sequences 42 936 -> 44 923 tokens/s, at 32
    // sequences 12 821 -> 12 661: with few (row, kv head) pairs the CTA-per-chunk kernels spread a row over more SMs)
    static const int mma_min_g = getenv("NCM_B200_ATTN_DEC_MMA_MIN_G") ? atoi(getenv("NCM_B200_ATTN_DEC_MMA_MIN_G")) : 12;
    static const int mma_max_ch = getenv("NCM_B200_ATTN_DEC_MMA_MAX_CHUNKS") ? atoi(getenv("NCM_B200_ATTN_DEC_MMA_MAX_CHUNKS")) : 16;
    const bool mma_pays = (gq_w >= mma_min_g && max_chunks <= mma_max_ch && pairs * 4 >= (int64_t)ctx().sm_count) ||
                          (gq_w >= 6 && pairs >= 2 * (int64_t)ctx().sm_count);
    if (mma_takes && (mma_env == 1 || (mma_env != 0 && mma_pays))) {
        // chunks per warp: as few CTAs per (row, kv head) as still give every SM about eight warps
        const int64_t want_ctas = std::max<int64_t>(1, cdiv((int64_t)ctx().sm_count * 2, pairs));
        int cpw = (int)cdiv(max_chunks, ADM_WARPS * want_ctas);
        if (cpw < 1) cpw = 1;
        if (cpw > 16) cpw = 16;
        const int max_split = (int)cdiv(max_chunks, ADM_WARPS * cpw);
        if (max_split <= AD_MAXSPLIT) {
            size_t need = (size_t)a.rows * a.Hkv * max_split * AD_MAXG * (a.hd + 2);
            if (need > part_cap) {
                if (part) { CUDA_CHECK(cudaStreamSynchronize(stream())); dev_free(part); }
                part = (float *)dev_alloc(need * 4); part_cap = need;
            }
            size_t nc = (size_t)a.rows * a.Hkv;
            if (nc > count_cap) {
                if (count) { CUDA_CHECK(cudaStreamSynchronize(stream())); dev_free(count); }
                count = (unsigned *)dev_alloc(nc * 4); count_cap = nc;
                CUDA_CHECK(cudaMemsetAsync(count, 0, nc * 4, stream()));
            }
            AttnDecDev d;
            d.q = a.q; d.ldq = a.ldq; d.k = a.k1; d.v = a.v1; d.ldk = a.ldk1;
            d.k2 = a.k2; d.v2 = a.v2; d.ldk2 = a.ldk2; d.k2_start = a.k2 ? a.k2_start : nullptr; d.out = a.out; d.out_lo = a.out_lo; d.out_fmt = a.out_fmt; d.ldo = a.ldo;
            d.q_start = a.q_start; d.k_start = a.k1_start; d.k_len = a.k1_len;
            d.step_d = a.step_d; d.len_step = a.k1_len_step;
            d.H = a.H; d.Hkv = a.Hkv; d.max_split = max_split; d.cps = cpw; d.hs = 1;
            d.scale = 1.0f / sqrtf((float)a.hd);
            d.part = part; d.count = count;
            dim3 grid((unsigned)max_split, (unsigned)a.Hkv, (unsigned)a.rows);
            ProfScope ps(NCMB_K_ATTN, 4.0 * (double)a.total_q * a.avg_keys * a.H * a.hd, 0);
            LAUNCH_PDL(k_attention_dec_mma, grid, ADM_WARPS * 32, 0, d);
            return;
        }
    }
    const int gmw = gq_w <= 1 ? 1 : (gq_w <= 8 ? 2 : 4);
    const int hs = (int)cdiv(gq_w, gmw);                                         // 1, 2, 3 or 4 warps per chunk
    const int cpc = hs <= 2 ? 4 : 2;                                             // chunks per CTA (128 or 64 keys): at most eight warps
    const int max_split_w = (int)cdiv(max_chunks, cpc);
    const bool warp_pays = warp_always || pairs * max_split_w <= 2 * (int64_t)ctx().sm_count;
    if (warp_kernel && warp_pays && a.hd == 64 && hs * cpc <= 8 && max_split_w <= AD_MAXSPLIT &&
        ((a.ldk1 & 3) == 0) && (!a.k2 || (a.ldk2 & 3) == 0)) {
        const int max_split = max_split_w;
        size_t need = (size_t)a.rows * a.Hkv * max_split * AD_MAXG * (a.hd + 2);
        if (need > part_cap) {
            if (part) { CUDA_CHECK(cudaStreamSynchronize(stream())); dev_free(part); }
            part = (float *)dev_alloc(need * 4); part_cap = need;
        }
        size_t nc = (size_t)a.rows * a.Hkv;
        if (nc > count_cap) {
            if (count) { CUDA_CHECK(cudaStreamSynchronize(stream())); dev_free(count); }
            count = (unsigned *)dev_alloc(nc * 4); count_cap = nc;
            CUDA_CHECK(cudaMemsetAsync(count, 0, nc * 4, stream()));
        }
        AttnDecDev d;
        d.q = a.q; d.ldq = a.ldq; d.k = a.k1; d.v = a.v1; d.ldk = a.ldk1;
        d.k2 = a.k2; d.v2 = a.v2; d.ldk2 = a.ldk2; d.k2_start = a.k2 ? a.k2_start : nullptr; d.out = a.out; d.out_lo = a.out_lo; d.out_fmt = a.out_fmt; d.ldo = a.ldo;
        d.q_start = a.q_start; d.k_start = a.k1_start; d.k_len = a.k1_len;
        d.step_d = a.step_d; d.len_step = a.k1_len_step;
        d.H = a.H; d.Hkv = a.Hkv; d.max_split = max_split; d.cps = cpc; d.hs = hs;
        d.scale = 1.0f / sqrtf((float)a.hd);
        d.part = part; d.count = count;
        dim3 grid((unsigned)max_split, (unsigned)a.Hkv, (unsigned)a.rows);
        ProfScope ps(NCMB_K_ATTN, 4.0 * (double)a.total_q * a.avg_keys * a.H * a.hd, 0);
        const int threads = hs * cpc * 32;
        if (gmw == 1) LAUNCH_PDL((k_attention_dec_warp<1>), grid, threads, 0, d);
        else if (gmw == 2) LAUNCH_PDL((k_attention_dec_warp<2>), grid, threads, 0, d);
        else LAUNCH_PDL((k_attention_dec_warp<4>), grid, threads, 0, d);
        return;
    }
    static const int per_sm = getenv("NCM_B200_ATTN_DEC_PER_SM") ? atoi(getenv("NCM_B200_ATTN_DEC_PER_SM")) : 8;
    int want_split = (int)std::min<int64_t>(max_chunks, cdiv((int64_t)ctx().sm_count * per_sm, pairs));
    if (want_split < 1) want_split = 1;
    static const int cps_env = getenv("NCM_B200_ATTN_DEC_CPS") ? atoi(getenv("NCM_B200_ATTN_DEC_CPS")) : 0;
    const int cps = cps_env > 0 ? std::min(cps_env, max_chunks) : (int)cdiv(max_chunks, want_split);
    const int max_split = (int)cdiv(max_chunks, cps);
    size_t need = (size_t)a.rows * a.Hkv * max_split * AD_MAXG * (a.hd + 2);
    if (need > part_cap) {
        if (part) { CUDA_CHECK(cudaStreamSynchronize(stream())); dev_free(part); }
        part = (float *)dev_alloc(need * 4); part_cap = need;
    }
    size_t nc = (size_t)a.rows * a.Hkv;
    if (nc > count_cap) {
        if (count) { CUDA_CHECK(cudaStreamSynchronize(stream())); dev_free(count); }
        count = (unsigned *)dev_alloc(nc * 4); count_cap = nc;
        CUDA_CHECK(cudaMemsetAsync(count, 0, nc * 4, stream()));
    }
    AttnDecDev d;
    d.q = a.q; d.ldq = a.ldq; d.k = a.k1; d.v = a.v1; d.ldk = a.ldk1;
    d.k2 = a.k2; d.v2 = a.v2; d.ldk2 = a.ldk2; d.k2_start = a.k2 ? a.k2_start : nullptr; d.out = a.out; d.out_lo = a.out_lo; d.out_fmt = a.out_fmt; d.ldo = a.ldo;
    d.q_start = a.q_start; d.k_start = a.k1_start; d.k_len = a.k1_len;
    d.step_d = a.step_d; d.len_step = a.k1_len_step;
    d.H = a.H; d.Hkv = a.Hkv; d.max_split = max_split; d.cps = cps;
    d.scale = 1.0f / sqrtf((float)a.hd);
    d.part = part; d.count = count;
    dim3 grid((unsigned)max_split, (unsigned)a.Hkv, (unsigned)a.rows);
    ProfScope ps(NCMB_K_ATTN, 4.0 * (double)a.total_q * a.avg_keys * a.H * a.hd, 0);
    const int gq = (a.H / a.Hkv) * a.max_q;
#define AD_LAUNCH(HD_)                                                                              \
    do {                                                                                            \
        if (gq <= 1) LAUNCH_PDL((k_attention_decode<HD_, 1>), grid, AD_THREADS, 0, d);              \
        else if (gq <= 4) LAUNCH_PDL((k_attention_decode<HD_, 4>), grid, AD_THREADS, 0, d);         \
        else if (gq <= 8) LAUNCH_PDL((k_attention_decode<HD_, 8>), grid, AD_THREADS, 0, d);         \
        else LAUNCH_PDL((k_attention_decode<HD_, 16>), grid, AD_THREADS, 0, d);                     \
    } while (0)
    switch (a.hd) {
        case 16: AD_LAUNCH(16); break;
        case 32: AD_LAUNCH(32); break;
        case 64: AD_LAUNCH(64); break;
        default: AD_LAUNCH(128); break;
    }
#undef AD_LAUNCH
}

} // namespace ncmb
