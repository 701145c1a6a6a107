// Device-side sampling of one level's positions for every row.
//
// One CTA per sequence row; positions are visited in order because the
// frequency / deficit / adjacency penalties of position t depend on the picks at
// positions < t (reference sample_level_rows, src/ncp.c:654-705). Per position:
//   CFG blend (1+w) cond - w uncond in fp64 (src/ncp.c:1112-1116), penalties in fp64,
//   then either first-index argmax (temp <= 0) or temperature / top-k / nucleus
//   sampling (src/kernels.c:794-825): the top `keep` logits are found with a
//   block-wide 4 x 8-bit radix select, sorted with a bitonic network, turned into
//   fp64 probabilities and walked sequentially in rank order exactly as the
//   reference does, using one pre-drawn uniform.
// The uniforms come either from the reference's xorshift64* stream (drawn on the
// host in the reference's (level, row, position) order) or from a counter-based
// generator keyed by (seed, global row, level, position).
#include "common.cuh"

#include <cub/device/device_radix_sort.cuh>
#include <vector>

namespace ncmb {

constexpr int SM_THREADS = 256;
constexpr int SM_MAXKEEP = 2048;           // exact sorted path handles keep <= this
constexpr int SM_SMEM_V = 16384;           // logits rows up to this many floats live in shared memory

struct SampleDev {
    SampleArgs a;
    int vals_in_smem;
};

__device__ __forceinline__ unsigned okey(float f) {      // order-preserving float -> uint
    unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float okey_inv(unsigned k) {
    unsigned u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
    return __uint_as_float(u);
}

// splitmix64-style counter hash -> uniform double in [0, 1)
__device__ __forceinline__ double counter_uniform(unsigned long long seed, long long row, int level, int t) {
    unsigned long long z = seed ^ (0x9E3779B97F4A7C15ULL * (unsigned long long)(row + 1));
    z += 0xBF58476D1CE4E5B9ULL * (unsigned long long)(level + 1) + 0x94D049BB133111EBULL * (unsigned long long)(t + 1);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    z = z ^ (z >> 31);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = z ^ (z >> 29);
    return (double)(z >> 11) * (1.0 / 9007199254740992.0);
}

// the draw of model row b at position t: keyed by the sequence's global index, never by the row's place in the call
__device__ __forceinline__ double counter_uniform_row(const SampleArgs &a, int b, int t) {
    const bool twin = a.rng_wrap > 0 && b >= a.rng_wrap;
    return counter_uniform(a.rng_seed, a.rng_row0 + (twin ? b - a.rng_wrap : b), a.rng_level + (twin ? 64 : 0), t);
}

__global__ void __launch_bounds__(SM_THREADS) k_sample(SampleDev sd) {
    const SampleArgs &a = sd.a;
    extern __shared__ __align__(16) unsigned char smraw[];
    // layout: cand u64[SM_MAXKEEP] | probs f64[SM_MAXKEEP] | vals f32[V] (optional)
    unsigned long long *cand = (unsigned long long *)smraw;
    double *probs = (double *)(smraw + sizeof(unsigned long long) * SM_MAXKEEP);
    float *vals = sd.vals_in_smem ? (float *)(smraw + 16 * SM_MAXKEEP) : a.scratch + (size_t)blockIdx.x * a.V;
    __shared__ int hist[256];
    __shared__ unsigned long long red[SM_THREADS];
    __shared__ unsigned s_prefix, s_mask;
    __shared__ double s_den;
    __shared__ int s_remaining, s_ncand, s_pick, s_eqbase[SM_THREADS + 1];

    const int b = blockIdx.x, tid = threadIdx.x, V = a.V, Lc = a.Lc;
    double *cnt = a.cnt ? a.cnt + (size_t)b * a.cnt_stride : nullptr;
    int *hst = a.hist ? a.hist + (size_t)b * a.hist_stride : nullptr;
    int hl = a.hist_len ? a.hist_len[b] : 0;
    const bool penal = (a.freq > 0.f) || (a.adj_a != 0.f);

    for (int t = 0; t < Lc; t++) {
        const float *lc = a.logits + ((size_t)b * Lc + t) * V;
        const float *lu = a.uncond_off ? a.logits + (((size_t)b + a.uncond_off) * Lc + t) * V : nullptr;
        float *bo = a.blend_out ? a.blend_out + ((size_t)b * Lc + t) * V : nullptr;
        for (int v = tid; v < V; v += SM_THREADS) {
            float x = lc[v];
            if (lu) x = (float)((1.0 + a.cfg_w) * (double)x - a.cfg_w * (double)lu[v]);
            if (bo) bo[v] = x;
            if (penal) {
                double lg = x;
                if (a.freq > 0.f) {
                    double al = a.allow_dev ? a.allow_dev[v] * Lc : 0.0;
                    double c = cnt[v];
                    double excess = c - al;
                    if (excess < 0) excess = 0;
                    lg -= (double)a.freq * excess;
                    if (a.mu > 0.f && a.allow_dev) {
                        double def = al - c;
                        if (def < 0) def = 0;
                        lg += (double)a.mu * ((Lc - t) / (double)Lc) * def;
                    }
                }
                x = (float)lg;
            }
            vals[v] = x;
        }
        __syncthreads();
        if (a.adj_a != 0.f && tid == 0) {            // sequential: the same id may repeat in the window
            int w = a.adj_w > 0 ? a.adj_w : 1;
            int start = hl - w;
            if (start < 0) start = 0;
            for (int h = start; h < hl; h++) {
                double pen = (double)a.adj_a * pow((double)a.adj_d, (double)(hl - 1 - h));
                vals[hst[h]] -= (float)pen;
            }
        }
        __syncthreads();

        if (!(a.temp > 0.f)) {
            // first-index argmax: max over (ordered key, inverted index)
            unsigned long long best = 0;
            for (int v = tid; v < V; v += SM_THREADS) {
                unsigned long long c = ((unsigned long long)okey(vals[v]) << 32) | (unsigned)(0xffffffffu - (unsigned)v);
                if (c > best) best = c;
            }
            red[tid] = best;
            __syncthreads();
            for (int s = SM_THREADS / 2; s > 0; s >>= 1) {
                if (tid < s && red[tid + s] > red[tid]) red[tid] = red[tid + s];
                __syncthreads();
            }
            if (tid == 0) s_pick = (int)(0xffffffffu - (unsigned)(red[0] & 0xffffffffu));
            __syncthreads();
        } else {
            for (int v = tid; v < V; v += SM_THREADS) vals[v] = vals[v] / a.temp;
            int keep = (a.top_k > 0) ? (a.top_k < V ? a.top_k : V) : V;
            // ---- radix select: key of the keep-th largest value ----
            if (tid == 0) { s_prefix = 0; s_mask = 0; s_remaining = keep; }
            __syncthreads();
            for (int pass = 3; pass >= 0; pass--) {
                hist[tid] = 0;
                __syncthreads();
                unsigned prefix = s_prefix, mask = s_mask;
                for (int v = tid; v < V; v += SM_THREADS) {
                    unsigned k = okey(vals[v]);
                    if ((k & mask) == prefix) atomicAdd(&hist[(k >> (8 * pass)) & 0xff], 1);
                }
                __syncthreads();
                if (tid < 32) {
                    // the bin, scanning from 255 down, where the running count first reaches `rem`: lane l owns bins
                    // 255-8l .. 248-8l; lane totals are scanned with shuffles instead of one thread walking 256 bins
                    const int rem = s_remaining, top = 255 - 8 * tid;
                    int h8[8], tot = 0;
#pragma unroll
                    for (int i = 0; i < 8; i++) { h8[i] = hist[top - i]; tot += h8[i]; }
                    int incl = tot;
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1) { int t2 = __shfl_up_sync(0xffffffffu, incl, o); if (tid >= o) incl += t2; }
                    int cum = incl - tot;                               // count in all bins above this lane's
                    const bool here = cum < rem && incl >= rem;          // the crossing lies in this lane's bins
                    const unsigned who = __ballot_sync(0xffffffffu, here);
                    if (who == 0) {                                      // fewer than rem values in total: bin 0, as the serial walk ends
                        if (tid == 31) {
                            s_remaining = rem - (incl - h8[7]);
                            s_prefix = prefix; s_mask = mask | (0xffu << (8 * pass));
                        }
                    } else if (tid == __ffs(who) - 1) {
                        int bin = top;
                        for (int i = 0; i < 8; i++) {
                            bin = top - i;
                            if (bin == 0 || cum + h8[i] >= rem) break;
                            cum += h8[i];
                        }
                        s_remaining = rem - cum;
                        s_prefix = prefix | ((unsigned)bin << (8 * pass));
                        s_mask = mask | (0xffu << (8 * pass));
                    }
                }
                __syncthreads();
            }
            const unsigned thr = s_prefix;
            const int need_eq = s_remaining;          // how many values equal to the threshold are kept
            if (tid == 0) s_ncand = 0;
            __syncthreads();
            for (int v = tid; v < V; v += SM_THREADS) {
                unsigned k = okey(vals[v]);
                if (k > thr) {
                    int p = atomicAdd(&s_ncand, 1);
                    cand[p] = ((unsigned long long)k << 32) | (unsigned)(0xffffffffu - (unsigned)v);
                }
            }
            // threshold ties: lowest indices first (contiguous chunk per thread + exclusive scan)
            const int chunk = (V + SM_THREADS - 1) / SM_THREADS;
            const int v0 = tid * chunk, v1 = (v0 + chunk < V) ? v0 + chunk : V;
            int eq = 0;
            for (int v = v0; v < v1; v++) if (okey(vals[v]) == thr) eq++;
            s_eqbase[tid + 1] = eq;
            __syncthreads();
            {   // inclusive scan of the per-thread tie counts: warp shuffles, then the eight warp totals
                const int lane = tid & 31, wp = tid >> 5;
                int v = eq;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) { int t2 = __shfl_up_sync(0xffffffffu, v, o); if (lane >= o) v += t2; }
                if (lane == 31) hist[wp] = v;
                __syncthreads();
                int base = 0;
                for (int i = 0; i < wp; i++) base += hist[i];
                s_eqbase[tid + 1] = base + v;
                if (tid == 0) s_eqbase[0] = 0;
            }
            __syncthreads();
            {
                int rank = s_eqbase[tid], gt = s_ncand;
                for (int v = v0; v < v1 && rank < need_eq; v++)
                    if (okey(vals[v]) == thr) {
                        cand[gt + rank] = ((unsigned long long)thr << 32) | (unsigned)(0xffffffffu - (unsigned)v);
                        rank++;
                    }
            }
            __syncthreads();
            // ---- bitonic sort, descending: value desc, index asc ----
            int n2 = 1;
            while (n2 < keep) n2 <<= 1;
            for (int i = keep + tid; i < n2; i += SM_THREADS) cand[i] = 0;
            __syncthreads();
            for (int k = 2; k <= n2; k <<= 1)
                for (int j = k >> 1; j > 0; j >>= 1) {
                    for (int i = tid; i < n2; i += SM_THREADS) {
                        int ixj = i ^ j;
                        if (ixj > i) {
                            unsigned long long x = cand[i], y = cand[ixj];
                            bool desc = ((i & k) == 0);
                            if (desc ? (x < y) : (x > y)) { cand[i] = y; cand[ixj] = x; }
                        }
                    }
                    __syncthreads();
                }
            // ---- probabilities in rank order (fp64), nucleus cut, renormalise, walk ----
            const double mx = (double)okey_inv((unsigned)(cand[0] >> 32));
            for (int r = tid; r < keep; r += SM_THREADS)
                probs[r] = exp((double)okey_inv((unsigned)(cand[r] >> 32)) - mx);
            __syncthreads();
            // the sums run in rank order on one thread, as the reference's do; the divisions are independent
            if (tid == 0) {
                double den = 0;
                for (int r = 0; r < keep; r++) den += probs[r];
                s_den = den;
            }
            __syncthreads();
            {
                const double den = s_den;
                for (int r = tid; r < keep; r += SM_THREADS) probs[r] /= den;
            }
            __syncthreads();
            if (tid == 0) {
                double den;
                double cum = 0;
                int nkeep = keep;
                for (int r = 0; r < keep; r++) {
                    if (cum - probs[r] > (double)a.top_p) { nkeep = r; break; }
                    cum += probs[r];
                }
                den = 0;
                for (int r = 0; r < nkeep; r++) den += probs[r];
                double u01 = a.uniforms ? a.uniforms[(size_t)b * Lc + t]
                                        : counter_uniform_row(a, b, t);
                double u = u01 * den, acc = 0;
                int pr = nkeep - 1;
                for (int r = 0; r < nkeep; r++) { acc += probs[r]; if (u <= acc) { pr = r; break; } }
                s_pick = (int)(0xffffffffu - (unsigned)(cand[pr] & 0xffffffffu));
            }
            __syncthreads();
        }
        if (tid == 0) {
            int pick = s_pick;
            a.out[(size_t)b * a.out_stride + a.out_off + t] = pick;
            if (cnt) cnt[pick] += 1.0;
            if (hst) hst[hl] = pick;
        }
        hl++;
        __syncthreads();
    }
    if (tid == 0 && a.hist_len) a.hist_len[b] = hl;
}

// ---------------------------------------------------------------------------------------------
// Two-phase sampling. The sequential kernel above spends most of a position on work that does not
// depend on earlier picks: the blend and the 4096-wide selection. Penalties that only LOWER logits
// (frequency excess, adjacency with a >= 0; no deficit bonus) touch at most P tokens, the ones
// picked so far in the row, so the `keep` best penalised logits of a position lie among its
// keep + P best raw ones: a token of the penalised top-keep is preceded in raw order by at most
// keep - 1 unpenalised tokens (which precede it in penalised order too) and P penalised ones.
//   k_sample_topc  one CTA per (row, position), all positions at once: blend, the Kc >= keep + P
//                  best raw logits (same radix select, ties to the lowest index) -> candidates
//   k_sample_seq   one CTA per row, positions in order, Kc entries each: the same penalty, temperature,
//                  ordering (value descending, index ascending), fp64 probabilities and walk as above
// Picks equal the one-kernel path's bit for bit: every number a pick depends on is computed by the
// same operations in the same order.
constexpr int SC_MAXC = 256;

struct SampleCand {
    SampleArgs a;
    int Kc;
    unsigned long long *cand;       // [Bn][Lc][Kc]: ordered key << 32 | ~index of the raw (blended) logit
};

__global__ void __launch_bounds__(SM_THREADS) k_sample_topc(SampleCand sc) {
    const SampleArgs &a = sc.a;
    extern __shared__ __align__(16) unsigned char smraw[];
    float *vals = (float *)smraw;
    __shared__ int hist[256];
    __shared__ unsigned s_prefix, s_mask;
    __shared__ int s_remaining, s_ncand, s_eqbase[SM_THREADS + 1];
    const int tid = threadIdx.x, V = a.V, Lc = a.Lc, keep = sc.Kc;
    const int b = blockIdx.x / Lc, t = blockIdx.x % Lc;
    const float *lc = a.logits + ((size_t)b * Lc + t) * V;
    const float *lu = a.uncond_off ? a.logits + (((size_t)b + a.uncond_off) * Lc + t) * V : nullptr;
    float *bo = a.blend_out ? a.blend_out + ((size_t)b * Lc + t) * V : nullptr;
    unsigned long long *out = sc.cand + ((size_t)b * Lc + t) * keep;
    for (int v = tid; v < V; v += SM_THREADS) {
        float x = lc[v];
        if (lu) x = (float)((1.0 + a.cfg_w) * (double)x - a.cfg_w * (double)lu[v]);
        if (bo) bo[v] = x;
        vals[v] = x;
    }
    if (tid == 0) { s_prefix = 0; s_mask = 0; s_remaining = keep; }
    __syncthreads();
    for (int pass = 3; pass >= 0; pass--) {
        hist[tid] = 0;
        __syncthreads();
        unsigned prefix = s_prefix, mask = s_mask;
        for (int v = tid; v < V; v += SM_THREADS) {
            unsigned k = okey(vals[v]);
            if ((k & mask) == prefix) atomicAdd(&hist[(k >> (8 * pass)) & 0xff], 1);
        }
        __syncthreads();
        if (tid < 32) {
            const int rem = s_remaining, top = 255 - 8 * tid;
            int h8[8], tot = 0;
#pragma unroll
            for (int i = 0; i < 8; i++) { h8[i] = hist[top - i]; tot += h8[i]; }
            int incl = tot;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { int t2 = __shfl_up_sync(0xffffffffu, incl, o); if (tid >= o) incl += t2; }
            int cum = incl - tot;
            const bool here = cum < rem && incl >= rem;
            const unsigned who = __ballot_sync(0xffffffffu, here);
            if (who == 0) {
                if (tid == 31) { s_remaining = rem - (incl - h8[7]); s_prefix = prefix; s_mask = mask | (0xffu << (8 * pass)); }
            } else if (tid == __ffs(who) - 1) {
                int bin = top;
                for (int i = 0; i < 8; i++) {
                    bin = top - i;
                    if (bin == 0 || cum + h8[i] >= rem) break;
                    cum += h8[i];
                }
                s_remaining = rem - cum;
                s_prefix = prefix | ((unsigned)bin << (8 * pass));
                s_mask = mask | (0xffu << (8 * pass));
            }
        }
        __syncthreads();
    }
    const unsigned thr = s_prefix;
    const int need_eq = s_remaining;
    if (tid == 0) s_ncand = 0;
    __syncthreads();
    for (int v = tid; v < V; v += SM_THREADS) {
        unsigned k = okey(vals[v]);
        if (k > thr) {
            int p = atomicAdd(&s_ncand, 1);
            out[p] = ((unsigned long long)k << 32) | (unsigned)(0xffffffffu - (unsigned)v);
        }
    }
    const int chunk = (V + SM_THREADS - 1) / SM_THREADS;
    const int v0 = tid * chunk, v1 = (v0 + chunk < V) ? v0 + chunk : V;
    int eq = 0;
    for (int v = v0; v < v1; v++) if (okey(vals[v]) == thr) eq++;
    {
        const int lane = tid & 31, wp = tid >> 5;
        int v = eq;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { int t2 = __shfl_up_sync(0xffffffffu, v, o); if (lane >= o) v += t2; }
        __syncthreads();                       // hist is reused for the warp totals
        if (lane == 31) hist[wp] = v;
        __syncthreads();
        int base = 0;
        for (int i = 0; i < wp; i++) base += hist[i];
        s_eqbase[tid + 1] = base + v;
        if (tid == 0) s_eqbase[0] = 0;
    }
    __syncthreads();
    {
        int rank = s_eqbase[tid], gt = s_ncand;
        for (int v = v0; v < v1 && rank < need_eq; v++)
            if (okey(vals[v]) == thr) {
                out[gt + rank] = ((unsigned long long)thr << 32) | (unsigned)(0xffffffffu - (unsigned)v);
                rank++;
            }
    }
}

__global__ void __launch_bounds__(SC_MAXC) k_sample_seq(SampleCand sc) {
    const SampleArgs &a = sc.a;
    __shared__ unsigned long long cand[SC_MAXC];
    __shared__ double probs[SC_MAXC];
    __shared__ double s_den;
    __shared__ int s_pick;
    const int b = blockIdx.x, tid = threadIdx.x, Lc = a.Lc, Kc = sc.Kc;
    double *cnt = a.cnt ? a.cnt + (size_t)b * a.cnt_stride : nullptr;
    int *hst = a.hist ? a.hist + (size_t)b * a.hist_stride : nullptr;
    int hl = a.hist_len ? a.hist_len[b] : 0;
    const bool penal = (a.freq > 0.f) || (a.adj_a != 0.f);
    const int keep = (a.top_k > 0) ? (a.top_k < a.V ? a.top_k : a.V) : a.V;
    unsigned long long c_next = tid < Kc ? sc.cand[(size_t)b * Lc * Kc + tid] : 0;
    for (int t = 0; t < Lc; t++) {
        unsigned long long key = 0;
        const unsigned long long c = c_next;
        if (t + 1 < Lc && tid < Kc) c_next = sc.cand[((size_t)b * Lc + t + 1) * Kc + tid];   // in flight under this position's work
        if (tid < Kc) {
            const int v = (int)(0xffffffffu - (unsigned)(c & 0xffffffffu));
            float x = okey_inv((unsigned)(c >> 32));
            if (penal) {
                double lg = x;
                if (a.freq > 0.f) {
                    double al = a.allow_dev ? a.allow_dev[v] * Lc : 0.0;
                    double cc = cnt[v];
                    double excess = cc - al;
                    if (excess < 0) excess = 0;
                    lg -= (double)a.freq * excess;
                }
                x = (float)lg;
                if (a.adj_a != 0.f) {                    // window entries in order: the same id may repeat
                    int w = a.adj_w > 0 ? a.adj_w : 1;
                    int start = hl - w;
                    if (start < 0) start = 0;
                    for (int h = start; h < hl; h++)
                        if (hst[h] == v) {
                            double pen = (double)a.adj_a * pow((double)a.adj_d, (double)(hl - 1 - h));
                            x -= (float)pen;
                        }
                }
            }
            x = x / a.temp;
            key = ((unsigned long long)okey(x) << 32) | (unsigned)(0xffffffffu - (unsigned)v);
        }
        // bitonic sort, descending, one entry per thread: exchanges within a warp by shuffle, the few across
        // warps (partner distance >= 32) through shared memory
        for (int k = 2; k <= Kc; k <<= 1)
            for (int j = k >> 1; j > 0; j >>= 1) {
                unsigned long long other;
                if (j >= 32) {
                    cand[tid] = key;
                    __syncthreads();
                    other = cand[tid ^ j];
                    __syncthreads();
                } else {
                    other = __shfl_xor_sync(0xffffffffu, key, j);
                }
                const bool keep_max = (((tid & k) == 0) == ((tid & j) == 0));   // descending run: the lower index keeps the larger
                key = keep_max ? (key > other ? key : other) : (key < other ? key : other);
            }
        cand[tid] = key;
        __syncthreads();
        const double mx = (double)okey_inv((unsigned)(cand[0] >> 32));
        if (tid < keep) probs[tid] = exp((double)okey_inv((unsigned)(cand[tid] >> 32)) - mx);
        __syncthreads();
        if (tid == 0) {
            double den = 0;
            for (int r = 0; r < keep; r++) den += probs[r];
            s_den = den;
        }
        __syncthreads();
        if (tid < keep) probs[tid] /= s_den;
        __syncthreads();
        if (tid == 0) {
            // nucleus cut. The running sum of the kept ranks is at once the reference's renormaliser (its second sum
            // adds the same numbers in the same order) and, rank by rank, the accumulator of its final walk.
            double cum = 0;
            int nkeep = keep;
            for (int r = 0; r < keep; r++) {
                if (cum - probs[r] > (double)a.top_p) { nkeep = r; break; }
                cum += probs[r];
                probs[r] = cum;                          // from here on: inclusive running sums
            }
            const double u01 = a.uniforms ? a.uniforms[(size_t)b * Lc + t]
                                          : counter_uniform_row(a, b, t);
            s_den = u01 * cum;
            s_pick = nkeep;                              // handed to the search below
        }
        __syncthreads();
        {   // first rank whose running sum reaches u; the last kept rank if none does
            const int nkeep = s_pick;
            const double u = s_den;
            const bool hit = tid < nkeep && u <= probs[tid];
            __shared__ int s_first;
            if (tid == 0) s_first = nkeep - 1;
            __syncthreads();
            if (hit) atomicMin(&s_first, tid);
            __syncthreads();
            if (tid == 0) {
                const int pick = (int)(0xffffffffu - (unsigned)(cand[s_first] & 0xffffffffu));
                a.out[(size_t)b * a.out_stride + a.out_off + t] = pick;
                if (cnt) cnt[pick] += 1.0;
                if (hst) hst[hl] = pick;
            }
        }
        hl++;
        __syncthreads();                 // cnt / hist of this position are visible to the next one
    }
    if (tid == 0 && a.hist_len) a.hist_len[b] = hl;
}

// Kc for the two-phase path, or 0 when it does not apply
static int two_phase_width(const SampleArgs &a) {
    if (!(a.temp > 0.f) || a.top_k <= 0 || a.V > SM_SMEM_V) return 0;
    const char *e = getenv("NCM_B200_SAMPLE_PHASES");          // 1 = one kernel always, 2 = two phases whenever valid
    const int mode = e ? atoi(e) : 0;
    if (mode == 1) return 0;
    const bool penal = (a.freq > 0.f) || (a.adj_a != 0.f);
    if (a.adj_a < 0.f || (a.adj_a != 0.f && a.adj_d < 0.f)) return 0;   // a negative adjacency weight (or decay) raises logits
    if (penal && a.freq > 0.f && a.mu > 0.f && a.allow_dev) return 0;   // so does the deficit bonus
    if (penal && a.picks_bound <= 0) return 0;
    const int keep = a.top_k < a.V ? a.top_k : a.V;
    int need = keep + (penal ? a.picks_bound : 0), Kc = 32;
    while (Kc < need) Kc <<= 1;
    if (Kc > SC_MAXC || Kc > a.V) return 0;
    if (mode != 2 && (a.V < 8 * Kc || a.Lc < 2)) return 0;      // nothing to gain on short rows or a single position
    return Kc;
}

size_t sample_scratch_floats(int Bn, int V) { return V > SM_SMEM_V ? (size_t)Bn * V : 0; }

// ---- large candidate sets (top_k = 0 or > 2048 over a big vocabulary, one position per row) ----
// The rows are sorted once (value descending, index ascending on ties: a stable device-wide
// radix sort) and one CTA per row then walks it with block-wide fp64 prefix sums: the
// nucleus cut "cum_before - p > top_p" and the draw "u <= cum" are monotone in the sorted
// rank, so each is the minimum rank that satisfies a predicate. Sums are formed in a
// different order than the reference's sequential loop (relative differences ~1e-16).
constexpr int SL_THREADS = 1024;

__global__ void k_sort_prep(const float *__restrict__ logits, float temp, int64_t n, int V, float *__restrict__ keys, int *__restrict__ idx) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        keys[i] = logits[i] / temp;
        idx[i] = (int)(i % V);
    }
}

// all rows in ONE device-wide sort: key = row << 32 | (0xffffffff - ordered value bits), ascending, so rows stay in
// order and every row comes out largest value first (the sort is stable: equal values keep ascending indices)
__global__ void k_sort_prep64(const float *__restrict__ logits, float temp, int64_t n, int V, unsigned long long *__restrict__ keys,
                              int *__restrict__ idx) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        keys[i] = ((unsigned long long)(i / V) << 32) | (unsigned long long)(0xffffffffu - okey(logits[i] / temp));
        idx[i] = (int)(i % V);
    }
}

__device__ __forceinline__ double block_excl_scan(double v, double *sm, double *total) {
    // exclusive scan of one value per thread over SL_THREADS threads
    int tid = threadIdx.x;
    sm[tid] = v;
    __syncthreads();
    for (int off = 1; off < SL_THREADS; off <<= 1) {
        double t = tid >= off ? sm[tid - off] : 0.0;
        __syncthreads();
        sm[tid] += t;
        __syncthreads();
    }
    double incl = sm[tid];
    *total = sm[SL_THREADS - 1];
    __syncthreads();
    return incl - v;
}

// K64: keys are the composite 64-bit keys of k_sort_prep64 (the value is recovered from the low word)
template <bool K64>
__global__ void __launch_bounds__(SL_THREADS) k_pick_sorted(const void *__restrict__ keys, const int *__restrict__ idx, double *__restrict__ pcache, int V, int keep,
                                                           float top_p, const double *__restrict__ uniforms,
                                                           unsigned long long seed, long long row0, int level,
                                                           int *__restrict__ out, int out_stride, int out_off) {
    __shared__ double sm[SL_THREADS];
    __shared__ int s_min;
    const int b = blockIdx.x, tid = threadIdx.x;
    const float *kf = (const float *)keys + (size_t)b * V;
    const unsigned long long *k8 = (const unsigned long long *)keys + (size_t)b * V;
    auto val = [&](int r) -> double {
        if (K64) return (double)okey_inv(0xffffffffu - (unsigned)(k8[r] & 0xffffffffull));
        return (double)kf[r];
    };
    const int *ir = idx + (size_t)b * V;
    const double mx = val(0);
    const int chunk = (keep + SL_THREADS - 1) / SL_THREADS;
    const int r0 = tid * chunk, r1 = min(r0 + chunk, keep);
    double local = 0;
    // the exponentials are taken once and kept: the passes below read them back. A thread's i-th entry sits at
    // [i][thread], so that a warp's accesses fall into one line although every thread walks its own run of ranks
    double *pc = pcache + (size_t)b * ((size_t)chunk * SL_THREADS) + tid;
    for (int r = r0; r < r1; r++) { const double p = exp(val(r) - mx); pc[(size_t)(r - r0) * SL_THREADS] = p; local += p; }
    double den;
    const double base = block_excl_scan(local, sm, &den);
    // nucleus cut: first rank with (cum_before - p) / den > top_p
    if (tid == 0) s_min = keep;
    __syncthreads();
    {
        double cum = base;
        for (int r = r0; r < r1; r++) {
            double p = pc[(size_t)(r - r0) * SL_THREADS];
            if ((cum - p) / den > (double)top_p) { atomicMin(&s_min, r); break; }
            cum += p;
        }
    }
    __syncthreads();
    const int nkeep = s_min;
    __syncthreads();
    // mass of the kept prefix
    double lk = 0;
    for (int r = r0; r < r1 && r < nkeep; r++) lk += pc[(size_t)(r - r0) * SL_THREADS];
    double den2;
    const double base2 = block_excl_scan(lk, sm, &den2);
    const double u01 = uniforms ? uniforms[b] : counter_uniform(seed, row0 + b, level, 0);
    const double u = u01 * den2;
    if (tid == 0) s_min = nkeep - 1;
    __syncthreads();
    {
        double acc = base2;
        for (int r = r0; r < r1 && r < nkeep; r++) {
            acc += pc[(size_t)(r - r0) * SL_THREADS];
            if (u <= acc) { atomicMin(&s_min, r); break; }
        }
    }
    __syncthreads();
    if (tid == 0) out[(size_t)b * out_stride + out_off] = ir[s_min < 0 ? 0 : s_min];
}

// ---- the same draw without sorting the row (top_k = 0: the nucleus is cut from the whole vocabulary) ----
// With seeded or near-uniform logits the nucleus holds most of a 150 K vocabulary, so the sort above is the
// sampler. Both the cut ("cum_before - p > top_p") and the draw ("u <= cum") are the first rank at which a
// monotone predicate over cumulative probability turns true, so each can be found the way a radix select finds
// a rank: three passes over the row's ordered 32-bit keys (11 + 11 + 10 bits), each building per-bin probability
// mass, element counts and the smallest / largest key of a bin, descending into the bin where the predicate
// flips. Probabilities are accumulated as 64-bit fixed point (2^-44 steps, exact and order-independent integer
// sums, so runs are reproducible whatever order the atomics land in); the absolute error of a cumulative sum is
// below 1e-11 of the row's mass, which moves a draw only when it falls that close to a boundary. Ties of equal
// logits are ranked by ascending index, like the stable sort.
constexpr int NS_THREADS = 1024;
constexpr int NS_BINS = 2048;
constexpr double NS_FIX = 17592186044416.0;                       // 2^44

struct NsHist {
    unsigned long long sum[NS_BINS];
    unsigned cnt[NS_BINS];
    unsigned kmin_inv[NS_BINS];       // ~(smallest key of the bin): zero-initialised storage, atomicMax
};
// A CTA's shared-memory copy. The 45-bit masses are added as three 15-bit limbs with native 32-bit atomics (a 64-bit
// shared-memory add is a compare-and-swap loop, and the rows' keys cluster in a few bins: it was 0.6 of the 0.7 ms
// the first sweep took at 256 rows). A limb sum stays below 2^32 for up to 2^17 elements per CTA.
constexpr int NS_MAX_PER_CTA = 1 << 17;
struct NsShHist {
    unsigned s0[NS_BINS], s1[NS_BINS], s2[NS_BINS];
    unsigned cnt[NS_BINS];
    unsigned kmin_inv[NS_BINS];
    __device__ __forceinline__ void clear(int nbins) {
        for (int i = threadIdx.x; i < nbins; i += NS_THREADS) { s0[i] = 0; s1[i] = 0; s2[i] = 0; cnt[i] = 0; kmin_inv[i] = 0; }
    }
    __device__ __forceinline__ void add(int bin, unsigned k, unsigned long long qv) {
        atomicAdd(&s0[bin], (unsigned)(qv & 0x7fffull));
        atomicAdd(&s1[bin], (unsigned)((qv >> 15) & 0x7fffull));
        atomicAdd(&s2[bin], (unsigned)(qv >> 30));
        atomicAdd(&cnt[bin], 1u);
        atomicMax(&kmin_inv[bin], ~k);
    }
    __device__ __forceinline__ void flush(int nbins, NsHist *gh) {
        for (int i = threadIdx.x; i < nbins; i += NS_THREADS)
            if (cnt[i]) {
                atomicAdd(&gh->sum[i], (unsigned long long)s0[i] + ((unsigned long long)s1[i] << 15) + ((unsigned long long)s2[i] << 30));
                atomicAdd(&gh->cnt[i], cnt[i]);
                atomicMax(&gh->kmin_inv[i], kmin_inv[i]);
            }
    }
};
// Per-row state handed from one kernel of the sequence to the next. A field is written by the first CTA of a row
// in one kernel and read only by LATER kernels (the CTAs of a kernel each repeat its decision for themselves), hence
// one slot per stage for the fields that change from stage to stage.
struct NsRow {
    unsigned maxkey;
    int n_done[2];                     // nucleus cut resolved by the first / second level (den2 valid)
    unsigned n_prefix[2];              // key bits fixed by the nucleus descent after its first / second level
    unsigned long long n_above[2];     // mass strictly above the nucleus descent's range after those levels
    unsigned long long total, den2;    // mass of the row / of the kept prefix
    unsigned p_prefix[2];
    unsigned long long p_above[2];
    double U;                          // the draw, in fixed-point units of mass
    unsigned n_cand;                   // entries the last histogram pass put on the row's candidate list
};
constexpr int NS_CAND = 2048;          // (key, index) pairs per row kept for the final index search

__device__ __forceinline__ unsigned long long ns_q_of_key(unsigned key, double mx) {
    return __double2ull_rn(exp((double)okey_inv(key) - mx) * NS_FIX);
}

// exclusive block scan of one u64 per thread (NS_THREADS threads); every thread gets its prefix
__device__ __forceinline__ unsigned long long ns_block_excl_scan(unsigned long long v, unsigned long long *wsum) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned long long x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        unsigned long long y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
    }
    __syncthreads();                                               // wsum may still be read from an earlier call
    if (lane == 31) wsum[warp] = x;
    __syncthreads();
    unsigned long long base = 0;
    for (int w = 0; w < warp; w++) base += wsum[w];
    return base + x - v;
}

// One level of a descent over a histogram of `nbins` bins, highest bin first. NUCLEUS: the first bin whose LAST
// element satisfies cum_before - p > T (the cut then lies inside that bin or exactly in front of it; the descent
// into the bin settles which). Otherwise: the first bin with cum_incl >= T. Results through shared memory:
// *sel = bin (-1: no bin satisfies), *sel_above = mass above that bin; *first_hit is always 0.
template <bool NUCLEUS>
__device__ void ns_decide(const NsHist *h, int nbins, unsigned long long above, double T, double mx, unsigned key_hi, int shift,
                          unsigned long long *wsum, int *sel, unsigned long long *sel_above, int *first_hit) {
    const int tid = threadIdx.x;
    unsigned long long s[2]; int bin[2];
#pragma unroll
    for (int e = 0; e < 2; e++) {
        const int d = 2 * tid + e;
        bin[e] = nbins - 1 - d;
        s[e] = (d < nbins) ? h->sum[bin[e]] : 0ull;
    }
    if (tid == 0) { *sel = 0x7fffffff; *first_hit = 0; }
    const unsigned long long ex = ns_block_excl_scan(s[0] + s[1], wsum);    // contains a __syncthreads after the init above
    unsigned long long ab = above + ex;
#pragma unroll
    for (int e = 0; e < 2; e++) {
        const int d = 2 * tid + e;
        if (d < nbins && h->cnt[bin[e]] > 0) {
            bool hit;
            if (NUCLEUS) {
                const unsigned kmin = ~h->kmin_inv[bin[e]];
                const long long g = (long long)(ab + s[e]) - 2ll * (long long)ns_q_of_key(kmin, mx);
                hit = (double)g > T;
            } else {
                hit = (double)(ab + s[e]) >= T;
            }
            if (hit) atomicMin(sel, d);
        }
        ab += s[e];
    }
    __syncthreads();
    const int dsel = *sel;
    __syncthreads();
    if (dsel == 0x7fffffff) { if (tid == 0) *sel = -1; __syncthreads(); return; }
    if (dsel >> 1 == tid) {
        const int e = dsel & 1;
        const unsigned long long a0 = above + ex + (e ? s[0] : 0ull);
        *sel = bin[e];
        *sel_above = a0;
    }
    __syncthreads();
}

__global__ void __launch_bounds__(NS_THREADS) k_ns_max(const float *__restrict__ logits, float temp, int V, NsRow *rows) {
    const int b = blockIdx.y;
    const float *lg = logits + (size_t)b * V;
    unsigned m = 0;
    for (int i = blockIdx.x * NS_THREADS + threadIdx.x; i < V; i += gridDim.x * NS_THREADS) m = max(m, okey(lg[i] / temp));
    for (int o = 16; o; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) atomicMax(&rows[b].maxkey, m);
}

// accumulates the elements of this CTA's slice whose key, shifted right by `fshift`, equals `want` (fshift = 32:
// every element) into the histogram of the next `bits` key bits below that; shared histogram, then one atomic
// per touched bin into the row's global one
__device__ void ns_histogram(const unsigned *__restrict__ keys, const unsigned long long *__restrict__ q, int V, int fshift, unsigned want,
                             int shift, int nbins, NsShHist *sh, NsHist *gh, unsigned *n_cand = nullptr, unsigned long long *cand = nullptr) {
    sh->clear(nbins);
    __syncthreads();
    // (Combining the lanes of a warp that fall into the same bin first -- match + warp reductions, one lane per
    // distinct bin touching shared memory -- measured slower than these plain shared-memory atomics: 2.6 against
    // 1.5 ms per step at 256 rows of 151 936 entries.)
    for (int i = blockIdx.x * NS_THREADS + threadIdx.x; i < V; i += gridDim.x * NS_THREADS) {
        const unsigned k = keys[i];
        if (fshift < 32 && (k >> fshift) != want) continue;
        const int bin = (int)((k >> shift) & (unsigned)(nbins - 1));
        sh->add(bin, k, q[i]);
        if (n_cand) {      // last level of the pick descent: the handful of entries left are kept with their indices
            const unsigned at = atomicAdd(n_cand, 1u);
            if (at < (unsigned)NS_CAND) cand[at] = ((unsigned long long)k << 32) | (unsigned)i;
        }
    }
    __syncthreads();
    sh->flush(nbins, gh);
}

// keys, fixed-point probabilities and the histogram of the top 11 key bits
__global__ void __launch_bounds__(NS_THREADS) k_ns_prob(const float *__restrict__ logits, float temp, int V, NsRow *rows, unsigned *keys,
                                                        unsigned long long *q, NsHist *hist) {
    __shared__ NsShHist sh;
    const int b = blockIdx.y;
    const float *lg = logits + (size_t)b * V;
    unsigned *kr = keys + (size_t)b * V;
    unsigned long long *qr = q + (size_t)b * V;
    const double mx = (double)okey_inv(rows[b].maxkey);
    NsHist *gh = hist + (size_t)b * 5;
    sh.clear(NS_BINS);
    __syncthreads();
    // keys and masses are stored for the later passes and enter the top-level histogram in the same sweep
    for (int i = blockIdx.x * NS_THREADS + threadIdx.x; i < V; i += gridDim.x * NS_THREADS) {
        const unsigned k = okey(lg[i] / temp);
        const unsigned long long qv = ns_q_of_key(k, mx);
        kr[i] = k;
        qr[i] = qv;
        sh.add((int)(k >> 21), k, qv);
    }
    __syncthreads();
    sh.flush(NS_BINS, gh);
}

// STAGE 2, 3: nucleus descent (decide on the previous histogram, build the next); 4: end of the nucleus descent,
// the draw, first level of the pick descent; 5: second level of the pick descent
template <int STAGE>
__global__ void __launch_bounds__(NS_THREADS) k_ns_refine(int V, float top_p, const double *__restrict__ uniforms, unsigned long long seed,
                                                          long long row0, int level, NsRow *rows, const unsigned *keys,
                                                          const unsigned long long *q, NsHist *hist, unsigned long long *cand) {
    __shared__ NsShHist sh;
    __shared__ unsigned long long wsum[32];
    __shared__ int s_sel, s_first;
    __shared__ unsigned long long s_above;
    const int b = blockIdx.y, tid = threadIdx.x;
    NsRow *row = rows + b;
    NsHist *H = hist + (size_t)b * 5;                              // 0: top bits | 1, 2: nucleus levels | 3, 4: pick levels
    const unsigned *kr = keys + (size_t)b * V;
    const unsigned long long *qr = q + (size_t)b * V;
    const double mx = (double)okey_inv(row->maxkey);
    const bool lead = blockIdx.x == 0 && tid == 0;
    const unsigned long long total = (STAGE == 2) ? 0ull : row->total;
    if (STAGE == 2) {
        // total mass = sum over the top-level bins (every CTA computes it; the leader records it)
        unsigned long long t = H[0].sum[2 * tid] + H[0].sum[2 * tid + 1];
        const unsigned long long ex = ns_block_excl_scan(t, wsum);
        __shared__ unsigned long long s_total;
        if (tid == NS_THREADS - 1) s_total = ex + t;
        __syncthreads();
        const unsigned long long tot = s_total;
        if (lead) row->total = tot;
        if (!(top_p < 1.0f)) { if (lead) { row->n_done[0] = 1; row->den2 = tot; } return; }
        const double T = (double)top_p * (double)tot;
        ns_decide<true>(&H[0], NS_BINS, 0ull, T, mx, 0u, 21, wsum, &s_sel, &s_above, &s_first);
        if (s_sel < 0) { if (lead) { row->n_done[0] = 1; row->den2 = tot; } return; }       // the cut is never reached
        if (s_first) { if (lead) { row->n_done[0] = 1; row->den2 = s_above; } return; }
        if (lead) { row->n_prefix[0] = (unsigned)s_sel; row->n_above[0] = s_above; }
        ns_histogram(kr, qr, V, 21, (unsigned)s_sel, 10, NS_BINS, &sh, &H[1]);
        return;
    }
    if (STAGE == 3) {
        if (row->n_done[0]) return;
        const double T = (double)top_p * (double)total;
        ns_decide<true>(&H[1], NS_BINS, row->n_above[0], T, mx, 0u, 10, wsum, &s_sel, &s_above, &s_first);
        // the parent bin's last element satisfies the predicate, so a bin is always found
        const unsigned pre = (row->n_prefix[0] << 11) | (unsigned)(s_sel < 0 ? 0 : s_sel);
        if (s_first || s_sel < 0) { __syncthreads(); if (lead) { row->n_done[1] = 1; row->den2 = s_sel < 0 ? total : s_above; } return; }
        __syncthreads();
        if (lead) { row->n_prefix[1] = pre; row->n_above[1] = s_above; }
        ns_histogram(kr, qr, V, 10, pre, 0, 1024, &sh, &H[2]);
        return;
    }
    if (STAGE == 4) {
        unsigned long long den2 = row->den2;
        if (!row->n_done[0] && !row->n_done[1]) {
            const double T = (double)top_p * (double)total;
            ns_decide<true>(&H[2], 1024, row->n_above[1], T, mx, 0u, 0, wsum, &s_sel, &s_above, &s_first);
            // the bin is one exact key held by cnt tied elements of mass qk each: the j-th of them (ascending index)
            // has cum_before - p = above + (j - 1) qk; the cut is the first j for which that exceeds T
            den2 = total;
            if (s_sel >= 0) {
                const unsigned long long qk = ns_q_of_key((row->n_prefix[1] << 10) | (unsigned)s_sel, mx);
                const long long cnt = (long long)H[2].cnt[s_sel];
                long long j = 0;
                if (qk > 0) {
                    j = (long long)floor((T - (double)s_above) / (double)qk) + 1;
                    if (j < 0) j = 0;
                    if (j > cnt) j = cnt;
                    while (j > 0 && (double)((long long)s_above + (j - 2) * (long long)qk) > T) j--;       // smallest j with the predicate true
                    while (j < cnt && !((double)((long long)s_above + (j - 1) * (long long)qk) > T)) j++;
                }
                den2 = s_above + (unsigned long long)j * qk;
            }
            __syncthreads();
        }
        const double u01 = uniforms ? uniforms[b] : counter_uniform(seed, row0 + b, level, 0);
        const double U = u01 * (double)den2;
        if (lead) { row->den2 = den2; row->U = U; }
        ns_decide<false>(&H[0], NS_BINS, 0ull, U, mx, 0u, 21, wsum, &s_sel, &s_above, &s_first);
        int sel = s_sel;
        unsigned long long ab = s_above;
        if (sel < 0) {                                              // rounding put the draw past the last mass: take the lowest occupied bin
            sel = 0; ab = 0;
            __syncthreads();
            if (tid == 0) { int bsel = -1; unsigned long long acc = 0, accb = 0; for (int i = NS_BINS - 1; i >= 0; i--) if (H[0].cnt[i]) { bsel = i; accb = acc; acc += H[0].sum[i]; } s_sel = bsel; s_above = accb; }
            __syncthreads();
            sel = s_sel; ab = s_above;
        }
        __syncthreads();
        if (lead) { row->p_prefix[0] = (unsigned)sel; row->p_above[0] = ab; }
        ns_histogram(kr, qr, V, 21, (unsigned)sel, 10, NS_BINS, &sh, &H[3]);
        return;
    }
    if (STAGE == 5) {
        ns_decide<false>(&H[3], NS_BINS, row->p_above[0], row->U, mx, 0u, 10, wsum, &s_sel, &s_above, &s_first);
        int sel = s_sel;
        unsigned long long ab = s_above;
        if (sel < 0) {
            __syncthreads();
            if (tid == 0) { int bsel = 0; unsigned long long acc = row->p_above[0], accb = acc; for (int i = NS_BINS - 1; i >= 0; i--) if (H[3].cnt[i]) { bsel = i; accb = acc; acc += H[3].sum[i]; } s_sel = bsel; s_above = accb; }
            __syncthreads();
            sel = s_sel; ab = s_above;
        }
        const unsigned pre = (row->p_prefix[0] << 11) | (unsigned)sel;
        __syncthreads();
        if (lead) { row->p_prefix[1] = pre; row->p_above[1] = ab; }
        ns_histogram(kr, qr, V, 10, pre, 0, 1024, &sh, &H[4], &row->n_cand, cand + (size_t)b * NS_CAND);
        return;
    }
}

// last level of the pick descent, then the index: the pick_tie-th (ascending index) element holding the chosen key
__global__ void __launch_bounds__(NS_THREADS) k_ns_pick(int V, NsRow *rows, const unsigned *keys, NsHist *hist, const unsigned long long *cand,
                                                        int *__restrict__ out, int out_stride, int out_off) {
    __shared__ unsigned long long wsum[32];
    __shared__ int s_sel, s_first, s_n, s_list[2048];
    __shared__ unsigned long long s_above;
    const int b = blockIdx.x, tid = threadIdx.x;
    NsRow *row = rows + b;
    NsHist *H = hist + (size_t)b * 5;
    const unsigned *kr = keys + (size_t)b * V;
    const double mx = (double)okey_inv(row->maxkey);
    ns_decide<false>(&H[4], 1024, row->p_above[1], row->U, mx, 0u, 0, wsum, &s_sel, &s_above, &s_first);
    if (s_sel < 0) {
        __syncthreads();
        if (tid == 0) { int bsel = 0; unsigned long long acc = row->p_above[1], accb = acc; for (int i = 1023; i >= 0; i--) if (H[4].cnt[i]) { bsel = i; accb = acc; acc += H[4].sum[i]; } s_sel = bsel; s_above = accb; }
        __syncthreads();
    }
    const unsigned key = (row->p_prefix[1] << 10) | (unsigned)s_sel;
    const long long cnt = (long long)H[4].cnt[s_sel];
    const unsigned long long qk = ns_q_of_key(key, mx);
    // the j-th tied element has cum_incl = above + (j + 1) qk: the first j for which that reaches U
    long long j = 0;
    if (qk > 0 && cnt > 1) {
        j = (long long)ceil((row->U - (double)s_above) / (double)qk) - 1;
        if (j < 0) j = 0;
        if (j > cnt - 1) j = cnt - 1;
        while (j > 0 && (double)(s_above + (unsigned long long)j * qk) >= row->U) j--;
        while (j < cnt - 1 && !((double)(s_above + (unsigned long long)(j + 1) * qk) >= row->U)) j++;
    }
    if (tid == 0) s_n = 0;
    __syncthreads();
    // indices holding the key (a handful at most for real logits; a constant row makes it the whole vocabulary)
    if (cnt <= 2048) {
        const unsigned nc = row->n_cand;
        if (nc <= (unsigned)NS_CAND) {
            // the entries sharing the key's upper 22 bits were listed by the last histogram pass: no sweep over the row
            const unsigned long long *cl = cand + (size_t)b * NS_CAND;
            for (unsigned i = tid; i < nc; i += NS_THREADS) {
                const unsigned long long e = cl[i];
                if ((unsigned)(e >> 32) == key) { int at = atomicAdd(&s_n, 1); if (at < 2048) s_list[at] = (int)(unsigned)(e & 0xffffffffull); }
            }
        } else {
            for (int i = tid; i < V; i += NS_THREADS)
                if (kr[i] == key) { int at = atomicAdd(&s_n, 1); if (at < 2048) s_list[at] = i; }
        }
        __syncthreads();
        const int n = s_n < 2048 ? s_n : 2048;
        for (int e = tid; e < n; e += NS_THREADS) {
            int r = 0;
            for (int f = 0; f < n; f++) r += s_list[f] < s_list[e];
            if (r == (int)j) out[(size_t)b * out_stride + out_off] = s_list[e];
        }
    } else {
        // many ties: the j-th match in index order, by counting matches per thread slice and scanning
        const int per = (V + NS_THREADS - 1) / NS_THREADS, i0 = tid * per, i1 = min(V, i0 + per);
        unsigned long long c = 0;
        for (int i = i0; i < i1; i++) c += kr[i] == key;
        const unsigned long long ex = ns_block_excl_scan(c, wsum);
        if ((unsigned long long)j >= ex && (unsigned long long)j < ex + c) {
            long long need = j - (long long)ex;
            for (int i = i0; i < i1; i++)
                if (kr[i] == key && need-- == 0) { out[(size_t)b * out_stride + out_off] = i; break; }
        }
    }
}

static bool sample_rows_select(const SampleArgs &a) {
    // NCM_B200_SORT_SAMPLER=1 keeps the sort-based path (read per call: tests compare the two on the same rows);
    // NCM_B200_SELECT_MIN_V lowers the vocabulary size from which the selection path is taken (default 4096)
    const char *e = getenv("NCM_B200_SORT_SAMPLER"), *mv = getenv("NCM_B200_SELECT_MIN_V");
    if ((e && atoi(e)) || a.V < (mv ? atoi(mv) : 4096)) return false;
    static Workspace ws;
    const size_t n = (size_t)a.Bn * a.V;
    const size_t head = ((size_t)a.Bn * sizeof(NsRow) + (size_t)a.Bn * 5 * sizeof(NsHist) + 255) & ~(size_t)255;
    const size_t need = head + n * 12 + (size_t)a.Bn * NS_CAND * 8 + 8192;
    if (need > ws.cap) ws.reserve(need + need / 8);
    ws.reset();
    char *base = (char *)ws.alloc(head);
    NsRow *rows = (NsRow *)base;
    NsHist *hist = (NsHist *)(base + (((size_t)a.Bn * sizeof(NsRow) + 15) & ~(size_t)15));
    unsigned long long *q = ws.get<unsigned long long>(n);
    unsigned *keys = ws.get<unsigned>(n);
    unsigned long long *cand = ws.get<unsigned long long>((size_t)a.Bn * NS_CAND);
    ProfScope ps(NCMB_K_SAMPLE, 0, (double)n * 40);
    CUDA_CHECK(cudaMemsetAsync(base, 0, head, stream()));
    // CTAs per row: enough to occupy the GPU when there are few rows
    int G = (2 * ctx().sm_count + a.Bn - 1) / a.Bn;
    const int gmax = (a.V + 4 * NS_THREADS - 1) / (4 * NS_THREADS);
    if (G > gmax) G = gmax;
    if (G > 32) G = 32;
    const int gmin = (a.V + NS_MAX_PER_CTA - 1) / NS_MAX_PER_CTA;          // the limb sums of a CTA's histogram must not wrap
    if (G < gmin) G = gmin;
    if (G < 1) G = 1;
    const dim3 grid((unsigned)G, (unsigned)a.Bn);
    LAUNCH(k_ns_max, grid, NS_THREADS, 0, a.logits, a.temp, a.V, rows);
    LAUNCH(k_ns_prob, grid, NS_THREADS, 0, a.logits, a.temp, a.V, rows, keys, q, hist);
    LAUNCH(k_ns_refine<2>, grid, NS_THREADS, 0, a.V, a.top_p, a.uniforms, a.rng_seed, a.rng_row0, a.rng_level, rows, (const unsigned *)keys, (const unsigned long long *)q, hist, cand);
    LAUNCH(k_ns_refine<3>, grid, NS_THREADS, 0, a.V, a.top_p, a.uniforms, a.rng_seed, a.rng_row0, a.rng_level, rows, (const unsigned *)keys, (const unsigned long long *)q, hist, cand);
    LAUNCH(k_ns_refine<4>, grid, NS_THREADS, 0, a.V, a.top_p, a.uniforms, a.rng_seed, a.rng_row0, a.rng_level, rows, (const unsigned *)keys, (const unsigned long long *)q, hist, cand);
    LAUNCH(k_ns_refine<5>, grid, NS_THREADS, 0, a.V, a.top_p, a.uniforms, a.rng_seed, a.rng_row0, a.rng_level, rows, (const unsigned *)keys, (const unsigned long long *)q, hist, cand);
    LAUNCH(k_ns_pick, (unsigned)a.Bn, NS_THREADS, 0, a.V, rows, (const unsigned *)keys, hist, (const unsigned long long *)cand, a.out, a.out_stride, a.out_off);
    return true;
}

static void sample_rows_large(const SampleArgs &a, int keep) {
    if (a.Lc != 1 || a.uncond_off || a.freq > 0.f || a.adj_a != 0.f)
        fatal("sampling: more than %d candidates (top_k=%d, V=%d) is supported for single-position rows "
              "without CFG or penalties only; set top_k <= %d", SM_MAXKEEP, a.top_k, a.V, SM_MAXKEEP);
    if (keep == a.V && sample_rows_select(a)) return;
    static Workspace ws;
    const int64_t n = (int64_t)a.Bn * a.V;
    // One row: a device-wide 32-bit radix sort. More rows: ONE device-wide sort of all rows on composite keys
    // (row index above the value bits); a segmented sort gives each row a single CTA, about a millisecond for a
    // 150 K vocabulary whatever the number of rows.
    const bool per_row = a.Bn == 1;
    int row_bits = 1;
    while ((1 << row_bits) < a.Bn) row_bits++;
    size_t temp_bytes = 0;
    if (per_row)
        cub::DeviceRadixSort::SortPairsDescending(nullptr, temp_bytes, (const float *)nullptr, (float *)nullptr,
                                                  (const int *)nullptr, (int *)nullptr, a.V, 0, 32, stream());
    else
        cub::DeviceRadixSort::SortPairs(nullptr, temp_bytes, (const unsigned long long *)nullptr, (unsigned long long *)nullptr,
                                        (const int *)nullptr, (int *)nullptr, n, 0, 32 + row_bits, stream());
    const size_t pc_per_row = (size_t)cdiv(keep, SL_THREADS) * SL_THREADS;
    size_t need = (size_t)n * 24 + (size_t)a.Bn * pc_per_row * 8 + temp_bytes + 8192;
    if (need > ws.cap) ws.reserve(need);
    ws.reset();
    ProfScope ps(NCMB_K_SAMPLE, 0, (double)n * 40);
    int64_t g = cdiv(n, 256), cap = (int64_t)ctx().sm_count * 16;
    cudaError_t e = cudaSuccess;
    if (per_row) {
        float *k_in = ws.get<float>(n), *k_out = ws.get<float>(n);
        int *i_in = ws.get<int>(n), *i_out = ws.get<int>(n);
        void *temp = ws.alloc(temp_bytes);
        double *pcache = ws.get<double>((size_t)a.Bn * pc_per_row);
        LAUNCH(k_sort_prep, (unsigned)(g > cap ? cap : g), 256, 0, a.logits, a.temp, n, a.V, k_in, i_in);
        e = cub::DeviceRadixSort::SortPairsDescending(temp, temp_bytes, k_in, k_out, i_in, i_out, a.V, 0, 32, stream());
        ctx().launches += 7;
        if (e != cudaSuccess) fatal("radix sort failed: %s", cudaGetErrorString(e));
        LAUNCH(k_pick_sorted<false>, (unsigned)a.Bn, SL_THREADS, 0, (const void *)k_out, (const int *)i_out, pcache, a.V, keep, a.top_p, a.uniforms, a.rng_seed,
               a.rng_row0, a.rng_level, a.out, a.out_stride, a.out_off);
    } else {
        unsigned long long *k_in = ws.get<unsigned long long>(n), *k_out = ws.get<unsigned long long>(n);
        int *i_in = ws.get<int>(n), *i_out = ws.get<int>(n);
        void *temp = ws.alloc(temp_bytes);
        double *pcache = ws.get<double>((size_t)a.Bn * pc_per_row);
        LAUNCH(k_sort_prep64, (unsigned)(g > cap ? cap : g), 256, 0, a.logits, a.temp, n, a.V, k_in, i_in);
        e = cub::DeviceRadixSort::SortPairs(temp, temp_bytes, k_in, k_out, i_in, i_out, n, 0, 32 + row_bits, stream());
        ctx().launches += 2 * ((32 + row_bits + 7) / 8) + 1;
        if (e != cudaSuccess) fatal("radix sort failed: %s", cudaGetErrorString(e));
        LAUNCH(k_pick_sorted<true>, (unsigned)a.Bn, SL_THREADS, 0, (const void *)k_out, (const int *)i_out, pcache, a.V, keep, a.top_p, a.uniforms, a.rng_seed,
               a.rng_row0, a.rng_level, a.out, a.out_stride, a.out_off);
    }
}

void sample_rows(const SampleArgs &a) {
    if (a.Bn <= 0 || a.Lc <= 0) return;
    if (a.temp > 0.f) {
        int keep = (a.top_k > 0) ? (a.top_k < a.V ? a.top_k : a.V) : a.V;
        if (keep > SM_MAXKEEP) { sample_rows_large(a, keep); return; }
    }
    if (const int Kc = two_phase_width(a)) {
        static unsigned long long *cand = nullptr; static size_t cand_cap = 0;
        const size_t need = (size_t)a.Bn * a.Lc * Kc;
        if (need > cand_cap) {
            if (cand) { CUDA_CHECK(cudaStreamSynchronize(stream())); dev_free(cand); }
            cand = (unsigned long long *)dev_alloc(need * 8); cand_cap = need;
        }
        SampleCand sc;
        sc.a = a; sc.Kc = Kc; sc.cand = cand;
        static bool set = false;
        if (!set) { CUDA_CHECK(cudaFuncSetAttribute(k_sample_topc, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * SM_SMEM_V)); set = true; }
        ProfScope ps(NCMB_K_SAMPLE, 0, (double)a.Bn * a.Lc * a.V * (a.uncond_off ? 8 : 4));
        LAUNCH(k_sample_topc, (unsigned)(a.Bn * a.Lc), SM_THREADS, sizeof(float) * (size_t)a.V, sc);
        LAUNCH(k_sample_seq, (unsigned)a.Bn, Kc, 0, sc);           // one thread per candidate
        return;
    }
    SampleDev sd;
    sd.a = a;
    sd.vals_in_smem = a.V <= SM_SMEM_V;
    if (!sd.vals_in_smem && !a.scratch) fatal("sampling: V=%d needs a scratch buffer", a.V);
    size_t smem = 16 * (size_t)SM_MAXKEEP + (sd.vals_in_smem ? sizeof(float) * (size_t)a.V : 0);
    static size_t attr = 0;
    if (smem > attr) {
        CUDA_CHECK(cudaFuncSetAttribute(k_sample, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(16 * SM_MAXKEEP + 4 * SM_SMEM_V)));
        attr = 16 * SM_MAXKEEP + 4 * SM_SMEM_V;
    }
    ProfScope ps(NCMB_K_SAMPLE, 0, (double)a.Bn * a.Lc * a.V * (a.uncond_off ? 8 : 4));
    LAUNCH(k_sample, (unsigned)a.Bn, SM_THREADS, smem, sd);
}

} // namespace ncmb

// Diagnostic: the device sampler on caller-supplied DEVICE rows, one position per row, no CFG and no penalties --
// sample_topkp's rule (src/kernels.c:794-825) with the uniform of row b taken from uniforms[b] (device doubles in
// [0, 1)). picks: device int[B].
extern "C" void ncmb_sample_rows_dev(const float *logits, int B, int V, float temp, int top_k, float top_p,
                                     const double *uniforms, int *picks) {
    using namespace ncmb;
    ensure_device();
    SampleArgs s{};
    s.logits = logits; s.Bn = B; s.Lc = 1; s.V = V; s.temp = temp; s.top_k = top_k; s.top_p = top_p;
    s.uniforms = uniforms; s.out = picks; s.out_stride = 1; s.out_off = 0; s.picks_bound = 1;
    float *scr = nullptr;
    const size_t need = sample_scratch_floats(B, V);
    if (need) { scr = (float *)dev_alloc(need * 4); s.scratch = scr; }
    sample_rows(s);
    CUDA_CHECK(cudaStreamSynchronize(stream()));
    if (scr) dev_free(scr);
}

// Host-side sampling helper of the reference kernel API (src/ncm.h:197): logits is a
// host row; same algorithm and the same single uniform draw per call.
static const float *g_sort_vals;
static int cmp_desc_idx(const void *pa, const void *pb) {
    float va = g_sort_vals[*(const int *)pa], vb = g_sort_vals[*(const int *)pb];
    return (va < vb) - (va > vb);
}
extern "C" int sample_topkp(const float *logits, int V, float temp, int top_k, float top_p, unsigned long long *rng) {
    if (!(temp > 0)) return argmax_row(logits, V);
    float *work = (float *)malloc((size_t)V * sizeof(float));
    int *ord = (int *)malloc((size_t)V * sizeof(int));
    double *probs = (double *)malloc((size_t)V * sizeof(double));
    if (!work || !ord || !probs) ncmb::fatal("oom in sample_topkp");
    for (int i = 0; i < V; i++) { work[i] = logits[i] / temp; ord[i] = i; }
    g_sort_vals = work;
    qsort(ord, (size_t)V, sizeof(int), cmp_desc_idx);
    int keep = (top_k > 0) ? (top_k < V ? top_k : V) : V;
    double mx = work[ord[0]], den = 0;
    for (int r = 0; r < keep; r++) { probs[r] = exp((double)work[ord[r]] - mx); den += probs[r]; }
    for (int r = 0; r < keep; r++) probs[r] /= den;
    double cum = 0;
    int nkeep = keep;
    for (int r = 0; r < keep; r++) { if (cum - probs[r] > top_p) { nkeep = r; break; } cum += probs[r]; }
    den = 0;
    for (int r = 0; r < nkeep; r++) den += probs[r];
    double u = (double)(rng_next(rng) >> 11) * (1.0 / 9007199254740992.0) * den, acc = 0;
    int pick = ord[nkeep - 1];
    for (int r = 0; r < nkeep; r++) { acc += probs[r]; if (u <= acc) { pick = ord[r]; break; } }
    free(work); free(ord); free(probs);
    return pick;
}
