// Tensor-core attention for head dim 64 on sm_100a (tcgen05 + TMEM + TMA).
//
// One CTA (512 threads) per (sequence row, head, 128-query tile):
//   S = Q K^T   tcgen05.mma.kind::tf32 into tensor memory; the query tile and ALL keys of the row (up to 288
//               padded keys: a 256-token prefix plus a 32-token level) are fetched together by TMA and stay
//               resident, so the score phase is one load, one split pass and one batch of MMAs
//   softmax     four threads per query row (each takes a quarter of the columns) read the scores with
//               tcgen05.ld; all keys of a row are resident, so the row maximum is known before
//               any exponential is taken and no rescaling is needed
//   O += P V    per 32-key chunk: P is written to shared memory by the softmax threads, V (fetched
//               for up to eight chunks ahead) is transposed on chip, tcgen05.mma accumulates the
//               128 x 64 output in TMEM; P / V^T are double-buffered so the MMAs of one chunk run
//               under the softmax of the next
// Scores are three TF32 MMAs over hi/lo splits (a = a_hi + a_lo), formed on chip from the fp32 tiles TMA
// brings in. P V runs on fp16 pairs (v = v1 + v2 * 2^-11, as the fp16-pair GEMM does): main += p1 v1 and
// cross += p1 v2 + p2 v1 in two accumulators, O = main + cross * 2^-11 -- six kind::f16 MMAs per chunk where
// TF32 needed twelve of half the depth, and that chain of small MMAs is what paces the chunk loop. Both
// are fp32-grade like the CUDA-core kernel. Two chunks share one hand-over: P and V^T tiles are 64 keys wide
// (one 128-byte-swizzled row of fp16), hi and lo in tiles of their own.
// Key rows come from up to two segments (cached prefix, tokens of the current pass); each
// segment is padded to a multiple of 32 score columns and the padding is masked in the softmax.
//
// Shared memory, reused between the two phases:
//   QA  (64 KB)   Q hi | Q lo                                 then  V^T pairs, two buffers (32 KB)
//   KA  (144 KB)  K hi atoms | K lo atoms, 288 rows each      then  raw V, one 8 KB slot per 32-key chunk (72 KB)
//                                                                   and P pairs, two buffers (64 KB)
#include "common.cuh"
#include "tc_common.cuh"
#include "split.cuh"

namespace ncmb {

constexpr int ATC_THREADS = 512;          // softmax team: four threads per query row, eight score columns of a chunk each
constexpr int ATC_BLOCK = ATC_THREADS + 32;  // + one warp whose first lane issues the PV MMAs while the team works on the next chunk
constexpr int ATC_MAXK = 288;            // padded keys per row the kernel keeps resident
constexpr int ATC_OCOL = 288;            // TMEM columns of the output accumulators (main, then cross terms); scores use [0, 288)
constexpr int ATC_PBUF = 32768, ATC_VBUF = 16384;  // P hi | lo tiles (128 rows x 128 B each) / V^T hi | lo tiles (64 rows x 128 B each) of a 64-key step
constexpr int ATC_VSLOTS = ATC_MAXK / 32;
constexpr int ATC_KATOM = ATC_MAXK * 128;                    // one 32-column atom of all key rows: 36 KB
constexpr int ATC_QA = 65536, ATC_KA = 4 * ATC_KATOM;        // 64 KB + 144 KB
constexpr int ATC_SMEM = 1024 + ATC_QA + ATC_KA + ATC_THREADS * 4 + 32 * 8 + 64;

struct AttnTcDev {
    float *out; float *out_lo; int64_t ldo; int out_fmt;
    const int *q_start, *k1_start, *k2_start, *k1_len;
    int H, Hkv, causal, causal_off, window;
    const float *v1; int64_t ldv1;   // segment-1 values as plain pointers (single-key shortcut)
    int pack;        // 1: the tile holds the (<= 32) queries of all H/Hkv (<= 4) heads that share one kv head, 32 rows per head
    float scale;
    int *err;
    // key-block mode (rows with more keys than the kernel keeps resident): this launch sees keys [kb_off, kb_off + kb_len)
    // of segment 1 only, writes its normalised context to `out` (a per-block scratch) and, per (token, head), the
    // block's maximum (log2 domain, scaled) and sum to ml, for k_attention_merge to combine the blocks
    int kb_off, kb_len;
    float *ml;
    // 1: the value tiles stay in their natural [key][dim] order and the P V MMAs read them as an MN-major B operand
    // (no transpose: a thread converts one float4 to four hi and four lo halves); 0: transposed on chip into [dim][key]
    int v_mn;
};

// byte offset of element (row, col) in a K-major tile of 32 floats per row with 128-byte swizzle
__device__ __forceinline__ uint32_t sw128_off(int row, int col) {
    return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((((col >> 2) ^ (row & 7)) & 7) << 4) + ((col & 3) << 2));
}
// byte offset of byte column cb (0..127) of a row in a 128-byte-swizzled tile
__device__ __forceinline__ uint32_t sw128_boff(int row, int cb) {
    return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((((cb >> 4) ^ (row & 7)) & 7) << 4) + (cb & 15));
}
__device__ __forceinline__ float atc_hi(float v) {
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v));
    return __uint_as_float(u);
}
// 2^x through the special-function unit (about 2 ulp): the probabilities are split into 22-bit pairs right after
__device__ __forceinline__ float atc_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t *r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// without the wait: issue all loads of a row, then tmem_ld_wait() once
__device__ __forceinline__ void tmem_ld8_issue(uint32_t taddr, uint32_t *r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr) : "memory");
}
// in place: tile -> hi, and lo into the twin buffer; n4 float4 elements, layout-agnostic
__device__ __forceinline__ void split_tile(unsigned char *hi, unsigned char *lo, int n4, int tid) {
    for (int i = tid; i < n4; i += ATC_THREADS) {
        float4 x = ((float4 *)hi)[i];
        float4 h = make_float4(atc_hi(x.x), atc_hi(x.y), atc_hi(x.z), atc_hi(x.w));
        ((float4 *)hi)[i] = h;
        ((float4 *)lo)[i] = make_float4(x.x - h.x, x.y - h.y, x.z - h.z, x.w - h.w);
    }
}

// A barrier wait that ran out marks the thread: its later waits return at once, so a CTA leaves within a
// few wait limits. Control flow never depends on the outcome (all threads keep meeting at the same
// __syncthreads); the host sees the code and discards the results.
struct BoundedWaiter {
    int *err; bool dead;
    __device__ __forceinline__ void wait(uint32_t bar, uint32_t parity, int code) {
        if (dead) return;
        if (!mbar_wait(bar, parity, err, code)) dead = true;
    }
};

__global__ void __launch_bounds__(ATC_BLOCK) k_attention_tc(const __grid_constant__ CUtensorMap mq,
                                                             const __grid_constant__ CUtensorMap mk1,
                                                             const __grid_constant__ CUtensorMap mk2,
                                                             AttnTcDev a) {
    pdl_launch_dependents();          // programmatic dependent launch: see launch_pdl()
    pdl_wait();
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char *R0 = smem;                                    // QA
    unsigned char *KA = smem + ATC_QA;                           // K hi atom 0 | hi atom 1 | lo atom 0 | lo atom 1
    unsigned char *R1 = KA;                                      // phase 2: raw V slots
    unsigned char *R2 = KA + ATC_VSLOTS * 8192;                  // phase 2: P buffers
    float *xch = (float *)(smem + ATC_QA + ATC_KA);                       // one float per thread: row max / row sum exchange
    uint64_t *bars = (uint64_t *)(xch + ATC_THREADS);
    uint32_t *tmem_slot = (uint32_t *)(bars + 32);
    // barriers: 0 Q | 1 K full | 3 S MMAs done | 5,6 PV MMAs of a buffer done | 8..16 V slots | 20,21 P / V^T buffer ready
    const uint32_t bar_q = smem_u32(bars), bar_k0 = smem_u32(bars + 1), bar_s0 = smem_u32(bars + 3);
    const uint32_t bar_pv0 = smem_u32(bars + 5), bar_v0 = smem_u32(bars + 8), bar_rdy0 = smem_u32(bars + 20);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row = blockIdx.z, qt = blockIdx.x;
    const int G = a.H / a.Hkv;
    const int kvh = a.pack ? (int)blockIdx.y : (int)blockIdx.y / G;
    const int q0 = a.q_start[row], nq = a.q_start[row + 1] - q0;
    if (qt * 128 >= nq) return;
    // one query, one key (the unconditional rows of a classifier-free-guidance batch: a one-token prefix):
    // the softmax weight is exactly 1, the context is the value row
    if (!a.pack && !a.ml && nq == 1 && !a.k2_start && (a.k1_len ? a.k1_len[row] : a.k1_start[row + 1] - a.k1_start[row]) == 1) {
        if (tid < 64) {
            const int kvh1 = (int)blockIdx.y / G;
            const float x = a.v1[(int64_t)a.k1_start[row] * a.ldv1 + kvh1 * 64 + tid];
            const int64_t at = (int64_t)q0 * a.ldo + (int)blockIdx.y * 64 + tid;
            if (a.out_lo) store_split1(a.out, a.out_lo, at, x, a.out_fmt);
            else a.out[at] = x;
        }
        return;
    }
    // a barrier wait that ran out anywhere earlier (this launch or a previous one) stops the rest of the grid
    __shared__ int s_abort;
    if (tid == 0) s_abort = *(volatile int *)a.err;
    __syncthreads();
    if (s_abort) return;
    int k10 = a.k1_start[row], n1 = a.k1_len ? a.k1_len[row] : a.k1_start[row + 1] - k10;
    int causal_off = a.causal_off;
    if (a.ml) {                                    // key-block mode: the block's slice of the row's keys
        k10 += a.kb_off; n1 -= a.kb_off; causal_off -= a.kb_off;
        n1 = n1 < 0 ? 0 : (n1 > a.kb_len ? a.kb_len : n1);
    }
    // causal rows: no query of this tile sees a key past its last query's position
    if (a.causal && !a.pack) { const int vis = qt * 128 + 128 + causal_off; n1 = n1 < vis ? n1 : (vis > 0 ? vis : 0); }
    const int k20 = a.k2_start ? a.k2_start[row] : 0, n2 = a.k2_start ? a.k2_start[row + 1] - k20 : 0;
    const int n1p = (n1 + 31) & ~31, n2p = (n2 + 31) & ~31, nkp = n1p + n2p;
    const int nchunks = nkp >> 5;
    const int vofs = a.Hkv * 64;
    BoundedWaiter w{a.err, false};

    if (tid == 0) {
        for (int i = 0; i < 7; i++) mbar_init(bar_q + 8 * i, 1);
        for (int i = 0; i < ATC_VSLOTS; i++) mbar_init(bar_v0 + 8 * i, 1);
        mbar_init(bar_rdy0, ATC_THREADS / 32); mbar_init(bar_rdy0 + 8, ATC_THREADS / 32);   // one arrival per team warp
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    // all (padded) key rows of the row -> KA as raw fp32, 32-row boxes, two 32-column atoms
    auto load_keys = [&]() {
        mbar_expect_tx(bar_k0, (uint32_t)nkp * 256);
        for (int g = 0; g < nkp / 32; g++) {
            int j0 = g * 32;
            const CUtensorMap *mk = j0 < n1p ? &mk1 : &mk2;
            int tok = j0 < n1p ? k10 + j0 : k20 + (j0 - n1p);
            tma_load_2d(smem_u32(KA + g * 4096), mk, kvh * 64, tok, bar_k0);
            tma_load_2d(smem_u32(KA + ATC_KATOM + g * 4096), mk, kvh * 64 + 32, tok, bar_k0);
        }
    };
    auto load_vchunk = [&](int c) {
        const int c0 = c * 32, slot = c % ATC_VSLOTS;
        const CUtensorMap *mk = c0 < n1p ? &mk1 : &mk2;
        int tok = c0 < n1p ? k10 + c0 : k20 + (c0 - n1p);
        const uint32_t bar = bar_v0 + 8 * slot;
        mbar_expect_tx(bar, 8192);
        tma_load_2d(smem_u32(R1 + slot * 8192), mk, vofs + kvh * 64, tok, bar);
        tma_load_2d(smem_u32(R1 + slot * 8192 + 4096), mk, vofs + kvh * 64 + 32, tok, bar);
    };

    // ================= phase 1: S = Q K^T =================
    if (tid == 0) {
        if (a.pack) {                                             // mq has 32-row boxes here: one per head of the group
            mbar_expect_tx(bar_q, (uint32_t)G * 8192);
            for (int g = 0; g < G; g++) {
                tma_load_2d(smem_u32(R0 + g * 4096), &mq, (kvh * G + g) * 64, q0, bar_q);
                tma_load_2d(smem_u32(R0 + 16384 + g * 4096), &mq, (kvh * G + g) * 64 + 32, q0, bar_q);
            }
        } else {
            mbar_expect_tx(bar_q, 32768);
            tma_load_2d(smem_u32(R0), &mq, (int)blockIdx.y * 64, q0 + qt * 128, bar_q);
            tma_load_2d(smem_u32(R0 + 16384), &mq, (int)blockIdx.y * 64 + 32, q0 + qt * 128, bar_q);
        }
        if (nkp > 0) load_keys();
    }
    w.wait(bar_q, 0, 11);
    if (tid < ATC_THREADS) split_tile(R0, R0 + 32768, 2048, tid);
    if (nkp > 0) {
        w.wait(bar_k0, 0, 12);
        if (tid < ATC_THREADS)
            for (int at = 0; at < 2; at++) split_tile(KA + at * ATC_KATOM, KA + (2 + at) * ATC_KATOM, nkp * 8, tid);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (nkp > 0) {
        if (tid == 0) {
            tc_fence_after();
            for (int r0 = 0; r0 < nkp; r0 += 256) {                   // N <= 256 per MMA: 256 + 32 for a full row
                const int nrows = (nkp - r0) < 256 ? (nkp - r0) : 256;
                const uint32_t idesc = umma_idesc_tf32(128, nrows);
                const uint32_t d = tmem + (uint32_t)r0;
                for (int at = 0; at < 2; at++) {
                    uint64_t qh = umma_desc_sw128(smem_u32(R0 + at * 16384)), ql = umma_desc_sw128(smem_u32(R0 + 32768 + at * 16384));
                    uint64_t kh = umma_desc_sw128(smem_u32(KA + at * ATC_KATOM + r0 * 128));
                    uint64_t kl = umma_desc_sw128(smem_u32(KA + (2 + at) * ATC_KATOM + r0 * 128));
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        umma_tf32(d, ql + (uint64_t)(k * 2), kh + (uint64_t)(k * 2), idesc, (at | k) ? 1u : 0u);
                        umma_tf32(d, qh + (uint64_t)(k * 2), kl + (uint64_t)(k * 2), idesc, 1u);
                        umma_tf32(d, qh + (uint64_t)(k * 2), kh + (uint64_t)(k * 2), idesc, 1u);
                    }
                }
            }
            umma_commit(bar_s0);
        }
        w.wait(bar_s0, 0, 13);
    }
    tc_fence_after();
    __syncthreads();                                              // every thread is past phase 1: regions may be reused

    // ================= phase 2: softmax and O = P V =================
    if (tid == 0)
        for (int c = 0; c < nchunks; c++) load_vchunk(c);      // one slot per chunk: every V load is in flight now
    auto team_sync = [&]() { asm volatile("bar.sync 1, %0;" ::"n"(ATC_THREADS) : "memory"); };
    if (warp == ATC_THREADS / 32) {
        // ---- MMA warp: O += P V for every chunk as soon as the team has filled a P / V^T buffer ----
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16(128, 64);
            const uint32_t dm = tmem + (uint32_t)ATC_OCOL, dc = dm + 64u;
            for (int c2 = 0; 2 * c2 < nchunks; c2++) {                 // a step = two 32-key chunks (the last one may have one)
                const int b = c2 & 1;
                w.wait(bar_rdy0 + 8 * b, (uint32_t)(c2 >> 1) & 1u, 17);
                tc_fence_after();
                const uint64_t p1 = umma_desc_sw128(smem_u32(R2 + b * ATC_PBUF)), p2 = umma_desc_sw128(smem_u32(R2 + b * ATC_PBUF + 16384));
                const uint64_t v1 = umma_desc_sw128(smem_u32(R0 + b * ATC_VBUF)), v2 = umma_desc_sw128(smem_u32(R0 + b * ATC_VBUF + 8192));
                const int nk = (nchunks - 2 * c2 >= 2) ? 4 : 2;                                   // 16 keys per MMA
                // 16 keys further along: 32 bytes in a [row][key] tile (P, transposed V), two 8-key groups of 1024 bytes
                // in a [key][dim] tile read as an MN-major operand
                const uint64_t vstep = a.v_mn ? 128u : 2u;
                const uint32_t idv = a.v_mn ? (idesc | (1u << 16)) : idesc;
                for (int k = 0; k < nk; k++) {
                    umma_f16(dm, p1 + (uint64_t)(k * 2), v1 + (uint64_t)k * vstep, idv, (c2 | k) ? 1u : 0u);
                    umma_f16(dc, p1 + (uint64_t)(k * 2), v2 + (uint64_t)k * vstep, idv, (c2 | k) ? 1u : 0u);
                    umma_f16(dc, p2 + (uint64_t)(k * 2), v1 + (uint64_t)k * vstep, idv, 1u);
                }
                umma_commit(bar_pv0 + 8 * b);
            }
        }
    } else {
        const int r = tid & 127, part = tid >> 7;                     // query row of the tile, which quarter of each chunk's columns
        const int qi = a.pack ? (r & 31) : qt * 128 + r;             // query index inside the sequence row
        const int h = a.pack ? kvh * G + (r >> 5) : (int)blockIdx.y;
        const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        // visible columns of chunk c for this thread's query, as [jlo, jhi) relative to the chunk start
        auto chunk_range = [&](int c, int &jlo, int &jhi) {
            const int c0 = c * 32;
            int lo, hi, base;                                         // key index = base + j
            if (c0 < n1p) {
                base = c0; lo = 0; hi = n1;
                if (a.causal) hi = min(hi, qi + causal_off + 1);
            } else {
                base = n1 + (c0 - n1p); lo = n1; hi = n1 + n2;
            }
            if (a.window > 0) { lo = max(lo, qi - a.window); hi = min(hi, qi + a.window + 1); }
            jlo = lo - base; jhi = hi - base;
        };
        // The thread's scores -- eight columns of every chunk -- are read from tensor memory ONCE, all loads in
        // flight together, and stay in registers for the maximum and for the exponentials: a tcgen05.ld round
        // trip costs about a microsecond, and one per chunk was most of the chunk loop.
        uint32_t sv[ATC_VSLOTS][8];
#pragma unroll
        for (int c = 0; c < ATC_VSLOTS; c++) tmem_ld8_issue(lane_addr + (uint32_t)(c * 32 + part * 8), sv[c]);
        tmem_ld_wait();
        float mx = -INFINITY;
#pragma unroll
        for (int c = 0; c < ATC_VSLOTS; c++) {
            if (c < nchunks) {
                int jlo, jhi;
                chunk_range(c, jlo, jhi);
                jlo -= part * 8; jhi -= part * 8;
#pragma unroll
                for (int j = 0; j < 8; j++)
                    if (j >= jlo && j < jhi) mx = fmaxf(mx, __uint_as_float(sv[c][j]));
            }
        }
        xch[tid] = mx;
        team_sync();
        mx = fmaxf(fmaxf(xch[r], xch[r + 128]), fmaxf(xch[r + 256], xch[r + 384]));
        team_sync();                                                  // xch is reused for the row sums
        const bool any = mx != -INFINITY;
        const float sl2 = a.scale * 1.4426950408889634f;

        // shared-memory offsets of the thread's four V elements (source: raw [key][d] atoms, destination: V^T)
        const int kk = tid & 31;
        uint32_t vsrc[4], vdst[4];                                   // vdst: offset in the hi tile; the lo tile takes the same offset
#pragma unroll
        for (int n = 0; n < 4; n++) {
            const int d = (tid >> 5) + 16 * n;
            vsrc[n] = (uint32_t)((d >> 5) * 4096) + sw128_off(kk, d & 31);
            vdst[n] = sw128_boff(d, kk * 2);
        }
        float l = 0.f;
        const uint32_t rowoff = (uint32_t)((r >> 3) * 1024 + (r & 7) * 128);
        // A step hands TWO 32-key chunks to the MMA warp: the fence, the barrier arrival and the wait for the
        // buffer are paid once per 64 keys.
#pragma unroll
        for (int c2 = 0; c2 < (ATC_VSLOTS + 1) / 2; c2++) {
            if (2 * c2 >= nchunks) break;
            const int b = c2 & 1;
            unsigned char *Pb = R2 + b * ATC_PBUF, *Vt = R0 + b * ATC_VBUF;
            if (c2 >= 2) w.wait(bar_pv0 + 8 * b, (uint32_t)((c2 >> 1) - 1) & 1u, 15);   // MMAs of step c2-2 are done with buffer b
#pragma unroll
            for (int hf = 0; hf < 2; hf++) {
                const int c = 2 * c2 + hf;
                if (c >= ATC_VSLOTS || c >= nchunks) break;
                {
                    const uint32_t *v = sv[c];
                    int jlo, jhi;
                    chunk_range(c, jlo, jhi);
                    jlo -= part * 8; jhi -= part * 8;
                    const bool inner = any && jlo <= 0 && jhi >= 8;
                    uint32_t hw[4], lw[4];                                 // eight probabilities as packed fp16 pairs
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        unsigned short h0, l0, h1, l1;
                        float x0 = atc_ex2((__uint_as_float(v[2 * e]) - mx) * sl2), x1 = atc_ex2((__uint_as_float(v[2 * e + 1]) - mx) * sl2);
                        if (!inner) {                                      // interior chunks skip the range tests
                            if (!(any && 2 * e >= jlo && 2 * e < jhi)) x0 = 0.f;
                            if (!(any && 2 * e + 1 >= jlo && 2 * e + 1 < jhi)) x1 = 0.f;
                        }
                        l += x0 + x1;
                        h16_pair(x0, h0, l0); h16_pair(x1, h1, l1);
                        hw[e] = (uint32_t)h0 | ((uint32_t)h1 << 16); lw[e] = (uint32_t)l0 | ((uint32_t)l1 << 16);
                    }
                    // the thread's eight keys are 16-byte chunk 4 hf + part of its row in the hi tile and in the lo tile
                    const uint32_t o = rowoff + ((uint32_t)(((4 * hf + part) ^ (r & 7)) & 7) << 4);
                    *(uint4 *)(Pb + o) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
                    *(uint4 *)(Pb + 16384 + o) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
                }
                w.wait(bar_v0 + 8 * (c % ATC_VSLOTS), (uint32_t)(c / ATC_VSLOTS) & 1u, 14);
                if (a.v_mn) {   // split only: Vraw[key][d] (two 32-column atoms) -> pair tiles [key][d], one float4 per thread
                    const unsigned char *Vraw = R1 + (c % ATC_VSLOTS) * 8192;
                    const int c0 = c * 32;
                    const int nvalid = c0 < n1p ? (n1 - c0) : (n2 - (c0 - n1p));
                    const int vk = tid >> 4, d4 = tid & 15;                   // key of the chunk, which four dims
                    float4 x = *(const float4 *)(Vraw + (d4 >> 3) * 4096 + sw128_off(vk, (d4 & 7) * 4));
                    if (vk >= nvalid) x = make_float4(0.f, 0.f, 0.f, 0.f);
                    unsigned short h0, l0, h1, l1, h2, l2, h3, l3;
                    h16_pair(x.x, h0, l0); h16_pair(x.y, h1, l1); h16_pair(x.z, h2, l2); h16_pair(x.w, h3, l3);
                    const uint32_t o = sw128_boff(hf * 32 + vk, d4 * 8);
                    *(uint2 *)(Vt + o) = make_uint2((uint32_t)h0 | ((uint32_t)h1 << 16), (uint32_t)h2 | ((uint32_t)h3 << 16));
                    *(uint2 *)(Vt + 8192 + o) = make_uint2((uint32_t)l0 | ((uint32_t)l1 << 16), (uint32_t)l2 | ((uint32_t)l3 << 16));
                } else {   // transpose + split: Vraw[key][d] (two 32-column atoms) -> Vt[d][key]; keys past the segment end read as 0
                    const unsigned char *Vraw = R1 + (c % ATC_VSLOTS) * 8192;
                    const int c0 = c * 32;
                    const int nvalid = c0 < n1p ? (n1 - c0) : (n2 - (c0 - n1p));
#pragma unroll
                    for (int n = 0; n < 4; n++) {
                        float x = *(const float *)(Vraw + vsrc[n]);
                        if (kk >= nvalid) x = 0.f;
                        unsigned short hi, lo;
                        h16_pair(x, hi, lo);
                        const uint32_t o = vdst[n] ^ (uint32_t)(hf * 64);      // keys 32..63 of the step: 64 B further along the row
                        *(unsigned short *)(Vt + o) = hi; *(unsigned short *)(Vt + 8192 + o) = lo;
                    }
                }
            }
            // hand the buffers to the MMA warp: this warp's writes are visible to the async proxy, one arrival per warp
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_rdy0 + 8 * b);
        }
        // the commits complete in order: the last one covers every earlier MMA
        if (nchunks > 0) { const int c2 = (nchunks - 1) >> 1; w.wait(bar_pv0 + 8 * (c2 & 1), (uint32_t)(c2 >> 1) & 1u, 16); }
        tc_fence_after();
        xch[tid] = l;
        team_sync();
        l = (xch[r] + xch[r + 128]) + (xch[r + 256] + xch[r + 384]);
        if (a.ml && part == 0 && qi < nq) {
            float *mlp = a.ml + ((int64_t)(q0 + qi) * a.H + (int)blockIdx.y) * 2;
            mlp[0] = any ? mx * sl2 : -INFINITY; mlp[1] = l;
        }
        // ---- output row: O / l; the four threads of a row take 16 columns each ----
        {
            const bool live = qi < nq && h < (kvh + 1) * G && !w.dead;
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            const int64_t ofs = (int64_t)(q0 + qi) * a.ldo + h * 64 + part * 16;
            uint32_t v[16], vc[16];
            if (nchunks > 0) {
                tmem_ld16(lane_addr + (uint32_t)(ATC_OCOL + part * 16), v);
                tmem_ld16(lane_addr + (uint32_t)(ATC_OCOL + 64 + part * 16), vc);
            }
            if (live) {
#pragma unroll
                for (int j = 0; j < 16; j += 4) {
                    float4 o4 = make_float4(fmaf(__uint_as_float(vc[j]), H16_LO_UNSCALE, __uint_as_float(v[j])) * inv,
                                            fmaf(__uint_as_float(vc[j + 1]), H16_LO_UNSCALE, __uint_as_float(v[j + 1])) * inv,
                                            fmaf(__uint_as_float(vc[j + 2]), H16_LO_UNSCALE, __uint_as_float(v[j + 2])) * inv,
                                            fmaf(__uint_as_float(vc[j + 3]), H16_LO_UNSCALE, __uint_as_float(v[j + 3])) * inv);
                    if (nchunks == 0) o4 = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (a.out_lo) store_split4(a.out, a.out_lo, ofs + j, o4, a.out_fmt);
                    else *(float4 *)(a.out + ofs + j) = o4;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

bool attention_tc_supported(const AttnArgs &a) {
    static const bool off = getenv("NCM_B200_ATTN_SIMT") != nullptr;
    if (off || a.hd != 64 || a.Hkv <= 0 || a.H % a.Hkv) return false;
    const int G = a.H / a.Hkv;
    const bool pack = a.max_q <= 32 && G >= 2 && G <= 4;         // grouped-query passes with few queries per row
    if (!pack && a.max_q < 64) return false;
    if (a.max_k1 <= 0 && a.max_k2 <= 0) return false;
    int n1p = (a.max_k1 + 31) & ~31, n2p = (a.max_k2 + 31) & ~31;
    if (n1p + n2p > ATC_MAXK || n1p + n2p == 0) return false;
    if (a.q_total <= 0 || a.k1_total <= 0 || (a.k2 && a.k2_total <= 0)) return false;
    if ((a.ldq | a.ldk1 | a.ldk2 | a.ldo) & 3) return false;
    if (a.v1 != a.k1 + a.Hkv * 64 || (a.k2 && a.v2 != a.k2 + a.Hkv * 64)) return false;
    auto al = [](const void *p) { return ((uintptr_t)p & 15) == 0; };
    if (!al(a.q) || !al(a.k1) || (a.k2 && !al(a.k2)) || !al(a.out) || (a.out_lo && !al(a.out_lo))) return false;
    return true;
}

// one launch; ml != null: key-block mode over keys [kb_off, kb_off + kb_len) into the scratch `out`
static void attention_tc_launch(const AttnArgs &a, float *out, float *out_lo, int64_t ldo, int kb_off, int kb_len, float *ml) {
    AttnTcDev d;
    d.out = out; d.out_lo = out_lo; d.ldo = ldo; d.out_fmt = a.out_fmt;
    d.q_start = a.q_start; d.k1_start = a.k1_start; d.k2_start = a.k2 ? a.k2_start : nullptr; d.k1_len = a.k1_len;
    d.v1 = a.v1; d.ldv1 = a.ldk1;
    d.H = a.H; d.Hkv = a.Hkv; d.causal = a.causal; d.causal_off = a.causal_off; d.window = a.window;
    d.scale = 1.0f / sqrtf(64.0f);
    d.err = tc_err_flag();
    d.kb_off = kb_off; d.kb_len = kb_len; d.ml = ml;
    static const int v_mn = getenv("NCM_B200_ATTN_VT") ? 0 : 1;       // A/B: NCM_B200_ATTN_VT=1 keeps the on-chip transpose
    d.v_mn = v_mn;
    const int G = a.H / a.Hkv;
    d.pack = (!ml && a.max_q <= 32 && G >= 2 && G <= 4) ? 1 : 0;
    const CUtensorMap mq = tc_get_map(a.q, a.q_total, a.H * 64, a.ldq, d.pack ? 32 : 128, false);
    const CUtensorMap mk1 = tc_get_map(a.k1, a.k1_total, 2 * a.Hkv * 64, a.ldk1, 32, false);
    const CUtensorMap mk2 = a.k2 ? tc_get_map(a.k2, a.k2_total, 2 * a.Hkv * 64, a.ldk2, 32, false) : mk1;
    static bool set = false;
    if (!set) {
        CUDA_CHECK(cudaFuncSetAttribute(k_attention_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, ATC_SMEM));
        set = true;
    }
    dim3 grid((unsigned)cdiv(a.max_q, 128), (unsigned)(d.pack ? a.Hkv : a.H), (unsigned)a.rows);
    LAUNCH_PDL_IF(pdl_small((int64_t)grid.x * grid.y * grid.z), k_attention_tc, grid, ATC_BLOCK, ATC_SMEM, mq, mk1, mk2, d);
}

void attention_tc(const AttnArgs &a) {
    ProfScope ps(NCMB_K_ATTN, 4.0 * (double)a.total_q * a.avg_keys * a.H * a.hd, 0);
    attention_tc_launch(a, a.out, a.out_lo, a.ldo, 0, 0, nullptr);
}

// ---- rows with more keys than one launch keeps resident: key blocks + merge ----
constexpr int ATC_KBLOCK = 256;

// out[token][h][d] = sum_b w_b ctx_b / sum_b w_b with w_b = 2^(m_b - M) l_b, the usual log-sum-exp merge of blocks
// whose contexts arrive normalised by their own sums
__global__ void k_attention_merge(const float *__restrict__ part, const float *__restrict__ ml, int nblk, int64_t ntok, int H,
                                  float *__restrict__ out, float *__restrict__ out_lo, int64_t ldo, int fmt) {
    const int64_t n4 = ntok * H * 16;                                   // float4 elements of the output
    const int64_t bstride = ntok * H * 64, mstride = ntok * H * 2;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t th = i >> 4;                                     // token * H + head
        const int d4 = (int)(i & 15);
        float M = -INFINITY;
        for (int b = 0; b < nblk; b++) M = fmaxf(M, ml[b * mstride + th * 2]);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float L = 0.f;
        for (int b = 0; b < nblk; b++) {
            const float m = ml[b * mstride + th * 2], l = ml[b * mstride + th * 2 + 1];
            if (!(l > 0.f)) continue;
            const float w = exp2f(m - M) * l;
            const float4 c = *(const float4 *)(part + b * bstride + th * 64 + d4 * 4);
            acc.x = fmaf(w, c.x, acc.x); acc.y = fmaf(w, c.y, acc.y); acc.z = fmaf(w, c.z, acc.z); acc.w = fmaf(w, c.w, acc.w);
            L += w;
        }
        const float inv = L > 0.f ? 1.0f / L : 0.f;
        const float4 o = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
        const int64_t tok = th / H; const int h = (int)(th % H);
        const int64_t at = tok * ldo + h * 64 + d4 * 4;
        if (out_lo) store_split4(out, out_lo, at, o, fmt);
        else *(float4 *)(out + at) = o;
    }
}

static size_t atc_long_scratch_floats(const AttnArgs &a, int nblk) { return (size_t)nblk * a.q_total * a.H * 66; }

bool attention_tc_long_supported(const AttnArgs &a) {
    static const bool off = getenv("NCM_B200_ATTN_SIMT") != nullptr || getenv("NCM_B200_NO_ATTN_BLOCKS") != nullptr;
    if (off || a.hd != 64 || a.Hkv <= 0 || a.H % a.Hkv || a.k2 || a.window > 0 || a.max_q < 64) return false;
    if (a.max_k1 <= ATC_MAXK || a.max_k1 > 16 * ATC_KBLOCK) return false;
    if (a.q_total <= 0 || a.k1_total <= 0) return false;
    if ((a.ldq | a.ldk1 | a.ldo) & 3) return false;
    if (a.v1 != a.k1 + a.Hkv * 64) return false;
    auto al = [](const void *p) { return ((uintptr_t)p & 15) == 0; };
    if (!al(a.q) || !al(a.k1) || !al(a.out) || (a.out_lo && !al(a.out_lo))) return false;
    return atc_long_scratch_floats(a, (int)cdiv(a.max_k1, ATC_KBLOCK)) * 4 <= ((size_t)2 << 30);      // at most 2 GB of block contexts
}

void attention_tc_long(const AttnArgs &a) {
    static float *scr = nullptr; static size_t scr_cap = 0;
    const int nblk = (int)cdiv(a.max_k1, ATC_KBLOCK);
    const size_t need = atc_long_scratch_floats(a, nblk);
    if (need > scr_cap) {
        if (scr) { CUDA_CHECK(cudaStreamSynchronize(stream())); dev_free(scr); }
        scr = (float *)dev_alloc(need * 4); scr_cap = need;
    }
    float *part = scr, *ml = scr + (size_t)nblk * a.q_total * a.H * 64;
    ProfScope ps(NCMB_K_ATTN, 4.0 * (double)a.total_q * a.avg_keys * a.H * a.hd, 0);
    for (int b = 0; b < nblk; b++)
        attention_tc_launch(a, part + (size_t)b * a.q_total * a.H * 64, nullptr, (int64_t)a.H * 64, b * ATC_KBLOCK, ATC_KBLOCK,
                            ml + (size_t)b * a.q_total * a.H * 2);
    const int64_t n4 = a.q_total * a.H * 16, g = cdiv(n4, 256), cap = (int64_t)ctx().sm_count * 32;
    LAUNCH(k_attention_merge, (unsigned)(g > cap ? cap : g), 256, 0, (const float *)part, (const float *)ml, nblk, (int64_t)a.q_total, a.H,
           a.out, a.out_lo, (int64_t)a.ldo, a.out_fmt);
}

} // namespace ncmb

// Diagnostic entry point: runs the token-major attention of the transformer blocks on caller-supplied
// device buffers with either engine (0: CUDA-core kernel, 1: tcgen05 kernel), so the two can be compared
// on the same inputs (engine 2: the split-key decode kernel, one query per row). q [q_total][H*64]; kv1 / kv2 [tokens][2*Hkv*64] (keys then values); the *_start
// arrays are host int[rows+1] prefix offsets (k2_start null: one key segment). Returns 0, -1 when the
// tensor-core engine does not take the shape, or the engine's timeout code.
extern "C" int ncmb_attention_check(const float *q, const float *kv1, const float *kv2, float *out,
                                    const int *q_start, const int *k1_start, const int *k2_start,
                                    int rows, int H, int Hkv, int causal, int window, int engine) {
    using namespace ncmb;
    ensure_device();
    int *d_q = (int *)dev_alloc((size_t)(rows + 1) * 4), *d_k1 = (int *)dev_alloc((size_t)(rows + 1) * 4), *d_k2 = nullptr;
    upload(d_q, q_start, (size_t)(rows + 1) * 4);
    upload(d_k1, k1_start, (size_t)(rows + 1) * 4);
    if (k2_start) { d_k2 = (int *)dev_alloc((size_t)(rows + 1) * 4); upload(d_k2, k2_start, (size_t)(rows + 1) * 4); }
    AttnArgs a;
    int kvd = Hkv * 64;
    a.q = q; a.ldq = H * 64; a.k1 = kv1; a.v1 = kv1 + kvd; a.ldk1 = 2 * kvd;
    if (k2_start) { a.k2 = kv2; a.v2 = kv2 + kvd; a.ldk2 = 2 * kvd; a.k2_start = d_k2; }
    a.out = out; a.ldo = H * 64; a.q_start = d_q; a.k1_start = d_k1;
    a.rows = rows; a.H = H; a.Hkv = Hkv; a.hd = 64; a.causal = causal; a.window = window;
    for (int r = 0; r < rows; r++) {
        a.max_q = std::max(a.max_q, q_start[r + 1] - q_start[r]);
        a.max_k1 = std::max(a.max_k1, k1_start[r + 1] - k1_start[r]);
        if (k2_start) a.max_k2 = std::max(a.max_k2, k2_start[r + 1] - k2_start[r]);
    }
    a.q_total = q_start[rows]; a.k1_total = k1_start[rows]; a.k2_total = k2_start ? k2_start[rows] : 0;
    a.total_q = a.q_total; a.avg_keys = rows ? (double)(a.k1_total + a.k2_total) / rows : 0;
    int rc = 0;
    if (engine == 1) {
        int saved_max_q = a.max_q;
        a.max_q = std::max(a.max_q, 64);               // the size threshold is a dispatch heuristic, not a limit
        if (attention_tc_supported(a)) { a.max_q = saved_max_q; attention_tc(a); rc = gemm_tc_check(); }
        else if (attention_tc_long_supported(a)) { attention_tc_long(a); rc = gemm_tc_check(); }
        else rc = -1;
    } else if (engine == 2) {
        if (!attention_decode_supported(a)) rc = -1;
        else attention_decode(a);
    } else {
        // the CUDA-core kernel, called directly: the dispatcher would pick the other engines where they apply
        int saved = ctx().gemm_mode, saved_q = a.max_q;
        ctx().gemm_mode = 0;
        if (attention_decode_supported(a)) a.max_q = 2;     // grid sizing only; rows still hold one query
        attention(a);
        a.max_q = saved_q;
        ctx().gemm_mode = saved;
    }
    CUDA_CHECK(cudaStreamSynchronize(stream()));
    dev_free(d_q); dev_free(d_k1); if (d_k2) dev_free(d_k2);
    return rc;
}
