// Tensor-core attention for head dim 64 on sm_100a (tcgen05 + TMEM + TMA).
//
// One CTA (16 softmax warps, one MMA warp, three converter warps) per (sequence row, group of heads that share a kv
// head, 128-query tile). The keys and values of the row (up to 288 padded keys: a 256-token prefix plus a 32-token
// level) are fetched ONCE by TMA, turned into fp16 pairs in place and stay resident; the CTA then walks its heads
// ("items") one after the other, so the fetch and the conversion are shared by the heads of the group and the phases
// of neighbouring items overlap: the query tile of item i+1 arrives and is converted by the converter warps while
// the team works on item i, and its score MMAs are issued in four batches between the P V MMAs of item i.
// The team raises its register allowance (setmaxnreg) with what the other four warps give up.
//   S = Q K^T   three kind::f16 MMAs per 16 dims over pairs x = x1 + x2 (x1 = rn_f16(x), x2 = rn_f16(x - x1), NOT
//               scaled: one accumulator takes q2 k1 + q1 k2 + q1 k1; where x2 falls into the fp16 subnormals,
//               |x| < 1/8, it is exact to 3e-8 absolute, below the dropped q2 k2 term for every |k| that matters)
//   softmax     four threads per query row (each takes a quarter of every 32-key chunk) read the scores with
//               tcgen05.ld once and keep them in registers; all keys of a row are resident, so the row maximum is
//               known before any exponential is taken and nothing is rescaled
//   O += P V    per 32-key chunk: the team writes P as fp16 pairs (p = p1 + p2 * 2^-11, as the fp16-pair GEMM does)
//               into the half of a 64-key tile, the MMA warp accumulates main += p1 v1 and cross += p1 v2 + p2 v1;
//               the value pairs are read in their natural [key][dim] order as an MN-major operand
// Both products are fp32-grade like the CUDA-core kernel. Key rows come from up to two segments (cached prefix,
// tokens of the current pass); each segment is padded to a multiple of 32 score columns, the padding is masked
// in the softmax and its value rows are zeroed.
//
// Shared memory (208 KB of tiles):
//   QB[2] (32 KB each)  raw query tile (two 32-column atoms) -> Q hi | Q lo -> after the item's score MMAs the P
//                       hi | lo tile of the same item (two 32-key halves, handed over one at a time)
//   KP    (72 KB)       raw keys -> K hi rows | K lo rows            VP (72 KB) the same for the values
// Tensor memory: scores [0, 288), output main [288, 352), cross [352, 416).
#include "common.cuh"
#include "tc_common.cuh"
#include "split.cuh"

namespace ncmb {

constexpr float ATC_LO_SCALE = 2048.0f, ATC_LO_UNSCALE = 1.0f / 2048.0f;   // P and V pairs: scaled remainders, cross terms apart
constexpr int ATC_THREADS = 512;          // softmax team: four threads per query row, eight score columns of a chunk each
constexpr int ATC_CONV = 96;              // converter threads: the query tiles' fp32 -> pair conversion, off the team's path
constexpr int ATC_BLOCK = ATC_THREADS + 32 + ATC_CONV;  // team + one warp whose first lane issues the MMAs + converters: five warpgroups
constexpr int ATC_MAXK = 288;            // padded keys per row the kernel keeps resident
constexpr int ATC_OCOL = 288;            // TMEM columns of the output accumulators (main, then cross terms); scores use [0, 288)
constexpr int ATC_QB = 32768;                                // a 128 x 64 tile as pairs: hi 16 KB | lo 16 KB
constexpr int ATC_KP = ATC_MAXK * 128;                       // all key rows, one half of the pair (or one raw atom): 36 KB
constexpr int ATC_SMEM = 1024 + 2 * ATC_QB + 4 * ATC_KP + 2 * ATC_THREADS * 4 + 32 * 8 + 64;

struct AttnTcDev {
    float *out; float *out_lo; int64_t ldo; int out_fmt;
    const int *q_start, *k1_start, *k2_start, *k1_len;
    int H, Hkv, causal, causal_off, window;
    const float *v1; int64_t ldv1;   // segment-1 values as plain pointers (single-key shortcut)
    int pack;        // 1: the tile holds the (<= 32) queries of all H/Hkv (<= 4) heads that share one kv head, 32 rows per head
    int hpc;         // heads a CTA walks (pack == 0): a divisor of H/Hkv; blockIdx.y * hpc is its first head
    float scale;
    int *err;
    // key-block mode (rows with more keys than the kernel keeps resident): this launch sees keys [kb_off, kb_off + kb_len)
    // of segment 1 only, writes its normalised context to `out` (a per-block scratch) and, per (token, head), the
    // block's maximum (log2 domain, scaled) and sum to ml, for k_attention_merge to combine the blocks
    int kb_off, kb_len;
    float *ml;
};

// 2^x through the special-function unit (about 2 ulp): the probabilities are split into 22-bit pairs right after
__device__ __forceinline__ float atc_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float atc_max3(float a, float b, float c) {
    float m;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(m) : "f"(a), "f"(b), "f"(c));
    return m;
}
// without the wait: issue all loads of a row, then tmem_ld_wait() once
__device__ __forceinline__ void tmem_ld8_issue(uint32_t taddr, uint32_t *r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, uint32_t *r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}

// A tile as TMA delivers it -- rows of 64 floats as two 32-float atoms (128-byte swizzle), the atoms `atom` bytes
// apart -- becomes fp16 pairs IN PLACE: hi rows (64 halves = 128 bytes, same swizzle) where atom 0 was, lo rows where
// atom 1 was. A unit is eight dims of one row: two float4 in, one 16-byte store per half out. The eight units of a
// row sit in eight neighbouring lanes of one warp and touch that row's two 128-byte lines only, so reading a batch
// of units into registers (atc_units_read), __syncwarp(), then writing them (atc_units_write) is all the ordering
// the in-place conversion needs.
template <int NU, int NT = ATC_THREADS>
__device__ __forceinline__ void atc_units_read(const unsigned char *base, uint32_t atom, int nrows, int tid, float4 (&x)[NU][2]) {
#pragma unroll
    for (int i = 0; i < NU; i++) {
        const int u = tid + i * NT, row = u >> 3, d8 = u & 7;
        if (row < nrows) {
            const unsigned char *rp = base + (size_t)(d8 >> 2) * atom + (row >> 3) * 1024 + (row & 7) * 128;
            const int c0 = (d8 & 3) * 2;
            x[i][0] = *(const float4 *)(rp + (((c0) ^ (row & 7)) << 4));
            x[i][1] = *(const float4 *)(rp + (((c0 + 1) ^ (row & 7)) << 4));
        }
    }
}
// lo_scale: 1 for the score operands, 2^11 for the values; rows whose index in its segment is past the segment's
// length (n1 of the first n1p rows, then n2) are written as zeros
template <int NU, int NT = ATC_THREADS>
__device__ __forceinline__ void atc_units_write(unsigned char *base, uint32_t atom, int nrows, int tid, const float4 (&x)[NU][2],
                                                float lo_scale, int n1p, int n1, int n2) {
#pragma unroll
    for (int i = 0; i < NU; i++) {
        const int u = tid + i * NT, row = u >> 3, d8 = u & 7;
        if (row < nrows) {
            const bool valid = row < n1p ? row < n1 : (row - n1p) < n2;
            const float v[8] = {x[i][0].x, x[i][0].y, x[i][0].z, x[i][0].w, x[i][1].x, x[i][1].y, x[i][1].z, x[i][1].w};
            uint32_t hw[4], lw[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                h16_pair2_raw(valid ? v[2 * e] : 0.f, valid ? v[2 * e + 1] : 0.f, hw[e], lw[e], lo_scale);
            }
            const uint32_t o = (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + (((d8) ^ (row & 7)) << 4));
            *(uint4 *)(base + o) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
            *(uint4 *)(base + atom + o) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
        }
    }
}

// A barrier wait that ran out marks the thread: its later waits return at once, so a CTA leaves within a
// few wait limits. Control flow never depends on the outcome (all threads keep meeting at the same
// barriers); the host sees the code and discards the results.
struct BoundedWaiter {
    int *err; bool dead;
    __device__ __forceinline__ void wait(uint32_t bar, uint32_t parity, int code) {
        if (dead) return;
        if (!mbar_wait(bar, parity, err, code)) dead = true;
    }
};

// NCH: 32-key chunks a thread keeps the scores of in registers (8 for rows of up to 256 padded keys, else 9)
template <int NCH>
__global__ void __launch_bounds__(ATC_BLOCK) k_attention_tc(const __grid_constant__ CUtensorMap mq,
                                                             const __grid_constant__ CUtensorMap mk1,
                                                             const __grid_constant__ CUtensorMap mk2,
                                                             AttnTcDev a) {
    pdl_launch_dependents();          // programmatic dependent launch: see launch_pdl()
    if (threadIdx.x == 0) {           // the descriptors are on their way while the predecessor finishes
        asm volatile("prefetch.tensormap [%0];" ::"l"(&mq) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&mk1) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&mk2) : "memory");
    }
    pdl_wait();
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char *QB = smem;                                    // two query / P tiles
    unsigned char *KP = smem + 2 * ATC_QB;                       // K hi | K lo
    unsigned char *VP = KP + 2 * ATC_KP;                         // V hi | V lo
    float *xmax = (float *)(VP + 2 * ATC_KP);                    // one float per thread: row maximum exchange
    float *xsum = xmax + ATC_THREADS;                            // ... and row sum exchange
    uint64_t *bars = (uint64_t *)(xsum + ATC_THREADS);
    uint32_t *tmem_slot = (uint32_t *)(bars + 32);
    // barriers: 0,1 query tile landed | 2 keys landed | 3 values landed | 4,5 query pairs of a tile ready | 6 score MMAs
    //           done | 7,8 P half ready | 9,10 PV MMAs of a P half done | 11 key pairs ready | 12 scores are in registers
    const uint32_t bar_q = smem_u32(bars), bar_k = smem_u32(bars + 2), bar_v = smem_u32(bars + 3), bar_qrdy = smem_u32(bars + 4);
    const uint32_t bar_s = smem_u32(bars + 6), bar_rdy0 = smem_u32(bars + 7), bar_pv0 = smem_u32(bars + 9);
    const uint32_t bar_krdy = smem_u32(bars + 11), bar_sfree = smem_u32(bars + 12);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row = blockIdx.z, qt = blockIdx.x;
    const int G = a.H / a.Hkv;
    const int h0 = a.pack ? (int)blockIdx.y * G : (int)blockIdx.y * a.hpc;     // first head of this CTA
    const int kvh = h0 / G;
    const int gn = a.pack ? 1 : a.hpc;                                         // items: one head each (pack: all heads in one)
    const int q0 = a.q_start[row], nq = a.q_start[row + 1] - q0;
    if (qt * 128 >= nq) return;
    // one query, one key (the unconditional rows of a classifier-free-guidance batch: a one-token prefix):
    // the softmax weight is exactly 1, the context is the value row
    if (!a.pack && !a.ml && nq == 1 && !a.k2_start && (a.k1_len ? a.k1_len[row] : a.k1_start[row + 1] - a.k1_start[row]) == 1) {
        if (tid < 64 * gn) {
            const float x = a.v1[(int64_t)a.k1_start[row] * a.ldv1 + kvh * 64 + (tid & 63)];
            const int64_t at = (int64_t)q0 * a.ldo + (h0 + (tid >> 6)) * 64 + (tid & 63);
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
    if (nkp == 0) {                                // no key in sight: zero context, empty block statistics
        if (tid < ATC_THREADS) {
            const int r = tid & 127, part = tid >> 7, qi = a.pack ? (r & 31) : qt * 128 + r;
            for (int it = 0; it < gn; it++) {
                const int h = a.pack ? h0 + (r >> 5) : h0 + it;
                if (qi >= nq || h >= (kvh + 1) * G) continue;
                if (a.ml && part == 0) { float *mlp = a.ml + ((int64_t)(q0 + qi) * a.H + h) * 2; mlp[0] = -INFINITY; mlp[1] = 0.f; }
                const int64_t ofs = (int64_t)(q0 + qi) * a.ldo + h * 64 + part * 16;
                const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int j = 0; j < 16; j += 4) {
                    if (a.out_lo) store_split4(a.out, a.out_lo, ofs + j, z, a.out_fmt);
                    else *(float4 *)(a.out + ofs + j) = z;
                }
            }
        }
        return;
    }
    BoundedWaiter w{a.err, false};

    if (tid == 0) {
        mbar_init(bar_q, 1); mbar_init(bar_q + 8, 1); mbar_init(bar_k, 1); mbar_init(bar_v, 1);
        mbar_init(bar_qrdy, ATC_CONV / 32); mbar_init(bar_qrdy + 8, ATC_CONV / 32);   // one arrival per converter warp
        mbar_init(bar_krdy, ATC_THREADS / 32); mbar_init(bar_sfree, ATC_THREADS / 32);   // one arrival per team warp
        mbar_init(bar_s, 1);
        mbar_init(bar_rdy0, ATC_THREADS / 32); mbar_init(bar_rdy0 + 8, ATC_THREADS / 32);
        mbar_init(bar_pv0, 1); mbar_init(bar_pv0 + 8, 1);
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

    // the query tile of item `it` -> QB[it & 1] as raw fp32 (two atoms)
    auto load_q = [&](int it) {
        const uint32_t bar = bar_q + 8 * (it & 1);
        const uint32_t dst = smem_u32(QB + (it & 1) * ATC_QB);
        if (a.pack) {                                             // mq has 32-row boxes here: one per head of the group
            mbar_expect_tx(bar, (uint32_t)G * 8192);
            for (int g = 0; g < G; g++) {
                tma_load_2d(dst + g * 4096, &mq, (h0 + g) * 64, q0, bar);
                tma_load_2d(dst + 16384 + g * 4096, &mq, (h0 + g) * 64 + 32, q0, bar);
            }
        } else {
            mbar_expect_tx(bar, 32768);
            tma_load_2d(dst, &mq, (h0 + it) * 64, q0 + qt * 128, bar);
            tma_load_2d(dst + 16384, &mq, (h0 + it) * 64 + 32, q0 + qt * 128, bar);
        }
    };
    // 32 (padded) key or value rows of the row -> dst as raw fp32: group g of 32 rows, two 32-column atoms
    auto load_row_group = [&](unsigned char *dst, int col0, uint32_t bar, int g) {
        const int j0 = g * 32;
        const CUtensorMap *mk = j0 < n1p ? &mk1 : &mk2;
        const int tok = j0 < n1p ? k10 + j0 : k20 + (j0 - n1p);
        tma_load_2d(smem_u32(dst + g * 4096), mk, col0, tok, bar);
        tma_load_2d(smem_u32(dst + ATC_KP + g * 4096), mk, col0 + 32, tok, bar);
    };
    auto team_sync = [&]() { asm volatile("bar.sync 1, %0;" ::"n"(ATC_THREADS) : "memory"); };

    // the first warp issues every load of the prologue, a lane per 32-row group of the keys (lanes 0..8) and of the
    // values (lanes 16..24): thirty-odd copies leave in the time of two
    if (warp == 0) {
        if (lane == 0) {
            load_q(0);
            mbar_expect_tx(bar_k, (uint32_t)nkp * 256);
            mbar_expect_tx(bar_v, (uint32_t)nkp * 256);
        }
        __syncwarp();
        if (lane < 16) { if (lane < nchunks) load_row_group(KP, kvh * 64, bar_k, lane); }
        else if (lane - 16 < nchunks) load_row_group(VP, vofs + kvh * 64, bar_v, lane - 16);
        if (lane == 0 && gn > 1) load_q(1);
    }

    if (warp > ATC_THREADS / 32) {
        // ================= converter warps: every item's query tile, fp32 -> pairs in place =================
        const int ct = tid - ATC_THREADS - 32;
        for (int it = 0; it < gn; it++) {
            unsigned char *Qn = QB + (it & 1) * ATC_QB;
            w.wait(bar_q + 8 * (it & 1), (uint32_t)(it >> 1) & 1u, 11);
            for (int i = 0; i < 12; i += 2) {                             // 1024 units over 96 threads, two at a time
                float4 xq[2][2];
                atc_units_read<2, ATC_CONV>(Qn, 16384, 128, ct + i * ATC_CONV, xq);
                __syncwarp();
                atc_units_write<2, ATC_CONV>(Qn, 16384, 128, ct + i * ATC_CONV, xq, 1.0f, 128, 128, 0);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_qrdy + 8 * (it & 1));
        }
    } else if (warp == ATC_THREADS / 32) {
        // ================= MMA warp =================
        if (lane == 0) {
            const uint32_t idpv = umma_idesc_f16(128, 64) | (1u << 16);       // B (values) MN-major
            const uint32_t dm = tmem + (uint32_t)ATC_OCOL, dc = dm + 64u;
            const uint64_t kh = umma_desc_sw128(smem_u32(KP)), kl = umma_desc_sw128(smem_u32(KP + ATC_KP));
            const uint64_t vh = umma_desc_sw128(smem_u32(VP)), vl = umma_desc_sw128(smem_u32(VP + ATC_KP));
            // the scores of item `it`, 16 dims (32 bytes along the swizzled rows) at a time: the first batch waits for
            // the item's query pairs and for the score columns to be free (the team holds the previous item's scores
            // in registers; for item 0, for the key pairs instead), the last one commits
            auto score_batch = [&](int it, int k) {
                if (k == 0) {
                    w.wait(bar_qrdy + 8 * (it & 1), (uint32_t)(it >> 1) & 1u, 12);
                    if (it > 0) w.wait(bar_sfree, (uint32_t)(it - 1) & 1u, 18);
                    else w.wait(bar_krdy, 0, 18);
                    tc_fence_after();
                }
                const uint64_t qh = umma_desc_sw128(smem_u32(QB + (it & 1) * ATC_QB)) + (uint64_t)(k * 2);
                const uint64_t ql = umma_desc_sw128(smem_u32(QB + (it & 1) * ATC_QB + 16384)) + (uint64_t)(k * 2);
                for (int r0 = 0; r0 < nkp; r0 += 256) {                   // N <= 256 per MMA: 256 + 32 for a full row
                    const int nrows = (nkp - r0) < 256 ? (nkp - r0) : 256;
                    const uint32_t idesc = umma_idesc_f16(128, nrows);
                    const uint32_t d = tmem + (uint32_t)r0;
                    const uint64_t ro = (uint64_t)(r0 * 8 + k * 2);       // r0 rows of 128 bytes, in 16-byte units
                    umma_f16(d, ql, kh + ro, idesc, k ? 1u : 0u);
                    umma_f16(d, qh, kl + ro, idesc, 1u);
                    umma_f16(d, qh, kh + ro, idesc, 1u);
                }
                if (k == 3) umma_commit(bar_s);
            };
            uint32_t use[2] = {0u, 0u};                                   // hand-overs seen so far per P half
            for (int k = 0; k < 4; k++) score_batch(0, k);
            for (int it = 0; it < gn; it++) {
                int sb = it + 1 < gn ? 0 : 4;                             // score batches of the next item still to issue
                const uint64_t p1 = umma_desc_sw128(smem_u32(QB + (it & 1) * ATC_QB)), p2 = umma_desc_sw128(smem_u32(QB + (it & 1) * ATC_QB + 16384));
                for (int c = 0; c < nchunks; c++) {
                    const int hf = c & 1;
                    w.wait(bar_rdy0 + 8 * hf, use[hf] & 1u, 17);
                    use[hf]++;
                    tc_fence_after();
#pragma unroll
                    for (int k = 0; k < 2; k++) {                         // 16 keys per MMA: 32 bytes of a P row, two 8-key groups of V rows
                        const uint64_t po = (uint64_t)((2 * hf + k) * 2), vo = (uint64_t)(c * 256 + k * 128);
                        umma_f16(dm, p1 + po, vh + vo, idpv, (c | k) ? 1u : 0u);
                        umma_f16(dc, p1 + po, vl + vo, idpv, (c | k) ? 1u : 0u);
                        umma_f16(dc, p2 + po, vh + vo, idpv, 1u);
                    }
                    umma_commit(bar_pv0 + 8 * hf);
                    // a quarter of the next item's scores behind each of chunks 1..4: short enough not to hold up the
                    // P V chain, early enough to be done when the team comes back for them
                    if (c >= 1 && sb < 4 && nchunks >= 5) score_batch(it + 1, sb++);
                }
                while (sb < 4) score_batch(it + 1, sb++);
            }
        }
    } else {
        // ================= softmax team =================
        const int r = tid & 127, part = tid >> 7;                     // query row of the tile, which quarter of each chunk's columns
        const int qi = a.pack ? (r & 31) : qt * 128 + r;             // query index inside the sequence row
        const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        // ---- prologue: the keys -> pairs, then the values ----
        {
            float4 xk[5][2];
            w.wait(bar_k, 0, 12);
            atc_units_read<5>(KP, ATC_KP, nkp, tid, xk);
            __syncwarp();
            atc_units_write<5>(KP, ATC_KP, nkp, tid, xk, 1.0f, nkp, nkp, 0);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_krdy);
            w.wait(bar_v, 0, 14);
            atc_units_read<5>(VP, ATC_KP, nkp, tid, xk);
            __syncwarp();
            atc_units_write<5>(VP, ATC_KP, nkp, tid, xk, ATC_LO_SCALE, n1p, n1, n2);
            // made visible to the MMA warp by the fence before the first P hand-over
        }
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
        const float sl2 = a.scale * 1.4426950408889634f;
        const uint32_t rowoff = (uint32_t)((r >> 3) * 1024 + (r & 7) * 128);
        uint32_t use0 = 0u, use1 = 0u;                                // hand-overs made so far per P half
        for (int it = 0; it < gn; it++) {
            unsigned char *Pb = QB + (it & 1) * ATC_QB;               // this item's query pairs, dead once its scores are in
            const int h = a.pack ? h0 + (r >> 5) : h0 + it;
            w.wait(bar_s, (uint32_t)it & 1u, 13);
            tc_fence_after();
            // The thread's scores -- eight columns of every chunk -- are read from tensor memory ONCE, all loads in
            // flight together, and stay in registers for the maximum and for the exponentials.
            uint32_t sv[NCH][8];
#pragma unroll
            for (int c = 0; c < NCH; c++) tmem_ld8_issue(lane_addr + (uint32_t)(c * 32 + part * 8), sv[c]);
            tmem_ld_wait();
            tc_fence_before();                                            // the score columns may take the next item's scores
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_sfree);
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < NCH; c++) {
                if (c < nchunks) {
                    // columns this query does not see (padding, causal / window limits) become -inf once, here: the
                    // maximum and the exponentials below then run without range tests (2^-inf = 0)
                    int jlo, jhi;
                    chunk_range(c, jlo, jhi);
                    jlo -= part * 8; jhi -= part * 8;
                    uint32_t *v = sv[c];
                    if (jlo > 0 || jhi < 8) {
#pragma unroll
                        for (int j = 0; j < 8; j++)
                            if (j < jlo || j >= jhi) v[j] = 0xff800000u;
                    }
                    const float m0 = atc_max3(__uint_as_float(v[0]), __uint_as_float(v[1]), __uint_as_float(v[2]));
                    const float m1 = atc_max3(__uint_as_float(v[3]), __uint_as_float(v[4]), __uint_as_float(v[5]));
                    mx = atc_max3(mx, m0, atc_max3(m1, __uint_as_float(v[6]), __uint_as_float(v[7])));
                }
            }
            xmax[tid] = mx;
            team_sync();
            mx = fmaxf(fmaxf(xmax[r], xmax[r + 128]), fmaxf(xmax[r + 256], xmax[r + 384]));
            const bool any = mx != -INFINITY;
            // 2^(s sl2 - mx sl2): one multiply-add per score; a row that sees no key keeps its -inf scores as they are
            const float nmx = any ? -mx * sl2 : 0.f;
            float l = 0.f;
#pragma unroll
            for (int c = 0; c < NCH; c++) {
                if (c >= nchunks) break;
                const int hf = c & 1;
                {
                    const uint32_t *v = sv[c];
                    uint32_t hw[4], lw[4];                                 // eight probabilities as packed fp16 pairs
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const float x0 = atc_ex2(fmaf(__uint_as_float(v[2 * e]), sl2, nmx)), x1 = atc_ex2(fmaf(__uint_as_float(v[2 * e + 1]), sl2, nmx));
                        l += x0 + x1;
                        h16_pair2_raw(x0, x1, hw[e], lw[e], ATC_LO_SCALE);
                    }
                    // the probabilities are ready in registers; only the stores need the half free: the MMAs of its
                    // previous hand-over are done with it
                    { const uint32_t n = hf ? use1 : use0; if (n >= 1u) w.wait(bar_pv0 + 8 * hf, (n - 1u) & 1u, 15); }
                    // the thread's eight keys are 16-byte chunk 4 hf + part of its row in the hi tile and in the lo tile
                    const uint32_t o = rowoff + ((uint32_t)(((4 * hf + part) ^ (r & 7)) & 7) << 4);
                    *(uint4 *)(Pb + o) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
                    *(uint4 *)(Pb + 16384 + o) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
                }
                // hand the half to the MMA warp: this warp's writes (and its reads of the previous item's output) are
                // ordered before the MMAs, one arrival per warp
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_rdy0 + 8 * hf);
                if (hf) use1++; else use0++;
            }
            // the commits complete in order: the last one covers every earlier MMA of the item
            { const int hf = (nchunks - 1) & 1; const uint32_t n = hf ? use1 : use0; w.wait(bar_pv0 + 8 * hf, (n - 1u) & 1u, 16); }
            tc_fence_after();
            xsum[tid] = l;
            team_sync();
            l = (xsum[r] + xsum[r + 128]) + (xsum[r + 256] + xsum[r + 384]);
            if (a.ml && part == 0 && qi < nq) {
                float *mlp = a.ml + ((int64_t)(q0 + qi) * a.H + h) * 2;
                mlp[0] = any ? mx * sl2 : -INFINITY; mlp[1] = l;
            }
            // ---- output rows: O / l; the four threads of a row take 16 columns each ----
            {
                const float inv = l > 0.f ? 1.0f / l : 0.f;
                float o[16];
                {
                    uint32_t v[16], vc[16];
                    tmem_ld16_issue(lane_addr + (uint32_t)(ATC_OCOL + part * 16), v);
                    tmem_ld16_issue(lane_addr + (uint32_t)(ATC_OCOL + 64 + part * 16), vc);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; j++) o[j] = fmaf(__uint_as_float(vc[j]), ATC_LO_UNSCALE, __uint_as_float(v[j])) * inv;
                }
                const bool h16 = a.out_lo && a.out_fmt == SPLIT_H16;
                if (a.out_lo && !h16) {
                    // TF32 hi / lo outputs (two fp32 arrays) go straight to global memory, a thread per 64-byte piece
                    if (tid == 0 && it + 2 < gn) load_q(it + 2);
                    if (qi < nq && h < (kvh + 1) * G && !w.dead) {
                        const int64_t ofs = (int64_t)(q0 + qi) * a.ldo + h * 64 + part * 16;
#pragma unroll
                        for (int j = 0; j < 16; j += 4) store_split4(a.out, a.out_lo, ofs + j, make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]), a.out_fmt);
                    }
                } else {
                    // fp16 pairs or plain fp32: the tile is staged in the item's P tile (every MMA that read it is done)
                    // and leaves as whole 128-byte lines; a thread writing its own row's piece would put 32 lines
                    // into every store instruction
                    unsigned char *St = Pb;
                    if (h16) {
#pragma unroll
                        for (int q = 0; q < 2; q++) {
                            uint32_t hw[4], lw[4];
#pragma unroll
                            for (int e = 0; e < 4; e++) h16_pair2(o[q * 8 + 2 * e], o[q * 8 + 2 * e + 1], hw[e], lw[e]);
                            const uint32_t so = rowoff + ((uint32_t)(((2 * part + q) ^ (r & 7)) & 7) << 4);
                            *(uint4 *)(St + so) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
                            *(uint4 *)(St + 16384 + so) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
                        }
                    } else {
#pragma unroll
                        for (int q = 0; q < 4; q++)                           // 256-byte rows, 16-byte pieces swizzled by the row
                            *(float4 *)(St + r * 256 + ((uint32_t)(((4 * part + q) ^ (r & 15)) & 15) << 4)) = make_float4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
                    }
                    team_sync();
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        const int idx = tid + k * ATC_THREADS;                // 2048 16-byte pieces
                        const int rr = h16 ? (idx >> 3) & 127 : idx >> 4;
                        const int qi2 = a.pack ? (rr & 31) : qt * 128 + rr, h2 = a.pack ? h0 + (rr >> 5) : h;
                        if (qi2 < nq && h2 < (kvh + 1) * G) {
                            const int64_t e0 = (int64_t)(q0 + qi2) * a.ldo + h2 * 64;
                            if (h16) {
                                const int tile = idx >> 10, j = idx & 7;
                                const uint4 x = *(const uint4 *)(St + tile * 16384 + (rr >> 3) * 1024 + (rr & 7) * 128 + (((j ^ (rr & 7)) & 7) << 4));
                                *(uint4 *)((unsigned short *)(tile ? a.out_lo : a.out) + e0 + j * 8) = x;
                            } else {
                                const int j = idx & 15;
                                *(float4 *)(a.out + e0 + j * 4) = *(const float4 *)(St + rr * 256 + (((j ^ (rr & 15)) & 15) << 4));
                            }
                        }
                    }
                    team_sync();                                              // the staged tile has left
                    // the tile now takes the query tile of the item after the next
                    if (tid == 0 && it + 2 < gn) {
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        load_q(it + 2);
                    }
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
    if (((a.ldq | a.ldk1 | a.ldk2) & 3) || (a.ldo & 7)) return false;
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
    const int G = a.H / a.Hkv;
    d.pack = (!ml && a.max_q <= 32 && G >= 2 && G <= 4) ? 1 : 0;
    // heads per CTA: all heads of a kv group share one fetch and conversion of its keys and values, as long as
    // that leaves at least two CTAs per SM; fewer heads per CTA (a divisor of the group) otherwise
    const char *hpc_s = getenv("NCM_B200_ATTN_HPC");                  // read per call: the tests force each grouping
    const int hpc_env = hpc_s ? atoi(hpc_s) : 0;
    d.hpc = 1;
    if (!d.pack) {
        const int64_t per_head = (int64_t)cdiv(a.max_q, 128) * a.rows * a.H;
        for (int c = G; c >= 1; c--)
            if (G % c == 0 && (c == 1 || per_head / c >= 2 * (int64_t)ctx().sm_count)) { d.hpc = c; break; }
        if (hpc_env > 0 && G % hpc_env == 0) d.hpc = hpc_env;
    }
    const CUtensorMap mq = tc_get_map(a.q, a.q_total, a.H * 64, a.ldq, d.pack ? 32 : 128, false);
    const CUtensorMap mk1 = tc_get_map(a.k1, a.k1_total, 2 * a.Hkv * 64, a.ldk1, 32, false);
    const CUtensorMap mk2 = a.k2 ? tc_get_map(a.k2, a.k2_total, 2 * a.Hkv * 64, a.ldk2, 32, false) : mk1;
    static bool set = false;
    if (!set) {
        CUDA_CHECK(cudaFuncSetAttribute(k_attention_tc<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATC_SMEM));
        CUDA_CHECK(cudaFuncSetAttribute(k_attention_tc<9>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATC_SMEM));
        set = true;
    }
    dim3 grid((unsigned)cdiv(a.max_q, 128), (unsigned)(d.pack ? a.Hkv : a.H / d.hpc), (unsigned)a.rows);
    const int max_n1 = ml ? std::min(kb_len, a.max_k1) : a.max_k1;
    const int max_keys = ((max_n1 + 31) & ~31) + (a.k2 ? ((a.max_k2 + 31) & ~31) : 0);
    if (max_keys <= 256) {
        LAUNCH_PDL_IF(pdl_small((int64_t)grid.x * grid.y * grid.z), k_attention_tc<8>, grid, ATC_BLOCK, ATC_SMEM, mq, mk1, mk2, d);
    } else {
        LAUNCH_PDL_IF(pdl_small((int64_t)grid.x * grid.y * grid.z), k_attention_tc<9>, grid, ATC_BLOCK, ATC_SMEM, mq, mk1, mk2, d);
    }
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
    if (((a.ldq | a.ldk1) & 3) || (a.ldo & 7)) return false;
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
