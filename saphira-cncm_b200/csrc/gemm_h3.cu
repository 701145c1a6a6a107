// fp32-grade GEMM on the fp16 tensor path of sm_100a: y = act(x W^T + bias) (+ res).
//
// Both operands are carried as pairs of fp16 arrays,
//     s v = v1 + v2,   v1 = rn_f16(s v),   v2 = rn_f16(s v - v1)
// (22 significant bits). s is a power of two that keeps the remainders clear of the fp16 subnormals: 16 for
// activations (fixed by the pair format), per matrix for weights (its largest element goes to [8192, 16384)).
// The product is
//     s_x s_w x W^T = x1 W1^T + x2 W1^T + x1 W2^T          (the x2 W2^T term, 2^-22 of the product, is dropped)
// so every k-step issues three tcgen05.mma.kind::f16 into ONE fp32 accumulator in tensor memory, smallest
// terms first, and the epilogue multiplies by 1 / (s_x s_w). Against three TF32 passes this moves half the
// operand bytes and runs on the twice-as-fast fp16 pipe.
//
// Structure: persistent CTAs (one per SM) walking output tiles of 128 x BN (BN = 256 for large problems: an MMA
// of 256 columns reads the 128-row activation tile once for twice the arithmetic, and it is the operand fetch from
// shared memory that paces 128-column MMAs); warp 0 feeds a ring of shared-memory stages by TMA (two 128 x 64
// and two BN x 64 fp16 tiles per stage, 128-byte swizzle), one lane of warp 1 issues the MMAs, warps 2-9 run the
// fused epilogue out of tensor memory (half of the tile's columns each). Two accumulators alternate so a tile's
// epilogue overlaps the next tile's MMAs (2 x 256 columns: all of tensor memory). Every mbarrier wait is bounded;
// a timeout records a code and drains.
#include "common.cuh"
#include "tc_common.cuh"
#include "tc_epilogue.cuh"

#include <algorithm>
#include <unordered_map>

namespace ncmb {

constexpr int H3_BM = 128, H3_BK = 64;                   // BK halfs = 128 bytes = one swizzle row
// Tile widths: 128 columns for large problems; 64 or 32 columns for small ones (batched decode steps, the first
// NCP levels), chosen per call so that the busiest CTA moves the fewest bytes.
// (256-column tiles: two stages of 96 KB. Four stages of 48 KB -- k-blocks of 32 halfs in 64-byte-swizzled rows --
// were measured 8% slower: the MMAs fetch 64-byte rows less efficiently)
constexpr int h3_stages(int BN) { return BN >= 256 ? 2 : BN >= 128 ? 3 : 4; }
constexpr int H3_EPI_WARPS = 8;                         // two per TMEM lane quadrant, 64 columns each
constexpr int H3_THREADS = 64 + 32 * H3_EPI_WARPS;
constexpr int H3_TILE = 128 * H3_BK * 2;                 // one 128-row operand tile: 16 KB
constexpr int h3_wtile(int BN) { return BN * H3_BK * 2; }  // one BN-row weight tile
constexpr int h3_stage(int BN) { return 2 * H3_TILE + 2 * h3_wtile(BN); }   // x1 | x2 | W1 | W2


// QKP: the epilogue applies the per-head RMSNorm / rotary embedding of a fused QKV projection (128-column tiles)
template <int H3_BN, bool QKP = false>
__global__ void __launch_bounds__(H3_THREADS, 1) k_gemm_h3(const __grid_constant__ CUtensorMap tmX1,
                                                       const __grid_constant__ CUtensorMap tmX2,
                                                       const __grid_constant__ CUtensorMap tmW1,
                                                       const __grid_constant__ CUtensorMap tmW2,
                                                       const __grid_constant__ CUtensorMap tmY,
                                                       TcEpi ep, int num_kb, int tiles_n, int num_tiles, int ksplit, int kb_per,
                                                       int m_pad, int skip_w2) {
    // skip_w2: every element of the W2 half is zero (a matrix whose scaled elements are all fp16 values, which is the
    // case for bf16 weights): the x1 W2 product is not issued -- two MMAs per k-step instead of three, same result
    // ksplit > 1: a work item is (output tile, slice of K); the item's raw sums go to slice s of a partial buffer whose
    // slices are m_pad rows apart (the tensor map of the stores covers all slices), and a second kernel adds the slices
    pdl_launch_dependents();          // programmatic dependent launch: see launch_pdl()
    pdl_wait();
    constexpr int H3_STAGES = h3_stages(H3_BN), H3_STAGE = h3_stage(H3_BN), H3_WTILE = h3_wtile(H3_BN);
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    // barriers: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
    unsigned char *stage0 = smem + H3_STAGES * H3_STAGE;         // one 4 KB store staging buffer per epilogue warp
    uint64_t *bars = (uint64_t *)(stage0 + H3_EPI_WARPS * 4096);
    uint32_t *tmem_slot = (uint32_t *)(bars + 2 * H3_STAGES + 4);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + H3_STAGES);
    const uint32_t afull0 = smem_u32(bars + 2 * H3_STAGES), aempty0 = smem_u32(bars + 2 * H3_STAGES + 2);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < H3_STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; a++) { mbar_init(afull0 + 8 * a, 1); mbar_init(aempty0 + 8 * a, H3_EPI_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmX1) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmX2) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmW1) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmW2) : "memory");
    }
    if (warp == 1) {   // two accumulators of BN columns: a tile's epilogue runs under the next tile's MMAs
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * H3_BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int kbg = 0, armed = 0;                       // k-block counter over all of this CTA's tiles
            bool ok = true;
            for (int w = blockIdx.x; w < num_tiles * ksplit && ok; w += gridDim.x) {
                const int t = w / ksplit, ks = w - t * ksplit;
                const int n0 = (t % tiles_n) * H3_BN, m0 = (t / tiles_n) * H3_BM;
                const int kb1 = min(num_kb, (ks + 1) * kb_per);
                for (int kb = ks * kb_per; kb < kb1; kb++, kbg++) {
                    int s = kbg % H3_STAGES; uint32_t ph = (uint32_t)(kbg / H3_STAGES) & 1u;
                    ok = mbar_wait(empty0 + 8 * s, ph ^ 1u, ep.err, 21);
                    if (!ok) break;
                    const uint32_t dst = smem_u32(smem + s * H3_STAGE), bar = full0 + 8 * s;
                    mbar_expect_tx(bar, skip_w2 ? H3_STAGE - H3_WTILE : H3_STAGE);       // an all-zero second half is neither fetched nor multiplied
                    tma_load_2d(dst, &tmX1, kb * H3_BK, m0, bar);
                    tma_load_2d(dst + H3_TILE, &tmX2, kb * H3_BK, m0, bar);
                    tma_load_2d(dst + 2 * H3_TILE, &tmW1, kb * H3_BK, n0, bar);
                    if (!skip_w2) tma_load_2d(dst + 2 * H3_TILE + H3_WTILE, &tmW2, kb * H3_BK, n0, bar);
                    armed = kbg + 1;
                }
            }
            if (!ok) {   // drain: wait (bounded) for the copies already in flight before leaving
                int first = armed - H3_STAGES < 0 ? 0 : armed - H3_STAGES;
                for (int k = first; k < armed; k++) mbar_wait(full0 + 8 * (k % H3_STAGES), (uint32_t)(k / H3_STAGES) & 1u, ep.err, 24);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_f16(H3_BM, H3_BN);
            int kbg = 0, it = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < num_tiles * ksplit && ok; w += gridDim.x, it++) {
                const int acc = it & 1; const uint32_t use = (uint32_t)(it >> 1);
                ok = mbar_wait(aempty0 + 8 * acc, (use & 1u) ^ 1u, ep.err, 25);    // epilogue has drained this accumulator pair
                if (!ok) break;
                tc_fence_after();
                const uint32_t tacc = tmem_base + (uint32_t)(acc * H3_BN);
                const int nkb = min(num_kb, (w % ksplit + 1) * kb_per) - (w % ksplit) * kb_per;
                for (int kb = 0; kb < nkb; kb++, kbg++) {
                    int s = kbg % H3_STAGES; uint32_t ph = (uint32_t)(kbg / H3_STAGES) & 1u;
                    ok = mbar_wait(full0 + 8 * s, ph, ep.err, 22);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t base = smem_u32(smem + s * H3_STAGE);
                    const uint64_t x1 = umma_desc_sw128(base), x2 = umma_desc_sw128(base + H3_TILE);
                    const uint64_t w1 = umma_desc_sw128(base + 2 * H3_TILE), w2 = umma_desc_sw128(base + 2 * H3_TILE + H3_WTILE);
#pragma unroll
                    for (int k = 0; k < H3_BK / 16; k++) {    // 16 halfs (32 bytes) per MMA: advance the start address
                        const uint64_t o = (uint64_t)(k * 2);
                        umma_f16(tacc, x2 + o, w1 + o, idesc, (kb | k) ? 1u : 0u);
                        if (!skip_w2) umma_f16(tacc, x1 + o, w2 + o, idesc, 1u);
                        umma_f16(tacc, x1 + o, w1 + o, idesc, 1u);
                    }
                    umma_commit(empty0 + 8 * s);             // stage reusable once these MMAs have read it
                }
                umma_commit(afull0 + 8 * acc);               // accumulators complete (also reached on the error path)
            }
        }
    } else {
        const int q = warp & 3;                              // TMEM lane quadrant this warp may read
        const int ch = (warp - 2) >> 2;                      // which half of the tile's 32-column chunks this warp drains
        constexpr int NCH = H3_BN / 64;                      // chunks per warp (BN = 32: the first four warps take the one chunk)
        constexpr int NCH1 = NCH > 0 ? NCH : 1;
        const bool has_cols = NCH > 0 || ch == 0;
        int it = 0;
        bool ok = true;
        const bool glu_fast = tc_glu_silu_h16(ep);
        unsigned char *stage = stage0 + (warp - 2) * 4096;
        for (int w = blockIdx.x; w < num_tiles * ksplit && ok; w += gridDim.x, it++) {
            const int t = w / ksplit;
            const int64_t slice_row0 = (int64_t)(w - t * ksplit) * m_pad;          // row offset of this K slice's partial sums
            const int acc = it & 1; const uint32_t use = (uint32_t)(it >> 1);
            const int n0 = (t % tiles_n) * H3_BN + ch * (H3_BN / 2);
            const int64_t m = (int64_t)(t / tiles_n) * H3_BM + q * 32 + lane;
            // the residual of this thread's 64 outputs is requested before the accumulators are waited for,
            // so its latency runs under the tile's MMAs
            // (two chunks are in flight at a time: a chunk's slot takes the chunk after the next once it is used)
            constexpr int NPRE = NCH1 < 2 ? NCH1 : 2;
            float4 resv[8 * NPRE];
            bool pre[NCH1];
            // fp32 tiles that leave by TMA store: the warp fetches the residual block together, full row segments per
            // request (see tc_epilogue_chunk_tma_coop); otherwise every thread fetches its own row
            const bool coop = ep.tma_store && ep.res && has_cols && ((ep.ldres & 3) == 0) && (((uintptr_t)ep.res & 15) == 0);
            auto fetch_res = [&](int c) {
                float4 *rv = &resv[(c % NPRE) * 8];
                if (coop && n0 + c * 32 + 32 <= ep.N) {
                    pre[c] = true;
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const int64_t row = (m - lane) + i * 4 + (lane >> 3);
                        rv[i] = row < ep.M ? *(const float4 *)(ep.res + row * ep.ldres + n0 + c * 32 + (lane & 7) * 4)
                                           : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                    return;
                }
                pre[c] = !coop && has_cols && tc_residual_prefetchable(ep, m, n0, c * 32);
                if (pre[c]) {
                    const float4 *rr = (const float4 *)(ep.res + m * ep.ldres + n0 + c * 32);
#pragma unroll
                    for (int j = 0; j < 8; j++) rv[j] = rr[j];
                }
            };
#pragma unroll
            for (int c = 0; c < NPRE; c++) fetch_res(c);
            ok = mbar_wait(afull0 + 8 * acc, use & 1u, ep.err, 23);
            tc_fence_after();
            if (!ok) break;
            const uint32_t trow = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * H3_BN + ch * (H3_BN / 2));
            if constexpr (QKP) {
                // both halves of the thread's head (64 columns) before anything is stored
                uint32_t r0[32], r1[32];
                tmem_ld32_issue(trow, r0);
                tmem_ld32_issue(trow + 32u, r1);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    r0[j] = __float_as_uint(__uint_as_float(r0[j]) * ep.acc_scale);
                    r1[j] = __float_as_uint(__uint_as_float(r1[j]) * ep.acc_scale);
                }
                tc_epilogue_head_qkpost(ep, r0, r1, m, m - lane, n0, stage, &tmY, lane);
            } else
#pragma unroll
            for (int c = 0; c < NCH1; c++) {
                if (!has_cols) break;
                uint32_t r[32];
                tmem_ld32(trow + (uint32_t)(c * 32), r);
#pragma unroll
                for (int j = 0; j < 32; j++) r[j] = __float_as_uint(__uint_as_float(r[j]) * ep.acc_scale);
                float4 *rv = &resv[(c % NPRE) * 8];
                if (glu_fast) tc_epilogue_glu_silu_h16(ep, r, m, n0, c * 32);
                else if (coop && n0 + c * 32 + 32 <= ep.N)
                    tc_epilogue_chunk_tma_coop(ep, r, m - lane, n0, c * 32, rv, stage, &tmY, lane);
                else if (ep.tma_store && n0 + c * 32 + 32 <= ep.N)
                    tc_epilogue_chunk_tma(ep, r, m, m - lane + slice_row0, n0, c * 32, pre[c] ? rv : nullptr, stage, &tmY, lane);
                else tc_epilogue_chunk(ep, r, m, n0, c * 32, pre[c] ? rv : nullptr);
                if (c + NPRE < NCH1) fetch_res(c + NPRE);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(aempty0 + 8 * acc);   // one arrival per epilogue warp frees the pair
        }
        // result tiles still on their way out of the staging buffer must be written before the CTA retires
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * H3_BN) : "memory");
    }
}

// ------------------------------------------------------------------ host side

// fp32 [rows][K] (row stride ldx) -> the fp16 pair, dense [rows][K] each
__global__ void k_split_h16(const float *__restrict__ x, int64_t ldx, unsigned short *__restrict__ v1,
                            unsigned short *__restrict__ v2, int64_t rows, int K4) {
    int64_t total = rows * K4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t r = i / K4; int c = (int)(i % K4);
        float4 v = *(const float4 *)(x + r * ldx + c * 4);
        store_split4((float *)v1, (float *)v2, i * 4, v, SPLIT_H16);
    }
}
static void split_h16(const float *x, int64_t ldx, void *v1, void *v2, int64_t rows, int K) {
    int64_t n = rows * (K / 4);
    int64_t g = cdiv(n, 256), cap = (int64_t)ctx().sm_count * 16;
    ProfScope ps(NCMB_K_ELEM, 0, (double)rows * K * 8);
    LAUNCH(k_split_h16, (unsigned)(g > cap ? cap : (g < 1 ? 1 : g)), 256, 0, x, ldx, (unsigned short *)v1,
           (unsigned short *)v2, rows, K / 4);
}

// ---- weight matrices: scaled pair + "second half all zero" test ----
__global__ void k_absmax(const float *__restrict__ w, int64_t n, unsigned *__restrict__ out) {
    unsigned m = 0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        m = max(m, __float_as_uint(fabsf(w[i])));                 // non-negative floats order like their bits
    for (int o = 16; o; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) atomicMax(out, m);
}
__global__ void k_split_h16_scaled(const float *__restrict__ w, float scale, unsigned short *__restrict__ v1, unsigned short *__restrict__ v2,
                                   int64_t n, unsigned *__restrict__ lo_seen) {
    unsigned any = 0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const float t = w[i] * scale;
        const unsigned short hi = f16_sat(t), lo = f16_sat(t - __half2float(__ushort_as_half(hi)));
        v1[i] = hi; v2[i] = lo;
        any |= (unsigned)(lo & 0x7fffu);
    }
    if (__any_sync(0xffffffffu, any != 0) && (threadIdx.x & 31) == 0) atomicOr(lo_seen, 1u);
}
// one-time conversion of a static weight matrix (a host synchronisation: the scale depends on the largest element)
static void split_h16_weights(const float *W, unsigned short *v1, unsigned short *v2, int64_t n, float *scale_out, bool *w2_zero) {
    static const bool no_scale = getenv("NCM_B200_H3_NO_WSCALE") != nullptr;
    unsigned *d = (unsigned *)dev_alloc(8);
    CUDA_CHECK(cudaMemsetAsync(d, 0, 8, stream()));
    const int64_t g = cdiv(n, 256), cap = (int64_t)ctx().sm_count * 16;
    const unsigned grid = (unsigned)(g > cap ? cap : (g < 1 ? 1 : g));
    float scale = 1.0f;
    if (!no_scale) {
        LAUNCH(k_absmax, grid, 256, 0, W, n, d);
        unsigned bits = 0;
        CUDA_CHECK(cudaMemcpyAsync(&bits, d, 4, cudaMemcpyDeviceToHost, stream()));
        CUDA_CHECK(cudaStreamSynchronize(stream()));
        float mx;
        memcpy(&mx, &bits, 4);
        if (mx > 0.f && std::isfinite(mx)) {
            int e = 0;
            frexpf(mx, &e);                                        // mx = f * 2^e, f in [0.5, 1)
            int sh = 14 - e;                                       // mx * 2^sh in [8192, 16384)
            if (sh > 24) sh = 24;
            if (sh < -24) sh = -24;
            scale = ldexpf(1.0f, sh);
        }
    }
    ProfScope ps(NCMB_K_ELEM, 0, (double)n * 8);
    LAUNCH(k_split_h16_scaled, grid, 256, 0, W, scale, v1, v2, n, d + 1);
    unsigned seen = 1;
    CUDA_CHECK(cudaMemcpyAsync(&seen, d + 1, 4, cudaMemcpyDeviceToHost, stream()));
    CUDA_CHECK(cudaStreamSynchronize(stream()));
    static const bool no_skip = getenv("NCM_B200_H3_NO_SKIP_W2") != nullptr;
    *scale_out = scale;
    *w2_zero = !seen && !no_skip;
    dev_free(d);
}

// cached pair of a weight matrix: formed from W * scale (a power of two that brings the largest element to
// [8192, 16384): small weights stay clear of the fp16 subnormals); w2_zero: no element needed its second half
struct ShadowH { unsigned short *v1, *v2; int64_t n; float scale; bool w2_zero; };
static std::unordered_map<const float *, ShadowH> &shadow_h() { static std::unordered_map<const float *, ShadowH> c; return c; }
static Workspace &split_ws_h() { static Workspace w; return w; }

// Drops the cached fp16 pairs of weights (call when weight memory is freed or rewritten).
void gemm_h3_forget_weights() {
    for (auto &kv : shadow_h()) dev_free(kv.second.v1);
    shadow_h().clear();
}

// Drops the cached pairs of every weight matrix that overlaps [p, p + bytes): called when that memory is rewritten
// or freed through the public memory functions, so a matrix never runs on copies of its old contents.
void gemm_h3_forget_range(const void *p, size_t bytes) {
    auto &sc = shadow_h();
    const char *lo = (const char *)p, *hi = lo + bytes;
    for (auto it = sc.begin(); it != sc.end();) {
        const char *w0 = (const char *)it->first, *w1 = w0 + (size_t)it->second.n * 4;
        if (w0 < hi && lo < w1) { CUDA_CHECK(cudaStreamSynchronize(stream())); dev_free(it->second.v1); it = sc.erase(it); }
        else ++it;
    }
}

static inline bool al16(const void *p) { return ((uintptr_t)p & 15) == 0; }

bool gemm_h3_supported(const GemmArgs &a) {
    int64_t ldx = a.ldx ? a.ldx : a.K, ldy = a.ldy ? a.ldy : (a.glu ? a.N / 2 : a.N);
    if (a.argmin_best) return false;                                // nearest-row search stays on the TF32 kernel
    if (a.M <= 16 || a.N < 32 || a.K < 32) return false;           // up to 16 rows: the weight-streaming GEMV kernel
    if ((a.K & 7) || (ldx & 7)) return false;                       // fp16 rows: TMA strides are multiples of 16 bytes
    if (a.x_lo && a.x_fmt != SPLIT_H16) return false;
    if (!al16(a.x) || (a.x_lo && !al16(a.x_lo)) || !al16(a.W) || !al16(a.y) || (a.y_lo && !al16(a.y_lo)) ||
        (a.bias && !al16(a.bias)) || (a.res && !al16(a.res))) return false;
    if (a.glu && ((a.N & 1) || (ldy & 1))) return false;
    if (a.y_lo && a.y_fmt == SPLIT_H16 && (ldy & 7)) return false;
    return true;
}

// y = act(sum_s part[s] + bias) + res, the slices added in order (N a multiple of 4, rows 16-byte aligned)
__global__ void k_splitk_reduce(const float *__restrict__ part, int ksplit, int64_t m_pad, int64_t M, int N, const float *__restrict__ bias,
                                int act, const float *__restrict__ res, int64_t ldres, float *__restrict__ y, int64_t ldy) {
    pdl_launch_dependents();
    pdl_wait();
    const int n4 = N / 4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < M * n4; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = i / n4; const int c = (int)(i % n4) * 4;
        float4 v = *(const float4 *)(part + m * N + c);
        for (int s = 1; s < ksplit; s++) {
            const float4 p = *(const float4 *)(part + ((int64_t)s * m_pad + m) * N + c);
            v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
        }
        if (bias) { const float4 b = *(const float4 *)(bias + c); v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w; }
        if (act != ACT_NONE) { v.x = tc_act(v.x, act); v.y = tc_act(v.y, act); v.z = tc_act(v.z, act); v.w = tc_act(v.w, act); }
        if (res) { const float4 r = *(const float4 *)(res + m * ldres + c); v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w; }
        *(float4 *)(y + m * ldy + c) = v;
    }
}

// The fused QKV epilogue is opt-in (NCM_B200_QK_EPILOGUE=1, read per call so that a test can switch it): it removes
// the norm / rotation pass (2.4 -> 0.6 ms of element-wise kernels per 12-layer generate step) but the K = 512
// projection is already paced by its fp32 epilogue, which grows by as much (25.3 -> 26.6 ms of GEMM), so the step
// as a whole measured 0.3 ms slower with it.
static bool qk_epilogue_on() {
    const char *e = getenv("NCM_B200_QK_EPILOGUE");
    return e && e[0] == '1';
}

void gemm_h3(const GemmArgs &a) {
    if (a.M <= 0 || a.N <= 0) return;
    TcEpi ep{};
    ep.bias = a.bias; ep.res = a.res; ep.ldres = a.ldres ? a.ldres : a.N;
    ep.y = a.y; ep.y_lo = a.y_lo; ep.y_fmt = a.y_fmt; ep.ldy = a.ldy ? a.ldy : (a.glu ? a.N / 2 : a.N);
    ep.M = a.M; ep.N = a.N; ep.act = a.act; ep.glu = a.glu; ep.err = tc_err_flag();
    ep.colnorm = nullptr; ep.best = nullptr;
    ep.qk_heads = a.qk_heads; ep.qk_H = a.qk_H; ep.qk_qw = a.qk_qw; ep.qk_kw = a.qk_kw; ep.qk_cos = a.qk_cos; ep.qk_sin = a.qk_sin; ep.qk_pos = a.qk_pos;
    ep.acc_scale = H16_X_UNSCALE * H16_X_UNSCALE;                  // weights split per call carry the activations' factor
    int skip_w2 = 0;
    const int64_t ldx = a.ldx ? a.ldx : a.K;
    const bool pre_split = a.x_lo != nullptr;
    const int64_t nx = pre_split ? 0 : a.M * a.K, nw = (int64_t)a.N * a.K;
    Workspace &ws = split_ws_h();
    const bool cache_w = ctx().w_static != 0;
    size_t need = (size_t)(2 * nx + (cache_w ? 0 : 2 * nw)) * 2 + 4096;
    if (need > ws.cap) ws.reserve(need + need / 4);
    ws.reset();
    const void *x1 = a.x, *x2 = a.x_lo;
    int64_t ldh = ldx;
    if (!pre_split) {
        unsigned short *p1 = ws.get<unsigned short>(nx), *p2 = ws.get<unsigned short>(nx);
        split_h16(a.x, ldx, p1, p2, a.M, a.K);
        x1 = p1; x2 = p2; ldh = a.K;
    }
    const unsigned short *w1, *w2;
    if (cache_w) {
        auto &sc = shadow_h();
        auto it = sc.find(a.W);
        if (it == sc.end() || it->second.n != nw) {
            if (it != sc.end()) dev_free(it->second.v1);
            unsigned short *buf = (unsigned short *)dev_alloc((size_t)2 * nw * 2);
            float scale = 1.0f; bool w2_zero = false;
            split_h16_weights(a.W, buf, buf + nw, nw, &scale, &w2_zero);
            it = sc.insert_or_assign(a.W, ShadowH{buf, buf + nw, nw, scale, w2_zero}).first;
        }
        w1 = it->second.v1; w2 = it->second.v2;
        ep.acc_scale = H16_X_UNSCALE / it->second.scale;
        skip_w2 = it->second.w2_zero ? 1 : 0;
    } else {
        unsigned short *p1 = ws.get<unsigned short>(nw), *p2 = ws.get<unsigned short>(nw);
        split_h16(a.W, a.K, p1, p2, a.N, a.K);
        w1 = p1; w2 = p2;
    }
    // Tile width. Small problems (decode steps, the first NCP levels) leave most SMs idle with 128-wide tiles and
    // are paced by what ONE CTA pulls through its shared memory: tiles per CTA x bytes per k-step (the 128-row
    // activation pair plus the bn-row weight pair). The width with the least of that wins; ties go to the wider.
    static const bool narrow_ok = !getenv("NCM_B200_NO_BN32");
    const char *bn_s = getenv("NCM_B200_H3_BN");                   // read per call: the tests force each tile width
    const int bn_env = bn_s ? atoi(bn_s) : 0;
    int bn = 128;
    static const bool wide_ok = !getenv("NCM_B200_NO_BN256");
    static const int wide_min_n = getenv("NCM_B200_BN256_MIN_N") ? atoi(getenv("NCM_B200_BN256_MIN_N")) : 1024;
    static const int wide_max_kb = getenv("NCM_B200_BN256_MAX_KB") ? atoi(getenv("NCM_B200_BN256_MAX_KB")) : 8;   // longest K, in 64s
    if (bn_env == 32 || bn_env == 64 || bn_env == 128 || bn_env == 256) bn = bn_env;
    else if (narrow_ok) {
        int64_t best = -1;
        int64_t cost128 = 0;
        for (int cand : {256, 128, 64, 32}) {
            // 256-column tiles run on two stages of 96 KB: enough for a short K, not for a long one, where three
            // stages of 128-column tiles measured faster (the down-projection, K = 2048); at 512 output columns the
            // 128-column tiles were no slower either
            if (cand == 256 && (!wide_ok || a.N % 256 != 0 || a.N < wide_min_n || cdiv(a.K, H3_BK) > wide_max_kb)) continue;
            const int64_t waves = cdiv(cdiv(a.N, cand) * cdiv(a.M, H3_BM), ctx().sm_count);
            const int64_t cost = waves * (2 * 128 + 2 * cand) * 128;     // bytes per 64 halfs of K
            if (cand == 128) cost128 = cost;
            if (best < 0 || cost < best) { best = cost; bn = cand; }
        }
        // a fused QKV projection needs 128-column tiles (two heads each) and saves a whole pass over q and k
        if (qk_epilogue_on() && a.qk_heads > 0 && a.qk_applied && a.N % 128 == 0 && cost128 <= 2 * best) bn = 128;
    }
    const CUtensorMap mx1 = tc_get_map_h16(x1, a.M, a.K, ldh, H3_BM), mx2 = tc_get_map_h16(x2, a.M, a.K, ldh, H3_BM);
    const CUtensorMap mw1 = tc_get_map_h16(w1, a.N, a.K, a.K, bn), mw2 = tc_get_map_h16(w2, a.N, a.K, a.K, bn);
    // fp32 results leave through TMA stores when the rows keep 16-byte strides
    ep.tma_store = (!a.glu && !a.y_lo && (ep.ldy & 3) == 0 && !getenv("NCM_B200_NO_TMA_STORE")) ? 1 : 0;
    int tiles_n = (int)cdiv(a.N, bn);
    int64_t tiles = (int64_t)tiles_n * cdiv(a.M, H3_BM);
    if (tiles > 0x7fffffff) fatal("gemm_h3: too many tiles");
    int num_kb = (int)cdiv(a.K, H3_BK);
    // Few tiles and a long K (batched decode steps): a CTA's serial chain of MMAs, about 53 ns each whatever their
    // width, is what the call takes. K is cut into slices that run as work items of their own; their raw sums go
    // to a partial buffer and k_splitk_reduce adds the slices in order and applies bias / activation / residual.
    static const bool splitk_ok = !getenv("NCM_B200_NO_SPLITK");
    static const int sk_min = getenv("NCM_B200_SPLITK_MINKB") ? atoi(getenv("NCM_B200_SPLITK_MINKB")) : 12;
    static const int sk_per = getenv("NCM_B200_SPLITK_PER") ? atoi(getenv("NCM_B200_SPLITK_PER")) : 2;
    int ksplit = 1, kb_per = num_kb, m_pad = 0;
    float *part = nullptr;
    auto al16 = [](const void *q) { return ((uintptr_t)q & 15) == 0; };
    if (splitk_ok && ep.tma_store && !a.qk_applied && tiles * 2 <= ctx().sm_count && num_kb >= sk_min && a.N % 32 == 0 &&
        al16(a.bias) && al16(a.res) && (ep.ldres & 3) == 0) {
        int want = (int)std::min<int64_t>(ctx().sm_count / tiles, num_kb / sk_per);
        if (want > 16) want = 16;
        if (want >= 2) {
            kb_per = (int)cdiv(num_kb, want);
            ksplit = (int)cdiv(num_kb, kb_per);                    // every slice has at least one k-block
            m_pad = (int)(cdiv(a.M, H3_BM) * H3_BM);
            static float *pbuf = nullptr; static size_t pcap = 0;
            const size_t need = (size_t)ksplit * m_pad * a.N;
            if (need > pcap) {
                if (pbuf) { CUDA_CHECK(cudaStreamSynchronize(stream())); dev_free(pbuf); }
                pbuf = (float *)dev_alloc(need * 4); pcap = need;
            }
            part = pbuf;
        }
    }
    TcEpi epf = ep;                                                // the call's own epilogue, for the reduce kernel
    if (ksplit > 1) { ep.bias = nullptr; ep.res = nullptr; ep.act = ACT_NONE; ep.y = part; ep.ldy = a.N; }
    const CUtensorMap my = !ep.tma_store ? mx1
                          : ksplit > 1 ? tc_get_map(part, (int64_t)ksplit * m_pad, a.N, a.N, 32, false)
                                       : tc_get_map(a.y, a.M, a.N, ep.ldy, 32, false);
    const int64_t items = tiles * ksplit;
    int grid = (int)(items < ctx().sm_count ? items : ctx().sm_count);     // persistent: one CTA per SM
    ProfScope ps(NCMB_K_GEMM, 2.0 * (double)a.M * a.N * a.K,
                 4.0 * ((double)a.M * a.K + (double)a.N * a.K + (double)a.M * a.N));
#define H3_LAUNCH(BN_)                                                                                                      \
    do {                                                                                                                    \
        constexpr size_t smem = 1024 + (size_t)h3_stages(BN_) * h3_stage(BN_) + H3_EPI_WARPS * 4096 + (2 * h3_stages(BN_) + 4) * 8 + 16; \
        static_assert(smem <= 227 * 1024, "stage ring + store staging exceed shared memory");                               \
        static bool set = false;                                                                                            \
        if (!set) { CUDA_CHECK(cudaFuncSetAttribute(k_gemm_h3<BN_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); set = true; } \
        LAUNCH_PDL_IF(pdl_small(tiles * 4), k_gemm_h3<BN_>, grid, H3_THREADS, smem, mx1, mx2, mw1, mw2, my, ep, num_kb, tiles_n, (int)tiles, ksplit, kb_per, m_pad, skip_w2);        \
    } while (0)
    // fused QKV projection: heads are 64 columns, a 128-column tile holds two, results leave as fp32 tiles
    const bool qkp = qk_epilogue_on() && a.qk_heads > 0 && a.qk_applied && bn == 128 && ep.tma_store && a.N % 128 == 0 && !a.res &&
                     a.act == ACT_NONE && (a.qk_qw || a.qk_kw || a.qk_cos) && (!a.qk_cos || a.qk_pos);
    if (a.qk_applied) *a.qk_applied = qkp;
    if (qkp) {
        constexpr size_t smem = 1024 + (size_t)h3_stages(128) * h3_stage(128) + H3_EPI_WARPS * 4096 + (2 * h3_stages(128) + 4) * 8 + 16;
        static bool set = false;
        if (!set) { CUDA_CHECK(cudaFuncSetAttribute((k_gemm_h3<128, true>), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); set = true; }
        LAUNCH_PDL_IF(pdl_small(tiles * 4), (k_gemm_h3<128, true>), grid, H3_THREADS, smem, mx1, mx2, mw1, mw2, my, ep, num_kb, tiles_n, (int)tiles, ksplit, kb_per, m_pad, skip_w2);
    } else if (bn == 32) H3_LAUNCH(32);
    else if (bn == 64) H3_LAUNCH(64);
    else if (bn == 256) H3_LAUNCH(256);
    else H3_LAUNCH(128);
#undef H3_LAUNCH
    if (ksplit > 1) {
        const int64_t n4 = a.M * (int64_t)(a.N / 4), g = cdiv(n4, 256), cap = (int64_t)ctx().sm_count * 8;
        LAUNCH_PDL(k_splitk_reduce, (unsigned)(g > cap ? cap : g), 256, 0, (const float *)part, ksplit, (int64_t)m_pad, a.M, a.N, epf.bias, epf.act,
                   epf.res, epf.ldres, epf.y, epf.ldy);
    }
}

} // namespace ncmb
