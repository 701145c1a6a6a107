// tcgen05 tensor-core GEMM for sm_100a: y = act(x W^T + bias) (+ res), fp32 operands
// consumed as TF32, fp32 accumulation in tensor memory.
//
// One CTA per 128 x BN output tile, six warps:
//   (persistent CTAs, one per SM, each walking a strided list of output tiles)
//   warp 0   TMA producer: cp.async.bulk.tensor tiles of x and W (128-byte swizzle)
//            into a ring of shared-memory stages, completion counted on mbarriers;
//   warp 1   allocates BN columns of tensor memory and (one lane) issues
//            tcgen05.mma.kind::tf32 over each stage, tcgen05.commit frees the stage;
//   warps 2-5 epilogue: tcgen05.ld the accumulator (lane = output row), fuse bias /
//            activation / gated product / residual, store fp32 rows.
// One persistent CTA per SM with two tensor-memory accumulators, so one tile's
// epilogue overlaps the next tile's main loop. Every mbarrier wait is bounded: on a
// timeout the kernel records an error code and drains instead of spinning.
#include "common.cuh"
#include "tc_common.cuh"
#include "tc_epilogue.cuh"

#include <unordered_map>

namespace ncmb {

constexpr int TC_BM = 128;
constexpr int TC_THREADS = 192;

// Persistent kernel: each CTA walks output tiles t = blockIdx.x, blockIdx.x + gridDim.x, ...
// (n-tile fastest, so CTAs running side by side share the same rows of x in L2). The
// shared-memory ring runs continuously across tiles, and two TMEM accumulators alternate:
// while the epilogue warps drain tile i, the MMA warp already accumulates tile i + 1.
//
// X3 = false: one TF32 pass over (A, B).  X3 = true: operands arrive split as
// a = a_hi + a_lo (both exactly representable in TF32) and the tile accumulates
// a_lo b_hi + a_hi b_lo + a_hi b_hi: fp32-grade products from three TF32 MMAs.
template <int BN, int STAGES, bool X3>
__global__ void __launch_bounds__(TC_THREADS) k_gemm_tc(const __grid_constant__ CUtensorMap tmA,
                                                       const __grid_constant__ CUtensorMap tmB,
                                                       const __grid_constant__ CUtensorMap tmAlo,
                                                       const __grid_constant__ CUtensorMap tmBlo,
                                                       TcEpi ep, int num_kb, int tiles_n, int num_tiles) {
    extern __shared__ unsigned char smem_raw[];
    // 1024-byte alignment for the swizzled tiles
    unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    constexpr int A_TILE = TC_BM * TC_BK * 4, B_TILE = BN * TC_BK * 4;
    constexpr int A_BYTES = A_TILE * (X3 ? 2 : 1), B_BYTES = B_TILE * (X3 ? 2 : 1);   // [hi | lo] per stage
    unsigned char *sA = smem, *sB = smem + STAGES * A_BYTES;
    // barriers: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
    uint64_t *bars = (uint64_t *)(sB + STAGES * B_BYTES);
    uint32_t *tmem_slot = (uint32_t *)(bars + 2 * STAGES + 4);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const uint32_t afull0 = smem_u32(bars + 2 * STAGES), aempty0 = smem_u32(bars + 2 * STAGES + 2);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; a++) { mbar_init(afull0 + 8 * a, 1); mbar_init(aempty0 + 8 * a, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB) : "memory");
        if (X3) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmAlo) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmBlo) : "memory");
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * BN) : "memory");
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
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                const int n0 = (t % tiles_n) * BN, m0 = (t / tiles_n) * TC_BM;
                for (int kb = 0; kb < num_kb; kb++, kbg++) {
                    int s = kbg % STAGES; uint32_t ph = (uint32_t)(kbg / STAGES) & 1u;
                    ok = mbar_wait(empty0 + 8 * s, ph ^ 1u, ep.err, 1);
                    if (!ok) break;
                    mbar_expect_tx(full0 + 8 * s, A_BYTES + B_BYTES);
                    tma_load_2d(smem_u32(sA + s * A_BYTES), &tmA, kb * TC_BK, m0, full0 + 8 * s);
                    tma_load_2d(smem_u32(sB + s * B_BYTES), &tmB, kb * TC_BK, n0, full0 + 8 * s);
                    if (X3) {
                        tma_load_2d(smem_u32(sA + s * A_BYTES + A_TILE), &tmAlo, kb * TC_BK, m0, full0 + 8 * s);
                        tma_load_2d(smem_u32(sB + s * B_BYTES + B_TILE), &tmBlo, kb * TC_BK, n0, full0 + 8 * s);
                    }
                    armed = kbg + 1;
                }
            }
            if (!ok) {   // drain: wait (bounded) for the copies already in flight before leaving
                int first = armed - STAGES < 0 ? 0 : armed - STAGES;
                for (int k = first; k < armed; k++) mbar_wait(full0 + 8 * (k % STAGES), (uint32_t)(k / STAGES) & 1u, ep.err, 4);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_tf32(TC_BM, BN);
            int kbg = 0, it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, it++) {
                const int acc = it & 1; const uint32_t use = (uint32_t)(it >> 1);
                ok = mbar_wait(aempty0 + 8 * acc, (use & 1u) ^ 1u, ep.err, 5);     // epilogue has drained this accumulator
                if (!ok) break;
                tc_fence_after();
                const uint32_t tacc = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < num_kb; kb++, kbg++) {
                    int s = kbg % STAGES; uint32_t ph = (uint32_t)(kbg / STAGES) & 1u;
                    ok = mbar_wait(full0 + 8 * s, ph, ep.err, 2);
                    if (!ok) break;
                    tc_fence_after();
                    uint64_t ad = umma_desc_sw128(smem_u32(sA + s * A_BYTES));
                    uint64_t bd = umma_desc_sw128(smem_u32(sB + s * B_BYTES));
                    if (X3) {
                        uint64_t al = umma_desc_sw128(smem_u32(sA + s * A_BYTES + A_TILE));
                        uint64_t bl = umma_desc_sw128(smem_u32(sB + s * B_BYTES + B_TILE));
#pragma unroll
                        for (int k = 0; k < TC_BK / 8; k++) {
                            umma_tf32(tacc, al + (uint64_t)(k * 2), bd + (uint64_t)(k * 2), idesc, (kb | k) ? 1u : 0u);
                            umma_tf32(tacc, ad + (uint64_t)(k * 2), bl + (uint64_t)(k * 2), idesc, 1u);
                        }
                    }
#pragma unroll
                    for (int k = 0; k < TC_BK / 8; k++)      // 8 tf32 (32 bytes) per MMA: advance the start address
                        umma_tf32(tacc, ad + (uint64_t)(k * 2), bd + (uint64_t)(k * 2), idesc, (X3 || (kb | k)) ? 1u : 0u);
                    umma_commit(empty0 + 8 * s);             // stage reusable once these MMAs have read it
                }
                umma_commit(afull0 + 8 * acc);               // accumulator complete (also reached on the error path)
            }
        }
    } else {
        const int q = warp & 3;                              // TMEM lane quadrant this warp may read
        int it = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, it++) {
            const int acc = it & 1; const uint32_t use = (uint32_t)(it >> 1);
            const int n0 = (t % tiles_n) * BN;
            const int64_t m = (int64_t)(t / tiles_n) * TC_BM + q * 32 + lane;
            ok = mbar_wait(afull0 + 8 * acc, use & 1u, ep.err, 3);
            tc_fence_after();
            if (!ok) break;
            float bestd = INFINITY; int bestn = 0x7fffffff;
            if (ep.best) {
                // Nearest row. The tile has one k-block (K = 64 for the codebook search), so this loop is the kernel:
                // the next 32 columns are on their way out of tensor memory while these are compared, the column
                // norms come as float4, and four independent running minima (columns j mod 4) break the
                // compare-select chain; they merge at the end by (distance, index), which keeps the first minimum.
                const uint32_t trow = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
                float bd[4] = {INFINITY, INFINITY, INFINITY, INFINITY};
                int bn[4] = {0x7fffffff, 0x7fffffff, 0x7fffffff, 0x7fffffff};
                uint32_t ra[32], rb[32];
                tmem_ld32_issue(trow, ra);
                tmem_ld_wait();
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 64) {
                    if (c0 + 32 < BN) tmem_ld32_issue(trow + (uint32_t)(c0 + 32), rb);
                    {
                        const int nb = n0 + c0;
                        if (nb + 32 <= ep.N) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                const float4 cn = *(const float4 *)(ep.colnorm + nb + j);
                                const float cc[4] = {cn.x, cn.y, cn.z, cn.w};
#pragma unroll
                                for (int e = 0; e < 4; e++) {
                                    const float d = fmaf(-2.0f, __uint_as_float(ra[j + e]), cc[e]);
                                    if (d < bd[e]) { bd[e] = d; bn[e] = nb + j + e; }
                                }
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++) {
                                const int n = nb + j;
                                if (n < ep.N) {
                                    const float d = fmaf(-2.0f, __uint_as_float(ra[j]), ep.colnorm[n]);
                                    if (d < bd[j & 3]) { bd[j & 3] = d; bn[j & 3] = n; }
                                }
                            }
                        }
                    }
                    tmem_ld_wait();
                    if (c0 + 64 < BN) tmem_ld32_issue(trow + (uint32_t)(c0 + 64), ra);
                    if (c0 + 32 < BN) {
                        const int nb = n0 + c0 + 32;
                        if (nb + 32 <= ep.N) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                const float4 cn = *(const float4 *)(ep.colnorm + nb + j);
                                const float cc[4] = {cn.x, cn.y, cn.z, cn.w};
#pragma unroll
                                for (int e = 0; e < 4; e++) {
                                    const float d = fmaf(-2.0f, __uint_as_float(rb[j + e]), cc[e]);
                                    if (d < bd[e]) { bd[e] = d; bn[e] = nb + j + e; }
                                }
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++) {
                                const int n = nb + j;
                                if (n < ep.N) {
                                    const float d = fmaf(-2.0f, __uint_as_float(rb[j]), ep.colnorm[n]);
                                    if (d < bd[j & 3]) { bd[j & 3] = d; bn[j & 3] = n; }
                                }
                            }
                        }
                    }
                    tmem_ld_wait();
                }
#pragma unroll
                for (int e = 0; e < 4; e++)
                    if (bd[e] < bestd || (bd[e] == bestd && bn[e] < bestn)) { bestd = bd[e]; bestn = bn[e]; }
            } else {
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c0), r);
                    tc_epilogue_chunk(ep, r, m, n0, c0);
                }
            }
            if (ep.best && m < ep.M && bestn != 0x7fffffff) {
                unsigned u = __float_as_uint(bestd);
                u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);           // order-preserving float -> uint
                atomicMin(ep.best + m, ((unsigned long long)u << 32) | (unsigned)bestn);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(aempty0 + 8 * acc);   // 4 arrivals (one per epilogue warp) free the accumulator
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN) : "memory");
    }
}

// ------------------------------------------------------------------ host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
        if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) fatal("cuTensorMapEncodeTiled is not available in this driver");
        fn = (EncodeTiledFn)p;
    }
    return fn;
}

struct MapKey {
    const void *p; int64_t rows, ld; int K, box_rows, dtype;
    bool operator==(const MapKey &o) const { return p == o.p && rows == o.rows && ld == o.ld && K == o.K && box_rows == o.box_rows && dtype == o.dtype; }
};
struct MapKeyHash {
    size_t operator()(const MapKey &k) const {
        size_t h = (size_t)(uintptr_t)k.p;
        h = h * 1000003u ^ (size_t)k.rows; h = h * 1000003u ^ (size_t)k.ld; h = h * 1000003u ^ (size_t)k.K;
        return h * 1000003u ^ (size_t)(k.box_rows * 4 + k.dtype);
    }
};

// Entries the tensor-map caches hold before they start over (ncmb_set_map_cache_limit; tests set it to 1 so that
// every lookup of one launch evicts the previous one).
static size_t g_map_cache_limit = 4096;
static size_t tc_map_cache_limit() { return g_map_cache_limit; }

static int tma_dtype_mode() {          // 1 (default): TMA rounds fp32 to tf32 while loading; 0: raw fp32 bits
    static int m = -1;
    if (m < 0) { const char *e = getenv("NCM_B200_TMA_TF32"); m = e ? atoi(e) : 1; }
    return m;
}

// 2-D map over a row-major [rows][K] fp32 matrix with row stride ld: box = 32 floats x box_rows.
// round_tf32: let the TMA unit round each element to TF32 on the way into shared memory.
// Returned by value: the cache may evict entries on a later lookup, so callers that fetch several maps for one
// launch never hold pointers into it.
CUtensorMap tc_get_map(const float *p, int64_t rows, int K, int64_t ld, int box_rows, bool round_tf32) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    int dt = (round_tf32 && tma_dtype_mode()) ? 1 : 0;
    MapKey key{p, rows, ld, K, box_rows, dt};
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
    if (cache.size() > tc_map_cache_limit()) cache.clear();
    CUtensorMap tm;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
    cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode_fn()(&tm, dt ? CU_TENSOR_MAP_DATA_TYPE_TFLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                             (void *)p, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) fatal("cuTensorMapEncodeTiled failed (%d) for [%lld][%d] ld %lld", (int)r, (long long)rows, K, (long long)ld);
    cache.emplace(key, tm);
    return tm;
}

// 2-D map over a row-major [rows][K] fp16 matrix with row stride ld (elements): box = 64 halfs x box_rows
CUtensorMap tc_get_map_h16(const void *p, int64_t rows, int K, int64_t ld, int box_rows) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    MapKey key{p, rows, ld, K, box_rows, 2};
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
    if (cache.size() > tc_map_cache_limit()) cache.clear();
    CUtensorMap tm;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode_fn()(&tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void *)p, dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) fatal("cuTensorMapEncodeTiled (fp16) failed (%d) for [%lld][%d] ld %lld", (int)r, (long long)rows, K, (long long)ld);
    cache.emplace(key, tm);
    return tm;
}

} // namespace ncmb
extern "C" void ncmb_set_map_cache_limit(int entries) { ncmb::g_map_cache_limit = entries < 1 ? 1 : (size_t)entries; }
namespace ncmb {

int *tc_err_flag() {
    static int *d = nullptr;
    if (!d) { d = (int *)dev_alloc(sizeof(int)); CUDA_CHECK(cudaMemsetAsync(d, 0, sizeof(int), stream())); }
    return d;
}

// reads and clears the device-side error word of the tensor-core engine (0 = no timeout seen)
int gemm_tc_check() {
    int v = 0;
    int *d = tc_err_flag();
    CUDA_CHECK(cudaMemcpyAsync(&v, d, sizeof(int), cudaMemcpyDeviceToHost, stream()));
    CUDA_CHECK(cudaStreamSynchronize(stream()));
    if (v) CUDA_CHECK(cudaMemsetAsync(d, 0, sizeof(int), stream()));
    return v;
}

// ---- hi / lo split for the three-pass mode: hi = rn_tf32(x), lo = x - hi (exact in fp32) ----
__global__ void k_split_tf32(const float *__restrict__ x, int64_t ldx, float *__restrict__ hi, float *__restrict__ lo,
                             int64_t rows, int K4) {
    int64_t total = rows * K4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t r = i / K4; int c = (int)(i % K4);
        float4 v = *(const float4 *)(x + r * ldx + c * 4);
        float4 h, l;
        uint32_t u;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v.x)); h.x = __uint_as_float(u); l.x = v.x - h.x;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v.y)); h.y = __uint_as_float(u); l.y = v.y - h.y;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v.z)); h.z = __uint_as_float(u); l.z = v.z - h.z;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v.w)); h.w = __uint_as_float(u); l.w = v.w - h.w;
        *(float4 *)(hi + i * 4) = h;
        *(float4 *)(lo + i * 4) = l;
    }
}
static void split_tf32(const float *x, int64_t ldx, float *hi, float *lo, int64_t rows, int K) {
    int64_t n = rows * (K / 4);
    int64_t g = cdiv(n, 256), cap = (int64_t)ctx().sm_count * 16;
    ProfScope ps(NCMB_K_ELEM, 0, (double)rows * K * 12);
    LAUNCH(k_split_tf32, (unsigned)(g > cap ? cap : (g < 1 ? 1 : g)), 256, 0, x, ldx, hi, lo, rows, K / 4);
}

struct Shadow { float *hi, *lo; int64_t n; };
static std::unordered_map<const float *, Shadow> &shadow_cache() { static std::unordered_map<const float *, Shadow> c; return c; }
static Workspace &split_ws() { static Workspace w; return w; }

// Drops the cached hi/lo copies of weights (call when weight memory is freed or rewritten).
void gemm_tc_forget_weights() {
    for (auto &kv : shadow_cache()) { dev_free(kv.second.hi); }
    shadow_cache().clear();
}

void gemm_tc_forget_range(const void *p, size_t bytes) {
    auto &sc = shadow_cache();
    const char *lo = (const char *)p, *hi = lo + bytes;
    for (auto it = sc.begin(); it != sc.end();) {
        const char *w0 = (const char *)it->first, *w1 = w0 + (size_t)it->second.n * 4;
        if (w0 < hi && lo < w1) { CUDA_CHECK(cudaStreamSynchronize(stream())); dev_free(it->second.hi); it = sc.erase(it); }
        else ++it;
    }
}

static inline bool al16(const void *p) { return ((uintptr_t)p & 15) == 0; }

bool gemm_tc_supported(const GemmArgs &a) {
    int64_t ldx = a.ldx ? a.ldx : a.K, ldy = a.ldy ? a.ldy : (a.glu ? a.N / 2 : a.N);
    if (a.M <= 16 || a.N < 32 || a.K < 32) return false;           // up to 16 rows: the weight-streaming GEMV kernel
    if ((a.K & 3) || (ldx & 3)) return false;                       // TMA strides: multiples of 16 bytes
    if (!al16(a.x) || !al16(a.W) || (!a.argmin_best && !al16(a.y)) || (a.bias && !al16(a.bias)) || (a.res && !al16(a.res))) return false;
    if (a.glu && ((a.N & 1) || (ldy & 1))) return false;
    return true;
}

template <int BN, int STAGES, bool X3>
static void launch_tc(const GemmArgs &a, const TcEpi &ep, const CUtensorMap *ma, const CUtensorMap *mb,
                      const CUtensorMap *mal, const CUtensorMap *mbl) {
    constexpr size_t smem = 1024 + (size_t)STAGES * (TC_BM + BN) * TC_BK * 4 * (X3 ? 2 : 1) + (2 * STAGES + 4) * 8 + 16;
    static_assert(smem <= 227 * 1024, "stage ring exceeds shared memory");
    static bool set = false;
    if (!set) {
        CUDA_CHECK(cudaFuncSetAttribute((k_gemm_tc<BN, STAGES, X3>), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        set = true;
    }
    int tiles_n = (int)cdiv(a.N, BN);
    int64_t tiles = (int64_t)tiles_n * cdiv(a.M, TC_BM);
    if (tiles > 0x7fffffff) fatal("gemm_tc: too many tiles");
    int grid = (int)(tiles < ctx().sm_count ? tiles : ctx().sm_count);     // persistent: one CTA per SM
    int num_kb = (int)cdiv(a.K, TC_BK);
    LAUNCH((k_gemm_tc<BN, STAGES, X3>), grid, TC_THREADS, smem, *ma, *mb, *mal, *mbl, ep, num_kb, tiles_n, (int)tiles);
}

void gemm_tc(const GemmArgs &a) {
    if (a.M <= 0 || a.N <= 0) return;
    TcEpi ep{};
    ep.bias = a.bias; ep.res = a.res; ep.ldres = a.ldres ? a.ldres : a.N;
    ep.y = a.y; ep.y_lo = a.y_lo; ep.y_fmt = a.y_fmt; ep.ldy = a.ldy ? a.ldy : (a.glu ? a.N / 2 : a.N);
    ep.M = a.M; ep.N = a.N; ep.act = a.act; ep.glu = a.glu; ep.err = tc_err_flag();
    ep.colnorm = a.argmin_colnorm; ep.best = a.argmin_best; ep.tma_store = 0;
    int64_t ldx = a.ldx ? a.ldx : a.K;
    const bool x3 = ctx().gemm_mode >= 2;
    if (!x3) {
        const CUtensorMap ma = tc_get_map(a.x, a.M, a.K, ldx, TC_BM, true);
        const CUtensorMap mb = tc_get_map(a.W, a.N, a.K, a.K, 128, true);
        ProfScope ps(NCMB_K_GEMM, 2.0 * (double)a.M * a.N * a.K,
                     4.0 * ((double)a.M * a.K + (double)a.N * a.K + (double)a.M * a.N));
        launch_tc<128, 6, false>(a, ep, &ma, &mb, &ma, &mb);
        return;
    }
    // three-pass mode: split both operands; static weights are split once and cached
    const bool pre_split = a.x_lo != nullptr;
    const int64_t nx = pre_split ? 0 : a.M * a.K, nw = (int64_t)a.N * a.K;
    float *whi, *wlo;
    Workspace &ws = split_ws();
    bool cache_w = ctx().w_static != 0;
    size_t need = (size_t)(2 * nx + (cache_w ? 0 : 2 * nw)) * 4 + 4096;
    if (need > ws.cap) ws.reserve(need + need / 4);
    ws.reset();
    const float *xhi = a.x, *xlo = a.x_lo;
    int64_t ldsplit = ldx;
    if (!pre_split) {
        float *h = ws.get<float>(nx), *l = ws.get<float>(nx);
        xhi = h; xlo = l; ldsplit = a.K;
    }
    if (cache_w) {
        auto &sc = shadow_cache();
        auto it = sc.find(a.W);
        if (it == sc.end() || it->second.n != nw) {
            if (it != sc.end()) dev_free(it->second.hi);
            float *buf = (float *)dev_alloc((size_t)2 * nw * 4);
            split_tf32(a.W, a.K, buf, buf + nw, a.N, a.K);
            it = sc.insert_or_assign(a.W, Shadow{buf, buf + nw, nw}).first;
        }
        whi = it->second.hi; wlo = it->second.lo;
    } else {
        whi = ws.get<float>(nw); wlo = ws.get<float>(nw);
        split_tf32(a.W, a.K, whi, wlo, a.N, a.K);
    }
    if (!pre_split) split_tf32(a.x, ldx, (float *)xhi, (float *)xlo, a.M, a.K);
    const CUtensorMap ma = tc_get_map(xhi, a.M, a.K, ldsplit, TC_BM, false), mal = tc_get_map(xlo, a.M, a.K, ldsplit, TC_BM, true);
    // 256-wide N tiles read a third less of the operands per MMA flop (from L2 and from shared memory);
    // they are used once the launch still fills every SM a few times over
    static const bool wide_ok = !getenv("NCM_B200_NO_BN256");
    const bool wide = wide_ok && a.N >= 256 && cdiv(a.N, 256) * cdiv(a.M, TC_BM) >= 2 * (int64_t)ctx().sm_count;
    const int bn = wide ? 256 : 128;
    const CUtensorMap mb = tc_get_map(whi, a.N, a.K, a.K, bn, false), mbl = tc_get_map(wlo, a.N, a.K, a.K, bn, true);
    ProfScope ps(NCMB_K_GEMM, 2.0 * (double)a.M * a.N * a.K,
                 4.0 * (2.0 * (double)a.M * a.K + 2.0 * (double)a.N * a.K + (double)a.M * a.N));
    if (wide) launch_tc<256, 2, true>(a, ep, &ma, &mb, &mal, &mbl);
    else launch_tc<128, 3, true>(a, ep, &ma, &mb, &mal, &mbl);
}


// ------------------------------------------------------------------ linear layer without any allocation
// The three-pass GEMM needs scratch for the hi/lo halves of both operands. linear_fwd
// takes it from a workspace that grows with cudaMalloc; the entry point below takes it
// from a fixed array that is part of the loaded module instead, so it can be called
// from places where allocating device memory is off the table.
constexpr size_t NOALLOC_SCRATCH_FLOATS = (size_t)8 << 20;           // 32 MiB, resident on every GPU that loads the library
static __device__ __align__(256) float g_noalloc_scratch[NOALLOC_SCRATCH_FLOATS];
static __device__ int g_noalloc_err;
static float *g_noalloc_scratch_of[64] = {nullptr};      // device addresses of the two symbols, per device ordinal
static int *g_noalloc_err_of[64] = {nullptr};

static void encode_map_now(CUtensorMap *tm, const float *p, int64_t rows, int K, int64_t ld, int box_rows, bool round_tf32) {
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
    cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    bool rt = round_tf32 && tma_dtype_mode();
    CUresult r = encode_fn()(tm, rt ? CU_TENSOR_MAP_DATA_TYPE_TFLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void *)p, dims,
                             strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) fatal("cuTensorMapEncodeTiled failed (%d)", (int)r);
}

} // namespace ncmb

// y = x W^T + b like linear_fwd (three-pass TF32, fp32-grade), allocating nothing:
// no cudaMalloc / cudaFree and no allocating library call on any path.
//
// Who needs this: code that runs where device allocation is not allowed or not
// safe -- a serving loop whose memory budget is fixed up front, a host callback or
// a region under stream capture (cudaMalloc is illegal there), or a process that
// shares the GPU and must never fail or stall on an allocation in steady state.
//
// Scratch: the split operands (2*batch*K + 2*M*K floats) live in a 32 MiB array
// compiled into the library. Sizes beyond it (or shapes the tensor-core kernel does
// not take: batch <= 16, M < 32, K < 32, K % 4 != 0, pointers not 16-byte aligned)
// are refused with -1 and a message; nothing is launched then. Returns 0 once the
// kernels are queued; whether a bounded wait inside them ran out is only known after
// ncmb_linear_fwd_noalloc_check(), which synchronises and reads the kernel's status word.
// The library keeps its per-process state (SM count, kernel attributes) for the device
// that was current at its first call; a call with another device current is refused.
// The first call on each device looks up the array's device address and clears its
// error word; make that first call outside any stream capture. Every call reuses
// the same array and overwrites all of the part it reads, so earlier contents never
// leak into a result -- but two calls running concurrently on one GPU (different
// streams, or different threads) would race on it: keep calls ordered on one stream.
extern "C" int ncmb_linear_fwd_noalloc(const float *x, const float *W, const float *b, float *y,
                                       int64_t batch, int M, int K) {
    using namespace ncmb;
    ensure_device();
    float **scratch_of = g_noalloc_scratch_of;
    int **err_of = g_noalloc_err_of;
    int dev = 0;
    CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) { fprintf(stderr, "ncmb_linear_fwd_noalloc: device index %d out of range\n", dev); return -1; }
    if (dev != ctx().device) {
        fprintf(stderr, "ncmb_linear_fwd_noalloc: device %d is current but the library was set up on device %d\n", dev, ctx().device);
        return -1;
    }
    if (!scratch_of[dev]) {
        // set-up, once per device, with that device current: the symbol name is only a
        // host-side handle; kernels must be given the address it resolves to on the device
        float *sp = nullptr; int *ep = nullptr;
        cudaError_t e1 = cudaGetSymbolAddress((void **)&sp, g_noalloc_scratch);
        cudaError_t e2 = cudaGetSymbolAddress((void **)&ep, g_noalloc_err);
        if (e1 != cudaSuccess || e2 != cudaSuccess || !sp || !ep) {
            fprintf(stderr, "ncmb_linear_fwd_noalloc: cudaGetSymbolAddress failed: %s\n",
                    cudaGetErrorString(e1 != cudaSuccess ? e1 : e2));
            return -1;
        }
        CUDA_CHECK(cudaMemsetAsync(ep, 0, sizeof(int), stream()));
        scratch_of[dev] = sp; err_of[dev] = ep;
    }
    GemmArgs a;
    a.x = x; a.ldx = K; a.W = W; a.bias = b; a.y = y; a.ldy = M; a.M = batch; a.N = M; a.K = K;
    if (!gemm_tc_supported(a)) {
        fprintf(stderr, "ncmb_linear_fwd_noalloc: shape [%lld x %d] * [%d x %d] not taken by the tensor-core kernel "
                        "(need batch > 16, M >= 32, K >= 32, K %% 4 == 0, 16-byte aligned pointers)\n",
                (long long)batch, K, M, K);
        return -1;
    }
    const size_t nx = (size_t)batch * K, nw = (size_t)M * K;
    if (2 * nx + 2 * nw > NOALLOC_SCRATCH_FLOATS) {
        fprintf(stderr, "ncmb_linear_fwd_noalloc: needs %zu scratch floats (2*batch*K + 2*M*K), the built-in array holds %zu\n",
                2 * nx + 2 * nw, NOALLOC_SCRATCH_FLOATS);
        return -1;
    }
    float *xhi = scratch_of[dev], *xlo = xhi + nx, *whi = xlo + nx, *wlo = whi + nw;
    split_tf32(x, K, xhi, xlo, batch, K);
    split_tf32(W, K, whi, wlo, M, K);
    CUtensorMap ma, mal, mb, mbl;
    encode_map_now(&ma, xhi, batch, K, K, TC_BM, false); encode_map_now(&mal, xlo, batch, K, K, TC_BM, true);
    encode_map_now(&mb, whi, M, K, K, 128, false); encode_map_now(&mbl, wlo, M, K, K, 128, true);
    TcEpi ep{};
    ep.bias = b; ep.res = nullptr; ep.ldres = M; ep.y = y; ep.y_lo = nullptr; ep.y_fmt = SPLIT_TF32; ep.tma_store = 0; ep.ldy = M; ep.colnorm = nullptr; ep.best = nullptr; ep.M = batch; ep.N = M; ep.act = ACT_NONE; ep.glu = 0;
    ep.err = err_of[dev];
    launch_tc<128, 3, true>(a, ep, &ma, &mb, &mal, &mbl);
    return 0;
}

// Status of the allocation-free entry point on the current device: waits for the stream, then returns and clears the
// word its kernels write when a bounded barrier wait runs out (0 = every call so far completed; -1 = the entry point
// has not been set up on this device). Allocates nothing: a 4-byte copy through the address looked up at set-up.
extern "C" int ncmb_linear_fwd_noalloc_check(void) {
    using namespace ncmb;
    ensure_device();
    int dev = 0;
    CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !g_noalloc_err_of[dev]) return -1;
    int v = 0;
    CUDA_CHECK(cudaMemcpyAsync(&v, g_noalloc_err_of[dev], sizeof(int), cudaMemcpyDeviceToHost, stream()));
    CUDA_CHECK(cudaStreamSynchronize(stream()));
    if (v) CUDA_CHECK(cudaMemsetAsync(g_noalloc_err_of[dev], 0, sizeof(int), stream()));
    return v;
}
