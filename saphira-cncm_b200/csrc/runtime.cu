// Runtime of libncm_b200.so: device context, tensors, arenas, NCM1 weight files,
// .conf parsing, kernel-class timers. Replaces the reference's src/tensor.c for a
// B200 build: weights live in one HBM slab per file instead of one cudaMalloc per
// tensor, and every copy goes through the library's stream.
#include "common.cuh"

#include <algorithm>
#include <map>
#include <string>
#include <tuple>

#include <stdarg.h>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace ncmb {

void fatal(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    fprintf(stderr, "[ncm_b200] fatal: ");
    vfprintf(stderr, fmt, ap);
    fprintf(stderr, "\n");
    va_end(ap);
    exit(1);
}

Ctx &ctx() {
    static Ctx c;
    return c;
}

void ensure_device() {
    Ctx &c = ctx();
    if (c.inited) return;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0)
        fatal("no CUDA device: this library has no CPU path (%s)",
              e != cudaSuccess ? cudaGetErrorString(e) : "device count 0");
    int dev = 0;
    CUDA_CHECK(cudaGetDevice(&dev));
    cudaDeviceProp p;
    CUDA_CHECK(cudaGetDeviceProperties(&p, dev));
    if (p.major < 10)
        fatal("device %s is sm_%d%d; this build targets sm_100a only", p.name, p.major, p.minor);
    c.sm_count = p.multiProcessorCount;
    c.device = dev;
    const char *gm = getenv("NCM_B200_GEMM");
    if (gm) c.gemm_mode = atoi(gm);
    const char *rm = getenv("NCM_B200_RNG");
    if (rm) c.rng_mode = atoi(rm);
    c.inited = true;
}

// ------------------------------------------------------------------ profiler
struct ProfRec { int klass; double flops, bytes; cudaEvent_t a, b; };
struct Prof {
    bool on = false;
    std::vector<cudaEvent_t> pool;
    std::vector<ProfRec> open;
    ProfRec cur; bool in_scope = false; int depth = 0;
    long long launches[NCMB_K_COUNT] = {0};
    double ms[NCMB_K_COUNT] = {0}, flops[NCMB_K_COUNT] = {0}, bytes[NCMB_K_COUNT] = {0};
    // one entry per distinct (class, flops, bytes) scope, i.e. per call shape
    std::map<std::tuple<int, double, double>, std::pair<long long, double>> shapes;
    bool by_shape = true;
    cudaEvent_t get() {
        if (!pool.empty()) { cudaEvent_t e = pool.back(); pool.pop_back(); return e; }
        cudaEvent_t e;
        CUDA_CHECK(cudaEventCreate(&e));
        return e;
    }
    void drain() {
        if (open.empty()) return;
        CUDA_CHECK(cudaEventSynchronize(open.back().b));
        for (auto &r : open) {
            float t = 0;
            CUDA_CHECK(cudaEventElapsedTime(&t, r.a, r.b));
            ms[r.klass] += t; flops[r.klass] += r.flops; bytes[r.klass] += r.bytes; launches[r.klass]++;
            if (by_shape) { auto &e = shapes[std::make_tuple(r.klass, r.flops, r.bytes)]; e.first++; e.second += t; }
            pool.push_back(r.a); pool.push_back(r.b);
        }
        open.clear();
    }
};
static Prof &prof() { static Prof p; return p; }

void prof_begin(int klass, double flops, double bytes) {
    Prof &p = prof();
    if (!p.on) return;
    if (p.depth++ > 0) return;               // nested scopes fold into the outermost one
    p.cur = ProfRec{klass, flops, bytes, p.get(), p.get()};
    CUDA_CHECK(cudaEventRecord(p.cur.a, stream()));
}
bool prof_enabled() { return prof().on; }
void prof_end() {
    Prof &p = prof();
    if (!p.on) return;
    if (--p.depth > 0) return;
    CUDA_CHECK(cudaEventRecord(p.cur.b, stream()));
    p.open.push_back(p.cur);
    if (p.open.size() >= 8192) p.drain();
}

// ------------------------------------------------------------------ workspace
void Workspace::reserve(size_t bytes) {
    if (bytes <= cap) return;
    ensure_device();
    if (base) { CUDA_CHECK(cudaStreamSynchronize(stream())); CUDA_CHECK(cudaFree(base)); }
    cudaError_t e = cudaMalloc((void **)&base, bytes);
    if (e != cudaSuccess) fatal("workspace of %.1f MB: %s", bytes / 1048576.0, cudaGetErrorString(e));
    cap = bytes; off = 0;
}
void *Workspace::alloc(size_t bytes) {
    off = (off + 255) & ~(size_t)255;
    if (measuring) { void *fake = (void *)(uintptr_t)(4096 + off); off += bytes; return fake; }
    if (off + bytes > cap) fatal("workspace overflow: need %zu of %zu bytes", off + bytes, cap);
    void *p = base + off;
    off += bytes;
    return p;
}
void Workspace::release() {
    if (base) { cudaStreamSynchronize(stream()); cudaFree(base); }
    base = nullptr; cap = off = 0;
}

} // namespace ncmb

using namespace ncmb;

// weight slabs: Tensor.data pointers that live inside a slab are not cudaFree'd one by one
static std::unordered_set<const void *> &slab_members() { static std::unordered_set<const void *> s; return s; }
static std::unordered_map<const void *, void *> &slab_of_store() { static std::unordered_map<const void *, void *> s; return s; }

extern "C" {

// ------------------------------------------------------------------ tensors
int64_t tensor_numel(int ndim, const int64_t *shape) {
    int64_t n = 1;
    for (int i = 0; i < ndim; i++) n *= shape[i];
    return n;
}

Tensor *tensor_alloc(int ndim, const int64_t *shape) {
    ensure_device();
    Tensor *t = (Tensor *)calloc(1, sizeof(Tensor));
    if (!t) fatal("oom tensor");
    t->ndim = ndim;
    for (int i = 0; i < ndim; i++) t->shape[i] = shape[i];
    t->n = tensor_numel(ndim, shape);
    CUDA_CHECK(cudaMalloc((void **)&t->data, (size_t)(t->n > 0 ? t->n : 1) * sizeof(float)));
    return t;
}

// memory that is rewritten or freed through the public functions no longer backs any cached weight copy
static void forget_copies_of(const void *p, size_t bytes) {
    gemm_h3_forget_range(p, bytes);
    gemm_tc_forget_range(p, bytes);
}

void tensor_free(Tensor *t) {
    if (!t) return;
    forget_copies_of(t->data, (size_t)(t->n > 0 ? t->n : 1) * sizeof(float));
    if (!slab_members().count(t->data)) {
        cudaStreamSynchronize(stream());
        cudaFree(t->data);
    }
    free(t);
}

void mem_d2h(void *h, const void *d, size_t n) {
    ensure_device();
    CUDA_CHECK(cudaMemcpyAsync(h, d, n, cudaMemcpyDeviceToHost, stream()));
    CUDA_CHECK(cudaStreamSynchronize(stream()));
    ctx().d2h_bytes += n;
}
void mem_h2d(void *d, const void *h, size_t n) {
    ensure_device();
    forget_copies_of(d, n);
    CUDA_CHECK(cudaMemcpyAsync(d, h, n, cudaMemcpyHostToDevice, stream()));
    CUDA_CHECK(cudaStreamSynchronize(stream()));   // h may be freed by the caller right after
    ctx().h2d_bytes += n;
}
void mem_d2d(void *d, const void *s, size_t n) {
    ensure_device();
    forget_copies_of(d, n);
    CUDA_CHECK(cudaMemcpyAsync(d, s, n, cudaMemcpyDeviceToDevice, stream()));
}
void tensor_to_host(const Tensor *t, float *out) { mem_d2h(out, t->data, (size_t)t->n * sizeof(float)); }
void tensor_to_backend(Tensor *t, const float *in) { mem_h2d(t->data, in, (size_t)t->n * sizeof(float)); }

void *backend_to_host(const float *d, size_t nbytes) {
    void *h = malloc(nbytes ? nbytes : 1);
    if (!h) fatal("oom host copy");
    mem_d2h(h, d, nbytes);
    return h;
}

// ------------------------------------------------------------------ arenas
static unsigned char *arena_base = nullptr, *parena_base = nullptr;
static size_t arena_size = 0, arena_off = 0, parena_size = 0, parena_off = 0;

void arena_free(void) {
    if (!arena_base) return;
    cudaStreamSynchronize(stream());
    cudaFree(arena_base);
    arena_base = nullptr; arena_size = arena_off = 0;
}
void arena_init(size_t bytes) {
    ensure_device();
    arena_free();
    cudaError_t e = cudaMalloc((void **)&arena_base, bytes);
    if (e != cudaSuccess) fatal("arena of %zu MB: %s", bytes >> 20, cudaGetErrorString(e));
    arena_size = bytes; arena_off = 0;
}
void arena_init_default(void) {
    const char *e = getenv("NCM_ARENA_MB");
    size_t mb = e ? (size_t)atol(e) : 4096;
    if (mb < 64) mb = 64;
    arena_init(mb << 20);
}
float *arena_alloc(size_t n_floats) {
    size_t need = n_floats * sizeof(float);
    arena_off = (arena_off + 255) & ~(size_t)255;
    if (!arena_base || arena_off + need > arena_size) {
        fprintf(stderr, "arena overflow (%zu > %zu MB); raise NCM_ARENA_MB\n", arena_off + need, arena_size >> 20);
        exit(1);
    }
    float *p = (float *)(arena_base + arena_off);
    arena_off += need;
    return p;
}
void arena_reset(void) { arena_off = 0; }

void parena_init(size_t bytes) {
    if (parena_base) return;
    ensure_device();
    CUDA_CHECK(cudaMalloc((void **)&parena_base, bytes));
    parena_size = bytes; parena_off = 0;
}
float *parena_alloc(size_t n_floats) {
    size_t need = n_floats * sizeof(float);
    parena_off = (parena_off + 255) & ~(size_t)255;
    if (!parena_base || parena_off + need > parena_size) {
        fprintf(stderr, "parena overflow (%zu > %zu)\n", parena_off + need, parena_size);
        exit(1);
    }
    float *p = (float *)(parena_base + parena_off);
    parena_off += need;
    return p;
}

// ------------------------------------------------------------------ NCM1 weight files
// Layout (reference loader, src/tensor.c:70-128): "NCM1", u32 count, then per tensor
// u8 name length, name, u8 ndim, u32 dims, u64 byte count, raw fp32. The whole file is
// read once; all tensor payloads go into one 256-byte-aligned HBM slab with one copy.
// ---- weight files -----------------------------------------------------------------------------
// NCM1 (reference weights_load src/tensor.c:70-130): "NCM1", u32 count, then per tensor u8 name length, name,
// u8 ndim, u32 dims, u64 payload bytes, fp32 payload. NCK1 training checkpoints (reference src/ckpt.c:200-262)
// hold the same per-tensor records after a run-state header and before the optimizer section, with an FNV-1a 64
// checksum of everything in the last eight bytes; like the reference (ckpt_load_weights_only src/ckpt.c:549-625,
// reached from weights_load src/tensor.c:73-80) only the tensor records are read. The file is staged once in
// pinned memory and every payload goes to one device slab.

// bf16 bits -> fp32 (exact): the payload of a 2-byte tensor record widened into the fp32 slab
__global__ void k_widen_bf16(const unsigned short *__restrict__ src, float *__restrict__ dst, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        dst[i] = __uint_as_float((uint32_t)src[i] << 16);
}
// stores whose matrices all came from 2-byte records (every 2-D or larger tensor holds bf16 values only)
static std::unordered_set<const void *> &bf16_stores() { static std::unordered_set<const void *> s; return s; }

namespace {
struct FileImage {
    unsigned char *buf = nullptr;
    size_t len = 0;
    ~FileImage() { if (buf) { memset(buf, 0, len); cudaFreeHost(buf); } }      // weights do not linger in host memory
};

int read_image(const char *path, FileImage &im, char *err, size_t errcap) {
    FILE *f = fopen(path, "rb");
    if (!f) { snprintf(err, errcap, "cannot open %s", path); return -1; }
    fseek(f, 0, SEEK_END);
    long fsz = ftell(f);
    fseek(f, 0, SEEK_SET);
    if (fsz < 8) { snprintf(err, errcap, "%s: bad magic", path); fclose(f); return -1; }
    if (cudaMallocHost((void **)&im.buf, (size_t)fsz) != cudaSuccess) { fclose(f); im.buf = nullptr; snprintf(err, errcap, "%s: pinned staging alloc failed", path); return -1; }
    im.len = (size_t)fsz;
    size_t got = fread(im.buf, 1, im.len, f);
    fclose(f);
    if (got != im.len) { snprintf(err, errcap, "%s: short read", path); return -1; }
    return 0;
}

// tensor records [pos, end) of a staged file -> ws (one device slab). strict: NCK1 rules (no empty names).
int load_tensor_records(WeightStore *ws, const char *path, const FileImage &im, size_t pos, size_t end, uint32_t count, bool strict,
                        char *err, size_t errcap, bool typed = false) {
    const unsigned char *buf = im.buf;
    // every record takes at least 10 bytes (name length, ndim, byte count): a count the file cannot hold is refused
    // before anything is allocated
    if (count > (1u << 24) || (uint64_t)count * 10 > (uint64_t)(end - pos)) { snprintf(err, errcap, "%s: bad tensor count", path); return -1; }
    ws->items = (NamedTensor *)calloc(count ? count : 1, sizeof(NamedTensor));
    ws->count = 0;
    if (!ws->items) { snprintf(err, errcap, "out of memory"); return -1; }
    auto fail = [&](const char *why) {
        if (!err[0]) snprintf(err, errcap, "%s: %s", path, why);
        for (int j = 0; j < ws->count; j++) free(ws->items[j].t);
        free(ws->items); ws->items = nullptr; ws->count = 0;
        return -1;
    };
    struct Span { size_t file_off, nbytes, slab_off; int dtype; };
    std::vector<Span> spans(count);
    size_t slab = 0, max16 = 0;
    bool all_matrices_16 = typed;
    const char *trunc = strict ? "truncated tensor section" : "truncated";
    for (uint32_t i = 0; i < count; i++) {
        if (pos + 1 > end) return fail(trunc);
        unsigned nl = buf[pos++];
        if ((strict && nl == 0) || nl >= sizeof(ws->items[0].name) || pos + nl + 1 > end) return fail(trunc);
        memcpy(ws->items[i].name, buf + pos, nl);
        ws->items[i].name[nl] = 0;
        pos += nl;
        unsigned nd = buf[pos++];
        if (nd > NCM_MAX_DIMS || pos + 4 * nd + 8 > end) return fail(trunc);
        Tensor *t = (Tensor *)calloc(1, sizeof(Tensor));
        t->ndim = (int)nd; t->n = 1;
        for (unsigned d = 0; d < nd; d++) { uint32_t v; memcpy(&v, buf + pos, 4); pos += 4; t->shape[d] = v; t->n *= v; }
        ws->items[i].t = t;
        ws->count = (int)i + 1;
        int dtype = 0;                                             // 0 = fp32, 1 = bf16 (typed records only)
        if (typed) {
            if (pos + 1 + 8 > end) return fail(trunc);
            dtype = buf[pos++];
            if (dtype > 1) return fail("unknown element type");
        }
        uint64_t nbytes;
        memcpy(&nbytes, buf + pos, 8); pos += 8;
        if (nbytes > end - pos) return fail(strict ? trunc : "truncated payload");
        if ((uint64_t)t->n * (dtype ? 2 : 4) != nbytes) {
            snprintf(err, errcap, "%s: tensor '%s' size mismatch", path, ws->items[i].name);
            return fail("size mismatch");
        }
        if (dtype && nbytes > max16) max16 = (size_t)nbytes;
        if (!dtype && nd >= 2) all_matrices_16 = false;
        spans[i] = Span{pos, (size_t)nbytes, slab, dtype};
        // an empty tensor still gets a slot of its own, so that no two tensors share an address
        const size_t room = (size_t)t->n * 4;
        slab += room ? ((room + 255) & ~(size_t)255) : 256;
        pos += nbytes;
    }
    char *dslab = nullptr;
    CUDA_CHECK(cudaMalloc((void **)&dslab, slab ? slab : 256));
    unsigned short *stage16 = nullptr;                             // 2-byte payloads pass through here, one at a time, in stream order
    if (max16) CUDA_CHECK(cudaMalloc((void **)&stage16, max16));
    for (uint32_t i = 0; i < count; i++) {
        ws->items[i].t->data = (float *)(dslab + spans[i].slab_off);
        slab_members().insert(ws->items[i].t->data);
        if (!spans[i].nbytes) continue;
        if (spans[i].dtype) {
            const int64_t n = ws->items[i].t->n;
            CUDA_CHECK(cudaMemcpyAsync(stage16, buf + spans[i].file_off, spans[i].nbytes, cudaMemcpyHostToDevice, stream()));
            const int64_t g = cdiv(n, 256), cap = (int64_t)ctx().sm_count * 16;
            LAUNCH(k_widen_bf16, (unsigned)(g > cap ? cap : g), 256, 0, (const unsigned short *)stage16, ws->items[i].t->data, n);
        } else {
            CUDA_CHECK(cudaMemcpyAsync(dslab + spans[i].slab_off, buf + spans[i].file_off, spans[i].nbytes,
                                       cudaMemcpyHostToDevice, stream()));
        }
    }
    CUDA_CHECK(cudaStreamSynchronize(stream()));
    if (stage16) CUDA_CHECK(cudaFree(stage16));
    slab_of_store()[ws->items] = dslab;
    if (all_matrices_16 && count) bf16_stores().insert(ws->items);
    return 0;
}

uint64_t fnv1a64(const unsigned char *b, size_t n) {
    uint64_t h = 14695981039346656037ULL;
    for (size_t i = 0; i < n; i++) { h ^= b[i]; h *= 1099511628211ULL; }
    return h;
}

// bounds-checked little-endian cursor over the checkpoint header
struct Cursor {
    const unsigned char *p, *end;
    bool bad = false;
    uint64_t le(int n) {
        if (bad || (size_t)(end - p) < (size_t)n) { bad = true; return 0; }
        uint64_t v = 0;
        for (int i = n - 1; i >= 0; i--) v = (v << 8) | p[i];
        p += n;
        return v;
    }
    void skip_str() {
        uint64_t n = le(2);
        if (bad || (size_t)(end - p) < n) { bad = true; return; }
        p += n;
    }
};
} // namespace

// a store whose tensors were placed in `slab` by another loader (the safetensors import): weights_free then treats it
// like a store of weights_load
void ncmb_store_adopt_slab(WeightStore *ws, void *slab) {
    for (int i = 0; i < ws->count; i++) slab_members().insert(ws->items[i].t->data);
    slab_of_store()[ws->items] = slab;
}

// Rows of token ids from an "NCMT" file (reference train_data_load src/tensor.c:375-397): a 20-byte header (magic,
// u64 rows, u64 row length) and rows * row_len little-endian int32. Host-only; the file's size is checked against the
// header before anything is allocated.
TrainData *train_data_load(const char *path, int max_rows) {
    FILE *f = fopen(path, "rb");
    if (!f) { fprintf(stderr, "cannot open %s\n", path); return nullptr; }
    struct __attribute__((packed)) { char magic[4]; uint64_t rows, row_len; } hd;
    if (fread(&hd, 1, sizeof(hd), f) != sizeof(hd) || memcmp(hd.magic, "NCMT", 4) != 0) {
        fprintf(stderr, "%s: bad magic\n", path);
        fclose(f);
        return nullptr;
    }
    uint64_t rows = hd.rows;
    if (max_rows > 0 && rows > (uint64_t)max_rows) rows = (uint64_t)max_rows;
    fseek(f, 0, SEEK_END);
    const uint64_t have = (uint64_t)ftell(f) - sizeof(hd);
    if (hd.row_len == 0 || hd.row_len > 0x7fffffffu || rows > 0x7fffffffu || rows * hd.row_len * sizeof(int) > have) {
        fprintf(stderr, "%s: short read\n", path);
        fclose(f);
        return nullptr;
    }
    TrainData *d = (TrainData *)calloc(1, sizeof(TrainData));
    const size_t n = (size_t)(rows * hd.row_len);
    int *ids = (int *)malloc((n ? n : 1) * sizeof(int));
    if (!d || !ids) fatal("oom reading %s", path);
    fseek(f, (long)sizeof(hd), SEEK_SET);
    const size_t got = fread(ids, sizeof(int), n, f);
    fclose(f);
    if (got != n) { fprintf(stderr, "%s: short read\n", path); free(ids); free(d); return nullptr; }
    d->rows = ids; d->n_rows = (int)rows; d->row_len = (int)hd.row_len;
    return d;
}
void train_data_free(TrainData *d) {
    if (!d) return;
    free(d->rows);
    free(d);
}

// 1 = NCK1 checkpoint, 0 = NCM1 weights, -1 = neither / unreadable (reference ckpt_probe src/ckpt.c:67-77)
int ckpt_probe(const char *path) {
    FILE *f = fopen(path, "rb");
    if (!f) return -1;
    char magic[4];
    size_t r = fread(magic, 1, 4, f);
    fclose(f);
    if (r != 4) return -1;
    if (memcmp(magic, "NCK1", 4) == 0) return 1;
    if (memcmp(magic, "NCM1", 4) == 0) return 0;
    return -1;
}

int ckpt_load_weights_only(const char *path, WeightStore *ws, char *err, size_t errcap) {
    ensure_device();
    char local[256];
    if (!err || !errcap) { err = local; errcap = sizeof(local); }
    err[0] = 0;
    ws->items = nullptr; ws->count = 0;
    FileImage im;
    if (read_image(path, im, err, errcap)) return -1;
    uint64_t file_sum;
    memcpy(&file_sum, im.buf + im.len - 8, 8);
    if (fnv1a64(im.buf, im.len - 8) != file_sum) { snprintf(err, errcap, "%s: checksum mismatch", path); return -1; }
    Cursor c{im.buf, im.buf + im.len - 8};
    const bool magic_ok = im.len - 8 >= 4 && memcmp(im.buf, "NCK1", 4) == 0;
    c.le(4);
    if (!magic_ok || c.le(4) != 1u || c.bad) { snprintf(err, errcap, "%s: not an NCK1 checkpoint", path); return -1; }
    // run state: step i64, batch rng u64, three f64 of the schedule, batch i32, pending i32, rows i64, row length i32,
    // data hash u64, data path, conf hash u64, tokenizer id, training config
    c.le(8); c.le(8); c.le(8); c.le(8); c.le(8); c.le(4); c.le(4); c.le(8); c.le(4); c.le(8);
    c.skip_str(); c.le(8); c.skip_str(); c.skip_str();
    uint32_t n = (uint32_t)c.le(4);
    if (c.bad || n > (1u << 24)) { snprintf(err, errcap, "%s: bad tensor count", path); return -1; }
    return load_tensor_records(ws, path, im, (size_t)(c.p - im.buf), im.len - 8, n, true, err, errcap);
}

int weights_load(WeightStore *ws, const char *path) {
    ensure_device();
    ws->items = nullptr; ws->count = 0;
    char err[256] = {0};
    if (ckpt_probe(path) == 1) {
        if (ckpt_load_weights_only(path, ws, err, sizeof(err))) { fprintf(stderr, "%s\n", err); return -1; }
        return 0;
    }
    FileImage im;
    int rc = read_image(path, im, err, sizeof(err));
    // "NCM2": the NCM1 layout with one byte of element type (0 fp32, 1 bf16) in front of each record's byte count;
    // bf16 payloads are widened on the device, so every consumer still sees fp32 tensors
    const bool typed = !rc && memcmp(im.buf, "NCM2", 4) == 0;
    if (!rc && !typed && memcmp(im.buf, "NCM1", 4) != 0) { snprintf(err, sizeof(err), "%s: bad magic", path); rc = -1; }
    if (!rc) {
        uint32_t count;
        memcpy(&count, im.buf + 4, 4);
        rc = load_tensor_records(ws, path, im, 8, im.len, count, false, err, sizeof(err), typed);
    }
    if (rc) fprintf(stderr, "%s\n", err);
    return rc;
}

void weights_free(WeightStore *ws) {
    if (!ws || !ws->items) return;
    gemm_tc_forget_weights();
    gemm_h3_forget_weights();        // cached hi/lo splits point at memory that is about to go away
    cudaStreamSynchronize(stream());
    auto it = slab_of_store().find(ws->items);
    for (int i = 0; i < ws->count; i++) {
        Tensor *t = ws->items[i].t;
        if (!t) continue;
        if (slab_members().count(t->data)) slab_members().erase(t->data);
        else cudaFree(t->data);
        free(t);
    }
    if (it != slab_of_store().end()) { cudaFree(it->second); slab_of_store().erase(it); }
    bf16_stores().erase(ws->items);
    free(ws->items);
    ws->items = nullptr; ws->count = 0;
}

Tensor *weights_get(WeightStore *ws, const char *name) {
    for (int i = 0; i < ws->count; i++)
        if (strcmp(ws->items[i].name, name) == 0) return ws->items[i].t;
    return nullptr;
}

// ------------------------------------------------------------------ .conf
// Flat key=value; unknown keys ignored; True/False accepted where the reference
// accepts them (src/tensor.c:151-156); defaults as src/tensor.c:173-177.
static int conf_boolish(const char *v) {
    while (*v == ' ') v++;
    if (*v == 'T' || *v == 't') return 1;
    if (*v == 'F' || *v == 'f') return 0;
    return atoi(v);
}
static int conf_int_list(const char *v, int *out, int cap) {
    int k = 0;
    const char *p = v;
    while (*p && k < cap) {
        while (*p == ' ' || *p == ',') p++;
        if (!*p) break;
        out[k++] = atoi(p);
        while (*p && *p != ',') p++;
    }
    return k;
}

int config_load(NCMConfig *c, const char *path) {
    memset(c, 0, sizeof(*c));
    c->bias = 1; c->rope_base = 10000; c->rope_theta = 10000.0; c->n_kv_heads = -1;
    c->prefix_pad_token_id = -1; c->eos_token_id = -1; c->pad_token_id = -1;
    c->attn_pattern_block_diag = 1; c->gen_top_k = 1; c->gen_top_p = 1.0f;
    FILE *f = fopen(path, "r");
    if (!f) { fprintf(stderr, "cannot open %s\n", path); return -1; }
    enum { BOOLISH, PLAIN };
    struct IntKey { const char *key; int *dst; int kind; };
    const IntKey ints[] = {
        {"model.n_layer", &c->n_layer, BOOLISH}, {"model.n_head", &c->n_head, BOOLISH},
        {"model.n_embd", &c->n_embd, BOOLISH}, {"model.context_length", &c->context_length, BOOLISH},
        {"model.prefix_len", &c->prefix_len, BOOLISH}, {"model.raw_token_prefix", &c->raw_token_prefix, BOOLISH},
        {"model.contextual_prefix", &c->contextual_prefix, BOOLISH},
        {"model.prefix_pad_token_id", &c->prefix_pad_token_id, BOOLISH},
        {"model.predict_level0", &c->predict_level0, BOOLISH}, {"model.query_level0", &c->query_level0, BOOLISH},
        {"model.l0_autoregressive", &c->l0_autoregressive, BOOLISH},
        {"model.use_positional_encoding", &c->use_positional_encoding, BOOLISH},
        {"model.use_level_encoding", &c->use_level_encoding, BOOLISH},
        {"model.use_rope", &c->use_rope, BOOLISH}, {"model.rope_base", &c->rope_base, BOOLISH},
        {"model.use_qk_norm", &c->use_qk_norm, BOOLISH}, {"model.use_flex_attention", &c->use_flex_attention, BOOLISH},
        {"model.n_kv_heads", &c->n_kv_heads, BOOLISH}, {"model.bias", &c->bias, PLAIN},
        {"model.ctx_enabled", &c->ctx_enabled, BOOLISH}, {"model.ctx_n_layer", &c->ctx_n_layer, BOOLISH},
        {"model.ctx_vocab", &c->ctx_vocab, BOOLISH}, {"model.puc_enabled", &c->puc_enabled, BOOLISH},
        {"model.puc_kernel", &c->puc_kernel, BOOLISH}, {"model.shared_output_head", &c->shared_output_head, BOOLISH},
        {"model.shared_head_per_level_bias", &c->shared_head_per_level_bias, BOOLISH},
        {"model.untied_head_bias", &c->untied_head_bias, BOOLISH},
        {"model.tie_heads_to_codebook", &c->tie_heads_to_codebook, BOOLISH},
        {"model.tie_heads_learn_scale", &c->tie_heads_learn_scale, BOOLISH},
        {"model.tie_heads_trainable", &c->tie_heads_trainable, BOOLISH},
        {"model.tie_heads_bias", &c->tie_heads_bias, BOOLISH},
        {"model.use_swiglu", &c->use_swiglu, BOOLISH}, {"model.use_geglu", &c->use_geglu, BOOLISH},
        {"model.use_relu2", &c->use_relu2, BOOLISH}, {"model.parallel_block", &c->parallel_block, BOOLISH},
        {"model.normformer", &c->normformer, BOOLISH}, {"model.use_layerscale", &c->use_layerscale, BOOLISH},
        {"model.use_rezero", &c->use_rezero, BOOLISH}, {"model.sudoku_size", &c->sudoku_size, PLAIN},
        {"vq.embed_dim", &c->vq_embed_dim, PLAIN}, {"vq.in_vocab", &c->vq_in_vocab, PLAIN},
        {"vq.context_length", &c->vq_context_length, PLAIN}, {"vq.n_layers", &c->vq_n_layers, PLAIN},
        {"vq.compression", &c->vq_compression, PLAIN}, {"vq.soft_levels", &c->vq_soft_levels, PLAIN},
        {"vq.qr_enabled", &c->quant_resi_enabled, PLAIN}, {"vq.qr_share", &c->quant_resi_share_mode, PLAIN},
        {"vq.l1_sampling", &c->learned_l1_sampling, PLAIN}, {"vq.l1_cascade", &c->learned_l1_cascade, PLAIN},
        {"vq.l1_base", &c->learned_l1_cascade_base, PLAIN}, {"vq.l1_norm", &c->learned_l1_norm, BOOLISH},
        {"vq.l1_norm_final", &c->learned_l1_norm_final, BOOLISH},
        {"vq.all_sampling", &c->learned_all_sampling, PLAIN}, {"vq.pre_quant_gn", &c->pre_quant_groupnorm, PLAIN},
        {"vq.qk_norm", &c->vq_qk_norm, BOOLISH}, {"vq.enc_layers", &c->enc_layers, PLAIN},
        {"vq.enc_window", &c->enc_attn_window, PLAIN}, {"vq.enc_convs", &c->enc_conv_layers, PLAIN},
        {"vq.enc_conv_kernel", &c->enc_conv_kernel, PLAIN}, {"vq.enc_positional", &c->enc_positional, PLAIN},
        {"vq.dec_layers", &c->dec_layers, PLAIN}, {"vq.dec_positional", &c->dec_positional, PLAIN},
        {"tok.eos_id", &c->eos_token_id, BOOLISH}, {"tok.pad_id", &c->pad_token_id, BOOLISH},
        {"gen.top_k", &c->gen_top_k, PLAIN},
    };
    struct FltKey { const char *key; float *dst; };
    const FltKey flts[] = {
        {"model.dropout", &c->dropout}, {"model.layerscale_init", &c->layerscale_init},
        {"vq.qr_ratio", &c->quant_resi_ratio}, {"gen.temperature", &c->gen_temperature},
        {"gen.top_p", &c->gen_top_p}, {"gen.cfg_scale", &c->gen_cfg_scale},
        {"gen.freq", &c->gen_freq}, {"gen.mu", &c->gen_mu},
    };
    char line[1024];
    while (fgets(line, sizeof line, f)) {
        char *eq = strchr(line, '=');
        if (!eq) continue;
        *eq = 0;
        const char *k = line;
        char *v = eq + 1;
        v[strcspn(v, "\r\n")] = 0;
        bool done = false;
        for (const IntKey &ik : ints)
            if (!strcmp(k, ik.key)) { *ik.dst = ik.kind == BOOLISH ? conf_boolish(v) : atoi(v); done = true; break; }
        if (done) continue;
        for (const FltKey &fk : flts)
            if (!strcmp(k, fk.key)) { *fk.dst = (float)atof(v); done = true; break; }
        if (done) continue;
        if (!strcmp(k, "task")) { strncpy(c->task, v, sizeof(c->task) - 1); }
        else if (!strcmp(k, "model.rope_theta")) c->rope_theta = atof(v);
        else if (!strcmp(k, "model.attn_pattern")) c->attn_pattern_block_diag = (strcmp(v, "block_diagonal") == 0);
        else if (!strcmp(k, "model.vocab_size")) c->n_levels_out = conf_int_list(v, c->vocab_size, NCM_MAX_VOCAB_LIST);
        else if (!strcmp(k, "vq.soft_tau")) c->vq_soft_tau = atof(v);
        else if (!strcmp(k, "vq.levels")) c->n_qlevels = conf_int_list(v, c->levels, NCM_MAX_LEVELS);
        else if (!strcmp(k, "vq.vocab")) conf_int_list(v, c->vq_vocab, NCM_MAX_LEVELS);
        else if (!strcmp(k, "tok.kind")) strncpy(c->pre_tok, v, sizeof(c->pre_tok) - 1);
        else if (!strcmp(k, "tok.model_id")) strncpy(c->hf_model_id, v, sizeof(c->hf_model_id) - 1);
        else if (!strcmp(k, "gen.adj")) {
            if (v[0]) {
                c->gen_adj_a = (float)atof(v);
                char *q = strchr(v, ',');
                c->gen_adj_w = q ? atoi(q + 1) : 1;
                q = q ? strchr(q + 1, ',') : nullptr;
                c->gen_adj_d = q ? (float)atof(q + 1) : 1.0f;
            }
        }
    }
    fclose(f);
    if (c->n_kv_heads < 0) c->n_kv_heads = c->n_head;
    return 0;
}

// ------------------------------------------------------------------ additions
const char *ncmb_version(void) { return "ncm_b200 0.1 (sm_100a)"; }
void ncmb_set_stream(void *s) { ensure_device(); ctx().stream = (cudaStream_t)s; }
void *ncmb_get_stream(void) { return (void *)ctx().stream; }
void ncmb_sync(void) { ensure_device(); CUDA_CHECK(cudaStreamSynchronize(stream())); }
void ncmb_set_gemm_mode(int mode) { ensure_device(); ctx().gemm_mode = mode; }
int ncmb_get_gemm_mode(void) { ensure_device(); return ctx().gemm_mode; }
int ncmb_gemm_tc_check(void) { ensure_device(); return gemm_tc_check(); }
void ncmb_set_rng_mode(int mode) { ensure_device(); ctx().rng_mode = mode; }
void ncmb_set_row_offset(long long off) { ctx().row_offset = off; }
long long ncmb_launch_count(void) { return ctx().launches; }
void ncmb_forget_weight_copies(void) { gemm_tc_forget_weights(); gemm_h3_forget_weights(); }
int ncmb_weights_are_bf16(const WeightStore *ws) { return ws && ws->items && bf16_stores().count(ws->items) ? 1 : 0; }
void ncmb_mem_info(unsigned long long *free_bytes, unsigned long long *total_bytes) {
    ensure_device();
    size_t f = 0, t = 0;
    CUDA_CHECK(cudaMemGetInfo(&f, &t));
    if (free_bytes) *free_bytes = f;
    if (total_bytes) *total_bytes = t;
}
void ncmb_copy_bytes(unsigned long long *h2d, unsigned long long *d2h) {
    if (h2d) *h2d = ctx().h2d_bytes;
    if (d2h) *d2h = ctx().d2h_bytes;
}

void ncmb_prof_enable(int on) {
    ensure_device();
    Prof &p = prof();
    if (!on) p.drain();
    p.on = on != 0; p.depth = 0;
}
void ncmb_prof_reset(void) {
    Prof &p = prof();
    p.drain();
    for (int i = 0; i < NCMB_K_COUNT; i++) { p.launches[i] = 0; p.ms[i] = p.flops[i] = p.bytes[i] = 0; }
    p.shapes.clear();
}
// the call shape of class `klass` with the largest total time since the last reset: its launch count,
// total ms, and the flops / bytes ONE call declared. Returns -1 when the class recorded nothing.
int ncmb_prof_top_shape(int klass, long long *launches, double *ms, double *flops, double *bytes) {
    Prof &p = prof();
    p.drain();
    const std::pair<const std::tuple<int, double, double>, std::pair<long long, double>> *best = nullptr;
    for (auto &kv : p.shapes)
        if (std::get<0>(kv.first) == klass && (!best || kv.second.second > best->second.second)) best = &kv;
    if (!best) return -1;
    if (launches) *launches = best->second.first;
    if (ms) *ms = best->second.second;
    if (flops) *flops = std::get<1>(best->first);
    if (bytes) *bytes = std::get<2>(best->first);
    return 0;
}

// prints the per-shape table to stderr, largest total first, and clears it
void ncmb_prof_dump_shapes(void) {
    Prof &p = prof();
    p.drain();
    std::vector<std::pair<double, std::string>> rows;
    for (auto &kv : p.shapes) {
        char buf[256];
        double fl = std::get<1>(kv.first), by = std::get<2>(kv.first), ms = kv.second.second;
        snprintf(buf, sizeof buf, "class %d  %6lld x %9.1f us = %9.2f ms  flops %.4g (%.1f TF/s)  bytes %.4g (%.0f GB/s)", std::get<0>(kv.first),
                 kv.second.first, 1e3 * ms / kv.second.first, ms, fl, fl * kv.second.first / ms / 1e9, by, by * kv.second.first / ms / 1e6);
        rows.emplace_back(-ms, buf);
    }
    std::sort(rows.begin(), rows.end());
    for (auto &r : rows) fprintf(stderr, "%s\n", r.second.c_str());
    p.shapes.clear();
}

int ncmb_prof_read(int klass, long long *launches, double *ms, double *flops, double *bytes) {
    if (klass < 0 || klass >= NCMB_K_COUNT) return -1;
    Prof &p = prof();
    p.drain();
    if (launches) *launches = p.launches[klass];
    if (ms) *ms = p.ms[klass];
    if (flops) *flops = p.flops[klass];
    if (bytes) *bytes = p.bytes[klass];
    return 0;
}

} // extern "C"
