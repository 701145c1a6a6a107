// Hugging Face safetensors -> WeightStore on the device, without the detour through an NCM1 file.
//
// The reference converts checkpoints offline (tools/gpt2import.c, tools/qwenimport.c: safetensors -> model.ncm
// on disk, later read by weights_load). The tensor rules are theirs:
//   * F32 is taken as is, F16 and BF16 are widened to fp32 (gpt2import.c:250-266, 393-408), fp16 subnormals the
//     way that converter does it;
//   * buffers whose name ends in ".attn.bias" (the causal mask) are dropped (gpt2import.c:385, qwenimport.c:383);
//   * GPT-2 only: 2-D "*.weight" tensors of c_attn / c_proj / c_fc (HF Conv1D, stored [in][out]) are transposed
//     to [out][in] (gpt2import.c:387-390, 409-417); Qwen2's nn.Linear weights already are [out][in]
//     (qwenimport.c:5-6);
//   * names and the order of the file's header are kept.
// Here the file is staged once in pinned memory, every tensor's bytes go to the device as they are, and one
// kernel per tensor widens and (where asked) transposes them into a slab that the WeightStore's tensors point
// into. Tokenizer assets (vocab / merges conversion) are host text work and stay with the reference's tools.
#include "common.cuh"

#include <string>
#include <vector>

namespace ncmb {

// dtype codes: 0 F32, 1 F16, 2 BF16
__global__ void k_import_tensor(const unsigned char *__restrict__ raw, float *__restrict__ out, int64_t n, int dtype,
                                int64_t R, int64_t C, int transpose) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        // i indexes the output; with a transpose the output is [C][R] and element (c, r) comes from in[r][c]
        int64_t src = i;
        if (transpose) { const int64_t c = i / R, r = i % R; src = r * C + c; }
        float v;
        if (dtype == 0) v = ((const float *)raw)[src];
        else if (dtype == 1) {
            // as the reference's converter widens fp16 (tools/gpt2import.c:250-259): IEEE for normal numbers,
            // infinities and NaNs; a subnormal with mantissa m becomes the float with BITS 0x33800000 + (m << 13)
            // (m * 2^-24 only for m = 1), so that an import equals the .ncm file the reference would have made
            const unsigned h = ((const unsigned short *)raw)[src];
            const unsigned sg = (h >> 15) & 1u, ex = (h >> 10) & 0x1Fu, m = h & 0x3FFu;
            unsigned f;
            if (ex == 0) f = m ? 0x33800000u + (m << 13) : 0u;
            else if (ex == 31) f = 0x7F800000u | (m << 13);
            else f = ((ex + 112u) << 23) | (m << 13);
            v = __uint_as_float((sg << 31) | f);
        }
        else v = __uint_as_float((unsigned)((const unsigned short *)raw)[src] << 16);
        out[i] = v;
    }
}

namespace {

// the few JSON forms a safetensors header uses
struct Json {
    const unsigned char *p, *end;
    bool bad = false;
    void ws() { while (p < end && (*p == ' ' || *p == '\t' || *p == '\n' || *p == '\r')) p++; }
    bool eat(char c) { ws(); if (p < end && *p == (unsigned char)c) { p++; return true; } return false; }
    bool peek(char c) { ws(); return p < end && *p == (unsigned char)c; }
    std::string str() {
        std::string s;
        ws();
        if (p >= end || *p != '"') { bad = true; return s; }
        p++;
        while (p < end && *p != '"') {
            if (*p == '\\') {
                p++;
                if (p >= end) { bad = true; return s; }
                const char e = (char)*p++;
                switch (e) {
                    case 'n': s.push_back('\n'); break;
                    case 't': s.push_back('\t'); break;
                    case 'r': s.push_back('\r'); break;
                    case 'b': s.push_back('\b'); break;
                    case 'f': s.push_back('\f'); break;
                    case 'u':                                  // kept verbatim: tensor names are plain ASCII
                        s += "\\u";
                        break;
                    default: s.push_back(e);
                }
            } else s.push_back((char)*p++);
        }
        if (p >= end) { bad = true; return s; }
        p++;
        return s;
    }
    long long integer() {
        ws();
        bool neg = false;
        if (p < end && *p == '-') { neg = true; p++; }
        if (p >= end || *p < '0' || *p > '9') { bad = true; return 0; }
        long long v = 0;
        while (p < end && *p >= '0' && *p <= '9') v = v * 10 + (*p++ - '0');
        return neg ? -v : v;
    }
    void skip() {                                              // any value
        ws();
        if (p >= end) { bad = true; return; }
        if (*p == '"') { str(); return; }
        if (*p == '{' || *p == '[') {
            const char close = *p == '{' ? '}' : ']';
            const bool obj = *p == '{';
            p++;
            if (eat(close)) return;
            for (;;) {
                if (obj) { str(); if (!eat(':')) { bad = true; return; } }
                skip();
                if (bad) return;
                if (eat(',')) continue;
                if (eat(close)) return;
                bad = true;
                return;
            }
        }
        while (p < end && *p != ',' && *p != '}' && *p != ']' && *p != ' ' && *p != '\t' && *p != '\n' && *p != '\r') p++;
    }
};

struct Entry {
    std::string name, dtype;
    std::vector<int64_t> shape;
    long long off0 = -1, off1 = -1;
};

bool ends_with(const std::string &s, const char *suf) {
    const size_t n = strlen(suf);
    return s.size() >= n && s.compare(s.size() - n, n, suf) == 0;
}

} // namespace
} // namespace ncmb

using namespace ncmb;

extern "C" void ncmb_store_adopt_slab(WeightStore *ws, void *slab);      // runtime.cu: the store frees the slab with its tensors

extern "C" int ncmb_weights_import_safetensors(WeightStore *ws, const char *path, int conv1d_transpose) {
    ensure_device();
    ws->items = nullptr; ws->count = 0;
    FILE *f = fopen(path, "rb");
    if (!f) { fprintf(stderr, "cannot open %s\n", path); return -1; }
    fseek(f, 0, SEEK_END);
    const long fsz = ftell(f);
    fseek(f, 0, SEEK_SET);
    unsigned char *buf = nullptr;
    auto fail = [&](const char *why) {
        fprintf(stderr, "%s: %s\n", path, why);
        if (buf) cudaFreeHost(buf);
        if (ws->items) { for (int i = 0; i < ws->count; i++) free(ws->items[i].t); free(ws->items); }
        ws->items = nullptr; ws->count = 0;
        return -1;
    };
    if (fsz < 8) { fclose(f); return fail("bad header"); }
    if (cudaMallocHost((void **)&buf, (size_t)fsz) != cudaSuccess) { buf = nullptr; fclose(f); return fail("pinned staging alloc failed"); }
    const size_t got = fread(buf, 1, (size_t)fsz, f);
    fclose(f);
    if (got != (size_t)fsz) return fail("short read");
    uint64_t hlen;
    memcpy(&hlen, buf, 8);
    if (hlen > (uint64_t)fsz - 8) return fail("short header");
    const size_t data0 = 8 + (size_t)hlen;
    Json j{buf + 8, buf + 8 + hlen};
    if (!j.eat('{')) return fail("bad json");
    std::vector<Entry> ents;
    if (!j.eat('}')) {
        for (;;) {
            Entry e;
            e.name = j.str();
            if (j.bad || !j.eat(':')) return fail("bad key");
            if (e.name == "__metadata__") j.skip();
            else {
                if (!j.eat('{')) return fail("bad tensor obj");
                if (!j.eat('}')) {
                    for (;;) {
                        const std::string fk = j.str();
                        if (j.bad || !j.eat(':')) return fail("bad field");
                        if (fk == "dtype") e.dtype = j.str();
                        else if (fk == "shape") {
                            if (!j.eat('[')) return fail("bad shape");
                            if (!j.eat(']')) {
                                for (;;) {
                                    e.shape.push_back(j.integer());
                                    if (j.bad) return fail("bad dim");
                                    if (j.eat(',')) continue;
                                    if (j.eat(']')) break;
                                    return fail("bad shape sep");
                                }
                            }
                        } else if (fk == "data_offsets") {
                            if (!j.eat('[')) return fail("bad offsets");
                            e.off0 = j.integer();
                            if (!j.eat(',')) return fail("bad offsets");
                            e.off1 = j.integer();
                            if (j.bad || !j.eat(']')) return fail("bad offsets");
                        } else j.skip();
                        if (j.bad) return fail("bad tensor obj");
                        if (j.eat(',')) continue;
                        if (j.eat('}')) break;
                        return fail("bad tensor sep");
                    }
                }
                if (!ends_with(e.name, ".attn.bias")) ents.push_back(std::move(e));
            }
            if (j.bad) return fail("bad json");
            if (j.eat(',')) continue;
            if (j.eat('}')) break;
            return fail("bad top sep");
        }
    }
    // sizes, slab layout
    struct Plan { int dtype; int64_t n; size_t raw_off, raw_bytes, slab_off; int transpose; };
    std::vector<Plan> plan(ents.size());
    size_t slab = 0, raw_max = 0;
    for (size_t i = 0; i < ents.size(); i++) {
        const Entry &e = ents[i];
        Plan &p = plan[i];
        if (e.dtype == "F32") p.dtype = 0;
        else if (e.dtype == "F16") p.dtype = 1;
        else if (e.dtype == "BF16") p.dtype = 2;
        else { fprintf(stderr, "unsupported dtype %s for %s\n", e.dtype.c_str(), e.name.c_str()); return fail("unsupported dtype"); }
        if (e.shape.empty() || e.shape.size() > NCM_MAX_DIMS) return fail("tensor rank outside 1..4");
        if (e.name.size() >= sizeof(ws->items[0].name)) return fail("tensor name too long");
        p.n = 1;
        for (int64_t d : e.shape) { if (d < 0) return fail("bad dim"); p.n *= d; }
        p.raw_bytes = (size_t)p.n * (p.dtype == 0 ? 4 : 2);
        if (e.off0 < 0 || (size_t)e.off0 + p.raw_bytes > (size_t)fsz - data0) return fail("tensor data outside the file");
        p.raw_off = data0 + (size_t)e.off0;
        const bool is_w = ends_with(e.name, ".weight");
        p.transpose = conv1d_transpose && e.shape.size() == 2 && is_w &&
                      (e.name.find("c_attn") != std::string::npos || e.name.find("c_proj") != std::string::npos ||
                       e.name.find("c_fc") != std::string::npos || e.name.find("proj") != std::string::npos);
        p.slab_off = slab;
        slab += ((size_t)p.n * 4 + 255) & ~(size_t)255;
        raw_max = raw_max > p.raw_bytes ? raw_max : p.raw_bytes;
    }
    ws->items = (NamedTensor *)calloc(ents.size() ? ents.size() : 1, sizeof(NamedTensor));
    char *dslab = nullptr;
    unsigned char *raw_d = nullptr;
    CUDA_CHECK(cudaMalloc((void **)&dslab, slab ? slab : 256));
    CUDA_CHECK(cudaMalloc((void **)&raw_d, raw_max ? raw_max : 256));
    for (size_t i = 0; i < ents.size(); i++) {
        const Entry &e = ents[i];
        const Plan &p = plan[i];
        Tensor *t = (Tensor *)calloc(1, sizeof(Tensor));
        t->ndim = (int)e.shape.size(); t->n = p.n;
        for (int d = 0; d < t->ndim; d++) t->shape[d] = e.shape[d];
        if (p.transpose) { t->shape[0] = e.shape[1]; t->shape[1] = e.shape[0]; }
        t->data = (float *)(dslab + p.slab_off);
        snprintf(ws->items[i].name, sizeof(ws->items[i].name), "%s", e.name.c_str());
        ws->items[i].t = t;
        ws->count = (int)i + 1;
        if (p.n == 0) continue;
        // a 2-byte or transposed tensor passes through the staging buffer and one kernel; plain fp32 is copied straight in
        if (p.dtype == 0 && !p.transpose) {
            CUDA_CHECK(cudaMemcpyAsync(t->data, buf + p.raw_off, p.raw_bytes, cudaMemcpyHostToDevice, stream()));
        } else {
            CUDA_CHECK(cudaMemcpyAsync(raw_d, buf + p.raw_off, p.raw_bytes, cudaMemcpyHostToDevice, stream()));
            const int64_t R = e.shape.size() == 2 ? e.shape[0] : 1, C = e.shape.size() == 2 ? e.shape[1] : p.n;
            const int64_t g = cdiv(p.n, 256), cap = (int64_t)ctx().sm_count * 16;
            LAUNCH(k_import_tensor, (unsigned)(g > cap ? cap : g), 256, 0, (const unsigned char *)raw_d, t->data, p.n, p.dtype, R, C, p.transpose);
        }
    }
    CUDA_CHECK(cudaStreamSynchronize(stream()));
    cudaFree(raw_d);
    cudaFreeHost(buf);
    ncmb_store_adopt_slab(ws, dslab);
    return 0;
}
