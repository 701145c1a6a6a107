/* Test infrastructure only.  The reference keeps gpt2_forward / gpt2_generate
 * (src/gpt2.c:92,179) and qwen_forward / qwen_generate (src/qwen.c:121,209)
 * file-static, so the only way to read their logits is to compile the
 * reference files, unchanged and from where they lie, into this translation
 * unit and export thin callers.  Nothing here restates reference code; the
 * build recipe passes -I<reference>/src and one of -DWRAP_GPT2 / -DWRAP_QWEN. */
#ifdef WRAP_GPT2
#include "gpt2.c"

void *ref_gpt2_open(const NCMConfig *c, const char *weights, const char *adir) {
    GPT2 *g = (GPT2 *)malloc(sizeof(GPT2));
    if (gpt2_open(g, c, weights, adir)) { free(g); return NULL; }
    return g;
}
int ref_gpt2_vocab(void *h) { return ((GPT2 *)h)->vocab_size; }
/* all-position logits [T][V] copied to out */
void ref_gpt2_logits(void *h, const int *ids, int T, float *out) {
    GPT2 *g = (GPT2 *)h;
    float *lg = gpt2_forward(g, ids, T);
    mem_d2h(out, lg, (size_t)T * g->vocab_size * sizeof(float));
}
double ref_gpt2_nll(void *h, const int *ids, int T) { return gpt2_nll((GPT2 *)h, ids, T); }
int ref_gpt2_generate(void *h, const int *prompt, int np, int n_new, float temp,
                      int top_k, float top_p, unsigned long long seed, int *out) {
    unsigned long long rng = seed ? seed : 0x12345678ULL;
    return gpt2_generate((GPT2 *)h, prompt, np, n_new, temp, top_k, top_p, &rng, out);
}
#endif

#ifdef WRAP_QWEN
#include "qwen.c"

void *ref_qwen_open(const NCMConfig *c, const char *weights, const char *adir) {
    QWEN *m = (QWEN *)malloc(sizeof(QWEN));
    if (qwen_open(m, c, weights, adir)) { free(m); return NULL; }
    return m;
}
int ref_qwen_vocab(void *h) { return ((QWEN *)h)->vocab_size; }
/* last_only=1: out gets [V]; else [T][V] */
void ref_qwen_logits(void *h, const int *ids, int T, int last_only, float *out) {
    QWEN *m = (QWEN *)h;
    float *lg = qwen_forward(m, ids, T, last_only);
    mem_d2h(out, lg, (size_t)(last_only ? 1 : T) * m->vocab_size * sizeof(float));
}
double ref_qwen_nll(void *h, const int *ids, int T) { return qwen_nll((QWEN *)h, ids, T); }
int ref_qwen_generate(void *h, const int *prompt, int np, int n_new, float temp,
                      int top_k, float top_p, unsigned long long seed, int *out) {
    unsigned long long rng = seed ? seed : 0x12345678ULL;
    return qwen_generate((QWEN *)h, prompt, np, n_new, temp, top_k, top_p, &rng, out);
}
#endif
