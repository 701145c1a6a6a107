// Persistent decode-step kernel of the decoder LMs (lm_mega.cu): argument block shared with lm.cu.
#pragma once
#include "common.cuh"

namespace ncmb {

constexpr int MG_MAXB = 4;            // sequences per step the persistent kernel takes

struct MegaLayer {
    const float *ln1w, *ln1b, *qkvw, *qkvb, *ow, *ob, *ln2w, *ln2b, *fcw, *fcb, *pw, *pb;
    float *kv;                        // this layer's cache [B][cap][2*nkv*hd]
};

struct MegaArgs {
    int B, C, H, nkv, I, NL, V;
    int norm;                         // 1 LayerNorm, 2 RMSNorm
    int gated, act, rope;
    float eps, eps_f;                 // block norms / final norm
    const MegaLayer *layers;          // device array [NL]
    const float *wte, *wpe, *lnfw, *lnfb, *cosb, *sinb;
    float *x, *qkv, *ctx, *h, *logits, *part;
    unsigned *count;
    const int *ids, *posmat, *lenmat;
    int *step_d;                      // tokens finalised so far (v); this step's position is np - 1 + v
    int np, cap, n_new, max_split;
    int64_t kv_seq_pitch;
    unsigned *bar, *bar_base;         // barrier counter (only grows) and its value at the start of this launch
    int *err;
    int greedy;                       // 1: pick the arg max and close the step in the kernel
    unsigned long long *amax;
    int *out, *ids_out;
};

void lm_mega_enable(int on);
bool lm_mega_eligible(int B, int hd, int C, int I, bool qk_norm);
size_t lm_mega_smem(const MegaArgs &a);
void lm_mega_launch(const MegaArgs &a);     // on stream(); fatal when the cooperative launch is refused

} // namespace ncmb
