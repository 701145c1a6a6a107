// VQ-VAE state shared with the NCP generate code.
#pragma once
#include <vector>
#include "common.cuh"
#include "vq.cuh"

struct VQVAEState {
    NCMConfig cfg;
    WeightStore *ws = nullptr;
    VQState *vq = nullptr;
    std::vector<ncmb::BlockWeights> dec, enc;
    const float *dec_lnf = nullptr, *dec_out = nullptr, *dec_wpe = nullptr;
    const float *enc_wte = nullptr, *enc_wpe = nullptr;
    bool enc_ready = false;
    ncmb::Workspace work, dec_ws, starts_ws, tok_ws;
    const int *starts = nullptr; int starts_B = -1, starts_T = -1;
};

namespace ncmb {
BlockWeights vae_block_weights(WeightStore *ws, const char *pre, int qk_norm);
const int *uniform_starts(VQVAEState *v, int B, int T);
void vqvae_decode_dev(VQVAEState *v, const float *zhat, float *logits, int B);
void decode_tokens_dev(VQVAEState *v, const int *codes_dev, int B, int *tokens_dev);
} // namespace ncmb
