// Quantizer state and device-side entry points shared with the VQ-VAE and NCP code.
#pragma once
#include "common.cuh"

struct VQState {
    int n_levels = 0, levels[NCM_MAX_LEVELS] = {0}, vocabs[NCM_MAX_LEVELS] = {0}, D = 0, L = 0;
    float *E[NCM_MAX_LEVELS] = {nullptr};                 // codebooks [V_k][D] (device, owned by the WeightStore)
    int resi = 0; float resi_ratio = 0.f; int n_phi = 0;
    float *phiW[NCM_MAX_LEVELS] = {nullptr}, *phiB[NCM_MAX_LEVELS] = {nullptr};
    double ticks[NCM_MAX_LEVELS] = {0};
    int has_l1 = 0, n_down = 0, n_up = 0, l1_norm = 0, l1_norm_final = 0;
    float *downW[16] = {nullptr}, *downB[16] = {nullptr}, *upW[16] = {nullptr}, *upB[16] = {nullptr};
    int downK[16] = {0}, upK[16] = {0};
    int has_all = 0;
    float *drefW[NCM_MAX_LEVELS] = {nullptr}, *drefB[NCM_MAX_LEVELS] = {nullptr};
    float *urefW[NCM_MAX_LEVELS] = {nullptr}, *urefB[NCM_MAX_LEVELS] = {nullptr};
    ncmb::Workspace work, codes_ws;
};

namespace ncmb {
// All pointers device memory. `scratch` sizes are in units of n = B*L*D floats.
void vq_increment_dev(VQState *v, const int *codes_dev, int stride, int rowmod, int level, int B, float *up, float *scratch /*4n*/);
void vq_next_input_dev(VQState *v, const int *codes_dev, int stride, int rowmod, int level, float *z_hat, float *x_out, int B, float *scratch /*5n*/);
void vq_encode_dev(VQState *v, const float *z, int B, int *idx_dev, float *scratch /*7n*/);
void vq_zhat_final_dev(VQState *v, const int *idx_dev, int B, float *z_hat, float **snapshots, float *scratch /*5n*/);
void vq_nearest(const float *x, const float *E, int64_t rows, int V, int D, int *idx_out, int out_tlen, int out_stride, int out_off);
int *vq_codes_to_dev(VQState *v, const int *host, size_t n);
} // namespace ncmb
