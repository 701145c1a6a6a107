// tcgen05 tensor-core GEMM engine (placeholder until the TMA/TMEM kernel lands).
#include "common.cuh"

namespace ncmb {
bool gemm_tc_supported(const GemmArgs &) { return false; }
void gemm_tc(const GemmArgs &a) { gemm_simt(a); }
} // namespace ncmb
