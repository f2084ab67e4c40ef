// placeholder until the register-tiled kernels land
#include "common.cuh"
namespace psig {
bool tiled_supported(int, int) { return false; }
int tiled_sig_forward(const PsigSigDesc &, const float *, float *, cudaStream_t) { return PSIG_ERR_UNSUPPORTED; }
int64_t tiled_sig_backward_workspace(const PsigSigDesc &) { return 0; }
int tiled_sig_backward(const PsigSigDesc &, const float *, const float *, const float *, float *, void *, cudaStream_t) { return PSIG_ERR_UNSUPPORTED; }
}
