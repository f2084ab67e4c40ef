// Signature <-> log-signature in word coordinates: choice between the two forms of the Horner kernels
// (horner_logsig.cu).  Rows whose lower degrees fit shared memory take the row-in-shared-memory form and
// need neither cache nor scratch; larger rows (for example d = 16 at depth 5) and `algo = GENERIC` take
// the streamed form, whose buffers are the caller's cache (forward: 2*lower of its S*depth scalars per
// row) and workspace (backward).  The reference instead stores the powers P_m = (S-1)^{(x)m} of every
// word (src/pathsig/forward/sig_kernels.cu:214-240) and scatters their adjoints with atomics
// (src/pathsig/backward/sig_backward_kernels.cu:449-476); nothing of that scheme is used here -- the
// cache argument keeps the reference's shape so that the operator signatures stay the same.
#include "common.cuh"

namespace psig {

template <typename T>
int generic_logsig_forward(const PsigLogDesc &desc, const LevelTable &lt, const T *sig, T *logsig, T *cache,
                           cudaStream_t stream)
{
    if (desc.rows == 0 || lt.total == 0) return PSIG_OK;
    if (horner_logsig_supported(desc, lt)) return horner_logsig_forward<T>(desc, lt, sig, logsig, nullptr, stream);
    if (streamed_logsig_forward_scratch(desc, lt) < 0) return PSIG_ERR_TOO_LARGE;
    if (!cache) return PSIG_ERR_NULL;
    return horner_logsig_forward<T>(desc, lt, sig, logsig, cache, stream);
}

template <typename T>
int generic_logsig_backward(const PsigLogDesc &desc, const LevelTable &lt, const T *sig, const T *,
                            const T *grad_logsig, T *grad_sig, T *workspace, cudaStream_t stream)
{
    if (desc.rows == 0 || lt.total == 0) return PSIG_OK;
    if (horner_logsig_supported(desc, lt))
        return horner_logsig_backward<T>(desc, lt, sig, grad_logsig, grad_sig, nullptr, stream);
    if (streamed_logsig_backward_scratch(desc, lt) < 0) return PSIG_ERR_TOO_LARGE;
    if (!workspace) return PSIG_ERR_NULL;
    return horner_logsig_backward<T>(desc, lt, sig, grad_logsig, grad_sig, workspace, stream);
}

template int generic_logsig_forward<float>(const PsigLogDesc &, const LevelTable &, const float *, float *, float *,
                                           cudaStream_t);
template int generic_logsig_forward<double>(const PsigLogDesc &, const LevelTable &, const double *, double *,
                                            double *, cudaStream_t);
template int generic_logsig_backward<float>(const PsigLogDesc &, const LevelTable &, const float *, const float *,
                                            const float *, float *, float *, cudaStream_t);
template int generic_logsig_backward<double>(const PsigLogDesc &, const LevelTable &, const double *, const double *,
                                             const double *, double *, double *, cudaStream_t);

}  // namespace psig
