// Shared declarations of the pathsig_b200 CUDA library (internal header).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/pathsig_b200.h"

namespace psig {

constexpr int kMaxDepth = PSIG_MAX_DEPTH;

// One row of the signature as the kernels see it: per degree the number of kept words, where
// the degree starts inside the row, and the explicit codes (nullptr = dense degree).
// Mirrors the bookkeeping of the reference launchers (src/pathsig/forward/sig_launch.cu:167-182).
struct LevelTable {
    int d;
    int depth;
    long long size[kMaxDepth + 1];
    long long offset[kMaxDepth + 1];
    const long long *words[kMaxDepth + 1];
    long long total;        // row width D
    long long dense_offset[kMaxDepth + 1];  // start of degree k in a fully dense row
    bool lower_dense[kMaxDepth + 1];        // all degrees below k are stored dense
};

// Builds the table; `top_only` selects the hybrid layout of the log operators.
int make_level_table(int d, int depth, bool projected, const int64_t *level_sizes, const int64_t *words,
                     bool top_only, LevelTable *out);

// 1/n as a compile-time-foldable constant (n = 1..12).
template <typename T>
__host__ __device__ __forceinline__ constexpr T recip(int n) { return T(1) / T(n); }

template <typename T> struct DType;
template <> struct DType<float> { static constexpr int id = PSIG_F32; };
template <> struct DType<double> { static constexpr int id = PSIG_F64; };

// ---- launch entry points implemented in the .cu files (host functions) ----
template <typename T>
int generic_sig_forward(const PsigSigDesc &desc, const LevelTable &lt, const T *path, T *out, cudaStream_t stream);
template <typename T>
int generic_sig_backward(const PsigSigDesc &desc, const LevelTable &lt, const T *path, const T *sig, const T *grad,
                         T *grad_path, T *inc_grad_ws, cudaStream_t stream);
template <typename T>
int generic_logsig_forward(const PsigLogDesc &desc, const LevelTable &lt, const T *sig, T *logsig, T *cache,
                           cudaStream_t stream);
template <typename T>
int generic_logsig_backward(const PsigLogDesc &desc, const LevelTable &lt, const T *sig, const T *cache,
                            const T *grad_logsig, T *grad_sig, T *grad_cache_ws, cudaStream_t stream);

// Horner-form log-signature kernels (horner_logsig.cu).  `supported` tells whether the row fits shared
// memory; it is a pure function of the description, so forward and backward of one call always agree
// on the form.  With `scratch` null the row-in-shared-memory form runs; otherwise the streamed form, on
// streamed_logsig_*_scratch() scalars of global memory (negative: the row does not fit 32-bit positions).
bool horner_logsig_supported(const PsigLogDesc &desc, const LevelTable &lt);
long long streamed_logsig_forward_scratch(const PsigLogDesc &desc, const LevelTable &lt);
long long streamed_logsig_backward_scratch(const PsigLogDesc &desc, const LevelTable &lt);
template <typename T>
int horner_logsig_forward(const PsigLogDesc &desc, const LevelTable &lt, const T *sig, T *logsig, T *scratch,
                          cudaStream_t stream);
template <typename T>
int horner_logsig_backward(const PsigLogDesc &desc, const LevelTable &lt, const T *sig, const T *grad_logsig,
                           T *grad_sig, T *scratch, cudaStream_t stream);

// Register-tiled dense kernels, float32 and float64 (tiled_sig.cu).  `supported` tells whether a kernel
// exists for this description (dense, or dense below a projected top degree).
bool tiled_supported(const PsigSigDesc &desc);
template <typename T>
int tiled_sig_forward(const PsigSigDesc &desc, const T *path, T *out, cudaStream_t stream);
int64_t tiled_sig_backward_workspace(const PsigSigDesc &desc);
bool tiled_sig_backward_reproducible(const PsigSigDesc &desc);
// Bounded wait of the bulk-copy staging: poll limit (test hook) and read-and-clear count of waits that ran out.
int tiled_set_bulk_wait_polls(int polls);
long long tiled_bulk_copy_timeouts();
int tiled_top_plan(const PsigSigDesc &desc, bool backward, unsigned char *items, int *active);
template <typename T>
int tiled_sig_backward(const PsigSigDesc &desc, const T *path, const T *sig, const T *grad, T *grad_path,
                       void *workspace, cudaStream_t stream);

// Prefix-closure kernels generated for the word set (closure_jit.cu).  `worthwhile` is a cheap test
// of the description; `supported` builds (and caches) the plan, which compiles on first use.
bool closure_worthwhile(const PsigSigDesc &desc, const LevelTable &lt);
bool closure_supported(const PsigSigDesc &desc, const LevelTable &lt);
template <typename T>
int closure_sig_forward(const PsigSigDesc &desc, const LevelTable &lt, const T *path, T *out, cudaStream_t stream);
template <typename T>
int closure_sig_backward(const PsigSigDesc &desc, const LevelTable &lt, const T *path, const T *sig, const T *grad,
                         T *grad_path, T *inc_grad_ws, cudaStream_t stream);
long long closure_source(const PsigSigDesc &desc, const LevelTable &lt, int target_bins, char *buffer, long long capacity,
                         long long *stats);
int closure_compile_only(const char *text, const char *arch, char *log, long long log_capacity);
bool closure_compiler_available();

// Launch attributes of a kernel (opt-in dynamic shared memory above 48 KB, preference for the largest
// shared-memory carveout) are properties of the function on a device: they are set the first time a
// kernel is launched on a device, and again only when a launch needs more dynamic shared memory than
// any launch before it -- not on every call.  Returns false when the runtime refuses.
bool prepare_kernel_once(const void *kernel, size_t dynamic_smem, bool prefer_shared_carveout);
template <typename Kernel>
inline bool prepare_kernel(Kernel kernel, size_t dynamic_smem, bool prefer_shared_carveout)
{
    return prepare_kernel_once(reinterpret_cast<const void *>(kernel), dynamic_smem, prefer_shared_carveout);
}

// Called once after every kernel launch: counts the launch (psig_kernel_launches) and reports a
// failed one.
void count_launch();
inline int check_launch()
{
    count_launch();
    return cudaGetLastError() == cudaSuccess ? PSIG_OK : PSIG_ERR_CUDA;
}

}  // namespace psig
