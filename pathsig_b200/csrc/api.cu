// C ABI of libpathsig_b200.so: argument checks, level bookkeeping and kernel selection.
// Declarations and the reference operators they stand in for: include/pathsig_b200.h.
#include "common.cuh"

#include <atomic>
#include <map>
#include <mutex>
#include <utility>

namespace psig {

namespace {
std::atomic<long long> g_kernel_launches{0};
}
void count_launch() { g_kernel_launches.fetch_add(1, std::memory_order_relaxed); }

bool prepare_kernel_once(const void *kernel, size_t dynamic_smem, bool prefer_shared_carveout)
{
    static std::mutex mutex;
    static std::map<std::pair<const void *, int>, size_t> granted;  // (kernel, device) -> shared memory + 1
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return false;
    std::lock_guard<std::mutex> lock(mutex);
    size_t &have = granted[std::make_pair(kernel, device)];
    if (have > dynamic_smem) return true;
    if (dynamic_smem > 48 * 1024 &&
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dynamic_smem) != cudaSuccess)
        return false;
    if (prefer_shared_carveout && have == 0)
        cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    have = dynamic_smem + 1;
    return true;
}

int make_level_table(int d, int depth, bool projected, const int64_t *level_sizes, const int64_t *words,
                     bool top_only, LevelTable *out)
{
    LevelTable &lt = *out;
    lt.d = d;
    lt.depth = depth;
    long long d_pow = 1, off = 0, dense_off = 0, used = 0;
    bool all_dense = true;
    for (int k = 0; k <= kMaxDepth; ++k) {
        lt.size[k] = 0; lt.offset[k] = 0; lt.words[k] = nullptr; lt.dense_offset[k] = 0; lt.lower_dense[k] = true;
    }
    for (int k = 1; k <= depth; ++k) {
        if (d_pow > (long long)(0x7fffffffffffffffLL / d)) return PSIG_ERR_PACKING;
        d_pow *= d;
        long long size = d_pow;
        const long long *w = nullptr;
        if (projected && (!top_only || k == depth)) {
            size = level_sizes[k];
            if (size < 0) return PSIG_ERR_SHAPE;
            if (size != d_pow) {
                if (size > 0 && !words) return PSIG_ERR_NULL;
                w = reinterpret_cast<const long long *>(words) + used;
                used += size;
            }
        }
        lt.size[k] = size;
        lt.offset[k] = off;
        lt.words[k] = w;
        lt.dense_offset[k] = dense_off;
        lt.lower_dense[k] = all_dense;
        if (w != nullptr || size != d_pow) all_dense = false;
        off += size;
        dense_off += d_pow;
    }
    lt.total = off;
    return PSIG_OK;
}

namespace {

int check_sig_desc(const PsigSigDesc *desc)
{
    if (!desc) return PSIG_ERR_NULL;
    if (desc->dtype != PSIG_F32 && desc->dtype != PSIG_F64) return PSIG_ERR_DTYPE;
    if (desc->depth < 1 || desc->depth > kMaxDepth) return PSIG_ERR_DEPTH;
    if (desc->B < 0 || desc->L < 2 || desc->d < 1 || desc->W < 0) return PSIG_ERR_SHAPE;
    if (desc->W > 0 && !desc->windows) return PSIG_ERR_NULL;
    return PSIG_OK;
}

int sig_table(const PsigSigDesc *desc, LevelTable *lt)
{
    const int rc = check_sig_desc(desc);
    if (rc != PSIG_OK) return rc;
    return make_level_table(desc->d, desc->depth, desc->projected != 0, desc->level_sizes, desc->words, false, lt);
}

int log_table(const PsigLogDesc *desc, LevelTable *lt)
{
    if (!desc) return PSIG_ERR_NULL;
    if (desc->dtype != PSIG_F32 && desc->dtype != PSIG_F64) return PSIG_ERR_DTYPE;
    if (desc->depth < 1 || desc->depth > kMaxDepth) return PSIG_ERR_DEPTH;
    if (desc->rows < 0 || desc->d < 1 || desc->top_size < 0) return PSIG_ERR_SHAPE;
    int64_t sizes[kMaxDepth + 1] = {0};
    sizes[desc->depth] = desc->top_size;
    return make_level_table(desc->d, desc->depth, true, sizes, desc->top_words, true, lt);
}

enum class Family { kGeneric, kTiled, kClosure };

// Kernel family for a description; the same function serves the forward call, the workspace query and
// the backward call, so the three always agree.
//   tiled:   dense rows (or dense below a listed top degree) of a shape with a register-tiled instance;
//   closure: other projected rows whose word set is known on the host, when there is enough work to
//            repay the one-off specialisation (where both exist the two measured within 6 % of each
//            other on a (4, 6) row with a Lyndon top degree, so the family without a compilation wins);
//   generic: everything else.
Family select_family(const PsigSigDesc *desc, const LevelTable &lt, int *rc)
{
    *rc = PSIG_OK;
    if (desc->algo == PSIG_ALGO_GENERIC) return Family::kGeneric;
    if (desc->algo == PSIG_ALGO_CLOSURE) {
        if (closure_supported(*desc, lt)) return Family::kClosure;
        *rc = PSIG_ERR_UNSUPPORTED;
        return Family::kGeneric;
    }
    const bool tiled = tiled_supported(*desc);
    if (desc->algo == PSIG_ALGO_TILED) {
        if (!tiled) *rc = PSIG_ERR_UNSUPPORTED;
        return tiled ? Family::kTiled : Family::kGeneric;
    }
    if (tiled) return Family::kTiled;
    if (closure_worthwhile(*desc, lt) && closure_supported(*desc, lt)) return Family::kClosure;
    return Family::kGeneric;
}

size_t dtype_size(int dtype) { return dtype == PSIG_F32 ? 4 : 8; }

}  // namespace
}  // namespace psig

using namespace psig;

extern "C" {

int psig_abi_version(void) { return PSIG_ABI_VERSION; }

int64_t psig_kernel_launches(void) { return g_kernel_launches.load(std::memory_order_relaxed); }

int64_t psig_bulk_copy_timeouts(void) { return tiled_bulk_copy_timeouts(); }

int psig_set_bulk_wait_polls(int polls) { return tiled_set_bulk_wait_polls(polls); }

int psig_tiled_top_plan(const PsigSigDesc *desc, int backward, unsigned char *items, int *active)
{
    if (!desc || !items || !active) return PSIG_ERR_NULL;
    LevelTable lt;
    const int rc = sig_table(desc, &lt);
    if (rc != PSIG_OK) return rc;
    return tiled_top_plan(*desc, backward != 0, items, active);
}

const char *psig_status_string(int status)
{
    switch (status) {
        case PSIG_OK: return "ok";
        case PSIG_ERR_NULL: return "a required pointer is NULL";
        case PSIG_ERR_DTYPE: return "dtype must be float32 or float64";
        case PSIG_ERR_DEPTH: return "depth must be in [1,12]";
        case PSIG_ERR_SHAPE: return "invalid shape (need B >= 0, L >= 2, d >= 1, W >= 0, consistent level sizes)";
        case PSIG_ERR_PACKING: return "d^depth does not fit a 64-bit word code";
        case PSIG_ERR_WORKSPACE: return "workspace missing or too small";
        case PSIG_ERR_CUDA: return "CUDA runtime call or kernel launch failed";
        case PSIG_ERR_TOO_LARGE: return "problem size exceeds what this entry point supports";
        case PSIG_ERR_UNSUPPORTED: return "no kernel for this configuration";
        default: return "unknown status";
    }
}

int64_t psig_sig_size(const PsigSigDesc *desc)
{
    LevelTable lt;
    const int rc = sig_table(desc, &lt);
    return rc != PSIG_OK ? rc : lt.total;
}

int64_t psig_closure_source(const PsigSigDesc *desc, int target_bins, char *buffer, int64_t capacity, int64_t *stats)
{
    LevelTable lt;
    const int rc = sig_table(desc, &lt);
    if (rc != PSIG_OK) return rc;
    if (target_bins < 1) return PSIG_ERR_SHAPE;
    long long st[5] = {0, 0, 0, 0, 0};
    const long long n = closure_source(*desc, lt, target_bins, buffer, capacity, st);
    if (stats) for (int i = 0; i < 5; ++i) stats[i] = st[i];
    return n;
}

int psig_closure_available(void) { return closure_compiler_available() ? 1 : 0; }

int psig_closure_compile(const char *source, const char *arch, char *log, int64_t log_capacity)
{
    if (!source || !arch) return PSIG_ERR_NULL;
    return closure_compile_only(source, arch, log, log_capacity);
}

int64_t psig_logsig_size(const PsigLogDesc *desc)
{
    LevelTable lt;
    const int rc = log_table(desc, &lt);
    return rc != PSIG_OK ? rc : lt.total;
}

int64_t psig_logsig_out_size(const PsigLogDesc *desc)
{
    LevelTable lt;
    const int rc = log_table(desc, &lt);
    if (rc != PSIG_OK) return rc;
    if (desc->lower_columns == nullptr && desc->n_lower_columns == 0) return lt.total;
    if (desc->lower_columns == nullptr || desc->n_lower_columns < 0) return PSIG_ERR_SHAPE;
    return desc->n_lower_columns + lt.size[lt.depth];
}

int psig_sig_forward(const PsigSigDesc *desc, const void *path, void *out, void *stream)
{
    LevelTable lt;
    int rc = sig_table(desc, &lt);
    if (rc != PSIG_OK) return rc;
    if (desc->B == 0 || lt.total == 0) return PSIG_OK;
    if (!path || !out) return PSIG_ERR_NULL;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const Family family = select_family(desc, lt, &rc);
    if (rc != PSIG_OK) return rc;
    if (family == Family::kTiled) {
        if (desc->dtype == PSIG_F32)
            return tiled_sig_forward<float>(*desc, static_cast<const float *>(path), static_cast<float *>(out), st);
        return tiled_sig_forward<double>(*desc, static_cast<const double *>(path), static_cast<double *>(out), st);
    }
    if (family == Family::kClosure) {
        if (desc->dtype == PSIG_F32)
            return closure_sig_forward<float>(*desc, lt, static_cast<const float *>(path), static_cast<float *>(out), st);
        return closure_sig_forward<double>(*desc, lt, static_cast<const double *>(path), static_cast<double *>(out), st);
    }
    if (desc->dtype == PSIG_F32)
        return generic_sig_forward<float>(*desc, lt, static_cast<const float *>(path), static_cast<float *>(out), st);
    return generic_sig_forward<double>(*desc, lt, static_cast<const double *>(path), static_cast<double *>(out), st);
}

int64_t psig_sig_backward_workspace(const PsigSigDesc *desc)
{
    LevelTable lt;
    int rc = sig_table(desc, &lt);
    if (rc != PSIG_OK) return rc;
    const Family family = select_family(desc, lt, &rc);
    if (rc != PSIG_OK) return rc;
    if (family == Family::kTiled) return tiled_sig_backward_workspace(*desc);
    return (int64_t)dtype_size(desc->dtype) * desc->B * (desc->L - 1) * desc->d;
}

int psig_sig_backward_reproducible(const PsigSigDesc *desc)
{
    LevelTable lt;
    int rc = sig_table(desc, &lt);
    if (rc != PSIG_OK) return rc;
    const Family family = select_family(desc, lt, &rc);
    if (rc != PSIG_OK) return rc;
    return family == Family::kTiled && tiled_sig_backward_reproducible(*desc) ? 1 : 0;
}

int psig_sig_backward(const PsigSigDesc *desc, const void *path, const void *sig, const void *grad_sig,
                      void *grad_path, void *workspace, int64_t workspace_bytes, void *stream)
{
    LevelTable lt;
    int rc = sig_table(desc, &lt);
    if (rc != PSIG_OK) return rc;
    if (desc->B == 0) return PSIG_OK;
    if (!path || !grad_path) return PSIG_ERR_NULL;
    if (lt.total > 0 && (!sig || !grad_sig)) return PSIG_ERR_NULL;
    const int64_t need = psig_sig_backward_workspace(desc);
    if (need < 0) return (int)need;
    if (need > 0 && (!workspace || workspace_bytes < need)) return PSIG_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const Family family = select_family(desc, lt, &rc);
    if (rc != PSIG_OK) return rc;
    if (family == Family::kClosure) {
        if (desc->dtype == PSIG_F32)
            return closure_sig_backward<float>(*desc, lt, static_cast<const float *>(path),
                                               static_cast<const float *>(sig), static_cast<const float *>(grad_sig),
                                               static_cast<float *>(grad_path), static_cast<float *>(workspace), st);
        return closure_sig_backward<double>(*desc, lt, static_cast<const double *>(path),
                                            static_cast<const double *>(sig), static_cast<const double *>(grad_sig),
                                            static_cast<double *>(grad_path), static_cast<double *>(workspace), st);
    }
    if (family == Family::kTiled) {
        if (desc->dtype == PSIG_F32)
            return tiled_sig_backward<float>(*desc, static_cast<const float *>(path), static_cast<const float *>(sig),
                                             static_cast<const float *>(grad_sig), static_cast<float *>(grad_path),
                                             workspace, st);
        return tiled_sig_backward<double>(*desc, static_cast<const double *>(path), static_cast<const double *>(sig),
                                          static_cast<const double *>(grad_sig), static_cast<double *>(grad_path),
                                          workspace, st);
    }
    if (desc->dtype == PSIG_F32)
        return generic_sig_backward<float>(*desc, lt, static_cast<const float *>(path),
                                           static_cast<const float *>(sig), static_cast<const float *>(grad_sig),
                                           static_cast<float *>(grad_path), static_cast<float *>(workspace), st);
    return generic_sig_backward<double>(*desc, lt, static_cast<const double *>(path),
                                        static_cast<const double *>(sig), static_cast<const double *>(grad_sig),
                                        static_cast<double *>(grad_path), static_cast<double *>(workspace), st);
}

int psig_logsig_forward(const PsigLogDesc *desc, const void *sig, void *logsig, void *cache, void *stream)
{
    LevelTable lt;
    const int rc = log_table(desc, &lt);
    if (rc != PSIG_OK) return rc;
    if (desc->rows == 0 || lt.total == 0) return PSIG_OK;
    if (!sig || !logsig || (!cache && psig_logsig_cache_size(desc) > 0)) return PSIG_ERR_NULL;
    if (desc->lower_columns != nullptr && !horner_logsig_supported(*desc, lt)) return PSIG_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (desc->dtype == PSIG_F32)
        return generic_logsig_forward<float>(*desc, lt, static_cast<const float *>(sig), static_cast<float *>(logsig),
                                             static_cast<float *>(cache), st);
    return generic_logsig_forward<double>(*desc, lt, static_cast<const double *>(sig), static_cast<double *>(logsig),
                                          static_cast<double *>(cache), st);
}

int64_t psig_logsig_cache_size(const PsigLogDesc *desc)
{
    LevelTable lt;
    const int rc = log_table(desc, &lt);
    if (rc != PSIG_OK) return rc;
    return horner_logsig_supported(*desc, lt) ? 0 : lt.total * desc->depth;
}

int64_t psig_logsig_backward_workspace(const PsigLogDesc *desc)
{
    LevelTable lt;
    const int rc = log_table(desc, &lt);
    if (rc != PSIG_OK) return rc;
    if (horner_logsig_supported(*desc, lt)) return 0;  // the row-in-shared-memory form needs none
    const long long scalars = streamed_logsig_backward_scratch(*desc, lt);
    if (scalars < 0) return PSIG_ERR_TOO_LARGE;
    return (int64_t)dtype_size(desc->dtype) * scalars;
}

int psig_logsig_backward(const PsigLogDesc *desc, const void *sig, const void *cache, const void *grad_logsig,
                         void *grad_sig, void *workspace, int64_t workspace_bytes, void *stream)
{
    LevelTable lt;
    const int rc = log_table(desc, &lt);
    if (rc != PSIG_OK) return rc;
    if (desc->rows == 0 || lt.total == 0) return PSIG_OK;
    if (!sig || !grad_logsig || !grad_sig || (!cache && psig_logsig_cache_size(desc) > 0)) return PSIG_ERR_NULL;
    if (desc->lower_columns != nullptr && !horner_logsig_supported(*desc, lt)) return PSIG_ERR_UNSUPPORTED;
    const int64_t need = psig_logsig_backward_workspace(desc);
    if (need > 0 && (!workspace || workspace_bytes < need)) return PSIG_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (desc->dtype == PSIG_F32)
        return generic_logsig_backward<float>(*desc, lt, static_cast<const float *>(sig),
                                              static_cast<const float *>(cache),
                                              static_cast<const float *>(grad_logsig), static_cast<float *>(grad_sig),
                                              static_cast<float *>(workspace), st);
    return generic_logsig_backward<double>(*desc, lt, static_cast<const double *>(sig),
                                           static_cast<const double *>(cache),
                                           static_cast<const double *>(grad_logsig), static_cast<double *>(grad_sig),
                                           static_cast<double *>(workspace), st);
}

}  // extern "C"
