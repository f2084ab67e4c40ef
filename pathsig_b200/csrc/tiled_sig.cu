// Register-tiled dense signature kernels (compile-time channel count D and depth N).
//
// The word tree is cut at a prefix length P.  One thread owns a prefix u (|u| = P) and, of the
// sub-tree below it, the DA first letters [a0, a0+DA): the values S(u.a), S(u.a.b), ... down
// to degree N live in registers (DA * (1 + D + ... ) scalars), the P values S(u[:j]) on the
// way to the root are kept redundantly by every thread that shares them.  One step of Chen's
// recurrence S <- S (x) exp(dx) is then, per target degree k, a Horner chain
//     B_j = B_{j-1} * dx[w_j] / (k-j+1) + S_j         (j = 1..k-1),   S_k += B_{k-1} * dx[w_k]
// whose scalar head (j <= P) costs P FMAs and whose tail is pure register FMA over the owned
// sub-tree: no shared-memory state, no barrier and no shuffle inside the step loop.  Shared
// prefixes are evaluated once per thread instead of once per word as in the reference
// (src/pathsig/forward/sig_kernels.cu:138-152), which is where the ~8x arithmetic saving at
// (d, depth) = (8, 4) comes from.  Increments are staged in shared memory a chunk of steps at a
// time; the factors 1/2, 1/3 of the Horner tail ride on the scalar multiplier.
//
// Backward is reverse-mode through the same recurrence.  Going back one step, degrees are
// visited bottom-up: the Horner values are rebuilt from the already rolled-back lower
// degrees, S_k is rolled back by subtracting exactly the term the forward step added (the top
// degree is never needed and is not tracked), and the adjoint G is pushed through the
// transposed chain, which also yields this thread's share of dL/d(dx_t).  Adjoints of the
// shared prefixes are kept as per-thread partial sums (everything downstream of them is
// linear), so the only cross-thread traffic is the per-step sum of the D-vector dL/d(dx_t)
// over the threads of a unit; it goes through shared memory in chunks of steps.  The reference
// instead evaluates an O(depth^3) two-sided product per word and reduces with warp shuffles and
// global atomics every step (src/pathsig/backward/sig_backward_kernels.cu:204-318).
//
// The kernels are written once, in tiled_sig_impl.inc, against a scalar type `real`; this file
// compiles them for float32 and for float64 (packed two-lane FMAs and the per-shape tuning exist for
// float32 only) and dispatches on the dtype of the description.
#include "common.cuh"

#include <algorithm>
#include <cstdint>
#include <type_traits>

namespace psig {
namespace {

__host__ __device__ constexpr int ipow(int b, int e) { int r = 1; for (int i = 0; i < e; ++i) r *= b; return r; }
__host__ __device__ constexpr int at_least_one(int n) { return n > 0 ? n : 1; }

namespace f32 {
using real = float;
constexpr int VEC = 4;  // scalars per 16-byte access
struct __align__(16) vec_t { real v[VEC]; };
#define PSIG_REAL_IS_DOUBLE 0
#include "tiled_sig_impl.inc"
#undef PSIG_REAL_IS_DOUBLE
}  // namespace f32

namespace f64 {
using real = double;
constexpr int VEC = 2;
struct __align__(16) vec_t { real v[VEC]; };
#define PSIG_REAL_IS_DOUBLE 1
#include "tiled_sig_impl.inc"
#undef PSIG_REAL_IS_DOUBLE
}  // namespace f64

}  // namespace

bool tiled_supported(const PsigSigDesc &desc)
{
    return desc.dtype == PSIG_F32 ? f32::tiled_supported(desc) : f64::tiled_supported(desc);
}

int64_t tiled_sig_backward_workspace(const PsigSigDesc &desc)
{
    return desc.dtype == PSIG_F32 ? f32::backward_scratch_bytes(desc, nullptr) : f64::backward_scratch_bytes(desc, nullptr);
}

bool tiled_sig_backward_reproducible(const PsigSigDesc &desc)
{
    bool repro = false;
    if (desc.dtype == PSIG_F32) f32::backward_scratch_bytes(desc, &repro); else f64::backward_scratch_bytes(desc, &repro);
    return repro;
}

int tiled_top_plan(const PsigSigDesc &desc, bool backward, unsigned char *items, int *active)
{
    return desc.dtype == PSIG_F32 ? f32::top_plan_of(desc, backward, items, active)
                                  : f64::top_plan_of(desc, backward, items, active);
}

int tiled_set_bulk_wait_polls(int polls)
{
    const int rc = f32::bulk_wait_control(true, polls, nullptr);
    return rc != PSIG_OK ? rc : f64::bulk_wait_control(true, polls, nullptr);
}

long long tiled_bulk_copy_timeouts()
{
    unsigned int a = 0, b = 0;
    if (f32::bulk_wait_control(false, 0, &a) != PSIG_OK || f64::bulk_wait_control(false, 0, &b) != PSIG_OK)
        return PSIG_ERR_CUDA;
    return (long long)a + (long long)b;
}

template <>
int tiled_sig_forward<float>(const PsigSigDesc &desc, const float *path, float *out, cudaStream_t stream)
{
    return f32::tiled_sig_forward(desc, path, out, stream);
}
template <>
int tiled_sig_forward<double>(const PsigSigDesc &desc, const double *path, double *out, cudaStream_t stream)
{
    return f64::tiled_sig_forward(desc, path, out, stream);
}
template <>
int tiled_sig_backward<float>(const PsigSigDesc &desc, const float *path, const float *sig, const float *grad,
                              float *grad_path, void *workspace, cudaStream_t stream)
{
    return f32::tiled_sig_backward(desc, path, sig, grad, grad_path, workspace, stream);
}
template <>
int tiled_sig_backward<double>(const PsigSigDesc &desc, const double *path, const double *sig, const double *grad,
                               double *grad_path, void *workspace, cudaStream_t stream)
{
    return f64::tiled_sig_backward(desc, path, sig, grad, grad_path, workspace, stream);
}

}  // namespace psig
