// Signature <-> log-signature in word coordinates (generic: any d, depth, dense or projected
// top degree, float32 / float64).
//
//   log S = sum_{m>=1} (-1)^(m+1) (S-1)^{(x)m} / m,
//   P_1(w) = S(w),  P_m(w) = sum_{k=m-1}^{n-1} P_{m-1}(w[:k]) * S(w[k:])      (n = |w|)
//
// which is the recursion of the reference (src/pathsig/forward/sig_kernels.cu:214-240) and its
// adjoint (src/pathsig/backward/sig_backward_kernels.cu:449-476).  Unlike the reference, which
// launches one kernel per degree because degree n reads the P values of shorter prefixes
// (src/pathsig/forward/sig_launch.cu:300-335), one thread block walks all degrees of one row
// with a block barrier in between, so a row is one launch and its P values stay in L2/L1.
#include "common.cuh"

namespace psig {
namespace {

constexpr int kLogBlock = 256;

struct LogPlan {
    LevelTable lt;
    long long rows;
    long long dpow[kMaxDepth + 1];
};

// Row positions of the proper prefixes and suffixes of word `code` (|w| = N):
//   pref[i] = position of w[:i], suf[i] = position of w[N-i:]   (i = 1..N-1, both dense degrees).
// IDX is a 32-bit type when every code and row position fits (64-bit integer division costs an
// order of magnitude more than the arithmetic of a word); one division by d per prefix.
template <typename IDX, int N>
__device__ __forceinline__ void split_word(const LogPlan &p, IDX code, IDX (&pref)[N + 1], IDX (&suf)[N + 1])
{
    const IDX d = (IDX)p.lt.d;
    IDX q = code;
#pragma unroll
    for (int i = N - 1; i >= 1; --i) {
        q /= d;  // code / d^(N-i)
        pref[i] = (IDX)p.lt.dense_offset[i] + q;
        suf[N - i] = (IDX)p.lt.dense_offset[N - i] + (code - q * (IDX)p.dpow[N - i]);
    }
}

template <typename T, typename IDX, int N>
__device__ __forceinline__ void logsig_word_forward(const LogPlan &p, long long idx, const T *__restrict__ sig,
                                                    T *__restrict__ P, T *__restrict__ logsig)
{
    const int depth = p.lt.depth;
    const IDX code = (IDX)(p.lt.words[N] ? p.lt.words[N][idx] : idx);
    T suf[N + 1];
    IDX pref_ind[N + 1], suf_ind[N + 1];
    split_word<IDX, N>(p, code, pref_ind, suf_ind);
#pragma unroll
    for (int i = 1; i < N; ++i) suf[i] = sig[suf_ind[i]];
    pref_ind[N] = (IDX)(p.lt.offset[N] + idx);
    suf[N] = sig[pref_ind[N]];
    const long long P_off = (long long)pref_ind[N] * depth;
    P[P_off] = suf[N];
    T lw = suf[N];
#pragma unroll
    for (int m = 2; m <= N; ++m) {
        T acc = T(0);
#pragma unroll
        for (int k = m - 1; k < N; ++k) acc = fma(P[(long long)pref_ind[k] * depth + (m - 2)], suf[N - k], acc);
        const T coeff = (m & 1) ? recip<T>(m) : -recip<T>(m);
        lw = fma(coeff, acc, lw);
        P[P_off + (m - 1)] = acc;
    }
    logsig[pref_ind[N]] = lw;
}

template <typename T, typename IDX, int N>
__device__ __forceinline__ void logsig_word_backward(const LogPlan &p, long long idx, const T *__restrict__ sig,
                                                     const T *__restrict__ P, const T *__restrict__ glog,
                                                     T *__restrict__ gsig, T *__restrict__ gP)
{
    const int depth = p.lt.depth;
    const IDX code = (IDX)(p.lt.words[N] ? p.lt.words[N][idx] : idx);
    IDX pref_ind[N + 1], suf_ind[N + 1];
    split_word<IDX, N>(p, code, pref_ind, suf_ind);
    const long long wg = p.lt.offset[N] + idx;
    const T g = glog[wg];
    T gPv[N];
#pragma unroll
    for (int m = 1; m <= N; ++m) {
        const T coeff = (m & 1) ? recip<T>(m) : -recip<T>(m);
        gPv[m - 1] = fma(coeff, g, gP[wg * depth + (m - 1)]);
    }
    atomicAdd(&gsig[wg], gPv[0]);
#pragma unroll
    for (int m = 2; m <= N; ++m) {
#pragma unroll
        for (int k = m - 1; k < N; ++k) {
            const long long pi = (long long)pref_ind[k], si = (long long)suf_ind[N - k];
            atomicAdd(&gP[pi * depth + (m - 2)], gPv[m - 1] * sig[si]);
            atomicAdd(&gsig[si], gPv[m - 1] * P[pi * depth + (m - 2)]);
        }
    }
}

#define PSIG_SWITCH_DEGREE(k, CALL)                                   \
    switch (k) {                                                      \
        case 1: { constexpr int N = 1; CALL; } break;                 \
        case 2: { constexpr int N = 2; CALL; } break;                 \
        case 3: { constexpr int N = 3; CALL; } break;                 \
        case 4: { constexpr int N = 4; CALL; } break;                 \
        case 5: { constexpr int N = 5; CALL; } break;                 \
        case 6: { constexpr int N = 6; CALL; } break;                 \
        case 7: { constexpr int N = 7; CALL; } break;                 \
        case 8: { constexpr int N = 8; CALL; } break;                 \
        case 9: { constexpr int N = 9; CALL; } break;                 \
        case 10: { constexpr int N = 10; CALL; } break;               \
        case 11: { constexpr int N = 11; CALL; } break;               \
        default: { constexpr int N = 12; CALL; } break;               \
    }

template <typename T, typename IDX>
__global__ void __launch_bounds__(kLogBlock) logsig_forward_rows(const LogPlan p, const T *__restrict__ sig,
                                                                 T *__restrict__ logsig, T *__restrict__ P)
{
    const long long S = p.lt.total;
    for (long long row = blockIdx.x; row < p.rows; row += gridDim.x) {
        const T *s = sig + row * S;
        T *l = logsig + row * S;
        T *c = P + row * S * p.lt.depth;
        for (int n = 1; n <= p.lt.depth; ++n) {
            for (long long idx = threadIdx.x; idx < p.lt.size[n]; idx += kLogBlock) {
                PSIG_SWITCH_DEGREE(n, (logsig_word_forward<T, IDX, N>(p, idx, s, c, l)));
            }
            __syncthreads();
        }
    }
}

template <typename T, typename IDX>
__global__ void __launch_bounds__(kLogBlock) logsig_backward_rows(const LogPlan p, const T *__restrict__ sig,
                                                                  const T *__restrict__ P,
                                                                  const T *__restrict__ glog,
                                                                  T *__restrict__ gsig, T *__restrict__ gP)
{
    const long long S = p.lt.total;
    for (long long row = blockIdx.x; row < p.rows; row += gridDim.x) {
        const T *s = sig + row * S;
        const T *c = P + row * S * p.lt.depth;
        const T *gl = glog + row * S;
        T *gs = gsig + row * S;
        T *gc = gP + row * S * p.lt.depth;
        for (int n = p.lt.depth; n >= 1; --n) {
            for (long long idx = threadIdx.x; idx < p.lt.size[n]; idx += kLogBlock) {
                PSIG_SWITCH_DEGREE(n, (logsig_word_backward<T, IDX, N>(p, idx, s, c, gl, gs, gc)));
            }
            __syncthreads();
        }
    }
}

LogPlan make_log_plan(const PsigLogDesc &desc, const LevelTable &lt)
{
    LogPlan p;
    p.lt = lt;
    p.rows = desc.rows;
    p.dpow[0] = 1;
    for (int k = 1; k <= kMaxDepth; ++k) p.dpow[k] = (k <= lt.depth) ? p.dpow[k - 1] * lt.d : 0;
    return p;
}

// Word codes (< d^depth) and positions inside a row both fit 32 bits.
bool narrow_indices(const LogPlan &p)
{
    return p.dpow[p.lt.depth] > 0 && p.dpow[p.lt.depth] <= 0x7fffffffLL && p.lt.total <= 0x7fffffffLL;
}

}  // namespace

template <typename T>
int generic_logsig_forward(const PsigLogDesc &desc, const LevelTable &lt, const T *sig, T *logsig, T *cache,
                           cudaStream_t stream)
{
    if (desc.rows == 0 || lt.total == 0) return PSIG_OK;
    if (horner_logsig_supported(desc, lt)) return horner_logsig_forward<T>(desc, lt, sig, logsig, stream);
    const LogPlan p = make_log_plan(desc, lt);
    const unsigned grid = (unsigned)(desc.rows < (1 << 20) ? desc.rows : (1 << 20));
    if (narrow_indices(p)) logsig_forward_rows<T, unsigned><<<grid, kLogBlock, 0, stream>>>(p, sig, logsig, cache);
    else logsig_forward_rows<T, long long><<<grid, kLogBlock, 0, stream>>>(p, sig, logsig, cache);
    return check_launch();
}

template <typename T>
int generic_logsig_backward(const PsigLogDesc &desc, const LevelTable &lt, const T *sig, const T *cache,
                            const T *grad_logsig, T *grad_sig, T *grad_cache_ws, cudaStream_t stream)
{
    if (desc.rows == 0 || lt.total == 0) return PSIG_OK;
    if (horner_logsig_supported(desc, lt))
        return horner_logsig_backward<T>(desc, lt, sig, grad_logsig, grad_sig, stream);
    const LogPlan p = make_log_plan(desc, lt);
    const size_t row_bytes = sizeof(T) * (size_t)lt.total;
    if (cudaMemsetAsync(grad_sig, 0, row_bytes * desc.rows, stream) != cudaSuccess) return PSIG_ERR_CUDA;
    if (cudaMemsetAsync(grad_cache_ws, 0, row_bytes * desc.rows * lt.depth, stream) != cudaSuccess)
        return PSIG_ERR_CUDA;
    const unsigned grid = (unsigned)(desc.rows < (1 << 20) ? desc.rows : (1 << 20));
    if (narrow_indices(p))
        logsig_backward_rows<T, unsigned><<<grid, kLogBlock, 0, stream>>>(p, sig, cache, grad_logsig, grad_sig,
                                                                         grad_cache_ws);
    else
        logsig_backward_rows<T, long long><<<grid, kLogBlock, 0, stream>>>(p, sig, cache, grad_logsig, grad_sig,
                                                                          grad_cache_ws);
    return check_launch();
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
