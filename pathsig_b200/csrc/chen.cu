// Chen product of truncated signatures in word coordinates (dense layout, float32 / float64).
//
//   (A (x) B)(w) = A(w) + B(w) + sum_{0<k<|w|} A(w[:k]) * B(w[k:])
//
// A and B are rows of signature coordinates of degrees 1..depth (the degree-0 coordinate is 1 and
// is not stored), so the product is the signature of the concatenation of the two paths (Chen's
// identity).  The reference has no such operator; its windows and batches are always recomputed
// from the increments (src/pathsig/forward/sig_kernels.cu:116-157).
//
// Forward: one thread per output word, |w|-1 gathered multiply-adds.  Backward is written as a
// gather as well (no atomics, deterministic):
//   dA(u) = G(u) + sum_{m=1}^{N-|u|} sum_{|v|=m} G(u.v) * B(v)      (contiguous runs of G)
//   dB(v) = G(v) + sum_{k=1}^{N-|v|} sum_{|u|=k} A(u)   * G(u.v)
// Words of low degree have long sums and are few: those are given a whole warp (lanes stride the
// run, shuffle reduction); the others one thread each.
#include "common.cuh"

namespace psig {
namespace {

constexpr int kChenBlock = 256;
constexpr long long kChenWarpRun = 96;  // sums at least this long get a warp

struct ChenPlan {
    int d, depth;
    long long rows, total;
    long long off[kMaxDepth + 2];   // off[k] = start of degree k in a row; off[depth+1] = total
    long long dpow[kMaxDepth + 1];  // d^k
    int warp_depth;                 // words of degree <= warp_depth are handled by a warp in backward
    long long warp_words;           // number of such words per side
};

__device__ __forceinline__ int degree_of(const ChenPlan &p, long long i)
{
    int n = 1;
    while (n < p.depth && i >= p.off[n + 1]) ++n;
    return n;
}

template <typename T>
__global__ void __launch_bounds__(kChenBlock) chen_forward_rows(const ChenPlan p, const T *__restrict__ a,
                                                                const T *__restrict__ b, T *__restrict__ out)
{
    for (long long row = blockIdx.y; row < p.rows; row += gridDim.y) {
        const T *ar = a + row * p.total;
        const T *br = b + row * p.total;
        T *orow = out + row * p.total;
        for (long long i = (long long)blockIdx.x * kChenBlock + threadIdx.x; i < p.total;
             i += (long long)gridDim.x * kChenBlock) {
            const int n = degree_of(p, i);
            const long long code = i - p.off[n];
            T acc = ar[i] + br[i];
            for (int k = 1; k < n; ++k) {
                const long long dm = p.dpow[n - k];
                acc = fma(ar[p.off[k] + code / dm], br[p.off[n - k] + code % dm], acc);
            }
            orow[i] = acc;
        }
    }
}

// Item numbering per row: [0, 2*warp_words) are warp items (side = item / warp_words), each taking
// 32 consecutive threads; the remaining words of both sides take one thread each.
template <typename T>
__global__ void __launch_bounds__(kChenBlock) chen_backward_rows(const ChenPlan p, const T *__restrict__ a,
                                                                 const T *__restrict__ b, const T *__restrict__ g,
                                                                 T *__restrict__ ga, T *__restrict__ gb)
{
    const long long warp_threads = 64 * p.warp_words;  // 2 sides * 32 lanes
    const long long thread_words = p.total - p.warp_words;
    const long long row_threads = warp_threads + 2 * thread_words;
    for (long long row = blockIdx.y; row < p.rows; row += gridDim.y) {
        const T *ar = a + row * p.total;
        const T *br = b + row * p.total;
        const T *gr = g + row * p.total;
        T *gar = ga + row * p.total;
        T *gbr = gb + row * p.total;
        // row_threads rounded up to whole warps, so that a warp is either all warp items or all
        // thread items and the shuffles below see full warps
        const long long span = (row_threads + 31) / 32 * 32;
        for (long long t = (long long)blockIdx.x * kChenBlock + threadIdx.x; t < span;
             t += (long long)gridDim.x * kChenBlock) {
            const bool team = t < warp_threads;
            long long word;
            int side, lane, stride;
            if (team) {
                const long long item = t >> 5;
                side = item >= p.warp_words ? 1 : 0;
                word = item - side * p.warp_words;
                lane = (int)(t & 31);
                stride = 32;
            } else {
                const long long item = t - warp_threads;
                side = item >= thread_words ? 1 : 0;
                word = p.warp_words + item - side * thread_words;
                lane = 0;
                stride = 1;
            }
            const bool live = team || t < row_threads;
            T acc = T(0);
            int n = 1;
            long long code = 0;
            if (live) {
                n = degree_of(p, word);
                code = word - p.off[n];
                if (side == 0) {
                    // dA(u), |u| = n: runs G[off[n+m] + code*d^m + v] * B[off[m] + v]
                    for (int m = 1; n + m <= p.depth; ++m) {
                        const long long dm = p.dpow[m];
                        const T *grun = gr + p.off[n + m] + code * dm;
                        const T *brun = br + p.off[m];
                        for (long long v = lane; v < dm; v += stride) acc = fma(grun[v], brun[v], acc);
                    }
                } else {
                    // dB(v), |v| = n: A[off[k] + u] * G[off[k+n] + u*d^n + code]
                    const long long dn = p.dpow[n];
                    for (int k = 1; k + n <= p.depth; ++k) {
                        const long long dk = p.dpow[k];
                        const T *arun = ar + p.off[k];
                        const T *gcol = gr + p.off[k + n] + code;
                        for (long long u = lane; u < dk; u += stride) acc = fma(arun[u], gcol[u * dn], acc);
                    }
                }
            }
            if (team) {
#pragma unroll
                for (int s = 16; s >= 1; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
            }
            if (live && lane == 0) {
                acc += gr[word];
                if (side == 0) gar[word] = acc;
                else gbr[word] = acc;
            }
        }
    }
}

int make_chen_plan(const PsigChenDesc &desc, ChenPlan *plan)
{
    ChenPlan &p = *plan;
    p.d = desc.d;
    p.depth = desc.depth;
    p.rows = desc.rows;
    p.dpow[0] = 1;
    p.off[0] = 0;
    p.off[1] = 0;
    const long long limit = (1LL << 62);
    for (int k = 1; k <= kMaxDepth; ++k) {
        if (k <= desc.depth) {
            if (p.dpow[k - 1] > limit / desc.d) return PSIG_ERR_PACKING;
            p.dpow[k] = p.dpow[k - 1] * desc.d;
            p.off[k + 1] = p.off[k] + p.dpow[k];
        } else {
            p.dpow[k] = 0;
            p.off[k + 1] = p.off[desc.depth + 1];
        }
    }
    p.total = p.off[desc.depth + 1];
    // the sum of a word of degree n runs over sum_{m=1}^{depth-n} d^m terms
    p.warp_depth = 0;
    p.warp_words = 0;
    for (int n = 1; n <= desc.depth; ++n) {
        long long run = 0;
        for (int m = 1; n + m <= desc.depth; ++m) run += p.dpow[m];
        if (run >= kChenWarpRun) {
            p.warp_depth = n;
            p.warp_words = p.off[n + 1];
        }
    }
    return PSIG_OK;
}

int check_chen(const PsigChenDesc *desc)
{
    if (desc == nullptr) return PSIG_ERR_NULL;
    if (desc->dtype != PSIG_F32 && desc->dtype != PSIG_F64) return PSIG_ERR_DTYPE;
    if (desc->depth < 1 || desc->depth > kMaxDepth) return PSIG_ERR_DEPTH;
    if (desc->d < 1 || desc->rows < 0) return PSIG_ERR_SHAPE;
    return PSIG_OK;
}

unsigned grid_y(long long rows) { return (unsigned)(rows < 65535 ? rows : 65535); }

template <typename T>
int chen_forward(const ChenPlan &p, const void *a, const void *b, void *out, cudaStream_t stream)
{
    long long bx = (p.total + kChenBlock - 1) / kChenBlock;
    if (bx > 4096) bx = 4096;
    const dim3 grid((unsigned)bx, grid_y(p.rows));
    chen_forward_rows<T><<<grid, kChenBlock, 0, stream>>>(p, static_cast<const T *>(a), static_cast<const T *>(b),
                                                         static_cast<T *>(out));
    return check_launch();
}

template <typename T>
int chen_backward(const ChenPlan &p, const void *a, const void *b, const void *g, void *ga, void *gb,
                  cudaStream_t stream)
{
    const long long row_threads = 64 * p.warp_words + 2 * (p.total - p.warp_words);
    long long bx = (row_threads + kChenBlock - 1) / kChenBlock;
    if (bx > 4096) bx = 4096;
    const dim3 grid((unsigned)bx, grid_y(p.rows));
    chen_backward_rows<T><<<grid, kChenBlock, 0, stream>>>(p, static_cast<const T *>(a), static_cast<const T *>(b),
                                                          static_cast<const T *>(g), static_cast<T *>(ga),
                                                          static_cast<T *>(gb));
    return check_launch();
}

}  // namespace
}  // namespace psig

using namespace psig;

extern "C" int64_t psig_chen_size(const PsigChenDesc *desc)
{
    const int rc = check_chen(desc);
    if (rc != PSIG_OK) return rc;
    ChenPlan p;
    const int rp = make_chen_plan(*desc, &p);
    return rp != PSIG_OK ? rp : p.total;
}

extern "C" int psig_chen_forward(const PsigChenDesc *desc, const void *a, const void *b, void *out, void *stream)
{
    const int rc = check_chen(desc);
    if (rc != PSIG_OK) return rc;
    if (desc->rows == 0) return PSIG_OK;
    if (a == nullptr || b == nullptr || out == nullptr) return PSIG_ERR_NULL;
    ChenPlan p;
    const int rp = make_chen_plan(*desc, &p);
    if (rp != PSIG_OK) return rp;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return desc->dtype == PSIG_F32 ? chen_forward<float>(p, a, b, out, s) : chen_forward<double>(p, a, b, out, s);
}

extern "C" int psig_chen_backward(const PsigChenDesc *desc, const void *a, const void *b, const void *grad_out,
                                  void *grad_a, void *grad_b, void *stream)
{
    const int rc = check_chen(desc);
    if (rc != PSIG_OK) return rc;
    if (desc->rows == 0) return PSIG_OK;
    if (a == nullptr || b == nullptr || grad_out == nullptr || grad_a == nullptr || grad_b == nullptr)
        return PSIG_ERR_NULL;
    ChenPlan p;
    const int rp = make_chen_plan(*desc, &p);
    if (rp != PSIG_OK) return rp;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return desc->dtype == PSIG_F32 ? chen_backward<float>(p, a, b, grad_out, grad_a, grad_b, s)
                                   : chen_backward<double>(p, a, b, grad_out, grad_a, grad_b, s);
}
