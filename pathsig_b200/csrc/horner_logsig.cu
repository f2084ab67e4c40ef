// Signature <-> log-signature with the row held in shared memory (float32 / float64).
//
// With x = S - 1 (degrees 1..N of the signature), the truncated logarithm is evaluated in Horner
// form instead of through the powers P_m = x^{(x)m} that the reference stores
// (src/pathsig/forward/sig_kernels.cu:214-240):
//
//   T_N = 1/N,   T_k = 1/k - x (x) T_{k+1}  (kept up to degree N-k),   log S = x (x) T_1.
//
// A product with x in word coordinates is (x (x) T)(w) = sum_{j=1}^{|w|} x(w[:j]) T(w[j:]), so only
// degrees below N of x and of the T_k are ever re-read: they live in shared memory (two or three
// copies of sum_{n<N} d^n scalars), the top degree of the row streams through once, and the
// (rows, S*depth) array of powers is neither written nor read.  One thread block per row.
//
// Backward is the adjoint of the same recurrences, written as gathers (contiguous runs of the
// incoming gradient, no atomics) except for the words of a projected top degree, which scatter
// with shared-memory atomics.  The T_k are recomputed, not stored.
//
// Rows whose lower degrees do not fit shared memory run the same kernels in "streamed" form: the buffers
// are per-row scratch in global memory (the caller's cache / workspace) and x is read from the signature
// row itself.  Word codes and row positions must fit 32 bits (rows below 2^31 scalars).
#include "common.cuh"

namespace psig {
namespace {

constexpr int kHornerBlock = 256;
// Backward, row in shared memory, few rows (at most eight per SM): config 4's 1 024 rows 0.113 -> 0.103 ms;
// 512 threads 0.105 ms; at 15 616 rows of dense (8,4) both are 20 % slower than 256.
constexpr int kHornerWideBlock = 384;
// The streamed form may run a row on a wider block when there are fewer rows than SMs can take.
constexpr int kStreamedMaxBlock = 1024;
// Resident blocks per SM the forward kernel is compiled for.  A row is a chain of short phases with a
// barrier each, so rows in flight per SM matter more than registers per thread (measured: 6 blocks
// against 2 cut the forward time by 40 %); the values below are the largest that do not spill.
template <typename T, int NMAX> constexpr int forward_blocks_per_sm()
{
    return sizeof(T) == 4 ? (NMAX <= 4 ? 8 : NMAX <= 8 ? 6 : 4) : 4;
}
constexpr size_t kHornerMaxSmem = 160 * 1024;
// Balance of the backward gathers: a word whose sum has at least kTeamTerms terms gets a warp (lanes stride the
// sum), shorter sums get a thread; sums over the first factor are cut into pieces of kPieceTerms terms.  With a
// warp only for sums of 96+ terms and pieces of 64, a few threads ran serial loops of 64-84 terms while the rest
// of the block waited at the phase barrier.
// Measured (config 4 at 1 024 rows / dense (8,4) at 15 616 rows): 96/64 0.117/0.772 ms, 48/32 0.111/0.620 ms,
// 32/16 0.110/0.633 ms, 16/8 0.185/0.652 ms.
constexpr unsigned kTeamTerms = 48, kPieceTerms = 32;

// Division of a 32-bit unsigned number by the channel count, which is fixed for a launch: the
// multiply-and-shift form of Granlund & Montgomery ("Division by invariant integers using
// multiplication", 1994) in its branch-free variant, exact for every 32-bit dividend.
struct FastDiv {
    unsigned mul, shift, one;  // one != 0: the divisor is 1
    __host__ void set(unsigned d)
    {
        one = d == 1u ? 1u : 0u;
        unsigned l = 0;
        while ((1ull << l) < d) ++l;  // ceil(log2 d)
        mul = (unsigned)((((1ull << l) - d) << 32) / d + 1ull);
        shift = l > 0 ? l - 1u : 0u;
    }
    __device__ __forceinline__ unsigned div(unsigned n) const
    {
        const unsigned t = __umulhi(n, mul);
        const unsigned q = (((n - t) >> 1) + t) >> shift;
        return one ? n : q;
    }
};

struct HornerPlan {
    FastDiv by_d;
    int d, depth;
    long long rows, width;       // row width S = lower + top
    unsigned lower;              // A = sum_{n<N} d^n: scalars of the dense degrees below the top
    unsigned top;                // words kept at degree N
    const long long *top_words;  // device codes, or nullptr when the top degree is dense
    unsigned off[kMaxDepth + 2];   // off[n] = start of degree n in a dense row; off[N] = lower
    unsigned dpow[kMaxDepth + 1];  // d^k (k < N; d^N only when it fits)
    unsigned t_off[kMaxDepth + 1];  // backward: start of T_k (degrees 1..N-k) in the T area
    unsigned t_total;
    unsigned stage_top;  // backward: hold a dense image of the top degree of the incoming gradient in shared memory
    unsigned top_dense;  // d^N (0 when it does not fit 31 bits)
    // Projected output: only these positions of the dense degrees below the top are written (forward) /
    // carry an incoming gradient (backward), followed by the whole top degree.  nullptr: every position.
    const long long *low_cols;
    unsigned n_low;      // entries of low_cols
    unsigned out_lower;  // columns of the output row ahead of the top degree: n_low, or `lower`
    long long out_width;  // out_lower + top
};

// Four scalars moved as one access (16 bytes of float, 32 of double).
template <typename T> struct __align__(4 * sizeof(T)) Quad { T v[4]; };

__device__ __forceinline__ int degree_at(const HornerPlan &p, unsigned i, int max_degree)
{
    int n = 1;
    while (n < max_degree && i >= p.off[n + 1]) ++n;
    return n;
}

// sum_{j=1}^{n-1} x(w[:j]) * t(w[j:]) for the word `code` of degree n; xs and ts are dense rows of the
// degrees below N (ts without its degree-0 term).
template <typename T>
__device__ __forceinline__ T split_sum(const HornerPlan &p, const T *xs, const T *ts, int n, unsigned code)
{
    T acc = T(0);
    unsigned q = code;
    for (int len = 1; len < n; ++len) {  // len = length of the suffix
        q = p.by_d.div(q);               // code of the prefix of length n - len
        const unsigned suf = code - q * p.dpow[len];
        acc = fma(xs[p.off[n - len] + q], ts[p.off[len] + suf], acc);
    }
    return acc;
}

// The same sums for all d children u.a of one parent word u (degree NDEG-1 >= 1) at once: the
// prefixes of the children are the prefixes of u, and their suffixes differ only in the last letter,
// so the x factors and the positions are worked out once per parent and the loop over a is N-1
// shared-memory loads and multiply-adds per word.  emit(a, sum) receives each child's sum.
template <typename T, int NDEG, class F>
__device__ __forceinline__ void children_sums(const HornerPlan &p, const T *xs, const T *ts, unsigned u, F &&emit)
{
    T xp[NDEG - 1];
    unsigned sb[NDEG - 1];
    unsigned q = u;
#pragma unroll
    for (int lp = 0; lp <= NDEG - 2; ++lp) {  // lp letters of u go to the suffix
        const unsigned rem = u - q * p.dpow[lp];  // q = u / d^lp, rem = u % d^lp
        xp[lp] = xs[p.off[NDEG - 1 - lp] + q];
        sb[lp] = p.off[lp + 1] + rem * (unsigned)p.d;
        q = p.by_d.div(q);
    }
    for (unsigned a = 0; a < (unsigned)p.d; ++a) {
        T acc = T(0);
#pragma unroll
        for (int lp = 0; lp <= NDEG - 2; ++lp) acc = fma(xp[lp], ts[sb[lp] + a], acc);
        emit(a, acc);
    }
}

// The same, four children at a time (d a multiple of 4): emit4(a, sums[4]) for a = 0, 4, 8, ...
template <typename T, int NDEG, class F>
__device__ __forceinline__ void children_sums4(const HornerPlan &p, const T *xs, const T *ts, unsigned u, F &&emit4)
{
    T xp[NDEG - 1];
    unsigned sb[NDEG - 1];
    unsigned q = u;
#pragma unroll
    for (int lp = 0; lp <= NDEG - 2; ++lp) {
        const unsigned rem = u - q * p.dpow[lp];
        xp[lp] = xs[p.off[NDEG - 1 - lp] + q];
        sb[lp] = p.off[lp + 1] + rem * (unsigned)p.d;
        q = p.by_d.div(q);
    }
    for (unsigned a = 0; a < (unsigned)p.d; a += 4) {
        T acc[4] = {T(0), T(0), T(0), T(0)};
#pragma unroll
        for (int lp = 0; lp <= NDEG - 2; ++lp) {
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[i] = fma(xp[lp], ts[sb[lp] + a + i], acc[i]);
        }
        emit4(a, acc);
    }
}

// NMAX (a template parameter of the enclosing function) bounds the depth an instance serves: deeper
// cases are not instantiated, which keeps the registers of the shallow instances low.
// One quad of children (a, a+1, a+2, a+3) of parent u: the unit of work when the threads of a warp take
// neighbouring quads, so that their 16-byte shared-memory reads and global accesses are consecutive
// (a thread looping over all children of its own parent reads at a stride of d scalars instead, which
// is an 8-way bank conflict at d = 8).  Needs d % 4 == 0.
template <typename T, int NDEG>
__device__ __forceinline__ void quad_sums(const HornerPlan &p, const T *xs, const T *ts, unsigned u, unsigned a,
                                          T (&acc)[4])
{
    unsigned q = u;
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = T(0);
#pragma unroll
    for (int lp = 0; lp <= NDEG - 2; ++lp) {
        const unsigned rem = u - q * p.dpow[lp];
        const T xp = xs[p.off[NDEG - 1 - lp] + q];
        const Quad<T> tq = *reinterpret_cast<const Quad<T> *>(ts + p.off[lp + 1] + rem * (unsigned)p.d + a);
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i] = fma(xp, tq.v[i], acc[i]);
        q = p.by_d.div(q);
    }
}

#define PSIG_QUAD_CASE(n, ...) \
    case n: if constexpr (n <= NMAX) quad_sums<T, n>(__VA_ARGS__); break;
#define PSIG_QUAD(n, ...)                                                                              \
    switch (n) {                                                                                       \
        PSIG_QUAD_CASE(2, __VA_ARGS__) PSIG_QUAD_CASE(3, __VA_ARGS__) PSIG_QUAD_CASE(4, __VA_ARGS__)   \
        PSIG_QUAD_CASE(5, __VA_ARGS__) PSIG_QUAD_CASE(6, __VA_ARGS__) PSIG_QUAD_CASE(7, __VA_ARGS__)   \
        PSIG_QUAD_CASE(8, __VA_ARGS__) PSIG_QUAD_CASE(9, __VA_ARGS__) PSIG_QUAD_CASE(10, __VA_ARGS__)  \
        PSIG_QUAD_CASE(11, __VA_ARGS__) PSIG_QUAD_CASE(12, __VA_ARGS__)                                \
        default: break;                                                                                \
    }

#define PSIG_CHILD4_CASE(n, ...) \
    case n: if constexpr (n <= NMAX) children_sums4<T, n>(__VA_ARGS__); break;
#define PSIG_CHILDREN4(n, ...)                                                                               \
    switch (n) {                                                                                             \
        PSIG_CHILD4_CASE(2, __VA_ARGS__) PSIG_CHILD4_CASE(3, __VA_ARGS__) PSIG_CHILD4_CASE(4, __VA_ARGS__)   \
        PSIG_CHILD4_CASE(5, __VA_ARGS__) PSIG_CHILD4_CASE(6, __VA_ARGS__) PSIG_CHILD4_CASE(7, __VA_ARGS__)   \
        PSIG_CHILD4_CASE(8, __VA_ARGS__) PSIG_CHILD4_CASE(9, __VA_ARGS__) PSIG_CHILD4_CASE(10, __VA_ARGS__)  \
        PSIG_CHILD4_CASE(11, __VA_ARGS__) PSIG_CHILD4_CASE(12, __VA_ARGS__)                                  \
        default: break;                                                                                      \
    }

#define PSIG_CHILD_CASE(n, ...) \
    case n: if constexpr (n <= NMAX) children_sums<T, n>(__VA_ARGS__); break;
// Dispatch on the children's degree (2..12).
#define PSIG_CHILDREN(n, ...)                                                                             \
    switch (n) {                                                                                          \
        PSIG_CHILD_CASE(2, __VA_ARGS__) PSIG_CHILD_CASE(3, __VA_ARGS__) PSIG_CHILD_CASE(4, __VA_ARGS__)   \
        PSIG_CHILD_CASE(5, __VA_ARGS__) PSIG_CHILD_CASE(6, __VA_ARGS__) PSIG_CHILD_CASE(7, __VA_ARGS__)   \
        PSIG_CHILD_CASE(8, __VA_ARGS__) PSIG_CHILD_CASE(9, __VA_ARGS__) PSIG_CHILD_CASE(10, __VA_ARGS__)  \
        PSIG_CHILD_CASE(11, __VA_ARGS__) PSIG_CHILD_CASE(12, __VA_ARGS__)                                 \
        default: break;                                                                                   \
    }

// emit(position, sum) for every word of degree 2..M (position = its place in a dense row), the block's
// threads taking parents in turn.  M <= N-1 here (words held in shared memory).
template <typename T, int NMAX, class F>
__device__ __forceinline__ void for_words_below_top(const HornerPlan &p, int M, const T *xs, const T *ts, F &&emit)
{
    if (M < 2) return;
    for (unsigned i = threadIdx.x; i < p.off[M]; i += blockDim.x) {  // parents: degrees 1..M-1
        const int m = degree_at(p, i, M - 1);
        const unsigned u = i - p.off[m];
        const unsigned first = p.off[m + 1] + u * (unsigned)p.d;
        PSIG_CHILDREN(m + 1, p, xs, ts, u, [&](unsigned a, T acc) { emit(first + a, acc); })
    }
}

// T_{N-1}, ..., T_1 in turn; T_k is built from T_{k+1} in the other buffer.  On return the result
// T_1 (degrees 1..N-1) is in the buffer the function returns.  `keep`, when not null, receives a
// copy of every T_k at keep + t_off[k].
template <typename T, int NMAX>
__device__ __forceinline__ T *build_t(const HornerPlan &p, const T *xs, T *ta, T *tb, T *keep)
{
    const int N = p.depth;
    T *cur = ta, *nxt = tb;  // cur holds T_{k+1}
    for (int k = N - 1; k >= 1; --k) {
        const T c = T(1) / T(k + 1);  // degree-0 term of T_{k+1}
        T *kept = keep ? keep + p.t_off[k] : nullptr;
        for (unsigned i = threadIdx.x; i < (unsigned)p.d; i += blockDim.x) {  // degree 1: no split
            const T v = -xs[i] * c;
            nxt[i] = v;
            if (kept) kept[i] = v;
        }
        for_words_below_top<T, NMAX>(p, N - k, xs, cur, [&](unsigned pos, T acc) {
            const T v = -fma(xs[pos], c, acc);
            nxt[pos] = v;
            if (kept) kept[pos] = v;
        });
        __syncthreads();
        T *tmp = cur; cur = nxt; nxt = tmp;
    }
    return cur;
}

// STREAMED is a compile-time switch so that the shared-memory instance keeps pointers the compiler knows
// to be shared memory (generic addressing cost it 11-13 %).
template <typename T, int NMAX, bool STREAMED>
__global__ void __launch_bounds__(STREAMED ? kStreamedMaxBlock : kHornerBlock, STREAMED ? 1 : forward_blocks_per_sm<T, NMAX>()) logsig_forward_horner(const HornerPlan p, const T *__restrict__ sig,
                                                                      T *__restrict__ logsig, T *scratch)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    // `scratch` null: the row's lower degrees and the two T buffers live in shared memory.  Otherwise
    // (rows too large for that) x is read from the signature row itself and the T buffers are this
    // row's 2*lower scalars of `scratch` in global memory -- the same code on other pointers.
    T *const xs_copy = reinterpret_cast<T *>(smem_raw);
    const int N = p.depth;
    for (long long row = blockIdx.x; row < p.rows; row += gridDim.x) {
        const T *s = sig + row * p.width;
        T *l = logsig + row * p.out_width;
        const T *xs;
        T *ta;
        if constexpr (STREAMED) { xs = s; ta = scratch + row * 2 * (long long)p.lower; }
        else { xs = xs_copy; ta = xs_copy + p.lower; }
        T *tb = ta + p.lower;
        __syncthreads();  // the previous row's readers are done with the buffers
        if constexpr (!STREAMED)
            for (unsigned i = threadIdx.x; i < p.lower; i += blockDim.x) xs_copy[i] = s[i];
        __syncthreads();
        const T *t1 = build_t<T, NMAX>(p, xs, ta, tb, nullptr);
        // log S = x (x) T_1: degrees below N from shared memory, the top degree streamed
        if (p.low_cols != nullptr) {
            // projected output: only the requested words below the top degree, each from its own splits
            for (unsigned i = threadIdx.x; i < p.n_low; i += blockDim.x) {
                const unsigned pos = (unsigned)p.low_cols[i];
                const int n = degree_at(p, pos, N - 1);
                l[i] = xs[pos] + (n >= 2 ? split_sum(p, xs, t1, n, pos - p.off[n]) : T(0));
            }
        } else {
            if (N >= 2)
                for (unsigned i = threadIdx.x; i < (unsigned)p.d; i += blockDim.x) l[i] = xs[i];
            for_words_below_top<T, NMAX>(p, N - 1, xs, t1, [&](unsigned pos, T acc) { l[pos] = xs[pos] + acc; });
        }
        if (p.top_words == nullptr && N >= 2) {
            // dense top degree: a thread takes a parent of degree N-1 and its d children
            const unsigned parents = p.dpow[N - 1];
            // 4 scalars per access when the runs of d children start on such boundaries
            const bool quads = (p.d & 3) == 0 && (p.lower & 3u) == 0 && (p.width & 3) == 0 &&
                               (p.out_lower & 3u) == 0 && (p.out_width & 3) == 0 &&
                               (reinterpret_cast<uintptr_t>(sig) & (4 * sizeof(T) - 1)) == 0 &&
                               (reinterpret_cast<uintptr_t>(logsig) & (4 * sizeof(T) - 1)) == 0;
            if (quads) {
                // a thread takes one quad of children; neighbouring threads take neighbouring quads
                const unsigned per_parent = (unsigned)p.d / 4u, items = parents * per_parent;
                for (unsigned it = threadIdx.x; it < items; it += blockDim.x) {
                    const unsigned u = it / per_parent, a = 4u * (it - u * per_parent);
                    T acc[4];
                    PSIG_QUAD(N, p, xs, t1, u, a, acc)
                    const size_t pos = (size_t)u * p.d + a;
                    const Quad<T> in = *reinterpret_cast<const Quad<T> *>(s + p.lower + pos);
                    Quad<T> o;
#pragma unroll
                    for (int i = 0; i < 4; ++i) o.v[i] = in.v[i] + acc[i];
                    *reinterpret_cast<Quad<T> *>(l + p.out_lower + pos) = o;
                }
            } else {
                for (unsigned u = threadIdx.x; u < parents; u += blockDim.x) {
                    const T *srun = s + p.lower + (size_t)u * p.d;
                    T *lrun = l + p.out_lower + (size_t)u * p.d;
                    PSIG_CHILDREN(N, p, xs, t1, u, [&](unsigned a, T acc) { lrun[a] = srun[a] + acc; })
                }
            }
        } else {
            for (unsigned i = threadIdx.x; i < p.top; i += blockDim.x) {
                const unsigned code = p.top_words ? (unsigned)p.top_words[i] : i;
                l[p.out_lower + i] = s[p.lower + i] + split_sum(p, xs, t1, N, code);
            }
        }
    }
}

// ---- backward ------------------------------------------------------------------------------

// Adjoint of  Y = X (x) Tn  restricted to words held in shared memory (degrees <= M <= N-1), where
// G is the adjoint of Y (degrees 1..M), X = xs and Tn has an implied degree-0 term handled by the
// caller:
//   gx[u] += sign * sum_{p=1}^{M-|u|} sum_{|v|=p} G(u.v) * Tn(v)       for 1 <= |u| <= M-1
//   gt[v] (+)= sign * sum_{m=1}^{M-|v|} sum_{|u|=m} X(u) * G(u.v)      for 1 <= |v| <= M-1
// `gt_assign`: overwrite gt (a fresh adjoint buffer) instead of adding to it.
// Words whose sums are long (low degrees) get a warp each, lanes striding the sum; the rest one
// thread each.  Every thread of the block must call this (it contains warp shuffles).
template <typename T>
__device__ __forceinline__ void adjoint_in_smem(const HornerPlan &p, int M, const T *xs, const T *tn, const T *G,
                                                T sign, T *gx, T *gt, bool gt_assign)
{
    if (M < 2) return;
    const unsigned words = p.off[M];  // words of degree <= M-1 (per side)
    // degrees 1..mw get warps: their sums have off[M-m+1] terms
    unsigned warp_words = 0;
    for (int m = 1; m <= M - 1; ++m)
        if (p.off[M - m + 1] >= kTeamTerms) warp_words = p.off[m + 1];
    const unsigned warp_threads = 64u * warp_words;
    const unsigned thread_words = words - warp_words;
    const unsigned total = warp_threads + 2u * thread_words;
    const unsigned span = (total + 31u) / 32u * 32u;
    for (unsigned t = threadIdx.x; t < span; t += blockDim.x) {
        const bool team = t < warp_threads;
        unsigned word, lane, stride;
        int side;
        if (team) {
            const unsigned item = t >> 5;
            side = item >= warp_words ? 1 : 0;
            word = item - (side ? warp_words : 0u);
            lane = t & 31u;
            stride = 32u;
        } else {
            const unsigned item = t - warp_threads;
            side = item >= thread_words ? 1 : 0;
            word = warp_words + item - (side ? thread_words : 0u);
            lane = 0u;
            stride = 1u;
        }
        const bool live = team || t < total;
        T acc = T(0);
        if (live) {
            const int n = degree_at(p, word, M - 1);
            const unsigned code = word - p.off[n];
            if (side == 0) {
                for (int q = 1; n + q <= M; ++q) {
                    const unsigned dq = p.dpow[q];
                    const T *grun = G + p.off[n + q] + code * dq;
                    const T *trun = tn + p.off[q];
                    for (unsigned v = lane; v < dq; v += stride) acc = fma(grun[v], trun[v], acc);
                }
            } else {
                const unsigned dn = p.dpow[n];
                for (int m = 1; m + n <= M; ++m) {
                    const unsigned dm = p.dpow[m];
                    const T *xrun = xs + p.off[m];
                    const T *gcol = G + p.off[m + n] + code;
                    for (unsigned u = lane; u < dm; u += stride) acc = fma(xrun[u], gcol[u * dn], acc);
                }
            }
        }
        if (team) {
#pragma unroll
            for (int sft = 16; sft >= 1; sft >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, sft);
        }
        if (live && lane == 0u) {
            if (side == 0) gx[word] += sign * acc;
            else if (gt_assign) gt[word] = sign * acc;
            else gt[word] += sign * acc;
        }
    }
}

template <typename T, int NMAX, bool STREAMED, int BLOCK>
__global__ void __launch_bounds__(BLOCK) logsig_backward_horner(const HornerPlan p, const T *__restrict__ sig,
                                                                       const T *__restrict__ glog,
                                                                       T *__restrict__ gsig, T *scratch)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    // `scratch` null: every buffer below lives in shared memory.  Otherwise x is read from the signature
    // row and the other buffers are this row's 4*lower + t_total scalars of `scratch` in global memory
    // (the top degree of the incoming gradient is then never staged).
    T *const xs_copy = reinterpret_cast<T *>(smem_raw);  // x, degrees below N
    const int N = p.depth;
    for (long long row = blockIdx.x; row < p.rows; row += gridDim.x) {
        const T *s = sig + row * p.width;
        const T *xs;
        T *gl;                                     // incoming gradient, degrees below N
        if constexpr (STREAMED) { xs = s; gl = scratch + row * (4 * (long long)p.lower + p.t_total); }
        else { xs = xs_copy; gl = xs_copy + p.lower; }
        T *gx = gl + p.lower;                      // gradient wrt x, degrees below N
        T *ga = gx + p.lower;                      // adjoint of T_k
        T *gb = ga + p.lower;                      // adjoint of T_{k+1}
        T *tk = gb + p.lower;                      // every T_k (degrees 1..N-k) at t_off[k]
        T *gts = tk + p.t_total;                   // dense top degree of the incoming gradient (when staged)
        const T *g = glog + row * p.out_width;
        const T *gtop_global = g + p.out_lower;
        const T *gtop = p.stage_top ? gts : gtop_global;  // re-read N-1 times by each side of the adjoint
        T *out = gsig + row * p.width;
        __syncthreads();
        for (unsigned i = threadIdx.x; i < p.lower; i += blockDim.x) {
            if constexpr (!STREAMED) xs_copy[i] = s[i];
            const T gi = p.low_cols != nullptr ? T(0) : g[i];
            gl[i] = gi;
            gx[i] = gi;   // log S = x * 1 + ...: the degree-0 term of T_1 is 1
            ga[i] = T(0);  // build_t scratch first, then the adjoint of T_1
            gb[i] = T(0);
        }
        if (p.low_cols != nullptr) {
            // projected gradient: spread it over the dense image of the lower degrees (a word may be
            // requested twice), then start gx from it
            __syncthreads();
            for (unsigned i = threadIdx.x; i < p.n_low; i += blockDim.x) atomicAdd(&gl[(unsigned)p.low_cols[i]], g[i]);
            __syncthreads();
            for (unsigned i = threadIdx.x; i < p.lower; i += blockDim.x) gx[i] = gl[i];
        }
        // the top degree of x enters only through that same term
        if (p.stage_top && p.top_words != nullptr) {
            // a projected top degree is scattered into a dense image (zeros elsewhere), after which it
            // goes through the same gathers as a dense one
            for (unsigned i = threadIdx.x; i < p.top_dense; i += blockDim.x) gts[i] = T(0);
            __syncthreads();
        }
        for (unsigned i = threadIdx.x; i < p.top; i += blockDim.x) {
            const T gi = gtop_global[i];
            out[p.lower + i] = gi;
            if (p.stage_top) {
                if (p.top_words != nullptr) atomicAdd(&gts[(unsigned)p.top_words[i]], gi);  // a word may be listed twice
                else gts[i] = gi;
            }
        }
        __syncthreads();
        build_t<T, NMAX>(p, xs, ga, gb, tk);  // ends with a barrier
        const T *t1 = tk + p.t_off[1];
        for (unsigned i = threadIdx.x; i < p.lower; i += blockDim.x) ga[i] = T(0);
        __syncthreads();

        // ---- log S = x (x) T_1: words below the top degree ----
        adjoint_in_smem<T>(p, N - 1, xs, t1, gl, T(1), gx, ga, false);
        __syncthreads();
        // ---- the same product at the top degree ----
        if (N >= 2) {
            if (p.top_words == nullptr || p.stage_top) {
                // dense (or its image): gx[u] += sum_v gtop[u.v] T_1(v), a warp per u while the run is long
                const unsigned long_words = [&] {
                    unsigned w = 0;
                    for (int m = 1; m <= N - 1; ++m)
                        if (p.dpow[N - m] >= kTeamTerms) w = p.off[m + 1];
                    return w;
                }();
                const unsigned span = ((32u * long_words + (p.lower - long_words)) + 31u) / 32u * 32u;
                for (unsigned t = threadIdx.x; t < span; t += blockDim.x) {
                    const bool team = t < 32u * long_words;
                    const unsigned word = team ? (t >> 5) : long_words + (t - 32u * long_words);
                    const unsigned lane = team ? (t & 31u) : 0u, stride = team ? 32u : 1u;
                    const bool live = word < p.lower;
                    T acc = T(0);
                    if (live) {
                        const int m = degree_at(p, word, N - 1);
                        const unsigned run = p.dpow[N - m];
                        const T *grun = gtop + (size_t)(word - p.off[m]) * run;
                        const T *trun = t1 + p.off[N - m];
#pragma unroll 4
                        for (unsigned v = lane; v < run; v += stride) acc = fma(grun[v], trun[v], acc);
                    }
                    if (team) {
#pragma unroll
                        for (int sft = 16; sft >= 1; sft >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, sft);
                    }
                    if (live && lane == 0u) gx[word] += acc;
                }
                // gT_1[v] += sum_u x(u) gtop[u.v]: neighbouring threads take neighbouring v (coalesced
                // reads of the top degree); long sums over u are cut into pieces of at most kPieceTerms terms
                unsigned items_before = 0;
                for (int q = 1; q <= N - 1; ++q) {
                    const unsigned dq = p.dpow[q], du = p.dpow[N - q];
                    const unsigned pieces = (du + kPieceTerms - 1u) / kPieceTerms;
                    const unsigned items = dq * pieces;
                    // this degree's items are dealt to the threads after those of the degrees before it
                    for (unsigned it = (threadIdx.x + blockDim.x - items_before % blockDim.x) % blockDim.x;
                         it < items; it += blockDim.x) {
                        const unsigned piece = it / dq, v = it - piece * dq;
                        const unsigned u0 = piece * kPieceTerms, u1 = min(du, u0 + kPieceTerms);
                        const T *xrun = xs + p.off[N - q];
                        T acc = T(0);
#pragma unroll 4
                        for (unsigned u = u0; u < u1; ++u) acc = fma(xrun[u], gtop[(size_t)u * dq + v], acc);
                        atomicAdd(&ga[p.off[q] + v], acc);
                    }
                    items_before += items;
                }
            } else {
                // projected: each listed word scatters its N-1 splits
                for (unsigned i = threadIdx.x; i < p.top; i += blockDim.x) {
                    const unsigned code = (unsigned)p.top_words[i];
                    const T gw = gtop[i];
                    unsigned q = code;
                    for (int len = 1; len < N; ++len) {
                        q = p.by_d.div(q);
                        const unsigned suf = code - q * p.dpow[len];
                        atomicAdd(&gx[p.off[N - len] + q], gw * t1[p.off[len] + suf]);
                        atomicAdd(&ga[p.off[len] + suf], xs[p.off[N - len] + q] * gw);
                    }
                }
            }
        }
        __syncthreads();

        // ---- T_k = 1/k - x (x) T_{k+1},  k = 1 .. N-1;  ga = adjoint of T_k (degrees 1..N-k) ----
        T *gk = ga, *gn = gb;
        for (int k = 1; k <= N - 1; ++k) {
            const int M = N - k;
            const T c = T(1) / T(k + 1);
            for (unsigned i = threadIdx.x; i < p.off[M + 1]; i += blockDim.x) gx[i] -= c * gk[i];
            for (unsigned i = threadIdx.x; i < p.off[M]; i += blockDim.x) gn[i] = T(0);
            __syncthreads();
            if (k < N - 1) adjoint_in_smem<T>(p, M, xs, tk + p.t_off[k + 1], gk, T(-1), gx, gn, true);
            __syncthreads();
            T *tmp = gk; gk = gn; gn = tmp;
        }
        for (unsigned i = threadIdx.x; i < p.lower; i += blockDim.x) out[i] = gx[i];
    }
}

int make_horner_plan(const PsigLogDesc &desc, const LevelTable &lt, HornerPlan *plan)
{
    HornerPlan &p = *plan;
    p.d = lt.d;
    p.by_d.set((unsigned)lt.d);
    p.depth = lt.depth;
    p.rows = desc.rows;
    p.width = lt.total;
    unsigned long long pw = 1, off = 0;
    p.dpow[0] = 1;
    p.off[0] = 0;
    for (int n = 1; n <= kMaxDepth; ++n) {
        p.off[n] = (unsigned)off;
        if (n < lt.depth) {
            pw *= (unsigned long long)lt.d;
            if (pw > 0x7fffffffULL) return PSIG_ERR_UNSUPPORTED;
            p.dpow[n] = (unsigned)pw;
            off += pw;
            if (off > 0x7fffffffULL) return PSIG_ERR_UNSUPPORTED;
        } else {
            p.dpow[n] = 0;
        }
    }
    p.off[kMaxDepth + 1] = (unsigned)off;
    p.lower = (unsigned)off;
    // the codes of the top degree must fit 32 bits too
    if (pw * (unsigned long long)lt.d > 0x7fffffffULL) return PSIG_ERR_UNSUPPORTED;
    if (lt.size[lt.depth] > 0x7fffffffLL) return PSIG_ERR_UNSUPPORTED;
    p.top = (unsigned)lt.size[lt.depth];
    p.top_dense = (unsigned)(pw * (unsigned long long)lt.d);
    p.top_words = lt.words[lt.depth];
    if ((long long)p.lower + (long long)p.top != lt.total) return PSIG_ERR_UNSUPPORTED;  // lower degrees must be dense
    unsigned t = 0;
    for (int k = 1; k <= kMaxDepth; ++k) {
        p.t_off[k] = t;
        if (k <= lt.depth - 1) t += p.off[lt.depth - k + 1];
    }
    p.t_total = t;
    p.stage_top = 0;
    p.low_cols = nullptr;
    p.n_low = 0;
    if (desc.lower_columns != nullptr || desc.n_lower_columns > 0) {
        if (desc.lower_columns == nullptr || desc.n_lower_columns < 0 || desc.n_lower_columns > 0x7fffffffLL) return PSIG_ERR_SHAPE;
        p.low_cols = reinterpret_cast<const long long *>(desc.lower_columns);
        p.n_low = (unsigned)desc.n_lower_columns;
    }
    p.out_lower = p.low_cols != nullptr ? p.n_low : p.lower;
    p.out_width = (long long)p.out_lower + (long long)p.top;
    return PSIG_OK;
}

template <typename T> size_t forward_smem(const HornerPlan &p) { return sizeof(T) * 3 * (size_t)p.lower; }
template <typename T> size_t backward_smem(const HornerPlan &p)
{
    return sizeof(T) * (5 * (size_t)p.lower + p.t_total + (p.stage_top ? (size_t)p.top_dense : 0));
}

// Threads per row (= per block).  The kernels stride by the launched block size; narrower blocks were
// measured (config 4 and a dense (8,4) row): 128 threads gain 15 % forward and lose 35 % backward, 64 and
// 32 threads lose up to 3.5x -- a row's phases are parallel inside the row, and rows in flight are limited
// by shared memory, not by threads.
unsigned horner_block(long long rows, bool streamed, bool backward = false)
{
    int device = 0, sms = 148;
    if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (!streamed) {
        if (backward) return rows <= 8LL * sms ? kHornerWideBlock : kHornerBlock;
        // forward, few rows: half-width blocks double the rows in flight, so that e.g. 1 024 rows are one wave
        // (config 4: 0.024 -> 0.020 ms)
        return rows <= 8LL * sms ? kHornerBlock / 2 : kHornerBlock;
    }
    // few large rows: a row is all the parallelism a block has
    return rows < 2LL * sms ? kStreamedMaxBlock : rows < 16LL * sms ? 512u : (unsigned)kHornerBlock;
}

unsigned row_grid(long long rows) { return (unsigned)(rows < (1 << 20) ? rows : (1 << 20)); }

}  // namespace

bool horner_logsig_supported(const PsigLogDesc &desc, const LevelTable &lt)
{
    if (desc.algo == PSIG_ALGO_GENERIC) return false;
    HornerPlan p;
    if (make_horner_plan(desc, lt, &p) != PSIG_OK) return false;
    const size_t scalar = desc.dtype == PSIG_F32 ? 4 : 8;
    return scalar * (5 * (size_t)p.lower + p.t_total) <= kHornerMaxSmem;  // backward needs the most
}

// Scalars of global scratch the streamed form needs per call, forward and backward, or a negative status
// when word codes or row positions do not fit 32 bits (a row of 2^31 scalars or more).
long long streamed_logsig_forward_scratch(const PsigLogDesc &desc, const LevelTable &lt)
{
    HornerPlan p;
    const int rc = make_horner_plan(desc, lt, &p);
    if (rc != PSIG_OK) return PSIG_ERR_TOO_LARGE;
    return desc.rows * 2 * (long long)p.lower;
}

long long streamed_logsig_backward_scratch(const PsigLogDesc &desc, const LevelTable &lt)
{
    HornerPlan p;
    const int rc = make_horner_plan(desc, lt, &p);
    if (rc != PSIG_OK) return PSIG_ERR_TOO_LARGE;
    return desc.rows * (4 * (long long)p.lower + (long long)p.t_total);
}

// `scratch` null: the row-in-shared-memory form (the caller has checked horner_logsig_supported).
// Otherwise the streamed form on streamed_logsig_forward_scratch() scalars of global memory.
template <typename T>
int horner_logsig_forward(const PsigLogDesc &desc, const LevelTable &lt, const T *sig, T *logsig, T *scratch,
                          cudaStream_t stream)
{
    HornerPlan p;
    const int rc = make_horner_plan(desc, lt, &p);
    if (rc != PSIG_OK) return scratch ? (int)PSIG_ERR_TOO_LARGE : rc;
    const size_t smem = scratch ? 0 : forward_smem<T>(p);
    auto launch = [&](auto kernel) {
        // rows in flight are limited by shared memory under the default L1 split
        if (smem > 0 && !prepare_kernel(kernel, smem, true)) return (int)PSIG_ERR_CUDA;
        kernel<<<row_grid(desc.rows), horner_block(desc.rows, scratch != nullptr), smem, stream>>>(p, sig, logsig, scratch);
        return check_launch();
    };
    if (scratch) {
        if (p.depth <= 4) return launch(logsig_forward_horner<T, 4, true>);
        if (p.depth <= 6) return launch(logsig_forward_horner<T, 6, true>);
        if (p.depth <= 8) return launch(logsig_forward_horner<T, 8, true>);
        return launch(logsig_forward_horner<T, 12, true>);
    }
    if (p.depth <= 4) return launch(logsig_forward_horner<T, 4, false>);
    if (p.depth <= 6) return launch(logsig_forward_horner<T, 6, false>);
    if (p.depth <= 8) return launch(logsig_forward_horner<T, 8, false>);
    return launch(logsig_forward_horner<T, 12, false>);
}

template <typename T>
int horner_logsig_backward(const PsigLogDesc &desc, const LevelTable &lt, const T *sig, const T *grad_logsig,
                           T *grad_sig, T *scratch, cudaStream_t stream)
{
    HornerPlan p;
    const int rc = make_horner_plan(desc, lt, &p);
    if (rc != PSIG_OK) return scratch ? (int)PSIG_ERR_TOO_LARGE : rc;
    // the top degree is staged (dense, or as a dense image of the listed words) while the block stays
    // under half of the largest supported footprint; the streamed form reads it where it is
    p.stage_top = (!scratch && p.depth >= 2 &&
                   sizeof(T) * (5 * (size_t)p.lower + p.t_total + (size_t)p.top_dense) <= kHornerMaxSmem / 2) ? 1u : 0u;
    const size_t smem = scratch ? 0 : backward_smem<T>(p);
    const unsigned block = horner_block(desc.rows, scratch != nullptr, true);
    auto launch = [&](auto kernel) {
        if (smem > 0 && !prepare_kernel(kernel, smem, true)) return (int)PSIG_ERR_CUDA;
        kernel<<<row_grid(desc.rows), block, smem, stream>>>(p, sig, grad_logsig, grad_sig, scratch);
        return check_launch();
    };
    // each block width is its own instance: a wider launch bound changed the code of the 256-thread case
    if (scratch) {
        if (p.depth <= 4) return launch(logsig_backward_horner<T, 4, true, kStreamedMaxBlock>);
        if (p.depth <= 6) return launch(logsig_backward_horner<T, 6, true, kStreamedMaxBlock>);
        if (p.depth <= 8) return launch(logsig_backward_horner<T, 8, true, kStreamedMaxBlock>);
        return launch(logsig_backward_horner<T, 12, true, kStreamedMaxBlock>);
    }
    if (block == (unsigned)kHornerWideBlock) {
        if (p.depth <= 4) return launch(logsig_backward_horner<T, 4, false, kHornerWideBlock>);
        if (p.depth <= 6) return launch(logsig_backward_horner<T, 6, false, kHornerWideBlock>);
        if (p.depth <= 8) return launch(logsig_backward_horner<T, 8, false, kHornerWideBlock>);
        return launch(logsig_backward_horner<T, 12, false, kHornerWideBlock>);
    }
    if (p.depth <= 4) return launch(logsig_backward_horner<T, 4, false, kHornerBlock>);
    if (p.depth <= 6) return launch(logsig_backward_horner<T, 6, false, kHornerBlock>);
    if (p.depth <= 8) return launch(logsig_backward_horner<T, 8, false, kHornerBlock>);
    return launch(logsig_backward_horner<T, 12, false, kHornerBlock>);
}

template int horner_logsig_backward<float>(const PsigLogDesc &, const LevelTable &, const float *, const float *,
                                           float *, float *, cudaStream_t);
template int horner_logsig_backward<double>(const PsigLogDesc &, const LevelTable &, const double *, const double *,
                                            double *, double *, cudaStream_t);
template int horner_logsig_forward<float>(const PsigLogDesc &, const LevelTable &, const float *, float *, float *,
                                          cudaStream_t);
template int horner_logsig_forward<double>(const PsigLogDesc &, const LevelTable &, const double *, double *, double *,
                                           cudaStream_t);

}  // namespace psig
