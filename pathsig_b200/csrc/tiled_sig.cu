// Register-tiled dense signature kernels (float32, compile-time channel count D and depth N).
//
// The word tree is cut at a prefix length P.  One thread owns a prefix u (|u| = P) and, of the
// sub-tree below it, the DA first letters [a0, a0+DA): the values S(u.a), S(u.a.b), ... down
// to degree N live in registers (DA * (1 + D + ... ) floats), the P values S(u[:j]) on the
// way to the root are kept redundantly by every thread that shares them.  One step of Chen's
// recurrence S <- S (x) exp(dx) is then, per target degree k, a Horner chain
//     B_j = B_{j-1} * dx[w_j] / (k-j+1) + S_j         (j = 1..k-1),   S_k += B_{k-1} * dx[w_k]
// whose scalar head (j <= P) costs P FMAs and whose tail is pure register FMA over the owned
// sub-tree: no shared-memory state, no barrier and no shuffle inside the step loop.  Shared
// prefixes are evaluated once per thread instead of once per word as in the reference
// (src/pathsig/forward/sig_kernels.cu:138-152), which is where the ~8x arithmetic saving at
// (d, depth) = (8, 4) comes from.  Increments (and their multiples 1/2, 1/3 needed by the
// Horner tail) are staged in shared memory a chunk of steps at a time.
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
#include "common.cuh"

#include <cstdint>

namespace psig {
namespace {

__host__ __device__ constexpr int ipow(int b, int e) { int r = 1; for (int i = 0; i < e; ++i) r *= b; return r; }
__host__ __device__ constexpr int at_least_one(int n) { return n > 0 ? n : 1; }

template <int D, int N, int P, int DA>
struct Shape {
    static_assert(P >= 1 && P < N, "prefix length must leave a sub-tree");
    static_assert(D % DA == 0, "DA must divide D");
    static constexpr int Q = N - P;  // depth of the register sub-tree
    static_assert(Q <= 3, "sub-tree depth above 3 is not implemented");
    static constexpr int SPLIT = D / DA;
    static constexpr int TPU = ipow(D, P) * SPLIT;  // threads per (path, window) unit
    // Blocks of NT threads cover a unit; when NT does not divide TPU the last block has idle threads.
    __host__ __device__ static constexpr int parts(int nt) { return (TPU + nt - 1) / nt; }
    static constexpr int n1 = DA;
    static constexpr int n2 = Q >= 2 ? DA * D : 0;
    static constexpr int n3 = Q >= 3 ? DA * D * D : 0;
    __host__ __device__ static constexpr long long dense_off(int k)
    {
        long long o = 0, p = 1;
        for (int j = 1; j < k; ++j) { p *= D; o += p; }
        return o;
    }
    static constexpr long long TOTAL = dense_off(N + 1);
    // 128-bit global accesses: runs at degree P+1 start at u*D + a0, deeper runs at multiples of D
    static constexpr bool kVecFirst = (D % 4 == 0) && (DA % 4 == 0);
    static constexpr bool kVecDeep = (D % 4 == 0);
};

template <int LEN>
__device__ __forceinline__ void load_run(float (&dst)[LEN], const float *src, bool vec)
{
    if constexpr (LEN % 4 == 0) {
        if (vec) {
#pragma unroll
            for (int i = 0; i < LEN / 4; ++i) {
                const float4 v = reinterpret_cast<const float4 *>(src)[i];
                dst[4 * i] = v.x; dst[4 * i + 1] = v.y; dst[4 * i + 2] = v.z; dst[4 * i + 3] = v.w;
            }
            return;
        }
    }
#pragma unroll
    for (int i = 0; i < LEN; ++i) dst[i] = src[i];
}

template <int LEN>
__device__ __forceinline__ void store_run(float *dst, const float (&src)[LEN], bool vec)
{
    if constexpr (LEN % 4 == 0) {
        if (vec) {
#pragma unroll
            for (int i = 0; i < LEN / 4; ++i)
                reinterpret_cast<float4 *>(dst)[i] = make_float4(src[4 * i], src[4 * i + 1], src[4 * i + 2], src[4 * i + 3]);
            return;
        }
    }
#pragma unroll
    for (int i = 0; i < LEN; ++i) dst[i] = src[i];
}

// Block-wide barrier; a block of one warp only needs warp convergence plus memory ordering.
template <int NT>
__device__ __forceinline__ void block_sync()
{
    if constexpr (NT <= 32) __syncwarp(); else __syncthreads();
}

__device__ __forceinline__ void window_of(long long unit, long long L, long long W, const int *windows,
                                          long long &b, int &start, int &steps)
{
    b = unit / W;
    start = 0;
    int end = (int)L;
    if (windows) {
        const long long w = unit % W;
        // clamped to the path: a window reaching outside reads only the points that exist
        start = max(windows[2 * w], 0);
        end = min(windows[2 * w + 1], (int)L);
    }
    steps = max(end - start - 1, 0);
}

// s_dx[0][t][a] = dx_{c0+t}[a]; with HALF also s_dx[1][t][a] = dx_{c0+t}[a] / 2.  Elsewhere the 1/2 and
// 1/3 factors of the Horner tail are applied to the scalar multiplier instead of to the vector; the
// halved table is kept for the backward sweep with a two-level sub-tree, where it measured faster.
template <int D, bool HALF, int CH, int NT>
__device__ __forceinline__ void stage_scaled_increments(const float *__restrict__ x, int c0, int n,
                                                        float (*s_dx)[CH][D])
{
    const float *lo = x + (long long)c0 * D;
    for (int i = threadIdx.x; i < n * D; i += NT) {
        const float v = lo[i + D] - lo[i];
        (&s_dx[0][0][0])[i] = v;
        if constexpr (HALF) (&s_dx[1][0][0])[i] = v * 0.5f;
    }
}

// ------------------------------------------------------------------------------------------
// Asynchronous staging of raw path points: bulk copies issued by one thread (cp.async.bulk, the
// TMA engine's untiled form) that land in this block's shared memory and signal an mbarrier.
// Two buffers, so the copy of the next chunk runs under the arithmetic of the current one.
// Every wait is bounded; if a copy has not landed in time the block reads the same bytes with
// plain loads (harmless if the copy lands later: same data) and counts the event.
// ------------------------------------------------------------------------------------------
__device__ unsigned int g_bulk_copy_timeouts = 0;

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long *bar, int count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void bulk_copy_g2s(void *dst, const void *src, uint32_t bytes, unsigned long long *bar)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_addr(dst)),
                 "l"(src), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(unsigned long long *bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

constexpr int kBulkWaitPolls = 1 << 20;

__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long *bar, uint32_t parity)
{
    for (int i = 0; i < kBulkWaitPolls; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

template <int D, int MAXPTS>
struct PointPipe {
    float raw[2][MAXPTS * D];
    unsigned long long bar[2];
    int failed;  // set (and never cleared) by any thread whose bounded wait ran out
};

// Thread 0 only.  Copies `npts` points (npts * D floats, a multiple of 16 bytes) starting at src.
template <int D, int MAXPTS>
__device__ __forceinline__ void pipe_issue(PointPipe<D, MAXPTS> &pp, int slot, const float *src, int npts)
{
    fence_proxy_async();  // earlier generic-proxy reads of this buffer are ordered before the copy
    bulk_copy_g2s(pp.raw[slot], src, (uint32_t)(npts * D * sizeof(float)), &pp.bar[slot]);
}

// s_dx tables from staged points: raw[t*D + a], t = 0..n.
template <int D, int CH, int NT>
__device__ __forceinline__ void scaled_increments_from_points(const float *raw, int n, float (*s_dx)[CH][D])
{
    for (int i = threadIdx.x; i < n * D; i += NT) {
        const float v = raw[i + D] - raw[i];
        (&s_dx[0][0][0])[i] = v;
    }
}

// Fetch the increments at the prefix letters one step ahead (measured: helps the backward sweep by
// about 1 %, costs registers and time in the forward sweep).
#ifndef PSIG_PREFETCH_XS_FWD
#define PSIG_PREFETCH_XS_FWD 0
#endif
#ifndef PSIG_PREFETCH_XS_BWD
#define PSIG_PREFETCH_XS_BWD 1
#endif
#ifndef PSIG_PACKED_FMA
#define PSIG_PACKED_FMA 1
#endif
// (x0, x1) += (a0, a1) * (b0, b1): one packed two-lane FMA (fma.rn.f32x2 of sm_100) instead of two
// scalar ones.  Same arithmetic and rounding per lane; it halves the issue slots of the inner loops.
__device__ __forceinline__ void fma_pair(float &x0, float &x1, float a0, float a1, float b0, float b1)
{
#if PSIG_PACKED_FMA
    const float2 r = __ffma2_rn(make_float2(a0, a1), make_float2(b0, b1), make_float2(x0, x1));
    x0 = r.x;
    x1 = r.y;
#else
    x0 = fmaf(a0, b0, x0);
    x1 = fmaf(a1, b1, x1);
#endif
}

// Whether the backward sweep keeps a second table of halved increments.  Measured: with a two-level
// sub-tree and few channels the table wins (about 3 % at d = 8); at d = 16 the registers it costs
// lose more than the multiplications it saves.
__host__ __device__ constexpr bool half_table(int D, int Q) { return Q == 2 && D <= 8; }

// The operands one step needs: the increment at this thread's prefix letters, the full
// increment vector, and the (scaled) slices at the owned first letters.
template <int D, int DA, int P, bool HALF = false>
struct StepOperands {
    float xs[P];
    float dxf1[D];                      // dx
    float dxa1[DA];                     // dx[a0..]
    float dxa2[HALF ? DA : 1];          // dx[a0..] / 2
};

template <int D, int DA, int P, bool HALF, int CH, bool XS_GIVEN = false>
__device__ __forceinline__ void load_operands(StepOperands<D, DA, P, HALF> &o, const float (*s_dx)[CH][D], int t,
                                              const int (&let)[P], int a0)
{
    if constexpr (HALF) load_run<DA>(o.dxa2, s_dx[1][t] + a0, true);
    const float *row = s_dx[0][t];
    if constexpr (!XS_GIVEN) {
#pragma unroll
        for (int j = 0; j < P; ++j) o.xs[j] = row[let[j]];
    }
    load_run<D>(o.dxf1, row, true);
    if constexpr (DA == D) {
#pragma unroll
        for (int a = 0; a < DA; ++a) o.dxa1[a] = o.dxf1[a];
    } else {
        load_run<DA>(o.dxa1, row + a0, true);
    }
}

// ------------------------------------------------------------------------------------------
// forward
// ------------------------------------------------------------------------------------------
#ifndef PSIG_FWD_CHUNK
#define PSIG_FWD_CHUNK 64
#endif
constexpr int kFwdChunk = PSIG_FWD_CHUNK;

template <int D, int N, int P, int DA>
struct ForwardState {
    using S = Shape<D, N, P, DA>;
    float pref[P + 1];
    float R1[S::n1], R2[at_least_one(S::n2)], R3[at_least_one(S::n3)];
};

template <int D, int N, int P, int DA>
__device__ __forceinline__ void forward_step(ForwardState<D, N, P, DA> &s, const StepOperands<D, DA, P> &o)
{
    constexpr int Q = N - P;
    if constexpr (Q >= 3) {  // target degree P+3
        constexpr int k = P + 3;
        float bb = 1.f;
#pragma unroll
        for (int j = 1; j <= P; ++j) bb = fmaf(bb, o.xs[j - 1] * recip<float>(k - j + 1), s.pref[j]);
        const float bb3 = bb * recip<float>(3);  // the stage's 1/3 rides on the scalar, not on the vector
#pragma unroll
        for (int a = 0; a < DA; ++a) {
            const float v1 = fmaf(bb3, o.dxa1[a], s.R1[a]);
            const float v1h = 0.5f * v1;
#pragma unroll
            for (int c = 0; c < D; ++c) {
                const float v2 = fmaf(v1h, o.dxf1[c], s.R2[a * D + c]);
#pragma unroll
                for (int e = 0; e + 1 < D; e += 2)
                    fma_pair(s.R3[(a * D + c) * D + e], s.R3[(a * D + c) * D + e + 1], v2, v2, o.dxf1[e], o.dxf1[e + 1]);
                if constexpr (D % 2 == 1)
                    s.R3[(a * D + c) * D + D - 1] = fmaf(v2, o.dxf1[D - 1], s.R3[(a * D + c) * D + D - 1]);
            }
        }
    }
    if constexpr (Q >= 2) {  // target degree P+2
        constexpr int k = P + 2;
        float bb = 1.f;
#pragma unroll
        for (int j = 1; j <= P; ++j) bb = fmaf(bb, o.xs[j - 1] * recip<float>(k - j + 1), s.pref[j]);
        const float bbh = 0.5f * bb;
#pragma unroll
        for (int a = 0; a < DA; ++a) {
            const float v1 = fmaf(bbh, o.dxa1[a], s.R1[a]);
#pragma unroll
            for (int c = 0; c + 1 < D; c += 2)
                fma_pair(s.R2[a * D + c], s.R2[a * D + c + 1], v1, v1, o.dxf1[c], o.dxf1[c + 1]);
            if constexpr (D % 2 == 1) s.R2[a * D + D - 1] = fmaf(v1, o.dxf1[D - 1], s.R2[a * D + D - 1]);
        }
    }
    {  // target degree P+1
        constexpr int k = P + 1;
        float bb = 1.f;
#pragma unroll
        for (int j = 1; j <= P; ++j) bb = fmaf(bb, o.xs[j - 1] * recip<float>(k - j + 1), s.pref[j]);
#pragma unroll
        for (int a = 0; a + 1 < DA; a += 2) fma_pair(s.R1[a], s.R1[a + 1], bb, bb, o.dxa1[a], o.dxa1[a + 1]);
        if constexpr (DA % 2 == 1) s.R1[DA - 1] = fmaf(bb, o.dxa1[DA - 1], s.R1[DA - 1]);
    }
    // the shared prefixes, highest first so each reads the previous step's lower values
#pragma unroll
    for (int m = P; m >= 1; --m) {
        float bm = 1.f;
#pragma unroll
        for (int j = 1; j <= m - 1; ++j) bm = fmaf(bm, o.xs[j - 1] * recip<float>(m - j + 1), s.pref[j]);
        s.pref[m] = fmaf(bm, o.xs[m - 1], s.pref[m]);
    }
}

// PROJ: the top degree is a word list (rows are dense below it).  BULK: stage points with bulk
// copies (needs 16-byte aligned path rows); otherwise plain loads.
template <int D, int N, int P, int DA, int NT, int MINB, bool PROJ, bool BULK>
__global__ void __launch_bounds__(NT, MINB) sig_forward_tiled(const float *__restrict__ path, float *__restrict__ out,
                                                              long long L, long long W,
                                                              const int *__restrict__ windows, int vec_ok,
                                                              const long long *__restrict__ top_words, int top_size)
{
    using S = Shape<D, N, P, DA>;
    constexpr int Q = S::Q, PARTS = S::parts(NT), CH = kFwdChunk;
    constexpr bool PADDED = S::TPU % NT != 0;  // the unit's last block has threads without work
    extern __shared__ __align__(16) float s_top[];  // D^N floats, only when the top degree is projected
    __shared__ __align__(16) float s_dx[1][CH][D];
    __shared__ __align__(16) PointPipe<D, BULK ? CH + 1 : 1> s_pipe;  // one float per buffer when unused

    const long long unit = blockIdx.x / PARTS;
    int tu = (int)(blockIdx.x % PARTS) * NT + threadIdx.x;
    bool active = true;
    if constexpr (PADDED) {
        // idle threads shadow the unit's last thread (they take part in staging and barriers) and
        // store nothing
        active = tu < S::TPU;
        tu = min(tu, S::TPU - 1);
    }
    const int u = tu / S::SPLIT;
    const int a0 = (tu % S::SPLIT) * DA;
    int let[P];
    {
        int c = u;
#pragma unroll
        for (int j = P - 1; j >= 0; --j) { let[j] = c % D; c /= D; }
    }
    long long b; int start, steps;
    window_of(unit, L, W, windows, b, start, steps);
    const float *x = path + (b * L + start) * D;

    ForwardState<D, N, P, DA> st;
#pragma unroll
    for (int j = 0; j <= P; ++j) st.pref[j] = 0.f;
#pragma unroll
    for (int i = 0; i < S::n1; ++i) st.R1[i] = 0.f;
#pragma unroll
    for (int i = 0; i < at_least_one(S::n2); ++i) st.R2[i] = 0.f;
#pragma unroll
    for (int i = 0; i < at_least_one(S::n3); ++i) st.R3[i] = 0.f;

    if constexpr (!BULK) {
        for (int c0 = 0; c0 < steps; c0 += CH) {
            const int n = min(CH, steps - c0);
            block_sync<NT>();
            stage_scaled_increments<D, false, CH, NT>(x, c0, n, s_dx);
            block_sync<NT>();
#if PSIG_PREFETCH_XS_FWD
            float xs_next[P];
#pragma unroll
            for (int j = 0; j < P; ++j) xs_next[j] = s_dx[0][0][let[j]];
#endif
#pragma unroll 1
            for (int t = 0; t < n; ++t) {
                StepOperands<D, DA, P> o;
#if PSIG_PREFETCH_XS_FWD
#pragma unroll
                for (int j = 0; j < P; ++j) o.xs[j] = xs_next[j];
                const int tn = min(t + 1, n - 1);
#pragma unroll
                for (int j = 0; j < P; ++j) xs_next[j] = s_dx[0][tn][let[j]];
                load_operands<D, DA, P, false, CH, true>(o, s_dx, t, let, a0);
#else
                load_operands<D, DA, P, false, CH>(o, s_dx, t, let, a0);
#endif
                forward_step<D, N, P, DA>(st, o);
            }
        }
    } else {
        // Points of chunk ci: [ci*CH, ci*CH + n] -> n+1 points; the copy of chunk ci+1 is in
        // flight while chunk ci computes.
        const int nchunks = (steps + CH - 1) / CH;
        bool bulk = true;
        if (nchunks > 0) {
            if (threadIdx.x == 0) {
                mbar_init(&s_pipe.bar[0], 1);
                mbar_init(&s_pipe.bar[1], 1);
                s_pipe.failed = 0;
                fence_mbar_init();
            }
            block_sync<NT>();
            if (threadIdx.x == 0) pipe_issue(s_pipe, 0, x, min(CH, steps) + 1);
        }
        int issued = 1;  // chunks whose copy has been issued (meaningful in thread 0 only)
        for (int ci = 0; ci < nchunks; ++ci) {
            const int c0 = ci * CH;
            const int n = min(CH, steps - c0);
            if (bulk) {
                if (threadIdx.x == 0 && ci + 1 < nchunks) {
                    pipe_issue(s_pipe, (ci + 1) & 1, x + (long long)(c0 + CH) * D, min(CH, steps - c0 - CH) + 1);
                    issued = ci + 2;
                }
                if (!mbar_wait_bounded(&s_pipe.bar[ci & 1], (uint32_t)((ci >> 1) & 1))) s_pipe.failed = 1;
                scaled_increments_from_points<D, CH, NT>(s_pipe.raw[ci & 1], n, s_dx);
            } else {
                stage_scaled_increments<D, false, CH, NT>(x, c0, n, s_dx);
            }
            block_sync<NT>();
            if (bulk && s_pipe.failed) {
                // a copy missed its deadline (never seen in practice): count it, read this and all
                // later chunks with plain loads instead
                if (threadIdx.x == 0) atomicAdd(&g_bulk_copy_timeouts, 1u);
                bulk = false;
                stage_scaled_increments<D, false, CH, NT>(x, c0, n, s_dx);
                block_sync<NT>();
            }
#if PSIG_PREFETCH_XS_FWD
            float xs_next[P];
#pragma unroll
            for (int j = 0; j < P; ++j) xs_next[j] = s_dx[0][0][let[j]];
#endif
#pragma unroll 1
            for (int t = 0; t < n; ++t) {
                StepOperands<D, DA, P> o;
#if PSIG_PREFETCH_XS_FWD
#pragma unroll
                for (int j = 0; j < P; ++j) o.xs[j] = xs_next[j];
                const int tn = min(t + 1, n - 1);
#pragma unroll
                for (int j = 0; j < P; ++j) xs_next[j] = s_dx[0][tn][let[j]];
                load_operands<D, DA, P, false, CH, true>(o, s_dx, t, let, a0);
#else
                load_operands<D, DA, P, false, CH>(o, s_dx, t, let, a0);
#endif
                forward_step<D, N, P, DA>(st, o);
            }
            block_sync<NT>();  // tables (and the staged points they came from) are free again
        }
        if (threadIdx.x == 0 && nchunks > 0 && s_pipe.failed) {
            // do not leave the block while one of its copies may still be in flight: one more
            // bounded wait on the last phase issued into each buffer
            for (int c = max(0, issued - 2); c < issued; ++c)
                mbar_wait_bounded(&s_pipe.bar[c & 1], (uint32_t)((c >> 1) & 1));
        }
    }

    // Row layout: dense degrees 1..N, or (PROJ) dense degrees 1..N-1 followed by
    // the top_size requested words of degree N in the caller's order.
    const long long width = PROJ ? S::dense_off(N) + top_size : S::TOTAL;
    float *row = out + unit * width;
    const bool vec1 = S::kVecFirst && vec_ok, vec = S::kVecDeep && vec_ok;
    if (active) {
#pragma unroll
        for (int j = 1; j <= P; ++j) {
            const int span = ipow(D, P - j) * S::SPLIT;  // threads sharing the prefix of length j
            if (tu % span == 0) row[S::dense_off(j) + tu / span] = st.pref[j];
        }
    }
    const long long base1 = (long long)u * D + a0;
    if constexpr (!PROJ) {
        if (active) {
            store_run<S::n1>(row + S::dense_off(P + 1) + base1, st.R1, vec1);
            if constexpr (Q >= 2) store_run<S::n2>(row + S::dense_off(P + 2) + base1 * D, st.R2, vec);
            if constexpr (Q >= 3) store_run<S::n3>(row + S::dense_off(P + 3) + base1 * D * D, st.R3, vec);
        }
    } else {
        // the block holds the whole unit (checked by the launcher): stage the dense top degree in
        // shared memory and copy out the requested words
        if (active) {
            if constexpr (Q == 1) {
                store_run<S::n1>(s_top + base1, st.R1, true);
            } else if constexpr (Q == 2) {
                store_run<S::n1>(row + S::dense_off(P + 1) + base1, st.R1, vec1);
                store_run<S::n2>(s_top + base1 * D, st.R2, true);
            } else {
                store_run<S::n1>(row + S::dense_off(P + 1) + base1, st.R1, vec1);
                store_run<S::n2>(row + S::dense_off(P + 2) + base1 * D, st.R2, vec);
                store_run<S::n3>(s_top + base1 * D * D, st.R3, true);
            }
        }
        block_sync<NT>();
        for (int i = threadIdx.x; i < top_size; i += NT) row[S::dense_off(N) + i] = s_top[top_words[i]];
    }
}

// ------------------------------------------------------------------------------------------
// backward
// ------------------------------------------------------------------------------------------

template <int D, int N, int P, int DA>
struct BackwardState {
    using S = Shape<D, N, P, DA>;
    float pref[P + 1], apref[P + 1];                      // S and partial adjoint at the shared prefixes
    float RS1[S::n1], RS2[at_least_one(S::n2)];           // S at degrees P+1, P+2 (tracked while below N)
    float RG1[S::n1], RG2[at_least_one(S::n2)], RG3[at_least_one(S::n3)];  // adjoints at degrees P+1..N
};

// Push the adjoint `adj` of the scalar Horner value at prefix length P of target degree K down
// to the root: adds to the partial adjoints of the shared prefixes and to the letter gradients.
template <int P, int K>
__device__ __forceinline__ void back_chain(float adj, const float (&bc)[P + 1], const float (&xs)[P],
                                           float (&apref)[P + 1], float (&lg)[P])
{
#pragma unroll
    for (int j = P; j >= 1; --j) {
        apref[j] += adj;
        const float c = 1.f / float(K - j + 1);
        lg[j - 1] = fmaf(adj * c, bc[j - 1], lg[j - 1]);
        adj = adj * (xs[j - 1] * c);
    }
}

template <int P, int K>
__device__ __forceinline__ void head_chain(float (&bc)[P + 1], const float (&xs)[P], const float (&pref)[P + 1])
{
    bc[0] = 1.f;
#pragma unroll
    for (int j = 1; j <= P; ++j) bc[j] = fmaf(bc[j - 1], xs[j - 1] * (1.f / float(K - j + 1)), pref[j]);
}

// One reverse step.  On return gdf[e] / gda[a] / lg[j] hold this thread's share of dL/d(dx_t)
// for letter e, for letter a0+a and for the prefix letter let[j].
template <int D, int N, int P, int DA>
__device__ __forceinline__ void backward_step(BackwardState<D, N, P, DA> &s, const StepOperands<D, DA, P, half_table(D, N - P)> &o,
                                              float (&gdf)[D], float (&gda)[DA], float (&lg)[P])
{
    constexpr int Q = N - P;
#pragma unroll
    for (int e = 0; e < D; ++e) gdf[e] = 0.f;
#pragma unroll
    for (int a = 0; a < DA; ++a) gda[a] = 0.f;
#pragma unroll
    for (int j = 0; j < P; ++j) lg[j] = 0.f;

    // shared prefixes, bottom-up: roll back, then transpose
#pragma unroll
    for (int m = 1; m <= P; ++m) {
        float bc[P + 1];
        bc[0] = 1.f;
#pragma unroll
        for (int j = 1; j <= m - 1; ++j) bc[j] = fmaf(bc[j - 1], o.xs[j - 1] * (1.f / float(m - j + 1)), s.pref[j]);
        s.pref[m] = fmaf(-bc[m - 1], o.xs[m - 1], s.pref[m]);
        const float a = s.apref[m];
        lg[m - 1] = fmaf(a, bc[m - 1], lg[m - 1]);
        float adj = a * o.xs[m - 1];
#pragma unroll
        for (int j = m - 1; j >= 1; --j) {
            s.apref[j] += adj;
            const float c = 1.f / float(m - j + 1);
            lg[j - 1] = fmaf(adj * c, bc[j - 1], lg[j - 1]);
            adj = adj * (o.xs[j - 1] * c);
        }
    }
    {  // target degree P+1
        constexpr int k = P + 1;
        float bc[P + 1];
        head_chain<P, k>(bc, o.xs, s.pref);
        const float bb = bc[P];
        float adj0 = 0.f, adj1 = 0.f;
#pragma unroll
        for (int a = 0; a + 1 < DA; a += 2) {
            if constexpr (Q >= 2) fma_pair(s.RS1[a], s.RS1[a + 1], -bb, -bb, o.dxa1[a], o.dxa1[a + 1]);
            fma_pair(adj0, adj1, s.RG1[a], s.RG1[a + 1], o.dxa1[a], o.dxa1[a + 1]);
            fma_pair(gda[a], gda[a + 1], s.RG1[a], s.RG1[a + 1], bb, bb);
        }
        if constexpr (DA % 2 == 1) {
            constexpr int a = DA - 1;
            if constexpr (Q >= 2) s.RS1[a] = fmaf(-bb, o.dxa1[a], s.RS1[a]);
            adj0 = fmaf(s.RG1[a], o.dxa1[a], adj0);
            gda[a] = fmaf(s.RG1[a], bb, gda[a]);
        }
        back_chain<P, k>(adj0 + adj1, bc, o.xs, s.apref, lg);
    }
    if constexpr (Q >= 2) {  // target degree P+2
        constexpr int k = P + 2;
        float bc[P + 1];
        head_chain<P, k>(bc, o.xs, s.pref);
        const float bb = bc[P];
        // the 1/2 of this stage comes with the halved table, or rides on the scalars
        constexpr bool kTable = half_table(D, Q);
        const float bbh = 0.5f * bb;
        float adj = 0.f;
#pragma unroll
        for (int a = 0; a < DA; ++a) {
            float v1;
            if constexpr (kTable) v1 = fmaf(bb, o.dxa2[a], s.RS1[a]);
            else v1 = fmaf(bbh, o.dxa1[a], s.RS1[a]);
            float av_even = 0.f, av_odd = 0.f;
#pragma unroll
            for (int c = 0; c + 1 < D; c += 2) {
                if constexpr (Q >= 3)
                    fma_pair(s.RS2[a * D + c], s.RS2[a * D + c + 1], -v1, -v1, o.dxf1[c], o.dxf1[c + 1]);
                const float g0 = s.RG2[a * D + c], g1 = s.RG2[a * D + c + 1];
                fma_pair(av_even, av_odd, g0, g1, o.dxf1[c], o.dxf1[c + 1]);
                fma_pair(gdf[c], gdf[c + 1], g0, g1, v1, v1);
            }
            if constexpr (D % 2 == 1) {
                constexpr int c = D - 1;
                if constexpr (Q >= 3) s.RS2[a * D + c] = fmaf(-v1, o.dxf1[c], s.RS2[a * D + c]);
                const float g0 = s.RG2[a * D + c];
                av_even = fmaf(g0, o.dxf1[c], av_even);
                gdf[c] = fmaf(g0, v1, gdf[c]);
            }
            const float av = av_even + av_odd;
            s.RG1[a] += av;
            if constexpr (kTable) {
                adj = fmaf(av, o.dxa2[a], adj);
                gda[a] = fmaf(av * 0.5f, bb, gda[a]);
            } else {
                adj = fmaf(av, o.dxa1[a], adj);
                gda[a] = fmaf(av, bbh, gda[a]);
            }
        }
        back_chain<P, k>(kTable ? adj : 0.5f * adj, bc, o.xs, s.apref, lg);
    }
    if constexpr (Q >= 3) {  // target degree P+3
        constexpr int k = P + 3;
        float bc[P + 1];
        head_chain<P, k>(bc, o.xs, s.pref);
        const float bb = bc[P];
        const float bb3 = bb * recip<float>(3);  // stage factors 1/3 and 1/2 ride on the scalars
        float adj = 0.f;
#pragma unroll
        for (int a = 0; a < DA; ++a) {
            const float v1 = fmaf(bb3, o.dxa1[a], s.RS1[a]);
            const float v1h = 0.5f * v1;
            float av1 = 0.f;
#pragma unroll
            for (int c = 0; c < D; ++c) {
                const float v2 = fmaf(v1h, o.dxf1[c], s.RS2[a * D + c]);
                float av2_even = 0.f, av2_odd = 0.f;
#pragma unroll
                for (int e = 0; e + 1 < D; e += 2) {
                    const float g0 = s.RG3[(a * D + c) * D + e], g1 = s.RG3[(a * D + c) * D + e + 1];
                    fma_pair(av2_even, av2_odd, g0, g1, o.dxf1[e], o.dxf1[e + 1]);
                    fma_pair(gdf[e], gdf[e + 1], g0, g1, v2, v2);
                }
                if constexpr (D % 2 == 1) {
                    constexpr int e = D - 1;
                    const float g0 = s.RG3[(a * D + c) * D + e];
                    av2_even = fmaf(g0, o.dxf1[e], av2_even);
                    gdf[e] = fmaf(g0, v2, gdf[e]);
                }
                const float av2 = av2_even + av2_odd;
                s.RG2[a * D + c] += av2;
                av1 = fmaf(av2, o.dxf1[c], av1);      // adjoint of v1h, before the 1/2
                gdf[c] = fmaf(av2, v1h, gdf[c]);
            }
            av1 *= 0.5f;                               // adjoint of v1
            s.RG1[a] += av1;
            adj = fmaf(av1, o.dxa1[a], adj);
            gda[a] = fmaf(av1, bb3, gda[a]);
        }
        back_chain<P, k>(adj * recip<float>(3), bc, o.xs, s.apref, lg);
    }
}

template <int D, int N, int P, int DA, int NT, int CHR>
struct BackwardSmem {
    static constexpr int Q = N - P;
    // One slot of D floats per thread and step; 4 floats of padding make 128-bit accesses at a
    // stride of one slot fall into distinct banks.
    static constexpr int kSlot = D + 4;
    static constexpr int kPartRow = NT * kSlot;
    static constexpr bool kHalf = half_table(D, Q);
    static constexpr int kTables = kHalf ? 2 : 1;
    static constexpr int kFloats = kTables * CHR * D + CHR * kPartRow + (CHR + 1) * D;
    static constexpr size_t kBytes = sizeof(float) * kFloats;
    // Block-wide sum of the partials: each group of kSlices adjacent lanes produces one float4
    // (4 letters of one step); used when the shape allows it, otherwise a scalar loop.
    static constexpr int kQuads = (D % 4 == 0) ? CHR * D / 4 : 1;
    static constexpr int kSlices = NT / kQuads;
#ifndef PSIG_VEC_REDUCE
#define PSIG_VEC_REDUCE 1
#endif
    static constexpr bool kVecReduce = PSIG_VEC_REDUCE && (D % 4 == 0) && (NT % kQuads == 0) && kSlices >= 1 && kSlices <= 32 &&
                                       (kSlices & (kSlices - 1)) == 0;
};

// Publish this thread's share of dL/d(dx_t) into its slot of the step's row of partials.  The
// slice for the owned first letters is folded into the full vector in registers; `split` (which
// slice this thread owns) is uniform over a block whenever the block size divides D^P, so the
// selection below does not diverge.
template <int D, int DA, int P>
__device__ __forceinline__ void publish_partials(float *mine, float (&gdf)[D], const float (&gda)[DA],
                                                 const float (&lg)[P], const int (&let)[P], int split)
{
    constexpr int SPLIT = D / DA;
#pragma unroll
    for (int s2 = 0; s2 < SPLIT; ++s2) {
        if (split == s2) {
#pragma unroll
            for (int a = 0; a < DA; ++a) gdf[s2 * DA + a] += gda[a];
        }
    }
    store_run<D>(mine, gdf, true);
#pragma unroll
    for (int j = 0; j < P; ++j) mine[let[j]] += lg[j];
}

// `accumulate` == 0: the block owns the whole path (no windows, one block per unit) and stores
// grad_path directly.  `accumulate` == 1: several blocks contribute to the same points
// (overlapping windows, or a unit split over several blocks); grad_path was zeroed and
// receives atomic adds.
template <int D, int N, int P, int DA, int NT, int CHR, int MINB>
__global__ void __launch_bounds__(NT, MINB) sig_backward_tiled(const float *__restrict__ path,
                                                               const float *__restrict__ sig,
                                                               const float *__restrict__ grad,
                                                               float *__restrict__ grad_path, long long L,
                                                               long long W, const int *__restrict__ windows,
                                                               int vec_ok, int accumulate,
                                                               const long long *__restrict__ top_words, int top_size)
{
    using S = Shape<D, N, P, DA>;
    using SM = BackwardSmem<D, N, P, DA, NT, CHR>;
    constexpr int Q = S::Q, PARTS = S::parts(NT);
    constexpr bool PADDED = S::TPU % NT != 0;  // the unit's last block has threads without work
    static_assert(NT % 4 == 0, "block size must be a multiple of 4");
    extern __shared__ __align__(16) float smem[];
    float (*s_dx)[CHR][D] = reinterpret_cast<float (*)[CHR][D]>(smem);
    float *s_part = smem + SM::kTables * CHR * D;
    float *s_red = s_part + CHR * SM::kPartRow;  // rows 0..CHR-1: reduced dL/d(dx); row CHR: carry

    const long long unit = blockIdx.x / PARTS;
    // slice-major thread order: all prefixes of slice 0, then slice 1, ... (keeps a0 block-uniform)
    constexpr int PREFIXES = ipow(D, P);
    int tu = (int)(blockIdx.x % PARTS) * NT + threadIdx.x;
    bool active = true;
    if constexpr (PADDED) {
        // idle threads shadow the unit's last thread in the loads and publish zeros
        active = tu < S::TPU;
        tu = min(tu, S::TPU - 1);
    }
    const int split = tu / PREFIXES;
    const int u = tu - split * PREFIXES;
    const int a0 = split * DA;
    int let[P];
    {
        int c = u;
#pragma unroll
        for (int j = P - 1; j >= 0; --j) { let[j] = c % D; c /= D; }
    }
    long long b; int start, steps;
    window_of(unit, L, W, windows, b, start, steps);
    if (steps == 0) return;
    const float *x = path + (b * L + start) * D;
    float *gx = grad_path + (b * L + start) * D;  // gradient at the first point of the unit

    const bool vec1 = S::kVecFirst && vec_ok, vec = S::kVecDeep && vec_ok;
    const long long width = top_words ? S::dense_off(N) + top_size : S::TOTAL;
    const float *srow = sig + unit * width;
    const float *grow = grad + unit * width;
    const long long base1 = (long long)u * D + a0;

    BackwardState<D, N, P, DA> st;
    st.pref[0] = 1.f; st.apref[0] = 0.f;
#pragma unroll
    for (int j = 1; j <= P; ++j) {
        const int span = ipow(D, P - j);  // prefixes u sharing u[:j]
        const long long idx = S::dense_off(j) + u / span;
        st.pref[j] = srow[idx];
        // the incoming gradient of a shared prefix is seeded in exactly one of its threads
        st.apref[j] = (split == 0 && u % span == 0) ? grow[idx] : 0.f;
    }
    if constexpr (Q >= 2) load_run<S::n1>(st.RS1, srow + S::dense_off(P + 1) + base1, vec1);
    if constexpr (Q >= 3) load_run<S::n2>(st.RS2, srow + S::dense_off(P + 2) + base1 * D, vec);
    if (top_words == nullptr) {
        load_run<S::n1>(st.RG1, grow + S::dense_off(P + 1) + base1, vec1);
        if constexpr (Q >= 2) load_run<S::n2>(st.RG2, grow + S::dense_off(P + 2) + base1 * D, vec);
        if constexpr (Q >= 3) load_run<S::n3>(st.RG3, grow + S::dense_off(P + 3) + base1 * D * D, vec);
    } else {
        // projected top degree: scatter the incoming gradient of the requested words into a dense
        // image of the degree (zeros elsewhere) in shared memory, then pick up the owned run
        float *s_top = s_part;  // the partials area is free until the first step
        for (int i = threadIdx.x; i < ipow(D, N); i += NT) s_top[i] = 0.f;
        block_sync<NT>();
        for (int i = threadIdx.x; i < top_size; i += NT) atomicAdd(&s_top[top_words[i]], grow[S::dense_off(N) + i]);
        block_sync<NT>();
        if constexpr (Q == 1) {
            load_run<S::n1>(st.RG1, s_top + base1, true);
        } else if constexpr (Q == 2) {
            load_run<S::n1>(st.RG1, grow + S::dense_off(P + 1) + base1, vec1);
            load_run<S::n2>(st.RG2, s_top + base1 * D, true);
        } else {
            load_run<S::n1>(st.RG1, grow + S::dense_off(P + 1) + base1, vec1);
            load_run<S::n2>(st.RG2, grow + S::dense_off(P + 2) + base1 * D, vec);
            load_run<S::n3>(st.RG3, s_top + base1 * D * D, true);
        }
        block_sync<NT>();
    }

    for (int i = threadIdx.x; i < D; i += NT) s_red[CHR * D + i] = 0.f;

    for (int c_hi = steps; c_hi > 0;) {
        const int n = min(CHR, c_hi);
        const int c0 = c_hi - n;
        block_sync<NT>();
        stage_scaled_increments<D, SM::kHalf, CHR, NT>(x, c0, n, s_dx);
        block_sync<NT>();

        float gdf[D], gda[DA], lg[P];
#if PSIG_PREFETCH_XS_BWD
        // the increments at the prefix letters feed the head of every Horner chain: fetch those
        // of the next step to be processed while the current one computes
        float xs_next[P];
#pragma unroll
        for (int j = 0; j < P; ++j) xs_next[j] = s_dx[0][n - 1][let[j]];
#endif
        if constexpr (PADDED) {
            if (!active) {
                for (int t = 0; t < n; ++t) {
                    float *slot = s_part + t * SM::kPartRow + threadIdx.x * SM::kSlot;
#pragma unroll
                    for (int e = 0; e < D; ++e) slot[e] = 0.f;
                }
            }
        }
#pragma unroll 1
        for (int t = active ? n - 1 : -1; t >= 0; --t) {
            StepOperands<D, DA, P, SM::kHalf> o;
#if PSIG_PREFETCH_XS_BWD
#pragma unroll
            for (int j = 0; j < P; ++j) o.xs[j] = xs_next[j];
            const int tn = max(t - 1, 0);
#pragma unroll
            for (int j = 0; j < P; ++j) xs_next[j] = s_dx[0][tn][let[j]];
            load_operands<D, DA, P, SM::kHalf, CHR, true>(o, s_dx, t, let, a0);
#else
            load_operands<D, DA, P, SM::kHalf, CHR>(o, s_dx, t, let, a0);
#endif
            backward_step<D, N, P, DA>(st, o, gdf, gda, lg);
            publish_partials<D, DA, P>(s_part + t * SM::kPartRow + threadIdx.x * SM::kSlot, gdf, gda, lg, let, split);
        }
        block_sync<NT>();
        // sum the partials of the block: s_red[t][e]
        if constexpr (SM::kVecReduce) {
            constexpr int SL = SM::kSlices, QPT = D / 4;
            const int quad = threadIdx.x / SL, slice = threadIdx.x % SL;
            const int t = quad / QPT, q4 = quad - t * QPT;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t < n) {
                const float *col = s_part + t * SM::kPartRow + 4 * q4;
#pragma unroll 4
                for (int i = slice; i < NT; i += SL) {
                    const float4 v = *reinterpret_cast<const float4 *>(col + i * SM::kSlot);
                    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                }
            }
#pragma unroll
            for (int off = SL / 2; off > 0; off >>= 1) {
                acc.x += __shfl_xor_sync(0xffffffffu, acc.x, off);
                acc.y += __shfl_xor_sync(0xffffffffu, acc.y, off);
                acc.z += __shfl_xor_sync(0xffffffffu, acc.z, off);
                acc.w += __shfl_xor_sync(0xffffffffu, acc.w, off);
            }
            if (slice == 0 && t < n) *reinterpret_cast<float4 *>(s_red + t * D + 4 * q4) = acc;
        } else {
            for (int o = threadIdx.x; o < n * D; o += NT) {
                const int t = o / D, e = o - t * D;
                const float *col = s_part + t * SM::kPartRow + e;
                float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
#pragma unroll 4
                for (int i = 0; i < NT; i += 4) {
                    acc0 += col[(i + 0) * SM::kSlot];
                    acc1 += col[(i + 1) * SM::kSlot];
                    acc2 += col[(i + 2) * SM::kSlot];
                    acc3 += col[(i + 3) * SM::kSlot];
                }
                s_red[o] = (acc0 + acc1) + (acc2 + acc3);
            }
        }
        block_sync<NT>();
        // grad at point p (p = c0+t+1) = g[p-1] - g[p]; g[c0+n] is the carry of the later chunk
        for (int o = threadIdx.x; o < n * D; o += NT) {
            const int t = o / D, e = o - t * D;
            const float later = (t + 1 < n) ? s_red[o + D] : s_red[CHR * D + e];
            const float v = s_red[o] - later;
            float *dst = gx + (long long)(c0 + t + 1) * D + e;
            if (accumulate) atomicAdd(dst, v); else *dst = v;
        }
        if (c0 == 0) {
            for (int e = threadIdx.x; e < D; e += NT) {
                if (accumulate) atomicAdd(gx + e, -s_red[e]); else gx[e] = -s_red[e];
            }
        }
        block_sync<NT>();
        for (int e = threadIdx.x; e < D; e += NT) s_red[CHR * D + e] = s_red[e];
        c_hi = c0;
    }
}

// ------------------------------------------------------------------------------------------
// configurations
// ------------------------------------------------------------------------------------------
template <int D_, int N_, int PF_, int DAF_, int NTF_, int MINBF_, int PB_, int DAB_, int NTB_, int CHR_, int MINBB_>
struct Config {
    static constexpr int D = D_, N = N_;
    static constexpr int PF = PF_, PB = PB_;  // prefix length owned by a thread, forward / backward
    static constexpr int DAF = DAF_, NTF = NTF_, MINBF = MINBF_;            // forward: first-letter tile, block, min blocks/SM
    static constexpr int DAB = DAB_, NTB = NTB_, CHR = CHR_, MINBB = MINBB_;  // backward
};

// Tunables (each overridable with -D for experiments): forward first-letter tile / block size /
// minimum resident blocks per SM, then the same for backward plus the steps per reduction chunk.
#ifndef PSIG_84_DAF
#define PSIG_84_DAF 8
#endif
#ifndef PSIG_84_NTF
#define PSIG_84_NTF 64
#endif
#ifndef PSIG_84_MINBF
#define PSIG_84_MINBF 1
#endif
#ifndef PSIG_84_DAB
#define PSIG_84_DAB 8
#endif
#ifndef PSIG_84_NTB
#define PSIG_84_NTB 64
#endif
#ifndef PSIG_84_CHR
#define PSIG_84_CHR 8
#endif
#ifndef PSIG_84_MINBB
#define PSIG_84_MINBB 8
#endif
#ifndef PSIG_164_DAF
#define PSIG_164_DAF 8
#endif
#ifndef PSIG_164_NTF
#define PSIG_164_NTF 128
#endif
#ifndef PSIG_164_MINBF
#define PSIG_164_MINBF 3
#endif
#ifndef PSIG_164_DAB
#define PSIG_164_DAB 8
#endif
#ifndef PSIG_164_NTB
#define PSIG_164_NTB 32
#endif
#ifndef PSIG_164_CHR
#define PSIG_164_CHR 8
#endif
#ifndef PSIG_164_MINBB
#define PSIG_164_MINBB 1
#endif
#ifndef PSIG_84_PF
#define PSIG_84_PF 2
#endif
#ifndef PSIG_84_PB
#define PSIG_84_PB 2
#endif
#define PSIG_CFG_8_4 8, 4, PSIG_84_PF, PSIG_84_DAF, PSIG_84_NTF, PSIG_84_MINBF, PSIG_84_PB, PSIG_84_DAB, PSIG_84_NTB, PSIG_84_CHR, PSIG_84_MINBB
#define PSIG_CFG_16_4 16, 4, 2, PSIG_164_DAF, PSIG_164_NTF, PSIG_164_MINBF, 2, PSIG_164_DAB, PSIG_164_NTB, PSIG_164_CHR, PSIG_164_MINBB
#define PSIG_CFG_16_3 16, 3, 1, 8, 32, 1, 1, 4, 64, 8, 1
#ifndef PSIG_46_DAF
#define PSIG_46_DAF 4
#endif
#ifndef PSIG_46_NTF
#define PSIG_46_NTF 64
#endif
#ifndef PSIG_46_MINBF
#define PSIG_46_MINBF 1
#endif
#ifndef PSIG_46_DAB
#define PSIG_46_DAB 4
#endif
#ifndef PSIG_46_NTB
#define PSIG_46_NTB 64
#endif
#ifndef PSIG_46_CHR
#define PSIG_46_CHR 8
#endif
#ifndef PSIG_46_MINBB
#define PSIG_46_MINBB 1
#endif
#define PSIG_CFG_4_6 4, 6, 3, PSIG_46_DAF, PSIG_46_NTF, PSIG_46_MINBF, 3, PSIG_46_DAB, PSIG_46_NTB, PSIG_46_CHR, PSIG_46_MINBB
using Cfg_8_4 = Config<PSIG_CFG_8_4>;
using Cfg_16_4 = Config<PSIG_CFG_16_4>;
using Cfg_16_3 = Config<PSIG_CFG_16_3>;
using Cfg_4_6 = Config<PSIG_CFG_4_6>;

// Further shapes, not tuned one by one: the prefix length leaves a sub-tree of two or three degrees
// that fits the registers, the block is the unit's thread count rounded up to whole warps (one
// block per unit where that is at most 256 threads, so that a projected top degree is served too).
//                      D  N  PF DAF NTF MINBF PB DAB NTB CHR MINBB
using Cfg_3_5 = Config<3, 5, 3, 3, 32, 1, 3, 3, 32, 8, 1>;
using Cfg_3_6 = Config<3, 6, 3, 3, 32, 1, 3, 3, 32, 8, 1>;
using Cfg_3_7 = Config<3, 7, 4, 3, 96, 1, 4, 3, 96, 8, 1>;
using Cfg_4_4 = Config<4, 4, 2, 4, 32, 1, 2, 4, 32, 8, 1>;
using Cfg_4_5 = Config<4, 5, 3, 4, 64, 1, 3, 4, 64, 8, 1>;
using Cfg_4_7 = Config<4, 7, 4, 4, 64, 1, 4, 4, 64, 8, 1>;
using Cfg_5_4 = Config<5, 4, 2, 5, 32, 1, 2, 5, 32, 8, 1>;
using Cfg_5_5 = Config<5, 5, 3, 5, 128, 1, 3, 5, 128, 8, 1>;
using Cfg_5_6 = Config<5, 6, 3, 1, 128, 1, 3, 1, 128, 8, 1>;
using Cfg_6_4 = Config<6, 4, 2, 3, 96, 1, 2, 3, 96, 8, 1>;
using Cfg_6_5 = Config<6, 5, 3, 6, 224, 1, 3, 6, 224, 8, 1>;
using Cfg_8_3 = Config<8, 3, 1, 2, 32, 1, 1, 2, 32, 8, 1>;
using Cfg_8_5 = Config<8, 5, 3, 8, 64, 1, 3, 8, 64, 8, 1>;
using Cfg_8_6 = Config<8, 6, 4, 8, 64, 1, 4, 8, 64, 8, 1>;
using Cfg_10_3 = Config<10, 3, 1, 2, 64, 1, 1, 2, 64, 8, 1>;
using Cfg_10_4 = Config<10, 4, 2, 5, 224, 1, 2, 5, 224, 8, 1>;
using Cfg_12_3 = Config<12, 3, 1, 2, 96, 1, 1, 2, 96, 8, 1>;
using Cfg_16_2 = Config<16, 2, 1, 8, 32, 1, 1, 8, 32, 8, 1>;
using Cfg_32_2 = Config<32, 2, 1, 8, 128, 1, 1, 8, 128, 8, 1>;
using Cfg_32_3 = Config<32, 3, 1, 2, 128, 1, 1, 2, 128, 4, 1>;

template <typename F>
bool dispatch(int d, int depth, F &&f)
{
#define PSIG_TRY(DD, NN) if (d == DD && depth == NN) { f(Cfg_##DD##_##NN{}); return true; }
    PSIG_TRY(8, 4) PSIG_TRY(16, 4) PSIG_TRY(16, 3) PSIG_TRY(4, 6)
    PSIG_TRY(3, 5) PSIG_TRY(3, 6) PSIG_TRY(3, 7)
    PSIG_TRY(4, 4) PSIG_TRY(4, 5) PSIG_TRY(4, 7)
    PSIG_TRY(5, 4) PSIG_TRY(5, 5) PSIG_TRY(5, 6)
    PSIG_TRY(6, 4) PSIG_TRY(6, 5)
    PSIG_TRY(8, 3) PSIG_TRY(8, 5) PSIG_TRY(8, 6)
    PSIG_TRY(10, 3) PSIG_TRY(10, 4) PSIG_TRY(12, 3)
    PSIG_TRY(16, 2) PSIG_TRY(32, 2) PSIG_TRY(32, 3)
#undef PSIG_TRY
    return false;
}

#ifndef PSIG_BULK_COPIES
#define PSIG_BULK_COPIES 1
#endif
constexpr bool kUseBulkCopies = PSIG_BULK_COPIES != 0;

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Largest dense top degree (floats) that the projected-top epilogue stages in shared memory.
constexpr long long kMaxStagedTop = 8192;

// Row layouts the tiled kernels accept: all degrees dense (also when a projection lists every
// degree as complete), or every degree below the top dense and the top degree an explicit word
// list (the layout LogSignature asks for).
enum class RowKind { kUnsupported, kDense, kProjectedTop };

RowKind classify_rows(const PsigSigDesc &desc, long long *top_size)
{
    *top_size = 0;
    if (!desc.projected) return RowKind::kDense;
    long long d_pow = 1;
    for (int k = 1; k < desc.depth; ++k) {
        d_pow *= desc.d;
        if (desc.level_sizes[k] != d_pow) return RowKind::kUnsupported;
    }
    d_pow *= desc.d;
    const long long top = desc.level_sizes[desc.depth];
    if (top == d_pow) return RowKind::kDense;
    if (top < 0 || top > 0x7fffffffLL || d_pow > kMaxStagedTop) return RowKind::kUnsupported;
    *top_size = top;
    return RowKind::kProjectedTop;
}

}  // namespace

bool tiled_supported(const PsigSigDesc &desc)
{
    if (desc.dtype != PSIG_F32) return false;
    bool one_block_per_unit = false;
    const bool known = dispatch(desc.d, desc.depth, [&](auto cfg) {
        using C = decltype(cfg);
        one_block_per_unit = Shape<C::D, C::N, C::PF, C::DAF>::parts(C::NTF) == 1 &&
                             Shape<C::D, C::N, C::PB, C::DAB>::parts(C::NTB) == 1;
    });
    if (!known) return false;
    long long top_size = 0;
    const RowKind kind = classify_rows(desc, &top_size);
    return kind == RowKind::kDense || (kind == RowKind::kProjectedTop && one_block_per_unit);
}

int tiled_sig_forward(const PsigSigDesc &desc, const float *path, float *out, cudaStream_t stream)
{
    const long long W = desc.W > 0 ? desc.W : 1;
    const long long units = desc.B * W;
    if (units == 0) return PSIG_OK;
    long long top_size = 0;
    const bool projected = classify_rows(desc, &top_size) == RowKind::kProjectedTop;
    int rc = PSIG_ERR_UNSUPPORTED;
    dispatch(desc.d, desc.depth, [&](auto cfg) {
        using C = decltype(cfg);
        using S = Shape<C::D, C::N, C::PF, C::DAF>;
        constexpr int PARTS = S::parts(C::NTF);
        const long long blocks = units * PARTS;
        if (blocks > 0x7fffffffLL) { rc = PSIG_ERR_TOO_LARGE; return; }
        const long long width = projected ? S::dense_off(C::N) + top_size : S::TOTAL;
        const size_t smem = projected ? sizeof(float) * (size_t)ipow(C::D, C::N) : 0;
        const int vec = (aligned16(out) && width % 4 == 0) ? 1 : 0;
        const int *win = desc.W > 0 ? desc.windows : nullptr;
        const long long *words = projected ? reinterpret_cast<const long long *>(desc.words) : nullptr;
        // Bulk (TMA) staging pays off when a unit has several chunks, so that the next chunk's copy
        // overlaps the current chunk's arithmetic; short units (one chunk) are faster with plain loads.
        const bool bulk = kUseBulkCopies && C::D % 4 == 0 && aligned16(path) && desc.W == 0 && desc.L - 1 > kFwdChunk;
        auto launch = [&](auto kernel) {
            kernel<<<(unsigned)blocks, C::NTF, smem, stream>>>(path, out, desc.L, W, win, vec, words, (int)top_size);
        };
        constexpr bool kBulkOk = C::D % 4 == 0;             // rows of whole 16-byte pieces
        constexpr bool kProjOk = S::parts(C::NTF) == 1;     // the block holds the whole unit
        if (projected) {
            if constexpr (kProjOk) {
                if constexpr (kBulkOk) {
                    if (bulk) { launch(sig_forward_tiled<C::D, C::N, C::PF, C::DAF, C::NTF, C::MINBF, true, true>); goto done; }
                }
                launch(sig_forward_tiled<C::D, C::N, C::PF, C::DAF, C::NTF, C::MINBF, true, false>);
            } else {
                return;  // tiled_supported() said no
            }
        } else {
            if constexpr (kBulkOk) {
                if (bulk) { launch(sig_forward_tiled<C::D, C::N, C::PF, C::DAF, C::NTF, C::MINBF, false, true>); goto done; }
            }
            launch(sig_forward_tiled<C::D, C::N, C::PF, C::DAF, C::NTF, C::MINBF, false, false>);
        }
    done:
        rc = check_launch();
    });
    return rc;
}

int64_t tiled_sig_backward_workspace(const PsigSigDesc &) { return 0; }

int tiled_sig_backward(const PsigSigDesc &desc, const float *path, const float *sig, const float *grad,
                       float *grad_path, void *, cudaStream_t stream)
{
    const long long W = desc.W > 0 ? desc.W : 1;
    const long long units = desc.B * W;
    long long top_size = 0;
    const bool projected = classify_rows(desc, &top_size) == RowKind::kProjectedTop;
    int rc = PSIG_ERR_UNSUPPORTED;
    dispatch(desc.d, desc.depth, [&](auto cfg) {
        using C = decltype(cfg);
        using S = Shape<C::D, C::N, C::PB, C::DAB>;
        using SM = BackwardSmem<C::D, C::N, C::PB, C::DAB, C::NTB, C::CHR>;
        constexpr int PARTS = S::parts(C::NTB);
        const long long blocks = units * PARTS;
        if (blocks > 0x7fffffffLL) { rc = PSIG_ERR_TOO_LARGE; return; }
        // Several blocks add into the same points when windows overlap or a unit spans blocks.
        const bool accumulate = desc.W > 0 || PARTS > 1;
        if (accumulate) {
            const size_t bytes = sizeof(float) * (size_t)desc.B * (size_t)desc.L * desc.d;
            if (cudaMemsetAsync(grad_path, 0, bytes, stream) != cudaSuccess) { rc = PSIG_ERR_CUDA; return; }
        }
        // the projected-top prologue stages D^N floats in the partials area
        size_t smem = SM::kBytes;
        if (projected) {
            const size_t need = sizeof(float) * ((size_t)SM::kTables * C::CHR * C::D + (size_t)ipow(C::D, C::N));
            if (need > smem) smem = need;
        }
        auto kernel = sig_backward_tiled<C::D, C::N, C::PB, C::DAB, C::NTB, C::CHR, C::MINBB>;
        if (smem > 48 * 1024) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
                rc = PSIG_ERR_CUDA; return;
            }
        }
        if (blocks > 0) {
            const long long width = projected ? S::dense_off(C::N) + top_size : S::TOTAL;
            const bool vec = aligned16(sig) && aligned16(grad) && width % 4 == 0;
            kernel<<<(unsigned)blocks, C::NTB, smem, stream>>>(
                path, sig, grad, grad_path, desc.L, W, desc.W > 0 ? desc.windows : nullptr, vec ? 1 : 0,
                accumulate ? 1 : 0, projected ? reinterpret_cast<const long long *>(desc.words) : nullptr,
                (int)top_size);
        }
        rc = check_launch();
    });
    return rc;
}

}  // namespace psig
