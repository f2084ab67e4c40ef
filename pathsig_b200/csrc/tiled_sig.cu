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
    static constexpr bool kVecLayout = (D % 4 == 0) && (DA % 4 == 0);
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

__device__ __forceinline__ void window_of(long long unit, long long L, long long W, const int *windows,
                                          long long &b, int &start, int &steps)
{
    b = unit / W;
    start = 0;
    int end = (int)L;
    if (windows) {
        const long long w = unit % W;
        start = windows[2 * w];
        end = windows[2 * w + 1];
    }
    steps = max(end - start - 1, 0);
}

// s_dx[r][t][a] = dx_{c0+t}[a] / (r+1) for r < Q.
template <int D, int Q, int CH, int NT>
__device__ __forceinline__ void stage_scaled_increments(const float *__restrict__ x, int c0, int n,
                                                        float (*s_dx)[CH][D])
{
    const float *lo = x + (long long)c0 * D;
    for (int i = threadIdx.x; i < n * D; i += NT) {
        const float v = lo[i + D] - lo[i];
        (&s_dx[0][0][0])[i] = v;
        if constexpr (Q >= 2) (&s_dx[1][0][0])[i] = v * 0.5f;
        if constexpr (Q >= 3) (&s_dx[2][0][0])[i] = v * recip<float>(3);
    }
}

// ------------------------------------------------------------------------------------------
// forward
// ------------------------------------------------------------------------------------------
constexpr int kFwdChunk = 32;

template <int D, int N, int P, int DA, int NT>
__global__ void __launch_bounds__(NT) sig_forward_tiled(const float *__restrict__ path, float *__restrict__ out,
                                                        long long L, long long W, const int *__restrict__ windows,
                                                        int vec_ok)
{
    using S = Shape<D, N, P, DA>;
    constexpr int Q = S::Q, PARTS = S::TPU / NT, CH = kFwdChunk;
    static_assert(S::TPU % NT == 0, "block size must divide the threads of a unit");
    __shared__ __align__(16) float s_dx[Q][CH][D];

    const long long unit = blockIdx.x / PARTS;
    const int tu = (int)(blockIdx.x % PARTS) * NT + threadIdx.x;
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

    float pref[P + 1];
    float R1[S::n1], R2[at_least_one(S::n2)], R3[at_least_one(S::n3)];
#pragma unroll
    for (int j = 0; j <= P; ++j) pref[j] = 0.f;
#pragma unroll
    for (int i = 0; i < S::n1; ++i) R1[i] = 0.f;
#pragma unroll
    for (int i = 0; i < at_least_one(S::n2); ++i) R2[i] = 0.f;
#pragma unroll
    for (int i = 0; i < at_least_one(S::n3); ++i) R3[i] = 0.f;

    for (int c0 = 0; c0 < steps; c0 += CH) {
        const int n = min(CH, steps - c0);
        __syncthreads();
        stage_scaled_increments<D, Q, CH, NT>(x, c0, n, s_dx);
        __syncthreads();
#pragma unroll 1
        for (int t = 0; t < n; ++t) {
            const float *row = s_dx[0][t];
            float xs[P];
#pragma unroll
            for (int j = 0; j < P; ++j) xs[j] = row[let[j]];
            float dxf1[D], dxa1[DA];
            load_run<D>(dxf1, row, true);
            if constexpr (DA == D) {
#pragma unroll
                for (int a = 0; a < DA; ++a) dxa1[a] = dxf1[a];
            } else {
                load_run<DA>(dxa1, row + a0, true);
            }

            if constexpr (Q >= 3) {  // target degree P+3
                constexpr int k = P + 3;
                float dxa3[DA], dxf2[D];
                load_run<DA>(dxa3, s_dx[2][t] + a0, true);
                load_run<D>(dxf2, s_dx[1][t], true);
                float bb = 1.f;
#pragma unroll
                for (int j = 1; j <= P; ++j) bb = fmaf(bb, xs[j - 1] * recip<float>(k - j + 1), pref[j]);
#pragma unroll
                for (int a = 0; a < DA; ++a) {
                    const float v1 = fmaf(bb, dxa3[a], R1[a]);
#pragma unroll
                    for (int c = 0; c < D; ++c) {
                        const float v2 = fmaf(v1, dxf2[c], R2[a * D + c]);
#pragma unroll
                        for (int e = 0; e < D; ++e) R3[(a * D + c) * D + e] = fmaf(v2, dxf1[e], R3[(a * D + c) * D + e]);
                    }
                }
            }
            if constexpr (Q >= 2) {  // target degree P+2
                constexpr int k = P + 2;
                float dxa2[DA];
                load_run<DA>(dxa2, s_dx[1][t] + a0, true);
                float bb = 1.f;
#pragma unroll
                for (int j = 1; j <= P; ++j) bb = fmaf(bb, xs[j - 1] * recip<float>(k - j + 1), pref[j]);
#pragma unroll
                for (int a = 0; a < DA; ++a) {
                    const float v1 = fmaf(bb, dxa2[a], R1[a]);
#pragma unroll
                    for (int c = 0; c < D; ++c) R2[a * D + c] = fmaf(v1, dxf1[c], R2[a * D + c]);
                }
            }
            {  // target degree P+1
                constexpr int k = P + 1;
                float bb = 1.f;
#pragma unroll
                for (int j = 1; j <= P; ++j) bb = fmaf(bb, xs[j - 1] * recip<float>(k - j + 1), pref[j]);
#pragma unroll
                for (int a = 0; a < DA; ++a) R1[a] = fmaf(bb, dxa1[a], R1[a]);
            }
            // the shared prefixes, highest first
#pragma unroll
            for (int m = P; m >= 1; --m) {
                float bm = 1.f;
#pragma unroll
                for (int j = 1; j <= m - 1; ++j) bm = fmaf(bm, xs[j - 1] * recip<float>(m - j + 1), pref[j]);
                pref[m] = fmaf(bm, xs[m - 1], pref[m]);
            }
        }
    }

    float *row = out + unit * S::TOTAL;
    const bool vec = S::kVecLayout && vec_ok;
#pragma unroll
    for (int j = 1; j <= P; ++j) {
        const int span = ipow(D, P - j) * S::SPLIT;  // threads sharing the prefix of length j
        if (tu % span == 0) row[S::dense_off(j) + tu / span] = pref[j];
    }
    const long long base1 = (long long)u * D + a0;
    store_run<S::n1>(row + S::dense_off(P + 1) + base1, R1, vec);
    if constexpr (Q >= 2) store_run<S::n2>(row + S::dense_off(P + 2) + base1 * D, R2, vec);
    if constexpr (Q >= 3) store_run<S::n3>(row + S::dense_off(P + 3) + base1 * D * D, R3, vec);
}

// ------------------------------------------------------------------------------------------
// backward
// ------------------------------------------------------------------------------------------

// Push the adjoint `adj` of the scalar Horner value at prefix length P of target degree k down
// to the root: adds to the partial adjoints of the shared prefixes and to the letter gradients.
template <int P, int K>
__device__ __forceinline__ void back_chain(float adj, const float (&bc)[P + 1], const float (&xs)[P],
                                           float (&apref)[P + 1], float (&lg)[P])
{
#pragma unroll
    for (int j = P; j >= 1; --j) {
        apref[j] += adj;
        constexpr float one = 1.f;
        const float c = one / float(K - j + 1);
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

template <int D, int N, int P, int DA, int NT, int CHR>
struct BackwardSmem {
    static constexpr int Q = N - P;
    static constexpr int kPartRow = NT * D + D;  // one step of per-thread partials (+D floats of padding)
    static constexpr int kFloats = Q * CHR * D + CHR * kPartRow + (CHR + 1) * D;
    static constexpr size_t kBytes = sizeof(float) * kFloats;
};

template <int D, int N, int P, int DA, int NT, int CHR>
__global__ void __launch_bounds__(NT) sig_backward_tiled(const float *__restrict__ path,
                                                         const float *__restrict__ sig,
                                                         const float *__restrict__ grad,
                                                         float *__restrict__ grad_path,
                                                         float *__restrict__ inc_grad, long long L, long long W,
                                                         const int *__restrict__ windows, int vec_ok)
{
    using S = Shape<D, N, P, DA>;
    using SM = BackwardSmem<D, N, P, DA, NT, CHR>;
    constexpr int Q = S::Q, PARTS = S::TPU / NT;
    static_assert(S::TPU % NT == 0, "block size must divide the threads of a unit");
    extern __shared__ __align__(16) float smem[];
    float (*s_dx)[CHR][D] = reinterpret_cast<float (*)[CHR][D]>(smem);
    float *s_part = smem + Q * CHR * D;
    float *s_red = s_part + CHR * SM::kPartRow;  // rows 0..CHR-1: reduced dL/d(dx); row CHR: carry

    const long long unit = blockIdx.x / PARTS;
    const int tu = (int)(blockIdx.x % PARTS) * NT + threadIdx.x;
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
    if (steps == 0) return;
    const float *x = path + (b * L + start) * D;
    // Direct mode: this block owns the whole path, so it writes grad_path itself.
    const bool direct = (inc_grad == nullptr);
    float *gx = grad_path + b * L * D;
    float *gd = direct ? nullptr : inc_grad + (b * (L - 1) + start) * D;

    const bool vec = S::kVecLayout && vec_ok;
    const float *srow = sig + unit * S::TOTAL;
    const float *grow = grad + unit * S::TOTAL;
    const long long base1 = (long long)u * D + a0;

    float pref[P + 1], apref[P + 1];
    pref[0] = 1.f; apref[0] = 0.f;
#pragma unroll
    for (int j = 1; j <= P; ++j) {
        const int span = ipow(D, P - j) * S::SPLIT;
        const long long idx = S::dense_off(j) + tu / span;
        pref[j] = srow[idx];
        apref[j] = (tu % span == 0) ? grow[idx] : 0.f;
    }
    float RS1[S::n1], RS2[at_least_one(S::n2)];          // S at degrees P+1, P+2 (when below N)
    float RG1[S::n1], RG2[at_least_one(S::n2)], RG3[at_least_one(S::n3)];
    if constexpr (Q >= 2) load_run<S::n1>(RS1, srow + S::dense_off(P + 1) + base1, vec);
    if constexpr (Q >= 3) load_run<S::n2>(RS2, srow + S::dense_off(P + 2) + base1 * D, vec);
    load_run<S::n1>(RG1, grow + S::dense_off(P + 1) + base1, vec);
    if constexpr (Q >= 2) load_run<S::n2>(RG2, grow + S::dense_off(P + 2) + base1 * D, vec);
    if constexpr (Q >= 3) load_run<S::n3>(RG3, grow + S::dense_off(P + 3) + base1 * D * D, vec);

    for (int i = threadIdx.x; i < D; i += NT) s_red[CHR * D + i] = 0.f;

    for (int c_hi = steps; c_hi > 0;) {
        const int n = min(CHR, c_hi);
        const int c0 = c_hi - n;
        __syncthreads();
        stage_scaled_increments<D, Q, CHR, NT>(x, c0, n, s_dx);
        __syncthreads();

#pragma unroll 1
        for (int t = n - 1; t >= 0; --t) {
            const float *row = s_dx[0][t];
            float xs[P], lg[P];
#pragma unroll
            for (int j = 0; j < P; ++j) { xs[j] = row[let[j]]; lg[j] = 0.f; }
            float dxf1[D], dxa1[DA], gdf[D], gda[DA];
            load_run<D>(dxf1, row, true);
            if constexpr (DA == D) {
#pragma unroll
                for (int a = 0; a < DA; ++a) dxa1[a] = dxf1[a];
            } else {
                load_run<DA>(dxa1, row + a0, true);
            }
#pragma unroll
            for (int e = 0; e < D; ++e) gdf[e] = 0.f;
#pragma unroll
            for (int a = 0; a < DA; ++a) gda[a] = 0.f;

            // shared prefixes, bottom-up: roll back, then transpose
#pragma unroll
            for (int m = 1; m <= P; ++m) {
                float bc[P + 1];
                bc[0] = 1.f;
#pragma unroll
                for (int j = 1; j <= m - 1; ++j) bc[j] = fmaf(bc[j - 1], xs[j - 1] * (1.f / float(m - j + 1)), pref[j]);
                pref[m] = fmaf(-bc[m - 1], xs[m - 1], pref[m]);
                const float a = apref[m];
                lg[m - 1] = fmaf(a, bc[m - 1], lg[m - 1]);
                float adj = a * xs[m - 1];
#pragma unroll
                for (int j = m - 1; j >= 1; --j) {
                    apref[j] += adj;
                    const float c = 1.f / float(m - j + 1);
                    lg[j - 1] = fmaf(adj * c, bc[j - 1], lg[j - 1]);
                    adj = adj * (xs[j - 1] * c);
                }
            }
            {  // target degree P+1
                constexpr int k = P + 1;
                float bc[P + 1];
                head_chain<P, k>(bc, xs, pref);
                const float bb = bc[P];
                float adj = 0.f;
#pragma unroll
                for (int a = 0; a < DA; ++a) {
                    if constexpr (Q >= 2) RS1[a] = fmaf(-bb, dxa1[a], RS1[a]);
                    adj = fmaf(RG1[a], dxa1[a], adj);
                    gda[a] = fmaf(RG1[a], bb, gda[a]);
                }
                back_chain<P, k>(adj, bc, xs, apref, lg);
            }
            if constexpr (Q >= 2) {  // target degree P+2
                constexpr int k = P + 2;
                float dxa2[DA];
                load_run<DA>(dxa2, s_dx[1][t] + a0, true);
                float bc[P + 1];
                head_chain<P, k>(bc, xs, pref);
                const float bb = bc[P];
                float adj = 0.f;
#pragma unroll
                for (int a = 0; a < DA; ++a) {
                    const float v1 = fmaf(bb, dxa2[a], RS1[a]);
                    float av = 0.f;
#pragma unroll
                    for (int c = 0; c < D; ++c) {
                        if constexpr (Q >= 3) RS2[a * D + c] = fmaf(-v1, dxf1[c], RS2[a * D + c]);
                        const float g = RG2[a * D + c];
                        av = fmaf(g, dxf1[c], av);
                        gdf[c] = fmaf(g, v1, gdf[c]);
                    }
                    RG1[a] += av;
                    adj = fmaf(av, dxa2[a], adj);
                    gda[a] = fmaf(av * 0.5f, bb, gda[a]);
                }
                back_chain<P, k>(adj, bc, xs, apref, lg);
            }
            if constexpr (Q >= 3) {  // target degree P+3
                constexpr int k = P + 3;
                float dxa3[DA], dxf2[D];
                load_run<DA>(dxa3, s_dx[2][t] + a0, true);
                load_run<D>(dxf2, s_dx[1][t], true);
                float bc[P + 1];
                head_chain<P, k>(bc, xs, pref);
                const float bb = bc[P];
                float adj = 0.f;
#pragma unroll
                for (int a = 0; a < DA; ++a) {
                    const float v1 = fmaf(bb, dxa3[a], RS1[a]);
                    float av1 = 0.f;
#pragma unroll
                    for (int c = 0; c < D; ++c) {
                        const float v2 = fmaf(v1, dxf2[c], RS2[a * D + c]);
                        float av2 = 0.f;
#pragma unroll
                        for (int e = 0; e < D; ++e) {
                            const float g = RG3[(a * D + c) * D + e];
                            av2 = fmaf(g, dxf1[e], av2);
                            gdf[e] = fmaf(g, v2, gdf[e]);
                        }
                        RG2[a * D + c] += av2;
                        av1 = fmaf(av2, dxf2[c], av1);
                        gdf[c] = fmaf(av2 * 0.5f, v1, gdf[c]);
                    }
                    RG1[a] += av1;
                    adj = fmaf(av1, dxa3[a], adj);
                    gda[a] = fmaf(av1 * recip<float>(3), bb, gda[a]);
                }
                back_chain<P, k>(adj, bc, xs, apref, lg);
            }

            // publish this thread's share of dL/d(dx_t)
            float *mine = s_part + t * SM::kPartRow + threadIdx.x * D;
            if constexpr (DA == D) {
#pragma unroll
                for (int e = 0; e < D; ++e) gdf[e] += gda[e];
            }
            store_run<D>(mine, gdf, true);
            if constexpr (DA != D) {
#pragma unroll
                for (int a = 0; a < DA; ++a) mine[a0 + a] += gda[a];
            }
#pragma unroll
            for (int j = 0; j < P; ++j) mine[let[j]] += lg[j];
        }
        __syncthreads();
        // sum the partials of the block: s_red[t][e]
        for (int o = threadIdx.x; o < n * D; o += NT) {
            const int t = o / D, e = o - t * D;
            const float *col = s_part + t * SM::kPartRow + e;
            float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
#pragma unroll 4
            for (int i = 0; i < NT; i += 4) {
                acc0 += col[(i + 0) * D];
                acc1 += col[(i + 1) * D];
                acc2 += col[(i + 2) * D];
                acc3 += col[(i + 3) * D];
            }
            s_red[o] = (acc0 + acc1) + (acc2 + acc3);
        }
        __syncthreads();
        if (direct) {
            // grad_path[p] = g[p-1] - g[p]; g[c0+n] is the carry of the chunk processed before
            for (int o = threadIdx.x; o < n * D; o += NT) {
                const int t = o / D, e = o - t * D;  // point p = c0 + t + 1
                const float later = (t + 1 < n) ? s_red[o + D] : s_red[CHR * D + e];
                gx[(long long)(start + c0 + t + 1) * D + e] = s_red[o] - later;
            }
            if (c0 == 0)
                for (int e = threadIdx.x; e < D; e += NT) gx[(long long)start * D + e] = -s_red[e];
            __syncthreads();
            for (int e = threadIdx.x; e < D; e += NT) s_red[CHR * D + e] = s_red[e];
        } else {
            for (int o = threadIdx.x; o < n * D; o += NT) atomicAdd(&gd[(long long)c0 * D + o], s_red[o]);
        }
        c_hi = c0;
    }
}

template <typename T>
__global__ void increments_to_points_f32(const T *__restrict__ inc_grad, T *__restrict__ path_grad, long long B,
                                         long long L, int d)
{
    const long long total = B * L * d;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long b = i / (L * d);
        const long long r = i - b * L * d;
        const long long t = r / d;
        const int a = (int)(r - t * d);
        const T *g = inc_grad + b * (L - 1) * d + a;
        const T after = (t < L - 1) ? g[t * d] : T(0);
        const T before = (t > 0) ? g[(t - 1) * d] : T(0);
        path_grad[i] = before - after;
    }
}

// ------------------------------------------------------------------------------------------
// configurations
// ------------------------------------------------------------------------------------------
template <int D_, int N_, int P_, int DAF_, int NTF_, int DAB_, int NTB_, int CHR_>
struct Config {
    static constexpr int D = D_, N = N_, P = P_;
    static constexpr int DAF = DAF_, NTF = NTF_;  // forward: first-letter tile, block size
    static constexpr int DAB = DAB_, NTB = NTB_, CHR = CHR_;  // backward
};

//                   D  N  P  fwd(DA,NT)  bwd(DA,NT,CHR)
using Cfg_8_4 = Config<8, 4, 2, 8, 64, 8, 64, 8>;
using Cfg_8_3 = Config<8, 3, 1, 8, 8, 8, 8, 8>;
using Cfg_16_4 = Config<16, 4, 2, 8, 256, 4, 256, 4>;
using Cfg_16_3 = Config<16, 3, 1, 8, 32, 4, 64, 8>;
using Cfg_4_6 = Config<4, 6, 3, 4, 64, 4, 64, 8>;
using Cfg_4_5 = Config<4, 5, 2, 4, 16, 4, 16, 8>;
using Cfg_4_4 = Config<4, 4, 2, 4, 16, 4, 16, 8>;

template <typename F>
bool dispatch(int d, int depth, F &&f)
{
    if (d == 8 && depth == 4) { f(Cfg_8_4{}); return true; }
    if (d == 16 && depth == 4) { f(Cfg_16_4{}); return true; }
    if (d == 16 && depth == 3) { f(Cfg_16_3{}); return true; }
    if (d == 4 && depth == 6) { f(Cfg_4_6{}); return true; }
    return false;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

bool tiled_supported(int d, int depth)
{
    return dispatch(d, depth, [](auto) {});
}

int tiled_sig_forward(const PsigSigDesc &desc, const float *path, float *out, cudaStream_t stream)
{
    const long long W = desc.W > 0 ? desc.W : 1;
    const long long units = desc.B * W;
    if (units == 0) return PSIG_OK;
    int rc = PSIG_ERR_UNSUPPORTED;
    dispatch(desc.d, desc.depth, [&](auto cfg) {
        using C = decltype(cfg);
        using S = Shape<C::D, C::N, C::P, C::DAF>;
        constexpr int PARTS = S::TPU / C::NTF;
        const long long blocks = units * PARTS;
        if (blocks > 0x7fffffffLL) { rc = PSIG_ERR_TOO_LARGE; return; }
        sig_forward_tiled<C::D, C::N, C::P, C::DAF, C::NTF><<<(unsigned)blocks, C::NTF, 0, stream>>>(
            path, out, desc.L, W, desc.W > 0 ? desc.windows : nullptr, aligned16(out) ? 1 : 0);
        rc = check_launch();
    });
    return rc;
}

namespace {
template <typename C>
bool backward_needs_scratch(const PsigSigDesc &desc)
{
    using S = Shape<C::D, C::N, C::P, C::DAB>;
    return desc.W > 0 || (S::TPU / C::NTB) > 1;
}
}  // namespace

int64_t tiled_sig_backward_workspace(const PsigSigDesc &desc)
{
    int64_t bytes = 0;
    dispatch(desc.d, desc.depth, [&](auto cfg) {
        using C = decltype(cfg);
        if (backward_needs_scratch<C>(desc)) bytes = (int64_t)sizeof(float) * desc.B * (desc.L - 1) * desc.d;
    });
    return bytes;
}

int tiled_sig_backward(const PsigSigDesc &desc, const float *path, const float *sig, const float *grad,
                       float *grad_path, void *workspace, cudaStream_t stream)
{
    const long long W = desc.W > 0 ? desc.W : 1;
    const long long units = desc.B * W;
    int rc = PSIG_ERR_UNSUPPORTED;
    dispatch(desc.d, desc.depth, [&](auto cfg) {
        using C = decltype(cfg);
        using S = Shape<C::D, C::N, C::P, C::DAB>;
        using SM = BackwardSmem<C::D, C::N, C::P, C::DAB, C::NTB, C::CHR>;
        constexpr int PARTS = S::TPU / C::NTB;
        const long long blocks = units * PARTS;
        if (blocks > 0x7fffffffLL) { rc = PSIG_ERR_TOO_LARGE; return; }
        const bool scratch = backward_needs_scratch<C>(desc);
        float *inc_grad = scratch ? static_cast<float *>(workspace) : nullptr;
        if (scratch) {
            const size_t bytes = sizeof(float) * (size_t)desc.B * (size_t)(desc.L - 1) * desc.d;
            if (cudaMemsetAsync(inc_grad, 0, bytes, stream) != cudaSuccess) { rc = PSIG_ERR_CUDA; return; }
        }
        auto kernel = sig_backward_tiled<C::D, C::N, C::P, C::DAB, C::NTB, C::CHR>;
        if (SM::kBytes > 48 * 1024) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SM::kBytes) !=
                cudaSuccess) { rc = PSIG_ERR_CUDA; return; }
        }
        if (blocks > 0) {
            const bool vec = aligned16(sig) && aligned16(grad);
            kernel<<<(unsigned)blocks, C::NTB, SM::kBytes, stream>>>(path, sig, grad, grad_path, inc_grad, desc.L, W,
                                                                      desc.W > 0 ? desc.windows : nullptr, vec ? 1 : 0);
            if (check_launch() != PSIG_OK) { rc = PSIG_ERR_CUDA; return; }
        }
        if (scratch) {
            const long long total = desc.B * desc.L * desc.d;
            long long nb = (total + 255) / 256;
            if (nb > 148 * 32) nb = 148 * 32;
            increments_to_points_f32<float><<<(unsigned)nb, 256, 0, stream>>>(inc_grad, grad_path, desc.B, desc.L,
                                                                               desc.d);
            rc = check_launch();
        } else {
            rc = PSIG_OK;
        }
    });
    return rc;
}

}  // namespace psig
