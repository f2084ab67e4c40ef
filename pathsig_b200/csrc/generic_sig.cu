// Generic signature kernels: any channel count d, any depth 1..12, dense or projected degrees,
// windows, float32 and float64.
//
// Work decomposition (differs from the reference, which gives every word its own thread and
// its own full prefix chain, src/pathsig/forward/sig_kernels.cu:95-157): one thread owns a
// prefix u of length K-1 together with a tile of TB last letters, i.e. the TB words u.b of
// degree K.  The Horner chain over the prefixes of u is evaluated once per step and shared by
// the whole tile; a projected degree degenerates to tiles of one word.  All degrees of all
// (path, window) units run in ONE launch: blockIdx.x selects degree and tile, blockIdx.y the
// unit.  Increments are staged in shared memory a chunk of steps at a time, so the step loop
// itself has no barrier and no global load.
//
// Backward is classical reverse mode on the thread-private chain: the prefix values are
// rolled back one step by subtracting exactly what the forward step added, and the adjoints
// of the prefixes are pushed through the transposed Horner chain, O(K^2) per step instead of
// the O(K^3) two-sided formula of the reference
// (src/pathsig/backward/sig_backward_kernels.cu:204-253).  Per-step increment gradients are
// summed in shared memory and flushed to a zeroed (B, L-1, d) scratch with atomics, then
// differenced into the path gradient (same data flow as
// src/pathsig/backward/sig_backward_kernels.cu:256-318 and 347-377).
#include "common.cuh"

#include <mutex>

namespace psig {
namespace {

constexpr int kBlock = 128;
constexpr size_t kStageBytes = 24 * 1024;
constexpr size_t kSlotBytes = 44 * 1024;
constexpr size_t kLaneBytes = 40 * 1024;   // staged increments (and gradients) of 32 units per block
constexpr long long kLaneMaxItems = 1024;  // above this the item-per-thread kernels fill their warps anyway

struct GenericPlan {
    LevelTable lt;
    long long items[kMaxDepth + 1];       // thread items per degree
    long long item_start[kMaxDepth + 2];  // first item of each degree in the packed order; [depth+1] = total
    int tiles;                            // letter tiles per dense prefix
    int chunk;                            // steps staged per refill
    int slot_stride;                      // backward: scalars per private gradient slot (0 = shared atomics)
    // "one lane per unit" kernels: items numbered without padding, 32 units per block
    long long lane_start[kMaxDepth + 2];  // first item of each degree; [depth+1] = total
    long long lane_items[kMaxDepth + 1];  // items per degree with tiles of lane_tb letters
    int lane_tb;                          // letters per dense tile in the lane kernels (1 or tile_letters)
    int lane_tiles;                       // letter tiles per dense prefix in the lane kernels
    int lane_chunk;                       // steps staged per refill (0 = lane kernels not used)
    int lane_stride;                      // scalars between two units' rows of staged increments (odd)
    long long B, L, W;                    // W >= 1
    const int *windows;
};

template <typename T>
__device__ __forceinline__ void kahan_add(T &sum, T add, T &comp)
{
    // Compensated summation in float32 (the explicit intrinsics keep the compiler from
    // re-associating).  In float64 the plain sum is already 5 orders of magnitude inside the 1e-11
    // parity bound over 10^4 steps, and the four extra dependent DADDs per term halve the throughput
    // of the FP64 pipe, so the compensation is left out there.
    if constexpr (sizeof(T) == 8) {
        (void)comp;
        sum = __dadd_rn(sum, add);
    } else {
        const float y = __fsub_rn(add, comp);
        const float t = __fadd_rn(sum, y);
        comp = __fsub_rn(__fsub_rn(t, sum), y);
        sum = t;
    }
}

// What one thread owns: degree K, the prefix u (|u| = K-1) and a tile of last letters.
// Items of all degrees are packed into one index space (each degree padded to a warp
// boundary), so a block may hold warps of several degrees; the per-step work is dispatched on K
// inside the step loop.
struct Item {
    int K;          // degree (1..depth); meaningless when nb == 0
    long long idx;  // index of the item within its degree
    long long u;    // code of the owned prefix
    int b0;         // first last-letter of the tile
    int nb;         // letters in the tile (0 = inactive thread)
};

template <int TB>
__device__ __forceinline__ Item decode_item(const GenericPlan &p, long long gi, const long long *first,
                                            const long long *items, int tiles)
{
    Item it{1, 0, 0, 0, 0};
    if (gi >= first[p.lt.depth + 1]) return it;
    int K = 1;
    while (K < p.lt.depth && gi >= first[K + 1]) ++K;
    it.K = K;
    it.idx = gi - first[K];
    if (it.idx >= items[K]) return it;  // padding between degrees
    const int d = p.lt.d;
    if (p.lt.words[K] == nullptr) {
        it.u = it.idx / tiles;
        it.b0 = (int)(it.idx % tiles) * TB;
        it.nb = min(TB, d - it.b0);
    } else {
        const long long code = p.lt.words[K][it.idx];
        it.u = code / d;
        it.b0 = (int)(code % d);
        it.nb = 1;
    }
    return it;
}

// Letters of the prefix, first letter in let[0]; entries at and beyond K-1 are zero.  MK bounds the
// degree a kernel instance handles and sizes its per-thread arrays.
template <int MK>
__device__ __forceinline__ void prefix_letters(const Item &it, int d, int (&let)[MK])
{
    long long c = it.u;
#pragma unroll
    for (int j = MK - 2; j >= 0; --j) {
        let[j] = 0;
        if (j < it.K - 1) { let[j] = (int)(c % d); c /= d; }
    }
    let[MK - 1] = 0;
}

__device__ __forceinline__ void unit_window(const GenericPlan &p, long long unit, long long &b, int &start, int &steps)
{
    b = unit / p.W;
    const long long w = unit % p.W;
    start = 0;
    int end = (int)p.L;
    if (p.windows) {
        // clamped to the path: a window reaching outside reads only the points that exist
        start = max(p.windows[2 * w], 0);
        end = min(p.windows[2 * w + 1], (int)p.L);
    }
    steps = max(end - start - 1, 0);
}

// Stage increments c0 .. c0+n-1 of one unit: s_dx[t*d + a] = x[c0+t+1][a] - x[c0+t][a].
template <typename T>
__device__ __forceinline__ void stage_increments(const T *__restrict__ x, int d, int c0, int n, T *s_dx)
{
    const T *lo = x + (long long)c0 * d;
    for (int i = threadIdx.x; i < n * d; i += kBlock) s_dx[i] = lo[i + d] - lo[i];
}

// ---- one forward step of an item of degree K (pref[j] = S(u[:j]), top[i] = S(u.b_i)) ----
// COMP: also compensate the sums of the private prefix copies (the owned words always are).
template <typename T, int K, int TB, int MK, bool COMP = true>
__device__ __forceinline__ void forward_step(const T *dx, const int (&let)[MK], const Item &it,
                                             T (&pref)[MK], T (&cpref)[MK], T (&top)[TB], T (&ctop)[TB])
{
    T xs[K > 1 ? K - 1 : 1];
#pragma unroll
    for (int j = 0; j < K - 1; ++j) xs[j] = dx[let[j]];
    // degree K: Horner chain over the prefixes of u, then one FMA per tile letter
    T bc = T(1);
#pragma unroll
    for (int j = 1; j <= K - 1; ++j) bc = fma(bc, xs[j - 1] * recip<T>(K - j + 1), pref[j]);
#pragma unroll
    for (int i = 0; i < TB; ++i)
        if (i < it.nb) kahan_add(top[i], bc * dx[it.b0 + i], ctop[i]);
    // private copies of the lower prefixes, highest first so each reads old values
#pragma unroll
    for (int m = K - 1; m >= 1; --m) {
        T bm = T(1);
#pragma unroll
        for (int j = 1; j <= m - 1; ++j) bm = fma(bm, xs[j - 1] * recip<T>(m - j + 1), pref[j]);
        if constexpr (COMP) kahan_add(pref[m], bm * xs[m - 1], cpref[m]);
        else pref[m] = fma(bm, xs[m - 1], pref[m]);
    }
}

// ---- forward step of the prefixes only (uncompensated), used to rebuild them for backward ----
template <typename T, int K, int MK>
__device__ __forceinline__ void prefix_step(const T *dx, const int (&let)[MK], T (&pref)[MK])
{
    T xs[K > 1 ? K - 1 : 1];
#pragma unroll
    for (int j = 0; j < K - 1; ++j) xs[j] = dx[let[j]];
#pragma unroll
    for (int m = K - 1; m >= 1; --m) {
        T bm = T(1);
#pragma unroll
        for (int j = 1; j <= m - 1; ++j) bm = fma(bm, xs[j - 1] * recip<T>(m - j + 1), pref[j]);
        pref[m] = fma(bm, xs[m - 1], pref[m]);
    }
}

// ---- one reverse step of an item of degree K ----
// Rolls pref back to the previous point, pushes the adjoints apref through the transposed
// chains and adds this thread's share of dL/d(dx_t) into sg (private slot, or the block's
// shared row with atomics).
template <typename T, int K, int TB, int MK>
__device__ __forceinline__ void backward_step(const T *dx, const int (&let)[MK], const Item &it,
                                              T (&pref)[MK], T (&apref)[MK], const T (&g)[TB], T *sg,
                                              bool slots)
{
    T xs[K > 1 ? K - 1 : 1], lg[K > 1 ? K - 1 : 1];
#pragma unroll
    for (int j = 0; j < K - 1; ++j) { xs[j] = dx[let[j]]; lg[j] = T(0); }

    // degrees 1..K-1 of the private chain: undo the step, then transpose it
#pragma unroll
    for (int m = 1; m <= K - 1; ++m) {
        T bc[K];  // bc[j] = Horner value after prefix length j (bc[0] = 1)
        bc[0] = T(1);
#pragma unroll
        for (int j = 1; j <= m - 1; ++j) bc[j] = fma(bc[j - 1], xs[j - 1] * recip<T>(m - j + 1), pref[j]);
        pref[m] = fma(-bc[m - 1], xs[m - 1], pref[m]);
        const T a = apref[m];
        lg[m - 1] = fma(a, bc[m - 1], lg[m - 1]);
        T adj = a * xs[m - 1];
#pragma unroll
        for (int j = m - 1; j >= 1; --j) {
            apref[j] += adj;
            const T c = recip<T>(m - j + 1);
            lg[j - 1] = fma(adj * c, bc[j - 1], lg[j - 1]);
            adj = adj * (xs[j - 1] * c);
        }
    }
    // degree K: the tile
    {
        T bc[K];
        bc[0] = T(1);
#pragma unroll
        for (int j = 1; j <= K - 1; ++j) bc[j] = fma(bc[j - 1], xs[j - 1] * recip<T>(K - j + 1), pref[j]);
        T adj = T(0);
#pragma unroll
        for (int i = 0; i < TB; ++i) {
            if (i < it.nb) {
                adj = fma(g[i], dx[it.b0 + i], adj);
                if (slots) sg[it.b0 + i] += g[i] * bc[K - 1];
                else atomicAdd(&sg[it.b0 + i], g[i] * bc[K - 1]);
            }
        }
#pragma unroll
        for (int j = K - 1; j >= 1; --j) {
            apref[j] += adj;
            const T c = recip<T>(K - j + 1);
            lg[j - 1] = fma(adj * c, bc[j - 1], lg[j - 1]);
            adj = adj * (xs[j - 1] * c);
        }
    }
#pragma unroll
    for (int j = 0; j < K - 1; ++j) {
        if (slots) sg[let[j]] += lg[j];
        else atomicAdd(&sg[let[j]], lg[j]);
    }
}

// Runs the statement with K = k as a compile-time constant; degrees above MK (the bound of the
// kernel instance) are not instantiated.
#define PSIG_DEGREE_CASE(n, MK, ...) \
    case n: { constexpr int K = n; if constexpr (K <= (MK)) { __VA_ARGS__; } } break;
#define PSIG_SWITCH_DEGREE(k, MK, ...)                                       \
    switch (k) {                                                             \
        PSIG_DEGREE_CASE(1, MK, __VA_ARGS__)                                 \
        PSIG_DEGREE_CASE(2, MK, __VA_ARGS__)                                 \
        PSIG_DEGREE_CASE(3, MK, __VA_ARGS__)                                 \
        PSIG_DEGREE_CASE(4, MK, __VA_ARGS__)                                 \
        PSIG_DEGREE_CASE(5, MK, __VA_ARGS__)                                 \
        PSIG_DEGREE_CASE(6, MK, __VA_ARGS__)                                 \
        PSIG_DEGREE_CASE(7, MK, __VA_ARGS__)                                 \
        PSIG_DEGREE_CASE(8, MK, __VA_ARGS__)                                 \
        PSIG_DEGREE_CASE(9, MK, __VA_ARGS__)                                 \
        PSIG_DEGREE_CASE(10, MK, __VA_ARGS__)                                \
        PSIG_DEGREE_CASE(11, MK, __VA_ARGS__)                                \
        PSIG_DEGREE_CASE(12, MK, __VA_ARGS__)                                \
        default: break;                                                      \
    }

template <typename T, int TB>
__global__ void __launch_bounds__(kBlock) sig_forward_generic(const GenericPlan p, const T *__restrict__ path,
                                                              T *__restrict__ out)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T *s_dx = reinterpret_cast<T *>(smem_raw);
    const int d = p.lt.d;
    const Item it = decode_item<TB>(p, (long long)blockIdx.x * kBlock + threadIdx.x, p.item_start, p.items, p.tiles);
    int let[kMaxDepth];
    prefix_letters<kMaxDepth>(it, d, let);
    const long long units = p.B * p.W;

    for (long long unit = blockIdx.y; unit < units; unit += gridDim.y) {
        long long b; int start, steps;
        unit_window(p, unit, b, start, steps);
        const T *x = path + (b * p.L + start) * d;

        T pref[kMaxDepth], cpref[kMaxDepth], top[TB], ctop[TB];
#pragma unroll
        for (int j = 0; j < kMaxDepth; ++j) { pref[j] = T(0); cpref[j] = T(0); }
#pragma unroll
        for (int i = 0; i < TB; ++i) { top[i] = T(0); ctop[i] = T(0); }

        for (int c0 = 0; c0 < steps; c0 += p.chunk) {
            const int n = min(p.chunk, steps - c0);
            __syncthreads();
            stage_increments(x, d, c0, n, s_dx);
            __syncthreads();
            if (it.nb == 0) continue;
            // dispatch on the degree once per chunk, so the step loop itself is branch-free
            PSIG_SWITCH_DEGREE(it.K, kMaxDepth, {
                for (int t = 0; t < n; ++t)
                    forward_step<T, K, TB, kMaxDepth>(s_dx + t * d, let, it, pref, cpref, top, ctop);
            });
        }
        if (it.nb == 0) continue;
        T *row = out + unit * p.lt.total + p.lt.offset[it.K];
        if (p.lt.words[it.K] == nullptr) {
#pragma unroll
            for (int i = 0; i < TB; ++i)
                if (i < it.nb) row[it.u * d + it.b0 + i] = top[i];
        } else {
            row[it.idx] = top[0];
        }
    }
}

template <typename T, int TB>
__global__ void __launch_bounds__(kBlock) sig_backward_generic(const GenericPlan p, const T *__restrict__ path,
                                                               const T *__restrict__ sig,
                                                               const T *__restrict__ grad,
                                                               T *__restrict__ inc_grad)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T *s_dx = reinterpret_cast<T *>(smem_raw);
    T *s_gd = s_dx + (size_t)p.chunk * p.lt.d;
    const int d = p.lt.d;
    const long long block_first = (long long)blockIdx.x * kBlock;
    const Item it = decode_item<TB>(p, block_first + threadIdx.x, p.item_start, p.items, p.tiles);
    int let[kMaxDepth];
    prefix_letters<kMaxDepth>(it, d, let);
    const bool slots = p.slot_stride > 0;
    const int nact = (int)max(0LL, min((long long)kBlock, p.item_start[p.lt.depth + 1] - block_first));
    // does any item of this block have to rebuild its prefix values with a forward sweep?
    const bool rebuild = it.nb > 0 && !p.lt.lower_dense[it.K];
    const bool any_rebuild = __syncthreads_or(rebuild ? 1 : 0) != 0;
    const long long units = p.B * p.W;

    for (long long unit = blockIdx.y; unit < units; unit += gridDim.y) {
        long long b; int start, steps;
        unit_window(p, unit, b, start, steps);
        if (steps == 0) continue;  // uniform over the block
        const T *x = path + (b * p.L + start) * d;
        T *gd = inc_grad + (b * (p.L - 1) + start) * d;

        T pref[kMaxDepth], apref[kMaxDepth], g[TB];
#pragma unroll
        for (int j = 0; j < kMaxDepth; ++j) { pref[j] = T(0); apref[j] = T(0); }
#pragma unroll
        for (int i = 0; i < TB; ++i) g[i] = T(0);

        if (it.nb > 0) {
            const T *grow = grad + unit * p.lt.total + p.lt.offset[it.K];
            if (p.lt.words[it.K] == nullptr) {
#pragma unroll
                for (int i = 0; i < TB; ++i)
                    if (i < it.nb) g[i] = grow[it.u * d + it.b0 + i];
            } else {
                g[0] = grow[it.idx];
            }
            // Prefix values at the end of the unit: read from the saved signature while all
            // lower degrees are stored dense ...
            if (!rebuild) {
                const T *srow = sig + unit * p.lt.total;
                long long c = it.u;
#pragma unroll
                for (int j = kMaxDepth - 1; j >= 1; --j)
                    if (j <= it.K - 1) { pref[j] = srow[p.lt.dense_offset[j] + c]; c /= d; }
            }
        }
        // ... otherwise recompute them with a forward sweep.
        if (any_rebuild) {
            for (int c0 = 0; c0 < steps; c0 += p.chunk) {
                const int n = min(p.chunk, steps - c0);
                __syncthreads();
                stage_increments(x, d, c0, n, s_dx);
                __syncthreads();
                if (!rebuild) continue;
                PSIG_SWITCH_DEGREE(it.K, kMaxDepth, {
                    for (int t = 0; t < n; ++t) prefix_step<T, K, kMaxDepth>(s_dx + t * d, let, pref);
                });
            }
        }

        // Reverse sweep, chunk by chunk from the end.
        const int nchunks = (steps + p.chunk - 1) / p.chunk;
        for (int ci = nchunks - 1; ci >= 0; --ci) {
            const int c0 = ci * p.chunk;
            const int n = min(p.chunk, steps - c0);
            __syncthreads();
            stage_increments(x, d, c0, n, s_dx);
            if (!slots)
                for (int i = threadIdx.x; i < n * d; i += kBlock) s_gd[i] = T(0);
            __syncthreads();
            // Where a step's increment gradients go: the block's shared row (atomics), or this
            // thread's private slot, zeroed first.  Padding threads between two degrees only zero
            // theirs (the column sums below run over them too).
            if (slots && (int)threadIdx.x < nact) {
                for (int t = 0; t < n; ++t) {
                    T *sg = s_gd + ((size_t)t * kBlock + threadIdx.x) * p.slot_stride;
                    for (int a = 0; a < d; ++a) sg[a] = T(0);
                }
            }
            if (it.nb > 0) {
                const size_t t_stride = slots ? (size_t)kBlock * p.slot_stride : (size_t)d;
                T *sg0 = slots ? s_gd + (size_t)threadIdx.x * p.slot_stride : s_gd;
                PSIG_SWITCH_DEGREE(it.K, kMaxDepth, {
                    for (int t = n - 1; t >= 0; --t)
                        backward_step<T, K, TB, kMaxDepth>(s_dx + t * d, let, it, pref, apref, g, sg0 + t * t_stride,
                                                           slots);
                });
            }
            __syncthreads();
            for (int i = threadIdx.x; i < n * d; i += kBlock) {
                T v;
                if (slots) {
                    // fixed-order sum over the active threads' slots
                    const int t = i / d, a = i - t * d;
                    const T *col = s_gd + (size_t)t * kBlock * p.slot_stride + a;
                    v = T(0);
                    for (int thr = 0; thr < nact; ++thr) v += col[(size_t)thr * p.slot_stride];
                } else {
                    v = s_gd[i];
                }
                if (v != T(0)) atomicAdd(&gd[(long long)c0 * d + i], v);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------
// "One lane per unit" kernels.  When a row has few items (a projection onto a few hundred words,
// or a small dense signature) but the batch has many units, the item-per-thread layout above
// leaves most lanes idle.  Here a warp takes ONE item and its 32 lanes take 32 different
// (path, window) units: every lane runs the same chain on its own unit's increments, so there is
// no divergence and no idle lane, and the warps of a block share one staging of the 32 units'
// increments.  Same step functions; the sums of the owned words are compensated, those of the
// private prefix copies are plain FMAs (as in the tiled kernels), which saves a fifth of the
// instructions of a deep word.
// ------------------------------------------------------------------------------------------
constexpr int kLaneWarps = 16;
constexpr int kLaneBlock = 32 * kLaneWarps;
constexpr int kLaneShallow = 6;  // depths up to this run an instance with per-thread arrays of this size

struct LaneUnit {  // per-unit facts, published once per unit group in shared memory
    long long b;
    int start, steps;
};

__device__ __forceinline__ void publish_units(const GenericPlan &p, long long group, LaneUnit *s_unit)
{
    if (threadIdx.x < 32) {
        const long long unit = group * 32 + threadIdx.x;
        LaneUnit lu{0, 0, 0};
        if (unit < p.B * p.W) unit_window(p, unit, lu.b, lu.start, lu.steps);
        s_unit[threadIdx.x] = lu;
    }
}

// s_dx[r * stride + t * d + a] = increment c0+t of unit r (r = 0..31), zero beyond its last step.
// Each warp takes whole units: coalesced reads along the unit's row, independent loads in flight.
template <typename T>
__device__ __forceinline__ void stage_unit_increments(const GenericPlan &p, const T *__restrict__ path,
                                                      const LaneUnit *s_unit, int c0, int n, T *s_dx)
{
    const int d = p.lt.d, row = n * d, lane = threadIdx.x & 31;
    for (int r = threadIdx.x >> 5; r < 32; r += (int)(blockDim.x >> 5)) {
        const LaneUnit lu = s_unit[r];
        const T *lo = path + (lu.b * p.L + lu.start + c0) * d;
        const int valid = max(0, min(n, lu.steps - c0)) * d;
        T *dst = s_dx + r * p.lane_stride;
        if constexpr (sizeof(T) == 4) {
            // 128-bit loads when rows are 16-byte aligned (d a multiple of 4, aligned base pointer)
            if ((d & 3) == 0 && (reinterpret_cast<uintptr_t>(lo) & 15u) == 0) {
#pragma unroll 2
                for (int j = 4 * lane; j < row; j += 128) {
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (j < valid) {
                        const float4 a = *reinterpret_cast<const float4 *>(lo + j);
                        const float4 c = *reinterpret_cast<const float4 *>(lo + j + d);
                        v = make_float4(c.x - a.x, c.y - a.y, c.z - a.z, c.w - a.w);
                    }
                    dst[j] = v.x; dst[j + 1] = v.y; dst[j + 2] = v.z; dst[j + 3] = v.w;
                }
                continue;
            }
        }
#pragma unroll 4
        for (int j = lane; j < row; j += 32) dst[j] = (j < valid) ? lo[j + d] - lo[j] : T(0);
    }
}

template <typename T, int TB, int MK>
__global__ void __launch_bounds__(kLaneBlock) sig_forward_lanes(const GenericPlan p, const T *__restrict__ path,
                                                                T *__restrict__ out)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T *s_dx = reinterpret_cast<T *>(smem_raw);
    __shared__ LaneUnit s_unit[32];
    const int d = p.lt.d, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const Item it = decode_item<TB>(p, (long long)blockIdx.x * (blockDim.x >> 5) + warp, p.lane_start, p.lane_items,
                                    p.lane_tiles);
    int let[MK];
    prefix_letters<MK>(it, d, let);
    const long long units = p.B * p.W, groups = (units + 31) / 32;

    for (long long group = blockIdx.y; group < groups; group += gridDim.y) {
        __syncthreads();
        publish_units(p, group, s_unit);
        __syncthreads();
        const int steps = s_unit[lane].steps;
        int max_steps = 0;
        for (int r = 0; r < 32; ++r) max_steps = max(max_steps, s_unit[r].steps);

        T pref[MK], cpref[MK], top[TB], ctop[TB];
#pragma unroll
        for (int j = 0; j < MK; ++j) { pref[j] = T(0); cpref[j] = T(0); }
#pragma unroll
        for (int i = 0; i < TB; ++i) { top[i] = T(0); ctop[i] = T(0); }

        for (int c0 = 0; c0 < max_steps; c0 += p.lane_chunk) {
            const int n = min(p.lane_chunk, max_steps - c0);
            __syncthreads();
            stage_unit_increments(p, path, s_unit, c0, n, s_dx);
            __syncthreads();
            if (it.nb == 0) continue;
            const T *mine = s_dx + lane * p.lane_stride;
            const int n_lane = min(n, steps - c0);  // steps of this lane's unit inside the chunk
            PSIG_SWITCH_DEGREE(it.K, MK, {
                for (int t = 0; t < n_lane; ++t)
                    forward_step<T, K, TB, MK, false>(mine + t * d, let, it, pref, cpref, top, ctop);
            });
        }
        const long long unit = group * 32 + lane;
        if (it.nb == 0 || unit >= units) continue;
        T *row = out + unit * p.lt.total + p.lt.offset[it.K];
        if (p.lt.words[it.K] == nullptr) {
#pragma unroll
            for (int i = 0; i < TB; ++i)
                if (i < it.nb) row[it.u * d + it.b0 + i] = top[i];
        } else {
            row[it.idx] = top[0];
        }
    }
}

template <typename T, int TB, int MK>
__global__ void __launch_bounds__(kLaneBlock) sig_backward_lanes(const GenericPlan p, const T *__restrict__ path,
                                                                 const T *__restrict__ sig,
                                                                 const T *__restrict__ grad,
                                                                 T *__restrict__ inc_grad)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T *s_dx = reinterpret_cast<T *>(smem_raw);
    T *s_gd = s_dx + 32 * (size_t)p.lane_stride;
    __shared__ LaneUnit s_unit[32];
    const int d = p.lt.d, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const Item it = decode_item<TB>(p, (long long)blockIdx.x * (blockDim.x >> 5) + warp, p.lane_start, p.lane_items,
                                    p.lane_tiles);
    int let[MK];
    prefix_letters<MK>(it, d, let);
    const bool rebuild = it.nb > 0 && !p.lt.lower_dense[it.K];
    const bool any_rebuild = __syncthreads_or(rebuild ? 1 : 0) != 0;
    const long long units = p.B * p.W, groups = (units + 31) / 32;

    for (long long group = blockIdx.y; group < groups; group += gridDim.y) {
        __syncthreads();
        publish_units(p, group, s_unit);
        __syncthreads();
        const long long unit = group * 32 + lane;
        const bool live = it.nb > 0 && unit < units;
        const int steps = s_unit[lane].steps;
        int max_steps = 0;
        for (int r = 0; r < 32; ++r) max_steps = max(max_steps, s_unit[r].steps);
        if (max_steps == 0) continue;  // uniform over the block

        T pref[MK], apref[MK], g[TB];
#pragma unroll
        for (int j = 0; j < MK; ++j) { pref[j] = T(0); apref[j] = T(0); }
#pragma unroll
        for (int i = 0; i < TB; ++i) g[i] = T(0);
        if (live) {
            const T *grow = grad + unit * p.lt.total + p.lt.offset[it.K];
            if (p.lt.words[it.K] == nullptr) {
#pragma unroll
                for (int i = 0; i < TB; ++i)
                    if (i < it.nb) g[i] = grow[it.u * d + it.b0 + i];
            } else {
                g[0] = grow[it.idx];
            }
            if (!rebuild) {
                const T *srow = sig + unit * p.lt.total;
                long long c = it.u;
#pragma unroll
                for (int j = MK - 1; j >= 1; --j)
                    if (j <= it.K - 1) { pref[j] = srow[p.lt.dense_offset[j] + c]; c /= d; }
            }
        }
        if (any_rebuild) {
            for (int c0 = 0; c0 < max_steps; c0 += p.lane_chunk) {
                const int n = min(p.lane_chunk, max_steps - c0);
                __syncthreads();
                stage_unit_increments(p, path, s_unit, c0, n, s_dx);
                __syncthreads();
                if (!rebuild || !live) continue;
                const T *mine = s_dx + lane * p.lane_stride;
                const int n_lane = min(n, steps - c0);
                PSIG_SWITCH_DEGREE(it.K, MK, {
                    for (int t = 0; t < n_lane; ++t) prefix_step<T, K, MK>(mine + t * d, let, pref);
                });
            }
        }

        const int nchunks = (max_steps + p.lane_chunk - 1) / p.lane_chunk;
        for (int ci = nchunks - 1; ci >= 0; --ci) {
            const int c0 = ci * p.lane_chunk;
            const int n = min(p.lane_chunk, max_steps - c0);
            __syncthreads();
            stage_unit_increments(p, path, s_unit, c0, n, s_dx);
            for (int i = threadIdx.x; i < 32 * p.lane_stride; i += blockDim.x) s_gd[i] = T(0);
            __syncthreads();
            if (live) {
                const T *mine = s_dx + lane * p.lane_stride;
                T *mine_gd = s_gd + lane * p.lane_stride;
                const int n_lane = min(n, steps - c0);
                PSIG_SWITCH_DEGREE(it.K, MK, {
                    for (int t = n_lane - 1; t >= 0; --t)
                        backward_step<T, K, TB, MK>(mine + t * d, let, it, pref, apref, g, mine_gd + t * d, false);
                });
            }
            __syncthreads();
            // flush the 32 units' rows of this chunk, one unit per warp at a time
            const int row = n * d;
            for (int r = warp; r < 32; r += (int)(blockDim.x >> 5)) {
                const LaneUnit lu = s_unit[r];
                T *dst = inc_grad + (lu.b * (p.L - 1) + lu.start + c0) * d;
                const T *src = s_gd + r * p.lane_stride;
                const int valid = max(0, min(n, lu.steps - c0)) * d;
                for (int j = lane; j < valid; j += 32) {
                    const T v = src[j];
                    if (v != T(0)) atomicAdd(&dst[j], v);
                }
            }
            (void)row;
        }
    }
}

// grad wrt increments -> grad wrt points (64-bit indexing).
template <typename T>
__global__ void increments_to_points(const T *__restrict__ inc_grad, T *__restrict__ path_grad, long long B,
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

// Warps per block of the lane kernels (16, 8 or 4): the choice that leaves the busiest SM the fewest
// warps when the blocks are dealt round-robin over the SMs; larger blocks win ties because a block
// stages the increments of its 32 units once for all its warps.
int lane_warps_for(long long items, long long groups)
{
    int kSmCount = 148, device = 0, queried = 0;
    if (cudaGetDevice(&device) == cudaSuccess &&
        cudaDeviceGetAttribute(&queried, cudaDevAttrMultiProcessorCount, device) == cudaSuccess && queried > 0)
        kSmCount = queried;
    int best = kLaneWarps;
    long long best_cost = -1;
    for (int lw = kLaneWarps; lw >= 4; lw /= 2) {
        const long long blocks = (items + lw - 1) / lw * groups;
        const long long cost = (blocks + kSmCount - 1) / kSmCount * lw;
        if (best_cost < 0 || cost < best_cost) { best = lw; best_cost = cost; }
    }
    return best;
}

template <typename T> constexpr int tile_letters() { return sizeof(T) == 4 ? 8 : 4; }

template <typename T>
int make_plan(const PsigSigDesc &desc, const LevelTable &lt, int buffers, GenericPlan *plan)
{
    constexpr int TB = tile_letters<T>();
    GenericPlan &p = *plan;
    p.lt = lt;
    p.B = desc.B;
    p.L = desc.L;
    p.W = desc.W > 0 ? desc.W : 1;
    p.windows = desc.W > 0 ? desc.windows : nullptr;
    p.tiles = (lt.d + TB - 1) / TB;
    long long total_items = 0;
    long long d_pow = 1;  // d^(k-1)
    for (int k = 1; k <= lt.depth; ++k) {
        p.items[k] = lt.words[k] ? lt.size[k] : (lt.size[k] == 0 ? 0 : d_pow * p.tiles);
        // every degree starts on a warp boundary: a warp never mixes degrees (no divergence in
        // the per-step dispatch), a block may hold warps of different degrees
        total_items = (total_items + 31) / 32 * 32;
        p.item_start[k] = total_items;
        total_items += p.items[k];
        if (k < lt.depth) d_pow *= lt.d;
    }
    for (int k = lt.depth + 1; k <= kMaxDepth + 1; ++k) p.item_start[k] = total_items;
    if ((total_items + kBlock - 1) / kBlock > 0x7fffffffLL) return PSIG_ERR_TOO_LARGE;
    const size_t per_step = sizeof(T) * (size_t)lt.d * buffers;
    if (per_step > 48 * 1024) return PSIG_ERR_TOO_LARGE;
    long long chunk = (long long)(kStageBytes / per_step);
    if (chunk < 1) chunk = 1;
    if (chunk > 64) chunk = 64;
    p.chunk = (int)chunk;
    // lane kernels: worth it when rows have few items and there are at least a warp's worth of units
    p.lane_chunk = 0;
    p.lane_stride = 0;
    // A warp of the lane kernels runs ONE item, so a tile wider than the item's word count is issued
    // in full and predicated off: rows with a projected degree use single-word items throughout.
    bool any_projected = false;
    for (int k = 1; k <= lt.depth; ++k) any_projected = any_projected || lt.words[k] != nullptr;
    p.lane_tb = any_projected ? 1 : TB;
    p.lane_tiles = (lt.d + p.lane_tb - 1) / p.lane_tb;
    long long lane_items = 0;
    d_pow = 1;
    p.lane_items[0] = 0;
    for (int k = 1; k <= kMaxDepth; ++k) p.lane_items[k] = 0;
    for (int k = 1; k <= lt.depth; ++k) {
        p.lane_items[k] = lt.words[k] ? lt.size[k] : (lt.size[k] == 0 ? 0 : d_pow * p.lane_tiles);
        p.lane_start[k] = lane_items;
        lane_items += p.lane_items[k];
        if (k < lt.depth) d_pow *= lt.d;
    }
    for (int k = lt.depth + 1; k <= kMaxDepth + 1; ++k) p.lane_start[k] = lane_items;
    {
        const long long units = p.B * p.W;
        const long long lane_steps = (long long)(kLaneBytes / (sizeof(T) * 32 * (size_t)lt.d * buffers));
        if (units >= 32 && lane_items <= kLaneMaxItems && lane_steps >= 2) {
            p.lane_chunk = (int)(lane_steps > 32 ? 32 : lane_steps);
            p.lane_stride = (p.lane_chunk * lt.d) | 1;
        }
    }
    p.slot_stride = 0;
    if (buffers == 2) {
        // Backward with few channels: float atomics on a handful of shared addresses serialise, so
        // every thread gets a private slot of d scalars per step instead (odd stride: no bank
        // conflicts in the column sums).  Needs at least two steps per chunk to be worth it.
        const int stride = lt.d | 1;
        const size_t slot_step = sizeof(T) * ((size_t)lt.d + (size_t)kBlock * stride);
        const long long slot_chunk = (long long)(kSlotBytes / slot_step);
        if (slot_chunk >= 2) {
            p.slot_stride = stride;
            p.chunk = (int)(slot_chunk > 32 ? 32 : slot_chunk);
        }
    }
    return PSIG_OK;
}

}  // namespace

template <typename T>
int generic_sig_forward(const PsigSigDesc &desc, const LevelTable &lt, const T *path, T *out, cudaStream_t stream)
{
    constexpr int TB = tile_letters<T>();
    GenericPlan plan;
    const int rc = make_plan<T>(desc, lt, 1, &plan);
    if (rc != PSIG_OK) return rc;
    const long long units = plan.B * plan.W;
    const long long blocks = (plan.item_start[kMaxDepth + 1] + kBlock - 1) / kBlock;
    if (units == 0 || blocks == 0) return PSIG_OK;
    if (plan.lane_chunk > 0) {
        const long long groups = (units + 31) / 32;
        const int lw = lane_warps_for(plan.lane_start[kMaxDepth + 1], groups);
        const long long lane_blocks = (plan.lane_start[kMaxDepth + 1] + lw - 1) / lw;
        const dim3 grid((unsigned)lane_blocks, (unsigned)(groups < 65535 ? groups : 65535));
        const unsigned block = 32u * lw;
        const size_t smem = sizeof(T) * 32 * (size_t)plan.lane_stride;
        const bool single = plan.lane_tb == 1, shallow = lt.depth <= kLaneShallow;
        auto launch = [&](auto kernel) {
            // the staged increments make shared memory the occupancy limit under the default L1 split
            prepare_kernel(kernel, smem, true);
            kernel<<<grid, block, smem, stream>>>(plan, path, out);
        };
        if (single && shallow) launch(sig_forward_lanes<T, 1, kLaneShallow>);
        else if (single) launch(sig_forward_lanes<T, 1, kMaxDepth>);
        else if (shallow) launch(sig_forward_lanes<T, TB, kLaneShallow>);
        else launch(sig_forward_lanes<T, TB, kMaxDepth>);
        return check_launch();
    }
    const dim3 grid((unsigned)blocks, (unsigned)(units < 65535 ? units : 65535));
    const size_t smem = sizeof(T) * (size_t)plan.chunk * lt.d;
    sig_forward_generic<T, TB><<<grid, kBlock, smem, stream>>>(plan, path, out);
    return check_launch();
}

template <typename T>
int generic_sig_backward(const PsigSigDesc &desc, const LevelTable &lt, const T *path, const T *sig, const T *grad,
                         T *grad_path, T *inc_grad_ws, cudaStream_t stream)
{
    constexpr int TB = tile_letters<T>();
    GenericPlan plan;
    const int rc = make_plan<T>(desc, lt, 2, &plan);
    if (rc != PSIG_OK) return rc;
    const long long units = plan.B * plan.W;
    const long long blocks = (plan.item_start[kMaxDepth + 1] + kBlock - 1) / kBlock;
    if (desc.B == 0) return PSIG_OK;
    const size_t inc_bytes = sizeof(T) * (size_t)desc.B * (size_t)(desc.L - 1) * lt.d;
    if (cudaMemsetAsync(inc_grad_ws, 0, inc_bytes, stream) != cudaSuccess) return PSIG_ERR_CUDA;
    if (units > 0 && blocks > 0 && plan.lane_chunk > 0) {
        const long long groups = (units + 31) / 32;
        const int lw = lane_warps_for(plan.lane_start[kMaxDepth + 1], groups);
        const long long lane_blocks = (plan.lane_start[kMaxDepth + 1] + lw - 1) / lw;
        const dim3 grid((unsigned)lane_blocks, (unsigned)(groups < 65535 ? groups : 65535));
        const unsigned block = 32u * lw;
        const size_t smem = 2 * sizeof(T) * 32 * (size_t)plan.lane_stride;
        const bool single = plan.lane_tb == 1, shallow = lt.depth <= kLaneShallow;
        auto launch = [&](auto kernel) {
            if (!prepare_kernel(kernel, smem, true)) return;  // the launch below then fails and reports the error
            kernel<<<grid, block, smem, stream>>>(plan, path, sig, grad, inc_grad_ws);
        };
        if (single && shallow) launch(sig_backward_lanes<T, 1, kLaneShallow>);
        else if (single) launch(sig_backward_lanes<T, 1, kMaxDepth>);
        else if (shallow) launch(sig_backward_lanes<T, TB, kLaneShallow>);
        else launch(sig_backward_lanes<T, TB, kMaxDepth>);
        if (check_launch() != PSIG_OK) return PSIG_ERR_CUDA;
    } else if (units > 0 && blocks > 0) {
        const dim3 grid((unsigned)blocks, (unsigned)(units < 65535 ? units : 65535));
        const size_t smem = plan.slot_stride > 0
                                ? sizeof(T) * (size_t)plan.chunk * ((size_t)lt.d + (size_t)kBlock * plan.slot_stride)
                                : 2 * sizeof(T) * (size_t)plan.chunk * lt.d;
        sig_backward_generic<T, TB><<<grid, kBlock, smem, stream>>>(plan, path, sig, grad, inc_grad_ws);
        if (check_launch() != PSIG_OK) return PSIG_ERR_CUDA;
    }
    const long long total = desc.B * desc.L * lt.d;
    long long nb = (total + 255) / 256;
    if (nb > 148 * 32) nb = 148 * 32;
    increments_to_points<T><<<(unsigned)nb, 256, 0, stream>>>(inc_grad_ws, grad_path, desc.B, desc.L, lt.d);
    return check_launch();
}

template int generic_sig_forward<float>(const PsigSigDesc &, const LevelTable &, const float *, float *, cudaStream_t);
template int generic_sig_forward<double>(const PsigSigDesc &, const LevelTable &, const double *, double *,
                                         cudaStream_t);
template int generic_sig_backward<float>(const PsigSigDesc &, const LevelTable &, const float *, const float *,
                                         const float *, float *, float *, cudaStream_t);
template int generic_sig_backward<double>(const PsigSigDesc &, const LevelTable &, const double *, const double *,
                                          const double *, double *, double *, cudaStream_t);

}  // namespace psig

// ----------------------------------------------------------------------------------------------
// psig_sig_backward_static: signature backward for callers that cannot hand us scratch memory
// ----------------------------------------------------------------------------------------------
// The generic backward kernel needs a zeroed accumulator of B*(L-1)*d scalars for the gradient
// with respect to the increments.  psig_sig_backward takes it from the caller; some callers have
// nothing to give: code that runs where a device allocation is off limits (a pre-sized inference
// arena owns all of the card's memory, an enqueue-style plugin hook that must not allocate, a
// latency-critical loop that cannot afford the device-wide synchronisation cudaMalloc/cudaFree
// imply).  For them the accumulator lives in this fixed array inside the library image.  Every
// device that loads the library carries these bytes until the process exits, which is why the
// limit is kept small.
#define PSIG_STATIC_SCRATCH_BYTES (8u << 20)
static __device__ __align__(256) unsigned char g_static_scratch[PSIG_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_scratch_mutex;
void *g_scratch_address[kMaxDevices] = {nullptr};

// Device address of g_static_scratch on the CURRENT device.  The array's name is only a host-side
// handle; the address a kernel can use has to be asked for, once per device, while that device
// is current.
int static_scratch_address(void **out)
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return PSIG_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_address[dev] == nullptr) {
        void *ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) return PSIG_ERR_CUDA;
        g_scratch_address[dev] = ptr;
    }
    *out = g_scratch_address[dev];
    return PSIG_OK;
}
}  // namespace

extern "C" int64_t psig_sig_backward_static_limit(void) { return (int64_t)PSIG_STATIC_SCRATCH_BYTES; }

extern "C" int psig_sig_backward_static(const PsigSigDesc *desc, const void *path, const void *sig,
                                        const void *grad_sig, void *grad_path, void *stream)
{
    using namespace psig;
    if (!desc) return PSIG_ERR_NULL;
    if (desc->dtype != PSIG_F32 && desc->dtype != PSIG_F64) return PSIG_ERR_DTYPE;
    if (desc->depth < 1 || desc->depth > kMaxDepth) return PSIG_ERR_DEPTH;
    if (desc->B < 0 || desc->L < 2 || desc->d < 1 || desc->W < 0) return PSIG_ERR_SHAPE;
    if (desc->W > 0 && !desc->windows) return PSIG_ERR_NULL;
    LevelTable lt;
    int rc = make_level_table(desc->d, desc->depth, desc->projected != 0, desc->level_sizes, desc->words, false, &lt);
    if (rc != PSIG_OK) return rc;
    if (desc->B == 0) return PSIG_OK;
    if (!path || !grad_path || (lt.total > 0 && (!sig || !grad_sig))) return PSIG_ERR_NULL;
    const size_t scalar = desc->dtype == PSIG_F32 ? 4 : 8;
    // B*(L-1)*d scalars must fit the fixed array; anything larger has to go through
    // psig_sig_backward with caller-provided scratch.
    const double need = (double)scalar * (double)desc->B * (double)(desc->L - 1) * (double)desc->d;
    if (need > (double)PSIG_STATIC_SCRATCH_BYTES) return PSIG_ERR_TOO_LARGE;
    void *scratch = nullptr;
    rc = static_scratch_address(&scratch);
    if (rc != PSIG_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // generic_sig_backward clears the part of the scratch it accumulates into before the kernel
    // runs, so contents left by an earlier call do not matter.
    if (desc->dtype == PSIG_F32)
        return generic_sig_backward<float>(*desc, lt, static_cast<const float *>(path),
                                           static_cast<const float *>(sig), static_cast<const float *>(grad_sig),
                                           static_cast<float *>(grad_path), static_cast<float *>(scratch), st);
    return generic_sig_backward<double>(*desc, lt, static_cast<const double *>(path),
                                        static_cast<const double *>(sig), static_cast<const double *>(grad_sig),
                                        static_cast<double *>(grad_path), static_cast<double *>(scratch), st);
}
