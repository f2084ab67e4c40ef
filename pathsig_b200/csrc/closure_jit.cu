// Prefix-closure signature kernels, specialised per word set at plan time.
//
// A projected signature asks for a set of words; the state Chen's recurrence needs is the prefix
// closure C of that set (every requested word and every prefix of one).  The reference gives each
// requested word a thread that recomputes the word's whole prefix chain privately
// (src/pathsig/forward/sig_kernels.cu:99-113, 138-152).  Here the closure is a trie, and one step is,
// per target degree m, a sweep over the trie nodes that have a descendant of degree m:
//     B_j[u] = B_{j-1}[parent(u)] * dx[letter(u)] / (m-j+1) + S[u]      (|u| = j < m)
//     S[w]  += B_{m-1}[parent(w)] * dx[letter(w)]                        (|w| = m)
// i.e. one FMA per (node, target degree) pair: the algorithmic minimum of the shared-prefix scheme.
//
// To keep every node value in a register the sweep has to be straight-line code, so the kernels are
// generated for the word set: the trie is laid out in depth-first order and cut into bins of about
// equal arithmetic; a bin holds its own nodes plus the (at most depth-1) ancestors of its first node,
// whose values it recomputes redundantly.  A warp runs ONE bin and its 32 lanes run 32 different
// (path, window) units, so the code of a bin is warp-uniform (no divergence) and needs no
// communication in forward.  In backward (reverse mode through the same sweep, degrees bottom-up:
// roll the values back one step, then push the adjoints through the transposed chains) each lane owns
// a unit, so the per-step gradient with respect to the increment is summed in registers over the
// bin's nodes; bins of the same units meet in shared memory and in a zeroed (B, L-1, d) accumulator.
//
// The generated CUDA C++ is compiled for the device at hand with NVRTC (loaded lazily; without it this
// family reports "unsupported" and the generic kernels serve the request) and launched through the
// driver entry points obtained from the runtime.  Plans are cached per (device, dtype, word set).
#include "common.cuh"

#include <dlfcn.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

namespace psig {
namespace {

constexpr long long kMaxClosureNodes = 16384;  // closure size beyond which the plan is refused

constexpr size_t kStageBytes = 192 * 1024;     // staged increments (and, in backward, their gradients) per block
constexpr size_t kOneBlockPerSmBytes = 116 * 1024;  // dynamic shared memory that leaves no room for a second block

// ------------------------------------------------------------------------------------------
// NVRTC and driver entry points, resolved at first use
// ------------------------------------------------------------------------------------------
typedef struct _nvrtcProgram *nvrtcProgram;
struct Nvrtc {
    int (*CreateProgram)(nvrtcProgram *, const char *, const char *, int, const char *const *, const char *const *);
    int (*DestroyProgram)(nvrtcProgram *);
    int (*CompileProgram)(nvrtcProgram, int, const char *const *);
    int (*GetCUBINSize)(nvrtcProgram, size_t *);
    int (*GetCUBIN)(nvrtcProgram, char *);
    int (*GetProgramLogSize)(nvrtcProgram, size_t *);
    int (*GetProgramLog)(nvrtcProgram, char *);
    bool ok = false;
};

typedef struct CUmod_st *CUmodule;
typedef struct CUfunc_st *CUfunction;
struct Driver {
    int (*ModuleLoadData)(CUmodule *, const void *);
    int (*ModuleGetFunction)(CUfunction *, CUmodule, const char *);
    int (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, void *, void **,
                        void **);
    int (*FuncSetAttribute)(CUfunction, int, int);
    bool ok = false;
};

std::once_flag g_nvrtc_once, g_driver_once;
Nvrtc g_nvrtc;
Driver g_driver;

const Nvrtc &nvrtc()
{
    std::call_once(g_nvrtc_once, [] {
        const char *names[] = {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12",
                               "/usr/local/cuda/lib64/libnvrtc.so"};
        void *h = nullptr;
        for (const char *n : names)
            if ((h = dlopen(n, RTLD_NOW | RTLD_LOCAL)) != nullptr) break;
        if (!h) return;
        bool all = true;
        auto get = [&](const char *sym) { void *p = dlsym(h, sym); all = all && p != nullptr; return p; };
        *(void **)&g_nvrtc.CreateProgram = get("nvrtcCreateProgram");
        *(void **)&g_nvrtc.DestroyProgram = get("nvrtcDestroyProgram");
        *(void **)&g_nvrtc.CompileProgram = get("nvrtcCompileProgram");
        *(void **)&g_nvrtc.GetCUBINSize = get("nvrtcGetCUBINSize");
        *(void **)&g_nvrtc.GetCUBIN = get("nvrtcGetCUBIN");
        *(void **)&g_nvrtc.GetProgramLogSize = get("nvrtcGetProgramLogSize");
        *(void **)&g_nvrtc.GetProgramLog = get("nvrtcGetProgramLog");
        g_nvrtc.ok = all;
    });
    return g_nvrtc;
}

const Driver &driver()
{
    std::call_once(g_driver_once, [] {
        bool all = true;
        auto get = [&](const char *sym) {
            void *p = nullptr;
            cudaDriverEntryPointQueryResult st;
            if (cudaGetDriverEntryPoint(sym, &p, cudaEnableDefault, &st) != cudaSuccess || st != cudaDriverEntryPointSuccess)
                p = nullptr;
            all = all && p != nullptr;
            return p;
        };
        *(void **)&g_driver.ModuleLoadData = get("cuModuleLoadData");
        *(void **)&g_driver.ModuleGetFunction = get("cuModuleGetFunction");
        *(void **)&g_driver.LaunchKernel = get("cuLaunchKernel");
        *(void **)&g_driver.FuncSetAttribute = get("cuFuncSetAttribute");
        g_driver.ok = all;
        (void)cudaGetLastError();
    });
    return g_driver;
}

// ------------------------------------------------------------------------------------------
// the trie of the closure and its bins
// ------------------------------------------------------------------------------------------
struct Node {
    int parent = -1;   // -1: child of the root (the empty word)
    int letter = 0;
    int depth = 0;     // 1..N
    long long col = -1;  // column in the output row, -1 for a closure-only prefix
    std::vector<int> children;
    unsigned below = 0;  // bit m set: the node or a descendant has depth m
};

struct Bin {
    std::vector<int> nodes;   // global node ids in depth-first order: ancestors of the first own node, then own nodes
    std::vector<int> parent;  // local index of the parent, -1 for children of the root
    std::vector<char> own;
    std::vector<unsigned> below;  // like Node::below, restricted to the bin
    bool rebuild = false;  // backward: some value the sweep needs is not in the saved signature
    int max_depth = 0;
};

struct Trie {
    int d = 0, depth = 0;
    long long width = 0;
    std::vector<Node> nodes;
    std::vector<int> roots;  // nodes of depth 1
    std::vector<int> order;  // depth-first preorder
};

void decode(long long code, int n, int d, int *letters)
{
    for (int i = n - 1; i >= 0; --i) { letters[i] = (int)(code % d); code /= d; }
}

// Builds the closure of the row layout `lt` (host word codes in `words_host`, laid out like the device
// array: non-complete degrees concatenated).  Returns false when it would exceed the node budget.
bool build_trie(const LevelTable &lt, const int64_t *words_host, Trie *out)
{
    Trie &t = *out;
    t.d = lt.d;
    t.depth = lt.depth;
    t.width = lt.total;
    // child lookup: (parent id + 1) * d + letter -> node id
    std::map<long long, int> child_of;
    auto descend = [&](int parent, int letter) -> int {
        const long long key = (long long)(parent + 1) * t.d + letter;
        auto it = child_of.find(key);
        if (it != child_of.end()) return it->second;
        Node n;
        n.parent = parent;
        n.letter = letter;
        n.depth = parent < 0 ? 1 : t.nodes[parent].depth + 1;
        const int id = (int)t.nodes.size();
        t.nodes.push_back(n);
        child_of[key] = id;
        if (parent >= 0) t.nodes[parent].children.push_back(id); else t.roots.push_back(id);
        return id;
    };
    long long used = 0, d_pow = 1;
    int letters[kMaxDepth];
    for (int k = 1; k <= lt.depth; ++k) {
        d_pow *= lt.d;
        const bool listed = lt.size[k] != d_pow;
        if ((long long)t.nodes.size() + lt.size[k] * k > 4 * kMaxClosureNodes) return false;
        for (long long i = 0; i < lt.size[k]; ++i) {
            long long code = i;
            if (listed) {
                if (!words_host) return false;
                code = words_host[used + i];
                if (code < 0 || code >= d_pow) return false;
            }
            decode(code, k, lt.d, letters);
            int node = -1;
            for (int j = 0; j < k; ++j) node = descend(node, letters[j]);
            // a word listed twice keeps its first column for the forward store; the duplicate column is
            // served by a copy node below (rare: handled by refusing the plan)
            if (t.nodes[node].col >= 0) return false;
            t.nodes[node].col = lt.offset[k] + i;
            if ((long long)t.nodes.size() > kMaxClosureNodes) return false;
        }
        if (listed) used += lt.size[k];
    }
    // children in letter order, then a depth-first preorder
    for (Node &n : t.nodes)
        std::sort(n.children.begin(), n.children.end(), [&](int a, int b) { return t.nodes[a].letter < t.nodes[b].letter; });
    std::sort(t.roots.begin(), t.roots.end(), [&](int a, int b) { return t.nodes[a].letter < t.nodes[b].letter; });
    std::vector<int> stack(t.roots.rbegin(), t.roots.rend());
    while (!stack.empty()) {
        const int u = stack.back();
        stack.pop_back();
        t.order.push_back(u);
        for (auto it = t.nodes[u].children.rbegin(); it != t.nodes[u].children.rend(); ++it) stack.push_back(*it);
    }
    for (auto it = t.order.rbegin(); it != t.order.rend(); ++it) {
        Node &n = t.nodes[*it];
        n.below |= 1u << n.depth;
        if (n.parent >= 0) t.nodes[n.parent].below |= n.below;
    }
    return !t.nodes.empty();
}

int popcount(unsigned v) { int c = 0; while (v) { c += v & 1u; v >>= 1; } return c; }

// Forward FMAs per step of the whole closure (one per node and target degree at or below it).
long long closure_fma(const Trie &t)
{
    long long total = 0;
    for (const Node &n : t.nodes) total += popcount(n.below);
    return total;
}

std::vector<Bin> make_bins(const Trie &t, int target_bins)
{
    const long long total = closure_fma(t);
    long long per_bin = (total + target_bins - 1) / target_bins;
    if (per_bin < 24) per_bin = 24;  // below this the per-step fixed cost of a warp dominates
    std::vector<Bin> bins;
    size_t i = 0;
    while (i < t.order.size()) {
        Bin b;
        // ancestors of the first own node, root first
        std::vector<int> anc;
        for (int a = t.nodes[t.order[i]].parent; a >= 0; a = t.nodes[a].parent) anc.push_back(a);
        std::reverse(anc.begin(), anc.end());
        for (int a : anc) { b.nodes.push_back(a); b.own.push_back(0); }
        long long cost = 0;
        while (i < t.order.size() && (cost < per_bin || b.nodes.size() == anc.size())) {
            const int u = t.order[i++];
            b.nodes.push_back(u);
            b.own.push_back(1);
            cost += popcount(t.nodes[u].below);
            if (b.nodes.size() >= 64) break;  // register budget of a lane (backward keeps two values per node)
        }
        std::map<int, int> local;
        for (size_t k = 0; k < b.nodes.size(); ++k) local[b.nodes[k]] = (int)k;
        b.parent.resize(b.nodes.size());
        b.below.assign(b.nodes.size(), 0u);
        for (size_t k = 0; k < b.nodes.size(); ++k) {
            const int p = t.nodes[b.nodes[k]].parent;
            b.parent[k] = p < 0 ? -1 : local.at(p);
        }
        for (size_t k = b.nodes.size(); k-- > 0;) {
            const Node &n = t.nodes[b.nodes[k]];
            b.below[k] |= 1u << n.depth;
            if (b.parent[k] >= 0) b.below[b.parent[k]] |= b.below[k];
            b.max_depth = std::max(b.max_depth, n.depth);
        }
        // values the reverse sweep reads: nodes with something below them inside the bin
        for (size_t k = 0; k < b.nodes.size(); ++k) {
            const Node &n = t.nodes[b.nodes[k]];
            const bool needed = (b.below[k] >> (n.depth + 1)) != 0;
            if (needed && n.col < 0) b.rebuild = true;
        }
        bins.push_back(std::move(b));
    }
    return bins;
}

// ------------------------------------------------------------------------------------------
// code generation
// ------------------------------------------------------------------------------------------
struct Emitter {
    std::string s;
    void line(const std::string &t) { s += t; s += '\n'; }
};

std::string str(long long v) { return std::to_string(v); }

// x{a}_{c} = dx[a] / c; c == 1 is the raw increment x{a}
struct ScaleSet {
    std::vector<char> used;  // [a * (kMaxDepth + 1) + c]
    int d;
    explicit ScaleSet(int d_) : used((size_t)d_ * (kMaxDepth + 1), 0), d(d_) {}
    std::string name(int a, int c)
    {
        used[(size_t)a * (kMaxDepth + 1) + c] = 1;
        used[(size_t)a * (kMaxDepth + 1) + 1] = 1;
        return c == 1 ? "x" + str(a) : "x" + str(a) + "_" + str(c);
    }
    void declare(Emitter &e) const
    {
        for (int a = 0; a < d; ++a) {
            if (!used[(size_t)a * (kMaxDepth + 1) + 1]) continue;
            e.line("    const real x" + str(a) + " = dx[" + str(a) + "];");
            for (int c = 2; c <= kMaxDepth; ++c)
                if (used[(size_t)a * (kMaxDepth + 1) + c])
                    e.line("    const real x" + str(a) + "_" + str(c) + " = x" + str(a) + " * (real)(1.0 / " + str(c) + ".0);");
        }
    }
};

// Emits the per-step code of one bin.  Siblings (children of one trie node) go through the sweep in
// pairs: their updates have the same shape with different letters, so each pair is one packed two-lane
// FMA (fma.rn.f32x2 in float32), which halves the issue slots wherever the trie branches.
struct BinGen {
    const Trie &t;
    const Bin &b;
    std::vector<std::vector<int>> kids;  // local children
    std::vector<int> top;                // local nodes of depth 1
    bool packed;                         // pair siblings into two-lane operations
    BinGen(const Trie &t_, const Bin &b_, bool packed_) : t(t_), b(b_), kids(b_.nodes.size()), packed(packed_)
    {
        for (size_t k = 0; k < b.nodes.size(); ++k) {
            if (b.parent[k] < 0) top.push_back((int)k); else kids[b.parent[k]].push_back((int)k);
        }
    }
    const Node &node(int k) const { return t.nodes[b.nodes[k]]; }
    static std::string S(int k) { return "S[" + str(k) + "]"; }
    static std::string A(int k) { return "A[" + str(k) + "]"; }
    std::vector<int> active(const std::vector<int> &list, int m) const
    {
        std::vector<int> out;
        for (int k : list)
            if ((b.below[k] >> m) & 1u) out.push_back(k);
        return out;
    }

    // ---- forward: S += ... for target degree m; `list` are siblings, bpar their parent's Horner value ----
    // The factor 1/(m-j+1) of a stage rides on the parent's value (one multiplication per parent and
    // degree) instead of on a table of scaled increments, which would cost a register per (letter, factor).
    void fwd_siblings(Emitter &e, ScaleSet &x, const std::vector<int> &list, int m, const std::string &bpar, int indent) const
    {
        const std::vector<int> act = active(list, m);
        if (act.empty()) return;
        const std::string pad((size_t)indent, ' ');
        const int depth = node(act[0]).depth;
        if (depth == m) {
            size_t i = 0;
            if (!bpar.empty() && packed)
                for (; i + 1 < act.size(); i += 2) {
                    const int k0 = act[i], k1 = act[i + 1];
                    e.line(pad + "fma2(" + S(k0) + ", " + S(k1) + ", " + bpar + ", " + bpar + ", " + x.name(node(k0).letter, 1) + ", " +
                           x.name(node(k1).letter, 1) + ", " + S(k0) + ", " + S(k1) + ");");
                }
            for (; i < act.size(); ++i) {
                const int k = act[i];
                if (bpar.empty()) e.line(pad + S(k) + " += " + x.name(node(k).letter, 1) + ";");
                else e.line(pad + S(k) + " = fma(" + bpar + ", " + x.name(node(k).letter, 1) + ", " + S(k) + ");");
            }
            return;
        }
        const std::string rc = "(real)(1.0 / " + str(m - depth + 1) + ".0)";
        const std::string b0 = "b" + str(depth) + "p", b1 = "b" + str(depth) + "q", bs = "s" + str(depth);
        e.line(pad + "{ const real " + bs + " = " + (bpar.empty() ? rc : bpar + " * " + rc) + ";");
        size_t i = 0;
        if (packed)
            for (; i + 1 < act.size(); i += 2) {
                const int k0 = act[i], k1 = act[i + 1];
                e.line(pad + "  { real " + b0 + ", " + b1 + ";");
                e.line(pad + "    fma2(" + b0 + ", " + b1 + ", " + bs + ", " + bs + ", " + x.name(node(k0).letter, 1) + ", " +
                       x.name(node(k1).letter, 1) + ", " + S(k0) + ", " + S(k1) + ");");
                fwd_siblings(e, x, kids[k0], m, b0, indent + 4);
                fwd_siblings(e, x, kids[k1], m, b1, indent + 4);
                e.line(pad + "  }");
            }
        for (; i < act.size(); ++i) {
            const int k = act[i];
            e.line(pad + "  { const real " + b0 + " = fma(" + bs + ", " + x.name(node(k).letter, 1) + ", " + S(k) + ");");
            fwd_siblings(e, x, kids[k], m, b0, indent + 4);
            e.line(pad + "  }");
        }
        e.line(pad + "}");
    }
    std::string forward_step(int index) const
    {
        Emitter body;
        ScaleSet x(t.d);
        for (int m = b.max_depth; m >= 1; --m)  // highest degree first: each reads the previous step's lower values
            fwd_siblings(body, x, top, m, "", 4);
        Emitter e;
        e.line("__device__ __forceinline__ void fwd_step_" + str(index) + "(real (&S)[SMAX], const real (&dx)[D])");
        e.line("{");
        x.declare(e);
        e.s += body.s;
        e.line("}");
        return e.s;
    }

    // ---- backward: one reverse step, target degrees bottom-up ----
    bool tracks_value(int k) const { return (b.below[k] >> (node(k).depth + 1)) != 0; }
    // `ap0`/`ap1`: the two partial accumulators of the adjoint of the parent's Horner value
    void bwd_siblings(Emitter &e, ScaleSet &x, const std::vector<int> &list, int m, const std::string &bpar,
                      const std::string &ap0, const std::string &ap1, int indent) const
    {
        const std::vector<int> act = active(list, m);
        if (act.empty()) return;
        const std::string pad((size_t)indent, ' ');
        const int depth = node(act[0]).depth;
        auto lg = [&](int k) { return "lg" + str(node(k).letter); };
        auto xr = [&](int k) { return x.name(node(k).letter, 1); };
        if (depth == m) {
            size_t i = 0;
            if (!bpar.empty() && packed) {
                for (; i + 1 < act.size(); i += 2) {
                    const int k0 = act[i], k1 = act[i + 1];
                    if (tracks_value(k0) && tracks_value(k1))
                        e.line(pad + "fma2(" + S(k0) + ", " + S(k1) + ", -" + bpar + ", -" + bpar + ", " + xr(k0) + ", " + xr(k1) + ", " + S(k0) + ", " + S(k1) + ");");
                    else {
                        if (tracks_value(k0)) e.line(pad + S(k0) + " = fma(-" + bpar + ", " + xr(k0) + ", " + S(k0) + ");");
                        if (tracks_value(k1)) e.line(pad + S(k1) + " = fma(-" + bpar + ", " + xr(k1) + ", " + S(k1) + ");");
                    }
                    e.line(pad + "fma2(" + lg(k0) + ", " + lg(k1) + ", " + A(k0) + ", " + A(k1) + ", " + bpar + ", " + bpar + ", " + lg(k0) + ", " + lg(k1) + ");");
                    e.line(pad + "fma2(" + ap0 + ", " + ap1 + ", " + A(k0) + ", " + A(k1) + ", " + xr(k0) + ", " + xr(k1) + ", " + ap0 + ", " + ap1 + ");");
                }
            }
            for (; i < act.size(); ++i) {
                const int k = act[i];
                if (tracks_value(k)) {
                    if (bpar.empty()) e.line(pad + S(k) + " -= " + xr(k) + ";");
                    else e.line(pad + S(k) + " = fma(-" + bpar + ", " + xr(k) + ", " + S(k) + ");");
                }
                if (bpar.empty()) e.line(pad + lg(k) + " += " + A(k) + ";");
                else {
                    e.line(pad + lg(k) + " = fma(" + A(k) + ", " + bpar + ", " + lg(k) + ");");
                    e.line(pad + ap0 + " = fma(" + A(k) + ", " + xr(k) + ", " + ap0 + ");");
                }
            }
            return;
        }
        const std::string rc = "(real)(1.0 / " + str(m - depth + 1) + ".0)";
        const std::string dn = str(depth), bs = "s" + dn;
        e.line(pad + "{ const real " + bs + " = " + (bpar.empty() ? rc : bpar + " * " + rc) + ";");
        size_t i = 0;
        if (packed)
            for (; i + 1 < act.size(); i += 2) {
                const int k0 = act[i], k1 = act[i + 1];
                const std::string bp = "b" + dn + "p", bq = "b" + dn + "q";
                const std::string p0 = "a" + dn + "p0", p1 = "a" + dn + "p1", q0 = "a" + dn + "q0", q1 = "a" + dn + "q1";
                e.line(pad + "  { real " + bp + ", " + bq + ", " + p0 + " = (real)0, " + p1 + " = (real)0, " + q0 + " = (real)0, " + q1 + " = (real)0;");
                e.line(pad + "    fma2(" + bp + ", " + bq + ", " + bs + ", " + bs + ", " + xr(k0) + ", " + xr(k1) + ", " + S(k0) + ", " + S(k1) + ");");
                bwd_siblings(e, x, kids[k0], m, bp, p0, p1, indent + 4);
                bwd_siblings(e, x, kids[k1], m, bq, q0, q1, indent + 4);
                e.line(pad + "    add2(" + p0 + ", " + q0 + ", " + p0 + ", " + q0 + ", " + p1 + ", " + q1 + ");");  // adjoints of the two Horner values
                e.line(pad + "    add2(" + A(k0) + ", " + A(k1) + ", " + A(k0) + ", " + A(k1) + ", " + p0 + ", " + q0 + ");");
                e.line(pad + "    mul2(" + p0 + ", " + q0 + ", " + p0 + ", " + q0 + ", " + rc + ", " + rc + ");");
                if (bpar.empty()) {
                    e.line(pad + "    add2(" + lg(k0) + ", " + lg(k1) + ", " + lg(k0) + ", " + lg(k1) + ", " + p0 + ", " + q0 + ");");
                } else {
                    e.line(pad + "    fma2(" + ap0 + ", " + ap1 + ", " + p0 + ", " + q0 + ", " + xr(k0) + ", " + xr(k1) + ", " + ap0 + ", " + ap1 + ");");
                    e.line(pad + "    fma2(" + lg(k0) + ", " + lg(k1) + ", " + p0 + ", " + q0 + ", " + bpar + ", " + bpar + ", " + lg(k0) + ", " + lg(k1) + ");");
                }
                e.line(pad + "  }");
            }
        // Unpaired siblings.  Their Horner values are b = S + s*x with the common s = bpar/(m-depth+1), so the
        // adjoint of s is gathered over the siblings (g) and scaled once; the letter gradient takes a*s.
        const std::string g = "g" + dn;
        const bool gather = i < act.size() && !bpar.empty();
        if (gather) e.line(pad + "  real " + g + " = (real)0;");
        for (; i < act.size(); ++i) {
            const int k = act[i];
            const std::string bp = "b" + dn + "p", p0 = "a" + dn + "p0", p1 = "a" + dn + "p1";
            e.line(pad + "  { const real " + bp + " = fma(" + bs + ", " + xr(k) + ", " + S(k) + "); real " + p0 + " = (real)0" +
                   (packed ? ", " + p1 + " = (real)0;" : ";"));
            bwd_siblings(e, x, kids[k], m, bp, p0, packed ? p1 : p0, indent + 4);
            if (packed) e.line(pad + "    " + p0 + " += " + p1 + ";");
            e.line(pad + "    " + A(k) + " += " + p0 + ";");
            e.line(pad + "    " + lg(k) + " = fma(" + p0 + ", " + bs + ", " + lg(k) + ");");
            if (!bpar.empty()) e.line(pad + "    " + g + " = fma(" + p0 + ", " + xr(k) + ", " + g + ");");
            e.line(pad + "  }");
        }
        if (gather) e.line(pad + "  " + ap0 + " = fma(" + g + ", " + rc + ", " + ap0 + ");");
        e.line(pad + "}");
    }
    std::string backward_step(int index) const
    {
        Emitter body;
        ScaleSet x(t.d);
        for (int m = 1; m <= b.max_depth; ++m) bwd_siblings(body, x, top, m, "", "", "", 4);
        Emitter e;
        e.line("__device__ __forceinline__ void bwd_step_" + str(index) +
               "(real (&S)[SMAX], real (&A)[SMAX], const real (&dx)[D], real *__restrict__ gd)");
        e.line("{");
        x.declare(e);
        std::vector<char> letter_used((size_t)t.d, 0);
        for (size_t k = 0; k < b.nodes.size(); ++k) letter_used[node((int)k).letter] = 1;
        for (int a = 0; a < t.d; ++a)
            if (letter_used[a]) e.line("    real lg" + str(a) + " = (real)0;");
        e.s += body.s;
        // this warp's slab of the step's gradient row: every letter is written, so the slab needs no clearing
        for (int a = 0; a < t.d; ++a)
            e.line("    gd[" + str(a) + "] = " + (letter_used[a] ? "lg" + str(a) : std::string("(real)0")) + ";");
        e.line("}");
        return e.s;
    }
};

// Fixed part of the generated source.  Macros defined ahead of it: D, NBINS, SMAX, WIDTH and the typedef
// `real`.  A block holds kBinsPerBlock bins times NG groups of 32 units (NG = blockDim.x / 128): warp w
// runs bin (w % kBinsPerBlock) on unit group (w / kBinsPerBlock), so the warps that share a scheduler of
// the SM (w mod 4) all run the same straight-line code, which is what keeps the loop of a bin resident
// in the scheduler's instruction cache.
const char *kCommon = R"SRC(
struct Params {
    const real *path;     // (B, L, D)
    real *out;            // forward: (units, WIDTH)
    const real *sig;      // backward: saved forward output
    const real *grad;     // backward: dL/d(out)
    real *inc_grad;       // backward: zeroed (B, L-1, D) accumulator
    long long B, L, W;    // W >= 1
    const int *windows;   // (W, 2) or null
    int chunk;            // steps staged per refill
    int stride;           // scalars between two units' rows of staged increments (odd)
};

struct Unit { long long b; int start, steps; };

// two-lane forms: one packed instruction in float32 (sm_100), two scalar ones in float64
__device__ __forceinline__ void fma2(real &d0, real &d1, real a0, real a1, real b0, real b1, real c0, real c1)
{
#if REAL_IS_FLOAT
    const float2 r = __ffma2_rn(make_float2(a0, a1), make_float2(b0, b1), make_float2(c0, c1));
    d0 = r.x; d1 = r.y;
#else
    d0 = fma(a0, b0, c0); d1 = fma(a1, b1, c1);
#endif
}
__device__ __forceinline__ void add2(real &d0, real &d1, real a0, real a1, real b0, real b1)
{
#if REAL_IS_FLOAT
    const float2 r = __fadd2_rn(make_float2(a0, a1), make_float2(b0, b1));
    d0 = r.x; d1 = r.y;
#else
    d0 = a0 + b0; d1 = a1 + b1;
#endif
}
__device__ __forceinline__ void mul2(real &d0, real &d1, real a0, real a1, real b0, real b1)
{
#if REAL_IS_FLOAT
    const float2 r = __fmul2_rn(make_float2(a0, a1), make_float2(b0, b1));
    d0 = r.x; d1 = r.y;
#else
    d0 = a0 * b0; d1 = a1 * b1;
#endif
}

#define MAX_ROWS 128   // 32 units times at most 4 groups per block

// facts of this block's units; returns the largest step count among them
__device__ __forceinline__ int publish_units(const Params &p, long long first_unit, int rows, Unit *s_unit, int *s_max)
{
    if (threadIdx.x == 0) *s_max = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < rows; i += blockDim.x) {
        const long long unit = first_unit + i;
        Unit u; u.b = 0; u.start = 0; u.steps = 0;
        if (unit < p.B * p.W) {
            u.b = unit / p.W;
            int end = (int)p.L;
            if (p.windows) {
                const long long w = unit % p.W;
                u.start = max(p.windows[2 * w], 0);
                end = min(p.windows[2 * w + 1], (int)p.L);
            }
            u.steps = max(end - u.start - 1, 0);
        }
        s_unit[i] = u;
        atomicMax(s_max, u.steps);
    }
    __syncthreads();
    return *s_max;
}

// Staging of raw path points: s_pts(r * stride + t * D + a) = coordinate a of point c0+t of unit r, for the
// points the unit has in [c0, c0+n].  The copies are asynchronous (cp.async, one scalar each, no
// alignment demand beyond the scalar's) and are committed as one group per call, so that the chunk
// after the one being computed is already on its way.  Increments are formed in registers, step by step.
__device__ __forceinline__ void stage_points_async(const Params &p, const Unit *s_unit, int rows, int c0, int n, real *s_pts)
{
    const int lane = threadIdx.x & 31;
    for (int r = threadIdx.x >> 5; r < rows; r += (int)(blockDim.x >> 5)) {
        const Unit u = s_unit[r];
        const real *src = p.path + (u.b * p.L + u.start + c0) * D;
        const int valid = (min(n, u.steps - c0) + 1) * D;  // <= 0 when the unit has ended before this chunk
        const unsigned dst = (unsigned)__cvta_generic_to_shared(s_pts + r * p.stride);
        for (int j = lane; j < valid; j += 32) {
            if (sizeof(real) == 4)
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + 4u * j), "l"(src + j) : "memory");
            else
                asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst + 8u * j), "l"(src + j) : "memory");
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}
__device__ __forceinline__ void wait_newest_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }
__device__ __forceinline__ void wait_all_copies() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
)SRC";

const char *kForwardKernel = R"SRC(
extern "C" __global__ void __launch_bounds__(512, 1) closure_forward(const Params p)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ Unit s_unit[MAX_ROWS];
    __shared__ int s_max;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int bin = blockIdx.x * BINS_PER_BLOCK + warp % BINS_PER_BLOCK, row = (warp / BINS_PER_BLOCK) * 32 + lane;
    const int rows = (int)(blockDim.x / (32 * BINS_PER_BLOCK)) * 32;
    real *const s_pts0 = reinterpret_cast<real *>(smem_raw), *const s_pts1 = s_pts0 + rows * (size_t)p.stride;
#define s_pts(i) ((i) ? s_pts1 : s_pts0)
    const long long units = p.B * p.W, blocks_of_units = (units + rows - 1) / rows;
    for (long long ub = blockIdx.y; ub < blocks_of_units; ub += gridDim.y) {
        const int max_steps = publish_units(p, ub * rows, rows, s_unit, &s_max);
        const int steps = s_unit[row].steps;
        real S[SMAX];
#pragma unroll
        for (int i = 0; i < SMAX; ++i) S[i] = (real)0;
        const int nchunks = (max_steps + p.chunk - 1) / p.chunk;
        if (nchunks > 0) stage_points_async(p, s_unit, rows, 0, min(p.chunk, max_steps), s_pts(0));
        for (int ci = 0; ci < nchunks; ++ci) {
            const int c0 = ci * p.chunk, n = min(p.chunk, max_steps - c0);
            if (ci + 1 < nchunks) {
                stage_points_async(p, s_unit, rows, c0 + p.chunk, min(p.chunk, max_steps - c0 - p.chunk), s_pts((ci + 1) & 1));
                wait_newest_but_one();
            } else {
                wait_all_copies();
            }
            __syncthreads();  // every thread's copies of this chunk have landed
            const real *mine = s_pts(ci & 1) + row * p.stride;
            const int n_lane = min(n, steps - c0);
            if (n_lane > 0) {
                real x[D], lo[D];
#pragma unroll
                for (int a = 0; a < D; ++a) lo[a] = mine[a];
                FORWARD_SWEEP
            }
            __syncthreads();  // the buffer may be refilled
        }
        const long long unit = ub * rows + row;
        if (unit < units) {
            real *orow = p.out + unit * (long long)WIDTH;
            FORWARD_STORE
        }
    }
}
)SRC";

const char *kBackwardKernel = R"SRC(
extern "C" __global__ void __launch_bounds__(512, 1) closure_backward(const Params p)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ Unit s_unit[MAX_ROWS];
    __shared__ int s_max;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int bin = blockIdx.x * BINS_PER_BLOCK + warp % BINS_PER_BLOCK, row = (warp / BINS_PER_BLOCK) * 32 + lane;
    const int rows = (int)(blockDim.x / (32 * BINS_PER_BLOCK)) * 32;
    real *const s_pts0 = reinterpret_cast<real *>(smem_raw), *const s_pts1 = s_pts0 + rows * (size_t)p.stride;
#define s_pts(i) ((i) ? s_pts1 : s_pts0)
    // per-step gradient rows, one slab per bin of the block: s_gd[bin_local][r * stride + t * D + a]
    real *s_gd = s_pts1 + rows * (size_t)p.stride;
    const size_t slab = rows * (size_t)p.stride;
    const long long units = p.B * p.W, blocks_of_units = (units + rows - 1) / rows;
    for (long long ub = blockIdx.y; ub < blocks_of_units; ub += gridDim.y) {
        const int max_steps = publish_units(p, ub * rows, rows, s_unit, &s_max);
        if (max_steps == 0) continue;  // uniform over the block
        const long long unit = ub * rows + row;
        const bool live = unit < units;
        const int steps = s_unit[row].steps;
        real S[SMAX], A[SMAX];
#pragma unroll
        for (int i = 0; i < SMAX; ++i) { S[i] = (real)0; A[i] = (real)0; }
        const real *srow = p.sig + (live ? unit : 0) * (long long)WIDTH;
        const real *grow = p.grad + (live ? unit : 0) * (long long)WIDTH;
        bool rebuild = false;
        BACKWARD_LOAD
        const int nchunks = (max_steps + p.chunk - 1) / p.chunk;
        // values that are not part of the saved signature are rebuilt with a forward sweep
        if (__syncthreads_or(rebuild ? 1 : 0)) {
            stage_points_async(p, s_unit, rows, 0, min(p.chunk, max_steps), s_pts(0));
            for (int ci = 0; ci < nchunks; ++ci) {
                const int c0 = ci * p.chunk, n = min(p.chunk, max_steps - c0);
                if (ci + 1 < nchunks) {
                    stage_points_async(p, s_unit, rows, c0 + p.chunk, min(p.chunk, max_steps - c0 - p.chunk), s_pts((ci + 1) & 1));
                    wait_newest_but_one();
                } else {
                    wait_all_copies();
                }
                __syncthreads();
                const real *mine = s_pts(ci & 1) + row * p.stride;
                const int n_lane = min(n, steps - c0);
                if (rebuild && n_lane > 0) {
                    real x[D], lo[D];
#pragma unroll
                    for (int a = 0; a < D; ++a) lo[a] = mine[a];
                    REBUILD_SWEEP
                }
                __syncthreads();
            }
        }
        // reverse sweep: chunks from the end, the copy of the chunk before running under the arithmetic
        {
            const int c_last = (nchunks - 1) * p.chunk;
            stage_points_async(p, s_unit, rows, c_last, max_steps - c_last, s_pts((nchunks - 1) & 1));
        }
        for (int ci = nchunks - 1; ci >= 0; --ci) {
            const int c0 = ci * p.chunk, n = min(p.chunk, max_steps - c0);
            if (ci > 0) {
                stage_points_async(p, s_unit, rows, c0 - p.chunk, p.chunk, s_pts((ci - 1) & 1));
                wait_newest_but_one();
            } else {
                wait_all_copies();
            }
            __syncthreads();
            const int n_lane = live ? min(n, steps - c0) : 0;
            {
                // steps of the chunk this lane does not run (its unit is shorter, or the bin does not exist)
                real *mine_gd = s_gd + (warp % BINS_PER_BLOCK) * slab + row * p.stride;
                for (int t = (bin < NBINS ? max(n_lane, 0) : 0); t < n; ++t)
                    for (int a = 0; a < D; ++a) mine_gd[t * D + a] = (real)0;
            }
            if (bin < NBINS && n_lane > 0) {
                const real *mine = s_pts(ci & 1) + row * p.stride;
                real *mine_gd = s_gd + (warp % BINS_PER_BLOCK) * slab + row * p.stride;
                real x[D], hi[D];
#pragma unroll
                for (int a = 0; a < D; ++a) hi[a] = mine[n_lane * D + a];
                BACKWARD_SWEEP
            }
            __syncthreads();
            // flush the units' rows of this chunk, one unit per warp at a time
            for (int r = warp; r < rows; r += (int)(blockDim.x >> 5)) {
                const Unit u = s_unit[r];
                real *dst = p.inc_grad + (u.b * (p.L - 1) + u.start + c0) * D;
                const real *src = s_gd + r * p.stride;
                const int valid = max(0, min(n, u.steps - c0)) * D;
                for (int j = lane; j < valid; j += 32) {
                    real v = src[j];
#pragma unroll
                    for (int k = 1; k < BINS_PER_BLOCK; ++k) v += src[k * slab + j];
                    if (v != (real)0) atomicAdd(&dst[j], v);
                }
            }
            __syncthreads();
        }
    }
}
)SRC";

// ------------------------------------------------------------------------------------------
// bin sizes and block shape
// ------------------------------------------------------------------------------------------
// Forward FMAs per bin and step that keep a bin's loop inside a scheduler's instruction cache (measured:
// a forward loop of about 250 FMAs and a backward loop grown from about 45 run from it; larger loops
// stall on instruction fetch as soon as two of them share a scheduler), and the least a bin should hold
// so that the per-step fixed cost of a warp does not dominate.
constexpr long long kForwardBinFma = 200, kBackwardBinFma = 45, kMinBinFma = 24;
constexpr int kBinsPerBlock = 4;   // one bin per scheduler of the SM
constexpr int kMaxGroupsPerBlock = 4;

void replace_all(std::string &s, const std::string &what, const std::string &with)
{
    for (size_t pos = s.find(what); pos != std::string::npos; pos = s.find(what, pos + with.size()))
        s.replace(pos, what.size(), with);
}

struct Source {
    std::string text;
    int nbins = 0, smax = 0;
    long long fma_forward = 0;  // FMAs the forward code of these bins executes per unit and step
};

// CUDA C++ of one pass (forward or backward) over the given bins.
Source generate(const Trie &t, const std::vector<Bin> &bins, bool is_double, bool backward, bool packed)
{
    Source src;
    src.nbins = (int)bins.size();
    for (const Bin &b : bins) src.smax = std::max(src.smax, (int)b.nodes.size());
    Emitter head;
    head.line(std::string("typedef ") + (is_double ? "double" : "float") + " real;");
    head.line(std::string("#define REAL_IS_FLOAT ") + (is_double ? "0" : "1"));
    head.line("#define D " + str(t.d));
    head.line("#define NBINS " + str(src.nbins));
    head.line("#define SMAX " + str(src.smax));
    head.line("#define BINS_PER_BLOCK " + str(kBinsPerBlock));
    head.line("#define WIDTH " + str(t.width));
    Emitter steps, fsweep, fstore, bload, bsweep, rsweep;
    rsweep.line("switch (bin) {");
    fsweep.line("switch (bin) {");
    fstore.line("switch (bin) {");
    bload.line("switch (bin) {");
    bsweep.line("switch (bin) {");
    for (int i = 0; i < src.nbins; ++i) {
        const Bin &b = bins[i];
        BinGen g(t, b, packed);
        if (!backward || b.rebuild) steps.s += g.forward_step(i);
        if (backward) steps.s += g.backward_step(i);
        long long bin_fma = 0;
        for (unsigned bits : b.below) bin_fma += popcount(bits);
        src.fma_forward += bin_fma;
        const std::string c = "case " + str(i) + ": ";
        // Two steps per trip of the forward loop let the compiler start a step's loads and increments under
        // the previous step's arithmetic (config 3 forward 0.086 -> 0.078 ms) as long as the doubled loop
        // stays inside the instruction cache; four steps, or two in the reverse sweep, fell out of it
        // (0.116 ms forward, 7x slower backward).
        const std::string unroll = 2 * bin_fma <= kForwardBinFma ? "\n#pragma unroll 2\n" : "";
        fsweep.line(c + unroll + "for (int t = 0; t < n_lane; ++t) { for (int a = 0; a < D; ++a) { const real hi = mine[(t + 1) * D + a]; x[a] = hi - lo[a]; lo[a] = hi; } fwd_step_" + str(i) + "(S, x); } break;");
        if (b.rebuild) rsweep.line(c + "for (int t = 0; t < n_lane; ++t) { for (int a = 0; a < D; ++a) { const real hi = mine[(t + 1) * D + a]; x[a] = hi - lo[a]; lo[a] = hi; } fwd_step_" + str(i) + "(S, x); } break;");
        bsweep.line(c + "for (int t = n_lane - 1; t >= 0; --t) { for (int a = 0; a < D; ++a) { const real lo = mine[t * D + a]; x[a] = hi[a] - lo; hi[a] = lo; } bwd_step_" + str(i) + "(S, A, x, mine_gd + t * D); } break;");
        fstore.s += c;
        bload.s += c;
        if (b.rebuild) bload.s += "rebuild = live; ";
        bload.s += "if (live) { ";
        for (size_t k = 0; k < b.nodes.size(); ++k) {
            const Node &n = t.nodes[b.nodes[k]];
            if (b.own[k] && n.col >= 0) {
                fstore.s += "orow[" + str(n.col) + "] = S[" + str((long long)k) + "]; ";
                bload.s += "A[" + str((long long)k) + "] = grow[" + str(n.col) + "]; ";
            }
            if (!b.rebuild && g.tracks_value((int)k)) bload.s += "S[" + str((long long)k) + "] = srow[" + str(n.col) + "]; ";
        }
        fstore.line("break;");
        bload.line("} break;");
    }
    fsweep.line("default: break; }");
    rsweep.line("default: break; }");
    fstore.line("default: break; }");
    bload.line("default: break; }");
    bsweep.line("default: break; }");
    std::string body = backward ? kBackwardKernel : kForwardKernel;
    replace_all(body, "REBUILD_SWEEP", rsweep.s);
    replace_all(body, "FORWARD_SWEEP", fsweep.s);
    replace_all(body, "FORWARD_STORE", fstore.s);
    replace_all(body, "BACKWARD_LOAD", bload.s);
    replace_all(body, "BACKWARD_SWEEP", bsweep.s);
    src.text = head.s + kCommon + steps.s + body;
    return src;
}

// ------------------------------------------------------------------------------------------
// plans
// ------------------------------------------------------------------------------------------
constexpr size_t kPackedMaxNodes = 24;  // node values per lane up to which the paired reverse sweep fits the registers

struct PassPlan {
    CUfunction fn = nullptr;
    int nbins = 0, smax = 0;
    long long fma_forward = 0;
};

struct Plan {
    bool usable = false;
    int d = 0;
    long long width = 0, nodes = 0, fma = 0;
    PassPlan pass[2];  // forward, backward
    std::string log;
};

struct PlanKey {
    int device, dtype, d, depth, bins_forward, bins_backward;
    std::vector<long long> sizes, words;
    bool operator<(const PlanKey &o) const
    {
        if (device != o.device) return device < o.device;
        if (dtype != o.dtype) return dtype < o.dtype;
        if (d != o.d) return d < o.d;
        if (depth != o.depth) return depth < o.depth;
        if (bins_forward != o.bins_forward) return bins_forward < o.bins_forward;
        if (bins_backward != o.bins_backward) return bins_backward < o.bins_backward;
        if (sizes != o.sizes) return sizes < o.sizes;
        return words < o.words;
    }
};

std::mutex g_plan_mutex;
std::map<PlanKey, std::shared_ptr<Plan>> g_plans;

int sm_count()
{
    int sms = 148, device = 0, v = 0;
    if (cudaGetDevice(&device) == cudaSuccess &&
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device) == cudaSuccess && v > 0)
        sms = v;
    return sms;
}

std::string arch_option(int device)
{
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return "";
    std::string a = "--gpu-architecture=sm_" + std::to_string(prop.major) + std::to_string(prop.minor);
    if (prop.major >= 9) a += "a";
    return a;
}

// Directory of compiled kernels kept across processes: $PATHSIG_B200_CACHE_DIR, else $XDG_CACHE_HOME/pathsig_b200,
// else ~/.cache/pathsig_b200; "" (the variable set to an empty string, or no home directory) turns the cache off.
std::string cache_dir()
{
    if (const char *e = getenv("PATHSIG_B200_CACHE_DIR")) return e;
    if (const char *x = getenv("XDG_CACHE_HOME")) { if (*x) return std::string(x) + "/pathsig_b200"; }
    if (const char *h = getenv("HOME")) { if (*h) return std::string(h) + "/.cache/pathsig_b200"; }
    return "";
}

long long spill_bytes(const std::string &log);

// mkdir -p
bool make_dirs(const std::string &dir)
{
    for (size_t pos = 1; pos <= dir.size(); ++pos) {
        if (pos != dir.size() && dir[pos] != '/') continue;
        const std::string part = dir.substr(0, pos);
        if (mkdir(part.c_str(), 0755) != 0 && errno != EEXIST) return false;
    }
    return true;
}

unsigned long long fnv1a(const std::string &s, unsigned long long h = 1469598103934665603ull)
{
    for (unsigned char c : s) { h ^= c; h *= 1099511628211ull; }
    return h;
}

// Compiles `text` to a cubin for `arch` ("--gpu-architecture=sm_100a"); empty result on failure (log filled).
// A cubin compiled before for the same text and options is read back from the cache directory (the file
// name is a hash of both, and the file starts with the text's length and a second hash as a check).
std::vector<char> compile(const std::string &text, const std::string &arch, std::string *log)
{
    std::vector<char> cubin;
    const std::string dir = cache_dir();
    const unsigned long long key = fnv1a(arch, fnv1a(text)), check_hash = fnv1a(text, 88172645463325252ull);
    char name[64];
    snprintf(name, sizeof(name), "/closure_%016llx.cubin", key);
    const std::string file = dir.empty() ? "" : dir + name;
    if (!file.empty()) {
        if (FILE *f = fopen(file.c_str(), "rb")) {
            unsigned long long head[3] = {0, 0, 0};
            if (fread(head, sizeof(head), 1, f) == 1 && head[0] == text.size() && head[1] == check_hash && head[2] > 0 &&
                head[2] < (1ull << 31)) {
                cubin.resize((size_t)head[2]);
                if (fread(cubin.data(), 1, cubin.size(), f) != cubin.size()) cubin.clear();
            }
            fclose(f);
            if (!cubin.empty()) { *log = "ptxas info    : read from " + file + "\n"; return cubin; }
        }
    }
    const Nvrtc &rt = nvrtc();
    if (!rt.ok) { *log = "NVRTC not available"; return cubin; }
    nvrtcProgram prog = nullptr;
    if (rt.CreateProgram(&prog, text.c_str(), "psig_closure.cu", 0, nullptr, nullptr) != 0) { *log = "nvrtcCreateProgram failed"; return cubin; }
    const char *opts[] = {arch.c_str(), "--std=c++17", "-lineinfo", "--ptxas-options=-v", "-diag-suppress=177"};
    const int rc = rt.CompileProgram(prog, 5, opts);
    size_t log_size = 0;
    if (rt.GetProgramLogSize(prog, &log_size) == 0 && log_size > 1) {
        log->resize(log_size);
        rt.GetProgramLog(prog, &(*log)[0]);
        while (!log->empty() && log->back() == '\0') log->pop_back();
    }
    if (rc == 0) {
        size_t size = 0;
        if (rt.GetCUBINSize(prog, &size) == 0 && size > 0) {
            cubin.resize(size);
            if (rt.GetCUBIN(prog, cubin.data()) != 0) cubin.clear();
        }
    }
    rt.DestroyProgram(&prog);
    // keep it for the next process, unless this version spilled (its caller will replace it)
    if (!cubin.empty() && !file.empty() && spill_bytes(*log) == 0) {
        if (make_dirs(dir)) {
            const std::string tmp = file + ".tmp" + std::to_string((long long)getpid());
            if (FILE *f = fopen(tmp.c_str(), "wb")) {
                const unsigned long long head[3] = {text.size(), check_hash, cubin.size()};
                const bool ok = fwrite(head, sizeof(head), 1, f) == 1 && fwrite(cubin.data(), 1, cubin.size(), f) == cubin.size();
                fclose(f);
                if (!ok || rename(tmp.c_str(), file.c_str()) != 0) remove(tmp.c_str());
            }
        }
    }
    return cubin;
}

// Bytes of register spills ptxas reported in a compile log ("N bytes spill stores").
long long spill_bytes(const std::string &log)
{
    long long total = 0;
    const std::string tag = " bytes spill stores";
    for (size_t pos = log.find(tag); pos != std::string::npos; pos = log.find(tag, pos + 1)) {
        size_t b = pos;
        while (b > 0 && log[b - 1] >= '0' && log[b - 1] <= '9') --b;
        total += atoll(log.substr(b, pos - b).c_str());
    }
    return total;
}

// Number of bins for a pass: enough that a bin's loop stays small, and, when the units alone cannot
// fill the SMs (one block per SM), more bins up to the point where bins get too small to pay.
int bins_for(long long units, long long fma, bool backward)
{
    const long long cap = backward ? kBackwardBinFma : kForwardBinFma;
    long long bins = std::max(1LL, (fma + cap - 1) / cap);
    const long long groups = std::max(1LL, (units + 31) / 32), sms = sm_count();
    const long long fill = kBinsPerBlock * (sms / std::min(groups, sms));  // bins that give every SM a block
    const long long most = std::max(1LL, fma / kMinBinFma);
    if (fill > bins) bins = std::min(fill, most);
    bins = (bins + kBinsPerBlock - 1) / kBinsPerBlock * kBinsPerBlock;
    return (int)std::min(bins, 4096LL);
}

std::shared_ptr<Plan> get_plan(const PsigSigDesc &desc, const LevelTable &lt, const int64_t *words_host, long long units)
{
    PlanKey key;
    if (cudaGetDevice(&key.device) != cudaSuccess) return nullptr;
    key.dtype = desc.dtype;
    key.d = lt.d;
    key.depth = lt.depth;
    long long listed = 0, d_pow = 1, width = 0;
    for (int k = 1; k <= lt.depth; ++k) {
        d_pow *= lt.d;
        key.sizes.push_back(lt.size[k]);
        width += lt.size[k];
        if (lt.size[k] != d_pow) listed += lt.size[k];
    }
    if (listed > 0 && !words_host) return nullptr;
    if (width > kMaxClosureNodes) return nullptr;
    key.words.assign(words_host, words_host + listed);
    // the bin counts depend on the closure, which is only known once the trie is built: look the
    // word set up with provisional counts first
    std::lock_guard<std::mutex> lock(g_plan_mutex);
    static std::map<PlanKey, long long> closure_fma_of;  // word set -> forward FMAs of its closure (bins fields zero)
    key.bins_forward = key.bins_backward = 0;
    Trie trie;
    bool have_trie = false;
    auto known = closure_fma_of.find(key);
    if (known == closure_fma_of.end()) {
        have_trie = build_trie(lt, words_host, &trie);
        known = closure_fma_of.emplace(key, have_trie ? closure_fma(trie) : -1).first;
    }
    const long long fma = known->second;
    PlanKey full = key;
    if (fma > 0) {
        full.bins_forward = bins_for(units, fma, false);
        full.bins_backward = bins_for(units, fma, true);
    }
    auto it = g_plans.find(full);
    if (it != g_plans.end()) return it->second;
    auto plan = std::make_shared<Plan>();
    g_plans[full] = plan;
    if (fma <= 0) { plan->log = "closure too large, or a word listed twice"; return plan; }
    if (!have_trie && !build_trie(lt, words_host, &trie)) { plan->log = "closure could not be rebuilt"; return plan; }
    const Driver &drv = driver();
    if (!drv.ok) { plan->log = "driver entry points not available"; return plan; }
    cudaFree(nullptr);  // make sure the primary context of the device is current
    const std::string arch = arch_option(key.device);
    for (int pass = 0; pass < 2; ++pass) {
        const std::vector<Bin> bins = make_bins(trie, pass == 0 ? full.bins_forward : full.bins_backward);
        // Sibling pairs as packed two-lane operations halve the issue slots of the reverse sweep wherever
        // the trie branches, at the price of registers (aligned pairs, two accumulators per degree): they
        // are used for bins of few nodes, and a version that spills is replaced by the scalar one.  The
        // forward sweep runs one warp per scheduler where it can and is bound by latency; pairing
        // measured no gain there.
        size_t most_nodes = 0;
        for (const Bin &b : bins) most_nodes = std::max(most_nodes, b.nodes.size());
        const bool packed = pass == 1 && desc.dtype == PSIG_F32 && most_nodes <= kPackedMaxNodes;
        Source src = generate(trie, bins, desc.dtype == PSIG_F64, pass == 1, packed);
        std::string log;
        std::vector<char> cubin = compile(src.text, arch, &log);
        if (packed && (cubin.empty() || spill_bytes(log) > 0)) {
            plan->log += log;
            log.clear();
            src = generate(trie, bins, desc.dtype == PSIG_F64, pass == 1, false);
            cubin = compile(src.text, arch, &log);
        }
        plan->log += log;
        if (cubin.empty()) return plan;
        CUmodule mod = nullptr;
        if (drv.ModuleLoadData(&mod, cubin.data()) != 0) { plan->log += "cuModuleLoadData failed"; return plan; }
        if (drv.ModuleGetFunction(&plan->pass[pass].fn, mod, pass == 0 ? "closure_forward" : "closure_backward") != 0) {
            plan->log += "kernel lookup failed";
            return plan;
        }
        plan->pass[pass].nbins = src.nbins;
        plan->pass[pass].smax = src.smax;
        plan->pass[pass].fma_forward = src.fma_forward;
    }
    plan->d = trie.d;
    plan->width = trie.width;
    plan->nodes = (long long)trie.nodes.size();
    plan->fma = fma;
    plan->usable = true;
    return plan;
}

// Mirrors `struct Params` of the generated source.
template <typename T>
struct LaunchParams {
    const T *path;
    T *out;
    const T *sig;
    const T *grad;
    T *inc_grad;
    long long B, L, W;
    const int *windows;
    int chunk;
    int stride;
};

template <typename T>
int launch(const Plan &plan, const PassPlan &pass, LaunchParams<T> &p, long long units, int buffers, cudaStream_t stream)
{
    const long long groups = (units + 31) / 32, sms = sm_count();
    const long long bin_blocks = (pass.nbins + kBinsPerBlock - 1) / kBinsPerBlock;
    // groups of 32 units per block: as few as lets the grid fit one block per SM (a warp alone on its
    // scheduler runs fastest), at most kMaxGroupsPerBlock
    int ng = 1;
    while (ng < kMaxGroupsPerBlock && (groups + ng - 1) / ng * bin_blocks > sms) ng *= 2;
    // `buffers` rows of about chunk*d scalars per unit: two buffers of points, plus the gradients in backward;
    // wide paths take fewer groups per block so that a chunk still holds a few steps
    auto chunk_for = [&](int g) { return (long long)(kStageBytes / (sizeof(T) * 32 * g * (size_t)plan.d * buffers)) - 1; };
    while (ng > 1 && chunk_for(ng) < 4) ng /= 2;
    const long long unit_blocks = (groups + ng - 1) / ng;
    const int rows = 32 * ng;
    long long chunk = chunk_for(ng);
    if (chunk < 1) return PSIG_ERR_TOO_LARGE;
    p.chunk = (int)std::min(chunk, 32LL);
    p.stride = ((p.chunk + 1) * plan.d) | 1;
    const size_t need = sizeof(T) * rows * (size_t)p.stride * buffers;
    // one block per SM: two blocks would put two different loops on each scheduler
    const unsigned smem = (unsigned)std::max(need, kOneBlockPerSmBytes);
    const unsigned gx = (unsigned)bin_blocks;
    const unsigned gy = (unsigned)std::min(unit_blocks, std::max(1LL, std::min(65535LL, sms / std::max(1LL, bin_blocks))));
    void *args[] = {&p};
    const Driver &drv = driver();
    if (drv.FuncSetAttribute(pass.fn, 8 /* max dynamic shared size */, (int)smem) != 0) return PSIG_ERR_CUDA;
    const int rc = drv.LaunchKernel(pass.fn, gx, gy, 1, 32 * kBinsPerBlock * ng, 1, 1, smem, stream, args, nullptr);
    count_launch();
    return rc == 0 ? PSIG_OK : PSIG_ERR_CUDA;
}

template <typename T>
__global__ void increments_to_points_closure(const T *__restrict__ inc_grad, T *__restrict__ path_grad, long long B,
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

}  // namespace

// Whether the closure kernels serve this description: a host copy of the word codes is there (or
// every degree is dense), the closure is small enough to live in registers bin by bin, and the
// specialised code could be built for the current device.  Compiles on first use.
bool closure_supported(const PsigSigDesc &desc, const LevelTable &lt)
{
    const long long units = desc.B * (desc.W > 0 ? desc.W : 1);
    if (units <= 0) return false;
    const auto plan = get_plan(desc, lt, desc.words_host, units);
    return plan && plan->usable;
}

// Whether the run-time compiler the family depends on can be loaded (host only).
bool closure_compiler_available() { return nvrtc().ok; }

// Cheap test (no compilation) used by the automatic selection: dense rows, or projected rows with a host
// copy of the codes; a closure of moderate size; enough work to repay the one-off compilation; and
// channels few enough that a chunk of staged points fits shared memory.
bool closure_worthwhile(const PsigSigDesc &desc, const LevelTable &lt)
{
    bool listed = false;
    long long d_pow = 1;
    for (int k = 1; k <= lt.depth; ++k) { d_pow *= lt.d; listed = listed || lt.size[k] != d_pow; }
    if (listed && !desc.words_host) return false;
    if (lt.d > 64) return false;
    const long long units = desc.B * (desc.W > 0 ? desc.W : 1);
    if (units < 256) return false;
    long long words = 0;
    for (int k = 1; k <= lt.depth; ++k) words += lt.size[k];
    if (words == 0 || words > kMaxClosureNodes) return false;
    return (double)units * (double)(desc.L - 1) * (double)words >= 2.0e7;
}

template <typename T>
int closure_sig_forward(const PsigSigDesc &desc, const LevelTable &lt, const T *path, T *out, cudaStream_t stream)
{
    const long long W = desc.W > 0 ? desc.W : 1, units = desc.B * W;
    if (units == 0) return PSIG_OK;
    const auto plan = get_plan(desc, lt, desc.words_host, units);
    if (!plan || !plan->usable) return PSIG_ERR_UNSUPPORTED;
    LaunchParams<T> p{path, out, nullptr, nullptr, nullptr, desc.B, desc.L, W, desc.W > 0 ? desc.windows : nullptr, 0, 0};
    return launch<T>(*plan, plan->pass[0], p, units, 2, stream);
}

template <typename T>
int closure_sig_backward(const PsigSigDesc &desc, const LevelTable &lt, const T *path, const T *sig, const T *grad,
                         T *grad_path, T *inc_grad_ws, cudaStream_t stream)
{
    const long long W = desc.W > 0 ? desc.W : 1, units = desc.B * W;
    if (desc.B == 0) return PSIG_OK;
    const auto plan = get_plan(desc, lt, desc.words_host, units);
    if (!plan || !plan->usable) return PSIG_ERR_UNSUPPORTED;
    const size_t inc_bytes = sizeof(T) * (size_t)desc.B * (size_t)(desc.L - 1) * lt.d;
    if (cudaMemsetAsync(inc_grad_ws, 0, inc_bytes, stream) != cudaSuccess) return PSIG_ERR_CUDA;
    if (units > 0) {
        LaunchParams<T> p{path, nullptr, sig, grad, inc_grad_ws, desc.B, desc.L, W, desc.W > 0 ? desc.windows : nullptr, 0, 0};
        const int rc = launch<T>(*plan, plan->pass[1], p, units, 2 + kBinsPerBlock, stream);
        if (rc != PSIG_OK) return rc;
    }
    const long long total = desc.B * desc.L * lt.d;
    long long nb = (total + 255) / 256;
    if (nb > 148 * 32) nb = 148 * 32;
    increments_to_points_closure<T><<<(unsigned)nb, 256, 0, stream>>>(inc_grad_ws, grad_path, desc.B, desc.L, lt.d);
    return check_launch();
}

// Generated source (forward pass followed by backward pass) and its statistics for a description,
// without compiling: returns the source length, writes up to `capacity` bytes.
long long closure_source(const PsigSigDesc &desc, const LevelTable &lt, int target_bins, char *buffer, long long capacity,
                         long long *stats)
{
    Trie trie;
    if (!build_trie(lt, desc.words_host, &trie)) return PSIG_ERR_UNSUPPORTED;
    const std::vector<Bin> bins = make_bins(trie, target_bins);
    const Source fwd = generate(trie, bins, desc.dtype == PSIG_F64, false, false);
    size_t most_nodes = 0;
    for (const Bin &b : bins) most_nodes = std::max(most_nodes, b.nodes.size());
    const Source bwd = generate(trie, bins, desc.dtype == PSIG_F64, true, desc.dtype == PSIG_F32 && most_nodes <= kPackedMaxNodes);
    // the two passes are separate translation units; the separator lets a caller split them
    const std::string text = fwd.text + "\n//---- backward pass ----\n" + bwd.text;
    if (stats) {
        stats[0] = (long long)trie.nodes.size();
        stats[1] = closure_fma(trie);
        stats[2] = fwd.fma_forward;
        stats[3] = fwd.nbins;
        stats[4] = std::max(fwd.smax, bwd.smax);
    }
    if (buffer && capacity > 0) {
        const long long n = std::min<long long>(capacity - 1, (long long)text.size());
        std::memcpy(buffer, text.data(), (size_t)n);
        buffer[n] = 0;
    }
    return (long long)text.size();
}

// Compiles a source produced by closure_source (both passes) for `arch` without touching a device.
int closure_compile_only(const char *text, const char *arch, char *log, long long log_capacity)
{
    const std::string all(text), sep = "\n//---- backward pass ----\n";
    const size_t cut = all.find(sep);
    std::vector<std::string> units;
    if (cut == std::string::npos) units.push_back(all);
    else { units.push_back(all.substr(0, cut)); units.push_back(all.substr(cut + sep.size())); }
    std::string logs;
    bool ok = true;
    for (const std::string &u : units) {
        std::string l;
        ok = !compile(u, std::string("--gpu-architecture=") + arch, &l).empty() && ok;
        logs += l;
    }
    if (log && log_capacity > 0) {
        const long long n = std::min<long long>(log_capacity - 1, (long long)logs.size());
        std::memcpy(log, logs.data(), (size_t)n);
        log[n] = 0;
    }
    return ok ? PSIG_OK : PSIG_ERR_CUDA;
}

template int closure_sig_forward<float>(const PsigSigDesc &, const LevelTable &, const float *, float *, cudaStream_t);
template int closure_sig_forward<double>(const PsigSigDesc &, const LevelTable &, const double *, double *, cudaStream_t);
template int closure_sig_backward<float>(const PsigSigDesc &, const LevelTable &, const float *, const float *,
                                         const float *, float *, float *, cudaStream_t);
template int closure_sig_backward<double>(const PsigSigDesc &, const LevelTable &, const double *, const double *,
                                          const double *, double *, double *, cudaStream_t);

}  // namespace psig
