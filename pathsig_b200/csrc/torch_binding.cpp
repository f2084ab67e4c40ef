// Operator registration of pathsig_b200 with the PyTorch dispatcher (libpathsig_b200_torch.so).
//
// Counterpart of the reference's src/pathsig/bindings.cpp:7-64 (schemas, pt2_compliant_tag) and of the
// TORCH_LIBRARY_IMPL(pathsig, CUDA, ...) blocks of its launchers (src/pathsig/forward/sig_launch.cu:345-348,
// src/pathsig/backward/sig_backward_launch.cu:468-471): the same four schemas, registered for the CUDA key
// only, in the namespace `pathsig_b200` (so that a build of the reference can be loaded in the same
// process), plus the operators the reference does not have (projected log-signature, Chen product).
// Every implementation validates like the reference launchers (src/pathsig/forward/sig_launch.cu:84-121,
// src/pathsig/backward/sig_backward_launch.cu:94-155), allocates its outputs with the caching allocator
// and hands raw pointers plus the current stream to the C ABI of include/pathsig_b200.h.  torch is used
// for memory, streams and dispatch only; fake (meta) implementations and autograd formulas are registered
// from Python (pathsig_b200/ops.py).
#include <ATen/ATen.h>
#include <ATen/Context.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGraphsC10Utils.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <nvtx3/nvToolsExt.h>

#include <atomic>
#include <list>
#include <mutex>
#include <tuple>
#include <vector>

#include "../../include/pathsig_b200.h"

namespace {

std::atomic<int> g_algo{PSIG_ALGO_AUTO};

// NVTX range around an operator call (host side: validation, allocation, enqueue), so that a timeline
// shows which operator a kernel belongs to.  Costs nothing measurable without a tool attached.
struct Range {
    explicit Range(const char *name) { nvtxRangePushA(name); }
    ~Range() { nvtxRangePop(); }
    Range(const Range &) = delete;
    Range &operator=(const Range &) = delete;
};

void check(int64_t status, const char *what)
{
    TORCH_CHECK(status >= 0, "pathsig_b200::", what, ": ", psig_status_string((int)status), " (status ", status, ")");
}

int dtype_id(const at::Tensor &t)
{
    if (t.scalar_type() == at::kFloat) return PSIG_F32;
    if (t.scalar_type() == at::kDouble) return PSIG_F64;
    TORCH_CHECK(false, "path must be float32 or float64");
}

void *stream_of(const at::Tensor &t) { return at::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

const void *ptr(const at::Tensor &t) { return t.numel() > 0 ? t.data_ptr() : nullptr; }

// Every tensor operand must live on the device the kernels are launched on.  The dispatcher checks this
// for operators with structured kernels only; a pointer into another GPU's memory would fault there.
void same_device(const at::Tensor &anchor, const at::Tensor &t, const char *name)
{
    TORCH_CHECK(t.device() == anchor.device(), name, " must be on the same device as the path/signature (", name,
                " is on ", t.device(), ", expected ", anchor.device(), ")");
}

void check_words(const at::Tensor &words)
{
    TORCH_CHECK(words.is_cuda(), "encoded_words must be CUDA");
    TORCH_CHECK(words.scalar_type() == at::kLong, "encoded_words must be int64");
    TORCH_CHECK(words.is_contiguous(), "encoded_words must be contiguous");
    TORCH_CHECK(words.dim() == 1, "encoded_words must be 1D");
}

// Host copies of word-code tensors.  The prefix-closure kernels are generated from the word set, so the
// library wants the codes in host memory; reading them back on every call would synchronise, so the copy
// is made once per (storage, version) and kept while the device tensor is alive.  An entry holds a
// reference to its device tensor, which keeps the address from being reused by another tensor.
struct HostWords {
    const void *data;
    int64_t version;
    int64_t numel;
    int device;
    at::Tensor on_device, on_host;
};
std::mutex g_words_mutex;
std::list<HostWords> g_words;  // most recently used first
constexpr size_t kHostWordsLimit = 64;

at::Tensor host_words(const at::Tensor &words)
{
    std::lock_guard<std::mutex> lock(g_words_mutex);
    for (auto it = g_words.begin(); it != g_words.end(); ++it) {
        if (it->data == words.data_ptr() && it->version == words._version() && it->numel == words.numel() &&
            it->device == words.get_device()) {
            g_words.splice(g_words.begin(), g_words, it);
            return g_words.front().on_host;
        }
    }
    // no device read inside a graph capture; the library then uses another kernel family
    if (c10::cuda::currentStreamCaptureStatusMayInitCtx() != c10::cuda::CaptureStatus::None) return at::Tensor();
    HostWords e{words.data_ptr(), words._version(), words.numel(), (int)words.get_device(), words,
                words.detach().to(at::kCPU).contiguous()};
    g_words.push_front(e);
    while (g_words.size() > kHostWordsLimit) g_words.pop_back();
    return g_words.front().on_host;
}

int64_t ipow(int64_t b, int64_t e) { int64_t r = 1; for (int64_t i = 0; i < e; ++i) r *= b; return r; }

int64_t row_width(int64_t d, int64_t depth, bool alt, at::IntArrayRef level_sizes)
{
    int64_t w = 0;
    for (int64_t k = 1; k <= depth; ++k) w += alt ? level_sizes[k] : ipow(d, k);
    return w;
}

// Validated PsigSigDesc; `keep` receives tensors that must stay alive during the call.
PsigSigDesc sig_desc(const at::Tensor &path, int64_t depth, bool alt, const at::Tensor &encoded_words,
                     at::IntArrayRef level_sizes, bool use_windows, const at::Tensor &windows, std::vector<at::Tensor> &keep)
{
    TORCH_CHECK(path.is_cuda(), "path must be CUDA");
    TORCH_CHECK(path.dim() == 3, "path must be [B,T,d]");
    TORCH_CHECK(depth >= 1 && depth <= PSIG_MAX_DEPTH, "depth must be in [1,12]");
    TORCH_CHECK(path.size(1) >= 2, "path must have at least 2 time steps");
    PsigSigDesc desc{};
    desc.dtype = dtype_id(path);
    desc.d = (int32_t)path.size(2);
    desc.depth = (int32_t)depth;
    desc.B = path.size(0);
    desc.L = path.size(1);
    desc.projected = alt ? 1 : 0;
    desc.algo = g_algo.load();
    // torch.use_deterministic_algorithms(True): ask for the fixed-order backward where the library has one
    if (at::globalContext().deterministicAlgorithms()) desc.flags |= PSIG_FLAG_DETERMINISTIC;
    if (alt) {
        check_words(encoded_words);
        same_device(path, encoded_words, "encoded_words");
        TORCH_CHECK((int64_t)level_sizes.size() >= depth + 1, "level_sizes must cover at least depth + 1 entries");
        int64_t need = 0;
        for (int64_t k = 1; k <= depth; ++k) {
            desc.level_sizes[k] = level_sizes[k];
            if (level_sizes[k] != ipow(desc.d, k)) need += level_sizes[k];
        }
        TORCH_CHECK(encoded_words.numel() >= need, "encoded_words holds fewer codes than level_sizes requires");
        if (encoded_words.numel() > 0) {
            desc.words = encoded_words.data_ptr<int64_t>();
            at::Tensor host = host_words(encoded_words);
            if (host.defined()) {
                desc.words_host = host.data_ptr<int64_t>();
                keep.push_back(host);
            }
        }
    }
    if (use_windows) {
        TORCH_CHECK(windows.is_cuda(), "windows must be CUDA");
        TORCH_CHECK(windows.dim() == 2 && windows.size(1) == 2, "windows must be [W,2]");
        TORCH_CHECK(windows.scalar_type() == at::kInt || windows.scalar_type() == at::kLong, "windows must be int32");
        same_device(path, windows, "windows");
        at::Tensor win = windows.to(at::kInt).contiguous();
        keep.push_back(win);
        desc.W = win.size(0);
        desc.windows = win.numel() > 0 ? win.data_ptr<int32_t>() : nullptr;
    }
    return desc;
}

at::Tensor compute_signature(const at::Tensor &path_in, int64_t depth, bool alt, const at::Tensor &encoded_words,
                             at::IntArrayRef level_sizes, bool use_windows, const at::Tensor &windows)
{
    Range range("pathsig_b200::compute_signature");
    TORCH_CHECK(path_in.is_cuda(), "path must be CUDA");
    c10::cuda::CUDAGuard guard(path_in.device());
    at::Tensor path = path_in.contiguous();
    std::vector<at::Tensor> keep;
    PsigSigDesc desc = sig_desc(path, depth, alt, encoded_words, level_sizes, use_windows, windows, keep);
    const int64_t D = row_width(desc.d, desc.depth, alt, level_sizes);
    at::Tensor out = use_windows ? at::empty({desc.B, desc.W, D}, path.options()) : at::empty({desc.B, D}, path.options());
    if (out.numel() == 0) return out;  // no paths, no windows or no requested words: nothing to launch
    check(psig_sig_forward(&desc, path.data_ptr(), out.data_ptr(), stream_of(path)), "compute_signature");
    return out;
}

at::Tensor signature_backward(const at::Tensor &path_in, const at::Tensor &signature_in, const at::Tensor &grad_in,
                              int64_t depth, bool alt, const at::Tensor &encoded_words, at::IntArrayRef level_sizes,
                              bool use_windows, const at::Tensor &windows)
{
    Range range("pathsig_b200::signature_backward");
    TORCH_CHECK(path_in.is_cuda(), "path must be CUDA");
    TORCH_CHECK(signature_in.is_cuda(), "signature must be CUDA");
    TORCH_CHECK(grad_in.is_cuda(), "grad_signature must be CUDA");
    TORCH_CHECK(signature_in.scalar_type() == path_in.scalar_type(), "signature must have same dtype as path");
    TORCH_CHECK(grad_in.scalar_type() == path_in.scalar_type(), "grad_signature must have same dtype as path");
    TORCH_CHECK(signature_in.sizes() == grad_in.sizes(), "grad_signature must match signature shape");
    same_device(path_in, signature_in, "signature");
    same_device(path_in, grad_in, "grad_signature");
    c10::cuda::CUDAGuard guard(path_in.device());
    at::Tensor path = path_in.contiguous(), sig = signature_in.contiguous(), grad = grad_in.contiguous();
    std::vector<at::Tensor> keep;
    PsigSigDesc desc = sig_desc(path, depth, alt, encoded_words, level_sizes, use_windows, windows, keep);
    const int64_t D = row_width(desc.d, desc.depth, alt, level_sizes);
    const bool shape_ok = use_windows ? (sig.dim() == 3 && sig.size(0) == desc.B && sig.size(1) == desc.W && sig.size(2) == D)
                                      : (sig.dim() == 2 && sig.size(0) == desc.B && sig.size(1) == D);
    if (!shape_ok) {
        TORCH_CHECK(!(use_windows && sig.dim() == 3 && sig.size(1) != desc.W), "windows.size(0) must match signature num_windows");
        TORCH_CHECK(false, "signature must be [B,S] or [B,W,S]");
    }
    if (sig.numel() == 0) return at::zeros_like(path);  // an empty signature carries no gradient
    at::Tensor grad_path = at::empty_like(path);
    const int64_t ws_bytes = psig_sig_backward_workspace(&desc);
    check(ws_bytes, "signature_backward");
    at::Tensor ws = at::empty({std::max<int64_t>(ws_bytes, 1)}, path.options().dtype(at::kByte));
    check(psig_sig_backward(&desc, path.data_ptr(), sig.data_ptr(), grad.data_ptr(), grad_path.data_ptr(), ws.data_ptr(),
                            ws_bytes, stream_of(path)),
          "signature_backward");
    return grad_path;
}

PsigLogDesc log_desc(const at::Tensor &signature, int64_t depth, int64_t d, bool alt, const at::Tensor &encoded_words,
                     at::IntArrayRef level_sizes)
{
    TORCH_CHECK(depth >= 1 && depth <= PSIG_MAX_DEPTH, "depth must be in [1,12]");
    TORCH_CHECK(d >= 1, "d must be >= 1");
    TORCH_CHECK(signature.dim() == 2 || signature.dim() == 3, "signature must be [B,S] or [B,W,S]");
    PsigLogDesc desc{};
    desc.dtype = dtype_id(signature);
    desc.d = (int32_t)d;
    desc.depth = (int32_t)depth;
    desc.algo = g_algo.load();
    desc.rows = signature.size(-1) > 0 ? signature.numel() / signature.size(-1) : 0;
    desc.top_size = ipow(d, depth);
    if (alt) {
        check_words(encoded_words);
        same_device(signature, encoded_words, "encoded_words");
        TORCH_CHECK((int64_t)level_sizes.size() >= depth + 1, "level_sizes must have entries up to depth");
        desc.top_size = level_sizes[depth];
        if (desc.top_size != ipow(d, depth)) {
            TORCH_CHECK(encoded_words.numel() >= desc.top_size, "encoded_words holds fewer codes than level_sizes[depth]");
            desc.top_words = encoded_words.numel() > 0 ? encoded_words.data_ptr<int64_t>() : nullptr;
        }
    }
    return desc;
}

std::vector<int64_t> with_last(const at::Tensor &t, int64_t last)
{
    std::vector<int64_t> shape(t.sizes().begin(), t.sizes().end());
    shape.back() = last;
    return shape;
}

std::tuple<at::Tensor, at::Tensor> sig_to_logsig(const at::Tensor &signature_in, int64_t depth, int64_t d, bool alt,
                                                 const at::Tensor &encoded_words, at::IntArrayRef level_sizes)
{
    Range range("pathsig_b200::sig_to_logsig");
    TORCH_CHECK(signature_in.is_cuda(), "signature must be CUDA");
    c10::cuda::CUDAGuard guard(signature_in.device());
    at::Tensor sig = signature_in.contiguous();
    PsigLogDesc desc = log_desc(sig, depth, d, alt, encoded_words, level_sizes);
    const int64_t S = psig_logsig_size(&desc);
    check(S, "sig_to_logsig");
    TORCH_CHECK(S == sig.size(-1), "signature width ", sig.size(-1), " does not match the layout width ", S);
    at::Tensor logsig = at::empty_like(sig);
    const int64_t per_row = psig_logsig_cache_size(&desc);
    check(per_row, "sig_to_logsig");
    at::Tensor cache = at::empty(with_last(sig, per_row), sig.options());
    check(psig_logsig_forward(&desc, ptr(sig), const_cast<void *>(ptr(logsig)), const_cast<void *>(ptr(cache)), stream_of(sig)),
          "sig_to_logsig");
    return std::make_tuple(logsig, cache);
}

at::Tensor logsig_backward(const at::Tensor &signature_in, const at::Tensor &P_in, const at::Tensor &grad_in, int64_t depth,
                           bool alt, const at::Tensor &encoded_words, at::IntArrayRef level_sizes)
{
    Range range("pathsig_b200::logsig_backward");
    TORCH_CHECK(signature_in.is_cuda(), "sig must be CUDA");
    TORCH_CHECK(P_in.is_cuda(), "P must be CUDA");
    TORCH_CHECK(grad_in.is_cuda(), "grad_logsig must be CUDA");
    TORCH_CHECK(P_in.scalar_type() == signature_in.scalar_type(), "P must have same dtype as sig");
    TORCH_CHECK(grad_in.scalar_type() == signature_in.scalar_type(), "grad_logsig must have same dtype as sig");
    TORCH_CHECK(grad_in.sizes() == signature_in.sizes(), "grad_logsig must match sig shape");
    same_device(signature_in, P_in, "P");
    same_device(signature_in, grad_in, "grad_logsig");
    TORCH_CHECK((int64_t)level_sizes.size() > depth, "level_sizes must have entries up to depth");
    const int64_t d = level_sizes[1];  // the channel count travels in level_sizes[1], as in the reference
    TORCH_CHECK(d >= 1, "level_sizes[1] must be >= 1 (infers path_dim)");
    c10::cuda::CUDAGuard guard(signature_in.device());
    at::Tensor sig = signature_in.contiguous(), cache = P_in.contiguous(), grad = grad_in.contiguous();
    PsigLogDesc desc = log_desc(sig, depth, d, alt, encoded_words, level_sizes);
    // The cache tells which form of the kernels produced it: S*depth scalars per row belong to the form
    // that streams through global scratch, an empty one to the row-in-shared-memory form.
    bool lead_ok = cache.dim() == sig.dim();
    for (int64_t i = 0; lead_ok && i + 1 < sig.dim(); ++i) lead_ok = cache.size(i) == sig.size(i);
    TORCH_CHECK(lead_ok && (cache.size(-1) == 0 || cache.size(-1) == sig.size(-1) * depth),
                "P must be [B,(W),S*depth] (or [B,(W),0] as returned by sig_to_logsig)");
    desc.algo = cache.size(-1) > 0 ? PSIG_ALGO_GENERIC : PSIG_ALGO_AUTO;
    TORCH_CHECK(psig_logsig_cache_size(&desc) == cache.size(-1), "P does not belong to a sig_to_logsig call with these arguments");
    at::Tensor grad_sig = at::empty_like(sig);
    const int64_t ws_bytes = psig_logsig_backward_workspace(&desc);
    check(ws_bytes, "logsig_backward");
    at::Tensor ws = at::empty({std::max<int64_t>(ws_bytes, 1)}, sig.options().dtype(at::kByte));
    check(psig_logsig_backward(&desc, ptr(sig), ptr(cache), ptr(grad), const_cast<void *>(ptr(grad_sig)), ws.data_ptr(), ws_bytes,
                               stream_of(sig)),
          "logsig_backward");
    return grad_sig;
}

PsigLogDesc projected_log_desc(const at::Tensor &sig, int64_t depth, int64_t d, const at::Tensor &top_words,
                               at::IntArrayRef level_sizes, const at::Tensor &lower_columns)
{
    PsigLogDesc desc = log_desc(sig, depth, d, true, top_words, level_sizes);
    TORCH_CHECK(lower_columns.dim() == 1 && lower_columns.scalar_type() == at::kLong, "lower_columns must be a 1D int64 tensor");
    TORCH_CHECK(lower_columns.is_cuda() && lower_columns.is_contiguous(), "lower_columns must be a contiguous CUDA tensor");
    same_device(sig, lower_columns, "lower_columns");
    desc.n_lower_columns = lower_columns.numel();
    // an empty list still selects the projected layout: any non-null pointer marks it
    static const int64_t kNoColumns = 0;
    desc.lower_columns = lower_columns.numel() > 0 ? lower_columns.data_ptr<int64_t>() : &kNoColumns;
    return desc;
}

at::Tensor logsig_projected(const at::Tensor &signature_in, int64_t depth, int64_t d, const at::Tensor &top_words,
                            at::IntArrayRef level_sizes, const at::Tensor &lower_columns)
{
    Range range("pathsig_b200::logsig_projected");
    TORCH_CHECK(signature_in.is_cuda(), "signature must be CUDA");
    c10::cuda::CUDAGuard guard(signature_in.device());
    at::Tensor sig = signature_in.contiguous();
    PsigLogDesc desc = projected_log_desc(sig, depth, d, top_words, level_sizes, lower_columns);
    const int64_t S = psig_logsig_size(&desc);
    check(S, "logsig_projected");
    TORCH_CHECK(S == sig.size(-1), "signature width ", sig.size(-1), " does not match the layout width ", S);
    const int64_t width = psig_logsig_out_size(&desc);
    check(width, "logsig_projected");
    at::Tensor out = at::empty(with_last(sig, width), sig.options());
    if (out.numel() == 0) return out;
    check(psig_logsig_forward(&desc, ptr(sig), out.data_ptr(), nullptr, stream_of(sig)), "logsig_projected");
    return out;
}

at::Tensor logsig_projected_backward(const at::Tensor &signature_in, const at::Tensor &grad_in, int64_t depth, int64_t d,
                                     const at::Tensor &top_words, at::IntArrayRef level_sizes, const at::Tensor &lower_columns)
{
    Range range("pathsig_b200::logsig_projected_backward");
    TORCH_CHECK(signature_in.is_cuda() && grad_in.is_cuda(), "signature and grad_out must be CUDA");
    TORCH_CHECK(grad_in.scalar_type() == signature_in.scalar_type(), "grad_out must have same dtype as signature");
    same_device(signature_in, grad_in, "grad_out");
    c10::cuda::CUDAGuard guard(signature_in.device());
    at::Tensor sig = signature_in.contiguous(), grad = grad_in.contiguous();
    PsigLogDesc desc = projected_log_desc(sig, depth, d, top_words, level_sizes, lower_columns);
    const int64_t width = psig_logsig_out_size(&desc);
    check(width, "logsig_projected_backward");
    TORCH_CHECK(grad.sizes().vec() == with_last(sig, width), "grad_out must be [B,(W),n_lower_columns + top_size]");
    at::Tensor grad_sig = at::empty_like(sig);
    if (grad_sig.numel() == 0) return grad_sig;
    check(psig_logsig_backward(&desc, ptr(sig), nullptr, ptr(grad), grad_sig.data_ptr(), nullptr, 0, stream_of(sig)),
          "logsig_projected_backward");
    return grad_sig;
}

PsigChenDesc chen_desc(const at::Tensor &a, const at::Tensor &b, int64_t depth, int64_t d)
{
    TORCH_CHECK(a.is_cuda() && b.is_cuda(), "signatures must be CUDA");
    TORCH_CHECK(depth >= 1 && depth <= PSIG_MAX_DEPTH, "depth must be in [1,12]");
    TORCH_CHECK(d >= 1, "d must be >= 1");
    TORCH_CHECK(a.scalar_type() == b.scalar_type(), "signatures must have the same dtype");
    same_device(a, b, "sig_b");
    TORCH_CHECK(a.sizes() == b.sizes() && a.dim() >= 1, "signatures must have the same shape (..., D)");
    const int64_t D = row_width(d, depth, false, {});
    TORCH_CHECK(a.size(-1) == D, "signature width ", a.size(-1), " is not the dense width ", D, " for d=", d, ", depth=", depth);
    PsigChenDesc desc{};
    desc.dtype = dtype_id(a);
    desc.d = (int32_t)d;
    desc.depth = (int32_t)depth;
    desc.rows = a.numel() / D;
    return desc;
}

at::Tensor chen_product(const at::Tensor &sig_a, const at::Tensor &sig_b, int64_t depth, int64_t d)
{
    Range range("pathsig_b200::chen_product");
    PsigChenDesc desc = chen_desc(sig_a, sig_b, depth, d);
    c10::cuda::CUDAGuard guard(sig_a.device());
    at::Tensor a = sig_a.contiguous(), b = sig_b.contiguous(), out = at::empty_like(a);
    if (out.numel() == 0) return out;
    check(psig_chen_forward(&desc, a.data_ptr(), b.data_ptr(), out.data_ptr(), stream_of(a)), "chen_product");
    return out;
}

std::tuple<at::Tensor, at::Tensor> chen_product_backward(const at::Tensor &sig_a, const at::Tensor &sig_b,
                                                         const at::Tensor &grad_out, int64_t depth, int64_t d)
{
    Range range("pathsig_b200::chen_product_backward");
    PsigChenDesc desc = chen_desc(sig_a, sig_b, depth, d);
    TORCH_CHECK(grad_out.is_cuda(), "grad_out must be CUDA");
    TORCH_CHECK(grad_out.scalar_type() == sig_a.scalar_type() && grad_out.sizes() == sig_a.sizes(),
                "grad_out must match the signatures in dtype and shape");
    same_device(sig_a, grad_out, "grad_out");
    c10::cuda::CUDAGuard guard(sig_a.device());
    at::Tensor a = sig_a.contiguous(), b = sig_b.contiguous(), g = grad_out.contiguous();
    at::Tensor ga = at::empty_like(a), gb = at::empty_like(a);
    if (ga.numel() == 0) return std::make_tuple(ga, gb);
    check(psig_chen_backward(&desc, a.data_ptr(), b.data_ptr(), g.data_ptr(), ga.data_ptr(), gb.data_ptr(), stream_of(a)),
          "chen_product_backward");
    return std::make_tuple(ga, gb);
}

}  // namespace

// Kernel family used by the signature operators (PsigAlgo); tests flip it to compare families.
extern "C" void psig_torch_set_algorithm(int algo) { g_algo.store(algo); }
extern "C" int psig_torch_get_algorithm(void) { return g_algo.load(); }

TORCH_LIBRARY(pathsig_b200, m)
{
    const auto tag = at::Tag::pt2_compliant_tag;
    m.set_python_module("pathsig_b200.ops");  // where the fake implementations and autograd formulas live
    m.def("compute_signature(Tensor path_in, int depth, bool alternative_projection, Tensor encoded_words, "
          "int[] level_sizes, bool use_windows, Tensor windows) -> Tensor", {tag});
    m.def("signature_backward(Tensor path_in, Tensor signature_in, Tensor grad_signature_in, int depth, "
          "bool alternative_projection, Tensor encoded_words, int[] level_sizes, bool use_windows, Tensor windows) -> Tensor", {tag});
    m.def("sig_to_logsig(Tensor signature_in, int depth, int d, bool alternative_projection, Tensor encoded_words, "
          "int[] level_sizes) -> (Tensor, Tensor)", {tag});
    m.def("logsig_backward(Tensor signature_in, Tensor P_in, Tensor grad_logsig_in, int depth, "
          "bool alternative_projection, Tensor encoded_words, int[] level_sizes) -> Tensor", {tag});
    m.def("logsig_projected(Tensor signature_in, int depth, int d, Tensor top_words, int[] level_sizes, "
          "Tensor lower_columns) -> Tensor", {tag});
    m.def("logsig_projected_backward(Tensor signature_in, Tensor grad_out, int depth, int d, Tensor top_words, "
          "int[] level_sizes, Tensor lower_columns) -> Tensor", {tag});
    m.def("chen_product(Tensor sig_a, Tensor sig_b, int depth, int d) -> Tensor", {tag});
    m.def("chen_product_backward(Tensor sig_a, Tensor sig_b, Tensor grad_out, int depth, int d) -> (Tensor, Tensor)", {tag});
}

TORCH_LIBRARY_IMPL(pathsig_b200, CUDA, m)
{
    m.impl("compute_signature", &compute_signature);
    m.impl("signature_backward", &signature_backward);
    m.impl("sig_to_logsig", &sig_to_logsig);
    m.impl("logsig_backward", &logsig_backward);
    m.impl("logsig_projected", &logsig_projected);
    m.impl("logsig_projected_backward", &logsig_projected_backward);
    m.impl("chen_product", &chen_product);
    m.impl("chen_product_backward", &chen_product_backward);
}
