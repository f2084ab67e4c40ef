/*
 * pathsig_b200 — C ABI of the B200 (sm_100a) signature / log-signature library.
 *
 * Plain pointers and sizes only: no C++ types, no torch types, no exceptions.  Every entry
 * point enqueues work on the given CUDA stream of the CURRENT device and returns without
 * synchronising.  Unless an entry point's comment says otherwise, nothing here allocates
 * device memory: outputs and scratch are supplied by the caller.  Return value: PSIG_OK (0)
 * or a negative PsigStatus; psig_status_string() gives the text.
 *
 * Each entry point replaces one operator of the reference (paths below are relative to the
 * reference project root):
 *   psig_sig_forward      <- pathsig::compute_signature   (src/pathsig/bindings.cpp:9-20,
 *                            launcher src/pathsig/forward/sig_launch.cu:75-225)
 *   psig_sig_backward     <- pathsig::signature_backward  (src/pathsig/bindings.cpp:23-36,
 *                            launcher src/pathsig/backward/sig_backward_launch.cu:83-303)
 *   psig_logsig_forward   <- pathsig::sig_to_logsig       (src/pathsig/bindings.cpp:39-49,
 *                            launcher src/pathsig/forward/sig_launch.cu:230-339)
 *   psig_logsig_backward  <- pathsig::logsig_backward     (src/pathsig/bindings.cpp:52-63,
 *                            launcher src/pathsig/backward/sig_backward_launch.cu:307-460)
 *
 * Data conventions (identical to the reference operators):
 *   path        (B, L, d) contiguous, float32 or float64, L >= 2
 *   windows     (W, 2) contiguous int32, half-open point ranges [start, end); a window with
 *               end - start < 2 yields zeros.  W == 0 / NULL: one unit per path, the whole path.
 *   signature   (B, D) or (B, W, D); degrees 1..depth concatenated; a dense degree k has d^k
 *               entries in lexicographic order, a projected degree keeps the caller's order.
 *   words       base-d codes (first letter most significant) of the NON-complete degrees,
 *               concatenated by degree, int64, device memory.
 *   level_sizes level_sizes[k] = number of words kept at degree k (entry 0 unused).  Ignored
 *               when `projected` is 0 (all degrees dense).
 */
#ifndef PATHSIG_B200_H
#define PATHSIG_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PSIG_MAX_DEPTH 12
#define PSIG_ABI_VERSION 2

typedef enum PsigStatus {
    PSIG_OK = 0,
    PSIG_ERR_NULL = -1,        /* a required pointer is NULL */
    PSIG_ERR_DTYPE = -2,       /* dtype is neither PSIG_F32 nor PSIG_F64 */
    PSIG_ERR_DEPTH = -3,       /* depth outside 1..12 */
    PSIG_ERR_SHAPE = -4,       /* B < 0, L < 2, d < 1, W < 0 or inconsistent level_sizes */
    PSIG_ERR_PACKING = -5,     /* d^depth does not fit a signed 64-bit word code */
    PSIG_ERR_WORKSPACE = -6,   /* workspace too small or NULL */
    PSIG_ERR_CUDA = -7,        /* a CUDA runtime call or launch failed (see cudaGetLastError) */
    PSIG_ERR_TOO_LARGE = -8,   /* a size exceeds what the entry point supports */
    PSIG_ERR_UNSUPPORTED = -9  /* configuration has no kernel */
} PsigStatus;

typedef enum PsigDtype { PSIG_F32 = 0, PSIG_F64 = 1 } PsigDtype;

/* Algorithm selection for psig_sig_forward / psig_sig_backward (desc.algo). */
typedef enum PsigAlgo {
    PSIG_ALGO_AUTO = 0,    /* register-tiled kernel when one exists for (dtype, d, depth); the prefix-closure
                              kernels for projected rows with enough work to repay their one-off
                              specialisation; else generic */
    PSIG_ALGO_GENERIC = 1, /* always the generic per-prefix kernel */
    PSIG_ALGO_TILED = 2,   /* register-tiled kernel or PSIG_ERR_UNSUPPORTED */
    PSIG_ALGO_CLOSURE = 3  /* prefix-closure kernels specialised for the word set, or PSIG_ERR_UNSUPPORTED */
} PsigAlgo;

/* PsigSigDesc.flags.  DETERMINISTIC: psig_sig_backward avoids floating-point atomics where a fixed-order
 * alternative exists -- today the register-tiled kernels on un-windowed paths whose unit spans several
 * blocks (d = 16): every block stores its share of the path gradient into its own slab of the workspace
 * and a second kernel sums the slabs in a fixed order (psig_sig_backward_workspace grows accordingly).
 * psig_sig_backward_reproducible tells whether the call selected by a description is bit-reproducible. */
#define PSIG_FLAG_DETERMINISTIC 1

/* Problem description shared by the signature entry points. */
typedef struct PsigSigDesc {
    int32_t dtype;                            /* PsigDtype */
    int32_t d;                                /* channels */
    int32_t depth;                            /* truncation depth, 1..12 */
    int32_t projected;                        /* 0: all degrees dense; 1: level_sizes / words in force */
    int64_t B;                                /* paths */
    int64_t L;                                /* points per path */
    int64_t W;                                /* windows; 0 = none */
    const int32_t *windows;                   /* device (W, 2) or NULL */
    const int64_t *words;                     /* device codes of non-complete degrees, or NULL */
    int64_t level_sizes[PSIG_MAX_DEPTH + 1];  /* host */
    int32_t algo;                             /* PsigAlgo */
    int32_t flags;                            /* PSIG_FLAG_* bits, 0 by default */
    const int64_t *words_host;                /* optional HOST copy of `words` (same layout).  The prefix-closure
                                                 kernels are generated from the word set, which has to be readable
                                                 on the host; NULL rules that family out for projected rows. */
} PsigSigDesc;

/* Problem description of the signature <-> log-signature entry points.  The signature is in
 * the hybrid layout: degrees below `depth` dense, the top degree dense (top_size == d^depth,
 * top_words NULL) or an explicit list of top_size words. */
typedef struct PsigLogDesc {
    int32_t dtype;
    int32_t d;
    int32_t depth;
    int32_t algo;               /* PsigAlgo: AUTO = row-in-shared-memory form of the kernels when the row fits,
                                   GENERIC = always the form streamed through global scratch (TILED is
                                   treated as AUTO) */
    int64_t rows;               /* B or B*W */
    int64_t top_size;           /* words kept at degree `depth` */
    const int64_t *top_words;   /* device codes of the top degree, or NULL when it is dense */
    /* Projected log-signature (row-in-shared-memory kernels only): the logarithm and the column selection
     * that follows it in the reference (src/pathsig/modules.py:134-135) as ONE kernel.  lower_columns
     * lists, in output order, the positions (in a dense row of the degrees below `depth`) of the words
     * kept below the top degree; the output row is those n_lower_columns values followed by the whole top
     * degree, and psig_logsig_backward takes the gradient in that same projected layout.  NULL / 0: every
     * position is kept (the layout of pathsig::sig_to_logsig). */
    const int64_t *lower_columns;   /* device, or NULL */
    int64_t n_lower_columns;
} PsigLogDesc;

int psig_abi_version(void);
/* Diagnostic with no counterpart in the reference: kernels this library has launched in this process
 * so far (all entry points, all threads).  A caller that wants to know how many kernels a step costs
 * reads it before and after the step. */
int64_t psig_kernel_launches(void);
/* Diagnostics of the bulk-copy (TMA) staging of the register-tiled forward kernel; no counterpart in the
 * reference.  A block waits for a staged chunk of points for a bounded number of polls; when the wait
 * runs out it reads the same bytes with plain loads (same result) and counts the event.
 * psig_bulk_copy_timeouts returns the count on the current device since the last call and clears it;
 * psig_set_bulk_wait_polls sets the bound on the current device (negative: the default, 2^20 polls;
 * 0: never wait, every staged chunk is read with plain loads) so that a test can make the wait run
 * out -- one poll is not enough for that, a poll may itself block for a short hardware-defined time.
 * Both synchronise the device; neither belongs in a hot loop. */
int64_t psig_bulk_copy_timeouts(void);
int psig_set_bulk_wait_polls(int polls);
/* Diagnostic, host only, no counterpart in the reference.  For a description whose top degree is a word
 * list over dense lower degrees (the LogSignature row layout) served by the register-tiled kernels, the
 * threads of a unit that own no listed word skip the arithmetic of the top target degree; the launcher
 * orders the unit's work items so that the skipping threads fill whole warps.  This call returns that
 * order for the forward (backward == 0) or the reverse sweep: items[s] = work item of thread slot s
 * (256 entries), *active = slots that run the top degree (a multiple of 32; at least the block size when
 * nothing is skipped, e.g. without desc->words_host).  Returns the block size, or PSIG_ERR_UNSUPPORTED
 * when the tiled kernels do not serve the description with a projected top degree. */
int psig_tiled_top_plan(const PsigSigDesc *desc, int backward, unsigned char *items, int *active);
const char *psig_status_string(int status);

/* Width D of one signature row for this description, or a negative PsigStatus. */
int64_t psig_sig_size(const PsigSigDesc *desc);
/* Width of one signature row in the hybrid layout of a PsigLogDesc, or a negative PsigStatus. */
int64_t psig_logsig_size(const PsigLogDesc *desc);
/* Width of one log-signature row: psig_logsig_size, or n_lower_columns + top_size when lower_columns is set. */
int64_t psig_logsig_out_size(const PsigLogDesc *desc);

/* out[(b*max(W,1)+w)*D + i] = signature coordinate i of path b over window w.
 * Replaces pathsig::compute_signature (src/pathsig/forward/sig_launch.cu:75-225). */
int psig_sig_forward(const PsigSigDesc *desc, const void *path, void *out, void *stream);

/* Scratch bytes psig_sig_backward needs for this description: 0 for the register-tiled kernels,
 * sizeof(scalar)*B*(L-1)*d for the generic and the prefix-closure ones.  May build the specialised
 * kernels of a projected description on first use (seconds, once per word set and device). */
int64_t psig_sig_backward_workspace(const PsigSigDesc *desc);

/* grad_path (B, L, d) = d/dpath of sum(signature * grad_sig).  `sig` is the forward output for
 * the same description.  Contributions of overlapping windows are summed.  `workspace` must hold
 * psig_sig_backward_workspace(desc) bytes, 256-byte aligned; its contents are overwritten.
 * Replaces pathsig::signature_backward (src/pathsig/backward/sig_backward_launch.cu:83-303). */
int psig_sig_backward(const PsigSigDesc *desc, const void *path, const void *sig, const void *grad_sig,
                      void *grad_path, void *workspace, int64_t workspace_bytes, void *stream);
/* Host only, no counterpart in the reference (whose backward always adds with float atomics,
 * src/pathsig/backward/sig_backward_kernels.cu:317): 1 when psig_sig_backward gives the same bits on every
 * run for this description (register-tiled kernels, no windows, and either one block per unit or
 * PSIG_FLAG_DETERMINISTIC), 0 when some sums are float atomics, negative PsigStatus on a bad description. */
int psig_sig_backward_reproducible(const PsigSigDesc *desc);

/* Scalars per row of the cache argument of psig_logsig_forward / psig_logsig_backward: 0 when the row
 * fits the row-in-shared-memory form of the kernels; S*depth -- the shape of the reference's table of
 * powers P_m, so that operator signatures stay the same -- when the row is streamed through global
 * memory, where the forward pass uses part of it as scratch (the backward pass reads nothing from it
 * and recomputes what it needs in its own workspace).  Host-only; depends on the description alone. */
int64_t psig_logsig_cache_size(const PsigLogDesc *desc);

/* logsig (rows, S) = word coordinates of the truncated tensor logarithm of `sig` (rows, S);
 * cache (rows, psig_logsig_cache_size(desc)) receives what psig_logsig_backward reads back (may be
 * NULL when that size is 0).  Forward and backward of one call must use the same desc.algo.
 * Replaces pathsig::sig_to_logsig (src/pathsig/forward/sig_launch.cu:230-339). */
int psig_logsig_forward(const PsigLogDesc *desc, const void *sig, void *logsig, void *cache, void *stream);

/* Scratch bytes psig_logsig_backward needs: 0 for the row-in-shared-memory form; for the streamed form
 * rows * (4 * lower + sum_k |T_k|) scalars, lower = the dense degrees below the top, T_k = degrees
 * 1..depth-k.  PSIG_ERR_TOO_LARGE for rows of 2^31 scalars or more. */
int64_t psig_logsig_backward_workspace(const PsigLogDesc *desc);

/* grad_sig (rows, S) = adjoint of psig_logsig_forward applied to grad_logsig.
 * Replaces pathsig::logsig_backward (src/pathsig/backward/sig_backward_launch.cu:307-460). */
int psig_logsig_backward(const PsigLogDesc *desc, const void *sig, const void *cache, const void *grad_logsig,
                         void *grad_sig, void *workspace, int64_t workspace_bytes, void *stream);

/* Prefix-closure kernels (no counterpart in the reference, whose threads each recompute the private
 * prefix chain of one word, src/pathsig/forward/sig_kernels.cu:99-113): diagnostics of the code
 * generator.  psig_closure_source writes the CUDA C++ generated for the row layout of `desc` (which must
 * carry words_host for listed degrees) cut into about `target_bins` bins, NUL-terminated, into `buffer`
 * (up to `capacity` bytes) and returns its full length, or a negative PsigStatus.  stats (5 entries, may
 * be NULL): closure nodes, algorithmic forward FMAs per path*step, FMAs the generated forward code
 * executes per path*step (bins recompute the ancestors of their first node), bins, node values per lane.
 * psig_closure_compile compiles such a source with NVRTC for `arch` (e.g. "sm_100a") without touching a
 * device; the compiler's log goes to `log`.  Neither call launches anything. */
int64_t psig_closure_source(const PsigSigDesc *desc, int target_bins, char *buffer, int64_t capacity, int64_t *stats);
int psig_closure_compile(const char *source, const char *arch, char *log, int64_t log_capacity);
/* 1 when the run-time compiler (libnvrtc.so.12) the prefix-closure kernels need can be loaded, else 0.  Host only. */
int psig_closure_available(void);

/* No counterpart in the reference.  Same result as psig_sig_backward computed by the generic
 * kernel, for callers that have no scratch memory to pass and may not allocate any: hosts whose
 * device memory is entirely owned by a pre-sized arena, enqueue-style hooks that are forbidden
 * to allocate, loops that cannot take the device-wide synchronisation of cudaMalloc/cudaFree.
 * The B*(L-1)*d-scalar accumulator the kernel needs is a fixed array inside the library; this
 * call allocates nothing (no cudaMalloc, no cudaFree, no allocating library routine).
 *   Limit: sizeof(scalar)*B*(L-1)*d <= psig_sig_backward_static_limit() (8 MiB); larger problems
 *   return PSIG_ERR_TOO_LARGE and must use psig_sig_backward.
 *   Every device that loads the library holds those 8 MiB until the process exits.
 *   The first call on each device looks up the array's device address (with that device
 *   current) and may make the CUDA runtime load the library's kernels onto the device; make it
 *   once as a warm-up, before starting any stream capture and before the phase in which
 *   allocations are forbidden.
 *   All calls on a device share the one array: the needed part is cleared on the stream before
 *   each use, and two calls whose GPU work overlaps (different streams, or different threads)
 *   would corrupt each other -- issue them on one stream or order them with events. */
int psig_sig_backward_static(const PsigSigDesc *desc, const void *path, const void *sig, const void *grad_sig,
                             void *grad_path, void *stream);
int64_t psig_sig_backward_static_limit(void);

/* Chen product of truncated signatures; no counterpart in the reference, which always recomputes
 * a signature from the increments (src/pathsig/forward/sig_kernels.cu:116-157).  Rows hold degrees
 * 1..depth, all dense, in the layout of psig_sig_forward; the degree-0 coordinate (1) is implied:
 *   out(w) = a(w) + b(w) + sum_{0<k<|w|} a(w[:k]) * b(w[k:])
 * so out is the signature of path A followed by path B (translated to start where A ends). */
typedef struct PsigChenDesc {
    int32_t dtype;   /* PsigDtype */
    int32_t d;       /* channels */
    int32_t depth;   /* 1..12 */
    int32_t reserved;
    int64_t rows;    /* signature rows in a, b and out */
} PsigChenDesc;

/* Width of one row (sum of d^k, k = 1..depth), or a negative PsigStatus. */
int64_t psig_chen_size(const PsigChenDesc *desc);
/* out (rows, D) = a (x) b, row by row.  `out` must not alias a or b. */
int psig_chen_forward(const PsigChenDesc *desc, const void *a, const void *b, void *out, void *stream);
/* grad_a, grad_b (rows, D) = adjoint of psig_chen_forward applied to grad_out.  Needs no scratch and
 * uses no atomics: results are bit-reproducible from run to run. */
int psig_chen_backward(const PsigChenDesc *desc, const void *a, const void *b, const void *grad_out,
                       void *grad_a, void *grad_b, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* PATHSIG_B200_H */
