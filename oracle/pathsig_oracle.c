/*
 * pathsig CPU oracle: a plain-C restatement of the reference's signature, signature-backward,
 * signature->log-signature and log-signature-backward algorithms in float32 and float64.
 *
 * TEST INFRASTRUCTURE ONLY.  It exists to check the CUDA library and to serve as the timed
 * CPU baseline (the reference has no CPU implementation of its own: both of its
 * TORCH_LIBRARY_IMPL blocks register for the CUDA key only,
 * src/pathsig/forward/sig_launch.cu:345-348, src/pathsig/backward/sig_backward_launch.cu:468-471).
 * Nothing in the shipped package may call into this file.
 *
 * Parity pin: the float64 routines are checked against outputs of the reference's own CUDA
 * build recorded on a B200 (tests/golden/), and against closed-form identities
 * (tests/test_oracle.py).
 *
 * Build: see oracle/Makefile (gcc -O2 -fopenmp -ffp-contract=off -shared -fPIC).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_MAX_DEPTH 12

typedef struct {
    int64_t size[ORACLE_MAX_DEPTH + 1];         /* words kept at each degree */
    int64_t offset[ORACLE_MAX_DEPTH + 1];       /* start of the degree inside one output row */
    const int64_t *words[ORACLE_MAX_DEPTH + 1]; /* base-d codes, or NULL when the degree is dense */
    int64_t total;
} oracle_levels;

/* Level bookkeeping of the launchers.
 * top_only == 0 (signature ops): src/pathsig/forward/sig_launch.cu:123-135,167-182 — explicit
 *   codes are stored for non-full levels only, concatenated in level order.
 * top_only == 1 (log ops): src/pathsig/forward/sig_launch.cu:300-315 — levels below depth are
 *   dense, the top level alone may be an explicit list.
 * level_sizes == NULL means every level is dense. */
static int oracle_make_levels(int d, int depth, const int64_t *encoded_words, const int64_t *level_sizes,
                              int top_only, oracle_levels *lv)
{
    if (depth < 1 || depth > ORACLE_MAX_DEPTH || d < 1) return -1;
    int64_t d_pow = 1, off = 0, enc_off = 0;
    memset(lv, 0, sizeof(*lv));
    for (int k = 1; k <= depth; ++k) {
        d_pow *= d;
        int64_t size = d_pow;
        const int64_t *words = NULL;
        const int projected = level_sizes && (!top_only || k == depth);
        if (projected) {
            size = level_sizes[k];
            if (size != d_pow) {
                if (!encoded_words && size > 0) return -1;
                words = encoded_words ? encoded_words + enc_off : NULL;
                enc_off += size;
            }
        }
        lv->size[k] = size;
        lv->offset[k] = off;
        lv->words[k] = (size != d_pow) ? words : NULL;
        off += size;
    }
    lv->total = off;
    return 0;
}

/* Base-d code -> letters, first letter most significant
 * (src/pathsig/utils/word_mappings.cuh:17-28, src/pathsig/projections.py:99-105). */
static void oracle_unpack(int64_t code, int k, int d, int *letters)
{
    for (int pos = k - 1; pos >= 0; --pos) {
        letters[pos] = (int)(code % d);
        code /= d;
    }
}

int64_t oracle_sig_size(int d, int depth, const int64_t *level_sizes, int top_only)
{
    oracle_levels lv;
    if (oracle_make_levels(d, depth, NULL, NULL, top_only, &lv)) return -1;
    if (!level_sizes) return lv.total;
    int64_t total = 0, d_pow = 1;
    for (int k = 1; k <= depth; ++k) {
        d_pow *= d;
        total += (!top_only || k == depth) ? level_sizes[k] : d_pow;
    }
    return total;
}

#define REAL float
#define SUFFIX _f32
#include "oracle_impl.inc"
#undef REAL
#undef SUFFIX

#define REAL double
#define SUFFIX _f64
#include "oracle_impl.inc"
#undef REAL
#undef SUFFIX
