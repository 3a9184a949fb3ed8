/*
 * barqkv - experiment knobs.  NOT part of the serving ABI.
 *
 * libbarqkv.so as built by default does not export barqkv_set_tuning and keeps no mutable
 * process-wide settings.  A library compiled with -DBARQKV_TUNING (barqtrain_b200/_build.py,
 * build_native(tuning=True) -> lib/libbarqkv_tuning.so) adds the function below so that kernel
 * parameters can be swept from one process.  The knobs are process-wide and not thread-safe.
 * No counterpart in the reference, which has no tunables.
 */
#ifndef BARQKV_EXPERIMENTAL_H
#define BARQKV_EXPERIMENTAL_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* value 0 restores the default unless stated otherwise */
#define BARQKV_KNOB_BULK_STAGES 1        /* ring stages of the bulk gather (3..32) */
#define BARQKV_KNOB_BULK_CTAS_PER_SM 2   /* persistent one-warp CTAs per SM of the bulk gather */
#define BARQKV_KNOB_VECTOR_CTAS_PER_SM 3 /* CTAs per SM of the vector gather */
#define BARQKV_KNOB_INTERLEAVE 4         /* static shares only. 1: every gridDim-th group of 32 pages; 0: contiguous */
#define BARQKV_KNOB_GROUP_TILES 5        /* pages handed out per atomic fetch by the bulk gather (1..32) */
#define BARQKV_KNOB_STATIC_SHARES 6      /* 1: ignore `work` and split pages statically among CTAs */
#define BARQKV_KNOB_PDL 7                /* 0: never launch with programmatic stream serialization (-1 = default: where allowed) */
#define BARQKV_KNOB_STATIC_PERMILLE 8    /* thousandths of the pages split evenly among CTAs before the atomic hand-out (-1 = default) */
#define BARQKV_KNOB_TENSOR_STORE 9       /* 0: token-major outputs use row copies only (-1 = default: tiled TMA store per full page) */
#define BARQKV_KNOB_ATTN_L2_PROMOTION 10 /* decode attention: L2 promotion of the page loads. 0 none, 1 128 B, 2 256 B (-1 = default) */
#define BARQKV_KNOB_ATTN_SPLIT_TOKENS 11 /* decode attention: tokens per split before adapting to the batch (0 = default 512) */
#define BARQKV_KNOB_APPEND_BULK 12       /* 0: appends always use the row kernel (-1 = default: copy engine for page-sized appends) */
#define BARQKV_KNOB_ATTN_WIDE 13         /* decode attention updates its softmax state every 32 tokens (1) or 16 (0); -1 = default: 32 for pages of 32 / 64 */
#define BARQKV_KNOB_LAYER_OVERLAP 14     /* 0: barqkv_update_layers keeps every layer on the caller's stream (default 1: odd layers on a second stream) */
#define BARQKV_KNOB_ATTN_PAGE_BOX 15     /* decode attention, pages per copy instruction. 0: half of K or V; 1: K or V; 2 (default): K and V where the pools allow it */
#define BARQKV_KNOB_ATTN_COMPACT 16      /* 0: decode attention launches one CTA per possible split of every sequence (default 1: only splits that can have pages, batches of up to 256) */
#define BARQKV_KNOB_ATTN_PROBE 17        /* timing probes, results are wrong. 1: decode attention loads pages but does not attend them; 2: writes no result; 3: both */
#define BARQKV_KNOB_ZERO_AHEAD 18         /* 0: every launch of barqkv_update_layers counts its finished CTAs and clears its own counter pair (default 1: a launch clears the pair of its neighbours in the chain) */

int barqkv_set_tuning(int32_t knob, int32_t value);

#ifdef __cplusplus
}
#endif
#endif /* BARQKV_EXPERIMENTAL_H */
