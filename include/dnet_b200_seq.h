/*
 * dnet_b200_seq.h -- C ABI of libdnet_b200_seq.so: the batched step of decoder models whose layers are a
 * sequence mixer (softmax attention over a paged cache -- block-masked or sliding-window, the window optionally followed
 * by mean-pooled blocks of older tokens, capped, with a sink and head gates --, latent attention that caches one
 * compressed row per token, a gated delta-rule recurrence, a generalized delta rule with a decay and a removal rate per
 * key channel, decayed outer-product recurrences, or attention beside one of those) plus an optional dense, gated or
 * routed feed-forward, tied together by S residual streams; a span of layers may run several times on the same weights;
 * every sublayer's input may pass a short causal convolution first, and the embedding may add a hashed bigram row.
 *
 * Same conventions as dnet_b200.h: plain C, opaque handles, 0 or a negative DN_E* code, dn_seq_last_error() for
 * the text, caller-owned streams and buffers, weights BORROWED by pointer.  One handle serves one compute thread.
 *
 * A model holds a pool of 64-token cache pages and `max_seqs` state slots.  A sequence is opened into a slot, fed
 * by dn_seq_step in portions of any size next to other sequences, and closed; its pages and slot are then reused.
 */
#ifndef DNET_B200_SEQ_H
#define DNET_B200_SEQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DN_SEQ_BF16 0
#define DN_SEQ_F32 1

#define DN_MIX_ATTENTION 0
#define DN_MIX_DELTA 1
#define DN_MIX_PARALLEL 2   /* softmax attention and a gated linear attention side by side on the same input */
#define DN_MIX_WKV 3        /* token-shift mixing + a decayed outer-product state read with a bonus for the current token */
#define DN_MIX_LATENT 4     /* latent attention: keys and values are up-projections of one cached latent row per token */

#define DN_MASK_BLOCK 0     /* a query sees its own block of `chunk` positions, causally */
#define DN_MASK_WINDOW 1    /* a query sees itself and the `chunk` - 1 positions before it */

#define DN_ROT_INTERLEAVED 0   /* rotary pairs (2i, 2i + 1) */
#define DN_ROT_HALF 1          /* rotary pairs (i, i + dims / 2) */

#define DN_NORM_RMS 0       /* x / sqrt(mean(x^2) + eps) * w  (or 1 + w) */
#define DN_NORM_DYT 1       /* tanh(alpha x) * w + b, elementwise */
#define DN_NORM_LAYER 2     /* (x - mean) / sqrt(variance + eps) * w + b */

#define DN_QKNORM_NONE 0
#define DN_QKNORM_WHOLE 1   /* RMS norm over the whole q (k) projection, weight [heads dim] */
#define DN_QKNORM_HEAD 2    /* RMS norm over each head's dim, one weight [dim] for all heads */

#define DN_RIGHT_GLA 0      /* right half of DN_MIX_PARALLEL: gated linear attention, M <- diag(d) M + k v^T */
#define DN_RIGHT_GDELTA 1   /* generalized delta rule: S <- diag(w) S - (a u)(u^T S) + k v^T with u = k / |k|, read after the update */

#define DN_MLP_DENSE 0      /* gelu_tanh(gate) * up -> down, or (ff_act) an ungated activation between up and down */
#define DN_MLP_MOE 1        /* routed GLU experts (+ an optional shared one) */

#define DN_FF_GEGLU 0       /* dense feed-forward: gelu_tanh(W_gate h) * (W_up h) */
#define DN_FF_RELU2 1       /* dense feed-forward: relu(W_up h + b)^2, no gate; up and down may carry biases */

#define DN_ROUTER_TOPK 0    /* the `top` largest logits choose; softmax over the chosen logits weighs */
#define DN_ROUTER_SCORED 1  /* softmax over all experts scores; a correction is added for the choice only; experts form groups of
                               which the best are kept; weights = chosen scores / their sum * router_scale */

#define DN_EXPERT_CGLU 0    /* clamped GLU: g = min(gate, limit), u = clamp(up, +-limit), g sigmoid(1.702 g) (u + 1) */
#define DN_EXPERT_SWIGLU 1  /* silu(gate) * up */

typedef struct dn_seq_model dn_seq_model;
typedef void* dn_seq_stream;   /* cudaStream_t */

typedef struct dn_seq_layer_cfg {
  int32_t mixer;       /* DN_MIX_* */
  int32_t heads;       /* query heads (attention) / value heads (delta) */
  int32_t kv_heads;    /* key/value heads (attention) / query-key heads (delta) */
  int32_t dim;         /* per-head query/key size */
  int32_t vdim;        /* per-head value size */
  int32_t conv;        /* taps of the short causal convolution on q, k, v (0: none) */
  int32_t chunk;       /* attention: a query sees its own block of this many positions (0: plain causal) */
  int32_t rot_dims;    /* attention: rotated dims per head (0: none) */
  float rot_base;
  float scale;         /* attention: score scale */
  int32_t kv_from;     /* attention: layer whose pages hold this layer's keys and values (-1: its own) */
  int32_t ff;          /* feed-forward width, of one expert for DN_MLP_MOE (0: the layer has no feed-forward) */
  /* attention (also the attention half of DN_MIX_PARALLEL) */
  int32_t qk_norm;     /* DN_QKNORM_*: RMS norm of q and k with learned weights, before rotation */
  float softcap;       /* scores: cap * tanh(score / cap) after the scale (0: none) */
  int32_t sink;        /* 1: the softmax denominator holds one more term exp(sink_h), a learned number per head */
  int32_t out_gate;    /* 1: head h's output is multiplied by sigmoid(w_h . x), one gate per head */
  /* the linear-attention half of DN_MIX_PARALLEL; DN_MIX_WKV uses heads / dim / vdim above and rank here */
  int32_t r_heads, r_dim, r_vdim;
  int32_t rank;        /* inner size of the two-step decay projection */
  float tau;           /* DN_MIX_PARALLEL: decay = sigmoid(z)^(1/tau) */
  float left_scale, right_scale;   /* DN_MIX_PARALLEL: result = left_scale * attention + right_scale * linear attention */
  /* feed-forward */
  int32_t mlp_kind;    /* DN_MLP_* */
  int32_t experts, top;
  float limit;         /* clamped GLU: gate <= limit, |up| <= limit */
  int32_t shared_ff;   /* width of the shared expert (0: none) */
  float shared_limit;
  /* attention */
  int32_t mask_kind;   /* DN_MASK_*: what `chunk` means */
  int32_t rot_layout;  /* DN_ROT_* */
  /* DN_MIX_LATENT: per head `dim` unrotated and `rot_part` rotated query / key dims (of which the first rot_dims turn),
   * values of vdim; the cache holds kv_rank + rot_part numbers a token.  q_rank > 0: queries go through a normed latent too */
  int32_t kv_rank, q_rank, rot_part;
  /* feed-forward */
  int32_t ff_act;      /* DN_FF_*: dense feed-forward */
  int32_t router_kind; /* DN_ROUTER_* */
  int32_t expert_act;  /* DN_EXPERT_*: routed and shared experts */
  int32_t identity;    /* DN_ROUTER_SCORED: the router's last `identity` outputs stand for experts that return their input */
  int32_t groups, groups_keep;   /* DN_ROUTER_SCORED: experts (identity ones included) in `groups` equal runs, the best kept (0: no groups) */
  float router_scale;
  int32_t shared_gate; /* 1: the shared expert's output is multiplied by sigmoid(w . h), one number a token */
  /* attention */
  int32_t v_is_k;      /* 1: the values are the keys as projected (vdim = dim, no value projection, one pool) */
  float qtemp_coef;    /* queries at position p are multiplied by 1 + qtemp_coef ln(floor((p + 1) / qtemp_every) + 1) (qtemp_every 0: no) */
  int32_t qtemp_every;
  int32_t pool;        /* DN_MASK_WINDOW: beside the window's tokens a query sees one mean key / value for each block of `pool` tokens
                          that lies wholly before the window (0: none) */
  /* rotary frequencies scaled by interpolation between f / factor (slow dims) and f (fast dims); cos and sin times
   * 0.1 ln(factor) + 1.  yarn_factor 0: plain frequencies */
  float yarn_factor, yarn_original, yarn_fast, yarn_slow;
  /* DN_MIX_PARALLEL */
  int32_t r_kind;      /* DN_RIGHT_* */
  int32_t branch_norm; /* 1: each half's output is RMS-normed over the width (weights DN_SQ_L_OUT / DN_SQ_R_OUT) before the scaled sum */
} dn_seq_layer_cfg;

typedef struct dn_seq_cfg {
  int32_t width, vocab, n_layers;
  int32_t streams;           /* residual streams (0: plain residual) */
  int32_t dtype;             /* DN_SEQ_BF16: bf16 storage, fp32 sums;  DN_SEQ_F32: everything fp32 */
  float eps;                 /* of every RMS norm */
  float embed_scale;
  int32_t pool_pages;        /* 64-token pages in the cache pool */
  int32_t max_seqs;          /* state slots */
  int32_t max_batch_tokens;  /* most tokens one dn_seq_step may bring */
  int32_t norm_kind;         /* DN_NORM_*: of every norm that spans the width */
  int32_t post_norm;         /* 1: a sublayer's output is normed again before it joins the residual */
  int32_t embed_norm;        /* 1: the embedding is normed */
  float logit_softcap;       /* logits: cap * tanh(logit / cap) (0: none) */
  /* layers loop_start .. loop_stop-1 run loop_times times in a row on the same weights, every pass with its own cache and
   * state; before the first layer of each pass x <- W_in [x; x0] with x0 the embedding's output.  loop_times = 0: no loop */
  int32_t loop_start, loop_stop, loop_times;
  int32_t no_pre_norm;       /* 1: sublayers read the residual itself; only their outputs are normed (post_norm) */
  /* every sublayer's input h becomes h + conv(h), a causal depthwise convolution over time of canon_taps taps whose last
   * canon_taps - 1 inputs are carried per sequence, layer run and sublayer (0: none) */
  int32_t canon_taps;
  /* the embedding adds row (previous token * mul_prev + token * mul_cur) mod buckets of DN_SQ_BIGRAM, row `buckets` for a
   * sequence's first token; the previous token is carried per sequence (buckets 0: none) */
  int32_t bigram_buckets, bigram_mul_prev, bigram_mul_cur;
  float logit_scale;         /* logits are multiplied by this (0: by 1) */
} dn_seq_cfg;

/* tensors of a layer (dn_seq_bind: layer >= 0) and of the model (layer = -1) */
enum {
  DN_SQ_NORM1 = 0, DN_SQ_NORM2,
  DN_SQ_Q, DN_SQ_K, DN_SQ_V, DN_SQ_O, DN_SQ_Q_CONV, DN_SQ_K_CONV, DN_SQ_V_CONV, DN_SQ_Q_NORM, DN_SQ_K_NORM,
  DN_SQ_A, DN_SQ_B, DN_SQ_G, DN_SQ_A_LOG, DN_SQ_DT_BIAS, DN_SQ_OUT_NORM,
  DN_SQ_GATE, DN_SQ_UP, DN_SQ_DOWN,
  DN_SQ_HC1_IN, DN_SQ_HC1_OUT, DN_SQ_HC1_MIX, DN_SQ_HC2_IN, DN_SQ_HC2_OUT, DN_SQ_HC2_MIX,
  /* DN_NORM_DYT: bias and scalar alpha of the norms; the norms after a sublayer (post_norm) */
  DN_SQ_NORM1_B, DN_SQ_NORM1_ALPHA, DN_SQ_NORM2_B, DN_SQ_NORM2_ALPHA,
  DN_SQ_POST1, DN_SQ_POST1_B, DN_SQ_POST1_ALPHA, DN_SQ_POST2, DN_SQ_POST2_B, DN_SQ_POST2_ALPHA,
  /* attention extras: per-head sink [H], per-head output gate [H, W] */
  DN_SQ_SINK, DN_SQ_HEAD_GATE,
  /* linear-attention half of DN_MIX_PARALLEL */
  DN_SQ_R_Q, DN_SQ_R_K, DN_SQ_R_V, DN_SQ_R_G, DN_SQ_R_O, DN_SQ_R_NORM,
  /* two-step decay projection [rank, W], [C, rank] and its bias [C] (DN_MIX_PARALLEL's right half, DN_MIX_WKV) */
  DN_SQ_DECAY1, DN_SQ_DECAY2, DN_SQ_DECAY_B,
  /* DN_MIX_WKV: token-shift coefficients of r, k, v, g, w [W] each; the current token's bonus [H, dk] */
  DN_SQ_MU_R, DN_SQ_MU_K, DN_SQ_MU_V, DN_SQ_MU_G, DN_SQ_MU_W, DN_SQ_BONUS,
  /* DN_MLP_MOE: router [E, W] and its bias [E]; the shared expert */
  DN_SQ_ROUTER, DN_SQ_ROUTER_B, DN_SQ_SH_GATE, DN_SQ_SH_UP, DN_SQ_SH_DOWN,
  /* DN_MIX_LATENT: query latent [q_rank, W] and its norm [q_rank] (DN_SQ_Q is then [H (dim + rot_part), q_rank]); key/value
   * latent [kv_rank + rot_part, W] and its norm [kv_rank]; up-projections to keys [H dim, kv_rank] and values [H vdim, kv_rank] */
  DN_SQ_DQ, DN_SQ_DQ_NORM, DN_SQ_DKV, DN_SQ_DKV_NORM, DN_SQ_UK, DN_SQ_UV,
  /* biases of a dense feed-forward [ff], [W]; DN_ROUTER_SCORED: correction [experts + identity]; the shared expert's gate [W] */
  DN_SQ_UP_B, DN_SQ_DOWN_B, DN_SQ_ROUTER_CORR, DN_SQ_SH_SG,
  /* the sublayers' input convolutions [W, canon_taps]; the norms of a parallel mixer's two outputs [W] (branch_norm);
   * DN_RIGHT_GDELTA: the removal rate's projection [C, W] and bias [C] (DN_SQ_R_Q is the read vector's projection,
   * DN_SQ_DECAY1 / 2 / _B the decay's, DN_SQ_R_NORM [C] one weight per channel) */
  DN_SQ_CANON1, DN_SQ_CANON2, DN_SQ_L_OUT, DN_SQ_R_OUT, DN_SQ_R_A, DN_SQ_R_AB,
  DN_SQ_COUNT,
  DN_SQ_EMBED = 100, DN_SQ_FINAL_NORM, DN_SQ_HEAD, DN_SQ_FINAL_NORM_B, DN_SQ_FINAL_NORM_ALPHA,
  DN_SQ_EMBED_NORM, DN_SQ_EMBED_NORM_B, DN_SQ_EMBED_NORM_ALPHA, DN_SQ_LOOP_IN, DN_SQ_BIGRAM
};
/* matrices of a routed expert (dn_seq_bind_expert) */
enum { DN_SQ_E_GATE = 0, DN_SQ_E_UP, DN_SQ_E_DOWN };

int dn_seq_init(int device);
const char* dn_seq_last_error(void);
int64_t dn_seq_launch_count(void);

int dn_seq_model_create(const dn_seq_cfg* cfg, const dn_seq_layer_cfg* layers, dn_seq_model** out);
int dn_seq_model_destroy(dn_seq_model* m);
int dn_seq_bind(dn_seq_model* m, int layer, int which, const void* dev_ptr);
int dn_seq_bind_expert(dn_seq_model* m, int layer, int expert, int which, const void* dev_ptr);
/* layer runs of a step: n_layers plus the repeated passes of the loop (rows of dn_seq_step's layer trace) */
int dn_seq_layer_runs(dn_seq_model* m);

/* sequences: open takes a free state slot (zeroed behind the work queued on s); close returns slot and pages */
int dn_seq_open(dn_seq_model* m, dn_seq_stream s, int* slot_out);
int dn_seq_close(dn_seq_model* m, int slot);
int dn_seq_length(dn_seq_model* m, int slot);
int dn_seq_free_pages(dn_seq_model* m);
int dn_seq_free_slots(dn_seq_model* m);

/* One step: entry e brings counts[e] tokens (concatenated in tokens_host) of the sequence in slots[e]; the rows
 * want_host[0..n_want) of the concatenation get logits, written as fp32 [n_want, vocab] to logits_dev.
 * layer_trace_dev (optional): fp32 [layer runs, N, width], the residual (sum of the streams) after every layer run.
 * Asynchronous on s except for the staging of the previous step's arguments. */
int dn_seq_step(dn_seq_model* m, int n_entries, const int32_t* slots, const int32_t* counts, const int32_t* tokens_host,
                int n_want, const int32_t* want_host, float* logits_dev, float* layer_trace_dev, dn_seq_stream s);

/* Synchronises s and reports whether a bounded in-kernel wait ever ran out (negative code; the model's results are
 * then invalid).  Callers ask before they trust logits they have read. */
int dn_seq_check(dn_seq_model* m, dn_seq_stream s);

/* Phase profiler (off by default).  While on, every step records an event at each phase boundary; read adds the
 * elapsed milliseconds of all steps since the last read to per-phase totals and copies them to ms_out
 * [DN_SEQ_PH_COUNT] (reset != 0 zeroes the totals afterwards).  Synchronises the device. */
enum {
  DN_SEQ_PH_EMBED = 0, DN_SEQ_PH_NORM, DN_SEQ_PH_PROJ, DN_SEQ_PH_ATTN_PREP, DN_SEQ_PH_ATTN, DN_SEQ_PH_DELTA_PREP,
  DN_SEQ_PH_DELTA_RULE, DN_SEQ_PH_DELTA_OUT, DN_SEQ_PH_CARRY, DN_SEQ_PH_OUT_PROJ, DN_SEQ_PH_WRITE_BACK, DN_SEQ_PH_FF_UP,
  DN_SEQ_PH_FF_DOWN, DN_SEQ_PH_HEAD, DN_SEQ_PH_OTHER, DN_SEQ_PH_RECUR_PREP, DN_SEQ_PH_RECUR, DN_SEQ_PH_RECUR_OUT, DN_SEQ_PH_ROUTER,
  DN_SEQ_PH_MOE_UP, DN_SEQ_PH_MOE_DOWN,
  DN_SEQ_PH_LATENT_IN,    /* latent attention: the cached row, rotary, queries absorbed into the latent space */
  DN_SEQ_PH_LATENT_OUT,   /* latent attention: the heads' outputs taken out of the latent space */
  DN_SEQ_PH_CANON,        /* the sublayers' input convolutions and their carried rows */
  DN_SEQ_PH_COUNT
};
int dn_seq_profile(dn_seq_model* m, int on);
int dn_seq_profile_read(dn_seq_model* m, double* ms_out, int reset);

/* Decode steps (every entry brings one token, at most 8 entries) replay a CUDA graph captured at the first step of
 * each (entries, wanted rows) shape; on by default.  Off: every kernel is launched one by one (same kernels, same
 * results).  The profiler and the layer trace always take the one-by-one path. */
int dn_seq_set_graphs(dn_seq_model* m, int on);

#ifdef __cplusplus
}
#endif
#endif
