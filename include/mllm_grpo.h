/*
 * mllm_grpo.h -- C ABI of the B200 (sm_100a) fused GRPO / PPO-clip token loss.
 *
 * The library replaces one region of demon2036/MLLM-JAX: the token-level loss
 * computed from logits inside TrainGRPOModule.__call__
 * (MLLM_JAX/train_modules/__init__.py:118-180) and its gradient with respect
 * to the logits (jax.value_and_grad at plugins/training/update/train_step.py:24).
 * The policy part of PPOActorCriticModule.__call__
 * (plugins/training/ppo/module.py:66-102) is the same operator with per-token
 * advantages.  The reference has no FFI for this path (it is plain jax.numpy);
 * these entry points are what an XLA FFI handler / ctypes stub binds instead.
 *
 * Conventions
 *   - Every pointer in mllm_grpo_args is a DEVICE pointer owned by the caller.
 *     The library allocates nothing (except where an entry point says so),
 *     never synchronises the host, and enqueues all work on the caller's
 *     stream (`stream` is a cudaStream_t passed as void*).
 *   - Every entry point returns an mllm_grpo_status (0 = ok).  Nothing throws.
 *   - Geometry: logits hold n_seqs sequences of seq_rows rows each, row r of
 *     sequence b starts at element (b*seq_rows + r)*row_stride.  Only the first
 *     scored_rows rows of a sequence are scored; the reference layout is
 *     seq_rows = L, scored_rows = L-1 (logits[:, :-1, :] against
 *     input_ids[:, 1:], train_modules/__init__.py:118-126).  A flat [N, V]
 *     problem is n_seqs = N, seq_rows = scored_rows = 1, or any (B, T, T).
 *   - Per-token side arrays are dense [n_seqs * scored_rows] in (b, t) order.
 *   - Vocabulary sharding: a call sees columns
 *     [vocab_start, vocab_start + vocab) of a vocabulary of any total size;
 *     chosen_ids are GLOBAL ids.
 */
#ifndef MLLM_GRPO_H_
#define MLLM_GRPO_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MLLM_GRPO_ABI_VERSION 3
#define MLLM_GRPO_MAX_SHARDS 8

typedef enum mllm_grpo_status {
  MLLM_GRPO_OK = 0,
  MLLM_GRPO_ERR_NULL_POINTER = 1,   /* a required pointer is NULL */
  MLLM_GRPO_ERR_BAD_SHAPE = 2,      /* non-positive size, scored_rows > seq_rows, row_stride < vocab ... */
  MLLM_GRPO_ERR_BAD_ATTRIBUTE = 3,  /* temperature <= 0, negative epsilon, softcap < 0 ... */
  MLLM_GRPO_ERR_STRUCT_SIZE = 4,    /* args->struct_size does not match this library */
  MLLM_GRPO_ERR_ALIGNMENT = 5,      /* a side array is not 4-byte aligned / logits not 2-byte aligned */
  MLLM_GRPO_ERR_LAUNCH = 6,         /* the CUDA runtime refused the launch (see mllm_grpo_last_cuda_error) */
  MLLM_GRPO_ERR_UNSUPPORTED = 7,    /* combination not implemented (stated per entry point) */
  MLLM_GRPO_ERR_TOO_LARGE = 8,      /* problem exceeds a fixed capacity of the entry point */
  MLLM_GRPO_ERR_NO_DEVICE = 9       /* no CUDA device / wrong architecture */
} mllm_grpo_status;

/* Bits the kernels may OR into *args->device_status (an int32 in device memory,
 * read by the host after it has synchronised the stream itself). */
#define MLLM_GRPO_DEV_ID_CLAMPED 1   /* a chosen id fell outside [0, vocab_total) and was clamped */
#define MLLM_GRPO_DEV_WAIT_TIMEOUT 2 /* a bounded wait on a peer ran out: the call's loss is NaN, its dlogits of
                                        the affected rows are zero, and the bit stays set until the caller clears it */

/* One struct serves every entry point; each entry point documents the fields
 * it reads.  Zero-initialise it, set struct_size = sizeof(mllm_grpo_args). */
typedef struct mllm_grpo_args {
  uint64_t struct_size;

  /* ---- geometry ---- */
  int64_t n_seqs;       /* B  > 0 */
  int64_t seq_rows;     /* L  >= scored_rows */
  int64_t scored_rows;  /* T  > 0 */
  int64_t vocab;        /* columns held by this call (V, or V/k when sharded) */
  int64_t row_stride;   /* elements between consecutive rows of logits AND dlogits, >= vocab */
  int64_t vocab_start;  /* global id of local column 0 (0 when unsharded) */
  int64_t vocab_total;  /* global vocabulary size; 0 means vocab_start + vocab */

  /* ---- attributes: TrainGRPOModule fields, train_modules/__init__.py:89-93 ---- */
  float temperature;    /* > 0.  lp = log_softmax(x)[c] / temperature (:124-126) */
  float epsilon_low;    /* clip lower bound is 1 - epsilon_low  (:170) */
  float epsilon_high;   /* clip upper bound is 1 + epsilon_high (:170) */
  float beta;           /* weight of the k3 KL term; used only if ref_logps != NULL */
  float softcap;        /* 0 = off; else y = softcap*tanh(x/softcap) replaces x
                           (deprecated/MLLM_JAX/language/gemma/transformer.py:337-339) */
  int32_t adv_per_token;/* 0: advantages is [n_seqs] (train_modules :173);
                           1: [n_seqs*scored_rows] (ppo/module.py:87-94) */
  int32_t flags;        /* MLLM_GRPO_FLAG_* */
  float grad_scale;     /* upstream cotangent of the loss used when grad_scale_dev == NULL */
  float total_valid;    /* total_valid_token_count used when total_valid_dev == NULL (:179) */

  /* ---- inputs ---- */
  const void* logits;            /* bf16 [n_seqs, seq_rows, row_stride] */
  const int32_t* chosen_ids;     /* [B*T] global token ids (input_ids[:, 1:], :118) */
  const float* mask;             /* [B*T] completion mask as f32 0/1 (labels[:, 1:], :120) */
  const float* advantages;       /* [B] or [B*T] */
  const float* old_logps;        /* [B*T] or NULL: NULL means old = stop_gradient(lp) (:161-165) */
  const float* ref_logps;        /* [B*T] or NULL: reference-policy log-probs for the KL term */
  const float* total_valid_dev;  /* scalar in device memory or NULL (then total_valid is used) */
  const float* grad_scale_dev;   /* scalar in device memory or NULL (then grad_scale is used) */

  /* ---- outputs of the forward; inputs of the backward ---- */
  float* per_token_logps; /* [B*T]  lp  (returned by the reference as 'per_token_logps', :187) */
  float* token_entropy;   /* [B*T]  H_t = -sum p log p of softmax(x/temperature) (:136-138); may be NULL */
  float* lse;             /* [B*T]  log-sum-exp of the (soft-capped) row: residual for the backward */
  float* grad_coef;       /* [B*T]  mask*w_t/temperature, w_t = dloss_t/dlp_t sign-flipped: residual */
  float* loss;            /* [1]    sum_t mask_t*(-ppo_t + beta*kl_t) / total_valid (:178-180) */
  float* loss_terms;      /* [B*T]  scratch: per-token numerators, reduced in a fixed order */

  /* ---- output of the backward ---- */
  void* dlogits;          /* bf16 [n_seqs, seq_rows, row_stride]; may alias logits (in place) */

  /* ---- vocabulary-sharded path ---- */
  float* partials;        /* [B*T, 4] (max, sumexp, sum e*y, chosen-or-0) of THIS shard; [B*T, 6] when the entropy
                             is requested at temperature != 1 (then: max, sumexp, 0, chosen-or-0, and the two sums
                             of the entropy on y/temperature) */
  const float* gathered_partials; /* [n_shards, B*T, 4 or 6]: every shard's partials (after the exchange) */
  int32_t n_shards;
  int32_t shard_rank;     /* this call's shard index in [0, n_shards) (peer-exchange entry point only) */

  /* ---- error reporting ---- */
  int32_t* device_status; /* optional int32 in device memory; kernels OR MLLM_GRPO_DEV_* bits into it */

  /* ---- peer exchange of mllm_grpo_fwd_bwd_sharded ---- */
  void* peer_exchange[MLLM_GRPO_MAX_SHARDS]; /* peer_exchange[q]: address, valid on THIS device, of rank q's
                                                exchange buffer (mllm_grpo_exchange_bytes each, zeroed once);
                                                entry shard_rank is this rank's own buffer */
  int32_t exchange_epoch; /* > 0, the same on every rank, +1 on every call that uses the buffers */
  int32_t peer_wait_ms;   /* how long a row may wait for the other ranks' partials; 0 = 2000 ms.  This is the
                             skew between ranks the call tolerates (a rank held up by a checkpoint, a data
                             loader or a collector for longer than this poisons the step, see below) */

  /* ---- per-sample monitors of mllm_grpo_entropy_stats ---- */
  float* sample_entropy;        /* [B] sum_t H_t m_t / sum_t m_t                      (train_modules :141-143) */
  float* sample_entropy_window; /* [B] the same over valid tokens number 4..100 of a sample (:148-157) */

  /* ---- gradient of the entropy (mllm_grpo_bwd only) ---- */
  const float* entropy_cotangent; /* [B*T] or NULL: cotangent of token_entropy.  When given, mllm_grpo_bwd adds
                                     cot_t * dH_t/dlogits to dlogits (the -entropy_coef * entropy term of
                                     plugins/training/ppo/module.py:140 reaches the logits this way); it is
                                     not multiplied by grad_scale, which belongs to the loss */
  float* lse_scaled;              /* [B*T] or NULL: log-sum-exp of the row divided by the temperature, written
                                     by the forward when non-NULL; the entropy gradient reads it when
                                     temperature != 1 (at temperature 1 it equals lse and may stay NULL) */
} mllm_grpo_args;

#define MLLM_GRPO_FLAG_SKIP_ENTROPY 1 /* do not compute token_entropy (saves one FMA per element) */
#define MLLM_GRPO_FLAG_CE_LOSS 2      /* masked cross-entropy instead of the clipped surrogate: per-token loss
                                         -lp, loss = sum(mask * -lp) / total_valid, dlogits =
                                         mask/total_valid * (softmax - onehot); advantages, old_logps and
                                         ref_logps are ignored (plugins/sft/jax/sft_module.py:29-41) */

/* Forward over full rows (vocab_start = 0, vocab = vocab_total).
 * Replaces train_modules/__init__.py:118-180 (ppo/module.py:66-102 with adv_per_token = 1).
 * Reads logits once.  Writes per_token_logps, token_entropy (unless NULL or
 * SKIP_ENTROPY), lse, grad_coef, loss_terms and loss. */
int mllm_grpo_fwd(const mllm_grpo_args* args, void* stream);

/* Backward: dlogits[b, r, j] = g*(softmax_j - onehot_j) (times the soft-cap
 * derivative), g = grad_scale * grad_coef / total_valid; rows r >= scored_rows
 * and rows whose g is 0 are written as exact zeros without reading logits.
 * Replaces the autodiff of the region above (update/train_step.py:24).
 * Reads lse, grad_coef, chosen_ids, logits; writes dlogits (bf16).
 * With vocab sharding each shard calls it on its own columns; no exchange. */
int mllm_grpo_bwd(const mllm_grpo_args* args, void* stream);

/* Forward and backward in one launch, the shape of jax.value_and_grad in
 * training_step (update/train_step.py:24): every output of mllm_grpo_fwd and
 * of mllm_grpo_bwd.  The row is kept on chip between the two sweeps, so logits
 * are read from HBM once.  grad_scale must be known up front (1.0 in
 * training_step). */
int mllm_grpo_fwd_bwd(const mllm_grpo_args* args, void* stream);

/* Applies a late upstream cotangent to gradients that mllm_grpo_fwd_bwd already wrote with
 * grad_scale = 1 (the forward of a custom_vjp that computes its gradient eagerly): dlogits *= g with
 * g read from grad_scale_dev (or grad_scale).  Every CTA reads g first and returns at once when it is
 * exactly 1, the case of jax.value_and_grad on the loss itself (update/train_step.py:24), so the
 * common path moves no data.  Reads n_seqs, seq_rows, vocab, row_stride, dlogits, grad_scale(_dev). */
int mllm_grpo_scale_grad(const mllm_grpo_args* args, void* stream);

/* Vocabulary-sharded forward, step 1: per-token (max, sumexp, sum e*y,
 * chosen-logit-or-0) of this shard's columns -> partials[B*T, 4] (6 floats per token when the entropy is wanted
 * at temperature != 1: mllm_grpo_partial_width tells which).  This is the
 * per-shard part of the all-reduce(max)/all-reduce(sum) XLA inserts when
 * log_softmax runs on tp-sharded logits (MLLM_JAX/utils.py:245). */
int mllm_grpo_fwd_partials(const mllm_grpo_args* args, void* stream);

/* Vocabulary-sharded forward, step 2: merge gathered_partials[n_shards, B*T, width]
 * and run the per-token epilogue; same outputs as mllm_grpo_fwd. */
int mllm_grpo_combine(const mllm_grpo_args* args, void* stream);

/* Floats per token in partials / gathered_partials for these attributes: 6 when token_entropy is requested
 * (non-NULL, no SKIP_ENTROPY flag) at temperature != 1, else 4. */
int32_t mllm_grpo_partial_width(const mllm_grpo_args* args);

/* Vocabulary-sharded forward AND backward in one kernel per GPU, with the exchange inside it.
 * Each rank (one process per GPU) calls it on its own column shard at the same time.  A CTA
 * streams its row shard once and pushes (max, sumexp, sum e*y, chosen-or-0) into every rank's
 * exchange buffer with plain 8-byte peer stores over NVLink; every word carries one float and the
 * call's epoch, so a word that shows the epoch is complete by itself (no separate flag, no fence).
 * The CTA then polls its OWN buffer (bounded) until all ranks' words show the epoch, merges, runs
 * the per-token epilogue and streams the row shard a second time (served on chip) to write its
 * dlogits columns.  This is the fused form of mllm_grpo_fwd_partials -> all-gather ->
 * mllm_grpo_combine -> mllm_grpo_bwd, i.e. of the all-reduce(max)/all-reduce(sum) XLA inserts for
 * tp-sharded logits (MLLM_JAX/utils.py:245).  Every output of mllm_grpo_fwd is replicated on every
 * rank.  Needs temperature == 1 when the entropy is requested, n_shards <= MLLM_GRPO_MAX_SHARDS,
 * every rank's exchange buffer mapped on this device with store access (cuMem / symmetric-memory
 * mappings; NVLink multicast is not used), the same exchange_epoch on all ranks (buffers are
 * double-buffered by its parity, so consecutive calls need no barrier between them) and a
 * non-NULL device_status.
 * Failure behaviour: a row whose peers' words do not arrive within peer_wait_ms raises
 * MLLM_GRPO_DEV_WAIT_TIMEOUT in *device_status; from then on no CTA of this call (or of a later
 * call that starts with the bit still set) waits any more, so a dead peer costs about one wait
 * limit per call, not one per row.  Every row that gave up gets per_token_logps = NaN and a zero
 * dlogits row, and the call's loss is NaN, so a poisoned step cannot be consumed unnoticed.  The
 * caller clears the bit before the next healthy call. */
int mllm_grpo_fwd_bwd_sharded(const mllm_grpo_args* args, void* stream);

/* Bytes of one rank's exchange buffer for n_tokens = B*T and n_shards ranks. */
int64_t mllm_grpo_exchange_bytes(int64_t n_tokens, int32_t n_shards);

/* Forward-only log-probs and entropies (no loss, no residuals): the
 * reference-model pass (train_modules/__init__.py:129-132) and the first PPO
 * epoch's per_token_logps collection (plugins/training/update/ppo.py:39-43).
 * Reads logits, chosen_ids; writes per_token_logps, token_entropy (optional), lse (optional). */
int mllm_grpo_logprobs(const mllm_grpo_args* args, void* stream);

/* Forward for callers that can neither pass a scratch buffer nor allocate one (code running inside
 * another framework's memory plan, e.g. an XLA custom-call handler that was given operands and
 * results only, or a loop that may not touch the allocator after start-up).  This entry point has no
 * counterpart in the reference.  Same inputs, outputs and results as mllm_grpo_fwd, except that
 * args->loss_terms is ignored: the per-token loss terms go to a fixed array inside the library's
 * device image (MLLM_GRPO_STATIC_SCRATCH_TOKENS floats = 4 MiB, held by every GPU that loads the
 * library until the process exits).
 *   - n_seqs*scored_rows > MLLM_GRPO_STATIC_SCRATCH_TOKENS returns MLLM_GRPO_ERR_TOO_LARGE.
 *   - Calls no cudaMalloc/cudaFree and no allocating library routine.
 *   - The first call on each device looks the array's device address up (cudaGetSymbolAddress, with
 *     that device current); make that first call before any stream capture begins.
 *   - All calls on a device share the one array, and it keeps the previous call's contents.  Every
 *     entry a call reads is written by that call first, so nothing has to be cleared; but two calls
 *     that overlap on the GPU (different streams, no ordering between them) race on it. */
#define MLLM_GRPO_STATIC_SCRATCH_TOKENS (1 << 20)
int mllm_grpo_fwd_static_scratch(const mllm_grpo_args* args, void* stream);

/* Per-sample entropy monitors of the reference's return dict ('entropy', 'entropy_loss',
 * train_modules/__init__.py:141-157) from token_entropy [B*T] and mask [B*T]: one CTA per sample,
 * a block scan gives each token its running count of valid tokens.  A sample without valid tokens
 * yields 0/0 = NaN, as in the reference.  Reads n_seqs, scored_rows, token_entropy, mask; writes
 * sample_entropy and sample_entropy_window. */
int mllm_grpo_entropy_stats(const mllm_grpo_args* args, void* stream);

/* Value-loss tail of the PPO actor-critic module (replaces plugins/training/ppo/module.py:104-140):
 *   value_pred = values[:, :scored_rows]                                        (:104)
 *   returns    = given, else advantages + value_pred (and then moves with the values)   (:105-107)
 *   old_values = given, else the values themselves without gradient             (:116-118)
 *   term       = max((v - r)^2, (old + clip(v - old, -c, c) - r)^2), or (v - r)^2 without a range  (:131-136)
 *   value_loss = sum(term * mask) / total_valid_token_count                     (:138)
 * out[0] = value_loss, out[1] = mean(value_pred), out[2] = mean(returns) (:147-148, plain means over
 * all n_seqs x scored_rows positions).  dvalues = grad_scale x d value_loss / d values, zero at
 * positions >= scored_rows; pass grad_scale = value_coef x the cotangent of the total loss (:140).
 * All arrays are f32 in device memory; returns, old_values and mask are [n_seqs, scored_rows]
 * row-major, values and dvalues [n_seqs, seq_rows].  Sums are taken in double precision in a
 * fixed order.  Asynchronous on the stream, allocates nothing. */
typedef struct mllm_ppo_value_args {
  uint64_t struct_size; /* sizeof(mllm_ppo_value_args) */
  int64_t n_seqs;
  int64_t seq_rows;    /* L */
  int64_t scored_rows; /* L - 1 in the reference */
  float clip_range;    /* value_clip_range (:20); negative = None */
  float grad_scale;
  float total_valid;   /* total_valid_token_count, used when total_valid_dev is NULL */
  int32_t adv_per_token; /* advantages are [n_seqs, scored_rows] instead of [n_seqs] */
  const float* total_valid_dev; /* optional scalar in device memory */
  const float* values;
  const float* returns;    /* optional */
  const float* advantages; /* required when returns is NULL */
  const float* old_values; /* optional */
  const float* mask;       /* optional: NULL = every position counts */
  float* dvalues;          /* optional */
  float* out;              /* [3] */
  double* workspace;       /* mllm_ppo_value_workspace_bytes(n_seqs, seq_rows) bytes, 8-byte aligned */
} mllm_ppo_value_args;
int mllm_ppo_value_loss(const mllm_ppo_value_args* args, void* stream);
int64_t mllm_ppo_value_workspace_bytes(int64_t n_seqs, int64_t seq_rows);

/* lm_head projection folded into the forward of the loss: logits = hidden x weight^T
 * (logits = self.lm_head(hidden_states), MLLM_JAX/language/qwen2/modular_qwen2.py:182, feeding
 * MLLM_JAX/train_modules/__init__.py:124-138) are produced tile by tile on the tensor cores
 * (tcgen05.mma into tensor memory, operands staged by TMA) and reduced there to the per-row
 * (max, sumexp, sum e*y, chosen-or-0) of mllm_grpo_fwd_partials; the [n_rows, vocab] logits never reach
 * HBM.  The vocabulary is cut into mllm_lm_head_splits() column ranges whose partials land in
 * partials[split, row, 4]; mllm_grpo_combine with gathered_partials = partials and
 * n_shards = mllm_lm_head_splits() then finishes the forward exactly as for vocabulary shards
 * (per_token_logps, token_entropy, lse, grad_coef, loss).  The logits are the f32 accumulators themselves
 * (no rounding to bf16 in between), soft-capped when softcap > 0.
 * tp-sharded head (lm_head kernel partitioned over "tp", MLLM_JAX/utils.py:245): every rank calls it on its own
 * weight rows [vocab_start, vocab_start + vocab) with GLOBAL chosen ids; the ranks' partials, all-gathered into
 * [k * splits, n_rows, 4], go through one mllm_grpo_combine with n_shards = k * splits.
 *   hidden [n_rows, hidden_dim] bf16, rows hidden_stride elements apart;
 *   weight [vocab, hidden_dim] bf16 (one row per vocabulary entry), rows weight_stride elements apart; or, with
 *   MLLM_LM_HEAD_FLAG_WEIGHT_HV, [hidden_dim, vocab] (a flax Dense kernel as it is stored: vocabulary contiguous,
 *   a vocabulary shard being a column range of it), read as an MN-major tensor-core operand without a transpose;
 *   hidden_dim a multiple of 64, strides multiples of 8 elements, bases 16-byte aligned, else
 *   MLLM_GRPO_ERR_UNSUPPORTED / _ALIGNMENT.  Entropy only at temperature 1 (the combine step's rule).
 * Asynchronous on the stream, allocates nothing.  A pipeline wait that runs out (never in normal
 * operation) raises MLLM_GRPO_DEV_WAIT_TIMEOUT in *device_status and the call's partials are void. */
typedef struct mllm_lm_head_args {
  uint64_t struct_size; /* sizeof(mllm_lm_head_args) */
  int64_t n_rows;       /* B*T scored rows */
  int64_t vocab;
  int64_t hidden_dim;
  int64_t hidden_stride;
  int64_t weight_stride;
  int64_t vocab_start;  /* global id of weight row 0 (0 unless this call holds one vocabulary shard of the head) */
  int64_t vocab_total;  /* global vocabulary size; 0 means vocab_start + vocab */
  float softcap;        /* 0 = off */
  int32_t flags;        /* MLLM_GRPO_FLAG_SKIP_ENTROPY, MLLM_LM_HEAD_FLAG_WEIGHT_HV */
  const void* hidden;
  const void* weight;
  const int32_t* chosen_ids; /* [n_rows] */
  void* partials;            /* mllm_lm_head_partials_bytes(n_rows, vocab) bytes, 16-byte aligned */
  int32_t* device_status;    /* optional */
} mllm_lm_head_args;
#define MLLM_LM_HEAD_FLAG_WEIGHT_HV 256 /* weight is [hidden_dim, vocab] row-major instead of [vocab, hidden_dim] */
int mllm_lm_head_partials(const mllm_lm_head_args* args, void* stream);
int32_t mllm_lm_head_splits(int64_t n_rows, int64_t vocab);
int64_t mllm_lm_head_partials_bytes(int64_t n_rows, int64_t vocab);

/* Bytes of loss_terms scratch a problem of n_tokens = B*T needs. */
int64_t mllm_grpo_workspace_bytes(int64_t n_tokens);

/* Tuning / test hook: forces how mllm_grpo_fwd_bwd and mllm_grpo_fwd_bwd_sharded run in this process, until
 * called again.  sweeps != 0: mllm_grpo_fwd_bwd takes the separate forward and backward kernels.  cluster
 * (1/2/4/6/8 CTAs per row), threads (64/128/256/512 per CTA), load_batch (6/8/10 vectors per thread) and staged
 * (0/1: row shard held in shared memory) override the plan the library derives from the row length; 0 (-1 for
 * staged) leaves a field automatic.  Combinations a kernel cannot run fall back to the nearest one that it can.
 * Production code never needs this: the automatic plan is the measured one. */
int mllm_grpo_set_plan_override(int sweeps, int cluster, int threads, int load_batch, int staged);

int mllm_grpo_abi_version(void);
const char* mllm_grpo_status_string(int status);
/* Text of the last CUDA runtime error seen by this thread's launches ("" if none). */
const char* mllm_grpo_last_cuda_error(void);
/* Number of kernels the library has launched in this process (for launch accounting). */
int64_t mllm_grpo_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* MLLM_GRPO_H_ */
