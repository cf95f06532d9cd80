// C-ABI layer: argument validation, mllm_grpo_args -> KernelParams, kernel selection.
// Every entry point is asynchronous on the caller's stream and allocates nothing.
#include <atomic>
#include <cstring>

#include "grpo_launch.h"

namespace grpo {

static std::atomic<int64_t> g_launches{0};
static std::atomic<int> g_force_sweeps{0};  // tuning / test hook: mllm_grpo_fwd_bwd as two separate sweeps
static thread_local char g_last_error[256] = {0};

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

static int fail_cuda(cudaError_t e) {
  std::strncpy(g_last_error, cudaGetErrorString(e), sizeof(g_last_error) - 1);
  return MLLM_GRPO_ERR_LAUNCH;
}

int record_cuda_error(cudaError_t e) { return fail_cuda(e); }

// What an entry point needs from the argument struct.
enum Need : unsigned {
  kLogits = 1u << 0,
  kIds = 1u << 1,
  kEpilogueIn = 1u << 2,   // advantages (mask/old/ref are optional)
  kEpilogueOut = 1u << 3,  // per_token_logps, lse, grad_coef, loss, loss_terms
  kDlogits = 1u << 4,
  kResiduals = 1u << 5,  // lse, grad_coef as inputs
  kPartialsOut = 1u << 6,
  kGathered = 1u << 7,
  kLogpOut = 1u << 8,
};

static bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

static int validate(const mllm_grpo_args* a, unsigned need, KernelParams* k) {
  if (a == nullptr) return MLLM_GRPO_ERR_NULL_POINTER;
  if (a->struct_size != sizeof(mllm_grpo_args)) return MLLM_GRPO_ERR_STRUCT_SIZE;
  if (a->n_seqs <= 0 || a->seq_rows <= 0 || a->scored_rows <= 0 || a->vocab <= 0) return MLLM_GRPO_ERR_BAD_SHAPE;
  if (a->scored_rows > a->seq_rows || a->row_stride < a->vocab || a->vocab_start < 0) return MLLM_GRPO_ERR_BAD_SHAPE;
  const int64_t vt = a->vocab_total > 0 ? a->vocab_total : a->vocab_start + a->vocab;
  if (a->vocab_start + a->vocab > vt) return MLLM_GRPO_ERR_BAD_SHAPE;
  const int64_t N = a->n_seqs * a->scored_rows, R = a->n_seqs * a->seq_rows;
  if (N >= (int64_t(1) << 31) || R >= (int64_t(1) << 31)) return MLLM_GRPO_ERR_TOO_LARGE;
  if (!(a->temperature > 0.f) || a->epsilon_low < 0.f || a->epsilon_high < 0.f || a->softcap < 0.f)
    return MLLM_GRPO_ERR_BAD_ATTRIBUTE;
  if (a->temperature != a->temperature || a->beta != a->beta) return MLLM_GRPO_ERR_BAD_ATTRIBUTE;

  if ((need & kLogits) && !a->logits) return MLLM_GRPO_ERR_NULL_POINTER;
  if ((need & kIds) && !a->chosen_ids) return MLLM_GRPO_ERR_NULL_POINTER;
  if ((need & kEpilogueIn) && !a->advantages && !(a->flags & MLLM_GRPO_FLAG_CE_LOSS)) return MLLM_GRPO_ERR_NULL_POINTER;
  if ((need & kEpilogueOut) && (!a->per_token_logps || !a->lse || !a->grad_coef || !a->loss || !a->loss_terms))
    return MLLM_GRPO_ERR_NULL_POINTER;
  if ((need & kEpilogueOut) && !a->total_valid_dev && !(a->total_valid == a->total_valid))
    return MLLM_GRPO_ERR_BAD_ATTRIBUTE;
  if ((need & kDlogits) && !a->dlogits) return MLLM_GRPO_ERR_NULL_POINTER;
  if ((need & kResiduals) && (!a->lse || !a->grad_coef)) return MLLM_GRPO_ERR_NULL_POINTER;
  if ((need & kPartialsOut) && !a->partials) return MLLM_GRPO_ERR_NULL_POINTER;
  if ((need & kGathered) && (!a->gathered_partials || a->n_shards <= 0)) return MLLM_GRPO_ERR_NULL_POINTER;
  if ((need & kLogpOut) && !a->per_token_logps) return MLLM_GRPO_ERR_NULL_POINTER;

  if (!aligned(a->logits, 2) || !aligned(a->dlogits, 2)) return MLLM_GRPO_ERR_ALIGNMENT;
  const void* f32s[] = {a->chosen_ids, a->mask, a->advantages, a->old_logps, a->ref_logps, a->total_valid_dev,
                        a->grad_scale_dev, a->per_token_logps, a->token_entropy, a->lse, a->grad_coef, a->loss,
                        a->loss_terms, a->device_status, a->entropy_cotangent, a->lse_scaled};
  for (const void* q : f32s)
    if (!aligned(q, 4)) return MLLM_GRPO_ERR_ALIGNMENT;
  if (!aligned(a->partials, 16) || !aligned(a->gathered_partials, 16)) return MLLM_GRPO_ERR_ALIGNMENT;

  k->n_seqs = a->n_seqs;
  k->seq_rows = a->seq_rows;
  k->scored_rows = a->scored_rows;
  k->vocab = a->vocab;
  k->row_stride = a->row_stride;
  k->vocab_start = a->vocab_start;
  k->vocab_total = vt;
  k->inv_temperature = 1.0f / a->temperature;
  k->clip_lo = 1.0f - a->epsilon_low;
  k->clip_hi = 1.0f + a->epsilon_high;
  k->beta = a->beta;
  k->softcap = a->softcap;
  k->grad_scale = a->grad_scale;
  k->total_valid = a->total_valid;
  k->adv_per_token = a->adv_per_token;
  k->ce_loss = (a->flags & MLLM_GRPO_FLAG_CE_LOSS) ? 1 : 0;
  k->logits = static_cast<const __nv_bfloat16*>(a->logits);
  k->chosen_ids = a->chosen_ids;
  k->mask = a->mask;
  k->advantages = a->advantages;
  k->old_logps = a->old_logps;
  k->ref_logps = a->ref_logps;
  k->total_valid_dev = a->total_valid_dev;
  k->grad_scale_dev = a->grad_scale_dev;
  k->per_token_logps = a->per_token_logps;
  k->token_entropy = a->token_entropy;
  k->lse = a->lse;
  k->lse_scaled = a->lse_scaled;
  k->entropy_cotangent = nullptr;  // only mllm_grpo_bwd honours it
  k->grad_coef = a->grad_coef;
  k->loss = a->loss;
  k->loss_terms = a->loss_terms;
  k->dlogits = static_cast<__nv_bfloat16*>(a->dlogits);
  k->partials = a->partials;
  k->gathered_partials = a->gathered_partials;
  k->n_shards = a->n_shards;
  k->device_status = a->device_status;
  k->shard_rank = a->shard_rank;
  k->exchange_epoch = a->exchange_epoch;
  k->peer_wait_ns = (a->peer_wait_ms > 0 ? static_cast<unsigned long long>(a->peer_wait_ms) : 2000ull) * 1000000ull;
  for (int q = 0; q < MLLM_GRPO_MAX_SHARDS; ++q) k->peer_words[q] = nullptr;
  return MLLM_GRPO_OK;
}

// Entropy mode of a call: 0 off, 1 temperature == 1, 2 otherwise.
static int entropy_mode(const mllm_grpo_args* a) {
  if ((a->flags & MLLM_GRPO_FLAG_SKIP_ENTROPY) || a->token_entropy == nullptr) return 0;
  return a->temperature == 1.0f ? 1 : 2;
}

}  // namespace grpo

using namespace grpo;

extern "C" {

int mllm_grpo_fwd(const mllm_grpo_args* args, void* stream) {
  KernelParams k;
  int st = validate(args, kLogits | kIds | kEpilogueIn | kEpilogueOut, &k);
  if (st) return st;
  if (k.vocab_start != 0 || k.vocab != k.vocab_total) return MLLM_GRPO_ERR_BAD_SHAPE;  // full rows only
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = launch_row_stats(k, 0, entropy_mode(args), s);
  if (e != cudaSuccess) return fail_cuda(e);
  e = launch_loss_reduce(k, s);
  if (e != cudaSuccess) return fail_cuda(e);
  return MLLM_GRPO_OK;
}

int mllm_grpo_bwd(const mllm_grpo_args* args, void* stream) {
  KernelParams k;
  int st = validate(args, kLogits | kIds | kResiduals | kDlogits, &k);
  if (st) return st;
  if (args->entropy_cotangent) {
    // needs the forward's token_entropy, its lse_scaled when temperature != 1, and vector-aligned rows
    if (!args->token_entropy || (args->temperature != 1.0f && !args->lse_scaled)) return MLLM_GRPO_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(args->logits) ^ reinterpret_cast<uintptr_t>(args->dlogits)) & 15)
      return MLLM_GRPO_ERR_UNSUPPORTED;
    k.entropy_cotangent = args->entropy_cotangent;
  }
  cudaError_t e = launch_dlogits(k, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail_cuda(e);
  return MLLM_GRPO_OK;
}

int mllm_grpo_fwd_bwd(const mllm_grpo_args* args, void* stream) {
  KernelParams k;
  int st = validate(args, kLogits | kIds | kEpilogueIn | kEpilogueOut | kDlogits, &k);
  if (st) return st;
  if (k.vocab_start != 0 || k.vocab != k.vocab_total) return MLLM_GRPO_ERR_BAD_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  bool taken = false;
  cudaError_t e = cudaSuccess;
  // Both passes in one kernel, the second read served on chip (grpo_twopass.cu); the separate sweeps
  // serve row pairs whose logits and dlogits do not share their 16-byte phase.
  const int ent = entropy_mode(args);
  if (!g_force_sweeps.load(std::memory_order_relaxed)) e = launch_two_pass(k, ent, false, s, &taken);
  if (e != cudaSuccess) return fail_cuda(e);
  if (taken) {
    e = launch_loss_reduce(k, s);
    if (e != cudaSuccess) return fail_cuda(e);
    return MLLM_GRPO_OK;
  }
  e = launch_row_stats(k, 0, entropy_mode(args), s);
  if (e != cudaSuccess) return fail_cuda(e);
  e = launch_loss_reduce(k, s);
  if (e != cudaSuccess) return fail_cuda(e);
  e = launch_dlogits(k, s);
  if (e != cudaSuccess) return fail_cuda(e);
  return MLLM_GRPO_OK;
}

int mllm_grpo_scale_grad(const mllm_grpo_args* args, void* stream) {
  KernelParams k;
  int st = validate(args, kDlogits, &k);
  if (st) return st;
  cudaError_t e = launch_scale_grad(k, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail_cuda(e);
  return MLLM_GRPO_OK;
}

int mllm_grpo_fwd_partials(const mllm_grpo_args* args, void* stream) {
  KernelParams k;
  int st = validate(args, kLogits | kIds | kPartialsOut, &k);
  if (st) return st;
  // entropy at temperature != 1: records of 6 floats (two more sums on y/temperature), see the header
  const int ent = args->temperature == 1.0f ? ((args->flags & MLLM_GRPO_FLAG_SKIP_ENTROPY) ? 0 : 1) : entropy_mode(args);
  cudaError_t e = launch_row_stats(k, 1, ent, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail_cuda(e);
  return MLLM_GRPO_OK;
}

int mllm_grpo_combine(const mllm_grpo_args* args, void* stream) {
  KernelParams k;
  int st = validate(args, kEpilogueIn | kEpilogueOut | kGathered, &k);
  if (st) return st;
  const int ent = entropy_mode(args);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = launch_combine(k, ent, s);
  if (e != cudaSuccess) return fail_cuda(e);
  e = launch_loss_reduce(k, s);
  if (e != cudaSuccess) return fail_cuda(e);
  return MLLM_GRPO_OK;
}

int32_t mllm_grpo_partial_width(const mllm_grpo_args* args) {
  if (args == nullptr) return 4;
  return entropy_mode(args) == 2 ? 6 : 4;
}

int mllm_grpo_entropy_stats(const mllm_grpo_args* args, void* stream) {
  if (args == nullptr) return MLLM_GRPO_ERR_NULL_POINTER;
  if (args->struct_size != sizeof(mllm_grpo_args)) return MLLM_GRPO_ERR_STRUCT_SIZE;
  if (args->n_seqs <= 0 || args->scored_rows <= 0 || args->n_seqs >= (int64_t(1) << 31)) return MLLM_GRPO_ERR_BAD_SHAPE;
  if (!args->token_entropy || !args->mask || !args->sample_entropy || !args->sample_entropy_window)
    return MLLM_GRPO_ERR_NULL_POINTER;
  const cudaError_t e = launch_entropy_stats(args->token_entropy, args->mask, args->n_seqs, args->scored_rows,
                                             args->sample_entropy, args->sample_entropy_window,
                                             static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? MLLM_GRPO_OK : fail_cuda(e);
}

int mllm_grpo_set_plan_override(int sweeps, int cluster, int threads, int load_batch, int staged) {
  g_force_sweeps = sweeps != 0;
  set_two_pass_override(cluster, threads, load_batch, staged);
  return MLLM_GRPO_OK;
}

int64_t mllm_grpo_exchange_bytes(int64_t n_tokens, int32_t n_shards) {
  if (n_tokens <= 0 || n_shards <= 0 || n_shards > MLLM_GRPO_MAX_SHARDS) return 0;
  // two epoch parities x n_shards senders x n_tokens x 4 words of (float value, int32 epoch)
  return int64_t(2) * n_shards * n_tokens * 4 * int64_t(sizeof(unsigned long long));
}

int mllm_grpo_fwd_bwd_sharded(const mllm_grpo_args* args, void* stream) {
  KernelParams k;
  int st = validate(args, kLogits | kIds | kEpilogueIn | kEpilogueOut | kDlogits, &k);
  if (st) return st;
  if (args->n_shards <= 0 || args->n_shards > MLLM_GRPO_MAX_SHARDS) return MLLM_GRPO_ERR_TOO_LARGE;
  if (args->shard_rank < 0 || args->shard_rank >= args->n_shards || args->exchange_epoch <= 0)
    return MLLM_GRPO_ERR_BAD_ATTRIBUTE;
  const int ent = entropy_mode(args);
  if (ent == 2) return MLLM_GRPO_ERR_UNSUPPORTED;  // sharded entropy needs temperature 1
  if (args->device_status == nullptr) return MLLM_GRPO_ERR_NULL_POINTER;  // the waits report through it
  for (int q = 0; q < args->n_shards; ++q) {
    if (args->peer_exchange[q] == nullptr) return MLLM_GRPO_ERR_NULL_POINTER;
    if (!aligned(args->peer_exchange[q], 16)) return MLLM_GRPO_ERR_ALIGNMENT;
    k.peer_words[q] = static_cast<unsigned long long*>(args->peer_exchange[q]);
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  bool taken = false;
  cudaError_t e = launch_two_pass(k, ent, true, s, &taken);
  if (e != cudaSuccess) return fail_cuda(e);
  if (!taken) return MLLM_GRPO_ERR_ALIGNMENT;  // logits and dlogits rows must share their 16-byte phase
  e = launch_loss_reduce(k, s);
  if (e != cudaSuccess) return fail_cuda(e);
  return MLLM_GRPO_OK;
}

int mllm_grpo_logprobs(const mllm_grpo_args* args, void* stream) {
  KernelParams k;
  int st = validate(args, kLogits | kIds | kLogpOut, &k);
  if (st) return st;
  if (k.vocab_start != 0 || k.vocab != k.vocab_total) return MLLM_GRPO_ERR_BAD_SHAPE;
  cudaError_t e = launch_row_stats(k, 2, entropy_mode(args), static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail_cuda(e);
  return MLLM_GRPO_OK;
}

int64_t mllm_grpo_workspace_bytes(int64_t n_tokens) { return n_tokens > 0 ? n_tokens * int64_t(sizeof(float)) : 0; }

int mllm_grpo_abi_version(void) { return MLLM_GRPO_ABI_VERSION; }

const char* mllm_grpo_status_string(int status) {
  switch (status) {
    case MLLM_GRPO_OK: return "ok";
    case MLLM_GRPO_ERR_NULL_POINTER: return "a required pointer is NULL";
    case MLLM_GRPO_ERR_BAD_SHAPE: return "bad shape";
    case MLLM_GRPO_ERR_BAD_ATTRIBUTE: return "bad attribute";
    case MLLM_GRPO_ERR_STRUCT_SIZE: return "struct_size does not match this library";
    case MLLM_GRPO_ERR_ALIGNMENT: return "misaligned pointer";
    case MLLM_GRPO_ERR_LAUNCH: return "CUDA launch failed";
    case MLLM_GRPO_ERR_UNSUPPORTED: return "unsupported combination";
    case MLLM_GRPO_ERR_TOO_LARGE: return "problem too large";
    case MLLM_GRPO_ERR_NO_DEVICE: return "no usable CUDA device";
    default: return "unknown status";
  }
}

const char* mllm_grpo_last_cuda_error(void) { return g_last_error; }

int64_t mllm_grpo_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
