// XLA FFI handlers over the C ABI of libmllm_grpo.so, for jax.ffi.ffi_call.
//
// NOT BUILT OR RUN where this repository was developed: jaxlib (and with it xla/ffi/api/ffi.h) is
// installed neither there nor on the GPU hosts it was measured on.  Build where JAX exists:
//   g++ -std=c++17 -shared -fPIC -I$(python -c "import jax.ffi; print(jax.ffi.include_dir())") \
//       -I../../include -I/usr/local/cuda/include grpo_ffi.cc -L../lib -lmllm_grpo -o libmllm_grpo_ffi.so
// The handlers only decode arguments; every check and every kernel lives behind the C ABI.  They keep no
// state, allocate nothing and never synchronise, so XLA may call them from any of its host threads and
// capture them in CUDA graphs.
//
// Handlers (one per entry point a jitted train step needs):
//   MllmGrpoFwd         mllm_grpo_fwd           forward, residuals (lse, grad_coef) out
//   MllmGrpoBwd         mllm_grpo_bwd           backward sweep, dlogits may alias logits
//   MllmGrpoFwdBwd      mllm_grpo_fwd_bwd       loss AND dlogits from one kernel (cotangent 1)
//   MllmGrpoScaleGrad   mllm_grpo_scale_grad    late cotangent on those dlogits (returns at once for 1)
//   MllmGrpoLogprobs    mllm_grpo_logprobs      forward-only log-probs / entropy (reference model, epoch 0)
//   MllmGrpoEntropyStats mllm_grpo_entropy_stats per-sample entropy monitors
#include <cuda_runtime_api.h>

#include "mllm_grpo.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

ffi::Error ToError(int status) {
  if (status == MLLM_GRPO_OK) return ffi::Error::Success();
  const ffi::ErrorCode code = status <= MLLM_GRPO_ERR_ALIGNMENT ? ffi::ErrorCode::kInvalidArgument : ffi::ErrorCode::kInternal;
  return ffi::Error(code, mllm_grpo_status_string(status));
}

// Attributes every loss handler takes (all f32 / i64 / bool: pass numpy scalars of exactly these types).
struct Attrs {
  float temperature, epsilon_low, epsilon_high, beta, softcap;
  int64_t scored_rows;
};

// logits [B, L, V] bf16; ids / mask / old / ref [B, T]; adv [B] or [B, T]; nv scalar f32.
void FillCommon(mllm_grpo_args* a, ffi::Buffer<ffi::BF16>& logits, const Attrs& at) {
  *a = mllm_grpo_args{};
  a->struct_size = sizeof(*a);
  auto d = logits.dimensions();
  a->n_seqs = d[0];
  a->seq_rows = d[1];
  a->scored_rows = at.scored_rows;
  a->vocab = a->row_stride = d[2];
  a->temperature = at.temperature;
  a->epsilon_low = at.epsilon_low;
  a->epsilon_high = at.epsilon_high;
  a->beta = at.beta;
  a->softcap = at.softcap;
  a->grad_scale = 1.0f;
  a->logits = logits.typed_data();
}

void FillSide(mllm_grpo_args* a, ffi::Buffer<ffi::S32>& ids, ffi::Buffer<ffi::F32>& mask, ffi::Buffer<ffi::F32>& adv,
              ffi::Buffer<ffi::F32>& old_lp, ffi::Buffer<ffi::F32>& ref_lp, ffi::Buffer<ffi::F32>& nv, bool has_old,
              bool has_ref) {
  a->chosen_ids = ids.typed_data();
  a->mask = mask.typed_data();
  a->advantages = adv.typed_data();
  a->adv_per_token = adv.element_count() == static_cast<size_t>(a->n_seqs) ? 0 : 1;
  a->old_logps = has_old ? old_lp.typed_data() : nullptr;  // absent: old = stop_gradient(lp)
  a->ref_logps = has_ref ? ref_lp.typed_data() : nullptr;  // absent: no KL term
  a->total_valid_dev = nv.typed_data();
}

ffi::Error FwdImpl(cudaStream_t stream, ffi::Buffer<ffi::BF16> logits, ffi::Buffer<ffi::S32> ids,
                   ffi::Buffer<ffi::F32> mask, ffi::Buffer<ffi::F32> adv, ffi::Buffer<ffi::F32> old_lp,
                   ffi::Buffer<ffi::F32> ref_lp, ffi::Buffer<ffi::F32> nv, ffi::ResultBuffer<ffi::F32> loss,
                   ffi::ResultBuffer<ffi::F32> lp, ffi::ResultBuffer<ffi::F32> ent, ffi::ResultBuffer<ffi::F32> lse,
                   ffi::ResultBuffer<ffi::F32> gcoef, ffi::ResultBuffer<ffi::F32> terms, float temperature,
                   float epsilon_low, float epsilon_high, float beta, float softcap, int64_t scored_rows,
                   bool has_old, bool has_ref) {
  mllm_grpo_args a;
  FillCommon(&a, logits, Attrs{temperature, epsilon_low, epsilon_high, beta, softcap, scored_rows});
  FillSide(&a, ids, mask, adv, old_lp, ref_lp, nv, has_old, has_ref);
  a.loss = loss->typed_data();
  a.per_token_logps = lp->typed_data();
  a.token_entropy = ent->typed_data();
  a.lse = lse->typed_data();
  a.grad_coef = gcoef->typed_data();
  a.loss_terms = terms->typed_data();
  return ToError(mllm_grpo_fwd(&a, stream));
}

// Loss and dlogits from one kernel (the logits cross HBM once); dlogits may alias logits.
ffi::Error FwdBwdImpl(cudaStream_t stream, ffi::Buffer<ffi::BF16> logits, ffi::Buffer<ffi::S32> ids,
                      ffi::Buffer<ffi::F32> mask, ffi::Buffer<ffi::F32> adv, ffi::Buffer<ffi::F32> old_lp,
                      ffi::Buffer<ffi::F32> ref_lp, ffi::Buffer<ffi::F32> nv, ffi::ResultBuffer<ffi::F32> loss,
                      ffi::ResultBuffer<ffi::F32> lp, ffi::ResultBuffer<ffi::F32> ent, ffi::ResultBuffer<ffi::F32> lse,
                      ffi::ResultBuffer<ffi::F32> gcoef, ffi::ResultBuffer<ffi::F32> terms,
                      ffi::ResultBuffer<ffi::BF16> dlogits, float temperature, float epsilon_low, float epsilon_high,
                      float beta, float softcap, int64_t scored_rows, bool has_old, bool has_ref) {
  mllm_grpo_args a;
  FillCommon(&a, logits, Attrs{temperature, epsilon_low, epsilon_high, beta, softcap, scored_rows});
  FillSide(&a, ids, mask, adv, old_lp, ref_lp, nv, has_old, has_ref);
  a.loss = loss->typed_data();
  a.per_token_logps = lp->typed_data();
  a.token_entropy = ent->typed_data();
  a.lse = lse->typed_data();
  a.grad_coef = gcoef->typed_data();
  a.loss_terms = terms->typed_data();
  a.dlogits = dlogits->typed_data();
  return ToError(mllm_grpo_fwd_bwd(&a, stream));
}

// dlogits may alias logits (input_output_aliases={0: 0} at the call site).
ffi::Error BwdImpl(cudaStream_t stream, ffi::Buffer<ffi::BF16> logits, ffi::Buffer<ffi::S32> ids,
                   ffi::Buffer<ffi::F32> lse, ffi::Buffer<ffi::F32> gcoef, ffi::Buffer<ffi::F32> nv,
                   ffi::Buffer<ffi::F32> cotangent, ffi::ResultBuffer<ffi::BF16> dlogits, float temperature,
                   float softcap, int64_t scored_rows) {
  mllm_grpo_args a;
  FillCommon(&a, logits, Attrs{temperature, 0.f, 0.f, 0.f, softcap, scored_rows});
  a.chosen_ids = ids.typed_data();
  a.lse = lse.typed_data();
  a.grad_coef = gcoef.typed_data();
  a.total_valid_dev = nv.typed_data();
  a.grad_scale_dev = cotangent.typed_data();
  a.dlogits = dlogits->typed_data();
  return ToError(mllm_grpo_bwd(&a, stream));
}

// In place on the gradient the forward wrote with cotangent 1 (input_output_aliases={0: 0}).
ffi::Error ScaleGradImpl(cudaStream_t stream, ffi::Buffer<ffi::BF16> dlogits_in, ffi::Buffer<ffi::F32> cotangent,
                         ffi::ResultBuffer<ffi::BF16> dlogits) {
  mllm_grpo_args a = mllm_grpo_args{};
  a.struct_size = sizeof(a);
  auto d = dlogits_in.dimensions();
  a.n_seqs = d[0];
  a.seq_rows = a.scored_rows = d[1];
  a.vocab = a.row_stride = d[2];
  a.temperature = 1.0f;
  a.grad_scale_dev = cotangent.typed_data();
  a.dlogits = dlogits->typed_data();
  if (dlogits->typed_data() != dlogits_in.typed_data())
    return ffi::Error(ffi::ErrorCode::kInvalidArgument, "scale_grad works in place: alias operand 0 to result 0");
  return ToError(mllm_grpo_scale_grad(&a, stream));
}

ffi::Error LogprobsImpl(cudaStream_t stream, ffi::Buffer<ffi::BF16> logits, ffi::Buffer<ffi::S32> ids,
                        ffi::ResultBuffer<ffi::F32> lp, ffi::ResultBuffer<ffi::F32> ent, ffi::ResultBuffer<ffi::F32> lse,
                        float temperature, float softcap, int64_t scored_rows) {
  mllm_grpo_args a;
  FillCommon(&a, logits, Attrs{temperature, 0.f, 0.f, 0.f, softcap, scored_rows});
  a.chosen_ids = ids.typed_data();
  a.per_token_logps = lp->typed_data();
  a.token_entropy = ent->typed_data();
  a.lse = lse->typed_data();
  return ToError(mllm_grpo_logprobs(&a, stream));
}

ffi::Error EntropyStatsImpl(cudaStream_t stream, ffi::Buffer<ffi::F32> token_entropy, ffi::Buffer<ffi::F32> mask,
                            ffi::ResultBuffer<ffi::F32> entropy, ffi::ResultBuffer<ffi::F32> entropy_window) {
  mllm_grpo_args a = mllm_grpo_args{};
  a.struct_size = sizeof(a);
  auto d = token_entropy.dimensions();
  a.n_seqs = d[0];
  a.seq_rows = a.scored_rows = d[1];
  a.token_entropy = token_entropy.typed_data();
  a.mask = mask.typed_data();
  a.sample_entropy = entropy->typed_data();
  a.sample_entropy_window = entropy_window->typed_data();
  return ToError(mllm_grpo_entropy_stats(&a, stream));
}

}  // namespace

#define MLLM_LOSS_ARGS                                                          \
  .Arg<ffi::Buffer<ffi::BF16>>()     /* logits */                               \
      .Arg<ffi::Buffer<ffi::S32>>()  /* chosen ids */                           \
      .Arg<ffi::Buffer<ffi::F32>>()  /* mask */                                 \
      .Arg<ffi::Buffer<ffi::F32>>()  /* advantages */                           \
      .Arg<ffi::Buffer<ffi::F32>>()  /* old log-probs (dummy if absent) */      \
      .Arg<ffi::Buffer<ffi::F32>>()  /* ref log-probs (dummy if absent) */      \
      .Arg<ffi::Buffer<ffi::F32>>()  /* total_valid_token_count */              \
      .Ret<ffi::Buffer<ffi::F32>>()  /* loss */                                 \
      .Ret<ffi::Buffer<ffi::F32>>()  /* per_token_logps */                      \
      .Ret<ffi::Buffer<ffi::F32>>()  /* token_entropy */                        \
      .Ret<ffi::Buffer<ffi::F32>>()  /* lse */                                  \
      .Ret<ffi::Buffer<ffi::F32>>()  /* grad_coef */                            \
      .Ret<ffi::Buffer<ffi::F32>>()  /* loss_terms scratch */
#define MLLM_LOSS_ATTRS                                                                                   \
  .Attr<float>("temperature").Attr<float>("epsilon_low").Attr<float>("epsilon_high").Attr<float>("beta") \
      .Attr<float>("softcap").Attr<int64_t>("scored_rows").Attr<bool>("has_old").Attr<bool>("has_ref")

XLA_FFI_DEFINE_HANDLER_SYMBOL(MllmGrpoFwd, FwdImpl,
                              ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>() MLLM_LOSS_ARGS MLLM_LOSS_ATTRS);

XLA_FFI_DEFINE_HANDLER_SYMBOL(MllmGrpoFwdBwd, FwdBwdImpl,
                              ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>() MLLM_LOSS_ARGS
                                  .Ret<ffi::Buffer<ffi::BF16>>()  // dlogits
                              MLLM_LOSS_ATTRS);

XLA_FFI_DEFINE_HANDLER_SYMBOL(MllmGrpoBwd, BwdImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::Buffer<ffi::BF16>>()  // logits
                                  .Arg<ffi::Buffer<ffi::S32>>()   // chosen ids
                                  .Arg<ffi::Buffer<ffi::F32>>()   // lse
                                  .Arg<ffi::Buffer<ffi::F32>>()   // grad_coef
                                  .Arg<ffi::Buffer<ffi::F32>>()   // total_valid_token_count
                                  .Arg<ffi::Buffer<ffi::F32>>()   // cotangent of the loss
                                  .Ret<ffi::Buffer<ffi::BF16>>()  // dlogits
                                  .Attr<float>("temperature")
                                  .Attr<float>("softcap")
                                  .Attr<int64_t>("scored_rows"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(MllmGrpoScaleGrad, ScaleGradImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::Buffer<ffi::BF16>>()   // dlogits written with cotangent 1
                                  .Arg<ffi::Buffer<ffi::F32>>()    // cotangent of the loss
                                  .Ret<ffi::Buffer<ffi::BF16>>());  // the same buffer

XLA_FFI_DEFINE_HANDLER_SYMBOL(MllmGrpoLogprobs, LogprobsImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::Buffer<ffi::BF16>>()  // logits
                                  .Arg<ffi::Buffer<ffi::S32>>()   // chosen ids
                                  .Ret<ffi::Buffer<ffi::F32>>()   // per_token_logps
                                  .Ret<ffi::Buffer<ffi::F32>>()   // token_entropy
                                  .Ret<ffi::Buffer<ffi::F32>>()   // lse
                                  .Attr<float>("temperature")
                                  .Attr<float>("softcap")
                                  .Attr<int64_t>("scored_rows"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(MllmGrpoEntropyStats, EntropyStatsImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::Buffer<ffi::F32>>()   // token_entropy [B, T]
                                  .Arg<ffi::Buffer<ffi::F32>>()   // mask [B, T]
                                  .Ret<ffi::Buffer<ffi::F32>>()   // entropy [B]
                                  .Ret<ffi::Buffer<ffi::F32>>());  // entropy_loss [B]
