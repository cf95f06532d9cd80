// mllm_grpo_fwd_static_scratch: the forward of the loss for callers that cannot hand the
// library a scratch buffer and cannot allocate one either.
//
// Who that is: code that runs inside someone else's memory plan.  An XLA custom-call handler,
// for example, only ever sees the operand and result buffers the compiler laid out for it; if the
// call site did not declare an extra result to serve as workspace there is nothing to pass as
// `loss_terms`, and calling cudaMalloc from the handler is off the table (it synchronises the
// device and takes memory behind the back of the framework's own pool).  The same holds for a
// serving loop that promised "no allocator calls after start-up" to keep its latency bounded.
//
// What it does instead: the per-token loss terms go to a fixed array that lives in the library's
// own device image.  The array costs MLLM_GRPO_STATIC_SCRATCH_TOKENS * 4 bytes (4 MiB) on every
// GPU that loads the library, for as long as the process lives.  Its name is only a handle on the
// host; the device address is looked up once per device with cudaGetSymbolAddress and cached.
#include <mutex>

#include "grpo_launch.h"

namespace {

__device__ __align__(256) float g_static_loss_terms[MLLM_GRPO_STATIC_SCRATCH_TOKENS];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
float* g_scratch_ptr[kMaxDevices] = {nullptr};

// Device address of the array on the CURRENT device; resolved on first use per device.
int static_scratch(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return MLLM_GRPO_ERR_NO_DEVICE;
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_loss_terms);
    if (e != cudaSuccess || p == nullptr) {
      (void)cudaGetLastError();
      return MLLM_GRPO_ERR_LAUNCH;
    }
    g_scratch_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_scratch_ptr[dev];
  return MLLM_GRPO_OK;
}

}  // namespace

extern "C" int mllm_grpo_fwd_static_scratch(const mllm_grpo_args* args, void* stream) {
  if (args == nullptr) return MLLM_GRPO_ERR_NULL_POINTER;
  if (args->struct_size != sizeof(mllm_grpo_args)) return MLLM_GRPO_ERR_STRUCT_SIZE;
  if (args->n_seqs <= 0 || args->scored_rows <= 0) return MLLM_GRPO_ERR_BAD_SHAPE;
  // n_seqs * scored_rows without overflow
  if (args->n_seqs > MLLM_GRPO_STATIC_SCRATCH_TOKENS || args->scored_rows > MLLM_GRPO_STATIC_SCRATCH_TOKENS ||
      args->n_seqs * args->scored_rows > MLLM_GRPO_STATIC_SCRATCH_TOKENS)
    return MLLM_GRPO_ERR_TOO_LARGE;
  float* scratch = nullptr;
  const int st = static_scratch(&scratch);
  if (st != MLLM_GRPO_OK) return st;
  mllm_grpo_args with_scratch = *args;
  with_scratch.loss_terms = scratch;  // every token below n_seqs*scored_rows is overwritten; nothing needs clearing
  return mllm_grpo_fwd(&with_scratch, stream);
}
