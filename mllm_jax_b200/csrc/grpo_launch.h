// Internal interface between the C-ABI layer (grpo_api.cu) and the kernel files.
#pragma once

#include <cuda_runtime.h>

#include "../../include/mllm_grpo.h"
#include "grpo_common.cuh"

namespace grpo {

// Bumps the process-wide count of kernels launched by this library.
void count_launch();
// Stores the error's text for mllm_grpo_last_cuda_error() and returns MLLM_GRPO_ERR_LAUNCH.
int record_cuda_error(cudaError_t e);

// mode: 0 full forward, 1 shard partials, 2 log-probs only.  ent: 0 none, 1 temperature == 1, 2 otherwise.
cudaError_t launch_row_stats(const KernelParams& p, int mode, int ent, cudaStream_t s);
cudaError_t launch_combine(const KernelParams& p, int ent, cudaStream_t s);
cudaError_t launch_loss_reduce(const KernelParams& p, cudaStream_t s);
cudaError_t launch_dlogits(const KernelParams& p, cudaStream_t s);
cudaError_t launch_scale_grad(const KernelParams& p, cudaStream_t s);
// One-kernel forward+backward whose second read of a row is served by L2 (grpo_twopass.cu); long
// rows are split over a cluster, and with sharded == true the vocabulary shards' partials are
// exchanged over NVLink inside the kernel.  *taken is false (nothing launched) when logits and
// dlogits rows do not share their 16-byte phase.
cudaError_t launch_two_pass(const KernelParams& p, int ent, bool sharded, cudaStream_t s, bool* taken);
// Per-sample entropy monitors (grpo_monitors.cu).
cudaError_t launch_entropy_stats(const float* H, const float* mask, int64_t B, int64_t T, float* ent, float* ent_win,
                                 cudaStream_t s);
// The two kernel families behind launch_two_pass, one translation unit each.
cudaError_t launch_two_pass_unsharded(const KernelParams& p, int ent, int cluster, int threads, int unroll, bool smem,
                                      cudaStream_t s);
cudaError_t launch_two_pass_sharded(const KernelParams& p, int ent, int cluster, int threads, int unroll, bool smem,
                                    cudaStream_t s);
// Forced plan of launch_two_pass (tuning / test hook); 0 (-1 for staged) = automatic.
void set_two_pass_override(int cluster, int threads, int load_batch, int staged);

}  // namespace grpo
