// The vocabulary-sharded family of the one-kernel forward + backward (exchange over NVLink inside the kernel),
// in a translation unit of its own so that it compiles beside the unsharded family.
#include "grpo_twopass_impl.cuh"

namespace grpo {

cudaError_t launch_two_pass_sharded(const KernelParams& p, int ent, int cluster, int threads, int unroll, bool smem,
                                    cudaStream_t s) {
  return launch_two_pass_family<true>(p, ent, cluster, threads, unroll, smem, s);
}

}  // namespace grpo
