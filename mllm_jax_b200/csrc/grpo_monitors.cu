// Per-sample entropy monitors of the reference's return dict (MLLM_JAX/train_modules/__init__.py:141-157):
//   entropy[b]      = sum_t H_t*m_t / sum_t m_t
//   entropy_loss[b] = mean of H_t over valid tokens (m_t == 1) whose running count of valid tokens in
//                     the sample lies in [4, 100]
// One CTA per sample; every thread owns a contiguous run of positions, a block scan of the runs'
// valid counts gives each run its starting count, and four block sums finish the job in a fixed order.
#include "grpo_common.cuh"
#include "grpo_launch.h"

namespace grpo {

constexpr int kMonThreads = 256;

__global__ void __launch_bounds__(kMonThreads) entropy_stats_kernel(const float* __restrict__ H,
                                                                    const float* __restrict__ mask, int64_t T,
                                                                    float* __restrict__ ent, float* __restrict__ ent_win) {
  __shared__ int warp_counts[kMonThreads / 32];
  __shared__ float red[4][kMonThreads / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t b = blockIdx.x;
  const float* h = H + b * T;
  const float* m = mask + b * T;
  const int64_t per = (T + kMonThreads - 1) / kMonThreads;
  const int64_t lo = tid * per, hi = (lo + per < T) ? lo + per : T;

  int mine = 0;
  for (int64_t t = lo; t < hi; ++t) mine += (m[t] == 1.0f);
  // exclusive block scan of `mine`
  int incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) warp_counts[warp] = incl;
  __syncthreads();
  int base = 0;
  for (int w = 0; w < warp; ++w) base += warp_counts[w];
  int cum = base + incl - mine;  // valid tokens before this thread's run

  float s_all = 0.f, c_all = 0.f, s_win = 0.f, c_win = 0.f;
  for (int64_t t = lo; t < hi; ++t) {
    const float mt = m[t], ht = h[t];
    s_all = fmaf(ht, mt, s_all);
    c_all += mt;
    if (mt == 1.0f) {
      ++cum;
      if (cum >= 4 && cum <= 100) {
        s_win += ht;
        c_win += 1.0f;
      }
    }
  }
  float v[4] = {s_all, c_all, s_win, c_win};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    v[k] = warp_sum(v[k]);
    if (lane == 0) red[k][warp] = v[k];
  }
  __syncthreads();
  if (tid == 0) {
    float tot[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < 4; ++k)
      for (int w = 0; w < kMonThreads / 32; ++w) tot[k] += red[k][w];
    ent[b] = tot[0] / tot[1];
    ent_win[b] = tot[2] / tot[3];
  }
}

cudaError_t launch_entropy_stats(const float* H, const float* mask, int64_t B, int64_t T, float* ent, float* ent_win,
                                 cudaStream_t s) {
  entropy_stats_kernel<<<static_cast<unsigned>(B), kMonThreads, 0, s>>>(H, mask, T, ent, ent_win);
  count_launch();
  return cudaGetLastError();
}

}  // namespace grpo
