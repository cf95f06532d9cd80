// Value-loss tail of the PPO actor-critic module (plugins/training/ppo/module.py:104-140):
//   value_pred = values[:, :-1];  returns = given, else advantages + value_pred (:105-107)
//   old_values = given, else stop_gradient(value_pred) (:116-118)
//   clipped    = old + clip(value_pred - old, -c, c);  term = max((v - r)^2, (clipped - r)^2)   (:131-134)
//   value_loss = sum(term * mask) / total_valid_token_count                                     (:138)
// plus the monitors value_pred_mean and return_mean (:147-148) and the gradient with respect to the
// values.  [B, L] elementwise work: one thread per position, per-block sums in double precision,
// a single CTA adds the blocks in a fixed order (the result does not depend on scheduling).
#include "grpo_common.cuh"
#include "grpo_launch.h"

namespace grpo {

constexpr int kValThreads = 256;

struct ValueParams {
  int64_t n_seqs, seq_rows, scored_rows;
  float clip, grad_scale, total_valid;
  int adv_per_token;
  const float* total_valid_dev;
  const float* values;
  const float* returns;
  const float* advantages;
  const float* old_values;
  const float* mask;
  float* dvalues;
  float* out;
  double* work;
};

__device__ __forceinline__ double warp_sum_f64(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void __launch_bounds__(kValThreads) value_terms_kernel(const ValueParams p) {
  __shared__ double red[3][kValThreads / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t R = p.n_seqs * p.seq_rows;
  const int64_t i = int64_t(blockIdx.x) * kValThreads + tid;
  double s_loss = 0.0, s_v = 0.0, s_r = 0.0;
  if (i < R) {
    const int64_t b = i / p.seq_rows, t = i - b * p.seq_rows;
    float grad = 0.f;
    if (t < p.scored_rows) {
      const int64_t n = b * p.scored_rows + t;
      const float v = p.values[i];
      const float m = p.mask ? p.mask[n] : 1.0f;
      // returns default to advantages + value_pred and then move with the values (dr = 1)
      const bool own_returns = p.returns != nullptr;
      const float r = own_returns ? p.returns[n] : (p.adv_per_token ? p.advantages[n] : p.advantages[b]) + v;
      const float dr = own_returns ? 0.f : 1.f;
      const float e1 = v - r;
      float term = e1 * e1;
      float g = 2.f * e1 * (1.f - dr);
      if (p.clip >= 0.f) {
        const float old = p.old_values ? p.old_values[n] : v;
        const float d = v - old;
        const bool inside = d >= -p.clip && d <= p.clip;
        const float vc = old + fminf(fmaxf(d, -p.clip), p.clip);
        const float e2 = vc - r;
        const float term2 = e2 * e2;
        const float g2 = 2.f * e2 * ((inside ? 1.f : 0.f) - dr);
        if (term2 > term) {
          term = term2;
          g = g2;
        } else if (term2 == term) {
          g = 0.5f * (g + g2);  // a tie of maximum() passes half of each side
        }
      }
      const float nv = p.total_valid_dev ? *p.total_valid_dev : p.total_valid;
      grad = p.grad_scale * m * g / nv;
      s_loss = double(term) * double(m);
      s_v = double(v);
      s_r = double(r);
    }
    if (p.dvalues) p.dvalues[i] = grad;
  }
  double v3[3] = {s_loss, s_v, s_r};
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    v3[k] = warp_sum_f64(v3[k]);
    if (lane == 0) red[k][warp] = v3[k];
  }
  __syncthreads();
  if (tid < 3) {
    double tot = 0.0;
    for (int w = 0; w < kValThreads / 32; ++w) tot += red[tid][w];
    p.work[int64_t(blockIdx.x) * 3 + tid] = tot;
  }
}

__global__ void __launch_bounds__(kValThreads) value_finish_kernel(const ValueParams p, const int64_t n_blocks) {
  __shared__ double red[3][kValThreads];
  const int tid = threadIdx.x;
  double acc[3] = {0.0, 0.0, 0.0};
  for (int64_t j = tid; j < n_blocks; j += kValThreads)
    for (int k = 0; k < 3; ++k) acc[k] += p.work[j * 3 + k];
  for (int k = 0; k < 3; ++k) red[k][tid] = acc[k];
  __syncthreads();
  for (int o = kValThreads / 2; o > 0; o >>= 1) {
    if (tid < o)
      for (int k = 0; k < 3; ++k) red[k][tid] += red[k][tid + o];
    __syncthreads();
  }
  if (tid == 0) {
    const float nv = p.total_valid_dev ? *p.total_valid_dev : p.total_valid;
    const double count = double(p.n_seqs) * double(p.scored_rows);
    p.out[0] = float(red[0][0] / double(nv));
    p.out[1] = float(red[1][0] / count);
    p.out[2] = float(red[2][0] / count);
  }
}

static int64_t value_blocks(int64_t positions) { return (positions + kValThreads - 1) / kValThreads; }

}  // namespace grpo

using namespace grpo;

extern "C" {

int64_t mllm_ppo_value_workspace_bytes(int64_t n_seqs, int64_t seq_rows) {
  if (n_seqs <= 0 || seq_rows <= 0) return 0;
  return value_blocks(n_seqs * seq_rows) * 3 * int64_t(sizeof(double));
}

int mllm_ppo_value_loss(const mllm_ppo_value_args* a, void* stream) {
  if (a == nullptr) return MLLM_GRPO_ERR_NULL_POINTER;
  if (a->struct_size != sizeof(mllm_ppo_value_args)) return MLLM_GRPO_ERR_STRUCT_SIZE;
  if (a->n_seqs <= 0 || a->seq_rows <= 0 || a->scored_rows <= 0 || a->scored_rows > a->seq_rows)
    return MLLM_GRPO_ERR_BAD_SHAPE;
  if (a->n_seqs * a->seq_rows >= (int64_t(1) << 31) * kValThreads) return MLLM_GRPO_ERR_TOO_LARGE;
  if (!a->values || !a->out || !a->workspace) return MLLM_GRPO_ERR_NULL_POINTER;
  if (!a->returns && !a->advantages) return MLLM_GRPO_ERR_NULL_POINTER;
  if (!a->total_valid_dev && !(a->total_valid == a->total_valid)) return MLLM_GRPO_ERR_BAD_ATTRIBUTE;
  if (a->clip_range != a->clip_range || a->grad_scale != a->grad_scale) return MLLM_GRPO_ERR_BAD_ATTRIBUTE;
  const void* f32s[] = {a->values, a->returns, a->advantages, a->old_values, a->mask, a->dvalues, a->out,
                        a->total_valid_dev};
  for (const void* q : f32s)
    if (reinterpret_cast<uintptr_t>(q) & 3) return MLLM_GRPO_ERR_ALIGNMENT;
  if (reinterpret_cast<uintptr_t>(a->workspace) & 7) return MLLM_GRPO_ERR_ALIGNMENT;

  ValueParams p;
  p.n_seqs = a->n_seqs;
  p.seq_rows = a->seq_rows;
  p.scored_rows = a->scored_rows;
  p.clip = a->clip_range;
  p.grad_scale = a->grad_scale;
  p.total_valid = a->total_valid;
  p.adv_per_token = a->adv_per_token;
  p.total_valid_dev = a->total_valid_dev;
  p.values = a->values;
  p.returns = a->returns;
  p.advantages = a->advantages;
  p.old_values = a->old_values;
  p.mask = a->mask;
  p.dvalues = a->dvalues;
  p.out = a->out;
  p.work = a->workspace;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t blocks = value_blocks(a->n_seqs * a->seq_rows);
  value_terms_kernel<<<static_cast<unsigned>(blocks), kValThreads, 0, s>>>(p);
  count_launch();
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) {
    value_finish_kernel<<<1, kValThreads, 0, s>>>(p, blocks);
    count_launch();
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) return record_cuda_error(e);
  return MLLM_GRPO_OK;
}

}  // extern "C"
