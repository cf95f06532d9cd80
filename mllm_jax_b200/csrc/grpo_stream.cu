// Streaming kernels of the fused GRPO token loss that work for ANY vocabulary
// size, row stride and base alignment: 128-bit read-only loads over the aligned
// body of each row, scalar loads for the ragged head and tail.
//
//   row_stats_kernel  : one CTA per scored token; one pass over the row gives
//                       (M, S, U) by an online max / sum-exp, then either the
//                       per-token epilogue (full rows) or the shard's partials.
//   combine_kernel    : merges the partials of all vocabulary shards, runs the epilogue.
//   loss_reduce_kernel: fixed-order sum of the per-token loss terms / total_valid.
//   dlogits_kernel    : one CTA per logits row; second streaming pass writing
//                       g*(softmax - onehot) in bf16; zero rows are write-only.
//   scale_grad_kernel : applies a late cotangent to gradients written with cotangent 1
//                       (returns at once when it is exactly 1).
#include "grpo_common.cuh"
#include "grpo_launch.h"
#include "grpo_rowpass.cuh"

namespace grpo {

// MODE: 0 full forward (epilogue + residuals + loss terms), 1 shard partials, 2 log-probs only.
template <int THREADS, int UNROLL, int ENT, bool CAP, int MODE>
__global__ void __launch_bounds__(THREADS) row_stats_kernel(const KernelParams p) {
  __shared__ float red[160];
  const int tid = threadIdx.x;
  const int64_t n = blockIdx.x;  // scored token index
  const int64_t b = n / p.scored_rows;
  const int64_t t = n - b * p.scored_rows;
  const uint16_t* row16 = reinterpret_cast<const uint16_t*>(p.logits + (b * p.seq_rows + t) * p.row_stride);
  const int64_t V = p.vocab;
  const float inv_temp = p.inv_temperature;
  const SoftCap sc(CAP ? p.softcap : 1.0f);
  const RowStats st = row_pass1<THREADS, UNROLL, ENT, CAP, 0>(row16, V, inv_temp, sc, red, 0);

  if (tid == 0) {
    bool mine;
    int64_t cl;
    const float yc = chosen_logit<CAP>(p, n, row16, sc, &mine, &cl);
    if (MODE == 1) {
      if (ENT == 2) {
        // temperature != 1 with the entropy: two more sums, on y/temperature (records of 6 floats)
        float* rec = p.partials + n * 6;
        rec[0] = st.M;
        rec[1] = st.S;
        rec[2] = 0.f;
        rec[3] = mine ? yc : 0.f;
        rec[4] = st.S2;
        rec[5] = st.U2;
      } else {
        reinterpret_cast<float4*>(p.partials)[n] = make_float4(st.M, st.S, st.U, mine ? yc : 0.f);
      }
    } else if (MODE == 2) {
      const float lse = st.M + logf(st.S);
      p.per_token_logps[n] = (yc - lse) * inv_temp;
      if (p.lse) p.lse[n] = lse;
      if (p.lse_scaled) p.lse_scaled[n] = scaled_lse<ENT>(p, st, lse);
      if (ENT != 0 && p.token_entropy) {
        p.token_entropy[n] = (ENT == 1) ? lse - st.U / st.S
                                        : st.M * inv_temp + logf(st.S2) - inv_temp * st.U2 / st.S2;
      }
    } else {
      const TokenOut o = token_epilogue<ENT>(p, n, b, st, yc);
      p.per_token_logps[n] = o.lp;
      if (ENT != 0 && p.token_entropy) p.token_entropy[n] = o.entropy;
      p.lse[n] = o.lse;
      if (p.lse_scaled) p.lse_scaled[n] = scaled_lse<ENT>(p, st, o.lse);
      p.grad_coef[n] = o.grad_coef;
      p.loss_terms[n] = o.loss_term;
    }
  }
}

// Merge the shards' partials (max, sumexp, sum e*y, chosen; for ENT == 2 also the two sums on y/temperature,
// records of 6 floats) and run the epilogue.
template <int ENT>
__global__ void __launch_bounds__(256) combine_kernel(const KernelParams p) {
  const int64_t N = p.n_seqs * p.scored_rows;
  const int64_t n = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
  if (n >= N) return;
  constexpr int W = ENT == 2 ? 6 : 4;
  const float* g = p.gathered_partials;
  float M = kNegInit;
  for (int r = 0; r < p.n_shards; ++r) M = fmaxf(M, g[(int64_t(r) * N + n) * W]);
  RowStats st;
  st.M = M;
  st.S = 0.f;
  st.U = 0.f;
  st.S2 = 0.f;
  st.U2 = 0.f;
  float yc = 0.f;
  for (int r = 0; r < p.n_shards; ++r) {
    const float* q = g + (int64_t(r) * N + n) * W;
    const float d = (q[0] - M) * kLog2e;
    const float scl = ex2f(d);
    st.S = fmaf(q[1], scl, st.S);
    st.U = fmaf(q[2], scl, st.U);
    yc += q[3];
    if (ENT == 2) {
      const float scl2 = ex2f(d * p.inv_temperature);
      st.S2 = fmaf(q[4], scl2, st.S2);
      st.U2 = fmaf(q[5], scl2, st.U2);
    }
  }
  const int64_t b = n / p.scored_rows;
  const TokenOut o = token_epilogue<ENT>(p, n, b, st, yc);
  p.per_token_logps[n] = o.lp;
  if (ENT != 0 && p.token_entropy) p.token_entropy[n] = o.entropy;
  p.lse[n] = o.lse;
  if (p.lse_scaled) p.lse_scaled[n] = scaled_lse<ENT>(p, st, o.lse);
  p.grad_coef[n] = o.grad_coef;
  p.loss_terms[n] = o.loss_term;
}

// loss = (sum of loss_terms in a fixed order, accumulated in f64) / total_valid.
__global__ void __launch_bounds__(1024) loss_reduce_kernel(const KernelParams p) {
  __shared__ double part[1024];
  const int64_t N = p.n_seqs * p.scored_rows;
  double a = 0.0;
  for (int64_t i = threadIdx.x; i < N; i += 1024) a += double(p.loss_terms[i]);
  part[threadIdx.x] = a;
  __syncthreads();
  for (int s = 512; s > 0; s >>= 1) {
    if (threadIdx.x < s) part[threadIdx.x] += part[threadIdx.x + s];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const float nv = p.total_valid_dev ? *p.total_valid_dev : p.total_valid;
    *p.loss = float(part[0] / double(nv));
  }
}

// Backward sweep.  One CTA per logits row (scored or not).  ENTG: the cotangent of the token entropies
// is folded in as well (the -entropy_coef * entropy term of plugins/training/ppo/module.py:140).
template <int THREADS, int UNROLL, bool CAP, bool ENTG>
__global__ void __launch_bounds__(THREADS) dlogits_kernel(const KernelParams p) {
  const int64_t r = blockIdx.x;  // row index over n_seqs*seq_rows
  const int64_t b = r / p.seq_rows;
  const int64_t t = r - b * p.seq_rows;
  const uint16_t* x16 = reinterpret_cast<const uint16_t*>(p.logits + r * p.row_stride);
  uint16_t* d16 = reinterpret_cast<uint16_t*>(p.dlogits + r * p.row_stride);
  float g = 0.f, lse = 0.f;
  int64_t cl = -1;
  EntropyGrad eg{0.f, 0.f, 0.f, 1.f};
  if (t < p.scored_rows) {
    const int64_t n = b * p.scored_rows + t;
    const float nv = p.total_valid_dev ? *p.total_valid_dev : p.total_valid;
    const float gs = p.grad_scale_dev ? *p.grad_scale_dev : p.grad_scale;
    g = p.grad_coef[n] * gs / nv;
    lse = p.lse[n];
    int64_t c = p.chosen_ids[n];
    c = c < 0 ? 0 : (c >= p.vocab_total ? p.vocab_total - 1 : c);
    cl = c - p.vocab_start;
    if (ENTG) {
      eg.cot = p.entropy_cotangent[n];  // a cotangent of its own: grad_scale belongs to the loss
      eg.H = p.token_entropy[n];
      eg.lse2 = p.lse_scaled ? p.lse_scaled[n] : lse;
      eg.inv_temp = p.inv_temperature;
    }
  }
  const SoftCap sc(CAP ? p.softcap : 1.0f);
  row_pass2<THREADS, UNROLL, CAP, 1, -1, ENTG>(x16, d16, p.vocab, g, lse, cl, sc, 0, eg);
}

// Any-alignment fallback for the rare case where logits and dlogits rows do not share
// their offset from a 16-byte boundary: scalar loads and stores.
template <bool CAP>
__global__ void __launch_bounds__(256) dlogits_scalar_kernel(const KernelParams p) {
  const int64_t r = blockIdx.x;
  const int64_t b = r / p.seq_rows;
  const int64_t t = r - b * p.seq_rows;
  const uint16_t* x16 = reinterpret_cast<const uint16_t*>(p.logits + r * p.row_stride);
  uint16_t* d16 = reinterpret_cast<uint16_t*>(p.dlogits + r * p.row_stride);
  float g = 0.f, lse = 0.f;
  int64_t cl = -1;
  if (t < p.scored_rows) {
    const int64_t n = b * p.scored_rows + t;
    const float nv = p.total_valid_dev ? *p.total_valid_dev : p.total_valid;
    const float gs = p.grad_scale_dev ? *p.grad_scale_dev : p.grad_scale;
    g = p.grad_coef[n] * gs / nv;
    lse = p.lse[n];
    int64_t c = p.chosen_ids[n];
    c = c < 0 ? 0 : (c >= p.vocab_total ? p.vocab_total - 1 : c);
    cl = c - p.vocab_start;
  }
  const SoftCap sc(CAP ? p.softcap : 1.0f);
  for (int64_t j = threadIdx.x; j < p.vocab; j += blockDim.x) {
    float d = 0.f;
    if (g != 0.f) {
      const float x = __uint_as_float(uint32_t(x16[j]) << 16);
      float y = x, deriv = 1.f;
      if (CAP) {
        y = sc.y(x);
        deriv = sc.dydx(y);
      }
      d = g * ex2f((y - lse) * kLog2e);
      if (j == cl) d -= g;
      d *= deriv;
    }
    d16[j] = __bfloat16_as_ushort(__float2bfloat16_rn(d));
  }
}

// dlogits *= g for a cotangent that arrives after the gradient was written with g = 1; a no-op
// (one scalar load per CTA) when g == 1.
__global__ void __launch_bounds__(256) scale_grad_kernel(const KernelParams p) {
  const float g = p.grad_scale_dev ? *p.grad_scale_dev : p.grad_scale;
  if (g == 1.0f) return;
  uint16_t* d16 = reinterpret_cast<uint16_t*>(p.dlogits + int64_t(blockIdx.x) * p.row_stride);
  for (int64_t j = threadIdx.x; j < p.vocab; j += blockDim.x) {
    const float v = __uint_as_float(uint32_t(d16[j]) << 16) * g;
    d16[j] = __bfloat16_as_ushort(__float2bfloat16_rn(v));
  }
}

// ---------------------------------------------------------------------------------------------
// Host-side launchers
// ---------------------------------------------------------------------------------------------
namespace {
constexpr int kStatsThreads = 512;
constexpr int kStatsUnroll = 4;
constexpr int kBwdThreads = 512;
constexpr int kBwdUnroll = 4;

template <int MODE, int ENT, bool CAP>
cudaError_t launch_stats_t(const KernelParams& p, cudaStream_t s) {
  const int64_t N = p.n_seqs * p.scored_rows;
  row_stats_kernel<kStatsThreads, kStatsUnroll, ENT, CAP, MODE>
      <<<static_cast<unsigned>(N), kStatsThreads, 0, s>>>(p);
  count_launch();
  return cudaGetLastError();
}
template <int MODE>
cudaError_t launch_stats_m(const KernelParams& p, int ent, cudaStream_t s) {
  const bool cap = p.softcap > 0.f;
  if (ent == 0) return cap ? launch_stats_t<MODE, 0, true>(p, s) : launch_stats_t<MODE, 0, false>(p, s);
  if (ent == 1) return cap ? launch_stats_t<MODE, 1, true>(p, s) : launch_stats_t<MODE, 1, false>(p, s);
  return cap ? launch_stats_t<MODE, 2, true>(p, s) : launch_stats_t<MODE, 2, false>(p, s);
}
}  // namespace

cudaError_t launch_row_stats(const KernelParams& p, int mode, int ent, cudaStream_t s) {
  if (mode == 0) return launch_stats_m<0>(p, ent, s);
  if (mode == 1) return launch_stats_m<1>(p, ent, s);
  return launch_stats_m<2>(p, ent, s);
}

cudaError_t launch_combine(const KernelParams& p, int ent, cudaStream_t s) {
  const int64_t N = p.n_seqs * p.scored_rows;
  const unsigned grid = static_cast<unsigned>((N + 255) / 256);
  if (ent == 0)
    combine_kernel<0><<<grid, 256, 0, s>>>(p);
  else if (ent == 1)
    combine_kernel<1><<<grid, 256, 0, s>>>(p);
  else
    combine_kernel<2><<<grid, 256, 0, s>>>(p);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_scale_grad(const KernelParams& p, cudaStream_t s) {
  scale_grad_kernel<<<static_cast<unsigned>(p.n_seqs * p.seq_rows), 256, 0, s>>>(p);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_loss_reduce(const KernelParams& p, cudaStream_t s) {
  loss_reduce_kernel<<<1, 1024, 0, s>>>(p);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_dlogits(const KernelParams& p, cudaStream_t s) {
  const int64_t R = p.n_seqs * p.seq_rows;
  const bool cap = p.softcap > 0.f;
  const uintptr_t ax = reinterpret_cast<uintptr_t>(p.logits), ad = reinterpret_cast<uintptr_t>(p.dlogits);
  const bool same_phase = ((ax ^ ad) & 15) == 0;
  if (!same_phase) {
    if (cap)
      dlogits_scalar_kernel<true><<<static_cast<unsigned>(R), 256, 0, s>>>(p);
    else
      dlogits_scalar_kernel<false><<<static_cast<unsigned>(R), 256, 0, s>>>(p);
  } else if (p.entropy_cotangent) {
    if (cap)
      dlogits_kernel<kBwdThreads, kBwdUnroll, true, true><<<static_cast<unsigned>(R), kBwdThreads, 0, s>>>(p);
    else
      dlogits_kernel<kBwdThreads, kBwdUnroll, false, true><<<static_cast<unsigned>(R), kBwdThreads, 0, s>>>(p);
  } else if (cap) {
    dlogits_kernel<kBwdThreads, kBwdUnroll, true, false><<<static_cast<unsigned>(R), kBwdThreads, 0, s>>>(p);
  } else {
    dlogits_kernel<kBwdThreads, kBwdUnroll, false, false><<<static_cast<unsigned>(R), kBwdThreads, 0, s>>>(p);
  }
  count_launch();
  return cudaGetLastError();
}

}  // namespace grpo
