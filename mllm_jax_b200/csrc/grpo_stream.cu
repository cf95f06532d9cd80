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
#include <cstdlib>

#include "grpo_cluster.cuh"
#include "grpo_common.cuh"
#include "grpo_launch.h"
#include "grpo_rowpass.cuh"

namespace grpo {

// MODE: 0 full forward (epilogue + residuals + loss terms), 1 shard partials, 2 log-probs only.
template <int THREADS, int UNROLL, int ENT, bool CAP, int MODE>
__global__ void __launch_bounds__(THREADS) row_stats_kernel(const KernelParams p) {
  __shared__ float red[32];
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
      float4 out = make_float4(st.M, st.S, st.U, mine ? yc : 0.f);
      reinterpret_cast<float4*>(p.partials)[n] = out;
    } else if (MODE == 2) {
      const float lse = st.M + logf(st.S);
      p.per_token_logps[n] = (yc - lse) * inv_temp;
      if (p.lse) p.lse[n] = lse;
      if (ENT != 0 && p.token_entropy) {
        p.token_entropy[n] = (ENT == 1) ? lse - st.U / st.S
                                        : st.M * inv_temp + logf(st.S2) - inv_temp * st.U2 / st.S2;
      }
    } else {
      const TokenOut o = token_epilogue<ENT>(p, n, b, st, yc);
      p.per_token_logps[n] = o.lp;
      if (ENT != 0 && p.token_entropy) p.token_entropy[n] = o.entropy;
      p.lse[n] = o.lse;
      p.grad_coef[n] = o.grad_coef;
      p.loss_terms[n] = o.loss_term;
    }
  }
}

// Merge the shards' partials (max, sumexp, sum e*y, chosen) and run the epilogue.
template <int ENT>
__global__ void __launch_bounds__(256) combine_kernel(const KernelParams p) {
  const int64_t N = p.n_seqs * p.scored_rows;
  const int64_t n = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
  if (n >= N) return;
  const float4* g = reinterpret_cast<const float4*>(p.gathered_partials);
  float M = kNegInit;
  for (int r = 0; r < p.n_shards; ++r) M = fmaxf(M, g[int64_t(r) * N + n].x);
  RowStats st;
  st.M = M;
  st.S = 0.f;
  st.U = 0.f;
  st.S2 = 0.f;
  st.U2 = 0.f;
  float yc = 0.f;
  for (int r = 0; r < p.n_shards; ++r) {
    const float4 q = g[int64_t(r) * N + n];
    const float scl = ex2f((q.x - M) * kLog2e);
    st.S = fmaf(q.y, scl, st.S);
    st.U = fmaf(q.z, scl, st.U);
    yc += q.w;
  }
  const int64_t b = n / p.scored_rows;
  const TokenOut o = token_epilogue<ENT>(p, n, b, st, yc);
  p.per_token_logps[n] = o.lp;
  if (ENT != 0 && p.token_entropy) p.token_entropy[n] = o.entropy;
  p.lse[n] = o.lse;
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

// Backward sweep.  One CTA per logits row (scored or not).
template <int THREADS, int UNROLL, bool CAP>
__global__ void __launch_bounds__(THREADS) dlogits_kernel(const KernelParams p) {
  const int64_t r = blockIdx.x;  // row index over n_seqs*seq_rows
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
  row_pass2<THREADS, UNROLL, CAP, 1>(x16, d16, p.vocab, g, lse, cl, sc, 0);
}

// Forward and backward of a row by the same CTA: the row is read from HBM with an evict_last L2
// policy, reduced, and read again right away (an L2 hit while the number of rows in flight stays
// well inside the 126 MB L2), so the logits cross HBM once.  One CTA per logits row; CTAs per SM
// are capped through the dynamic shared memory request.
template <int THREADS, int UNROLL, int ENT, bool CAP>
__global__ void __launch_bounds__(THREADS) row_two_pass_kernel(const KernelParams p) {
  __shared__ float red[32];
  __shared__ float bc[2];
  const int tid = threadIdx.x;
  const int64_t r = blockIdx.x;
  const int64_t b = r / p.seq_rows;
  const int64_t t = r - b * p.seq_rows;
  const uint16_t* x16 = reinterpret_cast<const uint16_t*>(p.logits + r * p.row_stride);
  uint16_t* d16 = reinterpret_cast<uint16_t*>(p.dlogits + r * p.row_stride);
  const SoftCap sc(CAP ? p.softcap : 1.0f);
  const uint64_t keep = policy_evict_last(), drop = policy_evict_first();
  if (t >= p.scored_rows) {
    row_pass2<THREADS, UNROLL, CAP, 2>(x16, d16, p.vocab, 0.f, 0.f, -1, sc, drop);
    return;
  }
  const int64_t n = b * p.scored_rows + t;
  const RowStats st = row_pass1<THREADS, UNROLL, ENT, CAP, 2>(x16, p.vocab, p.inv_temperature, sc, red, keep);
  int64_t cl = -1;
  if (tid == 0) {
    bool mine;
    const float yc = chosen_logit<CAP>(p, n, x16, sc, &mine, &cl);
    const TokenOut o = token_epilogue<ENT>(p, n, b, st, yc);
    p.per_token_logps[n] = o.lp;
    if (ENT != 0 && p.token_entropy) p.token_entropy[n] = o.entropy;
    p.lse[n] = o.lse;
    p.grad_coef[n] = o.grad_coef;
    p.loss_terms[n] = o.loss_term;
    const float nv = p.total_valid_dev ? *p.total_valid_dev : p.total_valid;
    const float gs = p.grad_scale_dev ? *p.grad_scale_dev : p.grad_scale;
    bc[0] = o.grad_coef * gs / nv;
    bc[1] = o.lse;
  }
  __syncthreads();
  const float g = bc[0], lse = bc[1];
  int64_t c = p.chosen_ids[n];
  c = c < 0 ? 0 : (c >= p.vocab_total ? p.vocab_total - 1 : c);
  cl = c - p.vocab_start;
  row_pass2<THREADS, UNROLL, CAP, 2>(x16, d16, p.vocab, g, lse, cl, sc, drop);
}

// The same two passes with one logits row split over a cluster of CL CTAs (CTA r takes the r-th
// column slice).  Rows in flight drop by CL, so the bytes that pass through L2 between the first and
// the second read of a line shrink to a few tens of MB and the second read is an L2 hit.  The slices'
// (M, S, U, y_c) are pushed into every peer's shared memory and published by one cluster barrier.
// Needs 16-byte aligned rows (vocab and row stride multiples of 8, aligned bases).
template <int CL, int THREADS, int UNROLL, int ENT, bool CAP>
__global__ void __launch_bounds__(THREADS) row_two_pass_cluster_kernel(const KernelParams p, int64_t vec_per) {
  __shared__ float red[32];
  __shared__ float bc[2];
  __shared__ __align__(16) float4 slots[8];
  const int tid = threadIdx.x;
  const uint32_t rank = cl::cluster_rank();
  const int64_t r = cl::cluster_id_x();
  const int64_t b = r / p.seq_rows;
  const int64_t t = r - b * p.seq_rows;
  const int64_t col0 = int64_t(rank) * vec_per * 8;
  int64_t ncol = p.vocab - col0;
  if (ncol > vec_per * 8) ncol = vec_per * 8;
  const uint16_t* x16 = reinterpret_cast<const uint16_t*>(p.logits + r * p.row_stride) + col0;
  uint16_t* d16 = reinterpret_cast<uint16_t*>(p.dlogits + r * p.row_stride) + col0;
  const SoftCap sc(CAP ? p.softcap : 1.0f);
  const uint64_t keep = policy_evict_last(), drop = policy_evict_first();
  if (t >= p.scored_rows) {  // the whole cluster takes this branch together
    row_pass2<THREADS, UNROLL, CAP, 2>(x16, d16, ncol, 0.f, 0.f, -1, sc, drop);
    return;
  }
  // Tell the peers this CTA is running (its shared memory exists) without blocking yet.
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
  const int64_t n = b * p.scored_rows + t;
  const RowStats st = row_pass1<THREADS, UNROLL, ENT, CAP, 2>(x16, ncol, p.inv_temperature, sc, red, keep);
  int64_t c = p.chosen_ids[n];
  if (c < 0 || c >= p.vocab_total) {
    c = c < 0 ? 0 : p.vocab_total - 1;
    if (tid == 0 && rank == 0 && p.device_status) atomicOr(p.device_status, MLLM_GRPO_DEV_ID_CLAMPED);
  }
  const int64_t cl_local = c - p.vocab_start - col0;  // chosen column relative to this slice
  asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
  if (tid < CL) {
    float yc = 0.f;
    if (cl_local >= 0 && cl_local < ncol) {
      yc = __uint_as_float(uint32_t(x16[cl_local]) << 16);
      if (CAP) yc = sc.y(yc);
    }
    cl::st_cluster_f4(cl::map_to_cta(cl::smem_u32(&slots[rank]), tid), make_float4(st.M, st.S, st.U, yc));
  }
  cl::cluster_sync_all();  // release our pushes, acquire everyone else's
  if (tid == 0) {
    RowStats all;
    all.M = kNegInit;
    for (int q = 0; q < CL; ++q) all.M = fmaxf(all.M, slots[q].x);
    all.S = 0.f;
    all.U = 0.f;
    all.S2 = 0.f;
    all.U2 = 0.f;
    float yc = 0.f;
    for (int q = 0; q < CL; ++q) {
      const float4 part = slots[q];
      const float e = ex2f((part.x - all.M) * kLog2e);
      all.S = fmaf(part.y, e, all.S);
      all.U = fmaf(part.z, e, all.U);
      yc += part.w;
    }
    const TokenOut o = token_epilogue<ENT>(p, n, b, all, yc);
    if (rank == 0) {
      p.per_token_logps[n] = o.lp;
      if (ENT != 0 && p.token_entropy) p.token_entropy[n] = o.entropy;
      p.lse[n] = o.lse;
      p.grad_coef[n] = o.grad_coef;
      p.loss_terms[n] = o.loss_term;
    }
    const float nv = p.total_valid_dev ? *p.total_valid_dev : p.total_valid;
    const float gs = p.grad_scale_dev ? *p.grad_scale_dev : p.grad_scale;
    bc[0] = o.grad_coef * gs / nv;
    bc[1] = o.lse;
  }
  __syncthreads();
  row_pass2<THREADS, UNROLL, CAP, 2>(x16, d16, ncol, bc[0], bc[1], cl_local, sc, drop);
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
        const float rr = sc.r(x);
        y = fmaf(-2.0f * sc.cap, rr, sc.cap);
        deriv = 4.0f * rr * (1.0f - rr);
      }
      d = g * ex2f((y - lse) * kLog2e);
      if (j == cl) d -= g;
      d *= deriv;
    }
    d16[j] = __bfloat16_as_ushort(__float2bfloat16_rn(d));
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

namespace {
template <int THREADS, int ENT, bool CAP>
cudaError_t launch_two_pass_t(const KernelParams& p, int ctas_per_sm, cudaStream_t s) {
  auto kern = row_two_pass_kernel<THREADS, 4, ENT, CAP>;
  // A dynamic shared memory request caps the resident CTAs per SM (227 KB per SM in total).
  size_t smem = 0;
  if (ctas_per_sm > 0) {
    smem = size_t(220 * 1024) / size_t(ctas_per_sm) - 1024;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
      if (e != cudaSuccess) return e;
    }
  }
  const int64_t R = p.n_seqs * p.seq_rows;
  kern<<<static_cast<unsigned>(R), THREADS, smem, s>>>(p);
  count_launch();
  return cudaGetLastError();
}
template <int THREADS>
cudaError_t launch_two_pass_th(const KernelParams& p, int ent, int ctas, cudaStream_t s) {
  const bool cap = p.softcap > 0.f;
  if (ent == 0) return cap ? launch_two_pass_t<THREADS, 0, true>(p, ctas, s) : launch_two_pass_t<THREADS, 0, false>(p, ctas, s);
  if (ent == 1) return cap ? launch_two_pass_t<THREADS, 1, true>(p, ctas, s) : launch_two_pass_t<THREADS, 1, false>(p, ctas, s);
  return cap ? launch_two_pass_t<THREADS, 2, true>(p, ctas, s) : launch_two_pass_t<THREADS, 2, false>(p, ctas, s);
}
}  // namespace

namespace {
template <int CL, int THREADS, int UNROLL, int ENT, bool CAP>
cudaError_t launch_two_pass_cluster_t(const KernelParams& p, cudaStream_t s) {
  const int64_t R = p.n_seqs * p.seq_rows;
  const int64_t nvec = p.vocab / 8;
  const int64_t per = (nvec + CL - 1) / CL;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CL;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3(static_cast<unsigned>(R * CL), 1, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = s;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, row_two_pass_cluster_kernel<CL, THREADS, UNROLL, ENT, CAP>, p, per);
  count_launch();
  return e;
}
template <int CL, int THREADS, int UNROLL>
cudaError_t launch_two_pass_cluster_u(const KernelParams& p, int ent, cudaStream_t s) {
  const bool cap = p.softcap > 0.f;
  if (ent == 0)
    return cap ? launch_two_pass_cluster_t<CL, THREADS, UNROLL, 0, true>(p, s)
               : launch_two_pass_cluster_t<CL, THREADS, UNROLL, 0, false>(p, s);
  return cap ? launch_two_pass_cluster_t<CL, THREADS, UNROLL, 1, true>(p, s)
             : launch_two_pass_cluster_t<CL, THREADS, UNROLL, 1, false>(p, s);
}
template <int CL, int THREADS>
cudaError_t launch_two_pass_cluster_c(const KernelParams& p, int ent, int unroll, cudaStream_t s) {
  if (unroll <= 4) return launch_two_pass_cluster_u<CL, THREADS, 4>(p, ent, s);
  return launch_two_pass_cluster_u<CL, THREADS, 8>(p, ent, s);
}
template <int CL>
cudaError_t launch_two_pass_cluster_th(const KernelParams& p, int ent, int threads, int unroll, cudaStream_t s) {
  if (threads <= 128) return launch_two_pass_cluster_c<CL, 128>(p, ent, unroll, s);
  return launch_two_pass_cluster_c<CL, 256>(p, ent, unroll, s);
}
}  // namespace

// Two passes per row with the row split over a cluster.  *taken is false (nothing launched) unless
// rows are 16-byte aligned in both buffers, every slice is non-empty and the entropy mode is 0 or 1.
cudaError_t launch_two_pass_cluster(const KernelParams& p, int ent, int cluster, int threads, cudaStream_t s,
                                    bool* taken) {
  *taken = false;
  if (ent == 2) return cudaSuccess;
  if ((p.vocab & 7) || (p.row_stride & 7)) return cudaSuccess;
  if ((reinterpret_cast<uintptr_t>(p.logits) & 15) || (reinterpret_cast<uintptr_t>(p.dlogits) & 15)) return cudaSuccess;
  const int64_t nvec = p.vocab / 8;
  if (cluster != 2 && cluster != 4 && cluster != 8) return cudaSuccess;
  const int64_t per = (nvec + cluster - 1) / cluster;
  if (nvec - (cluster - 1) * per <= 0) return cudaSuccess;
  if (p.n_seqs * p.seq_rows * cluster >= (int64_t(1) << 31)) return cudaSuccess;
  *taken = true;
  const char* un = std::getenv("MLLM_GRPO_L2_UNROLL");
  const int unroll = un ? std::atoi(un) : 8;
  switch (cluster) {
    case 2: return launch_two_pass_cluster_th<2>(p, ent, threads, unroll, s);
    case 4: return launch_two_pass_cluster_th<4>(p, ent, threads, unroll, s);
    default: return launch_two_pass_cluster_th<8>(p, ent, threads, unroll, s);
  }
}

// Single-kernel forward+backward that relies on L2 for the second read.  *taken is false when
// logits and dlogits rows do not share their 16-byte phase (the caller then runs the two sweeps).
cudaError_t launch_two_pass(const KernelParams& p, int ent, int threads, int ctas_per_sm, cudaStream_t s,
                            bool* taken) {
  const uintptr_t ax = reinterpret_cast<uintptr_t>(p.logits), ad = reinterpret_cast<uintptr_t>(p.dlogits);
  *taken = ((ax ^ ad) & 15) == 0;
  if (!*taken) return cudaSuccess;
  if (threads >= 1024) return launch_two_pass_th<1024>(p, ent, ctas_per_sm, s);
  return launch_two_pass_th<512>(p, ent, ctas_per_sm, s);
}

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
  else
    combine_kernel<1><<<grid, 256, 0, s>>>(p);
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
  } else if (cap) {
    dlogits_kernel<kBwdThreads, kBwdUnroll, true><<<static_cast<unsigned>(R), kBwdThreads, 0, s>>>(p);
  } else {
    dlogits_kernel<kBwdThreads, kBwdUnroll, false><<<static_cast<unsigned>(R), kBwdThreads, 0, s>>>(p);
  }
  count_launch();
  return cudaGetLastError();
}

}  // namespace grpo
