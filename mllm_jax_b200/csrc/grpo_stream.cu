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
#include "grpo_common.cuh"
#include "grpo_launch.h"

namespace grpo {

// ---------------------------------------------------------------------------------------------
// Row geometry: split a row of V bf16 starting at `row` into a scalar head (until the first
// 16-byte boundary), nvec aligned 8-element vectors and a scalar tail.
// ---------------------------------------------------------------------------------------------
struct RowSplit {
  int head, tail;
  int64_t nvec;
  __device__ __forceinline__ RowSplit(const void* row, int64_t V) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(row);
    int64_t h = ((16 - (a & 15)) & 15) >> 1;
    if (h > V) h = V;
    head = static_cast<int>(h);
    nvec = (V - h) >> 3;
    tail = static_cast<int>(V - h - (nvec << 3));
  }
};

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// Coherent variant for the backward pass, whose output may alias its input.
__device__ __forceinline__ uint4 ldg_stream_rw(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void stg_stream(uint4* p, const uint4& v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

template <int THREADS>
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();  // protect `red` from the previous use
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = (lane < THREADS / 32) ? red[lane] : kNegInit;
  return warp_max(r);
}
template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = (lane < THREADS / 32) ? red[lane] : 0.f;
  return warp_sum(r);
}

// Fold a batch of NV vectors into the accumulator.
template <int ENT, bool CAP, int NV>
__device__ __forceinline__ void fold_vectors(RowAcc<ENT>& acc, const uint4 (&v)[NV], float inv_temp,
                                             float k2, const SoftCap& sc) {
  uint32_t mx2 = v[0].x;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (i) mx2 = bf16x2_max(mx2, v[i].x);
    mx2 = bf16x2_max(mx2, v[i].y);
    mx2 = bf16x2_max(mx2, v[i].z);
    mx2 = bf16x2_max(mx2, v[i].w);
  }
  float mx = fmaxf(bf16lo(mx2), bf16hi(mx2));
  if (CAP) mx = sc.y(mx);  // tanh is monotonic: max of capped values = capped max
  if (mx > acc.m) acc.raise(mx, inv_temp);
  const float mk = acc.m * kLog2e;
  const float mk2 = mk * inv_temp;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float a = bf16lo(w[j]), b = bf16hi(w[j]);
      if (CAP) {
        a = sc.y(a);
        b = sc.y(b);
      }
      acc.add(a, mk, k2, mk2);
      acc.add(b, mk, k2, mk2);
    }
  }
}

template <int ENT, bool CAP>
__device__ __forceinline__ void fold_scalar(RowAcc<ENT>& acc, float x, float inv_temp, float k2,
                                            const SoftCap& sc) {
  const float y = CAP ? sc.y(x) : x;
  if (y > acc.m) acc.raise(y, inv_temp);
  const float mk = acc.m * kLog2e;
  acc.add(y, mk, k2, mk * inv_temp);
}

// MODE: 0 full forward (epilogue + residuals + loss terms), 1 shard partials, 2 log-probs only.
template <int THREADS, int UNROLL, int ENT, bool CAP, int MODE>
__global__ void __launch_bounds__(THREADS) row_stats_kernel(const KernelParams p) {
  __shared__ float red[32];
  const int tid = threadIdx.x;
  const int64_t n = blockIdx.x;  // scored token index
  const int64_t b = n / p.scored_rows;
  const int64_t t = n - b * p.scored_rows;
  const __nv_bfloat16* row = p.logits + (b * p.seq_rows + t) * p.row_stride;
  const int64_t V = p.vocab;
  const float inv_temp = p.inv_temperature;
  const float k2 = kLog2e * inv_temp;
  const SoftCap sc(CAP ? p.softcap : 1.0f);

  RowAcc<ENT> acc;
  acc.init();

  const RowSplit sp(row, V);
  const uint16_t* row16 = reinterpret_cast<const uint16_t*>(row);
  if (tid < sp.head) {
    fold_scalar<ENT, CAP>(acc, __uint_as_float(uint32_t(row16[tid]) << 16), inv_temp, k2, sc);
  }
  if (tid < sp.tail) {
    const int64_t j = sp.head + (sp.nvec << 3) + tid;
    fold_scalar<ENT, CAP>(acc, __uint_as_float(uint32_t(row16[j]) << 16), inv_temp, k2, sc);
  }
  const uint4* vec = reinterpret_cast<const uint4*>(row16 + sp.head);
  int64_t i = tid;
  for (; i + int64_t(UNROLL - 1) * THREADS < sp.nvec; i += int64_t(UNROLL) * THREADS) {
    uint4 v[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) v[u] = ldg_stream(vec + i + int64_t(u) * THREADS);
    fold_vectors<ENT, CAP, UNROLL>(acc, v, inv_temp, k2, sc);
  }
  for (; i < sp.nvec; i += THREADS) {
    uint4 v[1];
    v[0] = ldg_stream(vec + i);
    fold_vectors<ENT, CAP, 1>(acc, v, inv_temp, k2, sc);
  }

  // Block reduction: common max first, then sums rescaled to it.
  RowStats st;
  st.M = block_max<THREADS>(acc.m, red);
  const float d = (acc.m - st.M) * kLog2e;
  const float scl = ex2f(d);
  st.S = block_sum<THREADS>(acc.s * scl, red);
  st.U = 0.f;
  st.S2 = 0.f;
  st.U2 = 0.f;
  if (ENT == 1) st.U = block_sum<THREADS>(acc.u * scl, red);
  if (ENT == 2) {
    const float scl2 = ex2f(d * inv_temp);
    st.S2 = block_sum<THREADS>(acc.s2 * scl2, red);
    st.U2 = block_sum<THREADS>(acc.u2 * scl2, red);
  }

  if (tid == 0) {
    // Chosen logit: global id -> local column (clamped into the vocabulary if out of range).
    int64_t c = p.chosen_ids[n];
    if (c < 0 || c >= p.vocab_total) {
      c = c < 0 ? 0 : p.vocab_total - 1;
      if (p.device_status) atomicOr(p.device_status, MLLM_GRPO_DEV_ID_CLAMPED);
    }
    const int64_t cl = c - p.vocab_start;
    float yc = 0.f;
    const bool mine = (cl >= 0 && cl < V);
    if (mine) {
      yc = __uint_as_float(uint32_t(row16[cl]) << 16);
      if (CAP) yc = sc.y(yc);
    }
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

// Second streaming pass.  One CTA per logits row (scored or not).
template <int THREADS, int UNROLL, bool CAP>
__global__ void __launch_bounds__(THREADS) dlogits_kernel(const KernelParams p) {
  const int tid = threadIdx.x;
  const int64_t r = blockIdx.x;  // row index over n_seqs*seq_rows
  const int64_t b = r / p.seq_rows;
  const int64_t t = r - b * p.seq_rows;
  const int64_t V = p.vocab;
  const uint16_t* x16 = reinterpret_cast<const uint16_t*>(p.logits + r * p.row_stride);
  uint16_t* d16 = reinterpret_cast<uint16_t*>(p.dlogits + r * p.row_stride);
  const RowSplit sp(d16, V);  // the caller guarantees logits and dlogits rows share alignment
  uint4* dvec = reinterpret_cast<uint4*>(d16 + sp.head);

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

  if (g == 0.f) {
    // Unscored row, masked token or zero advantage: exact zeros, logits are not read.
    if (tid < sp.head) d16[tid] = 0;
    if (tid < sp.tail) d16[sp.head + (sp.nvec << 3) + tid] = 0;
    const uint4 z = make_uint4(0, 0, 0, 0);
    for (int64_t i = tid; i < sp.nvec; i += THREADS) stg_stream(dvec + i, z);
    return;
  }

  // g*e^(y-lse) = sign(g) * 2^(y*log2e - lse*log2e + log2|g|): the scale rides in the exponent.
  const float off = lg2f(fabsf(g)) - lse * kLog2e;
  const uint32_t sgn = g < 0.f ? 0x80008000u : 0u;
  const SoftCap sc(CAP ? p.softcap : 1.0f);

  auto one = [&](float x, int64_t j) -> float {  // scalar path: signed f32 result
    float d;
    if (CAP) {
      const float rr = sc.r(x);
      const float y = fmaf(-2.0f * sc.cap, rr, sc.cap);
      d = ex2f(fmaf(y, kLog2e, off));
      d = g < 0.f ? -d : d;
      if (j == cl) d -= g;
      d *= 4.0f * rr * (1.0f - rr);
    } else {
      d = ex2f(fmaf(x, kLog2e, off));
      d = g < 0.f ? -d : d;
      if (j == cl) d -= g;
    }
    return d;
  };

  if (tid < sp.head) {
    const float x = __uint_as_float(uint32_t(x16[tid]) << 16);
    d16[tid] = __bfloat16_as_ushort(__float2bfloat16_rn(one(x, tid)));
  }
  if (tid < sp.tail) {
    const int64_t j = sp.head + (sp.nvec << 3) + tid;
    const float x = __uint_as_float(uint32_t(x16[j]) << 16);
    d16[j] = __bfloat16_as_ushort(__float2bfloat16_rn(one(x, j)));
  }

  const uint4* xvec = reinterpret_cast<const uint4*>(x16 + sp.head);
  // Vector that holds the chosen column (or -1), and its lane inside the vector.
  const int64_t cv = (cl >= sp.head && cl < sp.head + (sp.nvec << 3)) ? ((cl - sp.head) >> 3) : -1;
  const int clane = int((cl - sp.head) & 7);

  auto do_vec = [&](const uint4& v, int64_t idx) -> uint4 {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[4];
    if (!CAP && idx != cv) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float a = ex2f(fmaf(bf16lo(w[j]), kLog2e, off));
        const float c = ex2f(fmaf(bf16hi(w[j]), kLog2e, off));
        o[j] = pack_bf16x2(a, c) ^ sgn;
      }
    } else {
      const int64_t j0 = sp.head + (idx << 3);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float a = one(bf16lo(w[j]), j0 + 2 * j);
        const float c = one(bf16hi(w[j]), j0 + 2 * j + 1);
        o[j] = pack_bf16x2(a, c);
      }
      (void)clane;
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
  };

  int64_t i = tid;
  for (; i + int64_t(UNROLL - 1) * THREADS < sp.nvec; i += int64_t(UNROLL) * THREADS) {
    uint4 v[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) v[u] = ldg_stream_rw(xvec + i + int64_t(u) * THREADS);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      stg_stream(dvec + i + int64_t(u) * THREADS, do_vec(v[u], i + int64_t(u) * THREADS));
  }
  for (; i < sp.nvec; i += THREADS) {
    const uint4 v = ldg_stream_rw(xvec + i);
    stg_stream(dvec + i, do_vec(v, i));
  }
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
