// Forward AND backward of the GRPO token loss in one kernel (kernel and launch templates; the two .cu files
// that include this header instantiate the unsharded and the vocabulary-sharded family separately, so that
// they compile in parallel): each logits row (or this rank's column
// shard of it) is streamed twice by the same CTAs, and the second read is served on chip: by L2, or,
// for unsplit rows of at most 48 KB, by shared memory (SMEM variant: one bulk TMA copy with an mbarrier
// lands the row there and both passes read it from shared memory).
//
//   pass 1   128-bit loads with an L2 evict_last policy, online max / sum-exp -> (M, S, U, y_c)
//   merge    CL > 1: the row is split over a thread-block cluster of CL CTAs (CTA r takes the r-th
//            column slice), so that CL times fewer rows are in flight and a line is re-read after
//            only a few tens of MB have passed through L2; slices push their partial into every
//            peer CTA's shared memory (DSMEM) and one cluster barrier publishes them.
//   exchange SHARDED: the row's partial of this GPU's vocabulary shard is pushed to every rank's
//            exchange buffer as four 8-byte peer stores over NVLink, each word carrying one float
//            and the call's epoch as its flag (an aligned 8-byte store is single-copy atomic: no
//            fence, no separate flag); then threads 0..k-1 poll, bounded, their OWN buffer until
//            rank q's four words show the epoch.  Nothing is ever loaded from a peer; no multicast.
//   epilogue thread 0: ratio, clip, KL, mask -> (lse, g); outputs written once per row
//   pass 2   dlogits = g*(softmax - onehot) in bf16, evict_first loads and stores; g == 0 rows are
//            write-only
// While a CTA waits for peers the other resident CTAs of the SM keep streaming.  Ranks walk the rows
// in the same order and a CTA only waits for the row it owns, so the lowest unfinished row on every
// GPU can always make progress.  Waits are bounded by wall-clock time; a row that gives up raises a
// status bit, is poisoned (log-prob and loss term NaN, zero gradient) and makes every later wait of
// the call return after one look, so a dead peer costs one wait limit per call, not one per row.
// Exchange buffers are double-buffered by the parity of the epoch: a rank can start call e+2 only
// after every peer has published all of call e+1, i.e. finished call e.
#pragma once

#include "grpo_cluster.cuh"
#include "grpo_common.cuh"
#include "grpo_launch.h"
#include "grpo_rowpass.cuh"

namespace grpo {


// One exchanged word: value bits in the low half, the epoch in the high half.
__device__ __forceinline__ unsigned long long make_word(float v, int epoch) {
  return (static_cast<unsigned long long>(static_cast<uint32_t>(epoch)) << 32) |
         static_cast<unsigned long long>(__float_as_uint(v));
}
// Two words per instruction; each 8-byte element is still its own atomic unit.
__device__ __forceinline__ void st_words2_sys(unsigned long long* p, unsigned long long a, unsigned long long b) {
  asm volatile("st.relaxed.sys.global.v2.b64 [%0], {%1, %2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}
__device__ __forceinline__ void ld_words2_sys(const unsigned long long* p, unsigned long long& a,
                                              unsigned long long& b) {
  asm volatile("ld.relaxed.sys.global.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}

__device__ __forceinline__ void prefetch_l2(const void* p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

__device__ __forceinline__ float4 merge_partials(const float4* parts, int count) {
  float M = kNegInit;
  for (int q = 0; q < count; ++q) M = fmaxf(M, parts[q].x);
  float S = 0.f, U = 0.f, yc = 0.f;
  for (int q = 0; q < count; ++q) {
    const float4 part = parts[q];
    const float e = ex2f((part.x - M) * kLog2e);
    S = fmaf(part.y, e, S);
    U = fmaf(part.z, e, U);
    yc += part.w;
  }
  return make_float4(M, S, U, yc);
}

// Waits, bounded, until the four words at `src` (a slot of THIS rank's exchange buffer) carry the call's
// epoch and returns their value halves.  *lost is set when the wait was given up: its own limit ran out
// (the status bit is raised), or some wait of this call, or an uncleared earlier one, already had.
struct WaitedPartial {
  float4 v;
  int lost;
};
// Not inlined: the wait runs once per row in a few threads, and its loop state must not raise the register
// count of the streaming passes around it.
static __device__ __noinline__ WaitedPartial wait_partial_words(const unsigned long long* src, uint32_t want,
                                                        unsigned long long wait_ns, int32_t* status_word) {
  int lost = 0;
  unsigned long long w0, w1, w2, w3;
  unsigned long long t0 = 0;
  const volatile int32_t* status = status_word;
  for (int spin = 0;; ++spin) {
    ld_words2_sys(src, w0, w1);  // all four words in one round trip
    ld_words2_sys(src + 2, w2, w3);
    if (static_cast<uint32_t>(w0 >> 32) == want && static_cast<uint32_t>(w1 >> 32) == want &&
        static_cast<uint32_t>(w2 >> 32) == want && static_cast<uint32_t>(w3 >> 32) == want)
      break;
    if ((spin & 63) == 0 && (*status & MLLM_GRPO_DEV_WAIT_TIMEOUT)) {
      lost = 1;
      break;
    }
    if (t0 == 0) t0 = cl::globaltimer();
    if (cl::globaltimer() - t0 > wait_ns) {
      atomicOr(status_word, MLLM_GRPO_DEV_WAIT_TIMEOUT);
      lost = 1;
      break;
    }
    __nanosleep(32);
  }
  WaitedPartial r;
  r.v = make_float4(__uint_as_float(static_cast<uint32_t>(w0)), __uint_as_float(static_cast<uint32_t>(w1)),
                    __uint_as_float(static_cast<uint32_t>(w2)), __uint_as_float(static_cast<uint32_t>(w3)));
  r.lost = lost;
  return r;
}
__device__ __forceinline__ float4 wait_partial(const KernelParams& p, const unsigned long long* src, bool* lost) {
  const WaitedPartial r = wait_partial_words(src, static_cast<uint32_t>(p.exchange_epoch), p.peer_wait_ns, p.device_status);
  if (r.lost) *lost = true;
  return r.v;
}

__device__ __forceinline__ void push_partial(const KernelParams& p, unsigned long long* dst, const float4& v) {
  st_words2_sys(dst, make_word(v.x, p.exchange_epoch), make_word(v.y, p.exchange_epoch));
  st_words2_sys(dst + 2, make_word(v.z, p.exchange_epoch), make_word(v.w, p.exchange_epoch));
}

// SMEM: the CTA's row slice is brought into shared memory by one bulk (TMA) copy and both passes read
// it from there: no load registers, the whole slice in flight at once, and no second trip to L2.
// The unsplit sharded 256-thread kernels with short load batches are held to 5 CTAs per SM (51 registers): the
// warp-level exchange must not cost them a resident CTA.  0 = no minimum asked for.
template <int CL, int THREADS, int UNROLL, bool CAP, bool SHARDED, bool SMEM>
constexpr int kMinCtasPerSm = (SHARDED && CL == 1 && THREADS == 256 && !SMEM && !CAP && UNROLL <= 6) ? 5 : 0;

template <int CL, int THREADS, int UNROLL, int ENT, bool CAP, bool SHARDED, bool SMEM>
__global__ void __launch_bounds__(THREADS, kMinCtasPerSm<CL, THREADS, UNROLL, CAP, SHARDED, SMEM>) two_pass_kernel(const KernelParams p, const int64_t vec_per) {
  extern __shared__ __align__(128) unsigned char slice_smem[];
  __shared__ unsigned long long load_bar;
  __shared__ int abort_flag;
  __shared__ int peer_lost;  // SHARDED: a wait for another rank's partial of this row ran out
  __shared__ float red[160];
  __shared__ float bc[2];
  __shared__ __align__(16) float4 slots[8];  // cluster slices' partials
  __shared__ __align__(16) float4 parts[8];  // vocabulary shards' partials
  const int tid = threadIdx.x;
  const uint32_t rank = CL > 1 ? cl::cluster_rank() : 0u;
  const int64_t r = CL > 1 ? int64_t(cl::cluster_id_x()) : int64_t(blockIdx.x);
  const int64_t b = r / p.seq_rows;
  const int64_t t = r - b * p.seq_rows;
  int64_t col0 = 0, ncol = p.vocab;
  if (CL > 1) {
    col0 = int64_t(rank) * vec_per * 8;
    ncol = p.vocab - col0;
    if (ncol > vec_per * 8) ncol = vec_per * 8;
  }
  const uint16_t* x16 = reinterpret_cast<const uint16_t*>(p.logits + r * p.row_stride) + col0;
  uint16_t* d16 = reinterpret_cast<uint16_t*>(p.dlogits + r * p.row_stride) + col0;
  const SoftCap sc(CAP ? p.softcap : 1.0f);
  const uint64_t keep = policy_evict_last(), drop = policy_evict_first();
  if (t >= p.scored_rows) {  // every CTA of a cluster takes this branch together
    row_pass2<THREADS, UNROLL, CAP, 2>(x16, d16, ncol, 0.f, 0.f, -1, sc, drop);
    return;
  }
  // Tell the cluster peers this CTA is running (its shared memory exists) without blocking yet.
  if (CL > 1) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
  if (SHARDED && CL > 1 && tid == 0) peer_lost = 0;  // ordered before its writers by the barrier inside the first pass
  if (SMEM && tid == 0) {
    abort_flag = 0;
    const uint32_t bar = cl::smem_u32(&load_bar);
    cl::mbar_init(bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    cl::mbar_expect_tx(bar, uint32_t(ncol) * 2u);
    cl::bulk_load(cl::smem_u32(slice_smem), x16, uint32_t(ncol) * 2u, bar);
  }
  const int64_t n = b * p.scored_rows + t;
  // Everything the epilogue needs is requested before the first pass, so its latency is hidden.
  int64_t c = p.chosen_ids[n];
  if (c < 0 || c >= p.vocab_total) {
    c = c < 0 ? 0 : p.vocab_total - 1;
    if (tid == 0 && rank == 0 && p.device_status) atomicOr(p.device_status, MLLM_GRPO_DEV_ID_CLAMPED);
  }
  const int64_t cl_local = c - p.vocab_start - col0;  // chosen column relative to this CTA's columns
  float yc_own = 0.f;
  if (tid < 8 && cl_local >= 0 && cl_local < ncol) yc_own = __uint_as_float(uint32_t(x16[cl_local]) << 16);
  if (tid == 0) {  // pull the epilogue's side inputs towards L2 without holding registers for them
    if (p.mask) prefetch_l2(p.mask + n);
    prefetch_l2(p.advantages + (p.adv_per_token ? n : b));
    if (p.old_logps) prefetch_l2(p.old_logps + n);
    if (p.ref_logps) prefetch_l2(p.ref_logps + n);
  }

  const uint16_t* xs = x16;
  if (SMEM) {
    __syncthreads();  // the barrier is initialised
    cl::mbar_wait(cl::smem_u32(&load_bar), 0, &abort_flag, p.device_status);  // bounded
    xs = reinterpret_cast<const uint16_t*>(slice_smem);
  }
  const RowStats st = row_pass1<THREADS, UNROLL, ENT, CAP, SMEM ? 3 : 2>(xs, ncol, p.inv_temperature, sc, red, keep);
  if (CAP && tid < 8 && cl_local >= 0 && cl_local < ncol) yc_own = sc.y(yc_own);

  // Unsplit sharded rows: warp 0 alone pushes, waits, merges and finishes the token (every thread holds the
  // row's statistics and lanes < 8 the chosen logit), so no block barrier stands between the first pass's
  // reduction and the one that publishes (g, lse) to the second pass.
  constexpr bool WARP_EXCHANGE = SHARDED && CL == 1;
  if (CL > 1) {
    asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
    if (tid < CL)
      cl::st_cluster_f4(cl::map_to_cta(cl::smem_u32(&slots[rank]), tid), make_float4(st.M, st.S, st.U, yc_own));
    cl::cluster_sync_all();  // release our pushes, acquire everyone else's
  } else if (!WARP_EXCHANGE && tid == 0) {
    slots[0] = make_float4(st.M, st.S, st.U, yc_own);
  }

  TokenSide side = {};
  float4 merged = make_float4(0.f, 0.f, 0.f, 0.f);
  bool lost = false;
  if (WARP_EXCHANGE) {
    if (tid < 32) {
      const int k = p.n_shards, me = p.shard_rank;
      const int64_t N = p.n_seqs * p.scored_rows;
      const int64_t half = int64_t(p.exchange_epoch & 1) * int64_t(k) * N;  // parity half of every buffer
      float4 part = make_float4(kNegInit, 0.f, 0.f, 0.f);
      if (tid < k) push_partial(p, p.peer_words[tid] + (half + int64_t(me) * N + n) * 4, make_float4(st.M, st.S, st.U, yc_own));
      // The epilogue's side inputs are requested now, so that their latency runs beside the exchange's.
      if (tid == 0) side = load_token_side(p, n, b);
      if (tid < k) part = wait_partial(p, p.peer_words[me] + (half + int64_t(tid) * N + n) * 4, &lost);
      lost = __any_sync(0xffffffffu, lost);
      const float M = warp_max(part.x);
      const float e = tid < k ? ex2f((part.x - M) * kLog2e) : 0.f;
      merged = make_float4(M, warp_sum(part.y * e), warp_sum(part.z * e), warp_sum(tid < k ? part.w : 0.f));
    }
  } else if (SHARDED) {
    const int k = p.n_shards, me = p.shard_rank;
    const int64_t N = p.n_seqs * p.scored_rows;
    const int64_t half = int64_t(p.exchange_epoch & 1) * int64_t(k) * N;
    if (tid == 0) side = load_token_side(p, n, b);
    if (tid < k) {
      // one CTA per row talks to the other GPUs
      if (rank == 0) push_partial(p, p.peer_words[tid] + (half + int64_t(me) * N + n) * 4, merge_partials(slots, CL));
      // wait for rank `tid`'s partial of this row in OUR buffer
      bool gave_up = false;
      parts[tid] = wait_partial(p, p.peer_words[me] + (half + int64_t(tid) * N + n) * 4, &gave_up);
      if (gave_up) peer_lost = 1;
    }
    __syncthreads();  // parts[] were written by threads 0..k-1
    lost = peer_lost != 0;
  }
  // Unsharded: thread 0 reads slots it wrote itself (CL == 1) or acquired at the cluster barrier (CL > 1).
  if (tid == 0) {
    const float4 m = WARP_EXCHANGE ? merged : (SHARDED ? merge_partials(parts, p.n_shards) : merge_partials(slots, CL));
    RowStats all;
    all.M = m.x;
    all.S = m.y;
    all.U = m.z;
    all.S2 = st.S2;  // temperature != 1 entropy exists only unsplit (CL == 1, not sharded)
    all.U2 = st.U2;
    TokenOut o = SHARDED ? token_epilogue_core<ENT>(p, all, m.w, side) : token_epilogue<ENT>(p, n, b, all, m.w);
    if (SHARDED && lost) {  // merged stale words: make the row unusable instead of silently wrong
      o.lp = o.entropy = o.loss_term = __int_as_float(0x7fc00000);
      o.grad_coef = 0.f;
    }
    if (rank == 0) {
      p.per_token_logps[n] = o.lp;
      if (ENT != 0 && p.token_entropy) p.token_entropy[n] = o.entropy;
      p.lse[n] = o.lse;
      if (p.lse_scaled) p.lse_scaled[n] = scaled_lse<ENT>(p, all, o.lse);
      p.grad_coef[n] = o.grad_coef;
      p.loss_terms[n] = o.loss_term;
    }
    const float nv = p.total_valid_dev ? *p.total_valid_dev : p.total_valid;
    const float gs = p.grad_scale_dev ? *p.grad_scale_dev : p.grad_scale;
    bc[0] = o.grad_coef * gs / nv;
    bc[1] = o.lse;
  }
  __syncthreads();
  row_pass2<THREADS, UNROLL, CAP, 2, SMEM ? 3 : -1>(xs, d16, ncol, bc[0], bc[1], cl_local, sc, drop);
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
namespace twopass_detail {

template <int CL, int THREADS, int UNROLL, int ENT, bool CAP, bool SHARDED>
cudaError_t launch_k(const KernelParams& p, bool smem, cudaStream_t s) {
  const int64_t R = p.n_seqs * p.seq_rows;
  const int64_t nvec = p.vocab / 8;
  const int64_t per = (nvec + CL - 1) / CL;
  const size_t slice_bytes = size_t(CL > 1 ? per : nvec) * 16;
  // shared-memory loads are short: batches of 2 vectors keep the register count low
  auto kern = two_pass_kernel<CL, THREADS, UNROLL, ENT, CAP, SHARDED, false>;
  if constexpr (CL == 1 && ENT != 2) {  // only unsplit rows are staged (split ones measured slower)
    if (smem) kern = two_pass_kernel<1, THREADS, 2, ENT, CAP, SHARDED, true>;
  } else {
    smem = false;
  }
  const size_t dyn = smem ? slice_bytes : 0;
  cudaError_t e;
  // The 48 KB a launch gets without opting in covers static + dynamic shared memory, and the kernel
  // has about 1 KB of static: opt in from 44 KB of row on.
  if (smem && dyn > 44 * 1024) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    if (e != cudaSuccess) return e;
  }
  if (CL > 1) {
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CL;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.gridDim = dim3(static_cast<unsigned>(R * CL), 1, 1);
    cfg.blockDim = dim3(THREADS, 1, 1);
    cfg.dynamicSmemBytes = dyn;
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, kern, p, per);
  } else {
    kern<<<static_cast<unsigned>(R), THREADS, dyn, s>>>(p, per);
    e = cudaGetLastError();
  }
  count_launch();
  return e;
}

template <int CL, int THREADS, int UNROLL, bool SHARDED>
cudaError_t launch_e(const KernelParams& p, int ent, bool smem, cudaStream_t s) {
  const bool cap = p.softcap > 0.f;
  if (ent == 0) return cap ? launch_k<CL, THREADS, UNROLL, 0, true, SHARDED>(p, smem, s) : launch_k<CL, THREADS, UNROLL, 0, false, SHARDED>(p, smem, s);
  if (ent == 1) return cap ? launch_k<CL, THREADS, UNROLL, 1, true, SHARDED>(p, smem, s) : launch_k<CL, THREADS, UNROLL, 1, false, SHARDED>(p, smem, s);
  if constexpr (CL == 1 && !SHARDED)
    return cap ? launch_k<1, THREADS, UNROLL, 2, true, false>(p, false, s) : launch_k<1, THREADS, UNROLL, 2, false, false>(p, false, s);
  return cudaErrorInvalidValue;
}

template <int CL, bool SHARDED>
cudaError_t launch_t(const KernelParams& p, int ent, int threads, int unroll, bool smem, cudaStream_t s) {
  if (threads <= 64 && CL == 1) return launch_e<1, 64, 8, SHARDED>(p, ent, smem, s);
  if constexpr (CL >= 2) {  // batch sizes other than 8 exist for cluster slices only
    if (threads <= 128 && unroll == 6) return launch_e<CL, 128, 6, SHARDED>(p, ent, smem, s);
    if (threads <= 128 && unroll == 10) return launch_e<CL, 128, 10, SHARDED>(p, ent, smem, s);
  }
  if (threads <= 128) return launch_e<CL, 128, 8, SHARDED>(p, ent, smem, s);
  if constexpr (CL == 1) {  // unsplit rows through registers, 256 threads: batches of 4, 6 or 8 (the plan's choice)
    if (threads <= 256 && !smem && unroll == 6) return launch_e<1, 256, 6, SHARDED>(p, ent, smem, s);
    if (threads <= 256 && !smem && unroll == 8) return launch_e<1, 256, 8, SHARDED>(p, ent, smem, s);
  }
  if (threads <= 256 || CL > 1) return launch_e<CL, 256, 4, SHARDED>(p, ent, smem, s);
  return launch_e<CL, 512, 4, SHARDED>(p, ent, smem, s);
}

template <bool SHARDED>
cudaError_t launch_c(const KernelParams& p, int ent, int cluster, int threads, int unroll, bool smem, cudaStream_t s) {
  switch (cluster) {
    case 1: return launch_t<1, SHARDED>(p, ent, threads, unroll, smem, s);
    case 2: return launch_t<2, SHARDED>(p, ent, threads, unroll, smem, s);
    case 4: return launch_t<4, SHARDED>(p, ent, threads, unroll, smem, s);
    case 6:
      if constexpr (!SHARDED) return launch_t<6, SHARDED>(p, ent, threads, unroll, smem, s);
      return launch_t<4, SHARDED>(p, ent, threads, unroll, smem, s);
    default: return launch_t<8, SHARDED>(p, ent, threads, unroll, smem, s);
  }
}

}  // namespace twopass_detail

// Launches the family this translation unit instantiates (SHARDED fixed at compile time).
template <bool SHARDED>
cudaError_t launch_two_pass_family(const KernelParams& p, int ent, int cluster, int threads, int unroll, bool smem,
                                   cudaStream_t s) {
  return twopass_detail::launch_c<SHARDED>(p, ent, cluster, threads, unroll, smem, s);
}

}  // namespace grpo
