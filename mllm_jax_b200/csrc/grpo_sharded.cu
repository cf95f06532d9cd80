// Vocabulary-parallel forward+backward in ONE kernel per GPU with the exchange inside it.
//
// Every rank (one process per GPU) launches the same grid on its own column shard: one CTA per
// logits row.  A CTA
//   1. streams its row shard once (L2 evict_last) -> (M, S, U, y_c or 0),
//   2. threads 0..k-1 each push that partial into rank q's exchange buffer with a plain peer
//      store over NVLink, fence, then store a release flag (the call's epoch) next to it,
//   3. threads 0..k-1 each wait, bounded, until rank q's flag for this row shows up in this
//      rank's OWN buffer (local polling only; nothing is ever loaded from a peer),
//   4. thread 0 merges the k partials, runs the per-token epilogue, broadcasts (lse, g),
//   5. the CTA streams the row shard again (served by L2) and writes its dlogits columns.
// While a CTA waits in step 3 the other resident CTAs of the SM keep streaming, which hides the
// NVLink latency.  Ranks walk the rows in the same order, and a CTA only ever waits for the row
// it owns, so the lowest unfinished row on every GPU can always make progress.  Waits are bounded
// by wall-clock time: on a timeout the CTA raises MLLM_GRPO_DEV_WAIT_TIMEOUT and carries on.
//
// Buffers are double-buffered by the parity of the epoch: a rank can start call e+2 only after
// every peer has published all of call e+1, i.e. after every peer has finished call e, so a slot
// is never overwritten while somebody still waits on it.  No multicast, no TMA on peer memory.
#include "grpo_cluster.cuh"
#include "grpo_common.cuh"
#include "grpo_launch.h"
#include "grpo_rowpass.cuh"

namespace grpo {

constexpr unsigned long long kPeerWaitLimitNs = 2000000000ull;  // 2 s

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys_f4(float4* p, float4 v) {
  asm volatile("st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}
__device__ __forceinline__ float4 ld_relaxed_sys_f4(const float4* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

template <int THREADS, int UNROLL, int ENT, bool CAP>
__global__ void __launch_bounds__(THREADS) row_two_pass_sharded_kernel(const KernelParams p) {
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
  const int64_t N = p.n_seqs * p.scored_rows;
  const int k = p.n_shards, me = p.shard_rank;
  const int64_t half = int64_t(p.exchange_epoch & 1) * int64_t(k) * N;  // parity half of every buffer

  const RowStats st = row_pass1<THREADS, UNROLL, ENT, CAP, 2>(x16, p.vocab, p.inv_temperature, sc, red, keep);

  int64_t c = p.chosen_ids[n];
  if (c < 0 || c >= p.vocab_total) {
    c = c < 0 ? 0 : p.vocab_total - 1;
    if (tid == 0 && p.device_status) atomicOr(p.device_status, MLLM_GRPO_DEV_ID_CLAMPED);
  }
  const int64_t cl = c - p.vocab_start;

  if (tid < k) {
    float yc = 0.f;
    if (cl >= 0 && cl < p.vocab) {
      yc = __uint_as_float(uint32_t(x16[cl]) << 16);
      if (CAP) yc = sc.y(yc);
    }
    // push to rank `tid` (own buffer included), then publish
    const int64_t slot = half + int64_t(me) * N + n;
    st_relaxed_sys_f4(p.peer_data[tid] + slot, make_float4(st.M, st.S, st.U, yc));
    __threadfence_system();
    st_release_sys(p.peer_flags[tid] + slot, p.exchange_epoch);
    // wait for rank `tid`'s partial of this row in OUR buffer
    const int* flag = p.peer_flags[me] + half + int64_t(tid) * N + n;
    if (ld_acquire_sys(flag) != p.exchange_epoch) {
      const unsigned long long t0 = cl::globaltimer();
      while (ld_acquire_sys(flag) != p.exchange_epoch) {
        if (cl::globaltimer() - t0 > kPeerWaitLimitNs) {
          if (p.device_status) atomicOr(p.device_status, MLLM_GRPO_DEV_WAIT_TIMEOUT);
          break;
        }
        __nanosleep(64);
      }
    }
  }
  __syncthreads();
  if (tid == 0) {
    const float4* mine = p.peer_data[me] + half + n;
    RowStats all;
    all.M = kNegInit;
    for (int q = 0; q < k; ++q) all.M = fmaxf(all.M, ld_relaxed_sys_f4(mine + int64_t(q) * N).x);
    all.S = 0.f;
    all.U = 0.f;
    all.S2 = 0.f;
    all.U2 = 0.f;
    float yc = 0.f;
    for (int q = 0; q < k; ++q) {
      const float4 part = ld_relaxed_sys_f4(mine + int64_t(q) * N);
      const float e = ex2f((part.x - all.M) * kLog2e);
      all.S = fmaf(part.y, e, all.S);
      all.U = fmaf(part.z, e, all.U);
      yc += part.w;
    }
    const TokenOut o = token_epilogue<ENT>(p, n, b, all, yc);
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
  row_pass2<THREADS, UNROLL, CAP, 2>(x16, d16, p.vocab, bc[0], bc[1], cl, sc, drop);
}

namespace {
template <int THREADS, int UNROLL>
cudaError_t launch_sharded_t(const KernelParams& p, int ent, cudaStream_t s) {
  const int64_t R = p.n_seqs * p.seq_rows;
  const bool cap = p.softcap > 0.f;
  const unsigned grid = static_cast<unsigned>(R);
  if (ent == 0) {
    if (cap)
      row_two_pass_sharded_kernel<THREADS, UNROLL, 0, true><<<grid, THREADS, 0, s>>>(p);
    else
      row_two_pass_sharded_kernel<THREADS, UNROLL, 0, false><<<grid, THREADS, 0, s>>>(p);
  } else {
    if (cap)
      row_two_pass_sharded_kernel<THREADS, UNROLL, 1, true><<<grid, THREADS, 0, s>>>(p);
    else
      row_two_pass_sharded_kernel<THREADS, UNROLL, 1, false><<<grid, THREADS, 0, s>>>(p);
  }
  count_launch();
  return cudaGetLastError();
}
}  // namespace

// *taken is false (nothing launched) when logits and dlogits rows do not share their 16-byte phase.
cudaError_t launch_two_pass_sharded(const KernelParams& p, int ent, int threads, cudaStream_t s, bool* taken) {
  const uintptr_t ax = reinterpret_cast<uintptr_t>(p.logits), ad = reinterpret_cast<uintptr_t>(p.dlogits);
  *taken = ((ax ^ ad) & 15) == 0;
  if (!*taken) return cudaSuccess;
  if (threads <= 128) return launch_sharded_t<128, 4>(p, ent, s);
  if (threads <= 256) return launch_sharded_t<256, 4>(p, ent, s);
  return launch_sharded_t<512, 4>(p, ent, s);
}

}  // namespace grpo
