// Row-resident fused forward+backward of the GRPO token loss for sm_100a.
//
// A thread-block cluster of CL CTAs owns one logits row at a time; CTA r keeps the r-th slice of
// the row in its shared memory from the moment TMA (cp.async.bulk) lands it until TMA has stored
// the finished gradient slice back.  Logits therefore cross HBM once in each direction (4 bytes
// per element instead of 6 for separate forward and backward sweeps).
//
// Per CTA: one DMA warp (lane 0 issues every bulk load and bulk store) and NT consumer threads.
// Shared memory holds S stages of one slice each.  For the j-th row of a cluster the consumers run
//   sweep A  thread-local max over the thread's own 16-byte vectors (packed bf16 max, exact)
//   sweep B  p = e^(y - m_thread): accumulates S and U in fp32, overwrites the logits in place with
//            p as f16 (p <= 1), remembers the chosen logit
//   reduce   warp shuffles + one named barrier -> slice (M, S, U, y_c)
//   exchange lanes 0..CL-1 push the slice partial into every peer CTA's shared memory (DSMEM) and
//            arrive on the peer's mbarrier: no cluster-wide barrier in the steady state
//   epilogue warp 0 merges the CL partials, lane 0 runs the per-token epilogue (ratio, clip, KL,
//            mask) and publishes (lse, g)
//   sweep C  dlogits = g*e^(m_thread - lse) * p - g*onehot, f16 -> bf16 in place; then the DMA
//            thread bulk-stores the slice
// Sweep C of row j runs after sweeps A/B of row j+1, so the exchange latency of a row is hidden
// behind useful work.  Every wait is bounded (wall-clock limit, then an abort flag that makes all
// later waits fall through and a status bit for the host); no thread ever returns early, so the
// hardware barriers stay matched.
#include <cuda_fp16.h>

#include <cstdlib>
#include <mutex>

#include "grpo_cluster.cuh"
#include "grpo_common.cuh"
#include "grpo_launch.h"

namespace grpo {
namespace fused {

constexpr int kMaxStages = 8;
constexpr int kMaxCluster = 8;
constexpr int kSlots = 4;  // exchange slot sets: a peer can run at most three rows ahead of a reader

struct Ctl {
  unsigned long long full_bar[kMaxStages];   // TMA load of a stage landed
  unsigned long long store_bar[kMaxStages];  // consumers finished writing a stage
  unsigned long long xchg_bar[kSlots];       // all CL partials of a row arrived
  float4 xchg[kSlots][kMaxCluster];          // (M, S, U, y_c or 0) per peer
  float4 warp_part[2][32];                   // per-warp (M, S, U), double-buffered by row parity
  float4 rowinfo[2];                         // (lse, g, -, -) published by warp 0
  float4 chosen[kMaxStages];                 // (y_c, p_c, dy/dx at c, -) written by the owner thread
  int abort_flag;
};

using namespace cl;

struct Geometry {
  int64_t nvec_total;  // 16-byte vectors per row
  int64_t nvec_per;    // vectors per CTA slice (last slice may be shorter)
  int stages;
  int slice_bytes_max;
};

// NT consumer threads + 32 DMA threads per CTA; CL CTAs per cluster.
template <int CL, int NT, bool CAP, bool ENT>
__global__ void __launch_bounds__(NT + 32, 1) fused_row_kernel(const KernelParams p, const Geometry geo) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int S = geo.stages;
  Ctl* ctl = reinterpret_cast<Ctl*>(smem_raw + size_t(S) * geo.slice_bytes_max);
  const uint32_t stage0 = smem_u32(smem_raw);
  const int tid = threadIdx.x;
  const uint32_t rank = cluster_rank();
  const int64_t cid = cluster_id_x();
  const int64_t ncl = n_clusters_x();
  volatile int* abort_flag = &ctl->abort_flag;

  // This CTA's slice of every row.
  const int64_t v0 = int64_t(rank) * geo.nvec_per;
  int64_t nv = geo.nvec_total - v0;
  if (nv > geo.nvec_per) nv = geo.nvec_per;
  const uint32_t slice_bytes = uint32_t(nv) * 16u;
  const int64_t col0 = v0 * 8;  // first column of the slice

  const int64_t N = p.n_seqs * p.scored_rows;
  const int64_t my_rows = (N > cid) ? (N - cid + ncl - 1) / ncl : 0;  // rows cid, cid+ncl, ...

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&ctl->full_bar[s]), 1);
      mbar_init(smem_u32(&ctl->store_bar[s]), NT);
    }
    for (int q = 0; q < kSlots; ++q) mbar_init(smem_u32(&ctl->xchg_bar[q]), CL);
    ctl->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  cluster_sync_all();  // peers' barriers exist before anyone arrives on them remotely

  auto row_of = [&](int64_t j, int64_t& n, int64_t& b) -> int64_t {
    n = cid + j * ncl;
    b = n / p.scored_rows;
    const int64_t t = n - b * p.scored_rows;
    return b * p.seq_rows + t;
  };

  if (tid >= NT) {
    // ------------------------------- DMA warp -------------------------------
    if (tid == NT) {
      const int64_t pre = my_rows < S ? my_rows : S;
      for (int64_t j = 0; j < pre; ++j) {
        int64_t n, b;
        const int64_t r = row_of(j, n, b);
        const uint32_t bar = smem_u32(&ctl->full_bar[j]);
        mbar_expect_tx(bar, slice_bytes);
        bulk_load(stage0 + uint32_t(j) * geo.slice_bytes_max, p.logits + r * p.row_stride + col0, slice_bytes, bar);
      }
      for (int64_t j = 0; j < my_rows; ++j) {
        const int s = int(j % S);
        const uint32_t par = uint32_t((j / S) & 1);
        mbar_wait(smem_u32(&ctl->store_bar[s]), par, abort_flag, p.device_status);
        int64_t n, b;
        const int64_t r = row_of(j, n, b);
        bulk_store(p.dlogits + r * p.row_stride + col0, stage0 + uint32_t(s) * geo.slice_bytes_max, slice_bytes);
        if (j + S < my_rows) {
          bulk_wait_read();  // the store has read the stage: it may be overwritten
          const int64_t r2 = row_of(j + S, n, b);
          const uint32_t bar = smem_u32(&ctl->full_bar[s]);
          mbar_expect_tx(bar, slice_bytes);
          bulk_load(stage0 + uint32_t(s) * geo.slice_bytes_max, p.logits + r2 * p.row_stride + col0, slice_bytes, bar);
        }
      }
      bulk_wait_all();
    }
  } else {
    // ------------------------------- consumers -------------------------------
    const int lane = tid & 31, warp = tid >> 5;
    constexpr int NW = NT / 32;
    const SoftCap sc(CAP ? p.softcap : 1.0f);

    // Rows of the logits buffer that are not scored (positions >= scored_rows) get zeros.
    {
      const int64_t per_seq = p.seq_rows - p.scored_rows;
      const int64_t n_unscored = p.n_seqs * per_seq;
      const uint4 z = make_uint4(0, 0, 0, 0);
      for (int64_t u = cid; u < n_unscored; u += ncl) {
        const int64_t b = u / per_seq;
        const int64_t r = b * p.seq_rows + p.scored_rows + (u - b * per_seq);
        uint4* dst = reinterpret_cast<uint4*>(p.dlogits + r * p.row_stride + col0);
        for (int64_t i = tid; i < nv; i += NT) dst[i] = z;
      }
    }

    float m_prev = kNegInit, m_cur = kNegInit;
    // side inputs of the rows in flight, held by lane 0 of warp 0
    TokenSide side[2] = {};
    int64_t c_loc[2] = {-1, -1};  // chosen column relative to this slice, for rows j (cur) and j-1 (prev)

    for (int64_t j = 0; j <= my_rows; ++j) {
      if (j < my_rows) {
        // ---------------- sweeps A and B of row j ----------------
        int64_t n, b;
        row_of(j, n, b);
        const int s = int(j % S);
        const uint32_t base = stage0 + uint32_t(s) * geo.slice_bytes_max;
        int64_t c = p.chosen_ids[n];
        if (c < 0 || c >= p.vocab_total) {
          c = c < 0 ? 0 : p.vocab_total - 1;
          if (tid == 0 && rank == 0 && p.device_status) atomicOr(p.device_status, MLLM_GRPO_DEV_ID_CLAMPED);
        }
        c_loc[0] = c - col0;
        const bool mine = c_loc[0] >= 0 && c_loc[0] < nv * 8;
        const int64_t cv = mine ? (c_loc[0] >> 3) : -1;
        if (tid == 0) {  // prefetch the token's side inputs; they are needed one row later
          side[0] = load_token_side(p, n, b);
        }
        mbar_wait(smem_u32(&ctl->full_bar[s]), uint32_t((j / S) & 1), abort_flag, p.device_status);

        // sweep A: max over this thread's vectors
        uint32_t mx2 = 0xff7fff7fu;  // two copies of the most negative finite bf16
        for (int64_t i = tid; i < nv; i += NT) {
          const uint4 q = lds128(base + uint32_t(i) * 16u);
          mx2 = bf16x2_max(mx2, bf16x2_max(bf16x2_max(q.x, q.y), bf16x2_max(q.z, q.w)));
        }
        float mt = fmaxf(bf16lo(mx2), bf16hi(mx2));
        if (CAP) mt = sc.y(mt);
        mt = fmaxf(mt, kNegInit);
        m_cur = mt;

        // sweep B: p = e^(y - mt); S, U; p (times dy/dx with the soft-cap) goes back as f16
        const float mk = mt * kLog2e;
        float sS = 0.f, sU = 0.f;
        for (int64_t i = tid; i < nv; i += NT) {
          const uint32_t addr = base + uint32_t(i) * 16u;
          const uint4 q = lds128(addr);
          const uint32_t w[4] = {q.x, q.y, q.z, q.w};
          uint32_t o[4];
          float pe[8], de[8], ye[8];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            float x0 = bf16lo(w[k]), x1 = bf16hi(w[k]);
            float d0 = 1.f, d1 = 1.f;
            if (CAP) {
              x0 = sc.y(x0);
              x1 = sc.y(x1);
              d0 = sc.dydx(x0);
              d1 = sc.dydx(x1);
            }
            const float p0 = ex2f(fmaf(x0, kLog2e, -mk)), p1 = ex2f(fmaf(x1, kLog2e, -mk));
            sS += p0;
            sS += p1;
            if (ENT) {
              sU = fmaf(p0, x0, sU);
              sU = fmaf(p1, x1, sU);
            }
            pe[2 * k] = p0;
            pe[2 * k + 1] = p1;
            ye[2 * k] = x0;
            ye[2 * k + 1] = x1;
            de[2 * k] = d0;
            de[2 * k + 1] = d1;
            o[k] = CAP ? pack_f16x2(p0 * d0, p1 * d1) : pack_f16x2(p0, p1);
          }
          if (i == cv) {
            const int l = int(c_loc[0] & 7);
            float yc = 0.f, pc = 0.f, dc = 1.f;
#pragma unroll
            for (int k = 0; k < 8; ++k)
              if (k == l) {
                yc = ye[k];
                pc = pe[k];
                dc = de[k];
              }
            ctl->chosen[s] = make_float4(yc, pc, dc, 0.f);
          }
          sts128(addr, make_uint4(o[0], o[1], o[2], o[3]));
        }

        // slice reduce: warp shuffles, then one named barrier
        const float Mw = warp_max(mt);
        const float scl = ex2f((mt - Mw) * kLog2e);
        const float Sw = warp_sum(sS * scl);
        const float Uw = ENT ? warp_sum(sU * scl) : 0.f;
        if (lane == 0) ctl->warp_part[j & 1][warp] = make_float4(Mw, Sw, Uw, 0.f);
        consumer_bar(NT);
        if (warp == 0) {
          float4 wp = (lane < NW) ? ctl->warp_part[j & 1][lane] : make_float4(kNegInit, 0.f, 0.f, 0.f);
          const float Ms = warp_max(wp.x);
          const float sc2 = ex2f((wp.x - Ms) * kLog2e);
          const float Ss = warp_sum(wp.y * sc2);
          const float Us = ENT ? warp_sum(wp.z * sc2) : 0.f;
          const float ycs = mine ? ctl->chosen[s].x : 0.f;
          // push the slice partial to every CTA of the cluster (own CTA included)
          if (lane < CL) {
            const int q = int(j & (kSlots - 1));
            st_cluster_f4(map_to_cta(smem_u32(&ctl->xchg[q][rank]), lane), make_float4(Ms, Ss, Us, ycs));
            mbar_arrive_cluster(map_to_cta(smem_u32(&ctl->xchg_bar[q]), lane));
          }
        }
      }

      if (j >= 1) {
        // ---------------- epilogue and sweep C of row j-1 ----------------
        const int64_t jj = j - 1;
        int64_t n, b;
        row_of(jj, n, b);
        const int s = int(jj % S);
        const uint32_t base = stage0 + uint32_t(s) * geo.slice_bytes_max;
        const int q = int(jj & (kSlots - 1));
        if (warp == 0) {
          mbar_wait(smem_u32(&ctl->xchg_bar[q]), uint32_t((jj / kSlots) & 1), abort_flag, p.device_status);
          const float4 part = (lane < CL) ? ctl->xchg[q][lane] : make_float4(kNegInit, 0.f, 0.f, 0.f);
          RowStats st;
          st.M = warp_max(part.x);
          const float e = ex2f((part.x - st.M) * kLog2e);
          st.S = warp_sum(part.y * e);
          st.U = ENT ? warp_sum(part.z * e) : 0.f;
          st.S2 = 0.f;
          st.U2 = 0.f;
          const float yc = warp_sum(part.w);
          if (lane == 0) {
            const TokenOut o = token_epilogue_core<ENT ? 1 : 0>(p, st, yc, side[1]);
            const float nvt = p.total_valid_dev ? *p.total_valid_dev : p.total_valid;
            const float gs = p.grad_scale_dev ? *p.grad_scale_dev : p.grad_scale;
            ctl->rowinfo[jj & 1] = make_float4(o.lse, o.grad_coef * gs / nvt, 0.f, 0.f);
            if (rank == 0) {
              p.per_token_logps[n] = o.lp;
              if (ENT && p.token_entropy) p.token_entropy[n] = o.entropy;
              p.lse[n] = o.lse;
              p.grad_coef[n] = o.grad_coef;
              p.loss_terms[n] = o.loss_term;
            }
          }
        }
        consumer_bar(NT);
        const float4 ri = ctl->rowinfo[jj & 1];
        const float lse = ri.x, g = ri.y;
        if (g == 0.f) {
          const uint4 z = make_uint4(0, 0, 0, 0);
          for (int64_t i = tid; i < nv; i += NT) sts128(base + uint32_t(i) * 16u, z);
        } else {
          const float f = g * ex2f((m_prev - lse) * kLog2e);
          const bool mine = c_loc[1] >= 0 && c_loc[1] < nv * 8;
          const int64_t cv = mine ? (c_loc[1] >> 3) : -1;
          for (int64_t i = tid; i < nv; i += NT) {
            const uint32_t addr = base + uint32_t(i) * 16u;
            const uint4 qv = lds128(addr);
            const uint32_t w[4] = {qv.x, qv.y, qv.z, qv.w};
            float d[8];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float2 pp = unpack_f16x2(w[k]);
              d[2 * k] = pp.x * f;
              d[2 * k + 1] = pp.y * f;
            }
            if (i == cv) {
              const float4 ch = ctl->chosen[s];
              const int l = int(c_loc[1] & 7);
              const float fix = (f * ch.y - g) * ch.z;
#pragma unroll
              for (int k = 0; k < 8; ++k)
                if (k == l) d[k] = fix;
            }
            sts128(addr, make_uint4(pack_bf16x2(d[0], d[1]), pack_bf16x2(d[2], d[3]), pack_bf16x2(d[4], d[5]),
                                    pack_bf16x2(d[6], d[7])));
          }
        }
        fence_async_smem();
        mbar_arrive(smem_u32(&ctl->store_bar[s]));
      }
      // rotate the per-row registers
      m_prev = m_cur;
      c_loc[1] = c_loc[0];
      side[1] = side[0];
    }
  }
  // No CTA may exit while a peer can still write into its shared memory.
  __syncthreads();
  cluster_sync_all();
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
struct Plan {
  int cluster = 0, threads = 0, stages = 0, slice_bytes = 0, n_clusters = 0;
  size_t smem = 0;
};

static int env_int(const char* name, int dflt) {
  const char* v = std::getenv(name);
  return v ? std::atoi(v) : dflt;
}

template <int CL, int NT, bool CAP, bool ENT>
static cudaError_t launch_t(const KernelParams& p, const Geometry& geo, const Plan& plan, cudaStream_t s) {
  auto kern = fused_row_kernel<CL, NT, CAP, ENT>;
  static std::mutex mu;
  static size_t smem_set[64] = {0};
  static int max_clusters[64] = {0};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CL;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(NT + 32, 1, 1);
  cfg.dynamicSmemBytes = plan.smem;
  cfg.stream = s;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int ncl = 0;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 64 && smem_set[dev] != plan.smem) {
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(plan.smem));
      if (e != cudaSuccess) return e;
      cfg.gridDim = dim3(CL, 1, 1);
      e = cudaOccupancyMaxActiveClusters(&ncl, kern, &cfg);
      if (e != cudaSuccess) return e;
      smem_set[dev] = plan.smem;
      max_clusters[dev] = ncl;
    }
    ncl = dev < 64 ? max_clusters[dev] : 0;
  }
  if (ncl <= 0) return cudaErrorInvalidConfiguration;
  const int64_t N = p.n_seqs * p.scored_rows;
  const int forced = env_int("MLLM_GRPO_FUSED_CLUSTERS", 0);
  if (forced > 0 && forced < ncl) ncl = forced;
  if (ncl > N) ncl = int(N);
  cfg.gridDim = dim3(unsigned(ncl) * CL, 1, 1);
  e = cudaLaunchKernelEx(&cfg, kern, p, geo);
  count_launch();
  return e;
}

template <int CL, int NT>
static cudaError_t launch_cn(const KernelParams& p, const Geometry& geo, const Plan& plan, bool ent, cudaStream_t s) {
  const bool cap = p.softcap > 0.f;
  if (cap) return ent ? launch_t<CL, NT, true, true>(p, geo, plan, s) : launch_t<CL, NT, true, false>(p, geo, plan, s);
  return ent ? launch_t<CL, NT, false, true>(p, geo, plan, s) : launch_t<CL, NT, false, false>(p, geo, plan, s);
}

}  // namespace fused

// Returns true and fills the plan if the row-resident kernel can take this problem: full rows,
// 16-byte aligned rows in both buffers, temperature-1 entropy (or none), and at least two slices of
// the chosen cluster size fit in shared memory.
bool fused_supported(const KernelParams& p, int ent, fused::Plan* plan, fused::Geometry* geo) {
  if (ent == 2) return false;
  if (p.vocab_start != 0 || p.vocab != p.vocab_total) return false;
  if ((p.vocab & 7) || (p.row_stride & 7)) return false;
  if ((reinterpret_cast<uintptr_t>(p.logits) & 15) || (reinterpret_cast<uintptr_t>(p.dlogits) & 15)) return false;
  const int64_t nvec = p.vocab / 8;
  const size_t avail = 232448 - sizeof(fused::Ctl) - 256;
  int want_cl = fused::env_int("MLLM_GRPO_FUSED_CLUSTER", 0);
  const int min_stages = 3;
  for (int cl = 1; cl <= fused::kMaxCluster; cl *= 2) {
    if (want_cl && cl != want_cl) continue;
    const int64_t per = (nvec + cl - 1) / cl;
    if (nvec - (cl - 1) * per <= 0) continue;  // an empty last slice
    const size_t bytes = size_t(per) * 16;
    int stages = int(avail / bytes);
    if (stages > fused::kMaxStages) stages = fused::kMaxStages;
    const int cap_stages = fused::env_int("MLLM_GRPO_FUSED_STAGES", 0);
    if (cap_stages > 0 && stages > cap_stages) stages = cap_stages;
    if (stages < (want_cl ? 2 : min_stages)) continue;
    plan->cluster = cl;
    plan->stages = stages;
    plan->slice_bytes = int(bytes);
    plan->smem = size_t(stages) * bytes + sizeof(fused::Ctl) + 128;
    plan->threads = fused::env_int("MLLM_GRPO_FUSED_THREADS", per >= 3072 ? 512 : 256);
    geo->nvec_total = nvec;
    geo->nvec_per = per;
    geo->stages = stages;
    geo->slice_bytes_max = int(bytes);
    return true;
  }
  return false;
}

cudaError_t launch_fused(const KernelParams& p, int ent, cudaStream_t s, bool* taken) {
  fused::Plan plan;
  fused::Geometry geo;
  *taken = fused_supported(p, ent, &plan, &geo);
  if (!*taken) return cudaSuccess;
  const bool e = ent == 1;
  const bool t512 = plan.threads >= 512;
  switch (plan.cluster) {
    case 1: return t512 ? fused::launch_cn<1, 512>(p, geo, plan, e, s) : fused::launch_cn<1, 256>(p, geo, plan, e, s);
    case 2: return t512 ? fused::launch_cn<2, 512>(p, geo, plan, e, s) : fused::launch_cn<2, 256>(p, geo, plan, e, s);
    case 4: return t512 ? fused::launch_cn<4, 512>(p, geo, plan, e, s) : fused::launch_cn<4, 256>(p, geo, plan, e, s);
    default: return t512 ? fused::launch_cn<8, 512>(p, geo, plan, e, s) : fused::launch_cn<8, 256>(p, geo, plan, e, s);
  }
}

}  // namespace grpo
