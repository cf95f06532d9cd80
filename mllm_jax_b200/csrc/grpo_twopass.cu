// Plan and dispatch of the one-kernel forward + backward (see grpo_twopass_impl.cuh for the kernel), and the
// unsharded kernel family.
#include <atomic>

#include "grpo_twopass_impl.cuh"

namespace grpo {

// Forced plan of the tuning / test hook (mllm_grpo_set_plan_override); 0 (-1 for staged) = automatic.
static std::atomic<int> g_force_cluster{0}, g_force_threads{0}, g_force_batch{0}, g_force_staged{-1};
void set_two_pass_override(int cluster, int threads, int load_batch, int staged) {
  g_force_cluster = cluster;
  g_force_threads = threads;
  g_force_batch = load_batch;
  g_force_staged = staged;
}

cudaError_t launch_two_pass_unsharded(const KernelParams& p, int ent, int cluster, int threads, int unroll, bool smem,
                                      cudaStream_t s) {
  return launch_two_pass_family<false>(p, ent, cluster, threads, unroll, smem, s);
}

// Cluster size, thread count and load-batch size for a row of `vocab` columns.  Measured on one B200, 32768
// rows, ms per step (unsplit 256 threads / 2 CTAs x 128 / 4 CTAs x 128): 64 KB rows 0.673 / 0.827 / 1.133,
// 76 KB 0.821 / 0.893 / 1.147, 100 KB 1.129 / 1.134 / 1.323, 125 KB 1.523 / 1.469 / 1.723,
// 148 KB 1.875 / 1.731 / 1.790, 195 KB 2.554 / 2.398 / 2.252.
void two_pass_plan(const KernelParams& p, int ent, bool sharded, int* cluster, int* threads, bool* smem, int* unroll) {
  const int64_t row_bytes = p.vocab * 2;
  int cl = row_bytes >= 176 * 1024 ? 4 : (row_bytes >= 112 * 1024 ? 2 : 1);
  int un = 8;
  if (cl > 1) {
    // A thread of a 128-thread CTA loads its slice in batches of `un` 16-byte vectors; what is left over
    // (fewer than `un` vectors) is requested at once and folded vector by vector, except with batches of
    // 10, whose leftovers go one at a time (the tail buffers cost that kernel registers).  So: batches of
    // 10 where they leave under 5 % over, else batches of 8, on the coarser split (8 or 4 CTAs for rows of
    // 192 KB and more).  Measured on one B200: V=151936 4 CTAs x 8: 3.43 ms (8 CTAs x 6: 3.48; 4 x 10: 3.52);
    // V=128256 4 CTAs x 10: 11.6 ms (4 x 6: 11.9, 4 x 8: 12.1, 8 x 6: 12.2).  The soft-cap kernels need too
    // many registers for batches of 10 and take the (split, 8 or 6) pair with the smallest leftover share:
    // V=256000: 8 CTAs x 6 15.1 ms, 4 x 6 15.1, 4 x 8 15.6, 8 x 8 16.8.
    const bool cap = p.softcap > 0.f;
    const int c_hi = row_bytes >= 192 * 1024 ? 8 : cl, c_lo = row_bytes >= 192 * 1024 ? 4 : cl;
    auto leftover = [&](int c, int u) {
      const double n = double((p.vocab / 8 + c - 1) / c) / 128.0;
      return (n - double(u) * double(int64_t(n / double(u)))) / n;
    };
    if (cap) {
      double best = 2.0;
      for (int c = c_hi; c >= c_lo; c /= 2) {
        for (int u = 8; u >= 6; u -= 2) {
          const double share = leftover(c, u);
          if (share < best - 0.02) {
            best = share;
            cl = c;
            un = u;
          }
        }
      }
    } else if (row_bytes >= 192 * 1024) {
      // 6 CTAs x batches of 6 (64 registers, 8 CTAs per SM, about 200 rows = 60 MB between their passes):
      // V=151936 3.39 ms against 3.43 with 4 CTAs x 8; V=128256 11.58 against 11.75 with 4 CTAs x 10.
      cl = 6;
      un = 6;
    } else if (leftover(c_lo, 10) < 0.05) {
      cl = c_lo;
      un = 10;
    } else if (leftover(c_hi, 10) < 0.05) {
      cl = c_hi;
      un = 10;
    } else {
      cl = c_lo;
      un = 8;
    }
  }
  // With the exchange in the kernel every CTA sits through one store -> visible -> poll round trip (1-2 us)
  // between its passes, a fixed cost that weighs on short-lived CTAs: keep whole row shards per CTA unless
  // they are very long.  One GPU exchanging with itself, unsplit 256 threads vs the split an unsharded row
  // of that length gets: 76 KB 0.953 vs 1.002 ms, 125 KB 1.573 vs 1.895, 148 KB 1.923 vs 2.007,
  // 250 KB 3.304 vs 3.116 (the same rows without any exchange: 0.861 / 1.614 / 1.730 / 2.797 split).
  if (sharded && row_bytes < 192 * 1024) cl = 1;
  const bool aligned16 = !(p.vocab & 7) && !(p.row_stride & 7) && !(reinterpret_cast<uintptr_t>(p.logits) & 15) &&
                         !(reinterpret_cast<uintptr_t>(p.dlogits) & 15);
  const int f_cl = g_force_cluster.load(std::memory_order_relaxed), f_th = g_force_threads.load(std::memory_order_relaxed);
  const int f_un = g_force_batch.load(std::memory_order_relaxed), f_sm = g_force_staged.load(std::memory_order_relaxed);
  if (f_cl > 0) cl = f_cl;
  if (cl != 1 && cl != 2 && cl != 4 && cl != 6 && cl != 8) cl = 1;
  const int64_t nvec = p.vocab / 8;
  if (cl > 1) {
    const int64_t per = (nvec + cl - 1) / cl;
    if (!aligned16 || ent == 2 || nvec - (cl - 1) * per <= 0 || p.n_seqs * p.seq_rows * cl >= (int64_t(1) << 31)) cl = 1;
  }
  // measured on one B200 (unsplit rows): 38 KB rows 64 threads, 76 KB 256, 152 KB and longer 512
  int th = f_th > 0 ? f_th : (cl > 1 ? 128 : (row_bytes < 48 * 1024 ? 64 : (row_bytes < 112 * 1024 || sharded ? 256 : 512)));
  // Rows of at most 48 KB that are not split: stage the row in shared memory with one bulk (TMA) copy
  // and run both passes from there (38 KB rows on one B200: 0.400 ms against 0.452 ms through
  // registers).  Longer rows and cluster slices measured slower that way (too few CTAs per SM).
  const size_t slice_bytes = size_t(cl > 1 ? (nvec + cl - 1) / cl : nvec) * 16;
  bool sm = cl == 1 && aligned16 && ent != 2 && slice_bytes <= 48 * 1024 && slice_bytes >= 4096;
  if (f_sm >= 0) sm = f_sm != 0 && cl == 1 && aligned16 && ent != 2 && slice_bytes <= 99 * 1024;
  if (sm && f_th <= 0) th = 256;
  if (f_un > 0) un = f_un;
  *cluster = cl;
  *threads = th;
  *smem = sm;
  if (cl == 1 && f_un <= 0) {
    // Unsplit rows through registers with 256 threads: a thread owns n vectors per pass.  Longer rows want more of
    // them in flight per batch (64 instead of 48 registers, 4 instead of 5 CTAs per SM).  Measured on one B200,
    // batches of 4 / 6 / 8: n = 18.5 (76 KB) 0.821 / 0.834 / 0.826 ms unsharded, 0.863 / 0.828 / 0.887 sharded;
    // n = 24.4 (100 KB) 1.128 / 1.085 / 1.061 unsharded; n = 37.1 (148 KB) 1.904 / 1.875 / 1.774 sharded.
    // The soft-cap kernels (more registers per vector) stay at 4: 65536 rows, 128 KB shards 3.71 / 3.73 / 4.21 ms,
    // 64 KB shards 1.98 / 2.16 / 2.56, 100 KB unsharded 2.78 / 2.85 / 3.09.
    const double n = double(nvec) / 256.0;
    un = p.softcap > 0.f ? 4 : (n >= 22.0 ? 8 : (sharded && n >= 12.0 ? 6 : 4));
  }
  *unroll = (un == 4 || un == 6 || un == 10) ? un : 8;
}

// *taken is false (nothing launched) when logits and dlogits rows do not share their 16-byte phase.
cudaError_t launch_two_pass(const KernelParams& p, int ent, bool sharded, cudaStream_t s, bool* taken) {
  const uintptr_t ax = reinterpret_cast<uintptr_t>(p.logits), ad = reinterpret_cast<uintptr_t>(p.dlogits);
  *taken = ((ax ^ ad) & 15) == 0;
  if (!*taken) return cudaSuccess;
  int cluster = 1, threads = 256;
  bool smem = false;
  int unroll = 8;
  two_pass_plan(p, ent, sharded, &cluster, &threads, &smem, &unroll);
  return sharded ? launch_two_pass_sharded(p, ent, cluster, threads, unroll, smem, s)
                 : launch_two_pass_unsharded(p, ent, cluster, threads, unroll, smem, s);
}

}  // namespace grpo
