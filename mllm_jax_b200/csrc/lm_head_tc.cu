// lm_head projection folded into the loss statistics (forward): logits = hidden x weight^T are produced
// tile by tile in tensor memory and consumed there; they never reach HBM.
//
// Replaces logits = self.lm_head(hidden_states) (MLLM_JAX/language/qwen2/modular_qwen2.py:182) followed by
// the log-softmax / gather / entropy of MLLM_JAX/train_modules/__init__.py:124-138: per row, the running
// (max, sum e^(y-max), sum e^(y-max)*y, chosen logit) over the vocabulary, the same four numbers a
// vocabulary shard contributes (mllm_grpo_fwd_partials), so mllm_grpo_combine finishes the forward.
//
// One CTA = one tile of 128 rows x a run of 256-column vocabulary tiles; 192 threads in three roles:
//   warp 0      TMA producer: hidden[128 x 64] and weight[256 x 64] k-blocks (bf16, 128-byte swizzle) through a
//               ring of shared-memory stages, each guarded by a full / empty mbarrier pair
//   warp 1      allocates tensor memory (512 columns = two 128 x 256 f32 accumulators) and issues
//               tcgen05.mma (kind::f16, M = 128, N = 256, K = 16) from one thread; tcgen05.commit frees a
//               stage, and after the last k-block hands the accumulator to the epilogue
//   warps 2-5   epilogue: tcgen05.ld 32 columns at a time (thread = one row = one TMEM lane), online max /
//               sum-exp in registers across all vocabulary tiles of the CTA, while the MMA warp already
//               fills the other accumulator
// Every mbarrier wait is bounded by wall-clock time; a wait that runs out raises a status bit, makes all
// roles leave their loops, and the CTA still frees its tensor memory before it returns.
#include <cuda.h>

#include <mutex>

#include "grpo_cluster.cuh"
#include "grpo_common.cuh"
#include "grpo_launch.h"

namespace grpo {
namespace lmh {

constexpr int kBM = 128;      // rows per CTA tile (TMEM lanes)
constexpr int kBN = 256;      // vocabulary columns per tile (one accumulator)
constexpr int kBK = 64;       // k-block: 64 bf16 = 128 bytes = one swizzle row
constexpr int kStages = 4;
constexpr int kABytes = kBM * kBK * 2;  // 16 KB
constexpr int kBBytes = kBN * kBK * 2;  // 32 KB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kThreads = 192;
constexpr int kTmemCols = 512;
constexpr unsigned long long kWaitNs = 2000000000ull;  // 2 s per wait
constexpr size_t kSmemBytes = size_t(kStages) * kStageBytes + 1024 /* alignment slack */ + 256 /* barriers */;

struct Params {
  int64_t n_rows, vocab, hidden, vocab_start, vocab_total;
  int m_tiles, n_vtiles, splits, tiles_per_split, k_blocks;
  float softcap;
  int want_entropy;
  const int32_t* chosen_ids;
  float4* partials;  // [splits, n_rows]
  int32_t* device_status;
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// Shared-memory matrix descriptor of a K-major bf16 tile whose rows are 128 bytes (64 elements), stored
// with the 128-byte swizzle in groups of 8 rows (1024 bytes): start address and stride between row groups
// in units of 16 bytes, descriptor version 1, layout type 2 (128-byte swizzle).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= uint64_t((addr & 0x3FFFFu) >> 4);
  d |= uint64_t(1) << 16;            // leading byte offset: unused for swizzled K-major tiles
  d |= uint64_t(1024 >> 4) << 32;    // stride byte offset: next group of 8 rows
  d |= uint64_t(1) << 46;            // descriptor version
  d |= uint64_t(2) << 61;            // 128-byte swizzle
  return d;
}
// The same for an MN-major operand (the weight stored [hidden, vocab], vocabulary contiguous): 64 vocabulary
// entries (128 bytes) per row of the swizzle atom, 8 k-rows per atom (1024 bytes, the stride offset), and the
// leading offset is the distance between two 64-entry column blocks of the tile.
__device__ __forceinline__ uint64_t smem_desc_mn(uint32_t addr, uint32_t block_bytes) {
  uint64_t d = 0;
  d |= uint64_t((addr & 0x3FFFFu) >> 4);
  d |= uint64_t((block_bytes >> 4) & 0x3FFFu) << 16;  // leading byte offset: next block of 64 columns
  d |= uint64_t(1024 >> 4) << 32;                     // stride byte offset: next group of 8 k-rows
  d |= uint64_t(1) << 46;
  d |= uint64_t(2) << 61;
  return d;
}
// Instruction descriptor: D f32, A and B bf16, A K-major, B K-major or MN-major (bit 16), N at bits 17-22 (N/8),
// M at bits 24-28 (M/16).
__host__ __device__ constexpr uint32_t instr_desc(int M, int N, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | (uint32_t(N >> 3) << 17) |
         (uint32_t(M >> 4) << 24);
}
__device__ __forceinline__ void mma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Bounded mbarrier wait shared by the three roles: false once any wait of the CTA has run out.
__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int* abort_flag, int32_t* status) {
  if (cl::mbar_try(bar, parity)) return true;
  unsigned long long t0 = 0;
  for (uint32_t spin = 0;; ++spin) {
    if (cl::mbar_try(bar, parity)) return true;
    if (*abort_flag) return false;
    if ((spin & 255u) == 0) {
      const unsigned long long now = cl::globaltimer();
      if (t0 == 0) t0 = now;
      if (now - t0 > kWaitNs) {
        *abort_flag = 1;
        if (status) atomicOr(status, MLLM_GRPO_DEV_WAIT_TIMEOUT);
        return false;
      }
    }
  }
}

// WMN: the weight is [hidden, vocab] (vocabulary contiguous, a flax Dense kernel) instead of [vocab, hidden].
template <bool WMN>
__global__ void __launch_bounds__(kThreads, 1)
lm_head_stats_kernel(const __grid_constant__ CUtensorMap map_hidden, const __grid_constant__ CUtensorMap map_weight,
                     const Params p) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = cl::smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;              // swizzled tiles need 1024-byte alignment
  const uint32_t bars = tiles + uint32_t(kStages) * kStageBytes;  // 8-byte aligned
  // barrier slots: full[kStages], empty[kStages], acc_full[2], acc_empty[2]
  auto full_bar = [&](int s) { return bars + 8u * uint32_t(s); };
  auto empty_bar = [&](int s) { return bars + 8u * uint32_t(kStages + s); };
  auto acc_full = [&](int a) { return bars + 8u * uint32_t(2 * kStages + a); };
  auto acc_empty = [&](int a) { return bars + 8u * uint32_t(2 * kStages + 2 + a); };
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // CTA -> (row tile, vocabulary split).  Groups of 16 row tiles walk the splits together, so the CTAs that
  // run at the same time share their weight tiles in L2 and re-read only 16 row tiles of hidden states.
  const int per_group = 16 * p.splits;
  const int group = blockIdx.x / per_group, within = blockIdx.x - group * per_group;
  const int rows_in_group = min(16, p.m_tiles - group * 16);
  const int m_tile = group * 16 + within % rows_in_group;
  const int split = within / rows_in_group;
  const int vt0 = split * p.tiles_per_split;
  const int n_tiles = max(0, min(p.tiles_per_split, p.n_vtiles - vt0));

  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      cl::mbar_init(full_bar(s), 1);
      cl::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      cl::mbar_init(acc_full(a), 1);
      cl::mbar_init(acc_empty(a), 4);  // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tmap(&map_hidden);
    prefetch_tmap(&map_weight);
  }
  if (warp == 1) {  // the whole warp allocates; the same warp frees at the end
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(cl::smem_u32(&tmem_base_slot)),
                 "r"(uint32_t(kTmemCols))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = 0; t < n_tiles && ok; ++t) {
        const int n0 = (vt0 + t) * kBN;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          ok = wait_or_abort(empty_bar(stage), phase ^ 1u, &abort_flag, p.device_status);
          if (!ok) break;
          const uint32_t a_dst = tiles + uint32_t(stage) * kStageBytes, b_dst = a_dst + kABytes;
          cl::mbar_expect_tx(full_bar(stage), uint32_t(kStageBytes));
          tma_load_2d(a_dst, &map_hidden, kb * kBK, m_tile * kBM, full_bar(stage));
          if (WMN) {
            // four boxes of 64 vocabulary columns x 64 k-rows, 8 KB each, side by side
#pragma unroll
            for (int c = 0; c < kBN / 64; ++c)
              tma_load_2d(b_dst + uint32_t(c) * (64u * kBK * 2u), &map_weight, n0 + c * 64, kb * kBK, full_bar(stage));
          } else {
            tma_load_2d(b_dst, &map_weight, kb * kBK, n0, full_bar(stage));
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc(kBM, kBN, WMN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = 0; t < n_tiles && ok; ++t) {
        const int acc = t & 1;
        const uint32_t acc_phase = uint32_t(t >> 1) & 1u;
        ok = wait_or_abort(acc_empty(acc), acc_phase ^ 1u, &abort_flag, p.device_status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_addr = tmem_base + uint32_t(acc * kBN);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          ok = wait_or_abort(full_bar(stage), phase, &abort_flag, p.device_status);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_src = tiles + uint32_t(stage) * kStageBytes, b_src = a_src + kABytes;
          const uint64_t adesc = smem_desc(a_src);
          const uint64_t bdesc = WMN ? smem_desc_mn(b_src, 64u * kBK * 2u) : smem_desc(b_src);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            // K-major: 16 bf16 = 32 bytes further along K inside the swizzled row: +2 in the address field.
            // MN-major: 16 k-rows = two 1024-byte atoms further: +128.
            mma_bf16(d_addr, adesc + uint64_t(2 * k), bdesc + uint64_t(WMN ? 128 * k : 2 * k), idesc,
                     (kb | k) != 0 ? 1u : 0u);
          }
          mma_commit(empty_bar(stage));  // the stage is free once these MMAs have read it
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) mma_commit(acc_full(acc));  // the accumulator is complete
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue: warps 2..5, one row per thread ----------------
    const int quarter = warp & 3;  // the TMEM lanes a warp may read: 32*(warp id mod 4) ...
    const int row_in_tile = quarter * 32 + lane;
    const int64_t row = int64_t(m_tile) * kBM + row_in_tile;
    const bool row_ok = row < p.n_rows;
    int64_t c = row_ok ? p.chosen_ids[row] : 0;  // global id
    if (row_ok && (c < 0 || c >= p.vocab_total)) {
      c = c < 0 ? 0 : p.vocab_total - 1;
      if (p.device_status) atomicOr(p.device_status, MLLM_GRPO_DEV_ID_CLAMPED);
    }
    c -= p.vocab_start;  // column among this call's weight rows
    if (c < 0 || c >= p.vocab) c = -1;  // another vocabulary shard owns the chosen token
    const bool cap = p.softcap > 0.f;
    const SoftCap sc(cap ? p.softcap : 1.0f);
    float m = kNegInit, s = 0.f, u = 0.f, yc = 0.f;
    bool ok = true;
    for (int t = 0; t < n_tiles && ok; ++t) {
      const int acc = t & 1;
      const uint32_t acc_phase = uint32_t(t >> 1) & 1u;
      ok = wait_or_abort(acc_full(acc), acc_phase, &abort_flag, p.device_status);
      if (!ok) break;
      tc_fence_after();
      const int64_t n0 = int64_t(vt0 + t) * kBN;
      const int64_t c_local = c - n0;
      const int valid = (p.vocab - n0 < kBN) ? int(p.vocab - n0) : kBN;  // columns of this tile inside the vocabulary
      const uint32_t t_addr = tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(acc * kBN);
#pragma unroll 1
      for (int ch = 0; ch < kBN / 32; ++ch) {
        if (ch * 32 >= valid) break;  // uniform over the CTA: the vocabulary ends before this chunk
        uint32_t v[32];
        tmem_ld32(t_addr + uint32_t(ch * 32), v);
        tmem_ld_wait();
        float y[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float x = __uint_as_float(v[j]);
          if (cap) x = sc.y(x);
          y[j] = (ch * 32 + j < valid) ? x : kNegInit;  // columns past the vocabulary contribute nothing
        }
        if (c_local >= ch * 32 && c_local < ch * 32 + 32) {
          const int jj = int(c_local) - ch * 32;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j == jj) yc = y[j];
        }
        float cm = y[0];
#pragma unroll
        for (int j = 1; j < 32; ++j) cm = fmaxf(cm, y[j]);
        if (cm > m) {
          const float r = ex2f((m - cm) * kLog2e);
          s *= r;
          u *= r;
          m = cm;
        }
        const float mk = m * kLog2e;
        float s0 = 0.f, s1 = 0.f, u0 = 0.f, u1 = 0.f;
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const float e0 = ex2f(fmaf(y[j], kLog2e, -mk));
          const float e1 = ex2f(fmaf(y[j + 1], kLog2e, -mk));
          s0 += e0;
          s1 += e1;
          if (p.want_entropy) {
            u0 = fmaf(e0, y[j], u0);
            u1 = fmaf(e1, y[j + 1], u1);
          }
        }
        s += s0 + s1;
        u += u0 + u1;
      }
      // hand the accumulator back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) cl::mbar_arrive(acc_empty(acc));
    }
    if (row_ok && ok && n_tiles > 0) {
      const bool mine = c >= int64_t(vt0) * kBN && c < int64_t(vt0 + n_tiles) * kBN;
      p.partials[int64_t(split) * p.n_rows + row] = make_float4(m, s, u, mine ? yc : 0.f);
    } else if (row_ok) {
      // nothing computed (empty split, or a wait ran out): a neutral entry, the status bit tells the rest
      p.partials[int64_t(split) * p.n_rows + row] = make_float4(kNegInit, 0.f, 0.f, 0.f);
    }
  }

  // ---------------- teardown: every role arrives here, also after an abort ----------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (abort_flag) {
      // copies or MMAs may still be in flight after a wait ran out: give them time (bounded) before the
      // tensor memory goes back
      for (int i = 0; i < 4; ++i) __nanosleep(500000);
    }
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(uint32_t(kTmemCols)) : "memory");
  }
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link-time dependency on libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static std::once_flag once;
  static EncodeTiledFn fn = nullptr;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    else
      (void)cudaGetLastError();
  });
  return fn;
}

// bf16 [rows, cols] row-major with `ld` elements between rows -> tiles of box_rows x 64 columns, 128-byte swizzle.
static bool make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
  const cuuint64_t strides[1] = {cuuint64_t(ld) * 2};
  const cuuint32_t box[2] = {cuuint32_t(kBK), cuuint32_t(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace lmh
}  // namespace grpo

using namespace grpo;

extern "C" {

int32_t mllm_lm_head_splits(int64_t n_rows, int64_t vocab) {
  if (n_rows <= 0 || vocab <= 0) return 0;
  const int64_t vt = (vocab + lmh::kBN - 1) / lmh::kBN;
  // about 16 vocabulary tiles per CTA: long enough to amortise set-up, short enough for an even last wave
  return int32_t((vt + 15) / 16);
}

int64_t mllm_lm_head_partials_bytes(int64_t n_rows, int64_t vocab) {
  return int64_t(mllm_lm_head_splits(n_rows, vocab)) * (n_rows > 0 ? n_rows : 0) * 16;
}

int mllm_lm_head_partials(const mllm_lm_head_args* a, void* stream) {
  if (a == nullptr) return MLLM_GRPO_ERR_NULL_POINTER;
  if (a->struct_size != sizeof(mllm_lm_head_args)) return MLLM_GRPO_ERR_STRUCT_SIZE;
  if (a->n_rows <= 0 || a->vocab <= 0 || a->hidden_dim <= 0) return MLLM_GRPO_ERR_BAD_SHAPE;
  if (a->hidden_stride < a->hidden_dim) return MLLM_GRPO_ERR_BAD_SHAPE;
  if (a->weight_stride < ((a->flags & MLLM_LM_HEAD_FLAG_WEIGHT_HV) ? a->vocab : a->hidden_dim)) return MLLM_GRPO_ERR_BAD_SHAPE;
  if (a->vocab_start < 0 || (a->vocab_total > 0 && a->vocab_start + a->vocab > a->vocab_total)) return MLLM_GRPO_ERR_BAD_SHAPE;
  if (!a->hidden || !a->weight || !a->chosen_ids || !a->partials) return MLLM_GRPO_ERR_NULL_POINTER;
  // TMA: 16-byte aligned bases and row pitches; whole 64-element k-blocks keep the pipeline uniform
  if ((a->hidden_dim % lmh::kBK) || (a->hidden_stride % 8) || (a->weight_stride % 8)) return MLLM_GRPO_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(a->hidden) & 15) || (reinterpret_cast<uintptr_t>(a->weight) & 15) ||
      (reinterpret_cast<uintptr_t>(a->partials) & 15))
    return MLLM_GRPO_ERR_ALIGNMENT;
  if (a->softcap < 0.f) return MLLM_GRPO_ERR_BAD_ATTRIBUTE;
  if (a->n_rows >= (int64_t(1) << 31) || a->vocab >= (int64_t(1) << 31)) return MLLM_GRPO_ERR_TOO_LARGE;

  lmh::Params p;
  p.n_rows = a->n_rows;
  p.vocab = a->vocab;
  p.vocab_start = a->vocab_start;
  p.vocab_total = a->vocab_total > 0 ? a->vocab_total : a->vocab_start + a->vocab;
  p.hidden = a->hidden_dim;
  p.m_tiles = int((a->n_rows + lmh::kBM - 1) / lmh::kBM);
  p.n_vtiles = int((a->vocab + lmh::kBN - 1) / lmh::kBN);
  p.splits = mllm_lm_head_splits(a->n_rows, a->vocab);
  p.tiles_per_split = (p.n_vtiles + p.splits - 1) / p.splits;
  p.k_blocks = int(a->hidden_dim / lmh::kBK);
  p.softcap = a->softcap;
  p.want_entropy = (a->flags & MLLM_GRPO_FLAG_SKIP_ENTROPY) ? 0 : 1;
  p.chosen_ids = a->chosen_ids;
  p.partials = static_cast<float4*>(a->partials);
  p.device_status = a->device_status;
  const int64_t ctas = int64_t(p.m_tiles) * p.splits;
  if (ctas >= (int64_t(1) << 31)) return MLLM_GRPO_ERR_TOO_LARGE;

  CUtensorMap map_h, map_w;
  const bool wmn = (a->flags & MLLM_LM_HEAD_FLAG_WEIGHT_HV) != 0;
  const bool maps_ok =
      lmh::make_map(&map_h, a->hidden, a->n_rows, a->hidden_dim, a->hidden_stride, lmh::kBM) &&
      (wmn ? lmh::make_map(&map_w, a->weight, a->hidden_dim, a->vocab, a->weight_stride, lmh::kBK)  // [H, V]: 64 x 64 boxes
           : lmh::make_map(&map_w, a->weight, a->vocab, a->hidden_dim, a->weight_stride, lmh::kBN));
  if (!maps_ok) return MLLM_GRPO_ERR_NO_DEVICE;

  static std::once_flag attr_once[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MLLM_GRPO_ERR_NO_DEVICE;
  cudaError_t attr_err = cudaSuccess;
  std::call_once(attr_once[dev], [&] {
    attr_err = cudaFuncSetAttribute(lmh::lm_head_stats_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    int(lmh::kSmemBytes));
    if (attr_err == cudaSuccess)
      attr_err = cudaFuncSetAttribute(lmh::lm_head_stats_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      int(lmh::kSmemBytes));
  });
  if (attr_err != cudaSuccess) return record_cuda_error(attr_err);
  if (wmn)
    lmh::lm_head_stats_kernel<true><<<unsigned(ctas), lmh::kThreads, lmh::kSmemBytes, static_cast<cudaStream_t>(stream)>>>(
        map_h, map_w, p);
  else
    lmh::lm_head_stats_kernel<false><<<unsigned(ctas), lmh::kThreads, lmh::kSmemBytes, static_cast<cudaStream_t>(stream)>>>(
        map_h, map_w, p);
  count_launch();
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? MLLM_GRPO_OK : record_cuda_error(e);
}

}  // extern "C"
