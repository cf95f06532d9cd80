// Shared device helpers of the fused GRPO token-loss kernels (sm_100a only).
//
// Notation (one scored token = one logits row):
//   y_j  = x_j, or softcap*tanh(x_j/softcap) when the soft-cap is on
//   M    = max_j y_j      S = sum_j e^(y_j - M)      U = sum_j e^(y_j - M) * y_j
//   lse  = M + log S      lp = (y_c - lse)/temperature      H = lse - U/S
// which restates MLLM_JAX/train_modules/__init__.py:124-126 (log-prob) and
// :136-138 (entropy, without its +1e-9 guard) as streaming sums.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace grpo {

constexpr float kLog2e = 1.4426950408889634f;
// Finite stand-in for "no element seen yet": its product with log2(e) stays finite.
constexpr float kNegInit = -1.0e30f;

struct KernelParams {
  // geometry
  int64_t n_seqs, seq_rows, scored_rows, vocab, row_stride, vocab_start, vocab_total;
  // attributes
  float inv_temperature, clip_lo, clip_hi, beta, softcap;
  float grad_scale, total_valid;
  int adv_per_token;
  int ce_loss;  // 1: per-token loss is -lp (masked cross-entropy) instead of the clipped surrogate
  // inputs
  const __nv_bfloat16* logits;
  const int32_t* chosen_ids;
  const float* mask;
  const float* advantages;
  const float* old_logps;
  const float* ref_logps;
  const float* total_valid_dev;
  const float* grad_scale_dev;
  // outputs / residuals
  float* per_token_logps;
  float* token_entropy;
  float* lse;
  float* lse_scaled;  // optional: log-sum-exp of y/temperature (residual of the entropy gradient)
  const float* entropy_cotangent;  // optional, backward sweep only
  float* grad_coef;
  float* loss;
  float* loss_terms;
  __nv_bfloat16* dlogits;
  float* partials;
  const float* gathered_partials;
  int n_shards;
  int32_t* device_status;
  // peer exchange (mllm_grpo_fwd_bwd_sharded): rank q's buffer as seen from this device
  unsigned long long* peer_words[8];  // [2 parities][n_shards senders][N tokens][4] (float, epoch) words
  int shard_rank;
  int exchange_epoch;
  unsigned long long peer_wait_ns;  // limit of one wait for the other ranks' partials
};

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2f(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcpf(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// bf16 pair packed in one 32-bit word -> two f32 (exact: bf16 is the top half of f32).
__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// Exact packed max of two bf16 pairs (one HMNMX2 per two elements).
__device__ __forceinline__ uint32_t bf16x2_max(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("max.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
// Two f32 -> packed bf16 pair, round to nearest even (lo in the low half).
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}

// Packed fp32 pairs (Blackwell FFMA2/FMUL2/FADD2): two lanes of fp32 arithmetic per issue slot.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// Exact packed min of two bf16 pairs.
__device__ __forceinline__ uint32_t bf16x2_min(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("min.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// Soft-cap y = cap*tanh(x/cap) (deprecated/MLLM_JAX/language/gemma/transformer.py:337-339).
// |x| <= 0.75 cap (the common case: 0.75 * 30 is 5.6 sigma of Gemma-like logits): an odd polynomial
// y = x*P(x^2) of degree 9 evaluated on the FMA pipe, absolute error of tanh 2.6e-7 (8e-6 in y at
// cap 30) -- one SFU op per element is then left for the softmax exponential.  Beyond that:
// cap - 2cap/(1 + e^(2x/cap)), two SFU ops, exact at saturation.  (tanh.approx would be 5e-4
// relative, too coarse for a 2e-3 log-prob bound.  Fitted over the whole |x| <= cap a degree-9
// polynomial is 10x less accurate and broke the 1e-4 loss gate; degree 11 costs one more packed FMA
// per pair and pass.)
struct SoftCap {
  float cap, icap, c1, near;
  float d0, d1, d2, d3, d4;  // tanh(z)/z ~ sum_k t_k z^(2k) on [-0.75, 0.75]; d_k = t_k / cap^(2k)
  __device__ __forceinline__ explicit SoftCap(float cap_)
      : cap(cap_), icap(1.0f / cap_), c1(2.0f * kLog2e / cap_), near(0.75f * cap_) {
    const float i2 = icap * icap;
    d0 = 0.9999972581863403f;
    d1 = -0.33323079347610474f * i2;
    d2 = 0.13226120173931122f * i2 * i2;
    d3 = -0.04928125441074371f * i2 * i2 * i2;
    d4 = 0.012319567613303661f * i2 * i2 * i2 * i2;
  }
  __device__ __forceinline__ float y_far(float x) const { return fmaf(-2.0f * cap, rcpf(1.0f + ex2f(x * c1)), cap); }
  __device__ __forceinline__ float y(float x) const {
    if (fabsf(x) > near) return y_far(x);
    const float q = x * x;
    float p = fmaf(d4, q, d3);
    p = fmaf(p, q, d2);
    p = fmaf(p, q, d1);
    p = fmaf(p, q, d0);
    return x * p;
  }
  // Both lanes of a pair at once; only valid when |x| <= near in both lanes.
  __device__ __forceinline__ f32x2 y2_near(f32x2 x) const {
    const f32x2 q = mul2(x, x);
    f32x2 p = fma2(pack2(d4, d4), q, pack2(d3, d3));
    p = fma2(p, q, pack2(d2, d2));
    p = fma2(p, q, pack2(d1, d1));
    p = fma2(p, q, pack2(d0, d0));
    return mul2(x, p);
  }
  __device__ __forceinline__ f32x2 dydx2(f32x2 y) const {
    const f32x2 t = mul2(y, pack2(icap, icap));
    return fma2(mul2(y, pack2(-icap, -icap)), t, pack2(1.0f, 1.0f));
  }
  // dy/dx = 1 - tanh^2 = 1 - (y/cap)^2
  __device__ __forceinline__ float dydx(float y) const {
    const float t = y * icap;
    return fmaf(-t, t, 1.0f);
  }
};

// Streaming accumulator of one thread.  ENT: 0 none, 1 entropy at temperature 1
// (U shares S), 2 entropy at temperature != 1 (own S2/U2 on y/temperature).
template <int ENT>
struct RowAcc {
  float m, s, u, s2, u2;
  __device__ __forceinline__ void init() {
    m = kNegInit;
    s = 0.f;
    u = 0.f;
    s2 = 0.f;
    u2 = 0.f;
  }
  // Raise the running max to mnew (>= m) and rescale the sums.
  __device__ __forceinline__ void raise(float mnew, float inv_temp) {
    const float d = (m - mnew) * kLog2e;
    const float sc = ex2f(d);
    s *= sc;
    if (ENT == 1) u *= sc;
    if (ENT == 2) {
      const float sc2 = ex2f(d * inv_temp);
      s2 *= sc2;
      u2 *= sc2;
    }
    m = mnew;
  }
  // Add one element y given mk = m*log2e (and mk2 = mk*inv_temp for ENT == 2).
  __device__ __forceinline__ void add(float y, float mk, float k2, float mk2) {
    const float p = ex2f(fmaf(y, kLog2e, -mk));
    s += p;
    if (ENT == 1) u = fmaf(p, y, u);
    if (ENT == 2) {
      const float p2 = ex2f(fmaf(y, k2, -mk2));
      s2 += p2;
      u2 = fmaf(p2, y, u2);
    }
  }
};

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct RowStats {
  float M, S, U, S2, U2;
};

// Per-token quantities produced by the epilogue.
struct TokenOut {
  float lp, entropy, lse, grad_coef, loss_term;
};

// Everything after the vocabulary reduction, per token n = (b, t).
// Follows train_modules/__init__.py:161-180 (old log-probs, ratio, clip, surrogate,
// mask) and adds beta*k3 against ref_logps.  grad_coef = mask*w/temperature with
//   w = A*ratio*sel - beta*(1 - e^(ref - lp)),
// sel = 1 where the unclipped branch is the active minimum (closed clip interval
// included), so that dlogits = (grad_scale/total_valid)*grad_coef*(softmax - onehot).
// Per-token side inputs of the epilogue (old == lp when no old log-probs are given).
struct TokenSide {
  float mask, adv, old, ref;
  bool has_old, has_ref;
};

template <int ENT>
__device__ __forceinline__ TokenOut token_epilogue_core(const KernelParams& p, const RowStats& st, float yc,
                                                        const TokenSide& sd) {
  TokenOut o;
  const float lnS = logf(st.S);
  o.lse = st.M + lnS;
  o.lp = (yc - o.lse) * p.inv_temperature;
  if (ENT == 1) {
    o.entropy = o.lse - st.U / st.S;
  } else if (ENT == 2) {
    // softmax(y/temperature): lse2 = M/temp + ln S2, E[y/temp] = U2/(temp*S2)
    o.entropy = st.M * p.inv_temperature + logf(st.S2) - p.inv_temperature * st.U2 / st.S2;
  } else {
    o.entropy = 0.f;
  }
  const float m = sd.mask, A = sd.adv;
  if (p.ce_loss) {
    // masked cross-entropy (plugins/sft/jax/sft_module.py:36-41): loss_t = -lp_t, d loss_t / d lp_t = -1
    o.loss_term = -m * o.lp;
    o.grad_coef = m * p.inv_temperature;
    return o;
  }
  const float old = sd.has_old ? sd.old : o.lp;
  const float ratio = expf(o.lp - old);
  const float clipped = fminf(fmaxf(ratio, p.clip_lo), p.clip_hi);
  const float ppo = fminf(ratio * A, clipped * A);
  float sel;
  if (ratio > p.clip_hi)
    sel = (A < 0.f) ? 1.f : 0.f;
  else if (ratio < p.clip_lo)
    sel = (A > 0.f) ? 1.f : 0.f;
  else
    sel = 1.f;
  float term = -ppo;
  float w = A * ratio * sel;
  if (sd.has_ref && p.beta != 0.f) {
    const float d = sd.ref - o.lp;
    const float ed = expf(d);
    term += p.beta * (ed - d - 1.0f);
    w -= p.beta * (1.0f - ed);
  }
  o.loss_term = m * term;
  o.grad_coef = m * w * p.inv_temperature;
  return o;
}

// Log-sum-exp of y/temperature (residual of the entropy gradient): the row's lse at temperature 1, from the
// second pair of sums otherwise; NaN when those were not accumulated (temperature != 1 without the entropy).
template <int ENT>
__device__ __forceinline__ float scaled_lse(const KernelParams& p, const RowStats& st, float lse) {
  if (ENT == 2) return st.M * p.inv_temperature + logf(st.S2);
  return p.inv_temperature == 1.0f ? lse : __int_as_float(0x7fc00000);
}

__device__ __forceinline__ TokenSide load_token_side(const KernelParams& p, int64_t n, int64_t b) {
  TokenSide sd;
  sd.mask = p.mask ? p.mask[n] : 1.0f;
  sd.adv = p.advantages ? p.advantages[p.adv_per_token ? n : b] : 0.0f;
  sd.has_old = p.old_logps != nullptr;
  sd.old = sd.has_old ? p.old_logps[n] : 0.f;
  sd.has_ref = p.ref_logps != nullptr;
  sd.ref = sd.has_ref ? p.ref_logps[n] : 0.f;
  return sd;
}

template <int ENT>
__device__ __forceinline__ TokenOut token_epilogue(const KernelParams& p, int64_t n, int64_t b,
                                                   const RowStats& st, float yc) {
  return token_epilogue_core<ENT>(p, st, yc, load_token_side(p, n, b));
}

}  // namespace grpo
