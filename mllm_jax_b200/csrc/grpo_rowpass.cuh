// Device code shared by every kernel that streams logits rows: row geometry, load/store flavours,
// L2 policies, block reductions, the forward pass over a row (online max / sum-exp) and the
// backward pass over a row (g*(softmax - onehot) in bf16).
#pragma once

#include "../../include/mllm_grpo.h"
#include "grpo_common.cuh"

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

// L2 eviction-priority policies for the kernel that reads each row twice: the first read asks L2
// to keep the line (evict_last), the second read and the gradient stores mark theirs evict_first.
__device__ __forceinline__ uint64_t policy_evict_last() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint4 ldg_hint(const uint4* p, uint64_t pol) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p), "l"(pol)
               : "memory");
  return v;
}
__device__ __forceinline__ void stg_hint(uint4* p, const uint4& v, uint64_t pol) {
  asm volatile("st.global.L2::cache_hint.v4.u32 [%0], {%1,%2,%3,%4}, %5;" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w), "l"(pol)
               : "memory");
}
// LD: 0 read-only streaming load, 1 coherent streaming load, 2 load with an L2 policy.
// LD 3: the row slice sits in shared memory (landed there by a bulk copy).
__device__ __forceinline__ uint4 lds_row(const uint4* p) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(p))));
  return v;
}
template <int LD>
__device__ __forceinline__ uint4 ld_row(const uint4* p, uint64_t pol) {
  if (LD == 0) return ldg_stream(p);
  if (LD == 1) return ldg_stream_rw(p);
  if (LD == 3) return lds_row(p);
  return ldg_hint(p, pol);
}
template <int LD>
__device__ __forceinline__ void st_row(uint4* p, const uint4& v, uint64_t pol) {
  if (LD == 2)
    stg_hint(p, v, pol);
  else
    stg_stream(p, v);
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
  if (CAP && ENT != 2) {
    // Whole batch inside the polynomial's range (the common case): packed-pair polynomial tanh, two lanes per issue.
    uint32_t mn2 = v[0].x;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      if (i) mn2 = bf16x2_min(mn2, v[i].x);
      mn2 = bf16x2_min(mn2, v[i].y);
      mn2 = bf16x2_min(mn2, v[i].z);
      mn2 = bf16x2_min(mn2, v[i].w);
    }
    const float lo = fminf(bf16lo(mn2), bf16hi(mn2)), hi = fmaxf(bf16lo(mx2), bf16hi(mx2));
    if (lo >= -sc.near && hi <= sc.near) {
      const f32x2 kk = pack2(kLog2e, kLog2e), nmk = pack2(-mk, -mk);
      f32x2 s2 = pack2(0.f, 0.f), u2 = pack2(0.f, 0.f);
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const f32x2 y = sc.y2_near(pack2(bf16lo(w[j]), bf16hi(w[j])));
          float t0, t1;
          unpack2(fma2(y, kk, nmk), t0, t1);
          const f32x2 p = pack2(ex2f(t0), ex2f(t1));
          s2 = add2(s2, p);
          if (ENT == 1) u2 = fma2(p, y, u2);
        }
      }
      float a, b;
      unpack2(s2, a, b);
      acc.s += a + b;
      if (ENT == 1) {
        unpack2(u2, a, b);
        acc.u += a + b;
      }
      return;
    }
  }
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

// First streaming pass over one row: every thread returns the row's (M, S, U[, S2, U2]).
template <int THREADS, int UNROLL, int ENT, bool CAP, int LD>
__device__ __forceinline__ RowStats row_pass1(const uint16_t* row16, int64_t V, float inv_temp, const SoftCap& sc,
                                              float* red, uint64_t pol) {
  const int tid = threadIdx.x;
  const float k2 = kLog2e * inv_temp;
  RowAcc<ENT> acc;
  acc.init();
  const RowSplit sp(row16, V);
  if (tid < sp.head) {
    fold_scalar<ENT, CAP>(acc, __uint_as_float(uint32_t(row16[tid]) << 16), inv_temp, k2, sc);
  }
  if (tid < sp.tail) {
    const int64_t j = sp.head + (sp.nvec << 3) + tid;
    fold_scalar<ENT, CAP>(acc, __uint_as_float(uint32_t(row16[j]) << 16), inv_temp, k2, sc);
  }
  const uint4* vec = reinterpret_cast<const uint4*>(row16 + sp.head);
  int64_t i = tid;
  constexpr int64_t kStep = int64_t(UNROLL) * THREADS;
  for (; i + kStep - THREADS < sp.nvec; i += kStep) {
    uint4 v[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) v[u] = ld_row<LD>(vec + i + int64_t(u) * THREADS, pol);
    fold_vectors<ENT, CAP, UNROLL>(acc, v, inv_temp, k2, sc);
  }
  if constexpr (UNROLL > 8) {  // batches of 10 are only chosen where next to nothing is left over
    for (; i < sp.nvec; i += THREADS) {
      uint4 v[1];
      v[0] = ld_row<LD>(vec + i, pol);
      fold_vectors<ENT, CAP, 1>(acc, v, inv_temp, k2, sc);
    }
  } else if (UNROLL > 1 && i < sp.nvec) {
    // Tail (fewer than UNROLL vectors left for this thread): all of them requested at once, one latency
    // period instead of one per vector, then folded one by one so that nothing is computed on padding.
    uint4 v[UNROLL - 1];
#pragma unroll
    for (int u = 0; u < UNROLL - 1; ++u)
      if (i + int64_t(u) * THREADS < sp.nvec) v[u] = ld_row<LD>(vec + i + int64_t(u) * THREADS, pol);
#pragma unroll
    for (int u = 0; u < UNROLL - 1; ++u) {
      if (i + int64_t(u) * THREADS < sp.nvec) {
        const uint4 one[1] = {v[u]};
        fold_vectors<ENT, CAP, 1>(acc, one, inv_temp, k2, sc);
      }
    }
  }
  // Block reduction with ONE barrier: warps merge (m, s, u) by shuffles, lane 0 parks the warp's
  // result in shared memory, and after the barrier every warp merges the per-warp entries again by
  // shuffles.  `red` must hold 5 floats per warp (160 floats).
  constexpr int NW = THREADS / 32;
  const int lane = tid & 31, warp = tid >> 5;
  const float Mw = warp_max(acc.m);
  const float dw = (acc.m - Mw) * kLog2e;
  const float sw = ex2f(dw);
  const float Sw = warp_sum(acc.s * sw);
  float Uw = 0.f, S2w = 0.f, U2w = 0.f;
  if (ENT == 1) Uw = warp_sum(acc.u * sw);
  if (ENT == 2) {
    const float sw2 = ex2f(dw * inv_temp);
    S2w = warp_sum(acc.s2 * sw2);
    U2w = warp_sum(acc.u2 * sw2);
  }
  if (lane == 0) {
    red[warp] = Mw;
    red[32 + warp] = Sw;
    if (ENT == 1) red[64 + warp] = Uw;
    if (ENT == 2) {
      red[96 + warp] = S2w;
      red[128 + warp] = U2w;
    }
  }
  __syncthreads();
  const float m_in = lane < NW ? red[lane] : kNegInit;
  RowStats st;
  st.M = warp_max(m_in);
  const float db = (m_in - st.M) * kLog2e;
  const float sb = ex2f(db);
  st.S = warp_sum(lane < NW ? red[32 + lane] * sb : 0.f);
  st.U = 0.f;
  st.S2 = 0.f;
  st.U2 = 0.f;
  if (ENT == 1) st.U = warp_sum(lane < NW ? red[64 + lane] * sb : 0.f);
  if (ENT == 2) {
    const float sb2 = ex2f(db * inv_temp);
    st.S2 = warp_sum(lane < NW ? red[96 + lane] * sb2 : 0.f);
    st.U2 = warp_sum(lane < NW ? red[128 + lane] * sb2 : 0.f);
  }
  // A logit of -inf has probability 0 but poisons the entropy sums with 0 * -inf.  The reference's
  // p*log(p + 1e-9) is 0 there (MLLM_JAX/train_modules/__init__.py:138), so such a row (rare: every
  // thread sees the same NaN and takes the branch together) sums e*y once more with p == 0 skipped.
  if ((ENT == 1 && st.U != st.U) || (ENT == 2 && st.U2 != st.U2)) {
    const float scale = ENT == 2 ? k2 : kLog2e;
    const float mk = st.M * scale;
    float u = 0.f;
    for (int64_t j = tid; j < V; j += THREADS) {
      uint16_t raw;
      if (LD == 3) {
        raw = row16[j];
      } else {
        asm volatile("ld.global.u16 %0, [%1];" : "=h"(raw) : "l"(row16 + j));
      }
      const float x = __uint_as_float(uint32_t(raw) << 16);
      const float y = CAP ? sc.y(x) : x;
      const float e = ex2f(fmaf(y, scale, -mk));
      if (e > 0.f) u = fmaf(e, y, u);
    }
    __syncthreads();  // everyone has read the first reduction's entries
    const float uw = warp_sum(u);
    if (lane == 0) red[warp] = uw;
    __syncthreads();
    const float tot = warp_sum(lane < NW ? red[lane] : 0.f);
    if (ENT == 1) st.U = tot;
    if (ENT == 2) st.U2 = tot;
  }
  return st;
}

// Chosen logit of a token: global id -> local column (clamped into the vocabulary if out of range).
template <bool CAP>
__device__ __forceinline__ float chosen_logit(const KernelParams& p, int64_t n, const uint16_t* row16,
                                              const SoftCap& sc, bool* mine, int64_t* cl_out) {
  int64_t c = p.chosen_ids[n];
  if (c < 0 || c >= p.vocab_total) {
    c = c < 0 ? 0 : p.vocab_total - 1;
    if (p.device_status) atomicOr(p.device_status, MLLM_GRPO_DEV_ID_CLAMPED);
  }
  const int64_t cl = c - p.vocab_start;
  *cl_out = cl;
  *mine = (cl >= 0 && cl < p.vocab);
  float yc = 0.f;
  if (*mine) {
    yc = __uint_as_float(uint32_t(row16[cl]) << 16);
    if (CAP) yc = sc.y(yc);
  }
  return yc;
}

// Second streaming pass over one row: dlogits = g*(softmax - onehot) (times dy/dx with the soft-cap)
// in bf16.  g == 0 writes exact zeros without reading the logits.
// LDSRC: load flavour of the source row when it differs from the store flavour LD (3 = shared memory).
// ENTG adds cot * dH/dlogits, H the entropy of softmax(y/temperature):
//   dH/dy_j = -(1/temp) * q_j * ((y_j/temp - lse2) + H),  q = softmax(y/temp), lse2 = log-sum-exp of y/temp.
struct EntropyGrad {
  float cot, H, lse2, inv_temp;
};
template <int THREADS, int UNROLL, bool CAP, int LD, int LDSRC = -1, bool ENTG = false>
__device__ __forceinline__ void row_pass2(const uint16_t* x16, uint16_t* d16, int64_t V, float g, float lse,
                                          int64_t cl, const SoftCap& sc, uint64_t pol,
                                          const EntropyGrad eg = EntropyGrad{0.f, 0.f, 0.f, 1.f}) {
  const int tid = threadIdx.x;
  const RowSplit sp(d16, V);  // the caller guarantees logits and dlogits rows share alignment
  uint4* dvec = reinterpret_cast<uint4*>(d16 + sp.head);

  if (g == 0.f && (!ENTG || eg.cot == 0.f)) {
    // Unscored row, masked token or zero advantage: exact zeros, logits are not read.
    if (tid < sp.head) d16[tid] = 0;
    if (tid < sp.tail) d16[sp.head + (sp.nvec << 3) + tid] = 0;
    const uint4 z = make_uint4(0, 0, 0, 0);
    for (int64_t i = tid; i < sp.nvec; i += THREADS) st_row<LD>(dvec + i, z, pol);
    return;
  }

  // g*e^(y-lse) = sign(g) * 2^(y*log2e - lse*log2e + log2|g|): the scale rides in the exponent.
  const float off = lg2f(fabsf(g)) - lse * kLog2e;
  const uint32_t sgn = g < 0.f ? 0x80008000u : 0u;

  auto one = [&](float x, int64_t j) -> float {  // scalar path: signed f32 result
    float d;
    if (ENTG) {
      const float y = CAP ? sc.y(x) : x;
      d = g * ex2f((y - lse) * kLog2e);
      if (j == cl) d -= g;
      const float z = fmaf(y, eg.inv_temp, -eg.lse2);
      const float q = ex2f(z * kLog2e);
      if (q > 0.f) d -= eg.cot * eg.inv_temp * q * (z + eg.H);
      if (CAP) d *= sc.dydx(y);
    } else if (CAP) {
      const float y = sc.y(x);
      d = ex2f(fmaf(y, kLog2e, off));
      d = g < 0.f ? -d : d;
      if (j == cl) d -= g;
      d *= sc.dydx(y);
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
  // Vector that holds the chosen column (or -1).
  const int64_t cv = (cl >= sp.head && cl < sp.head + (sp.nvec << 3)) ? ((cl - sp.head) >> 3) : -1;

  auto do_vec = [&](const uint4& v, int64_t idx) -> uint4 {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[4];
    bool near = false;
    if (CAP && !ENTG && idx != cv) {
      const uint32_t mx2 = bf16x2_max(bf16x2_max(w[0], w[1]), bf16x2_max(w[2], w[3]));
      const uint32_t mn2 = bf16x2_min(bf16x2_min(w[0], w[1]), bf16x2_min(w[2], w[3]));
      near = fminf(bf16lo(mn2), bf16hi(mn2)) >= -sc.near && fmaxf(bf16lo(mx2), bf16hi(mx2)) <= sc.near;
    }
    if (!CAP && !ENTG && idx != cv) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float a = ex2f(fmaf(bf16lo(w[j]), kLog2e, off));
        const float c = ex2f(fmaf(bf16hi(w[j]), kLog2e, off));
        o[j] = pack_bf16x2(a, c) ^ sgn;
      }
    } else if (CAP && near) {
      // all eight inside the polynomial's range, chosen column elsewhere: packed-pair polynomial tanh
      const f32x2 kk = pack2(kLog2e, kLog2e), oo = pack2(off, off);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const f32x2 y = sc.y2_near(pack2(bf16lo(w[j]), bf16hi(w[j])));
        float t0, t1, a, c;
        unpack2(fma2(y, kk, oo), t0, t1);
        unpack2(mul2(pack2(ex2f(t0), ex2f(t1)), sc.dydx2(y)), a, c);
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
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
  };

  // never the non-coherent path: the output may alias the input
  constexpr int LDX = LDSRC >= 0 ? LDSRC : ((LD == 0) ? 1 : LD);
  int64_t i = tid;
  constexpr int64_t kStep = int64_t(UNROLL) * THREADS;
  for (; i + kStep - THREADS < sp.nvec; i += kStep) {
    uint4 v[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) v[u] = ld_row<LDX>(xvec + i + int64_t(u) * THREADS, pol);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      st_row<LD>(dvec + i + int64_t(u) * THREADS, do_vec(v[u], i + int64_t(u) * THREADS), pol);
  }
  if constexpr (UNROLL > 8) {
    for (; i < sp.nvec; i += THREADS) {
      const uint4 v = ld_row<LDX>(xvec + i, pol);
      st_row<LD>(dvec + i, do_vec(v, i), pol);
    }
  } else if (UNROLL > 1 && i < sp.nvec) {  // tail: every remaining load in flight at once
    uint4 v[UNROLL - 1];
#pragma unroll
    for (int u = 0; u < UNROLL - 1; ++u)
      if (i + int64_t(u) * THREADS < sp.nvec) v[u] = ld_row<LDX>(xvec + i + int64_t(u) * THREADS, pol);
#pragma unroll
    for (int u = 0; u < UNROLL - 1; ++u)
      if (i + int64_t(u) * THREADS < sp.nvec)
        st_row<LD>(dvec + i + int64_t(u) * THREADS, do_vec(v[u], i + int64_t(u) * THREADS), pol);
  }
}

}  // namespace grpo
