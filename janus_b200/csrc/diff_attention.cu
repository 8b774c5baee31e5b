// Differential attention over the paged cache, with a short causal convolution on the
// projected q, k and v, rotation of a leading part of every vector, a sliding window that
// keeps a sequence's first keys, and the per-head unit norm of the combined maps.
//
// A query head has two maps, each an attention of its own over the same values:
//   q row: [head][map][d]   k row: [kv head][map][d]   v row: [kv head][e]
// The key cache is [page][2 G][PAGE][d] (a kv head's two maps are neighbouring "heads"),
// the value cache [page][G][PAGE][e]; block_table[seq][i] is the page of keys [i PAGE, (i+1) PAGE).
//
//   conv_rope_cache:  y_t = sum_j w[c, j] u_(t - taps + 1 + j) per channel c, where u before the
//                     step's first token comes from the sequence's state (its last taps - 1
//                     projected values) and is zero before the sequence's start; then the first
//                     `rot` dimensions of every q and k vector turn by the token's position (pairs
//                     (i, i + rot/2), cos and sin from a table); q goes out in float32, k and v
//                     into the cache.
//   conv_state_update: the state takes the step's last projected values (steps of one token per sequence do
//                     this inside conv_rope_cache).
//   diff_attention:   one block per (token, query head); both maps' online softmax over the visible
//                     keys j <= i with (i - j < window or j < keep_first), in chunks of 32 keys that
//                     start at multiples of 32 of the key index and go to the block's warps in turn (so
//                     the result does not depend on how a sequence was cut into steps); o = a1 - lambda a2,
//                     divided by its root mean square over the head's e values (eps inside the root),
//                     times out_scale.  It serves single tokens in both dtypes and every float32 step.
// Scores, softmax weights and the sums are float32 whatever the cache holds.
#include <math_constants.h>
#include <stdio.h>

#include "common.cuh"

namespace {

typedef __nv_bfloat16 bf16;

template <typename TC>
__global__ void conv_rope_cache_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ conv_w, int taps,
                                       float* __restrict__ conv_state, int update_state, const int* __restrict__ token_seq,
                                       const int* __restrict__ q_start, const int* __restrict__ seq_slot,
                                       const int* __restrict__ positions, const float* __restrict__ cos_sin, int rot,
                                       float* __restrict__ q_out, const int* __restrict__ dest, TC* __restrict__ k_cache,
                                       TC* __restrict__ v_cache, int H, int G, int d, int e, int page_size) {
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int t = blockIdx.x;
  const int seq = token_seq[t];
  const int local = t - q_start[seq];                 // tokens of this sequence before t within the step
  const int Cq = H * 2 * d, Ck = G * 2 * d, Cv = G * e, C = Cq + Ck + Cv;
  float* st = (conv_w && taps > 1) ? conv_state + (size_t)seq_slot[seq] * (taps - 1) * C : nullptr;
  const int half = rot >> 1;
  const float* cs = cos_sin ? cos_sin + (size_t)positions[t] * half * 2 : nullptr;
  const int dst = dest[t];
  const int page = dst / page_size, off = dst % page_size;

  auto convolved = [&](int c) -> float {
    if (!conv_w) return proj[(size_t)t * ld + c];
    float y = 0.0f;
    for (int j = 0; j < taps; ++j) {
      const int back = taps - 1 - j;                  // how many tokens before t
      float u;
      if (back <= local) u = proj[(size_t)(t - back) * ld + c];
      else u = st[(size_t)(taps - 1 - (back - local)) * C + c];
      y = fmaf(conv_w[(size_t)c * taps + j], u, y);
    }
    return y;
  };
  auto put = [&](int c, float y) {
    if (c < Cq) {
      q_out[(size_t)t * Cq + c] = y;
    } else if (c < Cq + Ck) {
      const int kc = c - Cq, vec = kc / d, i = kc % d;
      k_cache[(((size_t)page * 2 * G + vec) * page_size + off) * d + i] = jb::from_f32<TC>(y);
    } else {
      const int vc = c - Cq - Ck, g = vc / e, i = vc % e;
      v_cache[(((size_t)page * G + g) * page_size + off) * e + i] = jb::from_f32<TC>(y);
    }
  };
  // steps of one token per sequence: the thread that read a channel's state also moves it on by that token
  auto shift = [&](int c) {
    if (!update_state || st == nullptr) return;
    for (int i = 0; i + 1 < taps - 1; ++i) st[(size_t)i * C + c] = st[(size_t)(i + 1) * C + c];
    st[(size_t)(taps - 2) * C + c] = proj[(size_t)t * ld + c];
  };
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  if (c >= Cq + Ck || cs == nullptr) {
    put(c, convolved(c));
    shift(c);
    return;
  }
  const int i = (c < Cq ? c : c - Cq) % d;
  if (i >= rot) {
    put(c, convolved(c));
    shift(c);
  } else if (i < half) {
    const float a = convolved(c), b = convolved(c + half);
    const float co = cs[2 * i], si = cs[2 * i + 1];
    put(c, a * co - b * si);
    put(c + half, b * co + a * si);
    shift(c);
    shift(c + half);
  }
}

// Four channels a thread (sizes and rotated dimensions that are multiples of 4 or 8, 16-byte aligned rows): the same
// sums in the same order as the kernel above, with 16-byte loads of the projections and stores of q, and one set of
// index arithmetic per four channels.
template <typename TC>
__device__ __forceinline__ void store4c(TC* p, float4 v);
template <>
__device__ __forceinline__ void store4c<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <>
__device__ __forceinline__ void store4c<bf16>(bf16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<unsigned*>(&a);
  raw.y = *reinterpret_cast<unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

template <typename TC>
__global__ void conv_rope_cache_vec_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ conv_w, int taps,
                                           float* __restrict__ conv_state, int update_state, const int* __restrict__ token_seq,
                                           const int* __restrict__ q_start, const int* __restrict__ seq_slot,
                                           const int* __restrict__ positions, const float* __restrict__ cos_sin, int rot,
                                           float* __restrict__ q_out, const int* __restrict__ dest, TC* __restrict__ k_cache,
                                           TC* __restrict__ v_cache, int H, int G, int d, int e, int page_size) {
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int t = blockIdx.x;
  const int Cq = H * 2 * d, Ck = G * 2 * d, Cv = G * e, C = Cq + Ck + Cv;
  const int c = 4 * (blockIdx.y * blockDim.x + threadIdx.x);
  if (c >= C) return;
  const int seq = token_seq[t];
  const int local = t - q_start[seq];
  float* st = (conv_w && taps > 1) ? conv_state + (size_t)seq_slot[seq] * (taps - 1) * C : nullptr;
  const int half = rot >> 1;
  const float* cs = cos_sin ? cos_sin + (size_t)positions[t] * half * 2 : nullptr;
  const int dst = dest[t];
  const int page = dst / page_size, off = dst % page_size;

  auto convolved = [&](int c0) -> float4 {
    if (!conv_w) return *reinterpret_cast<const float4*>(proj + (size_t)t * ld + c0);
    float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < taps; ++j) {
      const int back = taps - 1 - j;
      const float4 u = back <= local ? *reinterpret_cast<const float4*>(proj + (size_t)(t - back) * ld + c0)
                                     : *reinterpret_cast<const float4*>(st + (size_t)(taps - 1 - (back - local)) * C + c0);
      const float* w = conv_w + (size_t)c0 * taps + j;
      y.x = fmaf(w[0], u.x, y.x);
      y.y = fmaf(w[taps], u.y, y.y);
      y.z = fmaf(w[2 * taps], u.z, y.z);
      y.w = fmaf(w[3 * taps], u.w, y.w);
    }
    return y;
  };
  auto put = [&](int c0, float4 y) {
    if (c0 < Cq) {
      *reinterpret_cast<float4*>(q_out + (size_t)t * Cq + c0) = y;
    } else if (c0 < Cq + Ck) {
      const int kc = c0 - Cq, vec = kc / d, i = kc % d;
      store4c<TC>(k_cache + (((size_t)page * 2 * G + vec) * page_size + off) * d + i, y);
    } else {
      const int vc = c0 - Cq - Ck, g = vc / e, i = vc % e;
      store4c<TC>(v_cache + (((size_t)page * G + g) * page_size + off) * e + i, y);
    }
  };
  auto shift = [&](int c0) {
    if (!update_state || st == nullptr) return;
    for (int i = 0; i + 1 < taps - 1; ++i)
      *reinterpret_cast<float4*>(st + (size_t)i * C + c0) = *reinterpret_cast<const float4*>(st + (size_t)(i + 1) * C + c0);
    *reinterpret_cast<float4*>(st + (size_t)(taps - 2) * C + c0) = *reinterpret_cast<const float4*>(proj + (size_t)t * ld + c0);
  };
  if (c >= Cq + Ck || cs == nullptr) {
    put(c, convolved(c));
    shift(c);
    return;
  }
  const int i = (c < Cq ? c : c - Cq) % d;
  if (i >= rot) {
    put(c, convolved(c));
    shift(c);
  } else if (i < half) {
    const float4 a = convolved(c), b = convolved(c + half);
    const float4 t0 = *reinterpret_cast<const float4*>(cs + 2 * i), t1 = *reinterpret_cast<const float4*>(cs + 2 * i + 4);
    // (cos, sin) of the pairs i, i + 1 in t0 and of i + 2, i + 3 in t1
    put(c, make_float4(a.x * t0.x - b.x * t0.y, a.y * t0.z - b.y * t0.w, a.z * t1.x - b.z * t1.y, a.w * t1.z - b.w * t1.w));
    put(c + half, make_float4(b.x * t0.x + a.x * t0.y, b.y * t0.z + a.y * t0.w, b.z * t1.x + a.z * t1.y, b.w * t1.z + a.w * t1.w));
    shift(c);
    shift(c + half);
  }
}

__global__ void conv_state_update_kernel(const float* __restrict__ proj, int ld, float* __restrict__ conv_state, int taps,
                                         const int* __restrict__ q_start, const int* __restrict__ seq_slot, int C) {
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int seq = blockIdx.x;
  const int t0 = q_start[seq], n = q_start[seq + 1] - t0;
  float* st = conv_state + (size_t)seq_slot[seq] * (taps - 1) * C;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    for (int i = 0; i < taps - 1; ++i) {           // new[i] is the value n - (taps - 1) + i tokens into the step
      const int li = n - (taps - 1) + i;
      st[(size_t)i * C + c] = li >= 0 ? proj[(size_t)(t0 + li) * ld + c] : st[(size_t)(i + n) * C + c];
    }
  }
}

// warps of a block at most, by the value columns a lane holds (a block of 32 warps leaves a thread 64 registers,
// which the kernel for up to 64 value columns fits into)
__host__ __device__ constexpr int max_warps(int ej) { return ej <= 2 ? 32 : 16; }

// dot products of one key's two maps with the query's two maps, 8 (bf16) or 4 (float) elements a load when
// the rows allow it
template <typename TC>
__device__ __forceinline__ void dot2(const float* __restrict__ qw, const TC* __restrict__ k1, const TC* __restrict__ k2,
                                     int d, bool vec, float& d1, float& d2);

template <>
__device__ __forceinline__ void dot2<float>(const float* __restrict__ qw, const float* __restrict__ k1,
                                            const float* __restrict__ k2, int d, bool vec, float& d1, float& d2) {
  d1 = d2 = 0.0f;
  if (vec) {
    for (int i = 0; i < d; i += 4) {
      const float4 a = *reinterpret_cast<const float4*>(k1 + i), b = *reinterpret_cast<const float4*>(k2 + i);
      d1 = fmaf(qw[i], a.x, d1); d1 = fmaf(qw[i + 1], a.y, d1); d1 = fmaf(qw[i + 2], a.z, d1); d1 = fmaf(qw[i + 3], a.w, d1);
      d2 = fmaf(qw[d + i], b.x, d2); d2 = fmaf(qw[d + i + 1], b.y, d2); d2 = fmaf(qw[d + i + 2], b.z, d2);
      d2 = fmaf(qw[d + i + 3], b.w, d2);
    }
  } else {
    for (int i = 0; i < d; ++i) {
      d1 = fmaf(qw[i], k1[i], d1);
      d2 = fmaf(qw[d + i], k2[i], d2);
    }
  }
}

template <>
__device__ __forceinline__ void dot2<bf16>(const float* __restrict__ qw, const bf16* __restrict__ k1,
                                           const bf16* __restrict__ k2, int d, bool vec, float& d1, float& d2) {
  d1 = d2 = 0.0f;
  if (vec) {
#pragma unroll 4
    for (int i = 0; i < d; i += 8) {
      const uint4 a = *reinterpret_cast<const uint4*>(k1 + i), b = *reinterpret_cast<const uint4*>(k2 + i);
      const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&a);
      const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float2 af = __bfloat1622float2(ap[u]), bf = __bfloat1622float2(bp[u]);
        d1 = fmaf(qw[i + 2 * u], af.x, d1);
        d1 = fmaf(qw[i + 2 * u + 1], af.y, d1);
        d2 = fmaf(qw[d + i + 2 * u], bf.x, d2);
        d2 = fmaf(qw[d + i + 2 * u + 1], bf.y, d2);
      }
    }
  } else {
    for (int i = 0; i < d; ++i) {
      d1 = fmaf(qw[i], __bfloat162float(k1[i]), d1);
      d2 = fmaf(qw[d + i], __bfloat162float(k2[i]), d2);
    }
  }
}

// A lane's EJ neighbouring value columns of one row, in one load when the row's length is a multiple of EJ
template <int EJ>
__device__ __forceinline__ void load_columns_f32(const float* __restrict__ vr, int c0, int e, bool vec, float (&v)[EJ]) {
  if (vec && c0 < e) {
    if (EJ == 2) {
      const float2 t = *reinterpret_cast<const float2*>(vr + c0);
      v[0] = t.x; v[1] = t.y;
    } else {
#pragma unroll
      for (int j = 0; j < EJ; j += 4) {
        const float4 t = *reinterpret_cast<const float4*>(vr + c0 + j);
        v[j] = t.x; v[j + 1] = t.y; v[j + 2] = t.z; v[j + 3] = t.w;
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < EJ; ++j) v[j] = c0 + j < e ? vr[c0 + j] : 0.0f;
  }
}
template <int EJ>
__device__ __forceinline__ void load_columns_bf16(const bf16* __restrict__ vr, int c0, int e, bool vec, float (&v)[EJ]) {
  if (vec && c0 < e) {
    unsigned raw[EJ / 2];
    if (EJ == 2) raw[0] = *reinterpret_cast<const unsigned*>(vr + c0);
    else if (EJ == 4) *reinterpret_cast<uint2*>(raw) = *reinterpret_cast<const uint2*>(vr + c0);
    else *reinterpret_cast<uint4*>(raw) = *reinterpret_cast<const uint4*>(vr + c0);
#pragma unroll
    for (int j = 0; j < EJ / 2; ++j) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[j]));
      v[2 * j] = f.x;
      v[2 * j + 1] = f.y;
    }
  } else {
#pragma unroll
    for (int j = 0; j < EJ; ++j) v[j] = c0 + j < e ? __bfloat162float(vr[c0 + j]) : 0.0f;
  }
}
template <typename TC, int EJ> struct Columns;
template <int EJ> struct Columns<float, EJ> {
  static __device__ __forceinline__ void load(const float* vr, int c0, int e, bool vec, float (&v)[EJ]) {
    load_columns_f32<EJ>(vr, c0, e, vec, v);
  }
};
template <int EJ> struct Columns<bf16, EJ> {
  static __device__ __forceinline__ void load(const bf16* vr, int c0, int e, bool vec, float (&v)[EJ]) {
    load_columns_bf16<EJ>(vr, c0, e, vec, v);
  }
};

__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// One block per (token, query head); its warps take the chunks of 32 keys in turn (chunk n goes to warp
// n mod warps) and their partial results (maximum, sum, weighted values of each map) meet in warp order.
// EJ: value columns a lane holds, EJ lane .. EJ lane + EJ - 1 (e <= 32 EJ)
template <typename TC, typename TO, int EJ>
__global__ void __launch_bounds__(max_warps(EJ) * 32) diff_attention_kernel(
    const float* __restrict__ q, const TC* __restrict__ k_cache, const TC* __restrict__ v_cache, TO* __restrict__ out,
    const int* __restrict__ block_table, const int* __restrict__ token_seq, const int* __restrict__ positions, int T, int H,
    int G, int d, int e, int page_size, int max_pages, int window, int keep_first, float scale, float lambda, float eps,
    float out_scale, int vec) {
  extern __shared__ float smem[];                    // q [2 d], then per warp: m1 l1 m2 l2, a1 [32 EJ], a2 [32 EJ]
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int t = blockIdx.x / H, h = blockIdx.x % H;
  const int g = h / (H / G);
  const int pos = positions[t];
  const int* pages = block_table + (size_t)token_seq[t] * max_pages;
  const int kstart = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const bool prefetch = (vec & 4) != 0;
  const bool vvec = (vec & 2) != 0 && e % EJ == 0;         // a lane's EJ neighbouring value columns come in one load
  float* qw = smem;
  for (int i = threadIdx.x; i < 2 * d; i += blockDim.x) qw[i] = q[((size_t)t * H + h) * 2 * d + i];
  __syncthreads();

  float m1 = -CUDART_INF_F, l1 = 0.0f, m2 = -CUDART_INF_F, l2 = 0.0f;
  float a1[EJ], a2[EJ];
#pragma unroll
  for (int j = 0; j < EJ; ++j) a1[j] = a2[j] = 0.0f;

  auto chunk = [&](int c0) {
    const int key = c0 + lane;
    const bool valid = key <= pos && (key >= kstart || key < keep_first);
    float s1 = -CUDART_INF_F, s2 = -CUDART_INF_F;
    if (prefetch) {
      // what the warp reads next is asked for now: this key's value row (needed once the scores are known) and
      // the two key rows of this lane's key in the warp's next chunk
      const int nkey = key + 32 * warps;
      if (nkey <= pos) {
        const int npage = pages[nkey / page_size], nrow = nkey % page_size;
        const char* nk = reinterpret_cast<const char*>(k_cache + (((size_t)npage * 2 * G + 2 * g) * page_size + nrow) * d);
        for (int b = 0; b < d * (int)sizeof(TC); b += 128) {
          prefetch_l2(nk + b);
          prefetch_l2(nk + (size_t)page_size * d * sizeof(TC) + b);
        }
      }
    }
    if (valid) {
      const int page = pages[key / page_size], row = key % page_size;
      const TC* k1 = k_cache + (((size_t)page * 2 * G + 2 * g) * page_size + row) * d;
      if (prefetch) {
        const char* vrow = reinterpret_cast<const char*>(v_cache + (((size_t)page * G + g) * page_size + row) * e);
        for (int b = 0; b < e * (int)sizeof(TC); b += 128) prefetch_l2(vrow + b);
      }
      float d1, d2;
      dot2<TC>(qw, k1, k1 + (size_t)page_size * d, d, (vec & 1) != 0, d1, d2);
      s1 = d1 * scale;
      s2 = d2 * scale;
    }
    const float n1 = fmaxf(m1, jb::warp_max(s1)), n2 = fmaxf(m2, jb::warp_max(s2));
    if (n1 == -CUDART_INF_F) return;                 // no visible key in this chunk or before (uniform)
    const float p1 = valid ? expf(s1 - n1) : 0.0f, p2 = valid ? expf(s2 - n2) : 0.0f;
    const float c1 = expf(m1 - n1), c2 = expf(m2 - n2);   // exp(-inf) = 0 before the first key
    l1 = l1 * c1 + jb::warp_sum(p1);
    l2 = l2 * c2 + jb::warp_sum(p2);
#pragma unroll
    for (int j = 0; j < EJ; ++j) {
      a1[j] *= c1;
      a2[j] *= c2;
    }
    const unsigned seen = __ballot_sync(0xffffffffu, valid);
    if (page_size % 32 == 0) {
      // the chunk lies in one page, which is held because the chunk has a visible key: eight value rows are
      // loaded before their products are added, in key order (keys that are not seen carry the weight zero)
      const int page = pages[c0 / page_size];
      const TC* vbase = v_cache + (((size_t)page * G + g) * page_size + c0 % page_size) * e;
      const int kk_lo = __ffs(seen) - 1, kk_hi = 32 - __clz(seen);
      for (int kk0 = kk_lo & ~7; kk0 < kk_hi; kk0 += 8) {
        float vreg[8][EJ];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const TC* vr = vbase + (size_t)(kk0 + u) * e;
          Columns<TC, EJ>::load(vr, EJ * lane, e, vvec, vreg[u]);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float w1 = __shfl_sync(0xffffffffu, p1, kk0 + u), w2 = __shfl_sync(0xffffffffu, p2, kk0 + u);
#pragma unroll
          for (int j = 0; j < EJ; ++j) {
            a1[j] = fmaf(w1, vreg[u][j], a1[j]);
            a2[j] = fmaf(w2, vreg[u][j], a2[j]);
          }
        }
      }
    } else {
      for (int kk = 0; kk < 32; ++kk) {
        if (!((seen >> kk) & 1u)) continue;            // uniform across the warp
        const int key2 = c0 + kk;
        const int page = pages[key2 / page_size], row = key2 % page_size;
        const TC* vr = v_cache + (((size_t)page * G + g) * page_size + row) * e;
        const float w1 = __shfl_sync(0xffffffffu, p1, kk), w2 = __shfl_sync(0xffffffffu, p2, kk);
#pragma unroll
        for (int j = 0; j < EJ; ++j) {
          const int c = EJ * lane + j;
          if (c < e) {
            const float v = jb::to_f32(vr[c]);
            a1[j] = fmaf(w1, v, a1[j]);
            a2[j] = fmaf(w2, v, a2[j]);
          }
        }
      }
    }
    m1 = n1;
    m2 = n2;
  };

  // chunks are numbered by their place in the key index, so a key is always handled by the same warp of its
  // query's block and in the same order, however the sequence was cut into steps
  const int first_window_chunk = (kstart / 32) * 32;
  const int kept = min(keep_first, kstart);          // kept keys that the window has left behind
  for (int c0 = 32 * warp; c0 < kept && c0 < first_window_chunk; c0 += 32 * warps) chunk(c0);
  for (int c0 = first_window_chunk + 32 * warp; c0 <= pos; c0 += 32 * warps) chunk(c0);

  // the warps' parts meet in warp order in warp 0
  float* part = smem + 2 * d + (size_t)warp * (4 + 64 * EJ);
  if (lane == 0) {
    part[0] = m1; part[1] = l1; part[2] = m2; part[3] = l2;
  }
#pragma unroll
  for (int j = 0; j < EJ; ++j) {
    part[4 + 32 * j + lane] = a1[j];
    part[4 + 32 * EJ + 32 * j + lane] = a2[j];
  }
  __syncthreads();
  if (warp != 0) return;
  for (int w = 1; w < warps; ++w) {
    const float* pw = smem + 2 * d + (size_t)w * (4 + 64 * EJ);
    const float om1 = pw[0], ol1 = pw[1], om2 = pw[2], ol2 = pw[3];
    if (om1 == -CUDART_INF_F) continue;              // that warp saw no key
    const float n1 = fmaxf(m1, om1), n2 = fmaxf(m2, om2);
    const float c1 = expf(m1 - n1), e1 = expf(om1 - n1), c2 = expf(m2 - n2), e2 = expf(om2 - n2);
    l1 = l1 * c1 + ol1 * e1;
    l2 = l2 * c2 + ol2 * e2;
#pragma unroll
    for (int j = 0; j < EJ; ++j) {
      a1[j] = a1[j] * c1 + pw[4 + 32 * j + lane] * e1;
      a2[j] = a2[j] * c2 + pw[4 + 32 * EJ + 32 * j + lane] * e2;
    }
    m1 = n1;
    m2 = n2;
  }
  float o[EJ], ss = 0.0f;
#pragma unroll
  for (int j = 0; j < EJ; ++j) {
    o[j] = a1[j] / l1 - lambda * (a2[j] / l2);
    if (EJ * lane + j < e) ss += o[j] * o[j];
  }
  ss = jb::warp_sum(ss);
  const float rms = sqrtf(ss / (float)e + eps);
  TO* orow = out + ((size_t)t * H + h) * e;
#pragma unroll
  for (int j = 0; j < EJ; ++j) {
    const int c = EJ * lane + j;
    if (c < e) orow[c] = jb::from_f32<TO>((o[j] / rms) * out_scale);
  }
}

}  // namespace

// proj: float32 [T, ld], columns [q: H 2 d | k: G 2 d | v: G e]; conv_w: float32 [C, taps] or null (no convolution);
// conv_state: float32 [slots, taps - 1, C] (update_state: every sequence brings one token and the state takes it in
// the same launch; otherwise `jb_conv_state_update` follows); cos_sin: float32 [positions, rot / 2, 2] or null (no rotation);
// q_out: float32 [T, H 2 d]; dest[t] = page * page_size + row of token t in the caches (cache_dtype).
JB_EXPORT int jb_conv_rope_cache(const float* proj, int ld, const float* conv_w, int taps, float* conv_state,
                                 int update_state, const int* token_seq, const int* q_start, const int* seq_slot, const int* positions,
                                 const float* cos_sin, int rot, float* q_out, const int* dest, void* k_cache, void* v_cache,
                                 int cache_dtype, int T, int H, int G, int d, int e, int page_size, cudaStream_t stream) {
  if (T <= 0) return 0;
  JB_REFUSE(rot % 2 != 0 || rot > d || rot < 0, "conv_rope_cache: %d rotated dimensions do not fit vectors of %d", rot, d);
  JB_REFUSE(conv_w != nullptr && taps < 1, "conv_rope_cache: %d taps", taps);
  const int C = H * 2 * d + G * 2 * d + G * e;
  const int threads = C >= 1024 ? 256 : 128;
  const bool vec = d % 4 == 0 && e % 4 == 0 && rot % 8 == 0 && ld % 4 == 0 &&
                   (((uintptr_t)proj | (uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)conv_state |
                     (uintptr_t)cos_sin) & 15) == 0;
  if (vec) {
    const int vthreads = C / 4 >= 512 ? 256 : 128;
    jb::Launch vcfg(dim3(T, (C / 4 + vthreads - 1) / vthreads), dim3(vthreads), 0, stream);
    if (cache_dtype == JB_F32)
      return (int)cudaLaunchKernelEx(&vcfg.c, conv_rope_cache_vec_kernel<float>, proj, ld, conv_w, taps, conv_state,
                                     update_state, token_seq, q_start, seq_slot, positions, cos_sin, rot, q_out, dest,
                                     (float*)k_cache, (float*)v_cache, H, G, d, e, page_size);
    if (cache_dtype == JB_BF16)
      return (int)cudaLaunchKernelEx(&vcfg.c, conv_rope_cache_vec_kernel<bf16>, proj, ld, conv_w, taps, conv_state,
                                     update_state, token_seq, q_start, seq_slot, positions, cos_sin, rot, q_out, dest,
                                     (bf16*)k_cache, (bf16*)v_cache, H, G, d, e, page_size);
    return JB_ERR_BAD_DTYPE;
  }
  jb::Launch cfg(dim3(T, (C + threads - 1) / threads), dim3(threads), 0, stream);
  if (cache_dtype == JB_F32)
    return (int)cudaLaunchKernelEx(&cfg.c, conv_rope_cache_kernel<float>, proj, ld, conv_w, taps, conv_state, update_state, token_seq,
                                   q_start, seq_slot, positions, cos_sin, rot, q_out, dest, (float*)k_cache,
                                   (float*)v_cache, H, G, d, e, page_size);
  if (cache_dtype == JB_BF16)
    return (int)cudaLaunchKernelEx(&cfg.c, conv_rope_cache_kernel<bf16>, proj, ld, conv_w, taps, conv_state, update_state, token_seq,
                                   q_start, seq_slot, positions, cos_sin, rot, q_out, dest, (bf16*)k_cache, (bf16*)v_cache,
                                   H, G, d, e, page_size);
  return JB_ERR_BAD_DTYPE;
}

JB_EXPORT int jb_conv_state_update(const float* proj, int ld, float* conv_state, int taps, const int* q_start,
                                   const int* seq_slot, int n_seqs, int C, cudaStream_t stream) {
  if (n_seqs <= 0 || taps <= 1) return 0;
  jb::Launch cfg(dim3(n_seqs, (C + 255) / 256), dim3(256), 0, stream);
  return (int)cudaLaunchKernelEx(&cfg.c, conv_state_update_kernel, proj, ld, conv_state, taps, q_start, seq_slot, C);
}

// q: float32 [T, H 2 d]; out: [T, H e] in out_dtype; caches in cache_dtype; window 0 = every key.
JB_EXPORT int jb_diff_attention(const float* q, const void* k_cache, const void* v_cache, int cache_dtype, void* out,
                                int out_dtype, const int* block_table, const int* token_seq, const int* positions, int T,
                                int H, int G, int d, int e, int page_size, int max_pages, int window, int keep_first,
                                float scale, float lambda, float eps, float out_scale, cudaStream_t stream) {
  if (T <= 0) return 0;
  JB_REFUSE(G <= 0 || H % G != 0, "diff_attention: %d heads are not a multiple of %d key/value heads", H, G);
  JB_REFUSE(e < 1 || e > 256 || d < 1 || d > 1024, "diff_attention: sizes %d (keys) and %d (values) are not supported", d, e);
  JB_REFUSE((long long)T * H > 2147483647LL, "diff_attention: %d tokens of %d heads are too many blocks", T, H);
  // few (token, head) pairs (single tokens): a warp per chunk of 32 keys a query can see, up to 32 warps, so that
  // the chunks' loads are all in flight at once; prompts: four warps
  const int EJ_ = e <= 64 ? 2 : e <= 128 ? 4 : 8;
  const long long reach = (long long)max_pages * page_size;
  const long long keys = window > 0 ? (reach < (long long)window + keep_first ? reach : (long long)window + keep_first) : reach;
  // ... as long as all blocks still fit the SMs at once (a block's registers allow max_warps warps of them an SM)
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  const long long room = (long long)sms * max_warps(EJ_);
  int warps = 4;
  while (warps < max_warps(EJ_) && (long long)warps * 32 < keys && (long long)T * H * warps * 2 <= room) warps *= 2;
  static int forced = -1;                  // JANUS_DIFF_WARPS: warps of a block whatever the shape (experiments)
  if (forced < 0) {
    const char* env = getenv("JANUS_DIFF_WARPS");
    forced = env ? atoi(env) : 0;
  }
  if (forced > 0) warps = forced < max_warps(EJ_) ? forced : max_warps(EJ_);
  const size_t smem = (size_t)(2 * d + warps * (4 + 64 * EJ_)) * sizeof(float);
  const bool f32c = cache_dtype == JB_F32;
  // bit 0: key rows in 16-byte loads; bit 1: the value cache is aligned for a lane's columns in one load; bit 2: prefetch
  static int prefetch_on = -1;             // JANUS_DIFF_PREFETCH=0: no prefetch of the rows a warp reads next (experiments)
  if (prefetch_on < 0) {
    const char* env = getenv("JANUS_DIFF_PREFETCH");
    prefetch_on = (env && env[0] == '0') ? 0 : 1;
  }
  static int vvec_on = -1;                 // JANUS_DIFF_VVEC=0: value columns by single loads (experiments)
  if (vvec_on < 0) {
    const char* env = getenv("JANUS_DIFF_VVEC");
    vvec_on = (env && env[0] == '0') ? 0 : 1;
  }
  const int vec = ((d % (f32c ? 4 : 8) == 0 && (((uintptr_t)k_cache) & 15) == 0) ? 1 : 0) |
                  ((vvec_on && (((uintptr_t)v_cache) & 15) == 0) ? 2 : 0) | (prefetch_on ? 4 : 0);
  jb::Launch cfg(dim3((unsigned)(T * H)), dim3(warps * 32), smem, stream);
  cudaError_t err;
#define JB_LAUNCH_DA(TC, TO, EJ)                                                                                     \
  err = cudaLaunchKernelEx(&cfg.c, diff_attention_kernel<TC, TO, EJ>, q, (const TC*)k_cache, (const TC*)v_cache,     \
                           (TO*)out, block_table, token_seq, positions, T, H, G, d, e, page_size, max_pages, window, \
                           keep_first, scale, lambda, eps, out_scale, vec)
#define JB_LAUNCH_DA_E(TC, TO)            \
  do {                                    \
    if (e <= 64) JB_LAUNCH_DA(TC, TO, 2); \
    else if (e <= 128) JB_LAUNCH_DA(TC, TO, 4); \
    else JB_LAUNCH_DA(TC, TO, 8);         \
  } while (0)
  if (cache_dtype == JB_F32 && out_dtype == JB_F32) JB_LAUNCH_DA_E(float, float);
  else if (cache_dtype == JB_BF16 && out_dtype == JB_BF16) JB_LAUNCH_DA_E(bf16, bf16);
  else return JB_ERR_BAD_DTYPE;
#undef JB_LAUNCH_DA_E
#undef JB_LAUNCH_DA
  return (int)err;
}
