// Differential attention of prompt steps in bfloat16 on the tensor cores (mma.sync m16n8k16, float32
// accumulation), one build per (key size JB_DIFF_D, value size JB_DIFF_E), both multiples of 16 up to 128.
//
// A CTA of eight warps (four row groups x the two maps) owns 64 rows = floor(64 / R) neighbouring tokens of one sequence x the R query heads of one
// key/value head, so a page of keys and values is read once for the whole group.  It walks the pages its rows can
// see: the pages of the kept first keys that the window has left behind, then the pages from the window's start
// of its first token to its last token.  Per page and per map: S = Q K^T (the map's own keys), scale, mask
// (j <= i and (i - j < window or j < keep_first)), online softmax in float32 with exp2, P rounded to bfloat16 as
// the A operand of O += P V; both maps use the same value tile.  Pages come by cp.async into a ring of two stages.
// Warp w and warp w + 4 own the same 16 rows, one map each; at the end the second map's warps hand O2 / l2 over
// through shared memory and the first map's warps form o = O1 / l1 - lambda O2 / l2, divided by its root mean square over the head's values (eps inside the
// root), times out_scale.
//
// A page whose keys a row cannot see leaves that row's maximum, sum and values untouched (its weights are exact
// zeros), so a token's result does not depend on which other tokens share its tile or its step.
#include <math_constants.h>
#include <stdio.h>

#include "common.cuh"

#ifndef JB_DIFF_D
#define JB_DIFF_D 64
#endif
#ifndef JB_DIFF_E
#define JB_DIFF_E 128
#endif

namespace {

typedef __nv_bfloat16 bf16;
constexpr int D = JB_DIFF_D, E = JB_DIFF_E;
constexpr int PAGE = 64;                 // keys per page and per step of the walk
constexpr int ROWS = 64;                 // rows of a CTA's tile (four warps of 16)
constexpr int QLD = 2 * D + 8;           // row strides in shared memory, padded by 16 bytes against bank conflicts
constexpr int KLD = D + 8;
constexpr int VLD = E + 8;
constexpr int STAGES = 2;
constexpr int THREADS = 256;             // eight warps: four row groups x two maps
#ifndef JB_DIFF_CTAS
#define JB_DIFF_CTAS 2
#endif
constexpr int CTAS_PER_SM = JB_DIFF_CTAS;
constexpr size_t SMEM_BYTES = ((size_t)ROWS * QLD + (size_t)STAGES * 2 * PAGE * KLD + (size_t)STAGES * PAGE * VLD) * sizeof(bf16);

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                         unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// 2^x on the special-function unit (2^-inf = 0); two units in the last place are far below bfloat16's rounding of P
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

__global__ void __launch_bounds__(THREADS, CTAS_PER_SM) diff_prefill_kernel(
    const float* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache, bf16* __restrict__ out,
    const int* __restrict__ block_table, const int* __restrict__ q_start, const int* __restrict__ kv_len, int tiles_per_seq,
    int H, int G, int max_pages, int window, int keep_first, float scale_log2, float lambda, float eps, float out_scale) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);
  bf16* Ks = Qs + ROWS * QLD;                       // [stage][map][PAGE][KLD]
  bf16* Vs = Ks + STAGES * 2 * PAGE * KLD;          // [stage][PAGE][VLD]
  jb::pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = blockIdx.x / tiles_per_seq, tile = blockIdx.x % tiles_per_seq, g = blockIdx.y;
  const int R = H / G, tpt = ROWS / R;              // tokens of a tile
  jb::pdl_wait();
  const int t_first = q_start[seq], q_len = q_start[seq + 1] - t_first;
  const int tok0 = tile * tpt;
  if (tok0 >= q_len) return;
  const int base_pos = kv_len[seq] - q_len;          // position of the step's first token of this sequence
  const int n_tok = min(tpt, q_len - tok0);
  const int p_lo = base_pos + tok0, p_hi = p_lo + n_tok - 1;
  const int* pages = block_table + (size_t)seq * max_pages;

  // queries: float32 -> bfloat16 rows [map 1 | map 2]; rows without a token are zeros
  for (int idx = threadIdx.x; idx < ROWS * (2 * D / 4); idx += blockDim.x) {
    const int r = idx / (2 * D / 4), c4 = (idx % (2 * D / 4)) * 4;
    const int tok = r / R, hh = r % R;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (tok < n_tok) v = *reinterpret_cast<const float4*>(q + ((size_t)(t_first + tok0 + tok) * H + g * R + hh) * 2 * D + c4);
    uint2 packed;
    packed.x = pack_bf16(v.x, v.y);
    packed.y = pack_bf16(v.z, v.w);
    *reinterpret_cast<uint2*>(Qs + r * QLD + c4) = packed;
  }

  // the pages to walk: kept first keys behind the window, then the window's pages
  const int first_key = window > 0 ? max(0, p_lo - window + 1) : 0;
  const int blk_lo = first_key / PAGE, blk_hi = p_hi / PAGE;
  const int n_sink = (window > 0 && keep_first > 0) ? min((keep_first + PAGE - 1) / PAGE, blk_lo) : 0;
  const int n_blocks = n_sink + blk_hi - blk_lo + 1;

  auto load_block = [&](int it, int stage) {
    const int b = it < n_sink ? it : blk_lo + it - n_sink;
    const int page = pages[b];
    const bf16* kp = k_cache + ((size_t)page * 2 * G + 2 * g) * PAGE * D;      // two maps, one after the other
    bf16* ks = Ks + (size_t)stage * 2 * PAGE * KLD;
    for (int idx = threadIdx.x; idx < 2 * PAGE * (D / 8); idx += blockDim.x) {
      const int row = idx / (D / 8), c = (idx % (D / 8)) * 8;
      cp_async16(ks + row * KLD + c, kp + (size_t)row * D + c);
    }
    const bf16* vp = v_cache + ((size_t)page * G + g) * PAGE * E;
    bf16* vs = Vs + (size_t)stage * PAGE * VLD;
    for (int idx = threadIdx.x; idx < PAGE * (E / 8); idx += blockDim.x) {
      const int row = idx / (E / 8), c = (idx % (E / 8)) * 8;
      cp_async16(vs + row * VLD + c, vp + (size_t)row * E + c);
    }
  };

  load_block(0, 0);
  cp_async_commit();

  // Eight warps: warp w and warp w + 4 own the same 16 rows, the first for map 1 and the second for map 2, so
  // that a thread holds one map's O (a CTA's registers then leave room for the other map's warps to run beside it
  // and the two maps' softmax and MMAs overlap).  This thread's two rows (lane / 4 and + 8 of the 16) and their
  // positions (-1: no token):
  const int rw = warp & 3, mp = warp >> 2;
  const int r0 = rw * 16 + (lane >> 2), r1 = r0 + 8;
  const int pos0 = (r0 / R) < n_tok ? p_lo + r0 / R : -1;
  const int pos1 = (r1 / R) < n_tok ? p_lo + r1 / R : -1;

  float O[E / 8][4];
  float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.0f, l1 = 0.0f;
#pragma unroll
  for (int nt = 0; nt < E / 8; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) O[nt][i] = 0.0f;

  for (int it = 0; it < n_blocks; ++it) {
    const int stage = it & 1;
    if (it + 1 < n_blocks) load_block(it + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const int b = it < n_sink ? it : blk_lo + it - n_sink;
    const int key0 = b * PAGE;
    const bf16* vs = Vs + (size_t)stage * PAGE * VLD;
    const bf16* ks = Ks + ((size_t)stage * 2 + mp) * PAGE * KLD;
    // a page that every row of the warp sees whole needs no mask
    const int w_lo = p_lo + (rw * 16) / R, w_hi = p_lo + min((rw * 16 + 15) / R, n_tok - 1);
    const bool whole = (rw * 16 + 15) / R < n_tok && key0 + PAGE - 1 <= w_lo && (window <= 0 || w_hi - key0 < window);
    float S[PAGE / 8][4];
#pragma unroll
    for (int nt = 0; nt < PAGE / 8; ++nt) S[nt][0] = S[nt][1] = S[nt][2] = S[nt][3] = 0.0f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      unsigned a0, a1, a2, a3;
      ldmatrix_x4(a0, a1, a2, a3, Qs + (rw * 16 + (lane & 15)) * QLD + mp * D + kk * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int np = 0; np < PAGE / 16; ++np) {
        unsigned b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, ks + (np * 16 + (lane >> 4) * 8 + (lane & 7)) * KLD + kk * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(S[2 * np], a0, a1, a2, a3, b0, b1);
        mma_bf16(S[2 * np + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    // scale, mask, this page's row maxima
    float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F;
#pragma unroll
    for (int nt = 0; nt < PAGE / 8; ++nt) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int key = key0 + nt * 8 + (lane & 3) * 2 + (i & 1);
        const int pos = i < 2 ? pos0 : pos1;
        const bool seen = whole || (key <= pos && (window <= 0 || pos - key < window || key < keep_first));
        S[nt][i] = seen ? S[nt][i] * scale_log2 : -CUDART_INF_F;
      }
      mx0 = fmaxf(mx0, fmaxf(S[nt][0], S[nt][1]));
      mx1 = fmaxf(mx1, fmaxf(S[nt][2], S[nt][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
    const float u0 = n0 == -CUDART_INF_F ? 0.0f : n0, u1 = n1 == -CUDART_INF_F ? 0.0f : n1;
    const float al0 = fast_exp2(m0 - u0), al1 = fast_exp2(m1 - u1);     // 2^-inf = 0 before the first key
    m0 = n0;
    m1 = n1;
    float s0 = 0.0f, s1 = 0.0f;
    unsigned P[PAGE / 8][2];
#pragma unroll
    for (int nt = 0; nt < PAGE / 8; ++nt) {
      const float p0 = fast_exp2(S[nt][0] - u0), p1 = fast_exp2(S[nt][1] - u0);
      const float p2 = fast_exp2(S[nt][2] - u1), p3 = fast_exp2(S[nt][3] - u1);
      s0 += p0 + p1;
      s1 += p2 + p3;
      P[nt][0] = pack_bf16(p0, p1);
      P[nt][1] = pack_bf16(p2, p3);
    }
    l0 = l0 * al0 + s0;
    l1 = l1 * al1 + s1;
#pragma unroll
    for (int nt = 0; nt < E / 8; ++nt) {
      O[nt][0] *= al0;
      O[nt][1] *= al0;
      O[nt][2] *= al1;
      O[nt][3] *= al1;
    }
#pragma unroll
    for (int kk = 0; kk < PAGE / 16; ++kk) {
#pragma unroll
      for (int np = 0; np < E / 16; ++np) {
        unsigned b0, b1, b2, b3;
        ldmatrix_x4_trans(b0, b1, b2, b3, vs + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * VLD + np * 16 + (lane >> 4) * 8);
        mma_bf16(O[2 * np], P[2 * kk][0], P[2 * kk][1], P[2 * kk + 1][0], P[2 * kk + 1][1], b0, b1);
        mma_bf16(O[2 * np + 1], P[2 * kk][0], P[2 * kk][1], P[2 * kk + 1][0], P[2 * kk + 1][1], b2, b3);
      }
    }
    __syncthreads();       // the stage is free for the load after next
  }
  cp_async_wait<0>();

  // the rows' sums over their four lanes; map 2's warps leave a2 = O2 / l2 in shared memory (the key and value
  // stages are free now), map 1's warps take the difference and the head's unit norm
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  float* A2 = reinterpret_cast<float*>(Ks);         // [ROWS][E + 2] floats
  constexpr int ALD = E + 2;
  if (mp == 1) {
#pragma unroll
    for (int nt = 0; nt < E / 8; ++nt) {
      const int c = nt * 8 + (lane & 3) * 2;
      *reinterpret_cast<float2*>(A2 + r0 * ALD + c) = make_float2(O[nt][0] / l0, O[nt][1] / l0);
      *reinterpret_cast<float2*>(A2 + r1 * ALD + c) = make_float2(O[nt][2] / l1, O[nt][3] / l1);
    }
  }
  __syncthreads();
  if (mp == 1) return;
  float ss0 = 0.0f, ss1 = 0.0f;
#pragma unroll
  for (int nt = 0; nt < E / 8; ++nt) {
    const int c = nt * 8 + (lane & 3) * 2;
    const float2 x0 = *reinterpret_cast<const float2*>(A2 + r0 * ALD + c), x1 = *reinterpret_cast<const float2*>(A2 + r1 * ALD + c);
    O[nt][0] = O[nt][0] / l0 - lambda * x0.x;
    O[nt][1] = O[nt][1] / l0 - lambda * x0.y;
    O[nt][2] = O[nt][2] / l1 - lambda * x1.x;
    O[nt][3] = O[nt][3] / l1 - lambda * x1.y;
    ss0 += O[nt][0] * O[nt][0] + O[nt][1] * O[nt][1];
    ss1 += O[nt][2] * O[nt][2] + O[nt][3] * O[nt][3];
  }
  ss0 += __shfl_xor_sync(0xffffffffu, ss0, 1);
  ss0 += __shfl_xor_sync(0xffffffffu, ss0, 2);
  ss1 += __shfl_xor_sync(0xffffffffu, ss1, 1);
  ss1 += __shfl_xor_sync(0xffffffffu, ss1, 2);
  const float f0 = out_scale / sqrtf(ss0 / (float)E + eps), f1 = out_scale / sqrtf(ss1 / (float)E + eps);
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    const int r = hf ? r1 : r0;
    if ((hf ? pos1 : pos0) < 0) continue;
    const int tok = r / R, hh = r % R;
    bf16* orow = out + ((size_t)(t_first + tok0 + tok) * H + g * R + hh) * E;
    const float f = hf ? f1 : f0;
#pragma unroll
    for (int nt = 0; nt < E / 8; ++nt) {
      const unsigned packed = pack_bf16(O[nt][2 * hf] * f, O[nt][2 * hf + 1] * f);
      *reinterpret_cast<unsigned*>(orow + nt * 8 + (lane & 3) * 2) = packed;
    }
  }
}

}  // namespace

// q: float32 [T, H 2 D]; caches bfloat16 [pages, 2 G, 64, D] and [pages, G, 64, E]; out: bfloat16 [T, H E];
// q_start: [n_seqs + 1] rows of each sequence's tokens; kv_len: [n_seqs] keys of each sequence after the step.
JB_EXPORT int jb_diff_attention_prefill(const float* q, const void* k_cache, const void* v_cache, void* out,
                                        const int* block_table, const int* q_start, const int* kv_len, int n_seqs,
                                        int max_q_len, int H, int G, int d, int e, int page_size, int max_pages, int window,
                                        int keep_first, float scale, float lambda, float eps, float out_scale,
                                        cudaStream_t stream) {
  if (n_seqs <= 0 || max_q_len <= 0) return 0;
  JB_REFUSE(d != D || e != E, "diff_attention_prefill: built for sizes %d and %d, called with %d and %d", D, E, d, e);
  JB_REFUSE(page_size != PAGE, "diff_attention_prefill: pages of %d keys (built for %d)", page_size, PAGE);
  JB_REFUSE(G <= 0 || H % G != 0 || H / G > ROWS, "diff_attention_prefill: %d heads over %d key/value heads", H, G);
  static bool configured = false;
  if (!configured) {
    cudaError_t e0 = cudaFuncSetAttribute(diff_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (e0 != cudaSuccess) return (int)e0;
    configured = true;
  }
  const int tpt = ROWS / (H / G);
  const int tiles_per_seq = (max_q_len + tpt - 1) / tpt;
  jb::Launch cfg(dim3((unsigned)(n_seqs * tiles_per_seq), (unsigned)G), dim3(THREADS), SMEM_BYTES, stream);
  return (int)cudaLaunchKernelEx(&cfg.c, diff_prefill_kernel, q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out,
                                 block_table, q_start, kv_len, tiles_per_seq, H, G, max_pages, window, keep_first,
                                 scale * 1.4426950408889634f, lambda, eps, out_scale);
}
