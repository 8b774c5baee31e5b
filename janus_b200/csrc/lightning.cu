// Linear attention with a per-head decay ("lightning attention") as a recurrence over the
// tokens of each sequence, and the gated norm behind it.
//
//   per head:  S_t = lambda S_(t-1) + k_t v_t^T   (S: [d, e] float32, kept per sequence)
//              o_t = S_t^T q_t
//   with q = silu(.), k = silu(.), v = silu(.) of the projection's float32 output.
//
// lightning_scan: a block owns one (sequence, head, block of EB value columns); a thread owns
// two value columns and a quarter of the rows of S in registers, walks the tokens in order
// (chunks of CT tokens are staged in shared memory, activated on the way), and the four
// partial sums of o meet by shuffles in a fixed order.  The state is read from and written back
// to the sequence's slot, so prompts, portions of prompts and single tokens are the same code.
//
// Long prompts run in segments of `seg_len` tokens so that the segments of one sequence run side
// by side: (1) every segment but a sequence's last computes the state it would reach from zero,
// (2) a prefix pass turns these into every segment's starting state,
//     start_(s+1) = lambda^seg_len start_s + local_s, in float32, one thread per element,
// (3) every segment walks its tokens again from its starting state and writes the outputs; the
//     last one leaves the sequence's state.  The recurrence itself is the same code in all cases.
//
// gated_rmsnorm: out = o / sqrt(mean(o^2) + eps) * w * sigmoid(g), one block per token, over
// the concatenated heads.
#include <stdio.h>

#include "common.cuh"

namespace {

typedef __nv_bfloat16 bf16;

constexpr int PARTS = 4;      // threads that share a value column (each a quarter of the rows)
constexpr int EB = 64;        // value columns a block owns, two a thread
constexpr int CT = 16;        // tokens staged at a time
constexpr int THREADS = EB / 2 * PARTS;

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

enum { WHOLE = 0, LOCAL = 1, FROM_START = 3 };

// RMAX: rows of S a thread holds (a multiple of 4, 4 RMAX >= d); shared rows are padded to 4 RMAX with zeros
template <int RMAX, int PHASE>
__global__ void __launch_bounds__(EB / 2 * PARTS, RMAX <= 32 ? 4 : 2) lightning_scan_kernel(
    const float* __restrict__ proj, int ld, int q_col, int k_col, int v_col, float* __restrict__ out,
    float* __restrict__ state, const int* __restrict__ q_start, const int* __restrict__ seq_slot,
    const float* __restrict__ decay, int H, int d, int e, int seg_len, int tiles_per_seq, float* __restrict__ scratch) {
  constexpr int phase = PHASE;             // the pass from zero needs neither queries nor outputs
  constexpr int DP = PARTS * RMAX;         // padded rows
  // a part's rows start four floats after the part before ends: the four parts of a column read their 16 bytes
  // from different banks (with the parts RMAX floats apart, a multiple of 16, they would meet in one or two)
  constexpr int PS = RMAX + 4;             // floats from part to part
  constexpr int TS = PARTS * PS;           // floats from token to token
  extern __shared__ __align__(16) float smem[];          // q [CT][TS], k [CT][TS], v [CT][EB]
  float* q_s = smem;
  float* k_s = q_s + CT * TS;
  float* v_s = k_s + CT * TS;
  jb::pdl_launch_dependents();
  const int seq = blockIdx.x / tiles_per_seq, seg = blockIdx.x % tiles_per_seq;
  const int h = blockIdx.y, e0 = blockIdx.z * EB;
  const int part = threadIdx.x % PARTS, col = threadIdx.x / PARTS;
  const int j0 = e0 + 2 * col, j1 = j0 + 1;
  const float lam = decay[h];
  jb::pdl_wait();
  const int s0 = q_start[seq], q_len = q_start[seq + 1] - s0;
  if ((long long)seg * seg_len >= q_len) return;
  const int t0 = s0 + seg * seg_len, t1 = min(s0 + q_len, t0 + seg_len);
  const bool last = t1 == s0 + q_len;
  if (phase == LOCAL && last) return;              // nobody needs the last segment's state from zero
  float* st = state + (((size_t)seq_slot[seq] * H + h) * d) * e;     // [d][e]
  float* sc = scratch ? scratch + (((size_t)blockIdx.x * H + h) * d) * e : nullptr;
  const float* init = phase == WHOLE ? st : phase == FROM_START ? sc : nullptr;
  float S0[RMAX], S1[RMAX];
#pragma unroll
  for (int i = 0; i < RMAX; ++i) {
    const int r = part * RMAX + i;
    S0[i] = (init && r < d && j0 < e) ? init[(size_t)r * e + j0] : 0.0f;
    S1[i] = (init && r < d && j1 < e) ? init[(size_t)r * e + j1] : 0.0f;
  }
  for (int c0 = t0; c0 < t1; c0 += CT) {
    const int n = min(CT, t1 - c0);
    __syncthreads();
    // eight loads of each kind are in flight before their activations run (a load a time would leave the
    // block waiting on memory for most of a chunk)
    for (int base = 0; base < n * DP; base += 8 * THREADS) {
      float qv[8], kv[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int idx = base + u * THREADS + threadIdx.x;
        const int tt = idx / DP, r = idx % DP;
        const bool in = idx < n * DP && r < d;
        const float* row = proj + (size_t)(c0 + (in ? tt : 0)) * ld + h * d + (in ? r : 0);
        qv[u] = (in && phase != LOCAL) ? row[q_col] : 0.0f;
        kv[u] = in ? row[k_col] : 0.0f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int idx = base + u * THREADS + threadIdx.x;
        if (idx < n * DP) {
          const int r = idx % DP;
          const bool in = r < d;
          const int at = (idx / DP) * TS + (r / RMAX) * PS + r % RMAX;
          if (phase != LOCAL) q_s[at] = in ? silu_f(qv[u]) : 0.0f;
          k_s[at] = in ? silu_f(kv[u]) : 0.0f;
        }
      }
    }
    {
      float vv[CT * EB / THREADS];
#pragma unroll
      for (int u = 0; u < CT * EB / THREADS; ++u) {
        const int idx = u * THREADS + threadIdx.x;
        const int tt = idx / EB, c = idx % EB;
        const bool in = tt < n && e0 + c < e;
        vv[u] = in ? proj[(size_t)(c0 + tt) * ld + v_col + h * e + e0 + c] : 0.0f;
      }
#pragma unroll
      for (int u = 0; u < CT * EB / THREADS; ++u) {
        const int idx = u * THREADS + threadIdx.x;
        const int tt = idx / EB, c = idx % EB;
        v_s[idx] = (tt < n && e0 + c < e) ? silu_f(vv[u]) : 0.0f;
      }
    }
    __syncthreads();
    for (int tt = 0; tt < n; ++tt) {
      const float2 v = *reinterpret_cast<const float2*>(v_s + tt * EB + 2 * col);
      const float4* qr = reinterpret_cast<const float4*>(q_s + tt * TS + part * PS);
      const float4* kr = reinterpret_cast<const float4*>(k_s + tt * TS + part * PS);
      float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f, b0 = 0.0f, b1 = 0.0f, b2 = 0.0f, b3 = 0.0f;
#pragma unroll
      for (int i = 0; i < RMAX / 4; ++i) {
        const float4 k4 = kr[i];
        S0[4 * i] = fmaf(lam, S0[4 * i], k4.x * v.x);
        S0[4 * i + 1] = fmaf(lam, S0[4 * i + 1], k4.y * v.x);
        S0[4 * i + 2] = fmaf(lam, S0[4 * i + 2], k4.z * v.x);
        S0[4 * i + 3] = fmaf(lam, S0[4 * i + 3], k4.w * v.x);
        S1[4 * i] = fmaf(lam, S1[4 * i], k4.x * v.y);
        S1[4 * i + 1] = fmaf(lam, S1[4 * i + 1], k4.y * v.y);
        S1[4 * i + 2] = fmaf(lam, S1[4 * i + 2], k4.z * v.y);
        S1[4 * i + 3] = fmaf(lam, S1[4 * i + 3], k4.w * v.y);
        if (phase != LOCAL) {
          const float4 q4 = qr[i];
          a0 = fmaf(S0[4 * i], q4.x, a0);
          a1 = fmaf(S0[4 * i + 1], q4.y, a1);
          a2 = fmaf(S0[4 * i + 2], q4.z, a2);
          a3 = fmaf(S0[4 * i + 3], q4.w, a3);
          b0 = fmaf(S1[4 * i], q4.x, b0);
          b1 = fmaf(S1[4 * i + 1], q4.y, b1);
          b2 = fmaf(S1[4 * i + 2], q4.z, b2);
          b3 = fmaf(S1[4 * i + 3], q4.w, b3);
        }
      }
      if (phase != LOCAL) {
        float acc0 = (a0 + a1) + (a2 + a3), acc1 = (b0 + b1) + (b2 + b3);
        // the four parts of a column are neighbouring lanes: part 0 + 1, 2 + 3, then the two sums
        acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
        acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
        acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
        acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
        if (part == 0) {
          float* orow = out + (size_t)(c0 + tt) * H * e + (size_t)h * e;
          if (j0 < e) orow[j0] = acc0;
          if (j1 < e) orow[j1] = acc1;
        }
      }
    }
  }
  float* dst = phase == LOCAL ? sc : (last ? st : nullptr);
  if (dst == nullptr) return;
#pragma unroll
  for (int i = 0; i < RMAX; ++i) {
    const int r = part * RMAX + i;
    if (r < d && j0 < e) dst[(size_t)r * e + j0] = S0[i];
    if (r < d && j1 < e) dst[(size_t)r * e + j1] = S1[i];
  }
}

// scratch[seq][seg] holds segment seg's state from zero; afterwards it holds the state the segment starts from
__global__ void lightning_prefix_kernel(float* __restrict__ scratch, const float* __restrict__ state,
                                        const int* __restrict__ q_start, const int* __restrict__ seq_slot,
                                        const float* __restrict__ decay, int H, int d, int e, int seg_len,
                                        int tiles_per_seq) {
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int seq = blockIdx.x;
  const size_t per = (size_t)H * d * e;
  const size_t idx = (size_t)blockIdx.y * blockDim.x + threadIdx.x;
  if (idx >= per) return;
  const int h = (int)(idx / ((size_t)d * e));
  const int q_len = q_start[seq + 1] - q_start[seq];
  const int n_seg = (q_len + seg_len - 1) / seg_len;
  const float lam = decay[h];
  float lam_seg = 1.0f;
  for (int i = 0; i < seg_len; ++i) lam_seg *= lam;          // the decay of a whole segment, as the walk applies it
  float S = state[(size_t)seq_slot[seq] * per + idx];
  float* p = scratch + (size_t)seq * tiles_per_seq * per + idx;
  // four segments' states from zero are on their way before the first is used
  for (int seg0 = 0; seg0 < n_seg; seg0 += 4) {
    float local[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) local[u] = seg0 + u + 1 < n_seg ? p[(size_t)(seg0 + u) * per] : 0.0f;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (seg0 + u < n_seg) {
        p[(size_t)(seg0 + u) * per] = S;
        S = fmaf(lam_seg, S, local[u]);
      }
    }
  }
}

template <typename TG, typename TO>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ o, const TG* __restrict__ w, const float* __restrict__ gate,
                                     int gate_ld, float eps, TO* __restrict__ out, int N) {
  __shared__ float scratch[33];
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int t = blockIdx.x;
  const float* row = o + (size_t)t * N;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < N; i += blockDim.x) ss += row[i] * row[i];
  ss = jb::block_sum(ss, scratch);
  const float rms = sqrtf(ss / (float)N + eps);
  const float* g = gate + (size_t)t * gate_ld;
  for (int i = threadIdx.x; i < N; i += blockDim.x) {
    const float s = 1.0f / (1.0f + expf(-g[i]));
    out[(size_t)t * N + i] = jb::from_f32<TO>((row[i] / rms) * jb::to_f32(w[i]) * s);
  }
}

}  // namespace

// proj: float32 [T, ld], the raw projections: q at column q_col ([H][d]), k at k_col ([H][d]), v at v_col ([H][e]);
// out: float32 [T, H * e]; state: float32 [slots, H, d, e]; q_start: [n_seqs + 1] rows of each sequence's tokens;
// seq_slot: [n_seqs]; decay: [H] float32.  seg_len > 0 with scratch (float32, n_seqs * ceil(max_q_len / seg_len) *
// H * d * e) runs the three passes over segments; seg_len = 0 walks every sequence in one block per column block.
JB_EXPORT int jb_lightning_scan(const float* proj, int ld, int q_col, int k_col, int v_col, float* out, float* state,
                                const int* q_start, const int* seq_slot, const float* decay, int n_seqs, int H, int d,
                                int e, int max_q_len, int seg_len, float* scratch, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  JB_REFUSE(d < 1 || d > 256 || e < 1, "lightning_scan: key size %d is outside [1, 256]", d);
  JB_REFUSE(seg_len > 0 && scratch == nullptr, "lightning_scan: segments need scratch");
  const int rmax = d <= 64 ? 16 : d <= 128 ? 32 : 64;
  const size_t smem = (size_t)(2 * CT * PARTS * (rmax + 4) + CT * EB) * sizeof(float);
  const bool segmented = seg_len > 0;
  const int tiles = segmented ? (max_q_len + seg_len - 1) / seg_len : 1;
  const int seg = segmented ? seg_len : 0x40000000;
#define JB_LAUNCH_LS(RM, PHASE)                                                                                      \
  do {                                                                                                               \
    jb::Launch cfg(dim3(n_seqs * tiles, H, (e + EB - 1) / EB), dim3(EB / 2 * PARTS), smem, stream);                     \
    cudaError_t err = cudaLaunchKernelEx(&cfg.c, lightning_scan_kernel<RM, PHASE>, proj, ld, q_col, k_col, v_col,   \
                                         out, state, q_start, seq_slot, decay, H, d, e, seg, tiles, scratch);        \
    if (err != cudaSuccess) return (int)err;                                                                         \
  } while (0)
#define JB_LAUNCH_LS_R(PHASE)                       \
  do {                                              \
    if (rmax == 16) JB_LAUNCH_LS(16, PHASE);        \
    else if (rmax == 32) JB_LAUNCH_LS(32, PHASE);   \
    else JB_LAUNCH_LS(64, PHASE);                   \
  } while (0)
  if (!segmented) {
    JB_LAUNCH_LS_R(WHOLE);
    return 0;
  }
  JB_LAUNCH_LS_R(LOCAL);
  {
    const size_t per = (size_t)H * d * e;
    jb::Launch cfg(dim3(n_seqs, (unsigned)((per + 255) / 256)), dim3(256), 0, stream);
    cudaError_t err = cudaLaunchKernelEx(&cfg.c, lightning_prefix_kernel, scratch, (const float*)state, q_start, seq_slot,
                                         decay, H, d, e, seg_len, tiles);
    if (err != cudaSuccess) return (int)err;
  }
  JB_LAUNCH_LS_R(FROM_START);
#undef JB_LAUNCH_LS_R
#undef JB_LAUNCH_LS
  return 0;
}

// out[t] = o[t] / sqrt(mean(o[t]^2) + eps) * w * sigmoid(gate[t]); o: float32 [T, N]; gate: float32 rows of gate_ld.
JB_EXPORT int jb_gated_rmsnorm(const float* o, const void* w, int w_dtype, const float* gate, int gate_ld, float eps,
                               void* out, int out_dtype, int T, int N, cudaStream_t stream) {
  if (T <= 0) return 0;
  jb::Launch cfg(dim3(T), dim3(N >= 2048 ? 256 : 128), 0, stream);
  cudaError_t e;
#define JB_LAUNCH_GN(TG, TO) \
  e = cudaLaunchKernelEx(&cfg.c, gated_rmsnorm_kernel<TG, TO>, o, (const TG*)w, gate, gate_ld, eps, (TO*)out, N)
  if (w_dtype == JB_F32 && out_dtype == JB_F32) JB_LAUNCH_GN(float, float);
  else if (w_dtype == JB_F32 && out_dtype == JB_BF16) JB_LAUNCH_GN(float, bf16);
  else if (w_dtype == JB_BF16 && out_dtype == JB_F32) JB_LAUNCH_GN(bf16, float);
  else if (w_dtype == JB_BF16 && out_dtype == JB_BF16) JB_LAUNCH_GN(bf16, bf16);
  else return JB_ERR_BAD_DTYPE;
#undef JB_LAUNCH_GN
  return (int)e;
}
