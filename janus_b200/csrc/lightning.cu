// Linear attention with a per-head decay ("lightning attention") as a recurrence over the
// tokens of each sequence, and the gated norm behind it.
//
//   per head:  S_t = lambda S_(t-1) + k_t v_t^T   (S: [d, e] float32, kept per sequence)
//              o_t = S_t^T q_t
//   with q = silu(.), k = silu(.), v = silu(.) of the projection's float32 output.
//
// lightning_scan: a block owns one (sequence, head, block of EB value columns); a thread owns
// one value column and every PARTS-th row of S in registers, walks the sequence's new tokens in
// order (chunks of CT tokens are staged in shared memory, activated on the way), and the PARTS
// partial sums of o meet by shuffles in a fixed order.  The state is read from and written back
// to the sequence's slot, so prompts, portions of prompts and single tokens are the same code
// and give the same bits.
//
// gated_rmsnorm: out = o / sqrt(mean(o^2) + eps) * w * sigmoid(g), one block per token, over
// the concatenated heads.
#include <stdio.h>

#include "common.cuh"

namespace {

typedef __nv_bfloat16 bf16;

constexpr int PARTS = 4;      // threads that share a value column (rows r = part, part + 4, ...)
constexpr int EB = 32;        // value columns a block owns
constexpr int CT = 16;        // tokens staged at a time

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

// RMAX: rows of S a thread holds at most (ceil(d / PARTS) <= RMAX)
template <int RMAX>
__global__ void __launch_bounds__(EB * PARTS) lightning_scan_kernel(
    const float* __restrict__ proj, int ld, int q_col, int k_col, int v_col, float* __restrict__ out,
    float* __restrict__ state, const int* __restrict__ q_start, const int* __restrict__ seq_slot,
    const float* __restrict__ decay, int H, int d, int e) {
  extern __shared__ float smem[];          // q [CT][d], k [CT][d], v [CT][EB]
  float* q_s = smem;
  float* k_s = q_s + CT * d;
  float* v_s = k_s + CT * d;
  jb::pdl_launch_dependents();
  const int seq = blockIdx.x, h = blockIdx.y, e0 = blockIdx.z * EB;
  const int part = threadIdx.x % PARTS, col = threadIdx.x / PARTS;
  const int j = e0 + col;
  const float lam = decay[h];
  jb::pdl_wait();
  const int t0 = q_start[seq], t1 = q_start[seq + 1];
  float* st = state + (((size_t)seq_slot[seq] * H + h) * d) * e;     // [d][e]
  float S[RMAX];
#pragma unroll
  for (int i = 0; i < RMAX; ++i) {
    const int r = part + PARTS * i;
    S[i] = (r < d && j < e) ? st[(size_t)r * e + j] : 0.0f;
  }
  for (int c0 = t0; c0 < t1; c0 += CT) {
    const int n = min(CT, t1 - c0);
    __syncthreads();
    for (int idx = threadIdx.x; idx < n * d; idx += blockDim.x) {
      const int tt = idx / d, r = idx % d;
      const float* row = proj + (size_t)(c0 + tt) * ld;
      q_s[tt * d + r] = silu_f(row[q_col + h * d + r]);
      k_s[tt * d + r] = silu_f(row[k_col + h * d + r]);
    }
    for (int idx = threadIdx.x; idx < n * EB; idx += blockDim.x) {
      const int tt = idx / EB, c = idx % EB;
      v_s[tt * EB + c] = e0 + c < e ? silu_f(proj[(size_t)(c0 + tt) * ld + v_col + h * e + e0 + c]) : 0.0f;
    }
    __syncthreads();
    for (int tt = 0; tt < n; ++tt) {
      const float v = v_s[tt * EB + col];
      const float* qr = q_s + tt * d;
      const float* kr = k_s + tt * d;
      float acc = 0.0f;
#pragma unroll
      for (int i = 0; i < RMAX; ++i) {
        const int r = part + PARTS * i;
        if (r < d) {
          S[i] = fmaf(lam, S[i], kr[r] * v);
          acc = fmaf(S[i], qr[r], acc);
        }
      }
      // the four parts of a column are neighbouring lanes: part 0 + 1, 2 + 3, then the two sums
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      if (part == 0 && j < e) out[(size_t)(c0 + tt) * H * e + (size_t)h * e + j] = acc;
    }
  }
#pragma unroll
  for (int i = 0; i < RMAX; ++i) {
    const int r = part + PARTS * i;
    if (r < d && j < e) st[(size_t)r * e + j] = S[i];
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
// seq_slot: [n_seqs]; decay: [H] float32.
JB_EXPORT int jb_lightning_scan(const float* proj, int ld, int q_col, int k_col, int v_col, float* out, float* state,
                                const int* q_start, const int* seq_slot, const float* decay, int n_seqs, int H, int d,
                                int e, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  JB_REFUSE(d < 1 || d > 256 || e < 1, "lightning_scan: key size %d is outside [1, 256]", d);
  const size_t smem = (size_t)(2 * CT * d + CT * EB) * sizeof(float);
  jb::Launch cfg(dim3(n_seqs, H, (e + EB - 1) / EB), dim3(EB * PARTS), smem, stream);
  const int rows = (d + PARTS - 1) / PARTS;
  if (rows <= 16)
    return (int)cudaLaunchKernelEx(&cfg.c, lightning_scan_kernel<16>, proj, ld, q_col, k_col, v_col, out, state, q_start,
                                   seq_slot, decay, H, d, e);
  if (rows <= 32)
    return (int)cudaLaunchKernelEx(&cfg.c, lightning_scan_kernel<32>, proj, ld, q_col, k_col, v_col, out, state, q_start,
                                   seq_slot, decay, H, d, e);
  return (int)cudaLaunchKernelEx(&cfg.c, lightning_scan_kernel<64>, proj, ld, q_col, k_col, v_col, out, state, q_start,
                                 seq_slot, decay, H, d, e);
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
