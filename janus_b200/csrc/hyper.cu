// Several residual streams per token (hyper-connections).
//
// The residual buffer of a step is float32 [T, S, H]: S copies of the stream per token.
// A sublayer reads u = sum_s a[s] x_s and, after it has produced y, every stream is
// rewritten from the old ones at once: x_t <- sum_s M[s, t] x_s + b[t] y.
//
//   streams_rmsnorm: out[r] = u / sqrt(mean(u^2) + eps) * gamma, u as above (a null: plain sum),
//                    one block per row; it can clear the row r of a float32 [rows, H] buffer
//                    besides (the target the sublayer adds its output into).
//   streams_mix:     the rewrite, in place, one thread per (token, column).
//   streams_mix_rmsnorm: a sublayer's rewrite and the next sublayer's read in one launch.
//
// All sums run over s = 0, 1, ... in that order in float32, so a token's values do not depend
// on what else is in the step.
#include <stdio.h>

#include "common.cuh"

namespace {

typedef __nv_bfloat16 bf16;
constexpr int MAX_STREAMS = 8;

// A read can also clear a scratch buffer of the sublayer that runs next (the target of a product whose slices of K
// meet by atomic adds): each block clears its share.
__device__ __forceinline__ void clear_slice(float4* __restrict__ p, size_t n4) {
  if (p == nullptr) return;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x)
    p[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
}

template <typename TG, typename TO>
__global__ void streams_rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ row_index,
                                       const float* __restrict__ a, int S, const TG* __restrict__ gamma, float eps,
                                       TO* __restrict__ out, int H, float* __restrict__ clear,
                                       float4* __restrict__ clear2, size_t clear2_n4) {
  extern __shared__ __align__(16) float u_s[];          // H floats, then 33 of scratch
  float* scratch = u_s + H;
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  clear_slice(clear2, clear2_n4);
  const int r = blockIdx.x;
  const size_t src = row_index ? (size_t)row_index[r] : (size_t)r;
  const float* xr = x + src * (size_t)S * H;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float u = 0.0f;
    for (int s = 0; s < S; ++s) {
      const float v = xr[(size_t)s * H + i];
      u = a ? fmaf(a[s], v, u) : u + v;
    }
    u_s[i] = u;
    ss += u * u;
    if (clear) clear[(size_t)r * H + i] = 0.0f;
  }
  ss = jb::block_sum(ss, scratch);
  const float rms = sqrtf(ss / (float)H + eps);
  TO* o = out + (size_t)r * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    o[i] = jb::from_f32<TO>((u_s[i] / rms) * jb::to_f32(gamma[i]));
}

// The rewrite of the streams by the sublayer that has just run (y, M, b) and the read of the next sublayer
// (a, gamma) in one launch: a block owns a token, rewrites its streams in place, sums them with the next
// sublayer's weights as it goes, clears the row of y, and norms.  The same sums in the same order as
// streams_mix followed by streams_rmsnorm.
template <typename TG, typename TO>
__global__ void streams_mix_rmsnorm_kernel(float* __restrict__ x, float* __restrict__ y, const float* __restrict__ M,
                                           const float* __restrict__ b, const float* __restrict__ a, int S,
                                           const TG* __restrict__ gamma, float eps, TO* __restrict__ out, int H,
                                           float4* __restrict__ clear2, size_t clear2_n4) {
  extern __shared__ __align__(16) float u_s[];          // H floats, then 33 of scratch, then M, b, a
  float* scratch = u_s + H;
  float* m_s = scratch + 33;
  if (threadIdx.x < S * S) m_s[threadIdx.x] = M[threadIdx.x];
  if (threadIdx.x < S) {
    m_s[MAX_STREAMS * MAX_STREAMS + threadIdx.x] = b[threadIdx.x];
    m_s[MAX_STREAMS * MAX_STREAMS + MAX_STREAMS + threadIdx.x] = a[threadIdx.x];
  }
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  clear_slice(clear2, clear2_n4);
  __syncthreads();
  const int r = blockIdx.x;
  float* xr = x + (size_t)r * S * H;
  float ss = 0.0f;
  if ((H & 3) == 0) {
    // four columns a thread: 16-byte loads and stores of the streams, the same sums per column
    float4* yr = reinterpret_cast<float4*>(y + (size_t)r * H);
    for (int i4 = threadIdx.x; i4 < (H >> 2); i4 += blockDim.x) {
      float4 old[MAX_STREAMS];
#pragma unroll
      for (int s = 0; s < MAX_STREAMS; ++s)
        old[s] = s < S ? *reinterpret_cast<const float4*>(xr + (size_t)s * H + 4 * i4) : make_float4(0.f, 0.f, 0.f, 0.f);
      const float4 yv = yr[i4];
      float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int to = 0; to < MAX_STREAMS; ++to) {
        if (to < S) {
          float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int s = 0; s < MAX_STREAMS; ++s)
            if (s < S) {
              const float m = m_s[s * S + to];
              v.x = fmaf(m, old[s].x, v.x); v.y = fmaf(m, old[s].y, v.y);
              v.z = fmaf(m, old[s].z, v.z); v.w = fmaf(m, old[s].w, v.w);
            }
          const float bo = m_s[MAX_STREAMS * MAX_STREAMS + to], an = m_s[MAX_STREAMS * MAX_STREAMS + MAX_STREAMS + to];
          v.x = fmaf(bo, yv.x, v.x); v.y = fmaf(bo, yv.y, v.y); v.z = fmaf(bo, yv.z, v.z); v.w = fmaf(bo, yv.w, v.w);
          *reinterpret_cast<float4*>(xr + (size_t)to * H + 4 * i4) = v;
          u.x = fmaf(an, v.x, u.x); u.y = fmaf(an, v.y, u.y); u.z = fmaf(an, v.z, u.z); u.w = fmaf(an, v.w, u.w);
        }
      }
      *reinterpret_cast<float4*>(u_s + 4 * i4) = u;
      ss += u.x * u.x;
      ss += u.y * u.y;
      ss += u.z * u.z;
      ss += u.w * u.w;
      yr[i4] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  } else
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float old[MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < MAX_STREAMS; ++s) old[s] = s < S ? xr[(size_t)s * H + i] : 0.0f;
    const float yv = y[(size_t)r * H + i];
    float u = 0.0f;
#pragma unroll
    for (int to = 0; to < MAX_STREAMS; ++to) {
      if (to < S) {
        float v = 0.0f;
#pragma unroll
        for (int s = 0; s < MAX_STREAMS; ++s)
          if (s < S) v = fmaf(m_s[s * S + to], old[s], v);
        v = fmaf(m_s[MAX_STREAMS * MAX_STREAMS + to], yv, v);
        xr[(size_t)to * H + i] = v;
        u = fmaf(m_s[MAX_STREAMS * MAX_STREAMS + MAX_STREAMS + to], v, u);
      }
    }
    u_s[i] = u;
    ss += u * u;
    y[(size_t)r * H + i] = 0.0f;
  }
  ss = jb::block_sum(ss, scratch);
  const float rms = sqrtf(ss / (float)H + eps);
  TO* o = out + (size_t)r * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    o[i] = jb::from_f32<TO>((u_s[i] / rms) * jb::to_f32(gamma[i]));
}

__global__ void streams_mix_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ M,
                                   const float* __restrict__ b, int S, int H, size_t n) {
  __shared__ float m_s[MAX_STREAMS * MAX_STREAMS + MAX_STREAMS];
  if (threadIdx.x < S * S) m_s[threadIdx.x] = M[threadIdx.x];
  if (threadIdx.x < S) m_s[MAX_STREAMS * MAX_STREAMS + threadIdx.x] = b[threadIdx.x];
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  __syncthreads();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n) return;
  const size_t t = idx / H;
  const int i = (int)(idx % H);
  float* xr = x + t * (size_t)S * H + i;
  float old[MAX_STREAMS];
#pragma unroll
  for (int s = 0; s < MAX_STREAMS; ++s) old[s] = s < S ? xr[(size_t)s * H] : 0.0f;
  const float yv = y[idx];
#pragma unroll
  for (int to = 0; to < MAX_STREAMS; ++to) {
    if (to < S) {
      float v = 0.0f;
#pragma unroll
      for (int s = 0; s < MAX_STREAMS; ++s)
        if (s < S) v = fmaf(m_s[s * S + to], old[s], v);
      xr[(size_t)to * H] = fmaf(m_s[MAX_STREAMS * MAX_STREAMS + to], yv, v);
    }
  }
}

}  // namespace

// x: float32 [*, S, H]; a: S float32 weights or null (plain sum); out: [rows, H] in out_dtype;
// clear: null or a float32 [rows, H] buffer whose row r is set to zero (only without row_index);
// clear2: null or clear2_n floats (whole 16-byte vectors) that the launch sets to zero besides.
JB_EXPORT int jb_streams_rmsnorm(const float* x, const int* row_index, const float* a, int S, const void* gamma,
                                 int gamma_dtype, float eps, void* out, int out_dtype, int rows, int H, float* clear,
                                 float* clear2, long long clear2_n, cudaStream_t stream) {
  if (rows <= 0) return 0;
  JB_REFUSE(clear2 != nullptr && ((clear2_n & 3) != 0 || ((uintptr_t)clear2 & 15) != 0),
            "streams_rmsnorm: the buffer to clear is not made of whole 16-byte vectors");
  float4* clear2_4 = (float4*)clear2;
  const size_t clear2_n4 = clear2 ? (size_t)clear2_n >> 2 : 0;
  JB_REFUSE(S < 1 || S > MAX_STREAMS, "streams_rmsnorm: %d streams are outside [1, %d]", S, MAX_STREAMS);
  JB_REFUSE(clear != nullptr && row_index != nullptr, "streams_rmsnorm: a buffer is cleared row by row only without a row index");
  const size_t smem = (size_t)(H + 33) * sizeof(float);
  JB_REFUSE(smem > 200 * 1024, "streams_rmsnorm: rows of %d floats do not fit shared memory", H);
  jb::Launch cfg(dim3(rows), dim3(H >= 2048 ? 256 : 128), smem, stream);
  cudaError_t e = cudaSuccess;
#define JB_LAUNCH_SN(TG, TO)                                                                                    \
  do {                                                                                                          \
    if (smem > 48 * 1024)                                                                                       \
      cudaFuncSetAttribute(streams_rmsnorm_kernel<TG, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    e = cudaLaunchKernelEx(&cfg.c, streams_rmsnorm_kernel<TG, TO>, x, row_index, a, S, (const TG*)gamma, eps,   \
                           (TO*)out, H, clear, clear2_4, clear2_n4);                                            \
  } while (0)
  if (gamma_dtype == JB_F32 && out_dtype == JB_F32) JB_LAUNCH_SN(float, float);
  else if (gamma_dtype == JB_F32 && out_dtype == JB_BF16) JB_LAUNCH_SN(float, bf16);
  else if (gamma_dtype == JB_BF16 && out_dtype == JB_F32) JB_LAUNCH_SN(bf16, float);
  else if (gamma_dtype == JB_BF16 && out_dtype == JB_BF16) JB_LAUNCH_SN(bf16, bf16);
  else return JB_ERR_BAD_DTYPE;
#undef JB_LAUNCH_SN
  return (int)e;
}

// x: float32 [T, S, H] rewritten in place; y: float32 [T, H]; M: [S, S] indexed [from, to]; b: [S].
JB_EXPORT int jb_streams_mix(float* x, const float* y, const float* M, const float* b, int T, int S, int H,
                             cudaStream_t stream) {
  if (T <= 0) return 0;
  JB_REFUSE(S < 1 || S > MAX_STREAMS, "streams_mix: %d streams are outside [1, %d]", S, MAX_STREAMS);
  const size_t n = (size_t)T * H;
  jb::Launch cfg(dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream);
  return (int)cudaLaunchKernelEx(&cfg.c, streams_mix_kernel, x, y, M, b, S, H, n);
}

// x: float32 [T, S, H] rewritten in place by (y, M, b) as in jb_streams_mix; then out[t] = rmsnorm(sum_s a[s] x[t, s]) *
// gamma and y[t] = 0, as jb_streams_rmsnorm with `clear` would do next.
JB_EXPORT int jb_streams_mix_rmsnorm(float* x, float* y, const float* M, const float* b, const float* a, int S,
                                     const void* gamma, int gamma_dtype, float eps, void* out, int out_dtype, int T, int H,
                                     float* clear2, long long clear2_n, cudaStream_t stream) {
  if (T <= 0) return 0;
  JB_REFUSE(clear2 != nullptr && ((clear2_n & 3) != 0 || ((uintptr_t)clear2 & 15) != 0),
            "streams_mix_rmsnorm: the buffer to clear is not made of whole 16-byte vectors");
  float4* clear2_4 = (float4*)clear2;
  const size_t clear2_n4 = clear2 ? (size_t)clear2_n >> 2 : 0;
  JB_REFUSE(S < 1 || S > MAX_STREAMS, "streams_mix_rmsnorm: %d streams are outside [1, %d]", S, MAX_STREAMS);
  const size_t smem = (size_t)(H + 33 + MAX_STREAMS * MAX_STREAMS + 2 * MAX_STREAMS) * sizeof(float);
  JB_REFUSE(smem > 200 * 1024, "streams_mix_rmsnorm: rows of %d floats do not fit shared memory", H);
  jb::Launch cfg(dim3(T), dim3(H >= 2048 ? 256 : 128), smem, stream);
  cudaError_t e = cudaSuccess;
#define JB_LAUNCH_SMN(TG, TO)                                                                                       \
  do {                                                                                                              \
    if (smem > 48 * 1024)                                                                                           \
      cudaFuncSetAttribute(streams_mix_rmsnorm_kernel<TG, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    e = cudaLaunchKernelEx(&cfg.c, streams_mix_rmsnorm_kernel<TG, TO>, x, y, M, b, a, S, (const TG*)gamma, eps,     \
                           (TO*)out, H, clear2_4, clear2_n4);                                                       \
  } while (0)
  if (gamma_dtype == JB_F32 && out_dtype == JB_F32) JB_LAUNCH_SMN(float, float);
  else if (gamma_dtype == JB_F32 && out_dtype == JB_BF16) JB_LAUNCH_SMN(float, bf16);
  else if (gamma_dtype == JB_BF16 && out_dtype == JB_F32) JB_LAUNCH_SMN(bf16, float);
  else if (gamma_dtype == JB_BF16 && out_dtype == JB_BF16) JB_LAUNCH_SMN(bf16, bf16);
  else return JB_ERR_BAD_DTYPE;
#undef JB_LAUNCH_SMN
  return (int)e;
}

namespace {
// out[t, s, :] = row of the table for every stream s (the streams start as copies of the embedding).
template <typename TT>
__global__ void embed_streams_kernel(const TT* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                                     int H, int S, const int* __restrict__ feedback, const int* __restrict__ token_slot) {
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0) id = feedback[token_slot[t]];
  const TT* row = table + (size_t)id * H;
  float* o = out + (size_t)t * S * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = jb::to_f32(row[i]);
    for (int s = 0; s < S; ++s) o[(size_t)s * H + i] = v;
  }
}
}  // namespace

// The embedding gather into S streams: out float32 [T, S, H]; ids < 0 read feedback[token_slot[t]].
JB_EXPORT int jb_embed_streams(const void* table, int table_dtype, const int* ids, float* out, int T, int H, int S,
                               const int* feedback, const int* token_slot, cudaStream_t stream) {
  if (T <= 0) return 0;
  JB_REFUSE(S < 1 || S > MAX_STREAMS, "embed_streams: %d streams are outside [1, %d]", S, MAX_STREAMS);
  jb::Launch cfg(dim3(T), dim3(H >= 1024 ? 256 : 128), 0, stream);
  if (table_dtype == JB_F32)
    return (int)cudaLaunchKernelEx(&cfg.c, embed_streams_kernel<float>, (const float*)table, ids, out, H, S, feedback, token_slot);
  if (table_dtype == JB_BF16)
    return (int)cudaLaunchKernelEx(&cfg.c, embed_streams_kernel<bf16>, (const bf16*)table, ids, out, H, S, feedback, token_slot);
  return JB_ERR_BAD_DTYPE;
}
