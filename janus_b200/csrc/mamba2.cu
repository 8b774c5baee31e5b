// The selective state-space mixer (Mamba-2 form: one scalar decay per head and token), as a recurrence over
// the tokens of each sequence, with the short causal convolution in front of it and the gated, grouped norm
// behind it.  Everything here is float32.
//
//   u = the projection's columns [x | B | C]            (x: [heads][P], B and C: [groups][N])
//   xbc_t = silu(bias + sum_j w[:, j] u_(t - taps + 1 + j))   (zeros before a sequence's start; the last taps - 1
//                                                              inputs of a sequence are kept as state)
//   dt_t = softplus(dt_raw_t + dt_bias_h),  a_t = exp(-exp(A_log_h) dt_t)
//   per head h (group g = h / (heads / groups)):
//       S_t = a_t S_(t-1) + dt_t B_t x_t^T               (S: [N, P] float32, kept per sequence)
//       y_t = S_t^T C_t + D_h x_t
//   out = (y * silu(z)) / rms over each of `parts` equal pieces * w
//
// mamba2_scan: a block owns one (sequence, head, block of EB value columns); a thread owns four value columns and an
// eighth of the rows of S in registers, walks the tokens in order (chunks of CT tokens are staged in shared memory,
// dt and a computed on the way; the decays are applied late, see the kernel), and the eight partial sums of y meet by
// shuffles in a fixed order.  The state is read
// from and written back to the sequence's slot, so prompts, portions of prompts and single tokens are the same code.
//
// Long prompts run in segments of `seg_len` tokens so that the segments of one sequence run side by side: (1) every
// segment but a sequence's last computes the state it would reach from zero and the product of its decays, (2) a
// prefix pass turns these into every segment's starting state, start_(s+1) = decay_s start_s + local_s, (3) every
// segment walks its tokens again from its starting state and writes the outputs; the last one leaves the
// sequence's state.
#include <stdio.h>

#include "common.cuh"

namespace {

typedef __nv_bfloat16 bf16;

constexpr int PARTS = 8;      // threads that share a value column (each an eighth of the rows)
constexpr int COLS = 4;       // value columns a thread owns (the 16-byte state accesses below are written for four)
constexpr int EB = 64;        // value columns a block owns
constexpr int CT = 16;        // tokens staged at a time
constexpr int THREADS = EB / COLS * PARTS;

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
// log(1 + exp(z)); beyond 20 the sum is z itself in float32
__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

// ---- the short convolution ------------------------------------------------------------------------------
// proj rows of ld floats, the convolved channels in columns [col0, col0 + C); w [C][taps], bias [C] (may be null);
// state: per slot `slot_stride` floats, the convolution's part at `state_off`: [taps - 1][C], the inputs just before
// the tokens of this step; out [T, C].
__global__ void causal_conv_silu_kernel(const float* __restrict__ proj, int ld, int col0, int C,
                                        const float* __restrict__ w, const float* __restrict__ bias, int taps,
                                        const float* __restrict__ state, long long slot_stride, long long state_off,
                                        const int* __restrict__ token_seq, const int* __restrict__ q_start,
                                        const int* __restrict__ seq_slot, float* __restrict__ out, int shift_here) {
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int seq = token_seq[t];
  const int s0 = q_start[seq], li = t - s0;
  float* st = const_cast<float*>(state) + (size_t)seq_slot[seq] * slot_stride + state_off;
  float acc = bias != nullptr ? bias[c] : 0.0f;
  if (shift_here) {
    // every sequence brings one token: this thread is the only one that touches its channel of the state, so it
    // also moves the state on (row s takes row s + 1, the last row takes the new input)
    const float u_new = proj[(size_t)t * ld + col0 + c];
    for (int j = 0; j < taps - 1; ++j) {
      const float u = st[(size_t)j * C + c];
      acc = fmaf(w[(size_t)c * taps + j], u, acc);
      if (j > 0) st[(size_t)(j - 1) * C + c] = u;
    }
    if (taps > 1) st[(size_t)(taps - 2) * C + c] = u_new;
    out[(size_t)t * C + c] = silu_f(fmaf(w[(size_t)c * taps + taps - 1], u_new, acc));
    return;
  }
  for (int j = 0; j < taps; ++j) {
    const int src = li - (taps - 1) + j;
    const float u = src >= 0 ? proj[(size_t)(s0 + src) * ld + col0 + c] : st[(size_t)(taps - 1 + src) * C + c];
    acc = fmaf(w[(size_t)c * taps + j], u, acc);
  }
  out[(size_t)t * C + c] = silu_f(acc);
}

// Prompt steps whose rows are whole 16-byte vectors: a thread owns four channels and walks CONV_TOKENS tokens in a
// row, keeping the last taps - 1 inputs in registers, so an input is read once instead of `taps` times; where a
// sequence begins inside the tile (or the tile begins) the window is filled anew from the tokens before or the state.
constexpr int CONV_TOKENS = 16;
constexpr int CONV_MAX_TAPS = 8;

__device__ __forceinline__ float4 silu4(float4 v) {
  return make_float4(silu_f(v.x), silu_f(v.y), silu_f(v.z), silu_f(v.w));
}

__global__ void causal_conv_silu_vec_kernel(const float* __restrict__ proj, int ld, int col0, int C,
                                            const float* __restrict__ w, const float* __restrict__ bias, int taps,
                                            const float* __restrict__ state, long long slot_stride, long long state_off,
                                            const int* __restrict__ token_seq, const int* __restrict__ q_start,
                                            const int* __restrict__ seq_slot, float* __restrict__ out, int T) {
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  if (c >= C) return;
  float wr[4][CONV_MAX_TAPS];
#pragma unroll
  for (int k = 0; k < 4; ++k)
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) wr[k][j] = j < taps ? w[(size_t)(c + k) * taps + j] : 0.0f;
  const float4 b4 = bias != nullptr ? *reinterpret_cast<const float4*>(bias + c) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  float4 win[CONV_MAX_TAPS - 1];          // win[j]: the input taps - 1 - j tokens back (slots taps - 1 and up unused)
  const int t0 = blockIdx.x * CONV_TOKENS, t1 = min(T, t0 + CONV_TOKENS);
  int seq_before = -1;
  for (int t = t0; t < t1; ++t) {
    const int seq = token_seq[t];
    if (seq != seq_before) {               // the tile's first token, or a sequence's first: fill the window
      const int s0 = q_start[seq], li = t - s0;
      const float* st = state + (size_t)seq_slot[seq] * slot_stride + state_off;
#pragma unroll
      for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) {
        if (j < taps - 1) {
          const int src = li - (taps - 1) + j;
          win[j] = src >= 0 ? *reinterpret_cast<const float4*>(proj + (size_t)(s0 + src) * ld + col0 + c)
                            : *reinterpret_cast<const float4*>(st + (size_t)(taps - 1 + src) * C + c);
        }
      }
      seq_before = seq;
    }
    const float4 u = *reinterpret_cast<const float4*>(proj + (size_t)t * ld + col0 + c);
    float4 acc = b4;
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) {
      if (j < taps - 1) {
        acc.x = fmaf(wr[0][j], win[j].x, acc.x);
        acc.y = fmaf(wr[1][j], win[j].y, acc.y);
        acc.z = fmaf(wr[2][j], win[j].z, acc.z);
        acc.w = fmaf(wr[3][j], win[j].w, acc.w);
      }
    }
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) {
      if (j == taps - 1) {
        acc.x = fmaf(wr[0][j], u.x, acc.x);
        acc.y = fmaf(wr[1][j], u.y, acc.y);
        acc.z = fmaf(wr[2][j], u.z, acc.z);
        acc.w = fmaf(wr[3][j], u.w, acc.w);
      }
    }
    *reinterpret_cast<float4*>(out + (size_t)t * C + c) = silu4(acc);
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS - 2; ++j)
      if (j < taps - 2) win[j] = win[j + 1];
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
      if (j == taps - 2) win[j] = u;
  }
}

// After a step: the state becomes the last taps - 1 inputs of each sequence (older ones move up when the step
// brought fewer tokens than that).  One thread per (sequence, channel) walks the rows in order, so a row is read
// before it is written.
__global__ void conv_state_shift_kernel(const float* __restrict__ proj, int ld, int col0, int C, int taps,
                                        float* __restrict__ state, long long slot_stride, long long state_off,
                                        const int* __restrict__ q_start, const int* __restrict__ seq_slot) {
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int seq = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int s0 = q_start[seq], n = q_start[seq + 1] - s0;
  float* st = state + (size_t)seq_slot[seq] * slot_stride + state_off;
  for (int s = 0; s < taps - 1; ++s) {
    const int src = n - (taps - 1) + s;              // index among this step's tokens
    st[(size_t)s * C + c] = src >= 0 ? proj[(size_t)(s0 + src) * ld + col0 + c] : st[(size_t)(s + n) * C + c];
  }
}

// ---- the recurrence -----------------------------------------------------------------------------------------
enum { WHOLE = 0, LOCAL = 1, FROM_START = 3 };

// RMAX: rows of S a thread holds (a multiple of 4, PARTS * RMAX >= N); shared rows are padded to PARTS * RMAX with zeros
template <int RMAX, int PHASE>
__global__ void __launch_bounds__(THREADS, RMAX <= 16 ? 4 : 2) mamba2_scan_kernel(
    const float* __restrict__ xbc, int ldx, int b_col, int c_col, const float* __restrict__ dt_raw, int ld_dt,
    const float* __restrict__ dt_bias, const float* __restrict__ A_log, const float* __restrict__ Dskip,
    float* __restrict__ out, float* __restrict__ state, long long slot_stride, long long state_off,
    const int* __restrict__ q_start, const int* __restrict__ seq_slot, int H, int G, int N, int P, int seg_len,
    int tiles_per_seq, float* __restrict__ scratch, float* __restrict__ seg_decay) {
  constexpr int phase = PHASE;
  constexpr int DP = PARTS * RMAX;         // padded rows
  // a part's rows start four floats after the part before ends: the eight parts of a column read their 16 bytes
  // from different banks (with the parts RMAX floats apart they would meet in one, two or four banks)
  constexpr int PS = RMAX + 4;             // floats from part to part
  constexpr int TS = PARTS * PS;           // floats from token to token
  extern __shared__ __align__(16) float smem[];          // B [CT][TS], C [CT][TS], x [CT][EB], then 3 CT + 1 scalars
  float* b_s = smem;
  float* c_s = b_s + CT * TS;
  float* x_s = c_s + CT * TS;
  float* w_s = x_s + CT * EB;              // dt_t / A_t
  float* A_s = w_s + CT;                   // A_t: the product of the decays since the state was last rescaled
  float* sc_s = A_s + CT;                  // >= 0: rescale the state by this before token t (its own decay included)
  float* end_s = sc_s + CT;                // the product that is left when the chunk ends
  jb::pdl_launch_dependents();
  const int seq = blockIdx.x / tiles_per_seq, seg = blockIdx.x % tiles_per_seq;
  const int h = blockIdx.y, e0 = blockIdx.z * EB;
  const int g = h / (H / G);
  const int part = threadIdx.x % PARTS, col = threadIdx.x / PARTS;
  const int j0 = e0 + COLS * col;
  const float neg_a = -expf(A_log[h]), bias = dt_bias[h], dskip = Dskip[h];
  jb::pdl_wait();
  const int s0 = q_start[seq], q_len = q_start[seq + 1] - s0;
  if ((long long)seg * seg_len >= q_len) return;
  const int t0 = s0 + seg * seg_len, t1 = min(s0 + q_len, t0 + seg_len);
  const bool last = t1 == s0 + q_len;
  if (phase == LOCAL && last) return;              // nobody needs the last segment's state from zero
  const size_t per_head = (size_t)N * P;
  float* st = state + (size_t)seq_slot[seq] * slot_stride + state_off + (size_t)h * per_head;     // [N][P]
  float* sc = scratch ? scratch + ((size_t)blockIdx.x * H + h) * per_head : nullptr;
  const float* init = phase == WHOLE ? st : phase == FROM_START ? sc : nullptr;
  float S[COLS][RMAX];
  // a thread's four columns of a row are 16 bytes of the state: one load where the rows are aligned
  const bool vec_in = init != nullptr && (P & 3) == 0 && ((uintptr_t)init & 15) == 0;
  if (vec_in) {
#pragma unroll
    for (int i = 0; i < RMAX; ++i) {
      const int r = part * RMAX + i;
      float4 v4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (r < N && j0 < P) v4 = *reinterpret_cast<const float4*>(init + (size_t)r * P + j0);
      S[0][i] = v4.x;
      S[1][i] = v4.y;
      S[2][i] = v4.z;
      S[3][i] = v4.w;
    }
  } else {
#pragma unroll
    for (int c = 0; c < COLS; ++c)
#pragma unroll
      for (int i = 0; i < RMAX; ++i) {
        const int r = part * RMAX + i;
        S[c][i] = (init && r < N && j0 + c < P) ? init[(size_t)r * P + j0 + c] : 0.0f;
      }
  }
  float decay_all = 1.0f;
  for (int c0 = t0; c0 < t1; c0 += CT) {
    const int n = min(CT, t1 - c0);
    __syncthreads();
    // eight loads of each kind are in flight before the first is stored (a load a time would leave the block
    // waiting on memory for most of a chunk)
    for (int base = 0; base < n * DP; base += 8 * THREADS) {
      float bv[8], cv[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int idx = base + u * THREADS + threadIdx.x;
        const int tt = idx / DP, r = idx % DP;
        const bool in = idx < n * DP && r < N;
        const float* row = xbc + (size_t)(c0 + (in ? tt : 0)) * ldx + (size_t)g * N + (in ? r : 0);
        bv[u] = in ? row[b_col] : 0.0f;
        cv[u] = (in && phase != LOCAL) ? row[c_col] : 0.0f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int idx = base + u * THREADS + threadIdx.x;
        if (idx < n * DP) {
          const int tt = idx / DP, r = idx % DP;
          const int at = tt * TS + (r / RMAX) * PS + r % RMAX;
          b_s[at] = bv[u];
          if (phase != LOCAL) c_s[at] = cv[u];
        }
      }
    }
    {
      float xv[CT * EB / THREADS];
#pragma unroll
      for (int u = 0; u < CT * EB / THREADS; ++u) {
        const int idx = u * THREADS + threadIdx.x;
        const int tt = idx / EB, c = idx % EB;
        xv[u] = (tt < n && e0 + c < P) ? xbc[(size_t)(c0 + tt) * ldx + (size_t)h * P + e0 + c] : 0.0f;
      }
#pragma unroll
      for (int u = 0; u < CT * EB / THREADS; ++u) x_s[u * THREADS + threadIdx.x] = xv[u];
    }
    // The decays are applied late.  With A_t the product of the decays from the last rescaling up to token t, the
    // registers hold U_t = S_t / A_t, which follows U_t = U_(t-1) + B_t (dt_t x_t / A_t)^T: one FMA an element
    // instead of a product and an FMA; y_t = A_t U_t^T C_t.  When the product would fall below 2^-40 the registers
    // are rescaled before that token (its own decay included) and the product starts again at one, so nothing
    // over- or underflows whatever the step sizes; the chunk's end rescales once more.  Warp 0 computes dt and the
    // decays, one token a lane, and every lane walks the products in the same order.
    if (threadIdx.x < 32) {
      const int lane = threadIdx.x;
      float dt = 0.0f, a = 1.0f;
      if (lane < n) {
        dt = softplus_f(dt_raw[(size_t)(c0 + lane) * ld_dt + h] + bias);
        a = expf(neg_a * dt);
      }
      float run = 1.0f, my_A = 1.0f, my_sc = -1.0f;
      for (int tt = 0; tt < n; ++tt) {
        const float at = __shfl_sync(0xffffffffu, a, tt);
        const float next = run * at;
        const bool rescale = next < 9.094947e-13f;       // 2^-40
        run = rescale ? 1.0f : next;
        if (lane == tt) {
          my_A = run;
          my_sc = rescale ? next : -1.0f;
        }
        if (phase == LOCAL) decay_all *= at;
      }
      if (lane < n) {
        w_s[lane] = dt / my_A;
        A_s[lane] = my_A;
        sc_s[lane] = my_sc;
      }
      if (lane == 0) end_s[0] = run;
    }
    __syncthreads();
    for (int tt = 0; tt < n; ++tt) {
      const float w = w_s[tt], A = A_s[tt], sc = sc_s[tt];
      if (sc >= 0.0f) {                                  // the same for every thread of the block
#pragma unroll
        for (int c = 0; c < COLS; ++c)
#pragma unroll
          for (int i = 0; i < RMAX; ++i) S[c][i] *= sc;
      }
      const float4 x = *reinterpret_cast<const float4*>(x_s + tt * EB + COLS * col);
      const float v[COLS] = {w * x.x, w * x.y, w * x.z, w * x.w};
      const float4* cr = reinterpret_cast<const float4*>(c_s + tt * TS + part * PS);
      const float4* br = reinterpret_cast<const float4*>(b_s + tt * TS + part * PS);
      float acc[COLS][2];
#pragma unroll
      for (int c = 0; c < COLS; ++c) acc[c][0] = acc[c][1] = 0.0f;
#pragma unroll
      for (int i = 0; i < RMAX / 4; ++i) {
        const float4 k4 = br[i];
#pragma unroll
        for (int c = 0; c < COLS; ++c) {
          S[c][4 * i] = fmaf(k4.x, v[c], S[c][4 * i]);
          S[c][4 * i + 1] = fmaf(k4.y, v[c], S[c][4 * i + 1]);
          S[c][4 * i + 2] = fmaf(k4.z, v[c], S[c][4 * i + 2]);
          S[c][4 * i + 3] = fmaf(k4.w, v[c], S[c][4 * i + 3]);
        }
        if (phase != LOCAL) {
          const float4 q4 = cr[i];
#pragma unroll
          for (int c = 0; c < COLS; ++c) {
            acc[c][0] = fmaf(S[c][4 * i], q4.x, acc[c][0]);
            acc[c][1] = fmaf(S[c][4 * i + 1], q4.y, acc[c][1]);
            acc[c][0] = fmaf(S[c][4 * i + 2], q4.z, acc[c][0]);
            acc[c][1] = fmaf(S[c][4 * i + 3], q4.w, acc[c][1]);
          }
        }
      }
      if (phase != LOCAL) {
        float y[COLS];
#pragma unroll
        for (int c = 0; c < COLS; ++c) {
          // the eight parts of a column are neighbouring lanes: pairs, then fours, then all eight
          float t = acc[c][0] + acc[c][1];
          t += __shfl_xor_sync(0xffffffffu, t, 1);
          t += __shfl_xor_sync(0xffffffffu, t, 2);
          t += __shfl_xor_sync(0xffffffffu, t, 4);
          y[c] = t;
        }
        if (part == 0) {
          float* orow = out + (size_t)(c0 + tt) * H * P + (size_t)h * P;
          const float xs[COLS] = {x.x, x.y, x.z, x.w};
#pragma unroll
          for (int c = 0; c < COLS; ++c)
            if (j0 + c < P) orow[j0 + c] = fmaf(dskip, xs[c], A * y[c]);
        }
      }
    }
    const float left = end_s[0];                         // back to the state itself before the next chunk is staged
#pragma unroll
    for (int c = 0; c < COLS; ++c)
#pragma unroll
      for (int i = 0; i < RMAX; ++i) S[c][i] *= left;
  }
  if (phase == LOCAL && blockIdx.z == 0 && threadIdx.x == 0) seg_decay[(size_t)blockIdx.x * H + h] = decay_all;
  float* dst = phase == LOCAL ? sc : (last ? st : nullptr);
  if (dst == nullptr) return;
  if ((P & 3) == 0 && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
    for (int i = 0; i < RMAX; ++i) {
      const int r = part * RMAX + i;
      if (r < N && j0 < P)
        *reinterpret_cast<float4*>(dst + (size_t)r * P + j0) = make_float4(S[0][i], S[1][i], S[2][i], S[3][i]);
    }
    return;
  }
#pragma unroll
  for (int c = 0; c < COLS; ++c)
#pragma unroll
    for (int i = 0; i < RMAX; ++i) {
      const int r = part * RMAX + i;
      if (r < N && j0 + c < P) dst[(size_t)r * P + j0 + c] = S[c][i];
    }
}

// scratch[seq][seg] holds segment seg's state from zero; afterwards it holds the state the segment starts from
__global__ void mamba2_prefix_kernel(float* __restrict__ scratch, const float* __restrict__ seg_decay,
                                     const float* __restrict__ state, long long slot_stride, long long state_off,
                                     const int* __restrict__ q_start, const int* __restrict__ seq_slot, int H, int N,
                                     int P, int seg_len, int tiles_per_seq) {
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int seq = blockIdx.x;
  const size_t per = (size_t)H * N * P;
  const size_t idx = (size_t)blockIdx.y * blockDim.x + threadIdx.x;
  if (idx >= per) return;
  const int h = (int)(idx / ((size_t)N * P));
  const int q_len = q_start[seq + 1] - q_start[seq];
  const int n_seg = (q_len + seg_len - 1) / seg_len;
  float S = state[(size_t)seq_slot[seq] * slot_stride + state_off + idx];
  float* p = scratch + (size_t)seq * tiles_per_seq * per + idx;
  const float* dec = seg_decay + (size_t)seq * tiles_per_seq * H + h;
  // eight segments' states from zero and decays are on their way before the first is used (one at a time, every
  // segment would wait for its own load behind the store of the segment before)
  for (int seg0 = 0; seg0 < n_seg; seg0 += 8) {
    float local[8], d[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const bool has_local = seg0 + u + 1 < n_seg;   // the last segment left nothing
      local[u] = has_local ? p[(size_t)(seg0 + u) * per] : 0.0f;
      d[u] = has_local ? dec[(size_t)(seg0 + u) * H] : 0.0f;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (seg0 + u < n_seg) {
        p[(size_t)(seg0 + u) * per] = S;
        S = fmaf(d[u], S, local[u]);
      }
    }
  }
}

// ---- gate, then a norm over each of `parts` equal pieces ------------------------------------------------------
template <typename TO>
__global__ void gated_group_rmsnorm_kernel(const float* __restrict__ y, const float* __restrict__ gate, int gate_ld,
                                           const float* __restrict__ w, float eps, TO* __restrict__ out, int N,
                                           int parts) {
  __shared__ float scratch[33];
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int t = blockIdx.x, piece = blockIdx.y;
  const int n = N / parts, c0 = piece * n;
  const float* row = y + (size_t)t * N + c0;
  const float* g = gate + (size_t)t * gate_ld + c0;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = row[i] * silu_f(g[i]);
    ss += v * v;
  }
  ss = jb::block_sum(ss, scratch);
  const float rms = sqrtf(ss / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x)
    out[(size_t)t * N + c0 + i] = jb::from_f32<TO>(((row[i] * silu_f(g[i])) / rms) * w[c0 + i]);
}

__device__ __forceinline__ void store4_out(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4_out(bf16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<uint32_t*>(&a);
  raw.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

// Pieces made of whole 16-byte vectors: the gated values stay in shared memory between the two passes (the piece is
// read once), 16 bytes a thread.
template <typename TO>
__global__ void gated_group_rmsnorm_vec_kernel(const float* __restrict__ y, const float* __restrict__ gate, int gate_ld,
                                               const float* __restrict__ w, float eps, TO* __restrict__ out, int N,
                                               int parts) {
  extern __shared__ __align__(16) float gated_s[];       // the piece's gated values
  __shared__ float scratch[33];
  jb::pdl_launch_dependents();
  jb::pdl_wait();
  const int t = blockIdx.x, piece = blockIdx.y;
  const int n = N / parts, c0 = piece * n, n4 = n >> 2;
  const float4* row = reinterpret_cast<const float4*>(y + (size_t)t * N + c0);
  const float4* g = reinterpret_cast<const float4*>(gate + (size_t)t * gate_ld + c0);
  float4* gs = reinterpret_cast<float4*>(gated_s);
  float ss = 0.0f;
  for (int i = threadIdx.x; i < n4; i += blockDim.x) {
    const float4 a = row[i], z = g[i];
    const float4 v = make_float4(a.x * silu_f(z.x), a.y * silu_f(z.y), a.z * silu_f(z.z), a.w * silu_f(z.w));
    gs[i] = v;
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  ss = jb::block_sum(ss, scratch);
  const float rms = sqrtf(ss / (float)n + eps);
  const float4* w4 = reinterpret_cast<const float4*>(w + c0);
  for (int i = threadIdx.x; i < n4; i += blockDim.x) {     // a thread reads back what it wrote itself
    const float4 v = gs[i], ww = w4[i];
    store4_out(out + (size_t)t * N + c0 + 4 * i,
               make_float4((v.x / rms) * ww.x, (v.y / rms) * ww.y, (v.z / rms) * ww.z, (v.w / rms) * ww.w));
  }
}

}  // namespace

// out[t, c] = silu(bias[c] + sum_j w[c][j] u[t - taps + 1 + j][c]) over the columns [col0, col0 + C) of proj.
// update_state != 0: afterwards the state takes the last taps - 1 inputs of every sequence: a second launch, or, when
// every sequence brings one token (single_tokens != 0), the same launch.
JB_EXPORT int jb_causal_conv_silu(const float* proj, int ld, int col0, int C, const float* w, const float* bias, int taps,
                                  float* state, long long slot_stride, long long state_off, const int* token_seq,
                                  const int* q_start, const int* seq_slot, float* out, int T, int n_seqs,
                                  int update_state, int single_tokens, cudaStream_t stream) {
  if (T <= 0) return 0;
  JB_REFUSE(taps < 1 || ld < col0 + C, "causal_conv_silu: %d taps over columns %d..%d of %d", taps, col0, col0 + C, ld);
  JB_REFUSE(taps > 1 && state == nullptr, "causal_conv_silu: a convolution of %d taps needs its state", taps);
  JB_REFUSE(single_tokens && T != n_seqs, "causal_conv_silu: %d tokens are not one for each of %d sequences", T, n_seqs);
  const bool aligned = ((C | ld | col0) & 3) == 0 && ((slot_stride | state_off) & 3) == 0 &&
                       (((uintptr_t)proj | (uintptr_t)out | (uintptr_t)state | (uintptr_t)bias) & 15) == 0;
  if (!single_tokens && aligned && taps <= CONV_MAX_TAPS && T >= 4 * CONV_TOKENS) {
    jb::Launch cfg(dim3((T + CONV_TOKENS - 1) / CONV_TOKENS, (C / 4 + 127) / 128), dim3(128), 0, stream);
    cudaError_t e = cudaLaunchKernelEx(&cfg.c, causal_conv_silu_vec_kernel, proj, ld, col0, C, w, bias, taps,
                                       (const float*)state, slot_stride, state_off, token_seq, q_start, seq_slot, out, T);
    if (e != cudaSuccess) return (int)e;
  } else {
    const int shift_here = (update_state && single_tokens) ? 1 : 0;
    jb::Launch cfg(dim3(T, (C + 127) / 128), dim3(128), 0, stream);
    cudaError_t e = cudaLaunchKernelEx(&cfg.c, causal_conv_silu_kernel, proj, ld, col0, C, w, bias, taps,
                                       (const float*)state, slot_stride, state_off, token_seq, q_start, seq_slot, out,
                                       shift_here);
    if (e != cudaSuccess) return (int)e;
    if (shift_here) return 0;
  }
  if (update_state && taps > 1) {
    jb::Launch cfg(dim3(n_seqs, (C + 127) / 128), dim3(128), 0, stream);
    cudaError_t e = cudaLaunchKernelEx(&cfg.c, conv_state_shift_kernel, proj, ld, col0, C, taps, state, slot_stride,
                                       state_off, q_start, seq_slot);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

// xbc: float32 [T, ldx], x in columns [0, H P), B at b_col ([G][N]), C at c_col ([G][N]); dt_raw: float32 rows of
// ld_dt floats, head h in column h; dt_bias, A_log, Dskip: [H] float32; out: float32 [T, H P]; state: per slot
// slot_stride floats, the recurrence's [H][N][P] at state_off.  seg_len > 0 with scratch (n_seqs *
// ceil(max_q_len / seg_len) * H * N * P floats) and seg_decay (n_seqs * ceil(max_q_len / seg_len) * H floats)
// runs the three passes over segments; seg_len = 0 walks every sequence in one block per column block.
JB_EXPORT int jb_mamba2_scan(const float* xbc, int ldx, int b_col, int c_col, const float* dt_raw, int ld_dt,
                             const float* dt_bias, const float* A_log, const float* Dskip, float* out, float* state,
                             long long slot_stride, long long state_off, const int* q_start, const int* seq_slot,
                             int n_seqs, int H, int G, int N, int P, int max_q_len, int seg_len, float* scratch,
                             float* seg_decay, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  JB_REFUSE(N < 1 || N > 256 || P < 1, "mamba2_scan: state size %d is outside [1, 256]", N);
  JB_REFUSE(G < 1 || H % G != 0, "mamba2_scan: %d heads are not a multiple of %d groups", H, G);
  JB_REFUSE(seg_len > 0 && (scratch == nullptr || seg_decay == nullptr), "mamba2_scan: segments need scratch");
  const int rmax = N <= 64 ? 8 : N <= 128 ? 16 : 32;
  const size_t smem = (size_t)(2 * CT * PARTS * (rmax + 4) + CT * EB + 3 * CT + 4) * sizeof(float);
  const bool segmented = seg_len > 0;
  const int tiles = segmented ? (max_q_len + seg_len - 1) / seg_len : 1;
  const int seg = segmented ? seg_len : 0x40000000;
#define JB_LAUNCH_MS(RM, PHASE)                                                                                      \
  do {                                                                                                               \
    jb::Launch cfg(dim3(n_seqs * tiles, H, (P + EB - 1) / EB), dim3(THREADS), smem, stream);                         \
    cudaError_t err = cudaLaunchKernelEx(&cfg.c, mamba2_scan_kernel<RM, PHASE>, xbc, ldx, b_col, c_col, dt_raw,     \
                                         ld_dt, dt_bias, A_log, Dskip, out, state, slot_stride, state_off, q_start, \
                                         seq_slot, H, G, N, P, seg, tiles, scratch, seg_decay);                      \
    if (err != cudaSuccess) return (int)err;                                                                         \
  } while (0)
#define JB_LAUNCH_MS_R(PHASE)                       \
  do {                                              \
    if (rmax == 8) JB_LAUNCH_MS(8, PHASE);          \
    else if (rmax == 16) JB_LAUNCH_MS(16, PHASE);   \
    else JB_LAUNCH_MS(32, PHASE);                   \
  } while (0)
  if (!segmented) {
    JB_LAUNCH_MS_R(WHOLE);
    return 0;
  }
  JB_LAUNCH_MS_R(LOCAL);
  {
    const size_t per = (size_t)H * N * P;
    jb::Launch cfg(dim3(n_seqs, (unsigned)((per + 255) / 256)), dim3(256), 0, stream);
    cudaError_t err = cudaLaunchKernelEx(&cfg.c, mamba2_prefix_kernel, scratch, (const float*)seg_decay,
                                         (const float*)state, slot_stride, state_off, q_start, seq_slot, H, N, P,
                                         seg_len, tiles);
    if (err != cudaSuccess) return (int)err;
  }
  JB_LAUNCH_MS_R(FROM_START);
#undef JB_LAUNCH_MS_R
#undef JB_LAUNCH_MS
  return 0;
}

// out[t] = (y[t] * silu(gate[t])) divided, in each of `parts` equal pieces, by the piece's root mean square, times w.
// y: float32 [T, N]; gate: float32 rows of gate_ld; w: [N] float32; out [T, N] in out_dtype.
JB_EXPORT int jb_gated_group_rmsnorm(const float* y, const float* gate, int gate_ld, const float* w, float eps,
                                     void* out, int out_dtype, int T, int N, int parts, cudaStream_t stream) {
  if (T <= 0) return 0;
  JB_REFUSE(parts < 1 || N % parts != 0, "gated_group_rmsnorm: %d numbers do not fall into %d equal pieces", N, parts);
  const int n = N / parts;
  const bool aligned = ((n | N | gate_ld) & 3) == 0 && n * (int)sizeof(float) <= 48 * 1024 &&
                       (((uintptr_t)y | (uintptr_t)gate | (uintptr_t)w | (uintptr_t)out) & 15) == 0;
  if (aligned) {
    jb::Launch cfg(dim3(T, parts), dim3(n >= 2048 ? 256 : 128), (size_t)n * sizeof(float), stream);
    if (out_dtype == JB_F32)
      return (int)cudaLaunchKernelEx(&cfg.c, gated_group_rmsnorm_vec_kernel<float>, y, gate, gate_ld, w, eps, (float*)out,
                                     N, parts);
    if (out_dtype == JB_BF16)
      return (int)cudaLaunchKernelEx(&cfg.c, gated_group_rmsnorm_vec_kernel<bf16>, y, gate, gate_ld, w, eps, (bf16*)out,
                                     N, parts);
    return JB_ERR_BAD_DTYPE;
  }
  jb::Launch cfg(dim3(T, parts), dim3(n >= 2048 ? 256 : 128), 0, stream);
  if (out_dtype == JB_F32)
    return (int)cudaLaunchKernelEx(&cfg.c, gated_group_rmsnorm_kernel<float>, y, gate, gate_ld, w, eps, (float*)out, N,
                                   parts);
  if (out_dtype == JB_BF16)
    return (int)cudaLaunchKernelEx(&cfg.c, gated_group_rmsnorm_kernel<bf16>, y, gate, gate_ld, w, eps, (bf16*)out, N,
                                   parts);
  return JB_ERR_BAD_DTYPE;
}
