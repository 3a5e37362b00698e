// lm_ops.cu - element-wise and per-row kernels of token-id decoder models with a 32-bit residual stream:
//   embedding + learned positions, RMS norm with one gain ("gain norm"), the residual update of a parallel layer fused
//   with the next norm, the short causal convolution over time with its carried state fused with per-head q/k RMS norm
//   and the paged K/V write, the squared-ReLU activation, and the sigmoid top-k router with its expert grouping.
//
// Activations are `T` = bf16 (serving) or float (the all-32-bit mode); the residual stream, every norm, the router and
// all per-head constants are float in both.  Nothing allocates or synchronises; every launch is graph-capturable.
#include <math.h>

#include "common.cuh"

namespace b2 {

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

constexpr int ROW_THREADS = 256;

// sum over the block; every thread gets the result.  `red` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();                       // red may still be read from a previous call
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// h[row] = T(x[row] / sqrt(mean(x[row]^2) + eps) * gain) for the row this block owns (x just written by this block).
template <typename T>
__device__ __forceinline__ void gain_norm_tail(const float* xr, T* hr, int cols, float ssq, const float* gain, float eps,
                                               float* red) {
  const float tot = block_sum(ssq, red);
  const float inv = 1.0f / sqrtf(tot / static_cast<float>(cols) + eps);
  const float g = gain[0];
  for (int c = threadIdx.x; c < cols; c += blockDim.x) hr[c] = from_f<T>(xr[c] * inv * g);
}

// ------------------------------------------------------------------ embedding + learned position (+ first norm)
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
embed_pos_norm_kernel(const int32_t* __restrict__ tokens, const int32_t* __restrict__ positions, const T* __restrict__ embed,
                      const T* __restrict__ pos_table, float* __restrict__ x, T* __restrict__ h, const float* __restrict__ gain,
                      int cols, int vocab, int max_pos, float eps) {
  __shared__ float red[33];
  const int row = blockIdx.x;
  int tok = tokens[row], p = positions[row];
  tok = min(max(tok, 0), vocab - 1);
  p = min(max(p, 0), max_pos - 1);
  const T* er = embed + static_cast<size_t>(tok) * cols;
  const T* pr = pos_table + static_cast<size_t>(p) * cols;
  float* xr = x + static_cast<size_t>(row) * cols;
  float ssq = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float v = to_f(er[c]) + to_f(pr[c]);
    xr[c] = v;
    ssq += v * v;
  }
  if (h != nullptr) gain_norm_tail<T>(xr, h + static_cast<size_t>(row) * cols, cols, ssq, gain, eps, red);
}

// ------------------------------------------------------------------ residual update (+ next norm)
// x[row] += mult * (a[row] + b[row] + sum_k w[row, k] * z[row * top + k]) with every term optional; then, if h is
// given, h[row] = gain norm of the NEW x[row].  The expert terms are added in the order k = 0 .. top-1.
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
residual_norm_kernel(float* __restrict__ x, const T* __restrict__ a, const T* __restrict__ b, const T* __restrict__ z,
                     const float* __restrict__ zw, int top, float mult, T* __restrict__ h, const float* __restrict__ gain,
                     int cols, float eps) {
  __shared__ float red[33];
  const size_t row = blockIdx.x;
  float* xr = x + row * cols;
  float ssq = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float s = 0.f;
    if (a != nullptr) s += to_f(a[row * cols + c]);
    if (b != nullptr) s += to_f(b[row * cols + c]);
    if (z != nullptr) {
      float e = 0.f;
      for (int k = 0; k < top; ++k) e += zw[row * top + k] * to_f(z[(row * top + k) * cols + c]);
      s += e;
    }
    const float v = xr[c] + mult * s;
    xr[c] = v;
    ssq += v * v;
  }
  if (h != nullptr) gain_norm_tail<T>(xr, h + row * cols, cols, ssq, gain, eps, red);
}

// out[i] = gain norm of x[rows[i]] (the rows whose logits are wanted)
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
gather_gain_norm_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows, T* __restrict__ out,
                        const float* __restrict__ gain, int cols, float eps) {
  __shared__ float red[33];
  const size_t src = rows != nullptr ? rows[blockIdx.x] : blockIdx.x;
  const float* xr = x + src * cols;
  float ssq = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) ssq += xr[c] * xr[c];
  gain_norm_tail<T>(xr, out + static_cast<size_t>(blockIdx.x) * cols, cols, ssq, gain, eps, red);
}

// ------------------------------------------------------------------ squared ReLU, in place
template <typename T>
__global__ void relu_sq_kernel(T* __restrict__ y, size_t n) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const float v = fmaxf(to_f(y[i]), 0.f);
    y[i] = from_f<T>(v * v);
  }
}

// ------------------------------------------------------------------ short convolution + head norm + paged K/V write
// One warp per (token, head slot); head slots are the H query heads, then the G key heads, then the G value heads of the
// merged projection row u[n] = [q | k | v].  Tap j of the token at position p reads the projection of position
// p - taps + 1 + j: from this step's rows when that position is in the step's portion, from the sequence's carried
// state (its last taps - 1 projections, oldest first) when it came earlier, zero before the sequence's start.
constexpr int CONV_WARPS = 8;
constexpr int CONV_MAX_PER_LANE = 8;       // head sizes up to 256
constexpr int CONV_MAX_TAPS = 8;

template <typename T>
__global__ void __launch_bounds__(CONV_WARPS * 32)
conv_headnorm_kvwrite_kernel(const T* __restrict__ u, int64_t u_stride, const float* __restrict__ conv_w /* [C, taps] */,
                             const T* __restrict__ state /* [slots, taps-1, C] */, const int32_t* __restrict__ tok_seq,
                             const int32_t* __restrict__ positions, const int32_t* __restrict__ seq_start,
                             const int32_t* __restrict__ seq_pos0, const int32_t* __restrict__ seq_slot,
                             const int32_t* __restrict__ slot_mapping, const float* __restrict__ q_norm_w,
                             const float* __restrict__ k_norm_w, T* __restrict__ q_out /* [n, H*d] */,
                             T* __restrict__ k_cache /* [slots, G*d] */, T* __restrict__ v_cache /* [slots, G*dv] */,
                             int n_tokens, int H, int G, int d, int dv, int taps, float eps) {
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * CONV_WARPS + (threadIdx.x >> 5);
  const int heads = H + 2 * G;
  if (item >= n_tokens * heads) return;
  const int n = item / heads, hs = item % heads;
  const int slot = slot_mapping[n];
  if (slot < 0) return;                                  // padding row
  const int C = H * d + G * d + G * dv;
  int kind, head, width, c0;
  if (hs < H) { kind = 0; head = hs; width = d; c0 = head * d; }
  else if (hs < H + G) { kind = 1; head = hs - H; width = d; c0 = H * d + head * d; }
  else { kind = 2; head = hs - H - G; width = dv; c0 = H * d + G * d + head * dv; }
  const int b = tok_seq[n], p = positions[n];
  const int pos0 = seq_pos0[b], start = seq_start[b], sslot = seq_slot[b];
  const int R = taps - 1;
  // where tap j comes from: a row of u (>= 0), a state entry (encoded as -2 - r) or nothing (-1)
  int src[CONV_MAX_TAPS];
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS; ++j) {
    src[j] = -1;
    if (j < taps) {
      const int pj = p - R + j;
      if (pj >= pos0) src[j] = start + (pj - pos0);
      else if (pj >= 0) src[j] = -2 - (pj - (pos0 - R));  // state entry r holds position pos0 - R + r
    }
  }
  float y[CONV_MAX_PER_LANE];
  float ssq = 0.f;
#pragma unroll
  for (int i = 0; i < CONV_MAX_PER_LANE; ++i) {
    const int cc = lane + 32 * i;
    y[i] = 0.f;
    if (cc < width) {
      const int c = c0 + cc;
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < CONV_MAX_TAPS; ++j) {
        if (j < taps && src[j] != -1) {
          const float uv = src[j] >= 0 ? to_f(u[static_cast<int64_t>(src[j]) * u_stride + c])
                                       : to_f(state[(static_cast<size_t>(sslot) * R + (-2 - src[j])) * C + c]);
          acc += conv_w[c * taps + j] * uv;
        }
      }
      y[i] = acc;
      ssq += acc * acc;
    }
  }
  if (kind != 2) {
    // the projection and convolution outputs are activations: the norm reads them as stored in T
    ssq = 0.f;
#pragma unroll
    for (int i = 0; i < CONV_MAX_PER_LANE; ++i) { y[i] = to_f(from_f<T>(y[i])); ssq += y[i] * y[i]; }
    ssq = warp_sum(ssq);
    const float inv = 1.0f / sqrtf(ssq / static_cast<float>(width) + eps);
    const float* w = kind == 0 ? q_norm_w : k_norm_w;
#pragma unroll
    for (int i = 0; i < CONV_MAX_PER_LANE; ++i) {
      const int cc = lane + 32 * i;
      if (cc < width) y[i] = y[i] * inv * w[cc];
    }
  }
  T* dst = kind == 0 ? q_out + static_cast<size_t>(n) * H * d + head * d
         : kind == 1 ? k_cache + static_cast<size_t>(slot) * G * d + head * d
                     : v_cache + static_cast<size_t>(slot) * G * dv + head * dv;
#pragma unroll
  for (int i = 0; i < CONV_MAX_PER_LANE; ++i) {
    const int cc = lane + 32 * i;
    if (cc < width) dst[cc] = from_f<T>(y[i]);
  }
}

// The same with four adjacent channels per lane (8- or 16-byte loads and stores) for head sizes that are multiples of 4.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
  __device__ static void load(const float* p, float* f) { const float4 r = *reinterpret_cast<const float4*>(p); f[0] = r.x; f[1] = r.y; f[2] = r.z; f[3] = r.w; }
  __device__ static void store(float* p, const float* f) { *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]); }
};
template <> struct Vec4<__nv_bfloat16> {
  __device__ static void load(const __nv_bfloat16* p, float* f) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    f[0] = bf16lo(r.x); f[1] = bf16hi(r.x); f[2] = bf16lo(r.y); f[3] = bf16hi(r.y);
  }
  __device__ static void store(__nv_bfloat16* p, const float* f) { *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3])); }
};
constexpr int CONV4_CHUNKS = 2;            // head sizes up to 256
constexpr int CONV4_TOKENS = 8;            // consecutive rows of the step per warp: the taps' weights are loaded once for all

// One warp per (block of CONV4_TOKENS rows, head slice).  The lane keeps the taps of its four channels in registers.
template <typename T, int TAPS, int NCH>
__global__ void __launch_bounds__(CONV_WARPS * 32)
conv_headnorm_kvwrite_vec4_kernel(const T* __restrict__ u, int64_t u_stride, const float* __restrict__ conv_w,
                                  const T* __restrict__ state, const int32_t* __restrict__ tok_seq,
                                  const int32_t* __restrict__ positions, const int32_t* __restrict__ seq_start,
                                  const int32_t* __restrict__ seq_pos0, const int32_t* __restrict__ seq_slot,
                                  const int32_t* __restrict__ slot_mapping, const float* __restrict__ q_norm_w,
                                  const float* __restrict__ k_norm_w, T* __restrict__ q_out, T* __restrict__ k_cache,
                                  T* __restrict__ v_cache, int n_tokens, int H, int G, int d, int dv, float eps) {
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * CONV_WARPS + (threadIdx.x >> 5);
  const int heads = H + 2 * G;
  const int n_blocks = (n_tokens + CONV4_TOKENS - 1) / CONV4_TOKENS;
  if (item >= n_blocks * heads) return;
  const int n0 = (item / heads) * CONV4_TOKENS, hs = item % heads;
  const int C = H * d + G * d + G * dv;
  int kind, head, width, c0;
  if (hs < H) { kind = 0; head = hs; width = d; c0 = head * d; }
  else if (hs < H + G) { kind = 1; head = hs - H; width = d; c0 = H * d + head * d; }
  else { kind = 2; head = hs - H - G; width = dv; c0 = H * d + G * d + head * dv; }
  constexpr int R = TAPS - 1;
  float w[NCH][4][TAPS];
  float g4[NCH][4];
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    const int cc = (lane + 32 * i) * 4;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      g4[i][e] = 0.f;
#pragma unroll
      for (int j = 0; j < TAPS; ++j) w[i][e][j] = 0.f;
    }
    if (cc < width) {
      // the lane's 4 channels x TAPS taps are 16 * TAPS contiguous, 16-byte aligned bytes: TAPS vector loads
      float flat[4 * TAPS];
#pragma unroll
      for (int v = 0; v < TAPS; ++v) {
        const float4 r = *reinterpret_cast<const float4*>(conv_w + static_cast<size_t>(c0 + cc) * TAPS + 4 * v);
        flat[4 * v] = r.x; flat[4 * v + 1] = r.y; flat[4 * v + 2] = r.z; flat[4 * v + 3] = r.w;
      }
#pragma unroll
      for (int e = 0; e < 4; ++e)
#pragma unroll
        for (int j = 0; j < TAPS; ++j) w[i][e][j] = flat[e * TAPS + j];
      if (kind != 2) {
        const float4 r = *reinterpret_cast<const float4*>((kind == 0 ? q_norm_w : k_norm_w) + cc);
        g4[i][0] = r.x; g4[i][1] = r.y; g4[i][2] = r.z; g4[i][3] = r.w;
      }
    }
  }
  // the rows' bookkeeping (three dependent loads each) is fetched by one lane per row, all rows at once
  int m_slot = -1, m_p = 0, m_pos0 = 0, m_start = 0, m_sslot = 0;
  if (lane < CONV4_TOKENS && n0 + lane < n_tokens) {
    m_slot = slot_mapping[n0 + lane];
    if (m_slot >= 0) {
      const int b = tok_seq[n0 + lane];
      m_p = positions[n0 + lane];
      m_pos0 = seq_pos0[b]; m_start = seq_start[b]; m_sslot = seq_slot[b];
    }
  }
  // norm of a q / k head (the convolution's output rounded to T first), then the row's destination
  auto finish = [&](float (&y)[NCH][4], int n, int slot) {
    if (kind != 2) {
      float ssq = 0.f;
#pragma unroll
      for (int i = 0; i < NCH; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) { y[i][e] = to_f(from_f<T>(y[i][e])); ssq += y[i][e] * y[i][e]; }
      ssq = warp_sum(ssq);
      const float inv = 1.0f / sqrtf(ssq / static_cast<float>(width) + eps);
#pragma unroll
      for (int i = 0; i < NCH; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) y[i][e] *= inv * g4[i][e];
    }
    T* dst = kind == 0 ? q_out + static_cast<size_t>(n) * H * d + head * d
           : kind == 1 ? k_cache + static_cast<size_t>(slot) * G * d + head * d
                       : v_cache + static_cast<size_t>(slot) * G * dv + head * dv;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const int cc = (lane + 32 * i) * 4;
      if (cc < width) Vec4<T>::store(dst + cc, y[i]);
    }
  };
  // The usual block of a prompt portion: CONV4_TOKENS consecutive tokens of one sequence.  Their projections and the
  // taps - 1 before the first are loaded once, all loads issued before the first use; row t then reads entries t .. t + R.
  const int p0 = __shfl_sync(0xffffffffu, m_p, 0), start0 = __shfl_sync(0xffffffffu, m_start, 0);
  const bool mine = lane >= CONV4_TOKENS || (m_slot >= 0 && m_start == start0 && m_p == p0 + lane);
  if (__all_sync(0xffffffffu, mine)) {
    const int pos0 = __shfl_sync(0xffffffffu, m_pos0, 0), sslot = __shfl_sync(0xffffffffu, m_sslot, 0);
    float uv[CONV4_TOKENS + R][NCH][4];
#pragma unroll
    for (int k = 0; k < CONV4_TOKENS + R; ++k) {
      const int pk = p0 - R + k;
#pragma unroll
      for (int i = 0; i < NCH; ++i) {
        const int cc = (lane + 32 * i) * 4;
#pragma unroll
        for (int e = 0; e < 4; ++e) uv[k][i][e] = 0.f;             // before the sequence's start
        if (cc < width) {
          if (pk >= pos0) Vec4<T>::load(u + static_cast<int64_t>(start0 + pk - pos0) * u_stride + c0 + cc, uv[k][i]);
          else if (pk >= 0) Vec4<T>::load(state + (static_cast<size_t>(sslot) * R + (pk - (pos0 - R))) * C + c0 + cc, uv[k][i]);
        }
      }
    }
#pragma unroll
    for (int t = 0; t < CONV4_TOKENS; ++t) {
      float y[NCH][4];
#pragma unroll
      for (int i = 0; i < NCH; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          y[i][e] = 0.f;
#pragma unroll
          for (int j = 0; j < TAPS; ++j) y[i][e] = fmaf(w[i][e][j], uv[t + j][i][e], y[i][e]);
        }
      finish(y, n0 + t, __shfl_sync(0xffffffffu, m_slot, t));
    }
    return;
  }
  // anything else (decoded tokens, the seam of two sequences, padding): row by row
#pragma unroll
  for (int t = 0; t < CONV4_TOKENS; ++t) {
    const int n = n0 + t;
    const int slot = __shfl_sync(0xffffffffu, m_slot, t);
    if (slot < 0) continue;                  // padding row, or past the step's last row
    const int p = __shfl_sync(0xffffffffu, m_p, t), pos0 = __shfl_sync(0xffffffffu, m_pos0, t);
    const int start = __shfl_sync(0xffffffffu, m_start, t), sslot = __shfl_sync(0xffffffffu, m_sslot, t);
    const T* src[TAPS];                      // row of tap j (nullptr: before the sequence's start)
#pragma unroll
    for (int j = 0; j < TAPS; ++j) {
      const int pj = p - R + j;
      src[j] = nullptr;
      if (pj >= pos0) src[j] = u + static_cast<int64_t>(start + pj - pos0) * u_stride;
      else if (pj >= 0) src[j] = state + (static_cast<size_t>(sslot) * R + (pj - (pos0 - R))) * C;
    }
    float y[NCH][4];
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const int cc = (lane + 32 * i) * 4;
#pragma unroll
      for (int e = 0; e < 4; ++e) y[i][e] = 0.f;
      if (cc < width) {
#pragma unroll
        for (int j = 0; j < TAPS; ++j) {
          if (src[j] != nullptr) {
            float uv[4];
            Vec4<T>::load(src[j] + c0 + cc, uv);
#pragma unroll
            for (int e = 0; e < 4; ++e) y[i][e] = fmaf(w[i][e][j], uv[e], y[i][e]);
          }
        }
      }
    }
    finish(y, n, slot);
  }
}

// The carried state after the step: entry r holds the projection of position end - R + r (end = pos0 + new tokens).
// One thread per (sequence, channel) reads its old entries before it writes any, so the shift is safe in place.
template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ u, int64_t u_stride, T* __restrict__ state,
                                         const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_pos0,
                                         const int32_t* __restrict__ seq_len, const int32_t* __restrict__ seq_slot,
                                         int n_seqs, int C, int taps) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  if (c >= C || b >= n_seqs) return;
  const int len = seq_len[b];
  if (len <= 0) return;                                  // padding row
  const int R = taps - 1, pos0 = seq_pos0[b], start = seq_start[b];
  T* st = state + static_cast<size_t>(seq_slot[b]) * R * C + c;
  T old[CONV_MAX_TAPS];
#pragma unroll
  for (int r = 0; r < CONV_MAX_TAPS; ++r) if (r < R) old[r] = st[static_cast<size_t>(r) * C];
  const int end = pos0 + len;
#pragma unroll
  for (int r = 0; r < CONV_MAX_TAPS; ++r) {
    if (r < R) {
      const int pj = end - R + r;
      T v = from_f<T>(0.f);
      if (pj >= pos0) v = u[static_cast<int64_t>(start + pj - pos0) * u_stride + c];
      else if (pj >= 0) v = old[pj - (pos0 - R)];
      st[static_cast<size_t>(r) * C] = v;
    }
  }
}

// ------------------------------------------------------------------ top-k router
// One warp per token: logits over the experts in 32-bit, the `top` largest scores chosen (ties: the lower index).
// mode 0: scores = sigmoid, weights = score / (sum of the chosen scores + 1e-20) * scale.
// mode 1: scores = logits + bias, weights = softmax over the chosen scores * scale.
// mode 2: scores = softmax over ALL logits; the choice is made on score + bias, the weights are the chosen scores
//         themselves * scale, not renormalised.
constexpr int ROUTE_WARPS = 4;
constexpr int ROUTE_MAX_EXPERTS = 256;

template <typename T>
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_kernel(const T* __restrict__ h, const float* __restrict__ router /* [E, cols] */, int32_t* __restrict__ top_idx,
                 float* __restrict__ top_w, int n_tokens, int cols, int E, int top, float scale,
                 const float* __restrict__ bias /* [E] or null */, int mode) {
  __shared__ float score[ROUTE_WARPS][ROUTE_MAX_EXPERTS];
  __shared__ float weight[ROUTE_WARPS][ROUTE_MAX_EXPERTS];   // mode 2: the scores the weights are taken from
  const int softmax_chosen = mode == 1;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n = blockIdx.x * ROUTE_WARPS + warp;
  if (n >= n_tokens) return;
  const T* hr = h + static_cast<size_t>(n) * cols;
  // one expert at a time: the warps of a launch walk the router together, so a row is fetched once and then served by L1 / L2
  // (scoring 4 or 16 experts per pass over the token's row was measured slower, for 64 tokens and for 8192)
  for (int e = 0; e < E; ++e) {
    const float* wr = router + static_cast<size_t>(e) * cols;
    float acc = 0.f;
    for (int c = lane; c < cols; c += 32) acc += to_f(hr[c]) * wr[c];
    acc = warp_sum(acc);
    if (lane == 0) {
      if (mode == 2) {
        score[warp][e] = acc >= -3.0e38f ? acc : -3.0e38f;
      } else if (softmax_chosen) {
        const float sc = acc + (bias != nullptr ? bias[e] : 0.f);
        score[warp][e] = sc >= -3.0e38f ? sc : -3.0e38f;  // a NaN input still yields valid expert ids
      } else {
        const float sc = 1.0f / (1.0f + expf(-acc));
        score[warp][e] = sc >= 0.f ? sc : 0.f;
      }
    }
  }
  __syncwarp();
  if (mode == 2) {                                       // softmax over all experts, then the choice scores
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, score[warp][e]);
    mx = warp_max(mx);
    float den = 0.f;
    for (int e = lane; e < E; e += 32) den += expf(score[warp][e] - mx);
    den = warp_sum(den);
    for (int e = lane; e < E; e += 32) {
      const float p = expf(score[warp][e] - mx) / den;
      weight[warp][e] = p;
      score[warp][e] = p + (bias != nullptr ? bias[e] : 0.f);
    }
    __syncwarp();
  }
  float sum = 0.f, first = 0.f;
  float chosen_s = 0.f;          // lane k keeps the k-th choice
  int chosen_e = 0;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int be = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float s = score[warp][e];
      if (s > best) { best = s; be = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ob > best || (ob == best && oe < be)) { best = ob; be = oe; }
    }
    if (k == 0) first = best;
    if (softmax_chosen) best = expf(best - first);       // weights: the softmax over the chosen logits only
    if (mode == 2) best = weight[warp][be];
    if (lane == (k & 31)) { chosen_s = best; chosen_e = be; }
    sum += best;
    if (lane == 0) score[warp][be] = -INFINITY;
    __syncwarp();
  }
  if (lane < top) {
    top_idx[static_cast<size_t>(n) * top + lane] = chosen_e;
    top_w[static_cast<size_t>(n) * top + lane] = mode == 2 ? chosen_s * scale
                                                 : softmax_chosen ? chosen_s / sum * scale : chosen_s / (sum + 1e-20f) * scale;
  }
}

// Group the (token, choice) pairs by expert: offsets[e] .. offsets[e+1] index `sorted_pair`, which holds pair ids
// (token * top + choice).  One block; the order inside a group is arbitrary (no result depends on it).
__global__ void __launch_bounds__(1024)
moe_group_kernel(const int32_t* __restrict__ top_idx, int32_t* __restrict__ offsets, int32_t* __restrict__ sorted_pair,
                 int n_pairs, int E) {
  __shared__ int count[ROUTE_MAX_EXPERTS + 1];
  __shared__ int cursor[ROUTE_MAX_EXPERTS];
  for (int e = threadIdx.x; e <= E; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) atomicAdd(&count[top_idx[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) { const int c = count[e]; cursor[e] = run; offsets[e] = run; run += c; }
    offsets[E] = run;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) sorted_pair[atomicAdd(&cursor[top_idx[i]], 1)] = i;
}

template <typename T>
static void launch_conv(bool vec4, int grid, cudaStream_t st, const void* u, int64_t u_stride, const float* conv_w, void* state,
                        const int32_t* tok_seq, const int32_t* positions, const int32_t* seq_start, const int32_t* seq_pos0,
                        const int32_t* seq_len, const int32_t* seq_slot, const int32_t* slot_mapping, const float* q_norm_w,
                        const float* k_norm_w, void* q_out, void* k_cache, void* v_cache, int n_tokens, int n_seqs, int H, int G, int d,
                        int dv, int taps, float eps, int C) {
#define CONV4_GO_N(TP, NCH) conv_headnorm_kvwrite_vec4_kernel<T, TP, NCH><<<grid, CONV_WARPS * 32, 0, st>>>(static_cast<const T*>(u), u_stride, conv_w, \
      static_cast<const T*>(state), tok_seq, positions, seq_start, seq_pos0, seq_slot, slot_mapping, q_norm_w, k_norm_w, \
      static_cast<T*>(q_out), static_cast<T*>(k_cache), static_cast<T*>(v_cache), n_tokens, H, G, d, dv, eps)
#define CONV4_GO(TP) do { if (d <= 128 && dv <= 128) CONV4_GO_N(TP, 1); else CONV4_GO_N(TP, 2); } while (0)
  if (vec4) grid = ((n_tokens + CONV4_TOKENS - 1) / CONV4_TOKENS * (H + 2 * G) + CONV_WARPS - 1) / CONV_WARPS;
  if (vec4 && taps == 4) CONV4_GO(4);
  else if (vec4 && taps == 3) CONV4_GO(3);
  else if (vec4 && taps == 2) CONV4_GO(2);
  else if (vec4 && taps == 1) CONV4_GO(1);
  else
    conv_headnorm_kvwrite_kernel<T><<<grid, CONV_WARPS * 32, 0, st>>>(static_cast<const T*>(u), u_stride, conv_w, static_cast<const T*>(state),
        tok_seq, positions, seq_start, seq_pos0, seq_slot, slot_mapping, q_norm_w, k_norm_w, static_cast<T*>(q_out),
        static_cast<T*>(k_cache), static_cast<T*>(v_cache), n_tokens, H, G, d, dv, taps, eps);
#undef CONV4_GO
#undef CONV4_GO_N
  if (taps > 1)
    conv_state_update_kernel<T><<<dim3((C + 127) / 128, n_seqs), 128, 0, st>>>(static_cast<const T*>(u), u_stride, static_cast<T*>(state),
        seq_start, seq_pos0, seq_len, seq_slot, n_seqs, C, taps);
}

template <typename T>
static int launch_residual(float* x, const void* a, const void* b, const void* z, const float* zw, int top, float mult,
                           void* h, const float* gain, int rows, int cols, float eps, cudaStream_t st) {
  residual_norm_kernel<T><<<rows, ROW_THREADS, 0, st>>>(x, static_cast<const T*>(a), static_cast<const T*>(b),
                                                         static_cast<const T*>(z), zw, top, mult, static_cast<T*>(h), gain,
                                                         cols, eps);
  return 0;
}

}  // namespace b2

#define LM_DTYPE_OK(dt) ((dt) == B2TTS_DTYPE_BF16 || (dt) == B2TTS_DTYPE_F32)

extern "C" int b2tts_embed_pos_norm(const int32_t* tokens, const int32_t* positions, const void* embed, const void* pos_table,
                                    float* x, void* h, const float* gain, int rows, int cols, int vocab, int max_pos,
                                    float eps, int dtype, void* stream) {
  using namespace b2;
  B2_REQUIRE(rows >= 0 && cols > 0 && vocab > 0 && max_pos > 0, B2TTS_EINVAL, "embed_pos_norm: rows=%d cols=%d", rows, cols);
  B2_REQUIRE(LM_DTYPE_OK(dtype), B2TTS_EINVAL, "embed_pos_norm: dtype %d", dtype);
  if (rows == 0) return B2TTS_OK;
  B2_REQUIRE(tokens && positions && embed && pos_table && x && (!h || gain), B2TTS_EINVAL, "embed_pos_norm: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == B2TTS_DTYPE_BF16)
    embed_pos_norm_kernel<__nv_bfloat16><<<rows, ROW_THREADS, 0, st>>>(tokens, positions, static_cast<const __nv_bfloat16*>(embed),
        static_cast<const __nv_bfloat16*>(pos_table), x, static_cast<__nv_bfloat16*>(h), gain, cols, vocab, max_pos, eps);
  else
    embed_pos_norm_kernel<float><<<rows, ROW_THREADS, 0, st>>>(tokens, positions, static_cast<const float*>(embed),
        static_cast<const float*>(pos_table), x, static_cast<float*>(h), gain, cols, vocab, max_pos, eps);
  B2_CHECK_LAUNCH("embed_pos_norm");
  return B2TTS_OK;
}

extern "C" int b2tts_residual_norm(float* x, const void* a, const void* b, const void* z, const float* zw, int top, float mult,
                                   void* h, const float* gain, int rows, int cols, float eps, int dtype, void* stream) {
  using namespace b2;
  B2_REQUIRE(rows >= 0 && cols > 0 && top >= 0, B2TTS_EINVAL, "residual_norm: rows=%d cols=%d top=%d", rows, cols, top);
  B2_REQUIRE(LM_DTYPE_OK(dtype), B2TTS_EINVAL, "residual_norm: dtype %d", dtype);
  if (rows == 0) return B2TTS_OK;
  B2_REQUIRE(x && (!h || gain) && (!z || (zw && top > 0)), B2TTS_EINVAL, "residual_norm: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == B2TTS_DTYPE_BF16) launch_residual<__nv_bfloat16>(x, a, b, z, zw, top, mult, h, gain, rows, cols, eps, st);
  else launch_residual<float>(x, a, b, z, zw, top, mult, h, gain, rows, cols, eps, st);
  B2_CHECK_LAUNCH("residual_norm");
  return B2TTS_OK;
}

extern "C" int b2tts_gather_gain_norm(const float* x, const int32_t* rows_idx, void* out, const float* gain, int rows, int cols,
                                      float eps, int dtype, void* stream) {
  using namespace b2;
  B2_REQUIRE(rows >= 0 && cols > 0, B2TTS_EINVAL, "gather_gain_norm: rows=%d cols=%d", rows, cols);
  B2_REQUIRE(LM_DTYPE_OK(dtype), B2TTS_EINVAL, "gather_gain_norm: dtype %d", dtype);
  if (rows == 0) return B2TTS_OK;
  B2_REQUIRE(x && out && gain, B2TTS_EINVAL, "gather_gain_norm: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == B2TTS_DTYPE_BF16)
    gather_gain_norm_kernel<__nv_bfloat16><<<rows, ROW_THREADS, 0, st>>>(x, rows_idx, static_cast<__nv_bfloat16*>(out), gain, cols, eps);
  else
    gather_gain_norm_kernel<float><<<rows, ROW_THREADS, 0, st>>>(x, rows_idx, static_cast<float*>(out), gain, cols, eps);
  B2_CHECK_LAUNCH("gather_gain_norm");
  return B2TTS_OK;
}

extern "C" int b2tts_relu_sq(void* y, int64_t n, int dtype, void* stream) {
  using namespace b2;
  B2_REQUIRE(n >= 0 && LM_DTYPE_OK(dtype), B2TTS_EINVAL, "relu_sq: n=%lld dtype=%d", static_cast<long long>(n), dtype);
  if (n == 0) return B2TTS_OK;
  B2_REQUIRE(y, B2TTS_EINVAL, "relu_sq: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = static_cast<int>(std::min<int64_t>((n + 255) / 256, 148 * 16));
  if (dtype == B2TTS_DTYPE_BF16) relu_sq_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<__nv_bfloat16*>(y), static_cast<size_t>(n));
  else relu_sq_kernel<float><<<grid, 256, 0, st>>>(static_cast<float*>(y), static_cast<size_t>(n));
  B2_CHECK_LAUNCH("relu_sq");
  return B2TTS_OK;
}

extern "C" int b2tts_conv_headnorm_kvwrite(const void* u, int64_t u_stride, const float* conv_w, void* state,
                                           const int32_t* tok_seq, const int32_t* positions, const int32_t* seq_start,
                                           const int32_t* seq_pos0, const int32_t* seq_len, const int32_t* seq_slot,
                                           const int32_t* slot_mapping, const float* q_norm_w, const float* k_norm_w,
                                           void* q_out, void* k_cache, void* v_cache, int n_tokens, int n_seqs, int heads,
                                           int kv_heads, int dim, int vdim, int taps, float eps, int dtype, void* stream) {
  using namespace b2;
  B2_REQUIRE(n_tokens >= 0 && n_seqs >= 0 && heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0, B2TTS_EINVAL,
             "conv_headnorm_kvwrite: bad sizes");
  B2_REQUIRE(taps >= 1 && taps <= CONV_MAX_TAPS, B2TTS_EUNSUPPORTED, "conv_headnorm_kvwrite: taps %d not in 1..%d", taps, CONV_MAX_TAPS);
  B2_REQUIRE(dim <= 32 * CONV_MAX_PER_LANE && vdim <= 32 * CONV_MAX_PER_LANE, B2TTS_EUNSUPPORTED,
             "conv_headnorm_kvwrite: head size above %d", 32 * CONV_MAX_PER_LANE);
  B2_REQUIRE(LM_DTYPE_OK(dtype), B2TTS_EINVAL, "conv_headnorm_kvwrite: dtype %d", dtype);
  if (n_tokens == 0 || n_seqs == 0) return B2TTS_OK;
  B2_REQUIRE(u && conv_w && (state || taps == 1) && tok_seq && positions && seq_start && seq_pos0 && seq_len && seq_slot &&
             slot_mapping && q_norm_w && k_norm_w && q_out && k_cache && v_cache, B2TTS_EINVAL, "conv_headnorm_kvwrite: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int items = n_tokens * (heads + 2 * kv_heads);
  const int grid = (items + CONV_WARPS - 1) / CONV_WARPS;
  const int C = heads * dim + kv_heads * dim + kv_heads * vdim;
  // four channels per lane when every head slice and row starts on a 16-byte (float) / 8-byte (bf16) boundary
  const bool vec4 = dim % 4 == 0 && vdim % 4 == 0 && u_stride % 4 == 0 && dim <= 128 * CONV4_CHUNKS && vdim <= 128 * CONV4_CHUNKS &&
                    (taps == 1 || taps == 2 || taps == 3 || taps == 4) && aligned16(u) && aligned16(q_out) && aligned16(k_cache) &&
                    aligned16(v_cache) && aligned16(conv_w) && aligned16(q_norm_w) && aligned16(k_norm_w) && (taps == 1 || aligned16(state));
  if (dtype == B2TTS_DTYPE_BF16)
    launch_conv<__nv_bfloat16>(vec4, grid, st, u, u_stride, conv_w, state, tok_seq, positions, seq_start, seq_pos0, seq_len, seq_slot,
                               slot_mapping, q_norm_w, k_norm_w, q_out, k_cache, v_cache, n_tokens, n_seqs, heads, kv_heads, dim, vdim, taps, eps, C);
  else
    launch_conv<float>(vec4, grid, st, u, u_stride, conv_w, state, tok_seq, positions, seq_start, seq_pos0, seq_len, seq_slot,
                       slot_mapping, q_norm_w, k_norm_w, q_out, k_cache, v_cache, n_tokens, n_seqs, heads, kv_heads, dim, vdim, taps, eps, C);
  B2_CHECK_LAUNCH("conv_headnorm_kvwrite");
  return B2TTS_OK;
}

extern "C" int b2tts_moe_route(const void* h, const float* router, int32_t* top_idx, float* top_w, int32_t* offsets,
                               int32_t* sorted_pair, int n_tokens, int cols, int experts, int top, float scale,
                               const float* bias, int mode, int dtype, void* stream) {
  using namespace b2;
  B2_REQUIRE(n_tokens >= 0 && cols > 0 && experts > 0 && top > 0 && top <= experts, B2TTS_EINVAL, "moe_route: bad sizes");
  B2_REQUIRE(mode >= 0 && mode <= 2, B2TTS_EINVAL, "moe_route: mode %d", mode);
  B2_REQUIRE(experts <= ROUTE_MAX_EXPERTS && top <= 32, B2TTS_EUNSUPPORTED, "moe_route: experts %d > %d or top %d > 32", experts,
             ROUTE_MAX_EXPERTS, top);
  B2_REQUIRE(LM_DTYPE_OK(dtype), B2TTS_EINVAL, "moe_route: dtype %d", dtype);
  B2_REQUIRE(offsets && sorted_pair, B2TTS_EINVAL, "moe_route: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n_tokens > 0) {
    B2_REQUIRE(h && router && top_idx && top_w, B2TTS_EINVAL, "moe_route: null pointer");
    const int grid = (n_tokens + ROUTE_WARPS - 1) / ROUTE_WARPS;
    if (dtype == B2TTS_DTYPE_BF16)
      moe_route_kernel<__nv_bfloat16><<<grid, ROUTE_WARPS * 32, 0, st>>>(static_cast<const __nv_bfloat16*>(h), router, top_idx, top_w,
                                                                          n_tokens, cols, experts, top, scale, bias, mode);
    else
      moe_route_kernel<float><<<grid, ROUTE_WARPS * 32, 0, st>>>(static_cast<const float*>(h), router, top_idx, top_w, n_tokens, cols,
                                                                 experts, top, scale, bias, mode);
    B2_CHECK_LAUNCH("moe_route");
  }
  moe_group_kernel<<<1, 1024, 0, st>>>(top_idx, offsets, sorted_pair, n_tokens * top, experts);
  B2_CHECK_LAUNCH("moe_group");
  return B2TTS_OK;
}
