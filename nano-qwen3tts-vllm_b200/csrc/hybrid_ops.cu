// hybrid_ops.cu - per-row kernels of decoders that keep several copies of the residual stream ("streams", mixed by small
// learned matrices around every sublayer) and pair an attention branch with a recurrent branch in one mixer:
//   token + hashed-bigram embedding into all streams; the stream update after a sublayer fused with the read-out and
//   RMS norm in front of the next one; the final sum of the streams with its norm on gathered rows; the preparation of an
//   attention step (biases, RMS norm over a whole projection, half-split rotation, paged K/V write, values that are the
//   raw keys); a short causal convolution over time with an activation and its carried state; the gate and grouped RMS
//   norm on a recurrent branch's output.
//
// Activations are `T` = bf16 (serving) or float (the all-32-bit mode).  The streams, every norm, angle and gate are float
// in both.  Nothing allocates or synchronises; every launch is graph-capturable.
#include <algorithm>

#include "row_ops.cuh"

namespace b2 {
namespace row {

constexpr int ROW_THREADS = 256;
constexpr int MAX_STREAMS = 8;

// ------------------------------------------------------------------ embedding: token row + bigram row -> every stream
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
embed_bigram_kernel(const int32_t* __restrict__ tokens, const int32_t* __restrict__ prev_tokens, const T* __restrict__ embed,
                    const T* __restrict__ bigram, float* __restrict__ xs, int cols, int streams, int vocab, int buckets,
                    int mul_prev, int mul_cur) {
  const int r = blockIdx.x;
  int tok = tokens[r];
  const int prev = prev_tokens[r];
  const T* br = nullptr;
  if (bigram != nullptr) {
    long long h = buckets;                                                   // a sequence's first token: the extra row
    if (prev >= 0) h = (static_cast<long long>(prev) * mul_prev + static_cast<long long>(tok) * mul_cur) % buckets;
    br = bigram + static_cast<size_t>(h) * cols;
  }
  tok = min(max(tok, 0), vocab - 1);
  const T* er = embed + static_cast<size_t>(tok) * cols;
  float* xr = xs + static_cast<size_t>(r) * streams * cols;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float v = to_f(er[c]);
    if (br != nullptr) v += to_f(br[c]);
    for (int s = 0; s < streams; ++s) xr[static_cast<size_t>(s) * cols + c] = v;
  }
}

// ------------------------------------------------------------------ stream update + read-out + norm
// Row r holds `streams` copies x_0 .. x_(s-1) of `cols` floats.  If y1 is given, all copies are replaced at once from
// the old ones: x_t <- sum_s mix[s, t] x_s + out_w[t] * (c1 * y1 + c2 * y2).  Then, if h is given, the read-out
// u = sum_s in_w[s] x_s (in_w null: the plain sum) is RMS-normed with norm_w into h.
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
stream_mix_norm_kernel(float* __restrict__ xs, const T* __restrict__ y1, const T* __restrict__ y2, float c1, float c2,
                       const float* __restrict__ mix, const float* __restrict__ out_w, const float* __restrict__ in_w,
                       const float* __restrict__ norm_w, T* __restrict__ h, int cols, int streams, float eps) {
  __shared__ float red[33];
  __shared__ float s_mix[MAX_STREAMS * MAX_STREAMS], s_out[MAX_STREAMS], s_in[MAX_STREAMS];
  if (threadIdx.x < streams * streams && y1 != nullptr) s_mix[threadIdx.x] = mix[threadIdx.x];
  if (threadIdx.x < streams) {
    s_out[threadIdx.x] = y1 != nullptr ? out_w[threadIdx.x] : 0.f;
    s_in[threadIdx.x] = in_w != nullptr ? in_w[threadIdx.x] : 1.f;
  }
  __syncthreads();
  const size_t r = blockIdx.x;
  float* xr = xs + r * streams * cols;
  float ssq = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float x[MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < MAX_STREAMS; ++s) x[s] = s < streams ? xr[static_cast<size_t>(s) * cols + c] : 0.f;
    float u = 0.f;
    if (y1 != nullptr) {
      float y = c1 * to_f(y1[r * cols + c]);
      if (y2 != nullptr) y += c2 * to_f(y2[r * cols + c]);
#pragma unroll
      for (int t = 0; t < MAX_STREAMS; ++t) {
        if (t < streams) {
          float acc = 0.f;
#pragma unroll
          for (int s = 0; s < MAX_STREAMS; ++s) if (s < streams) acc += s_mix[s * streams + t] * x[s];
          acc += s_out[t] * y;
          xr[static_cast<size_t>(t) * cols + c] = acc;
          u += s_in[t] * acc;
        }
      }
    } else {
#pragma unroll
      for (int t = 0; t < MAX_STREAMS; ++t) if (t < streams) u += s_in[t] * x[t];
    }
    ssq += u * u;
  }
  if (h == nullptr) return;
  const float tot = block_sum(ssq, red);
  const float inv = 1.0f / sqrtf(tot / static_cast<float>(cols) + eps);
  T* hr = h + r * cols;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {             // the same thread wrote these columns above
    float u = 0.f;
    for (int t = 0; t < streams; ++t) u += s_in[t] * xr[static_cast<size_t>(t) * cols + c];
    hr[c] = from_f<T>(u * inv * norm_w[c]);
  }
}

// four consecutive activations <-> floats (16-byte loads for float, 8-byte for bf16); p must be aligned accordingly
template <typename T> __device__ __forceinline__ float4 load4(const T* p);
template <> __device__ __forceinline__ float4 load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 r = ldg_v2(p);
  return make_float4(bf16lo(r.x), bf16hi(r.x), bf16lo(r.y), bf16hi(r.y));
}
template <typename T> __device__ __forceinline__ void store4(T* p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  stg_v2(p, make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w)));
}

// The same update and read-out for rows of cols % 4 == 0 and cols <= 4 * SMV_KEEP * ROW_THREADS: a thread owns groups of
// four consecutive columns, moves them as vectors and keeps its read-out values in registers for the norm, so the
// streams are read once and written once.
constexpr int SMV_KEEP = 4;

template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
stream_mix_norm_vec4_kernel(float* __restrict__ xs, const T* __restrict__ y1, const T* __restrict__ y2, float c1, float c2,
                            const float* __restrict__ mix, const float* __restrict__ out_w, const float* __restrict__ in_w,
                            const float* __restrict__ norm_w, T* __restrict__ h, int cols, int streams, float eps) {
  __shared__ float red[33];
  __shared__ float s_mix[MAX_STREAMS * MAX_STREAMS], s_out[MAX_STREAMS], s_in[MAX_STREAMS];
  if (threadIdx.x < streams * streams && y1 != nullptr) s_mix[threadIdx.x] = mix[threadIdx.x];
  if (threadIdx.x < streams) {
    s_out[threadIdx.x] = y1 != nullptr ? out_w[threadIdx.x] : 0.f;
    s_in[threadIdx.x] = in_w != nullptr ? in_w[threadIdx.x] : 1.f;
  }
  __syncthreads();
  const size_t r = blockIdx.x;
  float* xr = xs + r * streams * cols;
  float4 keep[SMV_KEEP];
  float ssq = 0.f;
#pragma unroll
  for (int it = 0; it < SMV_KEEP; ++it) {
    const int c = (threadIdx.x + it * ROW_THREADS) * 4;
    keep[it] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c >= cols) continue;
    float4 x[MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < MAX_STREAMS; ++s)
      if (s < streams) x[s] = *reinterpret_cast<const float4*>(xr + static_cast<size_t>(s) * cols + c);
    float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
    if (y1 != nullptr) {
      float4 y = load4<T>(y1 + r * cols + c);
      y.x *= c1; y.y *= c1; y.z *= c1; y.w *= c1;
      if (y2 != nullptr) {
        const float4 z = load4<T>(y2 + r * cols + c);
        y.x += c2 * z.x; y.y += c2 * z.y; y.z += c2 * z.z; y.w += c2 * z.w;
      }
#pragma unroll
      for (int t = 0; t < MAX_STREAMS; ++t) {
        if (t < streams) {
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int s = 0; s < MAX_STREAMS; ++s) {
            if (s < streams) {
              const float m = s_mix[s * streams + t];
              acc.x += m * x[s].x; acc.y += m * x[s].y; acc.z += m * x[s].z; acc.w += m * x[s].w;
            }
          }
          const float ow = s_out[t], iw = s_in[t];
          acc.x += ow * y.x; acc.y += ow * y.y; acc.z += ow * y.z; acc.w += ow * y.w;
          *reinterpret_cast<float4*>(xr + static_cast<size_t>(t) * cols + c) = acc;
          u.x += iw * acc.x; u.y += iw * acc.y; u.z += iw * acc.z; u.w += iw * acc.w;
        }
      }
    } else {
#pragma unroll
      for (int t = 0; t < MAX_STREAMS; ++t) {
        if (t < streams) {
          const float iw = s_in[t];
          u.x += iw * x[t].x; u.y += iw * x[t].y; u.z += iw * x[t].z; u.w += iw * x[t].w;
        }
      }
    }
    keep[it] = u;
    ssq += u.x * u.x + u.y * u.y + u.z * u.z + u.w * u.w;
  }
  if (h == nullptr) return;
  const float tot = block_sum(ssq, red);
  const float inv = 1.0f / sqrtf(tot / static_cast<float>(cols) + eps);
  T* hr = h + r * cols;
#pragma unroll
  for (int it = 0; it < SMV_KEEP; ++it) {
    const int c = (threadIdx.x + it * ROW_THREADS) * 4;
    if (c >= cols) continue;
    const float4 w = *reinterpret_cast<const float4*>(norm_w + c);
    const float4 u = keep[it];
    store4<T>(hr + c, make_float4(u.x * inv * w.x, u.y * inv * w.y, u.z * inv * w.z, u.w * inv * w.w));
  }
}

// out[i] = rms_norm(sum_s in_w[s] x_s of row rows_idx[i]) * norm_w
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
stream_gather_norm_kernel(const float* __restrict__ xs, const int32_t* __restrict__ rows_idx, const float* __restrict__ in_w,
                          const float* __restrict__ norm_w, T* __restrict__ out, int cols, int streams, float eps) {
  __shared__ float red[33];
  const size_t r = rows_idx != nullptr ? static_cast<size_t>(rows_idx[blockIdx.x]) : blockIdx.x;
  const float* xr = xs + r * streams * cols;
  float ssq = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float u = 0.f;
    for (int t = 0; t < streams; ++t) u += (in_w != nullptr ? in_w[t] : 1.f) * xr[static_cast<size_t>(t) * cols + c];
    ssq += u * u;
  }
  const float tot = block_sum(ssq, red);
  const float inv = 1.0f / sqrtf(tot / static_cast<float>(cols) + eps);
  T* o = out + static_cast<size_t>(blockIdx.x) * cols;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float u = 0.f;
    for (int t = 0; t < streams; ++t) u += (in_w != nullptr ? in_w[t] : 1.f) * xr[static_cast<size_t>(t) * cols + c];
    o[c] = from_f<T>(u * inv * norm_w[c]);
  }
}

// ------------------------------------------------------------------ attention step preparation
// One block per token.  q = u[q_off : +H*d] + q_bias, k = u[k_off : +G*d] + k_bias, v = u[v_off : +G*dv] + v_bias, or,
// with v_off < 0, v = k as it stands here (before norm and rotation).  With norm weights, q and k are each divided by
// the root mean square of their WHOLE projection and multiplied by the weight.  With rot_dims > 0, coordinate
// i < rot_dims/2 of every head is paired with i + rot_dims/2 (or, `interleaved`, coordinate 2i with 2i + 1) and the pair
// turned by position * freq[i].  Without caches (a layer that reads another layer's keys and values) only q is made.
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
attn_prep_kernel(const T* __restrict__ u, int64_t ldu, int q_off, int k_off, int v_off, const float* __restrict__ q_bias,
                 const float* __restrict__ k_bias, const float* __restrict__ v_bias, const float* __restrict__ q_norm_w,
                 const float* __restrict__ k_norm_w, const float* __restrict__ freq, int rot_dims,
                 const int32_t* __restrict__ positions, const int32_t* __restrict__ slot_mapping, T* __restrict__ q_out,
                 T* __restrict__ k_cache, T* __restrict__ v_cache, int H, int G, int Gv, int d, int dv, float eps, int interleaved) {
  __shared__ float red[33];
  const size_t t = blockIdx.x;
  const int slot = slot_mapping[t];
  if (slot < 0) return;                                   // padding row (uniform over the block)
  const T* ur = u + t * ldu;
  const int nq = H * d, nk = G * d, nv = Gv * dv;
  const float pos = static_cast<float>(positions[t]);
  // values
  T* vr = v_cache + static_cast<size_t>(slot) * nv;
  for (int c = threadIdx.x; c < nv && v_cache != nullptr; c += blockDim.x) {
    float v;
    if (v_off >= 0) v = to_f(ur[v_off + c]) + (v_bias != nullptr ? v_bias[c] : 0.f);
    else v = to_f(ur[k_off + c]) + (k_bias != nullptr ? k_bias[c] : 0.f);
    vr[c] = from_f<T>(v);
  }
  float inv_q = 1.f, inv_k = 1.f;
  if (q_norm_w != nullptr) {
    float sq = 0.f, sk = 0.f;
    for (int c = threadIdx.x; c < nq; c += blockDim.x) {
      const float v = to_f(ur[q_off + c]) + (q_bias != nullptr ? q_bias[c] : 0.f);
      sq += v * v;
    }
    for (int c = threadIdx.x; c < nk; c += blockDim.x) {
      const float v = to_f(ur[k_off + c]) + (k_bias != nullptr ? k_bias[c] : 0.f);
      sk += v * v;
    }
    inv_q = 1.0f / sqrtf(block_sum(sq, red) / static_cast<float>(nq) + eps);
    inv_k = 1.0f / sqrtf(block_sum(sk, red) / static_cast<float>(nk) + eps);
  }
  const int half = rot_dims / 2;
  // a work item is one coordinate that passes unchanged, or one pair of rotated coordinates (owned by its first half)
  for (int part = 0; part < (k_cache != nullptr ? 2 : 1); ++part) {
    const int n = part == 0 ? nq : nk, off = part == 0 ? q_off : k_off;
    const float* bias = part == 0 ? q_bias : k_bias;
    const float* nw = part == 0 ? q_norm_w : k_norm_w;
    const float inv = part == 0 ? inv_q : inv_k;
    T* dst = part == 0 ? q_out + t * nq : k_cache + static_cast<size_t>(slot) * nk;
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
      const int i = c % d;
      const bool rotated = i < rot_dims;
      if (rotated && (interleaved ? (i & 1) : i >= half)) continue;     // second of a pair: written by its partner
      float a = to_f(ur[off + c]) + (bias != nullptr ? bias[c] : 0.f);
      if (nw != nullptr) a = a * inv * nw[c];
      if (rotated) {
        const int c2 = interleaved ? c + 1 : c + half;
        float b = to_f(ur[off + c2]) + (bias != nullptr ? bias[c2] : 0.f);
        if (nw != nullptr) b = b * inv * nw[c2];
        float sn, cs;
        sincosf(pos * freq[interleaved ? i >> 1 : i], &sn, &cs);
        dst[c] = from_f<T>(a * cs - b * sn);
        dst[c2] = from_f<T>(b * cs + a * sn);
      } else {
        dst[c] = from_f<T>(a);
      }
    }
  }
}

// ------------------------------------------------------------------ short causal convolution + activation
// y[t, c] = act(bias[c] + sum_j w[c, j] * u(position(t) - taps + 1 + j)[c]) over the C columns of u from c_off on.  An
// earlier position comes from this step's rows when it lies in the step's portion, from the sequence's carried state
// (its last taps - 1 rows, oldest first) when it came before, and is zero before the sequence's start.
constexpr int CONV_MAX_TAPS = 8;

template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
short_conv_act_kernel(const T* __restrict__ u, int64_t ldu, const float* __restrict__ w, const float* __restrict__ bias,
                      const T* __restrict__ state, const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ positions,
                      const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_pos0,
                      const int32_t* __restrict__ seq_len, const int32_t* __restrict__ seq_slot, T* __restrict__ out,
                      int64_t ldo, int C, int taps, int act) {
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const size_t t = blockIdx.x;
  if (c >= C) return;
  const int b = tok_seq[t];
  if (seq_len[b] <= 0) return;                            // padding row
  const int p = positions[t], pos0 = seq_pos0[b], start = seq_start[b], R = taps - 1;
  const T* st = state + static_cast<size_t>(seq_slot[b]) * R * C;
  float acc = bias != nullptr ? bias[c] : 0.f;
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS; ++j) {
    if (j < taps) {
      const int pj = p - R + j;
      float v = 0.f;
      if (pj >= pos0) v = to_f(u[static_cast<int64_t>(start + pj - pos0) * ldu + c]);
      else if (pj >= 0) v = to_f(st[static_cast<size_t>(pj - (pos0 - R)) * C + c]);   // entry r holds position pos0 - R + r
      acc += w[c * taps + j] * v;
    }
  }
  if (act == 1) acc = silu_f(acc);
  out[t * ldo + c] = from_f<T>(acc);
}

// The same convolution for TAPS known at compile time: a thread owns VEC = 16 / sizeof(T) consecutive channels and walks
// CONV_RUN consecutive tokens of one sequence with its filters and the last TAPS - 1 rows in registers, so every row is
// read once, as one 16-byte vector (channels, c_off and the row strides multiples of VEC; u, state, out 16-byte aligned).
constexpr int CONV_RUN = 8;

template <typename T> struct RowVec {
  static constexpr int VEC = 16 / static_cast<int>(sizeof(T));
  static __device__ __forceinline__ void load(const T* p, float* f) {
    const uint4 raw = ldg_v4(p);
    if constexpr (VEC == 8) {
      f[0] = bf16lo(raw.x); f[1] = bf16hi(raw.x); f[2] = bf16lo(raw.y); f[3] = bf16hi(raw.y);
      f[4] = bf16lo(raw.z); f[5] = bf16hi(raw.z); f[6] = bf16lo(raw.w); f[7] = bf16hi(raw.w);
    } else {
      f[0] = __uint_as_float(raw.x); f[1] = __uint_as_float(raw.y); f[2] = __uint_as_float(raw.z); f[3] = __uint_as_float(raw.w);
    }
  }
  static __device__ __forceinline__ void store(T* p, const float* f) {
    if constexpr (VEC == 8) stg_v4(p, make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7])));
    else stg_v4(p, make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3])));
  }
};

template <typename T, int TAPS>
__global__ void __launch_bounds__(128)
short_conv_act_run_kernel(const T* __restrict__ u, int64_t ldu, const float* __restrict__ w, const float* __restrict__ bias,
                          const T* __restrict__ state, const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_pos0,
                          const int32_t* __restrict__ seq_len, const int32_t* __restrict__ seq_slot, T* __restrict__ out,
                          int64_t ldo, int C, int act) {
  constexpr int VEC = RowVec<T>::VEC, R = TAPS - 1;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
  const int b = blockIdx.z, t0 = blockIdx.x * CONV_RUN;
  const int len = seq_len[b];
  if (c >= C || t0 >= len) return;
  const int pos0 = seq_pos0[b], start = seq_start[b];
  const T* st = state + static_cast<size_t>(seq_slot[b]) * R * C;
  float wt[TAPS][VEC], bs[VEC], win[TAPS][VEC];            // win[j]: the row TAPS - 1 - j tokens back
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    bs[e] = bias != nullptr ? bias[c + e] : 0.f;
#pragma unroll
    for (int j = 0; j < TAPS; ++j) wt[j][e] = w[(c + e) * TAPS + j];
  }
#pragma unroll
  for (int j = 0; j < R; ++j) {                            // the rows before the run's first token
    const int pj = pos0 + t0 - R + j;
#pragma unroll
    for (int e = 0; e < VEC; ++e) win[j][e] = 0.f;
    if (pj >= pos0) RowVec<T>::load(u + static_cast<int64_t>(start + pj - pos0) * ldu + c, win[j]);
    else if (pj >= 0) RowVec<T>::load(st + static_cast<size_t>(pj - (pos0 - R)) * C + c, win[j]);
  }
#pragma unroll
  for (int i = 0; i < CONV_RUN; ++i) {
    const int t = t0 + i;
    if (t >= len) break;
    RowVec<T>::load(u + static_cast<int64_t>(start + t) * ldu + c, win[R]);
    float acc[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      float a = bs[e];
#pragma unroll
      for (int j = 0; j < TAPS; ++j) a += wt[j][e] * win[j][e];
      acc[e] = act == 1 ? silu_f(a) : a;
    }
    RowVec<T>::store(out + static_cast<int64_t>(start + t) * ldo + c, acc);
#pragma unroll
    for (int j = 0; j < R; ++j)
#pragma unroll
      for (int e = 0; e < VEC; ++e) win[j][e] = win[j + 1][e];
  }
}

// The carried state after the step: entry r holds the row of position end - R + r (end = pos0 + new tokens).  One thread
// per (sequence, column) reads its old entries before it writes any, so the shift is safe in place.
template <typename T>
__global__ void conv_state_advance_kernel(const T* __restrict__ u, int64_t ldu, T* __restrict__ state,
                                          const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_pos0,
                                          const int32_t* __restrict__ seq_len, const int32_t* __restrict__ seq_slot, int C,
                                          int taps) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  if (c >= C) return;
  const int len = seq_len[b];
  if (len <= 0) return;
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
      if (pj >= pos0) v = u[static_cast<int64_t>(start + pj - pos0) * ldu + c];
      else if (pj >= 0 && pj - (pos0 - R) >= 0) v = old[pj - (pos0 - R)];
      st[static_cast<size_t>(r) * C] = v;
    }
  }
}

// ------------------------------------------------------------------ gate + grouped RMS norm on a branch output
// One block per (row, group): the row y [cols] (float) is cut into `groups` equal consecutive parts; each part is divided
// by its own root mean square and multiplied by w[c mod w_len]; the gate act(gate[r, c]) multiplies y before the norm
// (gate_first) or the normed result.  act 0: sigmoid, 1: SiLU.
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
gated_group_norm_kernel(const float* __restrict__ y, const T* __restrict__ gate, int64_t ldg, const float* __restrict__ w,
                        int w_len, int groups, int act, int gate_first, float eps, T* __restrict__ out, int cols) {
  __shared__ float red[33];
  const size_t r = blockIdx.x;
  const int gs = cols / groups, c0 = blockIdx.y * gs;
  const float* yr = y + r * cols + c0;
  const T* gr = gate != nullptr ? gate + r * ldg + c0 : nullptr;
  float ssq = 0.f;
  for (int c = threadIdx.x; c < gs; c += blockDim.x) {
    float v = yr[c];
    if (gr != nullptr && gate_first) {
      const float g = to_f(gr[c]);
      v *= act == 0 ? sigmoid_f(g) : silu_f(g);
    }
    ssq += v * v;
  }
  const float inv = 1.0f / sqrtf(block_sum(ssq, red) / static_cast<float>(gs) + eps);
  T* o = out + r * cols + c0;
  for (int c = threadIdx.x; c < gs; c += blockDim.x) {
    float v = yr[c];
    float g = 1.f;
    if (gr != nullptr) {
      g = to_f(gr[c]);
      g = act == 0 ? sigmoid_f(g) : silu_f(g);
    }
    if (gate_first) v = v * g * inv * w[(c0 + c) % w_len];
    else v = v * inv * w[(c0 + c) % w_len] * g;
    o[c] = from_f<T>(v);
  }
}

// The same for groups of a size that is a multiple of four (y 16-byte aligned rows, gate and out 8- / 16-byte aligned).
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
gated_group_norm_vec4_kernel(const float* __restrict__ y, const T* __restrict__ gate, int64_t ldg, const float* __restrict__ w,
                             int w_len, int groups, int act, int gate_first, float eps, T* __restrict__ out, int cols) {
  __shared__ float red[33];
  const size_t r = blockIdx.x;
  const int gs = cols / groups, c0 = blockIdx.y * gs;
  const float* yr = y + r * cols + c0;
  const T* gr = gate != nullptr ? gate + r * ldg + c0 : nullptr;
  auto gated = [&](int c, float4& v, float4& g) {
    v = *reinterpret_cast<const float4*>(yr + c);
    g = make_float4(1.f, 1.f, 1.f, 1.f);
    if (gr != nullptr) {
      const float4 z = load4<T>(gr + c);
      if (act == 0) g = make_float4(sigmoid_f(z.x), sigmoid_f(z.y), sigmoid_f(z.z), sigmoid_f(z.w));
      else g = make_float4(silu_f(z.x), silu_f(z.y), silu_f(z.z), silu_f(z.w));
    }
    if (gate_first) { v.x *= g.x; v.y *= g.y; v.z *= g.z; v.w *= g.w; }
  };
  // a group of up to GN_KEEP vectors per thread stays in registers between the sum of squares and the scaled write
  constexpr int GN_KEEP = 4;
  const bool keep = gs <= 4 * GN_KEEP * static_cast<int>(blockDim.x);
  float4 kv[GN_KEEP], kg[GN_KEEP];
  float ssq = 0.f;
  if (keep) {
#pragma unroll
    for (int it = 0; it < GN_KEEP; ++it) {
      const int c = (threadIdx.x + it * blockDim.x) * 4;
      kv[it] = make_float4(0.f, 0.f, 0.f, 0.f);
      kg[it] = kv[it];
      if (c < gs) {
        gated(c, kv[it], kg[it]);
        ssq += kv[it].x * kv[it].x + kv[it].y * kv[it].y + kv[it].z * kv[it].z + kv[it].w * kv[it].w;
      }
    }
  } else {
    for (int c = threadIdx.x * 4; c < gs; c += blockDim.x * 4) {
      float4 v, g;
      gated(c, v, g);
      ssq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  }
  const float inv = 1.0f / sqrtf(block_sum(ssq, red) / static_cast<float>(gs) + eps);
  T* o = out + r * cols + c0;
  auto emit = [&](int c, const float4& v, const float4& g) {
    const int wc = (c0 + c) % w_len;                       // w_len is a multiple of four here
    const float4 ww = *reinterpret_cast<const float4*>(w + wc);
    float4 res = make_float4(v.x * inv * ww.x, v.y * inv * ww.y, v.z * inv * ww.z, v.w * inv * ww.w);
    if (!gate_first) { res.x *= g.x; res.y *= g.y; res.z *= g.z; res.w *= g.w; }
    store4<T>(o + c, res);
  };
  if (keep) {
#pragma unroll
    for (int it = 0; it < GN_KEEP; ++it) {
      const int c = (threadIdx.x + it * blockDim.x) * 4;
      if (c < gs) emit(c, kv[it], kg[it]);
    }
  } else {
    for (int c = threadIdx.x * 4; c < gs; c += blockDim.x * 4) {
      float4 v, g;
      gated(c, v, g);
      emit(c, v, g);
    }
  }
}

// Small groups (a head each): one CTA per row, a warp per group in turn, the group's values in registers, no barrier.
constexpr int GNW_KEEP = 4;                                // groups of up to 4 * GNW_KEEP * 32 = 512 values

template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
gated_group_norm_warp_kernel(const float* __restrict__ y, const T* __restrict__ gate, int64_t ldg, const float* __restrict__ w,
                             int w_len, int groups, int act, int gate_first, float eps, T* __restrict__ out, int cols) {
  const size_t r = blockIdx.x;
  const int gs = cols / groups, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int grp = threadIdx.x >> 5; grp < groups; grp += nw) {
    const int c0 = grp * gs;
    const float* yr = y + r * cols + c0;
    const T* gr = gate != nullptr ? gate + r * ldg + c0 : nullptr;
    float4 kv[GNW_KEEP], kg[GNW_KEEP];
    float ssq = 0.f;
#pragma unroll
    for (int it = 0; it < GNW_KEEP; ++it) {
      const int c = (lane + it * 32) * 4;
      kv[it] = make_float4(0.f, 0.f, 0.f, 0.f);
      kg[it] = make_float4(1.f, 1.f, 1.f, 1.f);
      if (c < gs) {
        kv[it] = *reinterpret_cast<const float4*>(yr + c);
        if (gr != nullptr) {
          const float4 z = load4<T>(gr + c);
          if (act == 0) kg[it] = make_float4(sigmoid_f(z.x), sigmoid_f(z.y), sigmoid_f(z.z), sigmoid_f(z.w));
          else kg[it] = make_float4(silu_f(z.x), silu_f(z.y), silu_f(z.z), silu_f(z.w));
        }
        if (gate_first) { kv[it].x *= kg[it].x; kv[it].y *= kg[it].y; kv[it].z *= kg[it].z; kv[it].w *= kg[it].w; }
        ssq += kv[it].x * kv[it].x + kv[it].y * kv[it].y + kv[it].z * kv[it].z + kv[it].w * kv[it].w;
      }
    }
    const float inv = 1.0f / sqrtf(warp_sum(ssq) / static_cast<float>(gs) + eps);
    T* o = out + r * cols + c0;
#pragma unroll
    for (int it = 0; it < GNW_KEEP; ++it) {
      const int c = (lane + it * 32) * 4;
      if (c < gs) {
        const float4 ww = *reinterpret_cast<const float4*>(w + (c0 + c) % w_len);
        float4 res = make_float4(kv[it].x * inv * ww.x, kv[it].y * inv * ww.y, kv[it].z * inv * ww.z, kv[it].w * inv * ww.w);
        if (!gate_first) { res.x *= kg[it].x; res.y *= kg[it].y; res.z *= kg[it].z; res.w *= kg[it].w; }
        store4<T>(o + c, res);
      }
    }
  }
}

}  // namespace row
}  // namespace b2

// =================================================================================================== C ABI
using namespace b2;
using namespace b2::row;

extern "C" int b2tts_embed_bigram_streams(const int32_t* tokens, const int32_t* prev_tokens, const void* embed,
                                          const void* bigram, float* xs, int rows, int cols, int streams, int vocab,
                                          int buckets, int mul_prev, int mul_cur, int dtype, void* stream) {
  B2_REQUIRE(rows >= 0 && cols > 0 && vocab > 0 && streams >= 1 && streams <= MAX_STREAMS, B2TTS_EINVAL,
             "embed_bigram_streams: rows=%d cols=%d streams=%d (at most %d)", rows, cols, streams, MAX_STREAMS);
  B2_REQUIRE(B2_ROW_DTYPE_OK(dtype), B2TTS_EINVAL, "embed_bigram_streams: dtype %d", dtype);
  B2_REQUIRE(!bigram || buckets > 0, B2TTS_EINVAL, "embed_bigram_streams: buckets=%d", buckets);
  if (rows == 0) return B2TTS_OK;
  B2_REQUIRE(tokens && prev_tokens && embed && xs, B2TTS_EINVAL, "embed_bigram_streams: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == B2TTS_DTYPE_BF16)
    embed_bigram_kernel<__nv_bfloat16><<<rows, ROW_THREADS, 0, st>>>(tokens, prev_tokens, static_cast<const __nv_bfloat16*>(embed),
        static_cast<const __nv_bfloat16*>(bigram), xs, cols, streams, vocab, buckets, mul_prev, mul_cur);
  else
    embed_bigram_kernel<float><<<rows, ROW_THREADS, 0, st>>>(tokens, prev_tokens, static_cast<const float*>(embed),
        static_cast<const float*>(bigram), xs, cols, streams, vocab, buckets, mul_prev, mul_cur);
  B2_CHECK_LAUNCH("embed_bigram_streams");
  return B2TTS_OK;
}

extern "C" int b2tts_stream_mix_norm(float* xs, const void* y1, const void* y2, float c1, float c2, const float* mix,
                                     const float* out_w, const float* in_w, const float* norm_w, void* h, int rows, int cols,
                                     int streams, float eps, int dtype, void* stream) {
  B2_REQUIRE(rows >= 0 && cols > 0 && streams >= 1 && streams <= MAX_STREAMS, B2TTS_EINVAL,
             "stream_mix_norm: rows=%d cols=%d streams=%d (at most %d)", rows, cols, streams, MAX_STREAMS);
  B2_REQUIRE(B2_ROW_DTYPE_OK(dtype), B2TTS_EINVAL, "stream_mix_norm: dtype %d", dtype);
  if (rows == 0) return B2TTS_OK;
  B2_REQUIRE(xs && (!y1 || (mix && out_w)) && (y1 || !y2) && (!h || norm_w), B2TTS_EINVAL, "stream_mix_norm: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool vec4 = cols % 4 == 0 && cols <= 4 * SMV_KEEP * ROW_THREADS && aligned16(xs) && aligned16(norm_w) &&
                    (!y1 || aligned16(y1)) && (!y2 || aligned16(y2)) && (!h || aligned16(h));
  if (vec4 && dtype == B2TTS_DTYPE_BF16)
    stream_mix_norm_vec4_kernel<__nv_bfloat16><<<rows, ROW_THREADS, 0, st>>>(xs, static_cast<const __nv_bfloat16*>(y1),
        static_cast<const __nv_bfloat16*>(y2), c1, c2, mix, out_w, in_w, norm_w, static_cast<__nv_bfloat16*>(h), cols, streams, eps);
  else if (vec4)
    stream_mix_norm_vec4_kernel<float><<<rows, ROW_THREADS, 0, st>>>(xs, static_cast<const float*>(y1), static_cast<const float*>(y2),
        c1, c2, mix, out_w, in_w, norm_w, static_cast<float*>(h), cols, streams, eps);
  else if (dtype == B2TTS_DTYPE_BF16)
    stream_mix_norm_kernel<__nv_bfloat16><<<rows, ROW_THREADS, 0, st>>>(xs, static_cast<const __nv_bfloat16*>(y1),
        static_cast<const __nv_bfloat16*>(y2), c1, c2, mix, out_w, in_w, norm_w, static_cast<__nv_bfloat16*>(h), cols, streams, eps);
  else
    stream_mix_norm_kernel<float><<<rows, ROW_THREADS, 0, st>>>(xs, static_cast<const float*>(y1), static_cast<const float*>(y2),
        c1, c2, mix, out_w, in_w, norm_w, static_cast<float*>(h), cols, streams, eps);
  B2_CHECK_LAUNCH("stream_mix_norm");
  return B2TTS_OK;
}

extern "C" int b2tts_stream_gather_norm(const float* xs, const int32_t* rows_idx, const float* in_w, const float* norm_w,
                                        void* out, int rows, int cols, int streams, float eps, int dtype, void* stream) {
  B2_REQUIRE(rows >= 0 && cols > 0 && streams >= 1, B2TTS_EINVAL, "stream_gather_norm: rows=%d cols=%d streams=%d", rows, cols, streams);
  B2_REQUIRE(B2_ROW_DTYPE_OK(dtype), B2TTS_EINVAL, "stream_gather_norm: dtype %d", dtype);
  if (rows == 0) return B2TTS_OK;
  B2_REQUIRE(xs && norm_w && out, B2TTS_EINVAL, "stream_gather_norm: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == B2TTS_DTYPE_BF16)
    stream_gather_norm_kernel<__nv_bfloat16><<<rows, ROW_THREADS, 0, st>>>(xs, rows_idx, in_w, norm_w, static_cast<__nv_bfloat16*>(out), cols, streams, eps);
  else
    stream_gather_norm_kernel<float><<<rows, ROW_THREADS, 0, st>>>(xs, rows_idx, in_w, norm_w, static_cast<float*>(out), cols, streams, eps);
  B2_CHECK_LAUNCH("stream_gather_norm");
  return B2TTS_OK;
}

extern "C" int b2tts_attn_prep(const void* u, int64_t ldu, int q_off, int k_off, int v_off, const float* q_bias,
                               const float* k_bias, const float* v_bias, const float* q_norm_w, const float* k_norm_w,
                               const float* freq, int rot_dims, const int32_t* positions, const int32_t* slot_mapping,
                               void* q_out, void* k_cache, void* v_cache, int n_tokens, int heads, int kv_heads, int dim,
                               int vdim, float eps, int interleaved, int v_heads, int dtype, void* stream) {
  B2_REQUIRE(v_heads > 0 && (v_off >= 0 || v_heads == kv_heads), B2TTS_EINVAL, "attn_prep: %d value heads", v_heads);
  B2_REQUIRE(n_tokens >= 0 && heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0 && q_off >= 0 && k_off >= 0, B2TTS_EINVAL,
             "attn_prep: bad sizes");
  B2_REQUIRE((k_cache == nullptr) == (v_cache == nullptr), B2TTS_EINVAL, "attn_prep: both caches, or neither");
  B2_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dim, B2TTS_EINVAL, "attn_prep: %d rotated of %d coordinates", rot_dims, dim);
  B2_REQUIRE(v_off >= 0 || vdim == dim, B2TTS_EINVAL, "attn_prep: values that are the keys need vdim == dim");
  B2_REQUIRE((q_norm_w == nullptr) == (k_norm_w == nullptr), B2TTS_EINVAL, "attn_prep: norm weights for q and k, or neither");
  B2_REQUIRE(B2_ROW_DTYPE_OK(dtype), B2TTS_EINVAL, "attn_prep: dtype %d", dtype);
  if (n_tokens == 0) return B2TTS_OK;
  B2_REQUIRE(u && positions && slot_mapping && q_out && (rot_dims == 0 || freq), B2TTS_EINVAL, "attn_prep: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == B2TTS_DTYPE_BF16)
    attn_prep_kernel<__nv_bfloat16><<<n_tokens, ROW_THREADS, 0, st>>>(static_cast<const __nv_bfloat16*>(u), ldu, q_off, k_off, v_off,
        q_bias, k_bias, v_bias, q_norm_w, k_norm_w, freq, rot_dims, positions, slot_mapping, static_cast<__nv_bfloat16*>(q_out),
        static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), heads, kv_heads, v_heads, dim, vdim, eps, interleaved);
  else
    attn_prep_kernel<float><<<n_tokens, ROW_THREADS, 0, st>>>(static_cast<const float*>(u), ldu, q_off, k_off, v_off, q_bias, k_bias,
        v_bias, q_norm_w, k_norm_w, freq, rot_dims, positions, slot_mapping, static_cast<float*>(q_out),
        static_cast<float*>(k_cache), static_cast<float*>(v_cache), heads, kv_heads, v_heads, dim, vdim, eps, interleaved);
  B2_CHECK_LAUNCH("attn_prep");
  return B2TTS_OK;
}

template <typename T>
static void launch_conv_act(cudaStream_t st, const void* u, int64_t ldu, int c_off, const float* w, const float* bias, void* state,
                            const int32_t* tok_seq, const int32_t* positions, const int32_t* seq_start, const int32_t* seq_pos0,
                            const int32_t* seq_len, const int32_t* seq_slot, void* out, int64_t ldo, int n_tokens, int n_seqs,
                            int max_new, int C, int taps, int act) {
  const T* uu = static_cast<const T*>(u) + c_off;
  constexpr int VEC = 16 / static_cast<int>(sizeof(T));
  const bool vec = taps >= 2 && taps <= 4 && max_new > 0 && C % VEC == 0 && ldu % VEC == 0 && ldo % VEC == 0 && aligned16(uu) &&
                   aligned16(out) && aligned16(state) && n_seqs <= 65535;
  if (vec) {
    const int threads = std::min(128, (C / VEC + 31) / 32 * 32);
    const dim3 grid((max_new + CONV_RUN - 1) / CONV_RUN, (C / VEC + threads - 1) / threads, n_seqs);
#define CONV_RUN_GO(TP) short_conv_act_run_kernel<T, TP><<<grid, threads, 0, st>>>(uu, ldu, w, bias, static_cast<const T*>(state), seq_start, \
        seq_pos0, seq_len, seq_slot, static_cast<T*>(out), ldo, C, act)
    if (taps == 4) CONV_RUN_GO(4);
    else if (taps == 3) CONV_RUN_GO(3);
    else CONV_RUN_GO(2);
#undef CONV_RUN_GO
  } else {
    short_conv_act_kernel<T><<<dim3(n_tokens, (C + ROW_THREADS - 1) / ROW_THREADS), ROW_THREADS, 0, st>>>(
        uu, ldu, w, bias, static_cast<const T*>(state), tok_seq, positions, seq_start, seq_pos0, seq_len, seq_slot,
        static_cast<T*>(out), ldo, C, taps, act);
  }
  if (taps > 1)
    conv_state_advance_kernel<T><<<dim3((C + 127) / 128, n_seqs), 128, 0, st>>>(uu, ldu, static_cast<T*>(state), seq_start, seq_pos0,
                                                                               seq_len, seq_slot, C, taps);
}

extern "C" int b2tts_short_conv_act(const void* u, int64_t ldu, int c_off, const float* w, const float* bias, void* state,
                                    const int32_t* tok_seq, const int32_t* positions, const int32_t* seq_start,
                                    const int32_t* seq_pos0, const int32_t* seq_len, const int32_t* seq_slot, void* out,
                                    int64_t ldo, int n_tokens, int n_seqs, int max_new, int channels, int taps, int act,
                                    int dtype, void* stream) {
  B2_REQUIRE(n_tokens >= 0 && n_seqs >= 0 && channels > 0 && c_off >= 0, B2TTS_EINVAL, "short_conv_act: bad sizes");
  B2_REQUIRE(taps >= 1 && taps <= CONV_MAX_TAPS, B2TTS_EUNSUPPORTED, "short_conv_act: taps %d not in 1..%d", taps, CONV_MAX_TAPS);
  B2_REQUIRE(act == 0 || act == 1, B2TTS_EINVAL, "short_conv_act: act %d", act);
  B2_REQUIRE(B2_ROW_DTYPE_OK(dtype), B2TTS_EINVAL, "short_conv_act: dtype %d", dtype);
  if (n_tokens == 0 || n_seqs == 0) return B2TTS_OK;
  B2_REQUIRE(u && w && (state || taps == 1) && tok_seq && positions && seq_start && seq_pos0 && seq_len && seq_slot && out,
             B2TTS_EINVAL, "short_conv_act: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == B2TTS_DTYPE_BF16)
    launch_conv_act<__nv_bfloat16>(st, u, ldu, c_off, w, bias, state, tok_seq, positions, seq_start, seq_pos0, seq_len, seq_slot, out,
                                   ldo, n_tokens, n_seqs, max_new, channels, taps, act);
  else
    launch_conv_act<float>(st, u, ldu, c_off, w, bias, state, tok_seq, positions, seq_start, seq_pos0, seq_len, seq_slot, out, ldo,
                           n_tokens, n_seqs, max_new, channels, taps, act);
  B2_CHECK_LAUNCH("short_conv_act");
  return B2TTS_OK;
}

extern "C" int b2tts_gated_group_norm(const float* y, const void* gate, int64_t ldg, const float* w, int w_len, int groups,
                                      int gate_act, int gate_first, float eps, void* out, int rows, int cols, int dtype,
                                      void* stream) {
  B2_REQUIRE(rows >= 0 && cols > 0 && groups > 0 && cols % groups == 0 && w_len > 0, B2TTS_EINVAL,
             "gated_group_norm: rows=%d cols=%d groups=%d", rows, cols, groups);
  B2_REQUIRE(gate_act == 0 || gate_act == 1, B2TTS_EINVAL, "gated_group_norm: gate_act %d", gate_act);
  B2_REQUIRE(B2_ROW_DTYPE_OK(dtype), B2TTS_EINVAL, "gated_group_norm: dtype %d", dtype);
  if (rows == 0) return B2TTS_OK;
  B2_REQUIRE(y && w && out, B2TTS_EINVAL, "gated_group_norm: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int gs = cols / groups;
  const dim3 grid(rows, groups);
  const bool vec4 = gs % 4 == 0 && w_len % 4 == 0 && ldg % 4 == 0 && aligned16(y) && aligned16(w) && aligned16(out) &&
                    (!gate || aligned16(gate));
  if (vec4 && groups > 1 && gs <= 4 * GNW_KEEP * 32) {
    const int threads = 32 * std::min(groups, ROW_THREADS / 32);
    if (dtype == B2TTS_DTYPE_BF16)
      gated_group_norm_warp_kernel<__nv_bfloat16><<<rows, threads, 0, st>>>(y, static_cast<const __nv_bfloat16*>(gate), ldg, w, w_len,
          groups, gate_act, gate_first, eps, static_cast<__nv_bfloat16*>(out), cols);
    else
      gated_group_norm_warp_kernel<float><<<rows, threads, 0, st>>>(y, static_cast<const float*>(gate), ldg, w, w_len, groups, gate_act,
                                                                   gate_first, eps, static_cast<float*>(out), cols);
    B2_CHECK_LAUNCH("gated_group_norm");
    return B2TTS_OK;
  }
  if (vec4) {
    const int threads = std::min(ROW_THREADS, (gs / 4 + 31) / 32 * 32);
    if (dtype == B2TTS_DTYPE_BF16)
      gated_group_norm_vec4_kernel<__nv_bfloat16><<<grid, threads, 0, st>>>(y, static_cast<const __nv_bfloat16*>(gate), ldg, w, w_len,
          groups, gate_act, gate_first, eps, static_cast<__nv_bfloat16*>(out), cols);
    else
      gated_group_norm_vec4_kernel<float><<<grid, threads, 0, st>>>(y, static_cast<const float*>(gate), ldg, w, w_len, groups, gate_act,
                                                                   gate_first, eps, static_cast<float*>(out), cols);
    B2_CHECK_LAUNCH("gated_group_norm");
    return B2TTS_OK;
  }
  const int threads = std::min(ROW_THREADS, (gs + 31) / 32 * 32);
  if (dtype == B2TTS_DTYPE_BF16)
    gated_group_norm_kernel<__nv_bfloat16><<<grid, threads, 0, st>>>(y, static_cast<const __nv_bfloat16*>(gate), ldg, w, w_len, groups,
                                                                    gate_act, gate_first, eps, static_cast<__nv_bfloat16*>(out), cols);
  else
    gated_group_norm_kernel<float><<<grid, threads, 0, st>>>(y, static_cast<const float*>(gate), ldg, w, w_len, groups, gate_act,
                                                            gate_first, eps, static_cast<float*>(out), cols);
  B2_CHECK_LAUNCH("gated_group_norm");
  return B2TTS_OK;
}
