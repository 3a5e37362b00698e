// recurrent.cu - recurrent memories with a matrix state per head, carried from token to token in per-sequence state slots:
//
//   state space      S <- exp(-exp(A) dt) S + dt B x^T                     y = S^T C + D x            (S: state x vdim)
//   matrix memory    S <- a S + b k v^T,  n <- a n + b k                   o = S^T q / (max(|n.q|, exp(-m)) + 1e-6)
//                    with log gates i, f and the running maximum m = max(f + m, i), a = exp(f + m_old - m), b = exp(i - m)
//   delta rule       S <- g S;  u = beta (v - S^T k);  S <- S + k u^T      o = S^T q
//   gated linear     S <- diag(alpha) S + k v^T                            o = S^T q      (a decay per key channel and token)
//
// All three update every value column of S independently.  A column is shared by RS = ceil(key size / 32) lanes of one
// warp, each keeping 32 rows of it in registers for the whole portion; sums over the rows (the read-out, the delta rule's
// S^T k, the unit norms) are butterfly shuffles over those lanes.  The per-token vectors (k, q or B, C) are staged in
// shared memory one element per thread (one barrier per token), their loads run four tokens ahead through registers, and
// the tokens of the portion are walked in order.  What a token contributes besides its vectors - decay, step size, write
// strength - depends on the inputs only and is computed for all tokens at once by a kernel in front.  A decode step is the same kernel with one token.  The state is read from the
// sequence's slot (or starts at zero when the portion starts at position 0: a slot is never cleared between owners) and
// written back at the end.  State, decays, gates, step sizes and unit norms are float whatever the activation type.
//
// The matrix memory's scalar part (gates, running maximum, the normaliser vector n and the denominator) runs first in a
// kernel of its own, one CTA per (sequence, head), and hands (a, b, denominator) per token to the column kernel, so that
// CTAs which share a head share no state.
#include <algorithm>

#include "row_ops.cuh"

namespace b2 {
namespace row {

constexpr int SCAN_ROWS = 32;             // state rows a thread keeps in registers
constexpr int SCAN_COLS = 32;             // value columns per CTA
constexpr int SCAN_PER = 8;               // key elements per lane of the one-warp gate kernel: key sizes up to 256
constexpr int SCAN_DEPTH = 4;             // tokens whose inputs are in flight in registers

enum { SCAN_LINEAR = 0, SCAN_DELTA = 1, SCAN_GATED = 2 };

struct ScanArgs {
  const void* k; int64_t ldk;             // key-like vectors: (row, group g, i) at k[row * ldk + g * d + i]
  const void* q; int64_t ldq;             // query-like vectors, same layout
  const void* v; int64_t ldv;             // values: (row, head h, c) at v[row * ldv + h * dv + c]
  const float* coef;                      // [rows, H, 3] per-token scalars, see scan_kernel (SCAN_GATED: unused)
  const float* decay; int64_t ldd;        // SCAN_GATED: per key channel, (row, head h, i) at decay[row * ldd + h * d + i]
  const float* skip;                      // [H] or null: out += skip[h] * value
  float* state;                           // [slots, H, d, dv]
  float* out;                             // [rows, H * dv]
  const int32_t* seq_start; const int32_t* seq_pos0; const int32_t* seq_len; const int32_t* seq_slot;
  int H, G, d, dv;
  float qscale;
  int divide;                             // linear: out = S^T q * qscale / coef[2] instead of S^T q * qscale
};

// sum over the RS lanes that share a column (lane = slice * (32 / RS) + column): every one of them gets the total
template <int RS>
__device__ __forceinline__ float slice_sum(float v) {
#pragma unroll
  for (int o = 16; o >= 32 / RS; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Per-token scalars c = coef[row, h, :], computed beforehand (they depend on the inputs only, not on the state):
//   SCAN_LINEAR   S <- c0 S + k (c1 v)^T;                               out = S^T q * qscale [/ c2] [+ skip v]
//   SCAN_DELTA    S <- c0 S; u = c1 (v - S^T k^); S <- S + k^ u^T;      out = S^T q^ * qscale      (k^, q^: unit vectors)
//   SCAN_GATED    S[i, :] <- decay[i] S[i, :] + k[i] v^T;               out = S^T q * qscale       (decay staged like k and q)
// RS = threads per value column = ceil(d / 32) rounded up to a power of two; the CTA is RS warps and owns 32 columns.  A
// warp holds 32 / RS columns; thread (slice, column) keeps rows slice * 32 .. + 31 of its column in registers for the
// whole portion.  Thread i stages element i of a token's k and q (zero beyond d) in shared memory, SCAN_DEPTH tokens at a
// time; the loads run a group of tokens ahead through registers, so a token waits for its own arithmetic only.
template <typename T, int KIND, int RS>
__global__ void __launch_bounds__(32 * RS)
scan_kernel(const ScanArgs a) {
  constexpr int CW = 32 / RS;                              // columns per warp
  constexpr int DP = RS * SCAN_ROWS;                       // padded key size = threads
  constexpr int NV = KIND == SCAN_GATED ? 3 : 2;
  __shared__ __align__(16) float vec[2][SCAN_DEPTH][NV][DP];  // [buffer][token of the group][k | q | decay][row]
  const int b = blockIdx.z, h = blockIdx.y;
  const int len = a.seq_len[b];
  if (len <= 0) return;
  const int d = a.d, dv = a.dv, H = a.H;
  const int g = h / (H / a.G);
  const int start = a.seq_start[b], pos0 = a.seq_pos0[b];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int slice = lane / CW;
  const int col = blockIdx.x * SCAN_COLS + warp * CW + (lane % CW);
  const bool live = col < dv, mine = tid < d;
  const int r0 = slice * SCAN_ROWS;
  float S[SCAN_ROWS];
  float* Sg = a.state + ((static_cast<size_t>(a.seq_slot[b]) * H + h) * d) * dv + col;
#pragma unroll
  for (int x = 0; x < SCAN_ROWS; ++x) {
    const int i = r0 + x;
    S[x] = (live && pos0 > 0 && i < d) ? Sg[static_cast<size_t>(i) * dv] : 0.f;
  }
  const T* kp = static_cast<const T*>(a.k) + static_cast<size_t>(start) * a.ldk + g * d + tid;
  const T* qp = static_cast<const T*>(a.q) + static_cast<size_t>(start) * a.ldq + g * d + tid;
  const T* vp = static_cast<const T*>(a.v) + static_cast<size_t>(start) * a.ldv + h * dv + col;
  const float* cp = a.coef + (static_cast<size_t>(start) * H + h) * 3;
  const float* dp = KIND == SCAN_GATED ? a.decay + static_cast<size_t>(start) * a.ldd + h * d + tid : nullptr;
  float* op = a.out + static_cast<size_t>(start) * H * dv + h * dv + col;
  const float skip = a.skip != nullptr ? a.skip[h] : 0.f;

  // the loaded values stay as they came (type T) until their token is staged: converting them at once would make the
  // thread wait for the load, four tokens early
  T rk[SCAN_DEPTH], rq[SCAN_DEPTH], rv[SCAN_DEPTH];
  float rc[SCAN_DEPTH][3], rd[SCAN_DEPTH];
  auto fetch = [&](int u, int t) {                         // token t's inputs into register stage u
    rk[u] = rq[u] = rv[u] = from_f<T>(0.f);
    rc[u][0] = rc[u][1] = 0.f; rc[u][2] = 1.f;
    rd[u] = 0.f;
    if (t < len) {
      if (mine) { rk[u] = kp[static_cast<size_t>(t) * a.ldk]; rq[u] = qp[static_cast<size_t>(t) * a.ldq]; }
      if (live) rv[u] = vp[static_cast<size_t>(t) * a.ldv];
      if constexpr (KIND == SCAN_GATED) {
        if (mine) rd[u] = dp[static_cast<size_t>(t) * a.ldd];
      } else {
        const float* c = cp + static_cast<size_t>(t) * H * 3;
        rc[u][0] = c[0]; rc[u][1] = c[1]; rc[u][2] = c[2];
      }
    }
  };
#pragma unroll
  for (int u = 0; u < SCAN_DEPTH; ++u) fetch(u, u);
  // tokens go in groups of SCAN_DEPTH: the group's vectors are staged at once (one barrier per group, two buffers), the
  // next group's loads are issued, then the group's tokens are walked without a barrier between them
  for (int t0 = 0, grp = 0; t0 < len; t0 += SCAN_DEPTH, grp ^= 1) {
    float vals[SCAN_DEPTH], cs[SCAN_DEPTH][3];
#pragma unroll
    for (int u = 0; u < SCAN_DEPTH; ++u) {
      vec[grp][u][0][tid] = to_f(rk[u]);
      vec[grp][u][1][tid] = to_f(rq[u]);
      if constexpr (KIND == SCAN_GATED) vec[grp][u][2][tid] = rd[u];
      vals[u] = to_f(rv[u]);
      cs[u][0] = rc[u][0]; cs[u][1] = rc[u][1]; cs[u][2] = rc[u][2];
    }
#pragma unroll
    for (int u = 0; u < SCAN_DEPTH; ++u) fetch(u, t0 + SCAN_DEPTH + u);
    __syncthreads();                                       // group staged; the other buffer's readers finished a group ago
#pragma unroll
    for (int u = 0; u < SCAN_DEPTH; ++u) {
      const int t = t0 + u;
      if (t >= len) break;                                 // uniform over the CTA
      const float* ks = vec[grp][u][0];
      const float* qs = vec[grp][u][1];
      const float val = vals[u], c0 = cs[u][0], c1 = cs[u][1], c2 = cs[u][2];
      float kr[SCAN_ROWS];
#pragma unroll
      for (int x = 0; x < SCAN_ROWS; x += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(ks + r0 + x);
        kr[x] = k4.x; kr[x + 1] = k4.y; kr[x + 2] = k4.z; kr[x + 3] = k4.w;
      }
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f, o;
      if constexpr (KIND == SCAN_LINEAR) {
        const float w = c1 * val;
#pragma unroll
        for (int x = 0; x < SCAN_ROWS; x += 4) {
          const float4 q4 = *reinterpret_cast<const float4*>(qs + r0 + x);
          S[x] = c0 * S[x] + kr[x] * w;             o0 += S[x] * q4.x;
          S[x + 1] = c0 * S[x + 1] + kr[x + 1] * w; o1 += S[x + 1] * q4.y;
          S[x + 2] = c0 * S[x + 2] + kr[x + 2] * w; o2 += S[x + 2] * q4.z;
          S[x + 3] = c0 * S[x + 3] + kr[x + 3] * w; o3 += S[x + 3] * q4.w;
        }
        o = slice_sum<RS>((o0 + o1) + (o2 + o3)) * a.qscale;
        if (a.divide) o /= c2;
        o += skip * val;
      } else if constexpr (KIND == SCAN_GATED) {
        const float* as = vec[grp][u][2];
#pragma unroll
        for (int x = 0; x < SCAN_ROWS; x += 4) {
          const float4 q4 = *reinterpret_cast<const float4*>(qs + r0 + x);
          const float4 a4 = *reinterpret_cast<const float4*>(as + r0 + x);
          S[x] = a4.x * S[x] + kr[x] * val;             o0 += S[x] * q4.x;
          S[x + 1] = a4.y * S[x + 1] + kr[x + 1] * val; o1 += S[x + 1] * q4.y;
          S[x + 2] = a4.z * S[x + 2] + kr[x + 2] * val; o2 += S[x + 2] * q4.z;
          S[x + 3] = a4.w * S[x + 3] + kr[x + 3] * val; o3 += S[x + 3] * q4.w;
        }
        o = slice_sum<RS>((o0 + o1) + (o2 + o3)) * a.qscale;
        (void)c0; (void)c1; (void)c2;
      } else {
        // unit vectors: every thread sums the squares of its slice, the slices of a column add up to the whole vector
        float ssk = 0.f, ssq = 0.f, kv0 = 0.f, kv1 = 0.f;
#pragma unroll
        for (int x = 0; x < SCAN_ROWS; x += 2) {
          ssk += kr[x] * kr[x] + kr[x + 1] * kr[x + 1];
          S[x] *= c0;     kv0 += S[x] * kr[x];
          S[x + 1] *= c0; kv1 += S[x + 1] * kr[x + 1];
        }
        const float kn = 1.0f / sqrtf(slice_sum<RS>(ssk) + 1e-6f);
        const float kv = slice_sum<RS>(kv0 + kv1) * kn;
        const float w = c1 * (val - kv) * kn;              // k^ u^T = k (kn u)^T
#pragma unroll
        for (int x = 0; x < SCAN_ROWS; x += 4) {
          const float4 q4 = *reinterpret_cast<const float4*>(qs + r0 + x);
          S[x] += kr[x] * w;         o0 += S[x] * q4.x;     ssq += q4.x * q4.x;
          S[x + 1] += kr[x + 1] * w; o1 += S[x + 1] * q4.y; ssq += q4.y * q4.y;
          S[x + 2] += kr[x + 2] * w; o2 += S[x + 2] * q4.z; ssq += q4.z * q4.z;
          S[x + 3] += kr[x + 3] * w; o3 += S[x + 3] * q4.w; ssq += q4.w * q4.w;
        }
        o = slice_sum<RS>((o0 + o1) + (o2 + o3)) * (a.qscale / sqrtf(slice_sum<RS>(ssq) + 1e-6f));
      }
      if (live && slice == 0) op[static_cast<size_t>(t) * H * dv] = o;
    }
  }
  if (live) {
#pragma unroll
    for (int x = 0; x < SCAN_ROWS; ++x) {
      const int i = r0 + x;
      if (i < d) Sg[static_cast<size_t>(i) * dv] = S[x];
    }
  }
}

// ------------------------------------------------------------------ per-token scalars of the state space and the delta rule
// kind 0: dt = softplus(s1 + f1[h]); coef = (exp(-exp(f2[h]) dt), dt, 1)                       (f1 = dt_bias, f2 = A_log)
// kind 1: coef = (exp(-exp(f1[h]) softplus(s2 + f2[h])), sigmoid(s1), 1)                      (f1 = A_log, f2 = dt_bias)
// kind 2: coef = (log input gate, log forget gate, 1) of the matrix memory                   (f1, f2 = the gates' biases)
template <typename T>
__global__ void scan_coef_kernel(const T* __restrict__ s1, const T* __restrict__ s2, int64_t lds, const float* __restrict__ f1,
                                 const float* __restrict__ f2, float* __restrict__ coef, int n_tokens, int H, int kind, float cap) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_tokens * H) return;
  const size_t t = idx / H;
  const int h = idx % H;
  float c0, c1;
  if (kind == 2) {                                       // log gates: cap tanh((s1 + f1) / cap), logsigmoid(cap tanh((s2 + f2) / cap))
    c0 = cap * tanhf((to_f(s1[t * lds + h]) + f1[h]) / cap);
    c1 = logsigmoid_f(cap * tanhf((to_f(s2[t * lds + h]) + f2[h]) / cap));
  } else if (kind == 0) {
    const float dt = softplus_f(to_f(s1[t * lds + h]) + f1[h]);
    c0 = expf(-expf(f2[h]) * dt);
    c1 = dt;
  } else {
    c0 = expf(-expf(f1[h]) * softplus_f(to_f(s2[t * lds + h]) + f2[h]));
    c1 = sigmoid_f(to_f(s1[t * lds + h]));
  }
  float* c = coef + static_cast<size_t>(idx) * 3;
  c[0] = c0; c[1] = c1; c[2] = 1.f;
}

// ------------------------------------------------------------------ scalar part of the matrix memory
// One warp per (sequence, head).  The log gates i = cap tanh((ig + bi) / cap), f = logsigmoid(cap tanh((fg + bf) / cap)) of
// all tokens come from the kernel in front (they do not depend on the state); here, token by token:
// m' = max(f + m, i), a = exp(f + m - m'), b = exp(i - m'); n <- a n + b k; den = max(|n . q * qscale|, exp(-m')) + 1e-6.
// state_nm [slots, H, d + 1]: n, then m (m starts at 0).  The next token's inputs are fetched while this one is computed.
template <typename T>
__global__ void __launch_bounds__(32)
matrix_memory_gates_kernel(const T* __restrict__ k, const T* __restrict__ q, int64_t ldu, float qscale, float* __restrict__ state_nm,
                           float* __restrict__ gates, const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_pos0,
                           const int32_t* __restrict__ seq_len, const int32_t* __restrict__ seq_slot, int H, int d) {
  const int b = blockIdx.y, h = blockIdx.x;
  const int len = seq_len[b];
  if (len <= 0) return;
  const int start = seq_start[b], pos0 = seq_pos0[b], lane = threadIdx.x;
  float* nm = state_nm + (static_cast<size_t>(seq_slot[b]) * H + h) * (d + 1);
  float n[SCAN_PER];
  T rk[SCAN_PER], rq[SCAN_PER];                            // the next token's inputs, converted only when they are used
  float ri = 0.f, rf = 0.f;
#pragma unroll
  for (int x = 0; x < SCAN_PER; ++x) {
    const int i = lane + x * 32;
    n[x] = (i < d && pos0 > 0) ? nm[i] : 0.f;
  }
  float m = pos0 > 0 ? nm[d] : 0.f;
  auto fetch = [&](int t) {
    const size_t r = static_cast<size_t>(start + t);
#pragma unroll
    for (int x = 0; x < SCAN_PER; ++x) {
      const int i = lane + x * 32;
      rk[x] = rq[x] = from_f<T>(0.f);
      if (i < d) { rk[x] = k[r * ldu + h * d + i]; rq[x] = q[r * ldu + h * d + i]; }
    }
    const float* gp = gates + (r * H + h) * 3;             // the log gates, left there by the kernel in front
    ri = gp[0];
    rf = gp[1];
  };
  fetch(0);
  for (int t = 0; t < len; ++t) {
    const float li = ri, lf = rf;
    const float m_new = fmaxf(lf + m, li);
    const float ca = expf(lf + m - m_new), cb = expf(li - m_new);
    m = m_new;
    float nq = 0.f;
#pragma unroll
    for (int x = 0; x < SCAN_PER; ++x) {
      n[x] = ca * n[x] + cb * to_f(rk[x]);
      nq += n[x] * (to_f(rq[x]) * qscale);
    }
    if (t + 1 < len) fetch(t + 1);
    nq = warp_sum(nq);
    if (lane == 0) {
      float* gp = gates + (static_cast<size_t>(start + t) * H + h) * 3;
      gp[0] = ca; gp[1] = cb; gp[2] = fmaxf(fabsf(nq), expf(-m)) + 1e-6f;
    }
  }
#pragma unroll
  for (int x = 0; x < SCAN_PER; ++x) {
    const int i = lane + x * 32;
    if (i < d) nm[i] = n[x];
  }
  if (lane == 0) nm[d] = m;
}

// decay of the gated linear recurrence: alpha = sigmoid(z + bias)^(1 / tau) = exp(logsigmoid(z + bias) / tau), in float
template <typename T>
__global__ void gated_decay_kernel(const T* __restrict__ z, int64_t ldz, const float* __restrict__ bias, float inv_tau,
                                   float* __restrict__ decay, int n_tokens, int cols) {
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<size_t>(n_tokens) * cols) return;
  const size_t t = idx / cols;
  const int c = static_cast<int>(idx % cols);
  decay[idx] = expf(logsigmoid_f(to_f(z[t * ldz + c]) + (bias != nullptr ? bias[c] : 0.f)) * inv_tau);
}

template <typename T, int KIND, int RS>
static void launch_scan_rs(const ScanArgs& a, int n_seqs, cudaStream_t st) {
  const dim3 grid((a.dv + SCAN_COLS - 1) / SCAN_COLS, a.H, n_seqs);
  scan_kernel<T, KIND, RS><<<grid, 32 * RS, 0, st>>>(a);
}

template <typename T, int KIND>
static int launch_scan(const ScanArgs& a, int n_seqs, cudaStream_t st, const char* what) {
  B2_REQUIRE(a.d <= 8 * SCAN_ROWS, B2TTS_EUNSUPPORTED, "%s: key size %d above %d", what, a.d, 8 * SCAN_ROWS);
  if (a.d <= 32) launch_scan_rs<T, KIND, 1>(a, n_seqs, st);
  else if (a.d <= 64) launch_scan_rs<T, KIND, 2>(a, n_seqs, st);
  else if (a.d <= 128) launch_scan_rs<T, KIND, 4>(a, n_seqs, st);
  else launch_scan_rs<T, KIND, 8>(a, n_seqs, st);
  return B2TTS_OK;
}

template <typename T>
static void launch_coef(const void* s1, const void* s2, int64_t lds, const float* f1, const float* f2, float* coef, int n_tokens, int H,
                        int kind, cudaStream_t st, float cap = 1.f) {
  const int total = n_tokens * H;
  scan_coef_kernel<T><<<(total + 255) / 256, 256, 0, st>>>(static_cast<const T*>(s1), static_cast<const T*>(s2), lds, f1, f2, coef,
                                                          n_tokens, H, kind, cap);
}

}  // namespace row
}  // namespace b2

using namespace b2;
using namespace b2::row;

#define SCAN_COMMON_CHECKS(name)                                                                                        \
  B2_REQUIRE(n_seqs >= 0 && heads > 0 && dim > 0 && vdim > 0, B2TTS_EINVAL, name ": bad sizes");                        \
  B2_REQUIRE(B2_ROW_DTYPE_OK(dtype), B2TTS_EINVAL, name ": dtype %d", dtype);                                           \
  B2_REQUIRE(heads <= 65535 && n_seqs <= 65535, B2TTS_EUNSUPPORTED, name ": %d heads, %d sequences", heads, n_seqs);    \
  if (n_seqs == 0) return B2TTS_OK;                                                                                     \
  B2_REQUIRE(state && out && seq_start && seq_pos0 && seq_len && seq_slot, B2TTS_EINVAL, name ": null pointer")

extern "C" int b2tts_ssm_scan(const void* xbc, int64_t ldx, const void* dt, int64_t lddt, const float* dt_bias,
                              const float* a_log, const float* d_skip, float* state, float* coef, float* out, const int32_t* seq_start,
                              const int32_t* seq_pos0, const int32_t* seq_len, const int32_t* seq_slot, int n_tokens, int n_seqs,
                              int heads, int groups, int vdim, int dim, int dtype, void* stream) {
  SCAN_COMMON_CHECKS("ssm_scan");
  B2_REQUIRE(groups > 0 && heads % groups == 0 && n_tokens >= 0, B2TTS_EINVAL, "ssm_scan: %d heads over %d groups", heads, groups);
  B2_REQUIRE(xbc && dt && dt_bias && a_log && d_skip && coef, B2TTS_EINVAL, "ssm_scan: null pointer");
  if (n_tokens == 0) return B2TTS_OK;
  const size_t el = dtype == B2TTS_DTYPE_BF16 ? 2 : 4;
  const int inner = heads * vdim;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == B2TTS_DTYPE_BF16) launch_coef<__nv_bfloat16>(dt, nullptr, lddt, dt_bias, a_log, coef, n_tokens, heads, 0, st);
  else launch_coef<float>(dt, nullptr, lddt, dt_bias, a_log, coef, n_tokens, heads, 0, st);
  B2_CHECK_LAUNCH("ssm_scan (scalars)");
  ScanArgs a{};
  const char* base = static_cast<const char*>(xbc);
  a.v = base; a.ldv = ldx;
  a.k = base + static_cast<size_t>(inner) * el; a.ldk = ldx;
  a.q = base + (static_cast<size_t>(inner) + static_cast<size_t>(groups) * dim) * el; a.ldq = ldx;
  a.coef = coef; a.skip = d_skip;
  a.state = state; a.out = out;
  a.seq_start = seq_start; a.seq_pos0 = seq_pos0; a.seq_len = seq_len; a.seq_slot = seq_slot;
  a.H = heads; a.G = groups; a.d = dim; a.dv = vdim; a.qscale = 1.f; a.divide = 0;
  const int rc = dtype == B2TTS_DTYPE_BF16 ? launch_scan<__nv_bfloat16, SCAN_LINEAR>(a, n_seqs, st, "ssm_scan")
                                           : launch_scan<float, SCAN_LINEAR>(a, n_seqs, st, "ssm_scan");
  if (rc != B2TTS_OK) return rc;
  B2_CHECK_LAUNCH("ssm_scan");
  return B2TTS_OK;
}

extern "C" int b2tts_delta_rule_scan(const void* qkv, int64_t ldq, const void* beta, const void* a_in, int64_t ldu,
                                     const float* a_log, const float* dt_bias, float* state, float* coef, float* out,
                                     const int32_t* seq_start, const int32_t* seq_pos0, const int32_t* seq_len,
                                     const int32_t* seq_slot, int n_tokens, int n_seqs, int heads, int kv_heads, int dim, int vdim,
                                     int dtype, void* stream) {
  SCAN_COMMON_CHECKS("delta_rule_scan");
  B2_REQUIRE(kv_heads > 0 && heads % kv_heads == 0 && n_tokens >= 0, B2TTS_EINVAL, "delta_rule_scan: %d heads over %d key heads", heads, kv_heads);
  B2_REQUIRE(qkv && beta && a_in && a_log && dt_bias && coef, B2TTS_EINVAL, "delta_rule_scan: null pointer");
  if (n_tokens == 0) return B2TTS_OK;
  const size_t el = dtype == B2TTS_DTYPE_BF16 ? 2 : 4;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == B2TTS_DTYPE_BF16) launch_coef<__nv_bfloat16>(beta, a_in, ldu, a_log, dt_bias, coef, n_tokens, heads, 1, st);
  else launch_coef<float>(beta, a_in, ldu, a_log, dt_bias, coef, n_tokens, heads, 1, st);
  B2_CHECK_LAUNCH("delta_rule_scan (scalars)");
  ScanArgs a{};
  const char* base = static_cast<const char*>(qkv);
  const size_t gd = static_cast<size_t>(kv_heads) * dim;
  a.q = base; a.ldq = ldq;
  a.k = base + gd * el; a.ldk = ldq;
  a.v = base + 2 * gd * el; a.ldv = ldq;
  a.coef = coef;
  a.state = state; a.out = out;
  a.seq_start = seq_start; a.seq_pos0 = seq_pos0; a.seq_len = seq_len; a.seq_slot = seq_slot;
  a.H = heads; a.G = kv_heads; a.d = dim; a.dv = vdim; a.qscale = 1.0f / sqrtf(static_cast<float>(dim)); a.divide = 0;
  const int rc = dtype == B2TTS_DTYPE_BF16 ? launch_scan<__nv_bfloat16, SCAN_DELTA>(a, n_seqs, st, "delta_rule_scan")
                                           : launch_scan<float, SCAN_DELTA>(a, n_seqs, st, "delta_rule_scan");
  if (rc != B2TTS_OK) return rc;
  B2_CHECK_LAUNCH("delta_rule_scan");
  return B2TTS_OK;
}

extern "C" int b2tts_matrix_memory_scan(const void* q, const void* k, const void* v, const void* ig, const void* fg, int64_t ldu,
                                        const float* i_bias, const float* f_bias, float cap, float* state, float* state_nm,
                                        float* gates, float* out, const int32_t* seq_start, const int32_t* seq_pos0,
                                        const int32_t* seq_len, const int32_t* seq_slot, int n_tokens, int n_seqs, int heads,
                                        int dim, int vdim, int dtype, void* stream) {
  SCAN_COMMON_CHECKS("matrix_memory_scan");
  if (n_tokens <= 0) return B2TTS_OK;
  B2_REQUIRE(q && k && v && ig && fg && i_bias && f_bias && state_nm && gates && cap > 0.f, B2TTS_EINVAL,
             "matrix_memory_scan: null pointer or cap <= 0");
  B2_REQUIRE(dim <= SCAN_PER * 32, B2TTS_EUNSUPPORTED, "matrix_memory_scan: key size %d above %d", dim, SCAN_PER * 32);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const float qscale = 1.0f / sqrtf(static_cast<float>(dim));
  const dim3 ggrid(heads, n_seqs);
  const int gthreads = 32;
  if (dtype == B2TTS_DTYPE_BF16) {
    launch_coef<__nv_bfloat16>(ig, fg, ldu, i_bias, f_bias, gates, n_tokens, heads, 2, st, cap);
    matrix_memory_gates_kernel<__nv_bfloat16><<<ggrid, gthreads, 0, st>>>(static_cast<const __nv_bfloat16*>(k),
        static_cast<const __nv_bfloat16*>(q), ldu, qscale, state_nm, gates, seq_start, seq_pos0, seq_len, seq_slot, heads, dim);
  } else {
    launch_coef<float>(ig, fg, ldu, i_bias, f_bias, gates, n_tokens, heads, 2, st, cap);
    matrix_memory_gates_kernel<float><<<ggrid, gthreads, 0, st>>>(static_cast<const float*>(k), static_cast<const float*>(q), ldu, qscale,
                                                                 state_nm, gates, seq_start, seq_pos0, seq_len, seq_slot, heads, dim);
  }
  count_launch();
  B2_CHECK_LAUNCH("matrix_memory_gates");
  ScanArgs a{};
  a.q = q; a.ldq = ldu; a.k = k; a.ldk = ldu; a.v = v; a.ldv = ldu;
  a.coef = gates; a.divide = 1;
  a.state = state; a.out = out;
  a.seq_start = seq_start; a.seq_pos0 = seq_pos0; a.seq_len = seq_len; a.seq_slot = seq_slot;
  a.H = heads; a.G = heads; a.d = dim; a.dv = vdim; a.qscale = qscale;
  const int rc = dtype == B2TTS_DTYPE_BF16 ? launch_scan<__nv_bfloat16, SCAN_LINEAR>(a, n_seqs, st, "matrix_memory_scan")
                                           : launch_scan<float, SCAN_LINEAR>(a, n_seqs, st, "matrix_memory_scan");
  if (rc != B2TTS_OK) return rc;
  B2_CHECK_LAUNCH("matrix_memory_scan");
  return B2TTS_OK;
}

extern "C" int b2tts_gated_linear_scan(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv, const void* z,
                                       int64_t ldz, const float* z_bias, float tau, float* decay, float* state, float* out,
                                       const int32_t* seq_start, const int32_t* seq_pos0, const int32_t* seq_len,
                                       const int32_t* seq_slot, int n_tokens, int n_seqs, int heads, int dim, int vdim, int dtype,
                                       void* stream) {
  SCAN_COMMON_CHECKS("gated_linear_scan");
  if (n_tokens <= 0) return B2TTS_OK;
  B2_REQUIRE(q && k && v && z && decay && tau > 0.f, B2TTS_EINVAL, "gated_linear_scan: null pointer or tau <= 0");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int cols = heads * dim;
  const size_t total = static_cast<size_t>(n_tokens) * cols;
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
  if (dtype == B2TTS_DTYPE_BF16)
    gated_decay_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(z), ldz, z_bias, 1.0f / tau, decay, n_tokens, cols);
  else
    gated_decay_kernel<float><<<blocks, 256, 0, st>>>(static_cast<const float*>(z), ldz, z_bias, 1.0f / tau, decay, n_tokens, cols);
  B2_CHECK_LAUNCH("gated_linear_scan (decays)");
  ScanArgs a{};
  a.q = q; a.ldq = ldq; a.k = k; a.ldk = ldk; a.v = v; a.ldv = ldv;
  a.decay = decay; a.ldd = cols;
  a.state = state; a.out = out;
  a.seq_start = seq_start; a.seq_pos0 = seq_pos0; a.seq_len = seq_len; a.seq_slot = seq_slot;
  a.H = heads; a.G = heads; a.d = dim; a.dv = vdim; a.qscale = 1.0f / sqrtf(static_cast<float>(dim)); a.divide = 0;
  const int rc = dtype == B2TTS_DTYPE_BF16 ? launch_scan<__nv_bfloat16, SCAN_GATED>(a, n_seqs, st, "gated_linear_scan")
                                           : launch_scan<float, SCAN_GATED>(a, n_seqs, st, "gated_linear_scan");
  if (rc != B2TTS_OK) return rc;
  B2_CHECK_LAUNCH("gated_linear_scan");
  return B2TTS_OK;
}
