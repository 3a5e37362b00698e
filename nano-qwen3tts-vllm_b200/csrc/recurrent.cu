// recurrent.cu - recurrent memories with a matrix state per head, carried from token to token in per-sequence state slots:
//
//   state space      S <- exp(-exp(A) dt) S + dt B x^T                     y = S^T C + D x            (S: state x vdim)
//   matrix memory    S <- a S + b k v^T,  n <- a n + b k                   o = S^T q / (max(|n.q|, exp(-m)) + 1e-6)
//                    with log gates i, f and the running maximum m = max(f + m, i), a = exp(f + m_old - m), b = exp(i - m)
//   delta rule       S <- g S;  u = beta (v - S^T k);  S <- S + k u^T      o = S^T q
//
// All three update every value column of S independently, so one CTA owns up to 128 columns of one (sequence, head): the
// columns' state lives in shared memory for the whole portion (column-major, one thread per column, conflict-free), the
// per-token vectors (k, q or B, C) are staged in shared memory by all threads one token ahead of their use, and the
// tokens of the portion are walked in order.  A decode step is the same kernel with one token.  The state is read from the
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

constexpr int SCAN_MAX_COLS = 128;
constexpr int SCAN_PER = 8;               // vector elements a thread stages per token: key sizes up to 8 * blockDim

enum { SCAN_SSM = 0, SCAN_MATRIX = 1, SCAN_DELTA = 2 };

struct ScanArgs {
  const void* k; int64_t ldk;             // key-like vectors: (row, group g, i) at k[row * ldk + g * d + i]
  const void* q; int64_t ldq;             // query-like vectors, same layout
  const void* v; int64_t ldv;             // values: (row, head h, c) at v[row * ldv + h * dv + c]
  const void* s1; const void* s2; int64_t lds;   // per-head pre-activations: (row, h) at s[row * lds + h]
  const float* f1; const float* f2; const float* f3;   // per-head constants
  const float* gates;                     // matrix memory: [rows, H, 3] = (a, b, denominator)
  float* state;                           // [slots, H, d, dv]
  float* out;                             // [rows, H * dv]
  const int32_t* seq_start; const int32_t* seq_pos0; const int32_t* seq_len; const int32_t* seq_slot;
  int H, G, d, dv;
  float qscale;
};

template <typename T, int KIND>
__global__ void __launch_bounds__(SCAN_MAX_COLS)
scan_kernel(const ScanArgs a) {
  extern __shared__ float smem[];
  __shared__ float red[33];
  const int b = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * SCAN_MAX_COLS;
  const int len = a.seq_len[b];
  if (len <= 0) return;
  const int d = a.d, dv = a.dv, H = a.H;
  const int cols = min(SCAN_MAX_COLS, dv - c0);
  const int g = h / (H / a.G);
  const int start = a.seq_start[b], pos0 = a.seq_pos0[b];
  const int tid = threadIdx.x, nt = blockDim.x;
  float* S = smem;                                        // [d][cols]
  float* vec = smem + static_cast<size_t>(d) * cols;      // 2 x (k [d] | q [d])
  float* Sg = a.state + (static_cast<size_t>(a.seq_slot[b]) * H + h) * d * dv + c0;
  if (tid < cols) {
    if (pos0 == 0) for (int i = 0; i < d; ++i) S[i * cols + tid] = 0.f;
    else for (int i = 0; i < d; ++i) S[i * cols + tid] = Sg[static_cast<size_t>(i) * dv + tid];
  }
  const T* kp = static_cast<const T*>(a.k) + g * d;
  const T* qp = static_cast<const T*>(a.q) + g * d;
  const T* vp = static_cast<const T*>(a.v) + h * dv + c0;
  const T* s1 = static_cast<const T*>(a.s1);
  const T* s2 = static_cast<const T*>(a.s2);
  float c_f1 = 0.f, c_f2 = 0.f, c_f3 = 0.f;
  if (a.f1 != nullptr) c_f1 = a.f1[h];
  if (a.f2 != nullptr) c_f2 = a.f2[h];
  if (a.f3 != nullptr) c_f3 = a.f3[h];

  // registers holding the NEXT token's inputs
  float rk[SCAN_PER], rq[SCAN_PER], rv = 0.f, r1 = 0.f, r2 = 0.f, r3 = 0.f;
  auto fetch = [&](int t) {
    const size_t r = static_cast<size_t>(start + t);
#pragma unroll
    for (int x = 0; x < SCAN_PER; ++x) {
      const int i = tid + x * nt;
      if (i < d) { rk[x] = to_f(kp[r * a.ldk + i]); rq[x] = to_f(qp[r * a.ldq + i]); }
    }
    if (tid < cols) rv = to_f(vp[r * a.ldv + tid]);
    if constexpr (KIND == SCAN_SSM) r1 = to_f(s1[r * a.lds + h]);
    if constexpr (KIND == SCAN_DELTA) { r1 = to_f(s1[r * a.lds + h]); r2 = to_f(s2[r * a.lds + h]); }
    if constexpr (KIND == SCAN_MATRIX) {
      const float* gp = a.gates + (r * H + h) * 3;
      r1 = gp[0]; r2 = gp[1]; r3 = gp[2];
    }
  };
  fetch(0);
  for (int t = 0; t < len; ++t) {
    float* ks = vec + (t & 1) * 2 * d;
    float* qs = ks + d;
    float ssk = 0.f, ssq = 0.f;
#pragma unroll
    for (int x = 0; x < SCAN_PER; ++x) {
      const int i = tid + x * nt;
      if (i < d) { ks[i] = rk[x]; qs[i] = rq[x]; ssk += rk[x] * rk[x]; ssq += rq[x] * rq[x]; }
    }
    const float val = rv, p1 = r1, p2 = r2, p3 = r3;
    if (t + 1 < len) fetch(t + 1);
    float kn = 1.f, qn = a.qscale;
    if constexpr (KIND == SCAN_DELTA) {                   // unit vectors; the block sums also publish ks / qs
      kn = 1.0f / sqrtf(block_sum(ssk, red) + 1e-6f);
      qn = a.qscale / sqrtf(block_sum(ssq, red) + 1e-6f);
    } else {
      __syncthreads();
    }
    if (tid < cols) {
      float o = 0.f;
      if constexpr (KIND == SCAN_SSM) {
        const float dt = softplus_f(p1 + c_f1);
        const float dA = expf(-expf(c_f2) * dt);
        const float w = dt * val;
        for (int i = 0; i < d; ++i) {
          const float s = dA * S[i * cols + tid] + ks[i] * w;
          S[i * cols + tid] = s;
          o += s * qs[i];
        }
        o += c_f3 * val;
      } else if constexpr (KIND == SCAN_MATRIX) {
        const float w = p2 * val;
        for (int i = 0; i < d; ++i) {
          const float s = p1 * S[i * cols + tid] + ks[i] * w;
          S[i * cols + tid] = s;
          o += s * qs[i];
        }
        o = o * qn / p3;
      } else {
        const float beta = sigmoid_f(p1);
        const float decay = expf(-expf(c_f1) * softplus_f(p2 + c_f2));
        float kv = 0.f;
        for (int i = 0; i < d; ++i) {
          const float s = decay * S[i * cols + tid];
          S[i * cols + tid] = s;
          kv += s * (ks[i] * kn);
        }
        const float u = beta * (val - kv);
        for (int i = 0; i < d; ++i) {
          const float s = S[i * cols + tid] + (ks[i] * kn) * u;
          S[i * cols + tid] = s;
          o += s * (qs[i] * qn);
        }
      }
      a.out[static_cast<size_t>(start + t) * H * dv + h * dv + c0 + tid] = o;
    }
  }
  if (tid < cols)
    for (int i = 0; i < d; ++i) Sg[static_cast<size_t>(i) * dv + tid] = S[i * cols + tid];
}

// ------------------------------------------------------------------ scalar part of the matrix memory
// One CTA per (sequence, head).  i = cap tanh((ig + bi) / cap), f = logsigmoid(cap tanh((fg + bf) / cap));
// m' = max(f + m, i), a = exp(f + m - m'), b = exp(i - m'); n <- a n + b k; den = max(|n . q * qscale|, exp(-m')) + 1e-6.
// state_nm [slots, H, d + 1]: n, then m (m starts at 0).
template <typename T>
__global__ void __launch_bounds__(128)
matrix_memory_gates_kernel(const T* __restrict__ k, const T* __restrict__ q, const T* __restrict__ ig, const T* __restrict__ fg,
                           int64_t ldu, const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap,
                           float qscale, float* __restrict__ state_nm, float* __restrict__ gates,
                           const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_pos0,
                           const int32_t* __restrict__ seq_len, const int32_t* __restrict__ seq_slot, int H, int d) {
  __shared__ float red[33];
  const int b = blockIdx.y, h = blockIdx.x;
  const int len = seq_len[b];
  if (len <= 0) return;
  const int start = seq_start[b], pos0 = seq_pos0[b], tid = threadIdx.x, nt = blockDim.x;
  float* nm = state_nm + (static_cast<size_t>(seq_slot[b]) * H + h) * (d + 1);
  float n[SCAN_PER];
#pragma unroll
  for (int x = 0; x < SCAN_PER; ++x) {
    const int i = tid + x * nt;
    n[x] = (i < d && pos0 > 0) ? nm[i] : 0.f;
  }
  float m = pos0 > 0 ? nm[d] : 0.f;
  const float bi = i_bias[h], bf = f_bias[h];
  for (int t = 0; t < len; ++t) {
    const size_t r = static_cast<size_t>(start + t);
    const float li = cap * tanhf((to_f(ig[r * ldu + h]) + bi) / cap);
    const float lf = logsigmoid_f(cap * tanhf((to_f(fg[r * ldu + h]) + bf) / cap));
    const float m_new = fmaxf(lf + m, li);
    const float ca = expf(lf + m - m_new), cb = expf(li - m_new);
    m = m_new;
    float nq = 0.f;
#pragma unroll
    for (int x = 0; x < SCAN_PER; ++x) {
      const int i = tid + x * nt;
      if (i < d) {
        n[x] = ca * n[x] + cb * to_f(k[r * ldu + h * d + i]);
        nq += n[x] * (to_f(q[r * ldu + h * d + i]) * qscale);
      }
    }
    nq = block_sum(nq, red);
    if (tid == 0) {
      float* gp = gates + (r * H + h) * 3;
      gp[0] = ca; gp[1] = cb; gp[2] = fmaxf(fabsf(nq), expf(-m)) + 1e-6f;
    }
  }
#pragma unroll
  for (int x = 0; x < SCAN_PER; ++x) {
    const int i = tid + x * nt;
    if (i < d) nm[i] = n[x];
  }
  if (tid == 0) nm[d] = m;
}

template <typename T, int KIND>
static int launch_scan(const ScanArgs& a, int n_seqs, cudaStream_t st, const char* what) {
  const int cols = std::min(SCAN_MAX_COLS, a.dv);
  const int threads = std::max(32, (cols + 31) / 32 * 32);
  B2_REQUIRE(a.d <= SCAN_PER * threads, B2TTS_EUNSUPPORTED, "%s: key size %d above %d", what, a.d, SCAN_PER * threads);
  const size_t sm = (static_cast<size_t>(a.d) * cols + 4 * static_cast<size_t>(a.d)) * sizeof(float);
  B2_REQUIRE(sm <= 220 * 1024, B2TTS_EUNSUPPORTED, "%s: %d x %d columns of state do not fit shared memory", what, a.d, cols);
  static size_t opted = 0;                               // per instantiation
  if (sm > 48 * 1024 && sm > opted) {
    cudaError_t e = cudaFuncSetAttribute(scan_kernel<T, KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sm));
    if (e != cudaSuccess) return cuda_fail(e, what);
    opted = sm;
  }
  const dim3 grid((a.dv + SCAN_MAX_COLS - 1) / SCAN_MAX_COLS, a.H, n_seqs);
  scan_kernel<T, KIND><<<grid, threads, sm, st>>>(a);
  return B2TTS_OK;
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
                              const float* a_log, const float* d_skip, float* state, float* out, const int32_t* seq_start,
                              const int32_t* seq_pos0, const int32_t* seq_len, const int32_t* seq_slot, int n_seqs, int heads,
                              int groups, int vdim, int dim, int dtype, void* stream) {
  SCAN_COMMON_CHECKS("ssm_scan");
  B2_REQUIRE(groups > 0 && heads % groups == 0, B2TTS_EINVAL, "ssm_scan: %d heads over %d groups", heads, groups);
  B2_REQUIRE(xbc && dt && dt_bias && a_log && d_skip, B2TTS_EINVAL, "ssm_scan: null pointer");
  const size_t el = dtype == B2TTS_DTYPE_BF16 ? 2 : 4;
  const int inner = heads * vdim;
  ScanArgs a{};
  const char* base = static_cast<const char*>(xbc);
  a.v = base; a.ldv = ldx;
  a.k = base + static_cast<size_t>(inner) * el; a.ldk = ldx;
  a.q = base + (static_cast<size_t>(inner) + static_cast<size_t>(groups) * dim) * el; a.ldq = ldx;
  a.s1 = dt; a.lds = lddt;
  a.f1 = dt_bias; a.f2 = a_log; a.f3 = d_skip;
  a.state = state; a.out = out;
  a.seq_start = seq_start; a.seq_pos0 = seq_pos0; a.seq_len = seq_len; a.seq_slot = seq_slot;
  a.H = heads; a.G = groups; a.d = dim; a.dv = vdim; a.qscale = 1.f;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int rc = dtype == B2TTS_DTYPE_BF16 ? launch_scan<__nv_bfloat16, SCAN_SSM>(a, n_seqs, st, "ssm_scan")
                                           : launch_scan<float, SCAN_SSM>(a, n_seqs, st, "ssm_scan");
  if (rc != B2TTS_OK) return rc;
  B2_CHECK_LAUNCH("ssm_scan");
  return B2TTS_OK;
}

extern "C" int b2tts_delta_rule_scan(const void* qkv, int64_t ldq, const void* beta, const void* a_in, int64_t ldu,
                                     const float* a_log, const float* dt_bias, float* state, float* out,
                                     const int32_t* seq_start, const int32_t* seq_pos0, const int32_t* seq_len,
                                     const int32_t* seq_slot, int n_seqs, int heads, int kv_heads, int dim, int vdim, int dtype,
                                     void* stream) {
  SCAN_COMMON_CHECKS("delta_rule_scan");
  B2_REQUIRE(kv_heads > 0 && heads % kv_heads == 0, B2TTS_EINVAL, "delta_rule_scan: %d heads over %d key heads", heads, kv_heads);
  B2_REQUIRE(qkv && beta && a_in && a_log && dt_bias, B2TTS_EINVAL, "delta_rule_scan: null pointer");
  const size_t el = dtype == B2TTS_DTYPE_BF16 ? 2 : 4;
  ScanArgs a{};
  const char* base = static_cast<const char*>(qkv);
  const size_t gd = static_cast<size_t>(kv_heads) * dim;
  a.q = base; a.ldq = ldq;
  a.k = base + gd * el; a.ldk = ldq;
  a.v = base + 2 * gd * el; a.ldv = ldq;
  a.s1 = beta; a.s2 = a_in; a.lds = ldu;
  a.f1 = a_log; a.f2 = dt_bias;
  a.state = state; a.out = out;
  a.seq_start = seq_start; a.seq_pos0 = seq_pos0; a.seq_len = seq_len; a.seq_slot = seq_slot;
  a.H = heads; a.G = kv_heads; a.d = dim; a.dv = vdim; a.qscale = 1.0f / sqrtf(static_cast<float>(dim));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int rc = dtype == B2TTS_DTYPE_BF16 ? launch_scan<__nv_bfloat16, SCAN_DELTA>(a, n_seqs, st, "delta_rule_scan")
                                           : launch_scan<float, SCAN_DELTA>(a, n_seqs, st, "delta_rule_scan");
  if (rc != B2TTS_OK) return rc;
  B2_CHECK_LAUNCH("delta_rule_scan");
  return B2TTS_OK;
}

extern "C" int b2tts_matrix_memory_scan(const void* q, const void* k, const void* v, const void* ig, const void* fg, int64_t ldu,
                                        const float* i_bias, const float* f_bias, float cap, float* state, float* state_nm,
                                        float* gates, float* out, const int32_t* seq_start, const int32_t* seq_pos0,
                                        const int32_t* seq_len, const int32_t* seq_slot, int n_seqs, int heads, int dim,
                                        int vdim, int dtype, void* stream) {
  SCAN_COMMON_CHECKS("matrix_memory_scan");
  B2_REQUIRE(q && k && v && ig && fg && i_bias && f_bias && state_nm && gates && cap > 0.f, B2TTS_EINVAL,
             "matrix_memory_scan: null pointer or cap <= 0");
  B2_REQUIRE(dim <= SCAN_PER * 128, B2TTS_EUNSUPPORTED, "matrix_memory_scan: key size %d above %d", dim, SCAN_PER * 128);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const float qscale = 1.0f / sqrtf(static_cast<float>(dim));
  const dim3 ggrid(heads, n_seqs);
  const int gthreads = std::min(128, std::max(32, (dim + 31) / 32 * 32));
  if (dtype == B2TTS_DTYPE_BF16)
    matrix_memory_gates_kernel<__nv_bfloat16><<<ggrid, gthreads, 0, st>>>(static_cast<const __nv_bfloat16*>(k),
        static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(ig), static_cast<const __nv_bfloat16*>(fg), ldu, i_bias,
        f_bias, cap, qscale, state_nm, gates, seq_start, seq_pos0, seq_len, seq_slot, heads, dim);
  else
    matrix_memory_gates_kernel<float><<<ggrid, gthreads, 0, st>>>(static_cast<const float*>(k), static_cast<const float*>(q),
        static_cast<const float*>(ig), static_cast<const float*>(fg), ldu, i_bias, f_bias, cap, qscale, state_nm, gates, seq_start,
        seq_pos0, seq_len, seq_slot, heads, dim);
  B2_CHECK_LAUNCH("matrix_memory_gates");
  ScanArgs a{};
  a.q = q; a.ldq = ldu; a.k = k; a.ldk = ldu; a.v = v; a.ldv = ldu;
  a.gates = gates;
  a.state = state; a.out = out;
  a.seq_start = seq_start; a.seq_pos0 = seq_pos0; a.seq_len = seq_len; a.seq_slot = seq_slot;
  a.H = heads; a.G = heads; a.d = dim; a.dv = vdim; a.qscale = qscale;
  const int rc = dtype == B2TTS_DTYPE_BF16 ? launch_scan<__nv_bfloat16, SCAN_MATRIX>(a, n_seqs, st, "matrix_memory_scan")
                                           : launch_scan<float, SCAN_MATRIX>(a, n_seqs, st, "matrix_memory_scan");
  if (rc != B2TTS_OK) return rc;
  B2_CHECK_LAUNCH("matrix_memory_scan");
  return B2TTS_OK;
}
