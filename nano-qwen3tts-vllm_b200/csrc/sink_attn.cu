// sink_attn.cu - softmax attention over a paged K/V cache with a learned per-head sink in the denominator, under a
// sliding-window or a chunk mask, for every row of an engine step at once (prompt portions beside single decoded tokens).
//
//   w(i, j) = exp(q_ih . k_jg * scale - m) / (sum over the visible j of exp(. - m) + exp(sink_h - m)),   out = sum_j w v_jg
//   window mask: max(0, i - mask + 1) <= j <= i        chunk mask: floor(i / mask) * mask <= j <= i        mask <= 0: j <= i
//
// Both masks are a lower bound on j, so one kernel serves them.  The sink has no key and no value and is not scaled.  An
// optional per-head gate multiplies the head's output by sigmoid(gate[t, h]).
//
// Plain kernel (bf16 or float, any head size up to 256): one CTA of four warps per (token, query head).  A warp takes
// 32-key tiles: each lane scores one key against the query held in shared memory (float accumulation), the warp keeps a
// running maximum and denominator, and the lanes then split the value columns for the weighted sum.  The four warps'
// partial results are merged through shared memory.  Scores, weights and sums are float in both modes.
#include <math.h>

#include "row_ops.cuh"

namespace b2 {
namespace row {

constexpr int SA_WARPS = 4;
constexpr int SA_MAX_PER_LANE = 8;        // value sizes up to 256

template <typename T> struct Vec16;       // how many T fit 16 bytes
template <> struct Vec16<float> { static constexpr int N = 4; };
template <> struct Vec16<__nv_bfloat16> { static constexpr int N = 8; };

template <typename T>
__device__ __forceinline__ float dot_row(const T* __restrict__ kr, const float* __restrict__ q, int d, bool vec) {
  float acc = 0.f;
  if (vec) {
    constexpr int N = Vec16<T>::N;
    for (int c = 0; c < d; c += N) {
      const uint4 raw = ldg_v4(kr + c);
      if constexpr (N == 8) {
        acc += bf16lo(raw.x) * q[c] + bf16hi(raw.x) * q[c + 1] + bf16lo(raw.y) * q[c + 2] + bf16hi(raw.y) * q[c + 3] +
               bf16lo(raw.z) * q[c + 4] + bf16hi(raw.z) * q[c + 5] + bf16lo(raw.w) * q[c + 6] + bf16hi(raw.w) * q[c + 7];
      } else {
        acc += __uint_as_float(raw.x) * q[c] + __uint_as_float(raw.y) * q[c + 1] + __uint_as_float(raw.z) * q[c + 2] +
               __uint_as_float(raw.w) * q[c + 3];
      }
    }
  } else {
    for (int c = 0; c < d; ++c) acc += to_f(kr[c]) * q[c];
  }
  return acc;
}

template <typename T>
__global__ void __launch_bounds__(SA_WARPS * 32)
sink_attn_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache, T* __restrict__ out,
                 const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ positions, const int32_t* __restrict__ seq_len,
                 const int32_t* __restrict__ block_tables, int64_t bt_stride, const float* __restrict__ sink,
                 const T* __restrict__ gate, int64_t ldg, int H, int G, int d, int dv, int page, int mask_kind, int mask,
                 float scale) {
  extern __shared__ float smem[];
  float* qs = smem;                                   // [d]
  float* part = smem + ((d + 3) & ~3);                // [SA_WARPS][dv + 2]: sums, running maximum, denominator
  const size_t t = blockIdx.x;
  const int h = blockIdx.y, g = h / (H / G);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int b = tok_seq[t];
  T* orow = out + (t * H + h) * dv;
  if (seq_len[b] <= 0) {                              // padding row
    for (int c = threadIdx.x; c < dv; c += blockDim.x) orow[c] = from_f<T>(0.f);
    return;
  }
  const int i = positions[t];
  int lo = 0;
  if (mask > 0) lo = mask_kind == 0 ? max(0, i - mask + 1) : (i / mask) * mask;
  const T* qr = q + (t * H + h) * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) qs[c] = to_f(qr[c]);
  __syncthreads();
  const int32_t* bt = block_tables + static_cast<int64_t>(b) * bt_stride;
  const int nk = G * d, nv = G * dv;
  const bool vec = (d % Vec16<T>::N) == 0;            // rows then start on 16-byte boundaries (the cache base is aligned)
  float m = -INFINITY, l = 0.f;
  float acc[SA_MAX_PER_LANE];
#pragma unroll
  for (int x = 0; x < SA_MAX_PER_LANE; ++x) acc[x] = 0.f;
  const int n_keys = i - lo + 1;
  for (int j0 = warp * 32; j0 < n_keys; j0 += SA_WARPS * 32) {
    const int j = lo + j0 + lane;
    float s = -INFINITY;
    int slot = 0;
    if (j <= i) {
      slot = bt[j / page] * page + j % page;
      s = dot_row<T>(k_cache + static_cast<size_t>(slot) * nk + g * d, qs, d, vec) * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));        // finite: the tile's first key exists
    const float p = j <= i ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);               // 0 on the first tile (m = -inf)
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int x = 0; x < SA_MAX_PER_LANE; ++x) acc[x] *= corr;
    const int cnt = min(32, n_keys - j0);
    for (int kk = 0; kk < cnt; ++kk) {
      const float pk = __shfl_sync(0xffffffffu, p, kk);
      const int sk = __shfl_sync(0xffffffffu, slot, kk);
      const T* vr = v_cache + static_cast<size_t>(sk) * nv + g * dv;
#pragma unroll
      for (int x = 0; x < SA_MAX_PER_LANE; ++x) {
        const int c = lane + 32 * x;
        if (c < dv) acc[x] += pk * to_f(vr[c]);
      }
    }
  }
  float* mine = part + warp * (dv + 2);
#pragma unroll
  for (int x = 0; x < SA_MAX_PER_LANE; ++x) {
    const int c = lane + 32 * x;
    if (c < dv) mine[c] = acc[x];
  }
  if (lane == 0) { mine[dv] = m; mine[dv + 1] = l; }
  __syncthreads();
  const float sk = sink != nullptr ? sink[h] : -INFINITY;
  float mm = sk;
#pragma unroll
  for (int w = 0; w < SA_WARPS; ++w) mm = fmaxf(mm, part[w * (dv + 2) + dv]);
  float den = sink != nullptr ? expf(sk - mm) : 0.f;
  float cw[SA_WARPS];
#pragma unroll
  for (int w = 0; w < SA_WARPS; ++w) {
    const float mw = part[w * (dv + 2) + dv];
    cw[w] = mw == -INFINITY ? 0.f : expf(mw - mm);
    den += cw[w] * part[w * (dv + 2) + dv + 1];
  }
  float gv = 1.f;
  if (gate != nullptr) gv = sigmoid_f(to_f(gate[t * ldg + h]));
  const float inv = gv / den;
  for (int c = threadIdx.x; c < dv; c += blockDim.x) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < SA_WARPS; ++w) o += cw[w] * part[w * (dv + 2) + c];
    orow[c] = from_f<T>(o * inv);
  }
}

}  // namespace row
}  // namespace b2

using namespace b2;
using namespace b2::row;

extern "C" int b2tts_sink_attn(const void* q, const void* k_cache, const void* v_cache, void* out, const int32_t* tok_seq,
                               const int32_t* positions, const int32_t* seq_len, const int32_t* block_tables, int64_t bt_stride,
                               const float* sink, const void* gate, int64_t ldg, int n_tokens, int heads, int kv_heads, int dim,
                               int vdim, int page, int mask_kind, int mask, float scale, int dtype, void* stream) {
  B2_REQUIRE(n_tokens >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dim > 0 && vdim > 0 && page > 0, B2TTS_EINVAL,
             "sink_attn: bad sizes (heads=%d kv_heads=%d dim=%d vdim=%d page=%d)", heads, kv_heads, dim, vdim, page);
  B2_REQUIRE(vdim <= 32 * SA_MAX_PER_LANE, B2TTS_EUNSUPPORTED, "sink_attn: value size %d above %d", vdim, 32 * SA_MAX_PER_LANE);
  B2_REQUIRE(heads <= 65535, B2TTS_EUNSUPPORTED, "sink_attn: %d heads", heads);
  B2_REQUIRE(mask_kind == 0 || mask_kind == 1, B2TTS_EINVAL, "sink_attn: mask kind %d", mask_kind);
  B2_REQUIRE(B2_ROW_DTYPE_OK(dtype), B2TTS_EINVAL, "sink_attn: dtype %d", dtype);
  if (n_tokens == 0) return B2TTS_OK;
  B2_REQUIRE(q && k_cache && v_cache && out && tok_seq && positions && seq_len && block_tables, B2TTS_EINVAL, "sink_attn: null pointer");
  B2_REQUIRE(aligned16(k_cache) && aligned16(v_cache), B2TTS_EALIGN, "sink_attn: caches must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t sm = (((dim + 3) & ~3) + SA_WARPS * (vdim + 2)) * sizeof(float);
  const dim3 grid(n_tokens, heads);
  if (dtype == B2TTS_DTYPE_BF16)
    sink_attn_kernel<__nv_bfloat16><<<grid, SA_WARPS * 32, sm, st>>>(static_cast<const __nv_bfloat16*>(q),
        static_cast<const __nv_bfloat16*>(k_cache), static_cast<const __nv_bfloat16*>(v_cache), static_cast<__nv_bfloat16*>(out), tok_seq,
        positions, seq_len, block_tables, bt_stride, sink, static_cast<const __nv_bfloat16*>(gate), ldg, heads, kv_heads, dim, vdim, page,
        mask_kind, mask, scale);
  else
    sink_attn_kernel<float><<<grid, SA_WARPS * 32, sm, st>>>(static_cast<const float*>(q), static_cast<const float*>(k_cache),
        static_cast<const float*>(v_cache), static_cast<float*>(out), tok_seq, positions, seq_len, block_tables, bt_stride, sink,
        static_cast<const float*>(gate), ldg, heads, kv_heads, dim, vdim, page, mask_kind, mask, scale);
  B2_CHECK_LAUNCH("sink_attn");
  return B2TTS_OK;
}
