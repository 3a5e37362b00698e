// sink_attn.cu - softmax attention over a paged K/V cache with a learned per-head sink in the denominator, under a
// sliding-window or a chunk mask, for every row of an engine step at once (prompt portions beside single decoded tokens).
//
//   w(i, j) = exp(q_ih . k_jg * scale - m) / (sum over the visible j of exp(. - m) + exp(sink_h - m)),   out = sum_j w v_jg
//   window mask: max(0, i - mask + 1) <= j <= i        chunk mask: floor(i / mask) * mask <= j <= i        mask <= 0: j <= i
//
// Both masks are a lower bound on j, so one kernel serves them.  The sink has no key and no value and is not scaled.  An
// optional per-head gate multiplies the head's output by sigmoid(gate[t, h]).
//
// Three more switches, each off at its neutral value: keep_first F > 0 lets every token also see the keys j < F that its mask
// hides (the kernels then walk a virtual key list, [0, min(F, lo)) followed by [lo, i]); softcap c > 0 turns a scaled score
// s into c tanh(s / c) before the softmax; v_heads < kv_heads makes key head g read value head g mod v_heads (several key
// maps over one set of values).
//
// Three kernels share a launch: prompt portions in bf16 with head sizes 32..128 x 64, 128 run on the tensor cores
// (sink_attn_mma_kernel), rows with ONE new token and a head size of 4, 8, 16 or 32 16-byte pieces (dv = d or 2 d) in a kernel whose
// lanes split a cached row (sink_attn_decode_kernel), everything else in the plain kernel; each skips the rows of the others.
//
// Plain kernel (bf16 or float, any head size up to 256): one CTA of four warps per token and 1, 2 or 4 query heads of one
// key/value group, so a cached row is loaded once for all of them.  A warp takes 32-key tiles: each lane scores one key
// against the queries held in shared memory (float accumulation), the warp keeps a running maximum and denominator per
// head, and the lanes then split the value columns for the weighted sums.  The four warps' partial results are merged
// through shared memory.  Scores, weights and sums are float in both modes.
#include <math.h>

#include "row_ops.cuh"

namespace b2 {
namespace row {

constexpr int SA_WARPS = 4;
constexpr int SA_MAX_PER_LANE = 8;        // value sizes up to 256
constexpr int SA_ROWS_AHEAD = 8;          // value rows in flight per lane

// an output element: of the activation type, or a float where the caller asked for unrounded results (`f32`)
template <typename T>
__device__ __forceinline__ void put_out(T* out, size_t idx, float v, int f32) {
  if (f32) reinterpret_cast<float*>(out)[idx] = v;
  else out[idx] = from_f<T>(v);
}

template <typename T> struct Vec16;       // how many T fit 16 bytes
template <> struct Vec16<float> { static constexpr int N = 4; };
template <> struct Vec16<__nv_bfloat16> { static constexpr int N = 8; };

// `cpl` consecutive value columns of one cached row -> floats; `bytes` = cpl * sizeof(T) when the row allows vector loads, else 0
template <typename T>
__device__ __forceinline__ void load_cols(const T* __restrict__ p, int cpl, int bytes, int room, float* f) {
  if (bytes == 0) {
#pragma unroll
    for (int x = 0; x < SA_MAX_PER_LANE; ++x) f[x] = (x < cpl && x < room) ? to_f(p[x]) : 0.f;
    return;
  }
  uint32_t w[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (bytes == 4) w[0] = *reinterpret_cast<const uint32_t*>(p);
  else if (bytes == 8) { const uint2 r = ldg_v2(p); w[0] = r.x; w[1] = r.y; }
  else {
    const uint4 r = ldg_v4(p);
    w[0] = r.x; w[1] = r.y; w[2] = r.z; w[3] = r.w;
    if (bytes == 32) { const uint4 r2 = ldg_v4(reinterpret_cast<const char*>(p) + 16); w[4] = r2.x; w[5] = r2.y; w[6] = r2.z; w[7] = r2.w; }
  }
  if constexpr (sizeof(T) == 2) {
#pragma unroll
    for (int x = 0; x < 4; ++x) { f[2 * x] = bf16lo(w[x]); f[2 * x + 1] = bf16hi(w[x]); }
  } else {
#pragma unroll
    for (int x = 0; x < 8; ++x) f[x] = __uint_as_float(w[x]);
  }
}

// REP query heads of one key/value group share the CTA: a key row and a value row are loaded once and serve all of them.
template <typename T, int REP>
__device__ __forceinline__ void dot_rows(const T* __restrict__ kr, const float* __restrict__ q, int d, int qs_stride, bool vec, float* s) {
#pragma unroll
  for (int r = 0; r < REP; ++r) s[r] = 0.f;
  if (vec) {
    constexpr int N = Vec16<T>::N, B = 8;              // eight 16-byte pieces of the row are asked for before the first is used
    for (int c0 = 0; c0 < d; c0 += B * N) {
      uint4 raw[B];
#pragma unroll
      for (int i = 0; i < B; ++i) raw[i] = c0 + i * N < d ? ldg_v4(kr + c0 + i * N) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int i = 0; i < B; ++i) {
        const int c = c0 + i * N;
        if (c < d) {
          float f[8];
          if constexpr (N == 8) {
            f[0] = bf16lo(raw[i].x); f[1] = bf16hi(raw[i].x); f[2] = bf16lo(raw[i].y); f[3] = bf16hi(raw[i].y);
            f[4] = bf16lo(raw[i].z); f[5] = bf16hi(raw[i].z); f[6] = bf16lo(raw[i].w); f[7] = bf16hi(raw[i].w);
          } else {
            f[0] = __uint_as_float(raw[i].x); f[1] = __uint_as_float(raw[i].y); f[2] = __uint_as_float(raw[i].z); f[3] = __uint_as_float(raw[i].w);
          }
#pragma unroll
          for (int r = 0; r < REP; ++r) {
            const float4* qr = reinterpret_cast<const float4*>(q + r * qs_stride + c);
            const float4 qa = qr[0];
            s[r] += f[0] * qa.x + f[1] * qa.y + f[2] * qa.z + f[3] * qa.w;
            if constexpr (N == 8) {
              const float4 qb = qr[1];
              s[r] += f[4] * qb.x + f[5] * qb.y + f[6] * qb.z + f[7] * qb.w;
            }
          }
        }
      }
    }
  } else {
    for (int c = 0; c < d; ++c) {
      const float kv = to_f(kr[c]);
#pragma unroll
      for (int r = 0; r < REP; ++r) s[r] += kv * q[r * qs_stride + c];
    }
  }
}

template <typename T, int REP>
__global__ void __launch_bounds__(SA_WARPS * 32)
sink_attn_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache, T* __restrict__ out,
                 const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ positions, const int32_t* __restrict__ seq_len,
                 const int32_t* __restrict__ block_tables, int64_t bt_stride, const float* __restrict__ sink,
                 const T* __restrict__ gate, int64_t ldg, int H, int G, int Gv, int d, int dv, int page, int mask_kind, int mask,
                 int keep_first, float softcap, float scale, int only_single, int out_f32) {
  extern __shared__ float smem[];
  const int qstride = (d + 3) & ~3;
  float* qs = smem;                                   // [REP][qstride]
  float* part = smem + REP * qstride;                 // [SA_WARPS][REP][dv + 2]: sums, running maximum, denominator
  const size_t t = blockIdx.x;
  const int h0 = blockIdx.y * REP, g = h0 / (H / G);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int b = tok_seq[t];
  const size_t obase = (t * H + h0) * dv;             // the REP heads' outputs are adjacent
  if ((only_single & 1) && seq_len[b] > 1) return;    // the tensor-core kernel owns prompt portions
  if ((only_single & 2) && seq_len[b] == 1) return;   // the row-splitting kernel owns one-token rows
  if (seq_len[b] <= 0) {                              // padding row
    for (int c = threadIdx.x; c < REP * dv; c += blockDim.x) put_out(out, obase + c, 0.f, out_f32);
    return;
  }
  const int i = positions[t];
  int lo = 0;
  if (mask > 0) lo = mask_kind == 0 ? max(0, i - mask + 1) : (i / mask) * mask;
  const T* qr = q + (t * H + h0) * d;
  for (int c = threadIdx.x; c < REP * d; c += blockDim.x) qs[(c / d) * qstride + c % d] = to_f(qr[c]);
  __syncthreads();
  const int32_t* bt = block_tables + static_cast<int64_t>(b) * bt_stride;
  const int nk = G * d, nv = Gv * dv, gv = g % Gv;
  const int npre = min(keep_first, lo);                // kept first keys the mask hides: they come first in the key list
  const bool vec = (d % Vec16<T>::N) == 0;            // rows then start on 16-byte boundaries (the cache base is aligned)
  // a lane owns `cpl` consecutive value columns; with dv a multiple of 32 they are one aligned vector load per key
  const int cpl = (dv + 31) / 32, c_lane = lane * cpl;
  const int cbytes = cpl * static_cast<int>(sizeof(T));
  const int vbytes = (dv % 32 == 0 && (cbytes == 4 || cbytes == 8 || cbytes == 16 || cbytes == 32)) ? cbytes : 0;
  const int room = max(0, min(cpl, dv - c_lane));
  float m[REP], l[REP], acc[REP][SA_MAX_PER_LANE];
#pragma unroll
  for (int r = 0; r < REP; ++r) {
    m[r] = -INFINITY; l[r] = 0.f;
#pragma unroll
    for (int x = 0; x < SA_MAX_PER_LANE; ++x) acc[r][x] = 0.f;
  }
  const int n_keys = npre + i - lo + 1;
  for (int j0 = warp * 32; j0 < n_keys; j0 += SA_WARPS * 32) {
    const int vi = j0 + lane;
    const bool valid = vi < n_keys;
    const int j = vi < npre ? vi : lo + vi - npre;
    float sc[REP], p[REP];
    int slot = 0;
#pragma unroll
    for (int r = 0; r < REP; ++r) sc[r] = -INFINITY;
    if (valid) {
      slot = bt[j / page] * page + j % page;
      dot_rows<T, REP>(k_cache + static_cast<size_t>(slot) * nk + g * d, qs, d, qstride, vec, sc);
    }
#pragma unroll
    for (int r = 0; r < REP; ++r) {
      float s = -INFINITY;
      if (valid) {
        s = sc[r] * scale;
        if (softcap > 0.f) s = softcap * tanhf(s / softcap);
      }
      const float m_new = fmaxf(m[r], warp_max(s));   // finite: the tile's first key exists
      p[r] = valid ? expf(s - m_new) : 0.f;
      const float corr = expf(m[r] - m_new);          // 0 on the first tile (m = -inf)
      l[r] = l[r] * corr + warp_sum(p[r]);
      m[r] = m_new;
#pragma unroll
      for (int x = 0; x < SA_MAX_PER_LANE; ++x) acc[r][x] *= corr;
    }
    // four value rows are asked for before the first is used: their loads overlap
    const int cnt = min(32, n_keys - j0);
    for (int kk0 = 0; kk0 < cnt; kk0 += SA_ROWS_AHEAD) {
      float vf[SA_ROWS_AHEAD][SA_MAX_PER_LANE];
#pragma unroll
      for (int u = 0; u < SA_ROWS_AHEAD; ++u) {
        const int sk = __shfl_sync(0xffffffffu, slot, (kk0 + u) & 31);
        if (kk0 + u < cnt) {
          load_cols<T>(v_cache + static_cast<size_t>(sk) * nv + gv * dv + (room > 0 ? c_lane : 0), cpl, vbytes, room, vf[u]);
        } else {
#pragma unroll
          for (int x = 0; x < SA_MAX_PER_LANE; ++x) vf[u][x] = 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < SA_ROWS_AHEAD; ++u) {
#pragma unroll
        for (int r = 0; r < REP; ++r) {
          float pk = __shfl_sync(0xffffffffu, p[r], (kk0 + u) & 31);
          if (kk0 + u >= cnt) pk = 0.f;
#pragma unroll
          for (int x = 0; x < SA_MAX_PER_LANE; ++x) acc[r][x] += pk * vf[u][x];
        }
      }
    }
  }
  const int pstride = dv + 2;
#pragma unroll
  for (int r = 0; r < REP; ++r) {
    float* mine = part + (warp * REP + r) * pstride;
#pragma unroll
    for (int x = 0; x < SA_MAX_PER_LANE; ++x)
      if (x < room) mine[c_lane + x] = acc[r][x];
    if (lane == 0) { mine[dv] = m[r]; mine[dv + 1] = l[r]; }
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < REP; ++r) {
    const int h = h0 + r;
    const float sk = sink != nullptr ? sink[h] : -INFINITY;
    float mm = sk;
#pragma unroll
    for (int w = 0; w < SA_WARPS; ++w) mm = fmaxf(mm, part[(w * REP + r) * pstride + dv]);
    float den = sink != nullptr ? expf(sk - mm) : 0.f;
    float cw[SA_WARPS];
#pragma unroll
    for (int w = 0; w < SA_WARPS; ++w) {
      const float mw = part[(w * REP + r) * pstride + dv];
      cw[w] = mw == -INFINITY ? 0.f : expf(mw - mm);
      den += cw[w] * part[(w * REP + r) * pstride + dv + 1];
    }
    float gv = 1.f;
    if (gate != nullptr) gv = sigmoid_f(to_f(gate[t * ldg + h]));
    const float inv = gv / den;
    for (int c = threadIdx.x; c < dv; c += blockDim.x) {
      float o = 0.f;
#pragma unroll
      for (int w = 0; w < SA_WARPS; ++w) o += cw[w] * part[(w * REP + r) * pstride + c];
      put_out(out, obase + r * dv + c, o * inv, out_f32);
    }
  }
}

template <typename T, int REP>
static void launch_sink_plain(cudaStream_t st, const void* q, const void* kc, const void* vc, void* out, const int32_t* tok_seq,
                              const int32_t* positions, const int32_t* seq_len, const int32_t* bt, int64_t bt_stride, const float* sink,
                              const void* gate, int64_t ldg, int n_tokens, int H, int G, int Gv, int d, int dv, int page, int mask_kind,
                              int mask, int keep_first, float softcap, float scale, int only_single, int out_f32) {
  const size_t sm = (static_cast<size_t>(REP) * ((d + 3) & ~3) + static_cast<size_t>(SA_WARPS) * REP * (dv + 2)) * sizeof(float);
  sink_attn_kernel<T, REP><<<dim3(n_tokens, H / REP), SA_WARPS * 32, sm, st>>>(
      static_cast<const T*>(q), static_cast<const T*>(kc), static_cast<const T*>(vc), static_cast<T*>(out), tok_seq, positions, seq_len, bt,
      bt_stride, sink, static_cast<const T*>(gate), ldg, H, G, Gv, d, dv, page, mask_kind, mask, keep_first, softcap, scale, only_single, out_f32);
}

template <typename T>
static void launch_sink_plain_rep(int rep, cudaStream_t st, const void* q, const void* kc, const void* vc, void* out,
                                  const int32_t* tok_seq, const int32_t* positions, const int32_t* seq_len, const int32_t* bt,
                                  int64_t bt_stride, const float* sink, const void* gate, int64_t ldg, int n_tokens, int H, int G, int Gv,
                                  int d, int dv, int page, int mask_kind, int mask, int keep_first, float softcap, float scale,
                                  int only_single, int out_f32) {
#define SINK_PLAIN_ARGS st, q, kc, vc, out, tok_seq, positions, seq_len, bt, bt_stride, sink, gate, ldg, n_tokens, H, G, Gv, d, dv, page, mask_kind, mask, keep_first, softcap, scale, only_single, out_f32
  // heads of a group that share a CTA: as many as divide the group, up to four (two for wide values: registers)
  if (rep % 4 == 0 && dv <= 128) launch_sink_plain<T, 4>(SINK_PLAIN_ARGS);
  else if (rep % 2 == 0) launch_sink_plain<T, 2>(SINK_PLAIN_ARGS);
  else launch_sink_plain<T, 1>(SINK_PLAIN_ARGS);
#undef SINK_PLAIN_ARGS
}

// ------------------------------------------------------------------ one-token rows: the lanes split a cached row
// One CTA of eight warps per (sequence with ONE new token, REP query heads of a key/value group).  LPK lanes read one key
// row, 16 bytes each (N elements; d = dv = LPK * N), so a warp-wide load is contiguous and covers 32 / LPK keys; a lane
// keeps its slice of the REP queries (times scale * log2 e) and of the REP accumulators in registers.  Four key steps
// (K and V pieces of four keys per lane group) are in flight before the first is used.  A score is the slice's dot product
// summed over the LPK lanes by shuffles; every lane group keeps a running maximum and denominator per head (base 2), the
// groups of a warp are merged by shuffles and the warps through shared memory, where the sink joins the denominator.
// Values may be VR = 1 or 2 times as wide as keys (dv = VR * d): a lane then takes VR 16-byte pieces of a value row, LPK
// pieces apart, so that the warp's loads stay contiguous.
constexpr int SD_WARPS = 8, SD_AHEAD = 4;

template <typename T, int LPK, int REP, int VR>
__global__ void __launch_bounds__(SD_WARPS * 32)
sink_attn_decode_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache, T* __restrict__ out,
                        const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_pos0,
                        const int32_t* __restrict__ seq_len, const int32_t* __restrict__ block_tables, int64_t bt_stride,
                        const float* __restrict__ sink, const T* __restrict__ gate, int64_t ldg, int H, int G, int Gv, int page,
                        int mask_kind, int mask, int keep_first, float softcap, float scale, int out_f32) {
  constexpr int N = Vec16<T>::N, D = LPK * N, DV = D * VR, KPW = 32 / LPK;
  constexpr float LOG2E = 1.4426950408889634f;
  __shared__ float part[SD_WARPS][REP][DV + 2];
  // the head groups of a sequence are neighbours in launch order: key heads that share a value head (v_heads < kv_heads)
  // run at the same time and the second reader finds the value rows in L2
  const int b = blockIdx.y;
  if (seq_len[b] != 1) return;
  const int h0 = blockIdx.x * REP, g = h0 / (H / G);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane % LPK, kg = lane / LPK;
  const size_t t = seq_start[b];
  const int i = seq_pos0[b];
  int lo = 0;
  if (mask > 0) lo = mask_kind == 0 ? max(0, i - mask + 1) : (i / mask) * mask;
  const int32_t* bt = block_tables + static_cast<int64_t>(b) * bt_stride;
  const size_t row = static_cast<size_t>(G) * D;          // elements of a cached key row
  const size_t vrow = static_cast<size_t>(Gv) * DV;       // and of a value row
  const int gv = g % Gv;
  const int npre = min(keep_first, lo), n_keys = npre + i - lo + 1;    // kept first keys the mask hides, then [lo, i]
  const float cap2 = softcap * LOG2E;                      // the cap in the base-2 domain the scores live in
  float qv[REP][N], acc[REP][VR * N], m[REP], l[REP];
#pragma unroll
  for (int r = 0; r < REP; ++r) {
    const T* qr = q + (t * H + h0 + r) * D + sub * N;
#pragma unroll
    for (int e = 0; e < N; ++e) qv[r][e] = to_f(qr[e]) * (scale * LOG2E);
#pragma unroll
    for (int e = 0; e < VR * N; ++e) acc[r][e] = 0.f;
    m[r] = -1e30f; l[r] = 0.f;
  }
  auto unpack = [](const uint4& raw, float* f) {
    if constexpr (N == 8) {
      f[0] = bf16lo(raw.x); f[1] = bf16hi(raw.x); f[2] = bf16lo(raw.y); f[3] = bf16hi(raw.y);
      f[4] = bf16lo(raw.z); f[5] = bf16hi(raw.z); f[6] = bf16lo(raw.w); f[7] = bf16hi(raw.w);
    } else {
      f[0] = __uint_as_float(raw.x); f[1] = __uint_as_float(raw.y); f[2] = __uint_as_float(raw.z); f[3] = __uint_as_float(raw.w);
    }
  };
  constexpr int STEP = SD_WARPS * KPW;                     // keys the CTA takes per step
  for (int j0 = 0; j0 < n_keys; j0 += STEP * SD_AHEAD) {
    uint4 kraw[SD_AHEAD], vraw[SD_AHEAD][VR];
    bool ok[SD_AHEAD];
#pragma unroll
    for (int u = 0; u < SD_AHEAD; ++u) {
      const int vi = j0 + u * STEP + warp * KPW + kg;
      const int j = vi < npre ? vi : lo + vi - npre;
      ok[u] = vi < n_keys;
      kraw[u] = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int p = 0; p < VR; ++p) vraw[u][p] = make_uint4(0, 0, 0, 0);
      if (ok[u]) {
        const int pg = j / page;
        const size_t slot = static_cast<size_t>(bt[pg]) * page + (j - pg * page);
        kraw[u] = ldg_v4(k_cache + slot * row + g * D + sub * N);
#pragma unroll
        for (int p = 0; p < VR; ++p) vraw[u][p] = ldg_v4(v_cache + slot * vrow + gv * DV + (p * LPK + sub) * N);
      }
    }
    float sc[SD_AHEAD][REP];
#pragma unroll
    for (int u = 0; u < SD_AHEAD; ++u) {
      float f[N];
      unpack(kraw[u], f);
#pragma unroll
      for (int r = 0; r < REP; ++r) {
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < N; ++e) s += f[e] * qv[r][e];
#pragma unroll
        for (int o = LPK / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (softcap > 0.f) s = cap2 * tanhf(s / cap2);
        sc[u][r] = ok[u] ? s : -INFINITY;
      }
    }
#pragma unroll
    for (int r = 0; r < REP; ++r) {
      float mx = sc[0][r];
#pragma unroll
      for (int u = 1; u < SD_AHEAD; ++u) mx = fmaxf(mx, sc[u][r]);
      const float m_new = fmaxf(m[r], mx);                 // finite: m starts finite
      const float corr = exp2f(m[r] - m_new);
      m[r] = m_new;
      l[r] *= corr;
#pragma unroll
      for (int e = 0; e < VR * N; ++e) acc[r][e] *= corr;
#pragma unroll
      for (int u = 0; u < SD_AHEAD; ++u) sc[u][r] = exp2f(sc[u][r] - m_new);
    }
#pragma unroll
    for (int u = 0; u < SD_AHEAD; ++u) {
#pragma unroll
      for (int r = 0; r < REP; ++r) l[r] += sc[u][r];
#pragma unroll
      for (int p = 0; p < VR; ++p) {
        float f[N];
        unpack(vraw[u][p], f);
#pragma unroll
        for (int r = 0; r < REP; ++r)
#pragma unroll
          for (int e = 0; e < N; ++e) acc[r][p * N + e] += sc[u][r] * f[e];
      }
    }
  }
  // the lane groups of the warp
#pragma unroll
  for (int o = LPK; o < 32; o <<= 1) {
#pragma unroll
    for (int r = 0; r < REP; ++r) {
      const float m_o = __shfl_xor_sync(0xffffffffu, m[r], o), l_o = __shfl_xor_sync(0xffffffffu, l[r], o);
      const float m_new = fmaxf(m[r], m_o);
      const float ca = exp2f(m[r] - m_new), cb = exp2f(m_o - m_new);
      l[r] = l[r] * ca + l_o * cb;
#pragma unroll
      for (int e = 0; e < VR * N; ++e) acc[r][e] = acc[r][e] * ca + __shfl_xor_sync(0xffffffffu, acc[r][e], o) * cb;
      m[r] = m_new;
    }
  }
  if (kg == 0) {
#pragma unroll
    for (int r = 0; r < REP; ++r) {
#pragma unroll
      for (int p = 0; p < VR; ++p)
#pragma unroll
        for (int e = 0; e < N; ++e) part[warp][r][(p * LPK + sub) * N + e] = acc[r][p * N + e];
      if (sub == 0) { part[warp][r][DV] = m[r]; part[warp][r][DV + 1] = l[r]; }
    }
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < REP; ++r) {
    const int h = h0 + r;
    float mm = sink != nullptr ? sink[h] * LOG2E : -1e30f;
    const float sk = mm;
#pragma unroll
    for (int w = 0; w < SD_WARPS; ++w) mm = fmaxf(mm, part[w][r][DV]);
    float den = sink != nullptr ? exp2f(sk - mm) : 0.f;
    float cw[SD_WARPS];
#pragma unroll
    for (int w = 0; w < SD_WARPS; ++w) {
      cw[w] = exp2f(part[w][r][DV] - mm);
      den += cw[w] * part[w][r][DV + 1];
    }
    float gv = 1.f;
    if (gate != nullptr) gv = sigmoid_f(to_f(gate[t * ldg + h]));
    const float inv = gv / den;
    const size_t obase = (t * H + h) * DV;
    for (int c = threadIdx.x; c < DV; c += blockDim.x) {
      float o = 0.f;
#pragma unroll
      for (int w = 0; w < SD_WARPS; ++w) o += cw[w] * part[w][r][c];
      put_out(out, obase + c, o * inv, out_f32);
    }
  }
}

template <typename T, int LPK, int VR>
static void launch_sink_decode(int rep, cudaStream_t st, const void* q, const void* kc, const void* vc, void* out,
                               const int32_t* seq_start, const int32_t* seq_pos0, const int32_t* seq_len, const int32_t* bt,
                               int64_t bt_stride, const float* sink, const void* gate, int64_t ldg, int n_seqs, int H, int G, int Gv,
                               int page, int mask_kind, int mask, int keep_first, float softcap, float scale, int out_f32) {
#define SD_GO(REP) sink_attn_decode_kernel<T, LPK, REP, VR><<<dim3(H / REP, n_seqs), SD_WARPS * 32, 0, st>>>(static_cast<const T*>(q), \
      static_cast<const T*>(kc), static_cast<const T*>(vc), static_cast<T*>(out), seq_start, seq_pos0, seq_len, bt, bt_stride, sink, \
      static_cast<const T*>(gate), ldg, H, G, Gv, page, mask_kind, mask, keep_first, softcap, scale, out_f32)
  if constexpr (LPK * Vec16<T>::N * VR <= 128) {          // four heads' accumulators fit registers and shared memory
    if (rep % 4 == 0) { SD_GO(4); return; }
  }
  if (rep % 2 == 0) SD_GO(2);
  else SD_GO(1);
#undef SD_GO
}

// the row-splitting kernel takes d = LPK * (16 / sizeof(T)) with LPK in {4, 8, 16, 32} and dv = d or 2 d
template <typename T>
static bool launch_sink_decode_any(int d, int dv, int rep, cudaStream_t st, const void* q, const void* kc, const void* vc, void* out,
                                   const int32_t* seq_start, const int32_t* seq_pos0, const int32_t* seq_len, const int32_t* bt,
                                   int64_t bt_stride, const float* sink, const void* gate, int64_t ldg, int n_seqs, int H, int G, int Gv,
                                   int page, int mask_kind, int mask, int keep_first, float softcap, float scale, int out_f32) {
  constexpr int N = Vec16<T>::N;
  if ((dv != d && dv != 2 * d) || d % N != 0) return false;
  const bool wide = dv == 2 * d;
#define SD_ARGS rep, st, q, kc, vc, out, seq_start, seq_pos0, seq_len, bt, bt_stride, sink, gate, ldg, n_seqs, H, G, Gv, page, mask_kind, mask, keep_first, softcap, scale, out_f32
  switch (d / N) {
    case 4: if (wide) launch_sink_decode<T, 4, 2>(SD_ARGS); else launch_sink_decode<T, 4, 1>(SD_ARGS); return true;
    case 8: if (wide) launch_sink_decode<T, 8, 2>(SD_ARGS); else launch_sink_decode<T, 8, 1>(SD_ARGS); return true;
    case 16: if (wide) launch_sink_decode<T, 16, 2>(SD_ARGS); else launch_sink_decode<T, 16, 1>(SD_ARGS); return true;
    case 32: if (wide) launch_sink_decode<T, 32, 2>(SD_ARGS); else launch_sink_decode<T, 32, 1>(SD_ARGS); return true;
    default: return false;
  }
#undef SD_ARGS
}

// ------------------------------------------------------------------ prompt portions on the tensor cores (bf16)
// 64 query tokens of one head per CTA (4 warps x 16 rows); key tiles of 64 are gathered through the block table into
// padded shared-memory rows by 16-byte asynchronous copies, two stages deep.  S = Q K^T and O += P V run as m16n8k16 bf16
// MMAs with float accumulators in registers.  The softmax is the running one: a row keeps its maximum m and denominator
// l (both in the base-2 domain), rescales O when m grows, and the sink enters as the initial state m = sink, l = 1 with
// no value.  Weights are computed in float from the float scores and enter the second product as a bf16 pair hi + lo
// (lo = bf16(w - hi)), i.e. with 16 mantissa bits.  Both masks are a per-row lower bound lo(i) <= j <= i; tiles a warp
// cannot see are skipped, tiles it sees whole take a path without per-element tests.  With kept first keys, tiles over
// [0, min(F, lowest bound of the CTA)) run in front of the regular ones, and a regular tile that reaches below F is never
// skipped.
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void split_bf16(float x, float y, uint32_t& hi, uint32_t& lo) {
  hi = pack_bf16(x, y);
  lo = pack_bf16(x - bf16lo(hi), y - bf16hi(hi));
}

constexpr int SM_BM = 64, SM_BN = 64;

__device__ __forceinline__ int mask_lo(int i, int mask_kind, int mask) {
  if (mask <= 0) return 0;
  return mask_kind == 0 ? max(0, i - mask + 1) : (i / mask) * mask;
}

template <int D, int DV>
__global__ void __launch_bounds__(128)
sink_attn_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                     const __nv_bfloat16* __restrict__ v_cache, __nv_bfloat16* __restrict__ out,
                     const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_pos0,
                     const int32_t* __restrict__ seq_len, const int32_t* __restrict__ block_tables, int64_t bt_stride,
                     const float* __restrict__ sink, const __nv_bfloat16* __restrict__ gate, int64_t ldg, int H, int G, int Gv,
                     int page, int mask_kind, int mask, int keep_first, float softcap, float scale, int out_f32) {
  constexpr int QS = D + 8, VS = DV + 8;             // padded rows: 16-byte aligned, ldmatrix rows land in distinct banks
  constexpr float LOG2E = 1.4426950408889634f;
  extern __shared__ __align__(16) unsigned char sm_raw[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(sm_raw);        // [BM][QS]
  __nv_bfloat16* Ks = Qs + SM_BM * QS;                                 // [2][BN][QS]
  __nv_bfloat16* Vs = Ks + 2 * SM_BN * QS;                             // [2][BN][VS]
  const int b = blockIdx.z, h = blockIdx.y, g = h / (H / G), gv = g % Gv;
  const int len = seq_len[b];
  const int t0 = blockIdx.x * SM_BM;
  if (len <= 1 || t0 >= len) return;                 // one-token and padding rows belong to the plain kernel
  const int tid = threadIdx.x, lane = tid & 31, wr = tid >> 5;
  const int start = seq_start[b], pos0 = seq_pos0[b];
  const int32_t* bt = block_tables + static_cast<int64_t>(b) * bt_stride;
  for (int idx = tid; idx < SM_BM * (D / 8); idx += 128) {
    const int r = idx / (D / 8), ch = idx % (D / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (t0 + r < len) v = ldg_v4(q + (static_cast<size_t>(start + t0 + r) * H + h) * D + ch * 8);
    *reinterpret_cast<uint4*>(Qs + r * QS + ch * 8) = v;
  }
  const float scale2 = scale * LOG2E, cap2 = softcap * LOG2E;
  const int t_hi = min(len - 1, t0 + SM_BM - 1);
  const int j_lo = mask_lo(pos0 + t0, mask_kind, mask), j_hi = pos0 + t_hi;
  const int row_lo = wr * 16 + (lane >> 2);
  const int p_lo = pos0 + t0 + row_lo, p_hi = p_lo + 8;
  const bool ok_lo = t0 + row_lo < len, ok_hi = t0 + row_lo + 8 < len;
  const int lo_lo = mask_lo(p_lo, mask_kind, mask), lo_hi = mask_lo(p_hi, mask_kind, mask);
  const int wp_lo = pos0 + t0 + wr * 16, wp_hi = wp_lo + 15;
  const int w_first = mask_lo(wp_lo, mask_kind, mask), w_last = mask_lo(wp_hi, mask_kind, mask);
  float oacc[DV / 8][4];
#pragma unroll
  for (int i = 0; i < DV / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) oacc[i][e] = 0.f;
  // running maximum and (this thread's share of the) denominator of its two rows; the sink is counted by one lane of four
  float m0 = -1e30f, m1 = -1e30f, l0 = 0.f, l1 = 0.f;
  if (sink != nullptr) {
    m0 = m1 = sink[h] * LOG2E;
    if ((lane & 3) == 0) l0 = l1 = 1.f;
  }

  // two threads per key: the slot once, then the thread's 16-byte chunks lch, lch + 2, ... of the key's K and V rows
  const int lkey = tid >> 1, lch = tid & 1;
  // kept first keys that the lowest bound of the CTA hides: tiles of their own, in front of the regular ones
  const int pre_end = min(keep_first, j_lo), n_pre = (pre_end + SM_BN - 1) / SM_BN;
  auto tile_j0 = [&](int t) { return t < n_pre ? t * SM_BN : j_lo + (t - n_pre) * SM_BN; };
  auto load_tile = [&](int stage, int t) {
    const int j = tile_j0(t) + lkey;
    const bool ok = j <= (t < n_pre ? pre_end - 1 : j_hi);
    size_t slot = 0;
    if (ok) {
      const int pg = j / page;
      slot = static_cast<size_t>(bt[pg]) * page + (j - pg * page);
    }
    const __nv_bfloat16* ksrc = k_cache + (slot * G + g) * D + lch * 8;
    const __nv_bfloat16* vsrc = v_cache + (slot * Gv + gv) * DV + lch * 8;
    __nv_bfloat16* kd = Ks + (stage * SM_BN + lkey) * QS + lch * 8;
    __nv_bfloat16* vd = Vs + (stage * SM_BN + lkey) * VS + lch * 8;
#pragma unroll
    for (int i = 0; i < D / 16; ++i) cp_async_16(kd + i * 16, ksrc + i * 16, ok);
#pragma unroll
    for (int i = 0; i < DV / 16; ++i) cp_async_16(vd + i * 16, vsrc + i * 16, ok);
  };
  const int n_tiles = n_pre + (j_hi - j_lo) / SM_BN + 1;
  load_tile(0, 0);
  cp_async_commit();
  for (int t = 0; t < n_tiles; ++t) {
    const int j0 = tile_j0(t);
    const bool pre = t < n_pre;
    cp_async_wait<0>();
    __syncthreads();                                 // tile t has landed (Q too); tile t - 1 is consumed
    if (t + 1 < n_tiles) load_tile((t + 1) & 1, t + 1);
    cp_async_commit();
    const __nv_bfloat16* Kt = Ks + (t & 1) * SM_BN * QS;
    const __nv_bfloat16* Vt = Vs + (t & 1) * SM_BN * VS;
    if (t0 + wr * 16 >= len) continue;
    if (!pre && (j0 > wp_hi || (j0 + SM_BN - 1 < w_first && j0 >= keep_first))) continue;   // none of the warp's rows sees the tile
    float sacc[SM_BN / 8][4];
#pragma unroll
    for (int i = 0; i < SM_BN / 8; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) sacc[i][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t a[4];
      ldsm_x4(a[0], a[1], a[2], a[3], Qs + (wr * 16 + (lane & 15)) * QS + ks * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int np = 0; np < SM_BN / 16; ++np) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(b0, b1, b2, b3, Kt + (np * 16 + (lane >> 4) * 8 + (lane & 7)) * QS + ks * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16_16816(sacc[2 * np], a, b0, b1);
        mma_bf16_16816(sacc[2 * np + 1], a, b2, b3);
      }
    }
    const bool inner = !pre && j0 + SM_BN - 1 <= wp_lo && j0 >= w_last;
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < SM_BN / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float s = sacc[nt][e] * scale2;
        if (softcap > 0.f) s = cap2 * tanhf(s / cap2);
        if (!inner) {
          const int j = j0 + nt * 8 + 2 * (lane & 3) + (e & 1);
          bool ok;
          if (pre) ok = j < pre_end;                 // below every row's bound and position: seen by all, counted here only
          else ok = e < 2 ? (j <= p_lo && (j >= lo_lo || j < keep_first)) : (j <= p_hi && (j >= lo_hi || j < keep_first));
          if (!ok) s = -INFINITY;
        }
        sacc[nt][e] = s;
        if (e < 2) mx0 = fmaxf(mx0, s); else mx1 = fmaxf(mx1, s);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);      // finite: m starts finite
    const float c0 = ex2_approx(m0 - n0), c1 = ex2_approx(m1 - n1);
    m0 = n0; m1 = n1;
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < SM_BN / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float w = ex2_approx(sacc[nt][e] - (e < 2 ? n0 : n1));
        sacc[nt][e] = w;
        if (e < 2) s0 += w; else s1 += w;
      }
    }
    l0 = l0 * c0 + s0;
    l1 = l1 * c1 + s1;
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) { oacc[i][0] *= c0; oacc[i][1] *= c0; oacc[i][2] *= c1; oacc[i][3] *= c1; }
#pragma unroll
    for (int kk = 0; kk < SM_BN / 16; ++kk) {
      uint32_t ah[4], al[4];
      split_bf16(sacc[2 * kk][0], sacc[2 * kk][1], ah[0], al[0]);
      split_bf16(sacc[2 * kk][2], sacc[2 * kk][3], ah[1], al[1]);
      split_bf16(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1], ah[2], al[2]);
      split_bf16(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3], ah[3], al[3]);
#pragma unroll
      for (int np = 0; np < DV / 16; ++np) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(b0, b1, b2, b3, Vt + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * VS + np * 16 + (lane >> 4) * 8);
        mma_bf16_16816(oacc[2 * np], ah, b0, b1);
        mma_bf16_16816(oacc[2 * np], al, b0, b1);
        mma_bf16_16816(oacc[2 * np + 1], ah, b2, b3);
        mma_bf16_16816(oacc[2 * np + 1], al, b2, b3);
      }
    }
  }
  cp_async_wait<0>();
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    if (!(half ? ok_hi : ok_lo)) continue;
    const size_t row = static_cast<size_t>(start + t0 + row_lo + 8 * half);
    float inv = 1.0f / (half ? l1 : l0);
    if (gate != nullptr) inv *= sigmoid_f(__bfloat162float(gate[row * ldg + h]));
    const size_t obase = (row * H + h) * DV + 2 * (lane & 3);
    if (out_f32) {
      float* o = reinterpret_cast<float*>(out) + obase;
#pragma unroll
      for (int nt = 0; nt < DV / 8; ++nt)
        *reinterpret_cast<float2*>(o + nt * 8) = make_float2(oacc[nt][2 * half] * inv, oacc[nt][2 * half + 1] * inv);
    } else {
      __nv_bfloat16* o = out + obase;
#pragma unroll
      for (int nt = 0; nt < DV / 8; ++nt)
        *reinterpret_cast<uint32_t*>(o + nt * 8) = pack_bf16(oacc[nt][2 * half] * inv, oacc[nt][2 * half + 1] * inv);
    }
  }
}

template <int D, int DV>
static cudaError_t launch_sink_mma(int max_new, int n_seqs, cudaStream_t st, const void* q, const void* kc, const void* vc, void* out,
                                   const int32_t* seq_start, const int32_t* seq_pos0, const int32_t* seq_len, const int32_t* bt,
                                   int64_t bt_stride, const float* sink, const void* gate, int64_t ldg, int H, int G, int Gv, int page,
                                   int mask_kind, int mask, int keep_first, float softcap, float scale, int out_f32) {
  auto kern = sink_attn_mma_kernel<D, DV>;
  const size_t smem = sizeof(__nv_bfloat16) * ((SM_BM + 2 * SM_BN) * (D + 8) + 2 * SM_BN * (DV + 8));
  static bool opted = false;
  if (!opted) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    opted = true;
  }
  using B = __nv_bfloat16;
  const dim3 grid((max_new + SM_BM - 1) / SM_BM, H, n_seqs);
  kern<<<grid, 128, smem, st>>>(static_cast<const B*>(q), static_cast<const B*>(kc), static_cast<const B*>(vc), static_cast<B*>(out),
                                seq_start, seq_pos0, seq_len, bt, bt_stride, sink, static_cast<const B*>(gate), ldg, H, G, Gv, page,
                                mask_kind, mask, keep_first, softcap, scale, out_f32);
  return cudaSuccess;
}

// head sizes the tensor-core kernel is built for
static bool sink_mma_shape(int d, int dv) {
  return (d == 32 || d == 48 || d == 64 || d == 96 || d == 128) && (dv == 64 || dv == 128);
}

#define SINK_MMA_ARGS max_new, n_seqs, st, q, kc, vc, out, seq_start, seq_pos0, seq_len, bt, bt_stride, sink, gate, ldg, H, G, Gv, page, mask_kind, mask, keep_first, softcap, scale, out_f32
template <int D>
static cudaError_t launch_sink_mma_dv(int dv, int max_new, int n_seqs, cudaStream_t st, const void* q, const void* kc, const void* vc,
                                      void* out, const int32_t* seq_start, const int32_t* seq_pos0, const int32_t* seq_len,
                                      const int32_t* bt, int64_t bt_stride, const float* sink, const void* gate, int64_t ldg, int H,
                                      int G, int Gv, int page, int mask_kind, int mask, int keep_first, float softcap, float scale,
                                      int out_f32) {
  return dv == 64 ? launch_sink_mma<D, 64>(SINK_MMA_ARGS) : launch_sink_mma<D, 128>(SINK_MMA_ARGS);
}

}  // namespace row
}  // namespace b2

using namespace b2;
using namespace b2::row;

extern "C" int b2tts_sink_attn(const void* q, const void* k_cache, const void* v_cache, void* out, const int32_t* tok_seq,
                               const int32_t* positions, const int32_t* seq_start, const int32_t* seq_pos0, const int32_t* seq_len,
                               const int32_t* block_tables, int64_t bt_stride, const float* sink, const void* gate, int64_t ldg,
                               int n_tokens, int n_seqs, int max_new, int heads, int kv_heads, int v_heads, int dim, int vdim, int page,
                               int mask_kind, int mask, int keep_first, float softcap, float scale, int dtype, int path, int out_f32,
                               void* stream) {
  if (dtype == B2TTS_DTYPE_F32) out_f32 = 0;         // the outputs are floats already
  B2_REQUIRE(v_heads > 0 && kv_heads % v_heads == 0 && keep_first >= 0 && softcap >= 0.f, B2TTS_EINVAL,
             "sink_attn: bad switches (v_heads=%d of kv_heads=%d, keep_first=%d, softcap=%g)", v_heads, kv_heads, keep_first, softcap);
  if (mask <= 0) keep_first = 0;                     // nothing is hidden, nothing to keep
  B2_REQUIRE(n_tokens >= 0 && n_seqs >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dim > 0 && vdim > 0 && page > 0,
             B2TTS_EINVAL, "sink_attn: bad sizes (heads=%d kv_heads=%d dim=%d vdim=%d page=%d)", heads, kv_heads, dim, vdim, page);
  B2_REQUIRE(vdim <= 32 * SA_MAX_PER_LANE, B2TTS_EUNSUPPORTED, "sink_attn: value size %d above %d", vdim, 32 * SA_MAX_PER_LANE);
  B2_REQUIRE(heads <= 65535 && n_seqs <= 65535, B2TTS_EUNSUPPORTED, "sink_attn: %d heads, %d sequences", heads, n_seqs);
  B2_REQUIRE(mask_kind == 0 || mask_kind == 1, B2TTS_EINVAL, "sink_attn: mask kind %d", mask_kind);
  B2_REQUIRE(path >= 0 && path <= 2, B2TTS_EINVAL, "sink_attn: path %d", path);
  B2_REQUIRE(B2_ROW_DTYPE_OK(dtype), B2TTS_EINVAL, "sink_attn: dtype %d", dtype);
  if (n_tokens == 0 || n_seqs == 0) return B2TTS_OK;
  B2_REQUIRE(q && k_cache && v_cache && out && tok_seq && positions && seq_start && seq_pos0 && seq_len && block_tables, B2TTS_EINVAL,
             "sink_attn: null pointer");
  B2_REQUIRE(aligned16(k_cache) && aligned16(v_cache), B2TTS_EALIGN, "sink_attn: caches must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool mma_ok = dtype == B2TTS_DTYPE_BF16 && sink_mma_shape(dim, vdim) && aligned16(q) && aligned16(out);
  B2_REQUIRE(path != 2 || mma_ok, B2TTS_EUNSUPPORTED, "sink_attn: the tensor-core kernel takes bf16 with head sizes 32..128 / 64, 128");
  const bool use_mma = mma_ok && path != 1 && max_new > 1;
  if (use_mma) {
    const int H = heads, G = kv_heads, Gv = v_heads;
    const void* kc = k_cache; const void* vc = v_cache; const int32_t* bt = block_tables;
    cudaError_t e;
    switch (dim) {
      case 32: e = launch_sink_mma_dv<32>(vdim, SINK_MMA_ARGS); break;
      case 48: e = launch_sink_mma_dv<48>(vdim, SINK_MMA_ARGS); break;
      case 64: e = launch_sink_mma_dv<64>(vdim, SINK_MMA_ARGS); break;
      case 96: e = launch_sink_mma_dv<96>(vdim, SINK_MMA_ARGS); break;
      default: e = launch_sink_mma_dv<128>(vdim, SINK_MMA_ARGS); break;
    }
    if (e != cudaSuccess) return cuda_fail(e, "sink_attn (tensor cores)");
    B2_CHECK_LAUNCH("sink_attn (tensor cores)");
  }
  // one-token rows: the row-splitting kernel where the head size fits it (path 1 keeps everything in the plain kernel)
  bool split = false;
  if (path != 1 && aligned16(q) && n_seqs > 0) {
    if (dtype == B2TTS_DTYPE_BF16)
      split = launch_sink_decode_any<__nv_bfloat16>(dim, vdim, heads / kv_heads, st, q, k_cache, v_cache, out, seq_start, seq_pos0, seq_len,
                                                    block_tables, bt_stride, sink, gate, ldg, n_seqs, heads, kv_heads, v_heads, page, mask_kind,
                                                    mask, keep_first, softcap, scale, out_f32);
    else
      split = launch_sink_decode_any<float>(dim, vdim, heads / kv_heads, st, q, k_cache, v_cache, out, seq_start, seq_pos0, seq_len,
                                            block_tables, bt_stride, sink, gate, ldg, n_seqs, heads, kv_heads, v_heads, page, mask_kind, mask,
                                            keep_first, softcap, scale, out_f32);
    if (split) B2_CHECK_LAUNCH("sink_attn (one-token rows)");
  }
  const int skip = (use_mma ? 1 : 0) | (split ? 2 : 0);
  if (dtype == B2TTS_DTYPE_BF16)
    launch_sink_plain_rep<__nv_bfloat16>(heads / kv_heads, st, q, k_cache, v_cache, out, tok_seq, positions, seq_len, block_tables,
                                         bt_stride, sink, gate, ldg, n_tokens, heads, kv_heads, v_heads, dim, vdim, page, mask_kind, mask,
                                         keep_first, softcap, scale, skip, out_f32);
  else
    launch_sink_plain_rep<float>(heads / kv_heads, st, q, k_cache, v_cache, out, tok_seq, positions, seq_len, block_tables, bt_stride,
                                 sink, gate, ldg, n_tokens, heads, kv_heads, v_heads, dim, vdim, page, mask_kind, mask, keep_first,
                                 softcap, scale, skip, out_f32);
  B2_CHECK_LAUNCH("sink_attn");
  return B2TTS_OK;
}
