// latent_attn.cu - attention over a paged cache of LATENTS: every cached row is [c (r numbers) | kr (dr numbers)], one
// row per token shared by all heads.  Head h's key is [W_uk,h c | kr] and its value W_uv,h c; both expansions are moved
// out of the loop over keys: the caller multiplies the un-rotated query part by W_uk,h^T once ("absorbed" query
// ql [r]) and applies W_uv,h to the attention-weighted sum of latents afterwards, so that the kernel is multi-query
// attention with key [c | kr] and value c:
//
//   s_ij = scale * (ql_i . c_j + rot(qr_i) . kr_j),   j visible from i:  0 <= i - j (< window, if window > 0)
//   o_i  = sum_j exp(s_ij - m) c_j / (exp(sink_h - m) + sum_j exp(s_ij - m))          (a sink: a slot with no key or value)
//
// The rotated query part is turned here (pairs (2k, 2k+1), angle position * freq[k], cos and sin times rot_mult); the
// keys were turned when they were written.  Scores, weights, maxima and sums are float.  One launch serves a mixed step:
// rows of prompt portions and single decoded tokens, each reading its keys through its sequence's block table.
#include <math.h>

#include "common.cuh"

namespace b2 {
namespace lat {

template <typename T> __device__ __forceinline__ float a_to_f(T v);
template <> __device__ __forceinline__ float a_to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float a_to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T a_from_f(float v);
template <> __device__ __forceinline__ float a_from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 a_from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T> __device__ __forceinline__ float dot_chunk(const uint4& v, const float* q);
template <> __device__ __forceinline__ float dot_chunk<float>(const uint4& v, const float* q) {
  return __uint_as_float(v.x) * q[0] + __uint_as_float(v.y) * q[1] + __uint_as_float(v.z) * q[2] + __uint_as_float(v.w) * q[3];
}
template <> __device__ __forceinline__ float dot_chunk<__nv_bfloat16>(const uint4& v, const float* q) {
  // a bf16 is the upper half of a float
  return __uint_as_float(v.x << 16) * q[0] + __uint_as_float(v.x & 0xffff0000u) * q[1] +
         __uint_as_float(v.y << 16) * q[2] + __uint_as_float(v.y & 0xffff0000u) * q[3] +
         __uint_as_float(v.z << 16) * q[4] + __uint_as_float(v.z & 0xffff0000u) * q[5] +
         __uint_as_float(v.w << 16) * q[6] + __uint_as_float(v.w & 0xffff0000u) * q[7];
}

struct LatentAttnArgs {
  const void* ql; int64_t ql_tok, ql_head;      // absorbed queries [.., r]
  const void* qr; int64_t qr_tok, qr_head;      // un-rotated rotary query parts [.., dr]
  const void* cache;                            // [pages * page, r + dr]
  void* out; int64_t o_tok, o_head;             // weighted latent sums [.., r]
  const float* sink;                            // [H], or null: no sink, an ordinary softmax
  const float* freq; float rot_mult; int rot_dims;
  const int32_t *seq_start, *seq_pos0, *seq_len, *block_tables; int64_t bt_stride;
  int n_seqs, max_new, H, r, dr, page, window;
  float scale;
  int ql_vec;                                    // tensor-core kernel: ql rows, plain kernel: cache rows can be read 16 bytes at a time
  int splits; float* ws;                         // key ranges per query tile (tensor-core kernel, decode steps) and their partial results
};

// ------------------------------------------------------------------ plain kernel (any size, bf16 or float)
// One warp per (token, head).  A batch of 32 keys: lane l scores key l (dot product over the whole row, the query in
// shared memory as floats), then the lanes turn to the latent's coordinates and add the 32 weighted rows.
constexpr int LA_WARPS = 4;
constexpr int LA_MAX_R_PER_LANE = 32;           // latents up to 1024 numbers

template <typename T>
__global__ void __launch_bounds__(LA_WARPS * 32)
latent_attn_kernel(const LatentAttnArgs a) {
  extern __shared__ float q_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int b = blockIdx.y;
  const int len = a.seq_len[b];
  const int row = blockIdx.x * LA_WARPS + warp;
  const int tl = row / a.H, h = row % a.H;
  if (tl >= len) return;
  const int Dk = a.r + a.dr;
  float* q = q_smem + warp * Dk;
  const int tok = a.seq_start[b] + tl;
  const int pos = a.seq_pos0[b] + tl;
  const T* ql = static_cast<const T*>(a.ql) + tok * a.ql_tok + h * a.ql_head;
  const T* qr = static_cast<const T*>(a.qr) + tok * a.qr_tok + h * a.qr_head;
  for (int c = lane; c < a.r; c += 32) q[c] = a_to_f(ql[c]) * a.scale;
  for (int i = lane; i < (a.dr + 1) / 2; i += 32) {
    const int c0 = 2 * i, c1 = 2 * i + 1;
    const float u = a_to_f(qr[c0]);
    const float v = c1 < a.dr ? a_to_f(qr[c1]) : 0.f;
    if (c1 < a.rot_dims) {
      float sn, cs;
      sincosf(static_cast<float>(pos) * a.freq[i], &sn, &cs);
      sn *= a.rot_mult; cs *= a.rot_mult;
      q[a.r + c0] = (u * cs - v * sn) * a.scale;
      q[a.r + c1] = (v * cs + u * sn) * a.scale;
    } else {
      q[a.r + c0] = u * a.scale;
      if (c1 < a.dr) q[a.r + c1] = v * a.scale;
    }
  }
  __syncwarp();
  const int32_t* bt = a.block_tables + b * a.bt_stride;
  const T* cache = static_cast<const T*>(a.cache);
  const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  float m = -1.0e30f, l = 0.f;
  if (a.sink != nullptr) { m = a.sink[h]; l = 1.0f; }   // the sink: exp(sink - m) with m = sink; none: an ordinary softmax
  float o[LA_MAX_R_PER_LANE];
#pragma unroll
  for (int i = 0; i < LA_MAX_R_PER_LANE; ++i) o[i] = 0.f;
  for (int j0 = lo; j0 <= pos; j0 += 32) {
    const int j = j0 + lane;
    const bool ok = j <= pos;
    size_t slot = 0;
    float s = -INFINITY;
    if (ok) {
      slot = static_cast<size_t>(bt[j / a.page]) * a.page + j % a.page;
      const T* kr = cache + slot * Dk;
      float acc = 0.f;
      if (a.ql_vec) {                              // rows of whole 16-byte chunks: 8 bf16 or 4 floats per load
        constexpr int PER = 16 / static_cast<int>(sizeof(T));
        const uint4* k4 = reinterpret_cast<const uint4*>(kr);
        for (int c4 = 0; c4 < Dk / PER; ++c4) acc += dot_chunk<T>(k4[c4], q + c4 * PER);
      } else {
        for (int c = 0; c < Dk; ++c) acc += q[c] * a_to_f(kr[c]);
      }
      s = acc;
    }
    const float mn = fmaxf(m, warp_max(s));
    const float alpha = expf(m - mn);
    const float p = ok ? expf(s - mn) : 0.f;
    l = l * alpha + warp_sum(p);
    m = mn;
#pragma unroll
    for (int i = 0; i < LA_MAX_R_PER_LANE; ++i) o[i] *= alpha;
    const int nk = min(32, pos - j0 + 1);
    for (int jj = 0; jj < nk; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const size_t sj = __shfl_sync(0xffffffffu, slot, jj);
      const T* vr = cache + sj * Dk;
#pragma unroll
      for (int i = 0; i < LA_MAX_R_PER_LANE; ++i) {
        const int c = i * 32 + lane;
        if (c < a.r) o[i] += pj * a_to_f(vr[c]);
      }
    }
  }
  T* orow = static_cast<T*>(a.out) + tok * a.o_tok + h * a.o_head;
  const float inv = 1.0f / l;
#pragma unroll
  for (int i = 0; i < LA_MAX_R_PER_LANE; ++i) {
    const int c = i * 32 + lane;
    if (c < a.r) orow[c] = a_from_f<T>(o[i] * inv);
  }
}


// ------------------------------------------------------------------ tensor-core kernel (bf16)
// A CTA owns 16 query rows: G consecutive tokens of one sequence times up to 16 heads (G = 16 / heads when a sequence
// has fewer than 16 heads; a decoded token is a tile with one token).  All rows read the SAME cached rows, so a tile of
// 64 keys is staged once in shared memory ([key][c | kr], two stages filled by 16-byte asynchronous copies through the
// block table) and used twice: as the key operand of S = Q K^T (each warp scores its own 8 or 16 keys over the whole
// row width) and, its first r columns read transposed, as the value operand of O += P V (each warp owns r / NW
// columns of O in registers).  Between the two products the 16 x 64 scores cross shared memory as floats, where the
// running maximum, the sum and the weights are formed in float (the sink starts the maximum and the sum).
constexpr int LM_KT = 64;                       // keys per tile

__device__ __forceinline__ void ldsm_x2(uint32_t& r0, uint32_t& r1, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x2_t(uint32_t& r0, uint32_t& r1, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(smem_u32(p)));
}

// the same with 32-bit shared-space addresses, so that unrolled offsets fold into the instructions
__device__ __forceinline__ void ldsm_x4_a(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2_a(uint32_t& r0, uint32_t& r1, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2_t_a(uint32_t& r0, uint32_t& r1, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}

// How often a wait for a key tile ran out (it never should: the copies are this CTA's own); read by b2tts_latent_attn_timeouts().
__device__ int g_latent_attn_timeouts = 0;

// Wait for phase `parity` of an mbarrier, giving up after a bounded number of polls.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (int i = 0; i < (1 << 20); ++i) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}

struct LatentMmaSmem {
  int q_off, k_off, s_off, p_off, st_off, total, ldk;   // byte offsets; ldk = padded row length in elements
};
static LatentMmaSmem latent_mma_smem(int r, int dr, int stages = 2) {
  LatentMmaSmem m;
  const int dkp = (r + dr + 15) / 16 * 16;
  m.ldk = dkp + 8;
  m.q_off = 0;
  m.k_off = 16 * m.ldk * 2;
  m.s_off = m.k_off + stages * LM_KT * m.ldk * 2;
  m.p_off = m.s_off + 16 * LM_KT * 4;
  m.st_off = m.p_off + 16 * (LM_KT + 8) * 2;
  m.total = m.st_off + 16 * 4 * 4 + 2 * 8;      // row statistics, then one mbarrier per key stage
  return m;
}

// KSMAX > 0: two key stages and the query fragments in registers (one CTA per SM).  KSMAX == 0: one key stage, query
// fragments re-read from shared memory, half the registers - two CTAs share an SM and cover each other's waits.
template <int NW, int NT, int KSMAX>
__global__ void __launch_bounds__(NW * 32, KSMAX == 0 ? 2 : 1)
latent_attn_mma_kernel(const LatentAttnArgs a, const LatentMmaSmem sm) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw + sm.q_off);
  __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(smem_raw + sm.k_off);
  float* ss = reinterpret_cast<float*>(smem_raw + sm.s_off);
  __nv_bfloat16* ps = reinterpret_cast<__nv_bfloat16*>(smem_raw + sm.p_off);
  float* row_m = reinterpret_cast<float*>(smem_raw + sm.st_off);
  float* row_l = row_m + 16;
  float* row_alpha = row_l + 16;
  int* row_pos = reinterpret_cast<int*>(row_alpha + 16);
  constexpr int LDP = LM_KT + 8, SN = LM_KT / 8 / NW;      // SN: score n-tiles per warp
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int ldk = sm.ldk, dkp = ldk - 8, Dk = a.r + a.dr;
  const int b = blockIdx.y;
  const int len = a.seq_len[b];
  const int hpc = min(a.H, 16), hblocks = (a.H + 15) / 16, G = 16 / hpc;
  const int tile = blockIdx.x / hblocks, hb = blockIdx.x % hblocks;
  const int tl0 = tile * G;
  if (tl0 >= len) return;
  const int pos0 = a.seq_pos0[b], start = a.seq_start[b];
  const int n_tok = min(G, len - tl0);
  const int pos_first = pos0 + tl0, pos_last = pos_first + n_tok - 1;
  const __nv_bfloat16* cache = static_cast<const __nv_bfloat16*>(a.cache);
  const int32_t* bt = a.block_tables + b * a.bt_stride;
  const int j_lo = a.window > 0 ? max(0, pos_first - a.window + 1) : 0;
  const int n_tiles = (pos_last - j_lo) / LM_KT + 1;
  // with splits > 1, CTA z of a query tile takes the z-th run of key tiles and leaves (O, m, l) for the merge kernel
  const int tps = (n_tiles + a.splits - 1) / a.splits;
  const int t_begin = blockIdx.z * tps, t_end = min(n_tiles, t_begin + tps);

  // Key tiles arrive by bulk copies (the TMA unit: no load instructions, no registers, whole rows of r + dr numbers),
  // one per key, issued by the first 64 / NW lanes of every warp and counted on the stage's mbarrier.  Lane i owns the
  // i-th key of its warp's share; its table lookup runs one tile ahead of the copy.  Keys past the last query repeat
  // the last key (finite numbers; their weights are zero), so a tile is always 64 whole rows.
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + sm.st_off + 16 * 4 * 4);
  constexpr int STAGES = KSMAX > 0 ? 2 : 1;
  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < STAGES; ++i) mbar_init(&bars[i], 1);
    mbar_fence_init();
  }
  if (dkp > Dk)                                   // the padding chunk after every row is never copied to: zero it once
    for (int i = tid; i < STAGES * LM_KT; i += NW * 32) *reinterpret_cast<uint4*>(ks + i * ldk + Dk) = make_uint4(0u, 0u, 0u, 0u);
  __syncthreads();
  auto lookup = [&](int t) -> long long {
    long long off = -1;
    if (lane < LM_KT / NW && t < t_end) {
      const int j = min(j_lo + t * LM_KT + warp + lane * NW, pos_last);
      off = (static_cast<long long>(bt[j / a.page]) * a.page + j % a.page) * Dk;
    }
    return off;
  };
  const uint32_t ks_u = smem_u32(ks), ps_u = smem_u32(ps);
  const uint32_t row_bytes = static_cast<uint32_t>(Dk) * 2u;
  auto load_tile = [&](long long my, int stage) {
    if (tid == 0) mbar_expect_tx(&bars[stage], LM_KT * row_bytes);
    if (my >= 0) bulk_g2s(ks + (stage * LM_KT + warp + lane * NW) * ldk, cache + my, row_bytes, &bars[stage]);
  };
  long long slots_next = lookup(t_begin);
  if (t_begin < t_end) {
    load_tile(slots_next, 0);
    slots_next = lookup(t_begin + 1);
  }

  // ---- the 16 query rows: [ql | rotate(qr)] as bf16, zero rows where the tile has no token or head
  if (tid < 16) {
    const int tl = tid / hpc, h = hb * 16 + tid % hpc;
    const bool ok = tl < n_tok && h < a.H;
    row_pos[tid] = ok ? pos_first + tl : -1;
    // the sink counts once: the first split starts from it (m = sink, l = exp(sink - m) = 1), the others from nothing
    const bool sunk = blockIdx.z == 0 && a.sink != nullptr;
    row_m[tid] = ok && sunk ? a.sink[h] : -1.0e30f;
    row_l[tid] = sunk ? 1.0f : 0.f;
  }
  {
    // a warp stages rows warp, warp + NW, ..: first every load of its rows is issued (16 bytes of ql per lane and step,
    // one pair of qr per lane), then the rows are written, so one round trip to memory covers them all
    constexpr int ROWS = 16 / NW, QV = 4;                                  // QV steps of 32 x 8 numbers: latents up to 1024
    const bool vec = a.ql_vec;
    uint4 qv[ROWS][QV];
    float2 rv[ROWS][2];
#pragma unroll
    for (int k = 0; k < ROWS; ++k) {
      const int row = warp + k * NW;
      const int tl = row / hpc, h = hb * 16 + row % hpc;
      const bool ok = tl < n_tok && h < a.H;
      const int tok = start + tl0 + tl;
      const __nv_bfloat16* ql = static_cast<const __nv_bfloat16*>(a.ql) + tok * a.ql_tok + h * a.ql_head;
      const __nv_bfloat16* qr = static_cast<const __nv_bfloat16*>(a.qr) + tok * a.qr_tok + h * a.qr_head;
#pragma unroll
      for (int v = 0; v < QV; ++v) {
        const int c = (v * 32 + lane) * 8;
        qv[k][v] = make_uint4(0u, 0u, 0u, 0u);
        if (ok && c < a.r) {
          if (vec) qv[k][v] = *reinterpret_cast<const uint4*>(ql + c);
          else {
            const unsigned short* q16 = reinterpret_cast<const unsigned short*>(ql + c);
            qv[k][v] = make_uint4(q16[0] | (q16[1] << 16), q16[2] | (q16[3] << 16), q16[4] | (q16[5] << 16), q16[6] | (q16[7] << 16));
          }
        }
      }
#pragma unroll
      for (int v = 0; v < 2; ++v) {
        const int d = (v * 32 + lane) * 2;
        rv[k][v] = make_float2(0.f, 0.f);
        if (ok && d < a.dr) rv[k][v] = make_float2(__bfloat162float(qr[d]), __bfloat162float(qr[d + 1]));
      }
    }
#pragma unroll
    for (int k = 0; k < ROWS; ++k) {
      const int row = warp + k * NW;
      const int tl = row / hpc;
#pragma unroll
      for (int v = 0; v < QV; ++v) {
        const int c = (v * 32 + lane) * 8;
        if (c < a.r) *reinterpret_cast<uint4*>(qs + row * ldk + c) = qv[k][v];
      }
#pragma unroll
      for (int v = 0; v < 2; ++v) {
        const int d = (v * 32 + lane) * 2;
        if (d < dkp - a.r) {                                               // the rotary part and the zero padding after it
          float v0 = rv[k][v].x, v1 = rv[k][v].y;
          if (d + 1 < a.rot_dims) {
            float sn, cs;
            sincosf(static_cast<float>(pos_first + tl) * a.freq[d / 2], &sn, &cs);
            sn *= a.rot_mult; cs *= a.rot_mult;
            const float u = v0, w = v1;
            v0 = u * cs - w * sn;
            v1 = w * cs + u * sn;
          }
          *reinterpret_cast<__nv_bfloat162*>(qs + row * ldk + a.r + d) = __floats2bfloat162_rn(v0, v1);
        }
      }
    }
  }

  // every warp keeps the whole query tile as MMA fragments in registers (KSMAX k-steps of 16): the score product then
  // reads only key rows from shared memory, whose bandwidth is what bounds it otherwise
  __syncthreads();
  constexpr bool QREG = KSMAX > 0;
  uint32_t qf[QREG ? KSMAX : 1][4];
  if (QREG) {
#pragma unroll
    for (int u = 0; u < KSMAX; ++u) {
      if (u * 16 < dkp) ldsm_x4_a(qf[u], smem_u32(qs) + static_cast<uint32_t>((lane & 15) * ldk + (lane >> 4) * 8) * 2u + u * 32u);
      else qf[u][0] = qf[u][1] = qf[u][2] = qf[u][3] = 0u;
    }
  }
  const uint32_t q_lane = smem_u32(qs) + static_cast<uint32_t>((lane & 15) * ldk + (lane >> 4) * 8) * 2u;

  float acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
  const int col0 = warp * NT * 8;                                   // this warp's columns of O

  for (int t = t_begin; t < t_end; ++t) {
    const int stage = QREG ? (t - t_begin) & 1 : 0;
    if (QREG && t + 1 < t_end) {
      load_tile(slots_next, stage ^ 1);
      slots_next = lookup(t + 2);
    }
    const int use = QREG ? (t - t_begin) >> 1 : t - t_begin;      // how often this stage has been filled before
    const bool arrived = mbar_wait_bounded(&bars[stage], use & 1);
    if (__syncthreads_or(!arrived)) {              // never expected; all threads leave together
      if (tid == 0) atomicAdd(&g_latent_attn_timeouts, 1);
      break;
    }
    // ---- S = Q K^T for this warp's keys
    float sc[SN][4][4];                          // four accumulators per n-tile: the k-steps of a group do not wait on each other
#pragma unroll
    for (int i = 0; i < SN; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) sc[i][0][e] = sc[i][1][e] = sc[i][2][e] = sc[i][3][e] = 0.f;
    const uint32_t kt_u = ks_u + static_cast<uint32_t>(stage * LM_KT * ldk) * 2u;
    const uint32_t k_lane = kt_u + static_cast<uint32_t>((warp * SN * 8 + (lane & 7)) * ldk + ((lane >> 3) & 1) * 8) * 2u;
    if (QREG) {
#pragma unroll
      for (int u0 = 0; u0 < KSMAX; u0 += 4) {    // the key fragments of four k-steps are in flight before their products
        if (u0 * 16 < dkp) {
          uint32_t bf[4][SN][2];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if ((u0 + u) * 16 < dkp) {
#pragma unroll
              for (int i = 0; i < SN; ++i) ldsm_x2_a(bf[u][i][0], bf[u][i][1], k_lane + static_cast<uint32_t>(i * 8 * ldk) * 2u + (u0 + u) * 32u);
            }
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if ((u0 + u) * 16 < dkp) {
#pragma unroll
              for (int i = 0; i < SN; ++i) mma_bf16_16816(sc[i][u], qf[QREG ? u0 + u : 0], bf[u][i][0], bf[u][i][1]);
            }
          }
        }
      }
    } else {
      for (int k0 = 0; k0 < dkp; k0 += 64) {
        uint32_t af[4][4], bf[4][SN][2];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (k0 + 16 * u < dkp) {
            ldsm_x4_a(af[u], q_lane + (k0 + 16 * u) * 2u);
#pragma unroll
            for (int i = 0; i < SN; ++i) ldsm_x2_a(bf[u][i][0], bf[u][i][1], k_lane + static_cast<uint32_t>(i * 8 * ldk) * 2u + (k0 + 16 * u) * 2u);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (k0 + 16 * u < dkp) {
#pragma unroll
            for (int i = 0; i < SN; ++i) mma_bf16_16816(sc[i][u], af[u], bf[u][i][0], bf[u][i][1]);
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < SN; ++i) {
      const int n0 = (warp * SN + i) * 8 + (lane & 3) * 2, r0 = lane >> 2;
      ss[r0 * LM_KT + n0] = (sc[i][0][0] + sc[i][1][0]) + (sc[i][2][0] + sc[i][3][0]);
      ss[r0 * LM_KT + n0 + 1] = (sc[i][0][1] + sc[i][1][1]) + (sc[i][2][1] + sc[i][3][1]);
      ss[(r0 + 8) * LM_KT + n0] = (sc[i][0][2] + sc[i][1][2]) + (sc[i][2][2] + sc[i][3][2]);
      ss[(r0 + 8) * LM_KT + n0 + 1] = (sc[i][0][3] + sc[i][1][3]) + (sc[i][2][3] + sc[i][3][3]);
    }
    __syncthreads();
    // ---- running maximum, sum and weights, in float; a warp takes rows warp, warp + NW, ..
    for (int r2 = 2 * warp; r2 < 16; r2 += 2 * NW) {       // half a warp per row, four keys per lane
      const int row = r2 + (lane >> 4), l16 = lane & 15;
      const int rp = row_pos[row];
      float sv[4];
      float mx = -INFINITY;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int kk = l16 + 16 * e;
        const int j = j_lo + t * LM_KT + kk;
        const bool vis = j <= rp && (a.window == 0 || rp - j < a.window);
        sv[e] = vis ? ss[row * LM_KT + kk] * a.scale : -INFINITY;
        mx = fmaxf(mx, sv[e]);
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_old = row_m[row];
      const float m_new = fmaxf(m_old, mx);
      float sum = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pe = expf(sv[e] - m_new);                                  // exp(-inf) = 0 for hidden keys
        sum += pe;
        ps[row * LDP + l16 + 16 * e] = __float2bfloat16_rn(pe);
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      __syncwarp();
      if (l16 == 0) {
        const float alpha = expf(m_old - m_new);
        row_m[row] = m_new;
        row_l[row] = row_l[row] * alpha + sum;
        row_alpha[row] = alpha;
      }
    }
    __syncthreads();
    // ---- O = O * alpha + P V, V = the first r columns of the key tile
    {
      const float a0 = row_alpha[lane >> 2], a1 = row_alpha[(lane >> 2) + 8];
#pragma unroll
      for (int i = 0; i < NT; ++i) { acc[i][0] *= a0; acc[i][1] *= a0; acc[i][2] *= a1; acc[i][3] *= a1; }
      const uint32_t p_lane = ps_u + static_cast<uint32_t>((lane & 15) * LDP + (lane >> 4) * 8) * 2u;
      const uint32_t v_lane = kt_u + static_cast<uint32_t>((lane & 15) * ldk + col0) * 2u;
      const uint32_t v_step = static_cast<uint32_t>(16 * ldk) * 2u;
#pragma unroll
      for (int kk = 0; kk < LM_KT / 16; ++kk) {
        uint32_t pf[4];
        ldsm_x4_a(pf, p_lane + kk * 32u);
        uint32_t vb[NT][2];
#pragma unroll
        for (int i = 0; i < NT; ++i) ldsm_x2_t_a(vb[i][0], vb[i][1], v_lane + kk * v_step + i * 16u);
#pragma unroll
        for (int i = 0; i < NT; ++i) mma_bf16_16816(acc[i], pf, vb[i][0], vb[i][1]);
      }
    }
    __syncthreads();
    if (!QREG && t + 1 < t_end) {                 // one stage: the next tile may only land once everyone is done with this one
      load_tile(slots_next, 0);
      slots_next = lookup(t + 2);
    }
  }
  if (a.splits > 1) {
    // ---- partial result of this key range: un-normalised O, then m and l, per row
    __syncthreads();                               // row_m / row_l of the last tile (and of a CTA with no tile at all)
    float* wrow = a.ws + ((static_cast<size_t>(b) * gridDim.x + blockIdx.x) * a.splits + blockIdx.z) * 16 * (a.r + 2);
    const int r0 = lane >> 2;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float* w = wrow + static_cast<size_t>(r0 + 8 * half) * (a.r + 2);
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        const int c = col0 + i * 8 + (lane & 3) * 2;
        w[c] = acc[i][2 * half];
        w[c + 1] = acc[i][2 * half + 1];
      }
    }
    if (tid < 16) {
      wrow[static_cast<size_t>(tid) * (a.r + 2) + a.r] = row_m[tid];
      wrow[static_cast<size_t>(tid) * (a.r + 2) + a.r + 1] = row_l[tid];
    }
    return;
  }
  // ---- out = O / l
  {
    const int r0 = lane >> 2;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = r0 + 8 * half;
      if (row_pos[row] < 0) continue;
      const int tl = row / hpc, h = hb * 16 + row % hpc;
      const float inv = 1.0f / row_l[row];
      __nv_bfloat16* orow = static_cast<__nv_bfloat16*>(a.out) + (start + tl0 + tl) * a.o_tok + h * a.o_head;
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        const int c = col0 + i * 8 + (lane & 3) * 2;
        orow[c] = __float2bfloat16_rn(acc[i][2 * half] * inv);
        orow[c + 1] = __float2bfloat16_rn(acc[i][2 * half + 1] * inv);
      }
    }
  }
}

// Merge of the key ranges of one query row: out = sum_z O_z e^(m_z - M) / sum_z l_z e^(m_z - M), M = max_z m_z.
// grid (query tiles, sequences, 16 rows).
__global__ void __launch_bounds__(128)
latent_attn_merge_kernel(const LatentAttnArgs a) {
  const int b = blockIdx.y, row = blockIdx.z;
  const int len = a.seq_len[b];
  const int hpc = min(a.H, 16), hblocks = (a.H + 15) / 16, G = 16 / hpc;
  const int tile = blockIdx.x / hblocks, hb = blockIdx.x % hblocks;
  const int tl0 = tile * G;
  const int tl = row / hpc, h = hb * 16 + row % hpc;
  if (tl0 + tl >= len || tl >= G || h >= a.H) return;
  const int stride = 16 * (a.r + 2);
  const float* w = a.ws + (static_cast<size_t>(b) * gridDim.x + blockIdx.x) * a.splits * stride + static_cast<size_t>(row) * (a.r + 2);
  float M = -1.0e30f;
  for (int z = 0; z < a.splits; ++z) M = fmaxf(M, w[z * stride + a.r]);
  float L = 0.f;
  for (int z = 0; z < a.splits; ++z) L += w[z * stride + a.r + 1] * expf(w[z * stride + a.r] - M);
  const float inv = 1.0f / L;
  __nv_bfloat16* orow = static_cast<__nv_bfloat16*>(a.out) + (a.seq_start[b] + tl0 + tl) * a.o_tok + h * a.o_head;
  for (int c = threadIdx.x; c < a.r; c += blockDim.x) {
    float o = 0.f;
    for (int z = 0; z < a.splits; ++z) o += w[z * stride + c] * expf(w[z * stride + a.r] - M);
    orow[c] = __float2bfloat16_rn(o * inv);
  }
}

template <int NW, int NT, int KSMAX>
static cudaError_t launch_latent_mma(const LatentAttnArgs& a, const LatentMmaSmem& sm_in, dim3 grid, cudaStream_t st) {
  auto kern = latent_attn_mma_kernel<NW, NT, KSMAX>;
  const LatentMmaSmem sm = KSMAX == 0 ? latent_mma_smem(a.r, a.dr, 1) : sm_in;
  if (sm.total > 48 * 1024) {
    static bool raised = false;                  // one attribute per kernel instance: raise it to the device's limit once
    if (!raised) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
      if (e != cudaSuccess) return e;
      raised = true;
    }
  }
  kern<<<grid, NW * 32, sm.total, st>>>(a, sm);
  return cudaSuccess;
}

// Sizes the tensor-core kernel takes: r a multiple of 32 (four or eight warps own whole 8-column tiles of O, at most
// eight each), dr a multiple of 8, everything addressable by 16-byte copies, one tile pair within shared memory.
static bool latent_mma_fits(const LatentAttnArgs& a, int* nw, int* nt) {
  if (a.r % 8 || a.dr % 8) return false;
  const int tiles = a.r / 8;
  if (tiles % 8 == 0 && tiles / 8 <= 8) { *nw = 8; *nt = tiles / 8; }
  else if (tiles % 4 == 0 && tiles / 4 <= 8) { *nw = 4; *nt = tiles / 4; }
  else return false;
  if (latent_mma_smem(a.r, a.dr).total > 220 * 1024 || (a.r + a.dr + 15) / 16 > 40) return false;
  if (reinterpret_cast<uintptr_t>(a.cache) % 16) return false;
  if (a.rot_dims % 2 || a.r > 1024 || a.dr > 120) return false;
  return true;
}

static cudaError_t run_latent_mma(const LatentAttnArgs& a, int nw, int nt, bool shared_sm, cudaStream_t st) {
  const LatentMmaSmem sm = latent_mma_smem(a.r, a.dr);
  const int hpc = a.H < 16 ? a.H : 16, hblocks = (a.H + 15) / 16, G = 16 / hpc;
  const dim3 grid(static_cast<unsigned>((a.max_new + G - 1) / G) * hblocks, a.n_seqs, a.splits);
  // the query fragments a warp keeps: 8 k-steps cover keys up to 128 numbers wide, 40 up to 640
  const bool small = (a.r + a.dr + 15) / 16 <= 8;
#define LM_GO(NW, NT) return shared_sm ? launch_latent_mma<NW, NT, 0>(a, sm, grid, st) : small ? launch_latent_mma<NW, NT, 8>(a, sm, grid, st) \
                                                                                                : launch_latent_mma<NW, NT, 40>(a, sm, grid, st)
#define LM_NT(NW) switch (nt) { case 1: LM_GO(NW, 1); case 2: LM_GO(NW, 2); case 3: LM_GO(NW, 3); case 4: LM_GO(NW, 4); \
                                case 5: LM_GO(NW, 5); case 6: LM_GO(NW, 6); case 7: LM_GO(NW, 7); case 8: LM_GO(NW, 8); }
  if (nw == 8) { LM_NT(8) } else { LM_NT(4) }
#undef LM_NT
#undef LM_GO
  return cudaErrorInvalidValue;
}

}  // namespace lat
}  // namespace b2

extern "C" int b2tts_latent_attn(const void* ql, int64_t ql_tok, int64_t ql_head, const void* qr, int64_t qr_tok, int64_t qr_head,
                                 const void* cache, void* out, int64_t o_tok, int64_t o_head, const float* sink, const float* freq,
                                 float rot_mult, int rot_dims, const int32_t* seq_start, const int32_t* seq_pos0,
                                 const int32_t* seq_len, const int32_t* block_tables, int64_t bt_stride, int n_seqs, int max_new,
                                 int heads, int kv_rank, int rot_dim, int page, int window, float scale, int dtype, int path,
                                 int splits, float* ws, void* stream) {
  using namespace b2;
  using namespace b2::lat;
  B2_REQUIRE(n_seqs >= 0 && max_new >= 0 && heads > 0 && kv_rank > 0 && rot_dim >= 0 && page > 0 && window >= 0, B2TTS_EINVAL,
             "latent_attn: bad sizes");
  B2_REQUIRE(rot_dims >= 0 && rot_dims <= rot_dim && rot_dims % 2 == 0, B2TTS_EINVAL, "latent_attn: rot_dims %d of %d", rot_dims, rot_dim);
  B2_REQUIRE(dtype == B2TTS_DTYPE_BF16 || dtype == B2TTS_DTYPE_F32, B2TTS_EINVAL, "latent_attn: dtype %d", dtype);
  B2_REQUIRE(kv_rank <= 32 * LA_MAX_R_PER_LANE, B2TTS_EUNSUPPORTED, "latent_attn: latent size %d > %d", kv_rank, 32 * LA_MAX_R_PER_LANE);
  if (n_seqs == 0 || max_new == 0) return B2TTS_OK;
  B2_REQUIRE(ql && cache && out && seq_start && seq_pos0 && seq_len && block_tables && (rot_dim == 0 || qr) &&
             (rot_dims == 0 || freq), B2TTS_EINVAL, "latent_attn: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LatentAttnArgs a{ql, ql_tok, ql_head, qr, qr_tok, qr_head, cache, out, o_tok, o_head, sink, freq, rot_mult, rot_dims,
                   seq_start, seq_pos0, seq_len, block_tables, bt_stride, n_seqs, max_new, heads, kv_rank, rot_dim, page, window, scale, 0, 1, nullptr};
  int nw = 0, nt = 0;
  const bool fits = dtype == B2TTS_DTYPE_BF16 && latent_mma_fits(a, &nw, &nt);
  B2_REQUIRE(path != 2 || fits, B2TTS_EUNSUPPORTED, "latent_attn: the tensor-core kernel does not take kv_rank %d, rot_dim %d", kv_rank, rot_dim);
  B2_REQUIRE(path != 3 || fits, B2TTS_EUNSUPPORTED, "latent_attn: the tensor-core kernel does not take kv_rank %d, rot_dim %d", kv_rank, rot_dim);
  if (fits && path != 1) {
    a.ql_vec = reinterpret_cast<uintptr_t>(ql) % 16 == 0 && ql_tok % 8 == 0 && ql_head % 8 == 0;
    a.splits = (splits > 1 && ws != nullptr) ? splits : 1;
    a.ws = ws;
    // prompt portions: many CTAs, so two small ones per SM cover each other's waits; a decode step has few CTAs, each
    // of which hides its own loads behind a second key stage
    const bool shared_sm = path == 3 || (path == 0 && max_new > 1);
    cudaError_t e = run_latent_mma(a, nw, nt, shared_sm, st);
    if (e != cudaSuccess) return cuda_fail(e, "latent_attn (tensor)");
    B2_CHECK_LAUNCH("latent_attn (tensor)");
    if (a.splits > 1) {
      const int hpc = heads < 16 ? heads : 16, G = 16 / hpc;
      latent_attn_merge_kernel<<<dim3(static_cast<unsigned>((max_new + G - 1) / G) * ((heads + 15) / 16), n_seqs, 16), 128, 0, st>>>(a);
      B2_CHECK_LAUNCH("latent_attn (merge)");
    }
    return B2TTS_OK;
  }
  // (plain kernel) ql_vec: the cache rows can be read 16 bytes at a time
  a.ql_vec = reinterpret_cast<uintptr_t>(cache) % 16 == 0 &&
             ((kv_rank + rot_dim) * (dtype == B2TTS_DTYPE_BF16 ? 2 : 4)) % 16 == 0;
  const size_t smem = static_cast<size_t>(LA_WARPS) * (kv_rank + rot_dim) * sizeof(float);
  B2_REQUIRE(smem <= 48 * 1024, B2TTS_EUNSUPPORTED, "latent_attn: key size %d too large", kv_rank + rot_dim);
  const dim3 grid((static_cast<unsigned>(max_new) * heads + LA_WARPS - 1) / LA_WARPS, n_seqs);
  if (dtype == B2TTS_DTYPE_BF16) latent_attn_kernel<__nv_bfloat16><<<grid, LA_WARPS * 32, smem, st>>>(a);
  else latent_attn_kernel<float><<<grid, LA_WARPS * 32, smem, st>>>(a);
  B2_CHECK_LAUNCH("latent_attn");
  return B2TTS_OK;
}

/* How many key ranges a decode step's query tiles are cut into so that the tensor-core kernel fills the GPU (1 = no cut),
 * and the float workspace that many need. */
extern "C" int b2tts_latent_attn_splits(int n_seqs, int max_new, int heads) {
  if (max_new != 1 || n_seqs <= 0) return 1;
  const int ctas = n_seqs * ((heads + 15) / 16);
  int s = 148 / ctas;
  return s < 1 ? 1 : (s > 8 ? 8 : s);
}
extern "C" size_t b2tts_latent_attn_workspace_floats(int n_seqs, int max_new, int heads, int kv_rank, int splits) {
  const int hpc = heads < 16 ? heads : 16, G = 16 / hpc;
  return static_cast<size_t>(n_seqs) * ((max_new + G - 1) / G) * ((heads + 15) / 16) * splits * 16 * (kv_rank + 2);
}

/* Number of key-tile waits of the tensor-core kernel that ran out since the library was loaded (0 in a healthy run).
 * Synchronises the device. */
extern "C" int b2tts_latent_attn_timeouts(void) {
  int v = -1;
  if (cudaMemcpyFromSymbol(&v, b2::lat::g_latent_attn_timeouts, sizeof(int)) != cudaSuccess) return -1;
  return v;
}
