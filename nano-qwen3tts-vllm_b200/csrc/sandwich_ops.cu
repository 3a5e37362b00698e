// sandwich_ops.cu - per-row kernels of decoders whose sublayers are normed on the way in AND on the way out, both with a
// single-gain RMS norm ("sandwich" layers over a 32-bit residual stream):
//
//   x <- x + g_out N(y),   h = g_in N(x)          N(v) = v / sqrt(mean(v^2) + eps),  g_out / g_in one number each
//
// One launch does the residual update of a finished sublayer and the input norm of the next one.  What y is made of is
// chosen by the arguments:
//   a dense output                        y = a
//   an embedding row                      y = table[index[r]], and x starts from zero
//   two branches of a parallel mixer      y = c (N(a) * wa + N(b) * wb), each branch normed over the row with its weight vector
//   a mixture of experts                  y = sum_k zw[r, k] * (idx[r, k] < n_real ? z[r * top + k] : hin[r])
//                                         (choices >= n_real are identity experts: they return the sublayer's input)
// plus the small per-row pieces the same models need: PolyNorm, the combination of two attention maps that share their
// values (differential attention), and a tanh cap on logits.
//
// Activations are `T` = bf16 (serving) or float (the all-32-bit mode); the stream, every sum of squares and every norm
// are float in both.  Nothing allocates or synchronises; every launch is graph-capturable.
#include <algorithm>

#include "row_ops.cuh"

namespace b2 {
namespace row {

constexpr int SW_THREADS = 256;

struct SandwichArgs {
  float* x;                       // [rows, cols] the stream, updated in place
  const void* a;                  // [*, cols] dense output, first branch, or the embedding table
  const int32_t* a_index;         // row of `a` for stream row r (null: r)
  int a_rows;                     // rows of `a` when indexed (ids outside read as row 0)
  const void* b;                  // second branch (with wa, wb)
  const float* wa; const float* wb; float branch_scale;
  const void* z; const float* zw; const int32_t* z_idx; int top, n_real;
  const void* hin;                // the sublayer's input (identity experts)
  const float* g_out;             // [1]
  const float* g_in;              // [1] (with h)
  void* h;                        // [rows, cols] the next sublayer's input, or null
  int cols, init;
  float eps;
};

// V consecutive columns of a row <-> floats; V = 4 needs 4-column alignment of the pointer (8 bytes of bf16, 16 of float)
template <typename T, int V>
__device__ __forceinline__ void ld_cols(const T* p, float* f) {
  if constexpr (V == 1) {
    f[0] = to_f(p[0]);
  } else if constexpr (sizeof(T) == 4) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  } else {
    const uint2 r = ldg_v2(p);
    f[0] = bf16lo(r.x); f[1] = bf16hi(r.x); f[2] = bf16lo(r.y); f[3] = bf16hi(r.y);
  }
}
template <typename T, int V>
__device__ __forceinline__ void st_cols(T* p, const float* f) {
  if constexpr (V == 1) {
    p[0] = from_f<T>(f[0]);
  } else if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  } else {
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]));
  }
}

// One CTA per row; a thread owns groups of V consecutive columns (V = 4 when the row length and every pointer allow
// vector accesses).  y is kept in shared memory between the passes; every sum of squares is a block sum in a fixed order.
template <typename T, int V>
__global__ void __launch_bounds__(SW_THREADS)
sandwich_residual_kernel(const SandwichArgs p) {
  extern __shared__ __align__(16) float ybuf[];         // [cols]
  __shared__ float red[33];
  const size_t r = blockIdx.x;
  const int cols = p.cols, step = blockDim.x * V, c0 = threadIdx.x * V;
  const float fc = static_cast<float>(cols);
  const T* a = static_cast<const T*>(p.a);
  if (a != nullptr) {
    size_t ar = r;
    if (p.a_index != nullptr) {
      const int id = p.a_index[r];
      ar = (id >= 0 && id < p.a_rows) ? id : 0;
    }
    a += ar * cols;
  }
  float ssq = 0.f;
  if (p.wa != nullptr) {                                // two branches, each normed with its own weight vector
    const T* b = static_cast<const T*>(p.b) + r * cols;
    float sa = 0.f, sb = 0.f;
    for (int c = c0; c < cols; c += step) {
      float va[V], vb[V];
      ld_cols<T, V>(a + c, va); ld_cols<T, V>(b + c, vb);
#pragma unroll
      for (int i = 0; i < V; ++i) { sa += va[i] * va[i]; sb += vb[i] * vb[i]; }
    }
    const float ia = 1.0f / sqrtf(block_sum(sa, red) / fc + p.eps);
    const float ib = 1.0f / sqrtf(block_sum(sb, red) / fc + p.eps);
    for (int c = c0; c < cols; c += step) {
      float va[V], vb[V], wa[V], wb[V], y[V];
      ld_cols<T, V>(a + c, va); ld_cols<T, V>(b + c, vb);
      ld_cols<float, V>(p.wa + c, wa); ld_cols<float, V>(p.wb + c, wb);
#pragma unroll
      for (int i = 0; i < V; ++i) {
        y[i] = p.branch_scale * (va[i] * ia * wa[i] + vb[i] * ib * wb[i]);
        ssq += y[i] * y[i];
      }
      st_cols<float, V>(ybuf + c, y);
    }
  } else {
    const T* z = static_cast<const T*>(p.z);
    const T* hin = p.hin != nullptr ? static_cast<const T*>(p.hin) + r * cols : nullptr;
    for (int c = c0; c < cols; c += step) {
      float y[V];
      if (a != nullptr) {
        ld_cols<T, V>(a + c, y);
      } else {
#pragma unroll
        for (int i = 0; i < V; ++i) y[i] = 0.f;
      }
      for (int k = 0; k < p.top; ++k) {                 // choices in ascending order: a fixed order of additions
        const size_t pr = r * p.top + k;
        const bool real = p.z_idx == nullptr || p.z_idx[pr] < p.n_real;
        const float w = p.zw[pr];
        float zv[V];
        ld_cols<T, V>(real ? z + pr * cols + c : hin + c, zv);
#pragma unroll
        for (int i = 0; i < V; ++i) y[i] += w * zv[i];
      }
#pragma unroll
      for (int i = 0; i < V; ++i) ssq += y[i] * y[i];
      st_cols<float, V>(ybuf + c, y);
    }
  }
  const float inv = p.g_out[0] / sqrtf(block_sum(ssq, red) / fc + p.eps);
  float* xr = p.x + r * cols;
  float sx = 0.f;
  for (int c = c0; c < cols; c += step) {
    float y[V], xv[V];
    ld_cols<float, V>(ybuf + c, y);
    if (p.init) {
#pragma unroll
      for (int i = 0; i < V; ++i) xv[i] = 0.f;
    } else {
      ld_cols<float, V>(xr + c, xv);
    }
#pragma unroll
    for (int i = 0; i < V; ++i) { xv[i] += y[i] * inv; sx += xv[i] * xv[i]; }
    st_cols<float, V>(xr + c, xv);
    st_cols<float, V>(ybuf + c, xv);
  }
  if (p.h == nullptr) return;
  const float inv2 = p.g_in[0] / sqrtf(block_sum(sx, red) / fc + p.eps);
  T* hr = static_cast<T*>(p.h) + r * cols;
  for (int c = c0; c < cols; c += step) {
    float xv[V];
    ld_cols<float, V>(ybuf + c, xv);
#pragma unroll
    for (int i = 0; i < V; ++i) xv[i] *= inv2;
    st_cols<T, V>(hr + c, xv);
  }
}

// ------------------------------------------------------------------ PolyNorm, in place on the rows of y [rows, cols]
// y <- c0 N(y) + c1 N(y^2) + c2 N(y^3) + c3, powers element by element, N over the row.
template <typename T, int V>
__global__ void __launch_bounds__(SW_THREADS)
polynorm_kernel(T* __restrict__ y, const float* __restrict__ coef, int cols, float eps) {
  __shared__ float red[33];
  T* yr = y + static_cast<size_t>(blockIdx.x) * cols;
  const int step = blockDim.x * V, c0 = threadIdx.x * V;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int c = c0; c < cols; c += step) {
    float v[V];
    ld_cols<T, V>(yr + c, v);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const float v2 = v[i] * v[i];
      s2 += v2; s4 += v2 * v2; s6 += v2 * v2 * v2;
    }
  }
  const float fc = static_cast<float>(cols);
  const float i1 = coef[0] / sqrtf(block_sum(s2, red) / fc + eps);
  const float i2 = coef[1] / sqrtf(block_sum(s4, red) / fc + eps);
  const float i3 = coef[2] / sqrtf(block_sum(s6, red) / fc + eps);
  const float c3 = coef[3];
  for (int c = c0; c < cols; c += step) {
    float v[V];
    ld_cols<T, V>(yr + c, v);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const float v2 = v[i] * v[i];
      v[i] = v[i] * i1 + v2 * i2 + v2 * v[i] * i3 + c3;
    }
    st_cols<T, V>(yr + c, v);
  }
}

// ------------------------------------------------------------------ two attention maps over the same values -> one output
// maps [rows, 2, H, dv] (the first map's heads, then the second map's); out[r, h] = N_head(maps[r, 0, h] - lambda * maps[r, 1, h])
// * mult, N over the head's dv values without a weight.  One warp per (row, head).  The maps may be floats while the output
// has the activation type, so that the difference is taken before anything is rounded to 16 bits.
constexpr int DC_PER_LANE = 8;                          // value sizes up to 256

template <typename TI, typename T>
__global__ void __launch_bounds__(128)
diff_combine_kernel(const TI* __restrict__ maps, T* __restrict__ out, float lambda, float mult, int rows, int H, int dv, float eps) {
  const int lane = threadIdx.x & 31;
  const size_t w = static_cast<size_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= static_cast<size_t>(rows) * H) return;
  const size_t r = w / H;
  const int h = static_cast<int>(w % H);
  const TI* m1 = maps + (r * 2 * H + h) * dv;
  const TI* m2 = m1 + static_cast<size_t>(H) * dv;
  float o[DC_PER_LANE], ss = 0.f;
#pragma unroll
  for (int i = 0; i < DC_PER_LANE; ++i) {
    const int c = i * 32 + lane;
    o[i] = c < dv ? to_f(m1[c]) - lambda * to_f(m2[c]) : 0.f;
    ss += o[i] * o[i];
  }
  const float inv = mult / sqrtf(warp_sum(ss) / static_cast<float>(dv) + eps);
  T* orow = out + (r * H + h) * dv;
#pragma unroll
  for (int i = 0; i < DC_PER_LANE; ++i) {
    const int c = i * 32 + lane;
    if (c < dv) orow[c] = from_f<T>(o[i] * inv);
  }
}

__global__ void tanh_cap_kernel(float* __restrict__ y, size_t n, float cap) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) y[i] = cap * tanhf(y[i] / cap);
}

}  // namespace row
}  // namespace b2

using namespace b2;
using namespace b2::row;

extern "C" int b2tts_sandwich_residual(float* x, const void* a, const int32_t* a_index, int a_rows, const void* b, const float* wa,
                                       const float* wb, float branch_scale, const void* z, const float* zw, const int32_t* z_idx,
                                       int top, int n_real, const void* hin, const float* g_out, const float* g_in, void* h,
                                       int rows, int cols, int init, float eps, int dtype, void* stream) {
  B2_REQUIRE(rows >= 0 && cols > 0 && top >= 0, B2TTS_EINVAL, "sandwich_residual: rows=%d cols=%d top=%d", rows, cols, top);
  B2_REQUIRE(B2_ROW_DTYPE_OK(dtype), B2TTS_EINVAL, "sandwich_residual: dtype %d", dtype);
  B2_REQUIRE(cols <= 12 * 1024, B2TTS_EUNSUPPORTED, "sandwich_residual: %d columns above %d", cols, 12 * 1024);
  if (rows == 0) return B2TTS_OK;
  B2_REQUIRE(x && g_out && (!h || g_in), B2TTS_EINVAL, "sandwich_residual: null pointer");
  B2_REQUIRE((wa == nullptr) == (wb == nullptr) && (wa == nullptr || (a && b && top == 0)), B2TTS_EINVAL,
             "sandwich_residual: two branches need a, b and both weight vectors, and no experts");
  B2_REQUIRE(top == 0 || (z && zw && (z_idx == nullptr || hin)), B2TTS_EINVAL, "sandwich_residual: experts need z, zw (and hin with z_idx)");
  B2_REQUIRE(a || top > 0, B2TTS_EINVAL, "sandwich_residual: nothing to add");
  B2_REQUIRE(a_index == nullptr || (a && a_rows > 0), B2TTS_EINVAL, "sandwich_residual: indexed rows need a table");
  SandwichArgs p{x, a, a_index, a_rows, b, wa, wb, branch_scale, z, zw, z_idx, top, n_real, hin, g_out, g_in, h, cols, init, eps};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t sm = static_cast<size_t>(cols) * sizeof(float);
  // vector accesses: rows of whole 4-column groups and every tensor 16-byte aligned (rows of `a`, `z`, `h` then start on
  // 8-byte boundaries in bf16, 16-byte ones in float)
  bool vec = cols % 4 == 0;
  for (const void* q : {static_cast<const void*>(x), a, b, static_cast<const void*>(wa), static_cast<const void*>(wb), z, hin,
                        static_cast<const void*>(h)})
    vec = vec && (q == nullptr || aligned16(q));
  if (dtype == B2TTS_DTYPE_BF16) {
    if (vec) sandwich_residual_kernel<__nv_bfloat16, 4><<<rows, SW_THREADS, sm, st>>>(p);
    else sandwich_residual_kernel<__nv_bfloat16, 1><<<rows, SW_THREADS, sm, st>>>(p);
  } else {
    if (vec) sandwich_residual_kernel<float, 4><<<rows, SW_THREADS, sm, st>>>(p);
    else sandwich_residual_kernel<float, 1><<<rows, SW_THREADS, sm, st>>>(p);
  }
  B2_CHECK_LAUNCH("sandwich_residual");
  return B2TTS_OK;
}

extern "C" int b2tts_polynorm(void* y, const float* coef, int rows, int cols, float eps, int dtype, void* stream) {
  B2_REQUIRE(rows >= 0 && cols > 0, B2TTS_EINVAL, "polynorm: rows=%d cols=%d", rows, cols);
  B2_REQUIRE(B2_ROW_DTYPE_OK(dtype), B2TTS_EINVAL, "polynorm: dtype %d", dtype);
  if (rows == 0) return B2TTS_OK;
  B2_REQUIRE(y && coef, B2TTS_EINVAL, "polynorm: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool vec = cols % 4 == 0 && aligned16(y);
  if (dtype == B2TTS_DTYPE_BF16) {
    if (vec) polynorm_kernel<__nv_bfloat16, 4><<<rows, SW_THREADS, 0, st>>>(static_cast<__nv_bfloat16*>(y), coef, cols, eps);
    else polynorm_kernel<__nv_bfloat16, 1><<<rows, SW_THREADS, 0, st>>>(static_cast<__nv_bfloat16*>(y), coef, cols, eps);
  } else {
    if (vec) polynorm_kernel<float, 4><<<rows, SW_THREADS, 0, st>>>(static_cast<float*>(y), coef, cols, eps);
    else polynorm_kernel<float, 1><<<rows, SW_THREADS, 0, st>>>(static_cast<float*>(y), coef, cols, eps);
  }
  B2_CHECK_LAUNCH("polynorm");
  return B2TTS_OK;
}

extern "C" int b2tts_diff_combine(const void* maps, void* out, float lambda, float mult, int rows, int heads, int vdim, float eps,
                                  int maps_f32, int dtype, void* stream) {
  B2_REQUIRE(rows >= 0 && heads > 0 && vdim > 0, B2TTS_EINVAL, "diff_combine: rows=%d heads=%d vdim=%d", rows, heads, vdim);
  B2_REQUIRE(vdim <= 32 * DC_PER_LANE, B2TTS_EUNSUPPORTED, "diff_combine: value size %d above %d", vdim, 32 * DC_PER_LANE);
  B2_REQUIRE(B2_ROW_DTYPE_OK(dtype), B2TTS_EINVAL, "diff_combine: dtype %d", dtype);
  if (rows == 0) return B2TTS_OK;
  B2_REQUIRE(maps && out, B2TTS_EINVAL, "diff_combine: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t warps = static_cast<size_t>(rows) * heads;
  const unsigned blocks = static_cast<unsigned>((warps + 3) / 4);
  if (dtype == B2TTS_DTYPE_BF16 && maps_f32)
    diff_combine_kernel<float, __nv_bfloat16><<<blocks, 128, 0, st>>>(static_cast<const float*>(maps), static_cast<__nv_bfloat16*>(out),
                                                                      lambda, mult, rows, heads, vdim, eps);
  else if (dtype == B2TTS_DTYPE_BF16)
    diff_combine_kernel<__nv_bfloat16, __nv_bfloat16><<<blocks, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(maps),
                                                                              static_cast<__nv_bfloat16*>(out), lambda, mult, rows, heads, vdim, eps);
  else
    diff_combine_kernel<float, float><<<blocks, 128, 0, st>>>(static_cast<const float*>(maps), static_cast<float*>(out), lambda, mult, rows,
                                                              heads, vdim, eps);
  B2_CHECK_LAUNCH("diff_combine");
  return B2TTS_OK;
}

extern "C" int b2tts_tanh_cap(float* y, int64_t n, float cap, void* stream) {
  B2_REQUIRE(n >= 0 && cap > 0.f, B2TTS_EINVAL, "tanh_cap: n=%lld cap=%g", static_cast<long long>(n), cap);
  if (n == 0) return B2TTS_OK;
  B2_REQUIRE(y, B2TTS_EINVAL, "tanh_cap: null pointer");
  tanh_cap_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(y, static_cast<size_t>(n), cap);
  B2_CHECK_LAUNCH("tanh_cap");
  return B2TTS_OK;
}
