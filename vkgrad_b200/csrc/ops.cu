// Streaming and row kernels of the training step: everything the reference
// generates as GLSL in kernels.make_kernels (kernels.py:699-862) and
// tkernels.make_transformer_kernels (tkernels.py:17-389).  All are HBM-bound;
// accesses are coalesced and vectorised where alignment allows, reductions are
// warp/CTA shuffles, and the column sums are deterministic (fixed-order partial
// sums in caller-provided scratch) instead of float atomics.
#include "common.cuh"

namespace {

constexpr int TPB = 256;

// ---- flat elementwise -------------------------------------------------------

__global__ void k_bias_act(const float* __restrict__ acc, const float* __restrict__ bias,
                           float* __restrict__ z, __half* __restrict__ y16, int64_t n, int ncol,
                           int act) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    float v = acc[i] + bias[i % ncol];
    if (z) z[i] = v;
    if (y16) y16[i] = __float2half_rn(vkg_act(v, act));
  }
}

__global__ void k_bias_act_bwd(const float* __restrict__ dy, const float* __restrict__ z,
                               __half* __restrict__ dz16, float* __restrict__ dz32, int64_t n,
                               int act) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    float g = dy[i] * vkg_dact(z[i], act);
    if (dz16) dz16[i] = __float2half_rn(g);
    if (dz32) dz32[i] = g;
  }
}

__global__ void k_cast16(const float* __restrict__ src, __half* __restrict__ dst, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) dst[i] = __float2half_rn(src[i]);
}

__global__ void k_cast16_v4(const float4* __restrict__ src, uint2* __restrict__ dst, int64_t n4) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n4; i += stride) {
    float4 v = src[i];
    __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&a);
    o.y = *reinterpret_cast<uint32_t*>(&b);
    dst[i] = o;
  }
}

__global__ void k_residual(const float* __restrict__ acc, const float* __restrict__ bias,
                           const float* __restrict__ res, float* __restrict__ out, int64_t n, int D) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) out[i] = res[i] + acc[i] + bias[i % D];
}

__global__ void k_add(const float* __restrict__ a, const float* __restrict__ b,
                      float* __restrict__ out, __half* __restrict__ out16, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    float v = a[i] + b[i];
    if (out) out[i] = v;
    if (out16) out16[i] = __float2half_rn(v);
  }
}

__global__ void k_add_bias(float* __restrict__ x, const float* __restrict__ bias, int64_t n,
                           int ncol) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) x[i] += bias[i % ncol];
}

__global__ void k_grad_add(const float* __restrict__ g, float* __restrict__ arena, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) arena[i] += g[i];
}

__global__ void k_grad_pull(const float* __restrict__ arena, float* __restrict__ g, int64_t n,
                            float scale) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) g[i] = arena[i] * scale;
}

template <typename T16>
__global__ void k_pack16(const float* __restrict__ src, T16* __restrict__ dst, int64_t n,
                         float scale) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) dst[i] = T16(src[i] * scale);
}

template <typename T16>
__global__ void k_unpack16(const T16* __restrict__ src, float* __restrict__ dst, int64_t n,
                           float scale) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) dst[i] = float(src[i]) * scale;
}

// ---- head permutes ------------------------------------------------------------

__global__ void k_split_qkv(const float* __restrict__ qkv, const float* __restrict__ bias,
                            __half* __restrict__ q16, __half* __restrict__ k16,
                            __half* __restrict__ v16, int64_t n, int D, int T, int H, int hd) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    int d = (int)(i % D);
    int64_t bt = i / D;
    int t = (int)(bt % T);
    int64_t b = bt / T;
    int h = d / hd, j = d % hd;
    int64_t dst = ((b * H + h) * T + t) * hd + j;
    int64_t src = bt * 3 * D + d;
    q16[dst] = __float2half_rn(qkv[src] + bias[d]);
    k16[dst] = __float2half_rn(qkv[src + D] + bias[d + D]);
    v16[dst] = __float2half_rn(qkv[src + 2 * D] + bias[d + 2 * D]);
  }
}

__global__ void k_merge_qkv_grad(const float* __restrict__ dq, const float* __restrict__ dk,
                                 const float* __restrict__ dv, __half* __restrict__ dqkv16,
                                 int64_t n, int D, int T, int H, int hd) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    int d = (int)(i % D);
    int64_t bt = i / D;
    int t = (int)(bt % T);
    int64_t b = bt / T;
    int h = d / hd, j = d % hd;
    int64_t src = ((b * H + h) * T + t) * hd + j;
    int64_t dst = bt * 3 * D + d;
    dqkv16[dst] = __float2half_rn(dq[src]);
    dqkv16[dst + D] = __float2half_rn(dk[src]);
    dqkv16[dst + 2 * D] = __float2half_rn(dv[src]);
  }
}

__global__ void k_merge_heads(const float* __restrict__ src, __half* __restrict__ y16, int64_t n,
                              int D, int T, int H, int hd) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    int d = (int)(i % D);
    int64_t bt = i / D;
    int t = (int)(bt % T);
    int64_t b = bt / T;
    int h = d / hd, j = d % hd;
    y16[i] = __float2half_rn(src[((b * H + h) * T + t) * hd + j]);
  }
}

__global__ void k_split_heads(const float* __restrict__ src, __half* __restrict__ dst16, int64_t n,
                              int D, int T, int H, int hd) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    int d = (int)(i % D);
    int64_t bt = i / D;
    int t = (int)(bt % T);
    int64_t b = bt / T;
    int h = d / hd, j = d % hd;
    dst16[((b * H + h) * T + t) * hd + j] = __float2half_rn(src[i]);
  }
}

// ---- embeddings -----------------------------------------------------------------

__global__ void k_embed(const float* __restrict__ tok, const float* __restrict__ pos,
                        const uint32_t* __restrict__ ids, const uint32_t* __restrict__ seg,
                        float* __restrict__ x, int64_t n, int D, int T) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    int d = (int)(i % D);
    int64_t bt = i / D;
    int t = (int)(bt % T);
    if (seg) t -= (int)seg[bt];
    x[i] = tok[(int64_t)ids[bt] * D + d] + pos[(int64_t)t * D + d];
  }
}

__global__ void k_embed_bwd(const float* __restrict__ dx, const uint32_t* __restrict__ ids,
                            const uint32_t* __restrict__ seg, float* __restrict__ dtok,
                            float* __restrict__ dpos, int64_t n, int D, int T) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    int d = (int)(i % D);
    int64_t bt = i / D;
    int t = (int)(bt % T);
    if (seg) t -= (int)seg[bt];
    float g = dx[i];
    atomicAdd(dtok + (int64_t)ids[bt] * D + d, g);
    atomicAdd(dpos + (int64_t)t * D + d, g);
  }
}

// Four columns per thread (D a multiple of 4, 16-byte aligned tables): one 16-byte access
// per operand, and one 16-byte vector atomic per table in the backward.
__global__ void k_embed_v4(const float4* __restrict__ tok, const float4* __restrict__ pos,
                           const uint32_t* __restrict__ ids, const uint32_t* __restrict__ seg,
                           float4* __restrict__ x, int n4, int D4, int T) {
  pdl_trigger();
  pdl_wait();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += gridDim.x * blockDim.x) {
    const int bt = i / D4, d = i - bt * D4;
    int t = bt % T;
    if (seg) t -= (int)seg[bt];
    const float4 a = tok[(int64_t)ids[bt] * D4 + d], b = pos[(int64_t)t * D4 + d];
    x[i] = make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
  }
}

__global__ void k_embed_bwd_v4(const float4* __restrict__ dx, const uint32_t* __restrict__ ids,
                               const uint32_t* __restrict__ seg, float4* __restrict__ dtok,
                               float4* __restrict__ dpos, int n4, int D4, int T) {
  pdl_trigger();
  pdl_wait();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += gridDim.x * blockDim.x) {
    const int bt = i / D4, d = i - bt * D4;
    int t = bt % T;
    if (seg) t -= (int)seg[bt];
    const float4 g = dx[i];
    atomicAdd(dtok + (int64_t)ids[bt] * D4 + d, g);
    atomicAdd(dpos + (int64_t)t * D4 + d, g);
  }
}

// Deterministic scatter-add of the embedding backward (the reference adds with float atomics,
// tkernels.py:317-360, whose order changes from run to run).  Rows that hit the same table
// row are linked into a chain in row order; the warp that owns a chain's first row walks it,
// adds the rows in that order in registers and updates the table row once.
//
// Table `which`: 0 the token table (key = ids[r]), 1 the position table (key = r % T, minus
// the start of the row's packed sample).  keys[which][rows_p] (rows_p = rows rounded up to 4,
// the padding holds -2), next[which][rows] = the next row with r's key or -1,
// has_prev[which][rows] = 1 when an earlier row has it.
__device__ __forceinline__ int embed_key(int which, int r, const uint32_t* ids, const uint32_t* seg,
                                         int T) {
  if (which == 0) return (int)ids[r];
  int t = r % T;
  if (seg) t -= (int)seg[r];
  return t;
}

__global__ void k_embed_keys(const uint32_t* __restrict__ ids, const uint32_t* __restrict__ seg,
                             int* __restrict__ keys, int* __restrict__ has_prev, int rows, int rows_p,
                             int T) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= 2 * rows_p) return;
  const int which = i / rows_p, r = i - which * rows_p;
  keys[i] = r < rows ? embed_key(which, r, ids, seg, T) : -2;
  if (r < rows) has_prev[which * rows + r] = 0;
}

// One warp per (table, row): the lanes look through the later rows 128 keys at a time (one
// 16-byte load each) and stop at the first chunk that holds the row's key; the smallest such
// row is the successor, whatever the timing.
__global__ void __launch_bounds__(256)
k_embed_chain(const int* __restrict__ keys, int* __restrict__ next, int* __restrict__ has_prev,
              int rows, int rows_p) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= 2 * rows) return;
  const int which = w / rows, r = w - which * rows;
  const int* k = keys + (size_t)which * rows_p;
  const int key = k[r];
  int found = -1;
  // four chunks of 128 keys per round: the four loads are independent, so a round costs one
  // memory round trip instead of four
  for (int j0 = ((r + 1) & ~3) + lane * 4; found < 0; j0 += 512) {
    unsigned m[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = j0 + u * 128;
      m[u] = 0;
      if (j < rows_p) {
        const int4 v = *reinterpret_cast<const int4*>(k + j);
        m[u] = (v.x == key && j > r ? 1u : 0u) | (v.y == key && j + 1 > r ? 2u : 0u) |
               (v.z == key && j + 2 > r ? 4u : 0u) | (v.w == key && j + 3 > r ? 8u : 0u);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const unsigned any = __ballot_sync(0xffffffffu, m[u] != 0u);
      if (any && found < 0) {
        const int src = __ffs(any) - 1;
        const int mine = j0 + u * 128 + __ffs(m[u]) - 1;     // meaningful on lane `src` only
        found = __shfl_sync(0xffffffffu, mine, src);
      }
    }
    if (__all_sync(0xffffffffu, j0 + 512 - lane * 4 >= rows_p)) break;   // the warp is past the end
  }
  if (lane == 0) {
    next[which * rows + r] = found;
    if (found >= 0) has_prev[which * rows + found] = 1;   // one writer: its predecessor
  }
}

template <int NV>
__global__ void __launch_bounds__(256)
k_embed_bwd_chain(const float* __restrict__ dx, const uint32_t* __restrict__ ids,
                  const uint32_t* __restrict__ seg, const int* __restrict__ next,
                  const int* __restrict__ has_prev, float* __restrict__ dtok, float* __restrict__ dpos,
                  int rows, int T) {
  constexpr int D = NV * 128;
  pdl_trigger();
  pdl_wait();
  const int which = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r0 = blockIdx.x * (blockDim.x >> 5) + warp;
  if (r0 >= rows || has_prev[which * rows + r0]) return;
  float4 acc[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int r = r0; r >= 0; r = next[which * rows + r]) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const float4 g = *reinterpret_cast<const float4*>(dx + (size_t)r * D + (i * 32 + lane) * 4);
      acc[i].x += g.x; acc[i].y += g.y; acc[i].z += g.z; acc[i].w += g.w;
    }
  }
  float* row = (which == 0 ? dtok : dpos) + (size_t)embed_key(which, r0, ids, seg, T) * D;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    float4* p = reinterpret_cast<float4*>(row + (i * 32 + lane) * 4);
    float4 v = *p;
    v.x += acc[i].x; v.y += acc[i].y; v.z += acc[i].z; v.w += acc[i].w;
    *p = v;
  }
}

// ---- column sums ------------------------------------------------------------------

// The reference's col_sum: one thread per column over fp32 rows (kernels.py:753).
__global__ void k_col_sum(const float* __restrict__ g, float* __restrict__ sums, int ncol,
                          int nrow) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= ncol) return;
  float s = 0.f;
  for (int r = 0; r < nrow; ++r) s += g[(int64_t)r * ncol + c];
  sums[c] = s;
}

constexpr int CS_WARPS = 8;

template <typename T> struct ColVec;
template <> struct ColVec<__half> {   // 8 columns per lane: one 16-byte load per row
  static constexpr int N = 8;
  __device__ static void add(const __half* p, float* s) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __half22float2(h[j]);
      s[2 * j] += f.x;
      s[2 * j + 1] += f.y;
    }
  }
};
template <> struct ColVec<float> {    // 4 columns per lane
  static constexpr int N = 4;
  __device__ static void add(const float* p, float* s) {
    float4 u = *reinterpret_cast<const float4*>(p);
    s[0] += u.x; s[1] += u.y; s[2] += u.z; s[3] += u.w;
  }
};

// Stage 1: block (cx, chunk) sums rows [chunk*rpc, ...) of its 32*N columns into
// partial[chunk][col].  Warps stride the rows; each lane owns N adjacent columns and
// reads them with one 16-byte load per row (scalar loads when ncol is not a multiple
// of N or the base is unaligned).
template <typename T>
__global__ void __launch_bounds__(CS_WARPS * 32)
k_col_sum_partial(const T* __restrict__ g, float* __restrict__ partial, int ncol, int nrow,
                  int rows_per_chunk, int vec_ok) {
  constexpr int N = ColVec<T>::N;
  __shared__ float red[CS_WARPS][32 * N + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = (blockIdx.x * 32 + lane) * N;
  const int r0 = blockIdx.y * rows_per_chunk;
  const int r1 = min(nrow, r0 + rows_per_chunk);
  float s[N];
#pragma unroll
  for (int j = 0; j < N; ++j) s[j] = 0.f;
  if (vec_ok) {
    if (c < ncol) {
      int r = r0 + warp;
      for (; r + 3 * CS_WARPS < r1; r += 4 * CS_WARPS) {   // four rows in flight per lane
        ColVec<T>::add(g + (int64_t)r * ncol + c, s);
        ColVec<T>::add(g + (int64_t)(r + CS_WARPS) * ncol + c, s);
        ColVec<T>::add(g + (int64_t)(r + 2 * CS_WARPS) * ncol + c, s);
        ColVec<T>::add(g + (int64_t)(r + 3 * CS_WARPS) * ncol + c, s);
      }
      for (; r < r1; r += CS_WARPS) ColVec<T>::add(g + (int64_t)r * ncol + c, s);
    }
  } else {
    for (int r = r0 + warp; r < r1; r += CS_WARPS)
#pragma unroll
      for (int j = 0; j < N; ++j)
        if (c + j < ncol) s[j] += float(g[(int64_t)r * ncol + c + j]);
  }
#pragma unroll
  for (int j = 0; j < N; ++j) red[warp][lane * N + j] = s[j];
  __syncthreads();
  for (int t = threadIdx.x; t < 32 * N; t += CS_WARPS * 32) {
    float a = 0.f;
#pragma unroll
    for (int w = 0; w < CS_WARPS; ++w) a += red[w][t];
    int col = blockIdx.x * 32 * N + t;
    if (col < ncol) partial[(int64_t)blockIdx.y * ncol + col] = a;
  }
}

// Stage 2: fixed-order sum of the partials.  A CTA owns 32 columns; its 8 warps each
// add every 8th chunk, then the eight slices are added in order.
constexpr int CSF_SLICES = 8;
__global__ void __launch_bounds__(32 * CSF_SLICES)
k_col_sum_final(const float* __restrict__ partial, float* __restrict__ sums, int ncol, int nchunk,
                int accumulate) {
  __shared__ float red[CSF_SLICES][32];
  const int lane = threadIdx.x & 31, slice = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float s = 0.f;
  if (c < ncol)
    for (int k = slice; k < nchunk; k += CSF_SLICES) s += partial[(int64_t)k * ncol + c];
  red[slice][lane] = s;
  __syncthreads();
  if (slice == 0 && c < ncol) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < CSF_SLICES; ++k) t += red[k][lane];
    sums[c] = accumulate ? sums[c] + t : t;
  }
}

// ---- softmax + cross entropy ---------------------------------------------------------

// One CTA per row.  Online max/sum in one pass, then one pass writing the
// gradient; the second read of the row comes out of L2.
__global__ void __launch_bounds__(TPB)
k_softmax_ce(const float* __restrict__ logits, const uint32_t* __restrict__ labels,
             const float* __restrict__ w, __half* __restrict__ dl16, float* __restrict__ dl32,
             float* __restrict__ loss, int stride, int ncls, float grad_scale) {
  __shared__ float s_m[TPB / 32], s_s[TPB / 32];
  __shared__ float s_logz;
  const int row = blockIdx.x;
  const float* x = logits + (int64_t)row * stride;
  __half* d16 = dl16 ? dl16 + (int64_t)row * stride : nullptr;
  float* d32 = dl32 ? dl32 + (int64_t)row * stride : nullptr;
  float wi = grad_scale;
  if (w) {
    // per-row weights replace the mean; a non-zero grad_scale then is a static loss scale
    wi = w[row] * (grad_scale != 0.0f ? grad_scale : 1.0f);
    if (wi == 0.0f) {
      for (int c = threadIdx.x; c < stride; c += TPB) {
        if (d16) d16[c] = __float2half_rn(0.f);
        if (d32) d32[c] = 0.f;
      }
      if (threadIdx.x == 0) loss[row] = 0.f;
      return;
    }
  }
  float m = -1e30f, s = 0.f;
  for (int c = threadIdx.x; c < ncls; c += TPB) {
    float v = x[c];
    if (v > m) {
      s = s * __expf(m - v) + 1.0f;
      m = v;
    } else {
      s += __expf(v - m);
    }
  }
  // combine (m, s) pairs across the warp, then across warps
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    float s2 = __shfl_xor_sync(0xffffffffu, s, o);
    float mm = fmaxf(m, m2);
    s = s * __expf(m - mm) + s2 * __expf(m2 - mm);
    m = mm;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    s_m[warp] = m;
    s_s[warp] = s;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float mm = s_m[0], ss = s_s[0];
    for (int k = 1; k < TPB / 32; ++k) {
      float m2 = s_m[k], s2 = s_s[k];
      float mx = fmaxf(mm, m2);
      ss = ss * __expf(mm - mx) + s2 * __expf(m2 - mx);
      mm = mx;
    }
    float logz = mm + logf(ss);
    s_logz = logz;
    loss[row] = logz - x[labels[row]];
  }
  __syncthreads();
  const float logz = s_logz;
  const int y = (int)labels[row];
  for (int c = threadIdx.x; c < stride; c += TPB) {
    float gv = 0.f;
    if (c < ncls) gv = (__expf(x[c] - logz) - (c == y ? 1.0f : 0.0f)) * wi;
    if (d16) d16[c] = __float2half_rn(gv);
    if (d32) d32[c] = gv;
  }
}

// Register-resident variant for wide rows (the GPT head: 50 272 columns): one CTA of
// 768 threads per row, every thread keeps up to NV float4 of the row in registers, so
// the logits are read from HBM exactly once and the gradient is written from registers.
constexpr int CE_THREADS = 768;

template <int NV>
__global__ void __launch_bounds__(CE_THREADS)
k_softmax_ce_reg(const float* __restrict__ logits, const uint32_t* __restrict__ labels,
                 const float* __restrict__ w, __half* __restrict__ dl16, float* __restrict__ dl32,
                 float* __restrict__ loss, int stride, int ncls, float grad_scale, int pf_rows) {
  pdl_trigger();
  pdl_wait();
  __shared__ float s_red[CE_THREADS / 32];
  __shared__ float s_bcast;
  const int row = blockIdx.x;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const float* x = logits + (size_t)row * stride;
  const int n4 = stride >> 2;
  float wi = grad_scale;
  bool skip = false;
  if (w) {
    wi = w[row] * (grad_scale != 0.0f ? grad_scale : 1.0f);
    skip = wi == 0.0f;
  }
  float4 v[NV];
  float m = -1e30f;
  if (!skip) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c4 = tid + i * CE_THREADS;
      v[i] = c4 < n4 ? *reinterpret_cast<const float4*>(x + 4 * c4) : make_float4(0, 0, 0, 0);
      const int c = 4 * c4;
      if (c + 0 < ncls) m = fmaxf(m, v[i].x);
      if (c + 1 < ncls) m = fmaxf(m, v[i].y);
      if (c + 2 < ncls) m = fmaxf(m, v[i].z);
      if (c + 3 < ncls) m = fmaxf(m, v[i].w);
    }
  }
  // Only one CTA of this size fits an SM, so its load, reduce and store phases do not
  // overlap: pull the row that the CTA after this one on the same SM will want into L2
  // now, which keeps HBM streaming while this row is reduced and written.
  if (row + pf_rows < (int)gridDim.x) {
    const char* nx = reinterpret_cast<const char*>(logits + (size_t)(row + pf_rows) * stride);
    for (int o = tid * 128; o < stride * 4; o += CE_THREADS * 128)
      asm volatile("prefetch.global.L2 [%0];" ::"l"(nx + o));
  }
  m = warp_max(m);
  if (lane == 0) s_red[warp] = m;
  __syncthreads();
  if (warp == 0) {
    float t = lane < CE_THREADS / 32 ? s_red[lane] : -1e30f;
    t = warp_max(t);
    if (lane == 0) s_bcast = t;
  }
  __syncthreads();
  m = s_bcast;
  float sum = 0.f;
  if (!skip) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = 4 * (tid + i * CE_THREADS);
      // keep exp(x - m) in place of x: it is what the gradient needs
      v[i].x = c + 0 < ncls ? __expf(v[i].x - m) : 0.f;
      v[i].y = c + 1 < ncls ? __expf(v[i].y - m) : 0.f;
      v[i].z = c + 2 < ncls ? __expf(v[i].z - m) : 0.f;
      v[i].w = c + 3 < ncls ? __expf(v[i].w - m) : 0.f;
      sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
  }
  sum = warp_sum(sum);
  __syncthreads();
  if (lane == 0) s_red[warp] = sum;
  __syncthreads();
  if (warp == 0) {
    float t = warp_sum(lane < CE_THREADS / 32 ? s_red[lane] : 0.f);
    if (lane == 0) s_bcast = t;
  }
  __syncthreads();
  sum = s_bcast;
  const int y = (int)labels[row];
  if (tid == 0) loss[row] = skip ? 0.f : (m + logf(sum)) - x[y];
  const float k = skip ? 0.f : wi / sum;
  __half* d16 = dl16 ? dl16 + (size_t)row * stride : nullptr;
  float* d32 = dl32 ? dl32 + (size_t)row * stride : nullptr;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c4 = tid + i * CE_THREADS;
    if (c4 >= n4) continue;
    const int c = 4 * c4;
    float4 g = skip ? make_float4(0, 0, 0, 0)
                    : make_float4(v[i].x * k, v[i].y * k, v[i].z * k, v[i].w * k);
    if (!skip && y >= c && y < c + 4) {
      if (y == c) g.x -= wi;
      else if (y == c + 1) g.y -= wi;
      else if (y == c + 2) g.z -= wi;
      else g.w -= wi;
    }
    if (d16) {
      __half2 a = __floats2half2_rn(g.x, g.y), b = __floats2half2_rn(g.z, g.w);
      uint2 u;
      u.x = *reinterpret_cast<uint32_t*>(&a);
      u.y = *reinterpret_cast<uint32_t*>(&b);
      *reinterpret_cast<uint2*>(d16 + c) = u;
    }
    if (d32) *reinterpret_cast<float4*>(d32 + c) = g;
  }
}

// ---- layernorm ----------------------------------------------------------------------------

// One warp per row, lanes stride the row (the reference's layout, tkernels.py:32-54).
__global__ void k_layernorm(const float* __restrict__ x, const float* __restrict__ gamma,
                            const float* __restrict__ beta, __half* __restrict__ y16,
                            float* __restrict__ mu, float* __restrict__ rstd, int rows, int D) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + warp;
  if (row >= rows) return;
  const float* xr = x + (int64_t)row * D;
  float s = 0.f;
  for (int d = lane; d < D; d += 32) s += xr[d];
  const float m = warp_sum(s) / (float)D;
  float v = 0.f;
  for (int d = lane; d < D; d += 32) {
    float t = xr[d] - m;
    v += t * t;
  }
  const float r = rsqrtf(warp_sum(v) / (float)D + 1e-5f);
  if (lane == 0) {
    mu[row] = m;
    rstd[row] = r;
  }
  __half* yr = y16 + (int64_t)row * D;
  for (int d = lane; d < D; d += 32) yr[d] = __float2half_rn((xr[d] - m) * r * gamma[d] + beta[d]);
}

// D = 128 * NV: the row lives in registers (NV float4 per lane), one read of x.
template <int NV>
__global__ void k_layernorm_vec(const float* __restrict__ x, const float* __restrict__ gamma,
                                const float* __restrict__ beta, __half* __restrict__ y16,
                                float* __restrict__ mu, float* __restrict__ rstd, int rows) {
  constexpr int D = NV * 128;
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + warp;
  if (row >= rows) return;
  const float* xr = x + (size_t)row * D;
  float4 v[NV];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    v[i] = *reinterpret_cast<const float4*>(xr + (i * 32 + lane) * 4);
    s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
  }
  const float m = warp_sum(s) * (1.0f / D);
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    v[i].x -= m; v[i].y -= m; v[i].z -= m; v[i].w -= m;
    q += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
  }
  const float r = rsqrtf(warp_sum(q) * (1.0f / D) + 1e-5f);
  if (lane == 0) {
    mu[row] = m;
    rstd[row] = r;
  }
  __half* yr = y16 + (size_t)row * D;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (i * 32 + lane) * 4;
    const float4 g = *reinterpret_cast<const float4*>(gamma + c);
    const float4 b = *reinterpret_cast<const float4*>(beta + c);
    __half2 lo = __floats2half2_rn(v[i].x * r * g.x + b.x, v[i].y * r * g.y + b.y);
    __half2 hi = __floats2half2_rn(v[i].z * r * g.z + b.z, v[i].w * r * g.w + b.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&lo);
    u.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(yr + c) = u;
  }
}

constexpr int LNB_WARPS = 4;

// Backward.  Each CTA owns a contiguous band of rows; warp w handles rows
// band0+w, band0+w+4, ...  Per-column partial sums of dy*xhat and dy are kept
// in the warp's private shared-memory strip, combined across the CTA's warps
// and written to scratch[block][2][D]; k_ln_param_final adds the blocks up in
// a fixed order.
__global__ void __launch_bounds__(LNB_WARPS * 32)
k_layernorm_bwd(const float* __restrict__ dy, const float* __restrict__ x,
                const float* __restrict__ gamma, const float* __restrict__ mu,
                const float* __restrict__ rstd, const float* __restrict__ dres,
                float* __restrict__ dx, __half* __restrict__ dx16, __half* __restrict__ dyxh16,
                __half* __restrict__ dy16, float* __restrict__ scratch, int rows, int D,
                int rows_per_block) {
  extern __shared__ float acc[];  // [LNB_WARPS][2][D] when scratch != nullptr
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* a_g = acc + (size_t)warp * 2 * D;
  float* a_b = a_g + D;
  if (scratch) {
    for (int d = lane; d < D; d += 32) {
      a_g[d] = 0.f;
      a_b[d] = 0.f;
    }
  }
  const int r0 = blockIdx.x * rows_per_block;
  const int r1 = min(rows, r0 + rows_per_block);
  const float inv = 1.0f / (float)D;
  for (int row = r0 + warp; row < r1; row += LNB_WARPS) {
    const int64_t base = (int64_t)row * D;
    const float m = mu[row], r = rstd[row];
    float s1 = 0.f, s2 = 0.f;
    for (int d = lane; d < D; d += 32) {
      float dyv = dy[base + d];
      float xh = (x[base + d] - m) * r;
      float dxh = dyv * gamma[d];
      s1 += dxh;
      s2 += dxh * xh;
      if (dyxh16) dyxh16[base + d] = __float2half_rn(dyv * xh);
      if (dy16) dy16[base + d] = __float2half_rn(dyv);
      if (scratch) {
        a_g[d] += dyv * xh;
        a_b[d] += dyv;
      }
    }
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
    for (int d = lane; d < D; d += 32) {
      float xh = (x[base + d] - m) * r;
      float dxh = dy[base + d] * gamma[d];
      float o = r * (dxh - s1 * inv - xh * s2 * inv);
      if (dres) o += dres[base + d];
      if (dx) dx[base + d] = o;
      if (dx16) dx16[base + d] = __float2half_rn(o);
    }
  }
  if (scratch) {
    __syncthreads();
    float* out = scratch + (size_t)blockIdx.x * 2 * D;
    for (int d = threadIdx.x; d < 2 * D; d += blockDim.x) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < LNB_WARPS; ++w) s += acc[(size_t)w * 2 * D + d];
      out[d] = s;
    }
  }
}

constexpr int LNF_SLICES = 32;

// Fixed-order reduction of the per-block partials: 32 columns x 32 slices per CTA,
// each slice adds every 32nd block, then the slices are added in order.
__global__ void __launch_bounds__(32 * LNF_SLICES)
k_ln_param_final(const float* __restrict__ scratch, float* __restrict__ dgamma,
                 float* __restrict__ dbeta, float* __restrict__ dxsum, int D, int nblocks,
                 int nparts) {
  __shared__ float red[LNF_SLICES][32];
  const int lane = threadIdx.x & 31, slice = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;  // column in [0, nparts*D): gamma, beta, (dx) parts
  const int W = nparts * D;
  float s = 0.f;
  if (c < W)
    for (int k = slice; k < nblocks; k += LNF_SLICES) s += scratch[(size_t)k * W + c];
  red[slice][lane] = s;
  __syncthreads();
  if (slice == 0 && c < W) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < LNF_SLICES; ++k) t += red[k][lane];
    if (c < D) dgamma[c] = t;
    else if (c < 2 * D) dbeta[c - D] = t;
    else dxsum[c - 2 * D] = t;
  }
}

// Vectorised backward for D = 128 * NV: a warp owns a row, each lane holds NV float4
// of x and dy in registers, and keeps its columns' dgamma/dbeta partial sums in
// registers across all the rows it visits.
constexpr int LNV_WARPS = 8;

template <int NV>
__global__ void __launch_bounds__(LNV_WARPS * 32)
k_layernorm_bwd_vec(const float* __restrict__ dy, const float* __restrict__ x,
                    const float* __restrict__ gamma, const float* __restrict__ mu,
                    const float* __restrict__ rstd, const float* __restrict__ dres,
                    float* __restrict__ dx, __half* __restrict__ dx16,
                    float* __restrict__ scratch, int rows, int nparts) {
  constexpr int D = NV * 128;
  pdl_trigger();
  pdl_wait();
  __shared__ float red[LNV_WARPS][32 * 4 + 4];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float4 g[NV], ag[NV], ab[NV], ax[NV];   // ax: column sums of the output (nparts == 3)
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    g[i] = *reinterpret_cast<const float4*>(gamma + (i * 32 + lane) * 4);
    ag[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    ab[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    ax[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const float inv = 1.0f / (float)D;
  const int warps_total = gridDim.x * LNV_WARPS;
  for (int row = blockIdx.x * LNV_WARPS + warp; row < rows; row += warps_total) {
    const size_t base = (size_t)row * D;
    const float m = mu[row], r = rstd[row];
    // all three streams of the row are requested before anything is consumed: the kernel
    // holds one CTA per SM (its registers), so memory latency is hidden by loads in flight
    // per warp, not by other warps
    float4 xv[NV], dv[NV], rv[NV];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      xv[i] = *reinterpret_cast<const float4*>(x + base + (i * 32 + lane) * 4);
      dv[i] = *reinterpret_cast<const float4*>(dy + base + (i * 32 + lane) * 4);
    }
    if (dres) {
#pragma unroll
      for (int i = 0; i < NV; ++i)
        rv[i] = *reinterpret_cast<const float4*>(dres + base + (i * 32 + lane) * 4);
    } else {
#pragma unroll
      for (int i = 0; i < NV; ++i) rv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      xv[i].x = (xv[i].x - m) * r; xv[i].y = (xv[i].y - m) * r;
      xv[i].z = (xv[i].z - m) * r; xv[i].w = (xv[i].w - m) * r;
      float a0 = dv[i].x * g[i].x, a1 = dv[i].y * g[i].y, a2 = dv[i].z * g[i].z, a3 = dv[i].w * g[i].w;
      s1 += a0 + a1 + a2 + a3;
      s2 += a0 * xv[i].x + a1 * xv[i].y + a2 * xv[i].z + a3 * xv[i].w;
      ag[i].x += dv[i].x * xv[i].x; ag[i].y += dv[i].y * xv[i].y;
      ag[i].z += dv[i].z * xv[i].z; ag[i].w += dv[i].w * xv[i].w;
      ab[i].x += dv[i].x; ab[i].y += dv[i].y; ab[i].z += dv[i].z; ab[i].w += dv[i].w;
    }
    s1 = warp_sum(s1) * inv;
    s2 = warp_sum(s2) * inv;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float4 o;
      o.x = r * (dv[i].x * g[i].x - s1 - xv[i].x * s2);
      o.y = r * (dv[i].y * g[i].y - s1 - xv[i].y * s2);
      o.z = r * (dv[i].z * g[i].z - s1 - xv[i].z * s2);
      o.w = r * (dv[i].w * g[i].w - s1 - xv[i].w * s2);
      const size_t off = base + (i * 32 + lane) * 4;
      o.x += rv[i].x; o.y += rv[i].y; o.z += rv[i].z; o.w += rv[i].w;
      if (dx) *reinterpret_cast<float4*>(dx + off) = o;
      if (dx16) {
        __half2 a = __floats2half2_rn(o.x, o.y), b = __floats2half2_rn(o.z, o.w);
        uint2 u;
        u.x = *reinterpret_cast<uint32_t*>(&a);
        u.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(dx16 + off) = u;
      }
      ax[i].x += o.x; ax[i].y += o.y; ax[i].z += o.z; ax[i].w += o.w;
    }
  }
  if (scratch) {
    // add the CTA's warps in a fixed order, one 128-column group at a time
    float* out = scratch + (size_t)blockIdx.x * nparts * D;
#pragma unroll
    for (int part = 0; part < 3; ++part) {
      if (part >= nparts) break;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        float4 v = part == 0 ? ag[i] : part == 1 ? ab[i] : ax[i];
        __syncthreads();
        *reinterpret_cast<float4*>(&red[warp][lane * 4]) = v;
        __syncthreads();
        if (warp == 0) {
          float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int w = 0; w < LNV_WARPS; ++w) {
            float4 u = *reinterpret_cast<const float4*>(&red[w][lane * 4]);
            t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
          }
          *reinterpret_cast<float4*>(out + part * D + (i * 32 + lane) * 4) = t;
        }
      }
    }
  }
}

// ---- attention softmax ---------------------------------------------------------------------

// One warp per (batch*head, query) row; causal; optional packed-sample start.
__global__ void k_attn_softmax(const float* __restrict__ s, const uint32_t* __restrict__ seg,
                               __half* __restrict__ p16, int64_t rows, int T, int H, float scale,
                               int fill_block) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
  if (row >= rows) return;
  const int64_t base = row * T;
  const int q = (int)(row % T);
  int st = 0;
  if (seg) st = (int)seg[(row / T / H) * T + q];
  float mx = -1e30f;
  for (int j = st + lane; j <= q; j += 32) mx = fmaxf(mx, s[base + j] * scale);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int j = st + lane; j <= q; j += 32) sum += __expf(s[base + j] * scale - mx);
  sum = warp_sum(sum);
  const float inv = 1.0f / sum;
  // zeros above the diagonal: to the end of the row, or only to the end of the
  // fill_block-wide tile the consumer's causal K range stops at
  const int jend = fill_block > 0 ? min(T, (q / fill_block + 1) * fill_block) : T;
  for (int j = lane; j < jend; j += 32) {
    float v = 0.f;
    if (j >= st && j <= q) v = __expf(s[base + j] * scale - mx) * inv;
    p16[base + j] = __float2half_rn(v);
  }
}

__global__ void k_attn_softmax_bwd(const float* __restrict__ dp, const __half* __restrict__ p16,
                                   __half* __restrict__ ds16, int64_t rows, int T, float scale,
                                   int fill_block) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
  if (row >= rows) return;
  const int64_t base = row * T;
  const int q = (int)(row % T);
  float dot = 0.f;
  for (int j = lane; j <= q; j += 32) dot += dp[base + j] * __half2float(p16[base + j]);
  dot = warp_sum(dot);
  const int jend = fill_block > 0 ? min(T, (q / fill_block + 1) * fill_block) : T;
  for (int j = lane; j < jend; j += 32) {
    float v = 0.f;
    if (j <= q) v = __half2float(p16[base + j]) * (dp[base + j] - dot) * scale;
    ds16[base + j] = __float2half_rn(v);
  }
}

// ---- AdamW -----------------------------------------------------------------------------------

__device__ __forceinline__ void adamw_one(float& w, float g, float& m, float& v, float lr, float b1,
                                          float b2, float bc1, float bc2, float eps, float wd) {
  m = b1 * m + (1.0f - b1) * g;
  v = b2 * v + (1.0f - b2) * g * g;
  float mh = m / bc1;
  float vh = v / bc2;
  w -= lr * (mh / (sqrtf(vh) + eps) + wd * w);
}

__global__ void k_adamw(float* __restrict__ w, const float* __restrict__ g, float* __restrict__ m,
                        float* __restrict__ v, __half* __restrict__ w16,
                        const float* __restrict__ hp, int64_t n, float wd) {
  const float lr = hp[0], b1 = hp[1], b2 = hp[2], bc1 = hp[3], bc2 = hp[4], eps = hp[5];
  const float gs = hp[6] != 0.0f ? hp[6] : 1.0f;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    float wi = w[i], mi = m[i], vi = v[i];
    adamw_one(wi, g[i] * gs, mi, vi, lr, b1, b2, bc1, bc2, eps, wd);
    w[i] = wi;
    m[i] = mi;
    v[i] = vi;
    if (w16) w16[i] = __float2half_rn(wi);
  }
}

struct AdamTensor {
  float* w;
  const float* g;
  float* m;
  float* v;
  __half* w16;
  int64_t n;
  float wd;
  int pad;
};

constexpr int ADAM_CHUNK = 4096;  // elements per block

// One launch for every parameter tensor: block b looks up (tensor, chunk).
__global__ void __launch_bounds__(TPB)
k_adamw_multi(const AdamTensor* __restrict__ tensors, const int2* __restrict__ blockmap,
              const float* __restrict__ hp) {
  pdl_trigger();
  pdl_wait();
  const float lr = hp[0], b1 = hp[1], b2 = hp[2], bc1 = hp[3], bc2 = hp[4], eps = hp[5];
  const float gs = hp[6] != 0.0f ? hp[6] : 1.0f;
  const int2 bm = blockmap[blockIdx.x];
  const AdamTensor t = tensors[bm.x];
  const int64_t lo = (int64_t)bm.y * ADAM_CHUNK;
  const int64_t hi = min(t.n, lo + ADAM_CHUNK);
  const bool vec = (((uintptr_t)t.w | (uintptr_t)t.g | (uintptr_t)t.m | (uintptr_t)t.v) & 15) == 0 &&
                   ((uintptr_t)t.w16 & 7) == 0;
  if (vec) {
    for (int64_t i = lo + threadIdx.x * 4; i + 3 < hi; i += TPB * 4) {
      float4 w = *reinterpret_cast<float4*>(t.w + i);
      float4 g = *reinterpret_cast<const float4*>(t.g + i);
      float4 m = *reinterpret_cast<float4*>(t.m + i);
      float4 v = *reinterpret_cast<float4*>(t.v + i);
      adamw_one(w.x, g.x * gs, m.x, v.x, lr, b1, b2, bc1, bc2, eps, t.wd);
      adamw_one(w.y, g.y * gs, m.y, v.y, lr, b1, b2, bc1, bc2, eps, t.wd);
      adamw_one(w.z, g.z * gs, m.z, v.z, lr, b1, b2, bc1, bc2, eps, t.wd);
      adamw_one(w.w, g.w * gs, m.w, v.w, lr, b1, b2, bc1, bc2, eps, t.wd);
      *reinterpret_cast<float4*>(t.w + i) = w;
      *reinterpret_cast<float4*>(t.m + i) = m;
      *reinterpret_cast<float4*>(t.v + i) = v;
      if (t.w16) {
        __half2 a = __floats2half2_rn(w.x, w.y), b = __floats2half2_rn(w.z, w.w);
        uint2 o;
        o.x = *reinterpret_cast<uint32_t*>(&a);
        o.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(t.w16 + i) = o;
      }
    }
    // ragged tail of this chunk (chunk length not a multiple of 4)
    int64_t tail = lo + ((hi - lo) & ~(int64_t)3);
    for (int64_t i = tail + threadIdx.x; i < hi; i += TPB) {
      float wi = t.w[i], mi = t.m[i], vi = t.v[i];
      adamw_one(wi, t.g[i] * gs, mi, vi, lr, b1, b2, bc1, bc2, eps, t.wd);
      t.w[i] = wi; t.m[i] = mi; t.v[i] = vi;
      if (t.w16) t.w16[i] = __float2half_rn(wi);
    }
  } else {
    for (int64_t i = lo + threadIdx.x; i < hi; i += TPB) {
      float wi = t.w[i], mi = t.m[i], vi = t.v[i];
      adamw_one(wi, t.g[i] * gs, mi, vi, lr, b1, b2, bc1, bc2, eps, t.wd);
      t.w[i] = wi; t.m[i] = mi; t.v[i] = vi;
      if (t.w16) t.w16[i] = __float2half_rn(wi);
    }
  }
}

struct AdamTable {
  AdamTensor* tensors = nullptr;
  int2* blockmap = nullptr;
  int nblocks = 0;
};

inline unsigned flat_grid(vkg_device* dev, int64_t n) {
  return vkg_blocks(n, TPB, (int64_t)dev->sm_count * 16);
}

}  // namespace

// ---- C ABI -----------------------------------------------------------------------------------

extern "C" int vkg_bias_act(vkg_device* dev, const float* acc, const float* bias, float* z, void* y16,
                            int64_t n, int ncol, int act) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(acc && bias && n > 0 && ncol > 0, "bias_act: bad arguments");
  k_bias_act<<<flat_grid(dev, n), TPB, 0, dev->stream>>>(acc, bias, z, (__half*)y16, n, ncol, act);
  return vkg_check_launch("bias_act");
}

extern "C" int vkg_bias_act_bwd(vkg_device* dev, const float* dy, const float* z, void* dz16,
                                float* dz32, int64_t n, int act) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(dy && z && n > 0, "bias_act_bwd: bad arguments");
  k_bias_act_bwd<<<flat_grid(dev, n), TPB, 0, dev->stream>>>(dy, z, (__half*)dz16, dz32, n, act);
  return vkg_check_launch("bias_act_bwd");
}

extern "C" int vkg_bias(vkg_device* dev, const float* acc, const float* bias, float* z, int64_t n,
                        int ncol) {
  return vkg_bias_act(dev, acc, bias, z, nullptr, n, ncol, VKG_ACT_NONE);
}

extern "C" int vkg_col_sum(vkg_device* dev, const float* g, float* sums, int ncol, int nrow) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(g && sums && ncol > 0 && nrow > 0, "col_sum: bad arguments");
  k_col_sum<<<vkg_blocks(ncol, 128), 128, 0, dev->stream>>>(g, sums, ncol, nrow);
  return vkg_check_launch("col_sum");
}

static int col_sum_chunks(int ncol, int nrow) {
  int col_blocks = (ncol + 255) / 256;               // the fp16 block width (fp32 blocks are 128)
  int want = (1184 + col_blocks - 1) / col_blocks;   // ~8 CTAs per SM on 148 SMs
  int max_chunks = (nrow + 31) / 32;               // at least 32 rows per chunk
  if (want > max_chunks) want = max_chunks;
  if (want < 1) want = 1;
  if (want > 1024) want = 1024;
  return want;
}

extern "C" int64_t vkg_col_sum_scratch_floats(int ncol, int nrow) {
  if (ncol <= 0 || nrow <= 0) return 0;
  return (int64_t)col_sum_chunks(ncol, nrow) * ncol;
}

int vkg_launch_col_sum_final(vkg_device* dev, const float* partial, float* sums, int ncol, int nchunk,
                             int accumulate) {
  if (dev->defer_finals) {
    dev->finals.push_back(vkg_final_entry{partial, {sums, nullptr, nullptr}, ncol, ncol, nchunk,
                                          accumulate, 0, 0});
    return 0;
  }
  k_col_sum_final<<<(ncol + 31) / 32, 32 * CSF_SLICES, 0, dev->stream>>>(partial, sums, ncol, nchunk,
                                                                         accumulate);
  return vkg_check_launch("col_sum_final");
}

extern "C" int vkg_col_sum_det(vkg_device* dev, const void* g, int g_dtype, float* sums,
                               float* scratch, int ncol, int nrow, int accumulate) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(g && sums && scratch && ncol > 0 && nrow > 0, "col_sum_det: bad arguments");
  VKG_REQUIRE(g_dtype == VKG_F32 || g_dtype == VKG_F16, "col_sum_det: dtype must be f32 or f16");
  int nchunk = col_sum_chunks(ncol, nrow);
  int rpc = (nrow + nchunk - 1) / nchunk;
  const int per_block = 32 * (g_dtype == VKG_F16 ? 8 : 4);
  const int vec_ok = (ncol % (per_block / 32) == 0) && (((uintptr_t)g & 15) == 0);
  dim3 grid((ncol + per_block - 1) / per_block, nchunk);
  if (g_dtype == VKG_F16)
    k_col_sum_partial<__half><<<grid, CS_WARPS * 32, 0, dev->stream>>>((const __half*)g, scratch,
                                                                        ncol, nrow, rpc, vec_ok);
  else
    k_col_sum_partial<float><<<grid, CS_WARPS * 32, 0, dev->stream>>>((const float*)g, scratch, ncol,
                                                                       nrow, rpc, vec_ok);
  if (vkg_check_launch("col_sum_partial")) return 1;
  k_col_sum_final<<<(ncol + 31) / 32, 32 * CSF_SLICES, 0, dev->stream>>>(scratch, sums, ncol, nchunk,
                                                                         accumulate);
  return vkg_check_launch("col_sum_final");
}

// ---- deferred final passes -------------------------------------------------------------
//
// The second stage of a two-stage column sum is a few microseconds of work behind a launch;
// a GPT-2-small backward has 49 of them (layernorm parameters, qkv and fc1 bias gradients),
// each between two large kernels.  While deferral is on they are collected on the host and
// vkg_finals_flush runs them all as ONE launch: the table travels as the kernel's parameter,
// a CTA finds its entry by its block number.  Results do not depend on timing: each column is
// added by 32 slices (slice s takes rows s, s + 32, ...) that are then added in order.
constexpr int FIN_SLICES = 32;
constexpr int FIN_MAX = 64;      // entries per launch: 64 * 56 bytes stay under the 4 KB limit
struct FinalTable {
  int n, reserved;
  vkg_final_entry e[FIN_MAX];
};

__global__ void __launch_bounds__(32 * FIN_SLICES)
k_finals_multi(const __grid_constant__ FinalTable tab) {
  pdl_trigger();
  pdl_wait();
  __shared__ float4 red4[FIN_SLICES][32];
  int e = 0;
  while (e + 1 < tab.n && (int)blockIdx.x >= tab.e[e + 1].first_block) ++e;
  const float* __restrict__ partial = tab.e[e].partial;
  const int W = tab.e[e].W, D = tab.e[e].D, nchunk = tab.e[e].nchunk;
  const int lane = threadIdx.x & 31, slice = threadIdx.x >> 5;
  if (tab.e[e].reserved) {
    // four columns per lane (W, D multiples of 4, 16-byte aligned rows): a block covers 128
    // columns with one 16-byte load per lane and row.  Per column the order of the additions is
    // the same as below -- slice s takes rows s, s + 32, ..., the slices are added in order.
    const int c = (((int)blockIdx.x - tab.e[e].first_block) * 32 + lane) * 4;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < W)
      for (int k = slice; k < nchunk; k += FIN_SLICES) {
        const float4 v = *reinterpret_cast<const float4*>(partial + (size_t)k * W + c);
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
    red4[slice][lane] = s;
    __syncthreads();
    if (slice == 0 && c < W) {
      float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int k = 0; k < FIN_SLICES; ++k) {
        const float4 u = red4[k][lane];
        t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
      }
      float4* d = reinterpret_cast<float4*>(tab.e[e].dst[c / D] + (c % D));
      if (tab.e[e].accumulate) {
        const float4 o = *d;
        t.x += o.x; t.y += o.y; t.z += o.z; t.w += o.w;
      }
      *d = t;
    }
    return;
  }
  float* red = reinterpret_cast<float*>(red4);       // [FIN_SLICES][32] floats
  const int c = ((int)blockIdx.x - tab.e[e].first_block) * 32 + lane;
  float s = 0.f;
  if (c < W)
    for (int k = slice; k < nchunk; k += FIN_SLICES) s += partial[(size_t)k * W + c];
  red[slice * 32 + lane] = s;
  __syncthreads();
  if (slice == 0 && c < W) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < FIN_SLICES; ++k) t += red[k * 32 + lane];
    float* d = tab.e[e].dst[c / D] + (c % D);
    *d = tab.e[e].accumulate ? *d + t : t;
  }
}

extern "C" int vkg_finals_defer(vkg_device* dev, int on) {
  if (vkg_bind(dev)) return 1;
  if (on < 0) dev->finals.clear();     // drop what an abandoned recording left behind
  VKG_REQUIRE(on > 0 || dev->finals.empty(), "finals_defer: %d final passes are pending; call vkg_finals_flush",
              (int)dev->finals.size());
  dev->defer_finals = on > 0;
  return 0;
}

extern "C" int vkg_finals_flush(vkg_device* dev) {
  if (vkg_bind(dev)) return 1;
  dev->defer_finals = false;
  std::vector<vkg_final_entry> todo;
  todo.swap(dev->finals);
  for (size_t i0 = 0; i0 < todo.size(); i0 += FIN_MAX) {
    FinalTable tab;
    memset(&tab, 0, sizeof(tab));
    int blocks = 0;
    for (size_t i = i0; i < todo.size() && i < i0 + FIN_MAX; ++i) {
      vkg_final_entry en = todo[i];
      VKG_REQUIRE(en.partial && en.dst[0] && en.W > 0 && en.D > 0 && en.W <= 3 * en.D && en.nchunk > 0 &&
                      (en.W <= en.D || en.dst[1]) && (en.W <= 2 * en.D || en.dst[2]),
                  "finals_flush: malformed entry");
      en.first_block = blocks;
      // 16-byte columns when every row of the partials and every destination allows it
      bool vec = en.W % 4 == 0 && en.D % 4 == 0 && ((uintptr_t)en.partial & 15) == 0;
      for (int d = 0; d < 3; ++d)
        if (en.dst[d] && ((uintptr_t)en.dst[d] & 15)) vec = false;
      en.reserved = vec ? 1 : 0;
      blocks += vec ? (en.W + 127) / 128 : (en.W + 31) / 32;
      tab.e[tab.n++] = en;
    }
    VKG_CUDA(vkg_launch(dev, VKG_K_SMALL, k_finals_multi, dim3((unsigned)blocks), dim3(32 * FIN_SLICES), 0, 1, tab));
    if (vkg_check_launch("finals_multi")) return 1;
  }
  return 0;
}

// ---- column sums for callers that cannot allocate -----------------------------------
//
// Some hosts of this library may not call cudaMalloc once they are running: a plugin
// loaded into a process whose memory pool is owned by someone else, or a real-time loop
// that must not take the allocator's locks.  For them the partial sums of the
// two-stage column reduction live in a fixed array inside the library image instead
// of caller-provided scratch.  Every GPU that loads the library carries the array
// (4 MiB) until the process exits.
constexpr int64_t COLSUM_STATIC_FLOATS = 1 << 20;
static __device__ __align__(256) float g_colsum_static[COLSUM_STATIC_FLOATS];

namespace {
std::mutex g_colsum_static_mu;
std::map<int, float*> g_colsum_static_ptr;   // device ordinal -> device address of the array

// The array's name is only a host-side handle here; kernels need its device address,
// which differs per device and is looked up once per device with that device current.
int colsum_static_address(vkg_device* dev, float** out) {
  std::lock_guard<std::mutex> lock(g_colsum_static_mu);
  auto it = g_colsum_static_ptr.find(dev->ordinal);
  if (it != g_colsum_static_ptr.end()) {
    *out = it->second;
    return 0;
  }
  if (dev->capturing) {
    // the look-up may load the module, which is not allowed while a stream is being captured
    vkg_set_error("col_sum_static: the first call on a device sets the array's address up and "
                  "must come before any stream capture on that device");
    return 1;
  }
  float* ptr = nullptr;
  cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_colsum_static);
  if (e != cudaSuccess || ptr == nullptr) {
    vkg_set_error("col_sum_static: cudaGetSymbolAddress failed on device %d: %s", dev->ordinal,
                  cudaGetErrorString(e));
    return 1;
  }
  g_colsum_static_ptr[dev->ordinal] = ptr;
  *out = ptr;
  return 0;
}
}  // namespace

extern "C" int64_t vkg_col_sum_static_max_floats(void) { return COLSUM_STATIC_FLOATS; }

extern "C" int vkg_col_sum_static(vkg_device* dev, const void* g, int g_dtype, float* sums, int ncol,
                                  int nrow, int accumulate) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(g && sums && ncol > 0 && nrow > 0, "col_sum_static: bad arguments");
  VKG_REQUIRE(g_dtype == VKG_F32 || g_dtype == VKG_F16, "col_sum_static: dtype must be f32 or f16");
  const int64_t need = vkg_col_sum_scratch_floats(ncol, nrow);
  VKG_REQUIRE(need <= COLSUM_STATIC_FLOATS,
              "col_sum_static: %d columns x %d rows needs %lld floats of partial sums, the built-in "
              "array holds %lld; use vkg_col_sum_det with your own scratch",
              ncol, nrow, (long long)need, (long long)COLSUM_STATIC_FLOATS);
  float* scratch = nullptr;
  if (colsum_static_address(dev, &scratch)) return 1;
  // Every partial the final pass reads is overwritten by the first pass of this same
  // call, so nothing left behind by an earlier call needs clearing.
  int nchunk = col_sum_chunks(ncol, nrow);
  int rpc = (nrow + nchunk - 1) / nchunk;
  const int per_block = 32 * (g_dtype == VKG_F16 ? 8 : 4);
  const int vec_ok = (ncol % (per_block / 32) == 0) && (((uintptr_t)g & 15) == 0);
  dim3 grid((ncol + per_block - 1) / per_block, nchunk);
  if (g_dtype == VKG_F16)
    k_col_sum_partial<__half><<<grid, CS_WARPS * 32, 0, dev->stream>>>((const __half*)g, scratch,
                                                                        ncol, nrow, rpc, vec_ok);
  else
    k_col_sum_partial<float><<<grid, CS_WARPS * 32, 0, dev->stream>>>((const float*)g, scratch, ncol,
                                                                       nrow, rpc, vec_ok);
  if (vkg_check_launch("col_sum_static partial")) return 1;
  k_col_sum_final<<<(ncol + 31) / 32, 32 * CSF_SLICES, 0, dev->stream>>>(scratch, sums, ncol, nchunk,
                                                                         accumulate);
  return vkg_check_launch("col_sum_static final");
}

extern "C" int vkg_softmax_ce(vkg_device* dev, const float* logits, const uint32_t* labels,
                              const float* w, void* dl16, float* dl32, float* loss, int rows,
                              int stride, int ncls, float grad_scale) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(logits && labels && loss && rows > 0 && stride >= ncls && ncls > 0,
              "softmax_ce: bad arguments");
  const bool aligned = stride % 4 == 0 && (((uintptr_t)logits | (uintptr_t)dl32) & 15) == 0 &&
                       ((uintptr_t)dl16 & 7) == 0;
  const int n4 = stride / 4;
  if (aligned && n4 > 4 * CE_THREADS && n4 <= 17 * CE_THREADS) {
    // wide rows: one read of the logits, everything else from registers
    const int nv = (n4 + CE_THREADS - 1) / CE_THREADS;
#define VKG_CE(NV)                                                                              \
  VKG_CUDA(vkg_launch(dev, VKG_K_CE, k_softmax_ce_reg<NV>, dim3((unsigned)rows), dim3(CE_THREADS), 0, 1, logits, \
                      labels, w, (__half*)dl16, dl32, loss, stride, ncls, grad_scale,             \
                      dev->sm_count * (NV <= 8 ? 2 : 1)))
    if (nv <= 8) VKG_CE(8);
    else if (nv <= 12) VKG_CE(12);
    else VKG_CE(17);
#undef VKG_CE
    return vkg_check_launch("softmax_ce_reg");
  }
  k_softmax_ce<<<rows, TPB, 0, dev->stream>>>(logits, labels, w, (__half*)dl16, dl32, loss, stride,
                                              ncls, grad_scale);
  return vkg_check_launch("softmax_ce");
}

extern "C" int vkg_adamw(vkg_device* dev, float* w, const float* g, float* m, float* v, void* w16,
                         const float* hp, int64_t n, float wd) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(w && g && m && v && hp && n > 0, "adamw: bad arguments");
  k_adamw<<<flat_grid(dev, n), TPB, 0, dev->stream>>>(w, g, m, v, (__half*)w16, hp, n, wd);
  return vkg_check_launch("adamw");
}

extern "C" int vkg_adamw_table_create(vkg_device* dev, int ntensors, float* const* w,
                                      const float* const* g, float* const* m, float* const* v,
                                      void* const* w16, const int64_t* n, const float* wd,
                                      void** table) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(ntensors > 0 && w && g && m && v && n && wd && table, "adamw_table: bad arguments");
  std::vector<AdamTensor> ts(ntensors);
  std::vector<int2> map;
  for (int i = 0; i < ntensors; ++i) {
    VKG_REQUIRE(n[i] > 0 && w[i] && g[i] && m[i] && v[i], "adamw_table: tensor %d is empty", i);
    ts[i].w = w[i]; ts[i].g = g[i]; ts[i].m = m[i]; ts[i].v = v[i];
    ts[i].w16 = w16 ? (__half*)w16[i] : nullptr;
    ts[i].n = n[i]; ts[i].wd = wd[i]; ts[i].pad = 0;
    int chunks = (int)((n[i] + ADAM_CHUNK - 1) / ADAM_CHUNK);
    for (int c = 0; c < chunks; ++c) map.push_back(make_int2(i, c));
  }
  AdamTable* t = new AdamTable();
  t->nblocks = (int)map.size();
  cudaError_t e = cudaMalloc(&t->tensors, ts.size() * sizeof(AdamTensor));
  if (e == cudaSuccess) e = cudaMalloc(&t->blockmap, map.size() * sizeof(int2));
  if (e == cudaSuccess)
    e = cudaMemcpy(t->tensors, ts.data(), ts.size() * sizeof(AdamTensor), cudaMemcpyHostToDevice);
  if (e == cudaSuccess)
    e = cudaMemcpy(t->blockmap, map.data(), map.size() * sizeof(int2), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    if (t->tensors) cudaFree(t->tensors);
    if (t->blockmap) cudaFree(t->blockmap);
    delete t;
    VKG_FAIL("adamw_table: %s", cudaGetErrorString(e));
  }
  *table = t;
  return 0;
}

extern "C" int vkg_adamw_table_destroy(vkg_device* dev, void* table) {
  if (!table) return 0;
  if (vkg_bind(dev)) return 1;
  AdamTable* t = (AdamTable*)table;
  cudaFree(t->tensors);
  cudaFree(t->blockmap);
  delete t;
  return 0;
}

extern "C" int vkg_adamw_multi(vkg_device* dev, void* table, const float* hp) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(table && hp, "adamw_multi: bad arguments");
  AdamTable* t = (AdamTable*)table;
  VKG_CUDA(vkg_launch(dev, VKG_K_ADAMW, k_adamw_multi, dim3((unsigned)t->nblocks), dim3(TPB), 0, 1, t->tensors,
                      t->blockmap, hp));
  return vkg_check_launch("adamw_multi");
}

extern "C" int vkg_cast16(vkg_device* dev, const float* src, void* dst16, int64_t n) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(src && dst16 && n > 0, "cast16: bad arguments");
  if ((n & 3) == 0 && (((uintptr_t)src & 15) == 0) && (((uintptr_t)dst16 & 7) == 0)) {
    k_cast16_v4<<<flat_grid(dev, n / 4), TPB, 0, dev->stream>>>((const float4*)src, (uint2*)dst16,
                                                                n / 4);
  } else {
    k_cast16<<<flat_grid(dev, n), TPB, 0, dev->stream>>>(src, (__half*)dst16, n);
  }
  return vkg_check_launch("cast16");
}

extern "C" int vkg_layernorm(vkg_device* dev, const float* x, const float* gamma, const float* beta,
                             void* y16, float* mu, float* rstd, int rows, int D) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(x && gamma && beta && y16 && mu && rstd && rows > 0 && D > 0, "layernorm: bad arguments");
  const int wpb = 4;
  const bool aligned = ((((uintptr_t)x | (uintptr_t)gamma | (uintptr_t)beta) & 15) == 0) &&
                       (((uintptr_t)y16 & 7) == 0);
  if (aligned && D % 128 == 0 && D <= 1024) {
    const unsigned grid = (rows + wpb - 1) / wpb;
#define VKG_LN(NV) \
  VKG_CUDA(vkg_launch(dev, VKG_K_LN, k_layernorm_vec<NV>, dim3(grid), dim3(wpb * 32), 0, 1, x, gamma, beta, \
                      (__half*)y16, mu, rstd, rows))
    switch (D / 128) {
      case 1: VKG_LN(1); break;
      case 2: VKG_LN(2); break;
      case 3: VKG_LN(3); break;
      case 4: VKG_LN(4); break;
      case 5: VKG_LN(5); break;
      case 6: VKG_LN(6); break;
      case 7: VKG_LN(7); break;
      default: VKG_LN(8); break;
    }
#undef VKG_LN
    return vkg_check_launch("layernorm_vec");
  }
  k_layernorm<<<(rows + wpb - 1) / wpb, wpb * 32, 0, dev->stream>>>(x, gamma, beta, (__half*)y16, mu,
                                                                    rstd, rows, D);
  return vkg_check_launch("layernorm");
}

static int ln_bwd_blocks(int rows) {
  int b = (rows + LNB_WARPS - 1) / LNB_WARPS;  // at least one row per warp
  if (b > 296) b = 296;
  if (b < 1) b = 1;
  return b;
}

extern "C" int64_t vkg_layernorm_bwd_scratch_floats(int rows, int D) {
  if (rows <= 0 || D <= 0) return 0;
  return (int64_t)ln_bwd_blocks(rows) * 3 * D;
}

template <int NV>
static void launch_ln_bwd_vec(vkg_device* dev, int nblocks, const float* dy, const float* x,
                              const float* gamma, const float* mu, const float* rstd,
                              const float* dres, float* dx, void* dx16, float* scratch, int rows,
                              int nparts) {
  // a failed launch is picked up by the caller's vkg_check_launch
  vkg_launch(dev, VKG_K_LN_BWD, k_layernorm_bwd_vec<NV>, dim3((unsigned)nblocks), dim3(LNV_WARPS * 32), 0, 1, dy, x,
             gamma, mu, rstd, dres, dx, (__half*)dx16, scratch, rows, nparts);
}

extern "C" int vkg_layernorm_bwd(vkg_device* dev, const float* dy, const float* x, const float* gamma,
                                 const float* mu, const float* rstd, const float* dres, float* dx,
                                 void* dx16, void* dyxh16, void* dy16, float* dgamma, float* dbeta,
                                 float* dxsum, float* scratch, int rows, int D) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(dy && x && gamma && mu && rstd && rows > 0 && D > 0, "layernorm_bwd: bad arguments");
  const bool fused = dgamma != nullptr || dbeta != nullptr;
  if (fused) VKG_REQUIRE(dgamma && dbeta && scratch, "layernorm_bwd: dgamma, dbeta and scratch go together");
  const int nparts = dxsum ? 3 : 2;
  VKG_REQUIRE(!dxsum || (fused && D % 128 == 0 && D <= 1024 && !dyxh16 && !dy16),
              "layernorm_bwd: dxsum needs dgamma/dbeta and D a multiple of 128 up to 1024");
  int nblocks = ln_bwd_blocks(rows);
  const bool aligned = ((((uintptr_t)dy | (uintptr_t)x | (uintptr_t)gamma | (uintptr_t)dres |
                          (uintptr_t)dx | (uintptr_t)scratch) & 15) == 0) && (((uintptr_t)dx16 & 7) == 0);
  if (D % 128 == 0 && D <= 1024 && !dyxh16 && !dy16 && aligned) {
    // register-resident rows; every CTA writes its partial sums (possibly zero)
    int nb = (rows + LNV_WARPS - 1) / LNV_WARPS;
    if (nb > nblocks) nb = nblocks;
    // from D = 640 on a CTA's registers (three row streams and three sets of column sums per
    // lane) leave room for one CTA per SM only: a second CTA per SM would run as a second wave
    if (D >= 640 && nb > dev->sm_count) nb = dev->sm_count;
    float* sc = fused ? scratch : nullptr;
    switch (D / 128) {
      case 1: launch_ln_bwd_vec<1>(dev, nb, dy, x, gamma, mu, rstd, dres, dx, dx16, sc, rows, nparts); break;
      case 2: launch_ln_bwd_vec<2>(dev, nb, dy, x, gamma, mu, rstd, dres, dx, dx16, sc, rows, nparts); break;
      case 3: launch_ln_bwd_vec<3>(dev, nb, dy, x, gamma, mu, rstd, dres, dx, dx16, sc, rows, nparts); break;
      case 4: launch_ln_bwd_vec<4>(dev, nb, dy, x, gamma, mu, rstd, dres, dx, dx16, sc, rows, nparts); break;
      case 5: launch_ln_bwd_vec<5>(dev, nb, dy, x, gamma, mu, rstd, dres, dx, dx16, sc, rows, nparts); break;
      case 6: launch_ln_bwd_vec<6>(dev, nb, dy, x, gamma, mu, rstd, dres, dx, dx16, sc, rows, nparts); break;
      case 7: launch_ln_bwd_vec<7>(dev, nb, dy, x, gamma, mu, rstd, dres, dx, dx16, sc, rows, nparts); break;
      default: launch_ln_bwd_vec<8>(dev, nb, dy, x, gamma, mu, rstd, dres, dx, dx16, sc, rows, nparts); break;
    }
    if (vkg_check_launch("layernorm_bwd_vec")) return 1;
    nblocks = nb;
  } else {
    int rpb = (rows + nblocks - 1) / nblocks;
    nblocks = (rows + rpb - 1) / rpb;
    size_t smem = fused ? (size_t)LNB_WARPS * 2 * D * sizeof(float) : 0;
    VKG_REQUIRE(smem <= 48 * 1024, "layernorm_bwd: fused parameter sums support D <= %d",
                48 * 1024 / (LNB_WARPS * 8));
    k_layernorm_bwd<<<nblocks, LNB_WARPS * 32, smem, dev->stream>>>(
        dy, x, gamma, mu, rstd, dres, dx, (__half*)dx16, (__half*)dyxh16, (__half*)dy16,
        fused ? scratch : nullptr, rows, D, rpb);
    if (vkg_check_launch("layernorm_bwd")) return 1;
  }
  if (fused) {
    VKG_REQUIRE(!dxsum || (D % 128 == 0 && D <= 1024 && aligned),
                "layernorm_bwd: dxsum needs 16-byte aligned operands");
    if (dev->defer_finals) {
      dev->finals.push_back(vkg_final_entry{scratch, {dgamma, dbeta, dxsum}, nparts * D, D, nblocks,
                                            0, 0, 0});
      return 0;
    }
    k_ln_param_final<<<(nparts * D + 31) / 32, 32 * LNF_SLICES, 0, dev->stream>>>(
        scratch, dgamma, dbeta, dxsum, D, nblocks, nparts);
    return vkg_check_launch("ln_param_final");
  }
  return 0;
}

extern "C" int vkg_attn_softmax(vkg_device* dev, const float* s, const uint32_t* seg, void* p16,
                                int64_t rows, int T, int H, float scale, int fill_block) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(s && p16 && rows > 0 && T > 0, "attn_softmax: bad arguments");
  const int wpb = 8;
  k_attn_softmax<<<(unsigned)((rows + wpb - 1) / wpb), wpb * 32, 0, dev->stream>>>(
      s, seg, (__half*)p16, rows, T, H > 0 ? H : 1, scale, fill_block);
  return vkg_check_launch("attn_softmax");
}

extern "C" int vkg_attn_softmax_bwd(vkg_device* dev, const float* dp, const void* p16, void* ds16,
                                    int64_t rows, int T, float scale, int fill_block) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(dp && p16 && ds16 && rows > 0 && T > 0, "attn_softmax_bwd: bad arguments");
  const int wpb = 8;
  k_attn_softmax_bwd<<<(unsigned)((rows + wpb - 1) / wpb), wpb * 32, 0, dev->stream>>>(
      dp, (const __half*)p16, (__half*)ds16, rows, T, scale, fill_block);
  return vkg_check_launch("attn_softmax_bwd");
}

extern "C" int vkg_split_qkv(vkg_device* dev, const float* qkv, const float* bias, void* q16,
                             void* k16, void* v16, int64_t n, int D, int T, int H, int hd) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(qkv && bias && q16 && k16 && v16 && n > 0, "split_qkv: bad arguments");
  k_split_qkv<<<flat_grid(dev, n), TPB, 0, dev->stream>>>(qkv, bias, (__half*)q16, (__half*)k16,
                                                          (__half*)v16, n, D, T, H, hd);
  return vkg_check_launch("split_qkv");
}

extern "C" int vkg_merge_qkv_grad(vkg_device* dev, const float* dq, const float* dk, const float* dv,
                                  void* dqkv16, int64_t n, int D, int T, int H, int hd) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(dq && dk && dv && dqkv16 && n > 0, "merge_qkv_grad: bad arguments");
  k_merge_qkv_grad<<<flat_grid(dev, n), TPB, 0, dev->stream>>>(dq, dk, dv, (__half*)dqkv16, n, D, T,
                                                               H, hd);
  return vkg_check_launch("merge_qkv_grad");
}

extern "C" int vkg_merge_heads(vkg_device* dev, const float* src, void* y16, int64_t n, int D, int T,
                               int H, int hd) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(src && y16 && n > 0, "merge_heads: bad arguments");
  k_merge_heads<<<flat_grid(dev, n), TPB, 0, dev->stream>>>(src, (__half*)y16, n, D, T, H, hd);
  return vkg_check_launch("merge_heads");
}

extern "C" int vkg_split_heads(vkg_device* dev, const float* src, void* dst16, int64_t n, int D,
                               int T, int H, int hd) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(src && dst16 && n > 0, "split_heads: bad arguments");
  k_split_heads<<<flat_grid(dev, n), TPB, 0, dev->stream>>>(src, (__half*)dst16, n, D, T, H, hd);
  return vkg_check_launch("split_heads");
}

extern "C" int vkg_embed(vkg_device* dev, const float* tok, const float* pos, const uint32_t* ids,
                         const uint32_t* seg, float* x, int64_t n, int D, int T) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(tok && pos && ids && x && n > 0, "embed: bad arguments");
  if (D % 4 == 0 && n < (1ll << 31) && ((((uintptr_t)tok | (uintptr_t)pos | (uintptr_t)x) & 15) == 0)) {
    VKG_CUDA(vkg_launch(dev, VKG_K_SMALL, k_embed_v4, dim3(flat_grid(dev, n / 4)), dim3(TPB), 0, 1, (const float4*)tok,
                        (const float4*)pos, ids, seg, (float4*)x, (int)(n / 4), D / 4, T));
    return vkg_check_launch("embed_v4");
  }
  k_embed<<<flat_grid(dev, n), TPB, 0, dev->stream>>>(tok, pos, ids, seg, x, n, D, T);
  return vkg_check_launch("embed");
}

extern "C" int vkg_embed_bwd(vkg_device* dev, const float* dx, const uint32_t* ids,
                             const uint32_t* seg, float* dtok, float* dpos, int64_t n, int D, int T) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(dx && ids && dtok && dpos && n > 0, "embed_bwd: bad arguments");
  if (D % 4 == 0 && n < (1ll << 31) && ((((uintptr_t)dx | (uintptr_t)dtok | (uintptr_t)dpos) & 15) == 0)) {
    VKG_CUDA(vkg_launch(dev, VKG_K_SMALL, k_embed_bwd_v4, dim3(flat_grid(dev, n / 4)), dim3(TPB), 0, 1,
                        (const float4*)dx, ids, seg, (float4*)dtok, (float4*)dpos, (int)(n / 4), D / 4, T));
    return vkg_check_launch("embed_bwd_v4");
  }
  k_embed_bwd<<<flat_grid(dev, n), TPB, 0, dev->stream>>>(dx, ids, seg, dtok, dpos, n, D, T);
  return vkg_check_launch("embed_bwd");
}

extern "C" int64_t vkg_embed_bwd_scratch_bytes(int64_t rows) {
  // keys[2][rows rounded up to 4], next[2][rows], has_prev[2][rows]
  return rows > 0 ? (6 * rows + 8) * (int64_t)sizeof(int) : 0;
}

extern "C" int vkg_embed_bwd_det(vkg_device* dev, const float* dx, const uint32_t* ids,
                                 const uint32_t* seg, float* dtok, float* dpos, void* scratch,
                                 int64_t n, int D, int T) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(dx && ids && dtok && dpos && scratch && n > 0 && D > 0 && T > 0,
              "embed_bwd_det: bad arguments");
  VKG_REQUIRE(D % 128 == 0 && D <= 1024 && n % D == 0 && n / D < (1ll << 30) &&
                  ((((uintptr_t)dx | (uintptr_t)dtok | (uintptr_t)dpos | (uintptr_t)scratch) & 15) == 0),
              "embed_bwd_det: D must be a multiple of 128 up to 1024 and the tables 16-byte aligned "
              "(use vkg_embed_bwd otherwise)");
  const int rows = (int)(n / D), rows_p = (rows + 3) & ~3;
  int* keys = static_cast<int*>(scratch);
  int* next = keys + 2 * (size_t)rows_p;
  int* has_prev = next + 2 * (size_t)rows;
  VKG_CUDA(vkg_launch(dev, VKG_K_SMALL, k_embed_keys, dim3((unsigned)((2 * rows_p + 255) / 256)),
                      dim3(256), 0, 1, ids, seg, keys, has_prev, rows, rows_p, T));
  if (vkg_check_launch("embed_keys")) return 1;
  VKG_CUDA(vkg_launch(dev, VKG_K_SMALL, k_embed_chain, dim3((unsigned)((2 * rows + 7) / 8)), dim3(256), 0,
                      1, (const int*)keys, next, has_prev, rows, rows_p));
  if (vkg_check_launch("embed_chain")) return 1;
  const dim3 grid((unsigned)((rows + 7) / 8), 2);
#define VKG_EB(NV)                                                                               \
  VKG_CUDA(vkg_launch(dev, VKG_K_SMALL, k_embed_bwd_chain<NV>, grid, dim3(256), 0, 1, dx, ids, seg, \
                      (const int*)next, (const int*)has_prev, dtok, dpos, rows, T))
  switch (D / 128) {
    case 1: VKG_EB(1); break;
    case 2: VKG_EB(2); break;
    case 3: VKG_EB(3); break;
    case 4: VKG_EB(4); break;
    case 5: VKG_EB(5); break;
    case 6: VKG_EB(6); break;
    case 7: VKG_EB(7); break;
    default: VKG_EB(8); break;
  }
#undef VKG_EB
  return vkg_check_launch("embed_bwd_chain");
}

extern "C" int vkg_residual(vkg_device* dev, const float* acc, const float* bias, const float* res,
                            float* out, int64_t n, int D) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(acc && bias && res && out && n > 0, "residual: bad arguments");
  k_residual<<<flat_grid(dev, n), TPB, 0, dev->stream>>>(acc, bias, res, out, n, D);
  return vkg_check_launch("residual");
}

extern "C" int vkg_add(vkg_device* dev, const float* a, const float* b, float* out, void* out16,
                       int64_t n) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(a && b && (out || out16) && n > 0, "add: bad arguments");
  k_add<<<flat_grid(dev, n), TPB, 0, dev->stream>>>(a, b, out, (__half*)out16, n);
  return vkg_check_launch("add");
}

extern "C" int vkg_add_bias(vkg_device* dev, float* x, const float* bias, int64_t n, int ncol) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(x && bias && n > 0 && ncol > 0, "add_bias: bad arguments");
  k_add_bias<<<flat_grid(dev, n), TPB, 0, dev->stream>>>(x, bias, n, ncol);
  return vkg_check_launch("add_bias");
}

extern "C" int vkg_grad_add(vkg_device* dev, const float* g, float* arena, int64_t n, int64_t off) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(g && arena && n > 0 && off >= 0, "grad_add: bad arguments");
  k_grad_add<<<flat_grid(dev, n), TPB, 0, dev->stream>>>(g, arena + off, n);
  return vkg_check_launch("grad_add");
}

extern "C" int vkg_grad_pull(vkg_device* dev, const float* arena, float* g, int64_t n, int64_t off,
                             float scale) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(g && arena && n > 0 && off >= 0, "grad_pull: bad arguments");
  k_grad_pull<<<flat_grid(dev, n), TPB, 0, dev->stream>>>(arena + off, g, n, scale);
  return vkg_check_launch("grad_pull");
}

extern "C" int vkg_bucket_pack16(vkg_device* dev, const float* src, void* dst16, int dtype, int64_t n,
                                 float scale) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(src && dst16 && n > 0, "bucket_pack16: bad arguments");
  if (dtype == VKG_F16)
    k_pack16<__half><<<flat_grid(dev, n), TPB, 0, dev->stream>>>(src, (__half*)dst16, n, scale);
  else if (dtype == VKG_BF16)
    k_pack16<__nv_bfloat16><<<flat_grid(dev, n), TPB, 0, dev->stream>>>(src, (__nv_bfloat16*)dst16, n,
                                                                         scale);
  else
    VKG_FAIL("bucket_pack16: dtype must be f16 or bf16");
  return vkg_check_launch("bucket_pack16");
}

extern "C" int vkg_bucket_unpack16(vkg_device* dev, const void* src16, int dtype, float* dst,
                                   int64_t n, float scale) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(src16 && dst && n > 0, "bucket_unpack16: bad arguments");
  if (dtype == VKG_F16)
    k_unpack16<__half><<<flat_grid(dev, n), TPB, 0, dev->stream>>>((const __half*)src16, dst, n, scale);
  else if (dtype == VKG_BF16)
    k_unpack16<__nv_bfloat16><<<flat_grid(dev, n), TPB, 0, dev->stream>>>((const __nv_bfloat16*)src16,
                                                                           dst, n, scale);
  else
    VKG_FAIL("bucket_unpack16: dtype must be f16 or bf16");
  return vkg_check_launch("bucket_unpack16");
}
