// The GEMM trio (Y = X W, dX = dY W^T, dW = X^T dY) and its batched form for
// sm_100a: TMA -> 128B-swizzled shared memory ring -> tcgen05.mma issued by one
// thread -> fp32 accumulators in TMEM (two stages, so the epilogue of tile i
// overlaps the main loop of tile i+1) -> tcgen05.ld epilogue with the fused
// bias / activation / activation-derivative / residual / narrowing.
//
// One persistent CTA per SM, 576 threads:
//   warp 0       TMA producer (one lane)
//   warp 1       TMEM allocation + MMA issue (converged, one elected lane per instruction)
//   warps 2..17  epilogue; warp w reads TMEM lanes 32*(w%4) .. +31 and takes every
//                fourth 16-column chunk.  The epilogue is instruction-issue / latency
//                bound, so it gets four warps per scheduler and a compile-time mask.
//
// Transposed operands are never materialised (the reference makes the same
// point for its cooperative-matrix loads, kernels.py:45-49): "A stored K x M"
// and "B stored K x N" are loaded as MN-major tiles and the shared-memory /
// instruction descriptors say so.
//
// Two kernels share the role code: gemm_tcgen05_kernel (128 x {64..256} tiles, one CTA
// each) and gemm_cta_pair_kernel (256 x 256 tiles on 2-CTA clusters with
// tcgen05.mma.cta_group::2, each CTA loading its rows of A and half of the B tile), which
// the host picks for launches with many waves of tiles and for split-K shapes.
//
// Every mbarrier wait is bounded by a clock64 budget; a wait that gives up
// sets an error word the host reads at the next synchronisation, the CTA
// stops issuing work, frees its TMEM and returns.
#include "common.cuh"
#include "tcgen05.cuh"

namespace {

using namespace tc05;

constexpr int BM = 128;            // rows of C per tile = UMMA M
constexpr int BK = 64;             // K elements per stage = 128 bytes of f16 = one swizzle row
constexpr int UMMA_K = 16;         // K per tcgen05.mma.kind::f16
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int MAX_STAGES = 8;
constexpr int EPI_WARPS = 16;      // four per TMEM lane quarter, each takes every fourth 16-column chunk
constexpr int NUM_THREADS = (2 + EPI_WARPS) * 32;
constexpr int TMEM_COLS = 512;     // whole TMEM: two 256-column accumulators
constexpr int ACC_COLS = 256;
constexpr int RING_BYTES = 196608; // shared-memory ring budget
constexpr int EPI_STAGE_BYTES = 32 * 16 * 4;  // one 32x16 fp32 chunk per epilogue warp (XOR-swizzled)
constexpr int SMEM_BYTES = RING_BYTES + EPI_WARPS * EPI_STAGE_BYTES + 1024 /*align slack*/ +
                           256 /*barriers*/;
constexpr int GROUP_M = 8;         // m-tiles per rasterisation band

struct GemmParams {
  int M, N, K;
  int nb0, nb1;
  int tiles_m, tiles_n;
  int bn, stages, num_kb;
  int split_k, kb_per_split;   // split_k > 1: z1 is the K slice, not a batch index
  int causal;                  // 0 none, 1 skip tiles above the diagonal, 2/3 clip the K range
  int a_mn, b_mn;
  uint32_t idesc;
  int c_dtype, act, dact, vec_ok;
  long long ldc, sC0, sC1;
  void* C;
  void* C2;
  const float* bias;
  float* pre;
  const float* dact_z;
  const float* residual;
  float* colsum;               // optional: [4 * row blocks][N] partial column sums of the output
  float alpha;
  int tma_store;               // epilogue stores C (and pre) through tensor maps
  uint32_t* err;
};

struct TileCoord {
  int z0, z1, m0, n0;
};

// bm: rows of C per tile (BM, or 2 * BM for a CTA pair); m_off: this CTA's rows inside it.
__device__ __forceinline__ TileCoord tile_coord(const GemmParams& p, int t, int bm = BM, int m_off = 0) {
  int per_batch = p.tiles_m * p.tiles_n;
  int z = t / per_batch;
  int r = t - z * per_batch;
  int band = GROUP_M * p.tiles_n;
  int g = r / band;
  int first_m = g * GROUP_M;
  int gsize = min(p.tiles_m - first_m, GROUP_M);
  int in_band = r - g * band;
  TileCoord c;
  c.m0 = (first_m + in_band % gsize) * bm + m_off;
  c.n0 = (in_band / gsize) * p.bn;
  c.z0 = z % p.nb0;
  c.z1 = z / p.nb0;
  return c;
}

// K-block range of a work unit: everything, slice z1 when K is split, or the part of K
// a causal operand is non-zero in.  nkb == 0 means the tile is skipped by every role.
__device__ __forceinline__ void kb_range(const GemmParams& p, const TileCoord& c, int& kb0, int& nkb) {
  if (p.split_k > 1) {
    kb0 = c.z1 * p.kb_per_split;
    nkb = min(p.kb_per_split, p.num_kb - kb0);
  } else {
    kb0 = 0;
    nkb = p.num_kb;
    if (p.causal == 1) {
      if (c.n0 > c.m0 + BM - 1) nkb = 0;                  // wholly above the diagonal
    } else if (p.causal == 2) {
      nkb = min(p.num_kb, (c.m0 + BM + BK - 1) / BK);    // A[m, k] = 0 for k > m
    } else if (p.causal == 3) {
      kb0 = c.m0 / BK;                                    // A^T[k, m] = 0 for k < m
      nkb = p.num_kb - kb0;
    }
  }
}

// Compile-time epilogue feature mask.  E_GENERIC reads every flag (and the vector
// alignment flag) at run time; the specialised masks assume 16-byte aligned operands.
enum : int {
  E_BIAS = 1, E_PRE = 2, E_ACT = 4, E_DACT = 8, E_RES = 16, E_C2 = 32, E_F16 = 64, E_BF16 = 128,
  E_COLSUM = 256,
  E_GENERIC = 1 << 20
};

template <typename T2, typename T>
__device__ __forceinline__ void store4_16(T* c, const float* v, bool vec);

template <>
__device__ __forceinline__ void store4_16<__half2, __half>(__half* c, const float* v, bool vec) {
  if (vec) {
    __half2 h[2] = {__floats2half2_rn(v[0], v[1]), __floats2half2_rn(v[2], v[3])};
    *reinterpret_cast<uint2*>(c) = *reinterpret_cast<uint2*>(h);
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) c[j] = __float2half_rn(v[j]);
  }
}

template <>
__device__ __forceinline__ void store4_16<__nv_bfloat162, __nv_bfloat16>(__nv_bfloat16* c,
                                                                         const float* v, bool vec) {
  if (vec) {
    __nv_bfloat162 h[2] = {__floats2bfloat162_rn(v[0], v[1]), __floats2bfloat162_rn(v[2], v[3])};
    *reinterpret_cast<uint2*>(c) = *reinterpret_cast<uint2*>(h);
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) c[j] = __float2bfloat16_rn(v[j]);
  }
}

__device__ __forceinline__ float4 ld4(const float* p, long long off, bool vec) {
  if (vec) return *reinterpret_cast<const float4*>(p + off);
  return make_float4(p[off], p[off + 1], p[off + 2], p[off + 3]);
}

__device__ __forceinline__ void st4(float* p, long long off, float4 v, bool vec) {
  if (vec) {
    *reinterpret_cast<float4*>(p + off) = v;
  } else {
    p[off] = v.x; p[off + 1] = v.y; p[off + 2] = v.z; p[off + 3] = v.w;
  }
}

// One lane's share of a 32x16 chunk through the fused epilogue: four rows (8*i +
// sub_row), four consecutive columns each.  In this layout four lanes cover the 16
// columns (64 bytes) of one row, so every global access of the warp is eight
// row-contiguous 64-byte pieces.  All loads of one kind are issued before the first
// dependent use: C may alias the inputs as far as the compiler knows, so a
// load-compute-store loop would serialise eight memory round trips.
//
// lanes: the lanes of the warp that call this together (those whose columns exist).
// cs_row: which row of p.colsum this warp's 32 rows add up into.  The sums are taken over
// the values as stored (after the narrowing), rows in a fixed order: lanes first add their
// four rows, then the eight row groups are folded by shuffles.
template <int MODE>
__device__ __forceinline__ void epilogue_chunk(const GemmParams& p, float4 (&v)[4],
                                               const long long (&off)[4], unsigned ok, int col,
                                               int cs_row, unsigned lanes) {
  constexpr bool G = (MODE & E_GENERIC) != 0;
  const bool has_colsum = G ? (p.colsum != nullptr) : (MODE & E_COLSUM) != 0;
  const bool vec = G ? (p.vec_ok != 0) : true;
  const bool has_bias = G ? (p.bias != nullptr) : (MODE & E_BIAS) != 0;
  const bool has_pre = G ? (p.pre != nullptr) : (MODE & E_PRE) != 0;
  const bool has_act = G ? (p.act != 0) : (MODE & E_ACT) != 0;
  const bool has_dact = G ? (p.dact_z != nullptr) : (MODE & E_DACT) != 0;
  const bool has_res = G ? (p.residual != nullptr) : (MODE & E_RES) != 0;
  const bool has_c2 = G ? (p.C2 != nullptr) : (MODE & E_C2) != 0;
  const int c_dtype = G ? p.c_dtype : ((MODE & E_F16) ? VKG_F16 : (MODE & E_BF16) ? VKG_BF16 : VKG_F32);
  float4 extra[4];
  if (has_dact) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      extra[i] = (ok >> i) & 1u ? ld4(p.dact_z, off[i], vec) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
  if (has_bias) b = ld4(p.bias, col, vec);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[i].x = v[i].x * p.alpha + b.x; v[i].y = v[i].y * p.alpha + b.y;
    v[i].z = v[i].z * p.alpha + b.z; v[i].w = v[i].w * p.alpha + b.w;
  }
  if (has_pre) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if ((ok >> i) & 1u) st4(p.pre, off[i], v[i], vec);
  }
  if (has_act) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[i].x = vkg_act(v[i].x, p.act); v[i].y = vkg_act(v[i].y, p.act);
      v[i].z = vkg_act(v[i].z, p.act); v[i].w = vkg_act(v[i].w, p.act);
    }
  }
  if (has_dact) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[i].x *= vkg_dact(extra[i].x, p.dact); v[i].y *= vkg_dact(extra[i].y, p.dact);
      v[i].z *= vkg_dact(extra[i].z, p.dact); v[i].w *= vkg_dact(extra[i].w, p.dact);
    }
  }
  if (has_res) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      extra[i] = (ok >> i) & 1u ? ld4(p.residual, off[i], vec) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[i].x += extra[i].x; v[i].y += extra[i].y; v[i].z += extra[i].z; v[i].w += extra[i].w;
    }
  }
  if (has_colsum) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (!((ok >> i) & 1u)) continue;
      float4 t = v[i];
      if (c_dtype == VKG_F16) {
        t.x = __half2float(__float2half_rn(t.x)); t.y = __half2float(__float2half_rn(t.y));
        t.z = __half2float(__float2half_rn(t.z)); t.w = __half2float(__float2half_rn(t.w));
      } else if (c_dtype == VKG_BF16) {
        t.x = __bfloat162float(__float2bfloat16_rn(t.x)); t.y = __bfloat162float(__float2bfloat16_rn(t.y));
        t.z = __bfloat162float(__float2bfloat16_rn(t.z)); t.w = __bfloat162float(__float2bfloat16_rn(t.w));
      }
      s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
    }
#pragma unroll
    for (int d = 4; d < 32; d <<= 1) {
      s.x += __shfl_xor_sync(lanes, s.x, d);
      s.y += __shfl_xor_sync(lanes, s.y, d);
      s.z += __shfl_xor_sync(lanes, s.z, d);
      s.w += __shfl_xor_sync(lanes, s.w, d);
    }
    if ((threadIdx.x & 31) < 4) st4(p.colsum, (long long)cs_row * p.N + col, s, vec);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (!((ok >> i) & 1u)) continue;
    const float f[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
    if (c_dtype == VKG_F32) {
      st4(reinterpret_cast<float*>(p.C), off[i], v[i], vec);
    } else if (c_dtype == VKG_F16) {
      store4_16<__half2, __half>(reinterpret_cast<__half*>(p.C) + off[i], f, vec);
    } else {
      store4_16<__nv_bfloat162, __nv_bfloat16>(reinterpret_cast<__nv_bfloat16*>(p.C) + off[i], f, vec);
    }
    if (has_c2) store4_16<__half2, __half>(reinterpret_cast<__half*>(p.C2) + off[i], f, vec);
  }
}

// Epilogues that only WRITE (plain, bias, bias + keep z + activation, narrowing) can leave the
// transposition to the TMA: the warp keeps the TMEM layout (lane = row, 16 columns), applies
// the fused arithmetic in registers, writes its 32 x 16 chunk into the staging area in the
// hardware's swizzled layout and one lane issues a tensor-map store of the box.  Compared
// with the per-lane path this drops the shared-memory read-back, the address arithmetic, the
// predicates (the box is clipped at the tensor's edge) and the global store instructions.
constexpr int E_NO_TMA = E_DACT | E_RES | E_C2 | E_COLSUM | E_GENERIC;

// 32 x 16 fp32: 64-byte rows, 16-byte piece j of row r at ((j ^ ((r >> 1) & 3)) << 4) -- the
// 64-byte swizzle of the tensor map, and conflict-free for one-row-per-lane writes.
__device__ __forceinline__ void stage_chunk_f32(const float (&v)[16], uint8_t* stage, int lane) {
#pragma unroll
  for (int j = 0; j < 4; ++j)
    *reinterpret_cast<float4*>(stage + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4)) =
        make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
}

// 32 x 16 halves: 32-byte rows, piece j of row r at ((j ^ ((r >> 2) & 1)) << 4) (32-byte swizzle)
template <bool BF>
__device__ __forceinline__ void stage_chunk_16(const float (&v)[16], uint8_t* stage, int lane) {
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    uint4 pk;
    uint32_t* w = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (BF) {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * j + 2 * e], v[8 * j + 2 * e + 1]);
        w[e] = *reinterpret_cast<uint32_t*>(&h);
      } else {
        __half2 h = __floats2half2_rn(v[8 * j + 2 * e], v[8 * j + 2 * e + 1]);
        w[e] = *reinterpret_cast<uint32_t*>(&h);
      }
    }
    *reinterpret_cast<uint4*>(stage + lane * 32 + ((j ^ ((lane >> 2) & 1)) << 4)) = pk;
  }
}

// One 32 x 16 chunk (rows row0.., columns col..) through the write-only epilogue.  The staging
// area is reused as soon as the previous store has finished reading it; bulk async-groups
// belong to the issuing thread, so lane 0 waits and the warp meets it.
template <int MODE>
__device__ __forceinline__ void epilogue_chunk_tma(const GemmParams& p, const CUtensorMap* tmC,
                                                   const CUtensorMap* tmP, const uint32_t (&r)[16],
                                                   uint8_t* stage, int lane, int col, int row0, int z0,
                                                   int z1) {
  float v[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
  if (MODE & E_BIAS) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      if (col + 4 * g < p.N) {       // N is a multiple of 8, the chunk may reach 8 past it
        const float4 b = *reinterpret_cast<const float4*>(p.bias + col + 4 * g);
        v[4 * g] += b.x; v[4 * g + 1] += b.y; v[4 * g + 2] += b.z; v[4 * g + 3] += b.w;
      }
    }
  }
  const uint32_t stage_s = smem_u32(stage);
  if (MODE & E_PRE) {
    if (lane == 0) bulk_wait_read_all();
    __syncwarp();
    stage_chunk_f32(v, stage, lane);
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_4d(tmP, stage_s, col, row0, z0, z1);
      bulk_commit_group();
    }
  }
  if (MODE & E_ACT) {
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = vkg_act(v[j], p.act);
  }
  if (lane == 0) bulk_wait_read_all();
  __syncwarp();
  if (MODE & E_F16) stage_chunk_16<false>(v, stage, lane);
  else if (MODE & E_BF16) stage_chunk_16<true>(v, stage, lane);
  else stage_chunk_f32(v, stage, lane);
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) {
    tma_store_4d(tmC, stage_s, col, row0, z0, z1);
    bulk_commit_group();
  }
}

// Per-CTA constants shared by the three roles.
struct CtaCtx {
  uint32_t base, stage_bytes, full0, empty0, tfull0, tempty0, tmem_base;
  int n_stages;
  volatile uint32_t* abort_flag;
  uint8_t* epi_stage;
};

// TMA producer (one lane): stream the operand k-blocks of work unit t into the ring.
__device__ __forceinline__ bool produce_unit(const CtaCtx& cx, const GemmParams& p,
                                             const CUtensorMap* tmA, const CUtensorMap* tmB, int t,
                                             int& stage, uint32_t& phase) {
  TileCoord tc = tile_coord(p, t);
  int kb0, nkb;
  kb_range(p, tc, kb0, nkb);
  if (p.split_k > 1) tc.z1 = 0;   // operands are not batched along the slice index
  for (int kb = 0; kb < nkb; ++kb) {
    if (!mbar_wait(cx.empty0 + 8 * stage, phase ^ 1u, cx.abort_flag, p.err, 0x100u + stage)) return false;
    const uint32_t fb = cx.full0 + 8 * stage;
    mbar_expect_tx(fb, cx.stage_bytes);
    const uint32_t sa = cx.base + stage * cx.stage_bytes;
    const uint32_t sb = sa + A_STAGE_BYTES;
    const int k0 = (kb0 + kb) * BK;
    if (!p.a_mn) {
      tma_load_4d(sa, tmA, fb, k0, tc.m0, tc.z0, tc.z1);
    } else {
      tma_load_4d(sa, tmA, fb, tc.m0, k0, tc.z0, tc.z1);
      tma_load_4d(sa + 8192, tmA, fb, tc.m0 + 64, k0, tc.z0, tc.z1);
    }
    if (!p.b_mn) {
      tma_load_4d(sb, tmB, fb, k0, tc.n0, tc.z0, tc.z1);
    } else {
      for (int g = 0; g < p.bn / 64; ++g)
        tma_load_4d(sb + g * 8192, tmB, fb, tc.n0 + 64 * g, k0, tc.z0, tc.z1);
    }
    if (++stage == cx.n_stages) {
      stage = 0;
      phase ^= 1u;
    }
  }
  return true;
}

// MMA issue (the whole warp, converged; one elected lane issues each instruction): accumulate
// work unit t into one of the two TMEM accumulators.
__device__ __forceinline__ bool mma_unit(const CtaCtx& cx, const GemmParams& p, int t, int& stage,
                                         uint32_t& phase, int& acc, uint32_t& acc_phase) {
  int kb0, nkb;
  kb_range(p, tile_coord(p, t), kb0, nkb);
  if (nkb <= 0) return true;   // skipped tile: no accumulator, no epilogue
  if (!mbar_wait_warp(cx.tempty0 + 8 * acc, acc_phase ^ 1u, cx.abort_flag, p.err, 0x200u + acc)) return false;
  tcgen05_fence_after();
  const uint32_t d_tmem = cx.tmem_base + (uint32_t)(acc * ACC_COLS);
  // Descriptor halves of ring stage 0; a K step of 16 elements is 32 bytes further along the
  // 128-byte row for a K-major operand and two 8-row groups (2 x 1024 bytes) further down for
  // an MN-major one; a stage is stage_bytes further on.  All in units of 16 bytes.
  const uint32_t d_hi = smem_desc_hi(1024);
  const uint32_t a_lo0 = smem_desc_lo(cx.base, p.a_mn ? 8192 : 16);
  const uint32_t b_lo0 = smem_desc_lo(cx.base + A_STAGE_BYTES, p.b_mn ? 8192 : 16);
  const uint32_t a_step = p.a_mn ? 128u : 2u, b_step = p.b_mn ? 128u : 2u;
  const uint32_t stage16 = cx.stage_bytes >> 4;
  for (int kb = 0; kb < nkb; ++kb) {
    if (!mbar_wait_warp(cx.full0 + 8 * stage, phase, cx.abort_flag, p.err, 0x300u + stage)) return false;
    tcgen05_fence_after();
    const uint32_t a_lo = a_lo0 + (uint32_t)stage * stage16, b_lo = b_lo0 + (uint32_t)stage * stage16;
#pragma unroll
    for (int k = 0; k < BK / UMMA_K; ++k)
      if (elect_one())
        umma_f16(d_tmem, smem_desc_pack(a_lo + k * a_step, d_hi), smem_desc_pack(b_lo + k * b_step, d_hi),
                 p.idesc, (kb | k) != 0 ? 1u : 0u);
    umma_commit_one(cx.empty0 + 8 * stage);  // frees the stage when these MMAs retire
    if (++stage == cx.n_stages) {
      stage = 0;
      phase ^= 1u;
    }
  }
  umma_commit_one(cx.tfull0 + 8 * acc);  // accumulator complete -> epilogue
  acc ^= 1;
  if (acc == 0) acc_phase ^= 1u;
  return true;
}

// Epilogue warp: drain this warp's share of the accumulator of work unit t.
template <int MODE>
__device__ __forceinline__ bool epilogue_unit(const CtaCtx& cx, const GemmParams& p,
                                              const CUtensorMap* tmC, const CUtensorMap* tmP, int t,
                                              int warp, int lane, int& acc, uint32_t& acc_phase) {
  const int q = warp & 3;  // TMEM lane quarter this warp may read
  TileCoord tc = tile_coord(p, t);
  {
    int kb0, nkb;
    kb_range(p, tc, kb0, nkb);
    if (nkb <= 0) return true;
  }
  if (!mbar_wait_warp(cx.tfull0 + 8 * acc, acc_phase, cx.abort_flag, p.err, 0x400u + acc)) return false;
  tcgen05_fence_after();
  // TMEM gives each lane one row; the chunk is transposed through shared memory so
  // that global loads and stores are row-contiguous (4 lanes x 16 B per row).  Rows
  // are 64 B apart with the 16-byte chunk index XOR-ed by (row >> 1) & 3: conflict-free
  // both for the row-per-lane writes and the row-contiguous reads.
  uint8_t* stage = cx.epi_stage + (warp - 2) * EPI_STAGE_BYTES;
  const int sub_row = lane >> 2;        // 0..7: row within a group of eight
  const int sub_chunk = lane & 3;       // which 16-byte chunk (4 columns) of the row
  const long long batch_off = (long long)tc.z0 * p.sC0 + (long long)tc.z1 * p.sC1;
  const int row_base = tc.m0 + q * 32;
  const uint32_t t_row = cx.tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * ACC_COLS);
  const bool tma_out = (MODE & E_NO_TMA) == 0 && p.tma_store != 0;
  for (int c0 = 16 * ((warp - 2) >> 2); c0 < p.bn; c0 += 64) {
    if (tc.n0 + c0 >= p.N) break;  // uniform across the warp
    uint32_t r[16];
    tmem_ld16(t_row + c0, r);
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    if ((MODE & E_NO_TMA) == 0 && tma_out) {
      if (row_base < p.M)
        epilogue_chunk_tma<MODE>(p, tmC, tmP, r, stage, lane, tc.n0 + c0, row_base, tc.z0, tc.z1);
      continue;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
      *reinterpret_cast<uint4*>(stage + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4)) =
          make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
    __syncwarp();
    const int col = tc.n0 + c0 + sub_chunk * 4;
    const unsigned lanes = __ballot_sync(0xffffffffu, col < p.N);
    if (col < p.N) {
      float4 v[4];
      long long off[4];
      unsigned ok = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int rr = 8 * i + sub_row;
        const int row = row_base + rr;
        v[i] = *reinterpret_cast<const float4*>(stage + rr * 64 + ((sub_chunk ^ ((rr >> 1) & 3)) << 4));
        off[i] = batch_off + (long long)row * p.ldc + col;
        ok |= (row < p.M ? 1u : 0u) << i;
      }
      epilogue_chunk<MODE>(p, v, off, ok, col, (tc.m0 / BM) * 4 + q, lanes);
    }
    __syncwarp();
  }
  tcgen05_fence_before();
  __syncwarp();
  if (lane == 0) mbar_arrive(cx.tempty0 + 8 * acc);
  acc ^= 1;
  if (acc == 0) acc_phase ^= 1u;
  return true;
}

// Barriers, TMEM and the role-independent constants of a CTA.
__device__ __forceinline__ void cta_setup(CtaCtx& cx, uint8_t* smem_raw, int bn, int stages) {
  // 128B-swizzled tiles want 1024-byte alignment.
  cx.base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (cx.base - smem_u32(smem_raw));
  cx.stage_bytes = A_STAGE_BYTES + (uint32_t)bn * 128u;
  cx.n_stages = stages;
  // Epilogue staging (one swizzled 32x16 fp32 chunk per epilogue warp), then the barrier block.
  cx.epi_stage = gen_base + RING_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(gen_base + RING_BYTES + EPI_WARPS * EPI_STAGE_BYTES);
  const uint32_t bar_base = cx.base + RING_BYTES + EPI_WARPS * EPI_STAGE_BYTES;
  // full[s] at +8s, empty[s] at +64+8s, tmem_full[a] at +128+8a, tmem_empty[a] at +144+8a
  cx.full0 = bar_base;
  cx.empty0 = bar_base + 64;
  cx.tfull0 = bar_base + 128;
  cx.tempty0 = bar_base + 144;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 20);
  cx.abort_flag = reinterpret_cast<volatile uint32_t*>(bars + 21);
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(cx.full0 + 8 * s, 1);
      mbar_init(cx.empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(cx.tfull0 + 8 * a, 1);
      mbar_init(cx.tempty0 + 8 * a, EPI_WARPS);
    }
    *cx.abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32((const void*)tmem_slot)),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  cx.tmem_base = *tmem_slot;
}

// Teardown: everyone meets, then the allocating warp frees TMEM.
__device__ __forceinline__ void cta_teardown(const CtaCtx& cx) {
  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  if (*cx.abort_flag) {
    // Give copies that may still be in flight time to land before the CTA's
    // shared memory is released.
    long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) {
    }
  }
  if ((threadIdx.x >> 5) == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(cx.tmem_base),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
}

// One GEMM: CTA b takes tiles b, b + gridDim.x, ...
template <int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmP,
                    const GemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  pdl_trigger();
  if (threadIdx.x == 0) {
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
  }
  CtaCtx cx;
  cta_setup(cx, smem_raw, p.bn, p.stages);
  pdl_wait();      // barriers, TMEM and tensor maps are ready; operands may still be in flight
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_tiles = p.tiles_m * p.tiles_n * p.nb0 * (p.split_k > 1 ? p.split_k : p.nb1);
  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < total_tiles; t += gridDim.x)
        if (!produce_unit(cx, p, &tmA, &tmB, t, stage, phase)) break;
    }
  } else if (warp == 1) {
    int stage = 0, acc = 0;
    uint32_t phase = 0, acc_phase = 0;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x)
      if (!mma_unit(cx, p, t, stage, phase, acc, acc_phase)) break;
  } else {
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x)
      if (!epilogue_unit<MODE>(cx, p, &tmC, &tmP, t, warp, lane, acc, acc_phase)) break;
    if (lane == 0) bulk_wait_read_all();   // the staging area outlives its last tile store
  }
  cta_teardown(cx);
}

// ---- grouped launch ------------------------------------------------------------------------
//
// Many independent GEMMs of the same tile width in one persistent launch: the dW = X^T dY of
// every Linear of a model, which have few tiles each (18..72 against 148 SMs) but thousands
// together.  Their tiles form one list, CTA b takes list entries b, b + gridDim.x, ...; with
// equal K (the rows of the batch) all entries cost the same, so the SMs stay level without
// splitting K and without a reduction pass.  The table lives in device memory: tensor maps,
// kernel parameters and the index of each problem's first list entry.
struct __align__(128) GroupEntry {
  CUtensorMap tmA, tmB, tmC;
  GemmParams p;
  int first_unit;
};
constexpr int GROUP_MAX = 256;   // problems per launch (their first_unit values sit in shared memory)

// problem that list entry u belongs to: the last one whose first_unit is <= u
__device__ __forceinline__ int group_find(const int* first, int n, int u) {
  int lo = 0, hi = n - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (first[mid] <= u) lo = mid;
    else hi = mid - 1;
  }
  return lo;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_group_kernel(const GroupEntry* __restrict__ table, int n_problems, int total_units, int bn,
                  int stages) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ int first[GROUP_MAX];
  pdl_trigger();
  // the table was written by the host long before this launch, not by the kernel before it
  for (int i = threadIdx.x; i < n_problems; i += blockDim.x) first[i] = table[i].first_unit;
  CtaCtx cx;
  cta_setup(cx, smem_raw, bn, stages);     // its __syncthreads also publishes first[]
  pdl_wait();
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int u = blockIdx.x; u < total_units; u += gridDim.x) {
        const int pi = group_find(first, n_problems, u);
        const GemmParams p = table[pi].p;
        if (!produce_unit(cx, p, &table[pi].tmA, &table[pi].tmB, u - first[pi], stage, phase)) break;
      }
    }
  } else if (warp == 1) {
    int stage = 0, acc = 0;
    uint32_t phase = 0, acc_phase = 0;
    for (int u = blockIdx.x; u < total_units; u += gridDim.x) {
      const int pi = group_find(first, n_problems, u);
      const GemmParams p = table[pi].p;
      if (!mma_unit(cx, p, u - first[pi], stage, phase, acc, acc_phase)) break;
    }
  } else {
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int u = blockIdx.x; u < total_units; u += gridDim.x) {
      const int pi = group_find(first, n_problems, u);
      const GemmParams p = table[pi].p;
      if (!epilogue_unit<0>(cx, p, &table[pi].tmC, nullptr, u - first[pi], warp, lane, acc, acc_phase))
        break;
    }
    if (lane == 0) bulk_wait_read_all();
  }
  cta_teardown(cx);
}

// ---- CTA pairs -----------------------------------------------------------------------------
//
// 256 x 256 tiles on a 2-CTA cluster: each CTA loads its 128 rows of A and its 128 of the
// tile's 256 columns of B, the even-ranked CTA issues tcgen05.mma.cta_group::2 for both, and
// each CTA's TMEM receives the accumulators of its own 128 rows.  Per k-block a CTA pulls
// 32 KB through L2 instead of 48 KB for the same 128 x 256 outputs, which is what bounds the
// single-CTA kernel on the K = 768 shapes.  Barriers: TMA of both CTAs counts bytes on the
// leader's full[s]; the leader's commits arrive on empty[s] / tmem_full[a] of both CTAs;
// the epilogue warps of both CTAs arrive on the leader's tmem_empty[a].
constexpr int PAIR_BN = 256;        // widest pair tile; 192 is the other width (N = 768 shapes)
// Bytes of one CTA's half of the B tile per k-block: bn / 2 rows of 128 bytes when B is K-major,
// whole 64-column groups of 64 k-rows when it is MN-major (96 columns load two groups).
__host__ __device__ inline int pair_b_stage_bytes(int bn, int b_mn) {
  return b_mn ? ((bn / 2 + 63) / 64) * 8192 : (bn / 2) * 128;
}
__host__ __device__ inline int pair_stages(int bn, int b_mn) {
  const int n = RING_BYTES / (A_STAGE_BYTES + pair_b_stage_bytes(bn, b_mn));
  return n > MAX_STAGES ? MAX_STAGES : n;
}

// Barriers, TMEM and constants of one CTA of a pair; ends with a cluster-wide barrier so the
// peer's mbarriers exist before anything is signalled on them.
__device__ __forceinline__ void pair_setup(CtaCtx& cx, uint8_t* smem_raw, int bn, int b_mn) {
  const int warp = threadIdx.x >> 5;
  cx.base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (cx.base - smem_u32(smem_raw));
  cx.stage_bytes = (uint32_t)(A_STAGE_BYTES + pair_b_stage_bytes(bn, b_mn));
  cx.n_stages = pair_stages(bn, b_mn);
  cx.epi_stage = gen_base + RING_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(gen_base + RING_BYTES + EPI_WARPS * EPI_STAGE_BYTES);
  const uint32_t bar_base = cx.base + RING_BYTES + EPI_WARPS * EPI_STAGE_BYTES;
  cx.full0 = bar_base;
  cx.empty0 = bar_base + 64;
  cx.tfull0 = bar_base + 128;
  cx.tempty0 = bar_base + 144;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 20);
  cx.abort_flag = reinterpret_cast<volatile uint32_t*>(bars + 21);
  if (threadIdx.x == 0) {
    for (int s = 0; s < cx.n_stages; ++s) {
      mbar_init(cx.full0 + 8 * s, 1);     // the leader's own arrive.expect_tx
      mbar_init(cx.empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(cx.tfull0 + 8 * a, 1);
      mbar_init(cx.tempty0 + 8 * a, 2 * EPI_WARPS);   // the epilogue warps of both CTAs
    }
    *cx.abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    // each CTA takes the whole of its own TMEM, so accumulator addresses agree in the pair
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32((const void*)tmem_slot)),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();        // the peer's barriers exist before anything is signalled on them
  tcgen05_fence_after();
  cx.tmem_base = *tmem_slot;

}

// Neither CTA may leave while the other can still read its shared memory or signal its
// barriers.
__device__ __forceinline__ void pair_teardown(const CtaCtx& cx) {
  const int warp = threadIdx.x >> 5;
  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (*cx.abort_flag) {
    long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) {
    }
  }
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(cx.tmem_base),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
}

// TMA producer of one CTA of the pair: its 128 rows of A and its half of the B tile.
__device__ __forceinline__ bool pair_produce_unit(const CtaCtx& cx, const GemmParams& p,
                                                  const CUtensorMap* tmA, const CUtensorMap* tmB,
                                                  int t, uint32_t rank, int& stage, uint32_t& phase) {
  TileCoord tc = tile_coord(p, t, 2 * BM, (int)rank * BM);
  int kb0, nkb;
  kb_range(p, tc, kb0, nkb);
  if (p.split_k > 1) tc.z1 = 0;
  const int nb = tc.n0 + (int)rank * (p.bn / 2);       // this CTA's columns of B
  for (int kb = 0; kb < nkb; ++kb) {
    if (!mbar_wait(cx.empty0 + 8 * stage, phase ^ 1u, cx.abort_flag, p.err, 0x500u + stage)) return false;
    if (rank == 0) mbar_expect_tx(cx.full0 + 8 * stage, 2 * cx.stage_bytes);
    const uint32_t fb = mapa_shared(cx.full0 + 8 * stage, 0);
    const uint32_t sa = cx.base + stage * cx.stage_bytes;
    const uint32_t sb = sa + A_STAGE_BYTES;
    const int k0 = (kb0 + kb) * BK;
    if (!p.a_mn) {
      tma_load_4d_pair(sa, tmA, fb, k0, tc.m0, tc.z0, tc.z1);
    } else {
      tma_load_4d_pair(sa, tmA, fb, tc.m0, k0, tc.z0, tc.z1);
      tma_load_4d_pair(sa + 8192, tmA, fb, tc.m0 + 64, k0, tc.z0, tc.z1);
    }
    if (!p.b_mn) {
      tma_load_4d_pair(sb, tmB, fb, k0, nb, tc.z0, tc.z1);
    } else {
      // whole 64-column groups: a 96-column half loads two and uses one and a half
      tma_load_4d_pair(sb, tmB, fb, nb, k0, tc.z0, tc.z1);
      if (p.bn > 128) tma_load_4d_pair(sb + 8192, tmB, fb, nb + 64, k0, tc.z0, tc.z1);
    }
    if (++stage == cx.n_stages) {
      stage = 0;
      phase ^= 1u;
    }
  }
  return true;
}

// MMA issue for the pair (a converged warp of the even-ranked CTA).
__device__ __forceinline__ bool pair_mma_unit(const CtaCtx& cx, const GemmParams& p, int t, int& stage,
                                              uint32_t& phase, int& acc, uint32_t& acc_phase) {
  int kb0, nkb;
  kb_range(p, tile_coord(p, t, 2 * BM, 0), kb0, nkb);
  if (nkb <= 0) return true;
  if (!mbar_wait_warp(cx.tempty0 + 8 * acc, acc_phase ^ 1u, cx.abort_flag, p.err, 0x600u + acc)) return false;
  tcgen05_fence_after();
  const uint32_t d_tmem = cx.tmem_base + (uint32_t)(acc * ACC_COLS);
  const uint32_t d_hi = smem_desc_hi(1024);       // descriptor halves as in mma_unit
  const uint32_t a_lo0 = smem_desc_lo(cx.base, p.a_mn ? 8192 : 16);
  const uint32_t b_lo0 = smem_desc_lo(cx.base + A_STAGE_BYTES, p.b_mn ? 8192 : 16);
  const uint32_t a_step = p.a_mn ? 128u : 2u, b_step = p.b_mn ? 128u : 2u;
  for (int kb = 0; kb < nkb; ++kb) {
    if (!mbar_wait_warp(cx.full0 + 8 * stage, phase, cx.abort_flag, p.err, 0x700u + stage)) return false;
    tcgen05_fence_after();
    const uint32_t a_lo = a_lo0 + (uint32_t)stage * (cx.stage_bytes >> 4);
    const uint32_t b_lo = b_lo0 + (uint32_t)stage * (cx.stage_bytes >> 4);
#pragma unroll
    for (int k = 0; k < BK / UMMA_K; ++k)
      if (elect_one())
        umma2_f16(d_tmem, smem_desc_pack(a_lo + k * a_step, d_hi), smem_desc_pack(b_lo + k * b_step, d_hi),
                  p.idesc, (kb | k) != 0 ? 1u : 0u);
    if (elect_one()) umma2_commit(cx.empty0 + 8 * stage);
    if (++stage == cx.n_stages) {
      stage = 0;
      phase ^= 1u;
    }
  }
  if (elect_one()) umma2_commit(cx.tfull0 + 8 * acc);
  acc ^= 1;
  if (acc == 0) acc_phase ^= 1u;
  return true;
}

// Epilogue warp of one CTA of the pair: its 128 rows of the 256 x 256 tile.
template <int MODE>
__device__ __forceinline__ bool pair_epilogue_unit(const CtaCtx& cx, const GemmParams& p,
                                                   const CUtensorMap* tmC, const CUtensorMap* tmP, int t,
                                                   uint32_t rank, int warp, int lane, int& acc,
                                                   uint32_t& acc_phase) {
  const int q = warp & 3;
  const TileCoord tc = tile_coord(p, t, 2 * BM, (int)rank * BM);
  {
    int kb0, nkb;
    kb_range(p, tc, kb0, nkb);
    if (nkb <= 0) return true;
  }
  if (!mbar_wait_warp(cx.tfull0 + 8 * acc, acc_phase, cx.abort_flag, p.err, 0x800u + acc)) return false;
  tcgen05_fence_after();
  uint8_t* stage = cx.epi_stage + (warp - 2) * EPI_STAGE_BYTES;
  const int sub_row = lane >> 2;
  const int sub_chunk = lane & 3;
  const long long batch_off = (long long)tc.z0 * p.sC0 + (long long)tc.z1 * p.sC1;
  const int row_base = tc.m0 + q * 32;
  const uint32_t t_row = cx.tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * ACC_COLS);
  const bool tma_out = (MODE & E_NO_TMA) == 0 && p.tma_store != 0;
  for (int c0 = 16 * ((warp - 2) >> 2); c0 < p.bn; c0 += 64) {
    if (tc.n0 + c0 >= p.N) break;
    uint32_t r[16];
    tmem_ld16(t_row + c0, r);
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    if ((MODE & E_NO_TMA) == 0 && tma_out) {
      if (row_base < p.M)
        epilogue_chunk_tma<MODE>(p, tmC, tmP, r, stage, lane, tc.n0 + c0, row_base, tc.z0, tc.z1);
      continue;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
      *reinterpret_cast<uint4*>(stage + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4)) =
          make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
    __syncwarp();
    const int col = tc.n0 + c0 + sub_chunk * 4;
    const unsigned lanes = __ballot_sync(0xffffffffu, col < p.N);
    if (col < p.N) {
      float4 v[4];
      long long off[4];
      unsigned ok = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int rr = 8 * i + sub_row;
        const int row = row_base + rr;
        v[i] = *reinterpret_cast<const float4*>(stage + rr * 64 + ((sub_chunk ^ ((rr >> 1) & 3)) << 4));
        off[i] = batch_off + (long long)row * p.ldc + col;
        ok |= (row < p.M ? 1u : 0u) << i;
      }
      epilogue_chunk<MODE>(p, v, off, ok, col, (tc.m0 / BM) * 4 + q, lanes);
    }
    __syncwarp();
  }
  tcgen05_fence_before();
  __syncwarp();
  if (lane == 0) {
    if (rank == 0) mbar_arrive(cx.tempty0 + 8 * acc);
    else mbar_arrive_cluster(mapa_shared(cx.tempty0 + 8 * acc, 0));
  }
  acc ^= 1;
  if (acc == 0) acc_phase ^= 1u;
  return true;
}

template <int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_cta_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmP,
                     const GemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  pdl_trigger();
  if (threadIdx.x == 0) {
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
  }
  CtaCtx cx;
  pair_setup(cx, smem_raw, p.bn, p.b_mn);
  pdl_wait();
  const int n_pairs = (int)gridDim.x >> 1, pair = (int)blockIdx.x >> 1;
  const int total_tiles = p.tiles_m * p.tiles_n * p.nb0 * (p.split_k > 1 ? p.split_k : p.nb1);
  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = pair; t < total_tiles; t += n_pairs)
        if (!pair_produce_unit(cx, p, &tmA, &tmB, t, rank, stage, phase)) break;
    }
  } else if (warp == 1) {
    if (rank == 0) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      for (int t = pair; t < total_tiles; t += n_pairs)
        if (!pair_mma_unit(cx, p, t, stage, phase, acc, acc_phase)) break;
    }
  } else {
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = pair; t < total_tiles; t += n_pairs)
      if (!pair_epilogue_unit<MODE>(cx, p, &tmC, &tmP, t, rank, warp, lane, acc, acc_phase)) break;
    if (lane == 0) bulk_wait_read_all();
  }
  pair_teardown(cx);
}

// The grouped launch on CTA pairs: list entries are 256 x 256 tiles.
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_group_pair_kernel(const GroupEntry* __restrict__ table, int n_problems, int total_units) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ int first[GROUP_MAX];
  pdl_trigger();
  for (int i = threadIdx.x; i < n_problems; i += blockDim.x) first[i] = table[i].first_unit;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  CtaCtx cx;
  pair_setup(cx, smem_raw, PAIR_BN, 1);   // dW problems: both operands MN-major; publishes first[]
  pdl_wait();
  const int n_pairs = (int)gridDim.x >> 1, pair = (int)blockIdx.x >> 1;
  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int u = pair; u < total_units; u += n_pairs) {
        const int pi = group_find(first, n_problems, u);
        const GemmParams p = table[pi].p;
        if (!pair_produce_unit(cx, p, &table[pi].tmA, &table[pi].tmB, u - first[pi], rank, stage, phase))
          break;
      }
    }
  } else if (warp == 1) {
    if (rank == 0) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      for (int u = pair; u < total_units; u += n_pairs) {
        const int pi = group_find(first, n_problems, u);
        const GemmParams p = table[pi].p;
        if (!pair_mma_unit(cx, p, u - first[pi], stage, phase, acc, acc_phase)) break;
      }
    }
  } else {
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int u = pair; u < total_units; u += n_pairs) {
      const int pi = group_find(first, n_problems, u);
      const GemmParams p = table[pi].p;
      if (!pair_epilogue_unit<0>(cx, p, &table[pi].tmC, nullptr, u - first[pi], rank, warp, lane, acc,
                                 acc_phase))
        break;
    }
    if (lane == 0) bulk_wait_read_all();
  }
  pair_teardown(cx);
}

// Adds the K slices of a split GEMM in slice order and writes C (fp32, row pitch ldc).
__global__ void k_splitk_reduce(const float4* __restrict__ ws, float* __restrict__ C, int M, int N4,
                                long long ldc, int splits) {
  pdl_trigger();
  pdl_wait();
  const long long per = (long long)M * N4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < per;
       i += (long long)gridDim.x * blockDim.x) {
    float4 a = ws[i];
    for (int s = 1; s < splits; ++s) {
      const float4 b = ws[i + s * per];
      a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    }
    const long long r = i / N4, c = i - r * N4;
    *reinterpret_cast<float4*>(C + r * ldc + c * 4) = a;
  }
}

typedef void (*GemmKernel)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap,
                           const GemmParams);
struct Specialised {
  int mode;
  GemmKernel fn;
};
#define VKG_SPEC(m) {(m), gemm_tcgen05_kernel<(m)>}
// The epilogues the training step uses; anything else runs the generic kernel.
const Specialised kSpecialised[] = {
    VKG_SPEC(0),                                   // fp32 out: dW, dX into layernorm, scores
    VKG_SPEC(E_F16),                               // fp16 out: attention products, dO
    VKG_SPEC(E_BIAS),                              // fp32 out + bias: logits of an untied head
    VKG_SPEC(E_BIAS | E_F16),                      // qkv projection
    VKG_SPEC(E_BIAS | E_RES),                      // proj / fc2 forward: + bias + residual
    VKG_SPEC(E_BIAS | E_PRE | E_ACT | E_F16),      // fc1 forward: bias, keep z, GELU, narrow
    VKG_SPEC(E_DACT | E_F16),                      // fc2 dX: * GELU'(z), narrow
    VKG_SPEC(E_DACT | E_F16 | E_COLSUM),           // the same + column sums = fc1's bias gradient
};
const int kNumSpecialised = sizeof(kSpecialised) / sizeof(kSpecialised[0]);
#define VKG_SPEC_CP(m) {(m), gemm_cta_pair_kernel<(m)>}
// The same epilogues on 256 x 256 tiles computed by CTA pairs.
const Specialised kCtaPair[] = {
    VKG_SPEC_CP(0),
    VKG_SPEC_CP(E_F16),
    VKG_SPEC_CP(E_BIAS),
    VKG_SPEC_CP(E_BIAS | E_F16),
    VKG_SPEC_CP(E_BIAS | E_RES),
    VKG_SPEC_CP(E_BIAS | E_PRE | E_ACT | E_F16),
    VKG_SPEC_CP(E_DACT | E_F16),
    VKG_SPEC_CP(E_DACT | E_F16 | E_COLSUM),
};
const int kNumCtaPair = sizeof(kCtaPair) / sizeof(kCtaPair[0]);
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// 4-D map {inner, rows, nb0, nb1} over a 16-bit matrix with two batch strides.
int make_map(vkg_device* dev, CUtensorMap* map, const void* ptr, int dtype, int64_t inner,
             int64_t rows, int64_t ld, int nb0, int64_t s0, int nb1, int64_t s1, int box_inner,
             int box_rows, const char* what) {
  cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)nb0, (cuuint64_t)nb1};
  int64_t pitch = ld * 2;
  int64_t st0 = nb0 > 1 ? s0 * 2 : pitch * rows;
  int64_t st1 = nb1 > 1 ? s1 * 2 : (nb0 > 1 ? st0 * nb0 : pitch * rows);
  cuuint64_t strides[3] = {(cuuint64_t)pitch, (cuuint64_t)st0, (cuuint64_t)st1};
  cuuint32_t box[4] = {(cuuint32_t)box_inner, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  if (((uintptr_t)ptr & 15) || (pitch & 15) || (st0 & 15) || (st1 & 15)) {
    vkg_set_error("gemm operand %s: base address and strides must be multiples of 16 bytes "
                  "(ptr %p, ld %lld, batch strides %lld/%lld elements)",
                  what, ptr, (long long)ld, (long long)s0, (long long)s1);
    return 1;
  }
  CUresult r = ((EncodeTiledFn)dev->encode_tiled)(
      map, dtype == VKG_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
      const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    vkg_set_error("cuTensorMapEncodeTiled failed for operand %s with code %d", what, (int)r);
    return 1;
  }
  return 0;
}

// 4-D map {N, M, nb0, nb1} over the output (fp32 or 16-bit) for the epilogue's tile stores:
// boxes of 16 columns x 32 rows in the 64-byte (fp32) or 32-byte (16-bit) swizzle the staging
// area is written in.  *ok = false (and no error) when the layout cannot be described: the
// epilogue then stores per lane.
int make_out_map(vkg_device* dev, CUtensorMap* map, const void* ptr, int dtype, int64_t n_cols,
                 int64_t n_rows, int64_t ld, int nb0, int64_t s0, int nb1, int64_t s1, bool* ok) {
  *ok = false;
  const int64_t es = dtype == VKG_F32 ? 4 : 2;
  const int64_t pitch = ld * es;
  const int64_t st0 = nb0 > 1 ? s0 * es : pitch * n_rows;
  const int64_t st1 = nb1 > 1 ? s1 * es : (nb0 > 1 ? st0 * nb0 : pitch * n_rows);
  if (((uintptr_t)ptr & 15) || (pitch & 15) || (st0 & 15) || (st1 & 15) || st0 <= 0 || st1 <= 0 ||
      pitch >= (1ll << 40) || st0 >= (1ll << 40) || st1 >= (1ll << 40))
    return 0;
  cuuint64_t dims[4] = {(cuuint64_t)n_cols, (cuuint64_t)n_rows, (cuuint64_t)nb0, (cuuint64_t)nb1};
  cuuint64_t strides[3] = {(cuuint64_t)pitch, (cuuint64_t)st0, (cuuint64_t)st1};
  cuuint32_t box[4] = {16, 32, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt = dtype == VKG_F32    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : dtype == VKG_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                     : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = ((EncodeTiledFn)dev->encode_tiled)(
      map, dt, 4, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
      es == 4 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    vkg_set_error("cuTensorMapEncodeTiled failed for the output map with code %d", (int)r);
    return 1;
  }
  *ok = true;
  return 0;
}

// Tile width and K split for one GEMM, from a small time model (microseconds).
// Measured on B200: a k-block (64 K-elements, four tcgen05.mma) costs 0.33 us even for a
// 64-column tile and only 0.41 us for 256 columns, so narrow tiles waste the tensor
// core; an epilogue costs ~4.4 us per 128x256 tile.  When the grid cannot fill
// the SMs with wide tiles (the dW shapes: few output tiles, K = rows of the batch),
// K is split across CTAs and a second pass adds the slices.
void plan_gemm(int M, int N, int K, int batch, int sms, bool may_split, int64_t ws_bytes,
               int force_bn, int force_split, int* out_bn, int* out_split, int bm = BM,
               double* out_us = nullptr) {
  const int tiles_m = (M + bm - 1) / bm;
  const int num_kb = (K + BK - 1) / BK;
  const int n_round = ((N + 63) / 64) * 64;
  const int cand[4] = {256, 192, 128, 64};
  double best = -1.0;
  *out_bn = 64;
  *out_split = 1;
  for (int i = 0; i < 4; ++i) {
    const int bn = cand[i];
    if (force_bn ? bn != force_bn : (bn > n_round && bn != 64)) continue;
    const long long tiles = (long long)tiles_m * ((N + bn - 1) / bn) * batch;
    // measured per k-block at K = 6144: 0.41 / 0.36 / 0.33 / 0.33 us for 256 / 192 / 128 / 64
    const double t_kb = bn >= 256 ? 0.41 : bn >= 192 ? 0.36 : 0.33;
    const double t_epi = 4.4 * bn / 256.0;
    for (int sp = 1; sp <= 16; ++sp) {
      if (force_split > 0 && sp != force_split) continue;
      if (sp > 1) {
        if (!may_split || num_kb / sp < 4) break;
        if ((int64_t)sp * M * N * 4 > ws_bytes) break;
      }
      const long long waves = (tiles * sp + sms - 1) / sms;
      const int kbs = (num_kb + sp - 1) / sp;
      double t = waves * (kbs * t_kb + t_epi);
      if (sp > 1) t += (double)(sp + 1) * M * N * 4.0 / 4.0e6 + 4.0;
      if (best < 0 || t < best) {
        best = t;
        *out_bn = bn;
        *out_split = sp;
      }
    }
  }
  if (out_us) *out_us = best;
}

// One GEMM made ready to launch: kernel parameters, operand maps, epilogue mask.
struct Problem {
  GemmParams p;
  CUtensorMap tmA, tmB, tmC, tmP;
  int mode;
  bool vec;
  long long total_tiles;
};

// use_pair: 256 x pair_bn tiles for gemm_cta_pair_kernel (the caller has checked the shape).
int build_problem(vkg_device* dev, const vkg_gemm_args* a, int force_bn, Problem* out,
                  bool use_pair = false, int pair_bn = PAIR_BN) {
  VKG_REQUIRE(a, "null gemm args");
  VKG_REQUIRE(a->M > 0 && a->N > 0 && a->K > 0, "gemm: M, N, K must be positive (%d, %d, %d)",
              a->M, a->N, a->K);
  VKG_REQUIRE(a->N % 8 == 0, "gemm: N must be a multiple of 8 (got %d)", a->N);
  VKG_REQUIRE(a->in_dtype == VKG_F16 || a->in_dtype == VKG_BF16,
              "gemm: inputs must be f16 or bf16");
  VKG_REQUIRE(a->c_dtype == VKG_F32 || a->c_dtype == VKG_F16 || a->c_dtype == VKG_BF16,
              "gemm: unknown output dtype %d", a->c_dtype);
  VKG_REQUIRE(a->A && a->B && a->C, "gemm: null operand");
  const int nb0 = a->nb0 > 0 ? a->nb0 : 1, nb1 = a->nb1 > 0 ? a->nb1 : 1;
  const int batch = nb0 * nb1;
  VKG_REQUIRE(a->ldc >= a->N, "gemm: ldc %lld < N %d", (long long)a->ldc, a->N);

  VKG_REQUIRE(a->tile_n == 0 || a->tile_n == 64 || a->tile_n == 128 || a->tile_n == 192 ||
                  a->tile_n == 256, "gemm: tile_n %d not in {64,128,192,256}", a->tile_n);
  const bool plain_f32 = !a->bias && !a->pre && !a->act && !a->dact_z && !a->residual && !a->C2 &&
                         a->c_dtype == VKG_F32 && (a->alpha == 0.0f || a->alpha == 1.0f);
  const bool may_split = plain_f32 && batch == 1 && a->causal == 0 && a->workspace && a->N % 4 == 0 &&
                         a->ldc % 4 == 0 && (((uintptr_t)a->C | (uintptr_t)a->workspace) & 15) == 0;
  VKG_REQUIRE(a->split_k <= 1 || may_split,
              "gemm: split_k needs an unbatched GEMM with a plain fp32 output, a 16-byte aligned "
              "workspace, and N, ldc multiples of 4");
  int bn = 0, want_split = 1;
  const int bm = use_pair ? 2 * BM : BM;
  plan_gemm(a->M, a->N, a->K, batch, use_pair ? vkg_persistent_ctas(dev) / 2 : vkg_persistent_ctas(dev),
            may_split && a->split_k != 1, a->workspace_bytes,
            use_pair ? pair_bn : (force_bn ? force_bn : a->tile_n), a->split_k > 1 ? a->split_k : 0,
            &bn, &want_split, bm);

  GemmParams& p = out->p;
  memset(&p, 0, sizeof(p));
  p.M = a->M; p.N = a->N; p.K = a->K;
  p.nb0 = nb0; p.nb1 = nb1;
  p.tiles_m = (a->M + bm - 1) / bm;
  p.tiles_n = (a->N + bn - 1) / bn;
  p.bn = bn;
  p.num_kb = (a->K + BK - 1) / BK;
  int stage_bytes = A_STAGE_BYTES + bn * 128;
  p.stages = RING_BYTES / stage_bytes;
  if (p.stages > MAX_STAGES) p.stages = MAX_STAGES;
  p.a_mn = a->trans_a ? 1 : 0;
  p.b_mn = a->trans_b ? 0 : 1;
  const uint32_t fmt = a->in_dtype == VKG_BF16 ? 1u : 0u;
  p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)p.a_mn << 15) |
            ((uint32_t)p.b_mn << 16) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(bm >> 4) << 24);
  p.c_dtype = a->c_dtype; p.act = a->act; p.dact = a->dact;
  p.ldc = a->ldc; p.sC0 = a->sC0; p.sC1 = a->sC1;
  p.C = a->C; p.C2 = a->C2; p.bias = a->bias; p.pre = a->pre;
  p.dact_z = a->dact_z; p.residual = a->residual;
  if (a->colsum) {
    VKG_REQUIRE(a->colsum_scratch && batch == 1 && a->causal == 0 && a->split_k <= 1,
                "gemm: colsum needs colsum_scratch, one matrix, causal == 0 and an unsplit K");
    p.colsum = a->colsum_scratch;
  }
  p.alpha = a->alpha == 0.0f ? 1.0f : a->alpha;
  p.err = dev->err_dev;
  p.split_k = 1;
  p.kb_per_split = p.num_kb;
  VKG_REQUIRE(a->causal >= 0 && a->causal <= 3, "gemm: causal mode %d unknown", a->causal);
  p.causal = a->causal;
  if (want_split > 1) {
    int splits = want_split < p.num_kb ? want_split : p.num_kb;
    p.kb_per_split = (p.num_kb + splits - 1) / splits;
    splits = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;   // no empty slice
    if (splits > 1) {
      VKG_REQUIRE(a->workspace_bytes >= (int64_t)splits * a->M * a->N * 4,
                  "gemm: split_k workspace too small (%lld bytes for %d slices of %d x %d)",
                  (long long)a->workspace_bytes, splits, a->M, a->N);
      p.split_k = splits;
      p.C = a->workspace;
      p.ldc = a->N;
      p.sC0 = 0;
      p.sC1 = (long long)a->M * a->N;
    }
  }
  // 16-byte vector accesses in the epilogue need every touched array aligned
  // for its element width at every (row, 8-column group).
  bool vec = (a->ldc % 4 == 0) && (a->sC0 % 4 == 0) && (a->sC1 % 4 == 0);
  const void* ptrs[6] = {a->C, a->C2, a->pre, a->dact_z, a->residual, a->bias};
  for (int i = 0; i < 6; ++i)
    if (ptrs[i] && ((uintptr_t)ptrs[i] & 15)) vec = false;
  p.vec_ok = vec ? 1 : 0;

  CUtensorMap& tmA = out->tmA;
  CUtensorMap& tmB = out->tmB;
  if (!a->trans_a) {
    VKG_REQUIRE(a->lda >= a->K, "gemm: lda %lld < K %d", (long long)a->lda, a->K);
    if (make_map(dev, &tmA, a->A, a->in_dtype, a->K, a->M, a->lda, nb0, a->sA0, nb1, a->sA1, BK, BM, "A"))
      return 1;
  } else {
    VKG_REQUIRE(a->lda >= a->M, "gemm: lda %lld < M %d (A stored K x M)", (long long)a->lda, a->M);
    if (make_map(dev, &tmA, a->A, a->in_dtype, a->M, a->K, a->lda, nb0, a->sA0, nb1, a->sA1, 64, BK, "A^T"))
      return 1;
  }
  if (a->trans_b) {
    VKG_REQUIRE(a->ldb >= a->K, "gemm: ldb %lld < K %d (B stored N x K)", (long long)a->ldb, a->K);
    if (make_map(dev, &tmB, a->B, a->in_dtype, a->K, a->N, a->ldb, nb0, a->sB0, nb1, a->sB1, BK,
                 use_pair ? pair_bn / 2 : bn, "B^T"))
      return 1;
  } else {
    VKG_REQUIRE(a->ldb >= a->N, "gemm: ldb %lld < N %d", (long long)a->ldb, a->N);
    if (make_map(dev, &tmB, a->B, a->in_dtype, a->N, a->K, a->ldb, nb0, a->sB0, nb1, a->sB1, 64, BK, "B"))
      return 1;
  }

  out->vec = vec;
  out->total_tiles = (long long)p.tiles_m * p.tiles_n * batch * p.split_k;
  VKG_REQUIRE(out->total_tiles < (1ll << 30), "gemm: too many tiles");
  out->mode = (a->bias ? E_BIAS : 0) | (a->pre ? E_PRE : 0) | (a->act ? E_ACT : 0) |
              (a->dact_z ? E_DACT : 0) | (a->residual ? E_RES : 0) | (a->C2 ? E_C2 : 0) |
              (a->c_dtype == VKG_F16 ? E_F16 : a->c_dtype == VKG_BF16 ? E_BF16 : 0) |
              (a->colsum ? E_COLSUM : 0);
  if (!vec) out->mode = E_GENERIC;
  // write-only epilogues store their tiles through tensor maps over C (and pre); p.C, p.ldc
  // and the batch strides already describe the split-K workspace when K is split
  memset(&out->tmC, 0, sizeof(CUtensorMap));
  memset(&out->tmP, 0, sizeof(CUtensorMap));
  if (dev->tma_store && (out->mode & E_NO_TMA) == 0) {
    const int z1n = p.split_k > 1 ? p.split_k : nb1;
    bool ok_c = false, ok_p = true;
    if (make_out_map(dev, &out->tmC, p.C, p.split_k > 1 ? VKG_F32 : a->c_dtype, p.N, p.M, p.ldc, nb0,
                     p.sC0, z1n, p.sC1, &ok_c))
      return 1;
    if (ok_c && a->pre &&
        make_out_map(dev, &out->tmP, a->pre, VKG_F32, p.N, p.M, p.ldc, nb0, p.sC0, z1n, p.sC1, &ok_p))
      return 1;
    p.tma_store = (ok_c && ok_p) ? 1 : 0;
  }
  return 0;
}

int ensure_attrs(vkg_device* dev) {
  if (dev->gemm_attr_set) return 0;
  VKG_REQUIRE((size_t)SMEM_BYTES <= dev->gemm_smem_optin,
              "gemm needs %d bytes of shared memory, device offers %zu", SMEM_BYTES,
              dev->gemm_smem_optin);
  VKG_CUDA(cudaFuncSetAttribute(gemm_tcgen05_kernel<E_GENERIC>,
                                cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
  for (int i = 0; i < kNumSpecialised; ++i)
    VKG_CUDA(cudaFuncSetAttribute(kSpecialised[i].fn, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  SMEM_BYTES));
  VKG_CUDA(cudaFuncSetAttribute(gemm_cta_pair_kernel<E_GENERIC>,
                                cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
  for (int i = 0; i < kNumCtaPair; ++i)
    VKG_CUDA(cudaFuncSetAttribute(kCtaPair[i].fn, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  SMEM_BYTES));
  dev->gemm_attr_set = true;
  return 0;
}

GemmKernel pick_kernel(int mode) {
  for (int i = 0; i < kNumSpecialised; ++i)
    if (kSpecialised[i].mode == mode) return kSpecialised[i].fn;
  return gemm_tcgen05_kernel<E_GENERIC>;
}

int reduce_slices(vkg_device* dev, const vkg_gemm_args* a, const GemmParams& p) {
  if (p.split_k <= 1) return 0;
  const long long n4 = (long long)a->M * (a->N / 4);
  VKG_CUDA(vkg_launch(dev, VKG_K_SMALL, k_splitk_reduce, dim3(vkg_blocks(n4, 256, (int64_t)dev->sm_count * 8)),
                      dim3(256), 0, 1, (const float4*)a->workspace, (float*)a->C, a->M, a->N / 4,
                      (long long)a->ldc, p.split_k));
  return vkg_check_launch("splitk_reduce");
}

// A barrier that nothing ever arrives on, waited for with the kernels' own bounded wait and a
// small budget: the error path every device-side wait takes when its partner never shows up
// (flag the abort, record where, return), without a fault and with the context intact.
__global__ void k_wait_selftest(uint32_t* err, long long budget) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0u;
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_wait<true>(smem_u32(&bar), 0, &abort_flag, err, 0x5e1fu, budget);
  }
}

// Adds the per-warp partial column sums a launch left in colsum_scratch: four rows per
// 128-row block the kernel worked on (tile_rows = BM, or 2 * BM for CTA pairs, whose last tile
// may add a block that lies wholly past M and holds zeros).
int finish_colsum(vkg_device* dev, const vkg_gemm_args* a, int tile_rows) {
  if (!a->colsum) return 0;
  const int blocks = ((a->M + tile_rows - 1) / tile_rows) * (tile_rows / BM);
  return vkg_launch_col_sum_final(dev, a->colsum_scratch, a->colsum, a->N, 4 * blocks, 0);
}

}  // namespace

// four partial rows (one per 32-row warp slot) for every 128-row block of the M rows padded
// to the 256-row tiles of a CTA pair
extern "C" int64_t vkg_gemm_colsum_scratch_floats(int M, int N) {
  if (M <= 0 || N <= 0) return 0;
  return (int64_t)4 * 2 * ((M + 2 * BM - 1) / (2 * BM)) * N;
}

extern "C" int vkg_selftest_wait_timeout(vkg_device* dev, int64_t budget_cycles) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(budget_cycles > 0 && budget_cycles <= 100000000ll,
              "selftest: budget must be between 1 and 1e8 cycles");
  k_wait_selftest<<<1, 32, 0, dev->stream>>>(dev->err_dev, (long long)budget_cycles);
  return vkg_check_launch("wait_selftest");
}

extern "C" int64_t vkg_gemm_group_table_bytes(int n) {
  return n > 0 ? (int64_t)n * (int64_t)sizeof(GroupEntry) : 0;
}

// Builds the table of a grouped launch in `table` (device memory, 128-byte aligned,
// vkg_gemm_group_table_bytes(n) bytes).  Synchronous: call it outside a stream capture.
extern "C" int vkg_gemm_group_prepare(vkg_device* dev, const vkg_gemm_args* args, int n, void* table,
                                      int cta_pair, int* total_units) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(args && table && total_units && n > 0 && n <= GROUP_MAX,
              "gemm_group: between 1 and %d problems and a table", GROUP_MAX);
  VKG_REQUIRE(((uintptr_t)table & 127) == 0, "gemm_group: table must be 128-byte aligned");
  VKG_REQUIRE(!dev->capturing, "gemm_group: prepare the table before the stream capture begins");
  std::vector<GroupEntry> host(n);
  long long units = 0;
  // CTA-pair tiles (256 x 256) when asked for and every problem has more than one row block
  bool use_pair = cta_pair > 0 && dev->sm_count >= 2;
  for (int i = 0; i < n && use_pair; ++i) use_pair = args[i].M > BM && args[i].N >= PAIR_BN / 2;
  for (int i = 0; i < n; ++i) {
    const vkg_gemm_args* a = &args[i];
    const int nb = (a->nb0 > 0 ? a->nb0 : 1) * (a->nb1 > 0 ? a->nb1 : 1);
    VKG_REQUIRE(nb == 1 && a->causal == 0 && !a->bias && !a->pre && !a->act && !a->dact_z &&
                    !a->residual && !a->C2 && !a->colsum && a->c_dtype == VKG_F32 &&
                    (a->alpha == 0.0f || a->alpha == 1.0f),
                "gemm_group: problem %d is not a plain fp32-output, unbatched GEMM", i);
    VKG_REQUIRE(a->in_dtype == args[0].in_dtype, "gemm_group: operand types differ");
    vkg_gemm_args one = *a;
    one.split_k = 1;
    one.workspace = nullptr;
    one.workspace_bytes = 0;
    Problem q;
    if (build_problem(dev, &one, 256, &q, use_pair)) return 1;
    VKG_REQUIRE(q.mode == 0, "gemm_group: problem %d needs 16-byte aligned rows", i);
    memset(&host[i], 0, sizeof(GroupEntry));
    host[i].tmA = q.tmA;
    host[i].tmB = q.tmB;
    host[i].tmC = q.tmC;
    host[i].p = q.p;
    host[i].first_unit = (int)units;
    units += q.total_tiles;
    VKG_REQUIRE(units < (1ll << 30), "gemm_group: too many tiles");
  }
  VKG_CUDA(cudaMemcpy(table, host.data(), (size_t)n * sizeof(GroupEntry), cudaMemcpyHostToDevice));
  // a negative count tells vkg_gemm_group_launch that the entries are CTA-pair tiles
  *total_units = use_pair ? -(int)units : (int)units;
  return 0;
}

extern "C" int vkg_gemm_group_launch(vkg_device* dev, const void* table, int n, int total_units) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(table && n > 0 && n <= GROUP_MAX && total_units != 0, "gemm_group: bad arguments");
  if (ensure_attrs(dev)) return 1;
  if (!dev->group_attr_set) {
    VKG_CUDA(cudaFuncSetAttribute(gemm_group_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  SMEM_BYTES));
    VKG_CUDA(cudaFuncSetAttribute(gemm_group_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  SMEM_BYTES));
    dev->group_attr_set = true;
  }
  if (total_units < 0) {
    const int units = -total_units;
    int pairs = vkg_persistent_ctas(dev) / 2;
    if (pairs > units) pairs = units;
    VKG_CUDA(vkg_launch(dev, VKG_K_GEMM_GROUP, gemm_group_pair_kernel, dim3((unsigned)(2 * pairs)), dim3(NUM_THREADS),
                        SMEM_BYTES, 2, static_cast<const GroupEntry*>(table), n, units));
    return vkg_check_launch("gemm_group_pair_kernel");
  }
  int ctas = vkg_persistent_ctas(dev) < total_units ? vkg_persistent_ctas(dev) : total_units;
  const int stages = RING_BYTES / (A_STAGE_BYTES + 256 * 128);
  VKG_CUDA(vkg_launch(dev, VKG_K_GEMM_GROUP, gemm_group_kernel, dim3((unsigned)ctas), dim3(NUM_THREADS), SMEM_BYTES, 1,
                      static_cast<const GroupEntry*>(table), n, total_units, 256, stages));
  return vkg_check_launch("gemm_group_kernel");
}

// 256 x 192 pair tiles: for outputs a few 192-column tiles wide (the N = 768 shapes of a
// d_model-768 step) they fill the second wave better than 256-wide tiles and each CTA pulls
// 28 KB per k-block (K-major B) where a single-CTA 128 x 192 tile pulls 40 KB.
bool pair192_pays(vkg_device* dev, const vkg_gemm_args* a) {
  if (!dev->pair192 || a->N % 192 != 0 || a->N > 4 * 192) return false;
  const int nb = (a->nb0 > 0 ? a->nb0 : 1) * (a->nb1 > 0 ? a->nb1 : 1);
  if (nb != 1 || a->split_k > 1 || a->K < 1536) return false;     // K = 768: no gain measured
  const long long tiles = (long long)((a->M + 2 * BM - 1) / (2 * BM)) * (a->N / 192);
  return tiles >= vkg_persistent_ctas(dev) / 2;      // at least one full wave of pair tiles
}

extern "C" int vkg_gemm(vkg_device* dev, const vkg_gemm_args* a) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(a, "null gemm args");
  Problem q;
  // 256 x 256 tiles on CTA pairs: only where a pair has at least two full row blocks and a
  // full-width tile to work on, and never for the causal attention shortcuts
  const bool pair_ok = a->causal == 0 && a->M > BM && a->N >= PAIR_BN / 2 && dev->sm_count >= 2 &&
                       (a->tile_n == 0 || a->tile_n == PAIR_BN || a->tile_n == 192) && a->max_ctas == 0;
  bool use_pair = pair_ok && a->cta_pair > 0;
  int pair_bn = a->tile_n == 192 ? 192 : PAIR_BN;
  if (pair_ok && a->cta_pair == 0) {
    // Measured on B200: CTA-pair tiles are about 10 % faster on launches with six or more waves of
    // them (the vocabulary-sized GEMMs) and on few-tile dW shapes whose K is split; with a
    // handful of waves they time the same alone and a little slower inside a training step,
    // and with one wave and a bit they lose.
    if (build_problem(dev, a, 0, &q, true)) return 1;
    use_pair = q.p.split_k > 1 ||
               10ll * q.total_tiles >= (long long)dev->pair_min_waves_x10 * (vkg_persistent_ctas(dev) / 2);
    if (!use_pair && a->tile_n == 0 && pair192_pays(dev, a)) {
      use_pair = true;
      pair_bn = 192;
    }
  }
  if (use_pair) {
    if (build_problem(dev, a, 0, &q, true, pair_bn)) return 1;
    if (ensure_attrs(dev)) return 1;
    GemmKernel fn = gemm_cta_pair_kernel<E_GENERIC>;
    for (int i = 0; i < kNumCtaPair; ++i)
      if (kCtaPair[i].mode == q.mode) fn = kCtaPair[i].fn;
    long long pairs = vkg_persistent_ctas(dev) / 2;
    if (pairs > q.total_tiles) pairs = q.total_tiles;
    VKG_CUDA(vkg_launch(dev, VKG_K_GEMM_PAIR, fn, dim3((unsigned)(2 * pairs)), dim3(NUM_THREADS), SMEM_BYTES, 2, q.tmA,
                        q.tmB, q.tmC, q.tmP, q.p));
    if (vkg_check_launch("gemm_cta_pair_kernel")) return 1;
    if (reduce_slices(dev, a, q.p)) return 1;
    return finish_colsum(dev, a, 2 * BM);
  }
  if (build_problem(dev, a, 0, &q)) return 1;
  if (ensure_attrs(dev)) return 1;
  int ctas = a->max_ctas > 0 ? a->max_ctas : vkg_persistent_ctas(dev);
  if (ctas > q.total_tiles) ctas = (int)q.total_tiles;
  VKG_CUDA(vkg_launch(dev, VKG_K_GEMM, pick_kernel(q.mode), dim3((unsigned)ctas), dim3(NUM_THREADS), SMEM_BYTES, 1,
                      q.tmA, q.tmB, q.tmC, q.tmP, q.p));
  if (vkg_check_launch("gemm_tcgen05_kernel")) return 1;
  if (reduce_slices(dev, a, q.p)) return 1;
  return finish_colsum(dev, a, BM);
}
