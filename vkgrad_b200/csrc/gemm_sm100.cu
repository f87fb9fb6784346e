// The GEMM trio (Y = X W, dX = dY W^T, dW = X^T dY) and its batched form for
// sm_100a: TMA -> 128B-swizzled shared memory ring -> tcgen05.mma issued by one
// thread -> fp32 accumulators in TMEM (two stages, so the epilogue of tile i
// overlaps the main loop of tile i+1) -> tcgen05.ld epilogue with the fused
// bias / activation / activation-derivative / residual / narrowing.
//
// One persistent CTA per SM, 320 threads:
//   warp 0      TMA producer (one lane)
//   warp 1      TMEM allocation + MMA issue (one lane)
//   warps 2..9  epilogue; warp w reads TMEM lanes 32*(w%4) .. +31 and takes every
//               other 32-column chunk.  The epilogue is instruction-issue bound, so
//               it gets two warps per scheduler and a compile-time feature mask.
//
// Transposed operands are never materialised (the reference makes the same
// point for its cooperative-matrix loads, kernels.py:45-49): "A stored K x M"
// and "B stored K x N" are loaded as MN-major tiles and the shared-memory /
// instruction descriptors say so.
//
// Every mbarrier wait is bounded by a clock64 budget; a wait that gives up
// sets an error word the host reads at the next synchronisation, the CTA
// stops issuing work, frees its TMEM and returns.
#include "common.cuh"

namespace {

constexpr int BM = 128;            // rows of C per tile = UMMA M
constexpr int BK = 64;             // K elements per stage = 128 bytes of f16 = one swizzle row
constexpr int UMMA_K = 16;         // K per tcgen05.mma.kind::f16
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int MAX_STAGES = 8;
constexpr int EPI_WARPS = 8;       // two per TMEM lane quarter, each takes alternate 32-column chunks
constexpr int NUM_THREADS = (2 + EPI_WARPS) * 32;
constexpr int TMEM_COLS = 512;     // whole TMEM: two 256-column accumulators
constexpr int ACC_COLS = 256;
constexpr int RING_BYTES = 196608; // shared-memory ring budget
constexpr int EPI_STAGE_BYTES = 32 * 32 * 4;  // one 32x32 fp32 chunk per epilogue warp (XOR-swizzled)
constexpr int SMEM_BYTES = RING_BYTES + EPI_WARPS * EPI_STAGE_BYTES + 1024 /*align slack*/ +
                           256 /*barriers*/;
constexpr int GROUP_M = 8;         // m-tiles per rasterisation band
constexpr long long WAIT_BUDGET_CYCLES = 2000000000ll;  // ~1 s

struct GemmParams {
  int M, N, K;
  int nb0, nb1;
  int tiles_m, tiles_n;
  int bn, stages, num_kb;
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
  float alpha;
  uint32_t* err;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

// Bounded wait.  Returns false when the wait gave up or another role already
// flagged an abort; the caller then leaves its loop.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          uint32_t* err, uint32_t where) {
  if (mbar_try_wait(bar, parity)) return true;
  long long t0 = clock64();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 63u) == 0u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > WAIT_BUDGET_CYCLES) {
        *abort_flag = 1u;
        if (atomicCAS(err, 0u, VKG_ERR_WAIT_TIMEOUT) == 0u) err[1] = where;
        __threadfence_system();
        return false;
      }
    }
  }
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(dst), "l"((uint64_t)map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle, Blackwell version field.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFFu);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;  // descriptor version for sm_100
  d |= 2ull << 61;  // SWIZZLE_128B
  return d;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

struct TileCoord {
  int z0, z1, m0, n0;
};

__device__ __forceinline__ TileCoord tile_coord(const GemmParams& p, int t) {
  int per_batch = p.tiles_m * p.tiles_n;
  int z = t / per_batch;
  int r = t - z * per_batch;
  int band = GROUP_M * p.tiles_n;
  int g = r / band;
  int first_m = g * GROUP_M;
  int gsize = min(p.tiles_m - first_m, GROUP_M);
  int in_band = r - g * band;
  TileCoord c;
  c.m0 = (first_m + in_band % gsize) * BM;
  c.n0 = (in_band / gsize) * p.bn;
  c.z0 = z % p.nb0;
  c.z1 = z / p.nb0;
  return c;
}

// Compile-time epilogue feature mask.  E_GENERIC reads every flag (and the vector
// alignment flag) at run time; the specialised masks assume 16-byte aligned operands.
enum : int {
  E_BIAS = 1, E_PRE = 2, E_ACT = 4, E_DACT = 8, E_RES = 16, E_C2 = 32, E_F16 = 64, E_BF16 = 128,
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

// Four consecutive columns of one row through the fused epilogue.  Called in the
// coalesced layout: the 8 lanes of a quarter-warp cover 32 consecutive columns of
// one row, so every global access of the warp is four full 128-byte rows.
template <int MODE>
__device__ __forceinline__ void epilogue4(const GemmParams& p, float4 a, long long off, int col) {
  constexpr bool G = (MODE & E_GENERIC) != 0;
  const bool vec = G ? (p.vec_ok != 0) : true;
  const bool has_bias = G ? (p.bias != nullptr) : (MODE & E_BIAS) != 0;
  const bool has_pre = G ? (p.pre != nullptr) : (MODE & E_PRE) != 0;
  const bool has_act = G ? (p.act != 0) : (MODE & E_ACT) != 0;
  const bool has_dact = G ? (p.dact_z != nullptr) : (MODE & E_DACT) != 0;
  const bool has_res = G ? (p.residual != nullptr) : (MODE & E_RES) != 0;
  const bool has_c2 = G ? (p.C2 != nullptr) : (MODE & E_C2) != 0;
  const int c_dtype = G ? p.c_dtype : ((MODE & E_F16) ? VKG_F16 : (MODE & E_BF16) ? VKG_BF16 : VKG_F32);
  float v[4] = {a.x * p.alpha, a.y * p.alpha, a.z * p.alpha, a.w * p.alpha};
  if (has_bias) {
    const float4 b = vec ? __ldg(reinterpret_cast<const float4*>(p.bias + col))
                         : make_float4(p.bias[col], p.bias[col + 1], p.bias[col + 2], p.bias[col + 3]);
    v[0] += b.x; v[1] += b.y; v[2] += b.z; v[3] += b.w;
  }
  if (has_pre) {
    if (vec) {
      *reinterpret_cast<float4*>(p.pre + off) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) p.pre[off + j] = v[j];
    }
  }
  if (has_act) {
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = vkg_act(v[j], p.act);
  }
  if (has_dact) {
    float z[4];
    if (vec) {
      const float4 t = *reinterpret_cast<const float4*>(p.dact_z + off);
      z[0] = t.x; z[1] = t.y; z[2] = t.z; z[3] = t.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) z[j] = p.dact_z[off + j];
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] *= vkg_dact(z[j], p.dact);
  }
  if (has_res) {
    if (vec) {
      const float4 t = *reinterpret_cast<const float4*>(p.residual + off);
      v[0] += t.x; v[1] += t.y; v[2] += t.z; v[3] += t.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] += p.residual[off + j];
    }
  }
  if (c_dtype == VKG_F32) {
    float* c = reinterpret_cast<float*>(p.C) + off;
    if (vec) {
      *reinterpret_cast<float4*>(c) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) c[j] = v[j];
    }
  } else if (c_dtype == VKG_F16) {
    store4_16<__half2, __half>(reinterpret_cast<__half*>(p.C) + off, v, vec);
  } else {
    store4_16<__nv_bfloat162, __nv_bfloat16>(reinterpret_cast<__nv_bfloat16*>(p.C) + off, v, vec);
  }
  if (has_c2) store4_16<__half2, __half>(reinterpret_cast<__half*>(p.C2) + off, v, vec);
}

template <int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const GemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // 128B-swizzled tiles want 1024-byte alignment.
  uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t b_stage_bytes = (uint32_t)p.bn * 128u;
  const uint32_t stage_bytes = A_STAGE_BYTES + b_stage_bytes;
  // Epilogue staging (one swizzled 32x32 fp32 chunk per epilogue warp), then the barrier block.
  float* epi_stage = reinterpret_cast<float*>(gen_base + RING_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(gen_base + RING_BYTES + EPI_WARPS * EPI_STAGE_BYTES);
  const uint32_t bar_base = base + RING_BYTES + EPI_WARPS * EPI_STAGE_BYTES;
  // full[s] at +8s, empty[s] at +64+8s, tmem_full[a] at +128+8a, tmem_empty[a] at +144+8a
  const uint32_t full0 = bar_base, empty0 = bar_base + 64, tfull0 = bar_base + 128,
                 tempty0 = bar_base + 144;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 20);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars + 21);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull0 + 8 * a, 1);
      mbar_init(tempty0 + 8 * a, EPI_WARPS);
    }
    *abort_flag = 0u;
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
  const uint32_t tmem_base = *tmem_slot;

  const int total_tiles = p.tiles_m * p.tiles_n * p.nb0 * p.nb1;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        TileCoord tc = tile_coord(p, t);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(empty0 + 8 * stage, phase ^ 1u, abort_flag, p.err, 0x100u + stage)) {
            ok = false;
            break;
          }
          const uint32_t fb = full0 + 8 * stage;
          mbar_expect_tx(fb, stage_bytes);
          const uint32_t sa = base + stage * stage_bytes;
          const uint32_t sb = sa + A_STAGE_BYTES;
          const int k0 = kb * BK;
          if (!p.a_mn) {
            tma_load_4d(sa, &tmA, fb, k0, tc.m0, tc.z0, tc.z1);
          } else {
            tma_load_4d(sa, &tmA, fb, tc.m0, k0, tc.z0, tc.z1);
            tma_load_4d(sa + 8192, &tmA, fb, tc.m0 + 64, k0, tc.z0, tc.z1);
          }
          if (!p.b_mn) {
            tma_load_4d(sb, &tmB, fb, k0, tc.n0, tc.z0, tc.z1);
          } else {
            for (int g = 0; g < p.bn / 64; ++g)
              tma_load_4d(sb + g * 8192, &tmB, fb, tc.n0 + 64 * g, k0, tc.z0, tc.z1);
          }
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(tempty0 + 8 * acc, acc_phase ^ 1u, abort_flag, p.err, 0x200u + acc)) break;
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * ACC_COLS);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(full0 + 8 * stage, phase, abort_flag, p.err, 0x300u + stage)) {
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const uint32_t sa = base + stage * stage_bytes;
          const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // K-major: 16 elements further along the 128-byte row.  MN-major:
            // two 8-row groups (2 x 1024 bytes) further down.
            uint64_t ad = p.a_mn ? make_smem_desc(sa + k * 2048, 8192, 1024)
                                 : make_smem_desc(sa + k * 32, 16, 1024);
            uint64_t bd = p.b_mn ? make_smem_desc(sb + k * 2048, 8192, 1024)
                                 : make_smem_desc(sb + k * 32, 16, 1024);
            umma_f16(d_tmem, ad, bd, p.idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty0 + 8 * stage);  // frees the stage when these MMAs retire
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(tfull0 + 8 * acc);  // accumulator complete -> epilogue
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
      TileCoord tc = tile_coord(p, t);
      if (!mbar_wait(tfull0 + 8 * acc, acc_phase, abort_flag, p.err, 0x400u + acc)) break;
      tcgen05_fence_after();
      // TMEM gives each lane one row; the chunk is transposed through shared memory so
      // that global loads and stores are row-contiguous (8 lanes x 16 B per row).  Rows
      // are 128 B apart with the 16-byte chunk index XOR-ed by (row & 7): conflict-free
      // both for the row-per-lane writes and the row-contiguous reads.
      uint8_t* stage = reinterpret_cast<uint8_t*>(epi_stage) + (warp - 2) * EPI_STAGE_BYTES;
      const int sub_row = lane >> 3;        // 0..3: row within a group of four
      const int sub_chunk = lane & 7;       // which 16-byte chunk (4 columns) of the row
      const long long batch_off = (long long)tc.z0 * p.sC0 + (long long)tc.z1 * p.sC1;
      const int row_base = tc.m0 + q * 32;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * ACC_COLS);
      for (int c0 = 32 * ((warp - 2) >> 2); c0 < p.bn; c0 += 64) {
        if (tc.n0 + c0 >= p.N) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld16(t_row + c0, r);
        tmem_ld16(t_row + c0 + 16, r + 16);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<uint4*>(stage + lane * 128 + ((j ^ (lane & 7)) << 4)) =
              make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
        __syncwarp();
        const int col = tc.n0 + c0 + sub_chunk * 4;
        if (col < p.N) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rr = 4 * i + sub_row;
            const int row = row_base + rr;
            if (row < p.M) {
              const float4 a = *reinterpret_cast<const float4*>(
                  stage + rr * 128 + ((sub_chunk ^ (rr & 7)) << 4));
              epilogue4<MODE>(p, a, batch_off + (long long)row * p.ldc + col, col);
            }
          }
        }
        __syncwarp();
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty0 + 8 * acc);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  // Teardown: everyone meets, then the allocating warp frees TMEM.
  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // Give copies that may still be in flight time to land before the CTA's
    // shared memory is released.
    long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) {
    }
  }
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
}

typedef void (*GemmKernel)(const CUtensorMap, const CUtensorMap, const GemmParams);
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
};
const int kNumSpecialised = sizeof(kSpecialised) / sizeof(kSpecialised[0]);

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

int pick_tile_n(int M, int N, int batch, int sms) {
  int tiles_m = (M + BM - 1) / BM;
  int best = 64;
  long long best_cost = -1;
  const int cand[4] = {256, 192, 128, 64};
  int n_round = ((N + 63) / 64) * 64;
  for (int i = 0; i < 4; ++i) {
    int bn = cand[i];
    if (bn > n_round && bn != 64) continue;
    long long tiles = (long long)tiles_m * ((N + bn - 1) / bn) * batch;
    long long waves = (tiles + sms - 1) / sms;
    long long cost = waves * (bn + 24);
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best = bn;
    }
  }
  return best;
}

}  // namespace

extern "C" int vkg_gemm(vkg_device* dev, const vkg_gemm_args* a) {
  if (vkg_bind(dev)) return 1;
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

  int bn = a->tile_n;
  if (bn == 0) bn = pick_tile_n(a->M, a->N, batch, dev->sm_count);
  VKG_REQUIRE(bn == 64 || bn == 128 || bn == 192 || bn == 256, "gemm: tile_n %d not in {64,128,192,256}",
              bn);

  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = a->M; p.N = a->N; p.K = a->K;
  p.nb0 = nb0; p.nb1 = nb1;
  p.tiles_m = (a->M + BM - 1) / BM;
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
            ((uint32_t)p.b_mn << 16) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  p.c_dtype = a->c_dtype; p.act = a->act; p.dact = a->dact;
  p.ldc = a->ldc; p.sC0 = a->sC0; p.sC1 = a->sC1;
  p.C = a->C; p.C2 = a->C2; p.bias = a->bias; p.pre = a->pre;
  p.dact_z = a->dact_z; p.residual = a->residual;
  p.alpha = a->alpha == 0.0f ? 1.0f : a->alpha;
  p.err = dev->err_dev;
  // 16-byte vector accesses in the epilogue need every touched array aligned
  // for its element width at every (row, 8-column group).
  bool vec = (a->ldc % 4 == 0) && (a->sC0 % 4 == 0) && (a->sC1 % 4 == 0);
  const void* ptrs[6] = {a->C, a->C2, a->pre, a->dact_z, a->residual, a->bias};
  for (int i = 0; i < 6; ++i)
    if (ptrs[i] && ((uintptr_t)ptrs[i] & 15)) vec = false;
  p.vec_ok = vec ? 1 : 0;

  CUtensorMap tmA, tmB;
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
    if (make_map(dev, &tmB, a->B, a->in_dtype, a->K, a->N, a->ldb, nb0, a->sB0, nb1, a->sB1, BK, bn, "B^T"))
      return 1;
  } else {
    VKG_REQUIRE(a->ldb >= a->N, "gemm: ldb %lld < N %d", (long long)a->ldb, a->N);
    if (make_map(dev, &tmB, a->B, a->in_dtype, a->N, a->K, a->ldb, nb0, a->sB0, nb1, a->sB1, 64, BK, "B"))
      return 1;
  }

  if (!dev->gemm_attr_set) {
    VKG_REQUIRE((size_t)SMEM_BYTES <= dev->gemm_smem_optin,
                "gemm needs %d bytes of shared memory, device offers %zu", SMEM_BYTES,
                dev->gemm_smem_optin);
    VKG_CUDA(cudaFuncSetAttribute(gemm_tcgen05_kernel<E_GENERIC>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    for (int i = 0; i < kNumSpecialised; ++i)
      VKG_CUDA(cudaFuncSetAttribute(kSpecialised[i].fn, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    SMEM_BYTES));
    dev->gemm_attr_set = true;
  }
  long long total_tiles = (long long)p.tiles_m * p.tiles_n * batch;
  VKG_REQUIRE(total_tiles < (1ll << 31), "gemm: too many tiles");
  int ctas = a->max_ctas > 0 ? a->max_ctas : dev->sm_count;
  if (ctas > total_tiles) ctas = (int)total_tiles;
  int mode = (a->bias ? E_BIAS : 0) | (a->pre ? E_PRE : 0) | (a->act ? E_ACT : 0) |
             (a->dact_z ? E_DACT : 0) | (a->residual ? E_RES : 0) | (a->C2 ? E_C2 : 0) |
             (a->c_dtype == VKG_F16 ? E_F16 : a->c_dtype == VKG_BF16 ? E_BF16 : 0);
  GemmKernel fn = gemm_tcgen05_kernel<E_GENERIC>;
  if (vec) {
    for (int i = 0; i < kNumSpecialised; ++i)
      if (kSpecialised[i].mode == mode) fn = kSpecialised[i].fn;
  }
  fn<<<ctas, NUM_THREADS, SMEM_BYTES, dev->stream>>>(tmA, tmB, p);
  return vkg_check_launch("gemm_tcgen05_kernel");
}
