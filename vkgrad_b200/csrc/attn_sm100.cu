// Fused causal attention for sm_100a, head dimension 64: replaces the reference's
// per-layer chain  QK^T matmul -> attn_softmax -> PV matmul  (transformer.py:144-155)
// and its backward chain (transformer.py:167-182) without ever writing the T x T score,
// probability or gradient tensors to HBM.
//
// Forward, one CTA per (128-query tile, head, sequence), 320 threads, two CTAs per SM:
//   warp 0      TMA producer: Q once, then the K and V tiles
//   warp 1      TMEM allocation + tcgen05.mma issue (the warp runs converged, one elected lane
//               per instruction)
//   warps 2..9  softmax: TMEM lane = query row; two warps share a lane quarter, each takes 64
//               of a tile's 128 keys, so a thread owns half of one row
// Two kernels.  attn_fwd1_kernel (the default) makes one pass: S = Q K^T once per key tile,
// P~ = exp2(S c - m) against a running reference maximum m that is moved -- and O~ and the row
// sum rescaled -- only when a tile exceeds it by more than 2^8.  attn_fwd_kernel makes two:
//   pass 1  S = Q K^T  -> row maximum m only (no exponentials)
//   pass 2  S again, P~ = exp2(S c - m), O~ += P~ V, no rescaling at all
// (QK^T has K = 64, so doing it twice costs little: 45 vs 37 us per layer at 8 x 1024 x 12.)
// In both, P~ is rounded to fp16 -- into tensor memory in the one-pass kernel, where P~ V reads
// it as the A operand, into swizzled shared memory in the two-pass one --, O~ accumulates in
// TMEM, the row sum l of the UN-rounded P~ is kept in fp32, and O = O~ / l when the tile is
// stored.
// Backward: two persistent kernels, the dQ kernel (which also forms delta = rowsum(dO * O))
// and the dK / dV kernel; their comments are beside them.
// Rounding points against the reference: it rounds the NORMALISED probability P = P~ / l to
// fp16 before P V (tkernels.py:123); here the un-normalised P~ (in (0, 1], the row's largest
// entry exactly 1) is rounded and 1 / l is applied to the fp32 accumulator, so O carries the
// same relative rounding per product and one division less per score.  The backward kernels
// rebuild the normalised P from the saved log-sum-exp and round that, as the reference does
// (tkernels.py:123, 183); O, dQ, dK, dV are stored fp16 as there (tkernels.py:284, 228-230).
// Every wait is bounded (see tcgen05.cuh); a wait that gives up flags the error word,
// all roles leave their loops, TMEM is freed and the CTA returns.
#include "common.cuh"
#include "tcgen05.cuh"

namespace {

using namespace tc05;

constexpr int FA_T = 128;          // query / key tile
constexpr int FA_HD = 64;          // head dimension
constexpr int FA_TILE_BYTES = FA_T * FA_HD * 2;  // 16 KB: one 128 x 64 fp16 tile, 128 B rows
constexpr int FA_THREADS = 320;      // producer + MMA + eight softmax warps
constexpr int FA_SOFTMAX_WARPS = 8;
constexpr int BW_SOFTMAX_WARPS = 16;   // dK / dV kernel: four warps per TMEM lane quarter, 32 keys of a row each
constexpr int DQ_SOFTMAX_WARPS = 16;   // dQ kernel: 8 or 16 (2 or 4 per lane quarter; 8 measured 2 % slower)
constexpr int DQ_MMA2_WARP = 2 + DQ_SOFTMAX_WARPS;        // the warp that issues dQ += dS K
constexpr int DQ_THREADS = (3 + DQ_SOFTMAX_WARPS) * 32;
constexpr int KV_MMA2_WARP = 2 + BW_SOFTMAX_WARPS;        // the warp that issues dV / dK
constexpr int BW_THREADS = (3 + BW_SOFTMAX_WARPS) * 32;
constexpr float LOG2E = 1.4426950408889634f;
// The softmax warps' waits suspend (mbarrier.try_wait with a time hint); the producer's and the
// MMA warps', which sit on the critical chain, poll.  Polling in the softmax warps too measured
// the same to 1 us per layer.
constexpr bool SM_SPIN = false;

struct AttnParams {
  int B, T, H, D;
  int nqt;                 // query tiles per sequence
  float cscale;            // softmax scale * log2(e)
  float scale;
  const uint32_t* seg;     // optional packed-sample starts (b*T + t)
  __half* out;             // forward: O, head-merged (rows, D)
  float* lse2;             // (B*H, T): row log2-sum-exp of the scaled scores
  const float* delta;      // backward: rowsum(dO * O), (B*H, T); the dQ kernel writes it (delta_out),
  float* delta_out;        // the dK / dV kernel, launched after it, reads it
  __half* dqkv;            // backward: (rows, 3D)
  float* colsum;           // backward, optional: [B * nqt * 4][3D] partial column sums of dqkv
  uint32_t* err;
};

// forward shared memory map (offsets from a 1024-aligned base)
constexpr int FW_Q = 0;
constexpr int FW_K = FW_Q + FA_TILE_BYTES;            // two K stages
constexpr int FW_V = FW_K + 2 * FA_TILE_BYTES;        // one V stage
constexpr int FW_P = FW_V + FA_TILE_BYTES;            // P: two 64-key blocks of 128 rows x 128 B
constexpr int FW_BAR = FW_P + 2 * FA_TILE_BYTES;
constexpr int FW_XCHG = FW_BAR + 256;                 // row statistics exchange: [2][128] floats; the
                                                      // one-pass kernel: [2][2][128] tagged 8-byte
                                                      // slots, then [2][128] floats
constexpr int FW_SMEM = FW_XCHG + 4096 + 1024 + 1024;

// P and dS tiles use the 128B-swizzled layout of TMA and the UMMA descriptors: 16-byte
// piece c8 (8 keys) of row r of a 64-key block sits at r * 128 + ((c8 ^ (r & 7)) << 4).

// Row maximum over this thread's 64 raw scores of one key tile.  MASK adds the causal /
// packed-sample test and is compiled only into the tiles that need it.
template <bool MASK>
__device__ __forceinline__ float fwd_max_tile(const uint32_t (&r)[64], int key0, int qi, int st, float m) {
#pragma unroll
  for (int e = 0; e < 64; ++e) {
    if (MASK) {
      const int key = key0 + e;
      if (key > qi || key < st) continue;
    }
    m = fmaxf(m, __uint_as_float(r[e]));
  }
  return m;
}

// P = exp2(s * cscale - m) for this thread's 64 scores, rounded to fp16 into the swizzled
// row `prow` (x = row & 7); returns the fp32 sum of the row's part.
template <bool MASK>
__device__ __forceinline__ float fwd_p_tile(const uint32_t (&r)[64], int key0, int qi, int st, float cscale,
                                         float nm, uint8_t* prow, uint32_t x) {
  float l = 0.f;
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    __half2 hv[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float pv[2];
#pragma unroll
      for (int w = 0; w < 2; ++w) {
        const int idx = u * 8 + 2 * e + w;
        float pr = vkg_ex2(fmaf(__uint_as_float(r[idx]), cscale, nm));
        if (MASK) {
          const int key = key0 + idx;
          if (key > qi || key < st) pr = 0.f;
        }
        pv[w] = pr;
      }
      l += pv[0] + pv[1];
      hv[e] = __floats2half2_rn(pv[0], pv[1]);
    }
    *reinterpret_cast<uint4*>(prow + (((uint32_t)u ^ x) << 4)) = *reinterpret_cast<uint4*>(hv);
  }
  return l;
}

// The same exponentials for a P~ that stays in tensor memory: the fp16 pairs (keys 2i, 2i + 1)
// replace r[i], ready for tcgen05.st; returns the fp32 sum of the un-rounded values.
template <bool MASK>
__device__ __forceinline__ float fwd_p_pack(uint32_t (&r)[64], int key0, int qi, int st, float cscale,
                                            float nm) {
  float l = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    float pv[2];
#pragma unroll
    for (int w = 0; w < 2; ++w) {
      float pr = vkg_ex2(fmaf(__uint_as_float(r[2 * i + w]), cscale, nm));
      if (MASK) {
        const int key = key0 + 2 * i + w;
        if (key > qi || key < st) pr = 0.f;
      }
      pv[w] = pr;
    }
    l += pv[0] + pv[1];
    const __half2 h = __floats2half2_rn(pv[0], pv[1]);
    r[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return l;
}

// Store a warp's block of 32 rows x NU 16-byte groups (lane = row, v[u] = group u of the row)
// to global rows of `pitch` bytes so that every store instruction writes whole contiguous row
// segments: the block goes through the warp's private staging area (32 x NU x 16 bytes, XOR
// swizzled so both passes are conflict-free) and comes back with 32 / NU rows per instruction.
// One row per lane (128-byte rows 4608 bytes apart for a 768-wide model) measured 1.5 us per
// item on the softmax warps' critical path.  rows_ok = how many of the 32 rows exist.
template <int NU>
__device__ __forceinline__ void warp_store_rows(const uint4 (&v)[NU], uint8_t* stage, int lane,
                                                uint8_t* dst_row0, size_t pitch, int rows_ok) {
  static_assert(NU == 4 || NU == 8, "64- or 128-byte row segments");
#pragma unroll
  for (int u = 0; u < NU; ++u)
    *reinterpret_cast<uint4*>(stage + lane * (NU * 16) + ((u ^ (lane & (NU - 1))) << 4)) = v[u];
  __syncwarp();
  constexpr int RPI = 32 / NU;        // rows per store instruction
  const int u = lane % NU;
#pragma unroll
  for (int i = 0; i < NU; ++i) {
    const int row = i * RPI + lane / NU;
    const uint4 x = *reinterpret_cast<const uint4*>(stage + row * (NU * 16) + ((u ^ (row & (NU - 1))) << 4));
    if (row < rows_ok) *reinterpret_cast<uint4*>(dst_row0 + (size_t)row * pitch + u * 16) = x;
  }
  __syncwarp();
}

__global__ void __launch_bounds__(FA_THREADS, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm, const AttnParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar = base + FW_BAR;
  // barriers: 0 q_full, 1-2 k_full, 3-4 k_empty, 5 v_full, 6 v_empty, 7 s_full, 8 s_free,
  //           9 p_full, 10 p_free, 11 o_full
  auto B_ = [bar](int i) { return bar + 8u * i; };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + FW_BAR + 128);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(gbase + FW_BAR + 136);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int HB = p.H * p.B;
  const int qt = p.nqt - 1 - (int)(blockIdx.x / HB);   // heaviest query tiles first
  const int hb = blockIdx.x % HB;
  const int h = hb % p.H, b = hb / p.H;
  const int q0 = qt * FA_T;
  const int nj = qt + 1;                                 // key tiles 0..qt
  const int row0 = b * p.T;                              // first row of this sequence

  pdl_trigger();
  if (threadIdx.x == 0) {
    prefetch_tensormap(&tm);
    for (int i = 0; i < 12; ++i) mbar_init(B_(i), (i == 8 || i == 9) ? FA_SOFTMAX_WARPS : 1);
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, 256);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  pdl_wait();      // the projection that wrote qkv has completed
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tO = tmem + 128;

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      mbar_expect_tx(B_(0), FA_TILE_BYTES);
      tma_load_2d(base + FW_Q, &tm, B_(0), h * FA_HD, row0 + q0);
      int it = 0;
      for (int pass = 0; pass < 2 && ok; ++pass) {
        for (int j = 0; j < nj && ok; ++j, ++it) {
          const int s = it & 1;
          ok = mbar_wait<true>(B_(3 + s), ((it >> 1) & 1) ^ 1u, abort_flag, p.err, 0x1100u + s);
          if (!ok) break;
          mbar_expect_tx(B_(1 + s), FA_TILE_BYTES);
          tma_load_2d(base + FW_K + s * FA_TILE_BYTES, &tm, B_(1 + s), p.D + h * FA_HD,
                      row0 + j * FA_T);
          if (pass == 1) {
            ok = mbar_wait<true>(B_(6), (j & 1) ^ 1u, abort_flag, p.err, 0x1200u);
            if (!ok) break;
            mbar_expect_tx(B_(5), FA_TILE_BYTES);
            tma_load_2d(base + FW_V, &tm, B_(5), 2 * p.D + h * FA_HD, row0 + j * FA_T);
          }
        }
      }
    }
  } else if (warp == 1) {
    // the whole warp runs this converged; one elected lane issues each tcgen05 instruction
    const uint32_t idesc_s = make_idesc(0, 0, 0, FA_T);     // Q K^T: both K-major, N = 128 keys
    const uint32_t idesc_o = make_idesc(0, 0, 1, FA_HD);    // P V: P K-major, V MN-major, N = 64
    bool ok = mbar_wait_warp<true>(B_(0), 0, abort_flag, p.err, 0x2000u);
    // descriptor halves (tcgen05.cuh): start address and leading offset in the low word
    const uint32_t d_hi = smem_desc_hi(1024);
    const uint32_t q_lo = smem_desc_lo(base + FW_Q, 16), k_lo = smem_desc_lo(base + FW_K, 16);
    const uint32_t p_lo = smem_desc_lo(base + FW_P, 16), v_lo = smem_desc_lo(base + FW_V, 8192);
    // S number n (n counts both passes): wait for its K stage and for the softmax warps
    // to have pulled the previous S out of TMEM, then issue Q K^T.
    auto issue_s = [&](int n) -> bool {
      const int s = n & 1;
      if (!(mbar_wait_warp<true>(B_(1 + s), (n >> 1) & 1, abort_flag, p.err, 0x2100u + s) &&
            mbar_wait_warp<true>(B_(8), (n & 1) ^ 1u, abort_flag, p.err, 0x2200u)))
        return false;
      tcgen05_fence_after();
      umma_f16_chain<4>(tS, q_lo, 2, k_lo + (uint32_t)s * (FA_TILE_BYTES >> 4), 2, d_hi, idesc_s, 0u);
      umma_commit_one(B_(3 + s));   // K stage free once these retire
      umma_commit_one(B_(7));       // S ready
      return true;
    };
    // pass 1: S only.  Pass 2 is software-pipelined: S(j+1) is issued before P(j) V, so
    // the tensor core works on the next scores while the softmax warps finish P(j).
    int n = 0;
    for (; n < nj && ok; ++n) ok = issue_s(n);
    if (ok) ok = issue_s(n++);
    for (int j = 0; j < nj && ok; ++j) {
      if (j + 1 < nj) {
        ok = issue_s(n++);
        if (!ok) break;
      }
      ok = mbar_wait_warp<true>(B_(9), j & 1, abort_flag, p.err, 0x2300u) &&
           mbar_wait_warp<true>(B_(5), j & 1, abort_flag, p.err, 0x2400u);
      if (!ok) break;
      tcgen05_fence_after();
      // P: two 64-key blocks, K-major; V: MN-major, 16 keys = two 8-row groups further down
      umma_f16_chain<4>(tO, p_lo, 2, v_lo, 128, d_hi, idesc_o, j ? 1u : 0u);
      umma_f16_chain<4>(tO, p_lo + (FA_TILE_BYTES >> 4), 2, v_lo + 4 * 128, 128, d_hi, idesc_o, 1u);
      umma_commit_one(B_(6));     // V free
      umma_commit_one(B_(10));    // P free
    }
    if (ok) umma_commit_one(B_(11));
  } else {
    // Softmax: two warps per TMEM lane quarter; `half` picks which 64 of the tile's 128
    // keys this warp handles.  Each thread owns one query row of its half.
    const int half = (warp - 2) >> 2;
    const int qr = (warp & 3) * 32 + lane;      // row within the tile = TMEM lane
    const int qi = q0 + qr;                     // query index in the sequence
    const bool q_ok = qi < p.T;
    const int st = (p.seg && q_ok) ? (int)p.seg[row0 + qi] : 0;
    const uint32_t t_lane = ((uint32_t)((warp & 3) * 32)) << 16;
    float* xchg = reinterpret_cast<float*>(gbase + FW_XCHG);   // [2][128] row statistics
    float m = -1e30f, l = 0.f;
    bool ok = true;
    int it = 0;
    // pass 1: row maximum of the scaled scores (no exponentials)
    for (int j = 0; j < nj && ok; ++j, ++it) {
      ok = mbar_wait_warp<SM_SPIN>(B_(7), it & 1, abort_flag, p.err, 0x3100u);
      if (!ok) break;
      tcgen05_fence_after();
      const bool need_mask = (j == qt) || (p.seg != nullptr);
      uint32_t r[64];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld16(tS + t_lane + half * 64 + c * 16, r + c * 16);
      tmem_wait_ld();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(B_(8));        // S may be overwritten
      // the scale is positive, so the maximum of the raw scores is enough here
      if (need_mask) m = fwd_max_tile<true>(r, j * FA_T + half * 64, qi, st, m);
      else m = fwd_max_tile<false>(r, 0, 0, 0, m);
    }
    xchg[half * 128 + qr] = m;
    asm volatile("bar.sync 1, 256;" ::: "memory");   // the eight softmax warps
    m = fmaxf(xchg[qr], xchg[128 + qr]) * p.cscale;  // row maximum of the scaled scores
    const float nm = -m;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    // pass 2: P = exp2(t - m) rounded to fp16 (normalised by 1/l at the very end), l in fp32
    for (int j = 0; j < nj && ok; ++j, ++it) {
      ok = mbar_wait_warp<SM_SPIN>(B_(7), it & 1, abort_flag, p.err, 0x3150u);
      if (!ok) break;
      tcgen05_fence_after();
      const bool need_mask = (j == qt) || (p.seg != nullptr);
      uint32_t r[64];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld16(tS + t_lane + half * 64 + c * 16, r + c * 16);
      tmem_wait_ld();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(B_(8));
      ok = mbar_wait_warp<SM_SPIN>(B_(10), (j & 1) ^ 1u, abort_flag, p.err, 0x3200u);   // P buffer free
      if (!ok) break;
      uint8_t* prow = gbase + FW_P + half * FA_TILE_BYTES + qr * 128;
      if (need_mask) l += fwd_p_tile<true>(r, j * FA_T + half * 64, qi, st, p.cscale, nm, prow, qr & 7);
      else l += fwd_p_tile<false>(r, 0, 0, 0, p.cscale, nm, prow, qr & 7);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(B_(9));        // this warp's part of P is in shared memory
    }
    xchg[half * 128 + qr] = l;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    l = xchg[qr] + xchg[128 + qr];
    const float inv_l = 1.0f / l;               // l >= 1: key == query is always valid
    if (half == 0 && q_ok) p.lse2[(size_t)(b * p.H + h) * p.T + qi] = m + log2f(l);
    if (ok) ok = mbar_wait_warp<SM_SPIN>(B_(11), 0, abort_flag, p.err, 0x3300u);
    if (ok) {
      tcgen05_fence_after();
      uint32_t r[32];                            // this half's 32 of the 64 output columns
      tmem_ld16(tO + t_lane + half * 32, r);
      tmem_ld16(tO + t_lane + half * 32 + 16, r + 16);
      tmem_wait_ld();
      {
        uint4 hv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          __half2 h2[4];
#pragma unroll
          for (int e = 0; e < 4; ++e)
            h2[e] = __floats2half2_rn(__uint_as_float(r[u * 8 + 2 * e]) * inv_l,
                                      __uint_as_float(r[u * 8 + 2 * e + 1]) * inv_l);
          hv[u] = *reinterpret_cast<uint4*>(h2);
        }
        // every product has retired (o_full), so the P buffer serves as the staging area
        const int q_w = q0 + (warp & 3) * 32;
        __half* dst = p.out + (size_t)(row0 + q_w) * p.D + h * FA_HD + half * 32;
        warp_store_rows<4>(hv, gbase + FW_P + (warp - 2) * 2048, lane, reinterpret_cast<uint8_t*>(dst),
                           (size_t)p.D * 2, p.T - q_w);
      }
    }
  }

  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  if (*abort_flag) {
    long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) {
    }
  }
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem, 256);
  }
}

// ---- forward, one pass ------------------------------------------------------------------
//
// The same CTA shape and roles, but every S = Q K^T is computed once: the softmax warps keep a
// running reference maximum m per row, P~ = exp2(S c - m) goes to the tensor core as before,
// and O~ and the row sum l are rescaled only when a tile's row maximum exceeds the reference by
// more than 2^8 (then the warps multiply their columns of O~ in TMEM by exp2(m_old - m_new)).
// With the threshold P~ stays below 256, well inside fp16, and its relative rounding is that of
// the two-pass kernel; for ordinary score ranges no rescale ever runs.  The two warps that share
// a row (64 keys each) exchange their tile maxima through shared memory with a tagged slot and
// a bounded poll -- no named barrier inside the loop, so an aborting warp cannot strand its
// partner.  The rescale sits between "P V of the previous tile has retired" (the wait that
// guards the P buffer anyway) and this warp's arrival on p_full, so it needs no barrier of its
// own: O~ is quiet exactly there.
constexpr float FW1_LAZY = 8.0f;      // log2 of the largest P~ the running reference allows

__global__ void __launch_bounds__(FA_THREADS, 2)
attn_fwd1_kernel(const __grid_constant__ CUtensorMap tm, const AttnParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar = base + FW_BAR;
  // barriers: 0 q_full, 1-2 k_full, 3-4 k_empty, 5 v_full, 6 v_empty, 7 s_full, 8 s_free,
  //           9 p_full, 10 p_free, 11 o_full
  auto B_ = [bar](int i) { return bar + 8u * i; };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + FW_BAR + 128);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(gbase + FW_BAR + 136);
  // [parity][half][row] (tag, value) pairs for the per-tile maxima; the final row sums reuse it
  volatile unsigned long long* xslot = reinterpret_cast<volatile unsigned long long*>(gbase + FW_XCHG);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int HB = p.H * p.B;
  const int qt = p.nqt - 1 - (int)(blockIdx.x / HB);   // heaviest query tiles first
  const int hb = blockIdx.x % HB;
  const int h = hb % p.H, b = hb / p.H;
  const int q0 = qt * FA_T;
  const int nj = qt + 1;
  const int row0 = b * p.T;

  pdl_trigger();
  if (threadIdx.x == 0) {
    prefetch_tensormap(&tm);
    for (int i = 0; i < 12; ++i) mbar_init(B_(i), (i == 8 || i == 9) ? FA_SOFTMAX_WARPS : 1);
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  for (int i = threadIdx.x; i < 2 * 2 * FA_T; i += blockDim.x) xslot[i] = 0ull;   // tag 0 = empty
  if (warp == 1) tmem_alloc(tmem_slot, 256);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  pdl_wait();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tO = tmem + 128, tP = tmem + 192;   // P~: 128 keys, two per column

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(B_(0), FA_TILE_BYTES);
      tma_load_2d(base + FW_Q, &tm, B_(0), h * FA_HD, row0 + q0);
      for (int j = 0; j < nj; ++j) {
        const int s = j & 1;
        if (!mbar_wait<true>(B_(3 + s), ((j >> 1) & 1) ^ 1u, abort_flag, p.err, 0x6100u + s)) break;
        mbar_expect_tx(B_(1 + s), FA_TILE_BYTES);
        tma_load_2d(base + FW_K + s * FA_TILE_BYTES, &tm, B_(1 + s), p.D + h * FA_HD, row0 + j * FA_T);
        if (!mbar_wait<true>(B_(6), (j & 1) ^ 1u, abort_flag, p.err, 0x6200u)) break;
        mbar_expect_tx(B_(5), FA_TILE_BYTES);
        tma_load_2d(base + FW_V, &tm, B_(5), 2 * p.D + h * FA_HD, row0 + j * FA_T);
      }
    }
  } else if (warp == 1) {
    // the whole warp runs this converged; one elected lane issues each tcgen05 instruction
    const uint32_t idesc_s = make_idesc(0, 0, 0, FA_T);
    const uint32_t idesc_o = make_idesc(0, 0, 1, FA_HD);
    bool ok = mbar_wait_warp<true>(B_(0), 0, abort_flag, p.err, 0x7000u);
    // descriptor halves (tcgen05.cuh): start address and leading offset in the low word
    const uint32_t d_hi = smem_desc_hi(1024);
    const uint32_t q_lo = smem_desc_lo(base + FW_Q, 16), k_lo = smem_desc_lo(base + FW_K, 16);
    const uint32_t v_lo = smem_desc_lo(base + FW_V, 8192);
    auto issue_s = [&](int n) -> bool {
      const int s = n & 1;
      if (!(mbar_wait_warp<true>(B_(1 + s), (n >> 1) & 1, abort_flag, p.err, 0x7100u + s) &&
            mbar_wait_warp<true>(B_(8), (n & 1) ^ 1u, abort_flag, p.err, 0x7200u)))
        return false;
      tcgen05_fence_after();
      umma_f16_chain<4>(tS, q_lo, 2, k_lo + (uint32_t)s * (FA_TILE_BYTES >> 4), 2, d_hi, idesc_s, 0u);
      umma_commit_one(B_(3 + s));   // K stage free once these retire
      umma_commit_one(B_(7));       // S ready
      return true;
    };
    int n = 0;
    if (ok) ok = issue_s(n++);
    for (int j = 0; j < nj && ok; ++j) {
      if (j + 1 < nj) {          // the next scores first: the tensor core works while P(j) forms
        ok = issue_s(n++);
        if (!ok) break;
      }
      ok = mbar_wait_warp<true>(B_(9), j & 1, abort_flag, p.err, 0x7300u) &&
           mbar_wait_warp<true>(B_(5), j & 1, abort_flag, p.err, 0x7400u);
      if (!ok) break;
      tcgen05_fence_after();
      // P~ from tensor memory; V: MN-major, 16 keys = two 8-row groups further down
      umma_f16_ts_chain<8>(tO, tP, v_lo, 128, d_hi, idesc_o, j ? 1u : 0u);
      umma_commit_one(B_(6));     // V free
      umma_commit_one(B_(10));    // P free, and O~ quiet until the next p_full
    }
    if (ok) umma_commit_one(B_(11));
  } else {
    const int half = (warp - 2) >> 2;
    const int qr = (warp & 3) * 32 + lane;      // row within the tile = TMEM lane
    const int qi = q0 + qr;
    const bool q_ok = qi < p.T;
    const int st = (p.seg && q_ok) ? (int)p.seg[row0 + qi] : 0;
    const uint32_t t_lane = ((uint32_t)((warp & 3) * 32)) << 16;
    float m_ref = -1e30f, l = 0.f;              // reference maximum (scaled units), row sum
    bool ok = true;
    for (int j = 0; j < nj && ok; ++j) {
      ok = mbar_wait_warp<SM_SPIN>(B_(7), j & 1, abort_flag, p.err, 0x8100u);
      if (!ok) break;
      tcgen05_fence_after();
      const bool need_mask = (j == qt) || (p.seg != nullptr);
      uint32_t r[64];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld16(tS + t_lane + half * 64 + c * 16, r + c * 16);
      tmem_wait_ld();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(B_(8));        // S may be overwritten
      // this half's maximum of the row, then the partner's through its tagged slot
      float mt = need_mask ? fwd_max_tile<true>(r, j * FA_T + half * 64, qi, st, -1e30f)
                           : fwd_max_tile<false>(r, 0, 0, 0, -1e30f);
      const unsigned long long tag = (unsigned long long)(unsigned)(j + 1) << 32;
      xslot[((j & 1) * 2 + half) * FA_T + qr] = tag | (unsigned long long)__float_as_uint(mt);
      float mo = -1e30f;
      {
        volatile unsigned long long* theirs = xslot + ((j & 1) * 2 + (1 - half)) * FA_T + qr;
        long long t0 = 0;
        for (unsigned spins = 0;; ++spins) {
          const unsigned long long v = *theirs;
          if ((v >> 32) == (unsigned long long)(unsigned)(j + 1)) {
            mo = __uint_as_float((uint32_t)v);
            break;
          }
          if ((spins & 255u) == 255u) {
            if (*abort_flag) { ok = false; break; }
            if (t0 == 0) t0 = clock64();
            else if (clock64() - t0 > WAIT_BUDGET_CYCLES) {
              *abort_flag = 1u;
              if (atomicCAS(p.err, 0u, VKG_ERR_WAIT_TIMEOUT) == 0u) p.err[1] = 0x8150u;
              __threadfence_system();
              ok = false;
              break;
            }
          }
        }
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const float m_row = fmaxf(mt, mo) * p.cscale;
      // the previous P V has retired: the P buffer is free and O~ is quiet
      ok = mbar_wait_warp<SM_SPIN>(B_(10), (j & 1) ^ 1u, abort_flag, p.err, 0x8200u);
      if (!ok) break;
      if (j == 0) {
        m_ref = m_row;
      } else {
        const bool grow = m_row > m_ref + FW1_LAZY;
        if (__any_sync(0xffffffffu, grow)) {
          // rescale this half's 32 columns of O~ (aligned TMEM accesses: the whole warp goes)
          const float alpha = grow ? vkg_ex2(m_ref - m_row) : 1.0f;
          tcgen05_fence_after();
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {          // 16 columns at a time: r[] is still live
            uint32_t o[16];
            tmem_ld16(tO + t_lane + half * 32 + c * 16, o);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 16; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tmem_st16(tO + t_lane + half * 32 + c * 16, o);
          }
          tmem_wait_st();
          l *= alpha;
          if (grow) m_ref = m_row;
        }
      }
      const float nm = -m_ref;
      // P~ packed two keys per register, overwriting the scores they came from, then into
      // this half's 32 columns of the P~ area
      if (need_mask) l += fwd_p_pack<true>(r, j * FA_T + half * 64, qi, st, p.cscale, nm);
      else l += fwd_p_pack<false>(r, 0, 0, 0, p.cscale, nm);
      tmem_st16(tP + t_lane + half * 32, r);
      tmem_st16(tP + t_lane + half * 32 + 16, r + 16);
      tmem_wait_st();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(B_(9));        // this warp's part of P~ is in tensor memory
    }
    // row sums of the two halves (both hold the same reference maximum)
    float* xchg = reinterpret_cast<float*>(gbase + FW_XCHG + 2 * 2 * FA_T * 8);
    xchg[half * 128 + qr] = l;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    l = xchg[qr] + xchg[128 + qr];
    const float inv_l = 1.0f / l;               // l > 0: key == query is always valid
    if (half == 0 && q_ok) p.lse2[(size_t)(b * p.H + h) * p.T + qi] = m_ref + log2f(l);
    if (ok) ok = mbar_wait_warp<SM_SPIN>(B_(11), 0, abort_flag, p.err, 0x8300u);
    if (ok) {
      tcgen05_fence_after();
      uint32_t r[32];
      tmem_ld16(tO + t_lane + half * 32, r);
      tmem_ld16(tO + t_lane + half * 32 + 16, r + 16);
      tmem_wait_ld();
      uint4 hv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        __half2 h2[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
          h2[e] = __floats2half2_rn(__uint_as_float(r[u * 8 + 2 * e]) * inv_l,
                                    __uint_as_float(r[u * 8 + 2 * e + 1]) * inv_l);
        hv[u] = *reinterpret_cast<uint4*>(h2);
      }
      const int q_w = q0 + (warp & 3) * 32;
      __half* dst = p.out + (size_t)(row0 + q_w) * p.D + h * FA_HD + half * 32;
      warp_store_rows<4>(hv, gbase + FW_P + (warp - 2) * 2048, lane, reinterpret_cast<uint8_t*>(dst),
                         (size_t)p.D * 2, p.T - q_w);
    }
  }

  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  if (*abort_flag) {
    long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) {
    }
  }
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem, 256);
  }
}

// ---- backward --------------------------------------------------------------------------
//
// One 32-key chunk of a (query row, key tile) pair: rebuild P from S and the saved
// log-sum-exp and form dS = P (dP - delta) scale, both rounded to fp16 and packed into registers
// (four 16-byte groups each); bwd_chunk_store writes them into the swizzled [query row][key]
// layout once the buffer, which the tensor core may still be reading, is free.  nlse = -lse2
// (or -inf for a row past the end of the sequence, which makes its P exactly 0), dsc = -delta *
// scale: each element costs two FMAs, one exp2, one multiply and the conversions.  MASK adds the
// per-element causal / packed-sample test and is only compiled into the tiles that need it.
template <bool MASK>
__device__ __forceinline__ void bwd_chunk_regs(const uint32_t* rs, const uint32_t* rdp, int c,
                                               int key0, int qi, int st, float cscale, float scale,
                                               float nlse, float dsc, uint4* outp, uint4* outd) {
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    __half2 hp[4], hd[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float pv[2], dv[2];
#pragma unroll
      for (int w = 0; w < 2; ++w) {
        const int idx = u * 8 + 2 * e + w;
        float pr = vkg_ex2(fmaf(__uint_as_float(rs[idx]), cscale, nlse));
        if (MASK) {
          const int key = key0 + c * 32 + idx;
          if (key > qi || key < st) pr = 0.f;
        }
        pv[w] = pr;
        dv[w] = pr * fmaf(__uint_as_float(rdp[idx]), scale, dsc);
      }
      hp[e] = __floats2half2_rn(pv[0], pv[1]);
      hd[e] = __floats2half2_rn(dv[0], dv[1]);
    }
    outp[u] = *reinterpret_cast<uint4*>(hp);
    outd[u] = *reinterpret_cast<uint4*>(hd);
  }
}

__device__ __forceinline__ void bwd_chunk_store(int c, int r, const uint4* outp, const uint4* outd,
                                                uint8_t* sp, uint8_t* sds) {
  const uint32_t row_off = (uint32_t)(r * 128), rx = (uint32_t)(r & 7);
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int cc = c * 4 + u;
    const uint32_t off = (uint32_t)((cc >> 3) * FA_TILE_BYTES) + row_off + ((((uint32_t)cc & 7u) ^ rx) << 4);
    *reinterpret_cast<uint4*>(sp + off) = outp[u];
    *reinterpret_cast<uint4*>(sds + off) = outd[u];
  }
}

// Column sums of one warp's 32 rows x NC columns (lane = row; fp16 values as stored, 0 for rows
// that do not exist) without shared memory: a reduce-scatter over the lanes.  Each step halves
// the columns a lane holds and adds the partner lane's share of the half it keeps, so after five
// steps lane l holds the sums of columns l * NC / 32 .. (l + 1) * NC / 32 - 1 and writes them to
// dst.  The order of the additions is fixed, so the result does not depend on timing.
template <int NC>
__device__ __forceinline__ void warp_col_sums(float (&v)[NC], int lane, float* dst) {
  static_assert(NC == 32 || NC == 64, "one or two columns per lane");
#pragma unroll
  for (int step = 0; step < 5; ++step) {
    const int off = 16 >> step, n = NC >> (step + 1);
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int c = 0; c < n; ++c) {
      const float keep = upper ? v[c + n] : v[c];
      const float send = upper ? v[c] : v[c + n];
      v[c] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
  }
  constexpr int PER = NC / 32;
#pragma unroll
  for (int c = 0; c < PER; ++c) dst[lane * PER + c] = v[c];
}

// Item number j of persistent CTA c out of G: rows of G items are dealt left to right and right
// to left in turn, which spreads items sorted by falling cost almost evenly (within 3 % of the
// mean for 8 query tiles x 96 heads on 148 CTAs; plain round-robin is 16 % off).
__device__ __forceinline__ int snake_item(int j, int G, int c) {
  return j * G + ((j & 1) ? G - 1 - c : c);
}

// dK / dV: persistent CTAs, one per SM, each taking (key tile, head, sequence) items
// blockIdx.x, blockIdx.x + gridDim.x, ... (items are ordered heaviest key tile first) and, per
// item, looping over the query tiles at or below the diagonal.  The pipeline runs across item
// boundaries: barrier phases follow a per-CTA count of (item, query tile) steps, the producer
// reloads K / V as soon as the item's last S / dP products have retired (kv_free) and the tensor
// core starts the next item's first S / dP before this item's last dV / dK, so a CTA pays the
// load -> S -> softmax -> dV latency chain once per launch instead of once per item (measured
// at 5.6 us per item when every item was its own CTA).  The accumulators are handed back by the
// softmax warps (acc_free) before the next item's first dV / dK overwrites them.
// TMEM: S [0,128) dP [128,256) dV [256,320) dK [320,384).
// Q / dO go through a ring of three stages and P / dS have ONE buffer.  A Q / dO stage is read
// by S / dP of its step and again by dV / dK of the same step a softmax later; with two stages
// (and P / dS double-buffered, which is what the shared memory then allowed) the load of step
// g + 1 waited for dV / dK of step g - 1 and the chain dV / dK -> load -> S / dP set the pace:
// 2.25 us per step measured against 1.45 us of tensor work.  With one P / dS buffer the softmax
// warps form the next step's P / dS in registers while the tensor core still reads the buffer
// for dV / dK, and only their stores wait for it.
constexpr int KV_STAGES = 3;
constexpr int KV_K = 0, KV_V = FA_TILE_BYTES, KV_Q = 2 * FA_TILE_BYTES,
              KV_DO = (2 + KV_STAGES) * FA_TILE_BYTES, KV_P = (2 + 2 * KV_STAGES) * FA_TILE_BYTES,
              KV_DS = KV_P + 2 * FA_TILE_BYTES, KV_OUT = KV_DS + 2 * FA_TILE_BYTES,   // output staging
              KV_BAR = KV_OUT + 2 * FA_TILE_BYTES, KV_SMEM = KV_BAR + 256 + 1024;
constexpr int KV_NBAR = 14 + 2 * KV_STAGES, KV_QD_FULL = 14, KV_QD_EMPTY = 14 + KV_STAGES;
static_assert(KV_SMEM <= 227 * 1024, "dK / dV kernel: shared memory");

__global__ void __launch_bounds__(BW_THREADS, 1)
attn_bwd_kv_kernel(const __grid_constant__ CUtensorMap tm, const __grid_constant__ CUtensorMap tmdo,
                   const AttnParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar = base + KV_BAR;
  // 0 kv_full, 5 sdp_full, 6 sdp_free, 7 pds_full, 8 pds_free, 9 out_full, 12 kv_free,
  // 13 acc_free, 14.. qd_full[stage], then qd_empty[stage]
  auto B_ = [bar](int i) { return bar + 8u * i; };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + KV_BAR + 192);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(gbase + KV_BAR + 200);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int HB = p.H * p.B;
  const int n_items = p.nqt * HB, G = (int)gridDim.x;

  pdl_trigger();
  if (threadIdx.x == 0) {
    prefetch_tensormap(&tm);
    prefetch_tensormap(&tmdo);
    for (int i = 0; i < KV_NBAR; ++i)
      mbar_init(B_(i), (i == 6 || i == 7 || i == 13) ? BW_SOFTMAX_WARPS : 1);
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  pdl_wait();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tdP = tmem + 128, tdV = tmem + 256, tdK = tmem + 320;

  if (warp == 0) {
    if (lane == 0) {
      int g = 0, j = 0;        // steps and items this CTA has started
      bool ok = true;
      for (;; ++j) {
        const int item = snake_item(j, G, (int)blockIdx.x);
        if (item >= n_items || !ok) break;
        const int kt = item / HB, hb = item % HB;
        const int h = hb % p.H, b = hb / p.H;
        const int row0 = b * p.T, k0 = kt * FA_T, ni = p.nqt - kt;
        // K / V of the previous item are read by its S / dP products only
        if (j > 0 && !mbar_wait<true>(B_(12), (j - 1) & 1, abort_flag, p.err, 0x4900u)) break;
        mbar_expect_tx(B_(0), 2 * FA_TILE_BYTES);
        tma_load_2d(base + KV_K, &tm, B_(0), p.D + h * FA_HD, row0 + k0);
        tma_load_2d(base + KV_V, &tm, B_(0), 2 * p.D + h * FA_HD, row0 + k0);
        for (int it = 0; it < ni; ++it, ++g) {
          const int s = g % KV_STAGES;
          const uint32_t ph = (uint32_t)(g / KV_STAGES) & 1u;
          if (!mbar_wait<true>(B_(KV_QD_EMPTY + s), ph ^ 1u, abort_flag, p.err, 0x4100u + s)) {
            ok = false;
            break;
          }
          mbar_expect_tx(B_(KV_QD_FULL + s), 2 * FA_TILE_BYTES);
          const int qrow = row0 + (kt + it) * FA_T;
          tma_load_2d(base + KV_Q + s * FA_TILE_BYTES, &tm, B_(KV_QD_FULL + s), h * FA_HD, qrow);
          tma_load_2d(base + KV_DO + s * FA_TILE_BYTES, &tmdo, B_(KV_QD_FULL + s), h * FA_HD, qrow);
        }
      }
    }
  } else if (warp == 1) {
    // S = Q K^T and dP = dO V^T of every step (dV / dK are issued by a warp of their own, as in
    // the dQ kernel).  The whole warp runs this converged; one elected lane issues each tcgen05
    // instruction.
    const uint32_t idesc_s = make_idesc(0, 0, 0, FA_T);    // [q x hd] . [key x hd]^T
    const uint32_t d_hi = smem_desc_hi(1024);              // descriptor halves (tcgen05.cuh)
    const uint32_t k_lo = smem_desc_lo(base + KV_K, 16), v_lo = smem_desc_lo(base + KV_V, 16);
    const uint32_t q_lo = smem_desc_lo(base + KV_Q, 16), do_lo = smem_desc_lo(base + KV_DO, 16);
    int s = 0;
    uint32_t ph = 0, par = 0;
    bool ok = true;
    for (int j = 0; ok; ++j) {
      const int item = snake_item(j, G, (int)blockIdx.x);
      if (item >= n_items) break;
      const int ni = p.nqt - item / HB;
      ok = mbar_wait_warp<true>(B_(0), j & 1, abort_flag, p.err, 0x4200u);
      for (int it = 0; it < ni && ok; ++it) {
        ok = mbar_wait_warp<true>(B_(KV_QD_FULL + s), ph, abort_flag, p.err, 0x4300u + s) &&
             mbar_wait_warp<true>(B_(6), par ^ 1u, abort_flag, p.err, 0x4400u);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t so = (uint32_t)s * (FA_TILE_BYTES >> 4);
        umma_f16_chain<4>(tS, q_lo + so, 2, k_lo, 2, d_hi, idesc_s, 0u);
        umma_f16_chain<4>(tdP, do_lo + so, 2, v_lo, 2, d_hi, idesc_s, 0u);
        umma_commit_one(B_(5));
        if (it == ni - 1) umma_commit_one(B_(12));    // the item's K / V may be replaced
        par ^= 1u;
        if (++s == KV_STAGES) {
          s = 0;
          ph ^= 1u;
        }
      }
    }
  } else if (warp == KV_MMA2_WARP) {
    // dV += P^T dO and dK += dS^T Q of every step.  Its commits cover this warp's instructions
    // only; a Q / dO stage is free when dV / dK of its step have retired, because the S / dP
    // that read it retired before the softmax warps could produce the P / dS these waited for.
    const uint32_t idesc_g = make_idesc(0, 1, 1, FA_HD);   // [q x key]^T . [q x hd]
    const uint32_t d_hi = smem_desc_hi(1024);
    const uint32_t qm_lo = smem_desc_lo(base + KV_Q, 8192), dom_lo = smem_desc_lo(base + KV_DO, 8192);
    const uint32_t pt_lo = smem_desc_lo(base + KV_P, FA_TILE_BYTES);
    const uint32_t dst_lo = smem_desc_lo(base + KV_DS, FA_TILE_BYTES);
    int g = 0, s = 0;
    bool ok = true;
    for (int j = 0; ok; ++j) {
      const int item = snake_item(j, G, (int)blockIdx.x);
      if (item >= n_items) break;
      const int ni = p.nqt - item / HB;
      for (int it = 0; it < ni; ++it, ++g) {
        ok = mbar_wait_warp<true>(B_(7), g & 1, abort_flag, p.err, 0x4500u);     // P / dS written
        if (!ok) break;
        if (it == 0 && j > 0) {              // the previous item's dV / dK have been read out
          ok = mbar_wait_warp<true>(B_(13), (j - 1) & 1, abort_flag, p.err, 0x4a00u);
          if (!ok) break;
        }
        tcgen05_fence_after();
        // K = 128 query rows, 16 at a time: every operand is MN-major here (P^T, dS^T with their
        // two 64-key blocks a tile apart; dO, Q with their 8-row groups 1024 bytes apart)
        const uint32_t so = (uint32_t)s * (FA_TILE_BYTES >> 4);
        umma_f16_chain<8>(tdV, pt_lo, 128, dom_lo + so, 128, d_hi, idesc_g, it ? 1u : 0u);
        umma_f16_chain<8>(tdK, dst_lo, 128, qm_lo + so, 128, d_hi, idesc_g, it ? 1u : 0u);
        umma_commit_one(B_(KV_QD_EMPTY + s));   // Q / dO stage free
        umma_commit_one(B_(8));                 // P / dS may be overwritten
        if (it == ni - 1) umma_commit_one(B_(9));
        if (++s == KV_STAGES) s = 0;
      }
    }
  } else {
    const int part = (warp - 2) >> 2;            // which 32 of the tile's 128 keys
    const int r = (warp & 3) * 32 + lane;
    const uint32_t t_lane = ((uint32_t)((warp & 3) * 32)) << 16;
    bool ok = true;
    // dV / dK of a finished item: wait for its last products, read the accumulators, hand them
    // back, store.  Runs after the NEXT item's first step, so the hand-off to the tensor core
    // (S, dP -> P, dS) does not stall at an item boundary.
    int pend_item = -1, pend_j = 0;
    auto store_item = [&](int item, int jj) -> bool {
      const int kt = item / HB, hb = item % HB;
      const int h = hb % p.H, b = hb / p.H;
      const int row0 = b * p.T, k0 = kt * FA_T;
      if (!mbar_wait_warp<SM_SPIN>(B_(9), jj & 1, abort_flag, p.err, 0x4800u)) return false;
      tcgen05_fence_after();
      const int key = k0 + r;     // accumulator rows are keys here
      // parts 0, 1 store the two 32-column halves of dV (slice 2 of dqkv), parts 2, 3 those of
      // dK (slice 1)
      uint32_t rr[32];
      const int slice = part < 2 ? 2 : 1, col0 = (part & 1) * 32;
      const uint32_t t = (part < 2 ? tdV : tdK) + t_lane + (uint32_t)col0;
      tmem_ld16(t, rr);
      tmem_ld16(t + 16, rr + 16);
      tmem_wait_ld();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(B_(13));           // the accumulators may be overwritten
      {
        uint4 hv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          __half2 h2[4];
#pragma unroll
          for (int e = 0; e < 4; ++e)
            h2[e] = __floats2half2_rn(__uint_as_float(rr[u * 8 + 2 * e]),
                                      __uint_as_float(rr[u * 8 + 2 * e + 1]));
          hv[u] = *reinterpret_cast<uint4*>(h2);
        }
        const int key_w = k0 + (warp & 3) * 32;      // first key of this warp's 32 rows
        __half* dst = p.dqkv + (size_t)(row0 + key_w) * 3 * p.D + slice * p.D + h * FA_HD + col0;
        warp_store_rows<4>(hv, gbase + KV_OUT + (warp - 2) * 2048, lane, reinterpret_cast<uint8_t*>(dst),
                           (size_t)3 * p.D * 2, p.T - key_w);
      }
      if (p.colsum) {
        // the qkv bias gradient: column sums of dV / dK as stored
        float val[32];
#pragma unroll
        for (int c = 0; c < 32; ++c)
          val[c] = key < p.T ? __half2float(__float2half_rn(__uint_as_float(rr[c]))) : 0.f;
        float* dst = p.colsum + ((size_t)(b * p.nqt + kt) * 4 + (warp & 3)) * 3 * p.D + slice * p.D +
                     h * FA_HD + col0;
        warp_col_sums<32>(val, lane, dst);
      }
      return true;
    };
    // statistics of this thread's row in the first query tile of an item
    auto first_stat = [&](int item, float& lse, float& dl, int& st) {
      const int kt = item / HB, hb = item % HB;
      const int qi = kt * FA_T + r;
      const bool q_ok = qi < p.T;
      const size_t i = (size_t)((hb / p.H) * p.H + hb % p.H) * p.T + (q_ok ? qi : 0);
      lse = p.lse2[i];
      dl = p.delta[i];
      st = (p.seg && q_ok) ? (int)p.seg[(hb / p.H) * p.T + qi] : 0;
    };
    float lse_f = 0.f, dl_f = 0.f;
    int st_f = 0;
    if ((int)blockIdx.x < n_items) first_stat((int)blockIdx.x, lse_f, dl_f, st_f);
    int g = 0, j = 0;
    for (;; ++j) {
      const int item = snake_item(j, G, (int)blockIdx.x);
      if (item >= n_items || !ok) break;
      const int kt = item / HB, hb = item % HB;
      const int h = hb % p.H, b = hb / p.H;
      const int row0 = b * p.T, k0 = kt * FA_T, ni = p.nqt - kt;
      // row statistics of query tile kt + it; the next tile's are fetched one step ahead, the
      // first tile's of the next item one item ahead (a load from global memory at the start
      // of an item would sit on the critical path)
      const float* lse_h = p.lse2 + (size_t)(b * p.H + h) * p.T;
      const float* delta_h = p.delta + (size_t)(b * p.H + h) * p.T;
      auto row_stat = [&](int qi, float& lse, float& dl, int& st) {
        const bool q_ok = qi < p.T;
        const int i = q_ok ? qi : 0;
        lse = lse_h[i];
        dl = delta_h[i];
        st = (p.seg && q_ok) ? (int)p.seg[row0 + qi] : 0;
      };
      float lse_n = lse_f, dl_n = dl_f;
      int st_n = st_f;
      {
        const int nxt = snake_item(j + 1, G, (int)blockIdx.x);
        if (nxt < n_items) first_stat(nxt, lse_f, dl_f, st_f);
      }
      for (int it = 0; it < ni && ok; ++it, ++g) {
        const int qt = kt + it;
        const int qi = qt * FA_T + r;
        const bool q_ok = qi < p.T;
        // a row past the end of the sequence gets lse = +inf, hence P = 0 and dS = 0
        const float nlse = q_ok ? -lse_n : -INFINITY, dsc = -dl_n * p.scale;
        const int st = st_n;
        if (it + 1 < ni) row_stat(qi + FA_T, lse_n, dl_n, st_n);
        const bool need_mask = (qt == kt) || (p.seg != nullptr);
        ok = mbar_wait_warp<SM_SPIN>(B_(5), g & 1, abort_flag, p.err, 0x4600u);
        if (!ok) break;
        tcgen05_fence_after();
        uint32_t rs[32], rdp[32];
        tmem_ld16(tS + t_lane + part * 32, rs);
        tmem_ld16(tS + t_lane + part * 32 + 16, rs + 16);
        tmem_ld16(tdP + t_lane + part * 32, rdp);
        tmem_ld16(tdP + t_lane + part * 32 + 16, rdp + 16);
        tmem_wait_ld();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(B_(6));          // S / dP may be overwritten
        // P and dS of this step, packed, in registers; the buffer is still being read
        uint4 hp[4], hd[4];
        if (need_mask) bwd_chunk_regs<true>(rs, rdp, part, k0, qi, st, p.cscale, p.scale, nlse, dsc, hp, hd);
        else bwd_chunk_regs<false>(rs, rdp, part, k0, qi, st, p.cscale, p.scale, nlse, dsc, hp, hd);
        ok = mbar_wait_warp<SM_SPIN>(B_(8), (g & 1) ^ 1u, abort_flag, p.err, 0x4700u);   // dV / dK of step g - 1 done
        if (!ok) break;
        uint8_t* sp = gbase + KV_P;
        uint8_t* sds = gbase + KV_DS;
        bwd_chunk_store(part, r, hp, hd, sp, sds);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(B_(7));
        if (pend_item >= 0) {      // the previous item's accumulators, now surely complete
          ok = store_item(pend_item, pend_j);
          pend_item = -1;
        }
      }
      pend_item = item;       // read this item's dV / dK out after the next item's first step
      pend_j = j;
    }
    if (ok && pend_item >= 0) ok = store_item(pend_item, pend_j);
  }
  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  if (*abort_flag) {
    long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) {
    }
  }
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// dQ: persistent CTAs like the dK / dV kernel; an item is a (query tile, head, sequence),
// heaviest query tile first, and loops over the key tiles up to the diagonal.  Q / dO are the
// per-item operands (reloaded once the item's last S / dP have retired: qd_free), K / V the
// per-step ones, in a ring of three stages: a stage is read by S / dP of its step and again by
// dQ of the same step a softmax later.
// dS never passes through shared memory: the softmax warps write it (fp16 pairs) into one of
// two areas of tensor memory with tcgen05.st, and dQ += dS K reads it there as the A operand.
// What paces a step is the warp that issues the MMAs: it shares its scheduler with softmax
// warps, a wait that is already satisfied costs it about 180 cycles and a loop iteration 400,
// so its loop is kept as short as it can be (one elected lane per instruction, descriptor
// halves stepped by adds, no wait that another wait implies).  Splitting a step into two
// half-steps with two softmax groups half a step apart doubled that warp's waits and commits
// and measured 15 % slower, although the softmax warps then idled less.
// This kernel also forms delta = rowsum(dO * O) (tkernels.py:176-179 computes the same number
// as sum_j dP_ij P_ij): the O tile of an item is loaded beside Q and dO, every softmax thread
// sums its row's 64 products from shared memory at the start of the item, and the rows are
// written out for the dK / dV kernel, which is launched after this one.
// TMEM columns: S [0, 128) dP [128, 256) dQ [256, 320) dS [320 + 64 b, +64) for buffer b.
constexpr int DQ_STAGES = 3;
constexpr int DQ_Q = 0, DQ_DO = FA_TILE_BYTES, DQ_O = 2 * FA_TILE_BYTES, DQ_K = 3 * FA_TILE_BYTES,
              DQ_V = (3 + DQ_STAGES) * FA_TILE_BYTES,
              DQ_OUT = (3 + 2 * DQ_STAGES) * FA_TILE_BYTES,    // output staging, one tile
              DQ_BAR = DQ_OUT + FA_TILE_BYTES, DQ_SMEM = DQ_BAR + 256 + 1024;
static_assert(DQ_SMEM <= 227 * 1024, "dQ kernel: shared memory");
constexpr int DQ_NBAR = 14 + 2 * DQ_STAGES, DQ_KV_FULL = 14, DQ_KV_EMPTY = 14 + DQ_STAGES;

// dS = P (dP - delta) scale for 32 keys of one query row, as fp16 pairs (keys 2i, 2i + 1) in
// pk[i], ready for tcgen05.st; P is rebuilt from the saved log-sum-exp as in bwd_chunk_regs.
template <bool MASK>
__device__ __forceinline__ void bwd_ds_pack(const uint32_t* rs, const uint32_t* rdp, int key0, int qi,
                                            int st, float cscale, float scale, float nlse, float dsc,
                                            uint32_t* pk) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    float dv[2];
#pragma unroll
    for (int w = 0; w < 2; ++w) {
      const int idx = 2 * i + w;
      float pr = vkg_ex2(fmaf(__uint_as_float(rs[idx]), cscale, nlse));
      if (MASK) {
        const int key = key0 + idx;
        if (key > qi || key < st) pr = 0.f;
      }
      dv[w] = pr * fmaf(__uint_as_float(rdp[idx]), scale, dsc);
    }
    const __half2 h = __floats2half2_rn(dv[0], dv[1]);
    pk[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
}

__global__ void __launch_bounds__(DQ_THREADS, 1)
attn_bwd_q_kernel(const __grid_constant__ CUtensorMap tm, const __grid_constant__ CUtensorMap tmdo,
                  const __grid_constant__ CUtensorMap tmo, const AttnParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar = base + DQ_BAR;
  // 0 qd_full, 1 od_free (delta formed from the dO / O tiles), 5 sdp_full, 6 sdp_free,
  // 7/10 ds_full[2], 8/11 ds_free[2], 9 out_full, 12 qd_free, 13 acc_free, 14.. kv_full[stage],
  // then kv_empty[stage]
  auto B_ = [bar](int i) { return bar + 8u * i; };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + DQ_BAR + 192);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(gbase + DQ_BAR + 200);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int HB = p.H * p.B;
  const int n_items = p.nqt * HB, G = (int)gridDim.x;
  constexpr int OUT_WARPS = DQ_SOFTMAX_WARPS < 8 ? DQ_SOFTMAX_WARPS : 8;   // warps that read dQ out

  pdl_trigger();
  if (threadIdx.x == 0) {
    prefetch_tensormap(&tm);
    prefetch_tensormap(&tmdo);
    prefetch_tensormap(&tmo);
    for (int i = 0; i < DQ_NBAR; ++i)
      mbar_init(B_(i), (i == 1 || i == 6 || i == 7 || i == 10) ? DQ_SOFTMAX_WARPS : (i == 13 ? OUT_WARPS : 1));
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  pdl_wait();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tdP = tmem + 128, tdQ = tmem + 256, tdS = tmem + 320;

  if (warp == 0) {
    if (lane == 0) {
      int g = 0, j = 0;
      bool ok = true;
      for (;; ++j) {
        const int item = snake_item(j, G, (int)blockIdx.x);
        if (item >= n_items || !ok) break;
        const int qt = p.nqt - 1 - item / HB, hb = item % HB;
        const int h = hb % p.H, b = hb / p.H;
        const int row0 = b * p.T, q0 = qt * FA_T, nj = qt + 1;
        // the previous item's Q / dO have been read by its last S / dP, its dO / O by every
        // softmax warp
        if (j > 0 && !(mbar_wait<true>(B_(12), (j - 1) & 1, abort_flag, p.err, 0x5900u) &&
                       mbar_wait<true>(B_(1), (j - 1) & 1, abort_flag, p.err, 0x5b00u)))
          break;
        mbar_expect_tx(B_(0), 3 * FA_TILE_BYTES);
        tma_load_2d(base + DQ_Q, &tm, B_(0), h * FA_HD, row0 + q0);
        tma_load_2d(base + DQ_DO, &tmdo, B_(0), h * FA_HD, row0 + q0);
        tma_load_2d(base + DQ_O, &tmo, B_(0), h * FA_HD, row0 + q0);
        for (int kt = 0; kt < nj; ++kt, ++g) {
          const int s = g % DQ_STAGES;
          const uint32_t ph = (uint32_t)(g / DQ_STAGES) & 1u;
          if (!mbar_wait<true>(B_(DQ_KV_EMPTY + s), ph ^ 1u, abort_flag, p.err, 0x5100u + s)) {
            ok = false;
            break;
          }
          mbar_expect_tx(B_(DQ_KV_FULL + s), 2 * FA_TILE_BYTES);
          tma_load_2d(base + DQ_K + s * FA_TILE_BYTES, &tm, B_(DQ_KV_FULL + s), p.D + h * FA_HD,
                      row0 + kt * FA_T);
          tma_load_2d(base + DQ_V + s * FA_TILE_BYTES, &tm, B_(DQ_KV_FULL + s), 2 * p.D + h * FA_HD,
                      row0 + kt * FA_T);
        }
      }
    }
  } else if (warp == 1) {
    // S = Q K^T and dP = dO V^T of every step.  The whole warp runs this converged; one elected
    // lane issues each tcgen05 instruction.
    const uint32_t idesc_s = make_idesc(0, 0, 0, FA_T);
    const uint32_t d_hi = smem_desc_hi(1024);      // descriptor halves (tcgen05.cuh)
    const uint32_t q_lo = smem_desc_lo(base + DQ_Q, 16), do_lo = smem_desc_lo(base + DQ_DO, 16);
    const uint32_t k_lo = smem_desc_lo(base + DQ_K, 16), v_lo = smem_desc_lo(base + DQ_V, 16);
    int s = 0;
    uint32_t ph = 0, par = 0;
    bool ok = true;
    for (int j = 0; ok; ++j) {
      const int item = snake_item(j, G, (int)blockIdx.x);
      if (item >= n_items) break;
      const int nj = p.nqt - item / HB;               // key tiles of the item: qt + 1
      ok = mbar_wait_warp<true>(B_(0), j & 1, abort_flag, p.err, 0x5200u);
      for (int kt = 0; kt < nj && ok; ++kt) {
        ok = mbar_wait_warp<true>(B_(DQ_KV_FULL + s), ph, abort_flag, p.err, 0x5300u + s) &&
             mbar_wait_warp<true>(B_(6), par ^ 1u, abort_flag, p.err, 0x5400u);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t so = (uint32_t)s * (FA_TILE_BYTES >> 4);
        umma_f16_chain<4>(tS, q_lo, 2, k_lo + so, 2, d_hi, idesc_s, 0u);
        umma_f16_chain<4>(tdP, do_lo, 2, v_lo + so, 2, d_hi, idesc_s, 0u);
        umma_commit_one(B_(5));
        if (kt == nj - 1) umma_commit_one(B_(12));    // the item's Q / dO may be replaced
        par ^= 1u;
        if (++s == DQ_STAGES) {
          s = 0;
          ph ^= 1u;
        }
      }
    }
  } else if (warp == DQ_MMA2_WARP) {
    // dQ += dS K of every step, issued by a warp of its own: the instruction stream of one warp
    // for both (waits, 16 instructions, commits, about 1900 cycles per step next to busy softmax
    // warps) was what paced the kernel.  Its commits cover this warp's instructions only; a
    // K / V stage is free when dQ of its step has retired, because the S / dP that read it
    // retired before the softmax warps could produce the dS this dQ waited for.
    const uint32_t idesc_q = make_idesc(0, 0, 1, FA_HD);   // dS (tensor memory) . K (MN-major), N = 64
    const uint32_t d_hi = smem_desc_hi(1024);
    const uint32_t km_lo = smem_desc_lo(base + DQ_K, 8192);
    int g = 0, s = 0;
    bool ok = true;
    for (int j = 0; ok; ++j) {
      const int item = snake_item(j, G, (int)blockIdx.x);
      if (item >= n_items) break;
      const int nj = p.nqt - item / HB;
      for (int kt = 0; kt < nj; ++kt, ++g) {
        const int pb = g & 1;
        ok = mbar_wait_warp<true>(B_(7 + 3 * pb), (g >> 1) & 1, abort_flag, p.err, 0x5500u);
        if (!ok) break;
        if (kt == 0 && j > 0) {
          ok = mbar_wait_warp<true>(B_(13), (j - 1) & 1, abort_flag, p.err, 0x5a00u);
          if (!ok) break;
        }
        tcgen05_fence_after();
        // K = 128 keys: dS from tensor memory (8 columns per step), K MN-major
        umma_f16_ts_chain<8>(tdQ, tdS + 64 * pb, km_lo + (uint32_t)s * (FA_TILE_BYTES >> 4), 128, d_hi, idesc_q,
                             kt ? 1u : 0u);
        umma_commit_one(B_(DQ_KV_EMPTY + s));   // K / V stage free
        umma_commit_one(B_(8 + 3 * pb));        // this dS area free
        if (kt == nj - 1) umma_commit_one(B_(9));
        if (++s == DQ_STAGES) s = 0;
      }
    }
  } else {
    constexpr int PARTS = DQ_SOFTMAX_WARPS / 4;  // warps per TMEM lane quarter
    constexpr int CPT = FA_T / PARTS;            // keys of a row per thread: 32 or 64
    const int part = (warp - 2) >> 2;            // which CPT of a key tile's 128 keys
    const int r = (warp & 3) * 32 + lane;
    const uint32_t t_lane = ((uint32_t)((warp & 3) * 32)) << 16;
    bool ok = true;
    // dQ of a finished item, read out after the NEXT item's first step (see the dK / dV kernel)
    // by the first OUT_WARPS warps, 64 / (OUT_WARPS / 4) columns each
    constexpr int OC = FA_HD / (OUT_WARPS / 4);
    int pend_item = -1, pend_j = 0;
    auto store_item = [&](int item, int jj) -> bool {
      const int qt = p.nqt - 1 - item / HB, hb = item % HB;
      const int h = hb % p.H, b = hb / p.H;
      const int row0 = b * p.T, qi = qt * FA_T + r;
      const bool q_ok = qi < p.T;
      if (!mbar_wait_warp<SM_SPIN>(B_(9), jj & 1, abort_flag, p.err, 0x5800u)) return false;
      tcgen05_fence_after();
      uint32_t rr[OC];
#pragma unroll
      for (int c = 0; c < OC / 16; ++c) tmem_ld16(tdQ + t_lane + part * OC + c * 16, rr + c * 16);
      tmem_wait_ld();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(B_(13));           // dQ may be overwritten
      {
        uint4 hv[OC / 8];
#pragma unroll
        for (int u = 0; u < OC / 8; ++u) {
          __half2 h2[4];
#pragma unroll
          for (int e = 0; e < 4; ++e)
            h2[e] = __floats2half2_rn(__uint_as_float(rr[u * 8 + 2 * e]),
                                      __uint_as_float(rr[u * 8 + 2 * e + 1]));
          hv[u] = *reinterpret_cast<uint4*>(h2);
        }
        const int q_w = qt * FA_T + (warp & 3) * 32;   // first query row of this warp's 32
        __half* dst = p.dqkv + (size_t)(row0 + q_w) * 3 * p.D + h * FA_HD + part * OC;
        warp_store_rows<OC / 8>(hv, gbase + DQ_OUT + (warp - 2) * (OC * 64), lane,
                                reinterpret_cast<uint8_t*>(dst), (size_t)3 * p.D * 2, p.T - q_w);
      }
      if (p.colsum) {
        float val[OC];
#pragma unroll
        for (int c = 0; c < OC; ++c)
          val[c] = q_ok ? __half2float(__float2half_rn(__uint_as_float(rr[c]))) : 0.f;
        float* dst = p.colsum + ((size_t)(b * p.nqt + qt) * 4 + (warp & 3)) * 3 * p.D + h * FA_HD +
                     part * OC;
        warp_col_sums<OC>(val, lane, dst);
      }
      return true;
    };
    // statistics of this thread's query row in an item
    auto item_stat = [&](int item, float& lse, int& st) {
      const int qt = p.nqt - 1 - item / HB, hb = item % HB;
      const int qi = qt * FA_T + r;
      const bool q_ok = qi < p.T;
      const size_t i = (size_t)((hb / p.H) * p.H + hb % p.H) * p.T + (q_ok ? qi : 0);
      lse = p.lse2[i];
      st = (p.seg && q_ok) ? (int)p.seg[(hb / p.H) * p.T + qi] : 0;
    };
    float lse_f = 0.f;
    int st_f = 0;
    if ((int)blockIdx.x < n_items) item_stat((int)blockIdx.x, lse_f, st_f);
    int g = 0, j = 0;
    for (;; ++j) {
      const int item = snake_item(j, G, (int)blockIdx.x);
      if (item >= n_items || !ok) break;
      const int qt = p.nqt - 1 - item / HB, nj = qt + 1;
      const int qi = qt * FA_T + r;
      const bool q_ok = qi < p.T;
      // this row's statistics were fetched while the previous item was being worked on
      const float nlse = q_ok ? -lse_f : -INFINITY;
      const int st = st_f;
      {
        const int nxt = snake_item(j + 1, G, (int)blockIdx.x);
        if (nxt < n_items) item_stat(nxt, lse_f, st_f);
      }
      // delta of this row from the item's dO and O tiles (128-byte rows, 16-byte pieces XOR-ed
      // with the row's low three bits, as the tensor map wrote them)
      ok = mbar_wait_warp<SM_SPIN>(B_(0), j & 1, abort_flag, p.err, 0x5c00u);
      if (!ok) break;
      float dl = 0.f;
      {
        const uint8_t* dor = gbase + DQ_DO + r * 128;
        const uint8_t* orow = gbase + DQ_O + r * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint32_t off = ((uint32_t)c ^ (uint32_t)(r & 7)) << 4;
          const uint4 a = *reinterpret_cast<const uint4*>(dor + off);
          const uint4 o = *reinterpret_cast<const uint4*>(orow + off);
          const __half2* ah = reinterpret_cast<const __half2*>(&a);
          const __half2* oh = reinterpret_cast<const __half2*>(&o);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 x = __half22float2(ah[e]), y = __half22float2(oh[e]);
            dl = fmaf(x.x, y.x, dl);
            dl = fmaf(x.y, y.y, dl);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(B_(1));             // this warp is done with the dO / O tiles
      if (part == 0 && q_ok) {
        const int hb = item % HB;
        p.delta_out[(size_t)((hb / p.H) * p.H + hb % p.H) * p.T + qi] = dl;
      }
      const float dsc = -dl * p.scale;
      for (int kt = 0; kt < nj && ok; ++kt, ++g) {
        const bool need_mask = (kt == qt) || (p.seg != nullptr);
        ok = mbar_wait_warp<SM_SPIN>(B_(5), g & 1, abort_flag, p.err, 0x5600u);
        if (!ok) break;
        tcgen05_fence_after();
        uint32_t rs[CPT], rdp[CPT];
#pragma unroll
        for (int c = 0; c < CPT / 16; ++c) tmem_ld16(tS + t_lane + part * CPT + c * 16, rs + c * 16);
#pragma unroll
        for (int c = 0; c < CPT / 16; ++c) tmem_ld16(tdP + t_lane + part * CPT + c * 16, rdp + c * 16);
        tmem_wait_ld();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(B_(6));
        // dS as fp16 pairs, overwriting the scores they came from
        const int key0 = kt * FA_T + part * CPT;
#pragma unroll
        for (int c = 0; c < CPT / 32; ++c) {
          if (need_mask)
            bwd_ds_pack<true>(rs + 32 * c, rdp + 32 * c, key0 + 32 * c, qi, st, p.cscale, p.scale, nlse, dsc,
                              rs + 16 * c);
          else
            bwd_ds_pack<false>(rs + 32 * c, rdp + 32 * c, 0, 0, 0, p.cscale, p.scale, nlse, dsc, rs + 16 * c);
        }
        const int pb = g & 1;
        // dQ of step g - 2 has read this dS area
        ok = mbar_wait_warp<SM_SPIN>(B_(8 + 3 * pb), ((g >> 1) & 1) ^ 1u, abort_flag, p.err, 0x5700u);
        if (!ok) break;
        tcgen05_fence_after();
#pragma unroll
        for (int c = 0; c < CPT / 32; ++c)
          tmem_st16(tdS + 64 * pb + t_lane + part * (CPT / 2) + c * 16, rs + 16 * c);
        tmem_wait_st();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(B_(7 + 3 * pb));
        if (pend_item >= 0) {
          if (warp - 2 < OUT_WARPS) ok = store_item(pend_item, pend_j);
          pend_item = -1;
        }
      }
      pend_item = item;       // read this item's dQ out after the next item's first step
      pend_j = j;
    }
    if (ok && pend_item >= 0 && warp - 2 < OUT_WARPS) ok = store_item(pend_item, pend_j);
  }
  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  if (*abort_flag) {
    long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) {
    }
  }
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// 2-D map over a row-major fp16 matrix (rows x cols), 64-column x 128-row boxes.
int make_map_2d(vkg_device* dev, CUtensorMap* map, const void* ptr, int64_t cols, int64_t rows,
                const char* what) {
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(cols * 2)};
  cuuint32_t box[2] = {FA_HD, FA_T};
  cuuint32_t estr[2] = {1, 1};
  if (((uintptr_t)ptr & 15) || ((cols * 2) & 15)) {
    vkg_set_error("attention operand %s must be 16-byte aligned with a 16-byte row pitch", what);
    return 1;
  }
  CUresult r = ((EncodeTiledFn)dev->encode_tiled)(
      map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    vkg_set_error("cuTensorMapEncodeTiled failed for %s with code %d", what, (int)r);
    return 1;
  }
  return 0;
}

}  // namespace

extern "C" int vkg_attn_fwd(vkg_device* dev, const void* qkv16, const uint32_t* seg, void* out16,
                            float* lse2, int B, int T, int H, int hd, float scale) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(qkv16 && out16 && lse2 && B > 0 && T > 0 && H > 0, "attn_fwd: bad arguments");
  VKG_REQUIRE(hd == FA_HD, "attn_fwd: head dimension must be %d (got %d)", FA_HD, hd);
  VKG_REQUIRE(((uintptr_t)out16 & 15) == 0, "attn_fwd: output must be 16-byte aligned");
  const int D = H * hd;
  CUtensorMap tm;
  if (make_map_2d(dev, &tm, qkv16, 3 * (int64_t)D, (int64_t)B * T, "qkv")) return 1;
  AttnParams p;
  memset(&p, 0, sizeof(p));
  p.B = B; p.T = T; p.H = H; p.D = D;
  p.nqt = (T + FA_T - 1) / FA_T;
  p.scale = scale;
  p.cscale = scale * LOG2E;
  p.seg = seg;
  p.out = (__half*)out16;
  p.lse2 = lse2;
  p.err = dev->err_dev;
  if (!dev->attn_fwd_attr_set) {
    VKG_CUDA(cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  FW_SMEM));
    VKG_CUDA(cudaFuncSetAttribute(attn_fwd1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  FW_SMEM));
    dev->attn_fwd_attr_set = true;
  }
  const long long ctas = (long long)p.nqt * H * B;
  VKG_REQUIRE(ctas < (1ll << 31), "attn_fwd: too many tiles");
  VKG_CUDA(vkg_launch(dev, VKG_K_ATTN_FWD, dev->attn_one_pass ? attn_fwd1_kernel : attn_fwd_kernel,
                      dim3((unsigned)ctas), dim3(FA_THREADS), FW_SMEM, 1, tm, p));
  return vkg_check_launch("attn_fwd_kernel");
}

extern "C" int vkg_attn_bwd(vkg_device* dev, const void* qkv16, const void* dout16, const void* out16,
                            const float* lse2, const uint32_t* seg, void* dqkv16, float* delta,
                            float* dbias, float* dbias_scratch, int B, int T, int H, int hd,
                            float scale) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(qkv16 && dout16 && out16 && lse2 && dqkv16 && delta && B > 0 && T > 0 && H > 0,
              "attn_bwd: bad arguments");
  VKG_REQUIRE(hd == FA_HD, "attn_bwd: head dimension must be %d (got %d)", FA_HD, hd);
  VKG_REQUIRE(((uintptr_t)dqkv16 & 15) == 0, "attn_bwd: dqkv must be 16-byte aligned");
  const int D = H * hd;
  CUtensorMap tm, tmdo, tmo;
  if (make_map_2d(dev, &tm, qkv16, 3 * (int64_t)D, (int64_t)B * T, "qkv")) return 1;
  if (make_map_2d(dev, &tmdo, dout16, (int64_t)D, (int64_t)B * T, "dO")) return 1;
  if (make_map_2d(dev, &tmo, out16, (int64_t)D, (int64_t)B * T, "O")) return 1;
  AttnParams p;
  memset(&p, 0, sizeof(p));
  p.B = B; p.T = T; p.H = H; p.D = D;
  p.nqt = (T + FA_T - 1) / FA_T;
  p.scale = scale;
  p.cscale = scale * LOG2E;
  p.seg = seg;
  p.lse2 = const_cast<float*>(lse2);
  p.delta = delta;
  p.delta_out = delta;
  p.dqkv = (__half*)dqkv16;
  p.err = dev->err_dev;
  VKG_REQUIRE(!dbias || dbias_scratch, "attn_bwd: dbias needs dbias_scratch");
  p.colsum = dbias ? dbias_scratch : nullptr;
  if (!dev->attn_bwd_attr_set) {
    VKG_CUDA(cudaFuncSetAttribute(attn_bwd_kv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  KV_SMEM));
    VKG_CUDA(cudaFuncSetAttribute(attn_bwd_q_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  DQ_SMEM));
    dev->attn_bwd_attr_set = true;
  }
  VKG_REQUIRE((((uintptr_t)dout16 | (uintptr_t)out16) & 15) == 0, "attn_bwd: dO and O must be 16-byte aligned");
  const long long n_items = (long long)p.nqt * H * B;
  VKG_REQUIRE(n_items < (1ll << 31), "attn_bwd: too many tiles");
  // persistent kernels: one CTA per SM (their shared memory allows no more), items dealt in
  // snake order; the dQ kernel goes first because it also writes delta
  const int sms = vkg_persistent_ctas(dev);
  const unsigned ctas = (unsigned)(n_items < sms ? n_items : sms);
  VKG_CUDA(vkg_launch(dev, VKG_K_ATTN_BWD, attn_bwd_q_kernel, dim3(ctas), dim3(DQ_THREADS), DQ_SMEM, 1, tm, tmdo, tmo, p));
  if (vkg_check_launch("attn_bwd_q_kernel")) return 1;
  VKG_CUDA(vkg_launch(dev, VKG_K_ATTN_BWD, attn_bwd_kv_kernel, dim3(ctas), dim3(BW_THREADS), KV_SMEM, 1, tm, tmdo, p));
  if (vkg_check_launch("attn_bwd_kv_kernel")) return 1;
  if (dbias)
    return vkg_launch_col_sum_final(dev, dbias_scratch, dbias, 3 * D, B * p.nqt * 4, 0);
  return 0;
}

extern "C" int64_t vkg_attn_bwd_dbias_scratch_floats(int B, int T, int H, int hd) {
  if (B <= 0 || T <= 0 || H <= 0 || hd <= 0) return 0;
  return (int64_t)B * ((T + FA_T - 1) / FA_T) * 4 * 3 * H * hd;
}
