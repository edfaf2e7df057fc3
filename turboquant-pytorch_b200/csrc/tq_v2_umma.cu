// Tensor-core (tcgen05 / TMEM / TMA) path for the MSE + QJL compress stage (K4), fp16 vectors,
// head_dim 128 or 256.  The reference's three chained D x D contractions
// (turboquant/compressors.py:83-120) run as three launches of one contraction kernel with a
// different epilogue each; operands that are fp32 in the reference are carried as fp16 pieces
// hi + lo (lo reaches into fp16 subnormals), so products match an fp32 matmul to ~2^-21:
//
//   stage 1  y = x Pi^T            A = x (exact fp16), B = Pi hi/lo.  Epilogue: ||y|| = ||x||, scale,
//                                  nearest centroid by exact thresholds, centroid pieces hi/lo -> scratch
//   stage 2  k = (c Pi) ||x||      A = centroid pieces, B = Pi^T hi/lo (hi.hi + lo.hi + hi.lo).  Epilogue:
//                                  k_mse (fp16 out), residual r = x - k, ||r|| (out), residual pieces -> scratch
//   stage 3  p = r S^T             A = residual pieces, B = S hi/lo.  Epilogue: signs (int8 out)
//
// A persistent CTA per SM walks 128-vector tiles.  warp 0: TMA loads of the tile's A chunks
// (128 rows x 64 columns, 128-byte swizzle, one slot per k-chunk and piece) and bulk copies of
// B chunks (128 output columns x 64 k, 16 KB, pre-swizzled image in global memory, L2-resident)
// through a ring; warp 1: tcgen05.mma M=128 N=128 K=16 into one 128-column accumulator per
// block of 128 output columns; the other warps: per tile in flight (two) one epilogue warpgroup
// per block of 128 columns, thread = vector.  Every mbarrier wait is bounded; on expiry the CTA raises an abort flag, records a
// status word and leaves through the normal exit.

#include <cuda.h>
#include <cuda_fp16.h>

#include <atomic>
#include <cstdlib>

#include "tq_common.cuh"
#include "tq_internal.h"

namespace tq {

namespace {

#include "tq_tc_ptx.cuh"

constexpr int kRowsT = 128;                    // vectors per tile (MMA M)
constexpr uint32_t kChunk = 128 * 128;         // 128 rows x 64 fp16 = 16 KB (an A chunk or a B chunk)
constexpr int kNB = 4;                         // B ring stages

template <int D>
struct VCfg {
  static constexpr int KC = D / 64;            // k chunks
  static constexpr int NBLK = D / 128;         // blocks of 128 output columns
  // A: two k-chunk slots per piece (chunk kc lands in slot kc & 1 and is released as soon as its MMAs are done), so
  // that the B ring can hold stages of ALL output columns: one MMA of N = D per k-step instead of one per block of
  // 128 columns (an MMA takes ~127 clocks whatever its N, so N = 256 halves the tensor time at head_dim 256)
  static constexpr int kASlots = 2;
  static constexpr uint32_t kBStage = NBLK * kChunk;                     // one k-chunk of B for all D output columns
  static constexpr uint32_t kOffA = 0;                                   // [piece 2][slot 2] chunks
  static constexpr uint32_t kOffB = kOffA + 2u * kASlots * kChunk;       // ring
  static constexpr uint32_t kOffTab = kOffB + kNB * kBStage;             // thresholds, centroid piece pairs, cell table, partial sums
  static constexpr uint32_t kOffBar = kOffTab + 6144;
  static constexpr int kThreads = 64 + 2 * NBLK * 128;                   // two tiles in flight, one warpgroup per 128 columns
  static constexpr uint32_t kUsedBytes = kOffBar + 256;
  static constexpr uint32_t kSmemBytes = kUsedBytes + 1024;
  static constexpr uint32_t kImageBytes = 2u * KC * NBLK * kChunk;       // [piece][kc][nb] chunks of one operand
  static constexpr int kTmemCols = 2 * NBLK * 128;                       // two tiles in flight
};
static_assert(VCfg<256>::kSmemBytes <= 232448 && VCfg<128>::kSmemBytes <= 232448, "shared memory budget");

struct V2Stage {
  CUtensorMap a_hi_map;      // fp16 (D, n), box 64 x 128, 128-byte swizzle
  CUtensorMap a_lo_map;      // second piece of A (stages 2 and 3)
  const uint8_t* b_image;    // [piece][kc][nb][128 rows x 128 bytes swizzled]
  const float* codebook;     // stage 1
  const uint16_t* x;         // stage 2: the original vectors (n, D) fp16
  uint16_t* p_hi;            // scratch (n, D): centroid pieces after stage 1, residual pieces after stage 2
  uint16_t* p_lo;
  float* norms;              // scratch (n): ||x||
  uint8_t* idx_u8_out;       // stage 1: optional, one index per byte (n, D)
  uint8_t* idx_packed_out;   // stage 1: optional, bit-packed rows (n, G), first index in the high bits
  uint8_t* sign_bits_out;    // stage 3: optional, one bit per sign (n, D / 8), coordinate j in bit 7 - j % 8, set for +1
  uint16_t* k_mse_out;       // stage 2: optional
  uint16_t* rnorm_out;       // stage 2, fp16 bits
  int8_t* signs_out;         // stage 3
  int32_t* status;
  int64_t n;
  int32_t tiles;
  int32_t bits;
};

__device__ int g_v2_status;    // 0 = ok; otherwise (stage << 20) | (code << 16) | block

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

// Operand image of a D x D matrix B (rows = output columns n, columns = contraction index k):
// value hi + lo in fp16, [piece][kc][nb][row n % 128][64 columns], rows of 128 bytes, 16-byte
// chunk c at c ^ (row & 7).  B[n][k] = src[n * ld_n + k * ld_k].
template <int D>
__global__ void k_v2_operand_image(const float* __restrict__ src, int64_t ld_n, int64_t ld_k, uint8_t* __restrict__ image) {
  constexpr int KC = VCfg<D>::KC, NBLK = VCfg<D>::NBLK;
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= D * D) return;
  const int n = e / D, k = e % D;
  const float v = src[(int64_t)n * ld_n + (int64_t)k * ld_k];
  const __half hi = __float2half_rn(v);
  const __half lo = __float2half_rn(v - __half2float(hi));
  const int kc = k / 64, nb = n / 128, rr = n % 128, c = (k % 64) / 8, w = k % 8;
  const size_t off = ((size_t)kc * NBLK + nb) * (kChunk / 2) + (size_t)rr * 64 + (size_t)((c ^ (rr & 7)) * 8 + w);
  uint16_t* img = reinterpret_cast<uint16_t*>(image);
  img[off] = __half_as_ushort(hi);
  img[(size_t)KC * NBLK * (kChunk / 2) + off] = __half_as_ushort(lo);
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  tmem_issue16(taddr, r);
  tmem_wait16(r);
}

template <int D, int STAGE>
__global__ void __launch_bounds__(VCfg<D>::kThreads, 1) k_umma_v2_stage(const __grid_constant__ V2Stage p) {
  using C = VCfg<D>;
  constexpr int KC = C::KC, NBLK = C::NBLK;
  constexpr int PA = STAGE == 1 ? 1 : 2;       // pieces of A
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
  {
    uint32_t dyn_bytes;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_bytes));
    if (base - smem_u32(smem_raw) + C::kUsedBytes > dyn_bytes) {     // the layout does not fit: report, do nothing
      if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, (STAGE << 20) | (9 << 16) | (int)blockIdx.x);
      return;
    }
  }
  const uint32_t a_smem = base + C::kOffA;
  const uint32_t b_smem = base + C::kOffB;
  float* thr_s = reinterpret_cast<float*>(gbase + C::kOffTab);
  uint32_t* lut_s = reinterpret_cast<uint32_t*>(gbase + C::kOffTab + 1024);
  uint8_t* cells_s = gbase + C::kOffTab + 2048;                        // 1028 bytes
  float* part_s = reinterpret_cast<float*>(gbase + C::kOffTab + 4096); // [slot 2][row 128] partial sums of the upper block
  const uint32_t bar0 = base + C::kOffBar;
  const uint32_t bar_afull = bar0;                          // [kASlots] TMA -> MMA (all pieces of a k-chunk)
  const uint32_t bar_aempty = bar_afull + 8 * 4;            // [kASlots] MMA commit -> producer
  const uint32_t bar_bfull = bar_aempty + 8 * 4;            // [kNB] bulk copy -> MMA
  const uint32_t bar_bempty = bar_bfull + 8 * kNB;          // [kNB] MMA commit -> producer
  const uint32_t bar_tfull = bar_bempty + 8 * kNB;          // [2] MMA commit -> epilogue
  const uint32_t bar_tempty = bar_tfull + 16;               // [2] epilogue (4 arrivals) -> MMA
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + C::kOffBar + 200);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + C::kOffBar + 208);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total = p.tiles;
  const int t0 = (int)((int64_t)total * blockIdx.x / gridDim.x);
  const int t1 = (int)((int64_t)total * (blockIdx.x + 1) / gridDim.x);
  const int n_local = t1 - t0;

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::kASlots; ++i) { mbar_init(bar_afull + 8 * i, 1); mbar_init(bar_aempty + 8 * i, 1); }
    for (int i = 0; i < kNB; ++i) { mbar_init(bar_bfull + 8 * i, 1); mbar_init(bar_bempty + 8 * i, 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(bar_tfull + 8 * i, 1); mbar_init(bar_tempty + 8 * i, 4 * NBLK); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if constexpr (STAGE == 1) {
    if (threadIdx.x >= 64 && threadIdx.x < 64 + 256) {
      const int e = threadIdx.x - 64;
      thr_s[e] = __ldg(p.codebook + kThresholdOff + e);
      const float c = __ldg(p.codebook + kCentroidOff + e);
      const __half h = __float2half_rn(c);
      const __half l = __float2half_rn(c - __half2float(h));
      lut_s[e] = (uint32_t)__half_as_ushort(h) | ((uint32_t)__half_as_ushort(l) << 16);
      for (int w = e; w < 257; w += 256) reinterpret_cast<uint32_t*>(cells_s)[w] = __float_as_uint(__ldg(p.codebook + 528 + w));
    }
  }
  if (warp == 1) tmem_alloc(smem_u32((const void*)tmem_slot), C::kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      bool ok = true;
      int bc = 0;                                           // running B chunk counter
      int ac = 0;                                           // running A chunk counter: slot ac & 1, use ac / 2
      for (int i = 0; i < n_local && ok; ++i) {
        const int row0 = (t0 + i) * kRowsT;
        for (int kc = 0; kc < KC && ok; ++kc, ++ac) {
          const int as = ac % C::kASlots;
          ok = mbar_wait(bar_aempty + 8 * as, (uint32_t)(((ac / C::kASlots) & 1) ^ 1), abort_flag);
          if (!ok) break;
          mbar_arrive_expect_tx(bar_afull + 8 * as, PA * kChunk);
          tma_load_2d(a_smem + as * kChunk, &p.a_hi_map, kc * 64, row0, bar_afull + 8 * as);
          if constexpr (PA == 2) tma_load_2d(a_smem + (C::kASlots + as) * kChunk, &p.a_lo_map, kc * 64, row0, bar_afull + 8 * as);
          for (int pb = 0; pb < 2; ++pb) {
            const int s = bc % kNB;
            ok = mbar_wait(bar_bempty + 8 * s, (uint32_t)(((bc / kNB) & 1) ^ 1), abort_flag);
            if (!ok) break;
            mbar_arrive_expect_tx(bar_bfull + 8 * s, C::kBStage);
            bulk_load(b_smem + s * C::kBStage, p.b_image + (size_t)(pb * KC + kc) * C::kBStage, C::kBStage, bar_bfull + 8 * s);
            ++bc;
          }
        }
      }
      if (!ok) {
        *abort_flag = 1;
        if (p.status != nullptr) atomicCAS(p.status, 0, (STAGE << 20) | (1 << 16) | (int)blockIdx.x);
      }
      // none of this CTA's own copies may still be in flight when it exits
      for (int k = 0; k < C::kASlots && k < ac; ++k) {
        const int j = ac - 1 - k;
        mbar_wait(bar_afull + 8 * (j % C::kASlots), (uint32_t)((j / C::kASlots) & 1), abort_flag);
      }
      for (int k = 0; k < kNB && k < bc; ++k) {
        const int j = bc - 1 - k;
        mbar_wait(bar_bfull + 8 * (j % kNB), (uint32_t)((j / kNB) & 1), abort_flag);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (converged warp, one elected lane issues)
    bool ok = true;
    int bc = 0;
    // M = 128, N = D (all output columns in one instruction: rows 128.. of the B stage are the second block), fp16
    const uint32_t idesc = (idesc_f16(false) & ~(0x3Fu << 17)) | ((uint32_t)(D >> 3) << 17);
    int ac = 0;
    for (int i = 0; i < n_local && ok; ++i) {
      const int slot = i & 1;
      ok = mbar_wait(bar_tempty + 8 * slot, (uint32_t)(((i >> 1) & 1) ^ 1), abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
#pragma unroll 1
      for (int kc = 0; kc < KC && ok; ++kc, ++ac) {
        const int as = ac % C::kASlots;
        ok = mbar_wait(bar_afull + 8 * as, (uint32_t)((ac / C::kASlots) & 1), abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const uint64_t a_hi = smem_desc_sw128(a_smem + as * kChunk);
        const uint64_t a_lo = smem_desc_sw128(a_smem + (C::kASlots + as) * kChunk);
        {
          const uint32_t d_tmem = tmem_base + (uint32_t)(slot * NBLK * 128);
#pragma unroll 1
          for (int pb = 0; pb < 2; ++pb) {
            const int s = bc % kNB;
            ok = mbar_wait(bar_bfull + 8 * s, (uint32_t)((bc / kNB) & 1), abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint64_t b_desc = smem_desc_sw128(b_smem + s * C::kBStage);
            if (elect_one()) {
              if (pb == 0) {
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_f16(d_tmem, a_hi + (uint64_t)(k * 2), b_desc + (uint64_t)(k * 2), idesc, (kc | k) != 0 ? 1u : 0u);
                if constexpr (PA == 2) {
#pragma unroll
                  for (int k = 0; k < 4; ++k) umma_f16(d_tmem, a_lo + (uint64_t)(k * 2), b_desc + (uint64_t)(k * 2), idesc, 1u);
                }
              } else {
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_f16(d_tmem, a_hi + (uint64_t)(k * 2), b_desc + (uint64_t)(k * 2), idesc, 1u);
              }
              umma_commit(bar_bempty + 8 * s);              // the ring stage is free once these MMAs are done
              if (pb == 1) {
                umma_commit(bar_aempty + 8 * as);           // last use of this k-chunk of A
                if (kc == KC - 1) umma_commit(bar_tfull + 8 * slot);
              }
            }
            __syncwarp();
            ++bc;
          }
        }
      }
    }
    if (!ok && lane == 0) {
      *abort_flag = 1;
      if (p.status != nullptr) atomicCAS(p.status, 0, (STAGE << 20) | (2 << 16) | (int)blockIdx.x);
    }
  } else {
    // ------------------------------------------------------------ epilogue: per tile in flight one warpgroup per block
    // of 128 output columns, thread = vector
    const int ew = warp - 2;
    const int wgi = ew >> 2;
    const int slot = wgi / NBLK, blk = wgi % NBLK;
    const int quarter = warp & 3;                 // TMEM lanes this warp may touch: 32*quarter ..
    const int rloc = quarter * 32 + lane;
    bool ok = true;
    // search shortcut of the codebook (stage 1): 1 = polynomial, 2 = cell table, 0 = binary search
    int mode = 0;
    float sc_s = 0.f, sc_c1 = 0.f, sc_c2 = 0.f, sc_c3 = 0.f;
    if constexpr (STAGE == 1) {
      mode = (int)__ldg(p.codebook + 512);
      sc_s = __ldg(p.codebook + 513);
      sc_c1 = __ldg(p.codebook + 514);
      sc_c2 = __ldg(p.codebook + 515);
      sc_c3 = __ldg(p.codebook + 516);
    }
    for (int i = slot; i < n_local && ok; i += 2) {
      const int64_t row = (int64_t)(t0 + i) * kRowsT + rloc;
      const bool valid = row < p.n;
      // The exit decision is made uniform before anything collective: per warp (the TMEM loads are
      // warp-collective) and, where the two warpgroups of a tile later meet at a named barrier (stage 2,
      // head_dim 256), over those 256 threads, so that nobody waits at that barrier for a warp that left.
      ok = __all_sync(0xffffffffu, mbar_wait(bar_tfull + 8 * slot, (uint32_t)((i >> 1) & 1), abort_flag));
      if constexpr (STAGE == 2 && NBLK == 2) ok = bar_red_and(3 + slot, 256, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t tile_acc = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(slot * NBLK * 128);
      const uint32_t tacc = tile_acc + (uint32_t)(blk * 128);     // this warpgroup's block of columns
      const int col0 = blk * 128;
      uint32_t v[16];
      if constexpr (STAGE == 1) {
        float ssq = 0.f;                         // the norm needs every column: both warpgroups sweep the whole row
#pragma unroll 1
        for (int c = 0; c < D / 16; ++c) {
          tmem_ld16(tile_acc + c * 16, v);
#pragma unroll
          for (int e = 0; e < 16; ++e) ssq = fmaf(__uint_as_float(v[e]), __uint_as_float(v[e]), ssq);
        }
        const float norm = __fsqrt_rn(ssq);
        const float inv = __fdiv_rn(1.0f, norm + 1e-8f);
        if (valid && blk == 0) p.norms[row] = norm;
        const int bits = p.bits;
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          tmem_ld16(tacc + c * 16, v);
          uint32_t w[16];
          uint32_t ib[4] = {0u, 0u, 0u, 0u};
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const float y = __uint_as_float(v[e]) * inv;
            int idx;
            if (mode != 0) {
              // candidate e0 with index in {e0, e0 + 1} (verified on the host for every y), then one exact compare
              float t;
              asm("fma.rn.sat.f32 %0, %1, %2, 0f3F000000;" : "=f"(t) : "f"(y), "f"(sc_s));
              int e0;
              if (mode == 1) {
                float q = fmaf(sc_c3, t, sc_c2);
                q = fmaf(q, t, sc_c1);
                e0 = __float_as_int(fmaf(q, t, 8388608.0f)) & 0xFF;
              } else {
                e0 = cells_s[__float_as_int(fmaf(t, 1024.0f, 8388608.0f)) & 0x7FF];
              }
              idx = e0 + (y > thr_s[e0] ? 1 : 0);
            } else {
              int lo = 0, hi = (1 << bits) - 1;
              for (int step = 0; step < bits; ++step) {
                const int mid = (lo + hi) >> 1;
                if (y > thr_s[mid]) lo = mid + 1; else hi = mid;
              }
              idx = lo;
            }
            w[e] = lut_s[idx];
            ib[e >> 2] |= (uint32_t)idx << (8 * (e & 3));
          }
          if (valid && p.idx_u8_out != nullptr)
            *reinterpret_cast<uint4*>(p.idx_u8_out + row * D + col0 + c * 16) = make_uint4(ib[0], ib[1], ib[2], ib[3]);
          if (valid && p.idx_packed_out != nullptr) {
            // the 16 indices of this step as 16 / ipb packed bytes of the row
            const int ipb = 8 / bits;
            uint8_t* dst = p.idx_packed_out + row * (int64_t)(D / ipb) + (col0 + c * 16) / ipb;
            if (ipb == 1) {
              *reinterpret_cast<uint4*>(dst) = make_uint4(ib[0], ib[1], ib[2], ib[3]);
            } else if (ipb == 2) {           // 3- and 4-bit codes: byte k = idx[2k] << bits | idx[2k+1]
              uint32_t o[2];
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const uint32_t a = ib[2 * h], b = ib[2 * h + 1];
                const uint32_t b0 = (((a >> 0) & 0xFFu) << bits) | ((a >> 8) & 0xFFu), b1 = (((a >> 16) & 0xFFu) << bits) | (a >> 24);
                const uint32_t b2 = (((b >> 0) & 0xFFu) << bits) | ((b >> 8) & 0xFFu), b3 = (((b >> 16) & 0xFFu) << bits) | (b >> 24);
                o[h] = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
              }
              *reinterpret_cast<uint2*>(dst) = make_uint2(o[0], o[1]);
            } else if (ipb == 4) {           // 2-bit codes
              uint32_t o = 0u;
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const uint32_t a = ib[k];
                o |= ((((a >> 0) & 3u) << 6) | (((a >> 8) & 3u) << 4) | (((a >> 16) & 3u) << 2) | ((a >> 24) & 3u)) << (8 * k);
              }
              *reinterpret_cast<uint32_t*>(dst) = o;
            } else {                          // 1-bit codes
              uint32_t o = 0u;
#pragma unroll
              for (int e = 0; e < 16; ++e) o |= ((ib[e >> 2] >> (8 * (e & 3))) & 1u) << (8 * (e >> 3) + 7 - (e & 7));
              *reinterpret_cast<uint16_t*>(dst) = (uint16_t)o;
            }
          }
          if (valid) {
            uint32_t ph[8], pl[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              ph[j] = __byte_perm(w[2 * j], w[2 * j + 1], 0x5410);
              pl[j] = __byte_perm(w[2 * j], w[2 * j + 1], 0x7632);
            }
            uint4* dh = reinterpret_cast<uint4*>(p.p_hi + row * D + col0 + c * 16);
            uint4* dl = reinterpret_cast<uint4*>(p.p_lo + row * D + col0 + c * 16);
            dh[0] = make_uint4(ph[0], ph[1], ph[2], ph[3]); dh[1] = make_uint4(ph[4], ph[5], ph[6], ph[7]);
            dl[0] = make_uint4(pl[0], pl[1], pl[2], pl[3]); dl[1] = make_uint4(pl[4], pl[5], pl[6], pl[7]);
          }
        }
      } else if constexpr (STAGE == 2) {
        const float nv = valid ? p.norms[row] : 0.f;
        float ssq = 0.f;
        // the vector's own 16-coordinate pieces are fetched one step ahead of their use
        const uint4* xrow = reinterpret_cast<const uint4*>(p.x + (valid ? row : 0) * D + col0);
        uint4 nx0 = __ldg(xrow), nx1 = __ldg(xrow + 1);
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          const uint4 x0 = nx0, x1 = nx1;
          if (c + 1 < 8) { nx0 = __ldg(xrow + 2 * (c + 1)); nx1 = __ldg(xrow + 2 * (c + 1) + 1); }
          tmem_ld16(tacc + c * 16, v);
          if (valid) {
            const uint32_t xw[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
            uint32_t kq[8], rh[8], rl[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float k0 = __uint_as_float(v[2 * j]) * nv, k1 = __uint_as_float(v[2 * j + 1]) * nv;
              const __half2 xh = *reinterpret_cast<const __half2*>(&xw[j]);
              const float r0 = __low2float(xh) - k0, r1 = __high2float(xh) - k1;
              ssq = fmaf(r0, r0, ssq);
              ssq = fmaf(r1, r1, ssq);
              const __half2 kh = __floats2half2_rn(k0, k1);
              kq[j] = *reinterpret_cast<const uint32_t*>(&kh);
              const __half2 hh = __floats2half2_rn(r0, r1);
              rh[j] = *reinterpret_cast<const uint32_t*>(&hh);
              const __half2 ll = __floats2half2_rn(r0 - __low2float(hh), r1 - __high2float(hh));
              rl[j] = *reinterpret_cast<const uint32_t*>(&ll);
            }
            uint4* dh = reinterpret_cast<uint4*>(p.p_hi + row * D + col0 + c * 16);
            uint4* dl = reinterpret_cast<uint4*>(p.p_lo + row * D + col0 + c * 16);
            if (p.k_mse_out != nullptr) {
              uint4* dk = reinterpret_cast<uint4*>(p.k_mse_out + row * D + col0 + c * 16);
              dk[0] = make_uint4(kq[0], kq[1], kq[2], kq[3]); dk[1] = make_uint4(kq[4], kq[5], kq[6], kq[7]);
            }
            dh[0] = make_uint4(rh[0], rh[1], rh[2], rh[3]); dh[1] = make_uint4(rh[4], rh[5], rh[6], rh[7]);
            dl[0] = make_uint4(rl[0], rl[1], rl[2], rl[3]); dl[1] = make_uint4(rl[4], rl[5], rl[6], rl[7]);
          }
        }
        if constexpr (NBLK == 2) {
          // the residual norm spans both blocks: the upper block's warpgroup hands its partial sum over
          if (blk == 1) part_s[slot * 128 + rloc] = ssq;
          asm volatile("bar.sync %0, 256;" ::"r"(1 + slot) : "memory");
          if (blk == 0) ssq += part_s[slot * 128 + rloc];
          asm volatile("bar.sync %0, 256;" ::"r"(1 + slot) : "memory");     // part_s is reused by the next tile
        }
        if (valid && blk == 0) p.rnorm_out[row] = __half_as_ushort(__float2half_rn(__fsqrt_rn(ssq)));
      } else {
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          tmem_ld16(tacc + c * 16, v);
          if (valid && p.signs_out != nullptr) {
            uint32_t sw[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint32_t x = 0u;
#pragma unroll
              for (int b = 0; b < 4; ++b) {
                const uint32_t s8 = __uint_as_float(v[4 * j + b]) >= 0.f ? 0x01u : 0xFFu;
                x |= s8 << (8 * b);
              }
              sw[j] = x;
            }
            *reinterpret_cast<uint4*>(p.signs_out + row * D + col0 + c * 16) = make_uint4(sw[0], sw[1], sw[2], sw[3]);
          }
          if (valid && p.sign_bits_out != nullptr) {
            uint32_t o = 0u;
#pragma unroll
            for (int e = 0; e < 16; ++e) o |= (__uint_as_float(v[e]) >= 0.f ? 1u : 0u) << (8 * (e >> 3) + 7 - (e & 7));
            *reinterpret_cast<uint16_t*>(p.sign_bits_out + row * (D / 8) + (col0 + c * 16) / 8) = (uint16_t)o;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + 8 * slot);
    }
    if (!ok && lane == 0) {
      *abort_flag = 1;
      if (p.status != nullptr) atomicCAS(p.status, 0, (STAGE << 20) | (3 << 16) | (int)blockIdx.x);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

int encode_rows(TensorMapEncodeFn enc, CUtensorMap* map, const void* ptr, int64_t n, int D) {
  cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)n};
  cuuint64_t strides[1] = {(cuuint64_t)D * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)kRowsT};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { note_cuda_error(100000 + (int)r); return TQ_ELAUNCH; }
  return TQ_OK;
}

template <int D, int STAGE>
int launch_stage(const V2Stage& p, int grid, cudaStream_t st) {
  cudaError_t e = cudaFuncSetAttribute(k_umma_v2_stage<D, STAGE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)VCfg<D>::kSmemBytes);
  if (e != cudaSuccess) { note_cuda_error((int)e); return TQ_ELAUNCH; }
  k_umma_v2_stage<D, STAGE><<<grid, VCfg<D>::kThreads, VCfg<D>::kSmemBytes, st>>>(p);
  return check_launch();
}

template <int D>
int run(const TqQjlCompressJob& job, cudaStream_t st) {
  TensorMapEncodeFn enc = tensor_map_encoder();
  if (enc == nullptr) return TQ_ELAUNCH;
  const int64_t n = job.B * job.H * job.S;
  const int64_t tiles = (n + kRowsT - 1) / kRowsT;
  if (tiles >= ((int64_t)1 << 30)) return TQ_ETOOBIG;
  // workspace: three operand images, then the two piece arrays, then the norms
  uint8_t* ws = reinterpret_cast<uint8_t*>(((uintptr_t)job.workspace + 1023u) & ~(uintptr_t)1023u);
  const size_t img = VCfg<D>::kImageBytes;
  uint8_t* img1 = ws;
  uint8_t* img2 = ws + img;
  uint8_t* img3 = ws + 2 * img;
  const size_t piece = ((size_t)n * D * 2 + 1023) / 1024 * 1024;
  uint16_t* p_hi = reinterpret_cast<uint16_t*>(ws + 3 * img);
  uint16_t* p_lo = reinterpret_cast<uint16_t*>(ws + 3 * img + piece);
  float* norms = reinterpret_cast<float*>(ws + 3 * img + 2 * piece);
  const int ib = (D * D + 255) / 256;
  k_v2_operand_image<D><<<ib, 256, 0, st>>>(job.rotation, D, 1, img1);      // B[n][k] = Pi[n][k]
  k_v2_operand_image<D><<<ib, 256, 0, st>>>(job.rotation, 1, D, img2);      // B[j][n] = Pi[n][j]
  k_v2_operand_image<D><<<ib, 256, 0, st>>>(job.qjl_t, 1, job.M, img3);     // B[m][j] = S[m][j] = qjl_t[j][m]
  int rc = check_launch();
  if (rc != TQ_OK) return rc;
  static thread_local V2Stage p;
  void* status_ptr = nullptr;
  cudaGetSymbolAddress(&status_ptr, g_v2_status);
  p.status = reinterpret_cast<int32_t*>(status_ptr);
  p.codebook = job.codebook;
  p.x = reinterpret_cast<const uint16_t*>(job.x);
  p.p_hi = p_hi;
  p.p_lo = p_lo;
  p.norms = job.vec_norms_out != nullptr ? job.vec_norms_out : norms;
  p.idx_u8_out = job.idx_mode == TQ_IDX_PACKED ? nullptr : reinterpret_cast<uint8_t*>(job.idx_out);
  p.idx_packed_out = job.idx_mode == TQ_IDX_PACKED ? reinterpret_cast<uint8_t*>(job.idx_out) : nullptr;
  p.k_mse_out = job.k_mse_out;
  p.rnorm_out = reinterpret_cast<uint16_t*>(job.rnorm_out);
  p.signs_out = job.signs_dtype == 2 ? nullptr : reinterpret_cast<int8_t*>(job.signs_out);
  p.sign_bits_out = job.signs_dtype == 2 ? reinterpret_cast<uint8_t*>(job.signs_out) : nullptr;
  p.n = n;
  p.tiles = (int32_t)tiles;
  p.bits = job.bits;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = (int)(tiles < sms ? tiles : sms);
  // stage 1: A = x
  if ((rc = encode_rows(enc, &p.a_hi_map, job.x, n, D)) != TQ_OK) return rc;
  p.a_lo_map = p.a_hi_map;
  p.b_image = img1;
  if ((rc = launch_stage<D, 1>(p, grid, st)) != TQ_OK) return rc;
  // stages 2 and 3: A = the piece arrays
  if ((rc = encode_rows(enc, &p.a_hi_map, p_hi, n, D)) != TQ_OK) return rc;
  if ((rc = encode_rows(enc, &p.a_lo_map, p_lo, n, D)) != TQ_OK) return rc;
  p.b_image = img2;
  if ((rc = launch_stage<D, 2>(p, grid, st)) != TQ_OK) return rc;
  p.b_image = img3;
  return launch_stage<D, 3>(p, grid, st);
}

}  // namespace

size_t umma_v2_compress_workspace(int64_t n, int D) {
  if (D != 128 && D != 256) return 0;
  const size_t img = D == 256 ? VCfg<256>::kImageBytes : VCfg<128>::kImageBytes;
  const size_t piece = ((size_t)n * D * 2 + 1023) / 1024 * 1024;
  return 1024 + 3 * img + 2 * piece + (size_t)n * sizeof(float) + 1024;
}

bool umma_v2_compress_eligible(const TqQjlCompressJob& job) {
  if (force_simt()) return false;
  if (job.D != 128 && job.D != 256) return false;
  if (job.x_dtype != TQ_F16 || job.normalize != 1 || (job.signs_dtype != 0 && job.signs_dtype != 2) || job.rnorm_dtype != TQ_F16)
    return false;
  if (job.M != job.D || (job.idx_out != nullptr && job.idx_mode != TQ_IDX_U8 && job.idx_mode != TQ_IDX_PACKED)) return false;
  if (job.bits < 1 || job.bits > 8) return false;
  const int64_t n = job.B * job.H * job.S;
  if (n <= 0) return false;
  // rows must be contiguous: (B, H, S, D) without gaps
  if (job.S > 1 && job.stride_s != job.D) return false;
  if (job.H > 1 && job.stride_h != job.S * job.D) return false;
  if (job.B > 1 && job.stride_b != job.H * job.S * job.D) return false;
  if (((uintptr_t)job.x & 15u) || ((uintptr_t)job.k_mse_out & 15u) || ((uintptr_t)job.signs_out & 15u) ||
      ((uintptr_t)job.idx_out & 15u))
    return false;
  if (job.workspace == nullptr || job.workspace_bytes < umma_v2_compress_workspace(n, job.D)) return false;
  return true;
}

int umma_v2_compress(const TqQjlCompressJob& job, cudaStream_t st) {
  return job.D == 256 ? run<256>(job, st) : run<128>(job, st);
}

int umma_v2_device_status() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_v2_status, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

}  // namespace tq
