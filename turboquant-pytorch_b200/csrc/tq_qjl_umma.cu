// Tensor-core (tcgen05 / TMEM / TMA) kernel for the asymmetric scores of the MSE+QJL
// representation (K5), head_dim 128 or 256:
//
//   scores[q][key] = <Q_q, k_mse_key> + sqrt(pi/2)/D * ||r_key|| * <S Q_q, signs_key>
//
// is ONE contraction of length 2D when the key side is written as the row
// [k_mse_key | signs_key * ||r_key||] (both halves exact in fp16: k_mse and ||r|| are stored
// as fp16, signs are +-1) and the query side as [Q_q | sqrt(pi/2)/D * S Q_q], split into
// fp16 pieces hi + lo (lo reaches into fp16 subnormals, so both passes accumulate into one
// fp32 TMEM accumulator and the products match an fp32 matmul to ~1e-7).
//
// A persistent, warp-specialised CTA per SM walks 128-key tiles of one (batch*head, block of
// up to 64 queries) unit after the other:
//   warp 0       producer: TMA loads of k_mse chunks (128 keys x 64 coordinates, 128-byte
//                swizzle: already the operand layout) and of raw sign chunks (128 x 64 bytes);
//                the unit's query image (all chunks, hi and lo) by bulk copy on unit change
//   warps 2..9   expanders: signs -> fp16 +-||r|| written in the swizzled operand layout
//   warp 1       issues tcgen05.mma kind::f16, M=128 N=64 K=16: 2 pieces x 4 k-steps per chunk
//   warps 10..13 drain: TMEM -> 128-byte rows of scores[q][key0 .. key0+31]
// Every mbarrier wait is bounded; on expiry the CTA raises an abort flag, records a status
// word and leaves through the normal exit.

#include <cuda.h>

#include <atomic>
#include <cstdlib>

#include "tq_common.cuh"
#include "tq_internal.h"

namespace tq {

namespace {

#include "tq_tc_ptx.cuh"

constexpr int kKeys = 128;                     // keys per tile (MMA M)
constexpr int kQ = 64;                         // queries per unit (MMA N)
constexpr uint32_t kChunkA = kKeys * 128;      // one operand chunk: 128 rows x 64 fp16 = 16 KB
constexpr uint32_t kChunkRaw = kKeys * 64;     // raw signs of a chunk: 128 rows x 64 int8 = 8 KB
constexpr uint32_t kChunkB = kQ * 128;         // one query chunk: 64 rows x 64 fp16 = 8 KB
constexpr int kNSK = 3, kNSG = 2, kNSR = 2, kNT = 4;
constexpr int kExpWarps = 8, kDrainWarps = 4;
constexpr int kThreadsQ = 64 + 32 * (kExpWarps + kDrainWarps);   // 448

template <int D>
struct QCfg {
  static constexpr int kHalfChunks = D / 64;                     // chunks per operand half (k_mse | signs)
  static constexpr int kChunks = 2 * kHalfChunks;                // contraction length 2D in chunks of 64
  static constexpr uint32_t kImageBytes = 2u * kChunks * kChunkB;   // hi pieces then lo pieces
  static constexpr uint32_t kOffImg = 0;
  static constexpr uint32_t kOffK = kOffImg + kImageBytes;
  static constexpr uint32_t kOffG = kOffK + kNSK * kChunkA;
  static constexpr uint32_t kOffR = kOffG + kNSG * kChunkA;
  static constexpr uint32_t kOffBar = kOffR + kNSR * kChunkRaw;
  static constexpr uint32_t kUsedBytes = kOffBar + 256;
  static constexpr uint32_t kSmemBytes = kUsedBytes + 1024;      // + slack for aligning the base to 1024 bytes
};
static_assert(QCfg<256>::kSmemBytes <= 232448 && QCfg<128>::kSmemBytes <= 232448, "shared memory budget");

struct QjlBatch {
  CUtensorMap kmse_map;      // fp16 (D, Sk, BH), box 64 x 128, 128-byte swizzle
  CUtensorMap sign_map;      // uint8 (D, Sk, BH), box 64 x 128, no swizzle
  const uint16_t* rnorm;     // fp16 bits (BH, Sk)
  const uint8_t* images;     // [unit][hi | lo][chunk][64 rows x 128 bytes swizzled]
  float* scores;             // (BH, Sq, Sk)
  int32_t* status;
  int64_t Sq, Sk;
  int32_t n_qblocks;         // ceil(Sq / 64)
  int32_t tiles_per_unit;    // ceil(Sk / 128)
  int32_t total_tiles;
  int32_t pad_;
};

__device__ int g_qjl_status;   // 0 = ok; otherwise (code << 16) | block

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__device__ __forceinline__ uint32_t idesc_f16_n(uint32_t n) {
  // D = fp32, A and B fp16, both K-major, M = 128
  return (1u << 4) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

// Query image of one unit: row n = query q0 + n of head bh (zero past Sq), contraction index
// j < D -> Q[n][j], j >= D -> corr * (S Q)[n][j - D]; value = hi + lo in fp16.  Stored as
// [piece][chunk][row n][64 columns], rows of 128 bytes, 16-byte chunk c at c ^ (n & 7).
constexpr int kImageSplit = 16;               // blocks per unit in the image kernel
template <int D>
__global__ void k_qjl_query_image(const float* __restrict__ qf, const float* __restrict__ qproj, float corr, int64_t Sq,
                                  int n_qblocks, uint8_t* __restrict__ images) {
  constexpr int kChunks = QCfg<D>::kChunks;
  const int unit = blockIdx.x / kImageSplit, part = blockIdx.x % kImageSplit;
  const int64_t bh = unit / n_qblocks;
  const int q0 = (unit % n_qblocks) * kQ;
  uint16_t* img = reinterpret_cast<uint16_t*>(images + (size_t)unit * QCfg<D>::kImageBytes);
  constexpr int kPer = kQ * 2 * D / kImageSplit;
  for (int e = part * kPer + threadIdx.x; e < (part + 1) * kPer; e += blockDim.x) {
    const int n = e / (2 * D), j = e % (2 * D);
    float v = 0.f;
    if (q0 + n < Sq) {
      const int64_t row = bh * Sq + q0 + n;
      v = j < D ? qf[row * D + j] : corr * qproj[row * D + (j - D)];
    }
    const __half hi = __float2half_rn(v);
    const __half lo = __float2half_rn(v - __half2float(hi));
    const int chunk = j / 64, c = (j % 64) / 8, w = j % 8;
    const size_t off = (size_t)chunk * (kChunkB / 2) + (size_t)n * 64 + (size_t)((c ^ (n & 7)) * 8 + w);
    img[off] = __half_as_ushort(hi);
    img[(size_t)kChunks * (kChunkB / 2) + off] = __half_as_ushort(lo);
  }
}

template <int D>
__global__ void __launch_bounds__(kThreadsQ, 1) k_umma_qjl_scores(const __grid_constant__ QjlBatch batch) {
  using C = QCfg<D>;
  constexpr int kHalfChunks = C::kHalfChunks, kChunks = C::kChunks;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
  {
    uint32_t dyn_bytes;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_bytes));
    if (base - smem_u32(smem_raw) + C::kUsedBytes > dyn_bytes) {     // the layout does not fit: report, do nothing
      if (threadIdx.x == 0 && batch.status != nullptr) atomicCAS(batch.status, 0, (9 << 16) | (int)blockIdx.x);
      return;
    }
  }
  const uint32_t img_smem = base + C::kOffImg;
  const uint32_t k_smem = base + C::kOffK;
  const uint32_t g_smem = base + C::kOffG;
  const uint32_t r_smem = base + C::kOffR;
  const uint32_t bar0 = base + C::kOffBar;
  const uint32_t bar_kfull = bar0;                         // [kNSK] TMA -> MMA
  const uint32_t bar_kempty = bar_kfull + 8 * kNSK;        // [kNSK] MMA commit -> producer
  const uint32_t bar_rfull = bar_kempty + 8 * kNSK;        // [kNSR] TMA -> expanders
  const uint32_t bar_rempty = bar_rfull + 8 * kNSR;        // [kNSR] expanders (256 arrivals) -> producer
  const uint32_t bar_gfull = bar_rempty + 8 * kNSR;        // [kNSG] expanders (256 arrivals) -> MMA
  const uint32_t bar_gempty = bar_gfull + 8 * kNSG;        // [kNSG] MMA commit -> expanders
  const uint32_t bar_tfull = bar_gempty + 8 * kNSG;        // [kNT] MMA commit -> drain
  const uint32_t bar_tempty = bar_tfull + 8 * kNT;         // [kNT] drain (4 arrivals) -> MMA
  const uint32_t bar_imgfull = bar_tempty + 8 * kNT;
  const uint32_t bar_imgfree = bar_imgfull + 8;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + C::kOffBar + 200);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + C::kOffBar + 208);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total = batch.total_tiles;
  const int t0 = (int)((int64_t)total * blockIdx.x / gridDim.x);
  const int t1 = (int)((int64_t)total * (blockIdx.x + 1) / gridDim.x);
  const int n_local = t1 - t0;
  const int tpu = batch.tiles_per_unit;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kNSK; ++i) { mbar_init(bar_kfull + 8 * i, 1); mbar_init(bar_kempty + 8 * i, 1); }
    for (int i = 0; i < kNSR; ++i) { mbar_init(bar_rfull + 8 * i, 1); mbar_init(bar_rempty + 8 * i, 256); }
    for (int i = 0; i < kNSG; ++i) { mbar_init(bar_gfull + 8 * i, 256); mbar_init(bar_gempty + 8 * i, 1); }
    for (int i = 0; i < kNT; ++i) { mbar_init(bar_tfull + 8 * i, 1); mbar_init(bar_tempty + 8 * i, 4); }
    mbar_init(bar_imgfull, 1);
    mbar_init(bar_imgfree, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32((const void*)tmem_slot), 256);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      bool ok = true;
      int img_loads = 0, cur_unit = -1;
      int kc = 0, rc = 0;                                  // running chunk counters of the two rings
      for (int i = 0; i < n_local && ok; ++i) {
        const int t = t0 + i;
        const int unit = t / tpu, kt = t - unit * tpu;
        const int bh = unit / batch.n_qblocks;
        if (unit != cur_unit) {
          if (img_loads > 0) ok = mbar_wait(bar_imgfree, (uint32_t)((img_loads - 1) & 1), abort_flag);
          if (!ok) break;
          mbar_arrive_expect_tx(bar_imgfull, C::kImageBytes);
          bulk_load(img_smem, batch.images + (size_t)unit * C::kImageBytes, C::kImageBytes, bar_imgfull);
          ++img_loads;
          cur_unit = unit;
        }
        for (int c = 0; c < kHalfChunks && ok; ++c) {
          const int sk = kc % kNSK;
          ok = mbar_wait(bar_kempty + 8 * sk, (uint32_t)(((kc / kNSK) & 1) ^ 1), abort_flag);
          if (!ok) break;
          mbar_arrive_expect_tx(bar_kfull + 8 * sk, kChunkA);
          tma_load_3d(k_smem + sk * kChunkA, &batch.kmse_map, c * 64, kt * kKeys, bh, bar_kfull + 8 * sk);
          ++kc;
          const int sr = rc % kNSR;
          ok = mbar_wait(bar_rempty + 8 * sr, (uint32_t)(((rc / kNSR) & 1) ^ 1), abort_flag);
          if (!ok) break;
          mbar_arrive_expect_tx(bar_rfull + 8 * sr, kChunkRaw);
          tma_load_3d(r_smem + sr * kChunkRaw, &batch.sign_map, c * 64, kt * kKeys, bh, bar_rfull + 8 * sr);
          ++rc;
        }
      }
      if (!ok) {
        *abort_flag = 1;
        if (batch.status != nullptr) atomicCAS(batch.status, 0, (1 << 16) | (int)blockIdx.x);
      }
      // none of this CTA's own copies may still be in flight when it exits
      for (int k = 0; k < kNSK && k < kc; ++k) {
        const int j = kc - 1 - k;
        mbar_wait(bar_kfull + 8 * (j % kNSK), (uint32_t)((j / kNSK) & 1), abort_flag);
      }
      for (int k = 0; k < kNSR && k < rc; ++k) {
        const int j = rc - 1 - k;
        mbar_wait(bar_rfull + 8 * (j % kNSR), (uint32_t)((j / kNSR) & 1), abort_flag);
      }
      if (img_loads > 0) mbar_wait(bar_imgfull, (uint32_t)((img_loads - 1) & 1), abort_flag);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (converged warp, one elected lane issues)
    bool ok = true;
    int img_uses = 0, cur_unit = -1;
    int kc = 0, gc = 0;
    const uint32_t idesc = idesc_f16_n(kQ);
    const uint64_t b_hi = smem_desc_sw128(img_smem);
    const uint64_t b_lo = smem_desc_sw128(img_smem + kChunks * kChunkB);
    for (int i = 0; i < n_local && ok; ++i) {
      const int t = t0 + i;
      const int unit = t / tpu;
      if (unit != cur_unit) {
        ok = mbar_wait(bar_imgfull, (uint32_t)(img_uses & 1), abort_flag);
        ++img_uses;
        cur_unit = unit;
      }
      const int b = i % kNT;
      ok = ok && mbar_wait(bar_tempty + 8 * b, (uint32_t)(((i / kNT) & 1) ^ 1), abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const uint32_t d_tmem = tmem_base + (uint32_t)(b * kQ);
      const bool last_of_unit = i + 1 >= n_local || (t + 1) / tpu != unit;
#pragma unroll 1
      for (int c = 0; c < kChunks; ++c) {
        // chunks 0 .. D/64-1 come from the k_mse ring, the others from the expanded sign ring
        const bool from_k = c < kHalfChunks;
        uint32_t a_addr, full_bar, empty_bar, parity;
        if (from_k) {
          const int s = kc % kNSK;
          a_addr = k_smem + s * kChunkA; full_bar = bar_kfull + 8 * s; empty_bar = bar_kempty + 8 * s;
          parity = (uint32_t)((kc / kNSK) & 1);
          ++kc;
        } else {
          const int s = gc % kNSG;
          a_addr = g_smem + s * kChunkA; full_bar = bar_gfull + 8 * s; empty_bar = bar_gempty + 8 * s;
          parity = (uint32_t)((gc / kNSG) & 1);
          ++gc;
        }
        ok = mbar_wait(full_bar, parity, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const uint64_t a_base = smem_desc_sw128(a_addr);
        const uint64_t b_off = (uint64_t)((uint32_t)c * kChunkB / 16);
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16(d_tmem, a_base + (uint64_t)(k * 2), b_hi + b_off + (uint64_t)(k * 2), idesc, (c | k) != 0 ? 1u : 0u);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16(d_tmem, a_base + (uint64_t)(k * 2), b_lo + b_off + (uint64_t)(k * 2), idesc, 1u);
          umma_commit(empty_bar);                          // the operand stage is free once these MMAs are done
          if (c == kChunks - 1) {
            umma_commit(bar_tfull + 8 * b);
            if (last_of_unit) umma_commit(bar_imgfree);
          }
        }
        __syncwarp();
      }
    }
    if (!ok && lane == 0) {
      *abort_flag = 1;
      if (batch.status != nullptr) atomicCAS(batch.status, 0, (2 << 16) | (int)blockIdx.x);
    }
  } else if (warp < 2 + kExpWarps) {
    // ------------------------------------------------------------ expanders: thread = (key row, 32-sign half of the chunk)
    const int et = threadIdx.x - 64;
    const int row = et & 127, half = et >> 7;
    bool ok = true;
    int rc = 0, gc = 0;
    for (int i = 0; i < n_local && ok; ++i) {
      const int t = t0 + i;
      const int unit = t / tpu, kt = t - unit * tpu;
      const int64_t bh = unit / batch.n_qblocks;
      const int64_t key = (int64_t)kt * kKeys + row;
      const uint32_t rn = key < batch.Sk ? (uint32_t)__ldg(batch.rnorm + bh * batch.Sk + key) : 0u;
      const uint32_t rr = rn | (rn << 16);
      for (int c = 0; c < kHalfChunks && ok; ++c) {
        const int sr = rc % kNSR, sg = gc % kNSG;
        ok = mbar_wait(bar_rfull + 8 * sr, (uint32_t)((rc / kNSR) & 1), abort_flag);
        if (!ok) break;
        ok = mbar_wait(bar_gempty + 8 * sg, (uint32_t)(((gc / kNSG) & 1) ^ 1), abort_flag);
        if (!ok) break;
        const uint32_t src = r_smem + sr * kChunkRaw + (uint32_t)(row * 64 + half * 32);
        const uint32_t dst_row = g_smem + sg * kChunkA + (uint32_t)row * 128u;
        const uint4 x0 = ld_shared_v4(src), x1 = ld_shared_v4(src + 16);
        const uint32_t w[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {                      // 16-byte output chunk 4*half + q = signs 8q .. 8q+7 of this half
          uint32_t o[4];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t neg = w[2 * q + h] & 0x80808080u;             // sign bit of each of four int8 values
            o[2 * h] = rr ^ __byte_perm(neg, 0u, 0x1404u);                // bytes 0,1 -> bits 15, 31
            o[2 * h + 1] = rr ^ __byte_perm(neg, 0u, 0x3424u);            // bytes 2,3 -> bits 15, 31
          }
          const int cq = 4 * half + q;
          st_shared_v4(dst_row + (uint32_t)((cq ^ (row & 7)) << 4), o[0], o[1], o[2], o[3]);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // operand writes -> visible to the tensor core
        mbar_arrive(bar_gfull + 8 * sg);
        mbar_arrive(bar_rempty + 8 * sr);
        ++rc; ++gc;
      }
    }
    if (!ok && lane == 0) {
      *abort_flag = 1;
      if (batch.status != nullptr) atomicCAS(batch.status, 0, (3 << 16) | (int)blockIdx.x);
    }
  } else {
    // ------------------------------------------------------------ drain: thread = key, columns = queries
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    bool ok = true;
    for (int i = 0; i < n_local && ok; ++i) {
      const int t = t0 + i;
      const int unit = t / tpu, kt = t - unit * tpu;
      const int64_t bh = unit / batch.n_qblocks;
      const int q0 = (unit % batch.n_qblocks) * kQ;
      const int64_t key = (int64_t)kt * kKeys + row;
      const int b = i % kNT;
      ok = __all_sync(0xffffffffu, mbar_wait(bar_tfull + 8 * b, (uint32_t)((i / kNT) & 1), abort_flag));   // warp-collective TMEM loads follow
      if (!ok) break;
      tc_fence_after();
      const uint32_t tacc = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(b * kQ);
      float* out = batch.scores + (bh * batch.Sq + q0) * batch.Sk + key;
      const bool key_ok = key < batch.Sk;
      uint32_t ra[16], rb[16];
      tmem_issue16(tacc, ra);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t (&cur)[16] = (c & 1) ? rb : ra;
        uint32_t (&nxt)[16] = (c & 1) ? ra : rb;
        tmem_wait16(cur);
        if (c + 1 < 4) tmem_issue16(tacc + (c + 1) * 16, nxt);
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const int q = c * 16 + e;
          if (key_ok && q0 + q < batch.Sq) out[(int64_t)q * batch.Sk] = __uint_as_float(cur[e]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + 8 * b);
    }
    if (!ok && lane == 0) {
      *abort_flag = 1;
      if (batch.status != nullptr) atomicCAS(batch.status, 0, (4 << 16) | (int)blockIdx.x);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

template <int D>
int launch(const TqQjlScoreJob& job, const float* qf, const float* qproj, uint8_t* images, cudaStream_t st) {
  TensorMapEncodeFn enc = tensor_map_encoder();
  if (enc == nullptr) return TQ_ELAUNCH;
  static thread_local QjlBatch batch;
  const int n_qblocks = (int)((job.Sq + kQ - 1) / kQ);
  const int64_t tpu = (job.Sk + kKeys - 1) / kKeys;
  const int64_t units = job.BH * n_qblocks;
  const int64_t total = units * tpu;
  if (total >= ((int64_t)1 << 30)) return TQ_ETOOBIG;
  cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)job.Sk, (cuuint64_t)job.BH};
  cuuint32_t box[3] = {64, (cuuint32_t)kKeys, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  cuuint64_t strides_h[2] = {(cuuint64_t)D * 2, (cuuint64_t)job.Sk * D * 2};
  CUresult r = enc(&batch.kmse_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<uint16_t*>(job.k_mse), dims, strides_h,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { note_cuda_error(100000 + (int)r); return TQ_ELAUNCH; }
  cuuint64_t strides_b[2] = {(cuuint64_t)D, (cuuint64_t)job.Sk * D};
  r = enc(&batch.sign_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<int8_t*>(job.signs), dims, strides_b, box, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { note_cuda_error(100000 + (int)r); return TQ_ELAUNCH; }
  const float corr = (float)(1.2533141373155001 / (double)D);   // sqrt(pi/2) / m with m = D
  k_qjl_query_image<D><<<(unsigned)(units * kImageSplit), 256, 0, st>>>(qf, qproj, corr, job.Sq, n_qblocks, images);
  int rc = check_launch();
  if (rc != TQ_OK) return rc;
  batch.rnorm = job.rnorm;
  batch.images = images;
  batch.scores = job.scores;
  void* status_ptr = nullptr;
  cudaGetSymbolAddress(&status_ptr, g_qjl_status);
  batch.status = reinterpret_cast<int32_t*>(status_ptr);
  batch.Sq = job.Sq;
  batch.Sk = job.Sk;
  batch.n_qblocks = n_qblocks;
  batch.tiles_per_unit = (int32_t)tpu;
  batch.total_tiles = (int32_t)total;
  batch.pad_ = 0;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = (int)(total < sms ? total : sms);
  cudaError_t e = cudaFuncSetAttribute(k_umma_qjl_scores<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)QCfg<D>::kSmemBytes);
  if (e != cudaSuccess) { note_cuda_error((int)e); return TQ_ELAUNCH; }
  k_umma_qjl_scores<D><<<grid, kThreadsQ, QCfg<D>::kSmemBytes, st>>>(batch);
  return check_launch();
}

}  // namespace

bool umma_qjl_scores_eligible(const TqQjlScoreJob& job) {
  if (force_simt()) return false;
  if (job.D != 128 && job.D != 256) return false;
  if (job.BH <= 0 || job.Sq <= 0 || job.Sk <= 0 || job.BH > 65535) return false;
  if (((uintptr_t)job.k_mse & 15u) || ((uintptr_t)job.signs & 15u)) return false;
  if ((job.Sk * job.D) % 16 != 0) return false;           // tensor-map strides are multiples of 16 bytes
  return true;
}

size_t umma_qjl_scores_image_bytes(int64_t BH, int64_t Sq, int D) {
  if (D != 128 && D != 256) return 0;
  const int64_t units = BH * ((Sq + kQ - 1) / kQ);
  return (size_t)units * (D == 256 ? QCfg<256>::kImageBytes : QCfg<128>::kImageBytes) + 1024;
}

// qf: the queries as fp32 (BH, Sq, D); qproj: S-projected queries (BH, Sq, D); images: scratch
int umma_qjl_scores(const TqQjlScoreJob& job, const float* qf, const float* qproj, void* images, cudaStream_t st) {
  uint8_t* img = reinterpret_cast<uint8_t*>(((uintptr_t)images + 1023u) & ~(uintptr_t)1023u);
  return job.D == 256 ? launch<256>(job, qf, qproj, img, st) : launch<128>(job, qf, qproj, img, st);
}

int umma_qjl_device_status() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_qjl_status, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

}  // namespace tq
