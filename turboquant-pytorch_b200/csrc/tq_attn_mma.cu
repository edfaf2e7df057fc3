// Attention straight from packed keys (and packed values) on the tensor cores, head_dim 128.
//
// Logits  l[g][s] = scale * norm_s * sum_j (q_g Pi^T)_j * c[idx_sj]  are a contraction over the 128
// coordinates.  The FP32 kernel (tq_simt.cu) spends ~1 400 instructions per key on it; here the
// multiply-adds run as mma.sync.m16n8k16 (fp16 inputs, fp32 accumulate) and only the centroid look-ups
// stay on the CUDA cores:
//   * M = 16 rows = 16 keys, K = 16 coordinates per instruction (8 k-steps per key), N = 8 columns = up to
//     4 query rows (the query heads that share the KV head x query tokens) as fp16 pieces: columns 0..3
//     hold q_hi, columns 4..7 q_lo;
//   * the key operand is assembled IN REGISTERS: thread (gid = lane / 4, t = lane % 4) reads quarter t of
//     the packed rows of keys gid and gid + 8 (one 4..32-byte load each) and looks up the centroids each
//     k-step needs in a shared table of (hi | lo << 16) fp16 pieces.  A dot product does not care in which
//     order its terms are visited, so the coordinates are assigned to k-steps in the order that makes a
//     thread's operand elements come from its own contiguous bytes: k-step ks, thread t covers coordinates
//     32 t + 4 ks + 0..3 (the query operand uses the same order);
//   * two MMAs per k-step (centroid pieces hi, lo) into ONE accumulator: column g collects
//     (c_hi + c_lo).q_hi, column g + 4 collects (c_hi + c_lo).q_lo; their sum is the fp32-accurate logit
//     (all four cross terms), one shuffle away.
// The softmax partials per block of keys and the finishing pass are those of the FP32 path.

#include "tq_common.cuh"
#include "tq_internal.h"

namespace tq {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kRows = 4;                       // query rows per pass (columns g and g + 4 of the accumulator)
constexpr int kDimA = 128;

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_half2(float x, float y) {
  __half2 h = __floats2half2_rn(x, y);
  return *reinterpret_cast<uint32_t*>(&h);
}

// fp16 pieces of two floats: hi = rn(x), lo = rn(x - hi)
__device__ __forceinline__ void split2(float x, float y, uint32_t& hi, uint32_t& lo) {
  const __half hx = __float2half_rn(x), hy = __float2half_rn(y);
  hi = (uint32_t)__half_as_ushort(hx) | ((uint32_t)__half_as_ushort(hy) << 16);
  lo = pack_half2(x - __half2float(hx), y - __half2float(hy));
}

template <int BITS>
struct Packed {
  static constexpr int IPB = 8 / BITS;
  static constexpr int G = kDimA / IPB;        // packed bytes per key
  static constexpr int CB = G / 4;             // bytes per thread: a quarter row = 32 coordinates
  static constexpr int CW = CB / 4;            // 32-bit words per thread: 1, 2, 4 or 8
};

// the quarter row `t` of one key
template <int BITS>
__device__ __forceinline__ void load_quarter(const uint8_t* row, int t, uint32_t (&w)[Packed<BITS>::CW]) {
  constexpr int CW = Packed<BITS>::CW;
  const uint8_t* p = row + t * Packed<BITS>::CB;
  if constexpr (CW == 1) {
    w[0] = __ldg(reinterpret_cast<const uint32_t*>(p));
  } else if constexpr (CW == 2) {
    const uint2 v = __ldg(reinterpret_cast<const uint2*>(p));
    w[0] = v.x; w[1] = v.y;
  } else {
#pragma unroll
    for (int k = 0; k < CW / 4; ++k) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(p) + k);
      w[4 * k] = v.x; w[4 * k + 1] = v.y; w[4 * k + 2] = v.z; w[4 * k + 3] = v.w;
    }
  }
}

__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

// Shared-memory addresses of the table entries of one packed word's coordinates.  The table is 1024-byte
// aligned; for codes of up to 6 bits an entry's offset (index * 4) fits one byte, so the fields of a word are
// moved to byte position with one shift and mask per field position (shared by the word's four bytes) and
// each address is then ONE byte permute that drops the offset byte into the table's base address.
template <int BITS>
struct WordAddr {
  static constexpr int IPB = Packed<BITS>::IPB;
  static constexpr bool kFast = BITS <= 6;
  uint32_t f[IPB];                              // field position p of every byte, as offset bytes (fast path)
  uint32_t x, base;
  __device__ __forceinline__ WordAddr(uint32_t word, uint32_t lut_base) : x(word), base(lut_base) {
    if constexpr (kFast) {
      constexpr uint32_t M = (((1u << BITS) - 1u) << 2) * 0x01010101u;
#pragma unroll
      for (int p = 0; p < IPB; ++p) {
        const int sh = BITS * (IPB - 1 - p);    // field p sits sh bits up in its byte (first index in the high bits)
        f[p] = sh >= 2 ? ((word >> (sh - 2)) & M) : ((word << (2 - sh)) & M);
      }
    }
  }
  // address of the entry of coordinate c (0 .. 4 * IPB - 1) of this word
  __device__ __forceinline__ uint32_t operator()(int c) const {
    const int byte = c / IPB, p = c % IPB;
    if constexpr (kFast) {
      return __byte_perm(f[p], base, 0x7650u | (uint32_t)byte);
    } else {
      constexpr uint32_t MASK = ((1u << BITS) - 1u) << 2;
      const int sh = 8 * byte;
      return base + (sh >= 2 ? ((x >> (sh - 2)) & MASK) : ((x << (2 - sh)) & MASK));
    }
  }
};

// key operand of k-step ks for both centroid pieces: the thread's local coordinates 4 ks .. 4 ks + 3
template <int BITS>
__device__ __forceinline__ void key_fragment(const uint32_t (&w)[Packed<BITS>::CW], int ks, uint32_t lut_base,
                                             uint32_t (&bh)[2], uint32_t (&bl)[2]) {
  constexpr int CPW = 4 * Packed<BITS>::IPB;    // coordinates per word: 4 (wide codes) .. 32 (1 bit)
  const int u0 = 4 * ks;
  const WordAddr<BITS> wa(w[u0 / CPW], lut_base);
  uint32_t e[4];
#pragma unroll
  for (int p = 0; p < 4; ++p) e[p] = lds_u32(wa((u0 + p) % CPW));
  bh[0] = __byte_perm(e[0], e[1], 0x5410); bl[0] = __byte_perm(e[0], e[1], 0x7632);
  bh[1] = __byte_perm(e[2], e[3], 0x5410); bl[1] = __byte_perm(e[2], e[3], 0x7632);
}

// (max, sum of exp) running pair
__device__ __forceinline__ void stat_add(float& m, float& s, float l) {
  const float nm = fmaxf(m, l);
  if (nm != -INFINITY) s = s * __expf(m - nm) + __expf(l - nm);
  m = nm;
}
__device__ __forceinline__ void stat_merge(float& m, float& s, float m2, float s2) {
  const float nm = fmaxf(m, m2);
  if (nm != -INFINITY) s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - nm));
  m = nm;
}

// Query operand of one pass: column n = lane / 4 of the 8-column operand is row r0 + (n & 3) of the rotated
// queries, as its high piece (n < 4) or low piece (n >= 4); thread t holds coordinates 32 t + 4 ks + 0..3.
__device__ __forceinline__ void query_fragments(const float* __restrict__ qrot, int64_t row, bool row_ok, int lane,
                                                uint32_t (&bq)[8][2]) {
  const int t = lane & 3;
  const bool low = (lane >> 2) >= 4;
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row_ok) v = __ldg(reinterpret_cast<const float4*>(qrot + row * kDimA + 32 * t + 4 * ks));
    uint32_t h0, l0, h1, l1;
    split2(v.x, v.y, h0, l0);
    split2(v.z, v.w, h1, l1);
    bq[ks][0] = low ? l0 : h0;
    bq[ks][1] = low ? l1 : h1;
  }
}

// 16 keys x 4 query rows: c[0..1] = key gid, c[2..3] = key gid + 8, columns (2t, 2t + 1) of [q_hi | q_lo].
template <int BITS>
__device__ __forceinline__ void score_block(const uint32_t (&w0)[Packed<BITS>::CW], const uint32_t (&w1)[Packed<BITS>::CW],
                                            const uint32_t (&bq)[8][2], uint32_t lut_base, float (&c)[4]) {
  c[0] = c[1] = c[2] = c[3] = 0.f;
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    uint32_t h0[2], l0[2], h1[2], l1[2];
    key_fragment<BITS>(w0, ks, lut_base, h0, l0);
    key_fragment<BITS>(w1, ks, lut_base, h1, l1);
    mma_16816(c, h0[0], h1[0], h0[1], h1[1], bq[ks][0], bq[ks][1]);
    mma_16816(c, l0[0], l1[0], l0[1], l1[1], bq[ks][0], bq[ks][1]);
  }
  // column g + 4 (low query piece) lives two lanes away: afterwards lanes t and t ^ 2 both hold the full sums
#pragma unroll
  for (int j = 0; j < 4; ++j) c[j] += __shfl_xor_sync(0xffffffffu, c[j], 2);
}

// grid: B * Hkv * nblk CTAs, each over keys_per_block keys of one KV head; stats as in the FP32 path:
// stats[(row * nblk + blk) * 2 + {0, 1}] = (max, sum of exp(l - max)) of the block's keys.
template <int BITS>
__global__ void __launch_bounds__(kThreads, 2) k_score_mma(TqScoreJob job, const float* __restrict__ qrot, float* stats, int nblk,
                                                        int keys_per_block) {
  constexpr int G = Packed<BITS>::G;
  constexpr int CW = Packed<BITS>::CW;
  __shared__ __align__(1024) uint32_t lut[256];
  __shared__ float red_m[kWarps][kRows], red_s[kWarps][kRows];
  {
    const float c = __ldg(job.codebook + kCentroidOff + threadIdx.x);
    const __half h = __float2half_rn(c);
    const __half l = __float2half_rn(c - __half2float(h));
    lut[threadIdx.x] = (uint32_t)__half_as_ushort(h) | ((uint32_t)__half_as_ushort(l) << 16);
  }
  const uint32_t lut_base = (uint32_t)__cvta_generic_to_shared(lut);
  const int blk = blockIdx.x % nblk;
  const int64_t bh = blockIdx.x / nblk;
  const int64_t b = bh / job.Hkv, hkv = bh % job.Hkv;
  const int rep = (int)(job.Hq / job.Hkv);
  const int R = rep * (int)job.Sq;
  const int64_t s_begin = (int64_t)blk * keys_per_block;
  const int64_t s_end = min(s_begin + (int64_t)keys_per_block, job.Sk);
  const uint8_t* keys = job.idx_bytes + bh * job.Sk * G;
  const uint16_t* norms = job.norms + bh * job.Sk;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, t = lane & 3;
  __syncthreads();
  auto global_row = [&](int r) -> int64_t {
    const int64_t hq = hkv * rep + r / job.Sq, sq = r % job.Sq;
    return (b * job.Hq + hq) * job.Sq + sq;
  };
  for (int r0 = 0; r0 < R; r0 += kRows) {
    uint32_t bq[8][2];
    {
      const int r = r0 + (gid & 3);
      query_fragments(qrot, r < R ? global_row(r) : 0, r < R, lane, bq);
    }
    // after the shuffle in score_block this lane finishes ONE key (gid for t < 2, gid + 8 otherwise) and the
    // two query rows r0 + 2 (t & 1) + {0, 1}
    const int ra = r0 + 2 * (t & 1);
    const bool ok_a = ra < R, ok_b = ra + 1 < R;
    const int64_t row_a = ok_a ? global_row(ra) : 0, row_b = ok_b ? global_row(ra + 1) : 0;
    float m_a = -INFINITY, s_a = 0.f, m_b = -INFINITY, s_b = 0.f;
    // the packed quarter rows and the norm of the NEXT block of 16 keys are in flight while this one is scored
    uint32_t w0[CW], w1[CW], n0[CW], n1[CW];
    uint16_t nv_bits = 0, nn_bits = 0;
    auto fetch = [&](int64_t kb, uint32_t (&a0)[CW], uint32_t (&a1)[CW], uint16_t& nb) {
      const int64_t k_lo = kb + gid, k_hi = kb + 8 + gid;
      load_quarter<BITS>(keys + (k_lo < s_end ? k_lo : s_begin) * G, t, a0);
      load_quarter<BITS>(keys + (k_hi < s_end ? k_hi : s_begin) * G, t, a1);
      const int64_t key = t < 2 ? k_lo : k_hi;
      nb = __ldg(norms + (key < s_end ? key : s_begin));
    };
    int64_t kb = s_begin + warp * 16;
    if (kb < s_end) fetch(kb, w0, w1, nv_bits);
    for (; kb < s_end; kb += kWarps * 16) {
      const int64_t kn = kb + kWarps * 16;
      if (kn < s_end) fetch(kn, n0, n1, nn_bits);
      float c[4];
      score_block<BITS>(w0, w1, bq, lut_base, c);
      const int64_t key = (t < 2 ? kb : kb + 8) + gid;
      if (key < s_end) {
        const float nv = __half2float(__ushort_as_half(nv_bits)) * job.scale;
        const float la = (t < 2 ? c[0] : c[2]) * nv, lb = (t < 2 ? c[1] : c[3]) * nv;
        if (ok_a) job.logits[row_a * job.Sk + key] = la;
        if (ok_b) job.logits[row_b * job.Sk + key] = lb;
        if (stats != nullptr) { stat_add(m_a, s_a, la); stat_add(m_b, s_b, lb); }
      }
#pragma unroll
      for (int k = 0; k < CW; ++k) { w0[k] = n0[k]; w1[k] = n1[k]; }
      nv_bits = nn_bits;
    }
    if (stats != nullptr) {
      // lanes that share (t & 1) share the two rows: fold over the other lane bits, then over the warps
#pragma unroll
      for (int o = 2; o <= 16; o <<= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m_a, o), s2 = __shfl_xor_sync(0xffffffffu, s_a, o);
        stat_merge(m_a, s_a, m2, s2);
        const float m3 = __shfl_xor_sync(0xffffffffu, m_b, o), s3 = __shfl_xor_sync(0xffffffffu, s_b, o);
        stat_merge(m_b, s_b, m3, s3);
      }
      if (lane < 2) {
        red_m[warp][2 * lane] = m_a; red_s[warp][2 * lane] = s_a;
        red_m[warp][2 * lane + 1] = m_b; red_s[warp][2 * lane + 1] = s_b;
      }
      __syncthreads();
      if (threadIdx.x < kRows && r0 + (int)threadIdx.x < R) {
        float m = -INFINITY, s = 0.f;
        for (int wv = 0; wv < kWarps; ++wv) stat_merge(m, s, red_m[wv][threadIdx.x], red_s[wv][threadIdx.x]);
        const int64_t orow = global_row(r0 + threadIdx.x);
        stats[(orow * nblk + blk) * 2 + 0] = m;
        stats[(orow * nblk + blk) * 2 + 1] = s;
      }
      __syncthreads();
    }
  }
}

}  // namespace

bool mma_score_eligible(const TqScoreJob& job) {
  if (force_simt()) return false;
  return job.D == kDimA && (((uintptr_t)job.idx_bytes) & 15u) == 0 && (((uintptr_t)job.norms) & 1u) == 0;
}

// logits (and the per-block softmax partials when stats != NULL) for a job whose queries are already rotated
int mma_score_packed(const TqScoreJob& job, const float* qrot, float* stats, int nblk, int keys_per_block, cudaStream_t st) {
  const int64_t blocks = job.B * job.Hkv * nblk;
  switch (job.bits) {
    case 1: k_score_mma<1><<<(unsigned)blocks, kThreads, 0, st>>>(job, qrot, stats, nblk, keys_per_block); break;
    case 2: k_score_mma<2><<<(unsigned)blocks, kThreads, 0, st>>>(job, qrot, stats, nblk, keys_per_block); break;
    case 3: k_score_mma<3><<<(unsigned)blocks, kThreads, 0, st>>>(job, qrot, stats, nblk, keys_per_block); break;
    case 4: k_score_mma<4><<<(unsigned)blocks, kThreads, 0, st>>>(job, qrot, stats, nblk, keys_per_block); break;
    case 5: k_score_mma<5><<<(unsigned)blocks, kThreads, 0, st>>>(job, qrot, stats, nblk, keys_per_block); break;
    case 6: k_score_mma<6><<<(unsigned)blocks, kThreads, 0, st>>>(job, qrot, stats, nblk, keys_per_block); break;
    case 7: k_score_mma<7><<<(unsigned)blocks, kThreads, 0, st>>>(job, qrot, stats, nblk, keys_per_block); break;
    default: k_score_mma<8><<<(unsigned)blocks, kThreads, 0, st>>>(job, qrot, stats, nblk, keys_per_block); break;
  }
  return check_launch();
}

}  // namespace tq
