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

#include <atomic>

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

// ---------------------------------------------------------------------------------------------------
// Decode attention on packed keys AND packed values:  out = softmax(scale * q k_hat^T) v_hat  without
// reconstructing either.  With v_hat_s = norm_s * (c_v[idx_s] Pi_v), the weighted sum is taken in the
// rotated domain,  acc[g][j] = sum_s p[g][s] * norm_v[s] * c_v[idx_v[s][j]],  and Pi_v is applied once at the
// end (k_decode_finish).  Per block of 16 keys a warp
//   1. scores the keys as above (score_block), applies norm and scale;
//   2. keeps a running maximum and sum per query row (online softmax) and rescales its accumulators when
//      the maximum moves;
//   3. forms P' = exp(l - max) * norm_v as fp16 pieces, columns [P'_hi rows 0..3 | P'_lo rows 0..3], and
//      turns the accumulator-layout block (16 keys x 8 columns) into the B operand of the next product with
//      two 8x8 transposes (movmatrix);
//   4. accumulates  acc^T (16 coordinates x 8 columns) += V^T (16 coordinates x 16 keys) P'  for 8 blocks of
//      coordinates, value pieces hi and lo: thread (gid, t) assembles the value operand for keys
//      2t, 2t+1, 2t+8, 2t+9 and its own 16 coordinates 16 gid .. 16 gid + 15 from the packed value rows.
// Each CTA covers keys_per_block keys of one (batch, KV head) and writes one partial (max, sum, acc) per
// query row; k_decode_finish merges the partials, the 16-bit window tokens and applies Pi_v.

template <int BITS>
struct PackedV {
  static constexpr int IPB = 8 / BITS;
  static constexpr int G = kDimA / IPB;         // packed bytes per value row
  static constexpr int CB = G / 8;              // bytes per thread and key: an eighth of a row = 16 coordinates
  static constexpr int CW = CB >= 4 ? CB / 4 : 1;
};

// the eighth `e` of one packed value row (16 coordinates): 2 (1-bit), 4, 8 or 16 bytes
template <int BITS>
__device__ __forceinline__ void load_eighth(const uint8_t* row, int e, uint32_t (&w)[PackedV<BITS>::CW]) {
  constexpr int CB = PackedV<BITS>::CB;
  const uint8_t* p = row + e * CB;
  if constexpr (CB == 2) {
    w[0] = __ldg(reinterpret_cast<const uint16_t*>(p));
  } else if constexpr (CB == 4) {
    w[0] = __ldg(reinterpret_cast<const uint32_t*>(p));
  } else if constexpr (CB == 8) {
    const uint2 v = __ldg(reinterpret_cast<const uint2*>(p));
    w[0] = v.x; w[1] = v.y;
  } else {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
    w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
  }
}

// table entry (hi | lo << 16) of local coordinate v (0..15) of a thread's eighth row
template <int BITS>
__device__ __forceinline__ uint32_t value_entry(const uint32_t (&w)[PackedV<BITS>::CW], int v, uint32_t lut_base) {
  constexpr int CPW = 4 * PackedV<BITS>::IPB;
  const WordAddr<BITS> wa(w[v / CPW], lut_base);
  return lds_u32(wa(v % CPW));
}

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}

struct DecodeParams {
  const float* qrot;          // (rows, 128) rotated queries
  const uint8_t* k_idx; const uint16_t* k_norms;
  const uint8_t* v_idx; const uint16_t* v_norms;
  const float* k_codebook; const float* v_codebook;
  float* part;                // [rows][nblk][130]: max, sum, acc[128] (rotated domain, coordinates in natural order)
  int64_t B, Hq, Sq, Hkv, Sk;
  float scale;
  int nblk, keys_per_block;
};
constexpr int kPartStride = 130;

template <int KBITS, int VBITS>
__global__ void __launch_bounds__(kThreads, 1) k_decode_attn(DecodeParams P) {
  constexpr int GK = Packed<KBITS>::G, KW = Packed<KBITS>::CW;
  constexpr int GV = PackedV<VBITS>::G, VW = PackedV<VBITS>::CW;
  __shared__ __align__(1024) uint32_t lut_k[256];
  __shared__ __align__(1024) uint32_t lut_v[256];
  __shared__ float sm_m[kWarps][kRows], sm_l[kWarps][kRows];
  __shared__ float sm_acc[kWarps][kRows][kDimA];          // 16 KB
  {
    const float ck = __ldg(P.k_codebook + kCentroidOff + threadIdx.x);
    const __half hk = __float2half_rn(ck);
    lut_k[threadIdx.x] = (uint32_t)__half_as_ushort(hk) | ((uint32_t)__half_as_ushort(__float2half_rn(ck - __half2float(hk))) << 16);
    const float cv = __ldg(P.v_codebook + kCentroidOff + threadIdx.x);
    const __half hv = __float2half_rn(cv);
    lut_v[threadIdx.x] = (uint32_t)__half_as_ushort(hv) | ((uint32_t)__half_as_ushort(__float2half_rn(cv - __half2float(hv))) << 16);
  }
  const uint32_t lutk = (uint32_t)__cvta_generic_to_shared(lut_k);
  const uint32_t lutv = (uint32_t)__cvta_generic_to_shared(lut_v);
  const int blk = blockIdx.x % P.nblk;
  const int64_t bh = blockIdx.x / P.nblk;
  const int64_t b = bh / P.Hkv, hkv = bh % P.Hkv;
  const int rep = (int)(P.Hq / P.Hkv);
  const int R = rep * (int)P.Sq;
  const int64_t s_begin = (int64_t)blk * P.keys_per_block;
  const int64_t s_end = min(s_begin + (int64_t)P.keys_per_block, P.Sk);
  const uint8_t* keys = P.k_idx + bh * P.Sk * GK;
  const uint8_t* vals = P.v_idx + bh * P.Sk * GV;
  const uint16_t* k_norms = P.k_norms + bh * P.Sk;
  const uint16_t* v_norms = P.v_norms + bh * P.Sk;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, t = lane & 3;
  __syncthreads();
  auto global_row = [&](int r) -> int64_t {
    const int64_t hq = hkv * rep + r / P.Sq, sq = r % P.Sq;
    return (b * P.Hq + hq) * P.Sq + sq;
  };
  for (int r0 = 0; r0 < R; r0 += kRows) {
    uint32_t bq[8][2];
    {
      const int r = r0 + (gid & 3);
      query_fragments(P.qrot, r < R ? global_row(r) : 0, r < R, lane, bq);
    }
    // this lane's two query rows: r0 + 2 (t & 1) + {0, 1}; lanes t and t ^ 2 hold the same rows, the first as
    // the high pieces of P' (columns 0..3), the second as the low pieces (columns 4..7)
    float run_m[2] = {-INFINITY, -INFINITY}, run_l[2] = {0.f, 0.f};
    float acc[8][4];
#pragma unroll
    for (int mb = 0; mb < 8; ++mb) acc[mb][0] = acc[mb][1] = acc[mb][2] = acc[mb][3] = 0.f;
    uint32_t w0[KW], w1[KW], n0[KW], n1[KW];
    uint32_t vw[4][VW], vx[4][VW];                                   // value rows of this block and of the next
    uint32_t kn_bits = 0, kn_next = 0, vn_bits = 0, vn_next = 0;      // norms of keys gid (low half) and gid + 8 (high half)
    // keys, value rows and norms of a block: fetched one block ahead of their use (fetching the value rows at the
    // start of their own block left most of a memory latency exposed in every round)
    auto fetch = [&](int64_t kb, uint32_t (&a0)[KW], uint32_t (&a1)[KW], uint32_t (&av)[4][VW], uint32_t& kn, uint32_t& vn) {
      const int64_t k_lo = kb + gid, k_hi = kb + 8 + gid;
      const int64_t c_lo = k_lo < s_end ? k_lo : s_begin, c_hi = k_hi < s_end ? k_hi : s_begin;
      load_quarter<KBITS>(keys + c_lo * GK, t, a0);
      load_quarter<KBITS>(keys + c_hi * GK, t, a1);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int64_t key = kb + 2 * t + (q & 1) + 8 * (q >> 1);         // keys 2t, 2t+1, 2t+8, 2t+9
        load_eighth<VBITS>(vals + (key < s_end ? key : s_begin) * GV, gid, av[q]);
      }
      kn = (uint32_t)__ldg(k_norms + c_lo) | ((uint32_t)__ldg(k_norms + c_hi) << 16);
      vn = (uint32_t)__ldg(v_norms + c_lo) | ((uint32_t)__ldg(v_norms + c_hi) << 16);
    };
    int64_t kb = s_begin + warp * 16;
    if (kb < s_end) fetch(kb, w0, w1, vw, kn_bits, vn_bits);
    for (; kb < s_end; kb += kWarps * 16) {
      const int64_t kn = kb + kWarps * 16;
      if (kn < s_end) fetch(kn, n0, n1, vx, kn_next, vn_next);
      float c[4];
      score_block<KBITS>(w0, w1, bq, lutk, c);
      // logits of keys gid (c[0], c[1]) and gid + 8 (c[2], c[3]) for this lane's two rows
      const bool in_lo = kb + gid < s_end, in_hi = kb + 8 + gid < s_end;
      const float nk_lo = __half2float(__ushort_as_half((uint16_t)(kn_bits & 0xFFFFu))) * P.scale;
      const float nk_hi = __half2float(__ushort_as_half((uint16_t)(kn_bits >> 16))) * P.scale;
      float l[4];
      l[0] = in_lo ? c[0] * nk_lo : -INFINITY; l[1] = in_lo ? c[1] * nk_lo : -INFINITY;
      l[2] = in_hi ? c[2] * nk_hi : -INFINITY; l[3] = in_hi ? c[3] * nk_hi : -INFINITY;
      // block maximum per row over the 16 keys (lanes that differ in gid)
      float bm[2] = {fmaxf(l[0], l[2]), fmaxf(l[1], l[3])};
#pragma unroll
      for (int o = 4; o <= 16; o <<= 1) {
        bm[0] = fmaxf(bm[0], __shfl_xor_sync(0xffffffffu, bm[0], o));
        bm[1] = fmaxf(bm[1], __shfl_xor_sync(0xffffffffu, bm[1], o));
      }
      float alpha[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float nm = fmaxf(run_m[j], bm[j]);              // the block holds at least one valid key: finite
        alpha[j] = run_m[j] == -INFINITY ? 0.f : __expf(run_m[j] - nm);
        run_m[j] = nm;
      }
      float p[4];
      p[0] = __expf(l[0] - run_m[0]); p[1] = __expf(l[1] - run_m[1]);
      p[2] = __expf(l[2] - run_m[0]); p[3] = __expf(l[3] - run_m[1]);
      // row sums: every (row, key) pair is counted by exactly one of the lanes t and t ^ 2
      if (t < 2) { run_l[0] = run_l[0] * alpha[0] + p[0]; run_l[1] = run_l[1] * alpha[1] + p[1]; }
      else       { run_l[0] = run_l[0] * alpha[0] + p[2]; run_l[1] = run_l[1] * alpha[1] + p[3]; }
      // P' = p * norm_v as fp16 pieces; this lane contributes the high (t < 2) or low (t >= 2) piece
      const float nv_lo = __half2float(__ushort_as_half((uint16_t)(vn_bits & 0xFFFFu)));
      const float nv_hi = __half2float(__ushort_as_half((uint16_t)(vn_bits >> 16)));
      uint32_t x0, x1;
      {
        uint32_t h, lo2;
        split2(p[0] * nv_lo, p[1] * nv_lo, h, lo2);
        x0 = t < 2 ? h : lo2;
        split2(p[2] * nv_hi, p[3] * nv_hi, h, lo2);
        x1 = t < 2 ? h : lo2;
      }
      const uint32_t pb0 = movmatrix_trans(x0);               // keys 2t, 2t+1  x column gid
      const uint32_t pb1 = movmatrix_trans(x1);               // keys 2t+8, 2t+9 x column gid
      // rescale the accumulators when a maximum moved (columns 2t, 2t+1 are this lane's two rows in both halves)
      if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
        for (int mb = 0; mb < 8; ++mb) {
          acc[mb][0] *= alpha[0]; acc[mb][1] *= alpha[1]; acc[mb][2] *= alpha[0]; acc[mb][3] *= alpha[1];
        }
      }
      // acc^T += V^T P' for 8 blocks of 16 coordinates; this thread's rows are coordinates 16 gid + 2 mb + {0, 1}
#pragma unroll
      for (int mb = 0; mb < 8; ++mb) {
        uint32_t e[4][2];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          e[q][0] = value_entry<VBITS>(vw[q], 2 * mb, lutv);
          e[q][1] = value_entry<VBITS>(vw[q], 2 * mb + 1, lutv);
        }
        // A registers: (row gid, keys 2t, 2t+1), (row gid + 8, keys 2t, 2t+1), (row gid, keys 2t+8, 2t+9), (row gid + 8, ...)
        const uint32_t ah0 = __byte_perm(e[0][0], e[1][0], 0x5410), ah1 = __byte_perm(e[0][1], e[1][1], 0x5410);
        const uint32_t ah2 = __byte_perm(e[2][0], e[3][0], 0x5410), ah3 = __byte_perm(e[2][1], e[3][1], 0x5410);
        const uint32_t al0 = __byte_perm(e[0][0], e[1][0], 0x7632), al1 = __byte_perm(e[0][1], e[1][1], 0x7632);
        const uint32_t al2 = __byte_perm(e[2][0], e[3][0], 0x7632), al3 = __byte_perm(e[2][1], e[3][1], 0x7632);
        mma_16816(acc[mb], ah0, ah1, ah2, ah3, pb0, pb1);
        mma_16816(acc[mb], al0, al1, al2, al3, pb0, pb1);
      }
#pragma unroll
      for (int k = 0; k < KW; ++k) { w0[k] = n0[k]; w1[k] = n1[k]; }
#pragma unroll
      for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int k = 0; k < VW; ++k) vw[q][k] = vx[q][k];
      kn_bits = kn_next; vn_bits = vn_next;
    }
    // ---- fold the warp: sums over the lanes that share (t & 1), pieces hi + lo two lanes apart
#pragma unroll
    for (int o = 2; o <= 16; o <<= 1) {
      run_l[0] += __shfl_xor_sync(0xffffffffu, run_l[0], o);
      run_l[1] += __shfl_xor_sync(0xffffffffu, run_l[1], o);
    }
#pragma unroll
    for (int mb = 0; mb < 8; ++mb)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[mb][j] += __shfl_xor_sync(0xffffffffu, acc[mb][j], 2);
    // run_m is already uniform over gid (every block maximum was); lanes t < 2 publish rows 2t, 2t + 1
    if (lane < 2) {
      sm_m[warp][2 * lane] = run_m[0]; sm_m[warp][2 * lane + 1] = run_m[1];
      sm_l[warp][2 * lane] = run_l[0]; sm_l[warp][2 * lane + 1] = run_l[1];
    }
    if (t < 2) {
#pragma unroll
      for (int mb = 0; mb < 8; ++mb) {
        // acc[mb][0..1]: coordinate 16 gid + 2 mb, rows 2t, 2t+1;  acc[mb][2..3]: coordinate 16 gid + 2 mb + 1
        sm_acc[warp][2 * t][16 * gid + 2 * mb] = acc[mb][0];
        sm_acc[warp][2 * t + 1][16 * gid + 2 * mb] = acc[mb][1];
        sm_acc[warp][2 * t][16 * gid + 2 * mb + 1] = acc[mb][2];
        sm_acc[warp][2 * t + 1][16 * gid + 2 * mb + 1] = acc[mb][3];
      }
    }
    __syncthreads();
    // ---- fold the CTA's warps and write the partial of this block of keys
    for (int idx = threadIdx.x; idx < kRows * kDimA; idx += kThreads) {
      const int rr = idx / kDimA, j = idx % kDimA;
      if (r0 + rr >= R) continue;
      float m = -INFINITY;
      for (int wv = 0; wv < kWarps; ++wv) m = fmaxf(m, sm_m[wv][rr]);
      float a = 0.f, lsum = 0.f;
      for (int wv = 0; wv < kWarps; ++wv) {
        const float wm = sm_m[wv][rr];
        if (wm != -INFINITY) {
          const float f = __expf(wm - m);
          a += sm_acc[wv][rr][j] * f;
          lsum += sm_l[wv][rr] * f;
        }
      }
      float* dst = P.part + (global_row(r0 + rr) * P.nblk + blk) * kPartStride;
      dst[2 + j] = a;
      if (j == 0) { dst[0] = m; dst[1] = lsum; }
    }
    __syncthreads();
  }
}

// One CTA per query row: merge the partials of the packed tokens, add the 16-bit window tokens (their logits use
// the UNROTATED query), normalise, and rotate back:  out = (acc / L) Pi_v + sum_w p_w v_w / L.
struct FinishParams {
  const void* q; int q_dtype;
  const float* part; int nblk;
  const float* v_rotation;    // Pi_v (128 x 128, row-major): out = acc @ Pi_v
  const void* k_window; const void* v_window; int window_dtype;
  int64_t W, ws_b, ws_h, ws_s;
  int64_t B, Hq, Sq, Hkv, Sk;
  float scale;
  float* out;
};

template <int QDT, int WDT>
__global__ void __launch_bounds__(128) k_decode_finish(FinishParams F) {
  __shared__ float sh_q[kDimA], sh_acc[kDimA], sh_red[4];
  __shared__ float sh_m, sh_l;
  extern __shared__ float sh_w[];                 // window logits, then probabilities: W floats
  const int64_t row = blockIdx.x;
  const int64_t sq = row % F.Sq, hq = (row / F.Sq) % F.Hq, b = row / (F.Sq * F.Hq);
  const int64_t hkv = hq / (F.Hq / F.Hkv);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  (void)sq;
  sh_q[tid] = load_elem<QDT>(F.q, row * kDimA + tid);
  __syncthreads();
  // window logits
  const int64_t wbase = b * F.ws_b + hkv * F.ws_h;
  float wmax = -INFINITY;
  for (int64_t w = warp; w < F.W; w += 4) {
    float d = 0.f;
    for (int j = lane; j < kDimA; j += 32) d = fmaf(sh_q[j], load_elem<WDT>(F.k_window, wbase + w * F.ws_s + j), d);
    d = warp_sum(d) * F.scale;
    if (lane == 0) sh_w[w] = d;
    wmax = fmaxf(wmax, d);
  }
  // global maximum over the partials and the window
  float m = wmax;
  if (F.Sk > 0)
    for (int i = tid; i < F.nblk; i += 128) m = fmaxf(m, F.part[(row * F.nblk + i) * kPartStride]);
  m = warp_max(m);
  if (lane == 0) sh_red[warp] = m;
  __syncthreads();
  m = fmaxf(fmaxf(sh_red[0], sh_red[1]), fmaxf(sh_red[2], sh_red[3]));
  __syncthreads();
  // rotated-domain accumulator and sum of the packed part; thread = coordinate
  float acc = 0.f, lsum = 0.f;
  if (F.Sk > 0) {
    // eight partials per round: their loads are independent and in flight together (a loop that tests each
    // partial's maximum before loading the next spends one memory latency per partial)
    constexpr int kBatch = 8;
    for (int i0 = 0; i0 < F.nblk; i0 += kBatch) {
      float pm[kBatch], ps[kBatch], pv[kBatch];
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const int i = i0 + u < F.nblk ? i0 + u : F.nblk - 1;
        const float* pp = F.part + (row * F.nblk + i) * kPartStride;
        pm[u] = i0 + u < F.nblk ? pp[0] : -INFINITY;
        ps[u] = pp[1];
        pv[u] = pp[2 + tid];
      }
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        if (pm[u] != -INFINITY) {
          const float f = __expf(pm[u] - m);
          acc += pv[u] * f;
          lsum += ps[u] * f;
        }
      }
    }
  }
  sh_acc[tid] = acc;
  // window probabilities
  float wl = 0.f;
  for (int64_t w = tid; w < F.W; w += 128) {
    const float pw = __expf(sh_w[w] - m);
    sh_w[w] = pw;
    wl += pw;
  }
  wl = warp_sum(wl);
  if (lane == 0) sh_red[warp] = wl;
  __syncthreads();
  const float total = lsum + sh_red[0] + sh_red[1] + sh_red[2] + sh_red[3];
  // out[tid] = sum_j acc[j] Pi_v[j][tid] + sum_w p_w v_w[tid]
  float o = 0.f;
#pragma unroll 16
  for (int j = 0; j < kDimA; ++j) o = fmaf(sh_acc[j], __ldg(F.v_rotation + j * kDimA + tid), o);
  for (int64_t w = 0; w < F.W; ++w) o = fmaf(sh_w[w], load_elem<WDT>(F.v_window, wbase + w * F.ws_s + tid), o);
  F.out[row * kDimA + tid] = o / total;
  (void)sh_m; (void)sh_l;
}

}  // namespace

size_t decode_attention_workspace(int64_t B, int64_t Hq, int64_t Sq, int64_t Sk, int keys_per_block) {
  const int64_t rows = B * Hq * Sq;
  const int64_t nblk = Sk > 0 ? (Sk + keys_per_block - 1) / keys_per_block : 1;
  size_t q = ((size_t)rows * kDimA * sizeof(float) + 255) / 256 * 256;
  return q + (size_t)rows * nblk * kPartStride * sizeof(float);
}

template <int KB>
static int launch_decode_v(const DecodeParams& P, int vbits, unsigned blocks, cudaStream_t st) {
  switch (vbits) {
    case 1: k_decode_attn<KB, 1><<<blocks, kThreads, 0, st>>>(P); break;
    case 2: k_decode_attn<KB, 2><<<blocks, kThreads, 0, st>>>(P); break;
    case 3: k_decode_attn<KB, 3><<<blocks, kThreads, 0, st>>>(P); break;
    case 4: k_decode_attn<KB, 4><<<blocks, kThreads, 0, st>>>(P); break;
    case 5: k_decode_attn<KB, 5><<<blocks, kThreads, 0, st>>>(P); break;
    case 6: k_decode_attn<KB, 6><<<blocks, kThreads, 0, st>>>(P); break;
    case 7: k_decode_attn<KB, 7><<<blocks, kThreads, 0, st>>>(P); break;
    default: k_decode_attn<KB, 8><<<blocks, kThreads, 0, st>>>(P); break;
  }
  return check_launch();
}

// Keys per CTA such that the CTAs fill whole waves of `slots` resident CTAs: at least min_keys (the scratch is
// sized for blocks of min_keys), a multiple of 16.  With 8 KV heads and 131 072 keys, blocks of 2048 keys are
// 512 CTAs = 3.46 waves of 148, i.e. four rounds of which the last is half empty; 55 blocks of 2384 keys per head
// are 2.97 waves.
static int wave_keys_per_block(int64_t units, int64_t Sk, int min_keys, int slots) {
  const int64_t nblk_max = (Sk + min_keys - 1) / min_keys;
  if (units <= 0 || slots <= 0 || units * nblk_max <= slots) return min_keys;
  const int64_t waves = units * nblk_max / slots;
  int64_t nblk = waves * slots / units;
  if (nblk < 1) nblk = 1;
  int64_t kpb = (Sk + nblk - 1) / nblk;
  kpb = (kpb + 15) / 16 * 16;
  return (int)(kpb < min_keys ? min_keys : kpb);
}

static int device_sm_count() {
  static std::atomic<int> cached[64] = {};
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev >= 0 && dev < 64 && (n = cached[dev].load()) > 0) return n;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
  if (dev >= 0 && dev < 64) cached[dev].store(n);
  return n;
}

int decode_attention(const TqDecodeAttnJob& job, cudaStream_t st) {
  constexpr int kMinKeysPerBlock = 2048;          // decode_attention_workspace() sizes the partials for this
  const int kKeysPerBlock = wave_keys_per_block(job.B * job.Hkv, job.Sk, kMinKeysPerBlock, device_sm_count());
  const int64_t rows = job.B * job.Hq * job.Sq;
  const int nblk = job.Sk > 0 ? (int)((job.Sk + kKeysPerBlock - 1) / kKeysPerBlock) : 1;
  float* qrot = reinterpret_cast<float*>(job.workspace);
  const size_t qbytes = ((size_t)rows * kDimA * sizeof(float) + 255) / 256 * 256;
  float* part = reinterpret_cast<float*>(reinterpret_cast<char*>(job.workspace) + qbytes);
  int rc = TQ_OK;
  if (job.Sk > 0) {
    rc = simt_project(job.q, job.q_dtype, rows, kDimA, job.k_rotation_t, kDimA, qrot, st);
    if (rc != TQ_OK) return rc;
    DecodeParams P;
    P.qrot = qrot;
    P.k_idx = job.k_idx; P.k_norms = job.k_norms; P.v_idx = job.v_idx; P.v_norms = job.v_norms;
    P.k_codebook = job.k_codebook; P.v_codebook = job.v_codebook;
    P.part = part;
    P.B = job.B; P.Hq = job.Hq; P.Sq = job.Sq; P.Hkv = job.Hkv; P.Sk = job.Sk;
    P.scale = job.scale;
    P.nblk = nblk; P.keys_per_block = kKeysPerBlock;
    const unsigned blocks = (unsigned)(job.B * job.Hkv * nblk);
    switch (job.key_bits) {
      case 1: rc = launch_decode_v<1>(P, job.value_bits, blocks, st); break;
      case 2: rc = launch_decode_v<2>(P, job.value_bits, blocks, st); break;
      case 3: rc = launch_decode_v<3>(P, job.value_bits, blocks, st); break;
      case 4: rc = launch_decode_v<4>(P, job.value_bits, blocks, st); break;
      case 5: rc = launch_decode_v<5>(P, job.value_bits, blocks, st); break;
      case 6: rc = launch_decode_v<6>(P, job.value_bits, blocks, st); break;
      case 7: rc = launch_decode_v<7>(P, job.value_bits, blocks, st); break;
      default: rc = launch_decode_v<8>(P, job.value_bits, blocks, st); break;
    }
    if (rc != TQ_OK) return rc;
  }
  FinishParams F;
  F.q = job.q; F.q_dtype = job.q_dtype;
  F.part = part; F.nblk = nblk;
  F.v_rotation = job.v_rotation;
  F.k_window = job.k_window; F.v_window = job.v_window; F.window_dtype = job.window_dtype;
  F.W = job.k_window != nullptr ? job.W : 0;
  F.ws_b = job.wstride_b; F.ws_h = job.wstride_h; F.ws_s = job.wstride_s;
  F.B = job.B; F.Hq = job.Hq; F.Sq = job.Sq; F.Hkv = job.Hkv; F.Sk = job.Sk;
  F.scale = job.scale;
  F.out = job.out;
  const size_t smem = (size_t)(F.W > 0 ? F.W : 1) * sizeof(float);
  auto launch = [&](auto kern) {
    kern<<<(unsigned)rows, 128, smem, st>>>(F);
  };
  const int wdt = F.W > 0 ? job.window_dtype : TQ_F16;
#define TQ_FIN(QD, WD) launch(k_decode_finish<QD, WD>)
  if (job.q_dtype == TQ_F32) { if (wdt == TQ_F16) TQ_FIN(TQ_F32, TQ_F16); else if (wdt == TQ_BF16) TQ_FIN(TQ_F32, TQ_BF16); else TQ_FIN(TQ_F32, TQ_F32); }
  else if (job.q_dtype == TQ_F16) { if (wdt == TQ_F16) TQ_FIN(TQ_F16, TQ_F16); else if (wdt == TQ_BF16) TQ_FIN(TQ_F16, TQ_BF16); else TQ_FIN(TQ_F16, TQ_F32); }
  else { if (wdt == TQ_F16) TQ_FIN(TQ_BF16, TQ_F16); else if (wdt == TQ_BF16) TQ_FIN(TQ_BF16, TQ_BF16); else TQ_FIN(TQ_BF16, TQ_F32); }
#undef TQ_FIN
  return check_launch();
}

bool mma_score_eligible(const TqScoreJob& job) {
  if (force_simt()) return false;
  return job.D == kDimA && (((uintptr_t)job.idx_bytes) & 15u) == 0 && (((uintptr_t)job.norms) & 1u) == 0;
}

// logits (and the per-block softmax partials when stats != NULL) for a job whose queries are already rotated
int mma_score_keys_per_block(const TqScoreJob& job, int min_keys) {
  return wave_keys_per_block(job.B * job.Hkv, job.Sk, min_keys, 2 * device_sm_count());      // two CTAs per SM
}

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
