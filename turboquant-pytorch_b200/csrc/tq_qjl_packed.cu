// Packed storage of the MSE+QJL representation and the asymmetric scores straight from it.
//
// The reference stores per key  k_mse (fp16, 2D bytes) + signs (int8, D bytes) + ||r|| (fp16)  -- 770 bytes at
// head_dim 256, more than the 16-bit key itself.  The packed form keeps what those were computed from:
// the MSE indices bit-packed (D * bits / 8 bytes), one sign bit per coordinate (D / 8 bytes), ||x|| (fp32) and
// ||r|| (fp16): 102 bytes at head_dim 256 with a 2-bit MSE stage.
//
// Scores from the packed form:   <q, k_mse> = ||x|| <q Pi^T, c[idx]>,  so with the query side prepared once as
// [q Pi^T | sqrt(pi/2)/D * S q] (fp16 pieces hi + lo) a key's score is
//     ||x|| * sum_j (q Pi^T)_j c[idx_j]  +  ||r|| * sum_j (coef S q)_j sign_j
// -- two contractions over D whose key operands are assembled in registers from the packed bytes (centroid
// pieces from a shared table, signs from their bits), run as mma.sync.m16n8k16 like the packed-key logits of
// tq_attn_mma.cu: 16 keys x 8 queries per instruction.  The query operand of a block of 64 queries is laid out in
// shared memory in fragment order, so a thread fetches both pieces of a k-step with one 16-byte load.

#include "tq_common.cuh"
#include "tq_internal.h"

namespace tq {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kQB = 64;                        // queries per CTA
constexpr int kNT = kQB / 8;                   // 8-query tiles

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

// ---------------------------------------------------------------- pack
__global__ void __launch_bounds__(256) k_pack_mse_qjl(const uint8_t* __restrict__ idx, const int8_t* __restrict__ signs, int64_t n,
                                                      int D, int bits, uint8_t* __restrict__ idx_packed,
                                                      uint8_t* __restrict__ sign_bits) {
  const int ipb = 8 / bits;
  const int g = (D + ipb - 1) / ipb;
  const int sb = D / 8;
  const int64_t total = n * (int64_t)(g + sb);
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = e / (g + sb);
    const int col = (int)(e % (g + sb));
    if (col < g) {
      if (idx_packed == nullptr || idx == nullptr) continue;
      uint32_t byte = 0;
      for (int f = 0; f < ipb; ++f) {
        const int c = col * ipb + f;                                   // first index in the high bits; zero padding
        const uint32_t v = c < D ? idx[row * D + c] : 0u;
        byte |= v << (bits * (ipb - 1 - f));
      }
      idx_packed[row * g + col] = (uint8_t)byte;
    } else {
      if (sign_bits == nullptr || signs == nullptr) continue;
      const int b8 = col - g;
      uint32_t byte = 0;
      for (int f = 0; f < 8; ++f) byte |= (signs[row * D + b8 * 8 + f] > 0 ? 1u : 0u) << (7 - f);
      sign_bits[row * sb + b8] = (uint8_t)byte;
    }
  }
}

// ---------------------------------------------------------------- scores from the packed form
template <int BITS, int D>
struct PK {
  static constexpr int IPB = 8 / BITS;
  static constexpr int G = D / IPB;            // packed index bytes per key
  static constexpr int CB = G / 4;             // index bytes per thread and key (a quarter row = D / 4 coordinates)
  static constexpr int CW = CB / 4 > 0 ? CB / 4 : 1;
  static constexpr int SB = D / 8 / 4;         // sign bytes per thread and key: 4 (D = 128) or 8 (D = 256)
  static constexpr int SW = SB / 4;
  static constexpr int KS = D / 16;            // k-steps per half
  static constexpr int DQ = D / 4;             // coordinates per thread quarter
};

template <int BITS, int D>
__device__ __forceinline__ void load_idx_quarter(const uint8_t* row, int t, uint32_t (&w)[PK<BITS, D>::CW]) {
  constexpr int CB = PK<BITS, D>::CB;
  const uint8_t* p = row + t * CB;
  if constexpr (CB == 4) {
    w[0] = __ldg(reinterpret_cast<const uint32_t*>(p));
  } else if constexpr (CB == 8) {
    const uint2 v = __ldg(reinterpret_cast<const uint2*>(p));
    w[0] = v.x; w[1] = v.y;
  } else {
#pragma unroll
    for (int k = 0; k < CB / 16; ++k) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(p) + k);
      w[4 * k] = v.x; w[4 * k + 1] = v.y; w[4 * k + 2] = v.z; w[4 * k + 3] = v.w;
    }
  }
}

// shared address of the table entry of local coordinate u (0 .. D/4 - 1) of a thread's index quarter
template <int BITS, int D>
__device__ __forceinline__ uint32_t entry_addr(const uint32_t (&w)[PK<BITS, D>::CW], int u, uint32_t lut_base) {
  constexpr int IPB = PK<BITS, D>::IPB;
  constexpr uint32_t MASK = ((1u << BITS) - 1u) << 2;
  const int byte = u / IPB;
  const int sh = 8 * (byte & 3) + BITS * (IPB - 1 - (u % IPB));
  const uint32_t xw = w[byte >> 2];
  return lut_base + (sh >= 2 ? ((xw >> (sh - 2)) & MASK) : ((xw << (2 - sh)) & MASK));
}

struct PackedScoreParams {
  const float* qrot;          // (BH * Sq, D): q Pi^T
  const float* qproj;         // (BH * Sq, D): S q
  const uint8_t* idx; const uint8_t* sign_bits; const float* vec_norms; const uint16_t* rnorm;
  const float* codebook;
  float* scores;
  int64_t BH, Sq, Sk;
  float coef;
  int n_qblocks, n_ksplit;
};

// Shared memory: table (1 KB, 1024-byte aligned), then the query operand of this CTA's 64 queries:
// word (((nt * 2 KS + ks) * 32 + lane) * 4 + r), r = {hi k0, hi k1, lo k0, lo k1}: the B registers of
// 8-query tile nt, k-step ks (first KS steps: q Pi^T, then coef * S q), for lane (n = lane / 4, t = lane % 4)
// coordinates D/4 * t + 4 ks' + {0, 1} (k0) and + {2, 3} (k1).
template <int BITS, int D>
__global__ void __launch_bounds__(kThreads, 1) k_qjl_score_packed(PackedScoreParams P) {
  using C = PK<BITS, D>;
  constexpr int KS = C::KS, CW = C::CW, SW = C::SW, DQ = C::DQ;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = ((uint32_t)__cvta_generic_to_shared(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - (uint32_t)__cvta_generic_to_shared(smem_raw));
  uint32_t* lut = reinterpret_cast<uint32_t*>(gbase);                 // 256 entries (hi | lo << 16)
  uint32_t* sgn = lut + 256;                                          // 4 entries: +-1 pairs, index = (first << 1) | second
  uint4* qimg = reinterpret_cast<uint4*>(gbase + 2048);               // [kNT][2 KS][32]
  const uint32_t lut_base = base, sgn_base = base + 1024, img_base = base + 2048;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, t = lane & 3;
  const int split = blockIdx.x % P.n_ksplit;
  const int qb = (blockIdx.x / P.n_ksplit) % P.n_qblocks;
  const int64_t bh = blockIdx.x / ((int64_t)P.n_ksplit * P.n_qblocks);
  const int q0 = qb * kQB;
  {
    const float c = __ldg(P.codebook + kCentroidOff + threadIdx.x);
    const __half h = __float2half_rn(c);
    lut[threadIdx.x] = (uint32_t)__half_as_ushort(h) | ((uint32_t)__half_as_ushort(__float2half_rn(c - __half2float(h))) << 16);
    if (threadIdx.x < 4) {
      const uint32_t first = (threadIdx.x & 2) ? 0x3C00u : 0xBC00u, second = (threadIdx.x & 1) ? 0x3C00u : 0xBC00u;
      sgn[threadIdx.x] = first | (second << 16);
    }
  }
  // query operand: one 16-byte word group per (tile, k-step, lane)
  for (int e = threadIdx.x; e < kNT * 2 * KS * 32; e += kThreads) {
    const int ln = e & 31, ks = (e >> 5) % (2 * KS), nt = e / (64 * KS);
    const int n = ln >> 2, tt = ln & 3;
    const int q = q0 + nt * 8 + n;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (q < P.Sq) {
      const bool second = ks >= KS;
      const float* src = (second ? P.qproj : P.qrot) + (bh * P.Sq + q) * D + DQ * tt + 4 * (second ? ks - KS : ks);
      const float4 f = __ldg(reinterpret_cast<const float4*>(src));
      const float s = second ? P.coef : 1.0f;
      v[0] = f.x * s; v[1] = f.y * s; v[2] = f.z * s; v[3] = f.w * s;
    }
    uint32_t r[4];
    {
      const __half h0 = __float2half_rn(v[0]), h1 = __float2half_rn(v[1]), h2 = __float2half_rn(v[2]), h3 = __float2half_rn(v[3]);
      r[0] = (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16);
      r[1] = (uint32_t)__half_as_ushort(h2) | ((uint32_t)__half_as_ushort(h3) << 16);
      const __half l0 = __float2half_rn(v[0] - __half2float(h0)), l1 = __float2half_rn(v[1] - __half2float(h1));
      const __half l2 = __float2half_rn(v[2] - __half2float(h2)), l3 = __float2half_rn(v[3] - __half2float(h3));
      r[2] = (uint32_t)__half_as_ushort(l0) | ((uint32_t)__half_as_ushort(l1) << 16);
      r[3] = (uint32_t)__half_as_ushort(l2) | ((uint32_t)__half_as_ushort(l3) << 16);
    }
    qimg[e] = make_uint4(r[0], r[1], r[2], r[3]);
  }
  __syncthreads();
  // this CTA's keys: a contiguous split of the head's keys, in blocks of 16 per warp
  const int64_t per = ((P.Sk + P.n_ksplit - 1) / P.n_ksplit + 15) / 16 * 16;
  const int64_t s_begin = (int64_t)split * per;
  const int64_t s_end = min(s_begin + per, P.Sk);
  const uint8_t* idx = P.idx + bh * P.Sk * C::G;
  const uint8_t* sbits = P.sign_bits + bh * P.Sk * (D / 8);
  for (int64_t kb = s_begin + warp * 16; kb < s_end; kb += kWarps * 16) {
    const int64_t k_lo = kb + gid, k_hi = kb + 8 + gid;
    const int64_t c_lo = k_lo < s_end ? k_lo : s_begin, c_hi = k_hi < s_end ? k_hi : s_begin;
    uint32_t w0[CW], w1[CW], s0[SW], s1[SW];
    load_idx_quarter<BITS, D>(idx + c_lo * C::G, t, w0);
    load_idx_quarter<BITS, D>(idx + c_hi * C::G, t, w1);
    if constexpr (SW == 1) {
      s0[0] = __ldg(reinterpret_cast<const uint32_t*>(sbits + c_lo * (D / 8) + 4 * t));
      s1[0] = __ldg(reinterpret_cast<const uint32_t*>(sbits + c_hi * (D / 8) + 4 * t));
    } else {
      const uint2 a = __ldg(reinterpret_cast<const uint2*>(sbits + c_lo * (D / 8) + 8 * t));
      const uint2 b = __ldg(reinterpret_cast<const uint2*>(sbits + c_hi * (D / 8) + 8 * t));
      s0[0] = a.x; s0[1] = a.y; s1[0] = b.x; s1[1] = b.y;
    }
    const float vn_lo = __ldg(P.vec_norms + bh * P.Sk + c_lo), vn_hi = __ldg(P.vec_norms + bh * P.Sk + c_hi);
    const float rn_lo = __half2float(__ushort_as_half(__ldg(P.rnorm + bh * P.Sk + c_lo)));
    const float rn_hi = __half2float(__ushort_as_half(__ldg(P.rnorm + bh * P.Sk + c_hi)));
    float acc[kNT][4];
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
    // ---- sign half first: acc = sum_j (coef S q)_j sign_j  (signs are exact in fp16: one piece)
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      // local coordinates 4 ks .. 4 ks + 3 of the quarter: bits 7 - (u % 8) of byte u / 8, first coordinate highest
      const int byte = (4 * ks) / 8, hi_nib = ((4 * ks) % 8) == 0;
      const uint32_t b0 = (s0[byte >> 2] >> (8 * (byte & 3) + (hi_nib ? 4 : 0))) & 0xFu;
      const uint32_t b1 = (s1[byte >> 2] >> (8 * (byte & 3) + (hi_nib ? 4 : 0))) & 0xFu;
      const uint32_t a0 = lds_u32(sgn_base + ((b0 >> 2) << 2)), a2 = lds_u32(sgn_base + ((b0 & 3u) << 2));
      const uint32_t a1 = lds_u32(sgn_base + ((b1 >> 2) << 2)), a3 = lds_u32(sgn_base + ((b1 & 3u) << 2));
#pragma unroll
      for (int nt = 0; nt < kNT; ++nt) {
        const uint4 q = qimg[(nt * 2 * KS + KS + ks) * 32 + lane];
        mma_16816(acc[nt], a0, a1, a2, a3, q.x, q.y);
        mma_16816(acc[nt], a0, a1, a2, a3, q.z, q.w);
      }
    }
    // ---- weight by ||r|| / ||x|| so that the final multiplication by ||x|| gives ||r|| * (sign term)
    const float ratio_lo = vn_lo > 0.f ? rn_lo / vn_lo : 0.f, ratio_hi = vn_hi > 0.f ? rn_hi / vn_hi : 0.f;
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) {
      acc[nt][0] *= ratio_lo; acc[nt][1] *= ratio_lo; acc[nt][2] *= ratio_hi; acc[nt][3] *= ratio_hi;
    }
    // ---- MSE half: acc += sum_j (q Pi^T)_j c[idx_j], pieces hi.hi + hi.lo + lo.hi
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t e0[4], e1[4];
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        e0[p] = lds_u32(entry_addr<BITS, D>(w0, 4 * ks + p, lut_base));
        e1[p] = lds_u32(entry_addr<BITS, D>(w1, 4 * ks + p, lut_base));
      }
      const uint32_t h0 = __byte_perm(e0[0], e0[1], 0x5410), h2 = __byte_perm(e0[2], e0[3], 0x5410);
      const uint32_t h1 = __byte_perm(e1[0], e1[1], 0x5410), h3 = __byte_perm(e1[2], e1[3], 0x5410);
      const uint32_t l0 = __byte_perm(e0[0], e0[1], 0x7632), l2 = __byte_perm(e0[2], e0[3], 0x7632);
      const uint32_t l1 = __byte_perm(e1[0], e1[1], 0x7632), l3 = __byte_perm(e1[2], e1[3], 0x7632);
#pragma unroll
      for (int nt = 0; nt < kNT; ++nt) {
        const uint4 q = qimg[(nt * 2 * KS + ks) * 32 + lane];
        mma_16816(acc[nt], h0, h1, h2, h3, q.x, q.y);
        mma_16816(acc[nt], h0, h1, h2, h3, q.z, q.w);
        mma_16816(acc[nt], l0, l1, l2, l3, q.x, q.y);
      }
    }
    // ---- scores[q][key]: rows gid / gid + 8 are keys, columns 2t, 2t + 1 queries of tile nt
    float* out = P.scores + (bh * P.Sq) * P.Sk;
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) {
      const int qa = q0 + nt * 8 + 2 * t;
      if (k_lo < s_end) {
        if (qa < P.Sq) out[(int64_t)qa * P.Sk + k_lo] = acc[nt][0] * vn_lo;
        if (qa + 1 < P.Sq) out[(int64_t)(qa + 1) * P.Sk + k_lo] = acc[nt][1] * vn_lo;
      }
      if (k_hi < s_end) {
        if (qa < P.Sq) out[(int64_t)qa * P.Sk + k_hi] = acc[nt][2] * vn_hi;
        if (qa + 1 < P.Sq) out[(int64_t)(qa + 1) * P.Sk + k_hi] = acc[nt][3] * vn_hi;
      }
    }
  }
  (void)sgn; (void)img_base;
}

template <int D>
int launch_packed(const PackedScoreParams& P, int bits, unsigned grid, size_t smem, cudaStream_t st) {
  auto go = [&](auto kern) -> int {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { note_cuda_error((int)e); return TQ_ELAUNCH; }
    kern<<<grid, kThreads, smem, st>>>(P);
    return check_launch();
  };
  switch (bits) {
    case 1: return go(k_qjl_score_packed<1, D>);
    case 2: return go(k_qjl_score_packed<2, D>);
    case 3: return go(k_qjl_score_packed<3, D>);
    case 4: return go(k_qjl_score_packed<4, D>);
    case 5: return go(k_qjl_score_packed<5, D>);
    case 6: return go(k_qjl_score_packed<6, D>);
    case 7: return go(k_qjl_score_packed<7, D>);
    default: return go(k_qjl_score_packed<8, D>);
  }
}

}  // namespace

int pack_mse_qjl(const uint8_t* idx_u8, const int8_t* signs, int64_t n, int D, int bits, uint8_t* idx_packed,
                 uint8_t* sign_bits, cudaStream_t st) {
  const int ipb = 8 / bits;
  const int64_t total = n * (int64_t)((D + ipb - 1) / ipb + D / 8);
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  k_pack_mse_qjl<<<(unsigned)blocks, 256, 0, st>>>(idx_u8, signs, n, D, bits, idx_packed, sign_bits);
  return check_launch();
}

size_t qjl_scores_packed_workspace(int64_t BH, int64_t Sq, int D) {
  const size_t one = ((size_t)BH * Sq * D * sizeof(float) + 255) / 256 * 256;
  return 2 * one;
}

int qjl_scores_packed(const TqQjlPackedScoreJob& job, cudaStream_t st) {
  const int D = job.D;
  const int64_t rows = job.BH * job.Sq;
  const size_t one = ((size_t)rows * D * sizeof(float) + 255) / 256 * 256;
  float* qrot = reinterpret_cast<float*>(job.workspace);
  float* qproj = reinterpret_cast<float*>(reinterpret_cast<char*>(job.workspace) + one);
  int rc = simt_project(job.q, job.q_dtype, rows, D, job.rotation_t, D, qrot, st);
  if (rc != TQ_OK) return rc;
  rc = simt_project(job.q, job.q_dtype, rows, D, job.qjl_t, D, qproj, st);
  if (rc != TQ_OK) return rc;
  PackedScoreParams P;
  P.qrot = qrot; P.qproj = qproj;
  P.idx = job.idx_packed; P.sign_bits = job.sign_bits; P.vec_norms = job.vec_norms; P.rnorm = job.rnorm;
  P.codebook = job.codebook;
  P.scores = job.scores;
  P.BH = job.BH; P.Sq = job.Sq; P.Sk = job.Sk;
  P.coef = 1.2533141373155003f / (float)D;            // sqrt(pi / 2) / m, m = D rows of S
  P.n_qblocks = (int)((job.Sq + kQB - 1) / kQB);
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // enough key splits to fill the GPU, at least 256 keys each
  int64_t units = job.BH * P.n_qblocks;
  int64_t want = (2 * sms + units - 1) / units;
  int64_t max_split = (job.Sk + 255) / 256;
  if (want > max_split) want = max_split;
  if (want < 1) want = 1;
  P.n_ksplit = (int)want;
  const unsigned grid = (unsigned)(units * P.n_ksplit);
  const size_t smem = 2048 + (size_t)kNT * 2 * (D / 16) * 32 * 16 + 1024;
  return D == 128 ? launch_packed<128>(P, job.bits, grid, smem, st) : launch_packed<256>(P, job.bits, grid, smem, st);
}

}  // namespace tq
