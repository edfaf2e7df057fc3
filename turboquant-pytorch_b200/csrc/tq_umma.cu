// Tensor-core (tcgen05 / TMEM / TMA) kernels for the headline shape: head_dim 128,
// 16-bit vectors, packed indices.
//
// quantize: a persistent, warp-specialised CTA per SM walks a contiguous range of
// 128-vector tiles that may span several jobs (layers, K or V):
//   warp 0      TMA producer: x tiles (two 128x64 boxes, 128-byte swizzle) into a
//               4-stage shared-memory ring; the job's rotation image (64 KB) by bulk copy
//   warp 1      issues tcgen05.mma kind::f16, M=128 N=128 K=16: 8 k-steps against the
//               high fp16 piece of Pi and 8 against the low piece, all into ONE fp32
//               accumulator of 128 TMEM columns (4 accumulators rotate)
//   warps 2..17 epilogue, four warpgroups, one tile each: tcgen05.ld the accumulator
//               (thread = vector, registers = coordinates), sum of squares -> norm
//               (||Pi x|| = ||x||), scale, exact threshold search, bit pack, 16-byte stores
// x is exact in fp16/bf16 and Pi = hi + lo to ~2^-22 (lo sits in fp16 subnormals, which
// the tensor core handles), so the rotated values match an fp32 matmul to ~1e-8.
// kind::f16 wants A and B in the same format (a bf16 A against an fp16 B is an illegal
// instruction), so bf16 vectors run against three bf16 pieces of Pi (3 x 8 significant
// bits) and a 3-stage ring; fp16 vectors use two fp16 pieces and a 4-stage ring.
// Every mbarrier wait is bounded; on expiry the CTA raises an abort flag, records a
// status word, drains its own copies and leaves through the normal exit.

#include <cuda.h>

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "tq_common.cuh"
#include "tq_internal.h"

namespace tq {

namespace {

constexpr int kTileRows = 128;
constexpr int kDim = 128;
constexpr int kAccBufs = 4;
constexpr int kEpiWarps = 16;
constexpr int kThreads = 64 + kEpiWarps * 32;          // 576
constexpr uint32_t kTileBytes = kTileRows * kDim * 2;  // 32768
constexpr uint32_t kHalfBytes = kTileBytes / 2;        // one 64-column box
constexpr uint32_t kImageBytes = 5 * kTileBytes;       // fp16 hi, lo; then bf16 p0, p1, p2
constexpr int kMaxJobs = 96;
constexpr int kMaxCtas = 192;                          // upper bound of the grid (one CTA per SM)

// Timing-only switches that skip parts of the kernels exist only in builds made with
// -DTQ_ABLATION (build.py --ablate); the shipped library has none of these branches.
#ifdef TQ_ABLATION
#define TQ_ABL(batch, bits) (((batch).ablate & (bits)) != 0)
#else
#define TQ_ABL(batch, bits) false
#endif

// shared memory map (offsets from a 1024-byte aligned base)
template <bool BF16, bool WIDE = false>
struct Cfg {
  // x-tile ring: launches with wide codes give one stage to the look-up tables (their tiles take 1.7-2.5 us,
  // enough for a load to land with one tile of look-ahead less)
  static constexpr int kStages = (BF16 ? 3 : 4) - (WIDE ? 1 : 0);
  static constexpr int kPieces = BF16 ? 3 : 2;
  static constexpr uint32_t kPieceOff = BF16 ? 2 * kTileBytes : 0;            // offset of the pieces in the image
  static constexpr uint32_t kOffA = 0;
  static constexpr uint32_t kOffPi = kOffA + kStages * kTileBytes;
  // Narrow launches: 256 thresholds (fp32) per epilogue warpgroup.  Launches with wide codes: ONE set of
  // tables per CTA, shared by the four warpgroups and rebuilt at every job change (see the epilogue), every
  // entry stored once per lane so that random look-ups never collide in the banks:
  //   thresholds * 2^40 of 7/8-bit codes:        256 x 32 x 4 bytes   (6-bit codes: 64 x 32 x 4 bytes, same place),
  //   candidate index per cell of t (7/8 bits): 1025 x 32 x 1 byte    (four lanes share a word)
  static constexpr uint32_t kOffThr = kOffPi + kPieces * kTileBytes;
  static constexpr uint32_t kThrRegion = 1024;
  static constexpr uint32_t kOffCells = kOffThr + 32768;
  static constexpr uint32_t kOffBar = WIDE ? kOffCells + 32800 : kOffThr + 4 * kThrRegion;
  static constexpr uint32_t kSmemBytes = kOffBar + 256 + 1024;                // + alignment slack
};
static_assert(Cfg<false, true>::kSmemBytes <= 232448 && Cfg<true, true>::kSmemBytes <= 232448, "shared memory budget");

struct alignas(64) UmmaQuantJob {
  CUtensorMap tmap;          // (D, S, H, B) view of x, box 64 x 128 x 1 x 1, 128-byte swizzle
  const void* image;         // rotation image: hi piece then lo piece, swizzled K-major
  const float* codebook;
  uint8_t* idx_out;
  uint16_t* norms_out;
  int64_t S;
  int32_t H;
  int32_t tiles_per_slab;
  int32_t tile_begin;        // first global tile of this job
  int32_t bits;
  int32_t a_bf16;
  int32_t pad_;
};

struct UmmaQuantBatch {
  int32_t n_jobs;
  int32_t total_tiles;
  int32_t* status;           // device status word (may be null)
  int32_t ablate;            // -DTQ_ABLATION builds only (TQ_ABLATE): 1 skip stores, 2 skip the epilogue, 4 skip MMA,
                             // 32 half loads, 64 no loads, 256 / 512 skip the quantise / norm sweep
  int32_t pad_[3];
  int32_t cta_begin[kMaxCtas + 1];   // CTA c owns tiles [cta_begin[c], cta_begin[c + 1]): equal estimated cost, not equal count
  UmmaQuantJob jobs[kMaxJobs];
};

static_assert(sizeof(UmmaQuantBatch) < 32000, "kernel parameter space");

__device__ int g_umma_status;   // 0 = ok; otherwise (code << 16) | block

#include "tq_tc_ptx.cuh"

// Register copy of the job a role is working on.  The table lives in kernel-parameter space,
// where every field access with a run-time index is a slow dependent load; a role therefore
// reloads the fields only when its tile leaves the current job's range.
struct QuantJobView {
  int j = -1, begin = 0, end = 0;      // tiles [begin, end)
  int tps = 1, H = 1, bits = 0, g = 0; // tiles per slab, heads, code width, packed bytes per row
  int64_t S = 0;
  uint8_t* idx_out = nullptr;
  uint16_t* norms_out = nullptr;
  const float* codebook = nullptr;
  const void* image = nullptr;
  const CUtensorMap* tmap = nullptr;
};
// true when `tile` belongs to another job than the cached one (tiles only grow within a role)
__device__ __forceinline__ bool view_advance(const UmmaQuantBatch& b, int tile, QuantJobView& v) {
  if (v.j >= 0 && tile < v.end) return false;
  int j = v.j < 0 ? 0 : v.j;
  while (j + 1 < b.n_jobs && tile >= b.jobs[j + 1].tile_begin) ++j;
  const UmmaQuantJob& job = b.jobs[j];
  v.j = j;
  v.begin = job.tile_begin;
  v.end = (j + 1 < b.n_jobs) ? b.jobs[j + 1].tile_begin : b.total_tiles;
  v.tps = job.tiles_per_slab;
  v.H = job.H;
  v.bits = job.bits;
  v.g = kDim / (8 / job.bits);
  v.S = job.S;
  v.idx_out = job.idx_out;
  v.norms_out = job.norms_out;
  v.codebook = job.codebook;
  v.image = job.image;
  v.tmap = &job.tmap;
  return true;
}

// ---------------------------------------------------------------- epilogue
// One thread owns one vector (registers = coordinates).
// Generic (binary search) quantise sweep for codebooks without a search shortcut.  A thread
// owns all 128 coordinates of one vector; tmem_acc points at its first column.
template <int BITS>
__device__ __forceinline__ void quant_row_generic(uint32_t tmem_acc, float inv, const float* thr, uint8_t* idx_half,
                                                  bool valid) {
  constexpr int IPB = 8 / BITS;
  constexpr int BYTES_PER_CHUNK = 32 / IPB;     // packed bytes per 32 coordinates
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {
    float v[32];
    tmem_ld32(tmem_acc + c * 32, v);
    uint32_t words[BYTES_PER_CHUNK / 4 > 0 ? BYTES_PER_CHUNK / 4 : 1];
#pragma unroll
    for (int w = 0; w < BYTES_PER_CHUNK / 4; ++w) words[w] = 0u;
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      const float y = v[e] * inv;
      int lo = 0, hi = (1 << BITS) - 1;
#pragma unroll
      for (int step = 0; step < BITS; ++step) {
        const int mid = (lo + hi) >> 1;
        if (y > thr[mid]) lo = mid + 1; else hi = mid;
      }
      // coordinate e of this chunk -> byte e / IPB, field (IPB-1 - e % IPB) of that byte
      const int byte = e / IPB;
      const int shift = 8 * (byte & 3) + BITS * (IPB - 1 - (e % IPB));
      words[byte >> 2] |= (uint32_t)lo << shift;
    }
    if (valid) {
      if constexpr (BYTES_PER_CHUNK == 4) {
        *reinterpret_cast<uint32_t*>(idx_half + c * 4) = words[0];
      } else if constexpr (BYTES_PER_CHUNK == 8) {
        *reinterpret_cast<uint2*>(idx_half + c * 8) = make_uint2(words[0], words[1]);
      } else if constexpr (BYTES_PER_CHUNK == 16) {
        *reinterpret_cast<uint4*>(idx_half + c * 16) = make_uint4(words[0], words[1], words[2], words[3]);
      } else {
        *reinterpret_cast<uint4*>(idx_half + c * 32) = make_uint4(words[0], words[1], words[2], words[3]);
        *reinterpret_cast<uint4*>(idx_half + c * 32 + 16) = make_uint4(words[4], words[5], words[6], words[7]);
      }
    }
  }
}

// Codebooks without a verified shortcut (none of the Lloyd-Max codebooks): out of line, so that its
// registers and code do not weigh on the paths that run.
__device__ __noinline__ void quant_row_search(int bits, uint32_t tacc, float inv, const float* thr, uint8_t* idx_row,
                                              bool valid) {
  switch (bits) {
    case 1: quant_row_generic<1>(tacc, inv, thr, idx_row, valid); break;
    case 2: quant_row_generic<2>(tacc, inv, thr, idx_row, valid); break;
    case 3: quant_row_generic<3>(tacc, inv, thr, idx_row, valid); break;
    case 4: quant_row_generic<4>(tacc, inv, thr, idx_row, valid); break;
    case 5: quant_row_generic<5>(tacc, inv, thr, idx_row, valid); break;
    case 6: quant_row_generic<6>(tacc, inv, thr, idx_row, valid); break;
    case 7: quant_row_generic<7>(tacc, inv, thr, idx_row, valid); break;
    default: quant_row_generic<8>(tacc, inv, thr, idx_row, valid); break;
  }
}

// Search shortcut (see the codebook block): one cubic, one lane look-up of the candidate
// threshold, one compare.  Arithmetic is kept on the FMA pipe: the index is built as a
// float next to 2^23 and shifted into the packed word by an integer multiply-add; the
// 2^23 bit patterns that ride along are removed once per word as a constant.
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
  unsigned long long v;
  asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
  return v;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
// two fp32 fused multiply-adds in one instruction (sm_100): the same IEEE results per half as fmaf
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

struct Shortcut {
  float s, c1, c2, c3;
  float thr_lane_h;    // threshold[lane] * 2^40 (+inf past the last one)
  float s_inv, h_inv;  // per vector: s / (norm + 1e-8) and 2^40 / (norm + 1e-8)
};

// CH coordinates (16 here) per step: the loop body stays small enough to live in the
// instruction cache while four warps per scheduler run it out of phase.
// LDS: the candidate's threshold comes from a shared-memory table (thresholds times 2^40) instead of a
// lane look-up: codes with more than 31 thresholds whose cubic still brackets the index (6 bits).
// The table is stored once per lane ([64][32] floats, lane l reads column l: bank l, never a collision).
// thr_addr is the table's shared address plus 4 * lane minus 128 * 0x4B000000, so that the look-up
// address is one multiply-add on the bit pattern of u = 2^23 + e.
template <int BITS, int CH, bool LDS = false, bool LINEAR = false>
__device__ __forceinline__ void quant_chunk_words(const uint32_t (&raw)[CH], const Shortcut& sc, uint32_t thr_addr,
                                                  uint32_t (&acc)[(CH / (8 / BITS)) >= 4 ? (CH / (8 / BITS)) / 4 : 1]) {
  constexpr int IPB = 8 / BITS;
  constexpr int BYTES = CH / IPB;               // packed bytes for CH coordinates
  constexpr int WORDS = BYTES >= 4 ? BYTES / 4 : 1;
  constexpr uint32_t kMagicBits = 0x4B000000u;  // 2^23
#pragma unroll
  for (int w = 0; w < WORDS; ++w) acc[w] = 0u;
#pragma unroll
  for (int e = 0; e < CH; ++e) {
    // t and the compare both come straight from the raw accumulator: y = raw * inv is never
    // rounded on its own.  pf = sat((raw*inv - thr) * 2^40) is 1 when y > thr, 0 when y <= thr
    // (a positive difference below 2^-40 cannot occur between an fp32 product and an fp32
    // threshold unless they agree to ~1e-12, where either side is a valid answer).
    const float r = __uint_as_float(raw[e]);
    float t, pf;
    asm("fma.rn.sat.f32 %0, %1, %2, 0f3F000000;" : "=f"(t) : "f"(r), "f"(sc.s_inv));
    float u;
    if constexpr (LINEAR) {                      // c2 = c3 = 0: the same value as the cubic form below
      u = fmaf(sc.c1, t, 8388608.0f);
    } else {
      float q = fmaf(sc.c3, t, sc.c2);
      q = fmaf(q, t, sc.c1);
      u = fmaf(q, t, 8388608.0f);
    }
    float thr_h;
    if constexpr (LDS) {
      asm("ld.shared.f32 %0, [%1];" : "=f"(thr_h) : "r"(__float_as_uint(u) * 128u + thr_addr));
    } else {
      thr_h = __shfl_sync(0xffffffffu, sc.thr_lane_h, __float_as_int(u));
    }
    asm("fma.rn.sat.f32 %0, %1, %2, %3;" : "=f"(pf) : "f"(r), "f"(sc.h_inv), "f"(-thr_h));
    const float ui = u + pf;
    const int byte = e / IPB;
    const int shift = 8 * (byte & 3) + BITS * (IPB - 1 - (e % IPB));
    acc[byte >> 2] = __float_as_uint(ui) * (1u << shift) + acc[byte >> 2];
  }
  // remove the 2^23 bit patterns that rode along: sum(magic << shift) mod 2^32 per word
#pragma unroll
  for (int w = 0; w < WORDS; ++w) {
    uint32_t k = 0u;
#pragma unroll
    for (int e = 0; e < CH; ++e) {
      const int byte = e / IPB;
      if ((byte >> 2) == w) k += kMagicBits << (8 * (byte & 3) + BITS * (IPB - 1 - (e % IPB)));
    }
    acc[w] -= k;
  }
}

// Two 16-byte pieces of one row that sit side by side: one 32-byte store when the row allows it.  A warp's store touches 32 different rows either way, so the wider
// form halves the store traffic through the load/store unit.
__device__ __forceinline__ void store_index_pair(uint8_t* dst, const uint32_t (&a)[4], const uint32_t (&b)[4], bool wide) {
  if (wide) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "r"(a[0]), "r"(a[1]), "r"(a[2]),
                 "r"(a[3]), "r"(b[0]), "r"(b[1]), "r"(b[2]), "r"(b[3])
                 : "memory");
  } else {
    *reinterpret_cast<uint4*>(dst) = make_uint4(a[0], a[1], a[2], a[3]);
    *reinterpret_cast<uint4*>(dst + 16) = make_uint4(b[0], b[1], b[2], b[3]);
  }
}

template <int BITS, int CH, bool LDS = false, bool LINEAR = false>
__device__ __forceinline__ void quant_chunk_fast(const uint32_t (&raw)[CH], const Shortcut& sc, uint8_t* dst,
                                                 bool valid, uint32_t thr_addr = 0u) {
  constexpr int IPB = 8 / BITS;
  constexpr int BYTES = CH / IPB;               // packed bytes for CH coordinates
  constexpr int WORDS = BYTES >= 4 ? BYTES / 4 : 1;
  uint32_t acc[WORDS];
  quant_chunk_words<BITS, CH, LDS, LINEAR>(raw, sc, thr_addr, acc);
  if (valid) {
    if constexpr (BYTES == 2) {
      *reinterpret_cast<uint16_t*>(dst) = (uint16_t)acc[0];
    } else if constexpr (BYTES == 4) {
      *reinterpret_cast<uint32_t*>(dst) = acc[0];
    } else if constexpr (BYTES == 8) {
      *reinterpret_cast<uint2*>(dst) = make_uint2(acc[0], acc[1]);
    } else {
      *reinterpret_cast<uint4*>(dst) = make_uint4(acc[0], acc[1], acc[2], acc[3]);
    }
  }
}

// sum of squares on packed pairs: even coordinates accumulate in the low half, odd ones in the high half
template <int CH>
__device__ __forceinline__ unsigned long long ssq_chunk(const uint32_t (&raw)[CH], unsigned long long ssq2) {
#pragma unroll
  for (int e = 0; e < CH; e += 2) {
    const unsigned long long v = pack2(__uint_as_float(raw[e]), __uint_as_float(raw[e + 1]));
    ssq2 = fma2(v, v, ssq2);
  }
  return ssq2;
}

// A thread owns one vector: eight 16-column steps per sweep.  Two register buffers
// alternate so that a TMEM load is always in flight behind the math; the loops stay rolled
// (two inlined copies of the step body, one per buffer).
__device__ __forceinline__ float ssq_row_fast(uint32_t tacc, uint32_t (&a)[16], uint32_t (&b)[16]) {
  unsigned long long ssq2 = pack2(0.f, 0.f);
  tmem_issue16(tacc, a);
#pragma unroll 1
  for (int c = 0; c < 8; c += 2) {
    tmem_wait16(a); tmem_issue16(tacc + (c + 1) * 16, b);
    ssq2 = ssq_chunk<16>(a, ssq2);
    tmem_wait16(b); tmem_issue16(tacc + ((c + 2) & 7) * 16, a);      // wraps to step 0 for the second sweep
    ssq2 = ssq_chunk<16>(b, ssq2);
  }
  float lo, hi;
  unpack2(ssq2, lo, hi);
  return lo + hi;   // step 0 is in flight into `a`
}

template <int BITS, bool LDS = false, bool LINEAR = false>
__device__ __forceinline__ void quant_row_fast(uint32_t tacc, uint32_t (&a)[16], uint32_t (&b)[16], const Shortcut& sc,
                                               uint8_t* idx_row, bool valid, uint32_t thr_addr = 0u) {
  constexpr int BYTES = 16 / (8 / BITS);
  if constexpr (BYTES == 16) {                   // one-byte codes: 32 coordinates leave as one store
    const bool wide = (reinterpret_cast<uintptr_t>(idx_row) & 31u) == 0;
#pragma unroll 1
    for (int c = 0; c < 8; c += 2) {
      uint32_t wa[4], wb[4];
      tmem_wait16(a); tmem_issue16(tacc + (c + 1) * 16, b);
      quant_chunk_words<BITS, 16, LDS, LINEAR>(a, sc, thr_addr, wa);
      tmem_wait16(b);
      if (c + 2 < 8) tmem_issue16(tacc + (c + 2) * 16, a);
      quant_chunk_words<BITS, 16, LDS, LINEAR>(b, sc, thr_addr, wb);
      if (valid) store_index_pair(idx_row + c * 16, wa, wb, wide);
    }
  } else if constexpr (BYTES == 8) {             // 3- and 4-bit codes: a round (32 coordinates) leaves as one 16-byte store
#pragma unroll 1
    for (int c = 0; c < 8; c += 2) {
      uint32_t wa[2], wb[2];
      tmem_wait16(a); tmem_issue16(tacc + (c + 1) * 16, b);
      quant_chunk_words<BITS, 16, LDS, LINEAR>(a, sc, thr_addr, wa);
      tmem_wait16(b);
      if (c + 2 < 8) tmem_issue16(tacc + (c + 2) * 16, a);
      quant_chunk_words<BITS, 16, LDS, LINEAR>(b, sc, thr_addr, wb);
      if (valid) *reinterpret_cast<uint4*>(idx_row + c * 8) = make_uint4(wa[0], wa[1], wb[0], wb[1]);
    }
  } else if constexpr (BYTES == 4) {             // 2-bit codes: a round leaves as one 8-byte store
#pragma unroll 1
    for (int c = 0; c < 8; c += 2) {
      uint32_t wa[1], wb[1];
      tmem_wait16(a); tmem_issue16(tacc + (c + 1) * 16, b);
      quant_chunk_words<BITS, 16, LDS, LINEAR>(a, sc, thr_addr, wa);
      tmem_wait16(b);
      if (c + 2 < 8) tmem_issue16(tacc + (c + 2) * 16, a);
      quant_chunk_words<BITS, 16, LDS, LINEAR>(b, sc, thr_addr, wb);
      if (valid) *reinterpret_cast<uint2*>(idx_row + c * 4) = make_uint2(wa[0], wb[0]);
    }
  } else {
#pragma unroll 1
    for (int c = 0; c < 8; c += 2) {
      tmem_wait16(a); tmem_issue16(tacc + (c + 1) * 16, b);
      quant_chunk_fast<BITS, 16, LDS, LINEAR>(a, sc, idx_row + c * BYTES, valid, thr_addr);
      tmem_wait16(b);
      if (c + 2 < 8) tmem_issue16(tacc + (c + 2) * 16, a);
      quant_chunk_fast<BITS, 16, LDS, LINEAR>(b, sc, idx_row + (c + 1) * BYTES, valid, thr_addr);
    }
  }
}

// 7- and 8-bit codes (one index per byte): the candidate e comes from a byte table over the 1024 uniform
// cells of t, its threshold (times 2^40) from a second table, then the saturating-fma compare.  Random
// look-ups by 32 lanes cost a shared-memory wavefront per bank collision, and these two were the whole
// cost of the wide codes, so both tables are stored once per lane: a threshold look-up never collides
// (lane l reads bank l), a cell look-up only inside a group of four lanes that share a 32-bit word.
// cells_lane = table + lane - 32 * 0x4B000000 (mod 2^32), so that the cell address is one multiply-add
// on the bit pattern of u = 2^23 + cell;  thr_lane = table + 4 * lane.
__device__ __forceinline__ void quant_chunk_cells(const uint32_t (&raw)[16], const Shortcut& sc, uint32_t cells_lane,
                                                  uint32_t thr_lane, uint32_t (&acc)[4]) {
  acc[0] = acc[1] = acc[2] = acc[3] = 0u;
#pragma unroll
  for (int e = 0; e < 16; ++e) {
    const float r = __uint_as_float(raw[e]);
    float t, pf, thr_h;
    uint32_t e0;
    asm("fma.rn.sat.f32 %0, %1, %2, 0f3F000000;" : "=f"(t) : "f"(r), "f"(sc.s_inv));
    const float u = fmaf(t, 1024.0f, 8388608.0f);
    asm("ld.shared.u8 %0, [%1];" : "=r"(e0) : "r"(__float_as_uint(u) * 32u + cells_lane));
    asm("ld.shared.f32 %0, [%1];" : "=f"(thr_h) : "r"(e0 * 128u + thr_lane));
    asm("fma.rn.sat.f32 %0, %1, %2, %3;" : "=f"(pf) : "f"(r), "f"(sc.h_inv), "f"(-thr_h));
    const uint32_t idx = e0 + (__float_as_uint(pf) >> 29);          // pf is 1.0f (0x3F800000) or 0.0f
    acc[e >> 2] = idx * (1u << (8 * (e & 3))) + acc[e >> 2];
  }
}

__device__ __forceinline__ void quant_row_cells(uint32_t tacc, uint32_t (&a)[16], uint32_t (&b)[16], const Shortcut& sc,
                                                uint32_t cells_lane, uint32_t thr_lane, uint8_t* idx_row, bool valid) {
  const bool wide = (reinterpret_cast<uintptr_t>(idx_row) & 31u) == 0;
#pragma unroll 1
  for (int c = 0; c < 8; c += 2) {
    uint32_t wa[4], wb[4];
    tmem_wait16(a); tmem_issue16(tacc + (c + 1) * 16, b);
    quant_chunk_cells(a, sc, cells_lane, thr_lane, wa);
    tmem_wait16(b);
    if (c + 2 < 8) tmem_issue16(tacc + (c + 2) * 16, a);
    quant_chunk_cells(b, sc, cells_lane, thr_lane, wb);
    if (valid) store_index_pair(idx_row + c * 16, wa, wb, wide);
  }
}

// Rest of a role's walk after one of its waits ran out: only the two named barriers of every job
// change, so that the other warps of the group never wait for this one.  Out of line: cold.
__device__ __noinline__ void walk_job_barriers(const UmmaQuantBatch& batch, int job_index, int t0, int i, int step,
                                               int n_local, int bar_id, int threads) {
  QuantJobView job;
  job.j = job_index;
  job.end = (job_index + 1 < batch.n_jobs) ? batch.jobs[job_index + 1].tile_begin : batch.total_tiles;
  for (i += step; i < n_local; i += step)
    if (view_advance(batch, t0 + i, job)) {
      asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(threads) : "memory");
      asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(threads) : "memory");
    }
}

// WIDE: the launch holds a job with codes of 6 bits or more; the narrow instantiation carries none of
// the wide-code paths (its epilogue loop is sensitive to code size).
template <bool BF16, bool WIDE>
__global__ void __launch_bounds__(kThreads, 1) k_umma_quantize(const __grid_constant__ UmmaQuantBatch batch) {
  using C = Cfg<BF16, WIDE>;
  constexpr int kStages = C::kStages;
  constexpr int kPieces = C::kPieces;
  constexpr uint32_t kOffA = C::kOffA, kOffPi = C::kOffPi, kOffThr = C::kOffThr, kOffBar = C::kOffBar;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t a_smem = base + kOffA;
  const uint32_t pi_smem = base + kOffPi;
  float* thr_all = reinterpret_cast<float*>(gbase + kOffThr);
  const uint32_t bar0 = base + kOffBar;
  // barrier slots (8 bytes each)
  const uint32_t bar_full = bar0;                  // [kStages]
  const uint32_t bar_empty = bar0 + 8 * kStages;   // [kStages]
  const uint32_t bar_tfull = bar0 + 16 * kStages;  // [kAccBufs]
  const uint32_t bar_tempty = bar_tfull + 8 * kAccBufs;
  const uint32_t bar_pifull = bar_tempty + 8 * kAccBufs;
  const uint32_t bar_pifree = bar_pifull + 8;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + kOffBar + 200);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + kOffBar + 208);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = batch.cta_begin[blockIdx.x];
  const int t1 = batch.cta_begin[blockIdx.x + 1];
  const int n_local = t1 - t0;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) { mbar_init(bar_full + 8 * i, 1); mbar_init(bar_empty + 8 * i, 1); }
    for (int i = 0; i < kAccBufs; ++i) { mbar_init(bar_tfull + 8 * i, 1); mbar_init(bar_tempty + 8 * i, 4); }
    mbar_init(bar_pifull, 1);
    mbar_init(bar_pifree, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32((const void*)tmem_slot), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int pi_loads = 0;
      bool ok = true;
      QuantJobView job;
      for (int i = 0; i < n_local && ok; ++i) {
        const int t = t0 + i;
        if (view_advance(batch, t, job)) {
          if (pi_loads > 0) ok = mbar_wait(bar_pifree, (uint32_t)((pi_loads - 1) & 1), abort_flag);
          if (!ok) break;
          mbar_arrive_expect_tx(bar_pifull, kPieces * kTileBytes);
          const uint8_t* img = reinterpret_cast<const uint8_t*>(job.image) + C::kPieceOff;
#pragma unroll
          for (int p = 0; p < kPieces; ++p) bulk_load(pi_smem + p * kTileBytes, img + p * kTileBytes, kTileBytes, bar_pifull);
          ++pi_loads;
        }
        const int s = i % kStages;
        if (i >= kStages) {     // the stage is free once the MMAs of tile i - kStages are done (one commit serves both rings)
          const int d = i - kStages;
          ok = mbar_wait(bar_tfull + 8 * (d % kAccBufs), (uint32_t)((d / kAccBufs) & 1), abort_flag);
          if (!ok) break;
        }
        const int lt = t - job.begin;
        const int slab = lt / job.tps;
        const int row0 = (lt - slab * job.tps) * kTileRows;
        const int bb = slab / job.H, hh = slab - bb * job.H;
        if (TQ_ABL(batch, 64)) {
          mbar_arrive(bar_full + 8 * s);
        } else if (TQ_ABL(batch, 32)) {
          mbar_arrive_expect_tx(bar_full + 8 * s, kHalfBytes);
          tma_load_4d(a_smem + s * kTileBytes, job.tmap, 0, row0, hh, bb, bar_full + 8 * s);
        } else {
          mbar_arrive_expect_tx(bar_full + 8 * s, kTileBytes);
          tma_load_4d(a_smem + s * kTileBytes, job.tmap, 0, row0, hh, bb, bar_full + 8 * s);
          tma_load_4d(a_smem + s * kTileBytes + kHalfBytes, job.tmap, 64, row0, hh, bb, bar_full + 8 * s);
        }
      }
      if (!ok) {
        *abort_flag = 1;
        if (batch.status != nullptr) atomicCAS(batch.status, 0, (1 << 16) | (int)blockIdx.x);
      }
      // make sure none of this CTA's own copies is still in flight when it exits
      const int armed = n_local < kStages ? n_local : kStages;
      for (int k = 0; k < armed; ++k) {
        const int i = n_local - 1 - k;
        if (i >= 0) mbar_wait(bar_full + 8 * (i % kStages), (uint32_t)((i / kStages) & 1), abort_flag);
      }
      if (pi_loads > 0) mbar_wait(bar_pifull, (uint32_t)((pi_loads - 1) & 1), abort_flag);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // The whole warp runs the loop and the waits, so that tile counters and descriptor
    // bases are computed in converged code; one elected lane issues the MMAs and the commits.
    {
      int pi_uses = 0;
      bool ok = true;
      QuantJobView job;
      const uint32_t idesc = idesc_f16(BF16);
      const uint64_t b_base = smem_desc_sw128(pi_smem);
      for (int i = 0; i < n_local && ok; ++i) {
        const int t = t0 + i;
        if (view_advance(batch, t, job)) {
          ok = mbar_wait(bar_pifull, (uint32_t)(pi_uses & 1), abort_flag);
          ++pi_uses;
        }
        const int s = i % kStages, b = i % kAccBufs;
        ok = ok && mbar_wait(bar_full + 8 * s, (uint32_t)((i / kStages) & 1), abort_flag);
        ok = ok && mbar_wait(bar_tempty + 8 * b, (uint32_t)(((i / kAccBufs) & 1) ^ 1), abort_flag);
        ok = __all_sync(0xffffffffu, ok);        // lanes leave the loop together
        if (!ok) break;
        tc_fence_after();
        // The issue loop must stay a handful of instructions per MMA or the tensor pipe
        // starves: descriptors are a per-tile base plus compile-time offsets (the
        // start-address field counts 16-byte units and cannot carry out).
        const uint32_t d_tmem = tmem_base + (uint32_t)(b * 128);
        const uint64_t a_base = smem_desc_sw128(a_smem + s * kTileBytes);
        const bool last_of_job = i + 1 >= n_local || t + 1 >= job.end;
        if (elect_one()) {
          if (!TQ_ABL(batch, 4)) {
#pragma unroll
            for (int piece = 0; piece < kPieces; ++piece) {
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                constexpr uint32_t kUnit = 16;
                const uint64_t koff = (uint64_t)(((k >> 2) * kHalfBytes + (k & 3) * 32) / kUnit);
                const uint64_t poff = (uint64_t)((piece * kTileBytes) / kUnit);
                umma_f16(d_tmem, a_base + koff, b_base + poff + koff, idesc, (piece | k) != 0 ? 1u : 0u);
              }
            }
          }
          umma_commit(bar_tfull + 8 * b);      // one commit per tile: the epilogue and the producer both wait on it
          if (last_of_job) umma_commit(bar_pifree);
        }
        __syncwarp();
      }
      if (!ok && lane == 0) {
        *abort_flag = 1;
        if (batch.status != nullptr) atomicCAS(batch.status, 0, (2 << 16) | (int)blockIdx.x);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warpgroups
    // `ok` is made warp-uniform after each wait because the TMEM loads are warp-collective.  A warp
    // whose wait ran out leaves the working loop and walks the rest of its tiles for the named
    // barriers of the job changes alone, so that the other warps of the group never wait for it.
    const int ew = warp - 2;
    const int wg = ew >> 2;                    // 0..3, also the accumulator this group reads
    const int quarter = warp & 3;              // TMEM lanes this warp may touch: 32*quarter ..
    const int row = quarter * 32 + lane;
    float* thr = thr_all + wg * (C::kThrRegion / 4);                            // narrow launches: per warpgroup
    const int wg_tid = (ew & 3) * 32 + lane;
    const int ep_tid = threadIdx.x - 64;                                        // 0..511 over the epilogue warps
    int mode = 0;                               // 0 search, 1 cubic shortcut, 2 cell table
    bool ok = true;
    bool fast = false, fast_lds = false, linear = false;
    Shortcut sc = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    QuantJobView job;
    // Wide launches keep ONE set of tables per CTA.  Every epilogue warp walks the CTA's jobs in order,
    // one at a time: barrier (all warpgroups are done with the previous job's tables), rebuild, barrier.
    // All sixteen warps pass the same sequence of barriers whatever tiles they own, also after a wait ran
    // out and after their last tile, so nobody waits for a warp that has left.
    int seq_job = 0, last_job = -1;
    if constexpr (WIDE) {
      while (seq_job + 1 < batch.n_jobs && t0 >= batch.jobs[seq_job + 1].tile_begin) ++seq_job;
      last_job = seq_job;
      while (last_job + 1 < batch.n_jobs && t1 - 1 >= batch.jobs[last_job + 1].tile_begin) ++last_job;
      if (n_local <= 0) last_job = seq_job - 1;
      --seq_job;                                // nothing built yet
    }
    auto build_tables_up_to = [&](int target) {
      while (seq_job < target) {
        ++seq_job;
        asm volatile("bar.sync 5, 512;" ::: "memory");
        const float* cb = batch.jobs[seq_job].codebook;
        const int jbits = batch.jobs[seq_job].bits;
        const int jmode = (int)__ldg(cb + 512);
        if (jmode == 2 && jbits >= 5) {
          float* thr_rep = reinterpret_cast<float*>(gbase + C::kOffThr);        // [256][32]
          for (int k = ep_tid; k < 256 * 32; k += 512) thr_rep[k] = __ldg(cb + kThresholdOff + (k >> 5)) * 1099511627776.0f;
          const uint8_t* cell_e = reinterpret_cast<const uint8_t*>(cb + 528);
          uint32_t* cells_rep = reinterpret_cast<uint32_t*>(gbase + C::kOffCells);   // [1025][32 bytes]
          for (int k = ep_tid; k < 1025 * 8; k += 512) cells_rep[k] = (uint32_t)__ldg(cell_e + (k >> 3)) * 0x01010101u;
        } else if (jmode == 1 && jbits == 6) {
          float* thr6 = reinterpret_cast<float*>(gbase + C::kOffThr);           // [64][32]
          for (int k = ep_tid; k < 64 * 32; k += 512) thr6[k] = __ldg(cb + kThresholdOff + (k >> 5)) * 1099511627776.0f;
        }
        asm volatile("bar.sync 5, 512;" ::: "memory");
      }
    };
    int i = wg;
    for (; i < n_local; i += 4) {
      const int t = t0 + i;
      if (view_advance(batch, t, job)) {
        if constexpr (WIDE) {
          build_tables_up_to(job.j);
          mode = (int)__ldg(job.codebook + 512);
          fast = mode == 1 && job.bits <= 5;        // up to 31 thresholds: one per lane
          fast_lds = mode == 1 && job.bits == 6;    // 63 thresholds: the candidate's threshold comes from shared memory
          if ((mode == 2 && job.bits < 5) || (mode == 1 && job.bits > 6)) mode = 0;
        } else {
          asm volatile("bar.sync %0, 128;" ::"r"(wg + 1) : "memory");     // previous tile's readers are done
          mode = (int)__ldg(job.codebook + 512);
          fast = mode == 1 && job.bits <= 5;
          if (!fast) mode = 0;
          thr[wg_tid] = __ldg(job.codebook + kThresholdOff + wg_tid);
          thr[wg_tid + 128] = __ldg(job.codebook + kThresholdOff + 128 + wg_tid);
        }
        linear = __ldg(job.codebook + 518) == 1.0f;
        sc.s = __ldg(job.codebook + 513);
        sc.c1 = __ldg(job.codebook + 514);
        sc.c2 = __ldg(job.codebook + 515);
        sc.c3 = __ldg(job.codebook + 516);
        sc.thr_lane_h = __ldg(job.codebook + kThresholdOff + lane) * 1099511627776.0f;
        if constexpr (!WIDE) asm volatile("bar.sync %0, 128;" ::"r"(wg + 1) : "memory");
      }
      ok = __all_sync(0xffffffffu, mbar_wait(bar_tfull + 8 * wg, (uint32_t)((i / kAccBufs) & 1), abort_flag));
      if (!ok) break;
      tc_fence_after();
      const int lt = t - job.begin;
      const int slab = lt / job.tps;
      const int64_t s_row = (int64_t)(lt - slab * job.tps) * kTileRows + row;
      const bool valid = s_row < job.S && !TQ_ABL(batch, 1);
      const int64_t n = (int64_t)slab * job.S + s_row;
      const uint32_t tacc = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(wg * 128);
      uint8_t* idx_row = job.idx_out + n * (int64_t)job.g;
      if (!TQ_ABL(batch, 2)) {
        uint32_t ra[16], rb[16];
        float ssq;
        if (TQ_ABL(batch, 512)) { ssq = 1.0f; tmem_issue16(tacc, ra); }
        else ssq = ssq_row_fast(tacc, ra, rb);
        const float norm = __fsqrt_rn(ssq);
        const float inv = __fdiv_rn(1.0f, norm + 1e-8f);
        if (valid) job.norms_out[n] = __half_as_ushort(__float2half_rn(norm));
        sc.s_inv = sc.s * inv;
        sc.h_inv = 1099511627776.0f * inv;            // 2^40: exact scaling
        if (TQ_ABL(batch, 256)) {
          tmem_wait16(ra);
        } else if (WIDE && mode == 2) {
          if constexpr (WIDE)
            quant_row_cells(tacc, ra, rb, sc, base + C::kOffCells + (uint32_t)lane - 32u * 0x4B000000u,
                            base + C::kOffThr + 4u * (uint32_t)lane, idx_row, valid);
        } else if (WIDE && fast_lds) {
          if constexpr (WIDE)
            quant_row_fast<6, true>(tacc, ra, rb, sc, idx_row, valid, base + C::kOffThr + 4u * (uint32_t)lane - 128u * 0x4B000000u);
        } else if (fast) {
          switch (job.bits) {
            case 1:
              if (linear) quant_row_fast<1, false, true>(tacc, ra, rb, sc, idx_row, valid);
              else quant_row_fast<1>(tacc, ra, rb, sc, idx_row, valid);
              break;
            case 2:
              if (linear) quant_row_fast<2, false, true>(tacc, ra, rb, sc, idx_row, valid);
              else quant_row_fast<2>(tacc, ra, rb, sc, idx_row, valid);
              break;
            case 3:
              if (linear) quant_row_fast<3, false, true>(tacc, ra, rb, sc, idx_row, valid);
              else quant_row_fast<3>(tacc, ra, rb, sc, idx_row, valid);
              break;
            case 4: quant_row_fast<4>(tacc, ra, rb, sc, idx_row, valid); break;
            default: quant_row_fast<5>(tacc, ra, rb, sc, idx_row, valid); break;
          }
        } else {
          tmem_wait16(ra);                       // the norm sweep left a load in flight
          // wide launches have no plain threshold table in shared memory: the search reads the codebook block
          quant_row_search(job.bits, tacc, inv, WIDE ? job.codebook + kThresholdOff : thr, idx_row, valid);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + 8 * wg);
    }
    if (!ok && lane == 0) {
      *abort_flag = 1;
      if (batch.status != nullptr) atomicCAS(batch.status, 0, (3 << 16) | (int)blockIdx.x);
    }
    if constexpr (WIDE) {
      build_tables_up_to(last_job);              // the rest of the CTA's job sequence: barriers for the others
    } else {
      if (!ok) walk_job_barriers(batch, job.j, t0, i, 4, n_local, wg + 1, 128);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------- dequantize
// unpack + centroid lookup + inverse rotation + rescale, head_dim 128, packed indices.
// Each of NWG warpgroups owns one A buffer and one TMEM accumulator and alternates
// between expanding a tile (packed indices -> fp16 centroid pieces written straight
// into the swizzled K-major operand layout) and draining the previous result (TMEM ->
// x norm -> cache dtype -> 16-byte stores).  Warp 1 issues the MMAs, warp 0 brings in
// the rotation image when the job changes.  16-bit outputs need one pass (c_hi . Pi_hi,
// error ~3e-4 of a 2e-3 budget); fp32 output takes three (hi.hi + lo.hi + hi.lo ~ 2^-21).
struct alignas(64) UmmaDeqJob {
  CUtensorMap out_map;       // 16-bit outputs: (D, S, H, B) view of out, box 64 x 128, 128-byte swizzle
  const uint8_t* idx;
  const uint16_t* norms;
  const void* image;         // image of Pi^T
  const float* codebook;
  void* out;
  int64_t S;
  int64_t os_b, os_h, os_s;  // output strides in elements
  int32_t H;
  int32_t tiles_per_slab;
  int32_t tile_begin;
  int32_t bits;
  int32_t out_dtype;
  int32_t pad_;
};
constexpr int kMaxDeqJobs = 96;
struct UmmaDeqBatch {
  int32_t n_jobs;
  int32_t total_tiles;
  int32_t* status;
  int32_t ablate;            // -DTQ_ABLATION builds only (TQ_ABLATE): 1 skip stores, 2 skip expansion, 4 skip MMA, 8 skip the drain arithmetic
  int32_t pad_[3];
  int32_t cta_begin[kMaxCtas + 1];   // tiles [cta_begin[c], cta_begin[c + 1]) belong to CTA c (equal estimated cost)
  UmmaDeqJob jobs[kMaxDeqJobs];
};
static_assert(sizeof(UmmaDeqBatch) < 32000, "kernel parameter space");

// Decoupled pipeline: producer (bulk copies of packed tiles) -> 8 expander warps (packed
// bytes -> fp16 centroid pieces in the swizzled operand layout) -> MMA warp -> 8 drain warps
// (TMEM -> x norm -> cache dtype -> 16-byte stores).  Each stage has its own ring, so global
// load latency, expansion, tensor work and stores all overlap across tiles.
// NARROW: every job of the launch has codes of at most 4 bits, so a packed tile is at most
// 8 KB; the space saved buys a deeper packed ring and a third operand stage.
template <bool OUT32, bool NARROW>
struct DCfg {
  static constexpr int kPk = NARROW ? 4 : (OUT32 ? 2 : 3); // packed-tile ring
  static constexpr int kNA = (NARROW && !OUT32) ? 3 : 2;   // operand ring
  static constexpr int kNT = 4;                            // TMEM accumulators
  static constexpr int kPiecesA = OUT32 ? 2 : 1;
  static constexpr int kPiecesB = OUT32 ? 2 : 1;
  static constexpr int kExpWarps = 8, kDrainWarps = 8;
  static constexpr int kThreadsD = 64 + 32 * (kExpWarps + kDrainWarps);     // 576
  static constexpr uint32_t kPkBytes = NARROW ? 8192 : 16384;   // 128 rows x up to 64 / 128 packed bytes
  static constexpr uint32_t kOffA = 0;
  static constexpr uint32_t kOffPi = kOffA + kNA * kPiecesA * kTileBytes;
  static constexpr uint32_t kOffPk = kOffPi + kPiecesB * kTileBytes;
  static constexpr uint32_t kOffStage = kOffPk + kPk * kPkBytes;           // 16-bit outputs: one tile per drain group
  // 16-bit outputs of wide codes: replicated look-up table (see expand_half_wide16), 16 KB
  static constexpr bool kWide16 = !OUT32 && !NARROW;
  static constexpr uint32_t kOffLut16 = kOffStage + (OUT32 ? 0u : 2u * kTileBytes);
  static constexpr uint32_t kOffBar = kOffLut16 + (kWide16 ? 16384u : 0u);
  static constexpr uint32_t kSmemBytes = kOffBar + 256 + 1024;
};
// + 1 KB of static shared memory for the centroid look-up table
static_assert(DCfg<false, false>::kSmemBytes + 1024 <= 232448 && DCfg<true, false>::kSmemBytes + 1024 <= 232448 &&
              DCfg<false, true>::kSmemBytes + 1024 <= 232448 && DCfg<true, true>::kSmemBytes + 1024 <= 232448,
              "shared memory budget");

// Register copy of the current job (see QuantJobView).
struct DeqJobView {
  int j = -1, begin = 0, end = 0;
  int tps = 1, H = 1, bits = 0, g = 0, out_dtype = 0;
  int64_t S = 0, os_b = 0, os_h = 0, os_s = 0;
  const uint8_t* idx = nullptr;
  const uint16_t* norms = nullptr;
  const float* codebook = nullptr;
  const void* image = nullptr;
  void* out = nullptr;
  const CUtensorMap* out_map = nullptr;
};
__device__ __forceinline__ bool view_advance(const UmmaDeqBatch& b, int tile, DeqJobView& v) {
  if (v.j >= 0 && tile < v.end) return false;
  int j = v.j < 0 ? 0 : v.j;
  while (j + 1 < b.n_jobs && tile >= b.jobs[j + 1].tile_begin) ++j;
  const UmmaDeqJob& job = b.jobs[j];
  v.j = j;
  v.begin = job.tile_begin;
  v.end = (j + 1 < b.n_jobs) ? b.jobs[j + 1].tile_begin : b.total_tiles;
  v.tps = job.tiles_per_slab;
  v.H = job.H;
  v.bits = job.bits;
  v.g = kDim / (8 / job.bits);
  v.out_dtype = job.out_dtype;
  v.S = job.S; v.os_b = job.os_b; v.os_h = job.os_h; v.os_s = job.os_s;
  v.idx = job.idx;
  v.norms = job.norms;
  v.codebook = job.codebook;
  v.image = job.image;
  v.out = job.out;
  v.out_map = &job.out_map;
  return true;
}

#include "tq_tc_expand.cuh"

// The TMEM load is warp-collective: every lane of the warp must come through here, rows
// past the end of a slab included; `valid` only guards the stores.
template <int ODT>
__device__ __forceinline__ void drain_row(uint32_t tacc, float nv, void* out_row, bool valid) {
  uint32_t a[16], b[16];
  tmem_issue16(tacc, a);
#pragma unroll 1
  for (int c = 0; c < 8; c += 2) {
#pragma unroll
    for (int hb = 0; hb < 2; ++hb) {
      uint32_t (&cur)[16] = hb ? b : a;
      uint32_t (&nxt)[16] = hb ? a : b;
      tmem_wait16(cur);
      if (c + hb + 1 < 8) tmem_issue16(tacc + (c + hb + 1) * 16, nxt);
      if (valid) {
        float v[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = __uint_as_float(cur[e]) * nv;
        if constexpr (ODT == TQ_F32) {
          float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(out_row) + (c + hb) * 16);
#pragma unroll
          for (int e = 0; e < 4; ++e) o[e] = make_float4(v[4 * e], v[4 * e + 1], v[4 * e + 2], v[4 * e + 3]);
        } else {
          uint32_t pk[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            if constexpr (ODT == TQ_F16) {
              __half2 h = __floats2half2_rn(v[2 * e], v[2 * e + 1]);
              pk[e] = *reinterpret_cast<uint32_t*>(&h);
            } else {
              __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
              pk[e] = *reinterpret_cast<uint32_t*>(&h);
            }
          }
          uint4* o = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(out_row) + (c + hb) * 16);
          o[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          o[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        }
      }
    }
  }
}

// 16-bit outputs: scale, convert and write the row into a staging tile laid out like an
// operand tile (128-byte swizzle), from where one TMA store writes whole 128-byte lines to
// global memory; rows past the end of a slab are clipped by the tensor map.
template <int ODT>
__device__ __forceinline__ void drain_row_staged(uint32_t tacc, float nv, uint32_t stage, int row) {
  uint32_t a[16], b[16];
  tmem_issue16(tacc, a);
#pragma unroll 1
  for (int c = 0; c < 8; c += 2) {
#pragma unroll
    for (int hb = 0; hb < 2; ++hb) {
      uint32_t (&cur)[16] = hb ? b : a;
      uint32_t (&nxt)[16] = hb ? a : b;
      tmem_wait16(cur);
      if (c + hb + 1 < 8) tmem_issue16(tacc + (c + hb + 1) * 16, nxt);
      uint32_t pk[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float v0 = __uint_as_float(cur[2 * e]) * nv, v1 = __uint_as_float(cur[2 * e + 1]) * nv;
        if constexpr (ODT == TQ_F16) {
          __half2 h = __floats2half2_rn(v0, v1);
          pk[e] = *reinterpret_cast<uint32_t*>(&h);
        } else {
          __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
          pk[e] = *reinterpret_cast<uint32_t*>(&h);
        }
      }
      const int q0 = (c + hb) * 2;               // first 16-byte chunk of this step, 0..15
      const uint32_t half_base = stage + (uint32_t)(q0 >> 3) * kHalfBytes + (uint32_t)row * 128u;
      st_shared_v4(half_base + (uint32_t)((((q0 & 7)) ^ (row & 7)) << 4), pk[0], pk[1], pk[2], pk[3]);
      st_shared_v4(half_base + (uint32_t)((((q0 & 7) + 1) ^ (row & 7)) << 4), pk[4], pk[5], pk[6], pk[7]);
    }
  }
}

__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map),
               "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}

template <bool OUT32, bool NARROW>
__global__ void __launch_bounds__(DCfg<OUT32, NARROW>::kThreadsD, 1) k_umma_dequantize(const __grid_constant__ UmmaDeqBatch batch) {
  using C = DCfg<OUT32, NARROW>;
  constexpr int kPk = C::kPk, kNA = C::kNA, kNT = C::kNT;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t a_smem = base + C::kOffA;
  const uint32_t pi_smem = base + C::kOffPi;
  const uint32_t pk_smem = base + C::kOffPk;
  __shared__ uint32_t lut[256];                           // static: look-ups compile to [register + constant]
  const uint32_t bar0 = base + C::kOffBar;
  const uint32_t bar_pkfull = bar0;                       // [kPk] producer -> expanders
  const uint32_t bar_pkempty = bar_pkfull + 8 * kPk;      // [kPk] expanders (256 arrivals) -> producer
  const uint32_t bar_afull = bar_pkempty + 8 * kPk;       // [kNA] expanders (256 arrivals) -> MMA
  const uint32_t bar_aempty = bar_afull + 8 * kNA;        // [kNA] MMA commit -> expanders
  const uint32_t bar_tfull = bar_aempty + 8 * kNA;        // [kNT] MMA commit -> drain
  const uint32_t bar_tempty = bar_tfull + 8 * kNT;        // [kNT] drain (4 arrivals) -> MMA
  const uint32_t bar_pifull = bar_tempty + 8 * kNT;
  const uint32_t bar_pifree = bar_pifull + 8;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + C::kOffBar + 200);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + C::kOffBar + 208);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = batch.cta_begin[blockIdx.x];
  const int t1 = batch.cta_begin[blockIdx.x + 1];
  const int n_local = t1 - t0;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kPk; ++i) { mbar_init(bar_pkfull + 8 * i, 1); mbar_init(bar_pkempty + 8 * i, 256); }
    for (int i = 0; i < kNA; ++i) { mbar_init(bar_afull + 8 * i, 256); mbar_init(bar_aempty + 8 * i, 1); }
    for (int i = 0; i < kNT; ++i) { mbar_init(bar_tfull + 8 * i, 1); mbar_init(bar_tempty + 8 * i, 4); }
    mbar_init(bar_pifull, 1);
    mbar_init(bar_pifree, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32((const void*)tmem_slot), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---- producer: rotation image on job change, packed tiles into the ring
    if (lane == 0) {
      int pi_loads = 0;
      bool ok = true;
      DeqJobView job;
      for (int i = 0; i < n_local && ok; ++i) {
        const int t = t0 + i;
        if (view_advance(batch, t, job)) {
          if (pi_loads > 0) ok = mbar_wait(bar_pifree, (uint32_t)((pi_loads - 1) & 1), abort_flag);
          if (!ok) break;
          mbar_arrive_expect_tx(bar_pifull, C::kPiecesB * kTileBytes);
          const uint8_t* img = reinterpret_cast<const uint8_t*>(job.image);
#pragma unroll
          for (int p = 0; p < C::kPiecesB; ++p) bulk_load(pi_smem + p * kTileBytes, img + p * kTileBytes, kTileBytes, bar_pifull);
          ++pi_loads;
        }
        const int s = i % kPk;
        ok = mbar_wait(bar_pkempty + 8 * s, (uint32_t)(((i / kPk) & 1) ^ 1), abort_flag);
        if (!ok) break;
        const int lt = t - job.begin;
        const int slab = lt / job.tps;
        const int64_t s0 = (int64_t)(lt - slab * job.tps) * kTileRows;
        const int64_t rows = (job.S - s0) < kTileRows ? (job.S - s0) : kTileRows;
        const int g = job.g;
        const uint32_t bytes = (uint32_t)(rows * g);
        mbar_arrive_expect_tx(bar_pkfull + 8 * s, bytes);
        bulk_load(pk_smem + s * C::kPkBytes, job.idx + ((int64_t)slab * job.S + s0) * g, bytes, bar_pkfull + 8 * s);
      }
      if (!ok) {
        *abort_flag = 1;
        if (batch.status != nullptr) atomicCAS(batch.status, 0, (4 << 16) | (int)blockIdx.x);
      }
      const int armed = n_local < kPk ? n_local : kPk;
      for (int k = 0; k < armed; ++k) {
        const int i = n_local - 1 - k;
        if (i >= 0) mbar_wait(bar_pkfull + 8 * (i % kPk), (uint32_t)((i / kPk) & 1), abort_flag);
      }
      if (pi_loads > 0) mbar_wait(bar_pifull, (uint32_t)((pi_loads - 1) & 1), abort_flag);
    }
  } else if (warp == 1) {
    // ---- MMA issuer
    if (lane == 0) {
      int pi_uses = 0;
      bool ok = true;
      const uint32_t idesc = idesc_f16(false);
      DeqJobView job;
      for (int i = 0; i < n_local && ok; ++i) {
        const int t = t0 + i;
        if (view_advance(batch, t, job)) {
          ok = mbar_wait(bar_pifull, (uint32_t)(pi_uses & 1), abort_flag);
          if (!ok) break;
          ++pi_uses;
        }
        const int a = i % kNA, b = i % kNT;
        ok = mbar_wait(bar_afull + 8 * a, (uint32_t)((i / kNA) & 1), abort_flag);
        if (!ok) break;
        ok = mbar_wait(bar_tempty + 8 * b, (uint32_t)(((i / kNT) & 1) ^ 1), abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(b * 128);
        const uint64_t a_base = smem_desc_sw128(a_smem + a * C::kPiecesA * kTileBytes);
        const uint64_t b_base = smem_desc_sw128(pi_smem);
        constexpr int kPasses = OUT32 ? 3 : 1;      // hi.hi [, lo.hi, hi.lo]
        if (!TQ_ABL(batch, 4)) {
#pragma unroll
          for (int pass = 0; pass < kPasses; ++pass) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              // descriptor = per-tile base + compile-time offset in 16-byte units
              const uint64_t koff = (uint64_t)(((k >> 2) * kHalfBytes + (k & 3) * 32) / 16);
              const uint64_t pa = (uint64_t)(((pass == 1) ? kTileBytes : 0u) / 16);
              const uint64_t pb = (uint64_t)(((pass == 2) ? kTileBytes : 0u) / 16);
              umma_f16(d_tmem, a_base + pa + koff, b_base + pb + koff, idesc, (pass | k) != 0 ? 1u : 0u);
            }
          }
        }
        umma_commit(bar_tfull + 8 * b);      // one commit per tile: drain and expanders both wait on it
        if (i + 1 >= n_local || t + 1 >= job.end) umma_commit(bar_pifree);    // last tile of this job here
      }
      if (!ok) {
        *abort_flag = 1;
        if (batch.status != nullptr) atomicCAS(batch.status, 0, (5 << 16) | (int)blockIdx.x);
      }
    }
  } else if (warp < 2 + C::kExpWarps) {
    // ---- expanders: 256 threads, one half row each.  A warp whose wait ran out leaves the working
    // loop and walks on for the job-change barriers alone (see the quantize epilogue).
    const int et = threadIdx.x - 64;             // 0..255
    // a quarter warp = four consecutive rows x both k-halves: with the chunk order of expand_order() its packed
    // loads and its operand stores are free of bank conflicts
    const int row = (et >> 5) * 16 + (lane >> 1), half = lane & 1;
    const uint32_t lut16_lane = base + C::kOffLut16 + 4u * (uint32_t)lane;          // up to 7 bits: a copy per lane
    const uint32_t lut16_pair = base + C::kOffLut16 + 4u * (uint32_t)(lane >> 1);   // 8 bits: a copy per lane pair
    bool ok = true;
    DeqJobView job;
    int i = 0;
    for (; i < n_local; ++i) {
      const int t = t0 + i;
      if (view_advance(batch, t, job)) {
        asm volatile("bar.sync 1, 256;" ::: "memory");       // everyone is past the previous tile's look-ups
        const float c = __ldg(job.codebook + kCentroidOff + et);
        const __half h = __float2half_rn(c);
        const __half l = __float2half_rn(c - __half2float(h));
        lut[et] = (uint32_t)__half_as_ushort(h) | ((uint32_t)__half_as_ushort(l) << 16);
        if constexpr (C::kWide16) {
          if (job.bits >= 5) {                  // entry `et` (fp16 bits in both halves): 32 copies, or 16 for 8-bit codes
            const uint32_t hh = (uint32_t)__half_as_ushort(h) * 0x00010001u;
            if (job.bits == 8) {
              uint32_t* copies = reinterpret_cast<uint32_t*>(gbase + C::kOffLut16) + et * 16;
#pragma unroll
              for (int k = 0; k < 16; ++k) copies[k] = hh;
            } else if (et < 128) {
              uint32_t* copies = reinterpret_cast<uint32_t*>(gbase + C::kOffLut16) + et * 32;
#pragma unroll
              for (int k = 0; k < 32; ++k) copies[(k + lane) & 31] = hh;     // rotated: the warp's stores spread over the banks
            }
          }
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
      }
      const int s = i % kPk, a = i % kNA;
      ok = mbar_wait(bar_pkfull + 8 * s, (uint32_t)((i / kPk) & 1), abort_flag);
      if (ok && i >= kNA) {     // the operand stage is free once the MMAs of tile i - kNA are done
        const int d = i - kNA;
        ok = mbar_wait(bar_tfull + 8 * (d % kNT), (uint32_t)((d / kNT) & 1), abort_flag);
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const int lt = t - job.begin;
      const int slab = lt / job.tps;
      const int64_t s_row = (int64_t)(lt - slab * job.tps) * kTileRows + row;
      if (s_row < job.S && !TQ_ABL(batch, 2)) {
        const int g = job.g;
        const uint32_t src = pk_smem + s * C::kPkBytes + (uint32_t)(row * g + half * (g >> 1));
        const uint32_t a_stage = a_smem + a * C::kPiecesA * kTileBytes;
        switch (job.bits) {
          case 1: expand_half<1, C::kPiecesA>(src, lut, a_stage, row, half); break;
          case 2: expand_half<2, C::kPiecesA>(src, lut, a_stage, row, half); break;
          case 3: expand_half<3, C::kPiecesA>(src, lut, a_stage, row, half); break;
          case 4: expand_half<4, C::kPiecesA>(src, lut, a_stage, row, half); break;
          case 5:
            if constexpr (C::kWide16) expand_half_wide16<5>(src, lut16_lane, a_stage, row, half);
            else expand_half<5, C::kPiecesA>(src, lut, a_stage, row, half);
            break;
          case 6:
            if constexpr (C::kWide16) expand_half_wide16<6>(src, lut16_lane, a_stage, row, half);
            else expand_half<6, C::kPiecesA>(src, lut, a_stage, row, half);
            break;
          case 7:
            if constexpr (C::kWide16) expand_half_wide16<7>(src, lut16_lane, a_stage, row, half);
            else expand_half<7, C::kPiecesA>(src, lut, a_stage, row, half);
            break;
          default:
            if constexpr (C::kWide16) expand_half_wide16<8>(src, lut16_pair, a_stage, row, half);
            else expand_half<8, C::kPiecesA>(src, lut, a_stage, row, half);
            break;
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // operand writes -> visible to the tensor core
      mbar_arrive(bar_afull + 8 * a);
      mbar_arrive(bar_pkempty + 8 * s);
    }
    if (!ok) {
      if (lane == 0) {
        *abort_flag = 1;
        if (batch.status != nullptr) atomicCAS(batch.status, 0, (6 << 16) | (int)blockIdx.x);
      }
      for (++i; i < n_local; ++i)
        if (view_advance(batch, t0 + i, job)) {
          asm volatile("bar.sync 1, 256;" ::: "memory");
          asm volatile("bar.sync 1, 256;" ::: "memory");
        }
    }
  } else {
    // ---- drain: two warpgroups, alternate tiles.  `ok` is warp-uniform; a warp whose wait ran out
    // leaves the working loop and still passes the two named barriers of every remaining tile of its group.
    const int dw = warp - (2 + C::kExpWarps);    // 0..7
    const int wg = dw >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int wg_tid = (dw & 3) * 32 + lane;
    const uint32_t stage = base + C::kOffStage + (uint32_t)wg * kTileBytes;
    bool ok = true;
    DeqJobView job;
    int i = wg;
    for (; i < n_local; i += 2) {
      const int t = t0 + i;
      view_advance(batch, t, job);
      const int lt = t - job.begin;
      const int slab = lt / job.tps;
      const int s0 = (lt - slab * job.tps) * kTileRows;
      const int64_t s_row = (int64_t)s0 + row;
      const bool valid = s_row < job.S;
      const int64_t n = (int64_t)slab * job.S + s_row;
      const float nv = valid ? __half2float(__ushort_as_half(__ldg(job.norms + n))) : 0.f;   // in flight during the wait
      const int bb = slab / job.H, hh = slab - bb * job.H;
      const int b = i % kNT;
      ok = __all_sync(0xffffffffu, mbar_wait(bar_tfull + 8 * b, (uint32_t)((i / kNT) & 1), abort_flag));
      if (!ok) break;
      tc_fence_after();
      const uint32_t tacc = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(b * 128);
      if constexpr (OUT32) {
        const int64_t off = (int64_t)bb * job.os_b + (int64_t)hh * job.os_h + s_row * job.os_s;
        drain_row<TQ_F32>(tacc, nv, reinterpret_cast<float*>(job.out) + off, valid);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_tempty + 8 * b);
      } else {
        // the previous tile's store must have finished reading the staging tile
        if (wg_tid == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        asm volatile("bar.sync %0, 128;" ::"r"(wg + 2) : "memory");
        if (TQ_ABL(batch, 8)) {
        } else if (job.out_dtype == TQ_F16) drain_row_staged<TQ_F16>(tacc, nv, stage, row);
        else drain_row_staged<TQ_BF16>(tacc, nv, stage, row);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_tempty + 8 * b);               // the accumulator is free again
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // staging writes -> visible to the TMA engine
        // the tile is stored only if every warp of the group drained its rows
        const bool all_ok = bar_red_and(wg + 2, 128, true);
        if (wg_tid == 0 && all_ok && !TQ_ABL(batch, 1)) {
          tma_store_4d(job.out_map, stage, 0, s0, hh, bb);
          tma_store_4d(job.out_map, stage + kHalfBytes, 64, s0, hh, bb);
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
    }
    if constexpr (!OUT32) {
      if (!ok)                                     // keep the group's two barriers per tile complete
        for (; i < n_local; i += 2) {
          asm volatile("bar.sync %0, 128;" ::"r"(wg + 2) : "memory");
          bar_red_and(wg + 2, 128, false);
        }
    }
    if constexpr (!OUT32) {
      if (wg_tid == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // all stores done before exit
    }
    if (!ok && lane == 0) {
      *abort_flag = 1;
      if (batch.status != nullptr) atomicCAS(batch.status, 0, (7 << 16) | (int)blockIdx.x);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------- rotation image
// image[piece][khalf][row n][64 cols], rows of 128 bytes, 16-byte chunk c stored at c ^ (n & 7).
// Pieces 0-1: fp16 hi / lo (m = hi + lo, lo in fp16 subnormals).  Pieces 2-4: bf16 p0 + p1 + p2.
__global__ void k_rotation_image(const float* __restrict__ m, uint16_t* __restrict__ image) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;     // over 128 x 128
  if (idx >= kDim * kDim) return;
  const int n = idx / kDim, k = idx % kDim;
  const float v = m[idx];
  const __half hi = __float2half_rn(v);
  const __half lo = __float2half_rn(v - __half2float(hi));
  const __nv_bfloat16 p0 = __float2bfloat16_rn(v);
  const float r1 = v - __bfloat162float(p0);
  const __nv_bfloat16 p1 = __float2bfloat16_rn(r1);
  const __nv_bfloat16 p2 = __float2bfloat16_rn(r1 - __bfloat162float(p1));
  const int khalf = k >> 6, kk = k & 63;
  const int chunk = (kk >> 3) ^ (n & 7);
  const int off = khalf * (kTileRows * 64) + n * 64 + chunk * 8 + (kk & 7);
  const int piece = kTileRows * kDim;
  image[off] = __half_as_ushort(hi);
  image[piece + off] = __half_as_ushort(lo);
  image[2 * piece + off] = __bfloat16_as_ushort(p0);
  image[3 * piece + off] = __bfloat16_as_ushort(p1);
  image[4 * piece + off] = __bfloat16_as_ushort(p2);
}

// ---------------------------------------------------------------- host side
typedef TensorMapEncodeFn EncodeTiledFn;

EncodeTiledFn encode_fn() { return tensor_map_encoder(); }

int ablate_flags() {
#ifdef TQ_ABLATION
  const char* e = getenv("TQ_ABLATE");
  return e != nullptr ? atoi(e) : 0;
#else
  return 0;
#endif
}

// Contiguous tile ranges of equal estimated cost: job j has tiles[j] tiles that cost weight[j] each.
// A launch that mixes code widths would otherwise finish with the CTAs that drew the slow tiles.
void partition_tiles(const int64_t* tiles, const int* weight, int n_jobs, int grid, int32_t* cta_begin) {
  double total = 0.0;
  int64_t total_tiles = 0;
  for (int j = 0; j < n_jobs; ++j) { total += (double)tiles[j] * weight[j]; total_tiles += tiles[j]; }
  int j = 0;
  double cum = 0.0;          // cost of the jobs before j
  int64_t base = 0;          // tiles of the jobs before j
  cta_begin[0] = 0;
  for (int c = 1; c < grid; ++c) {
    const double target = total * c / grid;
    while (j < n_jobs && cum + (double)tiles[j] * weight[j] <= target) {
      cum += (double)tiles[j] * weight[j];
      base += tiles[j];
      ++j;
    }
    int64_t b = j >= n_jobs ? total_tiles : base + (int64_t)((target - cum) / weight[j]);
    if (b > total_tiles) b = total_tiles;
    if (b < cta_begin[c - 1]) b = cta_begin[c - 1];
    cta_begin[c] = (int32_t)b;
  }
  cta_begin[grid] = (int32_t)total_tiles;
}

// Cost of a 128-vector tile per code width, in units of about 10 ns on one SM; only the ratios matter.  Measured
// on (8, 8, 32768, 128) tensors one width at a time, then corrected with the per-CTA times of a mixed launch
// (K6/V4 layers with 8-bit protected layers, all widths running side by side under the power cap), where the
// CTAs of the 8-bit jobs finished 6 % after the average and those of the 4-bit jobs 5 % before it.
int quantize_tile_weight(int bits, bool bf16) {
  if (bf16) return bits <= 2 ? 133 : bits <= 5 ? 144 : bits == 6 ? 170 : 219;
  return bits <= 2 ? 117 : bits <= 4 ? 137 : bits == 5 ? 146 : bits == 6 ? 163 : 203;
}
int dequantize_tile_weight(int bits, bool out32) {
  if (out32) return bits <= 4 ? 250 : 300;
  return bits <= 2 ? 127 : bits <= 4 ? 130 : bits <= 7 ? 152 : 157;
}

}  // namespace

bool force_simt() {
  const char* e = getenv("TQ_FORCE_SIMT");
  return e != nullptr && e[0] == '1';
}

TensorMapEncodeFn tensor_map_encoder() {
  static std::atomic<void*> cached{nullptr};
  void* p = cached.load();
  if (p == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    cached.store(fn);
    p = fn;
  }
  return reinterpret_cast<TensorMapEncodeFn>(p);
}

size_t umma_rotation_image_bytes(int D) { return D == kDim ? (size_t)kImageBytes : 0; }

int umma_prepare_rotation_image(const float* m, int D, void* image, cudaStream_t st) {
  if (D != kDim) return TQ_EDIM;
  k_rotation_image<<<(kDim * kDim + 255) / 256, 256, 0, st>>>(m, reinterpret_cast<uint16_t*>(image));
  return check_launch();
}

// Prepared launch descriptions kept per thread: a few slots, least recently used one replaced.  A caller with static
// buffers submits the same job arrays again and again (one plan, or a few plans in rotation as the host-streamed
// cache does): a call whose array, device and switches match a slot only issues the kernel.
constexpr int kLaunchSlots = 4;
template <typename Batch>
struct LaunchSlot {
  Batch batch;
  std::vector<unsigned char> jobs;
  int dev = -1, ablate = 0, grid = 0;
  unsigned long long stamp = 0;
};
template <typename Batch>
static LaunchSlot<Batch>& pick_slot(LaunchSlot<Batch> (&slots)[kLaunchSlots], unsigned long long& clock, const void* jobs,
                                    size_t job_bytes, int dev, int ablate, bool cacheable, bool& reuse) {
  reuse = false;
  int victim = 0;
  for (int i = 0; i < kLaunchSlots; ++i) {
    LaunchSlot<Batch>& s = slots[i];
    if (cacheable && s.dev == dev && s.ablate == ablate && s.jobs.size() == job_bytes &&
        memcmp(s.jobs.data(), jobs, job_bytes) == 0) {
      reuse = true;
      s.stamp = ++clock;
      return s;
    }
    if (s.stamp < slots[victim].stamp) victim = i;
  }
  slots[victim].stamp = ++clock;
  return slots[victim];
}

bool umma_quantize_eligible(const TqQuantizeJob& j) {
  if (force_simt()) return false;
  if (j.rotation_image == nullptr || j.D != kDim || j.normalize != 1 || j.idx_mode != TQ_IDX_PACKED) return false;
  if (j.x_dtype != TQ_F16 && j.x_dtype != TQ_BF16) return false;
  if (j.B <= 0 || j.H <= 0 || j.S <= 0) return false;
  if (j.B > 65535 || j.H > 65535 || j.S > (int64_t)1 << 30) return false;
  if (((uintptr_t)j.x & 15u) || ((uintptr_t)j.idx_out & 15u) || ((uintptr_t)j.rotation_image & 15u)) return false;
  if ((j.S > 1 && (j.stride_s % 8 != 0 || j.stride_s < kDim)) || (j.H > 1 && j.stride_h % 8 != 0) ||
      (j.B > 1 && j.stride_b % 8 != 0))
    return false;
  if (j.stride_s < 0 || j.stride_h < 0 || j.stride_b < 0) return false;
  const int64_t tiles = j.B * j.H * ((j.S + kTileRows - 1) / kTileRows);
  return tiles < ((int64_t)1 << 30);
}

// Launch one persistent kernel over up to kMaxJobs eligible jobs (all of one input dtype).
int umma_quantize(const TqQuantizeJob* jobs, int n_jobs, cudaStream_t st) {
  EncodeTiledFn enc = encode_fn();
  if (enc == nullptr) return TQ_ELAUNCH;
  // The prepared launch description (tensor maps included) of an earlier call of this thread is reused when the
  // job array, the device and the switches are unchanged.  Per-thread, so calls stay re-entrant.
  static thread_local LaunchSlot<UmmaQuantBatch> slots[kLaunchSlots];      // large: kept off the stack
  static thread_local unsigned long long slot_clock = 0;
  int cur_dev = 0;
  cudaGetDevice(&cur_dev);
  const size_t job_bytes = (size_t)n_jobs * sizeof(TqQuantizeJob);
  bool reuse = false;
  LaunchSlot<UmmaQuantBatch>& slot = pick_slot(slots, slot_clock, jobs, job_bytes, cur_dev, ablate_flags(), n_jobs <= kMaxJobs, reuse);
  UmmaQuantBatch& batch = slot.batch;
  std::vector<unsigned char>& last_jobs = slot.jobs;
  int& last_dev = slot.dev;
  int& last_ablate = slot.ablate;
  int& last_grid = slot.grid;
  last_dev = -1;                                 // invalid until this call has rebuilt or reused the batch
  int done = 0;
  while (done < n_jobs) {
    const int take = (n_jobs - done) < kMaxJobs ? (n_jobs - done) : kMaxJobs;
    int64_t tile_cursor = 0;
    int64_t job_tiles[kMaxJobs];
    int job_weight[kMaxJobs];
    for (int i = 0; i < take && !reuse; ++i) {
      const TqQuantizeJob& j = jobs[done + i];
      UmmaQuantJob& u = batch.jobs[i];
      const int64_t tps = (j.S + kTileRows - 1) / kTileRows;
      job_tiles[i] = tps * j.B * j.H;
      job_weight[i] = quantize_tile_weight(j.bits, j.x_dtype == TQ_BF16);
      // size-1 dimensions get a harmless stride; TMA wants multiples of 16 bytes
      const int64_t ss = j.S > 1 ? j.stride_s : kDim;
      const int64_t sh = j.H > 1 ? j.stride_h : ss * j.S;
      const int64_t sb = j.B > 1 ? j.stride_b : (sh > ss ? sh : ss) * (j.H > 1 ? j.H : j.S);
      cuuint64_t dims[4] = {(cuuint64_t)kDim, (cuuint64_t)j.S, (cuuint64_t)j.H, (cuuint64_t)j.B};
      cuuint64_t strides[3] = {(cuuint64_t)ss * 2, (cuuint64_t)sh * 2, (cuuint64_t)sb * 2};
      cuuint32_t box[4] = {64, (cuuint32_t)kTileRows, 1, 1};
      cuuint32_t estr[4] = {1, 1, 1, 1};
      CUresult r = enc(&u.tmap, j.x_dtype == TQ_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                       const_cast<void*>(j.x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                       CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS) { note_cuda_error(100000 + (int)r); return TQ_ELAUNCH; }
      u.image = j.rotation_image;
      u.codebook = j.codebook;
      u.idx_out = reinterpret_cast<uint8_t*>(j.idx_out);
      u.norms_out = j.norms_out;
      u.S = j.S;
      u.H = (int32_t)j.H;
      u.tiles_per_slab = (int32_t)tps;
      u.tile_begin = (int32_t)tile_cursor;
      u.bits = j.bits;
      u.a_bf16 = j.x_dtype == TQ_BF16;
      u.pad_ = 0;
      tile_cursor += tps * j.B * j.H;
      if (tile_cursor >= ((int64_t)1 << 30)) return TQ_ETOOBIG;
    }
    int grid = last_grid;
    const bool bf16 = jobs[done].x_dtype == TQ_BF16;
    bool wide = false;
    for (int i = 0; i < take; ++i) wide = wide || jobs[done + i].bits > 5;
    const uint32_t smem = bf16 ? (wide ? Cfg<true, true>::kSmemBytes : Cfg<true, false>::kSmemBytes)
                               : (wide ? Cfg<false, true>::kSmemBytes : Cfg<false, false>::kSmemBytes);
    if (!reuse) {
      batch.n_jobs = take;
      batch.total_tiles = (int32_t)tile_cursor;
      batch.ablate = ablate_flags();
      void* status_ptr = nullptr;
      cudaGetSymbolAddress(&status_ptr, g_umma_status);
      batch.status = reinterpret_cast<int32_t*>(status_ptr);
      int sms = 148;
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, cur_dev);
      if (sms > kMaxCtas) sms = kMaxCtas;
      grid = (int)(tile_cursor < sms ? tile_cursor : sms);
      partition_tiles(job_tiles, job_weight, take, grid, batch.cta_begin);
    }
    auto launch = [&](auto kern) -> int {
      if (!reuse) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { note_cuda_error((int)e); return TQ_ELAUNCH; }
      }
      kern<<<grid, kThreads, smem, st>>>(batch);
      return TQ_OK;
    };
    int lrc;
    if (bf16 && wide) lrc = launch(k_umma_quantize<true, true>);
    else if (bf16) lrc = launch(k_umma_quantize<true, false>);
    else if (wide) lrc = launch(k_umma_quantize<false, true>);
    else lrc = launch(k_umma_quantize<false, false>);
    if (lrc != TQ_OK) return lrc;
    int rc = check_launch();
    if (rc != TQ_OK) return rc;
    last_grid = grid;
    done += take;
  }
  if (n_jobs <= kMaxJobs) {
    if (!reuse) last_jobs.assign(reinterpret_cast<const unsigned char*>(jobs), reinterpret_cast<const unsigned char*>(jobs) + job_bytes);
    last_ablate = ablate_flags();
    last_dev = cur_dev;
  }
  return TQ_OK;
}

bool umma_dequantize_eligible(const TqDequantizeJob& j) {
  if (force_simt()) return false;
  if (j.rotation_image == nullptr || j.D != kDim || j.idx_mode != TQ_IDX_PACKED || j.norms == nullptr) return false;
  if (j.B <= 0 || j.H <= 0 || j.S <= 0) return false;
  if (((uintptr_t)j.idx & 15u) || ((uintptr_t)j.out & 15u) || ((uintptr_t)j.rotation_image & 15u)) return false;
  const int64_t q = j.out_dtype == TQ_F32 ? 4 : 8;     // elements per 16 bytes
  if (j.ostride_s % q != 0 || j.ostride_h % q != 0 || j.ostride_b % q != 0) return false;
  if (j.ostride_s < 0 || j.ostride_h < 0 || j.ostride_b < 0) return false;
  if (j.out_dtype != TQ_F32 && (j.B > 65535 || j.H > 65535 || (j.S > 1 && j.ostride_s < kDim))) return false;
  const int64_t tiles = j.B * j.H * ((j.S + kTileRows - 1) / kTileRows);
  return tiles < ((int64_t)1 << 30);
}

// One persistent launch over a run of eligible jobs that share the output class (fp32 vs 16-bit).
int umma_dequantize(const TqDequantizeJob* jobs, int n_jobs, cudaStream_t st) {
  EncodeTiledFn enc = encode_fn();
  if (enc == nullptr) return TQ_ELAUNCH;
  // same reuse of earlier calls' launch descriptions as in umma_quantize
  static thread_local LaunchSlot<UmmaDeqBatch> slots[kLaunchSlots];
  static thread_local unsigned long long slot_clock = 0;
  int cur_dev = 0;
  cudaGetDevice(&cur_dev);
  const size_t job_bytes = (size_t)n_jobs * sizeof(TqDequantizeJob);
  bool reuse = false;
  LaunchSlot<UmmaDeqBatch>& slot = pick_slot(slots, slot_clock, jobs, job_bytes, cur_dev, ablate_flags(), n_jobs <= kMaxDeqJobs, reuse);
  UmmaDeqBatch& batch = slot.batch;
  std::vector<unsigned char>& last_jobs = slot.jobs;
  int& last_dev = slot.dev;
  int& last_ablate = slot.ablate;
  int& last_grid = slot.grid;
  last_dev = -1;
  int done = 0;
  while (done < n_jobs) {
    const int take = (n_jobs - done) < kMaxDeqJobs ? (n_jobs - done) : kMaxDeqJobs;
    int64_t tile_cursor = 0;
    int64_t job_tiles[kMaxDeqJobs];
    int job_weight[kMaxDeqJobs];
    for (int i = 0; i < take && !reuse; ++i) {
      const TqDequantizeJob& j = jobs[done + i];
      UmmaDeqJob& u = batch.jobs[i];
      const int64_t tps = (j.S + kTileRows - 1) / kTileRows;
      job_tiles[i] = tps * j.B * j.H;
      job_weight[i] = dequantize_tile_weight(j.bits, j.out_dtype == TQ_F32);
      if (j.out_dtype != TQ_F32) {
        const int64_t ss = j.S > 1 ? j.ostride_s : kDim;
        const int64_t sh = j.H > 1 ? j.ostride_h : ss * j.S;
        const int64_t sb = j.B > 1 ? j.ostride_b : (sh > ss ? sh : ss) * (j.H > 1 ? j.H : j.S);
        cuuint64_t dims[4] = {(cuuint64_t)kDim, (cuuint64_t)j.S, (cuuint64_t)j.H, (cuuint64_t)j.B};
        cuuint64_t strides[3] = {(cuuint64_t)ss * 2, (cuuint64_t)sh * 2, (cuuint64_t)sb * 2};
        cuuint32_t box[4] = {64, (cuuint32_t)kTileRows, 1, 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        CUresult r = enc(&u.out_map, j.out_dtype == TQ_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                         4, j.out, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { note_cuda_error(100000 + (int)r); return TQ_ELAUNCH; }
      }
      u.idx = reinterpret_cast<const uint8_t*>(j.idx);
      u.norms = j.norms;
      u.image = j.rotation_image;
      u.codebook = j.codebook;
      u.out = j.out;
      u.S = j.S;
      u.os_b = j.ostride_b; u.os_h = j.ostride_h; u.os_s = j.ostride_s;
      u.H = (int32_t)j.H;
      u.tiles_per_slab = (int32_t)tps;
      u.tile_begin = (int32_t)tile_cursor;
      u.bits = j.bits;
      u.out_dtype = j.out_dtype;
      u.pad_ = 0;
      tile_cursor += tps * j.B * j.H;
      if (tile_cursor >= ((int64_t)1 << 30)) return TQ_ETOOBIG;
    }
    int grid = last_grid;
    if (!reuse) {
      batch.n_jobs = take;
      batch.total_tiles = (int32_t)tile_cursor;
      batch.ablate = ablate_flags();
      void* status_ptr = nullptr;
      cudaGetSymbolAddress(&status_ptr, g_umma_status);
      batch.status = reinterpret_cast<int32_t*>(status_ptr);
      int sms = 148;
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, cur_dev);
      if (sms > kMaxCtas) sms = kMaxCtas;
      grid = (int)(tile_cursor < sms ? tile_cursor : sms);
      partition_tiles(job_tiles, job_weight, take, grid, batch.cta_begin);
    }
    const bool out32 = jobs[done].out_dtype == TQ_F32;
    bool narrow = true;
    for (int i = 0; i < take; ++i) narrow = narrow && jobs[done + i].bits <= 4;
    auto launch = [&](auto kern, uint32_t smem, int threads) -> int {
      if (!reuse) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { note_cuda_error((int)e); return TQ_ELAUNCH; }
      }
      kern<<<grid, threads, smem, st>>>(batch);
      return TQ_OK;
    };
    int lrc;
    if (out32 && narrow) lrc = launch(k_umma_dequantize<true, true>, DCfg<true, true>::kSmemBytes, DCfg<true, true>::kThreadsD);
    else if (out32) lrc = launch(k_umma_dequantize<true, false>, DCfg<true, false>::kSmemBytes, DCfg<true, false>::kThreadsD);
    else if (narrow) lrc = launch(k_umma_dequantize<false, true>, DCfg<false, true>::kSmemBytes, DCfg<false, true>::kThreadsD);
    else lrc = launch(k_umma_dequantize<false, false>, DCfg<false, false>::kSmemBytes, DCfg<false, false>::kThreadsD);
    if (lrc != TQ_OK) return lrc;
    int rc = check_launch();
    if (rc != TQ_OK) return rc;
    last_grid = grid;
    done += take;
  }
  if (n_jobs <= kMaxDeqJobs) {
    if (!reuse) last_jobs.assign(reinterpret_cast<const unsigned char*>(jobs), reinterpret_cast<const unsigned char*>(jobs) + job_bytes);
    last_ablate = ablate_flags();
    last_dev = cur_dev;
  }
  return TQ_OK;
}

int umma_device_status() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_umma_status, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

}  // namespace tq
