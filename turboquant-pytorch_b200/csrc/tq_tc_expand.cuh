// Packed indices -> fp16 centroid pieces in the swizzled K-major operand layout (head_dim 128).
// Included inside namespace tq { namespace { ... } } after tq_tc_ptx.cuh; expects
// kDim = 128, kTileBytes = 32768 and kHalfBytes = 16384 to be defined by the including file.
#pragma once

// Expand half a row (64 coordinates = one 128-byte swizzled operand row of k-half `half`):
// chunk q (8 coordinates, 16 bytes) goes to  half*16384 + row*128 + ((q ^ (row & 7)) << 4).
// lut[i] = {hi(c_i) | lo(c_i) << 16} in static shared memory; `src` is the shared address
// of this half row's packed bytes.  Look-ups use byte offsets (index * 4) so that the load
// is a plain [register + constant] shared-memory access; for 4- and 2-bit codes the offsets
// of a whole word are prepared with two shifts and masks and picked out bytewise.
//
// Lane mapping and bank conflicts.  The caller gives lane l of a warp the half row
// (row0 + l / 2, l & 1), so a quarter warp (the unit in which 16-byte shared accesses are served) holds
// four consecutive rows x both halves.  Each thread walks its chunks in an order XOR-ed with `qx`
// (expand_order): at every step the eight lanes then read eight different 16-byte bank groups of the
// packed tile and write eight different 16-byte positions of the swizzled operand rows, so the packed
// loads and the operand stores both run without bank conflicts.  (With lanes = consecutive rows of
// one half, the 128-byte rows of one-byte codes put all eight lanes on the same four banks.)
template <int BITS>
__device__ __forceinline__ uint32_t expand_order(int row, int half) {
  constexpr int HB = kDim / (8 / BITS) / 2;     // packed bytes per half row
  if constexpr (HB == 64) return (uint32_t)((((row & 3) ^ (half << 1))) << 1);   // four chunks: rows take different ones
  else if constexpr (HB == 32) return (uint32_t)((half ^ ((row >> 1) & 1)) << 2);   // two chunks
  else return (uint32_t)(half << 2);            // one load: the halves start at opposite ends
}

template <int BITS>
__device__ __forceinline__ uint32_t lut_at(const uint32_t* lut, uint32_t byte_off) {
  return *reinterpret_cast<const uint32_t*>(reinterpret_cast<const char*>(lut) + byte_off);
}

template <int BITS, int PIECES>
__device__ __forceinline__ void expand_half(uint32_t src, const uint32_t* lut, uint32_t a_stage, int row, int half) {
  constexpr int IPB = 8 / BITS;
  constexpr int HB = kDim / IPB / 2;            // packed bytes per half row: 8, 16, 32, 64
  constexpr uint32_t MASK = (1u << BITS) - 1u;
  // register k of w holds packed word k ^ (qx * HB / 32): the chunk walked at step q is q ^ qx
  const uint32_t qx = expand_order<BITS>(row, half);
  uint32_t w[HB / 4];
  if constexpr (HB == 8) {
    const uint2 v = ld_shared_v2(src);
    w[0] = qx ? v.y : v.x; w[1] = qx ? v.x : v.y;
  } else if constexpr (HB == 16) {
    const uint4 t = ld_shared_v4(src);
    w[0] = qx ? t.z : t.x; w[1] = qx ? t.w : t.y; w[2] = qx ? t.x : t.z; w[3] = qx ? t.y : t.w;
  } else {
    constexpr uint32_t kChunkShift = HB == 64 ? 3 : 2;       // qx -> byte offset of the chunk: (qx / (128 / HB)) * 16
#pragma unroll
    for (int v = 0; v < HB / 16; ++v) {
      const uint4 t = ld_shared_v4(src + ((16u * v) ^ (qx << kChunkShift)));
      w[4 * v] = t.x; w[4 * v + 1] = t.y; w[4 * v + 2] = t.z; w[4 * v + 3] = t.w;
    }
  }
  const uint32_t dst_row = a_stage + half * kHalfBytes + row * 128;
  const uint32_t px = qx ^ (uint32_t)(row & 7);
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    uint32_t e2[8];                             // look-ups of the 8 coordinates of this chunk
    if constexpr (BITS == 4) {
      const uint32_t x = w[q];                  // one word = 8 coordinates, two per byte
      const uint32_t even = (x >> 2) & 0x3C3C3C3Cu, odd = (x << 2) & 0x3C3C3C3Cu;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        e2[2 * k] = lut_at<BITS>(lut, __byte_perm(even, 0u, 0x4440u | k));
        e2[2 * k + 1] = lut_at<BITS>(lut, __byte_perm(odd, 0u, 0x4440u | k));
      }
    } else if constexpr (BITS == 2) {
      const uint32_t x = w[q >> 1];             // one word = 16 coordinates, four per byte
      const uint32_t f0 = (x >> 4) & 0x0C0C0C0Cu, f1 = (x >> 2) & 0x0C0C0C0Cu, f2 = x & 0x0C0C0C0Cu,
                     f3 = (x << 2) & 0x0C0C0C0Cu;
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const uint32_t sel = 0x4440u | ((q & 1) * 2 + k);
        e2[4 * k] = lut_at<BITS>(lut, __byte_perm(f0, 0u, sel));
        e2[4 * k + 1] = lut_at<BITS>(lut, __byte_perm(f1, 0u, sel));
        e2[4 * k + 2] = lut_at<BITS>(lut, __byte_perm(f2, 0u, sel));
        e2[4 * k + 3] = lut_at<BITS>(lut, __byte_perm(f3, 0u, sel));
      }
    } else {
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int e = q * 8 + u;                // coordinate within the half row
        const int byte = e / IPB;
        const int sh = 8 * (byte & 3) + BITS * (IPB - 1 - (e % IPB));
        const uint32_t xw = w[byte >> 2];
        const uint32_t off = sh >= 2 ? ((xw >> (sh - 2)) & (MASK << 2)) : ((xw << (2 - sh)) & (MASK << 2));
        e2[u] = lut_at<BITS>(lut, off);
      }
    }
    uint32_t hi[4], lo[4];
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      hi[p] = __byte_perm(e2[2 * p], e2[2 * p + 1], 0x5410);
      lo[p] = __byte_perm(e2[2 * p], e2[2 * p + 1], 0x7632);
    }
    const uint32_t dst = dst_row + ((q ^ px) << 4);
    st_shared_v4(dst, hi[0], hi[1], hi[2], hi[3]);
    if constexpr (PIECES == 2) st_shared_v4(dst + kTileBytes, lo[0], lo[1], lo[2], lo[3]);
  }
}

// Wide codes (one index per byte, 5..8 bits) for 16-bit outputs, which need the high fp16 piece only:
// the table is replicated so that look-ups do not collide in the banks.  An entry is a 32-bit word with the
// fp16 bits of the centroid in both halves (two look-ups merge into an operand word with one byte permute).
// Up to 7 bits: entry i is stored 32 times, copy l at byte i * 128 + 4 * l, and lane l reads its own copy:
// every lane stays in its own bank.  8 bits (256 entries, 16 KB of table space): 16 copies, copy l / 2 at
// byte i * 64 + 4 * (l / 2); two lanes can only meet in a bank when they form a pair and look up different
// entries of equal parity.  `lut_lane` is the table's shared address plus the lane's copy offset.
template <int BITS>
__device__ __forceinline__ void expand_half_wide16(uint32_t src, uint32_t lut_lane, uint32_t a_stage, int row, int half) {
  static_assert(BITS >= 5 && BITS <= 8, "one index per byte");
  constexpr int SH = BITS == 8 ? 6 : 7;         // log2 of the entry stride in bytes
  constexpr uint32_t MASK = ((1u << BITS) - 1u) << SH;
  const uint32_t qx = expand_order<BITS>(row, half);
  uint32_t w[16];                               // 64 packed bytes: this half row, chunk v ^ (qx / 2) in w[4v..4v+3]
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    const uint4 t = ld_shared_v4(src + ((16u * v) ^ (qx << 3)));
    w[4 * v] = t.x; w[4 * v + 1] = t.y; w[4 * v + 2] = t.z; w[4 * v + 3] = t.w;
  }
  const uint32_t dst_row = a_stage + half * kHalfBytes + row * 128;
  const uint32_t px = qx ^ (uint32_t)(row & 7);
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    uint32_t h[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const uint32_t xw = w[2 * q + (u >> 2)];
      const int sh = 8 * (u & 3);
      const uint32_t off = sh >= SH ? ((xw >> (sh - SH)) & MASK) : ((xw << (SH - sh)) & MASK);
      asm("ld.shared.b32 %0, [%1];" : "=r"(h[u]) : "r"(lut_lane + off));
    }
    const uint32_t dst = dst_row + ((q ^ px) << 4);
    st_shared_v4(dst, __byte_perm(h[0], h[1], 0x5410), __byte_perm(h[2], h[3], 0x5410), __byte_perm(h[4], h[5], 0x5410),
                 __byte_perm(h[6], h[7], 0x5410));
  }
}
