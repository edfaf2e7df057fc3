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
template <int BITS>
__device__ __forceinline__ uint32_t lut_at(const uint32_t* lut, uint32_t byte_off) {
  return *reinterpret_cast<const uint32_t*>(reinterpret_cast<const char*>(lut) + byte_off);
}

template <int BITS, int PIECES>
__device__ __forceinline__ void expand_half(uint32_t src, const uint32_t* lut, uint32_t a_stage, int row, int half) {
  constexpr int IPB = 8 / BITS;
  constexpr int HB = kDim / IPB / 2;            // packed bytes per half row: 8, 16, 32, 64
  constexpr uint32_t MASK = (1u << BITS) - 1u;
  uint32_t w[HB / 4];
  if constexpr (HB == 8) {
    const uint2 v = ld_shared_v2(src);
    w[0] = v.x; w[1] = v.y;
  } else {
#pragma unroll
    for (int v = 0; v < HB / 16; ++v) {
      const uint4 t = ld_shared_v4(src + 16 * v);
      w[4 * v] = t.x; w[4 * v + 1] = t.y; w[4 * v + 2] = t.z; w[4 * v + 3] = t.w;
    }
  }
  const uint32_t dst_row = a_stage + half * kHalfBytes + row * 128;
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
    const uint32_t dst = dst_row + ((q ^ (row & 7)) << 4);
    st_shared_v4(dst, hi[0], hi[1], hi[2], hi[3]);
    if constexpr (PIECES == 2) st_shared_v4(dst + kTileBytes, lo[0], lo[1], lo[2], lo[3]);
  }
}

// Wide codes (one index per byte, 5..8 bits) for 16-bit outputs, which need the high fp16 piece only:
// the table is replicated so that look-ups hardly ever collide.  Entry i (fp16 bits of the centroid)
// is stored 32 times, copy l at byte  i * 64 + 2 * l;  lane l reads its own copy, so two lanes can
// only meet in a bank when they form a pair (l, l ^ 1) and look up different entries of equal parity.
// `lut_lane` is the table's shared address plus 2 * lane.
template <int BITS>
__device__ __forceinline__ void expand_half_wide16(uint32_t src, uint32_t lut_lane, uint32_t a_stage, int row, int half) {
  static_assert(BITS >= 5 && BITS <= 8, "one index per byte");
  constexpr uint32_t MASK = ((1u << BITS) - 1u) << 6;
  uint32_t w[16];                               // 64 packed bytes: this half row
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    const uint4 t = ld_shared_v4(src + 16 * v);
    w[4 * v] = t.x; w[4 * v + 1] = t.y; w[4 * v + 2] = t.z; w[4 * v + 3] = t.w;
  }
  const uint32_t dst_row = a_stage + half * kHalfBytes + row * 128;
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    uint32_t h[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const uint32_t xw = w[2 * q + (u >> 2)];
      const int sh = 8 * (u & 3);
      const uint32_t off = sh >= 6 ? ((xw >> (sh - 6)) & MASK) : ((xw << (6 - sh)) & MASK);
      uint16_t v16;
      asm("ld.shared.u16 %0, [%1];" : "=h"(v16) : "r"(lut_lane + off));
      h[u] = v16;
    }
    const uint32_t dst = dst_row + ((q ^ (row & 7)) << 4);
    st_shared_v4(dst, h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16), h[6] | (h[7] << 16));
  }
}
