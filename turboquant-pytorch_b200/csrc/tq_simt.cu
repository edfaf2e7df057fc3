// FP32 CUDA-core kernels: the exact-arithmetic path of every entry point.
//
// All rotation work goes through one register-tiled FP32 contraction
// (tile_gemm) whose k-loop is a sequential fma chain per output, i.e. ordinary
// fp32 dot products.  A tile is 64 vectors; the CTA keeps the tile in shared
// memory across the chained stages of a kernel (normalise -> rotate ->
// quantise -> rotate back -> residual -> project), so intermediates never
// touch HBM.  These kernels serve fp32 inputs, head_dims other than 128 and
// every API surface that is not throughput critical; the 16-bit, head_dim-128
// quantise / dequantise traffic goes to the tensor-core kernels in tq_umma.cu.

#include <atomic>

#include "tq_common.cuh"
#include "tq_internal.h"

namespace tq {

constexpr int TM = 64;    // vectors per tile
constexpr int KC = 16;    // k rows of B staged per step
constexpr int NT = 256;   // threads per CTA
constexpr int BPAD = 4;

enum { B_KN = 0, B_NK = 1 };

__host__ __device__ inline int lda_for(int K) { return round_up(K, KC) + 4; }
__host__ __device__ inline int ldb_for(int N) { return round_up(N, 64) + BPAD; }

// acc[ri][4*j+c] += sum_k As[(ty*4+ri)*lda + k] * B[k][tx*4 + 64*j + c]
// B is global, fp32, either [K][N] row-major with row stride ldg (B_KN) or
// [N][K] row-major with row stride ldg (B_NK).  Columns >= N and rows >= K read
// as zero.  As must hold zeros in columns [K, round_up(K,16)).
template <int NJ, int BL>
__device__ __forceinline__ void tile_gemm(const float* As, int lda, int K, const float* __restrict__ Bg, int64_t ldg,
                                          int N, float* Bs, float (&acc)[4][4 * NJ]) {
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int npad = 64 * NJ;
  const int ldb = npad + BPAD;
  const int kpad = round_up(K, KC);
  for (int k0 = 0; k0 < kpad; k0 += KC) {
    __syncthreads();
    if constexpr (BL == B_KN) {
      for (int e = tid; e < KC * npad; e += NT) {
        int kk = e / npad, n = e - kk * npad;
        int k = k0 + kk;
        float v = 0.f;
        if (k < K && n < N) v = __ldg(Bg + (int64_t)k * ldg + n);
        Bs[kk * ldb + n] = v;
      }
    } else {
      for (int e = tid; e < KC * npad; e += NT) {
        int n = e / KC, kk = e - n * KC;
        int k = k0 + kk;
        float v = 0.f;
        if (k < K && n < N) v = __ldg(Bg + (int64_t)n * ldg + k);
        Bs[kk * ldb + n] = v;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < KC; kk += 4) {
      float4 a[4];
#pragma unroll
      for (int ri = 0; ri < 4; ++ri) a[ri] = *reinterpret_cast<const float4*>(As + (ty * 4 + ri) * lda + k0 + kk);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float4 b[NJ];
#pragma unroll
        for (int j = 0; j < NJ; ++j) b[j] = *reinterpret_cast<const float4*>(Bs + (kk + u) * ldb + tx * 4 + 64 * j);
#pragma unroll
        for (int ri = 0; ri < 4; ++ri) {
          float av = (u == 0) ? a[ri].x : (u == 1) ? a[ri].y : (u == 2) ? a[ri].z : a[ri].w;
#pragma unroll
          for (int j = 0; j < NJ; ++j) {
            acc[ri][4 * j + 0] = fmaf(av, b[j].x, acc[ri][4 * j + 0]);
            acc[ri][4 * j + 1] = fmaf(av, b[j].y, acc[ri][4 * j + 1]);
            acc[ri][4 * j + 2] = fmaf(av, b[j].z, acc[ri][4 * j + 2]);
            acc[ri][4 * j + 3] = fmaf(av, b[j].w, acc[ri][4 * j + 3]);
          }
        }
      }
    }
  }
}

template <int NJ>
__device__ __forceinline__ void zero_acc(float (&acc)[4][4 * NJ]) {
#pragma unroll
  for (int ri = 0; ri < 4; ++ri)
#pragma unroll
    for (int c = 0; c < 4 * NJ; ++c) acc[ri][c] = 0.f;
}

// registers -> Cs[r*ldc + n] for n < ncols (a multiple of 4, at most ldc); caller syncs around it
template <int NJ>
__device__ __forceinline__ void acc_to_smem(const float (&acc)[4][4 * NJ], float* Cs, int ldc, int ncols) {
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
  for (int ri = 0; ri < 4; ++ri)
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      const int col = tx * 4 + 64 * j;
      if (col < ncols)
        *reinterpret_cast<float4*>(Cs + (ty * 4 + ri) * ldc + col) =
            make_float4(acc[ri][4 * j], acc[ri][4 * j + 1], acc[ri][4 * j + 2], acc[ri][4 * j + 3]);
    }
}

// Load a tile of vectors as fp32 into Xs (zero padded to kpad columns, zero rows
// past n_total); per-row L2 norms into nrm[] when wanted.
template <int XDT>
__device__ __forceinline__ void load_tile_rows(const void* x, int64_t row0, int64_t n_total, int D, int64_t H, int64_t S,
                                               int64_t sb, int64_t sh, int64_t ss, float* Xs, int ld, float* nrm) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kpad = round_up(D, KC);
  for (int r = warp; r < TM; r += NT / 32) {
    int64_t n = row0 + r;
    float ssq = 0.f;
    if (n < n_total) {
      int64_t off = vec_offset(n, H, S, sb, sh, ss);
      for (int k = lane; k < kpad; k += 32) {
        float v = (k < D) ? load_elem<XDT>(x, off + k) : 0.f;
        Xs[r * ld + k] = v;
        ssq = fmaf(v, v, ssq);
      }
    } else {
      for (int k = lane; k < kpad; k += 32) Xs[r * ld + k] = 0.f;
    }
    if (nrm != nullptr) {
      ssq = warp_sum(ssq);
      if (lane == 0) nrm[r] = __fsqrt_rn(ssq);
    }
  }
}

__device__ __forceinline__ void load_codebook(const float* cb, float* cent_s, float* thr_s) {
  for (int i = threadIdx.x; i < 256; i += NT) {
    cent_s[i] = __ldg(cb + kCentroidOff + i);
    thr_s[i] = __ldg(cb + kThresholdOff + i);
  }
}

// Quantise the row Cs[r][0..D) and write it in the requested layout.
__device__ __forceinline__ void emit_indices_row(const float* row, int D, int bits, int mode, const float* thr_s,
                                                 void* out, int64_t n, int lane) {
  const int levels = 1 << bits;
  if (mode == TQ_IDX_PACKED) {
    const int ipb = 8 / bits;
    const int G = (D + ipb - 1) / ipb;
    uint8_t* o = reinterpret_cast<uint8_t*>(out) + n * (int64_t)G;
    for (int g = lane; g < G; g += 32) {
      unsigned byte = 0;
      for (int i = 0; i < ipb; ++i) {
        int c = g * ipb + i;
        unsigned q = (c < D) ? (unsigned)quantize_scalar(row[c], thr_s, levels) : 0u;
        byte |= q << (bits * (ipb - 1 - i));
      }
      o[g] = (uint8_t)byte;
    }
  } else if (mode == TQ_IDX_U8) {
    uint8_t* o = reinterpret_cast<uint8_t*>(out) + n * (int64_t)D;
    for (int c = lane; c < D; c += 32) o[c] = (uint8_t)quantize_scalar(row[c], thr_s, levels);
  } else {
    int64_t* o = reinterpret_cast<int64_t*>(out) + n * (int64_t)D;
    for (int c = lane; c < D; c += 32) o[c] = (int64_t)quantize_scalar(row[c], thr_s, levels);
  }
}

__device__ __forceinline__ int fetch_index(const void* idx, int mode, int64_t n, int c, int D, int bits) {
  if (mode == TQ_IDX_PACKED) {
    const int ipb = 8 / bits;
    const int G = (D + ipb - 1) / ipb;
    unsigned byte = reinterpret_cast<const uint8_t*>(idx)[n * (int64_t)G + c / ipb];
    return (int)((byte >> (bits * (ipb - 1 - c % ipb))) & ((1u << bits) - 1u));
  } else if (mode == TQ_IDX_U8) {
    return (int)reinterpret_cast<const uint8_t*>(idx)[n * (int64_t)D + c];
  }
  return (int)(reinterpret_cast<const int64_t*>(idx)[n * (int64_t)D + c] & 255);
}

// ---------------------------------------------------------------------------
// K0: rotated values -> indices
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(NT) k_quantize_rotated(const float* __restrict__ y, int64_t n, int D, int bits,
                                                        const float* __restrict__ cb, int mode, void* out) {
  __shared__ float thr_s[256];
  for (int i = threadIdx.x; i < 256; i += NT) thr_s[i] = __ldg(cb + kThresholdOff + i);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t wstride = (int64_t)gridDim.x * (NT / 32);
  for (int64_t r = (int64_t)blockIdx.x * (NT / 32) + warp; r < n; r += wstride)
    emit_indices_row(y + r * D, D, bits, mode, thr_s, out, r, lane);
}

// ---------------------------------------------------------------------------
// K1: norm + rotate + quantise + pack
// ---------------------------------------------------------------------------
template <int XDT, int NJ>
__global__ void __launch_bounds__(NT) k_quantize(TqQuantizeJob job) {
  extern __shared__ __align__(16) float smem[];
  const int D = job.D;
  const int lda = lda_for(D);
  float* As = smem;
  float* Bs = As + TM * lda;
  float* cent_s = Bs + KC * (64 * NJ + BPAD);
  float* thr_s = cent_s + 256;
  float* nrm = thr_s + 256;
  load_codebook(job.codebook, cent_s, thr_s);
  const int64_t n_total = job.B * job.H * job.S;
  const int64_t tiles = (n_total + TM - 1) / TM;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kpad = round_up(D, KC);
  for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const int64_t row0 = tile * TM;
    __syncthreads();
    load_tile_rows<XDT>(job.x, row0, n_total, D, job.H, job.S, job.stride_b, job.stride_h, job.stride_s, As, lda,
                        job.normalize ? nrm : nullptr);
    if (job.normalize) {
      __syncwarp();
      for (int r = warp; r < TM; r += NT / 32) {
        float nv = nrm[r];
        int64_t n = row0 + r;
        if (lane == 0 && n < n_total) job.norms_out[n] = __half_as_ushort(__float2half_rn(nv));
        float den = nv + 1e-8f;
        for (int k = lane; k < kpad; k += 32) As[r * lda + k] = __fdiv_rn(As[r * lda + k], den);
      }
    }
    float acc[4][4 * NJ];
    zero_acc<NJ>(acc);
    tile_gemm<NJ, B_KN>(As, lda, D, job.rotation_t, D, D, Bs, acc);
    __syncthreads();
    acc_to_smem<NJ>(acc, As, lda, kpad);
    __syncthreads();
    for (int r = warp; r < TM; r += NT / 32) {
      int64_t n = row0 + r;
      if (n < n_total) emit_indices_row(As + r * lda, D, job.bits, job.idx_mode, thr_s, job.idx_out, n, lane);
    }
  }
}

// ---------------------------------------------------------------------------
// K2: unpack + lookup + inverse rotation + rescale
// ---------------------------------------------------------------------------
template <int ODT, int NJ>
__global__ void __launch_bounds__(NT) k_dequantize(TqDequantizeJob job) {
  extern __shared__ __align__(16) float smem[];
  const int D = job.D;
  const int lda = lda_for(D);
  float* As = smem;
  float* Bs = As + TM * lda;
  float* cent_s = Bs + KC * (64 * NJ + BPAD);
  float* thr_s = cent_s + 256;
  load_codebook(job.codebook, cent_s, thr_s);
  const int64_t n_total = job.B * job.H * job.S;
  const int64_t tiles = (n_total + TM - 1) / TM;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int kpad = round_up(D, KC);
  for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const int64_t row0 = tile * TM;
    __syncthreads();
    for (int r = warp; r < TM; r += NT / 32) {
      int64_t n = row0 + r;
      for (int c = lane; c < kpad; c += 32) {
        float v = 0.f;
        if (n < n_total && c < D) v = cent_s[fetch_index(job.idx, job.idx_mode, n, c, D, job.bits)];
        As[r * lda + c] = v;
      }
    }
    float acc[4][4 * NJ];
    zero_acc<NJ>(acc);
    tile_gemm<NJ, B_KN>(As, lda, D, job.rotation, D, D, Bs, acc);
#pragma unroll
    for (int ri = 0; ri < 4; ++ri) {
      int64_t n = row0 + ty * 4 + ri;
      if (n >= n_total) continue;
      float nv = (job.norms != nullptr) ? __half2float(__ushort_as_half(job.norms[n])) : 1.f;
      int64_t off = vec_offset(n, job.H, job.S, job.ostride_b, job.ostride_h, job.ostride_s);
#pragma unroll
      for (int j = 0; j < NJ; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          int col = tx * 4 + 64 * j + c;
          if (col < D) {
            float v = (job.norms != nullptr) ? acc[ri][4 * j + c] * nv : acc[ri][4 * j + c];
            store_elem<ODT>(job.out, off + col, v);
          }
        }
    }
  }
}

// ---------------------------------------------------------------------------
// generic projection out = x @ m
// ---------------------------------------------------------------------------
template <int XDT, int NJ>
__global__ void __launch_bounds__(NT) k_project(const void* x, int64_t n_total, int K, const float* m, int N,
                                                float* out) {
  extern __shared__ __align__(16) float smem[];
  const int lda = lda_for(K);
  float* As = smem;
  float* Bs = As + TM * lda;
  const int64_t tiles = (n_total + TM - 1) / TM;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const int64_t row0 = tile * TM;
    __syncthreads();
    load_tile_rows<XDT>(x, row0, n_total, K, 1, n_total, 0, 0, K, As, lda, nullptr);
    float acc[4][4 * NJ];
    zero_acc<NJ>(acc);
    tile_gemm<NJ, B_KN>(As, lda, K, m, N, N, Bs, acc);
#pragma unroll
    for (int ri = 0; ri < 4; ++ri) {
      int64_t n = row0 + ty * 4 + ri;
      if (n >= n_total) continue;
#pragma unroll
      for (int j = 0; j < NJ; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          int col = tx * 4 + 64 * j + c;
          if (col < N) out[n * N + col] = acc[ri][4 * j + c];
        }
    }
  }
}

// ---------------------------------------------------------------------------
// K3: logits from packed keys.  One thread per key, RQ query rows at a time.
// qrot: (B, Hq, Sq, D) rotated queries.  stats: per (row, key block) {max, sum}.
// ---------------------------------------------------------------------------
constexpr int RQ = 4;
constexpr int SCORE_KEYS_PER_BLOCK = 1024;

__global__ void __launch_bounds__(NT) k_score_packed(TqScoreJob job, const float* __restrict__ qrot, float* stats,
                                                    int nblk) {
  __shared__ float cent_s[256];
  __shared__ __align__(16) float qs[TQ_MAX_DIM * RQ];
  __shared__ float red[NT / 32][RQ];
  const int D = job.D, bits = job.bits;
  const int ipb = 8 / bits;
  const int G = (D + ipb - 1) / ipb;
  const unsigned mask = (1u << bits) - 1u;
  for (int i = threadIdx.x; i < 256; i += NT) cent_s[i] = __ldg(job.codebook + kCentroidOff + i);
  const int blk = blockIdx.x % nblk;
  const int64_t bh = blockIdx.x / nblk;           // b * Hkv + hkv
  const int64_t b = bh / job.Hkv, hkv = bh % job.Hkv;
  const int rep = (int)(job.Hq / job.Hkv);
  const int R = rep * (int)job.Sq;               // query rows that read this KV head
  const int64_t s_begin = (int64_t)blk * SCORE_KEYS_PER_BLOCK;
  const int64_t s_end = min(s_begin + SCORE_KEYS_PER_BLOCK, job.Sk);
  const uint8_t* keys = job.idx_bytes + bh * job.Sk * G;
  const uint16_t* norms = job.norms + bh * job.Sk;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int r0 = 0; r0 < R; r0 += RQ) {
    __syncthreads();
    // stage RQ rotated query rows as qs[j][rq]
    for (int e = threadIdx.x; e < D * RQ; e += NT) {
      int j = e / RQ, rq = e % RQ;
      int r = r0 + rq;
      float v = 0.f;
      if (r < R) {
        int64_t hq = hkv * rep + r / job.Sq, sq = r % job.Sq;
        v = qrot[((b * job.Hq + hq) * job.Sq + sq) * D + j];
      }
      qs[e] = v;
    }
    __syncthreads();
    float run_max[RQ], run_sum[RQ];
#pragma unroll
    for (int rq = 0; rq < RQ; ++rq) { run_max[rq] = -INFINITY; run_sum[rq] = 0.f; }
    for (int64_t s0 = s_begin; s0 < s_end; s0 += NT) {
      int64_t s = s0 + threadIdx.x;
      float acc[RQ] = {0.f, 0.f, 0.f, 0.f};
      if (s < s_end) {
        const uint8_t* row = keys + s * G;
        for (int g = 0; g < G; ++g) {
          unsigned byte = row[g];
          for (int i = 0; i < ipb; ++i) {
            int j = g * ipb + i;
            if (j < D) {
              float c = cent_s[(byte >> (bits * (ipb - 1 - i))) & mask];
              float4 qv = *reinterpret_cast<const float4*>(qs + j * RQ);
              acc[0] = fmaf(qv.x, c, acc[0]);
              acc[1] = fmaf(qv.y, c, acc[1]);
              acc[2] = fmaf(qv.z, c, acc[2]);
              acc[3] = fmaf(qv.w, c, acc[3]);
            }
          }
        }
        float nv = __half2float(__ushort_as_half(norms[s]));
#pragma unroll
        for (int rq = 0; rq < RQ; ++rq) {
          int r = r0 + rq;
          if (r < R) {
            float l = acc[rq] * nv * job.scale;
            int64_t hq = hkv * rep + r / job.Sq, sq = r % job.Sq;
            job.logits[((b * job.Hq + hq) * job.Sq + sq) * job.Sk + s] = l;
            acc[rq] = l;
          }
        }
      }
      if (stats != nullptr) {
        // online (max, sum exp) per row over this thread's keys
#pragma unroll
        for (int rq = 0; rq < RQ; ++rq) {
          if (s < s_end && r0 + rq < R) {
            float l = acc[rq];
            float m = fmaxf(run_max[rq], l);
            if (m == -INFINITY) {
              run_sum[rq] += 0.f;
            } else {
              run_sum[rq] = run_sum[rq] * __expf(run_max[rq] - m) + __expf(l - m);
            }
            run_max[rq] = m;
          }
        }
      }
    }
    if (stats != nullptr) {
#pragma unroll
      for (int rq = 0; rq < RQ; ++rq) {
        float m = warp_max(run_max[rq]);
        float sc = (run_max[rq] == -INFINITY) ? 0.f : run_sum[rq] * __expf(run_max[rq] - m);
        float sm = warp_sum(sc);
        if (lane == 0) { red[warp][rq] = m; }
        __syncthreads();
        float bm = -INFINITY;
        for (int w = 0; w < NT / 32; ++w) bm = fmaxf(bm, red[w][rq]);
        __syncthreads();
        float contrib = (m == -INFINITY) ? 0.f : sm * __expf(m - bm);
        if (lane == 0) red[warp][rq] = contrib;
        __syncthreads();
        if (threadIdx.x == 0 && r0 + rq < R) {
          float tot = 0.f;
          for (int w = 0; w < NT / 32; ++w) tot += red[w][rq];
          int r = r0 + rq;
          int64_t hq = hkv * rep + r / job.Sq, sq = r % job.Sq;
          int64_t grow = (b * job.Hq + hq) * job.Sq + sq;
          stats[(grow * nblk + blk) * 2 + 0] = bm;
          stats[(grow * nblk + blk) * 2 + 1] = tot;
        }
        __syncthreads();
      }
    }
  }
}

// y = x @ m for up to a few thousand rows (queries): one block per RPB rows, one thread per
// output coordinate, the same sequential-k fma order as the tiled contraction.  A matrix
// element is loaded once and used for all RPB rows of the block.
template <int XDT, int RPB>
__global__ void k_project_rows(const void* x, int64_t n, int K, const float* __restrict__ m, int N, float* out) {
  __shared__ float xs[RPB][TQ_MAX_DIM];
  const int64_t row0 = (int64_t)blockIdx.x * RPB;
#pragma unroll
  for (int r = 0; r < RPB; ++r)
    for (int k = threadIdx.x; k < K; k += blockDim.x) xs[r][k] = row0 + r < n ? load_elem<XDT>(x, (row0 + r) * K + k) : 0.f;
  __syncthreads();
  for (int col = threadIdx.x; col < N; col += blockDim.x) {
    float acc[RPB];
#pragma unroll
    for (int r = 0; r < RPB; ++r) acc[r] = 0.f;
    int k = 0;
    constexpr int kBatch = RPB == 1 ? 64 : 16;   // independent loads in flight before the ordered fma chains
    for (; k + kBatch <= K; k += kBatch) {
      float mv[kBatch];
#pragma unroll
      for (int u = 0; u < kBatch; ++u) mv[u] = __ldg(m + (int64_t)(k + u) * N + col);
#pragma unroll
      for (int u = 0; u < kBatch; ++u)
#pragma unroll
        for (int r = 0; r < RPB; ++r) acc[r] = fmaf(xs[r][k + u], mv[u], acc[r]);
    }
    for (; k < K; ++k) {
      const float mv = __ldg(m + (int64_t)k * N + col);
#pragma unroll
      for (int r = 0; r < RPB; ++r) acc[r] = fmaf(xs[r][k], mv, acc[r]);
    }
#pragma unroll
    for (int r = 0; r < RPB; ++r)
      if (row0 + r < n) out[(row0 + r) * N + col] = acc[r];
  }
}

// head_dim 128 specialisation: a thread owns whole keys (two at a time, 64 keys per warp and
// round), so no partial sums cross lanes.  The packed row is read in 16-byte pieces; for every
// coordinate the centroid comes from a shared look-up (byte offsets prepared a word at a
// time, so the load is [register + constant]) and the four rotated query values of that
// coordinate come from one broadcast 16-byte shared load, used for both keys.  Lane L holds
// the logits of keys L and L + 32 of the round, so logits leave as 128-byte rows and the
// softmax partials are per lane.
__device__ __forceinline__ float lds_f32(uint32_t addr) {
  float v;
  asm("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}

// Shared-memory addresses of the centroids of the CPW coordinates packed in one 32-bit word,
// in coordinate order.  `base` is the shared address of the table, aligned to 1024 bytes, so
// it can be merged into the byte offsets (index * 4) by the same permute / logic instruction
// that isolates them: no separate address addition per look-up.
template <int BITS>
__device__ __forceinline__ void word_offsets(uint32_t x, uint32_t base, uint32_t (&off)[4 * (8 / BITS)]) {
  constexpr int IPB = 8 / BITS;
  constexpr int CPW = 4 * IPB;
  constexpr uint32_t MASK = (1u << BITS) - 1u;
  if constexpr (BITS == 4) {
    const uint32_t even = (x >> 2) & 0x3C3C3C3Cu, odd = (x << 2) & 0x3C3C3C3Cu;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      off[2 * k] = __byte_perm(even, base, 0x7650u | k);       // byte k of `even` under bytes 1..3 of base
      off[2 * k + 1] = __byte_perm(odd, base, 0x7650u | k);
    }
  } else if constexpr (BITS == 2) {
    const uint32_t f0 = (x >> 4) & 0x0C0C0C0Cu, f1 = (x >> 2) & 0x0C0C0C0Cu, f2 = x & 0x0C0C0C0Cu, f3 = (x << 2) & 0x0C0C0C0Cu;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      off[4 * k] = __byte_perm(f0, base, 0x7650u | k);
      off[4 * k + 1] = __byte_perm(f1, base, 0x7650u | k);
      off[4 * k + 2] = __byte_perm(f2, base, 0x7650u | k);
      off[4 * k + 3] = __byte_perm(f3, base, 0x7650u | k);
    }
  } else {
#pragma unroll
    for (int u = 0; u < CPW; ++u) {
      const int byte = u / IPB;
      const int sh = 8 * byte + BITS * (IPB - 1 - (u % IPB));
      off[u] = (sh >= 2 ? ((x >> (sh - 2)) & (MASK << 2)) : ((x << (2 - sh)) & (MASK << 2))) | base;
    }
  }
}

template <int BITS>
__global__ void __launch_bounds__(NT) k_score_packed_d128(TqScoreJob job, const float* __restrict__ qrot, float* stats,
                                                         int nblk) {
  constexpr int D = 128;
  constexpr int IPB = 8 / BITS;
  constexpr int G = D / IPB;                     // packed bytes per key: 16, 32, 64 or 128
  constexpr int PIECES = G / 16;                 // 16-byte pieces per key
  constexpr int CPW = 4 * IPB;                   // coordinates per 32-bit word
  __shared__ __align__(1024) float cent_s[256];
  __shared__ float4 q_s[D];
  __shared__ float red[NT / 32][RQ];
  for (int i = threadIdx.x; i < 256; i += NT) cent_s[i] = __ldg(job.codebook + kCentroidOff + i);
  const uint32_t cent_base = (uint32_t)__cvta_generic_to_shared(cent_s);
  const int blk = blockIdx.x % nblk;
  const int64_t bh = blockIdx.x / nblk;
  const int64_t b = bh / job.Hkv, hkv = bh % job.Hkv;
  const int rep = (int)(job.Hq / job.Hkv);
  const int R = rep * (int)job.Sq;
  const int64_t s_begin = (int64_t)blk * SCORE_KEYS_PER_BLOCK;
  const int64_t s_end = min(s_begin + SCORE_KEYS_PER_BLOCK, job.Sk);
  const uint8_t* keys = job.idx_bytes + bh * job.Sk * G;
  const uint16_t* norms = job.norms + bh * job.Sk;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int r0 = 0; r0 < R; r0 += RQ) {
    int64_t out_row[RQ];
#pragma unroll
    for (int rq = 0; rq < RQ; ++rq) {
      const int r = r0 + rq;
      int64_t grow = 0;
      if (r < R) {
        const int64_t hq = hkv * rep + r / job.Sq, sq = r % job.Sq;
        grow = (b * job.Hq + hq) * job.Sq + sq;
      }
      out_row[rq] = grow;
    }
    __syncthreads();                             // the previous group's readers of q_s are done
#pragma unroll
    for (int rq = 0; rq < RQ; ++rq)
      for (int e = threadIdx.x; e < D; e += NT)
        reinterpret_cast<float*>(q_s)[e * RQ + rq] = (r0 + rq < R) ? __ldg(qrot + out_row[rq] * D + e) : 0.f;
    __syncthreads();
    float run_max[RQ], run_sum[RQ];
#pragma unroll
    for (int rq = 0; rq < RQ; ++rq) { run_max[rq] = -INFINITY; run_sum[rq] = 0.f; }
    for (int64_t kb = s_begin + warp * 64; kb < s_end; kb += (NT / 32) * 64) {
      const int64_t key_a = kb + lane, key_b = kb + 32 + lane;
      const bool ok_a = key_a < s_end, ok_b = key_b < s_end;
      const uint4* src_a = reinterpret_cast<const uint4*>(keys + (ok_a ? key_a : s_begin) * G);
      const uint4* src_b = reinterpret_cast<const uint4*>(keys + (ok_b ? key_b : s_begin) * G);
      float acc_a[RQ] = {0.f, 0.f, 0.f, 0.f}, acc_b[RQ] = {0.f, 0.f, 0.f, 0.f};
      uint4 cur_a = __ldg(src_a), cur_b = __ldg(src_b);
#pragma unroll 1
      for (int pc = 0; pc < PIECES; ++pc) {
        uint4 nxt_a = cur_a, nxt_b = cur_b;
        if (pc + 1 < PIECES) { nxt_a = __ldg(src_a + pc + 1); nxt_b = __ldg(src_b + pc + 1); }
        const float4* qp = q_s + pc * 4 * CPW;
        const uint32_t wa[4] = {cur_a.x, cur_a.y, cur_a.z, cur_a.w};
        const uint32_t wb[4] = {cur_b.x, cur_b.y, cur_b.z, cur_b.w};
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          uint32_t oa[CPW], ob[CPW];
          word_offsets<BITS>(wa[w], cent_base, oa);
          word_offsets<BITS>(wb[w], cent_base, ob);
#pragma unroll
          for (int u = 0; u < CPW; ++u) {
            const float4 q = qp[w * CPW + u];
            const float ca = lds_f32(oa[u]), cb = lds_f32(ob[u]);
            acc_a[0] = fmaf(q.x, ca, acc_a[0]); acc_a[1] = fmaf(q.y, ca, acc_a[1]);
            acc_a[2] = fmaf(q.z, ca, acc_a[2]); acc_a[3] = fmaf(q.w, ca, acc_a[3]);
            acc_b[0] = fmaf(q.x, cb, acc_b[0]); acc_b[1] = fmaf(q.y, cb, acc_b[1]);
            acc_b[2] = fmaf(q.z, cb, acc_b[2]); acc_b[3] = fmaf(q.w, cb, acc_b[3]);
          }
        }
        cur_a = nxt_a; cur_b = nxt_b;
      }
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int64_t key = half ? key_b : key_a;
        if (half ? ok_b : ok_a) {
          const float nv = __half2float(__ushort_as_half(norms[key]));
#pragma unroll
          for (int rq = 0; rq < RQ; ++rq) {
            if (r0 + rq < R) {
              const float l = (half ? acc_b[rq] : acc_a[rq]) * nv * job.scale;
              job.logits[out_row[rq] * job.Sk + key] = l;
              if (stats != nullptr) {
                const float m = fmaxf(run_max[rq], l);
                if (m != -INFINITY) run_sum[rq] = run_sum[rq] * __expf(run_max[rq] - m) + __expf(l - m);
                run_max[rq] = m;
              }
            }
          }
        }
      }
    }
    if (stats != nullptr) {
#pragma unroll
      for (int rq = 0; rq < RQ; ++rq) {
        const float m = warp_max(run_max[rq]);
        const float sc = (run_max[rq] == -INFINITY) ? 0.f : run_sum[rq] * __expf(run_max[rq] - m);
        const float sm = warp_sum(sc);
        if (lane == 0) red[warp][rq] = m;
        __syncthreads();
        float bm = -INFINITY;
        for (int w = 0; w < NT / 32; ++w) bm = fmaxf(bm, red[w][rq]);
        __syncthreads();
        const float contrib = (m == -INFINITY) ? 0.f : sm * __expf(m - bm);
        if (lane == 0) red[warp][rq] = contrib;
        __syncthreads();
        if (threadIdx.x == 0 && r0 + rq < R) {
          float tot = 0.f;
          for (int w = 0; w < NT / 32; ++w) tot += red[w][rq];
          stats[(out_row[rq] * nblk + blk) * 2 + 0] = bm;
          stats[(out_row[rq] * nblk + blk) * 2 + 1] = tot;
        }
        __syncthreads();
      }
    }
  }
}

// probs = exp(l - M) / Z with (M, Z) folded from the per-block partials.
__global__ void __launch_bounds__(NT) k_softmax_finish(const float* __restrict__ logits, const float* __restrict__ stats,
                                                      int nblk, int64_t Sk, float* probs) {
  __shared__ float sh_m, sh_z;
  const int64_t row = blockIdx.x;
  if (threadIdx.x < 32) {
    float m = -INFINITY;
    for (int i = threadIdx.x; i < nblk; i += 32) m = fmaxf(m, stats[(row * nblk + i) * 2]);
    m = warp_max(m);
    float z = 0.f;
    for (int i = threadIdx.x; i < nblk; i += 32) {
      float pm = stats[(row * nblk + i) * 2];
      if (pm != -INFINITY) z += stats[(row * nblk + i) * 2 + 1] * __expf(pm - m);
    }
    z = warp_sum(z);
    if (threadIdx.x == 0) { sh_m = m; sh_z = z; }
  }
  __syncthreads();
  const float m = sh_m, inv = 1.f / sh_z;
  const int64_t per = ((Sk + gridDim.y - 1) / gridDim.y + 3) / 4 * 4;
  const int64_t lo = blockIdx.y * per, hi = min(lo + per, Sk);
  const float* src = logits + row * Sk;
  float* dst = probs + row * Sk;
  if ((Sk & 3) == 0 && (((uintptr_t)src | (uintptr_t)dst) & 15u) == 0) {     // 16-byte rows: four logits per access
    for (int64_t s = lo + 4 * (int64_t)threadIdx.x; s < hi; s += 4 * NT) {
      const float4 l = *reinterpret_cast<const float4*>(src + s);
      float4 p;
      p.x = __expf(l.x - m) * inv; p.y = __expf(l.y - m) * inv; p.z = __expf(l.z - m) * inv; p.w = __expf(l.w - m) * inv;
      *reinterpret_cast<float4*>(dst + s) = p;
    }
  } else {
    for (int64_t s = lo + threadIdx.x; s < hi; s += NT) dst[s] = __expf(src[s] - m) * inv;
  }
}

// ---------------------------------------------------------------------------
// K4: MSE stage + QJL signs on one resident tile
// ---------------------------------------------------------------------------
template <int XDT, int NJ, int NJM>
__global__ void __launch_bounds__(NT) k_qjl_compress(TqQjlCompressJob job) {
  extern __shared__ __align__(16) float smem[];
  const int D = job.D, M = job.M;
  const int lda = lda_for(D);
  constexpr int NJB = (NJ > NJM) ? NJ : NJM;
  float* Xs = smem;
  float* As = Xs + TM * lda;
  float* Bs = As + TM * lda;
  float* cent_s = Bs + KC * (64 * NJB + BPAD);
  float* thr_s = cent_s + 256;
  float* nrm = thr_s + 256;
  load_codebook(job.codebook, cent_s, thr_s);
  const int64_t n_total = job.B * job.H * job.S;
  const int64_t tiles = (n_total + TM - 1) / TM;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int kpad = round_up(D, KC);
  const int levels = 1 << job.bits;
  for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const int64_t row0 = tile * TM;
    __syncthreads();
    load_tile_rows<XDT>(job.x, row0, n_total, D, job.H, job.S, job.stride_b, job.stride_h, job.stride_s, Xs, lda,
                        job.normalize ? nrm : nullptr);
    __syncwarp();
    for (int r = warp; r < TM; r += NT / 32) {
      float den = job.normalize ? nrm[r] + 1e-8f : 1.f;
      for (int k = lane; k < kpad; k += 32)
        As[r * lda + k] = job.normalize ? __fdiv_rn(Xs[r * lda + k], den) : Xs[r * lda + k];
    }
    {
      float acc[4][4 * NJ];
      zero_acc<NJ>(acc);
      tile_gemm<NJ, B_KN>(As, lda, D, job.rotation_t, D, D, Bs, acc);
      __syncthreads();
      acc_to_smem<NJ>(acc, As, lda, kpad);
    }
    __syncthreads();
    // quantise in place: As <- centroid of the nearest level
    for (int r = warp; r < TM; r += NT / 32) {
      int64_t n = row0 + r;
      for (int c = lane; c < kpad; c += 32) {
        float v = 0.f;
        if (c < D) {
          int q = quantize_scalar(As[r * lda + c], thr_s, levels);
          v = cent_s[q];
          if (job.idx_out != nullptr && n < n_total) {
            if (job.idx_mode == TQ_IDX_I64) reinterpret_cast<int64_t*>(job.idx_out)[n * D + c] = q;
            else if (job.idx_mode == TQ_IDX_U8) reinterpret_cast<uint8_t*>(job.idx_out)[n * D + c] = (uint8_t)q;
          }
        }
        As[r * lda + c] = v;
      }
    }
    {
      float acc[4][4 * NJ];
      zero_acc<NJ>(acc);
      tile_gemm<NJ, B_KN>(As, lda, D, job.rotation, D, D, Bs, acc);
      __syncthreads();
      // k_mse (fp32) -> optional fp16 output; residual = x - k_mse back into As
#pragma unroll
      for (int ri = 0; ri < 4; ++ri) {
        int r = ty * 4 + ri;
        int64_t n = row0 + r;
        float nv = job.normalize ? nrm[r] : 1.f;
#pragma unroll
        for (int j = 0; j < NJ; ++j)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            int col = tx * 4 + 64 * j + c;
            if (col < kpad) {
              float km = job.normalize ? acc[ri][4 * j + c] * nv : acc[ri][4 * j + c];
              if (col >= D) km = 0.f;
              if (job.k_mse_out != nullptr && n < n_total && col < D)
                job.k_mse_out[n * D + col] = __half_as_ushort(__float2half_rn(km));
              As[r * lda + col] = (col < D) ? Xs[r * lda + col] - km : 0.f;
            }
          }
      }
    }
    __syncthreads();
    for (int r = warp; r < TM; r += NT / 32) {
      float ssq = 0.f;
      for (int k = lane; k < D; k += 32) ssq = fmaf(As[r * lda + k], As[r * lda + k], ssq);
      ssq = warp_sum(ssq);
      int64_t n = row0 + r;
      if (lane == 0 && n < n_total) {
        float rn = __fsqrt_rn(ssq);
        if (job.rnorm_dtype == TQ_F16) reinterpret_cast<uint16_t*>(job.rnorm_out)[n] = __half_as_ushort(__float2half_rn(rn));
        else reinterpret_cast<float*>(job.rnorm_out)[n] = rn;
        if (job.vec_norms_out != nullptr && job.normalize) job.vec_norms_out[n] = nrm[r];
      }
    }
    {
      float acc[4][4 * NJM];
      zero_acc<NJM>(acc);
      tile_gemm<NJM, B_KN>(As, lda, D, job.qjl_t, M, M, Bs, acc);
#pragma unroll
      for (int ri = 0; ri < 4; ++ri) {
        int64_t n = row0 + ty * 4 + ri;
        if (n >= n_total) continue;
#pragma unroll
        for (int j = 0; j < NJM; ++j)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            int col = tx * 4 + 64 * j + c;
            if (col < M) {
              float p = acc[ri][4 * j + c];
              if (job.signs_dtype == 0) {
                reinterpret_cast<int8_t*>(job.signs_out)[n * M + col] = (p >= 0.f) ? (int8_t)1 : (int8_t)-1;
              } else {
                float sg = (p > 0.f) ? 1.f : (p < 0.f) ? -1.f : (p == 0.f) ? 1.f : p;
                reinterpret_cast<float*>(job.signs_out)[n * M + col] = sg;
              }
            }
          }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// K5: scores = Q k_mse^T + sqrt(pi/2)/m * (Q S^T) signs^T * ||r||
// Tile rows are keys; columns are queries (chunks of up to 256).
// ---------------------------------------------------------------------------
template <int QDT, int NJ>
__global__ void __launch_bounds__(NT) k_qjl_scores(TqQjlScoreJob job, const float* __restrict__ qproj, float corr) {
  extern __shared__ __align__(16) float smem[];
  const int D = job.D;
  const int lda = lda_for(D);
  float* As = smem;
  float* Bs = As + TM * lda;
  float* Cs = Bs + KC * (64 * NJ + BPAD);   // [64*NJ][TM+1]
  const int ldc = TM + 1;
  const int64_t key_tiles = (job.Sk + TM - 1) / TM;
  const int64_t total = job.BH * key_tiles;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int kpad = round_up(D, KC);
  for (int64_t t = blockIdx.x; t < total; t += gridDim.x) {
    const int64_t bh = t / key_tiles;
    const int64_t s0 = (t % key_tiles) * TM;
    const uint16_t* km = job.k_mse + (bh * job.Sk) * D;
    const int8_t* sg = job.signs + (bh * job.Sk) * D;
    for (int q0 = 0; q0 < job.Sq; q0 += 64 * NJ) {
      const int nq = (int)min((int64_t)(64 * NJ), job.Sq - q0);
      float acc1[4][4 * NJ], acc2[4][4 * NJ];
      zero_acc<NJ>(acc1);
      zero_acc<NJ>(acc2);
      __syncthreads();
      for (int r = warp; r < TM; r += NT / 32) {
        int64_t s = s0 + r;
        for (int k = lane; k < kpad; k += 32)
          As[r * lda + k] = (s < job.Sk && k < D) ? __half2float(__ushort_as_half(km[s * D + k])) : 0.f;
      }
      // queries as B in [N][K] layout, converted to fp32 on the fly for 16-bit q
      if constexpr (QDT == TQ_F32) {
        tile_gemm<NJ, B_NK>(As, lda, D, reinterpret_cast<const float*>(job.q) + (bh * job.Sq + q0) * D, D, nq, Bs, acc1);
      } else {
        // 16-bit queries were upcast into the workspace behind qproj by the host wrapper
        tile_gemm<NJ, B_NK>(As, lda, D, qproj + (job.BH * job.Sq + bh * job.Sq + q0) * D, D, nq, Bs, acc1);
      }
      __syncthreads();
      for (int r = warp; r < TM; r += NT / 32) {
        int64_t s = s0 + r;
        for (int k = lane; k < kpad; k += 32) As[r * lda + k] = (s < job.Sk && k < D) ? (float)sg[s * D + k] : 0.f;
      }
      tile_gemm<NJ, B_NK>(As, lda, D, qproj + (bh * job.Sq + q0) * D, D, nq, Bs, acc2);
      __syncthreads();
#pragma unroll
      for (int ri = 0; ri < 4; ++ri) {
        int r = ty * 4 + ri;
        int64_t s = s0 + r;
        float rn = (s < job.Sk) ? __half2float(__ushort_as_half(job.rnorm[bh * job.Sk + s])) : 0.f;
#pragma unroll
        for (int j = 0; j < NJ; ++j)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            int col = tx * 4 + 64 * j + c;
            float t2 = (corr * acc2[ri][4 * j + c]) * rn;
            Cs[col * ldc + r] = acc1[ri][4 * j + c] + t2;
          }
      }
      __syncthreads();
      for (int col = warp; col < nq; col += NT / 32) {
        float* o = job.scores + (bh * job.Sq + q0 + col) * job.Sk + s0;
        for (int r = lane; r < TM; r += 32)
          if (s0 + r < job.Sk) o[r] = Cs[col * ldc + r];
      }
    }
  }
}

// upcast a 16-bit tensor to fp32
template <int XDT>
__global__ void k_upcast(const void* x, int64_t n, float* out) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = load_elem<XDT>(x, i);
}

// out[n] = <y_n, xhat_n> + (rnorm_n * corr) * <sy_n, signs_n>
__global__ void __launch_bounds__(NT) k_prod_inner(const float* __restrict__ y, int64_t ny, const float* __restrict__ xhat,
                                                  const float* __restrict__ sy, const float* __restrict__ signs,
                                                  const float* __restrict__ rnorm, int64_t n, int D, int M, float corr,
                                                  float* out) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t wstride = (int64_t)gridDim.x * (NT / 32);
  for (int64_t r = (int64_t)blockIdx.x * (NT / 32) + warp; r < n; r += wstride) {
    const int64_t yr = (ny == 1) ? 0 : r;
    float t1 = 0.f, ip = 0.f;
    for (int k = lane; k < D; k += 32) t1 = fmaf(y[yr * D + k], xhat[r * D + k], t1);
    for (int k = lane; k < M; k += 32) ip = fmaf(sy[yr * M + k], signs[r * M + k], ip);
    t1 = warp_sum(t1);
    ip = warp_sum(ip);
    if (lane == 0) out[r] = t1 + (rnorm[r] * corr) * ip;
  }
}

// ---------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------
static thread_local int g_last_cuda_error = 0;
static std::atomic<long long> g_launches{0};
int last_cuda_error() { return g_last_cuda_error; }
long long launch_count() { return g_launches.load(); }
void note_cuda_error(int e) { g_last_cuda_error = e; }

int check_launch() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return TQ_ELAUNCH; }
  g_launches.fetch_add(1);
  return TQ_OK;
}

static int sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
  return n;
}

static int grid_for(int64_t tiles, int per_sm) {
  int64_t cap = (int64_t)sm_count() * per_sm;
  return (int)(tiles < cap ? (tiles > 0 ? tiles : 1) : cap);
}

template <typename K>
static int set_smem(K kernel, size_t bytes) {
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) { g_last_cuda_error = (int)e; return TQ_ELAUNCH; }
  }
  return TQ_OK;
}

static inline int nj_for(int n) { return (n + 63) / 64; }

#define TQ_DISPATCH_NJ(nj, ...)                              \
  switch (nj) {                                              \
    case 1: { constexpr int NJ_ = 1; __VA_ARGS__; } break;   \
    case 2: { constexpr int NJ_ = 2; __VA_ARGS__; } break;   \
    case 3: { constexpr int NJ_ = 3; __VA_ARGS__; } break;   \
    default: { constexpr int NJ_ = 4; __VA_ARGS__; } break;  \
  }

#define TQ_DISPATCH_DT(dt, ...)                                         \
  switch (dt) {                                                         \
    case TQ_F32: { constexpr int DT_ = TQ_F32; __VA_ARGS__; } break;    \
    case TQ_F16: { constexpr int DT_ = TQ_F16; __VA_ARGS__; } break;    \
    default: { constexpr int DT_ = TQ_BF16; __VA_ARGS__; } break;       \
  }

int simt_quantize_rotated(const float* y, int64_t n, int D, int bits, const float* cb, int mode, void* out,
                          cudaStream_t st) {
  if (n == 0) return TQ_OK;
  int grid = grid_for((n + NT / 32 - 1) / (NT / 32), 8);
  k_quantize_rotated<<<grid, NT, 0, st>>>(y, n, D, bits, cb, mode, out);
  return check_launch();
}

int simt_quantize(const TqQuantizeJob& job, cudaStream_t st) {
  const int64_t n = job.B * job.H * job.S;
  if (n == 0) return TQ_OK;
  const int nj = nj_for(job.D);
  const size_t smem = sizeof(float) * (TM * lda_for(job.D) + KC * (64 * nj + BPAD) + 512 + TM);
  const int grid = grid_for((n + TM - 1) / TM, 2);
  int rc = TQ_OK;
  TQ_DISPATCH_DT(job.x_dtype, TQ_DISPATCH_NJ(nj, {
    auto kern = k_quantize<DT_, NJ_>;
    rc = set_smem(kern, smem);
    if (rc == TQ_OK) kern<<<grid, NT, smem, st>>>(job);
  }));
  return rc != TQ_OK ? rc : check_launch();
}

int simt_dequantize(const TqDequantizeJob& job, cudaStream_t st) {
  const int64_t n = job.B * job.H * job.S;
  if (n == 0) return TQ_OK;
  const int nj = nj_for(job.D);
  const size_t smem = sizeof(float) * (TM * lda_for(job.D) + KC * (64 * nj + BPAD) + 512);
  const int grid = grid_for((n + TM - 1) / TM, 2);
  int rc = TQ_OK;
  TQ_DISPATCH_DT(job.out_dtype, TQ_DISPATCH_NJ(nj, {
    auto kern = k_dequantize<DT_, NJ_>;
    rc = set_smem(kern, smem);
    if (rc == TQ_OK) kern<<<grid, NT, smem, st>>>(job);
  }));
  return rc != TQ_OK ? rc : check_launch();
}

int simt_project(const void* x, int x_dtype, int64_t n, int K, const float* m, int N, float* out, cudaStream_t st) {
  if (n == 0) return TQ_OK;
  if (n <= 8192) {         // few rows: a 64-row tile kernel would run on a handful of SMs
    const int threads = N <= 128 ? 128 : 256;
    if (n <= 512) {
      TQ_DISPATCH_DT(x_dtype, (k_project_rows<DT_, 1><<<(unsigned)n, threads, 0, st>>>(x, n, K, m, N, out)));
    } else {
      TQ_DISPATCH_DT(x_dtype, (k_project_rows<DT_, 4><<<(unsigned)((n + 3) / 4), threads, 0, st>>>(x, n, K, m, N, out)));
    }
    return check_launch();
  }
  const int nj = nj_for(N);
  const size_t smem = sizeof(float) * (TM * lda_for(K) + KC * (64 * nj + BPAD));
  const int grid = grid_for((n + TM - 1) / TM, 2);
  int rc = TQ_OK;
  TQ_DISPATCH_DT(x_dtype, TQ_DISPATCH_NJ(nj, {
    auto kern = k_project<DT_, NJ_>;
    rc = set_smem(kern, smem);
    if (rc == TQ_OK) kern<<<grid, NT, smem, st>>>(x, n, K, m, N, out);
  }));
  return rc != TQ_OK ? rc : check_launch();
}

size_t simt_score_workspace(int64_t B, int64_t Hq, int64_t Sq, int64_t Sk, int D) {
  const int64_t rows = B * Hq * Sq;
  const int64_t nblk = (Sk + SCORE_KEYS_PER_BLOCK - 1) / SCORE_KEYS_PER_BLOCK;
  size_t q = (size_t)rows * D * sizeof(float);
  q = (q + 255) / 256 * 256;
  return q + (size_t)rows * (nblk > 0 ? nblk : 1) * 2 * sizeof(float);
}

int simt_score_packed(const TqScoreJob& job, cudaStream_t st) {
  const int64_t rows = job.B * job.Hq * job.Sq;
  if (rows == 0 || job.Sk == 0) return TQ_OK;
  // the tensor-core kernel takes its block size as a parameter: blocks of at least SCORE_KEYS_PER_BLOCK keys (the
  // scratch is sized for that) chosen so that the CTAs fill whole waves
  const bool use_mma = mma_score_eligible(job);
  const int kpb = use_mma ? mma_score_keys_per_block(job, SCORE_KEYS_PER_BLOCK) : SCORE_KEYS_PER_BLOCK;
  const int nblk = (int)((job.Sk + kpb - 1) / kpb);
  float* qrot = reinterpret_cast<float*>(job.workspace);
  size_t qbytes = ((size_t)rows * job.D * sizeof(float) + 255) / 256 * 256;
  float* stats = reinterpret_cast<float*>(reinterpret_cast<char*>(job.workspace) + qbytes);
  int rc = simt_project(job.q, job.q_dtype, rows, job.D, job.rotation_t, job.D, qrot, st);
  if (rc != TQ_OK) return rc;
  const int64_t blocks = job.B * job.Hkv * nblk;
  float* st_ptr = job.probs != nullptr ? stats : nullptr;
  if (use_mma) {
    rc = mma_score_packed(job, qrot, st_ptr, nblk, kpb, st);
    if (rc != TQ_OK) return rc;
  } else if (job.D == 128 && ((uintptr_t)job.idx_bytes & 15u) == 0) {
    switch (job.bits) {
      case 1: k_score_packed_d128<1><<<(unsigned)blocks, NT, 0, st>>>(job, qrot, st_ptr, nblk); break;
      case 2: k_score_packed_d128<2><<<(unsigned)blocks, NT, 0, st>>>(job, qrot, st_ptr, nblk); break;
      case 3: k_score_packed_d128<3><<<(unsigned)blocks, NT, 0, st>>>(job, qrot, st_ptr, nblk); break;
      case 4: k_score_packed_d128<4><<<(unsigned)blocks, NT, 0, st>>>(job, qrot, st_ptr, nblk); break;
      case 5: k_score_packed_d128<5><<<(unsigned)blocks, NT, 0, st>>>(job, qrot, st_ptr, nblk); break;
      case 6: k_score_packed_d128<6><<<(unsigned)blocks, NT, 0, st>>>(job, qrot, st_ptr, nblk); break;
      case 7: k_score_packed_d128<7><<<(unsigned)blocks, NT, 0, st>>>(job, qrot, st_ptr, nblk); break;
      default: k_score_packed_d128<8><<<(unsigned)blocks, NT, 0, st>>>(job, qrot, st_ptr, nblk); break;
    }
  } else {
    k_score_packed<<<(unsigned)blocks, NT, 0, st>>>(job, qrot, st_ptr, nblk);
  }
  if (!use_mma) rc = check_launch();
  if (rc != TQ_OK || job.probs == nullptr) return rc;
  int chunks = (int)((job.Sk + 4095) / 4096);
  dim3 grid((unsigned)rows, (unsigned)chunks);
  k_softmax_finish<<<grid, NT, 0, st>>>(job.logits, stats, nblk, job.Sk, job.probs);
  return check_launch();
}

int simt_qjl_compress(const TqQjlCompressJob& job, cudaStream_t st) {
  const int64_t n = job.B * job.H * job.S;
  if (n == 0) return TQ_OK;
  const int nj = nj_for(job.D), njm = nj_for(job.M);
  const int njb = nj > njm ? nj : njm;
  const size_t smem = sizeof(float) * (2 * TM * lda_for(job.D) + KC * (64 * njb + BPAD) + 512 + TM);
  const int grid = grid_for((n + TM - 1) / TM, 1);
  int rc = TQ_OK;
  // the projection width shares the head_dim's tile class unless it is wider
  TQ_DISPATCH_DT(job.x_dtype, TQ_DISPATCH_NJ(njb, {
    auto kern = k_qjl_compress<DT_, NJ_, NJ_>;
    rc = set_smem(kern, smem);
    if (rc == TQ_OK) kern<<<grid, NT, smem, st>>>(job);
  }));
  return rc != TQ_OK ? rc : check_launch();
}

size_t simt_qjl_scores_workspace(int64_t BH, int64_t Sq, int D) {
  return (size_t)2 * BH * Sq * D * sizeof(float);   // projected queries + room for upcast queries
}

int simt_qjl_queries(const TqQjlScoreJob& job, const float** qf_out, const float** qproj_out, cudaStream_t st) {
  float* qproj = reinterpret_cast<float*>(job.workspace);
  const int64_t nq = job.BH * job.Sq;
  int rc = simt_project(job.q, job.q_dtype, nq, job.D, job.qjl_t, job.D, qproj, st);
  if (rc != TQ_OK) return rc;
  const float* qf = reinterpret_cast<const float*>(job.q);
  if (job.q_dtype != TQ_F32) {
    float* up = qproj + nq * job.D;
    int g = grid_for((nq * job.D + 255) / 256, 8);
    if (job.q_dtype == TQ_F16) k_upcast<TQ_F16><<<g, 256, 0, st>>>(job.q, nq * job.D, up);
    else k_upcast<TQ_BF16><<<g, 256, 0, st>>>(job.q, nq * job.D, up);
    rc = check_launch();
    if (rc != TQ_OK) return rc;
    qf = up;
  }
  *qf_out = qf;
  *qproj_out = qproj;
  return TQ_OK;
}

int simt_qjl_scores(const TqQjlScoreJob& job, cudaStream_t st) {
  if (job.BH == 0 || job.Sq == 0 || job.Sk == 0) return TQ_OK;
  const float* qf_unused = nullptr;
  const float* qproj_c = nullptr;
  int rc = simt_qjl_queries(job, &qf_unused, &qproj_c, st);
  if (rc != TQ_OK) return rc;
  const float* qproj = qproj_c;
  const int nj = nj_for((int)(job.Sq < 256 ? job.Sq : 256));
  const size_t smem = sizeof(float) * (TM * lda_for(job.D) + KC * (64 * nj + BPAD) + 64 * nj * (TM + 1));
  const int64_t tiles = job.BH * ((job.Sk + TM - 1) / TM);
  const int grid = grid_for(tiles, 1);
  const float corr = (float)(1.2533141373155001 / (double)job.D);   // sqrt(pi/2) / m with m = D
  if (job.q_dtype == TQ_F32) {
    TQ_DISPATCH_NJ(nj, {
      auto kern = k_qjl_scores<TQ_F32, NJ_>;
      rc = set_smem(kern, smem);
      if (rc == TQ_OK) kern<<<grid, NT, smem, st>>>(job, qproj, corr);
    });
  } else {
    TQ_DISPATCH_NJ(nj, {
      auto kern = k_qjl_scores<TQ_F16, NJ_>;
      rc = set_smem(kern, smem);
      if (rc == TQ_OK) kern<<<grid, NT, smem, st>>>(job, qproj, corr);
    });
  }
  return rc != TQ_OK ? rc : check_launch();
}

int simt_prod_inner_product(const float* y, int64_t ny, const int64_t* idx, const float* signs, const float* rnorm,
                            int64_t n, int D, int M, const float* rotation, const float* codebook, const float* qjl_t,
                            float* out, void* workspace, cudaStream_t st) {
  if (n == 0) return TQ_OK;
  float* xhat = reinterpret_cast<float*>(workspace);
  float* sy = xhat + n * 256;
  TqDequantizeJob dj{};
  dj.idx = idx; dj.norms = nullptr; dj.idx_mode = TQ_IDX_I64; dj.D = D; dj.bits = 8; dj.out_dtype = TQ_F32;
  dj.B = 1; dj.H = 1; dj.S = n; dj.out = xhat; dj.ostride_b = 0; dj.ostride_h = 0; dj.ostride_s = D;
  dj.rotation = rotation; dj.codebook = codebook;
  int rc = simt_dequantize(dj, st);
  if (rc != TQ_OK) return rc;
  rc = simt_project(y, TQ_F32, ny, D, qjl_t, M, sy, st);
  if (rc != TQ_OK) return rc;
  const float corr = (float)(1.2533141373155001 / (double)M);
  int grid = grid_for((n + NT / 32 - 1) / (NT / 32), 8);
  k_prod_inner<<<grid, NT, 0, st>>>(y, ny, xhat, sy, signs, rnorm, n, D, M, corr, out);
  return check_launch();
}

}  // namespace tq
