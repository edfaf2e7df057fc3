// C ABI of libturboquant_b200.so: argument checking, host helpers, dispatch.

#include <math.h>
#include <string.h>

#include "tq_internal.h"

namespace {

inline bool bad_dtype(int dt) { return dt != TQ_F32 && dt != TQ_F16 && dt != TQ_BF16; }
inline bool bad_mode(int m) { return m != TQ_IDX_PACKED && m != TQ_IDX_U8 && m != TQ_IDX_I64; }

// order-preserving map between fp32 values and int32
inline int32_t f2ord(float f) {
  int32_t i;
  memcpy(&i, &f, 4);
  return i < 0 ? (int32_t)(0x80000000u - (uint32_t)i) : i;
}
inline float ord2f(int32_t o) {
  int32_t i = o < 0 ? (int32_t)(0x80000000u - (uint32_t)o) : o;
  float f;
  memcpy(&f, &i, 4);
  return f;
}

// fl|y - a| <= fl|y - b| in IEEE single precision (volatile blocks contraction / widening)
inline bool prefers_lower(float y, float a, float b) {
  volatile float da = y - a;
  volatile float db = y - b;
  return fabsf(da) <= fabsf(db);
}

// ---- search shortcut --------------------------------------------------------------
// e(y) exactly as the kernels compute it (fp32 fma, saturate, round to nearest even).
inline int shortcut_e(float y, float s, float c1, float c2, float c3) {
  float t = fmaf(y, s, 0.5f);
  if (!(t > 0.f)) t = 0.f;          // NaN -> 0, like a saturating fma
  if (t > 1.f) t = 1.f;
  float q = fmaf(c3, t, c2);
  q = fmaf(q, t, c1);
  const float u = fmaf(q, t, 8388608.0f);
  int32_t bits;
  memcpy(&bits, &u, 4);
  return bits - 0x4B000000;
}

inline int exact_index(float y, const float* thr, int n) {
  int c = 0;
  for (int k = 0; k < n; ++k) c += (y > thr[k]) ? 1 : 0;
  return c;
}

// Least-squares cubic through the origin mapping the thresholds to k + 1/2, then an
// exhaustive check of "exact index is e or e+1" around every threshold and on a grid.
// Wide codes (more than 31 thresholds): a table over 1024 uniform cells of t = sat(y s + 1/2)
// gives the lower candidate e; thresholds are at least one cell apart, so the exact index is
// e or e + 1, which the same exhaustive check confirms.  cell(y) = round(t * 1024).
constexpr int kCells = 1024;
inline int cell_of(float y, float s) {
  float t = fmaf(y, s, 0.5f);
  if (!(t > 0.f)) t = 0.f;
  if (t > 1.f) t = 1.f;
  const float u = fmaf(t, (float)kCells, 8388608.0f);
  int32_t bits;
  memcpy(&bits, &u, 4);
  return bits - 0x4B000000;
}

void fit_cell_table(float* block, int n) {
  const float* thr = block + 256;
  const double lim = fmax(fabs((double)thr[0]), fabs((double)thr[n - 1])) * 1.001 + 1e-12;
  const float s = (float)(0.5 / lim);
  uint8_t* cells = reinterpret_cast<uint8_t*>(block + 528);
  // lower candidate of a cell = exact index at the smallest y that maps to it
  int c_prev = -1;
  // walk y upwards through every threshold and every cell boundary by scanning a fine grid, then
  // fix the table from the thresholds themselves: e[c] = number of thresholds whose cell is < c,
  // plus those in an earlier cell position; verified below in any case.
  for (int c = 0; c <= kCells; ++c) cells[c] = 0;
  (void)c_prev;
  // count thresholds per cell
  int per_cell[kCells + 1] = {0};
  for (int k = 0; k < n; ++k) {
    const int c = cell_of(thr[k], s);
    if (c < 0 || c > kCells) return;
    per_cell[c]++;
    if (per_cell[c] > 1) return;            // two thresholds in one cell: table cannot bracket
  }
  int below = 0;                            // thresholds in cells strictly below c
  for (int c = 0; c <= kCells; ++c) {
    if (below > 255) return;
    cells[c] = (uint8_t)below;              // inside cell c the exact index is `below` or `below + 1`
    below += per_cell[c];
  }
  const float s_lo = s * (1.0f - 4e-6f), s_hi = s * (1.0f + 4e-6f);
  auto ok_at = [&](float y) {
    const int i = exact_index(y, thr, n);
    for (float sv : {s_lo, s, s_hi}) {
      const int c = cell_of(y, sv);
      if (c < 0 || c > kCells) return false;
      const int e = cells[c];
      if (!((e == i || e + 1 == i) && (e < n || i == e))) return false;
    }
    return true;
  };
  for (int k = 0; k < n; ++k) {
    float y = thr[k];
    for (int step = 0; step < 4; ++step) y = nextafterf(y, -INFINITY);
    for (int step = 0; step < 9; ++step) {
      if (!ok_at(y)) return;
      y = nextafterf(y, INFINITY);
    }
  }
  const int grid = 1 << 18;
  for (int g = 0; g <= grid; ++g) {
    const float y = (float)(-1.25 + 2.5 * (double)g / grid);
    if (!ok_at(y)) return;
  }
  const float specials[] = {0.f, -0.f, 1.f, -1.f, 100.f, -100.f, 1000.f, -1000.f, INFINITY, -INFINITY, NAN};
  for (float y : specials) if (!ok_at(y)) return;
  block[512] = 2.f;
  block[513] = s;
  block[517] = (float)kCells;
}

void fit_shortcut(float* block, int n) {
  for (int i = 512; i < TQ_CODEBOOK_FLOATS; ++i) block[i] = 0.f;
  if (n > 63 && n <= 255) { fit_cell_table(block, n); return; }
  if (n < 1 || n > 255) return;
  const float* thr = block + 256;
  const double lim = fmax(fabs((double)thr[0]), fabs((double)thr[n - 1])) * 1.001 + 1e-12;
  const float s = (float)(0.5 / lim);
  // basis t, t^2, t^3 ; target k + 0.5 - 0.5 = k  (the constant 1/2 is the rounding offset)
  auto try_degree = [&](int deg, float& c1, float& c2, float& c3) -> bool {
  double ata[3][3] = {{0}}, atb[3] = {0};
  for (int k = 0; k < n; ++k) {
    const double t = (double)thr[k] * (double)s + 0.5;
    const double b[3] = {t, t * t, t * t * t};
    for (int i = 0; i < deg; ++i) {
      for (int j = 0; j < deg; ++j) ata[i][j] += b[i] * b[j];
      atb[i] += b[i] * (double)k;
    }
  }
  double c[3] = {0, 0, 0};
  // Gaussian elimination on the deg x deg normal equations (with a tiny ridge)
  double m[3][4];
  for (int i = 0; i < deg; ++i) {
    for (int j = 0; j < deg; ++j) m[i][j] = ata[i][j] + (i == j ? 1e-12 : 0.0);
    m[i][deg] = atb[i];
  }
  for (int i = 0; i < deg; ++i) {
    int piv = i;
    for (int r = i + 1; r < deg; ++r) if (fabs(m[r][i]) > fabs(m[piv][i])) piv = r;
    for (int j = 0; j <= deg; ++j) { double tmp = m[i][j]; m[i][j] = m[piv][j]; m[piv][j] = tmp; }
    if (fabs(m[i][i]) < 1e-300) return false;
    for (int r = i + 1; r < deg; ++r) {
      const double f = m[r][i] / m[i][i];
      for (int j = i; j <= deg; ++j) m[r][j] -= f * m[i][j];
    }
  }
  for (int i = deg - 1; i >= 0; --i) {
    double acc = m[i][deg];
    for (int j = i + 1; j < deg; ++j) acc -= m[i][j] * c[j];
    c[i] = acc / m[i][i];
  }
  c1 = (float)c[0]; c2 = (float)c[1]; c3 = (float)c[2];
  // Kernels may fold the per-vector scale into s, which moves t by an ulp or two; demand the
  // bracket for slightly perturbed scales as well so that such rounding can never matter.
  const float s_lo = s * (1.0f - 4e-6f), s_hi = s * (1.0f + 4e-6f);
  auto ok_at = [&](float y) {
    const int i = exact_index(y, thr, n);
    for (float sv : {s_lo, s, s_hi}) {
      const int e = shortcut_e(y, sv, c1, c2, c3);
      if (!(e >= 0 && e <= 63 && (e == i || e + 1 == i) && (e < n || i == e))) return false;
    }
    return true;
  };
  for (int k = 0; k < n; ++k) {
    float y = thr[k];
    for (int step = 0; step < 4; ++step) y = nextafterf(y, -INFINITY);
    for (int step = 0; step < 9; ++step) {
      if (!ok_at(y)) return false;
      y = nextafterf(y, INFINITY);
    }
  }
  const int grid = 1 << 16;
  for (int g = 0; g <= grid; ++g) {
    const float y = (float)(-1.25 + 2.5 * (double)g / grid);
    if (!ok_at(y)) return false;
  }
  const float specials[] = {0.f, -0.f, 1.f, -1.f, 100.f, -100.f, 1000.f, -1000.f, INFINITY, -INFINITY, NAN};
  for (float y : specials) if (!ok_at(y)) return false;
  return true;
  };
  // a straight line is tried first (it brackets the few thresholds of 1- and 2-bit codes and
  // saves two multiply-adds per coordinate), then the cubic
  float c1 = 0.f, c2 = 0.f, c3 = 0.f;
  int degree = 0;
  if (try_degree(1, c1, c2, c3)) degree = 1;
  else if (try_degree(n >= 3 ? 3 : n, c1, c2, c3)) degree = 3;
  if (degree == 0) {
    if (n > 31) fit_cell_table(block, n);    // 6-bit codes whose cubic does not bracket: cell table
    return;
  }
  block[512] = 1.f;
  block[513] = s;
  block[514] = c1;
  block[515] = c2;
  block[516] = c3;
  block[518] = degree == 1 ? 1.f : 0.f;     // 1: c2 = c3 = 0, kernels may skip those terms
}

int check_common(int D, int bits) {
  if (bits < 1 || bits > 8) return TQ_EBITS;
  if (D < 1 || D > TQ_MAX_DIM) return TQ_EDIM;
  return TQ_OK;
}

}  // namespace

extern "C" {

int tq_version(void) { return 100; }

const char* tq_strerror(int code) {
  switch (code) {
    case TQ_OK: return "ok";
    case TQ_EINVAL: return "invalid argument (sizes, counts or mode)";
    case TQ_EBITS: return "bits must be in 1..8";
    case TQ_EDIM: return "head_dim must be in 1..256";
    case TQ_ENULL: return "required pointer is NULL";
    case TQ_EALIGN: return "pointer or stride is misaligned";
    case TQ_EDTYPE: return "unknown element type";
    case TQ_ELAUNCH: return "CUDA launch failed";
    case TQ_EWORKSPACE: return "workspace too small";
    case TQ_ETOOBIG: return "problem exceeds the capacity of this entry point";
    case TQ_EDEVICE: return "device is not compute capability 10.x, or its ordinal is not served";
    default: return "unknown error code";
  }
}

int tq_last_cuda_error(void) { return tq::last_cuda_error(); }

int64_t tq_launch_count(void) { return (int64_t)tq::launch_count(); }

int tq_packed_row_bytes(int D, int bits) {
  int rc = check_common(D, bits);
  if (rc != TQ_OK) return rc;
  int ipb = 8 / bits;
  return (D + ipb - 1) / ipb;
}

int tq_build_codebook(const float* centroids, int bits, float* block) {
  if (centroids == nullptr || block == nullptr) return TQ_ENULL;
  if (bits < 1 || bits > 8) return TQ_EBITS;
  const int L = 1 << bits;
  for (int i = 0; i + 1 < L; ++i)
    if (!(centroids[i] < centroids[i + 1])) return TQ_EINVAL;
  for (int i = 0; i < TQ_CODEBOOK_FLOATS; ++i) block[i] = INFINITY;
  for (int i = 0; i < L; ++i) block[i] = centroids[i];
  for (int k = 0; k + 1 < L; ++k) {
    const float a = centroids[k], b = centroids[k + 1];
    // prefers_lower is true at y = a and false at y = b, and monotone in between
    // because rounding is monotone; bisect on the ordered bit patterns.
    int64_t lo = f2ord(a), hi = f2ord(b);
    while (hi - lo > 1) {
      int64_t mid = lo + (hi - lo) / 2;
      if (prefers_lower(ord2f((int32_t)mid), a, b)) lo = mid; else hi = mid;
    }
    block[256 + k] = ord2f((int32_t)lo);
  }
  fit_shortcut(block, L - 1);
  return TQ_OK;
}

size_t tq_rotation_image_bytes(int D) { return tq::umma_rotation_image_bytes(D); }

int tq_prepare_rotation_image(const float* m, int D, void* image, void* stream) {
  if (m == nullptr || image == nullptr) return TQ_ENULL;
  if (tq::umma_rotation_image_bytes(D) == 0) return TQ_EDIM;
  if (((uintptr_t)image & 1023u) != 0) return TQ_EALIGN;
  return tq::umma_prepare_rotation_image(m, D, image, (cudaStream_t)stream);
}

int tq_last_device_status(void) {
  const int a = tq::umma_device_status();
  if (a != 0) return a;
  const int b = tq::umma_qjl_device_status();
  return b != 0 ? b : tq::umma_v2_device_status();
}

int tq_quantize_rotated(const float* y, int64_t n, int D, int bits, const float* codebook, int idx_mode, void* out,
                        void* stream) {
  int rc = check_common(D, bits);
  if (rc != TQ_OK) return rc;
  if (n < 0 || bad_mode(idx_mode)) return TQ_EINVAL;
  if (n == 0) return TQ_OK;
  if (y == nullptr || codebook == nullptr || out == nullptr) return TQ_ENULL;
  return tq::simt_quantize_rotated(y, n, D, bits, codebook, idx_mode, out, (cudaStream_t)stream);
}

int tq_quantize(const TqQuantizeJob* jobs, int n_jobs, void* stream) {
  if (n_jobs < 0) return TQ_EINVAL;
  if (n_jobs == 0) return TQ_OK;
  if (jobs == nullptr) return TQ_ENULL;
  for (int i = 0; i < n_jobs; ++i) {
    const TqQuantizeJob& j = jobs[i];
    int rc = check_common(j.D, j.bits);
    if (rc != TQ_OK) return rc;
    if (bad_dtype(j.x_dtype)) return TQ_EDTYPE;
    if (bad_mode(j.idx_mode) || j.B < 0 || j.H < 0 || j.S < 0) return TQ_EINVAL;
    if (j.B * j.H * j.S == 0) continue;
    if (j.x == nullptr || j.rotation_t == nullptr || j.codebook == nullptr || j.idx_out == nullptr) return TQ_ENULL;
    if (j.normalize && j.norms_out == nullptr) return TQ_ENULL;
  }
  // maximal runs of tensor-core-eligible jobs go out as one persistent launch each
  int i = 0;
  while (i < n_jobs) {
    if (jobs[i].B * jobs[i].H * jobs[i].S == 0) { ++i; continue; }
    int rc;
    if (tq::umma_quantize_eligible(jobs[i])) {
      int k = i + 1;
      while (k < n_jobs && jobs[k].x_dtype == jobs[i].x_dtype && tq::umma_quantize_eligible(jobs[k])) ++k;
      rc = tq::umma_quantize(jobs + i, k - i, (cudaStream_t)stream);
      i = k;
    } else {
      rc = tq::simt_quantize(jobs[i], (cudaStream_t)stream);
      ++i;
    }
    if (rc != TQ_OK) return rc;
  }
  return TQ_OK;
}

int tq_dequantize(const TqDequantizeJob* jobs, int n_jobs, void* stream) {
  if (n_jobs < 0) return TQ_EINVAL;
  if (n_jobs == 0) return TQ_OK;
  if (jobs == nullptr) return TQ_ENULL;
  for (int i = 0; i < n_jobs; ++i) {
    const TqDequantizeJob& j = jobs[i];
    int rc = check_common(j.D, j.bits);
    if (rc != TQ_OK) return rc;
    if (bad_dtype(j.out_dtype)) return TQ_EDTYPE;
    if (bad_mode(j.idx_mode) || j.B < 0 || j.H < 0 || j.S < 0) return TQ_EINVAL;
    if (j.B * j.H * j.S == 0) continue;
    if (j.idx == nullptr || j.rotation == nullptr || j.codebook == nullptr || j.out == nullptr) return TQ_ENULL;
  }
  int i = 0;
  while (i < n_jobs) {
    if (jobs[i].B * jobs[i].H * jobs[i].S == 0) { ++i; continue; }
    int rc;
    if (tq::umma_dequantize_eligible(jobs[i])) {
      const bool out32 = jobs[i].out_dtype == TQ_F32;
      int k = i + 1;
      while (k < n_jobs && (jobs[k].out_dtype == TQ_F32) == out32 && tq::umma_dequantize_eligible(jobs[k])) ++k;
      rc = tq::umma_dequantize(jobs + i, k - i, (cudaStream_t)stream);
      i = k;
    } else {
      rc = tq::simt_dequantize(jobs[i], (cudaStream_t)stream);
      ++i;
    }
    if (rc != TQ_OK) return rc;
  }
  return TQ_OK;
}

int tq_ablation_build(void) {
#ifdef TQ_ABLATION
  return 1;
#else
  return 0;
#endif
}

int tq_copy_rows(const TqCopyJob* jobs, int n_jobs, void* stream) {
  if (n_jobs < 0) return TQ_EINVAL;
  if (n_jobs == 0) return TQ_OK;
  if (jobs == nullptr) return TQ_ENULL;
  for (int i = 0; i < n_jobs; ++i) {
    const TqCopyJob& j = jobs[i];
    if (j.elem_bytes != 2 && j.elem_bytes != 4) return TQ_EDTYPE;
    if (j.D < 1 || j.B < 0 || j.H < 0 || j.S < 0) return TQ_EINVAL;
    if (j.B * j.H * j.S == 0) continue;
    if (j.src == nullptr || j.dst == nullptr) return TQ_ENULL;
    const int64_t eb = j.elem_bytes;
    if ((j.D * eb) % 16 != 0 || ((uintptr_t)j.src & 15u) || ((uintptr_t)j.dst & 15u)) return TQ_EALIGN;
    const int64_t strides[6] = {j.sstride_b, j.sstride_h, j.sstride_s, j.dstride_b, j.dstride_h, j.dstride_s};
    const int64_t extent[6] = {j.B, j.H, j.S, j.B, j.H, j.S};
    for (int k = 0; k < 6; ++k)
      if (extent[k] > 1 && (strides[k] < 0 || (strides[k] * eb) % 16 != 0)) return TQ_EALIGN;
  }
  return tq::copy_rows(jobs, n_jobs, (cudaStream_t)stream);
}

int tq_project(const void* x, int x_dtype, int64_t n, int K, const float* m, int N, float* out, void* stream) {
  if (K < 1 || K > TQ_MAX_DIM || N < 1 || N > TQ_MAX_DIM) return TQ_EDIM;
  if (bad_dtype(x_dtype)) return TQ_EDTYPE;
  if (n < 0) return TQ_EINVAL;
  if (n == 0) return TQ_OK;
  if (x == nullptr || m == nullptr || out == nullptr) return TQ_ENULL;
  return tq::simt_project(x, x_dtype, n, K, m, N, out, (cudaStream_t)stream);
}

size_t tq_score_workspace_bytes(int64_t B, int64_t Hq, int64_t Sq, int64_t Sk, int D) {
  if (B < 0 || Hq < 0 || Sq < 0 || Sk < 0 || D < 1) return 0;
  return tq::simt_score_workspace(B, Hq, Sq, Sk, D);
}

int tq_score_packed(const TqScoreJob* job, void* stream) {
  if (job == nullptr) return TQ_ENULL;
  int rc = check_common(job->D, job->bits);
  if (rc != TQ_OK) return rc;
  if (bad_dtype(job->q_dtype)) return TQ_EDTYPE;
  if (job->B < 0 || job->Hq < 0 || job->Sq < 0 || job->Hkv < 1 || job->Sk < 0 || job->Hq % job->Hkv != 0) return TQ_EINVAL;
  if (job->B * job->Hq * job->Sq == 0 || job->Sk == 0) return TQ_OK;
  if (job->q == nullptr || job->idx_bytes == nullptr || job->norms == nullptr || job->rotation_t == nullptr ||
      job->codebook == nullptr || job->logits == nullptr || job->workspace == nullptr)
    return TQ_ENULL;
  if (((uintptr_t)job->workspace & 255u) != 0) return TQ_EALIGN;
  if (job->workspace_bytes < tq::simt_score_workspace(job->B, job->Hq, job->Sq, job->Sk, job->D)) return TQ_EWORKSPACE;
  return tq::simt_score_packed(*job, (cudaStream_t)stream);
}

size_t tq_decode_attention_workspace_bytes(int64_t B, int64_t Hq, int64_t Sq, int64_t Sk) {
  if (B < 0 || Hq < 0 || Sq < 0 || Sk < 0) return 0;
  return tq::decode_attention_workspace(B, Hq, Sq, Sk, 2048);
}

int tq_decode_attention(const TqDecodeAttnJob* job, void* stream) {
  if (job == nullptr) return TQ_ENULL;
  if (job->key_bits < 1 || job->key_bits > 8 || job->value_bits < 1 || job->value_bits > 8) return TQ_EBITS;
  if (job->D != 128) return TQ_EDIM;
  if (bad_dtype(job->q_dtype)) return TQ_EDTYPE;
  if (job->B < 0 || job->Hq < 0 || job->Sq < 0 || job->Hkv < 1 || job->Sk < 0 || job->W < 0 || job->Hq % job->Hkv != 0)
    return TQ_EINVAL;
  if (job->B * job->Hq * job->Sq == 0) return TQ_OK;
  const bool has_window = job->k_window != nullptr && job->W > 0;
  if (job->Sk == 0 && !has_window) return TQ_EINVAL;          // nothing to attend to
  if (job->q == nullptr || job->out == nullptr || job->v_rotation == nullptr || job->workspace == nullptr) return TQ_ENULL;
  if (job->Sk > 0 && (job->k_idx == nullptr || job->k_norms == nullptr || job->v_idx == nullptr || job->v_norms == nullptr ||
                      job->k_rotation_t == nullptr || job->k_codebook == nullptr || job->v_codebook == nullptr))
    return TQ_ENULL;
  if (has_window && (job->v_window == nullptr || bad_dtype(job->window_dtype))) return job->v_window == nullptr ? TQ_ENULL : TQ_EDTYPE;
  if (((uintptr_t)job->workspace & 255u) != 0 || ((uintptr_t)job->k_idx & 15u) != 0 || ((uintptr_t)job->v_idx & 15u) != 0)
    return TQ_EALIGN;
  if (job->workspace_bytes < tq::decode_attention_workspace(job->B, job->Hq, job->Sq, job->Sk, 2048)) return TQ_EWORKSPACE;
  return tq::decode_attention(*job, (cudaStream_t)stream);
}

int tq_qjl_compress(const TqQjlCompressJob* job, void* stream) {
  if (job == nullptr) return TQ_ENULL;
  int rc = check_common(job->D, job->bits);
  if (rc != TQ_OK) return rc;
  if (job->M < 1 || job->M > TQ_MAX_DIM) return TQ_EDIM;
  if (bad_dtype(job->x_dtype)) return TQ_EDTYPE;
  if (job->rnorm_dtype != TQ_F16 && job->rnorm_dtype != TQ_F32) return TQ_EDTYPE;
  if (job->B < 0 || job->H < 0 || job->S < 0 || job->signs_dtype < 0 || job->signs_dtype > 2) return TQ_EINVAL;
  const bool packed_idx = job->idx_out != nullptr && job->idx_mode == TQ_IDX_PACKED;
  if (job->idx_out != nullptr && job->idx_mode != TQ_IDX_U8 && job->idx_mode != TQ_IDX_I64 && !packed_idx) return TQ_EINVAL;
  const bool packed_outputs = packed_idx || job->signs_dtype == 2;
  if (job->B * job->H * job->S == 0) return TQ_OK;
  if (job->x == nullptr || job->rotation_t == nullptr || job->rotation == nullptr || job->codebook == nullptr ||
      job->qjl_t == nullptr || job->signs_out == nullptr || job->rnorm_out == nullptr)
    return TQ_ENULL;
  if (tq::umma_v2_compress_eligible(*job)) return tq::umma_v2_compress(*job, (cudaStream_t)stream);
  if (packed_outputs) return TQ_EINVAL;      // packed outputs are written by the tensor-core path only
  return tq::simt_qjl_compress(*job, (cudaStream_t)stream);
}

size_t tq_qjl_compress_workspace_bytes(int64_t n_vectors, int D) {
  if (n_vectors <= 0) return 0;
  return tq::umma_v2_compress_workspace(n_vectors, D);
}

int tq_pack_mse_qjl(const uint8_t* idx_u8, const int8_t* signs, int64_t n, int D, int bits, uint8_t* idx_packed,
                    uint8_t* sign_bits, void* stream) {
  int rc = check_common(D, bits);
  if (rc != TQ_OK) return rc;
  if (n < 0 || D % 8 != 0) return TQ_EINVAL;
  if (n == 0) return TQ_OK;
  if ((idx_packed != nullptr && idx_u8 == nullptr) || (sign_bits != nullptr && signs == nullptr)) return TQ_ENULL;
  if (idx_packed == nullptr && sign_bits == nullptr) return TQ_OK;
  return tq::pack_mse_qjl(idx_u8, signs, n, D, bits, idx_packed, sign_bits, (cudaStream_t)stream);
}

size_t tq_qjl_scores_packed_workspace_bytes(int64_t BH, int64_t Sq, int D) {
  if (BH < 0 || Sq < 0 || D < 1) return 0;
  return tq::qjl_scores_packed_workspace(BH, Sq, D);
}

int tq_qjl_scores_packed(const TqQjlPackedScoreJob* job, void* stream) {
  if (job == nullptr) return TQ_ENULL;
  if (job->bits < 1 || job->bits > 8) return TQ_EBITS;
  if (job->D != 128 && job->D != 256) return TQ_EDIM;
  if (bad_dtype(job->q_dtype)) return TQ_EDTYPE;
  if (job->BH < 0 || job->Sq < 0 || job->Sk < 0) return TQ_EINVAL;
  if (job->BH == 0 || job->Sq == 0 || job->Sk == 0) return TQ_OK;
  if (job->q == nullptr || job->idx_packed == nullptr || job->sign_bits == nullptr || job->vec_norms == nullptr ||
      job->rnorm == nullptr || job->rotation_t == nullptr || job->qjl_t == nullptr || job->codebook == nullptr ||
      job->scores == nullptr || job->workspace == nullptr)
    return TQ_ENULL;
  if (((uintptr_t)job->workspace & 255u) != 0 || ((uintptr_t)job->idx_packed & 15u) != 0 || ((uintptr_t)job->sign_bits & 7u) != 0)
    return TQ_EALIGN;
  if (job->workspace_bytes < tq::qjl_scores_packed_workspace(job->BH, job->Sq, job->D)) return TQ_EWORKSPACE;
  return tq::qjl_scores_packed(*job, (cudaStream_t)stream);
}

size_t tq_qjl_scores_workspace_bytes(int64_t BH, int64_t Sq, int D) {
  if (BH < 0 || Sq < 0 || D < 1) return 0;
  return tq::simt_qjl_scores_workspace(BH, Sq, D) + tq::umma_qjl_scores_image_bytes(BH, Sq, D);
}

int tq_qjl_scores(const TqQjlScoreJob* job, void* stream) {
  if (job == nullptr) return TQ_ENULL;
  if (job->D < 1 || job->D > TQ_MAX_DIM) return TQ_EDIM;
  if (bad_dtype(job->q_dtype)) return TQ_EDTYPE;
  if (job->BH < 0 || job->Sq < 0 || job->Sk < 0) return TQ_EINVAL;
  if (job->BH == 0 || job->Sq == 0 || job->Sk == 0) return TQ_OK;
  if (job->q == nullptr || job->k_mse == nullptr || job->signs == nullptr || job->rnorm == nullptr ||
      job->qjl_t == nullptr || job->scores == nullptr || job->workspace == nullptr)
    return TQ_ENULL;
  if (((uintptr_t)job->workspace & 15u) != 0) return TQ_EALIGN;
  const size_t simt_ws = tq::simt_qjl_scores_workspace(job->BH, job->Sq, job->D);
  if (job->workspace_bytes < simt_ws) return TQ_EWORKSPACE;
  if (tq::umma_qjl_scores_eligible(*job)) {
    const size_t img = tq::umma_qjl_scores_image_bytes(job->BH, job->Sq, job->D);
    if (job->workspace_bytes < simt_ws + img) return TQ_EWORKSPACE;
    const float* qf = nullptr;
    const float* qproj = nullptr;
    int rc = tq::simt_qjl_queries(*job, &qf, &qproj, (cudaStream_t)stream);
    if (rc != TQ_OK) return rc;
    return tq::umma_qjl_scores(*job, qf, qproj, reinterpret_cast<char*>(job->workspace) + simt_ws, (cudaStream_t)stream);
  }
  return tq::simt_qjl_scores(*job, (cudaStream_t)stream);
}

int tq_prod_inner_product(const float* y, int64_t ny, const int64_t* idx, const float* signs, const float* rnorm,
                          int64_t n, int D, int M, const float* rotation, const float* codebook, const float* qjl_t,
                          float* out, void* workspace, size_t workspace_bytes, void* stream) {
  if (D < 1 || D > TQ_MAX_DIM || M < 1 || M > TQ_MAX_DIM) return TQ_EDIM;
  if (n < 0 || (ny != n && ny != 1)) return TQ_EINVAL;
  if (n == 0) return TQ_OK;
  if (y == nullptr || idx == nullptr || signs == nullptr || rnorm == nullptr || rotation == nullptr ||
      codebook == nullptr || qjl_t == nullptr || out == nullptr || workspace == nullptr)
    return TQ_ENULL;
  if (((uintptr_t)workspace & 15u) != 0) return TQ_EALIGN;
  if (workspace_bytes < (size_t)(n + ny) * 256 * sizeof(float)) return TQ_EWORKSPACE;
  return tq::simt_prod_inner_product(y, ny, idx, signs, rnorm, n, D, M, rotation, codebook, qjl_t, out, workspace,
                                     (cudaStream_t)stream);
}

}  // extern "C"
