/*
 * turboquant_b200.h -- C ABI of libturboquant_b200.so
 *
 * B200 (sm_100a) kernels for the TurboQuant KV-cache compression hot path.
 * Every entry point takes plain pointers and sizes.  Device pointers are marked
 * [dev], host pointers [host].  The library never allocates, frees or retains
 * caller memory, never synchronises the device, and enqueues all work on the
 * stream that is passed in (a cudaStream_t, given as void*).  The caller makes
 * the right device current before the call.
 *
 * Each function returns TQ_OK (0) or a negative TQ_E* code; tq_strerror() turns
 * a code into text.  No function throws or aborts.
 *
 * The "Replaces:" lines cite the interface of the reference implementation
 * (tonbistudio/turboquant-pytorch, file:line in that tree) whose work the entry
 * point performs.
 */
#ifndef TURBOQUANT_B200_H
#define TURBOQUANT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- codes ------------------------------------------------------------ */
enum {
  TQ_OK = 0,
  TQ_EINVAL = -1,    /* inconsistent sizes / negative counts / bad mode        */
  TQ_EBITS = -2,     /* bits outside 1..8                                       */
  TQ_EDIM = -3,      /* head_dim outside 1..256                                 */
  TQ_ENULL = -4,     /* a required pointer is NULL                              */
  TQ_EALIGN = -5,    /* pointer or stride breaks the stated alignment           */
  TQ_EDTYPE = -6,    /* unknown element type code                               */
  TQ_ELAUNCH = -7,   /* the CUDA runtime refused the launch (see tq_last_cuda_error) */
  TQ_EWORKSPACE = -8,/* workspace smaller than tq_*_workspace_bytes says        */
  TQ_ETOOBIG = -9,   /* problem exceeds a fixed capacity of the entry point     */
  TQ_EDEVICE = -10   /* device is not compute capability 10.x, or its ordinal is not served */
};

/* element types of caller tensors */
enum { TQ_F32 = 0, TQ_F16 = 1, TQ_BF16 = 2 };

/* how indices are laid out in memory */
enum {
  TQ_IDX_PACKED = 0, /* 8/bits indices per byte, first index in the high bits,
                        row = ceil(D / (8/bits)) bytes, zero padded
                        (turboquant/compressors_v3.py:64-74)                     */
  TQ_IDX_U8 = 1,     /* one uint8 per index (turboquant/compressors.py:205)     */
  TQ_IDX_I64 = 2     /* one int64 per index (turboquant/turboquant.py:85)       */
};

#define TQ_MAX_DIM 256
#define TQ_CODEBOOK_FLOATS 800
/* A codebook block is 800 floats on the device: [0,L) centroids ascending,
 * [256, 256+L-1) decision thresholds, every other slot below 512 +inf, and
 * [512,528) the parameters of the search shortcut and [528,800) its cell table
 * (below).  Threshold k is
 * the largest fp32 y for which fl|y-c_k| <= fl|y-c_(k+1)|, so that
 * index(y) = #{k : y > threshold_k} equals the first-minimum argmin over
 * |y - c| evaluated in fp32 (turboquant/compressors_v3.py:60-61).  The identity
 * holds while ulp(y) is far below the centroid spacing (|y| < 1024 for every
 * codebook of head_dim 64..256; rotated unit vectors have |y| <= 1); beyond
 * that fp32 differences tie and the argmin itself stops being monotone.
 *
 * Search shortcut (slots 512..): [512] = 1.0 when valid, [513] = s, [514..516] =
 * c1, c2, c3.  With t = sat(y*s + 0.5) and e = round(t*(c1 + t*(c2 + t*c3))) the
 * host has verified, in the same fp32 arithmetic, that the exact index is e or
 * e+1 for every y, so index(y) = e + (y > threshold_e): one table look-up instead
 * of a binary search, with the same result.  Built for up to 31 thresholds.
 * [518] = 1.0 when a straight line passed the check (c2 = c3 = 0; it does for the
 * three thresholds of 2-bit codes), which lets kernels skip the two higher terms.
 * For 32..255 thresholds [512] = 2.0: e comes from a byte table over 1024 uniform
 * cells of t, stored from float slot 528 on, e = table[round(t * 1024)], under the
 * same verified guarantee.  When neither form passes the check, [512] is 0 and
 * kernels search.                                                              */

int tq_version(void);
const char* tq_strerror(int code);
/* cudaError_t value of the last failed launch on this host thread (0 if none) */
int tq_last_cuda_error(void);
/* kernels this library has launched in this process so far (all threads)      */
int64_t tq_launch_count(void);

/* ---- host-side helpers (no GPU needed) -------------------------------- */

/* Bytes per packed row: ceil(D / (8/bits)).
 * Replaces: turboquant/compressors_v3.py:64-69 and :112-113.                  */
int tq_packed_row_bytes(int D, int bits);

/* Fill a TQ_CODEBOOK_FLOATS codebook block [host] from L = 2^bits ascending centroids
 * [host].  Replaces the argmin rule of turboquant/compressors_v3.py:60-61.    */
int tq_build_codebook(const float* centroids, int bits, float* block);

/* Tensor-core operand image of a (D, D) row-major fp32 matrix m [dev]: two fp16 pieces
 * (m = hi + lo), K-major, 128-byte swizzled, tq_rotation_image_bytes(D) bytes (0 when D
 * has no tensor-core path; only D = 128 has one).  Built once per compressor.
 * For TqQuantizeJob pass m = Pi; for TqDequantizeJob pass m = Pi^T.
 * Replaces nothing in the reference (a constant of this implementation).       */
size_t tq_rotation_image_bytes(int D);
int tq_prepare_rotation_image(const float* m, int D, void* image, void* stream);

/* Status word written by a kernel whose bounded wait ran out: 0 = none, else
 * (role << 16) | block.  Reads the device synchronously; for diagnostics only. */
int tq_last_device_status(void);

/* ---- K0: rotated fp32 values -> indices (the bit-exact gate) ----------- */
/* y [dev] (n, D) contiguous fp32; out [dev] laid out per idx_mode.
 * Replaces: turboquant/compressors_v3.py:60-74, turboquant/lloyd_max.py:117-121. */
int tq_quantize_rotated(const float* y, int64_t n, int D, int bits, const float* codebook,
                        int idx_mode, void* out, void* stream);

/* ---- K1: norm + rotate + nearest centroid + pack ----------------------- */
typedef struct {
  const void* x;          /* [dev] vectors; element (b,h,s,d) at x[b*stride_b + h*stride_h + s*stride_s + d] */
  int32_t x_dtype;        /* TQ_F32 | TQ_F16 | TQ_BF16                                      */
  int32_t D;              /* head_dim, 1..256; the last dimension is contiguous             */
  int32_t bits;           /* 1..8                                                            */
  int32_t normalize;      /* 1: divide by (||x||+1e-8) and emit norms; 0: quantise x as is  */
  int64_t B, H, S;        /* vector count = B*H*S                                            */
  int64_t stride_b, stride_h, stride_s;   /* in elements                                     */
  const float* rotation_t;/* [dev] Pi^T, (D, D) row-major fp32: y = x @ rotation_t           */
  const float* codebook;  /* [dev] codebook block                                            */
  int32_t idx_mode;       /* TQ_IDX_*                                                        */
  int32_t reserved;
  void* idx_out;          /* [dev] (B*H*S, row) contiguous                                   */
  uint16_t* norms_out;    /* [dev] fp16 bit patterns (B*H*S); may be NULL when normalize==0  */
  const void* rotation_image; /* [dev] optional: tq_prepare_rotation_image(Pi) output.  With it, head_dim
                             128, 16-bit x, normalize=1 and TQ_IDX_PACKED the job runs on the tensor
                             cores; NULL keeps it on the FP32 path                              */
} TqQuantizeJob;

/* Runs n_jobs independent jobs [host array].
 * Replaces: MSECompressor.compress turboquant/compressors_v3.py:45-81 (and the
 * old-token half of TurboQuantV3.compress_kv :193-207, which it reads through
 * strides instead of copying); TurboQuantCompressorMSE.compress
 * turboquant/compressors.py:200-213 (TQ_IDX_U8); TurboQuantMSE.quantize
 * turboquant/turboquant.py:80-86 (normalize=0, TQ_IDX_I64).                    */
int tq_quantize(const TqQuantizeJob* jobs, int n_jobs, void* stream);

/* ---- K2: unpack + centroid lookup + inverse rotation + rescale --------- */
typedef struct {
  const void* idx;        /* [dev] (B*H*S, row) contiguous, layout idx_mode                  */
  const uint16_t* norms;  /* [dev] fp16 bit patterns, or NULL for no rescale                 */
  int32_t idx_mode;
  int32_t D, bits;
  int32_t out_dtype;      /* TQ_F32 (drop-in decompress) | TQ_F16 | TQ_BF16 (cache dtype)    */
  int64_t B, H, S;
  void* out;              /* [dev] element (b,h,s,d) at out[b*ostride_b + h*ostride_h + s*ostride_s + d] */
  int64_t ostride_b, ostride_h, ostride_s;
  const float* rotation;  /* [dev] Pi, (D, D) row-major fp32: x_hat = c[idx] @ rotation      */
  const float* codebook;  /* [dev] codebook block                                            */
  const void* rotation_image; /* [dev] optional: tq_prepare_rotation_image(Pi^T) output; with it, head_dim
                             128 and TQ_IDX_PACKED with norms run on the tensor cores            */
} TqDequantizeJob;

/* Replaces: MSECompressor.decompress turboquant/compressors_v3.py:83-105; with a
 * 16-bit out_dtype and strides into the final (B,H,S_total,D) buffer also the
 * cast + concatenate of TurboQuantV3.decompress_kv :225-232;
 * TurboQuantCompressorMSE.decompress turboquant/compressors.py:215-221;
 * TurboQuantMSE.dequantize turboquant/turboquant.py:88-91 (norms NULL).        */
int tq_dequantize(const TqDequantizeJob* jobs, int n_jobs, void* stream);

/* ---- residual window: strided copy of kept 16-bit tokens ------------------ */
typedef struct {
  const void* src;        /* [dev] element (b,h,s,d) at src[b*sstride_b + h*sstride_h + s*sstride_s + d] */
  void* dst;              /* [dev] same indexing with the dstride_* strides                    */
  int32_t elem_bytes;     /* 2 or 4                                                            */
  int32_t D;              /* contiguous last dimension; D*elem_bytes a multiple of 16          */
  int64_t B, H, S;
  int64_t sstride_b, sstride_h, sstride_s;   /* in elements; byte strides multiples of 16      */
  int64_t dstride_b, dstride_h, dstride_s;
} TqCopyJob;

/* Copies n_jobs blocks of rows in one launch: the kept window tokens of every layer's K and
 * V into the buffers tq_dequantize writes the reconstructed tokens into.  src and dst are
 * 16-byte aligned and do not overlap.
 * Replaces: the torch.cat with the "fp16" part in TurboQuantV3.decompress_kv
 * turboquant/compressors_v3.py:230-232.                                        */
int tq_copy_rows(const TqCopyJob* jobs, int n_jobs, void* stream);

/* 1 when the library was built with -DTQ_ABLATION (timing-only switches that skip parts
 * of the kernels, selected by the TQ_ABLATE environment variable), 0 for a normal build. */
int tq_ablation_build(void);

/* ---- generic projection: out = x @ m ---------------------------------- */
/* x [dev] (n, K) contiguous of x_dtype; m [dev] (K, N) row-major fp32; out (n, N) fp32.
 * K, N in 1..256.  Replaces: TurboQuantMSE.rotate/unrotate
 * turboquant/turboquant.py:71-78 and the query projections of
 * turboquant/compressors.py:147 and turboquant/turboquant.py:185.             */
int tq_project(const void* x, int x_dtype, int64_t n, int K, const float* m, int N, float* out, void* stream);

/* ---- K3: attention logits straight from packed keys -------------------- */
typedef struct {
  const void* q;          /* [dev] (B, Hq, Sq, D) contiguous                                 */
  int32_t q_dtype;
  int32_t D, bits;
  int32_t reserved;
  int64_t B, Hq, Sq, Hkv, Sk;  /* Hq % Hkv == 0; query head g reads KV head g / (Hq/Hkv)    */
  const uint8_t* idx_bytes;    /* [dev] (B, Hkv, Sk, row) TQ_IDX_PACKED                      */
  const uint16_t* norms;       /* [dev] (B, Hkv, Sk) fp16 bits                               */
  const float* rotation_t;     /* [dev] Pi^T (the key compressor's)                          */
  const float* codebook;
  float scale;                 /* logits are multiplied by this (1.0f: raw q.k)              */
  int32_t reserved2;
  float* logits;               /* [dev] (B, Hq, Sq, Sk)                                      */
  float* probs;                /* [dev] softmax over Sk, same shape, or NULL                 */
  void* workspace;             /* [dev] scratch, 256-byte aligned                            */
  size_t workspace_bytes;
} TqScoreJob;

size_t tq_score_workspace_bytes(int64_t B, int64_t Hq, int64_t Sq, int64_t Sk, int D);

/* logits = scale * q . k_hat with k_hat the reconstruction MSECompressor.decompress
 * would return, computed as norm_s * sum_j (q Pi^T)_j * c[idx_sj] without
 * materialising keys.
 * Replaces: compress -> decompress -> matmul of turboquant/validate_v3.py:83-87.  */
int tq_score_packed(const TqScoreJob* job, void* stream);

/* Same computation and results as tq_score_packed, for callers that cannot
 * provide scratch memory: hosts whose device memory is fully planned by another
 * framework, request paths that must stay off the allocator, or bindings that
 * can only pass the tensors they own.  job->workspace and workspace_bytes are
 * ignored; the scratch is a fixed array of TQ_SCORE_NOALLOC_SCRATCH_BYTES inside
 * the library image (each GPU that loads the library holds it until exit).  The
 * call allocates and frees nothing.  It returns TQ_ETOOBIG when
 * tq_score_workspace_bytes(B, Hq, Sq, Sk, D) exceeds that size.  The first call
 * on a device looks up the array's address (cudaGetSymbolAddress) with that
 * device current, so make the first call on each device before any stream
 * capture.  All calls on a device share the array, which keeps the previous
 * call's contents (nothing in it needs clearing); two calls whose kernels can
 * overlap on the GPU -- different streams without an ordering between them --
 * race on it, so keep such calls on one stream or order them with events.
 * The looked-up address is kept until the process exits: after cudaDeviceReset,
 * or once the device's primary context has been destroyed, it is stale and the
 * entry point must not be used again in that process.  Device ordinals of 64
 * and above are not served (TQ_EDEVICE).
 * This entry point has no counterpart in the reference.                       */
#define TQ_SCORE_NOALLOC_SCRATCH_BYTES (4u << 20)
int tq_score_packed_noalloc(const TqScoreJob* job, void* stream);

/* ---- decode attention on packed keys AND packed values ---------------------- */
typedef struct {
  const void* q;               /* [dev] (B, Hq, Sq, D) contiguous queries (unrotated)             */
  int32_t q_dtype;
  int32_t D;                   /* 128                                                              */
  int32_t key_bits, value_bits;
  int64_t B, Hq, Sq, Hkv, Sk;  /* Sk packed tokens; Hq % Hkv == 0                                  */
  const uint8_t* k_idx;        /* [dev] (B, Hkv, Sk, row_k) TQ_IDX_PACKED                          */
  const uint16_t* k_norms;     /* [dev] (B, Hkv, Sk) fp16 bits                                     */
  const uint8_t* v_idx;        /* [dev] (B, Hkv, Sk, row_v)                                        */
  const uint16_t* v_norms;
  const float* k_rotation_t;   /* [dev] Pi_k^T of the key compressor                               */
  const float* v_rotation;     /* [dev] Pi_v of the value compressor: v_hat = c_v[idx] @ Pi_v * norm */
  const float* k_codebook;     /* [dev] codebook blocks                                            */
  const float* v_codebook;
  const void* k_window;        /* [dev] kept 16-bit (or fp32) tokens that follow the packed ones,  */
  const void* v_window;        /*       element (b,h,w,d) at [b*wstride_b + h*wstride_h + w*wstride_s + d]; NULL: none */
  int32_t window_dtype;
  int32_t reserved;
  int64_t W;
  int64_t wstride_b, wstride_h, wstride_s;
  float scale;                 /* logits = scale * q . k                                           */
  int32_t reserved2;
  float* out;                  /* [dev] (B, Hq, Sq, D) fp32                                        */
  void* workspace;             /* [dev] 256-byte aligned scratch                                   */
  size_t workspace_bytes;      /* >= tq_decode_attention_workspace_bytes(B, Hq, Sq, Sk)            */
} TqDecodeAttnJob;

size_t tq_decode_attention_workspace_bytes(int64_t B, int64_t Hq, int64_t Sq, int64_t Sk);

/* out = softmax(scale * q K_hat^T) V_hat over the Sk packed tokens followed by the W window tokens, where
 * K_hat, V_hat are what MSECompressor.decompress would return for the packed rows.  Neither is
 * materialised: logits come from the packed keys (as tq_score_packed), the probability-weighted sum of
 * the packed values is accumulated in the rotated domain and Pi_v is applied once per query row.
 * head_dim 128 only (TQ_EDIM otherwise).
 * Replaces: the decompress-everything-then-attend step of the generation harness,
 * turboquant/generation_test_v2.py:131-147, i.e. the composition of turboquant/validate_v3.py:83-87
 * (scores) with the value path of turboquant/compressors_v3.py:83-105.          */
int tq_decode_attention(const TqDecodeAttnJob* job, void* stream);

/* ---- K4: MSE stage + QJL sign stage ------------------------------------ */
typedef struct {
  const void* x; int32_t x_dtype; int32_t D;
  int32_t bits;           /* width of the MSE stage (already bits-1 of the total budget)     */
  int32_t normalize;      /* 1: V2 (unit-normalise, rescale k_mse); 0: V1 TurboQuantProd      */
  int64_t B, H, S; int64_t stride_b, stride_h, stride_s;
  const float* rotation_t;/* [dev] Pi^T                                                       */
  const float* rotation;  /* [dev] Pi                                                         */
  const float* codebook;
  const float* qjl_t;     /* [dev] S^T, (D, M) row-major fp32: projected = residual @ qjl_t   */
  int32_t M;              /* QJL projection width, 1..256                                     */
  int32_t signs_dtype;    /* 0: int8 +-1 with >=0 -> +1; 1: fp32 +-1 with 0 -> +1;
                             2: one bit per sign, (N, M / 8) bytes, coordinate j in bit 7 - j % 8 of byte j / 8, set for
                             +1 (the form tq_qjl_scores_packed reads).  2, and idx_mode TQ_IDX_PACKED for idx_out
                             (bit-packed rows as tq_quantize writes them), are served by the tensor-core path only:
                             a job that asks for them and does not qualify for it returns TQ_EINVAL (write the unpacked
                             forms and call tq_pack_mse_qjl instead)                            */
  int32_t rnorm_dtype;    /* TQ_F16 | TQ_F32                                                  */
  int32_t idx_mode;       /* layout of idx_out when it is not NULL                            */
  uint16_t* k_mse_out;    /* [dev] fp16 (N, D) or NULL                                        */
  void* idx_out;          /* [dev] or NULL                                                    */
  void* signs_out;        /* [dev] (N, M)                                                     */
  void* rnorm_out;        /* [dev] (N)                                                        */
  void* workspace;        /* [dev] scratch for the tensor-core path, or NULL (FP32 kernels)   */
  size_t workspace_bytes; /* >= tq_qjl_compress_workspace_bytes(N, D) to enable that path     */
  float* vec_norms_out;   /* [dev] optional fp32 ||x|| per vector (N), normalize == 1 only: what the
                             packed form keeps in place of k_mse                              */
} TqQjlCompressJob;

/* Scratch the tensor-core path of tq_qjl_compress needs for N vectors (operand images of the three
 * matrices, two fp16 piece arrays of N x D, N norms); 0 when head_dim has no such path.  That path
 * serves contiguous fp16 vectors with head_dim 128 or 256, normalize = 1, M = D, int8 signs, fp16
 * residual norms, idx_out NULL or TQ_IDX_U8; every other job, and any job without enough scratch,
 * runs on the FP32 kernels with identical semantics.                                           */
size_t tq_qjl_compress_workspace_bytes(int64_t n_vectors, int D);

/* Replaces: TurboQuantCompressorV2.compress turboquant/compressors.py:83-120;
 * TurboQuantProd.quantize turboquant/turboquant.py:134-159.                    */
int tq_qjl_compress(const TqQjlCompressJob* job, void* stream);

/* ---- packed storage of the MSE+QJL representation ----------------------- */
/* idx_u8 [dev] (n, D) one index per byte, signs [dev] (n, D) int8 +-1  ->
 * idx_packed [dev] (n, ceil(D / (8/bits))) in the TQ_IDX_PACKED layout and sign_bits [dev] (n, D/8), coordinate j
 * in bit 7 - j % 8 of byte j / 8, set for +1.  D a multiple of 8.  Either output may be NULL.
 * Replaces nothing the reference runs: it is the storage layout the reference's own size accounting assumes
 * (turboquant/validate.py:120-134) in place of the fp16 k_mse + int8 signs it stores
 * (turboquant/compressors.py:115-120) and the int64 indices + fp32 signs of turboquant/turboquant.py:155-159. */
int tq_pack_mse_qjl(const uint8_t* idx_u8, const int8_t* signs, int64_t n, int D, int bits, uint8_t* idx_packed,
                    uint8_t* sign_bits, void* stream);

typedef struct {
  const void* q; int32_t q_dtype; int32_t D;    /* (BH, Sq, D) queries; D = 128 or 256              */
  int32_t bits;                                  /* width of the MSE stage                            */
  int32_t reserved;
  int64_t BH, Sq, Sk;
  const uint8_t* idx_packed;   /* [dev] (BH, Sk, row) TQ_IDX_PACKED                                   */
  const uint8_t* sign_bits;    /* [dev] (BH, Sk, D/8)                                                 */
  const float* vec_norms;      /* [dev] fp32 (BH, Sk)                                                 */
  const uint16_t* rnorm;       /* [dev] fp16 (BH, Sk)                                                 */
  const float* rotation_t;     /* [dev] Pi^T (D, D)                                                   */
  const float* qjl_t;          /* [dev] S^T (D, D)                                                    */
  const float* codebook;       /* [dev] codebook block of the MSE stage                               */
  float* scores;               /* [dev] (BH, Sq, Sk)                                                  */
  void* workspace; size_t workspace_bytes;   /* >= tq_qjl_scores_packed_workspace_bytes               */
} TqQjlPackedScoreJob;

size_t tq_qjl_scores_packed_workspace_bytes(int64_t BH, int64_t Sq, int D);

/* The estimator of tq_qjl_scores evaluated straight from the packed form:
 * <q, k_mse> = ||x|| * <q Pi^T, c[idx]> needs no reconstructed key, the sign term reads one bit per
 * coordinate.  Replaces: TurboQuantCompressorV2.asymmetric_attention_scores
 * turboquant/compressors.py:122-158 on the layout of turboquant/validate.py:120-134.               */
int tq_qjl_scores_packed(const TqQjlPackedScoreJob* job, void* stream);

/* ---- K5: asymmetric scores from the MSE+QJL representation ------------- */
typedef struct {
  const void* q; int32_t q_dtype; int32_t D;
  int64_t BH, Sq, Sk;          /* q (BH, Sq, D); keys (BH, Sk, ...)                           */
  const uint16_t* k_mse;       /* [dev] fp16 (BH, Sk, D)                                      */
  const int8_t* signs;         /* [dev] (BH, Sk, D)                                           */
  const uint16_t* rnorm;       /* [dev] fp16 (BH, Sk)                                         */
  const float* qjl_t;          /* [dev] S^T (D, D)                                            */
  float* scores;               /* [dev] (BH, Sq, Sk)                                          */
  void* workspace; size_t workspace_bytes;   /* >= tq_qjl_scores_workspace_bytes              */
} TqQjlScoreJob;

size_t tq_qjl_scores_workspace_bytes(int64_t BH, int64_t Sq, int D);

/* Replaces: TurboQuantCompressorV2.asymmetric_attention_scores
 * turboquant/compressors.py:122-158.                                           */
int tq_qjl_scores(const TqQjlScoreJob* job, void* stream);

/* Row-paired estimator <y_n, x_mse_n> + ||r_n|| sqrt(pi/2)/M <S y_n, signs_n>.
 * y (ny, D) fp32 with ny == n or ny == 1; idx int64 (n, D); signs fp32 (n, M);
 * rnorm fp32 (n); workspace >= (n + ny) * 256 * 4 bytes.
 * Replaces: TurboQuantProd.inner_product turboquant/turboquant.py:165-192.     */
int tq_prod_inner_product(const float* y, int64_t ny, const int64_t* idx, const float* signs, const float* rnorm,
                          int64_t n, int D, int M, const float* rotation, const float* codebook,
                          const float* qjl_t, float* out, void* workspace, size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TURBOQUANT_B200_H */
