// Internal launch interface between the C ABI layer and the kernel files.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/turboquant_b200.h"

namespace tq {

int last_cuda_error();
void note_cuda_error(int e);
long long launch_count();
int check_launch();   // cudaGetLastError -> TQ_OK / TQ_ELAUNCH, counts successful launches
bool force_simt();    // TQ_FORCE_SIMT=1 in the environment: route everything to the FP32 kernels (second opinion in tests)

// FP32 CUDA-core path (tq_simt.cu)
int simt_quantize_rotated(const float* y, int64_t n, int D, int bits, const float* cb, int mode, void* out,
                          cudaStream_t st);
int simt_quantize(const TqQuantizeJob& job, cudaStream_t st);
int simt_dequantize(const TqDequantizeJob& job, cudaStream_t st);
int simt_project(const void* x, int x_dtype, int64_t n, int K, const float* m, int N, float* out, cudaStream_t st);
size_t simt_score_workspace(int64_t B, int64_t Hq, int64_t Sq, int64_t Sk, int D);
int simt_score_packed(const TqScoreJob& job, cudaStream_t st);
int simt_qjl_compress(const TqQjlCompressJob& job, cudaStream_t st);
size_t simt_qjl_scores_workspace(int64_t BH, int64_t Sq, int D);
int simt_qjl_scores(const TqQjlScoreJob& job, cudaStream_t st);
// fp32 queries and their S-projection, laid out in the job's workspace (qf aliases job.q for fp32 queries)
int simt_qjl_queries(const TqQjlScoreJob& job, const float** qf, const float** qproj, cudaStream_t st);
int simt_prod_inner_product(const float* y, int64_t ny, const int64_t* idx, const float* signs, const float* rnorm,
                            int64_t n, int D, int M, const float* rotation, const float* codebook, const float* qjl_t,
                            float* out, void* workspace, cudaStream_t st);


// packed-key logits on the tensor cores, mma.sync (tq_attn_mma.cu); queries already rotated
bool mma_score_eligible(const TqScoreJob& job);
int mma_score_packed(const TqScoreJob& job, const float* qrot, float* stats, int nblk, int keys_per_block, cudaStream_t st);
// keys per CTA (>= min_keys, for which the caller's scratch is sized) that makes the CTAs fill whole waves
int mma_score_keys_per_block(const TqScoreJob& job, int min_keys);

// decode attention on packed keys and packed values (tq_attn_mma.cu)
size_t decode_attention_workspace(int64_t B, int64_t Hq, int64_t Sq, int64_t Sk, int keys_per_block);
int decode_attention(const TqDecodeAttnJob& job, cudaStream_t st);

// packed MSE+QJL storage and scores from it (tq_qjl_packed.cu)
int pack_mse_qjl(const uint8_t* idx_u8, const int8_t* signs, int64_t n, int D, int bits, uint8_t* idx_packed,
                 uint8_t* sign_bits, cudaStream_t st);
size_t qjl_scores_packed_workspace(int64_t BH, int64_t Sq, int D);
int qjl_scores_packed(const TqQjlPackedScoreJob& job, cudaStream_t st);

// strided row copy (tq_copy.cu)
int copy_rows(const TqCopyJob* jobs, int n_jobs, cudaStream_t st);

// tensor-core path (tq_umma.cu)
size_t umma_rotation_image_bytes(int D);
int umma_prepare_rotation_image(const float* m, int D, void* image, cudaStream_t st);
bool umma_quantize_eligible(const TqQuantizeJob& job);
int umma_quantize(const TqQuantizeJob* jobs, int n_jobs, cudaStream_t st);
bool umma_dequantize_eligible(const TqDequantizeJob& job);
int umma_dequantize(const TqDequantizeJob* jobs, int n_jobs, cudaStream_t st);
int umma_device_status();
// cuTensorMapEncodeTiled looked up through the runtime (no link-time dependency on libcuda); NULL if unavailable
typedef CUresult (*TensorMapEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                      const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                      CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
TensorMapEncodeFn tensor_map_encoder();

// tensor-core MSE + QJL compress stage (tq_v2_umma.cu)
size_t umma_v2_compress_workspace(int64_t n, int D);
bool umma_v2_compress_eligible(const TqQjlCompressJob& job);
int umma_v2_compress(const TqQjlCompressJob& job, cudaStream_t st);
int umma_v2_device_status();

// tensor-core asymmetric scores of the MSE+QJL representation (tq_qjl_umma.cu)
bool umma_qjl_scores_eligible(const TqQjlScoreJob& job);
size_t umma_qjl_scores_image_bytes(int64_t BH, int64_t Sq, int D);
int umma_qjl_scores(const TqQjlScoreJob& job, const float* qf, const float* qproj, void* images, cudaStream_t st);
int umma_qjl_device_status();

}  // namespace tq
