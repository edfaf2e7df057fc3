// Strided block copy of the 16-bit residual window into the reconstructed cache buffers:
// every layer's K and V window in one launch.

#include "tq_common.cuh"
#include "tq_internal.h"

namespace tq {

namespace {

constexpr int kMaxCopyJobs = 128;

struct CopyView {
  const uint8_t* src;
  uint8_t* dst;
  int64_t H, S;
  int64_t ss_b, ss_h, ss_s;   // source strides in bytes
  int64_t ds_b, ds_h, ds_s;   // destination strides in bytes
  int64_t chunks;             // 16-byte chunks of the whole job
  int32_t row_chunks;         // 16-byte chunks per row
  int32_t pad_;
};

struct CopyBatch {
  int32_t n_jobs;
  int32_t pad_;
  CopyView jobs[kMaxCopyJobs];
};

// blockIdx.y = job; the blocks of a job stride over its 16-byte chunks
__global__ void __launch_bounds__(256) k_copy_rows(const __grid_constant__ CopyBatch batch) {
  const CopyView& v = batch.jobs[blockIdx.y];
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < v.chunks; c += step) {
    const int64_t r = c / v.row_chunks;
    const int64_t k = c - r * v.row_chunks;
    const int64_t s = r % v.S;
    const int64_t t = r / v.S;
    const int64_t h = t % v.H;
    const int64_t b = t / v.H;
    const uint4 val = *reinterpret_cast<const uint4*>(v.src + b * v.ss_b + h * v.ss_h + s * v.ss_s + k * 16);
    *reinterpret_cast<uint4*>(v.dst + b * v.ds_b + h * v.ds_h + s * v.ds_s + k * 16) = val;
  }
}

}  // namespace

int copy_rows(const TqCopyJob* jobs, int n_jobs, cudaStream_t st) {
  static thread_local CopyBatch batch;
  int done = 0;
  while (done < n_jobs) {
    int take = 0;
    int64_t max_chunks = 0;
    while (done < n_jobs && take < kMaxCopyJobs) {
      const TqCopyJob& j = jobs[done++];
      const int64_t rows = j.B * j.H * j.S;
      if (rows == 0) continue;
      const int64_t eb = j.elem_bytes;
      CopyView& v = batch.jobs[take++];
      v.src = reinterpret_cast<const uint8_t*>(j.src);
      v.dst = reinterpret_cast<uint8_t*>(j.dst);
      v.H = j.H; v.S = j.S;
      v.ss_b = j.sstride_b * eb; v.ss_h = j.sstride_h * eb; v.ss_s = j.sstride_s * eb;
      v.ds_b = j.dstride_b * eb; v.ds_h = j.dstride_h * eb; v.ds_s = j.dstride_s * eb;
      v.row_chunks = (int32_t)(j.D * eb / 16);
      v.chunks = rows * v.row_chunks;
      v.pad_ = 0;
      if (v.chunks > max_chunks) max_chunks = v.chunks;
    }
    if (take == 0) continue;
    batch.n_jobs = take;
    int64_t bx = (max_chunks + 255) / 256;
    if (bx > 2048) bx = 2048;
    k_copy_rows<<<dim3((unsigned)bx, (unsigned)take), 256, 0, st>>>(batch);
    int rc = check_launch();
    if (rc != TQ_OK) return rc;
  }
  return TQ_OK;
}

}  // namespace tq
