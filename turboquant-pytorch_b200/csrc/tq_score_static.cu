// tq_score_packed_noalloc: packed-key attention scores for callers that cannot allocate.
//
// Some hosts of this library have no way to hand over scratch memory: code that
// runs inside another framework's memory plan (every byte of device memory is
// already assigned and cudaMalloc is forbidden or would fragment the pool), a
// real-time serving loop that must not touch the allocator on the request path,
// or a thin FFI binding that only knows how to pass the tensors it owns.  For
// them the scratch that tq_score_packed takes from the caller lives here, in a
// fixed array inside the library image.  Every GPU that loads the library
// carries the array until the process exits, so it is kept modest (4 MiB).

#include <mutex>

#include "tq_internal.h"

namespace {

constexpr size_t kScratchBytes = TQ_SCORE_NOALLOC_SCRATCH_BYTES;
constexpr int kMaxDevices = 64;

// Scratch for rotated queries and per-block softmax partials.  In host code this
// name is only a handle for cudaGetSymbolAddress; it is not a device address.
static __device__ __align__(256) unsigned char g_score_scratch[kScratchBytes];

std::mutex g_mu;
void* g_scratch_ptr[kMaxDevices] = {};   // device address of g_score_scratch, per device ordinal

// Resolve the array's device address once per device, with that device current.  The address is
// kept until the process exits: after cudaDeviceReset (or any other destruction of the device's
// primary context) it is stale and this entry point must not be called again in the process.
int scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { tq::note_cuda_error((int)e); return TQ_ELAUNCH; }
  if (dev < 0 || dev >= kMaxDevices) return TQ_EDEVICE;    // device ordinals beyond the table below
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_score_scratch);
    if (e != cudaSuccess || p == nullptr) { tq::note_cuda_error((int)e); return TQ_ELAUNCH; }
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return TQ_OK;
}

}  // namespace

extern "C" int tq_score_packed_noalloc(const TqScoreJob* job, void* stream) {
  if (job == nullptr) return TQ_ENULL;
  if (job->bits < 1 || job->bits > 8) return TQ_EBITS;
  if (job->D < 1 || job->D > TQ_MAX_DIM) return TQ_EDIM;
  if (job->q_dtype != TQ_F32 && job->q_dtype != TQ_F16 && job->q_dtype != TQ_BF16) return TQ_EDTYPE;
  if (job->B < 0 || job->Hq < 0 || job->Sq < 0 || job->Hkv < 1 || job->Sk < 0 || job->Hq % job->Hkv != 0) return TQ_EINVAL;
  if (job->B * job->Hq * job->Sq == 0 || job->Sk == 0) return TQ_OK;
  if (job->q == nullptr || job->idx_bytes == nullptr || job->norms == nullptr || job->rotation_t == nullptr ||
      job->codebook == nullptr || job->logits == nullptr)
    return TQ_ENULL;
  const size_t need = tq::simt_score_workspace(job->B, job->Hq, job->Sq, job->Sk, job->D);
  if (need > kScratchBytes) return TQ_ETOOBIG;      // beyond the built-in scratch: use tq_score_packed
  void* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != TQ_OK) return rc;
  TqScoreJob local = *job;
  local.workspace = scratch;
  local.workspace_bytes = kScratchBytes;
  // Nothing in the scratch has to start at zero: the rotated queries and every
  // (row, key block) partial are written by this call before they are read.
  return tq::simt_score_packed(local, (cudaStream_t)stream);
}
