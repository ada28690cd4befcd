// kv_attend.cuh — launcher of the single-token KV-cache attention (kv_attend.cu).  dk <= 128.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace axb {

int launch_kv_cache_attend(const float *K_cache, const float *V_cache, const float *Q_new, float *out, int64_t BH,
                           int64_t cur_len, int64_t max_seq, int64_t dk, float scale, int sm_count, cudaStream_t st);

}  // namespace axb
