// Launcher of the split-KV log-sum-exp merge, shared by fa_combine() and fa_kvcache().
#pragma once

#include "common.h"

namespace fa {

int launch_combine(const float* o_accum, const float* lse_accum, void* o, float* lse, int64_t rows,
                   int num_splits, int h, int seqlen_q, int d, int64_t o_batch_stride,
                   int64_t o_row_stride, int64_t o_head_stride, cudaStream_t stream);

}  // namespace fa
