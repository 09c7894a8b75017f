// Internal entry of the forward launcher, shared by fa_fwd() and the tiled path of fa_kvcache().
#pragma once

#include "common.h"

namespace fa {

// Same as fa_fwd(); seqused_k_add is added to every seqused_k[b] on the device.
int run_fwd(const FaFwdParams* p, int seqused_k_add, cudaStream_t stream);

}  // namespace fa
