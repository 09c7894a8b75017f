// placeholder: replaced by the kv-cache kernels
#include "common.h"
extern "C" int fa_kvcache_num_splits(const FaKvcacheParams*) { return 1; }
extern "C" size_t fa_kvcache_workspace_bytes(const FaKvcacheParams*) { return 0; }
extern "C" int fa_kvcache(const FaKvcacheParams*, fa_stream_t) { return fa::set_error(FA_ERR_UNSUPPORTED, "fa_kvcache: not built yet"); }
