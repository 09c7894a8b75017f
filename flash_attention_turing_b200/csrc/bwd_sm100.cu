// placeholder: replaced by the backward kernels
#include "common.h"
extern "C" size_t fa_bwd_workspace_bytes(const FaBwdParams*) { return 0; }
extern "C" int fa_bwd(const FaBwdParams*, fa_stream_t) { return fa::set_error(FA_ERR_UNSUPPORTED, "fa_bwd: not built yet"); }
