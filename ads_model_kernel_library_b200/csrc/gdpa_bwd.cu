// placeholder until the backward kernel lands
#include "gdpa_common.cuh"
#include "gdpa_launch.h"
namespace gdpa {
int launch_bwd_bf16(const BwdLaunch&, int, int) { return GDPA_ERR_UNSUPPORTED_ACT_; }
int launch_dq_convert(const float*, __nv_bfloat16*, long long, cudaStream_t) { return GDPA_ERR_UNSUPPORTED_ACT_; }
int launch_fwd_softmax_bf16(const FwdLaunch&, int) { return GDPA_ERR_UNSUPPORTED_ACT_; }
int launch_fwd_fp8(const FwdLaunch&, int, int) { return GDPA_ERR_UNSUPPORTED_ACT_; }
}
