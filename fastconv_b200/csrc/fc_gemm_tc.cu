// Tensor-core (tcgen05) GEMM launchers -- placeholder until the kernels land.
#include "fc_internal.h"

namespace fc {

int launch_wino_gemm_tc(fc_context *, const float *, const float *, float *, const WinoGeom &, int) {
    set_error("tensor-core TensorGEMM is not built yet");
    return FC_ERR_UNSUPPORTED;
}

int launch_igemm_tc(fc_context *, const float *, const float *, float *, const fc_conv_desc &, int, int, int) {
    set_error("tensor-core implicit GEMM is not built yet");
    return FC_ERR_UNSUPPORTED;
}

}  // namespace fc
