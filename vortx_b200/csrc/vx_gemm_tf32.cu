// placeholder until the tcgen05 kernel lands
#include "vx_internal.h"
namespace vx {
vx_status launch_gemm_tf32(vx_context*, float*, const float*, const float*, const vx_shapes3&, bool* eligible) {
    *eligible = false;
    return VX_OK;
}
}
