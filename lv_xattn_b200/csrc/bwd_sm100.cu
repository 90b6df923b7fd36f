// placeholder until the backward block lands
#include "lvx_internal.h"
namespace lvx {
int launch_bwd_block(const lvx_shape&, const void*, const void*, const float*, const float*, const void*, const void*,
                     const int32_t*, float, float*, float*, float*, int, int*, cudaStream_t) {
  return fail(LVX_ERR_SHAPE, "lvx_bwd_block: not built yet");
}
}  // namespace lvx
