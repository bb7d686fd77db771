// Kernel instantiations of the fused-dequant GEMV for one weight format.
#include "gemv_launch.cuh"

namespace runit {

int32_t gemv_launch_q8_0(runit_ctx* ctx, const GemvArgs& a, const GemvMaps& maps, uint32_t tiles, uint32_t total_rows,
                       int cpb, bool tma, uint32_t batch, bool xf16, bool simple, const char* name) {
    if (simple) return launch_simple<RUNIT_FMT_Q8_0>(ctx, a, total_rows, batch, xf16, name);
    return launch_fmt<RUNIT_FMT_Q8_0>(ctx, a, maps, tiles, cpb, tma, batch, xf16, name);
}

}  // namespace runit
