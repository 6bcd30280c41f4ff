// Schedule 1 ("stream"): placeholder until the fragment-major kernels land.
#include "lev_internal.h"

int lev_repack_weights(lev_ctx*, lev_weights*) { return LEV_OK; }
bool lev_stream_supported(const lev_weights*, int64_t, int64_t, int) { return false; }
int lev_launch_matvec_stream(lev_ctx* ctx, const lev_weights*, int64_t, int64_t, const float*, int, float*) {
    return lev_fail(ctx, LEV_UNSUPPORTED, "stream schedule not built");
}
