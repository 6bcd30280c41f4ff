// Entry points declared in leviathan_cuda.h whose kernels are not built yet.
#include "lev_internal.h"

#define NOT_YET(ctx, what) lev_fail((ctx), LEV_UNSUPPORTED, what " is not built yet")

extern "C" int lev_op_install_json(lev_ctx* ctx, const char*, size_t, lev_op**) { return NOT_YET(ctx, "lev_op_install_json"); }
extern "C" int lev_op_uninstall(lev_ctx* ctx, lev_op*) { return NOT_YET(ctx, "lev_op_uninstall"); }
extern "C" int lev_op_describe(const lev_op*, char*, int64_t*, int64_t*, int*, int*, char*, char*) { return LEV_UNSUPPORTED; }
extern "C" int lev_op_serves(const lev_op*, const lev_weights*, int64_t) { return 0; }
