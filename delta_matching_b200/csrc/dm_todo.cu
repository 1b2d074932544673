// temporary: entry points not written yet
#include "dm_host.h"
extern "C" int dm_delta_fp8(const void*, const void*, const void*, const void*, const float*, const float*, const float*, const float*, const float*, DmShape, int32_t, int32_t, float*, void*, char* err, size_t errlen) { return dmh::fail(err, errlen, DM_ERR_UNSUPPORTED, "not built yet"); }
extern "C" int dm_bwd_workspace_bytes(DmShape, int32_t, size_t*, size_t*) { return DM_ERR_UNSUPPORTED; }
extern "C" int dm_bwd_fp8_pass1(const void*, const void*, const void*, const void*, const float*, const float*, const float*, const float*, const float*, const float*, DmShape, int32_t, int32_t, void*, void*, void*, float*, void*, char* err, size_t errlen) { return dmh::fail(err, errlen, DM_ERR_UNSUPPORTED, "not built yet"); }
extern "C" int dm_bwd_fp8_pass2(const void*, const float*, const void*, DmShape, int32_t, int32_t, void*, void*, char* err, size_t errlen) { return dmh::fail(err, errlen, DM_ERR_UNSUPPORTED, "not built yet"); }
extern "C" int dm_bwd_dbg_rowsum(const void*, const void*, const void*, const void*, const float*, const float*, const float*, const float*, const float*, const float*, DmShape, float*, float*, void*, char* err, size_t errlen) { return dmh::fail(err, errlen, DM_ERR_UNSUPPORTED, "not built yet"); }
