// Composite entry points: the whole forward and the whole (unsplit) backward as one C call each, so a host language with
// an expensive foreign-function boundary (Python's ctypes costs ~20 us per call, more than most of these kernels run at
// small shapes) crosses it twice per training step instead of twelve times.  They only chain the entry points above
// them on the caller's stream; every buffer, including intermediates, is still the caller's.
#include "dm_host.h"

extern "C" int dm_attn_forward(const void* q, DmStrides qs, const void* k, DmStrides ks, const void* v, DmStrides vs, DmShape s,
                               void* q8, float* q8s, void* k8, float* k8s, void* v8, float* v8s, float* km, float* km_partials,
                               void* o, float* lse, void* stream, char* err, size_t errlen) {
    int rc;
    // three or four launches: {K column sums, Q codes, V codes}, the fold of the sums into the K mean and the K codes (one launch
    // up to 8192 keys, two beyond), attention
    if ((rc = dm_quant_qv_kpartials(q, qs, k, ks, v, vs, s, q8, q8s, v8, v8s, km_partials, stream, err, errlen))) return rc;
    if ((rc = dmh::launch_kmean_fold_quant_k(k, ks, km_partials, s, km, k8, k8s, stream, err, errlen))) return rc;
    return dm_fwd_fp8(q8, k8, v8, q8s, k8s, v8s, s, 0, s.H, o, lse, stream, err, errlen);
}

extern "C" int dm_attn_backward(const void* dO, DmStrides dos, const void* o, DmStrides os, const void* q8, const void* k8,
                                const void* v8, const float* q8s, const float* k8s, const float* v8s, const float* lse, DmShape s,
                                int32_t matched, void* do8, float* do8s, float* delta, void* dk_heads, void* dv_heads, void* ds8_ws,
                                float* psi_ws, void* dq, void* dk, void* dv, void* stream, char* err, size_t errlen) {
    int rc;
    DM_REQUIRE(delta != nullptr, DM_ERR_ARG, "delta buffer is NULL");
    if (matched) {
        if ((rc = dm_quant_do(dO, dos, nullptr, os, s.B, s.H, s.N, s.D, do8, do8s, nullptr, stream, err, errlen))) return rc;
        if ((rc = dm_delta_fp8(q8, k8, v8, do8, q8s, k8s, v8s, do8s, lse, s, 0, s.H, delta, stream, err, errlen))) return rc;
    } else {
        if ((rc = dm_quant_do(dO, dos, o, os, s.B, s.H, s.N, s.D, do8, do8s, delta, stream, err, errlen))) return rc;
    }
    const bool gqa = s.Hk < s.H;
    void* dkh = gqa ? dk_heads : dk;      // without GQA the per-query-head gradients are the result
    void* dvh = gqa ? dv_heads : dv;
    if ((rc = dm_bwd_fp8_pass1(q8, k8, v8, do8, q8s, k8s, v8s, do8s, lse, delta, s, 0, s.H, dkh, dvh, ds8_ws, psi_ws, stream, err, errlen)))
        return rc;
    if ((rc = dm_bwd_fp8_pass2(ds8_ws, psi_ws, k8, s, 0, s.H, dq, stream, err, errlen))) return rc;
    if (gqa) {      // dK and dV in one launch
        if ((rc = dmh::launch_gqa_fold(dkh, dk, dvh, dv, s.B, s.N, s.H, s.Hk, s.D, stream, err, errlen))) return rc;
    }
    return DM_OK;
}
