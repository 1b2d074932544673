// Arithmetic shared by the attention kernels (forward, pass 0, pass 1): the numerics constants of the reference and
// the single definition of P-hat that pass 0 and pass 1 must agree on bit for bit, so that the matched delta cancels
// rowsum(P-hat * (dP - delta)) to fp32 round-off.
#pragma once
#include "dm_sm100.cuh"

namespace dm {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLog2_448 = 8.8073549220576042f;   // csrc/softmax_fq8f.h:153 of the reference
constexpr float kPhatFloorB = 12.0f;               // P-hat basis floor in binades below the running max (softmax_fq8f.h:147)
constexpr float kMoE = 8.0f;                       // backward P-hat offset 2^8 (mainloop_bwd_sm90_fp8r.hpp:664)
constexpr float kMoInv = 1.0f / 256.0f;

// Score descale in log2 units for one (Q scale block, K scale group) pair.
__device__ __forceinline__ float descale_log2(float q8sc, float k8sc) { return __fmul_rn(__fmul_rn(q8sc, k8sc), kLog2e); }
// Per-row constant of the P-hat exponent: 8 - lse * log2(e), the product formed by one IEEE multiply.
__device__ __forceinline__ float phat_row_const(float lse) { return kMoE - __fmul_rn(lse, kLog2e); }
// P-hat = 2^min(S_raw * dsc - lse * log2e + 8, 12) (the F1 clamp of the reference, mainloop_bwd_sm90_fp8r.hpp:746).
__device__ __forceinline__ float phat(float s_raw, float dsc, float row_const) {
    return ex2(fminf(fmaf(s_raw, dsc, row_const), kMoE + 4.0f));
}

// Row map of the Q-side tensors (Q8, dO8, O, LSE, delta, dQ, dS' tiles): normally all N rows in order; under context
// parallelism a rank holds two chunks of the sequence (zig-zag), `half` 128-row blocks starting at global block off0
// followed by the rest starting at global block off1.  K-side tensors are always global.
struct RowMap {
    int nq, half, off0, off1;
};
__device__ __forceinline__ int global_block(const RowMap& m, int li) { return li < m.half ? m.off0 + li : m.off1 + (li - m.half); }

// Division by a run-time constant without the divide sequence (about thirty dependent instructions per quotient, paid by every
// role of a persistent kernel at every work item): q = (t + ((x - t) >> s1)) >> s2 with t = mulhi(x, m), exact for every
// 32-bit x and d >= 1 (round-up method of Granlund and Montgomery).  The host fills the constants.
struct FastDiv {
    uint32_t d, m, s1, s2;
};
inline FastDiv make_fastdiv(uint32_t d) {
    FastDiv f{d, 1u, 0u, 0u};
    uint32_t l = 0;
    while ((uint64_t(1) << l) < d) ++l;                          // l = ceil(log2 d)
    f.m = (uint32_t)(((uint64_t(1) << 32) * ((uint64_t(1) << l) - d)) / d + 1);
    f.s1 = l < 1 ? l : 1;
    f.s2 = l < 1 ? 0 : l - 1;
    return f;
}
__device__ __forceinline__ uint32_t fdiv(uint32_t x, const FastDiv& f) {
    const uint32_t t = __umulhi(x, f.m);
    return (t + ((x - t) >> f.s1)) >> f.s2;
}

// Problem coordinates of one CTA.
struct HeadCoord {
    int b, h, bh, bhk;
};
// The same with the two divisors (hcount, H / Hk) prepared by the host.
__device__ __forceinline__ HeadCoord head_coord(int y, int h0, const FastDiv& hcount, int H, int Hk, const FastDiv& rep) {
    HeadCoord c;
    c.b = (int)fdiv((uint32_t)y, hcount);
    c.h = h0 + y - c.b * (int)hcount.d;
    c.bh = c.b * H + c.h;
    c.bhk = c.b * Hk + (int)fdiv((uint32_t)c.h, rep);
    return c;
}
__device__ __forceinline__ HeadCoord head_coord(int y, int h0, int hcount, int H, int Hk) {
    HeadCoord c;
    c.b = y / hcount;
    c.h = h0 + y % hcount;
    c.bh = c.b * H + c.h;
    c.bhk = c.b * Hk + c.h / (H / Hk);
    return c;
}

}  // namespace dm
