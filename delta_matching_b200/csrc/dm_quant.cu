// Producers: per-head K mean, block quantizers bf16 -> e4m3 codes + fp32 scales for Q, K, V, dO (with the optional
// stale delta), and the GQA fold of per-query-head gradients.  All HBM-bound: a warp owns one 512-byte row or two
// 256-byte rows per step (16-byte loads, 8-byte code stores per lane; 8 / 4 bytes in the stale-delta mode at head_dim
// 128), the block maximum is a warp reduction plus eight values in shared memory.
//
// Bit-exactness contract (checked against the CPU oracle, which is pinned to the reference's Triton kernels):
//   * every arithmetic step is an explicitly rounded IEEE operation (__fmul_rn, __fsub_rn, __fdiv_rn, __fadd_rn), so
//     the compiler cannot contract or reassociate; this file must never be built with --use_fast_math;
//   * Q / K / V scale = max(amax, 1e-30) / 448 (division), dO scale = max(amax, 1e-30) * fp32(1/448) (multiplication);
//   * codes = cvt.rn.satfinite.e4m3(clamp(x / scale, +-448)) with the IEEE quotient RN(x / scale).  One division per
//     element costs about ten issue slots and a MUFU, which bounds these kernels before HBM does, so the quotient is
//     formed from the block's correctly rounded reciprocal r = RN(1 / scale): q0 = RN(x r), then twice
//     q <- RN(q + RN(x - q scale) r).  The residual is exact (FMA); the first correction leaves q within one ulp of
//     x / scale, and a correction of a faithful quotient with a correctly rounded reciprocal rounds correctly
//     (Markstein), so the result carries the bits of the division; the sign of a zero quotient is restored from the
//     element (copysign, or in all-finite Q / V / dO blocks the sign bits copied into the four codes at once).  That
//     holds while no intermediate leaves the normal range: blocks whose scale is outside [2^-60, 2^60] (all-tiny,
//     huge or non-finite data) take the plain division instead, a branch that is uniform over the block;
//   * K mean = (((0 + s_0) + s_1) + ...) / N with s_j the sum of the 64 rows of chunk j in ascending row order.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include <mutex>
#include <type_traits>

#include "dm_host.h"

namespace {

constexpr float kE4M3Max = 448.0f;
constexpr float kTiny = 1e-30f;

__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xFFFF0000u); }

__device__ __forceinline__ uint32_t e4m3x4(float a, float b, float c, float d) {
    uint16_t lo, hi;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
    return (uint32_t)lo | ((uint32_t)hi << 16);
}

// RN(x / s).  kExactRcp: r = RN(1 / s), 2^-60 <= s <= 2^60 and |x| <= 449 s (see the contract at the top of the file).
// Scalar on purpose: the same steps on packed fp32 pairs measured slower in the Q quantizer (59.5 against 53.4 us on
// 134 MB) and no faster in the others.
template <bool kExactRcp>
__device__ __forceinline__ float quotient_rn(float x, float s, float r) {
    if (!kExactRcp) return __fdiv_rn(x, s);
    float q = __fmul_rn(x, r);
    q = __fmaf_rn(__fmaf_rn(-q, s, x), r, q);
    q = __fmaf_rn(__fmaf_rn(-q, s, x), r, q);
    return copysignf(q, x);
}

// ---- K mean ---------------------------------------------------------------------------------------------------------
template <int D>
__device__ __forceinline__ void kmean_partial_block(int xblk, int bh, const __nv_bfloat16* __restrict__ k, int64_t sb, int64_t sn,
                                                    int64_t sh, int Hk, int N, float* __restrict__ partials) {
    constexpr int TPC = D / 2;            // threads per 64-row chunk (two columns each)
    constexpr int CPB = 256 / TPC;        // chunks per block
    const int b = bh / Hk, h = bh % Hk;
    const int chunk = xblk * CPB + threadIdx.x / TPC;
    const int c2 = threadIdx.x % TPC;
    const __nv_bfloat16* base = k + b * sb + h * sh + (int64_t)chunk * 64 * sn + 2 * c2;
    float s0 = 0.f, s1 = 0.f;
#pragma unroll 16
    for (int r = 0; r < 64; ++r) {
        uint32_t u = *reinterpret_cast<const uint32_t*>(base + (int64_t)r * sn);
        s0 = __fadd_rn(s0, bf16_lo(u));
        s1 = __fadd_rn(s1, bf16_hi(u));
    }
    float2* out = reinterpret_cast<float2*>(partials + ((int64_t)bh * (N / 64) + chunk) * D) + c2;
    *out = make_float2(s0, s1);
}
template <int D>
__global__ void __launch_bounds__(256) kmean_partial_kernel(const __nv_bfloat16* __restrict__ k, int64_t sb, int64_t sn, int64_t sh,
                                                            int Hk, int N, float* __restrict__ partials) {
    kmean_partial_block<D>(blockIdx.x, blockIdx.y, k, sb, sn, sh, Hk, N, partials);
}

template <int D>
__global__ void kmean_fold_kernel(const float* __restrict__ partials, int N, float* __restrict__ km) {
    const int bh = blockIdx.x, d = threadIdx.x;
    const float* p = partials + (int64_t)bh * (N / 64) * D + d;
    float acc = 0.f;
    for (int j = 0; j < N / 64; ++j) acc = __fadd_rn(acc, p[(int64_t)j * D]);
    km[(int64_t)bh * D + d] = __fdiv_rn(acc, (float)N);
}

// ---- block quantizer ------------------------------------------------------------------------------------------------
// MODE 0 = Q, 1 = K, 2 = V, 3 = dO, 4 = dO with the stale delta = rowsum(dO * O) (its own instantiation: the O loads
// and the row sums cost registers the matched mode does not have to pay).
template <int D, int MODE>
__device__ __forceinline__ void quant_block(int blk, int bh, const __nv_bfloat16* __restrict__ x, int64_t sb, int64_t sn, int64_t sh,
                                            const __nv_bfloat16* __restrict__ o, int64_t ob, int64_t on, int64_t oh,
                                            const float* __restrict__ km, uint8_t* __restrict__ codes, float* __restrict__ scales,
                                            float* __restrict__ delta, int heads, int N, float sm) {
    constexpr int BLK = (MODE == 1 || MODE == 2) ? (D == 128 ? 64 : 32) : (D == 128 ? 128 : 64);
    // A lane takes 16 bytes of a row where it can (half a warp per 256-byte row at head_dim 128, two rows per step): half
    // the loads, stores and address arithmetic per element.  The stale-delta mode keeps four elements per lane, because
    // its row sum is defined as per-lane partial sums of D / 32 elements under a butterfly over 32 lanes.
    constexpr int E = (D == 128 && MODE != 4) ? 8 : D / 32;   // elements per lane
    constexpr int LPR = D / E;            // lanes per row
    constexpr int RW = 32 / LPR;          // rows per warp and step
    constexpr int RPW = BLK / (8 * RW);   // steps per warp
    // Q, V and dO: the block maximum is a maximum of bf16 magnitudes (Q's multiply by a positive constant is monotone, so
    // it commutes with the maximum), which orders like their bit patterns: two elements per instruction, on the raw pairs.
    // K subtracts a per-column mean first and takes the float route.
    constexpr bool kPackedMax = MODE != 1;
    const int b = bh / heads, h = bh % heads;
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    const int col = (l % LPR) * E, sub = l / LPR;       // this lane's columns and its row within a step
    __shared__ float s_amax[8];
    __shared__ uint32_t s_bits[8];

    float kmv[E];
    if (MODE == 1) {
#pragma unroll
        for (int e = 0; e < E; ++e) kmv[e] = km[(int64_t)bh * D + col + e];
    }
    // the block stays in registers as raw bf16 pairs between the maximum and the codes
    uint32_t u[RPW][E / 2];
    const __nv_bfloat16* xbase = x + b * sb + h * sh + col;
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        const int row = blk * BLK + (r * 8 + w) * RW + sub;
        const __nv_bfloat16* p = xbase + (int64_t)row * sn;
        if (E == 4) {
            uint2 t = *reinterpret_cast<const uint2*>(p);
            u[r][0] = t.x; u[r][1] = t.y;
        } else {
            uint4 t = *reinterpret_cast<const uint4*>(p);
            u[r][0] = t.x; u[r][1] = t.y; u[r][E / 2 - 2] = t.z; u[r][E / 2 - 1] = t.w;
        }
    }
    // element e of row r as the float the block is quantized from
    auto value = [&](int r, int e) -> float {
        float f = (e & 1) ? bf16_hi(u[r][e >> 1]) : bf16_lo(u[r][e >> 1]);
        if (MODE == 0) f = __fmul_rn(f, sm);
        if (MODE == 1) f = __fsub_rn(f, kmv[e]);
        return f;
    };

    float amax = 0.f;
    bool finite = false;                  // every element of the block is finite (known on the packed route only)
    if (kPackedMax) {
        uint32_t m = 0;
#pragma unroll
        for (int r = 0; r < RPW; ++r)
#pragma unroll
            for (int e = 0; e < E / 2; ++e) m = __vmaxu2(m, u[r][e] & 0x7FFF7FFFu);
        m = max(m & 0xFFFFu, m >> 16);
        m = __reduce_max_sync(0xffffffffu, m);
        if (l == 0) s_bits[w] = m;
        __syncthreads();
        m = s_bits[0];
#pragma unroll
        for (int i = 1; i < 8; ++i) m = max(m, s_bits[i]);
        finite = m < 0x7F80u;
        amax = __uint_as_float(m << 16);
        if (MODE == 0) amax = __fmul_rn(amax, sm);
    }
    if (!kPackedMax || !finite) {         // uniform over the block.  A NaN is skipped by the maximum, an infinity wins it.
        amax = 0.f;
#pragma unroll
        for (int r = 0; r < RPW; ++r)
#pragma unroll
            for (int e = 0; e < E; ++e) amax = fmaxf(amax, fabsf(value(r, e)));
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        if (l == 0) s_amax[w] = amax;
        __syncthreads();
        amax = s_amax[0];
#pragma unroll
        for (int i = 1; i < 8; ++i) amax = fmaxf(amax, s_amax[i]);
    }
    const float base = fmaxf(amax, kTiny);
    const float s = (MODE >= 3) ? __fmul_rn(base, __fdiv_rn(1.0f, kE4M3Max)) : __fdiv_rn(base, kE4M3Max);
    if (threadIdx.x == 0) scales[(int64_t)bh * (N / BLK) + blk] = s;

    uint8_t* cbase = codes + ((int64_t)bh * N) * D + col;
    const float rcp = __frcp_rn(s);
    // kFinite: all elements finite and the scale inside the reciprocal's range.  Then the quotient is finite, so the
    // conversion's own saturation is the clamp, and its sign is the element's: the sign bits are copied from the bf16
    // pairs into the four codes at once instead of a copysign per element.
    auto emit = [&](auto exact_rcp, auto all_finite) {
        constexpr bool kExactRcp = decltype(exact_rcp)::value, kFinite = decltype(all_finite)::value;
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
            const int row = blk * BLK + (r * 8 + w) * RW + sub;
            uint32_t c4[E / 4];
#pragma unroll
            for (int g = 0; g < E / 4; ++g) {
                float qv[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float xv = value(r, 4 * g + e);
                    if (kFinite) {
                        float q = __fmul_rn(xv, rcp);
                        q = __fmaf_rn(__fmaf_rn(-q, s, xv), rcp, q);
                        qv[e] = __fmaf_rn(__fmaf_rn(-q, s, xv), rcp, q);
                    } else {
                        qv[e] = fminf(fmaxf(quotient_rn<kExactRcp>(xv, s, rcp), -kE4M3Max), kE4M3Max);
                    }
                }
                c4[g] = e4m3x4(qv[0], qv[1], qv[2], qv[3]);
                if (kFinite) {
                    const uint32_t sign = __byte_perm(u[r][2 * g], u[r][2 * g + 1], 0x7531);   // the high byte of each bf16
                    c4[g] = (c4[g] & 0x7F7F7F7Fu) | (sign & 0x80808080u);
                }
            }
            if (E == 4) {
                *reinterpret_cast<uint32_t*>(cbase + (int64_t)row * D) = c4[0];
            } else {
                *reinterpret_cast<uint2*>(cbase + (int64_t)row * D) = make_uint2(c4[0], c4[E / 4 - 1]);
            }
            if (MODE == 4) {
                // stale delta from the RAW dO and the bf16 O
                const __nv_bfloat16* po = o + b * ob + h * oh + (int64_t)row * on + col;
                uint32_t uo[E / 2];
                if (E == 4) {
                    uint2 t = *reinterpret_cast<const uint2*>(po);
                    uo[0] = t.x; uo[1] = t.y;
                } else {
                    uint4 t = *reinterpret_cast<const uint4*>(po);
                    uo[0] = t.x; uo[1] = t.y; uo[E / 2 - 2] = t.z; uo[E / 2 - 1] = t.w;
                }
                float acc = __fmul_rn(bf16_lo(u[r][0]), bf16_lo(uo[0]));
                acc = __fadd_rn(acc, __fmul_rn(bf16_hi(u[r][0]), bf16_hi(uo[0])));
#pragma unroll
                for (int e = 1; e < E / 2; ++e) {
                    acc = __fadd_rn(acc, __fmul_rn(bf16_lo(u[r][e]), bf16_lo(uo[e])));
                    acc = __fadd_rn(acc, __fmul_rn(bf16_hi(u[r][e]), bf16_hi(uo[e])));
                }
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, off));
                if (l == 0) delta[(int64_t)bh * N + row] = acc;
            }
        }
    };
    const bool in_range = s >= 0x1p-60f && s <= 0x1p60f;
    if (kPackedMax && finite && in_range) emit(std::true_type{}, std::true_type{});
    else if (in_range) emit(std::true_type{}, std::false_type{});
    else emit(std::false_type{}, std::false_type{});
}

template <int D, int MODE>
__global__ void __launch_bounds__(256) quant_kernel(const __nv_bfloat16* __restrict__ x, int64_t sb, int64_t sn, int64_t sh,
                                                    const __nv_bfloat16* __restrict__ o, int64_t ob, int64_t on, int64_t oh,
                                                    const float* __restrict__ km, uint8_t* __restrict__ codes,
                                                    float* __restrict__ scales, float* __restrict__ delta, int heads, int N, float sm) {
    quant_block<D, MODE>(blockIdx.x, blockIdx.y, x, sb, sn, sh, o, ob, on, oh, km, codes, scales, delta, heads, N, sm);
}

// The K quantizer with the K mean's fold in front of it, for short sequences: every block folds the head's chunk sums itself
// (same order and division as kmean_fold_kernel, so the same bits; N / 64 additions per column, read from L2), which saves
// the fold's launch; the first block of a head also writes the mean out.
template <int D>
__global__ void __launch_bounds__(256) quant_k_folded_kernel(const __nv_bfloat16* __restrict__ x, int64_t sb, int64_t sn, int64_t sh,
                                                             const float* __restrict__ partials, float* __restrict__ km_out,
                                                             uint8_t* __restrict__ codes, float* __restrict__ scales, int heads, int N) {
    __shared__ float s_km[D];
    const int bh = blockIdx.y;
    if (threadIdx.x < D) {
        const float* p = partials + (int64_t)bh * (N / 64) * D + threadIdx.x;
        float acc = 0.f;
        for (int j = 0; j < N / 64; ++j) acc = __fadd_rn(acc, p[(int64_t)j * D]);
        const float m = __fdiv_rn(acc, (float)N);
        s_km[threadIdx.x] = m;
        if (blockIdx.x == 0) km_out[(int64_t)bh * D + threadIdx.x] = m;
    }
    __syncthreads();
    quant_block<D, 1>(blockIdx.x, bh, x, sb, sn, sh, nullptr, 0, 0, 0, s_km - (int64_t)bh * D, codes, scales, nullptr, heads, N, 0.f);
}

// The three producers of the forward that depend on nothing but the inputs, in one launch: K's per-chunk column sums
// (first in the grid: the K quantizer waits for them through the fold), the Q quantizer and the V quantizer.  A block
// does exactly what a block of the separate kernels does, so the results carry the same bits.
struct PrologueArgs {
    const __nv_bfloat16 *q, *k, *v;
    DmStrides qs, ks, vs;
    uint8_t *q8, *v8;
    float *q8s, *v8s, *partials;
    int H, Hk, N;
    int n_p, pbx, n_q, qbx, vbx;      // blocks of the k-sum part and their count per head; the same for Q; per head for V
    float sm;
};
template <int D>
__global__ void __launch_bounds__(256) prologue_kernel(const PrologueArgs a) {
    int i = blockIdx.x;
    if (i < a.n_p) {
        kmean_partial_block<D>(i % a.pbx, i / a.pbx, a.k, a.ks.b, a.ks.n, a.ks.h, a.Hk, a.N, a.partials);
        return;
    }
    i -= a.n_p;
    if (i < a.n_q) {
        quant_block<D, 0>(i % a.qbx, i / a.qbx, a.q, a.qs.b, a.qs.n, a.qs.h, nullptr, 0, 0, 0, nullptr, a.q8, a.q8s, nullptr, a.H, a.N, a.sm);
        return;
    }
    i -= a.n_q;
    quant_block<D, 2>(i % a.vbx, i / a.vbx, a.v, a.vs.b, a.vs.n, a.vs.h, nullptr, 0, 0, 0, nullptr, a.v8, a.v8s, nullptr, a.Hk, a.N, a.sm);
}

// ---- GQA fold -------------------------------------------------------------------------------------------------------
// blockIdx.y picks one of up to two (input, output) pairs of the same shape: dK and dV of a backward fold in one launch.
__global__ void __launch_bounds__(256) gqa_fold_kernel(const uint4* __restrict__ x0, uint4* __restrict__ out0, const uint4* __restrict__ x1,
                                                       uint4* __restrict__ out1, int64_t total_vec, int H, int Hk, int D) {
    const uint4* __restrict__ x = blockIdx.y ? x1 : x0;
    uint4* __restrict__ out = blockIdx.y ? out1 : out0;
    const int vpr = D / 8;                                   // 16-byte vectors per head row
    const int rep = H / Hk;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total_vec; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / vpr;                         // (b, n, hk)
        const int c = (int)(i % vpr);
        const int64_t bn = row / Hk;
        const int hk = (int)(row % Hk);
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.f;
        for (int r = 0; r < rep; ++r) {
            uint4 t = x[((bn * H) + hk * rep + r) * vpr + c];
            uint32_t u[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                acc[2 * e] = (r == 0) ? bf16_lo(u[e]) : __fadd_rn(acc[2 * e], bf16_lo(u[e]));
                acc[2 * e + 1] = (r == 0) ? bf16_hi(u[e]) : __fadd_rn(acc[2 * e + 1], bf16_hi(u[e]));
            }
        }
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            __nv_bfloat162 p = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
            o[e] = *reinterpret_cast<uint32_t*>(&p);
        }
        out[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

int check_geometry(int B, int heads, int N, int D, char* err, size_t errlen) {
    DM_REQUIRE(D == 128 || D == 256, DM_ERR_ARG, "head_dim must be 128 or 256 (got %d)", D);
    const int mult = D == 128 ? 256 : 128;
    DM_REQUIRE(N > 0 && N % mult == 0, DM_ERR_ARG, "seqlen must be a positive multiple of %d at head_dim %d (got %d)", mult, D, N);
    DM_REQUIRE(B > 0 && heads > 0, DM_ERR_ARG, "empty batch or no heads");
    DM_REQUIRE((int64_t)B * heads <= 65535, DM_ERR_ARG, "batch * nheads must be at most 65535 (got %lld)", (long long)B * heads);
    return DM_OK;
}

int check_strides(const void* p, DmStrides s, int D, const char* name, char* err, size_t errlen) {
    DM_REQUIRE((reinterpret_cast<uintptr_t>(p) & 15u) == 0, DM_ERR_ARG, "%s is not 16-byte aligned", name);
    DM_REQUIRE(s.b % 8 == 0 && s.n % 8 == 0 && s.h % 8 == 0, DM_ERR_ARG,
               "%s: batch / seqlen / head strides must be multiples of 8 elements (16-byte aligned rows)", name);
    DM_REQUIRE(s.n >= D, DM_ERR_ARG, "%s: seqlen stride %lld is smaller than head_dim", name, (long long)s.n);
    return DM_OK;
}

}  // namespace

extern "C" size_t dm_kmean_scratch_bytes(int32_t B, int32_t Hk, int32_t N, int32_t D) {
    if (B <= 0 || Hk <= 0 || N <= 0 || D <= 0) return 0;
    return (size_t)B * Hk * (N / 64) * D * sizeof(float);
}

extern "C" int dm_kmean(const void* k, DmStrides ks, int32_t B, int32_t Hk, int32_t N, int32_t D, float* km, float* partials,
                        void* stream, char* err, size_t errlen) {
    int rc = check_geometry(B, Hk, N, D, err, errlen);
    if (rc) return rc;
    if ((rc = dmh::check_device_ptr(k, "k", err, errlen))) return rc;
    if ((rc = dmh::check_device_ptr(km, "km", err, errlen))) return rc;
    if ((rc = dmh::check_device_ptr(partials, "partials", err, errlen))) return rc;
    if ((rc = check_strides(k, ks, D, "k", err, errlen))) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const __nv_bfloat16* kp = static_cast<const __nv_bfloat16*>(k);
    if (D == 128) {
        kmean_partial_kernel<128><<<dim3(N / 64 / 4, B * Hk), 256, 0, st>>>(kp, ks.b, ks.n, ks.h, Hk, N, partials);
        kmean_fold_kernel<128><<<B * Hk, 128, 0, st>>>(partials, N, km);
    } else {
        kmean_partial_kernel<256><<<dim3(N / 64 / 2, B * Hk), 256, 0, st>>>(kp, ks.b, ks.n, ks.h, Hk, N, partials);
        kmean_fold_kernel<256><<<B * Hk, 256, 0, st>>>(partials, N, km);
    }
    DM_CUDA(cudaGetLastError());
    return DM_OK;
}

extern "C" int dm_quant_qv_kpartials(const void* q, DmStrides qs, const void* k, DmStrides ks, const void* v, DmStrides vs, DmShape s,
                                     void* q8, float* q8s, void* v8, float* v8s, float* partials, void* stream, char* err, size_t errlen) {
    int rc = check_geometry(s.B, s.H, s.N, s.D, err, errlen);
    if (rc) return rc;
    DM_REQUIRE(s.Hk > 0 && s.H % s.Hk == 0, DM_ERR_ARG, "nheads (%d) must be a positive multiple of nheads_k (%d)", s.H, s.Hk);
    const void* ptrs[] = {q, k, v, q8, q8s, v8, v8s, partials};
    const char* names[] = {"q", "k", "v", "q8", "q8s", "v8", "v8s", "partials"};
    for (int i = 0; i < 8; ++i)
        if ((rc = dmh::check_device_ptr(ptrs[i], names[i], err, errlen))) return rc;
    if ((rc = check_strides(q, qs, s.D, "q", err, errlen))) return rc;
    if ((rc = check_strides(k, ks, s.D, "k", err, errlen))) return rc;
    if ((rc = check_strides(v, vs, s.D, "v", err, errlen))) return rc;
    DM_REQUIRE(dmh::aligned16(q8) && dmh::aligned16(v8), DM_ERR_ARG, "codes are not 16-byte aligned");
    const int qblk = s.D == 128 ? 128 : 64, kblk = s.D == 128 ? 64 : 32, cpb = s.D == 128 ? 4 : 2;
    PrologueArgs a;
    a.q = static_cast<const __nv_bfloat16*>(q); a.k = static_cast<const __nv_bfloat16*>(k); a.v = static_cast<const __nv_bfloat16*>(v);
    a.qs = qs; a.ks = ks; a.vs = vs;
    a.q8 = static_cast<uint8_t*>(q8); a.v8 = static_cast<uint8_t*>(v8);
    a.q8s = q8s; a.v8s = v8s; a.partials = partials;
    a.H = s.H; a.Hk = s.Hk; a.N = s.N;
    a.pbx = s.N / 64 / cpb; a.n_p = a.pbx * s.B * s.Hk;
    a.qbx = s.N / qblk; a.n_q = a.qbx * s.B * s.H;
    a.vbx = s.N / kblk;
    a.sm = s.D == 128 ? 0.08838834764831845f : 0.0625f;
    const int64_t total = (int64_t)a.n_p + a.n_q + (int64_t)a.vbx * s.B * s.Hk;
    DM_REQUIRE(total < ((int64_t)1 << 31), DM_ERR_ARG, "problem too large for one launch");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (s.D == 128) prologue_kernel<128><<<(unsigned)total, 256, 0, st>>>(a);
    else prologue_kernel<256><<<(unsigned)total, 256, 0, st>>>(a);
    DM_CUDA(cudaGetLastError());
    return DM_OK;
}

// The two halves of dm_kmean on their own, for a sequence that is split across ranks: every rank sums its own 64-row
// chunks, the partial sums are exchanged and laid out in sequence order, and every rank folds all of them in that order,
// which gives the bits dm_kmean gives on the whole sequence.
extern "C" int dm_kmean_partials(const void* k, DmStrides ks, int32_t B, int32_t Hk, int32_t N, int32_t D, float* partials, void* stream,
                                 char* err, size_t errlen) {
    int rc = check_geometry(B, Hk, N, D, err, errlen);
    if (rc) return rc;
    if ((rc = dmh::check_device_ptr(k, "k", err, errlen))) return rc;
    if ((rc = dmh::check_device_ptr(partials, "partials", err, errlen))) return rc;
    if ((rc = check_strides(k, ks, D, "k", err, errlen))) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const __nv_bfloat16* kp = static_cast<const __nv_bfloat16*>(k);
    if (D == 128) kmean_partial_kernel<128><<<dim3(N / 64 / 4, B * Hk), 256, 0, st>>>(kp, ks.b, ks.n, ks.h, Hk, N, partials);
    else kmean_partial_kernel<256><<<dim3(N / 64 / 2, B * Hk), 256, 0, st>>>(kp, ks.b, ks.n, ks.h, Hk, N, partials);
    DM_CUDA(cudaGetLastError());
    return DM_OK;
}

extern "C" int dm_kmean_fold(const float* partials, int32_t B, int32_t Hk, int32_t N, int32_t D, float* km, void* stream, char* err,
                             size_t errlen) {
    int rc = check_geometry(B, Hk, N, D, err, errlen);
    if (rc) return rc;
    if ((rc = dmh::check_device_ptr(partials, "partials", err, errlen))) return rc;
    if ((rc = dmh::check_device_ptr(km, "km", err, errlen))) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (D == 128) kmean_fold_kernel<128><<<B * Hk, 128, 0, st>>>(partials, N, km);
    else kmean_fold_kernel<256><<<B * Hk, 256, 0, st>>>(partials, N, km);
    DM_CUDA(cudaGetLastError());
    return DM_OK;
}

// ---- ordered fp32 fold ----------------------------------------------------------------------------------------------
// out[o, i] = sum over c ascending of in[o, c, i]: the fold of fp32 dK / dV partials over the query heads of a KV group
// (count = H / Hk, inner = D) and over the ranks of a sequence split (outer = 1, count = ranks), in a fixed order so the
// result does not depend on timing.  Four floats per thread; the result is rounded once, to bf16 when asked.
namespace {
__global__ void __launch_bounds__(256) fold_f32_kernel(const float4* __restrict__ in, int64_t outer, int count, int64_t inner4,
                                                       float4* __restrict__ out_f32, uint2* __restrict__ out_bf16) {
    const int64_t total = outer * inner4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t o = i / inner4, r = i - o * inner4;
        const float4* p = in + o * count * inner4 + r;
        float4 a = p[0];
        for (int c = 1; c < count; ++c) {
            const float4 b = p[(int64_t)c * inner4];
            a.x = __fadd_rn(a.x, b.x);
            a.y = __fadd_rn(a.y, b.y);
            a.z = __fadd_rn(a.z, b.z);
            a.w = __fadd_rn(a.w, b.w);
        }
        if (out_bf16) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(a.x, a.y), hi = __floats2bfloat162_rn(a.z, a.w);
            out_bf16[i] = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        } else {
            out_f32[i] = a;
        }
    }
}
}  // namespace

extern "C" int dm_fold_f32(const float* in, int64_t outer, int32_t count, int64_t inner, int32_t out_is_bf16, void* out, void* stream,
                           char* err, size_t errlen) {
    DM_REQUIRE(outer > 0 && count > 0 && inner > 0 && inner % 4 == 0, DM_ERR_ARG,
               "dm_fold_f32: outer, count, inner must be positive and inner a multiple of 4 (got %lld, %d, %lld)", (long long)outer, count,
               (long long)inner);
    int rc;
    if ((rc = dmh::check_device_ptr(in, "in", err, errlen))) return rc;
    if ((rc = dmh::check_device_ptr(out, "out", err, errlen))) return rc;
    DM_REQUIRE(dmh::aligned16(in) && dmh::aligned16(out), DM_ERR_ARG, "dm_fold_f32: pointers must be 16-byte aligned");
    const int64_t total = outer * (inner / 4);
    const int64_t want = (total + 255) / 256;
    const int grid = (int)(want < 148 * 16 ? want : 148 * 16);
    fold_f32_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const float4*>(in), outer, count, inner / 4, out_is_bf16 ? nullptr : static_cast<float4*>(out),
        out_is_bf16 ? static_cast<uint2*>(out) : nullptr);
    DM_CUDA(cudaGetLastError());
    return DM_OK;
}

// ---- fold over the query heads straight into the owners' layout of a zig-zag sequence split ---------------------------
// out[d, kv, b, rl, g, :] = sum over j ascending of part_kv[b, key(d, rl), g * rep + j, :], where rank d of W owns the
// sequence chunks d and 2W-1-d of c = N / 2W keys each: key(d, rl) = d c + rl for rl < c, (2W-1-d) c + rl - c otherwise.
// Same order of additions as fold_f32_kernel over the query heads; slice d is what this rank sends to rank d.
namespace {
__global__ void __launch_bounds__(256) fold_to_owners_kernel(const float4* __restrict__ dkp, const float4* __restrict__ dvp, int B,
                                                             int N, int Hk, int rep, int d4, int W, float4* __restrict__ out) {
    const int c = N / (2 * W);
    const int64_t per_row = (int64_t)Hk * d4;                       // float4 per (kv, b, key) row of the output
    const int64_t total = (int64_t)W * 2 * B * 2 * c * per_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t row = i / per_row;
        const int64_t e = i - row * per_row;                        // g * d4 + i4
        const int g = (int)(e / d4), i4 = (int)(e - (int64_t)g * d4);
        const int rl = (int)(row % (2 * c)); row /= 2 * c;
        const int b = (int)(row % B); row /= B;
        const int kv = (int)(row & 1), d = (int)(row >> 1);
        const int key = rl < c ? d * c + rl : (2 * W - 1 - d) * c + (rl - c);
        const float4* p = (kv ? dvp : dkp) + (((int64_t)b * N + key) * Hk + g) * rep * d4 + i4;
        float4 a = p[0];
        for (int j = 1; j < rep; ++j) {
            const float4 x = p[(int64_t)j * d4];
            a.x = __fadd_rn(a.x, x.x);
            a.y = __fadd_rn(a.y, x.y);
            a.z = __fadd_rn(a.z, x.z);
            a.w = __fadd_rn(a.w, x.w);
        }
        out[i] = a;
    }
}
}  // namespace

extern "C" int dm_fold_to_owners(const float* dkp, const float* dvp, int32_t B, int32_t N, int32_t H, int32_t Hk, int32_t D, int32_t world,
                                 float* out, void* stream, char* err, size_t errlen) {
    DM_REQUIRE(B > 0 && N > 0 && Hk > 0 && H > 0 && H % Hk == 0 && D > 0 && D % 4 == 0 && world > 0 && N % (2 * world) == 0, DM_ERR_ARG,
               "dm_fold_to_owners: needs nheads a multiple of nheads_k, head_dim a multiple of 4 and seqlen a multiple of 2 x ranks "
               "(got B %d N %d H %d Hk %d D %d ranks %d)", B, N, H, Hk, D, world);
    int rc;
    if ((rc = dmh::check_device_ptr(dkp, "dkp", err, errlen))) return rc;
    if ((rc = dmh::check_device_ptr(dvp, "dvp", err, errlen))) return rc;
    if ((rc = dmh::check_device_ptr(out, "out", err, errlen))) return rc;
    DM_REQUIRE(dmh::aligned16(dkp) && dmh::aligned16(dvp) && dmh::aligned16(out), DM_ERR_ARG,
               "dm_fold_to_owners: pointers must be 16-byte aligned");
    const int64_t total = (int64_t)2 * B * N * Hk * (D / 4);
    const int64_t want = (total + 255) / 256;
    const int grid = (int)(want < 148 * 16 ? want : 148 * 16);
    fold_to_owners_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const float4*>(dkp), reinterpret_cast<const float4*>(dvp), B, N, Hk, H / Hk, D / 4, world,
        reinterpret_cast<float4*>(out));
    DM_CUDA(cudaGetLastError());
    return DM_OK;
}

template <int D, int MODE>
static void launch_quant(const void* x, DmStrides xs, const void* o, DmStrides os, const float* km, void* codes, float* scales,
                         float* delta, int B, int heads, int N, cudaStream_t st) {
    constexpr int BLK = (MODE == 1 || MODE == 2) ? (D == 128 ? 64 : 32) : (D == 128 ? 128 : 64);
    const float sm = D == 128 ? 0.08838834764831845f : 0.0625f;
    quant_kernel<D, MODE><<<dim3(N / BLK, B * heads), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), xs.b, xs.n, xs.h, static_cast<const __nv_bfloat16*>(o), os.b, os.n, os.h, km,
        static_cast<uint8_t*>(codes), scales, delta, heads, N, sm);
}

extern "C" int dm_quant(int32_t mode, const void* x, DmStrides xs, int32_t B, int32_t heads, int32_t N, int32_t D, const float* km,
                        void* codes, float* scales, void* stream, char* err, size_t errlen) {
    DM_REQUIRE(mode >= 0 && mode <= 2, DM_ERR_ARG, "mode must be 0 (Q), 1 (K) or 2 (V); got %d", mode);
    int rc = check_geometry(B, heads, N, D, err, errlen);
    if (rc) return rc;
    if ((rc = dmh::check_device_ptr(x, "x", err, errlen))) return rc;
    if ((rc = dmh::check_device_ptr(codes, "codes", err, errlen))) return rc;
    if ((rc = dmh::check_device_ptr(scales, "scales", err, errlen))) return rc;
    if (mode == 1 && (rc = dmh::check_device_ptr(km, "km", err, errlen))) return rc;
    if ((rc = check_strides(x, xs, D, "x", err, errlen))) return rc;
    DM_REQUIRE(dmh::aligned16(codes), DM_ERR_ARG, "codes is not 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    DmStrides z = {0, 0, 0};
#define DM_Q(DD, MM) launch_quant<DD, MM>(x, xs, nullptr, z, km, codes, scales, nullptr, B, heads, N, st)
    if (D == 128) { if (mode == 0) DM_Q(128, 0); else if (mode == 1) DM_Q(128, 1); else DM_Q(128, 2); }
    else          { if (mode == 0) DM_Q(256, 0); else if (mode == 1) DM_Q(256, 1); else DM_Q(256, 2); }
#undef DM_Q
    DM_CUDA(cudaGetLastError());
    return DM_OK;
}

namespace dmh {
// K mean from the chunk sums + K codes: one launch while the fold is short (N / 64 <= 128), else the fold and the quantizer.
int launch_kmean_fold_quant_k(const void* k, DmStrides ks, const float* partials, DmShape s, float* km, void* k8, float* k8s, void* stream,
                              char* err, size_t errlen) {
    int rc;
    if (s.N / 64 > 128 || s.D == 256) {
        if ((rc = dm_kmean_fold(partials, s.B, s.Hk, s.N, s.D, km, stream, err, errlen))) return rc;
        return dm_quant(1, k, ks, s.B, s.Hk, s.N, s.D, km, k8, k8s, stream, err, errlen);
    }
    if ((rc = check_geometry(s.B, s.Hk, s.N, s.D, err, errlen))) return rc;
    const void* ptrs[] = {k, partials, km, k8, k8s};
    const char* names[] = {"k", "partials", "km", "k8", "k8s"};
    for (int i = 0; i < 5; ++i)
        if ((rc = check_device_ptr(ptrs[i], names[i], err, errlen))) return rc;
    if ((rc = check_strides(k, ks, s.D, "k", err, errlen))) return rc;
    DM_REQUIRE(aligned16(k8), DM_ERR_ARG, "codes is not 16-byte aligned");
    quant_k_folded_kernel<128><<<dim3(s.N / 64, s.B * s.Hk), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(k), ks.b, ks.n, ks.h, partials, km, static_cast<uint8_t*>(k8), k8s, s.Hk, s.N);
    DM_CUDA(cudaGetLastError());
    return DM_OK;
}
}  // namespace dmh

extern "C" int dm_quant_do(const void* dO, DmStrides dos, const void* o, DmStrides os, int32_t B, int32_t H, int32_t N, int32_t D,
                           void* codes, float* scales, float* delta, void* stream, char* err, size_t errlen) {
    int rc = check_geometry(B, H, N, D, err, errlen);
    if (rc) return rc;
    if ((rc = dmh::check_device_ptr(dO, "dO", err, errlen))) return rc;
    if ((rc = dmh::check_device_ptr(codes, "codes", err, errlen))) return rc;
    if ((rc = dmh::check_device_ptr(scales, "scales", err, errlen))) return rc;
    if ((rc = check_strides(dO, dos, D, "dO", err, errlen))) return rc;
    DM_REQUIRE((o == nullptr) == (delta == nullptr), DM_ERR_ARG, "o and delta must be given together (stale delta) or both NULL");
    if (delta) {
        if ((rc = dmh::check_device_ptr(o, "o", err, errlen))) return rc;
        if ((rc = dmh::check_device_ptr(delta, "delta", err, errlen))) return rc;
        if ((rc = check_strides(o, os, D, "o", err, errlen))) return rc;
    }
    DM_REQUIRE(dmh::aligned16(codes), DM_ERR_ARG, "codes is not 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (delta) {
        if (D == 128) launch_quant<128, 4>(dO, dos, o, os, nullptr, codes, scales, delta, B, H, N, st);
        else          launch_quant<256, 4>(dO, dos, o, os, nullptr, codes, scales, delta, B, H, N, st);
    } else {
        if (D == 128) launch_quant<128, 3>(dO, dos, o, os, nullptr, codes, scales, delta, B, H, N, st);
        else          launch_quant<256, 3>(dO, dos, o, os, nullptr, codes, scales, delta, B, H, N, st);
    }
    DM_CUDA(cudaGetLastError());
    return DM_OK;
}

namespace dmh {
// One launch for one pair (x1 == nullptr) or two pairs of the same shape.
int launch_gqa_fold(const void* x0, void* out0, const void* x1, void* out1, int B, int N, int H, int Hk, int D, void* stream, char* err,
                    size_t errlen) {
    DM_REQUIRE(B > 0 && N > 0 && H > 0 && Hk > 0 && H % Hk == 0, DM_ERR_ARG, "nheads (%d) must be a positive multiple of nheads_k (%d)", H, Hk);
    DM_REQUIRE(D % 8 == 0, DM_ERR_ARG, "head_dim must be a multiple of 8");
    int rc;
    const void* ptrs[] = {x0, out0, x1, out1};
    const char* names[] = {"x", "out", "x (second pair)", "out (second pair)"};
    for (int i = 0; i < (x1 ? 4 : 2); ++i) {
        if ((rc = check_device_ptr(ptrs[i], names[i], err, errlen))) return rc;
        DM_REQUIRE(aligned16(ptrs[i]), DM_ERR_ARG, "x / out must be 16-byte aligned");
    }
    const int64_t total = (int64_t)B * N * Hk * (D / 8);
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    gqa_fold_kernel<<<dim3(blocks, x1 ? 2 : 1), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(x0), static_cast<uint4*>(out0), static_cast<const uint4*>(x1), static_cast<uint4*>(out1), total, H, Hk, D);
    DM_CUDA(cudaGetLastError());
    return DM_OK;
}
}  // namespace dmh

extern "C" int dm_gqa_fold(const void* x, int32_t B, int32_t N, int32_t H, int32_t Hk, int32_t D, void* out, void* stream, char* err,
                           size_t errlen) {
    return dmh::launch_gqa_fold(x, out, nullptr, nullptr, B, N, H, Hk, D, stream, err, errlen);
}

// ---- K mean without any allocation ------------------------------------------------------------------------------------
// Some callers cannot allocate device memory at all: a training process that has handed the whole of HBM to its own
// arena (so a raw cudaMalloc from a library would fail or steal from it), or a latency-critical loop that must not hit
// cudaMalloc's device-wide synchronisation.  For them dm_kmean_noalloc keeps the per-chunk partial sums in a fixed array
// inside the library image.  Every GPU that loads the library holds these 4 MiB until the process exits.
constexpr size_t kNoAllocMaxFloats = (size_t)1 << 20;   // 4 MiB: B * Hk * (N / 64) * D floats, e.g. 8 KV heads x 65536 keys x 128
static __device__ __align__(256) float g_kmean_noalloc_scratch[kNoAllocMaxFloats];

// In host code the array's name is only a handle; the device address comes from cudaGetSymbolAddress, asked once per
// device with that device current and cached.
static std::mutex g_noalloc_mu;
static float* g_noalloc_ptr[64] = {nullptr};

static int noalloc_scratch(float** out, char* err, size_t errlen) {
    int dev = -1;
    DM_CUDA(cudaGetDevice(&dev));
    DM_REQUIRE(dev >= 0 && dev < 64, DM_ERR_ARG, "device index %d is out of range", dev);
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    if (!g_noalloc_ptr[dev]) {
        float* p = nullptr;
        DM_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_kmean_noalloc_scratch));
        DM_REQUIRE(p != nullptr, DM_ERR_CUDA, "cudaGetSymbolAddress returned a NULL scratch address");
        g_noalloc_ptr[dev] = p;
    }
    *out = g_noalloc_ptr[dev];
    return DM_OK;
}

extern "C" size_t dm_kmean_noalloc_max_bytes(void) { return kNoAllocMaxFloats * sizeof(float); }

extern "C" int dm_kmean_noalloc(const void* k, DmStrides ks, int32_t B, int32_t Hk, int32_t N, int32_t D, float* km, void* stream,
                                char* err, size_t errlen) {
    int rc = check_geometry(B, Hk, N, D, err, errlen);
    if (rc) return rc;
    const size_t need = dm_kmean_scratch_bytes(B, Hk, N, D);
    DM_REQUIRE(need <= kNoAllocMaxFloats * sizeof(float), DM_ERR_ARG,
               "dm_kmean_noalloc: this shape needs %zu bytes of partial sums but the built-in scratch holds %zu "
               "(B * Hk * (N / 64) * D floats must be at most %zu); use dm_kmean with caller-provided scratch",
               need, kNoAllocMaxFloats * sizeof(float), kNoAllocMaxFloats);
    if ((rc = dmh::check_device_ptr(k, "k", err, errlen))) return rc;
    if ((rc = dmh::check_device_ptr(km, "km", err, errlen))) return rc;
    if ((rc = check_strides(k, ks, D, "k", err, errlen))) return rc;
    float* partials = nullptr;
    if ((rc = noalloc_scratch(&partials, err, errlen))) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const __nv_bfloat16* kp = static_cast<const __nv_bfloat16*>(k);
    // Every partial that the fold reads is written by the partial kernel of this same call first, so nothing in the
    // shared array has to start at zero; what the previous call left there is simply overwritten.
    if (D == 128) {
        kmean_partial_kernel<128><<<dim3(N / 64 / 4, B * Hk), 256, 0, st>>>(kp, ks.b, ks.n, ks.h, Hk, N, partials);
        kmean_fold_kernel<128><<<B * Hk, 128, 0, st>>>(partials, N, km);
    } else {
        kmean_partial_kernel<256><<<dim3(N / 64 / 2, B * Hk), 256, 0, st>>>(kp, ks.b, ks.n, ks.h, Hk, N, partials);
        kmean_fold_kernel<256><<<B * Hk, 256, 0, st>>>(partials, N, km);
    }
    DM_CUDA(cudaGetLastError());
    return DM_OK;
}
