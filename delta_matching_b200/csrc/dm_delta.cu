// Pass 0 of the backward, head_dim 128: the matched delta.  delta[row] = 2^-8 * sum over visible keys of
// P-hat * dP, built from the backward's own fp8 operands with exactly the P-hat arithmetic pass 1 uses, so that
// rowsum(P-hat * (dP - delta)) cancels to fp32 round-off (csrc/fp11_delta_v6.h:338-376,458-462 of the reference).
//
// One CTA = 128 query rows of one (batch, head); 256 threads; key tiles of 128 keys ascending; TWO CTAs per SM (256
// tensor-memory columns, < 113 KB shared memory and <= 128 registers each), so one CTA's MMAs run under the other's
// arithmetic.  Per tile
//   S  = Q  K^T   and   dP = dO V^T      8 x tcgen05.mma into tensor memory (S | dP, 256 columns)
// then thread (row, key group g) forms P-hat for its 64 keys, accumulates fma(P-hat, dP * (do8sc * v8sc), a) per 32-key
// half in ascending key order, and folds each half's fp32 partial (times 2^-8) into an fp64 accumulator.  The two key
// groups' fp64 sums are added at the end and rounded once.
// Also the debug row-sum kernel: the same loop with delta subtracted, producing rowsum and abs-rowsum of
// P-hat * (dP - delta) / 256.
#include "dm_attn_common.cuh"
#include "dm_host.h"

namespace dmh {
int check_shape(const DmShape& s, int h0, int hcount, char* err, size_t errlen);
}

namespace {

constexpr int kTile = 128 * 128;

// kD = 256: a code row is two 128-byte sub-tiles (8 MMA K steps), K / V scales per 32 keys (exactly the 32-key halves this
// kernel already reduces separately), Q / dO scales per 64 rows; 192 KB of shared memory, so one CTA per SM.
template <int kD>
struct DeltaSmem {
    static constexpr int kDH = kD / 128;
    alignas(1024) uint8_t q[kDH][kTile];
    alignas(1024) uint8_t dO[kDH][kTile];
    alignas(1024) uint8_t k[2][kDH][kTile];
    alignas(1024) uint8_t v[2][kDH][kTile];
    double part[2][128];
    double part_abs[2][128];
    uint64_t bar_qdo, bar_kv[2], bar_mma[2];
    uint32_t tmem_base;
    int abort_flag;
};

struct DeltaParams {
    const float* q8s;
    const float* k8s;
    const float* v8s;
    const float* do8s;
    const float* lse;
    const float* delta_in;   // debug mode only
    float* out;              // delta, or the row sums in debug mode
    float* out_abs;          // debug mode only
    int H, Hk, N, h0, hcount, causal;
    int* status;
    dm::RowMap rm;
};

template <bool kDebug, int kD>
__global__ void __launch_bounds__(256, kD == 128 ? 2 : 1)
delta_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                  const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, const DeltaParams p) {
    extern __shared__ uint8_t smem_raw[];
    constexpr int kDH = kD / 128;
    DeltaSmem<kD>& s = *reinterpret_cast<DeltaSmem<kD>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const dm::HeadCoord hc = dm::head_coord(blockIdx.x, p.h0, p.hcount, p.H, p.Hk);
    const int nblk = p.N / 128;
    const int nq_blk = p.rm.nq / 128;
    const int li = nq_blk - 1 - (int)blockIdx.y;      // local row block
    const int I = dm::global_block(p.rm, li);       // its place in the sequence
    const int n_tiles = p.causal ? I + 1 : nblk;
    dm::WaitCtx wc{&s.abort_flag, p.status};

    if (tid == 0) {
        s.abort_flag = 0;
        dm::mbar_init(&s.bar_qdo, 1);
        for (int i = 0; i < 2; ++i) {
            dm::mbar_init(&s.bar_kv[i], 1);
            dm::mbar_init(&s.bar_mma[i], 1);
        }
        dm::fence_mbar_init();
    }
    if (warp == 0) dm::tmem_alloc(&s.tmem_base, 256);
    dm::tc_fence_before();
    __syncthreads();
    dm::tc_fence_after();
    const uint32_t tmem = s.tmem_base;
    const uint32_t lane_base = (uint32_t)(warp & 3) * 32;
    const int q_row0 = hc.bh * p.rm.nq + li * 128;
    const int kv_row0 = hc.bhk * p.N;
    constexpr uint32_t idesc = dm::idesc_e4m3(128, 128, false, false);

    auto load_kv = [&](int it) {
        const int st = it & 1;
        dm::mbar_expect_tx(&s.bar_kv[st], 2 * kDH * kTile);
        for (int hh = 0; hh < kDH; ++hh) {
            dm::tma_load_2d(s.k[st][hh], &tm_k, 128 * hh, kv_row0 + it * 128, &s.bar_kv[st]);
            dm::tma_load_2d(s.v[st][hh], &tm_v, 128 * hh, kv_row0 + it * 128, &s.bar_kv[st]);
        }
    };
    auto issue = [&](int it) {   // S and dP of key tile `it`
        const int st = it & 1;
        dm::mbar_wait(&s.bar_kv[st], (it >> 1) & 1, wc);
        dm::tc_fence_after();
        const uint32_t t_s = tmem, t_dp = t_s + 128;
#pragma unroll
        for (int hh = 0; hh < kDH; ++hh) {
            const uint64_t qd = dm::smem_desc_sw128(dm::smem_u32(s.q[hh])), kd = dm::smem_desc_sw128(dm::smem_u32(s.k[st][hh]));
#pragma unroll
            for (int k = 0; k < 4; ++k) dm::umma_e4m3(t_s, qd + 2 * k, kd + 2 * k, idesc, (hh | k) != 0);
        }
#pragma unroll
        for (int hh = 0; hh < kDH; ++hh) {
            const uint64_t dd = dm::smem_desc_sw128(dm::smem_u32(s.dO[hh])), vd = dm::smem_desc_sw128(dm::smem_u32(s.v[st][hh]));
#pragma unroll
            for (int k = 0; k < 4; ++k) dm::umma_e4m3(t_dp, dd + 2 * k, vd + 2 * k, idesc, (hh | k) != 0);
        }
        dm::umma_commit(&s.bar_mma[0]);
    };

    if (tid == 0) {
        dm::mbar_expect_tx(&s.bar_qdo, 2 * kDH * kTile);
        for (int hh = 0; hh < kDH; ++hh) {
            dm::tma_load_2d(s.q[hh], &tm_q, 128 * hh, q_row0, &s.bar_qdo);
            dm::tma_load_2d(s.dO[hh], &tm_do, 128 * hh, q_row0, &s.bar_qdo);
        }
        load_kv(0);
        if (n_tiles > 1) load_kv(1);
        dm::mbar_wait(&s.bar_qdo, 0, wc);
        issue(0);
    }

    const int sq = kD == 128 ? (int)((int64_t)hc.bh * nq_blk + li) : (int)((int64_t)hc.bh * (p.rm.nq / 64) + 2 * li + (row >> 6));
    const float q8sc = p.q8s[sq];
    const float do8sc = p.do8s[sq];
    const int n_glob = li * 128 + row;              // row inside the (local) Q-side tensors
    const float rc = dm::phat_row_const(p.lse[(int64_t)hc.bh * p.rm.nq + n_glob]);
    const float dlt = kDebug ? p.delta_in[(int64_t)hc.bh * p.rm.nq + n_glob] : 0.f;
    double acc = 0.0, acc_abs = 0.0;

    for (int it = 0; it < n_tiles; ++it) {
        const int st = it & 1;
        // scale group of (key group g, 32-key half h): one per 64 keys at head_dim 128, one per 32 keys at head_dim 256
        float dsc2[2], dpsc2[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int64_t si = kD == 128 ? (int64_t)hc.bhk * (p.N / 64) + 2 * it + g : (int64_t)hc.bhk * (p.N / 32) + 4 * it + 2 * g + h;
            dsc2[h] = dm::descale_log2(q8sc, p.k8s[si]);
            dpsc2[h] = do8sc * p.v8s[si];
        }
        const bool diag = p.causal && it == I;
        dm::mbar_wait(&s.bar_mma[0], it & 1, wc);
        dm::tc_fence_after();
        const uint32_t t_s = tmem, t_dp = t_s + 128;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            float sv[32], dp[32];
            dm::tmem_ld32(dm::tmem_addr(t_s, lane_base, g * 64 + half * 32), reinterpret_cast<uint32_t*>(sv));
            dm::tmem_ld32(dm::tmem_addr(t_dp, lane_base, g * 64 + half * 32), reinterpret_cast<uint32_t*>(dp));
            dm::tmem_ld_wait();
            float a = 0.f, aa = 0.f;
            const float dsc = dsc2[half], dpsc = dpsc2[half];
#pragma unroll
            for (int c = 0; c < 32; c += 2) {               // P-hat = 2^min(S dsc + rc, 12), the exponent two at a time
                dm::fma2(sv[c], sv[c + 1], sv[c], sv[c + 1], dsc, rc, rc);
                sv[c] = dm::ex2(fminf(sv[c], dm::kMoE + 4.0f));
                sv[c + 1] = dm::ex2(fminf(sv[c + 1], dm::kMoE + 4.0f));
            }
            if (diag) {                                     // the diagonal tile only: keys above the row
#pragma unroll
                for (int c = 0; c < 32; ++c)
                    if (g * 64 + half * 32 + c > row) sv[c] = 0.f;
            }
            if (kDebug) {
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const float t = sv[c] * (dp[c] * dpsc - dlt);
                    a += t;
                    aa += fabsf(t);
                }
            } else {
#pragma unroll
                for (int c = 0; c < 32; c += 2) {
                    float d0, d1;
                    dm::mul2(d0, d1, dp[c], dp[c + 1], dpsc, dpsc);
                    a = fmaf(sv[c], d0, a);
                    a = fmaf(sv[c + 1], d1, a);
                }
            }
            acc += (double)(a * dm::kMoInv);
            if (kDebug) acc_abs += (double)(aa * dm::kMoInv);
        }
        dm::tc_fence_before();
        __syncthreads();                       // S | dP have been read; stage `st` tiles are free
        if (tid == 0) {
            if (it + 1 < n_tiles) issue(it + 1);
            if (it + 2 < n_tiles) load_kv(it + 2);
        }
    }

    s.part[g][row] = acc;
    if (kDebug) s.part_abs[g][row] = acc_abs;
    __syncthreads();
    if (g == 0) {
        p.out[(int64_t)hc.bh * p.rm.nq + n_glob] = (float)(s.part[0][row] + s.part[1][row]);
        if (kDebug) p.out_abs[(int64_t)hc.bh * p.rm.nq + n_glob] = (float)(s.part_abs[0][row] + s.part_abs[1][row]);
    }
    if (warp == 0) dm::tmem_dealloc(tmem, 256);
}

template <bool kDebug, int kD>
int launch(const void* q8, const void* k8, const void* v8, const void* do8, const DeltaParams& p, const DmShape& sh, void* stream,
           char* err, size_t errlen) {
    int rc;
    CUtensorMap tq, td, tk, tv;
    if ((rc = dmh::make_tmap_u8(&tq, q8, kD, (uint64_t)sh.B * sh.H * p.rm.nq, 128, err, errlen))) return rc;
    if ((rc = dmh::make_tmap_u8(&td, do8, kD, (uint64_t)sh.B * sh.H * p.rm.nq, 128, err, errlen))) return rc;
    if ((rc = dmh::make_tmap_u8(&tk, k8, kD, (uint64_t)sh.B * sh.Hk * sh.N, 128, err, errlen))) return rc;
    if ((rc = dmh::make_tmap_u8(&tv, v8, kD, (uint64_t)sh.B * sh.Hk * sh.N, 128, err, errlen))) return rc;
    if ((rc = dmh::prepare_delta(err, errlen))) return rc;
    const int smem = (int)sizeof(DeltaSmem<kD>) + 1024;
    delta_kernel<kDebug, kD><<<dim3(sh.B * p.hcount, p.rm.nq / 128), 256, smem, static_cast<cudaStream_t>(stream)>>>(tq, td, tk, tv, p);
    DM_CUDA(cudaGetLastError());
    return DM_OK;
}

}  // namespace

namespace dmh {
int check_cp(const DmShape& s, const DmCp& cp, char* err, size_t errlen);

int prepare_delta(char* err, size_t errlen) {
    static DeviceOnce once;
    return device_once(once, err, errlen, [&]() -> int {
        DM_CUDA(cudaFuncSetAttribute(delta_kernel<false, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(DeltaSmem<128>) + 1024));
        DM_CUDA(cudaFuncSetAttribute(delta_kernel<true, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(DeltaSmem<128>) + 1024));
        DM_CUDA(cudaFuncSetAttribute(delta_kernel<false, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(DeltaSmem<256>) + 1024));
        DM_CUDA(cudaFuncSetAttribute(delta_kernel<true, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(DeltaSmem<256>) + 1024));
        return DM_OK;
    });
}
}  // namespace dmh

extern "C" int dm_delta_fp8(const void* q8, const void* k8, const void* v8, const void* do8, const float* q8s, const float* k8s,
                            const float* v8s, const float* do8s, const float* lse, DmShape sh, int32_t h0, int32_t hcount, float* delta,
                            void* stream, char* err, size_t errlen) {
    DmCp cp{sh.N, sh.N / 128, 0, 0};
    return dm_delta_fp8_cp(q8, k8, v8, do8, q8s, k8s, v8s, do8s, lse, sh, cp, h0, hcount, delta, stream, err, errlen);
}

extern "C" int dm_delta_fp8_cp(const void* q8, const void* k8, const void* v8, const void* do8, const float* q8s, const float* k8s,
                               const float* v8s, const float* do8s, const float* lse, DmShape sh, DmCp cp, int32_t h0, int32_t hcount,
                               float* delta, void* stream, char* err, size_t errlen) {
    int rc = dmh::check_shape(sh, h0, hcount, err, errlen);
    if (rc) return rc;
    const bool plain = cp.nq == sh.N && cp.half_blocks == sh.N / 128 && cp.off0 == 0;
    if (!plain && (rc = dmh::check_cp(sh, cp, err, errlen))) return rc;
    const void* ptrs[] = {q8, k8, v8, do8, q8s, k8s, v8s, do8s, lse, delta};
    const char* names[] = {"q8", "k8", "v8", "do8", "q8s", "k8s", "v8s", "do8s", "lse", "delta"};
    for (int i = 0; i < 10; ++i)
        if ((rc = dmh::check_device_ptr(ptrs[i], names[i], err, errlen))) return rc;
    DM_REQUIRE(sh.N % 128 == 0, DM_ERR_ARG, "seqlen must be a 128-multiple (got %d)", sh.N);
    int* status = dmh::device_status_word(err, errlen);
    if (!status) return DM_ERR_CUDA;
    DeltaParams p{q8s, k8s, v8s, do8s, lse, nullptr, delta, nullptr, sh.H, sh.Hk, sh.N, h0, hcount, sh.causal, status,
                  dm::RowMap{cp.nq, cp.half_blocks, cp.off0, cp.off1}};
    return sh.D == 128 ? launch<false, 128>(q8, k8, v8, do8, p, sh, stream, err, errlen)
                       : launch<false, 256>(q8, k8, v8, do8, p, sh, stream, err, errlen);
}

extern "C" int dm_bwd_dbg_rowsum(const void* q8, const void* k8, const void* v8, const void* do8, const float* q8s, const float* k8s,
                                 const float* v8s, const float* do8s, const float* lse, const float* delta, DmShape sh, float* rows,
                                 float* rows_abs, void* stream, char* err, size_t errlen) {
    int rc = dmh::check_shape(sh, 0, sh.H, err, errlen);
    if (rc) return rc;
    const void* ptrs[] = {q8, k8, v8, do8, q8s, k8s, v8s, do8s, lse, delta, rows, rows_abs};
    const char* names[] = {"q8", "k8", "v8", "do8", "q8s", "k8s", "v8s", "do8s", "lse", "delta", "rows", "rows_abs"};
    for (int i = 0; i < 12; ++i)
        if ((rc = dmh::check_device_ptr(ptrs[i], names[i], err, errlen))) return rc;
    int* status = dmh::device_status_word(err, errlen);
    if (!status) return DM_ERR_CUDA;
    DeltaParams p{q8s, k8s, v8s, do8s, lse, delta, rows, rows_abs, sh.H, sh.Hk, sh.N, 0, sh.H, sh.causal, status,
                  dm::RowMap{sh.N, sh.N / 128, 0, 0}};
    return sh.D == 128 ? launch<true, 128>(q8, k8, v8, do8, p, sh, stream, err, errlen)
                       : launch<true, 256>(q8, k8, v8, do8, p, sh, stream, err, errlen);
}
