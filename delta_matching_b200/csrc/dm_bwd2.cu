// Pass 2 of the backward, head_dim 128: dQ = D^-0.5 / 256 * sum over key tiles of psi * (dS'8 K8), one CTA per
// 128-row block so the reduction order is fixed and the result deterministic (csrc/fq8_dq_pass2_hd128.h:204-396 of the
// reference, restated for tcgen05).
//
// The dS' tiles were stored by pass 1 as [key][row] (128 x 128 bytes); here they are the A operand read MN-major
// (bytes of a tile row = M = query rows, tile rows = K = keys), and the K8 tile [key][d] is the B operand read MN-major
// too, so no transposed copy of anything exists.  Per key tile: 4 x tcgen05.mma (M128 N128 K32) into one of two
// tensor-memory buffers, zero-initialised; then each thread (row, 64 d columns) folds dq += psi(row's m-block, tile) *
// tmp unless the tile is a pass-1 zero tile (psi == 0) or sits more than 8 decades below the row block's running psi
// max (the F2 / F2b skip rules).  Tiles stream through a 3-stage TMA ring; the pass is bound by the dS' read from HBM, so two CTAs share an SM (256 tensor-
// memory columns, 96 KB shared memory, <= 128 registers each) to keep more loads in flight.
#include "dm_attn_common.cuh"
#include "dm_host.h"

namespace dmh {
int check_shape(const DmShape& s, int h0, int hcount, char* err, size_t errlen);
}

namespace {

constexpr int kTile = 128 * 128;
constexpr int kStages = 3;

struct Bwd2Smem {
    alignas(1024) uint8_t a[kStages][kTile];   // dS' tile [key][row]
    alignas(1024) uint8_t b[kStages][kTile];   // K8 tile [key][d]
    uint64_t bar_ld[kStages], bar_mma[2];
    uint32_t tmem_base;
    int abort_flag;
};

struct Bwd2Params {
    const float* psi;
    __nv_bfloat16* dq;
    int H, Hk, N, h0, hcount, causal;
    float final_scale;
    int* status;
    dm::RowMap rm;
};

__global__ void __launch_bounds__(256, 2)
bwd2_d128_kernel(const __grid_constant__ CUtensorMap tm_ds, const __grid_constant__ CUtensorMap tm_k, const Bwd2Params p) {
    extern __shared__ uint8_t smem_raw[];
    Bwd2Smem& s = *reinterpret_cast<Bwd2Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const dm::HeadCoord hc = dm::head_coord(blockIdx.x, p.h0, p.hcount, p.H, p.Hk);
    const int bhl = hc.b * p.hcount + (hc.h - p.h0);
    const int nbn = p.N / 128, nbm = p.N / 64;
    const int nq_blk = p.rm.nq / 128, nbm_l = p.rm.nq / 64;
    const int rb = nq_blk - 1 - (int)blockIdx.y;       // local row block, longest first
    const int n_it = p.causal ? dm::global_block(p.rm, rb) + 1 : nbn;
    dm::WaitCtx wc{&s.abort_flag, p.status};

    if (tid == 0) {
        s.abort_flag = 0;
        for (int i = 0; i < kStages; ++i) dm::mbar_init(&s.bar_ld[i], 1);
        dm::mbar_init(&s.bar_mma[0], 1);
        dm::mbar_init(&s.bar_mma[1], 1);
        dm::fence_mbar_init();
    }
    if (warp == 0) dm::tmem_alloc(&s.tmem_base, 256);
    dm::tc_fence_before();
    __syncthreads();
    dm::tc_fence_after();
    const uint32_t tmem = s.tmem_base;
    const uint32_t lane_base = (uint32_t)(warp & 3) * 32;
    const int64_t tile0 = ((int64_t)bhl * nq_blk + rb) * nbn;   // dS' tile index of (local row block rb, key block 0)
    const int kv_row0 = hc.bhk * p.N;
    constexpr uint32_t idesc = dm::idesc_e4m3(128, 128, true, true);

    auto load = [&](int it) {
        const int st = it % kStages;
        dm::mbar_expect_tx(&s.bar_ld[st], 2 * kTile);
        dm::tma_load_2d(s.a[st], &tm_ds, 0, (int)((tile0 + it) * 128), &s.bar_ld[st]);
        dm::tma_load_2d(s.b[st], &tm_k, 0, kv_row0 + it * 128, &s.bar_ld[st]);
    };
    auto issue = [&](int it) {
        const int st = it % kStages;
        dm::mbar_wait(&s.bar_ld[st], (it / kStages) & 1, wc);
        dm::tc_fence_after();
        const uint32_t aa = dm::smem_u32(s.a[st]), ba = dm::smem_u32(s.b[st]);
#pragma unroll
        for (int k = 0; k < 4; ++k)
            dm::umma_e4m3(tmem + (it & 1) * 128, dm::smem_desc_sw128(aa + 4096 * k), dm::smem_desc_sw128(ba + 4096 * k), idesc, k > 0);
        dm::umma_commit(&s.bar_mma[it & 1]);
    };

    if (tid == 0) {
        for (int i = 0; i < kStages && i < n_it; ++i) load(i);
        issue(0);
    }

    const int mb = 2 * rb + (row >> 6);
    const float* psi_row = p.psi + ((int64_t)bhl * nbm_l + mb) * nbn;
    float psi_max = 0.f;
    float dq[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) dq[i] = 0.f;

    for (int it = 0; it < n_it; ++it) {
        if (tid == 0 && it + 1 < n_it) issue(it + 1);
        const float psi_cur = psi_row[it];
        const bool take = (psi_cur != 0.f) && !(psi_cur < psi_max * 1e-8f);
        dm::mbar_wait(&s.bar_mma[it & 1], (it >> 1) & 1, wc);
        dm::tc_fence_after();
        if (tid == 0 && it + kStages < n_it) load(it + kStages);   // the MMA that read this stage is complete
        if (take) {                                                // warp-uniform: a warp's 32 rows share one m-block
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float t[32];
                dm::tmem_ld32(dm::tmem_addr(tmem + (it & 1) * 128, lane_base, g * 64 + 32 * h), reinterpret_cast<uint32_t*>(t));
                dm::tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) dq[32 * h + i] = fmaf(t[i], psi_cur, dq[32 * h + i]);
            }
            psi_max = fmaxf(psi_max, psi_cur);
        }
        dm::tc_fence_before();
        __syncthreads();                                           // this buffer may be overwritten by tile it + 2
    }

    const int n_glob = rb * 128 + row;
    __nv_bfloat16* op = p.dq + (((int64_t)hc.b * p.rm.nq + n_glob) * p.H + hc.h) * 128 + g * 64;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        uint32_t w4[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            __nv_bfloat162 t = __floats2bfloat162_rn(dq[8 * c + 2 * e] * p.final_scale, dq[8 * c + 2 * e + 1] * p.final_scale);
            w4[e] = *reinterpret_cast<uint32_t*>(&t);
        }
        reinterpret_cast<uint4*>(op)[c] = make_uint4(w4[0], w4[1], w4[2], w4[3]);
    }
    if (warp == 0) dm::tmem_dealloc(tmem, 256);
}

// ---- head_dim 256 ---------------------------------------------------------------------------------------------------------
// psi is per 64 rows x 64 keys (csrc/fq8_dq_pass2.h:95-125,188 of the reference), so a 128-key tile is two reductions (keys
// 0..63 and 64..127: two K steps each) times two d halves = four M128 N128 accumulators = all 512 tensor-memory columns;
// a thread (row, d half) folds the two key halves in ascending order with its row's psi and the F2 / F2b skip rules.
struct Bwd2Smem256 {
    alignas(1024) uint8_t a[kStages][kTile];      // dS' tile [key][row]
    alignas(1024) uint8_t b[kStages][2][kTile];   // K8 tile [d half][key][128 bytes]
    uint64_t bar_ld[kStages], bar_mma;
    uint32_t tmem_base;
    int abort_flag;
};

__global__ void __launch_bounds__(256, 1)
bwd2_d256_kernel(const __grid_constant__ CUtensorMap tm_ds, const __grid_constant__ CUtensorMap tm_k, const Bwd2Params p) {
    extern __shared__ uint8_t smem_raw[];
    Bwd2Smem256& s = *reinterpret_cast<Bwd2Smem256*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = warp >> 2;                           // d half
    const int row = (warp & 3) * 32 + lane;
    const dm::HeadCoord hc = dm::head_coord(blockIdx.x, p.h0, p.hcount, p.H, p.Hk);
    const int bhl = hc.b * p.hcount + (hc.h - p.h0);
    const int nbn = p.N / 128, nbm = p.N / 64;
    const int rb = nbn - 1 - (int)blockIdx.y;
    const int n_it = p.causal ? rb + 1 : nbn;
    dm::WaitCtx wc{&s.abort_flag, p.status};

    if (tid == 0) {
        s.abort_flag = 0;
        for (int i = 0; i < kStages; ++i) dm::mbar_init(&s.bar_ld[i], 1);
        dm::mbar_init(&s.bar_mma, 1);
        dm::fence_mbar_init();
    }
    if (warp == 0) dm::tmem_alloc(&s.tmem_base, 512);
    dm::tc_fence_before();
    __syncthreads();
    dm::tc_fence_after();
    const uint32_t tmem = s.tmem_base;
    const uint32_t lane_base = (uint32_t)(warp & 3) * 32;
    const int64_t tile0 = ((int64_t)bhl * nbn + rb) * nbn;
    const int kv_row0 = hc.bhk * p.N;
    constexpr uint32_t idesc = dm::idesc_e4m3(128, 128, true, true);

    auto load = [&](int it) {
        const int st = it % kStages;
        dm::mbar_expect_tx(&s.bar_ld[st], 3 * kTile);
        dm::tma_load_2d(s.a[st], &tm_ds, 0, (int)((tile0 + it) * 128), &s.bar_ld[st]);
        dm::tma_load_2d(s.b[st][0], &tm_k, 0, kv_row0 + it * 128, &s.bar_ld[st]);
        dm::tma_load_2d(s.b[st][1], &tm_k, 128, kv_row0 + it * 128, &s.bar_ld[st]);
    };
    auto issue = [&](int it) {
        const int st = it % kStages;
        dm::mbar_wait(&s.bar_ld[st], (it / kStages) & 1, wc);
        dm::tc_fence_after();
        const uint64_t ad = dm::smem_desc_sw128(dm::smem_u32(s.a[st]));
#pragma unroll
        for (int kh = 0; kh < 2; ++kh)
#pragma unroll
            for (int dh = 0; dh < 2; ++dh) {
                const uint64_t bd = dm::smem_desc_sw128(dm::smem_u32(s.b[st][dh]));
#pragma unroll
                for (int k2 = 0; k2 < 2; ++k2)
                    dm::umma_e4m3(tmem + kh * 256 + dh * 128, ad + 256 * (2 * kh + k2), bd + 256 * (2 * kh + k2), idesc, k2 > 0);
            }
        dm::umma_commit(&s.bar_mma);
    };
    if (tid == 0) {
        for (int i = 0; i < kStages && i < n_it; ++i) load(i);
        issue(0);
    }

    const int mb = 2 * rb + (row >> 6);
    const float* psi_row = p.psi + ((int64_t)bhl * nbm + mb) * nbm;     // [heads, N/64, N/64]
    float psi_max = 0.f;
    float dq[128];
#pragma unroll
    for (int i = 0; i < 128; ++i) dq[i] = 0.f;

    for (int it = 0; it < n_it; ++it) {
        const float psi2[2] = {psi_row[2 * it], psi_row[2 * it + 1]};
        dm::mbar_wait(&s.bar_mma, it & 1, wc);
        dm::tc_fence_after();
        if (tid == 0 && it + kStages < n_it) load(it + kStages);
#pragma unroll
        for (int kh = 0; kh < 2; ++kh) {
            const float psi_cur = psi2[kh];
            const bool take = (psi_cur != 0.f) && !(psi_cur < psi_max * 1e-8f);
            if (take) {                                            // warp-uniform
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                    float t[32];
                    dm::tmem_ld32(dm::tmem_addr(tmem + kh * 256 + g * 128, lane_base, 32 * h), reinterpret_cast<uint32_t*>(t));
                    dm::tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) dq[32 * h + i] = fmaf(t[i], psi_cur, dq[32 * h + i]);
                }
                psi_max = fmaxf(psi_max, psi_cur);
            }
        }
        dm::tc_fence_before();
        __syncthreads();
        if (tid == 0 && it + 1 < n_it) issue(it + 1);
    }

    const int n_glob = rb * 128 + row;
    __nv_bfloat16* op = p.dq + (((int64_t)hc.b * p.N + n_glob) * p.H + hc.h) * 256 + g * 128;
#pragma unroll
    for (int c = 0; c < 16; ++c) {
        uint32_t w4[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            __nv_bfloat162 t = __floats2bfloat162_rn(dq[8 * c + 2 * e] * p.final_scale, dq[8 * c + 2 * e + 1] * p.final_scale);
            w4[e] = *reinterpret_cast<uint32_t*>(&t);
        }
        reinterpret_cast<uint4*>(op)[c] = make_uint4(w4[0], w4[1], w4[2], w4[3]);
    }
    __syncthreads();
    if (warp == 0) dm::tmem_dealloc(tmem, 512);
}

}  // namespace

namespace dmh {
int check_cp(const DmShape& s, const DmCp& cp, char* err, size_t errlen);

int prepare_bwd2(char* err, size_t errlen) {
    static DeviceOnce once;
    return device_once(once, err, errlen, [&]() -> int {
        DM_CUDA(cudaFuncSetAttribute(bwd2_d128_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Bwd2Smem) + 1024));
        DM_CUDA(cudaFuncSetAttribute(bwd2_d256_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Bwd2Smem256) + 1024));
        return DM_OK;
    });
}
}  // namespace dmh

extern "C" int dm_bwd_fp8_pass2(const void* ds8_ws, const float* psi_ws, const void* k8, DmShape sh, int32_t h0, int32_t hcount,
                                void* dq, void* stream, char* err, size_t errlen) {
    DmCp cp{sh.N, sh.N / 128, 0, 0};
    return dm_bwd_fp8_pass2_cp(ds8_ws, psi_ws, k8, sh, cp, h0, hcount, dq, stream, err, errlen);
}

extern "C" int dm_bwd_fp8_pass2_cp(const void* ds8_ws, const float* psi_ws, const void* k8, DmShape sh, DmCp cp, int32_t h0,
                                   int32_t hcount, void* dq, void* stream, char* err, size_t errlen) {
    int rc = dmh::check_shape(sh, h0, hcount, err, errlen);
    if (rc) return rc;
    const bool plain = cp.nq == sh.N && cp.half_blocks == sh.N / 128 && cp.off0 == 0;
    if (!plain && (rc = dmh::check_cp(sh, cp, err, errlen))) return rc;
    const void* ptrs[] = {ds8_ws, psi_ws, k8, dq};
    const char* names[] = {"ds8_ws", "psi_ws", "k8", "dq"};
    for (int i = 0; i < 4; ++i)
        if ((rc = dmh::check_device_ptr(ptrs[i], names[i], err, errlen))) return rc;
    DM_REQUIRE(dmh::aligned16(dq), DM_ERR_ARG, "dq must be 16-byte aligned");
    const uint64_t ntiles = (uint64_t)sh.B * hcount * (cp.nq / 128) * (sh.N / 128);
    DM_REQUIRE(ntiles * 128 < ((uint64_t)1 << 31), DM_ERR_ARG, "dS' workspace too large for one call: split the heads");
    CUtensorMap ts, tk;
    if ((rc = dmh::make_tmap_u8(&ts, ds8_ws, 128, ntiles * 128, 128, err, errlen))) return rc;
    if ((rc = dmh::make_tmap_u8(&tk, k8, sh.D, (uint64_t)sh.B * sh.Hk * sh.N, 128, err, errlen))) return rc;
    int* status = dmh::device_status_word(err, errlen);
    if (!status) return DM_ERR_CUDA;
    if ((rc = dmh::prepare_bwd2(err, errlen))) return rc;
    const float sm = sh.D == 128 ? 0.08838834764831845f : 0.0625f;
    Bwd2Params p{psi_ws, static_cast<__nv_bfloat16*>(dq), sh.H, sh.Hk, sh.N, h0, hcount, sh.causal, sm / 256.0f, status,
                 dm::RowMap{cp.nq, cp.half_blocks, cp.off0, cp.off1}};
    if (sh.D == 256) {
        const int smem = (int)sizeof(Bwd2Smem256) + 1024;
        bwd2_d256_kernel<<<dim3(sh.B * hcount, sh.N / 128), 256, smem, static_cast<cudaStream_t>(stream)>>>(ts, tk, p);
        DM_CUDA(cudaGetLastError());
        return DM_OK;
    }
    const int smem = (int)sizeof(Bwd2Smem) + 1024;
    bwd2_d128_kernel<<<dim3(sh.B * hcount, cp.nq / 128), 256, smem, static_cast<cudaStream_t>(stream)>>>(ts, tk, p);
    DM_CUDA(cudaGetLastError());
    return DM_OK;
}
