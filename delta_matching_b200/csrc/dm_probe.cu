// Self-test of the operand conventions every attention kernel here relies on: TMA tiled loads/stores with the
// 128-byte swizzle, thread-written swizzled tiles, K-major and MN-major shared-memory descriptors for the e4m3
// tcgen05 MMA (M = 128, N = 64 or 128, four K steps of 32), and the 32x32b tensor-memory load layout.
#include "dm_sm100.cuh"
#include "dm_host.h"

namespace {

struct ProbeSmem {
    alignas(1024) uint8_t a[128 * 128];
    alignas(1024) uint8_t b[128 * 128];
    alignas(1024) uint8_t a2[128 * 128];
    uint64_t bar_load;
    uint64_t bar_mma;
    uint32_t tmem_base;
    int abort_flag;
};

__global__ void __launch_bounds__(128, 1)
probe_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
             const __grid_constant__ CUtensorMap tm_echo, const uint8_t* __restrict__ a_gmem, int a_mn, int b_mn, int n_cols,
             int via_st, float* __restrict__ c_out, int* status) {
    extern __shared__ uint8_t smem_raw[];
    ProbeSmem& s = *reinterpret_cast<ProbeSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5;
    dm::WaitCtx wc{&s.abort_flag, status};

    if (tid == 0) {
        s.abort_flag = 0;
        dm::mbar_init(&s.bar_load, 1);
        dm::mbar_init(&s.bar_mma, 1);
        dm::fence_mbar_init();
    }
    if (warp == 0) dm::tmem_alloc(&s.tmem_base, 128);
    dm::tc_fence_before();
    __syncthreads();
    dm::tc_fence_after();
    const uint32_t tmem = s.tmem_base;

    if (tid == 0) {
        dm::mbar_expect_tx(&s.bar_load, 2 * 128 * 128);
        dm::tma_load_2d(s.a, &tm_a, 0, 0, &s.bar_load);
        dm::tma_load_2d(s.b, &tm_b, 0, 0, &s.bar_load);
    }
    if (via_st) {
        // thread t copies row t of A from global memory into the swizzled tile by the documented formula
        const uint4* src = reinterpret_cast<const uint4*>(a_gmem + tid * 128);
#pragma unroll
        for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(s.a2 + dm::sw128(tid, c * 16)) = src[c];
        dm::fence_proxy_async_smem();
    }
    dm::mbar_wait(&s.bar_load, 0, wc);
    __syncthreads();
    if (tid == 0) {
        if (via_st) {
            dm::tma_store_2d(&tm_echo, 0, 0, s.a2);
            dm::tma_store_commit();
        }
        dm::tc_fence_after();
        const uint32_t idesc = dm::idesc_e4m3(128, n_cols, a_mn != 0, b_mn != 0);
        const uint32_t a_addr = dm::smem_u32(via_st ? s.a2 : s.a), b_addr = dm::smem_u32(s.b);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint64_t ad = dm::smem_desc_sw128(a_addr + (a_mn ? 4096 * k : 32 * k));
            const uint64_t bd = dm::smem_desc_sw128(b_addr + (b_mn ? 4096 * k : 32 * k));
            dm::umma_e4m3(tmem, ad, bd, idesc, k > 0);
        }
        dm::umma_commit(&s.bar_mma);
        if (via_st) dm::tma_store_wait_all0();
    }
    dm::mbar_wait(&s.bar_mma, 0, wc);
    dm::tc_fence_after();
    for (int c0 = 0; c0 < n_cols; c0 += 32) {
        uint32_t r[32];
        dm::tmem_ld32(dm::tmem_addr(tmem, warp * 32, c0), r);
        dm::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) c_out[tid * n_cols + c0 + j] = __uint_as_float(r[j]);
    }
    dm::tc_fence_before();
    __syncthreads();
    if (warp == 0) dm::tmem_dealloc(tmem, 128);
}

}  // namespace

extern "C" int dm_probe_mma(const void* a_tile, const void* b_tile, int32_t a_mn, int32_t b_mn, int32_t n_cols, int32_t via_st,
                            float* c_out, void* a_echo, void* stream, char* err, size_t errlen) {
    int rc;
    if ((rc = dmh::check_device_ptr(a_tile, "a_tile", err, errlen))) return rc;
    if ((rc = dmh::check_device_ptr(b_tile, "b_tile", err, errlen))) return rc;
    if ((rc = dmh::check_device_ptr(c_out, "c_out", err, errlen))) return rc;
    if ((rc = dmh::check_device_ptr(a_echo, "a_echo", err, errlen))) return rc;
    DM_REQUIRE(n_cols == 64 || n_cols == 128, DM_ERR_ARG, "n_cols must be 64 or 128");
    DM_REQUIRE(!(b_mn && n_cols != 128), DM_ERR_ARG, "an MN-major B tile is always 128 columns wide");
    CUtensorMap ta, tb, te;
    if ((rc = dmh::make_tmap_u8(&ta, a_tile, 128, 128, 128, err, errlen))) return rc;
    if ((rc = dmh::make_tmap_u8(&tb, b_tile, 128, 128, 128, err, errlen))) return rc;
    if ((rc = dmh::make_tmap_u8(&te, a_echo, 128, 128, 128, err, errlen))) return rc;
    int* status = dmh::device_status_word(err, errlen);
    if (!status) return DM_ERR_CUDA;
    const int smem = (int)sizeof(ProbeSmem) + 1024;
    DM_CUDA(cudaFuncSetAttribute(probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    probe_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(ta, tb, te, static_cast<const uint8_t*>(a_tile), a_mn, b_mn,
                                                                     n_cols, via_st, c_out, status);
    DM_CUDA(cudaGetLastError());
    return DM_OK;
}
