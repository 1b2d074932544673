// Self-test of the operand conventions every attention kernel here relies on: TMA tiled loads/stores with the
// 128-byte swizzle, thread-written swizzled tiles, K-major and MN-major shared-memory descriptors for the e4m3
// tcgen05 MMA (M = 128, N = 64 or 128, four K steps of 32), the 32x32b tensor-memory load layout, and the A operand read
// from tensor memory (written there by tcgen05.st, four e4m3 per 32-bit column): contiguous, one K step every 32 columns,
// and overwritten by the accumulator of the MMA issued right behind the one that reads it.
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
    if (warp == 0) dm::tmem_alloc(&s.tmem_base, 256);
    dm::tc_fence_before();
    __syncthreads();
    dm::tc_fence_after();
    const uint32_t tmem = s.tmem_base;
    // via_st 2, 3, 4: A lives in tensor memory.  2: columns [128, 160); 3: K step k at columns [128 + 32 k, +8); 4: K step k at
    // columns [32 k, +8), the product goes to columns [128, 256), and a second product (A and B from shared memory) is issued
    // right behind it into columns [0, 128), over the A operand the first one reads.
    const int a_tmem_mode = via_st >= 2 ? via_st : 0;
    if (a_tmem_mode) via_st = 0;

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
    if (a_tmem_mode) {
        uint32_t w[32];
        const uint4* src = reinterpret_cast<const uint4*>(a_gmem + tid * 128);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const uint4 v = src[c];
            w[4 * c] = v.x, w[4 * c + 1] = v.y, w[4 * c + 2] = v.z, w[4 * c + 3] = v.w;
        }
        const uint32_t base = a_tmem_mode == 4 ? 0u : 128u, step = a_tmem_mode == 2 ? 8u : 32u;
#pragma unroll
        for (int k = 0; k < 4; ++k) dm::tmem_st8(dm::tmem_addr(tmem, warp * 32, base + step * k), w + 8 * k);
        dm::tmem_st_wait();
        dm::tc_fence_before();
    }
    dm::mbar_wait(&s.bar_load, 0, wc);
    __syncthreads();
    if (tid == 0 && a_tmem_mode) {
        dm::tc_fence_after();
        const uint32_t idesc = dm::idesc_e4m3(128, n_cols, false, b_mn != 0);
        const uint32_t b_lo = dm::smem_desc_lo_sw128(dm::smem_u32(s.b));
        const uint32_t base = a_tmem_mode == 4 ? 0u : 128u, step = a_tmem_mode == 2 ? 8u : 32u;
        const uint32_t d = a_tmem_mode == 4 ? tmem + 128 : tmem;
        dm::umma_e4m3_ts<false>(d, tmem + base, b_lo, idesc);
#pragma unroll
        for (int k = 1; k < 4; ++k) dm::umma_e4m3_ts<true>(d, tmem + base + step * k, b_lo + (b_mn ? 256 * k : 2 * k), idesc);
        if (a_tmem_mode == 4) {
            const uint32_t a_lo = dm::smem_desc_lo_sw128(dm::smem_u32(s.a));
            dm::umma_e4m3_lo<false>(tmem, a_lo, b_lo, idesc);
#pragma unroll
            for (int k = 1; k < 4; ++k) dm::umma_e4m3_lo<true>(tmem, a_lo + 2 * k, b_lo + (b_mn ? 256 * k : 2 * k), idesc);
        }
        dm::umma_commit(&s.bar_mma);
    } else if (tid == 0) {
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
        dm::tmem_ld32(dm::tmem_addr(tmem, warp * 32, (a_tmem_mode == 4 ? 128 : 0) + c0), r);
        dm::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) c_out[tid * n_cols + c0 + j] = __uint_as_float(r[j]);
        if (a_tmem_mode == 4) {     // the second product, as raw fp32 behind the first in the same output buffer
            dm::tmem_ld32(dm::tmem_addr(tmem, warp * 32, c0), r);
            dm::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) c_out[128 * n_cols + tid * n_cols + c0 + j] = __uint_as_float(r[j]);
        }
    }
    dm::tc_fence_before();
    __syncthreads();
    if (warp == 0) dm::tmem_dealloc(tmem, 256);
}

// One CTA, two warps.  Warp 0 waits on an mbarrier that nothing ever arrives on, with a limit of 1024 polls: the wait gives
// up, raises the CTA's abort flag and writes DM_DEV_TIMEOUT into the status word.  Warp 1 waits on a second such barrier with
// the library's normal limit and must come back early because it sees the abort flag.  The kernel then ends normally.
__global__ void __launch_bounds__(64, 1) wait_timeout_kernel(int* status, int* polls_out) {
    __shared__ uint64_t bar[2];
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        dm::mbar_init(&bar[0], 1);
        dm::mbar_init(&bar[1], 1);
        dm::fence_mbar_init();
    }
    __syncthreads();
    dm::WaitCtx wc{&abort_flag, status};
    const bool ok = warp == 0 ? dm::mbar_wait_limit(&bar[0], 0, wc, 1u << 10) : dm::mbar_wait(&bar[1], 0, wc);
    if ((threadIdx.x & 31) == 0) polls_out[warp] = ok ? 1 : 0;
}

}  // namespace

extern "C" int dm_selftest_wait_timeout(int32_t* waits_returned_ok, void* stream, char* err, size_t errlen) {
    DM_REQUIRE(waits_returned_ok != nullptr, DM_ERR_ARG, "waits_returned_ok is NULL");
    int rc;
    if ((rc = dmh::check_device_ptr(waits_returned_ok, "waits_returned_ok", err, errlen))) return rc;
    int* status = dmh::device_status_word(err, errlen);
    if (!status) return DM_ERR_CUDA;
    wait_timeout_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(status, waits_returned_ok);
    DM_CUDA(cudaGetLastError());
    return DM_OK;
}

extern "C" int dm_probe_mma(const void* a_tile, const void* b_tile, int32_t a_mn, int32_t b_mn, int32_t n_cols, int32_t via_st,
                            float* c_out, void* a_echo, void* stream, char* err, size_t errlen) {
    int rc;
    if ((rc = dmh::check_device_ptr(a_tile, "a_tile", err, errlen))) return rc;
    if ((rc = dmh::check_device_ptr(b_tile, "b_tile", err, errlen))) return rc;
    if ((rc = dmh::check_device_ptr(c_out, "c_out", err, errlen))) return rc;
    if ((rc = dmh::check_device_ptr(a_echo, "a_echo", err, errlen))) return rc;
    DM_REQUIRE(n_cols == 64 || n_cols == 128, DM_ERR_ARG, "n_cols must be 64 or 128");
    DM_REQUIRE(!(b_mn && n_cols != 128), DM_ERR_ARG, "an MN-major B tile is always 128 columns wide");
    DM_REQUIRE(via_st >= 0 && via_st <= 4, DM_ERR_ARG, "via_st must be 0 .. 4");
    DM_REQUIRE(via_st < 2 || !a_mn, DM_ERR_ARG, "an A operand in tensor memory is always K-major");
    DM_REQUIRE(via_st != 4 || n_cols == 128, DM_ERR_ARG, "the overwrite probe uses 128 columns");
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
