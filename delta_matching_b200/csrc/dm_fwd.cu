// Forward kernel, head_dim 128: O and LSE from e4m3 Q / K / V codes and their block scales, with the reference's
// faithful P basis (per row, per 64-key group) -- csrc/softmax_fq8f.h and csrc/mainloop_fwd_sm90_fp8f.hpp of the
// reference, restated for tcgen05.
//
// One CTA = 128 query rows of one (batch, head); 256 threads.  Key tiles of 128 keys (two 64-key groups) are visited
// from the diagonal tile downwards.  Per tile:
//   S = Q K^T            4 x tcgen05.mma (M128 N128 K32), accumulator in tensor memory columns [0, 128)
//   softmax              thread (quarter q, lane, warpgroup g) owns row 32q+lane and key group g: group max, running max
//                        exchanged through shared memory, basis ms_g = max(gm_g*l2, m*l2 - 12) - log2(448),
//                        codes = e4m3(2^(S*l2 - ms_g)) written to a swizzled K-major tile; the denominator is summed
//                        from the unrounded p
//   D_g = C_g V_g        2 x tcgen05.mma per group into zero-initialised tensor-memory temporaries [128,256), [256,384)
//   O += D_g * w_g       w_g = v8sc_g * 2^(ms_g - m*l2); O lives in registers (64 columns per thread) so the
//                        cross-tile rescale by alpha is a register multiply
// K / V tiles arrive by TMA into a 2-stage ring; the S MMA of the next tile is issued as soon as S has been read, so
// the tensor pipe works under the softmax arithmetic.  Every mbarrier wait is bounded.
#include "dm_attn_common.cuh"
#include "dm_host.h"

namespace {

constexpr int kTile = 128 * 128;   // bytes of one e4m3 tile (128 rows x 128 bytes)

struct FwdSmem {
    alignas(1024) uint8_t q[kTile];
    alignas(1024) uint8_t k[2][kTile];
    alignas(1024) uint8_t v[2][kTile];
    alignas(1024) uint8_t p[kTile];
    float gmax[2][128];
    float wgt[2][128];
    float lsum[2][128];
    uint64_t bar_q, bar_kv[2], bar_s, bar_d[2];
    uint32_t tmem_base;
    int abort_flag;
};

struct FwdParams {
    const float* q8s;
    const float* k8s;
    const float* v8s;
    __nv_bfloat16* o;
    float* lse;
    int H, Hk, N, h0, hcount, causal;
    int* status;
    dm::RowMap rm;
};

__global__ void __launch_bounds__(256, 1)
fwd_d128_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const FwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    FwdSmem& s = *reinterpret_cast<FwdSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = warp >> 2;                  // warpgroup = key group inside the tile, and the 64-column half of O
    const int row = (warp & 3) * 32 + lane;   // query row inside the block = tensor-memory lane
    const dm::HeadCoord hc = dm::head_coord(blockIdx.y, p.h0, p.hcount, p.H, p.Hk);
    const int nblk = p.N / 128;
    const int nq_blk = p.rm.nq / 128;
    const int li = nq_blk - 1 - (int)blockIdx.x;  // local row block, heaviest first
    const int I = dm::global_block(p.rm, li);   // its place in the sequence (decides the causal extent)
    const int n_tiles = p.causal ? I + 1 : nblk;
    dm::WaitCtx wc{&s.abort_flag, p.status};

    if (tid == 0) {
        s.abort_flag = 0;
        dm::mbar_init(&s.bar_q, 1);
        dm::mbar_init(&s.bar_kv[0], 1);
        dm::mbar_init(&s.bar_kv[1], 1);
        dm::mbar_init(&s.bar_s, 1);
        dm::mbar_init(&s.bar_d[0], 1);
        dm::mbar_init(&s.bar_d[1], 1);
        dm::fence_mbar_init();
        dm::tma_prefetch_desc(&tm_q);
        dm::tma_prefetch_desc(&tm_k);
        dm::tma_prefetch_desc(&tm_v);
    }
    if (warp == 0) dm::tmem_alloc(&s.tmem_base, 512);
    dm::tc_fence_before();
    __syncthreads();
    dm::tc_fence_after();
    const uint32_t tmem = s.tmem_base;
    const uint32_t t_s = tmem, t_d0 = tmem + 128, t_d1 = tmem + 256;
    const uint32_t lane_base = (uint32_t)(warp & 3) * 32;

    const int q_row0 = hc.bh * p.rm.nq + li * 128;
    const int kv_row0 = hc.bhk * p.N;
    constexpr uint32_t idesc_s = dm::idesc_e4m3(128, 128, false, false);
    constexpr uint32_t idesc_pv = dm::idesc_e4m3(128, 128, false, true);

    auto load_kv = [&](int it) {   // thread 0 only
        const int j = n_tiles - 1 - it, st = it & 1;
        dm::mbar_expect_tx(&s.bar_kv[st], 2 * kTile);
        dm::tma_load_2d(s.k[st], &tm_k, 0, kv_row0 + j * 128, &s.bar_kv[st]);
        dm::tma_load_2d(s.v[st], &tm_v, 0, kv_row0 + j * 128, &s.bar_kv[st]);
    };
    auto issue_s = [&](int it) {   // thread 0 only: S = Q K^T for iteration `it`
        const int st = it & 1;
        dm::mbar_wait(&s.bar_kv[st], (it >> 1) & 1, wc);
        dm::tc_fence_after();
        const uint32_t qa = dm::smem_u32(s.q), ka = dm::smem_u32(s.k[st]);
#pragma unroll
        for (int k = 0; k < 4; ++k)
            dm::umma_e4m3(t_s, dm::smem_desc_sw128(qa + 32 * k), dm::smem_desc_sw128(ka + 32 * k), idesc_s, k > 0);
        dm::umma_commit(&s.bar_s);
    };

    if (tid == 0) {
        dm::mbar_expect_tx(&s.bar_q, kTile);
        dm::tma_load_2d(s.q, &tm_q, 0, q_row0, &s.bar_q);
        load_kv(0);
        if (n_tiles > 1) load_kv(1);
        dm::mbar_wait(&s.bar_q, 0, wc);
        issue_s(0);
    }

    const float q8sc = p.q8s[(int64_t)hc.bh * nq_blk + li];
    float m_run = -INFINITY, l_part = 0.f;
    float o_acc[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) o_acc[i] = 0.f;

    for (int it = 0; it < n_tiles; ++it) {
        const int j = n_tiles - 1 - it, st = it & 1;
        const float ks = p.k8s[(int64_t)hc.bhk * (p.N / 64) + 2 * j + g];
        const float vs = p.v8s[(int64_t)hc.bhk * (p.N / 64) + 2 * j + g];

        // ---- S for this thread's (row, key group): 64 fp32 values
        dm::mbar_wait(&s.bar_s, it & 1, wc);
        dm::tc_fence_after();
        float sv[64];
        dm::tmem_ld32(dm::tmem_addr(t_s, lane_base, g * 64), reinterpret_cast<uint32_t*>(sv));
        dm::tmem_ld32(dm::tmem_addr(t_s, lane_base, g * 64 + 32), reinterpret_cast<uint32_t*>(sv) + 32);
        dm::tmem_ld_wait();
        dm::tc_fence_before();
        __syncthreads();                                   // S columns are free again
        if (tid == 0 && it + 1 < n_tiles) issue_s(it + 1);

        const float dsc = q8sc * ks;
        float gm = -INFINITY;
        if (p.causal && j == I) {
#pragma unroll
            for (int c = 0; c < 64; ++c) {
                sv[c] = (g * 64 + c > row) ? -INFINITY : sv[c] * dsc;
                gm = fmaxf(gm, sv[c]);
            }
        } else {
#pragma unroll
            for (int c = 0; c < 64; ++c) {
                sv[c] *= dsc;
                gm = fmaxf(gm, sv[c]);
            }
        }
        s.gmax[g][row] = gm;
        __syncthreads();
        const float tile_max = fmaxf(s.gmax[0][row], s.gmax[1][row]);
        const float m_new = fmaxf(m_run, tile_max);
        const float m_cur = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = dm::ex2((m_run - m_cur) * dm::kLog2e);
        const float ml2 = m_cur * dm::kLog2e;
        const float ms = fmaxf(gm * dm::kLog2e, ml2 - dm::kPhatFloorB) - dm::kLog2_448;
        float part = 0.f;
        uint32_t codes[16];
#pragma unroll
        for (int c = 0; c < 64; c += 4) {
            const float p0 = dm::ex2(fmaf(sv[c], dm::kLog2e, -ms));
            const float p1 = dm::ex2(fmaf(sv[c + 1], dm::kLog2e, -ms));
            const float p2 = dm::ex2(fmaf(sv[c + 2], dm::kLog2e, -ms));
            const float p3 = dm::ex2(fmaf(sv[c + 3], dm::kLog2e, -ms));
            part += (p0 + p1) + (p2 + p3);
            codes[c >> 2] = dm::cvt_e4m3x4(p0, p1, p2, p3);
        }
        const float sigma = dm::ex2(ms - ml2);
        l_part = fmaf(l_part, alpha, sigma * part);
        s.wgt[g][row] = vs * sigma;
#pragma unroll
        for (int c = 0; c < 4; ++c)
            *reinterpret_cast<uint4*>(s.p + dm::sw128(row, g * 64 + c * 16)) =
                make_uint4(codes[4 * c], codes[4 * c + 1], codes[4 * c + 2], codes[4 * c + 3]);
#pragma unroll
        for (int i = 0; i < 64; ++i) o_acc[i] *= alpha;
        m_run = m_new;
        dm::fence_proxy_async_smem();
        dm::tc_fence_before();
        __syncthreads();                                   // P codes and weights are visible

        if (tid == 0) {
            dm::tc_fence_after();
            const uint32_t pa = dm::smem_u32(s.p), va = dm::smem_u32(s.v[st]);
#pragma unroll
            for (int gg = 0; gg < 2; ++gg) {
#pragma unroll
                for (int k = 0; k < 2; ++k)
                    dm::umma_e4m3(gg ? t_d1 : t_d0, dm::smem_desc_sw128(pa + 64 * gg + 32 * k),
                                  dm::smem_desc_sw128(va + 8192 * gg + 4096 * k), idesc_pv, k > 0);
                dm::umma_commit(&s.bar_d[gg]);
            }
        }
        // ---- fold the two group products into O (this thread: row, columns [64 g, 64 g + 64))
#pragma unroll
        for (int gg = 0; gg < 2; ++gg) {
            dm::mbar_wait(&s.bar_d[gg], it & 1, wc);
            dm::tc_fence_after();
            const float w = s.wgt[gg][row];
            float dv[64];
            dm::tmem_ld32(dm::tmem_addr(gg ? t_d1 : t_d0, lane_base, g * 64), reinterpret_cast<uint32_t*>(dv));
            dm::tmem_ld32(dm::tmem_addr(gg ? t_d1 : t_d0, lane_base, g * 64 + 32), reinterpret_cast<uint32_t*>(dv) + 32);
            dm::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 64; ++i) o_acc[i] = fmaf(dv[i], w, o_acc[i]);
        }
        dm::tc_fence_before();
        // both PV products are complete: this stage's K / V tiles are free
        if (tid == 0 && it + 2 < n_tiles) load_kv(it + 2);
    }

    // ---- epilogue
    s.lsum[g][row] = l_part;
    __syncthreads();
    const float l = s.lsum[0][row] + s.lsum[1][row];
    const bool dead = (l == 0.f) || (l != l);
    const float inv = dead ? 0.f : 1.0f / l;
    const int n_glob = li * 128 + row;          // row inside the (local) Q-side tensors
    __nv_bfloat16* op = p.o + (((int64_t)hc.b * p.rm.nq + n_glob) * p.H + hc.h) * 128 + g * 64;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        uint32_t w4[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            __nv_bfloat162 t = __floats2bfloat162_rn(o_acc[8 * c + 2 * e] * inv, o_acc[8 * c + 2 * e + 1] * inv);
            w4[e] = *reinterpret_cast<uint32_t*>(&t);
        }
        reinterpret_cast<uint4*>(op)[c] = make_uint4(w4[0], w4[1], w4[2], w4[3]);
    }
    if (g == 0) p.lse[(int64_t)hc.bh * p.rm.nq + n_glob] = dead ? -INFINITY : m_run + logf(l);
    __syncthreads();
    if (warp == 0) dm::tmem_dealloc(tmem, 512);
}

}  // namespace

namespace dmh {
int check_shape(const DmShape& s, int h0, int hcount, char* err, size_t errlen) {
    DM_REQUIRE(s.D == 128 || s.D == 256, DM_ERR_ARG, "head_dim must be 128 or 256 (got %d)", s.D);
    const int mult = s.D == 128 ? 256 : 128;
    DM_REQUIRE(s.N > 0 && s.N % mult == 0, DM_ERR_ARG, "seqlen must be a positive multiple of %d at head_dim %d (got %d)", mult, s.D, s.N);
    DM_REQUIRE(s.B > 0, DM_ERR_ARG, "empty batch");
    DM_REQUIRE(s.Hk > 0 && s.H > 0 && s.H % s.Hk == 0, DM_ERR_ARG, "nheads (%d) must be a positive multiple of nheads_k (%d)", s.H, s.Hk);
    DM_REQUIRE((int64_t)s.B * s.H <= 65535, DM_ERR_ARG, "batch * nheads must be at most 65535 (got %lld)", (long long)s.B * s.H);
    DM_REQUIRE(h0 >= 0 && hcount > 0 && h0 + hcount <= s.H, DM_ERR_ARG, "head range [%d, %d) is outside [0, %d)", h0, h0 + hcount, s.H);
    DM_REQUIRE((int64_t)s.B * s.H * s.N < (int64_t)1 << 31, DM_ERR_ARG, "batch * nheads * seqlen must be below 2^31");
    return DM_OK;
}
}  // namespace dmh

namespace dmh {
int launch_fwd_d256(const void* q8, const void* k8, const void* v8, const float* q8s, const float* k8s, const float* v8s, DmShape sh,
                    int h0, int hcount, void* o, float* lse, void* stream, char* err, size_t errlen);
}

namespace dmh {
int check_cp(const DmShape& s, const DmCp& cp, char* err, size_t errlen) {
    DM_REQUIRE(s.D == 128, DM_ERR_UNSUPPORTED, "context-parallel row maps are built for head_dim 128 only");
    DM_REQUIRE(cp.nq > 0 && cp.nq % 256 == 0 && cp.nq <= s.N, DM_ERR_ARG, "local seqlen must be a positive multiple of 256 (got %d)", cp.nq);
    DM_REQUIRE(cp.half_blocks > 0 && cp.half_blocks % 2 == 0 && cp.half_blocks * 128 <= cp.nq, DM_ERR_ARG, "bad first-chunk size %d blocks", cp.half_blocks);
    DM_REQUIRE(cp.off0 >= 0 && cp.off0 % 2 == 0 && (cp.off0 + cp.half_blocks) * 128 <= s.N, DM_ERR_ARG, "first chunk lies outside the sequence");
    const int rest = cp.nq / 128 - cp.half_blocks;
    DM_REQUIRE(rest == 0 || (cp.off1 % 2 == 0 && cp.off1 >= cp.off0 + cp.half_blocks && (cp.off1 + rest) * 128 <= s.N), DM_ERR_ARG,
               "second chunk must follow the first and lie inside the sequence");
    return DM_OK;
}
}  // namespace dmh

extern "C" int dm_fwd_fp8(const void* q8, const void* k8, const void* v8, const float* q8s, const float* k8s, const float* v8s,
                          DmShape sh, int32_t h0, int32_t hcount, void* o, float* lse, void* stream, char* err, size_t errlen) {
    if (sh.D == 256) {
        int rc = dmh::check_shape(sh, h0, hcount, err, errlen);
        if (rc) return rc;
        const void* ptrs[] = {q8, k8, v8, q8s, k8s, v8s, o, lse};
        const char* names[] = {"q8", "k8", "v8", "q8s", "k8s", "v8s", "o", "lse"};
        for (int i = 0; i < 8; ++i)
            if ((rc = dmh::check_device_ptr(ptrs[i], names[i], err, errlen))) return rc;
        DM_REQUIRE(dmh::aligned16(q8) && dmh::aligned16(k8) && dmh::aligned16(v8) && dmh::aligned16(o), DM_ERR_ARG,
                   "code and output pointers must be 16-byte aligned");
        return dmh::launch_fwd_d256(q8, k8, v8, q8s, k8s, v8s, sh, h0, hcount, o, lse, stream, err, errlen);
    }
    DmCp cp{sh.N, sh.N / 128, 0, 0};
    return dm_fwd_fp8_cp(q8, k8, v8, q8s, k8s, v8s, sh, cp, h0, hcount, o, lse, stream, err, errlen);
}

extern "C" int dm_fwd_fp8_cp(const void* q8, const void* k8, const void* v8, const float* q8s, const float* k8s, const float* v8s,
                          DmShape sh, DmCp cp, int32_t h0, int32_t hcount, void* o, float* lse, void* stream, char* err, size_t errlen) {
    int rc = dmh::check_shape(sh, h0, hcount, err, errlen);
    if (rc) return rc;
    if ((rc = dmh::check_cp(sh, cp, err, errlen))) return rc;
    const void* ptrs[] = {q8, k8, v8, q8s, k8s, v8s, o, lse};
    const char* names[] = {"q8", "k8", "v8", "q8s", "k8s", "v8s", "o", "lse"};
    for (int i = 0; i < 8; ++i)
        if ((rc = dmh::check_device_ptr(ptrs[i], names[i], err, errlen))) return rc;
    DM_REQUIRE(dmh::aligned16(q8) && dmh::aligned16(k8) && dmh::aligned16(v8) && dmh::aligned16(o), DM_ERR_ARG,
               "code and output pointers must be 16-byte aligned");
    CUtensorMap tq, tk, tv;
    if ((rc = dmh::make_tmap_u8(&tq, q8, 128, (uint64_t)sh.B * sh.H * cp.nq, 128, err, errlen))) return rc;
    if ((rc = dmh::make_tmap_u8(&tk, k8, 128, (uint64_t)sh.B * sh.Hk * sh.N, 128, err, errlen))) return rc;
    if ((rc = dmh::make_tmap_u8(&tv, v8, 128, (uint64_t)sh.B * sh.Hk * sh.N, 128, err, errlen))) return rc;
    int* status = dmh::device_status_word(err, errlen);
    if (!status) return DM_ERR_CUDA;
    FwdParams p{q8s, k8s, v8s, static_cast<__nv_bfloat16*>(o), lse, sh.H, sh.Hk, sh.N, h0, hcount, sh.causal, status,
                dm::RowMap{cp.nq, cp.half_blocks, cp.off0, cp.off1}};
    const int smem = (int)sizeof(FwdSmem) + 1024;
    {
        static bool attr_done[64] = {false};      // the attribute is per device and sticky: set it once per device
        int dev = 0;
        DM_CUDA(cudaGetDevice(&dev));
        if (dev < 0 || dev >= 64 || !attr_done[dev]) {
            DM_CUDA(cudaFuncSetAttribute(fwd_d128_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
            if (dev >= 0 && dev < 64) attr_done[dev] = true;
        }
    }
    fwd_d128_kernel<<<dim3(cp.nq / 128, sh.B * hcount), 256, smem, static_cast<cudaStream_t>(stream)>>>(tq, tk, tv, p);
    DM_CUDA(cudaGetLastError());
    return DM_OK;
}
