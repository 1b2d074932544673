// Forward kernel, head_dim 256: the head_dim-128 design (dm_fwd.cu) in the head_dim-256 geometry of the reference
// (csrc/flash_fwd_fp8f_launch.h:40, csrc/softmax_fq8f.h kGroups = 4): Q scales per 64 rows, K / V scales per 32 keys,
// key tiles of 128 keys = FOUR 32-key P groups, each with its own per-row basis.
//
// One CTA = 128 query rows of one (batch, head); 256 threads.  A code row is 256 bytes = two 128-byte swizzled sub-tiles
// (d 0..127 and d 128..255), so S = Q K^T is 8 tcgen05.mma K steps.  Thread (row, warpgroup g) owns key groups 2g and
// 2g + 1 of the tile (its 64 scores stay in registers from the maxima to the codes, beside the 128 columns of O) and the
// d columns [128 g, 128 g + 128) of O.  Per group: D_grp = C_grp V_grp as two M128 N128 K32 MMAs (one per d half) into a
// zero-initialised 256-column temporary, then O += D_grp * w_grp.  The four groups of a tile go through that one temporary
// in turn.  Every mbarrier wait is bounded.
#include "dm_attn_common.cuh"
#include "dm_host.h"

namespace dmh {
int check_shape(const DmShape& s, int h0, int hcount, char* err, size_t errlen);
}

namespace {

constexpr int kTile = 128 * 128;

struct Fwd256Smem {
    alignas(1024) uint8_t q[2][kTile];          // [d half][128 rows x 128 bytes]
    alignas(1024) uint8_t k[2][2][kTile];       // [stage][d half]
    alignas(1024) uint8_t v[2][2][kTile];
    alignas(1024) uint8_t p[kTile];             // P codes [row][128 keys]
    float gmax[4][128];
    float wgt[4][128];
    float lsum[2][128];
    uint64_t bar_q, bar_kv[2], bar_s, bar_d;
    uint32_t tmem_base;
    int abort_flag;
};

struct Fwd256Params {
    const float* q8s;
    const float* k8s;
    const float* v8s;
    __nv_bfloat16* o;
    float* lse;
    int H, Hk, N, h0, hcount, causal;
    int* status;
};

__global__ void __launch_bounds__(256, 1)
fwd_d256_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const Fwd256Params p) {
    extern __shared__ uint8_t smem_raw[];
    Fwd256Smem& s = *reinterpret_cast<Fwd256Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const dm::HeadCoord hc = dm::head_coord(blockIdx.x, p.h0, p.hcount, p.H, p.Hk);
    const int nblk = p.N / 128;
    const int I = nblk - 1 - (int)blockIdx.y;
    const int n_tiles = p.causal ? I + 1 : nblk;
    dm::WaitCtx wc{&s.abort_flag, p.status};

    if (tid == 0) {
        s.abort_flag = 0;
        dm::mbar_init(&s.bar_q, 1);
        dm::mbar_init(&s.bar_kv[0], 1);
        dm::mbar_init(&s.bar_kv[1], 1);
        dm::mbar_init(&s.bar_s, 1);
        dm::mbar_init(&s.bar_d, 1);
        dm::fence_mbar_init();
    }
    if (warp == 0) dm::tmem_alloc(&s.tmem_base, 512);
    dm::tc_fence_before();
    __syncthreads();
    dm::tc_fence_after();
    const uint32_t tmem = s.tmem_base;
    const uint32_t t_s = tmem, t_d = tmem + 128;          // S: 128 columns; D_grp: 256 columns
    const uint32_t lane_base = (uint32_t)(warp & 3) * 32;
    const int q_row0 = hc.bh * p.N + I * 128;
    const int kv_row0 = hc.bhk * p.N;
    constexpr uint32_t idesc_s = dm::idesc_e4m3(128, 128, false, false);
    constexpr uint32_t idesc_pv = dm::idesc_e4m3(128, 128, false, true);

    auto load_kv = [&](int it) {   // thread 0 only
        const int j = n_tiles - 1 - it, st = it & 1;
        dm::mbar_expect_tx(&s.bar_kv[st], 4 * kTile);
        for (int hh = 0; hh < 2; ++hh) {
            dm::tma_load_2d(s.k[st][hh], &tm_k, 128 * hh, kv_row0 + j * 128, &s.bar_kv[st]);
            dm::tma_load_2d(s.v[st][hh], &tm_v, 128 * hh, kv_row0 + j * 128, &s.bar_kv[st]);
        }
    };
    auto issue_s = [&](int it) {   // thread 0 only
        const int st = it & 1;
        dm::mbar_wait(&s.bar_kv[st], (it >> 1) & 1, wc);
        dm::tc_fence_after();
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const uint64_t qd = dm::smem_desc_sw128(dm::smem_u32(s.q[hh])), kd = dm::smem_desc_sw128(dm::smem_u32(s.k[st][hh]));
#pragma unroll
            for (int k = 0; k < 4; ++k) dm::umma_e4m3(t_s, qd + 2 * k, kd + 2 * k, idesc_s, (hh | k) != 0);
        }
        dm::umma_commit(&s.bar_s);
    };

    if (tid == 0) {
        dm::mbar_expect_tx(&s.bar_q, 2 * kTile);
        dm::tma_load_2d(s.q[0], &tm_q, 0, q_row0, &s.bar_q);
        dm::tma_load_2d(s.q[1], &tm_q, 128, q_row0, &s.bar_q);
        load_kv(0);
        if (n_tiles > 1) load_kv(1);
        dm::mbar_wait(&s.bar_q, 0, wc);
        issue_s(0);
    }

    const float q8sc = p.q8s[(int64_t)hc.bh * (p.N / 64) + 2 * I + (row >> 6)];
    float m_run = -INFINITY, l_part = 0.f;
    float o_acc[128];
#pragma unroll
    for (int i = 0; i < 128; ++i) o_acc[i] = 0.f;
    int d_phase = 0;
    // the K / V scales of a tile are read one tile ahead: read at the tile's top they are two exposed global loads
    const float* ksb = p.k8s + (int64_t)hc.bhk * (p.N / 32) + 2 * g;
    const float* vsb = p.v8s + (int64_t)hc.bhk * (p.N / 32) + 2 * g;
    float2 ks_n = *reinterpret_cast<const float2*>(ksb + 4 * (n_tiles - 1));
    float2 vs_n = *reinterpret_cast<const float2*>(vsb + 4 * (n_tiles - 1));

    for (int it = 0; it < n_tiles; ++it) {
        const int j = n_tiles - 1 - it, st = it & 1;
        const float dsc[2] = {q8sc * ks_n.x, q8sc * ks_n.y};
        const float vs[2] = {vs_n.x, vs_n.y};
        if (it + 1 < n_tiles) {
            ks_n = *reinterpret_cast<const float2*>(ksb + 4 * (j - 1));
            vs_n = *reinterpret_cast<const float2*>(vsb + 4 * (j - 1));
        }
        const bool diag = p.causal && j == I;

        dm::mbar_wait(&s.bar_s, it & 1, wc);
        dm::tc_fence_after();
        // ---- pass A: maxima of this thread's two 32-key groups (true units)
        float gm[2];
        float s2[2][32];                                   // this thread's 64 scores, kept through both passes
        dm::tmem_ld32(dm::tmem_addr(t_s, lane_base, g * 64), reinterpret_cast<uint32_t*>(s2[0]));
        dm::tmem_ld32(dm::tmem_addr(t_s, lane_base, g * 64 + 32), reinterpret_cast<uint32_t*>(s2[1]));
        dm::tmem_ld_wait();
#pragma unroll
        for (int gg = 0; gg < 2; ++gg) {
            float* sv = s2[gg];
            if (diag) {                                    // the diagonal tile only: keys above the row never win the maximum
#pragma unroll
                for (int c = 0; c < 32; ++c)
                    if (g * 64 + gg * 32 + c > row) sv[c] = -INFINITY;
            }
            float mx[4] = {fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]), fmaxf(sv[4], sv[5]), fmaxf(sv[6], sv[7])};
#pragma unroll
            for (int c = 8; c < 32; c += 8) {
                mx[0] = dm::fmax3(mx[0], sv[c], sv[c + 1]);
                mx[1] = dm::fmax3(mx[1], sv[c + 2], sv[c + 3]);
                mx[2] = dm::fmax3(mx[2], sv[c + 4], sv[c + 5]);
                mx[3] = dm::fmax3(mx[3], sv[c + 6], sv[c + 7]);
            }
            gm[gg] = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * dsc[gg];
            s.gmax[2 * g + gg][row] = gm[gg];
        }
        __syncthreads();
        // every thread holds its scores: S of the next tile may overwrite the buffer, under pass B and the products
        if (tid == 0 && it + 1 < n_tiles) issue_s(it + 1);
        const float tile_max = fmaxf(fmaxf(s.gmax[0][row], s.gmax[1][row]), fmaxf(s.gmax[2][row], s.gmax[3][row]));
        const float m_new = fmaxf(m_run, tile_max);
        const float m_cur = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = dm::ex2((m_run - m_cur) * dm::kLog2e);
        const float ml2 = m_cur * dm::kLog2e;
        m_run = m_new;
        // ---- pass B: codes and the denominator
        float lacc = 0.f;
#pragma unroll
        for (int gg = 0; gg < 2; ++gg) {
            const float ms = fmaxf(gm[gg] * dm::kLog2e, ml2 - dm::kPhatFloorB) - dm::kLog2_448;
            const float dl2 = dsc[gg] * dm::kLog2e;
            float* sv = s2[gg];                            // still in registers, masked
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t codes[8];
            const float nms = -ms;
#pragma unroll
            for (int c = 0; c < 32; c += 4) {
                float x0, x1, x2, x3;
                dm::fma2(x0, x1, sv[c], sv[c + 1], dl2, nms, nms);
                dm::fma2(x2, x3, sv[c + 2], sv[c + 3], dl2, nms, nms);
                const float p0 = dm::ex2(x0), p1 = dm::ex2(x1), p2 = dm::ex2(x2), p3 = dm::ex2(x3);
                dm::add2(acc[0], acc[1], p0, p1);
                dm::add2(acc[2], acc[3], p2, p3);
                codes[c >> 2] = dm::cvt_e4m3x4(p0, p1, p2, p3);
            }
            const float sigma = dm::ex2(ms - ml2);
            lacc = fmaf(sigma, (acc[0] + acc[1]) + (acc[2] + acc[3]), lacc);
            s.wgt[2 * g + gg][row] = vs[gg] * sigma;
            *reinterpret_cast<uint4*>(s.p + dm::sw128(row, g * 64 + gg * 32)) = make_uint4(codes[0], codes[1], codes[2], codes[3]);
            *reinterpret_cast<uint4*>(s.p + dm::sw128(row, g * 64 + gg * 32 + 16)) = make_uint4(codes[4], codes[5], codes[6], codes[7]);
        }
        l_part = fmaf(l_part, alpha, lacc);
        if (!__all_sync(0xffffffffu, alpha == 1.0f)) {
#pragma unroll
            for (int i = 0; i < 128; ++i) o_acc[i] *= alpha;
        }
        dm::fence_proxy_async_smem();
        dm::tc_fence_before();
        __syncthreads();                                   // S consumed, P codes and weights visible

        // ---- the four groups through the one product buffer.  A group's last two 32-column pieces are held in registers
        // while thread 0 issues the next group's products, so those form under the additions instead of after them.
        auto issue_pv = [&](int grp) {   // thread 0 only
            dm::tc_fence_after();
            const uint64_t pd = dm::smem_desc_sw128(dm::smem_u32(s.p)) + 2 * grp;      // 32 bytes of keys per group
#pragma unroll
            for (int dh = 0; dh < 2; ++dh) {
                const uint64_t vd = dm::smem_desc_sw128(dm::smem_u32(s.v[st][dh])) + 256 * grp;   // 32 key rows = 4096 bytes
                dm::umma_e4m3(t_d + 128 * dh, pd, vd, idesc_pv, 0);
            }
            dm::umma_commit(&s.bar_d);
        };
        if (tid == 0) issue_pv(0);
#pragma unroll 1
        for (int grp = 0; grp < 4; ++grp) {
            dm::mbar_wait(&s.bar_d, d_phase & 1, wc);
            ++d_phase;
            dm::tc_fence_after();
            const float w = s.wgt[grp][row];
            const uint32_t src = dm::tmem_addr(t_d, lane_base, g * 128);
            uint32_t sa[32], sb[32];
            auto add32 = [&](int h, const uint32_t* piece) {
#pragma unroll
                for (int i = 0; i < 32; i += 2)
                    dm::fma2(o_acc[h * 32 + i], o_acc[h * 32 + i + 1], __uint_as_float(piece[i]), __uint_as_float(piece[i + 1]), w,
                             o_acc[h * 32 + i], o_acc[h * 32 + i + 1]);
            };
            dm::tmem_ld32(src, sa);
            dm::tmem_ld_wait();
            dm::tmem_ld32(src + 32, sb);
            add32(0, sa);
            dm::tmem_ld_wait();
            dm::tmem_ld32(src + 64, sa);
            add32(1, sb);
            dm::tmem_ld_wait();
            dm::tmem_ld32(src + 96, sb);
            dm::tmem_ld_wait();
            dm::tc_fence_before();
            __syncthreads();                               // every thread holds its last two pieces: the buffer is free
            if (tid == 0 && grp < 3) issue_pv(grp + 1);
            add32(2, sa);
            add32(3, sb);
        }
        if (tid == 0 && it + 2 < n_tiles) load_kv(it + 2);
    }

    // ---- epilogue
    s.lsum[g][row] = l_part;
    __syncthreads();
    const float l = s.lsum[0][row] + s.lsum[1][row];
    const bool dead = (l == 0.f) || (l != l);
    const float inv = dead ? 0.f : 1.0f / l;
    const int n_glob = I * 128 + row;
    __nv_bfloat16* op = p.o + (((int64_t)hc.b * p.N + n_glob) * p.H + hc.h) * 256 + g * 128;
#pragma unroll
    for (int c = 0; c < 16; ++c) {
        uint32_t w4[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            __nv_bfloat162 t = __floats2bfloat162_rn(o_acc[8 * c + 2 * e] * inv, o_acc[8 * c + 2 * e + 1] * inv);
            w4[e] = *reinterpret_cast<uint32_t*>(&t);
        }
        reinterpret_cast<uint4*>(op)[c] = make_uint4(w4[0], w4[1], w4[2], w4[3]);
    }
    if (g == 0) p.lse[(int64_t)hc.bh * p.N + n_glob] = dead ? -INFINITY : m_run + logf(l);
    __syncthreads();
    if (warp == 0) dm::tmem_dealloc(tmem, 512);
}

}  // namespace

namespace dmh {
int prepare_fwd256(char* err, size_t errlen) {
    static DeviceOnce once;
    return device_once(once, err, errlen, [&]() -> int {
        DM_CUDA(cudaFuncSetAttribute(fwd_d256_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Fwd256Smem) + 1024));
        return DM_OK;
    });
}

int launch_fwd_d256(const void* q8, const void* k8, const void* v8, const float* q8s, const float* k8s, const float* v8s, DmShape sh,
                    int h0, int hcount, void* o, float* lse, void* stream, char* err, size_t errlen) {
    int rc;
    CUtensorMap tq, tk, tv;
    if ((rc = make_tmap_u8(&tq, q8, 256, (uint64_t)sh.B * sh.H * sh.N, 128, err, errlen))) return rc;
    if ((rc = make_tmap_u8(&tk, k8, 256, (uint64_t)sh.B * sh.Hk * sh.N, 128, err, errlen))) return rc;
    if ((rc = make_tmap_u8(&tv, v8, 256, (uint64_t)sh.B * sh.Hk * sh.N, 128, err, errlen))) return rc;
    int* status = device_status_word(err, errlen);
    if (!status) return DM_ERR_CUDA;
    Fwd256Params p{q8s, k8s, v8s, static_cast<__nv_bfloat16*>(o), lse, sh.H, sh.Hk, sh.N, h0, hcount, sh.causal, status};
    const int smem = (int)sizeof(Fwd256Smem) + 1024;
    if ((rc = prepare_fwd256(err, errlen))) return rc;
    fwd_d256_kernel<<<dim3(sh.B * hcount, sh.N / 128), 256, smem, static_cast<cudaStream_t>(stream)>>>(tq, tk, tv, p);
    DM_CUDA(cudaGetLastError());
    return DM_OK;
}
}  // namespace dmh
