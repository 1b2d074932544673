// Pass 2 of the backward: dQ = D^-0.5 / 256 * sum over key tiles of psi * (dS'8 K8), one work item per 128-row block so
// the reduction order is fixed and the result deterministic (csrc/fq8_dq_pass2_hd128.h:204-396 of the reference, restated
// for tcgen05).
//
// The dS' tiles were stored by pass 1 as [key][row] (128 x 128 bytes); here they are the A operand read MN-major
// (bytes of a tile row = M = query rows, tile rows = K = keys), and the K8 tile [key][d] is the B operand read MN-major
// too, so no transposed copy of anything exists.  The pass is bound by the dS' read from HBM (16 KB per tile against 4
// MMAs), so the head_dim 128 kernel is built to keep that stream full: one persistent CTA per SM walks the (head, row block)
// items, heaviest first, in three roles that meet only through mbarriers:
//   warp 8       TMA loads: dS' + K8 tiles into a six-stage ring, running ahead across items
//   warp 9       tcgen05.mma: 4 x (M128 N128 K32) per tile, zero-initialised, into one of four tensor-memory buffers
//   warps 0..7   fold: thread (row, 64 d columns) adds psi(row's m-block, tile) * product into its dQ registers unless the
//                tile is a pass-1 zero tile (psi == 0) or sits more than 8 decades below the row block's running psi
//                maximum (the F2 / F2b skip rules); then the item's epilogue (scale, bf16, store)
// With four product buffers the loads and MMAs of the next item run under the current item's last folds and its epilogue.
#include "dm_attn_common.cuh"
#include "dm_host.h"

namespace dmh {
int check_shape(const DmShape& s, int h0, int hcount, char* err, size_t errlen);
}

namespace {

constexpr int kTile = 128 * 128;
constexpr int kStages = 3;        // head_dim 256 kernel
constexpr int kRing = 6;          // head_dim 128 kernel: dS' + K8 stages
constexpr int kAcc = 4;           // head_dim 128 kernel: product buffers in tensor memory
constexpr int kFoldThreads = 256;
constexpr int kThreads128 = kFoldThreads + 64;

struct Bwd2Smem {
    alignas(1024) uint8_t a[kRing][kTile];   // dS' tile [key][row]
    alignas(1024) uint8_t b[kRing][kTile];   // K8 tile [key][d]
    alignas(16) uint8_t stg[128 * 256];       // an item's bf16 dQ rows on their way out (16-byte chunks XOR-swizzled by the row)
    uint64_t bar_ld[kRing], bar_free[kRing], bar_acc[kAcc], bar_acc_free[kAcc];
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
    int n_heads;                  // batch * hcount
    dm::FastDiv fd_heads, fd_hcount, fd_rep;   // divisions by n_heads, hcount and H / Hk
};

// One work item = one local 128-row block of one (batch, head); numbered rank-major (rank 0 = the row blocks with the most key
// tiles, all heads, then rank 1, ...) and walked in a snake over the rounds, as in the forward.
struct Bwd2Item {
    dm::HeadCoord hc;
    int rb, n_it, bhl;
    bool valid;
};
__device__ __forceinline__ Bwd2Item bwd2_item(const Bwd2Params& p, int round) {
    Bwd2Item w;
    const int G = gridDim.x, c = blockIdx.x;
    const int nq_blk = p.rm.nq / 128;
    const int idx = round * G + ((round & 1) ? G - 1 - c : c);
    w.valid = idx < p.n_heads * nq_blk;
    const int rank = (int)dm::fdiv((uint32_t)idx, p.fd_heads);
    w.hc = dm::head_coord(idx - rank * p.n_heads, p.h0, p.fd_hcount, p.H, p.Hk, p.fd_rep);
    w.bhl = w.hc.b * p.hcount + (w.hc.h - p.h0);
    w.rb = nq_blk - 1 - rank;
    w.n_it = p.causal ? dm::global_block(p.rm, w.rb) + 1 : p.N / 128;
    return w;
}

__global__ void __launch_bounds__(kThreads128, 1)
bwd2_d128_kernel(const __grid_constant__ CUtensorMap tm_ds, const __grid_constant__ CUtensorMap tm_k, const Bwd2Params p) {
    extern __shared__ uint8_t smem_raw[];
    Bwd2Smem& s = *reinterpret_cast<Bwd2Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nbn = p.N / 128;
    const int nq_blk = p.rm.nq / 128, nbm_l = p.rm.nq / 64;
    dm::WaitCtx wc{&s.abort_flag, p.status};

    if (tid == 0) {
        s.abort_flag = 0;
        for (int i = 0; i < kRing; ++i) {
            dm::mbar_init(&s.bar_ld[i], 1);
            dm::mbar_init(&s.bar_free[i], 1);
        }
        for (int i = 0; i < kAcc; ++i) {
            dm::mbar_init(&s.bar_acc[i], 1);
            dm::mbar_init(&s.bar_acc_free[i], kFoldThreads / 32);
        }
        dm::fence_mbar_init();
        dm::tma_prefetch_desc(&tm_ds);
        dm::tma_prefetch_desc(&tm_k);
    }
    if (warp == 0) dm::tmem_alloc(&s.tmem_base, 512);
    dm::tc_fence_before();
    __syncthreads();
    dm::tc_fence_after();
    const uint32_t tmem = s.tmem_base;
    // Every role walks the same item list; `gt` counts the key tiles of the items before the current one, so ring stages,
    // buffer indices and mbarrier phases run on across items (t = gt + it).

    if (warp == 8) {
        // ---- TMA loads
        const bool leader = lane == 0;
        int gt = 0;
        for (int r = 0;; ++r) {
            const Bwd2Item w = bwd2_item(p, r);
            if (!w.valid) break;
            const int64_t tile0 = ((int64_t)w.bhl * nq_blk + w.rb) * nbn;   // dS' tile index of (local row block rb, key block 0)
            const int kv_row0 = w.hc.bhk * p.N;
            for (int it = 0; it < w.n_it; ++it) {
                const int t = gt + it, st = t % kRing;
                if (t >= kRing) dm::mbar_wait(&s.bar_free[st], (t / kRing - 1) & 1, wc);
                if (leader) {
                    dm::mbar_expect_tx(&s.bar_ld[st], 2 * kTile);
                    dm::tma_load_2d(s.a[st], &tm_ds, 0, (int)((tile0 + it) * 128), &s.bar_ld[st]);
                    dm::tma_load_2d(s.b[st], &tm_k, 0, kv_row0 + it * 128, &s.bar_ld[st]);
                }
                __syncwarp();
            }
            gt += w.n_it;
        }
    } else if (warp == 9) {
        // ---- MMA issue: both operands MN-major, one K step = 32 tile rows = 4096 bytes
        const bool leader = lane == 0;
        constexpr uint32_t idesc = dm::idesc_e4m3(128, 128, true, true);
        constexpr uint32_t kSub = kTile >> 4;
        const uint32_t a_lo = dm::smem_desc_lo_sw128(dm::smem_u32(s.a[0])), b_lo = dm::smem_desc_lo_sw128(dm::smem_u32(s.b[0]));
        int gt = 0;
        for (int r = 0;; ++r) {
            const Bwd2Item w = bwd2_item(p, r);
            if (!w.valid) break;
            for (int it = 0; it < w.n_it; ++it) {
                const int t = gt + it, st = t % kRing, b = t % kAcc;
                dm::mbar_wait(&s.bar_ld[st], (t / kRing) & 1, wc);
                if (t >= kAcc) dm::mbar_wait(&s.bar_acc_free[b], (t / kAcc - 1) & 1, wc);
                dm::tc_fence_after();
                const uint32_t aa = a_lo + st * kSub, ba = b_lo + st * kSub, d = tmem + b * 128;
                if (leader) {
                    dm::umma_e4m3_lo<false>(d, aa, ba, idesc);
#pragma unroll
                    for (int k = 1; k < 4; ++k) dm::umma_e4m3_lo<true>(d, aa + 256 * k, ba + 256 * k, idesc);
                    dm::umma_commit(&s.bar_acc[b]);
                    dm::umma_commit(&s.bar_free[st]);
                }
                __syncwarp();
            }
            gt += w.n_it;
        }
    } else {
        // ---- fold warps: thread = (row, 64 d columns)
        const int g = warp >> 2;
        const int row = (warp & 3) * 32 + lane;
        const uint32_t lane_base = (uint32_t)(warp & 3) * 32;
        int gt = 0;
        for (int r = 0;; ++r) {
            const Bwd2Item w = bwd2_item(p, r);
            if (!w.valid) break;
            const int mb = 2 * w.rb + (row >> 6);
            const float* psi_row = p.psi + ((int64_t)w.bhl * nbm_l + mb) * nbn;
            float psi_max = 0.f;
            float dq[64];
#pragma unroll
            for (int i = 0; i < 64; ++i) dq[i] = 0.f;
            // psi is read two tiles ahead: a new 32-byte sector of the row comes from DRAM every eighth tile
            float psi_n1 = psi_row[0], psi_n2 = w.n_it > 1 ? psi_row[1] : 0.f;
            for (int it = 0; it < w.n_it; ++it) {
                const int t = gt + it, b = t % kAcc;
                const float psi_cur = psi_n1;
                psi_n1 = psi_n2;
                if (it + 2 < w.n_it) psi_n2 = psi_row[it + 2];
                const bool take = (psi_cur != 0.f) && !(psi_cur < psi_max * 1e-8f);
                dm::mbar_wait(&s.bar_acc[b], (t / kAcc) & 1, wc);
                dm::tc_fence_after();
                if (take) {                                                // warp-uniform: a warp's 32 rows share one m-block
                    uint32_t ta[32], tb[32];
                    const uint32_t src = dm::tmem_addr(tmem + b * 128, lane_base, g * 64);
                    dm::tmem_ld32(src, ta);
                    dm::tmem_ld32(src + 32, tb);
                    dm::tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) dq[i] = fmaf(__uint_as_float(ta[i]), psi_cur, dq[i]);
#pragma unroll
                    for (int i = 0; i < 32; ++i) dq[32 + i] = fmaf(__uint_as_float(tb[i]), psi_cur, dq[32 + i]);
                    psi_max = fmaxf(psi_max, psi_cur);
                }
                dm::tc_fence_before();
                dm::mbar_arrive_warp(&s.bar_acc_free[b]);
            }
            gt += w.n_it;
            // The bf16 rows leave through shared memory: a thread holds half a row, so stored directly every 16-byte store
            // instruction would touch 32 different rows; from the staging tile each instruction writes two whole 256-byte rows.
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                uint32_t w4[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    __nv_bfloat162 tt = __floats2bfloat162_rn(dq[8 * c + 2 * e] * p.final_scale, dq[8 * c + 2 * e + 1] * p.final_scale);
                    w4[e] = *reinterpret_cast<uint32_t*>(&tt);
                }
                *reinterpret_cast<uint4*>(s.stg + row * 256 + (((g * 8 + c) ^ (row & 7)) << 4)) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
            }
            dm::named_bar_sync(1, kFoldThreads);
            {
                uint8_t* obase = reinterpret_cast<uint8_t*>(p.dq + (((int64_t)w.hc.b * p.rm.nq + w.rb * 128) * p.H + w.hc.h) * 128);
                const int64_t row_bytes = (int64_t)p.H * 128 * 2;
                const int j = lane & 15;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int rr = 2 * (warp * 8 + i) + (lane >> 4);
                    const uint4 val = *reinterpret_cast<const uint4*>(s.stg + rr * 256 + ((j ^ (rr & 7)) << 4));
                    *reinterpret_cast<uint4*>(obase + rr * row_bytes + (j << 4)) = val;
                }
            }
            dm::named_bar_sync(1, kFoldThreads);           // the staging tile may take the next item's rows
        }
    }
    dm::tc_fence_before();
    __syncthreads();
    if (warp == 0) dm::tmem_dealloc(tmem, 512);
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
                 dm::RowMap{cp.nq, cp.half_blocks, cp.off0, cp.off1}, sh.B * hcount, dm::make_fastdiv(sh.B * hcount), dm::make_fastdiv(hcount),
                 dm::make_fastdiv(sh.H / sh.Hk)};
    if (sh.D == 256) {
        const int smem = (int)sizeof(Bwd2Smem256) + 1024;
        bwd2_d256_kernel<<<dim3(sh.B * hcount, sh.N / 128), 256, smem, static_cast<cudaStream_t>(stream)>>>(ts, tk, p);
        DM_CUDA(cudaGetLastError());
        return DM_OK;
    }
    const int smem = (int)sizeof(Bwd2Smem) + 1024;
    int sms = 0;
    if ((rc = dmh::sm_count(&sms, err, errlen))) return rc;
    const int64_t items = (int64_t)sh.B * hcount * (cp.nq / 128);
    const int grid = (int)(items < sms ? items : sms);
    bwd2_d128_kernel<<<grid, kThreads128, smem, static_cast<cudaStream_t>(stream)>>>(ts, tk, p);
    DM_CUDA(cudaGetLastError());
    return DM_OK;
}
