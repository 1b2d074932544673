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

// ------------------------------------------------------------------------------------------------------------------------------
// The production kernel at head_dim 128: the same sums as delta_kernel<false, 128>, as a persistent kernel in roles.
// One CTA per SM walks the (head, row block) items, heaviest first; 640 threads:
//   warps 0..15  compute, four per scheduler, in two teams of eight: team 0 takes the even key tiles and team 1 the odd ones
//                (counted over the CTA's whole walk), so the two teams are half a tile apart in time and one team's waits
//                and tensor-memory loads run under the other team's exponentials.  Thread (row, 64-key group g) does
//                what a thread of delta_kernel does: per 32-key half, P-hat and a = fma(P-hat, dP * (do8sc v8sc), a) in
//                ascending key order, then acc_fp64 += a * 2^-8
//   warp 16      TMA loads: Q8 / dO8 of an item (double-buffered by item), K8 / V8 tiles in a three-stage ring
//   warp 17      tcgen05.mma: S = Q K^T and dP = dO V^T of a tile (8 x M128 N128 K32) into one of two (S | dP) buffers
// A row's four fp64 sums (team x group) meet in shared memory at the item's end: every warp leaves its sums and arrives on
// an mbarrier, and only the four warps that add them up and store the result (team 0, group 0) wait for it; the buffers
// rotate over four items (the teams are never more than two tiles apart, because the MMAs are issued in tile order).  An
// item's row constants and first scales are read one item ahead.
constexpr int kDzComputeWarps = 16;
constexpr int kDzThreads = 32 * kDzComputeWarps + 64;
constexpr int kDzStages = 3;

struct DeltaRolesSmem {
    alignas(1024) uint8_t q[2][kTile];
    alignas(1024) uint8_t dO[2][kTile];
    alignas(1024) uint8_t k[kDzStages][kTile];
    alignas(1024) uint8_t v[kDzStages][kTile];
    double part[4][4][128];          // [item % 4][2 * team + group][row]
    uint64_t bar_qdo[2], bar_qdo_free[2], bar_kv[kDzStages], bar_kv_free[kDzStages], bar_sp[2], bar_part[4];
    uint32_t tmem_base;
    int abort_flag;
};

struct DeltaItem {
    dm::HeadCoord hc;
    int li, I, n_tiles;
    bool valid;
};
struct DeltaDivs {
    dm::FastDiv heads, hcount, rep;   // divisions by batch * hcount, hcount and H / Hk
};
__device__ __forceinline__ DeltaItem delta_item(const DeltaParams& p, const DeltaDivs& fd, int round) {
    DeltaItem w;
    const int G = gridDim.x, c = blockIdx.x;
    const int nq_blk = p.rm.nq / 128, n_heads = (int)fd.heads.d;
    const int idx = round * G + ((round & 1) ? G - 1 - c : c);
    w.valid = idx < n_heads * nq_blk;
    const int rank = (int)dm::fdiv((uint32_t)idx, fd.heads);
    w.hc = dm::head_coord(idx - rank * n_heads, p.h0, fd.hcount, p.H, p.Hk, fd.rep);
    w.li = nq_blk - 1 - rank;
    w.I = dm::global_block(p.rm, w.li);
    w.n_tiles = p.causal ? w.I + 1 : p.N / 128;
    return w;
}

__global__ void __launch_bounds__(kDzThreads, 1)
delta_roles_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                   const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, const DeltaParams p,
                   const DeltaDivs fd) {
    extern __shared__ uint8_t smem_raw[];
    DeltaRolesSmem& s = *reinterpret_cast<DeltaRolesSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nq_blk = p.rm.nq / 128;
    dm::WaitCtx wc{&s.abort_flag, p.status};

    if (tid == 0) {
        s.abort_flag = 0;
        for (int i = 0; i < 2; ++i) {
            dm::mbar_init(&s.bar_qdo[i], 1);
            dm::mbar_init(&s.bar_qdo_free[i], 1);
            dm::mbar_init(&s.bar_sp[i], 1);
        }
        for (int i = 0; i < kDzStages; ++i) {
            dm::mbar_init(&s.bar_kv[i], 1);
            dm::mbar_init(&s.bar_kv_free[i], 1);
        }
        for (int i = 0; i < 4; ++i) dm::mbar_init(&s.bar_part[i], kDzComputeWarps);
        dm::fence_mbar_init();
        dm::tma_prefetch_desc(&tm_q);
        dm::tma_prefetch_desc(&tm_do);
        dm::tma_prefetch_desc(&tm_k);
        dm::tma_prefetch_desc(&tm_v);
    }
    if (warp == 0) dm::tmem_alloc(&s.tmem_base, 512);
    dm::tc_fence_before();
    __syncthreads();
    dm::tc_fence_after();
    const uint32_t tmem = s.tmem_base;
    constexpr uint32_t kSub = kTile >> 4;
    // `gt` counts the key tiles of the items before the current one: ring stages, buffers and phases run on across items

    if (warp == kDzComputeWarps) {
        // ---- TMA loads
        const bool leader = lane == 0;
        int gt = 0;
        for (int r = 0;; ++r) {
            const DeltaItem w = delta_item(p, fd, r);
            if (!w.valid) break;
            const int qb = r & 1;
            const int q_row0 = w.hc.bh * p.rm.nq + w.li * 128, kv_row0 = w.hc.bhk * p.N;
            if (r >= 2) dm::mbar_wait(&s.bar_qdo_free[qb], ((r - 2) >> 1) & 1, wc);
            if (leader) {
                dm::mbar_expect_tx(&s.bar_qdo[qb], 2 * kTile);
                dm::tma_load_2d(s.q[qb], &tm_q, 0, q_row0, &s.bar_qdo[qb]);
                dm::tma_load_2d(s.dO[qb], &tm_do, 0, q_row0, &s.bar_qdo[qb]);
            }
            for (int it = 0; it < w.n_tiles; ++it) {
                const int t = gt + it, st = t % kDzStages;
                if (t >= kDzStages) dm::mbar_wait(&s.bar_kv_free[st], (t / kDzStages - 1) & 1, wc);
                if (leader) {
                    dm::mbar_expect_tx(&s.bar_kv[st], 2 * kTile);
                    dm::tma_load_2d(s.k[st], &tm_k, 0, kv_row0 + it * 128, &s.bar_kv[st]);
                    dm::tma_load_2d(s.v[st], &tm_v, 0, kv_row0 + it * 128, &s.bar_kv[st]);
                }
                __syncwarp();
            }
            gt += w.n_tiles;
        }
    } else if (warp == kDzComputeWarps + 1) {
        // ---- MMA issue
        const bool leader = lane == 0;
        constexpr uint32_t idesc = dm::idesc_e4m3(128, 128, false, false);
        const uint32_t q_lo0 = dm::smem_desc_lo_sw128(dm::smem_u32(s.q[0])), do_lo0 = dm::smem_desc_lo_sw128(dm::smem_u32(s.dO[0]));
        const uint32_t k_lo = dm::smem_desc_lo_sw128(dm::smem_u32(s.k[0])), v_lo = dm::smem_desc_lo_sw128(dm::smem_u32(s.v[0]));
        int gt = 0;
        for (int r = 0;; ++r) {
            const DeltaItem w = delta_item(p, fd, r);
            if (!w.valid) break;
            const int qb = r & 1;
            dm::mbar_wait(&s.bar_qdo[qb], (r >> 1) & 1, wc);
            const uint32_t q_lo = q_lo0 + qb * kSub, do_lo = do_lo0 + qb * kSub;
            for (int it = 0; it < w.n_tiles; ++it) {
                const int t = gt + it, st = t % kDzStages, b = t & 1;
                dm::mbar_wait(&s.bar_kv[st], (t / kDzStages) & 1, wc);
                // a team says through a named barrier that it holds its buffer's values: a hand-off between warps costs a fifth
                // of what an mbarrier's does
                if (t >= 2) dm::named_bar_sync(2 + b, 16 * kDzComputeWarps + 32);
                dm::tc_fence_after();
                const uint32_t ks = k_lo + st * kSub, vs = v_lo + st * kSub, t_s = tmem + b * 256, t_dp = t_s + 128;
                if (leader) {
                    dm::umma_e4m3_lo<false>(t_s, q_lo, ks, idesc);
#pragma unroll
                    for (int k = 1; k < 4; ++k) dm::umma_e4m3_lo<true>(t_s, q_lo + 2 * k, ks + 2 * k, idesc);
                    dm::umma_e4m3_lo<false>(t_dp, do_lo, vs, idesc);
#pragma unroll
                    for (int k = 1; k < 4; ++k) dm::umma_e4m3_lo<true>(t_dp, do_lo + 2 * k, vs + 2 * k, idesc);
                    dm::umma_commit(&s.bar_sp[b]);
                    dm::umma_commit(&s.bar_kv_free[st]);
                    if (it == w.n_tiles - 1) dm::umma_commit(&s.bar_qdo_free[qb]);
                }
                __syncwarp();
            }
            gt += w.n_tiles;
        }
    } else if (warp < kDzComputeWarps) {
        // ---- compute warps: thread = (row, 64-key group g), team = parity of the tiles it takes (= the (S | dP) buffer)
        const int team = warp >> 3, g = (warp >> 2) & 1;
        const int row = (warp & 3) * 32 + lane;
        const uint32_t lane_base = (uint32_t)(warp & 3) * 32;
        const uint32_t t_s = dm::tmem_addr(tmem + team * 256, lane_base, g * 64), t_dp = t_s + 128;
        int gt = 0;
        // what the item's first tile needs from global memory is read one item ahead
        int64_t rowi_nx = 0;
        float q8sc_nx = 0.f, do8sc_nx = 0.f, lse_nx = 0.f, ks_nx = 0.f, vs_nx = 0.f;
        auto prefetch = [&](const DeltaItem& wi, int gt_at) {
            if (!wi.valid) return;
            rowi_nx = (int64_t)wi.hc.bh * p.rm.nq + wi.li * 128 + row;
            q8sc_nx = p.q8s[(int64_t)wi.hc.bh * nq_blk + wi.li];
            do8sc_nx = p.do8s[(int64_t)wi.hc.bh * nq_blk + wi.li];
            lse_nx = p.lse[rowi_nx];
            const int first = (gt_at ^ team) & 1;
            if (first < wi.n_tiles) {
                const int64_t so = (int64_t)wi.hc.bhk * (p.N / 64) + g + 2 * first;
                ks_nx = p.k8s[so];
                vs_nx = p.v8s[so];
            }
        };
        DeltaItem w = delta_item(p, fd, 0);
        prefetch(w, 0);
        for (int r = 0; w.valid; ++r) {
            const int n_tiles = w.n_tiles, I = w.I;
            const int64_t rowi = rowi_nx;
            const float q8sc = q8sc_nx, do8sc = do8sc_nx;
            const float rc = dm::phat_row_const(lse_nx);
            const float* ksp = p.k8s + (int64_t)w.hc.bhk * (p.N / 64) + g;
            const float* vsp = p.v8s + (int64_t)w.hc.bhk * (p.N / 64) + g;
            double acc = 0.0;
            const int it0 = (gt ^ team) & 1;                   // this team's first tile of the item
            float ks_n = ks_nx, vs_n = vs_nx;
            const DeltaItem w_next = delta_item(p, fd, r + 1);
            prefetch(w_next, gt + n_tiles);
            for (int it = it0; it < n_tiles; it += 2) {
                const int t = gt + it;
                const float dsc = dm::descale_log2(q8sc, ks_n), dpsc = do8sc * vs_n;
                if (it + 2 < n_tiles) {
                    ks_n = ksp[2 * (it + 2)];
                    vs_n = vsp[2 * (it + 2)];
                }
                const bool diag = p.causal && it == I;
                dm::mbar_wait(&s.bar_sp[team], (t >> 1) & 1, wc);
                dm::tc_fence_after();
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    float sv[32], dp[32];
                    dm::tmem_ld32(t_s + half * 32, reinterpret_cast<uint32_t*>(sv));
                    dm::tmem_ld32(t_dp + half * 32, reinterpret_cast<uint32_t*>(dp));
                    dm::tmem_ld_wait();
                    if (half == 1) {
                        dm::tc_fence_before();
                        dm::named_bar_arrive(2 + team, 16 * kDzComputeWarps + 32);     // the team's buffer may be overwritten
                    }
#pragma unroll
                    for (int c = 0; c < 32; c += 2) {           // P-hat = 2^min(S dsc + rc, 12), the exponent two at a time
                        dm::fma2(sv[c], sv[c + 1], sv[c], sv[c + 1], dsc, rc, rc);
                        sv[c] = dm::ex2(fminf(sv[c], dm::kMoE + 4.0f));
                        sv[c + 1] = dm::ex2(fminf(sv[c + 1], dm::kMoE + 4.0f));
                    }
                    if (diag) {                                 // the diagonal tile only: keys above the row
#pragma unroll
                        for (int c = 0; c < 32; ++c)
                            if (g * 64 + half * 32 + c > row) sv[c] = 0.f;
                    }
                    float a = 0.f;
#pragma unroll
                    for (int c = 0; c < 32; c += 2) {
                        float d0, d1;
                        dm::mul2(d0, d1, dp[c], dp[c + 1], dpsc, dpsc);
                        a = fmaf(sv[c], d0, a);
                        a = fmaf(sv[c + 1], d1, a);
                    }
                    acc += (double)(a * dm::kMoInv);
                }
            }
            gt += n_tiles;
            // the row's four sums meet in shared memory; only the four storing warps wait for the others
            const int pb = r & 3;
            s.part[pb][2 * team + g][row] = acc;
            dm::mbar_arrive_warp(&s.bar_part[pb]);             // (lane 0 arrives after __syncwarp: the warp's stores are ordered before it)
            if (warp < 4) {
                dm::mbar_wait(&s.bar_part[pb], (r >> 2) & 1, wc);
                p.out[rowi] = (float)((s.part[pb][0][row] + s.part[pb][1][row]) + (s.part[pb][2][row] + s.part[pb][3][row]));
            }
            w = w_next;
        }
    }
    dm::tc_fence_before();
    __syncthreads();
    if (warp == 0) dm::tmem_dealloc(tmem, 512);
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
    // head_dim 128, production: the persistent kernel once every CTA has a walk of at least 24 key tiles (measured: it wins at
    // 29 tiles per CTA, 0.041 against 0.044 ms, and by more on longer walks); the one-item-per-CTA kernel below stays for small problems, the debug row sums and head_dim 256
    const int64_t items = (int64_t)sh.B * p.hcount * (p.rm.nq / 128);
    const int64_t tiles = items * (sh.causal ? (sh.N / 128 + 1) / 2 : sh.N / 128);      // about: exact for the identity row map
    int sms = 0;
    if ((rc = dmh::sm_count(&sms, err, errlen))) return rc;
    if (!kDebug && kD == 128 && items >= 2 * (int64_t)sms && tiles >= 24 * (int64_t)sms) {
        const DeltaDivs fd{dm::make_fastdiv(sh.B * p.hcount), dm::make_fastdiv(p.hcount), dm::make_fastdiv(sh.H / sh.Hk)};
        delta_roles_kernel<<<sms, kDzThreads, (int)sizeof(DeltaRolesSmem) + 1024, static_cast<cudaStream_t>(stream)>>>(tq, td, tk, tv, p, fd);
        DM_CUDA(cudaGetLastError());
        return DM_OK;
    }
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
        DM_CUDA(cudaFuncSetAttribute(delta_roles_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(DeltaRolesSmem) + 1024));
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
