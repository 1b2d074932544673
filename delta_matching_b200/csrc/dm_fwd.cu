// Forward kernel, head_dim 128: O and LSE from e4m3 Q / K / V codes and their block scales, with the reference's
// faithful P basis (per row, per 64-key group) -- csrc/softmax_fq8f.h and csrc/mainloop_fwd_sm90_fp8f.hpp of the
// reference, restated for tcgen05.
//
// One CTA = 128 query rows of one (batch, head).  512 threads in four roles:
//   warps 0..7   softmax: thread (quarter q, lane, warpgroup g) owns row 32q+lane and key group g of every key tile
//   warps 8..11  fold: thread = row; they own O (128 fp32 columns per thread) and nothing else
//   warps 12..14 service (one issuing lane each, loops converged): 12 issues S, 13 issues the P V products, 14 the TMA loads
// Key tiles of 128 keys (two 64-key groups) are visited from the diagonal tile downwards.  Per tile:
//   S = Q K^T            4 x tcgen05.mma (M128 N128 K32) into one of two tensor-memory buffers, up to two tiles ahead
//   softmax              group max, running max exchanged through shared memory, basis
//                        ms_g = max(gm_g*l2, m*l2 - 12) - log2(448), codes = e4m3(2^(S*l2 - ms_g)) written back into tensor
//                        memory over the scores they came from (four codes per column, lane = row); the denominator is
//                        summed from the unrounded p; the tile's alpha and the two weights w_g = v8sc_g * 2^(ms_g - m*l2)
//                        per row go to a small ring for the fold warps
//   D_g = C_g V_g        2 x tcgen05.mma per group (A = the codes in tensor memory, B = the V tile) into zero-initialised
//                        tensor-memory temporaries, issued when the codes are stored and the previous products have been read
//   O = O * alpha + D_0 w_0 + D_1 w_1   by the fold warps, in that order, while the softmax warps are on the next tile
// K / V tiles arrive by TMA into a 3-stage ring.  The kernel is persistent: one CTA per SM walks a list of (head, row
// block) items, and since every role keeps its own place in the list, the loads and S of the next item start while the
// softmax and fold warps finish the current one.  Every mbarrier wait is bounded.
#include "dm_attn_common.cuh"
#include "dm_host.h"

namespace {

constexpr int kTile = 128 * 128;   // bytes of one e4m3 tile (128 rows x 128 bytes)
constexpr int kStages = 3;
constexpr int kThreads = 512;
constexpr int kSoftmaxThreads = 256;
constexpr int kRing = 4;           // depth of the per-tile row-constant ring between softmax and fold warps

struct FwdSmem {
    alignas(1024) uint8_t q[2][kTile];             // by work item parity: the next item's Q arrives under this item's tail
    alignas(1024) uint8_t k[kStages][kTile];
    alignas(1024) uint8_t v[kStages][kTile];
    float gmax[2][2][128];            // [tile parity][key group][row]
    float wgt[kRing][2][128];         // [tile % kRing][key group][row]
    float alpha[kRing][128];
    float lsum[4][2][128];            // [work item % 4][key group][row]: with one-tile items the softmax warps can be three
                                      // items ahead of the fold warps
    alignas(16) uint8_t stg[4][32 * 256];   // per fold warp: its 32 bf16 O rows on their way out (16-byte chunks XOR-swizzled by the row)
    uint64_t bar_q[2], bar_q_free[2], bar_kv[kStages], bar_kv_free[kStages], bar_s_full[2], bar_s_free[2], bar_codes[2],
        bar_d_full[2], bar_d_free, bar_l[4];
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
    int n_heads;                      // B * hcount: work items are (head, row block), heaviest row blocks first
    dm::FastDiv fd_heads, fd_hcount, fd_rep;   // divisions by n_heads, hcount and H / Hk
};

// One work item of a persistent CTA.  Items are numbered rank-major (rank 0 = the row blocks with the most key tiles, all
// heads, then rank 1, ...); CTA c of G takes item r G + c in even rounds r and r G + (G - 1 - c) in odd rounds, so a CTA that
// got a long item in one round gets a short one in the next.
struct FwdItem {
    dm::HeadCoord hc;
    int li, I, n_tiles;
    bool valid;
};
__device__ __forceinline__ FwdItem fwd_item(const FwdParams& p, int round) {
    FwdItem w;
    const int G = gridDim.x, c = blockIdx.x;
    const int nq_blk = p.rm.nq / 128;
    const int idx = round * G + ((round & 1) ? G - 1 - c : c);
    w.valid = idx < p.n_heads * nq_blk;
    const int rank = (int)dm::fdiv((uint32_t)idx, p.fd_heads);
    w.hc = dm::head_coord(idx - rank * p.n_heads, p.h0, p.fd_hcount, p.H, p.Hk, p.fd_rep);
    w.li = nq_blk - 1 - rank;
    w.I = dm::global_block(p.rm, w.li);
    w.n_tiles = p.causal ? w.I + 1 : p.N / 128;
    return w;
}

__global__ void __launch_bounds__(kThreads, 1)
fwd_d128_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const FwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    FwdSmem& s = *reinterpret_cast<FwdSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nq_blk = p.rm.nq / 128;
    dm::WaitCtx wc{&s.abort_flag, p.status};
    // Every role walks the same list of work items; `gt` counts the key tiles of the items before the current one, so
    // that ring stages, buffer parities and mbarrier phases run on across items (t = gt + it below).

    if (tid == 0) {
        s.abort_flag = 0;
        for (int i = 0; i < kStages; ++i) {
            dm::mbar_init(&s.bar_kv[i], 1);
            dm::mbar_init(&s.bar_kv_free[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            dm::mbar_init(&s.bar_s_full[i], 1);
            dm::mbar_init(&s.bar_s_free[i], 8);
            dm::mbar_init(&s.bar_codes[i], 8);
            dm::mbar_init(&s.bar_d_full[i], 1);
            dm::mbar_init(&s.bar_q[i], 1);
            dm::mbar_init(&s.bar_q_free[i], 1);
        }
        dm::mbar_init(&s.bar_d_free, 4);
        for (int i = 0; i < 4; ++i) dm::mbar_init(&s.bar_l[i], 8);
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
    const uint32_t t_d0 = tmem + 256, t_d1 = tmem + 384;      // S buffers at columns [0, 128) and [128, 256)
    const uint32_t lane_base = (uint32_t)(warp & 3) * 32;

    if (warp >= 12) {
        // =============================================================== service warps
        dm::reg_dec<40>();
        const bool leader = lane == 0;
        constexpr uint32_t kSub = kTile >> 4;
        if (warp == 12) {
            // ---- S = Q K^T of tile t into buffer t & 1.  The code tile of the same parity is rewritten by the softmax of
            // this tile, so the products of tile t - 2, which read it, must be complete: waiting for them here gates the
            // softmax warps through S.
            constexpr uint32_t idesc_s = dm::idesc_e4m3(128, 128, false, false);
            const uint32_t q_lo0 = dm::smem_desc_lo_sw128(dm::smem_u32(s.q[0])), k_lo = dm::smem_desc_lo_sw128(dm::smem_u32(s.k[0]));
            int gt = 0;
            for (int r = 0;; ++r) {
                const FwdItem w = fwd_item(p, r);
                if (!w.valid) break;
                const int qb = r & 1;
                const uint32_t q_lo = q_lo0 + qb * kSub;
                dm::mbar_wait(&s.bar_q[qb], (r >> 1) & 1, wc);
                for (int it = 0; it < w.n_tiles; ++it) {
                    const int t = gt + it, st = t % kStages, b = t & 1;
                    dm::mbar_wait(&s.bar_kv[st], (t / kStages) & 1, wc);
                    if (t >= 2) {
                        dm::mbar_wait(&s.bar_s_free[b], ((t - 2) >> 1) & 1, wc);
                        dm::mbar_wait(&s.bar_d_full[b], ((t - 2) >> 1) & 1, wc);
                    }
                    dm::tc_fence_after();
                    const uint32_t ks = k_lo + st * kSub, ts = tmem + b * 128;
                    if (leader) {
                        dm::umma_e4m3_lo<false>(ts, q_lo, ks, idesc_s);
#pragma unroll
                        for (int k = 1; k < 4; ++k) dm::umma_e4m3_lo<true>(ts, q_lo + 2 * k, ks + 2 * k, idesc_s);
                        dm::umma_commit(&s.bar_s_full[b]);
                        if (it == w.n_tiles - 1) dm::umma_commit(&s.bar_q_free[qb]);   // the item's Q tile has been read
                    }
                    __syncwarp();
                }
                gt += w.n_tiles;
            }
        } else if (warp == 13) {
            // ---- D_g = C_g V_g for both key groups once the codes of tile t are in shared memory and the fold warps
            // have read the products of tile t - 1
            constexpr uint32_t idesc_pv = dm::idesc_e4m3(128, 128, false, true);
            const uint32_t v_lo = dm::smem_desc_lo_sw128(dm::smem_u32(s.v[0]));
            int gt = 0;
            for (int r = 0;; ++r) {
                const FwdItem w = fwd_item(p, r);
                if (!w.valid) break;
                for (int it = 0; it < w.n_tiles; ++it) {
                    const int t = gt + it, st = t % kStages, b = t & 1;
                    dm::mbar_wait(&s.bar_kv[st], (t / kStages) & 1, wc);
                    dm::mbar_wait(&s.bar_codes[b], (t >> 1) & 1, wc);
                    if (t >= 1) dm::mbar_wait(&s.bar_d_free, (t - 1) & 1, wc);
                    dm::tc_fence_after();
                    const uint32_t pa = tmem + b * 128, va = v_lo + st * kSub;     // codes of group g: columns [64 g, 64 g + 16) of S buffer b
                    if (leader) {
                        // group gg: codes columns [64 gg, 64 gg + 64) (K-major, +4 per 64 bytes), V rows [64 gg, +64) (MN-major, +512)
                        dm::umma_e4m3_ts<false>(t_d0, pa, va, idesc_pv);
                        dm::umma_e4m3_ts<true>(t_d0, pa + 8, va + 256, idesc_pv);
                        dm::umma_e4m3_ts<false>(t_d1, pa + 64, va + 512, idesc_pv);
                        dm::umma_e4m3_ts<true>(t_d1, pa + 72, va + 768, idesc_pv);
                        dm::umma_commit(&s.bar_d_full[b]);
                        dm::umma_commit(&s.bar_kv_free[st]);       // K was read by S long ago, V just now
                    }
                    __syncwarp();
                }
                gt += w.n_tiles;
            }
        } else if (warp == 14) {
            // ---- TMA loads: every item's Q, then its K / V tiles, as far ahead as the rings allow (across items too)
            int gt = 0;
            for (int r = 0;; ++r) {
                const FwdItem w = fwd_item(p, r);
                if (!w.valid) break;
                const int qb = r & 1;
                const int q_row0 = w.hc.bh * p.rm.nq + w.li * 128, kv_row0 = w.hc.bhk * p.N;
                if (r >= 2) dm::mbar_wait(&s.bar_q_free[qb], ((r - 2) >> 1) & 1, wc);
                if (leader) {
                    dm::mbar_expect_tx(&s.bar_q[qb], kTile);
                    dm::tma_load_2d(s.q[qb], &tm_q, 0, q_row0, &s.bar_q[qb]);
                }
                for (int it = 0; it < w.n_tiles; ++it) {
                    const int t = gt + it, st = t % kStages, j = w.n_tiles - 1 - it;
                    if (t >= kStages) dm::mbar_wait(&s.bar_kv_free[st], (t / kStages - 1) & 1, wc);
                    if (leader) {
                        dm::mbar_expect_tx(&s.bar_kv[st], 2 * kTile);
                        dm::tma_load_2d(s.k[st], &tm_k, 0, kv_row0 + j * 128, &s.bar_kv[st]);
                        dm::tma_load_2d(s.v[st], &tm_v, 0, kv_row0 + j * 128, &s.bar_kv[st]);
                    }
                    __syncwarp();
                }
                gt += w.n_tiles;
            }
        }
    } else if (warp >= 8) {
        // =============================================================== fold warps: thread = row, all 128 columns of O
        dm::reg_inc<208>();
        const int row = (warp & 3) * 32 + lane;
        int gt = 0;
        for (int r = 0;; ++r) {
            const FwdItem w = fwd_item(p, r);
            if (!w.valid) break;
            float o_acc[128];
#pragma unroll
            for (int i = 0; i < 128; ++i) o_acc[i] = 0.f;
            for (int it = 0; it < w.n_tiles; ++it) {
                const int t = gt + it, b = t & 1, rg = t % kRing;
                dm::mbar_wait(&s.bar_d_full[b], (t >> 1) & 1, wc);      // also orders the ring slot written before the codes
                dm::tc_fence_after();
                const float alpha = s.alpha[rg][row], w0 = s.wgt[rg][0][row], w1 = s.wgt[rg][1][row];
                uint32_t sa[32], sb[32];
                dm::tmem_ld32(dm::tmem_addr(t_d0, lane_base, 0), sa);
                if (__any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll
                    for (int i = 0; i < 128; i += 2) dm::mul2(o_acc[i], o_acc[i + 1], o_acc[i], o_acc[i + 1], alpha, alpha);
                }
                // eight 32-column pieces (group 0 columns 0..127, then group 1), the next one in flight while one is added
#pragma unroll
                for (int pc = 0; pc < 8; ++pc) {
                    uint32_t* cur = (pc & 1) ? sb : sa;
                    uint32_t* nxt = (pc & 1) ? sa : sb;
                    dm::tmem_ld_wait();
                    if (pc < 7) dm::tmem_ld32(dm::tmem_addr((pc + 1 < 4) ? t_d0 : t_d1, lane_base, 32 * ((pc + 1) & 3)), nxt);
                    const float wg = (pc < 4) ? w0 : w1;
                    const int c0 = 32 * (pc & 3);
#pragma unroll
                    for (int i = 0; i < 32; i += 2)
                        dm::fma2(o_acc[c0 + i], o_acc[c0 + i + 1], __uint_as_float(cur[i]), __uint_as_float(cur[i + 1]), wg,
                                 o_acc[c0 + i], o_acc[c0 + i + 1]);
                }
                dm::tc_fence_before();
                dm::mbar_arrive_warp(&s.bar_d_free);
            }
            gt += w.n_tiles;
            // ---- the item's epilogue: the softmax warps have left both halves of the denominator
            dm::mbar_wait(&s.bar_l[r & 3], (r >> 2) & 1, wc);
            const float l = s.lsum[r & 3][0][row] + s.lsum[r & 3][1][row];
            const bool dead = (l == 0.f) || (l != l);
            const float inv = dead ? 0.f : 1.0f / l;
            // The bf16 rows leave through shared memory: a thread holds a whole row, so stored directly every 16-byte store
            // instruction would touch 32 different rows; from the warp's staging slice each instruction writes two whole 256-byte
            // rows.  A warp's 32 rows are its own, so the hand-over needs no more than the warp.
            uint8_t* stg = s.stg[warp & 3];
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                uint32_t w4[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    __nv_bfloat162 tt = __floats2bfloat162_rn(o_acc[8 * c + 2 * e] * inv, o_acc[8 * c + 2 * e + 1] * inv);
                    w4[e] = *reinterpret_cast<uint32_t*>(&tt);
                }
                *reinterpret_cast<uint4*>(stg + lane * 256 + ((c ^ (lane & 15)) << 4)) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
            }
            __syncwarp();
            {
                const int row0 = w.li * 128 + (warp & 3) * 32;          // first of the warp's rows inside the (local) Q-side tensors
                uint8_t* obase = reinterpret_cast<uint8_t*>(p.o + (((int64_t)w.hc.b * p.rm.nq + row0) * p.H + w.hc.h) * 128);
                const int64_t row_bytes = (int64_t)p.H * 128 * 2;
                const int j = lane & 15;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int rr = 2 * i + (lane >> 4);
                    const uint4 val = *reinterpret_cast<const uint4*>(stg + rr * 256 + ((j ^ (rr & 15)) << 4));
                    *reinterpret_cast<uint4*>(obase + rr * row_bytes + (j << 4)) = val;
                }
            }
            __syncwarp();                                  // the slice may take the next item's rows
        }
    } else {
        // =============================================================== softmax warps
        const int g = warp >> 2;                  // warpgroup = key group inside the tile
        const int row = (warp & 3) * 32 + lane;   // query row inside the block = tensor-memory lane
        int gt = 0;
        // An item's Q scale and the K / V scales of its first key tile are read one item ahead: read at the item's start
        // they would be three exposed global loads in front of its first tile.
        float q8sc_nx = 0.f, ks_nx = 0.f, vs_nx = 0.f;
        auto first_scales = [&](const FwdItem& wi) {
            if (!wi.valid) return;
            const int64_t ko = (int64_t)wi.hc.bhk * (p.N / 64) + g + 2 * (wi.n_tiles - 1);
            q8sc_nx = p.q8s[(int64_t)wi.hc.bh * nq_blk + wi.li];
            ks_nx = p.k8s[ko];
            vs_nx = p.v8s[ko];
        };
        first_scales(fwd_item(p, 0));
        for (int r = 0;; ++r) {
        const FwdItem w = fwd_item(p, r);
        if (!w.valid) break;
        const int n_tiles = w.n_tiles, I = w.I;
        const float q8sc = q8sc_nx;
        const float* ksp = p.k8s + (int64_t)w.hc.bhk * (p.N / 64) + g;
        const float* vsp = p.v8s + (int64_t)w.hc.bhk * (p.N / 64) + g;
        float m_run = -INFINITY, l_part = 0.f;

        float ks_n = ks_nx, vs_n = vs_nx;
        first_scales(fwd_item(p, r + 1));
        for (int it = 0; it < n_tiles; ++it) {
            const int t = gt + it, j = n_tiles - 1 - it, b = t & 1, rg = t % kRing;
            const float ks = ks_n, vs = vs_n;
            if (it + 1 < n_tiles) {
                ks_n = ksp[2 * (j - 1)];
                vs_n = vsp[2 * (j - 1)];
            }

            // ---- S for this thread's (row, key group): 64 fp32 values
            dm::mbar_wait(&s.bar_s_full[b], (t >> 1) & 1, wc);
            dm::tc_fence_after();
            float sv[64];
            dm::tmem_ld32(dm::tmem_addr(tmem + b * 128, lane_base, g * 64), reinterpret_cast<uint32_t*>(sv));
            dm::tmem_ld32(dm::tmem_addr(tmem + b * 128, lane_base, g * 64 + 32), reinterpret_cast<uint32_t*>(sv) + 32);
            dm::tmem_ld_wait();
            dm::tc_fence_before();
            dm::mbar_arrive_warp(&s.bar_s_free[b]);            // this S buffer may be overwritten

            // The group maximum is taken on the raw products: the group's scale is positive, so scaling the maximum gives the
            // maximum of the scaled scores bit for bit, and the scores themselves are scaled inside the exponent's one
            // multiply-add below (x = raw * (dsc * log2 e) - ms).  The scale is kept a normal number (it underflows only when a Q
            // block and a K group are both all zero, where every product is zero anyway), so that a masked -inf stays -inf.
            const float dsc = fmaxf(q8sc * ks, 1.2e-38f);
            if (p.causal && j == I) {
#pragma unroll
                for (int c = 0; c < 64; ++c)
                    if (g * 64 + c > row) sv[c] = -INFINITY;
            }
            float gm;
            {
                float m0 = fmaxf(sv[0], sv[1]), m1 = fmaxf(sv[2], sv[3]);
#pragma unroll
                for (int c = 4; c < 64; c += 4) {
                    m0 = dm::fmax3(m0, sv[c], sv[c + 1]);
                    m1 = dm::fmax3(m1, sv[c + 2], sv[c + 3]);
                }
                gm = fmaxf(m0, m1) * dsc;
            }
            s.gmax[b][g][row] = gm;
            dm::named_bar_sync(1, kSoftmaxThreads);
            const float tile_max = fmaxf(s.gmax[b][0][row], s.gmax[b][1][row]);
            const float m_new = fmaxf(m_run, tile_max);
            const float m_cur = (m_new == -INFINITY) ? 0.f : m_new;
            const float alpha = dm::ex2((m_run - m_cur) * dm::kLog2e);
            const float ml2 = m_cur * dm::kLog2e;
            const float ms = fmaxf(gm * dm::kLog2e, ml2 - dm::kPhatFloorB) - dm::kLog2_448;
            const float sigma = dm::ex2(ms - ml2);
            // the ring slot of tile it - kRing has been read: its fold came before the fold of tile it - 3, whose release
            // of the product buffers came before the products of tile it - 2, which S of this tile waited for
            s.wgt[rg][g][row] = vs * sigma;
            if (g == 0) s.alpha[rg][row] = alpha;
            float part0 = 0.f, part1 = 0.f;
            uint32_t codes[16];
            const float nms = -ms, cl = __fmul_rn(dsc, dm::kLog2e);
#pragma unroll
            for (int c = 0; c < 64; c += 4) {
                float x0, x1, x2, x3;
                dm::fma2(x0, x1, sv[c], sv[c + 1], cl, nms, nms);
                dm::fma2(x2, x3, sv[c + 2], sv[c + 3], cl, nms, nms);
                const float p0 = dm::ex2(x0), p1 = dm::ex2(x1), p2 = dm::ex2(x2), p3 = dm::ex2(x3);
                dm::add2(part0, part1, p0, p1);
                dm::add2(part0, part1, p2, p3);
                codes[c >> 2] = dm::cvt_e4m3x4(p0, p1, p2, p3);
            }
            const float part = part0 + part1;
            l_part = fmaf(l_part, alpha, sigma * part);
            // the codes go back into tensor memory, over the first 16 columns of this thread's own 64 scores (all read by
            // now): the P V products take them from there as their A operand, four e4m3 per column, lane = row
            dm::tmem_st16(dm::tmem_addr(tmem + b * 128, lane_base, g * 64), codes);
            m_run = m_new;
            dm::tmem_st_wait();
            dm::tc_fence_before();
            dm::mbar_arrive_warp(&s.bar_codes[b]);
        }

        gt += n_tiles;
        // ---- the item's epilogue: denominator halves to the fold warps, LSE
        s.lsum[r & 3][g][row] = l_part;
        dm::mbar_arrive_warp(&s.bar_l[r & 3]);
        dm::named_bar_sync(1, kSoftmaxThreads);
        if (g == 0) {
            const float l = s.lsum[r & 3][0][row] + s.lsum[r & 3][1][row];
            const bool dead = (l == 0.f) || (l != l);
            p.lse[(int64_t)w.hc.bh * p.rm.nq + w.li * 128 + row] = dead ? -INFINITY : m_run + logf(l);
        }
        }
    }
    dm::tc_fence_before();
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
// setmaxnreg requests of the forward's roles: 8 softmax warps keep 128, 4 fold warps take 208, 4 service warps keep 40
constexpr int kFwdRegPool = 256 * 128 + 128 * 208 + 128 * 40;
static_assert(kFwdRegPool <= kThreads * 128, "the roles' register requests must fit the launch pool");

int prepare_fwd(char* err, size_t errlen) {
    static DeviceOnce once;
    return device_once(once, err, errlen, [&]() -> int {
        DM_CUDA(cudaFuncSetAttribute(fwd_d128_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(FwdSmem) + 1024));
        return check_register_pool((const void*)fwd_d128_kernel, kThreads, kFwdRegPool, err, errlen);
    });
}

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
                dm::RowMap{cp.nq, cp.half_blocks, cp.off0, cp.off1}, sh.B * hcount, dm::make_fastdiv(sh.B * hcount), dm::make_fastdiv(hcount),
                dm::make_fastdiv(sh.H / sh.Hk)};
    if ((rc = dmh::prepare_fwd(err, errlen))) return rc;
    const int smem = (int)sizeof(FwdSmem) + 1024;
    int sms = 0;
    if ((rc = dmh::sm_count(&sms, err, errlen))) return rc;
    // persistent: one CTA per SM walks the (head, row block) items, heaviest first
    const int64_t items = (int64_t)sh.B * hcount * (cp.nq / 128);
    const int grid = (int)(items < sms ? items : sms);
    fwd_d128_kernel<<<grid, kThreads, smem, static_cast<cudaStream_t>(stream)>>>(tq, tk, tv, p);
    DM_CUDA(cudaGetLastError());
    return DM_OK;
}
