// Pass 1 of the backward, head_dim 128: dK and dV per query head, plus the e4m3 dS' code tiles and their psi scales for
// pass 2 (csrc/mainloop_bwd_sm90_fp8r.hpp:695-952 of the reference, restated for tcgen05).
//
// One work item = one 128-key block of one (batch, query head); 64-row m-blocks ascending from the causal start.  The
// kernel is persistent: one CTA per SM walks its share of the items, and the next item starts under the tail of the
// current one.  768 threads in three roles that meet only through mbarriers:
//   warps 0..15  softmax, four per scheduler: thread = (key, 16-row quarter of the m-block); P-hat, dS', the tile amax, psi
//                and the two code tiles of every m-block; they hold no accumulator (64 registers each)
//   warps 16..19 fold: thread = key; they own dK (128 fp32 columns in registers) and drive dV's accumulator in tensor memory
//   warps 20..23 service, one per scheduler, loops converged with one issuing lane: the S^T / dP^T tcgen05.mma, the dK / dV
//                tcgen05.mma and the dS' TMA store, the TMA loads, the per-row constants
// Registers move between the roles by setmaxnreg; the CTA's pool is what it was launched with (768 x 80), so what the
// softmax and service warps give up (16 x 16 + 4 x 40 per lane) is exactly what the fold warps take (4 x 104).
// Everything is computed transposed (keys x rows): tensor-memory lane = key, so the per-key scales are per-thread
// constants.  Per m-block:
//   S^T = K Q^T, dP^T = V dO^T     tcgen05.mma M128 N64 K32 x 4 each into the (S | dP) tensor-memory buffer, issued as soon
//                                  as the softmax warps have read the previous m-block's
//   softmax warps                  P-hat, dS' = P-hat (dP descaled - delta k8s), tile amax over the 64 x 128 tile (one named
//                                  barrier among the softmax threads), psi by the F2 / F2b rules, codes
//                                  P-hat8 = e4m3(P-hat), dS'8 = e4m3(dS' / psi) into two swizzled K-major tiles [key][row];
//                                  the finished 128 x 128 dS' tile of a row pair leaves by one TMA store
//   dV_tmp (+)= P-hat8^T dO8       M128 N128 K32 x 2, zero-initialised on the first m-block of a 128-row dO scale block
//   dK_tmp  = dS'8^T Q8            M128 N128 K32 x 2, zero-initialised
//   dK += dK_tmp * (psi 2^-8 q8sc)   by the fold warps, in registers, while the softmax warps are on the next m-block
//   dV += dV_tmp * (2^-8 do8sc)       once per 128-row dO scale block: dV's fp32 accumulator lives in tensor memory
//                                  (columns [384, 512)); the fold warps read product and accumulator, add, and store it back
// Q8 / dO8 m-block tiles serve twice: K-major as the B operand of S^T / dP^T and MN-major as the B operand of dK / dV.
// The dS' tile layout in global memory is [key][row] (128 x 128 bytes), which pass 2 reads as an MN-major A operand.
#include "dm_attn_common.cuh"
#include "dm_host.h"

namespace dmh {
int check_shape(const DmShape& s, int h0, int hcount, char* err, size_t errlen);
}

namespace {

constexpr int kTile = 128 * 128;
constexpr int kHalf = 64 * 128;
constexpr int kSoftmaxWarps = 16;      // four per scheduler: key quarter (warp & 3) x 16-row quarter of the m-block (warp >> 2)
constexpr int kComputeThreads = 32 * kSoftmaxWarps;
constexpr int kThreads = kComputeThreads + 256;   // + one fold warpgroup + one service warpgroup
constexpr int kRing = 4;               // depth of the per-m-block scale ring between softmax and fold warps

// Geometry per head dim.  head_dim 256 (csrc/mainloop_bwd_sm90_fp8v10.hpp:1674-1761 of the reference): a code row is two
// 128-byte sub-tiles, K / V scales per 32 keys, Q / dO scales per 64-row m-block, psi per 64 rows x 64 keys (so a CTA's 128
// keys carry two psi tiles per m-block, one per lane half), dV folded every m-block.  The dK / dV accumulators of 128 keys x
// 256 columns do not fit the registers, so two work items (d half 0 and 1) share a key block: both form S^T / dP^T, each
// keeps its 128 columns of dK / dV, and only d half 0 writes the dS' tiles and psi.
template <int kD>
struct Geo {
    static constexpr int kDH = kD / 128;                 // 128-byte sub-tiles per code row
    static constexpr int kStages = kD == 128 ? 4 : 3;    // Q / dO ring depth
    static constexpr int kKeysPerScale = kD == 128 ? 64 : 32;
    static constexpr int kGrp = 128 / kKeysPerScale;     // K / V scale groups per key block
};

template <int kD>
struct Bwd1Smem {
    static constexpr int kDH = Geo<kD>::kDH, kStages = Geo<kD>::kStages, kGrp = Geo<kD>::kGrp;
    alignas(1024) uint8_t k[kDH][kTile];
    alignas(1024) uint8_t v[kDH][kTile];
    alignas(1024) uint8_t q[kStages][kDH][kHalf];
    alignas(1024) uint8_t dO[kStages][kDH][kHalf];
    alignas(1024) uint8_t pt[kTile];      // P-hat codes, [key][row of the 128-row pair]; an m-block owns one 64-byte half
    alignas(1024) uint8_t ds[2][kTile];   // dS' codes, same layout, one tile per 128-row pair parity (a TMA store drains the other)
    alignas(1024) uint8_t stg[kD == 128 ? 2 * kTile : 16];   // head_dim 128: the epilogue's 128 rows x 256 bytes of bf16 dK / dV
    alignas(16) float rc[3][64];                      // 8 - lse * log2e per row of the m-block (ring of 3 m-blocks)
    alignas(16) float dlk[3][kGrp][64];               // -delta * k8s(group) per row
    float sc[3][2];                                   // q8sc, do8sc of the m-block (same ring)
    float gf[kRing][4];                               // per m-block: dK scale of key half 0, of key half 1, dV scale
    float amax[2][kSoftmaxWarps];
    uint64_t bar_kv, bar_qdo[kStages], bar_stage_free[kStages], bar_sp_full, bar_sp_free, bar_codes[2], bar_dkv_full[2],
        bar_dkv_free, bar_ds_free[2], bar_rows_full[3], bar_rows_free[3], bar_kv_free;
    uint32_t tmem_base;
    int abort_flag;
};

struct Bwd1Params {
    const float* q8s;
    const float* k8s;
    const float* v8s;
    const float* do8s;
    const float* lse;
    const float* delta;
    __nv_bfloat16* dk;
    __nv_bfloat16* dv;
    uint8_t* ds_ws;
    float* psi;
    int H, Hk, N, h0, hcount, causal;
    int* status;
    dm::RowMap rm;                                // which rows of the sequence the Q-side tensors hold
    int out_fp32;                                 // dK / dV leave as fp32 (partials that another rank's are added to)
    int n_heads;                                  // batch * hcount: (batch, query head) pairs of this call
    dm::FastDiv fd_heads, fd_hcount, fd_rep, fd_nbn;   // divisions by n_heads, hcount, H / Hk and N / 128
};

// The work list: one item = one 128-key block J of one (batch, query head) (and one d half at head_dim 256), ordered by
// key block, i.e. heaviest first when causal.  CTA c takes position c of the even rounds and G - 1 - c of the odd ones
// (a snake), so the long and the short items of a round pair up.
struct Bwd1Item {
    dm::HeadCoord hc;
    int J, zh, m_lo, n_it, bhl;
    bool valid;
};
template <int kD>
__device__ __forceinline__ Bwd1Item bwd1_item(const Bwd1Params& p, int round) {
    Bwd1Item w;
    const int G = gridDim.x, c = blockIdx.x;
    const int nbn = p.N / 128;
    const int idx = round * G + ((round & 1) ? G - 1 - c : c);
    w.valid = idx < p.n_heads * nbn * (kD / 128);
    const int jz = (int)dm::fdiv((uint32_t)idx, p.fd_heads);
    w.hc = dm::head_coord(idx - jz * p.n_heads, p.h0, p.fd_hcount, p.H, p.Hk, p.fd_rep);
    w.bhl = w.hc.b * p.hcount + (w.hc.h - p.h0);
    w.zh = kD == 128 ? 0 : (int)dm::fdiv((uint32_t)jz, p.fd_nbn);   // d half whose dK / dV columns the item keeps
    w.J = jz - w.zh * nbn;
    // m-blocks are counted in the local rows; global position grows with the local index, and both chunks of a row map
    // start on a 128-row pair, so local and global m-block parity agree.  Causal: start at the first local m-block that is
    // not wholly above the diagonal of key block J; a rank may hold none (n_it == 0: dK = dV = 0 for this block).
    const int nq_blk = p.rm.nq / 128, nbm = p.rm.nq / 64;
    w.m_lo = 0;
    if (p.causal) {
        const int rest = nq_blk - p.rm.half;
        if (w.J < p.rm.off0 + p.rm.half) w.m_lo = 2 * max(w.J - p.rm.off0, 0);
        else if (w.J < p.rm.off1 + rest) w.m_lo = 2 * (p.rm.half + max(w.J - p.rm.off1, 0));
        else w.m_lo = nbm;
    }
    w.n_it = nbm - w.m_lo;
    return w;
}

template <int kD>
__global__ void __launch_bounds__(kThreads, 1)
bwd1_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                 const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                 const __grid_constant__ CUtensorMap tm_ds, const Bwd1Params p) {
    extern __shared__ uint8_t smem_raw[];
    using G = Geo<kD>;
    constexpr int kDH = G::kDH, kStages = G::kStages, kGrp = G::kGrp, kKPS = G::kKeysPerScale;
    Bwd1Smem<kD>& s = *reinterpret_cast<Bwd1Smem<kD>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nbn = p.N / 128;
    const int nq_blk = p.rm.nq / 128, nbm = p.rm.nq / 64;   // local 128-row blocks and 64-row m-blocks
    // Persistent: one CTA per SM walks its items (bwd1_item).  Every role keeps its own place in the list; `gt` counts the
    // m-blocks of the items before the current one (always even), so ring stages, buffer parities and mbarrier phases
    // run on across items (t = gt + it below) and the next item's loads, S^T / dP^T and first m-blocks run under the
    // current item's last folds and its epilogue.  `kvn` counts the items that loaded K / V (those with m-blocks).
    dm::WaitCtx wc{&s.abort_flag, p.status};

    if (tid == 0) {
        s.abort_flag = 0;
        dm::mbar_init(&s.bar_kv, 1);
        for (int i = 0; i < kStages; ++i) {
            dm::mbar_init(&s.bar_qdo[i], 1);
            dm::mbar_init(&s.bar_stage_free[i], 1);
        }
        for (int i = 0; i < 3; ++i) {
            dm::mbar_init(&s.bar_rows_full[i], 1);
            dm::mbar_init(&s.bar_rows_free[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            dm::mbar_init(&s.bar_codes[i], kSoftmaxWarps);
            dm::mbar_init(&s.bar_ds_free[i], 1);
            dm::mbar_init(&s.bar_dkv_full[i], 1);
        }
        dm::mbar_init(&s.bar_sp_full, 1);
        dm::mbar_init(&s.bar_sp_free, kSoftmaxWarps);
        dm::mbar_init(&s.bar_dkv_free, 4);
        dm::mbar_init(&s.bar_kv_free, 1);
        dm::fence_mbar_init();
    }
    if (warp == 0) dm::tmem_alloc(&s.tmem_base, 512);
    dm::tc_fence_before();
    __syncthreads();
    dm::tc_fence_after();
    // tensor memory: S^T | dP^T at columns [0, 64) | [64, 128), dV product [128, 256), dK product [256, 384), dV accumulator
    // [384, 512)
    const uint32_t tmem = s.tmem_base;
    const uint32_t t_dv = tmem + 128, t_dk = tmem + 256, t_dva = tmem + 384;
    const uint32_t lane_base = (uint32_t)(warp & 3) * 32;
    const int key = (warp & 3) * 32 + lane;       // tensor-memory lane of the softmax and fold threads
    const int khalf = key >> 6;                   // 64-key half (the psi tile at head_dim 256)

    if (warp >= kSoftmaxWarps + 4) {
        // =============================================================== service warps (the last warpgroup), one per scheduler
        // Each runs its loop converged (all lanes wait and compute the same addresses, so they stay in uniform registers)
        // and lane 0 alone executes the asynchronous instruction.
        dm::reg_dec<40>();
        const bool leader = lane == 0;
        if (warp == kSoftmaxWarps + 4) {
            // ---- S^T = K Q^T and dP^T = V dO^T of every m-block, as soon as the softmax warps have read the previous pair
            constexpr uint32_t idesc_sp = dm::idesc_e4m3(128, 64, false, false);
            constexpr uint32_t kSub = kTile >> 4, kSubQ = kHalf >> 4, kStageQ = (kDH * kHalf) >> 4;   // descriptor strides
            const uint32_t k_lo = dm::smem_desc_lo_sw128(dm::smem_u32(s.k[0])), v_lo = dm::smem_desc_lo_sw128(dm::smem_u32(s.v[0]));
            const uint32_t q_lo = dm::smem_desc_lo_sw128(dm::smem_u32(s.q[0][0])), do_lo = dm::smem_desc_lo_sw128(dm::smem_u32(s.dO[0][0]));
            int gt = 0, kvn = 0;
            for (int r = 0;; ++r) {
                const Bwd1Item w = bwd1_item<kD>(p, r);
                if (!w.valid) break;
                if (w.n_it > 0) dm::mbar_wait(&s.bar_kv, kvn & 1, wc);
                for (int it = 0; it < w.n_it; ++it) {
                    const int t = gt + it, st = t % kStages;
                    dm::mbar_wait(&s.bar_qdo[st], (t / kStages) & 1, wc);
                    // the softmax warps read the row constants of this m-block once its products are there: waiting here
                    // saves them a wait of their own
                    dm::mbar_wait(&s.bar_rows_full[t % 3], (t / 3) & 1, wc);
                    if (t >= 1) dm::mbar_wait(&s.bar_sp_free, (t - 1) & 1, wc);
                    // The softmax warps rewrite, in this m-block, the P-hat half tile that the dV product of m-block t - 2 read,
                    // and (first m-block of a row pair) the dS' tile that the TMA store of the pair two back drains: both
                    // must be done.  Gating the products gates the softmax warps.
                    if (t >= 2) dm::mbar_wait(&s.bar_dkv_full[t & 1], ((t - 2) >> 1) & 1, wc);
                    const int pair = t >> 1;         // gt and m_lo are even: pairs start at even t
                    if ((t & 1) == 0 && pair >= 2) dm::mbar_wait(&s.bar_ds_free[pair & 1], ((pair - 2) >> 1) & 1, wc);
                    dm::tc_fence_after();
                    const uint32_t t_s = tmem, t_dp = tmem + 64;
                    const uint32_t qs = q_lo + st * kStageQ, dos = do_lo + st * kStageQ;
                    if (leader) {
#pragma unroll
                        for (int hh = 0; hh < kDH; ++hh) {
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                if ((hh | k) == 0) dm::umma_e4m3_lo<false>(t_s, k_lo, qs, idesc_sp);
                                else dm::umma_e4m3_lo<true>(t_s, k_lo + hh * kSub + 2 * k, qs + hh * kSubQ + 2 * k, idesc_sp);
                            }
                        }
#pragma unroll
                        for (int hh = 0; hh < kDH; ++hh) {
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                if ((hh | k) == 0) dm::umma_e4m3_lo<false>(t_dp, v_lo, dos, idesc_sp);
                                else dm::umma_e4m3_lo<true>(t_dp, v_lo + hh * kSub + 2 * k, dos + hh * kSubQ + 2 * k, idesc_sp);
                            }
                        }
                        dm::umma_commit(&s.bar_sp_full);
                        // K / V have been read for the last time: the loader may bring the next item's
                        if (it == w.n_it - 1) dm::umma_commit(&s.bar_kv_free);
                    }
                    __syncwarp();
                }
                if (w.n_it > 0) ++kvn;
                gt += w.n_it;
            }
        } else if (warp == kSoftmaxWarps + 5) {
            // ---- dV_tmp (+)= P-hat8^T dO8 and dK_tmp = dS'8^T Q8 once the codes of an m-block are in shared memory and the
            // fold warps have read the previous products; the finished dS' tile of a row pair leaves by one TMA store
            constexpr uint32_t idesc_dkv = dm::idesc_e4m3(128, 128, false, true);
            constexpr uint32_t kSub = kTile >> 4, kSubQ = kHalf >> 4, kStageQ = (kDH * kHalf) >> 4;
            const uint32_t q_lo = dm::smem_desc_lo_sw128(dm::smem_u32(s.q[0][0])), do_lo = dm::smem_desc_lo_sw128(dm::smem_u32(s.dO[0][0]));
            const uint32_t pt_lo = dm::smem_desc_lo_sw128(dm::smem_u32(s.pt)), ds_lo = dm::smem_desc_lo_sw128(dm::smem_u32(s.ds[0]));
            int gt = 0;
            for (int r = 0;; ++r) {
                const Bwd1Item w = bwd1_item<kD>(p, r);
                if (!w.valid) break;
                const int zh = w.zh;
                const int ds_row0 = (int)((((int64_t)w.bhl * nq_blk + (w.m_lo >> 1)) * nbn + w.J) * 128);   // dS' tile of the first row pair
                for (int it = 0; it < w.n_it; ++it) {
                    const int t = gt + it, st = t % kStages, par = t & 1, pp = (t >> 1) & 1;
                    dm::mbar_wait(&s.bar_codes[t & 1], (t >> 1) & 1, wc);
                    // every softmax warp is past the row constants of this m-block: their ring slot may be refilled
                    if (leader) dm::mbar_arrive(&s.bar_rows_free[t % 3]);
                    if (t >= 1) dm::mbar_wait(&s.bar_dkv_free, (t - 1) & 1, wc);
                    dm::tc_fence_after();
                    const uint32_t qs = q_lo + st * kStageQ + zh * kSubQ, dos = do_lo + st * kStageQ + zh * kSubQ;
                    const uint32_t pa = pt_lo + 4 * par, da = ds_lo + pp * kSub + 4 * par;
                    if (leader) {
                        // head_dim 128: dV_tmp accumulates the two m-blocks of a 128-row dO scale block; head_dim 256: one m-block
                        dm::umma_e4m3_lo_rt(t_dv, pa, dos, idesc_dkv, (kD == 128 && par != 0) ? 1u : 0u);
                        dm::umma_e4m3_lo<true>(t_dv, pa + 2, dos + 256, idesc_dkv);
                        dm::umma_e4m3_lo<false>(t_dk, da, qs, idesc_dkv);
                        dm::umma_e4m3_lo<true>(t_dk, da + 2, qs + 256, idesc_dkv);
                        dm::umma_commit(&s.bar_dkv_full[t & 1]);
                        dm::umma_commit(&s.bar_stage_free[st]);      // the Q / dO stage has been read for the last time
                        if (par == 1) {
                            // d half 1 (head_dim 256) stores nothing but arrives all the same: the phases run on across items
                            if (zh == 0) {
                                dm::tma_store_2d(&tm_ds, 0, ds_row0 + (it >> 1) * (nbn * 128), s.ds[pp]);
                                dm::tma_store_commit();
                                dm::tma_store_wait_read0();
                            }
                            dm::mbar_arrive(&s.bar_ds_free[pp]);
                        }
                    }
                    __syncwarp();
                }
                gt += w.n_it;
            }
            if (gt > 0) {
                // the last products: wait so shared memory stays valid until the tensor pipe has read it
                dm::mbar_wait(&s.bar_dkv_free, (gt - 1) & 1, wc);
                if (leader) dm::tma_store_wait_all0();
            }
        } else if (warp == kSoftmaxWarps + 6) {
            // ---- TMA loads: an item's K / V once the previous item's last S^T / dP^T have read theirs, then the Q8 / dO8
            // tiles of its m-blocks as far ahead as the ring allows
            int gt = 0, kvn = 0;
            for (int r = 0;; ++r) {
                const Bwd1Item w = bwd1_item<kD>(p, r);
                if (!w.valid) break;
                const int kv_row0 = w.hc.bhk * p.N + w.J * 128;
                const int q_row0 = w.hc.bh * p.rm.nq + w.m_lo * 64;
                if (w.n_it > 0) {
                    if (kvn >= 1) dm::mbar_wait(&s.bar_kv_free, (kvn - 1) & 1, wc);
                    if (leader) {
                        dm::mbar_expect_tx(&s.bar_kv, 2 * kDH * kTile);
                        for (int hh = 0; hh < kDH; ++hh) {
                            dm::tma_load_2d(s.k[hh], &tm_k, 128 * hh, kv_row0, &s.bar_kv);
                            dm::tma_load_2d(s.v[hh], &tm_v, 128 * hh, kv_row0, &s.bar_kv);
                        }
                    }
                    ++kvn;
                }
                for (int it = 0; it < w.n_it; ++it) {
                    const int t = gt + it, st = t % kStages;
                    if (t >= kStages) dm::mbar_wait(&s.bar_stage_free[st], (t / kStages - 1) & 1, wc);
                    if (leader) {
                        dm::mbar_expect_tx(&s.bar_qdo[st], 2 * kDH * kHalf);
#pragma unroll
                        for (int hh = 0; hh < kDH; ++hh) {
                            dm::tma_load_2d(s.q[st][hh], &tm_q, 128 * hh, q_row0 + it * 64, &s.bar_qdo[st]);
                            dm::tma_load_2d(s.dO[st][hh], &tm_do, 128 * hh, q_row0 + it * 64, &s.bar_qdo[st]);
                        }
                    }
                    __syncwarp();
                }
                gt += w.n_it;
            }
        } else {
            // ---- per-row constants of the m-blocks, three ahead: 8 - lse * log2e and -delta * k8s(group) for the 64 rows
            // (two per lane), and the Q / dO scales of the m-block
            const int nsq = kD == 128 ? nq_blk : nbm;
            int gt = 0;
            for (int r = 0;; ++r) {
                const Bwd1Item w = bwd1_item<kD>(p, r);
                if (!w.valid) break;
                float kk[kGrp];
#pragma unroll
                for (int gq = 0; gq < kGrp; ++gq) kk[gq] = p.k8s[(int64_t)w.hc.bhk * (p.N / kKPS) + kGrp * w.J + gq];
                for (int it = 0; it < w.n_it; ++it) {
                    const int t = gt + it, slot = t % 3, mb = w.m_lo + it;
                    const int64_t gi = (int64_t)w.hc.bh * p.rm.nq + (int64_t)mb * 64 + 2 * lane;
                    const float2 l2 = *reinterpret_cast<const float2*>(p.lse + gi);
                    const float2 d2 = *reinterpret_cast<const float2*>(p.delta + gi);
                    const int sq = (int)((int64_t)w.hc.bh * nsq) + (kD == 128 ? (mb >> 1) : mb);
                    const float sc_v = lane == 0 ? p.q8s[sq] : (lane == 1 ? p.do8s[sq] : 0.f);
                    if (t >= 3) dm::mbar_wait(&s.bar_rows_free[slot], (t / 3 - 1) & 1, wc);
                    *reinterpret_cast<float2*>(&s.rc[slot][2 * lane]) = make_float2(dm::phat_row_const(l2.x), dm::phat_row_const(l2.y));
#pragma unroll
                    for (int gq = 0; gq < kGrp; ++gq)
                        *reinterpret_cast<float2*>(&s.dlk[slot][gq][2 * lane]) = make_float2(-(d2.x * kk[gq]), -(d2.y * kk[gq]));
                    if (lane < 2) s.sc[slot][lane] = sc_v;
                    __syncwarp();
                    if (leader) dm::mbar_arrive(&s.bar_rows_full[slot]);
                }
                gt += w.n_it;
            }
        }
    } else if (warp >= kSoftmaxWarps) {
        // =============================================================== fold warps: thread = key, all 128 columns
        dm::reg_inc<184>();
        int gt = 0;
        for (int r = 0;; ++r) {
        const Bwd1Item w = bwd1_item<kD>(p, r);
        if (!w.valid) break;
        const int J = w.J, zh = w.zh, n_it = w.n_it;
        const dm::HeadCoord hc = w.hc;
        const int kgrp = key / kKPS;
        float dk_acc[128];
#pragma unroll
        for (int i = 0; i < 128; ++i) dk_acc[i] = 0.f;
        bool dv_started = false;                  // the tensor-memory accumulator holds something of this item
        const float ik = 1.0f / p.k8s[(int64_t)hc.bhk * (p.N / kKPS) + kGrp * J + kgrp];   // for the epilogue; read early
        for (int it = 0; it < n_it; ++it) {
            const int t = gt + it, r4 = t % kRing;
            dm::mbar_wait(&s.bar_dkv_full[t & 1], (t >> 1) & 1, wc);   // also orders the ring slot written before the codes
            dm::tc_fence_after();
            const float gk = s.gf[r4][kD == 128 ? 0 : khalf], fv = s.gf[r4][2];
            uint32_t sa[16], sb[16];
            // dK: eight 16-column pieces, the next one in flight while one is added
#define DM_DK_PIECE(PC, CUR, NXT)                                                                                       \
            dm::tmem_ld_wait();                                                                                         \
            if ((PC) < 7) dm::tmem_ld16(dm::tmem_addr(t_dk, lane_base, 16 * ((PC) + 1)), NXT);                           \
            _Pragma("unroll") for (int i = 0; i < 16; i += 2)                                                            \
                dm::fma2(dk_acc[16 * (PC) + i], dk_acc[16 * (PC) + i + 1], __uint_as_float(CUR[i]), __uint_as_float(CUR[i + 1]), gk, \
                         dk_acc[16 * (PC) + i], dk_acc[16 * (PC) + i + 1]);
            dm::tmem_ld16(dm::tmem_addr(t_dk, lane_base, 0), sa);
            DM_DK_PIECE(0, sa, sb)
            DM_DK_PIECE(1, sb, sa)
            DM_DK_PIECE(2, sa, sb)
            DM_DK_PIECE(3, sb, sa)
            DM_DK_PIECE(4, sa, sb)
            DM_DK_PIECE(5, sb, sa)
            DM_DK_PIECE(6, sa, sb)
            DM_DK_PIECE(7, sb, sa)
#undef DM_DK_PIECE
            // dV: the product of a whole dO scale block (two m-blocks at head_dim 128, one at 256) into the accumulator
            if (kD == 256 || (t & 1) == 1) {
#pragma unroll
                for (int pc = 0; pc < 8; ++pc) {
                    dm::tmem_ld16(dm::tmem_addr(t_dv, lane_base, 16 * pc), sa);
                    if (dv_started) dm::tmem_ld16(dm::tmem_addr(t_dva, lane_base, 16 * pc), sb);
                    dm::tmem_ld_wait();
                    if (dv_started) {
#pragma unroll
                        for (int i = 0; i < 16; i += 2) {
                            float y0, y1;
                            dm::fma2(y0, y1, __uint_as_float(sa[i]), __uint_as_float(sa[i + 1]), fv, __uint_as_float(sb[i]),
                                     __uint_as_float(sb[i + 1]));
                            sa[i] = __float_as_uint(y0);
                            sa[i + 1] = __float_as_uint(y1);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; i += 2) {
                            float y0, y1;
                            dm::fma2(y0, y1, __uint_as_float(sa[i]), __uint_as_float(sa[i + 1]), fv, 0.f, 0.f);
                            sa[i] = __float_as_uint(y0);
                            sa[i + 1] = __float_as_uint(y1);
                        }
                    }
                    dm::tmem_st16(dm::tmem_addr(t_dva, lane_base, 16 * pc), sa);
                }
                dm::tmem_st_wait();
                dv_started = true;
            }
            dm::tc_fence_before();
            dm::mbar_arrive_warp(&s.bar_dkv_free);
        }

        // ---- epilogue: dK *= 1 / k8s, dV from its accumulator, per query head.  A thread holds one row of 128 columns, and a
        // store of 16 bytes per lane to 32 different rows costs the load/store unit one pass per row; so the bf16 rows go
        // through shared memory (a buffer of their own, since the next item's tiles are already arriving; 16-byte chunks
        // XOR-swizzled by the row so both sides are conflict-free) and leave as whole 256-byte rows, two per instruction.
        // head_dim 256 has no room for that buffer and stores its rows directly, as the fp32 partials do.
        const int n_glob = J * 128 + key;
        const int64_t off = (((int64_t)hc.b * p.N + n_glob) * p.H + hc.h) * kD + zh * 128;
        if (p.out_fp32) {
#pragma unroll
            for (int pc = 0; pc < 8; ++pc) {
                float dvv[16];
                if (dv_started) {
                    dm::tmem_ld16(dm::tmem_addr(t_dva, lane_base, 16 * pc), reinterpret_cast<uint32_t*>(dvv));
                    dm::tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) dvv[i] = 0.f;
                }
                float4* ok = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.dk) + off + 16 * pc);
                float4* ov = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.dv) + off + 16 * pc);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    ok[c] = make_float4(dk_acc[16 * pc + 4 * c] * ik, dk_acc[16 * pc + 4 * c + 1] * ik, dk_acc[16 * pc + 4 * c + 2] * ik,
                                        dk_acc[16 * pc + 4 * c + 3] * ik);
                    ov[c] = make_float4(dvv[4 * c], dvv[4 * c + 1], dvv[4 * c + 2], dvv[4 * c + 3]);
                }
            }
        } else if (kD == 256) {
#pragma unroll
            for (int pc = 0; pc < 8; ++pc) {
                float dvv[16];
                if (dv_started) {
                    dm::tmem_ld16(dm::tmem_addr(t_dva, lane_base, 16 * pc), reinterpret_cast<uint32_t*>(dvv));
                    dm::tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) dvv[i] = 0.f;
                }
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t wk[4], wv[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int i = 16 * pc + 8 * c + 2 * e;
                        __nv_bfloat162 a2 = __floats2bfloat162_rn(dk_acc[i] * ik, dk_acc[i + 1] * ik);
                        __nv_bfloat162 b2 = __floats2bfloat162_rn(dvv[8 * c + 2 * e], dvv[8 * c + 2 * e + 1]);
                        wk[e] = *reinterpret_cast<uint32_t*>(&a2);
                        wv[e] = *reinterpret_cast<uint32_t*>(&b2);
                    }
                    reinterpret_cast<uint4*>(p.dk + off + 16 * pc)[c] = make_uint4(wk[0], wk[1], wk[2], wk[3]);
                    reinterpret_cast<uint4*>(p.dv + off + 16 * pc)[c] = make_uint4(wv[0], wv[1], wv[2], wv[3]);
                }
            }
        } else {
            uint8_t* stg = s.stg;                                   // 128 rows x 256 bytes
            const int wq = warp & 3;
            const int64_t row_stride = (int64_t)p.H * kD;           // elements between consecutive keys
            const int64_t off0 = (((int64_t)hc.b * p.N + J * 128) * p.H + hc.h) * kD + zh * 128;
            auto rows_out = [&](__nv_bfloat16* dst) {
                dm::named_bar_sync(2, 128);
#pragma unroll 4
                for (int j = 0; j < 16; ++j) {
                    const int row = 8 * j + 2 * wq + (lane >> 4), c = lane & 15;
                    const uint4 w = *reinterpret_cast<const uint4*>(stg + row * 256 + ((c ^ (row & 15)) << 4));
                    *reinterpret_cast<uint4*>(dst + off0 + row * row_stride + 8 * c) = w;
                }
                dm::named_bar_sync(2, 128);
            };
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                uint32_t wk[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    __nv_bfloat162 a = __floats2bfloat162_rn(dk_acc[8 * c + 2 * e] * ik, dk_acc[8 * c + 2 * e + 1] * ik);
                    wk[e] = *reinterpret_cast<uint32_t*>(&a);
                }
                *reinterpret_cast<uint4*>(stg + key * 256 + ((c ^ (key & 15)) << 4)) = make_uint4(wk[0], wk[1], wk[2], wk[3]);
            }
            rows_out(p.dk);
#pragma unroll
            for (int pc = 0; pc < 8; ++pc) {
                float dvv[16];
                if (dv_started) {
                    dm::tmem_ld16(dm::tmem_addr(t_dva, lane_base, 16 * pc), reinterpret_cast<uint32_t*>(dvv));
                    dm::tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) dvv[i] = 0.f;
                }
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t wv[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        __nv_bfloat162 b2 = __floats2bfloat162_rn(dvv[8 * c + 2 * e], dvv[8 * c + 2 * e + 1]);
                        wv[e] = *reinterpret_cast<uint32_t*>(&b2);
                    }
                    *reinterpret_cast<uint4*>(stg + key * 256 + (((2 * pc + c) ^ (key & 15)) << 4)) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
                }
            }
            rows_out(p.dv);
        }
        dm::tc_fence_before();
        gt += n_it;
        }
    } else {
        // =============================================================== softmax warps
        dm::reg_dec<64>();
        const int g = warp >> 2;                      // row quarter: rows [16 g, 16 g + 16) of the m-block
        const int kgrp = key / kKPS;                  // K / V scale group inside the block
        int gt = 0;
        for (int r = 0;; ++r) {
        const Bwd1Item w = bwd1_item<kD>(p, r);
        if (!w.valid) break;
        // few values live across the m-block loop (these warps run on 64 registers): the item's psi column as a pointer,
        // and whether its first row pair is the diagonal block of this key block (it is the first one of the causal loop)
        const int n_it = w.n_it;
        const float k8s_t = p.k8s[(int64_t)w.hc.bhk * (p.N / kKPS) + kGrp * w.J + kgrp];
        const float v8s_t = p.v8s[(int64_t)w.hc.bhk * (p.N / kKPS) + kGrp * w.J + kgrp];
        const bool diag_item = p.causal && n_it > 0 && dm::global_block(p.rm, w.m_lo >> 1) == w.J;
        constexpr bool kHalfPsi = kD == 256;     // psi per 64 keys: [heads, N/64, N/64]; else [heads, N/64, N/128]
        const int psi_stride = kHalfPsi ? nbm : nbn;
        float* psi_it = w.zh == 0 ? p.psi + ((int64_t)w.bhl * nbm + w.m_lo) * psi_stride + (kHalfPsi ? 2 * w.J + khalf : w.J) : nullptr;
        float g_max = 0.f;

        for (int it = 0; it < n_it; ++it) {
            const int t = gt + it, par = t & 1, sb = t & 1, rb = t % 3;     // gt and m_lo are even: t has the m-block's parity
            dm::mbar_wait(&s.bar_sp_full, t & 1, wc);
            dm::tc_fence_after();
            // the ring slot of this m-block's row constants and scales was complete before S^T / dP^T were issued
            const float q8sc = s.sc[rb][0], do8sc = s.sc[rb][1];
            const float dsc = dm::descale_log2(q8sc, k8s_t);
            const float dpk = do8sc * v8s_t * k8s_t;

            // ---- phase 1: P-hat, dS', tile amax; P-hat codes to shared memory.  S^T first: the exponentials run while
            // dP^T is still on its way from tensor memory.
            float sv[16], ds[16];
            dm::tmem_ld16(dm::tmem_addr(tmem, lane_base, g * 16), reinterpret_cast<uint32_t*>(sv));
            dm::tmem_ld_wait();
            dm::tmem_ld16(dm::tmem_addr(tmem + 64, lane_base, g * 16), reinterpret_cast<uint32_t*>(ds));
            const bool diag = diag_item && it < 2;
            const int row_in_pair = par * 64 + g * 16;     // row offset of column 0 inside the 128-row pair
            const float4* rc4 = reinterpret_cast<const float4*>(&s.rc[rb][g * 16]);
            const float4* dl4 = reinterpret_cast<const float4*>(&s.dlk[rb][kgrp][g * 16]);
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {                // P-hat = 2^min(S dsc + rc, 12), the exponent two at a time
                const float4 r4 = rc4[c4];
                const int c = 4 * c4;
                dm::fma2(sv[c], sv[c + 1], sv[c], sv[c + 1], dsc, r4.x, r4.y);
                dm::fma2(sv[c + 2], sv[c + 3], sv[c + 2], sv[c + 3], dsc, r4.z, r4.w);
#pragma unroll
                for (int e = 0; e < 4; ++e) sv[c + e] = dm::ex2(fminf(sv[c + e], dm::kMoE + 4.0f));
            }
            if (diag) {                                     // the diagonal 128 x 128 block only: keys above the row
#pragma unroll
                for (int c = 0; c < 16; ++c)
                    if (key > row_in_pair + c) sv[c] = 0.f;
            }
            dm::tmem_ld_wait();
            dm::tc_fence_before();
            dm::mbar_arrive_warp(&s.bar_sp_free);          // the (S | dP) buffer may be overwritten
            float am4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
                const float4 d4 = dl4[c4];                  // -delta * k8s per row
                const int c = 4 * c4;
                dm::fma2(ds[c], ds[c + 1], ds[c], ds[c + 1], dpk, d4.x, d4.y);
                dm::fma2(ds[c + 2], ds[c + 3], ds[c + 2], ds[c + 3], dpk, d4.z, d4.w);
                dm::mul2(ds[c], ds[c + 1], ds[c], ds[c + 1], sv[c], sv[c + 1]);
                dm::mul2(ds[c + 2], ds[c + 3], ds[c + 2], ds[c + 3], sv[c + 2], sv[c + 3]);
#pragma unroll
                for (int e = 0; e < 4; ++e) am4[e] = fmaxf(am4[e], fabsf(ds[c + e]));
            }
            float amax = fmaxf(fmaxf(am4[0], am4[1]), fmaxf(am4[2], am4[3]));
            {
                uint32_t w[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) w[c] = dm::cvt_e4m3x4(sv[4 * c], sv[4 * c + 1], sv[4 * c + 2], sv[4 * c + 3]);
                *reinterpret_cast<uint4*>(s.pt + dm::sw128(key, row_in_pair)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
            // the warp's maximum in one instruction: non-negative floats order like their bit patterns
            amax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(amax)));
            if (lane == 0) s.amax[sb][warp] = amax;
            dm::named_bar_sync(1, kComputeThreads);
            // the tile maximum over the warps' maxima: one load per lane and one warp reduction.  head_dim 256: the psi tile is
            // this thread's 64-key half, i.e. the warps of key quarters 2h and 2h+1 (warp & 2 selects the half)
            {
                const float a = s.amax[sb][lane & (kSoftmaxWarps - 1)];
                const bool mine = kD == 128 || (((lane & 3) >> 1) == khalf);
                amax = __uint_as_float(__reduce_max_sync(0xffffffffu, mine ? __float_as_uint(a) : 0u));
            }
            const bool tile_zero = amax * (1.0f / 448.0f) < 1e-30f;
            const float psi_raw = fmaxf(amax * (1.0f / 448.0f), 1e-30f);
            // psi = max(psi_raw, g_max * 256e-8 / q8sc); the quotient can only win when its numerator exceeds
            // psi_raw * q8sc, so the division is formed only then (the 1 % margin covers the rounding of both sides)
            float psi = psi_raw;
            const float fl_num = g_max * (256.0f * 1e-8f);
            if (fl_num > psi_raw * q8sc * 0.99f) psi = fmaxf(psi_raw, fl_num / q8sc);
            const float psi_inv = tile_zero ? 0.f : __frcp_rn(psi);     // the correctly rounded reciprocal, as 1 / psi
            const float g_cur = tile_zero ? 0.f : psi * dm::kMoInv * q8sc;
            g_max = fmaxf(g_max, g_cur);
            // psi for pass 2 and the scales of this m-block's products for the fold warps.  The ring slot was last read by
            // the fold of m-block it - kRing, which came before the products of m-block it - 2 that S^T of this one waited for.
            if (tid == 0 || (kD == 256 && tid == 64)) {
                s.gf[t % kRing][khalf] = g_cur;
                if (tid == 0) s.gf[t % kRing][2] = dm::kMoInv * do8sc;
                if (psi_it) psi_it[(int64_t)it * psi_stride] = tile_zero ? 0.f : psi;
            }

            // ---- phase 2: dS' codes, to shared memory for dK and to the workspace tile for pass 2
            uint8_t* dst = s.ds[(t >> 1) & 1];        // gt and m_lo are even: t >> 1 counts this CTA's row pairs
            {
                uint32_t w[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    float a0, a1, a2, a3;
                    dm::mul2(a0, a1, ds[4 * c], ds[4 * c + 1], psi_inv, psi_inv);
                    dm::mul2(a2, a3, ds[4 * c + 2], ds[4 * c + 3], psi_inv, psi_inv);
                    w[c] = dm::cvt_e4m3x4(a0, a1, a2, a3);
                }
                *reinterpret_cast<uint4*>(dst + dm::sw128(key, row_in_pair)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
            dm::fence_proxy_async_smem();
            dm::mbar_arrive_warp(&s.bar_codes[sb]);
        }
        gt += n_it;
        }
    }
    dm::tc_fence_before();
    __syncthreads();
    if (warp == 0) dm::tmem_dealloc(tmem, 512);
}

}  // namespace

namespace dmh {
int check_cp(const DmShape& s, const DmCp& cp, char* err, size_t errlen);
}

namespace dmh {
int prepare_bwd1(char* err, size_t errlen) {
    static DeviceOnce once;
    return device_once(once, err, errlen, [&]() -> int {
        DM_CUDA(cudaFuncSetAttribute(bwd1_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Bwd1Smem<128>) + 1024));
        DM_CUDA(cudaFuncSetAttribute(bwd1_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Bwd1Smem<256>) + 1024));
        // setmaxnreg requests: 16 softmax warps keep 64, 4 fold warps take 184, 4 service warps keep 40
        constexpr int kPool = kComputeThreads * 64 + 128 * 184 + 128 * 40;
        static_assert(kPool == kThreads * 80, "the roles' register requests must add up to the launch pool");
        if (int rc = check_register_pool((const void*)bwd1_kernel<128>, kThreads, kPool, err, errlen)) return rc;
        return check_register_pool((const void*)bwd1_kernel<256>, kThreads, kPool, err, errlen);
    });
}
}  // namespace dmh

extern "C" int dm_bwd_workspace_bytes(DmShape sh, int32_t hcount, size_t* ds8_bytes, size_t* psi_bytes) {
    if (!ds8_bytes || !psi_bytes || sh.N <= 0 || sh.N % 128 || sh.B <= 0 || hcount <= 0) return DM_ERR_ARG;
    const size_t kb = sh.D == 128 ? 128 : 64;
    *ds8_bytes = (size_t)sh.B * hcount * sh.N * sh.N;
    *psi_bytes = (size_t)sh.B * hcount * (sh.N / 64) * (sh.N / kb) * sizeof(float);
    return DM_OK;
}

extern "C" int dm_bwd_workspace_bytes_cp(DmShape sh, DmCp cp, int32_t hcount, size_t* ds8_bytes, size_t* psi_bytes) {
    if (!ds8_bytes || !psi_bytes || sh.N <= 0 || sh.N % 128 || sh.B <= 0 || hcount <= 0 || sh.D != 128) return DM_ERR_ARG;
    if (cp.nq <= 0 || cp.nq % 128 || cp.nq > sh.N) return DM_ERR_ARG;
    *ds8_bytes = (size_t)sh.B * hcount * cp.nq * sh.N;
    *psi_bytes = (size_t)sh.B * hcount * (cp.nq / 64) * (sh.N / 128) * sizeof(float);
    return DM_OK;
}

extern "C" int dm_bwd_fp8_pass1(const void* q8, const void* k8, const void* v8, const void* do8, const float* q8s, const float* k8s,
                                const float* v8s, const float* do8s, const float* lse, const float* delta, DmShape sh, int32_t h0,
                                int32_t hcount, void* dk, void* dv, void* ds8_ws, float* psi_ws, void* stream, char* err, size_t errlen) {
    DmCp cp{sh.N, sh.N / 128, 0, 0};
    return dm_bwd_fp8_pass1_cp(q8, k8, v8, do8, q8s, k8s, v8s, do8s, lse, delta, sh, cp, h0, hcount, 0, dk, dv, ds8_ws, psi_ws, stream, err,
                               errlen);
}

extern "C" int dm_bwd_fp8_pass1_cp(const void* q8, const void* k8, const void* v8, const void* do8, const float* q8s, const float* k8s,
                                   const float* v8s, const float* do8s, const float* lse, const float* delta, DmShape sh, DmCp cp,
                                   int32_t h0, int32_t hcount, int32_t out_fp32, void* dk, void* dv, void* ds8_ws, float* psi_ws,
                                   void* stream, char* err, size_t errlen) {
    int rc = dmh::check_shape(sh, h0, hcount, err, errlen);
    if (rc) return rc;
    const bool plain = cp.nq == sh.N && cp.half_blocks == sh.N / 128 && cp.off0 == 0;
    if (!plain && (rc = dmh::check_cp(sh, cp, err, errlen))) return rc;
    DM_REQUIRE(!out_fp32 || sh.D == 128, DM_ERR_UNSUPPORTED, "fp32 dK / dV partials are built for head_dim 128 only");
    const void* ptrs[] = {q8, k8, v8, do8, q8s, k8s, v8s, do8s, lse, delta, dk, dv, ds8_ws, psi_ws};
    const char* names[] = {"q8", "k8", "v8", "do8", "q8s", "k8s", "v8s", "do8s", "lse", "delta", "dk", "dv", "ds8_ws", "psi_ws"};
    for (int i = 0; i < 14; ++i)
        if ((rc = dmh::check_device_ptr(ptrs[i], names[i], err, errlen))) return rc;
    DM_REQUIRE(dmh::aligned16(dk) && dmh::aligned16(dv) && dmh::aligned16(ds8_ws), DM_ERR_ARG, "outputs and workspace must be 16-byte aligned");
    const uint64_t ntiles = (uint64_t)sh.B * hcount * (cp.nq / 128) * (sh.N / 128);
    DM_REQUIRE(ntiles * 128 < ((uint64_t)1 << 31), DM_ERR_ARG, "dS' workspace too large for one call: split the heads (got %llu tiles)",
               (unsigned long long)ntiles);
    CUtensorMap tq, td, tk, tv, ts;
    if ((rc = dmh::make_tmap_u8(&tq, q8, sh.D, (uint64_t)sh.B * sh.H * cp.nq, 64, err, errlen))) return rc;
    if ((rc = dmh::make_tmap_u8(&td, do8, sh.D, (uint64_t)sh.B * sh.H * cp.nq, 64, err, errlen))) return rc;
    if ((rc = dmh::make_tmap_u8(&tk, k8, sh.D, (uint64_t)sh.B * sh.Hk * sh.N, 128, err, errlen))) return rc;
    if ((rc = dmh::make_tmap_u8(&tv, v8, sh.D, (uint64_t)sh.B * sh.Hk * sh.N, 128, err, errlen))) return rc;
    if ((rc = dmh::make_tmap_u8(&ts, ds8_ws, 128, ntiles * 128, 128, err, errlen))) return rc;
    int* status = dmh::device_status_word(err, errlen);
    if (!status) return DM_ERR_CUDA;
    Bwd1Params p{q8s, k8s, v8s, do8s, lse, delta, static_cast<__nv_bfloat16*>(dk), static_cast<__nv_bfloat16*>(dv), static_cast<uint8_t*>(ds8_ws), psi_ws,
                 sh.H, sh.Hk, sh.N, h0, hcount, sh.causal, status, dm::RowMap{cp.nq, cp.half_blocks, cp.off0, cp.off1}, out_fp32,
                 sh.B * hcount, dm::make_fastdiv(sh.B * hcount), dm::make_fastdiv(hcount), dm::make_fastdiv(sh.H / sh.Hk),
                 dm::make_fastdiv(sh.N / 128)};
    // persistent: one CTA per SM walks the (key block, head[, d half]) items, heaviest first
    if ((rc = dmh::prepare_bwd1(err, errlen))) return rc;
    const int smem = (int)(sh.D == 128 ? sizeof(Bwd1Smem<128>) : sizeof(Bwd1Smem<256>)) + 1024;
    int sms = 0;
    if ((rc = dmh::sm_count(&sms, err, errlen))) return rc;
    const int64_t items = (int64_t)sh.B * hcount * (sh.N / 128) * (sh.D / 128);
    const int grid = (int)(items < sms ? items : sms);
    if (sh.D == 128) bwd1_kernel<128><<<grid, kThreads, smem, static_cast<cudaStream_t>(stream)>>>(tq, td, tk, tv, ts, p);
    else bwd1_kernel<256><<<grid, kThreads, smem, static_cast<cudaStream_t>(stream)>>>(tq, td, tk, tv, ts, p);
    DM_CUDA(cudaGetLastError());
    return DM_OK;
}
