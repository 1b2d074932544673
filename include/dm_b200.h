/* libdm_b200: C ABI of the B200 (sm_100a) Delta-Matching fp8 attention kernels.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, returns 0 or a negative DM_ERR_* code and, on
 * error, writes a message into `err` (may be NULL).  Nothing here exits, aborts or traps.  The caller owns every
 * buffer; all pointers are device pointers on the CURRENT device; `stream` is a cudaStream_t passed as void*.
 * Work is enqueued on `stream` and the call returns without synchronising.
 *
 * Layouts.  bf16 tensors use the flash-attention layout (batch, seqlen, heads, head_dim) with explicit element strides
 * for batch / seqlen / head (the head_dim stride must be 1).  fp8 code tensors are [batch*heads, seqlen, head_dim]
 * e4m3, contiguous, 16-byte aligned; scales are contiguous fp32 [batch*heads, seqlen / rows_per_scale] with
 * rows_per_scale = (128, 64) for (Q / dO, K / V) at head_dim 128 and (64, 32) at head_dim 256.  Query head h reads KV
 * head h / (H / Hk).
 *
 * Each declaration cites the reference interface it replaces (paths inside the haok1402/delta-matching project).
 */
#ifndef DM_B200_H
#define DM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    DM_OK = 0,
    DM_ERR_ARG = -1,        /* bad shape / pointer / alignment / size; nothing was launched */
    DM_ERR_CUDA = -2,       /* a CUDA runtime or driver call failed */
    DM_ERR_UNSUPPORTED = -3,/* valid request this build does not implement (message says which) */
    DM_ERR_DEVICE = -4      /* a kernel reported a bounded-wait timeout (see dm_device_status) */
};

/* Geometry of one attention problem. D in {128, 256}; N % 256 == 0 at D=128, N % 128 == 0 at D=256; H % Hk == 0. */
typedef struct DmShape {
    int32_t B, H, Hk, N, D;
    int32_t causal; /* 0 / 1 */
} DmShape;

/* Element strides of a (batch, seqlen, heads, head_dim) bf16 tensor; the head_dim stride is 1. */
typedef struct DmStrides {
    int64_t b, n, h;
} DmStrides;

/* Context parallelism (sequence split across ranks, used for the long-context config): a rank's Q-side tensors (Q8, dO8
 * and their scales, O, LSE, delta, dQ, the dS' workspace) hold only `nq` local rows = two chunks of the sequence (zig-zag
 * balance for causal attention): `half_blocks` 128-row blocks that start at global 128-row block `off0`, then the rest
 * starting at global block `off1` (off0 < off1, both even).  K-side tensors (K8, V8, their scales, dK, dV) always span the
 * whole sequence N.  The *_cp entry points take this map; the plain ones are the map {N, N / 128, 0, 0}.  head_dim 128 only.
 * No counterpart in the reference, which has no sequence parallelism (its long-context tool is the head split). */
typedef struct DmCp {
    int32_t nq, half_blocks, off0, off1;
} DmCp;

/* Library identity: version, numerics tag, build flags.  Replaces torch.ops.delta_matching.build_hd128 / build_gt /
 * build_bf16dp (csrc/delta_matching_api.cpp:684-704) and feeds kernel_version() (delta_matching/__init__.py:65-89). */
const char* dm_build_info(void);

/* Per-head K mean over the sequence, fp32 [B*Hk, D], bit-exact fold order: 64-row chunk sums (rows ascending), chunks
 * folded serially, one IEEE division by N.  `partials` is caller-provided scratch of dm_kmean_scratch_bytes() bytes.
 * Replaces _kmean_kernel (delta_matching/quant.py:17-29) and kmean_m17 (delta_matching/producers.py:75-94). */
size_t dm_kmean_scratch_bytes(int32_t B, int32_t Hk, int32_t N, int32_t D);
int dm_kmean(const void* k_bf16, DmStrides ks, int32_t B, int32_t Hk, int32_t N, int32_t D, float* km, float* partials,
             void* stream, char* err, size_t errlen);

/* dm_kmean for callers that cannot allocate device memory -- a process whose own arena already owns all of HBM, or a loop
 * that cannot afford cudaMalloc's device-wide synchronisation.  Same result as dm_kmean bit for bit, but the partial
 * sums live in a 4 MiB array built into the library (dm_kmean_noalloc_max_bytes(); every GPU that loads the library
 * holds it until the process exits), so the caller passes only the input and the output and the call makes no
 * cudaMalloc / cudaFree.  Shapes with B * Hk * (N / 64) * D * 4 bytes above that limit are refused with DM_ERR_ARG.
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device current)
 * and caches it: make that first call before any stream capture.  All calls on a device share the one array, which keeps
 * the previous call's contents (nothing needs clearing: each call overwrites every partial it reads); two calls that
 * overlap on the GPU (different streams, no dependency) race on it, so serialise them.
 * This entry point has no counterpart in the reference. */
size_t dm_kmean_noalloc_max_bytes(void);
int dm_kmean_noalloc(const void* k_bf16, DmStrides ks, int32_t B, int32_t Hk, int32_t N, int32_t D, float* km, void* stream,
                     char* err, size_t errlen);

/* Block quantizers: bf16 -> e4m3 codes + per-block fp32 scales.
 * mode 0 = Q (x * fp32(D^-0.5)), 1 = K (x - km[head, d]; `km` required), 2 = V (as is): scale = max(amax, 1e-30) / 448,
 * code = e4m3_rtne(clamp(x / scale, +-448)) with IEEE division.
 * Replaces _quant_kernel MODE 0/1/2 (delta_matching/quant.py:32-86) as launched by quant_q_m17 / quant_kv_m17
 * (delta_matching/producers.py:149-204).  No transposed twins are produced: the sm_100a MMAs read both majors. */
int dm_quant(int32_t mode, const void* x_bf16, DmStrides xs, int32_t B, int32_t heads, int32_t N, int32_t D, const float* km,
             void* codes, float* scales, void* stream, char* err, size_t errlen);

/* dO quantizer: scale = max(amax, 1e-30) * fp32(1/448) (a multiply), codes as above.  When `o_bf16` and `delta` are
 * non-NULL also writes the stale delta[b*H + h, n] = sum_d float(dO) * float(O) from the raw bf16 values.
 * Replaces _doq_m17_kernel / doq_m17 (delta_matching/producers.py:235-329) and _doq2_kernel (delta_matching/doq.py:12-70). */
int dm_quant_do(const void* do_bf16, DmStrides dos, const void* o_bf16, DmStrides os, int32_t B, int32_t H, int32_t N, int32_t D,
                void* codes, float* scales, float* delta, void* stream, char* err, size_t errlen);

/* Forward: O (B, N, H, D) bf16 contiguous, LSE [B*H, N] fp32 (natural log of the sm-scaled, K-centred scores).
 * h0 / hcount select a range of query heads (all batches); outputs are indexed by the full head number.
 * Replaces torch.ops.delta_matching.fwd_fp8 (csrc/delta_matching_api.cpp:105-199). */
int dm_fwd_fp8(const void* q8, const void* k8, const void* v8, const float* q8s, const float* k8s, const float* v8s,
               DmShape s, int32_t h0, int32_t hcount, void* o_bf16, float* lse, void* stream, char* err, size_t errlen);

/* The producers of the forward that depend only on the inputs, in one launch: K's per-64-row-chunk column sums
 * (partials [B*Hk, N/64, D], as dm_kmean's scratch), the Q codes / scales and the V codes / scales.  Same bits as dm_quant
 * (modes 0 and 2) and the first half of dm_kmean; the reference launches these producers one by one
 * (delta_matching/producers.py:75-94 and :149-204). */
int dm_quant_qv_kpartials(const void* q, DmStrides qs, const void* k, DmStrides ks, const void* v, DmStrides vs, DmShape s, void* q8,
                          float* q8s, void* v8, float* v8s, float* partials, void* stream, char* err, size_t errlen);

/* The two halves of dm_kmean for a sequence split across ranks: each rank's per-64-row-chunk sums [B*Hk, N_local/64, D],
 * then (after the exchange, partials in sequence order [B*Hk, N/64, D]) the fold and the division by N.  Same bits as
 * dm_kmean on the whole sequence.  No counterpart in the reference. */
int dm_kmean_partials(const void* k, DmStrides ks, int32_t B, int32_t Hk, int32_t N_local, int32_t D, float* partials, void* stream,
                      char* err, size_t errlen);
int dm_kmean_fold(const float* partials, int32_t B, int32_t Hk, int32_t N, int32_t D, float* km, void* stream, char* err, size_t errlen);

/* out[o, i] = sum over c (ascending) of in[o, c, i], fp32 in, fp32 or bf16 out: folds fp32 dK / dV partials over the query
 * heads of a KV group and over the ranks of a sequence split in a fixed order.  inner % 4 == 0.  No counterpart in the
 * reference (its GQA fold is dm_gqa_fold's). */
int dm_fold_f32(const float* in, int64_t outer, int32_t count, int64_t inner, int32_t out_is_bf16, void* out, void* stream, char* err,
                size_t errlen);

/* The same fold over the query heads for a zig-zag sequence split, written straight into the layout of the exchange that
 * follows: dkp / dvp are this rank's fp32 partials [B, N, H, D] over all keys; out is [ranks, 2 (dK, dV), B, N / ranks,
 * Hk, D] fp32 whose slice d holds the keys rank d owns (chunk d, then chunk 2 ranks - 1 - d, of N / (2 ranks) keys each).
 * Same bits as dm_fold_f32 over the heads followed by a gather of the rows.  No counterpart in the reference. */
int dm_fold_to_owners(const float* dkp, const float* dvp, int32_t B, int32_t N, int32_t H, int32_t Hk, int32_t D, int32_t world,
                      float* out, void* stream, char* err, size_t errlen);

int dm_fwd_fp8_cp(const void* q8, const void* k8, const void* v8, const float* q8s, const float* k8s, const float* v8s,
                  DmShape s, DmCp cp, int32_t h0, int32_t hcount, void* o_bf16, float* lse, void* stream, char* err, size_t errlen);

/* Pass 0: the matched delta [B*H, N] fp32 from the backward's own fp8 P-hat / dP pair.
 * Replaces torch.ops.delta_matching.delta_fp8 (csrc/delta_matching_api.cpp:471-600). */
int dm_delta_fp8(const void* q8, const void* k8, const void* v8, const void* do8, const float* q8s, const float* k8s,
                 const float* v8s, const float* do8s, const float* lse, DmShape s, int32_t h0, int32_t hcount, float* delta,
                 void* stream, char* err, size_t errlen);

int dm_delta_fp8_cp(const void* q8, const void* k8, const void* v8, const void* do8, const float* q8s, const float* k8s,
                    const float* v8s, const float* do8s, const float* lse, DmShape s, DmCp cp, int32_t h0, int32_t hcount,
                    float* delta, void* stream, char* err, size_t errlen);

/* Workspace of the backward for `hcount` query heads per batch: dS' code tiles (e4m3) and their psi scales (fp32).
 * Replaces the allocations in bwd_fp8_core (csrc/delta_matching_api.cpp:288-306). */
int dm_bwd_workspace_bytes(DmShape s, int32_t hcount, size_t* ds8_bytes, size_t* psi_bytes);

/* Pass 1: dK, dV (B, N, H, D) bf16 per QUERY head, the dS' code tiles and psi.  Pass 2: dQ (B, N, H, D) bf16.
 * Together they replace torch.ops.delta_matching.bwd_fp8_t (csrc/delta_matching_api.cpp:224-392, 429-438); the split
 * lets a caller run pass 2 of one head group on another stream (delta_matching/split.py:51-92). */
int dm_bwd_fp8_pass1(const void* q8, const void* k8, const void* v8, const void* do8, const float* q8s, const float* k8s,
                     const float* v8s, const float* do8s, const float* lse, const float* delta, DmShape s, int32_t h0,
                     int32_t hcount, void* dk_bf16, void* dv_bf16, void* ds8_ws, float* psi_ws, void* stream, char* err,
                     size_t errlen);
int dm_bwd_fp8_pass2(const void* ds8_ws, const float* psi_ws, const void* k8, DmShape s, int32_t h0, int32_t hcount,
                     void* dq_bf16, void* stream, char* err, size_t errlen);

/* Context-parallel forms.  The workspace holds the local rows only: dS' [B*hcount, nq/128, N/128, 128, 128], psi
 * [B*hcount, nq/64, N/128].  Pass 1 produces this rank's PARTIAL dK / dV over its local rows for every key of the sequence,
 * (B, N, H, D) per query head, as fp32 when out_fp32 != 0 (so the cross-rank sum is rounded once) else bf16. */
int dm_bwd_workspace_bytes_cp(DmShape s, DmCp cp, int32_t hcount, size_t* ds8_bytes, size_t* psi_bytes);
int dm_bwd_fp8_pass1_cp(const void* q8, const void* k8, const void* v8, const void* do8, const float* q8s, const float* k8s,
                        const float* v8s, const float* do8s, const float* lse, const float* delta, DmShape s, DmCp cp, int32_t h0,
                        int32_t hcount, int32_t out_fp32, void* dk, void* dv, void* ds8_ws, float* psi_ws, void* stream, char* err,
                        size_t errlen);
int dm_bwd_fp8_pass2_cp(const void* ds8_ws, const float* psi_ws, const void* k8, DmShape s, DmCp cp, int32_t h0, int32_t hcount,
                        void* dq_bf16, void* stream, char* err, size_t errlen);

/* GQA fold: per-query-head grads (B, N, H, D) bf16 -> (B, N, Hk, D) bf16, fp32 sum over the H/Hk heads of a KV head in
 * ascending head order, one bf16 rounding.  Replaces dk.reshape(B, Hk, rep, N, D).sum(2) (delta_matching/attn.py:111-118). */
int dm_gqa_fold(const void* x_bf16, int32_t B, int32_t N, int32_t H, int32_t Hk, int32_t D, void* out_bf16, void* stream,
                char* err, size_t errlen);

/* The whole forward in one call: Q / K / V quantizers (with the K mean) and the forward kernel, on the caller's stream and
 * in the caller's buffers (code and scale tensors are outputs the backward needs; km [B*Hk, D] and km_partials
 * (dm_kmean_scratch_bytes) are scratch).  Replaces the op sequence of _DMAttn._forward (delta_matching/attn.py:52-68). */
int dm_attn_forward(const void* q_bf16, DmStrides qs, const void* k_bf16, DmStrides ks, const void* v_bf16, DmStrides vs, DmShape s,
                    void* q8, float* q8s, void* k8, float* k8s, void* v8, float* v8s, float* km, float* km_partials, void* o_bf16,
                    float* lse, void* stream, char* err, size_t errlen);

/* The whole backward for all heads in one call: dO quantizer (stale delta from `o_bf16` when matched == 0), pass 0 when
 * matched != 0, pass 1, pass 2 and, with GQA, the fold of dK / dV to KV heads.  do8 / do8s / delta / ds8_ws / psi_ws and,
 * with GQA, dk_heads / dv_heads (B, N, H, D) are caller-provided intermediates; results dq (B, N, H, D), dk / dv
 * (B, N, Hk, D) bf16.  Replaces the op sequence of _DMAttn._backward without the head-group split
 * (delta_matching/attn.py:76-118); callers that need the split drive pass 0 / 1 / 2 per head range themselves. */
int dm_attn_backward(const void* do_bf16, DmStrides dos, const void* o_bf16, DmStrides os, const void* q8, const void* k8,
                     const void* v8, const float* q8s, const float* k8s, const float* v8s, const float* lse, DmShape s,
                     int32_t matched, void* do8, float* do8s, float* delta, void* dk_heads, void* dv_heads, void* ds8_ws,
                     float* psi_ws, void* dq_bf16, void* dk_bf16, void* dv_bf16, void* stream, char* err, size_t errlen);

/* Debug: row sums and absolute row sums of P-hat * (dP - delta) / 256 over all visible keys, fp32 [B*H, N] each, from
 * the same operands and arithmetic as pass 1.  Replaces the DM_DBG ops bwd_fp8_dbg / delta_fp8_dbg
 * (csrc/delta_matching_api.cpp:612-680). */
int dm_bwd_dbg_rowsum(const void* q8, const void* k8, const void* v8, const void* do8, const float* q8s, const float* k8s,
                      const float* v8s, const float* do8s, const float* lse, const float* delta, DmShape s, float* rows,
                      float* rows_abs, void* stream, char* err, size_t errlen);

/* Self-test of the tensor-core operand conventions: C[128, 128] fp32 = A * B on e4m3 tiles of 128 x 128 bytes.
 * a_mn / b_mn = 0: the tile's rows are M (or N) and its 128 bytes are K; 1: its rows are K and its 128 bytes are M (or N).
 * via_st = 1 also round-trips A through thread-written swizzled shared memory and stores it back with a TMA store into
 * `a_echo` (128 x 128 bytes).  via_st = 2, 3, 4 (a_mn = 0) put A into tensor memory with tcgen05.st and read it from there:
 * contiguous; one K step every 32 columns; and overwritten by a second product issued right behind the first (then c_out
 * is [256, n_cols]: the second product follows the first).  No counterpart in the reference (its wgmma path fixes the
 * majors in CuTe types). */
int dm_probe_mma(const void* a_tile, const void* b_tile, int32_t a_mn, int32_t b_mn, int32_t n_cols, int32_t via_st,
                 float* c_out, void* a_echo, void* stream, char* err, size_t errlen);

/* Reads (and clears) the current device's status word; synchronises the device.  0 = no kernel gave up a wait, 1 = some
 * wait on an mbarrier ran out of polls (the kernel then ran to its end without the data it waited for: its outputs are
 * invalid).  Every wait in every kernel is bounded this way; nothing spins for ever.  Mirrors the lesson of the reference's
 * pass-2 barrier bookkeeping (csrc/fq8_dq_pass2_hd128.h:323-349). */
int dm_device_status(int32_t* status, char* err, size_t errlen);

/* Self-test of that path: launches one CTA whose first warp waits, with a limit of 1024 polls, on an mbarrier nothing
 * arrives on, and whose second warp waits on another one with the normal limit.  Both waits must come back unsatisfied
 * (`waits_returned_ok`, two device ints, both 0), the kernel ends by itself, and the next dm_device_status reports 1, the one
 * after that 0.  No counterpart in the reference. */
int dm_selftest_wait_timeout(int32_t* waits_returned_ok, void* stream, char* err, size_t errlen);

/* One-time set-up of the current device: allocates the status word (the library's only allocation), sets the kernels'
 * shared-memory attributes, checks that each kernel was compiled with the register pool its roles redistribute
 * (DM_ERR_UNSUPPORTED otherwise), caches the SM count.  Every entry point does its own part of this lazily on first use;
 * a caller that captures CUDA graphs, or calls from several threads, calls dm_init once per device first, because the
 * lazy set-up allocates and synchronises.  No counterpart in the reference (its ops rely on torch's lazy initialisation). */
int dm_init(char* err, size_t errlen);

/* The rule dm_init applies to the kernels that move registers between their warp roles with setmaxnreg: 1 when a kernel
 * compiled with `compiled_regs_per_thread` registers and launched with `threads` threads owns at least the `regs_needed`
 * registers its roles request in all, else 0 (the launch is then refused: a setmaxnreg.inc would wait for ever).  Pure host
 * arithmetic, exported so it can be tested without a GPU.  No counterpart in the reference. */
int dm_register_pool_ok(int32_t compiled_regs_per_thread, int32_t threads, int32_t regs_needed);

#ifdef __cplusplus
}
#endif
#endif /* DM_B200_H */
