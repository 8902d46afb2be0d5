/* natsl_b200.h — C ABI of the B200 (sm_100a) NAtSL hybrid-attention kernels.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (as void*),
 * launches asynchronously on that stream and returns an int status: 0 on success, a
 * negative NATSL_ERR_* code otherwise, with a message available from natsl_last_error()
 * (per calling thread).  Nothing here allocates device memory: the caller owns every
 * buffer.  Tensors are contiguous, token-major:  q,k [B,T,H,K], v,o [B,T,H,V], g,beta
 * [B,T,H].  Activations are bf16; decays, scales and states are fp32.
 *
 * Reference = automl/NeuralAttentionSearchLinear; paths below are relative to its root.
 * The reference has no native FFI: its hot path is Triton launched from Python, so each
 * entry cites the Python/Triton function it replaces.
 */
#ifndef NATSL_B200_H
#define NATSL_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NATSL_B200_ABI_VERSION 1

/* element types of loosely-typed inputs */
#define NATSL_DT_BF16 0
#define NATSL_DT_F32 1
#define NATSL_DT_F16 2
#define NATSL_DT_I32 3

/* linear-branch update rule */
#define NATSL_RULE_GDN 0   /* gated delta rule */
#define NATSL_RULE_MAMBA 1 /* Mamba2 / SSD    */

/* flags */
#define NATSL_FLAG_DECAY_SKIPPED 1      /* decay_for_non_gdn_blocks / decay_for_non_mamba_blocks      */
#define NATSL_FLAG_ATTN_OWN_CHUNK 2     /* softmax branch also covers the query's own block ('all', 'attn') */
#define NATSL_FLAG_NO_TRAILING_QUIRK 4  /* carry the decay also over skipped blocks after the last selected one */
#define NATSL_FLAG_ATTN_MMA_SYNC 8      /* natsl_attn_fwd: use the mma.sync comparison kernel instead of tcgen05 */
#define NATSL_FLAG_ATTN_PERSISTENT 32   /* natsl_attn_fwd*: two resident CTAs per SM work through the query tiles (measured slower; off by default) */
#define NATSL_FLAG_BWD_REFERENCE_COMPAT 16 /* natsl_attn_bwd: drop the own-block terms, as the reference's default backward does */

#define NATSL_ATTN_BT 128 /* query rows per attention tile; the attn_n_iters table is built for it */

/* status codes */
#define NATSL_OK 0
#define NATSL_ERR_BAD_SHAPE (-1)
#define NATSL_ERR_UNSUPPORTED (-2)
#define NATSL_ERR_NULL (-3)
#define NATSL_ERR_CUDA (-4)
#define NATSL_ERR_TOO_LARGE (-5)

const char* natsl_last_error(void);
int natsl_abi_version(void);

/* Synchronises the current device and returns (and clears) its status word: 0 = every kernel ran to
 * completion; 1 = a kernel gave up a bounded wait (the tensor-core kernels never spin forever; they record
 * the failure here instead); 2 = misaligned shared memory; 3 = a capacity given by the caller was too small
 * (natsl_pack_selected_pairs).  Non-zero means the outputs of the kernels since the last call are invalid. */
int natsl_device_status(void);

/* Diagnostic: launches one warp that waits, with the kernels' bounded-wait loop and a limit of `polls` polls, on a
 * barrier nobody arrives at.  The wait runs out, the kernel returns, and natsl_device_status() then reads 1 (and
 * clears it).  Shows that an expired wait is reported and leaves the context usable.  No reference counterpart. */
int natsl_bounded_wait_selftest(int polls, void* stream);

/* Selection tables from the op types [B,TN,HN,2] (column 0 softmax, column 1 linear).
 * Replaces: round / index sort / block counts, src/nats/ops/mixed_ops/mixed_attn_gdn.py:88-100;
 * prepare_nats_block_indices src/nats/ops/nats_util.py:6-32; prepare_nats_chunk_offsets :35-64;
 * compute_attn_n_iters_per_block :67-121; compute_starting_idx_for_chunks :124-162.
 * Outputs (int32): types_i, indices [B,TN,HN,2]; n_blocks [B,HN,2]; n_chunks_lin [B*HN];
 * offsets [B*HN+1]; chunk_indices [B*HN*cdiv(T,64), 2] (first offsets[B*HN] rows valid, may be
 * NULL); starting_h_idx [B,cdiv(T,64),HN]; attn_n_iters [B,cdiv(T,attn_bt),HN]. */
int natsl_build_tables(const void* types, int types_dtype, int B, int TN, int HN, int T, int nbs, int attn_bt,
                       int32_t* types_i, int32_t* indices, int32_t* n_blocks, int32_t* n_chunks_lin, int32_t* offsets,
                       int32_t* chunk_indices, int32_t* starting_h_idx, int32_t* attn_n_iters, void* stream);

/* Chunk-masked softmax attention forward.  q [B,T,HQ,DK], k [B,T,HKV,DK], v [B,T,HKV,DV] bf16;
 * o [B,T,HQ,DV] bf16; lse [B,T,HQ] fp32 (base 2).  attn_n_iters must come from
 * natsl_build_tables with attn_bt = NATSL_ATTN_BT.
 * Replaces: parallel_attn_nats_fwd src/nats/ops/attns/attns.py:1421-1531 (kernel :62-353). */
int natsl_attn_fwd(const void* q, const void* k, const void* v, const int32_t* types_i, const int32_t* indices,
                   const int32_t* attn_n_iters, void* o, float* lse, int B, int T, int HQ, int HKV, int HN, int DK,
                   int DV, int nbs, float scale, int flags, void* stream);

/* Same, for a window of queries: q, o [B,Tq,HQ,.], lse [B,Tq,HQ] are the tokens [q_off, q_off+Tq) of the
 * T-key sequence the tables describe (q_off a multiple of 128 and of nbs).  Used by the sequence-parallel
 * path, where the keys are [gathered selected blocks of earlier ranks | own segment].  No reference
 * counterpart (the reference has no sequence parallelism). */
int natsl_attn_fwd_ex(const void* q, const void* k, const void* v, const int32_t* types_i, const int32_t* indices,
                      const int32_t* attn_n_iters, void* o, float* lse, int B, int T, int Tq, int q_off, int HQ,
                      int HKV, int HN, int DK, int DV, int nbs, float scale, int flags, void* stream);

/* Same, with the T keys held in two pairs of tensors: keys [0, k_split) in k_rem, v_rem (batch index b % B_rem:
 * blocks gathered from other segments, shared by the B / B_rem local segments that sit segment-major in the batch),
 * keys [k_split, T) in k, v [B, T - k_split, HKV, .].  k_split is a multiple of nbs and <= q_off; k_split = 0
 * ignores the gathered tensors.  Two layouts of the gathered part:
 *   rem_base = NULL: k_rem, v_rem [B_rem, k_split, HKV, .], token-major like k, v;
 *   rem_base [B_rem, G, HKV] int32: k_rem, v_rem [B_rem, rem_tokens, .] hold only the selected (block, head) pairs
 *     of the G gathered segments (natsl_pack_selected_pairs); the virtual key sequence gives every gathered
 *     segment rem_slots blocks per head (k_split = G * rem_slots * nbs) and virtual block g * rem_slots + j of
 *     head h is the nbs tokens starting at token (rem_base[b % B_rem, g, h] + j) * nbs.
 * No reference counterpart (sequence parallelism). */
int natsl_attn_fwd_split(const void* q, const void* k_rem, const void* v_rem, const int32_t* rem_base, int rem_slots,
                         int rem_tokens, const void* k, const void* v, const int32_t* types_i, const int32_t* indices,
                         const int32_t* attn_n_iters, void* o, float* lse, int B, int B_rem, int T, int Tq, int q_off,
                         int k_split, int HQ, int HKV, int HN, int DK, int DV, int nbs, float scale, int flags,
                         void* stream);

/* Debug/parity: dense 0/1 mask [B,HQ,T,T] (uint8) from the same tile walk as natsl_attn_fwd.
 * Counterpart: store_msk=True of the reference kernel, src/nats/ops/attns/attns.py:214-217,
 * 321-323, 1495-1498. */
int natsl_attn_dense_mask(const int32_t* types_i, const int32_t* indices, const int32_t* attn_n_iters, uint8_t* mask,
                          int B, int T, int HQ, int HN, int nbs, int flags, void* stream);

/* Chunk-local cumsum of the log decay, g and gcs [B,T,H] fp32.
 * Replaces: chunk_local_cumsum calls at src/nats/ops/mamba/chunk.py:49-51,
 * src/nats/ops/gated_delta_rule/chunk.py:52-54. */
int natsl_chunk_local_cumsum(const float* g, float* gcs, int B, int T, int H, void* stream);

/* Gated-delta-rule chunk preparation: k_rstd, gcs [B,T,H] fp32; w [B,T,H,K], u [B,T,H,V] bf16.
 * Replaces: l2norm_fwd(k) src/nats/ops/mixed_ops/mixed_attn_gdn.py:119-121; chunk_local_cumsum;
 * chunk_scaled_dot_kkt_nats_fwd src/nats/ops/common/chunk_scaled_dot_kkt.py:272-374;
 * solve_tril_nats src/nats/ops/utils/solve_tril.py:484-569;
 * recompute_w_u_nats_fwd src/nats/ops/gated_delta_rule/wy_fast.py:386-457. */
int natsl_gdn_chunk_prep(const void* k, const void* v, const float* g, const void* beta, int beta_dtype, void* w,
                         void* u, float* gcs, float* k_rstd, int B, int T, int H, int K, int V, int use_l2norm,
                         void* stream);

/* State recurrence.  h [B,cdiv(T,64),H,K,V] bf16 = the state each chunk reads; carry
 * [B,cdiv(T,64),H] fp32 = decay of skipped blocks before each chunk (h and carry may both be NULL when only
 * the final state is wanted); ht [B,H,K,V] fp32 or NULL;
 * h0 [B,H,K,V] fp32 or NULL.  For NATSL_RULE_MAMBA pass w = NULL, u = v, k_rstd = NULL.
 * Replaces: chunk_gated_delta_rule_nats_fwd_h src/nats/ops/common/chunk_delta_h.py:638-732
 * (kernel :40-324), chunk_mamaba_nats_fwd_h src/nats/ops/mamba/chunk_h.py:220-290 (kernel :35-218)
 * and chunk_cumsum_non_gated_chunks src/nats/ops/utils/cumsum.py:136-180. */
int natsl_linear_fwd_h(int rule, const void* k, const void* w, const void* u, const float* gcs, const float* k_rstd,
                       const int32_t* types_i, const int32_t* indices, const int32_t* n_blocks, const float* h0,
                       void* h, float* carry, float* ht, int B, int T, int H, int HN, int K, int V, int nbs, int flags,
                       void* stream);

/* Output of every chunk, o [B,T,H,V] bf16.  mode: bit 0 = l2-normalise q (k through k_rstd); bit 1 = leave out
 * the own-chunk term, o = scale e^{g} q S only (ops_for_incomplete_chunks='attn', chunk_o.py:210-211).
 * Replaces: l2norm_fwd(q) src/nats/ops/mixed_ops/mixed_attn_gdn.py:119-120; chunk_fwd_nats_o
 * src/nats/ops/common/chunk_o.py:1176-1259 (kernel :35-215); chunk_mamba_fwd_nats_o
 * src/nats/ops/mamba/chunk_o.py:200-277 (kernel :34-198). */
int natsl_linear_fwd_o(int rule, const void* q, const void* k, const void* w, const void* u, const float* gcs,
                       const float* k_rstd, const void* h, const float* carry, void* o, int B, int T, int H, int K,
                       int V, float scale, int mode, void* stream);

/* Chunk preparation that also emits what the fused walk needs: q_rstd [B,T,H] fp32 and the intra-chunk score
 * matrix P = tril(qn kn^T e^{gcs_i - gcs_j}) [B,T,H,64] bf16 (q, q_rstd, pmat may all be NULL = natsl_gdn_chunk_prep).
 * Replaces in addition: l2norm_fwd(q) src/nats/ops/mixed_ops/mixed_attn_gdn.py:119-120 and the q k^T part of
 * chunk_fwd_kernel_o src/nats/ops/common/chunk_o.py:166,188,202-203. */
int natsl_gdn_chunk_prep_ex(const void* q, const void* k, const void* v, const float* g, const void* beta,
                            int beta_dtype, void* w, void* u, float* gcs, float* k_rstd, float* q_rstd, void* pmat,
                            int B, int T, int H, int K, int V, int use_l2norm, void* stream);

/* The same preparation on tcgen05 for K = V = 128 (other head dims: natsl_gdn_chunk_prep_ex): TMA tile loads, one stacked
 * [k ; q] k^T product into TMEM, (I + A)^-1 formed like the reference's solve_tril (fp32 diagonal blocks, block
 * recursion below them) and applied as one product with the raw v / k tiles as operands.  Same arguments and outputs.
 * Replaces the same reference functions as natsl_gdn_chunk_prep / natsl_gdn_chunk_prep_ex. */
int natsl_gdn_chunk_prep_tc(const void* q, const void* k, const void* v, const float* g, const void* beta,
                            int beta_dtype, void* w, void* u, float* gcs, float* k_rstd, float* q_rstd, void* pmat,
                            int B, int T, int H, int K, int V, int use_l2norm, void* stream);

/* State recurrence and chunk output in one walk on tcgen05 (state kept in TMEM, never written to memory):
 * inputs from natsl_gdn_chunk_prep_ex, outputs o [B,T,H,V] bf16 and ht [B,H,K,V] fp32 (or NULL).
 * Built for K = V = 128 and nats_block_size = 64.
 * Replaces: chunk_gated_delta_rule_nats_fwd_h + chunk_fwd_nats_o (src/nats/ops/common/chunk_delta_h.py:638-732,
 * src/nats/ops/common/chunk_o.py:1176-1259) and chunk_cumsum_non_gated_chunks (src/nats/ops/utils/cumsum.py:136-180). */
int natsl_gdn_walk_fused(const void* q, const void* k, const void* w, const void* u, const void* pmat,
                         const float* gcs, const float* k_rstd, const float* q_rstd, const int32_t* types_i,
                         const int32_t* indices, const int32_t* n_blocks, const float* h0, void* o, float* ht, int B,
                         int T, int H, int HN, int K, int V, int nbs, float scale, int flags, void* stream);

/* The same walk with the value dimension split over two CTAs per (batch, head): 256 tensor-memory columns and about
 * 107 KB of shared memory per CTA, so that two of them, or one of them and one attention CTA, share an SM (the two
 * branches of the layer then overlap).  Same arguments and results; T <= 8192. */
int natsl_gdn_walk_fused_vsplit(const void* q, const void* k, const void* w, const void* u, const void* pmat,
                                const float* gcs, const float* k_rstd, const float* q_rstd, const int32_t* types_i,
                                const int32_t* indices, const int32_t* n_blocks, const float* h0, void* o, float* ht,
                                int B, int T, int H, int HN, int K, int V, int nbs, float scale, int flags, void* stream);

/* Mamba2 / SSD state recurrence and chunk output in one walk on tcgen05 (state kept in TMEM, never written to memory;
 * q k^T, the decay mask, the scaled v tile, all four products inside the walk): q, k [B,T,H,K] bf16, v [B,T,H,V] bf16,
 * gcs = chunk-local cumsum of the log decay (natsl_chunk_local_cumsum), outputs o [B,T,H,V] bf16 and ht [B,H,K,V]
 * fp32.  o == NULL (q may then be NULL): only the recurrence runs and ht is required.  Built for K = 128, V = 64
 * and any nats_block_size that is a multiple of 64 (an unselected block's chunks update a temporary state which is
 * rolled back at the end of the block); T <= 65536.
 * Replaces: chunk_mamba_fwd_h + chunk_fwd_o of the Mamba2 branch (src/nats/ops/mamba/chunk_h.py:139-218,
 * src/nats/ops/mamba/chunk_o.py:137-198) and chunk_cumsum_non_gated_chunks (src/nats/ops/utils/cumsum.py:136-180);
 * same results as natsl_linear_fwd_h + natsl_linear_fwd_o with rule NATSL_RULE_MAMBA. */
int natsl_mamba_walk_fused(const void* q, const void* k, const void* v, const float* gcs, const int32_t* types_i,
                           const int32_t* indices, const int32_t* n_blocks, const float* h0, void* o, float* ht, int B,
                           int T, int H, int HN, int K, int V, int nbs, float scale, int flags, void* stream);

/* Reference-precision (fp32 math, CUDA cores) path for fp32 or bf16 tensors (dtype = NATSL_DT_F32 / _BF16 for
 * q, k, v, beta, o): token-by-token linear recurrence with re-roll to the block-start state, and plain masked
 * softmax attention.  ht = state after the last selected block, hstart = block-start state at the end (both
 * [B,H,K,V] fp32, may be NULL).
 * Replaces: fused_recurrent_gated_delta_rule_fwd_nats_kernel src/nats/ops/gated_delta_rule/fused_recurrent.py:28-358,
 * fused_recurrent_mamba_fwd_nats_kernel src/nats/ops/mamba/fused_recurrent.py:28-322, and the masked SDPA of the
 * recurrent ops (src/nats/ops/mixed_ops/mixed_attn_gdn.py:475-504). */
int natsl_linear_recurrent_fwd(int rule, int dtype, const void* q, const void* k, const void* v, const float* g,
                               const void* beta, const int32_t* types_i, const float* h0, void* o, float* ht,
                               float* hstart, int B, int T, int H, int HN, int K, int V, int nbs, float scale,
                               int flags, int use_l2norm, void* stream);
/* Decoding step of the linear branch: T new tokens (T < nbs typically 1) continue a block that already holds t_off
 * tokens.  h_cur = current state, h_start = state at the start of the current block, gsum [B,H] = log decay of the
 * block so far (all fp32); types_i [B, cdiv(t_off + T, nbs), HN, 2] are the types of the blocks these tokens touch,
 * read only where a block ends inside the call.  Outputs: o [B,T,H,V], h_cur_out, h_start_out (may alias the inputs'
 * buffers only if distinct tensors are not needed; each thread reads its elements before writing them).  The caller
 * keeps gsum (adds the new tokens' g, resets it where a block ends).
 * Replaces: fused_recurrent_gated_delta_rule_fwd_nats_kernel with initial_state / initial_state_current / g_cumsum /
 * n_tokens_in_current_block, src/nats/ops/gated_delta_rule/fused_recurrent.py:28-358 (Mamba2: src/nats/ops/mamba/fused_recurrent.py:28-322). */
int natsl_linear_recurrent_step(int rule, int dtype, const void* q, const void* k, const void* v, const float* g,
                                const void* beta, const int32_t* types_i, const float* h_cur, const float* h_start,
                                const float* gsum, int t_off, void* o, float* h_cur_out, float* h_start_out, int B, int T,
                                int H, int HN, int K, int V, int nbs, float scale, int flags, int use_l2norm, void* stream);
int natsl_attn_fwd_fp32(int dtype, const void* q, const void* k, const void* v, const int32_t* types_i, void* o,
                        float* lse, int B, int T, int HQ, int HKV, int HN, int DK, int DV, int nbs, float scale,
                        int flags, void* stream);

/* Sequence-parallel helpers (no reference counterpart; the recurrence they split is
 * src/nats/ops/mamba/chunk_h.py:139-218).
 * natsl_sp_segment_decay: a [B,H] = exp(total log decay the carried state sees over this segment);
 *   trail [B,H] = exp(log decay of the skipped blocks after the last selected block).
 * natsl_sp_state_combine: h_in [B,H,K,V] = sum_{r<rank} (prod_{r<r'<rank} a[r']) S[r] from the all-gathered
 *   a [world,B,H], S [world,B,H,K,V] (fp32).
 * natsl_sp_prefix_states: for N consecutive segments (a [N,B,H], S [N,B,H,K,V] fp32) and the state h0 [B,H,K,V]
 *   (or NULL = zero) the first one starts from: P[0] = h0, P[i+1] = a[i] P[i] + S[i]; writes prefix [N,B,H,K,V] = P[0..N)
 *   (or NULL), total_S [B,H,K,V] = P[N] (or NULL) and total_a [B,H] = prod a (or NULL).
 * natsl_pack_selected_blocks: packed [B, cap_blocks*nbs, H, D] <- the selected blocks (column `op`) of
 *   x [B,T,H,D] bf16 in index-table order, per head; slots past the number of selected blocks are left untouched.
 * natsl_pack_selected_pairs: packed [B, cap_pairs*nbs, D] <- the same blocks with no padding: the selected
 *   (block, head) pairs of a batch entry back to back, head-major (all blocks of head 0, then head 1, ...).  A
 *   batch entry with more than cap_pairs pairs, or a head with more than max_per_head blocks (0 = no limit),
 *   sets device status 3 and the surplus is dropped. */
int natsl_sp_segment_decay(const float* gcs, const int32_t* types_i, float* a, float* trail, int B, int T, int H,
                           int HN, int nbs, int flags, void* stream);
int natsl_sp_state_combine(const float* a, const float* S, float* h_in, int rank, int world, int B, int H, int K, int V,
                           void* stream);
int natsl_sp_prefix_states(const float* a, const float* S, const float* h0, float* prefix, float* total_S,
                           float* total_a, int N, int B, int H, int K, int V, void* stream);
int natsl_pack_selected_blocks(const void* x, const int32_t* indices, const int32_t* n_blocks, void* packed, int B,
                               int T, int H, int HN, int D, int nbs, int op, int cap_blocks, void* stream);
int natsl_pack_selected_pairs(const void* x, const int32_t* indices, const int32_t* n_blocks, void* packed, int B,
                              int T, int H, int HN, int D, int nbs, int op, int cap_pairs, int max_per_head,
                              void* stream);

/* Output mixing: y = (x1 rstd1 w1 a + x2 rstd2 w2 b) * g * sigmoid(g) over rows of D (64/128/256) bf16
 * elements; xw [rows,2] = (a, b) or NULL; w1, w2 [D] or NULL; activation 0 = swish, 1 = sigmoid.
 * Replaces: FusedMultiInputRMSNormGated forward, src/nats/modules/fused_norm_gate.py:38-182, 1354-1429. */
int natsl_norm_gate_mix(const void* x1, const void* x2, const void* g, const void* xw, int xw_dtype, const void* w1,
                        const void* w2, int w_dtype, void* y, long rows, int D, float eps, int activation,
                        void* stream);

/* ---- backward pass ------------------------------------------------------------------------------------------- */

/* Backward of the softmax branch.  Inputs as natsl_attn_fwd plus o, lse (its outputs) and d_o [B,T,HQ,DV] bf16.
 * Outputs: dq [B,T,HQ,DK], dk [B,T,HKV,DK], dv [B,T,HKV,DV] bf16; delta [B,T,HQ] fp32 = rowsum(o * do) (scratch
 * the second kernel reads); dnats_part [B,cdiv(T,64),HQ] fp32 = per 64-key tile and query head the sum of the score
 * gradients over the queries of later blocks (the caller sums tiles of a block and heads of a selection group and
 * keeps selected blocks only: the reference's dnats column 0).  flags: NATSL_FLAG_ATTN_OWN_CHUNK as in the forward;
 * NATSL_FLAG_BWD_REFERENCE_COMPAT reproduces the reference's default backward, which leaves out every own-block term
 * (src/nats/ops/mixed_ops/mixed_attn_gdn.py:237 passes the flag only for sliding windows).
 * Replaces: parallel_attn_nats_bwd src/nats/ops/attns/attns.py:1562-1759 (preprocess :357-372, dq :383-708,
 * dk/dv :719-982). */
int natsl_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                   const int32_t* types_i, void* dq, void* dk, void* dv, float* delta, float* dnats_part, int B, int T,
                   int HQ, int HKV, int HN, int DK, int DV, int nbs, float scale, int flags, void* stream);

/* Backward of the linear branch, block size 64, in five stages that run after the forward's own preparation
 * (natsl_gdn_chunk_prep / natsl_chunk_local_cumsum -> w, u, gcs) and recurrence (natsl_linear_fwd_h -> h, carry).
 * For NATSL_RULE_MAMBA pass w = NULL, u = vp = v, and NULL for v, dw, beta, dv, dbeta.
 *  1 natsl_linear_bwd_pre    qn, kn [B,T,H,K] bf16 = l2-normalised q, k with q_rstd, k_rstd [B,T,H] (use_l2norm = 0:
 *                            nothing is written, pass q, k themselves on); dvl [B,T,H,V] bf16 = scale * P^T do.
 *  2 natsl_linear_bwd_dh     reverse walk over the chunks: dS_all [B,NT,H,K,V] bf16 = gradient w.r.t. the state after
 *                            every chunk that updates it (other slots are not written), dvp [B,T,H,V] bf16 = gradient
 *                            w.r.t. v', dh0 [B,H,K,V] fp32 (may be NULL); dht [B,H,K,V] fp32 or NULL.
 *  3 natsl_linear_bwd_state  vp [B,T,H,V] = v'; dw, dq1, dk1 [B,T,H,K] bf16 (dk1 is written for updating chunks only);
 *                            dkd [B,T,H] fp32; scal [B,NT,H,4] fp32 (slots 0-2); dnats_lin [B,NT,H] fp32 = the
 *                            reference's dnats column 1 before the sum over the heads of a selection group
 *                            (invalid_dnats: also for chunks that do not update the state, from the raw values and the
 *                            state gradient of the next updating chunk).
 *  4 natsl_linear_bwd_intra  dq, dk [B,T,H,K], dv [B,T,H,V] bf16, dbeta, dg_tok [B,T,H] fp32, scal slot 3.
 *  5 natsl_linear_bwd_dg     dg [B,T,H] fp32 from dg_tok and scal; flags as natsl_linear_fwd_h.
 * Replaces: chunk_gated_delta_rule_nats_bwd src/nats/ops/gated_delta_rule/chunk.py:170-332 (kernels
 * src/nats/ops/common/chunk_o.py:234-571, 927-1173, src/nats/ops/common/chunk_delta_h.py:346-635,
 * src/nats/ops/gated_delta_rule/wy_fast.py:169-334), chunk_mamba2_bwd src/nats/ops/mamba/chunk.py:112-240, the reversed
 * cumsums chunk.py:318-331 and l2norm_bwd src/nats/ops/mixed_ops/mixed_attn_gdn.py:273-275. */
int natsl_linear_bwd_pre(const void* q, const void* k, const void* d_o, const float* gcs, void* qn, void* kn, float* q_rstd,
                         float* k_rstd, void* dvl, int B, int T, int H, int K, int V, float scale, int use_l2norm,
                         void* stream);
int natsl_linear_bwd_dh(int rule, const void* qn, const void* kn, const void* w, const void* d_o, const void* dvl,
                        const float* gcs, const float* carry, const int32_t* types_i, const int32_t* indices,
                        const int32_t* n_blocks, const float* dht, void* dS_all, void* dvp, float* dh0, int B, int T, int H,
                        int HN, int K, int V, float scale, void* stream);
int natsl_linear_bwd_state(int rule, const void* kn, const void* v, const void* w, const void* u, const void* d_o,
                           const void* dvp, const float* gcs, const void* h, const float* carry, const void* dS_all,
                           const int32_t* types_i, const int32_t* indices, const int32_t* n_blocks,
                           const int32_t* starting_h_idx, void* vp, void* dw, void* dq1, void* dk1, float* dkd, float* scal,
                           float* dnats_lin, int B, int T, int H, int HN, int K, int V, float scale, int invalid_dnats,
                           void* stream);
int natsl_linear_bwd_intra(int rule, const void* qn, const void* kn, const void* v, const void* w, const void* u,
                           const void* vp, const void* dvp, const void* dw, const void* d_o, const void* dq1,
                           const void* dk1, const float* gcs, const void* beta, int beta_dtype, const float* q_rstd,
                           const float* k_rstd, const float* dkd, const int32_t* types_i, void* dq, void* dk, void* dv,
                           float* dbeta, float* dg_tok, float* scal, int B, int T, int H, int HN, int K, int V, float scale,
                           int use_l2norm, void* stream);
int natsl_linear_bwd_dg(const float* dg_tok, const float* scal, const int32_t* types_i, const int32_t* indices,
                        const int32_t* n_blocks, float* dg, int B, int T, int H, int HN, int flags, void* stream);

/* Backward of natsl_norm_gate_mix: dx1, dx2, dg [rows, D] bf16; dxw [rows, 2] fp32 (NULL iff xw is NULL); dw_part
 * [n_part, 2, D] fp32 = per-CTA partial sums of the gradients of w1 and w2 (n_part CTAs are launched, each strides over
 * the rows; the caller adds the partials up).
 * Replaces: the backward of FusedMultiInputRMSNormGated, src/nats/modules/fused_norm_gate.py:353, :657. */
int natsl_norm_gate_mix_bwd(const void* x1, const void* x2, const void* g, const void* xw, int xw_dtype, const void* w1,
                            const void* w2, int w_dtype, const void* dy, void* dx1, void* dx2, void* dg, float* dxw,
                            float* dw_part, int n_part, long rows, int D, float eps, int activation, void* stream);

/* ---- layer steps around the hybrid attention op (bandwidth kernels; bf16 tensors, fp32 math) ------------------- */

/* Short causal depthwise convolution over time + SiLU: x, y [B,T,D]; w [D,W] (W = 4); bias [D] or NULL; silu 0/1.
 * y[b,t,d] = act(bias[d] + sum_j w[d,j] x[b,t-(W-1)+j,d]).  Backward: dx [B,T,D] and per-(batch, token range)
 * partial sums dw_part [B*cdiv(T,span), D, W+1] fp32 of the weight (columns 0..W-1) and bias (column W) gradients,
 * which the caller adds up.
 * Replaces: fla ShortConvolution as used at src/nats/layers/natsl_attn_gdn.py:329-348, 430-447. */
int natsl_short_conv_fwd(const void* x, const void* w, const void* bias, void* y, int B, int T, int D, int W, int silu,
                         void* stream);
int natsl_short_conv_bwd(const void* x, const void* w, const void* bias, const void* dy, void* dx, float* dw_part, int B,
                         int T, int D, int W, int silu, int span, void* stream);

/* RMSNorm over rows of D (64 ... 2048) elements, optionally fused with a residual add in front of it:
 * s = x (+ res), y = s * rsqrt(mean(s^2) + eps) * w; sum_out (or NULL) receives s.  Backward: dx = gradient w.r.t. s
 * (+ dadd, the gradient arriving at s from elsewhere, or NULL) and dw_part [n_part, D] fp32 per-CTA partial sums.
 * Replaces: fla RMSNorm (src/nats/layers/natsl_attn_gdn.py:233-235, 504-505; the fused pre-norm residual at
 * src/nats/models/natsl_attn_gdn/modeling_natsl_attn_gdn.py:138-139). */
int natsl_rmsnorm_fwd(const void* x, const void* res, const void* w, int w_dtype, void* y, void* sum_out, long rows, int D,
                      float eps, void* stream);
int natsl_rmsnorm_bwd(const void* s, const void* w, int w_dtype, const void* dy, const void* dadd, void* dx, float* dw_part,
                      int n_part, long rows, int D, float eps, void* stream);

/* SwiGLU: y = silu(a) * b over n elements (a multiple of 8); backward da, db.
 * Replaces: the activation of fla GatedMLP, src/nats/models/natsl_attn_gdn/modeling_natsl_attn_gdn.py:111-117. */
int natsl_swiglu_fwd(const void* a, const void* b, void* y, long n, void* stream);
int natsl_swiglu_bwd(const void* a, const void* b, const void* dy, void* da, void* db, long n, void* stream);

/* Mean of x [B,T,D] over each block of nbs tokens (the last block may be shorter): y [B,cdiv(T,nbs),D].
 * Replaces: fla mean_pooling, src/nats/layers/natsl_attn_gdn.py:412-416 (src/nats/ops/utils/pooling.py:26-57). */
int natsl_block_mean(const void* x, void* y, int B, int T, int D, int nbs, void* stream);

/* Cross entropy of bf16 logits [rows, vocab] (vocab a multiple of 8), row by row: loss_rows[r] = logsumexp(l) - l[y_r]
 * (0 where y_r == ignore_index), and the logits are overwritten with (softmax(l) - onehot(y_r)) * inv_denom (0 for
 * ignored rows) in bf16 -- the slice-wise loss + gradient of the language-model head.  labels: int64.
 * Replaces: the loss part of FusedLinearCrossEntropyLoss as called at
 * src/nats/models/natsl_attn_gdn/modeling_natsl_attn_gdn.py:474-491. */
int natsl_xent_rows(void* logits, const void* labels, float* loss_rows, long rows, int vocab, long ignore_index,
                    float inv_denom, void* stream);

/* Gated-delta-rule branch forward (prep -> recurrence -> output) that allocates nothing and asks
 * the caller for no intermediate buffers: they live in a fixed NATSL_NOALLOC_SCRATCH_BYTES array
 * inside the library, one per GPU, shared by all calls (overlapping calls on one GPU race; the
 * first call on a device resolves the array's address and should be made outside stream capture).
 * Shapes whose intermediates exceed the array are rejected with NATSL_ERR_TOO_LARGE.
 * For hosts that may not allocate device memory (fixed memory plans, foreign-runtime callbacks).
 * No counterpart in the reference: its Python ops allocate their intermediates through torch. */
#define NATSL_NOALLOC_SCRATCH_BYTES (32u << 20)
int natsl_gdn_fwd_noalloc(const void* q, const void* k, const void* v, const float* g, const void* beta,
                          int beta_dtype, const int32_t* types_i, const int32_t* indices, const int32_t* n_blocks,
                          const float* h0, void* o, float* ht, int B, int T, int H, int HN, int K, int V, int nbs,
                          float scale, int flags, int use_l2norm, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NATSL_B200_H */
