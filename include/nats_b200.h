/* C-ABI of libnats_b200: the NAtS attention hot path (role-masked chunked prefill, KV-cache
 * eviction, decode over the compacted ragged cache) as hand-written CUDA for sm_100a.
 *
 * Conventions
 *   - every pointer named d_* is DEVICE memory owned by the caller; nothing here allocates or frees
 *     device memory (one exception is documented at the entry point that carries static scratch);
 *   - tensors are dense row-major with the shapes given, bf16 unless stated otherwise;
 *   - role codes are uint8: 0 = global, 1 = local, 2 = sliding window (the column order of the
 *     reference's one-hot ``token_states_info``, src/nats/components/cache/nats_chunk_layer_cache.py:188-190);
 *   - ``stream`` is a cudaStream_t passed as void*; work is only enqueued, never synchronised;
 *   - the return value is 0 on success, else one of NATS_ERR_*; nats_b200_last_error() gives the text;
 *   - kernels that wait on hardware barriers bound every wait and report a time-out through the
 *     caller's device status word (0 = ok) instead of spinning forever; a non-zero word also makes every
 *     later prefill launch return at once, so read the word back (after the stream has finished) before
 *     d_o is used, and clear it before the next call;
 *   - the library reads the CURRENT device (SM count, per-device kernel attributes, built-in scratch): make the
 *     device that owns the pointers and the stream current before a call;
 *   - host threads: calls are thread safe once a device has been used; the first call of an entry point on a
 *     device initialises per-device state without locking, so let one host thread make it before others call
 *     concurrently.
 *
 * File paths in the comments below are relative to the reference project root.
 */
#ifndef NATS_B200_H_
#define NATS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NATS_OK               0
#define NATS_ERR_INVALID_ARG  1   /* shape / alignment / null pointer */
#define NATS_ERR_UNSUPPORTED  2   /* valid for the reference, not built here (e.g. head_dim 16 or 32 at this level) */
#define NATS_ERR_CUDA         3   /* a CUDA runtime / driver call failed */
#define NATS_ERR_WORKSPACE    4   /* workspace too small */

#define NATS_ROLE_GLOBAL  0
#define NATS_ROLE_LOCAL   1
#define NATS_ROLE_SLIDING 2

/* Thread-local text of the last error returned on this host thread ("" if none). */
const char* nats_b200_last_error(void);

/* Compile-time facts: "sm_100a", tile sizes, limits.  Never fails. */
const char* nats_b200_build_info(void);

/* ------------------------------------------------------------------------------------------------
 * Role mask metadata.
 * Replaces: generate_hard_seq_masks (src/nats/components/masks/utils.py:81-94) and the sliding-window
 * part of NAtSChunkLayerCache._generate_local_mask (src/nats/components/cache/nats_chunk_layer_cache.py:589-620)
 * -- instead of a dense [N,N] bool mask it produces, per KV chunk c, the last query row that may still
 * see the chunk (INT32_MAX for global chunks and for the last chunk), and per 128-column KV tile the
 * max / min of those limits, which is all the prefill kernel needs to skip or to mask a tile.
 *   d_roles      uint8 [B,Hkv,Nc], Nc = ceil(N/C)
 *   d_lim        int32 [B,Hkv,Nc]            (out)
 *   d_tile_max   int32 [B,Hkv,Nt], Nt = ceil(N/128)   (out)
 *   d_tile_min   int32 [B,Hkv,Nt]            (out)
 *   d_kept_tiles int64 [B,Hkv] or NULL       (out) number of 128x128 (q tile, kv tile) pairs the prefill computes
 */
int nats_b200_role_prep(const uint8_t* d_roles, int B, int Hkv, int N, int C, int SW,
                        int32_t* d_lim, int32_t* d_tile_max, int32_t* d_tile_min, int64_t* d_kept_tiles,
                        void* stream);

/* Bytes of workspace nats_b200_prefill_fwd needs (lim + tile_max + tile_min, 256-byte aligned parts). */
size_t nats_b200_prefill_workspace_bytes(int B, int Hkv, int N, int C);

/* Role-masked causal flash attention of the first prefill call.
 * Replaces: nats_prefill without past (src/nats/models/transformer/triton/nats_flashattn_fwd.py:617-692),
 * nats_chunk_attention forward (src/nats/models/transformer/triton/nats_chunk_attention.py:1154-1185) and the
 * eager pair generate_mask + scaled_dot_product_attention
 * (src/nats/models/transformer/attention/nats_chunk_attention.py:130-142).  The mask is the eager one.
 *   d_q [B,Hq,N,D], d_k,d_v [B,Hkv,N,D], d_o [B,Hq,N,D]  bf16, 16-byte aligned (d_o 32-byte aligned is faster);
 *   D in {64,128,256} (16 and 32 run zero-padded to 64 through the Python wrapper); Hq % Hkv == 0
 *   d_roles uint8 [B,Hkv,ceil(N/C)];  SW % C == 0;  N <= 524288
 *   d_workspace: nats_b200_prefill_workspace_bytes bytes;  d_kept_tiles int64 [B,Hkv] or NULL
 *   d_status: one int32, must be 0 on entry; non-zero afterwards means a bounded wait gave up and d_o is invalid
 */
int nats_b200_prefill_fwd(const void* d_q, const void* d_k, const void* d_v, void* d_o, const uint8_t* d_roles,
                          int B, int Hq, int Hkv, int N, int D, int C, int SW, float sm_scale,
                          void* d_workspace, size_t workspace_bytes, int64_t* d_kept_tiles, int32_t* d_status,
                          void* stream);

/* The forward with the two per-row statistics the reference's training forward hands to its backward
 * (src/nats/models/transformer/triton/nats_chunk_attention.py:319-330): M = m_i + log2(l_i), the base-2 log of the row's
 * sum of exp2(score * sm_scale * log2 e) over its visible keys, and N_VALID_BLOCKS, the number of keys the row sees
 * (the reference sums its mask over the blocks it computes, :131-133, which is that number).
 *   d_lse float [B,Hq,N] (out);  d_n_visible int32 [B,Hq,N] (out);  everything else as nats_b200_prefill_fwd.
 * nats_b200_visible_counts alone: counts from the row limits nats_b200_role_prep made.
 */
int nats_b200_prefill_fwd_stats(const void* d_q, const void* d_k, const void* d_v, void* d_o, const uint8_t* d_roles,
                                int B, int Hq, int Hkv, int N, int D, int C, int SW, float sm_scale,
                                void* d_workspace, size_t workspace_bytes, int64_t* d_kept_tiles,
                                float* d_lse, int32_t* d_n_visible, int32_t* d_status, void* stream);
int nats_b200_visible_counts(const int32_t* d_lim, int B, int Hq, int Hkv, int N, int C, int32_t* d_n_visible, void* stream);

/* Same computation as nats_b200_prefill_fwd for callers that have no way to hand over a workspace: code running
 * where device allocation is off limits -- inside a latency-critical serving loop that must not touch the allocator,
 * in a process whose memory pool is owned and fully handed out by another framework, or in a plugin host that gives
 * a kernel library nothing but its input and output buffers.  (No counterpart in the reference: its Triton entry
 * points allocate freely through PyTorch.)
 * The role metadata goes to a scratch array built into the library: nats_b200_prefill_static_scratch_bytes() bytes
 * (1 MiB) of device memory per GPU that loads the library, held until the process exits.  Shapes whose metadata
 * does not fit -- B*Hkv*(ceil(N/C) + 2*ceil(N/128)) int32 values plus padding -- are rejected with NATS_ERR_WORKSPACE.
 * This call and the library allocate nothing: no cudaMalloc / cudaFree, no allocating library routine.
 * The first call on a device looks up the scratch array's device address (once per device, with that device
 * current); make that first call before any stream capture begins.
 * Every call on a device shares the one array and overwrites all of the metadata it reads, so nothing carries over
 * from the previous call; but two calls that overlap on the GPU (different streams, no ordering between them) race
 * on it -- keep calls on one device ordered.
 */
size_t nats_b200_prefill_static_scratch_bytes(void);
int nats_b200_prefill_fwd_static(const void* d_q, const void* d_k, const void* d_v, void* d_o, const uint8_t* d_roles,
                                 int B, int Hq, int Hkv, int N, int D, int C, int SW, float sm_scale,
                                 int64_t* d_kept_tiles, int32_t* d_status, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Eviction after the first prefill call, in two steps because the size of the compacted cache is data dependent.
 *
 * Step 1 -- keep-set and ranks.  Replaces NAtSChunkLayerCache.get_updated_cache_info
 * (src/nats/components/cache/nats_chunk_layer_cache.py:715-868) and the size bookkeeping of _post_update (:352-358).
 * Kept chunks of a (b,kv-head), in order: every global chunk, then the local chunks after the last global one;
 * an unfinished last chunk (N % C != 0) is never kept.
 *   d_rank         int32 [B,Hkv,Nc]  (out) destination chunk slot counted from the end of the ring; negative for a chunk
 *                                    that is not kept: -1 - (number of kept chunks in front of it)
 *   d_size_global  int64 [B,Hkv]     (out) SW + C * #global
 *   d_size_local   int64 [B,Hkv]     (out) C * #(local after the last global)
 *   d_state        int32 [4]         (in/out) cache state words, all zero before the first call:
 *                                    [0] = max over (b,h) of size_global + size_local (the common tail offset T0),
 *                                    [1],[2] = scratch of the cross-block reduction (zero between calls), [3] reserved
 */
int nats_b200_evict_plan(const uint8_t* d_roles, int B, int Hkv, int N, int C, int SW,
                         int32_t* d_rank, int64_t* d_size_global, int64_t* d_size_local, int32_t* d_state,
                         void* stream);

/* Step 2 -- data movement.  Replaces the first-call cache build of NAtSChunkLayerCache.update (:215-237),
 * move_sliding_window_tokens_to_head (:391-437), merge_local_to_global_caches
 * (src/nats/components/cache/cache_update.py:25-76), the tail zeroing (:361-362) and mask_invalid_tokens (:634-656).
 * Writes, per (b,h):  cache[0,SW) = ring (last SW/C complete chunks; zeros + invalid where the chunk is not a
 * sliding one), cache[SW,len) = kept chunks, cache[T0,T0+r) = the r = N % C tokens of the unfinished chunk with
 * T0 = d_state[0], everything else up to Lcap zero;  valid[] accordingly.
 *   d_k,d_v [B,Hkv,N,D] (source, untouched);  d_cache_k,d_cache_v [B,Hkv,Lcap,D];  d_valid uint8 [B,Hkv,Lcap]
 *   Lcap >= ceil((T0 + r)/C)*C  (the caller reads d_state[0] back, or passes the bound SW + ceil(N/C)*C)
 */
int nats_b200_evict_compact(const void* d_k, const void* d_v, const uint8_t* d_roles, const int32_t* d_rank,
                            const int64_t* d_size_global, const int64_t* d_size_local, const int32_t* d_state,
                            int B, int Hkv, int N, int D, int C, int SW,
                            void* d_cache_k, void* d_cache_v, uint8_t* d_valid, int Lcap, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Multi-token call over an existing compacted cache (segmented prefill, a further turn of a conversation).
 *
 * The reference handles it in NAtSChunkLayerCache.update (:239-256: the new K/V are written behind the unfinished chunk),
 * _generate_mask with _seen_tokens > 0 (:444-511, with _fit_sliding_queue_masks :658-713), its Triton twin nats_prefill
 * with HAS_PAST_INFO (src/nats/models/transformer/triton/nats_flashattn_fwd.py:164-380, 693-722), and the general branch of
 * _post_update (:331-385).  Semantics: the outputs equal those of ONE call over the whole sequence; evicted tokens
 * are exactly the ones no later query may see.
 *
 * Cache layout on entry, per (b,h): [ring SW | kept global [SW,size_global) | kept local [..,len) | gap up to t0 |
 * unfinished chunk [t0, t0+fill)], t0 = d_state[0] (a multiple of C), same for all heads; capacity = rows per head.
 *
 * Step 0 -- append the x_len new tokens at rows [pos, pos+x_len), pos = t0 + fill, and mark them valid.
 */
int nats_b200_cache_append(const void* d_k_new, const void* d_v_new, void* d_cache_k, void* d_cache_v, uint8_t* d_valid,
                           int B, int Hkv, int x_len, int D, int Lcap, int pos, void* stream);

/* Role metadata of such a call (what nats_b200_role_prep is to a first call), over the physical layout as KV sequence of
 * n_kv = t0 + fill + x_len rows; query row i sits at position t0 + fill + i.
 *   d_roles_new  uint8 [B,Hkv,ceil((fill+x_len)/C)]: roles of the chunks from the unfinished one on (what the reference
 *                passes as token_states_info; an unfinished last chunk is marked global by the caller)
 *   d_valid      uint8, valid_stride bytes per (b,h); only the ring flags [0,SW) of each are read
 *   tail         ring write position (sliding_queue_tail) before this call
 *   d_lim int32 [B,Hkv,ceil(n_kv/C)], d_tile_max / d_tile_min int32 [B,Hkv,ceil(n_kv/128)], d_kept_tiles int64 [B,Hkv] or NULL
 */
int nats_b200_role_prep_past(const uint8_t* d_roles_new, const uint8_t* d_valid, const int64_t* d_size_global,
                             const int64_t* d_size_local, int B, int Hkv, int x_len, int C, int SW, int valid_stride,
                             int t0, int fill, int tail, int32_t* d_lim, int32_t* d_tile_max, int32_t* d_tile_min,
                             int64_t* d_kept_tiles, void* stream);

size_t nats_b200_prefill_past_workspace_bytes(int B, int Hkv, int n_kv, int C);

/* Step 1 -- attention of the new queries over cache + new tokens (the new tokens already appended by step 0).
 *   d_q [B,Hq,x_len,D], d_o [B,Hq,x_len,D]; d_cache_k/v [B,Hkv,cache_capacity,D]; the other arguments as above;
 *   d_workspace: nats_b200_prefill_past_workspace_bytes(B,Hkv,t0+fill+x_len,C) bytes; d_status as in nats_b200_prefill_fwd.
 *   Rows of the gap [len, t0) must hold finite numbers (this library keeps them zero).
 */
int nats_b200_prefill_past_fwd(const void* d_q, const void* d_cache_k, const void* d_cache_v, void* d_o,
                               const uint8_t* d_roles_new, const uint8_t* d_valid, int valid_stride,
                               const int64_t* d_size_global, const int64_t* d_size_local, int B, int Hq, int Hkv, int x_len, int D, int C, int SW,
                               int cache_capacity, int t0, int fill, int tail, float sm_scale,
                               void* d_workspace, size_t workspace_bytes, int64_t* d_kept_tiles, int32_t* d_status,
                               void* stream);

/* Step 2 -- keep-set of the call's n_tokens = fill + x_len tokens (get_updated_cache_info :715-868 with a non-empty cache).
 * A global chunk among the completed chunks drops the kept locals in front of it.
 *   d_rank int32 [B,Hkv,ceil(n_tokens/C)] (out): destination slot of a kept chunk counted from d_base, negative otherwise
 *                                          (encoded as for nats_b200_evict_plan)
 *   d_base int32 [B,Hkv] (out): chunk slot (position / C) the first kept chunk goes to = what the cache keeps from before
 *   d_size_global / d_size_local (in/out);  d_state as in nats_b200_evict_plan
 */
int nats_b200_evict_plan_past(const uint8_t* d_roles_new, int B, int Hkv, int n_tokens, int C, int SW,
                              int32_t* d_rank, int32_t* d_base, int64_t* d_size_global, int64_t* d_size_local,
                              int32_t* d_state, void* stream);

/* Step 3 -- data movement, out of place: old cache (with the appended tokens) -> new cache buffer.  Ring slots behind
 * tail_old receive the last min(#completed chunks, SW/C) chunks (move_sliding_window_tokens_to_head :391-437), the
 * others are copied; [SW, base*C) is copied; kept chunks go to [base*C, len); the new unfinished chunk to
 * [T0', T0'+r), T0' = d_state[0]; everything else up to Lcap is zero; flags accordingly.  (The reference moves chunks
 * inside one buffer after cloning the sources, cache_update.py:65-74.)
 *   t0_old: tail offset before the call (the tokens of the call sit at old rows [t0_old, t0_old + n_tokens))
 *   Lcap >= ceil((T0' + r)/C)*C
 */
int nats_b200_evict_compact_past(const void* d_old_k, const void* d_old_v, const uint8_t* d_old_valid, int old_capacity,
                                 const uint8_t* d_roles_new, const int32_t* d_rank, const int32_t* d_base,
                                 const int64_t* d_size_global, const int64_t* d_size_local, const int32_t* d_state,
                                 int B, int Hkv, int n_tokens, int D, int C, int SW, int t0_old, int tail_old,
                                 void* d_cache_k, void* d_cache_v, uint8_t* d_valid, int Lcap, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Decode over the compacted ragged cache.
 *
 * Logical sequence a query of (b,h) attends to (the reference's ``valid_tokens[:, :, :n_ctx_data+1]``,
 * src/nats/components/cache/nats_chunk_layer_cache.py:622-632): the valid ring slots [0,SW), the kept tokens
 * [SW,len), the ``fill`` tokens of the unfinished chunk at [T0,T0+fill) and the new token itself.
 */
size_t nats_b200_decode_workspace_bytes(int B, int Hq, int Hkv, int D, int max_len);

/* One decode step: append + attention.  Replaces NAtSChunkLayerCache.update for x_len == 1 (:239-256),
 * _generate_mask_one_step (:622-632) and repeat_kv + scaled_dot_product_attention over the padded cache
 * (src/nats/models/transformer/attention/nats_chunk_attention.py:131-142).
 *   d_q [B,Hq,1,D]; d_k_new,d_v_new [B,Hkv,1,D] (written to cache position T0+fill, valid set); d_o [B,Hq,1,D]
 *   d_state[0] = T0;  fill = tokens already in the unfinished chunk (host knows it);  T0+fill < Lcap
 *   max_len_bound: host upper bound of T0 (sizes the grid; no host sync needed)
 *   d_workspace: nats_b200_decode_workspace_bytes(B,Hq,Hkv,D,max_len_bound+C) bytes; must be zero on first use
 *   (the kernel leaves its counters zero again);  D in {64,128};  Hq/Hkv from 1 to 8
 */
int nats_b200_decode_fwd(const void* d_q, const void* d_k_new, const void* d_v_new, void* d_o,
                         void* d_cache_k, void* d_cache_v, uint8_t* d_valid, int Lcap,
                         const int64_t* d_size_global, const int64_t* d_size_local, const int32_t* d_state,
                         int fill, int max_len_bound,
                         int B, int Hq, int Hkv, int D, int C, int SW, float sm_scale,
                         void* d_workspace, size_t workspace_bytes, void* stream);

/* Placement of a chunk that has just been completed by a decode step.  Replaces the x_len == 1 branch of
 * NAtSChunkLayerCache._post_update (:270-330, 356-371) incl. the ring write of move_sliding_window_tokens_to_head.
 *   d_roles uint8 [B,Hkv]: role of the completed chunk;  tail: ring write position before this call (host tracks it)
 *   global -> chunk to size_global, size_global += C, size_local = 0;  local -> chunk to size_global+size_local,
 *   size_local += C;  sliding -> ring only.  d_state[0] becomes the new maximum length (it can shrink: a global
 *   chunk drops the locals before it).  The reference's joint "every head is sliding" early exit (:283-288)
 *   changes nothing but the ring, which is what the per-head rule already does.
 */
int nats_b200_decode_place(const uint8_t* d_roles, void* d_cache_k, void* d_cache_v, uint8_t* d_valid, int Lcap,
                           int64_t* d_size_global, int64_t* d_size_local, int32_t* d_state,
                           int tail, int B, int Hkv, int D, int C, int SW, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Caller-side helper: rotary position embedding fused with the head split, in front of the attention kernels.
 * Replaces, in the reference's attention modules and Hugging Face patches, the chain
 * ``proj(x).view(B,N,H,D).transpose(1,2)`` + ``apply_rotary_pos_emb`` + ``.contiguous()``
 * (src/nats/models/transformer/hf/llama_nats_chunk.py:187-192,227,246; attention/base_attention.py:153-161).
 *   d_q_in [B,N,Hq*D], d_k_in,d_v_in [B,N,Hkv*D] bf16, rows *_token_stride elements apart (so a fused qkv projection works);
 *   d_cos,d_sin bf16 [B or 1, N, D] (cos_batch_stride 0 when shared), the layout of Hugging Face rotary embeddings;
 *   d_q_out [B,Hq,N,D], d_k_out,d_v_out [B,Hkv,N,D] bf16.  rotate_half convention: pairs (i, i + D/2).
 *   Products and sum are rounded to bf16 one by one, which reproduces the element-wise bf16 chain bit for bit.
 */
int nats_b200_rope_split_heads(const void* d_q_in, const void* d_k_in, const void* d_v_in, long long q_token_stride,
                               long long k_token_stride, long long v_token_stride, const void* d_cos, const void* d_sin,
                               long long cos_batch_stride, void* d_q_out, void* d_k_out, void* d_v_out,
                               int B, int N, int Hq, int Hkv, int D, void* stream);

/* ------------------------------------------------------------------------------------------------
 * The decode step with static launch parameters, for callers that record the step once (a CUDA graph) and replay it.
 * nats_b200_decode_fwd / nats_b200_decode_place take the number of tokens in the unfinished chunk and the ring position by
 * value, so a recorded launch would freeze them; here they live in the state words: d_state is int32[8] with
 * [4] = tokens in the unfinished chunk, [5] = ring write position ([0..3] as before).  One step is
 *     nats_b200_decode_step_fwd(...)      append + attention (reads [4])
 *     nats_b200_decode_step_place(...)    placement if this token completed a chunk (d_roles: its role per (b,kv-head),
 *                                         ignored otherwise), then [4], [5] advance
 * max_len_bound must bound d_state[0] for every replay (the cache capacity minus a chunk does); Lcap must hold
 * max_len_bound + C rows; the workspace is sized for max_len_bound + C.
 */
int nats_b200_decode_step_fwd(const void* d_q, const void* d_k_new, const void* d_v_new, void* d_o,
                              void* d_cache_k, void* d_cache_v, uint8_t* d_valid, int Lcap,
                              const int64_t* d_size_global, const int64_t* d_size_local, const int32_t* d_state,
                              int max_len_bound, int B, int Hq, int Hkv, int D, int C, int SW, float sm_scale,
                              void* d_workspace, size_t workspace_bytes, void* stream);
int nats_b200_decode_step_place(const uint8_t* d_roles, void* d_cache_k, void* d_cache_v, uint8_t* d_valid, int Lcap,
                                int64_t* d_size_global, int64_t* d_size_local, int32_t* d_state,
                                int B, int Hkv, int D, int C, int SW, void* stream);

#ifdef __cplusplus
}
#endif
#endif  /* NATS_B200_H_ */
