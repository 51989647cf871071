/*
 * ucmr.h - C ABI of the B200 (sm_100a) hash-code top-k block retrieval library.
 *
 * Every entry point takes raw device pointers, sizes and an explicit CUDA
 * stream (a cudaStream_t passed as void*; NULL = legacy default stream),
 * launches asynchronously on that stream, allocates nothing and returns an
 * int status (0 = ok, negative = error, see UCMR_ERR_*).  Nothing here throws
 * or aborts.  The caller owns all buffers.
 *
 * State kept by the library, all of it process-wide and none of it per call:
 *   - ucmr_hamming_topk_static uses one fixed device array per GPU and a
 *     mutex-guarded table of its per-device addresses (see its declaration);
 *   - the tuning switches UCMR_PDL, UCMR_SCAN, UCMR_SEL_CLUSTER,
 *     UCMR_FORCE_SIMT_ENCODE, UCMR_STEP_ENCODE, UCMR_FUSED_SELECT,
 *     UCMR_SMALL_BLOCKS and UCMR_ROWS_KERNEL are environment variables read
 *     once, on the first call that consults them, and cached for the life of
 *     the process;
 *   - the text of the last CUDA error is kept per host thread.
 * Everything else (scores between two kernels, work counters, device status)
 * lives in the caller's workspace.
 *
 * Each declaration names the interface of the reference project
 * (ModelEngine-Group/unified-cache-management, paths relative to its root) that it
 * stands in for.
 *
 * Data layouts
 *   codes        uint32 [NB, BS, Hkv, W]   paged hash-code cache; bit b of word w is projection
 *                                          column 32*w+b (little-endian view of the reference's
 *                                          LSB-first uint8 packing, hash_encoder.py:445-448)
 *   q_codes      uint32 [B, Hq, W]         one code per query head; G = Hq/Hkv heads share a kv head
 *   block_table  int32  [B, max_blocks]    logical block -> physical block (row stride in elements)
 *   seq_lens     int32  [B]                tokens per request
 */
#ifndef UCMR_H_
#define UCMR_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define UCMR_VERSION 100

#define UCMR_OK 0
#define UCMR_ERR_BAD_ARG (-1)     /* null pointer, negative size, k > max_blocks, ...            */
#define UCMR_ERR_UNSUPPORTED (-2) /* shape outside what the kernels are built for                */
#define UCMR_ERR_LAUNCH (-3)      /* the CUDA runtime refused the launch (see ucmr_last_cuda_error) */
#define UCMR_ERR_DEVICE (-4)      /* a kernel recorded a problem in the workspace status word     */
#define UCMR_ERR_WORKSPACE (-5)   /* workspace missing or too small                               */

/* Bits of the device status word (first int32 of a workspace). */
#define UCMR_DEV_BAD_BLOCK_ID 1 /* a block-table entry or selected id was outside [0, NB)        */
#define UCMR_DEV_WAIT_TIMEOUT 2 /* a bounded wait inside a kernel gave up                        */
#define UCMR_DEV_BAD_SLOT 4     /* reserved                                                      */

#define UCMR_REDUCE_MIN 0 /* block score = min over tokens (reference behaviour)                 */
#define UCMR_REDUCE_SUM 1 /* block score = sum over tokens (mean * BS * G)                       */
/* May be OR-ed into reduce_mode: the caller guarantees that seq_lens and block_table are NOT written by any
 * kernel that may still be in flight on the stream when this call's scan starts - not only the kernel right
 * before it: kernels that release their successor early (this library's scan and decode-step encode do, and so
 * may a caller's own programmatic-dependent-launch kernels) let a flagged scan become resident while a kernel
 * two or more positions earlier is still running.  True in a decode loop, where both arrays are prepared at
 * the start of the step and only read afterwards.  The scan then resolves its first work items (prefix sums,
 * block-table loads) while the earlier kernels drain instead of after them.                              */
#define UCMR_FLAG_INPUTS_STABLE 0x100
/* May be OR-ed in together with UCMR_FLAG_INPUTS_STABLE: of the code-cache blocks this call scans, the kernels that
 * may still be in flight (same reading as above) write at most the block that holds the last token (seq_len - 1)
 * of each request.  True for a decode step, where the only writer is the encode of the one new key per request.
 * The scan then starts copying its first blocks - never a request's last one - before those kernels have finished;
 * query codes are read and scores written only afterwards.  Ignored by the kernels that have no use for it.   */
#define UCMR_FLAG_CACHE_APPEND_ONLY 0x200

#define UCMR_MAX_MUST_SELECT 16
#define UCMR_WORKSPACE_HEADER_BYTES 256

int ucmr_version(void);
const char* ucmr_status_string(int status);
/* Text of the last CUDA runtime error seen by this thread inside the library ("" if none). */
const char* ucmr_last_cuda_error(void);

/* Step timeline, for a library built with -DUCMR_TRACE (python -m unified_cache_management_b200.build --trace);
 * any other build returns UCMR_ERR_UNSUPPORTED.  Thread 0 of CTA 0 of the decode-step kernels stores the device's
 * nanosecond timer at numbered points; this copies the table of one kernel (UCMR_TRACE_SLOTS values, as left by the
 * kernel's last launch; a synchronising device-to-host copy) to `stamps`.
 *   UCMR_TRACE_ENCODE (decode-step encode): 0 entry, 1 dependency wait passed, 2 inputs staged, 3 end
 *   UCMR_TRACE_SCAN (staged Hamming scan):  0 entry, 1 work items counted, 2 first item resolved, 3 first copy issued,
 *                                           4 dependency wait passed, 5 first block landed, 6 first item scored,
 *                                           7 this warp out of items
 *   UCMR_TRACE_SELECT (selection kernel):   0 entry, 1 dependency wait passed, 2 keys staged, 3 threshold known,
 *                                           4 chosen blocks listed, 5 end; peer exchange: 6 records fenced (CTA 0),
 *                                           7 step number published (the launch's last CTA); merge kernel (same
 *                                           table): 8 entry, 9 every rank's step number seen, 10 merged; over all CTAs of the
 *                                           selection, the latest: 11 records stored, 12 records fenced, 13 wait passed
 * No reference counterpart (the reference times its kernels from the host). */
#define UCMR_TRACE_SLOTS 32
#define UCMR_TRACE_ENCODE 0
#define UCMR_TRACE_SCAN 1
#define UCMR_TRACE_SELECT 2
int ucmr_trace_read(int unit, unsigned long long* stamps);

/* ------------------------------------------------------------------------------------------
 * (1) Hash encode.  Replaces HashEncoder.compute_hash / triton_hash_code
 *     (ucm/sparse/gsa_on_device/hash_encoder.py:37-134, 450-507; CPU form torch_hash_code :359-370).
 *     codes_out[r, w] bit b = (sum_k x[r,k] * R[k, 32w+b] > 0), bf16 inputs, float32 accumulate.
 *     x: bf16 [rows, in_dim], row stride in elements (multiple of 8); R: bf16 [in_dim, hash_bits]
 *     row-major.  in_dim and hash_bits are 128 on the tensor-core path; other multiples of 32 up to
 *     1024 run on a slower CUDA-core path.  status_word (device int32*, may be NULL) receives
 *     UCMR_DEV_WAIT_TIMEOUT if a bounded wait inside the tensor-core kernel gave up.
 * ------------------------------------------------------------------------------------------ */
int ucmr_hash_encode(const void* x, int64_t rows, int64_t row_stride, const void* R, int in_dim,
                     int hash_bits, uint32_t* codes_out, int32_t* status_word, void* stream);

/*     Query path of GSAOnDevice.hash_code (ucm/sparse/gsa_on_device/gsa_on_device.py:396-412):
 *     q bf16 [T, Hq, in_dim] (strides in elements).  group_mean = G > 1 first averages each run of
 *     G consecutive heads (float32 sum, one rounding to bf16, as torch's bf16 mean does) and emits
 *     Hq/G codes per token; group_mean = 1 emits one code per head.  codes_out [T, Hq/G, W].      */
int ucmr_hash_encode_query(const void* q, int64_t T, int Hq, int64_t stride_t, int64_t stride_h,
                           int group_mean, const void* R, int in_dim, int hash_bits,
                           uint32_t* codes_out, int32_t* status_word, void* stream);

/*     Replaces HashEncoder.compute_hash_and_cache / fused_hash_and_cache_kernel
 *     (hash_encoder.py:263-356, 548-662): encode x[T,H,in_dim] and write the codes of token t to
 *     slot slot_mapping[t] (= block*BS + row) of cache[NB,BS,H,W].  Slots < 0 or >= NB*BS are
 *     skipped (hash_encoder.py:340-344).  slot_mapping is int64 when slot_is_int64 != 0, else int32. */
int ucmr_hash_encode_and_cache(const void* x, int64_t T, int H, int64_t stride_t, int64_t stride_h,
                               const void* R, int in_dim, int hash_bits, const void* slot_mapping,
                               int slot_is_int64, uint32_t* cache, int64_t NB, int BS,
                               int32_t* status_word, void* stream);

/*     Re-hash of key blocks that already sit in the paged K cache (a prefix-cache hit): stands in for
 *     the torch gather kv_cache[0][0][prefix_block_ids] followed by compute_hash_and_cache with the
 *     prefix slot mapping (ucm/sparse/gsa_on_device/gsa_on_device.py:574-588), without the gathered
 *     copy.  k_cache is bf16 [NB, BS, H, in_dim] with strides in elements (stride_block between
 *     blocks, stride_t between tokens, stride_h between heads).  For every listed block i the codes of
 *     its first block_tokens[i] tokens (all BS when block_tokens is NULL) are written to block
 *     block_ids[i] of cache [NB_codes, BS, H, W] - the code cache uses the K cache's block ids.  Ids
 *     outside [0, NB) are flagged in status_word and skipped.                                        */
int ucmr_hash_encode_blocks(const void* k_cache, int64_t NB, int BS, int H, int64_t stride_block,
                            int64_t stride_t, int64_t stride_h, const int32_t* block_ids,
                            const int32_t* block_tokens, int64_t n_blocks, const void* R, int in_dim,
                            int hash_bits, uint32_t* cache, int64_t NB_codes, int32_t* status_word,
                            void* stream);

/*     Variants for code caches whose (token, head) row holds more than one code: the row has
 *     row_words 32-bit words and this call's code goes to words [word_offset, word_offset +
 *     hash_bits/32).  MLA keeps a 512-bit code of the latent vector and a 64-bit code of the rope part
 *     side by side in rows of 18 words (the reference hashes them with two encoders and joins them with
 *     vLLM's concat_and_cache_mla, gsa_on_device.py:426-455): two calls, word_offset 0 and 16.        */
int ucmr_hash_encode_and_cache_at(const void* x, int64_t T, int H, int64_t stride_t, int64_t stride_h,
                                  const void* R, int in_dim, int hash_bits, const void* slot_mapping,
                                  int slot_is_int64, uint32_t* cache, int64_t NB, int BS, int row_words,
                                  int word_offset, int32_t* status_word, void* stream);
int ucmr_hash_encode_blocks_at(const void* k_cache, int64_t NB, int BS, int H, int64_t stride_block,
                               int64_t stride_t, int64_t stride_h, const int32_t* block_ids,
                               const int32_t* block_tokens, int64_t n_blocks, const void* R, int in_dim,
                               int hash_bits, uint32_t* cache, int64_t NB_codes, int row_words,
                               int word_offset, int32_t* status_word, void* stream);

/*     The two encodes of one decode step in a single launch: the step's queries (as
 *     ucmr_hash_encode_query, hash_code at gsa_on_device.py:396-412) and its new key rows (as
 *     ucmr_hash_encode_and_cache, cache_k_hash_gqa_cuda at gsa_on_device.py:564-573).
 *     q and k (a few hundred KB per step) may also point to page-locked host memory that the
 *     device can address: the kernel then fetches them across the bus itself, which saves the
 *     caller a separate host-to-device copy per step.                                              */
int ucmr_hash_encode_decode_step(const void* q, int64_t Tq, int Hq, int64_t q_stride_t,
                                 int64_t q_stride_h, int group_mean, uint32_t* q_codes_out,
                                 const void* k, int64_t Tk, int Hk, int64_t k_stride_t,
                                 int64_t k_stride_h, const void* slot_mapping, int slot_is_int64,
                                 uint32_t* cache, int64_t NB, int BS, const void* R, int in_dim,
                                 int hash_bits, int32_t* status_word, void* stream);

/* ------------------------------------------------------------------------------------------
 * Workspace.  Holds the device status word and the block scores between the scan and the
 * selection kernel.  Clear it once with ucmr_workspace_init after allocating it; the status word
 * is sticky until the next init.  ucmr_workspace_status copies the word to the host and waits for
 * the stream.
 * ------------------------------------------------------------------------------------------ */
size_t ucmr_hamming_topk_workspace_bytes(int B, int Hkv, int max_blocks, int reduce_kvhead);
int ucmr_workspace_init(void* workspace, size_t bytes, void* stream);
int ucmr_workspace_status(const void* workspace, int* host_status, void* stream);

/* ------------------------------------------------------------------------------------------
 * (2)+(3) Hamming scan + per-request exact top-k.  Replaces cuda_hamming_topk
 *     (ucm/sparse/gsa_on_device/hamming_topk.py:15-54) = hamming.hamming_score
 *     (ucm/sparse/gsa_on_device/csrc/cuda/ham_dist/paged_ham_dist_mla.cu:332-443, kernel :111-248)
 *     followed by torch.min / topk / sort / gather, and update_seq_lens (hamming_topk.py:7-12).
 *
 *     Token distance d[b,h,p] = sum_{g<G} popcount(codes[..p.., h, :] ^ q_codes[b, h*G+g, :]).
 *     Block score S[b,h,j] = min or sum of d over the valid tokens of logical block j;
 *     reduce_kvhead != 0 further combines the kv heads with the same operator (Hout = 1),
 *     otherwise Hout = Hkv.  Forced blocks: entries of must_select (HOST array; >= 0 counts from
 *     the start, < 0 from the request's block count) and every block overlapping [0, sink_tokens)
 *     or [seq_len - recent_tokens, seq_len).  Forced blocks count toward k.  Selection = first k
 *     blocks under the order (forced first, then score ascending, ties by lower block id; blocks
 *     past the request's length last); the k results are written in ascending logical order.
 *
 *     k_per_request (device int32 [B], may be NULL): row b uses min(k_per_request[b], k) and pads
 *     with logical -1 / physical 0.  request_mask (device uint8 [B], may be NULL): rows with 0 are
 *     not retrieved; they get logical 0..k-1, the head of their own block table and their own
 *     seq_len.
 *
 *     Outputs (device; any of out_logical / out_scores / out_valid_count / out_new_seq_lens may
 *     be NULL): out_physical, out_logical, out_scores int32 [B, Hout, k]; out_valid_count,
 *     out_new_seq_lens int32 [B].  out_scores holds the raw block score (-1 for padding).
 *     out_physical may be page-locked host memory (the ids are then on the host when the stream
 *     has drained, without a separate device-to-host copy).
 * ------------------------------------------------------------------------------------------ */
int ucmr_hamming_topk(const uint32_t* codes, int64_t NB, int BS, int Hkv, int W,
                      const uint32_t* q_codes, int Hq, const int32_t* block_table, int max_blocks,
                      int64_t block_table_stride, const int32_t* seq_lens, int B, int k,
                      const int32_t* k_per_request, const uint8_t* request_mask, int reduce_mode,
                      int reduce_kvhead, const int32_t* must_select, int n_must, int sink_tokens,
                      int recent_tokens, int32_t* out_physical, int32_t* out_logical,
                      int32_t* out_scores, int32_t* out_valid_count, int32_t* out_new_seq_lens,
                      void* workspace, size_t workspace_bytes, void* stream);

/*     Same retrieval for callers that cannot provide a workspace (no counterpart in the reference:
 *     its op allocates its output with torch on every call).  An engine that has already handed all free
 *     GPU memory to its KV-cache pool, or a hook running inside its forward pass, has nowhere to
 *     allocate from; this variant keeps the scan -> selection scores in a fixed device array that is
 *     part of the library image, so it calls no cudaMalloc / cudaFree and no allocating library routine.
 *     Limits and rules:
 *       - the array is ucmr_static_workspace_capacity() bytes (4 MiB) on every GPU that loads the
 *         library, held until the process exits; shapes whose workspace (see
 *         ucmr_hamming_topk_workspace_bytes) is larger are refused with UCMR_ERR_WORKSPACE;
 *       - the first call on each device resolves the array's device address (with that device current);
 *         make that first call outside any stream capture;
 *       - all calls on a device share the one array: calls that may overlap on the GPU (different
 *         streams, no ordering between them) race on it and must be serialised by the caller;
 *       - the array keeps the previous call's contents; each call clears the header it needs to start at
 *         zero.  The status word is therefore not sticky here and cannot be read back.
 *     Arguments and outputs are those of ucmr_hamming_topk without the workspace pair.              */
size_t ucmr_static_workspace_capacity(void);
int ucmr_hamming_topk_static(const uint32_t* codes, int64_t NB, int BS, int Hkv, int W,
                             const uint32_t* q_codes, int Hq, const int32_t* block_table,
                             int max_blocks, int64_t block_table_stride, const int32_t* seq_lens, int B,
                             int k, const int32_t* k_per_request, const uint8_t* request_mask,
                             int reduce_mode, int reduce_kvhead, const int32_t* must_select, int n_must,
                             int sink_tokens, int recent_tokens, int32_t* out_physical,
                             int32_t* out_logical, int32_t* out_scores, int32_t* out_valid_count,
                             int32_t* out_new_seq_lens, void* stream);

/*     Scan only: block scores int32 [B, Hout, max_blocks] (-1 past the request's length).
 *     Same kernel as the first half of ucmr_hamming_topk.  status_word (device int32*, may be
 *     NULL) receives UCMR_DEV_* bits.                                                             */
int ucmr_block_scores(const uint32_t* codes, int64_t NB, int BS, int Hkv, int W,
                      const uint32_t* q_codes, int Hq, const int32_t* block_table, int max_blocks,
                      int64_t block_table_stride, const int32_t* seq_lens, int B, int reduce_mode,
                      int reduce_kvhead, int32_t* out_scores, int32_t* status_word, void* stream);

/*     Per-token output of the reference op hamming.hamming_score
 *     (ucm/sparse/gsa_on_device/csrc/cuda/ham_dist/cpy/hamming.cpp:5, paged_ham_dist_mla.cu:189-247):
 *     fp16 [B, reduce_kvhead ? 1 : Hkv, max_blocks*BS]; positions < sink or in
 *     [seq_len-recent, seq_len) -> 0, positions >= seq_len -> +inf, min over kv heads when
 *     reduce_kvhead.  Kept for callers of the old op; the retrieval path never materialises it.  */
int ucmr_hamming_score(const uint32_t* codes, int64_t NB, int BS, int Hkv, int W,
                       const uint32_t* q_codes, int Hq, const int32_t* block_table, int max_blocks,
                       int64_t block_table_stride, const int32_t* seq_lens, int B, int sink_tokens,
                       int recent_tokens, int reduce_kvhead, void* out_fp16, void* stream);

/*     update_seq_lens (hamming_topk.py:7-12): out[b] = seq - ceil(max(seq - topk_tokens, 0)/BS)*BS. */
int ucmr_update_seq_lens(const int32_t* seq_lens, int B, int topk_tokens, int BS, int32_t* out,
                         void* stream);

/* ------------------------------------------------------------------------------------------
 * Sequence-sharded retrieval (no counterpart in the reference, whose plugin is not
 * context-parallel aware; the per-shard computation is the same scan + selection as above).
 *     ucmr_topk_candidates: this shard holds logical blocks [block_id_offset, block_id_offset +
 *     ceil(seq_lens_local[b]/BS)) of request b.  Writes its best k blocks as records
 *     (float32 score, int32 global block id) [B, Hout, k], ascending id, padding = (+inf, -1).
 *     score = block score * score_scale; forced blocks (decided from the global block index and
 *     seq_lens_global) carry -1.0 so that they survive the merge.
 *     ucmr_merge_topk: cand_* [R, B, Hout, kl] gathered in ascending shard order -> first k under
 *     (score, id), written in ascending id order to out_* [B, Hout, k]; padding = (+inf, -1).
 *     rank_stride = distance in elements between two shards' arrays (0 = dense, B*Hout*kl), so that
 *     scores and ids may sit side by side in one all-gathered buffer.
 * ------------------------------------------------------------------------------------------ */
int ucmr_topk_candidates(const uint32_t* codes, int64_t NB, int BS, int Hkv, int W,
                         const uint32_t* q_codes, int Hq, const int32_t* block_table,
                         int max_blocks, int64_t block_table_stride,
                         const int32_t* seq_lens_local, const int32_t* seq_lens_global, int B,
                         int k, int block_id_offset, float score_scale, int reduce_mode,
                         int reduce_kvhead, const int32_t* must_select, int n_must,
                         int sink_tokens, int recent_tokens, float* cand_scores,
                         int32_t* cand_ids, void* workspace, size_t workspace_bytes, void* stream);

int ucmr_merge_topk(const float* cand_scores, const int32_t* cand_ids, int64_t rank_stride, int R, int B,
                    int Hout, int kl, int k, float* out_scores, int32_t* out_ids, void* stream);

/* ------------------------------------------------------------------------------------------
 * (4) Paged-KV gather.  out[b, i*BS + t, h, :] = pool[sel[b,(h),i], t, h, :] for the K pool and
 *     the V pool (either may be NULL).  Device-to-device form of the reference's
 *     kv_cache[block_ids] (ucm/sparse/gsa_on_device/gsa_on_device.py:579-580) and of the
 *     scattered-blocks-to-one-buffer copy CudaCopyKernel (ucm/shared/trans/cuda/cuda_sm_kernel.cu:66-78).
 *     block_bytes = BS*Hkv*D*elem_size (multiple of 16).  per_head = 0: sel is int32 [B, k] and
 *     whole blocks are copied.  per_head != 0: sel is int32 [B, Hkv, k] and each kv head takes its
 *     own blocks (row_bytes = D*elem_size, multiple of 16).  Ids outside [0, NB) are skipped and
 *     flagged in status_word (device int32*, may be NULL).
 * ------------------------------------------------------------------------------------------ */
int ucmr_gather_kv(const void* k_pool, const void* v_pool, int64_t NB, int64_t block_bytes,
                   const int32_t* sel, int B, int k, int per_head, int BS, int Hkv,
                   int64_t row_bytes, void* out_k, void* out_v, int32_t* status_word,
                   void* stream);

/* ---------------------------------------------------------------------------------------------
 *  Sequence-sharded retrieval without a collective call: the local selection writes its records
 *  straight into every rank's gather buffer over peer memory (NVLink) and publishes a step number;
 *  the merge waits for the step number of every rank, then merges.  One process per GPU; the buffers
 *  are peer-mapped by the caller (symmetric memory / IPC).
 *
 *  ucmr_topk_candidates_p2p: as ucmr_topk_candidates, but the records go to peer_scores[r] /
 *     peer_ids[r] for r < n_peers (<= 8; HOST arrays of device pointers, each pointing at THIS rank's
 *     [B, Hout, k] slice of rank r's buffer - the own buffer included), and when the launch's last CTA
 *     is done `seq` is stored (release, system scope) to *peer_flags[r] (this rank's flag word on rank
 *     r).  Needs k > 0.  Uses the workspace header as an arrival counter.
 *  ucmr_merge_topk_wait: as ucmr_merge_topk, after waiting (at most 1 s, then UCMR_DEV_WAIT_TIMEOUT in
 *     status_word and the output left as padding) until flags[r] == seq for every r < R.
 *  A step's records must not be overwritten while a slower rank still merges them: alternate between
 *  two buffers (and two flag arrays) by the parity of seq.
 * ------------------------------------------------------------------------------------------ */
int ucmr_topk_candidates_p2p(const uint32_t* codes, int64_t NB, int BS, int Hkv, int W,
                             const uint32_t* q_codes, int Hq, const int32_t* block_table, int max_blocks,
                             int64_t block_table_stride, const int32_t* seq_lens_local,
                             const int32_t* seq_lens_global, int B, int k, int block_id_offset,
                             float score_scale, int reduce_mode, int reduce_kvhead,
                             const int32_t* must_select, int n_must, int sink_tokens, int recent_tokens,
                             float* const* peer_scores, int32_t* const* peer_ids, int32_t* const* peer_flags,
                             int n_peers, int seq, void* workspace, size_t workspace_bytes, void* stream);
int ucmr_merge_topk_wait(const float* cand_scores, const int32_t* cand_ids, int64_t rank_stride, int R, int B,
                         int Hout, int kl, int k, float* out_scores, int32_t* out_ids, const int32_t* flags,
                         int seq, int32_t* status_word, void* stream);

/*  Replay-safe forms of the two calls above.  `seq` above is a by-value argument: a launch captured in a CUDA
 *  graph publishes and waits for the SAME step number on every replay, so after the first replay nothing waits any
 *  more and a rank may merge records that a faster peer is already overwriting.  Use these forms whenever the step is
 *  captured.  The step number lives in a device word of this rank: both kernels read s = *step_word + 1, the
 *  selection publishes s, the merge waits for s and its last CTA stores s back to *step_word.  The parity of s picks
 *  one of two pointer sets, so the captured launch alternates buffers by itself.
 *     ucmr_topk_candidates_p2p_step: peer_scores / peer_ids / peer_flags hold 2 * n_peers entries, the n_peers
 *        pointers of parity 0 followed by those of parity 1.
 *     ucmr_merge_topk_wait_step: cand_* and flags point at parity 0; parity 1 lies parity_stride (elements of the
 *        records arrays) resp. flags_parity_stride (flag words) further.  arrive_word is a device int32 that is
 *        zero between launches.  *step_word and *arrive_word start at 0; the first step is number 1.
 *  The merge of a step and the selection of the next step must be ordered on one stream (they are in a decode
 *  loop); no counterpart in the reference.                                                                    */
int ucmr_topk_candidates_p2p_step(const uint32_t* codes, int64_t NB, int BS, int Hkv, int W,
                                  const uint32_t* q_codes, int Hq, const int32_t* block_table, int max_blocks,
                                  int64_t block_table_stride, const int32_t* seq_lens_local,
                                  const int32_t* seq_lens_global, int B, int k, int block_id_offset,
                                  float score_scale, int reduce_mode, int reduce_kvhead,
                                  const int32_t* must_select, int n_must, int sink_tokens, int recent_tokens,
                                  float* const* peer_scores, int32_t* const* peer_ids, int32_t* const* peer_flags,
                                  int n_peers, const int32_t* step_word, void* workspace, size_t workspace_bytes,
                                  void* stream);
int ucmr_merge_topk_wait_step(const float* cand_scores, const int32_t* cand_ids, int64_t parity_stride,
                              int64_t rank_stride, int R, int B, int Hout, int kl, int k, float* out_scores,
                              int32_t* out_ids, const int32_t* flags, int64_t flags_parity_stride,
                              int32_t* step_word, int32_t* arrive_word, int32_t* status_word, void* stream);

/* ---------------------------------------------------------------------------------------------
 *  Block copies through pointer lists, on the bulk-copy engine.
 *     Stands in for the three CudaSMCopyAsync / CudaCopyKernel overloads
 *     (ucm/shared/trans/cuda/cuda_sm_kernel.cu:52-114) that land store-loaded blocks: `num` blocks of
 *     `size` bytes (a multiple of 16) go from src_ptrs[i] (a DEVICE array of pointers) or from
 *     src_base + i*size to dst_ptrs[i] or dst_base + i*size.  Exactly one of src_ptrs / src_base and one
 *     of dst_ptrs / dst_base is non-NULL.  List entries that are NULL or not 16-byte aligned are skipped
 *     and flagged (UCMR_DEV_BAD_BLOCK_ID) in status_word.
 * ------------------------------------------------------------------------------------------ */
int ucmr_copy_blocks(const void* const* src_ptrs, const void* src_base, void* const* dst_ptrs, void* dst_base,
                     int64_t size, int64_t num, int32_t* status_word, void* stream);

/* ---------------------------------------------------------------------------------------------
 *  Float block retrieval (the ESA / KVStar plugins' CPU path, on the device).
 *
 *  ucmr_block_repr_mean: representation of KV blocks = mean of the keys over groups of `merge` tokens
 *     (merge = BS: one vector per block, ucm/sparse/esa/esa.py:254-263; smaller: ucm/sparse/kvstar/
 *     multistep.py:322-327).  k_cache bf16 [NB, BS, row_elems] with strides in elements; for listed
 *     block i, out[i, m, :] = mean of tokens [m*merge, (m+1)*merge), float32 accumulation, bf16 result.
 *     out is [n_blocks, BS/merge, row_elems] bf16.
 *  ucmr_dot_topk: per request b the k candidates with the largest inner product <q[b], repr[idx]>,
 *     idx running over indexes[b, 0..n) (entries < 0 or >= N are not candidates) - what the reference's
 *     RetrievalWorkerBackend computes on worker threads (ucm/sparse/esa/retrieval/cpy/
 *     retrieval_backend.cpp:206-225).  repr bf16 [N, dim], q bf16 [B, dim], float32 accumulation.
 *     out_scores float32 / out_ids int32 [B, k]: the chosen candidates in the order of the index list
 *     (the reference returns them by descending score), equal scores go to the earlier candidate,
 *     missing entries are (-inf, -1).  workspace: ucmr_dot_topk_workspace_bytes(B, n) bytes.
 * ------------------------------------------------------------------------------------------ */
int ucmr_block_repr_mean(const void* k_cache, int64_t NB, int BS, int row_elems, int64_t stride_block,
                         int64_t stride_t, const int32_t* block_ids, int64_t n_blocks, int merge, void* out,
                         int32_t* status_word, void* stream);
size_t ucmr_dot_topk_workspace_bytes(int B, int n);
int ucmr_dot_topk(const void* repr, int64_t N, int dim, const void* q, const int32_t* indexes, int B, int n,
                  int k, float* out_scores, int32_t* out_ids, void* workspace, size_t workspace_bytes,
                  void* stream);

/*  ucmr_softmax_topk: KVStar's block scores for one request (ucm/sparse/kvstar/retrieve/core/domain/
 *     retrieve_task/simd_compute_kernel.cpp:884-960): repr bf16 [n_blocks*M, Hkv, D] (M representations per
 *     block), q bf16 [X, Hq, D] (X query tokens); for every (token, query head) the inner products with the
 *     representations of its kv head, a softmax over all n_blocks*M of them, and score(block) = sum over
 *     rows and over the block's M representations of the softmax.  out_block_scores float32 [n_blocks]
 *     (may be NULL); the k best blocks go to out_scores / out_ids [k] in ascending block order.        */
size_t ucmr_softmax_topk_workspace_bytes(int X, int Hq, int n_blocks, int M);
int ucmr_softmax_topk(const void* repr, int n_blocks, int M, int Hkv, int D, const void* q, int X, int Hq, int k,
                      float* out_block_scores, float* out_scores, int32_t* out_ids, void* workspace,
                      size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* UCMR_H_ */
