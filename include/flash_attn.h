/*
 * C ABI of the B200 (sm_100a) attention library, libflash_attn.
 *
 * The first ten symbols are exactly what luma's Rust crate `luma-flash-attn` binds in
 * luma-flash-attn/src/api/ffi.rs:13-193 (status constants ffi.rs:6-11); a build of that crate
 * that links this library instead of its own kernels/ *.cu needs no source change.
 * Everything after the "additive" marker does not exist in the reference.
 *
 * Conventions shared by every entry point (reference: kernels/flash_attn_func.cu:267-328,
 * kernels/flash_attn_varlen_func.cu:259-326, kernels/flash_attn_with_kvcache.cu:345-407):
 *   - all tensors are dense row-major device buffers; element offsets are already applied;
 *   - `o` is caller-allocated and may be uninitialised: every element is written, zeros for
 *     rows that are invalid or see no key;
 *   - `stream` is a CUstream / cudaStream_t (NULL = legacy default stream); launches are
 *     asynchronous, nothing synchronises; execution-time faults surface at the caller's sync;
 *   - the call makes the device that owns the pointers current for its own launches, so one
 *     host thread per GPU can drive different devices;
 *   - return value is a flash_attn_status; on failure flash_attn_last_error() holds a
 *     NUL-terminated message (thread-local, at most 255 chars); every call clears it first;
 *   - storage types f32 / f16 / bf16, arithmetic in f32, outputs rounded to nearest even;
 *   - head_size must be 32, 64 or 128; q heads must be a multiple of kv heads (GQA).
 * There is no CPU fallback: without a CUDA device every compute entry point returns
 * FLASH_ATTN_ERR_CUDA.
 */
#ifndef LUMA_B200_FLASH_ATTN_H_
#define LUMA_B200_FLASH_ATTN_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* luma-flash-attn/kernels/common.cuh:17-24 == src/api/ffi.rs:6-11 */
enum flash_attn_status {
    FLASH_ATTN_OK = 0,
    FLASH_ATTN_ERR_NULL_PTR = 1,
    FLASH_ATTN_ERR_INVALID_SHAPE = 2,
    FLASH_ATTN_ERR_INVALID_HEAD_SIZE = 3,
    FLASH_ATTN_ERR_INVALID_START_POS = 4,
    FLASH_ATTN_ERR_CUDA = 5
};

/* f16 / bf16 buffers are passed as raw 16-bit storage so that this header needs no CUDA include. */
typedef uint16_t flash_attn_f16_t;
typedef uint16_t flash_attn_bf16_t;

/*
 * Batched causal attention. Replaces flash_attn_{f32,f16,bf16}
 * (ffi.rs:15-66; kernels/flash_attn_func.cu:312-328).
 *   q, o : (batch, q_seq_len,  q_num_heads,  head_size)
 *   k, v : (batch, kv_seq_len, kv_num_heads, head_size)
 *   attn_mask : (batch, kv_seq_len) bytes, 1 = valid, 0 = padding, may be NULL. A masked key is
 *               invisible; a query row whose own position start_pos+i is masked or >= kv_seq_len
 *               outputs zeros (kernels/flash_attn_func.cu:74-84).
 *   query row i sits at global position start_pos + i and sees keys j <= that.
 * Check order: NULL q/k/v/o -> NULL_PTR; non-positive dims or Hq % Hkv != 0 -> INVALID_SHAPE;
 * start_pos < 0 -> INVALID_START_POS; head_size not in {32,64,128} -> INVALID_HEAD_SIZE.
 */
int flash_attn_f32(const float* q, const float* k, const float* v, float* o,
                   int batch, int q_seq_len, int kv_seq_len, int q_num_heads, int kv_num_heads,
                   int head_size, int start_pos, float scale, const uint8_t* attn_mask, void* stream);
int flash_attn_f16(const flash_attn_f16_t* q, const flash_attn_f16_t* k, const flash_attn_f16_t* v,
                   flash_attn_f16_t* o,
                   int batch, int q_seq_len, int kv_seq_len, int q_num_heads, int kv_num_heads,
                   int head_size, int start_pos, float scale, const uint8_t* attn_mask, void* stream);
int flash_attn_bf16(const flash_attn_bf16_t* q, const flash_attn_bf16_t* k, const flash_attn_bf16_t* v,
                    flash_attn_bf16_t* o,
                    int batch, int q_seq_len, int kv_seq_len, int q_num_heads, int kv_num_heads,
                    int head_size, int start_pos, float scale, const uint8_t* attn_mask, void* stream);

/*
 * Packed variable-length causal attention, bottom-right aligned, K/V contiguous or paged.
 * Replaces flash_attn_varlen_{f32,f16,bf16} (ffi.rs:68-132;
 * kernels/flash_attn_varlen_func.cu:308-326).
 *   q, o : (total_q, q_heads, head_size)
 *   k, v : (total_kv, kv_heads, head_size), or when k_paged != 0 a cache
 *          (num_blocks, block_size, kv_heads, head_size) addressed through
 *          block_tables (num_seqs, max_blocks)
 *   cu_seqlens_q / cu_seqlens_k : (num_seqs + 1) i32 prefix sums; with a paged cache only the
 *          differences of cu_seqlens_k are used (the per-sequence cached length).
 * Check order: NULL q/o/cu_seqlens -> NULL_PTR; NULL k/v (or block_tables when paged) -> NULL_PTR;
 * num_seqs/heads <= 0, Hq % Hkv, head_size not in {32,64,128} -> INVALID_SHAPE;
 * max_seqlen_q/max_seqlen_k/block_size <= 0 -> INVALID_SHAPE.
 */
int flash_attn_varlen_f32(const float* q, const float* k, const float* v, float* o,
                          const int* cu_seqlens_q, const int* cu_seqlens_k, const int* block_tables,
                          int num_seqs, int max_seqlen_q, int max_seqlen_k, int q_heads, int kv_heads,
                          int head_size, int block_size, int max_blocks, int k_paged, float scale,
                          void* stream);
int flash_attn_varlen_f16(const flash_attn_f16_t* q, const flash_attn_f16_t* k,
                          const flash_attn_f16_t* v, flash_attn_f16_t* o,
                          const int* cu_seqlens_q, const int* cu_seqlens_k, const int* block_tables,
                          int num_seqs, int max_seqlen_q, int max_seqlen_k, int q_heads, int kv_heads,
                          int head_size, int block_size, int max_blocks, int k_paged, float scale,
                          void* stream);
int flash_attn_varlen_bf16(const flash_attn_bf16_t* q, const flash_attn_bf16_t* k,
                           const flash_attn_bf16_t* v, flash_attn_bf16_t* o,
                           const int* cu_seqlens_q, const int* cu_seqlens_k, const int* block_tables,
                           int num_seqs, int max_seqlen_q, int max_seqlen_k, int q_heads, int kv_heads,
                           int head_size, int block_size, int max_blocks, int k_paged, float scale,
                           void* stream);

/*
 * ADDITIVE (no counterpart in the reference): the packed entry point with the row counts of the
 * packed buffers. The reference signature above only has them on the device (cu_seqlens[num_seqs]);
 * through it the tensor-core kernel's tensor maps carry no row bound and the tiles at the very end
 * of the packed buffers are fetched with plain loads, never past the last row. With the counts the
 * maps are bounded as well. Results are bit-identical. luma's high.rs knows both from the tensor
 * shapes (high.rs:170-182).
 *   total_q : rows of q and o (= cu_seqlens_q[num_seqs])
 *   total_k : rows of contiguous k and v (= cu_seqlens_k[num_seqs]); ignored when k_paged != 0
 * Same checks, results and status codes as flash_attn_varlen_{f16,bf16}; totals <= 0 mean
 * "unknown" and give exactly the behaviour of those.
 */
int flash_attn_varlen_f16_total(const flash_attn_f16_t* q, const flash_attn_f16_t* k, const flash_attn_f16_t* v,
                                flash_attn_f16_t* o, const int* cu_seqlens_q, const int* cu_seqlens_k,
                                const int* block_tables, int num_seqs, int max_seqlen_q, int max_seqlen_k,
                                int q_heads, int kv_heads, int head_size, int block_size, int max_blocks,
                                int k_paged, float scale, int total_q, int total_k, void* stream);
int flash_attn_varlen_bf16_total(const flash_attn_bf16_t* q, const flash_attn_bf16_t* k, const flash_attn_bf16_t* v,
                                 flash_attn_bf16_t* o, const int* cu_seqlens_q, const int* cu_seqlens_k,
                                 const int* block_tables, int num_seqs, int max_seqlen_q, int max_seqlen_k,
                                 int q_heads, int kv_heads, int head_size, int block_size, int max_blocks,
                                 int k_paged, float scale, int total_q, int total_k, void* stream);

/*
 * Attention over a paged KV cache: q_seq_len == 1 is single-token decode, > 1 is chunked
 * prefill (bottom-right causal: row i sits at context_lens[s] - q_seq_len + i).
 * Replaces flash_attn_with_kvcache_{f32,f16,bf16} (ffi.rs:134-189;
 * kernels/flash_attn_with_kvcache.cu:390-407).
 *   q, o : (num_seqs, q_seq_len, q_heads, head_size)
 *   k_cache, v_cache : (num_blocks, block_size, kv_heads, head_size)
 *   block_tables : (num_seqs, max_blocks) i32, logical block -> physical block
 *   context_lens : (num_seqs) i32, total cached length including the q tokens
 * Token j of sequence s lives at slot block_tables[s*max_blocks + j/block_size]*block_size +
 * j%block_size (kernels/common.cuh:89-108); element offsets are 64-bit.
 * Check order: any NULL -> NULL_PTR; num_seqs/heads <= 0, Hq % Hkv, head_size not in {32,64,128},
 * q_seq_len <= 0, block_size <= 0 -> INVALID_SHAPE.
 * The decode path keeps a per-device, per-stream split-K workspace inside the library; it is
 * grown with cudaMalloc on the first call that needs more (that call synchronises the device).
 */
int flash_attn_with_kvcache_f32(const float* q, const float* k_cache, const float* v_cache, float* o,
                                const int* block_tables, const int* context_lens,
                                int num_seqs, int q_seq_len, int q_heads, int kv_heads, int head_size,
                                int block_size, int max_blocks, float scale, void* stream);
int flash_attn_with_kvcache_f16(const flash_attn_f16_t* q, const flash_attn_f16_t* k_cache,
                                const flash_attn_f16_t* v_cache, flash_attn_f16_t* o,
                                const int* block_tables, const int* context_lens,
                                int num_seqs, int q_seq_len, int q_heads, int kv_heads, int head_size,
                                int block_size, int max_blocks, float scale, void* stream);
int flash_attn_with_kvcache_bf16(const flash_attn_bf16_t* q, const flash_attn_bf16_t* k_cache,
                                 const flash_attn_bf16_t* v_cache, flash_attn_bf16_t* o,
                                 const int* block_tables, const int* context_lens,
                                 int num_seqs, int q_seq_len, int q_heads, int kv_heads, int head_size,
                                 int block_size, int max_blocks, float scale, void* stream);

/* Thread-local message of the last failing call on this thread; never NULL
 * (ffi.rs:191-192; kernels/flash_attn_func.cu:308-310). */
const char* flash_attn_last_error(void);

/* ------------------------------------------------------------------------------------------
 * Additive symbols (no counterpart in the reference's ffi.rs).
 * ------------------------------------------------------------------------------------------ */

/*
 * flash_attn_<T> plus an fp32 log-sum-exp output: lse is (batch, q_num_heads, q_seq_len),
 * natural log of the sum of exp(scale * q.k) over the visible keys; -inf for rows that output
 * zeros. lse may be NULL (then identical to flash_attn_<T>). No counterpart in the reference.
 */
int flash_attn_f32_lse(const float* q, const float* k, const float* v, float* o, float* lse,
                       int batch, int q_seq_len, int kv_seq_len, int q_num_heads, int kv_num_heads,
                       int head_size, int start_pos, float scale, const uint8_t* attn_mask, void* stream);
int flash_attn_f16_lse(const flash_attn_f16_t* q, const flash_attn_f16_t* k, const flash_attn_f16_t* v,
                       flash_attn_f16_t* o, float* lse,
                       int batch, int q_seq_len, int kv_seq_len, int q_num_heads, int kv_num_heads,
                       int head_size, int start_pos, float scale, const uint8_t* attn_mask, void* stream);
int flash_attn_bf16_lse(const flash_attn_bf16_t* q, const flash_attn_bf16_t* k, const flash_attn_bf16_t* v,
                        flash_attn_bf16_t* o, float* lse,
                        int batch, int q_seq_len, int kv_seq_len, int q_num_heads, int kv_num_heads,
                        int head_size, int start_pos, float scale, const uint8_t* attn_mask, void* stream);

/*
 * Head-sharded causal prefill with the output all-gather fused into the kernel's epilogue. No
 * counterpart in the reference (its luma-dist all_gather, luma-dist/src/backends/nccl/backend.rs:
 * 167-180, is a separate collective with two layout copies and a memset around it).
 *   q : (batch, q_seq_len, q_num_heads, 128) — this rank's query heads;  k, v : this rank's KV heads
 *   o_peers : HOST array of n_peers device pointers, one per GPU of the group (this GPU's own
 *             buffer included), each to the FULL output (batch, q_seq_len, q_heads_total, 128).
 *             Peer buffers must be mapped into this process (CUDA IPC or symmetric memory).
 *   The kernel stores its heads at head index q_head_offset of every buffer with ordinary 16-byte
 *   stores (posted writes over NVLink for peers): no TMA towards peers, no multicast, no waiting
 *   on peers inside the kernel. Every GPU of the group starts its walk over the buffers one past its
 *   own (its index is taken as q_head_offset / q_num_heads), so that the group never aims at one
 *   GPU at a time. The caller synchronises the group (a barrier after the launch) before anyone reads
 *   the gathered tensor. lse (optional) is local: (batch, q_num_heads, q_seq_len). No tensor map is
 *   ever made over a peer's buffer.
 * f16/bf16, head_size 64 or 128 (else INVALID_HEAD_SIZE), scale > 0, 16-byte aligned buffers
 * (else INVALID_SHAPE), each with a message.
 *
 * The _lse forms gather the log-sum-exp the same way (the reference's all_gather along dim 1 of
 * (batch, heads, seq)): lse_peers is a HOST array of n_peers device pointers to the FULL
 * (batch, q_heads_total, q_seq_len) f32 tensor of every GPU; this call's heads are written at head
 * index q_head_offset of each.
 */
int flash_attn_f16_allgather(const flash_attn_f16_t* q, const flash_attn_f16_t* k, const flash_attn_f16_t* v,
                             void* const* o_peers, int n_peers, int q_heads_total, int q_head_offset, float* lse,
                             int batch, int q_seq_len, int kv_seq_len, int q_num_heads, int kv_num_heads,
                             int head_size, int start_pos, float scale, void* stream);
int flash_attn_bf16_allgather(const flash_attn_bf16_t* q, const flash_attn_bf16_t* k, const flash_attn_bf16_t* v,
                              void* const* o_peers, int n_peers, int q_heads_total, int q_head_offset, float* lse,
                              int batch, int q_seq_len, int kv_seq_len, int q_num_heads, int kv_num_heads,
                              int head_size, int start_pos, float scale, void* stream);

int flash_attn_f16_allgather_lse(const flash_attn_f16_t* q, const flash_attn_f16_t* k, const flash_attn_f16_t* v,
                                 void* const* o_peers, float* const* lse_peers, int n_peers, int q_heads_total,
                                 int q_head_offset, int batch, int q_seq_len, int kv_seq_len, int q_num_heads,
                                 int kv_num_heads, int head_size, int start_pos, float scale, void* stream);
int flash_attn_bf16_allgather_lse(const flash_attn_bf16_t* q, const flash_attn_bf16_t* k, const flash_attn_bf16_t* v,
                                  void* const* o_peers, float* const* lse_peers, int n_peers, int q_heads_total,
                                  int q_head_offset, int batch, int q_seq_len, int kv_seq_len, int q_num_heads,
                                  int kv_num_heads, int head_size, int start_pos, float scale, void* stream);

/*
 * The same fused all-gather through an NVSwitch multicast address: o_multicast is a device address that
 * the caller obtained by binding the full (batch, q_seq_len, q_heads_total, head_size) output tensors of
 * all GPUs of the group to one multicast object (cuMulticastCreate / cuMulticastBindMem, or a library
 * that does it); the epilogue issues ONE multimem.st per 16 bytes and the switch writes it into every
 * GPU's tensor, this GPU's own included, so that a GPU's outgoing volume is its shard once instead of
 * once per peer. Everything else as flash_attn_<T>_allgather (barrier by the caller before reading;
 * lse is local). No counterpart in the reference.
 */
int flash_attn_f16_allgather_multicast(const flash_attn_f16_t* q, const flash_attn_f16_t* k, const flash_attn_f16_t* v,
                                       void* o_multicast, int q_heads_total, int q_head_offset, float* lse, int batch,
                                       int q_seq_len, int kv_seq_len, int q_num_heads, int kv_num_heads, int head_size,
                                       int start_pos, float scale, void* stream);
int flash_attn_bf16_allgather_multicast(const flash_attn_bf16_t* q, const flash_attn_bf16_t* k, const flash_attn_bf16_t* v,
                                        void* o_multicast, int q_heads_total, int q_head_offset, float* lse, int batch,
                                        int q_seq_len, int kv_seq_len, int q_num_heads, int kv_num_heads, int head_size,
                                        int start_pos, float scale, void* stream);

/*
 * Head-sharded single-token paged decode (q_seq_len == 1) with the output all-gather fused into the
 * split-K merge kernel: every merged row is stored straight into the (num_seqs, 1, q_heads_total,
 * head_size) output of every GPU of the group at head index q_head_offset (plain stores, as above).
 * No counterpart in the reference (attention, then luma-dist's all_gather, luma-dist/src/backends/
 * nccl/backend.rs:167-180). q / caches / tables as flash_attn_with_kvcache_<T>; this rank's caches
 * hold its KV heads only. f16/bf16, head_size 64 or 128, 16-byte aligned caches, else INVALID_SHAPE.
 */
int flash_attn_with_kvcache_f16_allgather(const flash_attn_f16_t* q, const flash_attn_f16_t* k_cache,
                                          const flash_attn_f16_t* v_cache, void* const* o_peers, int n_peers,
                                          int q_heads_total, int q_head_offset, const int* block_tables,
                                          const int* context_lens, int num_seqs, int q_heads, int kv_heads, int head_size,
                                          int block_size, int max_blocks, float scale, void* stream);
int flash_attn_with_kvcache_bf16_allgather(const flash_attn_bf16_t* q, const flash_attn_bf16_t* k_cache,
                                           const flash_attn_bf16_t* v_cache, void* const* o_peers, int n_peers,
                                           int q_heads_total, int q_head_offset, const int* block_tables,
                                           const int* context_lens, int num_seqs, int q_heads, int kv_heads, int head_size,
                                           int block_size, int max_blocks, float scale, void* stream);

/*
 * KV-cache append: the step before every paged decode / chunked prefill. No counterpart in the
 * reference, which leaves writing the cache to the caller (src/api/high.rs:123-125).
 *   k_new, v_new : (num_seqs, n_new, kv_heads, head_size) rows of the newly processed tokens
 *   k_cache, v_cache : (num_blocks, block_size, kv_heads, head_size)
 *   context_lens : (num_seqs) lengths AFTER the append; token t of sequence s goes to logical
 *                  position context_lens[s] - n_new + t (positions < 0 are skipped), i.e. to slot
 *                  block_tables[s*max_blocks + pos/block_size]*block_size + pos%block_size.
 * Storage-type agnostic: elem_bytes is 2 (f16 / bf16) or 4 (f32); rows are copied bit for bit.
 */
int flash_attn_kvcache_append(const void* k_new, const void* v_new, void* k_cache, void* v_cache,
                              const int* block_tables, const int* context_lens, int num_seqs, int n_new,
                              int kv_heads, int head_size, int elem_bytes, int block_size, int max_blocks,
                              void* stream);

/*
 * Runs the device-side block_slot arithmetic of the paged kernels and writes, for every sequence
 * s and token j < context_lens[s], the physical token slot to out_slots[offsets[s] + j]
 * (offsets = exclusive prefix sum of context_lens, supplied by the caller, num_seqs entries).
 * Exists so that page indexing can be checked bit for bit against a host walk of the table.
 * No counterpart in the reference.
 */
int flash_attn_debug_block_slots(const int* block_tables, const int* context_lens, const int* offsets,
                                 int num_seqs, int block_size, int max_blocks, int* out_slots,
                                 void* stream);

/*
 * Paged single-token decode (bf16, head_size 64 or 128) that never allocates. It has no
 * counterpart in the reference.
 *
 * Same arguments and result as flash_attn_with_kvcache_bf16 with q_seq_len == 1, but the split-K
 * partials go to a fixed 16 MiB array inside the library image instead of a cudaMalloc'ed
 * workspace, and the call makes no cudaMalloc / cudaFree / allocating library call at all. It is
 * meant for callers that cannot allocate at this point: an engine that reserved all device
 * memory for its own pool at start-up (a later cudaMalloc inside a library would fail), or a
 * latency-critical step that must not take the driver's allocation lock and the device-wide
 * synchronisation that cudaMalloc and cudaFree imply.
 *   - Cost: every GPU whose context loads this library holds those 16 MiB until the process
 *     exits, whether or not this function is called.
 *   - Limit: the partials of one split, num_seqs * q_heads * (head_size*4 + 8) bytes, must fit in
 *     16 MiB (32 263 rows at head_size 128); larger problems return
 *     FLASH_ATTN_ERR_INVALID_SHAPE with a message naming the limit. Within the limit the context
 *     is cut into as many splits as fit.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress); make that first call before starting any stream capture.
 *   - That first call is also the moment the 16 MiB become real on that device: CUDA loads a
 *     library's device code lazily by default, so the array is backed with memory when the first
 *     kernel or symbol of its module is touched, not when the process starts. A caller that is
 *     about to hand all free device memory to its own pool must therefore make one call here first
 *     (one sequence of one token is enough), or run with CUDA_MODULE_LOADING=EAGER; if the array
 *     cannot be backed any more, the first call fails with FLASH_ATTN_ERR_CUDA and a message that
 *     says so. From the second call on nothing is allocated by anyone.
 *   - All calls on a device share the one array. Nothing in it has to start at zero (every slot
 *     that is read was written earlier in the same call), but two calls that overlap on the GPU —
 *     different streams, or different threads — race on it; serialise them.
 * Check order: NULL -> NULL_PTR; non-positive sizes, Hq % Hkv, head_size not in {64,128},
 * misaligned caches, scratch too small -> INVALID_SHAPE.
 */
int flash_attn_decode_bf16_noalloc(const flash_attn_bf16_t* q, const flash_attn_bf16_t* k_cache,
                                   const flash_attn_bf16_t* v_cache, flash_attn_bf16_t* o,
                                   const int* block_tables, const int* context_lens,
                                   int num_seqs, int q_heads, int kv_heads, int head_size,
                                   int block_size, int max_blocks, float scale, void* stream);

/*
 * Batched causal attention for tensors in HOST memory: q (batch, q_seq_len, q_num_heads, head_size),
 * k/v (batch, kv_seq_len, kv_num_heads, head_size) and o like q, dense row-major, page-locked for
 * the copies to be asynchronous. No counterpart in the reference (its callers hold device tensors,
 * luma-flash-attn/src/api/high.rs:157-290); this is the call the end-to-end figure of the benchmark
 * goes through. The work is cut into steps of one batch element and `chunk_rows` query rows (0 =
 * automatic: half of the sequence, the first and last step cut finer) and pipelined over three
 * streams of `device`: each chunk travels in with the K/V rows up to its own end (a chunked prefill
 * with start_pos advanced per chunk), runs through flash_attn_<T>, and travels out while the next
 * ones are in flight. Staging buffers are kept per device (two row slots, two K/V slots of the
 * largest shape seen) and freed by flash_attn_release_workspaces. `stream` is the caller's stream
 * on `device`: the pipeline starts after the work already in it and the stream continues when the
 * last row of o has reached the host. Check order: NULL -> NULL_PTR; non-positive sizes or
 * Hq % Hkv -> INVALID_SHAPE; start_pos < 0 -> INVALID_START_POS; head_size not in {32,64,128} ->
 * INVALID_HEAD_SIZE; CUDA failures -> CUDA.
 *   flash_attn_host_steps : the (batch element, first row, end row) triples such a call is cut
 *                           into, written to steps_out (3 ints each, up to `capacity` triples);
 *                           returns their number. Host arithmetic only.
 */
int flash_attn_host_f32(const float* q, const float* k, const float* v, float* o,
                        int batch, int q_seq_len, int kv_seq_len, int q_num_heads, int kv_num_heads,
                        int head_size, int start_pos, float scale, int device, int chunk_rows, void* stream);
int flash_attn_host_f16(const flash_attn_f16_t* q, const flash_attn_f16_t* k, const flash_attn_f16_t* v,
                        flash_attn_f16_t* o,
                        int batch, int q_seq_len, int kv_seq_len, int q_num_heads, int kv_num_heads,
                        int head_size, int start_pos, float scale, int device, int chunk_rows, void* stream);
int flash_attn_host_bf16(const flash_attn_bf16_t* q, const flash_attn_bf16_t* k, const flash_attn_bf16_t* v,
                         flash_attn_bf16_t* o,
                         int batch, int q_seq_len, int kv_seq_len, int q_num_heads, int kv_num_heads,
                         int head_size, int start_pos, float scale, int device, int chunk_rows, void* stream);
int flash_attn_host_steps(int batch, int q_seq_len, int chunk_rows, int* steps_out, int capacity);

/*
 * Tuning and introspection. No counterpart in the reference.
 *   flash_attn_version        : library version string.
 *   flash_attn_last_path      : name of the kernel family the last successful call on this
 *                               thread dispatched to ("prefill_tcgen05", "decode_splitk", "tile_simt").
 *   flash_attn_last_launches  : number of kernels that call launched.
 *   flash_attn_set_option     : named integer knobs (returns 0 if the name is known):
 *       "force_generic"       1 = route everything through the SIMT tile kernel
 *       "prefill_trace"       (builds with -DFA_TRACE only; ignored otherwise)
 *                             1 = record the timeline read by flash_attn_debug_read;
 *                             2 = stage the epilogue's rows in shared memory even for one output;
 *                             3 = log {start ns, end ns, SM id} of up to 2048 CTAs from byte 16384
 *       "prefill_trace_y"     blockIdx.y of the CTA whose timeline is recorded (0 = heaviest)
 *       "prefill_band"        tile pairs of one K/V stream launched next to each other (0 = automatic)
 *       "prefill_groups"      groups of K/V streams the prefill grid runs one after the other (0 = automatic:
 *                             about 16 MiB of K/V per group when no launch band shares them, whole batch
 *                             elements or sequences, about 48 MiB of K/V per group, for batched and packed GQA calls)
 *       "prefill_order"       1 = heaviest-first launch order also for head-sharded calls (0 = their first wave mixes all weights)
 *       "decode_chunk_tokens" tokens per split-K work item (0 = automatic)
 *       "prefill_wait_us"     bound of every wait inside the tcgen05 prefill kernel, microseconds
 *                             (0 = the default of 2 s)
 *       "prefill_test_skip_k" test hook: 1 + index of a K tile the kernel's producer never requests,
 *                             so that the wait for it runs out and the kernel returns early with its
 *                             status word set (0 = off). Only for testing the error path below.
 *     The knobs are atomics: they may be set while other threads launch.
 */
/*
 * Bounded waits and how their expiry is reported. Every wait inside the tcgen05 prefill kernel is
 * bounded; a CTA whose wait runs out stores the wait's code in a per-device status word (mapped
 * host memory), drains its copies, frees its tensor memory and returns: the launch ends, its output
 * is undefined. Launches are asynchronous, so the entry point that made the launch has returned
 * FLASH_ATTN_OK long before. The NEXT attention entry point called for that device looks at the
 * word first (a host read, no synchronisation): if it is set, that call clears it, launches
 * nothing and returns FLASH_ATTN_ERR_CUDA with a message naming the wait code; the call after is
 * clean again.
 *   flash_attn_device_status  : synchronises the current device, then reads and clears its status
 *                               word. 0 = healthy, non-zero = the code of an expired wait,
 *                               -1 = no device / not readable.
 *   flash_attn_release_workspaces : releases (stream-ordered) every split-K workspace the decode
 *                               path holds and the staging buffers of flash_attn_host_<T>; returns how many there were. The library keeps at most
 *                               32 of them (one per device and stream, least recently used first out).
 */
const char* flash_attn_version(void);
int flash_attn_device_status(void);
int flash_attn_release_workspaces(void);
/*
 *   flash_attn_debug_launch_rank : the host copy of the index arithmetic that orders the rows of a
 *                               head-sharded prefill grid (which band of tile pairs, by weight, grid row
 *                               `grid_row` runs when the first `first_wave_rows` rows take every
 *                               `stride`-th band); exists so that the mapping can be checked on the CPU.
 */
int flash_attn_debug_launch_rank(int grid_row, int first_wave_rows, int stride);
/*
 *   flash_attn_debug_read     : builds with -DFA_TRACE only (returns -1 otherwise): copies up to
 *                               `bytes` (max 65536) of the current device's debug area to host
 *                               memory: int status word at byte 0; from byte 256, when the option
 *                               "prefill_trace" is 1, clock64 stamps of one CTA of the last tcgen05
 *                               prefill launch, laid out [role 0..2][kv step 0..59][event 0..7] as
 *                               int64. Returns bytes copied or -1.
 */
int flash_attn_debug_read(void* dst, int bytes);
const char* flash_attn_last_path(void);
int flash_attn_last_launches(void);
int flash_attn_set_option(const char* name, int value);

#ifdef __cplusplus
}
#endif

#endif /* LUMA_B200_FLASH_ATTN_H_ */
