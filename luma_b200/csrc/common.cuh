// Shared declarations of the sm_100a attention library: the problem descriptor every kernel
// family takes, status/last-error plumbing, storage<->f32 helpers and the paged-slot arithmetic.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

#include "../../include/flash_attn.h"

namespace fa {

// Which C entry point family a problem came from; decides how per-sequence extents are found.
enum Mode : int {
    MODE_BATCH = 0,    // flash_attn_<T>           : uniform lengths, start_pos, optional padding mask
    MODE_VARLEN = 1,   // flash_attn_varlen_<T>    : cu_seqlens, bottom-right causal, optional paging
    MODE_KVCACHE = 2,  // flash_attn_with_kvcache_<T>: context_lens + block table, bottom-right causal
};

enum DType : int { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 2 };

struct AttnParams {
    const void* q;
    const void* k;
    const void* v;
    void* o;
    float* lse;                 // (batch, q_heads, q_seq_len) or null; MODE_BATCH only
    const int* cu_q;            // MODE_VARLEN
    const int* cu_k;            // MODE_VARLEN
    const int* block_tables;    // paged K/V
    const int* context_lens;    // MODE_KVCACHE
    const uint8_t* mask;        // MODE_BATCH, (batch, kv_seq_len), may be null
    int mode;
    int dtype;
    int num_seqs;               // batch
    int q_seq_len;              // uniform q length (BATCH/KVCACHE) or max_seqlen_q (VARLEN)
    int kv_seq_len;             // BATCH: uniform kv length; VARLEN: max_seqlen_k; KVCACHE: max_blocks*block_size
    int q_heads;
    int kv_heads;
    int head_size;
    int start_pos;              // MODE_BATCH
    int block_size;
    int max_blocks;
    int paged;
    // MODE_VARLEN only: rows of the packed q/o and of the packed (contiguous) k/v buffers, when the
    // caller can say (0 = unknown: the tensor-core path needs them to bound its bulk copies)
    int total_q;
    int total_k;
    float scale;
    // head-sharded output (tcgen05 prefill only): n_out > 0 replaces `o` by n_out buffers of
    // (batch, q_seq_len, o_heads, head_size) that each receive this call's heads at o_head0
    void* o_peers[8];
    int n_out;
    int multicast;              // o_peers[0] is an NVSwitch multicast address of the group's output tensors (n_out == 1)
    int o_heads;
    int o_head0;
    // the same for the log-sum-exp: n_lse > 0 buffers of (batch, o_heads, q_seq_len) f32
    float* lse_peers[8];
    int n_lse;
};

// Per-sequence extents. Query row i of the sequence sits at global position pos_off + i and
// sees keys j < kv_len with j <= pos_off + i.
struct SeqInfo {
    long long q_row0;   // first row of this sequence in q / o (rows of q_heads*head_size elements)
    long long kv_row0;  // first row in contiguous k / v (unused when paged)
    int q_len;
    int kv_len;
    int pos_off;
};

__device__ __forceinline__ SeqInfo seq_info(const AttnParams& p, int s) {
    SeqInfo r;
    if (p.mode == MODE_BATCH) {
        r.q_row0 = (long long)s * p.q_seq_len;
        r.kv_row0 = (long long)s * p.kv_seq_len;
        r.q_len = p.q_seq_len;
        r.kv_len = p.kv_seq_len;
        r.pos_off = p.start_pos;
    } else if (p.mode == MODE_VARLEN) {
        const int q0 = p.cu_q[s], q1 = p.cu_q[s + 1];
        const int k0 = p.cu_k[s], k1 = p.cu_k[s + 1];
        r.q_row0 = q0;
        r.kv_row0 = k0;
        r.q_len = q1 - q0;
        r.kv_len = k1 - k0;
        r.pos_off = r.kv_len - r.q_len;
    } else {
        r.q_row0 = (long long)s * p.q_seq_len;
        r.kv_row0 = 0;
        r.q_len = p.q_seq_len;
        r.kv_len = p.context_lens[s];
        r.pos_off = r.kv_len - r.q_len;
    }
    return r;
}

// Logical token j of sequence s -> physical token slot of the pooled cache. Same 32-bit integer
// arithmetic as the reference (luma-flash-attn/kernels/common.cuh:89-108); callers widen the
// slot to 64 bits before multiplying by the row pitch.
__device__ __forceinline__ int block_slot(const int* __restrict__ block_tables, int s, int max_blocks,
                                          int j, int block_size) {
    const int logical_block = j / block_size;
    const int offset = j - logical_block * block_size;
    return block_tables[s * max_blocks + logical_block] * block_size + offset;
}

// Launch order of the rows (blockIdx.y) of a head-sharded tensor-core prefill grid: row `by` of the grid
// runs the band of tile pairs with this rank by weight (0 = heaviest). w == 0: heaviest first. Otherwise
// the first w rows of the grid are every m-th rank (0, m, 2m, ...: a first wave that mixes all weights),
// the ranks in between follow in ascending order, and ranks from w * m on keep their place. A bijection
// of [0, rows) for every rows >= w * m, m >= 2.
__host__ __device__ inline int launch_rank(int by, int w, int m) {
    if (w <= 0) return by;
    if (by < w) return by * m;
    if (by - w < w * (m - 1)) return ((by - w) / (m - 1)) * m + 1 + (by - w) % (m - 1);
    return by;
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// round-to-nearest-even, as the reference's f_from_float (kernels/common.cuh:70-81)
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// ---- host side -------------------------------------------------------------------------

int release_host_pipes();   // host_pipe.cu: frees the staging buffers of flash_attn_host_<T>; returns how many devices held some
void set_last_error(const char* msg);
void set_last_errorf(const char* fmt, ...);
void note_path(const char* name, int launches);   // records flash_attn_last_path / _launches
int get_option_force_generic();
int get_option_decode_chunk();
int get_option_prefill_trace();
int get_option_prefill_trace_y();
int get_option_prefill_band();
int get_option_prefill_groups();        // groups of K/V streams the tensor-core prefill grid runs one after the other (0 = automatic)
int get_option_prefill_order();         // 1 = heaviest-first launch order even for head-sharded calls (0 = the default)
int get_option_prefill_wait_us();       // bound of the tcgen05 kernel's waits in microseconds (0 = the default, 2 s)
int get_option_prefill_test_skip_k();   // test hook: 1 + index of a K tile the producer never requests (0 = off)

// Returns FLASH_ATTN_OK or FLASH_ATTN_ERR_CUDA (with last error set) after a launch.
int check_launch(const char* what);

// Kernel families. Each returns a flash_attn_status, or -1 when the problem is outside what that
// family supports (the dispatcher then tries the next one).
int launch_tile_simt(const AttnParams& p, cudaStream_t stream);
int launch_decode_splitk(const AttnParams& p, cudaStream_t stream);
int launch_prefill_tcgen05(const AttnParams& p, cudaStream_t stream);
int launch_debug_block_slots(const int* block_tables, const int* context_lens, const int* offsets,
                             int num_seqs, int block_size, int max_blocks, int* out_slots,
                             cudaStream_t stream);

int launch_kv_append(int elem_bytes, const void* k_new, const void* v_new, void* k_cache, void* v_cache,
                     const int* block_tables, const int* context_lens, int num_seqs, int n_new, int kv_heads,
                     int head_size, int block_size, int max_blocks, cudaStream_t stream);

// Reads and clears the current device's status word of the tcgen05 kernel (0 = every bounded wait
// was satisfied; otherwise the code of a wait that expired). The word is in mapped host memory:
// prefill_take_status() only looks at it, prefill_device_status() synchronises the device first.
int prefill_take_status();
int prefill_device_status();
// Copies the per-device debug area (status word, then from byte 256 the optional kernel timeline)
// to host memory; returns the bytes copied or -1.
int prefill_debug_read(void* dst, int bytes);

// Split-K scratch of the decode path: one buffer per (device, stream), grown on demand.
void* decode_workspace(cudaStream_t stream, size_t bytes);
// Releases every workspace (stream-ordered); returns how many buffers were held.
int release_workspaces();

}  // namespace fa
