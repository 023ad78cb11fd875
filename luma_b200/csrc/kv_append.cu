// KV-cache append: scatters the K/V rows of newly processed tokens into their pages.
//
// The reference has no such kernel — flash_attn_with_kvcache expects "the caller writes the K/V"
// (luma-flash-attn/src/api/high.rs:123-125) — but it is the step that precedes every paged decode
// or chunked prefill, it shares block_slot() with them, and it is pure byte movement: each new
// token row (kv_heads * head_size elements) is copied once with 16-byte accesses to slot
// block_slot(table, s, context_len[s] - n_new + t).
#include "common.cuh"

namespace fa {

namespace {

template <int ELEM_BYTES>
__global__ void kv_append_kernel(const unsigned char* __restrict__ k_new, const unsigned char* __restrict__ v_new,
                                 unsigned char* __restrict__ k_cache, unsigned char* __restrict__ v_cache,
                                 const int* __restrict__ block_tables, const int* __restrict__ context_lens,
                                 int n_new, int row_elems, int block_size, int max_blocks) {
    const int s = blockIdx.y;
    const int t = blockIdx.x;                       // new token index within the sequence
    const int L = context_lens[s];                  // length AFTER the append
    const int j = L - n_new + t;                    // logical position of this token
    if (j < 0) return;                              // the sequence holds fewer than n_new tokens
    const int slot = block_slot(block_tables, s, max_blocks, j, block_size);
    const long long row_bytes = (long long)row_elems * ELEM_BYTES;
    const unsigned char* ks = k_new + ((long long)s * n_new + t) * row_bytes;
    const unsigned char* vs = v_new + ((long long)s * n_new + t) * row_bytes;
    unsigned char* kd = k_cache + (long long)slot * row_bytes;
    unsigned char* vd = v_cache + (long long)slot * row_bytes;
    const int vecs = (int)(row_bytes / 16);         // head_size >= 32 elements of >= 2 bytes: rows are 16-byte multiples
    for (int i = threadIdx.x; i < vecs; i += blockDim.x) {
        reinterpret_cast<uint4*>(kd)[i] = reinterpret_cast<const uint4*>(ks)[i];
        reinterpret_cast<uint4*>(vd)[i] = reinterpret_cast<const uint4*>(vs)[i];
    }
}

}  // namespace

int launch_kv_append(int elem_bytes, const void* k_new, const void* v_new, void* k_cache, void* v_cache,
                     const int* block_tables, const int* context_lens, int num_seqs, int n_new, int kv_heads,
                     int head_size, int block_size, int max_blocks, cudaStream_t stream) {
    if (num_seqs > 65535) {
        set_last_error("flash_attn_kvcache_append: num_seqs must be <= 65535");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    const int row_elems = kv_heads * head_size;
    const int threads = 128;
    dim3 grid(n_new, num_seqs);
    if (elem_bytes == 4) {
        kv_append_kernel<4><<<grid, threads, 0, stream>>>(
            static_cast<const unsigned char*>(k_new), static_cast<const unsigned char*>(v_new),
            static_cast<unsigned char*>(k_cache), static_cast<unsigned char*>(v_cache), block_tables, context_lens, n_new,
            row_elems, block_size, max_blocks);
    } else {
        kv_append_kernel<2><<<grid, threads, 0, stream>>>(
            static_cast<const unsigned char*>(k_new), static_cast<const unsigned char*>(v_new),
            static_cast<unsigned char*>(k_cache), static_cast<unsigned char*>(v_cache), block_tables, context_lens, n_new,
            row_elems, block_size, max_blocks);
    }
    const int rc = check_launch("kv_append_kernel");
    if (rc == FLASH_ATTN_OK) note_path("kv_append", 1);
    return rc;
}

}  // namespace fa
