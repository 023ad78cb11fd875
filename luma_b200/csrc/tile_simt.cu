// SIMT tile kernel: the catch-all implementation behind every entry point. It covers what the
// tensor-core kernels do not take — f32 storage, head size 32, page sizes that do not divide 128,
// unaligned buffers — for every entry
// point (batched with padding mask, packed variable-length, chunked prefill over a paged cache),
// with f32 arithmetic throughout. Semantics per entry point follow
//   luma-flash-attn/kernels/flash_attn_func.cu:29-226        (batched, start_pos, padding mask)
//   luma-flash-attn/kernels/flash_attn_varlen_func.cu:35-199 (packed, bottom-right causal, paged)
//   luma-flash-attn/kernels/flash_attn_with_kvcache.cu:157-277 (chunked prefill over pages)
// but the work decomposition is different: a CTA owns 16 query rows of one head, 8 lanes share a
// row (each lane keeps head_size/8 interleaved dims of q and of the running output), keys are
// staged 32 at a time in shared memory as f32 and folded in one by one with the online-softmax
// recurrence. Also hosts the block_slot check kernel.
#include "common.cuh"

namespace fa {

namespace {

constexpr int kRows = 16;     // query rows per CTA
constexpr int kLanes = 8;     // lanes sharing one query row
constexpr int kKeys = 32;     // keys staged per step
constexpr int kThreads = kRows * kLanes;

template <typename T, int D>
__global__ void __launch_bounds__(kThreads) tile_simt_kernel(const AttnParams p) {
    constexpr int E = D / kLanes;  // dims per lane, interleaved: x = lane + kLanes * e
    __shared__ float k_s[kKeys][D];
    __shared__ float v_s[kKeys][D];
    __shared__ long long row_s[kKeys];
    __shared__ unsigned char vis_s[kKeys];

    const int tid = threadIdx.x;
    const int r = tid / kLanes;
    const int c = tid % kLanes;
    const int s = blockIdx.z;
    const int h = blockIdx.y;
    const int row0 = blockIdx.x * kRows;

    const SeqInfo si = seq_info(p, s);
    if (row0 >= si.q_len) return;

    const int group = p.q_heads / p.kv_heads;
    const int kvh = h / group;
    const long long kv_pitch = (long long)p.kv_heads * D;
    const long long q_pitch = (long long)p.q_heads * D;

    const T* __restrict__ qg = static_cast<const T*>(p.q);
    const T* __restrict__ kg = static_cast<const T*>(p.k);
    const T* __restrict__ vg = static_cast<const T*>(p.v);
    T* __restrict__ og = static_cast<T*>(p.o);
    const uint8_t* mask_row = p.mask ? p.mask + (long long)s * p.kv_seq_len : nullptr;

    const int row = row0 + r;
    const bool row_in = row < si.q_len;
    const long long pos = (long long)si.pos_off + row;  // global position of this query row

    // the query row is valid unless a padding mask says otherwise (flash_attn_func.cu:77-84)
    bool q_valid = row_in;
    if (q_valid && mask_row != nullptr) {
        q_valid = pos >= 0 && pos < si.kv_len && mask_row[pos] != 0;
    }

    float qr[E], acc[E];
#pragma unroll
    for (int e = 0; e < E; ++e) {
        acc[e] = 0.0f;
        qr[e] = row_in ? to_f32<T>(qg[(si.q_row0 + row) * q_pitch + (long long)h * D + c + kLanes * e]) : 0.0f;
    }
    float m = -INFINITY, l = 0.0f;

    // keys beyond the last row's position are never visible
    const int last_row = min(si.q_len, row0 + kRows) - 1;
    const long long max_pos = (long long)si.pos_off + last_row;
    const int kv_end = (int)max(0LL, min((long long)si.kv_len, max_pos + 1));

    for (int j0 = 0; j0 < kv_end; j0 += kKeys) {
        __syncthreads();
        if (tid < kKeys) {
            const int j = j0 + tid;
            long long rowidx = -1;
            unsigned char vis = 0;
            if (j < kv_end) {
                rowidx = p.paged ? (long long)block_slot(p.block_tables, s, p.max_blocks, j, p.block_size)
                                 : si.kv_row0 + j;
                vis = (mask_row == nullptr || mask_row[j] != 0) ? 1 : 0;
            }
            row_s[tid] = rowidx;
            vis_s[tid] = vis;
        }
        __syncthreads();
        for (int idx = tid; idx < kKeys * D; idx += kThreads) {
            const int y = idx / D;
            const int x = idx - y * D;
            const long long rowidx = row_s[y];
            float kvl = 0.0f, vvl = 0.0f;
            if (rowidx >= 0) {
                const long long off = rowidx * kv_pitch + (long long)kvh * D + x;
                kvl = to_f32<T>(kg[off]);
                vvl = to_f32<T>(vg[off]);
            }
            k_s[y][x] = kvl;
            v_s[y][x] = vvl;
        }
        __syncthreads();

        const int ny = min(kKeys, kv_end - j0);
        for (int y = 0; y < ny; ++y) {
            float part = 0.0f;
#pragma unroll
            for (int e = 0; e < E; ++e) part += qr[e] * k_s[y][c + kLanes * e];
            part += __shfl_xor_sync(0xffffffffu, part, 1);
            part += __shfl_xor_sync(0xffffffffu, part, 2);
            part += __shfl_xor_sync(0xffffffffu, part, 4);
            const bool visible = row_in && vis_s[y] && (long long)(j0 + y) <= pos;
            if (visible) {
                const float sc = part * p.scale;
                const float m_new = fmaxf(m, sc);
                const float alpha = __expf(m - m_new);
                const float pr = __expf(sc - m_new);
                l = l * alpha + pr;
#pragma unroll
                for (int e = 0; e < E; ++e) acc[e] = acc[e] * alpha + pr * v_s[y][c + kLanes * e];
                m = m_new;
            }
        }
    }

    if (row_in) {
        const bool write_valid = q_valid && l > 0.0f;
        const float inv = write_valid ? 1.0f / l : 0.0f;
#pragma unroll
        for (int e = 0; e < E; ++e) {
            og[(si.q_row0 + row) * q_pitch + (long long)h * D + c + kLanes * e] = from_f32<T>(acc[e] * inv);
        }
        if (p.lse != nullptr && c == 0) {
            p.lse[((long long)s * p.q_heads + h) * p.q_seq_len + row] = write_valid ? m + __logf(l) : -INFINITY;
        }
    }
}

template <typename T, int D>
int launch_one(const AttnParams& p, cudaStream_t stream) {
    const int q_tiles = (p.q_seq_len + kRows - 1) / kRows;
    if (p.q_heads > 65535 || p.num_seqs > 65535) {
        set_last_error("flash_attn: q_heads and batch must each be <= 65535");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    dim3 grid(q_tiles, p.q_heads, p.num_seqs);
    tile_simt_kernel<T, D><<<grid, kThreads, 0, stream>>>(p);
    const int rc = check_launch("tile_simt_kernel");
    if (rc == FLASH_ATTN_OK) note_path("tile_simt", 1);
    return rc;
}

template <typename T>
int launch_by_head(const AttnParams& p, cudaStream_t stream) {
    switch (p.head_size) {
        case 32: return launch_one<T, 32>(p, stream);
        case 64: return launch_one<T, 64>(p, stream);
        case 128: return launch_one<T, 128>(p, stream);
        default:
            set_last_error("flash_attn: unsupported head_size (only 32/64/128)");
            return FLASH_ATTN_ERR_INVALID_HEAD_SIZE;
    }
}

__global__ void block_slots_kernel(const int* __restrict__ block_tables,
                                   const int* __restrict__ context_lens,
                                   const int* __restrict__ offsets, int block_size, int max_blocks,
                                   int* __restrict__ out_slots) {
    const int s = blockIdx.x;
    const int L = context_lens[s];
    const long long base = offsets[s];
    for (int j = threadIdx.x; j < L; j += blockDim.x) {
        out_slots[base + j] = block_slot(block_tables, s, max_blocks, j, block_size);
    }
}

}  // namespace

int launch_tile_simt(const AttnParams& p, cudaStream_t stream) {
    switch (p.dtype) {
        case DT_F32: return launch_by_head<float>(p, stream);
        case DT_F16: return launch_by_head<__half>(p, stream);
        case DT_BF16: return launch_by_head<__nv_bfloat16>(p, stream);
        default:
            set_last_error("flash_attn: unknown storage type");
            return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
}

int launch_debug_block_slots(const int* block_tables, const int* context_lens, const int* offsets,
                             int num_seqs, int block_size, int max_blocks, int* out_slots,
                             cudaStream_t stream) {
    block_slots_kernel<<<num_seqs, 256, 0, stream>>>(block_tables, context_lens, offsets, block_size,
                                                     max_blocks, out_slots);
    const int rc = check_launch("block_slots_kernel");
    if (rc == FLASH_ATTN_OK) note_path("block_slots", 1);
    return rc;
}

}  // namespace fa
