// Paged-KV single-token decode for f16/bf16 storage, head_size 32, 64 or 128.
//
// Replaces flash_attn_decode_kernel (luma-flash-attn/kernels/flash_attn_with_kvcache.cu:22-116;
// launch :123-145), which walks the context one token at a time with one warp per query head and
// re-reads K/V once per query head of a GQA group.
//
// Here the path is HBM-bound by construction:
//   * work item = (chunk of the context, KV head, sequence); a CTA reads each K/V row of its chunk
//     exactly once and serves every query head of the GQA group from it;
//   * rows are gathered through the block table with 16-byte cp.async copies into a per-warp ring
//     of shared-memory stages (3 tiles of 16 tokens in flight per warp, 2 CTAs per SM), no
//     CTA-wide barrier inside the loop;
//   * Q.K^T and P.V run on tensor cores (mma.sync m16n8k16, f32 accumulate) with the group's
//     query heads as the 16-row M dimension — at 8 query heads per KV head scalar FMA could not
//     keep up with the memory system;
//   * split-K over the context: every chunk writes an unnormalised f32 partial (acc, m, l) to a
//     workspace and a second kernel merges the chunks of a sequence with log-sum-exp weights.
// Token -> slot arithmetic is block_slot() from common.cuh (reference: kernels/common.cuh:89-108).
#include <mutex>

#include "common.cuh"

namespace fa {

namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kTile = 16;    // tokens per tile (one mma K step for P.V, two N blocks for Q.K^T)
constexpr int kStages = 3;   // tiles in flight per warp
constexpr int kMaxHeads = 16;  // query heads served per CTA (M of the mma)

struct DecodeArgs {
    const void* q;
    const void* k;
    const void* v;
    const int* block_tables;
    const int* context_lens;
    float* ws_acc;   // (num_seqs, q_heads, max_splits, D) f32, unnormalised
    float2* ws_ml;   // (num_seqs, q_heads, max_splits) {m (log2 domain), l}
    int num_seqs, q_heads, kv_heads, block_size, max_blocks;
    int chunk;       // tokens per work item, multiple of kWarps * kTile
    int max_splits;
    int head_blocks; // ceil(group / kMaxHeads)
    float scale_log2;  // scale * log2(e)
};

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
    const unsigned saddr = (unsigned)__cvta_generic_to_shared(smem);
    const int src_bytes = valid ? 16 : 0;  // 0 -> the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(saddr), "l"(gmem), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3,
                                            const void* smem) {
    const unsigned saddr = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(saddr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3,
                                                  const void* smem) {
    const unsigned saddr = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(saddr));
}

template <typename T>
__device__ __forceinline__ void mma_16816(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1);
template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&d)[4], const unsigned (&a)[4], unsigned b0,
                                                         unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_16816<__half>(float (&d)[4], const unsigned (&a)[4], unsigned b0,
                                                  unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename T>
__device__ __forceinline__ unsigned pack2(float lo, float hi);
template <>
__device__ __forceinline__ unsigned pack2<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&t);
}
template <>
__device__ __forceinline__ unsigned pack2<__half>(float lo, float hi) {
    __half2 t = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&t);
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// Shared memory of one CTA:
//   ring : kWarps x kStages x {K tile, V tile}, each tile kTile rows of D elements, 16-byte chunks
//          XOR-swizzled by the row (row & 7; row & 3 at head_size 32, whose rows hold only four chunks) against
//          ldmatrix bank conflicts
//   after the loop the same bytes hold the per-warp partials for the cross-warp merge.
template <int D>
struct Smem {
    static constexpr int kRowBytes = D * 2;
    static constexpr int kSwz = (D / 8 - 1) < 7 ? (D / 8 - 1) : 7;   // XOR mask of the 16-byte chunk index: stays inside the row
    static constexpr int kTileBytes = kTile * kRowBytes;
    static constexpr int kStageBytes = 2 * kTileBytes;
    static constexpr int kWarpBytes = kStages * kStageBytes;
    static constexpr int kRingBytes = kWarps * kWarpBytes;
    static constexpr int kMergeBytes = kWarps * kMaxHeads * (D + 2) * 4;
    static constexpr int kBytes = kRingBytes > kMergeBytes ? kRingBytes : kMergeBytes;
};

template <typename T, int D>
__global__ void __launch_bounds__(kThreads, 2) decode_splitk_kernel(const DecodeArgs a) {
    using S = Smem<D>;
    constexpr int kChunksPerRow = D / 8;          // 16-byte chunks per K/V row
    constexpr int kCopiesPerLane = kChunksPerRow / 2;  // a lane copies half a row of K and of V
    constexpr int kKSteps = D / 16;
    constexpr int kDBlocks = D / 8;
    extern __shared__ __align__(128) unsigned char smem_raw[];

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2;   // mma row group
    const int c4 = lane & 3;

    // A merge kernel launched with programmatic stream serialisation may take its place on the SMs as
    // soon as every CTA of this grid has started (it still waits for this grid to finish before it reads).
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");

    // KV heads vary fastest across the grid: the CTAs that read the adjacent 256-byte slices of the
    // same token rows (one slice per KV head) are launched together, which keeps DRAM pages open.
    const int kvh = blockIdx.x / a.head_blocks;
    const int hb = blockIdx.x - kvh * a.head_blocks;
    const int split = blockIdx.y;
    const int s = blockIdx.z;

    const int L = a.context_lens[s];
    const int chunk_begin = split * a.chunk;
    if (chunk_begin >= L) return;  // nothing cached here (L <= 0 included): the merge kernel writes zeros
    const int chunk_end = min(L, chunk_begin + a.chunk);

    const int group = a.q_heads / a.kv_heads;
    const int head0 = kvh * group + hb * kMaxHeads;            // first query head of this CTA
    const int nheads = min(kMaxHeads, group - hb * kMaxHeads);  // query heads served

    const T* __restrict__ qg = static_cast<const T*>(a.q);
    const T* __restrict__ kg = static_cast<const T*>(a.k);
    const T* __restrict__ vg = static_cast<const T*>(a.v);
    const long long kv_pitch = (long long)a.kv_heads * D;

    // Q fragments of the A operand, straight from global: row g and g+8 of the head block.
    unsigned qa[kKSteps][4];
    {
        const unsigned* q0 = reinterpret_cast<const unsigned*>(qg + ((long long)s * a.q_heads + head0 + g) * D);
        const unsigned* q1 = reinterpret_cast<const unsigned*>(qg + ((long long)s * a.q_heads + head0 + g + 8) * D);
        const bool v0 = g < nheads, v1 = g + 8 < nheads;
#pragma unroll
        for (int kk = 0; kk < kKSteps; ++kk) {
            qa[kk][0] = v0 ? q0[kk * 8 + c4] : 0u;
            qa[kk][1] = v1 ? q1[kk * 8 + c4] : 0u;
            qa[kk][2] = v0 ? q0[kk * 8 + 4 + c4] : 0u;
            qa[kk][3] = v1 ? q1[kk * 8 + 4 + c4] : 0u;
        }
    }

    float acc[kDBlocks][4];
#pragma unroll
    for (int n = 0; n < kDBlocks; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;
    float m0 = -INFINITY, m1 = -INFINITY;  // running max of rows g and g+8 (log2 domain)
    float l0 = 0.0f, l1 = 0.0f;            // this lane's share of the running sums

    unsigned char* ring = smem_raw + warp * S::kWarpBytes;
    const int n_tiles = (chunk_end - chunk_begin + kTile - 1) / kTile;   // tiles in the chunk
    const int my_tiles = (n_tiles - warp + kWarps - 1) / kWarps;         // tiles warp takes: warp, warp+4, ...

    // Copies of one tile: a K/V row (D*2 bytes) is moved by kChunksPerRow adjacent lanes, 16 bytes
    // each, so one warp instruction reads whole rows (full 128-byte lines). Lane r < 16 looks up the
    // slot of token row r once per tile; the other lanes get it by shuffle.
    constexpr int kRowsPerInstr = 32 / kChunksPerRow;      // 2 (D=128) or 4 (D=64)
    constexpr int kInstrPerTile = kTile / kRowsPerInstr;   // 8 or 4
    static_assert(kCopiesPerLane == kInstrPerTile, "a lane issues one 16-byte copy per instruction");
    const int cp_ch = lane % kChunksPerRow;
    const int cp_sub = lane / kChunksPerRow;
    auto issue = [&](int it) {
        if (it < my_tiles) {
            const int tile = warp + it * kWarps;
            const int j = chunk_begin + tile * kTile + (lane & 15);
            long long my_off = -1;   // element offset of token row (lane & 15), -1 when past the chunk
            if (j < chunk_end) {
                const int slot = block_slot(a.block_tables, s, a.max_blocks, j, a.block_size);
                my_off = (long long)slot * kv_pitch + (long long)kvh * D;
            }
            unsigned char* kst = ring + (it % kStages) * S::kStageBytes;
            unsigned char* vst = kst + S::kTileBytes;
#pragma unroll
            for (int i = 0; i < kInstrPerTile; ++i) {
                const int row = i * kRowsPerInstr + cp_sub;
                const long long off = __shfl_sync(0xffffffffu, my_off, row);
                const bool valid = off >= 0;
                const long long src = (valid ? off : 0) + cp_ch * 8;
                const int dst = row * S::kRowBytes + ((cp_ch ^ (row & S::kSwz)) << 4);
                cp_async_16(kst + dst, kg + src, valid);
                cp_async_16(vst + dst, vg + src, valid);
            }
        }
        cp_async_commit();  // committed even when empty so that group counting stays uniform
    };

#pragma unroll
    for (int it = 0; it < kStages - 1; ++it) issue(it);

    for (int it = 0; it < my_tiles; ++it) {
        issue(it + kStages - 1);
        cp_async_wait<kStages - 1>();
        __syncwarp();

        const unsigned char* kst = ring + (it % kStages) * S::kStageBytes;
        const unsigned char* vst = kst + S::kTileBytes;
        const int tile_tok0 = chunk_begin + (warp + it * kWarps) * kTile;

        // S = Q K^T : 16 heads x 16 tokens as two N blocks of 8 tokens
        float sc[2][4];
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) sc[nb][0] = sc[nb][1] = sc[nb][2] = sc[nb][3] = 0.0f;
        {
            const int mi = lane >> 3;                    // which 8x8 matrix this lane addresses
            const int tok = ((mi >> 1) << 3) + (lane & 7);  // token row
#pragma unroll
            for (int kk = 0; kk < kKSteps; ++kk) {
                const int ch = 2 * kk + (mi & 1);
                unsigned b0, b1, b2, b3;
                ldmatrix_x4(b0, b1, b2, b3, kst + tok * S::kRowBytes + ((ch ^ (tok & S::kSwz)) << 4));
                mma_16816<T>(sc[0], qa[kk], b0, b1);
                mma_16816<T>(sc[1], qa[kk], b2, b3);
            }
        }

        // scale, mask the tail of the chunk, online softmax over this tile's 16 tokens
        float tmax0 = -INFINITY, tmax1 = -INFINITY;
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int j = tile_tok0 + nb * 8 + 2 * c4 + e;
                const bool vis = j < chunk_end;
                sc[nb][e] = vis ? sc[nb][e] * a.scale_log2 : -INFINITY;
                sc[nb][2 + e] = vis ? sc[nb][2 + e] * a.scale_log2 : -INFINITY;
                tmax0 = fmaxf(tmax0, sc[nb][e]);
                tmax1 = fmaxf(tmax1, sc[nb][2 + e]);
            }
        }
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 1));
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 2));
        tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 1));
        tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 2));
        // every tile inside the chunk has at least its first token visible, so the maxima are finite
        const float mn0 = fmaxf(m0, tmax0), mn1 = fmaxf(m1, tmax1);
        const float alpha0 = fast_exp2(m0 - mn0), alpha1 = fast_exp2(m1 - mn1);
        m0 = mn0;
        m1 = mn1;
        float ps0 = 0.0f, ps1 = 0.0f;
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                sc[nb][e] = fast_exp2(sc[nb][e] - mn0);
                sc[nb][2 + e] = fast_exp2(sc[nb][2 + e] - mn1);
                ps0 += sc[nb][e];
                ps1 += sc[nb][2 + e];
            }
        }
        l0 = l0 * alpha0 + ps0;
        l1 = l1 * alpha1 + ps1;
#pragma unroll
        for (int n = 0; n < kDBlocks; ++n) {
            acc[n][0] *= alpha0;
            acc[n][1] *= alpha0;
            acc[n][2] *= alpha1;
            acc[n][3] *= alpha1;
        }

        // O += P V : P (16 heads x 16 tokens) re-used from the accumulator layout as the A operand
        unsigned pa[4];
        pa[0] = pack2<T>(sc[0][0], sc[0][1]);
        pa[1] = pack2<T>(sc[0][2], sc[0][3]);
        pa[2] = pack2<T>(sc[1][0], sc[1][1]);
        pa[3] = pack2<T>(sc[1][2], sc[1][3]);
        {
            const int mi = lane >> 3;
            const int tok = ((mi & 1) << 3) + (lane & 7);
#pragma unroll
            for (int n = 0; n < kDBlocks; n += 2) {
                const int ch = n + (mi >> 1);
                unsigned b0, b1, b2, b3;
                ldmatrix_x4_trans(b0, b1, b2, b3, vst + tok * S::kRowBytes + ((ch ^ (tok & S::kSwz)) << 4));
                mma_16816<T>(acc[n], pa, b0, b1);
                mma_16816<T>(acc[n + 1], pa, b2, b3);
            }
        }
        __syncwarp();  // the stage may be refilled by the next issue()
    }
    cp_async_wait<0>();

    // row sums: fold the four lanes that share a row
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    // cross-warp merge through shared memory (the ring is dead now)
    __syncthreads();
    float* merge = reinterpret_cast<float*>(smem_raw);
    float* macc = merge + warp * kMaxHeads * (D + 2);  // [head][D + 2]: acc, m, l
#pragma unroll
    for (int n = 0; n < kDBlocks; ++n) {
        const int d = n * 8 + 2 * c4;
        macc[g * (D + 2) + d] = acc[n][0];
        macc[g * (D + 2) + d + 1] = acc[n][1];
        macc[(g + 8) * (D + 2) + d] = acc[n][2];
        macc[(g + 8) * (D + 2) + d + 1] = acc[n][3];
    }
    if (c4 == 0) {
        macc[g * (D + 2) + D] = m0;
        macc[g * (D + 2) + D + 1] = l0;
        macc[(g + 8) * (D + 2) + D] = m1;
        macc[(g + 8) * (D + 2) + D + 1] = l1;
    }
    __syncthreads();

    for (int idx = threadIdx.x; idx < nheads * D; idx += kThreads) {
        const int hh = idx / D;
        const int d = idx - hh * D;
        float mw[kWarps];
        float mstar = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            mw[w] = merge[(w * kMaxHeads + hh) * (D + 2) + D];
            mstar = fmaxf(mstar, mw[w]);
        }
        float o = 0.0f, l = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float wgt = (mw[w] == -INFINITY) ? 0.0f : fast_exp2(mw[w] - mstar);
            o += wgt * merge[(w * kMaxHeads + hh) * (D + 2) + d];
            l += wgt * merge[(w * kMaxHeads + hh) * (D + 2) + D + 1];
        }
        const long long row = ((long long)s * a.q_heads + head0 + hh) * a.max_splits + split;
        a.ws_acc[row * D + d] = o;
        if (d == 0) a.ws_ml[row] = make_float2(mstar, l);
    }
}

// Where the merged rows go: one buffer of (num_seqs, 1, o_heads, D), or — head-sharded decode with
// the output all-gather fused in — the same tensor on every GPU of the group (peer memory, plain
// stores over NVLink), each receiving this call's heads at head offset o_head0.
struct MergeOut {
    void* o[8];
    int n_out, o_heads, o_head0, peer0;
};

// Merges the split-K partials of one (sequence, query head) and writes the output row.
template <typename T, int D>
__global__ void __launch_bounds__(D) decode_merge_kernel(const float* __restrict__ ws_acc,
                                                         const float2* __restrict__ ws_ml,
                                                         const int* __restrict__ context_lens,
                                                         const MergeOut out, int q_heads, int chunk,
                                                         int max_splits) {
    const int h = blockIdx.x;
    const int s = blockIdx.y;
    const int d = threadIdx.x;
    const int L = context_lens[s];
    const int n = L > 0 ? min(max_splits, (L + chunk - 1) / chunk) : 0;
    // the split-K grid this one depends on has finished and its partials are visible (returns at once
    // when the launch carries no programmatic dependency)
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    const long long row0 = ((long long)s * q_heads + h) * max_splits;
    float mstar = -INFINITY;
    for (int i = 0; i < n; ++i) mstar = fmaxf(mstar, ws_ml[row0 + i].x);
    float acc = 0.0f, l = 0.0f;
    for (int i = 0; i < n; ++i) {
        const float2 ml = ws_ml[row0 + i];
        const float w = (ml.x == -INFINITY) ? 0.0f : fast_exp2(ml.x - mstar);
        acc += w * ws_acc[(row0 + i) * D + d];
        l += w * ml.y;
    }
    // reference: inv = l > 0 ? 1/l : 0 (flash_attn_with_kvcache.cu:109)
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    const T val = from_f32<T>(acc * inv);
    const long long off = ((long long)s * out.o_heads + out.o_head0 + h) * D + d;
    int pe = out.peer0;
    for (int n = 0; n < out.n_out; ++n) {
        static_cast<T*>(out.o[pe])[off] = val;
        pe = pe + 1 == out.n_out ? 0 : pe + 1;
    }
}

MergeOut merge_out_single(void* o, int q_heads) {
    MergeOut m{};
    m.o[0] = o;
    m.n_out = 1;
    m.o_heads = q_heads;
    return m;
}

// Tokens per work item. A CTA needs several microseconds to fill its copy pipeline, so long
// chunks win as long as there are enough of them: the largest of 4096/2048/1024 that still yields
// >= 1500 work items (about 5 waves of 2 CTAs x 148 SMs, counted at the maximum length), else the
// largest chunk >= 256 that yields at least 256. `base` = work items per split.
static int auto_chunk(long long base, long long max_tokens) {
    auto items = [&](int c) { return base * ((max_tokens + c - 1) / c); };
    for (int c = 4096; c >= 1024; c >>= 1)
        if (items(c) >= 1500) return c;
    for (int c = 4096; c >= 256; c >>= 1)
        if (items(c) >= 256) return c;
    return 256;
}

template <typename T, int D>
int launch_typed(const AttnParams& p, cudaStream_t stream) {
    using S = Smem<D>;
    const int group = p.q_heads / p.kv_heads;
    const int head_blocks = (group + kMaxHeads - 1) / kMaxHeads;
    const long long max_tokens = (long long)p.max_blocks * p.block_size;
    if (max_tokens <= 0) return -1;

    const int unit = kWarps * kTile;
    int chunk = get_option_decode_chunk();
    if (chunk <= 0) chunk = auto_chunk((long long)p.num_seqs * p.kv_heads * head_blocks, max_tokens);
    chunk = ((chunk + unit - 1) / unit) * unit;
    const long long max_splits_ll = (max_tokens + chunk - 1) / chunk;
    if (max_splits_ll > 65535 || p.num_seqs > 65535 || (long long)p.kv_heads * head_blocks > 65535) return -1;
    const int max_splits = (int)max_splits_ll;

    const size_t rows = (size_t)p.num_seqs * p.q_heads * max_splits;
    const size_t acc_bytes = rows * D * sizeof(float);
    const size_t ml_bytes = rows * sizeof(float2);
    unsigned char* ws = static_cast<unsigned char*>(decode_workspace(stream, acc_bytes + ml_bytes));
    if (ws == nullptr) {
        set_last_errorf("flash_attn_with_kvcache: could not allocate %zu bytes of split-K workspace",
                        acc_bytes + ml_bytes);
        return FLASH_ATTN_ERR_CUDA;
    }

    DecodeArgs a{};
    a.q = p.q; a.k = p.k; a.v = p.v;
    a.block_tables = p.block_tables;
    a.context_lens = p.context_lens;
    a.ws_acc = reinterpret_cast<float*>(ws);
    a.ws_ml = reinterpret_cast<float2*>(ws + acc_bytes);
    a.num_seqs = p.num_seqs;
    a.q_heads = p.q_heads;
    a.kv_heads = p.kv_heads;
    a.block_size = p.block_size;
    a.max_blocks = p.max_blocks;
    a.chunk = chunk;
    a.max_splits = max_splits;
    a.head_blocks = head_blocks;
    a.scale_log2 = p.scale * 1.4426950408889634f;

    cudaError_t err = cudaFuncSetAttribute(decode_splitk_kernel<T, D>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, S::kBytes);
    if (err != cudaSuccess) {
        set_last_errorf("decode_splitk_kernel: %s", cudaGetErrorString(err));
        cudaGetLastError();
        return FLASH_ATTN_ERR_CUDA;
    }
    dim3 grid(p.kv_heads * head_blocks, max_splits, p.num_seqs);
    decode_splitk_kernel<T, D><<<grid, kThreads, S::kBytes, stream>>>(a);
    int rc = check_launch("decode_splitk_kernel");
    if (rc != FLASH_ATTN_OK) return rc;
    dim3 mgrid(p.q_heads, p.num_seqs);
    MergeOut mo = merge_out_single(p.o, p.q_heads);
    if (p.n_out > 0) {
        for (int i = 0; i < p.n_out && i < 8; ++i) mo.o[i] = p.o_peers[i];
        mo.n_out = p.n_out;
        mo.o_heads = p.o_heads;
        mo.o_head0 = p.o_head0;
        mo.peer0 = (p.o_head0 / p.q_heads + 1) % p.n_out;
    }
    {
        // programmatic dependent launch: the merge grid is set up while the split-K grid drains
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = mgrid;
        cfg.blockDim = dim3(D);
        cfg.dynamicSmemBytes = 0;
        cfg.stream = stream;
        cudaLaunchAttribute attr{};
        attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr.val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        const float* ws_acc = a.ws_acc;
        const float2* ws_ml = a.ws_ml;
        const int* lens = p.context_lens;
        const int q_heads = p.q_heads;
        cudaLaunchKernelEx(&cfg, decode_merge_kernel<T, D>, ws_acc, ws_ml, lens, mo, q_heads, chunk, max_splits);
    }
    rc = check_launch("decode_merge_kernel");
    if (rc == FLASH_ATTN_OK) note_path("decode_splitk", 2);
    return rc;
}

}  // namespace

int launch_decode_splitk(const AttnParams& p, cudaStream_t stream) {
    if (p.mode != MODE_KVCACHE || p.q_seq_len != 1) return -1;
    if (p.dtype != DT_F16 && p.dtype != DT_BF16) return -1;
    if (p.head_size != 32 && p.head_size != 64 && p.head_size != 128) return -1;
    if (p.q_heads > 65535) return -1;
    // 16-byte cp.async needs 16-byte aligned rows
    if ((reinterpret_cast<uintptr_t>(p.k) | reinterpret_cast<uintptr_t>(p.v)) & 15) return -1;
    if (reinterpret_cast<uintptr_t>(p.q) & 3) return -1;
    if (p.dtype == DT_BF16) {
        return p.head_size == 128 ? launch_typed<__nv_bfloat16, 128>(p, stream)
               : p.head_size == 64 ? launch_typed<__nv_bfloat16, 64>(p, stream)
                                   : launch_typed<__nv_bfloat16, 32>(p, stream);
    }
    return p.head_size == 128 ? launch_typed<__half, 128>(p, stream)
           : p.head_size == 64 ? launch_typed<__half, 64>(p, stream)
                               : launch_typed<__half, 32>(p, stream);
}

// ---------------------------------------------------------------------------------------------
// Decode without any allocation: the split-K partials live in a fixed array that is part of the
// library image instead of a cudaMalloc'ed workspace.
//
// Who needs this: a serving engine that hands all of HBM to its own pool at start-up leaves
// nothing for a library-side cudaMalloc to find, so the ordinary decode entry point can fail (or
// fragment the pool) the first time it has to size its workspace; and a caller in the middle of
// a latency-critical step cannot afford cudaMalloc / cudaFree, which take the driver's allocation
// lock and synchronise the whole device. For them the scratch is paid for once, when the library
// is loaded: every GPU whose context loads libflash_attn holds kStaticScratchBytes of it until
// the process exits, whether or not this entry point is ever called. "Loaded" is meant literally:
// with CUDA's default lazy module loading the array gets its memory when the first kernel or
// symbol of this translation unit is touched on a device — possibly the first call here — so a
// caller that is about to give away all free memory makes one small call first (or sets
// CUDA_MODULE_LOADING=EAGER); an out-of-memory answer at that point is reported as such.
//
// In host code `g_static_scratch` is only a handle for the symbol, not a device address; the
// device address is fetched once per device with cudaGetSymbolAddress (with that device current)
// and passed to the same two kernels the ordinary path launches.
// ---------------------------------------------------------------------------------------------
namespace {

constexpr size_t kStaticScratchBytes = size_t(16) << 20;   // 16 MiB per GPU
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_static_mutex;
unsigned char* g_static_ptr[kMaxDevices] = {nullptr};

// Device address of the static scratch on the CURRENT device; resolved on first use per device.
unsigned char* static_scratch_ptr() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        cudaGetLastError();
        set_last_error("flash_attn_decode_bf16_noalloc: cannot identify the current device");
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (g_static_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        const cudaError_t err = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (err != cudaSuccess || ptr == nullptr) {
            cudaGetLastError();
            if (err == cudaErrorMemoryAllocation) {
                // lazy module loading: this first call is what backs the array, and no memory is left for it
                set_last_errorf("flash_attn_decode_bf16_noalloc: the library's %zu-byte scratch array could not be backed with "
                                "device memory. CUDA loads device code lazily: make the first call on each device before "
                                "the application reserves all device memory, or set CUDA_MODULE_LOADING=EAGER",
                                kStaticScratchBytes);
            } else {
                set_last_errorf("flash_attn_decode_bf16_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(err));
            }
            return nullptr;
        }
        g_static_ptr[dev] = static_cast<unsigned char*>(ptr);
    }
    return g_static_ptr[dev];
}

template <int D>
int launch_static(const void* q, const void* k, const void* v, void* o, const int* block_tables,
                  const int* context_lens, int num_seqs, int q_heads, int kv_heads, int block_size,
                  int max_blocks, float scale, cudaStream_t stream) {
    using T = __nv_bfloat16;
    using S = Smem<D>;
    const int group = q_heads / kv_heads;
    const int head_blocks = (group + kMaxHeads - 1) / kMaxHeads;
    const long long max_tokens = (long long)max_blocks * block_size;
    const int unit = kWarps * kTile;

    // one split must always fit; beyond that the chunk grows until the partials fit the array
    const size_t row_bytes = (size_t)D * sizeof(float) + sizeof(float2);
    const size_t rows1 = (size_t)num_seqs * q_heads;
    if (rows1 * row_bytes > kStaticScratchBytes) {
        set_last_errorf("flash_attn_decode_bf16_noalloc: num_seqs*q_heads = %zu exceeds the static scratch "
                        "(%zu bytes hold at most %zu rows of head_size %d); use flash_attn_with_kvcache_bf16",
                        rows1, kStaticScratchBytes, kStaticScratchBytes / row_bytes, D);
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    long long chunk = auto_chunk((long long)num_seqs * kv_heads * head_blocks, max_tokens);
    {
        while (rows1 * (size_t)((max_tokens + chunk - 1) / chunk) * row_bytes > kStaticScratchBytes) chunk <<= 1;
    }
    chunk = ((chunk + unit - 1) / unit) * unit;
    const long long max_splits_ll = (max_tokens + chunk - 1) / chunk;
    if (chunk > 0x40000000LL || max_splits_ll > 65535 || num_seqs > 65535 || (long long)kv_heads * head_blocks > 65535 ||
        q_heads > 65535) {
        set_last_error("flash_attn_decode_bf16_noalloc: grid dimensions out of range");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    const int max_splits = (int)max_splits_ll;
    const size_t rows = rows1 * max_splits;
    const size_t acc_bytes = rows * D * sizeof(float);   // a multiple of 256 bytes, so the float2 part stays aligned

    unsigned char* ws = static_scratch_ptr();
    if (ws == nullptr) return FLASH_ATTN_ERR_CUDA;

    DecodeArgs a{};
    a.q = q; a.k = k; a.v = v;
    a.block_tables = block_tables;
    a.context_lens = context_lens;
    a.ws_acc = reinterpret_cast<float*>(ws);
    a.ws_ml = reinterpret_cast<float2*>(ws + acc_bytes);
    a.num_seqs = num_seqs;
    a.q_heads = q_heads;
    a.kv_heads = kv_heads;
    a.block_size = block_size;
    a.max_blocks = max_blocks;
    a.chunk = (int)chunk;
    a.max_splits = max_splits;
    a.head_blocks = head_blocks;
    a.scale_log2 = scale * 1.4426950408889634f;

    cudaError_t err = cudaFuncSetAttribute(decode_splitk_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           S::kBytes);
    if (err != cudaSuccess) {
        set_last_errorf("decode_splitk_kernel: %s", cudaGetErrorString(err));
        cudaGetLastError();
        return FLASH_ATTN_ERR_CUDA;
    }
    dim3 grid(kv_heads * head_blocks, max_splits, num_seqs);
    decode_splitk_kernel<T, D><<<grid, kThreads, S::kBytes, stream>>>(a);
    int rc = check_launch("decode_splitk_kernel");
    if (rc != FLASH_ATTN_OK) return rc;
    dim3 mgrid(q_heads, num_seqs);
    decode_merge_kernel<T, D><<<mgrid, D, 0, stream>>>(a.ws_acc, a.ws_ml, context_lens, merge_out_single(o, q_heads), q_heads,
                                                      (int)chunk, max_splits);
    rc = check_launch("decode_merge_kernel");
    if (rc == FLASH_ATTN_OK) note_path("decode_splitk_static", 2);
    return rc;
}

}  // namespace
}  // namespace fa

extern "C" int flash_attn_decode_bf16_noalloc(const flash_attn_bf16_t* q, const flash_attn_bf16_t* k_cache,
                                              const flash_attn_bf16_t* v_cache, flash_attn_bf16_t* o,
                                              const int* block_tables, const int* context_lens, int num_seqs,
                                              int q_heads, int kv_heads, int head_size, int block_size,
                                              int max_blocks, float scale, void* stream) {
    using namespace fa;
    set_last_error("");
    cudaGetLastError();
    if (!q || !k_cache || !v_cache || !o || !block_tables || !context_lens) {
        set_last_error("flash_attn_decode_bf16_noalloc: null pointer argument");
        return FLASH_ATTN_ERR_NULL_PTR;
    }
    if (num_seqs <= 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0 || block_size <= 0 || max_blocks <= 0) {
        set_last_error("flash_attn_decode_bf16_noalloc: num_seqs/heads/block_size/max_blocks must be > 0 and "
                       "q_heads a multiple of kv_heads");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    if (head_size != 64 && head_size != 128) {
        set_last_error("flash_attn_decode_bf16_noalloc: head_size must be 64 or 128");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    if (((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 15) ||
        (reinterpret_cast<uintptr_t>(q) & 3)) {
        set_last_error("flash_attn_decode_bf16_noalloc: k_cache/v_cache must be 16-byte aligned, q 4-byte aligned");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    // launch on the device that owns q, and resolve the scratch address on that same device
    int prev = -1;
    bool switched = false;
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, q) == cudaSuccess && attr.type == cudaMemoryTypeDevice &&
        cudaGetDevice(&prev) == cudaSuccess && attr.device != prev) {
        if (cudaSetDevice(attr.device) != cudaSuccess) {
            cudaGetLastError();
            set_last_error("flash_attn_decode_bf16_noalloc: could not select the device that owns q");
            return FLASH_ATTN_ERR_CUDA;
        }
        switched = true;
    }
    cudaGetLastError();
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int rc = head_size == 128
                       ? launch_static<128>(q, k_cache, v_cache, o, block_tables, context_lens, num_seqs, q_heads,
                                            kv_heads, block_size, max_blocks, scale, st)
                       : launch_static<64>(q, k_cache, v_cache, o, block_tables, context_lens, num_seqs, q_heads,
                                           kv_heads, block_size, max_blocks, scale, st);
    if (switched) cudaSetDevice(prev);
    return rc;
}
