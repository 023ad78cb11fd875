// Causal, GQA-capable flash-attention prefill forward for sm_100a: TMA-fed Q/K/V tiles,
// tcgen05.mma with the S and O accumulators in tensor memory, online softmax in registers,
// warp-specialised roles. Handles f16/bf16 storage with head_size 128, 64, or 32 on zero-padded 64-column tiles (template parameter D;
// the layout comments below give the D = 128 figures) for the batched entry point (optional
// key-padding mask: template parameter kMask), chunked prefill over a paged cache, and the packed varlen entry point (with
// or without the packed buffers' row counts). Replaces flash_attn_kernel
// (luma-flash-attn/kernels/flash_attn_func.cu:29-226), flash_attn_prefill_kernel
// (kernels/flash_attn_with_kvcache.cu:157-277) and flash_attn_varlen_kernel
// (kernels/flash_attn_varlen_func.cu:35-199), one-thread-per-query-row scalar kernels.
//
// One CTA (384 threads, 1 per SM) owns up to two query tiles of 128 rows that share a batch
// element and a KV head — two query heads of one GQA group at the same row block, or two
// consecutive row blocks of one head when the group is 1 (tile 0 the later one) — and streams that KV head's K/V tiles
// (128 keys) past both:
//   warps 0-3 / 4-7 : softmax warpgroup of query tile 0 / 1 — one thread per query row: read S
//                     from tensor memory (tcgen05.ld), running max / sum in registers (exp2 with
//                     the scale folded in), write P as packed 16-bit back over S (tcgen05.st),
//                     rescale O in tensor memory only when the row max moved by more than 2^8,
//                     final normalisation of O, staged in Q's shared memory and written with bulk
//                     tensor stores (and LSE); setmaxnreg gives these warps 208 registers
//   warp 8 / 10     : TMA producers — warp 8 loads Q once, then the K tiles; warp 10 the V tiles; two 2-stage rings
//   warp 9          : MMA issuer — S_t = Q_t K^T (SS form), O_t += P_t V (P from tensor memory),
//                     completion signalled with tcgen05.commit on mbarriers; the warp runs converged
//                     and one elected lane issues
//   warp 11         : idle (completes the third warpgroup, which setmaxnreg needs whole)
// While one warpgroup runs its softmax the tensor core works on the other tile.
// Tensor memory (512 columns): S0 | S1 | O0 | O1, 128 fp32 columns each; P_t aliases S_t.
// Shared memory: Q 2 x 32 KiB, K ring 2 x 32 KiB, V ring 2 x 32 KiB, all 128-byte swizzled
// exactly as TMA writes them, so the MMA descriptors address them in place.
//
// Every wait on an mbarrier is bounded (about 2 s of wall clock); on expiry the CTA records a
// status word in global memory, stops waiting everywhere, drains its own TMA copies, frees its
// tensor memory and returns.
#include <cuda.h>

#include <algorithm>
#include <cstring>
#include <mutex>
#include <type_traits>

#include "common.cuh"

namespace fa {

namespace {

constexpr int kBlockM = 128;   // query rows per tile
constexpr int kBlockN = 128;   // keys per K/V tile
// head size D (64 or 128) is a template parameter of the kernel
constexpr int kStages = 2;     // K ring depth
// V ring depth. Two, like K: a third stage fits the 227 KiB of shared memory and takes the MMA
// issuer's ~350-clock wait for V out of every step (a bulk copy needs about 2 us to land while 148
// CTAs stream their tiles out of L2, and a V stage is released later than a K stage), but measured
// 5 % slower on every prefill workload (1165 against 1228 TFLOP/s at S = 8192, same box).
constexpr int kStagesV = 2;
constexpr int kThreads = 384;   // three warpgroups: softmax 0, softmax 1, and producer + issuer (+ two idle warps)
constexpr int kLoadWarp = 8;
constexpr int kMmaWarp = 9;
constexpr int kLoadWarpV = 10;   // V-ring producer (K ring and Q: kLoadWarp)
constexpr int kHalfBytes = kBlockN * 64 * 2;   // 16 KiB: one 64-column half, 128 rows x 128 B
template <int D> struct TileBytes { static constexpr int value = kBlockN * D * 2; };   // one half at D = 64, two at D = 128
constexpr float kRescaleThreshold = 8.0f;            // log2 units

// Which element pairs of an unmasked chunk take their exponential on the FMA pipe (a cubic) instead
// of the special-function unit: one pair in eight. Measured on the S = 8192 GQA prefill, same box:
// none 1231, one in eight 1237, one in four 1207, three in eight 1128, one in two 1058 TFLOP/s — the
// cubic costs about as many issue slots as the special-function unit saves, so the share is small.
__device__ __forceinline__ constexpr bool fma_pipe_exp(int i) { return (i & 7) == 7; }

template <int D>
struct SharedStorage {
    alignas(1024) unsigned char q[2][TileBytes<D>::value];
    alignas(1024) unsigned char k[kStages][TileBytes<D>::value];
    alignas(1024) unsigned char v[kStagesV][TileBytes<D>::value];
    alignas(8) unsigned long long q_full[2];
    unsigned long long k_full[kStages], k_empty[kStages];
    unsigned long long v_full[kStagesV], v_empty[kStagesV];
    unsigned long long s_full[2];   // MMA -> softmax: S_t ready (and every earlier MMA finished)
    unsigned long long p_lo[2];     // softmax -> MMA: keys 0-63 of P_t written, O_t rescaled
    unsigned long long p_hi[2];     // softmax -> MMA: keys 64-127 of P_t written
    unsigned long long v_tail;      // copy engine -> V producer: the sequence's last, partly filled V tile has landed
    unsigned long long drain;       // MMA issuer, error path only: every product issued so far has finished
    unsigned int tmem_base;
    volatile int abort_flag;
};

constexpr int kMaxPeers = 8;
#ifdef FA_TRACE
constexpr int kCtaLogEntries = 2048;
#endif
constexpr unsigned long long kWaitLimitNs = 2000000000ULL;   // default bound of every mbarrier wait

struct PrefillArgs {
    // Output: n_out buffers of (batch, q_seq_len, o_heads, 128), each receiving this launch's heads
    // at head offset o_head0. n_out == 1 with o_heads == q_heads is the ordinary call; with n_out > 1
    // the buffers are the same tensor on every GPU of a head-sharded group (peer memory over
    // NVLink), which makes the output all-gather part of the epilogue.
    void* o[kMaxPeers];
    int n_out, o_heads, o_head0;
    int peer0;          // n_out > 1: the buffer this CTA's rows go to first; each CTA walks the buffers from there
    int multicast;      // o[0] is an NVSwitch multicast address of the group's output tensors: one multimem.st reaches all of them
    float* lse;         // (batch, q_heads, q_seq_len) of this call, or null
    float* lse_peers[kMaxPeers];   // n_lse > 0: (batch, o_heads, q_seq_len) on every GPU of the group, written at head o_head0
    int n_lse;
    int* status;        // word in mapped host memory, set to non-zero when a bounded wait expired
    unsigned long long wait_ns;    // bound of every mbarrier wait
    int test_skip_k;    // test hook: the K producer leaves out tile (test_skip_k - 1), so that a wait runs out; 0 = off
#ifdef FA_TRACE
    int staged_store;   // 1 = stage O rows in shared memory and store whole rows even for a single output
    long long* trace;  // optional timeline of one CTA (clock64 stamps), null unless the "prefill_trace" option is set
    int trace_y;       // blockIdx.y of the traced CTA (option "prefill_trace_y", default 0 = the heaviest)
    long long* cta_log;  // optional per-CTA {start ns, end ns, SM id} records ("prefill_trace" = 3), up to kCtaLogEntries
#endif
    int batch, q_seq_len, kv_seq_len, q_heads, kv_heads, start_pos;
    int d_real;     // head size of the tensors: D, or 32 when the D = 64 kernel runs a head size of 32 on zero-padded tiles
    int band;       // tile pairs of one (batch, KV head) that sit next to each other in blockIdx.x
    // Launch order of the bands (blockIdx.y), heaviest = 0. spread_w == 0: heaviest first. Otherwise the
    // first spread_w rows of the grid are every spread_m-th band (a first wave that mixes all weights,
    // so that CTAs end at spread-out times from the start), the other bands follow heaviest first.
    int spread_w, spread_m;
    // which entry point the problem came from (fa::Mode) and its per-sequence descriptors
    int mode;                   // MODE_BATCH: uniform q_seq_len / kv_seq_len / start_pos
    const void* q;              // MODE_VARLEN: the packed q / k / v buffers themselves, for the tiles at their very end
    const void* k;
    const void* v;
    const unsigned char* mask;  // MODE_BATCH: optional (batch, kv_seq_len) key-padding mask, 1 = valid key
    const int* cu_q;            // MODE_VARLEN: packed row offsets of q / o
    const int* cu_k;            // MODE_VARLEN: packed row offsets (or, paged, lengths by difference) of k / v
    const int* context_lens;    // MODE_KVCACHE: cached length per sequence, query tokens included
    const int* block_tables;    // paged K/V: (batch, max_blocks) logical -> physical block
    int paged, block_size, max_blocks;
    float scale_log2;
};

// ---- PTX wrappers -------------------------------------------------------------------------
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("{\n.reg .b64 st;\nmbarrier.arrive.shared::cta.b64 st, [%0];\n}\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("{\n.reg .b64 st;\nmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n}\n" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t));
    return t;
}

// Bounded wait. Returns false when the wait was abandoned (time limit, or another thread of the
// CTA already gave up); the caller then falls through to the end of the kernel.
// The status word lives in mapped host memory (the host reads it without touching the device), so it
// is written with a plain store: the code of one of the waits that expired.
template <typename Storage>
__device__ __forceinline__ bool mbar_wait(Storage& sm, unsigned long long* bar, unsigned parity, const PrefillArgs& a,
                                          int where) {
    if (mbar_try_wait(bar, parity)) return true;
    // the bound is counted in SM clocks (cheap to read, unlike the global nanosecond timer):
    // wait_ns x 2 clocks, i.e. at least wait_ns of wall time at any SM clock up to 2 GHz
    const long long t0 = clock64();
    const long long limit = (long long)(a.wait_ns * 2ULL);
    for (unsigned spin = 1;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 63u) == 0u) {
            if (sm.abort_flag) return false;
            if (clock64() - t0 > limit) {
                sm.abort_flag = 1;
                *reinterpret_cast<volatile int*>(a.status) = where;
                __threadfence_system();
                return false;
            }
        }
    }
}

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, unsigned long long* bar, int c0, int c1,
                                            int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];\n" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// Bulk tensor store shared -> global of one box, tracked by the issuing thread's bulk group.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, const void* src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];\n" ::"l"(map),
                 "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}

// 16 bytes to an NVSwitch multicast address: the switch replicates the store into the same offset of
// every GPU's memory bound to the multicast object (the bits are stored as they are).
__device__ __forceinline__ void multimem_st16(void* mc_addr, const uint4& w) {
    asm volatile("multimem.st.global.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"l"(mc_addr), "r"(w.x), "r"(w.y), "r"(w.z), "r"(w.w)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

// Executed by the whole (converged) issuer warp; one elected lane commits.
__device__ __forceinline__ void tc_commit(unsigned long long* bar) {
    asm volatile("{\n.reg .pred e;\nelect.sync _|e, 0xffffffff;\n@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n}\n" ::"r"(smem_u32(bar)) : "memory");
}

// The products as the issuer warp runs them: the whole warp executes the instruction stream
// converged and one elected lane issues. Keeping the warp uniform lets the descriptors live in
// uniform registers, so a product costs a handful of issue slots; issued from a single diverged
// lane each needs register-to-uniform moves and, next to ALU-heavy warps on the same scheduler,
// took ~130 clocks instead of the tensor pipe's 64. The accumulate flag is a compile-time constant.
// D[tmem] (+)= A[smem] * B[smem]
template <bool kAccumulate>
__device__ __forceinline__ void tc_mma_ss_imm(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc, unsigned idesc) {
    if (kAccumulate)
        asm volatile("{\n.reg .pred p, e;\nelect.sync _|e, 0xffffffff;\nsetp.ne.b32 p, 1, 0;\n@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
                     "l"(a_desc), "l"(b_desc), "r"(idesc)
                     : "memory");
    else
        asm volatile("{\n.reg .pred p, e;\nelect.sync _|e, 0xffffffff;\nsetp.ne.b32 p, 0, 0;\n@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
                     "l"(a_desc), "l"(b_desc), "r"(idesc)
                     : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
template <bool kAccumulate>
__device__ __forceinline__ void tc_mma_ts_imm(unsigned d_tmem, unsigned a_tmem, unsigned long long b_desc, unsigned idesc) {
    if (kAccumulate)
        asm volatile("{\n.reg .pred p, e;\nelect.sync _|e, 0xffffffff;\nsetp.ne.b32 p, 1, 0;\n@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d_tmem),
                     "r"(a_tmem), "l"(b_desc), "r"(idesc)
                     : "memory");
    else
        asm volatile("{\n.reg .pred p, e;\nelect.sync _|e, 0xffffffff;\nsetp.ne.b32 p, 0, 0;\n@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d_tmem),
                     "r"(a_tmem), "l"(b_desc), "r"(idesc)
                     : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp <-> TMEM lane (base + i)
__device__ __forceinline__ void tc_ld32(unsigned taddr, float (&r)[32]) {
    unsigned* u = reinterpret_cast<unsigned*>(r);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
          "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]), "=r"(u[16]),
          "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]), "=r"(u[24]),
          "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_st32(unsigned taddr, const unsigned (&u)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::"r"(
            taddr),
        "r"(u[0]), "r"(u[1]), "r"(u[2]), "r"(u[3]), "r"(u[4]), "r"(u[5]), "r"(u[6]), "r"(u[7]), "r"(u[8]), "r"(u[9]),
        "r"(u[10]), "r"(u[11]), "r"(u[12]), "r"(u[13]), "r"(u[14]), "r"(u[15]), "r"(u[16]), "r"(u[17]), "r"(u[18]),
        "r"(u[19]), "r"(u[20]), "r"(u[21]), "r"(u[22]), "r"(u[23]), "r"(u[24]), "r"(u[25]), "r"(u[26]), "r"(u[27]),
        "r"(u[28]), "r"(u[29]), "r"(u[30]), "r"(u[31])
        : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns
__device__ __forceinline__ void tc_st16(unsigned taddr, const unsigned (&u)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n" ::"r"(taddr),
        "r"(u[0]), "r"(u[1]), "r"(u[2]), "r"(u[3]), "r"(u[4]), "r"(u[5]), "r"(u[6]), "r"(u[7]), "r"(u[8]), "r"(u[9]),
        "r"(u[10]), "r"(u[11]), "r"(u[12]), "r"(u[13]), "r"(u[14]), "r"(u[15])
        : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// Two f32 lanes in one 64-bit register for the packed FMA-pipe instructions of sm_100.
__device__ __forceinline__ unsigned long long pack2(float a, float b) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack2(unsigned long long r, float& a, float& b) {
    asm("mov.b64 {%0, %1}, %2;\n" : "=f"(a), "=f"(b) : "l"(r));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
// 2^x for two finite x on the FMA pipe instead of the special-function unit: x = n + f with n the
// nearest integer (magic-number rounding), a cubic for 2^f on [-0.5, 0.5] (relative error 7.5e-5,
// far below the 16-bit rounding of P), and n added to the exponent field. x is clamped at -126,
// so the result is never below 2^-126 — callers use this only where no element is masked.
__device__ __forceinline__ void ex2_fma2(float x0, float x1, float& p0, float& p1) {
    x0 = fmaxf(x0, -126.0f);
    x1 = fmaxf(x1, -126.0f);
    const unsigned long long x2 = pack2(x0, x1);
    const unsigned long long t2 = add2(x2, pack2(12582912.0f, 12582912.0f));   // 1.5 * 2^23
    const unsigned long long n2 = add2(t2, pack2(-12582912.0f, -12582912.0f));
    const unsigned long long f2 = fma2(n2, pack2(-1.0f, -1.0f), x2);
    unsigned long long p2 = fma2(pack2(0.05517084f, 0.05517084f), f2, pack2(0.24260908f, 0.24260908f));
    p2 = fma2(p2, f2, pack2(0.69326109f, 0.69326109f));
    p2 = fma2(p2, f2, pack2(0.99992847f, 0.99992847f));
    float t0, t1, q0, q1;
    unpack2(t2, t0, t1);
    unpack2(p2, q0, q1);
    p0 = __uint_as_float(__float_as_uint(q0) + (__float_as_uint(t0) << 23));
    p1 = __uint_as_float(__float_as_uint(q1) + (__float_as_uint(t1) << 23));
}

template <typename T> __device__ __forceinline__ unsigned pack16(float lo, float hi);
template <> __device__ __forceinline__ unsigned pack16<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&t);
}
template <> __device__ __forceinline__ unsigned pack16<__half>(float lo, float hi) {
    __half2 t = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&t);
}

// Shared-memory matrix descriptor (tcgen05): 128-byte swizzle, descriptor version 1.
//   bits [0,14)  start address >> 4      bits [16,30) leading byte offset >> 4
//   bits [32,46) stride byte offset >> 4 bits [46,48) version = 1      bits [61,64) layout = 2 (SWIZZLE_128B)
__device__ __forceinline__ unsigned long long make_desc(unsigned smem_addr, unsigned lbo_bytes, unsigned sbo_bytes) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_addr & 0x3FFFFu) >> 4);
    d |= (unsigned long long)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (unsigned long long)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= 1ULL << 46;
    d |= 2ULL << 61;
    return d;
}

// Instruction descriptor, kind::f16: f32 accumulate, A/B both f16 or both bf16, M = 128, N = n.
//   bits [4,6) D format (1 = f32)  [7,10) A format  [10,13) B format (0 = f16, 1 = bf16)
//   bit 15 A major, bit 16 B major (0 = K-major, 1 = MN-major)  [17,23) N >> 3  [24,29) M >> 4
template <typename T>
__device__ __forceinline__ unsigned make_idesc(bool b_mn_major, int n) {
    const unsigned fmt = sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
    unsigned d = 0;
    d |= 1u << 4;
    d |= fmt << 7;
    d |= fmt << 10;
    d |= (b_mn_major ? 1u : 0u) << 16;
    d |= (unsigned)(n >> 3) << 17;
    d |= (unsigned)(kBlockM >> 4) << 24;
    return d;
}

// Timeline slots: role (0/1 = softmax warpgroup, 2 = MMA issuer) x kv step (< 60) x event (< 8).
// Compiled in with -DFA_TRACE only; the default build carries none of it.
[[maybe_unused]] constexpr int kTraceSteps = 60;
#ifdef FA_TRACE
__device__ __forceinline__ void trace_event(long long* trace, int role, int j, int ev) {
    if (trace != nullptr && j < kTraceSteps) trace[(role * kTraceSteps + j) * 8 + ev] = clock64();
}
#define FA_TRACE_EVENT(role, j, ev) trace_event(trace, role, j, ev)
#else
#define FA_TRACE_EVENT(role, j, ev) ((void)0)
#endif

struct TileInfo {
    int valid;    // this query tile exists
    int head;     // query head
    int row0;     // first query row
    int n_kv;     // K/V tiles it needs
};

// Extents of one sequence. Query row i sits at global position pos_off + i and sees keys
// j < kv_len with j <= pos_off + i (bottom-right aligned for the varlen and kv-cache entry points).
struct SeqExtent {
    int q_len, kv_len, pos_off;
    long long o_row0;     // first row of this sequence in o (rows of o_heads * 128 elements)
    int q_crow, q_cb;     // TMA coordinates (row, batch) of the sequence's first q row
    int kv_crow, kv_cb;   // same for contiguous K/V (unused when paged)
};

__device__ __forceinline__ SeqExtent seq_extent(const PrefillArgs& a, int s) {
    SeqExtent e;
    if (a.mode == MODE_BATCH) {
        e.q_len = a.q_seq_len; e.kv_len = a.kv_seq_len; e.pos_off = a.start_pos;
        e.o_row0 = (long long)s * a.q_seq_len;
        e.q_crow = 0; e.q_cb = s; e.kv_crow = 0; e.kv_cb = s;
    } else if (a.mode == MODE_VARLEN) {
        const int q0 = a.cu_q[s], k0 = a.cu_k[s];
        e.q_len = a.cu_q[s + 1] - q0; e.kv_len = a.cu_k[s + 1] - k0; e.pos_off = e.kv_len - e.q_len;
        e.o_row0 = q0;
        e.q_crow = q0; e.q_cb = 0; e.kv_crow = k0; e.kv_cb = 0;
    } else {
        e.q_len = a.q_seq_len; e.kv_len = a.context_lens[s]; e.pos_off = e.kv_len - e.q_len;
        e.o_row0 = (long long)s * a.q_seq_len;
        e.q_crow = 0; e.q_cb = s; e.kv_crow = 0; e.kv_cb = 0;
    }
    return e;
}

__device__ __forceinline__ TileInfo tile_info(const SeqExtent& a, int pair, int t, int kvh, int group, int num_mb) {
    TileInfo ti;
    // Tile 0 takes the later index of the pair: where the pair is two consecutive row blocks of one head
    // (group 1), that is the longer tile, and tile 0 is the one whose copies are requested first and whose
    // products the issuer serves first in every step, so the tile that decides when the CTA ends is never
    // the one that waits (S = 2048 MHA: 887-892 against 851 TFLOP/s; no difference for GQA pairs, whose
    // two tiles are equally long).
    const int idx = pair * 2 + (1 - t);
    ti.valid = idx < group * num_mb;
    const int mb = ti.valid ? idx / group : 0;
    ti.head = kvh * group + (ti.valid ? idx - mb * group : 0);
    ti.row0 = mb * kBlockM;
    const int last_row = min(ti.row0 + kBlockM, a.q_len) - 1;
    const long long last_key = min((long long)a.kv_len - 1, (long long)a.pos_off + last_row);
    ti.n_kv = (ti.valid && last_key >= 0) ? (int)(last_key / kBlockN) + 1 : 0;   // 0: the tile sees no key at all
    return ti;
}

// One K or V tile (128 keys x D dims, D / 64 halves of 64 columns) of sequence s, tile index j.
//   contiguous: two boxes of 128 rows starting at the sequence's row kv_crow + 128 j;
//   paged     : one box per page and half (block_size rows), the page looked up in the block
//               table; pages past the sequence's last one are requested at block -1, which is out
//               of range for the tensor map and therefore arrives as zeros.
template <int D>
__device__ __forceinline__ void load_kv_tile(const PrefillArgs& a, const SeqExtent& sq, int s, int kvh, unsigned char* dst,
                                             const CUtensorMap* map, unsigned long long* bar, int j) {
    mbar_expect_tx(bar, TileBytes<D>::value);
    if (!a.paged) {
        tma_load_4d(dst, map, bar, 0, kvh, sq.kv_crow + j * kBlockN, sq.kv_cb);
        if (D == 128) tma_load_4d(dst + kHalfBytes, map, bar, 64, kvh, sq.kv_crow + j * kBlockN, sq.kv_cb);
    } else {
        const int bs = a.block_size;
        const int per_tile = kBlockN / bs;
        const int n_pages = (sq.kv_len + bs - 1) / bs;
        for (int i = 0; i < per_tile; ++i) {
            const int pg = j * per_tile + i;
            const int blk = pg < n_pages ? a.block_tables[(long long)s * a.max_blocks + pg] : -1;
            tma_load_4d(dst + i * bs * 128, map, bar, 0, kvh, 0, blk);
            if (D == 128) tma_load_4d(dst + kHalfBytes + i * bs * 128, map, bar, 64, kvh, 0, blk);
        }
    }
}

// A 128-row tile of a packed (varlen) buffer that would reach past the buffer's last row, fetched by
// one warp with plain loads: the reference's varlen signature does not say how many rows the packed
// buffers hold, so their tensor maps carry no row bound, and a bulk copy must never be asked for
// rows that may not exist. Rows past the end are written as zeros (what an out-of-range bulk copy
// delivers). Same shared-memory image as the bulk copies: 64-column halves, 128 B per row, 16-byte
// chunks XOR-swizzled by the row. The barrier's phase is completed by one plain arrival.
template <int D>
__device__ __forceinline__ void edge_tile_copy(unsigned char* dst, const void* base, int heads, int head, long long row_start,
                                               long long total_rows, unsigned long long* bar, int lane, int d_real) {
    constexpr int kChunksPerRow = D / 8;   // 16-byte chunks per row of the tile (columns past d_real are zeros)
    const long long left = total_rows - row_start;
    const int nrows = left < 0 ? 0 : (left > kBlockN ? kBlockN : (int)left);
    const unsigned char* src = static_cast<const unsigned char*>(base);
#pragma unroll 4
    for (int idx = lane; idx < kBlockN * kChunksPerRow; idx += 32) {
        const int r = idx / kChunksPerRow, cc = idx % kChunksPerRow;
        uint4 w = make_uint4(0u, 0u, 0u, 0u);
        if (r < nrows && cc * 8 < d_real) w = *reinterpret_cast<const uint4*>(src + ((row_start + r) * heads + head) * (long long)(d_real * 2) + cc * 16);
        *reinterpret_cast<uint4*>(dst + (cc >> 3) * kHalfBytes + r * 128 + (((cc & 7) ^ (r & 7)) << 4)) = w;
    }
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // generic-proxy writes -> tensor-core reads
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
}

// kMask: the call carries a key-padding mask (a separate instantiation, so that calls without one
// pay nothing for it in the softmax loop)
template <typename T, int D, bool kMask>
__global__ void __launch_bounds__(kThreads, 1)
prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                       const __grid_constant__ CUtensorMap v_map, const __grid_constant__ CUtensorMap o_map, const PrefillArgs a) {
    extern __shared__ unsigned char smem_raw[];
    using Storage = SharedStorage<D>;
    Storage& sm = *reinterpret_cast<Storage*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
#ifdef FA_TRACE
    const long long t_entry = clock64();
    const unsigned long long ns_entry = a.cta_log != nullptr ? global_timer_ns() : 0ULL;
#endif

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int group = a.q_heads / a.kv_heads;
    // blockIdx.x = (batch element, KV head) x `band` neighbouring tile pairs, blockIdx.y = band of pairs,
    // heaviest (latest rows) first. CTAs are dispatched in index order, so the `band` CTAs that walk
    // the same K/V stream start together and meet its tiles in L2 instead of each pulling them from
    // HBM, while the order across bands stays heaviest first.
    // blockIdx.z = group of K/V streams: the grid runs group after group (each heaviest first), so that the
    // K/V of the streams in flight stay within L2 when every tile pair of a stream re-reads its stream's prefix
    const int stream_id = (int)blockIdx.z * (int)(gridDim.x / a.band) + (int)(blockIdx.x / a.band);
    if (stream_id >= a.kv_heads * a.batch) return;   // the last group may be short
    const SeqExtent sq = seq_extent(a, stream_id / a.kv_heads);
    const int num_mb = (sq.q_len + kBlockM - 1) / kBlockM;
    const int kvh = stream_id % a.kv_heads;
    const int b = stream_id / a.kv_heads;
    const int rank_y = launch_rank((int)blockIdx.y, a.spread_w, a.spread_m);   // this row's rank by weight, 0 = heaviest
    const int pair = ((int)gridDim.y - 1 - rank_y) * a.band + (a.band - 1 - (int)(blockIdx.x % a.band));

    const TileInfo t0 = tile_info(sq, pair, 0, kvh, group, num_mb);
    const TileInfo t1 = tile_info(sq, pair, 1, kvh, group, num_mb);
    if (!t0.valid && !t1.valid) return;   // this sequence is shorter than the grid's row range (whole CTA leaves)
    const int n_max = max(t0.n_kv, t1.n_kv);

    // The producer thread initialises the barriers itself and issues the first loads right away (Q,
    // and the K/V tiles that fill the empty ring), before the CTA-wide set-up barrier: the copies
    // then fly while tensor memory is being allocated and the other warps start up.
    const int n_pre = min(kStages, n_max);
    // Packed buffers end at row cu_seqlens[num_seqs]; a tile that reaches past that row is not asked
    // of the copy engine (see edge_tile_copy) but fetched by the producer warp after the set-up.
    const bool packed = a.mode == MODE_VARLEN;
    const long long tot_q = packed ? (long long)a.cu_q[a.batch] : 0;
    const long long tot_k = (packed && !a.paged) ? (long long)a.cu_k[a.batch] : 0;
    auto q_edge = [&](const TileInfo& ti) { return packed && ti.valid && (long long)sq.q_crow + ti.row0 + kBlockM > tot_q; };
    auto kv_edge = [&](int j) { return packed && !a.paged && (long long)sq.kv_crow + (long long)(j + 1) * kBlockN > tot_k; };
    if (warp == kLoadWarp && lane == 0) {
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&q_map) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&k_map) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&v_map) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&o_map) : "memory");
        sm.abort_flag = 0;
        for (int i = 0; i < 2; ++i) {
            mbar_init(&sm.q_full[i], 1);
            mbar_init(&sm.s_full[i], 1);
            mbar_init(&sm.p_lo[i], 128);
            mbar_init(&sm.p_hi[i], 128);
        }
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&sm.k_full[i], 1);
            mbar_init(&sm.k_empty[i], 1);
        }
        for (int i = 0; i < kStagesV; ++i) {
            mbar_init(&sm.v_full[i], 1);
            mbar_init(&sm.v_empty[i], 1);
        }
        mbar_init(&sm.v_tail, 1);
        mbar_init(&sm.drain, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        auto load_q = [&](const TileInfo& ti, int t) {
            if (!ti.valid || q_edge(ti)) return;
            mbar_expect_tx(&sm.q_full[t], TileBytes<D>::value);
            tma_load_4d(sm.q[t], &q_map, &sm.q_full[t], 0, ti.head, sq.q_crow + ti.row0, sq.q_cb);
            if (D == 128) tma_load_4d(sm.q[t] + kHalfBytes, &q_map, &sm.q_full[t], 64, ti.head, sq.q_crow + ti.row0, sq.q_cb);
        };
        auto load_kv = [&](unsigned char* dst, const CUtensorMap* map, unsigned long long* bar, int j) {
            load_kv_tile<D>(a, sq, b, kvh, dst, map, bar, j);
        };
        load_q(t0, 0);
        if (n_pre > 0 && !kv_edge(0) && a.test_skip_k != 1) load_kv(sm.k[0], &k_map, &sm.k_full[0], 0);
        load_q(t1, 1);
        for (int j = 1; j < n_pre; ++j)
            if (!kv_edge(j) && a.test_skip_k != j + 1) load_kv(sm.k[j], &k_map, &sm.k_full[j], j);
        // the V tiles come from a producer thread of their own (warp kLoadWarpV), after the set-up barrier
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;\n" ::"r"(smem_u32(&sm.tmem_base)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = sm.tmem_base;
#ifdef FA_TRACE
    // only the heaviest CTA of the first (batch, KV head) records its timeline, one thread per role
    long long* const trace = (a.trace != nullptr && blockIdx.x == 0 && blockIdx.y == (unsigned)a.trace_y && lane == 0 && (warp == kMmaWarp || (warp & 3) == 0)) ? a.trace : nullptr;
    // slot kTraceSteps - 1 of each role holds the CTA's life cycle instead of a kv step
    if (trace != nullptr && warp == kMmaWarp) {
        trace[(2 * kTraceSteps + kTraceSteps - 1) * 8 + 0] = t_entry;
        FA_TRACE_EVENT(2, kTraceSteps - 1, 1);   // set-up (barriers, tensor memory) done
    }
#endif

    // Register budget: the kernel is compiled for 168 registers per thread (384 threads); the
    // producer/issuer warpgroup hands most of its share to the two softmax warpgroups, which
    // keep a whole 128-column score row per thread in registers.
    if (warp >= 8) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 88;\n");
    if (warp == kLoadWarp || warp == kLoadWarpV) {
        // ------------------------------ TMA producers ------------------------------
        // One thread streams the K tiles (and loaded Q before), one the V tiles: with a paged cache a
        // tile is one copy per page and 64-column half plus a block-table read per page, and a single
        // thread issuing both rings cannot keep up with the tensor pipe at small page sizes.
        // The warps run their loops whole; lane 0 issues the bulk copies, and all lanes share the
        // plain-load copy of a tile at the very end of a packed buffer.
        {
            const bool is_v = warp == kLoadWarpV;
            unsigned char (*ring)[TileBytes<D>::value] = is_v ? sm.v : sm.k;
            unsigned long long* full = is_v ? sm.v_full : sm.k_full;
            unsigned long long* empty = is_v ? sm.v_empty : sm.k_empty;
            const CUtensorMap* map = is_v ? &v_map : &k_map;
            const void* kv_base = is_v ? a.v : a.k;
            const int n_stages = is_v ? kStagesV : kStages;
            bool alive = true;
            if (!is_v) {   // what the set-up left out: Q tiles and first K tiles at the end of the packed buffers
                if (q_edge(t0)) edge_tile_copy<D>(sm.q[0], a.q, a.q_heads, t0.head, (long long)sq.q_crow + t0.row0, tot_q, &sm.q_full[0], lane, a.d_real);
                if (q_edge(t1)) edge_tile_copy<D>(sm.q[1], a.q, a.q_heads, t1.head, (long long)sq.q_crow + t1.row0, tot_q, &sm.q_full[1], lane, a.d_real);
                for (int j = 0; j < n_pre; ++j)
                    if (kv_edge(j)) edge_tile_copy<D>(sm.k[j], a.k, a.kv_heads, kvh, (long long)sq.kv_crow + (long long)j * kBlockN, tot_k, &sm.k_full[j], lane, a.d_real);
            }
            // The sequence's last V tile, when the sequence does not end on a tile boundary, holds rows
            // that are not this sequence's: the unwritten rest of its last page, or the next sequence
            // of a packed buffer. P is exactly zero there, but 0 x NaN (an uninitialised pool, a page
            // recycled from other use) would still poison the whole output row, so those rows are
            // cleared in shared memory before the tile is handed to the MMA issuer: its copy completes
            // on a barrier of its own, the producer warp zeroes the rows and then completes the
            // ring's barrier with a plain arrival. (Garbage in K is harmless: the score mask is a select.)
            const bool tail_fix = is_v && (a.paged || packed) && (sq.kv_len % kBlockN) != 0;
            const int tail_j = sq.kv_len > 0 ? (sq.kv_len - 1) / kBlockN : -1;
            bool tail_pending = false;   // the tail tile's copy was issued and v_tail not yet seen complete
            int issued = is_v ? 0 : n_pre;   // K tiles 0 .. n_pre-1 were issued during set-up
            for (int j = issued; j < n_max && alive; ++j) {
                const int s = j % n_stages;
                if (j >= n_stages) {
                    alive = __all_sync(0xffffffffu, mbar_wait(sm, &empty[s], ((unsigned)(j / n_stages) & 1u) ^ 1u, a, is_v ? 2 : 1));
                    if (!alive) break;
                }
                const bool fix = tail_fix && j == tail_j;
                unsigned long long* const bar = fix ? &sm.v_tail : &full[s];
                if (!is_v && a.test_skip_k == j + 1) {
                    // test hook: this tile is never requested, the issuer's wait for it runs out
                } else if (kv_edge(j)) {
                    edge_tile_copy<D>(ring[s], kv_base, a.kv_heads, kvh, (long long)sq.kv_crow + (long long)j * kBlockN, tot_k, bar, lane, a.d_real);
                } else if (lane == 0) {
                    load_kv_tile<D>(a, sq, b, kvh, ring[s], map, bar, j);
                }
                issued = j + 1;
                if (fix) {
                    tail_pending = true;
                    alive = __all_sync(0xffffffffu, mbar_wait(sm, &sm.v_tail, 0u, a, 4));
                    if (!alive) break;
                    tail_pending = false;
                    const int first = sq.kv_len - j * kBlockN;   // first row of the tile that is not this sequence's
                    constexpr int kChunksPerHalfRow = 8;        // 128 B per row and 64-column half
                    const int n_chunks = (kBlockN - first) * kChunksPerHalfRow;
                    for (int h = 0; h < D / 64; ++h)
                        for (int idx = lane; idx < n_chunks; idx += 32)
                            *reinterpret_cast<uint4*>(ring[s] + h * kHalfBytes + first * 128 + idx * 16) = make_uint4(0u, 0u, 0u, 0u);
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // generic-proxy writes -> tensor-core reads
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&full[s]);
                }
            }
            // Make sure none of this warp's copies is still in flight when the CTA exits: wait
            // (bounded) for the last fill of every stage (and of the Q tiles). These waits ignore the
            // abort flag: they only depend on the copy engine.
            if (lane == 0) {
                if (!is_v) {
                    if (t0.valid) mbar_wait(sm, &sm.q_full[0], 0, a, 3);
                    if (t1.valid) mbar_wait(sm, &sm.q_full[1], 0, a, 3);
                }
                const unsigned long long t_begin = global_timer_ns();
                for (int s = 0; s < n_stages; ++s) {
                    if (issued <= s) continue;   // never filled
                    const int last = issued - 1 - (issued - 1 - s) % n_stages;   // last issued tile of this stage
                    if (!is_v && a.test_skip_k == last + 1) continue;          // test hook: never requested
                    if (tail_fix && last == tail_j) {
                        // that tile's copy completes on v_tail; the ring's barrier got (or, after an abort, never gets) a plain arrival
                        while (tail_pending && !mbar_try_wait(&sm.v_tail, 0u) && global_timer_ns() - t_begin < 100000000ULL) {}
                        continue;
                    }
                    while (!mbar_try_wait(&full[s], (unsigned)(last / n_stages) & 1u) && global_timer_ns() - t_begin < 100000000ULL) {}
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ------------------------------ MMA issuer ------------------------------
        {   // the whole warp runs this block converged (see tc_mma_ss_imm)
            const unsigned idesc_qk = make_idesc<T>(false, kBlockN);
            const unsigned idesc_pv = make_idesc<T>(true, D);   // N = head size
            const TileInfo ts[2] = {t0, t1};
            bool alive = true;
            // Descriptors are built once; inside the loops an MMA costs one 64-bit add per operand. A
            // single thread then issues a 128x128x16 product every ~64 clocks, the tensor pipe's own
            // rate — rebuilding the descriptors per product held it at ~90.
            const unsigned long long dq[2] = {make_desc(smem_u32(sm.q[0]), 16, 1024), make_desc(smem_u32(sm.q[1]), 16, 1024)};
            const unsigned long long dk[2] = {make_desc(smem_u32(sm.k[0]), 16, 1024), make_desc(smem_u32(sm.k[1]), 16, 1024)};
            const unsigned long long dv[3] = {make_desc(smem_u32(sm.v[0]), kHalfBytes, 1024), make_desc(smem_u32(sm.v[1]), kHalfBytes, 1024),
                                              make_desc(smem_u32(sm.v[kStagesV - 1]), kHalfBytes, 1024)};
            static_assert(kStages == 2 && (kStagesV == 3 || kStagesV == 2), "descriptor tables hold two K stages and up to three V stages");
            auto issue_s = [&](int t, int stage) {
                // S_t = Q_t K^T : D / 16 K-steps over d; both operands K-major, 128 B swizzle
                const unsigned long long qd = t ? dq[1] : dq[0];
                const unsigned long long kd = stage ? dk[1] : dk[0];
                const unsigned d_tmem = tmem + t * 128;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const unsigned long long inc = (unsigned long long)(((kk >> 2) * kHalfBytes + (kk & 3) * 32) >> 4);
                    if (kk == 0) tc_mma_ss_imm<false>(d_tmem, qd + inc, kd + inc, idesc_qk);
                    else tc_mma_ss_imm<true>(d_tmem, qd + inc, kd + inc, idesc_qk);
                }
            };
            auto issue_pv = [&](int t, int stage, bool accumulate, int half) {
                // O_t += P_t V : 8 K-steps of 16 keys; A = P from tensor memory (packed 16-bit, 8 columns
                // per step), B = V MN-major: 64-column halves 16 KiB apart, 8-key groups 1 KiB apart
                const unsigned long long vd = stage == 0 ? dv[0] : (stage == 1 ? dv[1] : dv[2]);
                const unsigned d_tmem = tmem + 256 + t * 128;
                const unsigned p_tmem = tmem + t * 128;
#pragma unroll
                for (int kk = half * 4; kk < half * 4 + 4; ++kk) {
                    const unsigned long long inc = (unsigned long long)((kk * 2048) >> 4);
                    if (kk == 0 && !accumulate) tc_mma_ts_imm<false>(d_tmem, p_tmem + kk * 8, vd + inc, idesc_pv);
                    else tc_mma_ts_imm<true>(d_tmem, p_tmem + kk * 8, vd + inc, idesc_pv);
                }
            };
            // The copies were requested in the order Q0, K0, Q1: the first S of tile 0 is issued as soon as
            // its two operands are there, without waiting for the other tile's Q.
            if (ts[0].valid) alive = (mbar_wait(sm, &sm.q_full[0], 0, a, 10));
            if (alive && n_max > 0) alive = (mbar_wait(sm, &sm.k_full[0], 0, a, 11));
            if (alive && ts[0].n_kv > 0) {
                tc_fence_after();
                issue_s(0, 0);
                tc_commit(&sm.s_full[0]);
            }
            if (alive && ts[1].valid) alive = (mbar_wait(sm, &sm.q_full[1], 0, a, 10));
            FA_TRACE_EVENT(2, kTraceSteps - 1, 2);       // Q and the first K tile have landed
            if (alive && n_max > 0) {
                tc_fence_after();
                if (ts[1].n_kv > 0) {
                    issue_s(1, 0);
                    tc_commit(&sm.s_full[1]);
                }
                tc_commit(&sm.k_empty[0]);
            }
            for (int j = 0; j < n_max && alive; ++j) {
                const int s = j % kStagesV;                              // V stage of this step
                const unsigned ph = (unsigned)(j / kStagesV) & 1u;
                const int s1 = (j + 1) % kStages;                        // K stage of the next step
                const unsigned ph1 = (unsigned)((j + 1) / kStages) & 1u;
                alive = (mbar_wait(sm, &sm.v_full[s], ph, a, 13));
                if (!alive) break;
                FA_TRACE_EVENT(2, j, 4);
                bool k_seen = j + 1 >= n_max;   // K(j+1) is first needed for S(j+1): looked at while P's second half is awaited
                for (int t = 0; t < 2; ++t) {
                    if (j >= ts[t].n_kv) continue;
                    // the first 64 keys of P_t arrive while the softmax still works on the other 64:
                    // their half of P.V leaves the critical path
                    alive = (mbar_wait(sm, &sm.p_lo[t], (unsigned)j & 1u, a, 14 + t));
                    if (!alive) break;
                    FA_TRACE_EVENT(2, j, t * 2);
                    tc_fence_after();
                    issue_pv(t, s, j > 0, 0);
                    if (!k_seen) {
                        alive = (mbar_wait(sm, &sm.k_full[s1], ph1, a, 12));
                        if (!alive) break;
                        k_seen = true;
                    }
                    alive = (mbar_wait(sm, &sm.p_hi[t], (unsigned)j & 1u, a, 16 + t));
                    if (!alive) break;
                    FA_TRACE_EVENT(2, j, 5 + t);
                    tc_fence_after();
                    issue_pv(t, s, true, 1);
                    if (j + 1 < ts[t].n_kv) issue_s(t, s1);
                    tc_commit(&sm.s_full[t]);   // S_t(j+1) ready, or after the last PV: O_t final
                    FA_TRACE_EVENT(2, j, t * 2 + 1);
                }
                if (!alive) break;
                tc_commit(&sm.v_empty[s]);
                if (j + 1 < n_max) tc_commit(&sm.k_empty[s1]);
            }
            if (!alive) {
                // error path: tensor memory is freed at the end of the kernel, so let every product issued
                // so far finish first (bounded; depends on the tensor pipe alone)
                tc_commit(&sm.drain);
                const unsigned long long t_begin = global_timer_ns();
                while (!mbar_try_wait(&sm.drain, 0u) && global_timer_ns() - t_begin < 100000000ULL) {}
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 208;\n");
        // ------------------------------ softmax warpgroups ------------------------------
        const int t = warp >> 2;
        const TileInfo ti = t == 0 ? t0 : t1;
        const int r = (warp & 3) * 32 + lane;                  // row within the tile == TMEM lane
        const unsigned lane_base = (unsigned)((warp & 3) * 32) << 16;
        const unsigned s_addr = tmem + lane_base + t * 128;
        const unsigned o_addr = tmem + lane_base + 256 + t * 128;
        const int row = ti.row0 + r;
        const long long pos = (long long)sq.pos_off + row;      // global position of this query row
        float m = -INFINITY;   // reference max, log2 domain (may lag the true max by <= 2^8)
        float l = 0.0f;
        bool alive = true;

        for (int j = 0; j < ti.n_kv && alive; ++j) {
            alive = __all_sync(0xffffffffu, mbar_wait(sm, &sm.s_full[t], (unsigned)j & 1u, a, 20 + t));
            if (!alive) break;
            FA_TRACE_EVENT(t, j, 0);
            tc_fence_after();
            const int key0 = j * kBlockN;
            // mask only where the causal diagonal or the end of K/V cuts through this tile
            const long long limit_ll = min(pos, (long long)sq.kv_len - 1) - key0;
            const bool need_mask = (long long)(key0 + kBlockN - 1) > min((long long)sq.pos_off + ti.row0, (long long)sq.kv_len - 1);
            const int limit = need_mask ? (int)max(-1LL, min(limit_ll, (long long)kBlockN)) : kBlockN;

            // An aligned diagonal tile (row i of the tile sees exactly keys 0..i of it) has a fixed shape
            // per warp: warp w sees chunks 0..w-1 of 32 columns in full, chunk w up to its own lane,
            // nothing after it. It is handled with the chunks rotated so that the diagonal one sits in
            // register slot 0 (the tensor-memory addresses are run-time values, the slots are not):
            // 32 compares instead of 128, FMA-pipe exponentials in the full chunks, no work in the
            // unseen ones. Any other masked tile (cut by the end of K/V, unaligned start) takes the
            // general code below.
            // Key-padding mask (batched entry point): the tile's 128 validity bytes become four ballots;
            // a tile whose keys are all valid — the usual case, padding sits at one end — runs as if
            // there were no mask, any other takes the general step with the bits applied first.
            unsigned kb0 = 0xffffffffu, kb1 = 0xffffffffu, kb2 = 0xffffffffu, kb3 = 0xffffffffu;
            bool pad = false;
            if (kMask) {
                const unsigned char* mrow = a.mask + (long long)b * a.kv_seq_len;
                const int kk = key0 + lane;
                kb0 = __ballot_sync(0xffffffffu, kk < sq.kv_len && mrow[kk < sq.kv_len ? kk : 0] != 0);
                kb1 = __ballot_sync(0xffffffffu, kk + 32 < sq.kv_len && mrow[kk + 32 < sq.kv_len ? kk + 32 : 0] != 0);
                kb2 = __ballot_sync(0xffffffffu, kk + 64 < sq.kv_len && mrow[kk + 64 < sq.kv_len ? kk + 64 : 0] != 0);
                kb3 = __ballot_sync(0xffffffffu, kk + 96 < sq.kv_len && mrow[kk + 96 < sq.kv_len ? kk + 96 : 0] != 0);
                // keys past kv_len are cut by `limit` already; only padding among the real keys counts here
                const int real = min(kBlockN, sq.kv_len - key0);
                const unsigned w0 = real >= 32 ? 0xffffffffu : ((1u << max(real, 0)) - 1u);
                const unsigned w1 = real >= 64 ? 0xffffffffu : (real <= 32 ? 0u : ((1u << (real - 32)) - 1u));
                const unsigned w2 = real >= 96 ? 0xffffffffu : (real <= 64 ? 0u : ((1u << (real - 64)) - 1u));
                const unsigned w3 = real >= 128 ? 0xffffffffu : (real <= 96 ? 0u : ((1u << (real - 96)) - 1u));
                pad = ((kb0 & w0) != w0) || ((kb1 & w1) != w1) || ((kb2 & w2) != w2) || ((kb3 & w3) != w3);
            }
            const bool diag_tile = !(kMask && pad) && need_mask && (long long)sq.pos_off + ti.row0 == (long long)key0 &&
                                   (long long)sq.pos_off + ti.row0 + kBlockM - 1 <= (long long)sq.kv_len - 1;
            if (diag_tile) {
                const int w = warp & 3;
                float dv[4][32];   // slot k holds chunk (w + k) & 3
#pragma unroll
                for (int k = 0; k < 4; ++k) tc_ld32(s_addr + ((w + k) & 3) * 32, dv[k]);
                tc_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (i > lane) dv[0][i] = -INFINITY;
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int i = 0; i < 32; i += 2) mx4[(i >> 1) & 3] = max3(mx4[(i >> 1) & 3], dv[0][i], dv[0][i + 1]);
#pragma unroll
                for (int k = 1; k < 4; ++k) {
                    if (((w + k) & 3) < w) {   // a chunk before the diagonal one: seen in full
#pragma unroll
                        for (int i = 0; i < 32; i += 2) mx4[(i >> 1) & 3] = max3(mx4[(i >> 1) & 3], dv[k][i], dv[k][i + 1]);
                    }
                }
                float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * a.scale_log2;
                FA_TRACE_EVENT(t, j, 1);
                float alpha = 1.0f;
                bool changed = false;
                if (mx > m + kRescaleThreshold) {
                    alpha = ex2(m - mx);
                    m = mx;
                    changed = true;
                }
                if (j > 0 && __any_sync(0xffffffffu, changed)) {
#pragma unroll 1
                    for (int c = 0; c < D / 32; ++c) {
                        float ov[32];
                        tc_ld32(o_addr + c * 32, ov);
                        tc_wait_ld();
                        unsigned ou[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) ou[i] = __float_as_uint(ov[i] * alpha);
                        tc_st32(o_addr + c * 32, ou);
                    }
                }
                const float m_use = (m == -INFINITY) ? 0.0f : m;
                const unsigned long long scale2 = pack2(a.scale_log2, a.scale_log2);
                const unsigned long long neg_m2 = pack2(-m_use, -m_use);
                unsigned long long sum2 = pack2(0.0f, 0.0f);
                {   // the diagonal chunk: every exponential on the special-function unit (-inf gives an exact zero)
                    unsigned pu[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        float x0, x1;
                        unpack2(fma2(pack2(dv[0][2 * i], dv[0][2 * i + 1]), scale2, neg_m2), x0, x1);
                        const float p0 = ex2(x0), p1 = ex2(x1);
                        sum2 = add2(sum2, pack2(p0, p1));
                        pu[i] = pack16<T>(p0, p1);
                    }
                    tc_st16(s_addr + w * 16, pu);   // P of chunk c lives in 16 packed columns at c * 16
                }
#pragma unroll
                for (int k = 1; k < 4; ++k) {
                    const int c = (w + k) & 3;
                    unsigned pu[16];
                    if (c < w) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            float x0, x1, p0, p1;
                            unpack2(fma2(pack2(dv[k][2 * i], dv[k][2 * i + 1]), scale2, neg_m2), x0, x1);
                            if (fma_pipe_exp(i)) {
                                ex2_fma2(x0, x1, p0, p1);
                            } else {
                                p0 = ex2(x0);
                                p1 = ex2(x1);
                            }
                            sum2 = add2(sum2, pack2(p0, p1));
                            pu[i] = pack16<T>(p0, p1);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; ++i) pu[i] = 0u;
                    }
                    tc_st16(s_addr + c * 16, pu);
                }
                tc_wait_st();
                tc_fence_before();
                mbar_arrive(&sm.p_lo[t]);
                FA_TRACE_EVENT(t, j, 2);
                mbar_arrive(&sm.p_hi[t]);
                float sum_lo, sum_hi;
                unpack2(sum2, sum_lo, sum_hi);
                l = l * alpha + (sum_lo + sum_hi);
            } else {
                float sv[4][32];
#pragma unroll
                for (int c = 0; c < 4; ++c) tc_ld32(s_addr + c * 32, sv[c]);
                tc_wait_ld();
                if (kMask && pad) {   // padded keys first: the bits are dead after this
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if (!((kb0 >> i) & 1u)) sv[0][i] = -INFINITY;
                        if (!((kb1 >> i) & 1u)) sv[1][i] = -INFINITY;
                        if (!((kb2 >> i) & 1u)) sv[2][i] = -INFINITY;
                        if (!((kb3 >> i) & 1u)) sv[3][i] = -INFINITY;
                    }
                }
                if (need_mask) {
#pragma unroll
                    for (int c = 0; c < 4; ++c)
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (c * 32 + i > limit) sv[c][i] = -INFINITY;
                }
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int i = 0; i < 32; i += 2) mx4[(i >> 1) & 3] = max3(mx4[(i >> 1) & 3], sv[c][i], sv[c][i + 1]);
                float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
                mx *= a.scale_log2;   // scale > 0 is guaranteed by the dispatcher
                FA_TRACE_EVENT(t, j, 1);

                float alpha = 1.0f;
                bool changed = false;
                if (mx > m + kRescaleThreshold) {   // also true for the first finite max (m == -inf)
                    alpha = ex2(m - mx);            // 0 when m == -inf
                    m = mx;
                    changed = true;
                }
                if (j > 0 && __any_sync(0xffffffffu, changed)) {
                    // rescale this warp's 32 rows of O in tensor memory (rows that did not move use 1.0)
#pragma unroll 1
                    for (int c = 0; c < D / 32; ++c) {
                        float ov[32];
                        tc_ld32(o_addr + c * 32, ov);
                        tc_wait_ld();
                        unsigned ou[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) ou[i] = __float_as_uint(ov[i] * alpha);
                        tc_st32(o_addr + c * 32, ou);
                    }
                }
                const float m_use = (m == -INFINITY) ? 0.0f : m;
                // exp2(s * scale - m) two columns at a time: packed FMA for the argument and the row sum;
                // one pair in four takes its exponential on the FMA pipe (unmasked tiles only), which
                // relieves the special-function unit the two warpgroups compete for.
                const unsigned long long scale2 = pack2(a.scale_log2, a.scale_log2);
                const unsigned long long neg_m2 = pack2(-m_use, -m_use);
                unsigned long long sum2 = pack2(0.0f, 0.0f);
                // two straight-line copies (masked tiles keep every exponential on the special-function
                // unit, where -inf gives an exact zero) rather than a branch inside the unrolled loop
                auto exp_phase = [&](auto fma_pipe_share) {
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        unsigned pu[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int cc = c * 2 + (i >> 4);
                            const int ii = (i & 15) * 2;
                            float x0, x1, p0, p1;
                            unpack2(fma2(pack2(sv[cc][ii], sv[cc][ii + 1]), scale2, neg_m2), x0, x1);
                            if (decltype(fma_pipe_share)::value && fma_pipe_exp(i)) {
                                ex2_fma2(x0, x1, p0, p1);
                            } else {
                                p0 = ex2(x0);
                                p1 = ex2(x1);
                            }
                            sum2 = add2(sum2, pack2(p0, p1));
                            pu[i] = pack16<T>(p0, p1);
                        }
                        tc_st32(s_addr + c * 32, pu);
                        tc_wait_st();
                        tc_fence_before();
                        mbar_arrive(c == 0 ? &sm.p_lo[t] : &sm.p_hi[t]);
                        if (c == 0) FA_TRACE_EVENT(t, j, 2);
                    }
                };
                if (need_mask || (kMask && pad)) exp_phase(std::false_type{});
                else exp_phase(std::true_type{});
                float sum_lo, sum_hi;
                unpack2(sum2, sum_lo, sum_hi);
                const float sum = sum_lo + sum_hi;
                l = l * alpha + sum;
            }
            FA_TRACE_EVENT(t, j, 3);
        }

        // epilogue: O_t is final once the commit after the last P.V has arrived
        if (alive && ti.n_kv > 0)
            alive = __all_sync(0xffffffffu, mbar_wait(sm, &sm.s_full[t], (unsigned)ti.n_kv & 1u, a, 30 + t));
        if (alive && ti.valid) {
            tc_fence_after();
            const bool row_ok = row < sq.q_len;
            // with a padding mask a query row at a padded (or out-of-range) position outputs zeros (flash_attn_func.cu:77-84)
            bool q_ok = true;
            if (kMask) q_ok = row_ok && pos >= 0 && pos < (long long)sq.kv_len && a.mask[(long long)b * a.kv_seq_len + pos] != 0;
            const float inv = (l > 0.0f && q_ok) ? 1.0f / l : 0.0f;
            // a bulk store writes every row of its box that lies inside the tensor: in a packed buffer the
            // rows after this sequence belong to the next one, so a tile that overhangs the end of its
            // sequence takes the row-guarded path
#ifdef FA_TRACE
            const bool staged_only = a.staged_store != 0;
#else
            constexpr bool staged_only = false;
#endif
            const bool bulk_ok = a.n_out == 1 && !a.multicast && !staged_only && (a.mode != MODE_VARLEN || ti.row0 + kBlockM <= sq.q_len);
            if (bulk_ok) {
                // Single output: the rows go out as bulk tensor stores. Each warp lays its 32 rows down in
                // the Q tile's shared memory (every MMA that read Q_t has finished) in the 128-byte-swizzled
                // box layout and one lane issues one store of 32 rows x 64 columns per half. Plain 16-byte stores
                // of 32 different rows per instruction would fill the SM's memory pipeline for thousands
                // of clocks and hold up the barrier traffic of the other tile's last steps. Rows past the
                // end of the sequence are outside the tensor map and are not written.
                float ov[D / 32][32];
#pragma unroll
                for (int c = 0; c < D / 32; ++c) tc_ld32(o_addr + c * 32, ov[c]);
                tc_wait_ld();
                if (ti.n_kv == 0) {   // the tile saw no key: tensor memory holds nothing of ours, the rows are zeros
#pragma unroll
                    for (int c = 0; c < D / 32; ++c)
#pragma unroll
                        for (int i = 0; i < 32; ++i) ov[c][i] = 0.0f;
                }
                unsigned char* stage = sm.q[t];
#pragma unroll
                for (int c = 0; c < D / 32; ++c) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint4 w;
                        w.x = pack16<T>(ov[c][8 * i] * inv, ov[c][8 * i + 1] * inv);
                        w.y = pack16<T>(ov[c][8 * i + 2] * inv, ov[c][8 * i + 3] * inv);
                        w.z = pack16<T>(ov[c][8 * i + 4] * inv, ov[c][8 * i + 5] * inv);
                        w.w = pack16<T>(ov[c][8 * i + 6] * inv, ov[c][8 * i + 7] * inv);
                        const int ch = (c & 1) * 4 + i;   // 16-byte chunk within the 64-column half c >> 1
                        *reinterpret_cast<uint4*>(stage + (c >> 1) * kHalfBytes + r * 128 + ((ch ^ (r & 7)) << 4)) = w;
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // generic-proxy writes -> bulk copy reads
                __syncwarp();
                if (lane == 0) {
                    const int warp_row0 = (warp & 3) * 32;
                    tma_store_4d(&o_map, stage + warp_row0 * 128, 0, a.o_head0 + ti.head, sq.q_crow + ti.row0 + warp_row0, sq.q_cb);
                    if (D == 128)
                        tma_store_4d(&o_map, stage + kHalfBytes + warp_row0 * 128, 64, a.o_head0 + ti.head, sq.q_crow + ti.row0 + warp_row0, sq.q_cb);
                    asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
                    asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");   // shared memory stays valid until read
                }
            } else {
                // Stage this warp's 32 rows (2 D bytes each) in the Q tile's shared memory — every MMA that read
                // Q_t has finished — so that the global stores are whole rows: D / 8 lanes x 16 B contiguous,
                // 256 / D rows per instruction. That matters most for the peer copies, which cross NVLink.
                constexpr int kRowBytes = D * 2;
                constexpr int kChunks = D / 8;          // 16-byte chunks per row
                unsigned char* stage = sm.q[t];
    #pragma unroll 1
                for (int c = 0; c < D / 32; ++c) {
                    float ov[32];
                    tc_ld32(o_addr + c * 32, ov);
                    tc_wait_ld();
                    if (ti.n_kv == 0) {   // the tile saw no key: tensor memory holds nothing of ours, the rows are zeros
                    #pragma unroll
                        for (int i = 0; i < 32; ++i) ov[i] = 0.0f;
                    }
    #pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint4 w;
                        w.x = pack16<T>(ov[8 * i] * inv, ov[8 * i + 1] * inv);
                        w.y = pack16<T>(ov[8 * i + 2] * inv, ov[8 * i + 3] * inv);
                        w.z = pack16<T>(ov[8 * i + 4] * inv, ov[8 * i + 5] * inv);
                        w.w = pack16<T>(ov[8 * i + 6] * inv, ov[8 * i + 7] * inv);
                        const int ch = c * 4 + i;   // 16-byte chunk of the row, XOR-swizzled against bank conflicts
                        *reinterpret_cast<uint4*>(stage + r * kRowBytes + ((ch ^ (r & (kChunks - 1))) << 4)) = w;
                    }
                }
                __syncwarp();
                {
                    const int ch = lane & (kChunks - 1);
                    const int sub = lane / kChunks;
                    constexpr int kRowsPerStep = 32 / kChunks;
                    const int warp_row0 = (warp & 3) * 32;
    #pragma unroll 4
                    for (int it = 0; it < 32 / kRowsPerStep; ++it) {
                        const int rr = warp_row0 + it * kRowsPerStep + sub;
                        const int grow = ti.row0 + rr;
                        if (grow < sq.q_len && ch * 8 < a.d_real) {
                            const uint4 w = *reinterpret_cast<const uint4*>(stage + rr * kRowBytes + ((ch ^ (rr & (kChunks - 1))) << 4));
                            const long long o_off = ((sq.o_row0 + grow) * a.o_heads + a.o_head0 + ti.head) * a.d_real + ch * 8;
                            // every GPU of a group starts its walk at a different buffer (peer0 = its own
                            // index + 1), so that at no time all of them store to the same GPU
                            if (a.multicast) {
                                // one store into the multicast address: the switch writes it into every GPU's tensor
                                multimem_st16(static_cast<T*>(a.o[0]) + o_off, w);
                            } else {
                                int pe = a.peer0;
                                for (int n = 0; n < a.n_out; ++n) {
                                    *reinterpret_cast<uint4*>(static_cast<T*>(a.o[pe]) + o_off) = w;
                                    pe = pe + 1 == a.n_out ? 0 : pe + 1;
                                }
                            }
                        }
                    }
                }
            }
            if (row_ok && (a.lse != nullptr || a.n_lse > 0)) {
                const float lse_val = (l > 0.0f && q_ok) ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
                if (a.lse != nullptr) a.lse[((long long)b * a.q_heads + ti.head) * a.q_seq_len + row] = lse_val;
                // head-sharded call: the same value into the (batch, o_heads, q_seq_len) LSE of every GPU of the group
                const long long g_off = ((long long)b * a.o_heads + a.o_head0 + ti.head) * a.q_seq_len + row;
                for (int n = 0; n < a.n_lse; ++n) a.lse_peers[n][g_off] = lse_val;
            }
            FA_TRACE_EVENT(t, kTraceSteps - 1, 0);       // epilogue stores issued
        }
    }

    tc_fence_before();
    __syncthreads();
    FA_TRACE_EVENT(2, kTraceSteps - 1, 3);               // every role done
    if (warp == kMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;\n" ::"r"(tmem) : "memory");
    }
#ifdef FA_TRACE
    if (a.cta_log != nullptr && threadIdx.x == 0) {
        const int idx = blockIdx.y * gridDim.x + blockIdx.x;
        if (idx < kCtaLogEntries) {
            unsigned smid;
            asm volatile("mov.u32 %0, %%smid;\n" : "=r"(smid));
            a.cta_log[idx * 3 + 0] = (long long)ns_entry;
            a.cta_log[idx * 3 + 1] = (long long)global_timer_ns();
            a.cta_log[idx * 3 + 2] = (long long)smid;
        }
    }
#endif
}

// ---- host side ---------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode_fn() {
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, []() {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeFn>(p);
        } else {
            cudaGetLastError();
        }
    });
    return fn;
}

// (batch, seq, heads, 128) 16-bit tensor viewed as 4-D {d, head, seq, batch}; box = 64 x 1 x 128 x 1
// seq <= 0: a packed buffer whose row count the caller did not give (batch is 1 then). The row extent is
// set beyond any buffer and the kernel never asks for a box that reaches past the real last row.
bool encode_map(CUtensorMap* map, const void* base, int dtype, int d, int batch, int seq, int heads, int box_rows = kBlockM) {
    EncodeFn fn = get_encode_fn();
    if (fn == nullptr) return false;
    const bool unbounded = seq <= 0;
    const cuuint64_t rows = unbounded ? (cuuint64_t)0x7fffffff : (cuuint64_t)seq;
    const cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)heads, rows, (cuuint64_t)batch};
    // the stride of the batch axis is never used when batch is 1; it only has to be a legal value
    const cuuint64_t strides[3] = {(cuuint64_t)d * 2, (cuuint64_t)heads * d * 2,
                                   unbounded ? (cuuint64_t)heads * d * 2 * 128 : (cuuint64_t)seq * heads * d * 2};
    const cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUtensorMapDataType dt = dtype == DT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const CUresult rc = fn(map, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS;
}

// Paged cache (num_blocks, block_size, heads, 128) viewed as 4-D {d, head, slot in block, block};
// box = 64 x 1 x block_size x 1: one page of one head and one 64-column half per copy. The C ABI
// does not say how many blocks the pool has, so the block extent is set far beyond any pool; only
// block ids read from the table are ever requested (and -1 for "no page": out of range, zeros).
bool encode_paged_map(CUtensorMap* map, const void* base, int dtype, int d, int block_size, int heads) {
    EncodeFn fn = get_encode_fn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)heads, (cuuint64_t)block_size, (cuuint64_t)1 << 30};
    const cuuint64_t strides[3] = {(cuuint64_t)d * 2, (cuuint64_t)heads * d * 2, (cuuint64_t)block_size * heads * d * 2};
    if (strides[2] >= ((cuuint64_t)1 << 40)) return false;
    const cuuint32_t box[4] = {64, 1, (cuuint32_t)block_size, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUtensorMapDataType dt = dtype == DT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const CUresult rc = fn(map, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS;
}

// Status words, one per device, in mapped pinned host memory: a kernel whose bounded wait ran out
// stores the wait's code there, and the host reads it at the next entry-point call without
// touching the device. One portable allocation for all devices, a cache line per device.
constexpr int kMaxDevices = 64;
constexpr int kStatusStride = 32;   // ints (128 bytes) between two devices' words
std::mutex g_status_mutex;
int* g_status_host = nullptr;

int* status_word() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(g_status_mutex);
    if (g_status_host == nullptr) {
        void* p = nullptr;
        if (cudaHostAlloc(&p, sizeof(int) * kStatusStride * kMaxDevices, cudaHostAllocPortable | cudaHostAllocMapped) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        std::memset(p, 0, sizeof(int) * kStatusStride * kMaxDevices);
        g_status_host = static_cast<int*>(p);
    }
    return g_status_host + dev * kStatusStride;
}

#ifdef FA_TRACE
// Per-device debug area in device memory: (from byte 256) the optional timeline, from byte 16384 the CTA log.
constexpr size_t kDebugBytes = 16384 + kCtaLogEntries * 24;
unsigned char* g_debug_area[kMaxDevices] = {nullptr};

unsigned char* debug_area() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(g_status_mutex);
    if (g_debug_area[dev] == nullptr) {
        void* p = nullptr;
        if (cudaMalloc(&p, kDebugBytes) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        cudaMemset(p, 0, kDebugBytes);
        g_debug_area[dev] = static_cast<unsigned char*>(p);
    }
    return g_debug_area[dev];
}
#endif

template <typename T, int D, bool kMask>
int launch_typed(const AttnParams& p, cudaStream_t stream) {
    CUtensorMap qm, km, vm, om;
    // packed varlen buffers are one "batch" of total rows
    const bool packed = p.mode == MODE_VARLEN;
    const int q_batch = packed ? 1 : p.num_seqs, q_rows = packed ? p.total_q : p.q_seq_len;
    const int k_batch = packed ? 1 : p.num_seqs, k_rows = packed ? p.total_k : p.kv_seq_len;
    // head size 32 runs on the D = 64 kernel: the maps carry the real inner extent (32), the 64-column
    // boxes read zeros past it and bulk stores write nothing there
    const int d_real = p.head_size;
    bool ok = encode_map(&qm, p.q, p.dtype, d_real, q_batch, q_rows, p.q_heads);
    // The output as 32-row boxes (one per softmax warp). Bulk stores are used for a single, local output
    // only: a head-sharded call (n_out > 0) stores every copy with plain stores, and no tensor map is
    // ever made over another GPU's memory — the kernel's fourth map is then a second one over q, unused.
    if (p.n_out > 0) om = qm;
    else ok = ok && encode_map(&om, p.o, p.dtype, d_real, q_batch, q_rows, p.q_heads, 32);
    if (p.paged) {
        ok = ok && encode_paged_map(&km, p.k, p.dtype, d_real, p.block_size, p.kv_heads) &&
             encode_paged_map(&vm, p.v, p.dtype, d_real, p.block_size, p.kv_heads);
    } else {
        ok = ok && encode_map(&km, p.k, p.dtype, d_real, k_batch, k_rows, p.kv_heads) &&
             encode_map(&vm, p.v, p.dtype, d_real, k_batch, k_rows, p.kv_heads);
    }
    if (!ok) return -1;  // let the SIMT kernel take it
    int* status = status_word();
    if (status == nullptr) return -1;

    PrefillArgs a{};
    if (p.n_out > 0) {
        if (p.n_out > kMaxPeers || p.n_lse > kMaxPeers) return -1;
        for (int i = 0; i < p.n_out; ++i) a.o[i] = p.o_peers[i];
        for (int i = 0; i < p.n_lse; ++i) a.lse_peers[i] = p.lse_peers[i];
        a.n_out = p.n_out;
        a.n_lse = p.n_lse;
        a.o_heads = p.o_heads;
        a.o_head0 = p.o_head0;
        // with equal shards this GPU's index in the group is o_head0 / q_heads: start one past it
        a.peer0 = (p.o_head0 / p.q_heads + 1) % p.n_out;
        a.multicast = p.multicast;
    } else {
        a.o[0] = p.o;
        a.n_out = 1;
        a.o_heads = p.q_heads;
        a.o_head0 = 0;
    }
    a.lse = p.lse;
    a.status = status;
    a.wait_ns = get_option_prefill_wait_us() > 0 ? (unsigned long long)get_option_prefill_wait_us() * 1000ULL : kWaitLimitNs;
    a.test_skip_k = get_option_prefill_test_skip_k();
#ifdef FA_TRACE
    {
        unsigned char* dbg = get_option_prefill_trace() != 0 ? debug_area() : nullptr;
        a.staged_store = get_option_prefill_trace() == 2 ? 1 : 0;
        a.trace_y = get_option_prefill_trace_y();
        a.cta_log = (dbg != nullptr && get_option_prefill_trace() == 3) ? reinterpret_cast<long long*>(dbg + 16384) : nullptr;
        a.trace = (dbg != nullptr && get_option_prefill_trace() == 1) ? reinterpret_cast<long long*>(dbg + 256) : nullptr;
    }
#endif
    a.batch = p.num_seqs;
    a.q_seq_len = p.q_seq_len;
    a.kv_seq_len = p.kv_seq_len;
    a.q_heads = p.q_heads;
    a.kv_heads = p.kv_heads;
    a.start_pos = p.start_pos;
    a.d_real = d_real;
    a.mode = p.mode;
    a.q = p.q;
    a.k = p.k;
    a.v = p.v;
    a.mask = p.mode == MODE_BATCH ? static_cast<const unsigned char*>(p.mask) : nullptr;
    a.cu_q = p.cu_q;
    a.cu_k = p.cu_k;
    a.context_lens = p.context_lens;
    a.block_tables = p.block_tables;
    a.paged = p.paged;
    a.block_size = p.block_size;
    a.max_blocks = p.max_blocks;
    a.scale_log2 = p.scale * 1.4426950408889634f;

    const int group = p.q_heads / p.kv_heads;
    const int num_mb = (p.q_seq_len + kBlockM - 1) / kBlockM;
    const int pairs = (group * num_mb + 1) / 2;
    const size_t smem = sizeof(SharedStorage<D>) + 1024;
    cudaError_t err = cudaFuncSetAttribute(prefill_tcgen05_kernel<T, D, kMask>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) {
        set_last_errorf("prefill_tcgen05_kernel: %s", cudaGetErrorString(err));
        cudaGetLastError();
        return FLASH_ATTN_ERR_CUDA;
    }
    // Band width: the pairs of a band start together, so their work must be about equal or the
    // heaviest-first order is lost (at S = 2048 without GQA, bands of 2 cost 13 %). A band of w
    // pairs spans 2w / group row blocks, i.e. that many K/V tiles of difference between its lightest
    // and heaviest pair: keep that within an eighth of the longest K/V range, at most 8 pairs (16 measured no better).
    int band = 1;
    {
        const int kv_rows = p.mode == MODE_KVCACHE ? p.max_blocks * p.block_size : p.kv_seq_len;   // upper bound per sequence
        const int kv_tiles = std::max(1, (kv_rows + kBlockN - 1) / kBlockN);
        while (band < 8 && band * 2 <= pairs && (long long)(band * 2) * 2 * 8 <= (long long)kv_tiles * group) band *= 2;
        if (get_option_prefill_band() > 0) band = std::min(get_option_prefill_band(), pairs);
    }
    a.band = band;
    // Head-sharded call (every CTA ends with stores to the other GPUs): heaviest-first makes the SMs end
    // their CTAs in waves, each wave a burst on the links that stalls every SM in it. A first wave that
    // mixes all weights staggers the SMs for the rest of the launch; the rest stays heaviest first, which
    // keeps the tail balanced.
    {
        const int rows = (pairs + band - 1) / band;
        const int per_row = p.kv_heads * p.num_seqs * band;
        int sms = 148;
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const int w = (sms + per_row - 1) / per_row;
        const int m = w > 0 ? rows / w : 0;
        const bool spread = p.n_out > 1 && get_option_prefill_order() != 1 && m >= 2;
        a.spread_w = spread ? w : 0;
        a.spread_m = spread ? m : 0;
    }
    if ((long long)p.kv_heads * p.num_seqs * band > 0x7fffffffLL) return -1;
    // Groups of K/V streams (blockIdx.z). Every tile pair of a (batch, KV head) stream re-reads the stream's
    // K/V prefix; with many streams and no sharing inside a launch band the prefixes in flight exceed L2 and
    // come from HBM again (B=4, H=32, S=2048: 523 MB read for 201 MB of q, k and v). Running the streams in
    // groups of about 16 MiB of K/V keeps the re-reads in L2 (the same launch: 201 MB read, 823 -> 851-871
    // TFLOP/s; 4 groups 843, 12-32 groups 810-834); within a group the order is unchanged.
    int groups = 1;
    {
        const long long streams = (long long)p.kv_heads * p.num_seqs;
        const long long kv_bytes_per_stream = 2LL * (p.mode == MODE_KVCACHE ? (long long)p.max_blocks * p.block_size : p.kv_seq_len) * D * 2;
        const long long budget = 16LL << 20;
        if (get_option_prefill_groups() > 0) groups = get_option_prefill_groups();
        else if (band == 1 && pairs > 1 && p.n_out <= 1 && streams * kv_bytes_per_stream > 2 * budget)
            groups = (int)std::min<long long>(streams, (streams * kv_bytes_per_stream + budget - 1) / budget);
        else if (band > 1 && p.n_out <= 1 && (p.mode == MODE_BATCH || p.mode == MODE_VARLEN) && p.num_seqs >= 2 &&
                 streams * kv_bytes_per_stream > (48LL << 20) * (p.mode == MODE_VARLEN ? 2 : 1)) {
            // GQA launches share K/V inside a band already; running whole batch elements (sequences) one after
            // the other, about 48 MiB of K/V at a time, still keeps more of q, k, v and o in L2 and with it
            // power for the tensor pipe: B=2, Hq=32, Hkv=8, S=8192 1235-1237 against 1223-1225 TFLOP/s; 32 packed
            // prompts of 1024-8192 tokens 1015-1075 against 989-993 (12 to 20 groups). A packed call gives only
            // the longest sequence: the others are taken as half as long on average.
            const long long per_elem = (long long)p.kv_heads * kv_bytes_per_stream / (p.mode == MODE_VARLEN ? 2 : 1);
            const long long elems = std::max<long long>(1, (48LL << 20) / per_elem);
            groups = (int)((p.num_seqs + elems - 1) / elems);
        }
        if (groups > 65535) groups = 65535;
        if (groups < 1) groups = 1;
    }
    const int streams_per_group = (int)(((long long)p.kv_heads * p.num_seqs + groups - 1) / groups);
    dim3 grid(streams_per_group * band, (pairs + band - 1) / band, groups);
    prefill_tcgen05_kernel<T, D, kMask><<<grid, kThreads, smem, stream>>>(qm, km, vm, om, a);
    const int rc = check_launch("prefill_tcgen05_kernel");
    if (rc == FLASH_ATTN_OK) note_path("prefill_tcgen05", 1);
    return rc;
}

}  // namespace

int prefill_take_status() {
    int* status = status_word();
    if (status == nullptr) return 0;
    volatile int* w = status;
    const int h = *w;
    if (h != 0) *w = 0;
    return h;
}

int prefill_device_status() {
    int* status = status_word();
    if (status == nullptr) return -1;
    if (cudaDeviceSynchronize() != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    return prefill_take_status();
}

int prefill_debug_read(void* dst, int bytes) {
#ifdef FA_TRACE
    unsigned char* dbg = debug_area();
    int* status = status_word();
    if (dbg == nullptr || status == nullptr || dst == nullptr || bytes <= 0) return -1;
    const size_t n = (size_t)bytes < kDebugBytes ? (size_t)bytes : kDebugBytes;
    if (cudaMemcpy(dst, dbg, n, cudaMemcpyDeviceToHost) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    if (n >= sizeof(int)) std::memcpy(dst, status, sizeof(int));
    return (int)n;
#else
    (void)dst;
    (void)bytes;
    return -1;   // the timeline is compiled in with -DFA_TRACE only
#endif
}

int launch_prefill_tcgen05(const AttnParams& p, cudaStream_t stream) {
    // batched entry point, chunked prefill over a paged cache (whole pages must tile the 128-key
    // K/V tile), and the packed varlen entry point. The reference's varlen signature does not say how
    // many rows the packed buffers have: their tensor maps then carry no row bound, and the kernel
    // fetches the tiles at the very end of the buffers with plain loads (edge_tile_copy).
    if (p.mask != nullptr && p.mode != MODE_BATCH) return -1;
    if (p.mode == MODE_KVCACHE) {
        if (!p.paged || p.max_blocks <= 0) return -1;
    } else if (p.mode == MODE_VARLEN) {
        if (p.paged && p.max_blocks <= 0) return -1;
    } else if (p.mode != MODE_BATCH) {
        return -1;
    }
    if (p.paged && (p.block_size < 8 || p.block_size > 128 || (128 % p.block_size) != 0)) return -1;
    if (p.dtype != DT_F16 && p.dtype != DT_BF16) return -1;
    if (p.head_size != 32 && p.head_size != 64 && p.head_size != 128) return -1;
    if (!(p.scale > 0.0f)) return -1;
    // (single-token calls of the kv-cache entry point never get here: the dispatcher tries the split-K
    // decode kernel first; single rows through the batched or packed entry points do)
    uintptr_t align = reinterpret_cast<uintptr_t>(p.q) | reinterpret_cast<uintptr_t>(p.k) |
                      reinterpret_cast<uintptr_t>(p.v) | reinterpret_cast<uintptr_t>(p.o);
    for (int i = 0; i < p.n_out && i < 8; ++i) align |= reinterpret_cast<uintptr_t>(p.o_peers[i]);
    if (align & 15) return -1;
    const long long pairs = ((long long)(p.q_heads / p.kv_heads) * ((p.q_seq_len + kBlockM - 1) / kBlockM) + 1) / 2;
    if (pairs > 65535) return -1;
    const bool masked = p.mask != nullptr;
    if (p.head_size == 64 || p.head_size == 32) {
        if (p.dtype == DT_BF16) return masked ? launch_typed<__nv_bfloat16, 64, true>(p, stream) : launch_typed<__nv_bfloat16, 64, false>(p, stream);
        return masked ? launch_typed<__half, 64, true>(p, stream) : launch_typed<__half, 64, false>(p, stream);
    }
    if (p.dtype == DT_BF16) return masked ? launch_typed<__nv_bfloat16, 128, true>(p, stream) : launch_typed<__nv_bfloat16, 128, false>(p, stream);
    return masked ? launch_typed<__half, 128, true>(p, stream) : launch_typed<__half, 128, false>(p, stream);
}

}  // namespace fa
