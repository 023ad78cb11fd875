// TEST INFRASTRUCTURE ONLY — never linked into, imported by or called from the product path.
//
// CPU restatement of the attention arithmetic the luma reference defines, used as the parity
// checker for the CUDA kernels and as the timed CPU baseline. Two families of functions:
//
//  1. oracle_sdpa_math_f32  — luma-cpu's "math path" scaled-dot-product attention in f32,
//     op for op: head-major view, KV-head expansion for GQA, f32 GEMM Q.K^T, multiply by the
//     scale cast to f32, causal mask to -inf (j <= start_pos + i), single-pass online softmax,
//     f32 GEMM P.V.
//       definition ........ luma-tensor/src/ops/nn/attention.rs:11-45 (forward),
//                           :95-103 (expand_heads), :118-127 (causal_mask)
//       scale as f32 ...... luma-cpu/src/ops/float_ops.rs:328-335
//       masked -> -inf .... luma-cpu/src/ops/float_ops.rs:746-787
//       online softmax .... luma-cpu/src/kernels/nn.rs:39-56
//       GEMM call site .... luma-cpu/src/kernels/matmul.rs:64-107 (per batch element, alpha=1,
//                           beta=0, row-major output)
//     The f32 GEMM inside luma-cpu is the third-party crate `gemm` 0.19.0 (Cargo.lock:579-582),
//     which is not part of the reference tree; its SIMD summation order cannot be reproduced,
//     so this file fixes its own order (8 interleaved partial sums folded pairwise for the
//     Q.K^T dot products, ascending key order for P.V). Parity with luma-cpu is therefore by
//     tolerance, not bit for bit. Pinned by the closed-form known-answer case of
//     luma-tensor/src/tests/nn.rs:289-304 and by agreement with the f64 loop below.
//
//  2. oracle_attn_f64 — the direct f64 triple loop the reference's own GPU tests compare
//     against, generalised over the three entry points:
//       batched + padding mask + start_pos .. luma-flash-attn/tests/low.rs:45-117
//       batched, no mask .................... luma-flash-attn/tests/high.rs:29-86
//       varlen / paged variants ............. luma-flash-attn/tests/high.rs:208-379 (built from
//                                             ref_attention with start_pos = k_len - q_len)
//       paged slot arithmetic ............... luma-flash-attn/kernels/common.cuh:89-108
//
//  plus the deterministic generators of those tests (xorshift64*, tests/low.rs:363-384 and
//  tests/high.rs:13-24) and a host block_slot table walk used for the bit-exact index check.
//
// Build: see oracle/Makefile (g++ -O3 -shared). Loaded through ctypes by tests/, the smoke check
// and the bench's cpu_baseline leg only.

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <thread>
#include <vector>

namespace {

template <typename F>
void parallel_for(int64_t n, int nthreads, F&& fn) {
    if (nthreads <= 1 || n <= 1) {
        for (int64_t i = 0; i < n; ++i) fn(i);
        return;
    }
    std::atomic<int64_t> next{0};
    std::vector<std::thread> pool;
    const int nt = static_cast<int>(std::min<int64_t>(nthreads, n));
    pool.reserve(nt);
    for (int t = 0; t < nt; ++t) {
        pool.emplace_back([&]() {
            for (;;) {
                const int64_t i = next.fetch_add(1);
                if (i >= n) break;
                fn(i);
            }
        });
    }
    for (auto& th : pool) th.join();
}

// f32 dot product with a fixed, documented summation order: 8 interleaved partial sums
// (element x goes to lane x % 8), folded as ((0+4)+(2+6)) + ((1+5)+(3+7)).
inline float dot_f32(const float* a, const float* b, int n) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int x = 0;
    for (; x + 8 <= n; x += 8) {
        for (int l = 0; l < 8; ++l) acc[l] += a[x + l] * b[x + l];
    }
    for (int l = 0; x < n; ++x, ++l) acc[l] += a[x] * b[x];
    const float s04 = acc[0] + acc[4], s26 = acc[2] + acc[6];
    const float s15 = acc[1] + acc[5], s37 = acc[3] + acc[7];
    return (s04 + s26) + (s15 + s37);
}

// luma-cpu/src/kernels/nn.rs:39-56 — running max m and running sum s; when a larger value
// appears the sum is rescaled by exp(m - x). Output exp(x - m) / s. In place.
inline void online_softmax_f32(float* row, int n, float* m_out, float* s_out) {
    if (n == 0) return;
    float m = row[0];
    float s = 1.0f;
    for (int i = 1; i < n; ++i) {
        const float x = row[i];
        if (x <= m) {
            s = s + std::exp(x - m);
        } else {
            s = s * std::exp(m - x) + 1.0f;
            m = x;
        }
    }
    for (int i = 0; i < n; ++i) row[i] = std::exp(row[i] - m) / s;
    if (m_out) *m_out = m;
    if (s_out) *s_out = s;
}

}  // namespace

extern "C" {

// Math-path SDPA in f32. q/o: (B, Lq, Hq, D); k/v: (B, Lk, Hkv, D); all dense row-major.
// lse (optional, may be null): (B, Hq, Lq) natural-log-sum-exp of the scaled, masked scores.
// Returns 0 on success, 1 on bad arguments.
int oracle_sdpa_math_f32(const float* q, const float* k, const float* v, float* o, float* lse,
                         int B, int Lq, int Lk, int Hq, int Hkv, int D,
                         double scale, int causal, int start_pos, int nthreads) {
    if (!q || !k || !v || !o || B <= 0 || Lq <= 0 || Lk <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0) return 1;
    if (Hq % Hkv != 0) return 1;
    const int group = Hq / Hkv;
    const float scale_f = static_cast<float>(scale);  // float_ops.rs:328-335
    const float neg_inf = -std::numeric_limits<float>::infinity();
    constexpr int kRowBlock = 32;
    const int row_blocks = (Lq + kRowBlock - 1) / kRowBlock;
    const int64_t jobs = static_cast<int64_t>(B) * Hq * row_blocks;

    parallel_for(jobs, nthreads, [&](int64_t job) {
        const int rb = static_cast<int>(job % row_blocks);
        const int h = static_cast<int>((job / row_blocks) % Hq);
        const int b = static_cast<int>(job / (static_cast<int64_t>(row_blocks) * Hq));
        const int kh = h / group;  // expand_heads: KV head kh repeated `group` times consecutively
        const int i0 = rb * kRowBlock;
        const int i1 = std::min(Lq, i0 + kRowBlock);

        // head-major contiguous copies of this KV head (the reference materialises
        // (B, Hq, Lk, D) with .contiguous(); same values, same order)
        std::vector<float> kh_buf(static_cast<size_t>(Lk) * D), vh_buf(static_cast<size_t>(Lk) * D);
        for (int j = 0; j < Lk; ++j) {
            const size_t src = ((static_cast<size_t>(b) * Lk + j) * Hkv + kh) * D;
            std::memcpy(&kh_buf[static_cast<size_t>(j) * D], k + src, sizeof(float) * D);
            std::memcpy(&vh_buf[static_cast<size_t>(j) * D], v + src, sizeof(float) * D);
        }
        std::vector<float> scores(Lk);
        std::vector<float> acc(D);
        for (int i = i0; i < i1; ++i) {
            const float* qi = q + ((static_cast<size_t>(b) * Lq + i) * Hq + h) * D;
            // GEMM Q.K^T over the FULL key range (the math path does not skip masked tiles),
            // then scale, then mask.
            for (int j = 0; j < Lk; ++j) scores[j] = dot_f32(qi, &kh_buf[static_cast<size_t>(j) * D], D) * scale_f;
            if (causal) {
                const int64_t limit = static_cast<int64_t>(start_pos) + i;
                for (int j = 0; j < Lk; ++j)
                    if (j > limit) scores[j] = neg_inf;
            }
            float m = 0.f, s = 0.f;
            online_softmax_f32(scores.data(), Lk, &m, &s);
            if (lse) lse[(static_cast<size_t>(b) * Hq + h) * Lq + i] = m + std::log(s);
            // GEMM P.V, ascending key order
            std::fill(acc.begin(), acc.end(), 0.0f);
            for (int j = 0; j < Lk; ++j) {
                const float p = scores[j];
                const float* vj = &vh_buf[static_cast<size_t>(j) * D];
                for (int x = 0; x < D; ++x) acc[x] += p * vj[x];
            }
            float* oi = o + ((static_cast<size_t>(b) * Lq + i) * Hq + h) * D;
            std::memcpy(oi, acc.data(), sizeof(float) * D);
        }
    });
    return 0;
}

// Logical token j of sequence s -> physical token slot (kernels/common.cuh:89-108):
//   block_tables[s * max_blocks + j / block_size] * block_size + j % block_size
// Writes, for every sequence s and every j < lens[s], the slot into out[offsets[s] + j] where
// offsets is the exclusive prefix sum of lens. 32-bit arithmetic like the reference.
int oracle_block_slots(const int* block_tables, const int* lens, int num_seqs, int max_blocks,
                       int block_size, int* out) {
    if (!block_tables || !lens || !out || block_size <= 0) return 1;
    int64_t off = 0;
    for (int s = 0; s < num_seqs; ++s) {
        for (int j = 0; j < lens[s]; ++j) {
            const int logical_block = j / block_size;
            const int offset = j % block_size;
            out[off + j] = block_tables[s * max_blocks + logical_block] * block_size + offset;
        }
        off += lens[s];
    }
    return 0;
}

// General f64 attention loop over packed sequences.
//   q, o : rows of Hq*D doubles; row index of (seq s, local row i) is q_start[s] + i
//   k, v : rows of Hkv*D doubles; row index of (seq s, key j) is
//            block_size == 0 : kv_start[s] + j
//            block_size  > 0 : block_slot(block_tables, s, max_blocks, j, block_size)
//   query row i of sequence s sits at global position g = pos_offset[s] + i and sees keys
//   j < kv_len[s] with j <= g and (mask == null or mask[s*mask_stride + j] != 0).
//   With a mask the query row itself is valid only if 0 <= g < mask_stride and mask[s*..+g] != 0.
//   Invalid rows and rows with no visible key produce zeros (tests/low.rs:95-98).
//   lse (optional): (num_seqs rows packed like q, Hq) natural log-sum-exp, -inf for empty rows.
int oracle_attn_f64(const double* q, const double* k, const double* v, double* o, double* lse,
                    int num_seqs, const int* q_start, const int* q_len, const int* kv_start,
                    const int* kv_len, const int* pos_offset, int Hq, int Hkv, int D, double scale,
                    const int* block_tables, int max_blocks, int block_size,
                    const uint8_t* mask, int mask_stride, int nthreads) {
    if (!q || !k || !v || !o || num_seqs <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || Hq % Hkv) return 1;
    const int group = Hq / Hkv;
    const int64_t jobs = static_cast<int64_t>(num_seqs) * Hq;
    parallel_for(jobs, nthreads, [&](int64_t job) {
        const int s = static_cast<int>(job / Hq);
        const int h = static_cast<int>(job % Hq);
        const int kh = h / group;
        const int L = kv_len[s];
        std::vector<double> sc(std::max(L, 1));
        std::vector<int64_t> krow(std::max(L, 1));
        for (int j = 0; j < L; ++j) {
            if (block_size > 0) {
                const int slot = block_tables[s * max_blocks + j / block_size] * block_size + j % block_size;
                krow[j] = slot;
            } else {
                krow[j] = static_cast<int64_t>(kv_start[s]) + j;
            }
        }
        std::vector<double> acc(D);
        for (int i = 0; i < q_len[s]; ++i) {
            const int64_t g = static_cast<int64_t>(pos_offset[s]) + i;
            const int64_t qrow = static_cast<int64_t>(q_start[s]) + i;
            const double* qi = q + (qrow * Hq + h) * D;
            double* oi = o + (qrow * Hq + h) * D;
            for (int x = 0; x < D; ++x) oi[x] = 0.0;
            if (lse) lse[qrow * Hq + h] = -std::numeric_limits<double>::infinity();
            bool q_valid = true;
            if (mask) q_valid = g >= 0 && g < mask_stride && mask[static_cast<int64_t>(s) * mask_stride + g] != 0;
            double m = -std::numeric_limits<double>::infinity();
            int nvis = 0;
            for (int j = 0; j < L; ++j) {
                bool visible = mask ? (mask[static_cast<int64_t>(s) * mask_stride + j] != 0) : true;
                if (visible) visible = g >= j;
                if (!visible) {
                    sc[j] = std::numeric_limits<double>::quiet_NaN();
                    continue;
                }
                const double* kj = k + (krow[j] * Hkv + kh) * D;
                double dot = 0.0;
                for (int x = 0; x < D; ++x) dot += qi[x] * kj[x];
                dot *= scale;
                sc[j] = dot;
                m = std::max(m, dot);
                ++nvis;
            }
            if (!q_valid || nvis == 0) continue;
            double denom = 0.0;
            std::fill(acc.begin(), acc.end(), 0.0);
            for (int j = 0; j < L; ++j) {
                if (std::isnan(sc[j])) continue;
                const double p = std::exp(sc[j] - m);
                denom += p;
                const double* vj = v + (krow[j] * Hkv + kh) * D;
                for (int x = 0; x < D; ++x) acc[x] += p * vj[x];
            }
            for (int x = 0; x < D; ++x) oi[x] = acc[x] / denom;
            if (lse) lse[qrow * Hq + h] = m + std::log(denom);
        }
    });
    return 0;
}

// xorshift64* stream of the reference tests: state = seed | 1; each draw is the top 24 bits
// of state * 0x2545F4914F6CDD1D mapped to [-1, 1).
//   f32 flavour: tests/low.rs:363-384 ((bits as f32 / 2^24) * 2 - 1, in f32)
//   f64 flavour: tests/high.rs:13-24  (same bits in f64)
// `state` is in/out so consecutive tensors continue one stream as tests/low.rs:148-152 does.
void oracle_xorshift_fill_f32(uint64_t* state, float* out, int64_t n) {
    uint64_t x = *state;
    for (int64_t i = 0; i < n; ++i) {
        x ^= x >> 12;
        x ^= x << 25;
        x ^= x >> 27;
        const uint64_t r = x * 0x2545F4914F6CDD1DULL;
        const uint32_t bits = static_cast<uint32_t>(r >> 40);
        out[i] = (static_cast<float>(bits) / static_cast<float>(1u << 24)) * 2.0f - 1.0f;
    }
    *state = x;
}

void oracle_xorshift_fill_f64(uint64_t* state, double* out, int64_t n) {
    uint64_t x = *state;
    for (int64_t i = 0; i < n; ++i) {
        x ^= x >> 12;
        x ^= x << 25;
        x ^= x >> 27;
        const uint64_t r = x * 0x2545F4914F6CDD1DULL;
        out[i] = (static_cast<double>(r >> 40) / static_cast<double>(1ULL << 24)) * 2.0 - 1.0;
    }
    *state = x;
}

int oracle_hardware_threads(void) {
    const unsigned n = std::thread::hardware_concurrency();
    return n == 0 ? 1 : static_cast<int>(n);
}


// Row softmax over the last dimension of a dense (rows, n) f32 matrix with luma-cpu's own routine
// (luma-cpu/src/kernels/nn.rs:10-56: contiguous last-dim case -> online_softmax per row).
int oracle_softmax_last_dim_f32(const float* in, float* out, long long rows, int n) {
    if (in == nullptr || out == nullptr || rows < 0 || n < 0) return 1;
    for (long long r = 0; r < rows; ++r) {
        float* row = out + r * n;
        for (int i = 0; i < n; ++i) row[i] = in[r * n + i];
        float m = 0.0f, s = 0.0f;
        online_softmax_f32(row, n, &m, &s);
    }
    return 0;
}

}  // extern "C"
