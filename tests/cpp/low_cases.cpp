// The reference's low-level suite (luma-flash-attn/tests/low.rs) driven through the C++ host
// mirror include/luma_flash_attn.hpp: the eleven numeric cases (same shapes, seeds, xorshift64*
// stream and 3e-3 + 3e-3*|x| bar, checked against the oracle's f64 loop) and the seven error
// cases. Links libflash_attn.so and, as the checker only, oracle/liboracle.so.
// Prints one line per case and exits non-zero on the first failure.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "../../include/luma_flash_attn.hpp"

extern "C" {
int oracle_attn_f64(const double* q, const double* k, const double* v, double* o, double* lse, int num_seqs,
                    const int* q_start, const int* q_len, const int* kv_start, const int* kv_len, const int* pos_offset,
                    int Hq, int Hkv, int D, double scale, const int* block_tables, int max_blocks, int block_size,
                    const uint8_t* mask, int mask_stride, int nthreads);
void oracle_xorshift_fill_f32(uint64_t* state, float* out, int64_t n);
}

using namespace luma_flash_attn;
using Kind = FlashAttnError::Kind;

enum MaskKind { kNone, kRandom, kAllOnes };
struct Case { const char* name; uint64_t seed; int batch, sq, skv, hq, hkv, d, start_pos; MaskKind mask; };

template <typename T>
struct DevBuf {
    T* p = nullptr;
    size_t n = 0;
    explicit DevBuf(size_t n_) : n(n_) { if (cudaMalloc(&p, (n ? n : 1) * sizeof(T)) != cudaSuccess) { std::fprintf(stderr, "cudaMalloc failed\n"); std::exit(2); } }
    ~DevBuf() { cudaFree(p); }
    void upload(const std::vector<T>& h) { cudaMemcpy(p, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice); }
    DeviceSlice<const T> cslice() const { return DeviceSlice<const T>(p, n); }
    DeviceSlice<T> slice() { return DeviceSlice<T>(p, n); }
};

static int run_case(const Case& c) {
    const size_t q_sz = (size_t)c.batch * c.sq * c.hq * c.d, kv_sz = (size_t)c.batch * c.skv * c.hkv * c.d;
    uint64_t state = c.seed | 1;   // one stream: q, k, v, then the mask (tests/low.rs:148-152)
    std::vector<float> q(q_sz), k(kv_sz), v(kv_sz);
    oracle_xorshift_fill_f32(&state, q.data(), q_sz);
    oracle_xorshift_fill_f32(&state, k.data(), kv_sz);
    oracle_xorshift_fill_f32(&state, v.data(), kv_sz);
    std::vector<uint8_t> mask;
    if (c.mask == kAllOnes) mask.assign((size_t)c.batch * c.skv, 1);
    if (c.mask == kRandom) {
        std::vector<float> r((size_t)c.batch * c.skv);
        oracle_xorshift_fill_f32(&state, r.data(), r.size());
        for (float x : r) mask.push_back(x > -0.2f ? 1 : 0);
    }
    DevBuf<float> dq(q_sz), dk(kv_sz), dv(kv_sz), dout(q_sz);
    DevBuf<uint8_t> dmask(mask.size());
    dq.upload(q); dk.upload(k); dv.upload(v);
    if (!mask.empty()) dmask.upload(mask);
    std::vector<float> poison(q_sz, NAN);
    dout.upload(poison);   // the op must overwrite every element
    auto o = dout.slice();
    DeviceSlice<const uint8_t> ms = dmask.cslice();
    try {
        low::flash_attn_f32(dq.cslice(), dk.cslice(), dv.cslice(), o, c.batch, c.sq, c.skv, c.hq, c.hkv, c.d, c.start_pos,
                            1.0f / std::sqrt((float)c.d), mask.empty() ? nullptr : &ms, nullptr);
    } catch (const FlashAttnError& e) {
        std::printf("FAIL %s: %s\n", c.name, e.what());
        return 1;
    }
    if (cudaDeviceSynchronize() != cudaSuccess) { std::printf("FAIL %s: sync\n", c.name); return 1; }
    std::vector<float> got(q_sz);
    cudaMemcpy(got.data(), dout.p, q_sz * sizeof(float), cudaMemcpyDeviceToHost);

    std::vector<double> qd(q.begin(), q.end()), kd(k.begin(), k.end()), vd(v.begin(), v.end()), want(q_sz);
    std::vector<int> qs(c.batch), ql(c.batch, c.sq), ks(c.batch), kl(c.batch, c.skv), po(c.batch, c.start_pos);
    for (int b = 0; b < c.batch; ++b) { qs[b] = b * c.sq; ks[b] = b * c.skv; }
    oracle_attn_f64(qd.data(), kd.data(), vd.data(), want.data(), nullptr, c.batch, qs.data(), ql.data(), ks.data(), kl.data(),
                    po.data(), c.hq, c.hkv, c.d, 1.0 / std::sqrt((double)c.d), nullptr, 0, 0, mask.empty() ? nullptr : mask.data(),
                    c.skv, 4);
    double worst = 0;
    for (size_t i = 0; i < q_sz; ++i) {
        const double diff = std::fabs((double)got[i] - want[i]);
        const double tol = 3e-3 + 3e-3 * std::fabs(want[i]);   // tests/low.rs:129
        if (!(diff <= tol)) { std::printf("FAIL %s: idx %zu got %g want %g\n", c.name, i, got[i], want[i]); return 1; }
        worst = diff > worst ? diff : worst;
    }
    std::printf("ok   %s (max abs err %.2e)\n", c.name, worst);
    return 0;
}

template <typename F>
static int expect_error(const char* name, Kind kind, F&& f) {
    try {
        f();
    } catch (const FlashAttnError& e) {
        if (e.kind() == kind) { std::printf("ok   %s -> %s\n", name, e.what()); return 0; }
        std::printf("FAIL %s: wrong kind: %s\n", name, e.what());
        return 1;
    }
    std::printf("FAIL %s: no error\n", name);
    return 1;
}

int main() {
    int dev_count = 0;
    if (cudaGetDeviceCount(&dev_count) != cudaSuccess || dev_count == 0) { std::printf("no CUDA device\n"); return 3; }
    const Case cases[] = {
        {"mha_head32_exact_tiles", 1, 2, 64, 64, 4, 4, 32, 0, kNone},
        {"mha_head64_unaligned_seq", 2, 1, 100, 100, 4, 4, 64, 0, kNone},
        {"mha_head32_uneven_seq", 3, 3, 129, 200, 6, 6, 32, 0, kNone},
        {"gqa_head128", 4, 2, 70, 70, 8, 2, 128, 0, kNone},
        {"causal_zero_start_pos", 5, 1, 32, 32, 1, 1, 64, 0, kNone},
        {"mask_random_padding", 6, 2, 128, 128, 4, 4, 32, 0, kRandom},
        {"mask_all_ones_equals_no_mask", 7, 1, 64, 64, 2, 2, 64, 0, kAllOnes},
        {"kv_cache_start_pos_offset", 8, 1, 40, 72, 8, 2, 64, 32, kNone},
        {"start_pos_unaligned_to_block", 9, 2, 50, 120, 4, 4, 32, 70, kNone},
        {"gqa_mask_with_start_pos", 10, 2, 33, 100, 8, 4, 128, 67, kRandom},
        {"single_token_decode", 11, 1, 1, 96, 4, 4, 64, 95, kNone},
    };
    int failures = 0;
    for (const Case& c : cases) failures += run_case(c);

    // error cases, tests/low.rs:278-358
    DevBuf<float> t(1);
    auto tiny = [&]() { return t.cslice(); };
    auto o1 = t.slice();
    failures += expect_error("err_invalid_head_size", Kind::InvalidHeadSize, [&] { low::flash_attn_f32(tiny(), tiny(), tiny(), o1, 1, 1, 1, 1, 1, 48, 0, 0.1f, nullptr, nullptr); });
    failures += expect_error("err_non_multiple_heads", Kind::InvalidShape, [&] { low::flash_attn_f32(tiny(), tiny(), tiny(), o1, 1, 1, 1, 3, 2, 32, 0, 0.1f, nullptr, nullptr); });
    failures += expect_error("err_negative_start_pos", Kind::InvalidStartPos, [&] { low::flash_attn_f32(tiny(), tiny(), tiny(), o1, 1, 1, 1, 1, 1, 32, -1, 0.1f, nullptr, nullptr); });
    failures += expect_error("err_zero_shape", Kind::InvalidShape, [&] { low::flash_attn_f32(tiny(), tiny(), tiny(), o1, 0, 1, 1, 1, 1, 32, 0, 0.1f, nullptr, nullptr); });
    failures += expect_error("err_buffer_too_small", Kind::BufferTooSmall, [&] { low::flash_attn_f32(tiny(), tiny(), tiny(), o1, 1, 64, 64, 4, 4, 32, 0, 0.1f, nullptr, nullptr); });
    {
        const size_t n = 64 * 4 * 32;
        DevBuf<float> a(n), b(n), c(n), d(n);
        DevBuf<uint8_t> m(1);
        auto od = d.slice();
        DeviceSlice<const uint8_t> ms = m.cslice();
        failures += expect_error("err_mask_buffer_too_small", Kind::BufferTooSmall, [&] { low::flash_attn_f32(a.cslice(), b.cslice(), c.cslice(), od, 1, 64, 64, 4, 4, 32, 0, 0.1f, &ms, nullptr); });
    }
    {
        const int code = flash_attn_f32(nullptr, nullptr, nullptr, nullptr, 1, 1, 1, 1, 1, 32, 0, 1.0f, nullptr, nullptr);
        const bool ok = code == FLASH_ATTN_ERR_NULL_PTR && flash_attn_last_error()[0] != '\0';
        failures += expect_error("err_null_ptr_from_c_abi", Kind::NullPtr, [&] { FlashAttnError::from_status(code); });
        if (!ok) { std::printf("FAIL null ptr code/message\n"); ++failures; }
    }
    std::printf("%s (%d failure(s))\n", failures ? "FAILED" : "PASSED", failures);
    return failures ? 1 : 0;
}
