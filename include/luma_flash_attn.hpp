// C++ host-side mirror of luma's Rust crate `luma-flash-attn` over the C ABI of flash_attn.h.
//
// The reference's host layer is Rust (luma-flash-attn/src/{error.rs, api/low.rs}); this header
// restates the part of it that sits directly above the FFI — same names, same argument order,
// same validation order, same error kinds and messages — for callers that are compiled code.
// It is header-only, needs only the CUDA runtime for the stream type, and adds no behaviour of
// its own: every function validates like its Rust counterpart and then calls the C symbol.
//
//   FlashAttnError            <- error.rs:7-51   (kinds, Display strings, from_status)
//   DeviceSlice<T>            <- the role cudarc's CudaSlice<T> / DevicePtr<T> plays in low.rs
//   low::flash_attn<T>        <- low.rs:146-197  (+ validate :360-407, check_len :409-416)
//   low::flash_attn_varlen<T> <- low.rs:231-295
//   low::flash_attn_with_kvcache<T> <- low.rs:305-357
//   FlashDtype<T>             <- low.rs:14-134   (f32 / f16 / bf16 -> the typed C symbols)
#ifndef LUMA_B200_LUMA_FLASH_ATTN_HPP_
#define LUMA_B200_LUMA_FLASH_ATTN_HPP_

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

#include "flash_attn.h"

namespace luma_flash_attn {

// 16-bit storage tags; the values are the raw bit patterns the C ABI takes.
struct f16 { uint16_t bits; };
struct bf16 { uint16_t bits; };

// error.rs:7-36
class FlashAttnError : public std::runtime_error {
public:
    enum class Kind { NullPtr, InvalidShape, InvalidHeadSize, InvalidStartPos, BufferTooSmall, Cuda, Unsupported, Unknown };
    FlashAttnError(Kind kind, const std::string& detail, int code = 0)
        : std::runtime_error(display(kind, detail, code)), kind_(kind), detail_(detail), code_(code) {}
    Kind kind() const noexcept { return kind_; }
    const std::string& detail() const noexcept { return detail_; }
    int code() const noexcept { return code_; }

    // error.rs:38-51: status code -> typed error carrying the library's thread-local message
    static void from_status(int status) {
        if (status == FLASH_ATTN_OK) return;
        const char* p = flash_attn_last_error();
        const std::string msg = p ? p : "";   // NULL is treated as "" (error.rs:66-75)
        switch (status) {
            case FLASH_ATTN_ERR_NULL_PTR: throw FlashAttnError(Kind::NullPtr, msg);
            case FLASH_ATTN_ERR_INVALID_SHAPE: throw FlashAttnError(Kind::InvalidShape, msg);
            case FLASH_ATTN_ERR_INVALID_HEAD_SIZE: throw FlashAttnError(Kind::InvalidHeadSize, msg);
            case FLASH_ATTN_ERR_INVALID_START_POS: throw FlashAttnError(Kind::InvalidStartPos, msg);
            case FLASH_ATTN_ERR_CUDA: throw FlashAttnError(Kind::Cuda, msg);
            default: throw FlashAttnError(Kind::Unknown, "", status);
        }
    }

private:
    static std::string display(Kind kind, const std::string& d, int code) {
        switch (kind) {   // the reference's #[error(...)] strings
            case Kind::NullPtr: return "flash_attn: null pointer parameter (" + d + ")";
            case Kind::InvalidShape: return "flash_attn: invalid shape parameter (" + d + ")";
            case Kind::InvalidHeadSize: return "flash_attn: unsupported head_size (" + d + ")";
            case Kind::InvalidStartPos: return "flash_attn: invalid start_pos (" + d + ")";
            case Kind::BufferTooSmall: return "flash_attn: buffer too small (" + d + ")";
            case Kind::Cuda: return "flash_attn: CUDA error (" + d + ")";
            case Kind::Unsupported: return "flash_attn: unsupported (" + d + ")";
            default: return "flash_attn: unknown error code " + std::to_string(code);
        }
    }
    Kind kind_;
    std::string detail_;
    int code_;
};

// A typed view of device memory: pointer + length in elements (what low.rs gets from cudarc).
template <typename T>
struct DeviceSlice {
    T* ptr = nullptr;
    size_t len = 0;
    DeviceSlice() = default;
    DeviceSlice(T* p, size_t n) : ptr(p), len(n) {}
};

// low.rs:14-134 — dtype -> typed C symbols
template <typename T> struct FlashDtype;
template <> struct FlashDtype<float> {
    using raw = float;
    static constexpr auto batch = &flash_attn_f32;
    static constexpr auto varlen = &flash_attn_varlen_f32;
    static constexpr auto kvcache = &flash_attn_with_kvcache_f32;
};
template <> struct FlashDtype<f16> {
    using raw = flash_attn_f16_t;
    static constexpr auto batch = &flash_attn_f16;
    static constexpr auto varlen = &flash_attn_varlen_f16;
    static constexpr auto varlen_total = &flash_attn_varlen_f16_total;
    static constexpr auto kvcache = &flash_attn_with_kvcache_f16;
};
template <> struct FlashDtype<bf16> {
    using raw = flash_attn_bf16_t;
    static constexpr auto batch = &flash_attn_bf16;
    static constexpr auto varlen = &flash_attn_varlen_bf16;
    static constexpr auto varlen_total = &flash_attn_varlen_bf16_total;
    static constexpr auto kvcache = &flash_attn_with_kvcache_bf16;
};

namespace low {

// low.rs:409-416
inline void check_len(const char* name, size_t actual, uint64_t need) {
    if (static_cast<uint64_t>(actual) >= need) return;
    throw FlashAttnError(FlashAttnError::Kind::BufferTooSmall,
                         std::string(name) + ": need at least " + std::to_string(need) + " elements, got " +
                             std::to_string(actual));
}

// low.rs:360-407 — same order: shape, GQA, start_pos, head size, then buffer lengths
template <typename T>
void validate(const DeviceSlice<const T>& q, const DeviceSlice<const T>& k, const DeviceSlice<const T>& v,
              const DeviceSlice<T>& o, int batch, int q_seq_len, int kv_seq_len, int q_num_heads, int kv_num_heads,
              int head_size, int start_pos, const DeviceSlice<const uint8_t>* attn_mask) {
    using K = FlashAttnError::Kind;
    if (batch <= 0 || q_seq_len <= 0 || kv_seq_len <= 0 || q_num_heads <= 0 || kv_num_heads <= 0) {
        throw FlashAttnError(K::InvalidShape,
                             "batch=" + std::to_string(batch) + " q_seq_len=" + std::to_string(q_seq_len) +
                                 " kv_seq_len=" + std::to_string(kv_seq_len) + " q_num_heads=" + std::to_string(q_num_heads) +
                                 " kv_num_heads=" + std::to_string(kv_num_heads) + " must be positive");
    }
    if (q_num_heads % kv_num_heads != 0) {
        throw FlashAttnError(K::InvalidShape, "q_num_heads=" + std::to_string(q_num_heads) +
                                                  " must be a multiple of kv_num_heads=" + std::to_string(kv_num_heads) + " (GQA)");
    }
    if (start_pos < 0) throw FlashAttnError(K::InvalidStartPos, "start_pos=" + std::to_string(start_pos));
    if (head_size != 32 && head_size != 64 && head_size != 128) {
        throw FlashAttnError(K::InvalidHeadSize, "head_size=" + std::to_string(head_size) + " (only 32/64/128)");
    }
    const uint64_t d = static_cast<uint64_t>(head_size);
    const uint64_t q_need = static_cast<uint64_t>(batch) * q_seq_len * q_num_heads * d;
    const uint64_t kv_need = static_cast<uint64_t>(batch) * kv_seq_len * kv_num_heads * d;
    check_len("q", q.len, q_need);
    check_len("k", k.len, kv_need);
    check_len("v", v.len, kv_need);
    check_len("o", o.len, q_need);
    if (attn_mask != nullptr) check_len("attn_mask", attn_mask->len, static_cast<uint64_t>(batch) * kv_seq_len);
}

// low.rs:146-197. q/o (batch, q_seq_len, q_num_heads, head_size); k/v (batch, kv_seq_len,
// kv_num_heads, head_size); attn_mask (batch, kv_seq_len) or null. Asynchronous on `stream`.
template <typename T>
void flash_attn(const DeviceSlice<const T>& q, const DeviceSlice<const T>& k, const DeviceSlice<const T>& v,
                DeviceSlice<T>& o, int batch, int q_seq_len, int kv_seq_len, int q_num_heads, int kv_num_heads,
                int head_size, int start_pos, float scale, const DeviceSlice<const uint8_t>* attn_mask, void* stream) {
    validate<T>(q, k, v, o, batch, q_seq_len, kv_seq_len, q_num_heads, kv_num_heads, head_size, start_pos, attn_mask);
    using R = typename FlashDtype<T>::raw;
    const int code = FlashDtype<T>::batch(reinterpret_cast<const R*>(q.ptr), reinterpret_cast<const R*>(k.ptr),
                                          reinterpret_cast<const R*>(v.ptr), reinterpret_cast<R*>(o.ptr), batch, q_seq_len,
                                          kv_seq_len, q_num_heads, kv_num_heads, head_size, start_pos, scale,
                                          attn_mask ? attn_mask->ptr : nullptr, stream);
    FlashAttnError::from_status(code);
}

// low.rs:199-218 — the historical f32 alias
inline void flash_attn_f32(const DeviceSlice<const float>& q, const DeviceSlice<const float>& k,
                           const DeviceSlice<const float>& v, DeviceSlice<float>& o, int batch, int q_seq_len,
                           int kv_seq_len, int q_num_heads, int kv_num_heads, int head_size, int start_pos, float scale,
                           const DeviceSlice<const uint8_t>* attn_mask, void* stream) {
    flash_attn<float>(q, k, v, o, batch, q_seq_len, kv_seq_len, q_num_heads, kv_num_heads, head_size, start_pos, scale,
                      attn_mask, stream);
}

// low.rs:231-295. block_tables == nullptr: contiguous K/V (total_kv, kv_heads, head_size); otherwise a
// paged cache addressed by block_tables (num_seqs, max_blocks), max_blocks = len / num_seqs.
template <typename T>
void flash_attn_varlen(const DeviceSlice<const T>& q, const DeviceSlice<const T>& k, const DeviceSlice<const T>& v,
                       DeviceSlice<T>& o, const DeviceSlice<const int>& cu_seqlens_q,
                       const DeviceSlice<const int>& cu_seqlens_k, int num_seqs, int max_seqlen_q, int max_seqlen_k,
                       int q_heads, int kv_heads, int head_size, float scale, const DeviceSlice<const int>* block_tables,
                       int block_size, void* stream) {
    using R = typename FlashDtype<T>::raw;
    const int k_paged = block_tables != nullptr ? 1 : 0;
    const int max_blocks = (block_tables != nullptr && num_seqs > 0) ? static_cast<int>(block_tables->len / num_seqs) : 0;
    const int code = FlashDtype<T>::varlen(
        reinterpret_cast<const R*>(q.ptr), reinterpret_cast<const R*>(k.ptr), reinterpret_cast<const R*>(v.ptr),
        reinterpret_cast<R*>(o.ptr), cu_seqlens_q.ptr, cu_seqlens_k.ptr, block_tables ? block_tables->ptr : nullptr, num_seqs,
        max_seqlen_q, max_seqlen_k, q_heads, kv_heads, head_size, block_size, max_blocks, k_paged, scale, stream);
    FlashAttnError::from_status(code);
}

// Additive (16-bit storage only): the same call with the row counts of the packed buffers, which the
// caller knows from its tensor shapes (high.rs:170-182) and a slice length does not tell (a slice
// may be longer than the packed data). With them head_size-128 calls run on the tensor-core kernel.
template <typename T>
void flash_attn_varlen_total(const DeviceSlice<const T>& q, const DeviceSlice<const T>& k, const DeviceSlice<const T>& v,
                             DeviceSlice<T>& o, const DeviceSlice<const int>& cu_seqlens_q,
                             const DeviceSlice<const int>& cu_seqlens_k, int num_seqs, int max_seqlen_q, int max_seqlen_k,
                             int q_heads, int kv_heads, int head_size, float scale, const DeviceSlice<const int>* block_tables,
                             int block_size, int total_q, int total_k, void* stream) {
    using R = typename FlashDtype<T>::raw;
    if (total_q > 0 && q_heads > 0 && head_size > 0) {
        const uint64_t q_need = static_cast<uint64_t>(total_q) * q_heads * head_size;
        check_len("q", q.len, q_need);
        check_len("o", o.len, q_need);
    }
    if (total_k > 0 && block_tables == nullptr && kv_heads > 0 && head_size > 0) {
        const uint64_t kv_need = static_cast<uint64_t>(total_k) * kv_heads * head_size;
        check_len("k", k.len, kv_need);
        check_len("v", v.len, kv_need);
    }
    const int k_paged = block_tables != nullptr ? 1 : 0;
    const int max_blocks = (block_tables != nullptr && num_seqs > 0) ? static_cast<int>(block_tables->len / num_seqs) : 0;
    const int code = FlashDtype<T>::varlen_total(
        reinterpret_cast<const R*>(q.ptr), reinterpret_cast<const R*>(k.ptr), reinterpret_cast<const R*>(v.ptr),
        reinterpret_cast<R*>(o.ptr), cu_seqlens_q.ptr, cu_seqlens_k.ptr, block_tables ? block_tables->ptr : nullptr, num_seqs,
        max_seqlen_q, max_seqlen_k, q_heads, kv_heads, head_size, block_size, max_blocks, k_paged, scale, total_q, total_k,
        stream);
    FlashAttnError::from_status(code);
}

// low.rs:305-357. q/o (num_seqs, q_seq_len, q_heads, head_size); q_seq_len == 1 decodes.
template <typename T>
void flash_attn_with_kvcache(const DeviceSlice<const T>& q, const DeviceSlice<const T>& k_cache,
                             const DeviceSlice<const T>& v_cache, DeviceSlice<T>& o,
                             const DeviceSlice<const int>& block_tables, const DeviceSlice<const int>& context_lens,
                             int num_seqs, int q_seq_len, int q_heads, int kv_heads, int head_size, int block_size,
                             int max_blocks, float scale, void* stream) {
    if (q_seq_len <= 0) {
        throw FlashAttnError(FlashAttnError::Kind::InvalidShape, "q_seq_len=" + std::to_string(q_seq_len) + " must be > 0");
    }
    const uint64_t q_need = static_cast<uint64_t>(num_seqs) * q_seq_len * q_heads * head_size;
    check_len("q", q.len, q_need);
    check_len("o", o.len, q_need);
    using R = typename FlashDtype<T>::raw;
    const int code = FlashDtype<T>::kvcache(
        reinterpret_cast<const R*>(q.ptr), reinterpret_cast<const R*>(k_cache.ptr), reinterpret_cast<const R*>(v_cache.ptr),
        reinterpret_cast<R*>(o.ptr), block_tables.ptr, context_lens.ptr, num_seqs, q_seq_len, q_heads, kv_heads, head_size,
        block_size, max_blocks, scale, stream);
    FlashAttnError::from_status(code);
}

}  // namespace low
}  // namespace luma_flash_attn

#endif  // LUMA_B200_LUMA_FLASH_ATTN_HPP_
