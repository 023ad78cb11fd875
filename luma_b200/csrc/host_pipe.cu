// flash_attn_host_<T>: batched causal attention for tensors that live in HOST memory. This library's
// addition (luma's callers hold device tensors; see luma-flash-attn/src/api/high.rs:157-290 for the
// device-tensor call this wraps).
//
// The work is cut into steps of one batch element and a chunk of query rows — a chunked prefill: the
// rows of a chunk see the keys up to their own position, so a chunk needs only the K/V rows up to its
// end, which travel with it — and the steps are pipelined over three streams of the device: while one
// chunk is in the kernel, the next chunk's q rows and K/V rows are on their way in and the previous
// chunk's result on its way out, which keeps both directions of the host link busy. Staging buffers
// (two row slots, two K/V slots), the streams and the events are kept per device and shape and
// reused by later calls; flash_attn_release_workspaces frees them.
#include <algorithm>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace fa {

namespace {

struct Step {
    int elem, r0, r1;
    int kv_end;   // K/V rows [0, kv_end) of the element are on the device (or on their way) when the step runs, before start_pos is added
};

// Query rows per pipeline step: half of the sequence in whole 128-row tiles (sequences below 4096
// rows go in one step per batch element). Measured on the B=2, S=8192, Hq=32, Hkv=8 call: steps of
// 1024 / 2048 / 4096 / 8192 rows took 6.67 / 6.53 / 6.31 / 6.31 ms on a box whose link moves the same
// bytes in 5.72 ms as plain copies.
int auto_chunk_rows(int sq) {
    if (sq < 4096) return sq;
    return ((sq + 1) / 2 + 127) / 128 * 128;
}

// Cuts [r0, r1) of one batch element into pieces of the given shares (whole 128-row tiles, the rest
// goes to the last piece). kv_whole: the K/V rows of the whole range travel with the first piece, in
// one copy each, instead of piece by piece.
void cut(std::vector<Step>& out, const Step& s, const std::vector<double>& parts, bool kv_whole) {
    const int n = s.r1 - s.r0;
    int at = s.r0;
    for (double frac : parts) {
        const int size = std::max(128, (int)(n * frac) / 128 * 128);
        const int end = std::min(s.r1, at + size);
        if (end > at) out.push_back({s.elem, at, end, kv_whole ? s.r1 : end});
        at = end;
    }
    if (at < s.r1) out.push_back({s.elem, at, s.r1, s.r1});
}

// The steps of one call. Every step is `rows` query rows of one batch element, except that the very
// first step and the very last one are cut into smaller pieces: the link idles while the first chunk
// travels in before any kernel can run, and again while the last result travels back after the last
// kernel, so those two are made short.
std::vector<Step> make_steps(int batch, int sq, int rows) {
    std::vector<Step> steps;
    for (int i = 0; i < batch; ++i)
        for (int r0 = 0; r0 < sq; r0 += rows) steps.push_back({i, r0, std::min(sq, r0 + rows), std::min(sq, r0 + rows)});
    if (rows < 1024 || steps.empty()) return steps;
    std::vector<Step> out;
    if (steps.size() == 1) {
        cut(out, steps[0], {0.0625, 0.0625, 0.125, 0.25, 0.25, 0.125, 0.0625, 0.0625}, false);
        return out;
    }
    // only the first chunk's K/V rows travel piece by piece (the first kernel waits for them); a copy
    // that starts while the other direction is busy pays a start-up gap, so later ones are few and large
    cut(out, steps.front(), {0.0625, 0.0625, 0.125, 0.25, 0.5}, false);
    out.insert(out.end(), steps.begin() + 1, steps.end() - 1);
    cut(out, steps.back(), {0.5, 0.25, 0.125, 0.0625, 0.0625}, true);
    return out;
}

struct RowSlot {
    void* q = nullptr;
    void* o = nullptr;
    cudaEvent_t arrived = nullptr, ran = nullptr, out = nullptr;
    bool ran_set = false, out_set = false;
};

struct KvSlot {
    void* k = nullptr;
    void* v = nullptr;
    cudaEvent_t ran = nullptr;
    bool ran_set = false;
};

struct HostPipe {
    int device = -1;
    cudaStream_t s_in = nullptr, s_run = nullptr, s_out = nullptr;   // rows in, kernels, results out
    cudaEvent_t start = nullptr;
    size_t row_bytes = 0, kv_bytes = 0;   // capacity of each slot
    RowSlot rows[2];
    KvSlot kv[2];
    std::mutex mutex;                      // one call at a time per device
};

std::mutex g_pipes_mutex;
std::vector<HostPipe*> g_pipes;

#define FA_HOST_CHECK(expr)                                                               \
    do {                                                                                  \
        const cudaError_t e_ = (expr);                                                    \
        if (e_ != cudaSuccess) {                                                          \
            set_last_errorf("flash_attn_host: %s failed: %s", #expr, cudaGetErrorString(e_)); \
            return FLASH_ATTN_ERR_CUDA;                                                   \
        }                                                                                 \
    } while (0)

void free_buffers(HostPipe& p) {
    for (RowSlot& r : p.rows) {
        if (r.q) cudaFree(r.q);
        if (r.o) cudaFree(r.o);
        r.q = r.o = nullptr;
        r.ran_set = r.out_set = false;
    }
    for (KvSlot& s : p.kv) {
        if (s.k) cudaFree(s.k);
        if (s.v) cudaFree(s.v);
        s.k = s.v = nullptr;
        s.ran_set = false;
    }
    p.row_bytes = p.kv_bytes = 0;
}

HostPipe* pipe_of(int device) {
    std::lock_guard<std::mutex> lock(g_pipes_mutex);
    for (HostPipe* p : g_pipes)
        if (p->device == device) return p;
    HostPipe* p = new HostPipe();
    p->device = device;
    g_pipes.push_back(p);
    return p;
}

int ensure(HostPipe& p, size_t row_bytes, size_t kv_bytes) {
    if (p.s_in == nullptr) {
        FA_HOST_CHECK(cudaStreamCreateWithFlags(&p.s_in, cudaStreamNonBlocking));
        FA_HOST_CHECK(cudaStreamCreateWithFlags(&p.s_run, cudaStreamNonBlocking));
        FA_HOST_CHECK(cudaStreamCreateWithFlags(&p.s_out, cudaStreamNonBlocking));
        FA_HOST_CHECK(cudaEventCreateWithFlags(&p.start, cudaEventDisableTiming));
        for (RowSlot& r : p.rows) {
            FA_HOST_CHECK(cudaEventCreateWithFlags(&r.arrived, cudaEventDisableTiming));
            FA_HOST_CHECK(cudaEventCreateWithFlags(&r.ran, cudaEventDisableTiming));
            FA_HOST_CHECK(cudaEventCreateWithFlags(&r.out, cudaEventDisableTiming));
        }
        for (KvSlot& s : p.kv) FA_HOST_CHECK(cudaEventCreateWithFlags(&s.ran, cudaEventDisableTiming));
    }
    if (row_bytes > p.row_bytes || kv_bytes > p.kv_bytes) {
        // the staging buffers grow: everything an earlier call still has in flight must be through first
        FA_HOST_CHECK(cudaStreamSynchronize(p.s_in));
        FA_HOST_CHECK(cudaStreamSynchronize(p.s_run));
        FA_HOST_CHECK(cudaStreamSynchronize(p.s_out));
        const size_t rb = std::max(row_bytes, p.row_bytes), kb = std::max(kv_bytes, p.kv_bytes);
        free_buffers(p);
        for (RowSlot& r : p.rows) {
            FA_HOST_CHECK(cudaMalloc(&r.q, rb));
            FA_HOST_CHECK(cudaMalloc(&r.o, rb));
        }
        for (KvSlot& s : p.kv) {
            FA_HOST_CHECK(cudaMalloc(&s.k, kb));
            FA_HOST_CHECK(cudaMalloc(&s.v, kb));
        }
        p.row_bytes = rb;
        p.kv_bytes = kb;
    }
    return FLASH_ATTN_OK;
}

int call_batch(int dtype, const void* q, const void* k, const void* v, void* o, int q_rows, int kv_rows, int hq, int hkv, int d,
               int start_pos, float scale, cudaStream_t stream) {
    switch (dtype) {
        case DT_F32:
            return flash_attn_f32(static_cast<const float*>(q), static_cast<const float*>(k), static_cast<const float*>(v),
                                  static_cast<float*>(o), 1, q_rows, kv_rows, hq, hkv, d, start_pos, scale, nullptr, stream);
        case DT_F16:
            return flash_attn_f16(static_cast<const flash_attn_f16_t*>(q), static_cast<const flash_attn_f16_t*>(k),
                                  static_cast<const flash_attn_f16_t*>(v), static_cast<flash_attn_f16_t*>(o), 1, q_rows, kv_rows, hq,
                                  hkv, d, start_pos, scale, nullptr, stream);
        default:
            return flash_attn_bf16(static_cast<const flash_attn_bf16_t*>(q), static_cast<const flash_attn_bf16_t*>(k),
                                   static_cast<const flash_attn_bf16_t*>(v), static_cast<flash_attn_bf16_t*>(o), 1, q_rows, kv_rows,
                                   hq, hkv, d, start_pos, scale, nullptr, stream);
    }
}

int host_impl(int dtype, const void* q, const void* k, const void* v, void* o, int batch, int sq, int skv, int hq, int hkv, int d,
              int start_pos, float scale, int device, int chunk_rows, void* stream) {
    set_last_error("");
    if (q == nullptr || k == nullptr || v == nullptr || o == nullptr) {
        set_last_error("flash_attn_host: q/k/v/o must not be null");
        return FLASH_ATTN_ERR_NULL_PTR;
    }
    if (batch <= 0 || sq <= 0 || skv <= 0 || hq <= 0 || hkv <= 0 || hq % hkv != 0) {
        set_last_error("flash_attn_host: shape parameters must be positive, q_num_heads a multiple of kv_num_heads");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    if (start_pos < 0) {
        set_last_error("flash_attn_host: start_pos must be >= 0");
        return FLASH_ATTN_ERR_INVALID_START_POS;
    }
    if (d != 32 && d != 64 && d != 128) {
        set_last_error("flash_attn_host: unsupported head_size (only 32/64/128)");
        return FLASH_ATTN_ERR_INVALID_HEAD_SIZE;
    }
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || device < 0 || device >= n_dev) {
        cudaGetLastError();
        set_last_errorf("flash_attn_host: no CUDA device %d", device);
        return FLASH_ATTN_ERR_CUDA;
    }
    int prev = -1;
    FA_HOST_CHECK(cudaGetDevice(&prev));
    if (prev != device) FA_HOST_CHECK(cudaSetDevice(device));
    struct Restore {
        int prev, device;
        ~Restore() {
            if (prev != device && prev >= 0) cudaSetDevice(prev);
        }
    } restore{prev, device};

    const size_t es = dtype == DT_F32 ? 4 : 2;
    int rows = chunk_rows > 0 ? chunk_rows : auto_chunk_rows(sq);
    rows = std::max(1, std::min(rows, sq));
    const size_t q_row = (size_t)hq * d * es, kv_row = (size_t)hkv * d * es;

    HostPipe& p = *pipe_of(device);
    std::lock_guard<std::mutex> lock(p.mutex);
    int rc = ensure(p, (size_t)rows * q_row, (size_t)skv * kv_row);
    if (rc != FLASH_ATTN_OK) return rc;

    cudaStream_t user = reinterpret_cast<cudaStream_t>(stream);
    FA_HOST_CHECK(cudaEventRecord(p.start, user));
    FA_HOST_CHECK(cudaStreamWaitEvent(p.s_in, p.start, 0));

    const char* qh = static_cast<const char*>(q);
    const char* kh = static_cast<const char*>(k);
    const char* vh = static_cast<const char*>(v);
    char* oh = static_cast<char*>(o);
    int kv_have = 0, cur_elem = -1, n = 0;
    RowSlot* last = nullptr;
    for (const Step& st : make_steps(batch, sq, rows)) {
        KvSlot& kv = p.kv[st.elem & 1];
        if (st.elem != cur_elem) {   // a new batch element: nothing of it is on the device yet, and its K/V buffer must be free
            cur_elem = st.elem;
            kv_have = 0;
            if (kv.ran_set) FA_HOST_CHECK(cudaStreamWaitEvent(p.s_in, kv.ran, 0));
        }
        const int n_rows = st.r1 - st.r0;
        const int kv_need = (int)std::min<long long>(skv, (long long)start_pos + st.r1);   // the chunk's rows see keys < start_pos + r1
        const int kv_send = (int)std::min<long long>(skv, (long long)start_pos + st.kv_end);
        RowSlot& sl = p.rows[n & 1];
        ++n;
        if (sl.ran_set) FA_HOST_CHECK(cudaStreamWaitEvent(p.s_in, sl.ran, 0));   // the slot's q is free once its previous kernel has run
        FA_HOST_CHECK(cudaMemcpyAsync(sl.q, qh + ((size_t)st.elem * sq + st.r0) * q_row, (size_t)n_rows * q_row, cudaMemcpyHostToDevice, p.s_in));
        if (kv_send > kv_have) {
            // (a second inbound stream for the K/V rows was measured: 5.05 against 4.67 ms per call, the copies of
            // the two streams get in each other's way)
            const size_t off = (size_t)kv_have * kv_row, bytes = (size_t)(kv_send - kv_have) * kv_row;
            const size_t src = (size_t)st.elem * skv * kv_row + off;
            FA_HOST_CHECK(cudaMemcpyAsync(static_cast<char*>(kv.k) + off, kh + src, bytes, cudaMemcpyHostToDevice, p.s_in));
            FA_HOST_CHECK(cudaMemcpyAsync(static_cast<char*>(kv.v) + off, vh + src, bytes, cudaMemcpyHostToDevice, p.s_in));
            kv_have = kv_send;
        }
        FA_HOST_CHECK(cudaEventRecord(sl.arrived, p.s_in));
        FA_HOST_CHECK(cudaStreamWaitEvent(p.s_run, sl.arrived, 0));
        if (sl.out_set) FA_HOST_CHECK(cudaStreamWaitEvent(p.s_run, sl.out, 0));   // the slot's o is free once it has been copied back
        if (kv_need > 0) {
            rc = call_batch(dtype, sl.q, kv.k, kv.v, sl.o, n_rows, kv_need, hq, hkv, d, start_pos + st.r0, scale, p.s_run);
            if (rc != FLASH_ATTN_OK) return rc;   // the entry point has set the message
        } else {
            FA_HOST_CHECK(cudaMemsetAsync(sl.o, 0, (size_t)n_rows * q_row, p.s_run));   // no key at all: the rows output zeros
        }
        FA_HOST_CHECK(cudaEventRecord(sl.ran, p.s_run));
        FA_HOST_CHECK(cudaEventRecord(kv.ran, p.s_run));
        sl.ran_set = kv.ran_set = true;
        FA_HOST_CHECK(cudaStreamWaitEvent(p.s_out, sl.ran, 0));
        FA_HOST_CHECK(cudaMemcpyAsync(oh + ((size_t)st.elem * sq + st.r0) * q_row, sl.o, (size_t)n_rows * q_row, cudaMemcpyDeviceToHost, p.s_out));
        FA_HOST_CHECK(cudaEventRecord(sl.out, p.s_out));
        sl.out_set = true;
        last = &sl;
    }
    // the caller's stream continues when the last result has left; the copies to the host are in step
    // order on one stream, so the last one is the last to finish
    if (last != nullptr) FA_HOST_CHECK(cudaStreamWaitEvent(user, last->out, 0));
    note_path("host_pipeline", n);
    return FLASH_ATTN_OK;
}

}  // namespace

int release_host_pipes() {
    std::lock_guard<std::mutex> lock(g_pipes_mutex);
    int n = 0;
    for (HostPipe* p : g_pipes) {
        std::lock_guard<std::mutex> pl(p->mutex);
        if (p->row_bytes == 0 && p->kv_bytes == 0) continue;
        int prev = -1;
        cudaGetDevice(&prev);
        cudaSetDevice(p->device);
        cudaStreamSynchronize(p->s_in);
        cudaStreamSynchronize(p->s_run);
        cudaStreamSynchronize(p->s_out);
        free_buffers(*p);
        if (prev >= 0) cudaSetDevice(prev);
        ++n;
    }
    return n;
}

}  // namespace fa

extern "C" {

int flash_attn_host_f32(const float* q, const float* k, const float* v, float* o, int batch, int q_seq_len, int kv_seq_len,
                        int q_num_heads, int kv_num_heads, int head_size, int start_pos, float scale, int device, int chunk_rows,
                        void* stream) {
    return fa::host_impl(fa::DT_F32, q, k, v, o, batch, q_seq_len, kv_seq_len, q_num_heads, kv_num_heads, head_size, start_pos, scale,
                         device, chunk_rows, stream);
}

int flash_attn_host_f16(const flash_attn_f16_t* q, const flash_attn_f16_t* k, const flash_attn_f16_t* v, flash_attn_f16_t* o, int batch,
                        int q_seq_len, int kv_seq_len, int q_num_heads, int kv_num_heads, int head_size, int start_pos, float scale,
                        int device, int chunk_rows, void* stream) {
    return fa::host_impl(fa::DT_F16, q, k, v, o, batch, q_seq_len, kv_seq_len, q_num_heads, kv_num_heads, head_size, start_pos, scale,
                         device, chunk_rows, stream);
}

int flash_attn_host_bf16(const flash_attn_bf16_t* q, const flash_attn_bf16_t* k, const flash_attn_bf16_t* v, flash_attn_bf16_t* o,
                         int batch, int q_seq_len, int kv_seq_len, int q_num_heads, int kv_num_heads, int head_size, int start_pos,
                         float scale, int device, int chunk_rows, void* stream) {
    return fa::host_impl(fa::DT_BF16, q, k, v, o, batch, q_seq_len, kv_seq_len, q_num_heads, kv_num_heads, head_size, start_pos, scale,
                         device, chunk_rows, stream);
}

int flash_attn_host_steps(int batch, int q_seq_len, int chunk_rows, int* steps_out, int capacity) {
    int rows = chunk_rows > 0 ? chunk_rows : fa::auto_chunk_rows(q_seq_len);
    rows = std::max(1, std::min(rows, std::max(1, q_seq_len)));
    const std::vector<fa::Step> steps = fa::make_steps(batch, q_seq_len, rows);
    for (size_t i = 0; steps_out != nullptr && i < steps.size() && (int)i < capacity; ++i) {
        steps_out[3 * i] = steps[i].elem;
        steps_out[3 * i + 1] = steps[i].r0;
        steps_out[3 * i + 2] = steps[i].r1;
    }
    return (int)steps.size();
}

}  // extern "C"
