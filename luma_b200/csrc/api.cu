// extern "C" entry points of libflash_attn: argument validation in the reference's order with the
// reference's status codes, thread-local last-error string, device selection, and dispatch to the
// kernel families (tcgen05 prefill, split-K paged decode, SIMT tile kernel for everything else).
//
// Validation order and codes follow
//   luma-flash-attn/kernels/flash_attn_func.cu:267-304
//   luma-flash-attn/kernels/flash_attn_varlen_func.cu:243-304
//   luma-flash-attn/kernels/flash_attn_with_kvcache.cu:313-386
#include <atomic>
#include <cstdarg>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace fa {

namespace {
thread_local char g_last_error[256] = {0};
thread_local const char* g_last_path = "";
thread_local int g_last_launches = 0;
// Option knobs: written by flash_attn_set_option on any thread, read by launches on any thread.
std::atomic<int> g_force_generic{0};
std::atomic<int> g_decode_chunk{0};
std::atomic<int> g_prefill_trace{0};
std::atomic<int> g_prefill_trace_y{0};
std::atomic<int> g_prefill_band{0};
std::atomic<int> g_prefill_order{0};
std::atomic<int> g_prefill_groups{0};
std::atomic<int> g_prefill_wait_us{0};
std::atomic<int> g_prefill_test_skip_k{0};
}  // namespace

void set_last_error(const char* msg) { std::snprintf(g_last_error, sizeof(g_last_error), "%s", msg); }

void set_last_errorf(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    std::vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
}

void note_path(const char* name, int launches) {
    g_last_path = name;
    g_last_launches = launches;
}

int get_option_force_generic() { return g_force_generic.load(std::memory_order_relaxed); }
int get_option_decode_chunk() { return g_decode_chunk.load(std::memory_order_relaxed); }
int get_option_prefill_trace() { return g_prefill_trace.load(std::memory_order_relaxed); }
int get_option_prefill_trace_y() { return g_prefill_trace_y.load(std::memory_order_relaxed); }
int get_option_prefill_band() { return g_prefill_band.load(std::memory_order_relaxed); }
int get_option_prefill_groups() { return g_prefill_groups.load(std::memory_order_relaxed); }
int get_option_prefill_order() { return g_prefill_order.load(std::memory_order_relaxed); }
int get_option_prefill_wait_us() { return g_prefill_wait_us.load(std::memory_order_relaxed); }
int get_option_prefill_test_skip_k() { return g_prefill_test_skip_k.load(std::memory_order_relaxed); }

int check_launch(const char* what) {
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) {
        set_last_errorf("%s: %s", what, cudaGetErrorString(err));
        return FLASH_ATTN_ERR_CUDA;
    }
    return FLASH_ATTN_OK;
}

// ---- decode split-K workspace: one buffer per (device, stream) ---------------------------
// Allocation and release are stream-ordered (cudaMallocAsync / cudaFreeAsync on the stream that
// uses the buffer): growing a workspace neither takes a device-wide synchronisation nor frees
// memory under work that still reads it. The table is bounded: beyond kMaxWorkspaces entries the
// least recently used one is released, so a program that keeps creating streams does not keep
// one buffer per stream it ever had (a stream handle that is destroyed and handed out again simply
// finds a scratch buffer that nobody else uses).
namespace {
struct WsEntry {
    int dev = -1;
    cudaStream_t stream = nullptr;
    void* ptr = nullptr;
    size_t bytes = 0;
    unsigned long long last_use = 0;
};
constexpr size_t kMaxWorkspaces = 32;
std::mutex g_ws_mutex;
std::vector<WsEntry> g_ws;
unsigned long long g_ws_clock = 0;

void release_entry(WsEntry& e) {
    if (e.ptr == nullptr) return;
    int cur = -1;
    cudaGetDevice(&cur);
    if (cur != e.dev) cudaSetDevice(e.dev);
    if (cudaFreeAsync(e.ptr, e.stream) != cudaSuccess) {
        cudaGetLastError();   // e.g. the stream is gone: fall back to the synchronising release
        cudaFree(e.ptr);
        cudaGetLastError();
    }
    if (cur != e.dev && cur >= 0) cudaSetDevice(cur);
    e.ptr = nullptr;
    e.bytes = 0;
}
}  // namespace

void* decode_workspace(cudaStream_t stream, size_t bytes) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    WsEntry* e = nullptr;
    for (WsEntry& w : g_ws)
        if (w.dev == dev && w.stream == stream) e = &w;
    if (e == nullptr) {
        if (g_ws.size() >= kMaxWorkspaces) {
            size_t lru = 0;
            for (size_t i = 1; i < g_ws.size(); ++i)
                if (g_ws[i].last_use < g_ws[lru].last_use) lru = i;
            release_entry(g_ws[lru]);
            g_ws.erase(g_ws.begin() + (long)lru);
        }
        g_ws.emplace_back();
        e = &g_ws.back();
        e->dev = dev;
        e->stream = stream;
    }
    e->last_use = ++g_ws_clock;
    if (e->bytes >= bytes && e->ptr != nullptr) return e->ptr;
    release_entry(*e);   // ordered after the work that still reads the old buffer
    size_t want = bytes + bytes / 4;
    if (want < (size_t(1) << 20)) want = size_t(1) << 20;
    void* ptr = nullptr;
    if (cudaMallocAsync(&ptr, want, stream) != cudaSuccess) {
        cudaGetLastError();
        want = bytes;
        if (cudaMallocAsync(&ptr, want, stream) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
    }
    e->ptr = ptr;
    e->bytes = want;
    return ptr;
}

int release_workspaces() {
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    int n = 0;
    for (WsEntry& w : g_ws) {
        if (w.ptr != nullptr) ++n;
        release_entry(w);
    }
    g_ws.clear();
    return n;
}

namespace {

// Makes the device that owns `ptr` current for the lifetime of the guard.
struct DeviceGuard {
    int prev = -1;
    bool switched = false;
    bool ok = true;
    explicit DeviceGuard(const void* ptr) {
        cudaPointerAttributes attr;
        if (cudaPointerGetAttributes(&attr, ptr) != cudaSuccess) {
            cudaGetLastError();
            return;  // not a CUDA pointer we can classify: launch on the current device
        }
        if (attr.type != cudaMemoryTypeDevice && attr.type != cudaMemoryTypeManaged) return;
        if (cudaGetDevice(&prev) != cudaSuccess) {
            ok = false;
            return;
        }
        if (attr.device != prev) {
            ok = cudaSetDevice(attr.device) == cudaSuccess;
            switched = ok;
        }
    }
    ~DeviceGuard() {
        if (switched) cudaSetDevice(prev);
    }
};

bool have_device() {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        set_last_error("flash_attn: no CUDA device available (this library has no CPU fallback)");
        return false;
    }
    return true;
}

// A bounded wait of an earlier tensor-core prefill launch on the current device ran out: that launch
// returned early and its output is undefined. The kernel left the wait's code in a host-mapped
// word; it is reported here — without touching the device — as the failure of the next call, which
// is the first moment the asynchronous ABI can say so (error contract: luma-flash-attn/src/error.rs:38-51).
bool report_earlier_wait_expiry() {
    const int code = prefill_take_status();
    if (code == 0) return true;
    set_last_errorf("flash_attn: a bounded wait (code %d) inside an earlier prefill_tcgen05 launch on this device ran out; "
                    "that launch's output is undefined. This call did not run.", code);
    return false;
}

int dispatch(const AttnParams& p, cudaStream_t stream) {
    if (!have_device()) return FLASH_ATTN_ERR_CUDA;
    DeviceGuard guard(p.q);
    if (!guard.ok) {
        set_last_error("flash_attn: could not select the device that owns q");
        return FLASH_ATTN_ERR_CUDA;
    }
    if (!report_earlier_wait_expiry()) return FLASH_ATTN_ERR_CUDA;
    if (!get_option_force_generic()) {
        int rc = launch_decode_splitk(p, stream);
        if (rc >= 0) return rc;
        rc = launch_prefill_tcgen05(p, stream);
        if (rc >= 0) return rc;
    }
    return launch_tile_simt(p, stream);
}

bool head_size_ok(int h) { return h == 32 || h == 64 || h == 128; }

int batch_impl(int dtype, const void* q, const void* k, const void* v, void* o, float* lse,
               int batch, int q_seq_len, int kv_seq_len, int q_num_heads, int kv_num_heads,
               int head_size, int start_pos, float scale, const uint8_t* attn_mask, void* stream) {
    g_last_error[0] = '\0';
    cudaGetLastError();  // swallow a sticky error left by someone else, as the reference does
    if (q == nullptr || k == nullptr || v == nullptr || o == nullptr) {
        set_last_error("flash_attn: q/k/v/o must not be null");
        return FLASH_ATTN_ERR_NULL_PTR;
    }
    if (batch <= 0 || q_seq_len <= 0 || kv_seq_len <= 0 || q_num_heads <= 0 || kv_num_heads <= 0) {
        set_last_error("flash_attn: shape parameters must be positive");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    if (q_num_heads % kv_num_heads != 0) {
        set_last_error("flash_attn: q_num_heads must be a multiple of kv_num_heads (GQA)");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    if (start_pos < 0) {
        set_last_error("flash_attn: start_pos must be >= 0");
        return FLASH_ATTN_ERR_INVALID_START_POS;
    }
    if (!head_size_ok(head_size)) {
        set_last_error("flash_attn: unsupported head_size (only 32/64/128)");
        return FLASH_ATTN_ERR_INVALID_HEAD_SIZE;
    }
    AttnParams p{};
    p.q = q; p.k = k; p.v = v; p.o = o; p.lse = lse;
    p.mask = attn_mask;
    p.mode = MODE_BATCH;
    p.dtype = dtype;
    p.num_seqs = batch;
    p.q_seq_len = q_seq_len;
    p.kv_seq_len = kv_seq_len;
    p.q_heads = q_num_heads;
    p.kv_heads = kv_num_heads;
    p.head_size = head_size;
    p.start_pos = start_pos;
    p.block_size = 1;
    p.scale = scale;
    return dispatch(p, reinterpret_cast<cudaStream_t>(stream));
}

int varlen_impl(int dtype, const void* q, const void* k, const void* v, void* o,
                const int* cu_seqlens_q, const int* cu_seqlens_k, const int* block_tables,
                int num_seqs, int max_seqlen_q, int max_seqlen_k, int q_heads, int kv_heads,
                int head_size, int block_size, int max_blocks, int k_paged, float scale, void* stream,
                int total_q = 0, int total_k = 0) {
    g_last_error[0] = '\0';
    cudaGetLastError();
    if (q == nullptr || o == nullptr || cu_seqlens_q == nullptr || cu_seqlens_k == nullptr) {
        set_last_error("flash_attn_varlen: q/o/cu_seqlens must not be null");
        return FLASH_ATTN_ERR_NULL_PTR;
    }
    if (k == nullptr || v == nullptr || (k_paged && block_tables == nullptr)) {
        set_last_error("flash_attn_varlen: k/v (and block_tables when paged) must not be null");
        return FLASH_ATTN_ERR_NULL_PTR;
    }
    if (num_seqs <= 0 || q_heads <= 0 || kv_heads <= 0) {
        set_last_error("flash_attn_varlen: num_seqs/q_heads/kv_heads must be > 0");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    if (q_heads % kv_heads != 0) {
        set_last_error("flash_attn_varlen: q_heads must be a multiple of kv_heads (GQA)");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    if (!head_size_ok(head_size)) {
        set_last_error("flash_attn_varlen: head_size must be 32/64/128");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    if (max_seqlen_q <= 0 || max_seqlen_k <= 0 || block_size <= 0) {
        set_last_error("flash_attn_varlen: max_seqlen_q/k and block_size must be > 0");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    AttnParams p{};
    p.q = q; p.k = k; p.v = v; p.o = o;
    p.cu_q = cu_seqlens_q;
    p.cu_k = cu_seqlens_k;
    p.block_tables = k_paged ? block_tables : nullptr;
    p.mode = MODE_VARLEN;
    p.dtype = dtype;
    p.num_seqs = num_seqs;
    p.q_seq_len = max_seqlen_q;
    p.kv_seq_len = max_seqlen_k;
    p.q_heads = q_heads;
    p.kv_heads = kv_heads;
    p.head_size = head_size;
    p.block_size = block_size;
    p.max_blocks = max_blocks;
    p.paged = k_paged ? 1 : 0;
    p.total_q = total_q > 0 ? total_q : 0;
    p.total_k = total_k > 0 ? total_k : 0;
    p.scale = scale;
    return dispatch(p, reinterpret_cast<cudaStream_t>(stream));
}

// Head-sharded prefill whose epilogue writes this rank's heads into the full output tensor of every
// GPU of the group (peer pointers): the all-gather of luma-dist's Comm::all_gather is part of the
// kernel. Only the tcgen05 path implements it.
int allgather_impl(int dtype, const void* q, const void* k, const void* v, void* const* o_peers, int n_peers,
                   int q_heads_total, int q_head_offset, float* lse, int batch, int q_seq_len, int kv_seq_len,
                   int q_num_heads, int kv_num_heads, int head_size, int start_pos, float scale, void* stream,
                   float* const* lse_peers = nullptr, int multicast = 0) {
    g_last_error[0] = '\0';
    cudaGetLastError();
    if (q == nullptr || k == nullptr || v == nullptr || o_peers == nullptr) {
        set_last_error("flash_attn_allgather: q/k/v/o_peers must not be null");
        return FLASH_ATTN_ERR_NULL_PTR;
    }
    if (n_peers < 1 || n_peers > 8) {
        set_last_error("flash_attn_allgather: n_peers must be in 1..8");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    for (int i = 0; i < n_peers; ++i) {
        if (o_peers[i] == nullptr) {
            set_last_error("flash_attn_allgather: every entry of o_peers must be a device pointer");
            return FLASH_ATTN_ERR_NULL_PTR;
        }
    }
    if (batch <= 0 || q_seq_len <= 0 || kv_seq_len <= 0 || q_num_heads <= 0 || kv_num_heads <= 0) {
        set_last_error("flash_attn_allgather: shape parameters must be positive");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    if (q_num_heads % kv_num_heads != 0) {
        set_last_error("flash_attn_allgather: q_num_heads must be a multiple of kv_num_heads (GQA)");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    if (q_head_offset < 0 || q_heads_total <= 0 || q_head_offset + q_num_heads > q_heads_total) {
        set_last_error("flash_attn_allgather: q_head_offset + q_num_heads must lie inside q_heads_total");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    if (start_pos < 0) {
        set_last_error("flash_attn_allgather: start_pos must be >= 0");
        return FLASH_ATTN_ERR_INVALID_START_POS;
    }
    if (head_size != 64 && head_size != 128) {
        set_last_error("flash_attn_allgather: the fused path takes head_size 64 or 128");
        return FLASH_ATTN_ERR_INVALID_HEAD_SIZE;
    }
    if (lse_peers != nullptr) {
        for (int i = 0; i < n_peers; ++i) {
            if (lse_peers[i] == nullptr) {
                set_last_error("flash_attn_allgather: every entry of lse_peers must be a device pointer");
                return FLASH_ATTN_ERR_NULL_PTR;
            }
        }
    }
    AttnParams p{};
    p.q = q; p.k = k; p.v = v; p.o = o_peers[0]; p.lse = lse;
    p.mode = MODE_BATCH;
    p.dtype = dtype;
    p.num_seqs = batch;
    p.q_seq_len = q_seq_len;
    p.kv_seq_len = kv_seq_len;
    p.q_heads = q_num_heads;
    p.kv_heads = kv_num_heads;
    p.head_size = head_size;
    p.start_pos = start_pos;
    p.block_size = 1;
    p.scale = scale;
    for (int i = 0; i < n_peers; ++i) p.o_peers[i] = o_peers[i];
    p.n_out = n_peers;
    p.multicast = multicast;
    p.o_heads = q_heads_total;
    p.o_head0 = q_head_offset;
    if (lse_peers != nullptr) {
        for (int i = 0; i < n_peers; ++i) p.lse_peers[i] = lse_peers[i];
        p.n_lse = n_peers;
    }
    if (!have_device()) return FLASH_ATTN_ERR_CUDA;
    DeviceGuard guard(q);
    if (!guard.ok) {
        set_last_error("flash_attn_allgather: could not select the device that owns q");
        return FLASH_ATTN_ERR_CUDA;
    }
    if (!report_earlier_wait_expiry()) return FLASH_ATTN_ERR_CUDA;
    const int rc = launch_prefill_tcgen05(p, reinterpret_cast<cudaStream_t>(stream));
    if (rc < 0) {
        set_last_error("flash_attn_allgather: this shape is outside the fused tensor-core path (needs f16/bf16, head_size 64 or 128, "
                       "scale > 0, 16-byte aligned buffers)");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    return rc;
}

int kvcache_impl(int dtype, const void* q, const void* k_cache, const void* v_cache, void* o,
                 const int* block_tables, const int* context_lens, int num_seqs, int q_seq_len,
                 int q_heads, int kv_heads, int head_size, int block_size, int max_blocks,
                 float scale, void* stream, void* const* o_peers = nullptr, int n_peers = 0,
                 int q_heads_total = 0, int q_head_offset = 0) {
    g_last_error[0] = '\0';
    cudaGetLastError();
    if (q == nullptr || k_cache == nullptr || v_cache == nullptr || (o == nullptr && o_peers == nullptr) ||
        block_tables == nullptr || context_lens == nullptr) {
        set_last_error("flash_attn_with_kvcache: null pointer argument");
        return FLASH_ATTN_ERR_NULL_PTR;
    }
    if (num_seqs <= 0 || q_heads <= 0 || kv_heads <= 0) {
        set_last_error("flash_attn_with_kvcache: num_seqs/q_heads/kv_heads must be > 0");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    if (q_heads % kv_heads != 0) {
        set_last_error("flash_attn_with_kvcache: q_heads must be a multiple of kv_heads (GQA)");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    if (!head_size_ok(head_size)) {
        set_last_error("flash_attn_with_kvcache: head_size must be 32/64/128");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    if (q_seq_len <= 0) {
        set_last_error("flash_attn_with_kvcache: q_seq_len must be > 0");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    if (block_size <= 0) {
        set_last_error("flash_attn_with_kvcache: block_size must be > 0");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    AttnParams p{};
    p.q = q; p.k = k_cache; p.v = v_cache; p.o = o;
    p.block_tables = block_tables;
    p.context_lens = context_lens;
    p.mode = MODE_KVCACHE;
    p.dtype = dtype;
    p.num_seqs = num_seqs;
    p.q_seq_len = q_seq_len;
    p.kv_seq_len = (max_blocks > 0 && (long long)max_blocks * block_size < 0x7fffffffLL)
                       ? max_blocks * block_size : 0x7fffffff;
    p.q_heads = q_heads;
    p.kv_heads = kv_heads;
    p.head_size = head_size;
    p.block_size = block_size;
    p.max_blocks = max_blocks;
    p.paged = 1;
    p.scale = scale;
    if (o_peers != nullptr) {
        // head-sharded single-token decode with the output all-gather fused into the merge kernel
        if (n_peers < 1 || n_peers > 8 || q_head_offset < 0 || q_heads_total <= 0 || q_head_offset + q_heads > q_heads_total) {
            set_last_error("flash_attn_with_kvcache_allgather: n_peers must be in 1..8 and q_head_offset + q_heads inside q_heads_total");
            return FLASH_ATTN_ERR_INVALID_SHAPE;
        }
        for (int i = 0; i < n_peers; ++i) {
            if (o_peers[i] == nullptr) {
                set_last_error("flash_attn_with_kvcache_allgather: every entry of o_peers must be a device pointer");
                return FLASH_ATTN_ERR_NULL_PTR;
            }
            p.o_peers[i] = o_peers[i];
        }
        p.n_out = n_peers;
        p.o_heads = q_heads_total;
        p.o_head0 = q_head_offset;
        if (!have_device()) return FLASH_ATTN_ERR_CUDA;
        DeviceGuard guard(q);
        if (!guard.ok) {
            set_last_error("flash_attn_with_kvcache_allgather: could not select the device that owns q");
            return FLASH_ATTN_ERR_CUDA;
        }
        const int rc = launch_decode_splitk(p, reinterpret_cast<cudaStream_t>(stream));
        if (rc < 0) {
            set_last_error("flash_attn_with_kvcache_allgather: outside the split-K decode path (needs q_seq_len 1, f16/bf16, "
                           "head_size 64 or 128, 16-byte aligned caches)");
            return FLASH_ATTN_ERR_INVALID_SHAPE;
        }
        return rc;
    }
    return dispatch(p, reinterpret_cast<cudaStream_t>(stream));
}

}  // namespace
}  // namespace fa

extern "C" {

const char* flash_attn_last_error(void) { return fa::g_last_error; }
const char* flash_attn_version(void) { return "luma-b200-flash-attn 0.1.0 (sm_100a)"; }
const char* flash_attn_last_path(void) { return fa::g_last_path; }
int flash_attn_last_launches(void) { return fa::g_last_launches; }

int flash_attn_device_status(void) {
    if (!fa::have_device()) return -1;
    return fa::prefill_device_status();
}

int flash_attn_debug_read(void* dst, int bytes) {
    if (!fa::have_device()) return -1;
    return fa::prefill_debug_read(dst, bytes);
}

int flash_attn_release_workspaces(void) { return fa::release_workspaces() + fa::release_host_pipes(); }

int flash_attn_debug_launch_rank(int grid_row, int first_wave_rows, int stride) {
    return fa::launch_rank(grid_row, first_wave_rows, stride);
}

int flash_attn_set_option(const char* name, int value) {
    if (name == nullptr) return 1;
    if (std::strcmp(name, "force_generic") == 0) {
        fa::g_force_generic = value;
        return 0;
    }
    if (std::strcmp(name, "prefill_trace") == 0) {
        fa::g_prefill_trace = value;
        return 0;
    }
    if (std::strcmp(name, "prefill_groups") == 0) {
        fa::g_prefill_groups = value;
        return 0;
    }
    if (std::strcmp(name, "prefill_order") == 0) {
        fa::g_prefill_order = value;
        return 0;
    }
    if (std::strcmp(name, "prefill_band") == 0) {
        fa::g_prefill_band = value;
        return 0;
    }
    if (std::strcmp(name, "prefill_trace_y") == 0) {
        fa::g_prefill_trace_y = value;
        return 0;
    }
    if (std::strcmp(name, "decode_chunk_tokens") == 0) {
        fa::g_decode_chunk = value;
        return 0;
    }
    if (std::strcmp(name, "prefill_wait_us") == 0) {
        fa::g_prefill_wait_us = value;
        return 0;
    }
    if (std::strcmp(name, "prefill_test_skip_k") == 0) {
        fa::g_prefill_test_skip_k = value;
        return 0;
    }
    return 1;
}

#define FA_DEFINE_BATCH(NAME, CTYPE, DT)                                                            \
    int NAME(const CTYPE* q, const CTYPE* k, const CTYPE* v, CTYPE* o, int batch, int q_seq_len,    \
             int kv_seq_len, int q_num_heads, int kv_num_heads, int head_size, int start_pos,       \
             float scale, const uint8_t* attn_mask, void* stream) {                                 \
        return fa::batch_impl(DT, q, k, v, o, nullptr, batch, q_seq_len, kv_seq_len, q_num_heads,   \
                              kv_num_heads, head_size, start_pos, scale, attn_mask, stream);        \
    }                                                                                               \
    int NAME##_lse(const CTYPE* q, const CTYPE* k, const CTYPE* v, CTYPE* o, float* lse, int batch, \
                   int q_seq_len, int kv_seq_len, int q_num_heads, int kv_num_heads, int head_size, \
                   int start_pos, float scale, const uint8_t* attn_mask, void* stream) {            \
        return fa::batch_impl(DT, q, k, v, o, lse, batch, q_seq_len, kv_seq_len, q_num_heads,       \
                              kv_num_heads, head_size, start_pos, scale, attn_mask, stream);        \
    }

FA_DEFINE_BATCH(flash_attn_f32, float, fa::DT_F32)
FA_DEFINE_BATCH(flash_attn_f16, flash_attn_f16_t, fa::DT_F16)
FA_DEFINE_BATCH(flash_attn_bf16, flash_attn_bf16_t, fa::DT_BF16)
#undef FA_DEFINE_BATCH

#define FA_DEFINE_VARLEN(NAME, CTYPE, DT)                                                           \
    int NAME(const CTYPE* q, const CTYPE* k, const CTYPE* v, CTYPE* o, const int* cu_seqlens_q,     \
             const int* cu_seqlens_k, const int* block_tables, int num_seqs, int max_seqlen_q,      \
             int max_seqlen_k, int q_heads, int kv_heads, int head_size, int block_size,            \
             int max_blocks, int k_paged, float scale, void* stream) {                              \
        return fa::varlen_impl(DT, q, k, v, o, cu_seqlens_q, cu_seqlens_k, block_tables, num_seqs,  \
                               max_seqlen_q, max_seqlen_k, q_heads, kv_heads, head_size,            \
                               block_size, max_blocks, k_paged, scale, stream);                     \
    }

FA_DEFINE_VARLEN(flash_attn_varlen_f32, float, fa::DT_F32)
FA_DEFINE_VARLEN(flash_attn_varlen_f16, flash_attn_f16_t, fa::DT_F16)
FA_DEFINE_VARLEN(flash_attn_varlen_bf16, flash_attn_bf16_t, fa::DT_BF16)
#undef FA_DEFINE_VARLEN

int flash_attn_varlen_f16_total(const flash_attn_f16_t* q, const flash_attn_f16_t* k, const flash_attn_f16_t* v,
                                flash_attn_f16_t* o, const int* cu_seqlens_q, const int* cu_seqlens_k,
                                const int* block_tables, int num_seqs, int max_seqlen_q, int max_seqlen_k, int q_heads,
                                int kv_heads, int head_size, int block_size, int max_blocks, int k_paged, float scale,
                                int total_q, int total_k, void* stream) {
    return fa::varlen_impl(fa::DT_F16, q, k, v, o, cu_seqlens_q, cu_seqlens_k, block_tables, num_seqs, max_seqlen_q,
                           max_seqlen_k, q_heads, kv_heads, head_size, block_size, max_blocks, k_paged, scale, stream,
                           total_q, total_k);
}
int flash_attn_varlen_bf16_total(const flash_attn_bf16_t* q, const flash_attn_bf16_t* k, const flash_attn_bf16_t* v,
                                 flash_attn_bf16_t* o, const int* cu_seqlens_q, const int* cu_seqlens_k,
                                 const int* block_tables, int num_seqs, int max_seqlen_q, int max_seqlen_k, int q_heads,
                                 int kv_heads, int head_size, int block_size, int max_blocks, int k_paged, float scale,
                                 int total_q, int total_k, void* stream) {
    return fa::varlen_impl(fa::DT_BF16, q, k, v, o, cu_seqlens_q, cu_seqlens_k, block_tables, num_seqs, max_seqlen_q,
                           max_seqlen_k, q_heads, kv_heads, head_size, block_size, max_blocks, k_paged, scale, stream,
                           total_q, total_k);
}

#define FA_DEFINE_KVCACHE(NAME, CTYPE, DT)                                                          \
    int NAME(const CTYPE* q, const CTYPE* k_cache, const CTYPE* v_cache, CTYPE* o,                  \
             const int* block_tables, const int* context_lens, int num_seqs, int q_seq_len,         \
             int q_heads, int kv_heads, int head_size, int block_size, int max_blocks, float scale, \
             void* stream) {                                                                        \
        return fa::kvcache_impl(DT, q, k_cache, v_cache, o, block_tables, context_lens, num_seqs,   \
                                q_seq_len, q_heads, kv_heads, head_size, block_size, max_blocks,    \
                                scale, stream);                                                     \
    }

FA_DEFINE_KVCACHE(flash_attn_with_kvcache_f32, float, fa::DT_F32)
FA_DEFINE_KVCACHE(flash_attn_with_kvcache_f16, flash_attn_f16_t, fa::DT_F16)
FA_DEFINE_KVCACHE(flash_attn_with_kvcache_bf16, flash_attn_bf16_t, fa::DT_BF16)
#undef FA_DEFINE_KVCACHE

int flash_attn_f16_allgather(const flash_attn_f16_t* q, const flash_attn_f16_t* k, const flash_attn_f16_t* v,
                             void* const* o_peers, int n_peers, int q_heads_total, int q_head_offset, float* lse,
                             int batch, int q_seq_len, int kv_seq_len, int q_num_heads, int kv_num_heads, int head_size,
                             int start_pos, float scale, void* stream) {
    return fa::allgather_impl(fa::DT_F16, q, k, v, o_peers, n_peers, q_heads_total, q_head_offset, lse, batch, q_seq_len,
                              kv_seq_len, q_num_heads, kv_num_heads, head_size, start_pos, scale, stream);
}
int flash_attn_bf16_allgather(const flash_attn_bf16_t* q, const flash_attn_bf16_t* k, const flash_attn_bf16_t* v,
                              void* const* o_peers, int n_peers, int q_heads_total, int q_head_offset, float* lse,
                              int batch, int q_seq_len, int kv_seq_len, int q_num_heads, int kv_num_heads, int head_size,
                              int start_pos, float scale, void* stream) {
    return fa::allgather_impl(fa::DT_BF16, q, k, v, o_peers, n_peers, q_heads_total, q_head_offset, lse, batch, q_seq_len,
                              kv_seq_len, q_num_heads, kv_num_heads, head_size, start_pos, scale, stream);
}

int flash_attn_f16_allgather_lse(const flash_attn_f16_t* q, const flash_attn_f16_t* k, const flash_attn_f16_t* v,
                                 void* const* o_peers, float* const* lse_peers, int n_peers, int q_heads_total,
                                 int q_head_offset, int batch, int q_seq_len, int kv_seq_len, int q_num_heads,
                                 int kv_num_heads, int head_size, int start_pos, float scale, void* stream) {
    return fa::allgather_impl(fa::DT_F16, q, k, v, o_peers, n_peers, q_heads_total, q_head_offset, nullptr, batch, q_seq_len,
                              kv_seq_len, q_num_heads, kv_num_heads, head_size, start_pos, scale, stream, lse_peers);
}
int flash_attn_bf16_allgather_lse(const flash_attn_bf16_t* q, const flash_attn_bf16_t* k, const flash_attn_bf16_t* v,
                                  void* const* o_peers, float* const* lse_peers, int n_peers, int q_heads_total,
                                  int q_head_offset, int batch, int q_seq_len, int kv_seq_len, int q_num_heads,
                                  int kv_num_heads, int head_size, int start_pos, float scale, void* stream) {
    return fa::allgather_impl(fa::DT_BF16, q, k, v, o_peers, n_peers, q_heads_total, q_head_offset, nullptr, batch, q_seq_len,
                              kv_seq_len, q_num_heads, kv_num_heads, head_size, start_pos, scale, stream, lse_peers);
}

int flash_attn_f16_allgather_multicast(const flash_attn_f16_t* q, const flash_attn_f16_t* k, const flash_attn_f16_t* v,
                                       void* o_multicast, int q_heads_total, int q_head_offset, float* lse, int batch,
                                       int q_seq_len, int kv_seq_len, int q_num_heads, int kv_num_heads, int head_size,
                                       int start_pos, float scale, void* stream) {
    void* one[1] = {o_multicast};
    return fa::allgather_impl(fa::DT_F16, q, k, v, o_multicast != nullptr ? one : nullptr, 1, q_heads_total, q_head_offset, lse,
                              batch, q_seq_len, kv_seq_len, q_num_heads, kv_num_heads, head_size, start_pos, scale, stream,
                              nullptr, 1);
}
int flash_attn_bf16_allgather_multicast(const flash_attn_bf16_t* q, const flash_attn_bf16_t* k, const flash_attn_bf16_t* v,
                                        void* o_multicast, int q_heads_total, int q_head_offset, float* lse, int batch,
                                        int q_seq_len, int kv_seq_len, int q_num_heads, int kv_num_heads, int head_size,
                                        int start_pos, float scale, void* stream) {
    void* one[1] = {o_multicast};
    return fa::allgather_impl(fa::DT_BF16, q, k, v, o_multicast != nullptr ? one : nullptr, 1, q_heads_total, q_head_offset, lse,
                              batch, q_seq_len, kv_seq_len, q_num_heads, kv_num_heads, head_size, start_pos, scale, stream,
                              nullptr, 1);
}

int flash_attn_with_kvcache_f16_allgather(const flash_attn_f16_t* q, const flash_attn_f16_t* k_cache,
                                          const flash_attn_f16_t* v_cache, void* const* o_peers, int n_peers,
                                          int q_heads_total, int q_head_offset, const int* block_tables,
                                          const int* context_lens, int num_seqs, int q_heads, int kv_heads, int head_size,
                                          int block_size, int max_blocks, float scale, void* stream) {
    if (o_peers == nullptr) {
        fa::set_last_error("flash_attn_with_kvcache_allgather: o_peers must not be null");
        return FLASH_ATTN_ERR_NULL_PTR;
    }
    return fa::kvcache_impl(fa::DT_F16, q, k_cache, v_cache, nullptr, block_tables, context_lens, num_seqs, 1, q_heads,
                            kv_heads, head_size, block_size, max_blocks, scale, stream, o_peers, n_peers, q_heads_total,
                            q_head_offset);
}
int flash_attn_with_kvcache_bf16_allgather(const flash_attn_bf16_t* q, const flash_attn_bf16_t* k_cache,
                                           const flash_attn_bf16_t* v_cache, void* const* o_peers, int n_peers,
                                           int q_heads_total, int q_head_offset, const int* block_tables,
                                           const int* context_lens, int num_seqs, int q_heads, int kv_heads, int head_size,
                                           int block_size, int max_blocks, float scale, void* stream) {
    if (o_peers == nullptr) {
        fa::set_last_error("flash_attn_with_kvcache_allgather: o_peers must not be null");
        return FLASH_ATTN_ERR_NULL_PTR;
    }
    return fa::kvcache_impl(fa::DT_BF16, q, k_cache, v_cache, nullptr, block_tables, context_lens, num_seqs, 1, q_heads,
                            kv_heads, head_size, block_size, max_blocks, scale, stream, o_peers, n_peers, q_heads_total,
                            q_head_offset);
}

int flash_attn_kvcache_append(const void* k_new, const void* v_new, void* k_cache, void* v_cache,
                              const int* block_tables, const int* context_lens, int num_seqs, int n_new,
                              int kv_heads, int head_size, int elem_bytes, int block_size, int max_blocks,
                              void* stream) {
    fa::g_last_error[0] = '\0';
    cudaGetLastError();
    if (!k_new || !v_new || !k_cache || !v_cache || !block_tables || !context_lens) {
        fa::set_last_error("flash_attn_kvcache_append: null pointer argument");
        return FLASH_ATTN_ERR_NULL_PTR;
    }
    if (num_seqs <= 0 || n_new <= 0 || kv_heads <= 0 || block_size <= 0 || max_blocks <= 0) {
        fa::set_last_error("flash_attn_kvcache_append: num_seqs/n_new/kv_heads/block_size/max_blocks must be > 0");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    if (!fa::head_size_ok(head_size) || (elem_bytes != 2 && elem_bytes != 4)) {
        fa::set_last_error("flash_attn_kvcache_append: head_size must be 32/64/128 and elem_bytes 2 or 4");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    if ((reinterpret_cast<uintptr_t>(k_new) | reinterpret_cast<uintptr_t>(v_new) | reinterpret_cast<uintptr_t>(k_cache) |
         reinterpret_cast<uintptr_t>(v_cache)) & 15) {
        fa::set_last_error("flash_attn_kvcache_append: buffers must be 16-byte aligned");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    if (!fa::have_device()) return FLASH_ATTN_ERR_CUDA;
    fa::DeviceGuard guard(k_cache);
    return fa::launch_kv_append(elem_bytes, k_new, v_new, k_cache, v_cache, block_tables, context_lens, num_seqs, n_new,
                                kv_heads, head_size, block_size, max_blocks, reinterpret_cast<cudaStream_t>(stream));
}

int flash_attn_debug_block_slots(const int* block_tables, const int* context_lens, const int* offsets,
                                 int num_seqs, int block_size, int max_blocks, int* out_slots,
                                 void* stream) {
    fa::g_last_error[0] = '\0';
    cudaGetLastError();
    if (!block_tables || !context_lens || !offsets || !out_slots) {
        fa::set_last_error("flash_attn_debug_block_slots: null pointer argument");
        return FLASH_ATTN_ERR_NULL_PTR;
    }
    if (num_seqs <= 0 || block_size <= 0 || max_blocks <= 0) {
        fa::set_last_error("flash_attn_debug_block_slots: num_seqs/block_size/max_blocks must be > 0");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    if (!fa::have_device()) return FLASH_ATTN_ERR_CUDA;
    fa::DeviceGuard guard(block_tables);
    return fa::launch_debug_block_slots(block_tables, context_lens, offsets, num_seqs, block_size,
                                        max_blocks, out_slots, reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
