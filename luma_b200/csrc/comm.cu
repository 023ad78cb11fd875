// The collective boundary of the head-sharded attention path (include/luma_dist_comm.h): NCCL
// communicators for one rank per process or one rank per thread, all_gather along an axis, a
// barrier, and CUDA IPC export / open for peer buffers between processes.
//
// Stands in for luma-dist's NCCL backend on this path: NcclBackend::from_devices / from_rank
// (luma-dist/src/backends/nccl/mod.rs:26-42,56-64), all_gather_float -> all_gather_into
// (backends/nccl/backend.rs:167-180) with the layout handling of luma-dist/src/utils.rs:12-37.
// The reference permutes the gather axis to the front, materialises, zero-fills the receive
// buffer, gathers, permutes back and materialises again; here the input is sent as it lies and the
// result takes one interleaving pass (none when the axis is the outermost one).
//
// NCCL is called directly through its C API; the library is opened at run time so that
// libflash_attn has no link-time dependency on it.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>

#include "../../include/luma_dist_comm.h"

namespace {

thread_local char g_comm_error[256] = {0};

int fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    std::vsnprintf(g_comm_error, sizeof(g_comm_error), fmt, ap);
    va_end(ap);
    return 1;
}

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommInitAll)(ncclComm_t*, int, const int*) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

NcclApi* nccl_api() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, []() {
        const char* names[3] = {std::getenv("LUMA_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
        for (const char* n : names) {
            if (n == nullptr || n[0] == '\0') continue;
            api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (api.handle != nullptr) break;
        }
        if (api.handle == nullptr) return;
        auto sym = [&](const char* s) { return dlsym(api.handle, s); };
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
        api.CommInitAll = reinterpret_cast<decltype(api.CommInitAll)>(sym("ncclCommInitAll"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
        api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
        if (!api.GetUniqueId || !api.CommInitRank || !api.CommInitAll || !api.CommDestroy || !api.AllGather ||
            !api.AllReduce || !api.GetErrorString) {
            dlclose(api.handle);
            api.handle = nullptr;
        }
    });
    return api.handle != nullptr ? &api : nullptr;
}

int nccl_fail(const char* what, ncclResult_t rc) {
    NcclApi* api = nccl_api();
    return fail("%s: %s", what, api != nullptr ? api->GetErrorString(rc) : "NCCL not loaded");
}

struct DeviceScope {
    int prev = -1;
    bool ok = true;
    explicit DeviceScope(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != dev) ok = cudaSetDevice(dev) == cudaSuccess;
    }
    ~DeviceScope() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

// (world, outer, chunk) -> (outer, world, chunk), 16 bytes per thread and step.
__global__ void interleave_kernel(const uint4* __restrict__ staging, uint4* __restrict__ out, long long outer,
                                  long long chunk_vecs, int world) {
    const long long total = outer * chunk_vecs * world;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long v = i % chunk_vecs;
        const long long t = i / chunk_vecs;
        const int r = (int)(t % world);
        const long long o = t / world;
        out[i] = staging[((long long)r * outer + o) * chunk_vecs + v];
    }
}

__global__ void interleave_bytes_kernel(const unsigned char* __restrict__ staging, unsigned char* __restrict__ out,
                                        long long outer, long long chunk_bytes, int world) {
    const long long total = outer * chunk_bytes * world;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long v = i % chunk_bytes;
        const long long t = i / chunk_bytes;
        const int r = (int)(t % world);
        const long long o = t / world;
        out[i] = staging[((long long)r * outer + o) * chunk_bytes + v];
    }
}

// An allocation can be opened only once per process, and allocators carve several tensors out of
// one allocation: mappings are kept by handle with a count of the pointers handed out from them.
struct IpcMapping {
    void* base = nullptr;
    int refs = 0;
};
std::mutex g_ipc_mutex;
std::map<std::string, IpcMapping> g_ipc_by_handle;
std::map<void*, std::string> g_ipc_handle_of;   // pointer handed out -> its allocation's handle

}  // namespace

struct luma_comm {
    ncclComm_t comm = nullptr;
    int rank = 0;
    int world = 1;
    int device = 0;
    void* staging = nullptr;
    size_t staging_bytes = 0;
    int* flag = nullptr;   // device word for the barrier's all-reduce
};

extern "C" {

const char* luma_comm_last_error(void) { return g_comm_error; }

int luma_comm_unique_id(void* id_out) {
    g_comm_error[0] = '\0';
    if (id_out == nullptr) return fail("luma_comm_unique_id: id_out must not be null");
    NcclApi* api = nccl_api();
    if (api == nullptr) return fail("luma_comm: libnccl.so.2 could not be opened (set LUMA_NCCL_LIB)");
    static_assert(sizeof(ncclUniqueId) == LUMA_COMM_UNIQUE_ID_BYTES, "ncclUniqueId is 128 bytes");
    ncclUniqueId id;
    const ncclResult_t rc = api->GetUniqueId(&id);
    if (rc != ncclSuccess) return nccl_fail("ncclGetUniqueId", rc);
    std::memcpy(id_out, &id, sizeof(id));
    return 0;
}

static int finish_comm(luma_comm* c) {
    DeviceScope scope(c->device);
    if (!scope.ok) return fail("luma_comm: cannot select device %d", c->device);
    if (cudaMalloc(reinterpret_cast<void**>(&c->flag), sizeof(int)) != cudaSuccess) {
        cudaGetLastError();
        return fail("luma_comm: cannot allocate the barrier word on device %d", c->device);
    }
    cudaMemset(c->flag, 0, sizeof(int));
    return 0;
}

int luma_comm_from_rank(luma_comm** out, int nranks, const void* id, int rank, int device) {
    g_comm_error[0] = '\0';
    if (out == nullptr || id == nullptr) return fail("luma_comm_from_rank: out / id must not be null");
    if (nranks <= 0 || rank < 0 || rank >= nranks) return fail("luma_comm_from_rank: rank %d of %d", rank, nranks);
    NcclApi* api = nccl_api();
    if (api == nullptr) return fail("luma_comm: libnccl.so.2 could not be opened (set LUMA_NCCL_LIB)");
    DeviceScope scope(device);
    if (!scope.ok) return fail("luma_comm_from_rank: cannot select device %d", device);
    ncclUniqueId uid;
    std::memcpy(&uid, id, sizeof(uid));
    luma_comm* c = new luma_comm();
    c->rank = rank;
    c->world = nranks;
    c->device = device;
    const ncclResult_t rc = api->CommInitRank(&c->comm, nranks, uid, rank);
    if (rc != ncclSuccess) {
        delete c;
        return nccl_fail("ncclCommInitRank", rc);
    }
    if (finish_comm(c) != 0) {
        api->CommDestroy(c->comm);
        delete c;
        return 1;
    }
    *out = c;
    return 0;
}

int luma_comm_from_devices(luma_comm** out, int ndev, const int* devices) {
    g_comm_error[0] = '\0';
    if (out == nullptr || devices == nullptr || ndev <= 0 || ndev > 64) return fail("luma_comm_from_devices: bad arguments");
    NcclApi* api = nccl_api();
    if (api == nullptr) return fail("luma_comm: libnccl.so.2 could not be opened (set LUMA_NCCL_LIB)");
    ncclComm_t comms[64];
    const ncclResult_t rc = api->CommInitAll(comms, ndev, devices);
    if (rc != ncclSuccess) return nccl_fail("ncclCommInitAll", rc);
    for (int i = 0; i < ndev; ++i) {
        luma_comm* c = new luma_comm();
        c->comm = comms[i];
        c->rank = i;
        c->world = ndev;
        c->device = devices[i];
        if (finish_comm(c) != 0) return 1;
        out[i] = c;
    }
    // one address space, several GPUs: let every device reach every other one's memory
    for (int i = 0; i < ndev; ++i) {
        DeviceScope scope(devices[i]);
        for (int j = 0; j < ndev; ++j) {
            if (i == j) continue;
            int can = 0;
            if (cudaDeviceCanAccessPeer(&can, devices[i], devices[j]) == cudaSuccess && can) {
                const cudaError_t e = cudaDeviceEnablePeerAccess(devices[j], 0);
                if (e != cudaSuccess) cudaGetLastError();   // already enabled counts as fine
            }
        }
    }
    return 0;
}

int luma_comm_rank(const luma_comm* c) { return c != nullptr ? c->rank : -1; }
int luma_comm_world_size(const luma_comm* c) { return c != nullptr ? c->world : -1; }
int luma_comm_device(const luma_comm* c) { return c != nullptr ? c->device : -1; }

int luma_comm_all_gather(luma_comm* c, const void* send, void* recv, long long outer, long long chunk_bytes,
                         void* stream) {
    g_comm_error[0] = '\0';
    if (c == nullptr || send == nullptr || recv == nullptr) return fail("luma_comm_all_gather: null argument");
    if (outer <= 0 || chunk_bytes <= 0) return fail("luma_comm_all_gather: outer and chunk_bytes must be positive");
    NcclApi* api = nccl_api();
    if (api == nullptr) return fail("luma_comm: libnccl.so.2 could not be opened (set LUMA_NCCL_LIB)");
    DeviceScope scope(c->device);
    if (!scope.ok) return fail("luma_comm_all_gather: cannot select device %d", c->device);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const size_t local_bytes = (size_t)outer * (size_t)chunk_bytes;
    if (outer == 1 || c->world == 1) {
        // the gather axis is the outermost one that matters: NCCL's rank-major result is the answer
        const ncclResult_t rc = api->AllGather(send, recv, local_bytes, ncclInt8, c->comm, st);
        return rc == ncclSuccess ? 0 : nccl_fail("ncclAllGather", rc);
    }
    const size_t need = local_bytes * (size_t)c->world;
    if (c->staging_bytes < need) {
        if (c->staging != nullptr) cudaFreeAsync(c->staging, st);   // ordered after the work that reads it
        c->staging = nullptr;
        c->staging_bytes = 0;
        if (cudaMallocAsync(&c->staging, need, st) != cudaSuccess) {
            cudaGetLastError();
            return fail("luma_comm_all_gather: cannot allocate %zu bytes of staging", need);
        }
        c->staging_bytes = need;
    }
    const ncclResult_t rc = api->AllGather(send, c->staging, local_bytes, ncclInt8, c->comm, st);
    if (rc != ncclSuccess) return nccl_fail("ncclAllGather", rc);
    const bool vec = (chunk_bytes % 16) == 0 && ((reinterpret_cast<uintptr_t>(recv) | reinterpret_cast<uintptr_t>(c->staging)) & 15) == 0;
    const long long units = vec ? (long long)(need / 16) : (long long)need;
    const int threads = 256;
    const long long want_blocks = (units + threads - 1) / threads;
    const int blocks = (int)(want_blocks < 148LL * 16 ? (want_blocks > 0 ? want_blocks : 1) : 148LL * 16);
    if (vec)
        interleave_kernel<<<blocks, threads, 0, st>>>(static_cast<const uint4*>(c->staging), static_cast<uint4*>(recv), outer,
                                                     chunk_bytes / 16, c->world);
    else
        interleave_bytes_kernel<<<blocks, threads, 0, st>>>(static_cast<const unsigned char*>(c->staging),
                                                           static_cast<unsigned char*>(recv), outer, chunk_bytes, c->world);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail("luma_comm_all_gather: interleave kernel: %s", cudaGetErrorString(e));
    return 0;
}

int luma_comm_barrier(luma_comm* c, void* stream) {
    g_comm_error[0] = '\0';
    if (c == nullptr) return fail("luma_comm_barrier: null communicator");
    NcclApi* api = nccl_api();
    if (api == nullptr) return fail("luma_comm: libnccl.so.2 could not be opened (set LUMA_NCCL_LIB)");
    DeviceScope scope(c->device);
    if (!scope.ok) return fail("luma_comm_barrier: cannot select device %d", c->device);
    const ncclResult_t rc = api->AllReduce(c->flag, c->flag, 1, ncclInt32, ncclSum, c->comm, reinterpret_cast<cudaStream_t>(stream));
    return rc == ncclSuccess ? 0 : nccl_fail("ncclAllReduce", rc);
}

int luma_comm_destroy(luma_comm* c) {
    g_comm_error[0] = '\0';
    if (c == nullptr) return 0;
    NcclApi* api = nccl_api();
    DeviceScope scope(c->device);
    if (scope.ok) {
        cudaDeviceSynchronize();
        if (c->staging != nullptr) cudaFree(c->staging);
        if (c->flag != nullptr) cudaFree(c->flag);
        cudaGetLastError();
    }
    if (api != nullptr && c->comm != nullptr) api->CommDestroy(c->comm);
    delete c;
    return 0;
}

int luma_ipc_export(const void* ptr, void* handle_out, long long* offset_out) {
    g_comm_error[0] = '\0';
    if (ptr == nullptr || handle_out == nullptr || offset_out == nullptr) return fail("luma_ipc_export: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "cudaIpcMemHandle_t is 64 bytes");
    // the handle names the whole allocation: find its base to tell the importer where ptr lies in it
    using RangeFn = int (*)(unsigned long long*, size_t*, unsigned long long);
    static RangeFn range_fn = nullptr;
    static std::once_flag once;
    std::call_once(once, []() {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            range_fn = reinterpret_cast<RangeFn>(p);
        else
            cudaGetLastError();
    });
    if (range_fn == nullptr) return fail("luma_ipc_export: cuMemGetAddressRange is not available");
    unsigned long long base = 0;
    size_t size = 0;
    if (range_fn(&base, &size, (unsigned long long)reinterpret_cast<uintptr_t>(ptr)) != 0)
        return fail("luma_ipc_export: the pointer is not inside a device allocation");
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>((uintptr_t)base));
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail("luma_ipc_export: cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
    }
    std::memcpy(handle_out, &h, sizeof(h));
    *offset_out = (long long)((unsigned long long)reinterpret_cast<uintptr_t>(ptr) - base);
    return 0;
}

int luma_ipc_open(const void* handle, long long offset, void** ptr_out) {
    g_comm_error[0] = '\0';
    if (handle == nullptr || ptr_out == nullptr || offset < 0) return fail("luma_ipc_open: bad argument");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    const std::string key(static_cast<const char*>(handle), sizeof(h));
    std::lock_guard<std::mutex> lock(g_ipc_mutex);
    IpcMapping& m = g_ipc_by_handle[key];
    if (m.base == nullptr) {
        const cudaError_t e = cudaIpcOpenMemHandle(&m.base, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            cudaGetLastError();
            g_ipc_by_handle.erase(key);
            return fail("luma_ipc_open: cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
        }
    }
    void* p = static_cast<unsigned char*>(m.base) + offset;
    if (g_ipc_handle_of.count(p) == 0) {
        g_ipc_handle_of[p] = key;
        m.refs += 1;
    }
    *ptr_out = p;
    return 0;
}

int luma_peer_copy(void* dst, const void* src, long long bytes, void* stream) {
    g_comm_error[0] = '\0';
    if (dst == nullptr || src == nullptr || bytes <= 0) return fail("luma_peer_copy: bad argument");
    const cudaError_t e = cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDefault, reinterpret_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail("luma_peer_copy: cudaMemcpyAsync: %s", cudaGetErrorString(e));
    }
    return 0;
}

int luma_ipc_close(void* ptr) {
    g_comm_error[0] = '\0';
    void* base = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_ipc_mutex);
        auto it = g_ipc_handle_of.find(ptr);
        if (it == g_ipc_handle_of.end()) return fail("luma_ipc_close: not a pointer returned by luma_ipc_open");
        auto mit = g_ipc_by_handle.find(it->second);
        g_ipc_handle_of.erase(it);
        if (mit == g_ipc_by_handle.end()) return 0;
        if (--mit->second.refs > 0) return 0;   // other pointers into the same allocation are still open
        base = mit->second.base;
        g_ipc_by_handle.erase(mit);
    }
    const cudaError_t e = cudaIpcCloseMemHandle(base);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail("luma_ipc_close: cudaIpcCloseMemHandle: %s", cudaGetErrorString(e));
    }
    return 0;
}

}  // extern "C"
