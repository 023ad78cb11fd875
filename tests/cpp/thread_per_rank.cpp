// Thread-per-rank use of the C ABI, the default launch scheme of the reference
// (luma-dist/src/scheme/multi_thread.rs:25-48: one host thread per rank, every thread driving its
// own device handle with its own stream, luma-cuda/src/device.rs:16-110,138-139).
//
// Two parts, both compared bit for bit with a single-threaded run of the same calls:
//   1. N host threads (N = 2, on one GPU each when the box has two, else both on GPU 0), each with
//      its own stream, call flash_attn_bf16 (tensor-core prefill) and flash_attn_with_kvcache_bf16
//      (split-K decode) concurrently, several rounds; flash_attn_last_error() must stay per thread
//      (one thread provokes an error every round, the other must never see its message).
//   2. With two or more GPUs: luma_comm_from_devices (ncclCommInitAll, peer access enabled), each
//      thread runs the head-sharded prefill whose epilogue stores into every rank's full output
//      (flash_attn_bf16_allgather with plain pointers into the other GPUs' memory — one address
//      space, no IPC), then luma_comm_barrier; every rank's gathered tensor must equal the
//      unsharded result. The same through luma_comm_all_gather (attention, then the collective).
// Prints one line per check and exits non-zero on the first failure.
#include <cuda_runtime.h>

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "../../include/flash_attn.h"
#include "../../include/luma_dist_comm.h"

namespace {

uint16_t to_bf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    const uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;   // round to nearest even
    return (uint16_t)(u >> 16);
}

// xorshift64* as the reference's tests use it (luma-flash-attn/tests/low.rs:363-384), values in [-1, 1)
struct Rng {
    uint64_t s;
    explicit Rng(uint64_t seed) : s(seed | 1) {}
    float next() {
        s ^= s >> 12;
        s ^= s << 25;
        s ^= s >> 27;
        const uint64_t r = s * 0x2545F4914F6CDD1DULL;
        return (float)((double)(r >> 11) / (double)(1ULL << 53) * 2.0 - 1.0);
    }
};

std::vector<uint16_t> random_bf16(size_t n, uint64_t seed) {
    Rng rng(seed);
    std::vector<uint16_t> v(n);
    for (auto& x : v) x = to_bf16(rng.next());
    return v;
}

#define CK(call)                                                                                  \
    do {                                                                                          \
        cudaError_t e_ = (call);                                                                  \
        if (e_ != cudaSuccess) {                                                                  \
            std::printf("FAIL cuda %s: %s\n", #call, cudaGetErrorString(e_));                     \
            std::exit(2);                                                                         \
        }                                                                                         \
    } while (0)

template <typename T>
T* dev_upload(const std::vector<T>& h) {
    T* p = nullptr;
    CK(cudaMalloc(&p, h.size() * sizeof(T)));
    CK(cudaMemcpy(p, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice));
    return p;
}

struct Problem {
    // prefill
    int b = 2, s = 384, hq = 8, hkv = 2, d = 128;
    // decode
    int n = 5, page = 16, max_blocks = 48;
    std::vector<uint16_t> q, k, v, qd, kc, vc;
    std::vector<int> lens, table;
    explicit Problem(uint64_t seed) {
        q = random_bf16((size_t)b * s * hq * d, seed + 1);
        k = random_bf16((size_t)b * s * hkv * d, seed + 2);
        v = random_bf16((size_t)b * s * hkv * d, seed + 3);
        qd = random_bf16((size_t)n * hq * d, seed + 4);
        const int pool = n * max_blocks;
        kc = random_bf16((size_t)pool * page * hkv * d, seed + 5);
        vc = random_bf16((size_t)pool * page * hkv * d, seed + 6);
        lens = {700, 33, 1, 512, 767};
        table.assign((size_t)n * max_blocks, -1);
        // pages dealt out in a scrambled order
        int next = 0;
        for (int i = 0; i < n; ++i)
            for (int p = 0; p < (lens[i] + page - 1) / page; ++p) table[(size_t)i * max_blocks + p] = (next++ * 37) % pool;
    }
};

struct Result {
    std::vector<uint16_t> o_prefill, o_decode;
};

// Runs the two calls on `device` with a stream of its own; returns the outputs.
bool run_once(const Problem& pr, int device, Result& out, std::string& err) {
    CK(cudaSetDevice(device));
    cudaStream_t st;
    CK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    uint16_t *q = dev_upload(pr.q), *k = dev_upload(pr.k), *v = dev_upload(pr.v), *qd = dev_upload(pr.qd), *kc = dev_upload(pr.kc),
             *vc = dev_upload(pr.vc);
    int *lens = dev_upload(pr.lens), *table = dev_upload(pr.table);
    uint16_t *o = nullptr, *od = nullptr;
    CK(cudaMalloc(&o, pr.q.size() * 2));
    CK(cudaMalloc(&od, pr.qd.size() * 2));
    CK(cudaMemset(o, 0xff, pr.q.size() * 2));
    CK(cudaMemset(od, 0xff, pr.qd.size() * 2));
    const float scale = 1.0f / std::sqrt((float)pr.d);
    bool ok = true;
    int rc = flash_attn_bf16(q, k, v, o, pr.b, pr.s, pr.s, pr.hq, pr.hkv, pr.d, 0, scale, nullptr, st);
    if (rc != 0) { err = std::string("flash_attn_bf16: ") + flash_attn_last_error(); ok = false; }
    if (ok && std::strcmp(flash_attn_last_path(), "prefill_tcgen05") != 0) { err = "prefill took another path"; ok = false; }
    if (ok) {
        rc = flash_attn_with_kvcache_bf16(qd, kc, vc, od, table, lens, pr.n, 1, pr.hq, pr.hkv, pr.d, pr.page, pr.max_blocks, scale, st);
        if (rc != 0) { err = std::string("flash_attn_with_kvcache_bf16: ") + flash_attn_last_error(); ok = false; }
    }
    CK(cudaStreamSynchronize(st));
    out.o_prefill.resize(pr.q.size());
    out.o_decode.resize(pr.qd.size());
    CK(cudaMemcpy(out.o_prefill.data(), o, pr.q.size() * 2, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(out.o_decode.data(), od, pr.qd.size() * 2, cudaMemcpyDeviceToHost));
    for (void* p : {(void*)q, (void*)k, (void*)v, (void*)qd, (void*)kc, (void*)vc, (void*)lens, (void*)table, (void*)o, (void*)od}) cudaFree(p);
    cudaStreamDestroy(st);
    return ok;
}

int part_concurrent_calls(int ndev) {
    const int nthreads = 2, rounds = 4;
    Problem prs[2] = {Problem(100), Problem(200)};
    Result want[2];
    std::string err;
    for (int t = 0; t < nthreads; ++t)
        if (!run_once(prs[t], 0, want[t], err)) { std::printf("FAIL single-threaded run: %s\n", err.c_str()); return 1; }
    std::atomic<int> failures{0};
    std::vector<std::thread> th;
    for (int t = 0; t < nthreads; ++t) {
        th.emplace_back([&, t]() {
            const int device = ndev >= 2 ? t : 0;
            for (int r = 0; r < rounds; ++r) {
                Result got;
                std::string e;
                if (!run_once(prs[t], device, got, e)) { std::printf("FAIL thread %d: %s\n", t, e.c_str()); failures++; return; }
                if (got.o_prefill != want[t].o_prefill || got.o_decode != want[t].o_decode) {
                    std::printf("FAIL thread %d round %d: result differs from the single-threaded run\n", t, r);
                    failures++;
                    return;
                }
                if (t == 0) {
                    // this thread's error message must be its own ...
                    const int rc = flash_attn_bf16(nullptr, nullptr, nullptr, nullptr, 1, 1, 1, 1, 1, 64, 0, 1.0f, nullptr, nullptr);
                    if (rc != FLASH_ATTN_ERR_NULL_PTR || std::strlen(flash_attn_last_error()) == 0) { std::printf("FAIL thread 0: expected a null-pointer error\n"); failures++; return; }
                } else if (std::strlen(flash_attn_last_error()) != 0) {
                    // ... and never show up on the other thread
                    std::printf("FAIL thread 1 sees an error message it did not cause: %s\n", flash_attn_last_error());
                    failures++;
                    return;
                }
            }
        });
    }
    for (auto& x : th) x.join();
    if (failures.load() == 0) std::printf("ok   concurrent calls from %d threads on %d device(s), %d rounds, bit-identical to single-threaded\n", nthreads, ndev >= 2 ? 2 : 1, rounds);
    return failures.load();
}

int part_sharded(int ndev) {
    const int world = ndev >= 4 ? 4 : 2;
    const int b = 1, s = 640, hq = 8, hkv = 4, d = 128;
    const int hq_l = hq / world, hkv_l = hkv / world;
    const size_t q_sz = (size_t)b * s * hq * d, kv_sz = (size_t)b * s * hkv * d;
    const std::vector<uint16_t> q = random_bf16(q_sz, 11), k = random_bf16(kv_sz, 12), v = random_bf16(kv_sz, 13);
    const float scale = 1.0f / std::sqrt((float)d);
    // unsharded result on device 0
    std::vector<uint16_t> want(q_sz);
    {
        CK(cudaSetDevice(0));
        uint16_t *dq = dev_upload(q), *dk = dev_upload(k), *dv = dev_upload(v), *dout = nullptr;
        CK(cudaMalloc(&dout, q_sz * 2));
        if (flash_attn_bf16(dq, dk, dv, dout, b, s, s, hq, hkv, d, 0, scale, nullptr, nullptr) != 0) { std::printf("FAIL unsharded: %s\n", flash_attn_last_error()); return 1; }
        CK(cudaDeviceSynchronize());
        CK(cudaMemcpy(want.data(), dout, q_sz * 2, cudaMemcpyDeviceToHost));
        cudaFree(dq); cudaFree(dk); cudaFree(dv); cudaFree(dout);
    }
    std::vector<int> devices(world);
    for (int i = 0; i < world; ++i) devices[i] = i;
    std::vector<luma_comm*> comms(world, nullptr);
    if (luma_comm_from_devices(comms.data(), world, devices.data()) != 0) { std::printf("FAIL luma_comm_from_devices: %s\n", luma_comm_last_error()); return 1; }
    // every rank's full output buffers (fused path and two-step path), allocated up front so that all pointers are known
    std::vector<uint16_t*> full(world), full2(world);
    for (int r = 0; r < world; ++r) {
        CK(cudaSetDevice(r));
        CK(cudaMalloc(&full[r], q_sz * 2));
        CK(cudaMalloc(&full2[r], q_sz * 2));
        CK(cudaMemset(full[r], 0xff, q_sz * 2));
        CK(cudaMemset(full2[r], 0xff, q_sz * 2));
        CK(cudaDeviceSynchronize());
    }
    std::atomic<int> failures{0};
    std::vector<std::thread> th;
    for (int r = 0; r < world; ++r) {
        th.emplace_back([&, r]() {
            CK(cudaSetDevice(r));
            cudaStream_t st;
            CK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
            // this rank's shard: query heads [r*hq_l, (r+1)*hq_l), KV heads [r*hkv_l, (r+1)*hkv_l)
            std::vector<uint16_t> ql((size_t)b * s * hq_l * d), kl((size_t)b * s * hkv_l * d), vl(kl.size());
            for (size_t row = 0; row < (size_t)b * s; ++row) {
                std::memcpy(&ql[row * hq_l * d], &q[(row * hq + (size_t)r * hq_l) * d], (size_t)hq_l * d * 2);
                std::memcpy(&kl[row * hkv_l * d], &k[(row * hkv + (size_t)r * hkv_l) * d], (size_t)hkv_l * d * 2);
                std::memcpy(&vl[row * hkv_l * d], &v[(row * hkv + (size_t)r * hkv_l) * d], (size_t)hkv_l * d * 2);
            }
            uint16_t *dq = dev_upload(ql), *dk = dev_upload(kl), *dv = dev_upload(vl), *o_local = nullptr;
            CK(cudaMalloc(&o_local, ql.size() * 2));
            std::vector<void*> peers(world);
            for (int i = 0; i < world; ++i) peers[i] = full[i];
            int rc = flash_attn_bf16_allgather(dq, dk, dv, peers.data(), world, hq, r * hq_l, nullptr, b, s, s, hq_l, hkv_l, d, 0, scale, st);
            if (rc != 0) { std::printf("FAIL rank %d fused: %s\n", r, flash_attn_last_error()); failures++; }
            if (luma_comm_barrier(comms[r], st) != 0) { std::printf("FAIL rank %d barrier: %s\n", r, luma_comm_last_error()); failures++; }
            // two-step: attention on the shard, then all_gather along the head axis (dim 2 of (b, s, h, d))
            rc = flash_attn_bf16(dq, dk, dv, o_local, b, s, s, hq_l, hkv_l, d, 0, scale, nullptr, st);
            if (rc != 0) { std::printf("FAIL rank %d local: %s\n", r, flash_attn_last_error()); failures++; }
            if (luma_comm_all_gather(comms[r], o_local, full2[r], (long long)b * s, (long long)hq_l * d * 2, st) != 0) {
                std::printf("FAIL rank %d all_gather: %s\n", r, luma_comm_last_error());
                failures++;
            }
            CK(cudaStreamSynchronize(st));
            std::vector<uint16_t> got(q_sz), got2(q_sz);
            CK(cudaMemcpy(got.data(), full[r], q_sz * 2, cudaMemcpyDeviceToHost));
            CK(cudaMemcpy(got2.data(), full2[r], q_sz * 2, cudaMemcpyDeviceToHost));
            if (got != want) { std::printf("FAIL rank %d: fused all-gather differs from the unsharded result\n", r); failures++; }
            if (got2 != want) { std::printf("FAIL rank %d: luma_comm_all_gather differs from the unsharded result\n", r); failures++; }
            cudaFree(dq); cudaFree(dk); cudaFree(dv); cudaFree(o_local);
            cudaStreamDestroy(st);
        });
    }
    for (auto& x : th) x.join();
    for (int r = 0; r < world; ++r) {
        luma_comm_destroy(comms[r]);
        CK(cudaSetDevice(r));
        cudaFree(full[r]);
        cudaFree(full2[r]);
    }
    if (failures.load() == 0) std::printf("ok   thread-per-rank head-sharded prefill on %d GPUs: fused and two-step all-gather equal the unsharded result on every rank\n", world);
    return failures.load();
}

int part_single_rank_comm() {
    // world of one: the communicator, the gather along an inner axis and the barrier still run
    int dev = 0;
    luma_comm* c = nullptr;
    if (luma_comm_from_devices(&c, 1, &dev) != 0) { std::printf("FAIL luma_comm_from_devices(1): %s\n", luma_comm_last_error()); return 1; }
    const std::vector<uint16_t> x = random_bf16(6 * 40, 5);
    CK(cudaSetDevice(0));
    uint16_t *dx = dev_upload(x), *dy = nullptr;
    CK(cudaMalloc(&dy, x.size() * 2));
    int bad = 0;
    if (luma_comm_all_gather(c, dx, dy, 6, 80, nullptr) != 0 || luma_comm_barrier(c, nullptr) != 0) { std::printf("FAIL: %s\n", luma_comm_last_error()); bad = 1; }
    CK(cudaDeviceSynchronize());
    std::vector<uint16_t> y(x.size());
    CK(cudaMemcpy(y.data(), dy, x.size() * 2, cudaMemcpyDeviceToHost));
    if (!bad && y != x) { std::printf("FAIL: all_gather over one rank is not the identity\n"); bad = 1; }
    if (luma_comm_rank(c) != 0 || luma_comm_world_size(c) != 1) { std::printf("FAIL: rank / world of a single communicator\n"); bad = 1; }
    luma_comm_destroy(c);
    cudaFree(dx); cudaFree(dy);
    if (!bad) std::printf("ok   single-rank communicator: all_gather is the identity, barrier completes\n");
    return bad;
}

}  // namespace

int main() {
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) { std::printf("no CUDA device\n"); return 3; }
    int failures = part_concurrent_calls(ndev);
    failures += part_single_rank_comm();
    if (ndev >= 2) failures += part_sharded(ndev);
    else std::printf("skip thread-per-rank sharded prefill: one GPU\n");
    if (flash_attn_device_status() != 0) { std::printf("FAIL: device status word is set\n"); failures++; }
    std::printf(failures == 0 ? "PASSED\n" : "FAILED (%d)\n", failures);
    return failures == 0 ? 0 : 1;
}
