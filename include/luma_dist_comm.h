/*
 * C ABI of the collective boundary the head-sharded attention path needs: what luma-dist's NCCL
 * backend gives the reference, behind plain pointers so that a Rust `Comm` can bind it.
 *
 * Each function names the reference interface it stands in for (paths inside MoleSir/luma):
 *   luma_comm_unique_id / luma_comm_from_rank   NcclBackend::from_rank + init_process_group's id
 *                                               exchange  luma-dist/src/backends/nccl/mod.rs:56-64,238-252
 *   luma_comm_from_devices                      NcclBackend::from_devices (one process, one thread
 *                                               per GPU)  luma-dist/src/backends/nccl/mod.rs:26-42,
 *                                               scheme luma-dist/src/scheme/multi_thread.rs:25-48
 *   luma_comm_all_gather                        Comm::all_gather(&tensor, dim)
 *                                               luma-dist/src/base/comm.rs:212-214 ->
 *                                               backends/nccl/backend.rs:167-180 (+ the layout
 *                                               round trip of luma-dist/src/utils.rs:12-37)
 *   luma_comm_barrier                           Comm::barrier  luma-dist/src/base/comm.rs
 *
 * NCCL itself is called directly (ncclCommInitRank / ncclCommInitAll / ncclAllGather /
 * ncclAllReduce); libnccl.so.2 is looked up at run time (environment variable LUMA_NCCL_LIB, else
 * the loader's search path), so the attention library carries no link-time dependency on it.
 *
 * Status: 0 = ok, non-zero = failure with a thread-local message in luma_comm_last_error().
 */
#ifndef LUMA_B200_DIST_COMM_H_
#define LUMA_B200_DIST_COMM_H_

#ifdef __cplusplus
extern "C" {
#endif

typedef struct luma_comm luma_comm;

#define LUMA_COMM_UNIQUE_ID_BYTES 128

/* Fills id_out (128 bytes) with a fresh NCCL unique id; rank 0 makes it and hands it to the others
 * (the reference sends it over TCP, mod.rs:238-252). */
int luma_comm_unique_id(void* id_out);

/* One communicator for `rank` of `nranks`, bound to CUDA device `device` (one process or thread per
 * rank; every rank calls this with the same id). */
int luma_comm_from_rank(luma_comm** out, int nranks, const void* id, int rank, int device);

/* All communicators of one process at once: out[i] drives devices[i] as rank i (thread-per-rank
 * scheme). Peer access between the devices is enabled where the hardware allows it, so that a
 * pointer into one GPU's memory can be handed to a kernel on another (the fused all-gather of
 * flash_attn_<T>_allgather needs nothing else in this scheme). */
int luma_comm_from_devices(luma_comm** out, int ndev, const int* devices);

int luma_comm_rank(const luma_comm* c);
int luma_comm_world_size(const luma_comm* c);
int luma_comm_device(const luma_comm* c);

/*
 * Concatenates every rank's tensor along one axis. The local tensor is dense row-major and seen
 * as (outer, chunk_bytes): `outer` = product of the dims before the gather axis, `chunk_bytes` =
 * bytes of one rank's slab per outer index (local extent of the axis x the dims after it x element
 * size). recv is (outer, world, chunk_bytes). With outer == 1 this is one ncclAllGather straight
 * into recv; otherwise one ncclAllGather into a staging buffer the communicator keeps (grown,
 * stream-ordered, when needed) and one interleaving copy kernel — no memset, no copy of the input.
 * Asynchronous on `stream`.
 */
int luma_comm_all_gather(luma_comm* c, const void* send, void* recv, long long outer, long long chunk_bytes,
                         void* stream);

/* Every rank's earlier work on `stream` (peer stores included) is complete everywhere once this
 * has completed on every rank: a 4-byte ncclAllReduce. Asynchronous on `stream`. */
int luma_comm_barrier(luma_comm* c, void* stream);

int luma_comm_destroy(luma_comm* c);

/*
 * Peer memory between processes (one process per GPU): export a device allocation, open it in
 * another process, close it. `handle` is 64 bytes (cudaIpcMemHandle_t); `offset` is where ptr lies
 * inside its allocation (allocators hand out sub-ranges). No counterpart in the reference.
 */
int luma_ipc_export(const void* ptr, void* handle_out, long long* offset_out);
int luma_ipc_open(const void* handle, long long offset, void** ptr_out);
int luma_ipc_close(void* ptr);

/* One asynchronous copy between two device buffers that may live on different GPUs (a pointer from
 * luma_ipc_open, or any device pointer of a process that enabled peer access): a point-to-point
 * send as one cudaMemcpyAsync on `stream`. Used to measure the peer bandwidth that bounds the fused
 * all-gather. No counterpart in the reference. */
int luma_peer_copy(void* dst, const void* src, long long bytes, void* stream);

const char* luma_comm_last_error(void);

#ifdef __cplusplus
}
#endif

#endif /* LUMA_B200_DIST_COMM_H_ */
