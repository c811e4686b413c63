/* C door onto the brt runtime (Session / RequestContext), for hosts that cannot
 * include the C++ headers: the Python tests and benchmark drive the runtime
 * through it with ctypes.  It adds nothing to the C++ API in include/brt/.
 *
 * Every function that returns int returns 0 on success; on failure the message of
 * the failed Status (or exception) is available from brt_last_error() on the same
 * thread.
 */
#ifndef BRT_C_API_H_
#define BRT_C_API_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct brt_session brt_session;
typedef struct brt_request brt_request;

const char *brt_last_error(void);

/* ExecutionProvider::StaticRegisterKernelsFromDynlib: load a kernel plug-in
 * before the providers that should see its kernels are created */
int brt_register_kernels_from_dynlib(const char *path);

brt_session *brt_session_create(void);
void brt_session_destroy(brt_session *s);
/* DistributedSession(rank, nranks): one rank of several, each loading its own module.  The
 * communicator its nccl.* ops run on is one of:
 *  - a function of the host program that runs one all-reduce on the process group it created once
 *    (DistributedBackendCallback): fn(user, send, recv, len, dtype (brt::DTypeEnum), op (0 sum, 1 max,
 *    2 min), group, group_len, stream (NULL for host buffers)) returns 0 on success;
 *  - the one-kernel sum over NVLink peer memory (DistributedBackendPeer): peer_inbox / peer_flags are
 *    nranks device addresses each (memory every rank has mapped, zeroed once), epoch_counter a zeroed
 *    device uint32, status a device int or NULL; sums f32 vectors of exactly `capacity` elements over
 *    all ranks. */
brt_session *brt_session_create_distributed(int rank, int nranks);
typedef int (*brt_allreduce_fn)(void *user, const void *send, void *recv, uint64_t len, int dtype, int op,
                                const int64_t *group, uint64_t group_len, void *stream);
int brt_session_set_allreduce_callback(brt_session *s, brt_allreduce_fn fn, void *user);
int brt_session_set_allreduce_peer(brt_session *s, uint64_t capacity, void *const *peer_inbox, void *const *peer_flags,
                                   void *epoch_counter, void *status);
/* NaiveCPUExecutionProviderFactory: "cpu" allocator + host provider */
int brt_session_add_cpu(brt_session *s);
/* CUDAAllocatorFactory(device) + DefaultCUDAExecutionProviderFactory */
int brt_session_add_cuda(brt_session *s, int device_id);
/* same, with device memory taken from caller functions void*(size_t) / void(void*) */
int brt_session_add_cuda_external(brt_session *s, int device_id, void *alloc_fn, void *free_fn);
int brt_session_load(brt_session *s, const char *path);                 /* Session::Load(path, "byre") */
int brt_session_load_from_memory(brt_session *s, const char *byre_text); /* Session::LoadFromMemory */
/* `size` bytes of ByRE text or ByRE bytecode (byre_serial 1.0.0) */
int brt_session_load_buffer(brt_session *s, const void *data, size_t size);

int64_t brt_session_arg_num(brt_session *s);
int brt_session_arg_offset(brt_session *s, const char *name); /* -1 if unknown */
/* dtype: brt::DTypeEnum value; argtype: 1 input, 2 output, 4 weight (bit mask);
 * shape receives up to 8 dims; space and name receive NUL-terminated strings */
int brt_session_arg_info(brt_session *s, int64_t offset, int *dtype, int *rank, int64_t *shape, char *space,
                         size_t space_cap, int *argtype, char *name, size_t name_cap);

/* cuda_stream != NULL: run on that stream (CUDAExternalStreamWorkQueue);
 * NULL: the session creates the queue its model needs */
brt_request *brt_request_create(brt_session *s, void *cuda_stream);
void brt_request_destroy(brt_request *r);
int brt_request_bind_arg(brt_request *r, int64_t offset, void *ptr); /* OwnedByExternal */
void *brt_request_get_arg(brt_request *r, int64_t offset);
int brt_request_finish_io_binding(brt_request *r);
int brt_session_run(brt_session *s, brt_request *r);
int brt_request_sync(brt_request *r);
/* records the key of every op run on this request (Before/AfterOpKernelRun
 * listeners); brt_request_op_trace copies "key;key;..." and returns its length */
int brt_request_enable_op_trace(brt_request *r);
int64_t brt_request_op_trace(brt_request *r, char *buf, size_t cap);

#ifdef __cplusplus
}
#endif
#endif /* BRT_C_API_H_ */
