/* Thin C ABI of the sm_100a kernels behind the ByRE compute ops of ByteIR's
 * default CUDA provider.  Every entry point only enqueues work on `stream`:
 * it never synchronises, never allocates device memory and never touches the
 * host copy of a tensor.  All pointers are device pointers unless said
 * otherwise; sizes are element counts unless the name says bytes.
 *
 * Return value: 0 on success, a negative B200_ERR_* otherwise.  After
 * B200_ERR_CUDA, b200_last_cuda_error() gives the cudaError_t of the failed
 * launch (thread-local).
 *
 * Each declaration names the reference interface it stands in for, by the
 * file's path inside bytedance/byteir.
 */
#ifndef B200_KERNELS_H_
#define B200_KERNELS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef __DRIVER_TYPES_H__
typedef struct CUstream_st *cudaStream_t;
#endif

#define B200_OK 0
#define B200_ERR_INVALID_ARG (-1)
#define B200_ERR_UNSUPPORTED (-2)
#define B200_ERR_WORKSPACE (-3) /* workspace missing or too small */
#define B200_ERR_CUDA (-4)
#define B200_ERR_ALIGNMENT (-5)

/* element types (the ByRE key suffixes f32 / f16 / bf16) */
#define B200_F32 0
#define B200_F16 1
#define B200_BF16 2

#define B200_REDUCE_SUM 0
#define B200_REDUCE_MAX 1

const char *b200_version(void);
int b200_last_cuda_error(void);
const char *b200_error_string(int code);

/* ---- ReduceSumOp / ReduceMaxOp -------------------------------------------
 * Replaces kernel::call_reduce<T, Op> and get_reduce_workspace_in_bytes
 * (runtime/lib/backends/cuda/providers/default/reduction/kernels/reduction.h,
 *  reduction.cu:411-434).  Input is viewed as A x B x C, row-major; B is
 * reduced; output is A x C in the input's element type.  Sum accumulates in
 * f32 (reduce_impl.h:63-69).  Max follows reduction_helper.h:159-180 folded in
 * ascending index order: any NaN gives NaN, equal values keep the later one.
 * Workspace bytes depend only on (op, dtype, A, B, C); the workspace may be
 * uninitialised.  Two calls that may overlap on the GPU need different
 * workspaces.
 */
size_t b200_reduce_workspace_bytes(int op, int dtype, int64_t A, int64_t B,
                                   int64_t C);
int b200_reduce(int op, int dtype, const void *in, void *out, int64_t A,
                int64_t B, int64_t C, void *workspace, size_t workspace_bytes,
                cudaStream_t stream);
/* Sum only: the same reduction with the A x C result left in f32, unrounded.
 * This is what a device contributes to nccl.AllReduce when the reduced axis is
 * itself sharded over devices (runtime/lib/backends/nccl/providers/
 * all_reduce.cc:44-69); b200_cast_from_f32 then rounds once.  Same workspace
 * size as b200_reduce. */
int b200_reduce_sum_to_f32(int dtype, const void *in, float *out_f32, int64_t A,
                           int64_t B, int64_t C, void *workspace,
                           size_t workspace_bytes, cudaStream_t stream);
int b200_cast_from_f32(int dtype, const float *in, void *out, int64_t n,
                       cudaStream_t stream);
/* The reductions size their grids to fill every SM exactly (one wave).  A small
 * kernel that runs BESIDE them on another stream -- the exchange below is the
 * case in point -- then takes the place of a block, which runs as a second wave
 * after all others.  b200_reduce_reserve_blocks(n) makes the following calls of
 * this process leave n block slots of the wave free (n = 1 is room for
 * b200_sharded_sum_finish); 0 restores the full wave.  Results do not change
 * bit for bit for max; for sums the split of the reduced axis, and with it the
 * order of the f32 additions, follows the grid. */
void b200_reduce_reserve_blocks(int blocks);

/* The exchange step of a sum whose reduced axis is sharded over `world` GPUs:
 * stands in for nccl.AllReduce(sum) on the f32 partials followed by the cast to the
 * storage type (runtime/lib/backends/nccl/providers/all_reduce.cc:44-69;
 * DistributedBackendNCCL::all_reduce, distributed_backend_nccl.cc:175-194), as ONE
 * kernel over NVLink peer memory.  Every rank calls it once per step, in the same
 * order, with:
 *   partial       this rank's n unrounded f32 partial sums (b200_reduce_sum_to_f32)
 *   peer_inbox[p] rank p's inbox, b200_sharded_sum_inbox_bytes(world, n) bytes,
 *   peer_flags[p] rank p's flag words, world * 4 bytes, zeroed once before first use;
 *                 both must be memory every rank can write (symmetric / IPC-mapped;
 *                 host arrays of device pointers, indexed by rank, own rank included)
 *   epoch_counter a device uint32 of this rank, zeroed once, owned by this call chain
 *   out           n elements of `dtype`, identical on every rank afterwards
 * The wait for the peers is bounded (2 s); on expiry *status (device int, may be
 * NULL) is set to 3, `out` is left as it was, the epoch does not advance, and the
 * kernel ends: check *status before trusting `out` (a caller that passes NULL
 * cannot tell), and zero the flags and counters of every rank again before the
 * next call.  Ranks must not run ahead of each other by more than this call
 * enforces itself (a rank needs every peer's epoch to finish one), so no other
 * synchronisation is needed between steps.  One block of 256 threads does the whole
 * exchange: it is meant for vectors of up to a few thousand elements (the partial sums of a
 * reduction); world <= 16.
 */
size_t b200_sharded_sum_inbox_bytes(int world, int64_t n);
int b200_sharded_sum_finish(int dtype, const float *partial, void *const *peer_inbox,
                            void *const *peer_flags, int rank, int world, int64_t n,
                            uint32_t *epoch_counter, void *out, int *status,
                            cudaStream_t stream);

/* Same reduction as b200_reduce, for callers that have no way to hand in scratch
 * memory.  (No counterpart in the reference: its reduce kernels always get their
 * workspace from the session's allocator.)  A kernel reached through the
 * byre.custom call, for instance, receives only tensor pointers, a packed
 * attribute blob and a stream: it sees no allocator and no workspace operand, and
 * a cudaMalloc in the middle of an enqueue-only op would synchronise the whole
 * device.  Here the partial sums go to a
 * fixed block of b200_reduce_no_alloc_max_bytes() (1 MiB) of device memory that is
 * part of the library image; every GPU that loads the library holds that block
 * until the process exits.  The call allocates and frees nothing.
 *  - A shape whose b200_reduce_workspace_bytes() exceeds the block is refused with
 *    B200_ERR_WORKSPACE; nothing is launched.
 *  - The first call made with a given device current looks up the block's device
 *    address (a host-side query, no device work).  Make that first call before any
 *    stream capture begins.
 *  - All calls on a device share the one block.  It keeps whatever the last call
 *    left in it, which is harmless: every partial is written before it is read, so
 *    nothing has to be cleared.  But two calls whose kernels overlap on the GPU
 *    (different streams, no ordering between them) would overwrite each other's
 *    partials: order such calls yourself.
 */
size_t b200_reduce_no_alloc_max_bytes(void);
int b200_reduce_no_alloc(int op, int dtype, const void *in, void *out, int64_t A,
                         int64_t B, int64_t C, cudaStream_t stream);

/* ---- IndexSelectOp --------------------------------------------------------
 * Replaces kernel::index_select<InputTy, IndexTy>
 * (indexing/kernels/index_select.h; index_select.cu:26-47):
 *   out[a, ob, c] = in[a, idx[ob], c],  in: A x IB x C, out: A x OB x C.
 * elt_bytes in {1,2,4,8,16}; idx_bytes 4 (ui32) or 8 (i64).  An index outside
 * [0, IB) copies nothing for that row, zero-fills it, and sets *status (a
 * device int, may be NULL) to 1; the reference reads out of bounds there.
 */
int b200_index_select(int elt_bytes, int idx_bytes, const void *in,
                      const void *idx, void *out, int64_t A, int64_t IB,
                      int64_t OB, int64_t C, int *status, cudaStream_t stream);

/* ---- IndexPutOp (accumulate) ---------------------------------------------
 * Replaces kernel::index_put<T, true> (indexing/kernels/index_put.h;
 * index_put.cu:28-55): out = in; out[idx[i], :] += upd[i, :] for every i.
 * in/out: rows x feature, upd: index_count x feature, idx: int64.
 * Unlike the reference's atomicAdd, the result does not depend on scheduling:
 * updates are ordered by (row, i), summed in f32 in a fixed tree, added to the
 * table value and rounded once.  in == out (in place) is allowed.  Indices
 * outside [0, rows) are skipped and set *status (device int, may be NULL).
 */
size_t b200_index_put_workspace_bytes(int dtype, int64_t rows,
                                      int64_t index_count, int64_t feature);
/* Out of place, the index sort runs on a helper stream beside the table copy.  The
 * helper stream and its two events belong to the pair (current device, caller
 * stream): b200_index_put_prepare creates them ahead of time (a host-side call,
 * no device work); otherwise the first b200_index_put_add on that pair does, so
 * make one of the two before a stream capture begins.  b200_index_put_release
 * destroys them; call it before destroying `stream`, whose handle value the
 * runtime may give to a later stream.  (No counterpart in the reference, whose
 * IndexPut is a copy and one atomicAdd kernel on the caller's stream.) */
int b200_index_put_prepare(cudaStream_t stream);
int b200_index_put_release(cudaStream_t stream);
int b200_index_put_add(int dtype, const void *in, const int64_t *idx,
                       const void *upd, void *out, int64_t rows,
                       int64_t index_count, int64_t feature, void *workspace,
                       size_t workspace_bytes, int *status,
                       cudaStream_t stream);

/* ---- TransposeOp ----------------------------------------------------------
 * Replaces kernel::transpose_naive_2d (tensor_manipulate/kernels/transpose.h;
 * transpose.cu:24-41) and the cudnnTransformTensor NCHW<->NHWC path
 * (tensor_manipulate/transpose.cc:68-123), both of which are a batched 2-D
 * transpose:  in: batch x rows x cols  ->  out: batch x cols x rows.
 * elt_bytes in {1,2,4,8}.
 */
int b200_transpose_batched(int elt_bytes, const void *in, void *out,
                           int64_t batch, int64_t rows, int64_t cols,
                           cudaStream_t stream);
/* General permutation, rank <= 8: out.shape[k] = shape[perm[k]].  Collapses
 * to b200_transpose_batched whenever the permutation allows it. */
int b200_permute(int elt_bytes, const void *in, void *out, int rank,
                 const int64_t *shape, const int64_t *perm,
                 cudaStream_t stream);

/* ---- FillOp -----------------------------------------------------------------
 * Replaces kernel::Fill (tensor_generate/kernels/fill.h; caller tensor_generate/
 * fill.cc:36-62): out[i] = value for i in [0, n).  elt_bytes in {1,2,4,8}; the
 * value is passed as its bit pattern in the low elt_bytes bytes of value_bits.
 */
int b200_fill(int elt_bytes, void *out, int64_t n, uint64_t value_bits, cudaStream_t stream);

/* ---- Flash attention ------------------------------------------------------
 * Typed doors behind the byre.custom entry points run_flash_attn_fwd / _bwd
 * (external_libs/runtime/flash_attn/lib/flash_api.h:75-82, argument unpacking
 * flash_api.cu:586-725).  Strides are in elements.  q,k,v,o: [B, S, H, D];
 * lse: f32 [B, H, Sq].  dtype B200_F16 or B200_BF16.
 */
typedef struct {
  int64_t q_batch_stride, k_batch_stride, v_batch_stride, o_batch_stride;
  int64_t q_row_stride, k_row_stride, v_row_stride, o_row_stride;
  int64_t q_head_stride, k_head_stride, v_head_stride, o_head_stride;
  int64_t b, h, h_k, d, d_rounded;
  float softmax_scale;
  int64_t seqlen_q, seqlen_k, seqlen_q_rounded, seqlen_k_rounded;
  float p_dropout;
  int64_t window_size_left, window_size_right;
} b200_flash_attn_params;

int b200_flash_attn_fwd(int dtype, const void *q, const void *k, const void *v,
                        void *out, float *softmax_lse,
                        const b200_flash_attn_params *params,
                        cudaStream_t stream);
/* d_softmax_sum: f32 [B, H, seqlen_q_rounded]; dq_accum: f32 scratch of
 * B * seqlen_q_rounded * H * d_rounded elements (both caller-provided, as in
 * the reference's custom call). */
int b200_flash_attn_bwd(int dtype, const void *dout, const void *q,
                        const void *k, const void *v, const void *out,
                        const float *softmax_lse, void *dq, void *dk, void *dv,
                        float *d_softmax_sum, float *dq_accum,
                        const b200_flash_attn_params *params,
                        cudaStream_t stream);

/* Every wait inside the forward and backward kernels is bounded (about 2 s).  If one
 * runs out, the block stops, stores nothing more (its part of out / dq / dk / dv
 * stays unwritten) and sets a sticky per-device status word: 2 = forward, 3 =
 * backward.  This call copies the word to *status and clears it.  It is a
 * synchronous device read: call it after synchronising the streams that ran
 * attention.  (No counterpart in the reference, whose kernels have no waits.) */
int b200_flash_attn_take_status(int *status);

/* Attention over a key/value cache (decode): the typed door behind
 * run_flash_attn_kvcache (flash_api.h:75-82, unpacking flash_api.cu:727-811, setup
 * flash_api.cu:434-566).  q, out: [B, seqlen_q, H, D]; kcache, vcache:
 * [B, seqlen_k, H_k, D] (seqlen_k = capacity of the cache); knew, vnew:
 * [B, seqlen_knew, H_k, D] or NULL; seqlens_k: i32 [B], rows of the cache in use
 * (NULL = all of it); softmax_lse: f32 [B, H, seqlen_q].  Per batch entry the new rows
 * are written into the cache at seqlens_k[b] and the queries attend to the first
 * seqlens_k[b] + seqlen_knew rows, the mask aligned to the end of the keys; new rows
 * that would not fit the cache are dropped.  D is a multiple of 8, at most 256.
 * workspace: scratch of b200_flash_attn_kvcache_workspace_bytes(params) bytes, or NULL
 * to take it from the stream's memory pool for the duration of the call. */
typedef struct {
  int64_t q_batch_stride, k_batch_stride, v_batch_stride, knew_batch_stride, vnew_batch_stride, o_batch_stride;
  int64_t q_row_stride, k_row_stride, v_row_stride, knew_row_stride, vnew_row_stride, o_row_stride;
  int64_t q_head_stride, k_head_stride, v_head_stride, knew_head_stride, vnew_head_stride, o_head_stride;
  int64_t b, h, h_k, d, d_rounded, seqlen_knew;
  float softmax_scale;
  int64_t seqlen_q, seqlen_k, seqlen_q_rounded, seqlen_k_rounded;
  int64_t window_size_left, window_size_right;
} b200_flash_kvcache_params;

int64_t b200_flash_attn_kvcache_workspace_bytes(const b200_flash_kvcache_params *params);
int b200_flash_attn_kvcache(int dtype, const void *q, void *kcache, void *vcache,
                            const void *knew, const void *vnew, const int32_t *seqlens_k,
                            void *out, float *softmax_lse,
                            const b200_flash_kvcache_params *params, void *workspace,
                            size_t workspace_bytes, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_KERNELS_H_ */
