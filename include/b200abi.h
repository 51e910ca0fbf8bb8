/* b200abi.h — C ABI of the device-primitive layer.
 *
 * Every `cl_cuda_*` / `cl_cublas_*` symbol below has the signature, the id
 * numbering and the 0 / -1 error convention of the symbol of the same name
 * that the reference runtime registers for its JIT'd host programs
 * (reference: base/src/jit.rs:47-88, bodies in base/src/ffi/cuda.rs; the
 * authoritative argument lists are lean/lib/AlgorithmLib/FFI.lean:347-408).
 * The implementation underneath is new: the CUDA driver API resolved with
 * dlopen at `cl_cuda_init`, so the library itself loads on a machine that
 * has no GPU driver.
 *
 * The `cl_b200_*` symbols are additions the reference has no counterpart
 * for; each says why it exists.
 *
 * Conventions (reference: base/src/ffi/cuda.rs:2840-2884 and the unit tests
 * at :1993-2891): a null context returns -1; ids are indices into
 * per-context tables, handed out sequentially from 0 and never reused;
 * every argument is validated before the driver is touched; nothing throws
 * across this boundary.
 */
#ifndef B200ABI_H
#define B200ABI_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#pragma GCC visibility push(default)

typedef struct B200CudaContext B200CudaContext;

/* ---- lifecycle (cuda.rs:338-358, 1318-1323) ------------------------------
 * `cl_cuda_init` writes a context pointer into *slot (null on failure: no
 * driver, no device).  Device ordinal = $B200_DEVICE, else $LOCAL_RANK,
 * else 0 (the reference hard-codes 0, cuda.rs:331-336).
 * `cl_cuda_cleanup` frees everything the context owns and nulls *slot; a
 * null slot or an already-null *slot is a no-op. */
void    cl_cuda_init(B200CudaContext **slot);
void    cl_cuda_cleanup(B200CudaContext **slot);

/* ---- buffers (cuda.rs:360-491, 1124-1243) --------------------------------
 * Buffers are zero-filled at creation.  size <= 0 -> -1.  Uploads and
 * downloads are synchronous; the *_offset forms bounds-check
 * offset + size against the buffer; the plain forms check size. */
int32_t cl_cuda_create_buffer(B200CudaContext *ctx, int64_t size);
int32_t cl_cuda_free_buffer(B200CudaContext *ctx, int32_t buf_id);
int32_t cl_cuda_upload(B200CudaContext *ctx, int32_t buf_id, const uint8_t *src, int64_t size);
int32_t cl_cuda_upload_ptr(B200CudaContext *ctx, int32_t buf_id, const uint8_t *src, int64_t size);
int32_t cl_cuda_upload_ptr_offset(B200CudaContext *ctx, int32_t buf_id, int64_t buf_offset,
                                  const uint8_t *src, int64_t size);
int32_t cl_cuda_download(B200CudaContext *ctx, int32_t buf_id, uint8_t *dst, int64_t size);
int32_t cl_cuda_download_ptr(B200CudaContext *ctx, int32_t buf_id, uint8_t *dst, int64_t size);
int32_t cl_cuda_download_ptr_offset(B200CudaContext *ctx, int32_t buf_id, int64_t buf_offset,
                                    uint8_t *dst, int64_t size);

/* ---- async copies (cuda.rs:1005-1122); stream_id < 0 = the context's main
 * stream.  The host pointer must stay valid until the stream is synced. */
int32_t cl_cuda_upload_ptr_async(B200CudaContext *ctx, int32_t buf_id, const uint8_t *src,
                                 int64_t size, int32_t stream_id);
int32_t cl_cuda_upload_ptr_offset_async(B200CudaContext *ctx, int32_t buf_id, int64_t buf_offset,
                                        const uint8_t *src, int64_t size, int32_t stream_id);
int32_t cl_cuda_download_ptr_async(B200CudaContext *ctx, int32_t buf_id, uint8_t *dst,
                                   int64_t size, int32_t stream_id);

/* ---- streams / events (cuda.rs:493-768) ----------------------------------
 * A new stream is non-blocking and is ordered after everything already
 * queued on the main stream.  `elapsed_ms_bits` returns the f32 bit pattern
 * of the milliseconds between two recorded events, -1 if either id is bad
 * or unrecorded. */
int32_t cl_cuda_stream_create(B200CudaContext *ctx);
int32_t cl_cuda_stream_sync(B200CudaContext *ctx, int32_t stream_id);
int32_t cl_cuda_stream_destroy(B200CudaContext *ctx, int32_t stream_id);
int32_t cl_cuda_event_create(B200CudaContext *ctx);
int32_t cl_cuda_event_record(B200CudaContext *ctx, int32_t event_id, int32_t stream_id);
int32_t cl_cuda_stream_wait_event(B200CudaContext *ctx, int32_t stream_id, int32_t event_id);
int32_t cl_cuda_event_elapsed_ms_bits(B200CudaContext *ctx, int32_t start_event_id, int32_t end_event_id);
int32_t cl_cuda_event_destroy(B200CudaContext *ctx, int32_t event_id);

/* ---- graphs (cuda.rs:770-926): relaxed-mode capture on a stream,
 * `end_capture` instantiates and returns a graph id. */
int32_t cl_cuda_graph_begin_capture(B200CudaContext *ctx, int32_t stream_id);
int32_t cl_cuda_graph_end_capture(B200CudaContext *ctx, int32_t stream_id);
int32_t cl_cuda_graph_upload(B200CudaContext *ctx, int32_t graph_id, int32_t stream_id);
int32_t cl_cuda_graph_launch(B200CudaContext *ctx, int32_t graph_id, int32_t stream_id);
int32_t cl_cuda_graph_destroy(B200CudaContext *ctx, int32_t graph_id);

/* ---- pinned host memory (cuda.rs:928-1003) ------------------------------ */
int32_t cl_cuda_pinned_alloc(B200CudaContext *ctx, int64_t size);
int64_t cl_cuda_pinned_ptr(B200CudaContext *ctx, int32_t pinned_id);
int32_t cl_cuda_pinned_free(B200CudaContext *ctx, int32_t pinned_id);

/* ---- launches of NUL-terminated PTX text (cuda.rs:1254-1298, 1329-1467) ---
 * The module is cached by the host address of the text.  Kernel parameters
 * are device pointers only, one per packed little-endian i32 buffer id in
 * `bind`.  Entry point "main" unless named.  No dynamic shared memory.
 * Any grid/block dimension <= 0, n_bufs < 0 or an unknown id -> -1. */
int32_t cl_cuda_launch(B200CudaContext *ctx, const uint8_t *kernel_text, int32_t n_bufs,
                       const uint8_t *bind, int32_t gx, int32_t gy, int32_t gz,
                       int32_t bx, int32_t by, int32_t bz);
int32_t cl_cuda_launch_named(B200CudaContext *ctx, const uint8_t *kernel_text, const uint8_t *name,
                             int32_t n_bufs, const uint8_t *bind, int32_t gx, int32_t gy, int32_t gz,
                             int32_t bx, int32_t by, int32_t bz);
int32_t cl_cuda_launch_on_stream(B200CudaContext *ctx, const uint8_t *kernel_text, int32_t n_bufs,
                                 const uint8_t *bind, int32_t gx, int32_t gy, int32_t gz,
                                 int32_t bx, int32_t by, int32_t bz, int32_t stream_id);
int32_t cl_cuda_launch_named_on_stream(B200CudaContext *ctx, const uint8_t *kernel_text,
                                       const uint8_t *name, int32_t n_bufs, const uint8_t *bind,
                                       int32_t gx, int32_t gy, int32_t gz,
                                       int32_t bx, int32_t by, int32_t bz, int32_t stream_id);
int32_t cl_cuda_sync(const B200CudaContext *ctx);

/* ---- f32 GEMV / GEMM with the reference's cuBLAS call convention
 * (cuda.rs:1530-1991): column-major, scalars alpha/beta passed as f32 bit
 * patterns, operands named by buffer id.  Implemented by this library's own
 * sm_100a kernels; no cuBLAS is loaded.  A row-major W[rows,cols] times x
 * is `sgemv(trans=1, m=cols, n=rows)` as in the reference's call sites
 * (lean/lib/AlgorithmLib/Cuda.lean:278-288). */
int32_t cl_cublas_sgemv(B200CudaContext *ctx, int32_t trans, int32_t m, int32_t n, int32_t alpha_bits,
                        int32_t a_buf, int32_t x_buf, int32_t beta_bits, int32_t y_buf);
int32_t cl_cublas_sgemv_on_stream(B200CudaContext *ctx, int32_t trans, int32_t m, int32_t n,
                                  int32_t alpha_bits, int32_t a_buf, int32_t x_buf,
                                  int32_t beta_bits, int32_t y_buf, int32_t stream_id);
int32_t cl_cublas_sgemm(B200CudaContext *ctx, int32_t transa, int32_t transb, int32_t m, int32_t n,
                        int32_t k, int32_t alpha_bits, int32_t a_buf, int32_t b_buf,
                        int32_t beta_bits, int32_t c_buf);
int32_t cl_cublas_sgemm_strided_batched(B200CudaContext *ctx, int32_t transa, int32_t transb,
                                        int32_t m, int32_t n, int32_t k, int32_t alpha_bits,
                                        int32_t a_buf, int64_t stride_a, int32_t b_buf, int64_t stride_b,
                                        int32_t beta_bits, int32_t c_buf, int64_t stride_c,
                                        int32_t batch_count);
int32_t cl_cublas_sgemm_strided_batched_on_stream(B200CudaContext *ctx, int32_t transa, int32_t transb,
                                                  int32_t m, int32_t n, int32_t k, int32_t alpha_bits,
                                                  int32_t a_buf, int64_t stride_a, int32_t b_buf,
                                                  int64_t stride_b, int32_t beta_bits, int32_t c_buf,
                                                  int64_t stride_c, int32_t batch_count,
                                                  int32_t stream_id);

/* ---- additions (no counterpart in the reference) -------------------------
 * The reference finds kernel text with a NUL-terminated read and passes
 * scalars through a device "meta" buffer (lean/algorithms/Qwen2Common.lean:
 * 658-671).  A cubin is binary and the sm_100a kernels want real scalar
 * parameters, dynamic shared memory above 48 KB and, for some, programmatic
 * dependent launch, so: */

/* Load a cubin (or PTX) image of `len` bytes; returns a module id. */
int32_t cl_b200_load_module(B200CudaContext *ctx, const uint8_t *image, int64_t len);

/* Module id of the kernels built into this library (loaded on first use). */
int32_t cl_b200_builtin_module(B200CudaContext *ctx);

/* Launch `name` from a module.  Kernel parameters are `n_bufs` device
 * pointers (from the packed i32 ids in `bind`; id -1 passes a null pointer)
 * followed, when scalar_bytes > 0, by ONE by-value struct of that size
 * copied from `scalars`.  flags bit 0: programmatic dependent launch (the
 * kernel may start before its predecessor on the stream has finished and
 * must order itself with griddepcontrol.wait).  flags bit 1: cooperative
 * launch (all CTAs of the grid resident at once; the launch fails instead of
 * running when the grid does not fit), for kernels with grid-wide barriers. */
int32_t cl_b200_launch(B200CudaContext *ctx, int32_t module_id, const uint8_t *name,
                       int32_t n_bufs, const uint8_t *bind,
                       const uint8_t *scalars, int32_t scalar_bytes,
                       int32_t gx, int32_t gy, int32_t gz, int32_t bx, int32_t by, int32_t bz,
                       int32_t dyn_smem_bytes, int32_t stream_id, int32_t flags);

/* Device address / byte size of a buffer (0 / -1 for a bad id). */
int64_t cl_b200_buffer_ptr(B200CudaContext *ctx, int32_t buf_id);
int64_t cl_b200_buffer_size(B200CudaContext *ctx, int32_t buf_id);

/* Fill `size` bytes at `buf_offset` with `value` on a stream. */
int32_t cl_b200_memset_async(B200CudaContext *ctx, int32_t buf_id, int64_t buf_offset,
                             int32_t value, int64_t size, int32_t stream_id);

/* Device-to-device copy on a stream, bounds-checked on both sides. */
int32_t cl_b200_copy_async(B200CudaContext *ctx, int32_t dst_buf, int64_t dst_offset,
                           int32_t src_buf, int64_t src_offset, int64_t size, int32_t stream_id);

/* Copy `size` bytes of a buffer to a raw device address of the same device (memory owned by another
 * library in the process, e.g. a tensor handed to a collective), on a stream.  No counterpart in the
 * reference (its buffers never leave its tables). */
int32_t cl_b200_copy_to_device_ptr(B200CudaContext *ctx, int32_t src_buf, int64_t src_offset,
                                   uint64_t dst_device_ptr, int64_t size, int32_t stream_id);

/* Device ordinal in use, number of SMs, free device memory in bytes. */
int32_t cl_b200_device_ordinal(B200CudaContext *ctx);
int32_t cl_b200_sm_count(B200CudaContext *ctx);
int64_t cl_b200_mem_free(B200CudaContext *ctx);

/* The CUstream / cudaStream_t behind a stream id of this context (-1 = the main stream), as an
 * integer; 0 for a bad id.  For handing a stream of this library to code that takes raw stream
 * handles (cl_b200_argmax_noalloc below, another library in the process).  Every stream of this
 * library is non-blocking: work on the legacy default stream (handle 0) is NOT ordered with it. */
int64_t cl_b200_stream_handle(B200CudaContext *ctx, int32_t stream_id);

/* Collectives for the expert-parallel decode step, over NCCL (libnccl.so.2, loaded on first use).  No
 * counterpart in the reference, which has no multi-device path (base/src/ffi/cuda.rs:331-336 opens device 0).
 * One process per GPU: rank 0 makes a 128-byte id (cl_b200_comm_unique_id), every rank gets it by any host
 * channel and calls cl_b200_comm_init on its context (outside any stream capture).  The two collectives run
 * on a stream of the context and can be captured into a CUDA graph:
 *   all_gather: recv[r*bytes .. (r+1)*bytes) on every rank = rank r's send[send_offset .. +bytes);
 *   all_to_all: rank r receives send[r*bytes .. +bytes) of every rank q into recv[q*bytes .. +bytes).
 * Every call returns 0 or -1. */
int32_t cl_b200_comm_unique_id(uint8_t *out128);
int32_t cl_b200_comm_init(B200CudaContext *ctx, const uint8_t *id128, int32_t rank, int32_t world);
int32_t cl_b200_comm_world(B200CudaContext *ctx);
int32_t cl_b200_comm_all_gather(B200CudaContext *ctx, int32_t send_buf, int64_t send_offset, int32_t recv_buf,
                                int64_t bytes, int32_t stream_id);
int32_t cl_b200_comm_all_to_all(B200CudaContext *ctx, int32_t send_buf, int32_t recv_buf, int64_t bytes,
                                int32_t stream_id);

/* Peer memory, for kernels that write to and read from another process's buffers over NVLink themselves
 * (the batched decode step's dispatch and combine).  No counterpart in the reference (cuda.rs has one
 * device per process and no inter-process memory).  export: a 64-byte handle of a buffer made by
 * cl_cuda_create_buffer; open: the address, in this process, of the buffer behind a handle another process
 * exported (peer access is enabled by the call); close: unmaps it.  Handles travel by any host channel.
 * The exported buffer must outlive every mapping of it.  open returns 0 on error. */
int32_t cl_b200_ipc_export(B200CudaContext *ctx, int32_t buf_id, uint8_t *out64);
int64_t cl_b200_ipc_open(B200CudaContext *ctx, const uint8_t *handle64);
int32_t cl_b200_ipc_close(B200CudaContext *ctx, int64_t address);


/* Last error text of the calling thread ("" if none); never null. */
const char *cl_b200_last_error(void);

/* Greedy argmax without any allocation (no counterpart in the reference).
 * For callers that must not allocate device memory: code living inside a
 * fixed memory pool, a serving loop that cannot afford cudaMalloc's
 * device-wide stall, a host that has handed all device memory to someone
 * else.  out_dev[b] = smallest index of the maximum of
 * logits_dev[b*stride .. b*stride + vocab), for b < tokens.  All pointers are
 * device pointers on the current device, `stream` a CUstream / cudaStream_t
 * (null = legacy default stream).  The scratch the regular argmax kernel
 * needs is a fixed ~66 KB array inside the library image, held on every GPU
 * that loads the library until exit; tokens <= 64, more is rejected with -1.
 * Calls share that array: calls that overlap on the GPU race.  The first
 * call on a device resolves the array's device address; make it before any
 * stream capture.  The address is remembered per device: after a
 * cudaDeviceReset by the host program it is looked up again when the first
 * operation on it fails.
 * Ordering: the work runs on `stream` and nowhere else.  Logits produced by
 * this library (cl_b200_launch, a stage program) are on one of its own
 * non-blocking streams, with which the default stream does not synchronise:
 * pass cl_b200_stream_handle(ctx, id) of the producing stream (-1 = main
 * stream), or cl_cuda_sync on both sides of the call.
 * Returns 0, or -1 with text in cl_b200_argmax_noalloc_error(). */
int32_t cl_b200_argmax_noalloc(const float *logits_dev, int32_t vocab, int32_t tokens, int32_t stride,
                               int32_t *out_dev, void *stream);
const char *cl_b200_argmax_noalloc_error(void);

#pragma GCC visibility pop
#ifdef __cplusplus
}
#endif
#endif /* B200ABI_H */
